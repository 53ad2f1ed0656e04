// Gradient summation across the GPUs of one job through NCCL, behind the C ABI (cct_comm_*): what replaces the
// host-staged gather + serial CPU sum of ParallelizedBridge::backward (src/bridges/ParallelizedBridge_impl.hxx:876-971).
//
// NCCL is looked up at run time (dlopen of libnccl.so.2, the one the process already holds if any), so the library has
// no link-time dependency on it and single-GPU users never load it.  A communicator owns a communication stream: a
// reduction is ordered behind the work already queued on the context's stream, runs on the communication stream (so
// it overlaps whatever the context's stream is given next), and cct_comm_wait orders the context's stream behind it.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "cct_internal.h"

namespace {

// The slice of the NCCL API this file uses, declared here so that no NCCL header is needed to build the library.
typedef struct ncclComm* ncclComm_t;
typedef int ncclResult_t;  // 0 = ncclSuccess
struct NcclUniqueId { char internal[CCT_COMM_ID_BYTES]; };
enum { kNcclFloat = 7, kNcclSum = 0 };  // ncclFloat32, ncclSum

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(NcclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) {
    api.error = std::string("NCCL could not be loaded: ") + dlerror();
    return nullptr;
  }
  bool ok = true;
  auto sym = [&](const char* name) {
    void* p = dlsym(api.handle, name);
    if (!p) { ok = false; api.error = std::string("NCCL symbol missing: ") + name; }
    return p;
  };
  api.GetUniqueId = (ncclResult_t(*)(NcclUniqueId*))sym("ncclGetUniqueId");
  api.CommInitRank = (ncclResult_t(*)(ncclComm_t*, int, NcclUniqueId, int))sym("ncclCommInitRank");
  api.AllReduce = (ncclResult_t(*)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t))sym("ncclAllReduce");
  api.AllGather = (ncclResult_t(*)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t))sym("ncclAllGather");
  api.ReduceScatter =
      (ncclResult_t(*)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t))sym("ncclReduceScatter");
  api.CommDestroy = (ncclResult_t(*)(ncclComm_t))sym("ncclCommDestroy");
  api.CommGetAsyncError = (ncclResult_t(*)(ncclComm_t, ncclResult_t*))sym("ncclCommGetAsyncError");
  api.GetErrorString = (const char* (*)(ncclResult_t))sym("ncclGetErrorString");
  if (!ok) {
    dlclose(api.handle);
    api.handle = nullptr;
    return nullptr;
  }
  return &api;
}

}  // namespace

struct cct_comm {
  cct_ctx* ctx = nullptr;
  int nranks = 1, rank = 0;
  ncclComm_t comm = nullptr;
  cudaStream_t stream = nullptr;      // the communication stream
  cudaEvent_t ready = nullptr;        // context stream -> communication stream
  cudaEvent_t done = nullptr;         // communication stream -> context stream
  bool pending = false;               // reductions issued since the last cct_comm_wait
};

constexpr int kCommSms = 8;           // SMs left to NCCL while reductions are in flight
const char* const kCommCtas = "8";    // NCCL_MAX_CTAS unless the environment already has one

extern "C" {

int cct_comm_unique_id(unsigned char id[CCT_COMM_ID_BYTES]) {
  if (!id) return CCT_ERR_INVALID;
  NcclApi* api = nccl_api();
  if (!api) return CCT_ERR_UNSUPPORTED;
  NcclUniqueId u;
  if (api->GetUniqueId(&u) != 0) return CCT_ERR_CUDA;
  std::memcpy(id, u.internal, CCT_COMM_ID_BYTES);
  return CCT_OK;
}

int cct_comm_init_rank(cct_ctx* ctx, int nranks, int rank, const unsigned char id[CCT_COMM_ID_BYTES], cct_comm** out) {
  if (!ctx || !out || nranks < 1 || rank < 0 || rank >= nranks || (nranks > 1 && !id)) return CCT_ERR_INVALID;
  *out = nullptr;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  cct_comm* c = new (std::nothrow) cct_comm();
  if (!c) return CCT_ERR_NOMEM;
  c->ctx = ctx; c->nranks = nranks; c->rank = rank;
  if (nranks > 1) {
    NcclApi* api = nccl_api();
    if (!api) {
      ctx->last_error = "NCCL is not available (libnccl.so.2 could not be loaded or lacks a needed symbol)";
      delete c;
      return CCT_ERR_UNSUPPORTED;
    }
    // The reductions run beside the backward kernels: a few CTAs carry them at NVLink speed, and every SM NCCL does not
    // take stays with the persistent kernels (which leave kCommSms free while a reduction is in flight).  A value the
    // caller has set in the environment wins.
    setenv("NCCL_MAX_CTAS", kCommCtas, 0);
    ctx->comm_sms = kCommSms;  // plans created from now on count on that many SMs fewer during the backward pass
    NcclUniqueId u;
    std::memcpy(u.internal, id, CCT_COMM_ID_BYTES);
    const ncclResult_t r = api->CommInitRank(&c->comm, nranks, u, rank);
    if (r != 0) {
      ctx->last_error = std::string("ncclCommInitRank: ") + api->GetErrorString(r);
      delete c;
      return CCT_ERR_CUDA;
    }
  }
  cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    ctx->last_error = std::string("communicator streams: ") + cudaGetErrorString(e);
    cct_comm_destroy(c);
    return CCT_ERR_CUDA;
  }
  *out = c;
  return CCT_OK;
}

int cct_comm_destroy(cct_comm* c) {
  if (!c) return CCT_ERR_INVALID;
  cudaSetDevice(c->ctx->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  if (c->comm) {
    NcclApi* api = nccl_api();
    if (api) api->CommDestroy(c->comm);
  }
  if (c->ready) cudaEventDestroy(c->ready);
  if (c->done) cudaEventDestroy(c->done);
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
  return CCT_OK;
}

int cct_comm_size(const cct_comm* c, int* nranks, int* rank) {
  if (!c) return CCT_ERR_INVALID;
  if (nranks) *nranks = c->nranks;
  if (rank) *rank = c->rank;
  return CCT_OK;
}

int cct_allreduce_sum_begin(cct_comm* c, float* buf, size_t count) {
  if (!c || (!buf && count)) return CCT_ERR_INVALID;
  cct_ctx* ctx = c->ctx;
  if (c->nranks == 1 || count == 0) return CCT_OK;  // one partition: the sum is the gradient itself
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  NcclApi* api = nccl_api();
  if (!api) return CCT_ERR_UNSUPPORTED;
  CCT_CUDA(ctx, cudaEventRecord(c->ready, ctx->stream));
  CCT_CUDA(ctx, cudaStreamWaitEvent(c->stream, c->ready, 0));
  const ncclResult_t r = api->AllReduce(buf, buf, count, kNcclFloat, kNcclSum, c->comm, c->stream);
  if (r != 0) {
    ctx->last_error = std::string("ncclAllReduce: ") + api->GetErrorString(r);
    return CCT_ERR_CUDA;
  }
  c->pending = true;
  ctx->reserved_sms = kCommSms;
  return CCT_OK;
}

int cct_comm_wait(cct_comm* c) {
  if (!c) return CCT_ERR_INVALID;
  cct_ctx* ctx = c->ctx;
  if (!c->pending) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaEventRecord(c->done, c->stream));
  CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, c->done, 0));
  c->pending = false;
  ctx->reserved_sms = 0;
  if (c->comm) {
    NcclApi* api = nccl_api();
    ncclResult_t async = 0;
    if (api && api->CommGetAsyncError(c->comm, &async) == 0 && async != 0) {
      ctx->last_error = std::string("NCCL asynchronous error: ") + api->GetErrorString(async);
      return CCT_ERR_CUDA;
    }
  }
  return CCT_OK;
}

int cct_allreduce_sum(cct_comm* c, float* buf, size_t count) {
  const int rc = cct_allreduce_sum_begin(c, buf, count);
  return rc != CCT_OK ? rc : cct_comm_wait(c);
}

// The two exchanges of a model-parallel fully connected layer (the split and concat bridges DeepNet puts around one,
// src/DeepNet.h:1213-1357): every rank's block to every rank, and the sum over ranks of the block a rank owns.  Both
// are ordered behind the work queued on the context's stream, and the context's stream behind them.
static int exchange(cct_comm* c, const float* send, float* recv, size_t count, bool gather) {
  if (!c || ((!send || !recv) && count)) return CCT_ERR_INVALID;
  cct_ctx* ctx = c->ctx;
  if (count == 0) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  if (c->nranks == 1) {
    if (send != recv) CCT_CUDA(ctx, cudaMemcpyAsync(recv, send, count * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return CCT_OK;
  }
  NcclApi* api = nccl_api();
  if (!api) return CCT_ERR_UNSUPPORTED;
  CCT_CUDA(ctx, cudaEventRecord(c->ready, ctx->stream));
  CCT_CUDA(ctx, cudaStreamWaitEvent(c->stream, c->ready, 0));
  const ncclResult_t r = gather ? api->AllGather(send, recv, count, kNcclFloat, c->comm, c->stream)
                                : api->ReduceScatter(send, recv, count, kNcclFloat, kNcclSum, c->comm, c->stream);
  if (r != 0) {
    ctx->last_error = std::string(gather ? "ncclAllGather: " : "ncclReduceScatter: ") + api->GetErrorString(r);
    return CCT_ERR_CUDA;
  }
  c->pending = true;
  return cct_comm_wait(c);
}

int cct_allgather(cct_comm* c, const float* send, float* recv, size_t count_per_rank) {
  return exchange(c, send, recv, count_per_rank, true);
}

int cct_reduce_scatter_sum(cct_comm* c, const float* send, float* recv, size_t count_per_rank) {
  return exchange(c, send, recv, count_per_rank, false);
}

}  // extern "C"
