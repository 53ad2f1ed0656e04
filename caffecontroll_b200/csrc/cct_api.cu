// Context, memory and convolution-plan entry points of include/cct_b200.h.
#include <cstdio>
#include <new>

#include <algorithm>
#include <cmath>
#include <random>
#include <vector>

#include "cct_internal.h"

struct cct_conv_plan {
  cct_ctx* ctx = nullptr;
  cct_conv_desc desc{};
  ConvGeom G{};
  int algo = CCT_ALGO_SIMT_FP32;
  UmmaPlan* umma = nullptr;
  // Device staging for the host-buffer entry points, allocated on first use.
  float *sX = nullptr, *sW = nullptr, *sb = nullptr, *sY = nullptr, *sdY = nullptr, *sdX = nullptr, *sdW = nullptr,
        *sdb = nullptr;
  size_t staging_bytes = 0;
  bool staged_forward = false;  // sX / sW hold what the last cct_conv_forward_host uploaded
  float* mask_dY = nullptr;     // output gradient rebuilt from the pooled gradient (cct_conv_plan_reserve_fusion)
  bool staging_ready = false;   // every staging buffer, side stream and event below exists
  // Host-buffer calls move the batch in slices: slice c is uploaded (ev_in[c]), processed, downloaded (after ev_out[c]).
  static constexpr int kSlices = 8;
  cudaEvent_t ev_in[kSlices] = {}, ev_out[kSlices] = {}, ev_start = nullptr, ev_done = nullptr;
  PhaseTimer timer;
};

namespace {

int geom_from_desc(const cct_conv_desc* d, ConvGeom* G) {
  if (!d) return CCT_ERR_INVALID;
  if (d->batch <= 0 || d->in_depth <= 0 || d->in_size <= 0 || d->out_depth <= 0 || d->kernel <= 0 || d->stride <= 0 ||
      d->pad < 0 || d->groups <= 0)
    return CCT_ERR_INVALID;
  if (d->in_depth % d->groups || d->out_depth % d->groups) return CCT_ERR_INVALID;
  if (d->in_size + 2 * d->pad < d->kernel) return CCT_ERR_INVALID;
  G->B = d->batch; G->D = d->in_depth; G->n = d->in_size; G->o = d->out_depth;
  G->k = d->kernel; G->s = d->stride; G->p = d->pad; G->g = d->groups;
  G->m = (d->in_size + 2 * d->pad - d->kernel) / d->stride + 1;
  G->Dg = d->in_depth / d->groups;
  G->og = d->out_depth / d->groups;
  G->bias = d->bias_term != 0;
  // 32-bit index arithmetic inside the kernels: keep every tensor below 2^31 elements.
  const double lim = 2147483647.0;
  if ((double)G->B * G->D * G->n * G->n > lim || (double)G->B * G->o * G->m * G->m > lim) return CCT_ERR_UNSUPPORTED;
  return CCT_OK;
}

// All or nothing: a failed allocation releases what this call allocated, so that a retry starts from scratch.
int ensure_staging(cct_conv_plan* p) {
  if (p->staging_ready) return CCT_OK;
  cct_ctx* ctx = p->ctx;
  const ConvGeom& G = p->G;
  const size_t nx = (size_t)G.B * G.D * G.n * G.n, ny = (size_t)G.B * G.o * G.m * G.m,
               nw = (size_t)G.o * G.Dg * G.k * G.k;
  float** slots[] = {&p->sX, &p->sW, &p->sb, &p->sY, &p->sdY, &p->sdX, &p->sdW, &p->sdb};
  const size_t counts[] = {nx, nw, (size_t)G.o, ny, ny, nx, nw, (size_t)G.o};
  cudaError_t e = cudaSuccess;
  size_t bytes = 0;
  for (int i = 0; i < 8 && e == cudaSuccess; ++i) {
    e = cudaMalloc((void**)slots[i], counts[i] * sizeof(float));
    if (e == cudaSuccess) bytes += counts[i] * sizeof(float);
  }
  if (e == cudaSuccess && !ctx->copy_in) e = cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking);
  if (e == cudaSuccess && !ctx->copy_out) e = cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking);
  for (int c = 0; c < cct_conv_plan::kSlices && e == cudaSuccess; ++c) {
    if (!p->ev_in[c]) e = cudaEventCreateWithFlags(&p->ev_in[c], cudaEventDisableTiming);
    if (e == cudaSuccess && !p->ev_out[c]) e = cudaEventCreateWithFlags(&p->ev_out[c], cudaEventDisableTiming);
  }
  if (e == cudaSuccess && !p->ev_start) e = cudaEventCreateWithFlags(&p->ev_start, cudaEventDisableTiming);
  if (e == cudaSuccess && !p->ev_done) e = cudaEventCreateWithFlags(&p->ev_done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    for (float** s : slots) {
      if (*s) cudaFree(*s);
      *s = nullptr;
    }
    ctx->last_error = std::string("staging for the host-buffer calls: ") + cudaGetErrorString(e);
    return e == cudaErrorMemoryAllocation ? CCT_ERR_NOMEM : CCT_ERR_CUDA;
  }
  p->staging_bytes += bytes;
  p->staging_ready = true;
  return CCT_OK;
}

// Images per slice of the pipelined host-buffer calls (0: do not slice - tiny batches and the direct fp32 path).
int slice_images(const cct_conv_plan* p) {
  if (p->algo != CCT_ALGO_UMMA_3XTF32 || p->G.B < 2 * cct_conv_plan::kSlices) return 0;
  return (p->G.B + cct_conv_plan::kSlices - 1) / cct_conv_plan::kSlices;
}

// Both side streams start behind whatever the context's stream has queued; at the end the context's stream waits for
// the downloads, so that cct_sync() covers the whole call.
int host_call_begin(cct_conv_plan* p) {
  cct_ctx* ctx = p->ctx;
  CCT_CUDA(ctx, cudaEventRecord(p->ev_start, ctx->stream));
  CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_in, p->ev_start, 0));
  CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, p->ev_start, 0));
  return CCT_OK;
}
int host_call_end(cct_conv_plan* p) {
  cct_ctx* ctx = p->ctx;
  CCT_CUDA(ctx, cudaEventRecord(p->ev_done, ctx->copy_out));
  CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, p->ev_done, 0));
  CCT_CUDA(ctx, cudaEventRecord(p->ev_done, ctx->copy_in));
  CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, p->ev_done, 0));
  return cct_sync(ctx);
}

}  // namespace

extern "C" {

int cct_device_count(int* count) {
  if (!count) return CCT_ERR_INVALID;
  return cudaGetDeviceCount(count) == cudaSuccess ? CCT_OK : CCT_ERR_CUDA;
}

static int ctx_create_common(int device_id, cudaStream_t stream, bool make_stream, cct_ctx** out) {
  if (!out) return CCT_ERR_INVALID;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device_id < 0 || device_id >= count) return CCT_ERR_CUDA;
  cct_ctx* ctx = new (std::nothrow) cct_ctx();
  if (!ctx) return CCT_ERR_NOMEM;
  ctx->device = device_id;
  cudaError_t e = cudaSetDevice(device_id);
  cudaDeviceProp prop;
  if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device_id);
  if (e == cudaSuccess && prop.major != 10) {
    std::fprintf(stderr, "cct_b200: device %d is sm_%d%d; this library contains sm_100a code only\n", device_id,
                 prop.major, prop.minor);
    delete ctx;
    return CCT_ERR_UNSUPPORTED;
  }
  if (e == cudaSuccess) {
    ctx->sm_count = prop.multiProcessorCount;
    if (make_stream) {
      e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
      ctx->owns_stream = true;
    } else {
      ctx->stream = stream;
    }
  }
  int* hs = nullptr;
  if (e == cudaSuccess) e = cudaHostAlloc((void**)&hs, sizeof(int), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    *hs = 0;
    ctx->status_host = hs;
    e = cudaHostGetDevicePointer((void**)&ctx->status_dev, hs, 0);
  }
  if (e != cudaSuccess) {
    std::fprintf(stderr, "cct_b200: context creation failed: %s\n", cudaGetErrorString(e));
    if (hs) cudaFreeHost(hs);
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return CCT_ERR_CUDA;
  }
  *out = ctx;
  return CCT_OK;
}

int cct_ctx_create(int device_id, cct_ctx** out) { return ctx_create_common(device_id, nullptr, true, out); }

int cct_ctx_create_on_stream(int device_id, void* cuda_stream, cct_ctx** out) {
  return ctx_create_common(device_id, (cudaStream_t)cuda_stream, false, out);
}

int cct_ctx_destroy(cct_ctx* ctx) {
  if (!ctx) return CCT_ERR_INVALID;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
  if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
  if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
  if (ctx->status_host) cudaFreeHost((void*)ctx->status_host);
  delete ctx;
  return CCT_OK;
}

int cct_sync(cct_ctx* ctx) {
  if (!ctx) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (*ctx->status_host != 0) {
    char buf[96];
    std::snprintf(buf, sizeof buf, "device-side bounded wait gave up (status word 0x%x)", *ctx->status_host);
    ctx->last_error = buf;
    *ctx->status_host = 0;
    return CCT_ERR_TIMEOUT;
  }
  return CCT_OK;
}

const char* cct_last_error_string(cct_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int cct_malloc(cct_ctx* ctx, size_t bytes, void** dptr) {
  if (!ctx || !dptr) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaMalloc(dptr, bytes ? bytes : 1));
  return CCT_OK;
}

int cct_free(cct_ctx* ctx, void* dptr) {
  if (!ctx) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaFree(dptr));
  return CCT_OK;
}

int cct_malloc_host(cct_ctx* ctx, size_t bytes, void** hptr) {
  if (!ctx || !hptr) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocDefault));
  return CCT_OK;
}

int cct_free_host(cct_ctx* ctx, void* hptr) {
  if (!ctx) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaFreeHost(hptr));
  return CCT_OK;
}

static int copy_common(cct_ctx* ctx, void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
  if (!ctx || ((!dst || !src) && bytes)) return CCT_ERR_INVALID;
  if (!bytes) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, kind, ctx->stream));
  return CCT_OK;
}

int cct_memcpy_h2d(cct_ctx* ctx, void* dst, const void* src, size_t bytes) {
  return copy_common(ctx, dst, src, bytes, cudaMemcpyHostToDevice);
}
int cct_memcpy_d2h(cct_ctx* ctx, void* dst, const void* src, size_t bytes) {
  return copy_common(ctx, dst, src, bytes, cudaMemcpyDeviceToHost);
}
int cct_memcpy_d2d(cct_ctx* ctx, void* dst, const void* src, size_t bytes) {
  return copy_common(ctx, dst, src, bytes, cudaMemcpyDeviceToDevice);
}

int cct_memcpy2d_d2d(cct_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                     size_t rows) {
  if (!ctx || ((!dst || !src) && width_bytes && rows) || dst_pitch < width_bytes || src_pitch < width_bytes)
    return CCT_ERR_INVALID;
  if (!width_bytes || !rows) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDeviceToDevice, ctx->stream));
  return CCT_OK;
}

int cct_memset(cct_ctx* ctx, void* dptr, int byte_value, size_t bytes) {
  if (!ctx || (!dptr && bytes)) return CCT_ERR_INVALID;
  if (!bytes) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaMemsetAsync(dptr, byte_value, bytes, ctx->stream));
  return CCT_OK;
}

// The reference's fillers run on the host with the C++ standard generators (CPUDriver::sgaussian_initialize,
// sinitialize_xavier, sbernoulli_initialize: src/sched/DeviceDriver_CPU.cpp:661-699); the same calls here produce
// the same numbers for the same seed, and the result is uploaded.
int cct_fill_random(cct_ctx* ctx, float* dptr, size_t count, int kind, float a, float b, long seed) {
  if (!ctx || (!dptr && count) || kind < CCT_FILL_GAUSSIAN || kind > CCT_FILL_BERNOULLI) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  std::vector<float> host(count);
  std::random_device rd;
  std::mt19937 gen(seed == -1 ? rd() : (unsigned)seed);
  if (kind == CCT_FILL_GAUSSIAN) {
    std::normal_distribution<float> dist(a, b);
    for (size_t i = 0; i < count; ++i) host[i] = dist(gen);
  } else if (kind == CCT_FILL_XAVIER) {
    if (!(a > 0.f)) return CCT_ERR_INVALID;
    const float scale = (float)std::sqrt(3.0 / (size_t)a);
    std::uniform_real_distribution<float> dist(-scale, scale);
    for (size_t i = 0; i < count; ++i) host[i] = dist(gen);
  } else {
    std::bernoulli_distribution dist(a);
    for (size_t i = 0; i < count; ++i) host[i] = dist(gen);
  }
  CCT_CUDA(ctx, cudaMemcpyAsync(dptr, host.data(), count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  CCT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // `host` goes out of scope
  return CCT_OK;
}

int cct_conv_out_size(const cct_conv_desc* desc, int* out_size) {
  ConvGeom G;
  const int rc = geom_from_desc(desc, &G);
  if (rc != CCT_OK || !out_size) return rc != CCT_OK ? rc : CCT_ERR_INVALID;
  *out_size = G.m;
  return CCT_OK;
}

int cct_conv_plan_create(cct_ctx* ctx, const cct_conv_desc* desc, cct_conv_plan** out) {
  if (!ctx || !out) return CCT_ERR_INVALID;
  *out = nullptr;
  ConvGeom G;
  const int rc = geom_from_desc(desc, &G);
  if (rc != CCT_OK) {
    ctx->last_error = "invalid convolution descriptor";
    return rc;
  }
  int algo = desc->algo;
  if (algo == CCT_ALGO_AUTO) algo = umma_supported(G) ? CCT_ALGO_UMMA_3XTF32 : CCT_ALGO_SIMT_FP32;
  if (algo != CCT_ALGO_SIMT_FP32 && algo != CCT_ALGO_UMMA_3XTF32) return CCT_ERR_INVALID;
  if (algo == CCT_ALGO_UMMA_3XTF32 && !umma_supported(G)) {
    ctx->last_error = "shape not supported by the tcgen05 path";
    return CCT_ERR_UNSUPPORTED;
  }
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  cct_conv_plan* p = new (std::nothrow) cct_conv_plan();
  if (!p) return CCT_ERR_NOMEM;
  p->ctx = ctx;
  p->desc = *desc;
  p->G = G;
  p->algo = algo;
  if (algo == CCT_ALGO_UMMA_3XTF32) {
    const int rc2 = umma_plan_create(ctx, G, &p->umma);
    if (rc2 != CCT_OK) {
      delete p;
      return rc2;
    }
  }
  *out = p;
  return CCT_OK;
}

int cct_conv_plan_destroy(cct_conv_plan* plan) {
  if (!plan) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (plan->umma) umma_plan_destroy(ctx, plan->umma);
  for (cudaEvent_t e : plan->timer.ev)
    if (e) cudaEventDestroy(e);
  for (int c = 0; c < cct_conv_plan::kSlices; ++c) {
    if (plan->ev_in[c]) cudaEventDestroy(plan->ev_in[c]);
    if (plan->ev_out[c]) cudaEventDestroy(plan->ev_out[c]);
  }
  if (plan->ev_start) cudaEventDestroy(plan->ev_start);
  if (plan->ev_done) cudaEventDestroy(plan->ev_done);
  float* slots[] = {plan->sX, plan->sW, plan->sb, plan->sY, plan->sdY, plan->sdX, plan->sdW, plan->sdb, plan->mask_dY};
  for (float* s : slots)
    if (s) cudaFree(s);
  delete plan;
  return CCT_OK;
}

int cct_conv_plan_algo(const cct_conv_plan* plan, int* algo) {
  if (!plan || !algo) return CCT_ERR_INVALID;
  *algo = plan->algo;
  return CCT_OK;
}

int cct_conv_plan_workspace_bytes(const cct_conv_plan* plan, size_t* bytes) {
  if (!plan || !bytes) return CCT_ERR_INVALID;
  *bytes = (plan->umma ? umma_plan_workspace_bytes(plan->umma) : 0) + plan->staging_bytes;
  return CCT_OK;
}

int cct_conv_plan_reserve_fusion(cct_conv_plan* plan) {
  if (!plan) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  const ConvGeom& G = plan->G;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!plan->mask_dY) {
    const size_t bytes = (size_t)G.B * G.o * G.m * G.m * sizeof(float);
    CCT_CUDA(ctx, cudaMalloc((void**)&plan->mask_dY, bytes));
    plan->staging_bytes += bytes;
  }
  return CCT_OK;
}

int cct_conv_plan_enable_timing(cct_conv_plan* plan, int enable) {
  if (!plan) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  PhaseTimer& t = plan->timer;
  if (enable && !t.ev[0])
    for (cudaEvent_t& e : t.ev) CCT_CUDA(ctx, cudaEventCreate(&e));
  t.enabled = enable != 0;
  for (bool& h : t.have) h = false;
  return CCT_OK;
}

int cct_conv_plan_last_timings(cct_conv_plan* plan, float ms[5]) {
  if (!plan || !ms) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  CCT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (int i = 0; i < PhaseTimer::kSlots; ++i) {
    ms[i] = 0.f;
    if (plan->timer.have[i]) CCT_CUDA(ctx, cudaEventElapsedTime(&ms[i], plan->timer.ev[2 * i], plan->timer.ev[2 * i + 1]));
  }
  return CCT_OK;
}

int cct_conv_forward(cct_conv_plan* plan, const float* X, const float* W, const float* bias, float* Y, int relu) {
  if (!plan || !X || !W || !Y) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  if (plan->G.bias && !bias) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  if (plan->algo == CCT_ALGO_UMMA_3XTF32) return umma_conv_forward(ctx, plan->umma, X, W, bias, Y, relu, &plan->timer);
  return simt_conv_forward(ctx, plan->G, X, W, bias, Y, relu, &plan->timer);
}

int cct_conv_backward(cct_conv_plan* plan, const float* X, const float* W, const float* dY, float* dX, float* dW,
                      float* db) {
  if (!plan || !X || !W || !dY || !dW) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  if (plan->G.bias && !db) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  if (plan->algo == CCT_ALGO_UMMA_3XTF32)
    return umma_conv_backward(ctx, plan->umma, X, W, dY, dX, dW, db, &plan->timer);
  return simt_conv_backward(ctx, plan->G, X, W, dY, dX, dW, db, &plan->timer);
}

int cct_conv_backward_fused(cct_conv_plan* plan, const float* X, const float* W, const float* dY,
                            const cct_bwd_fusion* f, float* dX, float* dW, float* db) {
  if (!f) return cct_conv_backward(plan, X, W, dY, dX, dW, db);
  if (!plan || !X || !W || !dW) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  const ConvGeom& G = plan->G;
  if (G.bias && !db) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  if (f->dP) {
    // conv -> ReLU -> max-pool behind this layer: one pass builds the output gradient both kernels read.
    if ((!f->A && !f->P) || !f->idx || f->pool_k <= 0 || f->pool_s <= 0 || f->pool_k > G.m) return CCT_ERR_INVALID;
    if (!plan->mask_dY) {
      ctx->last_error = "cct_conv_backward_fused with a pooled gradient needs cct_conv_plan_reserve_fusion(plan) first";
      return CCT_ERR_INVALID;
    }
    const int rc = f->P ? pool_relu_backward_pooled(ctx, f->P, f->idx, f->dP, plan->mask_dY, G.B * G.o, G.m, f->pool_k, f->pool_s)
                        : cct_pool_relu_backward(ctx, f->A, f->idx, f->dP, plan->mask_dY, G.B * G.o, G.m, f->pool_k, f->pool_s);
    if (rc != CCT_OK) return rc;
    dY = plan->mask_dY;
  }
  if (!dY) return CCT_ERR_INVALID;
  // The ReLU bridge in front of the layer: dX *= [X > 0] as one HBM-bound pass behind the data-gradient kernel.
  // (Folded into that kernel's epilogue it cost more than the pass: one extra load per accumulator column in the four
  // epilogue warps made the epilogue the bottleneck of wide data gradients.)
  int rc = plan->algo == CCT_ALGO_UMMA_3XTF32 ? umma_conv_backward(ctx, plan->umma, X, W, dY, dX, dW, db, &plan->timer)
                                              : simt_conv_backward(ctx, G, X, W, dY, dX, dW, db, &plan->timer);
  if (rc == CCT_OK && f->relu_mask_dx && dX) rc = cct_relu_backward(ctx, X, dX, dX, (size_t)G.B * G.D * G.n * G.n);
  return rc;
}

int cct_conv_forward_host(cct_conv_plan* plan, const float* hX, const float* hW, const float* hbias, float* hY,
                          int relu) {
  if (!plan || !hX || !hW || !hY) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  const ConvGeom& G = plan->G;
  if (G.bias && !hbias) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  int rc = ensure_staging(plan);
  if (rc != CCT_OK) return rc;
  const size_t nx = (size_t)G.B * G.D * G.n * G.n, ny = (size_t)G.B * G.o * G.m * G.m,
               nw = (size_t)G.o * G.Dg * G.k * G.k;
  const int per = slice_images(plan);
  if (per > 0) {
    // Upload, kernel and download of consecutive batch slices overlap: PCIe runs in both directions at once.
    rc = host_call_begin(plan);
    if (rc != CCT_OK) return rc;
    const size_t ix = (size_t)G.D * G.n * G.n, iy = (size_t)G.o * G.m * G.m;  // elements per image
    CCT_CUDA(ctx, cudaMemcpyAsync(plan->sW, hW, nw * 4, cudaMemcpyHostToDevice, ctx->copy_in));
    if (G.bias) CCT_CUDA(ctx, cudaMemcpyAsync(plan->sb, hbias, (size_t)G.o * 4, cudaMemcpyHostToDevice, ctx->copy_in));
    int slices = 0;
    for (int b0 = 0; b0 < G.B; b0 += per, ++slices) {
      const int nb = std::min(per, G.B - b0);
      CCT_CUDA(ctx, cudaMemcpyAsync(plan->sX + b0 * ix, hX + b0 * ix, nb * ix * 4, cudaMemcpyHostToDevice, ctx->copy_in));
      CCT_CUDA(ctx, cudaEventRecord(plan->ev_in[slices], ctx->copy_in));
    }
    PhaseTimer untimed;
    slices = 0;
    for (int b0 = 0; b0 < G.B; b0 += per, ++slices) {
      const int nb = std::min(per, G.B - b0);
      CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, plan->ev_in[slices], 0));
      rc = umma_conv_forward(ctx, plan->umma, plan->sX + b0 * ix, plan->sW, plan->sb, plan->sY + b0 * iy, relu, &untimed, nb,
                             slices == 0);
      if (rc != CCT_OK) return rc;
      CCT_CUDA(ctx, cudaEventRecord(plan->ev_out[slices], ctx->stream));
      CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, plan->ev_out[slices], 0));
      CCT_CUDA(ctx, cudaMemcpyAsync(hY + b0 * iy, plan->sY + b0 * iy, nb * iy * 4, cudaMemcpyDeviceToHost, ctx->copy_out));
    }
    plan->staged_forward = true;
    return host_call_end(plan);
  }
  CCT_CUDA(ctx, cudaMemcpyAsync(plan->sX, hX, nx * 4, cudaMemcpyHostToDevice, ctx->stream));
  CCT_CUDA(ctx, cudaMemcpyAsync(plan->sW, hW, nw * 4, cudaMemcpyHostToDevice, ctx->stream));
  if (G.bias) CCT_CUDA(ctx, cudaMemcpyAsync(plan->sb, hbias, (size_t)G.o * 4, cudaMemcpyHostToDevice, ctx->stream));
  rc = cct_conv_forward(plan, plan->sX, plan->sW, plan->sb, plan->sY, relu);
  if (rc != CCT_OK) return rc;
  CCT_CUDA(ctx, cudaMemcpyAsync(hY, plan->sY, ny * 4, cudaMemcpyDeviceToHost, ctx->stream));
  plan->staged_forward = true;
  return cct_sync(ctx);
}

int cct_conv_backward_host(cct_conv_plan* plan, const float* hX, const float* hW, const float* hdY, float* hdX,
                           float* hdW, float* hdb) {
  if (!plan || !hdY || !hdW) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  const ConvGeom& G = plan->G;
  if (G.bias && !hdb) return CCT_ERR_INVALID;
  if ((!hX || !hW) && !plan->staged_forward) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  int rc = ensure_staging(plan);
  if (rc != CCT_OK) return rc;
  const size_t nx = (size_t)G.B * G.D * G.n * G.n, ny = (size_t)G.B * G.o * G.m * G.m,
               nw = (size_t)G.o * G.Dg * G.k * G.k;
  const int per = slice_images(plan);
  if (per > 0) {
    // dY arrives in slices; the data gradient of a slice runs as soon as the slice is there and its dX goes back while
    // the next slice is still arriving; the weight gradient (the whole batch) follows the last slice.
    rc = host_call_begin(plan);
    if (rc != CCT_OK) return rc;
    const size_t ix = (size_t)G.D * G.n * G.n, iy = (size_t)G.o * G.m * G.m;
    if (hW) CCT_CUDA(ctx, cudaMemcpyAsync(plan->sW, hW, nw * 4, cudaMemcpyHostToDevice, ctx->copy_in));
    if (hX) CCT_CUDA(ctx, cudaMemcpyAsync(plan->sX, hX, nx * 4, cudaMemcpyHostToDevice, ctx->copy_in));
    int slices = 0;
    for (int b0 = 0; b0 < G.B; b0 += per, ++slices) {
      const int nb = std::min(per, G.B - b0);
      CCT_CUDA(ctx, cudaMemcpyAsync(plan->sdY + b0 * iy, hdY + b0 * iy, nb * iy * 4, cudaMemcpyHostToDevice, ctx->copy_in));
      CCT_CUDA(ctx, cudaEventRecord(plan->ev_in[slices], ctx->copy_in));
    }
    PhaseTimer untimed;
    slices = 0;
    for (int b0 = 0; b0 < G.B; b0 += per, ++slices) {
      const int nb = std::min(per, G.B - b0);
      CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, plan->ev_in[slices], 0));
      if (!hdX) continue;
      rc = umma_conv_dgrad(ctx, plan->umma, plan->sW, plan->sdY + b0 * iy, plan->sdX + b0 * ix, &untimed, nb, slices == 0);
      if (rc != CCT_OK) return rc;
      CCT_CUDA(ctx, cudaEventRecord(plan->ev_out[slices], ctx->stream));
      CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, plan->ev_out[slices], 0));
      CCT_CUDA(ctx, cudaMemcpyAsync(hdX + b0 * ix, plan->sdX + b0 * ix, nb * ix * 4, cudaMemcpyDeviceToHost, ctx->copy_out));
    }
    rc = umma_conv_wgrad(ctx, plan->umma, plan->sX, plan->sdY, plan->sdW, plan->sdb, &untimed);
    if (rc != CCT_OK) return rc;
    CCT_CUDA(ctx, cudaEventRecord(plan->ev_out[0], ctx->stream));
    CCT_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_out, plan->ev_out[0], 0));
    CCT_CUDA(ctx, cudaMemcpyAsync(hdW, plan->sdW, nw * 4, cudaMemcpyDeviceToHost, ctx->copy_out));
    if (G.bias) CCT_CUDA(ctx, cudaMemcpyAsync(hdb, plan->sdb, (size_t)G.o * 4, cudaMemcpyDeviceToHost, ctx->copy_out));
    return host_call_end(plan);
  }
  if (hX) CCT_CUDA(ctx, cudaMemcpyAsync(plan->sX, hX, nx * 4, cudaMemcpyHostToDevice, ctx->stream));
  if (hW) CCT_CUDA(ctx, cudaMemcpyAsync(plan->sW, hW, nw * 4, cudaMemcpyHostToDevice, ctx->stream));
  CCT_CUDA(ctx, cudaMemcpyAsync(plan->sdY, hdY, ny * 4, cudaMemcpyHostToDevice, ctx->stream));
  rc = cct_conv_backward(plan, plan->sX, plan->sW, plan->sdY, hdX ? plan->sdX : nullptr, plan->sdW, plan->sdb);
  if (rc != CCT_OK) return rc;
  if (hdX) CCT_CUDA(ctx, cudaMemcpyAsync(hdX, plan->sdX, nx * 4, cudaMemcpyDeviceToHost, ctx->stream));
  CCT_CUDA(ctx, cudaMemcpyAsync(hdW, plan->sdW, nw * 4, cudaMemcpyDeviceToHost, ctx->stream));
  if (G.bias) CCT_CUDA(ctx, cudaMemcpyAsync(hdb, plan->sdb, (size_t)G.o * 4, cudaMemcpyDeviceToHost, ctx->stream));
  return cct_sync(ctx);
}

}  // extern "C"
