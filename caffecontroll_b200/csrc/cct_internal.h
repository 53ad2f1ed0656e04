// Internal declarations shared by the translation units behind include/cct_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <utility>

#include "../../include/cct_b200.h"

struct cct_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  // Side streams of the host-buffer entry points: uploads and downloads overlap each other and the kernels.
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  int sm_count = 148;
  // SMs the persistent kernels leave free while gradient reductions are in flight on the communicator's stream
  // (set by cct_allreduce_sum_begin, cleared by cct_comm_wait): NCCL's CTAs take whole SMs, and a persistent grid
  // sized for every SM would otherwise run its displaced CTAs as a second wave.
  int reserved_sms = 0;
  int launch_sms() const { return sm_count - reserved_sms > 0 ? sm_count - reserved_sms : 1; }
  // Set when a communicator of more than one rank is created on this context: plans created afterwards size their
  // work-unit counts (split counts, channel tilings) for the SMs that remain while reductions are in flight, because
  // that is when the backward kernels of a multi-GPU job run.
  int comm_sms = 0;
  int planning_sms() const { return sm_count - comm_sms > 0 ? sm_count - comm_sms : 1; }
  // One word in mapped pinned host memory that kernels set when a bounded wait runs out; read by cct_sync().
  volatile int* status_host = nullptr;
  int* status_dev = nullptr;
  std::string last_error;
};

#define CCT_CUDA(ctx, call)                                                                   \
  do {                                                                                        \
    cudaError_t e__ = (call);                                                                 \
    if (e__ != cudaSuccess) {                                                                 \
      (ctx)->last_error = std::string(#call) + ": " + cudaGetErrorString(e__);                \
      return e__ == cudaErrorMemoryAllocation ? CCT_ERR_NOMEM : CCT_ERR_CUDA;                 \
    }                                                                                         \
  } while (0)

// Programmatic dependent launch: every kernel of the library starts with pdl_wait() (griddepcontrol.wait: returns once
// the kernel before it in the stream has completed and its writes are visible) and is launched with the programmatic
// stream-serialisation attribute, so the launch itself - grid set-up, parameter upload - overlaps the tail of its
// predecessor instead of following it.  No kernel signals its dependents early: the order of execution stays the
// stream's order.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

#define CCT_CHECK_LAUNCH(ctx) CCT_CUDA(ctx, cudaGetLastError())

// Optional per-kernel-group timing with CUDA events on the context's stream (measurement only).
struct PhaseTimer {
  static constexpr int kSlots = 5;  // 0 forward, 1 wgrad, 2 wgrad reduce, 3 dgrad (with its repacking), 4 forward repack
  bool enabled = false;
  cudaEvent_t ev[2 * kSlots] = {};
  bool have[kSlots] = {};
  void begin(int slot, cudaStream_t s) {
    if (enabled) cudaEventRecord(ev[2 * slot], s);
  }
  void end(int slot, cudaStream_t s) {
    if (enabled) {
      cudaEventRecord(ev[2 * slot + 1], s);
      have[slot] = true;
    }
  }
};

// Geometry of one convolution layer, resolved once per plan.
struct ConvGeom {
  int B, D, n, o, k, s, p, g;
  int m;       // output size
  int Dg, og;  // per-group depths
  int bias;
};

// ---- SIMT fp32 path (conv_simt.cu) ----
int simt_conv_forward(cct_ctx* ctx, const ConvGeom& G, const float* X, const float* W, const float* bias, float* Y,
                      int relu, PhaseTimer* t);
int simt_conv_backward(cct_ctx* ctx, const ConvGeom& G, const float* X, const float* W, const float* dY, float* dX,
                       float* dW, float* db, PhaseTimer* t);

// ---- tcgen05 3xTF32 path (conv_umma.cu) ----
struct UmmaPlan;  // opaque: tables, packed weights, split-K scratch
int umma_plan_create(cct_ctx* ctx, const ConvGeom& G, UmmaPlan** out);
void umma_plan_destroy(cct_ctx* ctx, UmmaPlan* p);
size_t umma_plan_workspace_bytes(const UmmaPlan* p);
bool umma_supported(const ConvGeom& G);
// `batch` > 0 restricts a call to the first `batch` images of the tensors it is given; `repack` = rewrite the packed
// weight operand from W first (needed once per new W).
int umma_conv_forward(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* W, const float* bias, float* Y,
                      int relu, PhaseTimer* t, int batch = 0, bool repack = true);
int umma_conv_backward(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* W, const float* dY, float* dX,
                       float* dW, float* db, PhaseTimer* t);
int umma_conv_wgrad(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* dY, float* dW, float* db, PhaseTimer* t);
int umma_conv_dgrad(cct_ctx* ctx, UmmaPlan* p, const float* W, const float* dY, float* dX, PhaseTimer* t, int batch,
                    bool repack);

// ---- max pooling forward with the plane staged in shared memory (layers.cu)
int pool_relu_backward_pooled(cct_ctx* ctx, const float* P, const int32_t* idx, const float* dP, float* dA, int planes,
                              int n, int k, int s);
int maxpool_forward_staged(cct_ctx* ctx, const float* X, float* Y, int32_t* idx, int planes, int n, int m, int k, int s);
