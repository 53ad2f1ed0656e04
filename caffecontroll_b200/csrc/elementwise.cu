// Memory-bound companions of the convolution path: constant fill, fused SGD step, ReLU, max pooling and the
// combined pooling+ReLU backward mask.  All are grid-stride kernels sized to a multiple of the SM count; each is
// bounded by HBM bandwidth (bytes per element noted at each kernel).
#include <float.h>

#include "cct_internal.h"

namespace {

inline int grid_for(cct_ctx* ctx, size_t work, int threads) {
  size_t blocks = (work + threads - 1) / threads;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// 4 B written per element.
__global__ void fill_kernel(float* __restrict__ p, size_t count, float v) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    p[i] = v;
}

// 12 B read + 12 B written per parameter (g is written back only when decay is on: the reference's updater adds
// the decay term into the gradient buffer itself).
__global__ void sgd_kernel(size_t count, float* __restrict__ w, float* __restrict__ g, float* __restrict__ h,
                           float lr, float momentum, float lambda) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
    float gi = g[i];
    const float wi = w[i];
    if (lambda != 0.f) {
      gi = __fadd_rn(gi, __fmul_rn(lambda, wi));  // saxpy: separate multiply and add, as BLAS does without FMA contraction
      g[i] = gi;
    }
    const float hi = __fadd_rn(__fmul_rn(lr, gi), __fmul_rn(momentum, h[i]));
    h[i] = hi;
    w[i] = __fadd_rn(wi, -hi);
  }
}

__global__ void relu_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, size_t count) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    y[i] = fmaxf(x[i], 0.f);
}

// dy and dx may be the same buffer (in-place use by the fused backward of the SIMT path).
__global__ void relu_bwd_kernel(const float* __restrict__ x, const float* dy, float* dx, size_t count) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    dx[i] = dy[i] * (x[i] > 0.f ? 1.f : 0.f);
}

// One thread per pooled element; rows then columns, strict '>' so the first maximum wins.
__global__ void maxpool_fwd_kernel(const float* __restrict__ X, float* __restrict__ Y, int32_t* __restrict__ idx,
                                   int planes, int n, int m, int k, int s) {
  const size_t total = (size_t)planes * m * m;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int pw = (int)(t % m), ph = (int)((t / m) % m);
    const size_t plane = t / ((size_t)m * m);
    const float* in = X + plane * n * n;
    const int he = min(ph * s + k, n), we = min(pw * s + k, n);
    float best = -FLT_MAX;
    int where = 0;
    for (int h = ph * s; h < he; ++h)
      for (int w = pw * s; w < we; ++w) {
        const float v = in[h * n + w];
        if (v > best) { best = v; where = h * n + w; }
      }
    Y[t] = best;
    idx[t] = where;
  }
}

// Gather form of "zero-fill, then dX[idx] += dY in (ph, pw) order": each input element visits the windows that
// cover it in the same order, so the fp32 sum is the same.  RELU additionally multiplies by (A > 0).
template <bool RELU>
__global__ void maxpool_bwd_kernel(const float* __restrict__ A, const int32_t* __restrict__ idx,
                                   const float* __restrict__ dP, float* __restrict__ dA, int planes, int n, int m,
                                   int k, int s) {
  const size_t total = (size_t)planes * n * n;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int w = (int)(t % n), h = (int)((t / n) % n);
    const size_t plane = t / ((size_t)n * n);
    float acc = 0.f;
    bool live = true;
    if (RELU) live = A[t] > 0.f;
    if (live) {
      const int here = h * n + w;
      const int ph0 = h < k ? 0 : (h - k) / s + 1, pw0 = w < k ? 0 : (w - k) / s + 1;
      const int ph1 = min(h / s, m - 1), pw1 = min(w / s, m - 1);
      const int32_t* ip = idx + plane * m * m;
      const float* gp = dP + plane * m * m;
      for (int ph = ph0; ph <= ph1; ++ph)
        for (int pw = pw0; pw <= pw1; ++pw)
          if (ip[ph * m + pw] == here) acc += gp[ph * m + pw];
    }
    dA[t] = acc;
  }
}

}  // namespace

extern "C" {

int cct_fill_f32(cct_ctx* ctx, float* dptr, size_t count, float value) {
  if (!ctx || (!dptr && count)) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  fill_kernel<<<grid_for(ctx, count, 256), 256, 0, ctx->stream>>>(dptr, count, value);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_sgd_step(cct_ctx* ctx, size_t count, float* w, float* g, float* h, float lr, float momentum, float lambda) {
  if (!ctx || !w || !g || !h) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  sgd_kernel<<<grid_for(ctx, count, 256), 256, 0, ctx->stream>>>(count, w, g, h, lr, momentum, lambda);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_relu_forward(cct_ctx* ctx, const float* X, float* Y, size_t count) {
  if (!ctx || !X || !Y) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  relu_fwd_kernel<<<grid_for(ctx, count, 256), 256, 0, ctx->stream>>>(X, Y, count);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_relu_backward(cct_ctx* ctx, const float* X, const float* dY, float* dX, size_t count) {
  if (!ctx || !X || !dY || !dX) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  relu_bwd_kernel<<<grid_for(ctx, count, 256), 256, 0, ctx->stream>>>(X, dY, dX, count);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

static int pool_args_ok(int planes, int n, int k, int s) { return planes > 0 && n > 0 && k > 0 && s > 0 && k <= n; }

int cct_maxpool_forward(cct_ctx* ctx, const float* X, float* Y, int32_t* idx, int planes, int n, int k, int s) {
  if (!ctx || !X || !Y || !idx || !pool_args_ok(planes, n, k, s)) return CCT_ERR_INVALID;
  const int m = (n - k) / s + 1;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  maxpool_fwd_kernel<<<grid_for(ctx, (size_t)planes * m * m, 256), 256, 0, ctx->stream>>>(X, Y, idx, planes, n, m, k,
                                                                                        s);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_maxpool_backward(cct_ctx* ctx, const float* dY, const int32_t* idx, float* dX, int planes, int n, int k,
                         int s) {
  if (!ctx || !dY || !idx || !dX || !pool_args_ok(planes, n, k, s)) return CCT_ERR_INVALID;
  const int m = (n - k) / s + 1;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  maxpool_bwd_kernel<false><<<grid_for(ctx, (size_t)planes * n * n, 256), 256, 0, ctx->stream>>>(nullptr, idx, dY, dX,
                                                                                                planes, n, m, k, s);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_pool_relu_backward(cct_ctx* ctx, const float* A, const int32_t* idx, const float* dP, float* dA, int planes,
                           int n, int k, int s) {
  if (!ctx || !A || !idx || !dP || !dA || !pool_args_ok(planes, n, k, s)) return CCT_ERR_INVALID;
  const int m = (n - k) / s + 1;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  maxpool_bwd_kernel<true><<<grid_for(ctx, (size_t)planes * n * n, 256), 256, 0, ctx->stream>>>(A, idx, dP, dA, planes,
                                                                                               n, m, k, s);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

}  // extern "C"
