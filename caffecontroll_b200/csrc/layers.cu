// The remaining CaffeNet bridges between the contractions, as HBM-bound kernels: local response normalisation
// (LRNBridge), dropout (DropoutBridge), softmax with loss (SoftmaxLossBridge) and max pooling forward with the plane
// staged in shared memory.  Each kernel notes the bytes it moves per element; grids are multiples of the SM count.
#include <float.h>

#include <algorithm>

#include "cct_internal.h"

namespace {

inline int ew_grid(cct_ctx* ctx, size_t work, int threads) {
  const size_t blocks = (work + threads - 1) / threads;
  return (int)std::max<size_t>(1, std::min<size_t>(blocks, (size_t)ctx->sm_count * 16));
}

// ---------------------------------------------------------------------------------------------------- LRN
// Across-channel normalisation (src/bridges/LRNBridge_impl.hxx:46-120, src/kernels/lrn.hxx:38-124):
//   scale[b][d][p] = 1 + (alpha / local_size) * sum_{|c - d| <= local_size / 2} X[b][c][p]^2,   Y = X / scale^beta.
// One thread per (image, chunk of kLrnChunk channels, position): consecutive threads read consecutive positions of one
// channel plane (coalesced), a thread walks over its chunk with the window's squares in registers and reads
// local_size / 2 channels of halo on either side (they come from L1 / L2: the neighbouring chunk's thread block reads
// them as its own).  Splitting the channels keeps the grid large on the late layers (13 x 13 planes).  4 B read + 8 B
// written per element (Y and scale; the backward pass reads scale instead of recomputing a nine-channel window).
constexpr int kLrnChunk = 16;
constexpr int kLrnBwdChunk = 8;

// One short-lived block of 128 threads per 128 items (the kernels' loops then run once): a thread's item is some sixty
// loads and stores long, and with a grid of a few blocks per SM looping over the items the last round left a third of
// the SMs idle (5 - 7 % of the kernel).
inline int lrn_grid(size_t items) { return (int)std::max<size_t>(1, std::min<size_t>((items + 127) / 128, 1u << 30)); }

// s^(-beta) for s >= 1: exp2(-beta log2 s) on the special-function units (ex2.approx / lg2.approx, each within ~2 ulp:
// relative error below 1e-6 for the scales and exponents of a normalisation layer, two orders under the path's tolerance;
// powf costs some thirty instructions and made these kernels compute-bound).
__device__ __forceinline__ float inv_pow(float s, float beta) { return exp2f(-beta * __log2f(s)); }

template <int LOCAL>
__global__ void __launch_bounds__(128) lrn_fwd_kernel(const float* __restrict__ X, float* __restrict__ Y,
                                                      float* __restrict__ scale, size_t items, int D, int chunks, int plane,
                                                      float alpha_over_size, float beta) {
  pdl_wait();
  constexpr int W = LOCAL / 2, SPAN = kLrnChunk + 2 * W;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < items; t += (size_t)gridDim.x * blockDim.x) {
    const size_t bc = t / plane, p = t - bc * plane;
    const size_t b = bc / chunks;
    const int d0 = (int)(bc - b * chunks) * kLrnChunk;
    const size_t base = b * (size_t)D * plane + p;
    // the chunk and its halo, all loads issued before the first use (a thread keeps SPAN requests in flight)
    float x[SPAN];
#pragma unroll
    for (int i = 0; i < SPAN; ++i) {
      const int c = d0 + i - W;
      x[i] = (c >= 0 && c < D) ? __ldg(X + base + (size_t)c * plane) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kLrnChunk; ++j) {
      const int d = d0 + j;
      if (d < D) {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < LOCAL; ++i) sum += x[j + i] * x[j + i];
        const float s = alpha_over_size * sum + 1.f;
        const size_t at = base + (size_t)d * plane;
        if (scale != nullptr) scale[at] = s;
        Y[at] = x[j + W] * inv_pow(s, beta);
      }
    }
  }
}

// Any odd window: the squares are re-read (they sit in L1 from the previous channels' steps).
__global__ void lrn_fwd_generic_kernel(const float* __restrict__ X, float* __restrict__ Y, float* __restrict__ scale,
                                       size_t items, int D, int chunks, int plane, int local, float alpha_over_size,
                                       float beta) {
  pdl_wait();
  const int w = local / 2;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < items; t += (size_t)gridDim.x * blockDim.x) {
    const size_t bc = t / plane, p = t - bc * plane;
    const size_t b = bc / chunks;
    const int d0 = (int)(bc - b * chunks) * kLrnChunk, d1 = min(D, d0 + kLrnChunk);
    const size_t base = b * (size_t)D * plane + p;
    for (int d = d0; d < d1; ++d) {
      float sum = 0.f;
      for (int c = max(0, d - w); c <= min(D - 1, d + w); ++c) {
        const float v = X[base + (size_t)c * plane];
        sum += v * v;
      }
      const float s = alpha_over_size * sum + 1.f;
      if (scale != nullptr) scale[base + (size_t)d * plane] = s;
      Y[base + (size_t)d * plane] = X[base + (size_t)d * plane] / powf(s, beta);
    }
  }
}

// LRNBridge::backward (src/kernels/lrn.hxx:134-180) as a gather: the reference scatters, for every output channel o,
//   dX[c] += dY[o] * ([c == o] / scale[o]^beta - 2 beta (alpha / size) X[o] X[c] / scale[o]^(beta + 1))   for |c - o| <= w;
// collected per input channel c:
//   dX[c] = dY[c] / scale[c]^beta - 2 beta (alpha / size) X[c] * sum_{|o - c| <= w} dY[o] Y[o] / scale[o].
// Same decomposition as the forward kernel, the window terms t[o] = dY[o] Y[o] / scale[o] held in registers.  Y is not
// read: Y[o] = X[o] * scale[o]^-beta is formed again with the forward kernel's own expression (one power per element of
// the chunk and its halo, on the special-function units), which costs less than a fourth stream from HBM.  HAVE_SCALE =
// false forms the scales again as well, from X with a halo twice as wide and the forward kernel's summation order, for
// callers that did not keep them: 8 B read + 4 B written per element against 12 + 4 with the scale cube.
template <int LOCAL, bool HAVE_SCALE>
__global__ void __launch_bounds__(128) lrn_bwd_kernel(const float* __restrict__ X, const float* __restrict__ scale,
                                                      const float* __restrict__ dY, float* __restrict__ dX, size_t items,
                                                      int D, int chunks, int plane, float alpha_over_size, float beta) {
  pdl_wait();
  constexpr int kLrnChunk = kLrnBwdChunk;  // several arrays are read here: a shorter chunk keeps the registers in check
  constexpr int W = LOCAL / 2, SPAN = kLrnChunk + 2 * W;
  constexpr int XW = HAVE_SCALE ? 0 : W, XSPAN = SPAN + 2 * XW;  // channels of X a thread reads: d0 - W - XW ...
  const float coef = 2.f * beta * alpha_over_size;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < items; t += (size_t)gridDim.x * blockDim.x) {
    const size_t bc = t / plane, p = t - bc * plane;
    const size_t b = bc / chunks;
    const int d0 = (int)(bc - b * chunks) * kLrnChunk;
    const size_t base = b * (size_t)D * plane + p;
    // every load of the chunk and its halo is issued before the first use
    float gy[SPAN], sc[SPAN], xx[XSPAN];
#pragma unroll
    for (int i = 0; i < SPAN; ++i) {
      const int c = d0 + i - W;
      const bool in = c >= 0 && c < D;
      const size_t at = base + (size_t)(in ? c : 0) * plane;
      gy[i] = in ? __ldg(dY + at) : 0.f;
      if (HAVE_SCALE) sc[i] = in ? __ldg(scale + at) : 1.f;
    }
#pragma unroll
    for (int i = 0; i < XSPAN; ++i) {
      const int c = d0 + i - W - XW;
      xx[i] = (c >= 0 && c < D) ? __ldg(X + base + (size_t)c * plane) : 0.f;
    }
    if (!HAVE_SCALE) {
#pragma unroll
      for (int i = 0; i < SPAN; ++i) {
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < LOCAL; ++q) sum += xx[i + q] * xx[i + q];
        sc[i] = alpha_over_size * sum + 1.f;
      }
    }
    float pw[SPAN], tt[SPAN];
#pragma unroll
    for (int i = 0; i < SPAN; ++i) {
      pw[i] = inv_pow(sc[i], beta);
      tt[i] = __fdividef(gy[i] * (xx[i + XW] * pw[i]), sc[i]);  // the window terms; xx * pw is Y as the forward pass wrote it
    }
#pragma unroll
    for (int j = 0; j < kLrnChunk; ++j) {
      if (d0 + j < D) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < LOCAL; ++i) acc += tt[j + i];
        dX[base + (size_t)(d0 + j) * plane] = gy[j + W] * pw[j + W] - coef * xx[j + W + XW] * acc;
      }
    }
  }
}

__global__ void lrn_bwd_generic_kernel(const float* __restrict__ X, const float* __restrict__ Y,
                                       const float* __restrict__ scale, const float* __restrict__ dY,
                                       float* __restrict__ dX, size_t items, int D, int chunks, int plane, int local,
                                       float alpha_over_size, float beta) {
  pdl_wait();
  const int w = local / 2;
  const float coef = 2.f * beta * alpha_over_size;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < items; t += (size_t)gridDim.x * blockDim.x) {
    const size_t bc = t / plane, p = t - bc * plane;
    const size_t b = bc / chunks;
    const int d0 = (int)(bc - b * chunks) * kLrnChunk, d1 = min(D, d0 + kLrnChunk);
    const size_t base = b * (size_t)D * plane + p;
    for (int c = d0; c < d1; ++c) {
      float acc = 0.f;
      for (int o = max(0, c - w); o <= min(D - 1, c + w); ++o) {
        const size_t at = base + (size_t)o * plane;
        acc += dY[at] * Y[at] / scale[at];
      }
      const size_t at = base + (size_t)c * plane;
      dX[at] = dY[at] / powf(scale[at], beta) - coef * X[at] * acc;
    }
  }
}

// ------------------------------------------------------------------------------------------------ dropout
// DropoutBridge forward in training and backward (src/bridges/DropoutBridge_impl.hxx:71-74, 150-170): the same
// element-wise product with the mask (one unsigned int per element, non-zero = keep) and the scale 1 / (1 - ratio).
__global__ void dropout_kernel(const float* __restrict__ in, const uint32_t* __restrict__ mask, float scale,
                               float* __restrict__ out, size_t count) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    out[i] = in[i] * (float)(mask[i] != 0u) * scale;
}

// A fresh keep / drop mask on the device: element i of stream (seed, call) keeps its value with probability
// 1 - ratio.  Counter-based (a 64-bit mix of seed, call counter and index), so the result does not depend on the grid
// and a (seed, call) pair reproduces its mask.  The reference's GPU path thresholds cuRAND integers the same way
// (src/bridges/DropoutBridge_impl.hxx:100-104); its CPU path draws from boost::bernoulli on mt19937 - masks differ
// between the two there as well, which is why parity runs inject the CPU oracle's mask instead.
__global__ void dropout_mask_kernel(uint32_t* __restrict__ mask, size_t count, uint32_t threshold, uint64_t key) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
    uint64_t z = key + (uint64_t)i * 0x9E3779B97F4A7C15ull;  // splitmix64 finaliser
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    mask[i] = (uint32_t)(z >> 32) >= threshold ? 1u : 0u;
  }
}

// -------------------------------------------------------------------------------------------- softmax loss
// SoftmaxLossBridge (src/kernels/softmax.hxx:17-50): per image prob = exp(x - max) / sum, loss -= log(max(prob[label],
// FLT_MIN)).  One warp per image; the per-image losses are added in image order by one thread afterwards, so the
// result does not depend on the grid.  Labels are floats, as in the reference's label cube.
__global__ void softmax_fwd_kernel(const float* __restrict__ X, const float* __restrict__ labels, float* __restrict__ prob,
                                   float* __restrict__ image_loss, int B, int C) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int img = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5);
  if (img >= B) return;
  const float* x = X + (size_t)img * C;
  float* pr = prob + (size_t)img * C;
  float mx = -FLT_MAX;
  for (int i = lane; i < C; i += 32) mx = fmaxf(mx, x[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int i = lane; i < C; i += 32) sum += expf(x[i] - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  for (int i = lane; i < C; i += 32) pr[i] = expf(x[i] - mx) / sum;
  __syncwarp();
  if (lane == 0) {
    const int label = (int)labels[img];
    const float p = (label >= 0 && label < C) ? expf(x[label] - mx) / sum : 0.f;
    image_loss[img] = -logf(fmaxf(p, FLT_MIN));
  }
}

__global__ void sum_in_order_kernel(const float* __restrict__ v, float* __restrict__ out, int n) {
  pdl_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    float acc = 0.f;
    for (int i = 0; i < n; ++i) acc += v[i];
    *out = acc;
  }
}

// Gradient of the loss with respect to the bridge's input (src/kernels/softmax.hxx:62-80):
// dX = (prob - onehot(label)) * scale, scale = 1 / (batch the loss is averaged over).
__global__ void softmax_bwd_kernel(const float* __restrict__ prob, const float* __restrict__ labels,
                                   float* __restrict__ dX, size_t total, int C, float scale) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t img = i / C;
    const int c = (int)(i - img * C);
    dX[i] = (prob[i] - (c == (int)labels[img] ? 1.f : 0.f)) * scale;
  }
}

// ----------------------------------------------------------------------------- max pooling forward, staged
// MaxPoolingBridge::forward (src/sched/DeviceDriver_CPU.cpp:369-400): rows then columns, strict '>' so the first maximum
// wins; idx = offset inside the plane.  Output size by floor and no padding, so every window lies inside the plane
// ((m - 1) s + k <= n) and no clipping is needed.  One block per plane at a time: the plane is copied to shared memory
// with coalesced loads (every input element crosses HBM -> SM once, four loads in flight per thread), the windows are
// read from there, Y and idx leave in coalesced runs.  K, S > 0 fix the window at compile time (straight-line
// compare / select chain); K = 0 keeps run-time loops.  4 B read per input element + 8 B written per output element.
constexpr int kPoolFetch = 12;  // 256 * 12 elements: one 55 x 55 plane, four 27 x 27, sixteen 13 x 13
template <int K, int S>
__global__ void __launch_bounds__(256) maxpool_fwd_staged_kernel(const float* __restrict__ X, float* __restrict__ Y,
                                                                 int32_t* __restrict__ idx, int planes, int n, int m,
                                                                 int k_rt, int s_rt, int group) {
  pdl_wait();
  // `group` consecutive planes (contiguous in memory) are staged and pooled together, so that small planes (13 x 13)
  // still give every thread of the block work.
  extern __shared__ float plane_smem[];
  const int nn = n * n, mm = m * m;
  const int k = K > 0 ? K : k_rt, s = S > 0 ? S : s_rt;
  // Groups of up to 256 * kPoolFetch elements travel through registers: the next group's loads are issued before the
  // current group's windows are evaluated, so they are in flight during the compare chains and the stores.
  const bool via_regs = group * nn <= 256 * kPoolFetch;
  float r[kPoolFetch];
  auto fetch = [&](int p0) {
    const int total_in = min(group, planes - p0) * nn;
    const float* in = X + (size_t)p0 * nn;
#pragma unroll
    for (int j = 0; j < kPoolFetch; ++j) {
      const int i = threadIdx.x + j * 256;
      r[j] = i < total_in ? __ldg(in + i) : 0.f;
    }
  };
  if (via_regs && (int)blockIdx.x * group < planes) fetch(blockIdx.x * group);
  for (int p0 = blockIdx.x * group; p0 < planes; p0 += gridDim.x * group) {
    const int g = min(group, planes - p0);
    const float* in = X + (size_t)p0 * nn;
    const int total_in = g * nn, total_out = g * mm;
    __syncthreads();  // the previous group's windows have been read
    if (via_regs) {
#pragma unroll
      for (int j = 0; j < kPoolFetch; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < total_in) plane_smem[i] = r[j];
      }
      __syncthreads();
      const int next = p0 + gridDim.x * group;
      if (next < planes) fetch(next);
    } else {
      int i = threadIdx.x;
      for (; i + 3 * 256 < total_in; i += 4 * 256) {
        const float a = __ldg(in + i), b = __ldg(in + i + 256), c = __ldg(in + i + 512), d = __ldg(in + i + 768);
        plane_smem[i] = a; plane_smem[i + 256] = b; plane_smem[i + 512] = c; plane_smem[i + 768] = d;
      }
      for (; i < total_in; i += 256) plane_smem[i] = __ldg(in + i);
      __syncthreads();
    }
    for (int t = threadIdx.x; t < total_out; t += 256) {
      const int pl = t / mm, r = t - pl * mm;
      const int ph = r / m, pw = r - ph * m;
      const int origin = ph * s * n + pw * s;
      const float* win = plane_smem + pl * nn + origin;
      float best = -FLT_MAX;
      int where = 0;
      if (K > 0) {
#pragma unroll
        for (int h = 0; h < K; ++h)
#pragma unroll
          for (int w = 0; w < K; ++w) {
            const float v = win[h * n + w];
            const bool better = v > best;
            best = better ? v : best;
            where = better ? h * n + w : where;
          }
      } else {
        for (int h = 0; h < k; ++h)
          for (int w = 0; w < k; ++w) {
            const float v = win[h * n + w];
            if (v > best) { best = v; where = h * n + w; }
          }
      }
      Y[(size_t)p0 * mm + t] = best;
      idx[(size_t)p0 * mm + t] = origin + where;
    }
  }
}

}  // namespace

int maxpool_forward_staged(cct_ctx* ctx, const float* X, float* Y, int32_t* idx, int planes, int n, int m, int k, int s) {
  const size_t plane_bytes = (size_t)n * n * sizeof(float);
  if (plane_bytes > 200 * 1024) return CCT_ERR_UNSUPPORTED;
  const int group = (int)std::max<size_t>(1, std::min<size_t>(16, (12 * 1024) / plane_bytes));  // ~12 KB staged per block
  const size_t smem = plane_bytes * group;
  auto kernel = (k == 3 && s == 2) ? maxpool_fwd_staged_kernel<3, 2> : (k == 2 && s == 2) ? maxpool_fwd_staged_kernel<2, 2>
                                                                                         : maxpool_fwd_staged_kernel<0, 0>;
  if (smem > 48 * 1024) CCT_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / std::max<size_t>(smem, 1)));
  const int blocks_needed = (planes + group - 1) / group;
  const int grid = std::max(1, std::min(blocks_needed, ctx->sm_count * per_sm));
  launch_pdl(kernel, dim3(grid), dim3(256), smem, ctx->stream, X, Y, idx, planes, n, m, k, s, group);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

extern "C" {

int cct_lrn_forward(cct_ctx* ctx, const float* X, float* Y, float* scale, int batch, int depth, int plane, int local_size,
                    float alpha, float beta) {
  if (!ctx || !X || !Y || batch <= 0 || depth <= 0 || plane <= 0 || local_size <= 0 || !(local_size & 1))
    return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const int chunks = (depth + kLrnChunk - 1) / kLrnChunk;
  const size_t items = (size_t)batch * chunks * plane;
  const int grid = lrn_grid(items);
  const float aos = alpha / (float)local_size;
  if (local_size == 5)
    launch_pdl(lrn_fwd_kernel<5>, dim3(grid), dim3(128), 0, ctx->stream, X, Y, scale, items, depth, chunks, plane, aos, beta);
  else if (local_size == 3)
    launch_pdl(lrn_fwd_kernel<3>, dim3(grid), dim3(128), 0, ctx->stream, X, Y, scale, items, depth, chunks, plane, aos, beta);
  else
    launch_pdl(lrn_fwd_generic_kernel, dim3(grid), dim3(128), 0, ctx->stream, X, Y, scale, items, depth, chunks, plane, local_size, aos, beta);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_lrn_backward(cct_ctx* ctx, const float* X, const float* Y, const float* scale, const float* dY, float* dX,
                     int batch, int depth, int plane, int local_size, float alpha, float beta) {
  if (!ctx || !X || !dY || !dX || batch <= 0 || depth <= 0 || plane <= 0 || local_size <= 0 || !(local_size & 1))
    return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const bool fixed = local_size == 5 || local_size == 3;
  if (!fixed && (!Y || !scale)) {
    ctx->last_error = "windows other than 3 and 5 channels need the output and the scale cube of the forward pass";
    return CCT_ERR_UNSUPPORTED;
  }
  const int chunk = fixed ? kLrnBwdChunk : kLrnChunk;
  const int chunks = (depth + chunk - 1) / chunk;
  const size_t items = (size_t)batch * chunks * plane;
  const int grid = lrn_grid(items);
  const float aos = alpha / (float)local_size;
  auto go = [&](auto kernel) {
    launch_pdl(kernel, dim3(grid), dim3(128), 0, ctx->stream, X, scale, dY, dX, items, depth, chunks, plane, aos, beta);
  };
  if (local_size == 5) {
    if (scale) go(lrn_bwd_kernel<5, true>); else go(lrn_bwd_kernel<5, false>);
  } else if (local_size == 3) {
    if (scale) go(lrn_bwd_kernel<3, true>); else go(lrn_bwd_kernel<3, false>);
  } else {
    launch_pdl(lrn_bwd_generic_kernel, dim3(grid), dim3(128), 0, ctx->stream, X, Y, scale, dY, dX, items, depth, chunks, plane, local_size, aos,
                                                        beta);
  }
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_dropout_apply(cct_ctx* ctx, const float* in, const uint32_t* mask, float scale, float* out, size_t count) {
  if (!ctx || !in || !mask || !out) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(dropout_kernel, dim3(ew_grid(ctx, count, 256)), dim3(256), 0, ctx->stream, in, mask, scale, out, count);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_dropout_mask(cct_ctx* ctx, uint32_t* mask, size_t count, float ratio, uint64_t seed, uint64_t call) {
  if (!ctx || !mask || !(ratio >= 0.f && ratio < 1.f)) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const uint32_t threshold = (uint32_t)std::min(4294967295.0, (double)ratio * 4294967296.0);
  const uint64_t key = (seed * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull) ^ (call * 0xDA942042E4DD58B5ull);
  launch_pdl(dropout_mask_kernel, dim3(ew_grid(ctx, count, 256)), dim3(256), 0, ctx->stream, mask, count, threshold, key);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_softmax_loss_forward(cct_ctx* ctx, const float* X, const float* labels, float* prob, float* image_loss,
                             float* loss, int batch, int classes) {
  if (!ctx || !X || !labels || !prob || !image_loss || !loss || batch <= 0 || classes <= 0) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(softmax_fwd_kernel, dim3((batch + 3) / 4), dim3(128), 0, ctx->stream, X, labels, prob, image_loss, batch, classes);
  CCT_CHECK_LAUNCH(ctx);
  launch_pdl(sum_in_order_kernel, dim3(1), dim3(32), 0, ctx->stream, image_loss, loss, batch);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_softmax_loss_backward(cct_ctx* ctx, const float* prob, const float* labels, float* dX, int batch, int classes,
                              float scale) {
  if (!ctx || !prob || !labels || !dX || batch <= 0 || classes <= 0) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const size_t total = (size_t)batch * classes;
  launch_pdl(softmax_bwd_kernel, dim3(ew_grid(ctx, total, 256)), dim3(256), 0, ctx->stream, prob, labels, dX, total, classes, scale);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

}  // extern "C"
