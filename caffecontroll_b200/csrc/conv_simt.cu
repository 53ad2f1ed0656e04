// Direct convolution in fp32 FMA arithmetic (CCT_ALGO_SIMT_FP32).
//
// CCT_ALGO_AUTO picks it only where the tcgen05 path does not apply (kernels wider than 15, tables beyond shared
// memory); tests ask for it by name as a second on-device implementation to cross-check the tcgen05 path at full size.  Every output element is reduced by one thread (forward,
// data gradient) or one thread block (weight and bias gradients) in a fixed order, so results are deterministic.
#include "cct_internal.h"

namespace {

constexpr int kOcPerThread = 4;

// Y[b][o][r][c]: one thread per output pixel and kOcPerThread consecutive filters.
__global__ void simt_forward_kernel(const float* __restrict__ X, const float* __restrict__ W,
                                    const float* __restrict__ bias, float* __restrict__ Y, ConvGeom G, int relu) {
  pdl_wait();
  const int mm = G.m * G.m;
  const int ocb_per_group = (G.og + kOcPerThread - 1) / kOcPerThread;
  const long long total = (long long)G.B * G.g * ocb_per_group * mm;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int pix = (int)(t % mm);
    long long rest = t / mm;
    const int ocb = (int)(rest % ocb_per_group);
    rest /= ocb_per_group;
    const int gi = (int)(rest % G.g);
    const int b = (int)(rest / G.g);
    const int r = pix / G.m, c = pix % G.m;
    const int o0 = gi * G.og + ocb * kOcPerThread;
    const int o_lim = min(kOcPerThread, G.og - ocb * kOcPerThread);
    float acc[kOcPerThread];
#pragma unroll
    for (int j = 0; j < kOcPerThread; ++j) acc[j] = 0.f;
    const int kk = G.k * G.k;
    for (int d = 0; d < G.Dg; ++d) {
      const float* xp = X + ((size_t)b * G.D + gi * G.Dg + d) * G.n * G.n;
      for (int kr = 0; kr < G.k; ++kr) {
        const int y = r * G.s - G.p + kr;
        if ((unsigned)y >= (unsigned)G.n) continue;
        for (int kc = 0; kc < G.k; ++kc) {
          const int x = c * G.s - G.p + kc;
          if ((unsigned)x >= (unsigned)G.n) continue;
          const float v = xp[y * G.n + x];
#pragma unroll
          for (int j = 0; j < kOcPerThread; ++j)
            if (j < o_lim) acc[j] = fmaf(W[((size_t)(o0 + j) * G.Dg + d) * kk + kr * G.k + kc], v, acc[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kOcPerThread; ++j)
      if (j < o_lim) {
        float v = acc[j] + (bias ? bias[o0 + j] : 0.f);
        if (relu) v = fmaxf(v, 0.f);
        Y[((size_t)b * G.o + o0 + j) * mm + pix] = v;
      }
  }
}

// dX[b][d][y][x] = sum over filters and taps that touch (y, x): the inverse lowering written as a gather, so no
// two threads add to the same address.
__global__ void simt_dgrad_kernel(const float* __restrict__ W, const float* __restrict__ dY, float* __restrict__ dX,
                                  ConvGeom G) {
  pdl_wait();
  const int nn = G.n * G.n, mm = G.m * G.m, kk = G.k * G.k;
  const long long total = (long long)G.B * G.D * nn;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int pix = (int)(t % nn);
    const int d = (int)((t / nn) % G.D);
    const int b = (int)(t / ((long long)nn * G.D));
    const int y = pix / G.n, x = pix % G.n;
    const int gi = d / G.Dg, dl = d % G.Dg;
    float acc = 0.f;
    for (int kr = 0; kr < G.k; ++kr) {
      const int ty = y + G.p - kr;
      if (ty < 0 || ty % G.s) continue;
      const int r = ty / G.s;
      if (r >= G.m) continue;
      for (int kc = 0; kc < G.k; ++kc) {
        const int tx = x + G.p - kc;
        if (tx < 0 || tx % G.s) continue;
        const int c = tx / G.s;
        if (c >= G.m) continue;
        const float* wp = W + ((size_t)(gi * G.og) * G.Dg + dl) * kk + kr * G.k + kc;
        const float* gp = dY + ((size_t)b * G.o + gi * G.og) * mm + r * G.m + c;
        for (int o = 0; o < G.og; ++o) acc = fmaf(wp[(size_t)o * G.Dg * kk], gp[(size_t)o * mm], acc);
      }
    }
    dX[t] = acc;
  }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = v;
  __syncthreads();
  float total = 0.f;
  if (threadIdx.x == 0)
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += red[i];
  __syncthreads();
  return total;
}

// dW[o][d][kr][kc]: one block per element, fixed reduction tree.
__global__ void simt_wgrad_kernel(const float* __restrict__ X, const float* __restrict__ dY, float* __restrict__ dW,
                                  ConvGeom G) {
  pdl_wait();
  __shared__ float red[32];
  const int kk = G.k * G.k, mm = G.m * G.m;
  const size_t e = blockIdx.x;  // index into [o][Dg][k][k]
  const int kc = (int)(e % G.k), kr = (int)((e / G.k) % G.k);
  const int dl = (int)((e / kk) % G.Dg);
  const int o = (int)(e / ((size_t)kk * G.Dg));
  const int gi = o / G.og;
  float acc = 0.f;
  const long long total = (long long)G.B * mm;
  for (long long t = threadIdx.x; t < total; t += blockDim.x) {
    const int pix = (int)(t % mm);
    const int b = (int)(t / mm);
    const int r = pix / G.m, c = pix % G.m;
    const int y = r * G.s - G.p + kr, x = c * G.s - G.p + kc;
    if ((unsigned)y < (unsigned)G.n && (unsigned)x < (unsigned)G.n)
      acc = fmaf(dY[((size_t)b * G.o + o) * mm + pix],
                 X[(((size_t)b * G.D + gi * G.Dg + dl) * G.n + y) * G.n + x], acc);
  }
  const float total_sum = block_sum(acc, red);
  if (threadIdx.x == 0) dW[e] = total_sum;
}

__global__ void simt_bgrad_kernel(const float* __restrict__ dY, float* __restrict__ db, ConvGeom G) {
  pdl_wait();
  __shared__ float red[32];
  const int mm = G.m * G.m;
  const int o = blockIdx.x;
  float acc = 0.f;
  const long long total = (long long)G.B * mm;
  for (long long t = threadIdx.x; t < total; t += blockDim.x) {
    const int pix = (int)(t % mm);
    const int b = (int)(t / mm);
    acc += dY[((size_t)b * G.o + o) * mm + pix];
  }
  const float total_sum = block_sum(acc, red);
  if (threadIdx.x == 0) db[o] = total_sum;
}

int grid_for(long long work, int threads, int sm_count) {
  long long blocks = (work + threads - 1) / threads;
  const long long cap = (long long)sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

int simt_conv_forward(cct_ctx* ctx, const ConvGeom& G, const float* X, const float* W, const float* bias, float* Y,
                      int relu, PhaseTimer* t) {
  const int ocb = (G.og + kOcPerThread - 1) / kOcPerThread;
  const long long work = (long long)G.B * G.g * ocb * G.m * G.m;
  t->begin(0, ctx->stream);
  launch_pdl(simt_forward_kernel, dim3(grid_for(work, 256, ctx->sm_count)), dim3(256), 0, ctx->stream, X, W, G.bias ? bias : nullptr, Y,
                                                                                  G, relu);
  t->end(0, ctx->stream);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int simt_conv_backward(cct_ctx* ctx, const ConvGeom& G, const float* X, const float* W, const float* dY, float* dX,
                       float* dW, float* db, PhaseTimer* t) {
  if (G.bias && db) {
    launch_pdl(simt_bgrad_kernel, dim3(G.o), dim3(256), 0, ctx->stream, dY, db, G);
    CCT_CHECK_LAUNCH(ctx);
  }
  if (dX) {
    const long long work = (long long)G.B * G.D * G.n * G.n;
    t->begin(3, ctx->stream);
    launch_pdl(simt_dgrad_kernel, dim3(grid_for(work, 256, ctx->sm_count)), dim3(256), 0, ctx->stream, W, dY, dX, G);
    t->end(3, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  }
  const size_t nw = (size_t)G.o * G.Dg * G.k * G.k;
  t->begin(1, ctx->stream);
  launch_pdl(simt_wgrad_kernel, dim3((unsigned)nw), dim3(256), 0, ctx->stream, X, dY, dW, G);
  t->end(1, ctx->stream);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}
