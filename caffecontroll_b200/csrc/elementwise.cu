// Memory-bound companions of the convolution path: constant fill, fused SGD step, ReLU, max pooling and the
// combined pooling+ReLU backward mask.  All are grid-stride kernels sized to a multiple of the SM count; each is
// bounded by HBM bandwidth (bytes per element noted at each kernel).
#include <float.h>

#include <algorithm>
#include <initializer_list>

#include "cct_internal.h"

namespace {

inline int grid_for(cct_ctx* ctx, size_t work, int threads) {
  size_t blocks = (work + threads - 1) / threads;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// Magic for fast_div: valid when max_x * d < 2^32 and d > 1, else 0 (plain division).
inline uint32_t fast_div_magic(uint64_t max_x, uint32_t d) {
  return (d > 1 && max_x * d < (1ull << 32)) ? (uint32_t)((1ull << 32) / d) + 1u : 0u;
}

// Blocks for the per-plane kernels: a multiple of the SM count, at most one block per plane.
inline int plane_grid(cct_ctx* ctx, int planes) { return std::max(1, std::min(planes, ctx->sm_count * 8)); }

// 4 B written per element.
__global__ void fill_kernel(float* __restrict__ p, size_t count, float v) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    p[i] = v;
}

// The streaming kernels move four floats per thread and iteration (16-byte accesses) when every buffer is 16-byte
// aligned, so that enough bytes are in flight per SM to approach the HBM rate; the last count % 4 elements, and all
// of them for unaligned buffers, go through the scalar loop that follows.  Per-element arithmetic is identical.
__device__ __forceinline__ float sgd_one(float& gi, float wi, float& hi_io, float lr, float momentum, float lambda) {
  if (lambda != 0.f) gi = __fadd_rn(gi, __fmul_rn(lambda, wi));  // saxpy: separate multiply and add, as BLAS does without FMA contraction
  hi_io = __fadd_rn(__fmul_rn(lr, gi), __fmul_rn(momentum, hi_io));
  return __fadd_rn(wi, -hi_io);
}

// 12 B read + 12 B written per parameter (g is written back only when decay is on: the reference's updater adds
// the decay term into the gradient buffer itself).
__global__ void sgd_kernel(size_t count, size_t vec, float* __restrict__ w, float* __restrict__ g, float* __restrict__ h,
                           float lr, float momentum, float lambda) {
  pdl_wait();
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  float4* w4 = reinterpret_cast<float4*>(w);
  float4* g4 = reinterpret_cast<float4*>(g);
  float4* h4 = reinterpret_cast<float4*>(h);
  for (size_t i = tid; i < vec; i += nthreads) {
    float4 gi = g4[i], hi = h4[i];
    const float4 wi = w4[i];
    float4 wo;
    wo.x = sgd_one(gi.x, wi.x, hi.x, lr, momentum, lambda);
    wo.y = sgd_one(gi.y, wi.y, hi.y, lr, momentum, lambda);
    wo.z = sgd_one(gi.z, wi.z, hi.z, lr, momentum, lambda);
    wo.w = sgd_one(gi.w, wi.w, hi.w, lr, momentum, lambda);
    if (lambda != 0.f) g4[i] = gi;
    h4[i] = hi;
    w4[i] = wo;
  }
  for (size_t i = 4 * vec + tid; i < count; i += nthreads) {
    float gi = g[i], hi = h[i];
    const float wo = sgd_one(gi, w[i], hi, lr, momentum, lambda);
    if (lambda != 0.f) g[i] = gi;
    h[i] = hi;
    w[i] = wo;
  }
}

// y = alpha x + beta y (12 B moved per element): the saxpy / saxpby calls of the reference's SGD updater
// (src/algorithms/GradientUpdater.h:163-181), for callers that keep its three-call update.
__global__ void saxpby_kernel(size_t count, float alpha, const float* __restrict__ x, float beta, float* __restrict__ y) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    y[i] = __fadd_rn(__fmul_rn(alpha, x[i]), __fmul_rn(beta, y[i]));
}

// g += lambda * sign(w) with sign(0) = -1: DeviceDriver::L1_update as the host driver computes it
// (src/sched/DeviceDriver_CPU.cpp:111-117), the L1 branch of the SGD updater.
__global__ void l1_update_kernel(size_t count, float* __restrict__ g, float lambda, const float* __restrict__ w) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    g[i] = __fadd_rn(g[i], w[i] > 0.f ? lambda : -lambda);
}

__global__ void relu_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, size_t count, size_t vec) {
  pdl_wait();
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  for (size_t i = tid; i < vec; i += nthreads) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<float4*>(y)[i] = make_float4(fmaxf(v.x, 0.f), fmaxf(v.y, 0.f), fmaxf(v.z, 0.f), fmaxf(v.w, 0.f));
  }
  for (size_t i = 4 * vec + tid; i < count; i += nthreads) y[i] = fmaxf(x[i], 0.f);
}

// dy and dx may be the same buffer (in-place use by the fused backward of the SIMT path).
__global__ void relu_bwd_kernel(const float* __restrict__ x, const float* dy, float* dx, size_t count, size_t vec) {
  pdl_wait();
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  for (size_t i = tid; i < vec; i += nthreads) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    const float4 d = reinterpret_cast<const float4*>(dy)[i];
    reinterpret_cast<float4*>(dx)[i] = make_float4(d.x * (v.x > 0.f ? 1.f : 0.f), d.y * (v.y > 0.f ? 1.f : 0.f),
                                                   d.z * (v.z > 0.f ? 1.f : 0.f), d.w * (v.w > 0.f ? 1.f : 0.f));
  }
  for (size_t i = 4 * vec + tid; i < count; i += nthreads) dx[i] = dy[i] * (x[i] > 0.f ? 1.f : 0.f);
}

// Number of float4 groups the streaming kernels may take: all of count / 4 when every pointer is 16-byte aligned.
inline size_t vec_groups(size_t count, std::initializer_list<const void*> ptrs) {
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15u) return 0;
  return count / 4;
}

// One block per plane at a time (planes are small: 13x13 ... 55x55), so all index arithmetic is 32-bit and the
// plane offset is the only 64-bit product.  Rows then columns, strict '>' so the first maximum wins.
__global__ void maxpool_fwd_kernel(const float* __restrict__ X, float* __restrict__ Y, int32_t* __restrict__ idx,
                                   int planes, int n, int m, int k, int s) {
  pdl_wait();
  const int mm = m * m;
  for (int plane = blockIdx.x; plane < planes; plane += gridDim.x) {
    const float* in = X + (size_t)plane * n * n;
    for (int t = threadIdx.x; t < mm; t += blockDim.x) {
      const int ph = t / m, pw = t - ph * m;
      const int he = min(ph * s + k, n), we = min(pw * s + k, n);
      float best = -FLT_MAX;
      int where = 0;
      for (int h = ph * s; h < he; ++h)
        for (int w = pw * s; w < we; ++w) {
          const float v = in[h * n + w];
          if (v > best) { best = v; where = h * n + w; }
        }
      Y[(size_t)plane * mm + t] = best;
      idx[(size_t)plane * mm + t] = where;
    }
  }
}

// x / d for x * d < 2^32 as one multiply-high: inv = floor(2^32 / d) + 1 (host side, fast_div_magic); inv == 0 means
// "divide".  The GPU has no integer divider, and these kernels would otherwise spend more on index arithmetic than on
// memory.
__device__ __forceinline__ uint32_t fast_div(uint32_t x, uint32_t d, uint32_t inv) {
  return inv ? __umulhi(x, inv) : x / d;
}

// Gather form of "zero-fill, then dX[idx] += dY in (ph, pw) order": each input element visits the windows that
// cover it in the same order, so the fp32 sum is the same.  RELU additionally multiplies by (A > 0).
// One warp per plane at a time, eight elements per lane with their loads issued together; the pooled indices and
// gradients (each read by up to ceil(k/s)^2 elements) come through L1.  HBM-bound: reads A, idx, dP once and writes
// dA once.
// T = ceil(k / s) = the most windows that cover an element per axis, as a compile-time bound (1..3) so the window
// loop is straight-line code; T = 0 keeps runtime loops for larger ratios.  Adding 0.f for a window that does not
// point here leaves the sum bit-identical.
// One warp per plane at a time.  The warp first puts everything it will read in flight together - the plane's pooled
// indices and gradients (into its slice of shared memory) and the first sixteen rows-worth of A (into registers) -
// so a plane costs about two memory round trips; the window tests then run out of shared memory.
constexpr int kPoolWarps = 8;  // warps (= planes in flight) per block
constexpr int kPoolRows = 8;   // rows per step: their A values are loaded together
template <int T, bool RELU>
__global__ void __launch_bounds__(kPoolWarps * 32, 5) maxpool_bwd_kernel(const float* __restrict__ A,
                                                                      const int32_t* __restrict__ idx,
                                                                      const float* __restrict__ dP,
                                                                      const float* __restrict__ P,
                                                                      float* __restrict__ dA, int planes, int n, int m,
                                                                      int k, int s, uint32_t inv_s, int mm_pad) {
  pdl_wait();
  extern __shared__ uint32_t pool_smem[];
  const int mm = m * m, nn = n * n;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // [n] coordinate -> first | last << 16 pooled coordinate whose window covers it, then one slice per warp
  uint32_t* s_rng = pool_smem;
  int32_t* s_idx = reinterpret_cast<int32_t*>(pool_smem) + ((n + 31) & ~31) + warp * 2 * mm_pad;
  float* s_dp = reinterpret_cast<float*>(s_idx + mm_pad);
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const int p0 = c < k ? 0 : (int)fast_div((uint32_t)(c - k), (uint32_t)s, inv_s) + 1;
    const int p1 = min((int)fast_div((uint32_t)c, (uint32_t)s, inv_s), m - 1);
    s_rng[c] = (uint32_t)p0 | ((uint32_t)p1 << 16);
  }
  __syncthreads();
  const int warp0 = blockIdx.x * kPoolWarps + warp, nwarps = gridDim.x * kPoolWarps;
  for (int plane = warp0; plane < planes; plane += nwarps) {
    const int32_t* ip = idx + (size_t)plane * mm;
    const float* gp = dP + (size_t)plane * mm;
    const float* a = RELU ? A + (size_t)plane * nn : nullptr;
    float* out = dA + (size_t)plane * nn;
    __syncwarp();  // the previous plane's window tests are done with the shared slice
    for (int i = lane; i < mm; i += 32) {
      s_idx[i] = __ldg(ip + i);
      // With the pooled tensor P given, the ReLU mask is applied here: the element a window points at holds exactly
      // that window's maximum, so [A > 0] at the element equals [P > 0] at the window.
      s_dp[i] = (P == nullptr || __ldg(P + (size_t)plane * mm + i) > 0.f) ? __ldg(gp + i) : 0.f;
    }
    // lane = column (in chunks of 32), eight rows per step with their A values loaded together: no division and no
    // global load inside the window tests.
    for (int w0 = 0; w0 < n; w0 += 32) {
      const int w = w0 + lane;
      const bool wok = w < n;
      const uint32_t rw = s_rng[wok ? w : 0];
      int pwc[T > 0 ? T : 1];
      bool pwv[T > 0 ? T : 1];
#pragma unroll
      for (int jj = 0; jj < T; ++jj) {
        const int pw = (int)(rw >> 16) - (T - 1) + jj;
        pwv[jj] = wok && pw >= (int)(rw & 0xffffu);
        pwc[jj] = max(pw, 0);
      }
      float av[kPoolRows];
      auto fetch = [&](int h0) {
#pragma unroll
        for (int j = 0; j < kPoolRows; ++j) av[j] = (RELU && wok && h0 + j < n) ? __ldg(a + (h0 + j) * n + w) : 1.f;
      };
      fetch(0);
      __syncwarp();  // staged values visible (first column chunk) / harmless afterwards
      for (int h0 = 0; h0 < n; h0 += kPoolRows) {
        float res[kPoolRows];
#pragma unroll
        for (int j = 0; j < kPoolRows; ++j) {
          const int h = min(h0 + j, n - 1);
          const int here = h * n + w;
          const bool live = av[j] > 0.f;
          const uint32_t rh = s_rng[h];
          const int ph1 = (int)(rh >> 16), ph0 = (int)(rh & 0xffffu);
          float acc = 0.f;
          if (T > 0) {
#pragma unroll
            for (int i = 0; i < T; ++i) {
              const int ph = ph1 - (T - 1) + i;
              if (ph >= ph0) {  // the same for every lane (h is): a uniform branch that skips the row's dead windows
                const int base = ph * m;
#pragma unroll
                for (int jj = 0; jj < T; ++jj) {
                  // both reads are unconditional (the index is always inside the slice), so there is no branch
                  const int at = base + pwc[jj];
                  const int32_t where = s_idx[at];
                  const float g = s_dp[at];
                  acc += (live && pwv[jj] && where == here) ? g : 0.f;
                }
              }
            }
          } else if (live && wok) {
            for (int ph = ph0; ph <= ph1; ++ph)
              for (int pw = (int)(rw & 0xffffu); pw <= (int)(rw >> 16); ++pw)
                if (s_idx[ph * m + pw] == here) acc += s_dp[ph * m + pw];
          }
          res[j] = acc;
        }
        if (h0 + kPoolRows < n) fetch(h0 + kPoolRows);  // next rows' A in flight while these results are stored
#pragma unroll
        for (int j = 0; j < kPoolRows; ++j)
          if (wok && h0 + j < n) out[(h0 + j) * n + w] = res[j];
      }
    }
  }
}

// The same operation for ceil(k / s) <= 2 (3x3 / stride 2, 2x2 / stride 2, ...), where an element is covered by at most
// four windows, turned around: the block walks over the WINDOWS of a group of planes (a quarter as many as elements
// for 3x3 / 2), and each window drops its gradient into the slot (window row - first covering row, window column -
// first covering column) of the element it points at, in a shared-memory plane of four slots per element.  A slot has
// exactly one possible writer, so there is no read-modify-write; adding an element's four slots in slot order is the
// (ph, pw) order of the reference's scatter, empty slots adding 0.f.  The output is then written (and the slots
// zeroed again) by a flat, coalesced sweep, while the next group's indices and gradients are already in flight.
// Reads idx, dP (and P or A) once, writes dA once; shared-memory work per element: four words read and zeroed.
constexpr int kSlotThreads = 256;
constexpr int kSlotWin = 4;  // windows per thread and group: a group has at most kSlotThreads * kSlotWin windows
template <bool RELU>
__global__ void __launch_bounds__(kSlotThreads) maxpool_bwd_slots_kernel(
    const float* __restrict__ A, const int32_t* __restrict__ idx, const float* __restrict__ dP,
    const float* __restrict__ P, float* __restrict__ dA, int planes, int n, int m, int k, int s, int group,
    uint32_t inv_mm, uint32_t inv_m, uint32_t inv_n) {
  pdl_wait();
  extern __shared__ float slot_smem[];
  const int mm = m * m, nn = n * n, tid = threadIdx.x;
  const int span = group * nn;
  float* slots = slot_smem;                              // [4 slots][group][nn]: neighbouring elements, neighbouring banks
  int* first = reinterpret_cast<int*>(slots + 4 * span);  // [n]: first window that covers a coordinate
  for (int c = tid; c < n; c += kSlotThreads) first[c] = c < k ? 0 : (c - k) / s + 1;
  for (int j = tid; j < 4 * span; j += kSlotThreads) slots[j] = 0.f;
  __syncthreads();
  const int ngroups = (planes + group - 1) / group;
  int32_t e_r[kSlotWin];
  float g_r[kSlotWin];
  auto fetch = [&](int grp) {
    const int p0 = grp * group, count = min(group, planes - p0) * mm;
    const size_t off = (size_t)p0 * mm;
#pragma unroll
    for (int w = 0; w < kSlotWin; ++w) {
      const int i = tid + w * kSlotThreads;
      e_r[w] = -1;
      g_r[w] = 0.f;
      if (i < count) {
        e_r[w] = __ldg(idx + off + i);
        const float g = __ldg(dP + off + i);
        // With the pooled tensor P given, the ReLU mask is applied here: the element a window points at holds exactly
        // that window's maximum, so [A > 0] at the element equals [P > 0] at the window.
        g_r[w] = (P == nullptr || __ldg(P + off + i) > 0.f) ? g : 0.f;
      }
    }
  };
  int grp = blockIdx.x;
  if (grp < ngroups) fetch(grp);
  for (; grp < ngroups; grp += gridDim.x) {
    const int p0 = grp * group, np = min(group, planes - p0);
#pragma unroll
    for (int w = 0; w < kSlotWin; ++w) {
      if (e_r[w] >= 0) {
        const uint32_t i = (uint32_t)(tid + w * kSlotThreads);
        const uint32_t pl = fast_div(i, (uint32_t)mm, inv_mm), wi = i - pl * mm;
        const uint32_t ph = fast_div(wi, (uint32_t)m, inv_m), pw = wi - ph * m;
        const uint32_t e = (uint32_t)e_r[w];
        const uint32_t h = fast_div(e, (uint32_t)n, inv_n), c = e - h * n;
        const int slot = ((int)ph - first[h]) * 2 + ((int)pw - first[c]);
        slots[slot * span + (int)(pl * nn + e)] = g_r[w];
      }
    }
    __syncthreads();
    if (grp + (int)gridDim.x < ngroups) fetch(grp + gridDim.x);  // in flight during the sweep below
    const size_t obase = (size_t)p0 * nn;
    for (int j = tid; j < np * nn; j += kSlotThreads) {
      float acc = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc += slots[q * span + j];
        slots[q * span + j] = 0.f;
      }
      if (RELU) acc = __ldg(A + obase + j) > 0.f ? acc : 0.f;
      dA[obase + j] = acc;
    }
    __syncthreads();
  }
}

// 3x3 windows with stride 2 (the pooling layers of AlexNet / CaffeNet).  A block owns `group` consecutive planes: it
// brings their pooled indices and gradients (with the P-based ReLU mask already applied) into shared memory with aligned
// 16-byte loads, then one thread owns a 2 x 2 block of elements (rows 2a, 2a+1; columns 2b, 2b+1).  Only the windows
// (a-1 .. a) x (b-1 .. b) can point into it - four index / gradient pairs for four outputs - and each element visits its
// windows in (ph, pw) order like the reference's scatter:
//   (2a, 2b): all four;  (2a, 2b+1): (a-1, b), (a, b);  (2a+1, 2b): (a, b-1), (a, b);  (2a+1, 2b+1): (a, b).
// Reading the windows from global memory instead (each is wanted by four threads) ran at 3.7 TB/s, this at 4.9 TB/s;
// building the result in shared memory as well, to store it in 16-byte pieces, was slower than either.
constexpr int kPool32Threads = 256;
constexpr int kPool32Items = 12 * kPool32Threads;  // 2 x 2 blocks a thread block takes on per group
constexpr size_t kPool32SmemCap = 64 * 1024;

template <bool RELU>
__global__ void __launch_bounds__(kPool32Threads) maxpool_bwd_3x3s2_kernel(
    const float* __restrict__ A, const int32_t* __restrict__ idx, const float* __restrict__ dP, const float* __restrict__ P,
    float* __restrict__ dA, int planes, int n, int m, int half, uint32_t inv_half, int group, int vec_ok) {
  extern __shared__ __align__(16) float pool32_smem[];
  pdl_wait();
  const int nn = n * n, mm = m * m;
  const int in_pad = (group * mm + 3) & ~3;
  int32_t* s_idx = reinterpret_cast<int32_t*>(pool32_smem);
  float* s_g = pool32_smem + in_pad;
  for (int g0 = blockIdx.x * group; g0 < planes; g0 += gridDim.x * group) {
    const int cnt = min(group, planes - g0);
    const size_t in_base = (size_t)g0 * mm;
    const size_t out_base = (size_t)g0 * nn;
    const int tot = cnt * mm;
    // With the pooled tensor P given, the ReLU mask is applied here: the element a window points at holds exactly that
    // window's maximum, so [A > 0] at the element equals [P > 0] at the window.
    const int v = (vec_ok && (in_base & 3) == 0) ? tot >> 2 : 0;
    const int4* i4 = reinterpret_cast<const int4*>(idx + in_base);
    const float4* g4 = reinterpret_cast<const float4*>(dP + in_base);
    const float4* p4 = reinterpret_cast<const float4*>(P ? P + in_base : dP + in_base);
    for (int q = threadIdx.x; q < v; q += kPool32Threads) {
      const int4 iv = __ldg(i4 + q);
      float4 gv = __ldg(g4 + q);
      if (P != nullptr) {
        const float4 pv = __ldg(p4 + q);
        gv.x = pv.x > 0.f ? gv.x : 0.f;
        gv.y = pv.y > 0.f ? gv.y : 0.f;
        gv.z = pv.z > 0.f ? gv.z : 0.f;
        gv.w = pv.w > 0.f ? gv.w : 0.f;
      }
      reinterpret_cast<int4*>(s_idx)[q] = iv;
      reinterpret_cast<float4*>(s_g)[q] = gv;
    }
    for (int q = (v << 2) + threadIdx.x; q < tot; q += kPool32Threads) {
      s_idx[q] = __ldg(idx + in_base + q);
      const float gq = __ldg(dP + in_base + q);
      s_g[q] = (P == nullptr || __ldg(P + in_base + q) > 0.f) ? gq : 0.f;
    }
    __syncthreads();
    const uint32_t items = (uint32_t)cnt * half * half;
    for (uint32_t t = threadIdx.x; t < items; t += kPool32Threads) {
      const uint32_t row = fast_div(t, (uint32_t)half, inv_half);  // = plane in group * half + a
      const int b = (int)(t - row * half);
      const uint32_t pl = fast_div(row, (uint32_t)half, inv_half);
      const int a = (int)(row - pl * half);
      int32_t wi[2][2];
      float wg[2][2];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int ph = a - 1 + i, pw = b - 1 + j;
          const bool ok = ph >= 0 && ph < m && pw >= 0 && pw < m;
          const int at = ok ? (int)pl * mm + ph * m + pw : 0;
          wi[i][j] = ok ? s_idx[at] : -1;
          wg[i][j] = ok ? s_g[at] : 0.f;
        }
      const int h0 = 2 * a, w0 = 2 * b;
      const int e00 = h0 * n + w0, e01 = e00 + 1, e10 = e00 + n, e11 = e10 + 1;
      float r00 = 0.f, r01 = 0.f, r10 = 0.f, r11 = 0.f;
      r00 += wi[0][0] == e00 ? wg[0][0] : 0.f;
      r00 += wi[0][1] == e00 ? wg[0][1] : 0.f;
      r00 += wi[1][0] == e00 ? wg[1][0] : 0.f;
      r00 += wi[1][1] == e00 ? wg[1][1] : 0.f;
      r01 += wi[0][1] == e01 ? wg[0][1] : 0.f;
      r01 += wi[1][1] == e01 ? wg[1][1] : 0.f;
      r10 += wi[1][0] == e10 ? wg[1][0] : 0.f;
      r10 += wi[1][1] == e10 ? wg[1][1] : 0.f;
      r11 += wi[1][1] == e11 ? wg[1][1] : 0.f;
      const bool wide = w0 + 1 < n, tall = h0 + 1 < n;
      const size_t plane_at = out_base + (size_t)pl * nn;
      float* out = dA + plane_at;
      if (RELU) {
        const float* ap = A + plane_at;
        r00 = __ldg(ap + e00) > 0.f ? r00 : 0.f;
        if (wide) r01 = __ldg(ap + e01) > 0.f ? r01 : 0.f;
        if (tall) r10 = __ldg(ap + e10) > 0.f ? r10 : 0.f;
        if (wide && tall) r11 = __ldg(ap + e11) > 0.f ? r11 : 0.f;
      }
      out[e00] = r00;
      if (wide) out[e01] = r01;
      if (tall) out[e10] = r10;
      if (wide && tall) out[e11] = r11;
    }
    __syncthreads();
  }
}

template <bool RELU>
int launch_maxpool_bwd(cct_ctx* ctx, const float* A, const int32_t* idx, const float* dP, float* dA, int planes, int n,
                       int m, int k, int s, const float* P = nullptr) {
  const int grid = plane_grid(ctx, (planes + kPoolWarps - 1) / kPoolWarps);
  const uint32_t inv_s = fast_div_magic((uint64_t)n, (uint32_t)s);
  const int taps = (k + s - 1) / s;
  const int half = (n + 1) / 2;
  if (k == 3 && s == 2) {
    // Planes per block: a multiple of four, so that every group starts on a 16-byte boundary of the pooled tensors.
    const int group = std::max(4, (kPool32Items / (half * half) + 3) & ~3);
    const size_t smem = (size_t)2 * ((group * m * m + 3) & ~3) * 4;
    if (smem <= kPool32SmemCap) {
      const int vec_ok = ((reinterpret_cast<uintptr_t>(idx) | reinterpret_cast<uintptr_t>(dP) |
                           reinterpret_cast<uintptr_t>(P)) & 15) == 0;
      if (smem > 48 * 1024)
        CCT_CUDA(ctx, cudaFuncSetAttribute(maxpool_bwd_3x3s2_kernel<RELU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      const int blocks = std::max(1, std::min((planes + group - 1) / group, ctx->sm_count * 64));
      launch_pdl(maxpool_bwd_3x3s2_kernel<RELU>, dim3(blocks), dim3(kPool32Threads), smem, ctx->stream, A, idx, dP, P, dA,
                 planes, n, m, half, fast_div_magic((uint64_t)group * half * half, (uint32_t)half), group, vec_ok);
      return CCT_OK;
    }
  }
  constexpr int kSlotSmemCap = 56 * 1024;  // four blocks per SM
  if (taps <= 2 && m * m <= kSlotThreads * kSlotWin && (size_t)n * n * 16 + (size_t)n * 4 <= kSlotSmemCap) {
    const int nn = n * n, mm = m * m;
    const int group = std::max(1, std::min({planes, (int)((kSlotSmemCap - n * 4) / ((size_t)nn * 16)),
                                            kSlotThreads * kSlotWin / mm}));
    const size_t smem = (size_t)group * nn * 16 + (size_t)n * 4;
    if (smem > 48 * 1024)
      CCT_CUDA(ctx, cudaFuncSetAttribute(maxpool_bwd_slots_kernel<RELU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int ngroups = (planes + group - 1) / group;
    const int blocks = std::max(1, std::min(ngroups, ctx->sm_count * 4));
    launch_pdl(maxpool_bwd_slots_kernel<RELU>, dim3(blocks), dim3(kSlotThreads), smem, ctx->stream, 
        A, idx, dP, P, dA, planes, n, m, k, s, group, fast_div_magic((uint64_t)kSlotThreads * kSlotWin, (uint32_t)mm),
        fast_div_magic((uint64_t)mm, (uint32_t)m), fast_div_magic((uint64_t)nn, (uint32_t)n));
    return CCT_OK;
  }
  const int mm_pad = (m * m + 31) & ~31;
  const size_t smem = ((size_t)((n + 31) & ~31) + (size_t)kPoolWarps * 2 * mm_pad) * 4;
  if (smem > 200 * 1024) {
    ctx->last_error = "pooled plane too large for the shared-memory staging of maxpool backward";
    return CCT_ERR_UNSUPPORTED;
  }
  auto kernel = taps == 1 ? maxpool_bwd_kernel<1, RELU> : taps == 2 ? maxpool_bwd_kernel<2, RELU>
              : taps == 3 ? maxpool_bwd_kernel<3, RELU> : maxpool_bwd_kernel<0, RELU>;
  if (smem > 48 * 1024) CCT_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  launch_pdl(kernel, dim3(grid), dim3(kPoolWarps * 32), smem, ctx->stream, A, idx, dP, P, dA, planes, n, m, k, s, inv_s, mm_pad);
  return CCT_OK;
}

}  // namespace

static int pool_args_ok(int planes, int n, int k, int s) { return planes > 0 && n > 0 && k > 0 && s > 0 && k <= n; }

// cct_pool_relu_backward with the ReLU mask taken from the pooled tensor P instead of the full-size activation A
// (bit-identical: see the staging loop of the kernels); reads planes * m * m values where the other reads planes * n * n.
int pool_relu_backward_pooled(cct_ctx* ctx, const float* P, const int32_t* idx, const float* dP, float* dA, int planes,
                              int n, int k, int s) {
  if (!ctx || !P || !idx || !dP || !dA || !pool_args_ok(planes, n, k, s)) return CCT_ERR_INVALID;
  const int m = (n - k) / s + 1;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const int rc = launch_maxpool_bwd<false>(ctx, nullptr, idx, dP, dA, planes, n, m, k, s, P);
  if (rc != CCT_OK) return rc;
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

extern "C" {

int cct_fill_f32(cct_ctx* ctx, float* dptr, size_t count, float value) {
  if (!ctx || (!dptr && count)) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(fill_kernel, dim3(grid_for(ctx, count, 256)), dim3(256), 0, ctx->stream, dptr, count, value);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_sgd_step(cct_ctx* ctx, size_t count, float* w, float* g, float* h, float lr, float momentum, float lambda) {
  if (!ctx || !w || !g || !h) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(sgd_kernel, dim3(grid_for(ctx, (count + 3) / 4, 256)), dim3(256), 0, ctx->stream, count, vec_groups(count, {w, g, h}), w, g, h, lr,
                                                                        momentum, lambda);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_saxpby(cct_ctx* ctx, size_t count, float alpha, const float* x, float beta, float* y) {
  if (!ctx || ((!x || !y) && count)) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(saxpby_kernel, dim3(grid_for(ctx, count, 256)), dim3(256), 0, ctx->stream, count, alpha, x, beta, y);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_l1_update(cct_ctx* ctx, size_t count, float* g, float lambda, const float* w) {
  if (!ctx || ((!g || !w) && count)) return CCT_ERR_INVALID;
  if (!count) return CCT_OK;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(l1_update_kernel, dim3(grid_for(ctx, count, 256)), dim3(256), 0, ctx->stream, count, g, lambda, w);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_relu_forward(cct_ctx* ctx, const float* X, float* Y, size_t count) {
  if (!ctx || !X || !Y) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(relu_fwd_kernel, dim3(grid_for(ctx, (count + 3) / 4, 256)), dim3(256), 0, ctx->stream, X, Y, count, vec_groups(count, {X, Y}));
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_relu_backward(cct_ctx* ctx, const float* X, const float* dY, float* dX, size_t count) {
  if (!ctx || !X || !dY || !dX) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(relu_bwd_kernel, dim3(grid_for(ctx, (count + 3) / 4, 256)), dim3(256), 0, ctx->stream, X, dY, dX, count,
                                                                                vec_groups(count, {X, dY, dX}));
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}


int cct_maxpool_forward(cct_ctx* ctx, const float* X, float* Y, int32_t* idx, int planes, int n, int k, int s) {
  if (!ctx || !X || !Y || !idx || !pool_args_ok(planes, n, k, s)) return CCT_ERR_INVALID;
  const int m = (n - k) / s + 1;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  // planes that fit in shared memory are staged there (one HBM read per element); larger ones read through L1
  if ((size_t)n * n * sizeof(float) <= 200 * 1024) return maxpool_forward_staged(ctx, X, Y, idx, planes, n, m, k, s);
  launch_pdl(maxpool_fwd_kernel, dim3(plane_grid(ctx, planes)), dim3(256), 0, ctx->stream, X, Y, idx, planes, n, m, k, s);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_maxpool_backward(cct_ctx* ctx, const float* dY, const int32_t* idx, float* dX, int planes, int n, int k,
                         int s) {
  if (!ctx || !dY || !idx || !dX || !pool_args_ok(planes, n, k, s)) return CCT_ERR_INVALID;
  const int m = (n - k) / s + 1;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const int rc = launch_maxpool_bwd<false>(ctx, nullptr, idx, dY, dX, planes, n, m, k, s);
  if (rc != CCT_OK) return rc;
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_pool_relu_backward(cct_ctx* ctx, const float* A, const int32_t* idx, const float* dP, float* dA, int planes,
                           int n, int k, int s) {
  if (!ctx || !A || !idx || !dP || !dA || !pool_args_ok(planes, n, k, s)) return CCT_ERR_INVALID;
  const int m = (n - k) / s + 1;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const int rc = launch_maxpool_bwd<true>(ctx, A, idx, dP, dA, planes, n, m, k, s);
  if (rc != CCT_OK) return rc;
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

}  // extern "C"
