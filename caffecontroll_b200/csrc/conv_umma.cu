// Implicit-GEMM convolution on the Blackwell tensor cores (CCT_ALGO_UMMA_3XTF32).
//
// All three contractions of the convolution bridge run on tcgen05.mma (kind::tf32, M = 128, fp32 accumulators in
// tensor memory).  The lowered matrix of the reference (type-1 lowering, one row of k*k*D values per output pixel)
// is never written to global memory: producer threads gather each 128 x 32 tile of it straight from the NCHW input
// into shared memory, in the K-major 128-byte-swizzled layout the MMA unit reads, splitting every fp32 value into
// hi = tf32(x) and lo = x - hi on the way.  Three MMAs per k-step (hi*hi + hi*lo + lo*hi) recover fp32-level
// accuracy ("3xTF32"); flops are counted once.
//
//   forward        Y[pix][o]   = sum_k  Lowered(X)[pix][k] * W[o][k]            (+ bias, optional ReLU)
//   data gradient  dX[pix][d]  = sum_kk Gathered(dY)[pix][kk] * Wd[d][kk]       kk = (filter, tap)
//                  — the inverse lowering (col2im) written as a gather: every input pixel sums the taps that
//                  touch it inside the accumulator, so there is no scatter, no atomics, and the result is
//                  deterministic.  For stride s > 1 the input pixels are processed in s*s phases; a phase only
//                  sees the taps congruent to it, so no multiplication by structural zeros is issued.
//   weight gradient dW[kk][o]  = sum_pix Lowered(X)[pix][kk] * dY[pix][o]        split over pixel ranges across
//                  CTAs, partial sums to scratch, fixed-order reduction; one extra all-ones row of the lowered
//                  operand yields the bias gradient from the same MMAs.
//
// Pipeline inside a CTA (256 threads): a ring of S shared-memory stages; all threads fill stage s, fence to the
// async proxy, barrier; one thread issues the 12 MMAs of the stage and a tcgen05.commit onto the stage's mbarrier;
// the fill of the next stage overlaps the MMAs.  Every mbarrier wait is bounded: when it runs out the thread sets
// the context's status word, stops waiting on anything else, and the kernel still frees its tensor memory.
#include <algorithm>
#include <cstdlib>
#include <vector>

#include "cct_internal.h"

namespace {

constexpr int kThreads = 256;
constexpr int kTileM = 128;
constexpr int kBlockK = 32;  // fp32 per k-block: one 128-byte swizzled row
constexpr int kMaxStages = 4;
constexpr int kATileBytes = kTileM * 128;
constexpr int kSmemLimit = 227 * 1024;
#ifdef CCT_DBG
#define DBG(P, bit) ((P).dbg & (bit))
#else
#define DBG(P, bit) 0
#endif
constexpr int kPadTap = 0x4000;  // tap coordinate that fails every bounds test (marks padding rows of a table)

// One entry per reduction index of a gathered operand: element offset from the pixel's tap origin and the tap's
// (dy, dx) for the bounds test.
struct Tap {
  int off;
  short dy, dx;
};

// ---------------------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Bounded wait.  Returns false (and records `code` in the status word) after about 0.2 s without completion.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, bool& failed, int* status, int code) {
  if (failed) return false;
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > 400000000LL) break;
  }
  failed = true;
  *reinterpret_cast<volatile int*>(status) = code;
  return false;
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major, tf32 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The mbarrier receives one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// kind::tf32 instruction descriptor: fp32 accumulator, tf32 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}

// Byte offset of 16-byte chunk q (0..7) of row r inside a swizzled tile.
__device__ __forceinline__ uint32_t swz(int r, int q) { return (uint32_t)(r * 128 + ((q ^ (r & 7)) << 4)); }

// hi = x rounded to tf32 (10 explicit mantissa bits), lo = x - hi (exact in fp32).
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
  lo = x - hi;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void store_split4(uint32_t hi_addr, uint32_t lo_addr, const float* v) {
  float h[4], l[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) split_tf32(v[e], h[e], l[e]);
  st_shared_v4(hi_addr, h[0], h[1], h[2], h[3]);
  st_shared_v4(lo_addr, l[0], l[1], l[2], l[3]);
}

// The 12 MMAs of one stage: for each of the 4 k-steps (8 tf32 = 32 bytes), lo*hi, hi*lo, hi*hi.
__device__ __forceinline__ void issue_stage(uint32_t tmem_d, uint32_t a_hi, uint32_t a_lo, uint32_t b_hi, uint32_t b_lo,
                                            uint32_t idesc, bool first_stage) {
  const uint64_t dah = make_desc(a_hi), dal = make_desc(a_lo), dbh = make_desc(b_hi), dbl = make_desc(b_lo);
#pragma unroll
  for (int j = 0; j < kBlockK / 8; ++j) {
    const uint64_t adv = (uint64_t)(j * 2);  // 32 bytes >> 4
    umma_tf32(tmem_d, dal + adv, dbh + adv, idesc, (first_stage && j == 0) ? 0u : 1u);
    umma_tf32(tmem_d, dah + adv, dbl + adv, idesc, 1u);
    umma_tf32(tmem_d, dah + adv, dbh + adv, idesc, 1u);
  }
}

struct SmemLayout {
  uint32_t stage_bytes, b_tile_bytes;
  int stages;
};

__host__ __device__ inline SmemLayout smem_layout(int n_pad) {
  SmemLayout L;
  L.b_tile_bytes = (uint32_t)n_pad * 128u;
  L.stage_bytes = 2u * kATileBytes + 2u * L.b_tile_bytes;
  int s = (kSmemLimit - 2048) / (int)L.stage_bytes;
  L.stages = s > kMaxStages ? kMaxStages : s;
  return L;
}

inline size_t smem_bytes(int n_pad) {
  const SmemLayout L = smem_layout(n_pad);
  return (size_t)L.stages * L.stage_bytes + 1024 /*alignment slack*/ + 256 /*barriers, tmem slot*/;
}

__host__ __device__ inline uint32_t tmem_cols(int n_pad) {
  uint32_t c = 32;
  while ((int)c < n_pad) c <<= 1;
  return c;
}

// ------------------------------------------------------------------------------ gather kernel (forward, dgrad)
struct GatherParams {
  const float* in;    // gathered tensor: X (forward) or dY (data gradient)
  float* out;         // Y or dX
  const float* w_hi;  // packed B operand [vgroups][n_pad][k_pad], tf32-rounded part
  const float* w_lo;  // remainder part
  const Tap* taps;    // [k_pad]
  const float* bias;  // indexed by output channel, or null
  int n_pix, q_h, q_w;                 // pixels = batch * q_h * q_w
  int iy_mul, iy_add, ix_mul, ix_add;  // tap origin in the gathered tensor: iy0 = qy*iy_mul + iy_add
  int in_lim;                          // gathered tensor is in_lim x in_lim per channel
  long long in_batch_stride;
  int in_group_stride;   // elements between the channel blocks of consecutive groups
  int tiles_per_group;   // virtual groups per real group (output-channel tiles)
  int oy_mul, oy_add, ox_mul, ox_add;  // output pixel: oy = qy*oy_mul + oy_add
  int out_pitch, out_plane;
  long long out_batch_stride;
  int out_group_channels;  // output channels per real group
  int n, n_pad, k_pad;     // real / padded output channels per virtual group, padded reduction length
  int relu;
  int* status;
  int dbg;
};

__global__ void __launch_bounds__(kThreads, 1) gather_conv_kernel(const __grid_constant__ GatherParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const SmemLayout L = smem_layout(P.n_pad);
  const uint32_t bar0 = base + (uint32_t)L.stages * L.stage_bytes;  // mma_done[stage]
  const uint32_t tmem_slot = bar0 + 8u * kMaxStages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vg = blockIdx.y;
  const int grp = vg / P.tiles_per_group, ntile = vg % P.tiles_per_group;
  const uint32_t ncols = tmem_cols(P.n_pad);

  if (tid == 0) {
    for (int s = 0; s < L.stages; ++s) mbar_init(bar0 + 8u * s, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, ncols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_d;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_d) : "r"(tmem_slot));

  // This thread's A row = one output pixel of the tile.
  const int row = tid & 127, half = tid >> 7;
  const int pix = blockIdx.x * kTileM + row;
  const bool pix_ok = pix < P.n_pix;
  int b = 0, qy = 0, qx = 0;
  if (pix_ok) {
    const int per_img = P.q_h * P.q_w;
    b = pix / per_img;
    const int r = pix - b * per_img;
    qy = r / P.q_w;
    qx = r - qy * P.q_w;
  }
  const int iy0 = pix_ok ? qy * P.iy_mul + P.iy_add : -kPadTap * 2;
  const int ix0 = qx * P.ix_mul + P.ix_add;
  const float* in_px = P.in + (long long)b * P.in_batch_stride + (long long)grp * P.in_group_stride +
                       (long long)iy0 * P.in_lim + ix0;
  if (!pix_ok) in_px = P.in;
  const float* wh = P.w_hi + (size_t)vg * P.n_pad * P.k_pad;
  const float* wl = P.w_lo + (size_t)vg * P.n_pad * P.k_pad;
  const uint32_t idesc = make_idesc(P.n_pad);
  const int kblocks = P.k_pad / kBlockK;
  bool failed = false;

  for (int kb = 0; kb < kblocks; ++kb) {
    const int s = kb % L.stages, use = kb / L.stages;
    const uint32_t st = base + (uint32_t)s * L.stage_bytes;
    const uint32_t a_hi = st, a_lo = st + kATileBytes, b_hi = st + 2 * kATileBytes, b_lo = b_hi + L.b_tile_bytes;
    if (use > 0) mbar_wait(bar0 + 8u * s, (uint32_t)(use - 1) & 1u, failed, P.status, 0x1);

    // A: 4 chunks of 4 reduction indices for this thread's pixel.
    const Tap* tp = P.taps + kb * kBlockK + half * 16;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const Tap t = tp[c * 4 + e];
        const bool ok = (unsigned)(iy0 + t.dy) < (unsigned)P.in_lim && (unsigned)(ix0 + t.dx) < (unsigned)P.in_lim;
        v[e] = (ok && !DBG(P, 1)) ? __ldg(in_px + t.off) : 0.f;
      }
      const uint32_t o = swz(row, half * 4 + c);
      if (!DBG(P, 8)) store_split4(a_hi + o, a_lo + o, v);
    }
    // B: packed weights, already split; n_pad rows x 8 chunks, hi and lo.
    for (int i = tid; i < P.n_pad * 8 && !DBG(P, 2); i += kThreads) {
      const int r = i >> 3, q = i & 7;
      const size_t g = (size_t)r * P.k_pad + kb * kBlockK + q * 4;
      const float4 h = *reinterpret_cast<const float4*>(wh + g);
      const float4 l = *reinterpret_cast<const float4*>(wl + g);
      const uint32_t o = swz(r, q);
      st_shared_v4(b_hi + o, h.x, h.y, h.z, h.w);
      st_shared_v4(b_lo + o, l.x, l.y, l.z, l.w);
    }
    if (!DBG(P, 16)) fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      if (!DBG(P, 4)) issue_stage(tmem_d, a_hi, a_lo, b_hi, b_lo, idesc, kb == 0);
      umma_commit(bar0 + 8u * s);
    }
  }
  {
    const int last = kblocks - 1;
    mbar_wait(bar0 + 8u * (last % L.stages), (uint32_t)(last / L.stages) & 1u, failed, P.status, 0x2);
  }
  tc_fence_after();

  // Epilogue: warp w reads TMEM lanes 32*(w%4).., 16 columns at a time; warps 0-3 take even chunks, 4-7 odd ones.
  {
    const int erow = (warp & 3) * 32 + lane;
    const int epix = blockIdx.x * kTileM + erow;
    const bool eok = epix < P.n_pix && !failed;
    int eb = 0, ey = 0, ex = 0;
    if (epix < P.n_pix) {
      const int per_img = P.q_h * P.q_w;
      eb = epix / per_img;
      const int r = epix - eb * per_img;
      ey = r / P.q_w;
      ex = r - ey * P.q_w;
    }
    const int ch0 = grp * P.out_group_channels + ntile * P.n;
    float* op = P.out + (long long)eb * P.out_batch_stride + (long long)ch0 * P.out_plane +
                (long long)(ey * P.oy_mul + P.oy_add) * P.out_pitch + (ex * P.ox_mul + P.ox_add);
    const int chunks = P.n_pad / 16;
    for (int c = warp >> 2; c < chunks; c += 2) {
      float v[16];
      tmem_ld16(tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(c * 16), v);
      if (eok) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int ch = c * 16 + j;
          if (ch < P.n) {
            float y = v[j];
            if (P.bias) y += __ldg(P.bias + ch0 + ch);
            if (P.relu) y = fmaxf(y, 0.f);
            op[(long long)ch * P.out_plane] = y;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_d, ncols);
}

// ---------------------------------------------------------------------------------- weight-gradient kernel
struct WgradParams {
  const float* x;
  const float* dy;
  float* partial;   // [splits][vgroups][m_tiles*128][n_pad]
  const Tap* taps;  // [m_tiles*128]; row k_real is the all-ones row (dy == kOnesTap)
  int n_pix, m, mm, n, s, p;
  long long x_batch_stride;
  int x_group_stride;
  long long dy_batch_stride;
  int dy_group_channels;  // output channels per real group
  int tiles_per_group;
  int n_real, n_pad;
  int kblocks_total, kblocks_per_split;
  int* status;
  int dbg;
};
constexpr int kOnesTap = 0x2000;

__global__ void __launch_bounds__(kThreads, 1) wgrad_kernel(const __grid_constant__ WgradParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const SmemLayout L = smem_layout(P.n_pad);
  const uint32_t bar0 = base + (uint32_t)L.stages * L.stage_bytes;
  const uint32_t tmem_slot = bar0 + 8u * kMaxStages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mtile = blockIdx.x, split = blockIdx.y, vg = blockIdx.z;
  const int grp = vg / P.tiles_per_group, ntile = vg % P.tiles_per_group;
  const uint32_t ncols = tmem_cols(P.n_pad);

  if (tid == 0) {
    for (int s = 0; s < L.stages; ++s) mbar_init(bar0 + 8u * s, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, ncols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_d;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_d) : "r"(tmem_slot));

  // Thread (q, r0): 4 consecutive pixels (chunk q of the 32-pixel block) for rows r0, r0+32, r0+64, r0+96.
  const int q = tid & 7, r0 = tid >> 3;
  Tap tap[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) tap[i] = P.taps[mtile * kTileM + r0 + 32 * i];
  const float* xg = P.x + (long long)grp * P.x_group_stride;
  const float* dyg = P.dy + (long long)(grp * P.dy_group_channels + ntile * P.n_real) * P.mm;
  const uint32_t idesc = make_idesc(P.n_pad);
  const int kb_begin = split * P.kblocks_per_split;
  const int kb_end = min(P.kblocks_total, kb_begin + P.kblocks_per_split);
  const int kblocks = kb_end - kb_begin;  // >= 1 by construction of the grid
  bool failed = false;

  for (int it = 0; it < kblocks; ++it) {
    const int s = it % L.stages, use = it / L.stages;
    const uint32_t st = base + (uint32_t)s * L.stage_bytes;
    const uint32_t a_hi = st, a_lo = st + kATileBytes, b_hi = st + 2 * kATileBytes, b_lo = b_hi + L.b_tile_bytes;
    if (use > 0) mbar_wait(bar0 + 8u * s, (uint32_t)(use - 1) & 1u, failed, P.status, 0x4);

    // Decompose this thread's 4 pixels.
    long long xoff[4], dyoff[4];
    int iy0[4], ix0[4];
    bool ok[4];
    {
      int pix = (kb_begin + it) * kBlockK + q * 4;
      int b = pix / P.mm;
      int pin = pix - b * P.mm;
      int r = pin / P.m;
      int c = pin - r * P.m;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ok[e] = pix + e < P.n_pix;
        iy0[e] = r * P.s - P.p;
        ix0[e] = c * P.s - P.p;
        xoff[e] = (long long)b * P.x_batch_stride + (long long)iy0[e] * P.n + ix0[e];
        dyoff[e] = (long long)b * P.dy_batch_stride + r * P.m + c;
        if (++c == P.m) {
          c = 0;
          if (++r == P.m) { r = 0; ++b; }
        }
      }
    }
    // A: rows = reduction indices of the lowered input (kk), columns = pixels.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (tap[i].dy == kOnesTap) {
          v[e] = ok[e] ? 1.f : 0.f;
        } else {
          const bool in = ok[e] && (unsigned)(iy0[e] + tap[i].dy) < (unsigned)P.n &&
                          (unsigned)(ix0[e] + tap[i].dx) < (unsigned)P.n;
          v[e] = (in && !DBG(P, 1)) ? __ldg(xg + xoff[e] + tap[i].off) : 0.f;
        }
      }
      const uint32_t o = swz(r0 + 32 * i, q);
      if (!DBG(P, 8)) store_split4(a_hi + o, a_lo + o, v);
    }
    // B: rows = output channels, columns = the same pixels.
    for (int j = r0; j < P.n_pad && !DBG(P, 2); j += 32) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = (ok[e] && j < P.n_real) ? __ldg(dyg + dyoff[e] + (long long)j * P.mm) : 0.f;
      const uint32_t o = swz(j, q);
      store_split4(b_hi + o, b_lo + o, v);
    }
    if (!DBG(P, 16)) fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      if (!DBG(P, 4)) issue_stage(tmem_d, a_hi, a_lo, b_hi, b_lo, idesc, it == 0);
      umma_commit(bar0 + 8u * s);
    }
  }
  {
    const int last = kblocks - 1;
    mbar_wait(bar0 + 8u * (last % L.stages), (uint32_t)(last / L.stages) & 1u, failed, P.status, 0x8);
  }
  tc_fence_after();

  {
    const int erow = (warp & 3) * 32 + lane;
    float* op = P.partial +
                (((size_t)split * gridDim.z + vg) * gridDim.x * kTileM + (size_t)mtile * kTileM + erow) * P.n_pad;
    const int chunks = P.n_pad / 16;
    for (int c = warp >> 2; c < chunks; c += 2) {
      float v[16];
      tmem_ld16(tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(c * 16), v);
      float4* o4 = reinterpret_cast<float4*>(op + c * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) o4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_d, ncols);
}

// dW[o][kk] and db[o] from the split partial sums, added in split order (deterministic).
__global__ void wgrad_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dW, float* __restrict__ db,
                                    int splits, int vgroups, int tiles_per_group, int rows_pad, int n_real, int n_pad,
                                    int k_real, int og) {
  const size_t total = (size_t)vgroups * (k_real + 1) * n_real;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(t % n_real);
    const int kk = (int)((t / n_real) % (k_real + 1));
    const int vg = (int)(t / ((size_t)n_real * (k_real + 1)));
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(((size_t)s * vgroups + vg) * rows_pad + kk) * n_pad + j];
    const int ch = (vg / tiles_per_group) * og + (vg % tiles_per_group) * n_real + j;
    if (kk < k_real)
      dW[(size_t)ch * k_real + kk] = acc;
    else if (db)
      db[ch] = acc;
  }
}

// ------------------------------------------------------------------------------------------ weight packing
// Forward B operand: [vg][n_pad][k_pad] <- W[o][Dg*k*k], zero padded, split hi/lo.
__global__ void pack_fwd_kernel(const float* __restrict__ W, float* __restrict__ hi, float* __restrict__ lo, int vgroups,
                                int tiles_per_group, int og, int n_real, int n_pad, int k_real, int k_pad) {
  const size_t total = (size_t)vgroups * n_pad * k_pad;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int kk = (int)(t % k_pad);
    const int j = (int)((t / k_pad) % n_pad);
    const int vg = (int)(t / ((size_t)k_pad * n_pad));
    float v = 0.f;
    if (j < n_real && kk < k_real) {
      const int ch = (vg / tiles_per_group) * og + (vg % tiles_per_group) * n_real + j;
      v = W[(size_t)ch * k_real + kk];
    }
    float h, l;
    split_tf32(v, h, l);
    hi[t] = h;
    lo[t] = l;
  }
}

// Data-gradient B operand of one phase: [vg][n_pad][k_pad], row = input channel d (tile nt of group g),
// column kk = (oc, jy, jx) <- W[g*og + oc][d][py + jy*s][px + jx*s].
__global__ void pack_dgrad_kernel(const float* __restrict__ W, float* __restrict__ hi, float* __restrict__ lo,
                                  int vgroups, int tiles_per_group, int og, int Dg, int k, int s, int py, int px,
                                  int jh, int jw, int n_real, int n_pad, int k_real, int k_pad) {
  const size_t total = (size_t)vgroups * n_pad * k_pad;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int kk = (int)(t % k_pad);
    const int j = (int)((t / k_pad) % n_pad);
    const int vg = (int)(t / ((size_t)k_pad * n_pad));
    float v = 0.f;
    if (j < n_real && kk < k_real) {
      const int grp = vg / tiles_per_group;
      const int d = (vg % tiles_per_group) * n_real + j;
      const int jx = kk % jw, jy = (kk / jw) % jh, oc = kk / (jw * jh);
      v = W[(((size_t)(grp * og + oc)) * Dg + d) * k * k + (py + jy * s) * k + (px + jx * s)];
    }
    float h, l;
    split_tf32(v, h, l);
    hi[t] = h;
    lo[t] = l;
  }
}

// Measurement knobs of debug builds (-DCCT_DBG): a bit mask from the environment that removes one pipeline part.
int dbg_knobs() {
#ifdef CCT_DBG
  const char* e = getenv("CCT_DBG_KNOBS");
  return e ? atoi(e) : 0;
#else
  return 0;
#endif
}

int round_up(int v, int a) { return (v + a - 1) / a * a; }

// Smallest number of equal channel tiles such that a tile has at most 256 channels.
int channel_tiles(int channels) {
  for (int t = 1; t <= channels; ++t)
    if (channels % t == 0 && channels / t <= 256) return t;
  return channels;
}

}  // namespace

// One stride phase of the data gradient (stride 1 has a single phase).
struct DgradPhase {
  int py, px, jh, jw;      // phase and number of taps per axis
  int y0, x0, qh, qw;      // first input row/column of the phase and how many
  int ry0, rx0;            // dY coordinate of tap (0,0) for qy = 0 / qx = 0
  int k_real, k_pad;
  Tap* taps = nullptr;     // device
  float *w_hi = nullptr, *w_lo = nullptr;
};

struct UmmaPlan {
  ConvGeom G;
  // forward / weight gradient share the lowering table
  int f_tiles, f_n, f_npad, f_kreal, f_kpad;
  Tap* f_taps = nullptr;
  float *f_whi = nullptr, *f_wlo = nullptr;
  // weight gradient
  int w_mtiles, w_splits, w_kblocks_total, w_kblocks_per_split;
  Tap* w_taps = nullptr;
  float* w_partial = nullptr;
  // data gradient
  int d_tiles, d_n, d_npad;
  std::vector<DgradPhase> phases;
  size_t bytes = 0;
};

bool umma_supported(const ConvGeom& G) {
  const int fn = G.og / channel_tiles(G.og), dn = G.Dg / channel_tiles(G.Dg);
  if (fn > 256 || dn > 256) return false;
  if (G.k > 255 || G.n > 8000) return false;  // tap coordinates are 16-bit
  return true;
}

namespace {

template <class T>
int dev_alloc(cct_ctx* ctx, UmmaPlan* p, T** ptr, size_t count) {
  CCT_CUDA(ctx, cudaMalloc((void**)ptr, std::max<size_t>(count, 1) * sizeof(T)));
  p->bytes += count * sizeof(T);
  return CCT_OK;
}

int upload_taps(cct_ctx* ctx, UmmaPlan* p, Tap** dst, const std::vector<Tap>& host) {
  int rc = dev_alloc(ctx, p, dst, host.size());
  if (rc != CCT_OK) return rc;
  CCT_CUDA(ctx, cudaMemcpy(*dst, host.data(), host.size() * sizeof(Tap), cudaMemcpyHostToDevice));
  return CCT_OK;
}

template <class K>
int set_smem(cct_ctx* ctx, K kernel, size_t bytes) {
  CCT_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return CCT_OK;
}

int pack_grid(cct_ctx* ctx, size_t total) {
  size_t b = (total + 255) / 256;
  return (int)std::min<size_t>(std::max<size_t>(b, 1), (size_t)ctx->sm_count * 8);
}

}  // namespace

int umma_plan_create(cct_ctx* ctx, const ConvGeom& G, UmmaPlan** out) {
  UmmaPlan* p = new UmmaPlan();
  p->G = G;
  int rc = CCT_OK;
  const int kk = G.k * G.k;
  // ---- forward: rows = output channels of a tile, reduction = (d, kr, kc)
  p->f_tiles = channel_tiles(G.og);
  p->f_n = G.og / p->f_tiles;
  p->f_npad = round_up(p->f_n, 16);
  p->f_kreal = G.Dg * kk;
  p->f_kpad = round_up(p->f_kreal, kBlockK);
  {
    std::vector<Tap> t(p->f_kpad);
    for (int i = 0; i < p->f_kpad; ++i) {
      if (i < p->f_kreal) {
        const int d = i / kk, kr = (i / G.k) % G.k, kc = i % G.k;
        t[i] = Tap{d * G.n * G.n + kr * G.n + kc, (short)kr, (short)kc};
      } else {
        t[i] = Tap{0, (short)kPadTap, (short)kPadTap};
      }
    }
    rc = upload_taps(ctx, p, &p->f_taps, t);
  }
  const size_t fw = (size_t)G.g * p->f_tiles * p->f_npad * p->f_kpad;
  if (rc == CCT_OK) rc = dev_alloc(ctx, p, &p->f_whi, fw);
  if (rc == CCT_OK) rc = dev_alloc(ctx, p, &p->f_wlo, fw);
  // ---- weight gradient: rows = (d, kr, kc) plus the all-ones row, columns = output channels of a tile
  if (rc == CCT_OK) {
    p->w_mtiles = (p->f_kreal + 1 + kTileM - 1) / kTileM;
    std::vector<Tap> t((size_t)p->w_mtiles * kTileM);
    for (size_t i = 0; i < t.size(); ++i) {
      if ((int)i < p->f_kreal) {
        const int d = (int)i / kk, kr = ((int)i / G.k) % G.k, kc = (int)i % G.k;
        t[i] = Tap{d * G.n * G.n + kr * G.n + kc, (short)kr, (short)kc};
      } else if ((int)i == p->f_kreal) {
        t[i] = Tap{0, (short)kOnesTap, 0};
      } else {
        t[i] = Tap{0, (short)kPadTap, (short)kPadTap};
      }
    }
    rc = upload_taps(ctx, p, &p->w_taps, t);
    const int n_pix = G.B * G.m * G.m;
    p->w_kblocks_total = (n_pix + kBlockK - 1) / kBlockK;
    const int out_tiles = p->w_mtiles * G.g * p->f_tiles;
    int splits = std::max(1, ctx->sm_count / out_tiles);
    splits = std::min(splits, std::max(1, p->w_kblocks_total / 8));  // at least 8 k-blocks per CTA
    p->w_kblocks_per_split = (p->w_kblocks_total + splits - 1) / splits;
    p->w_splits = (p->w_kblocks_total + p->w_kblocks_per_split - 1) / p->w_kblocks_per_split;
    if (rc == CCT_OK)
      rc = dev_alloc(ctx, p, &p->w_partial,
                     (size_t)p->w_splits * G.g * p->f_tiles * p->w_mtiles * kTileM * p->f_npad);
  }
  // ---- data gradient: one gather problem per stride phase
  if (rc == CCT_OK) {
    p->d_tiles = channel_tiles(G.Dg);
    p->d_n = G.Dg / p->d_tiles;
    p->d_npad = round_up(p->d_n, 16);
    for (int py = 0; py < G.s && rc == CCT_OK; ++py)
      for (int px = 0; px < G.s && rc == CCT_OK; ++px) {
        DgradPhase ph;
        ph.py = py; ph.px = px;
        ph.jh = py < G.k ? (G.k - py + G.s - 1) / G.s : 0;
        ph.jw = px < G.k ? (G.k - px + G.s - 1) / G.s : 0;
        ph.y0 = ((py - G.p) % G.s + G.s) % G.s;
        ph.x0 = ((px - G.p) % G.s + G.s) % G.s;
        ph.qh = ph.y0 < G.n ? (G.n - ph.y0 + G.s - 1) / G.s : 0;
        ph.qw = ph.x0 < G.n ? (G.n - ph.x0 + G.s - 1) / G.s : 0;
        if (ph.qh == 0 || ph.qw == 0) continue;
        ph.ry0 = (ph.y0 + G.p - py) / G.s;
        ph.rx0 = (ph.x0 + G.p - px) / G.s;
        ph.k_real = G.og * ph.jh * ph.jw;
        ph.k_pad = std::max(kBlockK, round_up(ph.k_real, kBlockK));
        std::vector<Tap> t(ph.k_pad);
        for (int i = 0; i < ph.k_pad; ++i) {
          if (i < ph.k_real) {
            const int jx = i % ph.jw, jy = (i / ph.jw) % ph.jh, oc = i / (ph.jw * ph.jh);
            t[i] = Tap{oc * G.m * G.m - jy * G.m - jx, (short)-jy, (short)-jx};
          } else {
            t[i] = Tap{0, (short)kPadTap, (short)kPadTap};
          }
        }
        rc = upload_taps(ctx, p, &ph.taps, t);
        const size_t dw = (size_t)G.g * p->d_tiles * p->d_npad * ph.k_pad;
        if (rc == CCT_OK) rc = dev_alloc(ctx, p, &ph.w_hi, dw);
        if (rc == CCT_OK) rc = dev_alloc(ctx, p, &ph.w_lo, dw);
        p->phases.push_back(ph);
      }
  }
  if (rc == CCT_OK) rc = set_smem(ctx, gather_conv_kernel, kSmemLimit);
  if (rc == CCT_OK) rc = set_smem(ctx, wgrad_kernel, kSmemLimit);
  if (rc != CCT_OK) {
    umma_plan_destroy(ctx, p);
    return rc;
  }
  *out = p;
  return CCT_OK;
}

void umma_plan_destroy(cct_ctx* ctx, UmmaPlan* p) {
  if (!p) return;
  cudaFree(p->f_taps); cudaFree(p->f_whi); cudaFree(p->f_wlo);
  cudaFree(p->w_taps); cudaFree(p->w_partial);
  for (DgradPhase& ph : p->phases) { cudaFree(ph.taps); cudaFree(ph.w_hi); cudaFree(ph.w_lo); }
  delete p;
}

size_t umma_plan_workspace_bytes(const UmmaPlan* p) { return p->bytes; }

int umma_conv_forward(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* W, const float* bias, float* Y,
                      int relu, PhaseTimer* t) {
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;  // an earlier bounded wait gave up: do not pile up behind it
  const ConvGeom& G = p->G;
  const int vgroups = G.g * p->f_tiles;
  t->begin(4, ctx->stream);
  const size_t fw = (size_t)vgroups * p->f_npad * p->f_kpad;
  pack_fwd_kernel<<<pack_grid(ctx, fw), 256, 0, ctx->stream>>>(W, p->f_whi, p->f_wlo, vgroups, p->f_tiles, G.og, p->f_n,
                                                              p->f_npad, p->f_kreal, p->f_kpad);
  t->end(4, ctx->stream);
  CCT_CHECK_LAUNCH(ctx);
  GatherParams P{};
  P.in = X; P.out = Y; P.w_hi = p->f_whi; P.w_lo = p->f_wlo; P.taps = p->f_taps;
  P.bias = G.bias ? bias : nullptr;
  P.n_pix = G.B * G.m * G.m; P.q_h = G.m; P.q_w = G.m;
  P.iy_mul = G.s; P.iy_add = -G.p; P.ix_mul = G.s; P.ix_add = -G.p;
  P.in_lim = G.n;
  P.in_batch_stride = (long long)G.D * G.n * G.n;
  P.in_group_stride = G.Dg * G.n * G.n;
  P.tiles_per_group = p->f_tiles;
  P.oy_mul = 1; P.oy_add = 0; P.ox_mul = 1; P.ox_add = 0;
  P.out_pitch = G.m; P.out_plane = G.m * G.m;
  P.out_batch_stride = (long long)G.o * G.m * G.m;
  P.out_group_channels = G.og;
  P.n = p->f_n; P.n_pad = p->f_npad; P.k_pad = p->f_kpad;
  P.relu = relu;
  P.status = ctx->status_dev;
  P.dbg = dbg_knobs();
  dim3 grid((P.n_pix + kTileM - 1) / kTileM, vgroups);
  t->begin(0, ctx->stream);
  gather_conv_kernel<<<grid, kThreads, smem_bytes(P.n_pad), ctx->stream>>>(P);
  t->end(0, ctx->stream);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int umma_conv_backward(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* W, const float* dY, float* dX,
                       float* dW, float* db, PhaseTimer* t) {
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;
  const ConvGeom& G = p->G;
  // ---- weight + bias gradient
  {
    WgradParams P{};
    P.x = X; P.dy = dY; P.partial = p->w_partial; P.taps = p->w_taps;
    P.n_pix = G.B * G.m * G.m; P.m = G.m; P.mm = G.m * G.m; P.n = G.n; P.s = G.s; P.p = G.p;
    P.x_batch_stride = (long long)G.D * G.n * G.n;
    P.x_group_stride = G.Dg * G.n * G.n;
    P.dy_batch_stride = (long long)G.o * G.m * G.m;
    P.dy_group_channels = G.og;
    P.tiles_per_group = p->f_tiles;
    P.n_real = p->f_n; P.n_pad = p->f_npad;
    P.kblocks_total = p->w_kblocks_total; P.kblocks_per_split = p->w_kblocks_per_split;
    P.status = ctx->status_dev;
    P.dbg = dbg_knobs();
    const int vgroups = G.g * p->f_tiles;
    dim3 grid(p->w_mtiles, p->w_splits, vgroups);
    t->begin(1, ctx->stream);
    wgrad_kernel<<<grid, kThreads, smem_bytes(P.n_pad), ctx->stream>>>(P);
    t->end(1, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
    t->begin(2, ctx->stream);
    const size_t total = (size_t)vgroups * (p->f_kreal + 1) * p->f_n;
    wgrad_reduce_kernel<<<pack_grid(ctx, total), 256, 0, ctx->stream>>>(p->w_partial, dW, G.bias ? db : nullptr,
                                                                      p->w_splits, vgroups, p->f_tiles,
                                                                      p->w_mtiles * kTileM, p->f_n, p->f_npad,
                                                                      p->f_kreal, G.og);
    t->end(2, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  }
  // ---- data gradient
  if (dX) {
    const int vgroups = G.g * p->d_tiles;
    t->begin(3, ctx->stream);
    if ((int)p->phases.size() < G.s * G.s) {
      // some phase has no input pixels or was skipped: nothing writes those pixels otherwise
      CCT_CUDA(ctx, cudaMemsetAsync(dX, 0, (size_t)G.B * G.D * G.n * G.n * sizeof(float), ctx->stream));
    }
    for (DgradPhase& ph : p->phases) {
      const size_t dw = (size_t)vgroups * p->d_npad * ph.k_pad;
      pack_dgrad_kernel<<<pack_grid(ctx, dw), 256, 0, ctx->stream>>>(W, ph.w_hi, ph.w_lo, vgroups, p->d_tiles, G.og,
                                                                    G.Dg, G.k, G.s, ph.py, ph.px, ph.jh, ph.jw, p->d_n,
                                                                    p->d_npad, ph.k_real, ph.k_pad);
      CCT_CHECK_LAUNCH(ctx);
      GatherParams P{};
      P.in = dY; P.out = dX; P.w_hi = ph.w_hi; P.w_lo = ph.w_lo; P.taps = ph.taps; P.bias = nullptr;
      P.n_pix = G.B * ph.qh * ph.qw; P.q_h = ph.qh; P.q_w = ph.qw;
      P.iy_mul = 1; P.iy_add = ph.ry0; P.ix_mul = 1; P.ix_add = ph.rx0;
      P.in_lim = G.m;
      P.in_batch_stride = (long long)G.o * G.m * G.m;
      P.in_group_stride = G.og * G.m * G.m;
      P.tiles_per_group = p->d_tiles;
      P.oy_mul = G.s; P.oy_add = ph.y0; P.ox_mul = G.s; P.ox_add = ph.x0;
      P.out_pitch = G.n; P.out_plane = G.n * G.n;
      P.out_batch_stride = (long long)G.D * G.n * G.n;
      P.out_group_channels = G.Dg;
      P.n = p->d_n; P.n_pad = p->d_npad; P.k_pad = ph.k_pad;
      P.relu = 0;
      P.status = ctx->status_dev;
      P.dbg = dbg_knobs();
      dim3 grid((P.n_pix + kTileM - 1) / kTileM, vgroups);
      gather_conv_kernel<<<grid, kThreads, smem_bytes(P.n_pad), ctx->stream>>>(P);
      CCT_CHECK_LAUNCH(ctx);
    }
    t->end(3, ctx->stream);
  }
  return CCT_OK;
}
