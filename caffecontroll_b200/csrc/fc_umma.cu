// Fully connected layers on the Blackwell tensor cores (FullyConnectedBridge: src/bridges/FullyConnectedBridge_impl.hxx).
//
// The three contractions of the bridge
//   forward        Y[b][o]  = sum_k X[b][k]  * W[o][k]          (:196-215, sgemm_new NoTrans x Trans)
//   data gradient  dX[b][k] = sum_o dY[b][o] * W[o][k]          (:305, NoTrans x NoTrans)
//   weight gradient dW[o][k] = sum_b dY[b][o] * X[b][k]         (:311, Trans x NoTrans)
// are one kernel, fc_gemm_kernel:   out[n][m] = sum_r A(m, r) * B(n, r)   with M = 128 lanes per tile, N <= 256.
// Both operands are fetched from global memory by TMA as raw fp32 tiles of 32 reduction indices.  An operand whose
// reduction index is contiguous in memory ("K-major": W in the forward pass, X, dY) lands as rows of 128 bytes with
// the 128-byte swizzle; an operand whose row index is contiguous ("MN-major": W in the data gradient, X and dY in the
// weight gradient, where the reduction runs over the batch) lands as 32 x 32 boxes with the 128-byte swizzle of
// 32-byte atoms, the only shared-memory layout tcgen05.mma accepts for transposed 32-bit operands.  No operand is ever
// transposed or re-packed in global memory: the weights stream from HBM exactly once per contraction.
//
// 3xTF32: kind::tf32 reads the upper 19 bits of every fp32 operand word, so the raw tile is the "hi" operand as it
// stands; transform warps compute lo = x - hi element-wise into a second tile of the same layout (an element-wise pass
// is layout-agnostic, so it serves both swizzles), and three MMAs per k-step (lo*hi + hi*lo + hi*hi) accumulate in
// fp32 in tensor memory.  Long reductions are split over CTAs (bounded accumulation chains, as in the convolution
// kernels); a small kernel adds the partial sums in split order and applies bias / ReLU / dropout (forward) or the
// masks of the bridges in front of the layer (data gradient).
#include <algorithm>
#include <cstdio>
#include <new>

#include "cct_internal.h"
#include "umma_ptx.cuh"

namespace {

constexpr int kFcEpiWarps = 4, kFcTmaWarp = 4, kFcMmaWarp = 5, kFcXformWarp0 = 6, kFcXformWarps = 8;
constexpr int kFcThreads = (kFcXformWarp0 + kFcXformWarps) * 32;  // 448
constexpr int kFcMaxStages = 4;
constexpr int kFcMaxChainKblocks = 96;  // k-blocks of 32 per partial sum: the tensor core's fp32 accumulate truncates
constexpr uint32_t kFcATile = kTileM * 128u;  // bytes of one 128 x 32 fp32 tile

struct FcGemmParams {
  float* out;               // out[split * split_stride + n * ld_out + m]
  long long ld_out, split_stride;
  int M, N;                 // extents of the output (m fastest in memory)
  int n_pad;                // accumulator columns per tile: N rounded up (a multiple of 32 for MN-major B)
  int m_tiles, n_tiles, splits, kblocks_total, kblocks_per_split;
  int a_mn, b_mn;           // 1: the operand is MN-major (row index contiguous in memory)
  int a_tmem;               // 1: the A operand is split into tensor memory (hi and lo), the MMAs read it from there
  int stages, acc_bufs;
  int tmem_cols;            // tensor-memory columns the CTA allocates: 512, or 256 when two CTAs share an SM
  int* status;
};

struct FcSmem {
  uint32_t b_tile_bytes, b_off, stage_bytes, bars_off, total;
};
__host__ __device__ inline FcSmem fc_smem(int n_pad, int stages, int a_tmem) {
  FcSmem L;
  L.b_tile_bytes = (uint32_t)n_pad * 128u;
  L.b_off = (a_tmem ? 1u : 2u) * kFcATile;            // A raw, (A lo unless A's halves live in tensor memory,)
  L.stage_bytes = L.b_off + 2u * L.b_tile_bytes;      // B raw, B lo
  L.bars_off = (uint32_t)stages * L.stage_bytes;
  L.total = L.bars_off + 8u * (3 * kFcMaxStages + 4) + 16u;
  return L;
}

// Shared-memory descriptor of an MN-major fp32 operand: 32 x 32 boxes (row = one reduction index, 128 bytes = 32
// consecutive m), 128-byte swizzle with 32-byte atoms (layout type 1).  One MMA reads 8 reduction indices = two atoms
// of four rows, 512 bytes apart; consecutive 32-wide chunks of m are one box (4096 bytes) apart.
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(4096u >> 4) << 16) | ((uint64_t)(512u >> 4) << 32) |
         (1ull << 46) | (1ull << 61);
}

__global__ void __launch_bounds__(kFcThreads, 2)
    fc_gemm_kernel(const __grid_constant__ FcGemmParams P, const __grid_constant__ CUtensorMap a_map,
                   const __grid_constant__ CUtensorMap b_map) {
  pdl_wait();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const FcSmem L = fc_smem(P.n_pad, P.stages, P.a_tmem);
  const uint32_t bars = base + L.bars_off;
  // raw[s]: the stage's TMA bytes have landed; lo[s]: the transform warps have written the lo tiles; empty[s]: the
  // stage's MMAs have finished (tcgen05.commit), the TMA thread may refill it.
  const uint32_t raw_bar = bars, lo_bar = raw_bar + 8u * kFcMaxStages, empty_bar = lo_bar + 8u * kFcMaxStages,
                 acc_full = empty_bar + 8u * kFcMaxStages, acc_empty = acc_full + 16u, tmem_slot = acc_empty + 16u;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < kFcMaxStages; ++s) {
      mbar_init(raw_bar + 8u * s, 1);
      mbar_init(lo_bar + 8u * s, kFcXformWarps);
      mbar_init(empty_bar + 8u * s, 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + 8u * b, 1); mbar_init(acc_empty + 8u * b, kFcEpiWarps); }
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, (uint32_t)P.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  const uint32_t a_col0 = (uint32_t)(P.acc_bufs * P.n_pad);  // A stages (64 columns each) behind the accumulators
  const int total_tiles = P.m_tiles * P.n_tiles * P.splits;
  bool failed = false;
  // tile t -> (split, n-tile, m-tile), m-tile fastest; k-blocks [kb0, kb1)
  auto tile_of = [&](int t, int& mt, int& nt, int& split, int& kb0, int& kb1) {
    mt = t % P.m_tiles;
    const int r = t / P.m_tiles;
    nt = r % P.n_tiles;
    split = r / P.n_tiles;
    kb0 = split * P.kblocks_per_split;
    kb1 = min(P.kblocks_total, kb0 + P.kblocks_per_split);
  };

  if (warp == kFcTmaWarp) {
    if (lane == 0) {
      Ring ring;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        int mt, nt, split, kb0, kb1;
        tile_of(t, mt, nt, split, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb, ring.advance(P.stages)) {
          const int s = ring.idx;
          if (ring.use > 0) mbar_wait<false>(empty_bar + 8u * s, (uint32_t)(ring.use - 1) & 1u, failed, P.status, 0x1100);
          const uint32_t st = base + (uint32_t)s * L.stage_bytes, a_raw = st, b_raw = st + L.b_off;
          const uint32_t bar = raw_bar + 8u * s;
          mbar_expect_tx(bar, kFcATile + L.b_tile_bytes);
          if (P.a_mn) {
#pragma unroll
            for (int j = 0; j < 4; ++j) tma_load_2d(a_raw + j * 4096u, &a_map, mt * kTileM + j * 32, kb * kBlockK, bar);
          } else {
            tma_load_2d(a_raw, &a_map, kb * kBlockK, mt * kTileM, bar);
          }
          if (P.b_mn) {
            for (int j = 0; j < P.n_pad / 32; ++j)
              tma_load_2d(b_raw + j * 4096u, &b_map, nt * P.n_pad + j * 32, kb * kBlockK, bar);
          } else {
            tma_load_2d(b_raw, &b_map, kb * kBlockK, nt * P.n_pad, bar);
          }
        }
      }
    }
  } else if (warp == kFcMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(P.n_pad) | (P.a_mn ? 1u << 15 : 0u) | (P.b_mn ? 1u << 16 : 0u);
      const uint32_t idesc_ts = make_idesc(P.n_pad) | (P.b_mn ? 1u << 16 : 0u);  // A from tensor memory: lanes x K
      Ring ring;
      int tile_iter = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_iter) {
        int mt, nt, split, kb0, kb1;
        tile_of(t, mt, nt, split, kb0, kb1);
        const int buf = tile_iter & (P.acc_bufs - 1), use = tile_iter >> (P.acc_bufs - 1);
        if (use > 0) mbar_wait<false>(acc_empty + 8u * buf, (uint32_t)(use - 1) & 1u, failed, P.status, 0x1200);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * P.n_pad);
        for (int kb = kb0; kb < kb1; ++kb, ring.advance(P.stages)) {
          const int s = ring.idx;
          mbar_wait<false>(raw_bar + 8u * s, (uint32_t)ring.use & 1u, failed, P.status, 0x1300);
          mbar_wait<false>(lo_bar + 8u * s, (uint32_t)ring.use & 1u, failed, P.status, 0x1400);
          tc_fence_after();
          const uint32_t st = base + (uint32_t)s * L.stage_bytes;
          const uint32_t a_raw = st, a_lo = st + kFcATile, b_raw = st + L.b_off, b_lo = b_raw + L.b_tile_bytes;
          if (P.a_tmem) {
            const uint32_t t_hi = tmem_base + a_col0 + (uint32_t)(s * 64), t_lo = t_hi + 32u;
#pragma unroll
            for (int j = 0; j < kBlockK / 8; ++j) {
              const uint64_t bh = P.b_mn ? make_desc_mn(b_raw + j * 1024u) : make_desc(b_raw) + (uint64_t)(j * 2);
              const uint64_t bl = P.b_mn ? make_desc_mn(b_lo + j * 1024u) : make_desc(b_lo) + (uint64_t)(j * 2);
              umma_tf32_ts(d_tmem, t_lo + (uint32_t)(j * 8), bh, idesc_ts, (kb == kb0 && j == 0) ? 0u : 1u);
              umma_tf32_ts(d_tmem, t_hi + (uint32_t)(j * 8), bl, idesc_ts, 1u);
              umma_tf32_ts(d_tmem, t_hi + (uint32_t)(j * 8), bh, idesc_ts, 1u);
            }
            umma_commit(empty_bar + 8u * s);
            continue;
          }
#pragma unroll
          for (int j = 0; j < kBlockK / 8; ++j) {
            // K-major: 8 reduction indices = 32 bytes along the swizzled row; MN-major: 8 rows of 128 bytes
            const uint64_t ah = P.a_mn ? make_desc_mn(a_raw + j * 1024u) : make_desc(a_raw) + (uint64_t)(j * 2);
            const uint64_t al = P.a_mn ? make_desc_mn(a_lo + j * 1024u) : make_desc(a_lo) + (uint64_t)(j * 2);
            const uint64_t bh = P.b_mn ? make_desc_mn(b_raw + j * 1024u) : make_desc(b_raw) + (uint64_t)(j * 2);
            const uint64_t bl = P.b_mn ? make_desc_mn(b_lo + j * 1024u) : make_desc(b_lo) + (uint64_t)(j * 2);
            umma_tf32_ss(d_tmem, al, bh, idesc, (kb == kb0 && j == 0) ? 0u : 1u);
            umma_tf32_ss(d_tmem, ah, bl, idesc, 1u);
            umma_tf32_ss(d_tmem, ah, bh, idesc, 1u);
          }
          umma_commit(empty_bar + 8u * s);
        }
        umma_commit(acc_full + 8u * buf);
      }
    }
  } else if (warp >= kFcXformWarp0) {
    // ---- lo = x - (x with the low 13 mantissa bits cleared), element-wise over the stage's two raw tiles
    const int xt = tid - kFcXformWarp0 * 32;
    constexpr int kXThreads = kFcXformWarps * 32;
    const int a_vec = kFcATile / 16, b_vec = (int)(L.b_tile_bytes / 16);
    Ring ring;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      int mt, nt, split, kb0, kb1;
      tile_of(t, mt, nt, split, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ring.advance(P.stages)) {
        const int s = ring.idx;
        mbar_wait(raw_bar + 8u * s, (uint32_t)ring.use & 1u, failed, P.status, 0x1500);
        uint8_t* st = base_ptr + (size_t)s * L.stage_bytes;
        if (P.a_tmem) {
          // The stage's tensor-memory columns are free: the TMA thread refilled the stage only after the MMAs that read
          // them had completed (empty barrier), and this thread has just seen that refill land.
          tc_fence_after();
          // A: thread = (row m of the tile = tensor-memory lane, half of the k-block's 32 reduction indices).  Its 16
          // values come out of the swizzled tile the TMA wrote; hi and lo go to the stage's 64 tensor-memory columns.
          const int q = warp & 3, half = (warp - kFcXformWarp0) >> 2;
          const int m = q * 32 + lane;
          float x[16];
          if (P.a_mn) {
            // 32 x 32 boxes, row = reduction index (128 bytes), 32-byte chunks XORed with the row index mod 4
            const uint8_t* box = st + (size_t)(m >> 5) * 4096u;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t k = (uint32_t)(half * 16 + i);
              const uint32_t off = k * 128u + (uint32_t)(m & 31) * 4u;
              x[i] = *reinterpret_cast<const float*>(box + (off ^ ((k & 3u) << 5)));
            }
          } else {
            // rows of 128 bytes, 16-byte chunks XORed with the row index mod 8
            const uint8_t* rowp = st + (size_t)m * 128u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t c = (uint32_t)(half * 4 + i);
              const float4 v4 = *reinterpret_cast<const float4*>(rowp + ((c ^ (uint32_t)(m & 7)) << 4));
              x[4 * i] = v4.x; x[4 * i + 1] = v4.y; x[4 * i + 2] = v4.z; x[4 * i + 3] = v4.w;
            }
          }
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a_col0 + (uint32_t)(s * 64 + half * 16);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) split_tf32_trunc(x[c * 8 + e], hi[e], lo[e]);
            tmem_st8(taddr + (uint32_t)(c * 8), hi);
            tmem_st8(taddr + 32u + (uint32_t)(c * 8), lo);
          }
        }
        for (int i = P.a_tmem ? a_vec + xt : xt; i < a_vec + b_vec; i += kXThreads) {
          const bool in_a = i < a_vec;
          uint8_t* src = in_a ? st + (size_t)i * 16 : st + L.b_off + (size_t)(i - a_vec) * 16;
          const float4 x = *reinterpret_cast<const float4*>(src);
          float4 l;
          l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
          l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
          l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
          l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
          *reinterpret_cast<float4*>(src + (in_a ? kFcATile : L.b_tile_bytes)) = l;
        }
        fence_proxy_async_smem();
        if (P.a_tmem) {
          tmem_wait_st();
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(lo_bar + 8u * s);
      }
    }
  } else {
    // ---- epilogue: lane = m (contiguous in the output), one column = one n
    const int quarter = warp;  // warps 0-3 own tensor-memory lanes 32 * warp ...
    int tile_iter = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_iter) {
      int mt, nt, split, kb0, kb1;
      tile_of(t, mt, nt, split, kb0, kb1);
      const int buf = tile_iter & (P.acc_bufs - 1), use = tile_iter >> (P.acc_bufs - 1);
      mbar_wait(acc_full + 8u * buf, (uint32_t)use & 1u, failed, P.status, 0x1600);
      tc_fence_after();
      const int m = mt * kTileM + quarter * 32 + lane;
      const int n0 = nt * P.n_pad;
      float* op = P.out + (long long)split * P.split_stride + (long long)n0 * P.ld_out + m;
      const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P.n_pad);
      const uint32_t live = (m < P.M && !failed) ? 1u : 0u;
      for (int c = 0; c < P.n_pad / 16; ++c) {
        float v[16];
        tmem_ld16(acc + (uint32_t)(c * 16), v);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int n = n0 + c * 16 + j;
          if (live && n < P.N) op[(long long)(c * 16 + j) * P.ld_out] = v[j];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + 8u * buf);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, (uint32_t)P.tmem_cols);
}

// Y[b][o] = act(bias[o] + sum over splits of partial[s][b][o]), act = optional ReLU then optional dropout
// (DropoutBridge forward: x * mask * scale, src/bridges/DropoutBridge_impl.hxx:71-74).  Splits are added in order.
__global__ void fc_reduce_fwd_kernel(const float* __restrict__ partial, int splits, size_t split_stride,
                                     const float* __restrict__ bias, float* __restrict__ Y, size_t total, int O, int relu,
                                     const uint32_t* __restrict__ drop_mask, float drop_scale) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(size_t)s * split_stride + i];
    if (bias) acc += bias[i % O];
    if (relu) acc = fmaxf(acc, 0.f);
    if (drop_mask) acc = acc * (float)(drop_mask[i] != 0u) * drop_scale;
    Y[i] = acc;
  }
}

// dX[b][k] = (sum over splits) x [X > 0] (the ReLU bridge in front, src/kernels/relu.hxx:35-43) x mask * scale (the
// dropout bridge in front, DropoutBridge::backward).
__global__ void fc_reduce_dgrad_kernel(const float* __restrict__ partial, int splits, size_t split_stride,
                                       float* __restrict__ dX, size_t total, const float* __restrict__ X, int in_relu,
                                       const uint32_t* __restrict__ drop_mask, float drop_scale) {
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(size_t)s * split_stride + i];
    if (drop_mask) acc = acc * (float)(drop_mask[i] != 0u) * drop_scale;
    if (in_relu) acc = acc * (X[i] > 0.f ? 1.f : 0.f);
    dX[i] = acc;
  }
}

// db[o] = sum_b dY[b][o] (FullyConnectedBridge_impl.hxx:298: backward_bias_fc).  A block of 32 x 8 threads owns 32
// outputs: thread (x, y) adds the images y, y + 8, ... in order with sixteen loads in flight, then the eight partial sums
// of an output are added in a fixed order - deterministic, and two memory round trips instead of B.
__global__ void __launch_bounds__(256) fc_bias_grad_kernel(const float* __restrict__ dY, float* __restrict__ db, int B, int O) {
  pdl_wait();
  __shared__ float part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int o = blockIdx.x * 32 + tx;
  float acc = 0.f;
  if (o < O) {
    int b = ty;
    for (; b + 8 * 15 < B; b += 8 * 16) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __ldg(dY + (size_t)(b + 8 * j) * O + o);
#pragma unroll
      for (int j = 0; j < 16; ++j) acc += v[j];
    }
    for (; b < B; b += 8) acc += dY[(size_t)b * O + o];
  }
  part[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && o < O) {
    float t = part[0][tx];
#pragma unroll
    for (int y = 1; y < 8; ++y) t += part[y][tx];
    db[o] = t;
  }
}

int fc_round_up(int v, int a) { return (v + a - 1) / a * a; }

// rows x cols fp32 matrix, cols contiguous.  K-major use: box = 32 cols (reduction) x box_rows, 128-byte swizzle.
// MN-major use: box = 32 cols (the operand's row index) x 32 rows (reduction), 128-byte swizzle with 32-byte atoms.
int fc_make_map(cct_ctx* ctx, CUtensorMap* map, const float* ptr, size_t rows, size_t cols, int box_rows, bool mn_major) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    ctx->last_error = "cuTensorMapEncodeTiled is not available from this driver";
    return CCT_ERR_CUDA;
  }
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * sizeof(float)};
  const cuuint32_t box[2] = {32u, (cuuint32_t)(mn_major ? 32 : box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE,
                         mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    ctx->last_error = "cuTensorMapEncodeTiled (fully connected operand) failed with code " + std::to_string((int)r);
    return CCT_ERR_CUDA;
  }
  return CCT_OK;
}

}  // namespace

struct cct_fc_plan {
  cct_ctx* ctx = nullptr;
  int B = 0, K = 0, O = 0, bias = 0;
  float* partial = nullptr;  // split partial sums of the forward pass and of the data gradient
  size_t partial_elems = 0, bytes = 0;
  int f_splits = 1, f_kps = 1, d_splits = 1, d_kps = 1;
  PhaseTimer timer;
};

namespace {

// Splits of a reduction of `kblocks` k-blocks over `tiles` output tiles: about one CTA per SM, chains bounded.
void fc_pick_splits(int slots, int tiles, int kblocks, int* splits, int* kps) {
  int s = std::max(1, slots / std::max(1, tiles));
  s = std::max(s, (kblocks + kFcMaxChainKblocks - 1) / kFcMaxChainKblocks);
  s = std::min(s, std::max(1, kblocks / 4));
  *kps = (kblocks + s - 1) / s;
  *splits = (kblocks + *kps - 1) / *kps;
}

// Accumulator width of the forward pass and the data gradient (N = batch): at most 128 columns, so that two CTAs fit on
// an SM (256 tensor-memory columns and half the shared memory each) - two pipelines of TMA, transform and MMA issue per
// SM hide each other's latencies, which one CTA with two 96 KB stages cannot.
int fc_batch_tile(int batch) { return fc_round_up(std::min(batch, 128), 16); }

int fc_launch(cct_ctx* ctx, FcGemmParams& P, const CUtensorMap& a_map, const CUtensorMap& b_map) {
  const bool pair = P.a_tmem && P.n_pad <= 128;  // two CTAs per SM
  const uint32_t stage = fc_smem(P.n_pad, 1, P.a_tmem).stage_bytes;
  const uint32_t budget = pair ? 113u * 1024u : (uint32_t)kSmemLimit;
  P.stages = std::min(kFcMaxStages, (int)((budget - 2048) / stage));
  if (P.stages < 2) {
    ctx->last_error = "fully connected tile does not fit in shared memory twice";
    return CCT_ERR_UNSUPPORTED;
  }
  // Tensor memory = accumulator buffers (+ 64 columns per stage for an A operand kept there).
  P.tmem_cols = pair ? 256 : 512;
  if (P.a_tmem) P.stages = std::min(P.stages, (P.tmem_cols - P.n_pad) / 64);
  const int a_cols = P.a_tmem ? P.stages * 64 : 0;
  P.acc_bufs = 2 * P.n_pad + a_cols <= P.tmem_cols ? 2 : 1;
  const size_t smem = fc_smem(P.n_pad, P.stages, P.a_tmem).total + 1024;
  P.status = ctx->status_dev;
  const int tiles = P.m_tiles * P.n_tiles * P.splits;
  launch_pdl(fc_gemm_kernel, dim3(std::min(tiles, (pair ? 2 : 1) * ctx->launch_sms())), dim3(kFcThreads), smem, ctx->stream, P, a_map, b_map);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int fc_ew_grid(cct_ctx* ctx, size_t total) {
  return (int)std::max<size_t>(1, std::min<size_t>((total + 255) / 256, (size_t)ctx->sm_count * 8));
}

}  // namespace

extern "C" {

int cct_fc_plan_create(cct_ctx* ctx, int batch, int in_features, int out_features, int bias_term, cct_fc_plan** out) {
  if (!ctx || !out) return CCT_ERR_INVALID;
  *out = nullptr;
  if (batch <= 0 || in_features <= 0 || out_features <= 0) return CCT_ERR_INVALID;
  // TMA needs row pitches that are multiples of 16 bytes; the weight gradient reads X and dY with the batch as the
  // reduction, in boxes of 32 columns.
  if (in_features % 4 || out_features % 4) {
    ctx->last_error = "fully connected layers need in_features and out_features that are multiples of 4";
    return CCT_ERR_UNSUPPORTED;
  }
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  cct_fc_plan* p = new (std::nothrow) cct_fc_plan();
  if (!p) return CCT_ERR_NOMEM;
  p->ctx = ctx; p->B = batch; p->K = in_features; p->O = out_features; p->bias = bias_term != 0;
  const int n_tiles = (batch + fc_batch_tile(batch) - 1) / fc_batch_tile(batch);
  fc_pick_splits(2 * ctx->sm_count, ((out_features + kTileM - 1) / kTileM) * n_tiles, (in_features + kBlockK - 1) / kBlockK,
                 &p->f_splits, &p->f_kps);
  fc_pick_splits(2 * ctx->sm_count, ((in_features + kTileM - 1) / kTileM) * n_tiles, (out_features + kBlockK - 1) / kBlockK,
                 &p->d_splits, &p->d_kps);
  p->partial_elems = std::max((size_t)p->f_splits * batch * out_features, (size_t)p->d_splits * batch * in_features);
  if (cudaMalloc((void**)&p->partial, p->partial_elems * sizeof(float)) != cudaSuccess) {
    ctx->last_error = "cudaMalloc of the fully connected layer's split partial sums failed";
    delete p;
    return CCT_ERR_NOMEM;
  }
  p->bytes = p->partial_elems * sizeof(float);
  const cudaError_t e = cudaFuncSetAttribute(fc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
  if (e != cudaSuccess) {
    ctx->last_error = std::string("cudaFuncSetAttribute(fc_gemm_kernel): ") + cudaGetErrorString(e);
    cudaFree(p->partial);
    delete p;
    return CCT_ERR_CUDA;
  }
  *out = p;
  return CCT_OK;
}

int cct_fc_plan_destroy(cct_fc_plan* plan) {
  if (!plan) return CCT_ERR_INVALID;
  cudaSetDevice(plan->ctx->device);
  cudaStreamSynchronize(plan->ctx->stream);
  cudaFree(plan->partial);
  for (cudaEvent_t e : plan->timer.ev)
    if (e) cudaEventDestroy(e);
  delete plan;
  return CCT_OK;
}

int cct_fc_plan_workspace_bytes(const cct_fc_plan* plan, size_t* bytes) {
  if (!plan || !bytes) return CCT_ERR_INVALID;
  *bytes = plan->bytes;
  return CCT_OK;
}

int cct_fc_forward(cct_fc_plan* plan, const float* X, const float* W, const float* bias, float* Y, int relu,
                   const uint32_t* drop_mask, float drop_scale) {
  if (!plan || !X || !W || !Y || (plan->bias && !bias)) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const int B = plan->B, K = plan->K, O = plan->O;
  FcGemmParams P{};
  P.M = O; P.N = B;
  P.n_pad = fc_batch_tile(B);
  P.m_tiles = (O + kTileM - 1) / kTileM; P.n_tiles = (B + P.n_pad - 1) / P.n_pad;
  P.kblocks_total = (K + kBlockK - 1) / kBlockK; P.splits = plan->f_splits; P.kblocks_per_split = plan->f_kps;
  P.a_mn = 0; P.b_mn = 0; P.a_tmem = 1;
  P.out = plan->partial; P.ld_out = O; P.split_stride = (long long)B * O;
  CUtensorMap a_map, b_map;
  int rc = fc_make_map(ctx, &a_map, W, O, K, kTileM, false);
  if (rc == CCT_OK) rc = fc_make_map(ctx, &b_map, X, B, K, P.n_pad, false);
  if (rc != CCT_OK) return rc;
  plan->timer.begin(0, ctx->stream);
  rc = fc_launch(ctx, P, a_map, b_map);
  if (rc != CCT_OK) return rc;
  const size_t total = (size_t)B * O;
  launch_pdl(fc_reduce_fwd_kernel, dim3(fc_ew_grid(ctx, total)), dim3(256), 0, ctx->stream, plan->partial, P.splits, (size_t)P.split_stride,
                                                                      plan->bias ? bias : nullptr, Y, total, O, relu,
                                                                      drop_mask, drop_scale);
  plan->timer.end(0, ctx->stream);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int cct_fc_backward(cct_fc_plan* plan, const float* X, const float* W, const float* dY, float* dX, float* dW, float* db,
                    int in_relu, const uint32_t* in_drop_mask, float in_drop_scale) {
  if (!plan || !X || !W || !dY || !dW || (plan->bias && !db)) return CCT_ERR_INVALID;
  cct_ctx* ctx = plan->ctx;
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  const int B = plan->B, K = plan->K, O = plan->O;
  int rc;
  // ---- weight gradient: out = dW[o][k] (m = k, n = o), reduction over the batch; both operands MN-major
  {
    FcGemmParams P{};
    P.M = K; P.N = O;
    P.n_pad = fc_round_up(std::min(O, 256), 32);
    P.m_tiles = (K + kTileM - 1) / kTileM; P.n_tiles = (O + P.n_pad - 1) / P.n_pad;
    P.kblocks_total = (B + kBlockK - 1) / kBlockK; P.splits = 1; P.kblocks_per_split = P.kblocks_total;
    P.a_mn = 1; P.b_mn = 1;
    P.out = dW; P.ld_out = K; P.split_stride = 0;
    CUtensorMap a_map, b_map;
    rc = fc_make_map(ctx, &a_map, X, B, K, 32, true);
    if (rc == CCT_OK) rc = fc_make_map(ctx, &b_map, dY, B, O, 32, true);
    if (rc != CCT_OK) return rc;
    plan->timer.begin(1, ctx->stream);
    rc = fc_launch(ctx, P, a_map, b_map);
    if (rc != CCT_OK) return rc;
    if (plan->bias) launch_pdl(fc_bias_grad_kernel, dim3((O + 31) / 32), dim3(256), 0, ctx->stream, dY, db, B, O);
    plan->timer.end(1, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  }
  // ---- data gradient: out = dX[b][k] (m = k, n = b), reduction over o; A = W read MN-major, B = dY K-major
  if (dX) {
    FcGemmParams P{};
    P.M = K; P.N = B;
    P.n_pad = fc_batch_tile(B);
    P.m_tiles = (K + kTileM - 1) / kTileM; P.n_tiles = (B + P.n_pad - 1) / P.n_pad;
    P.kblocks_total = (O + kBlockK - 1) / kBlockK; P.splits = plan->d_splits; P.kblocks_per_split = plan->d_kps;
    P.a_mn = 1; P.b_mn = 0; P.a_tmem = 1;
    P.out = plan->partial; P.ld_out = K; P.split_stride = (long long)B * K;
    CUtensorMap a_map, b_map;
    rc = fc_make_map(ctx, &a_map, W, O, K, 32, true);
    if (rc == CCT_OK) rc = fc_make_map(ctx, &b_map, dY, B, O, P.n_pad, false);
    if (rc != CCT_OK) return rc;
    plan->timer.begin(3, ctx->stream);
    rc = fc_launch(ctx, P, a_map, b_map);
    if (rc != CCT_OK) return rc;
    const size_t total = (size_t)B * K;
    launch_pdl(fc_reduce_dgrad_kernel, dim3(fc_ew_grid(ctx, total)), dim3(256), 0, ctx->stream, plan->partial, P.splits, (size_t)P.split_stride,
                                                                          dX, total, X, in_relu, in_drop_mask, in_drop_scale);
    plan->timer.end(3, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  }
  return CCT_OK;
}

int cct_fc_plan_enable_timing(cct_fc_plan* plan, int enable) {
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

int cct_fc_plan_last_timings(cct_fc_plan* plan, float ms[5]) {
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

}  // extern "C"
