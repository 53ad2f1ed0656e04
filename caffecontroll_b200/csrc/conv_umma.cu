// Implicit-GEMM convolution on the Blackwell tensor cores (CCT_ALGO_UMMA_3XTF32).
//
// All three contractions of the convolution bridge run on tcgen05.mma (kind::tf32, M = 128, fp32 accumulators in
// tensor memory).  The lowered matrix of the reference (type-1 lowering, one row of k*k*D values per output pixel)
// is never written to global memory: producer threads gather each 128 x 32 tile of it straight from the NCHW
// tensors, splitting every fp32 value into hi = its tf32 part and lo = x - hi on the way.  Three MMAs per k-step
// (hi*hi + hi*lo + lo*hi) recover fp32-level accuracy ("3xTF32"); flops are counted once.
//
//   forward        Y[pix][o]   = sum_k  Lowered(X)[pix][k] * W[o][k]            (+ bias, optional ReLU)
//   data gradient  dX[q][(d,py,px)] = sum_kk Gathered(dY)[q][kk] * Wd[(d,py,px)][kk]   kk = (filter, jy, jx)
//                  - the inverse lowering (col2im) written as a gather over s x s blocks of input pixels q: every
//                  block sums the taps that touch it inside the accumulator and the epilogue scatters the columns
//                  (depth to space), so there is no atomics and the result is deterministic.
//   weight gradient dW[kk][o]  = sum_pix Lowered(X)[pix][kk] * dY[pix][o]        split over pixel ranges across
//                  CTAs, partial sums to scratch, fixed-order reduction.
//
// gather_conv_kernel serves the forward pass, the data gradient and (lanes = rows of the lowered matrix, dY as the
// pre-split TMA operand) the weight gradient of larger layers: gathered operand in tensor memory, the other operand
// streamed by TMA into swizzled shared memory, warp-specialised roles.  Shorter lowered matrices have their own weight-
// gradient kernels: wgrad_ts_kernel (257 .. 384 rows: dY through tensor memory, the lowered rows staged in shared memory)
// and wgrad_kernel (anything shorter, and the allocation-free entry point: both operands staged in shared memory).
// Every kernel starts with pdl_wait() and is launched with launch_pdl (cct_internal.h).  Every mbarrier wait is bounded: when it runs out the thread
// sets the context's status word, stops waiting on anything else, and the kernel still frees its tensor memory.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda.h>

#include "cct_internal.h"
#include "umma_ptx.cuh"

namespace {

constexpr int kMaxTapsPerAxis = 15;
// Longest accumulation chain of a weight-gradient partial sum, in k-blocks of 32 pixels.  Measured against a
// double-accumulating CPU reference, AlexNet conv1's dW was off by 7.7e-5 (max-norm relative) with chains of 327
// k-blocks, the error pointing towards zero (truncating accumulate), and it shrinks in proportion to the chain.
constexpr int kMaxChainKblocks = 176;
constexpr uint32_t kPadBit = 0x80000000u;  // never set in a pixel's validity mask: marks padding entries

// One entry per reduction index of a gathered operand: element offset from the pixel's tap origin, and the tap's
// row / column as mask bits.  The tap is in bounds for a pixel iff (pixel_mask & bits) == bits, where bit i (rows) and
// bit 16+j (columns) of the pixel's mask say whether tap row i / tap column j falls inside the gathered plane.
struct alignas(8) MaskTap {
  int off;
  uint32_t bits;
};

// Bits [lo, hi) set; 0 <= lo, hi <= 15.
__device__ __forceinline__ uint32_t bit_range(int lo, int hi) {
  lo = max(lo, 0);
  hi = min(hi, kMaxTapsPerAxis);
  return hi > lo ? ((1u << hi) - 1u) & ~((1u << lo) - 1u) : 0u;
}

// v = ((mask & bits) == bits) ? *p : 0 as straight-line predicated code: written through the compiler, each guarded
// load becomes a branch around the load, and the branch bookkeeping costs more issue slots than the load itself.
__device__ __forceinline__ float ldg_if_bits(const float* p, uint32_t mask, uint32_t bits) {
  float v;
  asm volatile(
      "{\n\t.reg .pred q;\n\t.reg .b32 t;\n\t"
      "and.b32 t, %2, %3;\n\t"
      "setp.eq.u32 q, t, %3;\n\t"
      "mov.f32 %0, 0f00000000;\n\t"
      "@q ld.global.nc.f32 %0, [%1];\n\t}"
      : "=f"(v)
      : "l"(p), "r"(mask), "r"(bits));
  return v;
}
// v = ((a & b) == 0) ? *p : 0, same form (a, b: "what is out of bounds here" against "what this entry needs").
__device__ __forceinline__ float ldg_if_clear(const float* p, uint32_t a, uint32_t b) {
  float v;
  asm volatile(
      "{\n\t.reg .pred q;\n\t.reg .b32 t;\n\t"
      "and.b32 t, %2, %3;\n\t"
      "setp.eq.u32 q, t, 0;\n\t"
      "mov.f32 %0, 0f00000000;\n\t"
      "@q ld.global.nc.f32 %0, [%1];\n\t}"
      : "=f"(v)
      : "l"(p), "r"(a), "r"(b));
  return v;
}
// v = flag ? *p : 0, same form.
__device__ __forceinline__ float ldg_if(const float* p, uint32_t flag) {
  float v;
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.u32 q, %2, 0;\n\t"
      "mov.f32 %0, 0f00000000;\n\t"
      "@q ld.global.nc.f32 %0, [%1];\n\t}"
      : "=f"(v)
      : "l"(p), "r"(flag));
  return v;
}

// if (flag) *p = v, as one predicated st.global.
__device__ __forceinline__ void stg_if(float* p, float v, uint32_t flag) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.u32 q, %2, 0;\n\t"
      "@q st.global.f32 [%0], %1;\n\t}" ::"l"(p), "f"(v), "r"(flag)
      : "memory");
}

// ------------------------------------------------------------------------------ gather kernel (forward, dgrad)
//
// Persistent, warp-specialised: one CTA per SM walks over (channel tile, 128-pixel tile) pairs.
//   producers   (4 * SETS warps) thread = one pixel of the tile = one TMEM lane.  Per k-block a thread gathers its
//               32 lowered values, splits them hi/lo and writes them with tcgen05.st into an A slot in tensor memory
//               (sets of four warps; set g takes the k-blocks with running index == g mod SETS, each set covers
//               all 128 lanes).
//   MMA warp    one thread issues the MMAs: A from tensor memory, B from shared memory.
//   TMA warp    one thread streams the pre-split weight tiles (B) into shared memory with TMA (128-byte swizzle).
//   epilogue    (4 warps) tcgen05.ld the finished accumulator, add bias / clamp, store NCHW (or depth-to-space for
//               the strided data gradient); overlaps the next tile's MMAs when two accumulators fit.
// Tensor memory: [accumulator(s) | A slots of 64 columns: 32 hi + 32 lo].
// The kernel comes in two shapes.  SETS = 4: sixteen producer warps (four sets of four; set g fills the k-blocks with
// running index == g mod 4), 704 threads, one CTA per SM with all 512 tensor-memory columns.  SETS = 2: eight producer
// warps, 448 threads, 256 columns, two stages, one accumulator - two such CTAs share an SM, so two threads issue MMAs
// into the SM's tensor pipe (one thread cannot issue them faster than one per ~75 cycles, however narrow they are)
// and one CTA's epilogue overlaps the other's main loop.
constexpr int kEpiWarps = 4;
__host__ __device__ constexpr int gather_threads(int sets) { return (4 * sets + 2 + kEpiWarps) * 32; }  // 704 or 448
constexpr int kMaxAStages = 4, kMaxAccBufs = 2;

struct alignas(8) ColEnt {  // one accumulator column -> where it lands in the output
  int off;       // element offset from the pixel's output origin
  short cy, cx;  // displacement of the output pixel (depth-to-space), for the bounds test
};

struct GatherParams {
  const float* in;    // gathered tensor: X (forward) or dY (data gradient)
  float* out;         // Y or dX
  const MaskTap* taps; // [k_pad]
  const ColEnt* cols;  // [n_pad]
  const float* bias;  // indexed by output channel, or null
  int n_pix, q_h, q_w;                 // pixels = batch * q_h * q_w
  int iy_mul, iy_add, ix_mul, ix_add;  // tap origin in the gathered tensor: iy0 = qy*iy_mul + iy_add
  int in_lim;                          // gathered tensor is in_lim x in_lim per channel
  int tap_sign, taps_per_axis;         // tap i of an axis sits at coordinate origin + tap_sign * i
  long long in_batch_stride;
  int in_group_stride;   // elements between the channel blocks of consecutive groups
  int tiles_per_group;   // virtual groups per real group (channel tiles)
  int oy_mul, oy_add, ox_mul, ox_add;  // output origin of a pixel: oy0 = qy*oy_mul + oy_add
  int out_lim, check_out;              // output plane is out_lim x out_lim; check_out: columns may fall outside
  int out_pitch, out_plane;
  long long out_batch_stride;
  int out_group_channels, out_tile_channels;  // output channels per real group / per channel tile
  int n, n_pad, k_pad;     // real / padded accumulator columns per virtual group, padded reduction length
  int n_pix_tiles, total_tiles;
  int a_stages, b_stages, acc_bufs;
  int tmem_cols;           // tensor-memory columns this CTA allocates: 512, or 256 when two CTAs share an SM
  int dual;                // 1: one MMA covers [B_hi; B_lo] (N = 2*n_pad) and the epilogue adds the two halves
  int acc_cols;            // accumulator width in tensor-memory columns: n_pad, or 2*n_pad when dual
  int n_bias;              // entries of `bias` (all output channels), staged in shared memory
  int lo_row_offset;       // first row of the "lo" half inside the packed-weight tensor map
  int relu;
  // Weight-gradient mode: the TMEM lanes are rows of the lowered matrix (taps), the reduction runs over pixels.
  // `taps` then points to a table in global memory with one entry per pixel (offset of the pixel's tap origin and
  // the set of tap rows / columns that fall outside the plane there), `out` to the split partial sums.
  int wg;
  int wg_mtiles, wg_vgroups;  // tiles = splits x channel tiles x M-tiles (M-tile fastest)
  int wg_rows_pad;            // rows of one split's partial-sum slice (M-tiles * 128)
  int wg_k, wg_kreal;         // kernel size, real rows of the lowered matrix
  int taps_smem;              // entries of `taps` staged in shared memory (0 in weight-gradient mode)
  int* status;
};

// Which tile a persistent CTA works on: channel tile, pixel tile (or M-tile), first k-block, split.
struct TileId {
  int vg, ptile, kb0, split;
};
__device__ __forceinline__ TileId decode_tile(const GatherParams& P, int t, int kblocks) {
  TileId id;
  if (!P.wg) {
    id.vg = t / P.n_pix_tiles;
    id.ptile = t - id.vg * P.n_pix_tiles;
    id.kb0 = 0;
    id.split = 0;
  } else {
    const int r = t / P.wg_mtiles;
    id.ptile = t - r * P.wg_mtiles;
    id.split = r / P.wg_vgroups;
    id.vg = r - id.split * P.wg_vgroups;
    id.kb0 = id.split * kblocks;
  }
  return id;
}

constexpr int kBiasPad = 256;  // zeros behind the staged bias: every accumulator column of a tile reads an entry
struct GatherSmem {
  uint32_t b_stage_bytes, taps_off, cols_off, bias_off, ptab_off, bars_off, total;
};
// ptab_warps: producer warps that keep a double-buffered 32-entry slice of the per-pixel table (weight-gradient mode).
__host__ __device__ inline GatherSmem gather_smem(int n_pad, int k_pad, int b_stages, int n_bias, int ptab_warps = 0) {
  GatherSmem L;
  L.b_stage_bytes = 2u * (uint32_t)n_pad * 128u;
  L.taps_off = (uint32_t)b_stages * L.b_stage_bytes;
  L.cols_off = L.taps_off + (uint32_t)k_pad * 8u;
  L.bias_off = L.cols_off + (uint32_t)n_pad * 8u;
  L.ptab_off = (L.bias_off + (uint32_t)(n_bias + kBiasPad) * 4u + 15u) & ~15u;
  L.bars_off = L.ptab_off + (uint32_t)ptab_warps * 512u;
  L.total = L.bars_off + 8u * (2 * kMaxAStages + 2 * kMaxAccBufs) + 16u;
  return L;
}

template <int SETS>
__global__ void __launch_bounds__(gather_threads(SETS), SETS == 2 ? 2 : 1)
    gather_conv_kernel(const __grid_constant__ GatherParams P, const __grid_constant__ CUtensorMap w_map) {
  pdl_wait();
  constexpr int kProducerWarps = 4 * SETS, kMmaWarp = kProducerWarps, kTmaWarp = kMmaWarp + 1;
  constexpr int kGatherThreads = gather_threads(SETS);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const GatherSmem L = gather_smem(P.n_pad, P.taps_smem, P.b_stages, P.n_bias, P.wg ? kProducerWarps : 0);
  const uint32_t bars = base + L.bars_off;
  // K-block i (running index over this CTA's tiles) uses A slot i % a_stages, weight slot i % b_stages and the
  // barrier pair i % 4: "ready" completes when the four producer warps of the block's set and the weight tile's TMA
  // bytes have arrived, "done" when the block's MMAs have finished (one tcgen05.commit), which frees both slots.
  // Rings of different depth share the barriers because no waiter can fall a whole barrier phase (4 blocks) behind:
  // block i + 4 cannot finish before the slots of block i + 3 were refilled, which waits for block i.
  const uint32_t ready_bar = bars, done_bar = ready_bar + 8u * kMaxAStages, acc_full = done_bar + 8u * kMaxAStages,
                 acc_empty = acc_full + 8u * kMaxAccBufs, tmem_slot = acc_empty + 8u * kMaxAccBufs;
  MaskTap* s_taps = reinterpret_cast<MaskTap*>(base_ptr + L.taps_off);
  ColEnt* s_cols = reinterpret_cast<ColEnt*>(base_ptr + L.cols_off);
  float* s_bias = reinterpret_cast<float*>(base_ptr + L.bias_off);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int i = tid; i < P.taps_smem; i += kGatherThreads) s_taps[i] = P.taps[i];
  if (P.cols)
    for (int i = tid; i < P.n_pad; i += kGatherThreads) s_cols[i] = P.cols[i];
  for (int i = tid; i < P.n_bias + kBiasPad; i += kGatherThreads) s_bias[i] = i < P.n_bias ? P.bias[i] : 0.f;
  if (tid == 0) {
    for (int s = 0; s < kMaxAStages; ++s) { mbar_init(ready_bar + 8u * s, 5); mbar_init(done_bar + 8u * s, 1); }  // 4 producer warps + the TMA thread
    for (int s = 0; s < kMaxAccBufs; ++s) { mbar_init(acc_full + 8u * s, 1); mbar_init(acc_empty + 8u * s, kEpiWarps); }
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, (uint32_t)P.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  const uint32_t a_col0 = (uint32_t)(P.acc_bufs * P.acc_cols);
  const int kblocks = P.k_pad / kBlockK;
  bool failed = false;

  if (warp < kProducerWarps) {
    // ------------------------------------------------------------------ producers
    // Set `group` fills the A stages of the k-blocks with running index == group (mod SETS).  The raw
    // values of the set's next k-block are already in flight (in registers) while the current one is split and
    // stored, so the global-load latency is paid once per k-block per set, off the critical path.
    const int group = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + a_col0;
    const int my_tiles = (P.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int my_stages = my_tiles * kblocks;
    const float* in_px = P.in;
    uint32_t mask = 0;                   // forward / data gradient: which taps are in bounds for this lane's pixel
    const MaskTap* pix_tab = P.taps;     // weight gradient: this tile's slice of the per-pixel table
    auto setup_tile = [&](int tile_local) {
      const int t = blockIdx.x + tile_local * gridDim.x;
      const TileId id = decode_tile(P, t, kblocks);
      const int grp = id.vg / P.tiles_per_group;
      in_px = P.in;
      if (P.wg) {
        // lane = row of the lowered matrix: (d, kr, kc); `mask` holds the tap's row and column bit
        const int r = id.ptile * kTileM + row;
        mask = kPadBit;
        if (r < P.wg_kreal) {
          const int kk = P.wg_k * P.wg_k;
          const int d = r / kk, rem = r - d * kk;
          const int kr = rem / P.wg_k, kc = rem - kr * P.wg_k;
          in_px = P.in + (long long)grp * P.in_group_stride + (long long)d * P.in_lim * P.in_lim + kr * P.in_lim + kc;
          mask = (1u << kr) | (1u << (16 + kc));
        }
        pix_tab = P.taps + (size_t)id.kb0 * kBlockK;
        return;
      }
      const int pix = id.ptile * kTileM + row;
      mask = 0;  // which tap rows (bits 0-14) and tap columns (bits 16-30) fall inside the plane
      if (pix < P.n_pix) {
        const int per_img = P.q_h * P.q_w;
        const int b = pix / per_img;
        const int r = pix - b * per_img;
        const int qy = r / P.q_w;
        const int qx = r - qy * P.q_w;
        const int iy0 = qy * P.iy_mul + P.iy_add, ix0 = qx * P.ix_mul + P.ix_add;
        in_px = P.in + (long long)b * P.in_batch_stride + (long long)grp * P.in_group_stride +
                (long long)iy0 * P.in_lim + ix0;
        if (P.tap_sign > 0)  // coordinate origin + i in [0, lim)
          mask = bit_range(-iy0, min(P.taps_per_axis, P.in_lim - iy0)) |
                 (bit_range(-ix0, min(P.taps_per_axis, P.in_lim - ix0)) << 16);
        else  // coordinate origin - i in [0, lim)
          mask = bit_range(iy0 - P.in_lim + 1, min(P.taps_per_axis, iy0 + 1)) |
                 (bit_range(ix0 - P.in_lim + 1, min(P.taps_per_axis, ix0 + 1)) << 16);
      }
    };
    float v[kBlockK];
    // Weight gradient: the 32 table entries of a k-block are the same for every lane.  Lane e fetches entry e one
    // step ahead (`ent_next`, in flight while the current block is split and stored), the warp passes them round
    // through its own slice of shared memory.
    uint2 ent_next = make_uint2(0u, 0xffffffffu);
    uint2* my_ptab = reinterpret_cast<uint2*>(base_ptr + L.ptab_off) + warp * 64;
    int pbuf = 0;
    auto prefetch_entries = [&](int kb) {
      if (P.wg) ent_next = __ldg(reinterpret_cast<const uint2*>(pix_tab + kb * kBlockK) + lane);
    };
    auto gather = [&](int kb) {
      if (P.wg) {
        // entry = (offset of the pixel's tap origin, tap rows / columns out of bounds there)
        uint2* slot = my_ptab + pbuf * 32;
        pbuf ^= 1;
        slot[lane] = ent_next;
        __syncwarp();
#pragma unroll
        for (int e = 0; e < kBlockK; ++e) {
          const uint2 ent = slot[e];
          v[e] = ldg_if_clear(in_px + (int)ent.x, ent.y, mask);
        }
        return;
      }
      const MaskTap* tp = s_taps + kb * kBlockK;
#pragma unroll
      for (int e = 0; e < kBlockK; ++e) {
        const MaskTap tap = tp[e];
        v[e] = ldg_if_bits(in_px + tap.off, mask, tap.bits);
      }
    };
    int tile_local = 0, kb = group;
    while (kb >= kblocks && tile_local < my_tiles) { kb -= kblocks; ++tile_local; }
    if (group < my_stages) {
      setup_tile(tile_local);
      prefetch_entries(kb);
      gather(kb);
    }
    for (int it = group; it < my_stages; it += SETS) {
      const int sa = it & (P.a_stages - 1);  // a_stages is 2 or 4
      const uint32_t st_addr = lane_addr + (uint32_t)(sa * 64);
      // The set's next k-block: its tile state and (weight gradient) its table entries, requested now so that
      // they have arrived when the gather is issued further down.  v[] still holds the current block.
      const bool has_next = it + SETS < my_stages;
      if (has_next) {
        const int before = tile_local;
        kb += SETS;
        while (kb >= kblocks) { kb -= kblocks; ++tile_local; }
        if (tile_local != before) setup_tile(tile_local);
        prefetch_entries(kb);
      }
      // The A slot was last read by the MMAs of k-block it - a_stages.
      const int prev = it - P.a_stages;
      if (prev >= 0) mbar_wait(done_bar + 8u * (prev & 3), (uint32_t)(prev >> 2) & 1u, failed, P.status, 0x10);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < kBlockK / 8; ++c) {
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) split_tf32_trunc(v[c * 8 + e], hi[e], lo[e]);
        tmem_st8(st_addr + (uint32_t)(c * 8), hi);
        tmem_st8(st_addr + 32u + (uint32_t)(c * 8), lo);
      }
      // With two stages the hand-over of a filled stage is on the critical path: arrive first, then fetch.
      if (P.a_stages == 2) {
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_bar + 8u * (it & 3));
      }
      if (has_next) gather(kb);  // loads in flight across the next wait
      if (P.a_stages != 2) {
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_bar + 8u * (it & 3));  // one arrival per warp: same-address arrivals serialise
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = make_idesc(P.acc_cols);
      int tile_iter = 0;
      Ring ra, rb, rbar;  // A slot, weight slot, barrier pair of the current k-block
      for (int t = blockIdx.x; t < P.total_tiles; t += gridDim.x, ++tile_iter) {
        const int buf = tile_iter & (P.acc_bufs - 1), ause = tile_iter >> (P.acc_bufs - 1);  // acc_bufs is 1 or 2
        if (ause > 0) mbar_wait<false>(acc_empty + 8u * buf, (uint32_t)(ause - 1) & 1u, failed, P.status, 0x20);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * P.acc_cols);
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait<false>(ready_bar + 8u * rbar.idx, (uint32_t)rbar.use & 1u, failed, P.status, 0x40);
          tc_fence_after();
          const uint32_t b_hi = base + (uint32_t)rb.idx * L.b_stage_bytes, b_lo = b_hi + (uint32_t)P.n_pad * 128u;
          const uint64_t dbh = make_desc(b_hi), dbl = make_desc(b_lo);
          const uint32_t a_hi = tmem_base + a_col0 + (uint32_t)(ra.idx * 64), a_lo = a_hi + 32u;
          if (P.dual) {
            // The lo tile sits right behind the hi tile: one descriptor spans both, so a single MMA of width
            // 2*n_pad produces A*B_hi in the first n_pad columns and A*B_lo in the next (issuing an MMA costs
            // this thread ~75 cycles however narrow it is, so two wide ones beat three narrow ones).
#pragma unroll
            for (int j = 0; j < kBlockK / 8; ++j) {
              const uint64_t adv = (uint64_t)(j * 2);
              umma_tf32_ts(d_tmem, a_lo + (uint32_t)(j * 8), dbh + adv, idesc, (kb == 0 && j == 0) ? 0u : 1u);
              umma_tf32_ts(d_tmem, a_hi + (uint32_t)(j * 8), dbh + adv, idesc, 1u);
            }
          } else {
#pragma unroll
            for (int j = 0; j < kBlockK / 8; ++j) {
              const uint64_t adv = (uint64_t)(j * 2);
              umma_tf32_ts(d_tmem, a_lo + (uint32_t)(j * 8), dbh + adv, idesc, (kb == 0 && j == 0) ? 0u : 1u);
              umma_tf32_ts(d_tmem, a_hi + (uint32_t)(j * 8), dbl + adv, idesc, 1u);
              umma_tf32_ts(d_tmem, a_hi + (uint32_t)(j * 8), dbh + adv, idesc, 1u);
            }
          }
          umma_commit(done_bar + 8u * rbar.idx);  // frees the A slot for the producers and the weight slot for the TMA thread
          ra.advance(P.a_stages);
          rb.advance(P.b_stages);
          rbar.advance(4);
        }
        umma_commit(acc_full + 8u * buf);
      }
    }
  } else if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ weight tiles by TMA
    if (lane == 0) {
      Ring rb;
      int i = 0;  // running k-block index
      for (int t = blockIdx.x; t < P.total_tiles; t += gridDim.x) {
        const TileId id = decode_tile(P, t, kblocks);
        const int vg = id.vg;
        for (int kb = 0; kb < kblocks; ++kb, ++i) {
          const int sb = rb.idx;
          const int prev = i - P.b_stages;  // the k-block whose MMAs read this weight slot last
          if (prev >= 0) mbar_wait<false>(done_bar + 8u * (prev & 3), (uint32_t)(prev >> 2) & 1u, failed, P.status, 0x100);
          const uint32_t b_hi = base + (uint32_t)sb * L.b_stage_bytes, b_lo = b_hi + (uint32_t)P.n_pad * 128u;
          const uint32_t bar = ready_bar + 8u * (i & 3);
          mbar_expect_tx(bar, L.b_stage_bytes);
          tma_load_2d(b_hi, &w_map, (id.kb0 + kb) * kBlockK, vg * P.n_pad, bar);
          tma_load_2d(b_lo, &w_map, (id.kb0 + kb) * kBlockK, P.lo_row_offset + vg * P.n_pad, bar);
          rb.advance(P.b_stages);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int tile_iter = 0;
    for (int t = blockIdx.x; t < P.total_tiles; t += gridDim.x, ++tile_iter) {
      const TileId id = decode_tile(P, t, kblocks);
      const int vg = id.vg, ptile = id.ptile;
      const int grp = vg / P.tiles_per_group, ntile = vg % P.tiles_per_group;
      const int buf = tile_iter & (P.acc_bufs - 1), ause = tile_iter >> (P.acc_bufs - 1);
      if (P.wg) {
        // The accumulator is a 128-row slice of this split's partial sums: row-contiguous stores.
        mbar_wait(acc_full + 8u * buf, (uint32_t)ause & 1u, failed, P.status, 0x200);
        tc_fence_after();
        const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P.acc_cols);
        float* op = P.out + ((size_t)(id.split * P.wg_vgroups + vg) * P.wg_rows_pad + (size_t)ptile * kTileM + row) * P.n_pad;
        for (int c = 0; c < P.n_pad / 16; ++c) {
          float v[16];
          tmem_ld16(acc + (uint32_t)(c * 16), v);
          if (P.dual) {
            float w[16];
            tmem_ld16(acc + (uint32_t)(P.n_pad + c * 16), w);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += w[j];
          }
          if (!failed) {
            float4* o4 = reinterpret_cast<float4*>(op + c * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) o4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + 8u * buf);
        continue;
      }
      const int pix = ptile * kTileM + row;
      int b = 0, qy = 0, qx = 0;
      if (pix < P.n_pix) {
        const int per_img = P.q_h * P.q_w;
        b = pix / per_img;
        const int r = pix - b * per_img;
        qy = r / P.q_w;
        qx = r - qy * P.q_w;
      }
      const int oy0 = qy * P.oy_mul + P.oy_add, ox0 = qx * P.ox_mul + P.ox_add;
      const int ch0 = grp * P.out_group_channels + ntile * P.out_tile_channels;
      float* op = P.out + (long long)b * P.out_batch_stride + (long long)ch0 * P.out_plane +
                  (long long)oy0 * P.out_pitch + ox0;
      const float* bias = s_bias + (P.n_bias ? ch0 : 0);  // zero padded: readable for every column of the tile
      mbar_wait(acc_full + 8u * buf, (uint32_t)ause & 1u, failed, P.status, 0x200);
      tc_fence_after();
      const uint32_t live = (pix < P.n_pix && !failed) ? 1u : 0u;
      const uint32_t unchecked = P.check_out ? 0u : 1u;
      const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P.acc_cols);
      const int chunks = P.n_pad / 16;
      for (int c = 0; c < chunks; ++c) {
        float v[16];
        tmem_ld16(acc + (uint32_t)(c * 16), v);
        if (P.dual) {
          float w[16];
          tmem_ld16(acc + (uint32_t)(P.n_pad + c * 16), w);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += w[j];
        }
        // Straight-line code: table and bias reads first, then predicated st.global (a generic store could alias
        // shared memory and would pin every following table read behind it; a branch per column costs more than
        // the store it guards).
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          ColEnt ce[8];
          float bv[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = c * 16 + h * 8 + j;
            ce[j] = s_cols[col];
            bv[j] = bias[col];
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = c * 16 + h * 8 + j;
            const uint32_t in_y = (unsigned)(oy0 + ce[j].cy) < (unsigned)P.out_lim ? 1u : 0u;
            const uint32_t in_x = (unsigned)(ox0 + ce[j].cx) < (unsigned)P.out_lim ? 1u : 0u;
            const uint32_t ok = live & (col < P.n ? 1u : 0u) & (unchecked | (in_y & in_x));
            float y = v[h * 8 + j] + bv[j];
            y = P.relu ? fmaxf(y, 0.f) : y;
            stg_if(op + ce[j].off, y, ok);
          }
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

// ---------------------------------------------------------------------------------- weight-gradient kernel
//
// dW[kk][o] (+ the bias row) = sum over pixels of Lowered(X)[pix][kk] * dY[pix][o], split over pixel ranges.
// Both operands are K-major shared-memory tiles whose rows are 32 consecutive pixels (one 128-byte swizzled row):
// a row of the lowered operand is one tap (d, kr, kc) seen by 32 consecutive output pixels, a row of the other
// operand is one output channel of dY for the same pixels.  With lane = pixel every global load is a coalesced run
// and every shared-memory store fills one row, conflict free.
// One CTA owns up to `subs` M-tiles of 128 taps (accumulators side by side in tensor memory), one channel tile of dY
// and a range of 32-pixel k-blocks; the dY tile of a k-block is staged once for all its M-tiles.
//   warps 0-15  tap producers: warp w stages rows w, w+16, ... of every M-tile of the stage: load, split hi/lo, two
//               st.shared per row; the loads of the next k-block are issued before the warp waits for the stage
//               buffer to drain.
//   warps 16-23 dY producers: warp 16+w stages channel rows w, w+8, ... of the dY tile the same way.
//   warp 24     one thread issues the MMAs (both operands from shared memory).
// The producers run at about one instruction per eight cycles each (latency bound), so their number, not their
// instruction count alone, sets the staging rate.  The finished accumulators are written to the split's slice of the
// scratch buffer by warps 0-15.
constexpr int kWgTapWarps = 16, kWgDyWarps = 8, kWgProdWarps = kWgTapWarps + kWgDyWarps, kWgMmaWarp = kWgProdWarps;
constexpr int kWgThreads = (kWgMmaWarp + 1) * 32;  // 800
constexpr int kWgMaxStages = 4, kWgMaxSubs = 2;
constexpr uint32_t kWgValidBit = 0x80000000u;      // set in a pixel's mask when the pixel exists
constexpr uint32_t kWgPadBit = 0x00008000u;        // never set in a pixel's mask: rows beyond the lowered matrix
constexpr uint32_t kWgOnesBits = kWgValidBit | kWgPadBit;  // the all-ones row: never loaded, patched in by its warp

struct WgradParams {
  const float* x;
  const float* dy;
  float* partial;       // [splits][vgroups][m_tiles*128][n_pad]
  const MaskTap* taps;  // [m_tiles*128]; row k_real is the all-ones row, rows beyond it are padding
  int n_pix, m, mm, n, s, p, k;
  long long x_batch_stride;
  int x_group_stride;
  long long dy_batch_stride;
  int dy_group_channels;  // output channels per real group
  int tiles_per_group;
  int n_real, n_pad;
  int m_tiles, subs, stages;
  int ones_row;           // index of the all-ones row among the lowered-matrix rows
  int kblocks_total, kblocks_per_split;  // end of this launch's k-block range, k-blocks per split
  int kb_first;                          // first k-block of this launch (a later round of a launch sequence starts further in)
  int* status;
};

struct WgSmem {
  uint32_t a_tile_bytes, b_tile_bytes, stage_bytes, taps_off, bars_off, total;
};
__host__ __device__ inline WgSmem wg_smem(int n_pad, int subs, int stages) {
  WgSmem L;
  L.a_tile_bytes = kTileM * 128u;           // one of hi / lo of one M-tile
  L.b_tile_bytes = (uint32_t)n_pad * 128u;  // one of hi / lo of the dY tile
  L.stage_bytes = 2u * (uint32_t)subs * L.a_tile_bytes + 2u * L.b_tile_bytes;
  L.taps_off = (uint32_t)stages * L.stage_bytes;
  L.bars_off = L.taps_off + (uint32_t)subs * kTileM * 8u;
  L.total = L.bars_off + 8u * (2 * kWgMaxStages + 1) + 16u;
  return L;
}


// SUBS: M-tiles per CTA (accumulators), NB: dY-tile rows per producer warp (= n_pad / 16).  With both fixed at
// compile time every warp stages exactly 8*SUBS tap rows and NB channel rows per k-block, all loads of a k-block are
// in flight together, and the shared-memory addresses are one per-warp base plus immediates: row warp+16*i of a
// 128-byte-swizzled tile has the same swizzle phase ((warp+16*i) & 7 == warp & 7) for every i.
template <int SUBS, int NB>
__global__ void __launch_bounds__(kWgThreads, 1) wgrad_kernel(const __grid_constant__ WgradParams P) {
  pdl_wait();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const WgSmem L = wg_smem(NB * 16, SUBS, P.stages);
  const uint32_t bars = base + L.bars_off;
  const uint32_t full = bars, empty = full + 8u * kWgMaxStages, acc_full = empty + 8u * kWgMaxStages,
                 tmem_slot = acc_full + 8u;
  MaskTap* s_taps = reinterpret_cast<MaskTap*>(base_ptr + L.taps_off);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mgroup = blockIdx.x, split = blockIdx.y, vg = blockIdx.z;
  const int grp = vg / P.tiles_per_group, ntile = vg % P.tiles_per_group;
  const int subs = min(SUBS, P.m_tiles - mgroup * SUBS);  // M-tiles this CTA really has
  constexpr int kARows = 8 * SUBS;                        // tap rows per producer warp and k-block
  constexpr uint32_t kATile = kTileM * 128u, kBTile = NB * 16u * 128u;
  constexpr int kNPad = NB * 16;
  // Narrow dY tiles run "dual": the lo tile sits right behind the hi tile, one MMA of width 2*kNPad covers both (an
  // MMA costs the issuing thread about 75 cycles however narrow it is), and the epilogue adds the two halves of the
  // accumulator.
  constexpr bool kDual = kNPad <= 64;  // operands from shared memory: an MMA wider than 128 is slower than two narrow ones
  constexpr int kAccCols = kDual ? 2 * kNPad : kNPad;

  for (int i = tid; i < SUBS * kTileM; i += kWgThreads)
    s_taps[i] = i < subs * kTileM ? P.taps[mgroup * SUBS * kTileM + i] : MaskTap{0, kWgPadBit};
  if (tid == 0) {
    for (int s = 0; s < kWgMaxStages; ++s) { mbar_init(full + 8u * s, kWgProdWarps); mbar_init(empty + 8u * s, 1); }
    mbar_init(acc_full, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  const int kb_begin = P.kb_first + split * P.kblocks_per_split;
  const int kb_end = min(P.kblocks_total, kb_begin + P.kblocks_per_split);
  const int kblocks = kb_end - kb_begin;  // >= 1 by construction of the grid
  bool failed = false;

  if (warp < kWgProdWarps) {
    // ------------------------------------------------------------------ producers (lane = pixel of the k-block)
    // this lane's pixel, advanced by 32 per k-block
    int pix = kb_begin * kBlockK + lane;
    int pb = pix / P.mm, pr, pc;
    {
      const int pin = pix - pb * P.mm;
      pr = pin / P.m;
      pc = pin - pr * P.m;
    }
    auto next_pixel = [&]() {
      pix += kBlockK;
      pc += kBlockK;
      while (pc >= P.m) { pc -= P.m; ++pr; }
      while (pr >= P.m) { pr -= P.m; ++pb; }
    };
    if (warp < kWgTapWarps) {
      // ---- tap rows: row warp + 16*i of every M-tile
      const float* xg = P.x + (long long)grp * P.x_group_stride;
      // The all-ones row (bias gradient) is one fixed row of one CTA column: its table entry never passes the
      // bounds test (so nothing is loaded for it) and the warp that owns it patches the value in.
      const int ones_local = P.ones_row - mgroup * SUBS * kTileM;
      const bool mine = ones_local >= 0 && ones_local < subs * kTileM && ((ones_local & (kTileM - 1)) % kWgTapWarps) == warp;
      const int ones_i = mine ? (ones_local / kTileM) * 8 + (ones_local & (kTileM - 1)) / kWgTapWarps : -1;
      // This lane's word in row `warp` of a tile; the warp's further rows are 2048 bytes apart.
      uint8_t* lane_ptr = base_ptr + warp * 128 + ((((lane >> 2) ^ (warp & 7)) << 4) + (lane & 3) * 4);
      const MaskTap* my_taps = s_taps + warp;
      float va[kARows];
      auto load_rows = [&]() {
        const bool ok = pix < P.n_pix;
        const int iy0 = pr * P.s - P.p, ix0 = pc * P.s - P.p;
        const float* xsrc = xg + (long long)pb * P.x_batch_stride + (long long)iy0 * P.n + ix0;
        const uint32_t mask =
            ok ? (kWgValidBit | bit_range(-iy0, min(P.k, P.n - iy0)) | (bit_range(-ix0, min(P.k, P.n - ix0)) << 16))
               : 0u;
#pragma unroll
        for (int i = 0; i < kARows; ++i) {
          const MaskTap tap = my_taps[kWgTapWarps * i];
          va[i] = ldg_if_bits(xsrc + tap.off, mask, tap.bits);
        }
        if (ones_i >= 0) {
#pragma unroll
          for (int i = 0; i < kARows; ++i) va[i] = i == ones_i ? (ok ? 1.f : 0.f) : va[i];
        }
      };
      load_rows();
      Ring ring;
      for (int kbl = 0; kbl < kblocks; ++kbl, ring.advance(P.stages)) {
        const int s = ring.idx, use = ring.use;
        uint8_t* st = lane_ptr + (size_t)s * L.stage_bytes;
        if (use > 0) mbar_wait(empty + 8u * s, (uint32_t)(use - 1) & 1u, failed, P.status, 0x10);
#pragma unroll
        for (int i = 0; i < kARows; ++i) {  // tile i/8 (hi then lo), row warp + 16*(i%8)
          uint32_t h, l;
          split_tf32_trunc(va[i], h, l);
          uint8_t* dst = st + (i / 8) * 2 * kATile + (i % 8) * 2048;
          *reinterpret_cast<uint32_t*>(dst) = h;
          *reinterpret_cast<uint32_t*>(dst + kATile) = l;
        }
        if (kbl + 1 < kblocks) {  // the next k-block's loads go in flight before the barrier work
          next_pixel();
          load_rows();
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(full + 8u * s);  // one arrival per warp: same-address arrivals serialise
      }
    } else {
      // ---- dY rows: channel w8 + 8*i of the tile (hi then lo), behind the SUBS tap tiles of the stage
      const int w8 = warp - kWgTapWarps;
      constexpr int kDyRows = kNPad / kWgDyWarps;
      const float* dyg = P.dy + (long long)(grp * P.dy_group_channels + ntile * P.n_real + w8) * P.mm;
      const int dy_step = kWgDyWarps * P.mm;  // elements between consecutive channel rows of this warp
      const int b_live = P.n_real > w8 ? (P.n_real - w8 + kWgDyWarps - 1) / kWgDyWarps : 0;  // real rows
      uint8_t* lane_ptr = base_ptr + SUBS * 2 * kATile + w8 * 128 + ((((lane >> 2) ^ (w8 & 7)) << 4) + (lane & 3) * 4);
      float vb[kDyRows];
      auto load_rows = [&]() {
        const bool ok = pix < P.n_pix;
        const float* dsrc = dyg + (long long)pb * P.dy_batch_stride + pr * P.m + pc;
#pragma unroll
        for (int i = 0; i < kDyRows; ++i) vb[i] = ldg_if(dsrc + i * dy_step, (ok && i < b_live) ? 1u : 0u);
      };
      load_rows();
      Ring ring;
      for (int kbl = 0; kbl < kblocks; ++kbl, ring.advance(P.stages)) {
        const int s = ring.idx, use = ring.use;
        uint8_t* st = lane_ptr + (size_t)s * L.stage_bytes;
        if (use > 0) mbar_wait(empty + 8u * s, (uint32_t)(use - 1) & 1u, failed, P.status, 0x11);
#pragma unroll
        for (int i = 0; i < kDyRows; ++i) {
          uint32_t h, l;
          split_tf32_trunc(vb[i], h, l);
          uint8_t* dst = st + i * (kWgDyWarps * 128);
          *reinterpret_cast<uint32_t*>(dst) = h;
          *reinterpret_cast<uint32_t*>(dst + kBTile) = l;
        }
        if (kbl + 1 < kblocks) {
          next_pixel();
          load_rows();
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(full + 8u * s);
      }
    }
    if (warp < kWgTapWarps) {
    // ---- epilogue: accumulator u, columns in chunks of 16; warp w takes lanes 32*(w%4).. and the (u, chunk) pairs
    //      with index == w/4 (mod 4)
    mbar_wait(acc_full, 0u, failed, P.status, 0x2000);
    tc_fence_after();
    const int quarter = warp & 3, row = quarter * 32 + lane;
    for (int w = warp >> 2; w < subs * NB; w += 4) {
      const int u = w / NB, c = w - u * NB;
      float acc[16];
      const uint32_t col = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(u * kAccCols + c * 16);
      tmem_ld16(col, acc);
      if (kDual) {
        float lo_part[16];
        tmem_ld16(col + kNPad, lo_part);
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] += lo_part[j];
      }
      float* op = P.partial + (((size_t)split * gridDim.z + vg) * P.m_tiles * kTileM +
                               (size_t)(mgroup * SUBS + u) * kTileM + row) * kNPad + c * 16;
      if (!failed) {
        float4* o4 = reinterpret_cast<float4*>(op);
#pragma unroll
        for (int j = 0; j < 4; ++j) o4[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
      }
    }
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kAccCols);
      Ring ring;
      for (int kbl = 0; kbl < kblocks; ++kbl, ring.advance(P.stages)) {
        const int s = ring.idx;
        mbar_wait(full + 8u * s, (uint32_t)ring.use & 1u, failed, P.status, 0x40);  // parked: this thread mostly waits for the producers
        tc_fence_after();
        const uint32_t st = base + (uint32_t)s * L.stage_bytes;
        const uint32_t b_hi = st + SUBS * 2u * kATile, b_lo = b_hi + kBTile;
        const uint64_t dbh = make_desc(b_hi), dbl = make_desc(b_lo);
        for (int u = 0; u < subs; ++u) {
          const uint32_t d_tmem = tmem_base + (uint32_t)(u * kAccCols);
          const uint32_t a_hi = st + (uint32_t)u * 2u * kATile;
          const uint64_t dah = make_desc(a_hi), dal = make_desc(a_hi + kATile);
#pragma unroll
          for (int j = 0; j < kBlockK / 8; ++j) {
            const uint64_t adv = (uint64_t)(j * 2);
            if (kDual) {
              umma_tf32_ss(d_tmem, dal + adv, dbh + adv, idesc, (kbl == 0 && j == 0) ? 0u : 1u);
              umma_tf32_ss(d_tmem, dah + adv, dbh + adv, idesc, 1u);
            } else {
              umma_tf32_ss(d_tmem, dal + adv, dbh + adv, idesc, (kbl == 0 && j == 0) ? 0u : 1u);
              umma_tf32_ss(d_tmem, dah + adv, dbl + adv, idesc, 1u);
              umma_tf32_ss(d_tmem, dah + adv, dbh + adv, idesc, 1u);
            }
          }
        }
        umma_commit(empty + 8u * s);
      }
      umma_commit(acc_full);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------------------------
// The same weight gradient with the operands' roles exchanged, for lowered matrices of 257 .. 384 rows (with the
// all-ones row) and at most 128 output channels per tile - AlexNet / CaffeNet conv1:
//     D[channel][row] = sum over pixels of dY[channel][pixel] * lowered[row][pixel].
// The small operand (dY: 128 lanes = channels, 32 pixels per k-block) goes through TENSOR memory, so the MMAs read only
// the lowered rows from shared memory, 192 of them per instruction (two accumulators of 192 columns): per k-block 24
// MMAs of 96 cycles each, none paying the shared-memory-A surcharge, where wgrad_kernel issues 36 of 91, and one CTA
// covers all rows, so dY is staged once per k-block for the whole SM.
//   warps 0-23  tap producers: warp w stages rows w, w+24, ... (16 rows) of the 384-row tile exactly as wgrad_kernel's.
//   warps 24-27 dY: warp 24+q owns channels 32q .. 32q+31 (= its tensor-memory lanes): coalesced loads with lane = pixel,
//               a turn through a private 32 x 33 shared-memory tile, then lane = channel: split and tcgen05.st.
//               After the last k-block the same warps write the accumulators out (lane = channel = fastest index of the
//               partial-sum buffer).
//   warp 28     one thread issues the MMAs.
// The partial sums have wgrad_kernel's layout ([split][tile][row][channel]), so the same reduction kernels follow.
constexpr int kTsTapWarps = 24, kTsDyWarps = 4, kTsMmaWarp = kTsTapWarps + kTsDyWarps;
constexpr int kTsThreads = (kTsMmaWarp + 1) * 32;  // 928
constexpr int kTsRows = 384, kTsNTile = 192, kTsStages = 2, kTsRowsPerWarp = kTsRows / kTsTapWarps;  // 16
constexpr uint32_t kTsTile = kTsRows * 128u;       // one of hi / lo of the lowered rows of a k-block
constexpr uint32_t kTsStage = 2u * kTsTile;
constexpr uint32_t kTsTapsOff = kTsStages * kTsStage, kTsTurnOff = kTsTapsOff + kTsRows * 8u,
                   kTsBarsOff = kTsTurnOff + kTsDyWarps * 32u * 33u * 4u, kTsSmem = kTsBarsOff + 8u * (2 * kTsStages + 1) + 16u;

__global__ void __launch_bounds__(kTsThreads, 1) wgrad_ts_kernel(const __grid_constant__ WgradParams P) {
  pdl_wait();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kTsBarsOff;
  const uint32_t full = bars, empty = full + 8u * kTsStages, acc_full = empty + 8u * kTsStages, tmem_slot = acc_full + 8u;
  MaskTap* s_taps = reinterpret_cast<MaskTap*>(base_ptr + kTsTapsOff);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.y, vg = blockIdx.z;
  const int grp = vg / P.tiles_per_group, ntile = vg % P.tiles_per_group;
  constexpr uint32_t kACol0 = 2 * kTsNTile;  // tensor memory: two accumulators of 192 columns, then 2 x 64 columns of A

  for (int i = tid; i < kTsRows; i += kTsThreads) s_taps[i] = P.taps[i];
  if (tid == 0) {
    for (int s = 0; s < kTsStages; ++s) { mbar_init(full + 8u * s, kTsTapWarps + kTsDyWarps); mbar_init(empty + 8u * s, 1); }
    mbar_init(acc_full, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  const int kb_begin = P.kb_first + split * P.kblocks_per_split;
  const int kb_end = min(P.kblocks_total, kb_begin + P.kblocks_per_split);
  const int kblocks = kb_end - kb_begin;
  bool failed = false;

  if (warp < kTsMmaWarp) {
    // this lane's pixel, advanced by 32 per k-block
    int pix = kb_begin * kBlockK + lane;
    int pb = pix / P.mm, pr, pc;
    {
      const int pin = pix - pb * P.mm;
      pr = pin / P.m;
      pc = pin - pr * P.m;
    }
    auto next_pixel = [&]() {
      pix += kBlockK;
      pc += kBlockK;
      while (pc >= P.m) { pc -= P.m; ++pr; }
      while (pr >= P.m) { pr -= P.m; ++pb; }
    };
    if (warp < kTsTapWarps) {
      // ---- lowered rows warp + 24*i: row offsets 3072 bytes apart, all with the swizzle phase of row `warp`
      const float* xg = P.x + (long long)grp * P.x_group_stride;
      const bool mine = P.ones_row % kTsTapWarps == warp;
      const int ones_i = mine ? P.ones_row / kTsTapWarps : -1;
      uint8_t* lane_ptr = base_ptr + warp * 128 + ((((lane >> 2) ^ (warp & 7)) << 4) + (lane & 3) * 4);
      const MaskTap* my_taps = s_taps + warp;
      float va[kTsRowsPerWarp];
      auto load_rows = [&]() {
        const bool ok = pix < P.n_pix;
        const int iy0 = pr * P.s - P.p, ix0 = pc * P.s - P.p;
        const float* xsrc = xg + (long long)pb * P.x_batch_stride + (long long)iy0 * P.n + ix0;
        const uint32_t mask =
            ok ? (kWgValidBit | bit_range(-iy0, min(P.k, P.n - iy0)) | (bit_range(-ix0, min(P.k, P.n - ix0)) << 16))
               : 0u;
#pragma unroll
        for (int i = 0; i < kTsRowsPerWarp; ++i) {
          const MaskTap tap = my_taps[kTsTapWarps * i];
          va[i] = ldg_if_bits(xsrc + tap.off, mask, tap.bits);
        }
        if (ones_i >= 0) {
#pragma unroll
          for (int i = 0; i < kTsRowsPerWarp; ++i) va[i] = i == ones_i ? (ok ? 1.f : 0.f) : va[i];
        }
      };
      load_rows();
      Ring ring;
      for (int kbl = 0; kbl < kblocks; ++kbl, ring.advance(kTsStages)) {
        const int s = ring.idx, use = ring.use;
        uint8_t* st = lane_ptr + (size_t)s * kTsStage;
        if (use > 0) mbar_wait(empty + 8u * s, (uint32_t)(use - 1) & 1u, failed, P.status, 0x3010);
#pragma unroll
        for (int i = 0; i < kTsRowsPerWarp; ++i) {
          uint32_t h, l;
          split_tf32_trunc(va[i], h, l);
          uint8_t* dst = st + i * (kTsTapWarps * 128);
          *reinterpret_cast<uint32_t*>(dst) = h;
          *reinterpret_cast<uint32_t*>(dst + kTsTile) = l;
        }
        if (kbl + 1 < kblocks) {  // the next k-block's loads go in flight before the barrier work
          next_pixel();
          load_rows();
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(full + 8u * s);
      }
    } else {
      // ---- dY: channels 32q .. 32q+31 of the tile; tensor-memory lanes of the same numbers
      const int q = warp - kTsTapWarps;
      const float* dyg = P.dy + (long long)(grp * P.dy_group_channels + ntile * P.n_real + q * 32) * P.mm;
      const int live = min(32, max(0, P.n_real - q * 32));  // real channels of this quadrant
      float* turn = reinterpret_cast<float*>(base_ptr + kTsTurnOff) + q * (32 * 33);
      const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + kACol0;
      float vb[32];
      auto load_rows = [&]() {
        const bool ok = pix < P.n_pix;
        const float* dsrc = dyg + (long long)pb * P.dy_batch_stride + pr * P.m + pc;
#pragma unroll
        for (int i = 0; i < 32; ++i) vb[i] = ldg_if(dsrc + (long long)i * P.mm, (ok && i < live) ? 1u : 0u);
      };
      load_rows();
      Ring ring;
      for (int kbl = 0; kbl < kblocks; ++kbl, ring.advance(kTsStages)) {
        const int s = ring.idx, use = ring.use;
#pragma unroll
        for (int i = 0; i < 32; ++i) turn[i * 33 + lane] = vb[i];  // row = channel, column = pixel
        __syncwarp();
        if (kbl + 1 < kblocks) {
          next_pixel();
          load_rows();
        }
        // The stage's 64 tensor-memory columns were last read by the MMAs of k-block kbl - 2.
        if (use > 0) mbar_wait(empty + 8u * s, (uint32_t)(use - 1) & 1u, failed, P.status, 0x3011);
        tc_fence_after();
        const uint32_t st_addr = lane_addr + (uint32_t)(s * 64);
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // lane = channel now: its 32 pixels, eight at a time
          uint32_t hi[8], lo[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) split_tf32_trunc(turn[lane * 33 + c * 8 + e], hi[e], lo[e]);
          tmem_st8(st_addr + (uint32_t)(c * 8), hi);
          tmem_st8(st_addr + 32u + (uint32_t)(c * 8), lo);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();  // also: every lane has read the tile before the next k-block overwrites it
        if (lane == 0) mbar_arrive(full + 8u * s);
      }
      // ---- epilogue: lane = channel, one accumulator column = one lowered row
      mbar_wait(acc_full, 0u, failed, P.status, 0x3020);
      tc_fence_after();
      const int ch = q * 32 + lane;
      float* op = P.partial + ((size_t)split * gridDim.z + vg) * kTsRows * P.n_pad + ch;
      for (int c = 0; c < kTsRows / 16; ++c) {
        float acc[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 16), acc);
        if (!failed && ch < P.n_pad) {
#pragma unroll
          for (int j = 0; j < 16; ++j) op[(size_t)(c * 16 + j) * P.n_pad] = acc[j];
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kTsNTile);
      Ring ring;
      for (int kbl = 0; kbl < kblocks; ++kbl, ring.advance(kTsStages)) {
        const int s = ring.idx;
        mbar_wait(full + 8u * s, (uint32_t)ring.use & 1u, failed, P.status, 0x3040);
        tc_fence_after();
        const uint32_t st = base + (uint32_t)s * kTsStage;
        const uint32_t a_hi = tmem_base + kACol0 + (uint32_t)(s * 64), a_lo = a_hi + 32u;
#pragma unroll
        for (int u = 0; u < kTsRows / kTsNTile; ++u) {
          const uint32_t d_tmem = tmem_base + (uint32_t)(u * kTsNTile);
          const uint64_t dbh = make_desc(st + (uint32_t)u * kTsNTile * 128u), dbl = make_desc(st + kTsTile + (uint32_t)u * kTsNTile * 128u);
#pragma unroll
          for (int j = 0; j < kBlockK / 8; ++j) {
            const uint64_t adv = (uint64_t)(j * 2);
            umma_tf32_ts(d_tmem, a_lo + (uint32_t)(j * 8), dbh + adv, idesc, (kbl == 0 && j == 0) ? 0u : 1u);
            umma_tf32_ts(d_tmem, a_hi + (uint32_t)(j * 8), dbl + adv, idesc, 1u);
            umma_tf32_ts(d_tmem, a_hi + (uint32_t)(j * 8), dbh + adv, idesc, 1u);
          }
        }
        umma_commit(empty + 8u * s);
      }
      umma_commit(acc_full);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

typedef void (*WgradKernel)(const WgradParams);
template <int SUBS>
WgradKernel wgrad_pick_nb(int nb) {
  switch (nb) {
    case 1: return wgrad_kernel<SUBS, 1>;   case 2: return wgrad_kernel<SUBS, 2>;
    case 3: return wgrad_kernel<SUBS, 3>;   case 4: return wgrad_kernel<SUBS, 4>;
    case 5: return wgrad_kernel<SUBS, 5>;   case 6: return wgrad_kernel<SUBS, 6>;
    case 7: return wgrad_kernel<SUBS, 7>;   case 8: return wgrad_kernel<SUBS, 8>;
    case 9: return wgrad_kernel<SUBS, 9>;   case 10: return wgrad_kernel<SUBS, 10>;
    case 11: return wgrad_kernel<SUBS, 11>; case 12: return wgrad_kernel<SUBS, 12>;
    case 13: return wgrad_kernel<SUBS, 13>; case 14: return wgrad_kernel<SUBS, 14>;
    case 15: return wgrad_kernel<SUBS, 15>; case 16: return wgrad_kernel<SUBS, 16>;
  }
  return nullptr;
}
WgradKernel wgrad_pick(int subs, int n_pad) {
  return subs == 2 ? wgrad_pick_nb<2>(n_pad / 16) : wgrad_pick_nb<1>(n_pad / 16);
}

// dW[o][kk] and db[o] from the split partial sums, added in split order (deterministic).  One block per 32 x 32
// tile of (kk, channel): the partial sums are read along the channels (their fastest index), the tile is turned in
// shared memory, and dW is written along kk (its fastest index) - both sides coalesced, no division per element.
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dW,
                                                           float* __restrict__ db, int splits, int vgroups,
                                                           int tiles_per_group, int rows_pad, int n_real, int n_pad,
                                                           int k_real, int og, int accumulate) {
  pdl_wait();
  __shared__ float tile[32][33];
  const int vg = blockIdx.z;
  const int kk0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int ch0 = (vg / tiles_per_group) * og + (vg % tiles_per_group) * n_real;
  const size_t split_stride = (size_t)vgroups * rows_pad * n_pad;
  const int last = db ? k_real : k_real - 1;  // the bias row exists only where the kernel produced it
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int kk = kk0 + ty + 8 * r, j = j0 + tx;
    float acc = 0.f;
    if (kk <= last && j < n_real) {
      const float* src = partial + ((size_t)vg * rows_pad + kk) * n_pad + j;
#pragma unroll 8
      for (int s = 0; s < splits; ++s) acc += src[(size_t)s * split_stride];
    }
    tile[ty + 8 * r][tx] = acc;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int j = j0 + ty + 8 * r, kk = kk0 + tx;
    if (j < n_real && kk <= last) {
      const float v = tile[tx][ty + 8 * r];
      float* dst = kk < k_real ? dW + (size_t)(ch0 + j) * k_real + kk : db + ch0 + j;
      *dst = accumulate ? *dst + v : v;  // accumulate: a later round of splits adds to what the earlier rounds left
    }
  }
}

// The same reduction for small outputs, where 32 x 32 tiles would leave most SMs idle: one block per row (channel
// tile, kk) of the partial sums; 32 channels x 8 interleaved slices of the splits per pass, the eight slice sums
// added in a fixed order - the result does not depend on the grid, and a thread's chain is splits / 8 long.
__global__ void __launch_bounds__(256) wgrad_reduce_rows_kernel(const float* __restrict__ partial, float* __restrict__ dW,
                                                                float* __restrict__ db, int splits, int vgroups,
                                                                int tiles_per_group, int rows_pad, int n_real,
                                                                int n_pad, int k_real, int og, int accumulate) {
  pdl_wait();
  __shared__ float part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int rows = vgroups * (k_real + 1);
  const size_t split_stride = (size_t)vgroups * rows_pad * n_pad;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const int vg = r / (k_real + 1), kk = r - vg * (k_real + 1);
    if (kk == k_real && !db) continue;  // no bias row in the partial sums (uniform over the block)
    const int ch0 = (vg / tiles_per_group) * og + (vg % tiles_per_group) * n_real;
    for (int j0 = 0; j0 < n_real; j0 += 32) {
      const int j = j0 + tx;
      float acc = 0.f;
      if (j < n_real) {
        const float* src = partial + ((size_t)vg * rows_pad + kk) * n_pad + j;
#pragma unroll 4
        for (int s = ty; s < splits; s += 8) acc += src[(size_t)s * split_stride];
      }
      __syncthreads();  // the previous pass has been read
      part[ty][tx] = acc;
      __syncthreads();
      if (ty == 0 && j < n_real) {
        float t = part[0][tx];
#pragma unroll
        for (int y = 1; y < 8; ++y) t += part[y][tx];
        float* dst = kk < k_real ? dW + (size_t)(ch0 + j) * k_real + kk : db + ch0 + j;
        *dst = accumulate ? *dst + t : t;
      }
    }
  }
}

// ------------------------------------------------------------------- dY as a pre-split TMA operand, bias sums
// dY[b][c][pix] -> hi / lo [row of channel c][b * mm + pix] with row = channel tile * n_pad + channel inside the
// tile (K-major rows of `row_len` floats, so a TMA box is 32 consecutive pixels x one channel tile), and the plane
// sum of dY[b][c] for the bias gradient.  One block per plane at a time; every access is a coalesced run.
__global__ void __launch_bounds__(256) split_dy_kernel(const float* __restrict__ dY, float* __restrict__ hi,
                                                       float* __restrict__ lo, float* __restrict__ plane_sums,
                                                       int planes, int channels, int mm, int og, int ch_tile,
                                                       int tiles_per_group, int n_pad, size_t row_len) {
  pdl_wait();
  // One warp per plane at a time, eight loads in flight per lane; no block-wide synchronisation.
  const int lane = threadIdx.x & 31;
  const int warp0 = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5), nwarps = (int)((gridDim.x * blockDim.x) >> 5);
  for (int plane = warp0; plane < planes; plane += nwarps) {
    const int b = plane / channels, c = plane - b * channels;
    const int grp = c / og, j = c - grp * og;
    const int tile = j / ch_tile, within = j - tile * ch_tile;
    const size_t row = (size_t)(grp * tiles_per_group + tile) * n_pad + within;
    const float* src = dY + (size_t)plane * mm;
    float* dh = hi + row * row_len + (size_t)b * mm;
    float* dl = lo + row * row_len + (size_t)b * mm;
    float sum = 0.f;
    // Lane l takes the plane's elements whose DESTINATION is l floats into a 128-byte line (rows of the operand are
    // multiples of 32 floats, so only the image's offset b * mm matters): every warp-wide store then fills whole lines.
    // Stores that straddle lines run at about two thirds of the bandwidth on this part; loads do not care.
    const int skew = (int)(((size_t)b * mm) & 31);
    for (int i0 = -skew; i0 < mm; i0 += 256) {
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * 32 + lane;
        x[u] = (i >= 0 && i < mm) ? __ldg(src + i) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * 32 + lane;
        uint32_t h, l;
        split_tf32_trunc(x[u], h, l);
        if (i >= 0 && i < mm) {
          dh[i] = __uint_as_float(h);
          dl[i] = __uint_as_float(l);
        }
        sum += x[u];
      }
    }
    if (plane_sums) {  // fixed-shape reduction: the result does not depend on the grid
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) plane_sums[plane] = sum;
    }
  }
}

// db[c] = sum over the batch of the plane sums (ConvolutionBridge_impl.hxx:575-599), in a fixed order.
__global__ void bias_grad_kernel(const float* __restrict__ plane_sums, float* __restrict__ db, int batch, int channels) {
  pdl_wait();
  // one warp per channel: lane l adds images l, l + 32, ... in order, then a fixed shuffle tree
  const int c = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (c >= channels) return;
  float t = 0.f;
  for (int b = lane; b < batch; b += 32) t += plane_sums[(size_t)b * channels + c];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  if (lane == 0) db[c] = t;
}

// ------------------------------------------------------------------------------------------ weight packing
// Forward B operand: [2 (hi, lo)][vg][n_pad][k_pad] <- W[o][Dg*k*k], zero padded.
__global__ void pack_fwd_kernel(const float* __restrict__ W, float* __restrict__ hi, float* __restrict__ lo, int vgroups,
                                int tiles_per_group, int og, int n_real, int n_pad, int k_real, int k_pad) {
  pdl_wait();
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

// Data-gradient B operand: [2][vg][n_pad][k_pad]; row j = (d, py, px) of channel tile nt of group g (py, px: position
// inside an s x s block of input pixels), column kk = (oc, jy, jx) <- W[g*og + oc][d][py + jy*s][px + jx*s], zero where
// the tap index exceeds the kernel.
__global__ void pack_dgrad_kernel(const float* __restrict__ W, float* __restrict__ hi, float* __restrict__ lo,
                                  int vgroups, int tiles_per_group, int og, int Dg, int k, int s, int taps, int d_tile,
                                  int n_real, int n_pad, int k_real, int k_pad) {
  pdl_wait();
  const size_t total = (size_t)vgroups * n_pad * k_pad;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int kk = (int)(t % k_pad);
    const int j = (int)((t / k_pad) % n_pad);
    const int vg = (int)(t / ((size_t)k_pad * n_pad));
    float v = 0.f;
    if (j < n_real && kk < k_real) {
      const int grp = vg / tiles_per_group;
      const int d = (vg % tiles_per_group) * d_tile + j / (s * s);
      const int py = (j / s) % s, px = j % s;
      const int jx = kk % taps, jy = (kk / taps) % taps, oc = kk / (taps * taps);
      const int kr = py + jy * s, kc = px + jx * s;
      if (kr < k && kc < k) v = W[(((size_t)(grp * og + oc)) * Dg + d) * k * k + kr * k + kc];
    }
    float h, l;
    split_tf32(v, h, l);
    hi[t] = h;
    lo[t] = l;
  }
}

int round_up(int v, int a) { return (v + a - 1) / a * a; }

// Smallest number of equal channel tiles such that a tile spans at most `limit` accumulator columns.
int channel_tiles(int channels, int cols_per_channel) {
  for (int t = 1; t <= channels; ++t)
    if (channels % t == 0 && (channels / t) * cols_per_channel <= 256) return t;
  return 0;
}

// Channel tiles of the data gradient.  The widest accumulator is not always the fastest: work units (pixel tile x
// channel tile) are spread over the resident CTAs in whole rounds, and accumulators of at most 128 columns run as two
// CTAs per SM, whose last, half-empty round costs about half a round.  Estimated cycles = rounds x k-blocks x cycles per
// k-block (MMA issue: 75 cycles each; MMA execution: half a cycle per column, shared by the SM's CTAs; gather: about
// 2 500 cycles per k-block and producer set), for the widest tiling and for the next narrower ones down to 64 columns.
int dgrad_channel_tiles(int sm_count, int channels, int cols_per_channel, long long pixel_tiles, int groups, int kblocks) {
  const int t0 = channel_tiles(channels, cols_per_channel);
  if (t0 == 0) return 0;
  int best_t = t0;
  double best = 0.0;
  for (int t = t0; t <= channels; ++t) {
    if (channels % t) continue;
    const int n_pad = round_up((channels / t) * cols_per_channel, 16);
    if (t > t0 && n_pad < 64) break;
    const bool dual = n_pad <= 64, two_per_sm = (dual ? 2 * n_pad : n_pad) <= 128;
    const int mmas = dual ? 8 : 12;
    const double exec = mmas * (dual ? n_pad : n_pad / 2.0);
    const double per_kb = two_per_sm ? std::max({mmas * 75.0, 2.0 * exec, 2500.0 / 2}) : std::max({mmas * 75.0, exec, 2500.0 / 4});
    const long long units = pixel_tiles * groups * t, slots = (long long)sm_count * (two_per_sm ? 2 : 1);
    const long long tail = units % slots;
    const double rounds = (double)(units / slots) + (tail == 0 ? 0.0 : (two_per_sm && 2 * tail <= slots) ? 0.55 : 1.0);
    const double cost = rounds * kblocks * per_kb;
    if (t == t0 || cost < 0.97 * best) {  // a narrower tiling gathers every pixel once more: it has to win clearly
      best = cost;
      best_t = t;
    }
  }
  return best_t;
}

}  // namespace

// One gather problem (forward, or the data gradient): tables, packed weights and their tensor map.
struct GatherProblem {
  int tiles = 1, ch_tile = 0;  // channel tiles per group, channels per tile
  int n = 0, n_pad = 0, k_real = 0, k_pad = 0;
  MaskTap* taps = nullptr;
  ColEnt* cols = nullptr;
  float* w = nullptr;  // [2][vgroups][n_pad][k_pad]
  size_t w_half = 0;   // elements in one half
  CUtensorMap map;
  int a_stages = 4, b_stages = 4, acc_bufs = 1, dual = 0, acc_cols = 0;
  int sets = 4, tmem_cols = 512;  // kernel shape: 4 producer sets and one CTA per SM, or 2 sets and two CTAs per SM
  int taps_smem = -1;             // tap-table entries staged in shared memory (-1: k_pad)
  size_t map_k = 0;               // extent of the packed operand along the reduction (0: k_pad)
  size_t smem = 0;
};

struct UmmaPlan {
  ConvGeom G;
  GatherProblem fwd, dgr;
  int dgr_taps = 0, dgr_q = 0, dgr_q0 = 0;  // taps per axis; super-pixels per axis and the first one that holds a pixel
  // weight gradient
  int w_mtiles, w_subs, w_stages, w_mgroups, w_splits, w_kblocks_total, w_kblocks_per_split, w_npad;
  size_t w_smem = 0;
  bool w_ts = false;  // weight gradient by wgrad_ts_kernel (dY through tensor memory) instead of wgrad_kernel
  MaskTap* w_taps = nullptr;
  float* w_partial = nullptr;
  // weight gradient through the gather kernel: lanes = rows of the lowered matrix, reduction over pixels, dY as the
  // pre-split TMA operand [hi|lo][channel tile][channel][pixel]
  bool wg_gather = false;
  GatherProblem wgp;
  MaskTap* wg_pix = nullptr;       // per pixel: offset of the tap origin, taps out of bounds (padded to splits * kps * 32)
  float* wg_plane_sums = nullptr;  // [batch][channel] sums of dY for the bias gradient
  int wg_splits = 1, wg_kps = 1, wg_mtiles = 1;
  size_t bytes = 0;
};

bool umma_supported(const ConvGeom& G) {
  if (channel_tiles(G.og, 1) == 0 || channel_tiles(G.Dg, G.s * G.s) == 0) return false;
  if (G.k > kMaxTapsPerAxis || G.n > 8000) return false;  // tap rows / columns are bits of a 32-bit validity mask
  const int taps = (G.k + G.s - 1) / G.s;
  const long long kf = (long long)G.Dg * G.k * G.k, kd = (long long)G.og * taps * taps;
  if (kf > 16384 || kd > 16384) return false;  // the tap table lives in shared memory next to the weight stages
  return true;
}

namespace {

template <class T>
int dev_alloc(cct_ctx* ctx, UmmaPlan* p, T** ptr, size_t count) {
  CCT_CUDA(ctx, cudaMalloc((void**)ptr, std::max<size_t>(count, 1) * sizeof(T)));
  p->bytes += count * sizeof(T);
  return CCT_OK;
}

template <class T>
int upload(cct_ctx* ctx, UmmaPlan* p, T** dst, const std::vector<T>& host) {
  int rc = dev_alloc(ctx, p, dst, host.size());
  if (rc != CCT_OK) return rc;
  CCT_CUDA(ctx, cudaMemcpy(*dst, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice));
  return CCT_OK;
}

template <class K>
int set_smem(cct_ctx* ctx, K kernel, size_t bytes) {
  CCT_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return CCT_OK;
}

// Split reduction: tiles when they fill the machine, rows otherwise (both add in split order).
void launch_wgrad_reduce(cct_ctx* ctx, const float* partial, float* dW, float* db, int splits, int vgroups,
                         int tiles_per_group, int rows_pad, int n_real, int n_pad, int k_real, int og,
                         int accumulate = 0) {
  const dim3 tiles((k_real + 1 + 31) / 32, (n_real + 31) / 32, vgroups);
  if ((int)(tiles.x * tiles.y * tiles.z) >= ctx->sm_count)
    launch_pdl(wgrad_reduce_kernel, dim3(tiles), dim3(256), 0, ctx->stream, partial, dW, db, splits, vgroups, tiles_per_group, rows_pad,
                                                       n_real, n_pad, k_real, og, accumulate);
  else
    launch_pdl(wgrad_reduce_rows_kernel, dim3(std::max(1, std::min(vgroups * (k_real + 1), ctx->sm_count * 8))), dim3(256), 0, ctx->stream, 
        partial, dW, db, splits, vgroups, tiles_per_group, rows_pad, n_real, n_pad, k_real, og, accumulate);
}

int pack_grid(cct_ctx* ctx, size_t total) {
  size_t b = (total + 255) / 256;
  return (int)std::min<size_t>(std::max<size_t>(b, 1), (size_t)ctx->sm_count * 8);
}

// Tensor-memory and shared-memory budget of a gather problem, packed-weight buffer and its tensor map.
int finish_problem(cct_ctx* ctx, UmmaPlan* p, GatherProblem& gp, int vgroups, int n_bias) {
  // Tensor memory (512 columns) = accumulator buffers + A stages of 64 columns.  Narrow problems run "dual" (see the
  // MMA loop): their accumulator is 2*n_pad wide.  Two accumulator buffers let the epilogue overlap the next tile.
  const int taps_smem = gp.taps_smem < 0 ? gp.k_pad : gp.taps_smem;
  const size_t map_k = gp.map_k ? gp.map_k : (size_t)gp.k_pad;
  gp.dual = gp.n_pad <= 64;  // 2 MMAs of width <= 128 instead of 3 narrow ones; wider ones gain nothing
  gp.acc_cols = gp.dual ? 2 * gp.n_pad : gp.n_pad;
  if (2 * gp.acc_cols + 4 * 64 <= 512) { gp.acc_bufs = 2; gp.a_stages = 4; }
  else if (2 * gp.acc_cols + 2 * 64 <= 512 && gp.k_pad / kBlockK <= 16) { gp.acc_bufs = 2; gp.a_stages = 2; }  // short K: the epilogue matters more
  else { gp.acc_bufs = 1; gp.a_stages = std::min(4, (512 - gp.acc_cols) / 64); }
  // Weight slots (hi and lo tile each) in shared memory: up to four, independent of the number of A slots.
  const int ptab = gp.taps_smem == 0 ? 16 : 0;  // weight-gradient mode: per-warp table slices (sized for 16 warps)
  auto slots_that_fit = [&](size_t limit) {
    int b = 4;
    while (b > 1 && gather_smem(gp.n_pad, taps_smem, b, n_bias, ptab).total + 1024 > limit) --b;
    return b;
  };
  gp.b_stages = slots_that_fit(kSmemLimit);
  // Accumulators of at most 128 columns leave room for two CTAs per SM: 256 columns each (accumulator + two A
  // slots) and half the shared memory (the SM holds 228 KB, 1 KB of it reserved per resident CTA).  Three weight slots
  // per CTA, or two when the accumulator is the full 128 columns (each MMA then lasts long enough to cover the refill:
  // CaffeNet conv5 forward 0.189 -> 0.153 ms).
  const int b_two = slots_that_fit(113 * 1024);
  if (gp.acc_cols <= 128 && (b_two >= 3 || (b_two == 2 && gp.acc_cols == 128))) {
    gp.sets = 2; gp.tmem_cols = 256; gp.acc_bufs = 1; gp.a_stages = 2; gp.b_stages = b_two;
  }
  gp.smem = gather_smem(gp.n_pad, taps_smem, gp.b_stages, n_bias, gp.taps_smem == 0 ? 4 * gp.sets : 0).total + 1024;
  gp.w_half = (size_t)vgroups * gp.n_pad * map_k;
  int rc = dev_alloc(ctx, p, &gp.w, 2 * gp.w_half);
  if (rc != CCT_OK) return rc;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    ctx->last_error = "cuTensorMapEncodeTiled is not available from this driver";
    return CCT_ERR_CUDA;
  }
  const cuuint64_t gdim[2] = {(cuuint64_t)map_k, (cuuint64_t)(2 * vgroups * gp.n_pad)};
  const cuuint64_t gstride[1] = {(cuuint64_t)map_k * sizeof(float)};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)gp.n_pad};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(&gp.map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, gp.w, gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    ctx->last_error = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r);
    return CCT_ERR_CUDA;
  }
  return CCT_OK;
}

}  // namespace

int umma_plan_create(cct_ctx* ctx, const ConvGeom& G, UmmaPlan** out) {
  UmmaPlan* p = new UmmaPlan();
  p->G = G;
  int rc = CCT_OK;
  const int kk = G.k * G.k;
  // ---- forward: accumulator columns = output channels of a tile, reduction = (d, kr, kc)
  {
    GatherProblem& f = p->fwd;
    f.tiles = channel_tiles(G.og, 1);
    f.ch_tile = f.n = G.og / f.tiles;
    f.n_pad = round_up(f.n, 16);
    f.k_real = G.Dg * kk;
    f.k_pad = round_up(f.k_real, kBlockK);
    std::vector<MaskTap> t(f.k_pad);
    for (int i = 0; i < f.k_pad; ++i) {
      if (i < f.k_real) {
        const int d = i / kk, kr = (i / G.k) % G.k, kc = i % G.k;
        t[i] = MaskTap{d * G.n * G.n + kr * G.n + kc, (1u << kr) | (1u << (16 + kc))};
      } else {
        t[i] = MaskTap{0, kPadBit};
      }
    }
    std::vector<ColEnt> c(f.n_pad);
    for (int j = 0; j < f.n_pad; ++j) c[j] = ColEnt{j * G.m * G.m, 0, 0};
    rc = upload(ctx, p, &f.taps, t);
    if (rc == CCT_OK) rc = upload(ctx, p, &f.cols, c);
    if (rc == CCT_OK) rc = finish_problem(ctx, p, f, G.g * f.tiles, G.bias ? G.o : 0);
  }
  // ---- data gradient as a stride-1 gather over dY: one "super pixel" = an s x s block of input pixels; accumulator
  //      columns = (d, py, px), reduction = (oc, jy, jx) with jy, jx < ceil(k/s); depth-to-space in the epilogue.
  if (rc == CCT_OK) {
    GatherProblem& d = p->dgr;
    const int ss = G.s * G.s;
    p->dgr_taps = (G.k + G.s - 1) / G.s;
    p->dgr_q0 = G.p / G.s;
    p->dgr_q = (G.n - 1 + G.p) / G.s + 1 - p->dgr_q0;
    {
      const int J0 = (G.k + G.s - 1) / G.s, q0 = G.p / G.s, q = (G.n - 1 + G.p) / G.s + 1 - q0;
      d.tiles = dgrad_channel_tiles(ctx->planning_sms(), G.Dg, ss, ((long long)G.B * q * q + kTileM - 1) / kTileM, G.g,
                                    (G.og * J0 * J0 + kBlockK - 1) / kBlockK);
    }
    d.ch_tile = G.Dg / d.tiles;
    d.n = d.ch_tile * ss;
    d.n_pad = round_up(d.n, 16);
    const int J = p->dgr_taps;
    d.k_real = G.og * J * J;
    d.k_pad = round_up(d.k_real, kBlockK);
    std::vector<MaskTap> t(d.k_pad);
    for (int i = 0; i < d.k_pad; ++i) {
      if (i < d.k_real) {
        const int jx = i % J, jy = (i / J) % J, oc = i / (J * J);
        t[i] = MaskTap{oc * G.m * G.m - jy * G.m - jx, (1u << jy) | (1u << (16 + jx))};
      } else {
        t[i] = MaskTap{0, kPadBit};
      }
    }
    std::vector<ColEnt> c(d.n_pad);
    for (int j = 0; j < d.n_pad; ++j) {
      const int dl = j / ss, py = (j / G.s) % G.s, px = j % G.s;
      c[j] = ColEnt{dl * G.n * G.n + py * G.n + px, (short)py, (short)px};
    }
    rc = upload(ctx, p, &d.taps, t);
    if (rc == CCT_OK) rc = upload(ctx, p, &d.cols, c);
    if (rc == CCT_OK) rc = finish_problem(ctx, p, d, G.g * d.tiles, 0);
  }
  // ---- weight gradient: rows = (d, kr, kc) plus the all-ones row, columns = output channels of a tile
  if (rc == CCT_OK) {
    const GatherProblem& f = p->fwd;
    p->w_npad = f.n_pad;
    p->w_mtiles = (f.k_real + 1 + kTileM - 1) / kTileM;
    std::vector<MaskTap> t((size_t)p->w_mtiles * kTileM);
    for (size_t i = 0; i < t.size(); ++i) {
      if ((int)i < f.k_real) {
        const int d = (int)i / kk, kr = ((int)i / G.k) % G.k, kc = (int)i % G.k;
        t[i] = MaskTap{d * G.n * G.n + kr * G.n + kc, kWgValidBit | (1u << kr) | (1u << (16 + kc))};
      } else if ((int)i == f.k_real) {
        t[i] = MaskTap{0, kWgOnesBits};
      } else {
        t[i] = MaskTap{0, kWgPadBit};
      }
    }
    rc = upload(ctx, p, &p->w_taps, t);
    // M-tiles per CTA: as many as leave room for two stages in shared memory (and whose accumulators fit in tensor
    // memory); the dY tile of a k-block is staged once for all of them.
    int subs = 1;
    for (int u = 2; u <= kWgMaxSubs; ++u)
      if (u <= p->w_mtiles && u * (f.n_pad <= 64 ? 2 : 1) * f.n_pad <= 512 && 2 * wg_smem(f.n_pad, u, 2).stage_bytes + 8192 <= (uint32_t)kSmemLimit)
        subs = u;
    p->w_subs = subs;
    p->w_mgroups = (p->w_mtiles + subs - 1) / subs;
    // 257 .. 384 rows and one channel tile of at most 128: the role-exchanged kernel, one CTA for all rows
    p->w_ts = p->w_mtiles * kTileM == kTsRows && f.n_pad <= kTileM;
    if (p->w_ts) p->w_mgroups = 1;
    const uint32_t stage_bytes = wg_smem(f.n_pad, subs, 2).stage_bytes;
    p->w_stages = std::max(2, std::min(kWgMaxStages, (int)((kSmemLimit - 8192) / stage_bytes)));
    p->w_smem = p->w_ts ? kTsSmem + 1024 : wg_smem(f.n_pad, subs, p->w_stages).total + 1024;
    const int n_pix = G.B * G.m * G.m;
    p->w_kblocks_total = (n_pix + kBlockK - 1) / kBlockK;
    const int out_tiles = p->w_mgroups * G.g * f.tiles;
    // Whole waves of CTAs (one CTA per SM), as few as keep a partial sum's accumulation chain within
    // kMaxChainKblocks: the tensor core's fp32 accumulation truncates, so the error of a partial sum grows with the
    // length of its chain, while the reduction over splits adds with proper rounding.
    int splits = 1;
    for (int waves = 1; waves <= 64; ++waves) {
      splits = std::max(1, waves * ctx->sm_count / out_tiles);
      if ((p->w_kblocks_total + splits - 1) / splits <= kMaxChainKblocks) break;
    }
    splits = std::min(splits, std::max(1, p->w_kblocks_total / 8));  // at least 8 k-blocks per CTA
    p->w_kblocks_per_split = (p->w_kblocks_total + splits - 1) / splits;
    p->w_splits = (p->w_kblocks_total + p->w_kblocks_per_split - 1) / p->w_kblocks_per_split;
    if (rc == CCT_OK)
      rc = dev_alloc(ctx, p, &p->w_partial, (size_t)p->w_splits * G.g * f.tiles * p->w_mtiles * kTileM * f.n_pad);
  }
  // ---- weight gradient through the gather kernel (the default): tiles = splits x channel tiles x M-tiles
  // It needs one extra pass over dY (split into hi / lo, 12 bytes moved per element), which pays when every dY
  // element takes part in many multiply-adds: measured faster from CaffeNet conv2 (1200 lowered rows) upwards,
  // slower for AlexNet conv1 (363 rows), so short lowered matrices keep the shared-memory kernel above.
  if (rc == CCT_OK && p->fwd.k_real >= 512) {
    const GatherProblem& f = p->fwd;
    GatherProblem& w = p->wgp;
    const int n_pix = G.B * G.m * G.m;
    const int kb_total = (n_pix + kBlockK - 1) / kBlockK;
    const int vgroups = G.g * f.tiles;
    w.tiles = f.tiles; w.ch_tile = f.ch_tile; w.n = f.n; w.n_pad = f.n_pad;
    w.k_real = n_pix;
    p->wg_mtiles = (f.k_real + kTileM - 1) / kTileM;  // no all-ones row here: the bias gradient comes from the dY pass
    const int base_tiles = vgroups * p->wg_mtiles;
    // Splits of the pixel range: all work units (base tiles x splits) cost the same, so the kernel's time is
    // (rounds of units over the resident CTAs) x (k-blocks per unit) - pick the split count that minimises it, plus the
    // traffic of the partial sums it creates (written once, read once by the reduction).  Chains stay bounded
    // (kMaxChainKblocks) and units no shorter than 16 k-blocks.  A last round that fills at most half of the slots of
    // the two-CTAs-per-SM shape costs about half a round: its CTAs have their SM's tensor pipe to themselves.
    {
      const bool two_per_sm = f.n_pad <= 128;  // the shape finish_problem() will pick for this accumulator width
      const int slots = ctx->planning_sms() * (two_per_sm ? 2 : 1);
      const double us_per_kblock = 12.0 * (f.n_pad / 2.0) / 1900.0 * (two_per_sm ? 2.0 : 1.0);
      double best = 0.0;
      int best_kps = 0;
      const int s_min = std::max(1, (kb_total + kMaxChainKblocks - 1) / kMaxChainKblocks);
      for (int s = s_min; s <= std::max(s_min, 8 * slots / base_tiles + 1); ++s) {
        const int kps = (kb_total + s - 1) / s;
        if (kps < 16 && best_kps) break;
        const int units = base_tiles * ((kb_total + kps - 1) / kps);
        const int tail = units % slots;
        const double rounds = units / slots + (tail == 0 ? 0.0 : (two_per_sm && 2 * tail <= slots) ? 0.55 : 1.0);
        const double reduce = 1.5 * units * (double)kTileM * f.n_pad * 8.0 / 6.5e6 / us_per_kblock;
        const double cost = rounds * kps + reduce;
        if (!best_kps || cost < best - 1e-9) { best = cost; best_kps = kps; }
      }
      p->wg_kps = best_kps;
    }
    p->wg_splits = (kb_total + p->wg_kps - 1) / p->wg_kps;
    w.k_pad = p->wg_kps * kBlockK;
    w.taps_smem = 0;
    w.map_k = (size_t)kb_total * kBlockK;
    std::vector<MaskTap> t((size_t)p->wg_splits * p->wg_kps * kBlockK);
    for (size_t i = 0; i < t.size(); ++i) {
      if ((long long)i < n_pix) {
        const int b = (int)(i / (G.m * G.m)), r = (int)(i % (G.m * G.m));
        const int iy0 = (r / G.m) * G.s - G.p, ix0 = (r % G.m) * G.s - G.p;
        uint32_t valid = 0;
        for (int a = 0; a < G.k; ++a) {
          if (iy0 + a >= 0 && iy0 + a < G.n) valid |= 1u << a;
          if (ix0 + a >= 0 && ix0 + a < G.n) valid |= 1u << (16 + a);
        }
        const long long off = (long long)b * G.D * G.n * G.n + (long long)iy0 * G.n + ix0;
        t[i] = MaskTap{(int)off, ~valid};
      } else {
        t[i] = MaskTap{0, 0xffffffffu};
      }
    }
    rc = upload(ctx, p, &p->wg_pix, t);
    if (rc == CCT_OK) rc = finish_problem(ctx, p, w, vgroups, 0);
    if (rc == CCT_OK && cudaMemsetAsync(w.w, 0, 2 * w.w_half * sizeof(float), ctx->stream) != cudaSuccess) {  // padded channel rows stay zero
      ctx->last_error = "cudaMemsetAsync of the pre-split dY buffer failed";
      rc = CCT_ERR_CUDA;
    }
    if (rc == CCT_OK && G.bias) rc = dev_alloc(ctx, p, &p->wg_plane_sums, (size_t)G.B * G.o);
    if (rc == CCT_OK) {
      cudaFree(p->w_partial);  // sized for the other kernel's split count
      p->bytes -= (size_t)p->w_splits * vgroups * p->w_mtiles * kTileM * f.n_pad * sizeof(float);
      p->w_partial = nullptr;
      rc = dev_alloc(ctx, p, &p->w_partial, (size_t)p->wg_splits * vgroups * p->wg_mtiles * kTileM * f.n_pad);
    }
    p->wg_gather = rc == CCT_OK;
  }
  if (rc == CCT_OK) rc = set_smem(ctx, gather_conv_kernel<4>, kSmemLimit);
  if (rc == CCT_OK) rc = set_smem(ctx, gather_conv_kernel<2>, 113 * 1024);
  if (rc == CCT_OK) rc = set_smem(ctx, wgrad_pick(p->w_subs, p->fwd.n_pad), kSmemLimit);
  if (rc == CCT_OK && p->w_ts) rc = set_smem(ctx, wgrad_ts_kernel, kSmemLimit);
  if (rc != CCT_OK) {
    umma_plan_destroy(ctx, p);
    return rc;
  }
  *out = p;
  return CCT_OK;
}

void umma_plan_destroy(cct_ctx* ctx, UmmaPlan* p) {
  if (!p) return;
  for (GatherProblem* gp : {&p->fwd, &p->dgr, &p->wgp}) { cudaFree(gp->taps); cudaFree(gp->cols); cudaFree(gp->w); }
  cudaFree(p->wg_pix); cudaFree(p->wg_plane_sums);
  cudaFree(p->w_taps); cudaFree(p->w_partial);
  delete p;
}

size_t umma_plan_workspace_bytes(const UmmaPlan* p) { return p->bytes; }

namespace {

void fill_common(GatherParams& P, const GatherProblem& gp, cct_ctx* ctx, int vgroups, int n_bias) {
  P.taps = gp.taps; P.cols = gp.cols;
  P.tiles_per_group = gp.tiles;
  P.out_tile_channels = gp.ch_tile;
  P.n = gp.n; P.n_pad = gp.n_pad; P.k_pad = gp.k_pad;
  P.taps_smem = gp.taps_smem < 0 ? gp.k_pad : gp.taps_smem;
  P.n_pix_tiles = (P.n_pix + kTileM - 1) / kTileM;
  P.total_tiles = P.n_pix_tiles * vgroups;
  P.a_stages = gp.a_stages; P.b_stages = gp.b_stages; P.acc_bufs = gp.acc_bufs;
  P.dual = gp.dual; P.acc_cols = gp.acc_cols; P.tmem_cols = gp.tmem_cols;
  P.n_bias = P.bias ? n_bias : 0;
  P.lo_row_offset = vgroups * gp.n_pad;
  P.status = ctx->status_dev;
}

// Persistent grid: one CTA per SM (4 producer sets) or two (2 sets).
void launch_gather(cct_ctx* ctx, const GatherParams& P, const GatherProblem& gp) {
  if (gp.sets == 2) {
    const int grid = std::min(P.total_tiles, 2 * ctx->launch_sms());
    launch_pdl(gather_conv_kernel<2>, dim3(grid), dim3(gather_threads(2)), gp.smem, ctx->stream, P, gp.map);
  } else {
    const int grid = std::min(P.total_tiles, ctx->launch_sms());
    launch_pdl(gather_conv_kernel<4>, dim3(grid), dim3(gather_threads(4)), gp.smem, ctx->stream, P, gp.map);
  }
}

}  // namespace

int umma_conv_forward(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* W, const float* bias, float* Y,
                      int relu, PhaseTimer* t, int batch, bool repack) {
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;  // an earlier bounded wait gave up: do not pile up behind it
  const ConvGeom& G = p->G;
  GatherProblem& f = p->fwd;
  const int vgroups = G.g * f.tiles;
  const int B = batch > 0 ? batch : G.B;  // a leading slice of the batch (host-buffer calls pipeline over slices)
  if (repack) {
    t->begin(4, ctx->stream);
    launch_pdl(pack_fwd_kernel, dim3(pack_grid(ctx, f.w_half)), dim3(256), 0, ctx->stream, W, f.w, f.w + f.w_half, vgroups, f.tiles, G.og,
                                                                     f.n, f.n_pad, f.k_real, f.k_pad);
    t->end(4, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  }
  GatherParams P{};
  P.in = X; P.out = Y;
  P.bias = G.bias ? bias : nullptr;
  P.n_pix = B * G.m * G.m; P.q_h = G.m; P.q_w = G.m;
  P.iy_mul = G.s; P.iy_add = -G.p; P.ix_mul = G.s; P.ix_add = -G.p;
  P.in_lim = G.n;
  P.tap_sign = 1; P.taps_per_axis = G.k;
  P.in_batch_stride = (long long)G.D * G.n * G.n;
  P.in_group_stride = G.Dg * G.n * G.n;
  P.oy_mul = 1; P.oy_add = 0; P.ox_mul = 1; P.ox_add = 0;
  P.out_lim = G.m; P.check_out = 0;
  P.out_pitch = G.m; P.out_plane = G.m * G.m;
  P.out_batch_stride = (long long)G.o * G.m * G.m;
  P.out_group_channels = G.og;
  P.relu = relu;
  fill_common(P, f, ctx, vgroups, G.o);
  t->begin(0, ctx->stream);
  launch_gather(ctx, P, f);
  t->end(0, ctx->stream);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}

int umma_conv_backward(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* W, const float* dY, float* dX,
                       float* dW, float* db, PhaseTimer* t) {
  int rc = umma_conv_wgrad(ctx, p, X, dY, dW, db, t);
  if (rc == CCT_OK && dX) rc = umma_conv_dgrad(ctx, p, W, dY, dX, t, 0, true);
  return rc;
}

// Weight + bias gradient over the whole batch.
int umma_conv_wgrad(cct_ctx* ctx, UmmaPlan* p, const float* X, const float* dY, float* dW, float* db, PhaseTimer* t) {
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;
  const ConvGeom& G = p->G;
  if (p->wg_gather) {
    const GatherProblem& f = p->fwd;
    GatherProblem& w = p->wgp;
    const int vgroups = G.g * f.tiles, mm = G.m * G.m;
    t->begin(1, ctx->stream);
    launch_pdl(split_dy_kernel, dim3(std::min((G.B * G.o + 7) / 8, ctx->sm_count * 8)), dim3(256), 0, ctx->stream, 
        dY, w.w, w.w + w.w_half, G.bias ? p->wg_plane_sums : nullptr, G.B * G.o, G.o, mm, G.og, f.ch_tile, f.tiles,
        f.n_pad, w.map_k);
    CCT_CHECK_LAUNCH(ctx);
    GatherParams P{};
    P.in = X; P.out = p->w_partial; P.bias = nullptr;
    P.n_pix = p->wg_mtiles * kTileM;  // lanes = rows of the lowered matrix
    P.in_lim = G.n;
    P.in_group_stride = G.Dg * G.n * G.n;
    P.wg = 1; P.wg_mtiles = p->wg_mtiles; P.wg_vgroups = vgroups; P.wg_rows_pad = p->wg_mtiles * kTileM;
    P.wg_k = G.k; P.wg_kreal = f.k_real;
    fill_common(P, w, ctx, vgroups, 0);
    P.taps = p->wg_pix; P.cols = nullptr;
    P.total_tiles = p->wg_splits * vgroups * p->wg_mtiles;
    launch_gather(ctx, P, w);
    t->end(1, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
    t->begin(2, ctx->stream);
    launch_wgrad_reduce(ctx, p->w_partial, dW, nullptr, p->wg_splits, vgroups, f.tiles, p->wg_mtiles * kTileM, f.n,
                        f.n_pad, f.k_real, G.og);
    if (G.bias) launch_pdl(bias_grad_kernel, dim3((G.o + 7) / 8), dim3(256), 0, ctx->stream, p->wg_plane_sums, db, G.B, G.o);
    t->end(2, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  } else {
    const GatherProblem& f = p->fwd;
    WgradParams P{};
    P.x = X; P.dy = dY; P.partial = p->w_partial; P.taps = p->w_taps;
    P.n_pix = G.B * G.m * G.m; P.m = G.m; P.mm = G.m * G.m; P.n = G.n; P.s = G.s; P.p = G.p; P.k = G.k;
    P.x_batch_stride = (long long)G.D * G.n * G.n;
    P.x_group_stride = G.Dg * G.n * G.n;
    P.dy_batch_stride = (long long)G.o * G.m * G.m;
    P.dy_group_channels = G.og;
    P.tiles_per_group = f.tiles;
    P.n_real = f.n; P.n_pad = f.n_pad;
    P.m_tiles = p->w_mtiles; P.subs = p->w_subs; P.stages = p->w_stages;
    P.ones_row = f.k_real;
    P.kblocks_total = p->w_kblocks_total; P.kblocks_per_split = p->w_kblocks_per_split;
    P.status = ctx->status_dev;
    const int vgroups = G.g * f.tiles;
    dim3 grid(p->w_mgroups, p->w_splits, vgroups);
    t->begin(1, ctx->stream);
    if (p->w_ts)
      launch_pdl(wgrad_ts_kernel, dim3(grid), dim3(kTsThreads), p->w_smem, ctx->stream, P);
    else
      launch_pdl(wgrad_pick(p->w_subs, f.n_pad), dim3(grid), dim3(kWgThreads), p->w_smem, ctx->stream, P);
    t->end(1, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
    t->begin(2, ctx->stream);
    launch_wgrad_reduce(ctx, p->w_partial, dW, G.bias ? db : nullptr, p->w_splits, vgroups, f.tiles,
                        p->w_mtiles * kTileM, f.n, f.n_pad, f.k_real, G.og);
    t->end(2, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  }
  return CCT_OK;
}

// Data gradient of the first `batch` images (0: all of them); `repack` rewrites the packed weights from W first.
int umma_conv_dgrad(cct_ctx* ctx, UmmaPlan* p, const float* W, const float* dY, float* dX, PhaseTimer* t, int batch,
                    bool repack) {
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;
  const ConvGeom& G = p->G;
  const int B = batch > 0 ? batch : G.B;
  {
    GatherProblem& d = p->dgr;
    const int vgroups = G.g * d.tiles;
    t->begin(3, ctx->stream);
    if (repack) {
      launch_pdl(pack_dgrad_kernel, dim3(pack_grid(ctx, d.w_half)), dim3(256), 0, ctx->stream, W, d.w, d.w + d.w_half, vgroups, d.tiles, G.og,
                                                                         G.Dg, G.k, G.s, p->dgr_taps, d.ch_tile, d.n,
                                                                         d.n_pad, d.k_real, d.k_pad);
      CCT_CHECK_LAUNCH(ctx);
    }
    GatherParams P{};
    P.in = dY; P.out = dX; P.bias = nullptr;
    P.n_pix = B * p->dgr_q * p->dgr_q; P.q_h = p->dgr_q; P.q_w = p->dgr_q;
    P.iy_mul = 1; P.iy_add = p->dgr_q0; P.ix_mul = 1; P.ix_add = p->dgr_q0;
    P.in_lim = G.m;
    P.tap_sign = -1; P.taps_per_axis = p->dgr_taps;
    P.in_batch_stride = (long long)G.o * G.m * G.m;
    P.in_group_stride = G.og * G.m * G.m;
    P.oy_mul = G.s; P.oy_add = p->dgr_q0 * G.s - G.p; P.ox_mul = G.s; P.ox_add = p->dgr_q0 * G.s - G.p;
    P.out_lim = G.n; P.check_out = 1;
    P.out_pitch = G.n; P.out_plane = G.n * G.n;
    P.out_batch_stride = (long long)G.D * G.n * G.n;
    P.out_group_channels = G.Dg;
    P.relu = 0;
    fill_common(P, d, ctx, vgroups, 0);
    launch_gather(ctx, P, d);
    t->end(3, ctx->stream);
    CCT_CHECK_LAUNCH(ctx);
  }
  return CCT_OK;
}

// ------------------------------------------------------------------ weight gradient without any allocation
// Scratch for cct_conv_weight_grad_noalloc: the lowered-matrix row table followed by the split partial sums.  It is a
// fixed part of the library image: every device that loads the library holds these 16 MiB until the process exits.
constexpr size_t kNoAllocScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
// Device address of the array above, per device ordinal, looked up once.  In host code the array's name is only a
// handle for the runtime, never an address a kernel may be given.
static void* g_noalloc_dev_ptr[64] = {};

namespace {

// Fills the weight-gradient row table on the device (the plan-based path builds it on the host and uploads it).
__global__ void noalloc_taps_kernel(MaskTap* taps, int rows, int k_real, int k, int n) {
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x) {
    MaskTap t;
    if (i < k_real) {
      const int d = i / (k * k), kr = (i / k) % k, kc = i % k;
      t.off = d * n * n + kr * n + kc;
      t.bits = kWgValidBit | (1u << kr) | (1u << (16 + kc));
    } else {
      t.off = 0;
      t.bits = i == k_real ? kWgOnesBits : kWgPadBit;
    }
    taps[i] = t;
  }
}

}  // namespace

extern "C" int cct_conv_weight_grad_noalloc(cct_ctx* ctx, const cct_conv_desc* desc, const float* X, const float* dY,
                                            float* dW, float* db) {
  if (!ctx || !desc || !X || !dY || !dW) return CCT_ERR_INVALID;
  if (desc->batch <= 0 || desc->in_depth <= 0 || desc->in_size <= 0 || desc->out_depth <= 0 || desc->kernel <= 0 ||
      desc->stride <= 0 || desc->pad < 0 || desc->groups <= 0 || desc->in_depth % desc->groups ||
      desc->out_depth % desc->groups || desc->in_size + 2 * desc->pad < desc->kernel)
    return CCT_ERR_INVALID;
  if (desc->bias_term && !db) return CCT_ERR_INVALID;
  ConvGeom G;
  G.B = desc->batch; G.D = desc->in_depth; G.n = desc->in_size; G.o = desc->out_depth;
  G.k = desc->kernel; G.s = desc->stride; G.p = desc->pad; G.g = desc->groups;
  G.m = (G.n + 2 * G.p - G.k) / G.s + 1;
  G.Dg = G.D / G.g; G.og = G.o / G.g; G.bias = desc->bias_term != 0;
  if ((double)G.B * G.D * G.n * G.n > 2147483647.0 || (double)G.B * G.o * G.m * G.m > 2147483647.0 ||
      !umma_supported(G)) {
    ctx->last_error = "cct_conv_weight_grad_noalloc: shape outside what the tensor-core path supports";
    return CCT_ERR_UNSUPPORTED;
  }
  if (ctx->device < 0 || ctx->device >= 64) return CCT_ERR_UNSUPPORTED;
  if (*ctx->status_host != 0) return CCT_ERR_TIMEOUT;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  // Set-up, once per device and with that device current: ask the runtime where the array lives on this device.
  if (!g_noalloc_dev_ptr[ctx->device]) {
    void* ptr = nullptr;
    CCT_CUDA(ctx, cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    g_noalloc_dev_ptr[ctx->device] = ptr;
  }
  unsigned char* scratch = static_cast<unsigned char*>(g_noalloc_dev_ptr[ctx->device]);

  // Same tiling rules as the plan-based path.
  const int tiles = channel_tiles(G.og, 1);
  const int n_real = G.og / tiles, n_pad = round_up(n_real, 16);
  const int k_real = G.Dg * G.k * G.k;
  const int m_tiles = (k_real + 1 + kTileM - 1) / kTileM;
  int subs = 1;
  for (int u = 2; u <= kWgMaxSubs; ++u)
    if (u <= m_tiles && u * (n_pad <= 64 ? 2 : 1) * n_pad <= 512 &&
        2 * wg_smem(n_pad, u, 2).stage_bytes + 8192 <= (uint32_t)kSmemLimit)
      subs = u;
  const int mgroups = (m_tiles + subs - 1) / subs;
  const int stages = std::max(2, std::min(kWgMaxStages, (int)((kSmemLimit - 8192) / wg_smem(n_pad, subs, 2).stage_bytes)));
  const size_t smem = wg_smem(n_pad, subs, stages).total + 1024;
  const int vgroups = G.g * tiles;
  const size_t taps_bytes = ((size_t)m_tiles * kTileM * sizeof(MaskTap) + 255) & ~(size_t)255;
  const size_t split_bytes = (size_t)vgroups * m_tiles * kTileM * n_pad * sizeof(float);
  if (taps_bytes + split_bytes > kNoAllocScratchBytes) {
    char msg[200];
    snprintf(msg, sizeof msg,
             "cct_conv_weight_grad_noalloc: this layer needs %zu bytes of scratch for one split, the built-in buffer "
             "holds %zu",
             taps_bytes + split_bytes, kNoAllocScratchBytes);
    ctx->last_error = msg;
    return CCT_ERR_UNSUPPORTED;
  }
  const int n_pix = G.B * G.m * G.m;
  const int kblocks_total = (n_pix + kBlockK - 1) / kBlockK;
  // Splits: one wave of CTAs, and - as in the plan-based path - enough of them that no partial sum's accumulation
  // chain exceeds kMaxChainKblocks (the tensor core's fp32 accumulate truncates; the split reduction rounds).  When
  // the array cannot hold that many partial-sum slices, the pixel range is covered in several rounds of (weight
  // gradient kernel, reduction), each round reusing the slices and the later reductions adding to dW / db.
  int want = std::max(1, ctx->sm_count / (mgroups * vgroups));
  want = std::max(want, (kblocks_total + kMaxChainKblocks - 1) / kMaxChainKblocks);
  want = std::min(want, std::max(1, kblocks_total / 8));  // at least 8 k-blocks per CTA (kMaxChainKblocks > 8)
  const int kblocks_per_split = (kblocks_total + want - 1) / want;
  const int total_splits = (kblocks_total + kblocks_per_split - 1) / kblocks_per_split;
  const int slots = (int)std::min<size_t>((kNoAllocScratchBytes - taps_bytes) / split_bytes, (size_t)total_splits);

  MaskTap* taps = reinterpret_cast<MaskTap*>(scratch);
  float* partial = reinterpret_cast<float*>(scratch + taps_bytes);
  WgradKernel kernel = wgrad_pick(subs, n_pad);
  CCT_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
  launch_pdl(noalloc_taps_kernel, dim3(8), dim3(256), 0, ctx->stream, taps, m_tiles * kTileM, k_real, G.k, G.n);
  CCT_CHECK_LAUNCH(ctx);
  WgradParams P{};
  P.x = X; P.dy = dY; P.partial = partial; P.taps = taps;
  P.n_pix = n_pix; P.m = G.m; P.mm = G.m * G.m; P.n = G.n; P.s = G.s; P.p = G.p; P.k = G.k;
  P.x_batch_stride = (long long)G.D * G.n * G.n;
  P.x_group_stride = G.Dg * G.n * G.n;
  P.dy_batch_stride = (long long)G.o * G.m * G.m;
  P.dy_group_channels = G.og;
  P.tiles_per_group = tiles;
  P.n_real = n_real; P.n_pad = n_pad;
  P.m_tiles = m_tiles; P.subs = subs; P.stages = stages;
  P.ones_row = k_real;
  P.kblocks_per_split = kblocks_per_split;
  P.status = ctx->status_dev;
  for (int first = 0, round = 0; first < total_splits; first += slots, ++round) {
    const int here = std::min(slots, total_splits - first);
    P.kb_first = first * kblocks_per_split;
    P.kblocks_total = std::min(kblocks_total, P.kb_first + here * kblocks_per_split);
    launch_pdl(kernel, dim3(dim3(mgroups, here, vgroups)), dim3(kWgThreads), smem, ctx->stream, P);
    CCT_CHECK_LAUNCH(ctx);
    launch_wgrad_reduce(ctx, partial, dW, G.bias ? db : nullptr, here, vgroups, tiles, m_tiles * kTileM, n_real, n_pad,
                        k_real, G.og, round > 0);
    CCT_CHECK_LAUNCH(ctx);
  }
  return CCT_OK;
}

// ------------------------------------------------------------------ the bounded wait, exercised on purpose
namespace {
// One warp waits - through the same mbar_wait the convolution kernels use - for a barrier phase that nothing will ever
// complete, with a short limit.  The wait gives up, records `code` in the status word and the kernel returns
// normally: no trap, no fault, the context stays usable.
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles, int code) {
  pdl_wait();
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  bool failed = false;
  mbar_wait(bar, 0u, failed, status, code, limit_cycles);
}
}  // namespace

extern "C" int cct_selftest_bounded_wait(cct_ctx* ctx, long long limit_cycles) {
  if (!ctx || limit_cycles <= 0 || limit_cycles > kWaitLimitCycles) return CCT_ERR_INVALID;
  CCT_CUDA(ctx, cudaSetDevice(ctx->device));
  launch_pdl(bounded_wait_selftest_kernel, dim3(1), dim3(32), 0, ctx->stream, ctx->status_dev, limit_cycles, 0x7e57);
  CCT_CHECK_LAUNCH(ctx);
  return CCT_OK;
}
