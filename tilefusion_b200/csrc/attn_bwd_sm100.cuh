// Attention backward for sm_100a: dQ, dK, dV from Q, K, V, O, dO and the
// log-sum-exp rows the forward kernels emit.  TileFusion has no backward pass
// (its attention path ends at include/kernels/flash_attention_device.cuh:130-312);
// this extends the path with the same building blocks as the forward kernel in
// attn_fwd_sm100.cuh: TMA tile loads with 128-byte swizzle, tcgen05.mma with
// accumulators in tensor memory, one thread per tile row for the element-wise
// stage, every wait bounded.
//
// Per (batch, head), with s = softmax_scale:
//   P  = exp(s Q K^T - LSE)            (recomputed tile by tile, never stored)
//   dV = P^T dO          dP = dO V^T          delta_i = sum_d dO_id O_id
//   dS = P o (dP - delta) * s          dQ = dS K          dK = dS^T Q
// Three kernels:
//   attn_bwd_delta_kernel   delta rows (fp32), D / 8 lanes per query row;
//   attn_bwd_dkv_kernel     work item = one 128-key tile, loops over the query tiles:
//                           S^T = K Q^T and dP^T = V dO^T into tensor memory
//                           (keys on the 128 lanes), threads turn them into P^T
//                           and dS^T (16-bit, written over the fp32 tiles they
//                           came from) and the second pair of MMAs reads those as
//                           TMEM A operands: dV += P^T dO, dK += dS^T Q.  The dO
//                           and Q tiles in shared memory serve both pairs: as
//                           K-major B operands of the first and MN-major B
//                           operands of the second, so nothing is transposed;
//   attn_bwd_dq_kernel      work item = one 128-query tile, loops over the key tiles:
//                           S = Q K^T, dP = dO V^T, dS over dP, dQ += dS K.
// A streamed tile is worked in two halves of 64 rows that alternate between two
// TMEM buffers, so the element-wise stage of one half runs under the MMAs of its
// neighbours.  TMEM: two buffers of (S | dP) = 2 x (64 + 64) columns, then dV | dK
// (D + D columns; dK/dV kernel) or dQ and, in the columns the dQ kernel has left,
// copies of its fixed tiles Q and dO as TMEM A operands of the first MMA pair.
// One warp issues all copies and MMAs (warp-uniform code, one elected lane),
// eight warps do the element-wise stage.  Both kernels are persistent: one CTA
// per SM walks the work items, and the barrier phases run on across them, so an
// item's loads and first MMAs overlap the previous item's epilogue.
// P and dS are rounded to the 16-bit input type before the second MMAs, all
// accumulation is fp32.  The two kernels recompute S and dP independently (7
// tile products per tile pair instead of 5), which keeps dQ free of atomics and
// the results deterministic.
#pragma once

#include <type_traits>

#include "attn_fwd_sm100.cuh"

namespace tfb {

struct AttnBwdArgs {
  const float* lse;        // [B, H, Lq] natural log, as written by the forward
  const float* delta;      // [B, H, Lq]
  void* dq;
  void* dk;
  void* dv;
  int len_q;
  int len_kv;
  int causal;
  float scale;             // softmax_scale
  float scale_log2;        // softmax_scale * log2(e)
  long long dq_stride_b, dq_stride_h, dq_stride_l;
  long long dk_stride_b, dk_stride_h, dk_stride_l;
  long long dv_stride_b, dv_stride_h, dv_stride_l;
  long long row_stride_b, row_stride_h;     // of lse and delta
  int heads;
  int batch;
};

struct AttnBwdDeltaArgs {
  const void* o;
  const void* d_o;
  float* delta;
  int len_q;
  int heads;
  long long rows;          // B * H * Lq
  long long o_stride_b, o_stride_h, o_stride_l;
  long long do_stride_b, do_stride_h, do_stride_l;
};

// delta[b, h, i] = sum_d O[b, h, i, d] * dO[b, h, i, d]; D / 8 lanes per row, 16 bytes per lane and tensor.
constexpr int kBwdDeltaThreads = 256;
template <int D>
struct BwdDeltaShape {
  static constexpr int kRowsPerBlock = kBwdDeltaThreads / (D / 8);
};

template <typename T, int D>
__global__ void __launch_bounds__(kBwdDeltaThreads) attn_bwd_delta_kernel(const AttnBwdDeltaArgs a) {
  constexpr int kLanes = D / 8;             // 16 (D = 128) or 8 (D = 64) lanes share a row
  const long long row = (long long)blockIdx.x * BwdDeltaShape<D>::kRowsPerBlock + threadIdx.x / kLanes;
  const int part = threadIdx.x % kLanes;
  float acc = 0.f;
  if (row < a.rows) {
    const long long bh = row / a.len_q;
    const int i = (int)(row - bh * a.len_q);
    const int b = (int)(bh / a.heads), h = (int)(bh - (long long)b * a.heads);
    const T* o = reinterpret_cast<const T*>(a.o) + b * a.o_stride_b + h * a.o_stride_h + i * a.o_stride_l;
    const T* g = reinterpret_cast<const T*>(a.d_o) + b * a.do_stride_b + h * a.do_stride_h + i * a.do_stride_l;
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(o + part * 8));
    const uint4 y = __ldg(reinterpret_cast<const uint4*>(g + part * 8));
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 xf = unpack2<T>(xw[e]), yf = unpack2<T>(yw[e]);
      acc = fmaf(xf.x, yf.x, acc);
      acc = fmaf(xf.y, yf.y, acc);
    }
  }
#pragma unroll
  for (int off = kLanes / 2; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (part == 0 && row < a.rows) a.delta[row] = acc;
}

template <int D>
struct AttnBwdSmem {
  static constexpr int kTileBytes = kAttnTile * D * 2;
  static constexpr int kBlockBytes = kAttnTile * 128;
  // fixed pair (K, V in the dK/dV kernel; Q, dO in the dQ kernel), then two slots of the streamed pair
  static constexpr int kOffFixed = 0;
  static constexpr int kOffStream = 2 * kTileBytes;
  static constexpr int kOffRows = 6 * kTileBytes;               // lse2 / delta of the streamed tile: [2][2][128] fp32
  static constexpr int kOffBar = kOffRows + 2 * 2 * kAttnTile * 4;
  static constexpr int kOffTmemSlot = kOffBar + 96;
  static constexpr int kOffAbort = kOffBar + 100;
  static constexpr int kBytes = kOffBar + 128 + 1024;
};

enum AttnBwdWaitCode {
  kBWaitFixed = 501, kBWaitStream = 502, kBWaitS = 503, kBWaitP = 504, kBWaitSlot = 505, kBWaitEpi = 506,
  kBWaitDrain = 507, kBWaitAcc = 508
};

// Element-wise warps: 4 (one thread per row of the fixed tile) or 8 (two threads per row, 32 of the 64
// streamed columns of a half tile each).  While the MMAs were issued from a branch on lane 0 (95 clocks per
// MMA) eight were no faster than four (520 against 534 TFLOP/s on the fp16 prefill config); with the
// warp-uniform issuer they are: 636 against 591.
constexpr int kBwdComputeWarps = 8;
constexpr int kBwdThreads = (kBwdComputeWarps + 1) * 32;  // + the TMA / MMA issuer warp

__device__ __forceinline__ void bwd_rows_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kBwdComputeWarps * 32) : "memory");
}

// Shared by the two kernels: which tensor plays which role is the only difference.
//   kDkv = true : fixed = (K, V) of key tile `tile`;  streamed = (Q, dO) of query tiles
//                 lanes = keys;   outputs dV (columns 256..) and dK
//   kDkv = false: fixed = (Q, dO) of query tile `tile`; streamed = (K, V) of key tiles
//                 lanes = queries; output dQ
// Persistent: one CTA per SM walks the work items (batch, head, fixed tile) number blockIdx.x,
// blockIdx.x + gridDim.x, ...; all barrier phases run on across items (counted in streamed tiles and
// items), so that the loads and the first MMAs of an item are issued while the element-wise warps
// still write the previous item's gradients out.  Items are head-major (the CTAs running at any
// moment stream the same few heads); under a causal mask the tiles of a head are taken heaviest
// first in even heads and lightest first in odd ones, which evens out what a CTA gets.
struct BwdItem {
  int tile, head, batch;
  int first, n;            // streamed tiles visited: [first, first + n), n >= 1
};

template <bool kDkv>
__device__ __forceinline__ BwdItem bwd_item_decode(const AttnBwdArgs& args, int item, int n_tiles, int n_q_tiles,
                                                   int n_kv_tiles) {
  BwdItem it;
  const int bh = item / n_tiles;
  int r = item - bh * n_tiles;
  if (args.causal && (bh & 1)) r = n_tiles - 1 - r;
  it.batch = bh / args.heads;
  it.head = bh - it.batch * args.heads;
  if (kDkv) {
    it.tile = r;                                            // key tile 0 is seen by every query tile
    it.first = args.causal ? it.tile : 0;                   // query tiles above the diagonal see none of these keys
    it.n = n_q_tiles - it.first;                            // (>= 1: key tiles no query sees are not items)
  } else {
    it.tile = args.causal ? n_tiles - 1 - r : r;            // the last query tile sees the most keys
    it.first = 0;
    it.n = args.causal ? min(n_kv_tiles, it.tile + 1) : n_kv_tiles;
  }
  return it;
}

template <typename T, int D, bool kDkv>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const AttnBwdArgs args) {
  using S = AttnBwdSmem<D>;
  constexpr int kIsBf16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr int kTmemCols = 512;
  // Two buffers of (S | dP) for 64 streamed rows each: buffer b has S in columns [128 b, 128 b + 64) and
  // dP in [128 b + 64, 128 b + 128); the accumulators follow.
  constexpr int kColAcc0 = 256, kColAcc1 = 256 + D;
  // dQ kernel: the accumulator takes D columns only, so the fixed tiles (Q, dO) are copied into the
  // remaining tensor memory (D / 2 columns each, two 16-bit values per column) and serve as TMEM A
  // operands of the first MMA pair: 43 instead of 76 clocks per M128 N64 K16 product.  At head dim
  // 64 the dK/dV kernel's two accumulators end at column 384 as well, and K and V go the same way.
  constexpr int kColFixA0 = 384, kColFixA1 = 384 + D / 2;
  constexpr bool kFixedInTmem = !kDkv || D == 64;
  static_assert(!kFixedInTmem || (kDkv ? 256 + 2 * D : 256 + D) <= kColFixA0, "accumulators overlap the fixed tiles");
  static_assert(kColFixA1 + D / 2 <= kTmemCols, "fixed tiles exceed tensor memory");
  constexpr int kBlocks = D / 64;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sFix0 = smem_base + S::kOffFixed;                    // K (dkv) / Q (dq)
  const uint32_t sFix1 = sFix0 + S::kTileBytes;                       // V (dkv) / dO (dq)
  auto sStr0 = [&](int slot) { return smem_base + S::kOffStream + slot * 2 * S::kTileBytes; };   // Q / K
  auto sStr1 = [&](int slot) { return sStr0(slot) + S::kTileBytes; };                            // dO / V
  float* s_rows = reinterpret_cast<float*>(smem_gen + S::kOffRows);   // [slot][lse2 | delta][128]
  const uint32_t bar_fix = smem_base + S::kOffBar + 0;
  const uint32_t bar_str = smem_base + S::kOffBar + 8;     // [2]
  const uint32_t bar_s = smem_base + S::kOffBar + 24;      // [2]  first MMA pair of a half tile is complete (per TMEM buffer)
  const uint32_t bar_p = smem_base + S::kOffBar + 40;      // [2]  P / dS of a half tile are in place (per TMEM buffer)
  const uint32_t bar_o = smem_base + S::kOffBar + 56;      // [2]  second MMA pairs of a streamed tile are complete (per slot)
  const uint32_t bar_fixt = smem_base + S::kOffBar + 72;   //      the fixed tiles are in tensor memory (where they are copied there)
  const uint32_t bar_acc = smem_base + S::kOffBar + 80;    //      the item's gradients have left the accumulators
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + S::kOffTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + S::kOffAbort);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_q_tiles = (args.len_q + kAttnTile - 1) / kAttnTile;
  const int n_kv_tiles = (args.len_kv + kAttnTile - 1) / kAttnTile;
  // Every item has at least one streamed tile: under a causal mask the key tiles that no query can see
  // (more keys than queries) are not items; their gradients are zero-filled after the loop.
  const int n_tiles = kDkv ? (args.causal ? min(n_kv_tiles, n_q_tiles) : n_kv_tiles) : n_q_tiles;
  const int n_items = n_tiles * args.heads * args.batch;

  if (threadIdx.x == 0) {
    mbar_init(bar_fix, 1);
    mbar_init(bar_str, 1);
    mbar_init(bar_str + 8, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_p, kBwdComputeWarps * 32);
    mbar_init(bar_p + 8, kBwdComputeWarps * 32);
    mbar_init(bar_o, 1);
    mbar_init(bar_o + 8, 1);
    mbar_init(bar_fixt, 128);
    mbar_init(bar_acc, kBwdComputeWarps * 32);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kBwdComputeWarps) {
    tmem_alloc<kTmemCols>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kBwdComputeWarps) {
    {
      // ------------------------------------------------ TMA + MMA issuer ----
      // The whole warp walks the schedule and one elected lane issues: in warp-uniform code the
      // descriptors stay in uniform registers and an MMA is issued every ~74 clocks, where a
      // branch on lane 0 took ~95 per MMA (bench.py --workload mma_rate) -- more than the tensor
      // pipe needs for the M128 N64 products of this kernel.
      const bool leader = elect_one();
      if (leader) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
      }
      const CUtensorMap* m_fix0 = kDkv ? &map_k : &map_q;
      const CUtensorMap* m_fix1 = kDkv ? &map_v : &map_do;
      const CUtensorMap* m_str0 = kDkv ? &map_q : &map_k;
      const CUtensorMap* m_str1 = kDkv ? &map_do : &map_v;
      // All operands are [128 rows][D] tiles, rows 128 B per 64-column block, 128-byte swizzle.
      // Descriptors are kept as 32-bit low halves (address and LBO; the high half is the same for all)
      // and advanced by constants: one thread issues every MMA, and building a 64-bit descriptor per
      // MMA costs it more clocks (96 per MMA, measured) than the tensor pipe needs for the MMA.
      //   K-major operand of a product over D (rows = the tile's own index): 32 bytes per K16 step
      //   within a 64-column block, LBO 16;
      //   MN-major B operand of a product over the tile's rows (N = D): 16 rows = 2048 bytes per K16
      //   step, LBO = one 64-column block.
      auto koff = [](int k) { return (uint32_t)(((k >> 2) * S::kBlockBytes + (k & 3) * 32) >> 4); };
      const uint32_t fix0_lo = desc_lo(sFix0, 16), fix1_lo = desc_lo(sFix1, 16);
      const uint32_t str0_k_lo[2] = {desc_lo(sStr0(0), 16), desc_lo(sStr0(1), 16)};
      const uint32_t str1_k_lo[2] = {desc_lo(sStr1(0), 16), desc_lo(sStr1(1), 16)};
      const uint32_t str0_r_lo[2] = {desc_lo(sStr0(0), S::kBlockBytes), desc_lo(sStr0(1), S::kBlockBytes)};
      const uint32_t str1_r_lo[2] = {desc_lo(sStr1(0), S::kBlockBytes), desc_lo(sStr1(1), S::kBlockBytes)};
      const uint32_t idesc_sd = make_idesc(128, 64, kIsBf16, 0, 0);
      const uint32_t idesc_acc = make_idesc(128, D, kIsBf16, 0, 1);

      uint32_t g = 0;          // streamed tiles of earlier items: slots and phases of bar_str / bar_s / bar_p / bar_o
      uint32_t k_item = 0;     // earlier items: phases of bar_fix / bar_fixt / bar_acc
      bool ok = true;
      for (int number = blockIdx.x; ok && number < n_items; number += gridDim.x, ++k_item) {
      const BwdItem item = bwd_item_decode<kDkv>(args, number, n_tiles, n_q_tiles, n_kv_tiles);
      const int n = item.n, first = item.first, head = item.head, batch = item.batch;
      const int t0 = item.tile * kAttnTile;
      auto load_tile = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int row0) {
#pragma unroll
        for (int blk = 0; blk < kBlocks; ++blk)
          tma_load_4d(dst + blk * S::kBlockBytes, map, bar, blk * 64, row0, head, batch);
      };
      auto load_stream = [&](int it) {
        if (!leader) return;
        const int slot = (g + it) & 1;
        mbar_arrive_expect_tx(bar_str + slot * 8, 2 * S::kTileBytes);
        load_tile(sStr0(slot), m_str0, bar_str + slot * 8, (first + it) * kAttnTile);
        load_tile(sStr1(slot), m_str1, bar_str + slot * 8, (first + it) * kAttnTile);
      };
      // Shared memory is free once every MMA of the previous item has completed: the commit of its
      // last streamed tile covers them all.
      if (g > 0) {
        ok = mbar_wait_warp(bar_o + ((g - 1) & 1) * 8, ((g - 1) >> 1) & 1, abort_flag, kBWaitDrain);
        if (!ok) break;
      }
      if (leader) {
        mbar_arrive_expect_tx(bar_fix, 2 * S::kTileBytes);
        load_tile(sFix0, m_fix0, bar_fix, t0);
        load_tile(sFix1, m_fix1, bar_fix, t0);
      }
      load_stream(0);
      if (n > 1) load_stream(1);

      // A streamed tile is worked in two halves of 64 rows (u = 2 it + half), alternating between
      // the two TMEM buffers, so that the element-wise stage of one half runs under the MMAs of its
      // neighbours.  Issue order:  P1(0) P1(1) | P2(0) P1(2) | P2(1) P1(3) | ...
      //   P1(u): lanes x 64 streamed rows, contraction over D, into buffer u & 1
      //          dkv: S^T = K Q^T, dP^T = V dO^T        dq: S = Q K^T, dP = dO V^T
      //   P2(u): A from tensor memory (16-bit P / dS of buffer u & 1: rows 0..31 of the half in columns
      //          0..15 of S resp. dP, rows 32..63 in columns 32..47), contraction over the 64 rows
      //          dkv: dV += P^T dO, dK += dS^T Q        dq: dQ += dS K
      // The tensor pipe executes in issue order, so P1(u + 2) overwrites buffer u & 1 only after P2(u)
      // has read it.
      const int n_half = 2 * n;
      ok = kFixedInTmem ? mbar_wait_warp(bar_fixt, k_item & 1, abort_flag, kBWaitFixed)
                        : mbar_wait_warp(bar_fix, k_item & 1, abort_flag, kBWaitFixed);
      if (kFixedInTmem) tc_fence_after();
      auto issue_p1 = [&](int u) -> bool {
        const int it = u >> 1, hh = u & 1, slot = (g + it) & 1, b = u & 1;
        if (hh == 0) {
          if (!mbar_wait_warp(bar_str + slot * 8, ((g + it) >> 1) & 1, abort_flag, kBWaitStream)) return false;
          tc_fence_after();
        }
        if (!leader) return true;
        const uint32_t rows = (hh * 64 * 128) >> 4;     // 64 rows of 128 B inside every 64-column block
        const uint32_t b0 = str0_k_lo[slot] + rows, b1 = str1_k_lo[slot] + rows;
        if (kFixedInTmem) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_ts_lohi(tmem_base + b * 128, tmem_base + kColFixA0 + k * 8, b0 + koff(k), kDescHiSw128, idesc_sd, k > 0);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_ts_lohi(tmem_base + b * 128 + 64, tmem_base + kColFixA1 + k * 8, b1 + koff(k), kDescHiSw128, idesc_sd, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_ss_lohi(tmem_base + b * 128, fix0_lo + koff(k), b0 + koff(k), kDescHiSw128, idesc_sd, k > 0);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_ss_lohi(tmem_base + b * 128 + 64, fix1_lo + koff(k), b1 + koff(k), kDescHiSw128, idesc_sd, k > 0);
        }
        umma_commit(bar_s + b * 8);
        return true;
      };
      if (ok) ok = issue_p1(0);
      for (int u = 0; ok && u < n_half; ++u) {
        const int it = u >> 1, hh = u & 1, slot = (g + it) & 1, b = u & 1;
        if (u + 1 < n_half) {
          ok = issue_p1(u + 1);
          if (!ok) break;
        }
        // the other slot is free once the second pairs of the previous tile have read it
        if (hh == 0 && it >= 1 && it + 1 < n) {
          ok = mbar_wait_warp(bar_o + (slot ^ 1) * 8, ((g + it - 1) >> 1) & 1, abort_flag, kBWaitSlot);
          if (!ok) break;
          load_stream(it + 1);
        }
        ok = mbar_wait_warp(bar_p + b * 8, ((2 * g + u) >> 1) & 1, abort_flag, kBWaitP);
        if (!ok) break;
        if (u == 0 && k_item > 0) {
          // the first accumulating MMAs overwrite the accumulators: the previous item's gradients must have left
          ok = mbar_wait_warp(bar_acc, (k_item - 1) & 1, abort_flag, kBWaitAcc);
          if (!ok) break;
        }
        tc_fence_after();
        if (!leader) continue;
        const uint32_t r0 = str0_r_lo[slot] + ((hh * 4 * 2048) >> 4), r1 = str1_r_lo[slot] + ((hh * 4 * 2048) >> 4);
        if (kDkv) {
#pragma unroll
          for (int k = 0; k < 4; ++k)      // dV += P^T dO
            umma_ts_lohi(tmem_base + kColAcc0, tmem_base + b * 128 + (k >> 1) * 32 + (k & 1) * 8, r1 + ((k * 2048) >> 4),
                         kDescHiSw128, idesc_acc, (u > 0) || (k > 0));
#pragma unroll
          for (int k = 0; k < 4; ++k)      // dK += dS^T Q
            umma_ts_lohi(tmem_base + kColAcc1, tmem_base + b * 128 + 64 + (k >> 1) * 32 + (k & 1) * 8, r0 + ((k * 2048) >> 4),
                         kDescHiSw128, idesc_acc, (u > 0) || (k > 0));
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k)      // dQ += dS K
            umma_ts_lohi(tmem_base + kColAcc0, tmem_base + b * 128 + 64 + (k >> 1) * 32 + (k & 1) * 8, r0 + ((k * 2048) >> 4),
                         kDescHiSw128, idesc_acc, (u > 0) || (k > 0));
        }
        if (hh == 1) umma_commit(bar_o + slot * 8);
      }
      g += n;
      }   // items
      if (ok && g > 0) {
        // the last MMAs (and with them every copy) are complete before the CTA gives up its shared memory
        ok = mbar_wait_warp(bar_o + ((g - 1) & 1) * 8, ((g - 1) >> 1) & 1, abort_flag, kBWaitDrain);
      }
      if (!ok) {
        // let copies still in flight land before the CTA gives up its shared memory
        const unsigned long long t_start = global_timer_ns();
        while (global_timer_ns() - t_start < 2000000ull) {
        }
      }
    }
  } else {
    // ------------------------------------------------- element-wise warps ---
    // Warp w works on TMEM lane quarter w & 3; with eight warps, on 32-column chunk w >> 2 of every
    // half tile (and every other chunk of the epilogue), with four on both chunks.
    constexpr int kChunkStep = kBwdComputeWarps / 4;
    const int quarter = warp & 3, chunk = warp >> 2;
    const int row = quarter * 32 + lane;                    // lane of tensor memory == row of the fixed tile
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    const uint64_t scale_log2_2 = f2_pack(args.scale_log2, args.scale_log2);
    // dQ kernel: log2(scale) rides in the exponent's addend, so the exponential yields P * scale, which is
    // all dS needs.  The dK/dV kernel needs P itself for dV += P^T dO (P * scale in 16 bits would put more
    // of the small probabilities into fp16's subnormal range: dV's error grew by half when that was tried)
    // and multiplies by scale afterwards.
    const uint64_t scale_2 = f2_pack(args.scale, args.scale);
    bool ok = true;
    uint32_t g = 0;                                         // streamed tiles of earlier items
    uint32_t k_item = 0;                                    // earlier items

    for (int number = blockIdx.x; ok && number < n_items; number += gridDim.x, ++k_item) {
    const BwdItem item = bwd_item_decode<kDkv>(args, number, n_tiles, n_q_tiles, n_kv_tiles);
    const int n = item.n, first = item.first, head = item.head, batch = item.batch;
    const int t0 = item.tile * kAttnTile;                   // first key (dkv) / query (dq) of this item
    const int fixed_idx = t0 + row;                         // key index (dkv) / query index (dq)
    const long long row_base = (long long)batch * args.row_stride_b + (long long)head * args.row_stride_h;

    // dq: this thread's query row keeps its own -lse2 / -delta (as packed pairs)
    uint64_t my_nlse2 = 0ull, my_ndelta = 0ull;
    if (!kDkv) {
      const bool valid = fixed_idx < args.len_q;
      const float l2 = valid ? log2f(args.scale) - args.lse[row_base + fixed_idx] * 1.4426950408889634f : -INFINITY;
      const float dl = valid ? -args.delta[row_base + fixed_idx] : 0.f;
      my_nlse2 = f2_pack(l2, l2);
      my_ndelta = f2_pack(dl, dl);
    }

    if (kFixedInTmem) {
      // The fixed tiles (Q and dO of this CTA's query tile; K and V of its key tile): shared memory (128-byte swizzle: the 16-byte unit u of row r
      // sits at unit u ^ (r & 7) of its 128-byte row) -> this thread's lane of tensor memory, in the
      // layout of a 16-bit A operand (two consecutive head dims per column).  (Every MMA that read
      // the previous item's copy completed before this thread left that item's epilogue.)
      ok = __all_sync(0xffffffffu, mbar_wait(bar_fix, k_item & 1, abort_flag, kBWaitFixed));
      if (ok && chunk == 0) {
#pragma unroll
        for (int f = 0; f < 2; ++f) {
          const uint8_t* tile_rows = smem_gen + S::kOffFixed + f * S::kTileBytes + row * 128;
#pragma unroll
          for (int blk = 0; blk < kBlocks; ++blk) {
            uint32_t w[32];
#pragma unroll
            for (int un = 0; un < 8; ++un) {
              const uint4 v4 = *reinterpret_cast<const uint4*>(tile_rows + blk * S::kBlockBytes + ((un ^ (row & 7)) << 4));
              w[4 * un + 0] = v4.x;
              w[4 * un + 1] = v4.y;
              w[4 * un + 2] = v4.z;
              w[4 * un + 3] = v4.w;
            }
            tmem_st32(t_lane + (f == 0 ? kColFixA0 : kColFixA1) + blk * 32, w);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_fixt);
      }
    }

    for (int it = 0; it < n; ++it) {
      const int s0 = (first + it) * kAttnTile;              // first streamed row (query for dkv, key for dq)
      float* rows_lse2 = s_rows + ((g + it) & 1) * 2 * kAttnTile;
      float* rows_delta = rows_lse2 + kAttnTile;
      if (kDkv) {
        // lse2 / delta of the streamed queries: one value per thread, shared through shared memory
        const int qi = s0 + row;
        const bool valid = qi < args.len_q;
        // (stored negated: they enter the arithmetic below as addends, two rows per 64-bit operand)
        if (kChunkStep == 1 || chunk == 0)
          rows_lse2[row] = valid ? -args.lse[row_base + qi] * 1.4426950408889634f : -INFINITY;   // P = 0 beyond len_q
        if (kChunkStep == 1 || chunk == 1) rows_delta[row] = valid ? -args.delta[row_base + qi] : 0.f;
        bwd_rows_sync();
      }
      for (int hh = 0; hh < 2; ++hh) {
        const uint32_t u = 2 * (g + it) + hh;
        const int b = u & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(bar_s + b * 8, (u >> 1) & 1, abort_flag, kBWaitS));
        if (!ok) break;
        tc_fence_after();
        const uint32_t col_s = b * 128, col_dp = b * 128 + 64;
        // Only a tile cut by the diagonal (or by the end of the keys) needs the element-wise mask.
        const bool need_mask = kDkv ? (args.causal && s0 < t0 + kAttnTile)
                                    : (s0 + kAttnTile > args.len_kv || (args.causal && s0 + kAttnTile - 1 > t0));
#pragma unroll
        for (int c = chunk; c < 2; c += kChunkStep) {
          uint32_t sr[32], dp[32];
          tmem_ld32(t_lane + col_s + c * 32, sr);
          tmem_ld32(t_lane + col_dp + c * 32, dp);
          tmem_wait_ld();
          uint32_t pk[16], dk[16];
          // Per pair of streamed rows, in packed fp32 pairs:  P = 2^(s * scale_log2 - lse2),
          // dS = (P * scale) * (dP - delta); in the dQ kernel the exponential gives P * scale
          // directly.  Two copies of the loop, with and without the mask:
          // a branch per pair of rows keeps the compiler from interleaving the pairs' dependency chains.
          auto rows = [&](auto masked_c) {
          constexpr bool kMasked = decltype(masked_c)::value;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int local = hh * 64 + c * 32 + i;           // first of four rows of the streamed tile
            uint64_t nl[2], nd[2];
            if (kDkv) {
              const ulonglong2 l4 = *reinterpret_cast<const ulonglong2*>(rows_lse2 + local);
              const ulonglong2 d4 = *reinterpret_cast<const ulonglong2*>(rows_delta + local);
              nl[0] = l4.x; nl[1] = l4.y;
              nd[0] = d4.x; nd[1] = d4.y;
            } else {
              nl[0] = nl[1] = my_nlse2;
              nd[0] = nd[1] = my_ndelta;
            }
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int j = i + 2 * h2;
              float x0, x1;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[j]), __uint_as_float(sr[j + 1])), scale_log2_2, nl[h2]), x0, x1);
              float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              if (kMasked) {
                const int col = s0 + local + 2 * h2;          // global index of the first of the two rows
                const bool m0 = kDkv ? fixed_idx > col : (col >= args.len_kv || (args.causal && col > fixed_idx));
                const bool m1 = kDkv ? fixed_idx > col + 1 : (col + 1 >= args.len_kv || (args.causal && col + 1 > fixed_idx));
                p0 = m0 ? 0.f : p0;
                p1 = m1 ? 0.f : p1;
              }
              const uint64_t p2 = f2_pack(p0, p1);
              float d0, d1;
              const uint64_t dpd = f2_add(f2_pack(__uint_as_float(dp[j]), __uint_as_float(dp[j + 1])), nd[h2]);
              f2_unpack(f2_mul(kDkv ? f2_mul(p2, scale_2) : p2, dpd), d0, d1);
              pk[j >> 1] = pack2<T>(p0, p1);
              dk[j >> 1] = pack2<T>(d0, d1);
            }
          }
          };
          if (need_mask) rows(std::true_type{}); else rows(std::false_type{});
          // 16-bit P over S and dS over dP, each thread over the start of the 32 fp32 columns it
          // has just read (so the row's other thread is never disturbed): chunk c lands in
          // columns [32c, 32c + 16) of the buffer.
          if (kDkv) tmem_st16(t_lane + col_s + c * 32, pk);
          tmem_st16(t_lane + col_dp + c * 32, dk);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p + b * 8);
      }
      if (!ok) break;
    }

    // ---------------------------------------------------- the item's epilogue --
    if (!ok) break;
    ok = __all_sync(0xffffffffu, mbar_wait(bar_o + ((g + n - 1) & 1) * 8, ((g + n - 1) >> 1) & 1, abort_flag, kBWaitEpi));
    if (!ok) break;
    tc_fence_after();
    {
      auto store_rows = [&](uint32_t col0, void* base, long long sb, long long sh, long long sl, int len) {
        const bool row_valid = fixed_idx < len;
        T* out = reinterpret_cast<T*>(base) + (long long)batch * sb + (long long)head * sh + (long long)fixed_idx * sl;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          if (kChunkStep == 2 && (c & 1) != chunk) continue;      // two threads per row take alternate chunks
          uint32_t acc[32];
          tmem_ld32(t_lane + col0 + c * 32, acc);
          tmem_wait_ld();
          if (row_valid) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o4;
              o4.x = pack2<T>(__uint_as_float(acc[v * 8 + 0]), __uint_as_float(acc[v * 8 + 1]));
              o4.y = pack2<T>(__uint_as_float(acc[v * 8 + 2]), __uint_as_float(acc[v * 8 + 3]));
              o4.z = pack2<T>(__uint_as_float(acc[v * 8 + 4]), __uint_as_float(acc[v * 8 + 5]));
              o4.w = pack2<T>(__uint_as_float(acc[v * 8 + 6]), __uint_as_float(acc[v * 8 + 7]));
              *reinterpret_cast<uint4*>(out + c * 32 + v * 8) = o4;
            }
          }
        }
      };
      if (kDkv) {
        store_rows(kColAcc0, args.dv, args.dv_stride_b, args.dv_stride_h, args.dv_stride_l, args.len_kv);
        store_rows(kColAcc1, args.dk, args.dk_stride_b, args.dk_stride_h, args.dk_stride_l, args.len_kv);
      } else {
        store_rows(kColAcc0, args.dq, args.dq_stride_b, args.dq_stride_h, args.dq_stride_l, args.len_q);
      }
    }
    // the accumulators are free for the next item's first accumulating MMAs
    tc_fence_before();
    mbar_arrive(bar_acc);
    g += n;
    }   // items

    if (kDkv && args.causal && ok) {
      // causal with more keys than queries: key tiles beyond the last query get zero gradients
      const int n_dead = n_kv_tiles - n_tiles;
      for (int idx = blockIdx.x; idx < n_dead * args.heads * args.batch; idx += gridDim.x) {
        const int bh = idx / n_dead;
        const int key = (n_tiles + (idx - bh * n_dead)) * kAttnTile + row;
        const int batch = bh / args.heads, head = bh - batch * args.heads;
        if (key < args.len_kv && chunk == 0) {
          T* dk_row = reinterpret_cast<T*>(args.dk) + (long long)batch * args.dk_stride_b +
                      (long long)head * args.dk_stride_h + (long long)key * args.dk_stride_l;
          T* dv_row = reinterpret_cast<T*>(args.dv) + (long long)batch * args.dv_stride_b +
                      (long long)head * args.dv_stride_h + (long long)key * args.dv_stride_l;
#pragma unroll
          for (int c = 0; c < D / 8; ++c) {
            reinterpret_cast<uint4*>(dk_row)[c] = make_uint4(0u, 0u, 0u, 0u);
            reinterpret_cast<uint4*>(dv_row)[c] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown --
  tc_fence_before();
  __syncthreads();
  if (warp == kBwdComputeWarps) {
    __syncwarp();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

}  // namespace tfb
