// Fused attention forward for sm_100a, two Q tiles per CTA (256 query rows),
// persistent over (head, Q-tile-pair) work items that the CTAs draw from a
// counter at run time (see pair_item_decode).
//
// Same arithmetic as attn_fwd_kernel (attn_fwd_sm100.cuh) and the same place
// in TileFusion's path (include/kernels/flash_attention_device.cuh:130-312);
// the difference is the schedule.  With one Q tile per CTA the tensor pipe and
// the exp unit take turns; here one thread fixes the MMA issue order
//     S0_0 S1_0 | PV0_0 S0_1 | PV1_0 S1_1 | PV0_1 S0_2 | ...
// so that while the tensor pipe works for tile 0 the softmax warps of tile 1
// run, and vice versa.  Roles (384 threads, one CTA per SM):
//   warps 0-3  softmax + epilogue of Q tile 0   (one row per thread)
//   warps 4-7  softmax + epilogue of Q tile 1
//   warp  8    tcgen05.mma issuer (the warp walks the schedule, one elected
//              lane issues), owns the TMEM allocation
//   warp  9    TMA producer and work-item scheduler (one thread)
//   warps 10-11 idle; they complete the third warpgroup so that it can hand
//              its registers to the softmax warpgroups (setmaxnreg)
// TMEM (512 columns): S0 | S1 | O0 | O1, each 128 fp32 columns (O: D columns);
// P overwrites the first 64 columns of its S and is the TMEM A operand of PV.
// Shared memory: Q0, Q1, a ring of three K/V stages (K_0 V_0 K_1 V_1 ...), each
// stage released by a tcgen05.commit after the last MMA that reads it, so both
// Q tiles share every K/V load, and one output staging tile per Q tile: the
// epilogue writes the 16-bit O tile there (swizzled) and one thread sends it
// to global memory with a TMA store.  While an item runs, the producer brings
// the next item's Q tiles and first K/V tiles into L2 if it belongs to another
// head, and the issuer starts the next item's first S tiles during the last
// KV tile of the current one.
//
// The same kernel serves grouped-query decoding in split-KV mode (see
// AttnPairArgs): the query heads of a group are the rows of Q tile 0, an item
// covers a range of KV tiles, and the epilogue writes fp32 partial rows.
#pragma once

#include <type_traits>

#include "attn_fwd_sm100.cuh"

namespace tfb {

constexpr int kPairThreads = 384;     // three warpgroups; warps 10-11 only donate registers
constexpr int kPairRegsSoftmax = 208;
constexpr int kPairRegsIssue = 88;
// setmaxnreg only moves registers between the warpgroups of the CTA: the CTA is
// launched with 168 registers per thread (65536 / 384, rounded down to 8), and a
// raise that does not fit into what the other warpgroups gave up blocks forever.
static_assert(2 * kPairRegsSoftmax + kPairRegsIssue <= 3 * 168, "register split exceeds the CTA's allocation");
constexpr int kPairStages = 3;        // K/V ring of a prefill launch (a deeper ring measured slower)
// In split-KV mode (decoding: K/V stream from HBM, nothing is staged for a TMA
// store) the two output staging tiles, which follow the ring in shared memory,
// serve as two more ring stages.
constexpr int kPairMaxStages = kPairStages + 2;
constexpr int kItemSlots = 4;         // ring of work-item coordinates in shared memory
// Largest sum of 64 values of P published without a look at the row maximum.
constexpr float kPairSumLimit = 4096.0f;

struct AttnPairArgs {
  AttnFwdArgs base;
  int heads;
  int batch;
  int n_pairs;          // ceil(len_q / 256)
  int n_items;          // batch * heads * n_pairs * max(kv_splits, 1)
  int tma_store;        // 1: O leaves through shared memory and a TMA store (map_o is valid)
  int* queue;           // item counter of this launch (zero when the kernel starts)
  int causal_block;     // causal item order: (batch, head) slices per block (see pair_item_decode)
  // Split-KV mode (kv_splits > 0; used for grouped-query decoding, where the
  // "query rows" of a head are the query heads that share one KV head): an item
  // covers KV tiles [split * tiles_per_split, ...), and instead of the final
  // output it writes one partial row per (query row, split): D fp32 of
  // normalised output to part_o and (log2-sum-exp, 1) to part_ml, in the layout
  // decode_combine_kernel reads ([row][split], row = (b * heads + h) * len_q + q).
  int kv_splits;
  int tiles_per_split;
  // kRepl instantiation (split-KV mode with at most 32 query rows per item): the rows are loaded
  // four times, once into every 32-lane quarter of Q tile 0, and the warp of quarter c takes keys
  // [32 c, 32 c + 32) of every KV tile for its copy of the rows; each copy writes a partial row of
  // its own, so a (row, split) has four partial rows: index split * 4 + c of kv_splits * 4.
  float* part_o;
  float* part_ml;
  // Paged KV cache (split-KV mode only; page_size > 0): the K and V tensor maps
  // cover [pages][heads][page_size][D] and a tile's page comes from the table.
  const int* block_table;   // [batch][max_pages]
  int page_size;
  int max_pages;
};

template <int D>
struct AttnPairSmem {
  static constexpr int kTileBytes = kAttnTile * D * 2;
  static constexpr int kBlockBytes = kAttnTile * 128;
  static constexpr int kOffQ = 0;                                   // Q0, Q1
  static constexpr int kOffKV = 2 * kTileBytes;                     // ring
  static constexpr int kOffOut = kOffKV + kPairStages * kTileBytes; // output staging, one tile per Q tile
  static constexpr int kOffBar = kOffOut + 2 * kTileBytes;
  // barrier slots (8 bytes each)
  static constexpr int kBarQFull = 0;      // [2]
  static constexpr int kBarQEmpty = 2;     // [2]
  static constexpr int kBarSFull = 4;      // [2]
  static constexpr int kBarPFull = 6;      // [2]
  static constexpr int kBarOFull = 8;      // [2]
  static constexpr int kBarOEmpty = 10;    // [2]
  static constexpr int kBarPFullHi = 12;   // [2]  second half of P (keys 64..127)
  static constexpr int kBarOutFree = 14;   // [2]  output staging of tile x may be overwritten
  static constexpr int kBarOutFull = 16;   // [2]  all 128 rows of tile x are in the staging buffer
  static constexpr int kBarOLoFull = 18;   // [2]  P.V MMAs of the first half of a tile are complete
  static constexpr int kBarItemFull = 20;   // [kItemSlots]  coordinates of an item are in the item ring
  static constexpr int kBarItemEmpty = 20 + kItemSlots;   // [kItemSlots]  every role has moved past the item
  static constexpr int kBarKVFull = 20 + 2 * kItemSlots;  // [kPairMaxStages]
  static constexpr int kBarKVEmpty = kBarKVFull + kPairMaxStages;
  static constexpr int kNumBars = kBarKVEmpty + kPairMaxStages;
  static constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
  static constexpr int kOffAbort = kOffTmemSlot + 4;
  static constexpr int kOffItems = kOffAbort + 4 + 8;                // kItemSlots x PairItem (16-byte aligned)
  static constexpr int kBytes = kOffItems + kItemSlots * 16 + 1024;  // + slack for 1024-B alignment
};

enum AttnPairWaitCode {
  kPWaitQFull = 301, kPWaitQEmpty = 302, kPWaitKVFull = 303, kPWaitKVEmpty = 304,
  kPWaitSFull = 305, kPWaitPFull = 306, kPWaitOFull = 307, kPWaitOEmpty = 308, kPWaitEpi = 309,
  kPWaitOutFree = 310, kPWaitOutFull = 311, kPWaitItemFull = 312, kPWaitItemEmpty = 313
};

// Work items are handed out at run time: the producer thread of a CTA draws
// item numbers from a counter in global memory (one atomicAdd per item) and
// publishes the decoded coordinates to the other roles of its CTA through a
// small ring in shared memory.  A CTA that runs slower, or that drew heavier
// items, simply draws fewer; and the CTAs running at any moment work on
// neighbouring item numbers.  Non-causal (all items cost the same):
//   number = ((b * heads + h) * n_pairs + pair) * splits + split
// so the tile pairs of one head, which read the same K/V, run at the same time
// and L2 serves all but the first read.  Causal (pair p costs 2p + 2 KV tiles):
// the (batch, head) slices are taken in blocks of `causal_block`; within a
// block all heaviest pairs come first, then the next lighter ones, and so on.
// Heavy items are thus drawn before light ones (a heavy item drawn last would
// run on alone after every other CTA has finished), while the K/V of a block
// stay in L2 from its first level to its last.
struct PairItem {
  int b, h, pair, split;      // b < 0: no more items
};

__device__ __forceinline__ PairItem pair_item_decode(const AttnPairArgs& a, int number) {
  PairItem it;
  if (number >= a.n_items) {
    it.b = -1;
    it.h = it.pair = it.split = 0;
    return it;
  }
  const int splits = a.kv_splits > 0 ? a.kv_splits : 1;
  it.split = number % splits;
  const int rest = number / splits;
  int bh;
  if (a.base.causal) {
    const int n_bh = a.batch * a.heads;
    const int per_block = a.causal_block * a.n_pairs;
    const int block = rest / per_block;
    const int r = rest - block * per_block;
    const int in_block = min(a.causal_block, n_bh - block * a.causal_block);   // the last block may be short
    const int level = r / in_block;
    bh = block * a.causal_block + (r - level * in_block);
    it.pair = a.n_pairs - 1 - level;
  } else {
    bh = rest / a.n_pairs;
    it.pair = rest - bh * a.n_pairs;
  }
  it.b = bh / a.heads;
  it.h = bh - it.b * a.heads;
  return it;
}

// Number of KV tiles visited by Q tile x (rows q0 .. q0+127) of a pair; the
// first one is tile `first` (non-zero only in split-KV mode).
__device__ __forceinline__ int kv_tiles_for(const AttnPairArgs& p, int q0, int split, int& first) {
  const AttnFwdArgs& a = p.base;
  first = 0;
  if (q0 >= a.len_q) return 0;
  int n = (a.len_kv + kAttnTile - 1) / kAttnTile;
  if (a.causal) n = min(n, q0 / kAttnTile + 1);
  if (p.kv_splits > 0) {
    first = split * p.tiles_per_split;
    n = max(0, min(p.tiles_per_split, n - first));
  }
  return n;
}

template <typename T, int D, bool kRepl = false>
__global__ void __launch_bounds__(kPairThreads, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap map_q,
                     const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v,
                     const __grid_constant__ CUtensorMap map_o, const AttnPairArgs pargs) {
  using S = AttnPairSmem<D>;
  const AttnFwdArgs& args = pargs.base;
  constexpr int kIsBf16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr int kTmemCols = 512;
  constexpr int kBlocks = D / 64;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + S::kOffBar;
  auto bar = [&](int slot) -> uint32_t { return bars + slot * 8; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + S::kOffTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + S::kOffAbort);

  const uint32_t n_stages = pargs.kv_splits > 0 ? kPairMaxStages : kPairStages;
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // provably warp-uniform
  const int lane = threadIdx.x & 31;

  // Item ring: the n-th item of this CTA sits in slot n % kItemSlots.
  volatile PairItem* item_ring = reinterpret_cast<volatile PairItem*>(smem_gen + S::kOffItems);
  // (consumer side) waits for the n-th item and reads it; false if the wait gave up
  auto item_get = [&](uint32_t n, PairItem& it) -> bool {
    const uint32_t slot = n % kItemSlots;
    if (!mbar_wait(bar(S::kBarItemFull + slot), (n / kItemSlots) & 1, abort_flag, kPWaitItemFull)) return false;
    it.b = item_ring[slot].b;
    it.h = item_ring[slot].h;
    it.pair = item_ring[slot].pair;
    it.split = item_ring[slot].split;
    return true;
  };

  if (threadIdx.x == 0) {
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar(S::kBarQFull + x), 1);
      mbar_init(bar(S::kBarQEmpty + x), 1);
      mbar_init(bar(S::kBarSFull + x), 1);
      mbar_init(bar(S::kBarPFull + x), 128);
      mbar_init(bar(S::kBarPFullHi + x), 128);
      mbar_init(bar(S::kBarOFull + x), 1);
      mbar_init(bar(S::kBarOLoFull + x), 1);
      mbar_init(bar(S::kBarOEmpty + x), 128);
      mbar_init(bar(S::kBarOutFree + x), 1);
      mbar_init(bar(S::kBarOutFull + x), 128);
    }
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(bar(S::kBarItemFull + s), 1);
      mbar_init(bar(S::kBarItemEmpty + s), 1 + 256);      // the issuer's leader and every softmax thread
    }
    for (int s = 0; s < kPairMaxStages; ++s) {
      mbar_init(bar(S::kBarKVFull + s), 1);
      mbar_init(bar(S::kBarKVEmpty + s), 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc<kTmemCols>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Each role's code sits under the register re-allocation that applies to it.
  if (warp >= 8) {
   setmaxnreg_dec<kPairRegsIssue>();
   if (warp == 9) {
    // ========================================================= TMA producer ==
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      uint32_t stage = 0, phase = 0;      // ring position; phase of the stage's barriers
      uint32_t q_uses[2] = {0, 0};        // loads issued so far into Q buffer x
      bool ok = true;
      // One K (kv = 0) or V (kv = 1) tile of 128 keys starting at key0: loaded
      // into shared memory at dst (signalling `full`), or, with dst == 0, only
      // brought into L2.
      auto kv_tile = [&](int kv, int key0, int b, int h, uint32_t dst, uint32_t full) {
        const bool natural = kv == 0 ? !args.k_mn_major : (args.v_mn_major != 0);
        const CUtensorMap* map = kv == 0 ? &map_k : &map_v;
        if (pargs.page_size > 0) {
          // paged cache (always the row-per-key layout): outer coordinate = page
          if (dst == 0) return;
          const int pg = key0 / pargs.page_size;
          const int page = pargs.block_table[(long long)b * pargs.max_pages + pg];
#pragma unroll
          for (int blk = 0; blk < kBlocks; ++blk)
            tma_load_4d(dst + blk * S::kBlockBytes, map, full, blk * 64, key0 - pg * pargs.page_size, h, page);
        } else if (natural) {
          // rows = keys, 64 head-dim elements per swizzle block
#pragma unroll
          for (int blk = 0; blk < kBlocks; ++blk) {
            if (dst != 0) tma_load_4d(dst + blk * S::kBlockBytes, map, full, blk * 64, key0, h, b);
            else tma_prefetch_l2_4d(map, blk * 64, key0, h, b);
          }
        } else {
          // rows = head dim, 64 keys per swizzle block
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            if (dst != 0) tma_load_4d(dst + blk * (D * 128), map, full, key0 + blk * 64, 0, h, b);
            else tma_prefetch_l2_4d(map, key0 + blk * 64, 0, h, b);
          }
        }
      };
      // Draws the n-th item of this CTA and publishes it (or the end marker).
      auto item_put = [&](uint32_t n, PairItem& it) -> bool {
        const uint32_t slot = n % kItemSlots;
        if (n >= kItemSlots &&
            !mbar_wait(bar(S::kBarItemEmpty + slot), ((n / kItemSlots) - 1) & 1, abort_flag, kPWaitItemEmpty))
          return false;
        it = pair_item_decode(pargs, atomicAdd(pargs.queue, 1));
        item_ring[slot].b = it.b;
        item_ring[slot].h = it.h;
        item_ring[slot].pair = it.pair;
        item_ring[slot].split = it.split;
        mbar_arrive(bar(S::kBarItemFull + slot));          // (release: orders the stores above)
        return true;
      };
      PairItem cur, nxt;
      ok = item_put(0, cur);
      for (uint32_t n_item = 0; ok && cur.b >= 0; ++n_item, cur = nxt) {
        // the next item is drawn before this one's loads start: the MMA issuer
        // looks one item ahead
        ok = item_put(n_item + 1, nxt);
        if (!ok) break;
        const int b = cur.b, h = cur.h, pair = cur.pair, split = cur.split;
        int j0, j0_unused;
        const int q0 = pair * 2 * kAttnTile;
        const int n0 = kv_tiles_for(pargs, q0, split, j0);          // tile 0 always exists; it sets j0
        const int n1 = kv_tiles_for(pargs, q0 + kAttnTile, split, j0_unused);
        const int n = max(n0, n1);
        // Q tile x of this item into its buffer, once the last S MMA of the
        // previous item has read the buffer.
        auto load_q = [&](int x) -> bool {
          if ((x == 0 ? n0 : n1) == 0) return true;
          if (q_uses[x] > 0 &&
              !mbar_wait(bar(S::kBarQEmpty + x), (q_uses[x] - 1) & 1, abort_flag, kPWaitQEmpty))
            return false;
          mbar_arrive_expect_tx(bar(S::kBarQFull + x), S::kTileBytes);
          if constexpr (kRepl) {
            // the same (at most 32) rows into every lane quarter: the tensor map's box is 32 rows high
#pragma unroll
            for (int copy = 0; copy < 4; ++copy)
#pragma unroll
              for (int blk = 0; blk < kBlocks; ++blk)
                tma_load_4d(smem_base + S::kOffQ + x * S::kTileBytes + blk * S::kBlockBytes + copy * 32 * 128, &map_q,
                            bar(S::kBarQFull + x), blk * 64, q0, h, b);
          } else {
#pragma unroll
            for (int blk = 0; blk < kBlocks; ++blk)
              tma_load_4d(smem_base + S::kOffQ + x * S::kTileBytes + blk * S::kBlockBytes, &map_q,
                          bar(S::kBarQFull + x), blk * 64, q0 + x * kAttnTile, h, b);
          }
          ++q_uses[x];
          return true;
        };
        // Order: Q0, the first K tile, Q1, then the rest of the ring.  The MMA
        // issuer starts this item's first S tile of Q tile 0 while Q tile 1 of
        // the previous item is still in its last KV tile, and the buffer of Q1
        // is released later than that of Q0.
        ok = load_q(0);
        // When the next item of this CTA belongs to another head, bring its Q
        // tiles and its first K and V tiles into L2 now, so that the loads at the
        // item boundary (which cannot be issued earlier: the Q buffers and the
        // ring are in use) do not wait for HBM.
        if (pargs.kv_splits == 0 && nxt.b >= 0 && (nxt.b != b || nxt.h != h)) {
          const int b2 = nxt.b, h2 = nxt.h, pair2 = nxt.pair;
          const int q2 = pair2 * 2 * kAttnTile;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            if (q2 + x * kAttnTile >= args.len_q) continue;
#pragma unroll
            for (int blk = 0; blk < kBlocks; ++blk)
              tma_prefetch_l2_4d(&map_q, blk * 64, q2 + x * kAttnTile, h2, b2);
          }
          kv_tile(0, 0, b2, h2, 0, 0);
          kv_tile(1, 0, b2, h2, 0, 0);
        }
        for (int t = 0; ok && t < 2 * n; ++t) {
          const int j = t >> 1, kv = t & 1;
          ok = mbar_wait(bar(S::kBarKVEmpty + stage), phase ^ 1, abort_flag, kPWaitKVEmpty);
          if (!ok) break;
          const uint32_t full = bar(S::kBarKVFull + stage);
          mbar_arrive_expect_tx(full, S::kTileBytes);
          kv_tile(kv, (j0 + j) * kAttnTile, b, h, smem_base + S::kOffKV + stage * S::kTileBytes, full);
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1;
          }
          if (t == 0) ok = load_q(1);
        }
        if (ok && n == 0) ok = load_q(1);
      }
      if (!ok) {
        // let copies still in flight land before the CTA gives up its shared memory
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
      }
    }
   } else if (warp == 8) {
    // =========================================================== MMA issuer ==
    // The whole warp walks the schedule (uniform control flow, uniform
    // operands); one elected lane executes the tcgen05 instructions.
    {
      const bool leader = elect_one();
      const uint32_t idesc_s = make_idesc(128, 128, kIsBf16, 0, args.k_mn_major);
      const uint32_t idesc_o = make_idesc(128, D, kIsBf16, 0, args.v_mn_major);
      uint32_t stage = 0, phase = 0;       // ring position of the next stage to consume
      uint32_t q_cnt[2] = {0, 0};          // Q loads consumed per buffer
      uint32_t p_cnt[2] = {0, 0};          // P tiles consumed per Q tile
      uint32_t items_done[2] = {0, 0};     // epilogues awaited per Q tile
      bool first_s_issued = false;         // the current item's first S tiles were issued during the previous item
      bool ok = true;

      // Operand B addressing, in 16-byte units: MMA step k (16 elements along the
      // contraction) starts at (k >> 2) * step_hi + (k & 3) * step_lo.
      //   K-major  (rows of 64 contraction elements): next 64-element block, 32 B within it
      //   MN-major (one 128-B row per contraction index): 16 rows = 2048 B per step
      const uint32_t k_step_hi = (args.k_mn_major ? 4 * 2048 : S::kBlockBytes) >> 4;
      const uint32_t k_step_lo = (args.k_mn_major ? 2048 : 32) >> 4;
      const uint32_t k_lbo = args.k_mn_major ? D * 128 : 16;
      const uint32_t v_step_hi = (args.v_mn_major ? 4 * 2048 : D * 128) >> 4;
      const uint32_t v_step_lo = (args.v_mn_major ? 2048 : 32) >> 4;
      const uint32_t v_lbo = args.v_mn_major ? S::kBlockBytes : 16;

      auto issue_s = [&](int x, uint32_t k_smem) {
        if (!leader) return;
        const uint32_t a0 = desc_lo(smem_base + S::kOffQ + x * S::kTileBytes, 16);
        const uint32_t b0 = desc_lo(k_smem, k_lbo);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          umma_ss_lohi(tmem_base + x * 128, a0 + (((k >> 2) * S::kBlockBytes + (k & 3) * 32) >> 4),
                       b0 + (k >> 2) * k_step_hi + (k & 3) * k_step_lo, kDescHiSw128, idesc_s, k > 0);
        }
        umma_commit(bar(S::kBarSFull + x));
      };
      // O_x += P_x V for keys [64*half, 64*half + 64) of the tile.
      auto issue_pv_half = [&](int x, int half, uint32_t v_smem, bool accumulate) {
        if (!leader) return;
        const uint32_t b0 = desc_lo(v_smem, v_lbo);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const int k = half * 4 + kk;
          umma_ts_lohi(tmem_base + 256 + x * 128, tmem_base + x * 128 + k * 8,
                       b0 + (k >> 2) * v_step_hi + (k & 3) * v_step_lo, kDescHiSw128, idesc_o,
                       accumulate || (k > 0));
        }
        umma_commit(bar((half == 0 ? S::kBarOLoFull : S::kBarOFull) + x));
      };
      // Waits for the next ring stage and returns its shared-memory address.
      auto next_stage = [&](uint32_t& smem_addr, uint32_t& stage_idx) -> bool {
        if (!mbar_wait_warp(bar(S::kBarKVFull + stage), phase, abort_flag, kPWaitKVFull)) return false;
        smem_addr = smem_base + S::kOffKV + stage * S::kTileBytes;
        stage_idx = stage;
        if (++stage == n_stages) {
          stage = 0;
          phase ^= 1;
        }
        return true;
      };

      PairItem cur, nxt;
      ok = __all_sync(0xffffffffu, item_get(0, cur));
      for (uint32_t n_item = 0; ok && cur.b >= 0; ++n_item, cur = nxt) {
        // (the producer publishes item n + 1 before it loads item n)
        ok = __all_sync(0xffffffffu, item_get(n_item + 1, nxt));
        if (!ok) break;
        if (leader && n_item > 0) mbar_arrive(bar(S::kBarItemEmpty + (n_item - 1) % kItemSlots));
        const int pair = cur.pair, split = cur.split;
        int j0_unused;
        const int q0 = pair * 2 * kAttnTile;
        const int nx[2] = {kv_tiles_for(pargs, q0, split, j0_unused),
                           kv_tiles_for(pargs, q0 + kAttnTile, split, j0_unused)};
        const int n = max(nx[0], nx[1]);
        // The first S tiles of the CTA's next item are issued during the last
        // KV tile of this one (below), so that the tensor pipe and the softmax
        // warps do not drain at the item boundary.  Only when both Q tiles end
        // on the same KV tile: with a causal mask Q tile 0 ends one tile early,
        // and waiting for the next item's operands at that point would hold up
        // the last P.V of Q tile 1 (measured slower).
        int nx2[2] = {0, 0};
        if (nx[0] == nx[1] && nxt.b >= 0) {
          const int pair2 = nxt.pair, split2 = nxt.split;
          nx2[0] = kv_tiles_for(pargs, pair2 * 2 * kAttnTile, split2, j0_unused);
          nx2[1] = kv_tiles_for(pargs, pair2 * 2 * kAttnTile + kAttnTile, split2, j0_unused);
        }
        uint32_t k_smem = 0, k_stage = 0, v_smem = 0, v_stage = 0;
        if (!first_s_issued) {
          // first item of this CTA: both first S tiles back to back
          for (int x = 0; x < 2 && ok; ++x) {
            if (nx[x] == 0) continue;
            ok = mbar_wait_warp(bar(S::kBarQFull + x), q_cnt[x] & 1, abort_flag, kPWaitQFull);
            ++q_cnt[x];
          }
          if (!ok) break;
          ok = next_stage(k_smem, k_stage);
          if (!ok) break;
          tc_fence_after();
          for (int x = 0; x < 2; ++x) {
            if (nx[x] == 0) continue;
            issue_s(x, k_smem);
            if (leader && (nx[x] == 1)) umma_commit(bar(S::kBarQEmpty + x));
          }
          if (leader) umma_commit(bar(S::kBarKVEmpty + k_stage));
        }

        for (int j = 0; ok && j < n; ++j) {
          ok = next_stage(v_smem, v_stage);
          if (!ok) break;
          bool have_k = false;
          for (int x = 0; x < 2 && ok; ++x) {
            if (j < nx[x]) {
              ok = mbar_wait_warp(bar(S::kBarPFull + x), p_cnt[x] & 1, abort_flag, kPWaitPFull);
              if (!ok) break;
              if (j == 0 && items_done[x] > 0) {
                // the previous item's epilogue must have read O_x out of TMEM
                ok = mbar_wait_warp(bar(S::kBarOEmpty + x), (items_done[x] - 1) & 1, abort_flag, kPWaitOEmpty);
                if (!ok) break;
              }
              tc_fence_after();
              issue_pv_half(x, 0, v_smem, j > 0);
              ok = mbar_wait_warp(bar(S::kBarPFullHi + x), p_cnt[x] & 1, abort_flag, kPWaitPFull);
              if (!ok) break;
              ++p_cnt[x];
              tc_fence_after();
              issue_pv_half(x, 1, v_smem, true);
            }
            if (leader && (x == 1)) umma_commit(bar(S::kBarKVEmpty + v_stage));
            if (j + 1 < nx[x]) {
              if (!have_k) {
                ok = next_stage(k_smem, k_stage);
                if (!ok) break;
                have_k = true;
              }
              issue_s(x, k_smem);
              if (leader && (j + 2 == nx[x])) umma_commit(bar(S::kBarQEmpty + x));
            } else if (j + 1 == n && nx2[x] > 0) {
              // first S tile of the next item (its K tile is the next ring stage)
              ok = mbar_wait_warp(bar(S::kBarQFull + x), q_cnt[x] & 1, abort_flag, kPWaitQFull);
              if (!ok) break;
              ++q_cnt[x];
              if (!have_k) {
                ok = next_stage(k_smem, k_stage);
                if (!ok) break;
                have_k = true;
              }
              tc_fence_after();
              issue_s(x, k_smem);
              if (leader && (nx2[x] == 1)) umma_commit(bar(S::kBarQEmpty + x));
            }
            if (leader && (x == 1 && have_k)) umma_commit(bar(S::kBarKVEmpty + k_stage));
          }
        }
        for (int x = 0; x < 2; ++x)
          if (nx[x] > 0) ++items_done[x];
        first_s_issued = n > 0 && nx2[0] > 0;
      }
    }
   }   // warps 10 and 11 only donate registers
  } else {
    setmaxnreg_inc<kPairRegsSoftmax>();
    // ======================================================== softmax warps ==
    const int x = warp >> 2;                                 // which Q tile of the pair
    const int quarter = warp & 3;                            // TMEM lane quarter of this warp
    const int row = quarter * 32 + lane;
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    const uint32_t col_s = x * 128, col_p = x * 128, col_o = 256 + x * 128;
    const uint32_t bar_s = bar(S::kBarSFull + x), bar_p = bar(S::kBarPFull + x);
    const uint32_t bar_p_hi = bar(S::kBarPFullHi + x);
    const uint32_t bar_o = bar(S::kBarOFull + x), bar_oe = bar(S::kBarOEmpty + x);
    const uint32_t bar_o_lo = bar(S::kBarOLoFull + x);
    uint32_t s_cnt = 0;      // S tiles consumed
    uint32_t out_cnt = 0;    // items whose output went through the staging buffer
    uint32_t o_base = 0;     // PV completions of earlier items
    bool ok = true;

    // Second part of an item's epilogue, run for the item in ring slot `slot`:
    // O / l out of TMEM to global memory, then the item's slot is given back.
    float pend_inv_l = 0.f;
    bool have_pending = false;
    auto flush_pending = [&](uint32_t slot) -> bool {
      if (!have_pending) return true;
      have_pending = false;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_o, (o_base - 1) & 1, abort_flag, kPWaitEpi))) return false;
      tc_fence_after();
      // (batch, head and split are read again here rather than kept in registers
      // through the KV loop; the slot is this thread's until it moves on)
      const int b = item_ring[slot].b, h = item_ring[slot].h;
      const int split = item_ring[slot].split;
      const int q0 = item_ring[slot].pair * 2 * kAttnTile + x * kAttnTile;
      const int q_idx = kRepl ? q0 + (row & 31) : q0 + row;
      const float inv_l = pend_inv_l;
      const bool row_valid = q_idx < args.len_q;
      if (pargs.kv_splits > 0) {
        // split-KV mode: one fp32 partial row (normalised O, log2-sum-exp) per split (and row copy)
        const long long prow =
            kRepl ? (((long long)b * pargs.heads + h) * args.len_q + q_idx) * (pargs.kv_splits * 4) + split * 4 + quarter
                  : (((long long)b * pargs.heads + h) * args.len_q + q_idx) * pargs.kv_splits + split;
        float* p_row = pargs.part_o + prow * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orow[32];
          tmem_ld32(t_lane + col_o + c * 32, orow);
          tmem_wait_ld();
          if (c == D / 32 - 1) {
            tc_fence_before();
            mbar_arrive(bar_oe);
          }
          if (row_valid) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<float4*>(p_row + c * 32 + v * 4) =
                  make_float4(__uint_as_float(orow[v * 4 + 0]) * inv_l, __uint_as_float(orow[v * 4 + 1]) * inv_l,
                              __uint_as_float(orow[v * 4 + 2]) * inv_l, __uint_as_float(orow[v * 4 + 3]) * inv_l);
          }
        }
        mbar_arrive(bar(S::kBarItemEmpty + slot));
        return true;
      }
      if (pargs.tma_store) {
        // O leaves through shared memory: each thread writes its row of the
        // 16-bit tile in the 128-byte-swizzle layout of the tensor map (16-byte
        // unit u of row r sits at unit u ^ (r & 7) of its 128-byte line, which
        // also keeps the writes of a warp free of bank conflicts), then one
        // thread issues a TMA store per 64-column block.  Rows past len_q are
        // clipped by the store.
        const uint32_t stage_out = smem_base + S::kOffOut + x * S::kTileBytes;
        if (row == 0) {
          bulk_wait_group_read0();                   // the previous item's store has read the buffer
          mbar_arrive(bar(S::kBarOutFree + x));
        }
        ok = __all_sync(0xffffffffu, mbar_wait(bar(S::kBarOutFree + x), out_cnt & 1, abort_flag, kPWaitOutFree));
        if (!ok) return false;
        // (all of O_x is read with one wait: the S registers are free by now)
        uint32_t orow[D / 32][32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld32(t_lane + col_o + c * 32, orow[c]);
        tmem_wait_ld();
        // O_x has been read out: the next item's first P V may overwrite it
        tc_fence_before();
        mbar_arrive(bar_oe);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          const uint32_t line = stage_out + (c >> 1) * S::kBlockBytes + row * 128;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint32_t w0 = pack2<T>(__uint_as_float(orow[c][v * 8 + 0]) * inv_l, __uint_as_float(orow[c][v * 8 + 1]) * inv_l);
            const uint32_t w1 = pack2<T>(__uint_as_float(orow[c][v * 8 + 2]) * inv_l, __uint_as_float(orow[c][v * 8 + 3]) * inv_l);
            const uint32_t w2 = pack2<T>(__uint_as_float(orow[c][v * 8 + 4]) * inv_l, __uint_as_float(orow[c][v * 8 + 5]) * inv_l);
            const uint32_t w3 = pack2<T>(__uint_as_float(orow[c][v * 8 + 6]) * inv_l, __uint_as_float(orow[c][v * 8 + 7]) * inv_l);
            const uint32_t unit = (uint32_t)((c & 1) * 4 + v) ^ (uint32_t)(row & 7);
            st_shared_v4(line + (unit << 4), w0, w1, w2, w3);
          }
        }
        fence_proxy_async_smem();                    // my writes are visible to the TMA engine
        mbar_arrive(bar(S::kBarOutFull + x));
        if (warp == 4 * x) {
          ok = mbar_wait_warp(bar(S::kBarOutFull + x), out_cnt & 1, abort_flag, kPWaitOutFull);
          if (!ok) return false;
        }
        ++out_cnt;
        if (row == 0) {
#pragma unroll
          for (int blk = 0; blk < kBlocks; ++blk)
            if (blk * 64 < args.dim_v)               // (a block of pure zero padding is not stored)
              tma_store_4d(&map_o, stage_out + blk * S::kBlockBytes, blk * 64, q0, h, b);
          bulk_commit_group();
        }
      } else {
      T* o_row = reinterpret_cast<T*>(args.o) + (long long)b * args.o_stride_b +
                 (long long)h * args.o_stride_h + (long long)q_idx * args.o_stride_l;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orow[32];
        tmem_ld32(t_lane + col_o + c * 32, orow);
        tmem_wait_ld();
        if (c == D / 32 - 1) {
          // O_x has been read out: the next item's first P V may overwrite it
          tc_fence_before();
          mbar_arrive(bar_oe);
        }
        if (row_valid) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (c * 32 + v * 8 >= args.dim_v) continue;      // zero padding of a smaller head dim
            uint4 out;
            out.x = pack2<T>(__uint_as_float(orow[v * 8 + 0]) * inv_l,
                             __uint_as_float(orow[v * 8 + 1]) * inv_l);
            out.y = pack2<T>(__uint_as_float(orow[v * 8 + 2]) * inv_l,
                             __uint_as_float(orow[v * 8 + 3]) * inv_l);
            out.z = pack2<T>(__uint_as_float(orow[v * 8 + 4]) * inv_l,
                             __uint_as_float(orow[v * 8 + 5]) * inv_l);
            out.w = pack2<T>(__uint_as_float(orow[v * 8 + 6]) * inv_l,
                             __uint_as_float(orow[v * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(o_row + c * 32 + v * 8) = out;
          }
        }
      }
      }
      mbar_arrive(bar(S::kBarItemEmpty + slot));
      return true;
    };

    for (uint32_t n_item = 0; ok; ++n_item) {
      PairItem cur;
      ok = __all_sync(0xffffffffu, item_get(n_item, cur));
      if (!ok) break;
      // The slot of the previous item is given back once this thread is done with
      // it: here if nothing of it is pending, else at the end of flush_pending.
      const uint32_t prev_slot = (n_item + kItemSlots - 1) % kItemSlots;
      if (n_item > 0 && !have_pending) mbar_arrive(bar(S::kBarItemEmpty + prev_slot));
      if (cur.b < 0) {
        ok = flush_pending(prev_slot);
        break;
      }
      int j0;
      const int q0 = cur.pair * 2 * kAttnTile + x * kAttnTile;
      const int n_kv = kv_tiles_for(pargs, q0, cur.split, j0);
      if (n_kv == 0) {
        ok = flush_pending(prev_slot);
        continue;
      }
      const int q_idx = kRepl ? q0 + (row & 31) : q0 + row;
      float m_used = -INFINITY;
      float l_run = 0.f;

      for (int j = 0; j < n_kv; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_s, s_cnt & 1, abort_flag, kPWaitSFull));
        if (!ok) break;
        ++s_cnt;
        tc_fence_after();

        if constexpr (kRepl) {
          // This warp's 32 keys of the tile for its copy of the rows; the other 96 keys of P are
          // zero in this copy, so the P.V MMAs add nothing for them.
          const int key0 = (j0 + j) * kAttnTile + quarter * 32;
          uint32_t s1[32];
          tmem_ld32(t_lane + col_s + quarter * 32, s1);
          tmem_wait_ld();
          if (key0 + 32 > args.len_kv) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (key0 + i >= args.len_kv) s1[i] = 0xff800000u;  // -inf
          }
          auto chunk_max = [&]() -> float {
            float ma = max3(__uint_as_float(s1[0]), __uint_as_float(s1[1]), __uint_as_float(s1[2]));
            float mb = max3(__uint_as_float(s1[3]), __uint_as_float(s1[4]), __uint_as_float(s1[5]));
#pragma unroll
            for (int i = 6; i + 3 < 32; i += 4) {
              ma = max3(ma, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
              mb = max3(mb, __uint_as_float(s1[i + 2]), __uint_as_float(s1[i + 3]));
            }
            return max3(ma, mb, fmaxf(__uint_as_float(s1[30]), __uint_as_float(s1[31])));
          };
          // Nothing has been accumulated under a maximum of -inf (every key so far was masked), so
          // the first finite maximum is taken over without a rescale.
          if (m_used == -INFINITY) m_used = chunk_max();
          uint32_t pk[16];
          float sum = 0.f;
          auto probs = [&]() {
            const float nm = -m_used * args.scale_log2;
            sum = 0.f;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              // (m_used = -inf only if every key of this chunk is masked as well: P = 0)
              const float p0 = m_used == -INFINITY ? 0.f : fast_exp2(fmaf(__uint_as_float(s1[i]), args.scale_log2, nm));
              const float p1 = m_used == -INFINITY ? 0.f : fast_exp2(fmaf(__uint_as_float(s1[i + 1]), args.scale_log2, nm));
              sum += p0 + p1;
              pk[i >> 1] = pack2<T>(p0, p1);
            }
          };
          probs();
          if (__any_sync(0xffffffffu, !(sum <= kPairSumLimit))) {
            // the maximum in use is stale by more than the limit allows: rescale what has been
            // accumulated (O only once the previous tile's P.V is complete) and compute again
            const float m_new = fmaxf(m_used, chunk_max());
            const float alpha = fast_exp2((m_used - m_new) * args.scale_log2);
            m_used = m_new;
            l_run *= alpha;
            if (j > 0) {
              ok = __all_sync(0xffffffffu, mbar_wait(bar_o, (o_base + j - 1) & 1, abort_flag, kPWaitOFull));
              if (!ok) break;
              tc_fence_after();
#pragma unroll
              for (int c = 0; c < D / 16; ++c) {
                uint32_t orow[16];
                tmem_ld16(t_lane + col_o + c * 16, orow);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                tmem_st16(t_lane + col_o + c * 16, orow);
              }
            }
            probs();
          }
          uint32_t zeros[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) zeros[i] = 0u;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c == quarter) tmem_st16(t_lane + col_p + c * 16, pk);
            else tmem_st16(t_lane + col_p + c * 16, zeros);
          }
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar_p);
          mbar_arrive(bar_p_hi);
          l_run += sum;
          if (j == 0) {
            ok = flush_pending(prev_slot);
            if (!ok) break;
          }
          continue;
        }

        // Load the whole S row (four 32-column chunks) into registers.
        const int kv0 = (j0 + j) * kAttnTile;
        const bool need_mask =
            (kv0 + kAttnTile > args.len_kv) || (args.causal && (kv0 + kAttnTile - 1 > q0));
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(t_lane + col_s + c * 32, sr[c]);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = kv0 + c * 32 + i;
              const bool masked = (col >= args.len_kv) || (args.causal && col > q_idx);
              if (masked) sr[c][i] = 0xff800000u;  // -inf
            }
          }
        }
        // Row maximum over chunks [c0, c1): two independent chains per chunk in
        // one straight line of code, so that the 3-input max instructions pipeline.
        auto row_max = [&](int c0, int c1) -> float {
          float ma[4], mb[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c < c0 || c >= c1) continue;
            ma[c] = max3(__uint_as_float(sr[c][0]), __uint_as_float(sr[c][1]), __uint_as_float(sr[c][2]));
            mb[c] = max3(__uint_as_float(sr[c][3]), __uint_as_float(sr[c][4]), __uint_as_float(sr[c][5]));
          }
#pragma unroll
          for (int i = 6; i + 3 < 32; i += 4) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              if (c < c0 || c >= c1) continue;
              ma[c] = max3(ma[c], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
              mb[c] = max3(mb[c], __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
            }
          }
          float m = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c < c0 || c >= c1) continue;
            m = fmaxf(m, max3(ma[c], mb[c], fmaxf(__uint_as_float(sr[c][30]), __uint_as_float(sr[c][31]))));
          }
          return m;
        };
        // Raises the maximum in use to at least m_seen and rescales what has been
        // accumulated under the old one: the running sum, `extra` (a partial sum
        // of this tile) and, once the P.V MMAs counted by `o_parity` on `o_bar`
        // are complete, O in TMEM.
        auto raise_max = [&](float m_seen, float& extra, bool rescale_o, uint32_t o_bar, uint32_t o_parity,
                             int code) -> bool {
          const float m_new = fmaxf(m_used, m_seen);
          const float alpha = fast_exp2((m_used - m_new) * args.scale_log2);
          m_used = m_new;
          l_run *= alpha;
          extra *= alpha;
          if (!rescale_o) return true;
          if (!__all_sync(0xffffffffu, mbar_wait(o_bar, o_parity, abort_flag, code))) return false;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            uint32_t orow[16];
            tmem_ld16(t_lane + col_o + c * 16, orow);
            tmem_wait_ld();
            const uint64_t alpha2 = f2_pack(alpha, alpha);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float lo, hi;
              f2_unpack(f2_mul(f2_pack(__uint_as_float(orow[i]), __uint_as_float(orow[i + 1])), alpha2), lo, hi);
              orow[i] = __float_as_uint(lo);
              orow[i + 1] = __float_as_uint(hi);
            }
            tmem_st16(t_lane + col_o + c * 16, orow);
          }
          return true;
        };
        // P = 2^(s*scale - m) for 64 keys (chunks 2*half, 2*half + 1), written as 16-bit over the
        // start of S; returns their sum.  Head dim 128: every exponential on the MUFU (an FMA-pipe
        // polynomial for 1, 2 or 3 of every 8 pairs measured 3-5 % slower).  Head dim 64, where a
        // step has half the tensor work under the same exponentials: 2 of every 8 pairs on the
        // FMA pipe measured 2 % faster (3 of 8 even, 4 of 8 4 % slower).
        constexpr int kPolyPairsOf8 = D == 64 ? 2 : 0;
        const uint64_t scale2 = f2_pack(args.scale_log2, args.scale_log2);
        auto p_half = [&](int half) -> float {
          const float m_scaled = m_used * args.scale_log2;
          const uint64_t negm2 = f2_pack(-m_scaled, -m_scaled);
          uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};    // four packed (even, odd) partial sums
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int c = 2 * half + cc;
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), scale2, negm2),
                        x0, x1);
              float p0, p1;
              if constexpr (kPolyPairsOf8 > 0) {
                if (((i >> 1) & 7) < kPolyPairsOf8) {
                  poly_exp2_x2(x0, x1, p0, p1);
                } else {
                  p0 = fast_exp2(x0);
                  p1 = fast_exp2(x1);
                }
              } else {
                p0 = fast_exp2(x0);
                p1 = fast_exp2(x1);
              }
              ls2[(i >> 1) & 3] = f2_add(ls2[(i >> 1) & 3], f2_pack(p0, p1));
              pk[i >> 1] = pack2<T>(p0, p1);
            }
            tmem_st16(t_lane + col_p + c * 16, pk);
          }
          float lo, hi;
          f2_unpack(f2_add(f2_add(ls2[0], ls2[1]), f2_add(ls2[2], ls2[3])), lo, hi);
          return lo + hi;
        };

        // The first tile of an item takes its row maximum before anything else.
        // Later tiles skip that pass: they compute P under the maximum in use and
        // look at the sum of each half before publishing it.  Every P is >= 0, so
        // a sum within kPairSumLimit bounds each of them (far below the 16-bit
        // overflow), and O and the running sum stay exact after the final 1/l
        // whatever maximum was in use.  A larger sum (or a NaN) means the
        // maximum in use is stale by more than the limit allows: only then is the
        // half's true maximum taken, the accumulated state rescaled and the half
        // computed again.  Nothing is published before its sum has passed.
        float no_extra = 0.f;
        if (j == 0) {
          ok = raise_max(row_max(0, 4), no_extra, false, 0, 0, 0);
        }
        float lo_sum = p_half(0);
        if (j > 0 && __any_sync(0xffffffffu, !(lo_sum <= kPairSumLimit))) {
          ok = raise_max(row_max(0, 4), no_extra, true, bar_o, (o_base + j - 1) & 1, kPWaitOFull);
          if (!ok) break;
          tmem_wait_st();            // the discarded half must not land after the new one
          lo_sum = p_half(0);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p);
        float hi_sum = p_half(1);
        if (j > 0 && __any_sync(0xffffffffu, !(hi_sum <= kPairSumLimit))) {
          // P.V of the first half (this tile) is in flight or done: wait for it,
          // then O holds everything accumulated so far and nothing else touches it
          // until the second half is published.
          ok = raise_max(row_max(2, 4), lo_sum, true, bar_o_lo, (o_base + j) & 1, kPWaitOFull);
          if (!ok) break;
          tmem_wait_st();
          hi_sum = p_half(1);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_hi);
        l_run += lo_sum + hi_sum;
        if (j == 0) {
          // the previous item's O can leave now: its last P.V has had a whole
          // tile's time to finish, and this item's first P.V waits for it
          ok = flush_pending(prev_slot);
          if (!ok) break;
        }
      }
      if (!ok) break;

      // ------------------------------------------------------ end of the item --
      // The log-sum-exp outputs are final now.  Reading O out of TMEM has to wait
      // for the last P.V MMAs; that part is deferred until this thread has
      // published the first tile of its next item (see flush_pending), so that it
      // does not sit idle meanwhile.
      {
        const int b = item_ring[n_item % kItemSlots].b, h = item_ring[n_item % kItemSlots].h;
        const int split = item_ring[n_item % kItemSlots].split;
        if (q_idx < args.len_q) {
          if (pargs.kv_splits > 0) {
            const long long prow =
                kRepl ? (((long long)b * pargs.heads + h) * args.len_q + q_idx) * (pargs.kv_splits * 4) + split * 4 + quarter
                      : (((long long)b * pargs.heads + h) * args.len_q + q_idx) * pargs.kv_splits + split;
            // (a row copy that saw no key at all: l = 0, m = -inf, which the combine gives weight 0)
            pargs.part_ml[prow * 2 + 0] = l_run > 0.f ? m_used * args.scale_log2 + log2f(l_run) : -INFINITY;
            pargs.part_ml[prow * 2 + 1] = 1.0f;
          } else if (args.lse != nullptr) {
            args.lse[(long long)b * args.lse_stride_b + (long long)h * args.lse_stride_h + q_idx] =
                0.6931471805599453f * (m_used * args.scale_log2 + log2f(l_run));
          }
        }
      }
      pend_inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
      have_pending = true;
      o_base += n_kv;
    }
  }

  // ---------------------------------------------------------------- teardown --
  // (threads that issued TMA stores wait for them; a no-op for the others)
  bulk_wait_group0();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

}  // namespace tfb
