// Flash decoding for sm_100a: one query row per (batch, head) against a long
// KV sequence, as split-KV partials followed by a log-sum-exp combine.
// TileFusion has no decode operator; these kernels extend its attention path
// (include/kernels/flash_attention_device.cuh:130-312 walks the whole KV
// length in one CTA) with the split the long-KV case needs.
//
// decode_split_kernel is bound by HBM bandwidth (about one flop per byte), so
// it is organised around the K/V byte stream:
//   * a persistent grid, two CTAs per SM; each work item is one (b, h, split)
//     and covers one or more kv_chunk-sized chunks of that head;
//   * one producer thread streams K then V of each chunk through a ring of
//     32-KB shared-memory stages with 1-D bulk TMA copies (evict-first in L2)
//     that complete on "full" mbarriers; eight consumer warps release stages
//     through "empty" mbarriers, so ~192 KB per SM stay in flight;
//   * consumers keep q (pre-multiplied by scale*log2 e) in registers; a group
//     of D/8 lanes reads one 16-byte-vectorised key row, partial dot products
//     are reduced with a transposing shuffle butterfly (one shuffle per key);
//   * softmax is per chunk with a running (m, l) across the chunks of a split;
//     P.V accumulates 8 output dims per lane in fp32 and is reduced across the
//     key groups once per work item.
// Each item writes D fp32 of un-normalised output plus (m, l), m in log2 units.
//
// decode_combine_kernel merges n partial rows per (b, h): it either writes the
// final O (16-bit) and LSE (natural log), or one merged partial row (used when
// the KV sequence is sharded across GPUs and the merge continues after an
// all-gather).
//
// KV sharded across GPUs: with DecodeFuseArgs set, decode_split_kernel carries
// the exchange itself.  A tenth warp (the "merger") of every CTA publishes the
// CTA's finished items: one flag word per item receives the step number, after
// a device-scope fence that covers every item signalled so far.  The CTA that
// runs the LAST split of a (b, h) owns that row's merge: its merger polls the
// row's flag words, merges the partials once all carry the step number, and
// stores the merged (O, m, l) row straight into the gather area of every rank
// through peer-mapped pointers; the merger that completes the rank's last row
// raises this rank's flag on every peer; and the CTAs then wait (bounded) for
// all ranks' flags and write the final O / LSE for their rows -- split,
// all-gather and combine in one launch.  The consumers only signal "item
// written" on an mbarrier and go on streaming.  (Counting arrivals per row with
// atomics instead costs tens of microseconds per item: the CTAs of a persistent
// grid work on the same one or two rows at any moment, so all of them hit the
// same counter at once.)  Only plain peer stores and system-scope
// release/acquire touch peer memory.
//
// 8-bit K/V (OCP e4m3 / e5m2 storage, the types TileFusion declares in
// include/types/base.hpp:13-39 and only converts, tests/cpp/types/test_fp8.cu):
// the KV template parameter selects the stored element.  The byte stream per key
// halves, a lane still reads 16 bytes of a row (16 head dims instead of 8), a
// stage keeps its size and holds 256 keys instead of 128 (so the per-stage
// barrier and shuffle work is spread over as many bytes as before), and the
// elements are widened e4m3/e5m2 -> f16x2 -> fp32 in registers; q, the scores,
// the softmax and the accumulators stay fp32.  Per-tensor dequantisation factors fold into
// the score scale (K) and into the partial row as it is written (V).
#pragma once

#include <cuda_fp8.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace tfb {

constexpr int kDecStageRows = 128;        // keys of a 16-bit cache per stage; an 8-bit cache takes twice as many
                                          // (one stage is 256 * D bytes either way); also the paging granule
constexpr int kDecConsumerThreads = 256;
constexpr int kDecThreads = kDecConsumerThreads + 64;   // + producer warp + merger warp
constexpr int kDecDoneSlots = 8;                        // items the consumers may be ahead of the merger
constexpr int kDecMaxChunk = 1024;        // keys; bounds the score buffers

// Fused merge / exchange / final combine of a KV-sharded decode step (all
// fields zero: the split pass only writes its partial rows).
struct DecodeFuseArgs {
  unsigned* item_flags;       // [items]: item i's partial row is in global memory once its word == step
                              // (words only grow from step to step; null = no fused tail)
  unsigned* rows_done;        // one word, zero between steps: merged rows of this rank
  int rows;                   // batch * heads
  // Destination of the merged rows: every peer's gather area (peer_bases[p] +
  // slot_offset floats; rows*D of O, then rows*2 of (m, l)), or out_slot alone.
  float* const* peer_bases;   // device array [n_peers], or null
  float* out_slot;
  int n_peers;
  int my_rank;
  long long slot_offset;
  long long flag_offset;      // floats from a peer base to its flag words (one per sender)
  unsigned step;              // value the flags receive; grows by one per step
  // Final phase (p2p only): wait for all senders' flags, then combine the
  // n_peers gathered rows of each (b,h) into O / LSE.
  int final_phase;
  const float* local_area;    // this rank's current gather area: [n_peers][rows*(D+2)]
  const unsigned* local_flags;
  void* o;
  long long o_stride_b, o_stride_h;
  float* lse;                 // [rows] or null
};

// Tags for 8-bit K/V storage (the KV template parameter; a 16-bit cache passes T).
struct Fp8E4M3 {};
struct Fp8E5M2 {};

template <typename KV>
struct KvBytes {
  static constexpr int value = 2;
};
template <>
struct KvBytes<Fp8E4M3> {
  static constexpr int value = 1;
};
template <>
struct KvBytes<Fp8E5M2> {
  static constexpr int value = 1;
};

// The 16 bytes a lane reads from a key or value row, widened to fp32: 8 elements
// of a 16-bit cache, 16 of an 8-bit one.
template <typename KV>
__device__ __forceinline__ void unpack_row16(const uint4 v, float (&out)[16 / KvBytes<KV>::value]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if constexpr (KvBytes<KV>::value == 2) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack2<KV>(w[e]);
      out[2 * e] = f.x;
      out[2 * e + 1] = f.y;
    }
  } else {
    constexpr __nv_fp8_interpretation_t kKind = std::is_same<KV, Fp8E4M3>::value ? __NV_E4M3 : __NV_E5M2;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __half2 lo(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[e] & 0xffffu), kKind));
      const __half2 hi(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[e] >> 16), kKind));
      const float2 a = __half22float2(lo), b = __half22float2(hi);
      out[4 * e] = a.x;
      out[4 * e + 1] = a.y;
      out[4 * e + 2] = b.x;
      out[4 * e + 3] = b.y;
    }
  }
}

struct DecodeSplitArgs {
  const void* q;
  const void* k;
  const void* v;
  float* part_o;      // [items][D]
  float* part_ml;     // [items][2]
  int heads;          // query heads
  int group;          // query heads per KV head: head h reads K/V head h / group
  int len_kv;
  int kv_chunk;
  int num_splits;
  int chunks_per_split;
  int items;          // B*H*num_splits
  float scale_log2;   // softmax_scale * log2(e) * the keys' dequantisation factor
  float v_scale;      // the values' dequantisation factor (1 for a 16-bit cache)
  long long q_stride_b, q_stride_h;
  long long k_stride_b, k_stride_h;
  long long v_stride_b, v_stride_h;
  // paged KV cache (page_size > 0): K/V are [pages][heads][page_size][D]
  const int* block_table;   // [batch][max_pages]
  int page_size;
  int max_pages;
  long long k_stride_page, v_stride_page;
  DecodeFuseArgs fuse;
};

template <int D, int kStages, int kKvBytes = 2>
struct DecodeSmem {
  static constexpr int kKeysPerStage = kDecStageRows * 2 / kKvBytes;
  static constexpr int kStageBytes = kKeysPerStage * D * kKvBytes;
  static constexpr int kOffStages = 0;
  static constexpr int kOffScores = kStages * kStageBytes;              // 2 x kDecMaxChunk fp32
  static constexpr int kOffRed = kOffScores + 2 * kDecMaxChunk * 4;     // [consumer warps][D] fp32
  static constexpr int kOffWarp = kOffRed + (kDecConsumerThreads / 32) * D * 4;   // 16 fp32 scratch
  static constexpr int kOffBar = kOffWarp + 64;                         // 2*kStages mbarriers
  static constexpr int kOffDone = kOffBar + 2 * kStages * 8;            // kDecDoneSlots "item written" + as many "slot free" mbarriers
  static constexpr int kOffAbort = kOffDone + 2 * kDecDoneSlots * 8;    // abort flag, then the gave-up flag of the final phase
  static constexpr int kBytes = kOffAbort + 16 + 128;                   // + alignment slack
};

enum DecodeWaitCode {
  kWaitDecEmpty = 201, kWaitDecFullK = 202, kWaitDecFullV = 203, kWaitDecDone = 204, kWaitDecFree = 205, kWaitDecRow = 206
};
enum CombineWaitCode { kWaitGatherFlag = 401 };

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until the flag word has reached `step` (flags only grow).  False
// when the wait gave up; the status word then holds kWaitGatherFlag.
__device__ __forceinline__ bool wait_gather_flag(const unsigned* flag, unsigned step) {
  const unsigned long long t0 = global_timer_ns();
  while ((int)(ld_acquire_sys(flag) - step) < 0) {
    if (global_timer_ns() - t0 > wait_limit_ns()) {
      report_wait_timeout((int)kWaitGatherFlag);
      return false;
    }
  }
  return true;
}

template <typename T>
__device__ __forceinline__ T to_out(float v);
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kDecConsumerThreads) : "memory");
}

template <typename T, typename KV, int D, int kStages>
__global__ void __launch_bounds__(kDecThreads, 2) decode_split_kernel(const DecodeSplitArgs args) {
  constexpr int kKvBytes = KvBytes<KV>::value;
  using S = DecodeSmem<D, kStages, kKvBytes>;
  constexpr int kRowBytes = D * kKvBytes;              // one key or value row
  constexpr int kEpl = 16 / kKvBytes;                  // head dims per lane (16 B of a row)
  constexpr int kLpr = D / kEpl;                       // lanes per key row
  constexpr int kGroups = kDecConsumerThreads / kLpr;  // key rows read per step
  constexpr int kKps = S::kKeysPerStage;               // keys per stage
  constexpr int kKpt = kKps / kGroups;                 // keys per thread per stage
  static_assert(kKpt == 8 || kKpt == 4 || kKpt == 2, "unexpected keys per thread");

  static_assert(kLpr >= kKpt, "butterfly needs at least kKpt lanes per row");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  float* scores = reinterpret_cast<float*>(smem_gen + S::kOffScores);
  float* red = reinterpret_cast<float*>(smem_gen + S::kOffRed);
  float* warp_scratch = reinterpret_cast<float*>(smem_gen + S::kOffWarp);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + S::kOffAbort);
  volatile int* s_gave_up = abort_flag + 1;    // the wait for the peers' flags ran out
  const uint32_t bar_full = smem_base + S::kOffBar;
  const uint32_t bar_empty = smem_base + S::kOffBar + kStages * 8;
  const uint32_t bar_done = smem_base + S::kOffDone;                      // [kDecDoneSlots] item n is in global memory
  const uint32_t bar_free = smem_base + S::kOffDone + kDecDoneSlots * 8;  // [kDecDoneSlots] the merger has taken item n
  const bool fused = args.fuse.item_flags != nullptr;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, kDecConsumerThreads / 32);
    }
    for (int s = 0; s < kDecDoneSlots; ++s) {
      mbar_init(bar_done + s * 8, kDecConsumerThreads / 32);
      mbar_init(bar_free + s * 8, 1);
    }
    *abort_flag = 0;
    *s_gave_up = 0;
    mbar_fence_init();
  }
  __syncthreads();

  const int chunk = args.kv_chunk;
  const int keys_per_split = chunk * args.chunks_per_split;

  if (warp == kDecConsumerThreads / 32 + 1) {
    // -------------------------------------------------------------- merger --
    // Publishes this CTA's finished items (flag word = step), merges the rows
    // whose last split this CTA runs, and sends them out.
    if (fused) {
      const DecodeFuseArgs& f = args.fuse;
      constexpr int kVec = D / 32;                     // output dims per lane
      constexpr int kMaxPending = 8;
      int pending[kMaxPending];                        // rows this CTA has to merge, oldest first
      int n_pending = 0;
      unsigned long long pending_since = 0;
      bool ok = true;
      uint32_t n = 0;                                  // items of this CTA published so far
      int item = blockIdx.x;

      // Publishes every item the consumers have signalled (at least one if `must`).
      auto publish = [&](bool must) -> bool {
        if (item >= args.items || n_pending >= kMaxPending) return true;
        if (must) {
          if (!mbar_wait_warp(bar_done + (n % kDecDoneSlots) * 8, (n / kDecDoneSlots) & 1, abort_flag, kWaitDecDone))
            return false;
        } else if (!__all_sync(0xffffffffu, mbar_try_wait(bar_done + (n % kDecDoneSlots) * 8, (n / kDecDoneSlots) & 1))) {
          return true;
        }
        int batch = 1;
        while (batch < kDecDoneSlots && item + batch * (int)gridDim.x < args.items && n_pending + batch < kMaxPending &&
               __all_sync(0xffffffffu, mbar_try_wait(bar_done + ((n + batch) % kDecDoneSlots) * 8,
                                                     ((n + batch) / kDecDoneSlots) & 1)))
          ++batch;
        if (lane == 0)
          for (int i = 0; i < batch; ++i) mbar_arrive(bar_free + ((n + i) % kDecDoneSlots) * 8);
        __threadfence();                               // the consumers' partial rows, before their flags
        for (int i = 0; i < batch; ++i, item += gridDim.x) {
          if (lane == 0) *reinterpret_cast<volatile unsigned*>(f.item_flags + item) = f.step;
          const int bh = item / args.num_splits;
          if (item - bh * args.num_splits == args.num_splits - 1) {      // the row's last split: the merge is ours
            if (n_pending == 0) pending_since = global_timer_ns();
            pending[n_pending++] = bh;
          }
        }
        n += batch;
        return true;
      };

      while (ok && (item < args.items || n_pending > 0)) {
        ok = publish(n_pending == 0);
        if (!ok || n_pending == 0) continue;
        // ---- is the oldest pending row complete? (flags written by other SMs: read past L1) ----
        const int bh = pending[0];
        const unsigned* flags = f.item_flags + (long long)bh * args.num_splits;
        bool all_in = true;
        for (int p = lane; p < args.num_splits; p += 32) all_in = all_in && (__ldcg(flags + p) == f.step);
        if (!__all_sync(0xffffffffu, all_in)) {
          if (global_timer_ns() - pending_since > wait_limit_ns()) {
            if (lane == 0) {
              *abort_flag = kWaitDecRow;
              report_wait_timeout(kWaitDecRow);
            }
            ok = false;
          }
          if (n_pending == kMaxPending || item >= args.items) __nanosleep(200);
          continue;
        }
        __threadfence();                               // (acquire side: the partial rows behind the flags)
        // ---- merge the splits of row bh ----
        const float* ml = args.part_ml + (long long)bh * args.num_splits * 2;
        const float* po = args.part_o + (long long)bh * args.num_splits * D + lane * kVec;
        float m = -INFINITY;
        for (int p = lane; p < args.num_splits; p += 32) m = fmaxf(m, __ldcg(ml + 2 * p));
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float acc_o[kVec], l = 0.f;
#pragma unroll
        for (int e = 0; e < kVec; ++e) acc_o[e] = 0.f;
        for (int p0 = 0; p0 < args.num_splits; p0 += 8) {
          // eight splits at a time: their loads are in flight together
          float2 mlp[8];
          float x[8][kVec];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int p = min(p0 + u, args.num_splits - 1);
            mlp[u] = __ldcg(reinterpret_cast<const float2*>(ml + 2 * p));
            if constexpr (kVec == 4) {
              const float4 t = __ldcg(reinterpret_cast<const float4*>(po + (long long)p * D));
              x[u][0] = t.x; x[u][1] = t.y; x[u][2] = t.z; x[u][3] = t.w;
            } else {
              const float2 t = __ldcg(reinterpret_cast<const float2*>(po + (long long)p * D));
              x[u][0] = t.x; x[u][1] = t.y;
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float w = (p0 + u >= args.num_splits || mlp[u].x == -INFINITY) ? 0.f : fast_exp2(mlp[u].x - m);
            l = fmaf(mlp[u].y, w, l);
#pragma unroll
            for (int e = 0; e < kVec; ++e) acc_o[e] = fmaf(x[u][e], w, acc_o[e]);
          }
          if ((p0 & 63) == 56) ok = ok && publish(false);      // keep the consumers' slots moving during a long merge
        }
        const int n_dst = f.peer_bases != nullptr ? f.n_peers : 1;
        for (int p = 0; p < n_dst; ++p) {
          float* base = f.peer_bases != nullptr ? f.peer_bases[p] + f.slot_offset : f.out_slot;
          float* dst = base + (long long)bh * D + lane * kVec;
          if constexpr (kVec == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(acc_o[0], acc_o[1], acc_o[2], acc_o[3]);
          } else {
            *reinterpret_cast<float2*>(dst) = make_float2(acc_o[0], acc_o[1]);
          }
          if (lane == 0)
            *reinterpret_cast<float2*>(base + (long long)f.rows * D + (long long)bh * 2) = make_float2(m, l);
        }
        __threadfence_system();                        // my peer stores are performed before the row is counted
        __syncwarp();
        if (lane == 0 && atomicAdd(f.rows_done, 1u) == (unsigned)f.rows - 1u) {
          // the rank's last row: re-arm the counter and raise this rank's flag everywhere
          *f.rows_done = 0;
          __threadfence_system();
          if (f.peer_bases != nullptr)
            for (int p = 0; p < f.n_peers; ++p)
              st_release_sys(reinterpret_cast<unsigned*>(f.peer_bases[p] + f.flag_offset) + f.my_rank, f.step);
        }
        // pop the row
        for (int i = 1; i < n_pending; ++i) pending[i - 1] = pending[i];
        --n_pending;
        pending_since = global_timer_ns();
      }
    }
  } else if (warp == kDecConsumerThreads / 32) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      const uint64_t policy = l2_policy_evict_first();
      uint32_t stage = 0, phase = 0;
      int issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < args.items; item += gridDim.x) {
        const int bh = item / args.num_splits;
        const int split = item - bh * args.num_splits;
        const int b = bh / args.heads, h = bh - b * args.heads;
        const bool paged = args.page_size > 0;
        // byte addresses: strides count elements of the stored type
        const int hk = h / args.group;                      // the KV head this query head reads
        const uint8_t* kbase = reinterpret_cast<const uint8_t*>(args.k) +
                               ((paged ? 0 : b * args.k_stride_b) + hk * args.k_stride_h) * kKvBytes;
        const uint8_t* vbase = reinterpret_cast<const uint8_t*>(args.v) +
                               ((paged ? 0 : b * args.v_stride_b) + hk * args.v_stride_h) * kKvBytes;
        const int* pages = paged ? args.block_table + (long long)b * args.max_pages : nullptr;
        const int key_begin = split * keys_per_split;
        const int key_end = min(args.len_kv, key_begin + keys_per_split);
        for (int c0 = key_begin; ok && c0 < key_end; c0 += chunk) {
          const int c1 = min(key_end, c0 + chunk);
          for (int pass = 0; ok && pass < 2; ++pass) {
            const uint8_t* base = pass == 0 ? kbase : vbase;
            for (int s0 = c0; s0 < c1; s0 += kKps) {
              const int n = min(kKps, c1 - s0);
              if (issued >= kStages) {
                ok = mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, kWaitDecEmpty);
                if (!ok) break;
              }
              const uint32_t bytes = uint32_t(n) * kRowBytes;
              mbar_arrive_expect_tx(bar_full + stage * 8, bytes);
              const uint32_t dst = smem_base + S::kOffStages + stage * S::kStageBytes;
              if (!paged) {
                tma_load_1d(dst, base + (long long)s0 * kRowBytes, bytes, bar_full + stage * 8, policy);
              } else {
                // one copy per 128-key granule: s0 is a multiple of 128 and so is page_size, so a
                // granule never straddles a page (a 256-key stage of an 8-bit cache may)
                const long long page_stride = (pass == 0 ? args.k_stride_page : args.v_stride_page) * kKvBytes;
                for (int u0 = 0; u0 < n; u0 += kDecStageRows) {
                  const int key = s0 + u0;
                  const int pg = key / args.page_size;
                  tma_load_1d(dst + u0 * kRowBytes,
                              base + (long long)pages[pg] * page_stride + (long long)(key - pg * args.page_size) * kRowBytes,
                              uint32_t(min(kDecStageRows, n - u0)) * kRowBytes, bar_full + stage * 8, policy);
                }
              }
              ++issued;
              if (++stage == kStages) {
                stage = 0;
                phase ^= 1;
              }
            }
          }
        }
      }
      // The consumers observe every copy through the full barriers before they
      // leave, so nothing is in flight at exit unless a wait gave up; in that
      // case let the outstanding copies land (bounded) before retiring.
      if (!ok) {
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else {
    // ----------------------------------------------------------- consumers --
    const int g = tid % kLpr;        // which kEpl head dims this lane owns
    const int r = tid / kLpr;        // key group
    uint32_t stage = 0, phase = 0;
    uint32_t n_done = 0;             // items this CTA has handed to the merger warp
    bool ok = true;

    // Index (within the kKpt keys this thread touches per stage) of the key
    // whose complete dot product the butterfly leaves in this lane.
    int own = 0;
    {
      int n = kKpt, bit = kLpr >> 1;
      while (n > 1) {
        n >>= 1;
        if (g & bit) own += n;
        bit >>= 1;
      }
    }
    // Lanes whose remaining low bits are zero publish the score.
    constexpr int kLowBits = kLpr / kKpt;   // lanes holding the same key after halving
    const bool publishes = (g % kLowBits) == 0;

    for (int item = blockIdx.x; ok && item < args.items; item += gridDim.x) {
      const int bh = item / args.num_splits;
      const int split = item - bh * args.num_splits;
      const int b = bh / args.heads, h = bh - b * args.heads;
      const int key_begin = split * keys_per_split;
      const int key_end = min(args.len_kv, key_begin + keys_per_split);

      // q * scale * log2(e) for this lane's dims
      float qf[kEpl];
      {
        const T* qp = reinterpret_cast<const T*>(args.q) + b * args.q_stride_b + h * args.q_stride_h + g * kEpl;
#pragma unroll
        for (int j = 0; j < kEpl / 8; ++j) {
          const uint4 qv = *reinterpret_cast<const uint4*>(qp + j * 8);
          const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = unpack2<T>(qw[i]);
            qf[j * 8 + 2 * i] = f.x * args.scale_log2;
            qf[j * 8 + 2 * i + 1] = f.y * args.scale_log2;

          }
        }
      }

      float acc[kEpl];
#pragma unroll
      for (int i = 0; i < kEpl; ++i) acc[i] = 0.f;
      float m_run = -INFINITY;
      float l_thread = 0.f;      // this thread's share of sum(p); reduced at the end
      int chunk_idx = 0;

      for (int c0 = key_begin; ok && c0 < key_end; c0 += chunk, ++chunk_idx) {
        const int c1 = min(key_end, c0 + chunk);
        const int n_chunk = c1 - c0;
        float* sc = scores + (chunk_idx & 1) * kDecMaxChunk;

        // ---- scores of this chunk ----
        for (int s0 = 0; s0 < n_chunk; s0 += kKps) {
          const int n = min(kKps, n_chunk - s0);
          ok = __all_sync(0xffffffffu,
                          mbar_wait(bar_full + stage * 8, phase, abort_flag, kWaitDecFullK));
          if (!ok) break;
          const uint8_t* st = smem_gen + S::kOffStages + stage * S::kStageBytes + r * kRowBytes + g * 16;
          // this thread's kKpt rows first (all loads in flight together), then the arithmetic
          uint4 raw[kKpt];
          if (n == kKps) {
#pragma unroll
            for (int i = 0; i < kKpt; ++i) raw[i] = *reinterpret_cast<const uint4*>(st + i * kGroups * kRowBytes);
          } else {
#pragma unroll
            for (int i = 0; i < kKpt; ++i)
              raw[i] = i * kGroups + r < n ? *reinterpret_cast<const uint4*>(st + i * kGroups * kRowBytes)
                                           : make_uint4(0u, 0u, 0u, 0u);
          }
          float part[kKpt];
#pragma unroll
          for (int i = 0; i < kKpt; ++i) {
            float d0 = 0.f, d1 = 0.f;          // two chains: half the dependent latency
            float kf[kEpl];
            unpack_row16<KV>(raw[i], kf);
#pragma unroll
            for (int e = 0; e < kEpl; e += 2) {
              d0 = fmaf(kf[e], qf[e], d0);
              d1 = fmaf(kf[e + 1], qf[e + 1], d1);
            }
            part[i] = d0 + d1;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty + stage * 8);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
          // Transposing butterfly over the kLpr lanes of a row: each step
          // halves the values held and doubles the lanes summed.
          {
            int n_live = kKpt;
#pragma unroll
            for (int bit = kLpr >> 1; bit >= 1; bit >>= 1) {
              if (n_live > 1) {
                const int half = n_live >> 1;
                const bool upper = (g & bit) != 0;
#pragma unroll
                for (int i = 0; i < kKpt / 2; ++i) {
                  if (i < half) {
                    const float send = upper ? part[i] : part[i + half];
                    const float keep = upper ? part[i + half] : part[i];
                    part[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                  }
                }
                n_live = half;
              } else {
                part[0] += __shfl_xor_sync(0xffffffffu, part[0], bit);
              }
            }
          }
          if (publishes) {
            const int key = own * kGroups + r;
            sc[s0 + key] = key < n ? part[0] : -INFINITY;
          }
        }
        if (!ok) break;
        consumer_sync();

        // ---- chunk maximum, probabilities ----
        float m_loc = -INFINITY;
        for (int i = tid; i < n_chunk; i += kDecConsumerThreads) m_loc = fmaxf(m_loc, sc[i]);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
          m_loc = fmaxf(m_loc, __shfl_xor_sync(0xffffffffu, m_loc, off));
        float* wmax = warp_scratch + (chunk_idx & 1) * 8;
        if (lane == 0) wmax[warp] = m_loc;
        consumer_sync();
        float m_chunk = wmax[0];
#pragma unroll
        for (int w = 1; w < kDecConsumerThreads / 32; ++w) m_chunk = fmaxf(m_chunk, wmax[w]);
        const float m_new = fmaxf(m_run, m_chunk);
        const float alpha = fast_exp2(m_run - m_new);   // 0 on the first chunk
        m_run = m_new;
        l_thread *= alpha;
#pragma unroll
        for (int i = 0; i < kEpl; ++i) acc[i] *= alpha;
        for (int i = tid; i < n_chunk; i += kDecConsumerThreads) {
          const float p = fast_exp2(sc[i] - m_new);
          sc[i] = p;
          l_thread += p;
        }
        consumer_sync();

        // ---- O += P V ----
        for (int s0 = 0; s0 < n_chunk; s0 += kKps) {
          const int n = min(kKps, n_chunk - s0);
          ok = __all_sync(0xffffffffu,
                          mbar_wait(bar_full + stage * 8, phase, abort_flag, kWaitDecFullV));
          if (!ok) break;
          const uint8_t* st = smem_gen + S::kOffStages + stage * S::kStageBytes + r * kRowBytes + g * 16;
          uint4 raw[kKpt];
          float pk[kKpt];
          if (n == kKps) {
#pragma unroll
            for (int i = 0; i < kKpt; ++i) {
              raw[i] = *reinterpret_cast<const uint4*>(st + i * kGroups * kRowBytes);
              pk[i] = sc[s0 + i * kGroups + r];
            }
          } else {
            // rows past the end of the chunk hold stale bytes: they enter as zero weight times zero
#pragma unroll
            for (int i = 0; i < kKpt; ++i) {
              const bool live = i * kGroups + r < n;
              raw[i] = live ? *reinterpret_cast<const uint4*>(st + i * kGroups * kRowBytes) : make_uint4(0u, 0u, 0u, 0u);
              pk[i] = live ? sc[s0 + i * kGroups + r] : 0.f;
            }
          }
#pragma unroll
          for (int i = 0; i < kKpt; ++i) {
            float vf[kEpl];
            unpack_row16<KV>(raw[i], vf);
#pragma unroll
            for (int e = 0; e < kEpl; ++e) acc[e] = fmaf(pk[i], vf[e], acc[e]);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty + stage * 8);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) break;

      // ---- reduce the key groups, write the partial row ----
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1)
        l_thread += __shfl_xor_sync(0xffffffffu, l_thread, off);
      // the key groups of a warp (lanes kLpr apart own the same dims) first, then the warps through shared memory
#pragma unroll
      for (int off = kLpr; off < 32; off <<= 1) {
#pragma unroll
        for (int e = 0; e < kEpl; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
      }
      consumer_sync();   // previous item's readers of red / warp_scratch are done
      if (lane == 0) warp_scratch[warp] = l_thread;
      if (lane < kLpr) {
        float4* dst = reinterpret_cast<float4*>(red + warp * D + lane * kEpl);
#pragma unroll
        for (int j = 0; j < kEpl / 4; ++j)
          dst[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
      }
      consumer_sync();
      if (tid < D) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kDecConsumerThreads / 32; ++w) o += red[w * D + tid];
        args.part_o[(long long)item * D + tid] = o * args.v_scale;
      } else if (tid == D) {
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < kDecConsumerThreads / 32; ++w) l += warp_scratch[w];
        args.part_ml[(long long)item * 2 + 0] = m_run;
        args.part_ml[(long long)item * 2 + 1] = l;
      }

      if (fused) {
        // Tell the merger warp that this item's partial row is written (one arrival
        // per warp; the arrival orders the warp's stores before it).  The slot must
        // have been taken kDecDoneSlots items ago, which it always has unless the
        // merger is that far behind.
        if (n_done >= kDecDoneSlots)
          ok = __all_sync(0xffffffffu, mbar_wait(bar_free + (n_done % kDecDoneSlots) * 8,
                                                 ((n_done / kDecDoneSlots) - 1) & 1, abort_flag, kWaitDecFree));
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_done + (n_done % kDecDoneSlots) * 8);
        ++n_done;
      }
    }

    if (ok && args.fuse.final_phase) {
      // ---- final combine of the gathered rows, once every sender's flag is up ----
      const DecodeFuseArgs& f = args.fuse;
      bool waited = false;
      for (int row = blockIdx.x; row < f.rows; row += gridDim.x) {
        if (!waited) {
          if (tid < f.n_peers && !wait_gather_flag(f.local_flags + tid, f.step)) *s_gave_up = 1;
          consumer_sync();
          waited = true;
        }
        if (tid < D) {
          const long long slot_floats = (long long)f.rows * (D + 2);
          const float* ml = f.local_area + (long long)f.rows * D + (long long)row * 2;
          const float* po = f.local_area + (long long)row * D + tid;
          float m = -INFINITY;
          for (int p = 0; p < f.n_peers; ++p) m = fmaxf(m, __ldcg(ml + p * slot_floats));
          float acc_o = 0.f, l = 0.f;
          for (int p = 0; p < f.n_peers; ++p) {
            const float mp = __ldcg(ml + p * slot_floats), lp = __ldcg(ml + p * slot_floats + 1);
            const float w = (mp == -INFINITY) ? 0.f : fast_exp2(mp - m);
            l = fmaf(lp, w, l);
            acc_o = fmaf(__ldcg(po + p * slot_floats), w, acc_o);
          }
          // a wait that gave up must not pass for a result: the rows read NaN
          const bool bad = *s_gave_up != 0;
          const int b = row / args.heads, h = row - b * args.heads;
          T* op = reinterpret_cast<T*>(f.o) + b * f.o_stride_b + h * f.o_stride_h;
          op[tid] = to_out<T>(bad ? __int_as_float(0x7fc00000) : acc_o / l);
          if (tid == 0 && f.lse != nullptr)
            f.lse[row] = bad ? __int_as_float(0x7fc00000) : 0.6931471805599453f * (m + log2f(l));
        }
      }
    }
  }
}

// ------------------------------------------------------------------ combine --
struct DecodeCombineArgs {
  const float* part_o;
  const float* part_ml;
  int n_parts;
  long long part_stride_o, row_stride_o;
  long long part_stride_ml, row_stride_ml;
  int heads;
  void* o;                 // final output (16-bit) or null
  long long o_stride_b, o_stride_h;
  float* lse;              // [rows] or null
  float* out_part_o;       // merged partial [rows][D] or null
  float* out_part_ml;      // merged partial [rows][2]
  // Fused all-gather over peer memory (merged form only).  When peer_bases is
  // non-null the merged row is stored straight into the gather buffer of every
  // rank (peer_bases[p] + scatter_offset floats; rows*D of O, then rows*2 of
  // (m, l)), and the CTA that finishes last publishes `step` in word my_rank of
  // every rank's flag array (peer_bases[p] + flag_offset floats).
  float* const* peer_bases;
  int n_peers;
  int my_rank;
  int rows_total;
  long long scatter_offset;
  long long flag_offset;
  unsigned step;
  // Final form only: wait until wait_flags[r] has reached wait_step for every r
  // (the slots of all ranks have landed) before reading the partials.
  const unsigned* wait_flags;
  int wait_n;
  unsigned wait_step;
};

// CTAs of the scatter kernel that have stored their rows (one sharded decode
// may be in flight per device).
__device__ unsigned int g_scatter_done = 0;

constexpr int kCombineGroups = 4;

// grid = rows, block = (D, kCombineGroups).  Thread (d, j) walks parts j,
// j + kCombineGroups, ... of output dim d.
template <typename T, int D>
__global__ void __launch_bounds__(D * kCombineGroups) decode_combine_kernel(const DecodeCombineArgs a) {
  __shared__ float s_red[kCombineGroups][D];
  __shared__ float s_m[kCombineGroups * D / 32];
  __shared__ float s_l[kCombineGroups];
  const int row = blockIdx.x;
  const int d = threadIdx.x;
  const int j = threadIdx.y;
  const int tid = j * D + d;
  const int n_threads = D * kCombineGroups;
  const float* ml = a.part_ml + (long long)row * a.row_stride_ml;
  const float* po = a.part_o + (long long)row * a.row_stride_o;

  __shared__ int s_gave_up;
  if (a.wait_flags != nullptr) {
    // Bounded wait for the peers' stores (flags are written with release
    // semantics after a system-scope fence on the sending GPU).
    if (tid == 0) s_gave_up = 0;
    __syncthreads();
    if (tid < a.wait_n && !wait_gather_flag(a.wait_flags + tid, a.wait_step)) s_gave_up = 1;
    __syncthreads();
  }
  // a wait that gave up must not pass for a result: the row reads NaN
  const bool bad = a.wait_flags != nullptr && s_gave_up != 0;

  // pass 1: global maximum
  float m = -INFINITY;
  for (int p = tid; p < a.n_parts; p += n_threads) m = fmaxf(m, ml[(long long)p * a.part_stride_ml]);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((tid & 31) == 0) s_m[tid >> 5] = m;
  __syncthreads();
  m = s_m[0];
#pragma unroll
  for (int w = 1; w < kCombineGroups * D / 32; ++w) m = fmaxf(m, s_m[w]);

  // pass 2: weighted sums
  float acc = 0.f, l = 0.f;
  for (int p = j; p < a.n_parts; p += kCombineGroups) {
    const float mp = ml[(long long)p * a.part_stride_ml];
    const float lp = ml[(long long)p * a.part_stride_ml + 1];
    const float w = (mp == -INFINITY) ? 0.f : fast_exp2(mp - m);
    l = fmaf(lp, w, l);
    acc = fmaf(po[(long long)p * a.part_stride_o + d], w, acc);
  }
  s_red[j][d] = acc;
  if (d == 0) s_l[j] = l;
  __syncthreads();
  if (j == 0) {
    float o = 0.f, lt = 0.f;
#pragma unroll
    for (int q = 0; q < kCombineGroups; ++q) {
      o += s_red[q][d];
      lt += s_l[q];
    }
    if (a.peer_bases != nullptr) {
      for (int p = 0; p < a.n_peers; ++p) {
        float* base = a.peer_bases[p] + a.scatter_offset;
        base[(long long)row * D + d] = o;
        if (d == 0) {
          float* mlp = base + (long long)a.rows_total * D + (long long)row * 2;
          mlp[0] = m;
          mlp[1] = lt;
        }
      }
    } else if (a.out_part_o != nullptr) {
      a.out_part_o[(long long)row * D + d] = o;
      if (d == 0) {
        a.out_part_ml[(long long)row * 2 + 0] = m;
        a.out_part_ml[(long long)row * 2 + 1] = lt;
      }
    } else {
      const int b = row / a.heads, h = row - b * a.heads;
      T* op = reinterpret_cast<T*>(a.o) + b * a.o_stride_b + h * a.o_stride_h;
      const float nan = __int_as_float(0x7fc00000);
      op[d] = to_out<T>(bad ? nan : o / lt);
      if (d == 0 && a.lse != nullptr) a.lse[row] = bad ? nan : 0.6931471805599453f * (m + log2f(lt));
    }
  }
  if (a.peer_bases != nullptr) {
    // Publish: every CTA fences its peer stores; the last one to finish raises
    // the flag on every rank and re-arms the counter for the next step.
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&g_scatter_done, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (s_last) {
      __threadfence_system();
      if (tid < a.n_peers)
        st_release_sys(reinterpret_cast<unsigned*>(a.peer_bases[tid] + a.flag_offset) + a.my_rank, a.step);
      if (tid == 0) g_scatter_done = 0;
    }
  }
}

}  // namespace tfb
