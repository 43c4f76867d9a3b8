// Fused attention forward for sm_100a: O = softmax(Q K^T * scale [+causal]) V.
//
// Stands in for TileFusion's ke_flash_attention
// (include/kernels/flash_attention_device.cuh:130-312), which runs the same
// loop with mma.sync fragments, a single-stage cp.async copy and an fp16
// softmax.  Here:
//   * one CTA owns a 128-row Q tile of one (batch, head) and walks the KV
//     length in 128-key tiles;
//   * Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle)
//     and complete on mbarriers;
//   * S = Q K^T and O += P V are tcgen05.mma instructions issued by one
//     thread, with S, P and O living in tensor memory: S is 128 fp32 columns,
//     P (16-bit) overwrites the first 64 of them and is read back by the
//     second MMA as its TMEM A operand, O takes D more columns;
//   * four softmax warps own one row per thread (tcgen05.ld 32x32b), keep the
//     running maximum and sum in fp32, use exp2 with scale*log2(e) folded in,
//     and rescale O only when the maximum moved by more than 2^8;
//   * two CTAs share an SM, so one CTA's softmax overlaps the other's MMAs.
// K may be stored [Lk, D] (K-major operand) or [D, Lk] (MN-major), V may be
// stored [Lk, Dv] (MN-major) or [Dv, Lk] (K-major); the shared-memory
// descriptors and the instruction descriptor carry the difference.
#pragma once

#include <type_traits>

#include "sm100_ptx.cuh"

namespace tfb {

constexpr int kAttnTile = 128;          // Q rows per CTA == keys per KV tile
constexpr int kAttnThreads = 160;       // 4 softmax warps + 1 TMA/MMA warp
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnFwdArgs {
  void* o;
  float* lse;            // may be null
  int len_q;
  int len_kv;
  int dim_v;             // columns of O actually stored (<= the kernel's D; the rest is zero padding)
  int causal;
  int k_mn_major;        // K stored [D, Lk]
  int v_mn_major;        // V stored [Lk, Dv]
  float scale_log2;      // softmax_scale * log2(e)
  long long o_stride_b, o_stride_h, o_stride_l;
  long long lse_stride_b, lse_stride_h;
};

template <int D>
struct AttnSmem {
  static constexpr int kTileBytes = kAttnTile * D * 2;      // one Q, K or V tile
  static constexpr int kBlockBytes = kAttnTile * 128;       // one 64-column swizzle block
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kTileBytes;
  static constexpr int kOffV = 2 * kTileBytes;
  static constexpr int kOffBar = 3 * kTileBytes;            // 6 mbarriers
  static constexpr int kOffTmemSlot = kOffBar + 64;
  static constexpr int kOffAbort = kOffBar + 68;
  static constexpr int kBytes = kOffBar + 128 + 1024;       // + slack for 1024-B alignment
};

enum AttnWaitCode {
  kWaitQ = 101, kWaitK = 102, kWaitV = 103, kWaitS = 104, kWaitP = 105, kWaitO = 106,
  kWaitSoftS = 111, kWaitSoftO = 112, kWaitEpiO = 113, kWaitDrain = 114
};

// kNoSoftmax = true turns the kernel into TileFusion's fused_two_gemms
// (include/kernels/fused_two_gemms_device.cuh:114-214): D = (A B^T) C^T with
// the intermediate product rounded to 16 bits, i.e. the same two MMAs with the
// softmax stage replaced by a conversion.  Q = A [M, K], K = B [N, K],
// V = C stored [P, N], O = D [M, P]; K == P == the template's D.
//
// D is the head-dim bucket the kernel is compiled for (64, 128 or 256).  A
// problem whose head dims are smaller runs on the next bucket: the tensor maps
// carry the true extents, TMA fills the missing columns of Q, K and V with
// zeros (which changes neither Q K^T nor P V), and only the first dim_v columns
// of O are stored.  D = 256 takes all 512 TMEM columns (S 128 + O 256) and 192
// KB of shared memory, so one CTA per SM.
template <typename T, int D, bool kNoSoftmax = false>
__global__ void __launch_bounds__(kAttnThreads, D <= 128 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q,
                const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const AttnFwdArgs args) {
  using S = AttnSmem<D>;
  constexpr int kIsBf16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr int kTmemCols = D <= 128 ? 256 : 512;   // S: 128, O: D; a power of two
  constexpr int kColS = 0, kColP = 0, kColO = 128;
  constexpr int kBlocks = D / 64;        // 64-element swizzle blocks per row

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + S::kOffQ;
  const uint32_t sK = smem_base + S::kOffK;
  const uint32_t sV = smem_base + S::kOffV;
  const uint32_t bar_q = smem_base + S::kOffBar + 0;
  const uint32_t bar_k = smem_base + S::kOffBar + 8;
  const uint32_t bar_v = smem_base + S::kOffBar + 16;
  const uint32_t bar_s = smem_base + S::kOffBar + 24;
  const uint32_t bar_p = smem_base + S::kOffBar + 32;
  const uint32_t bar_o = smem_base + S::kOffBar + 40;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + S::kOffTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + S::kOffAbort);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_tile = blockIdx.x;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int q0 = q_tile * kAttnTile;

  int n_kv = (args.len_kv + kAttnTile - 1) / kAttnTile;
  if (args.causal) n_kv = min(n_kv, q_tile + 1);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc<kTmemCols>(smem_u32(const_cast<uint32_t*>(tmem_slot)));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      // ------------------------------------------------ TMA + MMA issuer ----
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const uint32_t idesc_s = make_idesc(128, 128, kIsBf16, 0, args.k_mn_major);
      const uint32_t idesc_o = make_idesc(128, D, kIsBf16, 0, args.v_mn_major);

      auto load_q = [&]() {
        mbar_arrive_expect_tx(bar_q, S::kTileBytes);
#pragma unroll
        for (int blk = 0; blk < kBlocks; ++blk)
          tma_load_4d(sQ + blk * S::kBlockBytes, &map_q, bar_q, blk * 64, q0, head, batch);
      };
      auto load_k = [&](int j) {
        mbar_arrive_expect_tx(bar_k, S::kTileBytes);
        if (!args.k_mn_major) {
#pragma unroll
          for (int blk = 0; blk < kBlocks; ++blk)
            tma_load_4d(sK + blk * S::kBlockBytes, &map_k, bar_k, blk * 64, j * kAttnTile, head,
                        batch);
        } else {
          // [D rows][64 keys] per block, two key blocks per tile
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
            tma_load_4d(sK + blk * (D * 128), &map_k, bar_k, j * kAttnTile + blk * 64, 0, head,
                        batch);
        }
      };
      auto load_v = [&](int j) {
        mbar_arrive_expect_tx(bar_v, S::kTileBytes);
        if (args.v_mn_major) {
          // [128 keys][64 dv] per block
#pragma unroll
          for (int blk = 0; blk < kBlocks; ++blk)
            tma_load_4d(sV + blk * S::kBlockBytes, &map_v, bar_v, blk * 64, j * kAttnTile, head,
                        batch);
        } else {
          // [Dv rows][64 keys] per block
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
            tma_load_4d(sV + blk * (D * 128), &map_v, bar_v, j * kAttnTile + blk * 64, 0, head,
                        batch);
        }
      };
      auto issue_s = [&]() {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t a =
              make_smem_desc(sQ + (k >> 2) * S::kBlockBytes + (k & 3) * 32, 16, 1024);
          const uint64_t b =
              args.k_mn_major
                  ? make_smem_desc(sK + k * 2048, D * 128, 1024)
                  : make_smem_desc(sK + (k >> 2) * S::kBlockBytes + (k & 3) * 32, 16, 1024);
          umma_ss(tmem_base + kColS, a, b, idesc_s, k > 0);
        }
        umma_commit(bar_s);
      };
      auto issue_pv = [&](int j) {
#pragma unroll
        for (int k = 0; k < kAttnTile / 16; ++k) {
          const uint64_t b =
              args.v_mn_major
                  ? make_smem_desc(sV + k * 2048, S::kBlockBytes, 1024)
                  : make_smem_desc(sV + (k >> 2) * (D * 128) + (k & 3) * 32, 16, 1024);
          umma_ts(tmem_base + kColO, tmem_base + kColP + k * 8, b, idesc_o, (j > 0) || (k > 0));
        }
        umma_commit(bar_o);
      };

      // k_issued / v_issued count the tile loads sent to each barrier and
      // k_seen / v_seen the completions observed, so that an aborting CTA
      // knows which copies may still be in flight.
      bool ok = true;
      int k_issued = 0, k_seen = 0, v_issued = 0, v_seen = 0;
      load_q();
      load_k(0);
      ++k_issued;
      load_v(0);
      ++v_issued;
      ok = mbar_wait(bar_q, 0, abort_flag, kWaitQ) && mbar_wait(bar_k, 0, abort_flag, kWaitK);
      if (ok) {
        ++k_seen;
        issue_s();
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const uint32_t ph = j & 1;
        // K buffer is free once S_j has been computed.
        ok = mbar_wait(bar_s, ph, abort_flag, kWaitS);
        if (!ok) break;
        if (j + 1 < n_kv) {
          load_k(j + 1);
          ++k_issued;
        }
        ok = mbar_wait(bar_p, ph, abort_flag, kWaitP) && mbar_wait(bar_v, ph, abort_flag, kWaitV);
        if (!ok) break;
        ++v_seen;
        tc_fence_after();
        issue_pv(j);
        if (j + 1 < n_kv) {
          ok = mbar_wait(bar_k, ph ^ 1, abort_flag, kWaitK);
          if (!ok) break;
          ++k_seen;
          issue_s();
        }
        // V buffer is free once O += P_j V_j has completed.
        ok = mbar_wait(bar_o, ph, abort_flag, kWaitO);
        if (!ok) break;
        if (j + 1 < n_kv) {
          load_v(j + 1);
          ++v_issued;
        }
      }
      if (!ok) {
        // Give copies still in flight a bounded chance to land before the CTA
        // retires its shared memory.
        const unsigned long long t0 = global_timer_ns();
        while ((k_seen < k_issued || v_seen < v_issued) &&
               global_timer_ns() - t0 < wait_limit_ns()) {
          if (k_seen < k_issued && mbar_try_wait(bar_k, k_seen & 1)) ++k_seen;
          if (v_seen < v_issued && mbar_try_wait(bar_v, v_seen & 1)) ++v_seen;
        }
      }
    }
  } else {
    // ------------------------------------------------------ softmax warps ---
    const int row = warp * 32 + lane;                       // row of the Q tile == TMEM lane
    const uint32_t t_lane = tmem_base + (uint32_t(warp * 32) << 16);
    const int q_idx = q0 + row;
    float m_used = -INFINITY;    // maximum (raw scores) the running sums are relative to
    float l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const uint32_t ph = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_s, ph, abort_flag, kWaitSoftS));
      if (!ok) break;
      tc_fence_after();

      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_lane + kColS + c * 32, sr[c]);
      tmem_wait_ld();

      if constexpr (kNoSoftmax) {
        // P = S rounded to 16 bits (columns beyond len_kv are zero: TMA zero-fills K)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            pk[i >> 1] = pack2<T>(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
          tmem_st16(t_lane + kColP + c * 16, pk);
        }
        l_run = 1.f;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p);
        continue;
      }

      const int kv0 = j * kAttnTile;
      const bool need_mask =
          (kv0 + kAttnTile > args.len_kv) || (args.causal && (kv0 + kAttnTile - 1 > q0));
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = kv0 + c * 32 + i;
            const bool masked = (col >= args.len_kv) || (args.causal && col > q_idx);
            if (masked) sr[c][i] = 0xff800000u;  // -inf
          }
      }

      // Row maximum: eight independent chains (two per chunk) of 3-input max
      // instructions in one straight line of code, so that they pipeline.
      float m_tile;
      {
        float ma[4], mb[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          ma[c] = max3(__uint_as_float(sr[c][0]), __uint_as_float(sr[c][1]), __uint_as_float(sr[c][2]));
          mb[c] = max3(__uint_as_float(sr[c][3]), __uint_as_float(sr[c][4]), __uint_as_float(sr[c][5]));
        }
#pragma unroll
        for (int i = 6; i + 3 < 32; i += 4) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            ma[c] = max3(ma[c], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
            mb[c] = max3(mb[c], __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          ma[c] = max3(ma[c], mb[c], fmaxf(__uint_as_float(sr[c][30]), __uint_as_float(sr[c][31])));
        m_tile = fmaxf(fmaxf(ma[0], ma[1]), fmaxf(ma[2], ma[3]));
      }

      // Lazy rescale: keep the old reference maximum unless the new one is
      // more than 2^kRescaleThreshold above it.
      const bool grow = (m_tile - m_used) * args.scale_log2 > kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_used, m_tile);
        const float alpha = fast_exp2((m_used - m_new) * args.scale_log2);
        m_used = m_new;
        l_run *= alpha;
        if (j > 0) {
          // O holds the sum of tiles 0..j-1 once the previous P V has completed.
          ok = __all_sync(0xffffffffu, mbar_wait(bar_o, ph ^ 1, abort_flag, kWaitSoftO));
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            uint32_t orow[16];
            tmem_ld16(t_lane + kColO + c * 16, orow);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i)
              orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
            tmem_st16(t_lane + kColO + c * 16, orow);
          }
        }
      }

      // P = 2^(s*scale - m); scale-subtract and row sum as packed f32x2
      // instructions (they overlap with the MUFU, scalar FMAs only partly), the
      // sum in four independent accumulators.
      const float m_scaled = m_used * args.scale_log2;
      const uint64_t scale2 = f2_pack(args.scale_log2, args.scale_log2);
      const uint64_t negm2 = f2_pack(-m_scaled, -m_scaled);
      uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0, x1;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), scale2, negm2),
                    x0, x1);
          const float p0 = fast_exp2(x0);
          const float p1 = fast_exp2(x1);
          ls2[(i >> 1) & 3] = f2_add(ls2[(i >> 1) & 3], f2_pack(p0, p1));
          pk[i >> 1] = pack2<T>(p0, p1);
        }
        tmem_st16(t_lane + kColP + c * 16, pk);
      }
      {
        float lo, hi;
        f2_unpack(f2_add(f2_add(ls2[0], ls2[1]), f2_add(ls2[2], ls2[3])), lo, hi);
        l_run += lo + hi;
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p);
    }

    // ------------------------------------------------------------ epilogue --
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_o, (n_kv - 1) & 1, abort_flag, kWaitEpiO));
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l_run;
      const bool row_valid = q_idx < args.len_q;
      T* o_row = reinterpret_cast<T*>(args.o) + (long long)batch * args.o_stride_b +
                 (long long)head * args.o_stride_h + (long long)q_idx * args.o_stride_l;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orow[32];
        tmem_ld32(t_lane + kColO + c * 32, orow);
        tmem_wait_ld();
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
      if (row_valid && args.lse != nullptr) {
        args.lse[(long long)batch * args.lse_stride_b + (long long)head * args.lse_stride_h +
                 q_idx] = 0.6931471805599453f * (m_used * args.scale_log2 + log2f(l_run));
      }
    }
  }

  // ---------------------------------------------------------------- teardown --
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

}  // namespace tfb
