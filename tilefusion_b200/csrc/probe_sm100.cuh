// Measurement kernel: how long the tensor pipe of one SM takes per tcgen05.mma
// (M128, K16, kind::f16) when one thread issues them back to back -- the figures
// the roofline arguments for the attention kernels rest on.  It computes nothing
// useful: the operands are whatever shared and tensor memory hold.
//
//   a_from_tmem : 0 = both operands through shared-memory descriptors (the S = Q K^T form),
//                 1 = A operand in tensor memory (the O += P V form)
//   n           : 64, 128 or 256 accumulator columns
//   b_mn_major  : 0 = B rows run along the contraction (K-major, a [N][K] tile),
//                 1 = B rows run along N (MN-major, a [K][N] tile: V in P V)
//   desc32      : 0 = a 64-bit shared-memory descriptor is built for every MMA,
//                 1 = descriptors are 32-bit low halves advanced by constants (the
//                 issuing thread then spends fewer clocks per MMA than the pipe)
//   uniform_issue: 0 = the issuing thread is alone in a branch on its lane number,
//                 1 = the whole warp walks the loop and one elected lane issues
// Both layouts are the 128-byte-swizzle tiles the attention kernels use
// ([128 rows][64 16-bit columns] blocks of 16 KB).
#pragma once

#include "attn_fwd_sm100.cuh"

namespace tfb {

struct ProbeMmaArgs {
  int a_from_tmem;
  int n;
  int b_mn_major;
  int desc32;
  int uniform_issue;
  int n_mma;             // a multiple of 8
  long long* out;        // [2]: clocks until all are issued, clocks until all are complete
};

constexpr int kProbeSmemBytes = 2 * 32768 + 65536 + 1024;

__global__ void __launch_bounds__(128, 1) probe_mma_kernel(const ProbeMmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(8) uint64_t bar_mem;
  const uint32_t bar = smem_u32(&bar_mem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc<512>(smem_u32(&tmem_slot));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  if (warp == 0) {
    const uint32_t a_smem = base, b_smem = base + 32768;      // B: up to [128][256] 16-bit = 64 KB
    const uint32_t idesc = make_idesc(128, a.n, 0, 0, a.b_mn_major);
    const uint32_t b_block = 16384;                           // one [128 rows][64 columns] block
    const uint32_t a_lo = desc_lo(a_smem, 16);
    const uint32_t b_lo = a.b_mn_major ? desc_lo(b_smem, b_block) : desc_lo(b_smem, 16);
    const uint32_t b_hi_step = a.b_mn_major ? 4 * 2048 : a.n * 128, b_lo_step = a.b_mn_major ? 2048 : 32;
    // `issue` is true in the one lane that issues; with uniform_issue the other 31 lanes walk the
    // same loops beside it, otherwise they never enter.
    auto run = [&](bool issue, bool whole_warp) {
      const long long t0 = clock64();
      if (a.desc32) {
        for (int g = 0; g < a.n_mma / 8; ++g) {
          if (issue) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t bd = b_lo + (((k >> 2) * b_hi_step + (k & 3) * b_lo_step) >> 4);
              if (a.a_from_tmem)
                umma_ts_lohi(tm, tm + 384 + k * 8, bd, kDescHiSw128, idesc, 1);
              else
                umma_ss_lohi(tm, a_lo + (((k >> 2) * 16384 + (k & 3) * 32) >> 4), bd, kDescHiSw128, idesc, 1);
            }
          }
        }
      } else {
        for (int g = 0; g < a.n_mma / 8; ++g) {
          if (issue) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              // K-major: [n rows][64 contraction columns] blocks of n * 128 bytes, 32 bytes per K16 step;
              // MN-major: [128 contraction rows][64 columns] blocks of 16 KB, 16 rows = 2048 bytes per step.
              const uint64_t bd = a.b_mn_major ? make_smem_desc(b_smem + k * 2048, b_block, 1024)
                                               : make_smem_desc(b_smem + (k >> 2) * (a.n * 128) + (k & 3) * 32, 16, 1024);
              if (a.a_from_tmem)
                umma_ts(tm, tm + 384 + k * 8, bd, idesc, 1);
              else
                umma_ss(tm, make_smem_desc(a_smem + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), bd, idesc, 1);
            }
          }
        }
      }
      if (issue) umma_commit(bar);
      const long long t1 = clock64();
      if (whole_warp)
        mbar_wait_warp(bar, 0, &abort_flag, 901);
      else
        mbar_wait(bar, 0, &abort_flag, 901);
      const long long t2 = clock64();
      if (issue) {
        a.out[0] = t1 - t0;
        a.out[1] = t2 - t0;
      }
    };
    if (a.uniform_issue) {
      run(elect_one(), true);
    } else if (lane == 0) {
      run(true, false);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc<512>(tm);
  }
}

// ---------------------------------------------------------------------------
// The same measurement for the two-CTA form: a cluster of two CTAs on two SMs,
// tcgen05.mma.cta_group::2 with M = 256 (128 accumulator rows in each CTA's
// tensor memory) and N = `n`; each CTA's shared memory holds its own 128 rows of
// A and n / 2 of B's columns.  One elected lane of the first CTA issues for both
// (32-bit descriptor halves, the whole warp walking the loop).  Per SM the
// arithmetic of one such MMA equals that of an M128 single-CTA MMA of the same
// N, so the two probes' clocks compare directly.
struct ProbePairArgs {
  int a_from_tmem;
  int n;
  int b_mn_major;
  int n_mma;             // a multiple of 8
  long long* out;        // [2]: clocks until all are issued, clocks until all are complete
};

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void umma_pair_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                  uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_pair_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi,
                                                  uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 db;\n"
      "mov.b64 db, {%2, %3};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) probe_mma_pair_kernel(const ProbePairArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(8) uint64_t bar_mem;
  const uint32_t bar = smem_u32(&bar_mem);
  const int warp = threadIdx.x >> 5;
  uint32_t cta_rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {       // the same warp of both CTAs allocates (and later frees) the pair's columns
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "n"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  if (warp == 0 && cta_rank == 0) {
    const uint32_t a_smem = base, b_smem = base + 32768;
    const uint32_t idesc = make_idesc(256, a.n, 0, 0, a.b_mn_major);
    const uint32_t a_lo = desc_lo(a_smem, 16);
    const uint32_t b_lo = a.b_mn_major ? desc_lo(b_smem, 16384) : desc_lo(b_smem, 16);
    const uint32_t b_hi_step = a.b_mn_major ? 4 * 2048 : (a.n / 2) * 128, b_lo_step = a.b_mn_major ? 2048 : 32;
    const bool issue = elect_one();
    const long long t0 = clock64();
    for (int g = 0; g < a.n_mma / 8; ++g) {
      if (issue) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t bd = b_lo + (((k >> 2) * b_hi_step + (k & 3) * b_lo_step) >> 4);
          if (a.a_from_tmem)
            umma_pair_ts_lohi(tm, tm + 384 + k * 8, bd, kDescHiSw128, idesc, 1);
          else
            umma_pair_ss_lohi(tm, a_lo + (((k >> 2) * 16384 + (k & 3) * 32) >> 4), bd, kDescHiSw128, idesc, 1);
        }
      }
    }
    if (issue)
      asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    const long long t1 = clock64();
    mbar_wait_warp(bar, 0, &abort_flag, 902);
    const long long t2 = clock64();
    if (issue) {
      a.out[0] = t1 - t0;
      a.out[1] = t2 - t0;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // nothing of the pair is in flight in either CTA past this point
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tm), "n"(512) : "memory");
  }
}

}  // namespace tfb
