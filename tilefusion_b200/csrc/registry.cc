#include "registry.h"

#include <algorithm>
#include <cstdint>

namespace tfb {

namespace {
// tile_q 128: one Q tile per CTA, two CTAs per SM (attn_fwd_kernel).
// tile_q 256: two Q tiles per CTA, persistent, one CTA per SM (attn_fwd_pair_kernel).
constexpr AttnVariant kAttnVariants[] = {
    {TF_F16, 128, 256, 128, 1}, {TF_BF16, 128, 256, 128, 1},
    {TF_F16, 64, 256, 128, 1},  {TF_BF16, 64, 256, 128, 1},
    {TF_F16, 128, 128, 128, 2}, {TF_BF16, 128, 128, 128, 2},
    {TF_F16, 64, 128, 128, 2},  {TF_BF16, 64, 128, 128, 2},
    {TF_F16, 256, 128, 128, 1}, {TF_BF16, 256, 128, 128, 1},
    {0, 0, 0, 0, 0},
};
constexpr int kDecodeCtasPerSm = 2;
constexpr int kDecodeStages = 3;        // stages of 256 * D bytes: 128 keys of a 16-bit cache, 256 of an 8-bit one
}  // namespace

const AttnVariant* attn_variants() { return kAttnVariants; }

int head_dim_bucket(int head_dim, int head_dim_v) {
  const int need = std::max(head_dim, head_dim_v);
  return need <= 64 ? 64 : need <= 128 ? 128 : 256;
}

void plan_attn(const TfAttnDesc& d, int sm_count, TfAttnPlan* plan) {
  // Heuristic: a single Q tile cannot use the two-tile schedule, and a problem
  // with fewer tile pairs than SMs fills more of the GPU with one tile per CTA
  // -- unless the KV loop is long: measured on 148 SMs with 128 pairs, the
  // two-tile kernel is 1.14x / 1.23x faster at 2048 / 8192 keys, even at 1024
  // and 0.93x at 512; with 64 pairs and 2048 keys the two are even.
  const int64_t bh = (int64_t)d.batch * d.heads;
  const int64_t pairs = bh * ((d.len_q + 255) / 256);
  const int64_t singles = bh * ((d.len_q + 127) / 128);
  const bool few_pairs = pairs < sm_count && !(pairs * 4 >= (int64_t)sm_count * 3 && d.len_kv >= 2048);
  const int want_tile_q = (d.len_q <= 128 || (few_pairs && singles > pairs)) ? 128 : 256;
  // Kernels exist for head dims 64, 128 and 256; a problem runs on the smallest
  // one that holds both of its head dims, zero-padded (TMA fills the padding).
  const int bucket = head_dim_bucket(d.head_dim, d.head_dim_v);
  const AttnVariant* best = nullptr;
  const AttnVariant* any = nullptr;
  const AttnVariant* hinted = nullptr;
  for (const AttnVariant* v = kAttnVariants; v->head_dim != 0; ++v) {
    if (v->dtype != d.dtype || v->head_dim != bucket) continue;
    if (any == nullptr) any = v;
    if (v->tile_q == want_tile_q && best == nullptr) best = v;
    // A caller's tile hint wins when it names a compiled variant.
    if (d.tile_q == v->tile_q && d.tile_kv == v->tile_kv && hinted == nullptr) hinted = v;
  }
  if (best == nullptr) best = any;       // (head dim 256 has the one-tile kernel only)
  if (hinted != nullptr) best = hinted;
  plan->head_dim_kernel = bucket;
  plan->tile_q = best->tile_q;
  plan->tile_kv = best->tile_kv;
  plan->ctas_per_sm = best->ctas_per_sm;
  const int64_t q_tiles = (d.len_q + best->tile_q - 1) / best->tile_q;
  int64_t grid = q_tiles * d.heads * d.batch;
  if (best->tile_q == 256) grid = std::min<int64_t>(grid, std::max(1, sm_count));   // persistent
  plan->grid = (int32_t)std::min<int64_t>(grid, INT32_MAX);
  // With both strides 1 (a single key or a single head dim) either reading
  // is valid; the row-contiguous one is kept.
  plan->k_mn_major = d.k_stride_d == 1 ? 0 : 1;
  plan->v_mn_major = d.v_stride_d == 1 ? 1 : 0;
  plan->smem_bytes = 0;
}

int default_kv_chunk(const TfDecodeDesc& d) {
  // The per-chunk work that does not scale with the bytes (three block-wide barriers, the
  // softmax over the chunk's scores) is spread over half as many bytes with an 8-bit cache.
  return (d.kv_dtype == TF_FP8_E4M3 || d.kv_dtype == TF_FP8_E5M2) ? 1024 : 512;
}

void plan_decode(const TfDecodeDesc& d, int sm_count, TfDecodePlan* plan) {
  const bool kv8 = d.kv_dtype == TF_FP8_E4M3 || d.kv_dtype == TF_FP8_E5M2;
  if (d.heads_kv > 0 && d.heads_kv != d.heads && !kv8) {
    // Grouped-query decoding over a 16-bit cache runs on the two-tile attention kernel in split-KV
    // mode: work item = (batch, KV head, split), a split walks whole 128-key
    // tiles.  Enough splits for about two items per SM, never an empty one.
    const int64_t groups = (int64_t)d.batch * d.heads_kv;
    const int n_tiles = std::max(1, (d.len_kv + 127) / 128);
    const int grid = std::max(1, sm_count);
    int want = d.num_splits;
    if (want <= 0) {
      // Items are dealt round-robin to one persistent CTA per SM; take the fewest
      // splits whose makespan ceil(items / grid) * tiles_per_split is within 3 %
      // of the best over all split counts (fewer partial rows to combine).
      auto span = [&](int splits) {
        const int t = (n_tiles + splits - 1) / splits;
        const int64_t items = groups * ((n_tiles + t - 1) / t);
        return ((items + grid - 1) / grid) * (int64_t)t;
      };
      int64_t best = INT64_MAX;
      for (int sp = 1; sp <= n_tiles; ++sp) best = std::min(best, span(sp));
      want = 1;
      while (want < n_tiles && span(want) * 100 > best * 103) ++want;
    }
    const int tps = (n_tiles + want - 1) / want;
    const int splits = (n_tiles + tps - 1) / tps;
    // With at most 32 query heads per KV head the rows of a group are replicated in the four lane
    // quarters of the Q tile and every quarter takes a quarter of each KV tile's keys (a fourth of
    // the exponentials per thread and tile): four partial rows per (row, split).
    const int copies = d.heads / d.heads_kv <= 32 ? 4 : 1;
    plan->num_splits = splits * copies;
    plan->chunks_per_split = tps;
    plan->kv_chunk = 128;
    plan->grid = (int32_t)std::min<int64_t>(grid, groups * splits);
    plan->stages = 5;
    plan->reserved = copies;
    plan->workspace_bytes = (uint64_t)d.batch * d.heads * splits * copies * (d.head_dim + 2) * sizeof(float);
    return;
  }
  const int chunk = d.kv_chunk == 0 ? default_kv_chunk(d) : d.kv_chunk;
  const int64_t bh = (int64_t)d.batch * d.heads;
  const int n_chunks = std::max(1, (d.len_kv + chunk - 1) / chunk);
  const int grid = std::max(1, sm_count) * kDecodeCtasPerSm;

  int cps = 1;
  if (d.num_splits > 0) {
    const int want = std::min(d.num_splits, n_chunks);
    cps = (n_chunks + want - 1) / want;
  } else {
    // Items are dealt round-robin to a persistent grid, so the step takes
    // ceil(items / grid) item-times.  An item costs its K/V bytes plus a fixed
    // part (set-up, the cross-warp reduction, the partial row): about 1 us, the
    // time in which a CTA streams kItemOverheadBytes at its share of the HBM
    // bandwidth.  Measured on B200: with 64-KB chunks (8-bit cache, D = 64) 16
    // splits per row took 0.47 ms where 2 took 0.38.  Take the split with the
    // smallest makespan; the coarsest on a tie (fewest partial rows to combine).
    constexpr int64_t kItemOverheadBytes = 24 * 1024;
    const int64_t chunk_bytes = 2ll * chunk * d.head_dim * (kv8 ? 1 : 2);
    int64_t best_span = INT64_MAX;
    for (int c = n_chunks; c >= 1; --c) {
      const int64_t splits = (n_chunks + c - 1) / c;
      const int64_t items = bh * splits;
      const int64_t span = ((items + grid - 1) / grid) * (c * chunk_bytes + kItemOverheadBytes);
      if (span < best_span) {
        best_span = span;
        cps = c;
      }
    }
  }
  const int splits = (n_chunks + cps - 1) / cps;
  plan->num_splits = splits;
  plan->chunks_per_split = cps;
  plan->kv_chunk = chunk;
  plan->grid = (int32_t)std::min<int64_t>(grid, bh * splits);
  plan->stages = kDecodeStages;
  plan->reserved = 0;
  plan->workspace_bytes = (uint64_t)bh * splits * (d.head_dim + 2) * sizeof(float);
}

int QueueWords::eager(uintptr_t stream) {
  std::lock_guard<std::mutex> lock(mutex_);
  for (int i = 0; i < n_streams_; ++i)
    if (streams_[i] == stream) return i;
  if (n_streams_ == kEagerWords) return -1;
  streams_[n_streams_] = stream;
  return n_streams_++;
}

int QueueWords::captured() {
  std::lock_guard<std::mutex> lock(mutex_);
  if (n_captured_ == kCapturedWords) return -1;
  return kEagerWords + n_captured_++;
}

void shard_range(int64_t total, int rank, int world, int64_t* begin, int64_t* end) {
  const int64_t base = total / world, extra = total % world;
  *begin = rank * base + std::min<int64_t>(rank, extra);
  *end = *begin + base + (rank < extra ? 1 : 0);
}

}  // namespace tfb
