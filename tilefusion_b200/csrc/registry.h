// Variant registry: picks tile shapes (prefill) and split counts (decode) per
// (sequence length, head_dim).  TileFusion bakes caller-supplied tile sizes
// into a kernel it JIT-compiles per exact shape (src/kernels/flash_attn.cu:16-55,
// src/jit/compiler.cc:123-145); here the variants are compiled ahead of time,
// sequence lengths are run-time arguments, and this table chooses among them.
// Host-only code: it has no CUDA dependency and is unit-tested without a GPU.
#pragma once

#include <cstdint>
#include <mutex>

#include "tilefusion_b200.h"

namespace tfb {

// One compiled prefill variant.
struct AttnVariant {
  int dtype;        // TfDType
  int head_dim;
  int tile_q;
  int tile_kv;
  int ctas_per_sm;
};

// The table of compiled prefill variants (terminated by head_dim == 0).
const AttnVariant* attn_variants();

// Compiled head dim (64, 128 or 256) that a problem with these head dims runs on.
int head_dim_bucket(int head_dim, int head_dim_v);

// Fills `plan` for `desc` on a GPU with `sm_count` SMs.  `desc` must have been
// validated by the caller.
void plan_attn(const TfAttnDesc& desc, int sm_count, TfAttnPlan* plan);
void plan_decode(const TfDecodeDesc& desc, int sm_count, TfDecodePlan* plan);

// Keys per chunk when the descriptor leaves kv_chunk at 0: 512, or 1024 for an 8-bit cache.
int default_kv_chunk(const TfDecodeDesc& desc);

// Which work-item counter word a launch of the two-tile kernel uses (one table
// per device).  The kernel's CTAs draw item numbers from the word, so two
// launches that may run at the same time must never share one:
//   * launches on one stream run one after the other, so a stream keeps one word
//     for its lifetime (eager());
//   * a launch recorded into a CUDA graph keeps its word for every replay, and
//     graphs recorded on one stream may later replay side by side, so every
//     captured launch gets a word of its own (captured()).
// Both return the word's index, or -1 when the table is full.
class QueueWords {
 public:
  static constexpr int kEagerWords = 256;
  static constexpr int kCapturedWords = 4096;
  static constexpr int kWords = kEagerWords + kCapturedWords;
  int eager(uintptr_t stream);
  int captured();

 private:
  std::mutex mutex_;
  uintptr_t streams_[kEagerWords] = {};
  int n_streams_ = 0;
  int n_captured_ = 0;
};

// Contiguous [begin, end) share of `total` units for `rank` of `world`; the
// first total % world ranks take one unit more.
void shard_range(int64_t total, int rank, int world, int64_t* begin, int64_t* end);

}  // namespace tfb
