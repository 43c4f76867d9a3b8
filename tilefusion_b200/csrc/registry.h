// Variant registry: picks tile shapes (prefill) and split counts (decode) per
// (sequence length, head_dim).  TileFusion bakes caller-supplied tile sizes
// into a kernel it JIT-compiles per exact shape (src/kernels/flash_attn.cu:16-55,
// src/jit/compiler.cc:123-145); here the variants are compiled ahead of time,
// sequence lengths are run-time arguments, and this table chooses among them.
// Host-only code: it has no CUDA dependency and is unit-tested without a GPU.
#pragma once

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

// Fills `plan` for `desc` on a GPU with `sm_count` SMs.  `desc` must have been
// validated by the caller.
void plan_attn(const TfAttnDesc& desc, int sm_count, TfAttnPlan* plan);
void plan_decode(const TfDecodeDesc& desc, int sm_count, TfDecodePlan* plan);

}  // namespace tfb
