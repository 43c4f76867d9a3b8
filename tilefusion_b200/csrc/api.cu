// C-ABI of the library (declared in include/tilefusion_b200.h): argument
// validation, the variant registry's launch side, TMA tensor-map construction
// and kernel launches.  Host-only planning logic lives in registry.cc.
//
// This is the single CUDA translation unit of the library; it includes the
// kernel headers so that the device status word has one definition.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "attn_fwd_sm100.cuh"
#include "attn_fwd_pair_sm100.cuh"
#include "attn_bwd_sm100.cuh"
#include "decode_sm100.cuh"
#include "fp8_sm100.cuh"
#include "internal.h"
#include "probe_sm100.cuh"
#include "registry.h"
#include "tilefusion_b200.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

constexpr int kMaxDevices = 64;

#define TF_CUDA_TRY(expr)                                                          \
  do {                                                                             \
    cudaError_t e__ = (expr);                                                      \
    if (e__ != cudaSuccess)                                                        \
      return fail(TF_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));   \
  } while (0)

// cuTensorMapEncodeTiled is fetched through the runtime so that the library
// does not link libcuda (it must load on machines without a driver).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault,
                                         &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Rank-4 tensor map over a 16-bit tensor: dims[0] is innermost (stride 1),
// strides_elems[i] is the stride of dims[i+1] in elements.
int encode_map(CUtensorMap* map, int dtype, const void* base, const uint64_t dims[4],
               const int64_t strides_elems[3], uint32_t box0, uint32_t box1, const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return fail(TF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdims[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstr[3];
  uint64_t packed = dims[0] * 2;
  for (int i = 0; i < 3; ++i) {
    // A dimension of extent 1 never advances; give it the packed stride so
    // that any caller-provided value (0 for an expanded view) is acceptable.
    uint64_t s = dims[i + 1] == 1 ? packed : (uint64_t)strides_elems[i] * 2;
    if (strides_elems[i] < 0 && dims[i + 1] != 1)
      return fail(TF_ERR_BAD_ARG, "%s: negative stride", what);
    if (s % 16 != 0 || s == 0)
      return fail(TF_ERR_UNSUPPORTED, "%s: stride of dim %d (%llu bytes) is not a positive multiple of 16 bytes",
                  what, i + 1, (unsigned long long)s);
    gstr[i] = s;
    packed = s * dims[i + 1];
  }
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
    return fail(TF_ERR_UNSUPPORTED, "%s: base pointer is not 16-byte aligned", what);
  cuuint32_t box[4] = {box0, box1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, dtype == TF_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  4, const_cast<void*>(base), gdims, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TF_ERR_CUDA, "%s: cuTensorMapEncodeTiled returned %d", what, (int)r);
  return TF_OK;
}

int check_attn_desc(const TfAttnDesc* d) {
  if (d == nullptr) return fail(TF_ERR_BAD_ARG, "desc is null");
  if (d->dtype != TF_F16 && d->dtype != TF_BF16)
    return fail(TF_ERR_UNSUPPORTED, "the inputs and output must be half-precision (fp16 or bf16); got dtype code %d", d->dtype);
  if (d->batch < 1 || d->heads < 1 || d->len_q < 1 || d->len_kv < 1)
    return fail(TF_ERR_BAD_ARG, "batch, heads, len_q and len_kv must be positive (got %d, %d, %d, %d)",
                d->batch, d->heads, d->len_q, d->len_kv);
  if (d->head_dim < 8 || d->head_dim > 256 || d->head_dim % 8 != 0 || d->head_dim_v < 8 || d->head_dim_v > 256 ||
      d->head_dim_v % 8 != 0)
    return fail(TF_ERR_UNSUPPORTED,
                "head_dim (%d) and head_dim_v (%d) must be multiples of 8 in [8, 256] (kernels are compiled for "
                "64, 128 and 256; other widths run zero-padded on the next one)", d->head_dim, d->head_dim_v);
  if (!(d->softmax_scale > 0.f) || !std::isfinite(d->softmax_scale))
    return fail(TF_ERR_UNSUPPORTED, "softmax_scale must be positive and finite");
  if (d->heads > 65535 || d->batch > 65535) return fail(TF_ERR_UNSUPPORTED, "batch and heads must each be <= 65535");
  if (d->k_stride_d != 1 && d->k_stride_l != 1)
    return fail(TF_ERR_UNSUPPORTED, "K must be contiguous along the head dim or along the key index");
  if (d->v_stride_d != 1 && d->v_stride_l != 1)
    return fail(TF_ERR_UNSUPPORTED, "V must be contiguous along the head dim or along the key index");
  if (d->o_stride_l % 8 != 0 || d->o_stride_h % 8 != 0 || d->o_stride_b % 8 != 0)
    return fail(TF_ERR_UNSUPPORTED, "O strides must be multiples of 8 elements (16-byte rows)");
  return TF_OK;
}

int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  return n;
}

// Tensor maps and kernel arguments shared by the prefill variants.
struct AttnLaunch {
  CUtensorMap mq, mk, mv;
  CUtensorMap mo;        // output map for the TMA-store epilogue; valid when has_mo
  bool has_mo = false;
  tfb::AttnFwdArgs args;
};

int prepare_attn(const void* q, const void* k, const void* v, void* o, float* lse, const TfAttnDesc* d,
                 const TfAttnPlan& plan, AttnLaunch* out) {
  // The tensor maps carry the true head dims; boxes are as wide as the kernel's
  // bucket, and TMA zero-fills (loads) or clips (stores) what lies beyond.
  const int D = d->head_dim, Dv = d->head_dim_v;
  const int bucket = plan.head_dim_kernel;
  const uint64_t B = d->batch, H = d->heads;
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)d->len_q, H, B};
    const int64_t str[3] = {d->q_stride_l, d->q_stride_h, d->q_stride_b};
    if (int rc = encode_map(&out->mq, d->dtype, q, dims, str, 64, tfb::kAttnTile, "Q")) return rc;
  }
  if (!plan.k_mn_major) {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)d->len_kv, H, B};
    const int64_t str[3] = {d->k_stride_l, d->k_stride_h, d->k_stride_b};
    if (int rc = encode_map(&out->mk, d->dtype, k, dims, str, 64, tfb::kAttnTile, "K")) return rc;
  } else {
    const uint64_t dims[4] = {(uint64_t)d->len_kv, (uint64_t)D, H, B};
    const int64_t str[3] = {d->k_stride_d, d->k_stride_h, d->k_stride_b};
    if (int rc = encode_map(&out->mk, d->dtype, k, dims, str, 64, bucket, "K (stored [D, Lk])")) return rc;
  }
  if (plan.v_mn_major) {
    const uint64_t dims[4] = {(uint64_t)Dv, (uint64_t)d->len_kv, H, B};
    const int64_t str[3] = {d->v_stride_l, d->v_stride_h, d->v_stride_b};
    if (int rc = encode_map(&out->mv, d->dtype, v, dims, str, 64, tfb::kAttnTile, "V")) return rc;
  } else {
    const uint64_t dims[4] = {(uint64_t)d->len_kv, (uint64_t)Dv, H, B};
    const int64_t str[3] = {d->v_stride_d, d->v_stride_h, d->v_stride_b};
    if (int rc = encode_map(&out->mv, d->dtype, v, dims, str, 64, bucket, "V (stored [Dv, Lk])")) return rc;
  }
  {
    // The output leaves through a TMA store when its layout can be described
    // by a tensor map (16-byte aligned base, positive strides); otherwise the
    // kernels fall back to per-row stores.
    const uint64_t dims[4] = {(uint64_t)Dv, (uint64_t)d->len_q, H, B};
    const int64_t str[3] = {d->o_stride_l, d->o_stride_h, d->o_stride_b};
    bool ok = reinterpret_cast<uintptr_t>(o) % 16 == 0;
    for (int i = 0; i < 3; ++i) ok = ok && (dims[i + 1] == 1 || (str[i] > 0 && str[i] % 8 == 0));
    out->has_mo = false;
    if (ok) {
      if (int rc = encode_map(&out->mo, d->dtype, o, dims, str, 64, tfb::kAttnTile, "O")) return rc;
      out->has_mo = true;
    } else {
      out->mo = out->mq;
    }
  }
  tfb::AttnFwdArgs& args = out->args;
  args.o = o;
  args.lse = lse;
  args.len_q = d->len_q;
  args.len_kv = d->len_kv;
  args.dim_v = Dv;
  args.causal = d->causal ? 1 : 0;
  args.k_mn_major = plan.k_mn_major;
  args.v_mn_major = plan.v_mn_major;
  args.scale_log2 = d->softmax_scale * 1.4426950408889634f;
  args.o_stride_b = d->o_stride_b;
  args.o_stride_h = d->o_stride_h;
  args.o_stride_l = d->o_stride_l;
  args.lse_stride_b = (long long)d->heads * d->len_q;
  args.lse_stride_h = d->len_q;
  return TF_OK;
}

// One 128-row Q tile per CTA, two CTAs per SM.
template <typename T, int D>
int launch_attn(const AttnLaunch& L, const TfAttnDesc* d, cudaStream_t stream) {
  using Smem = tfb::AttnSmem<D>;
  auto kern = tfb::attn_fwd_kernel<T, D>;
  static thread_local int configured_device = -1;
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    TF_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
    configured_device = dev;
  }
  const int n_q_tiles = (d->len_q + tfb::kAttnTile - 1) / tfb::kAttnTile;
  dim3 grid(n_q_tiles, d->heads, d->batch);
  kern<<<grid, tfb::kAttnThreads, Smem::kBytes, stream>>>(L.mq, L.mk, L.mv, L.args);
  TF_CUDA_TRY(cudaGetLastError());
  return TF_OK;
}

// fused_two_gemms: the one-tile kernel with the softmax stage replaced by a cast.
template <typename T, int D>
int launch_two_gemms(const AttnLaunch& L, const TfAttnDesc* d, cudaStream_t stream) {
  using Smem = tfb::AttnSmem<D>;
  auto kern = tfb::attn_fwd_kernel<T, D, true>;
  static thread_local int configured_device = -1;
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    TF_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
    configured_device = dev;
  }
  dim3 grid((d->len_q + tfb::kAttnTile - 1) / tfb::kAttnTile, 1, 1);
  kern<<<grid, tfb::kAttnThreads, Smem::kBytes, stream>>>(L.mq, L.mk, L.mv, L.args);
  TF_CUDA_TRY(cudaGetLastError());
  return TF_OK;
}

// Item counters of the two-tile kernel.  A launch zeroes one of these words on
// its stream and hands it to the kernel, whose CTAs draw their work items from
// it.  tfb::QueueWords (registry.h) decides which word: one per stream for
// eager launches, a fresh one for every launch recorded into a CUDA graph.
static __device__ int g_pair_queue[tfb::QueueWords::kWords];

struct PairQueues {
  tfb::QueueWords words;
  std::mutex mutex;
  int* base = nullptr;      // device address of g_pair_queue on this device
};
PairQueues g_pair_queues[kMaxDevices];

int pair_queue_word(cudaStream_t stream, int** out) {
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(TF_ERR_UNSUPPORTED, "device index %d is out of range", dev);
  PairQueues& q = g_pair_queues[dev];
  {
    std::lock_guard<std::mutex> lock(q.mutex);
    if (q.base == nullptr) {
      void* p = nullptr;
      TF_CUDA_TRY(cudaGetSymbolAddress(&p, g_pair_queue));
      q.base = static_cast<int*>(p);
    }
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  TF_CUDA_TRY(cudaStreamIsCapturing(stream, &cap));
  const bool capturing = cap == cudaStreamCaptureStatusActive;
  const int idx = capturing ? q.words.captured() : q.words.eager(reinterpret_cast<uintptr_t>(stream));
  if (idx < 0)
    return fail(TF_ERR_UNSUPPORTED,
                capturing ? "more than %d launches of the two-tile kernel have been recorded into CUDA graphs on this device"
                          : "more than %d streams have launched the two-tile kernel on this device",
                capturing ? tfb::QueueWords::kCapturedWords : tfb::QueueWords::kEagerWords);
  *out = q.base + idx;
  return TF_OK;
}

// Two Q tiles per CTA, persistent grid of one CTA per SM.
// kRepl: split-KV mode with the (at most 32) query rows replicated in the four lane quarters of Q
// tile 0 (the Q tensor map's box is then 32 rows high); every (row, split) has four partial rows.
template <typename T, int D, bool kRepl = false>
int launch_attn_pair(const AttnLaunch& L, const TfAttnDesc* d, const TfAttnPlan& plan, cudaStream_t stream,
                     int kv_splits = 0, int tiles_per_split = 0, float* part_o = nullptr,
                     float* part_ml = nullptr, const int* block_table = nullptr, int page_size = 0,
                     int max_pages = 0) {
  using Smem = tfb::AttnPairSmem<D>;
  auto kern = tfb::attn_fwd_pair_kernel<T, D, kRepl>;
  static thread_local int configured_device = -1;
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    TF_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
    configured_device = dev;
  }
  tfb::AttnPairArgs a;
  a.base = L.args;
  a.heads = d->heads;
  a.batch = d->batch;
  a.n_pairs = (d->len_q + 2 * tfb::kAttnTile - 1) / (2 * tfb::kAttnTile);
  a.n_items = d->batch * d->heads * a.n_pairs * (kv_splits > 0 ? kv_splits : 1);
  a.tma_store = (kv_splits == 0 && L.has_mo) ? 1 : 0;
  {
    // Causal item order: equal blocks of (batch, head) slices whose K and V
    // together take about half of the 126 MB L2, and which hold at least one
    // item per CTA.  Measured on B8 H32 L2048 (1 MB of K+V per slice): blocks
    // of 16 / 40 / 64 / 128 / 256 slices give 772 / 820 / 853 / 796 / 777
    // TFLOP/s; on B16 H64 L8192 (4 MB per slice) 5 / 10 / 20 / 80 slices give
    // 1036 / 1027 / 1002 / 968.
    const long long n_bh = (long long)d->batch * d->heads;
    const long long kv_bytes_per_head = 2ll * d->len_kv * D * 2;
    long long fit = (64ll << 20) / std::max(1ll, kv_bytes_per_head);
    fit = std::max(fit, ((long long)plan.grid + a.n_pairs - 1) / a.n_pairs);
    fit = std::min(std::max(1ll, fit), n_bh);
    const long long n_blocks = std::max(1ll, (n_bh + fit / 2) / fit);
    a.causal_block = (int)((n_bh + n_blocks - 1) / n_blocks);
  }
  if (int rc = pair_queue_word(stream, &a.queue)) return rc;
  TF_CUDA_TRY(cudaMemsetAsync(a.queue, 0, sizeof(int), stream));
  a.kv_splits = kv_splits;
  a.tiles_per_split = tiles_per_split;
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.block_table = block_table;
  a.page_size = page_size;
  a.max_pages = max_pages;
  kern<<<kv_splits > 0 ? std::min(plan.grid, a.n_items) : plan.grid, tfb::kPairThreads, Smem::kBytes, stream>>>(L.mq, L.mk, L.mv, L.mo, a);
  TF_CUDA_TRY(cudaGetLastError());
  return TF_OK;
}

template <typename T, int D>
int run_attn(const void* q, const void* k, const void* v, void* o, float* lse, const TfAttnDesc* d,
             const TfAttnPlan& plan, cudaStream_t stream) {
  AttnLaunch L;
  if (int rc = prepare_attn(q, k, v, o, lse, d, plan, &L)) return rc;
  if constexpr (D <= 128) {
    if (plan.tile_q == 256) return launch_attn_pair<T, D>(L, d, plan, stream);
  }
  return launch_attn<T, D>(L, d, stream);
}

// Backward: delta rows, then the dK/dV kernel (items = live key tiles) and the dQ
// kernel (items = query tiles), each on a persistent grid of at most one CTA per
// SM that walks its items in a fixed order.
template <typename T, int D>
int launch_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                    void* dq, void* dk, void* dv, float* delta, const TfAttnDesc* d, cudaStream_t stream) {
  using Smem = tfb::AttnBwdSmem<D>;
  const uint64_t B = d->batch, H = d->heads;
  CUtensorMap mq, mk, mv, mdo;
  {
    const uint64_t dq_dims[4] = {(uint64_t)D, (uint64_t)d->len_q, H, B};
    const uint64_t dk_dims[4] = {(uint64_t)D, (uint64_t)d->len_kv, H, B};
    const int64_t qs[3] = {d->q_stride_l, d->q_stride_h, d->q_stride_b};
    const int64_t ks[3] = {d->k_stride_l, d->k_stride_h, d->k_stride_b};
    const int64_t vs[3] = {d->v_stride_l, d->v_stride_h, d->v_stride_b};
    const int64_t os[3] = {d->o_stride_l, d->o_stride_h, d->o_stride_b};
    if (int rc = encode_map(&mq, d->dtype, q, dq_dims, qs, 64, tfb::kAttnTile, "Q")) return rc;
    if (int rc = encode_map(&mk, d->dtype, k, dk_dims, ks, 64, tfb::kAttnTile, "K")) return rc;
    if (int rc = encode_map(&mv, d->dtype, v, dk_dims, vs, 64, tfb::kAttnTile, "V")) return rc;
    if (int rc = encode_map(&mdo, d->dtype, d_o, dq_dims, os, 64, tfb::kAttnTile, "dO")) return rc;
  }
  const long long rows = (long long)B * H * d->len_q;
  tfb::AttnBwdDeltaArgs da;
  da.o = o;
  da.d_o = d_o;
  da.delta = delta;
  da.len_q = d->len_q;
  da.heads = d->heads;
  da.rows = rows;
  da.o_stride_b = da.do_stride_b = d->o_stride_b;
  da.o_stride_h = da.do_stride_h = d->o_stride_h;
  da.o_stride_l = da.do_stride_l = d->o_stride_l;
  constexpr int kDeltaRows = tfb::BwdDeltaShape<D>::kRowsPerBlock;
  tfb::attn_bwd_delta_kernel<T, D><<<(unsigned)((rows + kDeltaRows - 1) / kDeltaRows), tfb::kBwdDeltaThreads, 0, stream>>>(da);
  TF_CUDA_TRY(cudaGetLastError());

  tfb::AttnBwdArgs a;
  a.lse = lse;
  a.delta = delta;
  a.dq = dq;
  a.dk = dk;
  a.dv = dv;
  a.len_q = d->len_q;
  a.len_kv = d->len_kv;
  a.causal = d->causal ? 1 : 0;
  a.scale = d->softmax_scale;
  a.scale_log2 = d->softmax_scale * 1.4426950408889634f;
  a.dq_stride_b = d->q_stride_b;
  a.dq_stride_h = d->q_stride_h;
  a.dq_stride_l = d->q_stride_l;
  a.dk_stride_b = d->k_stride_b;
  a.dk_stride_h = d->k_stride_h;
  a.dk_stride_l = d->k_stride_l;
  a.dv_stride_b = d->v_stride_b;
  a.dv_stride_h = d->v_stride_h;
  a.dv_stride_l = d->v_stride_l;
  a.row_stride_b = (long long)d->heads * d->len_q;
  a.row_stride_h = d->len_q;
  a.heads = d->heads;
  a.batch = d->batch;
  auto dkv = tfb::attn_bwd_kernel<T, D, true>;
  auto dqk = tfb::attn_bwd_kernel<T, D, false>;
  static thread_local int configured_device = -1;
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    TF_CUDA_TRY(cudaFuncSetAttribute(dkv, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
    TF_CUDA_TRY(cudaFuncSetAttribute(dqk, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
    configured_device = dev;
  }
  const int n_q_tiles = (d->len_q + tfb::kAttnTile - 1) / tfb::kAttnTile;
  const int n_kv_tiles = (d->len_kv + tfb::kAttnTile - 1) / tfb::kAttnTile;
  // persistent: one CTA per SM (or per work item when there are fewer); the kernels walk the items
  const long long bh = (long long)d->heads * d->batch;
  const int live_kv_tiles = d->causal ? std::min(n_kv_tiles, n_q_tiles) : n_kv_tiles;
  const int sms = sm_count();
  const int grid_dkv = (int)std::max<long long>(1, std::min<long long>((long long)live_kv_tiles * bh, sms));
  const int grid_dq = (int)std::max<long long>(1, std::min<long long>((long long)n_q_tiles * bh, sms));
  dkv<<<grid_dkv, tfb::kBwdThreads, Smem::kBytes, stream>>>(mq, mk, mv, mdo, a);
  TF_CUDA_TRY(cudaGetLastError());
  dqk<<<grid_dq, tfb::kBwdThreads, Smem::kBytes, stream>>>(mq, mk, mv, mdo, a);
  TF_CUDA_TRY(cudaGetLastError());
  return TF_OK;
}

bool kv_is_fp8(const TfDecodeDesc* d) { return d->kv_dtype == TF_FP8_E4M3 || d->kv_dtype == TF_FP8_E5M2; }

int check_decode_desc(const TfDecodeDesc* d) {
  if (d == nullptr) return fail(TF_ERR_BAD_ARG, "desc is null");
  if (d->dtype != TF_F16 && d->dtype != TF_BF16)
    return fail(TF_ERR_UNSUPPORTED, "the inputs and output must be half-precision (fp16 or bf16); got dtype code %d", d->dtype);
  if (d->batch < 1 || d->heads < 1 || d->len_kv < 0)
    return fail(TF_ERR_BAD_ARG, "batch and heads must be positive and len_kv non-negative (got %d, %d, %d)",
                d->batch, d->heads, d->len_kv);
  if (d->head_dim != 64 && d->head_dim != 128)
    return fail(TF_ERR_UNSUPPORTED, "head_dim %d has no compiled variant (64 and 128 do)", d->head_dim);
  if (!(d->softmax_scale > 0.f) || !std::isfinite(d->softmax_scale))
    return fail(TF_ERR_UNSUPPORTED, "softmax_scale must be positive and finite");
  const int chunk = d->kv_chunk == 0 ? tfb::default_kv_chunk(*d) : d->kv_chunk;
  if (chunk < 128 || chunk % 128 != 0 || chunk > tfb::kDecMaxChunk)
    return fail(TF_ERR_UNSUPPORTED, "kv_chunk must be a multiple of 128 in [128, %d] (got %d)", tfb::kDecMaxChunk, chunk);
  if (d->num_splits < 0) return fail(TF_ERR_BAD_ARG, "num_splits must be >= 0");
  if (d->heads_kv < 0 || (d->heads_kv > 0 && d->heads % d->heads_kv != 0))
    return fail(TF_ERR_BAD_ARG, "heads (%d) must be a multiple of heads_kv (%d)", d->heads, d->heads_kv);
  if (d->heads_kv > 0 && d->heads / d->heads_kv > 128)
    return fail(TF_ERR_UNSUPPORTED, "at most 128 query heads per KV head");
  if (d->page_size != 0) {
    if (d->page_size < 128 || d->page_size % 128 != 0)
      return fail(TF_ERR_UNSUPPORTED, "page_size must be a multiple of 128 keys (got %d)", d->page_size);
    if (d->block_table == nullptr) return fail(TF_ERR_BAD_ARG, "block_table is null although page_size > 0");
    if ((int64_t)d->max_pages * d->page_size < d->len_kv)
      return fail(TF_ERR_BAD_ARG, "block_table rows (%d pages of %d keys) do not cover len_kv %d", d->max_pages,
                  d->page_size, d->len_kv);
    if (d->num_pages < 1) return fail(TF_ERR_BAD_ARG, "num_pages must be positive for a paged cache");
    if (d->k_stride_page % 8 != 0 || d->v_stride_page % 8 != 0 || d->k_stride_page <= 0 || d->v_stride_page <= 0)
      return fail(TF_ERR_UNSUPPORTED, "page strides must be positive multiples of 8 elements (16 bytes)");
  }
  const int64_t s[] = {d->q_stride_b, d->q_stride_h, d->k_stride_b, d->k_stride_h,
                       d->v_stride_b, d->v_stride_h};
  for (int64_t x : s)
    if (x % 8 != 0 || x < 0) return fail(TF_ERR_UNSUPPORTED, "Q/K/V strides must be non-negative multiples of 8 elements (16 bytes)");
  if (d->kv_dtype != 0 && d->kv_dtype != d->dtype && !kv_is_fp8(d))
    return fail(TF_ERR_UNSUPPORTED, "kv_dtype must be 0, equal to dtype, TF_FP8_E4M3 or TF_FP8_E5M2 (got %d)", d->kv_dtype);
  if (kv_is_fp8(d)) {
    const int64_t kv[] = {d->k_stride_b, d->k_stride_h, d->v_stride_b, d->v_stride_h,
                          d->page_size != 0 ? d->k_stride_page : 0, d->page_size != 0 ? d->v_stride_page : 0};
    for (int64_t x : kv)
      if (x % 16 != 0) return fail(TF_ERR_UNSUPPORTED, "strides of an 8-bit K/V cache must be multiples of 16 elements (16 bytes)");
  }
  const float scales[] = {d->k_scale, d->v_scale};
  for (float x : scales)
    if (x != 0.f && (!(x > 0.f) || !std::isfinite(x)))
      return fail(TF_ERR_BAD_ARG, "k_scale and v_scale must be positive and finite (0 stands for 1)");
  return TF_OK;
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// KV: the stored K/V element (T itself, or an 8-bit tag).  Two CTAs share an SM;
// a CTA's ring is three stages of 256 * D bytes (128 keys of a 16-bit cache, 256
// of an 8-bit one).
template <typename T, typename KV, int D>
int launch_decode_split(const void* q, const void* k, const void* v, float* part_o, float* part_ml,
                        const TfDecodeDesc* d, const TfDecodePlan& plan, cudaStream_t stream,
                        const tfb::DecodeFuseArgs* fuse = nullptr) {
  constexpr int kKvBytes = tfb::KvBytes<KV>::value;
  constexpr int kStages = 3;
  using Smem = tfb::DecodeSmem<D, kStages, kKvBytes>;
  tfb::DecodeSplitArgs a;
  a.fuse = fuse != nullptr ? *fuse : tfb::DecodeFuseArgs{};
  a.q = q;
  a.k = k;
  a.v = v;
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.heads = d->heads;
  a.group = (d->heads_kv > 0 && d->heads_kv != d->heads) ? d->heads / d->heads_kv : 1;
  a.len_kv = d->len_kv;
  a.kv_chunk = plan.kv_chunk;
  a.num_splits = plan.num_splits;
  a.chunks_per_split = plan.chunks_per_split;
  a.items = d->batch * d->heads * plan.num_splits;
  a.scale_log2 = d->softmax_scale * 1.4426950408889634f * (d->k_scale != 0.f ? d->k_scale : 1.f);
  a.v_scale = d->v_scale != 0.f ? d->v_scale : 1.f;
  a.q_stride_b = d->q_stride_b;
  a.q_stride_h = d->q_stride_h;
  a.k_stride_b = d->k_stride_b;
  a.k_stride_h = d->k_stride_h;
  a.v_stride_b = d->v_stride_b;
  a.v_stride_h = d->v_stride_h;
  a.block_table = d->page_size > 0 ? d->block_table : nullptr;
  a.page_size = d->page_size;
  a.max_pages = d->max_pages;
  a.k_stride_page = d->k_stride_page;
  a.v_stride_page = d->v_stride_page;
  auto kern = tfb::decode_split_kernel<T, KV, D, kStages>;
  static thread_local int configured_device = -1;
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    TF_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
    configured_device = dev;
  }
  const int grid = plan.grid < a.items ? plan.grid : a.items;
  kern<<<grid, tfb::kDecThreads, Smem::kBytes, stream>>>(a);
  TF_CUDA_TRY(cudaGetLastError());
  return TF_OK;
}

template <typename T, int D>
int launch_combine(const tfb::DecodeCombineArgs& a, int rows, cudaStream_t stream) {
  dim3 block(D, tfb::kCombineGroups);
  tfb::decode_combine_kernel<T, D><<<rows, block, 0, stream>>>(a);
  TF_CUDA_TRY(cudaGetLastError());
  return TF_OK;
}

int dispatch_combine(const tfb::DecodeCombineArgs& a, int rows, int head_dim, int dtype, cudaStream_t stream) {
  if (head_dim == 128)
    return dtype == TF_F16 ? launch_combine<__half, 128>(a, rows, stream)
                           : launch_combine<__nv_bfloat16, 128>(a, rows, stream);
  if (head_dim == 64)
    return dtype == TF_F16 ? launch_combine<__half, 64>(a, rows, stream)
                           : launch_combine<__nv_bfloat16, 64>(a, rows, stream);
  return fail(TF_ERR_UNSUPPORTED, "head_dim %d has no compiled variant (64 and 128 do)", head_dim);
}

// Grouped-query decoding: the query heads that share a KV head become the rows
// of one attention problem per (batch, KV head), run by the two-tile kernel in
// split-KV mode (tensor cores; K/V streamed once through its TMA ring).
int launch_gqa_split(const void* q, const void* k, const void* v, float* part_o, float* part_ml,
                     const TfDecodeDesc* d, const TfDecodePlan& plan, cudaStream_t stream) {
  if (d->len_kv < 1) return fail(TF_ERR_UNSUPPORTED, "grouped-query decoding needs at least one key per call");
  const int group = d->heads / d->heads_kv;
  const int D = d->head_dim;
  TfAttnDesc ad{};
  ad.dtype = d->dtype;
  ad.batch = d->batch;
  ad.heads = d->heads_kv;
  ad.len_q = group;
  ad.len_kv = d->len_kv;
  ad.head_dim = ad.head_dim_v = D;
  ad.softmax_scale = d->softmax_scale;
  ad.tile_q = 256;
  ad.tile_kv = 128;
  ad.q_stride_b = d->q_stride_b;
  ad.q_stride_h = (int64_t)group * d->q_stride_h;
  ad.q_stride_l = d->q_stride_h;
  // (with a paged cache the batch strides are placeholders: the K and V maps
  // are rebuilt over the page pool below)
  ad.k_stride_b = d->page_size > 0 ? d->k_stride_page : d->k_stride_b;
  ad.k_stride_h = d->k_stride_h;
  ad.k_stride_l = D;
  ad.k_stride_d = 1;
  ad.v_stride_b = d->page_size > 0 ? d->v_stride_page : d->v_stride_b;
  ad.v_stride_h = d->v_stride_h;
  ad.v_stride_l = D;
  ad.v_stride_d = 1;
  ad.o_stride_l = D;      // unused in split-KV mode
  TfAttnPlan ap;
  tfb::plan_attn(ad, sm_count(), &ap);
  ap.grid = plan.grid;
  AttnLaunch L;
  if (int rc = prepare_attn(q, k, v, part_o, nullptr, &ad, ap, &L)) return rc;
  if (d->page_size > 0) {
    // K and V maps over the page pool: (D, page_size, H_kv, num_pages)
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)d->page_size, (uint64_t)d->heads_kv, (uint64_t)d->num_pages};
    const int64_t ks[3] = {D, d->k_stride_h, d->k_stride_page};
    const int64_t vs[3] = {D, d->v_stride_h, d->v_stride_page};
    if (int rc = encode_map(&L.mk, d->dtype, k, dims, ks, 64, tfb::kAttnTile, "K pages")) return rc;
    if (int rc = encode_map(&L.mv, d->dtype, v, dims, vs, 64, tfb::kAttnTile, "V pages")) return rc;
  }
  const int* table = d->page_size > 0 ? d->block_table : nullptr;
  // plan.reserved: partial rows per (row, split) -- 4 when the query rows of a group are replicated
  // in the four lane quarters (at most 32 query heads per KV head), else 1
  const int copies = plan.reserved == 4 ? 4 : 1;
  const int kv_splits = plan.num_splits / copies;
  if (copies == 4) {
    // Q map with a 32-row box: the group's rows are loaded once per lane quarter
    const uint64_t qdims[4] = {(uint64_t)D, (uint64_t)group, (uint64_t)d->heads_kv, (uint64_t)d->batch};
    const int64_t qstr[3] = {ad.q_stride_l, ad.q_stride_h, ad.q_stride_b};
    if (int rc = encode_map(&L.mq, d->dtype, q, qdims, qstr, 64, 32, "Q (grouped)")) return rc;
    if (D == 128)
      return d->dtype == TF_F16
                 ? launch_attn_pair<__half, 128, true>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages)
                 : launch_attn_pair<__nv_bfloat16, 128, true>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages);
    return d->dtype == TF_F16
               ? launch_attn_pair<__half, 64, true>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages)
               : launch_attn_pair<__nv_bfloat16, 64, true>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages);
  }
  if (D == 128)
    return d->dtype == TF_F16
               ? launch_attn_pair<__half, 128>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages)
               : launch_attn_pair<__nv_bfloat16, 128>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages);
  return d->dtype == TF_F16
             ? launch_attn_pair<__half, 64>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages)
             : launch_attn_pair<__nv_bfloat16, 64>(L, &ad, ap, stream, kv_splits, plan.chunks_per_split, part_o, part_ml, table, d->page_size, d->max_pages);
}

// Grouped-query heads over a 16-bit cache run on the two-tile (tensor-core) kernel.  Over an 8-bit
// cache they run on the split kernel, one work item per query head and split: each query head of a
// group streams its KV head's chunks itself (the re-reads within a group meet in L2).
bool is_grouped(const TfDecodeDesc* d) { return d->heads_kv > 0 && d->heads_kv != d->heads && !kv_is_fp8(d); }

// KvTag: an 8-bit storage tag, or void for a cache stored in the query's type.
template <typename KvTag>
int dispatch_split_kv(const void* q, const void* k, const void* v, float* part_o, float* part_ml,
                      const TfDecodeDesc* d, const TfDecodePlan& plan, cudaStream_t stream,
                      const tfb::DecodeFuseArgs* fuse) {
  using KvH = std::conditional_t<std::is_void<KvTag>::value, __half, KvTag>;
  using KvB = std::conditional_t<std::is_void<KvTag>::value, __nv_bfloat16, KvTag>;
  if (d->head_dim == 128)
    return d->dtype == TF_F16 ? launch_decode_split<__half, KvH, 128>(q, k, v, part_o, part_ml, d, plan, stream, fuse)
                              : launch_decode_split<__nv_bfloat16, KvB, 128>(q, k, v, part_o, part_ml, d, plan, stream, fuse);
  return d->dtype == TF_F16 ? launch_decode_split<__half, KvH, 64>(q, k, v, part_o, part_ml, d, plan, stream, fuse)
                            : launch_decode_split<__nv_bfloat16, KvB, 64>(q, k, v, part_o, part_ml, d, plan, stream, fuse);
}

// `fuse` (one query head per KV head only): merge, exchange and final combine in the same launch.
int dispatch_split(const void* q, const void* k, const void* v, float* part_o, float* part_ml,
                   const TfDecodeDesc* d, const TfDecodePlan& plan, cudaStream_t stream,
                   const tfb::DecodeFuseArgs* fuse = nullptr) {
  if (is_grouped(d)) return launch_gqa_split(q, k, v, part_o, part_ml, d, plan, stream);
  if (d->kv_dtype == TF_FP8_E4M3) return dispatch_split_kv<tfb::Fp8E4M3>(q, k, v, part_o, part_ml, d, plan, stream, fuse);
  if (d->kv_dtype == TF_FP8_E5M2) return dispatch_split_kv<tfb::Fp8E5M2>(q, k, v, part_o, part_ml, d, plan, stream, fuse);
  return dispatch_split_kv<void>(q, k, v, part_o, part_ml, d, plan, stream, fuse);
}

int plan_and_check_decode(const void* q, const void* k, const void* v, const void* workspace,
                          uint64_t workspace_bytes, const TfDecodeDesc* d, TfDecodePlan* plan) {
  if (int rc = check_decode_desc(d)) return rc;
  if (q == nullptr || (d->len_kv > 0 && (k == nullptr || v == nullptr)) || workspace == nullptr)
    return fail(TF_ERR_BAD_ARG, "q, k, v and workspace must be non-null");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(workspace))
    return fail(TF_ERR_UNSUPPORTED, "q, k, v and workspace must be 16-byte aligned");
  tfb::plan_decode(*d, sm_count(), plan);
  if (workspace_bytes < plan->workspace_bytes)
    return fail(TF_ERR_WORKSPACE, "workspace holds %llu bytes but %llu are needed",
                (unsigned long long)workspace_bytes, (unsigned long long)plan->workspace_bytes);
  return tfb::ensure_device_ready();
}

// ---- scratch for tf_decode_static -------------------------------------------
// Partial rows of the no-allocation decode entry point live here instead of in
// a caller-provided workspace.  Every GPU that loads the library holds these
// 4 MiB until the process exits.  In host code the name below is only a
// stand-in for the symbol; the device address is looked up once per device.
constexpr uint64_t kStaticScratchBytes = 4ull << 20;
static __device__ __align__(256) float g_decode_scratch[kStaticScratchBytes / sizeof(float)];

std::mutex g_scratch_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of g_decode_scratch on the current device (looked up on the
// first call for that device, with that device current).
int static_scratch(float** out) {
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(TF_ERR_UNSUPPORTED, "device index %d is out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(TF_ERR_CUDA, "cudaGetSymbolAddress(g_decode_scratch) failed: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return TF_OK;
}


// ---- per-device state shared by the entry points ----------------------------
struct DeviceState {
  bool ready = false;
  int* mirror_host = nullptr;                 // mapped host copy of the device status word
  unsigned long long limit_applied_ns = 0;    // value of g_wait_limit_ns on the device
};
std::mutex g_device_mutex;
DeviceState g_device[kMaxDevices];
std::atomic<unsigned long long> g_wait_limit_ns_host{2000000000ull};

}  // namespace

namespace tfb {

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int ensure_device_ready() {
  int dev = 0;
  TF_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(TF_ERR_UNSUPPORTED, "device index %d is out of range", dev);
  const unsigned long long limit = g_wait_limit_ns_host.load(std::memory_order_relaxed);
  static thread_local int ready_device = -1;
  static thread_local unsigned long long ready_limit = 0;
  if (ready_device == dev && ready_limit == limit) return TF_OK;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  DeviceState& st = g_device[dev];
  if (!st.ready) {
    // One mapped host word per device: a device-side wait that gives up stores its
    // code there too, so the host can see a failed launch without synchronising.
    void* host = nullptr;
    TF_CUDA_TRY(cudaHostAlloc(&host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
    *static_cast<volatile int*>(host) = 0;
    void* mapped = nullptr;
    TF_CUDA_TRY(cudaHostGetDevicePointer(&mapped, host, 0));
    TF_CUDA_TRY(cudaMemcpyToSymbol(tfb::g_status_mirror, &mapped, sizeof(mapped)));
    st.mirror_host = static_cast<int*>(host);
    st.limit_applied_ns = 2000000000ull;
    st.ready = true;
  }
  if (st.limit_applied_ns != limit) {
    TF_CUDA_TRY(cudaMemcpyToSymbol(tfb::g_wait_limit_ns, &limit, sizeof(limit)));
    st.limit_applied_ns = limit;
  }
  ready_device = dev;
  ready_limit = limit;
  return TF_OK;
}

int launch_sharded_decode(const void* q, const void* k, const void* v, void* o, float* lse,
                          const TfDecodeDesc* d, const ShardStep& st, cudaStream_t stream) {
  TfDecodePlan plan;
  if (int rc = plan_and_check_decode(q, k, v, st.workspace, st.workspace_bytes, d, &plan)) return rc;
  // (the item flags of the fused tail follow the partial rows in the workspace)
  const uint64_t ws_need = plan.workspace_bytes + (uint64_t)d->batch * d->heads * plan.num_splits * sizeof(unsigned);
  if (st.workspace_bytes < ws_need)
    return fail(TF_ERR_WORKSPACE, "workspace holds %llu bytes but %llu are needed", (unsigned long long)st.workspace_bytes,
                (unsigned long long)ws_need);
  const bool p2p = st.peer_table != nullptr;
  if (p2p && o == nullptr) return fail(TF_ERR_BAD_ARG, "o is null");
  if (int rc = ensure_device_ready()) return rc;
  const int rows = d->batch * d->heads;
  const int D = d->head_dim;
  const long long slot_floats = (long long)rows * (D + 2);
  const long long my_slot = st.area_offset + (long long)st.rank * slot_floats;
  float* part_o = static_cast<float*>(st.workspace);
  float* part_ml = part_o + (int64_t)rows * plan.num_splits * D;
  const unsigned* local_flags = reinterpret_cast<const unsigned*>(st.local_base + st.flag_offset);
  if (!is_grouped(d)) {
    // one launch: split, merge, exchange, final combine
    DecodeFuseArgs f{};
    f.item_flags = reinterpret_cast<unsigned*>(static_cast<char*>(st.workspace) + plan.workspace_bytes);
    f.rows_done = st.rows_done;
    f.rows = rows;
    f.peer_bases = st.peer_table;
    f.out_slot = st.local_base + my_slot;
    f.n_peers = st.n_ranks;
    f.my_rank = st.rank;
    f.slot_offset = my_slot;
    f.flag_offset = st.flag_offset;
    f.step = st.step;
    f.final_phase = p2p ? 1 : 0;
    f.local_area = st.local_base + st.area_offset;
    f.local_flags = local_flags;
    f.o = o;
    f.o_stride_b = d->o_stride_b;
    f.o_stride_h = d->o_stride_h;
    f.lse = lse;
    return dispatch_split(q, k, v, part_o, part_ml, d, plan, stream, &f);
  }
  // grouped-query heads run on the two-tile kernel, which has no fused tail:
  // split pass, merge (+ scatter to the peers), then the combine behind the flags
  if (int rc = dispatch_split(q, k, v, part_o, part_ml, d, plan, stream)) return rc;
  DecodeCombineArgs a{};
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.n_parts = plan.num_splits;
  a.part_stride_o = D;
  a.row_stride_o = (int64_t)plan.num_splits * D;
  a.part_stride_ml = 2;
  a.row_stride_ml = (int64_t)plan.num_splits * 2;
  a.heads = d->heads;
  if (p2p) {
    a.peer_bases = st.peer_table;
    a.n_peers = st.n_ranks;
    a.my_rank = st.rank;
    a.rows_total = rows;
    a.scatter_offset = my_slot;
    a.flag_offset = st.flag_offset;
    a.step = st.step;
  } else {
    a.out_part_o = st.local_base + my_slot;
    a.out_part_ml = a.out_part_o + (long long)rows * D;
  }
  if (int rc = dispatch_combine(a, rows, D, d->dtype, stream)) return rc;
  if (!p2p) return TF_OK;
  return tf_decode_gathered_wait(st.local_base + st.area_offset, local_flags, st.n_ranks, st.step, d->batch,
                                 d->heads, D, d->dtype, o, d->o_stride_b, d->o_stride_h, lse, stream);
}

}  // namespace tfb

namespace {

// Bulk conversion between a 16-bit tensor and 8-bit storage (both directions).
template <typename T, bool kE4M3>
int launch_convert_fp8(const void* src, void* dst, int64_t n, float factor, cudaStream_t stream, bool to_fp8) {
  const int64_t n_vec = n / tfb::kFp8ElemsPerThread;
  const int64_t want = std::max<int64_t>(1, (n_vec + tfb::kFp8ConvertThreads - 1) / tfb::kFp8ConvertThreads);
  const int grid = (int)std::min<int64_t>(want, (int64_t)sm_count() * 8);
  if (to_fp8)
    tfb::fp8_quantize_kernel<T, kE4M3><<<grid, tfb::kFp8ConvertThreads, 0, stream>>>(
        static_cast<const T*>(src), static_cast<uint8_t*>(dst), n, factor);
  else
    tfb::fp8_dequantize_kernel<T, kE4M3><<<grid, tfb::kFp8ConvertThreads, 0, stream>>>(
        static_cast<const uint8_t*>(src), static_cast<T*>(dst), n, factor);
  TF_CUDA_TRY(cudaGetLastError());
  return TF_OK;
}

int convert_fp8(const void* src, void* dst, int64_t n, int32_t wide_dtype, int32_t fp8_dtype, float factor,
                void* stream, bool to_fp8) {
  if (n < 0) return fail(TF_ERR_BAD_ARG, "n must be non-negative (got %lld)", (long long)n);
  if (wide_dtype != TF_F16 && wide_dtype != TF_BF16)
    return fail(TF_ERR_UNSUPPORTED, "the 16-bit side must be TF_F16 or TF_BF16 (got %d)", wide_dtype);
  if (fp8_dtype != TF_FP8_E4M3 && fp8_dtype != TF_FP8_E5M2)
    return fail(TF_ERR_UNSUPPORTED, "the 8-bit side must be TF_FP8_E4M3 or TF_FP8_E5M2 (got %d)", fp8_dtype);
  if (!(factor > 0.f) || !std::isfinite(factor)) return fail(TF_ERR_BAD_ARG, "factor must be positive and finite");
  if (n == 0) return TF_OK;
  if (src == nullptr || dst == nullptr) return fail(TF_ERR_BAD_ARG, "src and dst must be non-null");
  if (!aligned16(src) || !aligned16(dst)) return fail(TF_ERR_UNSUPPORTED, "src and dst must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool e4 = fp8_dtype == TF_FP8_E4M3;
  if (wide_dtype == TF_F16)
    return e4 ? launch_convert_fp8<__half, true>(src, dst, n, factor, st, to_fp8)
              : launch_convert_fp8<__half, false>(src, dst, n, factor, st, to_fp8);
  return e4 ? launch_convert_fp8<__nv_bfloat16, true>(src, dst, n, factor, st, to_fp8)
            : launch_convert_fp8<__nv_bfloat16, false>(src, dst, n, factor, st, to_fp8);
}

}  // namespace

extern "C" {

int tf_attn_plan(const TfAttnDesc* desc, TfAttnPlan* plan) {
  if (plan == nullptr) return fail(TF_ERR_BAD_ARG, "plan is null");
  if (int rc = check_attn_desc(desc)) return rc;
  tfb::plan_attn(*desc, sm_count(), plan);
  const int bucket = plan->head_dim_kernel;
  if (plan->tile_q == 256)
    plan->smem_bytes = bucket == 128 ? tfb::AttnPairSmem<128>::kBytes : tfb::AttnPairSmem<64>::kBytes;
  else
    plan->smem_bytes = bucket == 256 ? tfb::AttnSmem<256>::kBytes
                                     : bucket == 128 ? tfb::AttnSmem<128>::kBytes : tfb::AttnSmem<64>::kBytes;
  return TF_OK;
}

int tf_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const TfAttnDesc* desc,
                void* stream) {
  if (int rc = check_attn_desc(desc)) return rc;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr)
    return fail(TF_ERR_BAD_ARG, "q, k, v and o must be non-null");
  if (!aligned16(o)) return fail(TF_ERR_UNSUPPORTED, "o must be 16-byte aligned");
  if (int rc = tfb::ensure_device_ready()) return rc;
  TfAttnPlan plan;
  tfb::plan_attn(*desc, sm_count(), &plan);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (plan.head_dim_kernel) {
    case 256:
      return desc->dtype == TF_F16 ? run_attn<__half, 256>(q, k, v, o, lse, desc, plan, s)
                                   : run_attn<__nv_bfloat16, 256>(q, k, v, o, lse, desc, plan, s);
    case 128:
      return desc->dtype == TF_F16 ? run_attn<__half, 128>(q, k, v, o, lse, desc, plan, s)
                                   : run_attn<__nv_bfloat16, 128>(q, k, v, o, lse, desc, plan, s);
    default:
      return desc->dtype == TF_F16 ? run_attn<__half, 64>(q, k, v, o, lse, desc, plan, s)
                                   : run_attn<__nv_bfloat16, 64>(q, k, v, o, lse, desc, plan, s);
  }
}

uint64_t tf_attn_bwd_workspace_bytes(const TfAttnDesc* desc) {
  if (desc == nullptr || desc->batch < 1 || desc->heads < 1 || desc->len_q < 1) return 0;
  return (uint64_t)desc->batch * desc->heads * desc->len_q * sizeof(float);
}

int tf_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                void* dq, void* dk, void* dv, const TfAttnDesc* desc, void* workspace, uint64_t workspace_bytes,
                void* stream) {
  if (int rc = check_attn_desc(desc)) return rc;
  if (desc->head_dim != desc->head_dim_v || (desc->head_dim != 64 && desc->head_dim != 128))
    return fail(TF_ERR_UNSUPPORTED, "the backward pass is compiled for head_dim == head_dim_v in {64, 128} (got %d, %d)",
                desc->head_dim, desc->head_dim_v);
  if (desc->k_stride_d != 1 || desc->v_stride_d != 1)
    return fail(TF_ERR_UNSUPPORTED, "the backward pass reads K as [Lk, D] and V as [Lk, Dv] (rows contiguous)");
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || d_o == nullptr || lse == nullptr ||
      dq == nullptr || dk == nullptr || dv == nullptr)
    return fail(TF_ERR_BAD_ARG, "q, k, v, o, d_o, lse, dq, dk and dv must be non-null");
  if (!aligned16(o) || !aligned16(d_o) || !aligned16(dq) || !aligned16(dk) || !aligned16(dv))
    return fail(TF_ERR_UNSUPPORTED, "o, d_o, dq, dk and dv must be 16-byte aligned");
  const int64_t st[] = {desc->q_stride_b, desc->q_stride_h, desc->q_stride_l, desc->k_stride_b, desc->k_stride_h,
                        desc->k_stride_l, desc->v_stride_b, desc->v_stride_h, desc->v_stride_l};
  for (int64_t x : st)
    if (x % 8 != 0 || x < 0) return fail(TF_ERR_UNSUPPORTED, "strides must be non-negative multiples of 8 elements (16 bytes)");
  if (workspace == nullptr || !aligned16(workspace)) return fail(TF_ERR_BAD_ARG, "workspace must be non-null and 16-byte aligned");
  const uint64_t need = tf_attn_bwd_workspace_bytes(desc);
  if (workspace_bytes < need)
    return fail(TF_ERR_WORKSPACE, "workspace holds %llu bytes but %llu are needed", (unsigned long long)workspace_bytes,
                (unsigned long long)need);
  if (int rc = tfb::ensure_device_ready()) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* delta = static_cast<float*>(workspace);
  if (desc->head_dim == 128)
    return desc->dtype == TF_F16
               ? launch_attn_bwd<__half, 128>(q, k, v, o, d_o, lse, dq, dk, dv, delta, desc, s)
               : launch_attn_bwd<__nv_bfloat16, 128>(q, k, v, o, d_o, lse, dq, dk, dv, delta, desc, s);
  return desc->dtype == TF_F16 ? launch_attn_bwd<__half, 64>(q, k, v, o, d_o, lse, dq, dk, dv, delta, desc, s)
                               : launch_attn_bwd<__nv_bfloat16, 64>(q, k, v, o, d_o, lse, dq, dk, dv, delta, desc, s);
}

int tf_fused_two_gemms(const void* a, const void* b, const void* c, void* d, int32_t m, int32_t n, int32_t k,
                       int32_t p, int32_t dtype, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd,
                       void* stream) {
  if (a == nullptr || b == nullptr || c == nullptr || d == nullptr)
    return fail(TF_ERR_BAD_ARG, "a, b, c and d must be non-null");
  if (m < 1 || n < 1 || k < 1 || p < 1) return fail(TF_ERR_BAD_ARG, "m, n, k and p must be positive");
  if (dtype != TF_F16 && dtype != TF_BF16)
    return fail(TF_ERR_UNSUPPORTED, "the inputs and output must be half-precision (fp16 or bf16); got dtype code %d", dtype);
  if (k % 8 != 0 || p % 8 != 0 || k > 256 || p > 256)
    return fail(TF_ERR_UNSUPPORTED, "fused_two_gemms needs k and p to be multiples of 8 up to 256 (got k=%d, p=%d)", k, p);
  if (n % 8 != 0)
    return fail(TF_ERR_UNSUPPORTED, "fused_two_gemms needs n to be a multiple of 8 (rows of C are read in 16-byte units; got n=%d)", n);
  if (lda < k || ldb < k || ldc < n || ldd < p) return fail(TF_ERR_BAD_ARG, "a leading dimension is smaller than its row");
  if (!aligned16(d) || ldd % 8 != 0) return fail(TF_ERR_UNSUPPORTED, "d must be 16-byte aligned with ldd a multiple of 8");
  if (int rc = tfb::ensure_device_ready()) return rc;
  TfAttnDesc desc{};
  desc.dtype = dtype;
  desc.batch = desc.heads = 1;
  desc.len_q = m;
  desc.len_kv = n;
  desc.head_dim = k;
  desc.head_dim_v = p;
  desc.softmax_scale = 1.f;
  desc.tile_q = 128;
  desc.tile_kv = 128;
  desc.q_stride_l = lda;
  desc.k_stride_l = ldb;
  desc.k_stride_d = 1;
  desc.v_stride_d = ldc;      // C is stored [P, N]: the row-per-output-column form
  desc.v_stride_l = 1;
  desc.o_stride_l = ldd;
  TfAttnPlan plan;
  tfb::plan_attn(desc, sm_count(), &plan);
  AttnLaunch L;
  if (int rc = prepare_attn(a, b, c, d, nullptr, &desc, plan, &L)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (plan.head_dim_kernel) {
    case 256:
      return dtype == TF_F16 ? launch_two_gemms<__half, 256>(L, &desc, s) : launch_two_gemms<__nv_bfloat16, 256>(L, &desc, s);
    case 128:
      return dtype == TF_F16 ? launch_two_gemms<__half, 128>(L, &desc, s) : launch_two_gemms<__nv_bfloat16, 128>(L, &desc, s);
    default:
      return dtype == TF_F16 ? launch_two_gemms<__half, 64>(L, &desc, s) : launch_two_gemms<__nv_bfloat16, 64>(L, &desc, s);
  }
}

int tf_decode_plan(const TfDecodeDesc* desc, TfDecodePlan* plan) {
  if (plan == nullptr) return fail(TF_ERR_BAD_ARG, "plan is null");
  if (int rc = check_decode_desc(desc)) return rc;
  tfb::plan_decode(*desc, sm_count(), plan);
  return TF_OK;
}

int tf_decode_split(const void* q, const void* k, const void* v, void* workspace, uint64_t workspace_bytes,
                    const TfDecodeDesc* desc, void* stream) {
  TfDecodePlan plan;
  if (int rc = plan_and_check_decode(q, k, v, workspace, workspace_bytes, desc, &plan)) return rc;
  const int64_t rows = (int64_t)desc->batch * desc->heads * plan.num_splits;
  float* part_o = static_cast<float*>(workspace);
  float* part_ml = part_o + rows * desc->head_dim;
  return dispatch_split(q, k, v, part_o, part_ml, desc, plan, static_cast<cudaStream_t>(stream));
}

int tf_decode_combine(const float* part_o, const float* part_ml, int32_t n_parts, int64_t part_stride_o,
                      int64_t row_stride_o, int64_t part_stride_ml, int64_t row_stride_ml, int32_t rows,
                      int32_t heads, int32_t head_dim, int32_t dtype, void* o, int64_t o_stride_b,
                      int64_t o_stride_h, float* lse, float* out_part_o, float* out_part_ml, void* stream) {
  if (part_o == nullptr || part_ml == nullptr) return fail(TF_ERR_BAD_ARG, "partials are null");
  if (n_parts < 1 || rows < 1 || heads < 1) return fail(TF_ERR_BAD_ARG, "n_parts, rows and heads must be positive");
  if (dtype != TF_F16 && dtype != TF_BF16) return fail(TF_ERR_UNSUPPORTED, "dtype code %d is not fp16 or bf16", dtype);
  const bool merged = out_part_o != nullptr;
  if (merged && out_part_ml == nullptr) return fail(TF_ERR_BAD_ARG, "out_part_ml is null");
  if (!merged && o == nullptr) return fail(TF_ERR_BAD_ARG, "neither o nor out_part_o given");
  tfb::DecodeCombineArgs a;
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.n_parts = n_parts;
  a.part_stride_o = part_stride_o;
  a.row_stride_o = row_stride_o;
  a.part_stride_ml = part_stride_ml;
  a.row_stride_ml = row_stride_ml;
  a.heads = heads;
  a.o = merged ? nullptr : o;
  a.o_stride_b = o_stride_b;
  a.o_stride_h = o_stride_h;
  a.lse = lse;
  a.out_part_o = out_part_o;
  a.out_part_ml = out_part_ml;
  a.peer_bases = nullptr;
  a.n_peers = a.my_rank = a.rows_total = 0;
  a.scatter_offset = a.flag_offset = 0;
  a.step = 0;
  a.wait_flags = nullptr;
  a.wait_n = 0;
  a.wait_step = 0;
  return dispatch_combine(a, rows, head_dim, dtype, static_cast<cudaStream_t>(stream));
}

int tf_decode_partial_scatter(const void* q, const void* k, const void* v, void* workspace,
                              uint64_t workspace_bytes, const TfDecodeDesc* desc, const void* peer_table,
                              int32_t rank, int32_t n_ranks, int64_t slot_offset_floats,
                              int64_t flag_offset_floats, uint32_t step, void* stream) {
  TfDecodePlan plan;
  if (int rc = plan_and_check_decode(q, k, v, workspace, workspace_bytes, desc, &plan)) return rc;
  if (peer_table == nullptr) return fail(TF_ERR_BAD_ARG, "peer_table is null");
  if (n_ranks < 1 || n_ranks > 64 || rank < 0 || rank >= n_ranks)
    return fail(TF_ERR_BAD_ARG, "rank %d / n_ranks %d out of range (at most 64 ranks)", rank, n_ranks);
  if (slot_offset_floats < 0 || flag_offset_floats < 0) return fail(TF_ERR_BAD_ARG, "negative buffer offset");
  const int rows = desc->batch * desc->heads;
  const int D = desc->head_dim;
  float* part_o = static_cast<float*>(workspace);
  float* part_ml = part_o + (int64_t)rows * plan.num_splits * D;
  if (int rc = dispatch_split(q, k, v, part_o, part_ml, desc, plan, static_cast<cudaStream_t>(stream))) return rc;
  tfb::DecodeCombineArgs a{};
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.n_parts = plan.num_splits;
  a.part_stride_o = D;
  a.row_stride_o = (int64_t)plan.num_splits * D;
  a.part_stride_ml = 2;
  a.row_stride_ml = (int64_t)plan.num_splits * 2;
  a.heads = desc->heads;
  a.peer_bases = static_cast<float* const*>(peer_table);
  a.n_peers = n_ranks;
  a.my_rank = rank;
  a.rows_total = rows;
  a.scatter_offset = slot_offset_floats;
  a.flag_offset = flag_offset_floats;
  a.step = step;
  return dispatch_combine(a, rows, D, desc->dtype, static_cast<cudaStream_t>(stream));
}

int tf_decode_gathered_wait(const float* slots, const uint32_t* flags, int32_t n_ranks, uint32_t step,
                            int32_t batch, int32_t heads, int32_t head_dim, int32_t dtype, void* o,
                            int64_t o_stride_b, int64_t o_stride_h, float* lse, void* stream) {
  if (slots == nullptr || o == nullptr || flags == nullptr)
    return fail(TF_ERR_BAD_ARG, "slots, flags and o must be non-null");
  if (n_ranks < 1 || n_ranks > 64 || batch < 1 || heads < 1)
    return fail(TF_ERR_BAD_ARG, "n_ranks (<= 64), batch and heads must be positive");
  if (dtype != TF_F16 && dtype != TF_BF16) return fail(TF_ERR_UNSUPPORTED, "dtype code %d is not fp16 or bf16", dtype);
  if (int rc = tfb::ensure_device_ready()) return rc;
  const int64_t rows = (int64_t)batch * heads;
  const int64_t slot_floats = rows * (head_dim + 2);
  tfb::DecodeCombineArgs a{};
  a.part_o = slots;
  a.part_ml = slots + rows * head_dim;
  a.n_parts = n_ranks;
  a.part_stride_o = slot_floats;
  a.row_stride_o = head_dim;
  a.part_stride_ml = slot_floats;
  a.row_stride_ml = 2;
  a.heads = heads;
  a.o = o;
  a.o_stride_b = o_stride_b;
  a.o_stride_h = o_stride_h;
  a.lse = lse;
  a.wait_flags = flags;
  a.wait_n = n_ranks;
  a.wait_step = step;
  return dispatch_combine(a, (int)rows, head_dim, dtype, static_cast<cudaStream_t>(stream));
}

int tf_decode(const void* q, const void* k, const void* v, void* o, float* lse, void* workspace,
              uint64_t workspace_bytes, const TfDecodeDesc* desc, void* stream) {
  TfDecodePlan plan;
  if (int rc = plan_and_check_decode(q, k, v, workspace, workspace_bytes, desc, &plan)) return rc;
  if (o == nullptr) return fail(TF_ERR_BAD_ARG, "o is null");
  if (desc->len_kv < 1) return fail(TF_ERR_BAD_ARG, "len_kv must be positive for a full decode");
  const int rows = desc->batch * desc->heads;
  const int D = desc->head_dim;
  float* part_o = static_cast<float*>(workspace);
  float* part_ml = part_o + (int64_t)rows * plan.num_splits * D;
  if (int rc = dispatch_split(q, k, v, part_o, part_ml, desc, plan, static_cast<cudaStream_t>(stream))) return rc;
  return tf_decode_combine(part_o, part_ml, plan.num_splits, D, (int64_t)plan.num_splits * D, 2,
                           (int64_t)plan.num_splits * 2, rows, desc->heads, D, desc->dtype, o,
                           desc->o_stride_b, desc->o_stride_h, lse, nullptr, nullptr, stream);
}

int tf_decode_partial(const void* q, const void* k, const void* v, float* slot, void* workspace,
                      uint64_t workspace_bytes, const TfDecodeDesc* desc, void* stream) {
  TfDecodePlan plan;
  if (int rc = plan_and_check_decode(q, k, v, workspace, workspace_bytes, desc, &plan)) return rc;
  if (slot == nullptr) return fail(TF_ERR_BAD_ARG, "slot is null");
  const int rows = desc->batch * desc->heads;
  const int D = desc->head_dim;
  float* part_o = static_cast<float*>(workspace);
  float* part_ml = part_o + (int64_t)rows * plan.num_splits * D;
  if (int rc = dispatch_split(q, k, v, part_o, part_ml, desc, plan, static_cast<cudaStream_t>(stream))) return rc;
  return tf_decode_combine(part_o, part_ml, plan.num_splits, D, (int64_t)plan.num_splits * D, 2,
                           (int64_t)plan.num_splits * 2, rows, desc->heads, D, desc->dtype, nullptr, 0, 0,
                           nullptr, slot, slot + (int64_t)rows * D, stream);
}

int tf_decode_gathered(const float* slots, int32_t n_ranks, int32_t batch, int32_t heads, int32_t head_dim,
                       int32_t dtype, void* o, int64_t o_stride_b, int64_t o_stride_h, float* lse,
                       void* stream) {
  if (slots == nullptr || o == nullptr) return fail(TF_ERR_BAD_ARG, "slots and o must be non-null");
  if (n_ranks < 1 || batch < 1 || heads < 1) return fail(TF_ERR_BAD_ARG, "n_ranks, batch and heads must be positive");
  const int64_t rows = (int64_t)batch * heads;
  const int64_t slot_floats = rows * (head_dim + 2);
  return tf_decode_combine(slots, slots + rows * head_dim, n_ranks, slot_floats, head_dim, slot_floats, 2,
                           (int32_t)rows, heads, head_dim, dtype, o, o_stride_b, o_stride_h, lse, nullptr,
                           nullptr, stream);
}

int tf_decode_static(const void* q, const void* k, const void* v, void* o, float* lse,
                     const TfDecodeDesc* desc, void* stream) {
  if (int rc = check_decode_desc(desc)) return rc;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr)
    return fail(TF_ERR_BAD_ARG, "q, k, v and o must be non-null");
  if (desc->len_kv < 1) return fail(TF_ERR_BAD_ARG, "len_kv must be positive for a full decode");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v))
    return fail(TF_ERR_UNSUPPORTED, "q, k and v must be 16-byte aligned");
  TfDecodePlan plan;
  tfb::plan_decode(*desc, sm_count(), &plan);
  if (plan.workspace_bytes > kStaticScratchBytes)
    return fail(TF_ERR_WORKSPACE,
                "this problem needs %llu bytes of scratch but the built-in scratch holds %llu; lower "
                "num_splits or batch*heads, or use tf_decode with a caller-provided workspace",
                (unsigned long long)plan.workspace_bytes, (unsigned long long)kStaticScratchBytes);
  float* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  const int rows = desc->batch * desc->heads;
  const int D = desc->head_dim;
  float* part_o = scratch;
  float* part_ml = part_o + (int64_t)rows * plan.num_splits * D;
  if (int rc = dispatch_split(q, k, v, part_o, part_ml, desc, plan, static_cast<cudaStream_t>(stream))) return rc;
  return tf_decode_combine(part_o, part_ml, plan.num_splits, D, (int64_t)plan.num_splits * D, 2,
                           (int64_t)plan.num_splits * 2, rows, desc->heads, D, desc->dtype, o,
                           desc->o_stride_b, desc->o_stride_h, lse, nullptr, nullptr, stream);
}

uint64_t tf_decode_static_capacity(void) { return kStaticScratchBytes; }

const char* tf_last_error(void) { return g_err; }

int tf_device_status(int32_t* code_out) {
  int code = 0;
  TF_CUDA_TRY(cudaDeviceSynchronize());
  TF_CUDA_TRY(cudaMemcpyFromSymbol(&code, tfb::g_status_word, sizeof(int)));
  if (code != 0) {
    const int zero = 0;
    TF_CUDA_TRY(cudaMemcpyToSymbol(tfb::g_status_word, &zero, sizeof(int)));
  }
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices) {
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (g_device[dev].mirror_host != nullptr) *static_cast<volatile int*>(g_device[dev].mirror_host) = 0;
  }
  if (code_out != nullptr) *code_out = code;
  if (code != 0) return fail(TF_ERR_DEVICE_TIMEOUT, "a device-side wait gave up (site code %d)", code);
  return TF_OK;
}

int tf_device_status_peek(int32_t* code_out) {
  int code = 0, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices) {
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (g_device[dev].mirror_host != nullptr) code = *static_cast<volatile int*>(g_device[dev].mirror_host);
  }
  if (code_out != nullptr) *code_out = code;
  if (code != 0)
    return fail(TF_ERR_DEVICE_TIMEOUT, "a device-side wait of an earlier launch gave up (site code %d); its output is not valid",
                code);
  return TF_OK;
}

int tf_set_wait_limit_ms(uint32_t milliseconds) {
  if (milliseconds == 0) return fail(TF_ERR_BAD_ARG, "the wait limit must be positive");
  g_wait_limit_ns_host.store((unsigned long long)milliseconds * 1000000ull, std::memory_order_relaxed);
  return TF_OK;
}

int tf_fp8_quantize(const void* src, void* dst, int64_t n, int32_t src_dtype, int32_t fp8_dtype, float factor,
                    void* stream) {
  return convert_fp8(src, dst, n, src_dtype, fp8_dtype, factor, stream, /*to_fp8=*/true);
}

int tf_fp8_dequantize(const void* src, void* dst, int64_t n, int32_t fp8_dtype, int32_t dst_dtype, float factor,
                      void* stream) {
  return convert_fp8(src, dst, n, dst_dtype, fp8_dtype, factor, stream, /*to_fp8=*/false);
}

int tf_probe_mma_clocks(int32_t a_from_tmem, int32_t n, int32_t b_mn_major, int32_t desc32, int32_t uniform_issue,
                        int32_t n_mma, int64_t* issue_clocks, int64_t* complete_clocks) {
  if (n != 64 && n != 128 && n != 256) return fail(TF_ERR_BAD_ARG, "n must be 64, 128 or 256 (got %d)", n);
  if (n_mma < 8 || n_mma % 8 != 0 || n_mma > (1 << 20))
    return fail(TF_ERR_BAD_ARG, "n_mma must be a multiple of 8 in [8, 2^20] (got %d)", n_mma);
  if (issue_clocks == nullptr || complete_clocks == nullptr) return fail(TF_ERR_BAD_ARG, "the outputs must be non-null");
  if (int rc = tfb::ensure_device_ready()) return rc;
  long long* dev = nullptr;
  TF_CUDA_TRY(cudaMalloc(&dev, 2 * sizeof(long long)));
  tfb::ProbeMmaArgs a{a_from_tmem != 0, n, b_mn_major != 0, desc32 != 0, uniform_issue != 0, n_mma, dev};
  cudaError_t e = cudaFuncSetAttribute(tfb::probe_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tfb::kProbeSmemBytes);
  long long host[2] = {0, 0};
  if (e == cudaSuccess) {
    tfb::probe_mma_kernel<<<1, 128, tfb::kProbeSmemBytes>>>(a);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpy(host, dev, sizeof(host), cudaMemcpyDeviceToHost);    // (synchronises)
  cudaFree(dev);
  if (e != cudaSuccess) return fail(TF_ERR_CUDA, "the probe kernel failed: %s", cudaGetErrorString(e));
  *issue_clocks = host[0];
  *complete_clocks = host[1];
  return TF_OK;
}

int tf_probe_mma_pair_clocks(int32_t a_from_tmem, int32_t n, int32_t b_mn_major, int32_t n_mma,
                             int64_t* issue_clocks, int64_t* complete_clocks) {
  if (n != 64 && n != 128 && n != 256) return fail(TF_ERR_BAD_ARG, "n must be 64, 128 or 256 (got %d)", n);
  if (n_mma < 8 || n_mma % 8 != 0 || n_mma > (1 << 20))
    return fail(TF_ERR_BAD_ARG, "n_mma must be a multiple of 8 in [8, 2^20] (got %d)", n_mma);
  if (issue_clocks == nullptr || complete_clocks == nullptr) return fail(TF_ERR_BAD_ARG, "the outputs must be non-null");
  if (int rc = tfb::ensure_device_ready()) return rc;
  long long* dev = nullptr;
  TF_CUDA_TRY(cudaMalloc(&dev, 2 * sizeof(long long)));
  tfb::ProbePairArgs a{a_from_tmem != 0, n, b_mn_major != 0, n_mma, dev};
  cudaError_t e = cudaFuncSetAttribute(tfb::probe_mma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tfb::kProbeSmemBytes);
  long long host[2] = {0, 0};
  if (e == cudaSuccess) {
    tfb::probe_mma_pair_kernel<<<2, 128, tfb::kProbeSmemBytes>>>(a);     // one cluster of two CTAs
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpy(host, dev, sizeof(host), cudaMemcpyDeviceToHost);    // (synchronises)
  cudaFree(dev);
  if (e != cudaSuccess) return fail(TF_ERR_CUDA, "the probe kernel failed: %s", cudaGetErrorString(e));
  *issue_clocks = host[0];
  *complete_clocks = host[1];
  return TF_OK;
}

int tf_abi_version(void) { return 5; }

}  // extern "C"
