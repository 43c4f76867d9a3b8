// Operator layer: registers the attention operators with the torch dispatcher
// under the `tilefusion` namespace and forwards each to the C-ABI of
// libtilefusion_b200.so.  torch types stop here.
//
// `flash_attention` keeps the schema of TileFusion's operator verbatim
// (include/kernels/kernel_list.hpp:25-30; registered there through
// REGISTER_OP / KernelRegistry, include/kernel_registry.hpp:22-88, and
// src/torch_bind.cc:8-14).  The decode operators are additions registered the
// same way.  Differences from the reference's host operator
// (src/kernels/flash_attn.cu:58-152): leading (batch, head) dimensions and
// bf16 are accepted, operands may be strided views (no .contiguous() copy is
// needed), the launch goes to torch's current stream, and there is no device
// synchronisation.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <vector>

#include "tilefusion_b200.h"

namespace tilefusion_b200 {
namespace {

struct OpEntry {
  const char* name;
  const char* schema;
  void (*bind)(torch::Library&, const char*);
};

std::vector<OpEntry>& op_table() {
  static std::vector<OpEntry> table;
  return table;
}

// Adds an operator to the table at static-initialisation time; the
// TORCH_LIBRARY blocks below walk the table.
#define TF_REGISTER_OP(opname, schema_str, fn)                                         \
  static const bool opname##_added = [] {                                              \
    op_table().push_back({#opname, schema_str, [](torch::Library& m, const char* n) {  \
                            m.impl(n, c10::DispatchKey::CUDA, fn);                    \
                          }});                                                         \
    return true;                                                                       \
  }()

int dtype_code(const at::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kHalf || t.scalar_type() == at::kBFloat16,
              "the inputs and output must be half-precision (fp16 or bf16).");
  return t.scalar_type() == at::kHalf ? TF_F16 : TF_BF16;
}

// 8-bit storage code of a K/V tensor, or -1 when it is not an fp8 tensor.
int fp8_code(const at::Tensor& t) {
  if (t.scalar_type() == at::kFloat8_e4m3fn) return TF_FP8_E4M3;
  if (t.scalar_type() == at::kFloat8_e5m2) return TF_FP8_E5M2;
  return -1;
}

// K and V either share Q's type or are both the same 8-bit storage type.
void set_kv_dtype(TfDecodeDesc* d, const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, double k_scale,
                  double v_scale) {
  TORCH_CHECK(K.scalar_type() == V.scalar_type() && (K.scalar_type() == Q.scalar_type() || fp8_code(K) >= 0),
              "K and V must share Q's dtype, or both be float8_e4m3fn or float8_e5m2");
  if (fp8_code(K) >= 0) {
    d->kv_dtype = fp8_code(K);
    d->k_scale = (float)k_scale;
    d->v_scale = (float)v_scale;
  } else {
    TORCH_CHECK(k_scale == 1.0 && v_scale == 1.0, "k_scale / v_scale apply to an 8-bit K/V cache only");
  }
}

void check_status(int rc) { TORCH_CHECK(rc == TF_OK, "tilefusion_b200: ", tf_last_error()); }

// Raises if a device-side wait of an EARLIER launch on this device gave up (its
// output was left unwritten or NaN).  Costs one read of a host variable; the
// condition is cleared so that the error is raised once.
void check_earlier_launches() {
  int32_t code = 0;
  if (tf_device_status_peek(&code) != TF_OK) {
    tf_device_status(nullptr);
    TORCH_CHECK(false, "tilefusion_b200: a device-side wait of an earlier launch gave up (site code ", code,
                "); the output of that launch is not valid");
  }
}

// Splits leading dims of a [..., rows, cols] tensor into (batch, heads) with
// element strides; 2-D tensors are one (batch, head).
struct Lead {
  int64_t batch = 1, heads = 1, stride_b = 0, stride_h = 0;
};

Lead lead_dims(const at::Tensor& t, const char* name) {
  Lead l;
  const int64_t nd = t.dim();
  TORCH_CHECK(nd >= 2 && nd <= 4, name, " must have 2, 3 or 4 dimensions, got ", nd);
  if (nd == 3) {
    l.heads = t.size(0);
    l.stride_h = t.stride(0);
  } else if (nd == 4) {
    l.batch = t.size(0);
    l.heads = t.size(1);
    l.stride_b = t.stride(0);
    l.stride_h = t.stride(1);
  }
  return l;
}

void attention_impl(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& O,
                    at::Tensor* LSE, int64_t tile_q, int64_t tile_kv, double softmax_scale, bool causal) {
  TORCH_CHECK(Q.is_cuda() && K.is_cuda() && V.is_cuda() && O.is_cuda(), "Q, K, V and O must be CUDA tensors");
  TORCH_CHECK(Q.scalar_type() == K.scalar_type() && Q.scalar_type() == V.scalar_type() &&
                  Q.scalar_type() == O.scalar_type(),
              "Q, K, V and O must share one dtype");
  TORCH_CHECK(Q.dim() == K.dim() && Q.dim() == V.dim() && Q.dim() == O.dim(),
              "Q, K, V and O must have the same number of dimensions");
  TfAttnDesc d{};
  d.dtype = dtype_code(Q);
  const Lead lq = lead_dims(Q, "Q"), lk = lead_dims(K, "K"), lv = lead_dims(V, "V"), lo = lead_dims(O, "O");
  TORCH_CHECK(lq.batch == lk.batch && lq.batch == lv.batch && lq.batch == lo.batch && lq.heads == lk.heads &&
                  lq.heads == lv.heads && lq.heads == lo.heads,
              "leading (batch, head) dimensions of Q, K, V and O must match");
  d.batch = (int32_t)lq.batch;
  d.heads = (int32_t)lq.heads;
  d.len_q = (int32_t)Q.size(-2);
  d.head_dim = (int32_t)Q.size(-1);
  d.len_kv = (int32_t)K.size(-2);
  d.head_dim_v = (int32_t)O.size(-1);
  TORCH_CHECK(K.size(-1) == d.head_dim, "K must be [..., Lk, D] with D = Q.size(-1)");
  TORCH_CHECK(O.size(-2) == d.len_q, "O must be [..., Lq, Dv]");
  TORCH_CHECK(Q.stride(-1) == 1 && O.stride(-1) == 1, "Q and O rows must be contiguous");
  d.q_stride_b = lq.stride_b;
  d.q_stride_h = lq.stride_h;
  d.q_stride_l = Q.stride(-2);
  d.k_stride_b = lk.stride_b;
  d.k_stride_h = lk.stride_h;
  d.k_stride_l = K.stride(-2);
  d.k_stride_d = K.stride(-1);
  d.v_stride_b = lv.stride_b;
  d.v_stride_h = lv.stride_h;
  // The operand is V^T [..., Dv, Lk], as in the reference.  A caller holding V
  // as [..., Lk, Dv] passes V.transpose(-1, -2): a view, nothing is copied (the
  // kernels read either memory layout).  The shape alone cannot tell the two
  // apart when Lk == Dv, so no other form is accepted.
  TORCH_CHECK(V.size(-2) == d.head_dim_v && V.size(-1) == d.len_kv,
              "V must be V^T, [..., Dv, Lk], with Lk = K.size(-2) and Dv = O.size(-1); pass "
              "value.transpose(-1, -2) (a view) for a value stored [..., Lk, Dv]");
  d.v_stride_d = V.stride(-2);
  d.v_stride_l = V.stride(-1);
  d.o_stride_b = lo.stride_b;
  d.o_stride_h = lo.stride_h;
  d.o_stride_l = O.stride(-2);
  d.softmax_scale = (float)softmax_scale;
  d.causal = causal ? 1 : 0;
  d.tile_q = (int32_t)tile_q;
  d.tile_kv = (int32_t)tile_kv;
  float* lse_ptr = nullptr;
  if (LSE != nullptr) {
    TORCH_CHECK(LSE->is_cuda() && LSE->scalar_type() == at::kFloat && LSE->is_contiguous() &&
                    LSE->numel() == (int64_t)d.batch * d.heads * d.len_q,
                "LSE must be a contiguous fp32 CUDA tensor with batch*heads*Lq elements");
    lse_ptr = LSE->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(Q.device());
  check_earlier_launches();
  check_status(tf_attn_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), lse_ptr, &d,
                           at::cuda::getCurrentCUDAStream().stream()));
}

void flash_attention(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& O,
                     int64_t tile_length_q, int64_t tile_length_kv, int64_t tile_hidden_qk,
                     int64_t tile_hidden_v, double softmax_scale, bool causal) {
  (void)tile_hidden_qk;  // the head dimensions are never tiled on this path
  (void)tile_hidden_v;
  attention_impl(Q, K, V, O, nullptr, tile_length_q, tile_length_kv, softmax_scale, causal);
}

void flash_attention_lse(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& O,
                         at::Tensor& LSE, int64_t tile_length_q, int64_t tile_length_kv, double softmax_scale,
                         bool causal) {
  attention_impl(Q, K, V, O, &LSE, tile_length_q, tile_length_kv, softmax_scale, causal);
}

// Backward of flash_attention (no counterpart in the reference).  Operand
// conventions of the forward operator: K [..., Lk, D], V^T [..., Dv, Lk] -- here
// as a VIEW of a value stored [..., Lk, Dv], which is what
// value.transpose(-1, -2) gives (the backward kernels read V rows).  dQ / dK /
// dV^T are written in place and must have the shapes and strides of Q / K / V^T.
void flash_attention_bwd(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, const at::Tensor& O,
                         const at::Tensor& dO, const at::Tensor& LSE, at::Tensor& dQ, at::Tensor& dK, at::Tensor& dV,
                         double softmax_scale, bool causal) {
  const at::Tensor* all[] = {&Q, &K, &V, &O, &dO, &LSE, &dQ, &dK, &dV};
  for (const at::Tensor* t : all) TORCH_CHECK(t->is_cuda(), "all tensors must be CUDA tensors");
  TORCH_CHECK(Q.scalar_type() == K.scalar_type() && Q.scalar_type() == V.scalar_type() && Q.scalar_type() == O.scalar_type() &&
                  Q.scalar_type() == dO.scalar_type() && Q.scalar_type() == dQ.scalar_type() &&
                  Q.scalar_type() == dK.scalar_type() && Q.scalar_type() == dV.scalar_type(),
              "Q, K, V, O, dO, dQ, dK and dV must share one dtype");
  TORCH_CHECK(Q.dim() == K.dim() && Q.dim() == V.dim() && Q.dim() == O.dim(), "Q, K, V and O must have the same number of dimensions");
  TORCH_CHECK(dO.sizes() == O.sizes() && dO.strides() == O.strides(), "dO must have the shape and strides of O");
  TORCH_CHECK(dQ.sizes() == Q.sizes() && dQ.strides() == Q.strides(), "dQ must have the shape and strides of Q");
  TORCH_CHECK(dK.sizes() == K.sizes() && dK.strides() == K.strides(), "dK must have the shape and strides of K");
  TORCH_CHECK(dV.sizes() == V.sizes() && dV.strides() == V.strides(), "dV must have the shape and strides of V");
  TfAttnDesc d{};
  d.dtype = dtype_code(Q);
  const Lead lq = lead_dims(Q, "Q"), lk = lead_dims(K, "K"), lv = lead_dims(V, "V"), lo = lead_dims(O, "O");
  TORCH_CHECK(lq.batch == lk.batch && lq.batch == lv.batch && lq.batch == lo.batch && lq.heads == lk.heads &&
                  lq.heads == lv.heads && lq.heads == lo.heads,
              "leading (batch, head) dimensions of Q, K, V and O must match");
  d.batch = (int32_t)lq.batch;
  d.heads = (int32_t)lq.heads;
  d.len_q = (int32_t)Q.size(-2);
  d.head_dim = (int32_t)Q.size(-1);
  d.len_kv = (int32_t)K.size(-2);
  d.head_dim_v = (int32_t)O.size(-1);
  TORCH_CHECK(K.size(-1) == d.head_dim && O.size(-2) == d.len_q, "expected Q [.., Lq, D], K [.., Lk, D], O [.., Lq, Dv]");
  TORCH_CHECK(V.size(-2) == d.head_dim_v && V.size(-1) == d.len_kv, "V must be V^T, [..., Dv, Lk]");
  TORCH_CHECK(Q.stride(-1) == 1 && O.stride(-1) == 1 && K.stride(-1) == 1 && V.stride(-2) == 1,
              "rows of Q, K, O must be contiguous and V^T must be a transposed view of a value stored [..., Lk, Dv]");
  TORCH_CHECK(LSE.scalar_type() == at::kFloat && LSE.is_contiguous() && LSE.numel() == (int64_t)d.batch * d.heads * d.len_q,
              "LSE must be a contiguous fp32 tensor with batch*heads*Lq elements");
  d.q_stride_b = lq.stride_b;
  d.q_stride_h = lq.stride_h;
  d.q_stride_l = Q.stride(-2);
  d.k_stride_b = lk.stride_b;
  d.k_stride_h = lk.stride_h;
  d.k_stride_l = K.stride(-2);
  d.k_stride_d = 1;
  d.v_stride_b = lv.stride_b;
  d.v_stride_h = lv.stride_h;
  d.v_stride_l = V.stride(-1);
  d.v_stride_d = 1;
  d.o_stride_b = lo.stride_b;
  d.o_stride_h = lo.stride_h;
  d.o_stride_l = O.stride(-2);
  d.softmax_scale = (float)softmax_scale;
  d.causal = causal ? 1 : 0;
  const c10::cuda::CUDAGuard guard(Q.device());
  check_earlier_launches();
  const uint64_t need = tf_attn_bwd_workspace_bytes(&d);
  at::Tensor ws = at::empty({(int64_t)((need + 3) / 4)}, Q.options().dtype(at::kFloat));
  check_status(tf_attn_bwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), dO.data_ptr(), LSE.data_ptr<float>(),
                           dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(), &d, ws.data_ptr(), (uint64_t)ws.numel() * 4,
                           at::cuda::getCurrentCUDAStream().stream()));
}

TfDecodeDesc decode_desc(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, int64_t kv_chunk,
                         int64_t num_splits, double softmax_scale, double k_scale = 1.0, double v_scale = 1.0) {
  TORCH_CHECK(Q.is_cuda() && K.is_cuda() && V.is_cuda(), "Q, K and V must be CUDA tensors");
  TORCH_CHECK(Q.dim() == 4 && K.dim() == 4 && V.dim() == 4,
              "Q must be [B, H, 1, D] and K, V must be [B, H, Lk, D]");
  TORCH_CHECK(Q.size(2) == 1, "flash_decoding takes one query row per (batch, head)");
  TORCH_CHECK(K.sizes() == V.sizes() && K.size(0) == Q.size(0) && K.size(3) == Q.size(3) && K.size(1) >= 1 &&
                  Q.size(1) % K.size(1) == 0,
              "K and V must be [B, H_kv, Lk, D] with H_kv dividing Q's head count");
  TORCH_CHECK(Q.stride(3) == 1 && K.stride(3) == 1 && V.stride(3) == 1 &&
                  (K.size(2) <= 1 || (K.stride(2) == K.size(3) && V.stride(2) == V.size(3))),
              "rows of Q, K and V must be contiguous and consecutive keys D elements apart");
  TfDecodeDesc d{};
  set_kv_dtype(&d, Q, K, V, k_scale, v_scale);
  d.dtype = dtype_code(Q);
  d.batch = (int32_t)Q.size(0);
  d.heads = (int32_t)Q.size(1);
  d.heads_kv = (int32_t)K.size(1);
  d.len_kv = (int32_t)K.size(2);
  d.head_dim = (int32_t)Q.size(3);
  d.kv_chunk = (int32_t)kv_chunk;
  d.num_splits = (int32_t)num_splits;
  d.softmax_scale = (float)softmax_scale;
  d.q_stride_b = Q.stride(0);
  d.q_stride_h = Q.stride(1);
  d.k_stride_b = K.stride(0);
  d.k_stride_h = K.stride(1);
  d.v_stride_b = V.stride(0);
  d.v_stride_h = V.stride(1);
  return d;
}

at::Tensor decode_workspace(const TfDecodeDesc& d, const at::Tensor& like) {
  TfDecodePlan plan;
  check_status(tf_decode_plan(&d, &plan));
  return at::empty({(int64_t)((plan.workspace_bytes + 3) / 4)}, like.options().dtype(at::kFloat));
}

void flash_decoding(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& O,
                    at::Tensor& LSE, int64_t kv_chunk, int64_t num_splits, double softmax_scale, double k_scale,
                    double v_scale) {
  TfDecodeDesc d = decode_desc(Q, K, V, kv_chunk, num_splits, softmax_scale, k_scale, v_scale);
  TORCH_CHECK(O.is_cuda() && O.scalar_type() == Q.scalar_type() && O.dim() == 4 && O.size(0) == Q.size(0) &&
                  O.size(1) == Q.size(1) && O.size(2) == 1 && O.size(3) == Q.size(3) && O.stride(3) == 1,
              "O must be [B, H, 1, D] with contiguous rows and Q's dtype");
  TORCH_CHECK(LSE.is_cuda() && LSE.scalar_type() == at::kFloat && LSE.is_contiguous() &&
                  LSE.numel() == Q.size(0) * Q.size(1),
              "LSE must be a contiguous fp32 CUDA tensor with B*H elements");
  d.o_stride_b = O.stride(0);
  d.o_stride_h = O.stride(1);
  const c10::cuda::CUDAGuard guard(Q.device());
  check_earlier_launches();
  at::Tensor ws = decode_workspace(d, Q);
  check_status(tf_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), LSE.data_ptr<float>(),
                         ws.data_ptr(), (uint64_t)ws.numel() * 4, &d,
                         at::cuda::getCurrentCUDAStream().stream()));
}

// Paged KV cache: K/V pages [num_pages, H_kv, page_size, D], block_table int32 [B, max_pages].
void flash_decoding_paged(const at::Tensor& Q, const at::Tensor& Kp, const at::Tensor& Vp,
                          const at::Tensor& block_table, int64_t kv_len, at::Tensor& O, at::Tensor& LSE,
                          int64_t kv_chunk, int64_t num_splits, double softmax_scale, double k_scale,
                          double v_scale) {
  TORCH_CHECK(Q.is_cuda() && Kp.is_cuda() && Vp.is_cuda() && block_table.is_cuda(), "inputs must be CUDA tensors");
  TORCH_CHECK(Q.dim() == 4 && Q.size(2) == 1, "Q must be [B, H, 1, D]");
  TORCH_CHECK(Kp.dim() == 4 && Kp.sizes() == Vp.sizes() && Kp.size(3) == Q.size(3) && Q.size(1) % Kp.size(1) == 0,
              "K and V pages must be [num_pages, H_kv, page_size, D] with H_kv dividing Q's head count");
  TORCH_CHECK(Q.stride(3) == 1 && Kp.stride(3) == 1 && Vp.stride(3) == 1 && Kp.stride(2) == Kp.size(3) &&
                  Vp.stride(2) == Vp.size(3),
              "rows of Q, K and V must be contiguous and consecutive keys of a page D elements apart");
  TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.dim() == 2 && block_table.is_contiguous() &&
                  block_table.size(0) == Q.size(0),
              "block_table must be a contiguous int32 tensor [B, max_pages]");
  TORCH_CHECK(O.is_cuda() && O.scalar_type() == Q.scalar_type() && O.dim() == 4 && O.size(0) == Q.size(0) &&
                  O.size(1) == Q.size(1) && O.size(2) == 1 && O.size(3) == Q.size(3) && O.stride(3) == 1,
              "O must be [B, H, 1, D] with contiguous rows and Q's dtype");
  TORCH_CHECK(LSE.is_cuda() && LSE.scalar_type() == at::kFloat && LSE.is_contiguous() &&
                  LSE.numel() == Q.size(0) * Q.size(1),
              "LSE must be a contiguous fp32 CUDA tensor with B*H elements");
  TfDecodeDesc d{};
  set_kv_dtype(&d, Q, Kp, Vp, k_scale, v_scale);
  d.dtype = dtype_code(Q);
  d.batch = (int32_t)Q.size(0);
  d.heads = (int32_t)Q.size(1);
  d.heads_kv = (int32_t)Kp.size(1);
  d.len_kv = (int32_t)kv_len;
  d.head_dim = (int32_t)Q.size(3);
  d.kv_chunk = (int32_t)kv_chunk;
  d.num_splits = (int32_t)num_splits;
  d.softmax_scale = (float)softmax_scale;
  d.q_stride_b = Q.stride(0);
  d.q_stride_h = Q.stride(1);
  d.k_stride_h = Kp.stride(1);
  d.v_stride_h = Vp.stride(1);
  d.o_stride_b = O.stride(0);
  d.o_stride_h = O.stride(1);
  d.page_size = (int32_t)Kp.size(2);
  d.block_table = block_table.data_ptr<int>();
  d.max_pages = (int32_t)block_table.size(1);
  d.num_pages = (int32_t)Kp.size(0);
  d.k_stride_page = Kp.stride(0);
  d.v_stride_page = Vp.stride(0);
  const c10::cuda::CUDAGuard guard(Q.device());
  at::Tensor ws = decode_workspace(d, Q);
  check_status(tf_decode(Q.data_ptr(), Kp.data_ptr(), Vp.data_ptr(), O.data_ptr(), LSE.data_ptr<float>(),
                         ws.data_ptr(), (uint64_t)ws.numel() * 4, &d, at::cuda::getCurrentCUDAStream().stream()));
}

// Bulk conversion between a contiguous fp16/bf16 tensor and a float8 tensor of the same shape.
void fp8_quantize(const at::Tensor& src, at::Tensor& dst, double factor) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.is_contiguous() && dst.is_contiguous() &&
                  src.numel() == dst.numel() && fp8_code(dst) >= 0,
              "src must be a contiguous fp16/bf16 CUDA tensor and dst a contiguous float8 tensor of the same size");
  const c10::cuda::CUDAGuard guard(src.device());
  check_status(tf_fp8_quantize(src.data_ptr(), dst.data_ptr(), src.numel(), dtype_code(src), fp8_code(dst),
                               (float)factor, at::cuda::getCurrentCUDAStream().stream()));
}

void fp8_dequantize(const at::Tensor& src, at::Tensor& dst, double factor) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.is_contiguous() && dst.is_contiguous() &&
                  src.numel() == dst.numel() && fp8_code(src) >= 0,
              "src must be a contiguous float8 CUDA tensor and dst a contiguous fp16/bf16 tensor of the same size");
  const c10::cuda::CUDAGuard guard(src.device());
  check_status(tf_fp8_dequantize(src.data_ptr(), dst.data_ptr(), src.numel(), fp8_code(src), dtype_code(dst),
                                 (float)factor, at::cuda::getCurrentCUDAStream().stream()));
}

void flash_decoding_partial(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& slot,
                            int64_t kv_chunk, int64_t num_splits, double softmax_scale) {
  TfDecodeDesc d = decode_desc(Q, K, V, kv_chunk, num_splits, softmax_scale);
  TORCH_CHECK(slot.is_cuda() && slot.scalar_type() == at::kFloat && slot.is_contiguous() &&
                  slot.numel() == Q.size(0) * Q.size(1) * (Q.size(3) + 2),
              "slot must be a contiguous fp32 CUDA tensor with B*H*(D+2) elements");
  const c10::cuda::CUDAGuard guard(Q.device());
  at::Tensor ws = decode_workspace(d, Q);
  check_status(tf_decode_partial(Q.data_ptr(), K.data_ptr(), V.data_ptr(), slot.data_ptr<float>(),
                                 ws.data_ptr(), (uint64_t)ws.numel() * 4, &d,
                                 at::cuda::getCurrentCUDAStream().stream()));
}

void flash_decoding_gathered(const at::Tensor& slots, at::Tensor& O, at::Tensor& LSE) {
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kFloat && slots.is_contiguous() && slots.dim() == 2,
              "slots must be a contiguous fp32 CUDA tensor [n_ranks, B*H*(D+2)]");
  TORCH_CHECK(O.is_cuda() && O.dim() == 4 && O.size(2) == 1 && O.stride(3) == 1, "O must be [B, H, 1, D]");
  const int64_t B = O.size(0), H = O.size(1), D = O.size(3);
  TORCH_CHECK(slots.size(1) == B * H * (D + 2), "slots has the wrong row length for O");
  TORCH_CHECK(LSE.is_cuda() && LSE.scalar_type() == at::kFloat && LSE.is_contiguous() && LSE.numel() == B * H,
              "LSE must be a contiguous fp32 CUDA tensor with B*H elements");
  const c10::cuda::CUDAGuard guard(O.device());
  check_status(tf_decode_gathered(slots.data_ptr<float>(), (int32_t)slots.size(0), (int32_t)B, (int32_t)H,
                                  (int32_t)D, dtype_code(O), O.data_ptr(), O.stride(0), O.stride(1),
                                  LSE.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream()));
}

void flash_decoding_partial_scatter(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V,
                                    int64_t peer_table, int64_t rank, int64_t world, int64_t slot_offset,
                                    int64_t flag_offset, int64_t step, int64_t kv_chunk, int64_t num_splits,
                                    double softmax_scale) {
  TfDecodeDesc d = decode_desc(Q, K, V, kv_chunk, num_splits, softmax_scale);
  const c10::cuda::CUDAGuard guard(Q.device());
  at::Tensor ws = decode_workspace(d, Q);
  check_status(tf_decode_partial_scatter(Q.data_ptr(), K.data_ptr(), V.data_ptr(), ws.data_ptr(),
                                         (uint64_t)ws.numel() * 4, &d, reinterpret_cast<const void*>(peer_table),
                                         (int32_t)rank, (int32_t)world, slot_offset, flag_offset, (uint32_t)step,
                                         at::cuda::getCurrentCUDAStream().stream()));
}

void flash_decoding_gathered_wait(const at::Tensor& slots, const at::Tensor& flags, int64_t step, at::Tensor& O,
                                  at::Tensor& LSE) {
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kFloat && slots.is_contiguous() && slots.dim() == 2,
              "slots must be a contiguous fp32 CUDA tensor [n_ranks, B*H*(D+2)]");
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.is_contiguous() &&
                  flags.numel() >= slots.size(0),
              "flags must be a contiguous int32 CUDA tensor with one word per rank");
  TORCH_CHECK(O.is_cuda() && O.dim() == 4 && O.size(2) == 1 && O.stride(3) == 1, "O must be [B, H, 1, D]");
  const int64_t B = O.size(0), H = O.size(1), D = O.size(3);
  TORCH_CHECK(slots.size(1) == B * H * (D + 2), "slots has the wrong row length for O");
  TORCH_CHECK(LSE.is_cuda() && LSE.scalar_type() == at::kFloat && LSE.is_contiguous() && LSE.numel() == B * H,
              "LSE must be a contiguous fp32 CUDA tensor with B*H elements");
  const c10::cuda::CUDAGuard guard(O.device());
  check_status(tf_decode_gathered_wait(slots.data_ptr<float>(), reinterpret_cast<const uint32_t*>(flags.data_ptr<int>()),
                                       (int32_t)slots.size(0), (uint32_t)step, (int32_t)B, (int32_t)H, (int32_t)D,
                                       dtype_code(O), O.data_ptr(), O.stride(0), O.stride(1), LSE.data_ptr<float>(),
                                       at::cuda::getCurrentCUDAStream().stream()));
}

// Same schema and operand conventions as TileFusion's fused_two_gemms
// (include/kernels/kernel_list.hpp:20-23, src/kernels/fused_two_gemms.cu:66-144):
// A [M, K] and D [M, P] row-major, B given as [N, K], C given as [P, N].
void fused_two_gemms(const at::Tensor& A, const at::Tensor& B, const at::Tensor& C, at::Tensor& D, int64_t tm,
                     int64_t tn, int64_t tk, int64_t tp) {
  (void)tm; (void)tn; (void)tk; (void)tp;      // tile hints: the registry's tiles are used
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && C.is_cuda() && D.is_cuda(), "A, B, C and D must be CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && C.dim() == 2 && D.dim() == 2, "A, B, C and D must be matrices");
  TORCH_CHECK(A.scalar_type() == B.scalar_type() && A.scalar_type() == C.scalar_type() &&
                  A.scalar_type() == D.scalar_type(),
              "A, B, C and D must share one dtype");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && C.stride(1) == 1 && D.stride(1) == 1,
              "rows of A, B, C and D must be contiguous");
  const int64_t m = A.size(0), k = A.size(1), n = B.size(0), p = C.size(0);
  TORCH_CHECK(B.size(1) == k && C.size(1) == n && D.size(0) == m && D.size(1) == p,
              "expected A [M, K], B [N, K], C [P, N], D [M, P]");
  const c10::cuda::CUDAGuard guard(A.device());
  check_status(tf_fused_two_gemms(A.data_ptr(), B.data_ptr(), C.data_ptr(), D.data_ptr(), (int32_t)m, (int32_t)n,
                                  (int32_t)k, (int32_t)p, dtype_code(A), A.stride(0), B.stride(0), C.stride(0),
                                  D.stride(0), at::cuda::getCurrentCUDAStream().stream()));
}

TF_REGISTER_OP(flash_attention,
               "flash_attention(Tensor Q, Tensor K, Tensor V, Tensor(a!) O, "
               "int tile_length_q, int tile_length_kv, "
               "int tile_hidden_qk, int tile_hidden_v, "
               "float softmax_scale, bool causal) -> ()",
               &flash_attention);

TF_REGISTER_OP(flash_attention_lse,
               "flash_attention_lse(Tensor Q, Tensor K, Tensor V, Tensor(a!) O, Tensor(b!) LSE, "
               "int tile_length_q, int tile_length_kv, float softmax_scale, bool causal) -> ()",
               &flash_attention_lse);

TF_REGISTER_OP(flash_attention_bwd,
               "flash_attention_bwd(Tensor Q, Tensor K, Tensor V, Tensor O, Tensor dO, Tensor LSE, "
               "Tensor(a!) dQ, Tensor(b!) dK, Tensor(c!) dV, float softmax_scale, bool causal) -> ()",
               &flash_attention_bwd);

TF_REGISTER_OP(flash_decoding,
               "flash_decoding(Tensor Q, Tensor K, Tensor V, Tensor(a!) O, Tensor(b!) LSE, "
               "int kv_chunk, int num_splits, float softmax_scale, float k_scale=1.0, float v_scale=1.0) -> ()",
               &flash_decoding);

TF_REGISTER_OP(flash_decoding_paged,
               "flash_decoding_paged(Tensor Q, Tensor K_pages, Tensor V_pages, Tensor block_table, int kv_len, "
               "Tensor(a!) O, Tensor(b!) LSE, int kv_chunk, int num_splits, float softmax_scale, "
               "float k_scale=1.0, float v_scale=1.0) -> ()",
               &flash_decoding_paged);

TF_REGISTER_OP(flash_decoding_partial,
               "flash_decoding_partial(Tensor Q, Tensor K, Tensor V, Tensor(a!) slot, "
               "int kv_chunk, int num_splits, float softmax_scale) -> ()",
               &flash_decoding_partial);

TF_REGISTER_OP(flash_decoding_gathered,
               "flash_decoding_gathered(Tensor slots, Tensor(a!) O, Tensor(b!) LSE) -> ()",
               &flash_decoding_gathered);

TF_REGISTER_OP(flash_decoding_partial_scatter,
               "flash_decoding_partial_scatter(Tensor Q, Tensor K, Tensor V, int peer_table, int rank, int world, "
               "int slot_offset, int flag_offset, int step, int kv_chunk, int num_splits, "
               "float softmax_scale) -> ()",
               &flash_decoding_partial_scatter);

TF_REGISTER_OP(flash_decoding_gathered_wait,
               "flash_decoding_gathered_wait(Tensor slots, Tensor flags, int step, Tensor(a!) O, "
               "Tensor(b!) LSE) -> ()",
               &flash_decoding_gathered_wait);

TF_REGISTER_OP(fp8_quantize, "fp8_quantize(Tensor src, Tensor(a!) dst, float factor) -> ()", &fp8_quantize);

TF_REGISTER_OP(fp8_dequantize, "fp8_dequantize(Tensor src, Tensor(a!) dst, float factor) -> ()", &fp8_dequantize);

TF_REGISTER_OP(fused_two_gemms,
               "fused_two_gemms(Tensor A, Tensor B, Tensor C, Tensor(a!) D, "
               "int tm, int tn, int tk, int tp) ->()",
               &fused_two_gemms);

}  // namespace

TORCH_LIBRARY(tilefusion, m) {
  for (const OpEntry& e : op_table()) m.def(e.schema);
}

TORCH_LIBRARY_IMPL(tilefusion, CUDA, m) {
  for (const OpEntry& e : op_table()) e.bind(m, e.name);
}

}  // namespace tilefusion_b200
