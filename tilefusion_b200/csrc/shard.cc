// Host side of the single-box multi-GPU layer (one process per GPU).
//
// TileFusion has no distributed code; this file adds the two partitionings the
// attention path needs, as plain C entry points so that any host (torch, C,
// cgo, JNI) can drive them:
//   * prefill shards by (batch x heads) -- independent problems, no exchange:
//     tf_prefill_sharded computes this rank's contiguous slice of the flattened
//     (batch, head) axis and launches the attention kernel on it;
//   * long-context decode shards by KV length: every rank reduces its keys to
//     one (O, m, l) row per (batch, head) and the ranks exchange those rows.
//     A TfShardCtx owns everything a step needs (gather areas, flags, arrival
//     counters, split-KV workspace), so a step allocates nothing:
//       transport p2p  -- the gather buffers of all ranks are mapped into every
//         process (CUDA IPC); the decode kernel stores its merged rows into all
//         of them, raises a flag, waits for the other ranks' flags and writes
//         the final O / LSE: ONE launch per step, no collective;
//       transport nccl -- the kernel writes this rank's slot, ncclAllGather (in
//         place) moves the slots, a combine kernel finishes.
// NCCL is used through dlopen so that the library neither links it nor needs it
// for single-GPU use; it also carries the IPC handles at set-up.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "internal.h"
#include "registry.h"
#include "tilefusion_b200.h"

namespace {

using tfb::set_error;

#define TF_SHARD_CUDA(expr)                                                              \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return set_error(TF_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));    \
  } while (0)

// ---- NCCL, bound at run time ------------------------------------------------
// Only the handful of entry points used here; the types below are NCCL's stable
// public ABI (ncclUniqueId is 128 opaque bytes, ncclComm_t an opaque pointer).
struct NcclId {
  char bytes[TF_NCCL_ID_BYTES];
};
using NcclComm = void*;
constexpr int kNcclUint8 = 1, kNcclInt32 = 2, kNcclFloat32 = 7;   // ncclDataType_t
constexpr int kNcclMin = 3;                                       // ncclRedOp_t

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string why;      // non-empty when loading failed
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    // (a process that already has NCCL loaded, e.g. through torch, gets that copy)
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle != nullptr) break;
    }
    if (api.handle == nullptr) {
      api.why = std::string("libnccl.so.2 could not be loaded: ") + (dlerror() ? dlerror() : "unknown");
      return;
    }
    auto bind = [&](const char* sym) -> void* {
      void* p = dlsym(api.handle, sym);
      if (p == nullptr && api.why.empty()) api.why = std::string("NCCL symbol missing: ") + sym;
      return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(bind("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(bind("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(bind("ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(bind("ncclAllGather"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(bind("ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(bind("ncclGetErrorString"));
  });
  return api;
}

int nccl_fail(const char* what, int rc) {
  const char* text = nccl().GetErrorString != nullptr ? nccl().GetErrorString(rc) : "?";
  return set_error(TF_ERR_CUDA, "%s failed: NCCL error %d (%s)", what, rc, text);
}

constexpr int kMaxRanks = 64;
constexpr int kFlagWords = 64;

}  // namespace

// The context of one rank of a KV-sharded decoder (opaque to callers).
struct TfShardCtx {
  int rank = 0, world = 1, device = 0;
  int transport = TF_TRANSPORT_P2P;
  int batch = 0, heads = 0, head_dim = 0, dtype = 0;
  NcclComm comm = nullptr;
  float* buffer = nullptr;            // [2 areas][world][rows*(D+2)] floats, then kFlagWords flag words
  long long area_floats = 0;          // world * rows * (D+2)
  long long flag_offset = 0;          // 2 * area_floats
  float** peer_table_dev = nullptr;   // device array [world]: every rank's `buffer` as mapped here
  void* peer_mapping[kMaxRanks] = {}; // IPC mappings opened by this process (to close)
  void* workspace = nullptr;          // split-KV partial rows; grows on demand
  uint64_t workspace_bytes = 0;
  int splits_of_workspace = 0;        // split count the flag words in the workspace were laid out for
  unsigned* counters = nullptr;       // the merged-row count of the step in flight
  unsigned step = 0;
  std::string note;                   // why p2p was not used, if it was asked for
};

namespace {

void release(TfShardCtx* c) {
  if (c == nullptr) return;
  cudaDeviceSynchronize();
  for (int p = 0; p < c->world && p < kMaxRanks; ++p)
    if (c->peer_mapping[p] != nullptr) cudaIpcCloseMemHandle(c->peer_mapping[p]);
  if (c->peer_table_dev != nullptr) cudaFree(c->peer_table_dev);
  if (c->workspace != nullptr) cudaFree(c->workspace);
  if (c->counters != nullptr) cudaFree(c->counters);
  if (c->buffer != nullptr) cudaFree(c->buffer);
  if (c->comm != nullptr && nccl().CommDestroy != nullptr) nccl().CommDestroy(c->comm);
  delete c;
}

// Maps every rank's gather buffer into this process and builds the device-side
// pointer table.  Collective over the communicator.  Returns TF_OK with
// *all_ok = 0 when some rank could not map a peer (the caller then falls back
// to the NCCL transport on every rank alike).
int map_peers(TfShardCtx* c, int* all_ok) {
  NcclApi& api = nccl();
  cudaIpcMemHandle_t mine;
  int ok_local = 1;
  std::string why;
  if (cudaIpcGetMemHandle(&mine, c->buffer) != cudaSuccess) {
    ok_local = 0;
    why = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(cudaGetLastError());
    std::memset(&mine, 0, sizeof(mine));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "unexpected IPC handle size");
  unsigned char* stage = nullptr;
  TF_SHARD_CUDA(cudaMalloc(&stage, (size_t)c->world * 64 + 2 * sizeof(int)));
  TF_SHARD_CUDA(cudaMemcpy(stage + (size_t)c->rank * 64, &mine, 64, cudaMemcpyHostToDevice));
  int rc = api.AllGather(stage + (size_t)c->rank * 64, stage, 64, kNcclUint8, c->comm, nullptr);
  if (rc != 0) {
    cudaFree(stage);
    return nccl_fail("ncclAllGather (IPC handles)", rc);
  }
  TF_SHARD_CUDA(cudaStreamSynchronize(nullptr));
  cudaIpcMemHandle_t all[kMaxRanks];
  TF_SHARD_CUDA(cudaMemcpy(all, stage, (size_t)c->world * 64, cudaMemcpyDeviceToHost));
  float* table[kMaxRanks] = {};
  for (int p = 0; p < c->world && ok_local; ++p) {
    if (p == c->rank) {
      table[p] = c->buffer;
      continue;
    }
    void* mapped = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&mapped, all[p], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      ok_local = 0;
      why = std::string("cudaIpcOpenMemHandle(rank ") + std::to_string(p) + "): " + cudaGetErrorString(e);
      cudaGetLastError();
      break;
    }
    c->peer_mapping[p] = mapped;
    table[p] = static_cast<float*>(mapped);
  }
  // every rank must take the same transport
  int* flag_dev = reinterpret_cast<int*>(stage + (size_t)c->world * 64);
  TF_SHARD_CUDA(cudaMemcpy(flag_dev, &ok_local, sizeof(int), cudaMemcpyHostToDevice));
  rc = api.AllReduce(flag_dev, flag_dev + 1, 1, kNcclInt32, kNcclMin, c->comm, nullptr);
  if (rc != 0) {
    cudaFree(stage);
    return nccl_fail("ncclAllReduce (transport agreement)", rc);
  }
  TF_SHARD_CUDA(cudaStreamSynchronize(nullptr));
  TF_SHARD_CUDA(cudaMemcpy(all_ok, flag_dev + 1, sizeof(int), cudaMemcpyDeviceToHost));
  TF_SHARD_CUDA(cudaFree(stage));
  if (*all_ok) {
    TF_SHARD_CUDA(cudaMalloc(&c->peer_table_dev, sizeof(float*) * c->world));
    TF_SHARD_CUDA(cudaMemcpy(c->peer_table_dev, table, sizeof(float*) * c->world, cudaMemcpyHostToDevice));
  } else {
    for (int p = 0; p < c->world; ++p)
      if (c->peer_mapping[p] != nullptr) {
        cudaIpcCloseMemHandle(c->peer_mapping[p]);
        c->peer_mapping[p] = nullptr;
      }
    c->note = ok_local ? "another rank could not map its peers' gather buffers" : why;
  }
  return TF_OK;
}

int check_rank(int rank, int world) {
  if (world < 1 || world > kMaxRanks) return set_error(TF_ERR_BAD_ARG, "world size %d is outside [1, %d]", world, kMaxRanks);
  if (rank < 0 || rank >= world) return set_error(TF_ERR_BAD_ARG, "rank %d is outside a world of %d", rank, world);
  return TF_OK;
}

}  // namespace

extern "C" {

int tf_shard_head_slice(int64_t n_heads_total, int32_t rank, int32_t world, int64_t* begin, int64_t* end) {
  if (begin == nullptr || end == nullptr) return set_error(TF_ERR_BAD_ARG, "begin / end is null");
  if (int rc = check_rank(rank, world)) return rc;
  if (n_heads_total < 0) return set_error(TF_ERR_BAD_ARG, "n_heads_total must be non-negative");
  tfb::shard_range(n_heads_total, rank, world, begin, end);
  return TF_OK;
}

int tf_shard_kv_slice(int64_t len_kv, int32_t rank, int32_t world, int32_t align, int64_t* begin, int64_t* end) {
  if (begin == nullptr || end == nullptr) return set_error(TF_ERR_BAD_ARG, "begin / end is null");
  if (int rc = check_rank(rank, world)) return rc;
  if (len_kv < 0) return set_error(TF_ERR_BAD_ARG, "len_kv must be non-negative");
  if (align < 1) return set_error(TF_ERR_BAD_ARG, "align must be positive");
  int64_t b0, b1;
  tfb::shard_range((len_kv + align - 1) / align, rank, world, &b0, &b1);
  *begin = b0 * align < len_kv ? b0 * align : len_kv;
  *end = b1 * align < len_kv ? b1 * align : len_kv;
  return TF_OK;
}

int tf_shard_unique_id(void* id_out) {
  if (id_out == nullptr) return set_error(TF_ERR_BAD_ARG, "id_out is null");
  NcclApi& api = nccl();
  if (!api.why.empty()) return set_error(TF_ERR_UNSUPPORTED, "%s", api.why.c_str());
  NcclId id;
  if (int rc = api.GetUniqueId(&id)) return nccl_fail("ncclGetUniqueId", rc);
  std::memcpy(id_out, id.bytes, TF_NCCL_ID_BYTES);
  return TF_OK;
}

int tf_shard_create(int32_t rank, int32_t world, const void* nccl_id, int32_t transport, int32_t batch,
                    int32_t heads, int32_t head_dim, int32_t dtype, TfShardCtx** out) {
  if (out == nullptr) return set_error(TF_ERR_BAD_ARG, "out is null");
  *out = nullptr;
  if (int rc = check_rank(rank, world)) return rc;
  if (transport != TF_TRANSPORT_AUTO && transport != TF_TRANSPORT_P2P && transport != TF_TRANSPORT_NCCL)
    return set_error(TF_ERR_BAD_ARG, "transport %d is none of TF_TRANSPORT_AUTO / _P2P / _NCCL", transport);
  if (batch < 1 || heads < 1) return set_error(TF_ERR_BAD_ARG, "batch and heads must be positive (got %d, %d)", batch, heads);
  if (head_dim != 64 && head_dim != 128)
    return set_error(TF_ERR_UNSUPPORTED, "head_dim %d has no compiled decode variant (64 and 128 do)", head_dim);
  if (dtype != TF_F16 && dtype != TF_BF16) return set_error(TF_ERR_UNSUPPORTED, "dtype code %d is not fp16 or bf16", dtype);
  if (world > 1 && nccl_id == nullptr)
    return set_error(TF_ERR_BAD_ARG, "nccl_id is null: with more than one rank every rank passes the id rank 0 made");
  if (world > 1 && !nccl().why.empty()) return set_error(TF_ERR_UNSUPPORTED, "%s", nccl().why.c_str());

  TfShardCtx* c = new (std::nothrow) TfShardCtx;
  if (c == nullptr) return set_error(TF_ERR_CUDA, "out of host memory");
  c->rank = rank;
  c->world = world;
  c->batch = batch;
  c->heads = heads;
  c->head_dim = head_dim;
  c->dtype = dtype;
  auto give_up = [&](int rc) {
    release(c);
    return rc;
  };
#define TF_CREATE_CUDA(expr)                                                                        \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess)                                                                         \
      return give_up(set_error(TF_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)));      \
  } while (0)
  TF_CREATE_CUDA(cudaGetDevice(&c->device));
  const long long rows = (long long)batch * heads;
  c->area_floats = (long long)world * rows * (head_dim + 2);
  c->flag_offset = 2 * c->area_floats;
  const size_t buffer_bytes = (size_t)(c->flag_offset + kFlagWords) * sizeof(float);
  TF_CREATE_CUDA(cudaMalloc(&c->buffer, buffer_bytes));
  TF_CREATE_CUDA(cudaMemset(c->buffer, 0, buffer_bytes));
  TF_CREATE_CUDA(cudaMalloc(&c->counters, 64));
  TF_CREATE_CUDA(cudaMemset(c->counters, 0, 64));
  // flags and counters are zero on this rank before any peer can learn the buffer's address
  TF_CREATE_CUDA(cudaDeviceSynchronize());

  if (world > 1) {
    NcclId id;
    std::memcpy(id.bytes, nccl_id, TF_NCCL_ID_BYTES);
    if (int rc = nccl().CommInitRank(&c->comm, world, id, rank)) return give_up(nccl_fail("ncclCommInitRank", rc));
  }
  c->transport = transport == TF_TRANSPORT_NCCL ? TF_TRANSPORT_NCCL : TF_TRANSPORT_P2P;
  if (c->transport == TF_TRANSPORT_P2P) {
    if (world == 1) {
      TF_CREATE_CUDA(cudaMalloc(&c->peer_table_dev, sizeof(float*)));
      TF_CREATE_CUDA(cudaMemcpy(c->peer_table_dev, &c->buffer, sizeof(float*), cudaMemcpyHostToDevice));
    } else {
      int all_ok = 0;
      if (int rc = map_peers(c, &all_ok)) return give_up(rc);
      if (!all_ok) {
        if (transport == TF_TRANSPORT_P2P)
          return give_up(set_error(TF_ERR_UNSUPPORTED, "the peer-memory transport is not available: %s", c->note.c_str()));
        c->transport = TF_TRANSPORT_NCCL;
      }
    }
  }
#undef TF_CREATE_CUDA
  *out = c;
  return TF_OK;
}

int tf_shard_transport(const TfShardCtx* ctx) {
  if (ctx == nullptr) return set_error(TF_ERR_BAD_ARG, "ctx is null");
  return ctx->transport;
}

const char* tf_shard_note(const TfShardCtx* ctx) { return ctx == nullptr ? "" : ctx->note.c_str(); }

int tf_shard_destroy(TfShardCtx* ctx) {
  if (ctx == nullptr) return TF_OK;
  const int ctx_dev = ctx->device;
  int dev = ctx_dev;
  if (cudaGetDevice(&dev) == cudaSuccess && dev != ctx_dev) cudaSetDevice(ctx_dev);
  release(ctx);
  if (dev != ctx_dev) cudaSetDevice(dev);
  return TF_OK;
}

int tf_decode_sharded(TfShardCtx* c, const void* q, const void* k_local, const void* v_local, void* o,
                      float* lse, const TfDecodeDesc* desc, void* stream) {
  if (c == nullptr) return set_error(TF_ERR_BAD_ARG, "ctx is null");
  if (desc == nullptr) return set_error(TF_ERR_BAD_ARG, "desc is null");
  if (o == nullptr) return set_error(TF_ERR_BAD_ARG, "o is null");
  if (desc->batch != c->batch || desc->heads != c->heads || desc->head_dim != c->head_dim || desc->dtype != c->dtype)
    return set_error(TF_ERR_BAD_ARG,
                     "desc (batch %d, heads %d, head_dim %d, dtype %d) does not match the context (%d, %d, %d, %d)",
                     desc->batch, desc->heads, desc->head_dim, desc->dtype, c->batch, c->heads, c->head_dim, c->dtype);
  int dev = 0;
  TF_SHARD_CUDA(cudaGetDevice(&dev));
  if (dev != c->device) return set_error(TF_ERR_BAD_ARG, "the context belongs to device %d but device %d is current", c->device, dev);
  // A wait of an earlier step that gave up (a rank that never arrived) left NaN
  // rows and this code; it is reported before anything else is launched.
  if (int rc = tf_device_status_peek(nullptr)) return rc;
  TfDecodePlan plan;
  if (int rc = tf_decode_plan(desc, &plan)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // partial rows, then one flag word per (b, h, split) for the fused tail
  const uint64_t ws_need = plan.workspace_bytes + (uint64_t)c->batch * c->heads * plan.num_splits * sizeof(unsigned);
  if (ws_need > c->workspace_bytes || plan.num_splits != c->splits_of_workspace) {
    // first call, or a differently split shard than the last one: the only allocation a
    // step can make.  The flag words must start below every step number still to come.
    if (c->workspace != nullptr && ws_need > c->workspace_bytes) {
      TF_SHARD_CUDA(cudaStreamSynchronize(s));
      TF_SHARD_CUDA(cudaFree(c->workspace));
      c->workspace = nullptr;
      c->workspace_bytes = 0;
    }
    if (c->workspace == nullptr) {
      TF_SHARD_CUDA(cudaMalloc(&c->workspace, ws_need));
      c->workspace_bytes = ws_need;
    }
    TF_SHARD_CUDA(cudaMemsetAsync(c->workspace, 0, c->workspace_bytes, s));
    c->splits_of_workspace = plan.num_splits;
  }
  c->step += 1;
  const long long rows = (long long)c->batch * c->heads;
  tfb::ShardStep st;
  st.workspace = c->workspace;
  st.workspace_bytes = c->workspace_bytes;
  st.rows_done = c->counters;
  st.peer_table = c->transport == TF_TRANSPORT_P2P ? c->peer_table_dev : nullptr;
  st.local_base = c->buffer;
  st.n_ranks = c->world;
  st.rank = c->rank;
  st.area_offset = (long long)(c->step & 1u) * c->area_floats;
  st.flag_offset = c->flag_offset;
  st.step = c->step;
  if (int rc = tfb::launch_sharded_decode(q, k_local, v_local, o, lse, desc, st, s)) return rc;
  if (c->transport == TF_TRANSPORT_P2P) return TF_OK;
  float* area = c->buffer + st.area_offset;
  const size_t slot_floats = (size_t)rows * (c->head_dim + 2);
  if (c->world > 1) {
    if (int rc = nccl().AllGather(area + (size_t)c->rank * slot_floats, area, slot_floats, kNcclFloat32, c->comm, s))
      return nccl_fail("ncclAllGather", rc);
  }
  return tf_decode_gathered(area, c->world, c->batch, c->heads, c->head_dim, c->dtype, o, desc->o_stride_b,
                            desc->o_stride_h, lse, stream);
}

int tf_prefill_sharded(int32_t rank, int32_t world, const void* q, const void* k, const void* v, void* o,
                       float* lse, const TfAttnDesc* desc, void* stream, int64_t* begin_out, int64_t* end_out) {
  if (desc == nullptr) return set_error(TF_ERR_BAD_ARG, "desc is null");
  if (int rc = check_rank(rank, world)) return rc;
  if (desc->batch < 1 || desc->heads < 1) return set_error(TF_ERR_BAD_ARG, "batch and heads must be positive");
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr)
    return set_error(TF_ERR_BAD_ARG, "q, k, v and o must be non-null");
  int64_t h0, h1;
  tfb::shard_range((int64_t)desc->batch * desc->heads, rank, world, &h0, &h1);
  if (begin_out != nullptr) *begin_out = h0;
  if (end_out != nullptr) *end_out = h1;
  // The slice [h0, h1) of the flattened (batch, head) axis is covered by at most
  // three rectangular pieces: the tail of a first batch entry, whole entries,
  // and the head of a last one.
  const int64_t H = desc->heads;
  auto run = [&](int64_t b, int64_t nb, int64_t h, int64_t nh) -> int {
    if (nb <= 0 || nh <= 0) return TF_OK;
    TfAttnDesc d = *desc;
    d.batch = (int32_t)nb;
    d.heads = (int32_t)nh;
    auto at = [&](const void* base, int64_t sb, int64_t sh) {
      return static_cast<const char*>(base) + (b * sb + h * sh) * 2;
    };
    float* lse_piece = lse == nullptr ? nullptr : lse + (b * H + h) * (int64_t)desc->len_q;
    return tf_attn_fwd(at(q, desc->q_stride_b, desc->q_stride_h), at(k, desc->k_stride_b, desc->k_stride_h),
                       at(v, desc->v_stride_b, desc->v_stride_h),
                       const_cast<char*>(at(o, desc->o_stride_b, desc->o_stride_h)), lse_piece, &d, stream);
  };
  int64_t h = h0;
  if (h < h1 && h % H != 0) {                       // tail of a first batch entry
    const int64_t stop = (h / H + 1) * H < h1 ? (h / H + 1) * H : h1;
    if (int rc = run(h / H, 1, h % H, stop - h)) return rc;
    h = stop;
  }
  if (h1 - h >= H) {                                // whole batch entries
    const int64_t nb = (h1 - h) / H;
    if (int rc = run(h / H, nb, 0, H)) return rc;
    h += nb * H;
  }
  if (h < h1) return run(h / H, 1, 0, h1 - h);      // head of a last entry
  return TF_OK;
}

}  // extern "C"
