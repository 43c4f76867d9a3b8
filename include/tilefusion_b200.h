/*
 * tilefusion_b200 -- C-ABI of the fused-attention path (prefill + flash
 * decoding) for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and strides; no torch
 * types cross this boundary.  The torch operator layer
 * (tilefusion_b200/csrc/torch_bind.cc) and the tests bind exactly these
 * symbols.  All functions return 0 on success or a negative TfStatus; the
 * text of the last failure on the calling thread is available from
 * tf_last_error().  Nothing here calls exit() or abort().
 *
 * Which interface of microsoft/TileFusion each entry point stands in for is
 * cited as file:line (paths relative to the TileFusion source tree).
 */
#ifndef TILEFUSION_B200_H_
#define TILEFUSION_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TF_EXPORT __attribute__((visibility("default")))

typedef enum TfStatus {
  TF_OK = 0,
  TF_ERR_BAD_ARG = -1,       /* null pointer, non-positive size, bad stride   */
  TF_ERR_UNSUPPORTED = -2,   /* shape / dtype / layout with no compiled kernel */
  TF_ERR_CUDA = -3,          /* a CUDA runtime or driver call failed          */
  TF_ERR_DEVICE_TIMEOUT = -4,/* a bounded device-side wait ran out            */
  TF_ERR_WORKSPACE = -5      /* caller's workspace is too small               */
} TfStatus;

typedef enum TfDType {
  TF_F16 = 0,
  TF_BF16 = 1,
  /* 8-bit storage types (OCP 8-bit floating point: e4m3 without infinities,
   * e5m2 IEEE-like), the ones TileFusion declares in include/types/base.hpp:13-39.
   * Accepted only where a descriptor says so (TfDecodeDesc.kv_dtype).          */
  TF_FP8_E4M3 = 2,
  TF_FP8_E5M2 = 3
} TfDType;

/*
 * Prefill attention problem: O = softmax(Q K^T * scale [+ causal]) V, fp32
 * accumulation, one independent problem per (batch, head).
 *
 * All strides are in ELEMENTS.  Q and O rows must be contiguous (stride 1
 * along the head dimension).  K is addressed as K[l, d] and V as V[l, d]; for
 * each of them exactly one of (stride_l, stride_d) must be 1:
 *   k_stride_d == 1 : K stored [Lk, D] row-major  (the operand layout of
 *                     TileFusion's op, src/kernels/flash_attn.cu:73-76)
 *   k_stride_l == 1 : K stored [D, Lk] row-major  (the `key` argument of
 *                     python/ops/flash_attention.py:45-83 before its .t() copy)
 *   v_stride_d == 1 : V stored [Lk, Dv] row-major (the `value` argument there)
 *   v_stride_l == 1 : V stored [Dv, Lk] row-major (the op's V^T operand)
 * Both forms feed the tensor cores directly (K-major / MN-major shared-memory
 * descriptors); no transposing copy is ever made.
 */
typedef struct TfAttnDesc {
  int32_t dtype;        /* TfDType                                            */
  int32_t batch;        /* B                                                  */
  int32_t heads;        /* H                                                  */
  int32_t len_q;        /* Lq >= 1                                            */
  int32_t len_kv;       /* Lk >= 1                                            */
  int32_t head_dim;     /* D:  a multiple of 8 in [8, 256]                    */
  int32_t head_dim_v;   /* Dv: a multiple of 8 in [8, 256]; may differ from D.
                           Kernels are compiled for 64, 128 and 256; other
                           widths run zero-padded on the next one (TMA fills
                           the padding), which is exact.                      */
  int32_t causal;       /* 1: mask key index > query index (top-left aligned,
                           include/cell/mask.hpp:19-113)                      */
  float softmax_scale;  /* multiplies Q K^T before the softmax                */
  int32_t tile_q;       /* hint; 0 lets the registry choose                   */
  int32_t tile_kv;      /* hint; 0 lets the registry choose                   */
  int32_t reserved;
  int64_t q_stride_b, q_stride_h, q_stride_l;
  int64_t k_stride_b, k_stride_h, k_stride_l, k_stride_d;
  int64_t v_stride_b, v_stride_h, v_stride_l, v_stride_d;
  int64_t o_stride_b, o_stride_h, o_stride_l;
} TfAttnDesc;

/*
 * Flash-decoding problem: one query row per (batch, head) against Lk keys.
 * With heads_kv < heads (grouped-query attention) the query heads of a group
 * are processed together on the tensor cores as the rows of one small
 * attention problem per KV head, so K/V are still read from HBM once.
 * Q[B,H,D], K[B,H,Lk,D], V[B,H,Lk,D], O[B,H,D]; rows of K and V are
 * contiguous with stride D between consecutive keys.  Strides in elements.
 */
typedef struct TfDecodeDesc {
  int32_t dtype;        /* TfDType                                            */
  int32_t batch;
  int32_t heads;
  int32_t len_kv;       /* keys held by THIS call (a shard when KV is split
                           across GPUs); may be 0                             */
  int32_t head_dim;     /* D in {64, 128}                                     */
  int32_t kv_chunk;     /* keys per chunk, a multiple of 128, at most 1024;
                           0 -> 512 (1024 for an 8-bit cache)                 */
  int32_t num_splits;   /* splits per (b,h); 0 lets the registry choose       */
  float softmax_scale;
  int64_t q_stride_b, q_stride_h;
  int64_t k_stride_b, k_stride_h;
  int64_t v_stride_b, v_stride_h;
  int64_t o_stride_b, o_stride_h;
  int32_t heads_kv;     /* KV heads; 0 or == heads: one KV head per query head.
                           Otherwise grouped-query decoding: heads % heads_kv
                           == 0, K/V are [B, heads_kv, Lk, D] (k/v_stride_h
                           step over KV heads) and query head h reads KV head
                           h / (heads / heads_kv).                            */
  int32_t page_size;    /* paged KV cache: keys per page, a multiple of 128;
                           0 = K/V are contiguous per (batch, KV head)        */
  const int32_t* block_table; /* device pointer, [batch][max_pages]: page holding
                           keys [i*page_size, (i+1)*page_size) of a batch entry;
                           used only when page_size > 0                       */
  int32_t max_pages;    /* row length of block_table                          */
  int32_t num_pages;    /* pages in the pool (extent of K and V)              */
  int64_t k_stride_page, v_stride_page; /* elements between consecutive pages;
                           with paging K/V are [num_pages][H_kv][page_size][D]
                           addressed by (k/v_stride_page, k/v_stride_h) and
                           k/v_stride_b are ignored.  Rows of a sequence's last
                           page beyond len_kv must hold finite values.        */
  int32_t kv_dtype;     /* stored element of K and V: 0 or == dtype: the query's
                           type; TF_FP8_E4M3 / TF_FP8_E5M2: one byte per element
                           (K/V strides then count bytes and are multiples of
                           16).  Q, O stay `dtype`; all arithmetic is fp32.
                           With heads_kv < heads every query head is a work
                           item of its own that streams its KV head's bytes
                           (the re-reads of a group meet in L2): half the cache
                           memory of 16 bits, faster than the 16-bit grouped
                           path only up to two query heads per KV head.       */
  float k_scale;        /* dequantisation factors of an 8-bit cache: key =     */
  float v_scale;        /* k_scale * stored, value = v_scale * stored; 0 = 1   */
} TfDecodeDesc;

/* What the registry chose for a decode problem (tf_decode_plan). */
typedef struct TfDecodePlan {
  int32_t num_splits;        /* partial rows per (b,h)                        */
  int32_t chunks_per_split;  /* kv_chunk-sized chunks walked by one split     */
  int32_t kv_chunk;
  int32_t grid;              /* CTAs of the split kernel                      */
  int32_t stages;            /* depth of the shared-memory ring               */
  int32_t reserved;          /* grouped-query decoding: partial rows per (row,
                                split) -- 4 when the query rows of a group are
                                replicated in the kernel (num_splits counts
                                them all), else 0 or 1                        */
  uint64_t workspace_bytes;  /* fp32 partials: B*H*num_splits*(D+2)*4         */
} TfDecodePlan;

/* What the registry chose for a prefill problem (tf_attn_plan). */
typedef struct TfAttnPlan {
  int32_t tile_q;
  int32_t tile_kv;
  int32_t ctas_per_sm;
  int32_t grid;
  int32_t k_mn_major;   /* 1 when K is read as [D, Lk]                        */
  int32_t v_mn_major;   /* 1 when V is read as [Lk, Dv]                       */
  int32_t head_dim_kernel; /* compiled head dim the problem runs on (64/128/256) */
  uint64_t smem_bytes;
} TfAttnPlan;

/* ---- prefill ------------------------------------------------------------ */

/*
 * Fused attention forward on `stream` (a cudaStream_t; NULL = legacy stream).
 * Replaces the host operator tilefusion::kernels::flash_attention
 * (include/kernels/ops.hpp:54-58, src/kernels/flash_attn.cu:58-152) and the
 * kernel it JIT-compiles (include/kernels/flash_attention_device.cuh:130-312).
 * `lse` may be NULL; otherwise it receives log-sum-exp rows, fp32 [B,H,Lq],
 * natural log of sum(exp(scale * q.k)).  Asynchronous: no device sync.
 * Besides the kernel the call enqueues one 4-byte memset (the work-item
 * counter of the launch) on `stream`; both can be captured into a CUDA graph
 * once a first call on the device has been made outside a capture.  Calls on
 * different streams may overlap: every stream keeps a counter word of its own
 * (up to 256 streams per device), and every launch recorded into a CUDA graph
 * gets a word that no other launch ever uses (up to 4096 recorded launches per
 * device), so graphs may replay side by side.  Beyond those limits the call
 * returns TF_ERR_UNSUPPORTED.
 */
TF_EXPORT int tf_attn_fwd(const void* q, const void* k, const void* v, void* o,
                          float* lse, const TfAttnDesc* desc, void* stream);

/*
 * Attention backward: dQ, dK, dV from Q, K, V, O, dO and the log-sum-exp rows
 * (`lse`, fp32 [B,H,Lq], as tf_attn_fwd writes them).  No counterpart in the
 * reference, which has no backward pass; the forward's operand conventions are
 * kept.  `desc` describes the forward problem; K and V are read as [Lk, D] /
 * [Lk, Dv] (k_stride_d == v_stride_d == 1), head_dim == head_dim_v in
 * {64, 128}.  d_o is laid out like o (o's strides), dq like q, dk like k, dv
 * like v.  P and dS are rounded to the 16-bit type before the second products,
 * accumulation is fp32, results are deterministic (no atomics).  `workspace`
 * (tf_attn_bwd_workspace_bytes: B*H*Lq fp32 for the delta rows) is scratch.
 * Three launches on `stream`, asynchronous.
 */
TF_EXPORT int tf_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                          const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                          const TfAttnDesc* desc, void* workspace, uint64_t workspace_bytes,
                          void* stream);
TF_EXPORT uint64_t tf_attn_bwd_workspace_bytes(const TfAttnDesc* desc);

/*
 * Tile plan the registry would use for `desc`.  Stands in for the tile
 * arguments the reference bakes in as template constants
 * (src/kernels/flash_attn.cu:16-55, :87-99) and for its per-shape JIT cache
 * (src/jit/compiler.cc:123-145): variants here are compiled ahead of time and
 * looked up by (dtype, head_dim bucket); sequence lengths, scale and mask are
 * run-time arguments, and head dims between the compiled ones are zero-padded.
 */
TF_EXPORT int tf_attn_plan(const TfAttnDesc* desc, TfAttnPlan* plan);

/*
 * D[m, p] = (A[m, k] * B[n, k]^T) * C[p, n]^T with the intermediate product
 * rounded to the 16-bit dtype and fp32 accumulation in both products: the
 * attention kernel with its softmax stage replaced by a conversion.  Replaces
 * tilefusion::kernels::fused_two_gemms (include/kernels/ops.hpp:47-52,
 * src/kernels/fused_two_gemms.cu:66-144; kernel
 * include/kernels/fused_two_gemms_device.cuh:114-214) with the operand layouts
 * of that operator: A and D row-major, B given as [n, k] and C as [p, n]
 * ("column-major" B and C).  ld* are row strides in elements.  k and p are
 * multiples of 8 up to 256 (they may differ), n a multiple of 8, m arbitrary.
 */
TF_EXPORT int tf_fused_two_gemms(const void* a, const void* b, const void* c, void* d,
                                 int32_t m, int32_t n, int32_t k, int32_t p, int32_t dtype,
                                 int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd,
                                 void* stream);

/* ---- flash decoding (no counterpart in the reference: it has no decode
 *      op; registered in the style of include/kernels/kernel_list.hpp:25-30) */

/* Split count, grid and workspace size for `desc`. */
TF_EXPORT int tf_decode_plan(const TfDecodeDesc* desc, TfDecodePlan* plan);

/*
 * Split-KV pass: for every (b, h, split) writes one partial row into
 * `workspace`: D fp32 of un-normalised output, then (m, l) with m the running
 * maximum of scale*log2(e)*q.k and l the sum of 2^(s-m).
 * Workspace layout: [B*H*num_splits][D] fp32, then [B*H*num_splits][2] fp32.
 */
TF_EXPORT int tf_decode_split(const void* q, const void* k, const void* v,
                              void* workspace, uint64_t workspace_bytes,
                              const TfDecodeDesc* desc, void* stream);

/*
 * Log-sum-exp combine of `n_parts` partial rows per (b,h).
 *   part_o  : fp32, element (p, r, d) at part_o[p*part_stride_o + r*row_stride_o + d]
 *   part_ml : fp32 pairs, (p, r) at part_ml[p*part_stride_ml + r*row_stride_ml]
 * with r = b*H + h in [0, rows).  Exactly one output form is written:
 *   final   : o (dtype, element (r, d) at o[(r/H)*o_stride_b + (r%H)*o_stride_h + d])
 *             and, when non-NULL, lse fp32 [rows] (natural log);
 *   merged  : when out_part_o != NULL, one fp32 partial row per r in the same
 *             (O, then m,l) form: out_part_o[r*D + d], out_part_ml[r*2 + {0,1}].
 */
TF_EXPORT int tf_decode_combine(const float* part_o, const float* part_ml,
                                int32_t n_parts, int64_t part_stride_o,
                                int64_t row_stride_o, int64_t part_stride_ml,
                                int64_t row_stride_ml, int32_t rows,
                                int32_t heads, int32_t head_dim, int32_t dtype,
                                void* o, int64_t o_stride_b, int64_t o_stride_h,
                                float* lse, float* out_part_o,
                                float* out_part_ml, void* stream);

/* Split + combine: O[B,H,D] (dtype) and LSE[B,H] fp32 (may be NULL). */
TF_EXPORT int tf_decode(const void* q, const void* k, const void* v, void* o,
                        float* lse, void* workspace, uint64_t workspace_bytes,
                        const TfDecodeDesc* desc, void* stream);

/*
 * Split + local merge for a KV shard: writes ONE partial row per (b,h) into
 * `slot`, laid out [B*H][D] fp32 followed by [B*H][2] fp32 -- the send slot of
 * an all-gather over the GPUs that hold the other shards.  tf_decode_gathered
 * then combines the gathered slots.
 */
TF_EXPORT int tf_decode_partial(const void* q, const void* k, const void* v,
                                float* slot, void* workspace,
                                uint64_t workspace_bytes,
                                const TfDecodeDesc* desc, void* stream);

/* Final combine over `n_ranks` gathered slots (each B*H*(D+2) fp32). */
TF_EXPORT int tf_decode_gathered(const float* slots, int32_t n_ranks,
                                 int32_t batch, int32_t heads, int32_t head_dim,
                                 int32_t dtype, void* o, int64_t o_stride_b,
                                 int64_t o_stride_h, float* lse, void* stream);

/*
 * KV-sharded decode with the all-gather fused into the kernels (no library
 * collective): tf_decode_partial_scatter is tf_decode_partial whose merge
 * kernel stores its row straight into the gather buffer of EVERY rank through
 * peer-mapped pointers and then raises a flag there; tf_decode_gathered_wait
 * is tf_decode_gathered preceded by a bounded wait on those flags.  No
 * counterpart in the reference (it has no multi-GPU code).
 *
 * `peer_table` is a device array of n_ranks pointers, entry p = base of rank
 * p's symmetric buffer as mapped into this process (for example
 * torch.distributed._symmetric_memory's buffer_ptrs_dev).  Rank r's row block
 * lands at base + slot_offset_floats (the caller adds r * B*H*(D+2) and
 * alternates two buffer halves between consecutive steps); the flag word of
 * sender r is ((uint32_t*)(base + flag_offset_floats))[r] and receives `step`,
 * which must grow by one per step.  One sharded decode may be in flight per
 * device.  Plain peer stores and system-scope release/acquire only -- no TMA
 * and no multicast touch peer memory.
 */
TF_EXPORT int tf_decode_partial_scatter(const void* q, const void* k, const void* v,
                                        void* workspace, uint64_t workspace_bytes,
                                        const TfDecodeDesc* desc, const void* peer_table,
                                        int32_t rank, int32_t n_ranks,
                                        int64_t slot_offset_floats, int64_t flag_offset_floats,
                                        uint32_t step, void* stream);

TF_EXPORT int tf_decode_gathered_wait(const float* slots, const uint32_t* flags,
                                      int32_t n_ranks, uint32_t step, int32_t batch,
                                      int32_t heads, int32_t head_dim, int32_t dtype, void* o,
                                      int64_t o_stride_b, int64_t o_stride_h, float* lse,
                                      void* stream);

/*
 * Flash decoding for callers that cannot allocate device memory.  It has no
 * counterpart in the reference.
 *
 * Some hosts of this library may not call cudaMalloc on the serving path at
 * all: a runtime that hands out one fixed arena at start-up and forbids any
 * later allocation, a plugin loaded into a process whose memory pool it does
 * not own, or code running inside a region where an allocation would
 * synchronise the device.  tf_decode needs a workspace for its split-KV
 * partial rows, which such a caller has nowhere to get.  This variant keeps
 * the partial rows in a fixed 4 MiB array that is part of the library image
 * (each GPU that loads the library holds it until the process exits), so the
 * caller passes only inputs and outputs: same arguments and results as
 * tf_decode minus the workspace.  It calls no cudaMalloc / cudaFree and no
 * allocating routine of any library.
 *
 * Limits and rules:
 *  - the partial rows, B*H*num_splits*(D+2)*4 bytes as reported by
 *    tf_decode_plan, must fit in tf_decode_static_capacity() bytes; a larger
 *    problem is rejected with TF_ERR_WORKSPACE and a message that names both
 *    sizes (pass a smaller num_splits, or use tf_decode);
 *  - the first call on each device looks up the array's device address (with
 *    that device current) before it launches; make that first call outside
 *    any stream capture;
 *  - all calls on a device share the one array, which keeps whatever the last
 *    call left in it.  Nothing in it has to start at zero -- every row that
 *    the combine reads is first written by the split pass of the same call --
 *    but two calls whose kernels overlap on the GPU (different streams, or
 *    several host threads) race on it.  Issue them on one stream, or order
 *    them with events.
 */
TF_EXPORT int tf_decode_static(const void* q, const void* k, const void* v, void* o,
                               float* lse, const TfDecodeDesc* desc, void* stream);

/* Size in bytes of the built-in scratch that tf_decode_static uses. */
TF_EXPORT uint64_t tf_decode_static_capacity(void);

/* ---- single-box multi-GPU layer (one process per GPU) ----------------------
 * No counterpart in the reference: it has no NCCL / peer-access call site.
 * Prefill shards by (batch x heads) with no exchange; long-context decode
 * shards by KV length and exchanges one (O, m, l) row per (batch, head). */

/* [begin, end) of the flattened (batch x heads) axis that `rank` of `world`
 * processes (contiguous; the first n % world ranks take one more). */
TF_EXPORT int tf_shard_head_slice(int64_t n_heads_total, int32_t rank, int32_t world,
                                  int64_t* begin, int64_t* end);

/* [begin, end) of the key axis held by `rank`, boundaries on multiples of
 * `align` keys (128 keeps every TMA stage inside one shard). */
TF_EXPORT int tf_shard_kv_slice(int64_t len_kv, int32_t rank, int32_t world, int32_t align,
                                int64_t* begin, int64_t* end);

/*
 * Runs this rank's slice of a prefill problem described by `desc` (the FULL
 * problem: q, k, v, o, lse are the bases of the [B, H, ...] tensors; only the
 * slice is read or written, so a rank may map only that part).  At most three
 * tf_attn_fwd launches, no communication.  The slice is returned in
 * begin_out / end_out (either may be NULL).
 */
TF_EXPORT int tf_prefill_sharded(int32_t rank, int32_t world, const void* q, const void* k,
                                 const void* v, void* o, float* lse, const TfAttnDesc* desc,
                                 void* stream, int64_t* begin_out, int64_t* end_out);

#define TF_NCCL_ID_BYTES 128
enum { TF_TRANSPORT_AUTO = 0, TF_TRANSPORT_P2P = 1, TF_TRANSPORT_NCCL = 2 };

/* One rank's state of a KV-sharded decoder (opaque). */
typedef struct TfShardCtx TfShardCtx;

/* Rank 0 makes the 128-byte NCCL id that every rank passes to tf_shard_create;
 * the caller carries it to the other ranks by whatever means it has.  NCCL
 * (libnccl.so.2) is loaded at run time, on first use. */
TF_EXPORT int tf_shard_unique_id(void* id_out);

/*
 * Collective over all `world` ranks, each with its GPU current.  Creates the
 * rank's context for decode problems of (batch, heads, head_dim, dtype): an
 * NCCL communicator (world > 1), two alternating gather areas of
 * world * batch*heads * (head_dim+2) fp32 plus one flag word per sender,
 * arrival counters, and -- for the peer-memory transport -- a table of every
 * rank's gather buffer mapped into this process through CUDA IPC.
 * transport: TF_TRANSPORT_P2P (fails if a peer cannot be mapped),
 * TF_TRANSPORT_NCCL, or TF_TRANSPORT_AUTO (p2p, else nccl on every rank alike;
 * tf_shard_note then says why).  world == 1 needs no id.
 */
TF_EXPORT int tf_shard_create(int32_t rank, int32_t world, const void* nccl_id,
                              int32_t transport, int32_t batch, int32_t heads,
                              int32_t head_dim, int32_t dtype, TfShardCtx** out);

/* TF_TRANSPORT_P2P or TF_TRANSPORT_NCCL: what the context uses. */
TF_EXPORT int tf_shard_transport(const TfShardCtx* ctx);
TF_EXPORT const char* tf_shard_note(const TfShardCtx* ctx);

/*
 * One decode step over a KV sequence sharded across the ranks: q [B,H,D]
 * replicated, k_local / v_local this rank's keys (desc->len_kv of them, may be
 * 0), o [B,H,D] and lse [B,H] (may be NULL) written on EVERY rank.  Stream-
 * ordered, no host synchronisation, and every rank must call it once per step.
 *   p2p : ONE kernel launch -- split-KV pass; the CTA finishing a row's last
 *         split merges the row and stores it into every rank's gather area;
 *         the rank's last row raises its flag on every peer; CTAs then wait
 *         (bounded) for all flags and write the final O / LSE.  Plain peer
 *         stores and system-scope release/acquire only: no TMA, no multicast
 *         and no library kernel touch peer memory.  (Grouped-query problems
 *         take three launches: split, merge + scatter, combine.)
 *   nccl: the same kernel writes this rank's slot, ncclAllGather in place,
 *         then the combine kernel.
 * The split-KV workspace is allocated by the first call and grown only when a
 * later call needs more; otherwise a step allocates nothing.  If a rank never
 * arrives, the bounded wait gives up: o / lse of that step read NaN, and the
 * NEXT call returns TF_ERR_DEVICE_TIMEOUT before launching anything
 * (tf_device_status clears the condition).  The wait limit (default 2 s,
 * tf_set_wait_limit_ms) is therefore also the largest skew between ranks that
 * the p2p transport tolerates.
 */
TF_EXPORT int tf_decode_sharded(TfShardCtx* ctx, const void* q, const void* k_local,
                                const void* v_local, void* o, float* lse,
                                const TfDecodeDesc* desc, void* stream);

/* Frees the context (synchronises its device).  Collective in the sense that
 * no peer may still be running a step that stores into this rank's buffer. */
TF_EXPORT int tf_shard_destroy(TfShardCtx* ctx);

/* ---- diagnostics -------------------------------------------------------- */

/* Text of the last error raised on the calling thread ("" if none). */
TF_EXPORT const char* tf_last_error(void);

/*
 * Reads and clears the device-side status word of the current device
 * (synchronises the device).  0 = every bounded wait completed; otherwise the
 * code of the first wait that gave up, and TF_ERR_DEVICE_TIMEOUT is returned.
 * A kernel whose wait gave up leaves its output unwritten (prefill, split
 * pass) or NaN (the combine behind the gather flags).
 */
TF_EXPORT int tf_device_status(int32_t* code_out);

/*
 * The same word without synchronising: the device mirrors it into mapped host
 * memory the moment a wait gives up, so this only reads a host variable.  It
 * reports launches that have already failed; it neither waits for running
 * ones nor clears anything.
 */
TF_EXPORT int tf_device_status_peek(int32_t* code_out);

/*
 * Upper bound of every device-side wait (mbarrier waits of the kernels, the
 * flag wait of the sharded decode), in milliseconds; default 2000.  Takes
 * effect on each device with the next launch made through this library.
 */
TF_EXPORT int tf_set_wait_limit_ms(uint32_t milliseconds);

/* ---- 8-bit storage -------------------------------------------------------- */

/*
 * Bulk conversion of `n` contiguous elements between a 16-bit tensor (TF_F16 /
 * TF_BF16) and 8-bit storage (TF_FP8_E4M3 / TF_FP8_E5M2); both pointers 16-byte
 * aligned, any n >= 0.  The bulk form of TileFusion's per-value from_float /
 * to_float (include/types/base.hpp:70-107, the CUDA __nv_fp8 constructors):
 *   quantize  : dst[i] = fp8(float(src[i]) * factor), round to nearest even,
 *               values beyond the largest finite one saturate to it;
 *   dequantize: dst[i] = 16-bit(float(src[i]) * factor), round to nearest even.
 * A K/V cache written with factor f is read by tf_decode* with k_scale /
 * v_scale = 1 / f.  One HBM-bound kernel each (3 bytes per element).
 */
TF_EXPORT int tf_fp8_quantize(const void* src, void* dst, int64_t n,
                              int32_t src_dtype, int32_t fp8_dtype, float factor,
                              void* stream);
TF_EXPORT int tf_fp8_dequantize(const void* src, void* dst, int64_t n,
                                int32_t fp8_dtype, int32_t dst_dtype, float factor,
                                void* stream);

/* ---- measurement --------------------------------------------------------- */

/*
 * Tensor-pipe time of `n_mma` back-to-back tcgen05.mma (M128, K16, fp16 in,
 * fp32 accumulate, N = `n` in {64, 128, 256}) issued by one thread on one SM of
 * the current device: SM clocks until the last one is issued and until all are
 * complete.  a_from_tmem selects the A operand (0 shared memory, 1 tensor
 * memory), b_mn_major the layout of B (0: rows along the contraction, 1: rows
 * along N), desc32 how the issuing thread forms the shared-memory descriptors
 * (0: a 64-bit descriptor built per MMA, 1: 32-bit low halves advanced by
 * constants, as the kernels do), uniform_issue whether that thread is alone in
 * a branch on its lane number (0) or the elected lane of a warp that walks the
 * loop as a whole (1, as the kernels do).  Computes nothing useful; it exists so that the
 * per-MMA figures the design notes quote can be re-measured
 * (bench.py --workload mma_rate).
 * Synchronous; allocates 16 bytes for the duration of the call.
 */
TF_EXPORT int tf_probe_mma_clocks(int32_t a_from_tmem, int32_t n, int32_t b_mn_major,
                                  int32_t desc32, int32_t uniform_issue, int32_t n_mma,
                                  int64_t* issue_clocks, int64_t* complete_clocks);

/*
 * The same measurement for the two-CTA form (tcgen05.mma.cta_group::2, M = 256
 * over a cluster of two CTAs on two SMs, each holding its own 128 rows of A and
 * n / 2 columns of B): per SM the arithmetic of one such MMA equals that of an
 * M128 single-CTA MMA of the same n, so the clocks compare directly with
 * tf_probe_mma_clocks(..., desc32 = 1, uniform_issue = 1, ...).  No counterpart
 * in the reference.  Synchronous; allocates 16 bytes for the duration of the call.
 */
TF_EXPORT int tf_probe_mma_pair_clocks(int32_t a_from_tmem, int32_t n, int32_t b_mn_major,
                                       int32_t n_mma, int64_t* issue_clocks,
                                       int64_t* complete_clocks);

/* Library ABI version (bumped when a struct above changes). */
TF_EXPORT int tf_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TILEFUSION_B200_H_ */
