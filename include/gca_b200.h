/*
 * gca_b200.h -- C ABI of libgca_b200.so: Grouped Cross-Attention (GCA) and landmark
 * retrieval for the DRT long-context model, written for NVIDIA B200 (sm_100a).
 *
 * The reference project is pure Python; its boundary for this path is a set of Python
 * callables.  Each entry point below names the reference callable it stands in for
 * (paths relative to the reference project).  The Python host layer of this repository
 * binds these symbols with ctypes and re-exposes them under the reference's names.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller (also workspaces and the
 *     optional status word); the library keeps nothing after the call returns except work
 *     already enqueued on `stream`;
 *   - all launches are asynchronous on `stream` (a cudaStream_t passed as void*), which must
 *     belong to the device that holds the buffers; the entry points take the device from the
 *     pointers (not from the calling thread's current device) and restore the caller's
 *     current device before they return;
 *   - strides are in ELEMENTS; the innermost (head_dim) axis must be contiguous;
 *   - return value: 0 = ok, negative = argument rejected on the host before any launch
 *     (GCA_ERR_*), positive = CUDA runtime error code;
 *   - nothing throws or aborts; there is no CPU fallback.
 */
#ifndef GCA_B200_H_
#define GCA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GCA_ABI_VERSION 2

enum GcaDtype { GCA_BF16 = 0, GCA_F32 = 1 };

enum GcaError {
  GCA_OK = 0,
  GCA_ERR_NULL = -1,        /* a required pointer is NULL */
  GCA_ERR_DTYPE = -2,       /* unknown dtype / dtype not supported by this kernel */
  GCA_ERR_SHAPE = -3,       /* a dimension is outside the supported envelope */
  GCA_ERR_STRIDE = -4,      /* a stride is not usable (alignment, overlap) */
  GCA_ERR_ALIGN = -5,       /* a base pointer is not 16-byte aligned */
  GCA_ERR_WORKSPACE = -6,   /* workspace missing or too small */
  GCA_ERR_ALGO = -7,        /* requested kernel variant cannot run this problem */
  GCA_ERR_TMA = -8,         /* the driver rejected a tensor-map encoding */
  GCA_ERR_TOO_LARGE = -9,   /* a size exceeds a fixed built-in limit */
  GCA_ERR_STATIC_SCRATCH = -10 /* lmk_score_topk_static: the problem needs more than the built-in scratch */
};

/* kernel variants (GcaFwdArgs.algo / GcaBwdArgs.algo) */
enum GcaAlgo {
  GCA_ALGO_AUTO = 0,        /* bf16 + S=L=D=64 -> tensor-core kernel, everything else -> SIMT */
  GCA_ALGO_SIMT = 1,        /* fp32-accumulating CUDA-core kernel (bf16 or fp32 data) */
  GCA_ALGO_TC = 2,          /* tcgen05/TMEM/TMA kernel (bf16 only) */
  GCA_ALGO_TC_UNPAIRED = 3  /* forward only: the tensor-core kernel with ONE q head per work unit instead of a
                               pair (same per-row arithmetic, same bits; a cross-check of the pairing logic);
                               the backward treats it as GCA_ALGO_TC */
};

/* device-side soft status bits written (OR-ed) into *status when it is given */
enum GcaStatus {
  GCA_STATUS_OK = 0,
  GCA_STATUS_BAD_INDEX = 1, /* a retrieved chunk index was >= C; the slot was skipped */
  GCA_STATUS_TIMEOUT = 2    /* a bounded on-chip wait expired; outputs are not valid */
};

/*
 * Forward.  Stands in for `_attention.forward` (ltriton/gca.py:683-738, kernel
 * `_attn_fwd` :94-211) and, without `lse`, for `gca_kv_cache` (ltriton/gca.py:846-888,
 * kernel `_attn_inf` :214-314) -- with the chunk gather of
 * `ChunkKVManager.retrieve_chunks` (model/DRT.py:193-199) and the layout copy of
 * `TritonGroupCrossAttention.preprocess_chunk_kv_cache` (model/DRT.py:321-332) folded in:
 * K/V are read from the cache by retrieved chunk index.
 *
 *   q, out   (N, J, Hq, S, D)      addressed with *_stride = {n, j, h, s}
 *   k_cache, v_cache (N, C, L, Hkv, D) addressed with *_stride = {n, c, l, h}
 *   indices  (N, J, K) int32, contiguous; < 0 marks a padding slot (skipped)
 *   weights  (N, J, K) float32, contiguous (shared by all heads)
 *   lse      (N*J, Hq, K, S) float32 base-2 log-sum-exp per slot, or NULL
 *
 *   out[n,j,h] = sum_k weights[n,j,k] * softmax(sm_scale * q K_k^T) V_k,
 *   K_k = k_cache[n, indices[n,j,k], :, h / (Hq/Hkv), :].
 *
 * The pre-gathered call of the reference (k of shape (Z, Hkv, K, L, D)) is the same
 * kernel with N=Z, J=1, C=K, indices = 0..K-1 and the matching strides.
 * `off_by_one` > 0 adds a virtual zero logit of that weight to every softmax; 0 gives
 * the behaviour of the reference kernels (whose `sm_n` argument has no effect).
 */
typedef struct GcaFwdArgs {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int32_t* indices;
  const float* weights;
  void* out;
  float* lse;
  int32_t* status;
  int64_t q_stride[4];
  int64_t o_stride[4];
  int64_t k_stride[4];
  int64_t v_stride[4];
  int32_t N, J, Hq, Hkv, S, L, D, K, C;
  int32_t dtype;
  int32_t algo;
  float sm_scale;
  float off_by_one;
} GcaFwdArgs;

int gca_fwd(const GcaFwdArgs* args, void* stream);

/*
 * Decode / short-query forward: S in [1, 16] query rows (the model uses 1 or 2).
 * Stands in for `gca_kv_cache` with q of shape (N, Hq, 1|2, D) (model/DRT.py:382,
 * ltriton/gca.py:846-888).  Same argument block as gca_fwd; `lse` is ignored.
 */
int gca_decode(const GcaFwdArgs* args, void* stream);

/*
 * Backward.  Stands in for `_attention.backward` (ltriton/gca.py:740-841: the scaled copy
 * of K :776, kernels `kernel_attn_bwd_dkdv` :484-572 and `kernel_attn_bwd_dq` :575-675,
 * the `delta` reduction :839-840) plus the scatter-add into the chunk cache that autograd
 * performs behind the reference's gather (index_put_ with accumulate).
 *
 *   dout, dq        like q (strides do_stride / dq_stride)
 *   dk_cache, dv_cache like the caches (strides dk_stride / dv_stride); every (n, c, h)
 *                   tile is written: the sum over all (j, k) that retrieved chunk c, or 0
 *   dw              (N, J, K) float32: sum over heads and rows of <dout, O_k>
 *   lse             as written by gca_fwd with the same arguments
 *   workspace       gca_bwd_workspace_bytes() bytes, 256-byte aligned
 */
typedef struct GcaBwdArgs {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int32_t* indices;
  const float* weights;
  const void* dout;
  const float* lse;
  void* dq;
  void* dk_cache;
  void* dv_cache;
  float* dw;
  void* workspace;
  int32_t* status;
  size_t workspace_bytes;
  int64_t q_stride[4];
  int64_t do_stride[4];
  int64_t dq_stride[4];
  int64_t k_stride[4];
  int64_t v_stride[4];
  int64_t dk_stride[4];
  int64_t dv_stride[4];
  int32_t N, J, Hq, Hkv, S, L, D, K, C;
  int32_t dtype;
  int32_t algo;
  float sm_scale;
  float off_by_one;
} GcaBwdArgs;

int gca_bwd(const GcaBwdArgs* args, void* stream);
size_t gca_bwd_workspace_bytes(const GcaBwdArgs* args);

/*
 * The same backward, one stage at a time (gca_bwd == all three on one stream).  The reference
 * runs its two backward kernels back to back inside `_attention.backward`
 * (ltriton/gca.py:786-838); the stages exist here so that a caller can build the index early
 * (it depends on the indices only) and time the kernels separately.
 *   GCA_BWD_STAGE_INDEX  build the inverse retrieval index (chunk -> retrieving slots) in
 *                        `workspace`; must have completed before the other two stages run
 *   GCA_BWD_STAGE_Q      dq, dw, and the per-row terms (kept in `workspace`) that
 *                        GCA_BWD_STAGE_KV reads: it must run before GCA_BWD_STAGE_KV (same
 *                        stream, or ordered by the caller), as the reference's kernels hand
 *                        `delta` from one to the other (ltriton/gca.py:385,459)
 *   GCA_BWD_STAGE_KV     dk_cache, dv_cache
 * All calls of one backward pass the same argument block (same workspace).
 * GCA_BWD_INDEX_BY_SORT, a flag beside GCA_BWD_STAGE_INDEX, builds the index with the radix-sort
 * path that large problems take anyway; it has the same bits as the single-launch path.
 */
enum { GCA_BWD_STAGE_INDEX = 1, GCA_BWD_STAGE_KV = 2, GCA_BWD_STAGE_Q = 4, GCA_BWD_STAGE_ALL = 7,
       GCA_BWD_INDEX_BY_SORT = 8 };
int gca_bwd_stages(const GcaBwdArgs* args, unsigned stages, void* stream);

/*
 * Landmark scoring + causal chunk mask + top-k + retrieval weights, fused.  Stands in for
 * the tensor program of `DRT._perform_batch_retrieval` (model/DRT.py:612-627: einsum,
 * masked_fill with `_enc_dec_score_mask` :590-607, optional Gumbel noise, topk, softmax,
 * nan_to_num) and of the decode-time block (model/DRT.py:836-845).
 *
 *   lmk_q    (N, Cq, D)  bf16  query landmarks,  row stride q_row_stride, batch q_batch_stride
 *   lmk_k    (N, E, D)   bf16  cached landmarks, row stride k_row_stride, batch k_batch_stride
 *   noise    (N, Cq, E)  float32 or NULL; added for the selection only
 *   row i of a sequence sees cached chunk e iff  e_base + e < q_pos0 + i
 *   (the reference: q_pos0 = E_total - Cq, e_base = 0).
 *   head_dim == 0: one score per (row, chunk) over all D, scaled 1/sqrt(D)   (the reference)
 *   head_dim  > 0: one score per (row, head, chunk) over head_dim, scaled 1/sqrt(head_dim);
 *                  outputs gain a head axis after Cq.
 *   score_round 0: float32 scores; 1: scores rounded to bf16 twice like the reference
 *                  under autocast (bf16 einsum output, bf16 division).
 *
 * Outputs, R = N*Cq (*H in per-head mode) rows, contiguous:
 *   out_keys    (R, K) uint64   packed (orderable score << 32 | ~index), 0 = empty; descending
 *   out_indices (R, K) int32    global chunk ids (e_base + e), -1 = padding      (may be NULL)
 *   out_scores  (R, K) float32  noise-free scores of the selected chunks         (may be NULL)
 *   out_weights (R, K) float32  softmax over the valid slots, padding 0          (may be NULL)
 *   out_nvalid  (R)    int32                                                   (may be NULL)
 * Scores are float32 sums in one fixed order, ties go to the lower index, so the result
 * is bit-reproducible and independent of the launch geometry.
 *   workspace: lmk_topk_workspace_bytes() bytes (partial candidate lists).
 */
typedef struct LmkTopkArgs {
  const void* lmk_q;
  const void* lmk_k;
  const float* noise;
  uint64_t* out_keys;
  int32_t* out_indices;
  float* out_scores;
  float* out_weights;
  int32_t* out_nvalid;
  void* workspace;
  size_t workspace_bytes;
  int64_t q_batch_stride, q_row_stride;
  int64_t k_batch_stride, k_row_stride;
  int64_t q_pos0;
  int64_t e_base;
  int32_t N, Cq, E, D, K;
  int32_t head_dim;
  int32_t score_round;
  int32_t splits;            /* 0 = choose; otherwise number of E-ranges scanned by separate CTAs */
} LmkTopkArgs;

int lmk_score_topk(const LmkTopkArgs* args, void* stream);
size_t lmk_topk_workspace_bytes(const LmkTopkArgs* args);

/*
 * lmk_score_topk for callers that cannot provide device scratch.  (No counterpart in the
 * reference: it exists for hosts that must not allocate device memory around the call -- a
 * server that handed all HBM to its own pools, a plugin inside someone else's allocator, a
 * loop that cannot afford an allocator call.)
 *
 * Same arguments, same results, bit for bit; args->workspace / workspace_bytes are ignored.
 * The per-block candidate lists go into an array compiled into the library
 * (LMK_STATIC_SCRATCH_BYTES of device memory on every GPU that loads it, held until exit).
 * Limit: lmk_topk_workspace_bytes(args) must not exceed LMK_STATIC_SCRATCH_BYTES, i.e.
 * rows * splits * K * 8 bytes <= 1 MiB (rows = N*Cq, times D/64 in per-head mode); a larger
 * problem is refused with GCA_ERR_STATIC_SCRATCH and nothing is launched.  Passing
 * args->splits lets the caller shrink the need.
 * The call allocates nothing, on the host or on the device.  Its first use on a device looks
 * up the array's address; make that first call outside of any stream capture.  All calls
 * on one GPU share the array (contents left over from the previous call are never read), so
 * calls that could overlap on the same GPU must be serialised by the caller.
 */
#define LMK_STATIC_SCRATCH_BYTES (1 << 20)
int lmk_score_topk_static(const LmkTopkArgs* args, void* stream);

/*
 * Merge of candidate lists (the exchange step of the chunk-range-sharded cache; no
 * counterpart in the reference, which never shards retrieval): keys (R, P) packed uint64
 * candidates (P = shards * K, any order, 0 = empty) -> the K best per row, descending,
 * with indices / scores / weights / nvalid decoded as above.
 */
typedef struct LmkMergeArgs {
  const uint64_t* keys;
  uint64_t* out_keys;
  int32_t* out_indices;
  float* out_scores;
  float* out_weights;
  int32_t* out_nvalid;
  int32_t R, P, K;
} LmkMergeArgs;

int lmk_topk_merge(const LmkMergeArgs* args, void* stream);

/*
 * Candidate exchange between the GPUs of ONE node for the chunk-range-sharded cache, fused with
 * the merge (no counterpart in the reference, which parks the cache on the host instead,
 * model/DRT.py:87-128): one launch per rank and step.  Each rank stores its K packed candidates
 * per row into its slot of every rank's mailbox through peer mappings (stores only; nothing
 * reads remote memory), raises a flag, waits -- bounded by `wait_ms` -- for all ranks' flags in
 * its own mailbox, and merges the world x K candidates exactly like lmk_topk_merge, so every
 * rank ends with the identical global top-k.  If the wait expires, GCA_STATUS_TIMEOUT is OR-ed
 * into *status, the outputs of that row are not written, and the kernel returns; the host then
 * brings the ranks back in step (a barrier of its own, then lmk_exchange_mailbox_reset on every
 * rank).  The step counter lives in the mailbox, so the launch can be part of a CUDA graph.
 *
 * Set-up, once per rank: lmk_exchange_mailbox_create (allocates and clears the mailbox with
 * cudaMalloc on the current device and fills a 64-byte IPC handle), exchange the handles among the
 * ranks by any host means, lmk_exchange_mailbox_open for every other rank's handle, and put the
 * `world` pointers (own mailbox at index `rank`) into a device array: that array is `mailboxes`.
 */
typedef struct LmkExchangeArgs {
  const uint64_t* local_keys;   /* (R, K) this rank's candidates: out_keys of lmk_score_topk */
  void* const* mailboxes;       /* DEVICE array of `world` mailbox pointers as mapped in this process */
  uint64_t* out_keys;           /* (R, K) outputs as in lmk_topk_merge */
  int32_t* out_indices;
  float* out_scores;
  float* out_weights;
  int32_t* out_nvalid;
  int32_t* status;              /* device status word, or NULL */
  int32_t R, K, world, rank;
  int32_t R_max;                /* rows the mailboxes were created for (the same on every rank) */
  int32_t wait_ms;              /* bound of the wait for the other ranks' flags; 0 = 1000 */
} LmkExchangeArgs;

size_t lmk_exchange_mailbox_bytes(int r_max, int world);
int lmk_exchange_mailbox_create(int r_max, int world, void** mailbox, void* ipc_handle64);
int lmk_exchange_mailbox_open(const void* ipc_handle64, void** peer_ptr);
int lmk_exchange_mailbox_close(void* peer_ptr);
int lmk_exchange_mailbox_destroy(void* mailbox);
int lmk_exchange_mailbox_reset(void* mailbox, int r_max, int world, void* stream);
int lmk_topk_exchange(const LmkExchangeArgs* args, void* stream);

/*
 * Chunk cache append with the landmark row cleared.  Stands in for the tensor work of
 * model/DRT.py:770-784 + ChunkKVManager.append (:87-133): copies `count` new chunks of K
 * and V (N, count, L, Hkv*D) into a preallocated cache (N, capacity, L, Hkv*D) at chunk
 * position `pos`, writing zeros into the last row of every chunk when zero_landmark != 0,
 * and copies the landmark embeddings (N, count, Dm) into the landmark cache.
 * `capacity` / `lmk_capacity` are the chunk capacities of the destination buffers: a call with
 * pos + count beyond either is rejected with GCA_ERR_SHAPE before anything is launched.
 */
typedef struct CacheAppendArgs {
  const void* new_k;
  const void* new_v;
  const void* new_lmk;       /* may be NULL */
  void* k_cache;
  void* v_cache;
  void* lmk_cache;           /* may be NULL */
  int64_t new_batch_stride;  /* elements between sequences in new_k / new_v */
  int64_t cache_batch_stride;
  int64_t new_lmk_batch_stride, lmk_cache_batch_stride;
  int32_t N, count, pos, L, HD, Dm;
  int32_t dtype;
  int32_t zero_landmark;
  int32_t capacity;          /* chunks the k / v cache buffers hold per sequence */
  int32_t lmk_capacity;      /* rows the landmark cache holds per sequence (ignored when lmk_cache is NULL) */
} CacheAppendArgs;

int gca_cache_append(const CacheAppendArgs* args, void* stream);

/*
 * Chunk K/V projection with the cache append as its epilogue.  Stands in for
 * model/DRT.py:766-784 -- `lmk_embs = enc[:, :, -1]`, `chunk_k = chunk_k_proj(enc)`,
 * `chunk_v = chunk_v_proj(enc)`, the landmark row of both cleared, then
 * `ChunkKVManager.append` (:87-133) -- as ONE tensor-core GEMM whose epilogue writes K and V in
 * bf16 straight into the cache at chunk position `pos` (no intermediate tensors, no copy of the
 * existing cache), plus a copy of the landmark rows of `x` into the landmark cache.
 *
 *   x        (N, count, 64, D) bf16, contiguous: the chunk encoder's output
 *   wk, wv   (D, D) bf16, contiguous, nn.Linear layout (out_features, in_features), no bias
 *   k_cache, v_cache (N, capacity, 64, D) bf16, sequence stride cache_batch_stride elements
 *   lmk_cache (N, lmk_capacity, D) bf16 or NULL
 *   D must be a multiple of 256 (the model: 768).
 */
typedef struct KvProjectArgs {
  const void* x;
  const void* wk;
  const void* wv;
  void* k_cache;
  void* v_cache;
  void* lmk_cache;            /* may be NULL */
  int32_t* status;            /* device status word, or NULL */
  int64_t cache_batch_stride;
  int64_t lmk_cache_batch_stride;
  int32_t N, count, pos, D;
  int32_t capacity, lmk_capacity;
  int32_t zero_landmark;
} KvProjectArgs;

int gca_kv_project_append(const KvProjectArgs* args, void* stream);

/* ---- projections either side of GCA (reference: model/DRT.py:352-355 pre_norm + q_proj, :385 o_proj
 * and the residual add of the decoder layer, :476-484; the reference's RMSNorm is LlamaRMSNorm) ----
 *
 *   gca_row_rms:  row_scale[m] = rsqrt(mean(x[m, :]^2) + eps)                      (float32, M values)
 *   gca_linear:   out[m, :] = row_scale[m] * (x[m, :] . w^T) + residual[m, :]      (bf16 in / out, f32 accumulate)
 *
 * x (M, K) bf16, w (N, K) bf16 in nn.Linear layout, out / residual (M, N) bf16; strides in elements
 * between rows; row_scale and residual may be NULL.  K a multiple of 64, N a multiple of 16, row
 * strides multiples of 8 elements, every pointer 16-byte aligned.  With row_scale from gca_row_rms
 * and the norm's gain folded into w's columns (w' = w * gain[None, :]) this is RMSNorm + projection
 * without writing the normalised activations; with residual it is projection + residual add.
 * One tcgen05 GEMM launch (128 x 256 tiles, TMA ring, accumulators in tensor memory). */
typedef struct RowRmsArgs {
  const void* x;
  float* row_scale;
  int64_t M;
  int64_t x_stride;
  int32_t D;
  float eps;
} RowRmsArgs;

typedef struct LinearArgs {
  const void* x;
  const void* w;
  void* out;
  const void* residual;       /* may be NULL */
  const float* row_scale;     /* may be NULL */
  int32_t* status;            /* device status word, or NULL */
  int64_t M;
  int64_t x_stride, w_stride, out_stride, residual_stride;
  int32_t N, K;
} LinearArgs;

int gca_row_rms(const RowRmsArgs* args, void* stream);
int gca_linear(const LinearArgs* args, void* stream);

/* out[m, c] = silu(gate_up[m, c]) * gate_up[m, I + c] for c < I: the activation between ONE gate|up
 * projection (weights stacked) and down_proj -- the reference's fused SwiGLU, model/llama.py:290-300.
 * bf16; gate_up (M, 2 I) and out (M, I) by row strides in elements (multiples of 8); I % 8 == 0. */
int gca_silu_mul(const void* gate_up, void* out, int64_t M, int32_t I, int64_t in_stride, int64_t out_stride, void* stream);

/* ---- LM head fused with the cross-entropy loss, forward only (reference: model/DRT.py:1055-1064,
 * `logits = lm_head(hidden)` followed by CrossEntropyLoss(ignore_index=-100); evaluation / perplexity) ----
 *
 *   loss[m] = logsumexp_j(row_scale[m] * x[m, :] . w[j, :]) - (row_scale[m] * x[m, :] . w[targets[m], :])
 *
 * x (M, K) bf16, w (N, K) bf16 (N = vocabulary, any size), targets (M) int64 (negative: the row is
 * ignored, loss 0; a target >= N gives NaN), loss (M) float32, lse (M) float32 or NULL (natural log).
 * The (M, N) logits stay in tensor memory.  workspace: gca_linear_ce_workspace_bytes(M, N) bytes,
 * 16-byte aligned, caller-owned. */
typedef struct LinearCeArgs {
  const void* x;
  const void* w;
  const void* targets;
  const float* row_scale;     /* may be NULL */
  float* loss;
  float* lse;                 /* may be NULL */
  void* workspace;
  int32_t* status;            /* device status word, or NULL */
  int64_t M;
  int64_t x_stride, w_stride;
  int64_t workspace_bytes;
  int32_t N, K;
} LinearCeArgs;

size_t gca_linear_ce_workspace_bytes(int64_t M, int32_t N);
int gca_linear_cross_entropy(const LinearCeArgs* args, void* stream);

/* ---- sliding-window causal self-attention with ALiBi, decode form (reference call site:
 * model/llama.py:684-688, flash_attn_with_kvcache(..., causal=True, window_size=(W, 0), alibi_slopes=m)) ----
 *
 *   q, out (N, Hq, Sq, 64) bf16 by strides (n, head, row), k, v (N, Hkv, T, 64) bf16 by strides
 *   (n, kv head, position); the 64 head dimensions contiguous, rows 16-byte aligned.
 *   Query row i stands at position T - Sq + i and sees keys j with  pos - window <= j <= pos;
 *   score = sm_scale * q.k - slope[head] * (pos - j);  alibi_slopes (Hq) float32 or NULL.
 *   (Hq / Hkv) * Sq <= 4 rows per kv head.  HBM-bound: 2 * (window + 1) * 128 bytes per (n, kv head). */
typedef struct WindowDecodeArgs {
  const void* q;
  const void* k;
  const void* v;
  const float* alibi_slopes;  /* may be NULL */
  void* out;
  int64_t q_stride[3], o_stride[3], k_stride[3], v_stride[3];
  int32_t N, Hq, Hkv, Sq, T, window;
  float sm_scale;
} WindowDecodeArgs;

int gca_window_decode(const WindowDecodeArgs* args, void* stream);

/* The same attention for ONE new position per sequence (Sq = 1) over a window kept as a RING, with the
 * append folded in: attn.k / attn.v are the (N, Hkv, T, 64) ring buffers with T <= window + 1 valid rows,
 * k_new / v_new the new position's (N, Hkv, 64) rows by strides (n, kv head).  *rows_written (a device
 * int64 the caller advances by one per call sequence, e.g. inside a captured CUDA graph) gives the slot
 * p = rows_written mod T (the count must stay below 2^32: subtract a multiple of T before it gets there) that holds the oldest row: the new rows are attended to as the newest
 * position and stored at p; physical row j counts as logical position (j - p - 1) mod T.  With
 * rows_written = 0 and a linear window the result equals gca_window_shift_append followed by
 * gca_window_decode, without moving the window (which costs a read + write of the whole window per call). */
typedef struct WindowRingDecodeArgs {
  WindowDecodeArgs attn;
  const void* k_new;
  const void* v_new;
  const int64_t* rows_written;  /* device memory */
  int64_t new_stride[2];
} WindowRingDecodeArgs;

int gca_window_ring_decode(const WindowRingDecodeArgs* args, void* stream);

/* The cached window moved on by one position, in place: every (n, head) block of T rows (64 bf16 each,
 * contiguous: position stride 64) drops its oldest row and takes the new position's row at the end
 * (what the reference's KV cache does with torch.cat and a slice).  k_window / v_window (N, H, T, 64)
 * with strides (n, head) in elements; k_new / v_new (N, H, 64) rows with strides (n, head); T <= 640. */
typedef struct WindowAppendArgs {
  void* k_window;
  void* v_window;
  const void* k_new;
  const void* v_new;
  int64_t window_stride[2], new_stride[2];
  int32_t N, H, T;
} WindowAppendArgs;

int gca_window_shift_append(const WindowAppendArgs* args, void* stream);

/* ---- growable device buffers without copies (what the chunk cache of a growing context sits on;
 * the reference grows its cache with torch.cat on every append, model/DRT.py:87-133) ----
 *
 * A range of virtual addresses is reserved once for the largest size the buffer may reach;
 * physical memory is mapped behind it in multiples of gca_vmem_granularity() as the buffer grows.
 * Addresses never change, nothing is ever re-copied.  These are the library's only entry points,
 * besides lmk_exchange_mailbox_create, that obtain device memory, and they do so only when called.
 *   gca_vmem_reserve(bytes, alignment, &va)            reserve addresses (no memory yet)
 *   gca_vmem_map(va + off, bytes, device, &handle)     back a sub-range with new physical memory
 *   gca_vmem_unmap(va + off, bytes, handle)            undo one map (caller has synchronised)
 *   gca_vmem_free(va, bytes)                           give the addresses back (everything unmapped) */
size_t gca_vmem_granularity(int device);
int gca_vmem_reserve(size_t bytes, size_t alignment, void** va_out);
int gca_vmem_map(void* va, size_t bytes, int device, unsigned long long* handle_out);
int gca_vmem_unmap(void* va, size_t bytes, unsigned long long handle);
int gca_vmem_free(void* va, size_t bytes);

const char* gca_strerror(int code);
int gca_abi_version(void);
/* sizeof() of an argument block as the library was compiled (0 GcaFwdArgs, 1 GcaBwdArgs,
 * 2 LmkTopkArgs, 3 LmkMergeArgs, 4 CacheAppendArgs, 5 LmkExchangeArgs, 6 KvProjectArgs, 7 RowRmsArgs, 8 LinearArgs, 9 WindowDecodeArgs, 10 LinearCeArgs, 11 WindowAppendArgs, 12 WindowRingDecodeArgs): lets a foreign-language binding verify
 * its struct layout before the first call. */
size_t gca_sizeof(int which);

#ifdef __cplusplus
}
#endif
#endif /* GCA_B200_H_ */
