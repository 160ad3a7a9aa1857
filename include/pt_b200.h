/*
 * pt_b200.h — C-ABI of libpt_b200.so: sm_100a CUDA kernels for the PopTransformer
 * per-token decode step.
 *
 * This is the boundary a PopTransformer maintainer binds in place of
 * `ctypes.cdll.LoadLibrary('../../custom_ops.so')`
 * (poptransformer/ops/customized.py:17-18): one plain C function per custom op /
 * fused decode stage, keyed by the same op names and attribute meanings.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the parameter name ends in `_host`;
 *   - `stream` is a cudaStream_t passed as void*; calls only enqueue work;
 *   - fp16 tensors are IEEE binary16 (`uint16_t` storage), row-major, innermost
 *     dimension last;
 *   - every function returns 0 on success or a negative PT_ERR_* code and records a
 *     message retrievable with pt_last_error() (thread-local);
 *   - shape/dtype violations the reference reports at graph-build time
 *     (popart::error in each Op::setup) are reported here before any launch;
 *   - the library allocates no device memory: caches, workspaces and outputs belong to
 *     the caller.  `step` arguments named `step_dev` are read ON THE DEVICE so that a
 *     captured CUDA graph can be replayed for every token.
 */
#ifndef PT_B200_H
#define PT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PT_OK 0
#define PT_ERR_INVALID (-1)   /* bad shape / argument (reference: popart::error at setup) */
#define PT_ERR_CUDA (-2)      /* a CUDA runtime call failed                               */
#define PT_ERR_UNSUPPORTED (-3)

/* ---- library ---------------------------------------------------------------------- */
const char *pt_last_error(void);
int pt_version(void);
/* Number of kernel launches this library has enqueued from the calling process. */
uint64_t pt_launch_count(void);

/* Weight formats understood by the streaming skinny-matmul kernels. */
#define PT_W_INT4 0 /* signed nibbles, 2 per byte, high nibble = even k, fp16 group scales */
#define PT_W_FP16 1
#define PT_W_FP8 2  /* OCP E4M3, per-tensor fp32 scale                                    */

/* Prologues fused in front of a linear layer (applied to the activation rows). */
#define PT_PRO_NONE 0
#define PT_PRO_RMSNORM 1   /* poptransformer/layers/rms_layer_norm.py:26-36 */
#define PT_PRO_CAST_FP8 2  /* activations quantised to E4M3 with `act_scale` first */
#define PT_PRO_RMSNORM_CAST_FP8 3
#define PT_PRO_NORMCE 4    /* LayerNorm with the NormCE arithmetic (customized.py:69-102; custom_ops/NormCE.cpp), norm_gamma / norm_beta */

/* Epilogues fused behind a linear layer. */
#define PT_EPI_STORE 0        /* y = fp16(acc)                                         */
#define PT_EPI_RESIDUAL 1     /* y = fp16(res + fp16(acc))           (ops.add)        */
#define PT_EPI_SWIGLU 2       /* y = fp16(fp16(up) * swish(fp16(gate))) llama2/mlp.py:20-28 */
#define PT_EPI_BIAS 3         /* y = fp16(fp16(acc) + bias)          layers/linear.py:42-46 */
#define PT_EPI_BIAS_GELU 4    /* y = gelu(fp16(fp16(acc) + bias))    layers/mlp.py:34-41   */
#define PT_EPI_BIAS_RESIDUAL 5/* y = fp16(res + fp16(fp16(acc) + bias))                  */

/* ---- Int4ToHalf -------------------------------------------------------------------
 * Replaces the `Int4ToHalf` custom op (poptransformer/ops/customized.py:115-124;
 * custom_ops/int4_to_half_custom_op.cpp:168-380; codelets int4_to_half_codelets.cpp:18-73).
 * axis 1: w int8 [n, m], scale fp16 [n] (group == 0) or [n, 2m/group] -> out fp16 [2m, n].
 * axis 0: w int8 [n, m], scale fp16 [m] -> out fp16 [2n, m].  Bit-exact. */
int pt_int4_to_half(const void *w, const void *scale, int n, int m, int axis, int group,
                    void *out, void *stream);

/* ---- linear layers ----------------------------------------------------------------
 * Replaces Linear.__call__ -> ParamHandler.matmul -> (Int4ToHalf|CastToUint8) + matmul
 * (poptransformer/layers/linear.py:42-46, utils/param_handler/param_handler.py:57-83,
 * utils/param_handler/precision_strategy.py:56-81) for decode-sized batches.
 *
 * pt_linear_repack: one-time re-layout of a weight matrix W[n_out, k_in] stored with
 * k contiguous (INT4: the reference's int8 [n_out, k_in/2] + fp16 scales [n_out, k_in/group])
 * into the tile order the streaming kernel fetches with bulk async copies (INT4 tiles carry
 * their group scales).  Size of the output: pt_linear_packed_bytes.
 * `interleave_rows` = 1 builds the SwiGLU layout from a [2*f, k] matrix whose first f rows
 * are gate rows and last f rows are up rows (8 gate rows then 8 up rows per 16-row tile). */
size_t pt_linear_packed_bytes(int wfmt, int n_out, int k_in);
int pt_linear_repack(int wfmt, const void *w, const void *scale, int n_out, int k_in, int group,
                     int interleave_rows, void *packed_w, void *stream);

typedef struct pt_linear_args {
  int wfmt;              /* PT_W_*                                                  */
  int batch;             /* rows of x, 1..32                                        */
  int n_out, k_in;       /* logical weight shape (n_out counts gate+up rows for SWIGLU) */
  int group;             /* INT4 scale group along k (k_in for one scale per row)    */
  int prologue, epilogue;
  int ksplit;            /* 0 = let the library choose; >1 needs workspace          */
  const void *x;         /* fp16 [batch, k_in]                                      */
  const void *packed_w;  /* from pt_linear_repack                                   */
  const void *norm_gamma;/* fp16 [k_in]   (PT_PRO_RMSNORM*)                        */
  float norm_eps;
  float act_scale;       /* FP8: activation scale (x ~ act_scale * e4m3)            */
  float w_scale;         /* FP8: weight per-tensor scale                            */
  const void *bias;      /* fp16 [n_out]                                            */
  const void *residual;  /* fp16 [batch, n_out]; may alias `out`                    */
  void *out;             /* fp16 [batch, n_out] (SWIGLU: [batch, n_out/2])          */
  int out_ld;            /* row stride of `out` in elements; 0 = dense              */
  int pdl;               /* 1: launch with programmatic dependent launch: the kernel may start while the
                            preceding kernel of the stream is still running; it prefetches its (constant)
                            weights, then waits for that kernel to complete before it touches x, residual,
                            out or the workspace.  Safe after any kernel.                              */
  void *workspace;       /* split-k partials + counters (zeroed once by the caller; every launch
                            leaves the counters at zero), pt_linear_workspace_bytes             */
  size_t workspace_bytes;
  int32_t *error_flag;   /* optional device int, set non-zero if a bounded wait gave up        */
  const void *norm_beta; /* fp16 [k_in]   (PT_PRO_NORMCE)                           */
} pt_linear_args;

size_t pt_linear_workspace_bytes(int batch, int n_out, int max_ksplit);
int pt_linear(const pt_linear_args *args, void *stream);

/* pt_linear without any device allocation on the caller's side (no counterpart in the reference, whose ops get their
 * temporaries from the Poplar graph compiler).  Some hosts of this library cannot call cudaMalloc at the point where
 * they run a linear layer: a plugin loaded into a serving process whose memory pool is owned and sized by that process,
 * or a callback that runs inside a region where allocating is forbidden.  For them the split-k scratch (partial sums +
 * arrival counters) lives in a 4 MiB array inside the library image, one copy per GPU that loads the library, held until
 * the process exits.  `args->workspace` and `args->workspace_bytes` are ignored; x, weights and out are still the caller's.
 *   - Shapes whose scratch need exceeds 4 MiB are rejected with PT_ERR_INVALID (pt_last_error() names the need); use
 *     pt_linear with a workspace of your own for those.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first call
 *     before any stream capture begins.  Later calls only enqueue a small memset of the counters and the kernel.
 *   - Every call on a device shares the one array: calls that can overlap on the GPU (different streams without an
 *     ordering between them) race on it.  Serialise them on one stream or order them with events.
 *   - Nothing is allocated or freed, by this call or on its behalf. */
int pt_linear_static_scratch(const pt_linear_args *args, void *stream);

/* ---- tensor-core GEMMs for 16 or more activation rows (batched decode, prefill) ---------------------------------
 * The same layers as pt_linear (Linear.__call__ -> ParamHandler.matmul, poptransformer/layers/linear.py:42-46,
 * utils/param_handler/precision_strategy.py:56-81) when the batch no longer fits a matrix-vector kernel: the reference issues
 * one PopLibs matmul per layer whatever the batch (ops/popart.py:55-67); here 16 or more rows go to tcgen05 / tensor-memory
 * GEMMs fed by TMA.
 *   PT_W_FP8 : x = E4M3 bytes [m, k_in] (pt_cast_fp8 with x_scale), w = E4M3 bytes [n_out, k_in], out = fp16((x . w^T) * x_scale
 *              * w_scale) - the FP8MatMul op (custom_ops/matmul_fp8.cpp:885-1091).  w is either row-major as the checkpoint
 *              stores it (w_tiled = 0: what FP8MatMul passes; fetched with strided TMA boxes) or tiled once by pt_gemm_repack
 *              (w_tiled = 1: one contiguous bulk copy per stage, the layout for a model's weights).
 *   PT_W_INT4: x = fp16 [m, k_in], w = pt_gemm_repack of the reference's int8 [n_out, k_in/2] rows (w_tiled = 1), scales fp16
 *              [n_out, k_in/group]; every weight becomes fp16(q) * scale with one rounding (Int4ToHalf,
 *              custom_ops/int4_to_half_codelets.cpp:18-38) on its way to the tensor core.
 * k_in must be a multiple of 128.  Accumulation is fp32.  k-slices (ksplit, 0 = chosen by the library) are summed in a fixed
 * order; with more than one slice a workspace is needed (zeroed once by the caller; every launch leaves its counters at zero). */
typedef struct pt_gemm_args {
  int wfmt;               /* PT_W_FP8 or PT_W_INT4                                  */
  int m, n_out, k_in;
  int group;              /* INT4: scale group along k (a multiple of 128)          */
  int epilogue;           /* PT_EPI_STORE, PT_EPI_RESIDUAL or PT_EPI_BIAS            */
  int ksplit;             /* 0 = let the library choose                             */
  int w_tiled;            /* 1: w was tiled by pt_gemm_repack; 0: row-major (FP8 only) */
  const void *x, *w;
  const void *scales;     /* INT4: fp16 [n_out, k_in / group]                        */
  float x_scale, w_scale; /* FP8 per-tensor scales                                   */
  const void *residual;   /* fp16 [m, n_out]; may alias `out`                        */
  void *out;              /* fp16 [m, n_out]                                         */
  int out_ld;             /* row stride of `out` in elements; 0 = dense              */
  void *workspace;        /* pt_gemm_workspace_bytes                                 */
  size_t workspace_bytes;
  int32_t *error_flag;    /* optional device int, set non-zero (21..24) if a bounded wait gave up */
  const void *bias;       /* fp16 [n_out] (PT_EPI_BIAS)                              */
} pt_gemm_args;
size_t pt_gemm_workspace_bytes(int m, int n_out, int max_ksplit);
int pt_gemm(const pt_gemm_args *args, void *stream);
/* One-time tiling of a weight matrix for pt_gemm: [128-row tile][k block] with every tile contiguous.  FP8: E4M3 bytes
 * [n_out, k_in] -> 16 KB tiles in the 128-byte-swizzled image the tensor core reads.  INT4: the reference's int8
 * [n_out, k_in/2] rows (high nibble = even k, two's complement) -> 4 KB tiles of offset-binary nibbles in the word order
 * the transform step splits with two masks.  Rows are padded to a multiple of 128 (pt_gemm_packed_bytes). */
size_t pt_gemm_packed_bytes(int wfmt, int n_out, int k_in);
int pt_gemm_repack(int wfmt, const void *w, int n_out, int k_in, void *packed, void *stream);

/* ---- norms ------------------------------------------------------------------------
 * pt_norm_ce replaces the `NormCE` custom op (customized.py:69-102; custom_ops/NormCE.cpp:534-610):
 * fp16 rows, LayerNorm over `dim`; rows == 1 takes the GetInPlaceNorm arithmetic
 * (NormCECodelets.cpp:65-112), rows >= 2 the normInfKernel arithmetic (NormCECodelets.cpp:181-211).
 * Errors like the reference: dim % 4 != 0, dim >= 8192. */
int pt_norm_ce(const void *x, const void *gamma, const void *beta, int rows, int dim, float eps,
               void *out, void *stream);
/* RMSLayerNorm (layers/rms_layer_norm.py:26-36) with an optional fused residual add in front:
 * if residual != NULL: sum = fp16(x + residual) is written to sum_out and normalised. */
int pt_rms_norm(const void *x, const void *residual, const void *gamma, int rows, int dim, float eps,
                void *out, void *sum_out, void *stream);

/* ---- SoftmaxV3 --------------------------------------------------------------------
 * Replaces `SoftmaxV3` (customized.py:57-65; custom_ops/softmax.cpp:41-83). dtype: 0 = fp16, 1 = fp32. */
int pt_softmax(const void *x, int rows, int dim, int stable_mode, int dtype, void *out, void *stream);

/* ---- KVCache (reference layout) -----------------------------------------------------
 * Replaces `KVCache` (customized.py:21-35; custom_ops/kv_cache.cpp:94-187): `cache` is the op's
 * persistent state, viewed as [outer, max_len, inner] fp16 (sequence axis in the middle);
 * kv_new is [outer, step_len, inner].  cache <- concat(kv_new, (step==0 ? 0 : cache)[:max_len-step_len]).
 * `scratch` must hold outer*max_len*inner fp16 (the reference's clone). Bit-exact. */
int pt_kv_cache(const int32_t *step_dev, const void *kv_new, void *cache, void *scratch,
                int64_t outer, int max_len, int step_len, int64_t inner, void *stream);
/* `KVCachePipeline` (custom_ops/kv_cache_pipeline.cpp:374-451, kv_cache_codelet.cpp:18-212):
 * `caches` is [max_bps, outer, max_len, inner]; all caches are zeroed when step == 0; cache
 * step % max_bps receives the shifted insert and is copied to `out` [outer, max_len, inner]. */
int pt_kv_cache_pipeline(const int32_t *step_dev, const void *kv_new, void *caches, void *out,
                         int max_bps, int64_t outer, int max_len, int step_len, int64_t inner,
                         void *stream);
/* The two ops with 8-bit storage, the `fp8` attribute (customized.py:32; CastToUint8 / CastUint8ToFP16,
 * custom_ops/kv_cache.cpp:43-75, applied at :100-104 and :183-185; kv_cache_pipeline.cpp:386-388,
 * :437-439): kv_new (fp16) is cast to bytes before the shifted insert, the persistent caches hold bytes
 * ([outer, max_len, inner] / [max_bps, outer, max_len, inner] uint8) and `out` is the selected cache
 * cast back to fp16 [outer, max_len, inner].  The reference casts with Graphcore's F143 format; here the
 * bytes are OCP E4M3 (round to nearest even, saturating) of kv_new / scale, and out = fp16(decode * scale).
 * Bit-exact against that definition.  The shift is done in place: no scratch. */
int pt_kv_cache_fp8(const int32_t *step_dev, const void *kv_new, void *cache, void *out, float scale,
                    int64_t outer, int max_len, int step_len, int64_t inner, void *stream);
int pt_kv_cache_pipeline_fp8(const int32_t *step_dev, const void *kv_new, void *caches, void *out,
                             float scale, int max_bps, int64_t outer, int max_len, int step_len,
                             int64_t inner, void *stream);

/* ---- paged KV cache + fused decode attention ---------------------------------------------
 * Replaces, for one new token per sequence, the chain RoPE -> ops.kv_cache -> matmul(q,K^T) ->
 * scale/mask -> softmax_ce -> matmul(P,V) -> transpose/reshape
 * (llama2/attention.py:64-114; gpt2/attention.py:37-85; chatglm2/attention.py:166-312).
 * The cache is paged: pool[page][2][n_kv][page_size][head_dim] fp16, page_table[batch][max_pages].
 * Token t of sequence b lives in page page_table[b][t / page_size], slot t % page_size.
 * One block per (sequence, kv head, page): scores and P.V on the tensor cores (fp32 sums of exact fp16 products, scores rounded
 * to fp16 like the reference's matmul output), softmax statistics in fp32 (or the reference's fp16 exp), the pages of a head
 * combined in page order by the last block to arrive (deterministic). */
#define PT_ROPE_NONE 0
#define PT_ROPE_LLAMA 1    /* rotate_half, table [max_len, head_dim/2]  (llama2/attention.py:28-56) */
#define PT_ROPE_CHATGLM2 2 /* interleaved pairs on the first half of each head (chatglm2/attention.py:110-164) */
#define PT_SOFTMAX_F32 0   /* scores cast to fp32, exp in fp32 (llama2/attention.py:103-107) */
#define PT_SOFTMAX_F16 1   /* exp in fp16 (gpt2/attention.py:69, chatglm2/attention.py:289-291) */

typedef struct pt_attn_args {
  int batch, n_head, n_kv, head_dim; /* n_head % n_kv == 0                                   */
  int page_size, max_pages;          /* max_pages = pages per sequence in page_table          */
  int rope_mode, softmax_mode;
  float score_scale;                 /* multiplied onto fp16(q.k) in fp16; 1.0 = pre-folded    */
  const int32_t *step_dev;           /* position of the new token                             */
  const void *qkv;                   /* fp16 [batch, (n_head + 2*n_kv) * head_dim]: q | k | v  */
  const void *rope_sin, *rope_cos;   /* fp16 [max_len, rot_dim/2]                              */
  void *pool;                        /* this layer's page pool                                */
  const int32_t *page_table;         /* [batch, max_pages]                                    */
  void *out;                         /* fp16 [batch, n_head*head_dim]                          */
  int out_ld;                        /* row stride of `out` in elements; 0 = dense             */
  void *workspace;                   /* pt_attn_workspace_bytes                               */
  size_t workspace_bytes;
  int32_t *error_flag;               /* device int, set to 12 if *step_dev is out of range (the kernel has no waits) */
  int pdl;                           /* 1: programmatic dependent launch (see pt_linear_args.pdl) */
  int max_len;                       /* positions available: rows of rope_sin / rope_cos and of the id container; 0 = page_size *
                                        max_pages.  A launch that finds *step_dev outside [0, max_len) sets error_flag to 12 and
                                        does nothing else                                                                  */
  void *out_fp8;                     /* optional: E4M3 bytes [batch, n_head*head_dim] of out / out_fp8_scale, written beside `out`:
                                        the cast an FP8 linear applies to its input (precision_strategy.py:62-66) without a launch
                                        of its own                                                                          */
  float out_fp8_scale;
} pt_attn_args;

size_t pt_attn_workspace_bytes(int batch, int n_head, int head_dim, int max_pages);
int pt_kv_append_attn(const pt_attn_args *args, void *stream);
/* Logical view of a paged cache in the reference op's layout [2, batch, n_kv, max_len, head_dim],
 * newest token at index 0, zeros beyond `step` (custom_ops/kv_cache.cpp:118-132). */
int pt_kv_export(const void *pool, const int32_t *page_table, const int32_t *step_dev, int batch,
                 int n_kv, int head_dim, int page_size, int max_pages, int max_len, void *dense_out,
                 void *stream);
/* Beam reorder of a paged cache (no reference counterpart: the reference's BeamSearch op has no KV
 * reorder).  Row r continues from row parent[r].  Full pages are immutable and are shared by
 * permuting page-table rows; only the page that is still being filled (the one holding position
 * *step_dev) is copied, into the row's spare page, which then swaps roles with the row's old page.
 *   pt_kv_reorder_pages : per layer pool; copies the current page of row parent[r] into spare_pages[r].
 *   pt_kv_reorder_table : once per step, after every layer's copy; rewrites page_table and spare_pages.
 * `table_tmp` holds rows*max_pages int32. */
int pt_kv_reorder_pages(void *pool, const int32_t *page_table, const int32_t *spare_pages,
                        const int32_t *parent, const int32_t *step_dev, int rows, int n_kv, int head_dim,
                        int page_size, int max_pages, void *stream);
int pt_kv_reorder_table(int32_t *page_table, int32_t *table_tmp, int32_t *spare_pages, const int32_t *parent,
                        const int32_t *step_dev, int rows, int page_size, int max_pages, void *stream);

/* ---- prompt ingestion ("prefill") attention, Llama architecture ------------------------------------------------------
 * All tokens of a prompt in one pass: the attention of the reference's first stage, sequence_length = prompt length
 * (models/base_model.py:358-494; llama2/attention.py:64-114 with the causal mask and stable_mode = True).  qkv is fp16
 * [batch * n_tokens, 3 * n_head * head_dim] (row b * n_tokens + t holds q | k | v of token t of sequence b, position start + t);
 * q is rotated in place, rotated k and v are written to the paged cache (layout of pt_kv_append_attn), and out
 * [batch * n_tokens, n_head * head_dim] receives softmax(q K^T * score_scale + causal mask) V over positions 0 .. start + t.
 * head_dim 128, page_size 64, no grouped KV heads. */
typedef struct pt_prefill_attn_args {
  int batch, n_tokens, start, n_head, head_dim, page_size, max_pages, max_len;
  float score_scale;
  void *qkv;
  const void *rope_sin, *rope_cos;   /* fp16 [max_len, head_dim / 2] */
  void *pool;
  const int32_t *page_table;
  void *out;
} pt_prefill_attn_args;
int pt_prefill_attn(const pt_prefill_attn_args *args, void *stream);
/* Embedding rows of prompt tokens start .. start + n_tokens - 1 of every sequence (out row b * n_tokens + t), and the stop mask of
 * the reference's loop carry over them: sequence b is marked when ids[b, start + t + 1] == eos_id (models/base_model.py:313-346).
 * stop_mask may be NULL. */
int pt_prefill_embed(const void *table, const int32_t *ids, int ids_stride, int batch, int n_tokens, int start, int dim, int vocab,
                     int eos_id, int32_t *stop_mask, void *out, void *stream);

/* ---- persistent decode step (Llama architecture) ------------------------------------------------
 * One cooperative launch executes a whole iteration of the reference's decode loop body
 * (poptransformer/models/llama2/model.py:162-197, models/base_model.py:313-355) for batch <= 2: embedding, every
 * transformer block (INT4 linears packed by pt_linear_repack with PT_W_INT4; q|k|v fused, gate|up interleaved), final
 * RMSNorm, fp16 LM head (PT_W_FP16), greedy id and the loop-carry update (ids container, step, stop mask).
 * One block per SM streams its share of all weights through a shared-memory ring, so that HBM stays busy while the
 * SMs wait for each other's activations; those travel as tagged words that the consumers poll (no grid barrier between
 * phases).  INT4 linears run on the integer tensor-core path with the activations of every 128-k chunk in 16-bit block
 * fixed point (error far below the fp16 rounding of the result).  `layers` is a DEVICE array of n_layer entries.
 * The workspace and the x / qkv / attn / act scratch must be zeroed once before the first launch.
 * Weights: every matrix (q|k|v, o, gate|up, down, LM head) is first packed with pt_linear_repack and then re-ordered
 * with pt_llama_stream_permute into the order in which each SM's consumer warps read it (a permutation of the
 * packed tiles inside every SM's share; same size). */
int pt_llama_stream_permute(int wfmt, const void *packed, void *out, int n_out, int k_in, void *stream);
typedef struct pt_llama_layer {
  const void *qkv, *o, *gu, *down; /* packed INT4 weights                     */
  const void *ln1, *ln2;           /* fp16 RMSNorm weights [d_model]           */
  void *pool;                      /* this layer's KV page pool                */
} pt_llama_layer;

typedef struct pt_llama_step_args {
  int batch, d_model, n_head, head_dim, ffn, vocab, n_layer, max_len, page_size, max_pages, pad_id, eos_id;
  float norm_eps, score_scale;
  const pt_llama_layer *layers;
  const void *norm, *head, *emb;     /* final RMSNorm weight, packed fp16 LM head, fp16 embedding table [vocab, d_model] */
  const void *rope_sin, *rope_cos;   /* fp16 [max_len, head_dim/2]                                                   */
  int32_t *ids, *step_dev, *stop_mask, *next_ids; /* ids [batch, max_len]; stop_mask optional                          */
  const int32_t *page_table;         /* [batch, max_pages]                                                          */
  void *x, *qkv, *attn, *act;        /* scratch of 32-bit words, zeroed once: [batch, d_model], [batch, 3 d_model],
                                        [batch, d_model], [batch, ffn] (fp16 value + 16-bit phase tag per word)        */
  void *logits;                      /* optional fp16 [batch, vocab]                                                */
  void *workspace;                   /* pt_llama_step_workspace_bytes, zeroed once                                  */
  size_t workspace_bytes;
  int32_t *error_flag;               /* set non-zero if a bounded wait gave up (or, 12, if *step_dev is outside [0, max_len)) */
  uint64_t *trace;                   /* diagnostics, not a stable interface: optional [n_sm, n_layer, 32] global-timer stamps (ns) */
  int debug;                         /* diagnostics, not a stable interface: bit 0 = consume the weight tiles without the tile math;
                                        bits 16..31 = suspend-time hint (ns) of the shared-memory barrier waits (0 = default) */
  /* Tensor parallelism inside the kernel (tp_size > 1; one process and one launch per GPU, all ranks launch every step).
   * The reference's TP layers (layers/linear.py 'start' / 'end' strategies, layers/lm_head.py:75-116) map to: d_model = the
   * full hidden size, n_head = this rank's heads, ffn = width of this rank's k window of down_proj (a multiple of 128
   * holding its ffn_valid activations at ffn_offset; weights outside are zero), vocab = this rank's LM-head rows, first id
   * vocab_offset.  The all-reduce after o_proj / down_proj is fused into the kernel: every rank stores its fp16 partial
   * sums into its slot of every rank's exchange buffer (plain peer stores of tagged words, then one system-scope atomic
   * increment of an arrival counter per SM and rank), and the next staging step on every rank adds the slots in rank order.  tp_buffers[r] is rank r's exchange buffer as mapped in this process
   * (pt_llama_tp_buffer_bytes each, zeroed once); x must then hold two copies ([2, batch, d_model] words). */
  int tp_size, tp_rank, ffn_offset, ffn_valid, vocab_offset;
  int emb_rows;                      /* tp_size > 1: rows of the embedding table (the full vocabulary; the table is replicated) */
  void *tp_buffers[8];
  /* Early stop (HFDecBaseModel.early_stop, models/base_model.py:348-352).  Optional device int, zeroed by the caller before a
   * generation: the step that finds every stop_mask entry already set (the mask as it was before that step's own update, like
   * the reference's keep_going condition) sets it after finishing, and every later launch returns at once without touching
   * ids, step or the caches, so the host may poll it every few steps and still read the reference's final state. */
  int32_t *done_flag;
  /* 0: the kernel's polling loops on global memory give up after about two seconds (2^21 trips of one L2 / NVLink round trip);
   * non-zero: the short-wait build of the kernel is launched, which gives up after 2^12 trips (a few milliseconds).  A wait
   * that runs out sets error_flag, and the launch still terminates. */
  int wait_limit;
} pt_llama_step_args;

size_t pt_llama_step_workspace_bytes(int batch, int n_head, int head_dim, int max_pages);
size_t pt_llama_tp_buffer_bytes(int batch, int d_model, int tp_size);
int pt_llama_decode_step(const pt_llama_step_args *args, void *stream);

/* ---- top-k / LM-head ids / beam search --------------------------------------------------
 * pt_topk replaces ops.topk (popart.py:135-137) on [rows, dim] fp16 or fp32 (dtype 0/1): values
 * sorted descending, lowest index wins ties.  k <= 32. */
int pt_topk(const void *x, int rows, int dim, int k, int dtype, void *vals, int32_t *ids, void *stream);
/* Tensor-parallel LM head (layers/lm_head.py:75-116), k = 1.  pt_lm_head_local_topk: per-rank top-1 over the
 * rank's vocabulary slice with exact-zero logits read as -10000 (:86-88) and ids offset by
 * rank * ceil(V / tp) (:78-80, :90).  pt_lm_head_tp_pick: after the all-gather of (value, id) pairs laid out
 * [tp, rows], takes the first maximum over ranks (:110-115). */
int pt_lm_head_local_topk(const void *logits, int rows, int dim, int id_offset, void *vals, int32_t *ids, void *stream);
int pt_lm_head_tp_pick(const void *vals, const int32_t *ids, int tp, int rows, int32_t *next_ids, void *stream);

/* `BeamSearch` custom op (custom_ops/beam_search_custom_op.cpp:333-478): logits [b, beam, vocab]
 * (dtype 0 fp16 / 1 fp32), hyp int32 [b, max_len, beam] (in/out), prob [b, beam] (in/out, dtype of
 * logits), outputs next_id, global_best_id int32 [b, beam]; parent[b*beam] (optional) = flat cache
 * row each output slot continues from, for pt_kv_reorder.  Ties resolve to the lowest index. */
size_t pt_beam_search_workspace_bytes(int b, int beam, int max_len);
int pt_beam_search(const void *logits, int32_t *hyp, void *prob, const int32_t *step_dev, int b, int beam,
                   int vocab, int max_len, int dtype, int32_t *next_id, int32_t *global_best_id,
                   int32_t *parent, void *workspace, size_t workspace_bytes, void *stream);

/* ---- FP8 -----------------------------------------------------------------------------
 * `CastToUint8WithoutShapeInfer` (customized.py:127-135; custom_ops/cast_to_uint8.cpp:107-127) in the
 * OCP E4M3 + per-tensor fp32 scale form: out[i] = e4m3_rne_sat(x[i] / scale). */
int pt_cast_fp8(const void *x, float scale, int64_t n, void *out, void *stream);
/* `FP8MatMulWithoutShapeInfer` (customized.py:137-148; custom_ops/matmul_fp8.cpp:885-1091):
 * a e4m3 [m, k] (row-major), b e4m3 [n, k] (k contiguous), out fp16 [m, n] = (a.b^T) * sa * sb. */
int pt_fp8_matmul(const void *a, const void *b, float scale_a, float scale_b, int m, int n, int k,
                  void *out, void *stream);

/* ---- RWKV WKV ------------------------------------------------------------------------
 * poptransformer/models/rwkv/attention.py:66-105: k, v fp16 [b, c]; time_first/time_decay fp32 [c];
 * num/den/max fp32 [b, c] updated in place; out fp16 [b, c] = fp16(wkv). */
int pt_wkv(const void *k, const void *v, const float *time_first, const float *time_decay, float *num,
           float *den, float *max_state, int b, int c, void *out, void *stream);
/* Token-shift gates of RWKV (`gate`, rwkv/attention.py:59-64 and ffn.py:40-45): out_x = h * mix_x + (1 - mix_x) * state for up to
 * three fp16 mixing vectors [dim] (out_b / out_c optional), fp16 rounding after every op; then state <- hidden.
 * hidden, state, out_x fp16 [rows, dim]. */
int pt_rwkv_mix(const void *hidden, void *state, const void *mix_a, const void *mix_b, const void *mix_c, void *out_a,
                void *out_b, void *out_c, int rows, int dim, void *stream);
/* Element-wise steps of RWKV on fp16 [n]: mode 0 out = sigmoid(a) * b (receptance gate, attention.py:76,103, ffn.py:57-58);
 * mode 1 out = relu(a)^2 (ffn.py:53-54); mode 2 out = a / 2 (rescale_every, rwkv/model.py:115-116). */
int pt_rwkv_act(int mode, const void *a, const void *b, void *out, int64_t n, void *stream);

/* ---- loop-carry and small ops ----------------------------------------------------------
 * Embedding gather (layers/embedding.py:34-36): out[b] = table[ids[b*ids_stride + *step_dev]]. */
int pt_embedding(const void *table, const int32_t *ids, int ids_stride, const int32_t *step_dev,
                 int batch, int dim, int vocab, void *out, void *stream);
/* step_containers + step_loop_cond (models/base_model.py:313-355): step' = step+1; slot
 * ids[b, step'] takes next_ids[b] where it holds pad_id; stop_mask[b] |= (id == eos_id). */
int pt_step_containers(int32_t *ids, int batch, int max_len, int32_t *step_dev, const int32_t *next_ids,
                       int pad_id, int eos_id, int32_t *stop_mask, void *stream);
/* The same with the reference's early stop (models/base_model.py:348-352): when *done_flag is set the call changes nothing;
 * otherwise, if every stop_mask entry was already set before this update, it sets *done_flag after the update (the reference
 * evaluates keep_going on the incoming mask, so the loop body runs once more after the last sequence produced its eos id).
 * done_flag: device int, zeroed by the caller before a generation. */
int pt_step_containers_early_stop(int32_t *ids, int batch, int max_len, int32_t *step_dev, const int32_t *next_ids,
                                  int pad_id, int eos_id, int32_t *stop_mask, int32_t *done_flag, void *stream);
/* SwiGLU behind a fused gate|up linear (llama2/mlp.py:20-28, chatglm2/mlp.py:51-59): gate_up fp16 [rows, 2 f] with the gate
 * features first; out[r, j] = fp16(up[r, j] * swish(gate[r, j])), swish in float32 rounded once.  out_ld: row stride (0 = f). */
int pt_swiglu(const void *gate_up, int rows, int f, void *out, int out_ld, void *stream);
/* The activation side of an FP8 linear as its own kernel, for the layers that run on pt_gemm (the FP8 linear casts its
 * input with the scale stored beside the weight, utils/param_handler/precision_strategy.py:62-66):
 * pt_rms_norm_fp8: out bytes = e4m3(RMSNorm(x) / act_scale), the RMSNorm with the reference's fp16 roundings
 * (layers/rms_layer_norm.py:26-36); pt_swiglu_fp8: out bytes = e4m3(fp16(up * swish(gate)) / act_scale) from the fused
 * [gate features | up features] rows (chatglm2/mlp.py:51-59). */
int pt_rms_norm_fp8(const void *x, const void *gamma, int rows, int dim, float eps, float act_scale, void *out, void *stream);
int pt_swiglu_fp8(const void *gate_up, int rows, int f, float act_scale, void *out, int out_ld, void *stream);
/* Elementwise fp16: out = fp16(a + b) (ops.add). */
int pt_add_f16(const void *a, const void *b, int64_t n, void *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PT_B200_H */
