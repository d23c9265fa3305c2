/*
 * b200_decode.h — C-ABI of the B200-native decode path.
 *
 * The reference (psurabh/Enterprise-Inference v1.3.0) has NO in-process FFI for this path:
 * its boundary is the container contract of core/helm-charts/vllm (image + args + env + HTTP,
 * /root/reference/core/helm-charts/vllm/templates/deployment.yaml:57,66-87 and
 * /root/reference/docs/api-spec.yaml:6-49).  The arithmetic runs inside the third-party
 * image vllm-cpu-release-repo:v0.10.2 (values.yaml:23-28).  Each entry point below therefore
 * cites the step of that image's decode loop it replaces (the
 * [V22] citations are the vLLM 0.22 wheel used as the readable statement of the math).
 *
 * Conventions
 *  - every function returns 0 on success, a negative b200_status otherwise; the text of the
 *    last error of the calling thread is b200_last_error(); nothing throws across the ABI;
 *  - every tensor is a CALLER-OWNED DEVICE pointer (e.g. torch tensor.data_ptr()) unless the
 *    parameter name starts with host_; bf16 unless stated; row-major; explicit leading dims;
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing syncs
 *    unless documented;
 *  - no hidden allocation after b200_ctx_create(): scratch is either inside the ctx or passed
 *    by the caller as (workspace, workspace_bytes) with a *_workspace_bytes() query;
 *  - a ctx is not re-entrant: one engine thread per rank drives it; TP ranks are processes.
 */
#ifndef B200_DECODE_H
#define B200_DECODE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

typedef struct b200_ctx b200_ctx;

typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_INVALID = -1,      /* bad argument / shape */
  B200_ERR_CUDA = -2,         /* a CUDA runtime/driver call failed */
  B200_ERR_UNSUPPORTED = -3,  /* shape outside what the kernels were built for */
  B200_ERR_NCCL = -4,
  B200_ERR_STATE = -5         /* call order (weights not set, ...) */
} b200_status;

B200_API const char* b200_last_error(void);
B200_API int b200_abi_version(void);
/* 1 when a CUDA device of compute capability 10.x is current, else 0 (no error text). */
B200_API int b200_device_ok(void);

/* ---- model / context ------------------------------------------------------------------ */
typedef struct b200_model_cfg {
  int32_t hidden, n_layers, n_q_heads, n_kv_heads, head_dim; /* GLOBAL sizes; head_dim == 128 */
  int32_t intermediate, vocab;
  int32_t qkv_bias;            /* Qwen2: 1 */
  float rms_eps;
  int32_t block_size;          /* KV block, tokens: 128 (xeon-values.yaml:72-73 --block-size) */
  int32_t max_tokens;          /* max token rows in one step (--max-num-batched-tokens 2048) */
  int32_t max_blocks_per_seq;  /* ceil(max-model-len / block_size) */
  int32_t tp_rank, tp_world;   /* tensor parallel (deployment.yaml:72-78 --tensor-parallel-size) */
} b200_model_cfg;

typedef enum b200_weight_kind {
  B200_W_EMBED = 0,     /* [vocab, hidden]                      (a1)  replicated on every rank */
  B200_W_LN1 = 1,       /* [hidden]                             (a2)  */
  B200_W_QKV = 2,       /* [(hq+2hkv)_local*128, hidden]        (a3)  q|k|v rows, column-parallel */
  B200_W_QKV_BIAS = 3,  /* [(hq+2hkv)_local*128]                      */
  B200_W_O = 4,         /* [hidden, hq_local*128]               (a7)  row-parallel */
  B200_W_LN2 = 5,       /* [hidden]                                   */
  B200_W_GATE_UP = 6,   /* [2*I_local, hidden] gate rows then up rows (a8) */
  B200_W_DOWN = 7,      /* [hidden, I_local]                    (a8)  row-parallel */
  B200_W_FINAL_NORM = 8,/* [hidden]                             (a9)  */
  B200_W_LM_HEAD = 9,   /* [vocab_local, hidden]                (a9)  vocab-parallel */
  B200_W_GATE_UP_INTERLEAVED = 10 /* [2*I_local, hidden] in 128-row slabs: 64 gate rows, then the 64 matching
                                     up rows — lets the gate_up linear apply SiLU*mul in its epilogue (set
                                     this OR B200_W_GATE_UP; needs I_local % 64 == 0) */
} b200_weight_kind;

/* Replaces: model construction inside the image's worker (one per TP rank,
 * xeon-values.yaml:78-79 --distributed_executor_backend mp).  Allocates the ctx's private
 * activation/scratch buffers (the only cudaMalloc calls in the library). */
B200_API int b200_ctx_create(const b200_model_cfg* cfg, b200_ctx** out);
B200_API int b200_ctx_destroy(b200_ctx* ctx);
/* Bytes of device memory the ctx allocated in b200_ctx_create(). */
B200_API int64_t b200_ctx_workspace_bytes(const b200_ctx* ctx);

/* Replaces: weight loading ([V22] vllm/model_executor/models/llama.py:437-444 packing map).
 * The pointer is borrowed for the life of the ctx; `layer` is ignored for EMBED/FINAL_NORM/
 * LM_HEAD.  rows/cols are checked against the cfg (local TP shard sizes). */
B200_API int b200_set_weight(b200_ctx* ctx, int32_t layer, int32_t kind, const void* w, int64_t rows, int64_t cols);

/* KV cache, caller-owned, one allocation per K and V:
 *   [n_layers][n_blocks][n_kv_heads_local][block_size][head_dim] bf16
 * so one (block, kv head) is a contiguous 32 KiB tile — one bulk-async copy per tile.
 * Replaces the image-internal cache ([V22] vllm/v1/attention/backends/cpu_attn.py:88-100). */
B200_API int b200_set_kv_cache(b200_ctx* ctx, void* k_cache, void* v_cache, int64_t n_blocks);

/* cos|sin cache [max_pos][head_dim] bf16 ([V22] rotary_embedding/base.py:58-63,82-92). */
B200_API int b200_set_rope_cache(b200_ctx* ctx, const void* cos_sin, int64_t max_pos);

/* NCCL communicator for TP (replaces the image's shm all-reduce,
 * [V22] vllm/distributed/device_communicators/cpu_communicator.py:229-276).
 * b200_nccl_unique_id writes 128 bytes to host_id (rank 0 calls it and shares the bytes);
 * b200_nccl_init is collective over the tp_world ranks of the ctx. */
B200_API int b200_nccl_unique_id(void* host_id128);
B200_API int b200_nccl_init(b200_ctx* ctx, const void* host_id128);

/* Peer-memory all-reduce (optional, after b200_nccl_init): every rank exports the CUDA-IPC handle of its
 * all-reduce buffers (64 bytes), the ranks exchange them, and each imports all `world` handles (rank
 * order).  From then on the two all-reduces per layer run as ONE kernel per rank over NVLink peer loads
 * (flag barrier + rank-ordered fp32 sum) instead of NCCL; NCCL stays the fallback when this is skipped. */
B200_API int b200_tp_ipc_export(b200_ctx* ctx, void* host_handle64);
B200_API int b200_tp_ipc_import(b200_ctx* ctx, const void* host_handles, int32_t world);

/* ---- the hot path: one scheduler step ----------------------------
 * Replaces ModelRunner.execute_model of the image for one batch of token rows
 * ([V22] vllm/model_executor/models/llama.py:395-434 + sampler.py:235-236).
 * Row t is one new token: ids[t], positions[t], slot_mapping[t] = block_id*block_size+off,
 * ctx_lens[t] = tokens it attends to (position+1), row_to_seq[t] = its row of block_table
 * (NULL: row t).  Decode rows and (chunked) prefill rows have the same form, a prefill chunk
 * being T rows of one sequence with ctx_lens 1..T (+offset).
 * logit_rows[n_logit_rows] selects the rows that get lm_head + greedy sampling (NULL: all).
 * out_token_ids[n_logit_rows] int32; out_logits (nullable) bf16 [n_logit_rows][vocab].
 * max_ctx_len is a HOST hint >= max(ctx_lens) that sizes the split-KV grid.
 * With tp_world > 1 it is collective over the ranks. */
B200_API int b200_decode_step(b200_ctx* ctx, const int32_t* ids, const int32_t* positions,
                     const int32_t* slot_mapping, const int32_t* block_table, int32_t bt_stride,
                     const int32_t* row_to_seq, const int32_t* ctx_lens, int32_t n_tokens,
                     int32_t max_ctx_len, const int32_t* logit_rows, int32_t n_logit_rows,
                     int32_t* out_token_ids, void* out_logits, void* stream);

/* Same step, driven from PINNED HOST memory: one packed int32 buffer
 *   [ids | positions | slot_mapping | ctx_lens | row_to_seq | logit_rows](each n_tokens, the
 *   last n_logit_rows) followed by block_table [n_seqs][bt_stride] (and, for a ctx with per-sequence state slots,
 *   seq_slots [n_seqs]: see b200_stack_set_state),
 * copied H2D, the step, and the sampled ids copied D2H into host_out_token_ids.  The copies
 * are enqueued on `stream`; the caller synchronises.  This is the call the serving engine
 * makes every iteration (the `e2e` figure of bench.py).
 * An id of -(j+1) stands for the token the PREVIOUS b200_decode_step_host call on this ctx chose for
 * its logit row j (it is still on the device): an engine can enqueue step n+1 while step n runs and
 * read step n's tokens afterwards (vLLM's async scheduling).  host_packed and host_out_token_ids must
 * stay untouched until their copies have completed, so such an engine alternates two buffers of each. */
B200_API int b200_decode_step_host(b200_ctx* ctx, const int32_t* host_packed, int32_t n_tokens,
                          int32_t n_seqs, int32_t bt_stride, int32_t max_ctx_len,
                          int32_t n_logit_rows, int32_t* host_out_token_ids, void* stream);

/* Graph replay: 1 (default) captures each distinct step shape into a CUDA graph; 0 = eager
 * launches (the chart's --enforce-eager is accepted by the server but does not force this). */
B200_API int b200_ctx_set_graphs(b200_ctx* ctx, int32_t enabled);
/* Number of kernels one step of the given shape launches (bench.py's gpu_launches). */
B200_API int b200_ctx_last_step_launches(const b200_ctx* ctx);
/* Per-layer hidden/residual taps for parity tests: after a step, copies the layer's MLP
 * output and residual rows ([n_tokens][hidden] bf16 each) — only valid with graphs off. */
B200_API int b200_ctx_set_tap(b200_ctx* ctx, int32_t layer, void* out_hidden, void* out_residual);

/* ---- per-kernel entry points (unit tests, ncu) ------------------------------------------ */

/* Launch attribute for the per-kernel entry points called from THIS thread: 1 = programmatic dependent
 * launch (the kernels of b200_decode_step always use it unless B200_PDL=0): a kernel's prologue and first
 * weight tiles overlap the previous kernel's tail.  Default 0. */
B200_API int b200_set_launch_pdl(int32_t enabled);

/* y[T][n_out] = x[T][k] . w[n_out][k]^T (+bias), fp32 accumulate, one rounding to bf16.
 * Replaces sgl-kernel weight_packed_linear / oneDNN matmul of the image
 * ([V22] vllm/model_executor/layers/utils.py:277-299).  impl: 0 auto, 1 CUDA-core GEMV
 * (HBM-bound, T small), 2 tcgen05/TMEM weight-streaming GEMM.  Scratch (split-K partials
 * and slab tickets) comes from the caller: the first 64 KiB of the workspace must be ZERO before
 * its first use (cudaMemset once); every launch leaves them zero again. */
B200_API int64_t b200_linear_workspace_bytes(int32_t n_tokens, int32_t n_out, int32_t k);
B200_API int b200_linear_bf16(const void* x, int64_t ldx, const void* w, const void* bias, void* y,
                     int64_t ldy, int32_t n_tokens, int32_t n_out, int32_t k, int32_t impl,
                     void* workspace, int64_t workspace_bytes, void* stream);

/* Fused epilogues of the tcgen05 linear (what b200_decode_step uses): mode 1 = a8's SiLU*mul over
 * interleaved gate|up slabs (w as B200_W_GATE_UP_INTERLEAVED; y is [T][n_out/2]); mode 2 = a4+a5:
 * w is the fused qkv projection, RoPE is applied to q/k heads, q goes to y[T][ldy], k/v rows go to
 * the paged cache at slot_mapping[t] (pointers unused by mode 1 may be NULL).  Results are
 * bit-identical to b200_linear_bf16(impl=2) followed by b200_silu_mul / b200_rope_kv_append. */
B200_API int b200_linear_fused_bf16(const void* x, int64_t ldx, const void* w, const void* bias, void* y,
                           int64_t ldy, int32_t n_tokens, int32_t n_out, int32_t k, int32_t mode,
                           const int32_t* positions, const int32_t* slot_mapping, const void* cos_sin,
                           void* k_cache_layer, void* v_cache_layer, int32_t n_q_heads, int32_t n_kv_heads,
                           int32_t block_size, void* workspace, int64_t workspace_bytes, void* stream);

/* (a2 folded into a3/a7/a8/a9) RMSNorm without a kernel of its own, for steps of at most 64 rows.  The residual
 * stream lives in fp32: sres[T][hidden] holds s = x + res UNROUNDED (what [V22] vllm/ir/ops/layernorm.py:40-58
 * takes the variance of and normalises; the bf16 residual of the next layer is bf16(s), recomputed on read) and
 * ssq[T][hidden/128] the sums of squares of s per 128-wide slab.
 *  - b200_embed_stream: (a1) sres[t] = float(table[ids[t]]) and its ssq;
 *  - b200_linear_residual_bf16: (a7, a8-down) x = bf16(x_in . w^T + bias); sres = x + bf16(sres); ssq rewritten
 *    (n_out = hidden, a multiple of 128; no y is written);
 *  - b200_linear_normed_bf16: (a3, a8-gate_up, a9) the linear over y_in[t] = bf16(bf16(s * rinv) * norm_w),
 *    rinv = 1/sqrt(sum(ssq[row]) / k + eps), s = sres[rows ? rows[t] : t] (k = hidden); the rows are normalised
 *    inside the kernel while the weights stream.  mode / trailing arguments as b200_linear_fused_bf16 (0 = plain);
 *  - b200_rmsnorm_stream: the same normalised rows written out as bf16 [n_rows][hidden].
 * The summation order of the variance is the one b200_rmsnorm uses, so a step through these entry points is
 * bit-identical to embed -> rmsnorm -> linear -> ... with bf16 activations. */
B200_API int b200_embed_stream(const int32_t* ids, const void* table, float* sres, float* ssq, int32_t n_tokens,
                      int32_t hidden, int32_t vocab, void* stream);
B200_API int b200_linear_residual_bf16(const void* x, int64_t ldx, const void* w, const void* bias, float* sres,
                              float* ssq, int32_t n_tokens, int32_t n_out, int32_t k, void* workspace,
                              int64_t workspace_bytes, void* stream);
B200_API int b200_linear_normed_bf16(const float* sres, const float* ssq, const void* norm_w, float eps,
                            const int32_t* rows, const void* w, const void* bias, void* y, int64_t ldy,
                            int32_t n_tokens, int32_t n_out, int32_t k, int32_t mode, const int32_t* positions,
                            const int32_t* slot_mapping, const void* cos_sin, void* k_cache_layer,
                            void* v_cache_layer, int32_t n_q_heads, int32_t n_kv_heads, int32_t block_size,
                            void* workspace, int64_t workspace_bytes, void* stream);
B200_API int b200_rmsnorm_stream(const float* sres, const float* ssq, const int32_t* rows, const void* w, void* y,
                        int32_t n_rows, int32_t hidden, float eps, void* stream);

/* (a2) y = rmsnorm(x)*w, or with res != NULL: s=x+res; res=bf16(s); y=rmsnorm(s)*w
 * ([V22] vllm/ir/ops/layernorm.py:10-21,40-58). y may alias x. */
B200_API int b200_rmsnorm(const void* x, void* res, const void* w, void* y, int32_t n_tokens,
                 int32_t hidden, float eps, void* stream);

/* (a1) x[t] = table[ids[t]] ([V22] llama.py:371-375,392-393). */
B200_API int b200_embed(const int32_t* ids, const void* table, void* out, int32_t n_tokens,
               int32_t hidden, int32_t vocab, void* stream);

/* (a4+a5) in-place NeoX RoPE on the q and k heads of qkv[T][(hq+2hkv)*128] in bf16
 * arithmetic, then k,v rows written to the paged cache at slot_mapping[t]
 * ([V22] rotary_embedding/common.py:160-183; cpu_attn.py:342-362 reshape_and_cache). */
B200_API int b200_rope_kv_append(void* qkv, const int32_t* positions, const int32_t* slot_mapping,
                        const void* cos_sin, void* k_cache_layer, void* v_cache_layer,
                        int32_t n_tokens, int32_t n_q_heads, int32_t n_kv_heads,
                        int32_t block_size, void* stream);

/* (a6) paged attention, one query row per token, split-KV with LSE merge
 * ([V22] cpu_attn.py:377-396).  q rows are the first hq*128 columns of a [T][ldq] buffer. */
B200_API int64_t b200_paged_attn_workspace_bytes(int32_t n_tokens, int32_t n_q_heads, int32_t max_ctx_len,
                                        int32_t block_size);
B200_API int b200_paged_attn_decode(const void* q, int64_t ldq, const void* k_cache_layer,
                           const void* v_cache_layer, const int32_t* block_table, int32_t bt_stride,
                           const int32_t* row_to_seq, const int32_t* ctx_lens, void* out,
                           int64_t ldo, int32_t n_tokens, int32_t n_q_heads, int32_t n_kv_heads,
                           int32_t block_size, int32_t max_ctx_len, float scale, void* workspace,
                           int64_t workspace_bytes, void* stream);

/* (a6, prefill rows) Same contract and results as b200_paged_attn_decode, for steps dominated by the rows of
 * a prefill chunk: up to 4 consecutive rows that belong to one sequence (row_to_seq) share ONE pass over that
 * sequence's K/V cache with a per-row causal mask (their query heads fill the 16 MMA columns); rows of
 * different sequences inside a group fall back to one pass each.  Chunked prefill in the reference:
 * xeon-values.yaml:80-83 (--enable_chunked_prefill, --max-num-batched-tokens 2048). */
B200_API int b200_paged_attn_prefill(const void* q, int64_t ldq, const void* k_cache_layer,
                            const void* v_cache_layer, const int32_t* block_table, int32_t bt_stride,
                            const int32_t* row_to_seq, const int32_t* ctx_lens, void* out, int64_t ldo,
                            int32_t n_tokens, int32_t n_q_heads, int32_t n_kv_heads, int32_t block_size,
                            int32_t max_ctx_len, float scale, void* workspace, int64_t workspace_bytes,
                            void* stream);

/* No counterpart in the reference: a variant of b200_paged_attn_decode for callers that cannot
 * allocate device memory after start-up (engines with a fixed memory plan, bindings that cannot call
 * cudaMalloc).  Same inputs, outputs and results, but the split-KV partials live in a 2 MiB array
 * built into the library (b200_paged_attn_static_scratch_bytes(); held by every GPU that loads the
 * library until exit) and the call allocates nothing.  Shapes whose partials exceed the array return
 * B200_ERR_UNSUPPORTED with the sizes in b200_last_error().  The first call on each device looks up
 * the array's device address: make it before any stream capture.  All calls on a device share the
 * array — keep them on one stream; calls that overlap on the GPU race. */
B200_API int64_t b200_paged_attn_static_scratch_bytes(void);
B200_API int b200_paged_attn_decode_static(const void* q, int64_t ldq, const void* k_cache_layer,
                                  const void* v_cache_layer, const int32_t* block_table, int32_t bt_stride,
                                  const int32_t* row_to_seq, const int32_t* ctx_lens, void* out,
                                  int64_t ldo, int32_t n_tokens, int32_t n_q_heads, int32_t n_kv_heads,
                                  int32_t block_size, int32_t max_ctx_len, float scale, void* stream);

/* (a8) out[T][I] = bf16(bf16(silu(g))*u), gu = [T][2I] gate|up ([V22] activation.py:137-141). */
B200_API int b200_silu_mul(const void* gu, void* out, int32_t n_tokens, int32_t intermediate, void* stream);

/* (a10) greedy: fp32 argmax of bf16 logits, ties -> lowest index ([V22] sampler.py:90-91,235-236).
 * Also writes the winning value (fp32) when out_max != NULL (used by the TP (max,idx) reduce). */
B200_API int b200_argmax(const void* logits, int64_t ld, int32_t n_rows, int32_t vocab, int32_t index_offset,
                int32_t* out_ids, float* out_max, void* stream);

/* (a10, widened) stochastic sampling for requests that do not ask for greedy decoding: per row
 * logits / temperature, top-k mask (values below the k-th largest dropped, ties at it kept), top-p on the
 * renormalised rest (the smallest-probability tokens with cumulative mass <= 1 - p dropped), one draw
 * ([V22] vllm/v1/sample/sampler.py:90-91,235-256, ops/topk_topp_sampler.py; fields of docs/api-spec.yaml).
 * temperature[r] <= 0 -> the argmax of b200_argmax.  top_k[r] <= 0 and top_p[r] >= 1 disable the filters.
 * The draw is a function of (seeds[r], draws[r], logits row): same inputs, same token.  All arrays are device
 * pointers of n_rows elements; temperature/top_k/top_p/min_p/seeds/draws may be NULL (0, off, off, off, 0, 0).
 * min_p[r] in (0, 1]: tokens whose probability is below min_p x the largest one are dropped before top-k/top-p
 * ([V22] vllm/v1/sample/logits_processor/builtin.py:101).  vLLM compares in probability space; this kernel compares
 * the logit with max + T log(min_p), the same cut up to fp32 rounding of a token that sits exactly on it. */
B200_API int b200_sample(const void* logits, int64_t ld, int32_t n_rows, int32_t vocab, const float* temperature,
                const int32_t* top_k, const float* top_p, const float* min_p, const uint64_t* seeds,
                const uint64_t* draws, int32_t* out_ids, void* stream);

/* Sampling over the logit rows of the LAST b200_decode_step[_host] of this ctx (they are still in the ctx's
 * buffer; with tensor parallelism the vocab shards are all-gathered first: a collective, call it on every rank
 * with the same arguments).  host_params = five host arrays back to back,
 *   float temperature[n] | int32 top_k[n] | float top_p[n] | float min_p[n] (0: off) | uint64 seed[n] | uint64 draw[n],
 * 32 n bytes; host_out_ids receives n token ids (asynchronously: synchronise the stream before reading). */
B200_API int b200_ctx_sample_last(b200_ctx* ctx, int32_t n_rows, const void* host_params, int32_t* host_out_ids,
                         void* stream);

/* (a10, widened) OpenAI `logit_bias`, `frequency_penalty`, `presence_penalty` and vLLM's `repetition_penalty` on logit
 * rows [n_rows][ld] (bf16, modified in place), in the image's order and arithmetic ([V22] vllm/v1/sample/sampler.py:366-416,
 * vllm/model_executor/layers/utils.py:51-89, vllm/_custom_ops.py:360-373), fp32 per touched token:
 *   x += bias;  if the token is in the prompt or the output: x *= (x > 0 ? 1/rep : rep);
 *   x -= freq * (occurrences in the output);  x -= pres * (occurs in the output ? 1 : 0)
 * then ONE rounding back to bf16 (the image keeps the processed logits in fp32: the only deviation).  Sparse: row r owns
 * the entries offsets[r] .. offsets[r+1]-1 of (ids, counts, seen, bias), distinct tokens per row; row_params = (rep, freq,
 * pres) per row.  Device pointers.  b200_ctx_adjust_last applies the same to the logit rows of the LAST step of a ctx from
 * ONE packed host buffer (float row_params[3n] | int32 offsets[n+1] | int32 ids[E] | int32 counts[E] | int32 seen[E] |
 * float bias[E]); call it before b200_ctx_sample_last, on every tensor-parallel rank (each adjusts its vocabulary shard). */
B200_API int b200_logit_adjust(void* logits, int64_t ld, int32_t n_rows, int32_t vocab, const float* row_params,
                      const int32_t* offsets, const int32_t* ids, const int32_t* counts, const int32_t* seen,
                      const float* bias, void* stream);
B200_API int b200_ctx_adjust_last(b200_ctx* ctx, int32_t n_rows, const void* host_packed, int32_t n_entries, void* stream);

/* (a10, widened) OpenAI `logprobs` / `top_logprobs`: log softmax over the raw logits (vLLM's default logprobs mode,
 * [V22] vllm/v1/sample/sampler.py:90-118).  out_logprob[r] = l[token_ids[r]] - logsumexp(l); out_top_ids /
 * out_top_logprobs [r][n_top] = the n_top (<= 32) most likely tokens, value descending, ties by lowest index
 * (may be NULL when n_top == 0).  Device pointers. */
B200_API int b200_logprobs(const void* logits, int64_t ld, int32_t n_rows, int32_t vocab, const int32_t* token_ids,
                  int32_t n_top, float* out_logprob, int32_t* out_top_ids, float* out_top_logprobs, void* stream);

/* The same over the logit rows of the LAST step of this ctx (a collective under tensor parallelism, like
 * b200_ctx_sample_last).  host_out receives float logprob[n] | int32 top_ids[n][n_top] | float top_logprobs[n][n_top]
 * (4 n (1 + 2 n_top) bytes), asynchronously. */
B200_API int b200_ctx_logprobs_last(b200_ctx* ctx, int32_t n_rows, const int32_t* host_token_ids, int32_t n_top,
                           void* host_out, void* stream);

/* (a0) device-side scheduler advance for pure-decode rows: ids[t]=sampled[t], positions[t]+=1,
 * ctx_lens[t]=positions[t]+1, slot_mapping[t] from the block table.  The image's scheduler does this
 * on the host every iteration ([V22] vllm/v1/attention/backends/cpu_attn.py:107-117 metadata build);
 * on the device it lets several decode steps run without a host round trip.  The caller guarantees
 * the block table already covers the next position. */
B200_API int b200_advance_decode_rows(int32_t* ids, int32_t* positions, int32_t* slot_mapping,
                                      int32_t* ctx_lens, const int32_t* block_table, int32_t bt_stride,
                                      const int32_t* row_to_seq, const int32_t* sampled, int32_t n_rows,
                                      int32_t block_size, void* stream);

/* (a11) sum all-reduce of a bf16 buffer over the ctx's TP communicator. */
B200_API int b200_allreduce_bf16(b200_ctx* ctx, void* buf, int64_t count, void* stream);

/* (a11) The collective of one half-layer exactly as b200_decode_step runs it, as an entry point of its own (tests,
 * timing): `partial` [T][hidden] bf16 is this rank's row-parallel partial sum (NULL: reuse what the exchange buffer
 * holds); buf_idx 0 = the O projection's buffer, 1 = the down projection's (they alternate inside a step, and so
 * must consecutive calls).  norm_w == NULL: y = all-reduce(partial).  norm_w != NULL: the fused form the step uses,
 * s = bf16(all-reduce(partial)) + res; res = bf16(s); y = rmsnorm(s) * norm_w (above 16 rows the peer-memory path deals
 * the rows to the ranks: res is then current only for the rows t with t mod tp_world == tp_rank; res == NULL and
 * y == NULL: run on the ctx's own residual / normed rows without any copy, for timing).  Every rank must make the same call.
 * Replaces the shm all-reduce of the image's CPU communicator followed by its fused_add_rms_norm
 * ([V22] vllm/distributed/device_communicators/cpu_communicator.py:229-276; vllm/ir/ops/layernorm.py:40-58). */
B200_API int b200_tp_allreduce(b200_ctx* ctx, int32_t buf_idx, const void* partial, int32_t n_tokens, void* res,
                      const void* norm_w, void* y, void* stream);

/* ---- models described layer by layer ---------------------------------------------------------------------------------
 * No counterpart in the reference chart's model list: decoder-only designs whose layers differ from one another or use
 * mechanisms outside the Llama / Qwen2 stack are given as a list of layer descriptors.  The ctx they create is driven by
 * the SAME step, sampling, log-probability and logit-adjust entry points as above (b200_decode_step[_host],
 * b200_ctx_sample_last, ...); only construction, weights and caches differ.  Single GPU (tp_world 1).
 *
 * Layer = mixer sublayer + optional feed-forward sublayer over an fp32 residual stream x, each sublayer wrapped in bias-free
 * layer norms on both sides:  x += norm_post(sublayer(norm_pre(x))).
 *
 * B200_MIXER_ATTENTION: grouped-query causal softmax attention.  q and k are RMS-normalised over the WHOLE projection
 * (weights of that size) before rotation; the leading rot_dims dimensions of each q/k head rotate in the interleaved pair
 * layout by angles read from cos|sin table `rot_table` (frequency scaling and magnitude factors are baked into the table by
 * the host); values are scaled to unit RMS per head and, when vrot_table >= 0, rotated over all their dimensions by their
 * own position, with the attention output turned back by the query's position; score = q.k * scale.
 *
 * B200_MLP_MOE: routed experts.  Router softmax over all experts; choice by score + bias, group-limited (experts in
 * `groups` equal runs of neighbours, only the `keep` best groups eligible), `top` experts; mixing weights = the plain
 * softmax scores, not renormalised; expert = down(silu(gate x) * (up x)).
 *
 * Second layer form (b200_stack_cfg.form = B200_FORM_PARALLEL): both sublayers read the same stream,
 *   x_next = x + mixer(h1 + conv(h1)) + ff(h2),   h1 = x / rms(x) * g1,  h2 = x / rms(x) * g2   (g1, g2: one number each),
 * conv a causal per-channel convolution over `canon_taps` time steps (0: none), and, with depth_avg, the stream handed to
 * the next layer is a weighted sum of the embedding output and of every layer result so far.  Models of this form may
 * add a hashed bigram table to the embedding, cap the logits with cap * tanh(z / cap), and use
 *
 * B200_MIXER_LATENT: causal softmax attention whose keys and values are expanded from ONE cached vector per token.  The
 * fused projection gives, per token, the queries (per head `dim` plain and `rot_dim` rotated dimensions), a latent of
 * `kv_rank` dimensions (RMS-normalised with a weight) and one rotated key part of `rot_dim` dimensions shared by all heads;
 * a head's plain key is W_uk c and its value W_uv c.  The cache row is [c | rotated key part]; scores are taken in the
 * latent space (q' = W_uk^T q, one kv head of kv_rank + rot_dim dimensions whose value is the row's first kv_rank entries),
 * the weighted latent sum is expanded by W_uv.  mixer_flags: B200_MIXF_SINK adds exp(sink[head]) to the softmax
 * denominator; B200_MIXF_GATE multiplies the concatenated heads by sigmoid(W_g h).
 *
 * B200_MIXER_MLSTM: matrix-memory recurrence per head, fp32 state S [dim][vdim], n [dim], m carried per sequence in a state
 * slot: log gates i = cap tanh((W_i h + b_i) / cap), f = logsigmoid(cap tanh((W_f h + b_f) / cap));
 * m' = max(f + m, i); S' = exp(f + m - m') S + exp(i - m') k v^T (n' likewise with k); o = S'^T q / (max(|n'.q|, exp(-m')) + 1e-6)
 * with q scaled by dim^-1/2; each head's o is brought to unit RMS, times a weight, times sigmoid(W_g h).
 *
 * B200_MLP_DENSE: down(act(gate x) * (up x)).  Routed experts of this form may score with a sigmoid, apply the mixing
 * weight to the expert's INPUT, be ungated (down(act(up x))), and come with one shared expert of the same shape.
 *
 * Third layer form (b200_stack_cfg.form = B200_FORM_POSTNORM): the norm follows the sum,
 *   x = LN(residual_alpha * x + mixer(x)),   x = LN'(residual_alpha * x + ff(x))      (the second line only with a feed-forward),
 * LN a layer norm with weight and bias; both sublayers read the stream itself.  The output is LN_final(x) times the head.
 * Mixers of this form: B200_MIXER_ATTENTION with B200_MIXF_HEAD_NORM (q and k RMS-normalised per head with one weight of
 * `dim` entries), B200_MIXF_VALUE_IS_KEY (no value projection: the value of a token is its key projection before norm and
 * rotation, leading vdim entries) and B200_MIXF_SINK_ONE (one more unit in the softmax denominator);  B200_MIXER_LATENT
 * with q_rank > 0 (queries through a normed latent of their own: q = W_uq rms(W_dq h)), B200_MIXF_HEAD_GATE (one sigmoid
 * gate per head) and kv_share (the layer caches nothing and reads another layer's latent rows);  any attention mixer with
 * `window` > 0 sees only the last `window` positions, its own included;  and
 *
 * B200_MIXER_DELTA: delta-rule recurrence with one decay per head and key channel.  q, k (kv_heads x dim) and v (heads x vdim)
 * pass a causal per-channel convolution of `conv_taps` taps and silu; q and k become unit vectors per head (q times
 * dim^-1/2); beta = sigmoid(w_b . h) per head; decay = exp(-exp(a_log[head]) softplus(W_a2 (W_a1 h) + dt_bias)) per head and
 * key channel; per head  S = diag(decay) S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q;  o is brought to unit RMS per
 * head, times a weight, times sigmoid(W_g2 (W_g1 h)).  S (fp32) and the last conv_taps - 1 inputs of the convolution live
 * in the sequence's state slot.
 *
 * Fourth layer form (b200_stack_cfg.form = B200_FORM_HYPER): pre-norm sublayers over `streams` fp32 copies X_1..X_n of the
 * residual, all equal to the scaled embedding at the start.  Sublayer q of a layer has coefficients a_q [n], b_q [n], M_q [n][n]:
 *   u = sum_s a_q[s] X_s;   h = LN(u) * w + bias;   h += conv(h)   (causal per-channel convolution over canon_taps steps, its
 *   last canon_taps - 1 inputs in the state slot, for BOTH sublayers);   y = scale_q * sublayer(h)   (scale_q [width]);
 *   X_t = sum_s M_q[s][t] X_s + residual_mult * b_q[t] * y   for every t at once.
 * The output is LN_final(sum_s X_s) times the head.  Mixers of this form: B200_MIXER_ATTENTION with B200_MIXF_NO_QK_NORM (plain
 * q/k/v projections), B200_MIXF_ROT_HALF (dimension i of the rotated part turns with dimension i + rot_dims / 2) and
 * B200_MIXF_SINK (exp(sink[head]) in the softmax denominator);  B200_MIXER_DELTA with B200_MIXF_HEAD_DECAY: one decay per head,
 * g = exp(-exp(a_log[head]) softplus(w_a . h + dt_bias[head])), single-step projections, fused rows q | k | v | gate | b | a,
 * read-out times a weight shared by the heads ([vdim] repeated) and silu(gate);  and
 *
 * B200_MIXER_SSD: state-space recurrence with a scalar decay per head.  The fused projection is z | x | B | C | dt
 * (heads*vdim, heads*vdim, kv_heads*dim, kv_heads*dim, heads; kv_heads = groups of heads that share B and C, dim = state size);
 * x | B | C pass a causal per-channel convolution of conv_taps taps with bias and silu; dt = softplus(dt + dt_bias);
 * per head  S = exp(-exp(a_log) dt) S + dt B x^T  (S [dim][vdim], fp32, in the state slot);  y = S^T C + D x;  y *= silu(z);
 * y is brought to unit RMS in `norm_groups` equal parts and multiplied by a weight.
 *
 * Feed-forwards of this form: B200_MLP_DENSE with `ungated` and B200_ACT_POLYNORM: down(p(up h)), p(z) = c0 N(z) + c1 N(z^2) +
 * c2 N(z^3) + c3 with N(v) = v / sqrt(mean(v^2) + eps) over the ff entries of a token;  B200_MLP_MOE with route_chosen: the
 * router bias joins the logits, the `top` largest logits are chosen and the mixing weights are the softmax over the chosen logits
 * alone; experts with B200_ACT_SWIGLU_CLAMP: g = min(gate h, act_limit), u = clamp(up h, -act_limit, act_limit),
 * down(g * sigmoid(1.702 g) * (u + 1)). */
typedef enum b200_mixer_kind { B200_MIXER_ATTENTION = 1, B200_MIXER_LATENT = 2, B200_MIXER_MLSTM = 3, B200_MIXER_DELTA = 4, B200_MIXER_SSD = 5 } b200_mixer_kind;
typedef enum b200_mlp_kind { B200_MLP_NONE = 0, B200_MLP_MOE = 1, B200_MLP_DENSE = 2 } b200_mlp_kind;
typedef enum b200_act_kind { B200_ACT_SILU = 0, B200_ACT_GELU_TANH = 1, B200_ACT_RELU2 = 2, B200_ACT_RELU = 3, B200_ACT_SWIGLU_CLAMP = 4,
                             B200_ACT_POLYNORM = 5 } b200_act_kind;
typedef enum b200_stack_form { B200_FORM_SANDWICH = 0, B200_FORM_PARALLEL = 1, B200_FORM_POSTNORM = 2, B200_FORM_HYPER = 3 } b200_stack_form;
enum { B200_MIXF_SINK = 1, B200_MIXF_GATE = 2, B200_MIXF_HEAD_NORM = 4, B200_MIXF_VALUE_IS_KEY = 8, B200_MIXF_SINK_ONE = 16,
       B200_MIXF_HEAD_GATE = 32, B200_MIXF_ROT_HALF = 64, B200_MIXF_NO_QK_NORM = 128, B200_MIXF_HEAD_DECAY = 256 };
enum { B200_MAX_STREAMS = 8 };

typedef struct b200_stack_layer {
  int32_t mixer;                       /* b200_mixer_kind */
  int32_t heads, kv_heads, dim, vdim;  /* query heads, key/value heads, q/k head size, value head size */
  int32_t rot_dims;                    /* rotated leading dimensions of each q/k head (even; 0: none) */
  int32_t rot_table, vrot_table;       /* table indices (b200_stack_set_rot_table); -1: no rotation */
  float scale;                         /* score scale */
  int32_t mlp;                         /* b200_mlp_kind */
  int32_t experts, top, groups, keep, ff;
  /* everything below: 0 = the first form's behaviour */
  int32_t kv_rank, rot_dim;            /* latent mixer: latent size; rotated part of a query head and of the shared key
                                          (rot_dims <= rot_dim of them turn) */
  int32_t mixer_flags;                 /* B200_MIXF_* */
  float gate_cap;                      /* mLSTM */
  int32_t act;                         /* b200_act_kind of the feed-forward */
  int32_t ungated;                     /* experts without a gate projection */
  int32_t sigmoid_scores;              /* router scores are sigmoids of the logits (no softmax) */
  int32_t weight_input;                /* the mixing weight multiplies the expert's input instead of its output */
  int32_t shared_ff;                   /* intermediate size of the shared expert (0: none) */
  int32_t window;                      /* attention mixers: positions a query sees, its own included (0: all) */
  int32_t q_rank;                      /* latent mixer: size of the query latent (0: queries straight from the fused projection) */
  int32_t kv_share;                    /* latent mixer: 1 + the layer whose cached latent rows this layer reads (0: its own) */
  int32_t conv_taps;                   /* delta mixer: taps of the q/k/v convolution (>= 1) */
  int32_t decay_rank, gate_rank;       /* delta mixer: inner sizes of the two-step decay and output-gate projections */
  int32_t norm_groups;                 /* state-space mixer: equal parts of the gated output that are normalised on their own (>= 1) */
  float act_limit;                     /* B200_ACT_SWIGLU_CLAMP: the clamp */
  int32_t route_chosen;                /* router: bias inside the logits, mixing weights = softmax over the chosen logits */
} b200_stack_layer;

typedef struct b200_stack_cfg {
  int32_t width, vocab, n_layers;
  float embed_scale;                   /* x = table[id] * embed_scale */
  float norm_eps;
  int32_t f32;                         /* 0: bf16 activations, cache and matrix products (fp32 accumulation; residual stream,
                                          norms, rotations, scores, softmax and routers in fp32); 1: everything in true fp32 */
  int32_t block_size, max_tokens, max_blocks_per_seq, max_logit_rows;
  /* everything below: 0 = the first form's behaviour */
  int32_t form;                        /* b200_stack_form */
  int32_t canon_taps;                  /* taps of the input convolution of every mixer (0: none) */
  int32_t depth_avg;                   /* 1: weighted sum over all earlier layer results after every layer */
  int32_t bigram_buckets, bigram_mul_prev, bigram_mul_cur;   /* buckets > 0: hashed bigram rows are added to the embedding */
  float logit_softcap;                 /* > 0: logits = cap * tanh(logits / cap) */
  int32_t n_state_slots;               /* per-sequence state slots (previous token, convolution tails, recurrent state) */
  float residual_alpha;                /* post-norm form: the stream's factor inside the norm */
  int32_t streams;                     /* multi-stream form: copies of the residual (1 .. B200_MAX_STREAMS) */
  float residual_mult;                 /* multi-stream form: factor of every sublayer's result */
} b200_stack_cfg;

typedef enum b200_stack_weight {
  B200_SW_EMBED = 0,        /* bf16 [vocab][width] */
  B200_SW_FINAL_NORM = 1,   /* f32  [width]   (parallel form: [1]) */
  B200_SW_HEAD = 2,         /* bf16 [vocab][width] */
  B200_SW_NORM_MIX_PRE = 3, /* f32  [width]  the four layer norms of a layer (parallel form: PRE kinds only, [1] each) */
  B200_SW_NORM_MIX_POST = 4,
  B200_SW_NORM_MLP_PRE = 5,
  B200_SW_NORM_MLP_POST = 6,
  B200_SW_QKV = 7,          /* bf16, fused projection of the mixer's input.  attention: [heads*dim + kv_heads*dim + kv_heads*vdim][width]
                               (q, k, v rows); latent: [heads*(dim+rot_dim) + kv_rank + rot_dim (+ heads*vdim gate rows)][width];
                               mLSTM: [2*heads*dim + 2*heads*vdim][width] (q, k, v, output-gate rows) */
  B200_SW_Q_NORM = 8,       /* f32  [heads*dim] */
  B200_SW_K_NORM = 9,       /* f32  [kv_heads*dim]   (latent: [kv_rank], the latent's norm weight) */
  B200_SW_O = 10,           /* bf16 [width][heads*vdim] */
  B200_SW_ROUTER = 11,      /* bf16 [experts][width] */
  B200_SW_ROUTER_BIAS = 12, /* f32  [experts]  added to the scores for the choice only (may stay unset: zeros) */
  B200_SW_EXPERT_GATE_UP = 13, /* bf16 [experts][2*ff][width]: per expert the gate rows, then the up rows (ungated: [experts][ff][width]) */
  B200_SW_EXPERT_DOWN = 14, /* bf16 [experts][width][ff] */
  B200_SW_BIGRAM = 15,      /* bf16 [bigram_buckets + 1][width]; the last row serves a sequence's first token */
  B200_SW_CANON = 16,       /* f32  [width][canon_taps] */
  B200_SW_DEPTH_AVG = 17,   /* f32  [layer + 2] */
  B200_SW_UK_T = 18,        /* bf16 [heads][kv_rank][dim]: per head the TRANSPOSE of its key expansion */
  B200_SW_UV = 19,          /* bf16 [heads][vdim][kv_rank] */
  B200_SW_SINK = 20,        /* f32  [heads] */
  B200_SW_GATES = 21,       /* bf16 [2*heads][width]: mLSTM input-gate rows, then forget-gate rows */
  B200_SW_GATES_BIAS = 22,  /* f32  [2*heads] */
  B200_SW_HEAD_NORM = 23,   /* f32  [heads*vdim] */
  B200_SW_MLP_GATE_UP = 24, /* bf16 [2*ff][width]: gate rows, then up rows */
  B200_SW_MLP_DOWN = 25,    /* bf16 [width][ff] */
  B200_SW_SHARED_UP = 26,   /* bf16 [shared_ff][width] */
  B200_SW_SHARED_DOWN = 27, /* bf16 [width][shared_ff] */
  /* post-norm form: NORM_MIX_POST / NORM_MLP_POST / FINAL_NORM are the weights [width] of the norms after the two sums and of
     the output; their biases follow.  QKV is the fused projection of the stream: attention (values = keys) [heads*dim +
     kv_heads*dim][width]; latent [q_rank + (kv_rank unless shared) + heads][width] (query latent, key/value latent, gate rows);
     delta: q | k | v | a1 | g1 | b rows, each of the last three groups starting at a multiple of 8 rows (zero rows between),
     the total a multiple of 8 (b200_delta_fused_rows).  Q_NORM / K_NORM of a head-norm attention are [dim]. */
  B200_SW_NORM_MIX_POST_BIAS = 28, /* f32 [width] */
  B200_SW_NORM_MLP_POST_BIAS = 29, /* f32 [width] */
  B200_SW_FINAL_NORM_BIAS = 30,    /* f32 [width] */
  B200_SW_Q_LATENT_NORM = 31,      /* f32 [q_rank] */
  B200_SW_UQ = 32,                 /* bf16 [heads*dim][q_rank] */
  B200_SW_CONV = 33,               /* f32  [2*kv_heads*dim + heads*vdim][conv_taps]: q, k, v channels; the last tap is the current token's */
  B200_SW_DECAY_UP = 34,           /* bf16 [heads*dim][decay_rank] */
  B200_SW_DECAY_BIAS = 35,         /* f32  [heads*dim] */
  B200_SW_DECAY_LOG = 36,          /* f32  [heads] */
  B200_SW_GATE_UP = 37,            /* bf16 [heads*vdim][gate_rank] */
  B200_SW_MLP_GATE_UP_INTERLEAVED = 38, /* bf16 [2*ff][width] in 128-row slabs: 64 gate rows, then the 64 matching up rows; this OR
                                          B200_SW_MLP_GATE_UP.  bf16 mode, ff % 64 == 0, width % 8 == 0: the gate activation and the
                                          product run in the linear's epilogue */
  /* multi-stream form: NORM_MIX_PRE / NORM_MLP_PRE / FINAL_NORM are the weights [width] of the pre-norms and of the output norm,
     their biases follow (FINAL_NORM_BIAS above); CANON is the mixer's input convolution.  QKV: attention q | k | v rows; delta
     q | k | v | gate | b | a rows; state-space z | x | B | C | dt rows.  CONV of a state-space mixer: [heads*vdim + 2*kv_heads*dim]
     [conv_taps]; DECAY_BIAS of a head-decay delta or state-space mixer: [heads]; HEAD_NORM of a state-space mixer: [heads*vdim].
     MLP_GATE_UP of an ungated dense feed-forward: [ff][width]. */
  B200_SW_NORM_MIX_PRE_BIAS = 39,  /* f32 [width] */
  B200_SW_NORM_MLP_PRE_BIAS = 40,  /* f32 [width] */
  B200_SW_SCALE_MIX = 41,          /* f32 [width]: per-channel factor of the mixer's result */
  B200_SW_SCALE_MLP = 42,          /* f32 [width] */
  B200_SW_HC_MIX = 43,             /* f32 [2 n + n n]: a [n] | b [n] | M [n][n] (from, to) of the mixer sublayer, n = streams */
  B200_SW_HC_MLP = 44,             /* f32 [2 n + n n] */
  B200_SW_CANON_MLP = 45,          /* f32 [width][canon_taps]: input convolution of the feed-forward */
  B200_SW_CONV_BIAS = 46,          /* f32 [conv channels] */
  B200_SW_SKIP = 47,               /* f32 [heads]: D of a state-space mixer */
  B200_SW_MLP_ACT = 48             /* f32 [4]: c0..c3 of B200_ACT_POLYNORM */
} b200_stack_weight;

B200_API int b200_stack_create(const b200_stack_cfg* cfg, const b200_stack_layer* layers, b200_ctx** out);
/* Pointers are borrowed for the life of the ctx; rows/cols are checked ([rows][cols], vectors as [n][1]). */
B200_API int b200_stack_set_weight(b200_ctx* ctx, int32_t layer, int32_t kind, const void* w, int64_t rows, int64_t cols);
/* Row widths of one layer's cache: dim and vdim, or 128 for both where the layer runs on the attention kernels built for
 * 128-wide heads (bf16, blocks of 128 tokens, dim and vdim in [64, 128]); the tail of such rows is kept at zero. */
B200_API int b200_stack_cache_dims(b200_ctx* ctx, int32_t layer, int32_t* k_dim, int32_t* v_dim);
/* Paged cache of one layer, caller-owned: k [n_blocks][kv_heads][block_size][k_dim], v [...][v_dim] (b200_stack_cache_dims);
 * bf16, or fp32 when the ctx was created with f32.  Every layer gets the same n_blocks (one block table serves all layers). */
B200_API int b200_stack_set_kv_cache(b200_ctx* ctx, int32_t layer, void* k_cache, void* v_cache, int64_t n_blocks);
/* cos|sin table `index` (0..15): fp32 [n_pos][2][half] (the cos row of a position, then its sin row). */
B200_API int b200_stack_set_rot_table(b200_ctx* ctx, int32_t index, const float* table, int64_t n_pos, int32_t half);
/* After every layer of a step, the residual stream is copied to out[layer][n_tokens][width] fp32 (NULL: off; turns graph
 * replay off while set).  Parity tests. */
B200_API int b200_stack_set_stream_tap(b200_ctx* ctx, float* out);
/* Per-sequence state (models with n_state_slots > 0): caller-owned, n_state_slots * b200_stack_state_bytes(ctx) bytes, any
 * content (a sequence whose first row of a step is at position 0 starts from zeros).  A step names the slot of each of its
 * sequences: the host-buffer step reads seq_slots[n_seqs] behind the block tables of its packed buffer; device-pointer
 * steps use the array given here (device memory, n_seqs entries, read at every following step until replaced). */
B200_API int64_t b200_stack_state_bytes(b200_ctx* ctx);
B200_API int b200_stack_set_state(b200_ctx* ctx, void* state);
B200_API int b200_stack_set_step_slots(b200_ctx* ctx, const int32_t* seq_slots, int32_t n_seqs);
/* Rows of the delta mixer's fused projection and where its groups start: offsets[0..5] = q, k, v, a1, g1, b. */
B200_API int32_t b200_delta_fused_rows(int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t decay_rank, int32_t gate_rank,
                                       int32_t* offsets);
/* The logit rows of the LAST step as fp32 [n_rows][vocab] into host memory (asynchronously: synchronise the stream before
 * reading).  With f32 they are the unrounded logits; otherwise the bf16 logits widened.  Works for every ctx on one GPU. */
B200_API int b200_ctx_logits_last_f32(b200_ctx* ctx, int32_t n_rows, float* host_out, void* stream);

/* Per-kernel entry points of the mechanisms above (unit tests, profiling).  f32 selects the element type of activations
 * and caches (0: bf16, 1: fp32); vectors of norm weights, tables, queries and partial rows are always fp32. */
/* x (fp32 stream [T][width]) += LN(y) * w_post, where y is an activation row [T][width] or, when y is NULL, the sum over
 * n_parts fp32 partial rows yparts[T][n_parts][width] (both NULL: x is left alone); then, when w_next is given,
 * out[t] = LN(x[rows ? rows[t] : t]) * w_next.  LN: (v - mean) / sqrt(mean((v - mean)^2) + eps). */
B200_API int b200_layernorm_stream(int32_t f32, float* x, const void* y, const float* yparts, int32_t n_parts, const float* w_post,
                          const float* w_next, void* out, const int32_t* rows, int32_t n_tokens, int32_t width, float eps,
                          void* stream);
/* qkv [T][heads*dim + kv_heads*dim + kv_heads*vdim] -> q_out fp32 [T][heads*dim]; k, v into the paged caches at
 * slot_mapping[t].  rot / vrot: cos|sin tables [max_pos][2][rot_dims/2] / [max_pos][2][vdim/2] (NULL: no rotation). */
B200_API int b200_qk_norm_rotate_cache(int32_t f32, const void* qkv, const float* q_norm_w, const float* k_norm_w,
                              const int32_t* positions, const int32_t* slot_mapping, const float* rot, int32_t rot_dims,
                              const float* vrot, float* q_out, void* k_cache, void* v_cache, int32_t n_tokens, int32_t heads,
                              int32_t kv_heads, int32_t dim, int32_t vdim, int32_t block_size, float eps, int64_t max_pos,
                              void* stream);
/* The same over bf16 rows for attention kernels built for wider heads: bf16 queries [T][heads][k_row], cache rows of k_row /
 * v_row elements; the tail beyond dim / vdim is written as zero. */
B200_API int b200_qk_norm_rotate_cache_wide(const void* qkv, const float* q_norm_w, const float* k_norm_w, const int32_t* positions,
                                            const int32_t* slots, const float* rot, int32_t rot_dims, const float* vrot, void* q_out,
                                            void* k_cache, void* v_cache, int32_t n_tokens, int32_t heads, int32_t kv_heads, int32_t dim,
                                            int32_t vdim, int32_t block_size, float eps, int64_t max_pos, int32_t k_row, int32_t v_row,
                                            void* stream);
/* bf16 attention output rows [T][heads][in_row] -> [T][heads][vdim], each pair (2m, 2m+1) turned back by the row's position
 * (vrot: the value table, or null for packing alone).  in == out only when in_row == vdim. */
B200_API int b200_rotate_back_rows(const void* in, int32_t in_row, void* out, const int32_t* positions, const float* vrot,
                                   int32_t n_tokens, int32_t heads, int32_t vdim, int64_t max_pos, void* stream);
/* Causal paged attention of fp32 queries [T][heads*dim] over caches [block][kv_heads][block_size][dim | vdim]; out
 * [T][heads*vdim].  vrot != NULL: the output of row t is rotated by -positions[t].  shared_tiles 0: one CTA per (row, head);
 * 1: runs of consecutive rows of a sequence share K/V tiles (workspace: b200_paged_attn_anydim_workspace_bytes(T)). */
B200_API int64_t b200_paged_attn_anydim_workspace_bytes(int32_t n_tokens);
B200_API int b200_paged_attn_anydim(int32_t f32, const float* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                           int32_t bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions,
                           const float* vrot, int64_t max_pos, void* out, int32_t n_tokens, int32_t heads, int32_t kv_heads,
                           int32_t dim, int32_t vdim, int32_t block_size, float scale, int32_t shared_tiles, void* workspace,
                           void* stream);
/* ---- per-kernel entry points of the parallel form (unit tests, profiling); f32 as above ---- */
/* seq_start[s] = first row of sequence s of the step, seq_start[n_seqs] = n_tokens (row_to_seq NULL: every row its own). */
B200_API int b200_seq_bounds(const int32_t* row_to_seq, int32_t n_tokens, int32_t n_seqs, int32_t* seq_start, void* stream);
/* out[t] = table[id] * scale + bigram[(prev * mul_prev + id * mul_cur) mod buckets] (row `buckets` at position 0); prev is the
 * row before in the same sequence or state_prev[slot * slot_stride_ints]; with state_prev the last id of every sequence is
 * stored there afterwards. */
B200_API int b200_embed_bigram(const int32_t* ids, const void* table, const void* bigram, float* out, int32_t n_tokens, int32_t width,
                               int32_t vocab, float scale, const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start,
                               const int32_t* seq_slots, int32_t n_seqs, int32_t* state_prev, int64_t slot_stride_ints, int32_t buckets,
                               int32_t mul_prev, int32_t mul_cur, void* stream);
/* The closing pass of a layer over fp32 rows u [T][width]: with y_mix, X = u + (y_mix + y_ff + sum of n_parts fp32 partial rows +
 * y_sh) (each optional but y_mix); `results` [n_results][result_stride] receives X (or u) as entry n_results - 1; with dwa,
 * u = sum_j dwa[j] results[j], else u = X; with g1, h1 = u / rms(u) * g1[0] (fp32 and / or activation type) and h2 likewise. */
B200_API int b200_parallel_close(int32_t f32, float* u, const void* y_mix, const void* y_ff, const float* parts, int32_t n_parts,
                                 const void* y_sh, float* results, int64_t result_stride, int32_t n_results, const float* dwa,
                                 const float* g1, const float* g2, float* h1_f32, void* h1_act, void* h2, int32_t n_tokens, int32_t width,
                                 float eps, void* stream);
/* out[t] = h[t] + sum_j w[:, j] h[t - taps + 1 + j] along each sequence; tails [slot][taps - 1][width] (slot_stride floats apart)
 * hold the inputs before the step's portion and receive its last taps - 1 inputs. */
B200_API int b200_canon_conv(int32_t f32, const float* h, const float* w, void* out, int32_t n_tokens, int32_t width, int32_t taps,
                             const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots,
                             float* tails, int64_t slot_stride, void* stream);
/* Fused projection rows [heads*(dim+rot_dim) | kv_rank | rot_dim | ...] -> cache row [normed latent | rotated key part] at
 * slot_mapping[t], rotated query parts into qfull[t][h][kv_rank ..] (rows of kv_rank + rot_dim fp32). */
B200_API int b200_latent_prep(int32_t f32, const void* qkv, int64_t ld, const float* norm_w, const int32_t* positions,
                              const int32_t* slot_mapping, const float* rot, int32_t rot_dims, int64_t max_pos, float* qfull, void* cache,
                              int32_t n_tokens, int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, float eps, void* stream);
/* y[t][h][:n_out] = W[h] x[t][h][:k] for every head; element (t, h, i) of x at x[t * ldx + h * x_hs + i], likewise y and gate
 * (gate != NULL: y *= sigmoid(gate)).  W bf16 [heads][n_out][k]; y fp32 when y_f32. */
B200_API int b200_head_linear(int32_t f32, int32_t y_f32, const void* x, int64_t ldx, int32_t x_hs, const void* w, void* y, int64_t ldy,
                              int32_t y_hs, const void* gate, int64_t ldg, int32_t g_hs, int32_t n_tokens, int32_t heads, int32_t n_out,
                              int32_t k, void* stream);
/* b200_paged_attn_anydim with cache rows of k_row / v_row elements (0: dim / vdim; the value cache may be the key cache) and
 * an optional per-head sink term in the softmax denominator. */
B200_API int b200_paged_attn_anydim_ex(int32_t f32, const float* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                                       int32_t bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions,
                                       void* out, int32_t n_tokens, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                                       int32_t block_size, float scale, int32_t shared_tiles, void* workspace, int32_t k_row, int32_t v_row,
                                       const float* sink, void* stream);
/* The same attention over bf16 latent cache rows [block][block_size][k_row] on the tensor cores: one kv head, the value of a key
 * is the row's leading `rank` entries, fp32 queries [T][heads][k_row], bf16 output [T][heads][rank].  k_row and rank multiples
 * of 16, rank <= 512 (b200_latent_attn_supported).  workspace: b200_paged_attn_anydim_workspace_bytes(T).  n_splits > 1 with
 * part (n_tokens * heads * n_splits * (rank + 2) floats): the context is walked by n_splits CTAs per group of pairs and merged. */
B200_API int b200_latent_attn_supported(int32_t heads, int32_t k_row, int32_t rank);
B200_API int b200_latent_attn(const float* q, const void* cache, const int32_t* block_table, int32_t bt_stride, const int32_t* row_to_seq,
                              const int32_t* ctx_lens, void* out, int32_t n_tokens, int32_t heads, int32_t k_row, int32_t rank,
                              int32_t block_size, float scale, const float* sink, void* workspace, int32_t n_splits, float* part,
                              void* stream);
/* mLSTM: log gates [T][2 heads] (input gates, then forget gates) from w [2 heads][width] and bias; the recurrence over
 * fused rows (q at q_off, k at k_off, v at v_off) with the state of each sequence at state + slot * slot_stride floats
 * (b200_mlstm_state_floats per layer), out fp32 [T][heads*vdim]; then unit RMS per head, weight and sigmoid gate. */
B200_API int b200_mlstm_gates(int32_t f32, const void* x, const void* w, const float* bias, float* out, int32_t n_tokens, int32_t width,
                              int32_t heads, float cap, void* stream);
B200_API int64_t b200_mlstm_state_floats(int32_t heads, int32_t dim, int32_t vdim);
B200_API int b200_mlstm_scan(int32_t f32, const void* qkv, int64_t ld, int32_t q_off, int32_t k_off, int32_t v_off, const float* gates,
                             const int32_t* positions, const int32_t* seq_start, const int32_t* seq_slots, float* state,
                             int64_t slot_stride, float* out, int32_t n_seqs, int32_t heads, int32_t dim, int32_t vdim, void* stream);
B200_API int b200_head_norm_gate(int32_t f32, const float* o, const float* w, const void* gate, int64_t ldg, void* out, int32_t n_tokens,
                                 int32_t heads, int32_t vdim, float eps, void* stream);
/* gated: out[t][f] = act(in[t][f]) * in[t][ff + f] over rows of 2 ff; else out = act(in) (in place allowed). */
B200_API int b200_ff_act(int32_t f32, const void* in, void* out, int32_t n_tokens, int32_t ff, int32_t gated, int32_t act, void* stream);
/* Router without groups or bias; sigmoid_scores: scores are sigmoids of the logits instead of a softmax over the experts. */
B200_API int b200_moe_route_scores(int32_t f32, const void* x, const void* w_router, int32_t n_tokens, int32_t width, int32_t experts,
                                   int32_t top, int32_t sigmoid_scores, int32_t* out_ids, float* out_w, void* stream);
/* b200_moe_experts for the other expert shapes: gated 0 = down(act(up x)) over w_up [experts][ff][width]; weight_input: the
 * mixing weight scales the input row. */
B200_API int b200_moe_experts_form(int32_t f32, const void* x, const void* w_up, const void* w_down, const int32_t* ids, const float* wts,
                                   int32_t n_tokens, int32_t width, int32_t ff, int32_t experts, int32_t top, float* parts, void* ws,
                                   int32_t gated, int32_t act, int32_t weight_input, void* stream);
/* Router: out_ids / out_weights [T][top].  bias may be NULL. */
B200_API int b200_moe_route(int32_t f32, const void* x, const void* w_router, const float* bias, int32_t n_tokens, int32_t width,
                   int32_t experts, int32_t top, int32_t groups, int32_t keep, int32_t* out_ids, float* out_weights, void* stream);
/* The same router over bf16 rows with the logits from the tcgen05 linear: logits [n_tokens][experts] fp32 is written too. */
B200_API int b200_moe_route_linear(const void* x, const void* w_router, const float* bias, int32_t n_tokens, int32_t width,
                                   int32_t experts, int32_t top, int32_t groups, int32_t keep, int32_t* out_ids, float* out_w,
                                   float* logits, void* stream);
/* Chosen experts: parts [T][top][width] fp32, each row already times its weight.  workspace: b200_moe_workspace_bytes
   (width and ff > 0: room for the tensor-core form, which bf16 activations with width and ff multiples of 8 take). */
B200_API int64_t b200_moe_workspace_bytes(int32_t n_tokens, int32_t top, int32_t experts, int32_t width, int32_t ff);
B200_API int b200_moe_experts(int32_t f32, const void* x, const void* w_gate_up, const void* w_down, const int32_t* ids,
                     const float* weights, int32_t n_tokens, int32_t width, int32_t ff, int32_t experts, int32_t top, float* parts,
                     void* workspace, void* stream);
/* ---- per-kernel entry points of the post-norm form (unit tests, profiling); f32 as above ---- */
/* x[r] = LN(alpha * x_in[rows ? rows[r] : r] + y[r]) * w + b over fp32 rows (y optional, of the activation type); x_out fp32
 * and / or out_act (activation type) receive the result; x_out may be x_in when rows is NULL. */
B200_API int b200_postnorm_stream(int32_t f32, const float* x_in, const void* y, float alpha, const float* w, const float* b, float* x_out,
                                  void* out_act, const int32_t* rows, int32_t n_rows, int32_t width, float eps, void* stream);
/* Fused rows [heads*dim q | kv_heads*dim k] of leading dimension ld: values = the raw key rows' leading vdim entries into v_cache;
 * q and k RMS-normalised per head with qw / kw [dim], the leading rot_dims dimensions turned in neighbouring pairs by
 * table rot [max_pos][2][rot_dims/2]; q_out fp32 [T][heads*dim], k into k_cache; caches [block][kv_heads][block_size][dim | vdim]. */
B200_API int b200_qk_headnorm_rotate_cache(int32_t f32, const void* qk, int64_t ld, const float* qw, const float* kw, const int32_t* positions,
                                           const int32_t* slot_mapping, const float* rot, int32_t rot_dims, int64_t max_pos, float* q_out,
                                           void* k_cache, void* v_cache, int32_t n_tokens, int32_t heads, int32_t kv_heads, int32_t dim,
                                           int32_t vdim, int32_t block_size, float eps, void* stream);
/* b200_paged_attn_anydim_ex with a window: row t sees the last `window` keys of its context only (0: all). */
B200_API int b200_paged_attn_window(int32_t f32, const float* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                                    int32_t bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions,
                                    void* out, int32_t n_tokens, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                                    int32_t block_size, float scale, int32_t shared_tiles, void* workspace, int32_t k_row, int32_t v_row,
                                    const float* sink, int32_t window, void* stream);
/* b200_latent_attn with a window (n_splits 1). */
B200_API int b200_latent_attn_window(const float* q, const void* cache, const int32_t* block_table, int32_t bt_stride,
                                     const int32_t* row_to_seq, const int32_t* ctx_lens, void* out, int32_t n_tokens, int32_t heads,
                                     int32_t k_row, int32_t rank, int32_t block_size, float scale, const float* sink, void* workspace,
                                     int32_t window, void* stream);
/* Grouped-query attention over bf16 key and value caches [block][kv_heads][block_size][dim | vdim] on the tensor cores (dim and
 * vdim multiples of 16, vdim <= 512: b200_paged_attn_mma_supported): fp32 queries [T][heads][dim], bf16 output [T][heads][vdim],
 * optional sink [heads] and window; n_splits > 1 with part (n_tokens * heads * n_splits * (vdim + 2) floats) splits the context. */
B200_API int b200_paged_attn_mma_supported(int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim);
B200_API int b200_paged_attn_mma(const float* q, const void* k_cache, const void* v_cache, const int32_t* block_table, int32_t bt_stride,
                                 const int32_t* row_to_seq, const int32_t* ctx_lens, void* out, int32_t n_tokens, int32_t heads,
                                 int32_t kv_heads, int32_t dim, int32_t vdim, int32_t block_size, float scale, const float* sink,
                                 void* workspace, int32_t window, int32_t n_splits, float* part, void* stream);
/* Fused rows [q_rank | kv_rank ...] of leading dimension ld: cq[t] = rms(row[:q_rank]) * qw (activation type, rows of q_rank);
 * cache row at slot_mapping[t] = rms(row[q_rank : q_rank + kv_rank]) * kw (skipped when cache is NULL). */
B200_API int b200_latent_norms(int32_t f32, const void* fused, int64_t ld, int32_t q_rank, int32_t kv_rank, const float* qw, const float* kw,
                               const int32_t* slot_mapping, void* cq, void* cache, int32_t n_tokens, float eps, void* stream);
/* b200_head_linear whose gate is one number per head (gate[t * ldg + h]). */
B200_API int b200_head_linear_head_gate(int32_t f32, const void* x, int64_t ldx, int32_t x_hs, const void* w, void* y, int64_t ldy,
                                        int32_t y_hs, const void* gate, int64_t ldg, int32_t n_tokens, int32_t heads, int32_t n_out,
                                        int32_t k, void* stream);
/* Delta mixer, after the projections.  fused [T][ld] (groups at the offsets of b200_delta_fused_rows), a2 [T][heads*dim] =
 * W_a2 a1 (activation type).  prep: convolution (tails [slot][taps-1][C] fp32, slot_stride floats apart; a portion that
 * starts at position 0 sees zeros) + silu, unit q (times dim^-1/2) and k, beta, decay -> fp32 qn, kn [T][kv_heads*dim],
 * vn [T][heads*vdim], beta [T][heads], decay [T][heads*dim].  tails: the last taps-1 raw q|k|v rows of every sequence go into
 * its slot (after prep).  scan: the recurrence over state [slot][heads][vdim][dim] fp32, out fp32 [T][heads*vdim]. */
B200_API int b200_delta_prep(int32_t f32, const void* fused, int64_t ld, const void* a2, const float* conv_w, const float* dt_bias,
                             const float* a_log, const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start,
                             const int32_t* seq_slots, const float* tails, int64_t slot_stride, float* qn, float* kn, float* vn,
                             float* beta, float* decay, int32_t n_tokens, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                             int32_t taps, int32_t decay_rank, int32_t gate_rank, void* stream);
B200_API int b200_delta_tails(int32_t f32, const void* fused, int64_t ld, const int32_t* positions, const int32_t* seq_start,
                              const int32_t* seq_slots, float* tails, int64_t slot_stride, int32_t n_seqs, int32_t channels, int32_t taps,
                              void* stream);
B200_API int b200_delta_scan(const float* qn, const float* kn, const float* vn, const float* beta, const float* decay,
                             const int32_t* positions, const int32_t* seq_start, const int32_t* seq_slots, float* state,
                             int64_t slot_stride, float* out, int32_t n_seqs, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                             void* stream);
/* ---- per-kernel entry points of the multi-stream form (unit tests, profiling); f32 as above ---- */
/* Streams X [n][stream_stride] fp32 (row t of stream s at X + s * stream_stride + t * width).  init: every stream takes the row of
 * stream 0 first.  With hc_close (a | b | M of the sublayer that ends) X_t = sum_s M[s][t] X_s + mult * b[t] * scale * y, y an
 * activation row or the sum of n_parts fp32 partial rows.  Then u = sum_s open_in[s] X_s (open_in NULL: ones); with norm_w,
 * h = LN(u) * norm_w + norm_b into h_f32 and / or h_act, else u itself; sum_out receives sum_s X_s.  rows: only those rows are
 * read (outputs are dense, the streams are not written). */
B200_API int b200_hyper_step(int32_t f32, float* X, int64_t stream_stride, int32_t n, int32_t init, const void* y, const float* parts,
                             int32_t n_parts, const float* scale, const float* hc_close, float mult, const float* open_in,
                             const float* norm_w, const float* norm_b, float eps, const int32_t* rows, float* h_f32, void* h_act,
                             float* sum_out, int32_t n_rows, int32_t width, void* stream);
/* Fused rows [heads*dim q | kv_heads*dim k | kv_heads*vdim v] of leading dimension ld: the leading rot_dims dimensions of every q
 * and k head turn by table rot [max_pos][2][rot_dims/2], dimension i with i + rot_dims/2 (half_layout) or 2i with 2i + 1; q_out
 * fp32 [T][heads*dim]; k and v rows into the caches [block][kv_heads][block_size][dim | vdim] at slot_mapping[t]. */
B200_API int b200_qkv_rotate_cache(int32_t f32, const void* qkv, int64_t ld, const int32_t* positions, const int32_t* slot_mapping,
                                   const float* rot, int32_t rot_dims, int32_t half_layout, int64_t max_pos, float* q_out, void* k_cache,
                                   void* v_cache, int32_t n_tokens, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                                   int32_t block_size, void* stream);
/* out[t] = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 over rows z [T][ff], N(v) = v / sqrt(mean(v^2) + eps). */
B200_API int b200_polynorm(int32_t f32, const void* z, const float* coef, void* out, int32_t n_tokens, int32_t ff, float eps, void* stream);
/* b200_ff_act with the clamp of B200_ACT_SWIGLU_CLAMP. */
B200_API int b200_ff_act_limit(int32_t f32, const void* in, void* out, int32_t n_tokens, int32_t ff, int32_t gated, int32_t act, float limit,
                               void* stream);
/* Router whose bias joins the logits; the `top` largest are chosen, weights = softmax over the chosen logits. */
B200_API int b200_moe_route_chosen(int32_t f32, const void* x, const void* w_router, const float* bias, int32_t n_tokens, int32_t width,
                                   int32_t experts, int32_t top, int32_t* out_ids, float* out_w, void* stream);
/* b200_moe_experts_form with the clamp of B200_ACT_SWIGLU_CLAMP. */
B200_API int b200_moe_experts_limit(int32_t f32, const void* x, const void* w_up, const void* w_down, const int32_t* ids, const float* wts,
                                    int32_t n_tokens, int32_t width, int32_t ff, int32_t experts, int32_t top, float* parts, void* ws,
                                    int32_t gated, int32_t act, float limit, void* stream);
/* Delta mixer with one decay per head: fused rows q | k | v | gate | b | a (no padding); outputs as b200_delta_prep, decay [T][heads]. */
B200_API int b200_delta_prep_head(int32_t f32, const void* fused, int64_t ld, const float* conv_w, const float* dt_bias, const float* a_log,
                                  const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots,
                                  const float* tails, int64_t slot_stride, float* qn, float* kn, float* vn, float* beta, float* decay,
                                  int32_t n_tokens, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t taps, void* stream);
/* The recurrence S = g S; u = beta (v - S^T k) (delta_rule) or u = beta v (plain); S += k u^T; o = S^T q, with the decay of
 * (row t, head h, key channel d) at decay[t * g_row + h * g_head + d * g_chan]. */
B200_API int b200_linear_scan(int32_t delta_rule, const float* qn, const float* kn, const float* vn, const float* beta, const float* decay,
                              int64_t g_row, int32_t g_head, int32_t g_chan, const int32_t* positions, const int32_t* seq_start,
                              const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int32_t n_seqs, int32_t heads,
                              int32_t kv_heads, int32_t dim, int32_t vdim, void* stream);
/* b200_head_norm_gate whose gate is silu(gate) (gate_silu) instead of sigmoid(gate). */
B200_API int b200_head_norm_gate_act(int32_t f32, const float* o, const float* w, const void* gate, int64_t ldg, void* out, int32_t n_tokens,
                                     int32_t heads, int32_t vdim, float eps, int32_t gate_silu, void* stream);
/* State-space mixer, after the projection.  fused [T][ld] = z | x | B | C | dt.  prep: convolution with bias (tails
 * [slot][taps-1][heads*vdim + 2*groups*state] fp32) + silu -> fp32 xn [T][heads*vdim], bn, cn [T][groups*state]; dt = softplus(dt +
 * dt_bias) and decay = exp(-exp(a_log) dt) [T][heads].  The tails are written by b200_delta_tails over the x | B | C columns, the
 * recurrence is b200_linear_scan (plain) with q = cn, k = bn, v = xn, beta = dt.  gate_norm: y = (o + skip[head] xn) * silu(z), unit
 * RMS in norm_groups equal parts, times w. */
B200_API int b200_ssd_prep(int32_t f32, const void* fused, int64_t ld, const float* conv_w, const float* conv_b, const float* dt_bias,
                           const float* a_log, const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start,
                           const int32_t* seq_slots, const float* tails, int64_t slot_stride, float* xn, float* bn, float* cn, float* dt,
                           float* decay, int32_t n_tokens, int32_t heads, int32_t groups, int32_t state, int32_t vdim, int32_t taps,
                           void* stream);
B200_API int b200_ssd_gate_norm(int32_t f32, const float* o, const float* xn, const float* skip, const void* z, int64_t ldz, const float* w,
                                void* out, int32_t n_tokens, int32_t heads, int32_t vdim, int32_t norm_groups, float eps, void* stream);
/* y[T][n_out] = x[T][k] . w[n_out][k]^T on CUDA cores in true fp32; w bf16, x / y fp32 or bf16. */
B200_API int b200_linear_simt(int32_t x_f32, int32_t y_f32, const void* x, int64_t ldx, const void* w, void* y, int64_t ldy,
                     int32_t n_tokens, int32_t n_out, int32_t k, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_DECODE_H */
