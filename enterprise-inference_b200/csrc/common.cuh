// Shared device/host helpers for the sm_100a decode kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "b200_decode.h"

namespace b200 {

// ---- error plumbing (never throw across the C ABI) --------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define B200_CUDA(expr)                                                        \
  do {                                                                         \
    cudaError_t _e = (expr);                                                   \
    if (_e != cudaSuccess) return ::b200::cuda_fail(_e, #expr, __FILE__, __LINE__); \
  } while (0)

#define B200_REQUIRE(cond, code, ...)          \
  do {                                         \
    if (!(cond)) {                             \
      ::b200::set_error(__VA_ARGS__);          \
      return (code);                           \
    }                                          \
  } while (0)

#define B200_LAUNCH_CHECK() B200_CUDA(cudaGetLastError())

constexpr int kHeadDim = 128;
constexpr int kNumSMs = 148;

// ---- bf16 helpers -----------------------------------------------------------------------
// A bf16 is the top half of an fp32: widening is a shift / mask (exact).
__device__ __forceinline__ float bf16lo(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bf16hi(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Streaming 128-bit load that does not allocate in L1 (weights / KV are read once).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
// Cached 128-bit read-only load (activations re-read by every warp).
__device__ __forceinline__ uint4 ld_ro(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// (a8, R5) bf16(silu(g)) for a bf16-valued g: accurate expf, the division as a correctly rounded reciprocal
// times g (<= 1 fp32 ulp from g / d, i.e. the bf16 result differs once in ~2^15 elements; an IEEE division
// costs three times as much and this sits in the gate_up epilogue).  One definition for the fused epilogue
// and the stand-alone kernel: they stay bit-identical.
__device__ __forceinline__ float silu_to_bf16(float g) { return round_bf16(g * __frcp_rn(1.0f + expf(-g))); }

// Warp max of floats in ONE instruction (redux.sync on an order-preserving integer image of the float)
// instead of five shuffle + max rounds.  -inf maps through unchanged; NaNs do not occur where it is used
// (masked scores are -inf before the reduction).
__device__ __forceinline__ float warp_max_redux(float v) {
  int i = __float_as_int(v);
  i = i >= 0 ? i : (i ^ 0x7fffffff);
  i = __reduce_max_sync(0xffffffffu, i);
  return __int_as_float(i >= 0 ? i : (i ^ 0x7fffffff));
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// activations of the feed-forwards (b200_act_kind), fp32
__device__ __forceinline__ float act_apply(float z, int kind) {
  if (kind == B200_ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  if (kind == B200_ACT_RELU) return fmaxf(z, 0.f);
  if (kind == B200_ACT_RELU2) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  return z / (1.0f + expf(-z));
}
// gate and up value of a gated feed-forward -> the activated product.  B200_ACT_SWIGLU_CLAMP: g = min(g, limit),
// u = clamp(u, -limit, limit), g * sigmoid(1.702 g) * (u + 1)
__device__ __forceinline__ float gate_combine(float g, float u, int kind, float limit) {
  if (kind == B200_ACT_SWIGLU_CLAMP) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
  }
  return act_apply(g, kind) * u;
}

// ---- Programmatic dependent launch -------------------------------------------------------
// Every kernel of the step waits for its predecessor's memory here and lets its successor
// start its prologue early; with no PDL attribute on the launch both are no-ops.
// One lane of a converged warp (elect.sync): the predicate for single-thread instructions (tcgen05.mma, TMA) inside
// warp-uniform code, which keeps their operands in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
// Asks the lines of [p, p + bytes) into L2, the CTA's threads sharing the lines.  For what does not depend on the launch
// before (weights, step inputs, state of the step before) it runs ahead of pdl_wait, while that launch still computes.
__device__ __forceinline__ void prefetch_l2_span(const void* p, size_t bytes) {
  const char* c = static_cast<const char*>(p);
  for (size_t o = (size_t)threadIdx.x * 128; o < bytes; o += (size_t)blockDim.x * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(c + o));
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// ---- launch helper -----------------------------------------------------------------------
struct LaunchOpts {
  bool pdl = false;  // programmatic stream serialization (set by the ctx inside a step)
};
LaunchOpts& launch_opts();
int& launch_counter();

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  int na = 0;
  if (launch_opts().pdl) {
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = at;
  cfg.numAttrs = na;
  ++launch_counter();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same, with a thread-block cluster shape (1,1,1 = no cluster).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                  dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[2];
  int na = 0;
  if (launch_opts().pdl) {
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (cluster.x * cluster.y * cluster.z > 1) {
    at[na].id = cudaLaunchAttributeClusterDimension;
    at[na].val.clusterDim.x = cluster.x;
    at[na].val.clusterDim.y = cluster.y;
    at[na].val.clusterDim.z = cluster.z;
    ++na;
  }
  cfg.attrs = at;
  cfg.numAttrs = na;
  ++launch_counter();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-DEVICE property of a kernel: set it once per (instantiation,
// device) — `done` is a function-local static of the calling launcher — so that a process driving several GPUs works.
template <typename K>
inline cudaError_t ensure_dynamic_smem(K kernel, int bytes, bool (&done)[64]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
  return e;
}

// ---- kernels' host entry points (internal, C++ linkage) ----------------------------------
int linear_gemv(const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, const __nv_bfloat16* bias,
                __nv_bfloat16* y, int64_t ldy, int T, int n_out, int k, cudaStream_t s);
bool linear_tc_supported(int T, int n_out, int k);
int64_t linear_tc_workspace_bytes(int T, int n_out, int k);
// Optional fusions of the tcgen05 linear.  Epilogue modes: 0 plain, 1 silu*mul over an interleaved gate|up slab,
// 2 RoPE + KV append over a fused qkv projection, 3 add into the fp32 residual stream (sres/ssq, no y),
// 4 unrounded fp32 output rows in out_f32 [T][n_out] (no y).
// norm_in: the input rows are not read from x but normalised on the fly from the fp32 residual stream
// (RMSNorm folded into the consumer: sres, ssq, norm_w, eps, optional row indirection `rows`).
struct LinearExtra {
  int mode = 0;
  bool norm_in = false;
  float* sres = nullptr;         // [T][hidden] fp32: x + residual, unrounded
  float* ssq = nullptr;          // [T][hidden/128] fp32: per-slab sums of squares of sres
  const __nv_bfloat16* norm_w = nullptr;
  const int32_t* rows = nullptr;
  float eps = 0.f;
  const int32_t* positions = nullptr;
  const int32_t* slots = nullptr;
  const __nv_bfloat16* cos_sin = nullptr;
  __nv_bfloat16* kc = nullptr;
  __nv_bfloat16* vc = nullptr;
  int hq = 0, hkv = 0, block_size = 0;
  float* out_f32 = nullptr;
  int act = 0;                   // mode 1: b200_act_kind of the gate (0: silu)
};
int linear_tc(const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* w, const __nv_bfloat16* bias,
              __nv_bfloat16* y, int64_t ldy, int T, int n_out, int k, void* ws, int64_t ws_bytes,
              const LinearExtra* ex, cudaStream_t s);
// grouped form (gemm_tc.cu): one launch over the gathered token rows of every expert
int linear_tc_grouped_tile(int pairs, int experts);
int linear_tc_grouped(const __nv_bfloat16* x, int64_t ldx, int N, int n_tiles, const __nv_bfloat16* w, int experts, int n_out, int k,
                      const int32_t* tile_expert, __nv_bfloat16* y, int64_t ldy, const int32_t* row_pair, const float* wts,
                      float* out, cudaStream_t s);
int linear_tc_grouped_gate_up(const __nv_bfloat16* x, int64_t ldx, int N, int n_tiles, const __nv_bfloat16* w, int experts, int ff,
                              int k, const int32_t* tile_expert, __nv_bfloat16* y, cudaStream_t s, int act = 0, float act_limit = 0.f);
// act: b200_act_kind of the gate in the epilogue (0: silu; B200_ACT_SWIGLU_CLAMP with act_limit)
int rmsnorm(const __nv_bfloat16* x, __nv_bfloat16* res, const __nv_bfloat16* w, __nv_bfloat16* y, int T,
            int hidden, float eps, cudaStream_t s);
// fp32 residual stream (RMSNorm folded into the linears): embedding rows -> sres/ssq; stream rows -> normed bf16
// (prev, n_prev: tokens a negative id -(j+1) refers to, see elementwise.cu; nullptr = no such ids)
int embed_stream(const int32_t* ids, const __nv_bfloat16* table, float* sres, float* ssq, int T, int hidden, int vocab,
                 cudaStream_t s, const int32_t* prev = nullptr, int n_prev = 0);
int rmsnorm_stream(const float* sres, const float* ssq, const int32_t* rows, const __nv_bfloat16* w, __nv_bfloat16* y,
                   int R, int hidden, float eps, cudaStream_t s);
int embed(const int32_t* ids, const __nv_bfloat16* table, __nv_bfloat16* out, int T, int hidden, int vocab,
          cudaStream_t s, const int32_t* prev = nullptr, int n_prev = 0);
int rope_kv_append(__nv_bfloat16* qkv, const int32_t* positions, const int32_t* slots,
                   const __nv_bfloat16* cos_sin, __nv_bfloat16* kc, __nv_bfloat16* vc, int T, int hq,
                   int hkv, int block_size, cudaStream_t s);
int64_t paged_attn_workspace_bytes(int T, int hq, int max_ctx, int block_size);
int paged_attn(const __nv_bfloat16* q, int64_t ldq, const __nv_bfloat16* kc, const __nv_bfloat16* vc,
               const int32_t* block_table, int bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens,
               __nv_bfloat16* out, int64_t ldo, int T, int hq, int hkv, int block_size, int max_ctx,
               float scale, void* ws, int64_t ws_bytes, cudaStream_t s);
int paged_attn_ex(const __nv_bfloat16* q, int64_t ldq, const __nv_bfloat16* kc, const __nv_bfloat16* vc,
                  const int32_t* block_table, int bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens,
                  __nv_bfloat16* out, int64_t ldo, int T, int hq, int hkv, int block_size, int max_ctx,
                  float scale, void* ws, int64_t ws_bytes, int pack, cudaStream_t s);
int sample_rows(const __nv_bfloat16* logits, int64_t ld, int n_rows, int vocab, int seg_len, int64_t seg_stride,
                const float* temperature, const int32_t* top_k, const float* top_p, const float* min_p,
                const uint64_t* seeds, const uint64_t* draws, int32_t* out, cudaStream_t s);
int logit_adjust_rows(__nv_bfloat16* logits, int64_t ld, int n_rows, int vocab_local, int index_offset, const float* row_params,
                      const int32_t* offsets, const int32_t* ids, const int32_t* counts, const int32_t* seen, const float* bias,
                      cudaStream_t s);
int logprob_rows(const __nv_bfloat16* logits, int64_t ld, int n_rows, int vocab, int seg_len, int64_t seg_stride,
                 const int32_t* tok, int n_top, float* out_lp, int32_t* top_ids, float* top_lp, cudaStream_t s);
// once per step when pack > 0: builds the prefill attention's row plan in ws; 1 = built (use pack = 2), 0 = not used
int paged_attn_prefill_plan_step(const int32_t* row_to_seq, const int32_t* ctx_lens, int T, int hq, int hkv, int block_size,
                                 void* ws, int64_t ws_bytes, cudaStream_t s);
int advance_rows(int32_t* ids, int32_t* positions, int32_t* slots, int32_t* ctx_lens, const int32_t* block_table,
                 int bt_stride, const int32_t* row_to_seq, const int32_t* sampled, int n, int block_size,
                 cudaStream_t s);
int silu_mul(const __nv_bfloat16* gu, __nv_bfloat16* out, int T, int inter, cudaStream_t s);

// Peer-memory tensor-parallel all-reduce (allreduce.cu).  One IPC-shareable allocation per rank:
//   [ partial 0 | partial 1 | gather 0 | gather 1 | flags: 2 kinds x 2 buffers x 8 ranks x 128 B | state ]
struct ArParams {
  const __nv_bfloat16* bufs[8];   // every rank's partial for this buffer index (peer-mapped)
  unsigned int* flags[8];         // every rank's flag block
  unsigned int* state;            // local: counter[2] | ticket[2]
  __nv_bfloat16* out;
  long long n_chunks;             // 16-byte chunks
  int rank, world, buf_idx;
  __nv_bfloat16* gather[8];       // two-shot: every rank's normed-row buffer for this buffer index (peer-mapped)
};
int allreduce_oneshot(const ArParams& p, cudaStream_t s);
int allreduce_add_rmsnorm(const ArParams& p, int T, __nv_bfloat16* res, const __nv_bfloat16* w, __nv_bfloat16* y, int hidden,
                          float eps, cudaStream_t s);
int allreduce_twoshot_rmsnorm(const ArParams& p, int T, __nv_bfloat16* res, const __nv_bfloat16* w, int hidden, float eps,
                              cudaStream_t s);
int argmax_rows(const __nv_bfloat16* logits, int64_t ld, int rows, int vocab, int index_offset,
                int32_t* out_ids, float* out_max, cudaStream_t s);

// ---- mechanisms of models described layer by layer (stack.cu) -------------------------------------------------------
// fp32 residual stream: scaled embedding rows; bias-free layer norm with the sandwich form (post-norm of a sublayer's
// output added into the stream, then the pre-norm of the next sublayer) in one kernel
int embed_scaled(const int32_t* ids, const __nv_bfloat16* table, float* out, int T, int width, int vocab, float scale,
                 cudaStream_t s, const int32_t* prev = nullptr, int n_prev = 0);
int layernorm_stream(bool f32, float* x, const void* y, const float* yparts, int n_parts, const float* w_post,
                     const float* w_next, void* out, const int32_t* rows, int T, int width, float eps, cudaStream_t s);
// whole-projection RMS norm of q and k, interleaved partial rotation from a cos|sin table, unit-RMS (optionally rotated)
// values, k/v into the paged cache (rows of kstride / vstride elements, 0: dim / vdim; a wider row's tail is zeroed, and
// bf16 queries in qout16 get rows of kstride elements too)
int qk_norm_rotate_cache(bool f32, const void* qkv, const float* qw, const float* kw, const int32_t* positions,
                         const int32_t* slots, const float* rot, int rot_dims, const float* vrot, float* qout, void* kc,
                         void* vc, int T, int heads, int kv_heads, int dim, int vdim, int block_size, float eps,
                         int64_t max_pos, cudaStream_t s, __nv_bfloat16* qout16 = nullptr, int kstride = 0, int vstride = 0);
// attention output rows turned back by their position (bf16, in place): the closing step of rotated values when the
// attention kernel itself does not do it
int rotate_back_rows(const __nv_bfloat16* in, int in_stride, __nv_bfloat16* out, const int32_t* positions, const float* vrot, int T,
                     int heads, int vdim, int64_t max_pos, cudaStream_t s);
int convert_f32_to_bf16(const float* in, __nv_bfloat16* out, int64_t n, cudaStream_t s);
int convert_bf16_to_f32(const __nv_bfloat16* in, float* out, int64_t n, cudaStream_t s);
// paged softmax attention for any head sizes (attn_anydim.cu)
int64_t paged_attn_anydim_workspace_bytes(int T);
int paged_attn_anydim(bool f32, const float* q, const void* kc, const void* vc, const int32_t* block_table, int bt_stride,
                      const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions, const float* vrot,
                      int64_t max_pos, void* out, int T, int heads, int kv_heads, int dim, int vdim, int block_size, float scale,
                      int plan, void* ws, cudaStream_t s, int kstride = 0, int vstride = 0, const float* sink = nullptr, int window = 0);
// kstride / vstride: elements per cache row when they exceed dim / vdim (0: dim / vdim; the value cache may then be the key
// cache itself, a value being the leading vdim entries of the row); sink [heads]: exp(sink[h]) joins the softmax denominator
int paged_attn_runs_plan(const int32_t* row_to_seq, const int32_t* ctx_lens, int T, void* ws, cudaStream_t s);
// latent cache rows on the tensor cores (attn_latent.cu): bf16 cache, fp32 queries, bf16 output [T][heads][rank]
bool latent_attn_mma_supported(int heads, int krow, int rank);
int latent_attn_mma(const float* q, const __nv_bfloat16* kc, const int32_t* block_table, int bt_stride, const int32_t* row_to_seq,
                    const int32_t* ctx_lens, __nv_bfloat16* out, const int32_t* runs, const int32_t* n_runs, int T, int heads, int krow,
                    int rank, int block_size, float scale, const float* sink, cudaStream_t s, int n_splits = 1, float* part = nullptr,
                    int window = 0);
// the same kernel for grouped-query attention over key and value caches [block][kv_heads][block_size][dim | vdim]
bool paged_attn_mma_supported(int heads, int kv_heads, int dim, int vdim);
int paged_attn_mma(const float* q, const __nv_bfloat16* kc, const __nv_bfloat16* vc, const int32_t* block_table, int bt_stride,
                   const int32_t* row_to_seq, const int32_t* ctx_lens, __nv_bfloat16* out, const int32_t* runs, const int32_t* n_runs, int T,
                   int heads, int kv_heads, int dim, int vdim, int block_size, float scale, const float* sink, cudaStream_t s,
                   int n_splits = 1, float* part = nullptr, int window = 0);
// context splits for a step (1: none); part holds T * heads * n_splits * (rank + 2) floats
int latent_attn_splits(int T, int heads, int rank, int max_ctx, int64_t ws_bytes);
// mixture of experts (moe.cu)
int64_t moe_workspace_bytes(int T, int top, int experts, int width, int ff);
bool moe_tc_supported(int width, int ff);
// logits_ws ([T][experts] fp32) given and bf16 rows: the logits come from the tcgen05 linear (lin_ws: its split-K workspace)
// score_mode 0: softmax over all experts, the bias joins the choice only; 1: every expert's score is the sigmoid of its logit;
// 2: the bias joins the logits, the largest logits are chosen, weights = softmax over the chosen logits
int moe_route(bool f32, const void* x, const __nv_bfloat16* w_router, const float* bias, int T, int width, int experts, int top,
              int groups, int keep, int32_t* out_ids, float* out_w, cudaStream_t s, float* logits_ws = nullptr,
              void* lin_ws = nullptr, int64_t lin_ws_bytes = 0, int score_mode = 0);
// The shape of an expert: gated = down(act(gate x) * (up x)) over [expert][2 ff][width], else down(act(up x)) over
// [expert][ff][width]; weight_input: the mixing weight scales the expert's input row instead of its output row.
struct ExpertForm {
  bool gated = true;
  int act = B200_ACT_SILU;
  bool weight_input = false;
  float limit = 0.f;   // B200_ACT_SWIGLU_CLAMP
};
int moe_experts(bool f32, const void* x, const __nv_bfloat16* w_gu, const __nv_bfloat16* w_down, const int32_t* ids,
                const float* wts, int T, int width, int ff, int experts, int top, float* parts, void* ws, cudaStream_t s,
                ExpertForm form = ExpertForm());
// ---- the parallel layer form (stream_ops.cu, latent.cu, mlstm.cu) ------------------------------------------------------------
int seq_bounds(const int32_t* row_to_seq, int T, int S, int32_t* seq_start, cudaStream_t s);
int embed_bigram(const int32_t* ids, const __nv_bfloat16* table, const __nv_bfloat16* bigram, float* out, int T, int width, int vocab,
                 float scale, const int32_t* prev, int n_prev, const int32_t* positions, const int32_t* row_to_seq,
                 const int32_t* seq_slots, const int32_t* state_prev, int64_t slot_stride_ints, int buckets, int mul_prev, int mul_cur,
                 cudaStream_t s);
int prev_token_commit(const int32_t* ids, int vocab, const int32_t* prev, int n_prev, const int32_t* seq_start, const int32_t* seq_slots,
                      int S, int32_t* state_prev, int64_t slot_stride_ints, cudaStream_t s);
int parallel_close(bool f32, float* u, const void* y_mix, const void* y_ff, const float* parts, int n_parts, const void* y_sh,
                   float* results, int64_t result_stride, int n_results, const float* dwa, const float* g1, const float* g2,
                   float* h1_f32, void* h1_act, void* h2, int T, int width, float eps, cudaStream_t s);
int canon_conv(bool f32, const float* h, const float* w, void* out, int T, int width, int taps, const int32_t* positions,
               const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots, float* tails, int64_t slot_stride,
               cudaStream_t s);
int rms_rows(bool f32, const float* u, const int32_t* rows, const float* g, void* out, int R, int width, float eps, cudaStream_t s);
int ff_act(bool f32, const void* in, void* out, int T, int ff, bool gated, int kind, cudaStream_t s, float limit = 0.f);
int logit_cap(const float* in, float* out_f32, __nv_bfloat16* out_bf16, int R, int vocab, int ld, float cap, cudaStream_t s);
int latent_prep(bool f32, const void* qkv, int64_t ld, const float* norm_w, const int32_t* positions, const int32_t* slots,
                const float* rot, int rot_dims, int64_t max_pos, float* qfull, void* cache, int T, int heads, int dim, int rot_dim,
                int kv_rank, float eps, cudaStream_t s);
int head_linear(bool f32, bool y_f32, const void* x, int64_t ldx, int x_hs, const __nv_bfloat16* w, void* y, int64_t ldy, int y_hs,
                const void* gate, int64_t ldg, int g_hs, int T, int heads, int n_out, int k, cudaStream_t s, int g_es = 1);
int mlstm_gates(bool f32, const void* x, const __nv_bfloat16* w, const float* bias, float* out, int T, int width, int heads, float cap,
                cudaStream_t s);
int mlstm_col_blocks(int vd);
int64_t mlstm_state_floats(int heads, int dim, int vd);
int mlstm_scan(bool f32, const void* qkv, int64_t ld, int q_off, int k_off, int v_off, const float* gates, const int32_t* positions,
               const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int S, int heads,
               int dim, int vd, cudaStream_t s, bool single_rows = false);   // single_rows: every sequence of the step has one row
int head_norm_gate(bool f32, const float* o, const float* w, const void* gate, int64_t ldg, void* out, int T, int heads, int vd, float eps,
                   cudaStream_t s, bool gate_silu = false);   // gate_silu: times silu(gate) instead of sigmoid(gate)
// post-norm layer form (postnorm.cu): layer norm with bias after the sum; attention whose values are its raw keys with per-head
// q/k norms; the two norms of a latent mixer with a query latent
int postnorm_stream(bool f32, const float* x_in, const void* y, float alpha, const float* w, const float* b, float* x_out, void* out_act,
                    const int32_t* rows, int R, int width, float eps, cudaStream_t s);
int qk_headnorm_rotate_cache(bool f32, const void* qk, int64_t ld, const float* qw, const float* kw, const int32_t* positions,
                             const int32_t* slots, const float* rot, int rot_dims, int64_t max_pos, float* qout, void* kc, void* vc, int T,
                             int heads, int kv_heads, int dim, int vdim, int block_size, float eps, cudaStream_t s);
int latent_norms(bool f32, const void* fused, int64_t ld, int q_rank, int kv_rank, const float* qw, const float* kw, const int32_t* slots,
                 void* cq, void* cache, int T, float eps, cudaStream_t s);
// delta-rule recurrence with per-channel decays (delta.cu)
int delta_fused_rows(int heads, int kv_heads, int dim, int vdim, int decay_rank, int gate_rank, int* offsets);
int64_t delta_state_floats(int heads, int dim, int vd);
int64_t delta_tail_floats(int heads, int kv_heads, int dim, int vd, int taps);
int delta_prep(bool f32, const void* fused, int64_t ld, const void* a2, const float* conv_w, const float* dt_bias, const float* a_log,
               const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots, const float* tails,
               int64_t slot_stride, float* qn, float* kn, float* vn, float* beta, float* decay, int T, int heads, int kv_heads, int dim,
               int vdim, int taps, int decay_rank, int gate_rank, cudaStream_t s, bool head_decay = false);
// the scan with the decay of (row, head, channel) at decay[t * g_row + h * g_head + d * g_chan]; delta_rule false: u = beta v
int linear_scan(bool delta_rule, const float* qn, const float* kn, const float* vn, const float* beta, const float* decay, int64_t g_row,
                int g_head, int g_chan, const int32_t* positions, const int32_t* seq_start, const int32_t* seq_slots, float* state,
                int64_t slot_stride, float* out, int S, int heads, int kv_heads, int dim, int vd, cudaStream_t s);
// state-space mixer (ssd.cu)
int64_t ssd_tail_floats(int heads, int groups, int state, int vdim, int taps);
int ssd_prep(bool f32, const void* fused, int64_t ld, const float* conv_w, const float* conv_b, const float* dt_bias, const float* a_log,
             const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots, const float* tails,
             int64_t slot_stride, float* xn, float* bn, float* cn, float* dt, float* decay, int T, int heads, int groups, int state, int vdim,
             int taps, cudaStream_t s);
int ssd_gate_norm(bool f32, const float* o, const float* xn, const float* skip, const void* z, int64_t ldz, const float* w, void* out, int T,
                  int heads, int vdim, int norm_groups, float eps, cudaStream_t s);
// multi-stream pre-norm layer form (hyper.cu)
int hyper_step(bool f32, float* X, int64_t sstride, int n, bool init, const void* y, const float* parts, int n_parts, const float* scale,
               const float* hc, float mult, const float* open_in, const float* nw, const float* nb, float eps, const int32_t* rows,
               float* h_f32, void* h_act, float* sum_out, int R, int width, cudaStream_t s, const float* conv_w = nullptr, int taps = 0,
               const int32_t* positions = nullptr, const int32_t* row_to_seq = nullptr, const int32_t* seq_slots = nullptr,
               float* tails = nullptr, int64_t slot_stride = 0);
// conv_w [width][taps] given (steps whose sequences bring one row each): h + conv(h) goes to h_act and the tails
// [slot][taps - 1][width] (slot_stride floats apart) are shifted by the row
int qkv_rotate_cache(bool f32, const void* qkv, int64_t ld, const int32_t* positions, const int32_t* slots, const float* rot, int rot_dims,
                     bool half_layout, int64_t max_pos, float* qout, void* kc, void* vc, int T, int heads, int kv_heads, int dim, int vdim,
                     int block_size, cudaStream_t s);
int polynorm(bool f32, const void* z, const float* coef, void* out, int T, int ff, float eps, cudaStream_t s);
int delta_tails(bool f32, const void* fused, int64_t ld, const int32_t* positions, const int32_t* seq_start, const int32_t* seq_slots,
                float* tails, int64_t slot_stride, int S, int channels, int taps, cudaStream_t s);
int delta_scan(const float* qn, const float* kn, const float* vn, const float* beta, const float* decay, const int32_t* positions,
               const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int S, int heads,
               int kv_heads, int dim, int vd, cudaStream_t s);
// true-fp32 CUDA-core linear (linear_simt.cu)
int linear_simt(bool x_f32, bool y_f32, const void* x, int64_t ldx, const __nv_bfloat16* w, void* y, int64_t ldy, int T, int n_out,
                int k, cudaStream_t s);

}  // namespace b200
