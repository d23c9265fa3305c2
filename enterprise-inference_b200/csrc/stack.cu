// Models described layer by layer (b200_stack_create): construction, weights, per-layer caches and the step that
// strings the mechanisms together.  The ctx is the one every other entry point takes: the step runs through
// b200_decode_step[_host] (CUDA graphs, packed host metadata, token feedback), and sampling, log-probabilities and logit
// adjustment read the same logits buffer as for the fixed decoder stack.
//
// Step over T token rows (decode rows and rows of prefill chunks alike):
//   x = table[id] * embed_scale                                           fp32 residual stream
//   per layer:  h = LN(x) -> qkv = W_qkv h -> q/k RMS norm over the whole projection, rotation, unit-RMS rotated values,
//               k/v into the paged cache -> paged attention (+ output rotation) -> y = W_o a
//               x += LN(y); h = LN(x)            one kernel (sandwich norm)
//               router -> chosen experts -> per-slot partial rows;  x += LN(sum of slots); h = LN(x) for the next layer
//   logit rows: LN(x[rows]) -> W_head -> logits (bf16 for the samplers; fp32 mode keeps the unrounded rows too) -> argmax
//
// Parallel form (b200_stack_cfg.form = B200_FORM_PARALLEL), same step entry, cache and graph replay:
//   X_0 = table[id] * embed_scale + bigram row                            fp32; u = X_0
//   per layer:  h1 = u / rms(u) * g1, h2 = u / rms(u) * g2  ->  hc = h1 + conv(h1) (tail in the state slot)
//               mixer(hc): latent attention over the paged cache of [latent | rotated key part] rows, or the mLSTM
//               recurrence over the state slot;  ff(h2): dense gated, or routed experts + shared expert
//               X_{i+1} = u + (mixer + ff);  u = sum_j dwa[j] X_j;  norms of the next layer      one kernel
//   logit rows: u[rows] / rms * g -> W_head -> fp32 logits -> soft cap -> fp32 and bf16 copies -> argmax
//
// Post-norm form (b200_stack_cfg.form = B200_FORM_POSTNORM), same step entry, cache, state slots and graph replay:
//   x = table[id]                                                         fp32 residual stream (bf16 copy for the linears)
//   per layer:  y = mixer(x);  x = LN(alpha x + y) * w + b;   then, with a feed-forward,  x = LN'(alpha x + ff(x)) * w' + b'
//     attention: fused q | k -> per-head RMS norm, rotation, values = raw keys into the paged cache -> windowed attention with
//                one more unit in the denominator -> W_o
//     latent:    fused dq | dkv | g -> two RMS norms (dkv into the cache, unless the layer reads another layer's rows) -> W_uq ->
//                q' = W_uk^T q -> windowed attention over the latent rows -> W_uv with one sigmoid gate per head -> W_o
//     delta:     fused q | k | v | a1 | g1 | b -> W_a2, W_g2 -> convolution, unit vectors, beta, decays -> recurrence over the
//                state slot -> unit RMS per head, weight, gate -> W_o
//   logit rows: LN(x[rows]) * w + b -> W_head -> fp32 logits and their bf16 copy -> argmax
//
// Multi-stream pre-norm form (b200_stack_cfg.form = B200_FORM_HYPER), same step entry, cache, state slots and graph replay:
//   X_1..X_n = table[id] * embed_scale                                    n fp32 residual streams
//   per sublayer (mixer, then the feed-forward where the layer has one):
//     hyper_step: closes the sublayer before (X_t = sum_s M[s][t] X_s + mult b[t] scale y) and opens this one (u = sum_s a[s] X_s,
//                 h = LN(u) w + bias, fp32)  ->  canon_conv: h + conv(h) (tail in the state slot)  ->  the sublayer
//     attention:  fused q | k | v -> half-layout rotation, k and v into the paged cache -> attention with a learned sink -> W_o
//     delta:      fused q | k | v | gate | b | a -> convolution, unit vectors, beta, one decay per head -> recurrence -> unit RMS,
//                 weight, silu gate -> W_o
//     ssd:        fused z | x | B | C | dt -> convolution with bias, step sizes and decays -> recurrence without the correction
//                 term -> skip, gate, grouped RMS norm -> W_o
//     dense:      W_up -> polynomial of unit-RMS powers -> W_down;   experts: chosen-softmax router, clamped gated experts
//   logit rows: hyper_step over the rows (closes the last sublayer, a = ones, output norm) -> W_head -> fp32 logits -> argmax
#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "ctx.cuh"

namespace b200 {

struct StackLayerW {
  const float *n_mix_pre = nullptr, *n_mix_post = nullptr, *n_mlp_pre = nullptr, *n_mlp_post = nullptr, *q_norm = nullptr,
              *k_norm = nullptr, *router_bias = nullptr;
  const __nv_bfloat16 *qkv = nullptr, *o = nullptr, *router = nullptr, *e_gate_up = nullptr, *e_down = nullptr;
  void *kc = nullptr, *vc = nullptr;
  // parallel form
  const float *canon = nullptr, *dwa = nullptr, *sink = nullptr, *gates_bias = nullptr, *head_norm = nullptr;
  const __nv_bfloat16 *uk_t = nullptr, *uv = nullptr, *gates = nullptr, *mlp_gate_up = nullptr, *mlp_down = nullptr,
                      *shared_up = nullptr, *shared_down = nullptr;
  int64_t tail_off = 0, rec_off = 0;   // floats from the start of a state slot: convolution tail, recurrent state
  // post-norm form
  const float *n_mix_post_b = nullptr, *n_mlp_post_b = nullptr, *q_lat_norm = nullptr, *conv = nullptr, *decay_bias = nullptr,
              *decay_log = nullptr;
  const __nv_bfloat16 *uq = nullptr, *decay_up = nullptr, *gate_up = nullptr;
  bool gu_interleaved = false;   // mlp_gate_up holds 128-row slabs of 64 gate rows + the 64 matching up rows
  // multi-stream form
  const float *n_mix_pre_b = nullptr, *n_mlp_pre_b = nullptr, *scale_mix = nullptr, *scale_mlp = nullptr, *hc_mix = nullptr, *hc_mlp = nullptr,
              *canon_mlp = nullptr, *conv_b = nullptr, *skip = nullptr, *mlp_act = nullptr;
  int64_t tail2_off = 0, ctail_off = 0;   // floats from the start of a state slot: the feed-forward's input convolution tail, the mixer's own
};

struct StackModel {
  b200_stack_cfg cfg;
  std::vector<b200_stack_layer> layers;
  std::vector<StackLayerW> w;
  const __nv_bfloat16 *embed = nullptr, *head = nullptr;
  const float* final_norm = nullptr;
  const float* rot[16] = {};
  int64_t rot_pos[16] = {};
  int rot_half[16] = {};
  int64_t n_blocks = 0;
  int esz = 2;   // bytes per activation element
  // buffers (inside the ctx pool)
  float* x = nullptr;
  void *hn = nullptr, *qkv = nullptr, *attn = nullptr, *y = nullptr, *lm_in = nullptr;
  float* q = nullptr;
  int32_t* route_ids = nullptr;
  float *route_w = nullptr, *parts = nullptr, *route_logits = nullptr;
  void *attn_ws = nullptr, *moe_ws = nullptr;
  void* attn_wide = nullptr;    // [T][heads][128] bf16: what the 128-wide attention kernels write for narrower value heads
  void* attn_tc_ws = nullptr;   // row plan and split partials of the 128-wide tensor-core attention kernels
  int64_t attn_tc_ws_bytes = 0;
  float* tap = nullptr;
  // parallel form
  const __nv_bfloat16* bigram = nullptr;
  float* state = nullptr;              // caller-owned, n_state_slots slots of slot_floats floats
  int64_t slot_floats = 0;
  const int32_t* step_slots = nullptr; // device-pointer steps: the slots of the step's sequences
  int step_seqs = 0;
  float *results = nullptr, *h1f = nullptr, *gates_buf = nullptr, *oraw = nullptr, *head_f32 = nullptr;
  void *hc = nullptr, *lat = nullptr, *y2 = nullptr, *y3 = nullptr, *gu = nullptr, *ffa = nullptr;
  int32_t* seq_start = nullptr;
  float* lat_ws = nullptr;             // partial sums of the latent attention when a step's context is split over CTAs
  int64_t lat_ws_bytes = 0;
  // post-norm form
  const float* final_norm_b = nullptr;
  void *cq = nullptr, *qh = nullptr, *a2 = nullptr, *g2 = nullptr;   // query latent, queries, decay and gate projections
  float *dq = nullptr, *dk = nullptr, *dv = nullptr, *dbeta = nullptr, *ddecay = nullptr;   // what the recurrence reads
  float* zero_sink = nullptr;          // [heads] zeros: a sink of score 0 is one more unit in the denominator
  // multi-stream form
  float* xs = nullptr;                 // [streams][max_tokens][width]
};

bool paged_attn_tc_supported(int hq, int hkv, int block_size);   // attn_tc.cu

static bool is_latent(const b200_stack_layer& L) { return L.mixer == B200_MIXER_LATENT; }
static bool is_mlstm(const b200_stack_layer& L) { return L.mixer == B200_MIXER_MLSTM; }
static bool is_delta(const b200_stack_layer& L) { return L.mixer == B200_MIXER_DELTA; }
static bool is_ssd(const b200_stack_layer& L) { return L.mixer == B200_MIXER_SSD; }
static bool head_decay(const b200_stack_layer& L) { return (L.mixer_flags & B200_MIXF_HEAD_DECAY) != 0; }

// bf16 mode, keys and values of 64 to 128 dimensions in blocks of 128 tokens: the tcgen05 attention kernels of the fixed
// decoder stack serve the layer.  They are built for 128-wide heads, so the layer's cache rows and its bf16 queries are
// 128 wide with a zero tail (which adds nothing to a score, and whose outputs are dropped); the output rotation and the
// packing of narrower value heads are a step of their own.  Every other shape takes attn_anydim.cu.
static bool layer_attn_tc(const b200_stack_cfg& m, const b200_stack_layer& L) {
  static const int env = getenv("B200_STACK_ATTN_TC") ? atoi(getenv("B200_STACK_ATTN_TC")) : 1;
  return env && L.mixer == B200_MIXER_ATTENTION && m.form == B200_FORM_SANDWICH && !m.f32 && L.dim >= kHeadDim / 2 && L.dim <= kHeadDim && L.vdim >= kHeadDim / 2 && L.vdim <= kHeadDim &&
         L.scale > 0.f && paged_attn_tc_supported(L.heads, L.kv_heads, m.block_size);
}
// latent mixers cache one row [latent | rotated key part] per token (no value cache); mLSTM layers cache nothing
static int cache_kdim(const b200_stack_cfg& m, const b200_stack_layer& L) {
  if (is_latent(L)) return L.kv_share > 0 ? 0 : L.kv_rank + L.rot_dim;
  if (is_mlstm(L) || is_delta(L) || is_ssd(L)) return 0;
  return layer_attn_tc(m, L) ? kHeadDim : L.dim;
}
static int cache_vdim(const b200_stack_cfg& m, const b200_stack_layer& L) {
  if (is_latent(L) || is_mlstm(L) || is_delta(L) || is_ssd(L)) return 0;
  return layer_attn_tc(m, L) ? kHeadDim : L.vdim;
}

static int64_t up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// rows of the fused projection of the mixer's input
static int qkv_rows(const b200_stack_layer& L) {
  if (is_ssd(L)) return 2 * L.heads * L.vdim + 2 * L.kv_heads * L.dim + L.heads;             // z | x | B | C | dt
  if (is_delta(L) && head_decay(L)) return 2 * L.kv_heads * L.dim + 2 * L.heads * L.vdim + 2 * L.heads;   // q | k | v | gate | b | a
  if (is_delta(L)) return delta_fused_rows(L.heads, L.kv_heads, L.dim, L.vdim, L.decay_rank, L.gate_rank, nullptr);
  if (is_latent(L) && L.q_rank > 0)   // query latent | key/value latent (unless another layer's is read) | one gate row per head
    return L.q_rank + (L.kv_share > 0 ? 0 : L.kv_rank) + ((L.mixer_flags & B200_MIXF_HEAD_GATE) ? L.heads : 0);
  if (L.mixer == B200_MIXER_ATTENTION && (L.mixer_flags & B200_MIXF_VALUE_IS_KEY)) return (L.heads + L.kv_heads) * L.dim;
  if (is_latent(L))
    return L.heads * (L.dim + L.rot_dim) + L.kv_rank + L.rot_dim + ((L.mixer_flags & B200_MIXF_GATE) ? L.heads * L.vdim : 0);
  if (is_mlstm(L)) return 2 * L.heads * L.dim + 2 * L.heads * L.vdim;
  return L.heads * L.dim + L.kv_heads * (L.dim + L.vdim);
}

// bf16 mode: the tcgen05 weight-streaming linear wherever TMA can address the operands, else the CUDA-core tile kernel;
// fp32 mode: the CUDA-core kernel in true fp32.
static int stack_linear(b200_ctx* c, const void* x, int64_t ldx, const __nv_bfloat16* w, void* y, int64_t ldy, int T, int n_out,
                        int k, cudaStream_t s) {
  const StackModel* M = c->stack;
  if (M->cfg.f32) return linear_simt(true, true, x, ldx, w, y, ldy, T, n_out, k, s);
  static const int tc_env = getenv("B200_STACK_TC") ? atoi(getenv("B200_STACK_TC")) : 1;
  if (tc_env && k % 8 == 0 && ldx % 8 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
      linear_tc_supported(T, n_out, k) &&
      linear_tc_workspace_bytes(T, n_out, k) <= c->lin_ws_bytes)
    return linear_tc((const __nv_bfloat16*)x, ldx, w, nullptr, (__nv_bfloat16*)y, ldy, T, n_out, k, c->lin_ws, c->lin_ws_bytes,
                     nullptr, s);
  return linear_simt(false, false, x, ldx, w, y, ldy, T, n_out, k, s);
}

// Dense gated feed-forward, first half: act(gate x) * (up x) -> out [T][ff].  Interleaved weights: one tcgen05 launch whose
// epilogue activates and multiplies; else the plain linear and the activation kernel.
static int stack_gate_up(b200_ctx* c, const void* x, const StackLayerW& W, const b200_stack_layer& L, void* gu, void* out, int T, cudaStream_t s) {
  const StackModel* M = c->stack;
  const int Wd = M->cfg.width;
  if (W.gu_interleaved) {
    B200_REQUIRE(!M->cfg.f32 && linear_tc_supported(T, 2 * L.ff, Wd) && linear_tc_workspace_bytes(T, 2 * L.ff, Wd) <= c->lin_ws_bytes &&
                     reinterpret_cast<uintptr_t>(x) % 16 == 0,
                 B200_ERR_UNSUPPORTED, "feed-forward: interleaved gate|up weights need the tcgen05 linear (T=%d ff=%d width=%d)", T, L.ff, Wd);
    LinearExtra ex;
    ex.mode = 1;
    ex.act = L.act;
    return linear_tc((const __nv_bfloat16*)x, Wd, W.mlp_gate_up, nullptr, (__nv_bfloat16*)out, L.ff, T, 2 * L.ff, Wd, c->lin_ws, c->lin_ws_bytes, &ex, s);
  }
  int rc = stack_linear(c, x, Wd, W.mlp_gate_up, gu, 2 * L.ff, T, 2 * L.ff, Wd, s);
  if (rc) return rc;
  return ff_act(M->cfg.f32 != 0, gu, out, T, L.ff, true, L.act, s);
}

static int stack_ready_parallel(const b200_ctx* c) {
  const StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  B200_REQUIRE(m.bigram_buckets <= 0 || M->bigram, B200_ERR_STATE, "step: bigram table not set");
  B200_REQUIRE(m.n_state_slots <= 0 || M->state, B200_ERR_STATE, "step: state slots not set");
  for (size_t l = 0; l < M->layers.size(); ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    const int li = (int)l;
    B200_REQUIRE(W.n_mix_pre && W.qkv && W.o, B200_ERR_STATE, "step: layer %d mixer weights incomplete", li);
    B200_REQUIRE(m.canon_taps <= 0 || W.canon, B200_ERR_STATE, "step: layer %d convolution weights missing", li);
    B200_REQUIRE(!m.depth_avg || W.dwa, B200_ERR_STATE, "step: layer %d depth-average weights missing", li);
    if (is_latent(L)) {
      B200_REQUIRE(W.k_norm && W.uk_t && W.uv && W.kc, B200_ERR_STATE, "step: layer %d latent weights / cache incomplete", li);
      B200_REQUIRE(!(L.mixer_flags & B200_MIXF_SINK) || W.sink, B200_ERR_STATE, "step: layer %d sink missing", li);
      B200_REQUIRE(L.rot_dims == 0 || (L.rot_table >= 0 && M->rot[L.rot_table] && M->rot_half[L.rot_table] * 2 == L.rot_dims),
                   B200_ERR_STATE, "step: layer %d rotation table missing or of another size", li);
    } else {
      B200_REQUIRE(W.gates && W.head_norm, B200_ERR_STATE, "step: layer %d recurrent weights incomplete", li);
    }
    if (L.mlp != B200_MLP_NONE) B200_REQUIRE(W.n_mlp_pre, B200_ERR_STATE, "step: layer %d second norm missing", li);
    if (L.mlp == B200_MLP_DENSE) B200_REQUIRE(W.mlp_gate_up && W.mlp_down, B200_ERR_STATE, "step: layer %d feed-forward weights incomplete", li);
    if (L.mlp == B200_MLP_MOE) {
      B200_REQUIRE(W.router && W.e_gate_up && W.e_down, B200_ERR_STATE, "step: layer %d expert weights incomplete", li);
      B200_REQUIRE(L.shared_ff <= 0 || (W.shared_up && W.shared_down), B200_ERR_STATE, "step: layer %d shared expert incomplete", li);
    }
  }
  return B200_OK;
}

static int stack_ready_postnorm(const b200_ctx* c) {
  const StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  B200_REQUIRE(M->final_norm_b, B200_ERR_STATE, "step: the output norm's bias is not set");
  B200_REQUIRE(m.n_state_slots <= 0 || M->state, B200_ERR_STATE, "step: state slots not set");
  for (size_t l = 0; l < M->layers.size(); ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    const int li = (int)l;
    B200_REQUIRE(W.n_mix_post && W.n_mix_post_b && W.qkv && W.o, B200_ERR_STATE, "step: layer %d mixer weights incomplete", li);
    if (L.mixer == B200_MIXER_ATTENTION) {
      B200_REQUIRE(W.q_norm && W.k_norm && W.kc && W.vc, B200_ERR_STATE, "step: layer %d attention weights / cache incomplete", li);
      B200_REQUIRE(L.rot_dims == 0 || (L.rot_table >= 0 && M->rot[L.rot_table] && M->rot_half[L.rot_table] * 2 == L.rot_dims),
                   B200_ERR_STATE, "step: layer %d rotation table missing or of another size", li);
    } else if (is_latent(L)) {
      B200_REQUIRE(W.q_lat_norm && W.uq && W.uk_t && W.uv, B200_ERR_STATE, "step: layer %d latent weights incomplete", li);
      if (L.kv_share > 0) B200_REQUIRE(M->w[L.kv_share - 1].kc, B200_ERR_STATE, "step: layer %d reads the cache of layer %d, which has none", li, L.kv_share - 1);
      else B200_REQUIRE(W.k_norm && W.kc, B200_ERR_STATE, "step: layer %d latent norm / cache missing", li);
    } else {
      B200_REQUIRE(W.conv && W.decay_up && W.decay_bias && W.decay_log && W.gate_up && W.head_norm, B200_ERR_STATE,
                   "step: layer %d recurrent weights incomplete", li);
    }
    if (L.mlp == B200_MLP_DENSE)
      B200_REQUIRE(W.n_mlp_post && W.n_mlp_post_b && W.mlp_gate_up && W.mlp_down, B200_ERR_STATE, "step: layer %d feed-forward weights incomplete", li);
  }
  return B200_OK;
}

static int stack_ready_hyper(const b200_ctx* c) {
  const StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  B200_REQUIRE(M->final_norm_b, B200_ERR_STATE, "step: the output norm's bias is not set");
  B200_REQUIRE(m.n_state_slots <= 0 || M->state, B200_ERR_STATE, "step: state slots not set");
  for (size_t l = 0; l < M->layers.size(); ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    const int li = (int)l;
    B200_REQUIRE(W.n_mix_pre && W.n_mix_pre_b && W.scale_mix && W.hc_mix && W.qkv && W.o, B200_ERR_STATE, "step: layer %d mixer weights incomplete", li);
    B200_REQUIRE(m.canon_taps <= 0 || W.canon, B200_ERR_STATE, "step: layer %d convolution weights missing", li);
    if (L.mixer == B200_MIXER_ATTENTION) {
      B200_REQUIRE(W.kc && W.vc, B200_ERR_STATE, "step: layer %d cache missing", li);
      B200_REQUIRE(!(L.mixer_flags & B200_MIXF_SINK) || W.sink, B200_ERR_STATE, "step: layer %d sink missing", li);
      B200_REQUIRE(L.rot_dims == 0 || (L.rot_table >= 0 && M->rot[L.rot_table] && M->rot_half[L.rot_table] * 2 == L.rot_dims),
                   B200_ERR_STATE, "step: layer %d rotation table missing or of another size", li);
    } else if (is_delta(L)) {
      B200_REQUIRE(W.conv && W.decay_bias && W.decay_log && W.head_norm, B200_ERR_STATE, "step: layer %d recurrent weights incomplete", li);
    } else {
      B200_REQUIRE(W.conv && W.decay_bias && W.decay_log && W.head_norm && W.skip, B200_ERR_STATE, "step: layer %d recurrent weights incomplete", li);
    }
    if (L.mlp != B200_MLP_NONE) {
      B200_REQUIRE(W.n_mlp_pre && W.n_mlp_pre_b && W.scale_mlp && W.hc_mlp, B200_ERR_STATE, "step: layer %d feed-forward norm / stream weights missing", li);
      B200_REQUIRE(m.canon_taps <= 0 || W.canon_mlp, B200_ERR_STATE, "step: layer %d feed-forward convolution weights missing", li);
    }
    if (L.mlp == B200_MLP_DENSE)
      B200_REQUIRE(W.mlp_gate_up && W.mlp_down && (L.act != B200_ACT_POLYNORM || W.mlp_act), B200_ERR_STATE, "step: layer %d feed-forward weights incomplete", li);
    if (L.mlp == B200_MLP_MOE) B200_REQUIRE(W.router && W.e_gate_up && W.e_down, B200_ERR_STATE, "step: layer %d expert weights incomplete", li);
  }
  return B200_OK;
}

int stack_ready(const b200_ctx* c) {
  const StackModel* M = c->stack;
  B200_REQUIRE(M->embed && M->head && M->final_norm, B200_ERR_STATE, "step: embedding / output weights not set");
  if (M->cfg.form == B200_FORM_PARALLEL) return stack_ready_parallel(c);
  if (M->cfg.form == B200_FORM_POSTNORM) return stack_ready_postnorm(c);
  if (M->cfg.form == B200_FORM_HYPER) return stack_ready_hyper(c);
  for (size_t l = 0; l < M->layers.size(); ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    B200_REQUIRE(W.n_mix_pre && W.n_mix_post && W.qkv && W.q_norm && W.k_norm && W.o && W.kc && W.vc, B200_ERR_STATE,
                 "step: layer %d mixer weights / cache incomplete", (int)l);
    if (L.mlp == B200_MLP_MOE)
      B200_REQUIRE(W.n_mlp_pre && W.n_mlp_post && W.router && W.e_gate_up && W.e_down, B200_ERR_STATE,
                   "step: layer %d feed-forward weights incomplete", (int)l);
    B200_REQUIRE(L.rot_dims == 0 || (L.rot_table >= 0 && M->rot[L.rot_table] && M->rot_half[L.rot_table] * 2 == L.rot_dims),
                 B200_ERR_STATE, "step: layer %d rotation table missing or of another size", (int)l);
    B200_REQUIRE(L.vrot_table < 0 || (M->rot[L.vrot_table] && M->rot_half[L.vrot_table] * 2 == L.vdim), B200_ERR_STATE,
                 "step: layer %d value rotation table missing or of another size", (int)l);
  }
  return B200_OK;
}

int stack_state_slots(const b200_ctx* c) { return c->stack ? c->stack->cfg.n_state_slots : 0; }

void stack_step_slots(const b200_ctx* c, const int32_t** seq_slots, int* n_seqs) {
  *seq_slots = c->stack->step_slots;
  *n_seqs = c->stack->step_seqs;
}

void stack_destroy(b200_ctx* c) {
  delete c->stack;
  c->stack = nullptr;
}

// Logit rows of the forms that keep unrounded fp32 logits: lm_in [R][width] -> head_f32 [R][vocab] -> (cap) -> fp32 and bf16 rows
// with the ctx's leading dimension -> argmax.
static int stack_logits_f32(b200_ctx* c, const StepArgs& a, float cap, cudaStream_t s) {
  StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  const int Wd = m.width;
  int rc;
  if (m.f32) {
    rc = linear_simt(true, true, M->lm_in, Wd, M->head, M->head_f32, m.vocab, a.R, m.vocab, Wd, s);
  } else {
    // unrounded fp32 rows from the tcgen05 linear where it can address the operands, else the CUDA-core linear
    static const int tc_env = getenv("B200_STACK_TC") ? atoi(getenv("B200_STACK_TC")) : 1;
    if (tc_env && Wd % 8 == 0 && reinterpret_cast<uintptr_t>(M->head) % 16 == 0 && linear_tc_supported(a.R, m.vocab, Wd) &&
        linear_tc_workspace_bytes(a.R, m.vocab, Wd) <= c->lin_ws_bytes) {
      LinearExtra ex;
      ex.mode = 4;
      ex.out_f32 = M->head_f32;
      rc = linear_tc((const __nv_bfloat16*)M->lm_in, Wd, M->head, nullptr, nullptr, m.vocab, a.R, m.vocab, Wd, c->lin_ws, c->lin_ws_bytes, &ex, s);
    } else {
      rc = linear_simt(false, true, M->lm_in, Wd, M->head, M->head_f32, m.vocab, a.R, m.vocab, Wd, s);
    }
  }
  if (rc) return rc;
  rc = logit_cap(M->head_f32, c->logits_f32, c->logits, a.R, m.vocab, c->logits_ld, cap, s);
  if (rc) return rc;
  rc = argmax_rows(c->logits, c->logits_ld, a.R, m.vocab, 0, a.out_tokens, nullptr, s);
  if (rc) return rc;
  if (a.out_logits)
    B200_CUDA(cudaMemcpy2DAsync(a.out_logits, (size_t)m.vocab * 2, c->logits, (size_t)c->logits_ld * 2, (size_t)m.vocab * 2, a.R,
                                cudaMemcpyDeviceToDevice, s));
  return B200_OK;
}

// The step of the post-norm form.
static int stack_enqueue_step_postnorm(b200_ctx* c, const StepArgs& a, cudaStream_t s) {
  StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  const bool f32 = m.f32 != 0;
  const int T = a.T, Wd = m.width, nL = m.n_layers;
  const int64_t es = M->esz;
  int rc;
#define STEP(expr)     \
  do {                 \
    rc = (expr);       \
    if (rc) return rc; \
  } while (0)
  const bool stateful = m.n_state_slots > 0;
  const int S = a.n_seqs > 0 ? a.n_seqs : T;
  const int32_t* seq_slots = a.seq_slots;
  B200_REQUIRE(!stateful || seq_slots, B200_ERR_STATE, "step: the state slots of the step's sequences were not given");
  B200_REQUIRE(S <= T, B200_ERR_INVALID, "step: %d sequences in %d rows", S, T);
  int attn_plan = (a.row_to_seq && T >= 32 && T >= 2 * S) ? 1 : 0;
  static const int plan_env = getenv("B200_STACK_ATTN_RUNS") ? atoi(getenv("B200_STACK_ATTN_RUNS")) : 1;
  if (!plan_env) attn_plan = 0;
  bool runs_built = false;   // the step's run list is in the attention workspace
  // The run list is built by a launch of its own, once per step, before the first kernel that reads it: whether a layer's
  // attention takes a kernel that walks runs depends on the layer's shape, so no attention call can be trusted to leave it.
  auto step_runs = [&](bool& built) -> int {
    if (built) return B200_OK;
    built = true;
    return paged_attn_runs_plan(a.row_to_seq, a.ctx_lens, T, M->attn_ws, s);
  };
  float* x = M->x;
  // what the linears read: the stream itself in 32-bit mode, its rounded copy otherwise
  void* hin = f32 ? static_cast<void*>(x) : M->hn;
  void* hcopy = f32 ? nullptr : M->hn;
  if (stateful) STEP(seq_bounds(a.row_to_seq, T, S, M->seq_start, s));
  STEP(embed_scaled(a.ids, M->embed, x, T, Wd, m.vocab, m.embed_scale, s, a.prev_tokens, a.n_prev));
  if (!f32) STEP(convert_f32_to_bf16(x, (__nv_bfloat16*)M->hn, (int64_t)T * Wd, s));
  for (int l = 0; l < nL; ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    const int qr = qkv_rows(L), av = L.heads * L.vdim;
    STEP(stack_linear(c, hin, Wd, W.qkv, M->qkv, qr, T, qr, Wd, s));
    if (L.mixer == B200_MIXER_ATTENTION) {
      const float* rot = L.rot_dims > 0 ? M->rot[L.rot_table] : nullptr;
      const int64_t max_pos = rot ? M->rot_pos[L.rot_table] : (1ll << 40);
      STEP(qk_headnorm_rotate_cache(f32, M->qkv, qr, W.q_norm, W.k_norm, a.positions, a.slots, rot, L.rot_dims, max_pos, M->q, W.kc, W.vc, T,
                                    L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, m.norm_eps, s));
      const float* sink = (L.mixer_flags & B200_MIXF_SINK_ONE) ? M->zero_sink : nullptr;
      if (!f32 && paged_attn_mma_supported(L.heads, L.kv_heads, L.dim, L.vdim)) {
        STEP(step_runs(runs_built));
        const int seen = L.window > 0 ? std::min(a.max_ctx, L.window + 64) : a.max_ctx;
        STEP(paged_attn_mma(M->q, (const __nv_bfloat16*)W.kc, (const __nv_bfloat16*)W.vc, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens,
                            (__nv_bfloat16*)M->attn, static_cast<const int32_t*>(M->attn_ws) + 8, static_cast<const int32_t*>(M->attn_ws), T,
                            L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, L.scale, sink, s,
                            latent_attn_splits(T, L.heads, L.vdim, seen, M->lat_ws_bytes), M->lat_ws, L.window));
      } else {
      if (attn_plan) STEP(step_runs(runs_built));
      STEP(paged_attn_anydim(f32, M->q, W.kc, W.vc, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens, a.positions, nullptr, max_pos,
                             M->attn, T, L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, L.scale, attn_plan ? 2 : 0, M->attn_ws, s, 0, 0, sink,
                             L.window));
      }
    } else if (is_latent(L)) {
      const int kr = L.kv_rank, hd = L.heads * L.dim;
      void* cache = L.kv_share > 0 ? M->w[L.kv_share - 1].kc : W.kc;
      STEP(latent_norms(f32, M->qkv, qr, L.q_rank, kr, W.q_lat_norm, W.k_norm, a.slots, M->cq, L.kv_share > 0 ? nullptr : W.kc, T, m.norm_eps, s));
      STEP(stack_linear(c, M->cq, L.q_rank, W.uq, M->qh, hd, T, hd, L.q_rank, s));
      // q' = W_uk^T q: the scores are taken against the cached latent rows
      STEP(head_linear(f32, true, M->qh, hd, L.dim, W.uk_t, M->q, (int64_t)L.heads * kr, kr, nullptr, 0, 0, T, L.heads, kr, L.dim, s));
      if (!f32 && latent_attn_mma_supported(L.heads, kr, kr)) {
        STEP(step_runs(runs_built));
        const int seen = L.window > 0 ? std::min(a.max_ctx, L.window + 64) : a.max_ctx;
        STEP(latent_attn_mma(M->q, (const __nv_bfloat16*)cache, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens, (__nv_bfloat16*)M->lat,
                             static_cast<const int32_t*>(M->attn_ws) + 8, static_cast<const int32_t*>(M->attn_ws), T, L.heads, kr, kr,
                             m.block_size, L.scale, nullptr, s, latent_attn_splits(T, L.heads, kr, seen, M->lat_ws_bytes), M->lat_ws, L.window));
      } else {
        if (attn_plan) STEP(step_runs(runs_built));
        STEP(paged_attn_anydim(f32, M->q, cache, cache, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens, a.positions, nullptr, 1ll << 40,
                               M->lat, T, L.heads, 1, kr, kr, m.block_size, L.scale, attn_plan ? 2 : 0, M->attn_ws, s, kr, kr, nullptr, L.window));
      }
      const bool gate = (L.mixer_flags & B200_MIXF_HEAD_GATE) != 0;
      const char* gptr = static_cast<const char*>(M->qkv) + (int64_t)(L.q_rank + (L.kv_share > 0 ? 0 : kr)) * es;
      STEP(head_linear(f32, false, M->lat, (int64_t)L.heads * kr, kr, W.uv, M->attn, av, L.vdim, gate ? gptr : nullptr, qr, 1, T, L.heads,
                       L.vdim, kr, s, 0));
    } else {
      int off[6];
      delta_fused_rows(L.heads, L.kv_heads, L.dim, L.vdim, L.decay_rank, L.gate_rank, off);
      const int hd = L.heads * L.dim, C = 2 * L.kv_heads * L.dim + av;
      const char* fused = static_cast<const char*>(M->qkv);
      STEP(stack_linear(c, fused + off[3] * es, qr, W.decay_up, M->a2, hd, T, hd, L.decay_rank, s));
      STEP(stack_linear(c, fused + off[4] * es, qr, W.gate_up, M->g2, av, T, av, L.gate_rank, s));
      float* tails = L.conv_taps > 1 ? M->state + W.tail_off : nullptr;
      STEP(delta_prep(f32, M->qkv, qr, M->a2, W.conv, W.decay_bias, W.decay_log, a.positions, a.row_to_seq, M->seq_start, seq_slots, tails,
                      M->slot_floats, M->dq, M->dk, M->dv, M->dbeta, M->ddecay, T, L.heads, L.kv_heads, L.dim, L.vdim, L.conv_taps,
                      L.decay_rank, L.gate_rank, s));
      STEP(delta_tails(f32, M->qkv, qr, a.positions, M->seq_start, seq_slots, tails, M->slot_floats, S, C, L.conv_taps, s));
      STEP(delta_scan(M->dq, M->dk, M->dv, M->dbeta, M->ddecay, a.positions, M->seq_start, seq_slots, M->state + W.rec_off, M->slot_floats,
                      M->oraw, S, L.heads, L.kv_heads, L.dim, L.vdim, s));
      STEP(head_norm_gate(f32, M->oraw, W.head_norm, M->g2, av, M->attn, T, L.heads, L.vdim, m.norm_eps, s));
    }
    STEP(stack_linear(c, M->attn, av, W.o, M->y, Wd, T, Wd, av, s));
    STEP(postnorm_stream(f32, x, M->y, m.residual_alpha, W.n_mix_post, W.n_mix_post_b, x, hcopy, nullptr, T, Wd, m.norm_eps, s));
    if (L.mlp == B200_MLP_DENSE) {
      STEP(stack_gate_up(c, hin, W, L, M->gu, M->ffa, T, s));
      STEP(stack_linear(c, M->ffa, L.ff, W.mlp_down, M->y2, Wd, T, Wd, L.ff, s));
      STEP(postnorm_stream(f32, x, M->y2, m.residual_alpha, W.n_mlp_post, W.n_mlp_post_b, x, hcopy, nullptr, T, Wd, m.norm_eps, s));
    }
    if (M->tap) B200_CUDA(cudaMemcpyAsync(M->tap + (int64_t)l * T * Wd, x, (size_t)T * Wd * 4, cudaMemcpyDeviceToDevice, s));
  }
  STEP(postnorm_stream(f32, x, nullptr, 1.0f, M->final_norm, M->final_norm_b, nullptr, M->lm_in, a.logit_rows, a.R, Wd, m.norm_eps, s));
  STEP(stack_logits_f32(c, a, 0.f, s));
#undef STEP
  return B200_OK;
}

// The step of the parallel form.  Sequences of the step: a.n_seqs with their slots behind the block tables (host-buffer
// entry), or the array given by b200_stack_set_step_slots (device-pointer entry).
static int stack_enqueue_step_parallel(b200_ctx* c, const StepArgs& a, cudaStream_t s) {
  StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  const bool f32 = m.f32 != 0;
  const int T = a.T, Wd = m.width, nL = m.n_layers;
  const int64_t es = M->esz;
  int rc;
#define STEP(expr)     \
  do {                 \
    rc = (expr);       \
    if (rc) return rc; \
  } while (0)
  const bool stateful = m.n_state_slots > 0;
  const int S = a.n_seqs > 0 ? a.n_seqs : T;
  const int32_t* seq_slots = a.seq_slots;
  B200_REQUIRE(!stateful || seq_slots, B200_ERR_STATE, "step: the state slots of the step's sequences were not given");
  B200_REQUIRE(S <= T, B200_ERR_INVALID, "step: %d sequences in %d rows", S, T);
  int attn_plan = (a.row_to_seq && T >= 32 && T >= 2 * S) ? 1 : 0;
  static const int plan_env = getenv("B200_STACK_ATTN_RUNS") ? atoi(getenv("B200_STACK_ATTN_RUNS")) : 1;
  if (!plan_env) attn_plan = 0;
  bool runs_built = false;   // the step's run list is in the attention workspace
  // The run list is built by a launch of its own, once per step, before the first kernel that reads it: whether a layer's
  // attention takes a kernel that walks runs depends on the layer's shape, so no attention call can be trusted to leave it.
  auto step_runs = [&](bool& built) -> int {
    if (built) return B200_OK;
    built = true;
    return paged_attn_runs_plan(a.row_to_seq, a.ctx_lens, T, M->attn_ws, s);
  };
  const int64_t rstride = (int64_t)m.max_tokens * Wd;
  float* u = M->x;
  int32_t* st_prev = reinterpret_cast<int32_t*>(M->state);
  STEP(seq_bounds(a.row_to_seq, T, S, M->seq_start, s));
  STEP(embed_bigram(a.ids, M->embed, M->bigram, u, T, Wd, m.vocab, m.embed_scale, a.prev_tokens, a.n_prev, a.positions, a.row_to_seq,
                    seq_slots, stateful ? st_prev : nullptr, M->slot_floats, m.bigram_buckets, m.bigram_mul_prev, m.bigram_mul_cur, s));
  if (stateful && m.bigram_buckets > 0)
    STEP(prev_token_commit(a.ids, m.vocab, a.prev_tokens, a.n_prev, M->seq_start, seq_slots, S, st_prev, M->slot_floats, s));
  const bool conv = m.canon_taps >= 1;
  // X_0 and the first layer's norms
  STEP(parallel_close(f32, u, nullptr, nullptr, nullptr, 0, nullptr, m.depth_avg ? M->results : nullptr, rstride, 1, nullptr,
                      M->w[0].n_mix_pre, M->w[0].n_mlp_pre, conv ? M->h1f : nullptr, conv ? nullptr : M->hc, M->hn, T, Wd, m.norm_eps, s));
  for (int l = 0; l < nL; ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    const int qr = qkv_rows(L);
    if (conv)
      STEP(canon_conv(f32, M->h1f, W.canon, M->hc, T, Wd, m.canon_taps, a.positions, a.row_to_seq, M->seq_start, seq_slots,
                      M->state ? M->state + W.tail_off : nullptr, M->slot_floats, s));
    STEP(stack_linear(c, M->hc, Wd, W.qkv, M->qkv, qr, T, qr, Wd, s));
    const int av = L.heads * L.vdim;
    if (is_latent(L)) {
      const int qh = L.dim + L.rot_dim, krow = L.kv_rank + L.rot_dim;
      const float* rot = L.rot_dims > 0 ? M->rot[L.rot_table] : nullptr;
      const int64_t max_pos = rot ? M->rot_pos[L.rot_table] : (1ll << 40);
      STEP(latent_prep(f32, M->qkv, qr, W.k_norm, a.positions, a.slots, rot, L.rot_dims, max_pos, M->q, W.kc, T, L.heads, L.dim,
                       L.rot_dim, L.kv_rank, m.norm_eps, s));
      // q' = W_uk^T q_plain into the leading kv_rank entries of every query row
      STEP(head_linear(f32, true, M->qkv, qr, qh, W.uk_t, M->q, (int64_t)L.heads * krow, krow, nullptr, 0, 0, T, L.heads, L.kv_rank,
                       L.dim, s));
      const float* sink = (L.mixer_flags & B200_MIXF_SINK) ? W.sink : nullptr;
      if (!f32 && latent_attn_mma_supported(L.heads, krow, L.kv_rank)) {
        STEP(step_runs(runs_built));
        STEP(latent_attn_mma(M->q, (const __nv_bfloat16*)W.kc, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens,
                             (__nv_bfloat16*)M->lat, static_cast<const int32_t*>(M->attn_ws) + 8, static_cast<const int32_t*>(M->attn_ws), T,
                             L.heads, krow, L.kv_rank, m.block_size, L.scale, sink, s,
                             latent_attn_splits(T, L.heads, L.kv_rank, a.max_ctx, M->lat_ws_bytes), M->lat_ws));
      } else {
        if (attn_plan) STEP(step_runs(runs_built));
        STEP(paged_attn_anydim(f32, M->q, W.kc, W.kc, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens, a.positions, nullptr, max_pos,
                               M->lat, T, L.heads, 1, krow, L.kv_rank, m.block_size, L.scale, attn_plan ? 2 : 0, M->attn_ws, s, krow, krow, sink));
      }
      const bool gate = (L.mixer_flags & B200_MIXF_GATE) != 0;
      const char* gptr = static_cast<const char*>(M->qkv) + (int64_t)(L.heads * qh + krow) * es;
      STEP(head_linear(f32, false, M->lat, (int64_t)L.heads * L.kv_rank, L.kv_rank, W.uv, M->attn, av, L.vdim, gate ? gptr : nullptr, qr,
                       L.vdim, T, L.heads, L.vdim, L.kv_rank, s));
    } else {
      const int hd = L.heads * L.dim;
      STEP(mlstm_gates(f32, M->hc, W.gates, W.gates_bias, M->gates_buf, T, Wd, L.heads, L.gate_cap, s));
      STEP(mlstm_scan(f32, M->qkv, qr, 0, hd, 2 * hd, M->gates_buf, a.positions, M->seq_start, seq_slots, M->state + W.rec_off,
                      M->slot_floats, M->oraw, S, L.heads, L.dim, L.vdim, s, S == T));
      const char* gptr = static_cast<const char*>(M->qkv) + (int64_t)(2 * hd + av) * es;
      STEP(head_norm_gate(f32, M->oraw, W.head_norm, gptr, qr, M->attn, T, L.heads, L.vdim, m.norm_eps, s));
    }
    STEP(stack_linear(c, M->attn, av, W.o, M->y, Wd, T, Wd, av, s));
    const void *y_ff = nullptr, *y_sh = nullptr;
    const float* parts = nullptr;
    int n_parts = 0;
    if (L.mlp == B200_MLP_DENSE) {
      STEP(stack_gate_up(c, M->hn, W, L, M->gu, M->ffa, T, s));
      STEP(stack_linear(c, M->ffa, L.ff, W.mlp_down, M->y2, Wd, T, Wd, L.ff, s));
      y_ff = M->y2;
    } else if (L.mlp == B200_MLP_MOE) {
      STEP(moe_route(f32, M->hn, W.router, W.router_bias, T, Wd, L.experts, L.top, L.groups, L.keep, M->route_ids, M->route_w, s,
                     M->route_logits, c->lin_ws, c->lin_ws_bytes, L.sigmoid_scores != 0));
      ExpertForm form;
      form.gated = !L.ungated;
      form.act = L.act;
      form.weight_input = L.weight_input != 0;
      STEP(moe_experts(f32, M->hn, W.e_gate_up, W.e_down, M->route_ids, M->route_w, T, Wd, L.ff, L.experts, L.top, M->parts, M->moe_ws,
                       s, form));
      parts = M->parts;
      n_parts = L.top;
      if (L.shared_ff > 0) {
        const int sr = (L.ungated ? 1 : 2) * L.shared_ff;
        STEP(stack_linear(c, M->hn, Wd, W.shared_up, M->gu, sr, T, sr, Wd, s));
        STEP(ff_act(f32, M->gu, M->ffa, T, L.shared_ff, !L.ungated, L.act, s));
        STEP(stack_linear(c, M->ffa, L.shared_ff, W.shared_down, M->y3, Wd, T, Wd, L.shared_ff, s));
        y_sh = M->y3;
      }
    }
    const bool last = l + 1 == nL;
    STEP(parallel_close(f32, u, M->y, y_ff, parts, n_parts, y_sh, m.depth_avg ? M->results : nullptr, rstride, l + 2,
                        m.depth_avg ? W.dwa : nullptr, last ? nullptr : M->w[l + 1].n_mix_pre, last ? nullptr : M->w[l + 1].n_mlp_pre,
                        conv ? M->h1f : nullptr, conv ? nullptr : M->hc, M->hn, T, Wd, m.norm_eps, s));
    if (M->tap) B200_CUDA(cudaMemcpyAsync(M->tap + (int64_t)l * T * Wd, u, (size_t)T * Wd * 4, cudaMemcpyDeviceToDevice, s));
  }
  STEP(rms_rows(f32, u, a.logit_rows, M->final_norm, M->lm_in, a.R, Wd, m.norm_eps, s));
  STEP(stack_logits_f32(c, a, m.logit_softcap, s));
#undef STEP
  return B200_OK;
}

// The step of the multi-stream pre-norm form.
static int stack_enqueue_step_hyper(b200_ctx* c, const StepArgs& a, cudaStream_t s) {
  StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  const bool f32 = m.f32 != 0;
  const int T = a.T, Wd = m.width, nL = m.n_layers, n = m.streams;
  const int64_t es = M->esz;
  int rc;
#define STEP(expr)     \
  do {                 \
    rc = (expr);       \
    if (rc) return rc; \
  } while (0)
  const bool stateful = m.n_state_slots > 0;
  const int S = a.n_seqs > 0 ? a.n_seqs : T;
  const int32_t* seq_slots = a.seq_slots;
  B200_REQUIRE(!stateful || seq_slots, B200_ERR_STATE, "step: the state slots of the step's sequences were not given");
  B200_REQUIRE(S <= T, B200_ERR_INVALID, "step: %d sequences in %d rows", S, T);
  int attn_plan = (a.row_to_seq && T >= 32 && T >= 2 * S) ? 1 : 0;
  static const int plan_env = getenv("B200_STACK_ATTN_RUNS") ? atoi(getenv("B200_STACK_ATTN_RUNS")) : 1;
  if (!plan_env) attn_plan = 0;
  bool runs_built = false;   // the step's run list is in the attention workspace
  auto step_runs = [&](bool& built) -> int {
    if (built) return B200_OK;
    built = true;
    return paged_attn_runs_plan(a.row_to_seq, a.ctx_lens, T, M->attn_ws, s);
  };
  const int64_t sstride = (int64_t)m.max_tokens * Wd;
  const bool conv = m.canon_taps >= 1;
  float* X = M->xs;
  if (stateful) STEP(seq_bounds(a.row_to_seq, T, S, M->seq_start, s));
  STEP(embed_scaled(a.ids, M->embed, X, T, Wd, m.vocab, m.embed_scale, s, a.prev_tokens, a.n_prev));
  // what the sublayer before left to be closed: its result (an activation row or expert partial rows), scale and coefficients
  const void* y_prev = nullptr;
  const float *parts_prev = nullptr, *scale_prev = nullptr, *hc_prev = nullptr;
  int n_parts_prev = 0;
  bool first = true;
  // closes the sublayer before, opens one with coefficients hc / norm (w, b) / convolution cw (tail at tail_off) into `out`
  // every sequence brings one row (decode): the convolution runs behind the norm in the same launch
  static const int fuse_env = getenv("B200_STACK_FUSE_CANON") ? atoi(getenv("B200_STACK_FUSE_CANON")) : 1;
  const bool one_row_each = (a.n_seqs > 0 && a.n_seqs == T) || a.row_to_seq == nullptr;   // known, not assumed
  const bool conv_fused = conv && fuse_env && one_row_each && (m.canon_taps == 1 || M->state);
  auto open = [&](const float* hc, const float* w, const float* b, const float* cw, int64_t tail_off, void* out, float* tap) -> int {
    if (conv_fused) {
      const bool was_first = first;
      first = false;
      return hyper_step(f32, X, sstride, n, was_first, y_prev, parts_prev, n_parts_prev, scale_prev, hc_prev, m.residual_mult, hc, w, b, m.norm_eps,
                        nullptr, nullptr, out, tap, T, Wd, s, cw, m.canon_taps, a.positions, a.row_to_seq, seq_slots,
                        M->state ? M->state + tail_off : nullptr, M->slot_floats);
    }
    int r = hyper_step(f32, X, sstride, n, first, y_prev, parts_prev, n_parts_prev, scale_prev, hc_prev, m.residual_mult, hc, w, b, m.norm_eps,
                       nullptr, conv ? M->h1f : nullptr, conv ? nullptr : out, tap, T, Wd, s);
    first = false;
    if (r || !conv) return r;
    return canon_conv(f32, M->h1f, cw, out, T, Wd, m.canon_taps, a.positions, a.row_to_seq, M->seq_start, seq_slots,
                      M->state ? M->state + tail_off : nullptr, M->slot_floats, s);
  };
  for (int l = 0; l < nL; ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    const int qr = qkv_rows(L), av = L.heads * L.vdim;
    float* tap = (M->tap && l > 0) ? M->tap + (int64_t)(l - 1) * T * Wd : nullptr;   // the layer before is complete once its last sublayer is closed
    STEP(open(W.hc_mix, W.n_mix_pre, W.n_mix_pre_b, W.canon, W.tail_off, M->hc, tap));
    STEP(stack_linear(c, M->hc, Wd, W.qkv, M->qkv, qr, T, qr, Wd, s));
    if (L.mixer == B200_MIXER_ATTENTION) {
      const float* rot = L.rot_dims > 0 ? M->rot[L.rot_table] : nullptr;
      const int64_t max_pos = rot ? M->rot_pos[L.rot_table] : (1ll << 40);
      STEP(qkv_rotate_cache(f32, M->qkv, qr, a.positions, a.slots, rot, L.rot_dims, (L.mixer_flags & B200_MIXF_ROT_HALF) != 0, max_pos, M->q, W.kc,
                            W.vc, T, L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, s));
      const float* sink = (L.mixer_flags & B200_MIXF_SINK) ? W.sink : ((L.mixer_flags & B200_MIXF_SINK_ONE) ? M->zero_sink : nullptr);
      if (!f32 && paged_attn_mma_supported(L.heads, L.kv_heads, L.dim, L.vdim)) {
        STEP(step_runs(runs_built));
        const int seen = L.window > 0 ? std::min(a.max_ctx, L.window + 64) : a.max_ctx;
        STEP(paged_attn_mma(M->q, (const __nv_bfloat16*)W.kc, (const __nv_bfloat16*)W.vc, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens,
                            (__nv_bfloat16*)M->attn, static_cast<const int32_t*>(M->attn_ws) + 8, static_cast<const int32_t*>(M->attn_ws), T,
                            L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, L.scale, sink, s,
                            latent_attn_splits(T, L.heads, L.vdim, seen, M->lat_ws_bytes), M->lat_ws, L.window));
      } else {
        if (attn_plan) STEP(step_runs(runs_built));
        STEP(paged_attn_anydim(f32, M->q, W.kc, W.vc, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens, a.positions, nullptr, max_pos,
                               M->attn, T, L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, L.scale, attn_plan ? 2 : 0, M->attn_ws, s, 0, 0, sink,
                               L.window));
      }
    } else if (is_delta(L)) {
      const int C = 2 * L.kv_heads * L.dim + av;
      float* tails = L.conv_taps > 1 ? M->state + W.ctail_off : nullptr;
      STEP(delta_prep(f32, M->qkv, qr, nullptr, W.conv, W.decay_bias, W.decay_log, a.positions, a.row_to_seq, M->seq_start, seq_slots, tails,
                      M->slot_floats, M->dq, M->dk, M->dv, M->dbeta, M->ddecay, T, L.heads, L.kv_heads, L.dim, L.vdim, L.conv_taps, 0, 0, s, true));
      STEP(delta_tails(f32, M->qkv, qr, a.positions, M->seq_start, seq_slots, tails, M->slot_floats, S, C, L.conv_taps, s));
      STEP(linear_scan(true, M->dq, M->dk, M->dv, M->dbeta, M->ddecay, L.heads, 1, 0, a.positions, M->seq_start, seq_slots, M->state + W.rec_off,
                       M->slot_floats, M->oraw, S, L.heads, L.kv_heads, L.dim, L.vdim, s));
      const char* gptr = static_cast<const char*>(M->qkv) + (int64_t)C * es;
      STEP(head_norm_gate(f32, M->oraw, W.head_norm, gptr, qr, M->attn, T, L.heads, L.vdim, m.norm_eps, s, true));
    } else {
      const int gn = L.kv_heads * L.dim, C = av + 2 * gn;
      float* tails = L.conv_taps > 1 ? M->state + W.ctail_off : nullptr;
      STEP(ssd_prep(f32, M->qkv, qr, W.conv, W.conv_b, W.decay_bias, W.decay_log, a.positions, a.row_to_seq, M->seq_start, seq_slots, tails,
                    M->slot_floats, M->dv, M->dk, M->dq, M->dbeta, M->ddecay, T, L.heads, L.kv_heads, L.dim, L.vdim, L.conv_taps, s));
      const char* xbc = static_cast<const char*>(M->qkv) + (int64_t)av * es;
      STEP(delta_tails(f32, xbc, qr, a.positions, M->seq_start, seq_slots, tails, M->slot_floats, S, C, L.conv_taps, s));
      STEP(linear_scan(false, M->dq, M->dk, M->dv, M->dbeta, M->ddecay, L.heads, 1, 0, a.positions, M->seq_start, seq_slots, M->state + W.rec_off,
                       M->slot_floats, M->oraw, S, L.heads, L.kv_heads, L.dim, L.vdim, s));
      STEP(ssd_gate_norm(f32, M->oraw, M->dv, W.skip, M->qkv, qr, W.head_norm, M->attn, T, L.heads, L.vdim, L.norm_groups, m.norm_eps, s));
    }
    STEP(stack_linear(c, M->attn, av, W.o, M->y, Wd, T, Wd, av, s));
    y_prev = M->y, parts_prev = nullptr, n_parts_prev = 0, scale_prev = W.scale_mix, hc_prev = W.hc_mix;
    if (L.mlp == B200_MLP_NONE) continue;
    STEP(open(W.hc_mlp, W.n_mlp_pre, W.n_mlp_pre_b, W.canon_mlp, W.tail2_off, M->hn, nullptr));
    if (L.mlp == B200_MLP_DENSE) {
      if (L.ungated) {
        STEP(stack_linear(c, M->hn, Wd, W.mlp_gate_up, M->gu, L.ff, T, L.ff, Wd, s));
        if (L.act == B200_ACT_POLYNORM) STEP(polynorm(f32, M->gu, W.mlp_act, M->ffa, T, L.ff, m.norm_eps, s));
        else STEP(ff_act(f32, M->gu, M->ffa, T, L.ff, false, L.act, s));
      } else {
        STEP(stack_linear(c, M->hn, Wd, W.mlp_gate_up, M->gu, 2 * L.ff, T, 2 * L.ff, Wd, s));
        STEP(ff_act(f32, M->gu, M->ffa, T, L.ff, true, L.act, s, L.act_limit));
      }
      STEP(stack_linear(c, M->ffa, L.ff, W.mlp_down, M->y2, Wd, T, Wd, L.ff, s));
      y_prev = M->y2, scale_prev = W.scale_mlp, hc_prev = W.hc_mlp;
    } else {
      STEP(moe_route(f32, M->hn, W.router, W.router_bias, T, Wd, L.experts, L.top, 1, 1, M->route_ids, M->route_w, s, M->route_logits, c->lin_ws,
                     c->lin_ws_bytes, L.route_chosen ? 2 : (L.sigmoid_scores ? 1 : 0)));
      ExpertForm form;
      form.gated = !L.ungated;
      form.act = L.act;
      form.weight_input = L.weight_input != 0;
      form.limit = L.act_limit;
      STEP(moe_experts(f32, M->hn, W.e_gate_up, W.e_down, M->route_ids, M->route_w, T, Wd, L.ff, L.experts, L.top, M->parts, M->moe_ws, s, form));
      y_prev = nullptr, parts_prev = M->parts, n_parts_prev = L.top, scale_prev = W.scale_mlp, hc_prev = W.hc_mlp;
    }
  }
  if (M->tap) {   // the last layer's streams, closed over every row
    STEP(hyper_step(f32, X, sstride, n, false, y_prev, parts_prev, n_parts_prev, scale_prev, hc_prev, m.residual_mult, nullptr, nullptr, nullptr,
                    m.norm_eps, nullptr, nullptr, nullptr, M->tap + (int64_t)(nL - 1) * T * Wd, T, Wd, s));
    y_prev = nullptr, parts_prev = nullptr, hc_prev = nullptr;
  }
  // logit rows: the last close, the sum of the streams and the output norm over those rows only
  STEP(hyper_step(f32, X, sstride, n, false, y_prev, parts_prev, n_parts_prev, scale_prev, hc_prev, m.residual_mult, nullptr, M->final_norm,
                  M->final_norm_b, m.norm_eps, a.logit_rows, nullptr, M->lm_in, nullptr, a.R, Wd, s));
  STEP(stack_logits_f32(c, a, 0.f, s));
#undef STEP
  return B200_OK;
}

int stack_enqueue_step(b200_ctx* c, const StepArgs& a, cudaStream_t s) {
  StackModel* M = c->stack;
  const b200_stack_cfg& m = M->cfg;
  if (m.form == B200_FORM_PARALLEL) return stack_enqueue_step_parallel(c, a, s);
  if (m.form == B200_FORM_POSTNORM) return stack_enqueue_step_postnorm(c, a, s);
  if (m.form == B200_FORM_HYPER) return stack_enqueue_step_hyper(c, a, s);
  const bool f32 = m.f32 != 0;
  const int T = a.T, Wd = m.width, nL = m.n_layers;
  int rc;
#define STEP(expr)     \
  do {                 \
    rc = (expr);       \
    if (rc) return rc; \
  } while (0)
  // prefill-sized steps share K/V tiles between the rows of a run; the run list is built once per step
  int attn_plan = (a.row_to_seq && T >= 32 && (a.n_seqs > 0 ? T >= 2 * a.n_seqs : true)) ? 1 : 0;
  static const int plan_env = getenv("B200_STACK_ATTN_RUNS") ? atoi(getenv("B200_STACK_ATTN_RUNS")) : 1;
  if (!plan_env) attn_plan = 0;
  // the tensor-core kernels' view of the step (as in the fixed decoder stack): > 0 prefill-heavy, rows of a sequence
  // share a pass over its K/V (2: the row plan for `pack_group` query heads per kv head is in the workspace); -1 decode only
  int attn_pack = a.row_to_seq && (a.n_seqs > 0 ? (T >= 4 * a.n_seqs && T >= 32) : T >= 512);
  if (!attn_pack && (a.row_to_seq == nullptr || a.n_seqs == T)) attn_pack = -1;
  int pack_group = 0;
  STEP(embed_scaled(a.ids, M->embed, M->x, T, Wd, m.vocab, m.embed_scale, s, a.prev_tokens, a.n_prev));
  STEP(layernorm_stream(f32, M->x, nullptr, nullptr, 0, nullptr, M->w[0].n_mix_pre, M->hn, nullptr, T, Wd, m.norm_eps, s));
  for (int l = 0; l < nL; ++l) {
    const b200_stack_layer& L = M->layers[l];
    const StackLayerW& W = M->w[l];
    const float* next_pre = l + 1 < nL ? M->w[l + 1].n_mix_pre : nullptr;
    const int qr = qkv_rows(L);
    STEP(stack_linear(c, M->hn, Wd, W.qkv, M->qkv, qr, T, qr, Wd, s));
    const float* rot = L.rot_dims > 0 ? M->rot[L.rot_table] : nullptr;
    const float* vrot = L.vrot_table >= 0 ? M->rot[L.vrot_table] : nullptr;
    int64_t max_pos = 1ll << 40;
    if (rot) max_pos = std::min(max_pos, M->rot_pos[L.rot_table]);
    if (vrot) max_pos = std::min(max_pos, M->rot_pos[L.vrot_table]);
    if (layer_attn_tc(m, L)) {
      __nv_bfloat16* q16 = reinterpret_cast<__nv_bfloat16*>(M->q);
      STEP(qk_norm_rotate_cache(f32, M->qkv, W.q_norm, W.k_norm, a.positions, a.slots, rot, L.rot_dims, vrot, nullptr, W.kc, W.vc, T,
                                L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, m.norm_eps, max_pos, s, q16, kHeadDim, kHeadDim));
      __nv_bfloat16* wide = L.vdim == kHeadDim ? (__nv_bfloat16*)M->attn : (__nv_bfloat16*)M->attn_wide;
      int pack = attn_pack;
      if (pack > 0) {
        const int G = L.heads / L.kv_heads;
        if (pack_group != G) {
          const int built = paged_attn_prefill_plan_step(a.row_to_seq, a.ctx_lens, T, L.heads, L.kv_heads, m.block_size,
                                                         M->attn_tc_ws, M->attn_tc_ws_bytes, s);
          if (built < 0) return built;
          pack_group = built == 1 ? G : 0;
        }
        pack = pack_group == G ? 2 : 1;
      }
      STEP(paged_attn_ex(q16, L.heads * kHeadDim, (const __nv_bfloat16*)W.kc, (const __nv_bfloat16*)W.vc, a.block_table, a.bt_stride,
                         a.row_to_seq, a.ctx_lens, wide, L.heads * kHeadDim, T, L.heads, L.kv_heads, m.block_size, a.max_ctx,
                         L.scale, M->attn_tc_ws, M->attn_tc_ws_bytes, pack, s));
      if (vrot || L.vdim != kHeadDim)
        STEP(rotate_back_rows(wide, kHeadDim, (__nv_bfloat16*)M->attn, a.positions, vrot, T, L.heads, L.vdim, max_pos, s));
    } else {
      STEP(qk_norm_rotate_cache(f32, M->qkv, W.q_norm, W.k_norm, a.positions, a.slots, rot, L.rot_dims, vrot, M->q, W.kc, W.vc, T,
                                L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, m.norm_eps, max_pos, s));
      if (attn_plan == 1) {   // the run list, by a launch of its own (a layer's shape decides whether its kernel walks runs)
        STEP(paged_attn_runs_plan(a.row_to_seq, a.ctx_lens, T, M->attn_ws, s));
        attn_plan = 2;
      }
      STEP(paged_attn_anydim(f32, M->q, W.kc, W.vc, a.block_table, a.bt_stride, a.row_to_seq, a.ctx_lens, a.positions, vrot, max_pos,
                             M->attn, T, L.heads, L.kv_heads, L.dim, L.vdim, m.block_size, L.scale, attn_plan, M->attn_ws, s));
    }
    STEP(stack_linear(c, M->attn, L.heads * L.vdim, W.o, M->y, Wd, T, Wd, L.heads * L.vdim, s));
    if (L.mlp == B200_MLP_MOE) {
      STEP(layernorm_stream(f32, M->x, M->y, nullptr, 0, W.n_mix_post, W.n_mlp_pre, M->hn, nullptr, T, Wd, m.norm_eps, s));
      STEP(moe_route(f32, M->hn, W.router, W.router_bias, T, Wd, L.experts, L.top, L.groups, L.keep, M->route_ids, M->route_w, s,
                     M->route_logits, c->lin_ws, c->lin_ws_bytes));
      STEP(moe_experts(f32, M->hn, W.e_gate_up, W.e_down, M->route_ids, M->route_w, T, Wd, L.ff, L.experts, L.top, M->parts,
                       M->moe_ws, s));
      STEP(layernorm_stream(f32, M->x, nullptr, M->parts, L.top, W.n_mlp_post, next_pre, M->hn, nullptr, T, Wd, m.norm_eps, s));
    } else {
      STEP(layernorm_stream(f32, M->x, M->y, nullptr, 0, W.n_mix_post, next_pre, M->hn, nullptr, T, Wd, m.norm_eps, s));
    }
    if (M->tap)
      B200_CUDA(cudaMemcpyAsync(M->tap + (int64_t)l * T * Wd, M->x, (size_t)T * Wd * 4, cudaMemcpyDeviceToDevice, s));
  }
  // logit rows: final norm through the row indirection, output projection
  STEP(layernorm_stream(f32, M->x, nullptr, nullptr, 0, nullptr, M->final_norm, M->lm_in, a.logit_rows, a.R, Wd, m.norm_eps, s));
  if (f32) {
    STEP(linear_simt(true, true, M->lm_in, Wd, M->head, c->logits_f32, c->logits_ld, a.R, m.vocab, Wd, s));
    STEP(convert_f32_to_bf16(c->logits_f32, c->logits, (int64_t)a.R * c->logits_ld, s));
  } else {
    STEP(stack_linear(c, M->lm_in, Wd, M->head, c->logits, c->logits_ld, a.R, m.vocab, Wd, s));
  }
  STEP(argmax_rows(c->logits, c->logits_ld, a.R, m.vocab, 0, a.out_tokens, nullptr, s));
  if (a.out_logits)
    B200_CUDA(cudaMemcpy2DAsync(a.out_logits, (size_t)m.vocab * 2, c->logits, (size_t)c->logits_ld * 2, (size_t)m.vocab * 2, a.R,
                                cudaMemcpyDeviceToDevice, s));
#undef STEP
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_stack_create(const b200_stack_cfg* cfg, const b200_stack_layer* layers, b200_ctx** out) {
  B200_REQUIRE(cfg && layers && out, B200_ERR_INVALID, "stack_create: null argument");
  B200_REQUIRE(cfg->width > 0 && cfg->vocab > 0 && cfg->n_layers > 0 && cfg->block_size > 0 && cfg->max_tokens > 0 &&
                   cfg->max_blocks_per_seq > 0 && cfg->max_logit_rows > 0,
               B200_ERR_INVALID, "stack_create: bad sizes");
  int max_qkv = 0, max_q = 0, max_a = 0, max_top = 0, max_exp = 0, max_ff = 0, max_lat = 0, max_gates = 0, max_gu = 0, max_ffa = 0;
  int max_qrank = 0, max_qh = 0, max_dhd = 0, max_dqk = 0, max_dav = 0, max_dh = 0, max_heads = 0;
  int64_t moe_ws_bytes = 16;
  for (int l = 0; l < cfg->n_layers; ++l) {
    const b200_stack_layer& L = layers[l];
    if (cfg->form == B200_FORM_PARALLEL) {
      B200_REQUIRE(L.mixer == B200_MIXER_LATENT || L.mixer == B200_MIXER_MLSTM, B200_ERR_UNSUPPORTED,
                   "stack_create: layer %d: mixer %d is not served in the parallel form", l, L.mixer);
      B200_REQUIRE(L.heads > 0 && L.dim > 0 && L.vdim > 0, B200_ERR_INVALID, "stack_create: layer %d: bad mixer sizes", l);
      if (L.mixer == B200_MIXER_LATENT)
        B200_REQUIRE(L.kv_rank > 0 && L.rot_dim >= 0 && L.rot_dims >= 0 && L.rot_dims <= L.rot_dim && L.rot_dims % 2 == 0 &&
                         L.rot_table < 16 && L.kv_rank <= 512,
                     B200_ERR_INVALID, "stack_create: layer %d: bad latent sizes", l);
      else
        B200_REQUIRE(L.gate_cap > 0.f && L.dim <= 256 && cfg->n_state_slots > 0, B200_ERR_INVALID,
                     "stack_create: layer %d: bad recurrent sizes (or no state slots)", l);
      B200_REQUIRE(L.mlp == B200_MLP_NONE || L.mlp == B200_MLP_MOE || L.mlp == B200_MLP_DENSE, B200_ERR_UNSUPPORTED,
                   "stack_create: layer %d: unknown feed-forward %d", l, L.mlp);
      B200_REQUIRE(L.mlp == B200_MLP_NONE || (L.ff > 0 && L.act >= 0 && L.act <= B200_ACT_RELU && L.shared_ff >= 0), B200_ERR_INVALID,
                   "stack_create: layer %d: bad feed-forward sizes", l);
    } else if (cfg->form == B200_FORM_POSTNORM) {
      B200_REQUIRE(L.heads > 0 && L.dim > 0 && L.vdim > 0 && L.window >= 0, B200_ERR_INVALID, "stack_create: layer %d: bad mixer sizes", l);
      if (L.mixer == B200_MIXER_ATTENTION) {
        B200_REQUIRE((L.mixer_flags & B200_MIXF_HEAD_NORM) && (L.mixer_flags & B200_MIXF_VALUE_IS_KEY), B200_ERR_UNSUPPORTED,
                     "stack_create: layer %d: attention of the post-norm form has per-head norms and values that are its keys", l);
        B200_REQUIRE(L.kv_heads > 0 && L.heads % L.kv_heads == 0 && L.dim % 2 == 0 && L.vdim <= L.dim && L.rot_dims >= 0 &&
                         L.rot_dims <= L.dim && L.rot_dims % 2 == 0 && L.rot_table < 16,
                     B200_ERR_INVALID, "stack_create: layer %d: bad attention sizes", l);
      } else if (L.mixer == B200_MIXER_LATENT) {
        B200_REQUIRE(L.kv_rank > 0 && L.q_rank > 0 && L.rot_dim == 0 && L.rot_dims == 0 && L.kv_share >= 0 && L.kv_share <= l,
                     B200_ERR_INVALID, "stack_create: layer %d: bad latent sizes", l);
        if (L.kv_share > 0) {
          const b200_stack_layer& src = layers[L.kv_share - 1];
          B200_REQUIRE(src.mixer == B200_MIXER_LATENT && src.kv_share == 0 && src.kv_rank == L.kv_rank, B200_ERR_INVALID,
                       "stack_create: layer %d reads the latent rows of layer %d, which keeps none of that size", l, L.kv_share - 1);
        }
      } else if (L.mixer == B200_MIXER_DELTA) {
        B200_REQUIRE(L.kv_heads > 0 && L.heads % L.kv_heads == 0 && L.dim <= 256 && L.conv_taps >= 1 && L.conv_taps <= 64 &&
                         L.decay_rank > 0 && L.gate_rank > 0 && cfg->n_state_slots > 0,
                     B200_ERR_INVALID, "stack_create: layer %d: bad recurrent sizes (or no state slots)", l);
      } else {
        B200_REQUIRE(false, B200_ERR_UNSUPPORTED, "stack_create: layer %d: mixer %d is not served in the post-norm form", l, L.mixer);
      }
      B200_REQUIRE(L.mlp == B200_MLP_NONE || (L.mlp == B200_MLP_DENSE && L.ff > 0 && L.act >= 0 && L.act <= B200_ACT_RELU), B200_ERR_UNSUPPORTED,
                   "stack_create: layer %d: the post-norm form has dense feed-forwards", l);
    } else if (cfg->form == B200_FORM_HYPER) {
      B200_REQUIRE(L.heads > 0 && L.dim > 0 && L.vdim > 0 && L.window >= 0 && L.kv_heads > 0 && L.heads % L.kv_heads == 0, B200_ERR_INVALID,
                   "stack_create: layer %d: bad mixer sizes", l);
      if (L.mixer == B200_MIXER_ATTENTION) {
        B200_REQUIRE((L.mixer_flags & B200_MIXF_NO_QK_NORM) && !(L.mixer_flags & (B200_MIXF_HEAD_NORM | B200_MIXF_VALUE_IS_KEY)), B200_ERR_UNSUPPORTED,
                     "stack_create: layer %d: attention of the multi-stream form has plain q/k/v projections", l);
        B200_REQUIRE(L.rot_dims >= 0 && L.rot_dims <= L.dim && L.rot_dims % 2 == 0 && L.rot_table < 16, B200_ERR_INVALID,
                     "stack_create: layer %d: bad attention sizes", l);
      } else if (L.mixer == B200_MIXER_DELTA) {
        B200_REQUIRE(head_decay(L), B200_ERR_UNSUPPORTED, "stack_create: layer %d: the delta mixer of the multi-stream form has one decay per head", l);
        B200_REQUIRE(L.dim <= 256 && L.conv_taps >= 1 && L.conv_taps <= 64 && cfg->n_state_slots > 0, B200_ERR_INVALID,
                     "stack_create: layer %d: bad recurrent sizes (or no state slots)", l);
      } else if (L.mixer == B200_MIXER_SSD) {
        B200_REQUIRE(L.dim <= 256 && L.conv_taps >= 1 && L.conv_taps <= 64 && L.norm_groups >= 1 && (L.heads * L.vdim) % L.norm_groups == 0 &&
                         cfg->n_state_slots > 0,
                     B200_ERR_INVALID, "stack_create: layer %d: bad state-space sizes (or no state slots)", l);
      } else {
        B200_REQUIRE(false, B200_ERR_UNSUPPORTED, "stack_create: layer %d: mixer %d is not served in the multi-stream form", l, L.mixer);
      }
      B200_REQUIRE(L.mlp == B200_MLP_NONE || L.mlp == B200_MLP_MOE || L.mlp == B200_MLP_DENSE, B200_ERR_UNSUPPORTED,
                   "stack_create: layer %d: unknown feed-forward %d", l, L.mlp);
      B200_REQUIRE(L.mlp == B200_MLP_NONE || (L.ff > 0 && L.act >= 0 && L.act <= B200_ACT_POLYNORM && !L.shared_ff), B200_ERR_INVALID,
                   "stack_create: layer %d: bad feed-forward sizes", l);
      B200_REQUIRE(L.act != B200_ACT_POLYNORM || (L.mlp == B200_MLP_DENSE && L.ungated), B200_ERR_UNSUPPORTED,
                   "stack_create: layer %d: the polynomial activation belongs to an ungated dense feed-forward", l);
      B200_REQUIRE(L.act != B200_ACT_SWIGLU_CLAMP || (!L.ungated && L.act_limit > 0.f), B200_ERR_INVALID,
                   "stack_create: layer %d: the clamped gate needs a gate projection and a positive limit", l);
    } else {
    B200_REQUIRE(L.mixer == B200_MIXER_ATTENTION, B200_ERR_UNSUPPORTED, "stack_create: layer %d: unknown mixer %d", l, L.mixer);
    B200_REQUIRE(L.heads > 0 && L.kv_heads > 0 && L.heads % L.kv_heads == 0 && L.dim > 0 && L.vdim > 0 && L.dim % 2 == 0 &&
                     L.rot_dims >= 0 && L.rot_dims <= L.dim && L.rot_dims % 2 == 0 && (L.vrot_table < 0 || L.vdim % 2 == 0) &&
                     L.rot_table < 16 && L.vrot_table < 16,
                 B200_ERR_INVALID, "stack_create: layer %d: bad attention sizes", l);
    B200_REQUIRE(L.mlp == B200_MLP_NONE || L.mlp == B200_MLP_MOE, B200_ERR_UNSUPPORTED, "stack_create: layer %d: unknown feed-forward %d", l, L.mlp);
    B200_REQUIRE(!L.ungated && !L.sigmoid_scores && !L.weight_input && !L.shared_ff && L.act == B200_ACT_SILU, B200_ERR_UNSUPPORTED,
                 "stack_create: layer %d: this feed-forward shape is served in the parallel form only", l);
    }
    if (L.mlp == B200_MLP_MOE) {
      const int groups = L.groups < 1 ? 1 : L.groups;
      B200_REQUIRE(L.experts > 0 && L.top > 0 && L.top <= L.experts && L.ff > 0 && L.experts % groups == 0 && L.keep >= 1 &&
                       L.keep <= groups && L.top <= L.keep * (L.experts / groups),
                   B200_ERR_INVALID, "stack_create: layer %d: bad router sizes", l);
      max_top = std::max(max_top, L.top);
      max_exp = std::max(max_exp, L.experts);
      max_ff = std::max(max_ff, L.ff);
      moe_ws_bytes = std::max(moe_ws_bytes, moe_workspace_bytes(cfg->max_tokens, L.top, L.experts, cfg->f32 ? 0 : cfg->width, L.ff));
    }
    max_qkv = std::max(max_qkv, qkv_rows(L));
    max_q = std::max(max_q, L.heads * (is_latent(L) ? L.kv_rank + L.rot_dim : L.dim));
    max_a = std::max(max_a, L.heads * L.vdim);
    if (is_latent(L)) max_lat = std::max(max_lat, L.heads * L.kv_rank);
    if (is_mlstm(L)) max_gates = std::max(max_gates, 2 * L.heads);
    max_heads = std::max(max_heads, L.heads);
    if (is_latent(L) && L.q_rank > 0) max_qrank = std::max(max_qrank, L.q_rank), max_qh = std::max(max_qh, L.heads * L.dim);
    if (is_delta(L) || is_ssd(L)) {
      max_dhd = std::max(max_dhd, L.heads * (head_decay(L) || is_ssd(L) ? 1 : L.dim));
      max_dqk = std::max(max_dqk, L.kv_heads * L.dim);
      max_dav = std::max(max_dav, L.heads * L.vdim);
      max_dh = std::max(max_dh, L.heads);
    }
    if (L.mlp == B200_MLP_DENSE) max_gu = std::max(max_gu, (L.ungated ? 1 : 2) * L.ff), max_ffa = std::max(max_ffa, L.ff);
    if (L.shared_ff > 0) max_gu = std::max(max_gu, 2 * L.shared_ff), max_ffa = std::max(max_ffa, L.shared_ff);
  }
  const bool par = cfg->form == B200_FORM_PARALLEL, post = cfg->form == B200_FORM_POSTNORM, hyp = cfg->form == B200_FORM_HYPER;
  B200_REQUIRE(par || ((hyp || !cfg->canon_taps) && !cfg->depth_avg && !cfg->bigram_buckets && cfg->logit_softcap == 0.f), B200_ERR_UNSUPPORTED,
               "stack_create: depth average, bigram rows and the logit cap belong to the parallel form, the input convolution to it and the multi-stream form");
  B200_REQUIRE(!hyp || (cfg->streams >= 1 && cfg->streams <= B200_MAX_STREAMS && cfg->canon_taps >= 0 && cfg->canon_taps <= 16 &&
                        (cfg->canon_taps <= 1 || cfg->n_state_slots > 0)),
               B200_ERR_INVALID, "stack_create: bad stream count or convolution taps, or no state slots");
  B200_REQUIRE(!par || (cfg->canon_taps >= 0 && cfg->canon_taps <= 16 && cfg->n_state_slots >= 0 &&
                        ((cfg->canon_taps <= 1 && cfg->bigram_buckets <= 0) || cfg->n_state_slots > 0)),
               B200_ERR_INVALID, "stack_create: bad convolution taps or no state slots");
  b200_ctx* c = new b200_ctx();
  StackModel* M = new StackModel();
  c->stack = M;
  M->cfg = *cfg;
  M->layers.assign(layers, layers + cfg->n_layers);
  M->w.resize(cfg->n_layers);
  M->esz = cfg->f32 ? 4 : 2;
  if (par && cfg->n_state_slots > 0) {
    // one slot: [previous token (int32) + padding to 4 floats | per layer: convolution tail [taps - 1][width], recurrent state]
    int64_t off = 4;
    for (int l = 0; l < cfg->n_layers; ++l) {
      if (cfg->canon_taps > 1) {
        M->w[l].tail_off = off;
        off += (int64_t)(cfg->canon_taps - 1) * cfg->width;
      }
      if (is_mlstm(layers[l])) {
        M->w[l].rec_off = off;
        off += mlstm_state_floats(layers[l].heads, layers[l].dim, layers[l].vdim);
      }
      off = up(off, 4);
    }
    M->slot_floats = off;
  }
  if (post && cfg->n_state_slots > 0) {
    // one slot: per delta layer the convolution tail [taps - 1][q | k | v channels], then the state [heads][vdim][dim]
    int64_t off = 0;
    for (int l = 0; l < cfg->n_layers; ++l) {
      const b200_stack_layer& L = layers[l];
      if (!is_delta(L)) continue;
      M->w[l].tail_off = off;
      off = up(off + delta_tail_floats(L.heads, L.kv_heads, L.dim, L.vdim, L.conv_taps), 4);
      M->w[l].rec_off = off;
      off = up(off + delta_state_floats(L.heads, L.dim, L.vdim), 4);
    }
    M->slot_floats = std::max<int64_t>(off, 4);
  }
  if (hyp && cfg->n_state_slots > 0) {
    // one slot, per layer: the tails of the two input convolutions [taps - 1][width] (the second only with a feed-forward), then for
    // a recurrent mixer the tail of its own convolution [conv_taps - 1][channels] and its state [heads][vdim][dim]
    int64_t off = 0;
    for (int l = 0; l < cfg->n_layers; ++l) {
      const b200_stack_layer& L = layers[l];
      if (cfg->canon_taps > 1) {
        M->w[l].tail_off = off;
        off += (int64_t)(cfg->canon_taps - 1) * cfg->width;
        if (L.mlp != B200_MLP_NONE) {
          M->w[l].tail2_off = off;
          off += (int64_t)(cfg->canon_taps - 1) * cfg->width;
        }
      }
      if (is_delta(L) || is_ssd(L)) {
        M->w[l].ctail_off = off;
        off = up(off + (is_delta(L) ? delta_tail_floats(L.heads, L.kv_heads, L.dim, L.vdim, L.conv_taps)
                                    : ssd_tail_floats(L.heads, L.kv_heads, L.dim, L.vdim, L.conv_taps)), 4);
        M->w[l].rec_off = off;
        off = up(off + delta_state_floats(L.heads, L.dim, L.vdim), 4);
      }
    }
    M->slot_floats = std::max<int64_t>(off, 4);
  }
  b200_model_cfg& mc = c->cfg;
  memset(&mc, 0, sizeof(mc));
  mc.hidden = cfg->width;
  mc.n_layers = cfg->n_layers;
  mc.vocab = cfg->vocab;
  mc.rms_eps = cfg->norm_eps;
  mc.block_size = cfg->block_size;
  mc.max_tokens = cfg->max_tokens;
  mc.max_blocks_per_seq = cfg->max_blocks_per_seq;
  mc.tp_rank = 0;
  mc.tp_world = 1;
  c->hq = c->hkv = c->inter = c->qkv_w = 0;
  c->vocab_local = cfg->vocab;
  c->logits_ld = (int)up(cfg->vocab, 8);
  c->max_logit_rows = std::min(cfg->max_logit_rows, cfg->max_tokens);
  if (const char* e = getenv("B200_GRAPHS")) c->graphs = atoi(e) != 0;
  if (const char* e = getenv("B200_PDL")) c->pdl = atoi(e) != 0;
  c->x = c->res = c->normed = c->qkv_buf = c->attn_out = c->gu_buf = c->act = c->lm_in = nullptr;
  c->sres = c->ssq = nullptr;
  c->attn_ws = nullptr;
  c->attn_ws_bytes = 0;
  c->d_pairs = c->d_gathered = nullptr;
  c->logits_full = nullptr;

  const int64_t T = cfg->max_tokens, Wd = cfg->width, R = c->max_logit_rows, es = M->esz;
  int64_t lw = 0;
  if (!cfg->f32) {
    // the shapes of this model's linears over the row counts where the tcgen05 plan changes
    std::vector<std::pair<int, int>> shapes;   // (n_out, k)
    for (int l = 0; l < cfg->n_layers; ++l) {
      shapes.push_back({qkv_rows(layers[l]), (int)Wd});
      shapes.push_back({(int)Wd, layers[l].heads * layers[l].vdim});
      if (layers[l].mlp == B200_MLP_MOE) shapes.push_back({layers[l].experts, (int)Wd});
      if (layers[l].mlp == B200_MLP_DENSE) {
        shapes.push_back({(layers[l].ungated ? 1 : 2) * layers[l].ff, (int)Wd});
        shapes.push_back({(int)Wd, layers[l].ff});
      }
      if (layers[l].shared_ff > 0) {
        shapes.push_back({(layers[l].ungated ? 1 : 2) * layers[l].shared_ff, (int)Wd});
        shapes.push_back({(int)Wd, layers[l].shared_ff});
      }
      if (is_latent(layers[l]) && layers[l].q_rank > 0) shapes.push_back({layers[l].heads * layers[l].dim, layers[l].q_rank});
      if (is_delta(layers[l])) {
        shapes.push_back({layers[l].heads * layers[l].dim, layers[l].decay_rank});
        shapes.push_back({layers[l].heads * layers[l].vdim, layers[l].gate_rank});
      }
    }
    for (auto& sh : shapes) {
      if (sh.second % 8) continue;
      for (int t = 1; t <= T; t = (t < 16 ? 16 : (t % 2 == 0 ? t + 1 : (t - 1) * 2)))
        lw = std::max<int64_t>(lw, linear_tc_workspace_bytes(t, sh.first, sh.second));
      lw = std::max<int64_t>(lw, linear_tc_workspace_bytes((int)T, sh.first, sh.second));
    }
    if (Wd % 8 == 0) {
      for (int t = 1; t <= R; t = (t < 16 ? 16 : (t % 2 == 0 ? t + 1 : (t - 1) * 2)))
        lw = std::max<int64_t>(lw, linear_tc_workspace_bytes(t, cfg->vocab, (int)Wd));
      lw = std::max<int64_t>(lw, linear_tc_workspace_bytes((int)R, cfg->vocab, (int)Wd));
    }
  }
  c->lin_ws_bytes = std::max<int64_t>(lw, 64 * 1024);
  c->meta_ints = 7 * T + T * cfg->max_blocks_per_seq;
  const int64_t attn_ws_bytes = paged_attn_anydim_workspace_bytes((int)T);
  int tc_heads = 0;
  for (int l = 0; l < cfg->n_layers; ++l)
    if (layer_attn_tc(*cfg, layers[l])) {
      tc_heads = std::max(tc_heads, layers[l].heads);
      max_q = std::max(max_q, layers[l].heads * kHeadDim / 2);   // bf16 queries of 128 in the fp32 query buffer
    }
  M->attn_tc_ws_bytes = 16;
  if (tc_heads) {
    int max_ctx = 128;   // graph replay rounds a step's longest context up to a power of two
    while (max_ctx < cfg->max_blocks_per_seq * cfg->block_size) max_ctx *= 2;
    for (int t = 1; t <= T; t = t < 64 ? t + 1 : t * 2)   // the bound is not monotone in T: scan
      M->attn_tc_ws_bytes = std::max(M->attn_tc_ws_bytes, paged_attn_workspace_bytes(t, tc_heads, max_ctx, cfg->block_size));
    M->attn_tc_ws_bytes = std::max(M->attn_tc_ws_bytes, paged_attn_workspace_bytes((int)T, tc_heads, max_ctx, cfg->block_size));
  }

  M->lat_ws_bytes = 16;
  if ((par || post) && !cfg->f32)
    for (int l = 0; l < cfg->n_layers; ++l)
      if (is_latent(layers[l]) && latent_attn_mma_supported(layers[l].heads, layers[l].kv_rank + layers[l].rot_dim, layers[l].kv_rank))
        // splitting only happens below one CTA per SM: at most 148 * 16 pairs, 16 splits
        M->lat_ws_bytes = std::max<int64_t>(M->lat_ws_bytes, std::min<int64_t>(T * layers[l].heads, 148 * 16) * 16 * (layers[l].kv_rank + 2) * 4);
  if ((post || hyp) && !cfg->f32)
    for (int l = 0; l < cfg->n_layers; ++l)
      if (layers[l].mixer == B200_MIXER_ATTENTION && paged_attn_mma_supported(layers[l].heads, layers[l].kv_heads, layers[l].dim, layers[l].vdim))
        M->lat_ws_bytes = std::max<int64_t>(M->lat_ws_bytes, std::min<int64_t>(T * layers[l].heads, 148 * 16) * 16 * (layers[l].vdim + 2) * 4);
  struct Item {
    void** p;
    int64_t bytes;
  };
  std::vector<Item> items = {
      {(void**)&M->x, T * Wd * 4},
      {(void**)&M->hn, T * Wd * es},
      {(void**)&M->qkv, T * max_qkv * es},
      {(void**)&M->q, T * max_q * 4},
      {(void**)&M->attn, T * max_a * es},
      {(void**)&M->y, T * Wd * es},
      {(void**)&M->route_ids, T * std::max(max_top, 1) * 4},
      {(void**)&M->route_w, T * std::max(max_top, 1) * 4},
      {(void**)&M->parts, T * std::max(max_top, 1) * Wd * 4},
      {(void**)&M->route_logits, T * std::max(max_exp, 1) * 4},
      {(void**)&M->lm_in, R * Wd * es},
      {(void**)&M->attn_ws, attn_ws_bytes},
      {(void**)&M->moe_ws, moe_ws_bytes},
      {(void**)&M->attn_tc_ws, M->attn_tc_ws_bytes},
      {(void**)&M->attn_wide, tc_heads ? T * tc_heads * kHeadDim * 2 : 16},
      {(void**)&c->logits, R * (int64_t)c->logits_ld * 2},
      {(void**)&c->logits_f32, (cfg->f32 || par || post || hyp) ? R * (int64_t)c->logits_ld * 4 : 16},
      {(void**)&M->results, par && cfg->depth_avg ? (int64_t)(cfg->n_layers + 1) * T * Wd * 4 : 16},
      {(void**)&M->h1f, (par || hyp) && cfg->canon_taps >= 1 ? T * Wd * 4 : 16},
      {(void**)&M->hc, (par || hyp) ? T * Wd * es : 16},
      {(void**)&M->xs, hyp ? (int64_t)cfg->streams * T * Wd * 4 : 16},
      {(void**)&M->lat, T * std::max(max_lat, 1) * es},
      {(void**)&M->y2, (par || post || hyp) ? T * Wd * es : 16},
      {(void**)&M->y3, par ? T * Wd * es : 16},
      {(void**)&M->gu, T * std::max(max_gu, 1) * es},
      {(void**)&M->ffa, T * std::max(max_ffa, 1) * es},
      {(void**)&M->gates_buf, T * std::max(max_gates, 1) * 4},
      {(void**)&M->oraw, (max_gates || max_dav) ? T * max_a * 4 : 16},
      {(void**)&M->head_f32, (par || post || hyp) ? R * (int64_t)cfg->vocab * 4 : 16},
      {(void**)&M->seq_start, (T + 2) * 4},
      {(void**)&M->cq, T * std::max(max_qrank, 1) * es},
      {(void**)&M->qh, T * std::max(max_qh, 1) * es},
      {(void**)&M->a2, T * std::max(max_dhd, 1) * es},
      {(void**)&M->g2, T * std::max(max_dav, 1) * es},
      {(void**)&M->dq, T * std::max(max_dqk, 1) * 4},
      {(void**)&M->dk, T * std::max(max_dqk, 1) * 4},
      {(void**)&M->dv, T * std::max(max_dav, 1) * 4},
      {(void**)&M->dbeta, T * std::max(max_dh, 1) * 4},
      {(void**)&M->ddecay, T * std::max(max_dhd, 1) * 4},
      {(void**)&M->zero_sink, std::max(max_heads, 1) * 4},
      {(void**)&M->lat_ws, M->lat_ws_bytes},
      {(void**)&c->lin_ws, c->lin_ws_bytes},
      {(void**)&c->d_meta, c->meta_ints * 4},
      {(void**)&c->d_tokens, R * 4},
      {(void**)&c->d_max, R * 4},
      {(void**)&c->d_sample, R * 40},
      {(void**)&c->d_logprob, R * (8 + 32 * 8)},
      {(void**)&c->d_adjust, (4ll << 20) * 4},
  };
  (void)max_ff;
  int64_t total = 0;
  for (auto& it : items) total += up(std::max<int64_t>(it.bytes, 16), 1024);
  cudaError_t e = cudaMalloc(&c->pool, total);
  if (e == cudaSuccess) e = cudaMemset(c->pool, 0, total);
  if (e != cudaSuccess) {
    if (c->pool) cudaFree(c->pool);
    delete M;
    delete c;
    return cuda_fail(e, "cudaMalloc(ctx pool)", __FILE__, __LINE__);
  }
  c->pool_bytes = total;
  int64_t off = 0;
  for (auto& it : items) {
    *it.p = static_cast<char*>(c->pool) + off;
    off += up(std::max<int64_t>(it.bytes, 16), 1024);
  }
  if (!cfg->f32 && !par && !post && !hyp) c->logits_f32 = nullptr;
  *out = c;
  return B200_OK;
}

extern "C" int b200_stack_set_weight(b200_ctx* c, int32_t layer, int32_t kind, const void* w, int64_t rows, int64_t cols) {
  B200_REQUIRE(c && c->stack && w, B200_ERR_INVALID, "stack_set_weight: null argument or not a layer-list ctx");
  B200_REQUIRE(reinterpret_cast<uintptr_t>(w) % 16 == 0, B200_ERR_INVALID, "stack_set_weight: pointer not 16-byte aligned");
  StackModel* M = c->stack;
  const int64_t Wd = M->cfg.width, V = M->cfg.vocab;
  int64_t er = 0, ec = 1;
  const bool par = M->cfg.form == B200_FORM_PARALLEL;
  const bool post = M->cfg.form == B200_FORM_POSTNORM;
  const bool hyp = M->cfg.form == B200_FORM_HYPER;
  const bool global = kind == B200_SW_EMBED || kind == B200_SW_FINAL_NORM || kind == B200_SW_HEAD || kind == B200_SW_BIGRAM ||
                      kind == B200_SW_FINAL_NORM_BIAS;
  if (!global) B200_REQUIRE(layer >= 0 && layer < M->cfg.n_layers, B200_ERR_INVALID, "stack_set_weight: layer %d out of range", layer);
  const b200_stack_layer L = global ? b200_stack_layer{} : M->layers[layer];
  switch (kind) {
    case B200_SW_EMBED: case B200_SW_HEAD: er = V; ec = Wd; break;
    case B200_SW_FINAL_NORM: case B200_SW_NORM_MIX_PRE: case B200_SW_NORM_MIX_POST: case B200_SW_NORM_MLP_PRE:
    case B200_SW_NORM_MLP_POST: er = par ? 1 : Wd; break;
    case B200_SW_QKV: er = qkv_rows(L); ec = Wd; break;
    case B200_SW_Q_NORM: er = (L.mixer_flags & B200_MIXF_HEAD_NORM) ? L.dim : (int64_t)L.heads * L.dim; break;
    case B200_SW_K_NORM: er = is_latent(L) ? L.kv_rank : ((L.mixer_flags & B200_MIXF_HEAD_NORM) ? L.dim : (int64_t)L.kv_heads * L.dim); break;
    case B200_SW_NORM_MIX_POST_BIAS: case B200_SW_NORM_MLP_POST_BIAS: case B200_SW_FINAL_NORM_BIAS: er = Wd; break;
    case B200_SW_Q_LATENT_NORM: er = L.q_rank; break;
    case B200_SW_UQ: er = (int64_t)L.heads * L.dim; ec = L.q_rank; break;
    case B200_SW_CONV: er = 2 * (int64_t)L.kv_heads * L.dim + (int64_t)L.heads * L.vdim; ec = L.conv_taps; break;
    case B200_SW_CONV_BIAS: er = 2 * (int64_t)L.kv_heads * L.dim + (int64_t)L.heads * L.vdim; break;
    case B200_SW_DECAY_UP: er = (int64_t)L.heads * L.dim; ec = L.decay_rank; break;
    case B200_SW_DECAY_BIAS: er = (head_decay(L) || is_ssd(L)) ? L.heads : (int64_t)L.heads * L.dim; break;
    case B200_SW_NORM_MIX_PRE_BIAS: case B200_SW_NORM_MLP_PRE_BIAS: case B200_SW_SCALE_MIX: case B200_SW_SCALE_MLP: er = Wd; break;
    case B200_SW_HC_MIX: case B200_SW_HC_MLP: er = (int64_t)M->cfg.streams * (2 + M->cfg.streams); break;
    case B200_SW_CANON_MLP: er = Wd; ec = M->cfg.canon_taps; break;
    case B200_SW_SKIP: er = L.heads; break;
    case B200_SW_MLP_ACT: er = 4; break;
    case B200_SW_DECAY_LOG: er = L.heads; break;
    case B200_SW_GATE_UP: er = (int64_t)L.heads * L.vdim; ec = L.gate_rank; break;
    case B200_SW_O: er = Wd; ec = (int64_t)L.heads * L.vdim; break;
    case B200_SW_ROUTER: er = L.experts; ec = Wd; break;
    case B200_SW_ROUTER_BIAS: er = L.experts; break;
    case B200_SW_EXPERT_GATE_UP: er = (int64_t)L.experts * (L.ungated ? 1 : 2) * L.ff; ec = Wd; break;
    case B200_SW_EXPERT_DOWN: er = (int64_t)L.experts * Wd; ec = L.ff; break;
    case B200_SW_BIGRAM: er = (int64_t)M->cfg.bigram_buckets + 1; ec = Wd; break;
    case B200_SW_CANON: er = Wd; ec = M->cfg.canon_taps; break;
    case B200_SW_DEPTH_AVG: er = layer + 2; break;
    case B200_SW_UK_T: er = (int64_t)L.heads * L.kv_rank; ec = L.dim; break;
    case B200_SW_UV: er = (int64_t)L.heads * L.vdim; ec = L.kv_rank; break;
    case B200_SW_SINK: er = L.heads; break;
    case B200_SW_GATES: er = 2 * (int64_t)L.heads; ec = Wd; break;
    case B200_SW_GATES_BIAS: er = 2 * (int64_t)L.heads; break;
    case B200_SW_HEAD_NORM: er = (int64_t)L.heads * L.vdim; break;
    case B200_SW_MLP_GATE_UP: er = (int64_t)(L.ungated ? 1 : 2) * L.ff; ec = Wd; break;
    case B200_SW_MLP_GATE_UP_INTERLEAVED: er = 2 * (int64_t)L.ff; ec = Wd; break;
    case B200_SW_MLP_DOWN: er = Wd; ec = L.ff; break;
    case B200_SW_SHARED_UP: er = (int64_t)(L.ungated ? 1 : 2) * L.shared_ff; ec = Wd; break;
    case B200_SW_SHARED_DOWN: er = Wd; ec = L.shared_ff; break;
    default: B200_REQUIRE(false, B200_ERR_INVALID, "stack_set_weight: unknown kind %d", kind);
  }
  B200_REQUIRE(kind < B200_SW_BIGRAM || par || post || hyp, B200_ERR_INVALID, "stack_set_weight: kind %d belongs to another layer form", kind);
  B200_REQUIRE(kind < B200_SW_NORM_MIX_POST_BIAS || post || hyp || kind == B200_SW_MLP_GATE_UP_INTERLEAVED, B200_ERR_INVALID,
               "stack_set_weight: kind %d belongs to the post-norm form", kind);
  B200_REQUIRE(kind < B200_SW_NORM_MIX_PRE_BIAS || hyp, B200_ERR_INVALID, "stack_set_weight: kind %d belongs to the multi-stream form", kind);
  if (kind == B200_SW_CONV_BIAS || kind == B200_SW_SKIP)
    B200_REQUIRE(is_ssd(L), B200_ERR_INVALID, "stack_set_weight: layer %d has no state-space mixer", layer);
  if (kind == B200_SW_MLP_ACT)
    B200_REQUIRE(L.mlp == B200_MLP_DENSE && L.act == B200_ACT_POLYNORM, B200_ERR_INVALID, "stack_set_weight: layer %d has no polynomial activation", layer);
  if (kind == B200_SW_MLP_GATE_UP_INTERLEAVED) B200_REQUIRE(!L.ungated, B200_ERR_INVALID, "stack_set_weight: layer %d has no gate rows to interleave", layer);
  if (kind == B200_SW_Q_LATENT_NORM || kind == B200_SW_UQ)
    B200_REQUIRE(is_latent(L) && L.q_rank > 0, B200_ERR_INVALID, "stack_set_weight: layer %d has no query latent", layer);
  if (kind >= B200_SW_CONV && kind <= B200_SW_GATE_UP)
    B200_REQUIRE((is_delta(L) && (!head_decay(L) || (kind != B200_SW_DECAY_UP && kind != B200_SW_GATE_UP))) ||
                     (is_ssd(L) && (kind == B200_SW_CONV || kind == B200_SW_DECAY_BIAS || kind == B200_SW_DECAY_LOG)),
                 B200_ERR_INVALID, "stack_set_weight: layer %d has no recurrence that takes kind %d", layer, kind);
  if (kind == B200_SW_UK_T || kind == B200_SW_UV)
    B200_REQUIRE(is_latent(L), B200_ERR_INVALID, "stack_set_weight: layer %d has no latent attention", layer);
  if (kind == B200_SW_SINK)
    B200_REQUIRE(is_latent(L) || (L.mixer == B200_MIXER_ATTENTION && (L.mixer_flags & B200_MIXF_SINK)), B200_ERR_INVALID,
                 "stack_set_weight: layer %d has no sink", layer);
  if (kind == B200_SW_GATES || kind == B200_SW_GATES_BIAS || kind == B200_SW_HEAD_NORM)
    B200_REQUIRE(is_mlstm(L) || ((is_delta(L) || is_ssd(L)) && kind == B200_SW_HEAD_NORM), B200_ERR_INVALID, "stack_set_weight: layer %d has no recurrence", layer);
  if (kind == B200_SW_MLP_GATE_UP_INTERLEAVED)
    B200_REQUIRE(!M->cfg.f32 && L.ff % 64 == 0 && Wd % 8 == 0, B200_ERR_UNSUPPORTED,
                 "stack_set_weight: interleaved gate|up rows need the bf16 mode, ff %% 64 == 0 and width %% 8 == 0");
  if (kind == B200_SW_MLP_GATE_UP || kind == B200_SW_MLP_DOWN || kind == B200_SW_MLP_GATE_UP_INTERLEAVED)
    B200_REQUIRE(L.mlp == B200_MLP_DENSE, B200_ERR_INVALID, "stack_set_weight: layer %d has no dense feed-forward", layer);
  B200_REQUIRE(rows == er && cols == ec, B200_ERR_INVALID, "stack_set_weight: kind %d of layer %d expects [%lld,%lld], got [%lld,%lld]",
               kind, layer, (long long)er, (long long)ec, (long long)rows, (long long)cols);
  if ((kind >= B200_SW_ROUTER && kind <= B200_SW_EXPERT_DOWN && kind != B200_SW_ROUTER_BIAS) || kind == B200_SW_SHARED_UP ||
      kind == B200_SW_SHARED_DOWN)
    B200_REQUIRE(L.mlp == B200_MLP_MOE, B200_ERR_INVALID, "stack_set_weight: layer %d has no routed experts", layer);
  const float* f = static_cast<const float*>(w);
  const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(w);
  switch (kind) {
    case B200_SW_EMBED: M->embed = b; break;
    case B200_SW_HEAD: M->head = b; break;
    case B200_SW_FINAL_NORM: M->final_norm = f; break;
    case B200_SW_NORM_MIX_PRE: M->w[layer].n_mix_pre = f; break;
    case B200_SW_NORM_MIX_POST: M->w[layer].n_mix_post = f; break;
    case B200_SW_NORM_MLP_PRE: M->w[layer].n_mlp_pre = f; break;
    case B200_SW_NORM_MLP_POST: M->w[layer].n_mlp_post = f; break;
    case B200_SW_QKV: M->w[layer].qkv = b; break;
    case B200_SW_Q_NORM: M->w[layer].q_norm = f; break;
    case B200_SW_K_NORM: M->w[layer].k_norm = f; break;
    case B200_SW_O: M->w[layer].o = b; break;
    case B200_SW_ROUTER: M->w[layer].router = b; break;
    case B200_SW_ROUTER_BIAS: M->w[layer].router_bias = f; break;
    case B200_SW_EXPERT_GATE_UP: M->w[layer].e_gate_up = b; break;
    case B200_SW_EXPERT_DOWN: M->w[layer].e_down = b; break;
    case B200_SW_BIGRAM: M->bigram = b; break;
    case B200_SW_CANON: M->w[layer].canon = f; break;
    case B200_SW_DEPTH_AVG: M->w[layer].dwa = f; break;
    case B200_SW_UK_T: M->w[layer].uk_t = b; break;
    case B200_SW_UV: M->w[layer].uv = b; break;
    case B200_SW_SINK: M->w[layer].sink = f; break;
    case B200_SW_GATES: M->w[layer].gates = b; break;
    case B200_SW_GATES_BIAS: M->w[layer].gates_bias = f; break;
    case B200_SW_HEAD_NORM: M->w[layer].head_norm = f; break;
    case B200_SW_MLP_GATE_UP: M->w[layer].mlp_gate_up = b; M->w[layer].gu_interleaved = false; break;
    case B200_SW_MLP_GATE_UP_INTERLEAVED: M->w[layer].mlp_gate_up = b; M->w[layer].gu_interleaved = true; break;
    case B200_SW_MLP_DOWN: M->w[layer].mlp_down = b; break;
    case B200_SW_SHARED_UP: M->w[layer].shared_up = b; break;
    case B200_SW_SHARED_DOWN: M->w[layer].shared_down = b; break;
    case B200_SW_NORM_MIX_POST_BIAS: M->w[layer].n_mix_post_b = f; break;
    case B200_SW_NORM_MLP_POST_BIAS: M->w[layer].n_mlp_post_b = f; break;
    case B200_SW_FINAL_NORM_BIAS: M->final_norm_b = f; break;
    case B200_SW_Q_LATENT_NORM: M->w[layer].q_lat_norm = f; break;
    case B200_SW_UQ: M->w[layer].uq = b; break;
    case B200_SW_CONV: M->w[layer].conv = f; break;
    case B200_SW_DECAY_UP: M->w[layer].decay_up = b; break;
    case B200_SW_DECAY_BIAS: M->w[layer].decay_bias = f; break;
    case B200_SW_DECAY_LOG: M->w[layer].decay_log = f; break;
    case B200_SW_GATE_UP: M->w[layer].gate_up = b; break;
    case B200_SW_NORM_MIX_PRE_BIAS: M->w[layer].n_mix_pre_b = f; break;
    case B200_SW_NORM_MLP_PRE_BIAS: M->w[layer].n_mlp_pre_b = f; break;
    case B200_SW_SCALE_MIX: M->w[layer].scale_mix = f; break;
    case B200_SW_SCALE_MLP: M->w[layer].scale_mlp = f; break;
    case B200_SW_HC_MIX: M->w[layer].hc_mix = f; break;
    case B200_SW_HC_MLP: M->w[layer].hc_mlp = f; break;
    case B200_SW_CANON_MLP: M->w[layer].canon_mlp = f; break;
    case B200_SW_CONV_BIAS: M->w[layer].conv_b = f; break;
    case B200_SW_SKIP: M->w[layer].skip = f; break;
    case B200_SW_MLP_ACT: M->w[layer].mlp_act = f; break;
  }
  return B200_OK;
}

extern "C" int b200_stack_set_kv_cache(b200_ctx* c, int32_t layer, void* k_cache, void* v_cache, int64_t n_blocks) {
  B200_REQUIRE(c && c->stack && k_cache && n_blocks > 0, B200_ERR_INVALID, "stack_set_kv_cache: bad argument");
  StackModel* M = c->stack;
  B200_REQUIRE(layer >= 0 && layer < M->cfg.n_layers, B200_ERR_INVALID, "stack_set_kv_cache: layer %d out of range", layer);
  B200_REQUIRE(v_cache || cache_vdim(M->cfg, M->layers[layer]) == 0, B200_ERR_INVALID, "stack_set_kv_cache: layer %d needs a value cache", layer);
  B200_REQUIRE(M->n_blocks == 0 || M->n_blocks == n_blocks, B200_ERR_INVALID, "stack_set_kv_cache: every layer needs the same block count");
  M->n_blocks = n_blocks;
  c->n_blocks = n_blocks;
  M->w[layer].kc = k_cache;
  M->w[layer].vc = v_cache;
  return B200_OK;
}

extern "C" int b200_stack_cache_dims(b200_ctx* c, int32_t layer, int32_t* k_dim, int32_t* v_dim) {
  B200_REQUIRE(c && c->stack && k_dim && v_dim, B200_ERR_INVALID, "stack_cache_dims: bad argument");
  StackModel* M = c->stack;
  B200_REQUIRE(layer >= 0 && layer < M->cfg.n_layers, B200_ERR_INVALID, "stack_cache_dims: layer %d out of range", layer);
  *k_dim = cache_kdim(M->cfg, M->layers[layer]);
  *v_dim = cache_vdim(M->cfg, M->layers[layer]);
  return B200_OK;
}

extern "C" int b200_stack_set_rot_table(b200_ctx* c, int32_t index, const float* table, int64_t n_pos, int32_t half) {
  B200_REQUIRE(c && c->stack && table && index >= 0 && index < 16 && n_pos > 0 && half > 0, B200_ERR_INVALID,
               "stack_set_rot_table: bad argument");
  c->stack->rot[index] = table;
  c->stack->rot_pos[index] = n_pos;
  c->stack->rot_half[index] = half;
  return B200_OK;
}

extern "C" int64_t b200_stack_state_bytes(b200_ctx* c) { return c && c->stack ? c->stack->slot_floats * 4 : 0; }

extern "C" int b200_stack_set_state(b200_ctx* c, void* state) {
  B200_REQUIRE(c && c->stack && state && c->stack->slot_floats > 0, B200_ERR_INVALID, "stack_set_state: not a ctx with state slots");
  B200_REQUIRE(reinterpret_cast<uintptr_t>(state) % 16 == 0, B200_ERR_INVALID, "stack_set_state: pointer not 16-byte aligned");
  c->stack->state = static_cast<float*>(state);
  return B200_OK;
}

extern "C" int b200_stack_set_step_slots(b200_ctx* c, const int32_t* seq_slots, int32_t n_seqs) {
  B200_REQUIRE(c && c->stack && n_seqs >= 0, B200_ERR_INVALID, "stack_set_step_slots: bad argument");
  c->stack->step_slots = seq_slots;
  c->stack->step_seqs = n_seqs;
  return B200_OK;
}

extern "C" int b200_stack_set_stream_tap(b200_ctx* c, float* out) {
  B200_REQUIRE(c && c->stack, B200_ERR_INVALID, "stack_set_stream_tap: not a layer-list ctx");
  c->stack->tap = out;
  c->tap_layer = out ? (1 << 30) : -1;   // a set tap turns graph replay off (run_step)
  return B200_OK;
}

extern "C" int b200_ctx_logits_last_f32(b200_ctx* c, int32_t n_rows, float* host_out, void* stream) {
  B200_REQUIRE(c && host_out, B200_ERR_INVALID, "logits_last_f32: null argument");
  B200_REQUIRE(c->cfg.tp_world == 1, B200_ERR_UNSUPPORTED, "logits_last_f32: one GPU only");
  B200_REQUIRE(n_rows > 0 && n_rows <= c->max_logit_rows, B200_ERR_INVALID, "logits_last_f32: n_rows=%d outside (0,%d]", n_rows,
               c->max_logit_rows);
  cudaStream_t s = (cudaStream_t)stream;
  const int V = c->vocab_local, ld = c->logits_ld;
  if (c->logits_f32) {
    B200_CUDA(cudaMemcpy2DAsync(host_out, (size_t)V * 4, c->logits_f32, (size_t)ld * 4, (size_t)V * 4, n_rows, cudaMemcpyDeviceToHost, s));
    return B200_OK;
  }
  // widen on the device into the logit-adjust scratch (16 MiB), in slices when the rows exceed it
  float* tmp = static_cast<float*>(c->d_adjust);
  const int64_t cap_rows = std::max<int64_t>((4ll << 20) / ld, 1);
  B200_REQUIRE((int64_t)ld <= (4ll << 20), B200_ERR_UNSUPPORTED, "logits_last_f32: vocabulary too large for the scratch");
  for (int64_t r0 = 0; r0 < n_rows; r0 += cap_rows) {
    const int64_t nr = std::min<int64_t>(cap_rows, n_rows - r0);
    int rc = convert_bf16_to_f32(c->logits + r0 * ld, tmp, nr * ld, s);
    if (rc) return rc;
    B200_CUDA(cudaMemcpy2DAsync(host_out + r0 * V, (size_t)V * 4, tmp, (size_t)ld * 4, (size_t)V * 4, nr, cudaMemcpyDeviceToHost, s));
  }
  return B200_OK;
}

// ---- per-kernel entry points ---------------------------------------------------------------------------------------------
extern "C" int b200_layernorm_stream(int32_t f32, float* x, const void* y, const float* yparts, int32_t n_parts, const float* w_post,
                                     const float* w_next, void* out, const int32_t* rows, int32_t T, int32_t width, float eps,
                                     void* stream) {
  B200_REQUIRE(x && T >= 0 && width > 0, B200_ERR_INVALID, "layernorm_stream: bad argument");
  return layernorm_stream(f32 != 0, x, y, yparts, n_parts, w_post, w_next, out, rows, T, width, eps, (cudaStream_t)stream);
}

extern "C" int b200_qk_norm_rotate_cache(int32_t f32, const void* qkv, const float* qw, const float* kw, const int32_t* positions,
                                         const int32_t* slots, const float* rot, int32_t rot_dims, const float* vrot, float* q_out,
                                         void* kc, void* vc, int32_t T, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                                         int32_t block_size, float eps, int64_t max_pos, void* stream) {
  B200_REQUIRE(qkv && qw && kw && positions && slots && q_out && kc && vc && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 &&
                   block_size > 0 && max_pos > 0,
               B200_ERR_INVALID, "qk_norm_rotate_cache: bad argument");
  return qk_norm_rotate_cache(f32 != 0, qkv, qw, kw, positions, slots, rot, rot ? rot_dims : 0, vrot, q_out, kc, vc, T, heads, kv_heads,
                              dim, vdim, block_size, eps, max_pos, (cudaStream_t)stream);
}

extern "C" int b200_qk_norm_rotate_cache_wide(const void* qkv, const float* qw, const float* kw, const int32_t* positions,
                                              const int32_t* slots, const float* rot, int32_t rot_dims, const float* vrot, void* q_out,
                                              void* kc, void* vc, int32_t T, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                                              int32_t block_size, float eps, int64_t max_pos, int32_t k_row, int32_t v_row, void* stream) {
  B200_REQUIRE(qkv && qw && kw && positions && slots && q_out && kc && vc && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 &&
                   block_size > 0 && max_pos > 0 && k_row >= dim && v_row >= vdim && k_row % 2 == 0 && v_row % 2 == 0,
               B200_ERR_INVALID, "qk_norm_rotate_cache_wide: bad argument");
  return qk_norm_rotate_cache(false, qkv, qw, kw, positions, slots, rot, rot ? rot_dims : 0, vrot, nullptr, kc, vc, T, heads, kv_heads,
                              dim, vdim, block_size, eps, max_pos, (cudaStream_t)stream, (__nv_bfloat16*)q_out, k_row, v_row);
}

extern "C" int b200_rotate_back_rows(const void* in, int32_t in_row, void* out, const int32_t* positions, const float* vrot, int32_t T,
                                     int32_t heads, int32_t vdim, int64_t max_pos, void* stream) {
  B200_REQUIRE(in && out && positions && T >= 0 && heads > 0 && vdim > 0 && max_pos > 0, B200_ERR_INVALID, "rotate_back_rows: bad argument");
  return rotate_back_rows((const __nv_bfloat16*)in, in_row, (__nv_bfloat16*)out, positions, vrot, T, heads, vdim, max_pos,
                          (cudaStream_t)stream);
}

extern "C" int64_t b200_paged_attn_anydim_workspace_bytes(int32_t T) { return paged_attn_anydim_workspace_bytes(T); }

extern "C" int b200_paged_attn_anydim(int32_t f32, const float* q, const void* kc, const void* vc, const int32_t* block_table,
                                      int32_t bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions,
                                      const float* vrot, int64_t max_pos, void* out, int32_t T, int32_t heads, int32_t kv_heads,
                                      int32_t dim, int32_t vdim, int32_t block_size, float scale, int32_t shared_tiles, void* ws,
                                      void* stream) {
  B200_REQUIRE(q && kc && vc && block_table && ctx_lens && positions && out && block_size > 0, B200_ERR_INVALID,
               "paged_attn_anydim: bad argument");
  B200_REQUIRE(!shared_tiles || ws, B200_ERR_INVALID, "paged_attn_anydim: the shared-tile form needs its workspace");
  return paged_attn_anydim(f32 != 0, q, kc, vc, block_table, bt_stride, row_to_seq, ctx_lens, positions, vrot, max_pos, out, T, heads,
                           kv_heads, dim, vdim, block_size, scale, shared_tiles ? 1 : 0, ws, (cudaStream_t)stream);
}

extern "C" int b200_moe_route(int32_t f32, const void* x, const void* w_router, const float* bias, int32_t T, int32_t width,
                              int32_t experts, int32_t top, int32_t groups, int32_t keep, int32_t* out_ids, float* out_w, void* stream) {
  B200_REQUIRE(x && w_router && out_ids && out_w && width > 0, B200_ERR_INVALID, "moe_route: bad argument");
  return moe_route(f32 != 0, x, (const __nv_bfloat16*)w_router, bias, T, width, experts, top, groups, keep, out_ids, out_w,
                   (cudaStream_t)stream);
}

extern "C" int b200_moe_route_linear(const void* x, const void* w_router, const float* bias, int32_t T, int32_t width, int32_t experts,
                                     int32_t top, int32_t groups, int32_t keep, int32_t* out_ids, float* out_w, float* logits,
                                     void* stream) {
  B200_REQUIRE(x && w_router && out_ids && out_w && logits && width > 0, B200_ERR_INVALID, "moe_route_linear: bad argument");
  return moe_route(false, x, (const __nv_bfloat16*)w_router, bias, T, width, experts, top, groups, keep, out_ids, out_w,
                   (cudaStream_t)stream, logits, nullptr, 0);
}

extern "C" int64_t b200_moe_workspace_bytes(int32_t T, int32_t top, int32_t experts, int32_t width, int32_t ff) {
  return moe_workspace_bytes(T, top, experts, width, ff);
}

extern "C" int b200_moe_experts(int32_t f32, const void* x, const void* w_gu, const void* w_down, const int32_t* ids, const float* wts,
                                int32_t T, int32_t width, int32_t ff, int32_t experts, int32_t top, float* parts, void* ws,
                                void* stream) {
  B200_REQUIRE(x && w_gu && w_down && ids && wts && parts && width > 0 && ff > 0 && experts > 0 && top > 0, B200_ERR_INVALID,
               "moe_experts: bad argument");
  return moe_experts(f32 != 0, x, (const __nv_bfloat16*)w_gu, (const __nv_bfloat16*)w_down, ids, wts, T, width, ff, experts, top,
                     parts, ws, (cudaStream_t)stream);
}

extern "C" int b200_linear_simt(int32_t x_f32, int32_t y_f32, const void* x, int64_t ldx, const void* w, void* y, int64_t ldy,
                                int32_t T, int32_t n_out, int32_t k, void* stream) {
  B200_REQUIRE(x && w && y && T >= 0 && n_out > 0 && k > 0, B200_ERR_INVALID, "linear_simt: bad argument");
  return linear_simt(x_f32 != 0, y_f32 != 0, x, ldx, (const __nv_bfloat16*)w, y, ldy, T, n_out, k, (cudaStream_t)stream);
}

// ---- per-kernel entry points of the parallel form ---------------------------------------------------------------------------
extern "C" int b200_seq_bounds(const int32_t* row_to_seq, int32_t T, int32_t n_seqs, int32_t* seq_start, void* stream) {
  B200_REQUIRE(seq_start && T >= 0 && n_seqs >= 0, B200_ERR_INVALID, "seq_bounds: bad argument");
  return seq_bounds(row_to_seq, T, n_seqs, seq_start, (cudaStream_t)stream);
}

extern "C" int b200_embed_bigram(const int32_t* ids, const void* table, const void* bigram, float* out, int32_t T, int32_t width,
                                 int32_t vocab, float scale, const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start,
                                 const int32_t* seq_slots, int32_t n_seqs, int32_t* state_prev, int64_t slot_stride_ints, int32_t buckets,
                                 int32_t mul_prev, int32_t mul_cur, void* stream) {
  B200_REQUIRE(ids && table && out && width > 0 && vocab > 0, B200_ERR_INVALID, "embed_bigram: bad argument");
  int rc = embed_bigram(ids, (const __nv_bfloat16*)table, (const __nv_bfloat16*)bigram, out, T, width, vocab, scale, nullptr, 0, positions,
                        row_to_seq, seq_slots, state_prev, slot_stride_ints, buckets, mul_prev, mul_cur, (cudaStream_t)stream);
  if (rc || !state_prev) return rc;
  B200_REQUIRE(seq_start && seq_slots, B200_ERR_INVALID, "embed_bigram: sequence bounds / slots missing");
  return prev_token_commit(ids, vocab, nullptr, 0, seq_start, seq_slots, n_seqs, state_prev, slot_stride_ints, (cudaStream_t)stream);
}

extern "C" int b200_parallel_close(int32_t f32, float* u, const void* y_mix, const void* y_ff, const float* parts, int32_t n_parts,
                                   const void* y_sh, float* results, int64_t result_stride, int32_t n_results, const float* dwa,
                                   const float* g1, const float* g2, float* h1_f32, void* h1_act, void* h2, int32_t T, int32_t width,
                                   float eps, void* stream) {
  B200_REQUIRE(u && T >= 0 && width > 0 && n_results >= 1, B200_ERR_INVALID, "parallel_close: bad argument");
  return parallel_close(f32 != 0, u, y_mix, y_ff, parts, n_parts, y_sh, results, result_stride, n_results, dwa, g1, g2, h1_f32, h1_act, h2,
                        T, width, eps, (cudaStream_t)stream);
}

extern "C" int b200_canon_conv(int32_t f32, const float* h, const float* w, void* out, int32_t T, int32_t width, int32_t taps,
                               const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots,
                               float* tails, int64_t slot_stride, void* stream) {
  B200_REQUIRE(h && w && out && width > 0, B200_ERR_INVALID, "canon_conv: bad argument");
  return canon_conv(f32 != 0, h, w, out, T, width, taps, positions, row_to_seq, seq_start, seq_slots, tails, slot_stride,
                    (cudaStream_t)stream);
}

extern "C" int b200_latent_prep(int32_t f32, const void* qkv, int64_t ld, const float* norm_w, const int32_t* positions,
                                const int32_t* slots, const float* rot, int32_t rot_dims, int64_t max_pos, float* qfull, void* cache,
                                int32_t T, int32_t heads, int32_t dim, int32_t rot_dim, int32_t kv_rank, float eps, void* stream) {
  B200_REQUIRE(qkv && norm_w && positions && slots && qfull && cache && heads > 0 && kv_rank > 0 && max_pos > 0, B200_ERR_INVALID,
               "latent_prep: bad argument");
  return latent_prep(f32 != 0, qkv, ld, norm_w, positions, slots, rot, rot_dims, max_pos, qfull, cache, T, heads, dim, rot_dim, kv_rank, eps,
                     (cudaStream_t)stream);
}

extern "C" int b200_head_linear(int32_t f32, int32_t y_f32, const void* x, int64_t ldx, int32_t x_hs, const void* w, void* y, int64_t ldy,
                                int32_t y_hs, const void* gate, int64_t ldg, int32_t g_hs, int32_t T, int32_t heads, int32_t n_out, int32_t k,
                                void* stream) {
  B200_REQUIRE(x && w && y && heads > 0 && n_out > 0 && k > 0, B200_ERR_INVALID, "head_linear: bad argument");
  return head_linear(f32 != 0, y_f32 != 0, x, ldx, x_hs, (const __nv_bfloat16*)w, y, ldy, y_hs, gate, ldg, g_hs, T, heads, n_out, k,
                     (cudaStream_t)stream);
}

extern "C" int b200_paged_attn_anydim_ex(int32_t f32, const float* q, const void* kc, const void* vc, const int32_t* block_table,
                                         int32_t bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions,
                                         void* out, int32_t T, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t block_size,
                                         float scale, int32_t shared_tiles, void* ws, int32_t k_row, int32_t v_row, const float* sink,
                                         void* stream) {
  B200_REQUIRE(q && kc && vc && block_table && ctx_lens && positions && out && block_size > 0, B200_ERR_INVALID,
               "paged_attn_anydim_ex: bad argument");
  B200_REQUIRE(!shared_tiles || ws, B200_ERR_INVALID, "paged_attn_anydim_ex: the shared-tile form needs its workspace");
  return paged_attn_anydim(f32 != 0, q, kc, vc, block_table, bt_stride, row_to_seq, ctx_lens, positions, nullptr, 1ll << 40, out, T, heads,
                           kv_heads, dim, vdim, block_size, scale, shared_tiles ? 1 : 0, ws, (cudaStream_t)stream, k_row, v_row, sink);
}

extern "C" int b200_mlstm_gates(int32_t f32, const void* x, const void* w, const float* bias, float* out, int32_t T, int32_t width,
                                int32_t heads, float cap, void* stream) {
  B200_REQUIRE(x && w && out && width > 0 && heads > 0, B200_ERR_INVALID, "mlstm_gates: bad argument");
  return mlstm_gates(f32 != 0, x, (const __nv_bfloat16*)w, bias, out, T, width, heads, cap, (cudaStream_t)stream);
}

extern "C" int64_t b200_mlstm_state_floats(int32_t heads, int32_t dim, int32_t vdim) { return mlstm_state_floats(heads, dim, vdim); }

extern "C" int b200_mlstm_scan(int32_t f32, const void* qkv, int64_t ld, int32_t q_off, int32_t k_off, int32_t v_off, const float* gates,
                               const int32_t* positions, const int32_t* seq_start, const int32_t* seq_slots, float* state,
                               int64_t slot_stride, float* out, int32_t n_seqs, int32_t heads, int32_t dim, int32_t vdim, void* stream) {
  B200_REQUIRE(qkv && gates && out && heads > 0, B200_ERR_INVALID, "mlstm_scan: bad argument");
  return mlstm_scan(f32 != 0, qkv, ld, q_off, k_off, v_off, gates, positions, seq_start, seq_slots, state, slot_stride, out, n_seqs, heads,
                    dim, vdim, (cudaStream_t)stream);
}

extern "C" int b200_head_norm_gate(int32_t f32, const float* o, const float* w, const void* gate, int64_t ldg, void* out, int32_t T,
                                   int32_t heads, int32_t vdim, float eps, void* stream) {
  B200_REQUIRE(o && out && heads > 0 && vdim > 0, B200_ERR_INVALID, "head_norm_gate: bad argument");
  return head_norm_gate(f32 != 0, o, w, gate, ldg, out, T, heads, vdim, eps, (cudaStream_t)stream);
}

extern "C" int b200_ff_act(int32_t f32, const void* in, void* out, int32_t T, int32_t ff, int32_t gated, int32_t act, void* stream) {
  B200_REQUIRE(in && out && ff > 0 && act >= 0 && act <= B200_ACT_RELU2, B200_ERR_INVALID, "ff_act: bad argument");
  return ff_act(f32 != 0, in, out, T, ff, gated != 0, act, (cudaStream_t)stream);
}

extern "C" int b200_moe_route_scores(int32_t f32, const void* x, const void* w_router, int32_t T, int32_t width, int32_t experts,
                                     int32_t top, int32_t sigmoid_scores, int32_t* out_ids, float* out_w, void* stream) {
  B200_REQUIRE(x && w_router && out_ids && out_w && width > 0, B200_ERR_INVALID, "moe_route_scores: bad argument");
  return moe_route(f32 != 0, x, (const __nv_bfloat16*)w_router, nullptr, T, width, experts, top, 1, 1, out_ids, out_w, (cudaStream_t)stream,
                   nullptr, nullptr, 0, sigmoid_scores != 0);
}

extern "C" int b200_moe_experts_form(int32_t f32, const void* x, const void* w_up, const void* w_down, const int32_t* ids, const float* wts,
                                     int32_t T, int32_t width, int32_t ff, int32_t experts, int32_t top, float* parts, void* ws,
                                     int32_t gated, int32_t act, int32_t weight_input, void* stream) {
  B200_REQUIRE(x && w_up && w_down && ids && wts && parts && width > 0 && ff > 0 && experts > 0 && top > 0, B200_ERR_INVALID,
               "moe_experts_form: bad argument");
  ExpertForm form;
  form.gated = gated != 0;
  form.act = act;
  form.weight_input = weight_input != 0;
  return moe_experts(f32 != 0, x, (const __nv_bfloat16*)w_up, (const __nv_bfloat16*)w_down, ids, wts, T, width, ff, experts, top, parts, ws,
                     (cudaStream_t)stream, form);
}

extern "C" int b200_latent_attn_supported(int32_t heads, int32_t k_row, int32_t rank) { return latent_attn_mma_supported(heads, k_row, rank) ? 1 : 0; }

extern "C" int b200_latent_attn(const float* q, const void* cache, const int32_t* block_table, int32_t bt_stride, const int32_t* row_to_seq,
                                const int32_t* ctx_lens, void* out, int32_t T, int32_t heads, int32_t k_row, int32_t rank,
                                int32_t block_size, float scale, const float* sink, void* workspace, int32_t n_splits, float* part,
                                void* stream) {
  B200_REQUIRE(q && cache && block_table && ctx_lens && out && workspace && block_size > 0, B200_ERR_INVALID, "latent_attn: bad argument");
  int rc = paged_attn_runs_plan(row_to_seq, ctx_lens, T, workspace, (cudaStream_t)stream);
  if (rc) return rc;
  return latent_attn_mma(q, (const __nv_bfloat16*)cache, block_table, bt_stride, row_to_seq, ctx_lens, (__nv_bfloat16*)out,
                         static_cast<const int32_t*>(workspace) + 8, static_cast<const int32_t*>(workspace), T, heads, k_row, rank,
                         block_size, scale, sink, (cudaStream_t)stream, n_splits, part);
}

// ---- per-kernel entry points of the post-norm form ---------------------------------------------------------------------------
extern "C" int32_t b200_delta_fused_rows(int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t decay_rank, int32_t gate_rank,
                                         int32_t* offsets) {
  return delta_fused_rows(heads, kv_heads, dim, vdim, decay_rank, gate_rank, offsets);
}

extern "C" int b200_postnorm_stream(int32_t f32, const float* x_in, const void* y, float alpha, const float* w, const float* b, float* x_out,
                                    void* out_act, const int32_t* rows, int32_t R, int32_t width, float eps, void* stream) {
  B200_REQUIRE(x_in && w && width > 0 && R >= 0, B200_ERR_INVALID, "postnorm_stream: bad argument");
  return postnorm_stream(f32 != 0, x_in, y, alpha, w, b, x_out, out_act, rows, R, width, eps, (cudaStream_t)stream);
}

extern "C" int b200_qk_headnorm_rotate_cache(int32_t f32, const void* qk, int64_t ld, const float* qw, const float* kw, const int32_t* positions,
                                             const int32_t* slots, const float* rot, int32_t rot_dims, int64_t max_pos, float* q_out, void* kc,
                                             void* vc, int32_t T, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t block_size,
                                             float eps, void* stream) {
  B200_REQUIRE(qk && qw && kw && positions && slots && q_out && kc && vc && heads > 0 && kv_heads > 0 && dim > 0 && block_size > 0 && max_pos > 0,
               B200_ERR_INVALID, "qk_headnorm_rotate_cache: bad argument");
  return qk_headnorm_rotate_cache(f32 != 0, qk, ld, qw, kw, positions, slots, rot, rot ? rot_dims : 0, max_pos, q_out, kc, vc, T, heads, kv_heads,
                                  dim, vdim, block_size, eps, (cudaStream_t)stream);
}

extern "C" int b200_paged_attn_window(int32_t f32, const float* q, const void* kc, const void* vc, const int32_t* block_table, int32_t bt_stride,
                                      const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions, void* out, int32_t T,
                                      int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t block_size, float scale,
                                      int32_t shared_tiles, void* ws, int32_t k_row, int32_t v_row, const float* sink, int32_t window,
                                      void* stream) {
  B200_REQUIRE(q && kc && vc && block_table && ctx_lens && positions && out && block_size > 0 && window >= 0, B200_ERR_INVALID,
               "paged_attn_window: bad argument");
  B200_REQUIRE(!shared_tiles || ws, B200_ERR_INVALID, "paged_attn_window: the shared-tile form needs its workspace");
  return paged_attn_anydim(f32 != 0, q, kc, vc, block_table, bt_stride, row_to_seq, ctx_lens, positions, nullptr, 1ll << 40, out, T, heads,
                           kv_heads, dim, vdim, block_size, scale, shared_tiles ? 1 : 0, ws, (cudaStream_t)stream, k_row, v_row, sink, window);
}

extern "C" int b200_latent_attn_window(const float* q, const void* cache, const int32_t* block_table, int32_t bt_stride,
                                       const int32_t* row_to_seq, const int32_t* ctx_lens, void* out, int32_t T, int32_t heads, int32_t k_row,
                                       int32_t rank, int32_t block_size, float scale, const float* sink, void* workspace, int32_t window,
                                       void* stream) {
  B200_REQUIRE(q && cache && block_table && ctx_lens && out && workspace && block_size > 0 && window >= 0, B200_ERR_INVALID,
               "latent_attn_window: bad argument");
  int rc = paged_attn_runs_plan(row_to_seq, ctx_lens, T, workspace, (cudaStream_t)stream);
  if (rc) return rc;
  return latent_attn_mma(q, (const __nv_bfloat16*)cache, block_table, bt_stride, row_to_seq, ctx_lens, (__nv_bfloat16*)out,
                         static_cast<const int32_t*>(workspace) + 8, static_cast<const int32_t*>(workspace), T, heads, k_row, rank,
                         block_size, scale, sink, (cudaStream_t)stream, 1, nullptr, window);
}

extern "C" int b200_latent_norms(int32_t f32, const void* fused, int64_t ld, int32_t q_rank, int32_t kv_rank, const float* qw, const float* kw,
                                 const int32_t* slots, void* cq, void* cache, int32_t T, float eps, void* stream) {
  B200_REQUIRE(fused && q_rank >= 0 && kv_rank >= 0, B200_ERR_INVALID, "latent_norms: bad argument");
  return latent_norms(f32 != 0, fused, ld, q_rank, kv_rank, qw, kw, slots, cq, cache, T, eps, (cudaStream_t)stream);
}

extern "C" int b200_head_linear_head_gate(int32_t f32, const void* x, int64_t ldx, int32_t x_hs, const void* w, void* y, int64_t ldy, int32_t y_hs,
                                          const void* gate, int64_t ldg, int32_t T, int32_t heads, int32_t n_out, int32_t k, void* stream) {
  B200_REQUIRE(x && w && y && gate && heads > 0 && n_out > 0 && k > 0, B200_ERR_INVALID, "head_linear_head_gate: bad argument");
  return head_linear(f32 != 0, false, x, ldx, x_hs, (const __nv_bfloat16*)w, y, ldy, y_hs, gate, ldg, 1, T, heads, n_out, k, (cudaStream_t)stream, 0);
}

extern "C" int b200_delta_prep(int32_t f32, const void* fused, int64_t ld, const void* a2, const float* conv_w, const float* dt_bias,
                               const float* a_log, const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start,
                               const int32_t* seq_slots, const float* tails, int64_t slot_stride, float* qn, float* kn, float* vn, float* beta,
                               float* decay, int32_t T, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t taps,
                               int32_t decay_rank, int32_t gate_rank, void* stream) {
  B200_REQUIRE(fused && a2 && conv_w && dt_bias && a_log && positions && seq_start && qn && kn && vn && beta && decay, B200_ERR_INVALID,
               "delta_prep: null argument");
  return delta_prep(f32 != 0, fused, ld, a2, conv_w, dt_bias, a_log, positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, qn, kn, vn,
                    beta, decay, T, heads, kv_heads, dim, vdim, taps, decay_rank, gate_rank, (cudaStream_t)stream);
}

extern "C" int b200_delta_tails(int32_t f32, const void* fused, int64_t ld, const int32_t* positions, const int32_t* seq_start,
                                const int32_t* seq_slots, float* tails, int64_t slot_stride, int32_t S, int32_t channels, int32_t taps,
                                void* stream) {
  B200_REQUIRE(fused && channels > 0 && taps >= 1, B200_ERR_INVALID, "delta_tails: bad argument");
  return delta_tails(f32 != 0, fused, ld, positions, seq_start, seq_slots, tails, slot_stride, S, channels, taps, (cudaStream_t)stream);
}

extern "C" int b200_delta_scan(const float* qn, const float* kn, const float* vn, const float* beta, const float* decay, const int32_t* positions,
                               const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int32_t S,
                               int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, void* stream) {
  B200_REQUIRE(qn && kn && vn && beta && decay && out, B200_ERR_INVALID, "delta_scan: null argument");
  return delta_scan(qn, kn, vn, beta, decay, positions, seq_start, seq_slots, state, slot_stride, out, S, heads, kv_heads, dim, vdim,
                    (cudaStream_t)stream);
}

extern "C" int b200_paged_attn_mma_supported(int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim) {
  return paged_attn_mma_supported(heads, kv_heads, dim, vdim) ? 1 : 0;
}

extern "C" int b200_paged_attn_mma(const float* q, const void* kc, const void* vc, const int32_t* block_table, int32_t bt_stride,
                                   const int32_t* row_to_seq, const int32_t* ctx_lens, void* out, int32_t T, int32_t heads, int32_t kv_heads,
                                   int32_t dim, int32_t vdim, int32_t block_size, float scale, const float* sink, void* workspace, int32_t window,
                                   int32_t n_splits, float* part, void* stream) {
  B200_REQUIRE(q && kc && vc && block_table && ctx_lens && out && workspace && block_size > 0 && window >= 0, B200_ERR_INVALID,
               "paged_attn_mma: bad argument");
  int rc = paged_attn_runs_plan(row_to_seq, ctx_lens, T, workspace, (cudaStream_t)stream);
  if (rc) return rc;
  return paged_attn_mma(q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, bt_stride, row_to_seq, ctx_lens, (__nv_bfloat16*)out,
                        static_cast<const int32_t*>(workspace) + 8, static_cast<const int32_t*>(workspace), T, heads, kv_heads, dim, vdim,
                        block_size, scale, sink, (cudaStream_t)stream, n_splits, part, window);
}

// ---- per-kernel entry points of the multi-stream form ------------------------------------------------------------------------
extern "C" int b200_hyper_step(int32_t f32, float* X, int64_t stream_stride, int32_t n, int32_t init, const void* y, const float* parts,
                               int32_t n_parts, const float* scale, const float* hc_close, float mult, const float* open_in, const float* norm_w,
                               const float* norm_b, float eps, const int32_t* rows, float* h_f32, void* h_act, float* sum_out, int32_t R,
                               int32_t width, void* stream) {
  B200_REQUIRE(X && width > 0 && R >= 0, B200_ERR_INVALID, "hyper_step: bad argument");
  return hyper_step(f32 != 0, X, stream_stride, n, init != 0, y, parts, n_parts, scale, hc_close, mult, open_in, norm_w, norm_b, eps, rows, h_f32,
                    h_act, sum_out, R, width, (cudaStream_t)stream);
}

extern "C" int b200_qkv_rotate_cache(int32_t f32, const void* qkv, int64_t ld, const int32_t* positions, const int32_t* slots, const float* rot,
                                     int32_t rot_dims, int32_t half_layout, int64_t max_pos, float* q_out, void* kc, void* vc, int32_t T,
                                     int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t block_size, void* stream) {
  B200_REQUIRE(qkv && positions && slots && q_out && kc && vc && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && block_size > 0 && max_pos > 0,
               B200_ERR_INVALID, "qkv_rotate_cache: bad argument");
  return qkv_rotate_cache(f32 != 0, qkv, ld, positions, slots, rot, rot ? rot_dims : 0, half_layout != 0, max_pos, q_out, kc, vc, T, heads, kv_heads,
                          dim, vdim, block_size, (cudaStream_t)stream);
}

extern "C" int b200_polynorm(int32_t f32, const void* z, const float* coef, void* out, int32_t T, int32_t ff, float eps, void* stream) {
  B200_REQUIRE(z && coef && out && ff > 0, B200_ERR_INVALID, "polynorm: bad argument");
  return polynorm(f32 != 0, z, coef, out, T, ff, eps, (cudaStream_t)stream);
}

extern "C" int b200_ff_act_limit(int32_t f32, const void* in, void* out, int32_t T, int32_t ff, int32_t gated, int32_t act, float limit,
                                 void* stream) {
  B200_REQUIRE(in && out && ff > 0 && act >= 0 && act <= B200_ACT_SWIGLU_CLAMP, B200_ERR_INVALID, "ff_act_limit: bad argument");
  return ff_act(f32 != 0, in, out, T, ff, gated != 0, act, (cudaStream_t)stream, limit);
}

extern "C" int b200_moe_route_chosen(int32_t f32, const void* x, const void* w_router, const float* bias, int32_t T, int32_t width, int32_t experts,
                                     int32_t top, int32_t* out_ids, float* out_w, void* stream) {
  B200_REQUIRE(x && w_router && out_ids && out_w && width > 0, B200_ERR_INVALID, "moe_route_chosen: bad argument");
  return moe_route(f32 != 0, x, (const __nv_bfloat16*)w_router, bias, T, width, experts, top, 1, 1, out_ids, out_w, (cudaStream_t)stream, nullptr,
                   nullptr, 0, 2);
}

extern "C" int b200_moe_experts_limit(int32_t f32, const void* x, const void* w_up, const void* w_down, const int32_t* ids, const float* wts,
                                      int32_t T, int32_t width, int32_t ff, int32_t experts, int32_t top, float* parts, void* ws, int32_t gated,
                                      int32_t act, float limit, void* stream) {
  B200_REQUIRE(x && w_up && w_down && ids && wts && parts && width > 0 && ff > 0 && experts > 0 && top > 0, B200_ERR_INVALID,
               "moe_experts_limit: bad argument");
  ExpertForm form;
  form.gated = gated != 0;
  form.act = act;
  form.limit = limit;
  return moe_experts(f32 != 0, x, (const __nv_bfloat16*)w_up, (const __nv_bfloat16*)w_down, ids, wts, T, width, ff, experts, top, parts, ws,
                     (cudaStream_t)stream, form);
}

extern "C" int b200_delta_prep_head(int32_t f32, const void* fused, int64_t ld, const float* conv_w, const float* dt_bias, const float* a_log,
                                    const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots,
                                    const float* tails, int64_t slot_stride, float* qn, float* kn, float* vn, float* beta, float* decay, int32_t T,
                                    int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t taps, void* stream) {
  B200_REQUIRE(fused && conv_w && dt_bias && a_log && positions && seq_start && qn && kn && vn && beta && decay, B200_ERR_INVALID,
               "delta_prep_head: null argument");
  return delta_prep(f32 != 0, fused, ld, nullptr, conv_w, dt_bias, a_log, positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, qn, kn, vn,
                    beta, decay, T, heads, kv_heads, dim, vdim, taps, 0, 0, (cudaStream_t)stream, true);
}

extern "C" int b200_linear_scan(int32_t delta_rule, const float* qn, const float* kn, const float* vn, const float* beta, const float* decay,
                                int64_t g_row, int32_t g_head, int32_t g_chan, const int32_t* positions, const int32_t* seq_start,
                                const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int32_t S, int32_t heads, int32_t kv_heads,
                                int32_t dim, int32_t vdim, void* stream) {
  B200_REQUIRE(qn && kn && vn && beta && decay && out, B200_ERR_INVALID, "linear_scan: null argument");
  return linear_scan(delta_rule != 0, qn, kn, vn, beta, decay, g_row, g_head, g_chan, positions, seq_start, seq_slots, state, slot_stride, out, S,
                     heads, kv_heads, dim, vdim, (cudaStream_t)stream);
}

extern "C" int b200_head_norm_gate_act(int32_t f32, const float* o, const float* w, const void* gate, int64_t ldg, void* out, int32_t T,
                                       int32_t heads, int32_t vdim, float eps, int32_t gate_silu, void* stream) {
  B200_REQUIRE(o && out && heads > 0 && vdim > 0, B200_ERR_INVALID, "head_norm_gate_act: bad argument");
  return head_norm_gate(f32 != 0, o, w, gate, ldg, out, T, heads, vdim, eps, (cudaStream_t)stream, gate_silu != 0);
}

extern "C" int b200_ssd_prep(int32_t f32, const void* fused, int64_t ld, const float* conv_w, const float* conv_b, const float* dt_bias,
                             const float* a_log, const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start,
                             const int32_t* seq_slots, const float* tails, int64_t slot_stride, float* xn, float* bn, float* cn, float* dt,
                             float* decay, int32_t T, int32_t heads, int32_t groups, int32_t state, int32_t vdim, int32_t taps, void* stream) {
  B200_REQUIRE(fused && conv_w && dt_bias && a_log && positions && seq_start && xn && bn && cn && dt && decay, B200_ERR_INVALID,
               "ssd_prep: null argument");
  return ssd_prep(f32 != 0, fused, ld, conv_w, conv_b, dt_bias, a_log, positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, xn, bn, cn,
                  dt, decay, T, heads, groups, state, vdim, taps, (cudaStream_t)stream);
}

extern "C" int b200_ssd_gate_norm(int32_t f32, const float* o, const float* xn, const float* skip, const void* z, int64_t ldz, const float* w,
                                  void* out, int32_t T, int32_t heads, int32_t vdim, int32_t norm_groups, float eps, void* stream) {
  B200_REQUIRE(o && xn && skip && z && w && out && heads > 0 && vdim > 0, B200_ERR_INVALID, "ssd_gate_norm: bad argument");
  return ssd_gate_norm(f32 != 0, o, xn, skip, z, ldz, w, out, T, heads, vdim, norm_groups, eps, (cudaStream_t)stream);
}
