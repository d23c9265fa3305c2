// Delta-rule recurrence with one decay per head and key channel (B200_MIXER_DELTA).  Per head and sequence the state is
// S [dim][vdim], fp32, kept in the sequence's state slot between steps together with the last taps - 1 inputs of the
// q | k | v convolution:
//   x_t   = silu(sum_j w[:, j] raw_{t - taps + 1 + j})         per channel of the q | k | v projection, zeros before position 0
//   q_t   = x_q / sqrt(|x_q|^2 + 1e-6) * dim^-1/2              k_t = x_k / sqrt(|x_k|^2 + 1e-6)       per q/k head
//   b_t   = sigmoid(w_b . h_t)                                 per head
//   g_t   = exp(-exp(a_log) * softplus(W_a2 (W_a1 h_t) + dt_bias))          per head and key channel
//   S_t   = diag(g_t) S_{t-1};   u = b_t (v_t - S_t^T k_t);   S_t += k_t u^T;   o_t = S_t^T q_t
// Head h reads q/k head h / (heads / kv_heads).
//
//  * delta_prep: two CTAs per row (one for beta and the decays): convolution taps from the step's own rows or, before the portion's first row, from the
//    slot's tail; silu; the unit vectors; beta; the decays.  Everything leaves in fp32.
//  * delta_tails: CTAs of 256 channels per sequence, after prep: the last taps - 1 raw rows of the portion (or what is left of the old tail
//    when the portion is shorter) become the slot's tail.
//  * delta_scan: the recurrence.  The columns of S do not interact, so one CTA takes (sequence, head, 32 value columns); a warp
//    owns 4 columns, a lane the key channels lane, lane + 32, ...; the state lives in registers during the walk and is
//    stored [head][vdim][dim] so that a warp's loads are contiguous.  The step's rows are staged 16 at a time in shared memory,
//    the next stage travelling into registers while this one is walked.  The only reductions on the chain from one row to the
//    next are the four S^T k sums of a warp (interleaved shuffles); the read-out leaves per-lane partial sums in shared
//    memory that are added for the whole stage after its walk.
//    A sequence whose first row of the step is at position 0 starts from zeros, whatever the slot held.
//
// Two parameters widen the kernels to other recurrences of the same shape.  The decay of (row, head, key channel) is read at
// decay[t * g_row + h * g_head + d * g_chan]: channel decays are (heads*dim, dim, 1), ONE decay per head is (heads, 1, 0), and
// delta_prep then takes the decay's pre-activation straight from the fused row (one column per head, decay_dim 1) instead of a
// second-step projection.  DELTA false drops the correction: u = beta v, which is the state-space recurrence
// S = g S + dt B x^T, y = S^T C of ssd.cu with keys B, queries C, values x and beta = dt.
#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

constexpr int kPrepThreads = 256;

template <typename AT>
__global__ void __launch_bounds__(kPrepThreads)
delta_prep_kernel(const AT* __restrict__ fused, int64_t ld, const AT* __restrict__ a2, int64_t a2_ld, int decay_dim, const float* __restrict__ conv_w,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, const int32_t* __restrict__ positions,
                  const int32_t* __restrict__ row_to_seq, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slots,
                  const float* __restrict__ tails, int64_t slot_stride, float* __restrict__ qn, float* __restrict__ kn,
                  float* __restrict__ vn, float* __restrict__ beta, float* __restrict__ decay, int heads, int kv_heads, int dim, int vdim,
                  int taps, int off_b) {
  extern __shared__ float xs[];   // [C] convolved and activated channels
  const int64_t t = blockIdx.x;
  const int qk = kv_heads * dim, C = 2 * qk + heads * vdim;
  if (gridDim.x <= 128) {   // short steps wait on latency: weights and the sequence's tail go to L2 while the launch before runs
    if (blockIdx.y == 0) {
      prefetch_l2_span(conv_w, (size_t)C * taps * 4);
      if (tails) prefetch_l2_span(tails + (int64_t)seq_slots[row_to_seq ? row_to_seq[t] : (int)t] * slot_stride, (size_t)(taps - 1) * C * 4);
    } else {
      prefetch_l2_span(dt_bias, (size_t)heads * decay_dim * 4);
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  if (blockIdx.y == 1) {   // the second CTA of a row: beta and the decays (nothing of the convolution enters them)
    const int hd = heads * decay_dim;   // decay_dim: dim (one decay per key channel) or 1 (one per head)
    for (int h = threadIdx.x; h < heads; h += kPrepThreads) beta[t * heads + h] = sigmoid_f(ldx<AT>(fused, t * ld + off_b + h));
    for (int c = threadIdx.x; c < hd; c += kPrepThreads) {
      const float z = ldx<AT>(a2, t * a2_ld + c) + dt_bias[c];
      decay[t * hd + c] = expf(-expf(a_log[c / decay_dim]) * softplus_f(z));
    }
    return;
  }
  const int s = row_to_seq ? row_to_seq[t] : (int)t;
  const int start = seq_start[s], r = (int)t - start, pos = positions[t];
  const float* tail = tails ? tails + (int64_t)seq_slots[s] * slot_stride : nullptr;   // [taps - 1][C]
  for (int c = threadIdx.x; c < C; c += kPrepThreads) {
    float a = 0.f;
    for (int j = 0; j < taps; ++j) {   // lag j: the input of position pos - j
      if (pos - j < 0) break;
      const float x = r - j >= 0 ? ldx<AT>(fused, (t - j) * ld + c) : tail[(int64_t)(taps - 1 + r - j) * C + c];
      a = fmaf(conv_w[(int64_t)c * taps + taps - 1 - j], x, a);
    }
    xs[c] = a * sigmoid_f(a);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kPrepThreads / 32;
  const float qscale = rsqrtf((float)dim);
  for (int v = warp; v < 2 * kv_heads; v += nw) {   // q heads, then k heads
    const float* src = xs + (int64_t)v * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    const float inv = (1.0f / sqrtf(ss + 1e-6f)) * (v < kv_heads ? qscale : 1.0f);
    float* dst = v < kv_heads ? qn + t * qk + (int64_t)v * dim : kn + t * qk + (int64_t)(v - kv_heads) * dim;
    for (int d = lane; d < dim; d += 32) dst[d] = src[d] * inv;
  }
  const int hv = heads * vdim;
  for (int c = threadIdx.x; c < hv; c += kPrepThreads) vn[t * hv + c] = xs[2 * qk + c];
}

template <typename AT>
__global__ void __launch_bounds__(256)
delta_tails_kernel(const AT* __restrict__ fused, int64_t ld, const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_start,
                   const int32_t* __restrict__ seq_slots, float* __restrict__ tails, int64_t slot_stride, int C, int taps) {
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x;
  const int start = seq_start[s], n = seq_start[s + 1] - start;
  if (n <= 0) return;
  const bool fresh = positions[start] == 0;
  float* tail = tails + (int64_t)seq_slots[s] * slot_stride;
  // entry i holds the input of the position (taps - 2 - i) before the portion's last one.  A thread owns a channel and
  // walks i upwards: what it reads of the old tail lies above everything it has written.
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c < C)
    for (int i = 0; i < taps - 1; ++i) {
      const int ri = n - taps + 1 + i;   // row of the portion, negative: before it
      float v;
      if (ri >= 0) v = ldx<AT>(fused, (int64_t)(start + ri) * ld + c);
      else v = fresh ? 0.f : tail[(int64_t)(taps - 1 + ri) * C + c];
      tail[(int64_t)i * C + c] = v;
    }
}

constexpr int kDsCols = 4, kDsWarps = 8, kDsBlockCols = kDsCols * kDsWarps, kDsStage = 16, kDsThreads = kDsWarps * 32;

template <int DPL, bool DELTA>
__global__ void __launch_bounds__(kDsThreads)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vn, const float* __restrict__ beta,
                  const float* __restrict__ decay, int64_t g_row, int g_head, int g_chan, const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_start,
                  const int32_t* __restrict__ seq_slots, float* __restrict__ state, int64_t slot_stride, float* __restrict__ out, int heads,
                  int kv_heads, int dim, int vd) {
  extern __shared__ float stage[];
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y, zb = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int start = seq_start[s], n_rows = seq_start[s + 1] - start;
  if (n_rows <= 0) return;
  const bool fresh = positions[start] == 0;
  const int g = h / (heads / kv_heads);
  float* S_st = state + (int64_t)seq_slots[s] * slot_stride;   // [heads][vd][dim]
  const int jb = zb * kDsBlockCols, j0 = jb + warp * kDsCols;
  float Sr[kDsCols][DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < kDsCols; ++c) Sr[c][i] = (!fresh && d < dim && j0 + c < vd) ? S_st[((int64_t)h * vd + j0 + c) * dim + d] : 0.f;
  }
  const int qk = kv_heads * dim, hv = heads * vd;
  if (n_rows == 1) {
    // a decode row: nothing to stage; the row's inputs are fetched beside the state
    const int64_t t = start;
    const float b = beta[t * heads + h];
    float dot[kDsCols], acc[kDsCols], v[kDsCols], q[DPL], k[DPL];
#pragma unroll
    for (int c = 0; c < kDsCols; ++c) {
      dot[c] = 0.f;
      acc[c] = 0.f;
      v[c] = j0 + c < vd ? vn[t * hv + h * vd + j0 + c] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      const bool live = d < dim;
      q[i] = live ? qn[t * qk + g * dim + d] : 0.f;
      k[i] = live ? kn[t * qk + g * dim + d] : 0.f;
      const float gd = live ? decay[t * g_row + h * g_head + d * g_chan] : 0.f;
#pragma unroll
      for (int c = 0; c < kDsCols; ++c) {
        Sr[c][i] *= gd;
        if (DELTA) dot[c] = fmaf(Sr[c][i], k[i], dot[c]);
      }
    }
    if (DELTA) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int c = 0; c < kDsCols; ++c) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], o);
    }
#pragma unroll
    for (int c = 0; c < kDsCols; ++c) {
      const float u = b * (v[c] - dot[c]);
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        Sr[c][i] = fmaf(k[i], u, Sr[c][i]);
        acc[c] = fmaf(Sr[c][i], q[i], acc[c]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int c = 0; c < kDsCols; ++c) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
    float mine = 0.f;
#pragma unroll
    for (int c = 0; c < kDsCols; ++c)
      if (lane == c) mine = acc[c];
    if (lane < kDsCols && j0 + lane < vd) out[t * hv + h * vd + j0 + lane] = mine;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < dim) {
#pragma unroll
        for (int c = 0; c < kDsCols; ++c)
          if (j0 + c < vd) S_st[((int64_t)h * vd + j0 + c) * dim + d] = Sr[c][i];
      }
    }
    return;
  }
  float* sq = stage;                       // [kDsStage][dim]
  float* sk = sq + kDsStage * dim;
  float* sg = sk + kDsStage * dim;
  float* sv = sg + kDsStage * dim;         // [kDsStage][32]
  float* sb = sv + kDsStage * kDsBlockCols;   // [kDsStage]
  float* mypart = sb + kDsStage + warp * (kDsStage * kDsCols * 33);   // [kDsStage][kDsCols][32 lanes + 1]
  constexpr int EQ = 2 * DPL, EV = kDsStage * kDsBlockCols / kDsThreads;   // elements per thread of a [16][dim] / [16][32] tile
  float rq[EQ], rk[EQ], rg[EQ], rv[EV], rb = 0.f;
  auto prefetch = [&](int b0) {
    const int nb = min(kDsStage, n_rows - b0);
#pragma unroll
    for (int i = 0; i < EQ; ++i) {
      const int e = threadIdx.x + kDsThreads * i, r = e / dim, d = e - r * dim;
      const bool live = e < nb * dim;
      const int64_t t = start + b0 + (live ? r : 0);
      rq[i] = live ? qn[t * qk + g * dim + d] : 0.f;
      rk[i] = live ? kn[t * qk + g * dim + d] : 0.f;
      rg[i] = live ? decay[t * g_row + h * g_head + d * g_chan] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < EV; ++i) {
      const int e = threadIdx.x + kDsThreads * i, r = e / kDsBlockCols, j = jb + e % kDsBlockCols;
      rv[i] = (r < nb && j < vd) ? vn[(int64_t)(start + b0 + r) * hv + h * vd + j] : 0.f;
    }
    if (threadIdx.x < nb) rb = beta[(int64_t)(start + b0 + threadIdx.x) * heads + h];
  };
  prefetch(0);
  for (int b0 = 0; b0 < n_rows; b0 += kDsStage) {
    const int nb = min(kDsStage, n_rows - b0);
    __syncthreads();   // the stage before has been consumed
#pragma unroll
    for (int i = 0; i < EQ; ++i) {
      const int e = threadIdx.x + kDsThreads * i;
      if (e < kDsStage * dim) {
        sq[e] = rq[i];
        sk[e] = rk[i];
        sg[e] = rg[i];
      }
    }
#pragma unroll
    for (int i = 0; i < EV; ++i) sv[threadIdx.x + kDsThreads * i] = rv[i];
    if (threadIdx.x < kDsStage) sb[threadIdx.x] = rb;
    __syncthreads();
    if (b0 + kDsStage < n_rows) prefetch(b0 + kDsStage);
    // the walk: state update and per-lane partial read-out sums only; the one reduction on the chain from a row to the next is
    // S^T k.  The read-out sums over lanes follow for the whole stage.
    for (int r = 0; r < nb; ++r) {
      float q[DPL], k[DPL], dot[kDsCols], acc[kDsCols], v[kDsCols];
#pragma unroll
      for (int c = 0; c < kDsCols; ++c) {
        dot[c] = 0.f;
        acc[c] = 0.f;
        v[c] = sv[r * kDsBlockCols + warp * kDsCols + c];
      }
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        const bool live = d < dim;
        q[i] = live ? sq[r * dim + d] : 0.f;
        k[i] = live ? sk[r * dim + d] : 0.f;
        const float gd = live ? sg[r * dim + d] : 0.f;
#pragma unroll
        for (int c = 0; c < kDsCols; ++c) {
          Sr[c][i] *= gd;
          if (DELTA) dot[c] = fmaf(Sr[c][i], k[i], dot[c]);
        }
      }
      if (DELTA) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int c = 0; c < kDsCols; ++c) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], o);
      }
      const float b = sb[r];
#pragma unroll
      for (int c = 0; c < kDsCols; ++c) {
        const float u = b * (v[c] - dot[c]);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          Sr[c][i] = fmaf(k[i], u, Sr[c][i]);
          acc[c] = fmaf(Sr[c][i], q[i], acc[c]);
        }
        mypart[(r * kDsCols + c) * 33 + lane] = acc[c];
      }
    }
    __syncwarp();
    for (int x = lane; x < nb * kDsCols; x += 32) {   // lane x adds the 32 partials of sum x in lane order
      float sum = 0.f;
#pragma unroll 8
      for (int l = 0; l < 32; ++l) sum += mypart[x * 33 + l];
      const int r = x / kDsCols, c = x % kDsCols;
      if (j0 + c < vd) out[(int64_t)(start + b0 + r) * hv + h * vd + j0 + c] = sum;
    }
    __syncwarp();
  }
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < dim) {
#pragma unroll
      for (int c = 0; c < kDsCols; ++c)
        if (j0 + c < vd) S_st[((int64_t)h * vd + j0 + c) * dim + d] = Sr[c][i];
    }
  }
}

}  // namespace

static int up8(int v) { return (v + 7) / 8 * 8; }

// rows of the fused projection; offsets of q, k, v, a1, g1, b
int delta_fused_rows(int heads, int kv_heads, int dim, int vdim, int decay_rank, int gate_rank, int* off) {
  int o[6];
  o[0] = 0;
  o[1] = kv_heads * dim;
  o[2] = 2 * kv_heads * dim;
  o[3] = up8(o[2] + heads * vdim);
  o[4] = up8(o[3] + decay_rank);
  o[5] = up8(o[4] + gate_rank);
  if (off)
    for (int i = 0; i < 6; ++i) off[i] = o[i];
  return up8(o[5] + heads);
}

int64_t delta_state_floats(int heads, int dim, int vd) { return (int64_t)heads * vd * dim; }
int64_t delta_tail_floats(int heads, int kv_heads, int dim, int vd, int taps) {
  return (int64_t)(taps > 1 ? taps - 1 : 0) * (2 * kv_heads * dim + heads * vd);
}

int delta_prep(bool f32, const void* fused, int64_t ld, const void* a2, const float* conv_w, const float* dt_bias, const float* a_log,
               const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots, const float* tails,
               int64_t slot_stride, float* qn, float* kn, float* vn, float* beta, float* decay, int T, int heads, int kv_heads, int dim,
               int vdim, int taps, int decay_rank, int gate_rank, cudaStream_t s, bool head_decay) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && taps >= 1, B200_ERR_INVALID, "delta_prep: %d heads over %d, %d taps", heads,
               kv_heads, taps);
  B200_REQUIRE(taps == 1 || (tails && seq_slots), B200_ERR_INVALID, "delta_prep: the convolution needs its tails");
  int off[6];
  delta_fused_rows(heads, kv_heads, dim, vdim, decay_rank, gate_rank, off);
  int64_t a2_ld = (int64_t)heads * dim;
  int decay_dim = dim;
  if (head_decay) {   // fused rows q | k | v | gate | b | a without padding: the decay's pre-activation is the row's last group
    off[5] = 2 * kv_heads * dim + 2 * heads * vdim;
    a2 = static_cast<const char*>(fused) + (int64_t)(off[5] + heads) * (f32 ? 4 : 2);
    a2_ld = ld;
    decay_dim = 1;
  }
  const size_t smem = (size_t)(2 * kv_heads * dim + heads * vdim) * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "delta_prep: %zu bytes of channels do not fit shared memory", smem);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(delta_prep_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(delta_prep_kernel<float>, dim3(T, 2), dim3(kPrepThreads), smem, s, (const float*)fused, ld, (const float*)a2, a2_ld, decay_dim, conv_w, dt_bias,
                     a_log, positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, qn, kn, vn, beta, decay, heads, kv_heads, dim, vdim,
                     taps, off[5]));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(delta_prep_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(delta_prep_kernel<__nv_bfloat16>, dim3(T, 2), dim3(kPrepThreads), smem, s, (const __nv_bfloat16*)fused, ld,
                     (const __nv_bfloat16*)a2, a2_ld, decay_dim, conv_w, dt_bias, a_log, positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, qn, kn,
                     vn, beta, decay, heads, kv_heads, dim, vdim, taps, off[5]));
  }
  return B200_OK;
}

int delta_tails(bool f32, const void* fused, int64_t ld, const int32_t* positions, const int32_t* seq_start, const int32_t* seq_slots,
                float* tails, int64_t slot_stride, int S, int channels, int taps, cudaStream_t s) {
  if (S == 0 || taps <= 1) return B200_OK;
  B200_REQUIRE(tails && seq_slots && seq_start && positions, B200_ERR_INVALID, "delta_tails: null argument");
  if (f32)
    B200_CUDA(launch(delta_tails_kernel<float>, dim3(S, (channels + 255) / 256), dim3(256), (size_t)0, s, (const float*)fused, ld, positions, seq_start, seq_slots, tails,
                     slot_stride, channels, taps));
  else
    B200_CUDA(launch(delta_tails_kernel<__nv_bfloat16>, dim3(S, (channels + 255) / 256), dim3(256), (size_t)0, s, (const __nv_bfloat16*)fused, ld, positions, seq_start,
                     seq_slots, tails, slot_stride, channels, taps));
  return B200_OK;
}

int delta_scan(const float* qn, const float* kn, const float* vn, const float* beta, const float* decay, const int32_t* positions,
               const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int S, int heads,
               int kv_heads, int dim, int vd, cudaStream_t s) {
  return linear_scan(true, qn, kn, vn, beta, decay, (int64_t)heads * dim, dim, 1, positions, seq_start, seq_slots, state, slot_stride, out, S,
                     heads, kv_heads, dim, vd, s);
}

int linear_scan(bool delta_rule, const float* qn, const float* kn, const float* vn, const float* beta, const float* decay, int64_t g_row,
                int g_head, int g_chan, const int32_t* positions, const int32_t* seq_start, const int32_t* seq_slots, float* state,
                int64_t slot_stride, float* out, int S, int heads, int kv_heads, int dim, int vd, cudaStream_t s) {
  if (S == 0) return B200_OK;
  B200_REQUIRE(dim > 0 && dim <= 256 && vd > 0, B200_ERR_UNSUPPORTED, "delta_scan: key size %d outside (0, 256]", dim);
  B200_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0, B200_ERR_INVALID, "delta_scan: %d heads over %d", heads, kv_heads);
  B200_REQUIRE(positions && seq_start && seq_slots && state, B200_ERR_INVALID, "delta_scan: null argument");
  const dim3 grid(S, heads, (vd + kDsBlockCols - 1) / kDsBlockCols), block(kDsThreads);
  const int dpl = (dim + 31) / 32;
  const size_t smem = (size_t)kDsStage * (3 * dim + kDsBlockCols + 1 + kDsWarps * kDsCols * 33) * 4;   // <= 117 KiB
#define SCAN2(D, R)                                                                                                                   \
  do {                                                                                                                                \
    static bool done[64] = {};                                                                                                        \
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(delta_scan_kernel<D, R>, 128 * 1024, done));                                   \
    B200_CUDA(launch(delta_scan_kernel<D, R>, grid, block, smem, s, qn, kn, vn, beta, decay, g_row, g_head, g_chan, positions,        \
                     seq_start, seq_slots, state, slot_stride, out, heads, kv_heads, dim, vd));                                       \
  } while (0)
#define SCAN(D)              \
  do {                       \
    if (delta_rule) SCAN2(D, true); \
    else SCAN2(D, false);    \
  } while (0)
  if (dpl <= 1) SCAN(1);
  else if (dpl <= 2) SCAN(2);
  else if (dpl <= 4) SCAN(4);
  else SCAN(8);
#undef SCAN
#undef SCAN2
  return B200_OK;
}

}  // namespace b200
