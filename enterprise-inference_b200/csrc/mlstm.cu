// Matrix-memory recurrence (B200_MIXER_MLSTM).  Per head and sequence the state is S [dim][vdim], n [dim] and a running
// maximum m of the log gates, all fp32, kept in the sequence's state slot between steps:
//   i_t = cap tanh((w_i . h + b_i) / cap)              f_t = logsigmoid(cap tanh((w_f . h + b_f) / cap))
//   m_t = max(f_t + m_{t-1}, i_t)                      a = exp(f_t + m_{t-1} - m_t),  b = exp(i_t - m_t)
//   S_t = a S_{t-1} + b k_t v_t^T                      n_t = a n_{t-1} + b k_t
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t scaled by dim^-1/2
// then each head's o_t is brought to unit RMS, multiplied by a weight and by sigmoid(g_t).
//
//  * mlstm_gates: the two gate projections with fp32 accumulation and the gate transforms, [T][2 heads] fp32;
//  * mlstm_scan: the recurrence.  One CTA per (sequence, head, 32 value columns) walks the sequence's rows of the step in
//    order (a decode row is a walk of one), 16 rows staged in shared memory at a time; a warp owns 4 columns, a lane the
//    key dimensions lane, lane + 32, ...; the state lives in registers during the walk and is stored as [head][vdim][dim]
//    so that a warp's loads are contiguous.  Inside a stage the gate scalars (decays, input weights, exp(-m)) are computed
//    for all rows at once, the walk itself only updates the state and leaves per-lane partial dot products in shared memory,
//    and the sums over lanes, the normaliser and the division follow for the whole stage: no reduction sits on the chain
//    from one row to the next.
//    n and m are kept once per CTA (every CTA of a head needs them from the step before, so they cannot share one copy
//    that one of them overwrites).  A sequence whose first row is at position 0 starts from zeros.
//  * head_norm_gate: unit RMS per head, weight, sigmoid gate (or the gate's silu).
#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void stx(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename AT>
__global__ void __launch_bounds__(128)
mlstm_gates_kernel(const AT* __restrict__ x, const __nv_bfloat16* __restrict__ w, const float* __restrict__ bias, float* __restrict__ out,
                   int width, int heads, float cap) {
  extern __shared__ float xs[];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += 128) xs[c] = ldx<AT>(x, t * width + c);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int o = warp; o < 2 * heads; o += 4) {
    const __nv_bfloat16* wr = w + (int64_t)o * width;
    float a = 0.f;
    for (int c = lane; c < width; c += 32) a = fmaf(__bfloat162float(wr[c]), xs[c], a);
    a = warp_sum(a);
    if (lane == 0) {
      const float z = cap * tanhf((a + (bias ? bias[o] : 0.f)) / cap);
      out[t * 2 * heads + o] = o < heads ? z : log_sigmoid(z);
    }
  }
}

constexpr int kScanCols = 4;                 // value columns per warp
constexpr int kScanWarps = 8;
constexpr int kScanBlockCols = kScanCols * kScanWarps;
constexpr int kScanStage = 16;               // rows staged in shared memory at a time
constexpr int kScanSums = kScanCols + 1;     // per row and warp: one dot product per column and n . q

// STAGED false: the step has decode rows only (one row per sequence): no staging, no prefetch registers, so that several
// CTAs share an SM and the state's loads and stores, which are all of the work then, overlap.
template <typename AT, int DPL, bool STAGED>
__global__ void __launch_bounds__(kScanWarps * 32)
mlstm_scan_kernel(const AT* __restrict__ qkv, int64_t ld, int q_off, int k_off, int v_off, const float* __restrict__ gates,
                  const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slots,
                  float* __restrict__ state, int64_t slot_stride, float* __restrict__ out, int heads, int dim, int vd, float qscale) {
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y, zb = blockIdx.z, nz = gridDim.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int start = seq_start[s], n_rows = seq_start[s + 1] - start;
  if (n_rows <= 0) return;
  const bool fresh = positions[start] == 0;
  float* S_st = state + (int64_t)seq_slots[s] * slot_stride;                  // [heads][vd][dim]
  float* n_st = S_st + (int64_t)heads * vd * dim + ((int64_t)h * nz + zb) * dim;   // [heads][nz][dim]
  float* m_st = S_st + (int64_t)heads * vd * dim + (int64_t)heads * nz * dim + (int64_t)h * nz + zb;   // [heads][nz]
  const int j0 = zb * kScanBlockCols + warp * kScanCols;
  float Sr[kScanCols][DPL], nr[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    nr[i] = (!fresh && d < dim) ? n_st[d] : 0.f;
#pragma unroll
    for (int c = 0; c < kScanCols; ++c)
      Sr[c][i] = (!fresh && d < dim && j0 + c < vd) ? S_st[((int64_t)h * vd + j0 + c) * dim + d] : 0.f;
  }
  float m = fresh ? 0.f : *m_st;
  __syncthreads();   // every warp has read n and m before warp 0 may store them
  if constexpr (!STAGED) {
    for (int r = 0; r < n_rows; ++r) {
      const int t = start + r;
      const AT* row = qkv + (int64_t)t * ld;
      const float ig = gates[(int64_t)t * 2 * heads + h], fg = gates[(int64_t)t * 2 * heads + heads + h];
      const float m_new = fmaxf(fg + m, ig);
      const float a = expf(fg + m - m_new), b = expf(ig - m_new);
      m = m_new;
      float nq = 0.f, acc[kScanCols], v[kScanCols];
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) {
        acc[c] = 0.f;
        v[c] = j0 + c < vd ? ldx<AT>(row, v_off + h * vd + j0 + c) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        const float qv = d < dim ? ldx<AT>(row, q_off + h * dim + d) * qscale : 0.f;
        const float bk = b * (d < dim ? ldx<AT>(row, k_off + h * dim + d) : 0.f);
        nr[i] = fmaf(a, nr[i], bk);
        nq = fmaf(nr[i], qv, nq);
#pragma unroll
        for (int c = 0; c < kScanCols; ++c) {
          Sr[c][i] = fmaf(a, Sr[c][i], bk * v[c]);
          acc[c] = fmaf(Sr[c][i], qv, acc[c]);
        }
      }
      nq = warp_sum(nq);
      const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
      float mine = 0.f;
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) {
        const float o = warp_sum(acc[c]);
        if (lane == c) mine = o;
      }
      if (lane < kScanCols && j0 + lane < vd) out[((int64_t)t * heads + h) * vd + j0 + lane] = mine / den;
    }
  } else {
  // The rows of the step are staged kScanStage at a time: q (scaled), k, this CTA's 32 value columns and the two gates of
  // the head, loaded by the whole CTA with one round trip to memory per stage; the walk itself reads shared memory only.
  extern __shared__ float stage[];
  float* sq = stage;                          // [kScanStage][dim]
  float* sk = sq + kScanStage * dim;          // [kScanStage][dim]
  float* sv = sk + kScanStage * dim;          // [kScanStage][32]
  float* sg = sv + kScanStage * kScanBlockCols;   // [kScanStage][2]
  float* mypart = sg + kScanStage * 2 + warp * (kScanStage * kScanSums * 33);   // [kScanStage][5 sums][32 lanes + 1]
  const int jb = zb * kScanBlockCols;
  // The next stage's rows travel from memory into registers while this stage is walked, and move to shared memory once it
  // has been consumed: element e = tid + 256 i of a [rows][dim] (q, k) or [rows][32] (v) stage tile.
  constexpr int kThreads = kScanWarps * 32, EQ = 2 * DPL, EV = kScanStage * kScanBlockCols / kThreads;
  float rq[EQ], rk[EQ], rv[EV], rg = 0.f;
  auto prefetch = [&](int b0) {
    const int nb = min(kScanStage, n_rows - b0);
#pragma unroll
    for (int i = 0; i < EQ; ++i) {
      const int e = threadIdx.x + kThreads * i, r = e / dim, d = e - r * dim;
      const bool live = e < nb * dim;
      const AT* row = qkv + (int64_t)(start + b0 + (live ? r : 0)) * ld;
      rq[i] = live ? ldx<AT>(row, q_off + h * dim + d) * qscale : 0.f;
      rk[i] = live ? ldx<AT>(row, k_off + h * dim + d) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < EV; ++i) {
      const int e = threadIdx.x + kThreads * i, r = e / kScanBlockCols, j = jb + e % kScanBlockCols;
      rv[i] = (r < nb && j < vd) ? ldx<AT>(qkv + (int64_t)(start + b0 + r) * ld, v_off + h * vd + j) : 0.f;
    }
    if (threadIdx.x < 2 * nb) rg = gates[(int64_t)(start + b0 + (threadIdx.x >> 1)) * 2 * heads + (threadIdx.x & 1) * heads + h];
  };
  prefetch(0);
  for (int b0 = 0; b0 < n_rows; b0 += kScanStage) {
    const int nb = min(kScanStage, n_rows - b0);
    __syncthreads();   // the stage before has been consumed
#pragma unroll
    for (int i = 0; i < EQ; ++i) {
      const int e = threadIdx.x + kThreads * i;
      if (e < kScanStage * dim) {
        sq[e] = rq[i];
        sk[e] = rk[i];
      }
    }
#pragma unroll
    for (int i = 0; i < EV; ++i) sv[threadIdx.x + kThreads * i] = rv[i];
    if (threadIdx.x < 2 * kScanStage) sg[threadIdx.x] = rg;
    __syncthreads();
    if (b0 + kScanStage < n_rows) prefetch(b0 + kScanStage);
    if (nb == 1) {
      // a decode row: one walk step with its reductions in place
      const float ig = sg[0], fg = sg[1];
      const float m_new = fmaxf(fg + m, ig);
      const float a = expf(fg + m - m_new), b = expf(ig - m_new);
      m = m_new;
      float nq = 0.f, acc[kScanCols];
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) acc[c] = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        const float qv = d < dim ? sq[d] : 0.f, bk = b * (d < dim ? sk[d] : 0.f);
        nr[i] = fmaf(a, nr[i], bk);
        nq = fmaf(nr[i], qv, nq);
#pragma unroll
        for (int c = 0; c < kScanCols; ++c) {
          Sr[c][i] = fmaf(a, Sr[c][i], bk * sv[warp * kScanCols + c]);
          acc[c] = fmaf(Sr[c][i], qv, acc[c]);
        }
      }
      nq = warp_sum(nq);
      const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
      float mine = 0.f;
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) {
        const float o = warp_sum(acc[c]);
        if (lane == c) mine = o;
      }
      if (lane < kScanCols && j0 + lane < vd) out[((int64_t)(start + b0) * heads + h) * vd + j0 + lane] = mine / den;
      continue;
    }
    // gate scalars of the stage: the running maximum is a scalar chain of one add and one max per row; lane r then holds
    // row r's decay a, input weight b and exp(-m), computed for all rows of the stage at once
    const float ig_l = lane < nb ? sg[2 * lane] : 0.f, fg_l = lane < nb ? sg[2 * lane + 1] : 0.f;
    float m_prev_l = 0.f, m_l = 0.f;
    for (int r = 0; r < nb; ++r) {
      const float ig = __shfl_sync(0xffffffffu, ig_l, r), fg = __shfl_sync(0xffffffffu, fg_l, r);
      const float mn = fmaxf(fg + m, ig);
      if (lane == r) {
        m_prev_l = m;
        m_l = mn;
      }
      m = mn;
    }
    const float a_l = expf(fg_l + m_prev_l - m_l), b_l = expf(ig_l - m_l), e_l = expf(-m_l);
    // the walk: state update and per-lane partial dot products only; nothing here waits for a reduction
    for (int r = 0; r < nb; ++r) {
      const float a = __shfl_sync(0xffffffffu, a_l, r), b = __shfl_sync(0xffffffffu, b_l, r);
      float q[DPL], k[DPL], v[kScanCols];
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        q[i] = d < dim ? sq[r * dim + d] : 0.f;
        k[i] = d < dim ? sk[r * dim + d] : 0.f;
      }
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) v[c] = sv[r * kScanBlockCols + warp * kScanCols + c];
      float nq = 0.f, acc[kScanCols];
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) acc[c] = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const float bk = b * k[i];
        nr[i] = fmaf(a, nr[i], bk);
        nq = fmaf(nr[i], q[i], nq);
#pragma unroll
        for (int c = 0; c < kScanCols; ++c) {
          Sr[c][i] = fmaf(a, Sr[c][i], bk * v[c]);
          acc[c] = fmaf(Sr[c][i], q[i], acc[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < kScanCols; ++c) mypart[(r * kScanSums + c) * 33 + lane] = acc[c];
      mypart[(r * kScanSums + kScanCols) * 33 + lane] = nq;
    }
    __syncwarp();
    // the stage's reductions: lane x adds the 32 partials of sum x in lane order; then the outputs
    for (int x = lane; x < nb * kScanSums; x += 32) {
      float sum = 0.f;
      for (int l = 0; l < 32; ++l) sum += mypart[x * 33 + l];
      mypart[x * 33 + 32] = sum;
    }
    __syncwarp();
#pragma unroll
    for (int pass = 0; pass < kScanStage * kScanCols / 32; ++pass) {
      const int idx = lane + 32 * pass, r = idx / kScanCols, c = idx % kScanCols;
      const float e = __shfl_sync(0xffffffffu, e_l, r & 31);
      if (r < nb && j0 + c < vd) {
        const float den = fmaxf(fabsf(mypart[(r * kScanSums + kScanCols) * 33 + 32]), e) + 1e-6f;
        out[((int64_t)(start + b0 + r) * heads + h) * vd + j0 + c] = mypart[(r * kScanSums + c) * 33 + 32] / den;
      }
    }
    __syncwarp();
  }
  }   // STAGED
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < dim) {
      if (warp == 0) n_st[d] = nr[i];
#pragma unroll
      for (int c = 0; c < kScanCols; ++c)
        if (j0 + c < vd) S_st[((int64_t)h * vd + j0 + c) * dim + d] = Sr[c][i];
    }
  }
  if (warp == 0 && lane == 0) *m_st = m;
}

// one CTA per row, one warp per head (round robin)
template <typename AT>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const AT* __restrict__ gate, int64_t ldg,
                      AT* __restrict__ out, int heads, int vd, float eps, int gate_silu) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int h = warp; h < heads; h += 4) {
    const float* src = o + (t * heads + h) * vd;
    float ss = 0.f;
    for (int j = lane; j < vd; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vd + eps);
    for (int j = lane; j < vd; j += 32) {
      float v = src[j] * inv;
      if (w) v *= w[h * vd + j];
      if (gate) {
        const float gz = ldx<AT>(gate, t * ldg + h * vd + j);
        v *= (gate_silu ? gz : 1.0f) / (1.0f + expf(-gz));
      }
      stx<AT>(out, (t * heads + h) * vd + j, v);
    }
  }
}

}  // namespace

int mlstm_gates(bool f32, const void* x, const __nv_bfloat16* w, const float* bias, float* out, int T, int width, int heads, float cap,
                cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(cap > 0.f, B200_ERR_INVALID, "mlstm_gates: cap %f", (double)cap);
  const size_t smem = (size_t)width * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "mlstm_gates: width %d does not fit shared memory", width);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(mlstm_gates_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(mlstm_gates_kernel<float>, dim3(T), dim3(128), smem, s, (const float*)x, w, bias, out, width, heads, cap));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(mlstm_gates_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(mlstm_gates_kernel<__nv_bfloat16>, dim3(T), dim3(128), smem, s, (const __nv_bfloat16*)x, w, bias, out, width, heads,
                     cap));
  }
  return B200_OK;
}

int mlstm_col_blocks(int vd) { return (vd + kScanBlockCols - 1) / kScanBlockCols; }

// floats of one layer's recurrent state in a slot: S [heads][vd][dim], n [heads][col blocks][dim], m [heads][col blocks]
int64_t mlstm_state_floats(int heads, int dim, int vd) {
  const int64_t nz = mlstm_col_blocks(vd);
  return (int64_t)heads * vd * dim + (int64_t)heads * nz * dim + (int64_t)heads * nz;
}

template <typename AT>
static int mlstm_scan_t(const void* qkv, int64_t ld, int q_off, int k_off, int v_off, const float* gates, const int32_t* positions,
                        const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int S,
                        int heads, int dim, int vd, bool single_rows, cudaStream_t s) {
  const dim3 grid(S, heads, mlstm_col_blocks(vd)), block(kScanWarps * 32);
  const float qscale = 1.0f / sqrtf((float)dim);
  const int dpl = (dim + 31) / 32;
  const size_t smem = single_rows ? 0 : (size_t)kScanStage * (2 * dim + kScanBlockCols + 2 + kScanWarps * kScanSums * 33) * 4;   // <= 117 KiB
#define SCAN1(D, ST)                                                                                                                \
  do {                                                                                                                              \
    static bool done[64] = {};                                                                                                      \
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(mlstm_scan_kernel<AT, D, ST>, 128 * 1024, done));                           \
    B200_CUDA(launch(mlstm_scan_kernel<AT, D, ST>, grid, block, smem, s, (const AT*)qkv, ld, q_off, k_off, v_off, gates, positions, \
                     seq_start, seq_slots, state, slot_stride, out, heads, dim, vd, qscale));                                       \
  } while (0)
#define SCAN(D)                    \
  do {                             \
    if (single_rows) SCAN1(D, false); \
    else SCAN1(D, true);           \
  } while (0)
  if (dpl <= 1) SCAN(1);
  else if (dpl <= 2) SCAN(2);
  else if (dpl <= 4) SCAN(4);
  else SCAN(8);
#undef SCAN1
#undef SCAN
  return B200_OK;
}

int mlstm_scan(bool f32, const void* qkv, int64_t ld, int q_off, int k_off, int v_off, const float* gates, const int32_t* positions,
               const int32_t* seq_start, const int32_t* seq_slots, float* state, int64_t slot_stride, float* out, int S, int heads,
               int dim, int vd, cudaStream_t s, bool single_rows) {
  if (S == 0) return B200_OK;
  B200_REQUIRE(dim > 0 && dim <= 256 && vd > 0, B200_ERR_UNSUPPORTED, "mlstm_scan: key size %d outside (0, 256]", dim);
  B200_REQUIRE(positions && seq_start && seq_slots && state, B200_ERR_INVALID, "mlstm_scan: null argument");
  return f32 ? mlstm_scan_t<float>(qkv, ld, q_off, k_off, v_off, gates, positions, seq_start, seq_slots, state, slot_stride, out, S, heads,
                                   dim, vd, single_rows, s)
             : mlstm_scan_t<__nv_bfloat16>(qkv, ld, q_off, k_off, v_off, gates, positions, seq_start, seq_slots, state, slot_stride, out,
                                           S, heads, dim, vd, single_rows, s);
}

int head_norm_gate(bool f32, const float* o, const float* w, const void* gate, int64_t ldg, void* out, int T, int heads, int vd, float eps,
                   cudaStream_t s, bool gate_silu) {
  if (T == 0) return B200_OK;
  if (f32)
    B200_CUDA(launch(head_norm_gate_kernel<float>, dim3(T), dim3(128), (size_t)0, s, o, w, (const float*)gate, ldg, (float*)out, heads, vd,
                     eps, gate_silu ? 1 : 0));
  else
    B200_CUDA(launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, s, o, w, (const __nv_bfloat16*)gate, ldg,
                     (__nv_bfloat16*)out, heads, vd, eps, gate_silu ? 1 : 0));
  return B200_OK;
}

}  // namespace b200
