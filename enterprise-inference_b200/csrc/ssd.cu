// State-space recurrence with one scalar decay per head (B200_MIXER_SSD).  The fused projection of a token is
// z | x | B | C | dt  (heads*vdim, heads*vdim, groups*state, groups*state, heads); per head and sequence the state is
// S [state][vdim], fp32, kept in the sequence's state slot together with the last taps - 1 inputs of the x | B | C convolution:
//   c_t   = silu(bias + sum_j w[:, j] raw_{t - taps + 1 + j})      per channel of x | B | C, zeros before position 0
//   dt_t  = softplus(dt + dt_bias)                                 per head
//   S_t   = exp(-exp(a_log) dt_t) S_{t-1} + dt_t B_t x_t^T         head h reads B and C of group h / (heads / groups)
//   y_t   = S_t^T C_t + D x_t;   y_t *= silu(z_t);   unit RMS in norm_groups equal parts;   times a weight
// The recurrence is the delta mixer's scan without the correction term (delta.cu: linear_scan with delta_rule off, keys = B,
// queries = C, values = x, beta = dt, one decay per head), and the tails are written by delta_tails over the x | B | C
// columns.  Here:
//  * ssd_prep: two CTAs per row: convolution + bias + silu of the channels into fp32 x, B, C; dt and the decays.
//  * ssd_gate_norm: the skip term, the gate, the grouped RMS norm and the weight; one CTA per row, the row in shared memory.
#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void stx(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

constexpr int kSsdThreads = 256;

template <typename AT>
__global__ void __launch_bounds__(kSsdThreads)
ssd_prep_kernel(const AT* __restrict__ fused, int64_t ld, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const int32_t* __restrict__ positions,
                const int32_t* __restrict__ row_to_seq, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slots,
                const float* __restrict__ tails, int64_t slot_stride, float* __restrict__ xn, float* __restrict__ bn, float* __restrict__ cn,
                float* __restrict__ dt, float* __restrict__ decay, int heads, int groups, int state, int vdim, int taps) {
  const int64_t t = blockIdx.x;
  const int inner = heads * vdim, gn = groups * state, C = inner + 2 * gn;
  if (gridDim.x <= 128 && blockIdx.y == 0) {   // short steps wait on latency: weights and the tail go to L2 while the launch before runs
    prefetch_l2_span(conv_w, (size_t)C * taps * 4);
    if (conv_b) prefetch_l2_span(conv_b, (size_t)C * 4);
    if (tails) prefetch_l2_span(tails + (int64_t)seq_slots[row_to_seq ? row_to_seq[t] : (int)t] * slot_stride, (size_t)(taps - 1) * C * 4);
  }
  pdl_wait();
  pdl_launch_dependents();
  if (blockIdx.y == 1) {   // the second CTA of a row: step sizes and decays
    for (int h = threadIdx.x; h < heads; h += kSsdThreads) {
      const float d = softplus_f(ldx<AT>(fused, t * ld + inner + C + h) + dt_bias[h]);
      dt[t * heads + h] = d;
      decay[t * heads + h] = expf(-expf(a_log[h]) * d);
    }
    return;
  }
  const int s = row_to_seq ? row_to_seq[t] : (int)t;
  const int start = seq_start[s], r = (int)t - start, pos = positions[t];
  const float* tail = tails ? tails + (int64_t)seq_slots[s] * slot_stride : nullptr;   // [taps - 1][C]
  for (int c = threadIdx.x; c < C; c += kSsdThreads) {
    float a = conv_b ? conv_b[c] : 0.f;
    for (int j = 0; j < taps; ++j) {   // lag j: the input of position pos - j
      if (pos - j < 0) break;
      const float x = r - j >= 0 ? ldx<AT>(fused, (t - j) * ld + inner + c) : tail[(int64_t)(taps - 1 + r - j) * C + c];
      a = fmaf(conv_w[(int64_t)c * taps + taps - 1 - j], x, a);
    }
    a = a * sigmoid_f(a);
    if (c < inner) xn[t * inner + c] = a;
    else if (c < inner + gn) bn[t * gn + c - inner] = a;
    else cn[t * gn + c - inner - gn] = a;
  }
}

template <typename AT>
__global__ void __launch_bounds__(kSsdThreads)
ssd_gate_norm_kernel(const float* __restrict__ o, const float* __restrict__ xn, const float* __restrict__ skip, const AT* __restrict__ z,
                     int64_t ldz, const float* __restrict__ w, AT* __restrict__ out, int heads, int vdim, int norm_groups, float eps) {
  extern __shared__ float gy[];   // [inner] gated rows, then [norm_groups] scale factors
  if (gridDim.x <= 128) prefetch_l2_span(w, (size_t)heads * vdim * 4);
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const int inner = heads * vdim, per = inner / norm_groups;
  float* inv = gy + inner;
  for (int c = threadIdx.x; c < inner; c += kSsdThreads) {
    const float zv = ldx<AT>(z, t * ldz + c);
    gy[c] = fmaf(skip[c / vdim], xn[t * inner + c], o[t * inner + c]) * (zv * sigmoid_f(zv));
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < norm_groups; g += kSsdThreads / 32) {
    const float* src = gy + (int64_t)g * per;
    // four partial sums per lane shorten the chain of a long part; they are added in a fixed order
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int j = lane;
    for (; j + 96 < per; j += 128) {
      s0 = fmaf(src[j], src[j], s0);
      s1 = fmaf(src[j + 32], src[j + 32], s1);
      s2 = fmaf(src[j + 64], src[j + 64], s2);
      s3 = fmaf(src[j + 96], src[j + 96], s3);
    }
    for (; j < per; j += 32) s0 = fmaf(src[j], src[j], s0);
    const float ss = warp_sum((s0 + s1) + (s2 + s3));
    if (lane == 0) inv[g] = 1.0f / sqrtf(ss / (float)per + eps);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < inner; c += kSsdThreads) stx<AT>(out, t * inner + c, gy[c] * inv[c / per] * w[c]);
}

}  // namespace

int64_t ssd_tail_floats(int heads, int groups, int state, int vdim, int taps) {
  return (int64_t)(taps > 1 ? taps - 1 : 0) * (heads * vdim + 2 * groups * state);
}

int ssd_prep(bool f32, const void* fused, int64_t ld, const float* conv_w, const float* conv_b, const float* dt_bias, const float* a_log,
             const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots, const float* tails,
             int64_t slot_stride, float* xn, float* bn, float* cn, float* dt, float* decay, int T, int heads, int groups, int state, int vdim,
             int taps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && taps >= 1, B200_ERR_INVALID, "ssd_prep: %d heads over %d groups, %d taps", heads,
               groups, taps);
  B200_REQUIRE(taps == 1 || (tails && seq_slots), B200_ERR_INVALID, "ssd_prep: the convolution needs its tails");
  if (f32)
    B200_CUDA(launch(ssd_prep_kernel<float>, dim3(T, 2), dim3(kSsdThreads), (size_t)0, s, (const float*)fused, ld, conv_w, conv_b, dt_bias, a_log,
                     positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, xn, bn, cn, dt, decay, heads, groups, state, vdim, taps));
  else
    B200_CUDA(launch(ssd_prep_kernel<__nv_bfloat16>, dim3(T, 2), dim3(kSsdThreads), (size_t)0, s, (const __nv_bfloat16*)fused, ld, conv_w, conv_b,
                     dt_bias, a_log, positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, xn, bn, cn, dt, decay, heads, groups, state,
                     vdim, taps));
  return B200_OK;
}

int ssd_gate_norm(bool f32, const float* o, const float* xn, const float* skip, const void* z, int64_t ldz, const float* w, void* out, int T,
                  int heads, int vdim, int norm_groups, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  const int inner = heads * vdim;
  B200_REQUIRE(norm_groups >= 1 && inner % norm_groups == 0, B200_ERR_INVALID, "ssd_gate_norm: %d channels in %d parts", inner, norm_groups);
  const size_t smem = (size_t)(inner + norm_groups) * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "ssd_gate_norm: %d channels do not fit shared memory", inner);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(ssd_gate_norm_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(ssd_gate_norm_kernel<float>, dim3(T), dim3(kSsdThreads), smem, s, o, xn, skip, (const float*)z, ldz, w, (float*)out, heads,
                     vdim, norm_groups, eps));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(ssd_gate_norm_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(ssd_gate_norm_kernel<__nv_bfloat16>, dim3(T), dim3(kSsdThreads), smem, s, o, xn, skip, (const __nv_bfloat16*)z, ldz, w,
                     (__nv_bfloat16*)out, heads, vdim, norm_groups, eps));
  }
  return B200_OK;
}

}  // namespace b200
