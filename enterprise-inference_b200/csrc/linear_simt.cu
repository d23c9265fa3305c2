// y[T][n_out] = x[T][k] . w[n_out][k]^T on CUDA cores in true fp32 (no reduced-precision matrix mode): the linear of the
// 32-bit serving mode, and of shapes the tcgen05 path cannot address.  Weights stay bf16 in memory (their values are
// exact in fp32); activations are fp32 or bf16 on either side.  64 x 64 output tile per CTA, k in steps of 16 through
// shared memory, a 4 x 4 micro-tile per thread; the k loop runs in order, so a row's sums do not depend on what else is
// in the step.  Every 16-wide k block is summed on its own and then added to the running total: the rounding error of a
// sum over k terms grows with sqrt(16) + sqrt(k / 16) instead of sqrt(k).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kBM = 64, kBN = 64, kBK = 16;

template <typename T> __device__ __forceinline__ float ldf(const T* p, int64_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

template <typename XT, typename YT>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const XT* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w, YT* __restrict__ y, int64_t ldy,
                   int T, int n_out, int k) {
  __shared__ float xs[kBK][kBM + 1];
  __shared__ float ws[kBK][kBN + 1];
  pdl_wait();
  pdl_launch_dependents();
  const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx: 4 output features, ty: 4 token rows
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < k; k0 += kBK) {
    for (int i = threadIdx.x; i < kBM * kBK; i += 256) {
      const int r = i / kBK, c = i % kBK;
      xs[c][r] = (m0 + r < T && k0 + c < k) ? ldf<XT>(x, (int64_t)(m0 + r) * ldx + k0 + c) : 0.f;
    }
    for (int i = threadIdx.x; i < kBN * kBK; i += 256) {
      const int r = i / kBK, c = i % kBK;
      ws[c][r] = (n0 + r < n_out && k0 + c < k) ? __bfloat162float(w[(int64_t)(n0 + r) * k + k0 + c]) : 0.f;
    }
    __syncthreads();
    float part[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
    for (int c = 0; c < kBK; ++c) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[c][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = m0 + ty * 4 + i, cidx = n0 + tx * 4 + j;
      if (r < T && cidx < n_out) stf<YT>(y, (int64_t)r * ldy + cidx, acc[i][j]);
    }
}

}  // namespace

// x_f32 / y_f32: element type of the activations on either side (false: bf16)
int linear_simt(bool x_f32, bool y_f32, const void* x, int64_t ldx, const __nv_bfloat16* w, void* y, int64_t ldy, int T, int n_out,
                int k, cudaStream_t s) {
  if (T == 0) return B200_OK;
  const dim3 grid((n_out + kBN - 1) / kBN, (T + kBM - 1) / kBM), block(256);
  if (x_f32 && y_f32)
    B200_CUDA(launch(linear_simt_kernel<float, float>, grid, block, 0, s, (const float*)x, ldx, w, (float*)y, ldy, T, n_out, k));
  else if (!x_f32 && !y_f32)
    B200_CUDA(launch(linear_simt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)x, ldx, w,
                     (__nv_bfloat16*)y, ldy, T, n_out, k));
  else if (x_f32)
    B200_CUDA(launch(linear_simt_kernel<float, __nv_bfloat16>, grid, block, 0, s, (const float*)x, ldx, w, (__nv_bfloat16*)y, ldy,
                     T, n_out, k));
  else
    B200_CUDA(launch(linear_simt_kernel<__nv_bfloat16, float>, grid, block, 0, s, (const __nv_bfloat16*)x, ldx, w, (float*)y, ldy, T,
                     n_out, k));
  return B200_OK;
}

}  // namespace b200
