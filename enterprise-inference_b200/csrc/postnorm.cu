// Mechanisms of the post-norm layer form (B200_FORM_POSTNORM) that have no place in the other forms' kernels:
//  * postnorm_stream: x = LN(alpha * x + y) * w + b over the fp32 residual stream, a layer norm WITH bias taken after the
//    sum (mean removed, variance = mean of squared deviations, both in fp32 over the row held in shared memory); writes the
//    fp32 stream and, for the bf16 mode, the rounded copy the next linears read.  With a row list it is the output norm.
//  * qk_headnorm_rotate_cache: attention whose values are its keys.  The raw key projection's leading vdim entries go to the
//    value cache; q and k are RMS-normalised per head with ONE weight of `dim` entries each, their leading rot_dims
//    dimensions turn in neighbouring pairs (2i, 2i + 1) by the angles of an fp32 cos|sin table; k goes to the key cache, q
//    leaves as fp32 rows.
//  * latent_norms: the two RMS norms of a latent mixer whose queries pass a latent of their own: the query latent into an
//    activation buffer, the key/value latent into its cache row.
#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void stx(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

constexpr int kPnThreads = 256;

__device__ __forceinline__ float block_sum256(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float a = 0.f;
#pragma unroll
  for (int i = 0; i < kPnThreads / 32; ++i) a += red[i];
  return a;
}

template <typename AT>
__global__ void __launch_bounds__(kPnThreads)
postnorm_stream_kernel(const float* x_in, const AT* __restrict__ y, float alpha, const float* __restrict__ w, const float* __restrict__ b,
                       float* x_out, AT* __restrict__ out_act, const int32_t* __restrict__ rows, int width, float eps) {
  extern __shared__ float pn_row[];
  __shared__ float red[kPnThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const int64_t xr = (rows ? (int64_t)rows[t] : t) * width, yr = t * width;
  float sum = 0.f;
  for (int c = threadIdx.x; c < width; c += kPnThreads) {
    float v = alpha * x_in[xr + c];
    if (y != nullptr) v += ldx<AT>(y, yr + c);
    pn_row[c] = v;
    sum += v;
  }
  const float mean = block_sum256(sum, red) / (float)width;
  float sq = 0.f;
  for (int c = threadIdx.x; c < width; c += kPnThreads) {
    const float d = pn_row[c] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = 1.0f / sqrtf(block_sum256(sq, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += kPnThreads) {
    const float v = (pn_row[c] - mean) * rstd * w[c] + (b ? b[c] : 0.f);
    if (x_out) x_out[yr + c] = v;
    if (out_act) stx<AT>(out_act, yr + c, v);
  }
}

// one CTA per row; a warp takes head vectors round robin (query heads, then key heads); a lane owns pairs lane, lane + 32, ...
template <typename AT, typename CT>
__global__ void __launch_bounds__(256)
qk_headnorm_rotate_cache_kernel(const AT* __restrict__ qk, int64_t ld, const float* __restrict__ qw, const float* __restrict__ kw,
                                const int32_t* __restrict__ positions, const int32_t* __restrict__ slots, const float* __restrict__ rot,
                                int rot_dims, int64_t max_pos, float* __restrict__ qout, CT* __restrict__ kc, CT* __restrict__ vc, int heads,
                                int kv_heads, int dim, int vdim, int block_size, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
  const int half = rot_dims >> 1;
  const float* cs = rot ? rot + (int64_t)pos * 2 * half : nullptr;
  const int slot = slots[t];
  const int64_t blk = slot >= 0 ? slot / block_size : 0, off = slot >= 0 ? slot % block_size : 0;
  for (int v = warp; v < heads + kv_heads; v += 8) {
    const bool is_q = v < heads;
    const int g = is_q ? v : v - heads;
    const AT* src = qk + t * ld + (int64_t)v * dim;
    const float* w = is_q ? qw : kw;
    float ss = 0.f;
    for (int i = lane; 2 * i < dim; i += 32) {
      const float a = ldx<AT>(src, 2 * i), b = ldx<AT>(src, 2 * i + 1);
      ss = fmaf(a, a, fmaf(b, b, ss));
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    const int64_t crow = ((blk * kv_heads + g) * block_size + off);
    for (int i = lane; 2 * i < dim; i += 32) {
      const float a = ldx<AT>(src, 2 * i), b = ldx<AT>(src, 2 * i + 1);
      if (!is_q && slot >= 0) {
        if (2 * i < vdim) stx<CT>(vc, crow * vdim + 2 * i, a);
        if (2 * i + 1 < vdim) stx<CT>(vc, crow * vdim + 2 * i + 1, b);
      }
      float n0 = a * inv * w[2 * i], n1 = b * inv * w[2 * i + 1];
      if (cs && i < half) {
        const float c = cs[i], sn = cs[half + i];
        const float o0 = fmaf(n0, c, -n1 * sn), o1 = fmaf(n1, c, n0 * sn);
        n0 = o0;
        n1 = o1;
      }
      if (is_q) {
        qout[(t * heads + g) * dim + 2 * i] = n0;
        qout[(t * heads + g) * dim + 2 * i + 1] = n1;
      } else if (slot >= 0) {
        stx<CT>(kc, crow * dim + 2 * i, n0);
        stx<CT>(kc, crow * dim + 2 * i + 1, n1);
      }
    }
  }
}

template <typename AT>
__global__ void __launch_bounds__(128)
latent_norms_kernel(const AT* __restrict__ fused, int64_t ld, int q_rank, int kv_rank, const float* __restrict__ qw, const float* __restrict__ kw,
                    const int32_t* __restrict__ slots, AT* __restrict__ cq, AT* __restrict__ cache, float eps) {
  __shared__ float red[2][4];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const AT* row = fused + t * ld;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < q_rank; c += 128) {
    const float v = ldx<AT>(row, c);
    sq = fmaf(v, v, sq);
  }
  if (cache)
    for (int c = threadIdx.x; c < kv_rank; c += 128) {
      const float v = ldx<AT>(row, q_rank + c);
      sk = fmaf(v, v, sk);
    }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = sq;
    red[1][threadIdx.x >> 5] = sk;
  }
  __syncthreads();
  if (q_rank > 0) {
    const float inv = 1.0f / sqrtf(((red[0][0] + red[0][1]) + (red[0][2] + red[0][3])) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += 128) stx<AT>(cq, t * q_rank + c, ldx<AT>(row, c) * inv * qw[c]);
  }
  if (cache && slots[t] >= 0) {
    const float inv = 1.0f / sqrtf(((red[1][0] + red[1][1]) + (red[1][2] + red[1][3])) / (float)kv_rank + eps);
    AT* dst = cache + (int64_t)slots[t] * kv_rank;
    for (int c = threadIdx.x; c < kv_rank; c += 128) stx<AT>(dst, c, ldx<AT>(row, q_rank + c) * inv * kw[c]);
  }
}

}  // namespace

int postnorm_stream(bool f32, const float* x_in, const void* y, float alpha, const float* w, const float* b, float* x_out, void* out_act,
                    const int32_t* rows, int R, int width, float eps, cudaStream_t s) {
  if (R == 0) return B200_OK;
  B200_REQUIRE(x_in && w && (x_out || out_act), B200_ERR_INVALID, "postnorm: null argument");
  B200_REQUIRE(!(rows && x_out == x_in), B200_ERR_INVALID, "postnorm: gathered rows cannot be normalised in place");
  const size_t smem = (size_t)width * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "postnorm: width %d does not fit shared memory", width);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(postnorm_stream_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(postnorm_stream_kernel<float>, dim3(R), dim3(kPnThreads), smem, s, x_in, (const float*)y, alpha, w, b, x_out,
                     (float*)out_act, rows, width, eps));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(postnorm_stream_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(postnorm_stream_kernel<__nv_bfloat16>, dim3(R), dim3(kPnThreads), smem, s, x_in, (const __nv_bfloat16*)y, alpha, w, b,
                     x_out, (__nv_bfloat16*)out_act, rows, width, eps));
  }
  return B200_OK;
}

int qk_headnorm_rotate_cache(bool f32, const void* qk, int64_t ld, const float* qw, const float* kw, const int32_t* positions,
                             const int32_t* slots, const float* rot, int rot_dims, int64_t max_pos, float* qout, void* kc, void* vc, int T,
                             int heads, int kv_heads, int dim, int vdim, int block_size, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(dim % 2 == 0 && rot_dims % 2 == 0 && rot_dims <= dim && vdim <= dim && vdim > 0, B200_ERR_UNSUPPORTED,
               "head norm: key size %d (even), %d rotated, value size %d (at most the key size)", dim, rot_dims, vdim);
  if (f32)
    B200_CUDA(launch(qk_headnorm_rotate_cache_kernel<float, float>, dim3(T), dim3(256), (size_t)0, s, (const float*)qk, ld, qw, kw, positions,
                     slots, rot, rot ? rot_dims : 0, max_pos, qout, (float*)kc, (float*)vc, heads, kv_heads, dim, vdim, block_size, eps));
  else
    B200_CUDA(launch(qk_headnorm_rotate_cache_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), (size_t)0, s,
                     (const __nv_bfloat16*)qk, ld, qw, kw, positions, slots, rot, rot ? rot_dims : 0, max_pos, qout, (__nv_bfloat16*)kc,
                     (__nv_bfloat16*)vc, heads, kv_heads, dim, vdim, block_size, eps));
  return B200_OK;
}

int latent_norms(bool f32, const void* fused, int64_t ld, int q_rank, int kv_rank, const float* qw, const float* kw, const int32_t* slots,
                 void* cq, void* cache, int T, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(fused && (q_rank == 0 || (qw && cq)) && (!cache || (kw && slots && kv_rank > 0)), B200_ERR_INVALID, "latent_norms: null argument");
  if (f32)
    B200_CUDA(launch(latent_norms_kernel<float>, dim3(T), dim3(128), (size_t)0, s, (const float*)fused, ld, q_rank, kv_rank, qw, kw, slots,
                     (float*)cq, (float*)cache, eps));
  else
    B200_CUDA(launch(latent_norms_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, s, (const __nv_bfloat16*)fused, ld, q_rank, kv_rank, qw,
                     kw, slots, (__nv_bfloat16*)cq, (__nv_bfloat16*)cache, eps));
  return B200_OK;
}

}  // namespace b200
