// Latent attention (B200_MIXER_LATENT): what surrounds the paged attention kernel.
//
// Per token the fused projection gives queries (per head `dim` plain + `rot_dim` rotated dimensions), a latent of kv_rank
// dimensions and one rotated key part shared by all heads.  Only [normed latent | rotated key part] is cached.  A head's
// plain key is W_uk c, so q_plain . (W_uk c) = (W_uk^T q_plain) . c: the scores are taken against the cached rows directly
// with q' = [W_uk^T q_plain | rotated q] (one kv head of kv_rank + rot_dim dimensions), the weighted sum of the cached
// latents (the row's first kv_rank entries are the "values") is expanded by W_uv afterwards.
//
//  * latent_prep: RMS norm of the latent with its weight, rotation of the shared key part and of every head's rotated query
//    part (interleaved pairs, fp32 cos|sin table), cache append, rotated query parts into the fp32 query rows;
//  * head_linear: y[t][h] = W[h] x[t][h] for every head at once, strided rows in and out, fp32 accumulation, optional
//    sigmoid gate on the output (the output gate of the mixer reads the same input as the projections).
#include <stdlib.h>

#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void stx(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// one CTA (128 threads) per row
template <typename AT>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const AT* __restrict__ qkv, int64_t ld, const float* __restrict__ norm_w, const int32_t* __restrict__ positions,
                   const int32_t* __restrict__ slots, const float* __restrict__ rot, int rot_dims, int64_t max_pos,
                   float* __restrict__ qfull, AT* __restrict__ cache, int heads, int dim, int rot_dim, int kv_rank, float eps) {
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const AT* row = qkv + t * ld;
  const int qh = dim + rot_dim, krow = kv_rank + rot_dim;
  const AT* dkv = row + (int64_t)heads * qh;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
  const int half = rot_dims >> 1;
  const float* cs = rot ? rot + (int64_t)pos * 2 * half : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += 128) {
    const float v = ldx<AT>(dkv, c);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)kv_rank + eps);
  AT* dst = cache + (int64_t)slots[t] * krow;
  for (int c = threadIdx.x; c < kv_rank; c += 128) stx<AT>(dst, c, ldx<AT>(dkv, c) * inv * norm_w[c]);
  // rotated parts: index e over (heads + 1) vectors of rot_dim entries; vector `heads` is the shared key part
  for (int e = threadIdx.x; e < (heads + 1) * rot_dim; e += 128) {
    const int hv = e / rot_dim, i = e % rot_dim;
    const AT* src = hv < heads ? row + (int64_t)hv * qh + dim : dkv + kv_rank;
    float v = ldx<AT>(src, i);
    if (cs && i < 2 * half) {
      const float o = ldx<AT>(src, i ^ 1), c = cs[i >> 1], s = cs[half + (i >> 1)];
      v = (i & 1) ? fmaf(v, c, o * s) : fmaf(v, c, -o * s);
    }
    if (hv < heads) qfull[(t * heads + hv) * krow + kv_rank + i] = v;
    else stx<AT>(dst, kv_rank + i, v);
  }
}

// CTA = (tile of kHlRows rows, head).  The rows' inputs are staged in shared memory as fp32; warp w owns outputs w, w + 8,
// ...; a lane strides the inner dimension for all rows at once.
constexpr int kHlRows = 16;
template <typename AT, typename YT>
__global__ void __launch_bounds__(256)
head_linear_kernel(const AT* __restrict__ x, int64_t ldx_, int x_hs, const __nv_bfloat16* __restrict__ w, YT* __restrict__ y, int64_t ldy,
                   int y_hs, const AT* __restrict__ gate, int64_t ldg, int g_hs, int g_es, int T, int n_out, int k) {
  extern __shared__ float xs[];   // [kHlRows][k]
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * kHlRows, h = blockIdx.y, nr = min(kHlRows, T - t0);
  for (int i = threadIdx.x; i < kHlRows * k; i += 256) {
    const int r = i / k, c = i % k;
    xs[i] = r < nr ? ldx<AT>(x, (int64_t)(t0 + r) * ldx_ + (int64_t)h * x_hs + c) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* wh = w + (int64_t)h * n_out * k;
  for (int o = warp; o < n_out; o += 8) {
    const __nv_bfloat16* wr = wh + (int64_t)o * k;
    float acc[kHlRows];
#pragma unroll
    for (int r = 0; r < kHlRows; ++r) acc[r] = 0.f;
    for (int c = lane; c < k; c += 32) {
      const float wv = __bfloat162float(wr[c]);
#pragma unroll
      for (int r = 0; r < kHlRows; ++r) acc[r] = fmaf(wv, xs[r * k + c], acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kHlRows; ++r) {
      float v = warp_sum(acc[r]);
      if (lane == 0 && r < nr) {
        if (gate) v *= 1.0f / (1.0f + expf(-ldx<AT>(gate, (int64_t)(t0 + r) * ldg + (int64_t)h * g_hs + (int64_t)o * g_es)));
        stx<YT>(y, (int64_t)(t0 + r) * ldy + (int64_t)h * y_hs + o, v);
      }
    }
  }
}

// ---- the same per-head products on the tensor cores (bf16 inputs, inner size a multiple of 16) --------------------------------
// CTA = (64 rows, head, 64 outputs); warp w owns rows 16w .. 16w + 15.  Inputs and the head's weight rows are staged in
// shared memory in inner chunks of 128 (16-byte copies when the input rows allow it) and multiplied as bf16 mma.sync
// m16n8k16 with fp32 accumulators; the epilogue applies the optional sigmoid gate and stores fp32 or bf16.
constexpr int kHmRows = 64, kHmOuts = 64, kHmChunk = 128, kHmStride = kHmChunk + 8;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float& c0, float& c1, float& c2, float& c3, const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename YT, bool VEC>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx_, int x_hs, const __nv_bfloat16* __restrict__ w, YT* __restrict__ y,
                       int64_t ldy, int y_hs, const __nv_bfloat16* __restrict__ gate, int64_t ldg, int g_hs, int g_es, int T, int n_out, int k) {
  __shared__ __align__(16) __nv_bfloat16 Xs[kHmRows * kHmStride];
  __shared__ __align__(16) __nv_bfloat16 Ws[kHmOuts * kHmStride];
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * kHmRows, h = blockIdx.y, o0 = blockIdx.z * kHmOuts;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const __nv_bfloat16* wh = w + ((int64_t)h * n_out + o0) * k;
  for (int k0 = 0; k0 < k; k0 += kHmChunk) {
    const int kc = min(kHmChunk, k - k0), cpr = kc >> 3;
    // two threads per row (input rows and weight rows alike), alternate 16-byte chunks
    const int r = tid >> 1;
    {
      const bool live = t0 + r < T;
      const __nv_bfloat16* src = x + (int64_t)(t0 + r) * ldx_ + (int64_t)h * x_hs + k0;
      __nv_bfloat16* dst = Xs + r * kHmStride;
      for (int c = tid & 1; c < cpr; c += 2) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (live) {
          if (VEC) {
            v = __ldg(reinterpret_cast<const uint4*>(src + c * 8));
          } else {
            const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src + c * 8);
            v.x = s16[0] | ((uint32_t)s16[1] << 16);
            v.y = s16[2] | ((uint32_t)s16[3] << 16);
            v.z = s16[4] | ((uint32_t)s16[5] << 16);
            v.w = s16[6] | ((uint32_t)s16[7] << 16);
          }
        }
        *reinterpret_cast<uint4*>(dst + c * 8) = v;
      }
    }
    {
      const bool live = o0 + r < n_out;
      const __nv_bfloat16* src = wh + (int64_t)r * k + k0;
      __nv_bfloat16* dst = Ws + r * kHmStride;
      for (int c = tid & 1; c < cpr; c += 2)
        *reinterpret_cast<uint4*>(dst + c * 8) = live ? __ldg(reinterpret_cast<const uint4*>(src + c * 8)) : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    const __nv_bfloat16* ap = Xs + (warp * 16 + (lane & 15)) * kHmStride + (lane >> 4) * 8;
    const __nv_bfloat16* bp = Ws + ((lane & 7) + (lane >> 4) * 8) * kHmStride + ((lane >> 3) & 1) * 8;
    for (int kk = 0; kk < kc; kk += 16) {
      uint32_t a[4];
      ldsm_x4(a, ap + kk);
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t b[4];
        ldsm_x4(b, bp + n2 * 16 * kHmStride + kk);
        mma_bf16(acc[2 * n2][0], acc[2 * n2][1], acc[2 * n2][2], acc[2 * n2][3], a, b[0], b[1]);
        mma_bf16(acc[2 * n2 + 1][0], acc[2 * n2 + 1][1], acc[2 * n2 + 1][2], acc[2 * n2 + 1][3], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int t = t0 + warp * 16 + (lane >> 2) + half * 8;
    if (t >= T) continue;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int o = o0 + nt * 8 + (lane & 3) * 2 + e;
        if (o >= n_out) continue;
        float v = acc[nt][half * 2 + e];
        if (gate) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(int64_t)t * ldg + (int64_t)h * g_hs + (int64_t)o * g_es])));
        stx<YT>(y, (int64_t)t * ldy + (int64_t)h * y_hs + o, v);
      }
    }
  }
}

}  // namespace

int latent_prep(bool f32, const void* qkv, int64_t ld, const float* norm_w, const int32_t* positions, const int32_t* slots,
                const float* rot, int rot_dims, int64_t max_pos, float* qfull, void* cache, int T, int heads, int dim, int rot_dim,
                int kv_rank, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0, B200_ERR_INVALID, "latent_prep: %d of %d dimensions rotate",
               rot_dims, rot_dim);
  if (f32)
    B200_CUDA(launch(latent_prep_kernel<float>, dim3(T), dim3(128), (size_t)0, s, (const float*)qkv, ld, norm_w, positions, slots, rot,
                     rot ? rot_dims : 0, max_pos, qfull, (float*)cache, heads, dim, rot_dim, kv_rank, eps));
  else
    B200_CUDA(launch(latent_prep_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, s, (const __nv_bfloat16*)qkv, ld, norm_w, positions,
                     slots, rot, rot ? rot_dims : 0, max_pos, qfull, (__nv_bfloat16*)cache, heads, dim, rot_dim, kv_rank, eps));
  return B200_OK;
}

template <typename AT, typename YT>
static int head_linear_t(const void* x, int64_t ldx_, int x_hs, const __nv_bfloat16* w, void* y, int64_t ldy, int y_hs, const void* gate,
                         int64_t ldg, int g_hs, int g_es, int T, int heads, int n_out, int k, cudaStream_t s) {
  const size_t smem = (size_t)kHlRows * k * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "head_linear: inner size %d does not fit shared memory", k);
  static bool done[64] = {};
  if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(head_linear_kernel<AT, YT>, 200 * 1024, done));
  B200_CUDA(launch(head_linear_kernel<AT, YT>, dim3((T + kHlRows - 1) / kHlRows, heads), dim3(256), smem, s, (const AT*)x, ldx_, x_hs, w,
                   (YT*)y, ldy, y_hs, (const AT*)gate, ldg, g_hs, g_es, T, n_out, k));
  return B200_OK;
}

// x, gate: activation type (fp32 when f32, else bf16); y: fp32 when y_f32, else the activation type.  g_es: stride of the gate
// inside a head (1: one gate per output, 0: one gate per head)
int head_linear(bool f32, bool y_f32, const void* x, int64_t ldx_, int x_hs, const __nv_bfloat16* w, void* y, int64_t ldy, int y_hs,
                const void* gate, int64_t ldg, int g_hs, int T, int heads, int n_out, int k, cudaStream_t s, int g_es) {
  if (T == 0) return B200_OK;
  static const int mma_env = getenv("B200_HEAD_LINEAR_MMA") ? atoi(getenv("B200_HEAD_LINEAR_MMA")) : 1;
  if (!f32 && mma_env && k % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
    const bool vec = ldx_ % 8 == 0 && x_hs % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
    const dim3 grid((T + kHmRows - 1) / kHmRows, heads, (n_out + kHmOuts - 1) / kHmOuts), block(128);
#define HM(YT, VEC)                                                                                                               \
  B200_CUDA(launch(head_linear_mma_kernel<YT, VEC>, grid, block, (size_t)0, s, (const __nv_bfloat16*)x, ldx_, x_hs, w, (YT*)y, ldy, y_hs, \
                   (const __nv_bfloat16*)gate, ldg, g_hs, g_es, T, n_out, k))
    if (y_f32) {
      if (vec) HM(float, true); else HM(float, false);
    } else {
      if (vec) HM(__nv_bfloat16, true); else HM(__nv_bfloat16, false);
    }
#undef HM
    return B200_OK;
  }
  if (f32) return head_linear_t<float, float>(x, ldx_, x_hs, w, y, ldy, y_hs, gate, ldg, g_hs, g_es, T, heads, n_out, k, s);
  if (y_f32) return head_linear_t<__nv_bfloat16, float>(x, ldx_, x_hs, w, y, ldy, y_hs, gate, ldg, g_hs, g_es, T, heads, n_out, k, s);
  return head_linear_t<__nv_bfloat16, __nv_bfloat16>(x, ldx_, x_hs, w, y, ldy, y_hs, gate, ldg, g_hs, g_es, T, heads, n_out, k, s);
}

}  // namespace b200
