// Mechanisms of the multi-stream pre-norm layer form (B200_FORM_HYPER) that have no place in the other forms' kernels:
//  * hyper_step: the residual is n fp32 streams X_1..X_n.  One launch closes a sublayer and opens the next:
//      close:  X_t = sum_s M[s][t] X_s + mult * b[t] * scale[c] * y        for every t from the OLD streams (M indexed from, to)
//      open:   u = sum_s a[s] X_s;   h = (u - mean) / sqrt(var + eps) * w + bias      (var = mean of squared deviations)
//    Streams are elementwise in the channel, so a thread keeps the n values of its channels in registers; only u is
//    staged (one row in shared memory) for the two statistics passes.  The first launch of a step copies stream 0 (the
//    scaled embedding) into every stream; the last one runs over the logit rows only, with a = ones and the output norm.
//    y is an activation row or the sum, in slot order, of n_parts fp32 partial rows (routed experts).  A step whose sequences
//    bring one row each (decode) also runs the input convolution here: its earlier taps are the tail in the state slot.
//  * qkv_rotate_cache: plain q | k | v projections; the leading rot_dims dimensions of every q and k head turn by the
//    angles of an fp32 cos|sin table, dimension i paired with i + rot_dims / 2 (half layout) or 2i with 2i + 1; q leaves
//    as fp32 rows, k and v go to the paged caches.
//  * polynorm: p(z) = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 over the ff entries of a token, N(v) = v / sqrt(mean(v^2) + eps);
//    the three mean squares come from one pass over the row (z^2, z^4, z^6), all in fp32.
#include <algorithm>

#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ldx(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ldx<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void stx(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void stx<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stx<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

constexpr int kHyThreads = 256;
constexpr int kMaxN = B200_MAX_STREAMS;
constexpr int kHyMaxTaps = 16;

// sum over the CTA (any number of warps up to 32)
__device__ __forceinline__ float block_sum_hy(float v, float* red) {
  v = warp_sum(v);
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float a = 0.f;
  for (int i = 0; i < nw; ++i) a += red[i];
  return a;
}

template <typename AT, int V> __device__ __forceinline__ void ldv(const AT* p, int64_t i, float* o);
template <> __device__ __forceinline__ void ldv<float, 1>(const float* p, int64_t i, float* o) { o[0] = p[i]; }
template <> __device__ __forceinline__ void ldv<__nv_bfloat16, 1>(const __nv_bfloat16* p, int64_t i, float* o) { o[0] = __bfloat162float(p[i]); }
template <> __device__ __forceinline__ void ldv<float, 4>(const float* p, int64_t i, float* o) {
  const float4 v = *reinterpret_cast<const float4*>(p + i);
  o[0] = v.x, o[1] = v.y, o[2] = v.z, o[3] = v.w;
}
template <> __device__ __forceinline__ void ldv<__nv_bfloat16, 4>(const __nv_bfloat16* p, int64_t i, float* o) {
  const uint2 v = *reinterpret_cast<const uint2*>(p + i);
  o[0] = bf16lo(v.x), o[1] = bf16hi(v.x), o[2] = bf16lo(v.y), o[3] = bf16hi(v.y);
}
template <typename AT, int V> __device__ __forceinline__ void stv(AT* p, int64_t i, const float* o);
template <> __device__ __forceinline__ void stv<float, 1>(float* p, int64_t i, const float* o) { p[i] = o[0]; }
template <> __device__ __forceinline__ void stv<__nv_bfloat16, 1>(__nv_bfloat16* p, int64_t i, const float* o) { p[i] = __float2bfloat16_rn(o[0]); }
template <> __device__ __forceinline__ void stv<float, 4>(float* p, int64_t i, const float* o) {
  *reinterpret_cast<float4*>(p + i) = make_float4(o[0], o[1], o[2], o[3]);
}
template <> __device__ __forceinline__ void stv<__nv_bfloat16, 4>(__nv_bfloat16* p, int64_t i, const float* o) {
  *reinterpret_cast<uint2*>(p + i) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// The input convolution of a step whose sequences bring ONE row each (decode steps), fused behind the norm: the taps before
// the row's own come from the sequence's tail in its state slot, which is shifted by one place and takes the row.
struct HyperConv {
  const float* w = nullptr;            // [width][taps]; nullptr: no fused convolution
  int taps = 0;
  const int32_t* positions = nullptr;
  const int32_t* row_to_seq = nullptr;
  const int32_t* seq_slots = nullptr;
  float* tails = nullptr;              // this sublayer's tail of slot 0: [taps - 1][width]
  int64_t slot_stride = 0;
};

// V channels per thread and trip (4: 16-byte accesses; the row length and every pointer then are multiples of 4 floats)
template <typename AT, int N, int V>
__global__ void __launch_bounds__(1024)
hyper_step_kernel(float* X, int64_t sstride, int init, const AT* __restrict__ y, const float* __restrict__ parts, int n_parts,
                  const float* __restrict__ scale, const float* __restrict__ hc, float mult, const float* __restrict__ open_in,
                  const float* __restrict__ nw, const float* __restrict__ nb, float eps, const int32_t* __restrict__ rows,
                  float* __restrict__ h_f32, AT* __restrict__ h_act, float* __restrict__ sum_out, int width, HyperConv cv) {
  extern __shared__ __align__(16) float hy_row[];
  __shared__ float red[32];
  __shared__ float coef[2 * kMaxN + kMaxN * kMaxN + kMaxN];   // a | b | M of the closing sublayer, then the opening a
  __shared__ float* cv_slot_tail;
  __shared__ int cv_pos;
  // Weights do not depend on the launch before: the coefficients are fetched, and the rows of weights the later phases
  // read are asked into L2, while that launch still runs (programmatic dependent launch).
  const int nt = blockDim.x;
  for (int i = threadIdx.x; i < 2 * N + N * N; i += nt) coef[i] = hc ? hc[i] : 0.f;
  if (threadIdx.x < N) coef[2 * N + N * N + threadIdx.x] = open_in ? open_in[threadIdx.x] : 1.0f;
  if (gridDim.x <= 256) {   // short steps: every CTA is on an SM at once and waits on latency, not on bandwidth
    for (int c = threadIdx.x * 32; c < width; c += nt * 32) {
      if (hc) prefetch_l2(scale + c);
      if (nw) prefetch_l2(nw + c);
      if (nb) prefetch_l2(nb + c);
    }
    if (cv.w)
      for (int c = threadIdx.x * 32; c < width * cv.taps; c += nt * 32) prefetch_l2(cv.w + c);
  }
  if (cv.w) {
    // the row's sequence, slot and position are step inputs (copied in before the step's first launch): the chain of lookups
    // and the tail's way into L2 also run ahead of the wait
    const int sq = cv.row_to_seq ? cv.row_to_seq[blockIdx.x] : (int)blockIdx.x;
    const int hist0 = cv.taps - 1;
    const float* tl = hist0 ? cv.tails + (int64_t)cv.seq_slots[sq] * cv.slot_stride : nullptr;
    if (threadIdx.x == 0) {
      cv_slot_tail = const_cast<float*>(tl);
      cv_pos = cv.positions[blockIdx.x];
    }
    if (tl)
      for (int c = threadIdx.x * 32; c < width * hist0; c += nt * 32) prefetch_l2(tl + c);
  }
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const int64_t src = rows ? (int64_t)rows[t] : t;
  __syncthreads();
  const float* cb = coef + N;
  const float* cm = coef + 2 * N;
  const float* ca = coef + 2 * N + N * N;
  float sum = 0.f;
  for (int c = threadIdx.x * V; c < width; c += nt * V) {
    float xs[N][V], u[V], all[V];
#pragma unroll
    for (int s = 0; s < N; ++s) ldv<float, V>(X, (init ? 0 : s) * sstride + src * width + c, xs[s]);
#pragma unroll
    for (int v = 0; v < V; ++v) u[v] = all[v] = 0.f;
    if (hc) {
      float yv[V];
      if (y) {
        ldv<AT, V>(y, src * width + c, yv);
      } else {
#pragma unroll
        for (int v = 0; v < V; ++v) yv[v] = 0.f;
        for (int j = 0; j < n_parts; ++j) {
          float pv[V];
          ldv<float, V>(parts, (src * n_parts + j) * width + c, pv);
#pragma unroll
          for (int v = 0; v < V; ++v) yv[v] += pv[v];
        }
      }
      float sc[V];
      ldv<float, V>(scale, c, sc);
#pragma unroll
      for (int v = 0; v < V; ++v) yv[v] = yv[v] * sc[v] * mult;
#pragma unroll
      for (int q = 0; q < N; ++q) {
        float a[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < N; ++s) acc = fmaf(cm[s * N + q], xs[s][v], acc);
          a[v] = fmaf(cb[q], yv[v], acc);
          u[v] = fmaf(ca[q], a[v], u[v]);
          all[v] += a[v];
        }
        if (!rows) stv<float, V>(X, q * sstride + src * width + c, a);
      }
    } else {
#pragma unroll
      for (int q = 0; q < N; ++q) {
#pragma unroll
        for (int v = 0; v < V; ++v) {
          u[v] = fmaf(ca[q], xs[q][v], u[v]);
          all[v] += xs[q][v];
        }
        if (init && !rows && q > 0) stv<float, V>(X, q * sstride + src * width + c, xs[q]);
      }
    }
    if (sum_out) stv<float, V>(sum_out, t * width + c, all);
    stv<float, V>(hy_row, c, u);
#pragma unroll
    for (int v = 0; v < V; ++v) sum += u[v];
  }
  if (!h_f32 && !h_act) return;
  if (!nw) {
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += nt) {
      if (h_f32) h_f32[t * width + c] = hy_row[c];
      if (h_act) stv<AT, 1>(h_act, t * width + c, hy_row + c);
    }
    return;
  }
  const float mean = block_sum_hy(sum, red) / (float)width;
  float sq = 0.f;
  for (int c = threadIdx.x * V; c < width; c += nt * V) {
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const float d = hy_row[c + v] - mean;
      sq = fmaf(d, d, sq);
    }
  }
  const float rstd = 1.0f / sqrtf(block_sum_hy(sq, red) / (float)width + eps);
  if (cv.w == nullptr) {
    for (int c = threadIdx.x * V; c < width; c += nt * V) {
      float wv[V], bv[V], o[V];
      ldv<float, V>(nw, c, wv);
      if (nb) ldv<float, V>(nb, c, bv);
#pragma unroll
      for (int v = 0; v < V; ++v) o[v] = (hy_row[c + v] - mean) * rstd * wv[v] + (nb ? bv[v] : 0.f);
      if (h_f32) stv<float, V>(h_f32, t * width + c, o);
      if (h_act) stv<AT, V>(h_act, t * width + c, o);
    }
    return;
  }
  // one row per sequence: out = h + sum_j w[:, j] in_j with in_(taps-1) = h and the earlier inputs from the tail
  const int hist = cv.taps - 1, p0 = cv_pos;
  float* tail = cv_slot_tail;
  for (int c = threadIdx.x; c < width; c += nt) {
    const float h = (hy_row[c] - mean) * rstd * nw[c] + (nb ? nb[c] : 0.f);
    float old[kHyMaxTaps];
#pragma unroll
    for (int i = 0; i < kHyMaxTaps; ++i) old[i] = (i < hist && p0 - hist + i >= 0) ? tail[(int64_t)i * width + c] : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < kHyMaxTaps; ++j)
      if (j < cv.taps) acc = fmaf(cv.w[c * cv.taps + j], j == hist ? h : old[j], acc);
    const float o = h + acc;
    stv<AT, 1>(h_act, t * width + c, &o);
#pragma unroll
    for (int i = 0; i < kHyMaxTaps; ++i)
      if (i < hist) tail[(int64_t)i * width + c] = i + 1 < hist ? old[i + 1] : h;
  }
}

// one CTA per row; a warp takes head vectors round robin (query heads, key heads, value heads)
template <typename AT, typename CT>
__global__ void __launch_bounds__(256)
qkv_rotate_cache_kernel(const AT* __restrict__ qkv, int64_t ld, const int32_t* __restrict__ positions, const int32_t* __restrict__ slots,
                        const float* __restrict__ rot, int rot_dims, int half_layout, int64_t max_pos, float* __restrict__ qout,
                        CT* __restrict__ kc, CT* __restrict__ vc, int heads, int kv_heads, int dim, int vdim, int block_size) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
  const int half = rot ? rot_dims >> 1 : 0;
  const float* cs = rot ? rot + (int64_t)pos * 2 * half : nullptr;
  const int slot = slots[t];
  const int64_t blk = slot >= 0 ? slot / block_size : 0, off = slot >= 0 ? slot % block_size : 0;
  const int nqk = heads + kv_heads;
  for (int v = warp; v < nqk + kv_heads; v += 8) {
    if (v >= nqk) {   // a value head: copied
      if (slot < 0) continue;
      const int g = v - nqk;
      const AT* src = qkv + t * ld + (int64_t)nqk * dim + (int64_t)g * vdim;
      CT* dst = vc + ((blk * kv_heads + g) * block_size + off) * vdim;
      for (int i = lane; i < vdim; i += 32) stx<CT>(dst, i, ldx<AT>(src, i));
      continue;
    }
    const bool is_q = v < heads;
    const int g = is_q ? v : v - heads;
    if (!is_q && slot < 0) continue;
    const AT* src = qkv + t * ld + (int64_t)v * dim;
    float* qd = qout + (t * heads + g) * dim;
    CT* kd = kc + ((blk * kv_heads + g) * block_size + off) * dim;
    for (int i = lane; i < half; i += 32) {   // the pairs that turn
      const int i0 = half_layout ? i : 2 * i, i1 = half_layout ? i + half : 2 * i + 1;
      const float a = ldx<AT>(src, i0), b = ldx<AT>(src, i1), c = cs[i], sn = cs[half + i];
      const float o0 = fmaf(a, c, -b * sn), o1 = fmaf(b, c, a * sn);
      if (is_q) {
        qd[i0] = o0;
        qd[i1] = o1;
      } else {
        stx<CT>(kd, i0, o0);
        stx<CT>(kd, i1, o1);
      }
    }
    for (int i = 2 * half + lane; i < dim; i += 32) {   // the rest passes
      const float a = ldx<AT>(src, i);
      if (is_q) qd[i] = a;
      else stx<CT>(kd, i, a);
    }
  }
}

template <typename AT>
__global__ void __launch_bounds__(kHyThreads)
polynorm_kernel(const AT* __restrict__ z, const float* __restrict__ coef, AT* __restrict__ out, int ff, float eps) {
  extern __shared__ float pz[];
  __shared__ float red[kHyThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int c = threadIdx.x; c < ff; c += kHyThreads) {
    const float v = ldx<AT>(z, t * ff + c), v2 = v * v, v3 = v2 * v;
    pz[c] = v;
    s2 += v2;
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v3, v3, s6);
  }
  const float r1 = 1.0f / sqrtf(block_sum_hy(s2, red) / (float)ff + eps);
  const float r2 = 1.0f / sqrtf(block_sum_hy(s4, red) / (float)ff + eps);
  const float r3 = 1.0f / sqrtf(block_sum_hy(s6, red) / (float)ff + eps);
  const float c0 = coef[0] * r1, c1 = coef[1] * r2, c2 = coef[2] * r3, c3 = coef[3];
  for (int c = threadIdx.x; c < ff; c += kHyThreads) {
    const float v = pz[c], v2 = v * v;
    stx<AT>(out, t * ff + c, fmaf(c0, v, fmaf(c1, v2, fmaf(c2, v2 * v, c3))));
  }
}

template <typename AT, int N>
int hyper_step_n(float* X, int64_t sstride, int init, const void* y, const float* parts, int n_parts, const float* scale, const float* hc,
                 float mult, const float* open_in, const float* nw, const float* nb, float eps, const int32_t* rows, float* h_f32, void* h_act,
                 float* sum_out, int R, int width, const HyperConv& cv, cudaStream_t s) {
  const size_t smem = (size_t)width * 4;
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(parts) |
                         reinterpret_cast<uintptr_t>(scale) | reinterpret_cast<uintptr_t>(nw) | reinterpret_cast<uintptr_t>(nb) |
                         reinterpret_cast<uintptr_t>(h_f32) | reinterpret_cast<uintptr_t>(h_act) | reinterpret_cast<uintptr_t>(sum_out);
  if (N <= 4 && width % 4 == 0 && sstride % 4 == 0 && ptrs % 16 == 0) {
    // short steps: one trip per thread (latency); long steps: CTAs of 128 threads, so that many share an SM and one's block sums
    // hide behind the others' loads (2048 rows of width 2048, 4 streams: 45 us with 512 threads, 34 us with 128)
    int threads = std::min(1024, std::max(128, (width / 4 + 31) / 32 * 32));
    if (R >= 512) threads = 128;
    static bool done[64] = {};
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(hyper_step_kernel<AT, N, 4>, 200 * 1024, done));
    B200_CUDA(launch(hyper_step_kernel<AT, N, 4>, dim3(R), dim3(threads), smem, s, X, sstride, init, (const AT*)y, parts, n_parts, scale, hc, mult,
                     open_in, nw, nb, eps, rows, h_f32, (AT*)h_act, sum_out, width, cv));
    return B200_OK;
  }
  const int threads = std::min(1024, std::max(128, (width / 2 + 31) / 32 * 32));
  static bool done1[64] = {};
  if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(hyper_step_kernel<AT, N, 1>, 200 * 1024, done1));
  B200_CUDA(launch(hyper_step_kernel<AT, N, 1>, dim3(R), dim3(threads), smem, s, X, sstride, init, (const AT*)y, parts, n_parts, scale, hc, mult,
                   open_in, nw, nb, eps, rows, h_f32, (AT*)h_act, sum_out, width, cv));
  return B200_OK;
}

template <typename AT>
int hyper_step_t(int n, float* X, int64_t sstride, int init, const void* y, const float* parts, int n_parts, const float* scale, const float* hc,
                 float mult, const float* open_in, const float* nw, const float* nb, float eps, const int32_t* rows, float* h_f32, void* h_act,
                 float* sum_out, int R, int width, const HyperConv& cv, cudaStream_t s) {
#define HY(N) \
  case N: return hyper_step_n<AT, N>(X, sstride, init, y, parts, n_parts, scale, hc, mult, open_in, nw, nb, eps, rows, h_f32, h_act, sum_out, R, width, cv, s)
  switch (n) {
    HY(1);
    HY(2);
    HY(3);
    HY(4);
    HY(5);
    HY(6);
    HY(7);
    HY(8);
  }
#undef HY
  return B200_ERR_UNSUPPORTED;
}

}  // namespace

int hyper_step(bool f32, float* X, int64_t sstride, int n, bool init, const void* y, const float* parts, int n_parts, const float* scale,
               const float* hc, float mult, const float* open_in, const float* nw, const float* nb, float eps, const int32_t* rows,
               float* h_f32, void* h_act, float* sum_out, int R, int width, cudaStream_t s, const float* conv_w, int taps,
               const int32_t* positions, const int32_t* row_to_seq, const int32_t* seq_slots, float* tails, int64_t slot_stride) {
  if (R == 0) return B200_OK;
  B200_REQUIRE(X && n >= 1 && n <= kMaxN, B200_ERR_INVALID, "hyper_step: %d streams outside [1, %d]", n, kMaxN);
  B200_REQUIRE(!hc || ((y || (parts && n_parts > 0)) && scale), B200_ERR_INVALID, "hyper_step: a closing sublayer needs its result and its scale");
  B200_REQUIRE((size_t)width * 4 <= 200 * 1024, B200_ERR_UNSUPPORTED, "hyper_step: width %d does not fit shared memory", width);
  HyperConv cv;
  if (conv_w) {
    B200_REQUIRE(taps >= 1 && taps <= kHyMaxTaps && nw && h_act && !rows && positions && (taps == 1 || (seq_slots && tails)), B200_ERR_INVALID,
                 "hyper_step: the fused convolution needs 1 to %d taps, a norm, an output, positions and the tails", kHyMaxTaps);
    cv.w = conv_w, cv.taps = taps, cv.positions = positions, cv.row_to_seq = row_to_seq, cv.seq_slots = seq_slots, cv.tails = tails;
    cv.slot_stride = slot_stride;
  }
  return f32 ? hyper_step_t<float>(n, X, sstride, init ? 1 : 0, y, parts, n_parts, scale, hc, mult, open_in, nw, nb, eps, rows, h_f32, h_act,
                                   sum_out, R, width, cv, s)
             : hyper_step_t<__nv_bfloat16>(n, X, sstride, init ? 1 : 0, y, parts, n_parts, scale, hc, mult, open_in, nw, nb, eps, rows, h_f32,
                                           h_act, sum_out, R, width, cv, s);
}

int qkv_rotate_cache(bool f32, const void* qkv, int64_t ld, const int32_t* positions, const int32_t* slots, const float* rot, int rot_dims,
                     bool half_layout, int64_t max_pos, float* qout, void* kc, void* vc, int T, int heads, int kv_heads, int dim, int vdim,
                     int block_size, cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(rot_dims % 2 == 0 && rot_dims <= dim && rot_dims >= 0, B200_ERR_UNSUPPORTED, "qkv_rotate_cache: %d rotated dimensions in heads of %d",
               rot_dims, dim);
  if (f32)
    B200_CUDA(launch(qkv_rotate_cache_kernel<float, float>, dim3(T), dim3(256), (size_t)0, s, (const float*)qkv, ld, positions, slots, rot,
                     rot ? rot_dims : 0, half_layout ? 1 : 0, max_pos, qout, (float*)kc, (float*)vc, heads, kv_heads, dim, vdim, block_size));
  else
    B200_CUDA(launch(qkv_rotate_cache_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), (size_t)0, s, (const __nv_bfloat16*)qkv, ld,
                     positions, slots, rot, rot ? rot_dims : 0, half_layout ? 1 : 0, max_pos, qout, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, heads,
                     kv_heads, dim, vdim, block_size));
  return B200_OK;
}

int polynorm(bool f32, const void* z, const float* coef, void* out, int T, int ff, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  const size_t smem = (size_t)ff * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "polynorm: %d entries do not fit shared memory", ff);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(polynorm_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(polynorm_kernel<float>, dim3(T), dim3(kHyThreads), smem, s, (const float*)z, coef, (float*)out, ff, eps));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(polynorm_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(polynorm_kernel<__nv_bfloat16>, dim3(T), dim3(kHyThreads), smem, s, (const __nv_bfloat16*)z, coef, (__nv_bfloat16*)out, ff, eps));
  }
  return B200_OK;
}

}  // namespace b200
