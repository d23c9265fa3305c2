// Row-wise mechanisms of layer-list models in the parallel form (b200_stack_cfg.form = B200_FORM_PARALLEL), all over an
// fp32 residual stream:
//   * sequence bounds of a step (first row of every sequence) for the kernels that walk a sequence's rows in order;
//   * scaled embedding plus a hashed bigram row, with the previous token of a sequence kept in its state slot;
//   * the layer's closing sum, the depth-weighted average over all layer results so far, and the two scalar-weight RMS
//     norms of the next layer, in one pass over the row;
//   * the causal per-channel input convolution with its tail (the last taps - 1 inputs) in the state slot;
//   * gated / plain activations of a feed-forward, the final norm over the logit rows, the logit soft cap.
// Every kernel works on one row (or one sequence) per CTA with a fixed summation order, so a row's result does not depend
// on what else is in the step.
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

__device__ __forceinline__ int resolve_token(int id, int vocab, const int32_t* prev, int n_prev) {
  if (id < 0 && prev != nullptr && -id - 1 < n_prev) id = prev[-id - 1];
  return id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
}

__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < nw; ++i) r += red[i];
  return r;
}

// seq_start[s] = first row of sequence s, seq_start[S] = T.  Rows of a sequence are contiguous and sequences appear in
// index order (the scheduler builds steps so); without row_to_seq every row is a sequence of its own.
__global__ void seq_bounds_kernel(const int32_t* __restrict__ row_to_seq, int T, int S, int32_t* __restrict__ seq_start) {
  pdl_wait();
  pdl_launch_dependents();
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t <= T; t += gridDim.x * blockDim.x) {
    if (t == T) {
      seq_start[S] = T;
    } else if (row_to_seq == nullptr) {
      if (t < S) seq_start[t] = t;
    } else {
      const int s = row_to_seq[t];
      if ((t == 0 || row_to_seq[t - 1] != s) && s >= 0 && s < S) seq_start[s] = t;
    }
  }
}

__global__ void __launch_bounds__(128)
embed_bigram_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table, const __nv_bfloat16* __restrict__ bigram,
                    float* __restrict__ out, int width, int vocab, float scale, const int32_t* prev, int n_prev,
                    const int32_t* __restrict__ positions, const int32_t* __restrict__ row_to_seq,
                    const int32_t* __restrict__ seq_slots, const int32_t* __restrict__ state_prev, int64_t slot_stride_ints,
                    int buckets, int mul_prev, int mul_cur) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = resolve_token(ids[t], vocab, prev, n_prev);
  const __nv_bfloat16* src = table + (int64_t)id * width;
  const __nv_bfloat16* bsrc = nullptr;
  if (bigram != nullptr && buckets > 0) {
    int64_t row = buckets;
    if (positions[t] > 0) {
      const int s = row_to_seq ? row_to_seq[t] : t;
      int pid;
      if (t > 0 && row_to_seq != nullptr && row_to_seq[t - 1] == s) pid = resolve_token(ids[t - 1], vocab, prev, n_prev);
      else pid = state_prev ? state_prev[(int64_t)seq_slots[s] * slot_stride_ints] : 0;
      row = ((int64_t)pid * mul_prev + (int64_t)id * mul_cur) % buckets;
      if (row < 0) row += buckets;
    }
    bsrc = bigram + row * width;
  }
  float* dst = out + (int64_t)t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = __bfloat162float(src[c]) * scale;
    if (bsrc) v += __bfloat162float(bsrc[c]);
    dst[c] = v;
  }
}

// after the embedding has read the slots: the last token of every sequence of the step becomes its previous token
__global__ void prev_token_commit_kernel(const int32_t* __restrict__ ids, int vocab, const int32_t* prev, int n_prev,
                                         const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slots, int S,
                                         int32_t* __restrict__ state_prev, int64_t slot_stride_ints) {
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  const int last = seq_start[s + 1] - 1;
  if (last < seq_start[s]) return;
  state_prev[(int64_t)seq_slots[s] * slot_stride_ints] = resolve_token(ids[last], vocab, prev, n_prev);
}

// One CTA per row.  (1) with y_mix: X_new = u + (y_mix + y_ff + sum of parts + y_sh); X_new (or, without y_mix, u itself:
// the embedding output) is stored as result n_results - 1 when `results` is given; (2) with dwa:
// u = sum_j dwa[j] * results[j] over the n_results earlier results (result n_results - 1 being X_new); else u = X_new;
// (3) with g1: unit = u / sqrt(mean(u^2) + eps); h1 = unit * g1[0] (fp32 and / or activation type), h2 = unit * g2[0].
template <typename AT>
__global__ void __launch_bounds__(1024)
parallel_close_kernel(float* __restrict__ u, const AT* __restrict__ y_mix, const AT* __restrict__ y_ff, const float* __restrict__ parts,
                      int n_parts, const AT* __restrict__ y_sh, float* __restrict__ results, int64_t result_stride, int n_results,
                      const float* __restrict__ dwa, const float* __restrict__ g1, const float* __restrict__ g2,
                      float* __restrict__ h1_f32, AT* __restrict__ h1_act, AT* __restrict__ h2, int width, float eps) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = blockIdx.x, o = t * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = u[o + c];
    if (y_mix != nullptr) {
      float a = ldx<AT>(y_mix, o + c);
      if (y_ff) a += ldx<AT>(y_ff, o + c);
      for (int k = 0; k < n_parts; ++k) a += parts[(t * n_parts + k) * width + c];
      if (y_sh) a += ldx<AT>(y_sh, o + c);
      v += a;
    }
    if (results) results[(int64_t)(n_results - 1) * result_stride + o + c] = v;
    if (dwa != nullptr) {
      float a = 0.f;
      for (int j = 0; j < n_results - 1; ++j) a = fmaf(dwa[j], results[(int64_t)j * result_stride + o + c], a);
      v = fmaf(dwa[n_results - 1], v, a);
    }
    if (y_mix != nullptr || dwa != nullptr) u[o + c] = v;
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  if (g1 == nullptr) return;
  ss = block_sum_f(ss, red);
  const float inv = rsqrtf(ss / (float)width + eps);
  const float a1 = g1[0], a2 = g2 ? g2[0] : 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float n = row[c] * inv;
    if (h1_f32) h1_f32[o + c] = n * a1;
    if (h1_act) stx<AT>(h1_act, o + c, n * a1);
    if (h2) stx<AT>(h2, o + c, n * a2);
  }
}

// hc[t] = h[t] + sum_j w[:, j] * h[t - taps + 1 + j] along each sequence (zeros before position 0).  Rows whose window
// stays inside the step's portion of the sequence are one CTA each.  The first row of a portion also serves the next
// taps - 2 rows (those whose window reaches into the state slot's tail), then writes the new tail: every read of the old
// tail happens in the one CTA that overwrites it.  This form serves short steps and more than 8 taps (one row per CTA:
// rows_per_cta is 1); steps of 64 rows and more with at most 8 taps take canon_conv_run_kernel below.
constexpr int kMaxTaps = 16;
template <typename AT>
__global__ void __launch_bounds__(256)
canon_conv_kernel(const float* __restrict__ h, const float* __restrict__ w, AT* __restrict__ out, int width, int taps,
                  const int32_t* __restrict__ positions, const int32_t* __restrict__ row_to_seq, const int32_t* __restrict__ seq_start,
                  const int32_t* __restrict__ seq_slots, float* __restrict__ tails, int64_t slot_stride, int T, int rows_per_cta) {
  pdl_wait();
  pdl_launch_dependents();
  const int hist = taps - 1;
  const int t_end = min(T, (int)(blockIdx.x + 1) * rows_per_cta);
  for (int t = blockIdx.x * rows_per_cta; t < t_end; ++t) {
  const int s = row_to_seq ? row_to_seq[t] : t;
  const int start = hist ? seq_start[s] : t, n = hist ? seq_start[s + 1] - start : 1, r = t - start;
  if (r >= hist) {
    for (int c = blockIdx.y * 256 + threadIdx.x; c < width; c += gridDim.y * 256) {
      float a = h[(int64_t)t * width + c];
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) acc = fmaf(w[c * taps + j], h[(int64_t)(t - hist + j) * width + c], acc);
      stx<AT>(out, (int64_t)t * width + c, a + acc);
    }
    continue;
  }
  if (r != 0) continue;
  const int p0 = positions[t];
  float* tail = tails + (int64_t)seq_slots[s] * slot_stride;   // [hist][width]: inputs at positions p0 - hist .. p0 - 1
  for (int c = blockIdx.y * 256 + threadIdx.x; c < width; c += gridDim.y * 256) {
    float old[kMaxTaps], wv[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) {
      old[i] = (i < hist && p0 - hist + i >= 0) ? tail[(int64_t)i * width + c] : 0.f;
      wv[i] = i < taps ? w[c * taps + i] : 0.f;
    }
    // value of the input at offset o from the portion's first row (o < 0: the tail)
    auto at = [&](int o) -> float {
      if (o >= 0) return h[(int64_t)(start + o) * width + c];
      float v = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxTaps; ++i)
        if (i == hist + o) v = old[i];
      return v;
    };
    const int head_rows = n < hist ? n : hist;
    for (int rr = 0; rr < head_rows; ++rr) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxTaps; ++j)
        if (j < taps) acc = fmaf(wv[j], at(rr - hist + j), acc);
      stx<AT>(out, (int64_t)(start + rr) * width + c, at(rr) + acc);
    }
    for (int i = 0; i < hist; ++i) tail[(int64_t)i * width + c] = at(n - hist + i);
  }
  }
}

// The same for a known number of taps: a thread owns one channel over a run of consecutive rows and keeps the last TAPS - 1
// inputs in registers, so every input is fetched once instead of TAPS times.  A row at least TAPS - 1 places into its
// portion reads nothing but the rows before it in the step's buffer, whatever sequence those first rows of the run belong
// to; the first row of a portion takes the path through the tail as above.
constexpr int kConvRun = 16;
template <typename AT, int TAPS>
__global__ void __launch_bounds__(256)
canon_conv_run_kernel(const float* __restrict__ h, const float* __restrict__ w, AT* __restrict__ out, int width,
                      const int32_t* __restrict__ positions, const int32_t* __restrict__ row_to_seq, const int32_t* __restrict__ seq_start,
                      const int32_t* __restrict__ seq_slots, float* __restrict__ tails, int64_t slot_stride, int T) {
  constexpr int H = TAPS - 1;
  __shared__ int row_r[kConvRun], row_s[kConvRun];
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * kConvRun, t1 = min(T, t0 + kConvRun);
  if (threadIdx.x < t1 - t0) {
    const int t = t0 + threadIdx.x;
    const int s = row_to_seq ? row_to_seq[t] : t;
    row_s[threadIdx.x] = s;
    row_r[threadIdx.x] = H ? t - seq_start[s] : 0;
  }
  __syncthreads();
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c >= width) return;
  float wv[TAPS], win[H > 0 ? H : 1];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) wv[j] = w[c * TAPS + j];
#pragma unroll
  for (int j = 0; j < H; ++j) win[j] = t0 - H + j >= 0 ? h[(int64_t)(t0 - H + j) * width + c] : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float cur = h[(int64_t)t * width + c];
    const int r = row_r[t - t0];
    if (r >= H) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < H; ++j) acc = fmaf(wv[j], win[j], acc);
      acc = fmaf(wv[H], cur, acc);
      stx<AT>(out, (int64_t)t * width + c, cur + acc);
    } else if (r == 0) {
      const int s = row_s[t - t0], n = seq_start[s + 1] - t, p0 = positions[t];
      float* tail = tails + (int64_t)seq_slots[s] * slot_stride;   // [H][width]: inputs at positions p0 - H .. p0 - 1
      float old[H > 0 ? H : 1];
#pragma unroll
      for (int i = 0; i < H; ++i) old[i] = p0 - H + i >= 0 ? tail[(int64_t)i * width + c] : 0.f;
      auto at = [&](int o) -> float {   // the input at offset o from the portion's first row (o < 0: the tail)
        if (o >= 0) return h[(int64_t)(t + o) * width + c];
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < H; ++i)
          if (i == H + o) v = old[i];
        return v;
      };
      const int head_rows = n < H ? n : H;
      for (int rr = 0; rr < head_rows; ++rr) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) acc = fmaf(wv[j], at(rr - H + j), acc);
        stx<AT>(out, (int64_t)(t + rr) * width + c, at(rr) + acc);
      }
#pragma unroll
      for (int i = 0; i < H; ++i) tail[(int64_t)i * width + c] = at(n - H + i);
    }
#pragma unroll
    for (int j = 0; j + 1 < H; ++j) win[j] = win[j + 1];
    if (H > 0) win[H - 1] = cur;
  }
}

template <typename AT>
__global__ void __launch_bounds__(256)
rms_rows_kernel(const float* __restrict__ u, const int32_t* __restrict__ rows, const float* __restrict__ g, AT* __restrict__ out,
                int width, float eps) {
  extern __shared__ float row[];
  __shared__ float red[8];
  pdl_wait();
  pdl_launch_dependents();
  const int64_t src = (int64_t)(rows ? rows[blockIdx.x] : blockIdx.x) * width, dst = (int64_t)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += 256) {
    const float v = u[src + c];
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum_f(ss, red);
  const float a = rsqrtf(ss / (float)width + eps) * g[0];
  for (int c = threadIdx.x; c < width; c += 256) stx<AT>(out, dst + c, row[c] * a);
}

// gated rows of bf16 whose ff is a multiple of 8: eight neighbours per thread and trip (16-byte accesses), fp32 arithmetic
__global__ void __launch_bounds__(256)
ff_act_gated8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t rows, int ff, int kind, float limit) {
  pdl_wait();
  pdl_launch_dependents();
  const int chunks = ff >> 3;
  const int64_t n = rows * chunks;
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += gridDim.x * 256ll) {
    const int64_t t = i / chunks;
    const int f = (int)(i - t * chunks) << 3;
    const uint4 g = *reinterpret_cast<const uint4*>(in + t * 2 * ff + f), u = *reinterpret_cast<const uint4*>(in + t * 2 * ff + ff + f);
    uint4 o;
    o.x = pack_bf16(gate_combine(bf16lo(g.x), bf16lo(u.x), kind, limit), gate_combine(bf16hi(g.x), bf16hi(u.x), kind, limit));
    o.y = pack_bf16(gate_combine(bf16lo(g.y), bf16lo(u.y), kind, limit), gate_combine(bf16hi(g.y), bf16hi(u.y), kind, limit));
    o.z = pack_bf16(gate_combine(bf16lo(g.z), bf16lo(u.z), kind, limit), gate_combine(bf16hi(g.z), bf16hi(u.z), kind, limit));
    o.w = pack_bf16(gate_combine(bf16lo(g.w), bf16lo(u.w), kind, limit), gate_combine(bf16hi(g.w), bf16hi(u.w), kind, limit));
    *reinterpret_cast<uint4*>(out + t * ff + f) = o;
  }
}

// gated: out[t][f] = act(in[t][f]) * in[t][ff + f] over rows of 2 ff; plain: out[t][f] = act(in[t][f]) (in place allowed)
template <typename AT>
__global__ void __launch_bounds__(256)
ff_act_kernel(const AT* __restrict__ in, AT* __restrict__ out, int64_t total, int ff, int gated, int kind, float limit) {
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    if (gated) {
      const int64_t t = i / ff, f = i % ff;
      stx<AT>(out, i, gate_combine(ldx<AT>(in, t * 2 * ff + f), ldx<AT>(in, t * 2 * ff + ff + f), kind, limit));
    } else {
      stx<AT>(out, i, act_apply(ldx<AT>(in, i), kind));
    }
  }
}

// dense fp32 rows [R][vocab] -> capped fp32 rows and their bf16 rounding, both with leading dimension ld (tail zeroed)
__global__ void __launch_bounds__(256)
logit_cap_kernel(const float* __restrict__ in, float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16, int vocab, int ld,
                 float cap) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t r = blockIdx.x;
  for (int c = blockIdx.y * 256 + threadIdx.x; c < ld; c += gridDim.y * 256) {
    float v = 0.f;
    if (c < vocab) {
      v = in[r * vocab + c];
      if (cap > 0.f) v = cap * tanhf(v / cap);
    }
    out_f32[r * ld + c] = v;
    out_bf16[r * ld + c] = __float2bfloat16_rn(v);
  }
}

}  // namespace

int seq_bounds(const int32_t* row_to_seq, int T, int S, int32_t* seq_start, cudaStream_t s) {
  B200_CUDA(launch(seq_bounds_kernel, dim3((T + 256) / 256), dim3(256), (size_t)0, s, row_to_seq, T, S, seq_start));
  return B200_OK;
}

int embed_bigram(const int32_t* ids, const __nv_bfloat16* table, const __nv_bfloat16* bigram, float* out, int T, int width, int vocab,
                 float scale, const int32_t* prev, int n_prev, const int32_t* positions, const int32_t* row_to_seq,
                 const int32_t* seq_slots, const int32_t* state_prev, int64_t slot_stride_ints, int buckets, int mul_prev, int mul_cur,
                 cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(!bigram || buckets <= 0 || (positions && (!state_prev || seq_slots)), B200_ERR_INVALID, "embed_bigram: positions / slots missing");
  B200_CUDA(launch(embed_bigram_kernel, dim3(T), dim3(128), (size_t)0, s, ids, table, bigram, out, width, vocab, scale, prev, n_prev,
                   positions, row_to_seq, seq_slots, state_prev, slot_stride_ints, buckets, mul_prev, mul_cur));
  return B200_OK;
}

int prev_token_commit(const int32_t* ids, int vocab, const int32_t* prev, int n_prev, const int32_t* seq_start, const int32_t* seq_slots,
                      int S, int32_t* state_prev, int64_t slot_stride_ints, cudaStream_t s) {
  if (S == 0) return B200_OK;
  B200_CUDA(launch(prev_token_commit_kernel, dim3((S + 127) / 128), dim3(128), (size_t)0, s, ids, vocab, prev, n_prev, seq_start,
                   seq_slots, S, state_prev, slot_stride_ints));
  return B200_OK;
}

int parallel_close(bool f32, float* u, const void* y_mix, const void* y_ff, const float* parts, int n_parts, const void* y_sh,
                   float* results, int64_t result_stride, int n_results, const float* dwa, const float* g1, const float* g2,
                   float* h1_f32, void* h1_act, void* h2, int T, int width, float eps, cudaStream_t s) {
  if (T == 0) return B200_OK;
  const size_t smem = (size_t)width * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "parallel_close: width %d does not fit shared memory", width);
  static bool done[2][64] = {};
  // steps of few rows: few elements per thread, so that a row's loads are in flight together; long steps fill the SMs anyway
  const int threads = T >= 512 ? 256 : (width >= 2048 ? 1024 : (width >= 1024 ? 512 : 256));
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(parallel_close_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(parallel_close_kernel<float>, dim3(T), dim3(threads), smem, s, u, (const float*)y_mix, (const float*)y_ff, parts,
                     n_parts, (const float*)y_sh, results, result_stride, n_results, dwa, g1, g2, h1_f32, (float*)h1_act, (float*)h2,
                     width, eps));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(parallel_close_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(parallel_close_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, s, u, (const __nv_bfloat16*)y_mix,
                     (const __nv_bfloat16*)y_ff, parts, n_parts, (const __nv_bfloat16*)y_sh, results, result_stride, n_results, dwa,
                     g1, g2, h1_f32, (__nv_bfloat16*)h1_act, (__nv_bfloat16*)h2, width, eps));
  }
  return B200_OK;
}

int canon_conv(bool f32, const float* h, const float* w, void* out, int T, int width, int taps, const int32_t* positions,
               const int32_t* row_to_seq, const int32_t* seq_start, const int32_t* seq_slots, float* tails, int64_t slot_stride,
               cudaStream_t s) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(taps >= 1 && taps <= kMaxTaps, B200_ERR_UNSUPPORTED, "canon_conv: %d taps outside [1, %d]", taps, kMaxTaps);
  B200_REQUIRE(taps == 1 || (positions && seq_start && seq_slots && tails), B200_ERR_INVALID, "canon_conv: null argument");
  if (taps <= 8 && T >= 64) {   // long steps: runs of rows with the window in registers
    const dim3 rgrid((T + kConvRun - 1) / kConvRun, (width + 255) / 256);
#define CONV_RUN(N)                                                                                                                         \
  case N:                                                                                                                                   \
    if (f32)                                                                                                                                \
      B200_CUDA(launch(canon_conv_run_kernel<float, N>, rgrid, dim3(256), (size_t)0, s, h, w, (float*)out, width, positions, row_to_seq,    \
                       seq_start, seq_slots, tails, slot_stride, T));                                                                       \
    else                                                                                                                                    \
      B200_CUDA(launch(canon_conv_run_kernel<__nv_bfloat16, N>, rgrid, dim3(256), (size_t)0, s, h, w, (__nv_bfloat16*)out, width, positions, \
                       row_to_seq, seq_start, seq_slots, tails, slot_stride, T));                                                           \
    return B200_OK;
    switch (taps) {
      CONV_RUN(1)
      CONV_RUN(2)
      CONV_RUN(3)
      CONV_RUN(4)
      CONV_RUN(5)
      CONV_RUN(6)
      CONV_RUN(7)
      CONV_RUN(8)
    }
#undef CONV_RUN
  }
  const int rpc = 1;
  const dim3 grid((T + rpc - 1) / rpc, (width + 255) / 256);
  if (f32)
    B200_CUDA(launch(canon_conv_kernel<float>, grid, dim3(256), (size_t)0, s, h, w, (float*)out, width, taps, positions, row_to_seq,
                     seq_start, seq_slots, tails, slot_stride, T, rpc));
  else
    B200_CUDA(launch(canon_conv_kernel<__nv_bfloat16>, grid, dim3(256), (size_t)0, s, h, w, (__nv_bfloat16*)out, width, taps,
                     positions, row_to_seq, seq_start, seq_slots, tails, slot_stride, T, rpc));
  return B200_OK;
}

int rms_rows(bool f32, const float* u, const int32_t* rows, const float* g, void* out, int R, int width, float eps, cudaStream_t s) {
  if (R == 0) return B200_OK;
  const size_t smem = (size_t)width * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "rms_rows: width %d does not fit shared memory", width);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(rms_rows_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(rms_rows_kernel<float>, dim3(R), dim3(256), smem, s, u, rows, g, (float*)out, width, eps));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(rms_rows_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(rms_rows_kernel<__nv_bfloat16>, dim3(R), dim3(256), smem, s, u, rows, g, (__nv_bfloat16*)out, width, eps));
  }
  return B200_OK;
}

int ff_act(bool f32, const void* in, void* out, int T, int ff, bool gated, int kind, cudaStream_t s, float limit) {
  const int64_t total = (int64_t)T * ff;
  if (total == 0) return B200_OK;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, 148 * 16);
  if (!f32 && gated && ff % 8 == 0 && (reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
    const int g8 = (int)std::min<int64_t>((total / 8 + 255) / 256, 148 * 16);
    B200_CUDA(launch(ff_act_gated8_kernel, dim3(g8), dim3(256), (size_t)0, s, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, (int64_t)T, ff, kind, limit));
    return B200_OK;
  }
  if (f32)
    B200_CUDA(launch(ff_act_kernel<float>, dim3(grid), dim3(256), (size_t)0, s, (const float*)in, (float*)out, total, ff, gated ? 1 : 0, kind, limit));
  else
    B200_CUDA(launch(ff_act_kernel<__nv_bfloat16>, dim3(grid), dim3(256), (size_t)0, s, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, total,
                     ff, gated ? 1 : 0, kind, limit));
  return B200_OK;
}

int logit_cap(const float* in, float* out_f32, __nv_bfloat16* out_bf16, int R, int vocab, int ld, float cap, cudaStream_t s) {
  if (R == 0) return B200_OK;
  B200_CUDA(launch(logit_cap_kernel, dim3(R, std::max(1, std::min(ld / 1024, 64))), dim3(256), (size_t)0, s, in, out_f32, out_bf16, vocab, ld, cap));
  return B200_OK;
}

}  // namespace b200
