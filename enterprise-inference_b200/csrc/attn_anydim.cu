// Paged causal softmax attention (optionally over a sliding window of the last `window` keys) for heads of any size
// (query/key size `dim`, value size `vdim`, dim != vdim allowed),
// any block size, a caller-given score scale, fp32 queries and a bf16 or fp32 cache.  The tcgen05 kernels of attn_tc.cu /
// attn_prefill.cu are built for 128-wide heads; this file serves every other head shape on CUDA cores with fp32 scores,
// fp32 softmax weights and fp32 accumulation.
//
// Optional output rotation: when the cached values were rotated by their own position (pair 2m, 2m+1 of a value turned by
// j * f_m), the weighted sum of a query at position i is turned back by -i * f_m before it is written, which leaves each
// value rotated by the DISTANCE j - i.  The table is the one the cache writer used: [pos][2][vdim/2] fp32.
//
// Two kernels over the same cache layout ([block][kv head][block_size][dim | vdim]):
//  * rows kernel (decode rows, short steps): one CTA per (row, query head); a tile is 128 keys, one key per thread for the
//    scores, one value dimension per thread for the weighted sum; online softmax across tiles.
//  * tile kernel (prefill chunks): one CTA per (run of up to 16 consecutive rows of one sequence, kv head): K/V tiles are
//    staged in shared memory once and shared by the rows and by the query heads of the group.
// Both produce the same sums up to fp32 rounding: the per-row arithmetic is the same online softmax.
#include <algorithm>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kAdThreads = 128;
constexpr int kAdMaxVPer = 4;   // value dims per thread: vdim <= 512

template <typename CT> __device__ __forceinline__ float cache_load(const CT* p, int64_t i);
template <> __device__ __forceinline__ float cache_load<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float cache_load<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename AT> __device__ __forceinline__ void out_store(AT* p, int64_t i, float v);
template <> __device__ __forceinline__ void out_store<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void out_store<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_max128(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
}
__device__ __forceinline__ float block_sum128(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

template <typename CT, typename AT>
__global__ void __launch_bounds__(kAdThreads)
paged_attn_rows_kernel(const float* __restrict__ q, const CT* __restrict__ kc, const CT* __restrict__ vc,
                       const int32_t* __restrict__ block_table, int bt_stride, const int32_t* __restrict__ row_to_seq,
                       const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ positions,
                       const float* __restrict__ vrot, int64_t max_pos, AT* __restrict__ out, int heads, int kv_heads,
                       int dim, int vdim, int block_size, float scale, int kst, int vst, const float* __restrict__ sink, int window) {
  extern __shared__ float sm[];
  float* qs = sm;                 // [dim]
  float* ps = qs + dim;           // [128] weights of the tile
  float* os = ps + kAdThreads;    // [vdim] the finished row before the output rotation
  __shared__ float red[4];
  __shared__ int blk_of[kAdThreads];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (heads / kv_heads);
  const int ctx = ctx_lens[t];
  const int32_t* bt = block_table + (int64_t)(row_to_seq ? row_to_seq[t] : t) * bt_stride;
  for (int d = tid; d < dim; d += kAdThreads) qs[d] = q[((int64_t)t * heads + h) * dim + d];
  float m = -INFINITY, l = 0.f;
  float acc[kAdMaxVPer];
#pragma unroll
  for (int i = 0; i < kAdMaxVPer; ++i) acc[i] = 0.f;
  __syncthreads();
  const int lo = window > 0 ? max(ctx - window, 0) : 0;   // the first key the row sees; the tile that holds it is the first walked
  for (int base = lo - lo % kAdThreads; base < ctx; base += kAdThreads) {
    const int j = base + tid;
    float sc = -INFINITY;
    int blk = 0;
    if (j < ctx && j >= lo) {
      blk = bt[j / block_size];
      const CT* kp = kc + (((int64_t)blk * kv_heads + g) * block_size + j % block_size) * kst;
      float a = 0.f;
      for (int d = 0; d < dim; ++d) a = fmaf(qs[d], cache_load<CT>(kp, d), a);
      sc = a * scale;
    }
    const float tm = block_max128(sc, red);
    const float mn = fmaxf(m, tm);
    const float p = (j < ctx && j >= lo) ? expf(sc - mn) : 0.f;
    const float corr = expf(m - mn);      // first tile: exp(-inf) = 0
    const float ts = block_sum128(p, red);
    l = l * corr + ts;
    m = mn;
    ps[tid] = p;
    blk_of[tid] = blk;
    __syncthreads();
    const int n = min(kAdThreads, ctx - base);
#pragma unroll
    for (int i = 0; i < kAdMaxVPer; ++i) {
      const int d = tid + i * kAdThreads;
      if (d < vdim) {
        float a = acc[i] * corr;
        for (int jj = max(lo - base, 0); jj < n; ++jj) {
          const CT* vp = vc + (((int64_t)blk_of[jj] * kv_heads + g) * block_size + (base + jj) % block_size) * vst;
          a = fmaf(ps[jj], cache_load<CT>(vp, d), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();
  }
  if (sink != nullptr) {   // one more term of the denominator, without key or value
    const float sk = sink[h], mn = fmaxf(m, sk), corr = expf(m - mn);
    l = l * corr + expf(sk - mn);
#pragma unroll
    for (int i = 0; i < kAdMaxVPer; ++i) acc[i] *= corr;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < kAdMaxVPer; ++i) {
    const int d = tid + i * kAdThreads;
    if (d < vdim) os[d] = acc[i] * inv;
  }
  __syncthreads();
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
  const int vhalf = vdim >> 1;
  const float* cs = vrot ? vrot + (int64_t)pos * 2 * vhalf : nullptr;
  for (int d = tid; d < vdim; d += kAdThreads) {
    float v = os[d];
    if (cs && d < 2 * vhalf) {
      const float c = cs[d >> 1], s = cs[vhalf + (d >> 1)];
      const float o = os[d ^ 1];
      v = (d & 1) ? fmaf(v, c, -o * s) : fmaf(v, c, o * s);   // rotation by -angle
    }
    out_store<AT>(out, ((int64_t)t * heads + h) * vdim + d, v);
  }
}

// ---- prefill chunks: runs of consecutive rows of one sequence share the K/V tiles ------------------------------------------
// Work item = (run of up to kRunRows rows of one sequence whose context lengths rise by one, kv head).  The item list is
// built on the device once per step.  Warp w serves query (row r, head hh) pairs round-robin; a tile is 32 keys: lane =
// key for the scores, lanes stride the value dimensions for the weighted sum.
constexpr int kRunRows = 16;
constexpr int kTileKeys = 32;
constexpr int kTcThreads = 256;

// One CTA of 1024 threads.  Row t opens a segment when it is the step's first row, belongs to another sequence than row
// t - 1, or does not continue its context length by one; inside a segment a run starts every kRunRows rows.  Per chunk of
// 1024 rows: an inclusive max-scan carries every row's segment start, a prefix sum of the run starts gives each run its place.
__global__ void __launch_bounds__(1024)
attn_runs_plan_kernel(const int32_t* __restrict__ row_to_seq, const int32_t* __restrict__ ctx_lens, int T, int32_t* __restrict__ runs,
                      int32_t* __restrict__ n_runs) {
  __shared__ int wseg[32], wcnt[32];
  __shared__ int carry_seg, carry_cnt;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    carry_seg = 0;
    carry_cnt = 0;
  }
  __syncthreads();
  for (int c0 = 0; c0 < T; c0 += 1024) {
    const int t = c0 + tid;
    const bool live = t < T;
    const bool brk = live && (t == 0 || row_to_seq == nullptr || row_to_seq[t] != row_to_seq[t - 1] || ctx_lens[t] != ctx_lens[t - 1] + 1);
    int seg = brk ? t : -1;                       // latest segment start at or before t (within the warp, then the chunk)
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, seg, o);
      if (lane >= o) seg = max(seg, v);
    }
    if (lane == 31) wseg[warp] = seg;
    __syncthreads();
    int before = carry_seg;
    for (int w = 0; w < warp; ++w) before = max(before, wseg[w]);
    seg = max(seg, before);
    const bool starts = live && (t - seg) % kRunRows == 0;
    int cnt = starts ? 1 : 0;                     // inclusive prefix count of run starts
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, cnt, o);
      if (lane >= o) cnt += v;
    }
    if (lane == 31) wcnt[warp] = cnt;
    __syncthreads();
    int base = carry_cnt;
    for (int w = 0; w < warp; ++w) base += wcnt[w];
    if (starts) runs[2 * (base + cnt - 1)] = t;
    __syncthreads();
    if (tid == 1023) {
      carry_seg = seg;
      carry_cnt = base + cnt;
    }
    __syncthreads();
  }
  // lengths: a run ends where the next one starts
  const int n = carry_cnt;
  for (int i = tid; i < n; i += 1024) runs[2 * i + 1] = (i + 1 < n ? runs[2 * (i + 1)] : T) - runs[2 * i];
  if (tid == 0) *n_runs = n;
}

template <typename CT, typename AT>
__global__ void __launch_bounds__(kTcThreads)
paged_attn_runs_kernel(const float* __restrict__ q, const CT* __restrict__ kc, const CT* __restrict__ vc,
                       const int32_t* __restrict__ block_table, int bt_stride, const int32_t* __restrict__ row_to_seq,
                       const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ positions,
                       const float* __restrict__ vrot, int64_t max_pos, AT* __restrict__ out,
                       const int32_t* __restrict__ runs, const int32_t* __restrict__ n_runs, int heads, int kv_heads, int dim,
                       int vdim, int block_size, float scale, int kcs, int vcs, const float* __restrict__ sink, int window) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int item = blockIdx.x, g = blockIdx.y;
  if (item >= *n_runs) return;
  const int t0 = runs[2 * item], nr = runs[2 * item + 1];
  const int G = heads / kv_heads;          // query heads per kv head
  const int nq = nr * G;                   // queries of this item
  const int kst = dim + 1, vst = vdim;     // K rows padded: lane = key reads stride kst (conflict-free for odd strides)
  float* Ks = sm;                               // [32][dim+1]
  float* Vs = Ks + kTileKeys * kst;             // [32][vdim]
  float* Qs = Vs + kTileKeys * vst;             // [nq][dim]
  float* Os = Qs + kRunRows * G * dim;          // [nq][vdim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kTcThreads / 32;
  const int32_t* bt = block_table + (int64_t)(row_to_seq ? row_to_seq[t0] : t0) * bt_stride;
  const int ctx_max = ctx_lens[t0 + nr - 1];
  for (int i = threadIdx.x; i < nq * dim; i += kTcThreads) {
    const int qi = i / dim, d = i % dim;
    const int r = qi / G, hh = qi % G;
    Qs[i] = q[((int64_t)(t0 + r) * heads + g * G + hh) * dim + d];
  }
  for (int i = threadIdx.x; i < nq * vdim; i += kTcThreads) Os[i] = 0.f;
  // per-warp running statistics of its queries live in registers: query qi = warp + k * nw
  constexpr int kMaxQPerWarp = 16;   // nq <= 16 * G; the launcher bounds G so that nq <= nw * kMaxQPerWarp
  float m[kMaxQPerWarp], l[kMaxQPerWarp];
#pragma unroll
  for (int k = 0; k < kMaxQPerWarp; ++k) {
    m[k] = -INFINITY;
    l[k] = 0.f;
  }
  __syncthreads();
  // with a window the run's first row sees the oldest key of all: the walk starts at the tile that holds it
  const int lo_run = window > 0 ? max(ctx_lens[t0] - window, 0) : 0;
  for (int base = lo_run - lo_run % kTileKeys; base < ctx_max; base += kTileKeys) {
    const int n = min(kTileKeys, ctx_max - base);
    for (int i = threadIdx.x; i < n * dim; i += kTcThreads) {
      const int jj = i / dim, d = i % dim, j = base + jj;
      Ks[jj * kst + d] = cache_load<CT>(kc, (((int64_t)bt[j / block_size] * kv_heads + g) * block_size + j % block_size) * kcs + d);
    }
    for (int i = threadIdx.x; i < n * vdim; i += kTcThreads) {
      const int jj = i / vdim, d = i % vdim, j = base + jj;
      Vs[jj * vst + d] = cache_load<CT>(vc, (((int64_t)bt[j / block_size] * kv_heads + g) * block_size + j % block_size) * vcs + d);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kMaxQPerWarp; ++k) {
      const int qi = warp + k * nw;
      if (qi < nq) {
        const int r = qi / G;
        const int ctx = ctx_lens[t0 + r];
        const int lo = window > 0 ? max(ctx - window, 0) : 0;
        if (base < ctx && base + n > lo) {
          const int j = base + lane;
          float sc = -INFINITY;
          if (j < ctx && j >= lo) {
            const float* qp = Qs + qi * dim;
            const float* kp = Ks + lane * kst;
            float a = 0.f;
            for (int d = 0; d < dim; ++d) a = fmaf(qp[d], kp[d], a);
            sc = a * scale;
          }
          const float mn = fmaxf(m[k], warp_max(sc));
          const float p = (j < ctx && j >= lo) ? expf(sc - mn) : 0.f;
          const float corr = expf(m[k] - mn);
          l[k] = l[k] * corr + warp_sum(p);
          m[k] = mn;
          const int nn = min(n, ctx - base);
          float* op = Os + qi * vdim;
          for (int d0 = 0; d0 < vdim; d0 += 32) {   // the whole warp walks every slice: the shuffles need all lanes
            const int d = d0 + lane;
            const bool live = d < vdim;
            float a = live ? op[d] * corr : 0.f;
            for (int jj = 0; jj < nn; ++jj) {
              const float pj = __shfl_sync(0xffffffffu, p, jj);
              if (live) a = fmaf(pj, Vs[jj * vst + d], a);
            }
            if (live) op[d] = a;
          }
        }
      }
    }
    __syncthreads();
  }
  const int vhalf = vdim >> 1;
#pragma unroll
  for (int k = 0; k < kMaxQPerWarp; ++k) {
    const int qi = warp + k * nw;
    if (qi < nq) {
      const int r = qi / G, hh = qi % G, t = t0 + r;
      float lk = l[k], osc = 1.f;
      if (sink != nullptr) {
        const float sk = sink[g * G + hh], mn = fmaxf(m[k], sk);
        osc = expf(m[k] - mn);
        lk = lk * osc + expf(sk - mn);
      }
      const float inv = lk > 0.f ? osc / lk : 0.f;
      int pos = positions[t];
      pos = pos < 0 ? 0 : (pos >= max_pos ? (int)max_pos - 1 : pos);
      const float* cs = vrot ? vrot + (int64_t)pos * 2 * vhalf : nullptr;
      const float* op = Os + qi * vdim;
      for (int d = lane; d < vdim; d += 32) {
        float v = op[d] * inv;
        if (cs && d < 2 * vhalf) {
          const float c = cs[d >> 1], s = cs[vhalf + (d >> 1)];
          const float o = op[d ^ 1] * inv;
          v = (d & 1) ? fmaf(v, c, -o * s) : fmaf(v, c, o * s);
        }
        out_store<AT>(out, ((int64_t)t * heads + g * G + hh) * vdim + d, v);
      }
    }
  }
}

}  // namespace

int64_t paged_attn_anydim_workspace_bytes(int T) { return ((int64_t)2 * T + 8) * 4; }

// The run list of a step in ws (n_runs at ws[0], (first row, rows) pairs from ws[8]): what plan = 1 builds, as a call of its
// own for the kernels that share it.
int paged_attn_runs_plan(const int32_t* row_to_seq, const int32_t* ctx_lens, int T, void* ws, cudaStream_t s) {
  int32_t* runs = static_cast<int32_t*>(ws) + 8;
  int32_t* n_runs = static_cast<int32_t*>(ws);
  B200_CUDA(launch(attn_runs_plan_kernel, dim3(1), dim3(1024), (size_t)0, s, row_to_seq, ctx_lens, T, runs, n_runs));
  return B200_OK;
}

template <typename CT, typename AT>
static int paged_attn_anydim_t(const float* q, const void* kc, const void* vc, const int32_t* block_table, int bt_stride,
                               const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions, const float* vrot,
                               int64_t max_pos, void* out, int T, int heads, int kv_heads, int dim, int vdim, int block_size,
                               float scale, int plan, void* ws, cudaStream_t s, int kst, int vst, const float* sink, int window) {
  const int G = heads / kv_heads;
  const size_t smem_runs = ((size_t)kTileKeys * (dim + 1 + vdim) + (size_t)kRunRows * G * (dim + vdim)) * 4;
  if (plan != 0 && ws != nullptr && kRunRows * G <= 16 * (kTcThreads / 32) && smem_runs <= 200 * 1024) {
    int32_t* runs = static_cast<int32_t*>(ws) + 8;
    int32_t* n_runs = static_cast<int32_t*>(ws);
    if (plan == 1) B200_CUDA(launch(attn_runs_plan_kernel, dim3(1), dim3(1024), 0, s, row_to_seq, ctx_lens, T, runs, n_runs));
    static bool done[64] = {};
    if (smem_runs > 48 * 1024) B200_CUDA(ensure_dynamic_smem(paged_attn_runs_kernel<CT, AT>, 200 * 1024, done));
    B200_CUDA(launch(paged_attn_runs_kernel<CT, AT>, dim3(T, kv_heads), dim3(kTcThreads), smem_runs, s, q, (const CT*)kc,
                     (const CT*)vc, block_table, bt_stride, row_to_seq, ctx_lens, positions, vrot, max_pos, (AT*)out,
                     (const int32_t*)runs, (const int32_t*)n_runs, heads, kv_heads, dim, vdim, block_size, scale, kst, vst, sink, window));
    return B200_OK;
  }
  const size_t smem = ((size_t)dim + kAdThreads + vdim) * 4;
  B200_CUDA(launch(paged_attn_rows_kernel<CT, AT>, dim3(T, heads), dim3(kAdThreads), smem, s, q, (const CT*)kc, (const CT*)vc,
                   block_table, bt_stride, row_to_seq, ctx_lens, positions, vrot, max_pos, (AT*)out, heads, kv_heads, dim, vdim,
                   block_size, scale, kst, vst, sink, window));
  return B200_OK;
}

// plan: 0 = one CTA per (row, head); 1 = build the run list of the step in ws, then the shared-tile kernel; 2 = the
// shared-tile kernel over the run list already in ws (later layers of the same step).
int paged_attn_anydim(bool f32, const float* q, const void* kc, const void* vc, const int32_t* block_table, int bt_stride,
                      const int32_t* row_to_seq, const int32_t* ctx_lens, const int32_t* positions, const float* vrot,
                      int64_t max_pos, void* out, int T, int heads, int kv_heads, int dim, int vdim, int block_size, float scale,
                      int plan, void* ws, cudaStream_t s, int kstride, int vstride, const float* sink, int window) {
  if (T == 0) return B200_OK;
  const int kst = kstride > 0 ? kstride : dim, vst = vstride > 0 ? vstride : vdim;
  B200_REQUIRE(kst >= dim && vst >= vdim, B200_ERR_INVALID, "attention: cache rows of %d / %d elements for heads of %d / %d", kst, vst, dim, vdim);
  B200_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0, B200_ERR_INVALID, "attention: %d heads over %d kv heads", heads, kv_heads);
  B200_REQUIRE(vdim <= kAdThreads * kAdMaxVPer && dim <= 8192, B200_ERR_UNSUPPORTED, "attention: head sizes %d / %d too large", dim, vdim);
  return f32 ? paged_attn_anydim_t<float, float>(q, kc, vc, block_table, bt_stride, row_to_seq, ctx_lens, positions, vrot, max_pos,
                                                 out, T, heads, kv_heads, dim, vdim, block_size, scale, plan, ws, s, kst, vst, sink, window)
             : paged_attn_anydim_t<__nv_bfloat16, __nv_bfloat16>(q, kc, vc, block_table, bt_stride, row_to_seq, ctx_lens,
                                                                 positions, vrot, max_pos, out, T, heads, kv_heads, dim, vdim,
                                                                 block_size, scale, plan, ws, s, kst, vst, sink, window);
}

}  // namespace b200
