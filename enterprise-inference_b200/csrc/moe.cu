// Mixture-of-experts feed-forward: a softmax router with a selection bias and group-limited top-k choice, and the chosen
// experts' gated feed-forward (down(silu(gate x) * (up x))).
//
// Router (fp32 throughout; fp32 rows: one CTA per token computes logits and choice; bf16 rows: the logits are a tcgen05
// linear with unrounded fp32 output, then one warp per token chooses): z = W_r x, s = softmax(z) over all experts; the CHOICE uses s + bias, the
// mixing weights use s itself, not renormalised.  With groups: the experts form `groups` equal runs of neighbours, a
// group's score is its largest choice score, only the `keep` best groups stay eligible (the others count as -inf), then
// the `top` largest eligible choice scores win.  Ties go to the lowest index.
//
// Experts: three forms over the same weights ([expert][2 ff][width]: gate rows then up rows; [expert][width][ff]):
//  * token form (decode-sized steps): one CTA per (token, chosen slot) streams that expert's three matrices once;
//  * grouped form (prefill-sized steps): tokens are bucketed by expert on the device (deterministic order: by token, then
//    slot), and one CTA per (expert, tile of 16 of its tokens) streams the expert's weights once for the whole tile.
//  * tensor-core form (bf16 serving mode, width and ff multiples of 8; every step size): the (token, slot) pairs are
//    grouped by expert into whole token tiles, the token rows gathered, and two launches of the grouped tcgen05 linear
//    (gemm_tc.cu) run gate|up and down for all experts at once; the second one scatters the weighted fp32 rows.
// Score mode 2 (chosen-softmax router): the bias is part of the logits, the `top` largest logits win and the mixing weights are
// the softmax over those `top` logits alone.  Experts may also be gated by B200_ACT_SWIGLU_CLAMP (gate_combine, common.cuh).
// All write one fp32 partial row per (token, slot), already multiplied by the mixing weight; the consumer (the norm that
// follows the feed-forward) adds the slots in slot order, so the result does not depend on which form ran or on what else
// was in the step beyond fp32 rounding.
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"

namespace b200 {
namespace {

template <typename AT> __device__ __forceinline__ float ld_act(const AT* p, int64_t i);
template <> __device__ __forceinline__ float ld_act<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_act<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

constexpr int kRouteThreads = 128;

// (value, index) arg-max over a warp, ties to the lowest index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

// One warp: softmax over the logits in sc[experts] (replaced by the scores), choice scores in ch, the group limit, top-k.
__device__ __forceinline__ void route_select(float* sc, float* ch, float* gs, const float* __restrict__ bias, int lane, int t,
                                             int experts, int top, int groups, int keep, int32_t* __restrict__ out_ids,
                                             float* __restrict__ out_w, int sigmoid_scores) {
  if (sigmoid_scores == 2) {   // the logits themselves compete; the weights follow the choice
    for (int e = lane; e < experts; e += 32) {
      const float z = sc[e] + (bias ? bias[e] : 0.f);
      sc[e] = z;
      ch[e] = z;
    }
  } else if (sigmoid_scores) {   // every expert scored on its own
    for (int e = lane; e < experts; e += 32) {
      const float s = 1.0f / (1.0f + expf(-sc[e]));
      sc[e] = s;
      ch[e] = s + (bias ? bias[e] : 0.f);
    }
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, sc[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) sum += expf(sc[e] - mx);
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < experts; e += 32) {
      const float s = expf(sc[e] - mx) * inv;
      sc[e] = s;
      ch[e] = s + (bias ? bias[e] : 0.f);
    }
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float b = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, ch[e]);
      gs[g] = b;
    }
    __syncwarp();
    // drop the groups - keep worst groups: pick the keep best, mark them, then mask the rest
    for (int k = 0; k < keep; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (bi == 0x7fffffff || v > bv)) {   // +inf marks "already kept"
          bv = v;
          bi = g;
        }
      }
      if (bi == 0x7fffffff) bv = -INFINITY;
      // lanes without a candidate carry (-inf, big index) and lose every tie
      warp_argmax(bv, bi);
      __syncwarp();
      if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gs[e / per] != INFINITY) ch[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = ch[e];
      if (!isnan(v) && (bi == 0x7fffffff || v > bv)) {   // NaN marks "already chosen"
        bv = v;
        bi = e;
      }
    }
    if (bi == 0x7fffffff) bv = -INFINITY;
    warp_argmax(bv, bi);
    __syncwarp();
    if (lane == 0) {
      const int e = bi == 0x7fffffff ? 0 : bi;
      out_ids[(int64_t)t * top + k] = e;
      out_w[(int64_t)t * top + k] = bi == 0x7fffffff ? 0.f : sc[e];
      if (bi != 0x7fffffff) ch[e] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  if (sigmoid_scores == 2 && lane == 0) {   // softmax over the chosen logits (the first one is the largest)
    float* w = out_w + (int64_t)t * top;
    const float mx = w[0];
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      w[k] = expf(w[k] - mx);
      sum += w[k];
    }
    const float inv = 1.0f / sum;
    for (int k = 0; k < top; ++k) w[k] *= inv;
  }
}

// Selection over logits that a linear already produced ([T][experts] fp32): one warp per token.
constexpr int kSelWarps = 4;
__global__ void __launch_bounds__(kSelWarps * 32)
moe_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int experts, int top, int groups,
                  int keep, int32_t* __restrict__ out_ids, float* __restrict__ out_w, int sigmoid_scores) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kSelWarps + warp;
  if (t >= T) return;
  float* sc = sm + (size_t)warp * (2 * experts + groups);
  float* ch = sc + experts;
  float* gs = ch + experts;
  for (int e = lane; e < experts; e += 32) sc[e] = logits[(int64_t)t * experts + e];
  __syncwarp();
  route_select(sc, ch, gs, bias, lane, t, experts, top, groups, keep, out_ids, out_w, sigmoid_scores);
}

template <typename AT>
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const AT* __restrict__ x, const __nv_bfloat16* __restrict__ wr, const float* __restrict__ bias, int width,
                 int experts, int top, int groups, int keep, int32_t* __restrict__ out_ids, float* __restrict__ out_w,
                 int sigmoid_scores) {
  extern __shared__ float sm[];
  float* xs = sm;                 // [width]
  float* sc = xs + width;         // [experts] scores
  float* ch = sc + experts;       // [experts] choice scores (eligible) / -inf
  float* gs = ch + experts;       // [groups]
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kRouteThreads / 32;
  for (int c = threadIdx.x; c < width; c += kRouteThreads) xs[c] = ld_act<AT>(x, (int64_t)t * width + c);
  __syncthreads();
  for (int e = warp; e < experts; e += nw) {
    const __nv_bfloat16* w = wr + (int64_t)e * width;
    float a = 0.f;
    for (int c = lane; c < width; c += 32) a = fmaf(__bfloat162float(w[c]), xs[c], a);
    a = warp_sum(a);
    if (lane == 0) sc[e] = a;
  }
  __syncthreads();
  if (warp != 0) return;
  route_select(sc, ch, gs, bias, lane, t, experts, top, groups, keep, out_ids, out_w, sigmoid_scores);
}

// ---- token form ---------------------------------------------------------------------------------------------------------
constexpr int kExpThreads = 256;

template <typename AT>
__global__ void __launch_bounds__(kExpThreads)
moe_expert_rows_kernel(const AT* __restrict__ x, const __nv_bfloat16* __restrict__ w_gu, const __nv_bfloat16* __restrict__ w_down,
                       const int32_t* __restrict__ ids, const float* __restrict__ wts, int width, int ff, int top,
                       float* __restrict__ parts, ExpertForm form) {
  extern __shared__ float sm[];
  float* xs = sm;            // [width]
  float* as = xs + width;    // [ff]
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, slot = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kExpThreads / 32;
  const int e = ids[(int64_t)t * top + slot];
  const float wt = wts[(int64_t)t * top + slot];
  const float w_in = form.weight_input ? wt : 1.0f, w_out = form.weight_input ? 1.0f : wt;
  for (int c = threadIdx.x; c < width; c += kExpThreads) xs[c] = ld_act<AT>(x, (int64_t)t * width + c) * w_in;
  __syncthreads();
  const __nv_bfloat16* wg = w_gu + (int64_t)e * (form.gated ? 2 : 1) * ff * width;
  const __nv_bfloat16* wu = wg + (int64_t)ff * width;
  for (int f = warp; f < ff; f += nw) {
    const __nv_bfloat16* g = wg + (int64_t)f * width;
    const __nv_bfloat16* u = wu + (int64_t)f * width;
    float a = 0.f, b = 0.f;
    if (form.gated) {
      for (int c = lane; c < width; c += 32) {
        const float xv = xs[c];
        a = fmaf(__bfloat162float(g[c]), xv, a);
        b = fmaf(__bfloat162float(u[c]), xv, b);
      }
      b = warp_sum(b);
    } else {
      for (int c = lane; c < width; c += 32) a = fmaf(__bfloat162float(g[c]), xs[c], a);
      b = 1.0f;
    }
    a = warp_sum(a);
    if (lane == 0) as[f] = form.gated ? gate_combine(a, b, form.act, form.limit) : act_apply(a, form.act);
  }
  __syncthreads();
  const __nv_bfloat16* wd = w_down + (int64_t)e * width * ff;
  float* dst = parts + ((int64_t)t * top + slot) * width;
  for (int o = warp; o < width; o += nw) {
    const __nv_bfloat16* d = wd + (int64_t)o * ff;
    float a = 0.f;
    for (int c = lane; c < ff; c += 32) a = fmaf(__bfloat162float(d[c]), as[c], a);
    a = warp_sum(a);
    if (lane == 0) dst[o] = a * w_out;
  }
}

// ---- grouped form -------------------------------------------------------------------------------------------------------
// Bucketing: counts per expert, exclusive scan, then a stable fill (one thread per expert walks the (token, slot) pairs in
// order: deterministic lists without atomics on the order).
__global__ void moe_bucket_kernel(const int32_t* __restrict__ ids, int n_pairs, int experts, int32_t* __restrict__ offsets,
                                  int32_t* __restrict__ list) {
  extern __shared__ int32_t cnt[];   // [experts + 1]
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      const int c = cnt[e];
      cnt[e] = run;
      offsets[e] = run;
      run += c;
    }
    cnt[experts] = run;
    offsets[experts] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int o = cnt[e];
    const int end = cnt[e + 1];
    for (int i = 0; i < n_pairs && o < end; ++i)
      if (ids[i] == e) list[o++] = i;
  }
}

constexpr int kGrpTokens = 16;

template <typename AT>
__global__ void __launch_bounds__(kExpThreads)
moe_expert_grouped_kernel(const AT* __restrict__ x, const __nv_bfloat16* __restrict__ w_gu, const __nv_bfloat16* __restrict__ w_down,
                          const int32_t* __restrict__ offsets, const int32_t* __restrict__ list, const float* __restrict__ wts,
                          int width, int ff, int top, float* __restrict__ parts, ExpertForm form) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int e = blockIdx.y;
  const int lo = offsets[e] + blockIdx.x * kGrpTokens, hi = min(offsets[e + 1], lo + kGrpTokens);
  if (lo >= hi) return;
  const int n = hi - lo;
  float* xs = sm;                          // [16][width]
  float* as = xs + kGrpTokens * width;     // [16][ff]
  __shared__ int pair_of[kGrpTokens];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kExpThreads / 32;
  if (threadIdx.x < kGrpTokens) pair_of[threadIdx.x] = threadIdx.x < n ? list[lo + threadIdx.x] : -1;
  __syncthreads();
  for (int i = threadIdx.x; i < kGrpTokens * width; i += kExpThreads) {
    const int r = i / width, c = i % width;
    xs[i] = r < n ? ld_act<AT>(x, (int64_t)(pair_of[r] / top) * width + c) * (form.weight_input ? wts[pair_of[r]] : 1.0f) : 0.f;
  }
  __syncthreads();
  const __nv_bfloat16* wg = w_gu + (int64_t)e * (form.gated ? 2 : 1) * ff * width;
  const __nv_bfloat16* wu = form.gated ? wg + (int64_t)ff * width : wg;
  for (int f = warp; f < ff; f += nw) {
    const __nv_bfloat16* g = wg + (int64_t)f * width;
    const __nv_bfloat16* u = wu + (int64_t)f * width;
    float a[kGrpTokens], b[kGrpTokens];
#pragma unroll
    for (int r = 0; r < kGrpTokens; ++r) a[r] = b[r] = 0.f;
    for (int c = lane; c < width; c += 32) {
      const float gv = __bfloat162float(g[c]), uv = __bfloat162float(u[c]);
#pragma unroll
      for (int r = 0; r < kGrpTokens; ++r) {
        const float xv = xs[r * width + c];
        a[r] = fmaf(gv, xv, a[r]);
        b[r] = fmaf(uv, xv, b[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < kGrpTokens; ++r) {
      const float av = warp_sum(a[r]), bv = warp_sum(b[r]);
      if (lane == 0) as[r * ff + f] = form.gated ? gate_combine(av, bv, form.act, form.limit) : act_apply(av, form.act);
    }
  }
  __syncthreads();
  const __nv_bfloat16* wd = w_down + (int64_t)e * width * ff;
  for (int o = warp; o < width; o += nw) {
    const __nv_bfloat16* d = wd + (int64_t)o * ff;
    float a[kGrpTokens];
#pragma unroll
    for (int r = 0; r < kGrpTokens; ++r) a[r] = 0.f;
    for (int c = lane; c < ff; c += 32) {
      const float dv = __bfloat162float(d[c]);
#pragma unroll
      for (int r = 0; r < kGrpTokens; ++r) a[r] = fmaf(dv, as[r * ff + c], a[r]);
    }
#pragma unroll
    for (int r = 0; r < kGrpTokens; ++r) {
      const float av = warp_sum(a[r]);
      if (lane == 0 && r < n) parts[(int64_t)pair_of[r] * width + o] = form.weight_input ? av : av * wts[pair_of[r]];
    }
  }
}


// ---- tensor-core form: grouping and gather --------------------------------------------------------------------------------
// One CTA of 32 warps.  Every expert's run of (token, slot) pairs starts on a tile boundary (tiles of N rows); tile_expert
// names the owner of each tile (-1 past the last one), row_pair the pair of each row (-1 for the padding of a run).
// Within a run the pairs keep their order (by token, then slot).  Warp w owns a contiguous stretch of the pair list and
// walks it 32 pairs at a time; __match_any_sync gives every lane the lanes with the same expert, so a row of 32 pairs
// costs one step whatever the number of experts.  First walk: counts per (warp, expert).  Then the runs' first rows
// (a scan over experts) and every warp's first row inside each run (a scan over warps).  Second walk: places.
constexpr int kGroupThreads = 1024;
constexpr int kGroupWarps = kGroupThreads / 32;

__global__ void __launch_bounds__(kGroupThreads)
moe_group_kernel(const int32_t* __restrict__ ids, int n_pairs, int experts, int N, int n_tiles, int32_t* __restrict__ tile_expert,
                 int32_t* __restrict__ row_pair) {
  extern __shared__ int32_t gsm[];
  int32_t* start = gsm;                 // [experts] first row of the expert's run
  int32_t* wcnt = start + experts;      // [32 warps][experts] count, then next free row, of (warp, expert)
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kGroupWarps * experts; i += kGroupThreads) wcnt[i] = 0;
  for (int i = threadIdx.x; i < n_tiles * N; i += kGroupThreads) row_pair[i] = -1;
  for (int i = threadIdx.x; i < n_tiles; i += kGroupThreads) tile_expert[i] = -1;
  const int rows = (n_pairs + 31) / 32, rpw = (rows + kGroupWarps - 1) / kGroupWarps;
  const int r0 = warp * rpw, r1 = min(r0 + rpw, rows);
  int32_t* mine = wcnt + warp * experts;
  __syncthreads();
  for (int pass = 0; pass < 2; ++pass) {
    for (int rb = r0; rb < r1; rb += 8) {
      int ev[8];   // eight rows' experts are requested before the first is used: the walk below is a dependent chain
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = (rb + u) * 32 + lane;
        ev[u] = (rb + u < r1 && i < n_pairs) ? __ldg(ids + i) : -1;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (rb + u >= r1) break;   // warp-uniform
        const int i = (rb + u) * 32 + lane;
        const int e = ev[u] < experts ? ev[u] : -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
          const int before = __popc(same & ((1u << lane) - 1u));
          if (pass == 1) {
            const int row = mine[e] + before;
            if (row < n_tiles * N) row_pair[row] = i;
          }
          __syncwarp(same);
          if (before == 0) mine[e] += __popc(same);   // the group's first lane
        }
        __syncwarp();
      }
    }
    if (pass == 1) break;
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += kGroupThreads) {
      int c = 0;
      for (int w = 0; w < kGroupWarps; ++w) c += wcnt[w * experts + e];
      start[e] = c;   // the expert's pairs; turned into its first row below
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int e = 0; e < experts; ++e) {
        const int nt = (start[e] + N - 1) / N;
        start[e] = run * N;
        for (int j = 0; j < nt && run + j < n_tiles; ++j) tile_expert[run + j] = e;
        run += nt;
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += kGroupThreads) {
      int at = start[e];
      for (int w = 0; w < kGroupWarps; ++w) {
        const int c = wcnt[w * experts + e];
        wcnt[w * experts + e] = at;
        at += c;
      }
    }
    __syncthreads();
  }
}

// xg[row] = x[row_pair[row] / top] (zeros for padding rows); rows of unused tiles are left alone.  width % 8 == 0.
// in_wts given (the mixing weight belongs to the expert's input): the row is scaled by its pair's weight (fp32 product,
// rounded once), and ones[pair] = 1 so that the closing linear's per-pair factor is neutral.
__global__ void __launch_bounds__(128)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ row_pair,
                  int N, int top, int width, __nv_bfloat16* __restrict__ xg, const float* __restrict__ in_wts, float* __restrict__ ones) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  if (tile_expert[row / N] < 0) return;
  const int pair = row_pair[row];
  const int chunks = width >> 3;
  uint4* dst = reinterpret_cast<uint4*>(xg + (int64_t)row * width);
  if (pair < 0) {
    for (int c = threadIdx.x; c < chunks; c += 128) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(pair / top) * width);
  if (in_wts == nullptr) {
    for (int c = threadIdx.x; c < chunks; c += 128) dst[c] = __ldg(src + c);
    return;
  }
  const float wt = in_wts[pair];
  if (threadIdx.x == 0) ones[pair] = 1.0f;
  for (int c = threadIdx.x; c < chunks; c += 128) {
    const uint4 v = __ldg(src + c);
    dst[c] = make_uint4(pack_bf16(bf16lo(v.x) * wt, bf16hi(v.x) * wt), pack_bf16(bf16lo(v.y) * wt, bf16hi(v.y) * wt),
                        pack_bf16(bf16lo(v.z) * wt, bf16hi(v.z) * wt), pack_bf16(bf16lo(v.w) * wt, bf16hi(v.w) * wt));
  }
}

}  // namespace

static int64_t al256(int64_t v) { return (v + 255) / 256 * 256; }

// tensor-core form: rows and tiles of a step of T tokens (every expert's run padded to whole tiles of N rows)
static void moe_tc_shape(int T, int top, int experts, int* N, int* n_tiles) {
  const int pairs = T * top;
  *N = linear_tc_grouped_tile(pairs, experts);
  *n_tiles = pairs / *N + std::min(experts, pairs);
}

bool moe_tc_supported(int width, int ff) { return width % 8 == 0 && ff % 8 == 0; }

// CUDA-core forms: the bucket lists.  Tensor-core form (width > 0, supported shape): tile and row tables, the gathered
// rows, the gate|up rows and the activated rows, for any step of at most T tokens (at most pairs + experts * 128 rows).
int64_t moe_workspace_bytes(int T, int top, int experts, int width, int ff) {
  int64_t b = al256(((int64_t)T * top + experts + 8) * 4);
  if (width > 0 && ff > 0 && moe_tc_supported(width, ff)) {
    const int64_t rows = (int64_t)T * top + (int64_t)experts * 128, tiles = (int64_t)T * top / 16 + experts + 1;
    b = std::max(b, al256(tiles * 4) + al256(rows * 4) + al256(rows * width * 2) + al256(rows * 2 * ff * 2) + al256(rows * ff * 2) +
                        al256((int64_t)T * top * 4));
  }
  return b;
}

static int moe_experts_tc(const __nv_bfloat16* x, const __nv_bfloat16* w_gu, const __nv_bfloat16* w_down, const int32_t* ids,
                          const float* wts, int T, int width, int ff, int experts, int top, float* parts, void* ws,
                          cudaStream_t s, ExpertForm form) {
  int N, n_tiles;
  moe_tc_shape(T, top, experts, &N, &n_tiles);
  const int64_t rows = (int64_t)n_tiles * N;
  char* p = static_cast<char*>(ws);
  int32_t* tile_expert = reinterpret_cast<int32_t*>(p);
  p += al256(((int64_t)T * top / 16 + experts + 1) * 4);
  int32_t* row_pair = reinterpret_cast<int32_t*>(p);
  p += al256(rows * 4);
  __nv_bfloat16* xg = reinterpret_cast<__nv_bfloat16*>(p);
  p += al256(rows * width * 2);
  __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(p);
  p += al256(rows * 2 * ff * 2);
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(p);
  p += al256(rows * ff * 2);
  float* ones = reinterpret_cast<float*>(p);
  const size_t smem_grp = (size_t)experts * (1 + kGroupWarps) * 4;
  B200_REQUIRE(smem_grp <= 200 * 1024, B200_ERR_UNSUPPORTED, "experts: %d experts exceed the grouping kernel", experts);
  static bool done_grp[64] = {};
  if (smem_grp > 48 * 1024) B200_CUDA(ensure_dynamic_smem(moe_group_kernel, 200 * 1024, done_grp));
  B200_CUDA(launch(moe_group_kernel, dim3(1), dim3(kGroupThreads), smem_grp, s, ids, T * top, experts, N, n_tiles,
                   tile_expert, row_pair));
  B200_CUDA(launch(moe_gather_kernel, dim3((unsigned)rows), dim3(128), (size_t)0, s, x, (const int32_t*)tile_expert,
                   (const int32_t*)row_pair, N, top, width, xg, form.weight_input ? wts : (const float*)nullptr, ones));
  if (form.weight_input) wts = ones;
  int rc;
  static const int fuse_env = getenv("B200_MOE_FUSE_SILU") ? atoi(getenv("B200_MOE_FUSE_SILU")) : 1;
  if (!form.gated) {
    // one projection, activated in place
    rc = linear_tc_grouped(xg, width, N, n_tiles, w_gu, experts, ff, width, tile_expert, act, ff, nullptr, nullptr, nullptr, s);
    if (rc) return rc;
    rc = ff_act(false, act, act, (int)rows, ff, false, form.act, s);
    if (rc) return rc;
  } else if (form.act == B200_ACT_SWIGLU_CLAMP && fuse_env && ff % 64 == 0 && (N <= 64 || fuse_env > 1)) {
    // the clamped gate in the same epilogue (it sees the bf16-rounded gate and up values the separate kernel would read)
    rc = linear_tc_grouped_gate_up(xg, width, N, n_tiles, w_gu, experts, ff, width, tile_expert, act, s, form.act, form.limit);
    if (rc) return rc;
  } else if (form.act != B200_ACT_SILU) {
    rc = linear_tc_grouped(xg, width, N, n_tiles, w_gu, experts, 2 * ff, width, tile_expert, gu, 2 * ff, nullptr, nullptr, nullptr, s);
    if (rc) return rc;
    rc = ff_act(false, gu, act, (int)rows, ff, true, form.act, s, form.limit);
    if (rc) return rc;
  } else if (fuse_env && ff % 64 == 0 && (N <= 64 || fuse_env > 1)) {
    // gate and up rows of a slab come in as two 64-row boxes; the epilogue activates (as the dense gate|up linear does).
    // Decode-sized tiles only: at 128 tokens per tile the epilogue's exponentials cost more than the pass they save
    // (measured: 145 us against 119 + 19 us for 8192 rows of width 2048 into ff 1024)
    rc = linear_tc_grouped_gate_up(xg, width, N, n_tiles, w_gu, experts, ff, width, tile_expert, act, s);
    if (rc) return rc;
  } else {
    rc = linear_tc_grouped(xg, width, N, n_tiles, w_gu, experts, 2 * ff, width, tile_expert, gu, 2 * ff, nullptr, nullptr, nullptr, s);
    if (rc) return rc;
    rc = silu_mul(gu, act, (int)rows, ff, s);
    if (rc) return rc;
  }
  return linear_tc_grouped(act, ff, N, n_tiles, w_down, experts, width, ff, tile_expert, nullptr, 0, row_pair, wts, parts, s);
}

int moe_route(bool f32, const void* x, const __nv_bfloat16* w_router, const float* bias, int T, int width, int experts, int top,
              int groups, int keep, int32_t* out_ids, float* out_w, cudaStream_t s, float* logits_ws, void* lin_ws,
              int64_t lin_ws_bytes, int score_mode) {
  const int sg = score_mode;
  if (T == 0) return B200_OK;
  B200_REQUIRE(experts > 0 && top > 0 && top <= experts, B200_ERR_INVALID, "router: top %d of %d experts", top, experts);
  if (groups < 1) groups = 1;
  B200_REQUIRE(experts % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (experts / groups), B200_ERR_INVALID,
               "router: %d experts in %d groups, keep %d, top %d", experts, groups, keep, top);
  static const int tc_env = getenv("B200_STACK_TC") ? atoi(getenv("B200_STACK_TC")) : 1;
  const size_t smem_sel = (size_t)kSelWarps * (2 * experts + groups) * 4;
  if (!f32 && tc_env && logits_ws && width % 8 == 0 && reinterpret_cast<uintptr_t>(w_router) % 16 == 0 && smem_sel <= 48 * 1024 &&
      linear_tc_supported(T, experts, width) && (lin_ws == nullptr || linear_tc_workspace_bytes(T, experts, width) <= lin_ws_bytes)) {
    // bf16 rows: the logits are a tcgen05 linear with unrounded fp32 output (bf16 products are exact in fp32, the sum is
    // fp32), then one warp per token selects
    LinearExtra ex;
    ex.mode = 4;
    ex.out_f32 = logits_ws;
    const int rc = linear_tc((const __nv_bfloat16*)x, width, w_router, nullptr, nullptr, experts, T, experts, width, lin_ws,
                             lin_ws_bytes, &ex, s);
    if (rc) return rc;
    B200_CUDA(launch(moe_select_kernel, dim3((T + kSelWarps - 1) / kSelWarps), dim3(kSelWarps * 32), smem_sel, s,
                     (const float*)logits_ws, bias, T, experts, top, groups, keep, out_ids, out_w, sg));
    return B200_OK;
  }
  const size_t smem = ((size_t)width + 2 * experts + groups) * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "router: row of %zu bytes does not fit shared memory", smem);
  static bool done[2][64] = {};
  if (f32) {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(moe_route_kernel<float>, 200 * 1024, done[0]));
    B200_CUDA(launch(moe_route_kernel<float>, dim3(T), dim3(kRouteThreads), smem, s, (const float*)x, w_router, bias, width, experts,
                     top, groups, keep, out_ids, out_w, sg));
  } else {
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(moe_route_kernel<__nv_bfloat16>, 200 * 1024, done[1]));
    B200_CUDA(launch(moe_route_kernel<__nv_bfloat16>, dim3(T), dim3(kRouteThreads), smem, s, (const __nv_bfloat16*)x, w_router,
                     bias, width, experts, top, groups, keep, out_ids, out_w, sg));
  }
  return B200_OK;
}

template <typename AT>
static int moe_experts_t(const AT* x, const __nv_bfloat16* w_gu, const __nv_bfloat16* w_down, const int32_t* ids, const float* wts,
                         int T, int width, int ff, int experts, int top, float* parts, void* ws, bool grouped, cudaStream_t s,
                         ExpertForm form) {
  const size_t smem_g = (size_t)kGrpTokens * (width + ff) * 4;
  if (grouped && ws != nullptr && smem_g <= 200 * 1024) {
    int32_t* offsets = static_cast<int32_t*>(ws);
    int32_t* list = offsets + experts + 8;
    B200_CUDA(launch(moe_bucket_kernel, dim3(1), dim3(256), (size_t)(experts + 1) * 4, s, ids, T * top, experts, offsets, list));
    static bool done[64] = {};
    if (smem_g > 48 * 1024) B200_CUDA(ensure_dynamic_smem(moe_expert_grouped_kernel<AT>, 200 * 1024, done));
    const int tiles = (T * top + kGrpTokens - 1) / kGrpTokens;   // upper bound of any expert's tiles
    B200_CUDA(launch(moe_expert_grouped_kernel<AT>, dim3(std::min(tiles, (T + kGrpTokens - 1) / kGrpTokens + 1), experts),
                     dim3(kExpThreads), smem_g, s, x, w_gu, w_down, (const int32_t*)offsets, (const int32_t*)list, wts, width, ff,
                     top, parts, form));
    return B200_OK;
  }
  const size_t smem = ((size_t)width + ff) * 4;
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_UNSUPPORTED, "experts: width %d + ff %d do not fit shared memory", width, ff);
  static bool done2[64] = {};
  if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(moe_expert_rows_kernel<AT>, 200 * 1024, done2));
  B200_CUDA(launch(moe_expert_rows_kernel<AT>, dim3(T, top), dim3(kExpThreads), smem, s, x, w_gu, w_down, ids, wts, width, ff, top,
                   parts, form));
  return B200_OK;
}

// parts [T][top][width] fp32: the chosen experts' outputs times their mixing weights, one row per (token, slot).
int moe_experts(bool f32, const void* x, const __nv_bfloat16* w_gu, const __nv_bfloat16* w_down, const int32_t* ids,
                const float* wts, int T, int width, int ff, int experts, int top, float* parts, void* ws, cudaStream_t s,
                ExpertForm form) {
  if (T == 0) return B200_OK;
  static const int tc_env = getenv("B200_STACK_TC") ? atoi(getenv("B200_STACK_TC")) : 1;
  if (!f32 && tc_env && ws && moe_tc_supported(width, ff))
    return moe_experts_tc((const __nv_bfloat16*)x, w_gu, w_down, ids, wts, T, width, ff, experts, top, parts, ws, s, form);
  // an expert is chosen at most once per token, so it has at most T tokens: ceil(T / 16) tiles bound every expert
  const bool grouped = (int64_t)T * top >= 4 * (int64_t)experts && T >= 64;
  return f32 ? moe_experts_t<float>((const float*)x, w_gu, w_down, ids, wts, T, width, ff, experts, top, parts, ws, grouped, s, form)
             : moe_experts_t<__nv_bfloat16>((const __nv_bfloat16*)x, w_gu, w_down, ids, wts, T, width, ff, experts, top, parts,
                                            ws, grouped, s, form);
}

}  // namespace b200
