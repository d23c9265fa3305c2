// Paged causal attention over latent cache rows on the tensor cores (bf16 serving mode of B200_MIXER_LATENT), over the whole
// context or over a sliding window of its last `window` keys.
//
// One kv head serves every query head, and a key row's leading `rank` entries are its value, so all heads of a token share
// every byte of the cache: a CTA takes 16 (row, head) pairs of one run of consecutive rows of a sequence and walks the
// context in tiles of 64 keys.  Per tile the key rows are gathered once into shared memory (cp.async, 16-byte chunks through
// the block table), S = Q K^T and O += P V run as bf16 mma.sync m16n8k16 with fp32 accumulators, and the softmax between
// them is fp32: scores scaled and masked per pair (a pair sees keys below its own context length), running maximum and sum
// per pair, weights rounded to bf16 only as the second product's operand.  An optional per-head sink joins the denominator
// at the end.  Warp w (of 8) owns keys 8w..8w+7 of a tile for the scores and value columns 16(w + 8g) .. for the output.
//
// Steps with few (row, head) pairs and long contexts split the context over several CTAs per pair group (n_splits): each
// leaves unnormalised sums with its maximum and denominator, a merge kernel combines them.
//
// The same kernel serves grouped-query attention with a value cache of its own (paged_attn_mma): the pairs of a CTA are then
// (row, head) pairs of ONE kv head's group, the key tile [64][dim] and the value tile [64][vdim] are gathered side by side.
//
// Queries come as fp32 rows [T][heads][krow] (rounded to bf16 when staged); output rows are bf16 [T][heads][rank].
// Shapes: krow and rank multiples of 16, rank <= 512.  Everything else (and the 32-bit mode) takes attn_anydim.cu; both walk
// the same cache and the same run list, and agree within bf16 rounding of the operands.
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kLaKeys = 64, kLaPairs = 16, kLaWarps = 8, kLaThreads = kLaWarps * 32;
constexpr int kSsStride = kLaKeys + 4;    // fp32 score rows
constexpr int kPsStride = kLaKeys + 8;    // bf16 weight rows (144 bytes: 16-byte aligned, conflict-free for ldmatrix)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float& c0, float& c1, float& c2, float& c3, const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int NG>   // 16-column output groups per warp: rank <= 128 NG
__global__ void __launch_bounds__(kLaThreads)
latent_attn_mma_kernel(const float* __restrict__ q, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                       int kv_heads, const int32_t* __restrict__ block_table,
                       int bt_stride, const int32_t* __restrict__ row_to_seq, const int32_t* __restrict__ ctx_lens,
                       __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ runs, const int32_t* __restrict__ n_runs, int heads,
                       int krow, int rank, int block_size, float scale, const float* __restrict__ sink, int n_splits,
                       float* __restrict__ part, int window) {
  extern __shared__ __align__(16) unsigned char smraw[];
  pdl_wait();
  pdl_launch_dependents();
  // G query heads share kv head g; a pair i of the group is (row t0 + i / G, head g G + i % G).  Latent rows: one kv head, G = heads.
  const int G = heads / kv_heads;
  const int item = blockIdx.x, chunk = blockIdx.y % G, g = blockIdx.y / G;
  if (item >= *n_runs) return;
  const int t0 = runs[2 * item], nr = runs[2 * item + 1];
  const int nq = nr * G, i0 = chunk * kLaPairs;
  if (i0 >= nq) return;
  const int ks = krow + 8;   // bf16 elements per staged row: 16-byte aligned, 4 words off a bank multiple
  // a value cache of its own (vc) is staged beside the keys in rows of rank + 8; else a key row's leading entries are its value
  const int vs = vc ? rank + 8 : ks;
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);      // [64][ks]
  __nv_bfloat16* Vs = vc ? Ks + kLaKeys * ks : Ks;                  // [64][vs]
  __nv_bfloat16* Qs = Vs + (vc ? kLaKeys * vs : kLaKeys * ks);      // [16][ks]
  float* Ss = reinterpret_cast<float*>(Qs + kLaPairs * ks);         // [16][68]
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(Ss + kLaPairs * kSsStride);   // [16][72]
  float* corr = reinterpret_cast<float*>(Ps + kLaPairs * kPsStride);                 // [16]
  float* mrow = corr + kLaPairs;
  float* lrow = mrow + kLaPairs;
  int* ctxp = reinterpret_cast<int*>(lrow + kLaPairs);
  int* lop = ctxp + kLaPairs;   // the first key a pair sees (0 without a window)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kLaPairs) {
    const int i = i0 + tid;
    ctxp[tid] = i < nq ? ctx_lens[t0 + i / G] : 0;
    lop[tid] = window > 0 ? max(ctxp[tid] - window, 0) : 0;
    mrow[tid] = -INFINITY;
    lrow[tid] = 0.f;
  }
  for (int e = tid; e < kLaPairs * krow; e += kLaThreads) {
    const int p = e / krow, d = e % krow, i = i0 + p;
    Qs[p * ks + d] = __float2bfloat16_rn(i < nq ? q[((int64_t)(t0 + i / G) * heads + g * G + i % G) * krow + d] : 0.f);
  }
  const int last_row = min(nr - 1, (i0 + kLaPairs - 1) / G);
  const int ctx_max = ctx_lens[t0 + last_row];
  const int32_t* bt = block_table + (int64_t)(row_to_seq ? row_to_seq[t0] : t0) * bt_stride;
  const int cpr = krow >> 3, cpv = rank >> 3;   // 16-byte chunks per key / value row
  float o[NG][8];
#pragma unroll
  for (int cg = 0; cg < NG; ++cg)
#pragma unroll
    for (int j = 0; j < 8; ++j) o[cg][j] = 0.f;
  __syncthreads();

  // with n_splits > 1 this CTA walks only its share of the tiles and leaves unnormalised sums for the merge kernel
  // (with a window the walk starts at the tile that holds the oldest key the group's first row sees)
  const int tile0 = window > 0 ? max(ctx_lens[t0 + i0 / G] - window, 0) / kLaKeys : 0;
  const int tiles = (ctx_max + kLaKeys - 1) / kLaKeys - tile0, per = (tiles + n_splits - 1) / n_splits;
  const int base_lo = (tile0 + blockIdx.z * per) * kLaKeys, base_hi = min(ctx_max, (tile0 + (int)(blockIdx.z + 1) * per) * kLaKeys);
  for (int base = base_lo; base < base_hi; base += kLaKeys) {
    const int n = min(kLaKeys, ctx_max - base);
    {
      // four threads per key row, alternate 16-byte chunks: one block-table lookup per thread and tile
      const int r = tid >> 2;
      __nv_bfloat16* dst = Ks + r * ks;
      __nv_bfloat16* dstv = Vs + r * vs;
      if (r < n) {
        const int j = base + r;
        const int64_t crow = ((int64_t)bt[j / block_size] * kv_heads + g) * block_size + j % block_size;
        const __nv_bfloat16* src = kc + crow * krow;
        for (int c = tid & 3; c < cpr; c += 4) cp_async16(dst + c * 8, src + c * 8);
        if (vc) {
          const __nv_bfloat16* srcv = vc + crow * rank;
          for (int c = tid & 3; c < cpv; c += 4) cp_async16(dstv + c * 8, srcv + c * 8);
        }
      } else {
        // rows past the context: finite values under zero weights
        for (int c = tid & 3; c < cpr; c += 4) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        if (vc)
          for (int c = tid & 3; c < cpv; c += 4) *reinterpret_cast<uint4*>(dstv + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_wait_all();
    __syncthreads();
    // scores of this warp's 8 keys for all 16 pairs
    {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      const __nv_bfloat16* ap = Qs + (lane & 15) * ks + (lane >> 4) * 8;
      const __nv_bfloat16* bp = Ks + (warp * 8 + (lane & 7)) * ks + ((lane >> 3) & 1) * 8;
#pragma unroll 4
      for (int k0 = 0; k0 < krow; k0 += 16) {
        uint32_t a[4], b[2];
        ldsm_x4(a, ap + k0);
        ldsm_x2(b, bp + k0);
        mma_bf16(s0, s1, s2, s3, a, b[0], b[1]);
      }
      const int row = lane >> 2, col = warp * 8 + (lane & 3) * 2;
      Ss[row * kSsStride + col] = s0;
      Ss[row * kSsStride + col + 1] = s1;
      Ss[(row + 8) * kSsStride + col] = s2;
      Ss[(row + 8) * kSsStride + col + 1] = s3;
    }
    __syncthreads();
    // softmax bookkeeping: this warp's 2 pairs, two keys per lane
#pragma unroll
    for (int rr = 0; rr < kLaPairs / kLaWarps; ++rr) {
      const int row = warp * (kLaPairs / kLaWarps) + rr, c = ctxp[row], lo = lop[row];
      const int j0 = base + lane, j1 = j0 + 32;
      const bool see0 = j0 < c && j0 >= lo, see1 = j1 < c && j1 >= lo;
      const float s0 = see0 ? Ss[row * kSsStride + lane] * scale : -INFINITY;
      const float s1 = see1 ? Ss[row * kSsStride + lane + 32] * scale : -INFINITY;
      const float m_old = mrow[row];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
      float p0 = 0.f, p1 = 0.f, cr = 1.f;
      if (m_new != -INFINITY) {
        p0 = see0 ? expf(s0 - m_new) : 0.f;
        p1 = see1 ? expf(s1 - m_new) : 0.f;
        cr = expf(m_old - m_new);
      }
      const float sum = warp_sum(p0 + p1);
      Ps[row * kPsStride + lane] = __float2bfloat16_rn(p0);
      Ps[row * kPsStride + lane + 32] = __float2bfloat16_rn(p1);
      __syncwarp();
      if (lane == 0) {
        mrow[row] = m_new;
        lrow[row] = lrow[row] * cr + sum;
        corr[row] = cr;
      }
    }
    __syncthreads();
    // O = O * corr + P V over this warp's column groups
    {
      const float c_lo = corr[lane >> 2], c_hi = corr[(lane >> 2) + 8];
#pragma unroll
      for (int cg = 0; cg < NG; ++cg) {
        o[cg][0] *= c_lo; o[cg][1] *= c_lo; o[cg][4] *= c_lo; o[cg][5] *= c_lo;
        o[cg][2] *= c_hi; o[cg][3] *= c_hi; o[cg][6] *= c_hi; o[cg][7] *= c_hi;
      }
      const __nv_bfloat16* ap = Ps + (lane & 15) * kPsStride + (lane >> 4) * 8;
      const __nv_bfloat16* vp = Vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * vs + (lane >> 4) * 8;
#pragma unroll
      for (int kk = 0; kk < kLaKeys / 16; ++kk) {
        uint32_t a[4];
        ldsm_x4(a, ap + kk * 16);
#pragma unroll
        for (int cg = 0; cg < NG; ++cg) {
          const int col0 = (warp + kLaWarps * cg) * 16;
          if (col0 < rank) {
            uint32_t b[4];
            ldsm_x4_t(b, vp + kk * 16 * vs + col0);
            mma_bf16(o[cg][0], o[cg][1], o[cg][2], o[cg][3], a, b[0], b[1]);
            mma_bf16(o[cg][4], o[cg][5], o[cg][6], o[cg][7], a, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
  }
  if (n_splits > 1) {
    // partial rows [pair][split][rank | m | l] fp32
    const int prow = rank + 2;
    if (tid < kLaPairs && i0 + tid < nq) {
      const int i = i0 + tid;
      float* dst = part + (((int64_t)(t0 + i / G) * heads + g * G + i % G) * n_splits + blockIdx.z) * prow;
      dst[rank] = mrow[tid];
      dst[rank + 1] = lrow[tid];
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int p = (lane >> 2) + half * 8, i = i0 + p;
      if (i >= nq) continue;
      float* dst = part + (((int64_t)(t0 + i / G) * heads + g * G + i % G) * n_splits + blockIdx.z) * prow;
#pragma unroll
      for (int cg = 0; cg < NG; ++cg) {
        const int col0 = (warp + kLaWarps * cg) * 16;
        if (col0 < rank) {
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            const int col = col0 + nt * 8 + (lane & 3) * 2;
            dst[col] = o[cg][nt * 4 + half * 2];
            dst[col + 1] = o[cg][nt * 4 + half * 2 + 1];
          }
        }
      }
    }
    return;
  }
  // finish: sink, normalise, store
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int p = (lane >> 2) + half * 8, i = i0 + p;
    if (i >= nq) continue;
    const int t = t0 + i / G, h = g * G + i % G;
    float l = lrow[p], osc = 1.f;
    if (sink != nullptr) {
      const float m = mrow[p], sk = sink[h], mn = fmaxf(m, sk);
      osc = expf(m - mn);
      l = l * osc + expf(sk - mn);
    }
    const float inv = l > 0.f ? osc / l : 0.f;
    __nv_bfloat16* dst = out + ((int64_t)t * heads + h) * rank;
#pragma unroll
    for (int cg = 0; cg < NG; ++cg) {
      const int col0 = (warp + kLaWarps * cg) * 16;
      if (col0 < rank) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = col0 + nt * 8 + (lane & 3) * 2;
          *reinterpret_cast<__nv_bfloat162*>(dst + col) =
              __floats2bfloat162_rn(o[cg][nt * 4 + half * 2] * inv, o[cg][nt * 4 + half * 2 + 1] * inv);
        }
      }
    }
  }
}

// One warp per (row, head): the splits' sums are brought to one maximum (the sink's included), added and normalised.
// Lane z holds split z's maximum and denominator; the per-split factors are then shared by shuffles and every lane's loads
// of a column are independent of one another.
constexpr int kLaMaxSplits = 16;
__global__ void __launch_bounds__(128)
latent_attn_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int n_pairs, int heads, int rank, int n_splits,
                         const float* __restrict__ sink) {
  pdl_wait();
  pdl_launch_dependents();
  const int pair = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (pair >= n_pairs) return;
  const int prow = rank + 2;
  const float* src = part + (int64_t)pair * n_splits * prow;
  const float mz = lane < n_splits ? src[lane * prow + rank] : -INFINITY;
  const float lz = lane < n_splits ? src[lane * prow + rank + 1] : 0.f;
  const float sk = sink ? sink[pair % heads] : -INFINITY;
  const float m = fmaxf(warp_max(mz), sk);
  const float ez = mz != -INFINITY ? expf(mz - m) : 0.f;
  const float l = warp_sum(lz * ez) + (sink ? expf(sk - m) : 0.f);
  const float fz = l > 0.f ? ez / l : 0.f;
  float f[kLaMaxSplits];
#pragma unroll
  for (int z = 0; z < kLaMaxSplits; ++z) f[z] = __shfl_sync(0xffffffffu, fz, z);
  for (int c = lane; c < rank; c += 32) {
    float v[kLaMaxSplits];
#pragma unroll
    for (int z = 0; z < kLaMaxSplits; ++z) v[z] = z < n_splits ? src[z * prow + c] : 0.f;
    float a = 0.f;
#pragma unroll
    for (int z = 0; z < kLaMaxSplits; ++z) a = fmaf(v[z], f[z], a);
    out[(int64_t)pair * rank + c] = __float2bfloat16_rn(a);
  }
}

}  // namespace

// Splits of the context for a step of T rows whose longest context is max_ctx: 1 when the (row, head) pairs fill the SMs
// anyway or the context is short; else enough CTAs for two per SM, at least two tiles each, within a workspace of ws_bytes.
int latent_attn_splits(int T, int heads, int rank, int max_ctx, int64_t ws_bytes) {
  const int ctas = (T * heads + kLaPairs - 1) / kLaPairs;
  // measured at 513 tokens: with 64 pair groups the merge launch costs what the split saves, with one it pays
  if (ctas >= kNumSMs || max_ctx <= (ctas < 16 ? 4 : 16) * kLaKeys) return 1;
  const int tiles = (max_ctx + kLaKeys - 1) / kLaKeys;
  int n = std::min(std::min((tiles + 1) / 2, (2 * kNumSMs + ctas - 1) / ctas), kLaMaxSplits);
  const int64_t per_split = (int64_t)T * heads * (rank + 2) * 4;
  while (n > 1 && n * per_split > ws_bytes) --n;
  return std::max(n, 1);
}

static size_t la_smem(int krow, int rank, bool own_values) {
  return (size_t)(kLaKeys + kLaPairs) * (krow + 8) * 2 + (own_values ? (size_t)kLaKeys * (rank + 8) * 2 : 0) +
         kLaPairs * (kSsStride * 4 + kPsStride * 2 + 20);
}

bool latent_attn_mma_supported(int heads, int krow, int rank) {
  static const int env = getenv("B200_LATENT_MMA") ? atoi(getenv("B200_LATENT_MMA")) : 1;
  return env && heads > 0 && krow % 16 == 0 && rank % 16 == 0 && rank > 0 && rank <= 512 && rank <= krow && la_smem(krow, rank, false) <= 200 * 1024;
}

// grouped-query attention with a value cache of its own on the same kernel: key rows of `dim`, value rows of `vdim` entries
bool paged_attn_mma_supported(int heads, int kv_heads, int dim, int vdim) {
  static const int env = getenv("B200_ATTN_MMA") ? atoi(getenv("B200_ATTN_MMA")) : 1;
  return env && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim % 16 == 0 && vdim % 16 == 0 && vdim > 0 && vdim <= 512 &&
         la_smem(dim, vdim, true) <= 200 * 1024;
}

static int attn_mma_launch(const float* q, const __nv_bfloat16* kc, const __nv_bfloat16* vc, int kv_heads, const int32_t* block_table,
                           int bt_stride, const int32_t* row_to_seq, const int32_t* ctx_lens, __nv_bfloat16* out, const int32_t* runs,
                           const int32_t* n_runs, int T, int heads, int krow, int rank, int block_size, float scale, const float* sink,
                           cudaStream_t s, int n_splits, float* part, int window) {
  if (n_splits < 1 || part == nullptr) n_splits = 1;
  B200_REQUIRE(n_splits <= kLaMaxSplits, B200_ERR_INVALID, "attention: %d splits (at most %d)", n_splits, kLaMaxSplits);
  B200_REQUIRE(reinterpret_cast<uintptr_t>(kc) % 16 == 0 && reinterpret_cast<uintptr_t>(vc) % 16 == 0, B200_ERR_INVALID,
               "attention: cache not 16-byte aligned");
  const size_t smem = la_smem(krow, rank, vc != nullptr);
  // a run has at most 16 rows, so a kv head's group has at most 16 G pairs: G chunks of 16
  const dim3 grid(T, heads, n_splits), block(kLaThreads);
#define LA(NGV)                                                                                                                     \
  do {                                                                                                                              \
    static bool done[64] = {};                                                                                                      \
    if (smem > 48 * 1024) B200_CUDA(ensure_dynamic_smem(latent_attn_mma_kernel<NGV>, 200 * 1024, done));                            \
    B200_CUDA(launch(latent_attn_mma_kernel<NGV>, grid, block, smem, s, q, kc, vc, kv_heads, block_table, bt_stride, row_to_seq, ctx_lens, \
                     out, runs, n_runs, heads, krow, rank, block_size, scale, sink, n_splits, part, window));                       \
  } while (0)
  if (rank <= 128) LA(1);
  else if (rank <= 256) LA(2);
  else LA(4);
#undef LA
  if (n_splits > 1)
    B200_CUDA(launch(latent_attn_merge_kernel, dim3((T * heads + 3) / 4), dim3(128), (size_t)0, s, (const float*)part, out, T * heads, heads,
                     rank, n_splits, sink));
  return B200_OK;
}

// runs / n_runs: the run list of the step (attn_anydim.cu builds it: runs of at most 16 consecutive rows of one sequence)
int latent_attn_mma(const float* q, const __nv_bfloat16* kc, const int32_t* block_table, int bt_stride, const int32_t* row_to_seq,
                    const int32_t* ctx_lens, __nv_bfloat16* out, const int32_t* runs, const int32_t* n_runs, int T, int heads, int krow,
                    int rank, int block_size, float scale, const float* sink, cudaStream_t s, int n_splits, float* part, int window) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(latent_attn_mma_supported(heads, krow, rank), B200_ERR_UNSUPPORTED, "latent_attn_mma: shape %d / %d / %d", heads, krow, rank);
  return attn_mma_launch(q, kc, nullptr, 1, block_table, bt_stride, row_to_seq, ctx_lens, out, runs, n_runs, T, heads, krow, rank, block_size,
                         scale, sink, s, n_splits, part, window);
}

// caches [block][kv_heads][block_size][dim | vdim] bf16, fp32 queries [T][heads][dim], bf16 output [T][heads][vdim]
int paged_attn_mma(const float* q, const __nv_bfloat16* kc, const __nv_bfloat16* vc, const int32_t* block_table, int bt_stride,
                   const int32_t* row_to_seq, const int32_t* ctx_lens, __nv_bfloat16* out, const int32_t* runs, const int32_t* n_runs, int T,
                   int heads, int kv_heads, int dim, int vdim, int block_size, float scale, const float* sink, cudaStream_t s, int n_splits,
                   float* part, int window) {
  if (T == 0) return B200_OK;
  B200_REQUIRE(vc && paged_attn_mma_supported(heads, kv_heads, dim, vdim), B200_ERR_UNSUPPORTED, "paged_attn_mma: shape %d / %d / %d / %d", heads,
               kv_heads, dim, vdim);
  return attn_mma_launch(q, kc, vc, kv_heads, block_table, bt_stride, row_to_seq, ctx_lens, out, runs, n_runs, T, heads, dim, vdim, block_size,
                         scale, sink, s, n_splits, part, window);
}

}  // namespace b200
