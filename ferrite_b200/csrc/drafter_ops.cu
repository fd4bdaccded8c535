// Drafter-side kernels: GEMV over affine 4-bit weights (groups of 64, the MLX layout the block drafter ships in) and
// the top-16 selection over the vocabulary that seeds a draft block.
//
//   w4_gemv   y[m][n] = sum_k x[m][k] (scale[n][k/64] * q[n][k] + bias[n][k/64]) (+ res), q = 4-bit codes packed
//             eight per 32-bit word, low nibble first; up to 8 rows; one warp per output feature
//   topk16    the 16 largest logits of every row in descending order (ties: lower index first), 16 bounded passes of
//             a block-wide arg-max that only admits candidates ordered after the previous pick
// Counterparts in the reference: `fe_df_gemv4*`, `fe_df_topk16` (`kernels/k-dflash/src`), host `quant4`
// (`crates/fe-dflash/src/lib.rs:66`).
#include "api_ext.h"
#include "common.cuh"

namespace fb {

template <int M>
__global__ void __launch_bounds__(256) w4_gemv_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                                      const uint32_t* __restrict__ qw, const __nv_bfloat16* __restrict__ scales,
                                                      const __nv_bfloat16* __restrict__ biases,
                                                      const __nv_bfloat16* __restrict__ res, int rows, int N, int K, long ldx,
                                                      long ldy) {
  extern __shared__ float xs_w4[];                             // [M][K] fp32 + [M][K / 64] group sums
  float* gs = xs_w4 + (size_t)M * K;
  for (int i = threadIdx.x; i < M * K; i += blockDim.x) {
    const int m = i / K, k = i % K;
    xs_w4[i] = m < rows ? bf2f(x[(size_t)m * ldx + k]) : 0.f;
  }
  __syncthreads();
  const int ng = K / 64;
  for (int i = threadIdx.x; i < M * ng; i += blockDim.x) {     // sum of x over each group: the bias term factors out
    const int m = i / ng, g = i % ng;
    float s = 0.f;
    for (int j = 0; j < 64; ++j) s += xs_w4[m * K + g * 64 + j];
    gs[i] = s;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const uint32_t* qrow = qw + (size_t)n * (K / 8);
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int w = lane; w < K / 8; w += 32) {                     // one word = 8 codes of one group
    const uint32_t q = __ldg(qrow + w);
    const float sc = bf2f(scales[(size_t)n * ng + (w >> 3)]);
    float part[M];
#pragma unroll
    for (int m = 0; m < M; ++m) part[m] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = (float)((q >> (4 * j)) & 0xF);
#pragma unroll
      for (int m = 0; m < M; ++m) part[m] = fmaf(c, xs_w4[m * K + w * 8 + j], part[m]);
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(sc, part[m], acc[m]);
  }
  for (int g = lane; g < ng; g += 32) {
    const float b = bf2f(biases[(size_t)n * ng + g]);
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(b, gs[m * ng + g], acc[m]);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m < rows) {
      float o = v;
      if (res) o += bf2f(res[(size_t)m * ldy + n]);
      y[(size_t)m * ldy + n] = f2bf(o);
    }
  }
}

// ordering: a before b  <=>  a.v > b.v, or equal values and a.i < b.i
__device__ __forceinline__ bool tk_before(float av, int ai, float bv, int bi) { return av > bv || (av == bv && ai < bi); }

template <typename T>
__global__ void __launch_bounds__(1024) topk16_kernel(int* __restrict__ ids, float* __restrict__ vals,
                                                      const T* __restrict__ logits, long stride, int vocab) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float pv_s;
  __shared__ int pi_s;
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* lp = logits + (size_t)row * stride;
  float pv = INFINITY;
  int pi = -1;                                                 // previous pick: everything is ordered after (+inf, -1)
  for (int r = 0; r < 16; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = sizeof(T) == 2 ? bf2f(reinterpret_cast<const __nv_bfloat16*>(lp)[i]) : reinterpret_cast<const float*>(lp)[i];
      if (v == v && tk_before(pv, pi, v, i) && tk_before(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (tk_before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < (int)(blockDim.x >> 5) ? sv[lane] : -INFINITY;
      bi = lane < (int)(blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (tk_before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0) {
        pv_s = bv; pi_s = bi;
        ids[row * 16 + r] = bi == 0x7fffffff ? 0 : bi;
        if (vals) vals[row * 16 + r] = bv;
      }
    }
    __syncthreads();
    pv = pv_s; pi = pi_s;
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_w4_gemv(void* y, const void* x, const void* qweight, const void* scales, const void* biases,
                          const void* res, int M, int N, int K, long ldx, long ldy, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 8 || K % 64) return -1;
  const int MT = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
  const size_t smem = (size_t)MT * (K + K / 64) * sizeof(float);
  if (smem > 200 * 1024) return -2;
#define FB_W4(MTT)                                                                                                  \
  do {                                                                                                              \
    static bool done = false;                                                                                       \
    if (!done) {                                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(w4_gemv_kernel<MTT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      if (e != cudaSuccess) return (int)e;                                                                          \
      done = true;                                                                                                  \
    }                                                                                                               \
    w4_gemv_kernel<MTT><<<(N + 7) / 8, 256, smem, s>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const uint32_t*)qweight, \
        (const __nv_bfloat16*)scales, (const __nv_bfloat16*)biases, (const __nv_bfloat16*)res, M, N, K, ldx, ldy);    \
  } while (0)
  if (MT == 1) FB_W4(1); else if (MT == 2) FB_W4(2); else if (MT == 4) FB_W4(4); else FB_W4(8);
#undef FB_W4
  return (int)cudaGetLastError();
}

extern "C" int fb_topk16(int* ids, float* vals, const void* logits, long stride, int rows, int vocab, int is_f32,
                         cudaStream_t s) {
  if (rows <= 0) return 0;
  if (vocab < 16) return -1;
  if (is_f32) topk16_kernel<float><<<rows, 1024, 0, s>>>(ids, vals, (const float*)logits, stride, vocab);
  else topk16_kernel<__nv_bfloat16><<<rows, 1024, 0, s>>>(ids, vals, (const __nv_bfloat16*)logits, stride, vocab);
  return (int)cudaGetLastError();
}

// ---- block-drafter sublayers ---------------------------------------------------------------------------------------
namespace fb {

// Grouped dynamic causal conv over the rows of a draft block (two taps, causal inside the block):
//   y[t][j] = (base[0][j] + c[t][g]) x[t][j] + [t % blk != 0] (base[1][j] + c[t][groups + g]) x[t-1][j],  g = j / group
// c = coef + coff (row stride ldc): per-row kernel offsets from a projection of the row. With `res` the result is
// added into res (bf16) instead of written to out. One thread per 8 channels (`group` is a multiple of 8 or divides 8).
// Counterpart of `fe_df_dynconv` (`kernels/k-dflash/src/lib.rs:28`), with run-time width and group size.
__global__ void dynconv_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                               const __nv_bfloat16* __restrict__ coef, long ldc, const __nv_bfloat16* __restrict__ base,
                               __nv_bfloat16* __restrict__ res, int H, int group, int blk) {
  const int t = blockIdx.x;
  const int j0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (j0 >= H) return;
  const int groups = H / group;
  const bool prev = (t % blk) != 0;
  const __nv_bfloat16* c = coef + (size_t)t * ldc;
  const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)t * H + j0);
  const uint4 pv = prev ? *reinterpret_cast<const uint4*>(x + (size_t)(t - 1) * H + j0) : make_uint4(0, 0, 0, 0);
  const uint4 b0 = *reinterpret_cast<const uint4*>(base + j0), b1 = *reinterpret_cast<const uint4*>(base + H + j0);
  const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w}, pu[4] = {pv.x, pv.y, pv.z, pv.w};
  const uint32_t b0u[4] = {b0.x, b0.y, b0.z, b0.w}, b1u[4] = {b1.x, b1.y, b1.z, b1.w};
  float y[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int g = (j0 + e) / group;
    const float xe = (e & 1) ? bf_hi(xu[e >> 1]) : bf_lo(xu[e >> 1]);
    const float pe = (e & 1) ? bf_hi(pu[e >> 1]) : bf_lo(pu[e >> 1]);
    const float w0 = ((e & 1) ? bf_hi(b0u[e >> 1]) : bf_lo(b0u[e >> 1])) + bf2f(c[g]);
    float v = w0 * xe;
    if (prev) v = fmaf(((e & 1) ? bf_hi(b1u[e >> 1]) : bf_lo(b1u[e >> 1])) + bf2f(c[groups + g]), pe, v);
    y[e] = v;
  }
  __nv_bfloat16* dst = res ? res + (size_t)t * H + j0 : out + (size_t)t * H + j0;
  if (res) {
    const uint4 rv = *reinterpret_cast<const uint4*>(dst);
    const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = bf2f(f2bf(y[e])) + ((e & 1) ? bf_hi(ru[e >> 1]) : bf_lo(ru[e >> 1]));
  }
  *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf2(y[0], y[1]), pack_bf2(y[2], y[3]), pack_bf2(y[4], y[5]), pack_bf2(y[6], y[7]));
}

// Merge W ranks' per-row top-16 lists (vals / ids [W][rows][16], ids already global) into one descending top-16 per
// row, ties to the lower id. One warp per row: every lane holds up to four of the W * 16 candidates (W <= 8), sixteen
// rounds of a warp-wide arg-max. Counterpart of `fe_df_topk_pack` + `fe_df_topk_merge`
// (`kernels/k-dflash/src/lib.rs:571,582`: two ranks, one lane merging), for up to eight ranks.
__global__ void topk16_merge_kernel(float* __restrict__ ovals, int* __restrict__ oids, const float* __restrict__ vals,
                                    const int* __restrict__ ids, int rows, int W) {
  const int r = blockIdx.x, lane = threadIdx.x;
  float v[4];
  int id[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int cidx = lane + 32 * k;                          // candidate = (rank, position)
    const bool ok = cidx < W * 16;
    const size_t src = ((size_t)(cidx / 16) * rows + r) * 16 + cidx % 16;
    v[k] = ok ? vals[src] : -INFINITY;
    id[k] = ok ? ids[src] : 0x7fffffff;
  }
  for (int n = 0; n < 16; ++n) {
    float bv = v[0];
    int bi = id[0], bk = 0;
#pragma unroll
    for (int k = 1; k < 4; ++k)
      if (v[k] > bv || (v[k] == bv && id[k] < bi)) { bv = v[k]; bi = id[k]; bk = k; }
    float wv = bv;
    int wi = bi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, wv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, wi, off);
      if (ov > wv || (ov == wv && oi < wi)) { wv = ov; wi = oi; }
    }
    if (lane == 0) { ovals[(size_t)r * 16 + n] = wv; oids[(size_t)r * 16 + n] = wi; }
    if (bv == wv && bi == wi) {                              // the winner's owner retires it (ids are distinct per row)
#pragma unroll
      for (int k = 0; k < 4; ++k) if (k == bk) { v[k] = -INFINITY; id[k] = 0x7fffffff; }
    }
  }
}

// Candidate selector walk over a drafted block: pred = anchor; for each row i
//   score[c] = vals[i][c] + sum_r A[pred][r] * gate[i][r] * B[ids[i][c]][r];  pred = ids[i][argmax_c score] -> out[i]
// with rank-R codebooks A, B [vocab][R] (bf16) and gate [rows][R]. One CTA, warp c scores candidate c. The rows are a
// chain (each row's winner is the next row's predecessor), so the kernel walks them in order.
// Counterpart of `fe_df_select` (`kernels/k-dflash/src/lib.rs:613`), with run-time rank (a multiple of 256).
__global__ void __launch_bounds__(512) select_kernel(int* __restrict__ out, const float* __restrict__ vals,
                                                      const int* __restrict__ ids, const __nv_bfloat16* __restrict__ gate,
                                                      const __nv_bfloat16* __restrict__ a_cb,
                                                      const __nv_bfloat16* __restrict__ b_cb, int anchor, int rows, int R) {
  __shared__ float sc[16];
  __shared__ int pred_s;
  const int c = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) pred_s = anchor;
  __syncthreads();
  for (int i = 0; i < rows; ++i) {
    const int pred = pred_s;
    const int cand = ids[(size_t)i * 16 + c];
    float s = 0.f;
    for (int r0 = lane * 8; r0 < R; r0 += 256) {
      const uint4 av = *reinterpret_cast<const uint4*>(a_cb + (size_t)pred * R + r0);
      const uint4 bv = *reinterpret_cast<const uint4*>(b_cb + (size_t)cand * R + r0);
      const uint4 gv = *reinterpret_cast<const uint4*>(gate + (size_t)i * R + r0);
      const uint32_t au[4] = {av.x, av.y, av.z, av.w}, bu[4] = {bv.x, bv.y, bv.z, bv.w}, gu[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        s = fmaf(bf_lo(au[q]) * bf_lo(gu[q]), bf_lo(bu[q]), s);
        s = fmaf(bf_hi(au[q]) * bf_hi(gu[q]), bf_hi(bu[q]), s);
      }
    }
    s = warp_sum(s);
    if (lane == 0) sc[c] = vals[(size_t)i * 16 + c] + s;
    __syncthreads();
    if (threadIdx.x == 0) {
      int best = 0;
      for (int k = 1; k < 16; ++k) if (sc[k] > sc[best]) best = k;
      const int id = ids[(size_t)i * 16 + best];
      out[i] = id;
      pred_s = id;
    }
    __syncthreads();
  }
}

}  // namespace fb

extern "C" int fb_dynconv(void* out, const void* x, const void* coef, long ldc, const void* base, void* res, int rows, int H,
                          int group, int blk, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8 || group <= 0 || H % group || blk <= 0 || !(group % 8 == 0 || 8 % group == 0)) return -1;
  const int threads = 256;
  dim3 grid(rows, (H / 8 + threads - 1) / threads);
  fb::dynconv_kernel<<<grid, threads, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)coef, ldc,
                                             (const __nv_bfloat16*)base, (__nv_bfloat16*)res, H, group, blk);
  return (int)cudaGetLastError();
}

extern "C" int fb_topk16_merge(float* ovals, int* oids, const float* vals, const int* ids, int rows, int W, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (W < 1 || W > 8) return -1;
  fb::topk16_merge_kernel<<<rows, 32, 0, s>>>(ovals, oids, vals, ids, rows, W);
  return (int)cudaGetLastError();
}

extern "C" int fb_draft_select(int* out, const float* vals, const int* ids, const void* gate, const void* a_cb,
                               const void* b_cb, int anchor, int rows, int R, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (R <= 0 || R % 256) return -1;
  fb::select_kernel<<<1, 512, 0, s>>>(out, vals, ids, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)a_cb,
                                      (const __nv_bfloat16*)b_cb, anchor, rows, R);
  return (int)cudaGetLastError();
}
