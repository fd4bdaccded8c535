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
