// One small linear per attention head over a few rows: y[t][h][0..N) = W[h] (N x K) . x[t][h][0..K), t < T <= 8 per
// row tile (grid.z covers more). Multi-head latent attention needs two of these per layer and step: the key
// up-projection folded into the query (N = latent width, K = head width) and the value up-projection after the
// attention (N = value width, K = latent width). One launch streams the whole [heads][N][K] stack once; the reference
// issues its per-head products from the attention kernels' prologue / epilogue (`kernels/k-ds/src/attn.rs:151-548`).
//
// CTA = (32 outputs, one head, one tile of 8 rows), 8 warps. The head's x rows sit in shared memory as fp32; a group of
// LPO = min(32, K / 8) lanes owns one output at a time and reads its weight row with 16-byte loads; sums go over the
// lanes of the group in a fixed xor tree, so a row's bits do not depend on the other rows of the step.
#include "common.cuh"

namespace fb {

constexpr int HL_ROWS = 8;
constexpr int HL_OUT = 32;
constexpr int HL_MAX_K = 1024;

__global__ void __launch_bounds__(256) head_linear_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ W, int T, int N, int K,
                                                          long x_rs, long x_hs, long y_rs, long y_hs) {
  __shared__ float xs[HL_ROWS][HL_MAX_K];
  const int h = blockIdx.y, t0 = blockIdx.z * HL_ROWS, n0 = blockIdx.x * HL_OUT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < HL_ROWS * (K / 8); i += blockDim.x) {
    const int r = i / (K / 8), c = i % (K / 8);
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (t0 + r < T) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * x_rs + (size_t)h * x_hs + c * 8);
      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { v[2 * j] = bf_lo(u[j]); v[2 * j + 1] = bf_hi(u[j]); }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) xs[r][c * 8 + j] = v[j];
  }
  __syncthreads();
  const int chunks = K / 8;
  const int lpo = chunks < 32 ? chunks : 32;          // lanes per output: a power of two (K is 32, 64, 128, ...)
  const int per_pass = 32 / lpo;                      // outputs a warp works on together
  const int sub = lane / lpo, l = lane % lpo;
  const __nv_bfloat16* Wh = W + (size_t)h * N * K;
  // a warp owns HL_OUT / 8 = 4 consecutive outputs
  for (int o0 = 0; o0 < HL_OUT / 8; o0 += per_pass) {       // the same trip count for every lane: shuffles below
    const int o = o0 + sub;
    const int n = n0 + warp * (HL_OUT / 8) + o;
    const bool live = o < HL_OUT / 8 && n < N;
    float acc[HL_ROWS];
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) acc[r] = 0.f;
    if (live) {
      for (int c = l; c < chunks; c += lpo) {
        const uint4 raw = ldg_stream(reinterpret_cast<const uint4*>(Wh + (size_t)n * K) + c);
        const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
        float wv[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { wv[2 * j] = bf_lo(u[j]); wv[2 * j + 1] = bf_hi(u[j]); }
#pragma unroll
        for (int r = 0; r < HL_ROWS; ++r) {
          const float4 a = *reinterpret_cast<const float4*>(&xs[r][c * 8]);
          const float4 b = *reinterpret_cast<const float4*>(&xs[r][c * 8 + 4]);
          float s = acc[r];
          s = fmaf(wv[0], a.x, s); s = fmaf(wv[1], a.y, s); s = fmaf(wv[2], a.z, s); s = fmaf(wv[3], a.w, s);
          s = fmaf(wv[4], b.x, s); s = fmaf(wv[5], b.y, s); s = fmaf(wv[6], b.z, s); s = fmaf(wv[7], b.w, s);
          acc[r] = s;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r)
      for (int off = lpo >> 1; off > 0; off >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
    if (l == 0 && live) {
#pragma unroll
      for (int r = 0; r < HL_ROWS; ++r)
        if (t0 + r < T) y[(size_t)(t0 + r) * y_rs + (size_t)h * y_hs + n] = __float2bfloat16(acc[r]);
    }
  }
}

}  // namespace fb

using namespace fb;

// x: rows of stride x_rs elements, head h at offset h * x_hs (16-byte aligned); y likewise (any element alignment).
extern "C" int fb_head_linear(void* y, const void* x, const void* W, int T, int heads, int N, int K, long x_rs, long x_hs,
                              long y_rs, long y_hs, cudaStream_t s) {
  if (T <= 0 || heads <= 0) return 0;
  if (K < 8 || K > HL_MAX_K || (K & (K - 1)) || x_rs % 8 || x_hs % 8 || heads > 65535) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15) return -1;
  dim3 grid((N + HL_OUT - 1) / HL_OUT, heads, (T + HL_ROWS - 1) / HL_ROWS);
  head_linear_kernel<<<grid, 256, 0, s>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const __nv_bfloat16*)W, T, N, K,
                                          x_rs, x_hs, y_rs, y_hs);
  return (int)cudaGetLastError();
}
