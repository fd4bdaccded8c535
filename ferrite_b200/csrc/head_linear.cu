// One small linear per attention head over a few rows: y[t][h][0..N) = W[h] (N x K) . x[t][h][0..K), t < T <= 8 per
// row tile (grid.z covers more). Multi-head latent attention needs two of these per layer and step: the key
// up-projection folded into the query (N = latent width, K = head width) and the value up-projection after the
// attention (N = value width, K = latent width). One launch streams the whole [heads][N][K] stack once; the reference
// issues its per-head products from the attention kernels' prologue / epilogue (`kernels/k-ds/src/attn.rs:151-548`).
//
// CTA = (64 outputs, one head, one tile of ROWS rows), 8 warps x 8 outputs, no shared memory. A group of LPO =
// min(32, K / 8) lanes owns an output and reads its weight row with 16-byte loads (CPL = K / 8 / LPO of them per lane).
// A lane meets the same K chunks in every output, so it keeps its slice of the x rows in registers (packed bf16) for the
// whole CTA. A warp works on U outputs per lane group at a time and issues all their weight loads before it uses any.
// Sums go over the lanes of a group in a fixed xor tree: a row's bits do not depend on the other rows of the step.
#include "common.cuh"

namespace fb {

constexpr int HL_OUT = 64;
constexpr int HL_MAX_K = 1024;

template <int CPL, int ROWS, int HL_U>
__global__ void __launch_bounds__(256, 2) head_linear_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ W, int T, int N, int K,
                                                          long x_rs, long x_hs, long y_rs, long y_hs) {
  const int h = blockIdx.y, t0 = blockIdx.z * ROWS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = K / 8;
  const int lpo = chunks < 32 ? chunks : 32;          // lanes per output: a power of two
  const int per_pass = 32 / lpo;                      // outputs a warp covers in one pass
  const int passes = (HL_OUT / 8) / per_pass > 0 ? (HL_OUT / 8) / per_pass : 1;
  const int sub = lane / lpo, l = lane % lpo;
  const int n_base = blockIdx.x * HL_OUT + warp * (HL_OUT / 8);
  const __nv_bfloat16* Wh = W + (size_t)h * N * K;
  uint4 raw[HL_U][CPL];
  auto out_of = [&](int pass) { return n_base + pass * per_pass + sub; };
  auto live = [&](int pass) { return pass < passes && pass * per_pass + sub < HL_OUT / 8 && out_of(pass) < N; };
  auto load_batch = [&](int p0) {
#pragma unroll
    for (int u = 0; u < HL_U; ++u) {
      const bool ok = live(p0 + u);
#pragma unroll
      for (int c = 0; c < CPL; ++c)
        raw[u][c] = ok ? ldg_stream(reinterpret_cast<const uint4*>(Wh + (size_t)out_of(p0 + u) * K) + l + c * lpo)
                       : make_uint4(0, 0, 0, 0);
    }
  };
  load_batch(0);
  // this lane's K chunks of the x rows: as floats while they fit the register budget (no unpacking per output), else
  // packed bf16
  constexpr bool XF = ROWS * CPL <= 8;
  uint4 xr[XF ? 1 : ROWS][XF ? 1 : CPL];
  float xf[XF ? ROWS : 1][XF ? CPL : 1][8];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const uint4 v = t0 + r < T ? *reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * x_rs + (size_t)h * x_hs + (l + c * lpo) * 8)
                                 : make_uint4(0, 0, 0, 0);
      if constexpr (XF) {
        const uint32_t v4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { xf[r][c][2 * j] = bf_lo(v4[j]); xf[r][c][2 * j + 1] = bf_hi(v4[j]); }
      } else {
        xr[r][c] = v;
      }
    }
  }
  for (int p0 = 0; p0 < passes; p0 += HL_U) {          // the same trip count for every lane: shuffles below
    if (p0 > 0) load_batch(p0);
#pragma unroll
    for (int u = 0; u < HL_U; ++u) {
      float acc[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const uint32_t w4[4] = {raw[u][c].x, raw[u][c].y, raw[u][c].z, raw[u][c].w};
        float wv[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { wv[2 * j] = bf_lo(w4[j]); wv[2 * j + 1] = bf_hi(w4[j]); }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          float s = acc[r];
          if constexpr (XF) {
#pragma unroll
            for (int j = 0; j < 8; ++j) s = fmaf(wv[j], xf[r][c][j], s);
          } else {
            const uint32_t x4[4] = {xr[r][c].x, xr[r][c].y, xr[r][c].z, xr[r][c].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { s = fmaf(wv[2 * j], bf_lo(x4[j]), s); s = fmaf(wv[2 * j + 1], bf_hi(x4[j]), s); }
          }
          acc[r] = s;
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
        for (int off = lpo >> 1; off > 0; off >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
      if (l == 0 && live(p0 + u)) {
        const int n = out_of(p0 + u);
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
          if (t0 + r < T) y[(size_t)(t0 + r) * y_rs + (size_t)h * y_hs + n] = __float2bfloat16(acc[r]);
      }
    }
  }
}

}  // namespace fb

using namespace fb;

// x: rows of stride x_rs elements, head h at offset h * x_hs (16-byte aligned); y likewise (any element alignment).
// T > 8 runs as row tiles of 8 (grid.z).
extern "C" int fb_head_linear(void* y, const void* x, const void* W, int T, int heads, int N, int K, long x_rs, long x_hs,
                              long y_rs, long y_hs, cudaStream_t s) {
  if (T <= 0 || heads <= 0) return 0;
  if (K < 8 || K > HL_MAX_K || (K & (K - 1)) || x_rs % 8 || x_hs % 8 || heads > 65535) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15) return -1;
  const int rows = T >= 8 ? 8 : T > 2 ? 4 : T;        // rows per tile: 1, 2, 4 or 8
  dim3 grid((N + HL_OUT - 1) / HL_OUT, heads, (T + rows - 1) / rows);
  const int chunks = K / 8, cpl = chunks <= 32 ? 1 : chunks / 32;
#define FB_HL(C, R)                                                                                                      \
  head_linear_kernel<C, R, (C == 1 ? (R == 8 ? 2 : 4) : C == 2 ? (R == 8 ? 1 : 2) : 1)><<<grid, 256, 0, s>>>(                \
      (__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const __nv_bfloat16*)W, T, N, K, x_rs, x_hs, y_rs, y_hs)
#define FB_HL_R(C)                                                                                                       \
  { if (rows == 1) FB_HL(C, 1); else if (rows == 2) FB_HL(C, 2); else if (rows == 4) FB_HL(C, 4); else FB_HL(C, 8); }
  if (cpl == 1) FB_HL_R(1) else if (cpl == 2) FB_HL_R(2) else if (cpl == 4) FB_HL_R(4) else return -1;
#undef FB_HL_R
#undef FB_HL
  return (int)cudaGetLastError();
}
