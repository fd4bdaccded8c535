// bf16 GEMV for 1..8 activation rows with fused prologue (RMSNorm) and epilogue (residual add, SwiGLU).
// Replaces `fe_gemv_bf16`, `fe_gemv_bf16_kw` (`kernels/k-core/src/gemm.rs:149-194`) and, with its fused forms,
// the separate `fe_rmsnorm` / `fe_silu_mul` / `fe_add_bf16` launches around them on the decode path.
#include "api.h"
#include "gemv_core.cuh"

namespace fb {

template <int M, int R, bool SWIGLU>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __shared__ float scratch[32];
  __shared__ float rscale[M];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (a.norm_w) gemv_row_scales<M>(a, rscale, scratch);

  const int row0 = blockIdx.x * a.rows_per_cta;
  const int row_end = min(a.N, row0 + a.rows_per_cta);
  const int nchunks = (a.K + a.kc - 1) / a.kc;
  constexpr int RW = SWIGLU ? 1 : R;     // output rows a warp produces per pass

  if (nchunks == 1) {
    gemv_stage_x<M>(a, xs, rscale, 0, a.kc);
    __syncthreads();
    for (int n = row0 + warp * RW; n < row_end; n += GEMV_WARPS * RW) {
      float acc[R][M];
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
      const __nv_bfloat16* wrow[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        int rr = SWIGLU ? (n + r * a.N) : min(n + r, a.N - 1);
        wrow[r] = a.W + (size_t)rr * a.K;
      }
      gemv_accumulate<M, R>(acc, wrow, xs, a.kc, a.K);
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          if (m >= a.M) break;
          if (SWIGLU) {
            float v = siluf_(acc[0][m]) * acc[R - 1][m];
            reinterpret_cast<__nv_bfloat16*>(a.Y)[(size_t)m * a.ldy + n] = f2bf(v);
          } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              int nn = n + r;
              if (nn >= row_end) break;
              float v = acc[r][m];
              if (a.res) v += bf2f(a.res[(size_t)m * a.ldy + nn]);
              if (a.out_f32) reinterpret_cast<float*>(a.Y)[(size_t)m * a.ldy + nn] = v;
              else reinterpret_cast<__nv_bfloat16*>(a.Y)[(size_t)m * a.ldy + nn] = f2bf(v);
            }
          }
        }
      }
    }
  } else {
    // K does not fit one staged chunk: one row group per warp, chunks in the outer loop
    int n = row0 + warp * RW;
    bool active = n < row_end;
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
    for (int c = 0; c < nchunks; ++c) {
      int k0 = c * a.kc;
      __syncthreads();
      gemv_stage_x<M>(a, xs, rscale, k0, a.kc);
      __syncthreads();
      if (active) {
        const __nv_bfloat16* wrow[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          int rr = SWIGLU ? (n + r * a.N) : min(n + r, a.N - 1);
          wrow[r] = a.W + (size_t)rr * a.K + k0;
        }
        gemv_accumulate<M, R>(acc, wrow, xs, a.kc, a.K - k0);
      }
    }
    if (active) {
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          if (m >= a.M) break;
          if (SWIGLU) {
            float v = siluf_(acc[0][m]) * acc[R - 1][m];
            reinterpret_cast<__nv_bfloat16*>(a.Y)[(size_t)m * a.ldy + n] = f2bf(v);
          } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              int nn = n + r;
              if (nn >= row_end) break;
              float v = acc[r][m];
              if (a.res) v += bf2f(a.res[(size_t)m * a.ldy + nn]);
              if (a.out_f32) reinterpret_cast<float*>(a.Y)[(size_t)m * a.ldy + nn] = v;
              else reinterpret_cast<__nv_bfloat16*>(a.Y)[(size_t)m * a.ldy + nn] = f2bf(v);
            }
          }
        }
      }
    }
  }
}

template <int M, int R, bool SWIGLU>
static int launch_gemv(GemvArgs a, int sm_count, cudaStream_t s) {
  a.kc = gemv_chunk_len(M, a.K);
  int nchunks = (a.K + a.kc - 1) / a.kc;
  constexpr int RW = SWIGLU ? 1 : R;
  int group = GEMV_WARPS * RW;
  if (nchunks > 1) {
    a.rows_per_cta = group;
  } else {
    int target = sm_count * 4;
    int rpc = (a.N + target - 1) / target;
    a.rows_per_cta = (rpc + group - 1) / group * group;
  }
  int grid = (a.N + a.rows_per_cta - 1) / a.rows_per_cta;
  size_t smem = (size_t)M * a.kc * sizeof(__nv_bfloat16);
  auto kern = gemv_kernel<M, R, SWIGLU>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  kern<<<grid, GEMV_THREADS, smem, s>>>(a);
  return (int)cudaGetLastError();
}

}  // namespace fb

using namespace fb;

// mode: 0 = plain (optional residual), 1 = SwiGLU (W has 2N rows: gate rows then up rows)
extern "C" int fb_gemv_bf16(void* Y, const void* X, const void* W, const void* norm_w, const void* res, int M, int N,
                            int K, long ldx, long ldy, float eps, int centred, int out_f32, int mode, int sm_count,
                            cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 8 || (K % 8) != 0 || (ldx % 8) != 0) return -1;
  GemvArgs a;
  a.X = (const __nv_bfloat16*)X; a.W = (const __nv_bfloat16*)W; a.norm_w = (const __nv_bfloat16*)norm_w;
  a.res = (const __nv_bfloat16*)res; a.Y = Y; a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.eps = eps;
  a.centred = centred; a.out_f32 = out_f32; a.rows_per_cta = 0; a.kc = 0;
  if (sm_count <= 0) sm_count = 148;
  if (mode == 1) {
    if (M == 1) return launch_gemv<1, 2, true>(a, sm_count, s);
    if (M == 2) return launch_gemv<2, 2, true>(a, sm_count, s);
    if (M <= 4) return launch_gemv<4, 2, true>(a, sm_count, s);
    return launch_gemv<8, 2, true>(a, sm_count, s);
  }
  if (M == 1) return launch_gemv<1, 2, false>(a, sm_count, s);
  if (M == 2) return launch_gemv<2, 2, false>(a, sm_count, s);
  if (M <= 4) return launch_gemv<4, 2, false>(a, sm_count, s);
  return launch_gemv<8, 2, false>(a, sm_count, s);
}
