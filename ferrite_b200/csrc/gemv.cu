// bf16 GEMV for 1..8 activation rows with fused prologue (RMSNorm) and epilogue (residual add, SwiGLU).
// Replaces `fe_gemv_bf16`, `fe_gemv_bf16_kw` (`kernels/k-core/src/gemm.rs:149-194`) and, with its fused forms,
// the separate `fe_rmsnorm` / `fe_silu_mul` / `fe_add_bf16` launches around them on the decode path.
//
// Launched with programmatic stream serialization: the grid may become resident while the previous kernel of
// the stream drains; it issues its first batch of weight loads (weights never depend on the previous kernel)
// and only then executes griddepcontrol.wait before touching X. The reference overlaps the same way
// ("L2 prefetch before griddepcontrol.wait", `crates/fe-exl3/src/gpu/pdl.rs`).
#include "api.h"
#include "gemv_core.cuh"

namespace fb {

template <int M, int R, bool SWIGLU>
__global__ void __launch_bounds__(GEMV_THREADS, (M <= 2 ? 4 : (M <= 4 ? 3 : 2))) gemv_kernel(GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __shared__ float scratch[32];
  __shared__ float rscale[M];
  const int row_end = min(a.N, (int)(blockIdx.x + 1) * a.rows_per_cta);
  gemv_main<M, R, SWIGLU>(a, xs, rscale, scratch, [&](float (&acc)[R][M], int n) {
    if ((threadIdx.x & 31) != 0) return;
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
  });
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
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GEMV_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, a);
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
