// Single-GPU entry points of the tcgen05 bf16 GEMM (kernel and planning in gemm_core.cuh).
#include "gemm_core.cuh"

using namespace fb;

extern "C" long fb_gemm_workspace_bytes(int M, int N, int split_k) {
  if (M > 64 || split_k <= 1) return 0;
  int bn = ((M + 15) / 16) * 16;
  long tiles = (N + GM_BM - 1) / GM_BM;
  return tiles * split_k * 2L * bn * GM_BM * (long)sizeof(float);
}

// mode bit 0: SwiGLU over gate|up rows; bit 1: Y is fp32 (residual stays bf16 with the same leading dimension)
extern "C" int fb_gemm_bf16(void* Y, const void* X, const void* W, const void* res, int M, int N, int K, long ldx,
                            long ldy, int mode, int split_k, float* workspace, int* counters, int* status,
                            int sm_count, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  const int out_f32 = (mode >> 1) & 1;
  mode &= 1;
  if (K % 8 || ldx % 8 || (ldy % 8 && M > 64)) return -1;
  if (sm_count <= 0) sm_count = 148;
  GemmPlan p{};
  int rc = plan_gemm(p, M, N, K, mode, split_k, sm_count);
  if (rc) return rc;
  GemmArgs& a = p.a;
  if (a.split_k > 1 && (!workspace || !counters)) return -6;
  a.Y = Y; a.res = (const __nv_bfloat16*)res; a.workspace = workspace; a.counters = counters; a.status = status;
  a.ldy = ldy; a.out_f32 = out_f32;
  const int w_rows = a.dual ? 2 * N : N;
  CUtensorMap tmA, tmB;
  if (a.swap) {
    rc = make_tmap_bf16_2d(&tmA, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, GM_BM);
    if (rc) return rc;
    rc = make_tmap_bf16_2d(&tmB, X, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, (uint32_t)a.b_box_rows);
  } else {
    rc = make_tmap_bf16_2d(&tmA, X, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, GM_BM);
    if (rc) return rc;
    rc = make_tmap_bf16_2d(&tmB, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, (uint32_t)a.b_box_rows);
  }
  if (rc) return rc;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  gemm_bf16_tc_kernel<0><<<p.grid, GM_THREADS, p.smem, s>>>(tmA, tmB, a);
  return (int)cudaGetLastError();
}

// ---- FP8 (e4m3) operands ----------------------------------------------------------------------------------
// Y[M][N] (bf16) = (Xq[M][K] Wq[N][K]^T) * scale_m[m] * scale_n[n] (+ res, or SwiGLU over gate|up features), Xq / Wq
// e4m3 bytes, fp32 accumulation in TMEM. Per-row activation scales and per-feature weight scales; the reference's
// per-tensor variant is the case of constant vectors (`fe_gemm_fp8`, `kernels/k-fp4/src/fp8.rs`). The 128x128 /
// 1x128 block-scaled form is not built: it needs the partial sums of every 128-wide k block rescaled before they
// are added, which this accumulate-in-TMEM pipeline does not do.
#include <cuda_fp8.h>

namespace fb {

// one warp per row: amax -> scale = amax / 448, codes = e4m3(x / scale); optional RMSNorm(1 + w) first
__global__ void quant_fp8_kernel(unsigned char* __restrict__ q, float* __restrict__ scale, const __nv_bfloat16* __restrict__ x,
                                 const __nv_bfloat16* __restrict__ norm_w, int rows, int K, long ldx, float eps) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  float ss = 0.f, amax = 0.f;
  for (int k = lane; k < K; k += 32) { const float v = bf2f(xr[k]); ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float r = norm_w ? rsqrtf(ss / (float)K + eps) : 1.f;
  for (int k = lane; k < K; k += 32) {
    float v = bf2f(xr[k]) * r;
    if (norm_w) v *= 1.f + bf2f(norm_w[k]);
    amax = fmaxf(amax, fabsf(v));
  }
  amax = warp_max(amax);
  const float sc = amax > 0.f ? amax / 448.f : 1.f, inv = 1.f / sc;
  for (int k = lane; k < K; k += 32) {
    float v = bf2f(xr[k]) * r;
    if (norm_w) v *= 1.f + bf2f(norm_w[k]);
    q[(size_t)row * K + k] = (unsigned char)__nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, __NV_E4M3);
  }
  if (lane == 0) scale[row] = sc;
}

}  // namespace fb

extern "C" int fb_quant_fp8(void* q, float* scale, const void* x, const void* norm_w, int rows, int K, long ldx, float eps,
                            cudaStream_t s) {
  if (rows <= 0) return 0;
  quant_fp8_kernel<<<(rows * 32 + 255) / 256, 256, 0, s>>>((unsigned char*)q, scale, (const __nv_bfloat16*)x,
                                                           (const __nv_bfloat16*)norm_w, rows, K, ldx, eps);
  return (int)cudaGetLastError();
}

extern "C" int fb_gemm_fp8(void* Y, const void* Xq, const void* Wq, const float* scale_m, const float* scale_n,
                           const void* res, int M, int N, int K, long ldy, int mode, int split_k, float* workspace,
                           int* counters, int* status, int sm_count, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 16 || (ldy % 8 && M > 64)) return -1;
  if (sm_count <= 0) sm_count = 148;
  GemmPlan p{};
  int rc = plan_gemm(p, M, N, K, mode, split_k, sm_count, 1);
  if (rc) return rc;
  GemmArgs& a = p.a;
  if (a.split_k > 1 && (!workspace || !counters)) return -6;
  a.Y = Y; a.res = (const __nv_bfloat16*)res; a.workspace = workspace; a.counters = counters; a.status = status;
  a.ldy = ldy; a.scale_m = scale_m; a.scale_n = scale_n;
  const int w_rows = a.dual ? 2 * N : N;
  CUtensorMap tmA, tmB;
  if (a.swap) {
    rc = make_tmap_u8_2d(&tmA, Wq, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, GM_BM);
    if (rc) return rc;
    rc = make_tmap_u8_2d(&tmB, Xq, (uint64_t)M, (uint64_t)K, (uint64_t)K, (uint32_t)a.b_box_rows);
  } else {
    rc = make_tmap_u8_2d(&tmA, Xq, (uint64_t)M, (uint64_t)K, (uint64_t)K, GM_BM);
    if (rc) return rc;
    rc = make_tmap_u8_2d(&tmB, Wq, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, (uint32_t)a.b_box_rows);
  }
  if (rc) return rc;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  gemm_bf16_tc_kernel<0><<<p.grid, GM_THREADS, p.smem, s>>>(tmA, tmB, a);
  return (int)cudaGetLastError();
}
