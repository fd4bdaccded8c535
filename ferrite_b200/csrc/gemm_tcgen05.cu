// Single-GPU entry points of the tcgen05 bf16 GEMM (kernel and planning in gemm_core.cuh).
#include "gemm_core.cuh"

using namespace fb;

extern "C" long fb_gemm_workspace_bytes(int M, int N, int split_k) {
  if (M > 64 || split_k <= 1) return 0;
  int bn = ((M + 15) / 16) * 16;
  long tiles = (N + GM_BM - 1) / GM_BM;
  return tiles * split_k * 2L * bn * GM_BM * (long)sizeof(float);
}

extern "C" int fb_gemm_bf16(void* Y, const void* X, const void* W, const void* res, int M, int N, int K, long ldx,
                            long ldy, int mode, int split_k, float* workspace, int* counters, int* status,
                            int sm_count, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 || ldx % 8 || (ldy % 8 && M > 64)) return -1;
  if (sm_count <= 0) sm_count = 148;
  GemmPlan p{};
  int rc = plan_gemm(p, M, N, K, mode, split_k, sm_count);
  if (rc) return rc;
  GemmArgs& a = p.a;
  if (a.split_k > 1 && (!workspace || !counters)) return -6;
  a.Y = Y; a.res = (const __nv_bfloat16*)res; a.workspace = workspace; a.counters = counters; a.status = status;
  a.ldy = ldy;
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
