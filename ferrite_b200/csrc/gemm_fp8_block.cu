// Block-scaled FP8 GEMM: e4m3 activations with one fp32 scale per (row, 128 k) and e4m3 weights with one fp32 scale
// per (128 output features, 128 k) block, y[m][n] = sum_kb sx[m][kb] * sw[n/128][kb] * (xq[m][kb] . wq[n][kb]).
//
// The scales change along k, so the tensor core cannot accumulate the whole reduction in one TMEM tile. One CTA owns a
// 128 x 128 output tile; per k block of 128 (128 bytes of e4m3 = one swizzled row) the MMA warp issues four
// tcgen05.mma kind::f8f6f4 (K = 32 each) into one of two TMEM buffers, and the four epilogue warps read that buffer,
// multiply by the block's scale pair and add it into fp32 registers ("promotion") while the tensor pipe already works
// on the next k block in the other buffer. Operand tiles arrive through a four-stage TMA ring.
//
// Warp roles: warp 0 lane 0 TMA, warp 1 lane 0 MMA, warps 2..5 promotion + store (one output row per thread).
// Every wait is bounded; a wait that runs out sets the status word and an abort flag, all roles leave, TMEM is freed.
//
// Counterpart of the reference's FP8 prompt linear (`crates/fe-fp4/src/lib.rs`, `FE_FP8_KERNEL`), in the block-scaled
// form that 671B-class MLA MoE checkpoints ship (128 x 128 weight blocks, 1 x 128 activation blocks).
#include <cuda_fp8.h>

#include "api.h"
#include "common.cuh"
#include "gemm_core.cuh"

namespace fb {

constexpr int FBK_BM = 128, FBK_BN = 128, FBK_BK = 128, FBK_STAGES = 4, FBK_THREADS = 192;
constexpr int FBK_TILE = FBK_BM * FBK_BK;          // bytes of one operand tile (e4m3)

// activations -> e4m3 codes + one scale per (row, 128 columns): scale = amax / 448. One warp per (row, block).
__global__ void quant_fp8_block_kernel(unsigned char* __restrict__ q, float* __restrict__ scale,
                                       const __nv_bfloat16* __restrict__ x, int rows, int K, long ldx, int kblocks) {
  pdl_launch_dependents();
  pdl_wait();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * kblocks) return;
  const int row = w / kblocks, kb = w % kblocks;
  const int c0 = kb * FBK_BK + lane * 4;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = (c0 + j < K) ? bf2f(x[(size_t)row * ldx + c0 + j]) : 0.f;
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float sc = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / sc;
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    packed |= (uint32_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
  // the code matrix is padded to whole k blocks (kblocks * 128 columns), so the store never needs a tail case
  *reinterpret_cast<uint32_t*>(q + (size_t)row * kblocks * FBK_BK + c0) = packed;
  if (lane == 0) scale[(size_t)row * kblocks + kb] = sc;
}

__global__ void __launch_bounds__(FBK_THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                      __nv_bfloat16* __restrict__ Y, const float* __restrict__ sx, const float* __restrict__ sw,
                      const __nv_bfloat16* __restrict__ res, int M, int N, int kblocks, long ldy, int* status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[FBK_STAGES], empty_bar[FBK_STAGES], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tm = blockIdx.x, tn = blockIdx.y;          // row tiles vary fastest: CTAs running together share weight tiles
  volatile int* abort_flag = &abort_s;
  pdl_launch_dependents();
  pdl_wait();

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int i = 0; i < FBK_STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 128); }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 2 * FBK_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX); tma_prefetch_desc(&tmW);
      int armed = 0;
      bool ok = true;
      for (int kb = 0; kb < kblocks; ++kb) {
        const int st = kb % FBK_STAGES;
        if (kb >= FBK_STAGES && !mbar_wait_or_flag(&empty_bar[st], ((kb / FBK_STAGES) - 1) & 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&full_bar[st], 2 * FBK_TILE);
        tma_load_2d(tiles + st * 2 * FBK_TILE, &tmX, &full_bar[st], kb * FBK_BK, tm * FBK_BM);
        tma_load_2d(tiles + st * 2 * FBK_TILE + FBK_TILE, &tmW, &full_bar[st], kb * FBK_BK, tn * FBK_BN);
        armed = kb + 1;
      }
      if (!ok) { set_status(status, ST_MBAR_TIMEOUT); abort_s = 1; }
      if (*abort_flag)      // loads of this thread may still be landing: bounded wait before the CTA's memory goes away
        for (int kb = max(0, armed - FBK_STAGES); kb < armed; ++kb)
          mbar_wait(&full_bar[kb % FBK_STAGES], (kb / FBK_STAGES) & 1, 1u << 20);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(0, 0, FBK_BM, FBK_BN);      // e4m3 x e4m3 -> fp32
      const uint32_t base = smem_u32(tiles);
      bool ok = true;
      for (int kb = 0; kb < kblocks; ++kb) {
        const int st = kb % FBK_STAGES, buf = kb & 1;
        if (!mbar_wait_or_flag(&full_bar[st], (kb / FBK_STAGES) & 1, abort_flag)) { ok = false; break; }
        if (kb >= 2 && !mbar_wait_or_flag(&tempty_bar[buf], ((kb >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a = base + st * 2 * FBK_TILE, b = a + FBK_TILE;
#pragma unroll
        for (int kk = 0; kk < FBK_BK / 32; ++kk)
          tc_mma_f8f6f4(tmem + buf * FBK_BN, umma_desc_k128(a + kk * 32), umma_desc_k128(b + kk * 32), idesc, kk > 0 ? 1u : 0u);
        tc_commit(&empty_bar[st]);
        tc_commit(&tfull_bar[buf]);
      }
      if (!ok) { set_status(status, ST_MBAR_TIMEOUT); abort_s = 1; }
    }
  } else {
    // ---- promotion: acc += scale(kb) * partial(kb), then the store ---------------------------------------------------
    const int quad = warp & 3;
    const int row = tm * FBK_BM + quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const bool row_ok = row < M;
    float acc[FBK_BN];
#pragma unroll
    for (int c = 0; c < FBK_BN; ++c) acc[c] = 0.f;
    bool ok = true;
    for (int kb = 0; kb < kblocks; ++kb) {
      const int buf = kb & 1;
      const float sc = (row_ok ? sx[(size_t)row * kblocks + kb] : 0.f) * sw[(size_t)tn * kblocks + kb];
      ok = __all_sync(0xffffffffu, mbar_wait_or_flag(&tfull_bar[buf], (kb >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < FBK_BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem + lane_addr + buf * FBK_BN + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) acc[c0 + c] = fmaf(__uint_as_float(v[c]), sc, acc[c0 + c]);
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[buf]);
    }
    if (!ok) {
      if (lane == 0) { set_status(status, ST_MBAR_TIMEOUT); abort_s = 1; }
    } else if (row_ok) {
      const int n0 = tn * FBK_BN;
      __nv_bfloat16* dst = Y + (size_t)row * ldy + n0;
      const __nv_bfloat16* rs = res ? res + (size_t)row * ldy + n0 : nullptr;
      if (n0 + FBK_BN <= N && (ldy % 8) == 0) {
#pragma unroll
        for (int c0 = 0; c0 < FBK_BN; c0 += 8) {
          uint32_t w[4];
          uint4 r4 = make_uint4(0, 0, 0, 0);
          if (rs) r4 = *reinterpret_cast<const uint4*>(rs + c0);
          const uint32_t ru[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a = acc[c0 + 2 * e], b = acc[c0 + 2 * e + 1];
            if (rs) { a += bf_lo(ru[e]); b += bf_hi(ru[e]); }
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            w[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst + c0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < FBK_BN; ++c)
          if (n0 + c < N) dst[c] = f2bf(acc[c] + (rs ? bf2f(rs[c]) : 0.f));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 2 * FBK_BN);
}

}  // namespace fb

using namespace fb;

extern "C" long fb_fp8_block_kblocks(int K) { return (K + FBK_BK - 1) / FBK_BK; }

// q: [rows][kblocks*128] e4m3 codes (columns past K are zero), scale: [rows][kblocks]
extern "C" int fb_quant_fp8_block(void* q, float* scale, const void* x, int rows, int K, long ldx, cudaStream_t s) {
  if (rows <= 0) return 0;
  const int kblocks = (K + FBK_BK - 1) / FBK_BK;
  const long warps = (long)rows * kblocks;
  launch_pdl(quant_fp8_block_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), (size_t)0, s, (unsigned char*)q,
             scale, (const __nv_bfloat16*)x, rows, K, ldx, kblocks);
  return (int)cudaGetLastError();
}

// Xq [M][kblocks*128], sx [M][kblocks]; Wq [N][kblocks*128], sw [ceil(N/128)][kblocks]; Y (and res) bf16 [M][ldy]
extern "C" int fb_gemm_fp8_block(void* Y, const void* Xq, const float* sx, const void* Wq, const float* sw, const void* res,
                                 int M, int N, int K, long ldy, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  const int kblocks = (K + FBK_BK - 1) / FBK_BK;
  const uint64_t kp = (uint64_t)kblocks * FBK_BK;
  CUtensorMap tmX, tmW;
  int rc;
  if ((rc = make_tmap_u8_2d(&tmX, Xq, (uint64_t)M, kp, kp, FBK_BM))) return rc;
  if ((rc = make_tmap_u8_2d(&tmW, Wq, (uint64_t)N, kp, kp, FBK_BN))) return rc;
  const size_t smem = (size_t)FBK_STAGES * 2 * FBK_TILE + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((M + FBK_BM - 1) / FBK_BM, (N + FBK_BN - 1) / FBK_BN);
  launch_pdl(gemm_fp8_block_kernel, grid, dim3(FBK_THREADS), smem, s, tmX, tmW, (__nv_bfloat16*)Y, sx, sw,
             (const __nv_bfloat16*)res, M, N, kblocks, ldy, status);
  return (int)cudaGetLastError();
}
