// Weight-streaming linear for 2..32 token rows on the warp-level tensor cores: y[m][n] = sum_k x[m][k] W[n][k].
//
// Between one row (the SIMT GEMV) and prompt-sized batches (the tcgen05 GEMM) the work is still bound by streaming the
// weights once, but there are too many FMAs per weight for the CUDA cores and too few rows to fill a 128-wide UMMA
// tile. Here every warp streams 16 weight rows straight from global memory into mma.sync m16n8k16 A fragments with
// 16-byte loads and no shared-memory round trip: a dot product does not care about the order of k, so the thread that
// the fragment layout makes owner of k pairs {2t, 2t+1} and {2t+8, 2t+9} of two consecutive k steps simply takes the
// 8 contiguous elements k0 + 8t .. 8t+7 of its row, and the activations (staged in shared memory, token-major) are read
// with the same permutation - one 16-byte shared load per 8-token tile. The 8 warps of a CTA split K and are summed in
// warp order, so results do not depend on scheduling. Epilogues: residual add, SwiGLU over gate|up rows, fp32 output;
// prologue: RMSNorm(1 + w) of the rows (scales computed in-kernel).
//
// This is the decode path for 2..8 concurrent streams and the verify path of speculative decoding (1 + 16 drafted
// rows). The tensor path is mma.sync by necessity: tcgen05 needs a 64/128-row A tile from shared memory, which is what
// the swapped orientation of gemm_core.cuh does for 33..64 rows. Replaces `exl3_gemv8*` / `fe_gemv_bf16` multi-row forms
// (`kernels/k-exl3/src`, `kernels/k-core/src/gemv.rs`).
#include "api.h"
#include "common.cuh"

namespace fb {

struct GemvMmaArgs {
  void* y;                        // bf16 or fp32 [M][ldy]
  const __nv_bfloat16* x;         // [M][ldx]
  const __nv_bfloat16* w;         // [N or 2N][K]
  const __nv_bfloat16* norm_w;    // [K] or null
  const __nv_bfloat16* res;       // [M][ldy] or null
  int M, N, K;
  long ldx, ldy;
  float eps;
  int out_f32;
};

__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int GM2_WARPS = 8;
template <int MT> struct Gm2 {                       // MT = 8-token tiles
  static constexpr int KC = MT == 1 ? 4096 : MT == 2 ? 2048 : 1024;   // k values of x staged per pass
  static constexpr int LDX = KC + 32;                // row stride: 64 bytes off a multiple of 128 -> conflict-free reads
  static constexpr size_t SMEM = (size_t)8 * MT * LDX * 2 + (size_t)GM2_WARPS * 16 * 8 * MT * 4 * 2 + 8 * MT * 4;
};

// grid = ceil(N / 16); 256 threads; DUAL: rows n (gate) and N + n (up), output silu(gate) * up
template <int MT, bool DUAL>
__global__ void __launch_bounds__(GM2_WARPS * 32, 2) gemv_mma_kernel(GemvMmaArgs a) {
  using C = Gm2<MT>;
  extern __shared__ __align__(16) unsigned char smem_g2[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_g2);                    // [8 MT][LDX]
  float* red = reinterpret_cast<float*>(smem_g2 + (size_t)8 * MT * C::LDX * 2);     // [2][warps][16][8 MT]
  float* rscale = red + 2 * GM2_WARPS * 16 * 8 * MT;                                // [8 MT]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  // weight rows of this thread's fragments (clamped: rows past N are computed and dropped)
  const int ra = min(n0 + g, a.N - 1), rb = min(n0 + g + 8, a.N - 1);
  const __nv_bfloat16* wa = a.w + (size_t)ra * a.K;
  const __nv_bfloat16* wb = a.w + (size_t)rb * a.K;
  const __nv_bfloat16* ua = DUAL ? a.w + (size_t)(a.N + ra) * a.K : nullptr;
  const __nv_bfloat16* ub = DUAL ? a.w + (size_t)(a.N + rb) * a.K : nullptr;
  pdl_wait();
  // RMSNorm scales of the token rows (one warp per row, round robin)
  if (a.norm_w) {
    for (int m = warp; m < 8 * MT; m += GM2_WARPS) {
      float ss = 0.f;
      if (m < a.M)
        for (int k = lane * 8; k < a.K; k += 256) {
          const uint4 v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + k);
          const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float lo = bf_lo(u[j]), hi = bf_hi(u[j]); ss = fmaf(lo, lo, fmaf(hi, hi, ss)); }
        }
      ss = warp_sum(ss);
      if (lane == 0) rscale[m] = rsqrtf(ss / (float)a.K + a.eps);
    }
  }
  float acc[MT][4], acu[DUAL ? MT : 1][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (DUAL) acu[i][j] = 0.f; }

  for (int kc = 0; kc < a.K; kc += C::KC) {
    const int kn = min(C::KC, a.K - kc);
    __syncthreads();                                    // previous pass is done with xs (and rscale is visible)
    for (int i = threadIdx.x; i < 8 * MT * (kn / 8); i += blockDim.x) {
      const int m = i / (kn / 8), c8 = (i % (kn / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < a.M) {
        v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + kc + c8);
        if (a.norm_w) {
          const uint4 nw = *reinterpret_cast<const uint4*>(a.norm_w + kc + c8);
          const float r = rscale[m];
          uint32_t u[4] = {v.x, v.y, v.z, v.w};
          const uint32_t wv[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            u[j] = pack_bf2(bf_lo(u[j]) * r * (1.f + bf_lo(wv[j])), bf_hi(u[j]) * r * (1.f + bf_hi(wv[j])));
          v = make_uint4(u[0], u[1], u[2], u[3]);
        }
      }
      *reinterpret_cast<uint4*>(xs + (size_t)m * C::LDX + c8) = v;
    }
    __syncthreads();
    // this warp's k range inside the pass, in steps of 32 (two mma k steps)
    const int per = ((kn / 32) + GM2_WARPS - 1) / GM2_WARPS;
    const int it0 = warp * per, it1 = min(kn / 32, it0 + per);
#pragma unroll 4
    for (int it = it0; it < it1; ++it) {
      const int kl = it * 32 + t * 8;                   // local k of this thread's 8 elements
      const uint4 A0 = ldg_stream(wa + kc + kl), A1 = ldg_stream(wb + kc + kl);
      uint4 U0, U1;
      if (DUAL) { U0 = ldg_stream(ua + kc + kl); U1 = ldg_stream(ub + kc + kl); }
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const uint4 B = *reinterpret_cast<const uint4*>(xs + (size_t)(i * 8 + g) * C::LDX + kl);
        mma_bf16_16816(acc[i], A0.x, A1.x, A0.y, A1.y, B.x, B.y);
        mma_bf16_16816(acc[i], A0.z, A1.z, A0.w, A1.w, B.z, B.w);
        if (DUAL) {
          mma_bf16_16816(acu[i], U0.x, U1.x, U0.y, U1.y, B.x, B.y);
          mma_bf16_16816(acu[i], U0.z, U1.z, U0.w, U1.w, B.z, B.w);
        }
      }
    }
  }
  // partial sums of the 8 warps -> shared memory, summed in warp order
  float* rg = red + (size_t)warp * 16 * 8 * MT;
  float* ru = red + (size_t)(GM2_WARPS + warp) * 16 * 8 * MT;
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    // c0,c1: (row g, tokens 2t, 2t+1); c2,c3: (row g + 8, same tokens)
    rg[(g) * 8 * MT + i * 8 + 2 * t] = acc[i][0];
    rg[(g) * 8 * MT + i * 8 + 2 * t + 1] = acc[i][1];
    rg[(g + 8) * 8 * MT + i * 8 + 2 * t] = acc[i][2];
    rg[(g + 8) * 8 * MT + i * 8 + 2 * t + 1] = acc[i][3];
    if (DUAL) {
      ru[(g) * 8 * MT + i * 8 + 2 * t] = acu[i][0];
      ru[(g) * 8 * MT + i * 8 + 2 * t + 1] = acu[i][1];
      ru[(g + 8) * 8 * MT + i * 8 + 2 * t] = acu[i][2];
      ru[(g + 8) * 8 * MT + i * 8 + 2 * t + 1] = acu[i][3];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * 8 * MT; i += blockDim.x) {
    const int m = i / 16, r = i % 16;                   // consecutive threads -> consecutive output features
    const int n = n0 + r;
    if (m >= a.M || n >= a.N) continue;
    float gsum = 0.f, usum = 0.f;
#pragma unroll
    for (int wdx = 0; wdx < GM2_WARPS; ++wdx) {
      gsum += red[((size_t)wdx * 16 + r) * 8 * MT + m];
      if (DUAL) usum += red[((size_t)(GM2_WARPS + wdx) * 16 + r) * 8 * MT + m];
    }
    float v = DUAL ? siluf_(gsum) * usum : gsum;
    if (a.res) v += bf2f(a.res[(size_t)m * a.ldy + n]);
    if (a.out_f32) reinterpret_cast<float*>(a.y)[(size_t)m * a.ldy + n] = v;
    else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)m * a.ldy + n] = f2bf(v);
  }
}

template <int MT, bool DUAL>
static int launch_g2(const GemvMmaArgs& a, cudaStream_t s) {
  static bool done = false;
  if (!done) {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<MT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Gm2<MT>::SMEM);
    if (e != cudaSuccess) return (int)e;
    done = true;
  }
  return (int)launch_pdl(gemv_mma_kernel<MT, DUAL>, dim3((a.N + 15) / 16), dim3(GM2_WARPS * 32), Gm2<MT>::SMEM, s, a);
}

}  // namespace fb

using namespace fb;

// mode 1: SwiGLU (W = [gate rows | up rows], 2N rows). M <= 32, K % 32 == 0, ldx % 8 == 0.
extern "C" int fb_gemv_mma(void* y, const void* x, const void* w, const void* norm_w, const void* res, int M, int N, int K,
                           long ldx, long ldy, float eps, int mode, int out_f32, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32 || K % 32 || ldx % 8) return -1;
  GemvMmaArgs a;
  a.y = y; a.x = (const __nv_bfloat16*)x; a.w = (const __nv_bfloat16*)w; a.norm_w = (const __nv_bfloat16*)norm_w;
  a.res = (const __nv_bfloat16*)res; a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.eps = eps; a.out_f32 = out_f32;
  const int mt = (M + 7) / 8;
  if (mode == 1) {
    if (mt == 1) return launch_g2<1, true>(a, s);
    if (mt == 2) return launch_g2<2, true>(a, s);
    if (mt == 3) return launch_g2<3, true>(a, s);
    return launch_g2<4, true>(a, s);
  }
  if (mt == 1) return launch_g2<1, false>(a, s);
  if (mt == 2) return launch_g2<2, false>(a, s);
  if (mt == 3) return launch_g2<3, false>(a, s);
  return launch_g2<4, false>(a, s);
}
