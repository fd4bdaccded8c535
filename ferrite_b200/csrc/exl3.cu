// EXL3 (trellis-quantised) linears on the GPU. A weight W [k][n] (y = x W) is stored in a rotated basis,
//   W = diag(suh) H_k W_hat H_n diag(svh) / 128   (H = 128-point Hadamard blocks),
// W_hat in 16x16 tiles, each a cyclic stream of 256*bits bits; position t owns the 16-bit window ending at bit
// (t+1)*bits and decodes through the `mul1` codebook: x = state * 0x83DCD12D, s = byte sum of x,
// value = fp16(1024 + s) * fp16(0x1EEE) + fp16(0xC931) (one fp16 fma). Position t = lane*8 + j sits at tile row
// 2*(lane&3) + (j&1) + 8*((j>>1)&1), column (lane>>2) + 8*(j>>2).
//
// Kernels:
//   exl3_had      rows of 128-blocks: out = H128(in * pre) * post * scale (+ residual); the input and output rotations
//   exl3_gemv     z[m][n] = sum_k xh[m][k] W_hat[k][n] for up to 8 rows, tiles decoded in registers, the 8 warps of a
//                 CTA split K and are summed in warp order (deterministic)
//   exl3_decode   W_hat as bf16 [n][k] (K-major) for the tensor-core GEMM of the prompt path
// Counterparts in the reference: `exl3_rot_in`, `exl3_had_*`, `exl3_gemv*`, `exl3_recon_*` (`kernels/k-exl3/src`);
// host statement `formats/exl3.py` (after `crates/fe-exl3/src/cpu.rs`).
#include <cuda_fp16.h>

#include "api_ext.h"
#include "common.cuh"

namespace fb {

constexpr float EXL3_HAD_SCALE = 0.08838834764831845f;      // 1 / sqrt(128)

// unnormalised Sylvester Hadamard over 128 values held 4 per lane (index = lane * 4 + e)
__device__ __forceinline__ void had128(float v[4]) {
  float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
  v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float o = __shfl_xor_sync(0xffffffffu, v[e], m);
      v[e] = (lane & m) ? o - v[e] : v[e] + o;
    }
  }
}

// one warp per 128-block; in: bf16 (IN_F32 = 0) or fp32; out: fp32 (OUT_BF16 = 0) or bf16 with optional residual
template <int IN_F32, int OUT_BF16>
__global__ void exl3_had_kernel(void* __restrict__ out, const void* __restrict__ in, const __half* __restrict__ pre,
                                const __half* __restrict__ post, const __nv_bfloat16* __restrict__ res, int rows,
                                int width, float scale) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int blocks_per_row = width / 128;
  if (warp >= rows * blocks_per_row) return;
  const int row = warp / blocks_per_row, c0 = (warp % blocks_per_row) * 128 + lane * 4;
  float v[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const size_t idx = (size_t)row * width + c0 + e;
    float x = IN_F32 ? reinterpret_cast<const float*>(in)[idx] : bf2f(reinterpret_cast<const __nv_bfloat16*>(in)[idx]);
    if (pre) x *= __half2float(pre[c0 + e]);
    v[e] = x;
  }
  had128(v);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const size_t idx = (size_t)row * width + c0 + e;
    float y = v[e] * scale;
    if (post) y *= __half2float(post[c0 + e]);
    if (OUT_BF16) {
      if (res) y += bf2f(res[idx]);
      reinterpret_cast<__nv_bfloat16*>(out)[idx] = f2bf(y);
    } else {
      reinterpret_cast<float*>(out)[idx] = y;
    }
  }
}

// 16-bit window of the cyclic stream ending at bit `end` (exclusive); bit 0 = most significant bit of word 0
__device__ __forceinline__ uint32_t exl3_window(const uint32_t* words, int n_words, int end) {
  const int total = n_words * 32;
  int start = end - 16;
  if (start < 0) start += total;
  const int w0 = start >> 5, off = start & 31;
  const uint32_t a = words[w0], b = words[(w0 + 1) % n_words];
  const uint64_t both = ((uint64_t)a << 32) | b;
  return (uint32_t)((both >> (48 - off)) & 0xFFFFu);
}

__device__ __forceinline__ float exl3_mul1(uint32_t state) {
  const uint32_t x = state * 0x83DCD12Du;
  const uint32_t s = __dp4a(x, 0x01010101u, 0u);
  const __half v = __hfma(__int2half_rn(1024 + (int)s), __ushort_as_half((unsigned short)0x1EEE),
                          __ushort_as_half((unsigned short)0xC931));
  return __half2float(v);
}

constexpr int EXL3_KC = 4096;        // k values of xh staged per pass (fp16, up to 8 rows: 64 KB)

// grid = n / 16 column tiles; 8 warps split the k tiles of every pass
template <int M>
__global__ void __launch_bounds__(256) exl3_gemv_kernel(float* __restrict__ z, const float* __restrict__ xh,
                                                        const unsigned short* __restrict__ trellis, int rows, int k,
                                                        int n, int bits) {
  extern __shared__ __align__(16) unsigned char smem_exl3[];
  __half* xs = reinterpret_cast<__half*>(smem_exl3);                               // [M][EXL3_KC]
  uint32_t* wbuf = reinterpret_cast<uint32_t*>(smem_exl3 + (size_t)M * EXL3_KC * 2);   // [8 warps][64 words]
  float* part = reinterpret_cast<float*>(wbuf + 8 * 64);                            // [8 warps][M][16]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = blockIdx.x, n_tiles = n / 16;
  const int n_words = 8 * bits;
  uint32_t* my_words = wbuf + warp * 64;
  float acc[M][2];
#pragma unroll
  for (int m = 0; m < M; ++m) { acc[m][0] = 0.f; acc[m][1] = 0.f; }
  int rr[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) rr[j] = 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1);
  for (int kc = 0; kc < k; kc += EXL3_KC) {
    const int kn = min(EXL3_KC, k - kc);
    __syncthreads();
    for (int i = threadIdx.x; i < M * kn; i += blockDim.x) {
      const int m = i / kn, kk = i % kn;
      xs[m * EXL3_KC + kk] = __float2half_rn(m < rows ? xh[(size_t)m * k + kc + kk] : 0.f);
    }
    __syncthreads();
    for (int kt = warp; kt < kn / 16; kt += 8) {
      const unsigned short* tile = trellis + ((size_t)((kc >> 4) + kt) * n_tiles + nt) * (16 * bits);
      __syncwarp();
      for (int w = lane; w < n_words; w += 32) my_words[w] = (uint32_t)tile[2 * w] | ((uint32_t)tile[2 * w + 1] << 16);
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float wv = exl3_mul1(exl3_window(my_words, n_words, (lane * 8 + j + 1) * bits));
        const int krow = kt * 16 + rr[j];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m][j >> 2] = fmaf(__half2float(xs[m * EXL3_KC + krow]), wv, acc[m][j >> 2]);
      }
    }
  }
  // lanes sharing lane>>2 hold the 16 rows of the same two columns
#pragma unroll
  for (int m = 0; m < M; ++m) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float v = acc[m][c];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if ((lane & 3) == 0) part[(warp * M + m) * 16 + (lane >> 2) + 8 * c] = v;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < M * 16; i += blockDim.x) {
    const int m = i / 16, c = i % 16;
    if (m >= rows) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[(w * M + m) * 16 + c];
    z[(size_t)m * n + nt * 16 + c] = s;
  }
}

// W_hat as bf16 [n][k]: one warp per tile
__global__ void exl3_decode_kernel(__nv_bfloat16* __restrict__ out, const unsigned short* __restrict__ trellis, int k,
                                   int n, int bits) {
  __shared__ uint32_t wbuf[8][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long tile_id = (long)blockIdx.x * 8 + warp;
  const int n_tiles = n / 16;
  if (tile_id >= (long)(k / 16) * n_tiles) return;
  const int kt = (int)(tile_id / n_tiles), nt = (int)(tile_id % n_tiles);
  const int n_words = 8 * bits;
  const unsigned short* tile = trellis + (size_t)tile_id * (16 * bits);
  for (int w = lane; w < n_words; w += 32) wbuf[warp][w] = (uint32_t)tile[2 * w] | ((uint32_t)tile[2 * w + 1] << 16);
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float wv = exl3_mul1(exl3_window(wbuf[warp], n_words, (lane * 8 + j + 1) * bits));
    const int r = 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1), c = (lane >> 2) + 8 * (j >> 2);
    out[(size_t)(nt * 16 + c) * k + kt * 16 + r] = f2bf(wv);
  }
}

}  // namespace fb

using namespace fb;

// out = H128(in * pre) * post * scale (+ res). in_f32 / out_bf16 select the element types; width % 128 == 0.
extern "C" int fb_exl3_had(void* out, const void* in, const void* pre_f16, const void* post_f16, const void* res, int rows,
                           int width, float scale, int in_f32, int out_bf16, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (width % 128) return -1;
  const long warps = (long)rows * (width / 128);
  const unsigned grid = (unsigned)((warps * 32 + 255) / 256);
#define FB_HAD(I, O)                                                                                            \
  exl3_had_kernel<I, O><<<grid, 256, 0, s>>>(out, in, (const __half*)pre_f16, (const __half*)post_f16,          \
                                             (const __nv_bfloat16*)res, rows, width, scale)
  if (in_f32 && out_bf16) FB_HAD(1, 1); else if (in_f32) FB_HAD(1, 0); else if (out_bf16) FB_HAD(0, 1); else FB_HAD(0, 0);
#undef FB_HAD
  return (int)cudaGetLastError();
}

extern "C" int fb_exl3_gemv(float* z, const float* xh, const void* trellis, int rows, int k, int n, int bits,
                            cudaStream_t s) {
  if (rows <= 0) return 0;
  if (rows > 8 || k % 16 || n % 16 || bits < 1 || bits > 8) return -1;
  const int M = rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : 8;
  const size_t smem = (size_t)M * EXL3_KC * 2 + 8 * 64 * 4 + (size_t)8 * M * 16 * 4;
#define FB_EX(MT)                                                                                                   \
  do {                                                                                                              \
    static bool done = false;                                                                                       \
    if (!done) {                                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(exl3_gemv_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
      if (e != cudaSuccess) return (int)e;                                                                          \
      done = true;                                                                                                  \
    }                                                                                                               \
    exl3_gemv_kernel<MT><<<n / 16, 256, smem, s>>>(z, xh, (const unsigned short*)trellis, rows, k, n, bits);        \
  } while (0)
  if (M == 1) FB_EX(1); else if (M == 2) FB_EX(2); else if (M == 4) FB_EX(4); else FB_EX(8);
#undef FB_EX
  return (int)cudaGetLastError();
}

extern "C" int fb_exl3_decode(void* w_hat_t_bf16, const void* trellis, int k, int n, int bits, cudaStream_t s) {
  if (k % 16 || n % 16 || bits < 1 || bits > 8) return -1;
  const long tiles = (long)(k / 16) * (n / 16);
  exl3_decode_kernel<<<(unsigned)((tiles + 7) / 8), 256, 0, s>>>((__nv_bfloat16*)w_hat_t_bf16, (const unsigned short*)trellis,
                                                                k, n, bits);
  return (int)cudaGetLastError();
}
