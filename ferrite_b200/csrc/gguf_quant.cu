// GGUF block formats on the GPU: dequantisation to bf16 (load path: a GGUF checkpoint becomes bf16 or is requantised
// to NVFP4 for the tensor-core kernels), the q8_1 activation quantiser, and a dequantising GEMV for decode rows that
// reads the checkpoint's own blocks. One device routine decodes a 32-value group of any supported type, so the
// dequantiser and the GEMV cannot disagree.
//
// Types: Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, IQ4_NL, MXFP4 (32-value blocks) and Q4_K, Q5_K, Q6_K, IQ4_XS (256-value
// super-blocks of eight 32-value groups). The codebook types (IQ1/IQ2/IQ3) and Q2_K/Q3_K are parsed by the reader
// but not decoded here. Counterparts in the reference: `ggq_deq_*`, `ggq_q8_1`, `ggq_gemv_*`
// (`kernels/k-gguf/src/{deq,q8,gemv}.rs`), host reference `crates/fe-ggq/src/refq.rs`.
#include <cuda_fp16.h>

#include "api_ext.h"
#include "common.cuh"

namespace fb {

enum GgmlType { GT_Q4_0 = 2, GT_Q4_1 = 3, GT_Q5_0 = 6, GT_Q5_1 = 7, GT_Q8_0 = 8, GT_Q4_K = 12, GT_Q5_K = 13,
                GT_Q6_K = 14, GT_IQ4_NL = 20, GT_IQ4_XS = 23, GT_MXFP4 = 39 };

__device__ __constant__ float kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
__device__ __constant__ float kMxfp4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

__host__ __device__ inline int gg_block_values(int t) {
  return (t == GT_Q4_K || t == GT_Q5_K || t == GT_Q6_K || t == GT_IQ4_XS) ? 256 : 32;
}
__host__ __device__ inline int gg_block_bytes(int t) {
  switch (t) {
    case GT_Q4_0: return 18; case GT_Q4_1: return 20; case GT_Q5_0: return 22; case GT_Q5_1: return 24;
    case GT_Q8_0: return 34; case GT_Q4_K: return 144; case GT_Q5_K: return 176; case GT_Q6_K: return 210;
    case GT_IQ4_NL: return 18; case GT_IQ4_XS: return 136; case GT_MXFP4: return 17;
  }
  return 0;
}

__device__ __forceinline__ float ld_half(const unsigned char* p) {
  const unsigned short u = (unsigned short)p[0] | ((unsigned short)p[1] << 8);
  return __half2float(__ushort_as_half(u));
}

// six-bit (scale, min) pair j of a K-quant super-block (12 packed bytes)
__device__ __forceinline__ void k4_scale_min(const unsigned char* sc, int j, float& s, float& m) {
  if (j < 4) { s = (float)(sc[j] & 63); m = (float)(sc[j + 4] & 63); }
  else { s = (float)((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4)); m = (float)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)); }
}

// Decode value `l` (0..31) of the 32-value group `g` of the block at `b`.
__device__ __forceinline__ float gg_value(int type, const unsigned char* b, int g, int l) {
  switch (type) {
    case GT_Q8_0: return ld_half(b) * (float)(signed char)b[2 + l];
    case GT_Q4_0: { const unsigned char q = b[2 + (l & 15)]; return ld_half(b) * ((float)(l < 16 ? (q & 0xF) : (q >> 4)) - 8.f); }
    case GT_Q4_1: { const unsigned char q = b[4 + (l & 15)]; return ld_half(b) * (float)(l < 16 ? (q & 0xF) : (q >> 4)) + ld_half(b + 2); }
    case GT_IQ4_NL: { const unsigned char q = b[2 + (l & 15)]; return ld_half(b) * kIq4nl[l < 16 ? (q & 0xF) : (q >> 4)]; }
    case GT_MXFP4: { const unsigned char q = b[1 + (l & 15)]; return ldexpf(0.5f, (int)b[0] - 127) * kMxfp4[l < 16 ? (q & 0xF) : (q >> 4)]; }
    case GT_Q5_0:
    case GT_Q5_1: {
      const int o = type == GT_Q5_1 ? 4 : 2;
      const unsigned qh = (unsigned)b[o] | ((unsigned)b[o + 1] << 8) | ((unsigned)b[o + 2] << 16) | ((unsigned)b[o + 3] << 24);
      const unsigned char q = b[o + 4 + (l & 15)];
      const int v = (l < 16 ? (q & 0xF) : (q >> 4)) | (((qh >> l) & 1) << 4);
      return type == GT_Q5_0 ? ld_half(b) * ((float)v - 16.f) : ld_half(b) * (float)v + ld_half(b + 2);
    }
    case GT_Q4_K: {
      float s, m;
      k4_scale_min(b + 4, g, s, m);
      const unsigned char q = b[16 + (g >> 1) * 32 + l];
      return ld_half(b) * s * (float)((g & 1) ? (q >> 4) : (q & 0xF)) - ld_half(b + 2) * m;
    }
    case GT_Q5_K: {
      float s, m;
      k4_scale_min(b + 4, g, s, m);
      const unsigned char q = b[48 + (g >> 1) * 32 + l];
      const int v = ((g & 1) ? (q >> 4) : (q & 0xF)) + (((b[16 + l] >> g) & 1) << 4);
      return ld_half(b) * s * (float)v - ld_half(b + 2) * m;
    }
    case GT_Q6_K: {
      const int h = g >> 2, k = g & 3;                       // half of the super-block, 32-value quarter inside it
      const unsigned char* ql = b + h * 64;
      const unsigned char hh = b[128 + h * 32 + l];
      const unsigned char lo = (k & 1) ? ql[32 + l] : ql[l];
      const int nib = (k < 2) ? (lo & 0xF) : (lo >> 4);
      const int v = (nib | (((hh >> (2 * k)) & 3) << 4)) - 32;
      const float sc = (float)(signed char)b[192 + h * 8 + (l >> 4) + 2 * k];
      return ld_half(b + 208) * sc * (float)v;
    }
    case GT_IQ4_XS: {
      const unsigned sh = (unsigned)b[2] | ((unsigned)b[3] << 8);
      const int ls = ((b[4 + (g >> 1)] >> (4 * (g & 1))) & 0xF) | (((sh >> (2 * g)) & 3) << 4);
      const unsigned char q = b[8 + g * 16 + (l & 15)];
      return ld_half(b) * (float)(ls - 32) * kIq4nl[l < 16 ? (q & 0xF) : (q >> 4)];
    }
  }
  return 0.f;
}

// one thread per value; consecutive threads take consecutive values, so the bf16 stores coalesce
__global__ void gguf_dequant_kernel(__nv_bfloat16* __restrict__ out, const unsigned char* __restrict__ raw, int type,
                                    long n) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int bv = gg_block_values(type), bb = gg_block_bytes(type);
  const long blk = i / bv;
  const int in = (int)(i % bv);
  out[i] = f2bf(gg_value(type, raw + blk * bb, in >> 5, in & 31));
}

// q8_1 blocks of 32 activations: {half d, half d * sum(q), int8 q[32]} = 36 bytes; one warp per block
__global__ void q8_1_quant_kernel(unsigned char* __restrict__ out, const __nv_bfloat16* __restrict__ x, long n_blocks) {
  const long blk = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (blk >= n_blocks) return;
  const float v = bf2f(x[blk * 32 + lane]);
  const float amax = warp_max(fabsf(v));
  const float d = amax / 127.f;
  const int q = d > 0.f ? __float2int_rn(v / d) : 0;
  const float s = warp_sum((float)q);
  unsigned char* o = out + blk * 36;
  o[4 + lane] = (unsigned char)(signed char)q;
  if (lane == 0) {
    __half2 hh = __floats2half2_rn(d, d * s);                 // blocks are 36 bytes, so `o` is 4-byte aligned
    *reinterpret_cast<__half2*>(o) = hh;
  }
}

// y[m][n] = sum_k x[m][k] * W[n][k], W in GGUF blocks, M <= 8 decode rows. One warp per output row n; lane l decodes
// value l of every group, so a warp reads whole groups; x is staged in shared memory as fp32.
template <int M>
__global__ void __launch_bounds__(256) gguf_gemv_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                                        const unsigned char* __restrict__ raw,
                                                        const __nv_bfloat16* __restrict__ res, int type, int rows, int N,
                                                        int K, long ldx, long ldy) {
  extern __shared__ float xs_gg[];                            // [M][K]
  for (int i = threadIdx.x; i < M * K; i += blockDim.x) {
    const int m = i / K, k = i % K;
    xs_gg[i] = m < rows ? bf2f(x[(size_t)m * ldx + k]) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const int bv = gg_block_values(type), bb = gg_block_bytes(type);
  const unsigned char* wrow = raw + (size_t)n * (K / bv) * bb;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int g0 = 0; g0 < K / 32; ++g0) {
    const int blk = (g0 * 32) / bv, g = ((g0 * 32) % bv) >> 5;
    const float w = gg_value(type, wrow + (size_t)blk * bb, g, lane);
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = fmaf(w, xs_gg[m * K + g0 * 32 + lane], acc[m]);
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

static bool gg_supported(int t) { return gg_block_bytes(t) != 0; }

}  // namespace fb

using namespace fb;

extern "C" int fb_gguf_dequant(void* out_bf16, const void* raw, int type, long n_values, cudaStream_t s) {
  if (n_values <= 0) return 0;
  if (!gg_supported(type) || n_values % gg_block_values(type)) return -1;
  gguf_dequant_kernel<<<(unsigned)((n_values + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)out_bf16, (const unsigned char*)raw,
                                                                         type, n_values);
  return (int)cudaGetLastError();
}

extern "C" int fb_q8_1_quant(void* out, const void* x_bf16, long n_values, cudaStream_t s) {
  if (n_values <= 0) return 0;
  if (n_values % 32) return -1;
  const long nb = n_values / 32;
  q8_1_quant_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, s>>>((unsigned char*)out, (const __nv_bfloat16*)x_bf16, nb);
  return (int)cudaGetLastError();
}

extern "C" int fb_gguf_gemv(void* y, const void* x, const void* raw, const void* res, int type, int M, int N, int K,
                            long ldx, long ldy, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (!gg_supported(type) || M > 8 || K % gg_block_values(type)) return -1;
  const size_t smem = (size_t)(M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8) * K * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const dim3 grid((N + 7) / 8), block(256);
#define FB_GG(MT)                                                                                                   \
  do {                                                                                                              \
    static bool done = false;                                                                                       \
    if (!done) {                                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(gguf_gemv_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      if (e != cudaSuccess) return (int)e;                                                                          \
      done = true;                                                                                                  \
    }                                                                                                               \
    gguf_gemv_kernel<MT><<<grid, block, smem, s>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const unsigned char*)raw, \
                                                   (const __nv_bfloat16*)res, type, M, N, K, ldx, ldy);             \
  } while (0)
  if (M == 1) FB_GG(1); else if (M == 2) FB_GG(2); else if (M <= 4) FB_GG(4); else FB_GG(8);
#undef FB_GG
  return (int)cudaGetLastError();
}
