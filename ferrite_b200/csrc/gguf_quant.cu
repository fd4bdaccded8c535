// GGUF block formats on the GPU: dequantisation to bf16 (load path: a GGUF checkpoint becomes bf16 or is requantised
// to NVFP4 for the tensor-core kernels), the q8_1 activation quantiser, and a dequantising GEMV for decode rows that
// reads the checkpoint's own blocks. One device routine decodes a 32-value group of any supported type, so the
// dequantiser and the GEMV cannot disagree.
//
// Types: Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, IQ4_NL, MXFP4 (32-value blocks) and Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_XS and the
// codebook types IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S (256-value super-blocks of eight 32-value
// groups; grids in `gguf_tables.cuh`). Every product is written with explicit single roundings in the order of the
// host decoder (`formats/gguf.py`), so device and host agree bit for bit. Counterparts in the reference: `ggq_deq_*`,
// `ggq_q8_1`, `ggq_gemv_*` (`kernels/k-gguf/src/{deq,q8,gemv}.rs`), block decoders `dec.rs` / `vq.rs` / `tables.rs`,
// host reference `crates/fe-ggq/src/refq.rs`.
#include <cuda_fp16.h>

#include "api_ext.h"
#include "common.cuh"
#include "gguf_tables.cuh"

namespace fb {

enum GgmlType { GT_Q4_0 = 2, GT_Q4_1 = 3, GT_Q5_0 = 6, GT_Q5_1 = 7, GT_Q8_0 = 8, GT_Q2_K = 10, GT_Q3_K = 11, GT_Q4_K = 12,
                GT_Q5_K = 13, GT_Q6_K = 14, GT_IQ2_XXS = 16, GT_IQ2_XS = 17, GT_IQ3_XXS = 18, GT_IQ1_S = 19, GT_IQ4_NL = 20,
                GT_IQ3_S = 21, GT_IQ2_S = 22, GT_IQ4_XS = 23, GT_IQ1_M = 29, GT_MXFP4 = 39 };

__device__ __constant__ float kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
__device__ __constant__ float kMxfp4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

__host__ __device__ inline int gg_block_values(int t) {
  switch (t) {
    case GT_Q2_K: case GT_Q3_K: case GT_Q4_K: case GT_Q5_K: case GT_Q6_K: case GT_IQ4_XS: case GT_IQ2_XXS: case GT_IQ2_XS:
    case GT_IQ2_S: case GT_IQ3_XXS: case GT_IQ3_S: case GT_IQ1_S: case GT_IQ1_M: return 256;
  }
  return 32;
}
__host__ __device__ inline int gg_block_bytes(int t) {
  switch (t) {
    case GT_Q4_0: return 18; case GT_Q4_1: return 20; case GT_Q5_0: return 22; case GT_Q5_1: return 24;
    case GT_Q8_0: return 34; case GT_Q4_K: return 144; case GT_Q5_K: return 176; case GT_Q6_K: return 210;
    case GT_IQ4_NL: return 18; case GT_IQ4_XS: return 136; case GT_MXFP4: return 17;
    case GT_Q2_K: return 84; case GT_Q3_K: return 110; case GT_IQ2_XXS: return 66; case GT_IQ2_XS: return 74;
    case GT_IQ2_S: return 82; case GT_IQ3_XXS: return 98; case GT_IQ3_S: return 110; case GT_IQ1_S: return 50;
    case GT_IQ1_M: return 56;
  }
  return 0;
}

__device__ __forceinline__ float ld_half(const unsigned char* p) {
  const unsigned short u = (unsigned short)p[0] | ((unsigned short)p[1] << 8);
  return __half2float(__ushort_as_half(u));
}

__device__ __forceinline__ unsigned ld_u16(const unsigned char* p) { return (unsigned)p[0] | ((unsigned)p[1] << 8); }
__device__ __forceinline__ unsigned ld_u32(const unsigned char* p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }
// value j (int8) of an 8-value / 4-value grid entry, with the sign bit j of `signs` applied
__device__ __forceinline__ float grid8(uint64_t e, int j, unsigned signs) {
  const float v = (float)(signed char)((e >> (8 * j)) & 0xFF);
  return ((signs >> j) & 1) ? -v : v;
}
__device__ __forceinline__ float grid4(uint32_t e, int j) { return (float)(signed char)((e >> (8 * j)) & 0xFF); }

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
    case GT_Q2_K: {
      const unsigned char sc = b[g * 2 + (l >> 4)];
      const float q = (float)((b[16 + (g >> 2) * 32 + l] >> (2 * (g & 3))) & 3);
      return __fsub_rn(__fmul_rn(__fmul_rn(ld_half(b + 80), (float)(sc & 0xF)), q), __fmul_rn(ld_half(b + 82), (float)(sc >> 4)));
    }
    case GT_Q3_K: {
      const int k = g * 2 + (l >> 4);
      const unsigned char* sc = b + 96;
      const int low = k < 8 ? (sc[k] & 0xF) : (sc[k - 8] >> 4);
      const int scale = (low | (((sc[8 + (k & 3)] >> (2 * (k >> 2))) & 3) << 4)) - 32;
      const int q = ((b[32 + (g >> 2) * 32 + l] >> (2 * (g & 3))) & 3) - ((b[l] >> g) & 1 ? 0 : 4);
      return __fmul_rn(__fmul_rn(ld_half(b + 108), (float)scale), (float)q);
    }
    case GT_IQ2_XXS: {
      const unsigned char* q = b + 2 + 8 * g;
      const unsigned aux = ld_u32(q + 4);
      const float db = __fmul_rn(__fmul_rn(ld_half(b), 0.5f + (float)(aux >> 28)), 0.25f);
      const int e = l >> 3;
      return __fmul_rn(db, grid8(gguf_iq2xxs_grid[q[e]], l & 7, gguf_ksigns[(aux >> (7 * e)) & 127]));
    }
    case GT_IQ2_XS: {
      const int e = l >> 3;
      const unsigned q = ld_u16(b + 2 + (g * 4 + e) * 2);
      const unsigned char sc = b[66 + g];
      const float db = __fmul_rn(__fmul_rn(ld_half(b), 0.5f + (float)(e < 2 ? (sc & 0xF) : (sc >> 4))), 0.25f);
      return __fmul_rn(db, grid8(gguf_iq2xs_grid[q & 511], l & 7, gguf_ksigns[q >> 9]));
    }
    case GT_IQ2_S: {
      const int e = l >> 3;
      const unsigned idx = (unsigned)b[2 + g * 4 + e] | (((unsigned)b[66 + g] << (8 - 2 * e)) & 0x300);
      const unsigned char sc = b[74 + g];
      const float db = __fmul_rn(__fmul_rn(ld_half(b), 0.5f + (float)(e < 2 ? (sc & 0xF) : (sc >> 4))), 0.25f);
      return __fmul_rn(db, grid8(gguf_iq2s_grid[idx], l & 7, b[34 + g * 4 + e]));
    }
    case GT_IQ3_XXS: {
      const unsigned aux = ld_u32(b + 66 + 4 * g);
      const float db = __fmul_rn(__fmul_rn(ld_half(b), 0.5f + (float)(aux >> 28)), 0.5f);
      const float v = grid4(gguf_iq3xxs_grid[b[2 + g * 8 + (l >> 2)]], l & 3);
      const unsigned signs = gguf_ksigns[(aux >> (7 * (l >> 3))) & 127];
      return __fmul_rn(db, ((signs >> (l & 7)) & 1) ? -v : v);
    }
    case GT_IQ3_S: {
      const unsigned char sc = b[106 + (g >> 1)];
      const float db = __fmul_rn(ld_half(b), 1.f + 2.f * (float)((g & 1) ? (sc >> 4) : (sc & 0xF)));
      const int e4 = l >> 2;
      const unsigned idx = (unsigned)b[2 + g * 8 + e4] | ((((unsigned)b[66 + g] >> e4) & 1) << 8);
      const float v = grid4(gguf_iq3s_grid[idx], l & 3);
      return __fmul_rn(db, ((b[74 + g * 4 + (l >> 3)] >> (l & 7)) & 1) ? -v : v);
    }
    case GT_IQ1_S: {
      const unsigned qh = ld_u16(b + 34 + 2 * g);
      const float dl = __fmul_rn(ld_half(b), (float)(2 * ((qh >> 12) & 7) + 1));
      const int e = l >> 3;
      const unsigned idx = (unsigned)b[2 + g * 4 + e] | (((qh >> (3 * e)) & 7) << 8);
      const float v = (float)(signed char)((gguf_iq1s_grid[idx] >> (8 * (l & 7))) & 0xFF);
      return __fmul_rn(dl, v + ((qh & 0x8000) ? -0.125f : 0.125f));
    }
    case GT_IQ1_M: {
      const unsigned s0 = ld_u16(b + 48), s1 = ld_u16(b + 50), s2 = ld_u16(b + 52), s3 = ld_u16(b + 54);
      const unsigned short dbits = (unsigned short)((s0 >> 12) | ((s1 >> 8) & 0x00F0) | ((s2 >> 4) & 0x0F00) | (s3 & 0xF000));
      const float d = __half2float(__ushort_as_half(dbits));
      const int e = l >> 3;
      const unsigned w = (g >> 1) == 0 ? s0 : (g >> 1) == 1 ? s1 : (g >> 1) == 2 ? s2 : s3;
      const float dl = __fmul_rn(d, (float)(2 * ((w >> (6 * (g & 1) + 3 * (e >> 1))) & 7) + 1));
      const unsigned char qhb = b[32 + g * 2 + (e >> 1)];
      const unsigned h = (e & 1) ? (qhb >> 4) : (qhb & 0xF);
      const unsigned idx = (unsigned)b[g * 4 + e] | ((h & 7) << 8);
      const float v = (float)(signed char)((gguf_iq1s_grid[idx] >> (8 * (l & 7))) & 0xFF);
      return __fmul_rn(dl, v + ((h & 8) ? -0.125f : 0.125f));
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
