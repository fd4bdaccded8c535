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

// ---- few-row GEMV on mma.sync fragments ---------------------------------------------------------------------------
// The trellis tile layout IS a tensor-core fragment layout: lane l's eight weights of a 16 x 16 tile sit at k rows
// 2 (l & 3) + {0, 1} + {0, 8} and columns (l >> 2) + {0, 8}, which are the four A registers of mma.m16n8k16 when the tile
// is read as W^T [16 columns][16 k]. So a lane decodes its eight codes straight into four f16x2 registers and one
// mma.sync multiplies the tile with up to eight activation rows (the B operand, from shared memory), fp32 accumulation.
// No weight is converted to fp32 and no conversion instruction is issued at all: 1024 + s as f16 is the bit pattern
// 0x6400 + s (s <= 1020 keeps the exponent), two of them are packed into one word and one HFMA2 applies the codebook's
// affine map to both. With 4 bits per weight a tile is 32 words, one per lane; the 16-bit window of a code is a funnel
// shift over the lane's word and its left neighbour's (one shuffle per tile). Four tiles per warp are in flight.
__device__ __forceinline__ uint32_t exl3_pair_f16x2(uint32_t st0, uint32_t st1) {
  // byte sum of the scrambled state, started at 0x6400: the f16 bit pattern of 1024 + s
  const uint32_t h0 = __dp4a(st0 * 0x83DCD12Du, 0x01010101u, 0x6400u);
  const uint32_t h1 = __dp4a(st1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
  const uint32_t packed = __byte_perm(h0, h1, 0x5410);
  const __half2 v = __hfma2(*reinterpret_cast<const __half2*>(&packed), __half2half2(__ushort_as_half((unsigned short)0x1EEE)),
                            __half2half2(__ushort_as_half((unsigned short)0xC931)));
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void exl3_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// the B fragment of k tile kt for this lane: activation row g (zero beyond `rows`), k = 16 kt + 2t + {0, 1} and + {8, 9};
// the rotated activations are a few KB that every CTA reads: they stay in L1 / L2, no staging pass
__device__ __forceinline__ void exl3_bfrag(uint32_t& b0, uint32_t& b1, const float* __restrict__ xh, int rows, int k, int kt,
                                           int g, int t) {
  b0 = 0u; b1 = 0u;
  if (g < rows) {
    const float* xr = xh + (size_t)g * k + kt * 16 + 2 * t;
    const float2 lo = __ldg(reinterpret_cast<const float2*>(xr));
    const float2 hi = __ldg(reinterpret_cast<const float2*>(xr + 8));
    const __half2 hlo = __float22half2_rn(lo), hhi = __float22half2_rn(hi);
    b0 = *reinterpret_cast<const uint32_t*>(&hlo);
    b1 = *reinterpret_cast<const uint32_t*>(&hhi);
  }
}

// grid = n / 16 column tiles; the 8 warps of a CTA split the k tiles.
template <bool BITS4>
__global__ void __launch_bounds__(256) exl3_gemv_mma_kernel(float* __restrict__ z, const float* __restrict__ xh,
                                                            const unsigned short* __restrict__ trellis, int rows, int k,
                                                            int n, int bits) {
  __shared__ float part[8 * 16 * 8];                         // [8 warps][16 columns][8 rows]
  __shared__ uint32_t wbuf[8 * 64];                          // [8 warps][64 words] (bits != 4)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int nt = blockIdx.x, n_tiles = n / 16;
  const int n_words = 8 * bits;
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  const int ntile = k / 16;
  const uint32_t* tiles = reinterpret_cast<const uint32_t*>(trellis) + (size_t)nt * n_words;
  const size_t tstride = (size_t)n_tiles * n_words;          // words between consecutive k tiles
  if (BITS4) {
    constexpr int DEPTH = 4;
    uint32_t nxt[DEPTH];
#pragma unroll
    for (int u = 0; u < DEPTH; ++u) {
      const int kt = warp + 8 * u;
      nxt[u] = kt < ntile ? __ldg(tiles + (size_t)kt * tstride + lane) : 0u;
    }
    for (int kt0 = warp; kt0 < ntile; kt0 += 8 * DEPTH) {
      uint32_t cur[DEPTH];
#pragma unroll
      for (int u = 0; u < DEPTH; ++u) {
        cur[u] = nxt[u];
        const int ktn = kt0 + 8 * (u + DEPTH);
        nxt[u] = ktn < ntile ? __ldg(tiles + (size_t)ktn * tstride + lane) : 0u;
      }
#pragma unroll
      for (int u = 0; u < DEPTH; ++u) {
        const int kt = kt0 + 8 * u;
        if (kt < ntile) {                                    // uniform over the warp
          const uint32_t prev = __shfl_sync(0xffffffffu, cur[u], (lane + 31) & 31);
          uint32_t st[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) st[j] = __funnelshift_r(cur[u], prev, 28 - 4 * j) & 0xFFFFu;
          // A registers: (col g, k 2t..2t+1), (col g + 8, same k), (col g, k + 8), (col g + 8, k + 8)
          const uint32_t a[4] = {exl3_pair_f16x2(st[0], st[1]), exl3_pair_f16x2(st[4], st[5]),
                                 exl3_pair_f16x2(st[2], st[3]), exl3_pair_f16x2(st[6], st[7])};
          uint32_t b0, b1;
          exl3_bfrag(b0, b1, xh, rows, k, kt, g, t);
          exl3_mma(d, a, b0, b1);
        }
      }
    }
  } else {
    uint32_t* my_words = wbuf + warp * 64;
    for (int kt = warp; kt < ntile; kt += 8) {
      __syncwarp();
      for (int w = lane; w < n_words; w += 32) my_words[w] = __ldg(tiles + (size_t)kt * tstride + w);
      __syncwarp();
      uint32_t st[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) st[j] = exl3_window(my_words, n_words, (lane * 8 + j + 1) * bits);
      const uint32_t a[4] = {exl3_pair_f16x2(st[0], st[1]), exl3_pair_f16x2(st[4], st[5]),
                             exl3_pair_f16x2(st[2], st[3]), exl3_pair_f16x2(st[6], st[7])};
      uint32_t b0, b1;
      exl3_bfrag(b0, b1, xh, rows, k, kt, g, t);
      exl3_mma(d, a, b0, b1);
    }
  }
  // D fragment: rows = columns of the tile (g, g + 8), columns = activation rows (2t, 2t + 1)
  float* mine = part + warp * 128;
  mine[g * 8 + 2 * t] = d[0]; mine[g * 8 + 2 * t + 1] = d[1];
  mine[(g + 8) * 8 + 2 * t] = d[2]; mine[(g + 8) * 8 + 2 * t + 1] = d[3];
  __syncthreads();
  for (int i = threadIdx.x; i < 128; i += blockDim.x) {
    const int c = i >> 3, m = i & 7;
    if (m >= rows) continue;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += part[w * 128 + i];
    z[(size_t)m * n + nt * 16 + c] = sum;
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
  if (((uintptr_t)trellis & 3)) return -1;
  if (bits == 4) exl3_gemv_mma_kernel<true><<<n / 16, 256, 0, s>>>(z, xh, (const unsigned short*)trellis, rows, k, n, bits);
  else exl3_gemv_mma_kernel<false><<<n / 16, 256, 0, s>>>(z, xh, (const unsigned short*)trellis, rows, k, n, bits);
  return (int)cudaGetLastError();
}

extern "C" int fb_exl3_decode(void* w_hat_t_bf16, const void* trellis, int k, int n, int bits, cudaStream_t s) {
  if (k % 16 || n % 16 || bits < 1 || bits > 8) return -1;
  const long tiles = (long)(k / 16) * (n / 16);
  exl3_decode_kernel<<<(unsigned)((tiles + 7) / 8), 256, 0, s>>>((__nv_bfloat16*)w_hat_t_bf16, (const unsigned short*)trellis,
                                                                k, n, bits);
  return (int)cudaGetLastError();
}
