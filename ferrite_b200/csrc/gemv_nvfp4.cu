// NVFP4-weight GEMV for 1..8 activation rows (W4A16): e2m1 codes become f16x2 by bit placement (two shifts and two
// logic ops per pair of weights, no conversion instruction), are multiplied against f16 activations with HFMA2 inside
// each 16-value block, and the block sums are scaled (e4m3 block scale) into fp32 accumulators. 0.5625 bytes per
// weight cross HBM instead of 2.
//
// Why no `cvt.rn.f16x2.e2m1x2`: measured on B200 (ncu, gate|up 2 x 17408 x 5120, 1 row) the conversion pipe was 86 %
// busy and the kernel ran at 2.15 TB/s; the packed-format conversions issue at a fraction of the ALU rate. The bit
// placement: a nibble S E E M put at f16 bits 15 and 11..9 is the f16 number e2m1 * 2^-14 (exponent field 000EE,
// mantissa M0..0; EE = 0 is an f16 subnormal, which is exactly M * 0.5 * 2^-14), so the factor 2^14 moves into the
// activations: every activation row is staged as x * 2^s with s = min(14, floor(log2(32768 / max|x|))), which also
// keeps the f16 products in the normal range, and the epilogue multiplies by 2^(14 - s). The staged activations are
// laid out so that a warp's 16-byte reads of them are contiguous (the first version's reads were 64 bytes apart:
// 4-way bank conflicts, 67 % of the shared-memory pipe).
//
// The decode-side role of the reference's low-bit GEMVs (`exl3_gemv*`, `kernels/k-exl3/src/gemv.rs:227`; NVFP4
// itself serves only its prompt path, `kernels/k-fp4/src/lib.rs`). Same structure as the bf16 GEMV: the next
// weight batch is always in flight, the first one requested before griddepcontrol.wait, RMSNorm prologue,
// residual / SwiGLU epilogue, and an optional one-shot all-reduce over NVLink peers fused into the epilogue for
// row-parallel projections under tensor parallelism.
//
// Layouts: codes [rows][K/2] bytes, element 2i in the low nibble; scales tiled per row as
// [group of 4 spans][lane 32][span 4][2 blocks] (see formats/nvfp4.py `tile_scales_gemv`).
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "api_ext.h"
#include "comm_core.cuh"

namespace fb {

constexpr int G4_THREADS = 256;
constexpr int G4_WARPS = 8;
constexpr int G4_R = 2;                       // weight rows per warp
constexpr int G4_SPAN = 1024;                 // weights per warp load (32 lanes x 32 codes)
constexpr int G4_GROUP = 4;                   // spans per batch
constexpr int G4_BATCH = G4_SPAN * G4_GROUP;  // 4096 weights
constexpr int G4_SMEM = 96 * 1024;

struct Gemv4Args {
  const __nv_bfloat16* X;       // [M][ldx]
  const uint8_t* Wq;            // [rows][K/2]
  const uint8_t* Sc;            // [rows][sc_stride] tiled scales
  const __nv_bfloat16* norm_w;
  const __nv_bfloat16* res;
  void* Y;
  float global_scale;
  const float* row_alpha;       // null, or one tensor scale per weight row (fused checkpoint parts); replaces global_scale
  int M, N, K;
  long ldx, ldy;
  long sc_stride;
  float eps;
  int out_f32;
  int rows_per_cta;
  int kc;
  int one;                      // the value 1 (spare: lets an experiment keep a constant out of the compiler's sight)
};

struct Batch4 {
  uint4 w[G4_R][G4_GROUP];
  uint2 s[G4_R];
};

__host__ __device__ inline int gemv4_chunk_len(int M, int K) {
  int kpad = (K + G4_BATCH - 1) / G4_BATCH * G4_BATCH;
  int cap = (G4_SMEM / 2 / M) / G4_BATCH * G4_BATCH;
  if (cap < G4_BATCH) cap = G4_BATCH;
  return kpad < cap ? kpad : cap;
}

template <bool SWIGLU>
__device__ __forceinline__ void g4_rows(const Gemv4Args& a, int (&rows)[G4_R], int n) {
#pragma unroll
  for (int r = 0; r < G4_R; ++r) rows[r] = SWIGLU ? (min(n, a.N - 1) + r * a.N) : min(n + r, a.N - 1);
}

// loads of the batch that starts at absolute k = kb (a multiple of 4096)
__device__ __forceinline__ void g4_load(Batch4& b, const Gemv4Args& a, const int (&rows)[G4_R], int kb) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int r = 0; r < G4_R; ++r) {
    const uint8_t* wrow = a.Wq + (size_t)rows[r] * (a.K / 2);
#pragma unroll
    for (int u = 0; u < G4_GROUP; ++u) {
      int k = kb + u * G4_SPAN + lane * 32;
      b.w[r][u] = (k < a.K) ? ldg_stream(wrow + k / 2) : make_uint4(0, 0, 0, 0);
    }
    b.s[r] = ldg_stream8(a.Sc + (size_t)rows[r] * a.sc_stride + (size_t)(kb / G4_BATCH) * 256 + lane * 8);
  }
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(byte & 0xffu), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Eight e2m1 codes of one 32-bit word -> four f16x2 holding (code j, code j + 4) * 2^-14, j = 0..3: nibble j sits
// 16 bits below nibble j + 4, so one shift lines both up with the two halves of the result.
//
// (Writing the shifts as integer multiply-adds, to move them off the integer pipe, measured slower: 150 vs 142 us on
// the vocabulary head.)
__device__ __forceinline__ void e2m1x8_to_half2x4(uint32_t w, __half2 (&h)[4], uint32_t one) {
  constexpr uint32_t SGN = 0x80008000u, MAG = 0x0E000E00u;
  uint32_t o[4];
  (void)one;
  o[0] = ((w << 12) & SGN) | ((w << 9) & MAG);
  o[1] = ((w << 8) & SGN) | ((w << 5) & MAG);
  o[2] = ((w << 4) & SGN) | ((w << 1) & MAG);
  o[3] = (w & SGN) | ((w >> 3) & MAG);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = *reinterpret_cast<__half2*>(&o[j]);
}

// Position (in halfs, inside a staged row) of the 16-byte chunk that holds the activations of weight word `wi`
// (8 codes) of lane `lane` in the span that starts at `span0`: chunks of one word index are contiguous over the lanes.
__device__ __forceinline__ int g4_xpos(int span0, int lane, int wi) { return span0 + (wi * 32 + lane) * 8; }

// `klim`: end of the valid k range inside the staged chunk, rounded up to a span. Spans past it hold only padding
// (K = 5120 fills 5 of the 8 spans of two batches): they are skipped, not multiplied by zero.
template <int M>
__device__ __forceinline__ void g4_consume(float (&acc)[G4_R][M], const Batch4& b, const __half* xs, int kc, int koff,
                                           int klim, uint32_t one) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int u = 0; u < G4_GROUP; ++u) {
    const int span0 = koff + u * G4_SPAN;
    if (span0 >= klim) continue;
    float sc[G4_R][2];
#pragma unroll
    for (int r = 0; r < G4_R; ++r) {
      const uint32_t sw = (u < 2) ? b.s[r].x : b.s[r].y;
      sc[r][0] = e4m3_to_float(sw >> ((u & 1) * 16));
      sc[r][1] = e4m3_to_float(sw >> ((u & 1) * 16 + 8));
    }
    __half2 s0[G4_R][M], s1[G4_R][M];                         // two chains per (row, activation row) inside a block
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      if ((wi & 1) == 0) {
#pragma unroll
        for (int r = 0; r < G4_R; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) { s0[r][m] = __float2half2_rn(0.f); s1[r][m] = __float2half2_rn(0.f); }
      }
      __half2 wh[G4_R][4];
#pragma unroll
      for (int r = 0; r < G4_R; ++r) {
        const uint32_t word = wi == 0 ? b.w[r][u].x : wi == 1 ? b.w[r][u].y : wi == 2 ? b.w[r][u].z : b.w[r][u].w;
        e2m1x8_to_half2x4(word, wh[r], one);
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)m * kc + g4_xpos(span0, lane, wi));
        const __half2 x0 = *reinterpret_cast<const __half2*>(&xv.x), x1 = *reinterpret_cast<const __half2*>(&xv.y);
        const __half2 x2 = *reinterpret_cast<const __half2*>(&xv.z), x3 = *reinterpret_cast<const __half2*>(&xv.w);
#pragma unroll
        for (int r = 0; r < G4_R; ++r) {
          s0[r][m] = __hfma2(wh[r][0], x0, s0[r][m]);
          s1[r][m] = __hfma2(wh[r][1], x1, s1[r][m]);
          s0[r][m] = __hfma2(wh[r][2], x2, s0[r][m]);
          s1[r][m] = __hfma2(wh[r][3], x3, s1[r][m]);
        }
      }
      if (wi & 1) {                                           // words 0,1 = block 0 of this lane, words 2,3 = block 1
#pragma unroll
        for (int r = 0; r < G4_R; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const float2 f = __half22float2(__hadd2(s0[r][m], s1[r][m]));
            acc[r][m] = fmaf(f.x + f.y, sc[r][wi >> 1], acc[r][m]);
          }
      }
    }
  }
}

// Stage X[:, k0:k0+kc) as f16 scaled by 2^s of its row (normalised when asked), in the chunk order `g4_xpos` reads;
// positions past K are zero. A thread writes one 16-byte chunk: the 8 activations of one weight word as the pairs
// (j, j + 4).
template <int M>
__device__ __forceinline__ void g4_stage(const Gemv4Args& a, __half* xs, const float* rscale, const float* xpow, int k0,
                                         int kc) {
  for (int idx = threadIdx.x; idx < M * (kc / 8); idx += blockDim.x) {
    const int m = idx / (kc / 8), c = idx % (kc / 8);
    const int k = k0 + c * 8;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (m < a.M && k < a.K) {
      uint4 xv = *reinterpret_cast<const uint4*>(a.X + (size_t)m * a.ldx + k);
      uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
      const float p = xpow[m];
      if (a.norm_w) {
        uint4 wv = __ldg(reinterpret_cast<const uint4*>(a.norm_w + k));
        uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
        const float r = rscale[m];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // round through bf16 first so this path sees the same normalised activations as the bf16 kernels
          v[2 * j] = bf2f(f2bf(bf_lo(xu[j]) * r * (bf_lo(wu[j]) + 1.f))) * p;
          v[2 * j + 1] = bf2f(f2bf(bf_hi(xu[j]) * r * (bf_hi(wu[j]) + 1.f))) * p;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) { v[2 * j] = bf_lo(xu[j]) * p; v[2 * j + 1] = bf_hi(xu[j]) * p; }
      }
    }
    __half2 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __floats2half2_rn(v[j], v[j + 4]);
    uint4 ov;
    ov.x = *reinterpret_cast<uint32_t*>(&o[0]); ov.y = *reinterpret_cast<uint32_t*>(&o[1]);
    ov.z = *reinterpret_cast<uint32_t*>(&o[2]); ov.w = *reinterpret_cast<uint32_t*>(&o[3]);
    const int rel = c * 8;                                    // position inside the staged chunk
    const int span0 = rel / G4_SPAN * G4_SPAN, r = rel % G4_SPAN;
    *reinterpret_cast<uint4*>(xs + (size_t)m * kc + g4_xpos(span0, r / 32, (r % 32) / 8)) = ov;
  }
}

// Per row: rscale[m] = rsqrt(mean(x_m^2) + eps) (when a norm weight is given, else 1), xpow[m] = 2^s, the power of
// two the staged row is multiplied by (s = min(14, floor(log2(32768 / max|staged x|)))), and xinv[m] = 2^(14 - s)
// for the epilogue. All threads of the CTA take part.
template <int M>
__device__ __forceinline__ void g4_row_scales(const Gemv4Args& a, float* rscale, float* xpow, float* xinv, float* scratch) {
  for (int m = 0; m < M; ++m) {
    float ss = 0.f, am = 0.f;
    if (m < a.M) {
      for (int k = threadIdx.x * 8; k < a.K; k += blockDim.x * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(a.X + (size_t)m * a.ldx + k);
        uint32_t u[4] = {v.x, v.y, v.z, v.w};
        if (a.norm_w) {
          uint4 wv = __ldg(reinterpret_cast<const uint4*>(a.norm_w + k));
          uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float x0 = bf_lo(u[j]), x1 = bf_hi(u[j]);
            ss += x0 * x0 + x1 * x1;
            am = fmaxf(am, fmaxf(fabsf(x0 * (bf_lo(wu[j]) + 1.f)), fabsf(x1 * (bf_hi(wu[j]) + 1.f))));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) am = fmaxf(am, fmaxf(fabsf(bf_lo(u[j])), fabsf(bf_hi(u[j]))));
        }
      }
    }
    const float tot = block_sum(ss, scratch);
    const float amax = block_max(am, scratch);
    if (threadIdx.x == 0) {
      const float r = a.norm_w ? rsqrtf(tot / (float)a.K + a.eps) : 1.f;
      rscale[m] = r;
      const float top = amax * r * 1.01f;                      // the staged values are rounded to bf16 first: a margin
      int s = 14;
      if (top > 0.f) {
        int e;
        frexpf(32768.f / top, &e);                             // 32768 / top = f * 2^e, f in [0.5, 1)
        s = min(14, max(-14, e - 1));
      }
      xpow[m] = ldexpf(1.f, s);
      xinv[m] = ldexpf(1.f, 14 - s);
    }
  }
  __syncthreads();
}

template <int M, bool SWIGLU, class Store>
__device__ __forceinline__ void gemv4_main(const Gemv4Args& a, __half* xs, float* rscale, float* scratch, Store store) {
  __shared__ float xpow[M], xinv[M];
  const int warp = threadIdx.x >> 5;
  const int row0 = blockIdx.x * a.rows_per_cta;
  const int row_end = min(a.N, row0 + a.rows_per_cta);
  const int nchunks = (a.K + a.kc - 1) / a.kc;
  constexpr int RW = SWIGLU ? 1 : G4_R;
  int n = row0 + warp * RW;

  pdl_launch_dependents();
  Batch4 b;
  int rows[G4_R];
  g4_rows<SWIGLU>(a, rows, n);
  g4_load(b, a, rows, 0);
  pdl_wait();

  g4_row_scales<M>(a, rscale, xpow, xinv, scratch);

  const int passes = (row_end - row0 + G4_WARPS * RW - 1) / (G4_WARPS * RW);
  for (int pass = 0; pass < passes; ++pass, n += G4_WARPS * RW) {
    const bool active = n < row_end;
    float acc[G4_R][M] = {};
    for (int c = 0; c < nchunks; ++c) {
      const int k0 = c * a.kc;
      if (nchunks > 1 || pass == 0) {
        __syncthreads();
        g4_stage<M>(a, xs, rscale, xpow, k0, a.kc);
        __syncthreads();
      }
      if (active) {
        const int klim = min(a.kc, (a.K - k0 + G4_SPAN - 1) / G4_SPAN * G4_SPAN);
        for (int base = 0; base < klim; base += G4_BATCH) {
          g4_consume<M>(acc, b, xs, a.kc, base, klim, (uint32_t)a.one);
          const int knext = k0 + base + G4_BATCH;
          if (knext < a.K) {
            g4_load(b, a, rows, knext);
          } else if (c == nchunks - 1 && base + G4_BATCH >= klim && n + G4_WARPS * RW < row_end) {
            g4_rows<SWIGLU>(a, rows, n + G4_WARPS * RW);
            g4_load(b, a, rows, 0);
          }
        }
      }
    }
    if (active) {
#pragma unroll
      for (int r = 0; r < G4_R; ++r) {
        const int wr = SWIGLU ? (min(n, a.N - 1) + r * a.N) : min(n + r, a.N - 1);
        const float gs = a.row_alpha ? __ldg(a.row_alpha + wr) : a.global_scale;
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]) * (gs * xinv[m]);
      }
      store(acc, n);
    }
  }
}

template <int M, bool SWIGLU>
__global__ void __launch_bounds__(G4_THREADS, (M == 1 ? 3 : 2)) gemv_nvfp4_kernel(Gemv4Args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  __shared__ float scratch[32];
  __shared__ float rscale[M];
  const int row_end = min(a.N, (int)(blockIdx.x + 1) * a.rows_per_cta);
  gemv4_main<M, SWIGLU>(a, xs, rscale, scratch, [&](float (&acc)[G4_R][M], int n) {
    if ((threadIdx.x & 31) != 0) return;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      if (m >= a.M) break;
      if (SWIGLU) {
        float v = siluf_(acc[0][m]) * acc[1][m];
        reinterpret_cast<__nv_bfloat16*>(a.Y)[(size_t)m * a.ldy + n] = f2bf(v);
      } else {
#pragma unroll
        for (int r = 0; r < G4_R; ++r) {
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

// Row-parallel projection under tensor parallelism: GEMV partial -> one-shot all-reduce over peers -> + residual.
template <int M>
__global__ void __launch_bounds__(G4_THREADS, 2) gemv_nvfp4_allreduce_kernel(Gemv4Args a, CommBuf cb) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  float* tile = reinterpret_cast<float*>(smem_raw + (size_t)M * a.kc * sizeof(__half));      // [M][rows_per_cta]
  __shared__ float scratch[32];
  __shared__ float rscale[M];
  const int row0 = blockIdx.x * a.rows_per_cta;
  const int row_end = min(a.N, row0 + a.rows_per_cta);
  const int nrows = row_end - row0;
  const int rpc = a.rows_per_cta;
  for (int i = threadIdx.x; i < M * rpc; i += blockDim.x) tile[i] = 0.f;
  __syncthreads();
  gemv4_main<M, false>(a, xs, rscale, scratch, [&](float (&acc)[G4_R][M], int n) {
    if ((threadIdx.x & 31) != 0) return;
#pragma unroll
    for (int r = 0; r < G4_R; ++r)
      if (n + r < row_end)
#pragma unroll
        for (int m = 0; m < M; ++m) tile[m * rpc + (n + r - row0)] = acc[r][m];
  });
  __syncthreads();
  const uint32_t epoch = comm_epoch_begin(cb);
  cta_exchange_sum(cb, tile, M * rpc, (long)blockIdx.x * M * rpc, epoch);
  __syncthreads();
  for (int i = threadIdx.x; i < a.M * nrows; i += blockDim.x) {
    int m = i / nrows, j = i % nrows;
    float v = tile[m * rpc + j];
    size_t o = (size_t)m * a.ldy + row0 + j;
    if (a.res) v += bf2f(a.res[o]);
    reinterpret_cast<__nv_bfloat16*>(a.Y)[o] = f2bf(v);
  }
  comm_epoch_end(cb, epoch);
}

template <typename Kern, typename... Args>
static int g4_launch(Kern kern, int grid, size_t smem, cudaStream_t s, Args... args) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G4_SMEM + 16 * 1024);
  if (e != cudaSuccess) return (int)e;
  return (int)launch_pdl(kern, dim3(grid), dim3(G4_THREADS), smem, s, args...);
}

}  // namespace fb

using namespace fb;

static int fill_args(Gemv4Args& a, void* Y, const void* X, const void* Wq, const void* Sc, float gs,
                     const void* norm_w, const void* res, int M, int N, int K, long ldx, long ldy, long sc_stride,
                     float eps, int out_f32, const float* row_alpha) {
  if (M > 8 || (K % 32) != 0 || (ldx % 8) != 0) return -1;
  a.X = (const __nv_bfloat16*)X; a.Wq = (const uint8_t*)Wq; a.Sc = (const uint8_t*)Sc; a.global_scale = gs;
  a.row_alpha = row_alpha;
  a.norm_w = (const __nv_bfloat16*)norm_w; a.res = (const __nv_bfloat16*)res; a.Y = Y; a.M = M; a.N = N; a.K = K;
  a.ldx = ldx; a.ldy = ldy; a.sc_stride = sc_stride; a.eps = eps; a.out_f32 = out_f32; a.rows_per_cta = 0; a.kc = 0;
  a.one = 1;
  return 0;
}

// mode: 0 plain (+res), 1 SwiGLU (2N weight rows: gate then up)
extern "C" int fb_gemv_nvfp4(void* Y, const void* X, const void* Wq, const void* Sc, float global_scale,
                             const void* norm_w, const void* res, int M, int N, int K, long ldx, long ldy,
                             long sc_stride, float eps, int out_f32, int mode, int sm_count, const float* row_alpha,
                             cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  Gemv4Args a;
  int rc = fill_args(a, Y, X, Wq, Sc, global_scale, norm_w, res, M, N, K, ldx, ldy, sc_stride, eps, out_f32, row_alpha);
  if (rc) return rc;
  if (sm_count <= 0) sm_count = 148;
  const int Mt = M == 1 ? 1 : (M == 2 ? 2 : (M <= 4 ? 4 : 8));
  a.kc = gemv4_chunk_len(Mt, K);
  const int group = G4_WARPS * (mode == 1 ? 1 : G4_R);
  int rpc = (N + sm_count * 3 - 1) / (sm_count * 3);
  a.rows_per_cta = (rpc + group - 1) / group * group;
  const int grid = (N + a.rows_per_cta - 1) / a.rows_per_cta;
  const size_t smem = (size_t)Mt * a.kc * sizeof(__half);
#define G4_GO(MV)                                                                                  \
  return mode == 1 ? g4_launch(gemv_nvfp4_kernel<MV, true>, grid, smem, s, a)                       \
                   : g4_launch(gemv_nvfp4_kernel<MV, false>, grid, smem, s, a);
  if (Mt == 1) { G4_GO(1) } else if (Mt == 2) { G4_GO(2) } else if (Mt == 4) { G4_GO(4) } else { G4_GO(8) }
#undef G4_GO
}

extern "C" int fb_gemv_nvfp4_allreduce(void* Y, const void* X, const void* Wq, const void* Sc, float global_scale,
                                       const void* res, int M, int N, int K, long ldx, long ldy, long sc_stride,
                                       const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                                       uint32_t* epochs, int* status, unsigned spin_limit, int max_resident,
                                       const float* row_alpha, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  Gemv4Args a;
  int rc = fill_args(a, Y, X, Wq, Sc, global_scale, nullptr, res, M, N, K, ldx, ldy, sc_stride, 0.f, 0, row_alpha);
  if (rc) return rc;
  if (world > COMM_MAX_RANKS) return -1;
  CommBuf cb;
  fill_comm(cb, peers, rank, world, max_ctas, slot_floats, epochs, status, spin_limit);
  const int Mt = M == 1 ? 1 : (M == 2 ? 2 : (M <= 4 ? 4 : 8));
  a.kc = gemv4_chunk_len(Mt, K);
  const int group = G4_WARPS * G4_R;
  int rpc = (N + max_resident - 1) / max_resident;
  a.rows_per_cta = (rpc + group - 1) / group * group;
  const int grid = (N + a.rows_per_cta - 1) / a.rows_per_cta;
  if (grid > max_resident || grid > max_ctas) return -7;
  if ((long)grid * Mt * a.rows_per_cta * 2 > slot_floats - COMM_TOP_RESERVE) return -8;
  const size_t smem = (size_t)Mt * a.kc * sizeof(__half) + (size_t)Mt * a.rows_per_cta * sizeof(float);
  if (Mt == 1) return g4_launch(gemv_nvfp4_allreduce_kernel<1>, grid, smem, s, a, cb);
  if (Mt == 2) return g4_launch(gemv_nvfp4_allreduce_kernel<2>, grid, smem, s, a, cb);
  if (Mt == 4) return g4_launch(gemv_nvfp4_allreduce_kernel<4>, grid, smem, s, a, cb);
  return g4_launch(gemv_nvfp4_allreduce_kernel<8>, grid, smem, s, a, cb);
}
