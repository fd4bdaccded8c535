// Small-M weight-streaming dot-product core shared by the plain GEMV kernels and the fused
// GEMV + all-reduce kernels. Y[m][n] = sum_k X[m][k] * W[n][k] for M <= 8 activation rows.
//
// The reference's decode GEMVs (`fe_gemv_bf16` `kernels/k-core/src/gemm.rs:149`, the EXL3 family
// `kernels/k-exl3/src/gemv.rs:227`) are bandwidth kernels; on a B200 the same job needs ~35 KB of loads in
// flight per SM to cover HBM3e latency, so every lane keeps R x U independent 16-byte weight loads in flight
// and the activations are staged once per CTA in shared memory (normalised on the way in when asked).
//
// A lane accumulates its k positions in increasing order whatever M is, so a row's bits do not depend on
// how many other rows ride in the same launch (the reference's batch-invariance rule, `TP2.md:99-105`).
#pragma once
#include "common.cuh"

namespace fb {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int GEMV_U = 4;                 // 16-byte loads in flight per lane per weight row
constexpr int GEMV_STEP = 256;            // k elements a warp covers per load (32 lanes x 8 bf16)
constexpr int GEMV_SMEM_BYTES = 96 * 1024;

struct GemvArgs {
  const __nv_bfloat16* X;       // [M][ldx]
  const __nv_bfloat16* W;       // [N or 2N][K]
  const __nv_bfloat16* norm_w;  // [K] or null: RMSNorm prologue on X rows
  const __nv_bfloat16* res;     // [M][ldy] or null: residual added in the epilogue
  void* Y;                      // [M][ldy] bf16, or fp32 when out_f32
  int M, N, K;
  long ldx, ldy;
  float eps;
  int centred;
  int out_f32;
  int rows_per_cta;
  int kc;                       // staged chunk length (multiple of GEMV_STEP)
};

__host__ __device__ inline int gemv_chunk_len(int M, int K) {
  int kpad = (K + GEMV_STEP - 1) / GEMV_STEP * GEMV_STEP;
  int cap = (GEMV_SMEM_BYTES / 2 / M) / (GEMV_STEP * GEMV_U) * (GEMV_STEP * GEMV_U);
  return kpad < cap ? kpad : cap;
}

// Stage X[:, k0:k0+kc) into shared memory as bf16, applying the RMSNorm scale when present.
template <int M>
__device__ __forceinline__ void gemv_stage_x(const GemvArgs& a, __nv_bfloat16* xs, const float* rscale, int k0,
                                             int kc) {
  for (int idx = threadIdx.x; idx < M * (kc / 8); idx += blockDim.x) {
    int m = idx / (kc / 8), c = idx % (kc / 8);
    int k = k0 + c * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m < a.M && k < a.K) {
      v = *reinterpret_cast<const uint4*>(a.X + (size_t)m * a.ldx + k);
      if (a.norm_w) {
        uint4 wv = __ldg(reinterpret_cast<const uint4*>(a.norm_w + k));
        uint32_t xu[4] = {v.x, v.y, v.z, v.w}, wu[4] = {wv.x, wv.y, wv.z, wv.w}, o[4];
        float r = rscale[m];
        float add = a.centred ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          o[j] = pack_bf2(bf_lo(xu[j]) * r * (bf_lo(wu[j]) + add), bf_hi(xu[j]) * r * (bf_hi(wu[j]) + add));
        v = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    *reinterpret_cast<uint4*>(xs + (size_t)m * kc + c * 8) = v;
  }
}

// rscale[m] = rsqrt(mean(x_m^2) + eps) for every row (all threads of the CTA take part)
template <int M>
__device__ __forceinline__ void gemv_row_scales(const GemvArgs& a, float* rscale, float* scratch) {
  for (int m = 0; m < M; ++m) {
    float ss = 0.f;
    if (m < a.M) {
      for (int k = threadIdx.x * 8; k < a.K; k += blockDim.x * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(a.X + (size_t)m * a.ldx + k);
        uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { float x0 = bf_lo(u[j]), x1 = bf_hi(u[j]); ss += x0 * x0 + x1 * x1; }
      }
    }
    float tot = block_sum(ss, scratch);
    if (threadIdx.x == 0) rscale[m] = rsqrtf(tot / (float)a.K + a.eps);
  }
  __syncthreads();
}

// Issue the R x U weight loads of the batch starting at k = base (elements, relative to wrow).
template <int R>
__device__ __forceinline__ void gemv_load_batch(uint4 (&wv)[R][GEMV_U], const __nv_bfloat16* const (&wrow)[R], int base,
                                                int kvalid) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int u = 0; u < GEMV_U; ++u) {
    int k = base + u * GEMV_STEP + lane * 8;
#pragma unroll
    for (int r = 0; r < R; ++r) wv[r][u] = (k < kvalid) ? ldg_stream(wrow[r] + k) : make_uint4(0, 0, 0, 0);
  }
}

// acc += W batch (registers) x staged activations. koff = position of the batch inside the staged chunk.
template <int M, int R>
__device__ __forceinline__ void gemv_consume_batch(float (&acc)[R][M], const uint4 (&wv)[R][GEMV_U],
                                                   const __nv_bfloat16* xs, int kc, int koff) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int u = 0; u < GEMV_U; ++u) {
    const int k = koff + u * GEMV_STEP + lane * 8;
    if (k >= kc) continue;
    float wf[R][8];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint32_t wu[4] = {wv[r][u].x, wv[r][u].y, wv[r][u].z, wv[r][u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { wf[r][2 * j] = bf_lo(wu[j]); wf[r][2 * j + 1] = bf_hi(wu[j]); }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)m * kc + k);
      uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
      float xf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { xf[2 * j] = bf_lo(xu[j]); xf[2 * j + 1] = bf_hi(xu[j]); }
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[r][m] = fmaf(wf[r][j], xf[j], acc[r][m]);
      }
    }
  }
}

template <int R, bool SWIGLU>
__device__ __forceinline__ void gemv_row_ptrs(const GemvArgs& a, const __nv_bfloat16* (&wrow)[R], int n) {
#pragma unroll
  for (int r = 0; r < R; ++r) {
    int rr = SWIGLU ? (min(n, a.N - 1) + r * a.N) : min(n + r, a.N - 1);
    wrow[r] = a.W + (size_t)rr * a.K;
  }
}

// The whole GEMV main loop of one CTA, shared by the plain and the fused-collective kernels.
//
// The weight batch a warp will consume next is always already in flight: the first one is requested before
// griddepcontrol.wait (weights never depend on the previous kernel of the stream, so under programmatic
// dependent launch those loads overlap its tail and this kernel's own prologue), and each later one right
// after the previous batch was consumed, across row-group boundaries too. `store(acc, n)` is called by every
// lane of the warp with the warp-reduced sums of row group n.
// How the main loop learns that its activations are ready. As a kernel of its own: programmatic dependent launch.
struct GemvPdlWait {
  __device__ __forceinline__ void before_loads() const { pdl_launch_dependents(); }
  __device__ __forceinline__ void wait() const { pdl_wait(); }
};

template <int M, int R, bool SWIGLU, int NWARPS, class Store, class Wait>
__device__ __forceinline__ void gemv_main_w(const GemvArgs& a, __nv_bfloat16* xs, float* rscale, float* scratch,
                                            Store store, Wait waiter, unsigned long long* wait_stamp = nullptr) {
  constexpr int GEMV_WARPS = NWARPS;                   // (shadows the default: row groups stride by this CTA's warps)
  const int warp = threadIdx.x >> 5;
  const int row0 = blockIdx.x * a.rows_per_cta;
  const int row_end = min(a.N, row0 + a.rows_per_cta);
  const int nchunks = (a.K + a.kc - 1) / a.kc;
  constexpr int RW = SWIGLU ? 1 : R;
  constexpr int BATCH = GEMV_STEP * GEMV_U;
  int n = row0 + warp * RW;

  waiter.before_loads();
  uint4 wv[R][GEMV_U];
  const __nv_bfloat16* wrow[R];
  gemv_row_ptrs<R, SWIGLU>(a, wrow, n);
  gemv_load_batch<R>(wv, wrow, 0, a.K);
  waiter.wait();
  if (wait_stamp != nullptr && threadIdx.x == 0)       // profiling: when the previous kernel of the stream had finished
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(*wait_stamp));

  if (a.norm_w) gemv_row_scales<M>(a, rscale, scratch);

  if (nchunks == 1) {
    gemv_stage_x<M>(a, xs, rscale, 0, a.kc);
    __syncthreads();
    for (; n < row_end; n += GEMV_WARPS * RW) {
      float acc[R][M] = {};
      for (int base = 0; base < a.kc; base += BATCH) {
        gemv_consume_batch<M, R>(acc, wv, xs, a.kc, base);
        if (base + BATCH < a.kc) {
          gemv_load_batch<R>(wv, wrow, base + BATCH, a.K);
        } else if (n + GEMV_WARPS * RW < row_end) {
          gemv_row_ptrs<R, SWIGLU>(a, wrow, n + GEMV_WARPS * RW);
          gemv_load_batch<R>(wv, wrow, 0, a.K);
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
      store(acc, n);
    }
  } else {
    // K does not fit one staged chunk: per pass one row group per warp, the chunks re-staged inside the pass
    // (the loop bounds are uniform over the CTA because of the barriers)
    const int passes = (row_end - row0 + GEMV_WARPS * RW - 1) / (GEMV_WARPS * RW);
    for (int pass = 0; pass < passes; ++pass, n += GEMV_WARPS * RW) {
      const bool active = n < row_end;
      float acc[R][M] = {};
      for (int c = 0; c < nchunks; ++c) {
        const int k0 = c * a.kc;
        __syncthreads();
        gemv_stage_x<M>(a, xs, rscale, k0, a.kc);
        __syncthreads();
        if (active) {
          for (int base = 0; base < a.kc; base += BATCH) {
            gemv_consume_batch<M, R>(acc, wv, xs, a.kc, base);
            const int knext = k0 + base + BATCH;
            if (knext < a.K) {
              gemv_load_batch<R>(wv, wrow, knext, a.K);
            } else if (c == nchunks - 1 && base + BATCH >= a.kc && n + GEMV_WARPS * RW < row_end) {
              gemv_row_ptrs<R, SWIGLU>(a, wrow, n + GEMV_WARPS * RW);
              gemv_load_batch<R>(wv, wrow, 0, a.K);
            }
          }
        }
      }
      if (active) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
        store(acc, n);
      }
    }
  }
}

template <int M, int R, bool SWIGLU, class Store>
__device__ __forceinline__ void gemv_main(const GemvArgs& a, __nv_bfloat16* xs, float* rscale, float* scratch,
                                          Store store, unsigned long long* wait_stamp = nullptr) {
  gemv_main_w<M, R, SWIGLU, GEMV_WARPS>(a, xs, rscale, scratch, store, GemvPdlWait(), wait_stamp);
}

}  // namespace fb
