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
  // split-K over blockIdx.y: partial tiles (and partial sums of squares) go to `ws`, the last CTA of a tile to arrive
  // adds them up in split order (deterministic) and runs the epilogue; counters clean themselves
  int split, klen;                // klen = k values per split (multiple of 32)
  float* ws;                      // [tiles][split][16 RT * 8 MT * (1 or 2) + 8 MT]
  int* counters;                  // [tiles]
};

__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int GM2_WARPS = 8;
template <int MT> struct Gm2 {                       // MT = 8-token tiles
  static constexpr int KC = MT == 1 ? 4096 : MT == 2 ? 2048 : 1024;   // k values of x staged per pass
  static constexpr int LDX = KC + 32;                // row stride: 64 bytes off a multiple of 128 -> conflict-free reads
  static constexpr size_t SMEM = (size_t)8 * MT * LDX * 2 + (size_t)GM2_WARPS * 16 * 8 * MT * 4 * 2 + 8 * MT * 4;
};

// One batch of A fragments: U iterations of 32 k for rows g and g + 8 (and the up rows for SwiGLU).
template <int U, bool DUAL>
struct FragBatch {
  uint4 a0[U], a1[U], u0[DUAL ? U : 1], u1[DUAL ? U : 1];
  __device__ __forceinline__ void load(const __nv_bfloat16* wa, const __nv_bfloat16* wb, const __nv_bfloat16* ua,
                                       const __nv_bfloat16* ub, int k, int it, int it1) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (it + u < it1) {
        a0[u] = ldg_stream(wa + k + u * 32);
        a1[u] = ldg_stream(wb + k + u * 32);
        if (DUAL) { u0[u] = ldg_stream(ua + k + u * 32); u1[u] = ldg_stream(ub + k + u * 32); }
      } else {
        a0[u] = a1[u] = make_uint4(0, 0, 0, 0);
        if (DUAL) u0[u] = u1[u] = make_uint4(0, 0, 0, 0);
      }
    }
  }
};

// grid = ceil(N / (16 RT)); 256 threads = RT row tiles x (8 / RT) k slices. DUAL: rows n (gate) and N + n (up), output
// silu(gate) * up. The RMSNorm scale of a token row is a scalar, so it is applied in the epilogue; x is staged as
// x * (1 + w) and its sum of squares is collected on the way (each token row is staged by one warp: deterministic).
template <int MT, int RT, bool DUAL>
__global__ void __launch_bounds__(GM2_WARPS * 32, 2) gemv_mma_kernel(GemvMmaArgs a) {
  using C = Gm2<MT>;
  constexpr int KS = GM2_WARPS / RT;                  // k slices
  constexpr int U = DUAL ? 2 : 4;                     // iterations per load batch
  extern __shared__ __align__(16) unsigned char smem_g2[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_g2);                    // [8 MT][LDX]
  float* red = reinterpret_cast<float*>(smem_g2 + (size_t)8 * MT * C::LDX * 2);     // [2][warps][16][8 MT]
  float* ssq = red + 2 * GM2_WARPS * 16 * 8 * MT;                                   // [8 MT] sums of squares
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rt = warp % RT, ks = warp / RT;
  const int n0 = (blockIdx.x * RT + rt) * 16;
  // weight rows of this thread's fragments (clamped: rows past N are computed and dropped)
  const int ra = min(n0 + g, a.N - 1), rb = min(n0 + g + 8, a.N - 1);
  const __nv_bfloat16* wa = a.w + (size_t)ra * a.K;
  const __nv_bfloat16* wb = a.w + (size_t)rb * a.K;
  const __nv_bfloat16* ua = DUAL ? a.w + (size_t)(a.N + ra) * a.K : nullptr;
  const __nv_bfloat16* ub = DUAL ? a.w + (size_t)(a.N + rb) * a.K : nullptr;
  float acc[MT][4], acu[DUAL ? MT : 1][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (DUAL) acu[i][j] = 0.f; }
  float ss_row[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) ss_row[i] = 0.f;
  const int kbeg = blockIdx.y * a.klen, kend = min(a.K, kbeg + a.klen);     // this CTA's share of K

  // first batch of weights is independent of the previous kernel's output: issue it before waiting for it
  FragBatch<U, DUAL> cur, nxt;
  {
    const int kn = min(C::KC, kend - kbeg);
    const int per = ((kn / 32) + KS - 1) / KS;
    const int it0 = ks * per, it1 = min(kn / 32, it0 + per);
    cur.load(wa, wb, ua, ub, kbeg + it0 * 32 + t * 8, it0, it1);
  }
  pdl_wait();
  for (int kc = kbeg; kc < kend; kc += C::KC) {
    const int kn = min(C::KC, kend - kc);
    __syncthreads();                                    // previous pass is done with xs
    // warp `warp` stages token rows warp, warp + 8, ...
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int m = warp + 8 * i;
      float ss = 0.f;
      for (int c8 = lane * 8; c8 < kn; c8 += 256) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < a.M) {
          v = *reinterpret_cast<const uint4*>(a.x + (size_t)m * a.ldx + kc + c8);
          if (a.norm_w) {
            const uint4 nw = *reinterpret_cast<const uint4*>(a.norm_w + kc + c8);
            uint32_t u[4] = {v.x, v.y, v.z, v.w};
            const uint32_t wv[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lo = bf_lo(u[j]), hi = bf_hi(u[j]);
              ss = fmaf(lo, lo, fmaf(hi, hi, ss));
              u[j] = pack_bf2(lo * (1.f + bf_lo(wv[j])), hi * (1.f + bf_hi(wv[j])));
            }
            v = make_uint4(u[0], u[1], u[2], u[3]);
          }
        }
        *reinterpret_cast<uint4*>(xs + (size_t)m * C::LDX + c8) = v;
      }
      ss_row[i] += warp_sum(ss);
    }
    __syncthreads();
    // this warp's k range inside the pass, in steps of 32 (two mma k steps), walked in batches of U with the next
    // batch (or the first batch of the next pass) always in flight
    const int per = ((kn / 32) + KS - 1) / KS;
    const int it0 = ks * per, it1 = min(kn / 32, it0 + per);
    for (int it = it0; it < it1; it += U) {
      if (it + U < it1) {
        nxt.load(wa, wb, ua, ub, kc + (it + U) * 32 + t * 8, it + U, it1);
      } else if (kc + C::KC < kend) {
        const int kn2 = min(C::KC, kend - kc - C::KC);
        const int per2 = ((kn2 / 32) + KS - 1) / KS;
        const int jt0 = ks * per2, jt1 = min(kn2 / 32, jt0 + per2);
        nxt.load(wa, wb, ua, ub, kc + C::KC + jt0 * 32 + t * 8, jt0, jt1);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int kl = (it + u) * 32 + t * 8;           // local k of this thread's 8 elements (zero fragments past it1)
        if (it + u < it1) {
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            const uint4 B = *reinterpret_cast<const uint4*>(xs + (size_t)(i * 8 + g) * C::LDX + kl);
            mma_bf16_16816(acc[i], cur.a0[u].x, cur.a1[u].x, cur.a0[u].y, cur.a1[u].y, B.x, B.y);
            mma_bf16_16816(acc[i], cur.a0[u].z, cur.a1[u].z, cur.a0[u].w, cur.a1[u].w, B.z, B.w);
            if (DUAL) {
              mma_bf16_16816(acu[i], cur.u0[u].x, cur.u1[u].x, cur.u0[u].y, cur.u1[u].y, B.x, B.y);
              mma_bf16_16816(acu[i], cur.u0[u].z, cur.u1[u].z, cur.u0[u].w, cur.u1[u].w, B.z, B.w);
            }
          }
        }
      }
      cur = nxt;
    }
    if (it0 >= it1) cur = nxt;                          // a slice with no work in this pass still rotates the buffers
  }
  if (a.norm_w && lane == 0) {
#pragma unroll
    for (int i = 0; i < MT; ++i) ssq[warp + 8 * i] = ss_row[i];
  }
  // partial sums of the warps -> shared memory, summed in slice order
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
  constexpr int TILE = RT * 16 * 8 * MT;                // outputs of a CTA
  constexpr int REC = TILE * (DUAL ? 2 : 1) + 8 * MT;   // floats per (tile, split) record in the workspace
  __shared__ int last_s;
  if (a.split > 1) {
    // slice sums of this CTA -> workspace record; the last CTA of the tile adds the records in split order
    float* rec = a.ws + ((size_t)blockIdx.x * a.split + blockIdx.y) * REC;
    for (int i = threadIdx.x; i < TILE; i += blockDim.x) {
      const int m = i / (RT * 16), rr = i % (RT * 16), tile = rr / 16, r = rr % 16;
      float gsum = 0.f, usum = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < KS; ++s2) {
        const int wdx = s2 * RT + tile;
        gsum += red[((size_t)wdx * 16 + r) * 8 * MT + m];
        if (DUAL) usum += red[((size_t)(GM2_WARPS + wdx) * 16 + r) * 8 * MT + m];
      }
      rec[i] = gsum;
      if (DUAL) rec[TILE + i] = usum;
    }
    if (threadIdx.x < 8 * MT) rec[TILE * (DUAL ? 2 : 1) + threadIdx.x] = a.norm_w ? ssq[threadIdx.x] : 0.f;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_s = atomicAdd(&a.counters[blockIdx.x], 1) == a.split - 1 ? 1 : 0;
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    if (threadIdx.x == 0) a.counters[blockIdx.x] = 0;
  }
  for (int i = threadIdx.x; i < TILE; i += blockDim.x) {
    const int m = i / (RT * 16), rr = i % (RT * 16);    // consecutive threads -> consecutive output features
    const int tile = rr / 16, r = rr % 16;
    const int n = (blockIdx.x * RT + tile) * 16 + r;
    if (m >= a.M || n >= a.N) continue;
    float gsum = 0.f, usum = 0.f, ssm = 0.f;
    if (a.split > 1) {
      const float* rec0 = a.ws + (size_t)blockIdx.x * a.split * REC;
      for (int sp = 0; sp < a.split; ++sp) {
        const float* rec = rec0 + (size_t)sp * REC;
        gsum += __ldcg(rec + i);
        if (DUAL) usum += __ldcg(rec + TILE + i);
        ssm += __ldcg(rec + TILE * (DUAL ? 2 : 1) + m);
      }
    } else {
#pragma unroll
      for (int s2 = 0; s2 < KS; ++s2) {
        const int wdx = s2 * RT + tile;
        gsum += red[((size_t)wdx * 16 + r) * 8 * MT + m];
        if (DUAL) usum += red[((size_t)(GM2_WARPS + wdx) * 16 + r) * 8 * MT + m];
      }
      ssm = a.norm_w ? ssq[m] : 0.f;
    }
    if (a.norm_w) {
      const float rs = rsqrtf(ssm / (float)a.K + a.eps);
      gsum *= rs;
      usum *= rs;
    }
    float v = DUAL ? siluf_(gsum) * usum : gsum;
    if (a.res) v += bf2f(a.res[(size_t)m * a.ldy + n]);
    if (a.out_f32) reinterpret_cast<float*>(a.y)[(size_t)m * a.ldy + n] = v;
    else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)m * a.ldy + n] = f2bf(v);
  }
}

template <int MT, int RT, bool DUAL>
static int launch_g2(GemvMmaArgs a, int split, float* ws, long ws_floats, int* counters, int n_counters, cudaStream_t s) {
  static bool done = false;
  if (!done) {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<MT, RT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Gm2<MT>::SMEM);
    if (e != cudaSuccess) return (int)e;
    done = true;
  }
  const int tiles = (a.N + 16 * RT - 1) / (16 * RT);
  constexpr long REC = (long)RT * 16 * 8 * MT * (DUAL ? 2 : 1) + 8 * MT;
  if (split > 1 && (!ws || !counters || (long)tiles * split * REC > ws_floats || tiles > n_counters)) split = 1;
  a.split = split;
  a.klen = ((a.K / 32 + split - 1) / split) * 32;
  a.ws = ws; a.counters = counters;
  return (int)launch_pdl(gemv_mma_kernel<MT, RT, DUAL>, dim3(tiles, split), dim3(GM2_WARPS * 32), Gm2<MT>::SMEM, s, a);
}

// Row tiles per CTA (RT x 16 weight rows) and k split. Two CTAs are resident per SM; a CTA first stages its k range of
// x (8 * MT rows) and then streams its weight rows, so what a launch costs is roughly
//   (resident slots / slots actually filled, counting a nearly empty last wave as a whole one)
//   x (1 + (staged x bytes + a fixed per-CTA cost) / weight bytes per CTA).
// Measured on B200 at N 5120, K 17408 (the 27B down projection, 4 rows): 16-row tiles split in two (640 CTAs, 278 KB of
// weights against 139 KB of x each) took 70 us, where one row took 52 us on the SIMT kernel; 64-row tiles split in three
// (240 CTAs, 745 KB against 93 KB) fill one wave.
template <int MT, bool DUAL>
static int pick_rt(const GemvMmaArgs& a, int sm_count, float* ws, long ws_floats, int* counters, int n_counters,
                   cudaStream_t s) {
  const int slots = 2 * sm_count;
  int best_rt = 1, best_split = 1;
  double best = 1e30;
  for (int rt = 4; rt >= 1; rt >>= 1) {
    const int tiles = (a.N + 16 * rt - 1) / (16 * rt);
    int split = 1;
    if (tiles < slots) {
      split = slots / tiles;
      split = min(split, min(8, a.K / 2048));
      split = max(split, 1);
      while (split > 1 && (long)(split - 1) * (((a.K / 32 + split - 1) / split) * 32) >= a.K) --split;
    }
    const long ctas = (long)tiles * split;
    const long waves = (ctas + slots - 1) / slots;
    const double fill = (double)ctas / (double)(waves * slots);
    const double klen = (double)a.K / split;
    const double wbytes = 16.0 * rt * klen * 2.0 * (DUAL ? 2 : 1), xbytes = 8.0 * MT * klen * 2.0;
    const double cost = (1.0 / fill) * (1.0 + (xbytes + 65536.0 + (split > 1 ? 16384.0 : 0.0)) / wbytes);
    if (cost < best) { best = cost; best_rt = rt; best_split = split; }
  }
  if (best_rt == 4) return launch_g2<MT, 4, DUAL>(a, best_split, ws, ws_floats, counters, n_counters, s);
  if (best_rt == 2) return launch_g2<MT, 2, DUAL>(a, best_split, ws, ws_floats, counters, n_counters, s);
  return launch_g2<MT, 1, DUAL>(a, best_split, ws, ws_floats, counters, n_counters, s);
}

}  // namespace fb

using namespace fb;

// mode 1: SwiGLU (W = [gate rows | up rows], 2N rows). M <= 32, K % 32 == 0, ldx % 8 == 0.
extern "C" int fb_gemv_mma(void* y, const void* x, const void* w, const void* norm_w, const void* res, int M, int N, int K,
                           long ldx, long ldy, float eps, int mode, int out_f32, float* ws, long ws_floats, int* counters,
                           int n_counters, int sm_count, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32 || K % 32 || ldx % 8) return -1;
  if (sm_count <= 0) sm_count = 148;
  GemvMmaArgs a;
  a.y = y; a.x = (const __nv_bfloat16*)x; a.w = (const __nv_bfloat16*)w; a.norm_w = (const __nv_bfloat16*)norm_w;
  a.res = (const __nv_bfloat16*)res; a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.eps = eps; a.out_f32 = out_f32;
  a.split = 1; a.klen = K; a.ws = nullptr; a.counters = nullptr;
  const int mt = (M + 7) / 8;
#define FB_G2(MTT, D) return pick_rt<MTT, D>(a, sm_count, ws, ws_floats, counters, n_counters, s)
  if (mode == 1) {
    if (mt == 1) FB_G2(1, true);
    if (mt == 2) FB_G2(2, true);
    if (mt == 3) FB_G2(3, true);
    FB_G2(4, true);
  }
  if (mt == 1) FB_G2(1, false);
  if (mt == 2) FB_G2(2, false);
  if (mt == 3) FB_G2(3, false);
  FB_G2(4, false);
#undef FB_G2
}
