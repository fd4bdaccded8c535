// NVFP4 decode on the block-scaled tensor cores with 16-bit-accurate activations.
//
// Few-row steps (decode, a handful of concurrent streams) are bound by how fast the 4-bit weights stream from HBM.
// A SIMT dequantising GEMV spends about five instructions per weight and stalls at a third of the memory rate, so
// here the weights go from HBM to shared memory by TMA and are multiplied, still packed, by
// `tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X` (128 weight rows x 16 activation columns x K 64, ue4m3 scale
// per 16 values read from TMEM). No thread ever touches a weight.
//
// The tensor core wants e2m1 activations too. A single e2m1 rendering of a row is too coarse, but the instruction's
// N = 16 columns are free when there is one token, so each activation row is expanded into up to three NVFP4 rows:
// the row, the residual the first quantisation left, and the residual of that. Their products are summed in the
// epilogue with their per-term scales (each term's global scale is a quarter of the one before), which brings the
// activation error down to bf16 level while the weights stay untouched.
//
// Structure: persistent CTAs, one TMA producer thread, one MMA thread that owns TMEM, four epilogue warps. The k
// blocks of all 128-row tiles form one linear list that is cut into equal contiguous runs, one per CTA ("stream-K"),
// so every SM streams the same number of bytes whatever N and K are. A run that covers part of a tile's K leaves a
// partial in a workspace slot; the CTA that completes the tile's k-block count sums the slots in CTA order
// (deterministic) and writes the result. The producer fills its ring before `griddepcontrol.wait` (weights do not
// depend on the previous kernel); then all six warps normalise (optional RMSNorm(1+w)) and quantise the k blocks this
// CTA will use, once, into a resident B operand, and the pipeline runs with nothing but TMA and MMA on it.
//
// Stands where the reference's decode-shape NVFP4 kernels do (`fe_gemv_nvfp4*`, `fe_gemm_nvfp4_swiglu` with few
// rows, `kernels/k-fp4/src/lib.rs:167-866`, mma.sync m16n8k64 with scale registers).
#include <cuda.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "api_ext.h"
#include "common.cuh"

namespace fb {

constexpr int T4_BM = 128;               // weight rows per tile
constexpr int T4_BKB = 128;              // bytes of K per stage row = 256 e2m1 values = 4 MMAs of K 64
constexpr int T4_BK = 256;
constexpr int T4_MAX_STAGES = 8;
constexpr int T4_THREADS = 192;
constexpr int T4_A_BYTES = T4_BM * T4_BKB;        // 16 KB
constexpr int T4_SF_ATOM = 512;                   // 128 rows x 4 k-blocks of 16
constexpr int T4_SFA_STAGE = 4 * T4_SF_ATOM;
constexpr int T4_MAX_R = 8;                       // activation rows x terms
constexpr int T4_BN = 16;                         // MMA N; columns >= R hold whatever the next k block holds
constexpr int T4_B_BLOCK = 8 * T4_BKB;            // resident B: 8 rows x 128 bytes per k block
constexpr int T4_SFB_STEP = 8 * 16;               // resident B scales per K-64 step: the first 8 rows of a scale atom
constexpr int T4_SFB_BLOCK = 4 * T4_SFB_STEP;     // ... per k block (the copy to TMEM reads a whole 512-byte atom: rows
                                                  // 8..31 of it are the following steps' bytes, scales of unused columns)

struct T4Args {
  void* Y;
  const __nv_bfloat16* res;
  const __nv_bfloat16* X;
  const __nv_bfloat16* norm_w;
  const uint8_t* sf_a;          // tiled weight scales [row tile][K/64][512]
  const float* row_alpha;       // per weight row tensor scale (nullptr: w_scale for every row)
  float w_scale;
  float eps;
  float* workspace;
  int* counters;
  int* status;
  int M, N, K;
  long ldy, ldx;
  int dual;                     // gate|up pairs with the SwiGLU epilogue
  int terms, R;                 // NVFP4 renderings per activation row; R = M * terms <= 8
  int stages, out_f32;
  int kblocks, items;           // k blocks of 256 per row; tiles (dual: gate/up tile pairs)
  int max_slots;                // workspace slots per item
  int nres;                     // resident k blocks per CTA
  int tmem_cols;
  // L2 prefetch of the weights the next few-row call will stream (nullptr: none): while this kernel drains, waits for
  // its successor to be released and the successor prepares its activations, HBM would otherwise idle
  const unsigned char* pf_w;    // next codes [rows][pf_row_bytes]
  const unsigned char* pf_sf;   // next tiled scales
  long pf_row_bytes, pf_sf_item_bytes, pf_cta_bytes;
  int pf_items, pf_kblocks, pf_grid, pf_n, pf_dual;
  unsigned long long* trace;    // optional [CTA][8] %globaltimer stamps (entry, set-up, dependency, row statistics,
                                // quantised, first stage landed, last MMA issued, epilogue done)
};

__device__ __forceinline__ void t4_stamp(const T4Args& a, int i) {
  if (a.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.trace[(size_t)blockIdx.x * 8 + i] = t;
  }
}

__device__ __forceinline__ bool t4_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < FB_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}

__device__ __forceinline__ void t4_bulk_load(void* smem_dst, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void t4_prefetch_l2(const unsigned char* p, long bytes) {
  for (long o = 0; o < bytes; o += 32768) {
    const uint32_t n = (uint32_t)((bytes - o) < 32768 ? (bytes - o) : 32768);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + o), "r"(n) : "memory");
  }
}

// position of the producer in the CTA's run of (item, k block) units
struct T4Cursor {
  long long u, u1;
  int stage;
  uint32_t phase;
};

__global__ void __launch_bounds__(T4_THREADS, 2)
gemv_nvfp4_tc_kernel(const __grid_constant__ CUtensorMap tmA, T4Args a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[T4_MAX_STAGES], empty_bar[T4_MAX_STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int last_flag_s;
  __shared__ float rn_s[T4_MAX_R], gst_s[T4_MAX_R];        // RMSNorm factor per row (of the segment in the epilogue);
                                                           // global scale per (row, term)
  __shared__ float red_s[T4_THREADS / 32][T4_MAX_R];

  pdl_launch_dependents();
  if (threadIdx.x == 0) t4_stamp(a, 0);
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_a = a.dual ? 2 : 1;
  const int stage_bytes = n_a * (T4_A_BYTES + T4_SFA_STAGE);
  unsigned char* bq = tiles + (size_t)a.stages * stage_bytes;                  // resident B codes (+ one block of pad)
  unsigned char* bsf = bq + (size_t)(a.nres + 1) * T4_B_BLOCK;                 // resident B scales (+ 384 bytes of pad)
  float* ssq = reinterpret_cast<float*>(bsf + (size_t)a.nres * T4_SFB_BLOCK + 384);   // sum of x^2 per (resident block, row)
  const int kt_total = a.K / 64;
  const long long U = (long long)a.items * a.kblocks;
  const long long u0 = (long long)blockIdx.x * U / gridDim.x, u1 = (long long)(blockIdx.x + 1) * U / gridDim.x;
  const int kbfirst = (int)(u0 % a.kblocks);
  const int nres_used = (int)((u1 - u0) < (long long)a.kblocks ? (u1 - u0) : (long long)a.kblocks);
  const int acc_cols = n_a * T4_BN;
  const int sf_cols_stage = n_a * 16 + 16;
  const int sf_col0 = 2 * acc_cols;
  volatile int* abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int i = 0; i < a.stages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 4); }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, (uint32_t)a.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  if (threadIdx.x == 0) t4_stamp(a, 1);

  // ---------------- producer: weights and their scales, TMA + bulk copies ----------------
  T4Cursor cur{u0, u1, 0, 0u};
  auto produce = [&](int limit) -> bool {                 // issues up to `limit` stages; false on a wait that ran out
    const uint32_t tx = (uint32_t)(n_a * (T4_A_BYTES + T4_SFA_STAGE));
    while (cur.u < cur.u1 && limit-- > 0) {
      const int item = (int)(cur.u / a.kblocks), kb = (int)(cur.u % a.kblocks);
      if (!t4_wait(&empty_bar[cur.stage], cur.phase ^ 1u, abort_flag)) return false;
      unsigned char* sa = tiles + (size_t)cur.stage * stage_bytes;
      unsigned char* ssfa = sa + n_a * T4_A_BYTES;
      mbar_expect_tx(&full_bar[cur.stage], tx);
      for (int i = 0; i < n_a; ++i) {
        const int row = item * T4_BM + i * a.N;            // gate rows, then up rows N further
        tma_load_2d(sa + i * T4_A_BYTES, &tmA, &full_bar[cur.stage], kb * T4_BKB, row);
        t4_bulk_load(ssfa + i * T4_SFA_STAGE, a.sf_a + ((size_t)(row / 128) * kt_total + (size_t)kb * 4) * T4_SF_ATOM,
                     T4_SFA_STAGE, &full_bar[cur.stage]);
      }
      if (++cur.stage == a.stages) { cur.stage = 0; cur.phase ^= 1u; }
      ++cur.u;
    }
    return true;
  };
  const bool is_producer = warp == 0 && elect_one();
  bool prod_ok = true;
  if (is_producer) {
    tma_prefetch_desc(&tmA);
    prod_ok = produce(a.stages);                           // the ring fills while the previous kernel still runs
  }

  // ---------------- all warps: normalise and quantise the activation rows this CTA multiplies ----------------
  pdl_wait();
  if (threadIdx.x == 0) t4_stamp(a, 2);
  {
    // One task = 16 values of one row of one resident k block. Every thread loads its tasks once (the first two stay
    // in registers), the CTA takes the largest |x (1 + w)| of each row over ITS blocks as that row's scale base, and
    // the values are quantised term by term. The RMSNorm factor is a per-row constant: it is applied in the epilogue
    // from the per-block sums of squares gathered here, so nothing waits for a pass over the whole row.
    const int ntask = nres_used * a.M * 16;
    auto load_task = [&](int q, float (&xv)[16]) -> float {      // fills xv with x (1 + w); returns the sum of x^2
      const int m = (q >> 4) % a.M, js = (q >> 4) / a.M;
      int kb = kbfirst + js;
      if (kb >= a.kblocks) kb -= a.kblocks;
      const int k = kb * T4_BK + (q & 15) * 16;
      const uint4* xp = reinterpret_cast<const uint4*>(a.X + (size_t)m * a.ldx + k);
      const uint4 v0 = xp[0], v1 = xp[1];
      const uint32_t u[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xv[2 * j] = bf_lo(u[j]); xv[2 * j + 1] = bf_hi(u[j]);
        ss += xv[2 * j] * xv[2 * j] + xv[2 * j + 1] * xv[2 * j + 1];
      }
      if (a.norm_w) {
        const uint4* wp = reinterpret_cast<const uint4*>(a.norm_w + k);
        const uint4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
        const uint32_t wu[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) { xv[2 * j] *= 1.f + bf_lo(wu[j]); xv[2 * j + 1] *= 1.f + bf_hi(wu[j]); }
      }
      return ss;
    };
    float keep0[16], keep1[16];
    float am[T4_MAX_R];
#pragma unroll
    for (int m = 0; m < T4_MAX_R; ++m) am[m] = 0.f;
    const int ntask_warp = (ntask + 31) & ~31;             // whole warps run the loop: it shuffles
    for (int q = threadIdx.x, it = 0; q < ntask_warp; q += T4_THREADS, ++it) {
      float xv[16];
      float ss = 0.f;
      if (q < ntask) {
        ss = load_task(q, xv);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) xv[j] = 0.f;
      }
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(xv[j]));
      const int m = (q >> 4) % a.M;
#pragma unroll
      for (int mm = 0; mm < T4_MAX_R; ++mm) am[mm] = (mm == m) ? fmaxf(am[mm], bm) : am[mm];
      // the 16 tasks of a (k block, row) sit in 16 consecutive lanes
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((q & 15) == 0 && q < ntask) ssq[(q >> 4)] = ss;        // index = js * M + m
      if (it == 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) keep0[j] = xv[j];
      } else if (it == 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) keep1[j] = xv[j];
      }
    }
#pragma unroll
    for (int m = 0; m < T4_MAX_R; ++m)
      if (m < a.M) {
        const float a2 = warp_max(am[m]);
        if (lane == 0) red_s[warp][m] = a2;
      }
    __syncthreads();
    if (threadIdx.x < a.M) {
      const int m = threadIdx.x;
      float amx = 0.f;
      for (int w = 0; w < T4_THREADS / 32; ++w) amx = fmaxf(amx, red_s[w][m]);
      float gs = amx > 0.f ? amx / (6.f * 448.f) : 1.f;
      for (int t = 0; t < a.terms; ++t) { gst_s[m * a.terms + t] = gs; gs *= 0.25f; }
    }
    __syncthreads();
    if (threadIdx.x == 0) t4_stamp(a, 3);
    for (int q = threadIdx.x, it = 0; q < ntask; q += T4_THREADS, ++it) {
      float xv[16];
      if (it == 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) xv[j] = keep0[j];
      } else if (it == 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) xv[j] = keep1[j];
      } else {
        (void)load_task(q, xv);
      }
      const int qb = q & 15, m = (q >> 4) % a.M, js = (q >> 4) / a.M;
      for (int t = 0; t < a.terms; ++t) {
        const int r = m * a.terms + t;
        const float gs = gst_s[r];
        float bm = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(xv[j]));
        __nv_fp8_storage_t sc8 = __nv_cvt_float_to_fp8(bm / (6.f * gs), __NV_SATFINITE, __NV_E4M3);
        __half_raw hr = __nv_cvt_fp8_to_halfraw(sc8, __NV_E4M3);
        const float step = __half2float(*reinterpret_cast<__half*>(&hr)) * gs;      // value of code 1.0
        const float inv = step > 0.f ? 1.f / step : 0.f;
        uint32_t packed[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          __nv_fp4x2_storage_t c2 = __nv_cvt_float2_to_fp4x2(make_float2(xv[j] * inv, xv[j + 1] * inv), __NV_E2M1, cudaRoundNearest);
          packed[j / 8] |= (uint32_t)c2 << (8 * ((j / 2) % 4));
          __half2_raw d2 = __nv_cvt_fp4x2_to_halfraw2(c2, __NV_E2M1);
          const float2 df = __half22float2(*reinterpret_cast<__half2*>(&d2));
          xv[j] -= df.x * step;                            // what this term did not represent goes to the next
          xv[j + 1] -= df.y * step;
        }
        // 128-byte swizzle of the K-major tile: 16-byte chunk c of row r lives at chunk c ^ (r % 8)
        const int chunk = (qb >> 1) ^ (r & 7);
        *reinterpret_cast<uint2*>(bq + (size_t)js * T4_B_BLOCK + r * 128 + chunk * 16 + (qb & 1) * 8) = make_uint2(packed[0], packed[1]);
        bsf[(size_t)js * T4_SFB_BLOCK + (qb >> 2) * T4_SFB_STEP + r * 16 + (qb & 3)] = sc8;
      }
    }
    fence_proxy_async();
  }
  __syncthreads();
  if (threadIdx.x == 0) t4_stamp(a, 4);

  if (warp == 0) {
    if (is_producer) {
      if (prod_ok) prod_ok = produce(0x7fffffff);
      if (!prod_ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
      if (prod_ok && a.pf_w) {
        // all of this CTA's own loads are issued: ask L2 for the head of the runs the next call's CTAs will walk
        const long long U2 = (long long)a.pf_items * a.pf_kblocks;
        for (int c2 = blockIdx.x; c2 < a.pf_grid; c2 += gridDim.x) {
          const long long v0 = (long long)c2 * U2 / a.pf_grid, v1 = (long long)(c2 + 1) * U2 / a.pf_grid;
          const int item0 = (int)(v0 / a.pf_kblocks), item1 = (int)((v1 - 1) / a.pf_kblocks);
          const long row0 = (long)item0 * T4_BM;
          long row1 = (long)(item1 + 1) * T4_BM;
          if (row1 > a.pf_n) row1 = a.pf_n;
          long bytes = (row1 - row0) * a.pf_row_bytes;
          if (bytes > a.pf_cta_bytes) bytes = a.pf_cta_bytes;
          bytes &= ~15L;
          for (int part = 0; part <= a.pf_dual; ++part)
            t4_prefetch_l2(a.pf_w + (row0 + (long)part * a.pf_n) * a.pf_row_bytes, bytes);
          long sfb = (long)(item1 - item0 + 1) * a.pf_sf_item_bytes;
          if (sfb > a.pf_cta_bytes / 8) sfb = (a.pf_cta_bytes / 8) & ~15L;
          for (int part = 0; part <= a.pf_dual; ++part)
            t4_prefetch_l2(a.pf_sf + (long)(item0 + part * (a.pf_n / T4_BM)) * a.pf_sf_item_bytes, sfb);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_nvfp4(T4_BM, T4_BN, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int buf = 0; uint32_t tphase[2] = {0, 0};
      bool ok = true;
      for (long long u = u0; u < u1 && ok;) {
        const int kb0 = (int)(u % a.kblocks);
        const int kb1 = (int)((u1 - u) < (long long)(a.kblocks - kb0) ? kb0 + (u1 - u) : a.kblocks);
        if (!t4_wait(&tempty_bar[buf], tphase[buf] ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(buf * acc_cols);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!t4_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (u == u0 && kb == kb0) t4_stamp(a, 5);
          int js = kb - kbfirst;
          if (js < 0) js += a.kblocks;
          const uint32_t sa = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint32_t ssfa = sa + n_a * T4_A_BYTES;
          const uint32_t tsfa = tmem_base + (uint32_t)(sf_col0 + stage * sf_cols_stage);
          const uint32_t tsfb = tsfa + (uint32_t)(n_a * 16);
          for (int i = 0; i < n_a; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc_cp_32x128b_warpx4(tsfa + (uint32_t)(i * 16 + j * 4),
                                   umma_desc_noswz(ssfa + i * T4_SFA_STAGE + j * T4_SF_ATOM, 16, 128));
          // every K-64 step gets its own 4-column group: a scale address that is not a multiple of 4 columns makes
          // the MMA fault with "misaligned address"
#pragma unroll
          for (int j = 0; j < 4; ++j)
            tc_cp_32x128b_warpx4(tsfb + (uint32_t)(j * 4),
                                 umma_desc_noswz(smem_u32(bsf) + (uint32_t)(js * T4_SFB_BLOCK + j * T4_SFB_STEP), 16, 128));
          const uint64_t db = umma_desc_k128(smem_u32(bq) + (uint32_t)(js * T4_B_BLOCK));
          for (int i = 0; i < n_a; ++i) {
            const uint64_t da = umma_desc_k128(sa + i * T4_A_BYTES);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc_mma_nvfp4(d0 + (uint32_t)(i * T4_BN), da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc,
                           tsfa + (uint32_t)(i * 16 + j * 4), tsfb + (uint32_t)(j * 4), (kb > kb0 || j > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == a.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[buf]);
        tphase[buf] ^= 1u;
        buf ^= 1;
        u += kb1 - kb0;
      }
      t4_stamp(a, 6);
      if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quad = warp & 3;
    const int etid = quad * 32 + lane;
    int buf = 0; uint32_t tphase[2] = {0, 0};
    bool ok = true;
    __nv_bfloat16* Yb = reinterpret_cast<__nv_bfloat16*>(a.Y);
    // a partial is [gate rows | up rows | one column of per-row sums of x^2] x 128 weight rows, already scaled by this
    // CTA's activation scales (CTAs that share a tile quantised their k ranges with their own)
    const int ncol = n_a * a.M + 1;
    for (long long u = u0; u < u1 && ok;) {
      const int item = (int)(u / a.kblocks), kb0 = (int)(u % a.kblocks);
      const int kb1 = (int)((u1 - u) < (long long)(a.kblocks - kb0) ? kb0 + (u1 - u) : a.kblocks);
      const bool whole = kb0 == 0 && kb1 == a.kblocks;
      if (a.norm_w && etid < a.M) {                       // sum of x^2 of this segment's k range, per row
        float ss = 0.f;
        for (int kb = kb0; kb < kb1; ++kb) {
          int js = kb - kbfirst;
          if (js < 0) js += a.kblocks;
          ss += ssq[js * a.M + etid];
        }
        rn_s[etid] = ss;
      }
      ok = t4_wait(&tfull_bar[buf], tphase[buf], abort_flag);
      {                                                   // everyone agrees on ok; rn_s is visible
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.red.and.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
        ok = all_ok != 0;
      }
      if (!ok) break;
      tphase[buf] ^= 1u;
      tc_fence_after();
      const uint32_t tbase = tmem_base + (uint32_t)(buf * acc_cols) + ((uint32_t)(quad * 32) << 16);
      uint32_t r0[16], r1[16];
      tmem_ld16(tbase, r0);
      if (a.dual) tmem_ld16(tbase + (uint32_t)T4_BN, r1);
      tmem_ld_wait();
      tc_fence_before();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      const int n = item * T4_BM + etid;
      const bool n_ok = n < a.N;
      float g[T4_MAX_R], up[T4_MAX_R], ssr[T4_MAX_R];     // per activation row
#pragma unroll
      for (int m = 0; m < T4_MAX_R; ++m) { g[m] = 0.f; up[m] = 0.f; ssr[m] = (a.norm_w && m < a.M) ? rn_s[m] : 0.f; }
#pragma unroll
      for (int c = 0; c < T4_MAX_R; ++c)
        if (c < a.R) {
          const int m = c / a.terms;
          const float sc = gst_s[c];
#pragma unroll
          for (int mm = 0; mm < T4_MAX_R; ++mm)
            if (mm == m) { g[mm] += __uint_as_float(r0[c]) * sc; if (a.dual) up[mm] += __uint_as_float(r1[c]) * sc; }
        }
      bool finish = whole;
      if (!whole) {
        const long long ui0 = (long long)item * a.kblocks;
        const int c_first = (int)(((ui0 + 1) * gridDim.x - 1) / U);
        const int c_last = (int)(((ui0 + a.kblocks) * gridDim.x - 1) / U);
        const int slot = (int)blockIdx.x - c_first;
        float* ws = a.workspace + ((size_t)item * a.max_slots + slot) * ncol * T4_BM;
#pragma unroll
        for (int m = 0; m < T4_MAX_R; ++m)
          if (m < a.M) {
            ws[(size_t)m * T4_BM + etid] = g[m];
            if (a.dual) ws[(size_t)(a.M + m) * T4_BM + etid] = up[m];
            if (etid == m) ws[(size_t)(ncol - 1) * T4_BM + m] = ssr[m];
          }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (etid == 0) {
          const int old = atomicAdd(&a.counters[item], kb1 - kb0);
          last_flag_s = (old + (kb1 - kb0) == a.kblocks) ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finish = last_flag_s != 0;
        if (finish) {
          __threadfence();
          const float* wt = a.workspace + (size_t)item * a.max_slots * ncol * T4_BM;
          const int ns = c_last - c_first + 1;
#pragma unroll
          for (int m = 0; m < T4_MAX_R; ++m) { g[m] = 0.f; up[m] = 0.f; ssr[m] = 0.f; }
          for (int s2 = 0; s2 < ns; ++s2) {                // CTA order, whoever arrived last
            const float* p = wt + (size_t)s2 * ncol * T4_BM;
#pragma unroll
            for (int m = 0; m < T4_MAX_R; ++m)
              if (m < a.M) {
                g[m] += __ldcg(p + (size_t)m * T4_BM + etid);
                if (a.dual) up[m] += __ldcg(p + (size_t)(a.M + m) * T4_BM + etid);
                ssr[m] += __ldcg(p + (size_t)(ncol - 1) * T4_BM + m);
              }
          }
          if (etid == 0) a.counters[item] = 0;
        }
      }
      if (finish && n_ok) {
        const float ag = a.row_alpha ? a.row_alpha[n] : a.w_scale;
        const float au = a.dual ? (a.row_alpha ? a.row_alpha[a.N + n] : a.w_scale) : 0.f;
#pragma unroll
        for (int m = 0; m < T4_MAX_R; ++m)
          if (m < a.M) {
            const float rn = a.norm_w ? rsqrtf(ssr[m] / (float)a.K + a.eps) : 1.f;
            float x = g[m] * rn * ag;
            if (a.dual) x = siluf_(x) * (up[m] * rn * au);
            if (a.res) x += bf2f(a.res[(size_t)m * a.ldy + n]);
            if (a.out_f32) reinterpret_cast<float*>(a.Y)[(size_t)m * a.ldy + n] = x;
            else Yb[(size_t)m * a.ldy + n] = f2bf(x);
          }
      }
      // rn_s and last_flag_s are rewritten for the next segment: everyone is done reading them
      asm volatile("bar.sync 1, 128;" ::: "memory");
      buf ^= 1;
      u += kb1 - kb0;
    }
    if (etid == 0) t4_stamp(a, 7);
    if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_s && threadIdx.x == 0) {
    // loads already issued still target this CTA's shared memory: give them a bounded time to land
    for (int i = 0; i < a.stages; ++i)
      for (uint32_t p = 0; p < 2; ++p) (void)mbar_wait(&full_bar[i], p, 1u << 12);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
  }
}

typedef CUresult (*EncodeTiledFnT4)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnT4 t4_encode() {
  static EncodeTiledFnT4 fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
  if (qres != cudaDriverEntryPointSuccess) return nullptr;
  fn = (EncodeTiledFnT4)p;
  return fn;
}

struct T4Plan {
  int ok, terms, R, stages, kblocks, items, max_slots, nres, tmem_cols, grid;
  size_t smem;
  long ws_bytes;
};

static int t4_pow2_at_least(int v) { int p = 32; while (p < v) p <<= 1; return p; }

static T4Plan t4_plan(int M, int N, int K, int dual, int terms, int sm_count, int ctas_per_sm) {
  T4Plan p = {};
  if (M <= 0 || M > T4_MAX_R || N <= 0 || K <= 0 || K % T4_BK) return p;
  if (dual && (N % 128)) return p;                    // gate and up scale tiles start on a 128-row tile
  if (terms < 1) terms = 1;
  if (terms > 3) terms = 3;
  while (M * terms > T4_MAX_R) --terms;
  p.terms = terms; p.R = M * terms;
  p.kblocks = K / T4_BK;
  p.items = (N + T4_BM - 1) / T4_BM;
  if (sm_count <= 0) sm_count = 148;
  if (ctas_per_sm < 1) ctas_per_sm = 1;
  const long long U = (long long)p.items * p.kblocks;
  long long grid = (long long)sm_count * ctas_per_sm;
  if (grid > U) grid = U;
  // nearly as many tiles as CTAs: one whole tile each (no partials to combine) beats a perfectly even split
  if (p.items <= grid && (long long)p.items * 8 >= grid * 7) grid = p.items;
  p.grid = (int)grid;
  const long long per_lo = U / grid, per_hi = (U + grid - 1) / grid;
  p.nres = (int)(per_hi < p.kblocks ? per_hi : p.kblocks);
  long long slots = p.kblocks / (per_lo > 0 ? per_lo : 1) + 2;
  if (slots > p.kblocks) slots = p.kblocks;
  if (slots > grid) slots = grid;
  p.max_slots = (int)slots;
  const int n_a = dual ? 2 : 1;
  const int stage_bytes = n_a * (T4_A_BYTES + T4_SFA_STAGE);
  const size_t fixed = 1024 + (size_t)(p.nres + 1) * T4_B_BLOCK + (size_t)p.nres * T4_SFB_BLOCK + 384 +
                       (size_t)p.nres * T4_MAX_R * sizeof(float) + 16;
  const size_t cap = (ctas_per_sm > 1 ? 110 : 220) * 1024;
  if (fixed + 2 * (size_t)stage_bytes > cap) return p;
  int stages = (int)((cap - fixed) / stage_bytes);
  if (stages > T4_MAX_STAGES) stages = T4_MAX_STAGES;
  const int tm_fixed = 2 * n_a * T4_BN, tm_stage = n_a * 16 + 16;
  while (stages > 2 && tm_fixed + stages * tm_stage > (ctas_per_sm > 1 ? 256 : 512)) --stages;
  p.stages = stages;
  p.tmem_cols = t4_pow2_at_least(tm_fixed + stages * tm_stage);
  p.smem = fixed + (size_t)stages * stage_bytes;
  p.ws_bytes = (long)p.items * p.max_slots * (n_a * M + 1) * T4_BM * (long)sizeof(float);
  p.ok = 1;
  return p;
}

}  // namespace fb

using namespace fb;

static unsigned long long* g_t4_trace = nullptr;
static int g_t4_trace_call = 0;

// Debug aid: a device buffer of [8 calls][1024 CTAs][8] 64-bit words; later calls stamp it, call after call in turn
// (nullptr switches it off).
extern "C" void fb_gemv_nvfp4_tc_trace_set(void* buf) { g_t4_trace = (unsigned long long*)buf; g_t4_trace_call = 0; }

// Workspace bytes for a call of this shape (0 when the shape is not served by this kernel).
extern "C" long fb_gemv_nvfp4_tc_workspace_bytes(int M, int N, int K, int dual, int terms, int sm_count, int ctas_per_sm) {
  T4Plan p = t4_plan(M, N, K, dual, terms, sm_count, ctas_per_sm);
  return p.ok ? p.ws_bytes : 0;
}

// Renderings per activation row this shape would get (0: shape not served).
extern "C" int fb_gemv_nvfp4_tc_terms(int M, int N, int K, int dual, int terms) {
  T4Plan p = t4_plan(M, N, K, dual, terms, 148, 1);
  return p.ok ? p.terms : 0;
}

// Y[M, N] = act(X[M, K] (optionally RMSNorm(1+w))) @ Wq^T, M <= 8 rows. Wq: e2m1 codes [rows][K/2]; w_sf: tiled
// ue4m3 scales; w_scale or row_alpha[rows]: tensor scale. mode 1: rows are gate|up and the output is silu(g) * u.
// counters: `ceil(N/128)` zeroed ints, left zeroed. The items counter array must not be shared with a kernel that
// may run concurrently.
// next_Wq / next_sf / next_N / next_K / next_mode: the NVFP4 weight the next few-row call on this stream will use
// (nullptr: unknown); up to prefetch_bytes of it are requested into L2 as this kernel's own loads run out.
extern "C" int fb_gemv_nvfp4_tc(void* Y, const void* X, long ldx, const void* norm_w, float eps, const void* Wq,
                                const void* w_sf, float w_scale, const float* row_alpha, const void* res, int M, int N,
                                int K, long ldy, int mode, int terms, int out_f32, float* workspace, int* counters,
                                int* status, int sm_count, int ctas_per_sm, const void* next_Wq, const void* next_sf,
                                int next_N, int next_K, int next_mode, long prefetch_bytes, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  const int dual = mode == 1;
  T4Plan p = t4_plan(M, N, K, dual, terms, sm_count, ctas_per_sm);
  if (!p.ok || (ldx % 8)) return -1;
  if (((uintptr_t)X & 15) || (norm_w && ((uintptr_t)norm_w & 15))) return -1;
  if (p.ws_bytes && (!workspace || !counters)) return -6;
  T4Args a;
  a.Y = Y; a.res = (const __nv_bfloat16*)res; a.X = (const __nv_bfloat16*)X; a.norm_w = (const __nv_bfloat16*)norm_w;
  a.sf_a = (const uint8_t*)w_sf; a.row_alpha = row_alpha; a.w_scale = w_scale; a.eps = eps;
  a.workspace = workspace; a.counters = counters; a.status = status;
  a.M = M; a.N = N; a.K = K; a.ldy = ldy; a.ldx = ldx; a.dual = dual; a.terms = p.terms; a.R = p.R;
  a.stages = p.stages; a.out_f32 = out_f32; a.kblocks = p.kblocks; a.items = p.items; a.max_slots = p.max_slots;
  a.nres = p.nres; a.tmem_cols = p.tmem_cols; a.trace = (g_t4_trace && p.grid <= 1024) ? g_t4_trace + (size_t)(g_t4_trace_call++ % 8) * 1024 * 8 : nullptr;
  a.pf_w = nullptr; a.pf_sf = nullptr;
  a.pf_row_bytes = a.pf_sf_item_bytes = a.pf_cta_bytes = 0; a.pf_items = a.pf_kblocks = a.pf_grid = a.pf_n = a.pf_dual = 0;
  if (next_Wq && next_sf && prefetch_bytes > 0) {
    T4Plan q = t4_plan(M, next_N, next_K, next_mode == 1, terms, sm_count, ctas_per_sm);
    // a gate|up pair is addressed as two row ranges N apart, and the scale tiles of the parts as item ranges: both
    // need whole tiles
    if (q.ok && !(((uintptr_t)next_Wq | (uintptr_t)next_sf) & 15) && (next_mode != 1 || next_N % T4_BM == 0)) {
      a.pf_w = (const unsigned char*)next_Wq; a.pf_sf = (const unsigned char*)next_sf;
      a.pf_row_bytes = next_K / 2; a.pf_sf_item_bytes = (long)(next_K / 64) * T4_SF_ATOM;
      a.pf_items = q.items; a.pf_kblocks = q.kblocks; a.pf_grid = q.grid; a.pf_n = next_N; a.pf_dual = next_mode == 1;
      a.pf_cta_bytes = (prefetch_bytes / q.grid / (a.pf_dual ? 2 : 1)) & ~15L;
      if (a.pf_cta_bytes < 4096) a.pf_w = nullptr;
    }
  }
  EncodeTiledFnT4 fn = t4_encode();
  if (!fn) return -10;
  const uint64_t w_rows = (uint64_t)(dual ? 2 * N : N), row_bytes = (uint64_t)K / 2;
  if (((uintptr_t)Wq & 15) || (row_bytes & 15) || ((uintptr_t)w_sf & 15)) return -11;
  CUtensorMap tmA;
  cuuint64_t dims[2] = {row_bytes, w_rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)T4_BKB, (cuuint32_t)T4_BM};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(Wq), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -12;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemv_nvfp4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  return (int)launch_pdl(gemv_nvfp4_tc_kernel, dim3(p.grid), dim3(T4_THREADS), p.smem, s, tmA, a);
}
