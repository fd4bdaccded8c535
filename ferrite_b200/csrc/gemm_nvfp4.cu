// Block-scaled NVFP4 GEMM on the 5th-generation tensor cores (W4A4): Y = (X_q * W_q^T) * alpha, with e2m1 operands,
// one ue4m3 scale per 16 values, fp32 accumulation in TMEM. `tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X`
// reads the scale factors from TMEM; they arrive there from shared memory with `tcgen05.cp 32x128b.warpx4`, and in
// shared memory by bulk copies of pre-tiled 512-byte atoms (128 rows x 4 k-blocks, laid out [row%32][row/32][kb]).
//
// Same warp-specialised, persistent structure as the bf16 GEMM (TMA producer warp, single-thread MMA issuer that
// owns TMEM, four epilogue warps, two accumulator buffers) and the same two orientations: weights as the
// 128-row operand with the few activation rows as N (decode / verify, split-K), or activations as the 128-row
// operand for prompts. The activation side is quantised on the fly by `fb_quant_nvfp4` (optionally fused with
// RMSNorm), with a per-row global scale that the epilogue multiplies back in.
//
// Replaces `fe_fp4_quant`, `fe_gemm_nvfp4*` and `fe_gemm_nvfp4_swiglu` (`kernels/k-fp4/src/lib.rs:167-866`,
// mma.sync m16n8k64 with scale registers) with the TMEM-scaled tcgen05 form.
#include <cuda.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "api_ext.h"
#include "common.cuh"

namespace fb {

constexpr int Q4_BM = 128;            // rows of the A box
constexpr int Q4_BKB = 128;           // bytes of K per stage row = 256 e2m1 values = 4 MMAs of K 64
constexpr int Q4_BK = 256;
constexpr int Q4_MAX_STAGES = 4;
constexpr int Q4_THREADS = 192;
constexpr int Q4_A_BYTES = Q4_BM * Q4_BKB;     // 16 KB
constexpr int Q4_SF_ATOM = 512;                // bytes: 128 rows x 4 k-blocks
constexpr int Q4_SF_STAGE = 4 * Q4_SF_ATOM;    // scale bytes per 128 rows per stage

struct Q4Args {
  void* Y;
  const __nv_bfloat16* res;
  const uint8_t* sf_a;        // tiled scales of the A operand [row tile][K/64][512]
  const uint8_t* sf_b;        // tiled scales of the B operand
  const float* row_scale;     // per activation row (token) global scale
  float w_scale;              // weight tensor global scale
  float* workspace;
  int* counters;
  int* status;
  int M, N, K;
  long ldy;
  int swap, dual, bn, n_a, n_b, b_box_rows, stages, split_k, tiles_a, tiles_b, acc_cols, tmem_cols;
  int sf_col0;                // first TMEM column of the scale-factor area
  int sf_cols_stage;          // scale columns per pipeline stage
  int b_sf_tiles;             // 128-row scale tiles of the B operand per stage
  int n_bm;                   // B boxes that get their own MMA + accumulator (normal SwiGLU: gate, up)
  int n_buf;                  // accumulator buffers in TMEM (2 = epilogue overlaps the next tile)
  // fused activation quantiser (swapped orientation, <= 8 rows): the epilogue warps read the bf16 rows,
  // normalise + quantise them stage by stage straight into the B tile and its scale atoms
  int fuseq;
  const __nv_bfloat16* X;
  long ldx;
  const __nv_bfloat16* norm_w;
  float eps;
  int out_f32;
  // SwiGLU output re-quantised to NVFP4 by the epilogue (normal orientation): codes [M][N / 2], scales in the tiled
  // layout of an A operand with K = N, one static global scale for every row
  uint8_t* q_codes;
  uint8_t* q_sf;
  float* q_row_scale;
  float q_gs;
};

__device__ __forceinline__ bool q4_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
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

// 1-D bulk copy global -> shared, completion on an mbarrier (both addresses 16-byte aligned, size % 16 == 0)
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(Q4_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Q4Args a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[Q4_MAX_STAGES], empty_bar[Q4_MAX_STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int last_flag_s;
  __shared__ float rs_s[8], rn_s[8];      // fused quantiser: per-row global scale and RMSNorm factor
  __shared__ float red_s[4][8];

  pdl_launch_dependents();
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b_bytes = a.n_b * a.b_box_rows * Q4_BKB;
  const int b_bytes_pad = (b_bytes + 1023) & ~1023;
  const int sfa_bytes = a.n_a * Q4_SF_STAGE;
  const int sfb_bytes = a.b_sf_tiles * Q4_SF_STAGE;
  const int stage_bytes = a.n_a * Q4_A_BYTES + b_bytes_pad + sfa_bytes + sfb_bytes;
  const int kblocks_total = a.K / Q4_BK;
  const int kb_per_split = (kblocks_total + a.split_k - 1) / a.split_k;
  const int total_work = a.tiles_a * a.tiles_b * a.split_k;
  const int kt_total = a.K / 64;                      // scale atoms along K per row tile
  volatile int* abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int i = 0; i < a.stages; ++i) { mbar_init(&full_bar[i], a.fuseq ? 5 : 1); mbar_init(&empty_bar[i], 1); }
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

  auto decode_work = [&](int w, int& ta, int& tb, int& ks) {
    ks = w % a.split_k;
    int t = w / a.split_k;
    if (a.swap) { tb = t % a.tiles_b; ta = t / a.tiles_b; }
    else { ta = t % a.tiles_a; tb = t / a.tiles_a; }
  };

  if (warp == 0) {
    // ---------------- producer: TMA tiles + bulk copies of the scale atoms ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0; uint32_t phase = 0;
      const uint32_t tx = (uint32_t)(a.n_a * Q4_A_BYTES + sfa_bytes + (a.fuseq ? 0 : b_bytes + sfb_bytes));
      bool ok = true;
      // weights never depend on the previous kernel: with the fused quantiser this warp starts streaming them
      // at once; otherwise it also loads the quantised activations and has to wait for their producer
      if (!a.fuseq) pdl_wait();
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int ta, tb, ks;
        decode_work(w, ta, tb, ks);
        const int kb0 = ks * kb_per_split, kb1 = min(kblocks_total, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!q4_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          unsigned char* sa = tiles + (size_t)stage * stage_bytes;
          unsigned char* sb = sa + a.n_a * Q4_A_BYTES;
          unsigned char* ssfa = sb + b_bytes_pad;
          unsigned char* ssfb = ssfa + sfa_bytes;
          mbar_expect_tx(&full_bar[stage], tx);
          const int kx = kb * Q4_BKB;                 // byte coordinate along K
          for (int i = 0; i < a.n_a; ++i) {
            const int row = ta * Q4_BM + i * a.N;     // swapped SwiGLU: gate rows, then up rows N further
            tma_load_2d(sa + i * Q4_A_BYTES, &tmA, &full_bar[stage], kx, row);
            bulk_load(ssfa + i * Q4_SF_STAGE, a.sf_a + ((size_t)(row / 128) * kt_total + (size_t)kb * 4) * Q4_SF_ATOM,
                      Q4_SF_STAGE, &full_bar[stage]);
          }
          for (int i = 0; i < (a.fuseq ? 0 : a.n_b); ++i) {
            const int row = tb * a.b_box_rows + i * a.N;
            tma_load_2d(sb + (size_t)i * a.b_box_rows * Q4_BKB, &tmB, &full_bar[stage], kx, row);
          }
          for (int i = 0; i < (a.fuseq ? 0 : a.b_sf_tiles); ++i) {
            // normal SwiGLU: scale tile 0 = gate rows, tile 1 = up rows; otherwise consecutive 128-row tiles
            const int row = a.swap ? 0 : tb * a.b_box_rows + i * a.N;
            bulk_load(ssfb + i * Q4_SF_STAGE, a.sf_b + ((size_t)(row / 128) * kt_total + (size_t)kb * 4) * Q4_SF_ATOM,
                      Q4_SF_STAGE, &full_bar[stage]);
          }
          if (++stage == a.stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_nvfp4(Q4_BM, (uint32_t)a.bn, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int buf = 0; uint32_t tphase[2] = {0, 0};
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int ta, tb, ks;
        decode_work(w, ta, tb, ks);
        const int kb0 = ks * kb_per_split, kb1 = min(kblocks_total, kb0 + kb_per_split);
        if (!q4_wait(&tempty_bar[buf], tphase[buf] ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(buf * a.acc_cols);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!q4_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint32_t sb = sa + a.n_a * Q4_A_BYTES;
          const uint32_t ssfa = sb + b_bytes_pad;
          const uint32_t ssfb = ssfa + sfa_bytes;
          // scale factors of this stage: shared memory -> TMEM (4 columns per 128 rows per K-64 step)
          const uint32_t tsf = tmem_base + (uint32_t)(a.sf_col0 + stage * a.sf_cols_stage);
          const uint32_t tsfa = tsf, tsfb = tsf + (uint32_t)(a.n_a * 16);
          for (int i = 0; i < a.n_a; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc_cp_32x128b_warpx4(tsfa + (uint32_t)(i * 16 + j * 4),
                                   umma_desc_noswz(ssfa + i * Q4_SF_STAGE + j * Q4_SF_ATOM, 16, 128));
          for (int i = 0; i < a.b_sf_tiles; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc_cp_32x128b_warpx4(tsfb + (uint32_t)(i * 16 + j * 4),
                                   umma_desc_noswz(ssfb + i * Q4_SF_STAGE + j * Q4_SF_ATOM, 16, 128));
          for (int i = 0; i < a.n_a; ++i) {
            const uint64_t da = umma_desc_k128(sa + i * Q4_A_BYTES);
            for (int bi = 0; bi < a.n_bm; ++bi) {
              const uint64_t db = umma_desc_k128(sb + (uint32_t)(bi * a.b_box_rows * Q4_BKB));
#pragma unroll
              for (int j = 0; j < 4; ++j)
                tc_mma_nvfp4(d0 + (uint32_t)((i * a.n_bm + bi) * a.bn), da + (uint64_t)(2 * j), db + (uint64_t)(2 * j),
                             idesc, tsfa + (uint32_t)(i * 16 + j * 4), tsfb + (uint32_t)(bi * 16 + j * 4),
                             (kb > kb0 || j > 0) ? 1u : 0u);
            }
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == a.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[buf]);
        tphase[buf] ^= 1u;
        if (++buf == a.n_buf) buf = 0;
      }
      if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quad = warp & 3;
    const int etid = quad * 32 + lane;
    int buf = 0; uint32_t tphase[2] = {0, 0};
    bool ok = true;
    __nv_bfloat16* Yb = reinterpret_cast<__nv_bfloat16*>(a.Y);
    pdl_wait();                                  // everything below reads X or writes Y / the split-K workspace
    int qstage = 0; uint32_t qphase = 0;
    if (a.fuseq) {
      // zero the B tiles and their scale atoms once: rows >= M of the 16-row box stay zero for the whole kernel
      for (int st = 0; st < a.stages; ++st) {
        unsigned char* sb = tiles + (size_t)st * stage_bytes + a.n_a * Q4_A_BYTES;
        for (int i = etid * 16; i < b_bytes_pad; i += 128 * 16) *reinterpret_cast<uint4*>(sb + i) = make_uint4(0, 0, 0, 0);
        unsigned char* sf = sb + b_bytes_pad + sfa_bytes;
        for (int i = etid * 16; i < sfb_bytes; i += 128 * 16) *reinterpret_cast<uint4*>(sf + i) = make_uint4(0, 0, 0, 0);
      }
      // per-row RMSNorm factor, then per-row amax of the (normalised, bf16-rounded) values -> global scale
      for (int pass = 0; pass < 2; ++pass) {
        if (pass == 0 && !a.norm_w) { if (etid < 8) rn_s[etid] = 1.f; asm volatile("bar.sync 1, 128;" ::: "memory"); continue; }
        float acc[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) acc[m] = 0.f;
        for (int m = 0; m < a.M; ++m) {
          const __nv_bfloat16* xr = a.X + (size_t)m * a.ldx;
          const float rn = pass ? rn_s[m] : 0.f;
          for (int k = etid * 8; k < a.K; k += 128 * 8) {
            uint4 v = *reinterpret_cast<const uint4*>(xr + k);
            uint32_t u[4] = {v.x, v.y, v.z, v.w};
            if (pass == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) { float x0 = bf_lo(u[j]), x1 = bf_hi(u[j]); acc[m] += x0 * x0 + x1 * x1; }
            } else if (a.norm_w) {
              uint4 wv = __ldg(reinterpret_cast<const uint4*>(a.norm_w + k));
              uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                acc[m] = fmaxf(acc[m], fabsf(bf2f(f2bf(bf_lo(u[j]) * rn * (1.f + bf_lo(wu[j]))))));
                acc[m] = fmaxf(acc[m], fabsf(bf2f(f2bf(bf_hi(u[j]) * rn * (1.f + bf_hi(wu[j]))))));
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[m] = fmaxf(acc[m], fmaxf(fabsf(bf_lo(u[j])), fabsf(bf_hi(u[j]))));
            }
          }
        }
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          float v = acc[m];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            float t = __shfl_xor_sync(0xffffffffu, v, o);
            v = pass ? fmaxf(v, t) : v + t;
          }
          if (lane == 0) red_s[quad][m] = v;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (etid < 8) {
          float v = pass ? fmaxf(fmaxf(red_s[0][etid], red_s[1][etid]), fmaxf(red_s[2][etid], red_s[3][etid]))
                         : red_s[0][etid] + red_s[1][etid] + red_s[2][etid] + red_s[3][etid];
          if (pass == 0) rn_s[etid] = rsqrtf(v / (float)a.K + a.eps);
          else rs_s[etid] = v > 0.f ? v / (6.f * 448.f) : 1.f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      int ta, tb, ks;
      decode_work(w, ta, tb, ks);
      if (a.fuseq) {
        // quantise this item's k blocks into the B tiles: thread = (row, 16-value block) of the 256-wide stage
        const int qm = etid >> 4, qb = etid & 15;
        const int kb0 = ks * kb_per_split, kb1 = min(kblocks_total, kb0 + kb_per_split);
        // the activation (and norm weight) values of the next k block are requested before this one is
        // quantised, so their L2 latency overlaps the work instead of adding to every stage
        const bool qact = qm < a.M;
        uint4 nx0 = make_uint4(0, 0, 0, 0), nx1 = nx0, nw0 = nx0, nw1 = nx0;
        if (qact && kb0 < kb1) {
          const int k = kb0 * Q4_BK + qb * 16;
          const uint4* xp = reinterpret_cast<const uint4*>(a.X + (size_t)qm * a.ldx + k);
          nx0 = xp[0]; nx1 = xp[1];
          if (a.norm_w) { const uint4* wp = reinterpret_cast<const uint4*>(a.norm_w + k); nw0 = __ldg(wp); nw1 = __ldg(wp + 1); }
        }
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          const uint4 v0 = nx0, v1 = nx1, w0 = nw0, w1 = nw1;
          if (qact && kb + 1 < kb1) {
            const int k = (kb + 1) * Q4_BK + qb * 16;
            const uint4* xp = reinterpret_cast<const uint4*>(a.X + (size_t)qm * a.ldx + k);
            nx0 = xp[0]; nx1 = xp[1];
            if (a.norm_w) { const uint4* wp = reinterpret_cast<const uint4*>(a.norm_w + k); nw0 = __ldg(wp); nw1 = __ldg(wp + 1); }
          }
          ok = q4_wait(&empty_bar[qstage], qphase ^ 1u, abort_flag);
          if (ok && qact) {
            unsigned char* sb = tiles + (size_t)qstage * stage_bytes + a.n_a * Q4_A_BYTES;
            unsigned char* sf = sb + b_bytes_pad + sfa_bytes;
            uint32_t u[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            float xv[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) { xv[2 * j] = bf_lo(u[j]); xv[2 * j + 1] = bf_hi(u[j]); }
            if (a.norm_w) {
              uint32_t wu[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
              const float rn = rn_s[qm];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                xv[2 * j] = bf2f(f2bf(xv[2 * j] * rn * (1.f + bf_lo(wu[j]))));
                xv[2 * j + 1] = bf2f(f2bf(xv[2 * j + 1] * rn * (1.f + bf_hi(wu[j]))));
              }
            }
            float bm = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(xv[j]));
            const float gs = rs_s[qm];
            __nv_fp8_storage_t sc8 = __nv_cvt_float_to_fp8(bm * (1.f / gs) * (1.f / 6.f), __NV_SATFINITE, __NV_E4M3);
            __half_raw hr = __nv_cvt_fp8_to_halfraw(sc8, __NV_E4M3);
            const float scf = __half2float(*reinterpret_cast<__half*>(&hr));
            const float inv = scf > 0.f ? 1.f / (scf * gs) : 0.f;
            uint32_t packed[2] = {0, 0};
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              __nv_fp4x2_storage_t c2 = __nv_cvt_float2_to_fp4x2(make_float2(xv[j] * inv, xv[j + 1] * inv), __NV_E2M1, cudaRoundNearest);
              packed[j / 8] |= (uint32_t)c2 << (8 * ((j / 2) % 4));
            }
            // 128-byte swizzle of the K-major tile: 16-byte chunk c of row r lives at chunk c ^ (r % 8)
            const int chunk = (qb >> 1) ^ (qm & 7);
            *reinterpret_cast<uint2*>(sb + qm * 128 + chunk * 16 + (qb & 1) * 8) = make_uint2(packed[0], packed[1]);
            sf[(qb >> 2) * Q4_SF_ATOM + qm * 16 + (qb & 3)] = sc8;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[qstage]);
          if (++qstage == a.stages) { qstage = 0; qphase ^= 1u; }
        }
        if (!ok) break;
      }
      ok = q4_wait(&tfull_bar[buf], tphase[buf], abort_flag);
      if (a.split_k > 1) {
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.red.and.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
        ok = all_ok != 0;
      }
      if (!ok) break;
      tphase[buf] ^= 1u;
      tc_fence_after();
      const uint32_t tbase = tmem_base + (uint32_t)(buf * a.acc_cols) + ((uint32_t)(quad * 32) << 16);
      if (!a.swap) {
        const int m = ta * Q4_BM + etid;
        const int ncols_out = a.bn;
        const int n0 = tb * ncols_out;
        const float alpha = (m < a.M) ? a.w_scale * a.row_scale[m] : 0.f;
        for (int c = 0; c < ncols_out; c += 32) {
          uint32_t r0[32], r1[32];
          tmem_ld32(tbase + (uint32_t)c, r0);
          if (a.dual) tmem_ld32(tbase + (uint32_t)(c + a.bn), r1);
          tmem_ld_wait();
          if (m < a.M) {
            const int n = n0 + c;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = __uint_as_float(r0[j]) * alpha;
              v[j] = a.dual ? siluf_(x) * (__uint_as_float(r1[j]) * alpha) : x;
            }
            if (a.q_codes) {
              // the next GEMM's A operand, written here: per 16 columns an e4m3 scale (block amax / 6 / global scale)
              // and 8 bytes of e2m1 codes; this thread owns row m, so a block never straddles threads
              const float inv_gs = 1.f / a.q_gs;
              uint8_t* sf_row = a.q_sf + (size_t)(m / 128) * (a.N / 64) * Q4_SF_ATOM + (size_t)(m % 32) * 16 +
                                (size_t)((m % 128) / 32) * 4;
#pragma unroll
              for (int blk = 0; blk < 2; ++blk) {
                float bm = 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(v[blk * 16 + j]));
                const __nv_fp8_storage_t sc8 = __nv_cvt_float_to_fp8(bm * inv_gs * (1.f / 6.f), __NV_SATFINITE, __NV_E4M3);
                __half_raw hr = __nv_cvt_fp8_to_halfraw(sc8, __NV_E4M3);
                const float scf = __half2float(*reinterpret_cast<__half*>(&hr));
                const float inv = scf > 0.f ? 1.f / (scf * a.q_gs) : 0.f;
                uint32_t packed[2] = {0, 0};
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                  const float2 pr = make_float2(v[blk * 16 + j] * inv, v[blk * 16 + j + 1] * inv);
                  const __nv_fp4x2_storage_t c2 = __nv_cvt_float2_to_fp4x2(pr, __NV_E2M1, cudaRoundNearest);
                  packed[j / 8] |= (uint32_t)c2 << (8 * ((j / 2) % 4));
                }
                const int b = (n >> 4) + blk;
                *reinterpret_cast<uint2*>(a.q_codes + (size_t)m * (a.N / 2) + (size_t)b * 8) = make_uint2(packed[0], packed[1]);
                sf_row[(size_t)(b / 4) * Q4_SF_ATOM + (b % 4)] = sc8;
              }
              if (n == 0) a.q_row_scale[m] = a.q_gs;
            } else if (n + 32 <= a.N) {
              if (a.res) {
                const uint4* rp = reinterpret_cast<const uint4*>(a.res + (size_t)m * a.ldy + n);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 rv = rp[q];
                  uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) { v[q * 8 + 2 * j] += bf_lo(ru[j]); v[q * 8 + 2 * j + 1] += bf_hi(ru[j]); }
                }
              }
              uint4* yp = reinterpret_cast<uint4*>(Yb + (size_t)m * a.ldy + n);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                yp[q] = make_uint4(pack_bf2(v[q * 8], v[q * 8 + 1]), pack_bf2(v[q * 8 + 2], v[q * 8 + 3]),
                                   pack_bf2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf2(v[q * 8 + 6], v[q * 8 + 7]));
            } else {
              for (int j = 0; j < 32 && n + j < a.N; ++j) {
                float x = v[j];
                if (a.res) x += bf2f(a.res[(size_t)m * a.ldy + n + j]);
                Yb[(size_t)m * a.ldy + n + j] = f2bf(x);
              }
            }
          }
        }
        tc_fence_before();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      } else {
        const int n = ta * Q4_BM + etid;
        const int m0 = tb * a.bn;
        const bool n_ok = n < a.N;
        if (a.split_k == 1) {
          for (int c = 0; c < a.bn; c += 16) {
            uint32_t r0[16], r1[16];
            tmem_ld16(tbase + (uint32_t)c, r0);
            if (a.dual) tmem_ld16(tbase + (uint32_t)(a.bn + c), r1);
            tmem_ld_wait();
            if (n_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int m = m0 + c + j;
                if (m < a.M) {
                  const float alpha = a.w_scale * (a.fuseq ? rs_s[m] : a.row_scale[m]);
                  float x = __uint_as_float(r0[j]) * alpha;
                  if (a.dual) x = siluf_(x) * (__uint_as_float(r1[j]) * alpha);
                  if (a.res) x += bf2f(a.res[(size_t)m * a.ldy + n]);
                  if (a.out_f32) reinterpret_cast<float*>(a.Y)[(size_t)m * a.ldy + n] = x;
                  else Yb[(size_t)m * a.ldy + n] = f2bf(x);
                }
              }
            }
          }
          tc_fence_before();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        } else {
          const int tile_id = ta * a.tiles_b + tb;
          const int cols = a.acc_cols;
          float* ws = a.workspace + ((size_t)(tile_id * a.split_k + ks) * cols) * Q4_BM;
          for (int c = 0; c < cols; c += 16) {
            uint32_t r0[16];
            tmem_ld16(tbase + (uint32_t)c, r0);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) ws[(size_t)(c + j) * Q4_BM + etid] = __uint_as_float(r0[j]);
          }
          tc_fence_before();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (etid == 0) {
            int old = atomicAdd(&a.counters[tile_id], 1);
            last_flag_s = (old == a.split_k - 1) ? 1 : 0;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (last_flag_s) {
            __threadfence();
            const float* wt = a.workspace + ((size_t)(tile_id * a.split_k) * cols) * Q4_BM;
            for (int c = 0; c < a.bn; ++c) {
              const int m = m0 + c;
              if (m >= a.M) break;
              float g = 0.f, u = 0.f;
              for (int s2 = 0; s2 < a.split_k; ++s2) {
                const float* p = wt + ((size_t)s2 * cols) * Q4_BM;
                g += __ldcg(p + (size_t)c * Q4_BM + etid);
                if (a.dual) u += __ldcg(p + (size_t)(a.bn + c) * Q4_BM + etid);
              }
              if (n_ok) {
                const float alpha = a.w_scale * (a.fuseq ? rs_s[m] : a.row_scale[m]);
                float x = a.dual ? siluf_(g * alpha) * (u * alpha) : g * alpha;
                if (a.res) x += bf2f(a.res[(size_t)m * a.ldy + n]);
                if (a.out_f32) reinterpret_cast<float*>(a.Y)[(size_t)m * a.ldy + n] = x;
                else Yb[(size_t)m * a.ldy + n] = f2bf(x);
              }
            }
            if (etid == 0) a.counters[tile_id] = 0;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
      if (++buf == a.n_buf) buf = 0;
    }
    if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_s && threadIdx.x == 0) {
    for (int i = 0; i < a.stages; ++i)
      for (uint32_t p = 0; p < 2; ++p) (void)mbar_wait(&full_bar[i], p, 1u << 12);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
  }
}

// ---- activation quantiser ---------------------------------------------------------------------------------
// One CTA per row: optional RMSNorm(1+w), per-row global scale = amax / (6 * 448), e4m3 block scales, e2m1 codes.
// Scales are written straight into the tiled layout the GEMM's bulk copies read.
__global__ void __launch_bounds__(256)
quant_nvfp4_kernel(uint8_t* __restrict__ codes, uint8_t* __restrict__ sf, float* __restrict__ row_scale,
                   const __nv_bfloat16* __restrict__ x, long ldx, const __nv_bfloat16* __restrict__ norm_w, int K,
                   float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];                  // K floats
  __shared__ float scratch[32];
  const int m = blockIdx.x;
  const __nv_bfloat16* xr = x + (size_t)m * ldx;
  float ss = 0.f, amax = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + k);
    uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a0 = bf_lo(u[j]), a1 = bf_hi(u[j]);
      xs[k + 2 * j] = a0; xs[k + 2 * j + 1] = a1;
      ss += a0 * a0 + a1 * a1;
    }
  }
  if (norm_w) {
    float tot = block_sum(ss, scratch);
    float r = rsqrtf(tot / (float)K + eps);
    for (int k = threadIdx.x; k < K; k += blockDim.x)
      xs[k] = bf2f(f2bf(xs[k] * r * (1.f + bf2f(norm_w[k]))));     // same rounding as the bf16 norm kernel
  }
  __syncthreads();
  for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(xs[k]));
  amax = block_max(amax, scratch);
  const float gs = amax > 0.f ? amax / (6.f * 448.f) : 1.f;
  if (threadIdx.x == 0) row_scale[m] = gs;
  const float inv_gs = 1.f / gs;
  const int kt_total = K / 64;
  uint8_t* sf_tile = sf + (size_t)(m / 128) * kt_total * Q4_SF_ATOM + (size_t)(m % 32) * 16 + (size_t)((m % 128) / 32) * 4;
  // one thread per block of 16 values
  for (int b = threadIdx.x; b < K / 16; b += blockDim.x) {
    float bm = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(xs[b * 16 + j]));
    __nv_fp8_storage_t sc8 = __nv_cvt_float_to_fp8(bm * inv_gs * (1.f / 6.f), __NV_SATFINITE, __NV_E4M3);
    __half_raw hr = __nv_cvt_fp8_to_halfraw(sc8, __NV_E4M3);
    float scf = __half2float(*reinterpret_cast<__half*>(&hr));
    float inv = scf > 0.f ? 1.f / (scf * gs) : 0.f;
    uint32_t packed[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      float2 pr = make_float2(xs[b * 16 + j] * inv, xs[b * 16 + j + 1] * inv);
      __nv_fp4x2_storage_t c2 = __nv_cvt_float2_to_fp4x2(pr, __NV_E2M1, cudaRoundNearest);
      packed[j / 8] |= (uint32_t)c2 << (8 * ((j / 2) % 4));
    }
    *reinterpret_cast<uint2*>(codes + (size_t)m * (K / 2) + b * 8) = make_uint2(packed[0], packed[1]);
    sf_tile[(size_t)(b / 4) * Q4_SF_ATOM + (b % 4)] = sc8;
  }
}

// ---- host side ----------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn4)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn4 get_encode4() {
  static EncodeTiledFn4 fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
  if (qres != cudaDriverEntryPointSuccess) return nullptr;
  fn = (EncodeTiledFn4)p;
  return fn;
}

// tensor map over packed codes seen as bytes: [rows][K/2], box = {128 bytes, box_rows}, 128-byte swizzle
static int make_tmap_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn4 fn = get_encode4();
  if (!fn) return -10;
  if (((uintptr_t)base & 15) || (row_bytes & 15)) return -11;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)Q4_BKB, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

static int pow2_at_least(int v) { int p = 32; while (p < v) p <<= 1; return p; }

}  // namespace fb

using namespace fb;

extern "C" long fb_nvfp4_sf_bytes(int rows, int K) {
  return (long)((rows + 127) / 128) * (K / 64) * Q4_SF_ATOM;
}

extern "C" int fb_quant_nvfp4(void* codes, void* sf, float* row_scale, const void* x, long ldx, const void* norm_w,
                              int M, int K, float eps, cudaStream_t s) {
  if (M <= 0) return 0;
  if (K % 64 || ldx % 8) return -1;
  size_t smem = (size_t)K * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(quant_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)launch_pdl(quant_nvfp4_kernel, dim3(M), dim3(256), smem, s, (uint8_t*)codes, (uint8_t*)sf, row_scale,
                         (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)norm_w, K, eps);
}

extern "C" long fb_gemm_nvfp4_workspace_bytes(int M, int N, int split_k) {
  if (M > 64 || split_k <= 1) return 0;
  int bn = ((M + 15) / 16) * 16;
  long tiles = (N + Q4_BM - 1) / Q4_BM;
  return tiles * split_k * 2L * bn * Q4_BM * (long)sizeof(float);
}

// Xq/x_sf/row_scale: quantised activations from fb_quant_nvfp4. Wq/w_sf: weight codes [rows][K/2] and tiled scales.
static int gemm_nvfp4_impl(void* Y, const void* Xq, const void* x_sf, const float* row_scale, const void* Wq,
                           const void* w_sf, float w_scale, const void* res, int M, int N, int K, long ldy, int mode,
                           int split_k, float* workspace, int* counters, int* status, int sm_count, cudaStream_t s,
                           const void* X16, long ldx, const void* norm_w, float eps, int out_f32,
                           void* q_codes = nullptr, void* q_sf = nullptr, float* q_row_scale = nullptr, float q_gs = 0.f) {
  if (M <= 0 || N <= 0) return 0;
  if (q_codes && (M <= 64 || mode != 1 || res || !q_sf || !q_row_scale || !(q_gs > 0.f))) return -1;
  if (K % Q4_BK || (ldy % 8 && M > 64)) return -1;
  if (sm_count <= 0) sm_count = 148;
  Q4Args a;
  a.fuseq = X16 != nullptr; a.X = (const __nv_bfloat16*)X16; a.ldx = ldx; a.norm_w = (const __nv_bfloat16*)norm_w;
  a.eps = eps; a.out_f32 = out_f32;
  a.q_codes = (uint8_t*)q_codes; a.q_sf = (uint8_t*)q_sf; a.q_row_scale = q_row_scale; a.q_gs = q_gs;
  if (a.fuseq && (M > 8 || (ldx % 8))) return -1;
  if (out_f32 && M > 64) return -1;
  a.M = M; a.N = N; a.K = K; a.dual = mode == 1; a.swap = M <= 64;
  const int w_rows = a.dual ? 2 * N : N;
  if (a.dual && (N % 128)) return -2;                 // gate and up scale tiles must start on a 128-row tile
  if (a.swap) {
    a.bn = ((M + 15) / 16) * 16;
    a.n_a = a.dual ? 2 : 1; a.n_b = 1; a.b_box_rows = a.bn; a.b_sf_tiles = 1;
    a.tiles_a = (N + Q4_BM - 1) / Q4_BM; a.tiles_b = 1;
    a.split_k = split_k < 1 ? 1 : split_k;
  } else {
    a.bn = 128;
    a.n_a = 1; a.n_b = a.dual ? 2 : 1; a.b_box_rows = 128; a.b_sf_tiles = a.dual ? 2 : 1;
    a.tiles_a = (M + Q4_BM - 1) / Q4_BM;
    a.tiles_b = (N + 127) / 128;
    a.split_k = 1;
  }
  const int kblocks = K / Q4_BK;
  if (a.split_k > kblocks) a.split_k = kblocks;
  {
    int per = (kblocks + a.split_k - 1) / a.split_k;
    a.split_k = (kblocks + per - 1) / per;
  }
  if (a.split_k > 1 && (!workspace || !counters)) return -6;
  a.n_bm = a.swap ? 1 : a.n_b;
  a.acc_cols = a.n_a * a.n_bm * a.bn;
  const int b_bytes = a.n_b * a.b_box_rows * Q4_BKB;
  const int stage_bytes = a.n_a * Q4_A_BYTES + ((b_bytes + 1023) & ~1023) + (a.n_a + a.b_sf_tiles) * Q4_SF_STAGE;
  a.stages = (200 * 1024) / stage_bytes;
  if (a.stages > Q4_MAX_STAGES) a.stages = Q4_MAX_STAGES;
  if (a.stages < 2) return -5;
  a.sf_cols_stage = a.n_a * 16 + a.b_sf_tiles * 16;
  a.n_buf = (2 * a.acc_cols + a.stages * a.sf_cols_stage <= 512) ? 2 : 1;
  a.sf_col0 = a.n_buf * a.acc_cols;
  const int need_cols = a.sf_col0 + a.stages * a.sf_cols_stage;
  a.tmem_cols = pow2_at_least(need_cols);
  if (a.tmem_cols > 512) return -4;
  a.Y = Y; a.res = (const __nv_bfloat16*)res; a.workspace = workspace; a.counters = counters; a.status = status;
  a.ldy = ldy; a.row_scale = row_scale; a.w_scale = w_scale;
  CUtensorMap tmA, tmB;
  int rc;
  if (a.swap) {
    a.sf_a = (const uint8_t*)w_sf; a.sf_b = (const uint8_t*)x_sf;
    rc = make_tmap_u8(&tmA, Wq, (uint64_t)w_rows, (uint64_t)K / 2, Q4_BM);
    if (rc) return rc;
    // fused quantiser: the B tile is written by the kernel itself; the map is never used (any valid one will do)
    rc = a.fuseq ? make_tmap_u8(&tmB, Wq, (uint64_t)w_rows, (uint64_t)K / 2, (uint32_t)a.b_box_rows)
                 : make_tmap_u8(&tmB, Xq, (uint64_t)M, (uint64_t)K / 2, (uint32_t)a.b_box_rows);
  } else {
    a.sf_a = (const uint8_t*)x_sf; a.sf_b = (const uint8_t*)w_sf;
    rc = make_tmap_u8(&tmA, Xq, (uint64_t)M, (uint64_t)K / 2, Q4_BM);
    if (rc) return rc;
    rc = make_tmap_u8(&tmB, Wq, (uint64_t)w_rows, (uint64_t)K / 2, (uint32_t)a.b_box_rows);
  }
  if (rc) return rc;
  size_t smem = (size_t)a.stages * stage_bytes + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  int total = a.tiles_a * a.tiles_b * a.split_k;
  int grid = total < sm_count ? total : sm_count;
  return (int)launch_pdl(gemm_nvfp4_kernel, dim3(grid), dim3(Q4_THREADS), smem, s, tmA, tmB, a);
}

extern "C" int fb_gemm_nvfp4(void* Y, const void* Xq, const void* x_sf, const float* row_scale, const void* Wq,
                             const void* w_sf, float w_scale, const void* res, int M, int N, int K, long ldy, int mode,
                             int split_k, float* workspace, int* counters, int* status, int sm_count, cudaStream_t s) {
  return gemm_nvfp4_impl(Y, Xq, x_sf, row_scale, Wq, w_sf, w_scale, res, M, N, K, ldy, mode, split_k, workspace,
                         counters, status, sm_count, s, nullptr, 0, nullptr, 0.f, 0);
}

// Decode form (<= 8 rows): bf16 activations in, RMSNorm + NVFP4 quantisation fused into the GEMM kernel.
extern "C" int fb_gemm_nvfp4_fused(void* Y, const void* X, long ldx, const void* norm_w, float eps, const void* Wq,
                                   const void* w_sf, float w_scale, const void* res, int M, int N, int K, long ldy,
                                   int mode, int split_k, int out_f32, float* workspace, int* counters, int* status,
                                   int sm_count, cudaStream_t s) {
  return gemm_nvfp4_impl(Y, nullptr, nullptr, nullptr, Wq, w_sf, w_scale, res, M, N, K, ldy, mode, split_k, workspace,
                         counters, status, sm_count, s, X, ldx, norm_w, eps, out_f32);
}

// Prompt rows: gate|up GEMM + SwiGLU whose epilogue writes the activation already quantised for the down projection
// (codes [M][N / 2], tiled scales of fb_nvfp4_sf_bytes(M, N) bytes, row_scale[m] = q_gs), instead of bf16 rows that a
// second kernel would read back and quantise. `q_gs` is a static global scale (a checkpoint's input scale of the
// down projection, or a default that puts block maxima of 6e-3 .. 168 on normal e4m3 scales). Counterpart of
// `fe_gemm_nvfp4_swiglu` with its fp4 output (`kernels/k-fp4/src/lib.rs:747-764`).
extern "C" int fb_gemm_nvfp4_swiglu_q(void* q_codes, void* q_sf, float* q_row_scale, float q_gs, const void* Xq,
                                      const void* x_sf, const float* row_scale, const void* Wq, const void* w_sf,
                                      float w_scale, int M, int N, int K, int* status, int sm_count, cudaStream_t s) {
  return gemm_nvfp4_impl(q_codes, Xq, x_sf, row_scale, Wq, w_sf, w_scale, nullptr, M, N, K, N, 1, 1, nullptr, nullptr,
                         status, sm_count, s, nullptr, 0, nullptr, 0.f, 0, q_codes, q_sf, q_row_scale, q_gs);
}
