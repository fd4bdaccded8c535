// Causal flash attention for prompt chunks on the 5th-generation tensor cores (tcgen05 + TMEM), over the paged KV cache.
//
// One CTA = 128 query rows of one q head; keys stream in tiles of 64 (one or part of one KV page) through a two-stage
// TMA pipeline. Warp roles: warp 0 lane 0 issues the TMA loads, warp 1 lane 0 issues every tcgen05.mma, warps 2..9
// (256 threads, two per query row = TMEM lane, each taking half of a tile's keys and half of the O columns) run the
// online softmax and the epilogue: two warps per SM sub-partition, so one's TMEM / ex2 latencies hide behind the other.
//
//   S = Q K^T        SS form: Q and K tiles in shared memory (K-major, 128-byte swizzle), S in TMEM (2 buffers x 64 cols)
//   P = exp2(S - m)  softmax threads read S with tcgen05.ld, write P as packed bf16 back into TMEM with tcgen05.st
//   O += P V         TS form: A = P from TMEM, B = the V tile in shared memory read MN-major (V rows are keys, the
//                    head dim is contiguous), O in TMEM (head_dim columns) for the whole key loop
//
// The running maximum only moves when a row's new maximum exceeds it by more than 2^8 (then the O accumulator is
// rescaled in TMEM; between such events P may exceed 1, which bf16 and the fp32 row sum absorb), so the common key
// tile costs one TMEM read of S and one TMEM write of P per thread. Tensor-pipe order is S(0) S(1) PV(0) S(2) PV(1) ...:
// the softmax of tile j overlaps PV(j-1) and S(j+1). Every mbarrier wait is bounded; a wait that runs out sets the
// status word and an abort flag, all roles leave their loops, and the CTA frees its TMEM and returns.
//
// Counterpart of the reference's `fe_flash_prefill` (`kernels/k-core/src/flash.rs:50`: BQ 64 / BKV 32 on mma.sync with
// the gate epilogue); same contract as `fb_attn_prefill` (sigmoid output gate fused, paged cache with a prefix).
#include "api.h"
#include "common.cuh"
#include "gemm_core.cuh"

namespace fb {

constexpr int FT_BQ = 128, FT_BKV = 64, FT_THREADS = 64 + 256;

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// MN-major operand tile with the 128-byte swizzle: rows are K (here: keys), each row holds 64 contiguous MN elements
// (128 bytes). Eight rows form one swizzle atom; SBO = bytes between 8-row groups along K, LBO = bytes between
// 64-element chunks along MN.
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD>
__global__ void __launch_bounds__(FT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out,
                       const __nv_bfloat16* __restrict__ proj, long proj_stride, const int* __restrict__ seg_slot,
                       const int* __restrict__ seg_row0, const int* __restrict__ seg_nrows,
                       const int* __restrict__ seg_pos0, const int* __restrict__ block_table, int max_blocks,
                       int kv_block, int nq, int nkv, int gated, float scale_log2, int* status) {
  constexpr int NCH = HD / 64;                     // 64-element (128-byte) chunks of the head dim
  constexpr int Q_CH = FT_BQ * 128;                // bytes of one Q chunk box (128 rows x 128 B)
  constexpr int KV_CH = FT_BKV * 128;              // bytes of one K / V chunk box (64 rows x 128 B)
  constexpr int Q_BYTES = NCH * Q_CH, KV_BYTES = NCH * KV_CH;
  constexpr uint32_t COL_O = 0, COL_S = HD, COL_P = HD + 2 * FT_BKV;   // TMEM columns: O | S0 S1 | P0 P1
  constexpr uint32_t TMEM_COLS = 512;
  // K runs three tiles ahead at head_dim 256 (S(j+1) is issued a whole tile before PV(j), so with two K buffers a K
  // load had one tile period to arrive and its latency set the pace), four below; V two / three.
  constexpr int KS = HD == 256 ? 3 : 4, VS = HD == 256 ? 2 : 3;
  // All shared state lives in the dynamic allocation (no static shared memory), so the tile area starts at the
  // 1024-byte aligned base: [Q][K x KS][V x VS][row maxima 2 KB][barriers][flags]
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sQ = smem_raw;
  unsigned char* sK = sQ + Q_BYTES;                         // [KS][KV_BYTES]
  unsigned char* sV = sK + KS * KV_BYTES;                   // [VS][KV_BYTES]
  float (*mx_s)[2][FT_BQ] = reinterpret_cast<float (*)[2][FT_BQ]>(sV + VS * KV_BYTES);   // [2][2][128] by tile parity
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + VS * KV_BYTES + 2 * 2 * FT_BQ * 4);
  uint64_t* q_full = bars;
  uint64_t* s_full = bars + 2;                              // [2]
  uint64_t* s_empty = bars + 4;                             // [2]
  uint64_t* p_full = bars + 6;                              // [2]
  uint64_t* p_empty = bars + 8;                             // [2]: PV(j) has completed (P buffer free, O up to date)
  uint64_t* k_full = bars + 10;                             // [KS]
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;                          // [VS]
  uint64_t* v_empty = v_full + VS;
  uint32_t* tmem_base_p = reinterpret_cast<uint32_t*>(v_empty + VS);
  int* abort_p = reinterpret_cast<int*>(tmem_base_p + 1);
  int* fail_s = abort_p + 1;                                // [3]: a softmax wait ran out (tile parity; [2]: after the loop)

  const int seg = blockIdx.z, qh = blockIdx.y;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;      // long (late) query tiles first
  pdl_launch_dependents();
  pdl_wait();
  const int n = seg_nrows[seg];
  const int q0 = qt * FT_BQ;
  if (q0 >= n) return;                                      // uniform for the CTA, before any barrier or allocation
  if (smem_u32(smem_raw) & 1023u) {                         // the swizzled tiles need the 1024-byte base
    if (threadIdx.x == 0) set_status(status, ST_BOUNDS);
    return;
  }
  const int row0 = seg_row0[seg], pos0 = seg_pos0[seg], slot = seg_slot[seg];
  const int kvh = qh / (nq / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = (pos0 + min(q0 + FT_BQ, n) + FT_BKV - 1) / FT_BKV;   // key tiles the last query row of the tile sees
  volatile int* abort_flag = abort_p;

  if (threadIdx.x == 0) {
    *abort_p = 0;
    fail_s[0] = fail_s[1] = fail_s[2] = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 256); mbar_init(&p_full[i], 256); mbar_init(&p_empty[i], 1);
    }
    for (int i = 0; i < KS; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < VS; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_p, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_base_p;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: K(j+1) is issued before V(j), so the K ring really runs KS - 1 tiles ahead ----------------
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_2d(sQ + c * Q_CH, &tmQ, q_full, qh * HD + c * 64, row0 + q0);
      const int* bt = block_table + (size_t)slot * max_blocks;
      int k_armed = 0, v_armed = 0;                           // tiles whose K / V loads were issued
      bool ok = true;
      auto tile_row = [&](int j) -> int {
        const int t0 = j * FT_BKV;
        const int blk = bt[t0 / kv_block];
        return blk < 0 ? -1 : blk * kv_block + t0 % kv_block;
      };
      auto load_k = [&](int j) -> bool {
        const int st = j % KS, krow = tile_row(j);
        if (krow < 0) { set_status(status, ST_BOUNDS); return false; }
        if (j >= KS && !mbar_wait_or_flag(&k_empty[st], ((j / KS) - 1) & 1, abort_flag)) { set_status(status, ST_MBAR_TIMEOUT); return false; }
        mbar_expect_tx(&k_full[st], KV_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_2d(sK + st * KV_BYTES + c * KV_CH, &tmK, &k_full[st], kvh * HD + c * 64, krow);
        k_armed = j + 1;
        return true;
      };
      auto load_v = [&](int j) -> bool {
        const int st = j % VS, krow = tile_row(j);
        if (krow < 0) { set_status(status, ST_BOUNDS); return false; }
        if (j >= VS && !mbar_wait_or_flag(&v_empty[st], ((j / VS) - 1) & 1, abort_flag)) { set_status(status, ST_MBAR_TIMEOUT); return false; }
        mbar_expect_tx(&v_full[st], KV_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_2d(sV + st * KV_BYTES + c * KV_CH, &tmV, &v_full[st], kvh * HD + c * 64, krow);
        v_armed = j + 1;
        return true;
      };
      ok = load_k(0);
      for (int j = 0; ok && j < nt; ++j) {
        if (j + 1 < nt) ok = load_k(j + 1);
        if (ok) ok = load_v(j);
      }
      if (!ok) *abort_p = 1;
      if (*abort_flag) {
        // loads issued by this thread may still be landing: give them a bounded time before the CTA's memory goes away
        mbar_wait(q_full, 0, 1u << 20);
        for (int j = max(0, k_armed - KS); j < k_armed; ++j) mbar_wait(&k_full[j % KS], (j / KS) & 1, 1u << 20);
        for (int j = max(0, v_armed - VS); j < v_armed; ++j) mbar_wait(&v_full[j % VS], (j / VS) & 1, 1u << 20);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ---------------------------------------------------------------------------------------
      constexpr uint32_t idesc_s = umma_idesc(1, 1, FT_BQ, FT_BKV);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, FT_BQ, HD) | (1u << 16);     // B read MN-major
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait_or_flag(q_full, 0, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1, st = j % KS;
        if (!mbar_wait_or_flag(&k_full[st], (j / KS) & 1, abort_flag)) return false;
        if (j >= 2 && !mbar_wait_or_flag(&s_empty[s], ((j >> 1) - 1) & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk & 3) * 32u;
          tc_mma_f16(tmem + COL_S + s * FT_BKV, umma_desc_k128(aQ + (kk >> 2) * Q_CH + off),
                     umma_desc_k128(aK + st * KV_BYTES + (kk >> 2) * KV_CH + off), idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[s]);
        tc_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < nt; ++j) {
        const int s = j & 1, st = j % VS;
        if (j + 1 < nt && !issue_s(j + 1)) { ok = false; break; }
        if (!mbar_wait_or_flag(&p_full[s], (j >> 1) & 1, abort_flag) ||
            !mbar_wait_or_flag(&v_full[st], (j / VS) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < FT_BKV / 16; ++kk)
          tc_mma_f16_ts(tmem + COL_O, tmem + COL_P + s * (FT_BKV / 2) + kk * 8,
                        umma_desc_mn128(aV + st * KV_BYTES + kk * 16 * 128, KV_CH, 1024), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        tc_commit(&v_empty[st]);
        tc_commit(&p_empty[s]);
      }
      if (!ok) { set_status(status, ST_MBAR_TIMEOUT); *abort_p = 1; }
    }
  } else {
    // ---- softmax + epilogue: two threads per query row (warps 2..5 take keys 0..31 of a tile, warps 6..9 keys 32..63;
    // a row's two threads sit in the same TMEM lane quadrant) -----------------------------------------------------
    // The halves of a row exchange their tile maxima through shared memory around a named barrier of the 256 softmax
    // threads. A failed wait is published through fail_s BEFORE that barrier and acted on AFTER it, so the 256 threads
    // always leave the loop in the same iteration and nobody is left alone at the barrier.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int qpos = pos0 + q0 + row;
    constexpr int HC = FT_BKV / 2;                          // keys per thread and tile
    constexpr int OC = HD / 2;                              // O columns per thread (rescale, epilogue)
    float m_ref = -INFINITY, l = 0.f;
    bool broke = false;
    bool late_fail = false;                                 // a wait after the barrier ran out: reported at the next one
    for (int j = 0; j < nt; ++j) {
      const int s = j & 1;
      bool ok = !late_fail && mbar_wait_or_flag(&s_full[s], (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      uint32_t sr[HC];
      float mx = -INFINITY;
      if (ok) {
        tc_fence_after();
        tmem_ld32(tmem + lane_addr + COL_S + s * FT_BKV + half * HC, sr);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_empty[s]);
        const int t0 = j * FT_BKV + half * HC;
        const bool need_mask = t0 + HC - 1 > pos0 + q0;
#pragma unroll
        for (int c = 0; c < HC; ++c) {
          float v = __uint_as_float(sr[c]) * scale_log2;
          if (need_mask && t0 + c > qpos) v = -INFINITY;
          sr[c] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      } else {
        fail_s[s] = 1;
      }
      mx_s[s][half][row] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (fail_s[s]) { broke = true; break; }
      mx = fmaxf(mx, mx_s[s][half ^ 1][row]);               // the row's maximum over the whole tile
      const bool any = __any_sync(0xffffffffu, mx > m_ref + 8.f);
      // The P buffer of this parity was last read by PV(j-2); O may only be rescaled once PV(j-1) has completed. Both
      // are phases of p_empty; neither wait sits on the common path's critical chain (PV(j-1) runs while this tile's
      // softmax does, and P(j) is handed over without waiting for it).
      ok = true;
      if (j >= 2) ok = mbar_wait_or_flag(&p_empty[s], ((j >> 1) - 1) & 1, abort_flag);
      if (ok && any && j > 0) ok = mbar_wait_or_flag(&p_empty[s ^ 1], ((j - 1) >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { late_fail = true; continue; }
      tc_fence_after();
      if (any) {
        const float m_new = fmaxf(m_ref, mx);
        const float f = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
        l *= f;
        if (j > 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < OC; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tmem + lane_addr + COL_O + half * OC + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
            tmem_st32(tmem + lane_addr + COL_O + half * OC + c0, o);
          }
          tmem_st_wait();
        }
        m_ref = m_new;
      }
      const float mr = (m_ref == -INFINITY) ? 0.f : m_ref;
      uint32_t pr[HC / 2];
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < HC / 2; ++c) {
        const float p0 = fast_exp2(__uint_as_float(sr[2 * c]) - mr);
        const float p1 = fast_exp2(__uint_as_float(sr[2 * c + 1]) - mr);
        sum += p0 + p1;
        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);     // .x (low half) = even key
        pr[c] = *reinterpret_cast<uint32_t*>(&h);
      }
      l += sum;
      tmem_st16(tmem + lane_addr + COL_P + s * (FT_BKV / 2) + half * (HC / 2), pr);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
    }
    // final hand-over: the row sum of the other half, and agreement on whether the output is complete
    bool ok = !broke && !late_fail;
    if (ok) ok = mbar_wait_or_flag(&p_empty[(nt - 1) & 1], ((nt - 1) >> 1) & 1, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) fail_s[2] = 1;
    // row sums go through the maxima buffer of the parity the last tile did NOT use: nobody reads that one any more
    float (*l_s)[FT_BQ] = mx_s[nt & 1];
    l_s[half][row] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!fail_s[2]) {
      tc_fence_after();
      const float lt = l + l_s[half ^ 1][row];
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      const bool valid = q0 + row < n;
      const size_t grow = (size_t)(row0 + q0 + row);
      __nv_bfloat16* dst = out + grow * (size_t)nq * HD + (size_t)qh * HD + half * OC;
      const __nv_bfloat16* gate = proj + grow * proj_stride + (size_t)qh * 2 * HD + HD + half * OC;
#pragma unroll 1
      for (int c0 = 0; c0 < OC; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_addr + COL_O + half * OC + c0, o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint32_t w[4];
            uint4 g4 = make_uint4(0, 0, 0, 0);
            if (gated) g4 = *reinterpret_cast<const uint4*>(gate + c0 + v4 * 8);
            const uint32_t gu[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float a = __uint_as_float(o[v4 * 8 + 2 * e]) * inv, b = __uint_as_float(o[v4 * 8 + 2 * e + 1]) * inv;
              if (gated) { a *= sigmoidf_(bf_lo(gu[e])); b *= sigmoidf_(bf_hi(gu[e])); }
              __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
              w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(dst + c0 + v4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    } else if (threadIdx.x == 64) {
      set_status(status, ST_MBAR_TIMEOUT);
      *abort_p = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace fb

using namespace fb;

// q: [q_rows][nq*hd] bf16 (post norm / RoPE); caches: [cache_rows = blocks*kv_block][nkv*hd] bf16; same outputs as
// fb_attn_prefill. Returns -20 when the shape is outside what this kernel takes (the caller uses fb_attn_prefill).
extern "C" int fb_attn_prefill_tc(void* out, const void* q, const void* k_cache, const void* v_cache, const void* proj,
                                  long proj_stride, const int* seg_slot, const int* seg_row0, const int* seg_nrows,
                                  const int* seg_pos0, const int* block_table, int max_blocks, int kv_block, int nseg,
                                  int max_rows, long q_rows, long cache_rows, int nq, int nkv, int hd, int gated,
                                  int* status, cudaStream_t s) {
  if (nseg <= 0 || max_rows <= 0) return 0;
  if (nq % nkv) return -1;
  if ((hd != 64 && hd != 128 && hd != 256) || kv_block % FT_BKV) return -20;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tmQ, q, (uint64_t)q_rows, (uint64_t)nq * hd, (uint64_t)nq * hd, FT_BQ))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmK, k_cache, (uint64_t)cache_rows, (uint64_t)nkv * hd, (uint64_t)nkv * hd, FT_BKV))) return rc;
  if ((rc = make_tmap_bf16_2d(&tmV, v_cache, (uint64_t)cache_rows, (uint64_t)nkv * hd, (uint64_t)nkv * hd, FT_BKV))) return rc;
  dim3 grid((max_rows + FT_BQ - 1) / FT_BQ, nq, nseg);
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
#define FB_FT(HDV)                                                                                                 \
  {                                                                                                                \
    const size_t smem = (size_t)(FT_BQ + ((HDV == 256 ? 3 : 4) + (HDV == 256 ? 2 : 3)) * FT_BKV) * HDV * 2 + 2048 + 512;                                             \
    auto kern = attn_prefill_tc_kernel<HDV>;                                                                       \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    if (e != cudaSuccess) return (int)e;                                                                           \
    launch_pdl(kern, grid, dim3(FT_THREADS), smem, s, tmQ, tmK, tmV, (__nv_bfloat16*)out, (const __nv_bfloat16*)proj, \
               proj_stride, seg_slot, seg_row0, seg_nrows, seg_pos0, block_table, max_blocks, kv_block, nq, nkv,   \
               gated, scale_log2, status);                                                                         \
  }
  if (hd == 256) FB_FT(256) else if (hd == 128) FB_FT(128) else FB_FT(64)
#undef FB_FT
  return (int)cudaGetLastError();
}
