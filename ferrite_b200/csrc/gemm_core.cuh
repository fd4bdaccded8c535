// bf16 GEMM on the 5th-generation tensor cores: Y[M][N] = X[M][K] * W[N][K]^T with fp32 accumulation in TMEM.
//
// One persistent, warp-specialised kernel: warp 0 drives TMA (cp.async.bulk.tensor, 128-byte swizzle, no
// multicast), warp 1 owns TMEM and issues tcgen05.mma from one elected thread, warps 2-5 drain the accumulator
// with tcgen05.ld and run the epilogue (bf16 store, + residual, or SwiGLU over a gate|up weight). Two
// accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
//
// Two orientations share the code, because both operands are K-major and UMMA N is a run-time field of the
// instruction descriptor:
//   normal (M > 64): A = 128 token rows, B = 256 output features (or 128 gate + 128 up rows for SwiGLU).
//   swapped (M <= 64, decode / verify rows): A = 128 output features, B = the token rows (N = 16..64), with
//     deterministic split-K so the few weight tiles still cover every SM; partial tiles go to an fp32
//     workspace and the last CTA of a tile sums them in split order.
//
// Replaces `fe_gemm_bf16`, `fe_gemm_swiglu` (`kernels/k-core/src/gemm.rs:113-285`, mma.sync m16n8k16 with
// cp.async) and `ggq_gemm16_bf16_*` (`kernels/k-gguf/src/gemm16.rs:121`).
//
// The kernel is a template over a communication mode so the tensor-parallel variants (reduce-scatter epilogue,
// all-gather prologue; gemm_comm.cu) share the pipeline with the single-GPU GEMM (gemm_tcgen05.cu).
#pragma once
#include <cuda.h>

#include "api.h"
#include "common.cuh"

namespace fb {

constexpr int GM_BM = 128;        // UMMA M (rows of the A box)
constexpr int GM_BK = 64;         // k elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int GM_MAX_STAGES = 8;
constexpr int GM_THREADS = 192;
constexpr int GM_A_BYTES = GM_BM * GM_BK * 2;   // 16 KB

// Communication fused into the kernel (template parameter COMM):
//   0  none
//   1  reduce-scatter epilogue: bf16 partial tiles are stored into the row owner's staging slot over NVLink, a flag
//      per (source rank, tile) is released, and after its GEMM work every CTA reduces tiles of the rows this rank owns
//      (rank order, + residual) into the local output shard
//   2  all-gather prologue: two extra warps per CTA pull the peers' row shards of X into this GPU's full-X buffer
//      with plain peer loads while the tensor cores work on the rows already present; the TMA producer waits for a
//      row tile's arrival count before loading it
struct GemmComm {
  void* peer[8];            // base of the large symmetric workspace on every rank (peer[rank] = local)
  int rank, world;
  int rows_per_rank;        // Ms: rank o owns rows [o * Ms, (o + 1) * Ms)
  uint32_t* ctr;            // local: [0] call counter (epoch), [1] CTAs finished, [2..] per-row-tile arrival counts
  unsigned spin_limit;
  long flags_off;           // u32 [2 parity][8 src][max_tiles]
  long ready_off;           // u32 [8 src]: epoch in which that rank's X shard became readable
  long stage_off;           // bf16 [2 parity][world src][slot_elems]
  long slot_elems;
  long xfull_off;           // bf16 [M][K] gathered X
  int max_tiles;
  __nv_bfloat16* y_shard;   // mode 1: local output [Ms][N]
  const __nv_bfloat16* res_shard;   // mode 1: local residual [Ms][N] or null
};

//   3  grouped (mixture-of-experts): the rows of X are sorted by expert; row tile -> expert comes from two device
//      tables (prefix sums of rows and of 128-row tiles per expert), each expert multiplies by its own weight block
struct GemmGroups {
  const int* tile_start;    // [experts + 1] prefix sum of 128-row tiles
  const int* row_base;      // [experts + 1] prefix sum of rows
  int experts;
  int w_rows;               // weight rows per expert in the stacked [experts * w_rows][K] matrix
  int uniform_rows;         // > 0: every group has this many rows (batched GEMM); the two prefix arrays are not read
};

struct GemmArgs {
  GemmComm cm;
  GemmGroups gr;
  // FP8 (e4m3) operands on kind::f8f6f4: one stage still holds 128 bytes of K per row (128 elements instead of 64),
  // so the shared-memory layout, the descriptors and their k advance are those of the bf16 path. The epilogue
  // multiplies by a per-token-row and a per-output-feature scale (either may be null).
  int fp8;
  const float* scale_m;     // [M]
  const float* scale_n;     // [N] (SwiGLU: [2N], gate features then up features)
  int out_f32;              // Y is fp32 [M][ldy] instead of bf16 (router logits, lm_head rows)
  void* Y;
  const __nv_bfloat16* res;
  float* workspace;
  int* counters;
  int* status;
  int M, N, K;              // problem: Y is [M][N]
  long ldy;
  int swap;                 // 1: A operand = weights, B = activations
  int dual;                 // SwiGLU: two weight row blocks (gate at n, up at N + n)
  int bn;                   // UMMA N per MMA (columns of one accumulator)
  int n_a;                  // A boxes per stage (2 for swapped SwiGLU)
  int n_b;                  // B boxes per stage (2 for normal SwiGLU)
  int b_box_rows;           // rows per B box
  int stages;
  int split_k;
  int tiles_a, tiles_b;     // tile counts along the A-row and B-row dimensions
  int acc_cols;             // TMEM columns per accumulator buffer (n_a * bn)
  int tmem_cols;            // allocated columns (power of two >= 2 * acc_cols)
};

__device__ __forceinline__ bool mbar_wait_or_flag(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
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

constexpr int GM_COPY_WARPS = 2;   // mode 2: warps 6 and 7 gather remote rows
constexpr int GM_COPY_COLS = 512;  // columns of X per gather work item (two 16-byte loads per lane and row)
constexpr int GM_RS_COLS = 128;   // mode 1: columns staged per warp before the coalesced peer stores
constexpr int GM_COPY_ROWS = 8;    // rows per gather work item: 16 loads of 16 bytes in flight per lane

__device__ __forceinline__ uint32_t* gc_flag(void* base, const GemmComm& cm, int parity, int src, int tile) {
  return reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(base) + cm.flags_off) +
         ((size_t)parity * 8 + src) * cm.max_tiles + tile;
}
__device__ __forceinline__ __nv_bfloat16* gc_stage(void* base, const GemmComm& cm, int parity, int src) {
  return reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(base) + cm.stage_off) +
         ((size_t)parity * cm.world + src) * cm.slot_elems;
}

template <int COMM>
__global__ void __launch_bounds__(COMM == 2 ? GM_THREADS + 32 * GM_COPY_WARPS : GM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[GM_MAX_STAGES], empty_bar[GM_MAX_STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int last_flag_s;

  // 1024-byte aligned tile area (the swizzle atom is 8 rows x 128 B)
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b_bytes = a.n_b * a.b_box_rows * GM_BK * 2;
  const int stage_bytes = a.n_a * GM_A_BYTES + ((b_bytes + 1023) & ~1023);
  const int bk_elems = a.fp8 ? 2 * GM_BK : GM_BK;
  const int kblocks_total = (a.K + bk_elems - 1) / bk_elems;
  const int kb_per_split = (kblocks_total + a.split_k - 1) / a.split_k;
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
  uint32_t epoch = 0;
  int parity = 0;
  // Row-tile order of the communicating modes. The row tiles are walked as a ring that starts just after this
  // rank's own tiles (mode 1: own rows LAST, so every peer's partial for them is already staged when their epilogue
  // adds it up, and no rank ever waits inside a tile another rank is waiting for) or at its own tiles (mode 2: own
  // rows FIRST, they need no transfer). The ring is cut into two phases (own / not own) and each phase into groups of
  // `gs` row tiles; inside a group the row tiles vary fastest so the CTAs running together share weight panels.
  int seq0 = 0, n_first = 0, gs = 1, groups_first = 0, total_work = a.tiles_a * a.tiles_b * a.split_k;
  if constexpr (COMM == 3)
    total_work = (a.gr.uniform_rows > 0 ? a.gr.experts * ((a.gr.uniform_rows + GM_BM - 1) / GM_BM)
                                        : a.gr.tile_start[a.gr.experts]) * a.tiles_b;
  if constexpr (COMM == 1 || COMM == 2) {
    epoch = *reinterpret_cast<volatile uint32_t*>(&a.cm.ctr[0]) + 1;
    parity = (int)(epoch & 1u);
    const int my0 = min(a.M, a.cm.rank * a.cm.rows_per_rank), my1 = min(a.M, my0 + a.cm.rows_per_rank);
    const int t_lo = my0 / GM_BM, t_hi = my1 > my0 ? (my1 - 1) / GM_BM : t_lo - 1;
    const int n_own = t_hi - t_lo + 1;
    if (COMM == 1) { seq0 = (t_hi + 1) % a.tiles_a; n_first = a.tiles_a - n_own; }
    else { seq0 = t_lo % a.tiles_a; n_first = n_own; }
    gs = max(1, a.cm.rows_per_rank / GM_BM);
    groups_first = (n_first + gs - 1) / gs;
    const int groups_second = (a.tiles_a - n_first + gs - 1) / gs;
    total_work = (groups_first + groups_second) * gs * a.tiles_b;      // padded: short groups leave invalid items
  }
  (void)parity;

  // work item -> (tile along A rows, tile along B rows, k split); A-row tiles vary fastest in the normal
  // orientation so CTAs running together share weight panels through L2.
  int g_row0 = 0, g_row_end = 0, g_wrow = 0;          // grouped mode: set by decode_work
  auto decode_work = [&](int w, int& ta, int& tb, int& ks) -> bool {
    if constexpr (COMM == 3) {
      ks = 0;
      ta = w / a.tiles_b;                              // global row tile; weight panels of one row tile run together
      tb = w % a.tiles_b;
      if (a.gr.uniform_rows > 0) {
        const int per = (a.gr.uniform_rows + GM_BM - 1) / GM_BM, g = ta / per;
        g_row0 = g * a.gr.uniform_rows + (ta - g * per) * GM_BM;
        g_row_end = min((g + 1) * a.gr.uniform_rows, a.M);
        g_wrow = g * a.gr.w_rows;
        return true;
      }
      int lo = 0, hi = a.gr.experts;                   // last expert whose first tile is <= ta
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (a.gr.tile_start[mid] <= ta) lo = mid; else hi = mid;
      }
      g_row0 = a.gr.row_base[lo] + (ta - a.gr.tile_start[lo]) * GM_BM;
      g_row_end = min(a.gr.row_base[lo + 1], a.M);     // a.M = capacity of the row buffers
      g_wrow = lo * a.gr.w_rows;
      return true;
    }
    if constexpr (COMM == 1 || COMM == 2) {
      ks = 0;
      const int pos = w / (gs * a.tiles_b), rem = w % (gs * a.tiles_b);
      int base, sz;
      if (pos < groups_first) { base = pos * gs; sz = min(gs, n_first - base); }
      else { base = n_first + (pos - groups_first) * gs; sz = min(gs, a.tiles_a - base); }
      if (rem >= sz * a.tiles_b) return false;
      ta = (seq0 + base + rem % sz) % a.tiles_a;
      tb = rem / sz;
      return true;
    }
    ks = w % a.split_k;
    int t = w / a.split_k;
    if (a.swap) { tb = t % a.tiles_b; ta = t / a.tiles_b; }
    else { ta = t % a.tiles_a; tb = t / a.tiles_a; }
    return true;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0; uint32_t phase = 0;
      const uint32_t tx = (uint32_t)(a.n_a * GM_A_BYTES + b_bytes);
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int ta, tb, ks;
        if (!decode_work(w, ta, tb, ks)) continue;
        const int kb0 = ks * kb_per_split, kb1 = min(kblocks_total, kb0 + kb_per_split);
        if constexpr (COMM == 2) {
          // rows of this tile that live on other ranks must have arrived in the local full-X buffer
          const int trows = min(GM_BM, a.M - ta * GM_BM);
          const uint32_t want = (uint32_t)(((a.K + GM_COPY_COLS - 1) / GM_COPY_COLS) *
                                           ((trows + GM_COPY_ROWS - 1) / GM_COPY_ROWS));
          bool here = false;
          for (uint32_t i = 0; i < a.cm.spin_limit; ++i) {
            if (ld_acquire_gpu(&a.cm.ctr[2 + ta]) >= want) { here = true; break; }
            if ((i & 1023u) == 1023u && *abort_flag) break;
          }
          if (!here) { set_status(a.status, ST_PEER_TIMEOUT); ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_or_flag(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          unsigned char* sa = tiles + (size_t)stage * stage_bytes;
          unsigned char* sb = sa + a.n_a * GM_A_BYTES;
          mbar_expect_tx(&full_bar[stage], tx);
          const int kx = kb * bk_elems;
          // A boxes: swapped SwiGLU loads gate rows and up rows (N apart) as two boxes
          for (int i = 0; i < a.n_a; ++i)
            tma_load_2d(sa + i * GM_A_BYTES, &tmA, &full_bar[stage], kx, (COMM == 3 ? g_row0 : ta * GM_BM) + i * a.N);
          // B boxes: normal SwiGLU stacks 128 gate rows and 128 up rows into one N = 256 operand
          for (int i = 0; i < a.n_b; ++i)
            tma_load_2d(sb + (size_t)i * a.b_box_rows * GM_BK * 2, &tmB, &full_bar[stage], kx,
                        tb * a.b_box_rows + i * a.N + (COMM == 3 ? g_wrow : 0));
          if (++stage == a.stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
    }
  } else if (COMM == 2 && warp >= 6) {
    // ---------------- gather warps: peers' row shards of X -> local full-X buffer ----------------
    const GemmComm& cm = a.cm;
    if (blockIdx.x == 0 && warp == 6 && lane < cm.world)
      st_release_sys(reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(cm.peer[lane]) + cm.ready_off) + cm.rank, epoch);
    const int n_kc = (a.K + GM_COPY_COLS - 1) / GM_COPY_COLS;
    const int gw = blockIdx.x * GM_COPY_WARPS + (warp - 6), nw = gridDim.x * GM_COPY_WARPS;
    const uint32_t* ready = reinterpret_cast<const uint32_t*>(reinterpret_cast<char*>(cm.peer[cm.rank]) + cm.ready_off);
    __nv_bfloat16* xl = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(cm.peer[cm.rank]) + cm.xfull_off);
    uint32_t seen = 1u << cm.rank;
    bool ok = true;
    constexpr int RG = GM_BM / GM_COPY_ROWS;          // row groups per tile
    for (int item = gw; item < a.tiles_a * RG * n_kc && ok; item += nw) {
      const int ta = (item / (RG * n_kc) + seq0) % a.tiles_a;     // same ring order as the consumers
      const int rg = (item / n_kc) % RG, kc = item % n_kc;
      const int mb = ta * GM_BM + rg * GM_COPY_ROWS;
      if (mb >= a.M) continue;                        // row group past the end of the last tile: not counted
      const int m1 = min(a.M, mb + GM_COPY_ROWS);
      const int c0 = kc * GM_COPY_COLS;
      uint4 v[2 * GM_COPY_ROWS];
      bool on[2 * GM_COPY_ROWS];
#pragma unroll
      for (int q = 0; q < 2 * GM_COPY_ROWS; ++q) {
        const int m = mb + (q >> 1), c = c0 + ((q & 1) * 32 + lane) * 8;
        on[q] = false;
        if (ok && m < m1 && c < a.K) {
          const int o = m / cm.rows_per_rank;
          if (o != cm.rank) {
            if (!((seen >> o) & 1u)) {
              if (!wait_flag_ge(ready + o, epoch, cm.spin_limit)) ok = false;
              seen |= 1u << o;
            }
            if (ok) {
              const __nv_bfloat16* xr = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const char*>(cm.peer[o]) + cm.xfull_off);
              v[q] = __ldcg(reinterpret_cast<const uint4*>(xr + (size_t)m * a.K + c));
              on[q] = true;
            }
          }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#pragma unroll
      for (int q = 0; q < 2 * GM_COPY_ROWS; ++q) {
        const int m = mb + (q >> 1), c = c0 + ((q & 1) * 32 + lane) * 8;
        if (on[q]) *reinterpret_cast<uint4*>(xl + (size_t)m * a.K + c) = v[q];
      }
      __threadfence();
      __syncwarp();
      if (lane == 0) atomicAdd(&a.cm.ctr[2 + ta], 1u);
    }
    if (!ok && lane == 0) { set_status(a.status, ST_PEER_TIMEOUT); abort_s = 1; }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      const uint32_t idesc = a.fp8 ? umma_idesc(0, 0, GM_BM, (uint32_t)a.bn) : umma_idesc(1, 1, GM_BM, (uint32_t)a.bn);
      int stage = 0; uint32_t phase = 0;
      int buf = 0; uint32_t tphase[2] = {0, 0};
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int ta, tb, ks;
        if (!decode_work(w, ta, tb, ks)) continue;
        const int kb0 = ks * kb_per_split, kb1 = min(kblocks_total, kb0 + kb_per_split);
        if (!mbar_wait_or_flag(&tempty_bar[buf], tphase[buf] ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(buf * a.acc_cols);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_or_flag(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint32_t sb = sa + a.n_a * GM_A_BYTES;
          const uint64_t db = umma_desc_k128(sb);
          for (int i = 0; i < a.n_a; ++i) {
            const uint64_t da = umma_desc_k128(sa + i * GM_A_BYTES);
#pragma unroll
            for (int k = 0; k < GM_BK / 16; ++k)
              if (a.fp8)
                tc_mma_f8f6f4(d0 + (uint32_t)(i * a.bn), da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                              (kb > kb0 || k > 0) ? 1u : 0u);
              else
                tc_mma_f16(d0 + (uint32_t)(i * a.bn), da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                           (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);               // frees the smem slot once these MMAs have read it
          if (++stage == a.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[buf]);                   // accumulator complete
        tphase[buf] ^= 1u;
        buf ^= 1;
      }
      if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
    }
  } else {
    // ---------------- epilogue: warps 2..5, lane quadrant = warp % 4 ----------------
    const int quad = warp & 3;
    const int etid = quad * 32 + lane;                // 0..127: the accumulator lane this thread reads
    int buf = 0; uint32_t tphase[2] = {0, 0};
    bool ok = true;
    __nv_bfloat16* Yb = reinterpret_cast<__nv_bfloat16*>(a.Y);
    // mode 1: per-warp transpose buffer behind the pipeline stages (32 rows x GM_RS_COLS bf16)
    unsigned char* tbuf = tiles + (size_t)a.stages * stage_bytes + (size_t)quad * (32 * GM_RS_COLS * 2);
    (void)tbuf;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      int ta, tb, ks;
      if (!decode_work(w, ta, tb, ks)) continue;
      ok = mbar_wait_or_flag(&tfull_bar[buf], tphase[buf], abort_flag);
      if (a.split_k > 1 || COMM == 1) {
        // the four epilogue warps meet at named barriers below: agree on the outcome before anyone leaves
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
      if constexpr (COMM == 1) {
        // Reduce-scatter epilogue (normal orientation, lanes = token rows). Rows owned by other ranks: bf16 partials
        // go through this warp's transpose buffer and leave as 256-byte row pieces for the owner's staging slot of
        // this source rank, then one release flag per (owner, tile). Rows this rank owns (they come last in the tile
        // order): wait for the other ranks' flags of this tile, add their staged partials in rank order to the fp32
        // accumulator, add the residual, store the final bf16 rows of the local output shard.
        const GemmComm& cm = a.cm;
        const int Ms = cm.rows_per_rank;
        const int m = ta * GM_BM + etid;
        const int ncols_out = a.bn;
        const int n0 = tb * ncols_out;
        const int tile_id = ta * a.tiles_b + tb;
        const int row_end = min(a.M, ta * GM_BM + GM_BM);
        const int o_lo = (ta * GM_BM) / Ms, o_hi = (row_end - 1) / Ms;
        const bool has_remote = o_lo != cm.rank || o_hi != cm.rank;
        const bool has_own = o_lo <= cm.rank && cm.rank <= o_hi;
        const bool mine = m < a.M && m / Ms == cm.rank;
        if (has_remote) {
          for (int c = 0; c < ncols_out; c += 32) {
            uint32_t r0[32];
            tmem_ld32(tbase + (uint32_t)c, r0);
            tmem_ld_wait();
            if (m < a.M && !mine) {
              // 16-byte slots XOR-swizzled by row inside each 128-byte group: the row-per-lane writes here and the
              // row-contiguous reads below are both free of bank conflicts
              unsigned char* tb_row = tbuf + (size_t)lane * (GM_RS_COLS * 2);
              const int cbase = (c % GM_RS_COLS) / 8;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int slot = cbase + q;
                const int phys = (slot & ~7) | ((slot & 7) ^ (lane & 7));
                *reinterpret_cast<uint4*>(tb_row + phys * 16) = make_uint4(
                    pack_bf2(__uint_as_float(r0[q * 8]), __uint_as_float(r0[q * 8 + 1])),
                    pack_bf2(__uint_as_float(r0[q * 8 + 2]), __uint_as_float(r0[q * 8 + 3])),
                    pack_bf2(__uint_as_float(r0[q * 8 + 4]), __uint_as_float(r0[q * 8 + 5])),
                    pack_bf2(__uint_as_float(r0[q * 8 + 6]), __uint_as_float(r0[q * 8 + 7])));
              }
            }
            if (((c + 32) % GM_RS_COLS) == 0 || c + 32 >= ncols_out) {
              __syncwarp();
              const int cgrp = (c / GM_RS_COLS) * GM_RS_COLS;
              const int slots = min(GM_RS_COLS, ncols_out - cgrp) / 8;
              const int slot = lane & 15;
#pragma unroll 4
              for (int rr = 0; rr < 32; rr += 2) {
                const int row = rr + (lane >> 4);
                const int mm = ta * GM_BM + quad * 32 + row;
                const int nn = n0 + cgrp + slot * 8;
                const int o = mm / Ms;
                if (mm < a.M && o != cm.rank && nn < a.N && slot < slots) {
                  const int phys = (slot & ~7) | ((slot & 7) ^ (row & 7));
                  const uint4 val = *reinterpret_cast<const uint4*>(tbuf + (size_t)row * (GM_RS_COLS * 2) + phys * 16);
                  __nv_bfloat16* dst = gc_stage(cm.peer[o], cm, parity, cm.rank) + (size_t)(mm - o * Ms) * a.N + nn;
                  *reinterpret_cast<uint4*>(dst) = val;
                }
              }
              __syncwarp();
            }
          }
          __threadfence_system();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (etid <= o_hi - o_lo && o_lo + etid != cm.rank)
            st_release_sys(gc_flag(cm.peer[o_lo + etid], cm, parity, cm.rank, tile_id), epoch);
        }
        if (has_own) {
          uint32_t good = 1;
          if (etid < cm.world && etid != cm.rank)
            good = wait_flag_ge(gc_flag(cm.peer[cm.rank], cm, parity, etid, tile_id), epoch, cm.spin_limit) ? 1u : 0u;
          uint32_t all_ok;
          asm volatile(
              "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.red.and.pred p, 1, 128, q;\n\t"
              "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(all_ok) : "r"(good) : "memory");
          if (!all_ok) {
            ok = false;
            set_status(a.status, ST_PEER_TIMEOUT);
          } else {
            const int lr = m - cm.rank * Ms;
            for (int c = 0; c < ncols_out; c += 32) {
              uint32_t r0[32];
              tmem_ld32(tbase + (uint32_t)c, r0);
              tmem_ld_wait();
              const int n = n0 + c;
              if (mine && n < a.N) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r0[j]);
                const int nv = min(32, a.N - n) / 8;                  // 16-byte pieces of this row inside N
                for (int src = 0; src < cm.world; ++src) {
                  if (src == cm.rank) continue;
                  const uint4* sp = reinterpret_cast<const uint4*>(gc_stage(cm.peer[cm.rank], cm, parity, src) +
                                                                   (size_t)lr * a.N + n);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    if (q < nv) {
                      const uint4 raw = __ldcg(sp + q);
                      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                      for (int j = 0; j < 4; ++j) { v[q * 8 + 2 * j] += bf_lo(u[j]); v[q * 8 + 2 * j + 1] += bf_hi(u[j]); }
                    }
                  }
                }
                if (cm.res_shard) {
                  const uint4* rp = reinterpret_cast<const uint4*>(cm.res_shard + (size_t)lr * a.N + n);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    if (q < nv) {
                      const uint4 raw = rp[q];
                      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                      for (int j = 0; j < 4; ++j) { v[q * 8 + 2 * j] += bf_lo(u[j]); v[q * 8 + 2 * j + 1] += bf_hi(u[j]); }
                    }
                  }
                }
                uint4* yp = reinterpret_cast<uint4*>(cm.y_shard + (size_t)lr * a.N + n);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  if (q < nv)
                    yp[q] = make_uint4(pack_bf2(v[q * 8], v[q * 8 + 1]), pack_bf2(v[q * 8 + 2], v[q * 8 + 3]),
                                       pack_bf2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf2(v[q * 8 + 6], v[q * 8 + 7]));
              }
            }
          }
        }
        tc_fence_before();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        if (!ok) break;
      } else if (!a.swap) {
        // lanes = token rows, columns = output features
        const int m = (COMM == 3 ? g_row0 : ta * GM_BM) + etid;
        const int m_end = COMM == 3 ? g_row_end : a.M;
        const int ncols_out = a.dual ? a.bn / 2 : a.bn;
        const int n0 = tb * ncols_out;
        for (int c = 0; c < ncols_out; c += 32) {
          uint32_t r0[32], r1[32];
          tmem_ld32(tbase + (uint32_t)c, r0);
          if (a.dual) tmem_ld32(tbase + (uint32_t)(c + a.bn / 2), r1);
          tmem_ld_wait();
          if (m < m_end) {
            const int n = n0 + c;
            float v[32];
#pragma unroll
            const float sm_row = a.scale_m ? a.scale_m[m] : 1.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = __uint_as_float(r0[j]) * sm_row;
              float u = a.dual ? __uint_as_float(r1[j]) * sm_row : 0.f;
              if (a.scale_n && n + j < a.N) {
                x *= a.scale_n[n + j];
                if (a.dual) u *= a.scale_n[a.N + n + j];
              }
              v[j] = a.dual ? siluf_(x) * u : x;
            }
            if (n + 32 <= a.N) {
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
              if (a.out_f32) {
                float4* yf = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.Y) + (size_t)m * a.ldy + n);
#pragma unroll
                for (int q = 0; q < 8; ++q) yf[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              } else {
                uint4* yp = reinterpret_cast<uint4*>(Yb + (size_t)m * a.ldy + n);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  yp[q] = make_uint4(pack_bf2(v[q * 8], v[q * 8 + 1]), pack_bf2(v[q * 8 + 2], v[q * 8 + 3]),
                                     pack_bf2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf2(v[q * 8 + 6], v[q * 8 + 7]));
              }
            } else {
              for (int j = 0; j < 32 && n + j < a.N; ++j) {
                float x = v[j];
                if (a.res) x += bf2f(a.res[(size_t)m * a.ldy + n + j]);
                if (a.out_f32) reinterpret_cast<float*>(a.Y)[(size_t)m * a.ldy + n + j] = x;
                else Yb[(size_t)m * a.ldy + n + j] = f2bf(x);
              }
            }
          }
        }
        tc_fence_before();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      } else {
        // lanes = output features, columns = token rows
        const int n = ta * GM_BM + etid;
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
                  const float sc = (a.scale_m ? a.scale_m[m] : 1.f);
                  float x = __uint_as_float(r0[j]) * sc * (a.scale_n ? a.scale_n[n] : 1.f);
                  if (a.dual) x = siluf_(x) * (__uint_as_float(r1[j]) * sc * (a.scale_n ? a.scale_n[a.N + n] : 1.f));
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
          // split-K: park the fp32 partial, count arrivals, the last CTA of the tile reduces in split order
          const int tile_id = ta * a.tiles_b + tb;
          const int cols = a.acc_cols;                      // n_a * bn columns
          float* ws = a.workspace + ((size_t)(tile_id * a.split_k + ks) * cols) * GM_BM;
          for (int c = 0; c < cols; c += 16) {
            uint32_t r0[16];
            tmem_ld16(tbase + (uint32_t)c, r0);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) ws[(size_t)(c + j) * GM_BM + etid] = __uint_as_float(r0[j]);
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
            const float* wt = a.workspace + ((size_t)(tile_id * a.split_k) * cols) * GM_BM;
            for (int c = 0; c < a.bn; ++c) {
              const int m = m0 + c;
              if (m >= a.M) break;
              float g = 0.f, u = 0.f;
              for (int s2 = 0; s2 < a.split_k; ++s2) {
                const float* p = wt + ((size_t)s2 * cols) * GM_BM;
                g += __ldcg(p + (size_t)c * GM_BM + etid);
                if (a.dual) u += __ldcg(p + (size_t)(a.bn + c) * GM_BM + etid);
              }
              if (n_ok) {
                const float sc = (a.scale_m ? a.scale_m[m] : 1.f);
                g *= sc * (a.scale_n ? a.scale_n[n] : 1.f);
                if (a.dual) u *= sc * (a.scale_n ? a.scale_n[a.N + n] : 1.f);
                float x = a.dual ? siluf_(g) * u : g;
                if (a.res) x += bf2f(a.res[(size_t)m * a.ldy + n]);
                if (a.out_f32) reinterpret_cast<float*>(a.Y)[(size_t)m * a.ldy + n] = x;
                else Yb[(size_t)m * a.ldy + n] = f2bf(x);
              }
            }
            if (etid == 0) a.counters[tile_id] = 0;       // self-cleaning for the next launch
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
      buf ^= 1;
    }
    if (!ok) { set_status(a.status, ST_MBAR_TIMEOUT); abort_s = 1; }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (abort_s && threadIdx.x == 0) {
    // give copies that were already issued a bounded time to land before the CTA (and its smem) goes away
    for (int i = 0; i < a.stages; ++i) {
      for (uint32_t p = 0; p < 2; ++p) (void)mbar_wait(&full_bar[i], p, 1u << 12);
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
  }
  if constexpr (COMM == 1 || COMM == 2) {
    // the last CTA to finish advances the call counter (and clears the arrival counts for the next call)
    if (threadIdx.x == 0) {
      __threadfence();
      const uint32_t done = atomicAdd(&a.cm.ctr[1], 1u);
      if (done == gridDim.x - 1) {
        if (COMM == 2)
          for (int i = 0; i < a.tiles_a; ++i) a.cm.ctr[2 + i] = 0;
        a.cm.ctr[1] = 0;
        __threadfence();
        a.cm.ctr[0] = epoch;
      }
    }
  }
}

// ---- host side -------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
  if (qres != cudaDriverEntryPointSuccess) return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows][cols] matrix with row stride ld (elements): box = {64, box_rows},
// 128-byte swizzle, zero fill outside the tensor.
static int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -10;
  if (((uintptr_t)base & 15) || ((ld * 2) & 15)) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)GM_BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

// 2-D byte tensor map (FP8 operands): box = {128 bytes, box_rows}, 128-byte swizzle
static int make_tmap_u8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -10;
  if ((uintptr_t)base % 16 || ld % 16) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

static int round_up_pow2(int v) { int p = 32; while (p < v) p <<= 1; return p; }

struct GemmPlan { GemmArgs a; int grid; size_t smem; };

static int plan_gemm(GemmPlan& p, int M, int N, int K, int mode, int split_k, int sm_count, int fp8 = 0) {
  GemmArgs& a = p.a;
  a.fp8 = fp8; a.scale_m = nullptr; a.scale_n = nullptr; a.out_f32 = 0;
  a.M = M; a.N = N; a.K = K;
  a.dual = mode == 1;
  a.swap = M <= 64;
  if (a.swap) {
    a.bn = ((M + 15) / 16) * 16;
    a.n_a = a.dual ? 2 : 1;
    a.n_b = 1;
    a.b_box_rows = a.bn;
    a.tiles_a = (N + GM_BM - 1) / GM_BM;
    a.tiles_b = 1;
    a.split_k = split_k < 1 ? 1 : split_k;
  } else {
    a.bn = (a.dual || N > 128) ? 256 : 128;
    a.n_a = 1;
    a.n_b = a.dual ? 2 : 1;
    a.b_box_rows = a.dual ? 128 : a.bn;
    a.tiles_a = (M + GM_BM - 1) / GM_BM;
    int ncols_out = a.dual ? 128 : a.bn;
    a.tiles_b = (N + ncols_out - 1) / ncols_out;
    a.split_k = 1;
  }
  const int bk_elems = fp8 ? 2 * GM_BK : GM_BK;
  int kblocks = (K + bk_elems - 1) / bk_elems;
  if (a.split_k > kblocks) a.split_k = kblocks;
  {
    // every split must own at least one k block (an empty split would publish an unwritten accumulator)
    int per = (kblocks + a.split_k - 1) / a.split_k;
    a.split_k = (kblocks + per - 1) / per;
  }
  a.acc_cols = a.n_a * a.bn;
  a.tmem_cols = round_up_pow2(2 * a.acc_cols);
  if (a.tmem_cols > 512) return -4;
  int b_bytes = a.n_b * a.b_box_rows * GM_BK * 2;
  int stage_bytes = a.n_a * GM_A_BYTES + ((b_bytes + 1023) & ~1023);
  int budget = 200 * 1024;
  a.stages = budget / stage_bytes;
  if (a.stages > GM_MAX_STAGES) a.stages = GM_MAX_STAGES;
  if (a.stages < 2) return -5;
  // more than half the shared memory of an SM, so one CTA (and one TMEM allocation) per SM
  p.smem = (size_t)a.stages * stage_bytes + 1024;
  if (p.smem < 120 * 1024) p.smem = 120 * 1024;
  int total = a.tiles_a * a.tiles_b * a.split_k;
  p.grid = total < sm_count ? total : sm_count;
  return 0;
}

}  // namespace fb

