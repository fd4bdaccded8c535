// Tensor-parallel GEMMs with the collective inside the kernel (kernel body: gemm_core.cuh, COMM = 1 and 2).
//
//   fb_gemm_rs   row-parallel projection -> reduce-scatter over rows (+ residual): every rank multiplies its K slice,
//                the epilogue stores bf16 partial tiles straight into the row owner's staging slot over NVLink and
//                releases a per-tile flag; owners sum the W partials in rank order. Replaces the reference's
//                prompt-sized `fe_gemm_*` + NCCL all-reduce (`crates/fe-model/src/model.rs:1761-1797`,
//                `crates/fe-fabric/src/lib.rs:161`).
//   fb_ag_gemm   all-gather -> column-parallel projection (+ SwiGLU): X lives row-sharded in a symmetric buffer; two
//                warps per CTA pull the peers' shards with plain 16-byte peer loads into this GPU's copy (every remote
//                byte crosses NVLink once) while the tensor cores start on the rows already present.
//
// Protocol rules shared by both (the callers in parallel/tp.py keep them):
//   * every rank makes the same sequence of calls with the same shapes; a device-side call counter is the epoch of
//     the flags, so CUDA-graph replays work;
//   * the grid is at most one CTA per SM, so all CTAs of a launch are resident (the gather warps and the tile
//     consumers of one GPU wait on each other);
//   * no wait is unbounded: on expiry a kernel records ST_PEER_TIMEOUT in the status word, stops issuing work,
//     drains its copies, frees its TMEM and returns;
//   * between two fb_ag_gemm calls that reuse the X buffer there must be a collective every rank only enters after
//     finishing the first (in the layer that is the fb_gemm_rs of the same block), because peers read the shard in place.
//   * no TMA or bulk load reads peer memory and nothing here uses cluster multicast.
#include "api_ext.h"
#include "gemm_core.cuh"

using namespace fb;

namespace {

struct BigLayout {
  long flags_off, ready_off, stage_off, slot_elems, xfull_off, total;
  int max_tiles;
};

BigLayout big_layout(int world, long max_rows, long max_cols) {
  BigLayout l;
  const long tiles_a = (max_rows + GM_BM - 1) / GM_BM, tiles_b = (max_cols + 127) / 128;
  l.max_tiles = (int)(tiles_a * tiles_b);
  l.flags_off = 0;
  l.ready_off = ((long)2 * 8 * l.max_tiles * 4 + 255) & ~255l;
  l.stage_off = l.ready_off + 256;
  const long rows_per = (max_rows + world - 1) / world + 1;
  l.slot_elems = (rows_per * max_cols + 127) & ~127l;
  l.xfull_off = l.stage_off + 2l * world * l.slot_elems * 2;
  l.total = l.xfull_off + ((max_rows * max_cols * 2 + 255) & ~255l);
  return l;
}

int fill(GemmComm& cm, const void* const* peers, int rank, int world, int M, long max_rows, long max_cols,
         uint32_t* ctr, unsigned spin_limit) {
  if (world < 2 || world > 8) return -20;
  BigLayout l = big_layout(world, max_rows, max_cols);
  for (int i = 0; i < 8; ++i) cm.peer[i] = i < world ? const_cast<void*>(peers[i]) : nullptr;
  cm.rank = rank; cm.world = world;
  cm.rows_per_rank = (M + world - 1) / world;
  cm.ctr = ctr;
  cm.spin_limit = spin_limit ? spin_limit : (1u << 24);
  cm.flags_off = l.flags_off; cm.ready_off = l.ready_off; cm.stage_off = l.stage_off; cm.slot_elems = l.slot_elems;
  cm.xfull_off = l.xfull_off; cm.max_tiles = l.max_tiles;
  cm.y_shard = nullptr; cm.res_shard = nullptr;
  return 0;
}

constexpr size_t RS_STAGING = 4 * 32 * GM_RS_COLS * 2;      // transpose buffers of the four epilogue warps

template <int COMM>
int launch(const GemmPlan& p, const CUtensorMap& tmA, const CUtensorMap& tmB, cudaStream_t s) {
  const size_t smem = p.smem + (COMM == 1 ? RS_STAGING : 0);
  constexpr size_t limit = 226 * 1024;                     // 227 KB per CTA minus the kernel's static shared memory
  if (smem > limit) return -23;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tc_kernel<COMM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  const int threads = COMM == 2 ? GM_THREADS + 32 * GM_COPY_WARPS : GM_THREADS;
  gemm_bf16_tc_kernel<COMM><<<p.grid, threads, smem, s>>>(tmA, tmB, p.a);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" long fb_big_workspace_bytes(int world, long max_rows, long max_cols) {
  return big_layout(world, max_rows, max_cols).total;
}

extern "C" long fb_big_xfull_offset(int world, long max_rows, long max_cols) {
  return big_layout(world, max_rows, max_cols).xfull_off;
}

// Y_shard[Ms][N] = (sum over ranks of X_r[M][K_r] W_r[N][K_r]^T)[rows of this rank] + res_shard.  M > 64.
extern "C" int fb_gemm_rs(void* y_shard, const void* X, const void* W, const void* res_shard, int M, int N, int K,
                          long ldx, const void* const* peers, int rank, int world, long max_rows, long max_cols,
                          uint32_t* ctr, int* status, unsigned spin_limit, int sm_count, cudaStream_t s) {
  if (M <= 64 || K % 8 || ldx % 8 || N % 8) return -1;
  if (M > max_rows || N > max_cols) return -21;
  if (sm_count <= 0) sm_count = 148;
  GemmPlan p{};
  int rc = plan_gemm(p, M, N, K, 0, 1, sm_count);
  if (rc) return rc;
  GemmArgs& a = p.a;
  if (a.tiles_a * a.tiles_b > big_layout(world, max_rows, max_cols).max_tiles) return -22;
  rc = fill(a.cm, peers, rank, world, M, max_rows, max_cols, ctr, spin_limit);
  if (rc) return rc;
  a.cm.y_shard = (__nv_bfloat16*)y_shard;
  a.cm.res_shard = (const __nv_bfloat16*)res_shard;
  a.Y = nullptr; a.res = nullptr; a.workspace = nullptr; a.counters = nullptr; a.status = status; a.ldy = N;
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, X, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, GM_BM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)a.b_box_rows);
  if (rc) return rc;
  return launch<1>(p, tmA, tmB, s);
}

// Y[M][N] = Xfull[M][K] W[N or 2N][K]^T (mode 1: SwiGLU over gate|up rows), where Xfull is the all-gather of the
// ranks' row shards; this rank's rows must already be in its full-X buffer (offset fb_big_xfull_offset).  M > 64.
extern "C" int fb_ag_gemm(void* Y, const void* W, const void* res, int M, int N, int K, long ldy, int mode,
                          const void* const* peers, int rank, int world, long max_rows, long max_cols, uint32_t* ctr,
                          int* status, unsigned spin_limit, int sm_count, cudaStream_t s) {
  if (M <= 64 || K % 8 || ldy % 8) return -1;
  if (M > max_rows || K > max_cols) return -21;
  if (sm_count <= 0) sm_count = 148;
  GemmPlan p{};
  int rc = plan_gemm(p, M, N, K, mode, 1, sm_count);
  if (rc) return rc;
  GemmArgs& a = p.a;
  rc = fill(a.cm, peers, rank, world, M, max_rows, max_cols, ctr, spin_limit);
  if (rc) return rc;
  a.Y = Y; a.res = (const __nv_bfloat16*)res; a.workspace = nullptr; a.counters = nullptr; a.status = status; a.ldy = ldy;
  const void* xfull = reinterpret_cast<const char*>(peers[rank]) + a.cm.xfull_off;
  const int w_rows = a.dual ? 2 * N : N;
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, xfull, (uint64_t)M, (uint64_t)K, (uint64_t)K, GM_BM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, (uint32_t)a.b_box_rows);
  if (rc) return rc;
  return launch<2>(p, tmA, tmB, s);
}

// ---- grouped GEMM over expert-sorted rows (mixture of experts, prompt-sized) ------------------------------------
// Y[r][N] = X[r][K] W[e(r)][N or 2N][K]^T (+ SwiGLU) for the rows r of every expert e: rows are contiguous per
// expert, `row_base` / `tile_start` are device-side prefix sums (experts + 1 entries) so the call needs no host
// synchronisation. `max_rows` bounds the rows (the tensor map's extent). Counterpart of the reference's segmented
// prompt GEMM over sorted (token, expert) pairs (`ggq_mmq_moe*`, `kernels/k-gguf/src/mmq.rs:522`).
extern "C" int fb_gemm_grouped(void* Y, const void* X, const void* W, const int* tile_start, const int* row_base,
                               int experts, int max_rows, int N, int K, long ldx, long ldy, int mode, int* status,
                               int sm_count, cudaStream_t s) {
  if (experts <= 0 || max_rows <= 0) return 0;
  if (K % 8 || ldx % 8 || ldy % 8) return -1;
  if (sm_count <= 0) sm_count = 148;
  GemmPlan p{};
  int rc = plan_gemm(p, max_rows > 64 ? max_rows : 65, N, K, mode, 1, sm_count);     // normal orientation
  if (rc) return rc;
  GemmArgs& a = p.a;
  const int w_rows = a.dual ? 2 * N : N;
  a.gr.tile_start = tile_start; a.gr.row_base = row_base; a.gr.experts = experts; a.gr.w_rows = w_rows;
  a.gr.uniform_rows = 0;
  a.Y = Y; a.res = nullptr; a.workspace = nullptr; a.counters = nullptr; a.status = status; a.ldy = ldy;
  a.M = max_rows;
  p.grid = sm_count;                               // the real tile count is only known on the device
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, X, (uint64_t)max_rows, (uint64_t)K, (uint64_t)ldx, GM_BM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, (uint64_t)experts * w_rows, (uint64_t)K, (uint64_t)K, (uint32_t)a.b_box_rows);
  if (rc) return rc;
  return launch<3>(p, tmA, tmB, s);
}

// ---- batched GEMM: Y[g] = X[g] W[g]^T for `groups` problems of the same shape ---------------------------------------
// X is [groups * rows][K] (group-major), W [groups][N][K], Y [groups * rows][N]: the grouped kernel with every group
// `rows` long, so no prefix arrays and nothing computed on the device beforehand. Used for the per-head projections of
// multi-head latent attention on prompt-sized steps (reference: one `mma` launch per head group,
// `kernels/k-ds/src/attn.rs:151-548`).
extern "C" int fb_gemm_batched(void* Y, const void* X, const void* W, int groups, int rows, int N, int K, int* status,
                               int sm_count, cudaStream_t s) {
  if (groups <= 0 || rows <= 0) return 0;
  if (K % 8 || N % 8) return -1;
  if (sm_count <= 0) sm_count = 148;
  const long total = (long)groups * rows;
  if (total > 0x7fffffffL) return -1;
  GemmPlan p{};
  int rc = plan_gemm(p, total > 64 ? (int)total : 65, N, K, 0, 1, sm_count);
  if (rc) return rc;
  GemmArgs& a = p.a;
  a.gr.tile_start = nullptr; a.gr.row_base = nullptr; a.gr.experts = groups; a.gr.w_rows = N; a.gr.uniform_rows = rows;
  a.Y = Y; a.res = nullptr; a.workspace = nullptr; a.counters = nullptr; a.status = status; a.ldy = N;
  a.M = (int)total;
  p.grid = sm_count;
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, X, (uint64_t)total, (uint64_t)K, (uint64_t)K, GM_BM);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, (uint64_t)groups * N, (uint64_t)K, (uint64_t)K, (uint32_t)a.b_box_rows);
  if (rc) return rc;
  return launch<3>(p, tmA, tmB, s);
}
