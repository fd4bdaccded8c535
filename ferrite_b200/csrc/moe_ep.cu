// Expert parallelism for prompt-sized batches: router output -> all-to-all dispatch -> grouped expert GEMMs ->
// all-to-all combine, with both all-to-alls done by these kernels over NVLink peer memory (no NCCL on the path).
//
// Tokens are sharded by rows over the ranks (the sequence-parallel layout of the prompt path); experts are owned by
// ranks in contiguous blocks. One call runs, on every rank, in stream order:
//   1. ep_plan      one CTA: histogram of the local (token, pick) pairs per expert and each pair's position inside
//                   its (source, expert) bucket; the per-expert counts are exchanged with every rank as
//                   (value, epoch) pairs; from the full count matrix every rank derives, without further talk, where
//                   its buckets start inside each owner's receive buffer (experts ascending, sources ascending
//                   inside an expert) and, for the experts it owns, the row / tile prefix sums of the grouped GEMM.
//   2. ep_dispatch  one warp per pair: the token's hidden row is stored into the owner's receive buffer (16-byte peer
//                   stores); the last CTA to finish releases one "rows are in" flag per owner.
//   3. ep_wait      one CTA: bounded wait for the W dispatch flags.
//   4. two grouped tcgen05 GEMMs (gate|up + SwiGLU, down) over the expert-sorted rows (gemm_comm.cu), the second
//      writing into the symmetric result buffer; 5. ep_signal: "results are ready" flag to every rank.
//   6. ep_combine   one CTA per local token: bounded wait for the owners' flags, then the K result rows are PULLED from
//                   the owners (16-byte peer loads) and summed in pick order with the routing weights, the shared
//                   expert and the residual. The last CTA advances the call counter (the epoch of every flag), so the
//                   sequence replays inside CUDA graphs.
// Buffer reuse is safe by data flow: a rank dispatches call n+1 only after its combine n saw every owner's
// "results ready" (so every owner is done reading its receive buffer), and an owner overwrites its result buffer
// only after every source dispatched call n+1, i.e. after that source's combine n pulled its rows.
//
// Replaces the reference's expert dispatch by peer copies (`layer_zc`, `crates/fe-dsc/src/engine.rs:2409-2496`), its
// pair sort (`ggq_moe_sort_*`, `kernels/k-gguf/src/sort.rs`) and ownership masks (`fx_mask_own`,
// `kernels/k-fnext/src/fast.rs:1718`). No TMA or bulk copy touches peer memory; every wait is bounded.
#include "api_ext.h"
#include "common.cuh"

namespace fb {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_MAX_EXPERTS = 1024;

struct EpComm {
  void* peer[EP_MAX_RANKS];    // base of the symmetric EP workspace on each rank
  int rank, world;
  int n_experts, per_rank;     // experts are owned in blocks of per_rank
  int hidden, cap_rows;        // receive / result buffers hold cap_rows rows of `hidden` bf16
  uint32_t* ctr;               // local: [0] call counter, [1] dispatch CTAs done, [2] combine CTAs done
  int* status;
  unsigned spin_limit;
  long cnt_off;                // u32 pairs [2 parity][W src][E] (value, epoch)
  long flag_off;               // u32 [2 kinds][W]: kind 0 "rows are in" (written by sources), kind 1 "results ready"
  long recv_off;               // bf16 [cap_rows][hidden]
  long out_off;                // bf16 [cap_rows][hidden]
};

__device__ __forceinline__ uint2* ep_cnt(void* base, const EpComm& c, int parity, int src) {
  return reinterpret_cast<uint2*>(reinterpret_cast<char*>(base) + c.cnt_off) + ((size_t)parity * EP_MAX_RANKS + src) * c.n_experts;
}
__device__ __forceinline__ uint32_t* ep_flag(void* base, const EpComm& c, int kind, int src) {
  return reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(base) + c.flag_off) + kind * EP_MAX_RANKS + src;
}
__device__ __forceinline__ __nv_bfloat16* ep_recv(void* base, const EpComm& c) {
  return reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(base) + c.recv_off);
}
__device__ __forceinline__ __nv_bfloat16* ep_out(void* base, const EpComm& c) {
  return reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(base) + c.out_off);
}

// ---- 1. plan ---------------------------------------------------------------------------------------------------
// pos[pair]: position of the pair inside its (this rank, expert) bucket; send_off[e]: first row of this rank's
// bucket for expert e inside the owner's buffers; row_base / tile_start: prefix sums over the experts this rank owns.
__global__ void __launch_bounds__(1024) ep_plan_kernel(EpComm c, const int* __restrict__ ids, int n_pairs,
                                                       int* __restrict__ pos, int* __restrict__ send_off,
                                                       int* __restrict__ row_base, int* __restrict__ tile_start) {
  __shared__ int hist[EP_MAX_EXPERTS];
  __shared__ int rows_e[EP_MAX_EXPERTS];
  __shared__ int before_me[EP_MAX_EXPERTS];
  const int E = c.n_experts, tid = threadIdx.x;
  const uint32_t epoch = c.ctr[0] + 1;
  const int parity = epoch & 1;
  for (int e = tid; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int p = tid; p < n_pairs; p += blockDim.x) pos[p] = atomicAdd(&hist[ids[p]], 1);
  __syncthreads();
  for (int r = 0; r < c.world; ++r) {
    if (r == c.rank) continue;
    uint2* dst = ep_cnt(c.peer[r], c, parity, c.rank);
    for (int e = tid; e < E; e += blockDim.x) st_relaxed_sys_v2(dst + e, (uint32_t)hist[e], epoch);
  }
  bool fail = false;
  for (int e = tid; e < E; e += blockDim.x) {
    int total = 0, before = 0;
    for (int r = 0; r < c.world; ++r) {
      int v;
      if (r == c.rank) {
        v = hist[e];
      } else {
        const uint2* src = ep_cnt(c.peer[c.rank], c, parity, r) + e;
        uint2 w = ld_relaxed_sys_v2(src);
        for (uint32_t spin = 0; w.y != epoch && spin < c.spin_limit; ++spin) w = ld_relaxed_sys_v2(src);
        if (w.y != epoch) fail = true;
        v = (int)w.x;
      }
      if (r < c.rank) before += v;
      total += v;
    }
    rows_e[e] = total;
    before_me[e] = before;
  }
  if (fail) set_status(c.status, ST_PEER_TIMEOUT);
  __syncthreads();
  // prefix over the experts of each owner (per_rank <= 128 entries per owner: one thread per owner is plenty)
  if (tid < c.world) {
    int acc = 0, tiles = 0;
    const int e0 = tid * c.per_rank;
    for (int j = 0; j < c.per_rank; ++j) {
      const int e = e0 + j;
      send_off[e] = acc + before_me[e];
      if (tid == c.rank) { row_base[j] = acc; tile_start[j] = tiles; }
      acc += rows_e[e];
      tiles += (rows_e[e] + 127) / 128;
    }
    if (tid == c.rank) {
      row_base[c.per_rank] = acc;
      tile_start[c.per_rank] = tiles;
      if (acc > c.cap_rows) set_status(c.status, ST_CAPACITY);
    }
  }
}

// ---- 2. dispatch -----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpComm c, const __nv_bfloat16* __restrict__ x,
                                                          const int* __restrict__ ids, const int* __restrict__ pos,
                                                          const int* __restrict__ send_off, int n_pairs, int top_k) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * 8 + warp;
  if (pair < n_pairs) {
    const int e = ids[pair], o = e / c.per_rank;
    const int row = send_off[e] + pos[pair];
    if (row < c.cap_rows) {
      const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / top_k) * c.hidden);
      uint4* dst = reinterpret_cast<uint4*>(ep_recv(c.peer[o], c) + (size_t)row * c.hidden);
      for (int i = lane; i < c.hidden / 8; i += 32) dst[i] = src[i];
    }
  }
  // the last CTA to finish tells every owner that this rank's rows are in place
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = (atomicAdd(&c.ctr[1], 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (last) {
    const uint32_t epoch = c.ctr[0] + 1;
    __threadfence_system();
    if (threadIdx.x < c.world) st_release_sys(ep_flag(c.peer[threadIdx.x], c, 0, c.rank), epoch);
    if (threadIdx.x == 0) c.ctr[1] = 0;
  }
}

// ---- 3 / 5. flags ----------------------------------------------------------------------------------------------
__global__ void ep_wait_kernel(EpComm c) {
  if (threadIdx.x < c.world) {
    const uint32_t epoch = c.ctr[0] + 1;
    if (!wait_flag_ge(ep_flag(c.peer[c.rank], c, 0, threadIdx.x), epoch, c.spin_limit)) set_status(c.status, ST_PEER_TIMEOUT);
  }
}

__global__ void ep_signal_kernel(EpComm c) {
  if (threadIdx.x < c.world) {
    const uint32_t epoch = c.ctr[0] + 1;
    __threadfence_system();
    st_release_sys(ep_flag(c.peer[threadIdx.x], c, 1, c.rank), epoch);
  }
}

// ---- 6. combine ------------------------------------------------------------------------------------------------
// grid = local tokens; out[t] = res[t] + shared[t] * sigmoid(gate[t]) + sum_k wts[t][k] * result_row(t, k), pick order
__global__ void __launch_bounds__(256) ep_combine_kernel(EpComm c, __nv_bfloat16* __restrict__ out,
                                                         const int* __restrict__ ids, const float* __restrict__ wts,
                                                         const int* __restrict__ pos, const int* __restrict__ send_off,
                                                         const __nv_bfloat16* __restrict__ shared,
                                                         const float* __restrict__ shared_gate,
                                                         const __nv_bfloat16* __restrict__ res, int rows, int top_k) {
  __shared__ int fail_s;
  const int t = blockIdx.x;
  const uint32_t epoch = c.ctr[0] + 1;
  if (threadIdx.x == 0) fail_s = 0;
  __syncthreads();
  if (threadIdx.x < c.world)
    if (!wait_flag_ge(ep_flag(c.peer[c.rank], c, 1, threadIdx.x), epoch, c.spin_limit)) { fail_s = 1; set_status(c.status, ST_PEER_TIMEOUT); }
  __syncthreads();
  const int H = c.hidden;
  if (!fail_s && t < rows) {
    const float g = shared ? (shared_gate ? sigmoidf_(shared_gate[t]) : 1.f) : 0.f;
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < top_k; ++k) {
        const int pair = t * top_k + k;
        const int e = ids[pair], o = e / c.per_rank;
        const int row = send_off[e] + pos[pair];
        if (row >= c.cap_rows) continue;
        const float w = wts[pair];
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(ep_out(c.peer[o], c) + (size_t)row * H) + i);
        const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[2 * j] = fmaf(w, bf_lo(u[j]), acc[2 * j]); acc[2 * j + 1] = fmaf(w, bf_hi(u[j]), acc[2 * j + 1]); }
      }
      if (shared) {
        const uint4 raw = reinterpret_cast<const uint4*>(shared + (size_t)t * H)[i];
        const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[2 * j] = fmaf(g, bf_lo(u[j]), acc[2 * j]); acc[2 * j + 1] = fmaf(g, bf_hi(u[j]), acc[2 * j + 1]); }
      }
      if (res) {
        const uint4 raw = reinterpret_cast<const uint4*>(res + (size_t)t * H)[i];
        const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[2 * j] += bf_lo(u[j]); acc[2 * j + 1] += bf_hi(u[j]); }
      }
      reinterpret_cast<uint4*>(out + (size_t)t * H)[i] =
          make_uint4(pack_bf2(acc[0], acc[1]), pack_bf2(acc[2], acc[3]), pack_bf2(acc[4], acc[5]), pack_bf2(acc[6], acc[7]));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&c.ctr[2], 1u) == gridDim.x - 1) {      // last CTA: the call is over on this rank
      c.ctr[2] = 0;
      __threadfence();
      c.ctr[0] = epoch;
    }
  }
}

struct EpLayout { long cnt_off, flag_off, recv_off, out_off, total; };

static EpLayout ep_layout(int n_experts, int hidden, long cap_rows) {
  EpLayout l;
  l.cnt_off = 0;
  l.flag_off = ((long)2 * EP_MAX_RANKS * n_experts * 8 + 255) & ~255l;
  l.recv_off = l.flag_off + 256;
  const long buf = (cap_rows * hidden * 2 + 255) & ~255l;
  l.out_off = l.recv_off + buf;
  l.total = l.out_off + buf;
  return l;
}

}  // namespace fb

using namespace fb;

extern "C" long fb_ep_workspace_bytes(int n_experts, int hidden, long cap_rows) {
  return ep_layout(n_experts, hidden, cap_rows).total;
}
extern "C" long fb_ep_recv_offset(int n_experts, int hidden, long cap_rows) { return ep_layout(n_experts, hidden, cap_rows).recv_off; }
extern "C" long fb_ep_out_offset(int n_experts, int hidden, long cap_rows) { return ep_layout(n_experts, hidden, cap_rows).out_off; }

// One expert-parallel MoE block over this rank's `rows` tokens. `act` is scratch [cap_rows][inter] bf16; `plan` is int
// scratch of rows * top_k + 3 * n_experts + 8 entries. w_gu / w_down hold only the experts this rank owns.
extern "C" int fb_ep_moe(void* out, const void* x, const int* ids, const float* wts, const void* w_gu, const void* w_down,
                         const void* shared, const float* shared_gate, const void* res, void* act, int* plan, int rows,
                         int top_k, int n_experts, int hidden, int inter, long cap_rows, const void* const* peers, int rank,
                         int world, uint32_t* ctr, int* status, unsigned spin_limit, int sm_count, cudaStream_t s) {
  if (world < 1 || world > EP_MAX_RANKS || n_experts > EP_MAX_EXPERTS || n_experts % world || hidden % 8 || inter % 8)
    return -1;
  EpLayout l = ep_layout(n_experts, hidden, cap_rows);
  EpComm c;
  for (int i = 0; i < EP_MAX_RANKS; ++i) c.peer[i] = i < world ? const_cast<void*>(peers[i]) : nullptr;
  c.rank = rank; c.world = world; c.n_experts = n_experts; c.per_rank = n_experts / world; c.hidden = hidden;
  c.cap_rows = (int)cap_rows; c.ctr = ctr; c.status = status; c.spin_limit = spin_limit ? spin_limit : (1u << 23);
  c.cnt_off = l.cnt_off; c.flag_off = l.flag_off; c.recv_off = l.recv_off; c.out_off = l.out_off;
  const int n_pairs = rows * top_k;
  int* pos = plan;
  int* send_off = pos + n_pairs;
  int* row_base = send_off + n_experts;
  int* tile_start = row_base + c.per_rank + 1;
  ep_plan_kernel<<<1, 1024, 0, s>>>(c, ids, n_pairs, pos, send_off, row_base, tile_start);
  const int dgrid = n_pairs > 0 ? (n_pairs + 7) / 8 : 1;
  ep_dispatch_kernel<<<dgrid, 256, 0, s>>>(c, (const __nv_bfloat16*)x, ids, pos, send_off, n_pairs, top_k);
  ep_wait_kernel<<<1, 32, 0, s>>>(c);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const char* local = reinterpret_cast<const char*>(peers[rank]);
  int rc = fb_gemm_grouped(act, local + l.recv_off, w_gu, tile_start, row_base, c.per_rank, (int)cap_rows, inter, hidden,
                           hidden, inter, 1, status, sm_count, s);
  if (rc) return rc;
  rc = fb_gemm_grouped(const_cast<char*>(local) + l.out_off, act, w_down, tile_start, row_base, c.per_rank, (int)cap_rows,
                       hidden, inter, inter, hidden, 0, status, sm_count, s);
  if (rc) return rc;
  ep_signal_kernel<<<1, 32, 0, s>>>(c);
  ep_combine_kernel<<<rows > 0 ? rows : 1, 256, 0, s>>>(c, (__nv_bfloat16*)out, ids, wts, pos, send_off,
                                                        (const __nv_bfloat16*)shared, shared_gate,
                                                        (const __nv_bfloat16*)res, rows, top_k);
  return (int)cudaGetLastError();
}
