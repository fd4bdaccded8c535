// Fused compute + collective kernels over NVLink peer memory (one process per GPU, symmetric buffers mapped
// on every rank). No NCCL call and no TMA load touches peer memory here: peers are reached with plain
// st/ld (system scope) through the peer-pointer table.
//
//  * fb_gemv_allreduce   row-parallel GEMV (o_proj / out_proj / down_proj, <= 8 rows) whose epilogue is a
//                        one-shot all-reduce: every CTA pushes its fp32 partial tile to all ranks, releases a
//                        flag per (rank, CTA), waits (bounded) for the same tile from every rank, sums in RANK
//                        ORDER, adds the residual and rounds to bf16. All ranks therefore hold identical bits.
//  * fb_allreduce_oneshot the same exchange for a partial that another kernel produced (tcgen05 GEMM for 9..64
//                        verify rows), bf16 or fp32 partials.
//  * fb_argmax_gather    vocab-parallel head: per-row (max, index) of the local logits shard pushed to all ranks
//                        and merged in rank order, so only 8 bytes per row cross NVLink instead of the logits.
//
// The reference does this job with a NIC: `fab_gather_sum_bf16[in]` stages the partial, rings a doorbell, a CPU
// proxy thread posts an RDMA write, and the kernel spins on the peer's sequence flag, giving up after a poll
// limit and setting a poison word (`kernels/k-fabric/src/lib.rs:82-135`, `crates/fe-fabric/src/roce.rs:375-455`,
// call site `crates/fe-model/src/model.rs:1761-1797`). Here the wait is bounded the same way and reports
// ST_PEER_TIMEOUT through the status word; epochs live in device memory so the kernels replay inside CUDA graphs.
#include "api_ext.h"
#include "comm_core.cuh"
#include "gemv_core.cuh"

namespace fb {

// ---- K1: GEMV + one-shot all-reduce + residual ------------------------------------------------------------
template <int M, int R>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_allreduce_kernel(GemvArgs a, CommBuf cb) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float* tile = reinterpret_cast<float*>(smem_raw + (size_t)M * a.kc * sizeof(__nv_bfloat16));  // [M][rows_per_cta]
  __shared__ float rscale[M];
  __shared__ float scratch[32];
  __shared__ unsigned long long stamps[6];
  const bool traced = cb.trace != nullptr && blockIdx.x == 0;
  const int row0 = blockIdx.x * a.rows_per_cta;
  const int row_end = min(a.N, row0 + a.rows_per_cta);
  const int nrows = row_end - row0;
  for (int i = threadIdx.x; i < M * a.rows_per_cta; i += blockDim.x) tile[i] = 0.f;
  __syncthreads();
  const int rpc = a.rows_per_cta;
  gemv_main<M, R, false>(a, xs, rscale, scratch, [&](float (&acc)[R][M], int n) {
    if ((threadIdx.x & 31) != 0) return;
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (n + r < row_end)
#pragma unroll
        for (int m = 0; m < M; ++m) tile[m * rpc + (n + r - row0)] = acc[r][m];
  }, traced ? &stamps[0] : nullptr);
  __syncthreads();
  // slot layout: CTA-major, so a CTA's tile is one contiguous run of M * rows_per_cta floats
  const uint32_t epoch = comm_epoch_begin(cb);
  cta_exchange_sum(cb, tile, M * a.rows_per_cta, (long)blockIdx.x * M * a.rows_per_cta, epoch, traced ? stamps : nullptr);
  __syncthreads();
  for (int i = threadIdx.x; i < a.M * nrows; i += blockDim.x) {
    int m = i / nrows, j = i % nrows;
    float v = tile[m * a.rows_per_cta + j];
    size_t o = (size_t)m * a.ldy + row0 + j;
    if (a.res) v += bf2f(a.res[o]);
    reinterpret_cast<__nv_bfloat16*>(a.Y)[o] = f2bf(v);
  }
  if (traced) comm_trace_flush(cb, stamps, epoch);
  comm_epoch_end(cb, epoch);
}

// ---- standalone one-shot all-reduce of [rows][n] partials ---------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(__nv_bfloat16* __restrict__ y, const T* __restrict__ part,
                                                                const __nv_bfloat16* __restrict__ res, long count,
                                                                int per_cta, CommBuf cb) {
  extern __shared__ __align__(16) float tile_s[];
  const long i0 = (long)blockIdx.x * per_cta;
  const int cnt = (int)min((long)per_cta, count - i0);
  for (int i = threadIdx.x; i < per_cta; i += blockDim.x) {
    float v = 0.f;
    if (i < cnt) {
      if (sizeof(T) == 2) v = bf2f(reinterpret_cast<const __nv_bfloat16*>(part)[i0 + i]);
      else v = reinterpret_cast<const float*>(part)[i0 + i];
    }
    tile_s[i] = v;
  }
  const uint32_t epoch = comm_epoch_begin(cb);          // (its barrier also orders the tile fill above)
  cta_exchange_sum(cb, tile_s, cnt, i0, epoch);          // only the live values travel: nothing is written past `count`
  for (int i = threadIdx.x; i < cnt; i += blockDim.x) {  // same thread <-> index map as the exchange: no barrier needed
    float v = tile_s[i];
    if (res) v += bf2f(res[i0 + i]);
    y[i0 + i] = f2bf(v);
  }
  comm_epoch_end(cb, epoch);
}

// ---- K4: vocab-parallel argmax merged over ranks ------------------------------------------------------------
// grid = rows. Each CTA finds (max, lowest index) of its rank's logits shard, publishes it to every rank and
// merges the world's candidates: larger value wins, ties go to the lower global index.
__global__ void __launch_bounds__(1024) argmax_gather_kernel(int* __restrict__ ids, float* __restrict__ vals,
                                                             const float* __restrict__ logits, long stride,
                                                             int n_local, int vocab_offset, CommBuf cb) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cand[2];
  const int row = blockIdx.x;
  const float* lp = logits + (size_t)row * stride;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n_local; i += blockDim.x) {
    float v = lp[i];
    if (v > best) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { cand[0] = best; cand[1] = __int_as_float(bi == 0x7fffffff ? 0 : bi + vocab_offset); }
  }
  __syncthreads();
  // Each rank's candidate travels as one 16-byte store {value, epoch, index, epoch}: both halves carry the epoch,
  // so a reader that sees two matching epoch words has the whole candidate (8-byte halves are written atomically).
  // The candidates live in the top COMM_TOP_RESERVE words of the data slots, apart from the all-reduce pairs.
  __shared__ int s_fail;
  const int cta = blockIdx.x;
  if (threadIdx.x == 0) s_fail = 0;
  const uint32_t epoch = comm_epoch_begin(cb);
  const int parity = epoch & 1;
  const long top = cb.slot_floats - COMM_TOP_RESERVE + (long)cta * 4;
  __shared__ float rv[COMM_MAX_RANKS];
  __shared__ int ri[COMM_MAX_RANKS];
  if (threadIdx.x < cb.world) {
    const int r = threadIdx.x;
    if (r != cb.rank) {
      st_relaxed_sys_v4(comm_data(cb.peer[r], cb, parity, cb.rank) + top,
                        make_uint4(__float_as_uint(cand[0]), epoch, __float_as_uint(cand[1]), epoch));
      const float* src = comm_data(cb.peer[cb.rank], cb, parity, r) + top;
      uint4 v = ld_relaxed_sys_v4(src);
      for (uint32_t spin = 0; (v.y != epoch || v.w != epoch) && spin < cb.spin_limit; ++spin) v = ld_relaxed_sys_v4(src);
      if (v.y != epoch || v.w != epoch) { s_fail = 1; set_status(cb.status, ST_PEER_TIMEOUT); }
      rv[r] = __uint_as_float(v.x);
      ri[r] = (int)v.z;
    } else {
      rv[r] = cand[0];
      ri[r] = __float_as_int(cand[1]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bv = -INFINITY;
    int bidx = 0;
    if (!s_fail) {
      for (int r = 0; r < cb.world; ++r)
        if (rv[r] > bv || (rv[r] == bv && ri[r] < bidx)) { bv = rv[r]; bidx = ri[r]; }
    }
    ids[row] = bidx;
    if (vals) vals[row] = bv;
  }
  comm_epoch_end(cb, epoch);
}

// Start-up self-test of every ordered pair of GPUs: this rank stores a pattern that names (source, destination, word)
// into its own lane of every peer's workspace with the same plain peer stores the fused kernels use. The host then
// compares what arrived with what each source must have written (`parallel/selftest.py`).
__global__ void p2p_pattern_kernel(CommBuf cb, long word_off, int n_words, uint32_t seed) {
  for (int p = 0; p < cb.world; ++p) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(comm_data(cb.peer[p], cb, 0, cb.rank)) + word_off;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += gridDim.x * blockDim.x) {
      uint32_t v = seed ^ ((uint32_t)cb.rank * 0x9E3779B1u) ^ ((uint32_t)p * 0x85EBCA77u) ^ ((uint32_t)i * 0xC2B2AE3Du);
      v ^= v >> 15; v *= 0x2C1B3C6Du; v ^= v >> 12;
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst + i), "r"(v) : "memory");
    }
  }
}

// A wait that is made to run out on purpose by a flag nobody sets: exercises the timeout path on one GPU
// without faulting anything. Returns through the status word.
__global__ void comm_wait_probe_kernel(const uint32_t* flag, uint32_t want, unsigned limit, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (!wait_flag_eq(flag, want, limit)) set_status(status, ST_PEER_TIMEOUT);
  }
}

template <int M>
static int launch_gemv_ar(GemvArgs a, CommBuf cb, int max_resident, cudaStream_t s) {
  constexpr int R = 2;
  a.kc = gemv_chunk_len(M, a.K);
  const int group = GEMV_WARPS * R;
  int nchunks = (a.K + a.kc - 1) / a.kc;
  int rpc;
  (void)nchunks;
  rpc = (a.N + max_resident - 1) / max_resident;
  rpc = (rpc + group - 1) / group * group;
  a.rows_per_cta = rpc;
  int grid = (a.N + rpc - 1) / rpc;
  // every CTA waits on its peers: all of them must be resident at once
  if (grid > max_resident || grid > cb.max_ctas) return -7;
  if ((long)grid * M * rpc * 2 > cb.slot_floats - COMM_TOP_RESERVE) return -8;
  size_t smem = (size_t)M * a.kc * sizeof(__nv_bfloat16) + (size_t)M * rpc * sizeof(float);
  auto kern = gemv_allreduce_kernel<M, R>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM_BYTES + 16 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GEMV_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, a, cb);
}

}  // namespace fb

using namespace fb;

// Profiling switches shared by every file that fills a CommBuf. The trace buffer must be set before a CUDA
// graph is captured (kernel arguments are baked into the graph).
static unsigned long long* g_comm_trace = nullptr;
static int g_comm_serial = -1;
extern "C" unsigned long long* fb_comm_trace_get() { return g_comm_trace; }
extern "C" void fb_comm_trace_set(unsigned long long* buf) { g_comm_trace = buf; }
extern "C" int fb_comm_serial_polls_get() {
  if (g_comm_serial < 0) { const char* e = getenv("FB_COMM_SERIAL_POLLS"); g_comm_serial = (e && e[0] == '1') ? 1 : 0; }
  return g_comm_serial;
}
extern "C" void fb_comm_serial_polls_set(int on) { g_comm_serial = on ? 1 : 0; }
extern "C" int fb_comm_trace_recs() { return COMM_TRACE_RECS; }
extern "C" int fb_comm_trace_words() { return COMM_TRACE_WORDS; }

extern "C" long fb_comm_workspace_bytes(int max_ctas, long slot_floats) {
  return (long)2 * COMM_MAX_RANKS * max_ctas * 4 + (long)2 * COMM_MAX_RANKS * slot_floats * 4;
}

extern "C" int fb_gemv_allreduce(void* Y, const void* X, const void* W, const void* res, int M, int N, int K, long ldx,
                                 long ldy, const void* const* peers, int rank, int world, int max_ctas,
                                 long slot_floats, uint32_t* epochs, int* status, unsigned spin_limit,
                                 int max_resident, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > COMM_MAX_ROWS || world > COMM_MAX_RANKS || (K % 8) || (ldx % 8)) return -1;
  GemvArgs a;
  a.X = (const __nv_bfloat16*)X; a.W = (const __nv_bfloat16*)W; a.norm_w = nullptr; a.res = (const __nv_bfloat16*)res;
  a.Y = Y; a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldy = ldy; a.eps = 0.f; a.centred = 0; a.out_f32 = 0;
  a.rows_per_cta = 0; a.kc = 0;
  CommBuf cb;
  fill_comm(cb, peers, rank, world, max_ctas, slot_floats, epochs, status, spin_limit);
  if (M == 1) return launch_gemv_ar<1>(a, cb, max_resident, s);
  if (M == 2) return launch_gemv_ar<2>(a, cb, max_resident, s);
  if (M <= 4) return launch_gemv_ar<4>(a, cb, max_resident, s);
  return launch_gemv_ar<8>(a, cb, max_resident, s);
}

extern "C" int fb_allreduce_oneshot(void* y, const void* part, const void* res, long count, int part_f32,
                                    const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                                    uint32_t* epochs, int* status, unsigned spin_limit, int max_resident,
                                    cudaStream_t s) {
  if (count <= 0) return 0;
  if (count * 2 > slot_floats - COMM_TOP_RESERVE) return -8;     // pairs stay below the argmax candidates
  CommBuf cb;
  fill_comm(cb, peers, rank, world, max_ctas, slot_floats, epochs, status, spin_limit);
  int grid = max_resident < max_ctas ? max_resident : max_ctas;
  int per = (int)((count + grid - 1) / grid);
  per = (per + 3) / 4 * 4;
  if (per < 256) per = 256;
  if (per > 8192) return -9;
  grid = (int)((count + per - 1) / per);
  size_t smem = (size_t)per * sizeof(float);
  if (part_f32) allreduce_oneshot_kernel<float><<<grid, 256, smem, s>>>((__nv_bfloat16*)y, (const float*)part, (const __nv_bfloat16*)res, count, per, cb);
  else allreduce_oneshot_kernel<__nv_bfloat16><<<grid, 256, smem, s>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)part, (const __nv_bfloat16*)res, count, per, cb);
  return (int)cudaGetLastError();
}

extern "C" int fb_argmax_gather(int* ids, float* vals, const float* logits, long stride, int rows, int n_local,
                                int vocab_offset, const void* const* peers, int rank, int world, int max_ctas,
                                long slot_floats, uint32_t* epochs, int* status, unsigned spin_limit, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (rows > max_ctas || (long)rows * 4 > COMM_TOP_RESERVE) return -8;
  CommBuf cb;
  fill_comm(cb, peers, rank, world, max_ctas, slot_floats, epochs, status, spin_limit);
  argmax_gather_kernel<<<rows, 1024, 0, s>>>(ids, vals, logits, stride, n_local, vocab_offset, cb);
  return (int)cudaGetLastError();
}

extern "C" int fb_p2p_pattern(const void* const* peers, int rank, int world, int max_ctas, long slot_floats, long word_off,
                              int n_words, uint32_t seed, cudaStream_t s) {
  if (n_words <= 0 || word_off < 0 || word_off + n_words > slot_floats - COMM_TOP_RESERVE) return -8;
  CommBuf cb;
  fill_comm(cb, peers, rank, world, max_ctas, slot_floats, nullptr, nullptr, 0);
  p2p_pattern_kernel<<<8, 256, 0, s>>>(cb, word_off, n_words, seed);
  return (int)cudaGetLastError();
}

extern "C" int fb_comm_wait_probe(const uint32_t* flag, uint32_t want, unsigned limit, int* status, cudaStream_t s) {
  comm_wait_probe_kernel<<<1, 32, 0, s>>>(flag, want, limit, status);
  return (int)cudaGetLastError();
}
