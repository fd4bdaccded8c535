// One decoder layer of a plain decode step (one row per sequence, a handful of sequences) as ONE persistent kernel.
//
// With the weights cut over several GPUs, or stored in 4 bits, a decode step no longer has enough bytes per kernel to
// hide a kernel boundary: at tensor-parallel 8 the 27B hybrid's five per-layer kernels each stream 1 - 3 MB (a
// microsecond of HBM time) and then pay the grid drain, the dependent launch and their own prologue, about 10 us each.
// Here the five phases of a layer
//     1  proj  = W_in  * rmsnorm(x)                      (Gated DeltaNet layers)
//     2  o     = conv + delta rule + gated norm of every local head
//     3  x_mid = x + sum over ranks (W_out * o)
//     4  act   = silu(W_gate * rmsnorm(x_mid)) * (W_up * rmsnorm(x_mid))
//     5  x_out = x_mid + sum over ranks (W_down * act)
// run inside one cooperative launch of one CTA per SM, separated by grid barriers (an atomic counter in global memory
// with a bounded wait) instead of kernel boundaries. Every phase issues its first weight loads BEFORE it waits at the
// barrier in front of it, so HBM latency hides behind the barrier. The two sums over ranks are the same one-shot
// (value, epoch)-pair exchange over NVLink peer memory that the stand-alone fused GEMV + all-reduce uses, executed by
// the CTA that owns the rows. Attention layers enter at phase 3 with o computed by the attention kernels.
//
// The reference reaches the same end with one CUDA graph per step over separate kernels (`enqueue_layer`,
// `crates/fe-model/src/model.rs:2981-3204`) and its NCCL-free `fx_ar_ll` exchange (`kernels/k-fnext/src/fast.rs:1376`);
// the arithmetic per phase here is that of `gemv_core.cuh` / `gdn_step.cuh`, the kernels the separate-launch path runs.
#include "api_ext.h"
#include "comm_core.cuh"
#include "gdn_step.cuh"
#include "gemv_core.cuh"

namespace fb {

constexpr int DL_THREADS = 512;
constexpr int DL_WARPS = DL_THREADS / 32;
constexpr int DL_R = 2;

struct DLSync {
  uint32_t* counter;      // arrivals, monotonic over all launches
  uint32_t* base;         // counter value at which the running launch started (written by the last arrival of a launch)
  int* status;
  unsigned spin_limit;
};

struct DLArgs {
  GemvArgs g_in, g_out, g_gu, g_down;
  // phase 2
  __nv_bfloat16* o;
  float* rec_state;
  __nv_bfloat16* conv_state;
  const __nv_bfloat16* conv_w;
  const float* A_log;
  const float* dt_bias;
  const __nv_bfloat16* gnorm_w;
  const int* seg_slot;
  int nk, nv, dk;
  float eps;
  int start_phase;        // 1: Gated DeltaNet layer, 3: enter with o given (attention layers)
  int M;
  int xs_bytes;           // bytes of the staged-activation area; the exchange tile follows it
  int rpc_out, rpc_down;  // rows per CTA of the two exchanged phases (tile row stride)
  CommBuf cb;             // world 1: no exchange
  DLSync sync;
};

struct DLBarrier {
  DLSync s;
  uint32_t base;
  int* abort_s;           // shared: a barrier ran out; later barriers return at once
  int n;                  // barriers passed so far
  int last;               // index of the launch's last barrier

  // Everyone has finished what it wrote before; nobody continues before all have arrived.
  __device__ __forceinline__ void sync() {
    __syncthreads();
    if (threadIdx.x == 0 && !*abort_s) {
      const uint32_t target = base + (uint32_t)(n + 1) * gridDim.x;
      __threadfence();
      const uint32_t old = atomicAdd(s.counter, 1u);
      if (old + 1 == target) {
        if (n == last) *reinterpret_cast<volatile uint32_t*>(s.base) = target;      // the next launch starts from here
      } else {
        bool ok = false;
        for (unsigned i = 0; i < s.spin_limit; ++i) {
          if ((int32_t)(ld_acquire_gpu(s.counter) - target) >= 0) { ok = true; break; }
        }
        if (!ok) { set_status(s.status, ST_PEER_TIMEOUT); *abort_s = 1; }
      }
      __threadfence();
    }
    ++n;
    __syncthreads();
  }
};

struct DLNoWait {
  __device__ __forceinline__ void before_loads() const {}
  __device__ __forceinline__ void wait() const {}
};
struct DLBarrierWait {
  DLBarrier* b;
  __device__ __forceinline__ void before_loads() const {}
  __device__ __forceinline__ void wait() const { b->sync(); }
};

template <int M, class Wait>
__device__ __forceinline__ void dl_gemv_store(const GemvArgs& g, __nv_bfloat16* xs, float* rscale, float* scratch, Wait w) {
  const int row_end = min(g.N, (int)(blockIdx.x + 1) * g.rows_per_cta);
  gemv_main_w<M, DL_R, false, DL_WARPS>(g, xs, rscale, scratch, [&](float (&acc)[DL_R][M], int n) {
    if ((threadIdx.x & 31) != 0) return;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      if (m >= g.M) break;
#pragma unroll
      for (int r = 0; r < DL_R; ++r) {
        const int nn = n + r;
        if (nn >= row_end) break;
        float v = acc[r][m];
        if (g.res) v += bf2f(g.res[(size_t)m * g.ldy + nn]);
        reinterpret_cast<__nv_bfloat16*>(g.Y)[(size_t)m * g.ldy + nn] = f2bf(v);
      }
    }
  }, w);
}

// W * x into the CTA's tile, the sum over ranks (world > 1), residual, bf16 rows out
template <int M, class Wait>
__device__ __forceinline__ void dl_gemv_reduce(const GemvArgs& g, const CommBuf& cb, uint32_t epoch, __nv_bfloat16* xs,
                                               float* tile, float* rscale, float* scratch, Wait w) {
  const int rpc = g.rows_per_cta;
  const int row0 = blockIdx.x * rpc;
  const int row_end = min(g.N, row0 + rpc);
  const int nrows = max(0, row_end - row0);
  for (int i = threadIdx.x; i < M * rpc; i += blockDim.x) tile[i] = 0.f;
  __syncthreads();
  gemv_main_w<M, DL_R, false, DL_WARPS>(g, xs, rscale, scratch, [&](float (&acc)[DL_R][M], int n) {
    if ((threadIdx.x & 31) != 0) return;
#pragma unroll
    for (int r = 0; r < DL_R; ++r)
      if (n + r < row_end)
#pragma unroll
        for (int m = 0; m < M; ++m) tile[m * rpc + (n + r - row0)] = acc[r][m];
  }, w);
  __syncthreads();
  if (cb.world > 1 && nrows > 0) cta_exchange_sum(cb, tile, M * rpc, (long)blockIdx.x * M * rpc, epoch);
  __syncthreads();
  for (int i = threadIdx.x; i < g.M * nrows; i += blockDim.x) {
    const int m = i / nrows, j = i % nrows;
    float v = tile[m * rpc + j];
    const size_t o = (size_t)m * g.ldy + row0 + j;
    if (g.res) v += bf2f(g.res[o]);
    reinterpret_cast<__nv_bfloat16*>(g.Y)[o] = f2bf(v);
  }
}

template <int M>
__global__ void __launch_bounds__(DL_THREADS, 1) decode_layer_kernel(DLArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float* tile = reinterpret_cast<float*>(smem_raw + a.xs_bytes);
  __shared__ float rscale[M];
  __shared__ float scratch[32];
  __shared__ uint32_t base_s;
  __shared__ int abort_s;
  if (threadIdx.x == 0) {
    base_s = *reinterpret_cast<volatile uint32_t*>(a.sync.base);
    abort_s = 0;
  }
  __syncthreads();
  DLBarrier bar{a.sync, base_s, &abort_s, 0, a.start_phase == 1 ? 3 : 1};
  uint32_t epoch = 0;
  if (a.cb.world > 1) epoch = comm_epoch_begin(a.cb);        // this launch uses epoch and epoch + 1

  if (a.start_phase == 1) {
    dl_gemv_store<M>(a.g_in, xs, rscale, scratch, DLNoWait());
    bar.sync();
    // every (head, sequence) pair has a CTA of its own (the host checks nv * M <= grid): the heads of a key group read
    // the conv tail their first head rewrites at the end
    const int pair = blockIdx.x;
    if (pair < a.nv * a.M) {
      const int h = pair % a.nv, seg = pair / a.nv;
      if (a.dk == 128)
        gdn_step_body<128, 128, 4>(a.o, a.rec_state, a.conv_state, reinterpret_cast<const __nv_bfloat16*>(a.g_in.Y),
                                   a.g_in.ldy, a.conv_w, a.A_log, a.dt_bias, a.gnorm_w, 1, seg, a.seg_slot[seg], h, a.nk,
                                   a.nv, a.eps, 1);
      else
        gdn_step_body<64, 64, 8>(a.o, a.rec_state, a.conv_state, reinterpret_cast<const __nv_bfloat16*>(a.g_in.Y),
                                 a.g_in.ldy, a.conv_w, a.A_log, a.dt_bias, a.gnorm_w, 1, seg, a.seg_slot[seg], h, a.nk,
                                 a.nv, a.eps, 1);
    }
    dl_gemv_reduce<M>(a.g_out, a.cb, epoch, xs, tile, rscale, scratch, DLBarrierWait{&bar});
  } else {
    dl_gemv_reduce<M>(a.g_out, a.cb, epoch, xs, tile, rscale, scratch, DLNoWait());
  }

  {
    const GemvArgs& g = a.g_gu;
    gemv_main_w<M, DL_R, true, DL_WARPS>(g, xs, rscale, scratch, [&](float (&acc)[DL_R][M], int n) {
      if ((threadIdx.x & 31) != 0) return;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        if (m >= g.M) break;
        reinterpret_cast<__nv_bfloat16*>(g.Y)[(size_t)m * g.ldy + n] = f2bf(siluf_(acc[0][m]) * acc[DL_R - 1][m]);
      }
    }, DLBarrierWait{&bar});
  }

  dl_gemv_reduce<M>(a.g_down, a.cb, epoch + 1, xs, tile, rscale, scratch, DLBarrierWait{&bar});
  if (a.cb.world > 1) comm_epoch_end(a.cb, epoch + 1);
}

struct DLPlan { int grid; size_t smem; };

static void dl_plan_gemv(GemvArgs& g, int M, int grid, bool swiglu) {
  g.kc = gemv_chunk_len(M, g.K);
  const int nchunks = (g.K + g.kc - 1) / g.kc;
  (void)nchunks; (void)swiglu;
  g.rows_per_cta = (g.N + grid - 1) / grid;
}

template <int M>
static int dl_launch(DLArgs& a, int grid, cudaStream_t s) {
  dl_plan_gemv(a.g_in, M, grid, false);
  dl_plan_gemv(a.g_out, M, grid, false);
  dl_plan_gemv(a.g_gu, M, grid, true);
  dl_plan_gemv(a.g_down, M, grid, false);
  int kc = a.g_out.kc > a.g_gu.kc ? a.g_out.kc : a.g_gu.kc;
  if (a.g_down.kc > kc) kc = a.g_down.kc;
  if (a.start_phase == 1 && a.g_in.kc > kc) kc = a.g_in.kc;
  a.xs_bytes = (int)((size_t)M * kc * sizeof(__nv_bfloat16));
  const int rpc = a.g_out.rows_per_cta > a.g_down.rows_per_cta ? a.g_out.rows_per_cta : a.g_down.rows_per_cta;
  const size_t smem = (size_t)a.xs_bytes + (size_t)M * rpc * sizeof(float);
  if (smem > 160 * 1024) return -5;
  if (a.cb.world > 1) {
    if (grid > a.cb.max_ctas) return -7;
    if ((long)grid * M * rpc * 2 > a.cb.slot_floats - COMM_TOP_RESERVE) return -8;
  }
  auto kern = decode_layer_kernel<M>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  // every CTA waits for every other: a cooperative launch makes the driver refuse a grid that cannot be resident at once
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(DL_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace fb

using namespace fb;

// Persistent decode layer. x_in/x_mid/x_out/act/proj/o: bf16 rows [M][...] (contiguous). start_phase 1: Gated DeltaNet
// layer (w_in, input_norm, states and head parameters used); 3: o is given. sync: two zero-initialised u32 words owned by
// the caller (counter, base), shared by all launches of a stream. world 1: peers may be null.
extern "C" int fb_decode_layer(int start_phase, int M, int hidden, void* x_out, void* x_mid, void* act, void* proj, void* o,
                               const void* x_in, const void* w_in, int n_in, const void* input_norm, const void* w_out,
                               int k_out, const void* post_norm, const void* w_gu, int inter, const void* w_down,
                               float* rec_state, void* conv_state, const void* conv_w, const float* A_log,
                               const float* dt_bias, const void* gnorm_w, const int* seg_slot, int nk, int nv, int dk,
                               float eps, const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                               uint32_t* epochs, int* status, unsigned spin_limit, uint32_t* sync_words, int sm_count,
                               cudaStream_t s) {
  if (M <= 0 || M > 4 || world > COMM_MAX_RANKS) return -1;
  if ((hidden % 8) || (k_out % 8) || (inter % 8)) return -1;
  if (sm_count <= 0) sm_count = 148;
  if (start_phase == 1 && (nv * M > sm_count || !(dk == 128 || dk == 64))) return -2;
  typedef const __nv_bfloat16* cbf;
  DLArgs a;
  auto fill = [&](GemvArgs& g, const void* X, long ldx, const void* W, const void* norm_w, const void* res, void* Y,
                  long ldy, int N, int K) {
    g.X = (cbf)X; g.W = (cbf)W; g.norm_w = (cbf)norm_w; g.res = (cbf)res; g.Y = Y; g.M = M; g.N = N; g.K = K;
    g.ldx = ldx; g.ldy = ldy; g.eps = eps; g.centred = 1; g.out_f32 = 0; g.rows_per_cta = 0; g.kc = 0;
  };
  fill(a.g_in, x_in, hidden, w_in ? w_in : w_out, input_norm, nullptr, proj, n_in, start_phase == 1 ? n_in : 1, hidden);
  fill(a.g_out, o, k_out, w_out, nullptr, x_in, x_mid, hidden, hidden, k_out);
  fill(a.g_gu, x_mid, hidden, w_gu, post_norm, nullptr, act, inter, inter, hidden);
  fill(a.g_down, act, inter, w_down, nullptr, x_mid, x_out, hidden, hidden, inter);
  a.o = (__nv_bfloat16*)o; a.rec_state = rec_state; a.conv_state = (__nv_bfloat16*)conv_state; a.conv_w = (cbf)conv_w;
  a.A_log = A_log; a.dt_bias = dt_bias; a.gnorm_w = (cbf)gnorm_w; a.seg_slot = seg_slot; a.nk = nk; a.nv = nv; a.dk = dk;
  a.eps = eps; a.start_phase = start_phase; a.M = M; a.xs_bytes = 0; a.rpc_out = a.rpc_down = 0;
  if (world > 1) {
    fill_comm(a.cb, peers, rank, world, max_ctas, slot_floats, epochs, status, spin_limit);
  } else {
    for (int i = 0; i < COMM_MAX_RANKS; ++i) a.cb.peer[i] = nullptr;
    a.cb.rank = 0; a.cb.world = 1; a.cb.max_ctas = 0; a.cb.slot_floats = 0; a.cb.epochs = nullptr; a.cb.status = status;
    a.cb.spin_limit = 0; a.cb.serial_polls = 0; a.cb.trace = nullptr;
  }
  a.cb.trace = nullptr;
  a.sync.counter = sync_words; a.sync.base = sync_words + 1; a.sync.status = status;
  a.sync.spin_limit = spin_limit ? spin_limit : (1u << 22);
  const int grid = sm_count;
  if (M == 1) return dl_launch<1>(a, grid, s);
  if (M == 2) return dl_launch<2>(a, grid, s);
  return dl_launch<4>(a, grid, s);
}
