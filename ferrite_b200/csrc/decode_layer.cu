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
// run inside one launch of one CTA per SM, separated by grid barriers (an atomic counter in global memory
// with a bounded wait) instead of kernel boundaries. Every phase issues its first weight loads BEFORE it waits at the
// barrier in front of it, so HBM latency hides behind the barrier. (Asking L2 for the whole next phase's rows with
// cp.async.bulk.prefetch.L2 while a phase runs was measured too: the step got 11 % slower at tensor-parallel 8.)
// The two sums over ranks are the same one-shot (value, epoch)-pair exchange over NVLink peer memory that the
// stand-alone fused GEMV + all-reduce uses, executed by
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
constexpr int DL_TRACE_RECS = 1024;
constexpr int DL_TRACE_WORDS = 16;   // 0 start, 1 in_proj done, 2 barrier, 3 heads done, 4 barrier, 5 out_proj done, 6 summed + stored,
                                     // 7 barrier, 8 gate|up done, 9 barrier, 10 down done, 11 summed + stored, 12 start phase

struct DLSync {
  uint32_t* counter;      // arrivals, monotonic over all launches
  uint32_t* base;         // counter value at which the running launch started (written by the last arrival of a launch)
  int* status;
  unsigned spin_limit;
};

constexpr int DL_MAX_LAYERS = 4;

struct DLLayer {
  GemvArgs g_in, g_out, g_gu, g_down;
  // phase 2
  __nv_bfloat16* o;
  float* rec_state;
  __nv_bfloat16* conv_state;
  const __nv_bfloat16* conv_w;
  const float* A_log;
  const float* dt_bias;
  const __nv_bfloat16* gnorm_w;
  int start_phase;        // 1: Gated DeltaNet layer, 3: enter with o given (attention layers)
};

// A run of consecutive layers in one launch: only the first may enter at phase 3.
struct DLArgs {
  DLLayer L[DL_MAX_LAYERS];
  int n_layers;
  const int* seg_slot;
  int nk, nv, dk;
  float eps;
  int M;
  int xs_bytes;           // bytes of the staged-activation area; the exchange tile follows it
  int n_barriers;         // grid barriers of the whole launch
  unsigned long long* trace;   // null, or [DL_TRACE_RECS][DL_TRACE_WORDS] %globaltimer stamps of CTA 0 (profiling)
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

// What a phase waits for once its first weight loads are in flight. FIRST (first phase of a launch): the previous
// kernel of the stream (programmatic dependent launch); only then are the words that kernel may have written read, the
// barrier base and the exchange epoch. BARRIER: the grid barrier in front of the phase.
struct DLWait {
  enum Mode { FIRST, BARRIER };
  Mode mode;
  DLBarrier* b;
  uint32_t* base_s;
  const CommBuf* cb;
  uint32_t* epoch;
  __device__ __forceinline__ void before_loads() const { if (mode == FIRST) pdl_launch_dependents(); }
  __device__ __forceinline__ void wait() const {
    if (mode == BARRIER) { b->sync(); return; }
    pdl_wait();
    if (threadIdx.x == 0) *base_s = *reinterpret_cast<volatile uint32_t*>(b->s.base);
    __syncthreads();
    b->base = *base_s;
    if (cb->world > 1) *epoch = comm_epoch_begin(*cb);      // the launch uses epoch, epoch + 1, ...
  }
};

template <int M, class Wait>
__device__ __forceinline__ void dl_gemv_store(const GemvArgs& g, __nv_bfloat16* xs, float* rscale, float* scratch, Wait w,
                                              unsigned long long* wait_stamp = nullptr) {
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
  }, w, wait_stamp);
}

// W * x into the CTA's tile, the sum over ranks (world > 1), residual, bf16 rows out
__device__ __forceinline__ void dl_stamp(unsigned long long* st, int i) {
  if (st != nullptr && threadIdx.x == 0) st[i] = comm_now();
}

template <int M, class Wait>
__device__ __forceinline__ void dl_gemv_reduce(const GemvArgs& g, const CommBuf& cb, const uint32_t& epoch0,
                                               uint32_t epoch_add, __nv_bfloat16* xs, float* tile, float* rscale,
                                               float* scratch, Wait w, unsigned long long* st = nullptr, int st0 = 0) {
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
  }, w, st ? st + st0 : nullptr);
  __syncthreads();
  dl_stamp(st, st0 + 1);
  // (epoch0 is set by the launch's first wait, which may be the one inside the loop above)
  if (cb.world > 1 && nrows > 0) cta_exchange_sum(cb, tile, M * rpc, (long)blockIdx.x * M * rpc, epoch0 + epoch_add);
  __syncthreads();
  for (int i = threadIdx.x; i < g.M * nrows; i += blockDim.x) {
    const int m = i / nrows, j = i % nrows;
    float v = tile[m * rpc + j];
    const size_t o = (size_t)m * g.ldy + row0 + j;
    if (g.res) v += bf2f(g.res[o]);
    reinterpret_cast<__nv_bfloat16*>(g.Y)[o] = f2bf(v);
  }
  dl_stamp(st, st0 + 2);
}

template <int M>
__global__ void __launch_bounds__(DL_THREADS, 1) decode_layer_kernel(const __grid_constant__ DLArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float* tile = reinterpret_cast<float*>(smem_raw + a.xs_bytes);
  __shared__ float rscale[M];
  __shared__ float scratch[32];
  __shared__ uint32_t base_s;
  __shared__ int abort_s;
  __shared__ unsigned long long stamps_s[DL_TRACE_WORDS];
  unsigned long long* st = (a.trace != nullptr && blockIdx.x == 0) ? stamps_s : nullptr;
  if (threadIdx.x == 0) abort_s = 0;
  __syncthreads();
  DLBarrier bar{a.sync, 0u, &abort_s, 0, a.n_barriers - 1};
  uint32_t epoch = 0;
  const DLWait first{DLWait::FIRST, &bar, &base_s, &a.cb, &epoch};
  const DLWait at_barrier{DLWait::BARRIER, &bar, &base_s, &a.cb, &epoch};

  for (int li = 0; li < a.n_layers; ++li) {
    const DLLayer& L = a.L[li];
    const DLWait& enter = li == 0 ? first : at_barrier;
    const int n_at_start = bar.n;
    if (st != nullptr && threadIdx.x == 0) {
      for (int i = 0; i < DL_TRACE_WORDS; ++i) st[i] = 0;
      st[0] = comm_now(); st[12] = (unsigned long long)L.start_phase; st[14] = (unsigned long long)li;
    }
    if (L.start_phase == 1) {
      dl_gemv_store<M>(L.g_in, xs, rscale, scratch, enter, st ? st + 13 : nullptr);
      dl_stamp(st, 1);
      bar.sync();
      dl_stamp(st, 2);
      // every (head, sequence) pair has a CTA of its own (the host checks nv * M <= grid): the heads of a key group
      // read the conv tail their first head rewrites at the end
      const int pair = blockIdx.x;
      if (pair < a.nv * a.M) {
        const int h = pair % a.nv, seg = pair / a.nv;
        if (a.dk == 128)
          gdn_step_body<128, 128, 4>(L.o, L.rec_state, L.conv_state, reinterpret_cast<const __nv_bfloat16*>(L.g_in.Y),
                                     L.g_in.ldy, L.conv_w, L.A_log, L.dt_bias, L.gnorm_w, 1, seg, a.seg_slot[seg], h, a.nk,
                                     a.nv, a.eps, 1);
        else
          gdn_step_body<64, 64, 8>(L.o, L.rec_state, L.conv_state, reinterpret_cast<const __nv_bfloat16*>(L.g_in.Y),
                                   L.g_in.ldy, L.conv_w, L.A_log, L.dt_bias, L.gnorm_w, 1, seg, a.seg_slot[seg], h, a.nk,
                                   a.nv, a.eps, 1);
      }
      dl_stamp(st, 3);
      dl_gemv_reduce<M>(L.g_out, a.cb, epoch, 2u * li, xs, tile, rscale, scratch, at_barrier, st, 4);
    } else {
      dl_gemv_reduce<M>(L.g_out, a.cb, epoch, 2u * li, xs, tile, rscale, scratch, enter, st, 4);
      if (st != nullptr && threadIdx.x == 0) st[13] = st[4];
    }

    {
      const GemvArgs& g = L.g_gu;
      gemv_main_w<M, DL_R, true, DL_WARPS>(g, xs, rscale, scratch, [&](float (&acc)[DL_R][M], int n) {
        if ((threadIdx.x & 31) != 0) return;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          if (m >= g.M) break;
          reinterpret_cast<__nv_bfloat16*>(g.Y)[(size_t)m * g.ldy + n] = f2bf(siluf_(acc[0][m]) * acc[DL_R - 1][m]);
        }
      }, at_barrier, st ? st + 7 : nullptr);
      dl_stamp(st, 8);
    }

    dl_gemv_reduce<M>(L.g_down, a.cb, epoch, 2u * li + 1u, xs, tile, rscale, scratch, at_barrier, st, 9);
    if (st != nullptr && threadIdx.x == 0) {
      unsigned long long* rec = a.trace + (size_t)((base_s / gridDim.x + (uint32_t)n_at_start) % DL_TRACE_RECS) * DL_TRACE_WORDS;
      for (int i = 0; i < DL_TRACE_WORDS; ++i) rec[i] = st[i];
    }
  }
  if (a.cb.world > 1) comm_epoch_end(a.cb, epoch + 2u * a.n_layers - 1u);
}

static void dl_plan_gemv(GemvArgs& g, int M, int grid) {
  g.kc = gemv_chunk_len(M, g.K);
  g.rows_per_cta = (g.N + grid - 1) / grid;
}

constexpr size_t DL_SMEM_MAX = 160 * 1024;

// Attribute set-up and the residency check, once per instantiation and never inside a stream capture (the engine calls
// fb_decode_layers_prepare when it is built): one CTA of the largest shared-memory size must fit an SM.
template <int M>
static int dl_prepare() {
  static int state = 0;                       // 0: not yet, 1: ready, < 0: error
  if (state == 0) {
    auto kern = decode_layer_kernel<M>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DL_SMEM_MAX);
    int per_sm = 0;
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, DL_THREADS, DL_SMEM_MAX);
    state = (e == cudaSuccess && per_sm >= 1) ? 1 : -9;
  }
  return state == 1 ? 0 : state;
}

template <int M>
static int dl_launch(DLArgs& a, int grid, cudaStream_t s) {
  int kc = 0, rpc = 0;
  a.n_barriers = a.n_layers - 1;
  for (int li = 0; li < a.n_layers; ++li) {
    DLLayer& L = a.L[li];
    dl_plan_gemv(L.g_in, M, grid);
    dl_plan_gemv(L.g_out, M, grid);
    dl_plan_gemv(L.g_gu, M, grid);
    dl_plan_gemv(L.g_down, M, grid);
    if (L.start_phase == 1 && L.g_in.kc > kc) kc = L.g_in.kc;
    if (L.g_out.kc > kc) kc = L.g_out.kc;
    if (L.g_gu.kc > kc) kc = L.g_gu.kc;
    if (L.g_down.kc > kc) kc = L.g_down.kc;
    if (L.g_out.rows_per_cta > rpc) rpc = L.g_out.rows_per_cta;
    if (L.g_down.rows_per_cta > rpc) rpc = L.g_down.rows_per_cta;
    a.n_barriers += L.start_phase == 1 ? 4 : 2;
  }
  a.xs_bytes = (int)((size_t)M * kc * sizeof(__nv_bfloat16));
  const size_t smem = (size_t)a.xs_bytes + (size_t)M * rpc * sizeof(float);
  if (smem > DL_SMEM_MAX) return -5;
  if (a.cb.world > 1) {
    if (grid > a.cb.max_ctas) return -7;
    if ((long)grid * M * rpc * 2 > a.cb.slot_floats - COMM_TOP_RESERVE) return -8;
  }
  auto kern = decode_layer_kernel<M>;
  if (int rc = dl_prepare<M>()) return rc;
  // Every CTA waits for every other, so all of them must be resident together: one per SM, checked against what the
  // occupancy calculator allows. (A cooperative launch would have the driver check the same, but measured 15 us from the
  // end of one such launch to the start of the next inside a CUDA graph; a plain launch with programmatic dependent
  // launch lets the next launch's CTAs start, and request their first weights, as SMs free up. CTAs of earlier kernels
  // never wait for this one, so they drain and every CTA of this grid gets its SM; the barrier waits are bounded.)
  return (int)launch_pdl(kern, dim3(grid), dim3(DL_THREADS), smem, s, a);
}

}  // namespace fb

using namespace fb;

static unsigned long long* g_dl_trace = nullptr;
// Profiling: a device buffer of [1024][16] 64-bit words that CTA 0 of every later launch stamps (nullptr: off). Set it
// before a CUDA graph is captured.
extern "C" void fb_decode_layer_trace_set(void* buf) { g_dl_trace = (unsigned long long*)buf; }

extern "C" int fb_decode_layers_max() { return DL_MAX_LAYERS; }

// Call once outside any stream capture before the first fb_decode_layers.
extern "C" int fb_decode_layers_prepare() {
  if (int rc = dl_prepare<1>()) return rc;
  if (int rc = dl_prepare<2>()) return rc;
  return dl_prepare<4>();
}

// A run of n_layers consecutive decoder layers (<= fb_decode_layers_max()) for M <= 4 one-row sequences. Per layer, in
// arrays of n_layers entries: start_phase (1: Gated DeltaNet layer from the hidden rows; 3: the rest of a layer whose
// mixer output o is given, first layer of the run only), the buffers x_out / x_mid / act / proj / o (bf16, contiguous
// rows) and the weights; layer l reads the rows layer l - 1 wrote (x_in for the first). sync: two zero-initialised
// u32 words owned by the caller (counter, base), shared by all launches of a stream. world 1: peers may be null.
extern "C" int fb_decode_layers(int n_layers, const int* start_phase, int M, int hidden, const void* x_in,
                                void* const* x_out, void* const* x_mid, void* const* act, void* const* proj,
                                void* const* o, const void* const* w_in, const int* n_in,
                                const void* const* input_norm, const void* const* w_out, const int* k_out,
                                const void* const* post_norm, const void* const* w_gu, int inter,
                                const void* const* w_down, float* const* rec_state, void* const* conv_state,
                                const void* const* conv_w, const float* const* A_log, const float* const* dt_bias,
                                const void* const* gnorm_w, const int* seg_slot, int nk, int nv, int dk, float eps,
                                const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                                uint32_t* epochs, int* status, unsigned spin_limit, uint32_t* sync_words, int sm_count,
                                cudaStream_t s) {
  if (M <= 0 || M > 4 || world > COMM_MAX_RANKS || n_layers < 1 || n_layers > DL_MAX_LAYERS) return -1;
  if ((hidden % 8) || (inter % 8)) return -1;
  if (sm_count <= 0) sm_count = 148;
  typedef const __nv_bfloat16* cbf;
  DLArgs a;
  auto fill = [&](GemvArgs& g, const void* X, long ldx, const void* W, const void* norm_w, const void* res, void* Y,
                  long ldy, int N, int K) {
    g.X = (cbf)X; g.W = (cbf)W; g.norm_w = (cbf)norm_w; g.res = (cbf)res; g.Y = Y; g.M = M; g.N = N; g.K = K;
    g.ldx = ldx; g.ldy = ldy; g.eps = eps; g.centred = 1; g.out_f32 = 0; g.rows_per_cta = 0; g.kc = 0;
  };
  const void* x_prev = x_in;
  for (int li = 0; li < n_layers; ++li) {
    DLLayer& L = a.L[li];
    const int sp = start_phase[li];
    if (sp != 1 && !(sp == 3 && li == 0)) return -2;
    if (sp == 1 && (nv * M > sm_count || !(dk == 128 || dk == 64))) return -2;
    if (k_out[li] % 8) return -1;
    fill(L.g_in, x_prev, hidden, sp == 1 ? w_in[li] : w_out[li], sp == 1 ? input_norm[li] : nullptr, nullptr, proj[li],
         sp == 1 ? n_in[li] : 1, sp == 1 ? n_in[li] : 1, hidden);
    fill(L.g_out, o[li], k_out[li], w_out[li], nullptr, x_prev, x_mid[li], hidden, hidden, k_out[li]);
    fill(L.g_gu, x_mid[li], hidden, w_gu[li], post_norm[li], nullptr, act[li], inter, inter, hidden);
    fill(L.g_down, act[li], inter, w_down[li], nullptr, x_mid[li], x_out[li], hidden, hidden, inter);
    L.o = (__nv_bfloat16*)o[li];
    L.rec_state = sp == 1 ? rec_state[li] : nullptr;
    L.conv_state = sp == 1 ? (__nv_bfloat16*)conv_state[li] : nullptr;
    L.conv_w = sp == 1 ? (cbf)conv_w[li] : nullptr;
    L.A_log = sp == 1 ? A_log[li] : nullptr;
    L.dt_bias = sp == 1 ? dt_bias[li] : nullptr;
    L.gnorm_w = sp == 1 ? (cbf)gnorm_w[li] : nullptr;
    L.start_phase = sp;
    x_prev = x_out[li];
  }
  a.n_layers = n_layers; a.seg_slot = seg_slot; a.nk = nk; a.nv = nv; a.dk = dk; a.eps = eps; a.M = M; a.xs_bytes = 0;
  a.n_barriers = 0; a.trace = g_dl_trace;
  if (world > 1) {
    fill_comm(a.cb, peers, rank, world, max_ctas, slot_floats, epochs, status, spin_limit);
  } else {
    for (int i = 0; i < COMM_MAX_RANKS; ++i) a.cb.peer[i] = nullptr;
    a.cb.rank = 0; a.cb.world = 1; a.cb.max_ctas = 0; a.cb.slot_floats = 0; a.cb.epochs = nullptr; a.cb.status = status;
    a.cb.spin_limit = 0; a.cb.serial_polls = 0;
  }
  a.cb.trace = nullptr;
  a.sync.counter = sync_words; a.sync.base = sync_words + 1; a.sync.status = status;
  a.sync.spin_limit = spin_limit ? spin_limit : (1u << 22);
  const int grid = sm_count;
  if (M == 1) return dl_launch<1>(a, grid, s);
  if (M == 2) return dl_launch<2>(a, grid, s);
  return dl_launch<4>(a, grid, s);
}
