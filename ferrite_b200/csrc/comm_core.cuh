// Shared pieces of the kernels that exchange data over NVLink peer memory: the symmetric workspace layout, the
// flag protocol and the per-CTA push / bounded wait / rank-ordered sum. Included by every .cu file that fuses a
// collective into its epilogue.
#pragma once
#include "common.cuh"

namespace fb {

constexpr int COMM_MAX_RANKS = 8;
constexpr int COMM_MAX_ROWS = 8;
constexpr int COMM_TOP_RESERVE = 1024;   // words at the top of every data slot kept for the argmax candidates

// Layout of the symmetric workspace (identical on every rank):
//   flags : [2 parity][COMM_MAX_RANKS][max_ctas] u32            (kept for layout compatibility; unused)
//   data  : [2 parity][COMM_MAX_RANKS][slot_floats] 4-byte words: (value, epoch) pairs of the all-reduce
struct CommBuf {
  void* peer[COMM_MAX_RANKS];      // base of the workspace on each rank (peer[rank] = local)
  int rank, world;
  int max_ctas;
  long slot_floats;
  uint32_t* epochs;                // local: [0] = epoch of the last finished call, [1] = CTAs of the running call done
  int* status;
  unsigned spin_limit;
  int serial_polls;                // 1: poll the sources one after the other (kept for A/B timing)
  unsigned long long* trace;       // null, or [COMM_TRACE_RECS][COMM_TRACE_WORDS] device timestamps (profiling)
};

constexpr int COMM_TRACE_RECS = 1024;
constexpr int COMM_TRACE_WORDS = 8;   // predecessor done, exchange begin, stores issued, first peer, last peer, end, epoch, grid

__device__ __forceinline__ unsigned long long comm_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t* comm_flags(void* base, const CommBuf& cb, int parity, int src, int cta) {
  return reinterpret_cast<uint32_t*>(base) + ((size_t)parity * COMM_MAX_RANKS + src) * cb.max_ctas + cta;
}
__device__ __forceinline__ float* comm_data(void* base, const CommBuf& cb, int parity, int src) {
  char* p = reinterpret_cast<char*>(base) + (size_t)2 * COMM_MAX_RANKS * cb.max_ctas * sizeof(uint32_t);
  return reinterpret_cast<float*>(p) + ((size_t)parity * COMM_MAX_RANKS + src) * cb.slot_floats;
}

// ---- one epoch per call ------------------------------------------------------------------------------------
// Every kernel that exchanges through this workspace is one "call". All CTAs of a call use the same epoch,
// epochs[0] + 1, read at entry (after griddepcontrol.wait, so the previous call of the stream has finished and
// published its epoch); the last CTA to finish publishes the new epoch. Invariants that make the pairs safe:
//   * epochs grow by one per call whatever the kernel, grid or tile layout, so a pair left anywhere in the
//     slots by an earlier call carries a smaller epoch and can never be mistaken for this call's;
//   * a call writes the parity (epoch & 1) half of the slots. A rank starts call e + 2 only after it finished
//     call e + 1, which needed every peer's pairs of call e + 1, which a peer sends only after its own call e
//     has finished reading: nobody overwrites pairs that are still being read.
// All ranks must issue the same sequence of calls (the engine runs in lockstep).
__device__ __forceinline__ uint32_t comm_epoch_begin(const CommBuf& cb) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(cb.epochs) + 1;
  __syncthreads();
  return s_epoch;
}
// Called by every thread of every CTA once its exchanges are done (the barrier inside orders them first).
__device__ __forceinline__ void comm_epoch_end(const CommBuf& cb, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(cb.epochs + 1, 1u) == total - 1) {
      cb.epochs[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(cb.epochs) = epoch;
    }
  }
}

// Exchange one CTA's tile. `tile` = fp32 values in shared memory, `count` of them, living at value offset `off`
// of the slot. After the call `tile` holds the rank-ordered sum. All threads of the CTA call this.
//
// Low-latency protocol: every value travels as an 8-byte (value, epoch) pair written with one store, so the
// receiver needs no separate flag and the sender no system-wide fence: a pair whose epoch word matches is complete.
// (The reference's host-memory all-reduce uses the same idea, `fx_ar_ll` in `kernels/k-fnext/src/fast.rs:1376`.)
// A slot therefore holds slot_floats / 2 values. The polls of all sources are in flight together; they are
// bounded, and on expiry the status word is set, the sum is left incomplete and the kernel returns normally.
__device__ __forceinline__ void cta_exchange_sum(const CommBuf& cb, float* tile, int count, long off, uint32_t epoch,
                                                 unsigned long long* stamps = nullptr) {
  const int parity = epoch & 1;
  const bool tr = stamps != nullptr && threadIdx.x == 0;
  if (tr) stamps[1] = comm_now();
  for (int p = 0; p < cb.world; ++p) {
    if (p == cb.rank) continue;
    uint2* dst = reinterpret_cast<uint2*>(comm_data(cb.peer[p], cb, parity, cb.rank)) + off;
    for (int i = threadIdx.x; i < count; i += blockDim.x) st_relaxed_sys_v2(dst + i, __float_as_uint(tile[i]), epoch);
  }
  if (tr) { stamps[2] = comm_now(); stamps[3] = 0; }
  bool fail = false;
  const uint2* mine = reinterpret_cast<const uint2*>(comm_data(cb.peer[cb.rank], cb, parity, 0)) + off;
  const size_t src_stride = (size_t)cb.slot_floats / 2;           // uint2 elements between two sources' slots
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    uint2 v[COMM_MAX_RANKS];
    if (cb.serial_polls) {
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r) {
        if (r >= cb.world || r == cb.rank) continue;
        const uint2* src = mine + r * src_stride + i;
        v[r] = ld_relaxed_sys_v2(src);
        for (uint32_t spin = 0; v[r].y != epoch && spin < cb.spin_limit; ++spin) v[r] = ld_relaxed_sys_v2(src);
        if (v[r].y != epoch) fail = true;
      }
    } else {
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r) v[r] = make_uint2(0u, epoch - 1);
      bool pending = true;
      for (uint32_t spin = 0; pending && spin < cb.spin_limit; ++spin) {
        pending = false;
#pragma unroll
        for (int r = 0; r < COMM_MAX_RANKS; ++r)            // all missing sources are requested before any is tested
          if (r < cb.world && r != cb.rank && v[r].y != epoch) v[r] = ld_relaxed_sys_v2(mine + r * src_stride + i);
#pragma unroll
        for (int r = 0; r < COMM_MAX_RANKS; ++r)
          if (r < cb.world && r != cb.rank && v[r].y != epoch) pending = true;
        if (tr && i == 0 && stamps[3] == 0) {
          bool any = false;
#pragma unroll
          for (int r = 0; r < COMM_MAX_RANKS; ++r) any |= (r < cb.world && r != cb.rank && v[r].y == epoch);
          if (any) stamps[3] = comm_now();
        }
      }
      if (pending) fail = true;
    }
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < COMM_MAX_RANKS; ++r) {               // rank order: every rank adds the same bits the same way
      if (r >= cb.world) continue;
      acc += (r == cb.rank) ? tile[i] : __uint_as_float(v[r].x);
    }
    tile[i] = acc;
    if (tr && i == 0) { stamps[4] = comm_now(); if (stamps[3] == 0) stamps[3] = stamps[4]; }
  }
  if (fail) set_status(cb.status, ST_PEER_TIMEOUT);
}

// Flush the stamps of CTA 0 into the trace ring (profiling runs only).
__device__ __forceinline__ void comm_trace_flush(const CommBuf& cb, const unsigned long long* stamps, uint32_t epoch) {
  if (cb.trace == nullptr || blockIdx.x != 0 || threadIdx.x != 0) return;
  unsigned long long* rec = cb.trace + (size_t)(epoch % COMM_TRACE_RECS) * COMM_TRACE_WORDS;
  for (int j = 0; j < 5; ++j) rec[j] = stamps[j];
  rec[5] = comm_now();
  rec[6] = epoch;
  rec[7] = gridDim.x;
}

}  // namespace fb

// Process-wide profiling switches, defined in comm.cu.
extern "C" unsigned long long* fb_comm_trace_get();
extern "C" int fb_comm_serial_polls_get();

namespace fb {

static inline void fill_comm(CommBuf& cb, const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                      uint32_t* epochs, int* status, unsigned spin_limit) {
  for (int i = 0; i < COMM_MAX_RANKS; ++i) cb.peer[i] = i < world ? const_cast<void*>(peers[i]) : nullptr;
  cb.rank = rank; cb.world = world; cb.max_ctas = max_ctas; cb.slot_floats = slot_floats; cb.epochs = epochs;
  cb.status = status; cb.spin_limit = spin_limit ? spin_limit : (1u << 23);   // a few seconds of polling
  cb.serial_polls = fb_comm_serial_polls_get();
  cb.trace = fb_comm_trace_get();
}

}  // namespace fb
