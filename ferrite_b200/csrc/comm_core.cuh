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
//   flags : [2 parity][COMM_MAX_RANKS][max_ctas] u32            (argmax gather)
//   data  : [2 parity][COMM_MAX_RANKS][slot_floats] 4-byte words: (value, epoch) pairs of the all-reduce
struct CommBuf {
  void* peer[COMM_MAX_RANKS];      // base of the workspace on each rank (peer[rank] = local)
  int rank, world;
  int max_ctas;
  long slot_floats;
  uint32_t* epochs;                // local, [max_ctas]: per-CTA launch counter
  int* status;
  unsigned spin_limit;
};

__device__ __forceinline__ uint32_t* comm_flags(void* base, const CommBuf& cb, int parity, int src, int cta) {
  return reinterpret_cast<uint32_t*>(base) + ((size_t)parity * COMM_MAX_RANKS + src) * cb.max_ctas + cta;
}
__device__ __forceinline__ float* comm_data(void* base, const CommBuf& cb, int parity, int src) {
  char* p = reinterpret_cast<char*>(base) + (size_t)2 * COMM_MAX_RANKS * cb.max_ctas * sizeof(uint32_t);
  return reinterpret_cast<float*>(p) + ((size_t)parity * COMM_MAX_RANKS + src) * cb.slot_floats;
}

// Exchange one CTA's tile. `tile` = fp32 values in shared memory, `count` of them, living at value offset `off`
// of the slot. After the call `tile` holds the rank-ordered sum. All threads of the CTA call this.
//
// Low-latency protocol: every value travels as an 8-byte (value, epoch) pair written with one store, so the
// receiver needs no separate flag and the sender no system-wide fence: a pair whose epoch word matches is complete.
// (The reference's host-memory all-reduce uses the same idea, `fx_ar_ll` in `kernels/k-fnext/src/fast.rs:1376`.)
// A slot therefore holds slot_floats / 2 values. Polls are bounded; on expiry the status word is set, the sum is
// left incomplete and the kernel returns normally.
__device__ __forceinline__ void cta_exchange_sum(const CommBuf& cb, float* tile, int count, long off) {
  __shared__ uint32_t s_epoch;
  const int cta = blockIdx.x;
  if (threadIdx.x == 0) s_epoch = cb.epochs[cta] + 1;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int parity = epoch & 1;
  for (int p = 0; p < cb.world; ++p) {
    if (p == cb.rank) continue;
    uint2* dst = reinterpret_cast<uint2*>(comm_data(cb.peer[p], cb, parity, cb.rank)) + off;
    for (int i = threadIdx.x; i < count; i += blockDim.x) st_relaxed_sys_v2(dst + i, __float_as_uint(tile[i]), epoch);
  }
  bool fail = false;
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < cb.world; ++r) {                       // rank order: every rank adds the same bits the same way
      if (r == cb.rank) { acc += tile[i]; continue; }
      const uint2* src = reinterpret_cast<const uint2*>(comm_data(cb.peer[cb.rank], cb, parity, r)) + off + i;
      uint2 v = ld_relaxed_sys_v2(src);
      for (uint32_t spin = 0; v.y != epoch && spin < cb.spin_limit; ++spin) v = ld_relaxed_sys_v2(src);
      if (v.y != epoch) fail = true;
      acc += __uint_as_float(v.x);
    }
    tile[i] = acc;
  }
  if (fail) set_status(cb.status, ST_PEER_TIMEOUT);
  __syncthreads();
  if (threadIdx.x == 0) cb.epochs[cta] = epoch;
}

static inline void fill_comm(CommBuf& cb, const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                      uint32_t* epochs, int* status, unsigned spin_limit) {
  for (int i = 0; i < COMM_MAX_RANKS; ++i) cb.peer[i] = i < world ? const_cast<void*>(peers[i]) : nullptr;
  cb.rank = rank; cb.world = world; cb.max_ctas = max_ctas; cb.slot_floats = slot_floats; cb.epochs = epochs;
  cb.status = status; cb.spin_limit = spin_limit ? spin_limit : (1u << 23);   // a few seconds of polling
}

}  // namespace fb
