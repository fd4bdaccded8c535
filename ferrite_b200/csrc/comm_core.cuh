// Shared pieces of the kernels that exchange data over NVLink peer memory: the symmetric workspace layout, the
// flag protocol and the per-CTA push / bounded wait / rank-ordered sum. Included by every .cu file that fuses a
// collective into its epilogue.
#pragma once
#include "common.cuh"

namespace fb {

constexpr int COMM_MAX_RANKS = 8;
constexpr int COMM_MAX_ROWS = 8;

// Layout of the symmetric workspace (identical on every rank):
//   flags : [2 parity][COMM_MAX_RANKS][max_ctas] u32
//   data  : [2 parity][COMM_MAX_RANKS][slot_floats] f32
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

// Exchange one CTA's tile. `tile` = fp32 values in shared memory, `count` of them, living at float offset
// `off` of the slot. After the call `tile` holds the rank-ordered sum. All threads of the CTA call this.
__device__ __forceinline__ void cta_exchange_sum(const CommBuf& cb, float* tile, int count, long off) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_fail;
  const int cta = blockIdx.x;
  if (threadIdx.x == 0) { s_epoch = cb.epochs[cta] + 1; s_fail = 0; }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int parity = epoch & 1;
  // push to every rank (self included, so the sum below reads one layout)
  for (int p = 0; p < cb.world; ++p) {
    float* dst = comm_data(cb.peer[p], cb, parity, cb.rank) + off;
    for (int i = threadIdx.x * 4; i < count; i += blockDim.x * 4) {
      if (i + 4 <= count) {
        st_relaxed_sys_v4(dst + i, *reinterpret_cast<const uint4*>(tile + i));
      } else {
        for (int j = i; j < count; ++j) dst[j] = tile[j];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < cb.world) {
    st_release_sys(comm_flags(cb.peer[threadIdx.x], cb, parity, cb.rank, cta), epoch);
  }
  // wait for the same tile from every rank
  if (threadIdx.x < cb.world) {
    const uint32_t* f = comm_flags(cb.peer[cb.rank], cb, parity, threadIdx.x, cta);
    if (!wait_flag_eq(f, epoch, cb.spin_limit)) { s_fail = 1; set_status(cb.status, ST_PEER_TIMEOUT); }
  }
  __syncthreads();
  if (!s_fail) {
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
      float acc = 0.f;
      for (int r = 0; r < cb.world; ++r)
        acc += __ldcg(comm_data(cb.peer[cb.rank], cb, parity, r) + off + i);     // rank order, L2 (peer-written)
      tile[i] = acc;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) cb.epochs[cta] = epoch;
}

static inline void fill_comm(CommBuf& cb, const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                      uint32_t* epochs, int* status, unsigned spin_limit) {
  for (int i = 0; i < COMM_MAX_RANKS; ++i) cb.peer[i] = i < world ? const_cast<void*>(peers[i]) : nullptr;
  cb.rank = rank; cb.world = world; cb.max_ctas = max_ctas; cb.slot_floats = slot_floats; cb.epochs = epochs;
  cb.status = status; cb.spin_limit = spin_limit ? spin_limit : FB_PEER_SPIN_LIMIT;
}

}  // namespace fb
