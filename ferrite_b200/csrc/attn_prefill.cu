// Causal flash attention for prompt chunks over the paged KV cache (the chunk's own K/V rows are already in
// the cache, written by attn-prep). One CTA = 64 query rows of one q head; keys stream through shared memory
// in 32-key tiles with a two-stage cp.async pipeline; online softmax in registers; sigmoid output gate fused
// into the epilogue.
//
// This is the warp-level tensor-core (mma.sync m16n8k16) formulation: attention is under 1% of the FLOPs of a
// 2K-token prefill of this model, so the tcgen05 budget went to the GEMMs first. Counterpart of the
// reference's `fe_flash_prefill` (`kernels/k-core/src/flash.rs:50`, BQ 64 / BKV 32 / hd 256 with the gate
// epilogue), generalised to run-time head counts, head_dim 64/128/256 and a paged cache with a prefix.
#include "api.h"
#include "common.cuh"

namespace fb {

constexpr int FP_BQ = 64, FP_BKV = 32, FP_WARPS = 4;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int HD>
__global__ void __launch_bounds__(FP_WARPS * 32)
attn_prefill_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
                    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                    const __nv_bfloat16* __restrict__ proj, long proj_stride, const int* __restrict__ seg_slot,
                    const int* __restrict__ seg_row0, const int* __restrict__ seg_nrows,
                    const int* __restrict__ seg_pos0, const int* __restrict__ block_table, int max_blocks,
                    int kv_block, int nq, int nkv, int gated, float scale_log2) {
  constexpr int LD = HD + 8;                    // padded row (elements): conflict-free ldmatrix
  constexpr int CPR = HD / 8;                   // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [BQ][LD]
  __nv_bfloat16* sK = sQ + FP_BQ * LD;                                      // [2][BKV][LD]
  __nv_bfloat16* sV = sK + 2 * FP_BKV * LD;                                 // [2][BKV][LD]
  const int seg = blockIdx.z, qh = blockIdx.y, qt = blockIdx.x;
  const int n = seg_nrows[seg];
  const int q0 = qt * FP_BQ;
  if (q0 >= n) return;
  const int row0 = seg_row0[seg], pos0 = seg_pos0[seg], slot = seg_slot[seg];
  const int kvh = qh / (nq / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int* bt = block_table + (size_t)slot * max_blocks;
  const int q_last = min(n, q0 + FP_BQ) - 1;
  const int kv_end = pos0 + q_last + 1;                     // keys [0, kv_end) can be visible to this tile
  const int ntiles = (kv_end + FP_BKV - 1) / FP_BKV;

  // Q tile -> smem
  for (int c = tid; c < FP_BQ * CPR; c += blockDim.x) {
    int r = c / CPR, cc = c % CPR;
    bool ok = q0 + r < n;
    const __nv_bfloat16* src = q + ((size_t)(row0 + (ok ? q0 + r : 0)) * nq + qh) * HD + cc * 8;
    cp_async16(sQ + r * LD + cc * 8, src, ok);
  }
  auto load_kv = [&](int tile, int stage) {
    const int t0 = tile * FP_BKV;
    for (int c = tid; c < FP_BKV * CPR; c += blockDim.x) {
      int r = c / CPR, cc = c % CPR;
      int t = t0 + r;
      bool ok = t < kv_end;
      size_t off = 0;
      if (ok) {
        int blk = bt[t / kv_block];
        off = (((size_t)blk * kv_block + (t % kv_block)) * nkv + kvh) * HD + cc * 8;
      }
      cp_async16(sK + (stage * FP_BKV + r) * LD + cc * 8, k_cache + off, ok);
      cp_async16(sV + (stage * FP_BKV + r) * LD + cc * 8, v_cache + off, ok);
    }
  };
  load_kv(0, 0);
  cp_async_commit();

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int r_lo = warp * 16 + lane / 4;                   // this thread's two query rows within the tile
  const int qpos_lo = pos0 + q0 + r_lo, qpos_hi = qpos_lo + 8;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < ntiles) { load_kv(tile + 1, stage ^ 1); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const __nv_bfloat16* K = sK + stage * FP_BKV * LD;
    const __nv_bfloat16* V = sV + stage * FP_BKV * LD;
    // S = Q K^T for 16 rows x 32 keys
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < 2; ++np) {                     // two n-tiles (16 keys) per ldmatrix.x4
        uint32_t b[4];
        ldsm_x4(b, K + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[np * 2], a, b[0], b[1]);
        mma_bf16(s[np * 2 + 1], a, b[2], b[3]);
      }
    }
    // scale, causal mask, online softmax
    const int kbase = tile * FP_BKV + (lane & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int kpos = kbase + nt * 8 + (e & 1);
        int qpos = (e < 2) ? qpos_lo : qpos_hi;
        float v = s[nt][e] * scale_log2;
        if (kpos > qpos || kpos >= kv_end) v = -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float sc[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      float mn = fmaxf(mrow[h], mx[h]);
      sc[h] = (mn == -INFINITY) ? 1.f : exp2f(mrow[h] - mn);
      mrow[h] = mn;
    }
    float ls[2] = {0.f, 0.f};
    uint32_t pa[2][4];                                      // P as A fragments: two k-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float p0 = (mrow[0] == -INFINITY) ? 0.f : exp2f(s[nt][0] - mrow[0]);
      float p1 = (mrow[0] == -INFINITY) ? 0.f : exp2f(s[nt][1] - mrow[0]);
      float p2 = (mrow[1] == -INFINITY) ? 0.f : exp2f(s[nt][2] - mrow[1]);
      float p3 = (mrow[1] == -INFINITY) ? 0.f : exp2f(s[nt][3] - mrow[1]);
      ls[0] += p0 + p1; ls[1] += p2 + p3;
      // n-tile nt covers keys nt*8..+8: k-step nt/2, low (nt even) or high (nt odd) half of its 16 keys
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf2(p0, p1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf2(p2, p3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) lrow[h] = lrow[h] * sc[h] + ls[h];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] *= sc[0]; o[i][1] *= sc[0]; o[i][2] *= sc[1]; o[i][3] *= sc[1]; }
    // O += P V
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int np = 0; np < HD / 16; ++np) {
        uint32_t b[4];
        ldsm_x4_t(b, V + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + np * 16 + (lane >> 4) * 8);
        mma_bf16(o[np * 2], pa[ks], b[0], b[1]);
        mma_bf16(o[np * 2 + 1], pa[ks], b[2], b[3]);
      }
    }
    __syncthreads();                                        // the stage is free for the load after next
  }
  // epilogue: normalise, gate, store
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 1);
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = q0 + r_lo + h * 8;
    if (r >= n) continue;
    const float inv = lrow[h] > 0.f ? 1.f / lrow[h] : 0.f;
    const size_t grow = (size_t)(row0 + r);
    const __nv_bfloat16* gate = proj + grow * proj_stride + (size_t)qh * 2 * HD + HD;
    __nv_bfloat16* op = out + (grow * nq + qh) * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      int d = i * 8 + (lane & 3) * 2;
      float v0 = o[i][h * 2] * inv, v1 = o[i][h * 2 + 1] * inv;
      if (gated) {
        uint32_t g = *reinterpret_cast<const uint32_t*>(gate + d);
        v0 *= sigmoidf_(bf_lo(g)); v1 *= sigmoidf_(bf_hi(g));
      }
      *reinterpret_cast<uint32_t*>(op + d) = pack_bf2(v0, v1);
    }
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_attn_prefill(void* out, const void* q, const void* k_cache, const void* v_cache, const void* proj,
                               long proj_stride, const int* seg_slot, const int* seg_row0, const int* seg_nrows,
                               const int* seg_pos0, const int* block_table, int max_blocks, int kv_block, int nseg,
                               int max_rows, int nq, int nkv, int hd, int gated, cudaStream_t s) {
  if (nseg <= 0 || max_rows <= 0) return 0;
  if (nq % nkv) return -1;
  dim3 grid((max_rows + FP_BQ - 1) / FP_BQ, nq, nseg);
  float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
#define FB_FP(HDV)                                                                                               \
  {                                                                                                              \
    size_t smem = (size_t)(FP_BQ + 4 * FP_BKV) * (HDV + 8) * 2;                                                  \
    auto kern = attn_prefill_kernel<HDV>;                                                                        \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    if (e != cudaSuccess) return (int)e;                                                                         \
    kern<<<grid, FP_WARPS * 32, smem, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)q,                         \
        (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (const __nv_bfloat16*)proj, proj_stride,   \
        seg_slot, seg_row0, seg_nrows, seg_pos0, block_table, max_blocks, kv_block, nq, nkv, gated, scale_log2); \
  }
  if (hd == 256) FB_FP(256) else if (hd == 128) FB_FP(128) else if (hd == 64) FB_FP(64) else return -2;
#undef FB_FP
  return (int)cudaGetLastError();
}
