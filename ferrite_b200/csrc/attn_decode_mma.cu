// Decode / verify / tree attention on tensor cores (mma.sync m16n8k16), split over the keys.
//
// The SIMT decode kernel (`attn.cu`) walks the keys of one row at a time: every q head of the group multiplies every key
// in fp32 FMAs with a shuffle reduction per key, and the rows of a verify segment each read the slot's K/V again. It
// tops out near 0.9 TB/s. Here the M dimension of the MMA is (row of the segment, q head of the GQA group): up to
// 64 / G rows of one segment share one pass over the K/V tiles of a kv head, QK^T and PV run on the tensor cores, and
// the K/V stream through shared memory with a two-stage cp.async pipeline. grid = (segment x row group, kv head,
// key split); a CTA writes the unnormalised partial (o, m, l) of its split in the layout `attn_combine_kernel` merges
// (fixed split order, sigmoid gate), so results do not depend on how many CTAs ran.
//
// Visibility of key t for a row: t < kvlen[row], and, with a verify tree, t < base[row] or bit (t - base[row]) of the
// row's ancestor mask. Counterpart of the reference's `fe_attn_vk` (`kernels/k-core/src/attn.rs:331`: decode / verify /
// tree attention on mma.sync with 16-key tiles and ancestor masks) and `fe_attn_combine` (`:99`).
#include <cuda_fp8.h>

#include "api.h"
#include "common.cuh"

namespace fb {

constexpr int DM_BM = 64, DM_BKV = 32, DM_WARPS = 4;

__device__ __forceinline__ void dm_cp_async16(void* smem, const void* gmem, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void dm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void dm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void dm_ldsm(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void dm_ldsm_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void dm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void dm_cp_async8(void* smem, const void* gmem, bool valid) {
  int sz = valid ? 8 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(sz) : "memory");
}
// 16 e4m3 codes -> 16 bf16 (exact: e4m3 values are representable in bf16)
__device__ __forceinline__ void dm_e4m3x16_to_bf16(const uint4& c, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {c.x, c.y, c.z, c.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w[i] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      o[i * 2 + h] = pack_bf2(f.x, f.y);
    }
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// KV8: e4m3 cache (codes [..][HD] bytes, scales [token * nkv + head][2] fp32 for K and V). The byte tiles stream through
// a two-stage cp.async ring and are expanded to bf16 tiles in shared memory before the MMAs; the per-key scales are
// applied to the scores (K) and to P (V) instead of to every element.
template <int HD, bool KV8>
__global__ void __launch_bounds__(DM_WARPS * 32)
attn_decode_mma_kernel(float* __restrict__ o_part, float* __restrict__ ml_part, const __nv_bfloat16* __restrict__ q,
                       const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                       const float* __restrict__ kv_scale, const int* __restrict__ seg_slot, const int* __restrict__ seg_row0,
                       const int* __restrict__ seg_nrows, const int* __restrict__ row_kvlen,
                       const int* __restrict__ row_base, const unsigned long long* __restrict__ row_mask,
                       const int* __restrict__ block_table, int max_blocks, int kv_block, int nq, int nkv, int nsplit,
                       int groups_per_seg, float scale_log2) {
  constexpr int LD = HD + 8;                    // padded row (elements): conflict-free ldmatrix
  constexpr int CPR = HD / 8;                   // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char dm_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dm_smem);           // [BM][LD]
  constexpr int NST = KV8 ? 1 : 2;              // bf16 tile buffers (the e4m3 form double-buffers the byte tiles instead)
  __nv_bfloat16* sK = sQ + DM_BM * LD;                                      // [NST][BKV][LD]
  __nv_bfloat16* sV = sK + NST * DM_BKV * LD;                               // [NST][BKV][LD]
  unsigned char* rK = reinterpret_cast<unsigned char*>(sV + NST * DM_BKV * LD);   // KV8: [2][BKV][HD] codes
  unsigned char* rV = rK + 2 * DM_BKV * HD;
  float* ssc = reinterpret_cast<float*>(rV + 2 * DM_BKV * HD);              // KV8: [2][BKV][2] scales (K, V)
  // No early launch of the dependent grid here: measured inside the decode graph, the dependents' CTAs (which only
  // wait) took the shared memory this kernel's 101 KB CTAs needed and a 27B decode step slowed from 8.9 to 10.8 ms.
  pdl_wait();
  const int G = nq / nkv, RG = DM_BM / G;       // q heads per kv head, rows of a segment per CTA
  const int seg = blockIdx.x / groups_per_seg, gi = blockIdx.x % groups_per_seg;
  const int kvh = blockIdx.y, split = blockIdx.z;
  const int n = seg_nrows[seg];
  const int r_first = gi * RG;
  if (r_first >= n) return;
  const int rows_here = min(RG, n - r_first);
  const int valid_m = rows_here * G;            // M rows in use: m = local row * G + head of the group
  const int row0 = seg_row0[seg] + r_first, slot = seg_slot[seg];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int* bt = block_table + (size_t)slot * max_blocks;
  int kv_end = 0;
  for (int r = 0; r < rows_here; ++r) kv_end = max(kv_end, row_kvlen[row0 + r]);
  int per = (kv_end + nsplit - 1) / nsplit;
  per = (per + DM_BKV - 1) / DM_BKV * DM_BKV;
  const int lo = split * per, hi = min(kv_end, lo + per);

  // this thread's two M rows
  const int m_lo = warp * 16 + lane / 4, m_hi = m_lo + 8;
  int kvl[2] = {0, 0}, base[2] = {0, 0};
  unsigned long long msk[2] = {0ull, 0ull};
  size_t pidx[2] = {0, 0};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int m = h ? m_hi : m_lo;
    if (m < valid_m) {
      const int grow = row0 + m / G, qh = kvh * G + m % G;
      kvl[h] = row_kvlen[grow];
      base[h] = row_base ? row_base[grow] : kvl[h];
      msk[h] = row_mask ? row_mask[grow] : 0ull;
      pidx[h] = ((size_t)grow * nq + qh) * nsplit + split;
    }
  }
  if (lo >= hi) {                                // an empty split: nothing visible, the merge skips it
#pragma unroll
    for (int h = 0; h < 2; ++h)
      if ((h ? m_hi : m_lo) < valid_m && (lane & 3) == 0) { ml_part[pidx[h] * 2] = -INFINITY; ml_part[pidx[h] * 2 + 1] = 0.f; }
    return;
  }

  // Q rows -> smem (rows past valid_m are zero)
  for (int c = tid; c < DM_BM * CPR; c += blockDim.x) {
    const int m = c / CPR, cc = c % CPR;
    const bool ok = m < valid_m;
    const __nv_bfloat16* src = q + ((size_t)(row0 + (ok ? m / G : 0)) * nq + kvh * G + (ok ? m % G : 0)) * HD + cc * 8;
    dm_cp_async16(sQ + m * LD + cc * 8, src, ok);
  }
  auto load_kv = [&](int t0, int stage) {
    if (KV8) {
      const unsigned char* k8 = reinterpret_cast<const unsigned char*>(k_cache);
      const unsigned char* v8 = reinterpret_cast<const unsigned char*>(v_cache);
      constexpr int CPR8 = HD / 16;
      for (int c = tid; c < DM_BKV * CPR8; c += blockDim.x) {
        const int r = c / CPR8, cc = c % CPR8;
        const int t = t0 + r;
        const bool ok = t < hi;
        size_t tok = 0;
        if (ok) tok = ((size_t)bt[t / kv_block] * kv_block + (t % kv_block)) * nkv + kvh;
        dm_cp_async16(rK + ((size_t)stage * DM_BKV + r) * HD + cc * 16, k8 + tok * HD + cc * 16, ok);
        dm_cp_async16(rV + ((size_t)stage * DM_BKV + r) * HD + cc * 16, v8 + tok * HD + cc * 16, ok);
        if (cc == 0) dm_cp_async8(ssc + ((size_t)stage * DM_BKV + r) * 2, kv_scale + tok * 2, ok);
      }
      return;
    }
    for (int c = tid; c < DM_BKV * CPR; c += blockDim.x) {
      const int r = c / CPR, cc = c % CPR;
      const int t = t0 + r;
      const bool ok = t < hi;
      size_t off = 0;
      if (ok) {
        const int blk = bt[t / kv_block];
        off = (((size_t)blk * kv_block + (t % kv_block)) * nkv + kvh) * HD + cc * 8;
      }
      dm_cp_async16(sK + (stage * DM_BKV + r) * LD + cc * 8, k_cache + off, ok);
      dm_cp_async16(sV + (stage * DM_BKV + r) * LD + cc * 8, v_cache + off, ok);
    }
  };
  load_kv(lo, 0);
  dm_commit();

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const bool warp_on = warp * 16 < valid_m;      // warps whose 16 M rows are all unused only help with the loads
  const int ntiles = (hi - lo + DM_BKV - 1) / DM_BKV;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < ntiles) { load_kv(lo + (tile + 1) * DM_BKV, stage ^ 1); dm_commit(); dm_wait<1>(); }
    else dm_wait<0>();
    __syncthreads();
    if (KV8) {
      // expand this tile's codes to bf16 (the MMAs of the previous tile finished before the barrier above)
      constexpr int CPR8 = HD / 16;
      for (int c = tid; c < DM_BKV * CPR8; c += blockDim.x) {
        const int r = c / CPR8, cc = c % CPR8;
        uint4 lo4, hi4;
        dm_e4m3x16_to_bf16(*reinterpret_cast<const uint4*>(rK + ((size_t)stage * DM_BKV + r) * HD + cc * 16), lo4, hi4);
        *reinterpret_cast<uint4*>(sK + r * LD + cc * 16) = lo4;
        *reinterpret_cast<uint4*>(sK + r * LD + cc * 16 + 8) = hi4;
        dm_e4m3x16_to_bf16(*reinterpret_cast<const uint4*>(rV + ((size_t)stage * DM_BKV + r) * HD + cc * 16), lo4, hi4);
        *reinterpret_cast<uint4*>(sV + r * LD + cc * 16) = lo4;
        *reinterpret_cast<uint4*>(sV + r * LD + cc * 16 + 8) = hi4;
      }
      __syncthreads();
    }
    if (warp_on) {
      const __nv_bfloat16* K = sK + (KV8 ? 0 : stage) * DM_BKV * LD;
      const __nv_bfloat16* V = sV + (KV8 ? 0 : stage) * DM_BKV * LD;
      const float* tsc = ssc + (size_t)stage * DM_BKV * 2;   // KV8: (K scale, V scale) of the tile's keys
      float s[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t a[4];
        dm_ldsm(a, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b[4];
          dm_ldsm(b, K + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
          dm_mma(s[np * 2], a, b[0], b[1]);
          dm_mma(s[np * 2 + 1], a, b[2], b[3]);
        }
      }
      const int kbase = lo + tile * DM_BKV + (lane & 3) * 2;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int t = kbase + nt * 8 + (e & 1), h = e >> 1;
          bool vis = t < kvl[h] && t < hi;
          if (vis && t >= base[h]) vis = ((msk[h] >> (t - base[h])) & 1ull) != 0ull;
          float sv = s[nt][e];
          if (KV8) sv *= tsc[((lane & 3) * 2 + nt * 8 + (e & 1)) * 2];
          const float v = vis ? sv * scale_log2 : -INFINITY;
          s[nt][e] = v;
          mx[h] = fmaxf(mx[h], v);
        }
      }
      float sc[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float mn = fmaxf(mrow[h], mx[h]);
        sc[h] = (mn == -INFINITY) ? 1.f : exp2f(mrow[h] - mn);
        mrow[h] = mn;
      }
      float ls[2] = {0.f, 0.f};
      uint32_t pa[2][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float p0 = (mrow[0] == -INFINITY) ? 0.f : exp2f(s[nt][0] - mrow[0]);
        const float p1 = (mrow[0] == -INFINITY) ? 0.f : exp2f(s[nt][1] - mrow[0]);
        const float p2 = (mrow[1] == -INFINITY) ? 0.f : exp2f(s[nt][2] - mrow[1]);
        const float p3 = (mrow[1] == -INFINITY) ? 0.f : exp2f(s[nt][3] - mrow[1]);
        ls[0] += p0 + p1; ls[1] += p2 + p3;
        float v0 = 1.f, v1 = 1.f;                           // KV8: the V scale of the two keys rides on P
        if (KV8) { v0 = tsc[((lane & 3) * 2 + nt * 8) * 2 + 1]; v1 = tsc[((lane & 3) * 2 + nt * 8 + 1) * 2 + 1]; }
        pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf2(p0 * v0, p1 * v1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf2(p2 * v0, p3 * v1);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) lrow[h] = lrow[h] * sc[h] + ls[h];
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) { o[i][0] *= sc[0]; o[i][1] *= sc[0]; o[i][2] *= sc[1]; o[i][3] *= sc[1]; }
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int np = 0; np < HD / 16; ++np) {
          uint32_t b[4];
          dm_ldsm_t(b, V + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + np * 16 + (lane >> 4) * 8);
          dm_mma(o[np * 2], pa[ks], b[0], b[1]);
          dm_mma(o[np * 2 + 1], pa[ks], b[2], b[3]);
        }
      }
    }
    __syncthreads();                                        // the stage is free for the load after next
  }
  if (!warp_on) return;
  // this split's partial: unnormalised o relative to m, and (m, l)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 1);
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if ((h ? m_hi : m_lo) >= valid_m) continue;
    float* op = o_part + pidx[h] * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(op + d) = make_float2(o[i][h * 2], o[i][h * 2 + 1]);
    }
    if ((lane & 3) == 0) { ml_part[pidx[h] * 2] = mrow[h]; ml_part[pidx[h] * 2 + 1] = lrow[h]; }
  }
}

}  // namespace fb

using namespace fb;

// Same outputs as fb_attn_decode (bf16 cache) / fb_attn_decode_kv8 (kv_scale != null: e4m3 cache); rows are addressed
// through their segments (rows of one segment share a slot). Returns -20 for shapes this kernel does not take (the
// caller uses the SIMT kernel).
extern "C" int fb_attn_decode_mma(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache,
                                  const void* v_cache, const float* kv_scale, const void* proj, long proj_stride,
                                  const int* seg_slot, const int* seg_row0, const int* seg_nrows, const int* row_kvlen,
                                  const int* row_base, const unsigned long long* row_mask, const int* block_table,
                                  int max_blocks, int kv_block, int nseg, int max_rows, int rows, int nq, int nkv, int hd,
                                  int nsplit, int gated, cudaStream_t s) {
  if (nseg <= 0 || rows <= 0) return 0;
  if (nq % nkv) return -1;
  const int G = nq / nkv;
  if (G > DM_BM || (hd != 64 && hd != 128 && hd != 256)) return -20;
  const int RG = DM_BM / G;
  const int gps = (max_rows + RG - 1) / RG;
  dim3 grid(nseg * gps, nkv, nsplit);
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
#define FB_DM(HDV, K8)                                                                                              \
  {                                                                                                                 \
    const size_t smem = K8 ? (size_t)(DM_BM + 2 * DM_BKV) * (HDV + 8) * 2 + (size_t)4 * DM_BKV * HDV + 4 * DM_BKV * 4 * 2 \
                           : (size_t)(DM_BM + 4 * DM_BKV) * (HDV + 8) * 2;                                          \
    auto kern = attn_decode_mma_kernel<HDV, K8>;                                                                    \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
    if (e != cudaSuccess) return (int)e;                                                                            \
    launch_pdl(kern, grid, dim3(DM_WARPS * 32), smem, s, o_part, ml_part, (const __nv_bfloat16*)q,                   \
               (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, kv_scale, seg_slot, seg_row0, seg_nrows, \
               row_kvlen, row_base, row_mask, block_table, max_blocks, kv_block, nq, nkv, nsplit, gps, scale_log2);  \
  }
  if (kv_scale) {
    if (hd == 256) FB_DM(256, true) else if (hd == 128) FB_DM(128, true) else FB_DM(64, true)
  } else {
    if (hd == 256) FB_DM(256, false) else if (hd == 128) FB_DM(128, false) else FB_DM(64, false)
  }
#undef FB_DM
  int rc = (int)cudaGetLastError();
  if (rc) return rc;
  return fb_attn_combine(out, o_part, ml_part, proj, proj_stride, rows, nq, hd, nsplit, gated, s);
}
