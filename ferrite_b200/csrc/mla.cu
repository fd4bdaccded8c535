// Multi-head latent attention (absorbed form) over a paged latent cache.
//
// Per token the cache holds one row [kv_lora | rope_dim] (512 + 64 bf16): the RMS-normalised latent and the rotated
// shared key part. With the key up-projection folded into the query (q' = q_nope W_uk per head) every head attends the
// same cache rows: score = q'.latent + q_rope.k_rope, output = P latent (kv_lora wide), up-projected by W_uv afterwards.
//
//   mla_prep      per token: RMSNorm(1+w) of the latent and rotate-half RoPE of the key part into the paged cache;
//                 RoPE of every head's query rope part into the tail of its absorbed query row
//   mla_attn      one CTA per (token row, head, key split): warps stride over the keys, online softmax, value = latent;
//                 rows of a prompt attend causally through their own kvlen
//   mla_combine   merge of the splits in split order
// SIMT fp32 throughout: this is the functional path of the MLA model family (prefill cost is quadratic per row here).
// Counterparts in the reference: `ds_rope`, `ds_kv_window`, `ds_attn`, `ds_attn16`, `ds_attn_mq(_fin)`
// (`kernels/k-ds/src`), f32 oracle `crates/fe-dsc/src/refmodel.rs`.
#include "api_ext.h"
#include "common.cuh"

namespace fb {

constexpr int MLA_WARPS = 4;

// grid = rows, 256 threads. kva: [rows][L + R]; q: [rows][nq][dn + R]; qabs: [rows][nq][L + R] (rope tail written here)
__global__ void __launch_bounds__(256) mla_prep_kernel(__nv_bfloat16* __restrict__ cache, __nv_bfloat16* __restrict__ qabs,
                                                       const __nv_bfloat16* __restrict__ kva, long kva_stride,
                                                       const __nv_bfloat16* __restrict__ q, long q_stride,
                                                       const __nv_bfloat16* __restrict__ norm_w,
                                                       const float* __restrict__ inv_freq, const int* __restrict__ row_slot,
                                                       const int* __restrict__ row_pos, const int* __restrict__ block_table,
                                                       int max_blocks, int kv_block, int nq, int dn, int L, int R,
                                                       float eps, int* status) {
  __shared__ float red[32];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int slot = row_slot[row], pos = row_pos[row];
  const int blk = block_table[(size_t)slot * max_blocks + pos / kv_block];
  if (blk < 0) { if (tid == 0) set_status(status, ST_BOUNDS); return; }
  __nv_bfloat16* crow = cache + ((size_t)blk * kv_block + pos % kv_block) * (L + R);
  const __nv_bfloat16* kr = kva + (size_t)row * kva_stride;
  float ss = 0.f;
  for (int i = tid; i < L; i += blockDim.x) { const float v = bf2f(kr[i]); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)L + eps);
  for (int i = tid; i < L; i += blockDim.x) crow[i] = f2bf(bf2f(kr[i]) * r * (1.f + bf2f(norm_w[i])));
  const int half = R / 2;
  // key rope part, then every head's query rope part: pair (i, i + R/2)
  for (int idx = tid; idx < (nq + 1) * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    if (h == nq) {
      const float a = bf2f(kr[L + i]), b = bf2f(kr[L + half + i]);
      crow[L + i] = f2bf(a * c - b * s);
      crow[L + half + i] = f2bf(b * c + a * s);
    } else {
      const __nv_bfloat16* qh = q + (size_t)row * q_stride + (size_t)h * (dn + R) + dn;
      __nv_bfloat16* oh = qabs + ((size_t)row * nq + h) * (L + R) + L;
      const float a = bf2f(qh[i]), b = bf2f(qh[half + i]);
      oh[i] = f2bf(a * c - b * s);
      oh[half + i] = f2bf(b * c + a * s);
    }
  }
}

// grid (rows, nq, nsplit); D = L + R must be a multiple of 64 with D / 64 <= 9, L a multiple of 64
template <int DJ, int LJ>
__global__ void __launch_bounds__(MLA_WARPS * 32) mla_attn_kernel(float* __restrict__ o_part, float* __restrict__ ml_part,
                                                                  const __nv_bfloat16* __restrict__ qabs,
                                                                  const __nv_bfloat16* __restrict__ cache,
                                                                  const int* __restrict__ row_slot,
                                                                  const int* __restrict__ row_kvlen,
                                                                  const int* __restrict__ block_table, int max_blocks,
                                                                  int kv_block, int nq, int nsplit, float scale_log2) {
  constexpr int D = DJ * 64, L = LJ * 64;
  __shared__ float so[MLA_WARPS][L];
  __shared__ float sml[MLA_WARPS][2];
  const int row = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvlen = row_kvlen[row], slot = row_slot[row];
  int per = (kvlen + nsplit - 1) / nsplit;
  per = (per + 31) / 32 * 32;
  const int lo = split * per, hi = min(kvlen, lo + per);
  // lane owns dims {64 j + 2 lane, 64 j + 2 lane + 1}
  float qf[DJ][2];
  const __nv_bfloat16* qr = qabs + ((size_t)row * nq + h) * D;
#pragma unroll
  for (int j = 0; j < DJ; ++j) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(qr + 64 * j + 2 * lane);
    qf[j][0] = bf_lo(u) * scale_log2; qf[j][1] = bf_hi(u) * scale_log2;
  }
  float m = -INFINITY, l = 0.f, o[LJ][2];
#pragma unroll
  for (int j = 0; j < LJ; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; }
  for (int t = lo + warp; t < hi; t += MLA_WARPS) {
    const int blk = block_table[(size_t)slot * max_blocks + t / kv_block];
    const __nv_bfloat16* kr = cache + ((size_t)blk * kv_block + t % kv_block) * D;
    uint32_t ku[DJ];
#pragma unroll
    for (int j = 0; j < DJ; ++j) ku[j] = *reinterpret_cast<const uint32_t*>(kr + 64 * j + 2 * lane);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < DJ; ++j) s = fmaf(qf[j][0], bf_lo(ku[j]), fmaf(qf[j][1], bf_hi(ku[j]), s));
    s = warp_sum(s);
    const float mn = fmaxf(m, s);
    const float a = exp2f(m - mn), p = exp2f(s - mn);
    l = l * a + p;
#pragma unroll
    for (int j = 0; j < LJ; ++j) {
      o[j][0] = fmaf(p, bf_lo(ku[j]), o[j][0] * a);
      o[j][1] = fmaf(p, bf_hi(ku[j]), o[j][1] * a);
    }
    m = mn;
  }
#pragma unroll
  for (int j = 0; j < LJ; ++j) { so[warp][64 * j + 2 * lane] = o[j][0]; so[warp][64 * j + 2 * lane + 1] = o[j][1]; }
  if (lane == 0) { sml[warp][0] = m; sml[warp][1] = l; }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < MLA_WARPS; ++w) M = fmaxf(M, sml[w][0]);
  const size_t pidx = ((size_t)row * nq + h) * nsplit + split;
  for (int d = threadIdx.x; d < L; d += blockDim.x) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < MLA_WARPS; ++w) {
      const float mw = sml[w][0];
      acc += so[w][d] * (mw == -INFINITY ? 0.f : exp2f(mw - M));
    }
    o_part[pidx * L + d] = acc;
  }
  if (threadIdx.x == 0) {
    float Ls = 0.f;
#pragma unroll
    for (int w = 0; w < MLA_WARPS; ++w) {
      const float mw = sml[w][0];
      Ls += sml[w][1] * (mw == -INFINITY ? 0.f : exp2f(mw - M));
    }
    ml_part[pidx * 2] = M;
    ml_part[pidx * 2 + 1] = Ls;
  }
}

// grid (rows, nq); out: bf16 [rows][nq][L]
__global__ void mla_combine_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ o_part,
                                   const float* __restrict__ ml_part, int nq, int nsplit, int L) {
  const int row = blockIdx.x, h = blockIdx.y;
  const size_t pbase = ((size_t)row * nq + h) * nsplit;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ml_part[(pbase + s) * 2]);
  float Ls = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = ml_part[(pbase + s) * 2];
    if (ms != -INFINITY) Ls += ml_part[(pbase + s) * 2 + 1] * exp2f(ms - M);
  }
  const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
  for (int d = threadIdx.x; d < L; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = ml_part[(pbase + s) * 2];
      if (ms != -INFINITY) acc += o_part[(pbase + s) * L + d] * exp2f(ms - M);
    }
    out[((size_t)row * nq + h) * L + d] = f2bf(acc * inv);
  }
}

// ---- prompt rows on the tensor-core flash kernel: the expanded (per-head key / value) form -----------------------------
// The absorbed form above reads 576-wide latent rows per head per key, which is right for a few rows and quadratic SIMT
// work for a prompt. For prompt chunks the context's latent rows are expanded once per layer by one dense GEMM with
// kv_b ([nq (dn + dv)] x L), and packed here into ordinary per-head K / V rows padded to the flash kernel's head width
// HP (64 / 128 / 256): K = [k_nope | k_rope (shared by the heads) | 0], V = [v | 0], Q = [q_nope | q_rope | 0] * s with
// s = sqrt(HP / (dn + R)) so that the kernel's 1 / sqrt(HP) becomes the model's 1 / sqrt(dn + R). Zero padding changes
// neither q . k nor the first dv output columns.
// grid = context rows, 256 threads, 8 elements per thread step.
__global__ void __launch_bounds__(256) mla_expand_kernel(__nv_bfloat16* __restrict__ kp, __nv_bfloat16* __restrict__ vp,
                                                         const __nv_bfloat16* __restrict__ kvx, const __nv_bfloat16* __restrict__ lat,
                                                         int nq, int dn, int dv, int L, int R, int HP) {
  const size_t t = blockIdx.x;
  const int per = HP / 8;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < nq * per; i += blockDim.x) {
    const int h = i / per, c = (i % per) * 8;
    uint4 kv = zero, vv = zero;
    if (c < dn) kv = *reinterpret_cast<const uint4*>(kvx + (t * nq + h) * (dn + dv) + c);
    else if (c < dn + R) kv = *reinterpret_cast<const uint4*>(lat + t * (L + R) + L + (c - dn));
    if (c < dv) vv = *reinterpret_cast<const uint4*>(kvx + (t * nq + h) * (dn + dv) + dn + c);
    *reinterpret_cast<uint4*>(kp + (t * nq + h) * HP + c) = kv;
    *reinterpret_cast<uint4*>(vp + (t * nq + h) * HP + c) = vv;
  }
}

// q [rows][nq][dn + R] (rope part not yet rotated), qabs [rows][nq][L + R] (rotated rope part in its tail).
__global__ void __launch_bounds__(256) mla_qpad_kernel(__nv_bfloat16* __restrict__ qp, const __nv_bfloat16* __restrict__ q,
                                                       long q_stride, const __nv_bfloat16* __restrict__ qabs, int nq, int dn,
                                                       int L, int R, int HP, float s) {
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < nq * HP; i += blockDim.x) {
    const int h = i / HP, c = i % HP;
    float v = 0.f;
    if (c < dn) v = bf2f(q[t * q_stride + (size_t)h * (dn + R) + c]);
    else if (c < dn + R) v = bf2f(qabs[(t * nq + h) * (L + R) + L + (c - dn)]);
    qp[(t * nq + h) * HP + c] = f2bf(v * s);
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_mla_expand(void* kp, void* vp, const void* kvx, const void* lat, long rows, int nq, int dn, int dv, int L,
                             int R, int HP, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (dn % 8 || dv % 8 || R % 8 || L % 8 || HP % 8 || dn + R > HP || dv > HP) return -1;
  mla_expand_kernel<<<(unsigned)rows, 256, 0, s>>>((__nv_bfloat16*)kp, (__nv_bfloat16*)vp, (const __nv_bfloat16*)kvx,
                                                   (const __nv_bfloat16*)lat, nq, dn, dv, L, R, HP);
  return (int)cudaGetLastError();
}

extern "C" int fb_mla_qpad(void* qp, const void* q, long q_stride, const void* qabs, long rows, int nq, int dn, int L, int R,
                           int HP, float scale, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (dn + R > HP) return -1;
  mla_qpad_kernel<<<(unsigned)rows, 256, 0, s>>>((__nv_bfloat16*)qp, (const __nv_bfloat16*)q, q_stride,
                                                 (const __nv_bfloat16*)qabs, nq, dn, L, R, HP, scale);
  return (int)cudaGetLastError();
}


extern "C" int fb_mla_prep(void* cache, void* qabs, const void* kva, long kva_stride, const void* q, long q_stride,
                           const void* norm_w, const float* inv_freq, const int* row_slot, const int* row_pos,
                           const int* block_table, int max_blocks, int kv_block, int rows, int nq, int dn, int L, int R,
                           float eps, int* status, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (R % 2) return -1;
  mla_prep_kernel<<<rows, 256, 0, s>>>((__nv_bfloat16*)cache, (__nv_bfloat16*)qabs, (const __nv_bfloat16*)kva, kva_stride,
                                       (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)norm_w, inv_freq, row_slot,
                                       row_pos, block_table, max_blocks, kv_block, nq, dn, L, R, eps, status);
  return (int)cudaGetLastError();
}

// o_part: rows * nq * nsplit * L floats, ml_part: rows * nq * nsplit * 2 floats
extern "C" int fb_mla_attn(void* out, float* o_part, float* ml_part, const void* qabs, const void* cache,
                           const int* row_slot, const int* row_kvlen, const int* block_table, int max_blocks, int kv_block,
                           int rows, int nq, int L, int R, int nsplit, float scale, cudaStream_t s) {
  if (rows <= 0) return 0;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(rows, nq, nsplit);
  if (L == 512 && R == 64)
    mla_attn_kernel<9, 8><<<grid, MLA_WARPS * 32, 0, s>>>(o_part, ml_part, (const __nv_bfloat16*)qabs,
                                                          (const __nv_bfloat16*)cache, row_slot, row_kvlen, block_table,
                                                          max_blocks, kv_block, nq, nsplit, scale_log2);
  else if (L == 64 && R == 64)
    mla_attn_kernel<2, 1><<<grid, MLA_WARPS * 32, 0, s>>>(o_part, ml_part, (const __nv_bfloat16*)qabs,
                                                          (const __nv_bfloat16*)cache, row_slot, row_kvlen, block_table,
                                                          max_blocks, kv_block, nq, nsplit, scale_log2);
  else if (L == 128 && R == 64)
    mla_attn_kernel<3, 2><<<grid, MLA_WARPS * 32, 0, s>>>(o_part, ml_part, (const __nv_bfloat16*)qabs,
                                                          (const __nv_bfloat16*)cache, row_slot, row_kvlen, block_table,
                                                          max_blocks, kv_block, nq, nsplit, scale_log2);
  else return -2;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  mla_combine_kernel<<<dim3(rows, nq), 128, 0, s>>>((__nv_bfloat16*)out, o_part, ml_part, nq, nsplit, L);
  return (int)cudaGetLastError();
}
