// Sparse-attention selection: latent compressor, indexer scores, exact top-k, candidate-block masks and the block
// table of a selected-block (QSA) attention.
//
//   comp_stash / comp_close   a slot keeps the last `ring_len` rows of the compressor linears' outputs (value kvc and
//                             score sc, fp32); a row that closes a group of `ratio` tokens emits the group's latent
//                             sum_t kvc_t * softmax_t(sc_t) per channel (ratio 1: the value itself), other rows zeros
//   index_score               score[r][e] = sum_h w[r][h] * relu(q[r][h] . key[slot(r)][e]) for e < len(r), -inf
//                             elsewhere (and where a candidate mask drops the entry's block): mma.sync m16n8k16 with
//                             entries as M, heads as N, the key width (permuted for 16-byte loads) as K
//   topk_select               exact top-k of a score row by 4 x 8-bit radix selection on order-preserving keys; ties to
//                             the lower index; -inf entries never count; output ascending indices, -1 padded
//   block_max / sel_to_mask   candidate pool of a later layer: block maxima (the block of the last valid entry always
//                             kept), top blocks -> byte mask
//   qsa_pool                  pooled key of a finished block of kp cells: rope(rmsnorm(mean) * w) at its first position
//   qsa_table                 per-row block table of the selected blocks (+ the open tail block) in page ids, so the
//                             paged decode attention kernel runs the sparse attention unchanged: selection is a table
//                             rewrite, not a second attention kernel
//
// Counterparts of the reference's `ds_comp_stash`, `ds_comp_pair`, `ds_idx_score(_tc)`, `ds_topk(_part/_fin)`,
// `ds_block_max`, `ds_sel_to_mask` (`kernels/k-ds/src/index.rs:11-399`) and `fx_idx_pool`, `fx_idx_score`, `fx_topk`
// (`kernels/k-fnext/src/fast.rs:157-247`; there the selection is a cell list read by a second attention kernel).
#include "api_ext.h"
#include "common.cuh"

namespace fb {

// ---- compressor -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) comp_stash_kernel(float* __restrict__ tail, const float* __restrict__ kvc,
                                                         const float* __restrict__ sc, const int* __restrict__ row_slot,
                                                         const int* __restrict__ row_pos, int dim, int ring_len) {
  const int r = blockIdx.x;
  float* dst = tail + ((size_t)row_slot[r] * ring_len + (row_pos[r] % ring_len)) * 2 * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    dst[i] = kvc[(size_t)r * dim + i];
    dst[dim + i] = sc ? sc[(size_t)r * dim + i] : 0.f;
  }
}

__global__ void __launch_bounds__(256) comp_close_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ tail,
                                                         const int* __restrict__ row_slot, const int* __restrict__ row_pos,
                                                         int ratio, int dim, int ring_len) {
  const int r = blockIdx.x, pos = row_pos[r];
  const bool closes = (pos + 1) % ratio == 0;
  const float* tb = tail + (size_t)row_slot[r] * ring_len * 2 * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = 0.f;
    if (closes) {
      float m = -INFINITY;
      for (int t = 0; t < ratio; ++t) m = fmaxf(m, tb[(size_t)((pos - t) % ring_len) * 2 * dim + dim + i]);
      float den = 0.f, num = 0.f;
      for (int t = ratio - 1; t >= 0; --t) {          // oldest token first
        const float* row = tb + (size_t)((pos - t) % ring_len) * 2 * dim;
        const float e = ratio == 1 ? 1.f : __expf(row[dim + i] - m);
        den += e;
        num = fmaf(row[i], e, num);
      }
      v = num / den;
    }
    out[(size_t)r * dim + i] = __float2bfloat16(v);
  }
}

// ---- indexer scores ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void idx_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int IDX_MAX_HEADS = 64;

// grid = (ceil(ld / 128), rows), 256 threads: a warp takes 16 entries. q [rows][nh][D] bf16, w [rows][nh] fp32 (null:
// every head weighs `scale`), keys [slots][key_stride] bf16 with entry e at e * D, D a multiple of 32 and <= 128.
//
// A dot product does not care in which order K is walked, so the K dimension is permuted to suit the loads: lane t of a
// row's four lanes reads 16 contiguous bytes (8 values) per pair of k16 steps, words {0, 1} feed the first step's two
// A registers and words {2, 3} the second's; the query fragments are read with the same pattern. All of a warp's key
// loads (two rows x D / 32 uint4 per lane) are in flight before the first MMA.
constexpr int IDX_MAX_D = 128;

__global__ void __launch_bounds__(256) index_score_kernel(float* __restrict__ score, int ld, const __nv_bfloat16* __restrict__ q,
                                                          const float* __restrict__ w, float scale,
                                                          const __nv_bfloat16* __restrict__ keys, long key_stride,
                                                          const int* __restrict__ row_slot, const int* __restrict__ row_len,
                                                          const uint8_t* __restrict__ mask, int mask_ld, int mask_block,
                                                          int nh, int D) {
  const int r = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int e0 = blockIdx.x * 128 + warp * 16;
  if (e0 >= ld) return;                                 // whole warps leave together
  const int len = min(row_len[r], ld);
  const __nv_bfloat16* kb = keys + (size_t)row_slot[r] * key_stride;
  const __nv_bfloat16* qr = q + (size_t)r * nh * D;
  const int ea = e0 + g, eb = e0 + g + 8;
  auto kept = [&](int e) { return e < len && (!mask || mask[(size_t)r * mask_ld + e / mask_block] != 0); };
  const bool ka = kept(ea), kb8 = kept(eb);
  const int ntiles = (nh + 7) / 8, npair = D / 32;      // pairs of k16 steps
  uint4 ra[IDX_MAX_D / 32], rb[IDX_MAX_D / 32];
#pragma unroll
  for (int j = 0; j < IDX_MAX_D / 32; ++j) {
    ra[j] = (ka && j < npair) ? ldg_stream(reinterpret_cast<const uint4*>(kb + (size_t)ea * D) + j * 4 + t) : make_uint4(0, 0, 0, 0);
    rb[j] = (kb8 && j < npair) ? ldg_stream(reinterpret_cast<const uint4*>(kb + (size_t)eb * D) + j * 4 + t) : make_uint4(0, 0, 0, 0);
  }
  float acc[IDX_MAX_HEADS / 8][4];
#pragma unroll
  for (int n = 0; n < IDX_MAX_HEADS / 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
#pragma unroll
  for (int j = 0; j < IDX_MAX_D / 32; ++j) {
    if (j < npair) {
      const uint32_t a0[4] = {ra[j].x, rb[j].x, ra[j].y, rb[j].y};      // first k16 step: (row g, row g + 8) x words {0, 1}
      const uint32_t a1[4] = {ra[j].z, rb[j].z, ra[j].w, rb[j].w};      // second: words {2, 3}
#pragma unroll
      for (int n = 0; n < IDX_MAX_HEADS / 8; ++n) {
        if (n < ntiles) {
          const int h = n * 8 + g;
          uint4 bq = make_uint4(0, 0, 0, 0);
          if (h < nh) bq = __ldg(reinterpret_cast<const uint4*>(qr + (size_t)h * D) + j * 4 + t);
          idx_mma(acc[n], a0, bq.x, bq.y);
          idx_mma(acc[n], a1, bq.z, bq.w);
        }
      }
    }
  }
  // relu, head weights, sum over heads: this thread's two columns per tile, then the four lanes of a row, fixed order
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int n = 0; n < IDX_MAX_HEADS / 8; ++n) {
    if (n < ntiles) {
      const int h0 = n * 8 + 2 * t;
      const float w0 = h0 < nh ? (w ? w[(size_t)r * nh + h0] : scale) : 0.f;
      const float w1 = h0 + 1 < nh ? (w ? w[(size_t)r * nh + h0 + 1] : scale) : 0.f;
      sa += fmaxf(acc[n][0], 0.f) * w0 + fmaxf(acc[n][1], 0.f) * w1;
      sb += fmaxf(acc[n][2], 0.f) * w0 + fmaxf(acc[n][3], 0.f) * w1;
    }
  }
  sa += __shfl_xor_sync(0xffffffffu, sa, 1); sa += __shfl_xor_sync(0xffffffffu, sa, 2);
  sb += __shfl_xor_sync(0xffffffffu, sb, 1); sb += __shfl_xor_sync(0xffffffffu, sb, 2);
  if (t == 0) {
    if (ea < ld) score[(size_t)r * ld + ea] = ka ? sa : -INFINITY;
    if (eb < ld) score[(size_t)r * ld + eb] = kb8 ? sb : -INFINITY;
  }
}

// ---- exact top-k ------------------------------------------------------------------------------------------------
// order-preserving key of a float: larger float -> larger key
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive scan of one int per thread over the block (1024 threads); `total` gets the block sum. scratch >= 33 ints.
__device__ __forceinline__ int block_excl_scan(int v, int* scratch, int& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += u;
  }
  __syncthreads();
  if (lane == 31) scratch[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    int s = lane < nw ? scratch[lane] : 0, si = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, si, o);
      if (lane >= o) si += u;
    }
    scratch[lane] = si - s;                  // exclusive warp offsets
    if (lane == 31) scratch[32] = si;
  }
  __syncthreads();
  total = scratch[32];
  return scratch[wid] + inc - v;
}

constexpr int TOPK_THREADS = 1024;

// grid = rows, 1024 threads. sel [rows][k] int; score rows of stride ld, the first n (row_n[r] when given) entries count.
__global__ void __launch_bounds__(TOPK_THREADS) topk_select_kernel(int* __restrict__ sel, const float* __restrict__ score,
                                                                   int ld, int n_all, const int* __restrict__ row_n, int k) {
  __shared__ int hist[256];
  __shared__ int scan_s[33];
  __shared__ uint32_t prefix_s;
  __shared__ int want_s;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = score + (size_t)r * ld;
  const int n = min(row_n ? row_n[r] : n_all, ld);
  uint32_t prefix = 0, pmask = 0;
  int want = k;                              // entries still to take among those matching the prefix
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += TOPK_THREADS) hist[i] = 0;
    __syncthreads();
    for (int e = tid; e < n; e += TOPK_THREADS) {
      const float f = row[e];
      if (f == -INFINITY) continue;
      const uint32_t key = order_key(f);
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int w = want;
      if (pass == 0) {                       // fewer valid entries than k: take them all
        int valid = 0;
        for (int b = 0; b < 256; ++b) valid += hist[b];
        if (w > valid) w = valid;
      }
      int b = 255, above = 0;
      for (; b > 0; --b) {
        if (above + hist[b] >= w) break;
        above += hist[b];
      }
      prefix_s = prefix | ((uint32_t)b << shift);
      want_s = w - above;                    // to take from bin b (all of the bins above it are taken)
    }
    __syncthreads();
    prefix = prefix_s;
    want = want_s;
    pmask |= 0xffu << shift;
    __syncthreads();
  }
  // `prefix` is the key of the last entry taken; `want` of the entries equal to it are taken, lowest index first
  const uint32_t thr = prefix;
  int out_base = 0, eq_base = 0;
  for (int c0 = 0; c0 < n; c0 += TOPK_THREADS) {
    const int e = c0 + tid;
    bool gt = false, eq = false;
    if (e < n) {
      const float f = row[e];
      if (f != -INFINITY) {
        const uint32_t key = order_key(f);
        gt = key > thr;
        eq = key == thr;
      }
    }
    int eq_total, take_total;
    const int eq_rank = block_excl_scan(eq ? 1 : 0, scan_s, eq_total);
    const bool take = gt || (eq && eq_base + eq_rank < want);
    const int pos = block_excl_scan(take ? 1 : 0, scan_s, take_total);
    if (take && out_base + pos < k) sel[(size_t)r * k + out_base + pos] = e;
    out_base += take_total;
    eq_base += eq_total;
  }
  for (int i = out_base + tid; i < k; i += TOPK_THREADS) sel[(size_t)r * k + i] = -1;
}

// ---- candidate blocks -------------------------------------------------------------------------------------------
// bmax[r][b] = max of the row's valid scores in block b (bsize entries); the block of the last valid entry reads +inf
// (always kept); blocks past it -inf. grid = (ceil(mask_ld / 8), rows), 256 threads: a warp per block.
__global__ void __launch_bounds__(256) block_max_kernel(float* __restrict__ bmax, int mask_ld, const float* __restrict__ score,
                                                        int ld, const int* __restrict__ row_n, int bsize) {
  const int r = blockIdx.y, b = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (b >= mask_ld) return;
  const int n = min(row_n[r], ld);
  float m = -INFINITY;
  for (int e = b * bsize + lane; e < min(n, (b + 1) * bsize); e += 32) m = fmaxf(m, score[(size_t)r * ld + e]);
  m = warp_max(m);
  if (n > 0 && b == (n - 1) / bsize) m = INFINITY;
  if (lane == 0) bmax[(size_t)r * mask_ld + b] = m;
}

__global__ void __launch_bounds__(256) sel_to_mask_kernel(uint8_t* __restrict__ mask, int mask_ld, const int* __restrict__ sel,
                                                          int k) {
  const int r = blockIdx.x;
  for (int b = threadIdx.x; b < mask_ld; b += blockDim.x) mask[(size_t)r * mask_ld + b] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const int b = sel[(size_t)r * k + i];
    if (b >= 0 && b < mask_ld) mask[(size_t)r * mask_ld + b] = 1;
  }
}

// ---- selected-block attention: pooled keys and the per-row block table ---------------------------------------------
// pooled[b][:] = rope(rmsnorm(mean_c raw[b][c][:]) * w) at position pos0[b]; raw fp32 [blocks][kp][D], rotation over the
// first `rot` dims in halves (inv_freq [rot / 2]). grid = blocks, 128 threads, D <= 512.
__global__ void __launch_bounds__(128) qsa_pool_kernel(__nv_bfloat16* __restrict__ pooled, const float* __restrict__ raw,
                                                       const float* __restrict__ w, const int* __restrict__ pos0,
                                                       const float* __restrict__ inv_freq, int kp, int D, int rot, float eps) {
  __shared__ float v[512];
  __shared__ float red[32];
  const int b = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f;
    for (int c = 0; c < kp; ++c) s += raw[((size_t)b * kp + c) * D + i];
    s /= (float)kp;
    v[i] = s;
    ss += s * s;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)D + eps);
  __syncthreads();
  const int half = rot / 2;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float x = v[i] * inv * w[i];
    if (i < rot) {
      const int j = i < half ? i : i - half;
      const float other = v[i < half ? i + half : i - half] * inv * w[i < half ? i + half : i - half];
      float sn, cs;
      sincosf((float)pos0[b] * inv_freq[j], &sn, &cs);
      x = i < half ? x * cs - other * sn : x * cs + other * sn;
    }
    pooled[(size_t)b * D + i] = __float2bfloat16(x);
  }
}

// Row r at position pos sees nv = (pos + 1) / kp finished blocks. nv <= top: the dense table (every block up to pos).
// Otherwise the `top` selected blocks (sel ascending) and, when (pos + 1) % kp != 0, the open tail block last; kvlen
// counts the cells the attention reads. table [rows][top + 1] holds page ids of the slot's block table. One thread a
// row entry; grid = rows, 128 threads.
__global__ void __launch_bounds__(128) qsa_table_kernel(int* __restrict__ table, int* __restrict__ kvlen,
                                                        const int* __restrict__ sel, const int* __restrict__ row_slot,
                                                        const int* __restrict__ row_pos, const int* __restrict__ block_table,
                                                        int max_blocks, int kp, int top, int* __restrict__ status) {
  const int r = blockIdx.x, pos = row_pos[r], nv = (pos + 1) / kp, tail = (pos + 1) % kp;
  const int* bt = block_table + (size_t)row_slot[r] * max_blocks;
  int* out = table + (size_t)r * (top + 1);
  const bool dense = nv <= top;
  const int used = dense ? nv + (tail ? 1 : 0) : top + (tail ? 1 : 0);
  for (int j = threadIdx.x; j <= top; j += blockDim.x) {
    int logical = -1;
    if (j < used) {
      if (dense) logical = j;
      else logical = j < top ? sel[(size_t)r * top + j] : nv;
    }
    int page = 0;
    if (logical >= 0) {
      if (logical < max_blocks) page = bt[logical];
      else set_status(status, ST_BOUNDS);
    }
    out[j] = page;
  }
  if (threadIdx.x == 0) kvlen[r] = dense ? pos + 1 : top * kp + tail;
}

}  // namespace fb

using namespace fb;

extern "C" int fb_comp_step(void* out, float* tail, const float* kvc, const float* sc, const int* row_slot, const int* row_pos,
                            int rows, int ratio, int dim, int ring_len, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (ratio < 1 || ratio > ring_len || (ratio > 1 && !sc)) return -1;
  comp_stash_kernel<<<rows, 256, 0, s>>>(tail, kvc, sc, row_slot, row_pos, dim, ring_len);
  comp_close_kernel<<<rows, 256, 0, s>>>((__nv_bfloat16*)out, tail, row_slot, row_pos, ratio, dim, ring_len);
  return (int)cudaGetLastError();
}

extern "C" int fb_index_score(float* score, int ld, const void* q, const float* w, float scale, const void* keys,
                              long key_stride, const int* row_slot, const int* row_len, const uint8_t* mask, int mask_ld,
                              int mask_block, int rows, int nh, int D, cudaStream_t s) {
  if (rows <= 0 || ld <= 0) return 0;
  if (nh < 1 || nh > IDX_MAX_HEADS || D % 32 || D > IDX_MAX_D || rows > 65535 || (mask && mask_block < 1)) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(keys)) & 15 || key_stride % 8) return -1;
  dim3 grid((ld + 127) / 128, rows);
  index_score_kernel<<<grid, 256, 0, s>>>(score, ld, (const __nv_bfloat16*)q, w, scale, (const __nv_bfloat16*)keys,
                                          key_stride, row_slot, row_len, mask, mask_ld, mask_block, nh, D);
  return (int)cudaGetLastError();
}

extern "C" int fb_topk_select(int* sel, const float* score, int ld, int n, const int* row_n, int rows, int k,
                              cudaStream_t s) {
  if (rows <= 0 || k <= 0) return 0;
  topk_select_kernel<<<rows, TOPK_THREADS, 0, s>>>(sel, score, ld, n, row_n, k);
  return (int)cudaGetLastError();
}

extern "C" int fb_block_max(float* bmax, int mask_ld, const float* score, int ld, const int* row_n, int rows, int bsize,
                            cudaStream_t s) {
  if (rows <= 0 || mask_ld <= 0) return 0;
  if (bsize < 1 || rows > 65535) return -1;
  dim3 grid((mask_ld + 7) / 8, rows);
  block_max_kernel<<<grid, 256, 0, s>>>(bmax, mask_ld, score, ld, row_n, bsize);
  return (int)cudaGetLastError();
}

extern "C" int fb_sel_to_mask(uint8_t* mask, int mask_ld, const int* sel, int rows, int k, cudaStream_t s) {
  if (rows <= 0) return 0;
  sel_to_mask_kernel<<<rows, 256, 0, s>>>(mask, mask_ld, sel, k);
  return (int)cudaGetLastError();
}

extern "C" int fb_qsa_pool(void* pooled, const float* raw, const float* w, const int* pos0, const float* inv_freq,
                           int blocks, int kp, int D, int rot, float eps, cudaStream_t s) {
  if (blocks <= 0) return 0;
  if (D > 512 || rot > D || rot % 2) return -1;
  qsa_pool_kernel<<<blocks, 128, 0, s>>>((__nv_bfloat16*)pooled, raw, w, pos0, inv_freq, kp, D, rot, eps);
  return (int)cudaGetLastError();
}

extern "C" int fb_qsa_table(int* table, int* kvlen, const int* sel, const int* row_slot, const int* row_pos,
                            const int* block_table, int max_blocks, int rows, int kp, int top, int* status, cudaStream_t s) {
  if (rows <= 0) return 0;
  qsa_table_kernel<<<rows, 128, 0, s>>>(table, kvlen, sel, row_slot, row_pos, block_table, max_blocks, kp, top, status);
  return (int)cudaGetLastError();
}
