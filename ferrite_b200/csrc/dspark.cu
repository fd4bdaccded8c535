// Drafting heads that run on top of a target model's hidden rows: the Markov (bigram-bias) head loop and the
// confidence head, plus the two reductions over hyper-connection streams that feed them.
//
//   markov_bias    bias[r][v] = head[v] . emb[tok[r]] (low-rank bigram logits, rank <= 512) for rows whose token has no
//                  cached bias row (slot[r] < 0); bf16 out, fp32 accumulation in a fixed lane order
//   markov_score   best (value, index) of logits[r] + bias over a column slice, in the order of an arg-max that puts
//                  NaN first, then the larger value, then the lower index: a total order, so any split of the columns
//                  over CTAs or ranks gives the same pick
//   markov_pick    the pick over all slices (and ranks), appended to the draft, with the next step's bias slot
//   conf_head      conf[j] = [xc row | emb[prev]] . w: how much the drafter trusts draft j
//   stream_mean    out[r] = bf16(mean over the hc residual streams), summed in stream order
//   stream_collapse xc[r] = bf16(sum_j pre[r][j] * h[r][j])
//
// Counterparts of the reference's `markov_bias`, `markov_score`, `markov_pick`, `markov_begin`, `conf_head`,
// `dspark_tap`, `dspark_collapse` (`kernels/k-dspark/src/lib.rs:57-275`).
#include "api_ext.h"
#include "common.cuh"

namespace fb {

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// (v1, i1) ahead of (v2, i2)?
__device__ __forceinline__ bool mk_better(float v1, uint32_t i1, float v2, uint32_t i2) {
  const bool n1 = v1 != v1, n2 = v2 != v2;
  if (n1 || n2) return (n1 && n2) ? i1 < i2 : n1;
  return v1 > v2 || (v1 == v2 && i1 < i2);
}

// grid = (ceil(V / 8), rows), 256 threads: a warp per vocabulary entry. head [V][rank], emb [vocab][rank] bf16.
__global__ void __launch_bounds__(256) markov_bias_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ head,
                                                          const __nv_bfloat16* __restrict__ emb, const int* __restrict__ tok,
                                                          const int* __restrict__ slot, int V, int rank) {
  const int r = blockIdx.y, v = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (slot[r] >= 0 || v >= V) return;
  const __nv_bfloat16* e = emb + (size_t)tok[r] * rank;
  const __nv_bfloat16* hrow = head + (size_t)v * rank;
  float acc = 0.f;
  for (int k = lane * 8; k < rank; k += 256) {
    const uint4 a = ldg_stream(hrow + k), b = *reinterpret_cast<const uint4*>(e + k);
    const uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc = fmaf(bf_lo(au[j]), bf_lo(bu[j]), acc); acc = fmaf(bf_hi(au[j]), bf_hi(bu[j]), acc); }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[(size_t)r * V + v] = __float2bfloat16(acc);
}

// grid = (rows, parts), 256 threads. pair [parts][rows] = (value bits, global index col0 + c).
__global__ void __launch_bounds__(256) markov_score_kernel(uint2* __restrict__ pair, const float* __restrict__ logits, long ld,
                                                           const __nv_bfloat16* __restrict__ stage,
                                                           const __nv_bfloat16* __restrict__ cache,
                                                           const int* __restrict__ slot, int n, int col0) {
  __shared__ float sv[8];
  __shared__ uint32_t si[8];
  const int r = blockIdx.x, p = blockIdx.y, parts = gridDim.y;
  const int chunk = (n + parts - 1) / parts, end = min(n, (p + 1) * chunk);
  const int s = slot[r];
  const uint16_t* bias = reinterpret_cast<const uint16_t*>(s >= 0 ? cache + (size_t)s * n : stage + (size_t)r * n);
  const float* lg = logits + (size_t)r * ld;
  float bv = -INFINITY;
  uint32_t bi = 0xffffffffu;
  for (int c = p * chunk + threadIdx.x; c < end; c += blockDim.x) {
    const float v = lg[c] + bf16_bits_to_float(bias[c]);
    const uint32_t i = (uint32_t)(col0 + c);
    if (mk_better(v, i, bv, bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (mk_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (mk_better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    pair[(size_t)p * gridDim.x + r] = make_uint2(__float_as_uint(bv), bi);
  }
}

// One block, a thread a row: draft[r][step + 1] = tok[r] = the best of `n_pairs` candidates (rank-major: the lower index
// wins a tie whatever the order); slot[r] = slot_of[best]. step < 0: the start of a loop, tok[r] = draft[r][0].
__global__ void markov_pick_kernel(int* __restrict__ draft, int* __restrict__ tok, int* __restrict__ slot,
                                   const uint2* __restrict__ pairs, const int* __restrict__ slot_of, int n_pairs, int rows,
                                   int stride, int step, int vocab, int* __restrict__ status) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  uint32_t bi;
  if (step < 0) {
    bi = (uint32_t)draft[(size_t)r * stride];
  } else {
    float bv = __uint_as_float(pairs[r].x);
    bi = pairs[r].y;
    for (int k = 1; k < n_pairs; ++k) {
      const uint2 p = pairs[(size_t)k * rows + r];
      if (mk_better(__uint_as_float(p.x), p.y, bv, bi)) { bv = __uint_as_float(p.x); bi = p.y; }
    }
    if (bi >= (uint32_t)vocab) { set_status(status, ST_BOUNDS); bi = 0; }      // an empty slice set: keep indices legal
    draft[(size_t)r * stride + step + 1] = (int)bi;
  }
  tok[r] = (int)bi;
  slot[r] = slot_of[bi];
}

// grid = streams * steps, 256 threads. Row j = s * steps + i reads xc row s * block + i and the embedding of the
// token that draft i + 1 followed (draft[s][i]); w fp32 [d + rank].
__global__ void __launch_bounds__(256) conf_head_kernel(float* __restrict__ conf, const __nv_bfloat16* __restrict__ xc,
                                                        const __nv_bfloat16* __restrict__ emb, const int* __restrict__ draft,
                                                        const float* __restrict__ w, int d, int rank, int steps, int block,
                                                        int stride) {
  __shared__ float red[32];
  const int j = blockIdx.x, s = j / steps, i = j % steps;
  const __nv_bfloat16* x = xc + (size_t)(s * block + i) * d;
  const __nv_bfloat16* e = emb + (size_t)draft[(size_t)s * stride + i] * rank;
  float acc = 0.f;
  for (int c = threadIdx.x; c < d + rank; c += blockDim.x)
    acc = fmaf(__bfloat162float(c < d ? x[c] : e[c - d]), w[c], acc);
  const float tot = block_sum(acc, red);
  if (threadIdx.x == 0) conf[j] = tot;
}

// h [rows][hc][dim] bf16 -> out[r * ld + c] = bf16(((h0 + h1) + h2 ...) / hc). grid = rows, 256 threads.
__global__ void __launch_bounds__(256) stream_mean_kernel(__nv_bfloat16* __restrict__ out, long ld,
                                                          const __nv_bfloat16* __restrict__ h, int hc, int dim) {
  const int r = blockIdx.x;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < hc; ++j) s += __bfloat162float(h[((size_t)r * hc + j) * dim + c]);
    out[(size_t)r * ld + c] = __float2bfloat16(s / (float)hc);
  }
}

// xc[r][c] = bf16(sum_j pre[r * pre_ld + j] * h[r][j][c]). grid = rows, 256 threads.
__global__ void __launch_bounds__(256) stream_collapse_kernel(__nv_bfloat16* __restrict__ xc, const __nv_bfloat16* __restrict__ h,
                                                              const float* __restrict__ pre, long pre_ld, int hc, int dim) {
  const int r = blockIdx.x;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < hc; ++j) s = fmaf(pre[(size_t)r * pre_ld + j], __bfloat162float(h[((size_t)r * hc + j) * dim + c]), s);
    xc[(size_t)r * dim + c] = __float2bfloat16(s);
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_markov_bias(void* out, const void* head, const void* emb, const int* tok, const int* slot, int rows, int V,
                              int rank, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (rank % 8 || rows > 65535) return -1;
  dim3 grid((V + 7) / 8, rows);
  markov_bias_kernel<<<grid, 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)head, (const __nv_bfloat16*)emb, tok,
                                          slot, V, rank);
  return (int)cudaGetLastError();
}

extern "C" int fb_markov_score(void* pair, const float* logits, long ld, const void* stage, const void* cache,
                               const int* slot, int rows, int parts, int n, int col0, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (parts < 1 || parts > 65535) return -1;
  dim3 grid(rows, parts);
  markov_score_kernel<<<grid, 256, 0, s>>>((uint2*)pair, logits, ld, (const __nv_bfloat16*)stage,
                                           (const __nv_bfloat16*)cache, slot, n, col0);
  return (int)cudaGetLastError();
}

extern "C" int fb_markov_pick(int* draft, int* tok, int* slot, const void* pairs, const int* slot_of, int n_pairs, int rows,
                              int stride, int step, int vocab, int* status, cudaStream_t s) {
  if (rows <= 0) return 0;
  markov_pick_kernel<<<(rows + 127) / 128, 128, 0, s>>>(draft, tok, slot, (const uint2*)pairs, slot_of, n_pairs, rows, stride,
                                                        step, vocab, status);
  return (int)cudaGetLastError();
}

extern "C" int fb_conf_head(float* conf, const void* xc, const void* emb, const int* draft, const float* w, int streams,
                            int steps, int d, int rank, int block, int stride, cudaStream_t s) {
  if (streams * steps <= 0) return 0;
  conf_head_kernel<<<streams * steps, 256, 0, s>>>(conf, (const __nv_bfloat16*)xc, (const __nv_bfloat16*)emb, draft, w, d,
                                                   rank, steps, block, stride);
  return (int)cudaGetLastError();
}

extern "C" int fb_stream_mean(void* out, long ld, const void* h, int rows, int hc, int dim, cudaStream_t s) {
  if (rows <= 0) return 0;
  stream_mean_kernel<<<rows, 256, 0, s>>>((__nv_bfloat16*)out, ld, (const __nv_bfloat16*)h, hc, dim);
  return (int)cudaGetLastError();
}

extern "C" int fb_stream_collapse(void* xc, const void* h, const float* pre, long pre_ld, int rows, int hc, int dim,
                                  cudaStream_t s) {
  if (rows <= 0) return 0;
  stream_collapse_kernel<<<rows, 256, 0, s>>>((__nv_bfloat16*)xc, (const __nv_bfloat16*)h, pre, pre_ld, hc, dim);
  return (int)cudaGetLastError();
}
