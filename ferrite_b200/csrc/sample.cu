// Token selection on the device: greedy argmax, temperature / top-k / top-p / min-p sampling with presence,
// frequency and repetition penalties, a finite check, and the accept-while-match walk of a verified draft.
// Counterparts in the reference: `fe_argmax` (`kernels/k-core/src/misc.rs:89`), the host sampler
// (`crates/fe-model/src/sched.rs:2103-2200`, `crates/fe-server/src/sampler.rs`) and `tree_walk` (`sched.rs:125`).
#include "api.h"
#include "common.cuh"

namespace fb {

template <typename T> __device__ __forceinline__ float ld_logit(const T* p, size_t i);
template <> __device__ __forceinline__ float ld_logit<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return bf2f(p[i]); }

// ids[row] = lowest index of the maximum; finite[row] = 0 when a non-finite logit was seen.
template <typename T>
__global__ void argmax_kernel(int* __restrict__ ids, float* __restrict__ vals, int* __restrict__ finite,
                              const T* __restrict__ logits, long stride, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int sbad;
  const int row = blockIdx.x;
  const T* lp = logits + (size_t)row * stride;
  if (threadIdx.x == 0) sbad = 0;
  __syncthreads();
  float best = -INFINITY;
  int bi = 0x7fffffff;
  bool bad = false;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = ld_logit<T>(lp, i);
    if (!isfinite(v)) bad = true;
    if (v > best) { best = v; bi = i; }
  }
  if (bad) sbad = 1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      ids[row] = bi == 0x7fffffff ? 0 : bi;
      if (vals) vals[row] = best;
      if (finite) finite[row] = sbad ? 0 : 1;
    }
  }
}

// Two-stage argmax for wide vocabularies: stage 1 scans a slice of the row per CTA, stage 2 merges the slices in
// slice order (ties to the lower index), so one row is spread over many SMs instead of one.
constexpr int AM_SLICES = 64;
template <typename T>
__global__ void argmax_part_kernel(float* __restrict__ pv, int* __restrict__ pi, int* __restrict__ pbad,
                                   const T* __restrict__ logits, long stride, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int sbad;
  const int row = blockIdx.x, slice = blockIdx.y;
  const int per = (vocab + AM_SLICES - 1) / AM_SLICES;
  const int lo = slice * per, hi = min(vocab, lo + per);
  const T* lp = logits + (size_t)row * stride;
  if (threadIdx.x == 0) sbad = 0;
  __syncthreads();
  float best = -INFINITY;
  int bi = 0x7fffffff;
  bool bad = false;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float v = ld_logit<T>(lp, i);
    if (!isfinite(v)) bad = true;
    if (v > best) { best = v; bi = i; }
  }
  if (bad) sbad = 1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < (int)(blockDim.x >> 5); ++k)
      if (sv[k] > best || (sv[k] == best && si[k] < bi)) { best = sv[k]; bi = si[k]; }
    pv[row * AM_SLICES + slice] = best;
    pi[row * AM_SLICES + slice] = bi;
    pbad[row * AM_SLICES + slice] = sbad;
  }
}

__global__ void argmax_fin_kernel(int* __restrict__ ids, float* __restrict__ vals, int* __restrict__ finite,
                                  const float* __restrict__ pv, const int* __restrict__ pi,
                                  const int* __restrict__ pbad) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff, bad = 0;
  for (int k = lane; k < AM_SLICES; k += 32) {
    float v = pv[row * AM_SLICES + k];
    int ix = pi[row * AM_SLICES + k];
    bad |= pbad[row * AM_SLICES + k];
    if (v > best || (v == best && ix < bi)) { best = v; bi = ix; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) {
    ids[row] = bi == 0x7fffffff ? 0 : bi;
    if (vals) vals[row] = best;
    if (finite) finite[row] = bad ? 0 : 1;
  }
}

// SplitMix64 step, the generator family the reference's server sampler uses (`crates/fe-server/src/sampler.rs`).
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long& s) {
  s += 0x9E3779B97F4A7C15ull;
  unsigned long long z = s;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct SampleParams {
  float temperature, top_p, min_p, presence, frequency, repetition;
  int top_k;
  unsigned long long seed;
};

// One CTA per row. Penalties use counts[row][vocab] (int32, may be null). Sampling works on a candidate set
// found by threshold refinement: the top-k / top-p / min-p cut is expressed as a probability threshold found
// by bisection over the value range, so no sort of the vocabulary is needed.
template <typename T>
__global__ void sample_kernel(int* __restrict__ ids, const T* __restrict__ logits, long stride, int vocab,
                              const SampleParams* __restrict__ params, const int* __restrict__ counts,
                              float* __restrict__ work) {
  __shared__ float scratch[32];
  __shared__ float s_thr;
  __shared__ int s_pick;
  const int row = blockIdx.x;
  const SampleParams sp = params[row];
  const T* lp = logits + (size_t)row * stride;
  float* wk = work + (size_t)row * vocab;
  const int* cnt = counts ? counts + (size_t)row * vocab : nullptr;
  const float invt = sp.temperature > 0.f ? 1.f / sp.temperature : 1.f;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = ld_logit<T>(lp, i);
    if (cnt) {
      int c = cnt[i];
      if (c > 0) {
        if (sp.repetition != 1.f && sp.repetition > 0.f) v = v > 0.f ? v / sp.repetition : v * sp.repetition;
        v -= sp.presence + sp.frequency * (float)c;
      }
    }
    v *= invt;
    wk[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, scratch);
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) { float p = __expf(wk[i] - mx); wk[i] = p; sum += p; }
  sum = block_sum(sum, scratch);
  // The kept set is the intersection of the three filters, applied in the host sampler's order: top-k first, top-p
  // over the mass that top-k kept, min-p relative to the largest probability. Each filter is a probability threshold
  // (wk holds p / p_max, so the largest value is 1) found by bisection; the final threshold is the largest of them.
  const bool need_k = sp.top_k > 0 && sp.top_k < vocab;
  const bool need_p = sp.top_p > 0.f && sp.top_p < 1.f;
  float thr_k = 0.f, mass_k = sum;
  if (need_k) {
    float a = 0.f, b = 1.0f;                          // a keeps >= k tokens, b (pushed just above 1) keeps fewer
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (a + b);
      float c = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += wk[i] >= mid ? 1.f : 0.f;
      c = block_sum(c, scratch);
      if (c >= (float)sp.top_k) a = mid; else b = mid;
    }
    thr_k = a;
    float m = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const float p = wk[i]; if (p >= thr_k) m += p; }
    mass_k = block_sum(m, scratch);
  }
  float thr_p = thr_k;
  if (need_p) {
    // largest threshold whose kept mass still reaches top_p of the top-k mass: the shortest prefix of the sorted
    // distribution that covers top_p
    float a = thr_k, b = 1.0f;
    const float want = sp.top_p * mass_k;
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (a + b);
      float m = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const float p = wk[i]; if (p >= mid) m += p; }
      m = block_sum(m, scratch);
      if (m >= want) a = mid; else b = mid;
    }
    thr_p = a;
  }
  float thr = fmaxf(thr_k, thr_p);
  if (sp.min_p > 0.f) thr = fmaxf(thr, sp.min_p);
  thr = fminf(thr, 1.0f);                             // the most likely token always survives
  if (threadIdx.x == 0) s_thr = thr;
  __syncthreads();
  thr = s_thr;
  float kept = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) { float p = wk[i]; if (p >= thr) kept += p; }
  kept = block_sum(kept, scratch);
  // draw u in [0, kept) and walk the kept tokens in index order (deterministic for a seed)
  unsigned long long st = sp.seed;
  float u = (float)((splitmix64(st) >> 40) * (1.0 / 16777216.0)) * kept;
  // serial prefix over blockDim-sized strips: each thread sums its strip, then thread 0 finds the strip
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int b0 = threadIdx.x * per, b1 = min(vocab, b0 + per);
  float mine = 0.f;
  for (int i = b0; i < b1; ++i) { float p = wk[i]; if (p >= thr) mine += p; }
  extern __shared__ float strip[];
  strip[threadIdx.x] = mine;
  if (threadIdx.x == 0) s_pick = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float acc = 0.f;
    int t = 0;
    for (; t < (int)blockDim.x; ++t) { if (acc + strip[t] > u) break; acc += strip[t]; }
    if (t == (int)blockDim.x) t = blockDim.x - 1;
    int s0 = t * per, s1 = min(vocab, s0 + per);
    int pick = -1, last = -1;
    for (int i = s0; i < s1; ++i) {
      float p = wk[i];
      if (p >= thr) { last = i; acc += p; if (acc > u) { pick = i; break; } }
    }
    if (pick < 0) pick = last;
    s_pick = pick;
  }
  __syncthreads();
  if (s_pick < 0) {
    // numerical corner: fall back to the arg-max of the kept set
    float best = -1.f; int bi = 0;
    if (threadIdx.x == 0) {
      for (int i = 0; i < vocab; ++i) if (wk[i] > best) { best = wk[i]; bi = i; }
      ids[row] = bi;
    }
  } else if (threadIdx.x == 0) {
    ids[row] = s_pick;
  }
}

// Accept-while-match over a verified chain: draft[i] was fed at row i+1; target[i] is the model's pick after
// row i. n_accept = number of leading drafts equal to the target's pick; the bonus token is target[n_accept].
__global__ void chain_accept_kernel(int* __restrict__ n_accept, int* __restrict__ out_tokens,
                                    const int* __restrict__ target, const int* __restrict__ draft,
                                    const int* __restrict__ seg_row0, const int* __restrict__ seg_ndraft,
                                    int max_draft) {
  const int seg = blockIdx.x;
  if (threadIdx.x != 0) return;
  const int r0 = seg_row0[seg], nd = seg_ndraft[seg];
  int acc = 0;
  while (acc < nd && draft[r0 + acc] == target[r0 + acc]) ++acc;
  n_accept[seg] = acc;
  for (int i = 0; i <= acc; ++i) out_tokens[(size_t)seg * (max_draft + 1) + i] = target[r0 + i];
}

// Compaction of an accepted tree path's K/V rows: move i of a segment copies cache row src[i] onto row dst[i] (flat row
// = page * kv_block + offset) in up to three tensors at once (K codes, V codes, scales; blockIdx.z picks the tensor).
// The moves of a segment are listed root first, where dst <= src and both ascend: a thread owns one 16-byte column of
// the row and walks the moves in order, so it never reads a row it has already overwritten and needs no staging copy.
// grid = (column chunks, segments, tensors), 128 threads.
struct KvMoveArgs {
  unsigned char* base[3];
  long row_bytes[3];
  int vec[3];                 // bytes a thread moves per row: 16 when the rows allow it, else 4
};

__global__ void __launch_bounds__(128) kv_move_rows_kernel(KvMoveArgs a, const int* __restrict__ src,
                                                           const int* __restrict__ dst, const int* __restrict__ seg_off) {
  const int z = blockIdx.z, seg = blockIdx.y;
  if (!a.base[z]) return;
  const long col = ((long)blockIdx.x * blockDim.x + threadIdx.x) * a.vec[z];
  if (col >= a.row_bytes[z]) return;
  for (int i = seg_off[seg]; i < seg_off[seg + 1]; ++i) {
    const unsigned char* from = a.base[z] + (size_t)src[i] * a.row_bytes[z] + col;
    unsigned char* to = a.base[z] + (size_t)dst[i] * a.row_bytes[z] + col;
    if (a.vec[z] == 16) *reinterpret_cast<uint4*>(to) = *reinterpret_cast<const uint4*>(from);
    else *reinterpret_cast<uint32_t*>(to) = *reinterpret_cast<const uint32_t*>(from);
  }
}

}  // namespace fb

using namespace fb;

// rows of every tensor are multiples of 4 bytes; tensors not given are null
extern "C" int fb_kv_move_rows(void* k, long k_row_bytes, void* v, long v_row_bytes, void* sc, long sc_row_bytes,
                               const int* src, const int* dst, const int* seg_off, int nseg, cudaStream_t s) {
  if (nseg <= 0) return 0;
  KvMoveArgs a;
  a.base[0] = (unsigned char*)k; a.base[1] = (unsigned char*)v; a.base[2] = (unsigned char*)sc;
  a.row_bytes[0] = k_row_bytes; a.row_bytes[1] = v_row_bytes; a.row_bytes[2] = sc_row_bytes;
  long most = 0;               // threads the widest tensor needs per row
  for (int i = 0; i < 3; ++i) {
    a.vec[i] = 16;
    if (!a.base[i]) continue;
    if (a.row_bytes[i] % 4 || (reinterpret_cast<uintptr_t>(a.base[i]) & 15)) return -1;
    if (a.row_bytes[i] % 16) a.vec[i] = 4;
    const long need = a.row_bytes[i] / a.vec[i];
    if (need > most) most = need;
  }
  if (most == 0) return 0;
  dim3 grid((unsigned)((most + 127) / 128), nseg, 3);
  kv_move_rows_kernel<<<grid, 128, 0, s>>>(a, src, dst, seg_off);
  return (int)cudaGetLastError();
}

// scratch: rows * 64 * 3 words (slice maxima, indices, non-finite flags); when null the one-CTA kernel runs
extern "C" int fb_argmax2(int* ids, float* vals, int* finite, const void* logits, long stride, int rows, int vocab,
                          int is_f32, void* scratch, cudaStream_t s) {
  if (rows <= 0) return 0;
  float* pv = (float*)scratch;
  int* pi = (int*)scratch + (size_t)rows * AM_SLICES;
  int* pbad = (int*)scratch + (size_t)2 * rows * AM_SLICES;
  dim3 grid(rows, AM_SLICES);
  if (is_f32) launch_pdl(argmax_part_kernel<float>, dim3(grid), dim3(256), (size_t)(0), s, pv, pi, pbad, (const float*)logits, stride, vocab);
  else launch_pdl(argmax_part_kernel<__nv_bfloat16>, dim3(grid), dim3(256), (size_t)(0), s, pv, pi, pbad, (const __nv_bfloat16*)logits, stride, vocab);
  launch_pdl(argmax_fin_kernel, dim3(rows), dim3(32), (size_t)(0), s, ids, vals, finite, pv, pi, pbad);
  return (int)cudaGetLastError();
}

extern "C" int fb_argmax(int* ids, float* vals, int* finite, const void* logits, long stride, int rows, int vocab,
                         int is_f32, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (is_f32) launch_pdl(argmax_kernel<float>, dim3(rows), dim3(1024), (size_t)(0), s, ids, vals, finite, (const float*)logits, stride, vocab);
  else launch_pdl(argmax_kernel<__nv_bfloat16>, dim3(rows), dim3(1024), (size_t)(0), s, ids, vals, finite, (const __nv_bfloat16*)logits, stride, vocab);
  return (int)cudaGetLastError();
}

extern "C" int fb_sample(int* ids, const void* logits, long stride, int rows, int vocab, const void* params,
                         const int* counts, float* work, int is_f32, cudaStream_t s) {
  if (rows <= 0) return 0;
  const int threads = 1024;
  size_t smem = threads * sizeof(float);
  if (is_f32) sample_kernel<float><<<rows, threads, smem, s>>>(ids, (const float*)logits, stride, vocab, (const SampleParams*)params, counts, work);
  else sample_kernel<__nv_bfloat16><<<rows, threads, smem, s>>>(ids, (const __nv_bfloat16*)logits, stride, vocab, (const SampleParams*)params, counts, work);
  return (int)cudaGetLastError();
}

extern "C" int fb_chain_accept(int* n_accept, int* out_tokens, const int* target, const int* draft,
                               const int* seg_row0, const int* seg_ndraft, int nseg, int max_draft, cudaStream_t s) {
  if (nseg <= 0) return 0;
  chain_accept_kernel<<<nseg, 32, 0, s>>>(n_accept, out_tokens, target, draft, seg_row0, seg_ndraft, max_draft);
  return (int)cudaGetLastError();
}
