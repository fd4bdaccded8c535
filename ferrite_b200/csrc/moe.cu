// Mixture-of-experts decode path: router (softmax top-k, or sigmoid scores with group-limited top-k and a
// selection bias), grouped-expert GEMVs over (token, expert) pairs with fused SwiGLU, and the fixed-order combine
// with the shared expert and the residual. Expert parallelism: a rank computes only the pairs whose expert it
// owns ([e_lo, e_hi)); the other pairs contribute zero and the partial sums are reduced over ranks afterwards.
//
// Counterparts in the reference: `fx_route` / `fx_route8` (`kernels/k-fnext/src/fast.rs:393,667`), `ds_router`
// (`kernels/k-ds/src/moe.rs:11`), `ggq_moe_gu_*` / `ggq_moe_down_*` / `ggq_moe_combine` (`kernels/k-gguf/src/moe.rs:271-362`),
// `fx_mask_own` (`fast.rs:1718`). Ties go to the lower expert id and pairs are combined in pick order, so results
// do not depend on scheduling.
#include "api_ext.h"
#include "common.cuh"

namespace fb {

constexpr int RT_MAXPL = 32;      // experts per lane (up to 1024 experts)

// mode 0: softmax over all experts, top-k, renormalise, * scale.
// mode 1: scores = sigmoid(logit); choose by score + bias inside the best `topk_groups` of `n_groups` groups
//         (group score = sum of its two best biased scores); weights = chosen scores / sum * scale.
__global__ void __launch_bounds__(32) route_kernel(int* __restrict__ ids, float* __restrict__ wts,
                                                   const float* __restrict__ logits, const float* __restrict__ bias,
                                                   int n_exp, int top_k, int mode, int n_groups, int topk_groups,
                                                   float scale, int ld, int shared_col, int shared_id) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;
  const float* lp = logits + (size_t)row * ld;
  // `shared_id` >= 0: the always-on shared expert rides along as pick number top_k (expert id shared_id of the stack),
  // weighted by sigmoid(logit[shared_col]) or 1; ids / wts rows are then top_k + 1 wide
  const int kout = top_k + (shared_id >= 0 ? 1 : 0);
  const int per = (n_exp + 31) / 32;                 // contiguous experts per lane: lane owns [lane*per, +per)
  float sc[RT_MAXPL], sel[RT_MAXPL];
  float mx = -INFINITY;
  for (int j = 0; j < per; ++j) {
    int e = lane * per + j;
    sc[j] = e < n_exp ? lp[e] : -INFINITY;
    mx = fmaxf(mx, sc[j]);
  }
  if (mode == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
    for (int j = 0; j < per; ++j) { sc[j] = sc[j] == -INFINITY ? 0.f : __expf(sc[j] - mx); sum += sc[j]; }
    sum = warp_sum(sum);
    for (int j = 0; j < per; ++j) { sc[j] /= sum; sel[j] = (lane * per + j < n_exp) ? sc[j] : -INFINITY; }
  } else {
    for (int j = 0; j < per; ++j) {
      int e = lane * per + j;
      sc[j] = e < n_exp ? sigmoidf_(sc[j]) : 0.f;
      sel[j] = e < n_exp ? sc[j] + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    if (n_groups > 1 && topk_groups < n_groups) {
      // a group spans gl = (experts per group) / (experts per lane) lanes; its score is the sum of its two best
      // biased scores
      const int gl = (n_exp / n_groups) / per;
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int j = 0; j < per; ++j) { float v = sel[j]; if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v; }
      for (int o = 1; o < gl; o <<= 1) {
        float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        float n1 = fmaxf(b1, o1), n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1; b2 = n2;
      }
      const float gscore = b1 + b2;
      const int g = lane / gl;
      int better = 0;                                // groups that beat this one (ties: the lower group wins)
      for (int og = 0; og < n_groups; ++og) {
        float os = __shfl_sync(0xffffffffu, gscore, og * gl);
        if (os > gscore || (os == gscore && og < g)) ++better;
      }
      if (better >= topk_groups)
        for (int j = 0; j < per; ++j) sel[j] = -INFINITY;
    }
  }
  float wsum = 0.f;
  float myw = 0.f;
  int myid = 0;
  for (int k = 0; k < top_k; ++k) {
    float bv = -INFINITY;
    int bj = -1;
    for (int j = 0; j < per; ++j)
      if (sel[j] > bv) { bv = sel[j]; bj = j; }
    int be = bj >= 0 ? lane * per + bj : 0x7fffffff;
    float v = bv;
    int e = be;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, v, o);
      int oe = __shfl_xor_sync(0xffffffffu, e, o);
      if (ov > v || (ov == v && oe < e)) { v = ov; e = oe; }
    }
    // the owning lane retires the pick and reports its (unbiased) score
    float w = 0.f;
    if (e == be && bj >= 0) { w = sc[bj]; sel[bj] = -INFINITY; }
    w = warp_sum(w);
    wsum += w;
    if (lane == k) { myw = w; myid = e; }
  }
  if (lane < top_k) {
    ids[(size_t)row * kout + lane] = myid;
    wts[(size_t)row * kout + lane] = myw / (wsum + 1e-20f) * scale;
  }
  if (shared_id >= 0 && lane == 0) {
    ids[(size_t)row * kout + top_k] = shared_id;
    wts[(size_t)row * kout + top_k] = shared_col >= 0 ? sigmoidf_(lp[shared_col]) : 1.f;
  }
}

// Pair GEMVs. Weight rows are bf16; a CTA handles 16 output rows of one (token, expert) pair.
constexpr int MOE_THREADS = 256;

// act[p][j] = silu(Wg[e][j] . x[t]) * (Wu[e][j] . x[t]);  W_gu[e] = [2*inter][hidden] (gate rows then up rows)
__global__ void __launch_bounds__(MOE_THREADS)
moe_gate_up_kernel(__nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_gu,
                   const int* __restrict__ ids, int top_k, int hidden, int inter, int e_lo, int e_hi) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) __nv_bfloat16 xs_moe[];
  pdl_wait();                                                // ids come from the router kernel before this one
  const int p = blockIdx.y, e = ids[p];
  if (e < e_lo || e >= e_hi) return;                         // another rank owns this expert
  const int t = p / top_k;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(xs_moe)[i] = reinterpret_cast<const uint4*>(x + (size_t)t * hidden)[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* we = w_gu + (size_t)(e - e_lo) * 2 * inter * hidden;
  // the warp's two outputs run together: four weight rows stream at once, twice unrolled (8 loads of 16 bytes in flight)
  const int j0 = blockIdx.x * 16 + warp * 2;
  if (j0 >= inter) return;
  const int j1 = min(j0 + 1, inter - 1);
  const __nv_bfloat16* wg0 = we + (size_t)j0 * hidden;
  const __nv_bfloat16* wu0 = we + (size_t)(inter + j0) * hidden;
  const __nv_bfloat16* wg1 = we + (size_t)j1 * hidden;
  const __nv_bfloat16* wu1 = we + (size_t)(inter + j1) * hidden;
  float g0 = 0.f, u0 = 0.f, g1 = 0.f, u1 = 0.f;
  auto dot8 = [](const uint4& a, const uint4& xv, float acc) {
    const uint32_t au[4] = {a.x, a.y, a.z, a.w}, xu[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) acc = fmaf(bf_lo(au[q]), bf_lo(xu[q]), fmaf(bf_hi(au[q]), bf_hi(xu[q]), acc));
    return acc;
  };
  int k = lane * 8;
  for (; k + 256 < hidden; k += 512) {
    const uint4 a0 = ldg_stream(wg0 + k), b0 = ldg_stream(wu0 + k), c0 = ldg_stream(wg1 + k), d0 = ldg_stream(wu1 + k);
    const uint4 a1 = ldg_stream(wg0 + k + 256), b1 = ldg_stream(wu0 + k + 256), c1 = ldg_stream(wg1 + k + 256),
                d1 = ldg_stream(wu1 + k + 256);
    const uint4 x0 = *reinterpret_cast<const uint4*>(xs_moe + k), x1 = *reinterpret_cast<const uint4*>(xs_moe + k + 256);
    g0 = dot8(a1, x1, dot8(a0, x0, g0)); u0 = dot8(b1, x1, dot8(b0, x0, u0));
    g1 = dot8(c1, x1, dot8(c0, x0, g1)); u1 = dot8(d1, x1, dot8(d0, x0, u1));
  }
  for (; k < hidden; k += 256) {
    const uint4 a0 = ldg_stream(wg0 + k), b0 = ldg_stream(wu0 + k), c0 = ldg_stream(wg1 + k), d0 = ldg_stream(wu1 + k);
    const uint4 x0 = *reinterpret_cast<const uint4*>(xs_moe + k);
    g0 = dot8(a0, x0, g0); u0 = dot8(b0, x0, u0); g1 = dot8(c0, x0, g1); u1 = dot8(d0, x0, u1);
  }
  g0 = warp_sum(g0); u0 = warp_sum(u0); g1 = warp_sum(g1); u1 = warp_sum(u1);
  if (lane == 0) {
    act[(size_t)p * inter + j0] = f2bf(siluf_(g0) * u0);
    if (j0 + 1 < inter) act[(size_t)p * inter + j0 + 1] = f2bf(siluf_(g1) * u1);
  }
}

// yp[p][n] = Wd[e][n] . act[p];  W_down[e] = [hidden][inter]; fp32 out (zero for pairs of other ranks)
__global__ void __launch_bounds__(MOE_THREADS)
moe_down_kernel(float* __restrict__ yp, const __nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ w_down,
                const int* __restrict__ ids, int hidden, int inter, int e_lo, int e_hi) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) __nv_bfloat16 as_moe[];
  pdl_wait();
  const int p = blockIdx.y, e = ids[p];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 16 + warp * 2;
  if (e < e_lo || e >= e_hi) {
    if (lane == 0) for (int r = 0; r < 2; ++r) if (n0 + r < hidden) yp[(size_t)p * hidden + n0 + r] = 0.f;
    return;
  }
  for (int i = threadIdx.x; i < inter / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(as_moe)[i] = reinterpret_cast<const uint4*>(act + (size_t)p * inter)[i];
  __syncthreads();
  const __nv_bfloat16* we = w_down + (size_t)(e - e_lo) * hidden * inter;
  if (n0 >= hidden) return;
  const int n1 = min(n0 + 1, hidden - 1);
  const __nv_bfloat16* w0 = we + (size_t)n0 * inter;
  const __nv_bfloat16* w1 = we + (size_t)n1 * inter;
  float s0 = 0.f, s1 = 0.f;
  for (int k = lane * 8; k < inter; k += 256) {               // both rows of the warp stream together
    const uint4 a = ldg_stream(w0 + k), b = ldg_stream(w1 + k);
    const uint4 xv = *reinterpret_cast<const uint4*>(as_moe + k);
    const uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w}, xu[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      s0 = fmaf(bf_lo(au[q]), bf_lo(xu[q]), fmaf(bf_hi(au[q]), bf_hi(xu[q]), s0));
      s1 = fmaf(bf_lo(bu[q]), bf_lo(xu[q]), fmaf(bf_hi(bu[q]), bf_hi(xu[q]), s1));
    }
  }
  s0 = warp_sum(s0); s1 = warp_sum(s1);
  if (lane == 0) {
    yp[(size_t)p * hidden + n0] = s0;
    if (n0 + 1 < hidden) yp[(size_t)p * hidden + n0 + 1] = s1;
  }
}

// out[t] = (res[t]) + sum_k wts[t][k] * yp[t*K + k]  (pick order) + shared[t] * gate[t]; fp32 or bf16 out
__global__ void moe_combine_kernel(void* __restrict__ out, const float* __restrict__ yp, const float* __restrict__ wts,
                                   const __nv_bfloat16* __restrict__ shared, const float* __restrict__ shared_gate,
                                   const __nv_bfloat16* __restrict__ res, int top_k, int hidden, int out_f32) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= hidden) return;
  float acc = 0.f;
  for (int k = 0; k < top_k; ++k) acc = fmaf(wts[(size_t)t * top_k + k], yp[((size_t)t * top_k + k) * hidden + n], acc);
  if (shared) acc += bf2f(shared[(size_t)t * hidden + n]) * (shared_gate ? sigmoidf_(shared_gate[t]) : 1.f);
  if (res) acc += bf2f(res[(size_t)t * hidden + n]);
  if (out_f32) reinterpret_cast<float*>(out)[(size_t)t * hidden + n] = acc;
  else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)t * hidden + n] = f2bf(acc);
}

}  // namespace fb

using namespace fb;

extern "C" int fb_moe_route(int* ids, float* wts, const float* logits, const float* bias, int rows, int n_exp, int top_k,
                            int mode, int n_groups, int topk_groups, float scale, int ld, int shared_col, int shared_id,
                            cudaStream_t s) {
  if (rows <= 0) return 0;
  if (ld < n_exp || shared_col >= ld) return -1;
  if (n_exp > 32 * RT_MAXPL || top_k > 32 || top_k > n_exp) return -1;
  if (mode == 1 && n_groups > 1) {
    // a group must cover a power-of-two number of whole lanes
    const int per = (n_exp + 31) / 32;
    if (n_exp % n_groups || (n_exp / n_groups) % per) return -2;
    const int gl = (n_exp / n_groups) / per;
    if (gl < 1 || (gl & (gl - 1)) || n_groups * gl > 32) return -2;
  }
  return (int)launch_pdl(route_kernel, dim3(rows), dim3(32), 0, s, ids, wts, logits, bias, n_exp, top_k, mode,
                         n_groups, topk_groups, scale, ld, shared_col, shared_id);
}

extern "C" int fb_moe_gate_up(void* act, const void* x, const void* w_gu, const int* ids, int pairs, int top_k,
                              int hidden, int inter, int e_lo, int e_hi, cudaStream_t s) {
  if (pairs <= 0) return 0;
  if (hidden % 8) return -1;
  return (int)launch_pdl(moe_gate_up_kernel, dim3((inter + 15) / 16, pairs), dim3(MOE_THREADS), (size_t)hidden * 2, s,
                         (__nv_bfloat16*)act, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gu, ids, top_k, hidden,
                         inter, e_lo, e_hi);
}

extern "C" int fb_moe_down(float* yp, const void* act, const void* w_down, const int* ids, int pairs, int hidden,
                           int inter, int e_lo, int e_hi, cudaStream_t s) {
  if (pairs <= 0) return 0;
  if (inter % 8) return -1;
  return (int)launch_pdl(moe_down_kernel, dim3((hidden + 15) / 16, pairs), dim3(MOE_THREADS), (size_t)inter * 2, s, yp,
                         (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, ids, hidden, inter, e_lo, e_hi);
}

extern "C" int fb_moe_combine(void* out, const float* yp, const float* wts, const void* shared, const float* shared_gate,
                              const void* res, int rows, int top_k, int hidden, int out_f32, cudaStream_t s) {
  if (rows <= 0) return 0;
  return (int)launch_pdl(moe_combine_kernel, dim3((hidden + 255) / 256, rows), dim3(256), 0, s, out, yp, wts,
                         (const __nv_bfloat16*)shared, shared_gate, (const __nv_bfloat16*)res, top_k, hidden, out_f32);
}
