// Gated DeltaNet: causal depthwise conv1d + SiLU, and the gated delta-rule recurrence
//   S = S * g;  delta = (v - S^T k) * beta;  S += k (x) delta;  y = S^T q
// with q, k L2-normalised per head (q also scaled by 1/sqrt(dk)), g = exp(-exp(A_log) * softplus(a + dt_bias)),
// beta = sigmoid(b). State S is fp32 [slot][head][dk][dv].
//
// Counterparts in the reference: `fe_gdn_conv` (`kernels/k-core/src/gdn.rs:30`), `fe_gdn_rec` / `fe_gdn_rec2`
// (`:117`, `:241`) and, through the `commit` flag and saved projections, `fe_gdn_replay` (`:260`).
// The conv kernel never writes state; the recurrence kernel (which runs after it on the stream) commits both
// the recurrent state and the conv tail, so no CTA reads state another CTA of the same launch writes.
#include "api.h"
#include "common.cuh"
#include "gdn_step.cuh"

namespace fb {

// proj row layout: [q (nk*dk) | k (nk*dk) | v (nv*dv) | z (nv*dv) | b (nv) | a (nv)]
// conv_state: [slot][conv_k-1][conv_dim] bf16, oldest input first.
// grid = (ceil(conv_dim/256), row chunks of 32, segments)
__global__ void gdn_conv_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ proj,
                                long proj_stride, const __nv_bfloat16* __restrict__ conv_w,
                                const __nv_bfloat16* __restrict__ conv_state, const int* __restrict__ seg_slot,
                                const int* __restrict__ seg_row0, const int* __restrict__ seg_nrows, int conv_dim) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CK = 4, CHUNK = 32;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seg = blockIdx.z;
  const int n = seg_nrows[seg];
  const int r0 = blockIdx.y * CHUNK;
  if (c >= conv_dim || r0 >= n) return;
  const int row0 = seg_row0[seg];
  const int slot = seg_slot[seg];
  float w[CK];
#pragma unroll
  for (int j = 0; j < CK; ++j) w[j] = bf2f(conv_w[(size_t)c * CK + j]);
  const __nv_bfloat16* st = conv_state + (size_t)slot * (CK - 1) * conv_dim + c;
  float win[CK - 1];
#pragma unroll
  for (int j = 0; j < CK - 1; ++j) {
    int r = r0 - (CK - 1) + j;                      // time index relative to the segment start
    win[j] = r >= 0 ? bf2f(proj[(size_t)(row0 + r) * proj_stride + c]) : bf2f(st[(size_t)(CK - 1 + r) * conv_dim]);
  }
  const int rend = min(n, r0 + CHUNK);
  for (int r = r0; r < rend; ++r) {
    float x = bf2f(proj[(size_t)(row0 + r) * proj_stride + c]);
    float acc = w[0] * win[0] + w[1] * win[1] + w[2] * win[2] + w[3] * x;
    out[(size_t)(row0 + r) * conv_dim + c] = f2bf(siluf_(acc));
    win[0] = win[1]; win[1] = win[2]; win[2] = x;
  }
}

// Verify-tree form of the conv: the window of a row is its three nearest ancestors (then the slot's conv tail), found
// by walking `row_parent` (parent row inside the segment, -1 for the root row). Counterpart of the tree variant of
// `fe_gdn_conv` (`kernels/k-core/src/gdn.rs:30`). grid = (ceil(conv_dim/256), segments); never writes state.
__global__ void gdn_conv_tree_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ proj,
                                     long proj_stride, const __nv_bfloat16* __restrict__ conv_w,
                                     const __nv_bfloat16* __restrict__ conv_state, const int* __restrict__ seg_slot,
                                     const int* __restrict__ seg_row0, const int* __restrict__ seg_nrows,
                                     const int* __restrict__ row_parent, int conv_dim) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CK = 4;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seg = blockIdx.y;
  const int n = seg_nrows[seg];
  if (c >= conv_dim || n <= 0) return;
  const int row0 = seg_row0[seg];
  const int slot = seg_slot[seg];
  float w[CK];
#pragma unroll
  for (int j = 0; j < CK; ++j) w[j] = bf2f(conv_w[(size_t)c * CK + j]);
  const __nv_bfloat16* st = conv_state + (size_t)slot * (CK - 1) * conv_dim + c;
  for (int r = 0; r < n; ++r) {
    float acc = w[CK - 1] * bf2f(proj[(size_t)(row0 + r) * proj_stride + c]);
    int i = r;
#pragma unroll
    for (int j = CK - 2; j >= 0; --j) {
      // one step back in time: the parent row, or (past the root) one entry further into the saved tail
      i = i >= 0 ? row_parent[row0 + i] : i - 1;
      if (i >= n) i = -1;                                    // malformed parent: treat as the root's predecessor
      const float x = i >= 0 ? bf2f(proj[(size_t)(row0 + i) * proj_stride + c]) : bf2f(st[(size_t)(CK - 1 + i) * conv_dim]);
      acc = fmaf(w[j], x, acc);
    }
    out[(size_t)(row0 + r) * conv_dim + c] = f2bf(siluf_(acc));
  }
}

// Recurrence over the rows of one segment for one value head. blockDim = DV * 8; thread (col = tid % DV,
// part = tid / DV) keeps DK/8 rows of state column `col` in registers across the whole segment.
// TREE: the rows of a segment form a verify tree. A row starts from the state its parent left (`row_parent`, -1 = the
// slot's committed state); states are parked in `node_state` [row][head][DK][DV] only where `row_flags` asks for it
// (bit 0: this row's parent is not the previous row, reload; bit 1: a later row branches from this one, store). A
// thread reloads exactly the elements it stored, so no barrier is needed. Tree launches never commit. Counterpart of
// the tree variant of `fe_gdn_rec` (`kernels/k-core/src/gdn.rs:117`).
template <int DK, int DV, bool TREE>
__global__ void __launch_bounds__(DV * 8)
gdn_rec_kernel(float* __restrict__ y, float* __restrict__ rec_state, __nv_bfloat16* __restrict__ conv_state,
               const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ proj, long proj_stride,
               const float* __restrict__ A_log, const float* __restrict__ dt_bias, const int* __restrict__ seg_slot,
               const int* __restrict__ seg_row0, const int* __restrict__ seg_nrows, int nk, int nv, float eps,
               int commit, const int* __restrict__ row_parent, const int* __restrict__ row_flags,
               float* __restrict__ node_state) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int PARTS = 8, RP = DK / PARTS, CK = 4;
  __shared__ float qs[DK], ks[DK], vs[DV];
  __shared__ float red1[PARTS][DV], red2[PARTS][DV];
  __shared__ float ssq[2][DK / 32];
  const int h = blockIdx.x, seg = blockIdx.y;
  const int tid = threadIdx.x, col = tid % DV, part = tid / DV;
  const int n = seg_nrows[seg];
  if (n <= 0) return;
  const int row0 = seg_row0[seg], slot = seg_slot[seg];
  const int kh = h / (nv / nk);
  const int conv_dim = 2 * nk * DK + nv * DV;
  const int q_off = kh * DK, k_off = nk * DK + kh * DK, v_off = 2 * nk * DK + h * DV;
  const int b_off = conv_dim + nv * DV + h, a_off = b_off + nv;
  float* Sg = rec_state + (((size_t)slot * nv + h) * DK) * DV;
  float S[RP];
#pragma unroll
  for (int i = 0; i < RP; ++i) S[i] = Sg[(size_t)(part * RP + i) * DV + col];
  const float expA = __expf(A_log[h]);
  const float dtb = dt_bias[h];
  const float qscale = rsqrtf((float)DK);

  for (int r = 0; r < n; ++r) {
    int flags = 0;
    if (TREE) {
      flags = row_flags[row0 + r];
      if (flags & 1) {
        const int par = row_parent[row0 + r];
        const float* src = (par < 0 || par >= r) ? Sg : node_state + (((size_t)(row0 + par) * nv + h) * DK) * DV;
#pragma unroll
        for (int i = 0; i < RP; ++i) S[i] = src[(size_t)(part * RP + i) * DV + col];
      }
    }
    const __nv_bfloat16* xr = qkv + (size_t)(row0 + r) * conv_dim;
    if (tid < DK) {
      float qv = bf2f(xr[q_off + tid]), kv = bf2f(xr[k_off + tid]);
      qs[tid] = qv; ks[tid] = kv;
      float sq = warp_sum(qv * qv), sk = warp_sum(kv * kv);
      if ((tid & 31) == 0) { ssq[0][tid >> 5] = sq; ssq[1][tid >> 5] = sk; }
    }
    if (tid < DV) vs[tid] = bf2f(xr[v_off + tid]);
    __syncthreads();
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int i = 0; i < DK / 32; ++i) { sq += ssq[0][i]; sk += ssq[1][i]; }
    const float rq = rsqrtf(sq + eps) * qscale, rk = rsqrtf(sk + eps);
    const __nv_bfloat16* pr = proj + (size_t)(row0 + r) * proj_stride;
    const float beta = sigmoidf_(bf2f(pr[b_off]));
    const float g = __expf(-expA * softplusf_(bf2f(pr[a_off]) + dtb));
    float p = 0.f;
#pragma unroll
    for (int i = 0; i < RP; ++i) p = fmaf(S[i], ks[part * RP + i], p);
    red1[part][col] = p;
    __syncthreads();
    float kvv = 0.f;
#pragma unroll
    for (int i = 0; i < PARTS; ++i) kvv += red1[i][col];
    kvv *= g * rk;
    const float delta = (vs[col] - kvv) * beta;
    float yp = 0.f;
#pragma unroll
    for (int i = 0; i < RP; ++i) {
      S[i] = fmaf(ks[part * RP + i] * rk, delta, S[i] * g);
      yp = fmaf(S[i], qs[part * RP + i], yp);
    }
    red2[part][col] = yp;
    __syncthreads();
    if (part == 0) {
      float yy = 0.f;
#pragma unroll
      for (int i = 0; i < PARTS; ++i) yy += red2[i][col];
      y[((size_t)(row0 + r) * nv + h) * DV + col] = yy * rq;
    }
    if (TREE && (flags & 2)) {
      float* dst = node_state + (((size_t)(row0 + r) * nv + h) * DK) * DV;
#pragma unroll
      for (int i = 0; i < RP; ++i) dst[(size_t)(part * RP + i) * DV + col] = S[i];
    }
  }
  if (commit && !TREE) {
#pragma unroll
    for (int i = 0; i < RP; ++i) Sg[(size_t)(part * RP + i) * DV + col] = S[i];
    // conv tail: the last CK-1 raw inputs of the channels this head owns (q/k channels: first head of the group)
    __nv_bfloat16* st = conv_state + (size_t)slot * (CK - 1) * conv_dim;
    const bool own_qk = (h % (nv / nk)) == 0;
    const int nch = DV + (own_qk ? 2 * DK : 0);
    for (int idx = tid; idx < nch; idx += blockDim.x) {
      int c = idx < DV ? v_off + idx : (idx < DV + DK ? q_off + (idx - DV) : k_off + (idx - DV - DK));
      __nv_bfloat16 nw[CK - 1];
#pragma unroll
      for (int j = 0; j < CK - 1; ++j) {
        int t = n - (CK - 1) + j;
        nw[j] = t >= 0 ? proj[(size_t)(row0 + t) * proj_stride + c] : st[(size_t)(CK - 1 + t) * conv_dim + c];
      }
#pragma unroll
      for (int j = 0; j < CK - 1; ++j) st[(size_t)j * conv_dim + c] = nw[j];
    }
  }
}

// The decode-row fusion of the three kernels above lives in gdn_step.cuh (also used by the persistent decode-layer kernel).
template <int DK, int DV, int PARTS>
__global__ void __launch_bounds__(DV * PARTS)
gdn_step_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ rec_state, __nv_bfloat16* __restrict__ conv_state,
                const __nv_bfloat16* __restrict__ proj, long proj_stride, const __nv_bfloat16* __restrict__ conv_w,
                const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                const __nv_bfloat16* __restrict__ gnorm_w, const int* __restrict__ seg_slot,
                const int* __restrict__ seg_row0, const int* __restrict__ seg_nrows, int nk, int nv, float eps,
                int commit) {
  pdl_launch_dependents();
  pdl_wait();
  const int seg = blockIdx.y;
  gdn_step_body<DK, DV, PARTS>(out, rec_state, conv_state, proj, proj_stride, conv_w, A_log, dt_bias, gnorm_w,
                               seg_nrows[seg], seg_row0[seg], seg_slot[seg], blockIdx.x, nk, nv, eps, commit);
}

}  // namespace fb

using namespace fb;

extern "C" int fb_gdn_conv(void* out, const void* proj, long proj_stride, const void* conv_w, const void* conv_state,
                           const int* seg_slot, const int* seg_row0, const int* seg_nrows, int nseg, int max_rows,
                           int conv_dim, cudaStream_t s) {
  if (nseg <= 0 || max_rows <= 0) return 0;
  dim3 grid((conv_dim + 255) / 256, (max_rows + 31) / 32, nseg);
  launch_pdl(gdn_conv_kernel, dim3(grid), dim3(256), (size_t)(0), s, (__nv_bfloat16*)out, (const __nv_bfloat16*)proj, proj_stride,
                                       (const __nv_bfloat16*)conv_w, (const __nv_bfloat16*)conv_state, seg_slot,
                                       seg_row0, seg_nrows, conv_dim);
  return (int)cudaGetLastError();
}

extern "C" int fb_gdn_rec(float* y, float* rec_state, void* conv_state, const void* qkv, const void* proj,
                          long proj_stride, const float* A_log, const float* dt_bias, const int* seg_slot,
                          const int* seg_row0, const int* seg_nrows, int nseg, int nk, int nv, int dk, int dv,
                          float eps, int commit, cudaStream_t s) {
  if (nseg <= 0) return 0;
  if (nv % nk) return -1;
  dim3 grid(nv, nseg);
  if (dk == 128 && dv == 128)
    launch_pdl(gdn_rec_kernel<128, 128, false>, dim3(grid), dim3(1024), (size_t)(0), s, y, rec_state, (__nv_bfloat16*)conv_state, (const __nv_bfloat16*)qkv,
        (const __nv_bfloat16*)proj, proj_stride, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, nk, nv, eps, commit,
        (const int*)nullptr, (const int*)nullptr, (float*)nullptr);
  else if (dk == 64 && dv == 64)
    launch_pdl(gdn_rec_kernel<64, 64, false>, dim3(grid), dim3(512), (size_t)(0), s, y, rec_state, (__nv_bfloat16*)conv_state, (const __nv_bfloat16*)qkv,
        (const __nv_bfloat16*)proj, proj_stride, A_log, dt_bias, seg_slot, seg_row0, seg_nrows, nk, nv, eps, commit,
        (const int*)nullptr, (const int*)nullptr, (float*)nullptr);
  else return -2;
  return (int)cudaGetLastError();
}

// Verify trees: conv over ancestor windows, then the recurrence from each row's parent state. `node_state` holds
// rows x nv x dk x dv floats (rows = all rows of the step); nothing is committed.
extern "C" long fb_gdn_tree_scratch_bytes(int rows, int nv, int dk, int dv) {
  return (long)rows * nv * dk * dv * (long)sizeof(float);
}

extern "C" int fb_gdn_conv_tree(void* out, const void* proj, long proj_stride, const void* conv_w, const void* conv_state,
                                const int* seg_slot, const int* seg_row0, const int* seg_nrows, const int* row_parent,
                                int nseg, int conv_dim, cudaStream_t s) {
  if (nseg <= 0) return 0;
  dim3 grid((conv_dim + 255) / 256, nseg);
  launch_pdl(gdn_conv_tree_kernel, dim3(grid), dim3(256), (size_t)(0), s, (__nv_bfloat16*)out, (const __nv_bfloat16*)proj,
             proj_stride, (const __nv_bfloat16*)conv_w, (const __nv_bfloat16*)conv_state, seg_slot, seg_row0, seg_nrows,
             row_parent, conv_dim);
  return (int)cudaGetLastError();
}

extern "C" int fb_gdn_rec_tree(float* y, float* rec_state, const void* qkv, const void* proj, long proj_stride,
                               const float* A_log, const float* dt_bias, const int* seg_slot, const int* seg_row0,
                               const int* seg_nrows, const int* row_parent, const int* row_flags, float* node_state,
                               int nseg, int nk, int nv, int dk, int dv, float eps, cudaStream_t s) {
  if (nseg <= 0) return 0;
  if (nv % nk) return -1;
  if (!row_parent || !row_flags || !node_state) return -3;
  dim3 grid(nv, nseg);
  if (dk == 128 && dv == 128)
    launch_pdl(gdn_rec_kernel<128, 128, true>, dim3(grid), dim3(1024), (size_t)(0), s, y, rec_state, (__nv_bfloat16*)nullptr,
               (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)proj, proj_stride, A_log, dt_bias, seg_slot, seg_row0, seg_nrows,
               nk, nv, eps, 0, row_parent, row_flags, node_state);
  else if (dk == 64 && dv == 64)
    launch_pdl(gdn_rec_kernel<64, 64, true>, dim3(grid), dim3(512), (size_t)(0), s, y, rec_state, (__nv_bfloat16*)nullptr,
               (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)proj, proj_stride, A_log, dt_bias, seg_slot, seg_row0, seg_nrows,
               nk, nv, eps, 0, row_parent, row_flags, node_state);
  else return -2;
  return (int)cudaGetLastError();
}

extern "C" int fb_gdn_step(void* out, float* rec_state, void* conv_state, const void* proj, long proj_stride,
                           const void* conv_w, const float* A_log, const float* dt_bias, const void* gnorm_w,
                           const int* seg_slot, const int* seg_row0, const int* seg_nrows, int nseg, int nk, int nv, int dk,
                           int dv, float eps, int commit, cudaStream_t s) {
  if (nseg <= 0) return 0;
  if (nv % nk) return -1;
  dim3 grid(nv, nseg);
  if (dk == 128 && dv == 128)
    launch_pdl(gdn_step_kernel<128, 128, 4>, dim3(grid), dim3(512), (size_t)(0), s, (__nv_bfloat16*)out, rec_state,
               (__nv_bfloat16*)conv_state, (const __nv_bfloat16*)proj, proj_stride, (const __nv_bfloat16*)conv_w, A_log, dt_bias,
               (const __nv_bfloat16*)gnorm_w, seg_slot, seg_row0, seg_nrows, nk, nv, eps, commit);
  else if (dk == 64 && dv == 64)
    launch_pdl(gdn_step_kernel<64, 64, 8>, dim3(grid), dim3(512), (size_t)(0), s, (__nv_bfloat16*)out, rec_state,
               (__nv_bfloat16*)conv_state, (const __nv_bfloat16*)proj, proj_stride, (const __nv_bfloat16*)conv_w, A_log, dt_bias,
               (const __nv_bfloat16*)gnorm_w, seg_slot, seg_row0, seg_nrows, nk, nv, eps, commit);
  else return -2;
  return (int)cudaGetLastError();
}
