// Gated DeltaNet, chunked scan for prompt-sized segments (same recurrence as gdn.cu, see its header):
//   S_t = g_t S_{t-1} + k_t d_t^T,   d_t = beta_t (v_t - g_t S_{t-1}^T k_t),   y_t = S_t^T q_t.
//
// Over a chunk of C = 64 rows that starts from state S_0, with c_t = sum_{i<=t} log g_i:
//   (I + A) D = diag(beta) (V - diag(e^{c}) K S_0),     A[t][i] = beta_t e^{c_t - c_i} (k_t . k_i)   (i < t)
//   Y   = diag(e^{c}) Q S_0 + P D,                      P[t][i] = e^{c_t - c_i} (q_t . k_i)          (i <= t)
//   S_C = e^{c_C} S_0 + sum_i e^{c_C - c_i} k_i d_i^T
// so the work splits in two kernels:
//   prep  (parallel over chunk x head): normalise q/k, decays, T' = (I + A)^{-1} diag(beta), P        -> scratch
//   scan  (sequential over the chunks of a segment, parallel over head x 16-column slices of the state):
//         five small fp32 matrix products per chunk, operands double-buffered through cp.async.
// State columns never interact, which is what lets the scan split the value dimension over CTAs.
// All products run in fp32 FMA: the state carries hundreds of chunks of history and the reference needs a
// three-way TF32 split to hold its accuracy (`fe_gdn_chunk_tc`, `kernels/k-gdn/src/lib.rs`); per 2048-row prompt
// and layer this is ~5 GFLOP, far from the bound that matters here (the serial chain of chunks).
//
// Counterparts in the reference: `fe_gdn_chunk`, `fe_gdn_chunk_tc`, `fe_gdn_chunk_tc1` (`kernels/k-gdn/src/lib.rs`),
// `fx_gdn_chunk*` (`kernels/k-fnext/src/gdn.rs`); host wrapper `Gdn::run` (`crates/fe-gdn/src/lib.rs`).
#include "api.h"
#include "common.cuh"

namespace fb {

constexpr int GC = 64;            // rows per chunk
constexpr int GC_W = 16;          // state columns per scan CTA
constexpr int GC_THREADS = 256;

__device__ __forceinline__ void gc_cp16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void gc_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void gc_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// floats of scratch per (chunk, head): Kn[C][DK] | Qn[C][DK] | Tp[C][C] | P[C][C] | c[C]
__host__ __device__ constexpr long gc_rec_floats(int dk) { return 2l * GC * dk + 2l * GC * GC + GC; }

// ---- prep ------------------------------------------------------------------------------------------------
// grid (max chunks per segment, nv, nseg); 256 threads.
template <int DK>
__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_prep_kernel(float* __restrict__ scratch, const __nv_bfloat16* __restrict__ qkv,
                      const __nv_bfloat16* __restrict__ proj, long proj_stride, const float* __restrict__ A_log,
                      const float* __restrict__ dt_bias, const int* __restrict__ seg_row0,
                      const int* __restrict__ seg_nrows, int nk, int nv, int dv, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int LDK = DK + 4;              // padded rows: 8 rows x float4 hit 32 distinct banks
  constexpr int LDA = GC + 1;
  extern __shared__ __align__(16) float sm_prep[];
  float* Ks = sm_prep;                     // [GC][LDK]
  float* Qs = Ks + GC * LDK;               // [GC][LDK]
  float* Am = Qs + GC * LDK;               // [GC][LDA]
  float* cs = Am + GC * LDA;               // [GC] cumulative log decay
  float* bs = cs + GC;                     // [GC] beta
  const int chunk = blockIdx.x, h = blockIdx.y, seg = blockIdx.z;
  const int n = seg_nrows[seg];
  if (chunk * GC >= n) return;
  const int row0 = seg_row0[seg] + chunk * GC;
  const int valid = min(GC, n - chunk * GC);
  const int kh = h / (nv / nk);
  const int conv_dim = 2 * nk * DK + nv * dv;
  const int q_off = kh * DK, k_off = nk * DK + kh * DK;
  const int b_off = conv_dim + nv * dv + h, a_off = b_off + nv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* rec = scratch + ((size_t)(seg_row0[seg] / GC + seg + chunk) * nv + h) * gc_rec_floats(DK);
  float* gK = rec;
  float* gQ = gK + GC * DK;
  float* gT = gQ + GC * DK;
  float* gP = gT + GC * GC;
  float* gc = gP + GC * GC;

  // normalised q (scaled by 1/sqrt(dk)) and k, one warp per row; rows past the segment end are zero
  constexpr int EPL = DK / 32;
  const float qscale = rsqrtf((float)DK);
  for (int t = warp; t < GC; t += GC_THREADS / 32) {
    float qv[EPL], kv[EPL];
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      if (t < valid) {
        const __nv_bfloat16* xr = qkv + (size_t)(row0 + t) * conv_dim;
        qv[j] = bf2f(xr[q_off + lane * EPL + j]);
        kv[j] = bf2f(xr[k_off + lane * EPL + j]);
      } else {
        qv[j] = 0.f; kv[j] = 0.f;
      }
      sq = fmaf(qv[j], qv[j], sq);
      sk = fmaf(kv[j], kv[j], sk);
    }
    sq = warp_sum(sq); sk = warp_sum(sk);
    const float rq = rsqrtf(sq + eps) * qscale, rk = rsqrtf(sk + eps);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const float qn = qv[j] * rq, kn = kv[j] * rk;
      Qs[t * LDK + lane * EPL + j] = qn;
      Ks[t * LDK + lane * EPL + j] = kn;
      gQ[t * DK + lane * EPL + j] = qn;
      gK[t * DK + lane * EPL + j] = kn;
    }
  }
  if (tid < GC) {
    float lg = 0.f, beta = 0.f;
    if (tid < valid) {
      const __nv_bfloat16* pr = proj + (size_t)(row0 + tid) * proj_stride;
      beta = sigmoidf_(bf2f(pr[b_off]));
      lg = -__expf(A_log[h]) * softplusf_(bf2f(pr[a_off]) + dt_bias[h]);
    }
    bs[tid] = beta;
    cs[tid] = lg;
  }
  __syncthreads();
  if (tid == 0) {
    float acc = 0.f;
    for (int t = 0; t < GC; ++t) { acc += cs[t]; cs[t] = acc; }
  }
  __syncthreads();
  if (tid < GC) gc[tid] = cs[tid];

  // Gram products: thread (t, iq) covers i = ii * 4 + iq
  {
    const int t = tid >> 2, iq = tid & 3;
    float gkk[16], gqk[16];
#pragma unroll
    for (int ii = 0; ii < 16; ++ii) { gkk[ii] = 0.f; gqk[ii] = 0.f; }
    for (int kk = 0; kk < DK; kk += 4) {
      const float4 kt = *reinterpret_cast<const float4*>(Ks + t * LDK + kk);
      const float4 qt = *reinterpret_cast<const float4*>(Qs + t * LDK + kk);
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) {
        const float4 ki = *reinterpret_cast<const float4*>(Ks + (ii * 4 + iq) * LDK + kk);
        gkk[ii] = fmaf(kt.x, ki.x, fmaf(kt.y, ki.y, fmaf(kt.z, ki.z, fmaf(kt.w, ki.w, gkk[ii]))));
        gqk[ii] = fmaf(qt.x, ki.x, fmaf(qt.y, ki.y, fmaf(qt.z, ki.z, fmaf(qt.w, ki.w, gqk[ii]))));
      }
    }
    const float ct = cs[t], bt = bs[t];
#pragma unroll
    for (int ii = 0; ii < 16; ++ii) {
      const int i = ii * 4 + iq;
      const float dec = i <= t ? __expf(ct - cs[i]) : 0.f;
      Am[t * LDA + i] = i < t ? bt * dec * gkk[ii] : 0.f;
      gP[t * GC + i] = dec * gqk[ii];
    }
  }
  __syncthreads();
  // T = (I + A)^{-1}: thread j solves column j by forward substitution; T' = T diag(beta)
  if (tid < GC) {
    const int j = tid;
    float x[GC];
#pragma unroll
    for (int t = 0; t < GC; ++t) {
      float a0 = (t == j) ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
      for (int i = 0; i + 1 < t; i += 2) {
        a0 = fmaf(-Am[t * LDA + i], x[i], a0);
        a1 = fmaf(-Am[t * LDA + i + 1], x[i + 1], a1);
      }
      if (t & 1) a0 = fmaf(-Am[t * LDA + t - 1], x[t - 1], a0);
      x[t] = a0 + a1;
    }
    const float bj = bs[j];
#pragma unroll
    for (int t = 0; t < GC; ++t) gT[t * GC + j] = x[t] * bj;
  }
}

// ---- scan ------------------------------------------------------------------------------------------------
// grid (DV / GC_W, nv, nseg); 256 threads; dynamic shared memory = two operand stages + state slice + work arrays.
template <int DK>
struct ScanSmem {
  static constexpr int LDK = DK + 4, LDT = GC + 4;
  static constexpr int STAGE = 2 * GC * LDK + 2 * GC * LDT + GC;       // floats: K, Q, T', P, c
  static constexpr int TOTAL = 2 * STAGE + DK * GC_W + 3 * GC * GC_W;  // + S, B, D, D'
};

template <int DK>
__device__ __forceinline__ void scan_issue_loads(float* st, const float* rec, int tid) {
  using L = ScanSmem<DK>;
  float* Ks = st;
  float* Qs = Ks + GC * L::LDK;
  float* Ts = Qs + GC * L::LDK;
  float* Ps = Ts + GC * L::LDT;
  float* cs = Ps + GC * L::LDT;
  const float* gK = rec;
  const float* gQ = gK + GC * DK;
  const float* gT = gQ + GC * DK;
  const float* gP = gT + GC * GC;
  const float* gc = gP + GC * GC;
  for (int idx = tid; idx < GC * DK / 4; idx += GC_THREADS) {
    const int r = idx / (DK / 4), c4 = idx % (DK / 4);
    gc_cp16(Ks + r * L::LDK + c4 * 4, gK + r * DK + c4 * 4);
    gc_cp16(Qs + r * L::LDK + c4 * 4, gQ + r * DK + c4 * 4);
  }
  for (int idx = tid; idx < GC * GC / 4; idx += GC_THREADS) {
    const int r = idx / (GC / 4), c4 = idx % (GC / 4);
    gc_cp16(Ts + r * L::LDT + c4 * 4, gT + r * GC + c4 * 4);
    gc_cp16(Ps + r * L::LDT + c4 * 4, gP + r * GC + c4 * 4);
  }
  if (tid < GC / 4) gc_cp16(cs + tid * 4, gc + tid * 4);
}

template <int DK>
__global__ void __launch_bounds__(GC_THREADS)
gdn_chunk_scan_kernel(float* __restrict__ y, float* __restrict__ rec_state, __nv_bfloat16* __restrict__ conv_state,
                      const float* __restrict__ scratch, const __nv_bfloat16* __restrict__ qkv,
                      const __nv_bfloat16* __restrict__ proj, long proj_stride, const int* __restrict__ seg_slot,
                      const int* __restrict__ seg_row0, const int* __restrict__ seg_nrows, int nk, int nv, int dv,
                      int commit) {
  pdl_launch_dependents();
  using L = ScanSmem<DK>;
  constexpr int W = GC_W, CK = 4;
  extern __shared__ __align__(16) float sm_scan[];
  float* Ss = sm_scan + 2 * L::STAGE;      // [DK][W] state slice
  float* Bs = Ss + DK * W;                 // [GC][W]  right-hand side
  float* Ds = Bs + GC * W;                 // [GC][W]  deltas
  float* Es = Ds + GC * W;                 // [GC][W]  deltas scaled by e^{c_C - c_i}
  const int slice = blockIdx.x, h = blockIdx.y, seg = blockIdx.z;
  const int tid = threadIdx.x;
  const int n = seg_nrows[seg];
  if (n <= 0) return;
  const int row0 = seg_row0[seg], slot = seg_slot[seg];
  const int kh = h / (nv / nk);
  const int conv_dim = 2 * nk * DK + nv * dv;
  const int v_off = 2 * nk * DK + h * dv + slice * W;
  float* Sg = rec_state + (((size_t)slot * nv + h) * DK) * dv + slice * W;
  pdl_wait();                              // the prep kernel's records (and everything before it on the stream)
  for (int idx = tid; idx < DK * W / 4; idx += GC_THREADS) {
    const int kk = idx / (W / 4), c4 = idx % (W / 4);
    *reinterpret_cast<float4*>(Ss + kk * W + c4 * 4) = *reinterpret_cast<const float4*>(Sg + (size_t)kk * dv + c4 * 4);
  }
  const int nchunks = (n + GC - 1) / GC;
  const size_t rec_stride = (size_t)nv * gc_rec_floats(DK);
  const float* rec0 = scratch + ((size_t)(row0 / GC + seg) * nv + h) * gc_rec_floats(DK);
  scan_issue_loads<DK>(sm_scan, rec0, tid);
  gc_commit();

  const int t = tid >> 2, wq = tid & 3;    // products over rows: thread owns row t, columns wq*4..+3
  const int kk2 = tid >> 1, half = tid & 1;  // state update: thread owns state row kk2, columns half*8..+7
  for (int ch = 0; ch < nchunks; ++ch) {
    float* st = sm_scan + (ch & 1) * L::STAGE;
    const int valid = min(GC, n - ch * GC);
    float vv[4] = {0.f, 0.f, 0.f, 0.f};
    if (t < valid) {
      const uint2 raw = *reinterpret_cast<const uint2*>(qkv + (size_t)(row0 + ch * GC + t) * conv_dim + v_off + wq * 4);
      vv[0] = bf_lo(raw.x); vv[1] = bf_hi(raw.x); vv[2] = bf_lo(raw.y); vv[3] = bf_hi(raw.y);
    }
    gc_wait<0>();
    __syncthreads();                       // stage `ch` landed for everyone; the previous chunk's reads and its new
                                           // state slice are complete, so the other stage can be refilled
    if (ch + 1 < nchunks) {
      scan_issue_loads<DK>(sm_scan + ((ch + 1) & 1) * L::STAGE, rec0 + (size_t)(ch + 1) * rec_stride, tid);
      gc_commit();
    }
    const float* Ks = st;
    const float* Qs = Ks + GC * L::LDK;
    const float* Ts = Qs + GC * L::LDK;
    const float* Ps = Ts + GC * L::LDT;
    const float* cs = Ps + GC * L::LDT;
    // U = K S0, R = Q S0
    float u[4] = {0.f, 0.f, 0.f, 0.f}, r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int kk = 0; kk < DK; kk += 4) {
      const float4 kt = *reinterpret_cast<const float4*>(Ks + t * L::LDK + kk);
      const float4 qt = *reinterpret_cast<const float4*>(Qs + t * L::LDK + kk);
      const float ka[4] = {kt.x, kt.y, kt.z, kt.w}, qa[4] = {qt.x, qt.y, qt.z, qt.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + (kk + e) * W + wq * 4);
        u[0] = fmaf(ka[e], s4.x, u[0]); u[1] = fmaf(ka[e], s4.y, u[1]);
        u[2] = fmaf(ka[e], s4.z, u[2]); u[3] = fmaf(ka[e], s4.w, u[3]);
        r[0] = fmaf(qa[e], s4.x, r[0]); r[1] = fmaf(qa[e], s4.y, r[1]);
        r[2] = fmaf(qa[e], s4.z, r[2]); r[3] = fmaf(qa[e], s4.w, r[3]);
      }
    }
    const float ect = __expf(cs[t]);
    *reinterpret_cast<float4*>(Bs + t * W + wq * 4) =
        make_float4(vv[0] - ect * u[0], vv[1] - ect * u[1], vv[2] - ect * u[2], vv[3] - ect * u[3]);
    __syncthreads();
    // D = T' B (lower triangular)
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i <= t; i += 4) {
      const float4 tt = *reinterpret_cast<const float4*>(Ts + t * L::LDT + i);
      const float ta[4] = {tt.x, tt.y, tt.z, tt.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float4 b4 = *reinterpret_cast<const float4*>(Bs + (i + e) * W + wq * 4);
        d[0] = fmaf(ta[e], b4.x, d[0]); d[1] = fmaf(ta[e], b4.y, d[1]);
        d[2] = fmaf(ta[e], b4.z, d[2]); d[3] = fmaf(ta[e], b4.w, d[3]);
      }
    }
    const float cC = cs[GC - 1];
    const float tail = __expf(cC - cs[t]);
    *reinterpret_cast<float4*>(Ds + t * W + wq * 4) = make_float4(d[0], d[1], d[2], d[3]);
    *reinterpret_cast<float4*>(Es + t * W + wq * 4) = make_float4(d[0] * tail, d[1] * tail, d[2] * tail, d[3] * tail);
    __syncthreads();
    // Y = e^{c} R + P D
    float o[4] = {ect * r[0], ect * r[1], ect * r[2], ect * r[3]};
    for (int i = 0; i <= t; i += 4) {
      const float4 pp = *reinterpret_cast<const float4*>(Ps + t * L::LDT + i);
      const float pa[4] = {pp.x, pp.y, pp.z, pp.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float4 d4 = *reinterpret_cast<const float4*>(Ds + (i + e) * W + wq * 4);
        o[0] = fmaf(pa[e], d4.x, o[0]); o[1] = fmaf(pa[e], d4.y, o[1]);
        o[2] = fmaf(pa[e], d4.z, o[2]); o[3] = fmaf(pa[e], d4.w, o[3]);
      }
    }
    if (t < valid)
      *reinterpret_cast<float4*>(y + ((size_t)(row0 + ch * GC + t) * nv + h) * dv + slice * W + wq * 4) =
          make_float4(o[0], o[1], o[2], o[3]);
    // S = e^{c_C} S0 + K^T D'
    if (kk2 < DK) {
      const float eC = __expf(cC);
      float s[8];
      {
        const float4 a = *reinterpret_cast<const float4*>(Ss + kk2 * W + half * 8);
        const float4 b = *reinterpret_cast<const float4*>(Ss + kk2 * W + half * 8 + 4);
        s[0] = a.x * eC; s[1] = a.y * eC; s[2] = a.z * eC; s[3] = a.w * eC;
        s[4] = b.x * eC; s[5] = b.y * eC; s[6] = b.z * eC; s[7] = b.w * eC;
      }
#pragma unroll 4
      for (int i = 0; i < GC; ++i) {
        const float ki = Ks[i * L::LDK + kk2];
        const float4 a = *reinterpret_cast<const float4*>(Es + i * W + half * 8);
        const float4 b = *reinterpret_cast<const float4*>(Es + i * W + half * 8 + 4);
        s[0] = fmaf(ki, a.x, s[0]); s[1] = fmaf(ki, a.y, s[1]); s[2] = fmaf(ki, a.z, s[2]); s[3] = fmaf(ki, a.w, s[3]);
        s[4] = fmaf(ki, b.x, s[4]); s[5] = fmaf(ki, b.y, s[5]); s[6] = fmaf(ki, b.z, s[6]); s[7] = fmaf(ki, b.w, s[7]);
      }
      *reinterpret_cast<float4*>(Ss + kk2 * W + half * 8) = make_float4(s[0], s[1], s[2], s[3]);
      *reinterpret_cast<float4*>(Ss + kk2 * W + half * 8 + 4) = make_float4(s[4], s[5], s[6], s[7]);
    }
  }
  __syncthreads();
  if (commit) {
    for (int idx = tid; idx < DK * W / 4; idx += GC_THREADS) {
      const int kk = idx / (W / 4), c4 = idx % (W / 4);
      *reinterpret_cast<float4*>(Sg + (size_t)kk * dv + c4 * 4) = *reinterpret_cast<const float4*>(Ss + kk * W + c4 * 4);
    }
    if (slice == 0) {
      // conv tail: the last CK-1 raw inputs of the channels this head owns (q/k channels: first head of the group)
      const int q_off = kh * DK, k_off = nk * DK + kh * DK, vh_off = 2 * nk * DK + h * dv;
      __nv_bfloat16* cst = conv_state + (size_t)slot * (CK - 1) * conv_dim;
      const bool own_qk = (h % (nv / nk)) == 0;
      const int nch = dv + (own_qk ? 2 * DK : 0);
      for (int idx = tid; idx < nch; idx += GC_THREADS) {
        const int c = idx < dv ? vh_off + idx : (idx < dv + DK ? q_off + (idx - dv) : k_off + (idx - dv - DK));
        __nv_bfloat16 nw[CK - 1];
#pragma unroll
        for (int j = 0; j < CK - 1; ++j) {
          const int tt = n - (CK - 1) + j;
          nw[j] = tt >= 0 ? proj[(size_t)(row0 + tt) * proj_stride + c] : cst[(size_t)(CK - 1 + tt) * conv_dim + c];
        }
#pragma unroll
        for (int j = 0; j < CK - 1; ++j) cst[(size_t)j * conv_dim + c] = nw[j];
      }
    }
  }
}

template <int DK>
static int launch_chunk(float* y, float* rec_state, void* conv_state, float* scratch, const void* qkv, const void* proj,
                        long proj_stride, const float* A_log, const float* dt_bias, const int* seg_slot,
                        const int* seg_row0, const int* seg_nrows, int nseg, int max_rows, int nk, int nv, int dv,
                        float eps, int commit, cudaStream_t s) {
  constexpr size_t prep_smem = (size_t)(2 * GC * (DK + 4) + GC * (GC + 1) + 2 * GC) * sizeof(float);
  constexpr size_t scan_smem = (size_t)ScanSmem<DK>::TOTAL * sizeof(float);
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gdn_chunk_prep_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prep_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gdn_chunk_scan_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)scan_smem);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  const int max_chunks = (max_rows + GC - 1) / GC;
  cudaError_t e = launch_pdl(gdn_chunk_prep_kernel<DK>, dim3(max_chunks, nv, nseg), dim3(GC_THREADS), prep_smem, s, scratch,
                             (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)proj, proj_stride, A_log, dt_bias, seg_row0,
                             seg_nrows, nk, nv, dv, eps);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(gdn_chunk_scan_kernel<DK>, dim3(dv / GC_W, nv, nseg), dim3(GC_THREADS), scan_smem, s, y, rec_state,
                 (__nv_bfloat16*)conv_state, (const float*)scratch, (const __nv_bfloat16*)qkv,
                 (const __nv_bfloat16*)proj, proj_stride, seg_slot, seg_row0, seg_nrows, nk, nv, dv, commit);
  return (int)e;
}

}  // namespace fb

using namespace fb;

extern "C" long fb_gdn_chunk_scratch_bytes(int rows, int nseg, int nv, int dk) {
  return ((long)rows / GC + nseg + 1) * nv * gc_rec_floats(dk) * (long)sizeof(float);
}

extern "C" int fb_gdn_chunk(float* y, float* rec_state, void* conv_state, float* scratch, const void* qkv,
                            const void* proj, long proj_stride, const float* A_log, const float* dt_bias,
                            const int* seg_slot, const int* seg_row0, const int* seg_nrows, int nseg, int max_rows,
                            int nk, int nv, int dk, int dv, float eps, int commit, cudaStream_t s) {
  if (nseg <= 0 || max_rows <= 0) return 0;
  if (nv % nk || dv % GC_W || !scratch) return -1;
  if (dk == 128)
    return launch_chunk<128>(y, rec_state, conv_state, scratch, qkv, proj, proj_stride, A_log, dt_bias, seg_slot, seg_row0,
                             seg_nrows, nseg, max_rows, nk, nv, dv, eps, commit, s);
  return -2;
}
