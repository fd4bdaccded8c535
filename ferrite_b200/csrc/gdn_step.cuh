// One decode-row step of a Gated DeltaNet head as a device function, shared by the stand-alone kernel (`gdn.cu`) and the
// persistent decode-layer kernel (`decode_layer.cu`).
#pragma once
#include "common.cuh"

namespace fb {

// Decode-row fusion of the three kernels above: causal conv + SiLU of this head's q / k / v channels, the delta-rule
// recurrence, and the gated per-head RMSNorm (y * rsqrt(mean y^2 + eps) * w * silu(z)) in one pass.
// Same arithmetic as the separate kernels (the conv output is rounded to bf16 as it would be when stored), so both
// paths agree to fp32 rounding of the norm's sum. blockDim = DV * 8 as in gdn_rec_kernel.
// Called by all DV * PARTS threads of a CTA for head h and the segment (n rows from row0, state slot `slot`).
template <int DK, int DV, int PARTS>
__device__ __forceinline__ void gdn_step_body(__nv_bfloat16* __restrict__ out, float* __restrict__ rec_state,
                                              __nv_bfloat16* __restrict__ conv_state, const __nv_bfloat16* __restrict__ proj,
                                              long proj_stride, const __nv_bfloat16* __restrict__ conv_w,
                                              const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                              const __nv_bfloat16* __restrict__ gnorm_w, int n, int row0, int slot, int h,
                                              int nk, int nv, float eps, int commit) {
  constexpr int RP = DK / PARTS, CK = 4;
  __shared__ __align__(16) float qs[DK], ks[DK], vs[DV];
  __shared__ float red1[PARTS][DV], red2[PARTS][DV];
  __shared__ float ssq[2][DK / 32], ssn[DV / 32];
  const int tid = threadIdx.x, col = tid % DV, part = tid / DV;
  if (n <= 0) return;
  const int kh = h / (nv / nk);
  const int conv_dim = 2 * nk * DK + nv * DV;
  const int q_off = kh * DK, k_off = nk * DK + kh * DK, v_off = 2 * nk * DK + h * DV;
  const int z_off = conv_dim + h * DV;
  const int b_off = conv_dim + nv * DV + h, a_off = b_off + nv;
  float* Sg = rec_state + (((size_t)slot * nv + h) * DK) * DV;
  __nv_bfloat16* st = conv_state + (size_t)slot * (CK - 1) * conv_dim;
  float S[RP];
#pragma unroll
  for (int i = 0; i < RP; ++i) S[i] = Sg[(size_t)(part * RP + i) * DV + col];
  const float expA = __expf(A_log[h]);
  const float dtb = dt_bias[h];
  const float qscale = rsqrtf((float)DK);
  // conv roles: threads [0, DK) produce the q channels, [DK, 2 DK) the k channels, [2 DK, 2 DK + DV) the v channels
  // (one channel and one sliding window per thread, so the three convs of a row run side by side)
  static_assert(2 * DK + DV <= DV * PARTS, "block too small for the conv roles");
  const int crole = tid < DK ? 0 : (tid < 2 * DK ? 1 : (tid < 2 * DK + DV ? 2 : -1));
  const int cch = crole == 0 ? q_off + tid : (crole == 1 ? k_off + tid - DK : v_off + tid - 2 * DK);   // channel in the row
  const int cidx = crole == 0 ? tid : (crole == 1 ? tid - DK : tid - 2 * DK);                           // index in qs / ks / vs
  float cw[CK], cwin[CK - 1];
  if (crole >= 0) {
#pragma unroll
    for (int j = 0; j < CK; ++j) cw[j] = bf2f(conv_w[(size_t)cch * CK + j]);
#pragma unroll
    for (int j = 0; j < CK - 1; ++j) cwin[j] = bf2f(st[(size_t)j * conv_dim + cch]);
  }
  const float gw = bf2f(gnorm_w[col]);

  // The rows of a segment are sequential, so a row's inputs are fetched while the row before it is computed: without
  // this every row paid a full global-memory round trip before its first FMA (3.2 us per row on B200, 55 us for a
  // 17-row verify segment).
  struct RowIn { float x, b, a, z; };
  auto fetch = [&](int r) {
    RowIn in = {0.f, 0.f, 0.f, 0.f};
    const __nv_bfloat16* pr = proj + (size_t)(row0 + r) * proj_stride;
    if (crole >= 0) in.x = bf2f(pr[cch]);
    in.b = bf2f(pr[b_off]); in.a = bf2f(pr[a_off]);
    if (part == 0) in.z = bf2f(pr[z_off + col]);
    return in;
  };
  RowIn nxt = fetch(0);
  for (int r = 0; r < n; ++r) {
    const RowIn cur = nxt;
    if (r + 1 < n) nxt = fetch(r + 1);
    if (crole >= 0) {
      const float cv = bf2f(f2bf(siluf_(cw[0] * cwin[0] + cw[1] * cwin[1] + cw[2] * cwin[2] + cw[3] * cur.x)));
      cwin[0] = cwin[1]; cwin[1] = cwin[2]; cwin[2] = cur.x;
      if (crole == 2) {
        vs[cidx] = cv;
      } else {                                               // warps are uniform in their role (DK is a multiple of 32)
        (crole == 0 ? qs : ks)[cidx] = cv;
        const float sq2 = warp_sum(cv * cv);
        if ((tid & 31) == 0) ssq[crole][cidx >> 5] = sq2;
      }
    }
    __syncthreads();
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int i = 0; i < DK / 32; ++i) { sq += ssq[0][i]; sk += ssq[1][i]; }
    const float rq = rsqrtf(sq + eps) * qscale, rk = rsqrtf(sk + eps);
    const float beta = sigmoidf_(cur.b);
    const float g = __expf(-expA * softplusf_(cur.a + dtb));
    // k and q are read as float4 (one shared-memory instruction per four FMAs: with one word per FMA the 16 warps of
    // the CTA spent 640 + 980 cycles per row in the load / store unit); the FMA order is unchanged
    const float4* k4 = reinterpret_cast<const float4*>(ks + part * RP);
    const float4* q4 = reinterpret_cast<const float4*>(qs + part * RP);
    float p = 0.f;
#pragma unroll
    for (int i = 0; i < RP / 4; ++i) {
      const float4 kk = k4[i];
      p = fmaf(S[4 * i], kk.x, p); p = fmaf(S[4 * i + 1], kk.y, p); p = fmaf(S[4 * i + 2], kk.z, p); p = fmaf(S[4 * i + 3], kk.w, p);
    }
    red1[part][col] = p;
    __syncthreads();
    float kvv = 0.f;
#pragma unroll
    for (int i = 0; i < PARTS; ++i) kvv += red1[i][col];
    kvv *= g * rk;
    const float delta = (vs[col] - kvv) * beta;
    float yp = 0.f;
#pragma unroll
    for (int i = 0; i < RP / 4; ++i) {
      const float4 kk = k4[i], qq = q4[i];
      const float kx[4] = {kk.x, kk.y, kk.z, kk.w}, qx[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        S[4 * i + e] = fmaf(kx[e] * rk, delta, S[4 * i + e] * g);
        yp = fmaf(S[4 * i + e], qx[e], yp);
      }
    }
    red2[part][col] = yp;
    __syncthreads();
    float yy = 0.f;
    if (part == 0) {
#pragma unroll
      for (int i = 0; i < PARTS; ++i) yy += red2[i][col];
      yy *= rq;
      const float s2 = warp_sum(yy * yy);
      if ((tid & 31) == 0) ssn[tid >> 5] = s2;
    }
    __syncthreads();
    if (part == 0) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < DV / 32; ++i) ss += ssn[i];
      const float rn = rsqrtf(ss / (float)DV + eps);
      out[((size_t)(row0 + r) * nv + h) * DV + col] = f2bf(yy * rn * gw * siluf_(cur.z));
    }
  }
  if (commit) {
#pragma unroll
    for (int i = 0; i < RP; ++i) Sg[(size_t)(part * RP + i) * DV + col] = S[i];
    // conv tail = the windows after the last row (q / k channels: first head of the group writes them)
    const bool own_qk = (h % (nv / nk)) == 0;
    if (crole == 2 || (crole >= 0 && own_qk)) {
#pragma unroll
      for (int j = 0; j < CK - 1; ++j) st[(size_t)j * conv_dim + cch] = f2bf(cwin[j]);
    }
  }
}

}  // namespace fb
