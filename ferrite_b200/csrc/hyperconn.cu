// Hyper-connection kernels: a block's residual is kept as `hc` parallel streams per token; a block reads a gated mix of
// the normalised streams and its output is injected back into every stream with a learned per-stream weight.
//
//   hc_norm     y[g][i]      = bf16(x[g][i] * inv_g * w[(g % ngw)][i]),  inv_g = rsqrt(mean_i x[g][i]^2 + eps),  g = row * hc + s
//   hc_mix      mixed[r][i]  = mean_s( res[r][s][i] * inv[r * hc + s] * w[s][i] * sigmoid(gate[r][s][i]) )
//   hc_combine  res[r][s][i] += out[r][i] * 2 * sigmoid(inj[r][s])
//   engram_gate out[r][s][:] = bf16(h[r][s][:] + gate * value[r][:]),  gate = sigmoid(signed_sqrt(max(|dot|, 1e-6))),
//               dot = <h[r][s] * qk[s], key[r][s]> * rstd(h[r][s]) * rstd(key[r][s]) / sqrt(d); key / value are the
//               (hc + 1) slices of a memory lookup's projection, given summed (bf16) or as per-rank fp32 partials that
//               are summed here in rank order and rounded to bf16 first
//
// Residual streams are fp32 (they accumulate over every block of the model). Counterparts of the reference's
// `fx_hc_norm_bf16`, `fx_hc_mix_res` and `fx_hc_combine` (`kernels/k-fnext/src/fast.rs:1010,1039,768`) and `engram_gate`
// (`kernels/k-engram/src/lib.rs:38`); the models of this
// repo's presets do not use hyper-connections, the ops are provided for checkpoints of that family.
#include "api_ext.h"
#include "common.cuh"

namespace fb {

__global__ void __launch_bounds__(256) hc_norm_kernel(__nv_bfloat16* __restrict__ y, float* __restrict__ rinv,
                                                       const float* __restrict__ x, const float* __restrict__ w, int d,
                                                       int ngw, float eps) {
  __shared__ float red[32];
  const int g = blockIdx.x;
  const float* xr = x + (size_t)g * d;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / (float)d + eps);
  if (threadIdx.x == 0) rinv[g] = inv;
  const float* wr = w + (size_t)(g % ngw) * d;
  for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i), ww = *reinterpret_cast<const float4*>(wr + i);
    *reinterpret_cast<uint2*>(y + (size_t)g * d + i) =
        make_uint2(pack_bf2(v.x * inv * ww.x, v.y * inv * ww.y), pack_bf2(v.z * inv * ww.z, v.w * inv * ww.w));
  }
}

__global__ void hc_mix_kernel(float* __restrict__ mixed, const float* __restrict__ res, const float* __restrict__ rinv,
                              const float* __restrict__ w, const float* __restrict__ gate, long n, int d, int hc) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const long r = idx / d;
  const int i = (int)(idx % d);
  float acc = 0.f;
  for (int s = 0; s < hc; ++s) {
    const size_t e = ((size_t)r * hc + s) * d + i;
    acc += res[e] * rinv[r * hc + s] * w[(size_t)s * d + i] * sigmoidf_(gate[e]);
  }
  mixed[idx] = acc / (float)hc;
}

__global__ void hc_combine_kernel(float* __restrict__ res, const float* __restrict__ out, const float* __restrict__ inj,
                                  long n, int d, int hc, long ldi) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const int i = (int)(idx % d);
  const long rs = idx / d;
  const long r = rs / hc;
  const int s = (int)(rs % hc);
  res[idx] += out[r * d + i] * 2.f * sigmoidf_(inj[r * ldi + s]);
}

// grid = (rows, hc), 256 threads. h / out [rows][hc][d] bf16; kvb bf16 [rows][(hc + 1) d] or kvp fp32 [world][rows][(hc + 1) d].
__global__ void __launch_bounds__(256) engram_gate_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ h,
                                                          const float* __restrict__ kvp, const __nv_bfloat16* __restrict__ kvb,
                                                          const float* __restrict__ qk, int rows, int hc, int d, int world,
                                                          float eps) {
  __shared__ float red[3][32];
  const int r = blockIdx.x, s = blockIdx.y;
  const size_t wd = (size_t)(hc + 1) * d, part = (size_t)rows * wd;
  auto kv_at = [&](size_t i) -> float {
    if (world == 0) return __bfloat162float(kvb[(size_t)r * wd + i]);
    float acc = kvp[(size_t)r * wd + i];
    for (int k = 1; k < world; ++k) acc += kvp[(size_t)k * part + (size_t)r * wd + i];
    return __bfloat162float(__float2bfloat16(acc));
  };
  const __nv_bfloat16* hrow = h + ((size_t)r * hc + s) * d;
  float sh = 0.f, sk = 0.f, sd = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float x = __bfloat162float(hrow[i]), k = kv_at((size_t)s * d + i);
    sh = fmaf(x, x, sh);
    sk = fmaf(k, k, sk);
    sd = fmaf(x * qk[(size_t)s * d + i], k, sd);
  }
  sh = block_sum(sh, red[0]);
  sk = block_sum(sk, red[1]);
  sd = block_sum(sd, red[2]);
  const float df = (float)d;
  const float dot = sd * rsqrtf(sh / df + eps) * rsqrtf(sk / df + eps) * rsqrtf(df);
  const float mag = sqrtf(fmaxf(fabsf(dot), 1e-6f));
  const float gate = sigmoidf_(dot < 0.f ? -mag : mag);
  __nv_bfloat16* orow = out + ((size_t)r * hc + s) * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    orow[i] = __float2bfloat16(__bfloat162float(hrow[i]) + gate * kv_at((size_t)hc * d + i));
}

}  // namespace fb

using namespace fb;

extern "C" int fb_engram_gate(void* out, const void* h, const float* kvp, const void* kvb, const float* qk, int rows, int hc,
                              int d, int world, float eps, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (hc < 1 || hc > 65535 || (world == 0 ? !kvb : !kvp)) return -1;
  engram_gate_kernel<<<dim3(rows, hc), 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)h, kvp,
                                                    (const __nv_bfloat16*)kvb, qk, rows, hc, d, world, eps);
  return (int)cudaGetLastError();
}


extern "C" int fb_hc_norm(void* y, float* rinv, const float* x, const float* w, int groups, int d, int ngw, float eps,
                          cudaStream_t s) {
  if (groups <= 0) return 0;
  if (d % 4 || ngw <= 0) return -1;
  hc_norm_kernel<<<groups, 256, 0, s>>>((__nv_bfloat16*)y, rinv, x, w, d, ngw, eps);
  return (int)cudaGetLastError();
}

extern "C" int fb_hc_mix(float* mixed, const float* res, const float* rinv, const float* w, const float* gate, int rows,
                         int d, int hc, cudaStream_t s) {
  const long n = (long)rows * d;
  if (n <= 0) return 0;
  hc_mix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(mixed, res, rinv, w, gate, n, d, hc);
  return (int)cudaGetLastError();
}

extern "C" int fb_hc_combine(float* res, const float* out, const float* inj, int rows, int d, int hc, long ldi,
                             cudaStream_t s) {
  const long n = (long)rows * hc * d;
  if (n <= 0) return 0;
  hc_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(res, out, inj, n, d, hc, ldi);
  return (int)cudaGetLastError();
}
