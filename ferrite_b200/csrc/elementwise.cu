// Row-wise glue kernels: embedding gather, RMSNorm (with the pending residual add folded in), SiLU*mul,
// gated per-head RMSNorm, row gathers, casts and adds. All are bandwidth-bound SIMT kernels with 128-bit IO.
// Counterparts in the reference: `fe_embed`, `fe_rmsnorm`, `fe_silu_mul`, `fe_gather_rows`, `fe_bf16_to_f32`,
// `fe_add_bf16` (`kernels/k-core/src/misc.rs:7-179`) and `fe_gdn_norm` (`kernels/k-core/src/gdn.rs:417`).
#include "api.h"
#include "common.cuh"

namespace fb {

__global__ void embed_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ table,
                             const int* __restrict__ ids, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = __ldg(src + i);
}

// out = bf16( x' * rsqrt(mean(x'^2) + eps) * (centred ? 1 + w : w) ), x' = x (+ res). When res != null the sum
// x' is also written back to x_out (the residual stream), so a block's output add costs no extra pass.
__global__ void rmsnorm_kernel(__nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ x_out,
                               const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                               const __nv_bfloat16* __restrict__ w, int hidden, float eps, int centred) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];          // hidden floats
  __shared__ float scratch[32];
  int row = blockIdx.x;
  const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)row * hidden);
  const uint4* rp = res ? reinterpret_cast<const uint4*>(res + (size_t)row * hidden) : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    uint4 a = xp[i];
    uint32_t u[4] = {a.x, a.y, a.z, a.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[2 * j] = bf_lo(u[j]); v[2 * j + 1] = bf_hi(u[j]); }
    if (rp) {
      uint4 b = rp[i];
      uint32_t ub[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the residual stream is bf16: round the sum before it is normalised, as a separate add kernel would
        v[2 * j] = bf2f(f2bf(v[2 * j] + bf_lo(ub[j])));
        v[2 * j + 1] = bf2f(f2bf(v[2 * j + 1] + bf_hi(ub[j])));
      }
      uint4 o;
      o.x = pack_bf2(v[0], v[1]); o.y = pack_bf2(v[2], v[3]); o.z = pack_bf2(v[4], v[5]); o.w = pack_bf2(v[6], v[7]);
      reinterpret_cast<uint4*>(x_out + (size_t)row * hidden)[i] = o;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { xs[i * 8 + j] = v[j]; ss += v[j] * v[j]; }
  }
  float tot = block_sum(ss, scratch);
  float r = rsqrtf(tot / (float)hidden + eps);
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    uint4 a = __ldg(wp + i);
    uint32_t u[4] = {a.x, a.y, a.z, a.w};
    float o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float w0 = bf_lo(u[j]), w1 = bf_hi(u[j]);
      if (centred) { w0 += 1.f; w1 += 1.f; }
      o[2 * j] = xs[i * 8 + 2 * j] * r * w0;
      o[2 * j + 1] = xs[i * 8 + 2 * j + 1] * r * w1;
    }
    uint4 ov;
    ov.x = pack_bf2(o[0], o[1]); ov.y = pack_bf2(o[2], o[3]); ov.z = pack_bf2(o[4], o[5]); ov.w = pack_bf2(o[6], o[7]);
    reinterpret_cast<uint4*>(out + (size_t)row * hidden)[i] = ov;
  }
}

// out[r][i] = silu(gu[r][i]) * gu[r][inter + i]
__global__ void silu_mul_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu, int inter,
                                float clamp) {
  int row = blockIdx.y;
  int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= inter) return;
  uint4 g = *reinterpret_cast<const uint4*>(gu + (size_t)row * 2 * inter + i);
  uint4 u = *reinterpret_cast<const uint4*>(gu + (size_t)row * 2 * inter + inter + i);
  uint32_t ga[4] = {g.x, g.y, g.z, g.w}, ua[4] = {u.x, u.y, u.z, u.w}, o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float g0 = bf_lo(ga[j]), g1 = bf_hi(ga[j]), u0 = bf_lo(ua[j]), u1 = bf_hi(ua[j]);
    if (clamp > 0.f) {
      g0 = fminf(g0, clamp); g1 = fminf(g1, clamp);
      u0 = fminf(fmaxf(u0, -clamp), clamp); u1 = fminf(fmaxf(u1, -clamp), clamp);
    }
    o[j] = pack_bf2(siluf_(g0) * u0, siluf_(g1) * u1);
  }
  *reinterpret_cast<uint4*>(out + (size_t)row * inter + i) = make_uint4(o[0], o[1], o[2], o[3]);
}

// Gated per-head RMSNorm of the GDN output: out[r][h][d] = bf16( y * rsqrt(mean_d y^2 + eps) * w[d] * silu(z) ).
// y is fp32 [rows][heads][dv]; z is a bf16 column block of the fused projection (row stride z_stride).
__global__ void gated_norm_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ y,
                                  const __nv_bfloat16* __restrict__ z, long z_stride,
                                  const __nv_bfloat16* __restrict__ w, int heads, int dv, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  int row = blockIdx.x;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int nw = blockDim.x >> 5;
  for (int h = warp; h < heads; h += nw) {
    const float* yp = y + ((size_t)row * heads + h) * dv;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) { float v = yp[d]; ss += v * v; }
    ss = warp_sum(ss);
    float r = rsqrtf(ss / (float)dv + eps);
    const __nv_bfloat16* zp = z + (size_t)row * z_stride + (size_t)h * dv;
    for (int d = lane; d < dv; d += 32) {
      float v = yp[d] * r * bf2f(w[d]) * siluf_(bf2f(zp[d]));
      out[((size_t)row * heads + h) * dv + d] = f2bf(v);
    }
  }
}

__global__ void gather_rows_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in,
                                   const int* __restrict__ idx, int width) {
  int row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(in + (size_t)idx[row] * width);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * width);
  for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void add_bf16_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y, long n) {
  long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  uint4 a = *reinterpret_cast<const uint4*>(x + i), b = *reinterpret_cast<const uint4*>(y + i);
  uint32_t ua[4] = {a.x, a.y, a.z, a.w}, ub[4] = {b.x, b.y, b.z, b.w}, o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = pack_bf2(bf_lo(ua[j]) + bf_lo(ub[j]), bf_hi(ua[j]) + bf_hi(ub[j]));
  *reinterpret_cast<uint4*>(x + i) = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void bf16_to_f32_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ in, long n) {
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = bf2f(in[i]);
}

}  // namespace fb

using namespace fb;

extern "C" int fb_embed(void* out, const void* table, const int* ids, int rows, int hidden, int vocab, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (hidden % 8) return -1;
  launch_pdl(embed_kernel, dim3(rows), dim3(256), (size_t)(0), s, (__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids, hidden, vocab);
  return (int)cudaGetLastError();
}

extern "C" int fb_rmsnorm(void* out, void* x_out, const void* x, const void* res, const void* w, int rows, int hidden,
                          float eps, int centred, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (hidden % 8) return -1;
  size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int threads = hidden >= 4096 ? 512 : 256;
  launch_pdl(rmsnorm_kernel, dim3(rows), dim3(threads), (size_t)(smem), s, (__nv_bfloat16*)out, (__nv_bfloat16*)x_out, (const __nv_bfloat16*)x,
                                             (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, hidden, eps, centred);
  return (int)cudaGetLastError();
}

extern "C" int fb_silu_mul(void* out, const void* gu, int rows, int inter, float clamp, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (inter % 8) return -1;
  dim3 grid((inter / 8 + 255) / 256, rows);
  silu_mul_kernel<<<grid, 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gu, inter, clamp);
  return (int)cudaGetLastError();
}

extern "C" int fb_gated_norm(void* out, const float* y, const void* z, long z_stride, const void* w, int rows,
                             int heads, int dv, float eps, cudaStream_t s) {
  if (rows <= 0) return 0;
  int threads = heads >= 8 ? 256 : 32 * heads;
  launch_pdl(gated_norm_kernel, dim3(rows), dim3(threads), (size_t)(0), s, (__nv_bfloat16*)out, y, (const __nv_bfloat16*)z, z_stride,
                                             (const __nv_bfloat16*)w, heads, dv, eps);
  return (int)cudaGetLastError();
}

extern "C" int fb_gather_rows(void* out, const void* in, const int* idx, int rows, int width, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (width % 8) return -1;
  gather_rows_kernel<<<rows, 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, idx, width);
  return (int)cudaGetLastError();
}

extern "C" int fb_add_bf16(void* x, const void* y, long n, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n % 8) return -1;
  add_bf16_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)y, n);
  return (int)cudaGetLastError();
}

extern "C" int fb_bf16_to_f32(float* out, const void* in, long n, cudaStream_t s) {
  if (n <= 0) return 0;
  bf16_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out, (const __nv_bfloat16*)in, n);
  return (int)cudaGetLastError();
}
