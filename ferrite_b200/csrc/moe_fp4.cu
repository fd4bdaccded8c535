// Routed-expert GEMVs over NVFP4 expert weights (decode rows of the MoE models), and the dequantiser that feeds the
// grouped bf16 tensor-core GEMM on prompt-sized steps.
//
// Layout per expert tensor: e2m1 codes [experts][rows][K/2] (low nibble = even element), one e4m3 scale per 16
// elements [experts][rows][K/16], one fp32 scale for the whole tensor; value = code * block scale * tensor scale.
// A decode step touches top_k experts per token, so expert weights dominate the bytes of an MoE decode step; at 4.5
// bits per weight the pair GEMVs stream 3.5x fewer bytes than the bf16 ones in `moe.cu`, whose structure they keep
// (one CTA = 16 outputs of one (token, expert) pair, activations staged once in shared memory, fp32 partials combined
// in pick order by `moe_combine`).
//
// Counterpart of the reference's low-bit expert GEMVs (`moe_gu` / `moe_down`, `crates/fe-ggq/src/gpu.rs:645,697`, over
// GGUF block formats); the format here is NVFP4 as the 80B-A3B configuration asks.
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"

namespace fb {

constexpr int MF_THREADS = 256;

__device__ __forceinline__ __half2 mf_e2m1x2(uint32_t byte) {
  __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xffu), __NV_E2M1);
  return *reinterpret_cast<__half2*>(&h);
}
__device__ __forceinline__ float mf_e4m3(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(byte & 0xffu), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// 16 weights (8 bytes of codes, one block scale) against 16 staged activations (f16)
__device__ __forceinline__ float mf_dot16(uint2 codes, uint32_t scale_byte, const __half* xs) {
  const uint4 xa = *reinterpret_cast<const uint4*>(xs), xb = *reinterpret_cast<const uint4*>(xs + 8);
  const uint32_t xu[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
  const uint32_t cw[2] = {codes.x, codes.y};
  __half2 s0 = __float2half2_rn(0.f), s1 = __float2half2_rn(0.f);
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    s0 = __hfma2(mf_e2m1x2(cw[j >> 2] >> (8 * (j & 3))), *reinterpret_cast<const __half2*>(&xu[j]), s0);
    s1 = __hfma2(mf_e2m1x2(cw[(j + 1) >> 2] >> (8 * ((j + 1) & 3))), *reinterpret_cast<const __half2*>(&xu[j + 1]), s1);
  }
  const float2 f0 = __half22float2(s0), f1 = __half22float2(s1);
  return ((f0.x + f0.y) + (f1.x + f1.y)) * mf_e4m3(scale_byte);
}

__device__ __forceinline__ uint2 mf_ld8(const unsigned char* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// act[p][j] = silu(Wg[e][j] . x[t]) * (Wu[e][j] . x[t]); W_gu[e] = [2*inter][hidden] (gate rows then up rows)
__global__ void __launch_bounds__(MF_THREADS)
moe_gate_up_fp4_kernel(__nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ x,
                       const unsigned char* __restrict__ wq, const unsigned char* __restrict__ ws, float gscale,
                       const int* __restrict__ ids, int top_k, int hidden, int inter, int e_lo, int e_hi) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) __half xs_mf[];
  pdl_wait();
  const int p = blockIdx.y, e = ids[p];
  if (e < e_lo || e >= e_hi) return;
  const int t = p / top_k;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs_mf[i] = __float2half(bf2f(x[(size_t)t * hidden + i]));
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j0 = blockIdx.x * 16 + warp * 2;
  if (j0 >= inter) return;
  const int j1 = min(j0 + 1, inter - 1);
  const size_t erow = (size_t)(e - e_lo) * 2 * inter;
  const int kb = hidden / 2, ksb = hidden / 16;              // bytes of codes / scales per weight row
  const size_t rows[4] = {erow + j0, erow + inter + j0, erow + j1, erow + inter + j1};   // g0 u0 g1 u1
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int b0 = 0; b0 < ksb; b0 += 64) {                      // two 16-element blocks per lane and pass
    uint2 c[4][2];
    uint32_t s[4][2];
    const int ba = b0 + lane, bb = b0 + 32 + lane;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      c[r][0] = ba < ksb ? mf_ld8(wq + rows[r] * kb + (size_t)ba * 8) : make_uint2(0, 0);
      c[r][1] = bb < ksb ? mf_ld8(wq + rows[r] * kb + (size_t)bb * 8) : make_uint2(0, 0);
      s[r][0] = ba < ksb ? ws[rows[r] * ksb + ba] : 0;
      s[r][1] = bb < ksb ? ws[rows[r] * ksb + bb] : 0;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (ba < ksb) acc[r] += mf_dot16(c[r][0], s[r][0], xs_mf + ba * 16);
      if (bb < ksb) acc[r] += mf_dot16(c[r][1], s[r][1], xs_mf + bb * 16);
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) acc[r] = warp_sum(acc[r]) * gscale;
  if (lane == 0) {
    act[(size_t)p * inter + j0] = f2bf(siluf_(acc[0]) * acc[1]);
    if (j0 + 1 < inter) act[(size_t)p * inter + j0 + 1] = f2bf(siluf_(acc[2]) * acc[3]);
  }
}

// yp[p][n] = Wd[e][n] . act[p]; W_down[e] = [hidden][inter]; fp32 out (zero for pairs of other ranks)
__global__ void __launch_bounds__(MF_THREADS)
moe_down_fp4_kernel(float* __restrict__ yp, const __nv_bfloat16* __restrict__ act, const unsigned char* __restrict__ wq,
                    const unsigned char* __restrict__ ws, float gscale, const int* __restrict__ ids, int hidden, int inter,
                    int e_lo, int e_hi) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) __half as_mf[];
  pdl_wait();
  const int p = blockIdx.y, e = ids[p];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 16 + warp * 2;
  if (e < e_lo || e >= e_hi) {
    if (lane == 0) for (int r = 0; r < 2; ++r) if (n0 + r < hidden) yp[(size_t)p * hidden + n0 + r] = 0.f;
    return;
  }
  for (int i = threadIdx.x; i < inter; i += blockDim.x) as_mf[i] = __float2half(bf2f(act[(size_t)p * inter + i]));
  __syncthreads();
  if (n0 >= hidden) return;
  const int n1 = min(n0 + 1, hidden - 1);
  const size_t erow = (size_t)(e - e_lo) * hidden;
  const int kb = inter / 2, ksb = inter / 16;
  const size_t rows[2] = {erow + n0, erow + n1};
  float acc[2] = {0.f, 0.f};
  for (int b0 = 0; b0 < ksb; b0 += 64) {
    const int ba = b0 + lane, bb = b0 + 32 + lane;
    uint2 c[2][2];
    uint32_t s[2][2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      c[r][0] = ba < ksb ? mf_ld8(wq + rows[r] * kb + (size_t)ba * 8) : make_uint2(0, 0);
      c[r][1] = bb < ksb ? mf_ld8(wq + rows[r] * kb + (size_t)bb * 8) : make_uint2(0, 0);
      s[r][0] = ba < ksb ? ws[rows[r] * ksb + ba] : 0;
      s[r][1] = bb < ksb ? ws[rows[r] * ksb + bb] : 0;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (ba < ksb) acc[r] += mf_dot16(c[r][0], s[r][0], as_mf + ba * 16);
      if (bb < ksb) acc[r] += mf_dot16(c[r][1], s[r][1], as_mf + bb * 16);
    }
  }
  acc[0] = warp_sum(acc[0]) * gscale;
  acc[1] = warp_sum(acc[1]) * gscale;
  if (lane == 0) {
    yp[(size_t)p * hidden + n0] = acc[0];
    if (n0 + 1 < hidden) yp[(size_t)p * hidden + n0 + 1] = acc[1];
  }
}

// out[row][k] (bf16) = code * block scale * tensor scale; one thread per 16-element block
__global__ void nvfp4_dequant_kernel(__nv_bfloat16* __restrict__ out, const unsigned char* __restrict__ wq,
                                     const unsigned char* __restrict__ ws, float gscale, long blocks) {
  const long b = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= blocks) return;
  const uint2 c = mf_ld8(wq + b * 8);
  const float sc = mf_e4m3(ws[b]) * gscale;
  const uint32_t cw[2] = {c.x, c.y};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 f = __half22float2(mf_e2m1x2(cw[j >> 2] >> (8 * (j & 3))));
    __nv_bfloat162 h = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    o[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

}  // namespace fb

using namespace fb;

extern "C" int fb_moe_gate_up_fp4(void* act, const void* x, const void* wq, const void* ws, float gscale, const int* ids,
                                  int pairs, int top_k, int hidden, int inter, int e_lo, int e_hi, cudaStream_t s) {
  if (pairs <= 0) return 0;
  if (hidden % 16 || inter <= 0) return -1;
  launch_pdl(moe_gate_up_fp4_kernel, dim3((inter + 15) / 16, pairs), dim3(MF_THREADS), (size_t)hidden * 2, s,
             (__nv_bfloat16*)act, (const __nv_bfloat16*)x, (const unsigned char*)wq, (const unsigned char*)ws, gscale, ids,
             top_k, hidden, inter, e_lo, e_hi);
  return (int)cudaGetLastError();
}

extern "C" int fb_moe_down_fp4(float* yp, const void* act, const void* wq, const void* ws, float gscale, const int* ids,
                               int pairs, int hidden, int inter, int e_lo, int e_hi, cudaStream_t s) {
  if (pairs <= 0) return 0;
  if (inter % 16) return -1;
  launch_pdl(moe_down_fp4_kernel, dim3((hidden + 15) / 16, pairs), dim3(MF_THREADS), (size_t)inter * 2, s, yp,
             (const __nv_bfloat16*)act, (const unsigned char*)wq, (const unsigned char*)ws, gscale, ids, hidden, inter, e_lo,
             e_hi);
  return (int)cudaGetLastError();
}

extern "C" int fb_nvfp4_dequant(void* out, const void* wq, const void* ws, float gscale, long elements, cudaStream_t s) {
  if (elements <= 0) return 0;
  if (elements % 16) return -1;
  const long blocks = elements / 16;
  nvfp4_dequant_kernel<<<(unsigned)((blocks + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)out, (const unsigned char*)wq,
                                                                        (const unsigned char*)ws, gscale, blocks);
  return (int)cudaGetLastError();
}
