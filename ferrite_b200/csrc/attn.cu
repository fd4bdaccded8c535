// GQA attention over a paged KV cache: attn-prep (q/k RMSNorm + partial RoPE + KV page write), split-KV
// decode / verify / tree attention, and the fixed-order merge with the sigmoid output gate.
//
// Counterparts in the reference: `fe_attn_prep` (`kernels/k-core/src/attn.rs:17`), `fe_attn_split` +
// `fe_attn_combine` (`:99`, `:219`) and the tree masks of `fe_attn_vk` (`:331`). Differences: the cache is
// paged (a block table per slot, so parking a sequence is a table move), heads and head_dim are run-time /
// template parameters rather than compiled-in dims, and split boundaries depend only on the row's own
// length so a row's result does not depend on what else is in the batch.
#include <cuda_fp8.h>

#include "api.h"
#include "common.cuh"

namespace fb {

// ---------------------------------------------------------------------------------------------------
// attn-prep. One CTA per row, one warp per head (q heads first, then kv heads). The fused projection row is
// [per q head: q(hd) | gate(hd)] [k heads] [v heads].
template <int HD, int KVM>
__global__ void attn_prep_kernel(__nv_bfloat16* __restrict__ q_out, void* __restrict__ k_cache_v,
                                 void* __restrict__ v_cache_v, float* __restrict__ kv_scale,
                                 const __nv_bfloat16* __restrict__ proj,
                                 long proj_stride, const __nv_bfloat16* __restrict__ q_norm,
                                 const __nv_bfloat16* __restrict__ k_norm, const float* __restrict__ inv_freq,
                                 const int* __restrict__ row_slot, const int* __restrict__ row_pos,
                                 const int* __restrict__ row_cpos,
                                 const int* __restrict__ block_table, int max_blocks, int kv_block, int nq, int nkv,
                                 int rot, int gated, float eps, int* status, int hrot) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int EPL = HD / 32;
  const int row = blockIdx.x;
  // one warp per (q or kv) head; blockIdx.y carries the heads beyond the first 32
  const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (warp >= nq + nkv) return;
  const bool is_q = warp < nq;
  const int qw = gated ? 2 * HD : HD;
  const __nv_bfloat16* src = proj + (size_t)row * proj_stride + (is_q ? (size_t)warp * qw : (size_t)nq * qw + (size_t)(warp - nq) * HD);
  float v[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) v[j] = bf2f(src[lane * EPL + j]);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < EPL; ++j) ss += v[j] * v[j];
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)HD + eps);
  const __nv_bfloat16* nw = is_q ? q_norm : k_norm;
#pragma unroll
  for (int j = 0; j < EPL; ++j) v[j] = v[j] * r * (1.f + bf2f(nw[lane * EPL + j]));
  // partial RoPE, rotate-half pairing (i, i + rot/2) inside the first `rot` dims
  const int pos = row_pos[row];
  const int half = rot / 2;
  const int partner_lanes = half / EPL;                  // lane distance between the two halves of a pair
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    float other = __shfl_xor_sync(0xffffffffu, v[j], partner_lanes);
    int d = lane * EPL + j;
    if (d < rot) {
      int i = d < half ? d : d - half;
      float ang = (float)pos * inv_freq[i];
      float sn, cs;
      sincosf(ang, &sn, &cs);
      v[j] = d < half ? (v[j] * cs - other * sn) : (v[j] * cs + other * sn);
    }
  }
  if (hrot) {
    // Walsh-Hadamard rotation of the head (queries and keys alike, so q . k is unchanged): it spreads a few large
    // channels over all of them before the keys are quantised. Element d = lane * EPL + j: the low bits of d are
    // register indices, the high five bits the lane. Values stay unrotated.
#pragma unroll
    for (int st = 1; st < EPL; st <<= 1) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        if (!(j & st)) { const float a = v[j], b = v[j | st]; v[j] = a + b; v[j | st] = a - b; }
      }
    }
#pragma unroll
    for (int o2 = 1; o2 < 32; o2 <<= 1) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], o2);
        v[j] = (lane & o2) ? other - v[j] : v[j] + other;
      }
    }
    const float hs = rsqrtf((float)HD);
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] *= hs;
  }
  if (is_q) {
    __nv_bfloat16* dst = q_out + ((size_t)row * nq + warp) * HD;
#pragma unroll
    for (int j = 0; j < EPL; ++j) dst[lane * EPL + j] = f2bf(v[j]);
  } else {
    const int kvh = warp - nq;
    const int slot = row_slot[row];
    // rows of a verify tree rotate by their depth but are stored by their row index: siblings share a position
    const int cpos = row_cpos ? row_cpos[row] : pos;
    const int blk = block_table[(size_t)slot * max_blocks + cpos / kv_block];
    if (blk < 0) { set_status(status, ST_BOUNDS); return; }
    const size_t tok = ((size_t)blk * kv_block + (cpos % kv_block)) * nkv + kvh;
    const size_t off = tok * HD;
    const __nv_bfloat16* vsrc = proj + (size_t)row * proj_stride + (size_t)nq * qw + (size_t)(nkv + kvh) * HD;
    if (KVM == 3) {
      // 6-bit codes (value = (code - 32) * scale, scale = group amax / 31) with one fp32 scale per 32 elements, packed
      // little-endian: element d of a row owns bits [6 d, 6 d + 6) of its hd * 3 / 4 bytes
      constexpr int NG = HD / 32, GL = 32 / EPL;
      unsigned char* kc6 = reinterpret_cast<unsigned char*>(k_cache_v) + tok * (HD * 3 / 4);
      unsigned char* vc6 = reinterpret_cast<unsigned char*>(v_cache_v) + tok * (HD * 3 / 4);
      float vv[EPL], ka = 0.f, va = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) { vv[j] = bf2f(vsrc[lane * EPL + j]); ka = fmaxf(ka, fabsf(v[j])); va = fmaxf(va, fabsf(vv[j])); }
#pragma unroll
      for (int o2 = GL / 2; o2 > 0; o2 >>= 1) {
        ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o2));
        va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o2));
      }
      const float ks = ka > 0.f ? ka / 31.f : 1.f, vs = va > 0.f ? va / 31.f : 1.f;
      auto code = [](float x, float sc) { return (unsigned long long)(min(31, max(-32, __float2int_rn(x / sc))) + 32); };
      unsigned long long kb = 0ull, vb = 0ull;
#pragma unroll
      for (int j = 0; j < EPL; ++j) { kb |= code(v[j], ks) << (6 * j); vb |= code(vv[j], vs) << (6 * j); }
      if (EPL == 2) {
        // 12 bits per lane: an even lane writes its own and its right neighbour's codes as three bytes
        const unsigned long long ko = __shfl_down_sync(0xffffffffu, kb, 1), vo = __shfl_down_sync(0xffffffffu, vb, 1);
        kb |= ko << 12; vb |= vo << 12;
        if (!(lane & 1)) {
#pragma unroll
          for (int b = 0; b < 3; ++b) {
            kc6[lane / 2 * 3 + b] = (unsigned char)(kb >> (8 * b));
            vc6[lane / 2 * 3 + b] = (unsigned char)(vb >> (8 * b));
          }
        }
      } else {
        constexpr int NB = EPL * 6 / 8;                     // 3 bytes (4 elements) or 6 bytes (8 elements) per lane
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          kc6[lane * NB + b] = (unsigned char)(kb >> (8 * b));
          vc6[lane * NB + b] = (unsigned char)(vb >> (8 * b));
        }
      }
      if (lane % GL == 0) {
        kv_scale[tok * 2 * NG + lane / GL] = ks;
        kv_scale[tok * 2 * NG + NG + lane / GL] = vs;
      }
    } else if (KVM == 2) {
      // 4-bit codes (value = (code - 8) * scale) with one fp32 scale per 32 elements: scales of a (token, kv head) row
      // are [K groups | V groups]
      constexpr int NG = HD / 32, GL = 32 / EPL;                 // groups per row, lanes per group
      unsigned char* kc4 = reinterpret_cast<unsigned char*>(k_cache_v);
      unsigned char* vc4 = reinterpret_cast<unsigned char*>(v_cache_v);
      float vv[EPL], ka = 0.f, va = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) { vv[j] = bf2f(vsrc[lane * EPL + j]); ka = fmaxf(ka, fabsf(v[j])); va = fmaxf(va, fabsf(vv[j])); }
#pragma unroll
      for (int o2 = GL / 2; o2 > 0; o2 >>= 1) {
        ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o2));
        va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o2));
      }
      const float ks = ka > 0.f ? ka / 7.f : 1.f, vs = va > 0.f ? va / 7.f : 1.f;
      auto code = [](float x, float sc) { return (uint32_t)(min(7, max(-8, __float2int_rn(x / sc))) + 8); };
#pragma unroll
      for (int j = 0; j < EPL; j += 2) {
        kc4[(off + lane * EPL + j) / 2] = (unsigned char)(code(v[j], ks) | (code(v[j + 1], ks) << 4));
        vc4[(off + lane * EPL + j) / 2] = (unsigned char)(code(vv[j], vs) | (code(vv[j + 1], vs) << 4));
      }
      if (lane % GL == 0) {
        kv_scale[tok * 2 * NG + lane / GL] = ks;
        kv_scale[tok * 2 * NG + NG + lane / GL] = vs;
      }
    } else if (KVM == 1) {
      // e4m3 codes with one fp32 scale per (token, kv head) for K and for V
      unsigned char* kc8 = reinterpret_cast<unsigned char*>(k_cache_v);
      unsigned char* vc8 = reinterpret_cast<unsigned char*>(v_cache_v);
      float vv[EPL], ka = 0.f, va = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) { vv[j] = bf2f(vsrc[lane * EPL + j]); ka = fmaxf(ka, fabsf(v[j])); va = fmaxf(va, fabsf(vv[j])); }
      ka = warp_max(ka); va = warp_max(va);
      const float ks = ka > 0.f ? ka / 448.f : 1.f, vs = va > 0.f ? va / 448.f : 1.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        kc8[off + lane * EPL + j] = (unsigned char)__nv_cvt_float_to_fp8(v[j] / ks, __NV_SATFINITE, __NV_E4M3);
        vc8[off + lane * EPL + j] = (unsigned char)__nv_cvt_float_to_fp8(vv[j] / vs, __NV_SATFINITE, __NV_E4M3);
      }
      if (lane == 0) { kv_scale[tok * 2] = ks; kv_scale[tok * 2 + 1] = vs; }
    } else {
      __nv_bfloat16* k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache_v);
      __nv_bfloat16* v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache_v);
#pragma unroll
      for (int j = 0; j < EPL; ++j) k_cache[off + lane * EPL + j] = f2bf(v[j]);
#pragma unroll
      for (int j = 0; j < EPL; ++j) v_cache[off + lane * EPL + j] = vsrc[lane * EPL + j];
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Split-KV decode attention. grid = (rows, kv heads, splits), 8 warps per CTA. A lane group of HD/8 lanes
// owns one key at a time; every lane keeps 8 dims of K, V and of the G query heads of the group.
constexpr int ATT_WARPS = 8;

__device__ __forceinline__ void e4m3x8_to_float(uint2 raw, float* f) {
  const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w[i] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
      const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      f[i * 4 + h * 2] = f2.x;
      f[i * 4 + h * 2 + 1] = f2.y;
    }
  }
}

template <int HD, int G, int KVM>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_decode_kernel(float* __restrict__ o_part, float* __restrict__ ml_part, const __nv_bfloat16* __restrict__ q,
                   const void* __restrict__ k_cache_v, const void* __restrict__ v_cache_v,
                   const float* __restrict__ kv_scale,
                   const int* __restrict__ row_slot, const int* __restrict__ row_kvlen,
                   const int* __restrict__ row_base, const unsigned long long* __restrict__ row_mask,
                   const int* __restrict__ block_table, int max_blocks, int kv_block, int nq, int nkv, int nsplit,
                   float scale_log2) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int LPK = HD / 8;           // lanes per key
  constexpr int KPI = 32 / LPK;         // keys per warp iteration
  extern __shared__ float sm[];         // [ATT_WARPS][G][HD] o, then [ATT_WARPS][G][2] m,l
  const int row = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPK, kslot = lane / LPK;
  const int kvlen = row_kvlen[row];
  const int base = row_base ? row_base[row] : kvlen;
  const unsigned long long mask = row_mask ? row_mask[row] : 0ull;
  const int slot = row_slot[row];
  // split boundaries depend on the row's own length only
  int per = (kvlen + nsplit - 1) / nsplit;
  per = (per + 31) / 32 * 32;
  const int lo = split * per, hi = min(kvlen, lo + per);

  float qf[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    uint4 qv = *reinterpret_cast<const uint4*>(q + ((size_t)row * nq + (size_t)kvh * G + g) * HD + sub * 8);
    uint32_t u[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { qf[g][2 * j] = bf_lo(u[j]) * scale_log2; qf[g][2 * j + 1] = bf_hi(u[j]) * scale_log2; }
  }
  float m[G], l[G], o[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) o[g][j] = 0.f;
  }
  const int* bt = block_table + (size_t)slot * max_blocks;
  // UN keys per lane group are in flight at once: all their K/V loads are issued before any is consumed
  constexpr int UN = (G <= 6) ? 4 : 2;
  for (int t0 = lo + warp * KPI * UN; t0 < hi; t0 += ATT_WARPS * KPI * UN) {
    uint4 kraw[UN], vraw[UN];
    float2 sc2[UN];
    bool visb[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int t = t0 + u * KPI + kslot;
      bool vis = t < hi;
      if (vis && t >= base) vis = ((mask >> (t - base)) & 1ull) != 0ull;
      visb[u] = vis;
      kraw[u] = make_uint4(0, 0, 0, 0); vraw[u] = make_uint4(0, 0, 0, 0);
      if (vis) {
        const int blk = bt[t / kv_block];
        const size_t tok = ((size_t)blk * kv_block + (t % kv_block)) * nkv + kvh;
        const size_t off = tok * HD + sub * 8;
        if (KVM == 3) {
          constexpr int NG = HD / 32;
          const unsigned short* kp = reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(k_cache_v) + tok * (HD * 3 / 4) + sub * 6);
          const unsigned short* vp = reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(v_cache_v) + tok * (HD * 3 / 4) + sub * 6);
          kraw[u] = make_uint4((uint32_t)__ldg(kp) | ((uint32_t)__ldg(kp + 1) << 16), (uint32_t)__ldg(kp + 2), 0, 0);
          vraw[u] = make_uint4((uint32_t)__ldg(vp) | ((uint32_t)__ldg(vp + 1) << 16), (uint32_t)__ldg(vp + 2), 0, 0);
          sc2[u] = make_float2(kv_scale[tok * 2 * NG + sub / 4], kv_scale[tok * 2 * NG + NG + sub / 4]);
        } else if (KVM == 2) {
          constexpr int NG = HD / 32;
          kraw[u] = make_uint4(__ldg(reinterpret_cast<const unsigned int*>(reinterpret_cast<const unsigned char*>(k_cache_v) + off / 2)), 0, 0, 0);
          vraw[u] = make_uint4(__ldg(reinterpret_cast<const unsigned int*>(reinterpret_cast<const unsigned char*>(v_cache_v) + off / 2)), 0, 0, 0);
          sc2[u] = make_float2(kv_scale[tok * 2 * NG + sub / 4], kv_scale[tok * 2 * NG + NG + sub / 4]);
        } else if (KVM == 1) {
          const uint2 k8 = ldg_stream8(reinterpret_cast<const unsigned char*>(k_cache_v) + off);
          const uint2 v8 = ldg_stream8(reinterpret_cast<const unsigned char*>(v_cache_v) + off);
          kraw[u] = make_uint4(k8.x, k8.y, 0, 0);
          vraw[u] = make_uint4(v8.x, v8.y, 0, 0);
          sc2[u] = *reinterpret_cast<const float2*>(kv_scale + tok * 2);
        } else {
          kraw[u] = ldg_stream(reinterpret_cast<const __nv_bfloat16*>(k_cache_v) + off);
          vraw[u] = ldg_stream(reinterpret_cast<const __nv_bfloat16*>(v_cache_v) + off);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const bool vis = visb[u];
      uint32_t ku[4] = {kraw[u].x, kraw[u].y, kraw[u].z, kraw[u].w}, vu[4] = {vraw[u].x, vraw[u].y, vraw[u].z, vraw[u].w};
      float kf[8], vf[8];
      if (KVM == 3) {
        const unsigned long long kb = (unsigned long long)ku[0] | ((unsigned long long)ku[1] << 32);
        const unsigned long long vb = (unsigned long long)vu[0] | ((unsigned long long)vu[1] << 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          kf[j] = vis ? (float)((int)((kb >> (6 * j)) & 63ull) - 32) * sc2[u].x : 0.f;
          vf[j] = vis ? (float)((int)((vb >> (6 * j)) & 63ull) - 32) * sc2[u].y : 0.f;
        }
      } else if (KVM == 2) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          kf[j] = vis ? (float)((int)((ku[0] >> (4 * j)) & 15u) - 8) * sc2[u].x : 0.f;
          vf[j] = vis ? (float)((int)((vu[0] >> (4 * j)) & 15u) - 8) * sc2[u].y : 0.f;
        }
      } else if (KVM == 1) {
        e4m3x8_to_float(make_uint2(ku[0], ku[1]), kf);
        e4m3x8_to_float(make_uint2(vu[0], vu[1]), vf);
        if (vis) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { kf[j] *= sc2[u].x; vf[j] *= sc2[u].y; }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          kf[2 * j] = bf_lo(ku[j]); kf[2 * j + 1] = bf_hi(ku[j]);
          vf[2 * j] = bf_lo(vu[j]); vf[2 * j + 1] = bf_hi(vu[j]);
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s = fmaf(qf[g][j], kf[j], s);
#pragma unroll
        for (int off = LPK / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (vis) {
          float mn = fmaxf(m[g], s);
          float sc = exp2f(m[g] - mn);
          float p = exp2f(s - mn);
          l[g] = l[g] * sc + p;
#pragma unroll
          for (int j = 0; j < 8; ++j) o[g][j] = fmaf(p, vf[j], o[g][j] * sc);
          m[g] = mn;
        }
      }
    }
  }
  // merge the lane groups of the warp (keys were interleaved over them)
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
      float lo_ = __shfl_xor_sync(0xffffffffu, l[g], off);
      float mn = fmaxf(m[g], mo);
      float a = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
      float b = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
      l[g] = l[g] * a + lo_ * b;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float oo = __shfl_xor_sync(0xffffffffu, o[g][j], off);
        o[g][j] = o[g][j] * a + oo * b;
      }
      m[g] = mn;
    }
  }
  float* so = sm;                                   // [ATT_WARPS][G][HD]
  float* sml = sm + ATT_WARPS * G * HD;             // [ATT_WARPS][G][2]
  if (kslot == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int j = 0; j < 8; ++j) so[((size_t)warp * G + g) * HD + sub * 8 + j] = o[g][j];
      if (sub == 0) { sml[(warp * G + g) * 2] = m[g]; sml[(warp * G + g) * 2 + 1] = l[g]; }
    }
  }
  __syncthreads();
  // merge the warps in warp order and write this split's partial (unnormalised o, m, l)
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    int g = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, sml[(w * G + g) * 2]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      float mw = sml[(w * G + g) * 2];
      float a = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      acc += so[((size_t)w * G + g) * HD + d] * a;
      L += sml[(w * G + g) * 2 + 1] * a;
    }
    size_t qh = (size_t)kvh * G + g;
    size_t pidx = ((size_t)row * nq + qh) * nsplit + split;
    o_part[pidx * HD + d] = acc;
    if (d == 0) { ml_part[pidx * 2] = M; ml_part[pidx * 2 + 1] = L; }
  }
}

constexpr int ATT_MAX_SPLITS = 1025;     // most key splits the combine kernel takes (1024), plus one slot for the sum

// Merge the splits in split order, normalise, apply the sigmoid gate, write bf16 [rows][nq*HD].
template <int HD>
__global__ void attn_combine_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ o_part,
                                    const float* __restrict__ ml_part, const __nv_bfloat16* __restrict__ proj,
                                    long proj_stride, int nq, int nsplit, int gated) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, qh = blockIdx.y;
  const size_t pbase = ((size_t)row * nq + qh) * nsplit;
  // The first warp turns the splits' (max, sum) pairs into one weight per split (two dependent memory round trips for
  // the whole kernel instead of three per thread); then every thread sums its dimensions over the splits in split order.
  __shared__ float wgt[ATT_MAX_SPLITS];
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float M = -INFINITY;
    for (int s0 = lane; s0 < nsplit; s0 += 32) M = fmaxf(M, ml_part[(pbase + s0) * 2]);
    M = warp_max(M);
    for (int s0 = lane; s0 < nsplit; s0 += 32) {
      const float ms = ml_part[(pbase + s0) * 2];
      wgt[s0] = ms != -INFINITY ? exp2f(ms - M) : 0.f;
    }
    __syncwarp();
    if (lane == 0) {                                       // the normaliser, summed in split order
      float Ls = 0.f;
      for (int s0 = 0; s0 < nsplit; ++s0) Ls += ml_part[(pbase + s0) * 2 + 1] * wgt[s0];
      wgt[nsplit] = Ls;                                    // (nsplit < ATT_MAX_SPLITS is checked on the host)
    }
  }
  __syncthreads();
  const float L = wgt[nsplit];
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int s0 = 0; s0 < nsplit; ++s0) {
      const float e = wgt[s0];
      if (e != 0.f) acc += o_part[(pbase + s0) * HD + d] * e;
    }
    float v = acc * inv;
    if (gated) v *= sigmoidf_(bf2f(proj[(size_t)row * proj_stride + (size_t)qh * 2 * HD + HD + d]));
    out[((size_t)row * nq + qh) * HD + d] = f2bf(v);
  }
}

// bf16 rows of the keys / values a prompt chunk can see, decoded from the e4m3 cache into a scratch laid out per
// slot ([slot][position][kv head][hd]) so the prompt attention kernel reads it through an identity block table.
// grid (max kvlen, nkv, segments); blockDim = hd / 8 (8 elements per thread)
__global__ void kv_dequant_kernel(__nv_bfloat16* __restrict__ k_out, __nv_bfloat16* __restrict__ v_out,
                                  const unsigned char* __restrict__ k8, const unsigned char* __restrict__ v8,
                                  const float* __restrict__ kv_scale, const int* __restrict__ seg_slot,
                                  const int* __restrict__ seg_pos0, const int* __restrict__ seg_nrows,
                                  const int* __restrict__ block_table, int max_blocks, int kv_block, int nkv, int hd,
                                  int scratch_tokens_per_slot, int bits) {
  const int t = blockIdx.x, kvh = blockIdx.y, seg = blockIdx.z;
  const int n = seg_nrows[seg];
  if (n <= 0 || t >= seg_pos0[seg] + n) return;
  const int slot = seg_slot[seg];
  const int blk = block_table[(size_t)slot * max_blocks + t / kv_block];
  if (blk < 0) return;
  const size_t tok = ((size_t)blk * kv_block + (t % kv_block)) * nkv + kvh;
  const size_t dst = (((size_t)slot * scratch_tokens_per_slot + t) * nkv + kvh) * hd + threadIdx.x * 8;
  float kf[8], vf[8], ks, vs;
  if (bits == 6) {
    const int ng = hd / 32;
    ks = kv_scale[tok * 2 * ng + threadIdx.x / 4];
    vs = kv_scale[tok * 2 * ng + ng + threadIdx.x / 4];
    const unsigned short* kp = reinterpret_cast<const unsigned short*>(k8 + tok * (hd * 3 / 4) + threadIdx.x * 6);
    const unsigned short* vp = reinterpret_cast<const unsigned short*>(v8 + tok * (hd * 3 / 4) + threadIdx.x * 6);
    const unsigned long long kb = (unsigned long long)kp[0] | ((unsigned long long)kp[1] << 16) | ((unsigned long long)kp[2] << 32);
    const unsigned long long vb = (unsigned long long)vp[0] | ((unsigned long long)vp[1] << 16) | ((unsigned long long)vp[2] << 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      kf[j] = (float)((int)((kb >> (6 * j)) & 63ull) - 32);
      vf[j] = (float)((int)((vb >> (6 * j)) & 63ull) - 32);
    }
  } else if (bits == 4) {
    const int ng = hd / 32;
    ks = kv_scale[tok * 2 * ng + threadIdx.x / 4];
    vs = kv_scale[tok * 2 * ng + ng + threadIdx.x / 4];
    const uint32_t kw = *reinterpret_cast<const uint32_t*>(k8 + (tok * hd + threadIdx.x * 8) / 2);
    const uint32_t vw = *reinterpret_cast<const uint32_t*>(v8 + (tok * hd + threadIdx.x * 8) / 2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      kf[j] = (float)((int)((kw >> (4 * j)) & 15u) - 8);
      vf[j] = (float)((int)((vw >> (4 * j)) & 15u) - 8);
    }
  } else {
    ks = kv_scale[tok * 2]; vs = kv_scale[tok * 2 + 1];
    e4m3x8_to_float(*reinterpret_cast<const uint2*>(k8 + tok * hd + threadIdx.x * 8), kf);
    e4m3x8_to_float(*reinterpret_cast<const uint2*>(v8 + tok * hd + threadIdx.x * 8), vf);
  }
  *reinterpret_cast<uint4*>(k_out + dst) = make_uint4(pack_bf2(kf[0] * ks, kf[1] * ks), pack_bf2(kf[2] * ks, kf[3] * ks),
                                                      pack_bf2(kf[4] * ks, kf[5] * ks), pack_bf2(kf[6] * ks, kf[7] * ks));
  *reinterpret_cast<uint4*>(v_out + dst) = make_uint4(pack_bf2(vf[0] * vs, vf[1] * vs), pack_bf2(vf[2] * vs, vf[3] * vs),
                                                      pack_bf2(vf[4] * vs, vf[5] * vs), pack_bf2(vf[6] * vs, vf[7] * vs));
}

template <int HD, int KVM>
static int launch_decode(int G, dim3 grid, size_t smem, cudaStream_t s, float* o_part, float* ml_part, const void* q,
                         const void* kc, const void* vc, const float* kv_scale, const int* row_slot, const int* row_kvlen,
                         const int* row_base, const unsigned long long* row_mask, const int* bt, int max_blocks,
                         int kv_block, int nq, int nkv, int nsplit, float scale_log2) {
#define FB_LAUNCH_G(GV)                                                                                          \
  case GV: {                                                                                                     \
    auto kern = attn_decode_kernel<HD, GV, KVM>;                                                                 \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    launch_pdl(kern, dim3(grid), dim3(ATT_WARPS * 32), (size_t)(smem), s, o_part, ml_part, (const __nv_bfloat16*)q, kc,  \
                                            vc, kv_scale, row_slot, row_kvlen, row_base, row_mask,               \
                                            bt, max_blocks, kv_block, nq, nkv, nsplit, scale_log2);              \
    break;                                                                                                       \
  }
  switch (G) {
    FB_LAUNCH_G(1) FB_LAUNCH_G(2) FB_LAUNCH_G(3) FB_LAUNCH_G(4) FB_LAUNCH_G(6) FB_LAUNCH_G(8)
    default: return -2;
  }
#undef FB_LAUNCH_G
  return (int)cudaGetLastError();
}

}  // namespace fb

using namespace fb;

static int attn_prep_impl(void* q_out, void* k_cache, void* v_cache, float* kv_scale, const void* proj, long proj_stride,
                          const void* q_norm, const void* k_norm, const float* inv_freq, const int* row_slot,
                          const int* row_pos, const int* row_cpos, const int* block_table, int max_blocks, int kv_block,
                          int rows, int nq, int nkv, int hd, int rot, int gated, float eps, int* status, cudaStream_t s,
                          int bits = 8, int hrot = 0) {
  if (rows <= 0) return 0;
  const int heads = nq + nkv;
  const int threads = 32 * (heads < 32 ? heads : 32);
  const int hgroups = (heads + 31) / 32;
  int epl = hd / 32;
  if (rot % 2 || (rot / 2) % epl || ((rot / 2 / epl) & (rot / 2 / epl - 1))) return -3;
#define FB_PREP(HDV, K8)                                                                                          \
  launch_pdl(attn_prep_kernel<HDV, K8>, dim3(rows, hgroups), dim3(threads), (size_t)(0), s, (__nv_bfloat16*)q_out, k_cache, v_cache, \
      kv_scale, (const __nv_bfloat16*)proj, proj_stride, (const __nv_bfloat16*)q_norm,                            \
      (const __nv_bfloat16*)k_norm, inv_freq, row_slot, row_pos, row_cpos, block_table, max_blocks, kv_block, nq, nkv, rot, \
      gated, eps, status, hrot)
  if (kv_scale && bits == 6) {
    if (hd == 256) FB_PREP(256, 3); else if (hd == 128) FB_PREP(128, 3); else if (hd == 64) FB_PREP(64, 3); else return -2;
  } else if (kv_scale && bits == 4) {
    if (hd == 256) FB_PREP(256, 2); else if (hd == 128) FB_PREP(128, 2); else if (hd == 64) FB_PREP(64, 2); else return -2;
  } else if (kv_scale) {
    if (hd == 256) FB_PREP(256, 1); else if (hd == 128) FB_PREP(128, 1); else if (hd == 64) FB_PREP(64, 1); else return -2;
  } else {
    if (hd == 256) FB_PREP(256, 0); else if (hd == 128) FB_PREP(128, 0); else if (hd == 64) FB_PREP(64, 0); else return -2;
  }
#undef FB_PREP
  return (int)cudaGetLastError();
}

// merge of the per-split partials in split order + sigmoid output gate (shared by the SIMT and the mma decode kernels)
extern "C" int fb_attn_combine(void* out, const float* o_part, const float* ml_part, const void* proj, long proj_stride,
                               int rows, int nq, int hd, int nsplit, int gated, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (nsplit < 1 || nsplit >= ATT_MAX_SPLITS) return -1;
  dim3 cgrid(rows, nq);
  int cthreads = hd >= 128 ? 128 : 64;
  if (hd == 256) launch_pdl(attn_combine_kernel<256>, dim3(cgrid), dim3(cthreads), (size_t)(0), s, (__nv_bfloat16*)out, o_part, ml_part, (const __nv_bfloat16*)proj, proj_stride, nq, nsplit, gated);
  else if (hd == 128) launch_pdl(attn_combine_kernel<128>, dim3(cgrid), dim3(cthreads), (size_t)(0), s, (__nv_bfloat16*)out, o_part, ml_part, (const __nv_bfloat16*)proj, proj_stride, nq, nsplit, gated);
  else if (hd == 64) launch_pdl(attn_combine_kernel<64>, dim3(cgrid), dim3(cthreads), (size_t)(0), s, (__nv_bfloat16*)out, o_part, ml_part, (const __nv_bfloat16*)proj, proj_stride, nq, nsplit, gated);
  else return -2;
  return (int)cudaGetLastError();
}

static int attn_decode_impl(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache,
                            const void* v_cache, const float* kv_scale, const void* proj, long proj_stride,
                            const int* row_slot, const int* row_kvlen, const int* row_base,
                            const unsigned long long* row_mask, const int* block_table, int max_blocks, int kv_block,
                            int rows, int nq, int nkv, int hd, int nsplit, int gated, cudaStream_t s, int bits = 8) {
  if (rows <= 0) return 0;
  if (nq % nkv) return -1;
  int G = nq / nkv;
  dim3 grid(rows, nkv, nsplit);
  size_t smem = (size_t)ATT_WARPS * G * (hd + 2) * sizeof(float);
  float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  int rc;
#define FB_DEC(HDV, K8) rc = launch_decode<HDV, K8>(G, grid, smem, s, o_part, ml_part, q, k_cache, v_cache, kv_scale, row_slot, row_kvlen, row_base, row_mask, block_table, max_blocks, kv_block, nq, nkv, nsplit, scale_log2)
  if (kv_scale && bits == 6) {
    if (hd == 256) FB_DEC(256, 3); else if (hd == 128) FB_DEC(128, 3); else if (hd == 64) FB_DEC(64, 3); else return -2;
  } else if (kv_scale && bits == 4) {
    if (hd == 256) FB_DEC(256, 2); else if (hd == 128) FB_DEC(128, 2); else if (hd == 64) FB_DEC(64, 2); else return -2;
  } else if (kv_scale) {
    if (hd == 256) FB_DEC(256, 1); else if (hd == 128) FB_DEC(128, 1); else if (hd == 64) FB_DEC(64, 1); else return -2;
  } else {
    if (hd == 256) FB_DEC(256, 0); else if (hd == 128) FB_DEC(128, 0); else if (hd == 64) FB_DEC(64, 0); else return -2;
  }
#undef FB_DEC
  if (rc) return rc;
  return fb_attn_combine(out, o_part, ml_part, proj, proj_stride, rows, nq, hd, nsplit, gated, s);
}

extern "C" int fb_attn_prep(void* q_out, void* k_cache, void* v_cache, const void* proj, long proj_stride,
                            const void* q_norm, const void* k_norm, const float* inv_freq, const int* row_slot,
                            const int* row_pos, const int* block_table, int max_blocks, int kv_block, int rows, int nq,
                            int nkv, int hd, int rot, int gated, float eps, int* status, cudaStream_t s) {
  return attn_prep_impl(q_out, k_cache, v_cache, nullptr, proj, proj_stride, q_norm, k_norm, inv_freq, row_slot, row_pos,
                        nullptr, block_table, max_blocks, kv_block, rows, nq, nkv, hd, rot, gated, eps, status, s);
}

// Verify-tree form: `row_pos` is the rotary position (depth in the tree), `row_cpos` the cache row the K/V go to.
// `kv_scale` non-null selects the e4m3 cache.
extern "C" int fb_attn_prep_tree(void* q_out, void* k_cache, void* v_cache, float* kv_scale, const void* proj,
                                 long proj_stride, const void* q_norm, const void* k_norm, const float* inv_freq,
                                 const int* row_slot, const int* row_pos, const int* row_cpos, const int* block_table,
                                 int max_blocks, int kv_block, int rows, int nq, int nkv, int hd, int rot, int gated,
                                 float eps, int* status, cudaStream_t s) {
  return attn_prep_impl(q_out, k_cache, v_cache, kv_scale, proj, proj_stride, q_norm, k_norm, inv_freq, row_slot, row_pos,
                        row_cpos, block_table, max_blocks, kv_block, rows, nq, nkv, hd, rot, gated, eps, status, s);
}

extern "C" int fb_attn_decode(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache,
                              const void* v_cache, const void* proj, long proj_stride, const int* row_slot,
                              const int* row_kvlen, const int* row_base, const unsigned long long* row_mask,
                              const int* block_table, int max_blocks, int kv_block, int rows, int nq, int nkv, int hd,
                              int nsplit, int gated, cudaStream_t s) {
  return attn_decode_impl(out, o_part, ml_part, q, k_cache, v_cache, nullptr, proj, proj_stride, row_slot, row_kvlen,
                          row_base, row_mask, block_table, max_blocks, kv_block, rows, nq, nkv, hd, nsplit, gated, s);
}

// FP8 (e4m3) KV cache: codes [blocks][kv_block][nkv][hd] bytes + scales [blocks][kv_block][nkv][2] fp32 (K, V)
extern "C" int fb_attn_prep_kv8(void* q_out, void* k_cache8, void* v_cache8, float* kv_scale, const void* proj,
                                long proj_stride, const void* q_norm, const void* k_norm, const float* inv_freq,
                                const int* row_slot, const int* row_pos, const int* block_table, int max_blocks,
                                int kv_block, int rows, int nq, int nkv, int hd, int rot, int gated, float eps, int* status,
                                cudaStream_t s) {
  if (!kv_scale) return -4;
  return attn_prep_impl(q_out, k_cache8, v_cache8, kv_scale, proj, proj_stride, q_norm, k_norm, inv_freq, row_slot, row_pos,
                        nullptr, block_table, max_blocks, kv_block, rows, nq, nkv, hd, rot, gated, eps, status, s);
}

extern "C" int fb_attn_decode_kv8(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache8,
                                  const void* v_cache8, const float* kv_scale, const void* proj, long proj_stride,
                                  const int* row_slot, const int* row_kvlen, const int* row_base,
                                  const unsigned long long* row_mask, const int* block_table, int max_blocks,
                                  int kv_block, int rows, int nq, int nkv, int hd, int nsplit, int gated, cudaStream_t s) {
  if (!kv_scale) return -4;
  return attn_decode_impl(out, o_part, ml_part, q, k_cache8, v_cache8, kv_scale, proj, proj_stride, row_slot, row_kvlen,
                          row_base, row_mask, block_table, max_blocks, kv_block, rows, nq, nkv, hd, nsplit, gated, s);
}

// decode the e4m3 rows the segments of a prompt step can see into the per-slot bf16 scratch
extern "C" int fb_kv_dequant(void* k_out, void* v_out, const void* k_cache8, const void* v_cache8, const float* kv_scale,
                             const int* seg_slot, const int* seg_pos0, const int* seg_nrows, const int* block_table,
                             int max_blocks, int kv_block, int nseg, int max_kvlen, int nkv, int hd,
                             int scratch_tokens_per_slot, cudaStream_t s) {
  if (nseg <= 0 || max_kvlen <= 0) return 0;
  if (hd % 8 || max_kvlen > scratch_tokens_per_slot) return -1;
  kv_dequant_kernel<<<dim3(max_kvlen, nkv, nseg), hd / 8, 0, s>>>((__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out,
      (const unsigned char*)k_cache8, (const unsigned char*)v_cache8, kv_scale, seg_slot, seg_pos0, seg_nrows, block_table,
      max_blocks, kv_block, nkv, hd, scratch_tokens_per_slot, 8);
  return (int)cudaGetLastError();
}

// ---- 4-bit KV cache: codes [blocks][kv_block][nkv][hd/2] bytes (low nibble = even element, value = (code - 8) * scale),
// scales [blocks][kv_block][nkv][2 * hd/32] fp32 (K groups then V groups, one per 32 elements). Counterparts of the
// reference's `fe_attn_prep_q4`, `fe_attn_vk_q*` and the q4 flash path (`kernels/k-core/src/kvq.rs`).
extern "C" int fb_attn_prep_q4(void* q_out, void* k_cache4, void* v_cache4, float* kv_scale, const void* proj,
                               long proj_stride, const void* q_norm, const void* k_norm, const float* inv_freq,
                               const int* row_slot, const int* row_pos, const int* row_cpos, const int* block_table,
                               int max_blocks, int kv_block, int rows, int nq, int nkv, int hd, int rot, int gated,
                               float eps, int* status, cudaStream_t s) {
  if (!kv_scale) return -4;
  return attn_prep_impl(q_out, k_cache4, v_cache4, kv_scale, proj, proj_stride, q_norm, k_norm, inv_freq, row_slot, row_pos,
                        row_cpos, block_table, max_blocks, kv_block, rows, nq, nkv, hd, rot, gated, eps, status, s, 4);
}

extern "C" int fb_attn_decode_q4(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache4,
                                 const void* v_cache4, const float* kv_scale, const void* proj, long proj_stride,
                                 const int* row_slot, const int* row_kvlen, const int* row_base,
                                 const unsigned long long* row_mask, const int* block_table, int max_blocks,
                                 int kv_block, int rows, int nq, int nkv, int hd, int nsplit, int gated, cudaStream_t s) {
  if (!kv_scale) return -4;
  return attn_decode_impl(out, o_part, ml_part, q, k_cache4, v_cache4, kv_scale, proj, proj_stride, row_slot, row_kvlen,
                          row_base, row_mask, block_table, max_blocks, kv_block, rows, nq, nkv, hd, nsplit, gated, s, 4);
}

extern "C" int fb_kv_dequant_q4(void* k_out, void* v_out, const void* k_cache4, const void* v_cache4, const float* kv_scale,
                                const int* seg_slot, const int* seg_pos0, const int* seg_nrows, const int* block_table,
                                int max_blocks, int kv_block, int nseg, int max_kvlen, int nkv, int hd,
                                int scratch_tokens_per_slot, cudaStream_t s) {
  if (nseg <= 0 || max_kvlen <= 0) return 0;
  if (hd % 32 || max_kvlen > scratch_tokens_per_slot) return -1;
  kv_dequant_kernel<<<dim3(max_kvlen, nkv, nseg), hd / 8, 0, s>>>((__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out,
      (const unsigned char*)k_cache4, (const unsigned char*)v_cache4, kv_scale, seg_slot, seg_pos0, seg_nrows, block_table,
      max_blocks, kv_block, nkv, hd, scratch_tokens_per_slot, 4);
  return (int)cudaGetLastError();
}

// ---- low-bit KV cache, general form: bits = 4 (codes [..][hd / 2]) or 6 (codes [..][hd * 3 / 4], value = (code - 32) *
// scale), one fp32 scale per 32 elements in both; `hrot` != 0 stores keys (and hands out queries) in a Walsh-Hadamard
// rotated basis. Counterpart of the reference's 6-bit records and rotated 4-bit records (`kernels/k-core/src/kvq.rs:95,126`).
extern "C" int fb_attn_prep_qn(void* q_out, void* k_cache, void* v_cache, float* kv_scale, const void* proj,
                               long proj_stride, const void* q_norm, const void* k_norm, const float* inv_freq,
                               const int* row_slot, const int* row_pos, const int* row_cpos, const int* block_table,
                               int max_blocks, int kv_block, int rows, int nq, int nkv, int hd, int rot, int gated,
                               float eps, int* status, int bits, int hrot, cudaStream_t s) {
  if ((bits == 4 || bits == 6) && !kv_scale) return -4;
  if (bits != 4 && bits != 6 && bits != 8 && bits != 16) return -1;
  return attn_prep_impl(q_out, k_cache, v_cache, bits == 16 ? nullptr : kv_scale, proj, proj_stride, q_norm, k_norm, inv_freq,
                        row_slot, row_pos, row_cpos, block_table, max_blocks, kv_block, rows, nq, nkv, hd, rot, gated, eps,
                        status, s, bits, hrot);
}

extern "C" int fb_attn_decode_qn(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache,
                                 const void* v_cache, const float* kv_scale, const void* proj, long proj_stride,
                                 const int* row_slot, const int* row_kvlen, const int* row_base,
                                 const unsigned long long* row_mask, const int* block_table, int max_blocks,
                                 int kv_block, int rows, int nq, int nkv, int hd, int nsplit, int gated, int bits,
                                 cudaStream_t s) {
  if (!kv_scale || (bits != 4 && bits != 6)) return -4;
  return attn_decode_impl(out, o_part, ml_part, q, k_cache, v_cache, kv_scale, proj, proj_stride, row_slot, row_kvlen,
                          row_base, row_mask, block_table, max_blocks, kv_block, rows, nq, nkv, hd, nsplit, gated, s, bits);
}

extern "C" int fb_kv_dequant_qn(void* k_out, void* v_out, const void* k_cache, const void* v_cache, const float* kv_scale,
                                const int* seg_slot, const int* seg_pos0, const int* seg_nrows, const int* block_table,
                                int max_blocks, int kv_block, int nseg, int max_kvlen, int nkv, int hd,
                                int scratch_tokens_per_slot, int bits, cudaStream_t s) {
  if (nseg <= 0 || max_kvlen <= 0) return 0;
  if (hd % 32 || max_kvlen > scratch_tokens_per_slot || (bits != 4 && bits != 6)) return -1;
  kv_dequant_kernel<<<dim3(max_kvlen, nkv, nseg), hd / 8, 0, s>>>((__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out,
      (const unsigned char*)k_cache, (const unsigned char*)v_cache, kv_scale, seg_slot, seg_pos0, seg_nrows, block_table,
      max_blocks, kv_block, nkv, hd, scratch_tokens_per_slot, bits);
  return (int)cudaGetLastError();
}

// ---- allocation-free variant (declared in api_static.h) -----------------------------------------------------------
// The per-split partials live in an array that is part of the library image, so a caller that may not allocate device
// memory can still run split-KV decode attention. In host code the array's name is only a handle for the runtime's
// symbol table; the address the kernels need is looked up once per device with cudaGetSymbolAddress.
#include <cstdio>
#include <mutex>

#include "api_static.h"

namespace fb {
constexpr long ATT_STATIC_FLOATS = 2l * 1024 * 1024;                       // 8 MiB per GPU
static __device__ __align__(256) float g_attn_static_scratch[ATT_STATIC_FLOATS];
constexpr int ATT_STATIC_MAX_DEV = 64;
static float* g_attn_static_ptr[ATT_STATIC_MAX_DEV] = {};
static std::mutex g_attn_static_mu;
static thread_local char g_attn_static_err[256] = "";
}  // namespace fb

extern "C" long fb_attn_decode_static_scratch_bytes(void) { return fb::ATT_STATIC_FLOATS * (long)sizeof(float); }

extern "C" long fb_attn_decode_static_need_bytes(int rows, int nq, int hd, int nsplit) {
  if (rows < 0 || nq < 0 || hd < 0 || nsplit < 0) return -1;
  const long sat = 1l << 52;                       // the answer for sizes whose product would not fit
  if (hd > (1 << 16)) return sat;
  long v = (long)rows * (long)nq;                  // < 2^62
  if (v > (1l << 30)) return sat;
  v *= (long)nsplit;                               // < 2^61
  if (v > (1l << 30)) return sat;
  return v * ((long)hd + 2) * (long)sizeof(float); // < 2^30 * 2^17 * 4
}

extern "C" const char* fb_attn_decode_static_error(void) { return fb::g_attn_static_err; }

extern "C" int fb_attn_decode_static(void* out, const void* q, const void* k_cache, const void* v_cache,
                                     const void* proj, long proj_stride, const int* row_slot, const int* row_kvlen,
                                     const int* row_base, const unsigned long long* row_mask, const int* block_table,
                                     int max_blocks, int kv_block, int rows, int nq, int nkv, int hd, int nsplit,
                                     int gated, cudaStream_t s) {
  using namespace fb;
  g_attn_static_err[0] = 0;
  if (rows <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || hd <= 0 || nsplit <= 0) {
    snprintf(g_attn_static_err, sizeof g_attn_static_err, "fb_attn_decode_static: non-positive size");
    return -1;
  }
  // sizes no call can mean: refused before the byte count is formed, so the product below cannot wrap
  if (rows > (1 << 20) || nq > 4096 || nsplit > 1024 || (hd != 64 && hd != 128 && hd != 256)) {
    snprintf(g_attn_static_err, sizeof g_attn_static_err,
             "fb_attn_decode_static: rows=%d nq=%d hd=%d nsplit=%d outside rows<=2^20, nq<=4096, nsplit<=1024, hd in {64,128,256}",
             rows, nq, hd, nsplit);
    return -1;
  }
  const long need = fb_attn_decode_static_need_bytes(rows, nq, hd, nsplit);
  if (need > fb_attn_decode_static_scratch_bytes()) {
    snprintf(g_attn_static_err, sizeof g_attn_static_err,
             "fb_attn_decode_static: rows=%d nq=%d hd=%d nsplit=%d need %ld bytes of scratch, the built-in array holds %ld",
             rows, nq, hd, nsplit, need, fb_attn_decode_static_scratch_bytes());
    return -20;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    snprintf(g_attn_static_err, sizeof g_attn_static_err, "fb_attn_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (dev < 0 || dev >= ATT_STATIC_MAX_DEV) {
    snprintf(g_attn_static_err, sizeof g_attn_static_err, "fb_attn_decode_static: device %d beyond the set-up table", dev);
    return -21;
  }
  float* base;
  {
    std::lock_guard<std::mutex> lk(g_attn_static_mu);
    if (!g_attn_static_ptr[dev]) {                    // first call on this device (it is the current one)
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
      if (e != cudaSuccess || !p) {
        snprintf(g_attn_static_err, sizeof g_attn_static_err, "fb_attn_decode_static: cudaGetSymbolAddress: %s",
                 cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : -22;
      }
      g_attn_static_ptr[dev] = static_cast<float*>(p);
    }
    base = g_attn_static_ptr[dev];
  }
  float* o_part = base;                                              // [rows][nq][nsplit][hd]
  float* ml_part = base + (size_t)rows * nq * nsplit * hd;           // [rows][nq][nsplit][2]
  int rc = fb_attn_decode(out, o_part, ml_part, q, k_cache, v_cache, proj, proj_stride, row_slot, row_kvlen, row_base,
                          row_mask, block_table, max_blocks, kv_block, rows, nq, nkv, hd, nsplit, gated, s);
  if (rc)
    snprintf(g_attn_static_err, sizeof g_attn_static_err, "fb_attn_decode_static: launch failed with code %d%s%s", rc,
             rc > 0 ? ": " : "", rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "");
  return rc;
}
