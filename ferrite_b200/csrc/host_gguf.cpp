// GGUF block decoders on the load path, in C++: Q8_0, Q4_0, Q4_K, Q5_K, Q6_K (the formats dense GGUF checkpoints are made
// of) to fp32, bit for bit what the NumPy statements in `formats/gguf.py` produce (same operations in the same order, no
// fused multiply-add), several times faster and without the temporaries of the vectorised form. The other formats (IQ
// codebooks, Q2_K / Q3_K, the legacy 5-bit ones) stay with the NumPy decoders. Counterpart of the reference's host
// decoders (`crates/fe-gguf`, `crates/fe-ggq/src/refq.rs`).
#pragma GCC optimize("fp-contract=off")
#include <torch/extension.h>

#include <cstdint>
#include <cstring>
#include <string>

namespace {

inline float f16(const uint8_t* p) {
  const uint16_t h = (uint16_t)p[0] | ((uint16_t)p[1] << 8);
  const uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023;
  uint32_t u;
  if (e == 0) {
    if (m == 0) {
      u = s;
    } else {                                  // subnormal: renormalise
      int sh = 0;
      uint32_t mm = m;
      while (!(mm & 1024)) { mm <<= 1; ++sh; }
      u = s | ((uint32_t)(113 - sh) << 23) | ((mm & 1023) << 13);
    }
  } else if (e == 31) {
    u = s | 0x7f800000u | (m << 13);
  } else {
    u = s | ((e + 112) << 23) | (m << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// the 8 six-bit (scale, min) pairs of a K-quant super-block's 12 scale bytes
inline void scale_min_k4(const uint8_t* sc, float* s, float* m) {
  for (int j = 0; j < 8; ++j) {
    if (j < 4) {
      s[j] = (float)(sc[j] & 63);
      m[j] = (float)(sc[j + 4] & 63);
    } else {
      s[j] = (float)((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4));
      m[j] = (float)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
    }
  }
}

torch::Tensor gguf_dequant_host(const torch::Tensor& raw, const std::string& name) {
  TORCH_CHECK(raw.dtype() == torch::kUInt8 && raw.is_contiguous() && !raw.is_cuda(), "gguf_dequant_host: contiguous host bytes");
  const uint8_t* b = raw.data_ptr<uint8_t>();
  const int64_t nbytes = raw.numel();
  int bb, bv;
  if (name == "Q8_0") { bb = 34; bv = 32; }
  else if (name == "Q4_0") { bb = 18; bv = 32; }
  else if (name == "Q4_K") { bb = 144; bv = 256; }
  else if (name == "Q5_K") { bb = 176; bv = 256; }
  else if (name == "Q6_K") { bb = 210; bv = 256; }
  else TORCH_CHECK(false, "gguf_dequant_host: no decoder for ", name);
  TORCH_CHECK(nbytes % bb == 0, "gguf_dequant_host: ", nbytes, " bytes are not whole ", name, " blocks");
  const int64_t nb = nbytes / bb;
  torch::Tensor out = torch::empty({nb * bv}, torch::kFloat32);
  float* o = out.data_ptr<float>();
  for (int64_t i = 0; i < nb; ++i, b += bb, o += bv) {
    if (name == "Q8_0") {
      const float d = f16(b);
      for (int j = 0; j < 32; ++j) o[j] = d * (float)(int8_t)b[2 + j];
    } else if (name == "Q4_0") {
      const float d = f16(b);
      for (int j = 0; j < 16; ++j) {
        o[j] = d * ((float)(b[2 + j] & 0xF) - 8.f);
        o[16 + j] = d * ((float)(b[2 + j] >> 4) - 8.f);
      }
    } else if (name == "Q4_K") {
      const float d = f16(b), dmin = f16(b + 2);
      float s[8], m[8];
      scale_min_k4(b + 4, s, m);
      const uint8_t* qs = b + 16;
      for (int g = 0; g < 4; ++g)
        for (int j = 0; j < 32; ++j) {
          const uint8_t q = qs[g * 32 + j];
          o[(2 * g) * 32 + j] = (d * s[2 * g]) * (float)(q & 0xF) - dmin * m[2 * g];
          o[(2 * g + 1) * 32 + j] = (d * s[2 * g + 1]) * (float)(q >> 4) - dmin * m[2 * g + 1];
        }
    } else if (name == "Q5_K") {
      const float d = f16(b), dmin = f16(b + 2);
      float s[8], m[8];
      scale_min_k4(b + 4, s, m);
      const uint8_t *qh = b + 16, *qs = b + 48;
      for (int g = 0; g < 4; ++g)
        for (int j = 0; j < 32; ++j) {
          const uint8_t q = qs[g * 32 + j];
          const float lo = (float)((q & 0xF) + (((qh[j] >> (2 * g)) & 1) << 4));
          const float hi = (float)((q >> 4) + (((qh[j] >> (2 * g + 1)) & 1) << 4));
          o[(2 * g) * 32 + j] = (d * s[2 * g]) * lo - dmin * m[2 * g];
          o[(2 * g + 1) * 32 + j] = (d * s[2 * g + 1]) * hi - dmin * m[2 * g + 1];
        }
    } else {                                  // Q6_K
      const uint8_t *ql = b, *qh = b + 128;
      const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
      const float d = f16(b + 208);
      for (int h = 0; h < 2; ++h)
        for (int j = 0; j < 32; ++j) {
          const uint8_t l0 = ql[h * 64 + j], l1 = ql[h * 64 + 32 + j], hh = qh[h * 32 + j];
          const int q[4] = {(int)((l0 & 0xF) | (((hh >> 0) & 3) << 4)) - 32, (int)((l1 & 0xF) | (((hh >> 2) & 3) << 4)) - 32,
                            (int)((l0 >> 4) | (((hh >> 4) & 3) << 4)) - 32, (int)((l1 >> 4) | (((hh >> 6) & 3) << 4)) - 32};
          for (int k = 0; k < 4; ++k)
            o[h * 128 + 32 * k + j] = d * ((float)sc[h * 8 + j / 16 + 2 * k] * (float)q[k]);
        }
    }
  }
  return out;
}

}  // namespace

void register_gguf_host(pybind11::module_& m) { m.def("gguf_dequant_host", &gguf_dequant_host); }
