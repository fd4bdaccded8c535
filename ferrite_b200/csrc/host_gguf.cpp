// GGUF block decoders on the load path, in C++, to fp32: the legacy and K formats dense checkpoints are made of (Q8_0,
// Q4_0/1, Q5_0/1, Q2_K .. Q6_K), the 4-bit non-linear ones (IQ4_NL, IQ4_XS) and the codebook formats the large MoE
// checkpoints ship in (IQ1_S/M, IQ2_XXS/XS/S, IQ3_XXS/S; their grids and sign table come from the caller, one copy in
// `formats/gguf_tables.py`). Bit for bit what the NumPy statements in `formats/gguf.py` produce (same operations in the
// same order and width, no fused multiply-add), without the temporaries of the vectorised form, and with the blocks
// spread over the host's cores. Counterpart of the reference's host decoders (`crates/fe-gguf`,
// `crates/fe-ggq/src/refq.rs`).
#pragma GCC optimize("fp-contract=off")
#include <ATen/Parallel.h>
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

inline uint16_t u16(const uint8_t* p) { return (uint16_t)p[0] | ((uint16_t)p[1] << 8); }
inline uint32_t u32(const uint8_t* p) { return (uint32_t)u16(p) | ((uint32_t)u16(p + 2) << 16); }
inline float f16bits(uint16_t h) {
  const uint8_t b[2] = {(uint8_t)(h & 255), (uint8_t)(h >> 8)};
  return f16(b);
}

struct Tables {
  const int8_t* grid = nullptr;   // codebook rows (8 values for the 1- and 2-bit grids, 4 for the 3-bit ones)
  const uint8_t* ksigns = nullptr;  // 128 sign masks of the 7-bit sign codes
  const float* kvalues = nullptr;   // 16 levels of the non-linear 4-bit formats
};

inline void put8(float* o, float db, const int8_t* g, uint8_t mask) {
  for (int j = 0; j < 8; ++j) o[j] = (db * (float)g[j]) * (((mask >> j) & 1) ? -1.f : 1.f);
}

enum Kind { Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S,
            IQ1_S, IQ1_M };

void decode_block(Kind kind, const uint8_t* b, float* o, const Tables& t) {
  switch (kind) {
    case Q8_0: {
      const float d = f16(b);
      for (int j = 0; j < 32; ++j) o[j] = d * (float)(int8_t)b[2 + j];
      break;
    }
    case Q4_0: {
      const float d = f16(b);
      for (int j = 0; j < 16; ++j) {
        o[j] = d * ((float)(b[2 + j] & 0xF) - 8.f);
        o[16 + j] = d * ((float)(b[2 + j] >> 4) - 8.f);
      }
      break;
    }
    case Q4_1: {
      const float d = f16(b), m = f16(b + 2);
      for (int j = 0; j < 16; ++j) {
        o[j] = d * (float)(b[4 + j] & 0xF) + m;
        o[16 + j] = d * (float)(b[4 + j] >> 4) + m;
      }
      break;
    }
    case IQ4_NL: {
      const float d = f16(b);
      for (int j = 0; j < 16; ++j) {
        o[j] = d * t.kvalues[b[2 + j] & 0xF];
        o[16 + j] = d * t.kvalues[b[2 + j] >> 4];
      }
      break;
    }
    case Q5_0:
    case Q5_1: {
      const int off = kind == Q5_1 ? 4 : 2;
      const float d = f16(b), m = kind == Q5_1 ? f16(b + 2) : 0.f;
      const uint32_t qh = u32(b + off);
      const uint8_t* qs = b + off + 4;
      for (int j = 0; j < 16; ++j) {
        const float lo = (float)((qs[j] & 0xF) | (((qh >> j) & 1) << 4));
        const float hi = (float)((qs[j] >> 4) | (((qh >> (j + 16)) & 1) << 4));
        if (kind == Q5_0) {
          o[j] = d * (lo - 16.f);
          o[16 + j] = d * (hi - 16.f);
        } else {
          o[j] = d * lo + m;
          o[16 + j] = d * hi + m;
        }
      }
      break;
    }
    case Q2_K: {
      const uint8_t *sc = b, *qs = b + 16;
      const float d = f16(b + 80), dmin = f16(b + 82);
      for (int n = 0; n < 2; ++n)
        for (int j = 0; j < 4; ++j)
          for (int half = 0; half < 2; ++half) {
            const int i = n * 8 + j * 2 + half;
            const float dl = d * (float)(sc[i] & 0xF), ml = dmin * (float)(sc[i] >> 4);
            for (int k = 0; k < 16; ++k) o[i * 16 + k] = dl * (float)((qs[n * 32 + 16 * half + k] >> (2 * j)) & 3) - ml;
          }
      break;
    }
    case Q3_K: {
      const uint8_t *hm = b, *qs = b + 32;
      const uint32_t a0 = u32(b + 96), a1 = u32(b + 100), tmp = u32(b + 104), k1 = 0x03030303u, k2 = 0x0F0F0F0Fu;
      const uint32_t w[4] = {(a0 & k2) | (((tmp >> 0) & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
                             ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)};
      const float d = f16(b + 108);
      for (int n = 0; n < 2; ++n)
        for (int j = 0; j < 4; ++j)
          for (int half = 0; half < 2; ++half) {
            const int i = n * 8 + j * 2 + half;
            const float sc = (float)(int8_t)((w[i / 4] >> (8 * (i % 4))) & 255) - 32.f;
            const float dl = d * sc;
            const uint8_t bit = (uint8_t)(1u << (n * 4 + j));
            for (int k = 0; k < 16; ++k) {
              const float q = (float)((qs[n * 32 + 16 * half + k] >> (2 * j)) & 3) - ((hm[16 * half + k] & bit) ? 0.f : 4.f);
              o[i * 16 + k] = dl * q;
            }
          }
      break;
    }
    case Q4_K: {
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
      break;
    }
    case Q5_K: {
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
      break;
    }
    case Q6_K: {
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
      break;
    }
    case IQ4_XS: {
      // the NumPy statement multiplies the fp32 scale by an int32 (a double product) and that by the fp32 level: both
      // products are exact in double, one rounding to fp32 at the store
      const float d = f16(b);
      const int sh = (int)u16(b + 2);
      const uint8_t *sl = b + 4, *qs = b + 8;
      for (int ib = 0; ib < 8; ++ib) {
        const int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
        const double dl = (double)d * (double)(ls - 32);
        for (int j = 0; j < 16; ++j) {
          o[ib * 32 + j] = (float)(dl * (double)t.kvalues[qs[ib * 16 + j] & 0xF]);
          o[ib * 32 + 16 + j] = (float)(dl * (double)t.kvalues[qs[ib * 16 + j] >> 4]);
        }
      }
      break;
    }
    case IQ2_XXS: {
      const float d = f16(b);
      for (int ib = 0; ib < 8; ++ib) {
        const uint8_t* q = b + 2 + 8 * ib;
        const uint32_t aux = u32(q + 4);
        const float db = (d * (0.5f + (float)(aux >> 28))) * 0.25f;
        for (int l = 0; l < 4; ++l) put8(o + ib * 32 + l * 8, db, t.grid + 8 * (int)q[l], t.ksigns[(aux >> (7 * l)) & 127]);
      }
      break;
    }
    case IQ2_XS: {
      const float d = f16(b);
      const uint8_t* sc = b + 66;
      for (int ib = 0; ib < 8; ++ib) {
        const float db[2] = {(d * (0.5f + (float)(sc[ib] & 0xF))) * 0.25f, (d * (0.5f + (float)(sc[ib] >> 4))) * 0.25f};
        for (int l = 0; l < 4; ++l) {
          const uint16_t q = u16(b + 2 + 2 * (ib * 4 + l));
          put8(o + ib * 32 + l * 8, db[l / 2], t.grid + 8 * (int)(q & 511), t.ksigns[q >> 9]);
        }
      }
      break;
    }
    case IQ2_S: {
      const float d = f16(b);
      const uint8_t *qs = b + 2, *sg = b + 34, *qh = b + 66, *sc = b + 74;
      for (int ib = 0; ib < 8; ++ib) {
        const float db[2] = {(d * (0.5f + (float)(sc[ib] & 0xF))) * 0.25f, (d * (0.5f + (float)(sc[ib] >> 4))) * 0.25f};
        for (int l = 0; l < 4; ++l) {
          const int idx = (int)qs[ib * 4 + l] | (((int)qh[ib] << (8 - 2 * l)) & 0x300);
          put8(o + ib * 32 + l * 8, db[l / 2], t.grid + 8 * idx, sg[ib * 4 + l]);
        }
      }
      break;
    }
    case IQ3_XXS: {
      const float d = f16(b);
      const uint8_t* qs = b + 2;
      for (int ib = 0; ib < 8; ++ib) {
        const uint32_t aux = u32(b + 66 + 4 * ib);
        const float db = (d * (0.5f + (float)(aux >> 28))) * 0.5f;
        for (int l = 0; l < 4; ++l) {
          const uint8_t mask = t.ksigns[(aux >> (7 * l)) & 127];
          const int8_t *g0 = t.grid + 4 * (int)qs[ib * 8 + 2 * l], *g1 = t.grid + 4 * (int)qs[ib * 8 + 2 * l + 1];
          float* oo = o + ib * 32 + l * 8;
          for (int j = 0; j < 4; ++j) {
            oo[j] = (db * (float)g0[j]) * (((mask >> j) & 1) ? -1.f : 1.f);
            oo[4 + j] = (db * (float)g1[j]) * (((mask >> (4 + j)) & 1) ? -1.f : 1.f);
          }
        }
      }
      break;
    }
    case IQ3_S: {
      const float d = f16(b);
      const uint8_t *qs = b + 2, *qh = b + 66, *sg = b + 74, *sc = b + 106;
      for (int ib = 0; ib < 8; ++ib) {
        const int nib = (ib & 1) ? (sc[ib / 2] >> 4) : (sc[ib / 2] & 0xF);
        const float db = d * (1.f + 2.f * (float)nib);
        for (int l = 0; l < 4; ++l) {
          const uint8_t mask = sg[ib * 4 + l];
          float* oo = o + ib * 32 + l * 8;
          for (int e = 0; e < 2; ++e) {
            const int j = 2 * l + e;
            const int idx = (int)qs[ib * 8 + j] | ((((int)qh[ib] << 8) >> j) & 256);
            const int8_t* g = t.grid + 4 * idx;
            for (int k = 0; k < 4; ++k) oo[4 * e + k] = (db * (float)g[k]) * (((mask >> (4 * e + k)) & 1) ? -1.f : 1.f);
          }
        }
      }
      break;
    }
    case IQ1_S: {
      const float d = f16(b);
      const uint8_t* qs = b + 2;
      for (int ib = 0; ib < 8; ++ib) {
        const uint16_t qh = u16(b + 34 + 2 * ib);
        const float dl = d * (float)(2 * ((qh >> 12) & 7) + 1), dlt = (qh & 0x8000) ? -0.125f : 0.125f;
        for (int l = 0; l < 4; ++l) {
          const int8_t* g = t.grid + 8 * ((int)qs[ib * 4 + l] | (((qh >> (3 * l)) & 7) << 8));
          for (int j = 0; j < 8; ++j) o[ib * 32 + l * 8 + j] = dl * ((float)g[j] + dlt);
        }
      }
      break;
    }
    case IQ1_M: {
      const uint8_t *qs = b, *qh = b + 32;
      const uint16_t sc[4] = {u16(b + 48), u16(b + 50), u16(b + 52), u16(b + 54)};
      const uint16_t dbits = (uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00F0) | ((sc[2] >> 4) & 0x0F00) | (sc[3] & 0xF000));
      const float d = f16bits(dbits);
      for (int ib = 0; ib < 8; ++ib) {
        const uint16_t w = sc[ib / 2];
        const float dl[2] = {d * (float)(2 * ((w >> (6 * (ib % 2))) & 7) + 1), d * (float)(2 * ((w >> (6 * (ib % 2) + 3)) & 7) + 1)};
        for (int l = 0; l < 4; ++l) {
          const int h = (l & 1) ? (qh[ib * 2 + l / 2] >> 4) : qh[ib * 2 + l / 2];
          const int8_t* g = t.grid + 8 * ((int)qs[ib * 4 + l] | ((h & 7) << 8));
          const float dlt = (h & 8) ? -0.125f : 0.125f;
          for (int j = 0; j < 8; ++j) o[ib * 32 + l * 8 + j] = dl[l / 2] * ((float)g[j] + dlt);
        }
      }
      break;
    }
  }
}

struct Fmt { const char* name; Kind kind; int bytes, values, grid_rows, grid_cols; };
const Fmt FORMATS[] = {
    {"Q8_0", Q8_0, 34, 32, 0, 0},        {"Q4_0", Q4_0, 18, 32, 0, 0},       {"Q4_1", Q4_1, 20, 32, 0, 0},
    {"Q5_0", Q5_0, 22, 32, 0, 0},        {"Q5_1", Q5_1, 24, 32, 0, 0},       {"Q2_K", Q2_K, 84, 256, 0, 0},
    {"Q3_K", Q3_K, 110, 256, 0, 0},      {"Q4_K", Q4_K, 144, 256, 0, 0},     {"Q5_K", Q5_K, 176, 256, 0, 0},
    {"Q6_K", Q6_K, 210, 256, 0, 0},      {"IQ4_NL", IQ4_NL, 18, 32, 16, 1},  {"IQ4_XS", IQ4_XS, 136, 256, 16, 1},
    {"IQ2_XXS", IQ2_XXS, 66, 256, 256, 8}, {"IQ2_XS", IQ2_XS, 74, 256, 512, 8}, {"IQ2_S", IQ2_S, 82, 256, 1024, 8},
    {"IQ3_XXS", IQ3_XXS, 98, 256, 256, 4}, {"IQ3_S", IQ3_S, 110, 256, 512, 4},  {"IQ1_S", IQ1_S, 50, 256, 2048, 8},
    {"IQ1_M", IQ1_M, 56, 256, 2048, 8},
};

// raw: the tensor's block bytes. grid: the format's codebook as int8 [rows, 8 or 4] (codebook formats) or its 16 levels as
// fp32 (IQ4_NL / IQ4_XS); ksigns: the 128 sign masks (uint8), for the formats that code their signs in 7 bits.
torch::Tensor gguf_dequant_host(const torch::Tensor& raw, const std::string& name, c10::optional<torch::Tensor> grid,
                                c10::optional<torch::Tensor> ksigns) {
  TORCH_CHECK(raw.dtype() == torch::kUInt8 && raw.is_contiguous() && !raw.is_cuda(), "gguf_dequant_host: contiguous host bytes");
  const Fmt* f = nullptr;
  for (const Fmt& x : FORMATS)
    if (name == x.name) f = &x;
  TORCH_CHECK(f != nullptr, "gguf_dequant_host: no decoder for ", name);
  Tables t;
  if (f->grid_rows) {
    TORCH_CHECK(grid.has_value() && grid->is_contiguous() && !grid->is_cuda() && grid->numel() == (int64_t)f->grid_rows * f->grid_cols,
                "gguf_dequant_host: ", name, " needs its table of ", f->grid_rows, " x ", f->grid_cols);
    if (f->grid_cols == 1) {
      TORCH_CHECK(grid->dtype() == torch::kFloat32, "gguf_dequant_host: the 4-bit levels are fp32");
      t.kvalues = grid->data_ptr<float>();
    } else {
      TORCH_CHECK(grid->dtype() == torch::kInt8, "gguf_dequant_host: codebooks are int8");
      t.grid = grid->data_ptr<int8_t>();
    }
  }
  if (f->kind == IQ2_XXS || f->kind == IQ2_XS || f->kind == IQ3_XXS) {
    TORCH_CHECK(ksigns.has_value() && ksigns->dtype() == torch::kUInt8 && ksigns->is_contiguous() && ksigns->numel() == 128,
                "gguf_dequant_host: ", name, " needs the 128 sign masks");
    t.ksigns = ksigns->data_ptr<uint8_t>();
  }
  const int64_t nbytes = raw.numel();
  TORCH_CHECK(nbytes % f->bytes == 0, "gguf_dequant_host: ", nbytes, " bytes are not whole ", name, " blocks");
  const int64_t nb = nbytes / f->bytes;
  torch::Tensor out = torch::empty({nb * f->values}, torch::kFloat32);
  const uint8_t* b = raw.data_ptr<uint8_t>();
  float* o = out.data_ptr<float>();
  const Kind kind = f->kind;
  const int bb = f->bytes, bv = f->values;
  at::parallel_for(0, nb, std::max<int64_t>(1, (1 << 16) / bv), [&](int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) decode_block(kind, b + i * bb, o + i * bv, t);
  });
  return out;
}

}  // namespace

void register_gguf_host(pybind11::module_& m) {
  m.def("gguf_dequant_host", &gguf_dequant_host, pybind11::arg("raw"), pybind11::arg("name"), pybind11::arg("grid") = pybind11::none(),
        pybind11::arg("ksigns") = pybind11::none());
}
