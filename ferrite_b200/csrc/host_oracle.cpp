// Plain C++ restatements of the core ops in double precision: loops over scalars, no library calls. They exist to check
// the checker: the GPU tests compare every kernel with the fp32 PyTorch statement of its op (`ops/torch_ops.py`), and
// `tests/test_oracle_cpu.py` compares those statements with these, so an error in the PyTorch statement (a wrong axis,
// a broadcast that silently fits) cannot hide behind a kernel that copied it. Inputs are fp32 host tensors.
//
//   oracle_linear      y = [RMSNorm(1 + w)](x) W^T, optional SwiGLU over W = [gate | up], optional residual
//   oracle_attention   causal softmax attention of rows over the first kvlen[r] keys of their sequence, grouped heads
//   oracle_gdn         gated delta rule, one sequence: state decay, delta update, read-out, per row
//   oracle_nvfp4       x W^T with W given as e2m1 codes + e4m3 block scales + one tensor scale, decoded here
//
// The role of the reference's CPU references (`crates/fe-fp4/src/format.rs` `ref_gemm`, `crates/fe-dsc/src/refmodel.rs`,
// the f64 paths of `crates/fe-exl3/src/cpu.rs`).
#include <torch/extension.h>

#include <cmath>
#include <vector>

namespace {

using torch::Tensor;

const float* f32(const Tensor& t) {
  TORCH_CHECK(t.dtype() == torch::kFloat32 && t.is_contiguous() && !t.is_cuda(), "oracle: contiguous fp32 host tensors");
  return t.data_ptr<float>();
}

Tensor oracle_linear(const Tensor& x, const Tensor& w, c10::optional<Tensor> norm_w, double eps, c10::optional<Tensor> res,
                     bool swiglu) {
  const int64_t M = x.size(0), K = x.size(1), R = w.size(0), N = swiglu ? R / 2 : R;
  TORCH_CHECK(w.size(1) == K, "oracle_linear: K");
  const float *xp = f32(x), *wp = f32(w);
  const float* nw = norm_w.has_value() ? f32(*norm_w) : nullptr;
  const float* rp = res.has_value() ? f32(*res) : nullptr;
  Tensor y = torch::empty({M, N}, torch::kFloat32);
  float* yp = y.data_ptr<float>();
  std::vector<double> h(K);
  for (int64_t m = 0; m < M; ++m) {
    double ss = 0;
    for (int64_t k = 0; k < K; ++k) ss += (double)xp[m * K + k] * xp[m * K + k];
    const double r = nw ? 1.0 / std::sqrt(ss / (double)K + eps) : 1.0;
    for (int64_t k = 0; k < K; ++k) h[k] = nw ? xp[m * K + k] * r * (1.0 + nw[k]) : xp[m * K + k];
    for (int64_t n = 0; n < N; ++n) {
      double a = 0, b = 0;
      for (int64_t k = 0; k < K; ++k) a += h[k] * wp[n * K + k];
      if (swiglu) {
        for (int64_t k = 0; k < K; ++k) b += h[k] * wp[(N + n) * K + k];
        a = a / (1.0 + std::exp(-a)) * b;
      }
      if (rp) a += rp[m * N + n];
      yp[m * N + n] = (float)a;
    }
  }
  return y;
}

// q [T, nq, hd]; k, v [L, nkv, hd] (one sequence); kvlen [T] (int32): row r sees keys 0 .. kvlen[r] - 1
Tensor oracle_attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& kvlen) {
  const int64_t T = q.size(0), nq = q.size(1), hd = q.size(2), L = k.size(0), nkv = k.size(1), G = nq / nkv;
  const float *qp = f32(q), *kp = f32(k), *vp = f32(v);
  const int32_t* lp = kvlen.data_ptr<int32_t>();
  Tensor o = torch::zeros({T, nq, hd}, torch::kFloat32);
  float* op = o.data_ptr<float>();
  std::vector<double> s(L);
  for (int64_t t = 0; t < T; ++t)
    for (int64_t h = 0; h < nq; ++h) {
      const int64_t kh = h / G, n = std::min<int64_t>(lp[t], L);
      double mx = -INFINITY;
      for (int64_t j = 0; j < n; ++j) {
        double d = 0;
        for (int64_t c = 0; c < hd; ++c) d += (double)qp[(t * nq + h) * hd + c] * kp[(j * nkv + kh) * hd + c];
        s[j] = d / std::sqrt((double)hd);
        mx = std::max(mx, s[j]);
      }
      double den = 0;
      for (int64_t j = 0; j < n; ++j) { s[j] = std::exp(s[j] - mx); den += s[j]; }
      for (int64_t c = 0; c < hd; ++c) {
        double a = 0;
        for (int64_t j = 0; j < n; ++j) a += s[j] * vp[(j * nkv + kh) * hd + c];
        op[(t * nq + h) * hd + c] = n > 0 ? (float)(a / den) : 0.f;
      }
    }
  return o;
}

// qkv [T, 2 nk dk + nv dv] (after the conv), b / a [T, nv] (beta logit, decay input), state [nv, dk, dv], A_log / dt_bias
// [nv]. Returns (y [T, nv dv], final state).
std::pair<Tensor, Tensor> oracle_gdn(const Tensor& qkv, const Tensor& b, const Tensor& a, const Tensor& state, const Tensor& A_log,
                                     const Tensor& dt_bias, int64_t nk, int64_t nv, int64_t dk, int64_t dv, double eps) {
  const int64_t T = qkv.size(0), C = 2 * nk * dk + nv * dv, rep = nv / nk;
  TORCH_CHECK(qkv.size(1) == C, "oracle_gdn: row width");
  const float *xp = f32(qkv), *bp = f32(b), *ap = f32(a), *Al = f32(A_log), *db = f32(dt_bias), *sp = f32(state);
  std::vector<double> S(sp, sp + nv * dk * dv), qn(dk), kn(dk), kvv(dv);
  Tensor y = torch::empty({T, nv * dv}, torch::kFloat32);
  float* yp = y.data_ptr<float>();
  for (int64_t t = 0; t < T; ++t) {
    const float* x = xp + t * C;
    for (int64_t h = 0; h < nv; ++h) {
      const float* q = x + (h / rep) * dk;
      const float* k = x + nk * dk + (h / rep) * dk;
      const float* v = x + 2 * nk * dk + h * dv;
      double qs = 0, ks = 0;
      for (int64_t i = 0; i < dk; ++i) { qs += (double)q[i] * q[i]; ks += (double)k[i] * k[i]; }
      for (int64_t i = 0; i < dk; ++i) {
        qn[i] = q[i] / std::sqrt(qs + eps) / std::sqrt((double)dk);
        kn[i] = k[i] / std::sqrt(ks + eps);
      }
      const double z = (double)ap[t * nv + h] + db[h];
      const double softplus = z > 20 ? z : std::log1p(std::exp(z));
      const double g = std::exp(-std::exp((double)Al[h]) * softplus), beta = 1.0 / (1.0 + std::exp(-(double)bp[t * nv + h]));
      double* Sh = S.data() + h * dk * dv;
      for (int64_t i = 0; i < dk * dv; ++i) Sh[i] *= g;
      for (int64_t j = 0; j < dv; ++j) {
        double acc = 0;
        for (int64_t i = 0; i < dk; ++i) acc += Sh[i * dv + j] * kn[i];
        kvv[j] = (v[j] - acc) * beta;
      }
      for (int64_t i = 0; i < dk; ++i)
        for (int64_t j = 0; j < dv; ++j) Sh[i * dv + j] += kn[i] * kvv[j];
      for (int64_t j = 0; j < dv; ++j) {
        double acc = 0;
        for (int64_t i = 0; i < dk; ++i) acc += Sh[i * dv + j] * qn[i];
        yp[t * nv * dv + h * dv + j] = (float)acc;
      }
    }
  }
  Tensor out = torch::empty({nv, dk, dv}, torch::kFloat32);
  float* o = out.data_ptr<float>();
  for (size_t i = 0; i < S.size(); ++i) o[i] = (float)S[i];
  return {y, out};
}

double e2m1(int code) {
  static const double mag[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};
  return (code & 8) ? -mag[code & 7] : mag[code & 7];
}

double e4m3(int bits) {                    // finite e4m3 (bias 7, no infinities; 0x7f / 0xff are NaN and do not occur in scales)
  const int s = bits >> 7, e = (bits >> 3) & 15, m = bits & 7;
  const double v = e == 0 ? std::ldexp((double)m, -9) : std::ldexp(1.0 + m / 8.0, e - 7);
  return s ? -v : v;
}

// x [M, K] fp32; packed [N, K / 2] uint8 (low nibble = even element); scales [N, K / 16] uint8 (e4m3 bits); y [M, N]
Tensor oracle_nvfp4(const Tensor& x, const Tensor& packed, const Tensor& scales, double global_scale) {
  const int64_t M = x.size(0), K = x.size(1), N = packed.size(0);
  TORCH_CHECK(packed.size(1) * 2 == K && scales.size(1) * 16 == K && packed.dtype() == torch::kUInt8 &&
              scales.dtype() == torch::kUInt8 && packed.is_contiguous() && scales.is_contiguous(), "oracle_nvfp4: layout");
  const float* xp = f32(x);
  const uint8_t *cp = packed.data_ptr<uint8_t>(), *sp = scales.data_ptr<uint8_t>();
  Tensor y = torch::empty({M, N}, torch::kFloat32);
  float* yp = y.data_ptr<float>();
  std::vector<double> wrow(K);
  for (int64_t n = 0; n < N; ++n) {
    for (int64_t k = 0; k < K; ++k) {
      const int byte = cp[n * (K / 2) + k / 2], code = (k & 1) ? byte >> 4 : byte & 15;
      wrow[k] = e2m1(code) * e4m3(sp[n * (K / 16) + k / 16]) * global_scale;
    }
    for (int64_t m = 0; m < M; ++m) {
      double a = 0;
      for (int64_t k = 0; k < K; ++k) a += (double)xp[m * K + k] * wrow[k];
      yp[m * N + n] = (float)a;
    }
  }
  return y;
}

}  // namespace

void register_oracle(pybind11::module_& m) {
  m.def("oracle_linear", &oracle_linear);
  m.def("oracle_attention", &oracle_attention);
  m.def("oracle_gdn", &oracle_gdn);
  m.def("oracle_nvfp4", &oracle_nvfp4);
}
