// Host sampler over one row of logits, in C++: the per-token path of requests the device sampler does not take (penalised
// rows, the first token's stop ban, sampled verification of drafts). The same statements as `engine/sampler.py` (`dist`,
// `draw`): temperature softmax, top-k (ties at the k-th value stay), top-p inside the top-k set (a token stays while the
// mass before it is below top_p; order by probability, ties by index), min-p against the largest probability,
// renormalise; the draw is the inverse CDF in index order over a double-precision running sum. What differs from the
// PyTorch statement is rounding only (its softmax and sums are vectorised), so a pick can differ when the uniform lands
// within rounding of a boundary. The point is the cost: a 248K-entry row needs no full sort here. Top-p sorts only the
// entries that can reach the cut: those above eps = (1 - top_p) / (2 V) hold more than top_p of the mass (the rest
// hold at most V eps), and they precede every smaller entry in the order, so the cut falls among them.
// Counterpart of the reference's CPU sampler (`crates/fe-server/src/sampler.rs`, `crates/fe-model/src/sched.rs:2103-2200`).
#include <torch/extension.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

namespace {

torch::Tensor sample_probs(const torch::Tensor& logits, double temperature, int64_t top_k, double top_p, double min_p,
                           const std::vector<int64_t>& banned) {
  TORCH_CHECK(logits.dim() == 1 && logits.dtype() == torch::kFloat32 && logits.is_contiguous() && !logits.is_cuda(),
              "sample_probs: one contiguous fp32 host row");
  const int64_t V = logits.numel();
  const float* l = logits.data_ptr<float>();
  torch::Tensor out = torch::empty({V}, torch::kFloat32);
  float* p = out.data_ptr<float>();
  const float ninf = -std::numeric_limits<float>::infinity();
  std::vector<float> lf(l, l + V);
  for (int64_t b : banned)
    if (b >= 0 && b < V) lf[b] = ninf;
  const float t = temperature > 0 ? (float)temperature : 1.f;
  auto softmax = [&](float temp) {
    float mx = ninf;
    for (int64_t i = 0; i < V; ++i) mx = std::max(mx, lf[i] / temp);
    double sum = 0;
    for (int64_t i = 0; i < V; ++i) {
      p[i] = std::exp(lf[i] / temp - mx);
      sum += p[i];
    }
    const float inv = (float)(1.0 / sum);
    for (int64_t i = 0; i < V; ++i) p[i] *= inv;
  };
  softmax(t);
  if (top_k > 0 && top_k < V) {
    std::vector<float> tmp(p, p + V);
    std::nth_element(tmp.begin(), tmp.begin() + (top_k - 1), tmp.end(), std::greater<float>());
    const float kth = tmp[top_k - 1];
    for (int64_t i = 0; i < V; ++i)
      if (!(p[i] >= kth)) p[i] = 0.f;
  }
  if (top_p > 0.0 && top_p < 1.0) {
    double tot = 0;
    for (int64_t i = 0; i < V; ++i) tot += p[i];
    const float eps = (float)((1.0 - top_p) * tot / (2.0 * (double)V));
    std::vector<std::pair<float, int64_t>> big;
    for (int64_t i = 0; i < V; ++i)
      if (p[i] > eps) big.emplace_back(p[i], i);
    std::sort(big.begin(), big.end(), [](const std::pair<float, int64_t>& a, const std::pair<float, int64_t>& b) {
      return a.first > b.first || (a.first == b.first && a.second < b.second);
    });
    std::vector<char> keep(V, 0);
    double before = 0;
    for (const auto& e : big) {
      if (!(before / tot < top_p)) break;
      keep[e.second] = 1;
      before += e.first;
    }
    for (int64_t i = 0; i < V; ++i)
      if (!keep[i]) p[i] = 0.f;
  }
  if (min_p > 0.0) {
    float mx = 0.f;
    for (int64_t i = 0; i < V; ++i) mx = std::max(mx, p[i]);
    const float thr = (float)min_p * mx;
    for (int64_t i = 0; i < V; ++i)
      if (!(p[i] >= thr)) p[i] = 0.f;
  }
  double tot = 0;
  for (int64_t i = 0; i < V; ++i) tot += p[i];
  if (tot > 0) {
    const float inv = (float)(1.0 / tot);
    for (int64_t i = 0; i < V; ++i) p[i] *= inv;
  } else {
    softmax(1.f);
  }
  return out;
}

// Inverse-CDF draw in index order: the first index whose running sum (double) exceeds u * sum(p). `excluded` >= 0 draws
// from p with that entry removed (returns it when nothing else has mass).
int64_t sample_draw(const torch::Tensor& probs, double u, int64_t excluded) {
  TORCH_CHECK(probs.dim() == 1 && probs.dtype() == torch::kFloat32 && probs.is_contiguous() && !probs.is_cuda(),
              "sample_draw: one contiguous fp32 host row");
  const int64_t V = probs.numel();
  const float* p = probs.data_ptr<float>();
  double tot = 0;
  for (int64_t i = 0; i < V; ++i)
    if (i != excluded) tot += p[i];
  if (excluded >= 0 && !(tot > 0)) return excluded;
  const double target = u * tot;
  double c = 0;
  int64_t last = V - 1;
  for (int64_t i = 0; i < V; ++i) {
    if (i == excluded) continue;
    c += p[i];
    if (c > target) return i;
    if (p[i] > 0) last = i;
  }
  return excluded >= 0 ? last : V - 1;
}

}  // namespace

void register_sampler_host(pybind11::module_& m) {
  m.def("sample_probs", &sample_probs);
  m.def("sample_draw", &sample_draw, pybind11::arg("probs"), pybind11::arg("u"), pybind11::arg("excluded") = -1);
}
