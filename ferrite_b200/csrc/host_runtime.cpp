// Host-side pieces of the per-token path in C++: what the scheduler does between two device steps for every request.
//
//   CopyIndex     n-gram index over a request's tokens and the suffix-match proposal of context-copy speculation
//   tree_walk     the accepted path of a verified draft tree
//   grow_tree     best-first verify tree from per-depth candidates
//   graft         a copy proposal laid onto a draft tree
//   StopScanner   stop strings on a text stream, holding back text that may still become one
//   fill_step_meta the int32 staging block of an engine step (tokens, slots, positions, segment tables, verify-tree layout)
//
// Each has a plain-Python statement of the same behaviour (`engine/copy.py`, `engine/scheduler.py`, `server/stop.py`) that
// serves when the extension is not built and that the tests compare against, result for result. Counterparts of the
// reference's `Copier` (`crates/fe-model/src/copy.rs`), `tree_walk` (`crates/fe-model/src/sched.rs:125`), `grow_tree`
// (`crates/fe-dflash/src/lib.rs:306`) and `StopMatcher` (`crates/fe-server/src/stop.rs`).
#include <torch/extension.h>

#include <algorithm>
#include <cstdint>
#include <queue>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

namespace {

namespace py = pybind11;

// ---- context-copy speculation ------------------------------------------------------------------------------------
class CopyIndex {
 public:
  CopyIndex(int key, int min_match, int max_match, int scan)
      : key_(key), min_match_(min_match), max_match_(max_match), scan_(scan) {}

  // Bring the index up to date with the whole sequence; a sequence that is not an extension of the indexed one (a
  // rollback) rebuilds the index.
  void sync(const std::vector<int64_t>& tokens) {
    size_t n = t_.size();
    bool same = tokens.size() >= n;
    for (size_t i = 0; same && i < n; ++i) same = tokens[i] == t_[i];
    if (!same) {
      t_.clear();
      idx_.clear();
      n = 0;
    }
    for (size_t i = n; i < tokens.size(); ++i) {
      t_.push_back(tokens[i]);
      if ((int)i + 1 >= key_) idx_[hash(i + 1 - key_)].push_back((int)i + 1);      // position right after the n-gram
    }
  }

  // Append to a sequence the caller knows to be unchanged up to its current end (the per-step path: O(new tokens)).
  void extend(const std::vector<int64_t>& tail) {
    for (int64_t v : tail) {
      t_.push_back(v);
      const size_t i = t_.size() - 1;
      if ((int)i + 1 >= key_) idx_[hash(i + 1 - key_)].push_back((int)i + 1);
    }
  }

  // the last `k` tokens (fewer when the sequence is shorter): what the caller compares to tell an extension from a rollback
  std::vector<int64_t> tail(int k) const {
    const size_t n = t_.size(), m = std::min(n, (size_t)std::max(0, k));
    return std::vector<int64_t>(t_.end() - m, t_.end());
  }

  size_t size() const { return t_.size(); }

  // Up to `want` tokens that followed the latest longest earlier occurrence of the sequence's end; a continuation that
  // reaches the end of the sequence goes on with the copy itself.
  std::vector<int64_t> propose(int want) const {
    std::vector<int64_t> out;
    const int n = (int)t_.size();
    if (n < min_match_ + 1 || want <= 0) return out;
    auto it = idx_.find(hash(n - key_));
    if (it == idx_.end()) return out;
    const std::vector<int>& cands = it->second;
    int best_len = 0, best_pos = -1;
    const int first = std::max(0, (int)cands.size() - scan_);
    for (int c = (int)cands.size() - 1; c >= first; --c) {
      const int pos = cands[c];
      if (pos >= n) continue;
      int m = 0;
      while (m < max_match_ && pos - 1 - m >= 0 && t_[pos - 1 - m] == t_[n - 1 - m]) ++m;
      if (m > best_len) {
        best_len = m;
        best_pos = pos;
        if (m == max_match_) break;
      }
    }
    if (best_len < min_match_) return out;
    want = std::min(want, max_match_);
    out.reserve(want);
    for (int j = 0; j < want; ++j) {
      const int i = best_pos + j;
      out.push_back(i < n ? t_[i] : out[i - n]);
    }
    return out;
  }

 private:
  // the n-gram starting at `at`; colliding n-grams only add candidates that the backward match then rejects
  uint64_t hash(size_t at) const {
    uint64_t h = 1469598103934665603ull;
    for (int k = 0; k < key_; ++k) h = (h ^ (uint64_t)t_[at + k]) * 1099511628211ull;
    return h;
  }
  int key_, min_match_, max_match_, scan_;
  std::vector<int64_t> t_;
  std::unordered_map<uint64_t, std::vector<int>> idx_;
};

// ---- verify trees ------------------------------------------------------------------------------------------------
// `target[r]`: the target model's token after row r. Returns (rows of the accepted path, tokens to emit).
std::pair<std::vector<int>, std::vector<int64_t>> tree_walk(const std::vector<int64_t>& tokens, const std::vector<int>& parents,
                                                            const std::vector<int64_t>& target) {
  std::vector<int> path{0};
  std::vector<int64_t> emit;
  int node = 0;
  const int n = (int)parents.size();
  for (;;) {
    const int64_t t = target.at(node);
    emit.push_back(t);
    int next = -1;
    for (int c = node + 1; c < n; ++c)          // parents come before children; the first matching child wins
      if (parents[c] == node && tokens[c] == t) { next = c; break; }
    if (next < 0) return {path, emit};
    path.push_back(next);
    node = next;
  }
}

// cand_tok[d][i], cand_lp[d][i]: candidates of the draft token at depth d + 1, best first. Returns (tokens, parents) of
// up to `rows` draft rows in segment numbering (the root is row 0, draft row i is row i + 1).
std::pair<std::vector<int64_t>, std::vector<int>> grow_tree(const std::vector<std::vector<int64_t>>& cand_tok,
                                                            const std::vector<std::vector<double>>& cand_lp, int rows) {
  struct Item { double neg; int tie, prow, d, ci; };
  auto later = [](const Item& a, const Item& b) { return a.neg != b.neg ? a.neg > b.neg : a.tie > b.tie; };
  std::priority_queue<Item, std::vector<Item>, decltype(later)> heap(later);
  std::vector<int64_t> toks;
  std::vector<int> par;
  int tie = 0;
  if (!cand_tok.empty() && !cand_tok[0].empty()) heap.push({-cand_lp[0][0], tie, 0, 0, 0});
  while (!heap.empty() && (int)toks.size() < rows) {
    const Item it = heap.top();
    heap.pop();
    const double lp = cand_lp[it.d][it.ci];
    toks.push_back(cand_tok[it.d][it.ci]);
    par.push_back(it.prow);
    const int me = (int)toks.size();
    if (it.ci + 1 < (int)cand_tok[it.d].size())                               // next-best sibling under the same parent
      heap.push({it.neg + lp - cand_lp[it.d][it.ci + 1], ++tie, it.prow, it.d, it.ci + 1});
    if (it.d + 1 < (int)cand_tok.size() && !cand_tok[it.d + 1].empty())       // best child
      heap.push({it.neg - cand_lp[it.d + 1][0], ++tie, me, it.d + 1, 0});
  }
  return {toks, par};
}

// Lays `copy` (the tokens proposed after the root) onto the tree: follows the rows that already hold it, appends up to
// `room` of the rest as a chain. Returns (tokens, parents, copy tokens found in the tree, rows added).
std::tuple<std::vector<int64_t>, std::vector<int>, int, int> graft(std::vector<int64_t> toks, std::vector<int> parents,
                                                                   const std::vector<int64_t>& copy, int room) {
  int r = 0, i = 0;
  while (i < (int)copy.size()) {
    int next = -1;
    for (int c = r + 1; c < (int)toks.size(); ++c)
      if (parents[c] == r && toks[c] == copy[i]) { next = c; break; }
    if (next < 0) break;
    r = next;
    ++i;
  }
  const int add = std::min((int)copy.size() - i, std::max(0, room));
  for (int k = 0; k < add; ++k) {
    parents.push_back(r);
    toks.push_back(copy[i + k]);
    r = (int)toks.size() - 1;
  }
  return {toks, parents, i, add};
}

// ---- stop strings ------------------------------------------------------------------------------------------------
// Works on UTF-8 bytes; a hold-back never splits a character because stop strings and pushed text are whole characters
// and a proper prefix of a stop string that ends the buffer starts at a character boundary of the buffer.
class StopScanner {
 public:
  StopScanner(std::vector<std::string> stops, bool include) : include_(include) {
    for (auto& s : stops)
      if (!s.empty()) stops_.push_back(std::move(s));
  }

  // (text safe to emit, stopped)
  std::pair<py::bytes, bool> push(const std::string& text) {
    if (hit_) return {py::bytes(""), true};
    if (stops_.empty()) return {py::bytes(text), false};
    buf_ += text;
    size_t best = std::string::npos;
    const std::string* which = nullptr;
    for (const auto& s : stops_) {
      const size_t i = buf_.find(s);
      if (i != std::string::npos && (best == std::string::npos || i < best)) { best = i; which = &s; }
    }
    if (which) {
      std::string out = buf_.substr(0, best + (include_ ? which->size() : 0));
      hit_ = true;
      hit_text_ = *which;
      buf_.clear();
      return {py::bytes(out), true};
    }
    size_t hold = 0;                      // the longest suffix that is a proper prefix of some stop string
    for (const auto& s : stops_) {
      for (size_t k = std::min(s.size() - 1, buf_.size()); k > 0; --k) {
        if (buf_.compare(buf_.size() - k, k, s, 0, k) == 0) { hold = std::max(hold, k); break; }
      }
    }
    std::string out = buf_.substr(0, buf_.size() - hold);
    buf_.erase(0, buf_.size() - hold);
    return {py::bytes(out), false};
  }

  py::bytes flush() {
    std::string out;
    out.swap(buf_);
    return py::bytes(out);
  }

  py::object hit() const { return hit_ ? py::object(py::bytes(hit_text_)) : py::object(py::none()); }

 private:
  std::vector<std::string> stops_;
  bool include_, hit_ = false;
  std::string buf_, hit_text_;
};

// ---- step metadata -------------------------------------------------------------------------------------------------
// Fills the staging buffer of one engine step (int32, usually pinned): [tok T | slot T | pos T | kvlen T | lrow T |
// seg_slot S | seg_row0 S | seg_nrows S | seg_pos0 S] from the step's segments. `want`: 0 no logits, 1 the last row's,
// 2 every row's. With `parents` (one list per segment; empty = a chain) the rows are a verify tree: positions become
// pos0 + depth and the tree block `th` = [ancestor masks (int64 x R) | cache row R | base R | parent R | flags R] is
// filled too (flag bit 0: the row's parent is not the row before it; bit 1: a later row branches from this one).
// Returns the rows whose logits the step produces.
std::vector<int> fill_step_meta(torch::Tensor h, const std::vector<std::vector<int64_t>>& seg_tokens,
                                const std::vector<int>& seg_slot, const std::vector<int>& seg_pos0,
                                const std::vector<int>& seg_want, c10::optional<torch::Tensor> th, int64_t R,
                                const std::vector<std::vector<int>>& parents) {
  TORCH_CHECK(h.dtype() == torch::kInt32 && h.is_contiguous() && !h.is_cuda(), "fill_step_meta: host int32 buffer");
  const size_t S = seg_tokens.size();
  TORCH_CHECK(seg_slot.size() == S && seg_pos0.size() == S && seg_want.size() == S, "fill_step_meta: one entry per segment");
  size_t T = 0;
  for (const auto& t : seg_tokens) T += t.size();
  TORCH_CHECK((size_t)h.numel() >= 5 * T + 4 * S, "fill_step_meta: staging buffer too small");
  int32_t* p = h.data_ptr<int32_t>();
  int32_t *tok = p, *slot = p + T, *pos = p + 2 * T, *kvl = p + 3 * T, *lrow = p + 4 * T;
  int32_t *sslot = p + 5 * T, *srow0 = sslot + S, *snrows = srow0 + S, *spos0 = snrows + S;
  const bool tree = th.has_value() && th->defined();
  int64_t* tmask = nullptr;
  int32_t *tcpos = nullptr, *tbase = nullptr, *tpar = nullptr, *tflag = nullptr;
  if (tree) {
    TORCH_CHECK(th->dtype() == torch::kInt32 && th->is_contiguous() && th->numel() >= 6 * R && (int64_t)T <= R &&
                parents.size() == S, "fill_step_meta: tree block");
    int32_t* q = th->data_ptr<int32_t>();
    tmask = reinterpret_cast<int64_t*>(q);
    tcpos = q + 2 * R; tbase = q + 3 * R; tpar = q + 4 * R; tflag = q + 5 * R;
  }
  std::vector<int> logit_rows;
  size_t r = 0;
  for (size_t si = 0; si < S; ++si) {
    const auto& t = seg_tokens[si];
    const int n = (int)t.size(), p0 = seg_pos0[si];
    for (int j = 0; j < n; ++j) {
      tok[r + j] = (int32_t)t[j];
      slot[r + j] = seg_slot[si];
      pos[r + j] = p0 + j;
      kvl[r + j] = p0 + j + 1;
    }
    if (tree) {
      const auto& par = parents[si];
      TORCH_CHECK(par.empty() || (int)par.size() == n, "fill_step_meta: one parent per row");
      TORCH_CHECK(n > 0 && n <= 64, "a verify tree holds 1..64 rows");
      std::vector<int> depth(n, 0);
      for (int j = 0; j < n; ++j) {
        const int pj = par.empty() ? j - 1 : par[j];
        TORCH_CHECK((pj == -1 && j == 0) || (pj >= 0 && pj < j), "parents come before their children; row 0 is the root");
        depth[j] = pj < 0 ? 0 : depth[pj] + 1;
        tmask[r + j] = (int64_t)((1ull << j) | (pj < 0 ? 0ull : (uint64_t)tmask[r + pj]));
        tflag[r + j] = 0;
        if (pj != j - 1) {
          tflag[r + j] |= 1;
          if (pj >= 0) tflag[r + pj] |= 2;
        }
        pos[r + j] = p0 + depth[j];
        tcpos[r + j] = p0 + j;
        tbase[r + j] = p0;
        tpar[r + j] = pj;
      }
    }
    sslot[si] = seg_slot[si]; srow0[si] = (int32_t)r; snrows[si] = n; spos0[si] = p0;
    if (seg_want[si] == 2) for (int j = 0; j < n; ++j) logit_rows.push_back((int)r + j);
    else if (seg_want[si] == 1 && n > 0) logit_rows.push_back((int)r + n - 1);
    r += n;
  }
  for (size_t i = 0; i < logit_rows.size(); ++i) lrow[i] = logit_rows[i];
  return logit_rows;
}

}  // namespace

void register_host(pybind11::module_& m) {
  py::class_<CopyIndex>(m, "CopyIndex")
      .def(py::init<int, int, int, int>(), py::arg("key"), py::arg("min_match"), py::arg("max_match"), py::arg("scan"))
      .def("sync", &CopyIndex::sync)
      .def("extend", &CopyIndex::extend)
      .def("tail", &CopyIndex::tail)
      .def("size", &CopyIndex::size)
      .def("propose", &CopyIndex::propose);
  m.def("host_tree_walk", &tree_walk);
  m.def("host_grow_tree", &grow_tree);
  m.def("host_graft", &graft);
  m.def("fill_step_meta", &fill_step_meta);
  py::class_<StopScanner>(m, "StopScanner")
      .def(py::init<std::vector<std::string>, bool>(), py::arg("stops"), py::arg("include") = false)
      .def("push", &StopScanner::push)
      .def("flush", &StopScanner::flush)
      .def("hit", &StopScanner::hit);
}
