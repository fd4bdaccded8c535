// Python bindings, second part (fused collectives, quantised formats, MoE, MLA, drafter ops).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <vector>

#include "api.h"
#include "api_ext.h"

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }
inline void check(int rc, const char* what) {
  if (rc == 0) return;
  if (rc > 0) TORCH_CHECK(false, what, ": CUDA error ", rc, " (", cudaGetErrorString((cudaError_t)rc), ")");
  TORCH_CHECK(false, what, ": unsupported arguments (code ", rc, ")");
}
inline const void* cptr(const c10::optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// Handle to the symmetric communication workspace of one rank.
struct Comm {
  std::vector<const void*> peers;
  int rank = 0, world = 1, max_ctas = 0, max_resident = 0;
  long slot_floats = 0;
  Tensor epochs, status;
  unsigned spin_limit = 0;
};

Comm make_comm(std::vector<int64_t> peer_ptrs, int64_t rank, int64_t max_ctas, int64_t slot_floats, Tensor epochs,
               Tensor status, int64_t spin_limit, int64_t max_resident) {
  Comm c;
  for (auto p : peer_ptrs) c.peers.push_back(reinterpret_cast<const void*>(p));
  c.rank = (int)rank; c.world = (int)peer_ptrs.size(); c.max_ctas = (int)max_ctas; c.slot_floats = (long)slot_floats;
  c.epochs = epochs; c.status = status; c.spin_limit = (unsigned)spin_limit; c.max_resident = (int)max_resident;
  return c;
}

void gemv_allreduce(const Comm& c, Tensor Y, Tensor X, Tensor W, c10::optional<Tensor> res) {
  check(fb_gemv_allreduce(Y.data_ptr(), X.data_ptr(), W.data_ptr(), cptr(res), (int)X.size(0), (int)W.size(0),
                          (int)X.size(1), (long)X.stride(0), (long)Y.stride(0), c.peers.data(), c.rank, c.world,
                          c.max_ctas, c.slot_floats, (uint32_t*)c.epochs.data_ptr(), c.status.data_ptr<int>(),
                          c.spin_limit, c.max_resident, cur_stream()), "gemv_allreduce");
}

void allreduce_oneshot(const Comm& c, Tensor y, Tensor part, c10::optional<Tensor> res) {
  check(fb_allreduce_oneshot(y.data_ptr(), part.data_ptr(), cptr(res), (long)part.numel(),
                             part.scalar_type() == torch::kFloat32 ? 1 : 0, c.peers.data(), c.rank, c.world,
                             c.max_ctas, c.slot_floats, (uint32_t*)c.epochs.data_ptr(), c.status.data_ptr<int>(),
                             c.spin_limit, c.max_resident, cur_stream()), "allreduce_oneshot");
}

// A run of consecutive decoder layers for one-row-per-sequence steps in one persistent launch. Per-layer lists; entries a
// layer does not use (a layer entered after its attention has no input projection and no recurrent state) are empty tensors.
// comm: a Comm, or None on one GPU.
int64_t decode_layers_max() { return fb_decode_layers_max(); }
void decode_layers_prepare() { check(fb_decode_layers_prepare(), "decode_layers_prepare"); }

void decode_layers(pybind11::object comm, std::vector<int64_t> start_phase, Tensor x_in, std::vector<Tensor> x_out,
                   std::vector<Tensor> x_mid, std::vector<Tensor> act, std::vector<Tensor> proj, std::vector<Tensor> o,
                   std::vector<Tensor> w_in, std::vector<Tensor> input_norm, std::vector<Tensor> w_out,
                   std::vector<Tensor> post_norm, std::vector<Tensor> w_gu, std::vector<Tensor> w_down,
                   std::vector<Tensor> rec_state, std::vector<Tensor> conv_state, std::vector<Tensor> conv_w,
                   std::vector<Tensor> A_log, std::vector<Tensor> dt_bias, std::vector<Tensor> gnorm_w,
                   c10::optional<Tensor> seg_slot, int64_t nk, int64_t nv, int64_t dk, double eps, Tensor status,
                   Tensor sync_words) {
  const int n = (int)start_phase.size();
  const int M = (int)x_in.size(0), hidden = (int)x_in.size(1);
  TORCH_CHECK(n >= 1 && n <= fb_decode_layers_max(), "decode_layers: run length");
  for (auto* v : {&x_out, &x_mid, &act, &proj, &o, &w_in, &input_norm, &w_out, &post_norm, &w_gu, &w_down, &rec_state,
                  &conv_state, &conv_w, &A_log, &dt_bias, &gnorm_w})
    TORCH_CHECK((int)v->size() == n, "decode_layers: one entry per layer in every list");
  TORCH_CHECK(x_in.is_contiguous(), "decode_layers: contiguous rows");
  TORCH_CHECK(sync_words.numel() >= 2 && sync_words.scalar_type() == torch::kInt32, "decode_layers: sync words");
  const int inter = (int)w_down[0].size(1);
  std::vector<int> sp(n), n_in(n), k_outs(n);
  std::vector<void*> p_xout(n), p_xmid(n), p_act(n), p_proj(n), p_o(n), p_conv(n);
  std::vector<const void*> p_win(n), p_inorm(n), p_wout(n), p_pnorm(n), p_wgu(n), p_wdown(n), p_convw(n), p_gnorm(n);
  std::vector<float*> p_rec(n);
  std::vector<const float*> p_alog(n), p_dtb(n);
  auto ptr = [](const Tensor& t) -> void* { return (t.defined() && t.numel() > 0) ? t.data_ptr() : nullptr; };
  for (int i = 0; i < n; ++i) {
    sp[i] = (int)start_phase[i];
    const int k_out = (int)w_out[i].size(1);
    k_outs[i] = k_out;
    TORCH_CHECK(x_out[i].is_contiguous() && x_mid[i].is_contiguous() && act[i].is_contiguous() && o[i].is_contiguous() &&
                w_out[i].is_contiguous() && w_gu[i].is_contiguous() && w_down[i].is_contiguous(), "decode_layers: contiguous");
    TORCH_CHECK(w_out[i].size(0) == hidden && w_out[i].size(1) == k_out && o[i].size(1) == k_out &&
                w_gu[i].size(1) == hidden && w_gu[i].size(0) == 2 * inter && w_down[i].size(0) == hidden &&
                w_down[i].size(1) == inter && act[i].size(1) == inter && x_out[i].size(1) == hidden &&
                x_mid[i].size(1) == hidden, "decode_layers: shapes");
    if (sp[i] == 1) {
      TORCH_CHECK(w_in[i].is_contiguous() && w_in[i].size(1) == hidden && proj[i].is_contiguous() &&
                  proj[i].size(1) == w_in[i].size(0) && rec_state[i].numel() > 0 && conv_state[i].numel() > 0 &&
                  seg_slot.has_value() && seg_slot->numel() >= M && k_out == nv * dk,
                  "decode_layers: Gated DeltaNet operands");
      n_in[i] = (int)w_in[i].size(0);
    } else {
      n_in[i] = 0;
    }
    p_xout[i] = x_out[i].data_ptr(); p_xmid[i] = x_mid[i].data_ptr(); p_act[i] = act[i].data_ptr();
    p_proj[i] = ptr(proj[i]) ? ptr(proj[i]) : x_mid[i].data_ptr(); p_o[i] = o[i].data_ptr();
    p_win[i] = ptr(w_in[i]); p_inorm[i] = ptr(input_norm[i]); p_wout[i] = w_out[i].data_ptr();
    p_pnorm[i] = post_norm[i].data_ptr(); p_wgu[i] = w_gu[i].data_ptr(); p_wdown[i] = w_down[i].data_ptr();
    p_rec[i] = (float*)ptr(rec_state[i]); p_conv[i] = ptr(conv_state[i]); p_convw[i] = ptr(conv_w[i]);
    p_alog[i] = (const float*)ptr(A_log[i]); p_dtb[i] = (const float*)ptr(dt_bias[i]); p_gnorm[i] = ptr(gnorm_w[i]);
  }
  const Comm* c = comm.is_none() ? nullptr : comm.cast<const Comm*>();
  check(fb_decode_layers(n, sp.data(), M, hidden, x_in.data_ptr(), p_xout.data(), p_xmid.data(), p_act.data(),
                         p_proj.data(), p_o.data(), p_win.data(), n_in.data(), p_inorm.data(), p_wout.data(), k_outs.data(),
                         p_pnorm.data(), p_wgu.data(), inter, p_wdown.data(), p_rec.data(), p_conv.data(), p_convw.data(),
                         p_alog.data(), p_dtb.data(), p_gnorm.data(),
                         seg_slot.has_value() ? seg_slot->data_ptr<int>() : nullptr, (int)nk, (int)nv, (int)dk, (float)eps,
                         c ? c->peers.data() : nullptr, c ? c->rank : 0, c ? c->world : 1, c ? c->max_ctas : 0,
                         c ? c->slot_floats : 0, c ? (uint32_t*)c->epochs.data_ptr() : nullptr, status.data_ptr<int>(),
                         c ? c->spin_limit : 0u, (uint32_t*)sync_words.data_ptr(),
                         at::cuda::getCurrentDeviceProperties()->multiProcessorCount, cur_stream()), "decode_layers");
}

void decode_layer_trace_set(c10::optional<Tensor> buf) {
  if (buf.has_value()) TORCH_CHECK(buf->scalar_type() == torch::kInt64 && buf->numel() >= 1024 * 16, "trace: int64[1024 * 16]");
  fb_decode_layer_trace_set(buf.has_value() ? buf->data_ptr() : nullptr);
}

void argmax_gather(const Comm& c, Tensor ids, Tensor logits, int64_t vocab_offset, c10::optional<Tensor> vals) {
  check(fb_argmax_gather(ids.data_ptr<int>(), vals.has_value() ? vals->data_ptr<float>() : nullptr,
                         logits.data_ptr<float>(), (long)logits.stride(0), (int)logits.size(0), (int)logits.size(1),
                         (int)vocab_offset, c.peers.data(), c.rank, c.world, c.max_ctas, c.slot_floats,
                         (uint32_t*)c.epochs.data_ptr(), c.status.data_ptr<int>(), c.spin_limit, cur_stream()),
        "argmax_gather");
}

void comm_wait_probe(Tensor flag, int64_t want, int64_t limit, Tensor status) {
  check(fb_comm_wait_probe((const uint32_t*)flag.data_ptr(), (uint32_t)want, (unsigned)limit, status.data_ptr<int>(),
                           cur_stream()), "comm_wait_probe");
}

void gemv_nvfp4(Tensor Y, Tensor X, Tensor packed, Tensor scales, double global_scale, c10::optional<Tensor> norm_w,
                c10::optional<Tensor> res, double eps, int64_t mode, c10::optional<Tensor> row_alpha) {
  int M = (int)X.size(0), K = (int)X.size(1);
  int N = (int)(mode == 1 ? packed.size(0) / 2 : packed.size(0));
  TORCH_CHECK(packed.size(1) * 2 == K, "gemv_nvfp4: K mismatch");
  TORCH_CHECK(!row_alpha.has_value() || (row_alpha->scalar_type() == torch::kFloat32 && row_alpha->numel() == packed.size(0)),
              "gemv_nvfp4: row_alpha is fp32 [weight rows]");
  check(fb_gemv_nvfp4(Y.data_ptr(), X.data_ptr(), packed.data_ptr(), scales.data_ptr(), (float)global_scale,
                      cptr(norm_w), cptr(res), M, N, K, (long)X.stride(0), (long)Y.stride(0), (long)scales.stride(0),
                      (float)eps, Y.scalar_type() == torch::kFloat32 ? 1 : 0, (int)mode,
                      at::cuda::getCurrentDeviceProperties()->multiProcessorCount, (const float*)cptr(row_alpha),
                      cur_stream()), "gemv_nvfp4");
}

void gemv_nvfp4_allreduce(const Comm& c, Tensor Y, Tensor X, Tensor packed, Tensor scales, double global_scale,
                          c10::optional<Tensor> res, c10::optional<Tensor> row_alpha) {
  int M = (int)X.size(0), K = (int)X.size(1), N = (int)packed.size(0);
  TORCH_CHECK(packed.size(1) * 2 == K, "gemv_nvfp4_allreduce: K mismatch");
  check(fb_gemv_nvfp4_allreduce(Y.data_ptr(), X.data_ptr(), packed.data_ptr(), scales.data_ptr(), (float)global_scale,
                                cptr(res), M, N, K, (long)X.stride(0), (long)Y.stride(0), (long)scales.stride(0),
                                c.peers.data(), c.rank, c.world, c.max_ctas, c.slot_floats,
                                (uint32_t*)c.epochs.data_ptr(), c.status.data_ptr<int>(), c.spin_limit, c.max_resident,
                                (const float*)cptr(row_alpha), cur_stream()), "gemv_nvfp4_allreduce");
}

int64_t nvfp4_sf_bytes(int64_t rows, int64_t K) { return fb_nvfp4_sf_bytes((int)rows, (int)K); }

void quant_nvfp4(Tensor codes, Tensor sf, Tensor row_scale, Tensor x, c10::optional<Tensor> norm_w, double eps) {
  check(fb_quant_nvfp4(codes.data_ptr(), sf.data_ptr(), row_scale.data_ptr<float>(), x.data_ptr(), (long)x.stride(0),
                       cptr(norm_w), (int)x.size(0), (int)x.size(1), (float)eps, cur_stream()), "quant_nvfp4");
}

int64_t gemm_nvfp4_workspace_bytes(int64_t M, int64_t N, int64_t split_k) {
  return fb_gemm_nvfp4_workspace_bytes((int)M, (int)N, (int)split_k);
}

void gemm_nvfp4(Tensor Y, Tensor xq, Tensor x_sf, Tensor row_scale, Tensor wq, Tensor w_sf, double w_scale,
                c10::optional<Tensor> res, int64_t mode, int64_t split_k, c10::optional<Tensor> workspace,
                c10::optional<Tensor> counters, c10::optional<Tensor> status) {
  int M = (int)xq.size(0), K = (int)xq.size(1) * 2;
  int N = (int)(mode == 1 ? wq.size(0) / 2 : wq.size(0));
  TORCH_CHECK(wq.size(1) * 2 == K, "gemm_nvfp4: K mismatch");
  check(fb_gemm_nvfp4(Y.data_ptr(), xq.data_ptr(), x_sf.data_ptr(), row_scale.data_ptr<float>(), wq.data_ptr(),
                      w_sf.data_ptr(), (float)w_scale, cptr(res), M, N, K, (long)Y.stride(0), (int)mode, (int)split_k,
                      workspace.has_value() ? (float*)workspace->data_ptr() : nullptr,
                      counters.has_value() ? (int*)counters->data_ptr() : nullptr,
                      status.has_value() ? (int*)status->data_ptr() : nullptr,
                      at::cuda::getCurrentDeviceProperties()->multiProcessorCount, cur_stream()), "gemm_nvfp4");
}

void gemm_nvfp4_swiglu_q(Tensor q_codes, Tensor q_sf, Tensor q_row_scale, double q_gs, Tensor xq, Tensor x_sf,
                         Tensor row_scale, Tensor wq, Tensor w_sf, double w_scale, Tensor status) {
  int M = (int)xq.size(0), K = (int)xq.size(1) * 2, N = (int)wq.size(0) / 2;
  TORCH_CHECK(wq.size(1) * 2 == K && q_codes.size(0) == M && q_codes.size(1) * 2 == N && q_row_scale.numel() >= M,
              "gemm_nvfp4_swiglu_q: shapes");
  TORCH_CHECK(q_sf.numel() >= fb_nvfp4_sf_bytes(M, N), "gemm_nvfp4_swiglu_q: scale buffer too small");
  check(fb_gemm_nvfp4_swiglu_q(q_codes.data_ptr(), q_sf.data_ptr(), q_row_scale.data_ptr<float>(), (float)q_gs, xq.data_ptr(),
                               x_sf.data_ptr(), row_scale.data_ptr<float>(), wq.data_ptr(), w_sf.data_ptr(), (float)w_scale,
                               M, N, K, status.data_ptr<int>(),
                               at::cuda::getCurrentDeviceProperties()->multiProcessorCount, cur_stream()),
        "gemm_nvfp4_swiglu_q");
}

void gemm_nvfp4_fused(Tensor Y, Tensor X, c10::optional<Tensor> norm_w, double eps, Tensor wq, Tensor w_sf,
                      double w_scale, c10::optional<Tensor> res, int64_t mode, int64_t split_k,
                      c10::optional<Tensor> workspace, c10::optional<Tensor> counters, c10::optional<Tensor> status) {
  int M = (int)X.size(0), K = (int)X.size(1);
  int N = (int)(mode == 1 ? wq.size(0) / 2 : wq.size(0));
  TORCH_CHECK(wq.size(1) * 2 == K, "gemm_nvfp4_fused: K mismatch");
  check(fb_gemm_nvfp4_fused(Y.data_ptr(), X.data_ptr(), (long)X.stride(0), cptr(norm_w), (float)eps, wq.data_ptr(),
                            w_sf.data_ptr(), (float)w_scale, cptr(res), M, N, K, (long)Y.stride(0), (int)mode,
                            (int)split_k, Y.scalar_type() == torch::kFloat32 ? 1 : 0,
                            workspace.has_value() ? (float*)workspace->data_ptr() : nullptr,
                            counters.has_value() ? (int*)counters->data_ptr() : nullptr,
                            status.has_value() ? (int*)status->data_ptr() : nullptr,
                            at::cuda::getCurrentDeviceProperties()->multiProcessorCount, cur_stream()),
        "gemm_nvfp4_fused");
}

int64_t gemv_nvfp4_tc_workspace_bytes(int64_t M, int64_t N, int64_t K, bool dual, int64_t terms, int64_t ctas_per_sm) {
  return fb_gemv_nvfp4_tc_workspace_bytes((int)M, (int)N, (int)K, dual ? 1 : 0, (int)terms,
                                          at::cuda::getCurrentDeviceProperties()->multiProcessorCount, (int)ctas_per_sm);
}

int64_t gemv_nvfp4_tc_terms(int64_t M, int64_t N, int64_t K, bool dual, int64_t terms) {
  return fb_gemv_nvfp4_tc_terms((int)M, (int)N, (int)K, dual ? 1 : 0, (int)terms);
}

void gemv_nvfp4_tc_trace_set(c10::optional<Tensor> buf) {
  if (buf.has_value()) TORCH_CHECK(buf->scalar_type() == torch::kInt64 && buf->numel() >= 8 * 1024 * 8, "trace: int64[8 * 1024 * 8]");
  fb_gemv_nvfp4_tc_trace_set(buf.has_value() ? buf->data_ptr() : nullptr);
}

void gemv_nvfp4_tc(Tensor Y, Tensor X, c10::optional<Tensor> norm_w, double eps, Tensor wq, Tensor w_sf, double w_scale,
                   c10::optional<Tensor> row_alpha, c10::optional<Tensor> res, int64_t mode, int64_t terms,
                   c10::optional<Tensor> workspace, c10::optional<Tensor> counters, c10::optional<Tensor> status,
                   int64_t ctas_per_sm, c10::optional<Tensor> next_wq, c10::optional<Tensor> next_sf, int64_t next_mode,
                   int64_t prefetch_bytes) {
  int M = (int)X.size(0), K = (int)X.size(1);
  int N = (int)(mode == 1 ? wq.size(0) / 2 : wq.size(0));
  TORCH_CHECK(wq.size(1) * 2 == K, "gemv_nvfp4_tc: K mismatch");
  const bool pf = next_wq.has_value() && next_sf.has_value() && next_wq->is_contiguous();
  int next_N = pf ? (int)(next_mode == 1 ? next_wq->size(0) / 2 : next_wq->size(0)) : 0;
  int next_K = pf ? (int)next_wq->size(1) * 2 : 0;
  TORCH_CHECK(X.stride(1) == 1 && Y.stride(1) == 1 && wq.is_contiguous(), "gemv_nvfp4_tc: layout");
  check(fb_gemv_nvfp4_tc(Y.data_ptr(), X.data_ptr(), (long)X.stride(0), cptr(norm_w), (float)eps, wq.data_ptr(),
                         w_sf.data_ptr(), (float)w_scale, (const float*)cptr(row_alpha), cptr(res), M, N, K,
                         (long)Y.stride(0), (int)mode, (int)terms, Y.scalar_type() == torch::kFloat32 ? 1 : 0,
                         workspace.has_value() ? (float*)workspace->data_ptr() : nullptr,
                         counters.has_value() ? (int*)counters->data_ptr() : nullptr,
                         status.has_value() ? (int*)status->data_ptr() : nullptr,
                         at::cuda::getCurrentDeviceProperties()->multiProcessorCount, (int)ctas_per_sm,
                         pf ? next_wq->data_ptr() : nullptr, pf ? next_sf->data_ptr() : nullptr, next_N, next_K,
                         (int)next_mode, (long)prefetch_bytes, cur_stream()),
        "gemv_nvfp4_tc");
}

void moe_route(Tensor ids, Tensor wts, Tensor logits, c10::optional<Tensor> bias, int64_t mode, int64_t n_groups,
               int64_t topk_groups, double scale, int64_t n_exp, int64_t shared_col, int64_t shared_id) {
  // logits [rows, >= n_exp] fp32 (n_exp <= 0: every column is an expert); ids / wts [rows, top_k (+ 1 with a shared expert)]
  const int ne = n_exp > 0 ? (int)n_exp : (int)logits.size(1);
  const int top_k = (int)ids.size(1) - (shared_id >= 0 ? 1 : 0);
  check(fb_moe_route(ids.data_ptr<int>(), wts.data_ptr<float>(), logits.data_ptr<float>(),
                     bias.has_value() ? bias->data_ptr<float>() : nullptr, (int)logits.size(0), ne, top_k, (int)mode,
                     (int)n_groups, (int)topk_groups, (float)scale, (int)logits.stride(0), (int)shared_col, (int)shared_id,
                     cur_stream()), "moe_route");
}

void moe_experts(Tensor out, Tensor act, Tensor yp, Tensor x, Tensor w_gu, Tensor w_down, Tensor ids, Tensor wts,
                 int64_t e_lo, int64_t e_hi, c10::optional<Tensor> shared, c10::optional<Tensor> shared_gate,
                 c10::optional<Tensor> res) {
  int rows = (int)x.size(0), hidden = (int)x.size(1), top_k = (int)ids.size(1), inter = (int)w_down.size(2);
  int pairs = rows * top_k;
  check(fb_moe_gate_up(act.data_ptr(), x.data_ptr(), w_gu.data_ptr(), ids.data_ptr<int>(), pairs, top_k, hidden, inter,
                       (int)e_lo, (int)e_hi, cur_stream()), "moe_gate_up");
  check(fb_moe_down(yp.data_ptr<float>(), act.data_ptr(), w_down.data_ptr(), ids.data_ptr<int>(), pairs, hidden, inter,
                    (int)e_lo, (int)e_hi, cur_stream()), "moe_down");
  check(fb_moe_combine(out.data_ptr(), yp.data_ptr<float>(), wts.data_ptr<float>(), cptr(shared),
                       shared_gate.has_value() ? shared_gate->data_ptr<float>() : nullptr, cptr(res), rows, top_k,
                       hidden, out.scalar_type() == torch::kFloat32 ? 1 : 0, cur_stream()), "moe_combine");
}

void moe_experts_fp4(Tensor out, Tensor act, Tensor yp, Tensor x, Tensor gu_q, Tensor gu_s, double gu_scale, Tensor dn_q,
                     Tensor dn_s, double dn_scale, Tensor ids, Tensor wts, int64_t e_lo, int64_t e_hi,
                     c10::optional<Tensor> shared, c10::optional<Tensor> shared_gate, c10::optional<Tensor> res) {
  int rows = (int)x.size(0), hidden = (int)x.size(1), top_k = (int)ids.size(1), inter = (int)dn_q.size(2) * 2;
  int pairs = rows * top_k;
  TORCH_CHECK(gu_q.size(1) == 2 * inter && gu_q.size(2) * 2 == hidden && dn_q.size(1) == hidden, "moe_experts_fp4: shapes");
  check(fb_moe_gate_up_fp4(act.data_ptr(), x.data_ptr(), gu_q.data_ptr(), gu_s.data_ptr(), (float)gu_scale,
                           ids.data_ptr<int>(), pairs, top_k, hidden, inter, (int)e_lo, (int)e_hi, cur_stream()),
        "moe_gate_up_fp4");
  check(fb_moe_down_fp4(yp.data_ptr<float>(), act.data_ptr(), dn_q.data_ptr(), dn_s.data_ptr(), (float)dn_scale,
                        ids.data_ptr<int>(), pairs, hidden, inter, (int)e_lo, (int)e_hi, cur_stream()), "moe_down_fp4");
  check(fb_moe_combine(out.data_ptr(), yp.data_ptr<float>(), wts.data_ptr<float>(), cptr(shared),
                       shared_gate.has_value() ? shared_gate->data_ptr<float>() : nullptr, cptr(res), rows, top_k,
                       hidden, out.scalar_type() == torch::kFloat32 ? 1 : 0, cur_stream()), "moe_combine");
}

void nvfp4_dequant(Tensor out, Tensor wq, Tensor ws, double gscale) {
  TORCH_CHECK(out.numel() == wq.numel() * 2 && ws.numel() * 16 == out.numel(), "nvfp4_dequant: sizes");
  check(fb_nvfp4_dequant(out.data_ptr(), wq.data_ptr(), ws.data_ptr(), (float)gscale, (long)out.numel(), cur_stream()),
        "nvfp4_dequant");
}

// Handle to the large symmetric workspace used by the GEMMs with a fused reduce-scatter / all-gather.
struct BigComm {
  std::vector<const void*> peers;
  int rank = 0, world = 1, sm = 148;
  long max_rows = 0, max_cols = 0;
  Tensor ctr, status;
  unsigned spin_limit = 0;
};

BigComm make_big_comm(std::vector<int64_t> peer_ptrs, int64_t rank, int64_t max_rows, int64_t max_cols, Tensor ctr,
                      Tensor status, int64_t spin_limit, int64_t sm) {
  BigComm c;
  for (auto p : peer_ptrs) c.peers.push_back(reinterpret_cast<const void*>(p));
  c.rank = (int)rank; c.world = (int)peer_ptrs.size(); c.max_rows = max_rows; c.max_cols = max_cols;
  c.ctr = ctr; c.status = status; c.spin_limit = (unsigned)spin_limit; c.sm = (int)sm;
  TORCH_CHECK(ctr.numel() >= 2 + (max_rows + 127) / 128, "make_big_comm: counter array too small");
  return c;
}

void gemm_rs(const BigComm& c, Tensor y_shard, Tensor X, Tensor W, c10::optional<Tensor> res_shard) {
  check(fb_gemm_rs(y_shard.data_ptr(), X.data_ptr(), W.data_ptr(), cptr(res_shard), (int)X.size(0), (int)W.size(0),
                   (int)X.size(1), (long)X.stride(0), c.peers.data(), c.rank, c.world, c.max_rows, c.max_cols,
                   (uint32_t*)c.ctr.data_ptr(), c.status.data_ptr<int>(), c.spin_limit, c.sm, cur_stream()), "gemm_rs");
}

void ag_gemm(const BigComm& c, Tensor Y, Tensor W, c10::optional<Tensor> res, int64_t K, int64_t mode) {
  int M = (int)Y.size(0);
  int N = (int)(mode == 1 ? W.size(0) / 2 : W.size(0));
  TORCH_CHECK(W.size(1) == K, "ag_gemm: K mismatch");
  check(fb_ag_gemm(Y.data_ptr(), W.data_ptr(), cptr(res), M, N, (int)K, (long)Y.stride(0), (int)mode, c.peers.data(),
                   c.rank, c.world, c.max_rows, c.max_cols, (uint32_t*)c.ctr.data_ptr(), c.status.data_ptr<int>(),
                   c.spin_limit, c.sm, cur_stream()), "ag_gemm");
}

// Handle to the symmetric workspace of the expert-parallel MoE block.
struct EpHandle {
  std::vector<const void*> peers;
  int rank = 0, world = 1, n_experts = 0, hidden = 0, sm = 148;
  long cap_rows = 0;
  Tensor ctr, status;
  unsigned spin_limit = 0;
};

EpHandle make_ep_comm(std::vector<int64_t> peer_ptrs, int64_t rank, int64_t n_experts, int64_t hidden, int64_t cap_rows,
                      Tensor ctr, Tensor status, int64_t spin_limit, int64_t sm) {
  EpHandle c;
  for (auto p : peer_ptrs) c.peers.push_back(reinterpret_cast<const void*>(p));
  c.rank = (int)rank; c.world = (int)peer_ptrs.size(); c.n_experts = (int)n_experts; c.hidden = (int)hidden;
  c.cap_rows = cap_rows; c.ctr = ctr; c.status = status; c.spin_limit = (unsigned)spin_limit; c.sm = (int)sm;
  return c;
}

void ep_moe(const EpHandle& c, Tensor out, Tensor x, Tensor ids, Tensor wts, Tensor w_gu, Tensor w_down,
            c10::optional<Tensor> shared, c10::optional<Tensor> shared_gate, c10::optional<Tensor> res, Tensor act,
            Tensor plan) {
  int rows = (int)x.size(0), top_k = (int)ids.size(1), inter = (int)w_down.size(2);
  TORCH_CHECK(plan.numel() >= (int64_t)rows * top_k + 3 * c.n_experts + 8, "ep_moe: plan scratch too small");
  TORCH_CHECK(act.numel() >= c.cap_rows * inter, "ep_moe: activation scratch too small");
  check(fb_ep_moe(out.data_ptr(), x.data_ptr(), ids.data_ptr<int>(), wts.data_ptr<float>(), w_gu.data_ptr(),
                  w_down.data_ptr(), cptr(shared), shared_gate.has_value() ? shared_gate->data_ptr<float>() : nullptr,
                  cptr(res), act.data_ptr(), plan.data_ptr<int>(), rows, top_k, c.n_experts, c.hidden, inter, c.cap_rows,
                  c.peers.data(), c.rank, c.world, (uint32_t*)c.ctr.data_ptr(), c.status.data_ptr<int>(), c.spin_limit,
                  c.sm, cur_stream()), "ep_moe");
}

void gemm_grouped(Tensor Y, Tensor X, Tensor W, Tensor tile_start, Tensor row_base, int64_t mode, Tensor status) {
  int experts = (int)W.size(0);
  int N = (int)(mode == 1 ? W.size(1) / 2 : W.size(1));
  check(fb_gemm_grouped(Y.data_ptr(), X.data_ptr(), W.data_ptr(), tile_start.data_ptr<int>(), row_base.data_ptr<int>(),
                        experts, (int)X.size(0), N, (int)X.size(1), (long)X.stride(0), (long)Y.stride(0), (int)mode,
                        status.data_ptr<int>(), 0, cur_stream()), "gemm_grouped");
}

void gemm_batched(Tensor Y, Tensor X, Tensor W, Tensor status) {
  // X [groups, rows, K], W [groups, N, K], Y [groups, rows, N], all contiguous bf16
  TORCH_CHECK(X.is_contiguous() && W.is_contiguous() && Y.is_contiguous() && X.dim() == 3 && W.dim() == 3 && Y.dim() == 3,
              "gemm_batched: contiguous [groups, rows, K] x [groups, N, K] -> [groups, rows, N]");
  TORCH_CHECK(X.size(0) == W.size(0) && X.size(2) == W.size(2) && Y.size(0) == X.size(0) && Y.size(1) == X.size(1) &&
              Y.size(2) == W.size(1), "gemm_batched: shapes");
  check(fb_gemm_batched(Y.data_ptr(), X.data_ptr(), W.data_ptr(), (int)X.size(0), (int)X.size(1), (int)W.size(1),
                        (int)X.size(2), status.data_ptr<int>(), 0, cur_stream()), "gemm_batched");
}

void head_linear(Tensor y, Tensor x, Tensor W) {
  // x [T, heads, >= K] and y [T, heads, >= N]: views with unit stride in the last dimension; W [heads, N, K] contiguous
  TORCH_CHECK(x.dim() == 3 && y.dim() == 3 && W.dim() == 3 && W.is_contiguous() && x.stride(2) == 1 && y.stride(2) == 1,
              "head_linear: layouts");
  TORCH_CHECK(x.size(0) == y.size(0) && x.size(1) == W.size(0) && y.size(1) == W.size(0) && x.size(2) == W.size(2) &&
              y.size(2) == W.size(1), "head_linear: shapes");
  check(fb_head_linear(y.data_ptr(), x.data_ptr(), W.data_ptr(), (int)x.size(0), (int)W.size(0), (int)W.size(1),
                       (int)W.size(2), (long)x.stride(0), (long)x.stride(1), (long)y.stride(0), (long)y.stride(1),
                       cur_stream()), "head_linear");
}

// ---- sparse-attention selection, drafting heads, Engram gate -------------------------------------------------------
using OptT = c10::optional<Tensor>;

void engram_gate(Tensor out, Tensor h, OptT kvp, OptT kvb, Tensor qk, double eps) {
  // h / out [rows, hc, d] bf16; kvb [rows, (hc + 1) d] bf16 or kvp [world, rows, (hc + 1) d] fp32; qk [hc, d] fp32
  const int world = kvp.has_value() ? (int)kvp->size(0) : 0;
  check(fb_engram_gate(out.data_ptr(), h.data_ptr(), world ? kvp->data_ptr<float>() : nullptr, cptr(kvb),
                       qk.data_ptr<float>(), (int)h.size(0), (int)h.size(1), (int)h.size(2), world, (float)eps, cur_stream()),
        "engram_gate");
}

void comp_step(Tensor out, Tensor tail, Tensor kvc, OptT sc, Tensor row_slot, Tensor row_pos, int64_t ratio) {
  // tail [slots, ring_len, 2 dim] fp32; kvc / sc [rows, dim] fp32; out [rows, dim] bf16
  check(fb_comp_step(out.data_ptr(), tail.data_ptr<float>(), kvc.data_ptr<float>(),
                     sc.has_value() ? sc->data_ptr<float>() : nullptr, row_slot.data_ptr<int>(), row_pos.data_ptr<int>(),
                     (int)kvc.size(0), (int)ratio, (int)kvc.size(1), (int)tail.size(1), cur_stream()), "comp_step");
}

void index_score(Tensor score, Tensor q, OptT w, double scale, Tensor keys, Tensor row_slot, Tensor row_len, OptT mask,
                 int64_t mask_block) {
  // score [rows, ld] fp32; q [rows, nh, D] bf16; w [rows, nh] fp32; keys [slots, entries, D] bf16; mask [rows, mask_ld] u8
  TORCH_CHECK(q.is_contiguous() && keys.is_contiguous() && score.is_contiguous(), "index_score: contiguous tensors");
  check(fb_index_score(score.data_ptr<float>(), (int)score.size(1), q.data_ptr(), w.has_value() ? w->data_ptr<float>() : nullptr,
                       (float)scale, keys.data_ptr(), (long)keys.stride(0), row_slot.data_ptr<int>(), row_len.data_ptr<int>(),
                       mask.has_value() ? mask->data_ptr<uint8_t>() : nullptr, mask.has_value() ? (int)mask->size(1) : 0,
                       (int)mask_block, (int)q.size(0), (int)q.size(1), (int)q.size(2), cur_stream()), "index_score");
}

void topk_select(Tensor sel, Tensor score, OptT row_n) {
  // sel [rows, k] int32; score [rows, ld] fp32; row_n [rows] int32 (entries that count; all when absent)
  check(fb_topk_select(sel.data_ptr<int>(), score.data_ptr<float>(), (int)score.stride(0), (int)score.size(1),
                       row_n.has_value() ? row_n->data_ptr<int>() : nullptr, (int)score.size(0), (int)sel.size(1), cur_stream()),
        "topk_select");
}

void block_max(Tensor bmax, Tensor score, Tensor row_n, int64_t bsize) {
  check(fb_block_max(bmax.data_ptr<float>(), (int)bmax.size(1), score.data_ptr<float>(), (int)score.stride(0),
                     row_n.data_ptr<int>(), (int)score.size(0), (int)bsize, cur_stream()), "block_max");
}

void sel_to_mask(Tensor mask, Tensor sel) {
  check(fb_sel_to_mask(mask.data_ptr<uint8_t>(), (int)mask.size(1), sel.data_ptr<int>(), (int)sel.size(0), (int)sel.size(1),
                       cur_stream()), "sel_to_mask");
}

void qsa_pool(Tensor pooled, Tensor raw, Tensor w, Tensor pos0, Tensor inv_freq, double eps) {
  // raw [blocks, kp, D] fp32 -> pooled [blocks, D] bf16
  check(fb_qsa_pool(pooled.data_ptr(), raw.data_ptr<float>(), w.data_ptr<float>(), pos0.data_ptr<int>(),
                    inv_freq.data_ptr<float>(), (int)raw.size(0), (int)raw.size(1), (int)raw.size(2),
                    2 * (int)inv_freq.size(0), (float)eps, cur_stream()), "qsa_pool");
}

void qsa_table(Tensor table, Tensor kvlen, Tensor sel, Tensor row_slot, Tensor row_pos, Tensor block_table, int64_t kp,
               Tensor status) {
  // table [rows, top + 1], sel [rows, top]
  TORCH_CHECK(table.size(1) == sel.size(1) + 1, "qsa_table: table holds top + 1 blocks per row");
  check(fb_qsa_table(table.data_ptr<int>(), kvlen.data_ptr<int>(), sel.data_ptr<int>(), row_slot.data_ptr<int>(),
                     row_pos.data_ptr<int>(), block_table.data_ptr<int>(), (int)block_table.size(1), (int)sel.size(0),
                     (int)kp, (int)sel.size(1), status.data_ptr<int>(), cur_stream()), "qsa_table");
}

void markov_bias(Tensor out, Tensor head, Tensor emb, Tensor tok, Tensor slot) {
  check(fb_markov_bias(out.data_ptr(), head.data_ptr(), emb.data_ptr(), tok.data_ptr<int>(), slot.data_ptr<int>(),
                       (int)out.size(0), (int)head.size(0), (int)head.size(1), cur_stream()), "markov_bias");
}

void markov_score(Tensor pair, Tensor logits, Tensor stage, Tensor cache, Tensor slot, int64_t col0) {
  // pair [parts, rows, 2] int32; logits [rows, >= n] fp32; stage [rows, n] / cache [slots, n] bf16
  check(fb_markov_score(pair.data_ptr(), logits.data_ptr<float>(), (long)logits.stride(0), stage.data_ptr(), cache.data_ptr(),
                        slot.data_ptr<int>(), (int)pair.size(1), (int)pair.size(0), (int)stage.size(1), (int)col0, cur_stream()),
        "markov_score");
}

void markov_pick(Tensor draft, Tensor tok, Tensor slot, Tensor pairs, Tensor slot_of, int64_t step, Tensor status) {
  // pairs [n_pairs, rows, 2]; draft [rows, stride]; step < 0 starts a loop from draft[:, 0]
  check(fb_markov_pick(draft.data_ptr<int>(), tok.data_ptr<int>(), slot.data_ptr<int>(), pairs.data_ptr(),
                       slot_of.data_ptr<int>(), (int)pairs.size(0), (int)draft.size(0), (int)draft.stride(0), (int)step,
                       (int)slot_of.size(0), status.data_ptr<int>(), cur_stream()), "markov_pick");
}

void conf_head(Tensor conf, Tensor xc, Tensor emb, Tensor draft, Tensor w, int64_t steps, int64_t block) {
  // conf [streams * steps]; xc [streams * block, d]; emb [vocab, rank]; draft [streams, stride]; w [d + rank] fp32
  check(fb_conf_head(conf.data_ptr<float>(), xc.data_ptr(), emb.data_ptr(), draft.data_ptr<int>(), w.data_ptr<float>(),
                     (int)draft.size(0), (int)steps, (int)xc.size(1), (int)emb.size(1), (int)block, (int)draft.stride(0),
                     cur_stream()), "conf_head");
}

void stream_mean(Tensor out, Tensor h) {
  check(fb_stream_mean(out.data_ptr(), (long)out.stride(0), h.data_ptr(), (int)h.size(0), (int)h.size(1), (int)h.size(2),
                       cur_stream()), "stream_mean");
}

void stream_collapse(Tensor xc, Tensor h, Tensor pre) {
  check(fb_stream_collapse(xc.data_ptr(), h.data_ptr(), pre.data_ptr<float>(), (long)pre.stride(0), (int)h.size(0),
                           (int)h.size(1), (int)h.size(2), cur_stream()), "stream_collapse");
}

void gguf_dequant(Tensor out, Tensor raw, int64_t type) {
  check(fb_gguf_dequant(out.data_ptr(), raw.data_ptr(), (int)type, (long)out.numel(), cur_stream()), "gguf_dequant");
}

void q8_1_quant(Tensor out, Tensor x) {
  TORCH_CHECK(out.numel() >= x.numel() / 32 * 36, "q8_1_quant: output too small");
  check(fb_q8_1_quant(out.data_ptr(), x.data_ptr(), (long)x.numel(), cur_stream()), "q8_1_quant");
}

void gguf_gemv(Tensor y, Tensor x, Tensor raw, int64_t type, int64_t N, c10::optional<Tensor> res) {
  check(fb_gguf_gemv(y.data_ptr(), x.data_ptr(), raw.data_ptr(), cptr(res), (int)type, (int)x.size(0), (int)N,
                     (int)x.size(1), (long)x.stride(0), (long)y.stride(0), cur_stream()), "gguf_gemv");
}

void exl3_had(Tensor out, Tensor in, c10::optional<Tensor> pre, c10::optional<Tensor> post, c10::optional<Tensor> res,
              double scale) {
  check(fb_exl3_had(out.data_ptr(), in.data_ptr(), cptr(pre), cptr(post), cptr(res), (int)in.size(0), (int)in.size(1),
                    (float)scale, in.scalar_type() == torch::kFloat32 ? 1 : 0, out.scalar_type() == torch::kBFloat16 ? 1 : 0,
                    cur_stream()), "exl3_had");
}

void exl3_gemv(Tensor z, Tensor xh, Tensor trellis, int64_t bits) {
  check(fb_exl3_gemv(z.data_ptr<float>(), xh.data_ptr<float>(), trellis.data_ptr(), (int)xh.size(0), (int)xh.size(1),
                     (int)z.size(1), (int)bits, cur_stream()), "exl3_gemv");
}

void exl3_decode(Tensor out, Tensor trellis, int64_t bits) {
  check(fb_exl3_decode(out.data_ptr(), trellis.data_ptr(), (int)out.size(1), (int)out.size(0), (int)bits, cur_stream()),
        "exl3_decode");
}

void mla_prep(Tensor cache, Tensor qabs, Tensor kva, Tensor q, Tensor norm_w, Tensor inv_freq, Tensor row_slot,
              Tensor row_pos, Tensor block_table, int64_t kv_block, int64_t nq, int64_t dn, int64_t L, int64_t R, double eps,
              Tensor status) {
  check(fb_mla_prep(cache.data_ptr(), qabs.data_ptr(), kva.data_ptr(), (long)kva.stride(0), q.data_ptr(), (long)q.stride(0),
                    norm_w.data_ptr(), inv_freq.data_ptr<float>(), row_slot.data_ptr<int>(), row_pos.data_ptr<int>(),
                    block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block, (int)q.size(0), (int)nq, (int)dn,
                    (int)L, (int)R, (float)eps, status.data_ptr<int>(), cur_stream()), "mla_prep");
}

void mla_attn(Tensor out, Tensor o_part, Tensor ml_part, Tensor qabs, Tensor cache, Tensor row_slot, Tensor row_kvlen,
              Tensor block_table, int64_t kv_block, int64_t nq, int64_t L, int64_t R, int64_t nsplit, double scale) {
  check(fb_mla_attn(out.data_ptr(), o_part.data_ptr<float>(), ml_part.data_ptr<float>(), qabs.data_ptr(), cache.data_ptr(),
                    row_slot.data_ptr<int>(), row_kvlen.data_ptr<int>(), block_table.data_ptr<int>(),
                    (int)block_table.size(1), (int)kv_block, (int)qabs.size(0), (int)nq, (int)L, (int)R, (int)nsplit,
                    (float)scale, cur_stream()), "mla_attn");
}

void mla_expand(Tensor kp, Tensor vp, Tensor kvx, Tensor lat, int64_t nq, int64_t dn, int64_t dv, int64_t L, int64_t R) {
  // kp / vp [rows, nq, HP]; kvx [rows, nq (dn + dv)]; lat [rows, L + R]; all contiguous bf16
  TORCH_CHECK(kp.is_contiguous() && vp.is_contiguous() && kvx.is_contiguous() && lat.is_contiguous(), "mla_expand: contiguous");
  check(fb_mla_expand(kp.data_ptr(), vp.data_ptr(), kvx.data_ptr(), lat.data_ptr(), (long)lat.size(0), (int)nq, (int)dn,
                      (int)dv, (int)L, (int)R, (int)kp.size(-1), cur_stream()), "mla_expand");
}

void mla_qpad(Tensor qp, Tensor q, Tensor qabs, int64_t nq, int64_t dn, int64_t L, int64_t R, double scale) {
  check(fb_mla_qpad(qp.data_ptr(), q.data_ptr(), (long)q.stride(0), qabs.data_ptr(), (long)q.size(0), (int)nq, (int)dn,
                    (int)L, (int)R, (int)qp.size(-1), (float)scale, cur_stream()), "mla_qpad");
}

void w4_gemv(Tensor y, Tensor x, Tensor qweight, Tensor scales, Tensor biases, c10::optional<Tensor> res) {
  check(fb_w4_gemv(y.data_ptr(), x.data_ptr(), qweight.data_ptr(), scales.data_ptr(), biases.data_ptr(), cptr(res),
                   (int)x.size(0), (int)qweight.size(0), (int)x.size(1), (long)x.stride(0), (long)y.stride(0), cur_stream()),
        "w4_gemv");
}

void hc_norm(Tensor y, Tensor rinv, Tensor x, Tensor w, double eps) {
  check(fb_hc_norm(y.data_ptr(), rinv.data_ptr<float>(), x.data_ptr<float>(), w.data_ptr<float>(), (int)x.size(0),
                   (int)x.size(1), (int)w.size(0), (float)eps, cur_stream()), "hc_norm");
}

void hc_mix(Tensor mixed, Tensor res, Tensor rinv, Tensor w, Tensor gate) {
  check(fb_hc_mix(mixed.data_ptr<float>(), res.data_ptr<float>(), rinv.data_ptr<float>(), w.data_ptr<float>(),
                  gate.data_ptr<float>(), (int)res.size(0), (int)res.size(2), (int)res.size(1), cur_stream()), "hc_mix");
}

void hc_combine(Tensor res, Tensor out, Tensor inj) {
  check(fb_hc_combine(res.data_ptr<float>(), out.data_ptr<float>(), inj.data_ptr<float>(), (int)res.size(0), (int)res.size(2),
                      (int)res.size(1), (long)inj.stride(0), cur_stream()), "hc_combine");
}

void dynconv(Tensor out, Tensor x, Tensor coef, Tensor base, c10::optional<Tensor> res, int64_t group, int64_t blk) {
  check(fb_dynconv(out.data_ptr(), x.data_ptr(), coef.data_ptr(), (long)coef.stride(0), base.data_ptr(), res.has_value() ? res->data_ptr() : nullptr,
                   (int)x.size(0), (int)x.size(1), (int)group, (int)blk, cur_stream()), "dynconv");
}

void topk16_merge(Tensor ovals, Tensor oids, Tensor vals, Tensor ids) {
  check(fb_topk16_merge(ovals.data_ptr<float>(), oids.data_ptr<int>(), vals.data_ptr<float>(), ids.data_ptr<int>(),
                        (int)vals.size(1), (int)vals.size(0), cur_stream()), "topk16_merge");
}

void draft_select(Tensor out, Tensor vals, Tensor ids, Tensor gate, Tensor a_cb, Tensor b_cb, int64_t anchor) {
  check(fb_draft_select(out.data_ptr<int>(), vals.data_ptr<float>(), ids.data_ptr<int>(), gate.data_ptr(), a_cb.data_ptr(),
                        b_cb.data_ptr(), (int)anchor, (int)vals.size(0), (int)gate.size(1), cur_stream()), "draft_select");
}

void topk16(Tensor ids, c10::optional<Tensor> vals, Tensor logits) {
  check(fb_topk16(ids.data_ptr<int>(), vals.has_value() ? vals->data_ptr<float>() : nullptr, logits.data_ptr(),
                  (long)logits.stride(0), (int)logits.size(0), (int)logits.size(1),
                  logits.scalar_type() == torch::kFloat32 ? 1 : 0, cur_stream()), "topk16");
}

}  // namespace

void register_ext(pybind11::module_& m) {
  m.def("w4_gemv", &w4_gemv);
  m.def("topk16", &topk16);
  m.def("dynconv", &dynconv);
  m.def("mla_expand", &mla_expand);
  m.def("mla_qpad", &mla_qpad);
  m.def("hc_norm", &hc_norm);
  m.def("hc_mix", &hc_mix);
  m.def("hc_combine", &hc_combine);
  m.def("engram_gate", &engram_gate);
  m.def("comp_step", &comp_step);
  m.def("index_score", &index_score);
  m.def("topk_select", &topk_select);
  m.def("block_max", &block_max);
  m.def("sel_to_mask", &sel_to_mask);
  m.def("qsa_pool", &qsa_pool);
  m.def("qsa_table", &qsa_table);
  m.def("markov_bias", &markov_bias);
  m.def("markov_score", &markov_score);
  m.def("markov_pick", &markov_pick);
  m.def("conf_head", &conf_head);
  m.def("stream_mean", &stream_mean);
  m.def("stream_collapse", &stream_collapse);
  m.def("topk16_merge", &topk16_merge);
  m.def("draft_select", &draft_select);
  m.def("mla_prep", &mla_prep);
  m.def("mla_attn", &mla_attn);
  m.def("exl3_had", &exl3_had);
  m.def("exl3_gemv", &exl3_gemv);
  m.def("exl3_decode", &exl3_decode);
  m.def("gguf_dequant", &gguf_dequant);
  m.def("q8_1_quant", &q8_1_quant);
  m.def("gguf_gemv", &gguf_gemv);
  pybind11::class_<EpHandle>(m, "EpHandle");
  m.def("make_ep_comm", &make_ep_comm);
  m.def("ep_workspace_bytes", [](int64_t e, int64_t h, int64_t cap) { return (int64_t)fb_ep_workspace_bytes((int)e, (int)h, cap); });
  m.def("ep_moe", &ep_moe);
  m.def("gemm_grouped", &gemm_grouped);
  m.def("gemm_batched", &gemm_batched);
  m.def("head_linear", &head_linear);
  pybind11::class_<BigComm>(m, "BigComm");
  m.def("make_big_comm", &make_big_comm);
  m.def("big_workspace_bytes", [](int64_t world, int64_t max_rows, int64_t max_cols) {
    return (int64_t)fb_big_workspace_bytes((int)world, (long)max_rows, (long)max_cols);
  });
  m.def("big_xfull_offset", [](int64_t world, int64_t max_rows, int64_t max_cols) {
    return (int64_t)fb_big_xfull_offset((int)world, (long)max_rows, (long)max_cols);
  });
  m.def("gemm_rs", &gemm_rs);
  m.def("ag_gemm", &ag_gemm);
  pybind11::class_<Comm>(m, "Comm");
  m.def("make_comm", &make_comm);
  m.def("decode_layers", &decode_layers);
  m.def("decode_layers_max", &decode_layers_max);
  m.def("decode_layers_prepare", &decode_layers_prepare);
  m.def("decode_layer_trace_set", &decode_layer_trace_set);
  m.def("comm_workspace_bytes", [](int64_t max_ctas, int64_t slot_floats) {
    return (int64_t)fb_comm_workspace_bytes((int)max_ctas, (long)slot_floats);
  });
  m.def("gemv_allreduce", &gemv_allreduce);
  m.def("allreduce_oneshot", &allreduce_oneshot);
  m.def("argmax_gather", &argmax_gather);
  m.def("comm_wait_probe", &comm_wait_probe);
  m.def("p2p_pattern", [](const Comm& c, int64_t word_off, int64_t n_words, int64_t seed) {
    check(fb_p2p_pattern(c.peers.data(), c.rank, c.world, c.max_ctas, c.slot_floats, (long)word_off, (int)n_words,
                         (uint32_t)seed, cur_stream()), "p2p_pattern");
  });
  m.def("comm_trace_set", [](c10::optional<Tensor> buf) {
    if (buf.has_value() && buf->defined()) {
      TORCH_CHECK(buf->scalar_type() == torch::kInt64 && buf->is_cuda() && buf->is_contiguous() &&
                  buf->numel() >= (int64_t)fb_comm_trace_recs() * fb_comm_trace_words(), "comm_trace_set: int64 cuda buffer too small");
      fb_comm_trace_set(reinterpret_cast<unsigned long long*>(buf->data_ptr()));
    } else {
      fb_comm_trace_set(nullptr);
    }
  });
  m.def("comm_trace_shape", []() { return std::make_pair((int64_t)fb_comm_trace_recs(), (int64_t)fb_comm_trace_words()); });
  m.def("comm_serial_polls_set", [](bool on) { fb_comm_serial_polls_set(on ? 1 : 0); });
  m.def("gemv_nvfp4", &gemv_nvfp4);
  m.def("moe_route", &moe_route);
  m.def("moe_experts", &moe_experts);
  m.def("moe_experts_fp4", &moe_experts_fp4);
  m.def("nvfp4_dequant", &nvfp4_dequant);
  m.def("nvfp4_sf_bytes", &nvfp4_sf_bytes);
  m.def("quant_nvfp4", &quant_nvfp4);
  m.def("gemm_nvfp4_workspace_bytes", &gemm_nvfp4_workspace_bytes);
  m.def("gemm_nvfp4", &gemm_nvfp4);
  m.def("gemm_nvfp4_fused", &gemm_nvfp4_fused);
  m.def("gemm_nvfp4_swiglu_q", &gemm_nvfp4_swiglu_q);
  m.def("gemv_nvfp4_tc", &gemv_nvfp4_tc);
  m.def("gemv_nvfp4_tc_trace_set", &gemv_nvfp4_tc_trace_set);
  m.def("gemv_nvfp4_tc_workspace_bytes", &gemv_nvfp4_tc_workspace_bytes);
  m.def("gemv_nvfp4_tc_terms", &gemv_nvfp4_tc_terms);
  m.def("gemv_nvfp4_allreduce", &gemv_nvfp4_allreduce);
}
