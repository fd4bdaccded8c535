// Python bindings: thin glue from torch tensors to the C launch API in api.h. No kernel lives here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "api.h"
#include "api_ext.h"

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

inline void check(int rc, const char* what) {
  if (rc == 0) return;
  if (rc > 0) {
    TORCH_CHECK(false, what, ": CUDA error ", rc, " (", cudaGetErrorString((cudaError_t)rc), ")");
  }
  TORCH_CHECK(false, what, ": unsupported arguments (code ", rc, ")");
}

inline const void* cptr(const c10::optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }
inline void* mptr(const c10::optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

int sm_count() {
  static int n = 0;
  if (n == 0) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

void embed(Tensor out, Tensor table, Tensor ids) {
  check(fb_embed(out.data_ptr(), table.data_ptr(), ids.data_ptr<int>(), (int)ids.numel(), (int)table.size(1),
                 (int)table.size(0), cur_stream()), "embed");
}

void rmsnorm(Tensor out, Tensor x, Tensor w, double eps, bool centred, c10::optional<Tensor> res,
             c10::optional<Tensor> x_out) {
  int rows = (int)(x.numel() / x.size(-1));
  check(fb_rmsnorm(out.data_ptr(), mptr(x_out), x.data_ptr(), cptr(res), w.data_ptr(), rows, (int)x.size(-1),
                   (float)eps, centred ? 1 : 0, cur_stream()), "rmsnorm");
}

void silu_mul(Tensor out, Tensor gu, double clamp) {
  int rows = (int)gu.size(0);
  check(fb_silu_mul(out.data_ptr(), gu.data_ptr(), rows, (int)(gu.size(1) / 2), (float)clamp, cur_stream()), "silu_mul");
}

void gated_norm(Tensor out, Tensor y, Tensor z_base, int64_t z_off, int64_t z_stride, Tensor w, int64_t heads,
                int64_t dv, double eps) {
  int rows = (int)y.size(0);
  const char* zp = (const char*)z_base.data_ptr() + z_off * 2;
  check(fb_gated_norm(out.data_ptr(), y.data_ptr<float>(), zp, (long)z_stride, w.data_ptr(), rows, (int)heads, (int)dv,
                      (float)eps, cur_stream()), "gated_norm");
}

void gather_rows(Tensor out, Tensor in, Tensor idx) {
  check(fb_gather_rows(out.data_ptr(), in.data_ptr(), idx.data_ptr<int>(), (int)idx.numel(), (int)in.size(1),
                       cur_stream()), "gather_rows");
}

void add_bf16(Tensor x, Tensor y) { check(fb_add_bf16(x.data_ptr(), y.data_ptr(), (long)x.numel(), cur_stream()), "add_bf16"); }

// Y[M][N] (+)= X W^T, small M. mode 0 plain / 1 swiglu.
void gemv(Tensor Y, Tensor X, Tensor W, c10::optional<Tensor> norm_w, c10::optional<Tensor> res, double eps,
          bool centred, int64_t mode) {
  int M = (int)X.size(0), K = (int)X.size(1);
  int N = (int)(mode == 1 ? W.size(0) / 2 : W.size(0));
  check(fb_gemv_bf16(Y.data_ptr(), X.data_ptr(), W.data_ptr(), cptr(norm_w), cptr(res), M, N, K, (long)X.stride(0),
                     (long)Y.stride(0), (float)eps, centred ? 1 : 0, Y.scalar_type() == torch::kFloat32 ? 1 : 0,
                     (int)mode, sm_count(), cur_stream()), "gemv");
}

int64_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t split_k) {
  return fb_gemm_workspace_bytes((int)M, (int)N, (int)split_k);
}

void gemm(Tensor Y, Tensor X, Tensor W, c10::optional<Tensor> res, int64_t mode, int64_t split_k,
          c10::optional<Tensor> workspace, c10::optional<Tensor> counters, c10::optional<Tensor> status) {
  int M = (int)X.size(0), K = (int)X.size(1);
  int N = (int)((mode & 1) ? W.size(0) / 2 : W.size(0));
  check(fb_gemm_bf16(Y.data_ptr(), X.data_ptr(), W.data_ptr(), cptr(res), M, N, K, (long)X.stride(0),
                     (long)Y.stride(0), (int)mode, (int)split_k, (float*)mptr(workspace), (int*)mptr(counters),
                     (int*)mptr(status), sm_count(), cur_stream()), "gemm");
}

void gemv_mma(Tensor Y, Tensor X, Tensor W, c10::optional<Tensor> norm_w, c10::optional<Tensor> res, double eps,
              int64_t mode, c10::optional<Tensor> workspace, c10::optional<Tensor> counters) {
  int M = (int)X.size(0), K = (int)X.size(1);
  int N = (int)(mode == 1 ? W.size(0) / 2 : W.size(0));
  long wsf = workspace.has_value() ? (long)(workspace->numel() * workspace->element_size() / 4) : 0;
  int nc = counters.has_value() ? (int)counters->numel() : 0;
  check(fb_gemv_mma(Y.data_ptr(), X.data_ptr(), W.data_ptr(), cptr(norm_w), cptr(res), M, N, K, (long)X.stride(0),
                    (long)Y.stride(0), (float)eps, (int)mode, Y.scalar_type() == torch::kFloat32 ? 1 : 0,
                    (float*)mptr(workspace), wsf, (int*)mptr(counters), nc, sm_count(), cur_stream()), "gemv_mma");
}

void quant_fp8(Tensor q, Tensor scale, Tensor x, c10::optional<Tensor> norm_w, double eps) {
  check(fb_quant_fp8(q.data_ptr(), scale.data_ptr<float>(), x.data_ptr(), cptr(norm_w), (int)x.size(0), (int)x.size(1),
                     (long)x.stride(0), (float)eps, cur_stream()), "quant_fp8");
}

void quant_fp8_block(Tensor q, Tensor scale, Tensor x) {
  check(fb_quant_fp8_block(q.data_ptr(), scale.data_ptr<float>(), x.data_ptr(), (int)x.size(0), (int)x.size(1),
                           (long)x.stride(0), cur_stream()), "quant_fp8_block");
}

void gemm_fp8_block(Tensor Y, Tensor Xq, Tensor sx, Tensor Wq, Tensor sw, c10::optional<Tensor> res, int64_t K,
                    c10::optional<Tensor> status) {
  const int M = (int)Xq.size(0), N = (int)Wq.size(0);
  const long kb = fb_fp8_block_kblocks((int)K);
  TORCH_CHECK(Xq.size(1) == kb * 128 && Wq.size(1) == kb * 128 && Xq.is_contiguous() && Wq.is_contiguous(),
              "gemm_fp8_block: code matrices are [rows][kblocks * 128], contiguous");
  TORCH_CHECK(sx.numel() == (int64_t)M * kb && sw.numel() == (int64_t)((N + 127) / 128) * kb, "gemm_fp8_block: scale shapes");
  check(fb_gemm_fp8_block(Y.data_ptr(), Xq.data_ptr(), sx.data_ptr<float>(), Wq.data_ptr(), sw.data_ptr<float>(), cptr(res),
                          M, N, (int)K, (long)Y.stride(0), (int*)mptr(status), cur_stream()), "gemm_fp8_block");
}

void gemm_fp8(Tensor Y, Tensor Xq, Tensor Wq, c10::optional<Tensor> scale_m, c10::optional<Tensor> scale_n,
              c10::optional<Tensor> res, int64_t mode, int64_t split_k, c10::optional<Tensor> workspace,
              c10::optional<Tensor> counters, c10::optional<Tensor> status) {
  int M = (int)Xq.size(0), K = (int)Xq.size(1);
  int N = (int)(mode == 1 ? Wq.size(0) / 2 : Wq.size(0));
  check(fb_gemm_fp8(Y.data_ptr(), Xq.data_ptr(), Wq.data_ptr(), (const float*)cptr(scale_m), (const float*)cptr(scale_n),
                    cptr(res), M, N, K, (long)Y.stride(0), (int)mode, (int)split_k, (float*)mptr(workspace),
                    (int*)mptr(counters), (int*)mptr(status), sm_count(), cur_stream()), "gemm_fp8");
}

void attn_prep(Tensor q_out, Tensor k_cache, Tensor v_cache, Tensor proj, Tensor q_norm, Tensor k_norm,
               Tensor inv_freq, Tensor row_slot, Tensor row_pos, Tensor block_table, int64_t kv_block, int64_t nq,
               int64_t nkv, int64_t hd, int64_t rot, bool gated, double eps, c10::optional<Tensor> status,
               c10::optional<Tensor> kv_scale, c10::optional<Tensor> row_cpos, int64_t hrot) {
  const bool scaled = kv_scale.has_value() && kv_scale->defined();
  const bool bytes = k_cache.scalar_type() == torch::kByte;
  // a byte cache with hd * 3 / 4 bytes per head row is the 6-bit form; any form can keep its keys Hadamard-rotated
  const bool six = scaled && bytes && k_cache.size(3) * 4 == hd * 3;
  if (six || hrot) {
    const int bits = six ? 6 : (scaled && bytes && k_cache.size(3) * 2 == hd) ? 4 : scaled ? 8 : 16;
    check(fb_attn_prep_qn(q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                          scaled ? kv_scale->data_ptr<float>() : nullptr, proj.data_ptr(), (long)proj.stride(0),
                          q_norm.data_ptr(), k_norm.data_ptr(), inv_freq.data_ptr<float>(), row_slot.data_ptr<int>(),
                          row_pos.data_ptr<int>(), (const int*)cptr(row_cpos), block_table.data_ptr<int>(),
                          (int)block_table.size(1), (int)kv_block, (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd,
                          (int)rot, gated ? 1 : 0, (float)eps, (int*)mptr(status), bits, (int)hrot, cur_stream()),
          "attn_prep_qn");
    return;
  }
  // a byte cache with hd/2 bytes per head row is the 4-bit form
  if (kv_scale.has_value() && kv_scale->defined() && k_cache.scalar_type() == torch::kByte && k_cache.size(3) * 2 == hd) {
    check(fb_attn_prep_q4(q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), kv_scale->data_ptr<float>(),
                          proj.data_ptr(), (long)proj.stride(0), q_norm.data_ptr(), k_norm.data_ptr(),
                          inv_freq.data_ptr<float>(), row_slot.data_ptr<int>(), row_pos.data_ptr<int>(),
                          (const int*)cptr(row_cpos), block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                          (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd, (int)rot, gated ? 1 : 0, (float)eps,
                          (int*)mptr(status), cur_stream()), "attn_prep_q4");
    return;
  }
  if (row_cpos.has_value() && row_cpos->defined()) {
    const bool k8 = kv_scale.has_value() && kv_scale->defined();
    check(fb_attn_prep_tree(q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                            k8 ? kv_scale->data_ptr<float>() : nullptr, proj.data_ptr(), (long)proj.stride(0),
                            q_norm.data_ptr(), k_norm.data_ptr(), inv_freq.data_ptr<float>(), row_slot.data_ptr<int>(),
                            row_pos.data_ptr<int>(), row_cpos->data_ptr<int>(), block_table.data_ptr<int>(),
                            (int)block_table.size(1), (int)kv_block, (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd,
                            (int)rot, gated ? 1 : 0, (float)eps, (int*)mptr(status), cur_stream()), "attn_prep_tree");
    return;
  }
  if (kv_scale.has_value() && kv_scale->defined()) {
    check(fb_attn_prep_kv8(q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), kv_scale->data_ptr<float>(),
                           proj.data_ptr(), (long)proj.stride(0), q_norm.data_ptr(), k_norm.data_ptr(),
                           inv_freq.data_ptr<float>(), row_slot.data_ptr<int>(), row_pos.data_ptr<int>(),
                           block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block, (int)row_slot.numel(),
                           (int)nq, (int)nkv, (int)hd, (int)rot, gated ? 1 : 0, (float)eps, (int*)mptr(status),
                           cur_stream()), "attn_prep_kv8");
    return;
  }
  check(fb_attn_prep(q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), proj.data_ptr(), (long)proj.stride(0),
                     q_norm.data_ptr(), k_norm.data_ptr(), inv_freq.data_ptr<float>(), row_slot.data_ptr<int>(),
                     row_pos.data_ptr<int>(), block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                     (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd, (int)rot, gated ? 1 : 0, (float)eps,
                     (int*)mptr(status), cur_stream()), "attn_prep");
}

void attn_decode(Tensor out, Tensor o_part, Tensor ml_part, Tensor q, Tensor k_cache, Tensor v_cache, Tensor proj,
                 Tensor row_slot, Tensor row_kvlen, c10::optional<Tensor> row_base, c10::optional<Tensor> row_mask,
                 Tensor block_table, int64_t kv_block, int64_t nq, int64_t nkv, int64_t hd, int64_t nsplit,
                 bool gated, c10::optional<Tensor> kv_scale) {
  if (kv_scale.has_value() && kv_scale->defined() && k_cache.scalar_type() == torch::kByte && k_cache.size(3) * 4 == hd * 3) {
    check(fb_attn_decode_qn(out.data_ptr(), o_part.data_ptr<float>(), ml_part.data_ptr<float>(), q.data_ptr(),
                            k_cache.data_ptr(), v_cache.data_ptr(), kv_scale->data_ptr<float>(), proj.data_ptr(),
                            (long)proj.stride(0), row_slot.data_ptr<int>(), row_kvlen.data_ptr<int>(),
                            (const int*)cptr(row_base), (const unsigned long long*)cptr(row_mask),
                            block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                            (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd, (int)nsplit, gated ? 1 : 0, 6, cur_stream()),
          "attn_decode_q6");
    return;
  }
  if (kv_scale.has_value() && kv_scale->defined() && k_cache.scalar_type() == torch::kByte && k_cache.size(3) * 2 == hd) {
    check(fb_attn_decode_q4(out.data_ptr(), o_part.data_ptr<float>(), ml_part.data_ptr<float>(), q.data_ptr(),
                            k_cache.data_ptr(), v_cache.data_ptr(), kv_scale->data_ptr<float>(), proj.data_ptr(),
                            (long)proj.stride(0), row_slot.data_ptr<int>(), row_kvlen.data_ptr<int>(),
                            (const int*)cptr(row_base), (const unsigned long long*)cptr(row_mask),
                            block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                            (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd, (int)nsplit, gated ? 1 : 0, cur_stream()),
          "attn_decode_q4");
    return;
  }
  if (kv_scale.has_value() && kv_scale->defined()) {
    check(fb_attn_decode_kv8(out.data_ptr(), o_part.data_ptr<float>(), ml_part.data_ptr<float>(), q.data_ptr(),
                             k_cache.data_ptr(), v_cache.data_ptr(), kv_scale->data_ptr<float>(), proj.data_ptr(),
                             (long)proj.stride(0), row_slot.data_ptr<int>(), row_kvlen.data_ptr<int>(),
                             (const int*)cptr(row_base), (const unsigned long long*)cptr(row_mask),
                             block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                             (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd, (int)nsplit, gated ? 1 : 0, cur_stream()),
          "attn_decode_kv8");
    return;
  }
  check(fb_attn_decode(out.data_ptr(), o_part.data_ptr<float>(), ml_part.data_ptr<float>(), q.data_ptr(),
                       k_cache.data_ptr(), v_cache.data_ptr(), proj.data_ptr(), (long)proj.stride(0),
                       row_slot.data_ptr<int>(), row_kvlen.data_ptr<int>(), (const int*)cptr(row_base),
                       (const unsigned long long*)cptr(row_mask), block_table.data_ptr<int>(),
                       (int)block_table.size(1), (int)kv_block, (int)row_slot.numel(), (int)nq, (int)nkv, (int)hd,
                       (int)nsplit, gated ? 1 : 0, cur_stream()), "attn_decode");
}

int64_t attn_decode_mma(Tensor out, Tensor o_part, Tensor ml_part, Tensor q, Tensor k_cache, Tensor v_cache, Tensor proj,
                        Tensor seg_slot, Tensor seg_row0, Tensor seg_nrows, int64_t max_rows, Tensor row_kvlen,
                        c10::optional<Tensor> row_base, c10::optional<Tensor> row_mask, Tensor block_table,
                        int64_t kv_block, int64_t nq, int64_t nkv, int64_t hd, int64_t nsplit, bool gated,
                        c10::optional<Tensor> kv_scale) {
  int rc = fb_attn_decode_mma(out.data_ptr(), o_part.data_ptr<float>(), ml_part.data_ptr<float>(), q.data_ptr(),
                              k_cache.data_ptr(), v_cache.data_ptr(), (const float*)cptr(kv_scale), proj.data_ptr(),
                              (long)proj.stride(0),
                              seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(), seg_nrows.data_ptr<int>(),
                              row_kvlen.data_ptr<int>(), (const int*)cptr(row_base),
                              (const unsigned long long*)cptr(row_mask), block_table.data_ptr<int>(),
                              (int)block_table.size(1), (int)kv_block, (int)seg_slot.numel(), (int)max_rows,
                              (int)row_kvlen.numel(), (int)nq, (int)nkv, (int)hd, (int)nsplit, gated ? 1 : 0, cur_stream());
  if (rc == -20) return rc;
  check(rc, "attn_decode_mma");
  return 0;
}

void kv_dequant(Tensor k_out, Tensor v_out, Tensor k_cache8, Tensor v_cache8, Tensor kv_scale, Tensor seg_slot,
                Tensor seg_pos0, Tensor seg_nrows, Tensor block_table, int64_t kv_block, int64_t max_kvlen, int64_t nkv,
                int64_t hd, int64_t scratch_tokens_per_slot) {
  if (k_cache8.size(3) * 4 == hd * 3) {
    check(fb_kv_dequant_qn(k_out.data_ptr(), v_out.data_ptr(), k_cache8.data_ptr(), v_cache8.data_ptr(),
                           kv_scale.data_ptr<float>(), seg_slot.data_ptr<int>(), seg_pos0.data_ptr<int>(),
                           seg_nrows.data_ptr<int>(), block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                           (int)seg_slot.numel(), (int)max_kvlen, (int)nkv, (int)hd, (int)scratch_tokens_per_slot, 6,
                           cur_stream()), "kv_dequant_q6");
    return;
  }
  if (k_cache8.size(3) * 2 == hd) {
    check(fb_kv_dequant_q4(k_out.data_ptr(), v_out.data_ptr(), k_cache8.data_ptr(), v_cache8.data_ptr(),
                           kv_scale.data_ptr<float>(), seg_slot.data_ptr<int>(), seg_pos0.data_ptr<int>(),
                           seg_nrows.data_ptr<int>(), block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                           (int)seg_slot.numel(), (int)max_kvlen, (int)nkv, (int)hd, (int)scratch_tokens_per_slot,
                           cur_stream()), "kv_dequant_q4");
    return;
  }
  check(fb_kv_dequant(k_out.data_ptr(), v_out.data_ptr(), k_cache8.data_ptr(), v_cache8.data_ptr(),
                      kv_scale.data_ptr<float>(), seg_slot.data_ptr<int>(), seg_pos0.data_ptr<int>(),
                      seg_nrows.data_ptr<int>(), block_table.data_ptr<int>(), (int)block_table.size(1), (int)kv_block,
                      (int)seg_slot.numel(), (int)max_kvlen, (int)nkv, (int)hd, (int)scratch_tokens_per_slot, cur_stream()),
        "kv_dequant");
}

void attn_prefill(Tensor out, Tensor q, Tensor k_cache, Tensor v_cache, Tensor proj, Tensor seg_slot, Tensor seg_row0,
                  Tensor seg_nrows, Tensor seg_pos0, Tensor block_table, int64_t kv_block, int64_t max_rows,
                  int64_t nq, int64_t nkv, int64_t hd, bool gated) {
  check(fb_attn_prefill(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), proj.data_ptr(),
                        (long)proj.stride(0), seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(),
                        seg_nrows.data_ptr<int>(), seg_pos0.data_ptr<int>(), block_table.data_ptr<int>(),
                        (int)block_table.size(1), (int)kv_block, (int)seg_slot.numel(), (int)max_rows, (int)nq,
                        (int)nkv, (int)hd, gated ? 1 : 0, cur_stream()), "attn_prefill");
}

int64_t attn_prefill_tc(Tensor out, Tensor q, Tensor k_cache, Tensor v_cache, Tensor proj, Tensor seg_slot, Tensor seg_row0,
                        Tensor seg_nrows, Tensor seg_pos0, Tensor block_table, int64_t kv_block, int64_t max_rows,
                        int64_t nq, int64_t nkv, int64_t hd, bool gated, c10::optional<Tensor> status) {
  TORCH_CHECK(q.is_contiguous() && k_cache.is_contiguous() && v_cache.is_contiguous(), "attn_prefill_tc: contiguous inputs");
  int rc = fb_attn_prefill_tc(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), proj.data_ptr(),
                              (long)proj.stride(0), seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(),
                              seg_nrows.data_ptr<int>(), seg_pos0.data_ptr<int>(), block_table.data_ptr<int>(),
                              (int)block_table.size(1), (int)kv_block, (int)seg_slot.numel(), (int)max_rows,
                              (long)q.size(0), (long)(k_cache.size(0) * k_cache.size(1)), (int)nq, (int)nkv, (int)hd,
                              gated ? 1 : 0, (int*)mptr(status), cur_stream());
  if (rc == -20) return rc;                     // shape outside this kernel: the caller takes the mma.sync kernel
  check(rc, "attn_prefill_tc");
  return 0;
}

void gdn_conv(Tensor out, Tensor proj, Tensor conv_w, Tensor conv_state, Tensor seg_slot, Tensor seg_row0,
              Tensor seg_nrows, int64_t max_rows) {
  check(fb_gdn_conv(out.data_ptr(), proj.data_ptr(), (long)proj.stride(0), conv_w.data_ptr(), conv_state.data_ptr(),
                    seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(), seg_nrows.data_ptr<int>(),
                    (int)seg_slot.numel(), (int)max_rows, (int)out.size(1), cur_stream()), "gdn_conv");
}

void gdn_rec(Tensor y, Tensor rec_state, Tensor conv_state, Tensor qkv, Tensor proj, Tensor A_log, Tensor dt_bias,
             Tensor seg_slot, Tensor seg_row0, Tensor seg_nrows, int64_t nk, int64_t nv, int64_t dk, int64_t dv,
             double eps, bool commit) {
  check(fb_gdn_rec(y.data_ptr<float>(), rec_state.data_ptr<float>(), conv_state.data_ptr(), qkv.data_ptr(),
                   proj.data_ptr(), (long)proj.stride(0), A_log.data_ptr<float>(), dt_bias.data_ptr<float>(),
                   seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(), seg_nrows.data_ptr<int>(),
                   (int)seg_slot.numel(), (int)nk, (int)nv, (int)dk, (int)dv, (float)eps, commit ? 1 : 0, cur_stream()),
        "gdn_rec");
}

void gdn_conv_tree(Tensor out, Tensor proj, Tensor conv_w, Tensor conv_state, Tensor seg_slot, Tensor seg_row0,
                   Tensor seg_nrows, Tensor row_parent) {
  check(fb_gdn_conv_tree(out.data_ptr(), proj.data_ptr(), (long)proj.stride(0), conv_w.data_ptr(), conv_state.data_ptr(),
                         seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(), seg_nrows.data_ptr<int>(),
                         row_parent.data_ptr<int>(), (int)seg_slot.numel(), (int)out.size(1), cur_stream()),
        "gdn_conv_tree");
}

void gdn_rec_tree(Tensor y, Tensor rec_state, Tensor qkv, Tensor proj, Tensor A_log, Tensor dt_bias, Tensor seg_slot,
                  Tensor seg_row0, Tensor seg_nrows, Tensor row_parent, Tensor row_flags, Tensor node_state, int64_t nk,
                  int64_t nv, int64_t dk, int64_t dv, double eps) {
  TORCH_CHECK(node_state.numel() * (int64_t)node_state.element_size() >=
                  fb_gdn_tree_scratch_bytes((int)qkv.size(0), (int)nv, (int)dk, (int)dv), "gdn_rec_tree: scratch too small");
  check(fb_gdn_rec_tree(y.data_ptr<float>(), rec_state.data_ptr<float>(), qkv.data_ptr(), proj.data_ptr(),
                        (long)proj.stride(0), A_log.data_ptr<float>(), dt_bias.data_ptr<float>(), seg_slot.data_ptr<int>(),
                        seg_row0.data_ptr<int>(), seg_nrows.data_ptr<int>(), row_parent.data_ptr<int>(),
                        row_flags.data_ptr<int>(), (float*)node_state.data_ptr(), (int)seg_slot.numel(), (int)nk, (int)nv,
                        (int)dk, (int)dv, (float)eps, cur_stream()), "gdn_rec_tree");
}

void gdn_step(Tensor out, Tensor rec_state, Tensor conv_state, Tensor proj, Tensor conv_w, Tensor A_log, Tensor dt_bias,
              Tensor gnorm_w, Tensor seg_slot, Tensor seg_row0, Tensor seg_nrows, int64_t nk, int64_t nv, int64_t dk,
              int64_t dv, double eps, bool commit) {
  check(fb_gdn_step(out.data_ptr(), rec_state.data_ptr<float>(), conv_state.data_ptr(), proj.data_ptr(),
                    (long)proj.stride(0), conv_w.data_ptr(), A_log.data_ptr<float>(), dt_bias.data_ptr<float>(),
                    gnorm_w.data_ptr(), seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(), seg_nrows.data_ptr<int>(),
                    (int)seg_slot.numel(), (int)nk, (int)nv, (int)dk, (int)dv, (float)eps, commit ? 1 : 0, cur_stream()),
        "gdn_step");
}

int64_t gdn_chunk_scratch_bytes(int64_t rows, int64_t nseg, int64_t nv, int64_t dk) {
  return fb_gdn_chunk_scratch_bytes((int)rows, (int)nseg, (int)nv, (int)dk);
}

void gdn_chunk(Tensor y, Tensor rec_state, Tensor conv_state, Tensor scratch, Tensor qkv, Tensor proj, Tensor A_log,
               Tensor dt_bias, Tensor seg_slot, Tensor seg_row0, Tensor seg_nrows, int64_t max_rows, int64_t nk,
               int64_t nv, int64_t dk, int64_t dv, double eps, bool commit) {
  TORCH_CHECK((int64_t)(scratch.numel() * scratch.element_size()) >=
                  gdn_chunk_scratch_bytes(qkv.size(0), seg_slot.numel(), nv, dk), "gdn_chunk: scratch too small");
  check(fb_gdn_chunk(y.data_ptr<float>(), rec_state.data_ptr<float>(), conv_state.data_ptr(), (float*)scratch.data_ptr(),
                     qkv.data_ptr(), proj.data_ptr(), (long)proj.stride(0), A_log.data_ptr<float>(),
                     dt_bias.data_ptr<float>(), seg_slot.data_ptr<int>(), seg_row0.data_ptr<int>(),
                     seg_nrows.data_ptr<int>(), (int)seg_slot.numel(), (int)max_rows, (int)nk, (int)nv, (int)dk, (int)dv,
                     (float)eps, commit ? 1 : 0, cur_stream()), "gdn_chunk");
}

void argmax(Tensor ids, Tensor logits, c10::optional<Tensor> vals, c10::optional<Tensor> finite,
            c10::optional<Tensor> scratch) {
  if (scratch.has_value() && scratch->defined() && logits.size(1) >= 8192) {
    TORCH_CHECK(scratch->numel() * scratch->element_size() >= logits.size(0) * 64 * 12, "argmax scratch too small");
    check(fb_argmax2(ids.data_ptr<int>(), (float*)mptr(vals), (int*)mptr(finite), logits.data_ptr(),
                     (long)logits.stride(0), (int)logits.size(0), (int)logits.size(1),
                     logits.scalar_type() == torch::kFloat32 ? 1 : 0, scratch->data_ptr(), cur_stream()), "argmax2");
    return;
  }
  check(fb_argmax(ids.data_ptr<int>(), (float*)mptr(vals), (int*)mptr(finite), logits.data_ptr(),
                  (long)logits.stride(0), (int)logits.size(0), (int)logits.size(1),
                  logits.scalar_type() == torch::kFloat32 ? 1 : 0, cur_stream()), "argmax");
}

void sample(Tensor ids, Tensor logits, Tensor params, c10::optional<Tensor> counts, Tensor work) {
  check(fb_sample(ids.data_ptr<int>(), logits.data_ptr(), (long)logits.stride(0), (int)logits.size(0),
                  (int)logits.size(1), params.data_ptr(), (const int*)cptr(counts), work.data_ptr<float>(),
                  logits.scalar_type() == torch::kFloat32 ? 1 : 0, cur_stream()), "sample");
}

void chain_accept(Tensor n_accept, Tensor out_tokens, Tensor target, Tensor draft, Tensor seg_row0, Tensor seg_ndraft,
                  int64_t max_draft) {
  check(fb_chain_accept(n_accept.data_ptr<int>(), out_tokens.data_ptr<int>(), target.data_ptr<int>(),
                        draft.data_ptr<int>(), seg_row0.data_ptr<int>(), seg_ndraft.data_ptr<int>(),
                        (int)seg_row0.numel(), (int)max_draft, cur_stream()), "chain_accept");
}

void kv_move_rows(Tensor k, c10::optional<Tensor> v, c10::optional<Tensor> sc, Tensor src, Tensor dst, Tensor seg_off) {
  // caches [pages, kv_block, ...] contiguous: a row is everything behind the first two dimensions
  auto row_bytes = [](const Tensor& t) { return (long)(t.numel() / (t.size(0) * t.size(1))) * (long)t.element_size(); };
  const bool hv = v.has_value() && v->defined() && v->numel() > 0, hs = sc.has_value() && sc->defined() && sc->numel() > 0;
  check(fb_kv_move_rows(k.data_ptr(), row_bytes(k), hv ? v->data_ptr() : nullptr, hv ? row_bytes(*v) : 0,
                        hs ? sc->data_ptr() : nullptr, hs ? row_bytes(*sc) : 0, src.data_ptr<int>(), dst.data_ptr<int>(),
                        seg_off.data_ptr<int>(), (int)seg_off.numel() - 1, cur_stream()), "kv_move_rows");
}

}  // namespace

void register_ext(pybind11::module_& m);
void register_host(pybind11::module_& m);
void register_oracle(pybind11::module_& m);
void register_gguf_host(pybind11::module_& m);
void register_sampler_host(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("embed", &embed);
  m.def("rmsnorm", &rmsnorm);
  m.def("silu_mul", &silu_mul);
  m.def("gated_norm", &gated_norm);
  m.def("gather_rows", &gather_rows);
  m.def("add_bf16", &add_bf16);
  m.def("gemv", &gemv);
  m.def("gemm", &gemm);
  m.def("gemm_workspace_bytes", &gemm_workspace_bytes);
  m.def("attn_prep", &attn_prep);
  m.def("attn_decode", &attn_decode);
  m.def("attn_prefill", &attn_prefill);
  m.def("attn_prefill_tc", &attn_prefill_tc);
  m.def("attn_decode_mma", &attn_decode_mma);
  m.def("gdn_conv", &gdn_conv);
  m.def("gdn_rec", &gdn_rec);
  m.def("gdn_conv_tree", &gdn_conv_tree);
  m.def("gdn_rec_tree", &gdn_rec_tree);
  m.def("kv_dequant", &kv_dequant);
  m.def("gemv_mma", &gemv_mma);
  m.def("gdn_step", &gdn_step);
  m.def("quant_fp8", &quant_fp8);
  m.def("gemm_fp8", &gemm_fp8);
  m.def("quant_fp8_block", &quant_fp8_block);
  m.def("gemm_fp8_block", &gemm_fp8_block);
  m.def("gdn_chunk", &gdn_chunk);
  m.def("gdn_chunk_scratch_bytes", &gdn_chunk_scratch_bytes);
  m.def("argmax", &argmax);
  m.def("sample", &sample);
  m.def("chain_accept", &chain_accept);
  m.def("kv_move_rows", &kv_move_rows);
  register_ext(m);
  register_host(m);
  register_oracle(m);
  register_gguf_host(m);
  register_sampler_host(m);
}
