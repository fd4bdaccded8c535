// C launch API, second part: fused compute+collective kernels, quantised formats, MoE, MLA, drafter ops.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- comm.cu: kernels over NVLink peer memory. `peers` = base pointer of the symmetric workspace on every rank
// (host array, peers[rank] is the local mapping); epochs = local device array of two words: the epoch of the last
// finished call and the count of CTAs of the running call that have finished. ----
long fb_comm_workspace_bytes(int max_ctas, long slot_floats);
// Profiling: a device buffer of fb_comm_trace_recs() x fb_comm_trace_words() u64 that CTA 0 of every fused GEMV +
// all-reduce fills with device timestamps (null switches it off; set it before capturing a CUDA graph), and the
// switch that makes the exchange poll its sources one after the other (the earlier protocol, kept for comparison).
void fb_comm_trace_set(unsigned long long* buf);
int fb_comm_trace_recs();
int fb_comm_trace_words();
void fb_comm_serial_polls_set(int on);
int fb_gemv_allreduce(void* Y, const void* X, const void* W, const void* res, int M, int N, int K, long ldx, long ldy,
                      const void* const* peers, int rank, int world, int max_ctas, long slot_floats, uint32_t* epochs,
                      int* status, unsigned spin_limit, int max_resident, cudaStream_t s);
int fb_allreduce_oneshot(void* y, const void* part, const void* res, long count, int part_f32,
                         const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                         uint32_t* epochs, int* status, unsigned spin_limit, int max_resident, cudaStream_t s);
int fb_argmax_gather(int* ids, float* vals, const float* logits, long stride, int rows, int n_local, int vocab_offset,
                     const void* const* peers, int rank, int world, int max_ctas, long slot_floats, uint32_t* epochs,
                     int* status, unsigned spin_limit, cudaStream_t s);
// start-up self-test: this rank's pattern into its lane (parity 0, source = rank) of every rank's workspace
int fb_p2p_pattern(const void* const* peers, int rank, int world, int max_ctas, long slot_floats, long word_off,
                   int n_words, uint32_t seed, cudaStream_t s);
int fb_comm_wait_probe(const uint32_t* flag, uint32_t want, unsigned limit, int* status, cudaStream_t s);

// ---- gemv_nvfp4.cu: NVFP4-weight GEMV (W4A16), plain and with the fused one-shot all-reduce ----
int fb_gemv_nvfp4(void* Y, const void* X, const void* Wq, const void* Sc, float global_scale, const void* norm_w,
                  const void* res, int M, int N, int K, long ldx, long ldy, long sc_stride, float eps, int out_f32,
                  int mode, int sm_count, const float* row_alpha, cudaStream_t s);
int fb_gemv_nvfp4_allreduce(void* Y, const void* X, const void* Wq, const void* Sc, float global_scale,
                            const void* res, int M, int N, int K, long ldx, long ldy, long sc_stride,
                            const void* const* peers, int rank, int world, int max_ctas, long slot_floats,
                            uint32_t* epochs, int* status, unsigned spin_limit, int max_resident,
                            const float* row_alpha, cudaStream_t s);

// ---- gemm_nvfp4.cu: activation quantiser and block-scaled tcgen05 GEMM (W4A4) ----
long fb_nvfp4_sf_bytes(int rows, int K);
int fb_quant_nvfp4(void* codes, void* sf, float* row_scale, const void* x, long ldx, const void* norm_w, int M, int K,
                   float eps, cudaStream_t s);
long fb_gemm_nvfp4_workspace_bytes(int M, int N, int split_k);
int fb_gemm_nvfp4(void* Y, const void* Xq, const void* x_sf, const float* row_scale, const void* Wq, const void* w_sf,
                  float w_scale, const void* res, int M, int N, int K, long ldy, int mode, int split_k,
                  float* workspace, int* counters, int* status, int sm_count, cudaStream_t s);

int fb_gemm_nvfp4_fused(void* Y, const void* X, long ldx, const void* norm_w, float eps, const void* Wq,
                        const void* w_sf, float w_scale, const void* res, int M, int N, int K, long ldy, int mode,
                        int split_k, int out_f32, float* workspace, int* counters, int* status, int sm_count,
                        cudaStream_t s);

// gate|up GEMM + SwiGLU with the activation written as NVFP4 (codes, tiled scales, row scales) for the next GEMM
int fb_gemm_nvfp4_swiglu_q(void* q_codes, void* q_sf, float* q_row_scale, float q_gs, const void* Xq, const void* x_sf,
                           const float* row_scale, const void* Wq, const void* w_sf, float w_scale, int M, int N, int K,
                           int* status, int sm_count, cudaStream_t s);

// ---- gemv_nvfp4_tc.cu: few-row NVFP4 linear on the block-scaled tensor cores, activations as residual NVFP4 terms ----
long fb_gemv_nvfp4_tc_workspace_bytes(int M, int N, int K, int dual, int terms, int sm_count, int ctas_per_sm);
int fb_gemv_nvfp4_tc_terms(int M, int N, int K, int dual, int terms);
void fb_gemv_nvfp4_tc_trace_set(void* buf);
int fb_gemv_nvfp4_tc(void* Y, const void* X, long ldx, const void* norm_w, float eps, const void* Wq, const void* w_sf,
                     float w_scale, const float* row_alpha, const void* res, int M, int N, int K, long ldy, int mode,
                     int terms, int out_f32, float* workspace, int* counters, int* status, int sm_count,
                     int ctas_per_sm, const void* next_Wq, const void* next_sf, int next_N, int next_K, int next_mode,
                     long prefetch_bytes, cudaStream_t s);

// ---- decode_layer.cu: one decoder layer of a plain decode step as one persistent kernel ----
int fb_decode_layers_max();
int fb_decode_layers_prepare();
int fb_decode_layers(int n_layers, const int* start_phase, int M, int hidden, const void* x_in, void* const* x_out,
                     void* const* x_mid, void* const* act, void* const* proj, void* const* o, const void* const* w_in,
                     const int* n_in, const void* const* input_norm, const void* const* w_out, const int* k_out,
                     const void* const* post_norm, const void* const* w_gu, int inter, const void* const* w_down,
                     float* const* rec_state, void* const* conv_state, const void* const* conv_w,
                     const float* const* A_log, const float* const* dt_bias, const void* const* gnorm_w,
                     const int* seg_slot, int nk, int nv, int dk, float eps, const void* const* peers, int rank, int world,
                     int max_ctas, long slot_floats, uint32_t* epochs, int* status, unsigned spin_limit,
                     uint32_t* sync_words, int sm_count, cudaStream_t s);
void fb_decode_layer_trace_set(void* buf);

// ---- moe.cu: router, grouped-expert GEMVs over (token, expert) pairs, fixed-order combine ----
// `ld`: logit row stride (>= n_exp); shared_id >= 0 appends the shared expert as pick top_k (weight sigmoid(logit[shared_col])
// or 1 when shared_col < 0): ids / wts rows are top_k + 1 wide then
int fb_moe_route(int* ids, float* wts, const float* logits, const float* bias, int rows, int n_exp, int top_k, int mode,
                 int n_groups, int topk_groups, float scale, int ld, int shared_col, int shared_id, cudaStream_t s);
int fb_moe_gate_up(void* act, const void* x, const void* w_gu, const int* ids, int pairs, int top_k, int hidden,
                   int inter, int e_lo, int e_hi, cudaStream_t s);
int fb_moe_down(float* yp, const void* act, const void* w_down, const int* ids, int pairs, int hidden, int inter,
                int e_lo, int e_hi, cudaStream_t s);
// NVFP4 expert weights (moe_fp4.cu): codes [experts][rows][K/2], e4m3 block scales [experts][rows][K/16], one tensor scale
int fb_moe_gate_up_fp4(void* act, const void* x, const void* wq, const void* ws, float gscale, const int* ids, int pairs,
                       int top_k, int hidden, int inter, int e_lo, int e_hi, cudaStream_t s);
int fb_moe_down_fp4(float* yp, const void* act, const void* wq, const void* ws, float gscale, const int* ids, int pairs,
                    int hidden, int inter, int e_lo, int e_hi, cudaStream_t s);
int fb_nvfp4_dequant(void* out, const void* wq, const void* ws, float gscale, long elements, cudaStream_t s);
int fb_moe_combine(void* out, const float* yp, const float* wts, const void* shared, const float* shared_gate,
                   const void* res, int rows, int top_k, int hidden, int out_f32, cudaStream_t s);

// ---- gemm_comm.cu: tensor-parallel GEMMs with the collective inside the kernel ----
long fb_big_workspace_bytes(int world, long max_rows, long max_cols);
long fb_big_xfull_offset(int world, long max_rows, long max_cols);
int fb_gemm_rs(void* y_shard, const void* X, const void* W, const void* res_shard, int M, int N, int K, long ldx,
               const void* const* peers, int rank, int world, long max_rows, long max_cols, uint32_t* ctr, int* status,
               unsigned spin_limit, int sm_count, cudaStream_t s);
int fb_ag_gemm(void* Y, const void* W, const void* res, int M, int N, int K, long ldy, int mode,
               const void* const* peers, int rank, int world, long max_rows, long max_cols, uint32_t* ctr, int* status,
               unsigned spin_limit, int sm_count, cudaStream_t s);

int fb_gemm_grouped(void* Y, const void* X, const void* W, const int* tile_start, const int* row_base, int experts,
                    int max_rows, int N, int K, long ldx, long ldy, int mode, int* status, int sm_count, cudaStream_t s);

// Y[g] = X[g] W[g]^T for `groups` problems of one shape: X [groups * rows][K], W [groups][N][K], Y [groups * rows][N]
int fb_gemm_batched(void* Y, const void* X, const void* W, int groups, int rows, int N, int K, int* status, int sm_count,
                    cudaStream_t s);
// ---- head_linear.cu: one small linear per attention head over a few rows (strided x / y, W [heads][N][K]) ----
int fb_head_linear(void* y, const void* x, const void* W, int T, int heads, int N, int K, long x_rs, long x_hs, long y_rs,
                   long y_hs, cudaStream_t s);

// ---- moe_ep.cu: expert-parallel MoE block (dispatch / grouped GEMMs / combine over peer memory) ----
long fb_ep_workspace_bytes(int n_experts, int hidden, long cap_rows);
long fb_ep_recv_offset(int n_experts, int hidden, long cap_rows);
long fb_ep_out_offset(int n_experts, int hidden, long cap_rows);
int fb_ep_moe(void* out, const void* x, const int* ids, const float* wts, const void* w_gu, const void* w_down,
              const void* shared, const float* shared_gate, const void* res, void* act, int* plan, int rows, int top_k,
              int n_experts, int hidden, int inter, long cap_rows, const void* const* peers, int rank, int world,
              uint32_t* ctr, int* status, unsigned spin_limit, int sm_count, cudaStream_t s);

// ---- gguf_quant.cu: GGUF block formats ----
int fb_gguf_dequant(void* out_bf16, const void* raw, int type, long n_values, cudaStream_t s);
int fb_q8_1_quant(void* out, const void* x_bf16, long n_values, cudaStream_t s);
int fb_gguf_gemv(void* y, const void* x, const void* raw, const void* res, int type, int M, int N, int K, long ldx,
                 long ldy, cudaStream_t s);

// ---- exl3.cu: EXL3 trellis-quantised linears ----
int fb_exl3_had(void* out, const void* in, const void* pre_f16, const void* post_f16, const void* res, int rows, int width,
                float scale, int in_f32, int out_bf16, cudaStream_t s);
int fb_exl3_gemv(float* z, const float* xh, const void* trellis, int rows, int k, int n, int bits, cudaStream_t s);
int fb_exl3_decode(void* w_hat_t_bf16, const void* trellis, int k, int n, int bits, cudaStream_t s);

// ---- mla.cu: multi-head latent attention over a paged latent cache ----
int fb_mla_prep(void* cache, void* qabs, const void* kva, long kva_stride, const void* q, long q_stride, const void* norm_w,
                const float* inv_freq, const int* row_slot, const int* row_pos, const int* block_table, int max_blocks,
                int kv_block, int rows, int nq, int dn, int L, int R, float eps, int* status, cudaStream_t s);
int fb_mla_attn(void* out, float* o_part, float* ml_part, const void* qabs, const void* cache, const int* row_slot,
                const int* row_kvlen, const int* block_table, int max_blocks, int kv_block, int rows, int nq, int L, int R,
                int nsplit, float scale, cudaStream_t s);
// prompt rows of latent attention in the expanded form: per-head K / V rows (padded to the flash kernel's head width)
// from the kv_b GEMM output `kvx` [rows][nq][dn + dv] and the latent rows `lat` [rows][L + R]; padded, pre-scaled queries
int fb_mla_expand(void* kp, void* vp, const void* kvx, const void* lat, long rows, int nq, int dn, int dv, int L, int R, int HP,
                  cudaStream_t s);
int fb_mla_qpad(void* qp, const void* q, long q_stride, const void* qabs, long rows, int nq, int dn, int L, int R, int HP,
                float scale, cudaStream_t s);

// ---- drafter_ops.cu ----
int fb_w4_gemv(void* y, const void* x, const void* qweight, const void* scales, const void* biases, const void* res, int M,
               int N, int K, long ldx, long ldy, cudaStream_t s);
// hyper-connection streams (hyperconn.cu): per-stream RMSNorm to bf16, gated mix of the streams, output injection
int fb_hc_norm(void* y, float* rinv, const float* x, const float* w, int groups, int d, int ngw, float eps, cudaStream_t s);
int fb_hc_mix(float* mixed, const float* res, const float* rinv, const float* w, const float* gate, int rows, int d, int hc,
              cudaStream_t s);
int fb_hc_combine(float* res, const float* out, const float* inj, int rows, int d, int hc, long ldi, cudaStream_t s);
int fb_engram_gate(void* out, const void* h, const float* kvp, const void* kvb, const float* qk, int rows, int hc, int d,
                   int world, float eps, cudaStream_t s);

// ---- sparse_index.cu: compressor, indexer scores, exact top-k, candidate masks, selected-block tables ----
int fb_comp_step(void* out, float* tail, const float* kvc, const float* sc, const int* row_slot, const int* row_pos, int rows,
                 int ratio, int dim, int ring_len, cudaStream_t s);
int fb_index_score(float* score, int ld, const void* q, const float* w, float scale, const void* keys, long key_stride,
                   const int* row_slot, const int* row_len, const uint8_t* mask, int mask_ld, int mask_block, int rows, int nh,
                   int D, cudaStream_t s);
int fb_topk_select(int* sel, const float* score, int ld, int n, const int* row_n, int rows, int k, cudaStream_t s);
int fb_block_max(float* bmax, int mask_ld, const float* score, int ld, const int* row_n, int rows, int bsize, cudaStream_t s);
int fb_sel_to_mask(uint8_t* mask, int mask_ld, const int* sel, int rows, int k, cudaStream_t s);
int fb_qsa_pool(void* pooled, const float* raw, const float* w, const int* pos0, const float* inv_freq, int blocks, int kp,
                int D, int rot, float eps, cudaStream_t s);
int fb_qsa_table(int* table, int* kvlen, const int* sel, const int* row_slot, const int* row_pos, const int* block_table,
                 int max_blocks, int rows, int kp, int top, int* status, cudaStream_t s);

// ---- dspark.cu: Markov head loop, confidence head, reductions over residual streams ----
int fb_markov_bias(void* out, const void* head, const void* emb, const int* tok, const int* slot, int rows, int V, int rank,
                   cudaStream_t s);
int fb_markov_score(void* pair, const float* logits, long ld, const void* stage, const void* cache, const int* slot, int rows,
                    int parts, int n, int col0, cudaStream_t s);
int fb_markov_pick(int* draft, int* tok, int* slot, const void* pairs, const int* slot_of, int n_pairs, int rows, int stride,
                   int step, int vocab, int* status, cudaStream_t s);
int fb_conf_head(float* conf, const void* xc, const void* emb, const int* draft, const float* w, int streams, int steps, int d,
                 int rank, int block, int stride, cudaStream_t s);
int fb_stream_mean(void* out, long ld, const void* h, int rows, int hc, int dim, cudaStream_t s);
int fb_stream_collapse(void* xc, const void* h, const float* pre, long pre_ld, int rows, int hc, int dim, cudaStream_t s);
// block-drafter sublayers: grouped dynamic conv over a block, merge of per-rank top-16 lists, candidate selector walk
int fb_dynconv(void* out, const void* x, const void* coef, long ldc, const void* base, void* res, int rows, int H, int group,
               int blk, cudaStream_t s);
int fb_topk16_merge(float* ovals, int* oids, const float* vals, const int* ids, int rows, int W, cudaStream_t s);
int fb_draft_select(int* out, const float* vals, const int* ids, const void* gate, const void* a_cb, const void* b_cb,
                    int anchor, int rows, int R, cudaStream_t s);
int fb_topk16(int* ids, float* vals, const void* logits, long stride, int rows, int vocab, int is_f32, cudaStream_t s);

#ifdef __cplusplus
}
#endif
