// C launch API of the sm_100a kernels. Every function enqueues on the given stream, allocates nothing and
// returns 0 on success, a negative value for an unsupported argument, or a positive cudaError_t.
// The Python bindings (bindings.cpp) and C callers share these symbols.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- elementwise.cu ----
int fb_embed(void* out, const void* table, const int* ids, int rows, int hidden, int vocab, cudaStream_t s);
int fb_rmsnorm(void* out, void* x_out, const void* x, const void* res, const void* w, int rows, int hidden, float eps,
               int centred, cudaStream_t s);
int fb_silu_mul(void* out, const void* gu, int rows, int inter, float clamp, cudaStream_t s);
int fb_gated_norm(void* out, const float* y, const void* z, long z_stride, const void* w, int rows, int heads, int dv,
                  float eps, cudaStream_t s);
int fb_gather_rows(void* out, const void* in, const int* idx, int rows, int width, cudaStream_t s);
int fb_add_bf16(void* x, const void* y, long n, cudaStream_t s);
int fb_bf16_to_f32(float* out, const void* in, long n, cudaStream_t s);

// ---- gemv.cu ----
int fb_gemv_bf16(void* Y, const void* X, const void* W, const void* norm_w, const void* res, int M, int N, int K,
                 long ldx, long ldy, float eps, int centred, int out_f32, int mode, int sm_count, cudaStream_t s);

// ---- gemm_tcgen05.cu ----
// Y[M][N] = X[M][K] * W[N][K]^T (+ res), or SwiGLU over W = [gate rows | up rows] (2N rows). bf16 in/out,
// fp32 accumulation in TMEM. workspace/counters are needed only when split_k > 1.
int fb_gemm_bf16(void* Y, const void* X, const void* W, const void* res, int M, int N, int K, long ldx, long ldy,
                 int mode, int split_k, float* workspace, int* counters, int* status, int sm_count, cudaStream_t s);
long fb_gemm_workspace_bytes(int M, int N, int split_k);

// 2..32 rows: weight-streaming linear on mma.sync with in-register A fragments (gemv_mma.cu)
int fb_gemv_mma(void* y, const void* x, const void* w, const void* norm_w, const void* res, int M, int N, int K, long ldx,
                long ldy, float eps, int mode, int out_f32, float* ws, long ws_floats, int* counters, int n_counters,
                int sm_count, cudaStream_t s);
// FP8 (e4m3) GEMM with per-row / per-feature scales, and the activation quantiser (gemm_tcgen05.cu)
int fb_quant_fp8(void* q, float* scale, const void* x, const void* norm_w, int rows, int K, long ldx, float eps,
                 cudaStream_t s);
// block-scaled form (gemm_fp8_block.cu): activations scaled per (row, 128 k), weights per (128 features, 128 k);
// code matrices are padded to whole k blocks: [rows][kblocks * 128]
long fb_fp8_block_kblocks(int K);
int fb_quant_fp8_block(void* q, float* scale, const void* x, int rows, int K, long ldx, cudaStream_t s);
int fb_gemm_fp8_block(void* Y, const void* Xq, const float* sx, const void* Wq, const float* sw, const void* res, int M,
                      int N, int K, long ldy, int* status, cudaStream_t s);
int fb_gemm_fp8(void* Y, const void* Xq, const void* Wq, const float* scale_m, const float* scale_n, const void* res, int M,
                int N, int K, long ldy, int mode, int split_k, float* workspace, int* counters, int* status, int sm_count,
                cudaStream_t s);

// ---- attn.cu ----
int fb_attn_prep(void* q_out, void* k_cache, void* v_cache, const void* proj, long proj_stride, const void* q_norm,
                 const void* k_norm, const float* inv_freq, const int* row_slot, const int* row_pos,
                 const int* block_table, int max_blocks, int kv_block, int rows, int nq, int nkv, int hd, int rot,
                 int gated, float eps, int* status, cudaStream_t s);
// verify-tree rows: rotary position `row_pos` (depth) and cache row `row_cpos` differ; kv_scale != null: e4m3 cache
int fb_attn_prep_tree(void* q_out, void* k_cache, void* v_cache, float* kv_scale, const void* proj, long proj_stride,
                      const void* q_norm, const void* k_norm, const float* inv_freq, const int* row_slot,
                      const int* row_pos, const int* row_cpos, const int* block_table, int max_blocks, int kv_block,
                      int rows, int nq, int nkv, int hd, int rot, int gated, float eps, int* status, cudaStream_t s);
int fb_attn_decode(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache, const void* v_cache,
                   const void* proj, long proj_stride, const int* row_slot, const int* row_kvlen, const int* row_base,
                   const unsigned long long* row_mask, const int* block_table, int max_blocks, int kv_block, int rows,
                   int nq, int nkv, int hd, int nsplit, int gated, cudaStream_t s);
// FP8 (e4m3) KV cache variants: byte codes + one fp32 scale per (token, kv head) for K and V; fb_kv_dequant decodes
// the rows a prompt step can see into a per-slot bf16 scratch for the prompt attention kernel
int fb_attn_prep_kv8(void* q_out, void* k_cache8, void* v_cache8, float* kv_scale, const void* proj, long proj_stride,
                     const void* q_norm, const void* k_norm, const float* inv_freq, const int* row_slot, const int* row_pos,
                     const int* block_table, int max_blocks, int kv_block, int rows, int nq, int nkv, int hd, int rot,
                     int gated, float eps, int* status, cudaStream_t s);
int fb_attn_decode_kv8(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache8, const void* v_cache8,
                       const float* kv_scale, const void* proj, long proj_stride, const int* row_slot, const int* row_kvlen,
                       const int* row_base, const unsigned long long* row_mask, const int* block_table, int max_blocks,
                       int kv_block, int rows, int nq, int nkv, int hd, int nsplit, int gated, cudaStream_t s);
int fb_kv_dequant(void* k_out, void* v_out, const void* k_cache8, const void* v_cache8, const float* kv_scale,
                  const int* seg_slot, const int* seg_pos0, const int* seg_nrows, const int* block_table, int max_blocks,
                  int kv_block, int nseg, int max_kvlen, int nkv, int hd, int scratch_tokens_per_slot, cudaStream_t s);
int fb_attn_prefill(void* out, const void* q, const void* k_cache, const void* v_cache, const void* proj,
                    long proj_stride, const int* seg_slot, const int* seg_row0, const int* seg_nrows,
                    const int* seg_pos0, const int* block_table, int max_blocks, int kv_block, int nseg, int max_rows,
                    int nq, int nkv, int hd, int gated, cudaStream_t s);
int fb_attn_combine(void* out, const float* o_part, const float* ml_part, const void* proj, long proj_stride, int rows,
                    int nq, int hd, int nsplit, int gated, cudaStream_t s);
// tensor-core (mma.sync) decode / verify / tree attention over bf16 or e4m3 (kv_scale != null) caches, rows addressed
// through their segments
int fb_attn_decode_mma(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache, const void* v_cache,
                       const float* kv_scale, const void* proj, long proj_stride, const int* seg_slot, const int* seg_row0, const int* seg_nrows,
                       const int* row_kvlen, const int* row_base, const unsigned long long* row_mask,
                       const int* block_table, int max_blocks, int kv_block, int nseg, int max_rows, int rows, int nq,
                       int nkv, int hd, int nsplit, int gated, cudaStream_t s);
// 4-bit KV cache: codes [..][hd/2] bytes, scales [..][2 * hd/32] fp32 per (token, kv head) row (K groups, V groups)
int fb_attn_prep_q4(void* q_out, void* k_cache4, void* v_cache4, float* kv_scale, const void* proj, long proj_stride,
                    const void* q_norm, const void* k_norm, const float* inv_freq, const int* row_slot, const int* row_pos,
                    const int* row_cpos, const int* block_table, int max_blocks, int kv_block, int rows, int nq, int nkv,
                    int hd, int rot, int gated, float eps, int* status, cudaStream_t s);
int fb_attn_decode_q4(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache4, const void* v_cache4,
                      const float* kv_scale, const void* proj, long proj_stride, const int* row_slot, const int* row_kvlen,
                      const int* row_base, const unsigned long long* row_mask, const int* block_table, int max_blocks,
                      int kv_block, int rows, int nq, int nkv, int hd, int nsplit, int gated, cudaStream_t s);
int fb_kv_dequant_q4(void* k_out, void* v_out, const void* k_cache4, const void* v_cache4, const float* kv_scale,
                     const int* seg_slot, const int* seg_pos0, const int* seg_nrows, const int* block_table, int max_blocks,
                     int kv_block, int nseg, int max_kvlen, int nkv, int hd, int scratch_tokens_per_slot, cudaStream_t s);
// low-bit KV cache, general form (bits 4 or 6; `hrot`: keys stored / queries handed out Walsh-Hadamard rotated)
int fb_attn_prep_qn(void* q_out, void* k_cache, void* v_cache, float* kv_scale, const void* proj, long proj_stride,
                    const void* q_norm, const void* k_norm, const float* inv_freq, const int* row_slot, const int* row_pos,
                    const int* row_cpos, const int* block_table, int max_blocks, int kv_block, int rows, int nq, int nkv,
                    int hd, int rot, int gated, float eps, int* status, int bits, int hrot, cudaStream_t s);
int fb_attn_decode_qn(void* out, float* o_part, float* ml_part, const void* q, const void* k_cache, const void* v_cache,
                      const float* kv_scale, const void* proj, long proj_stride, const int* row_slot, const int* row_kvlen,
                      const int* row_base, const unsigned long long* row_mask, const int* block_table, int max_blocks,
                      int kv_block, int rows, int nq, int nkv, int hd, int nsplit, int gated, int bits, cudaStream_t s);
int fb_kv_dequant_qn(void* k_out, void* v_out, const void* k_cache, const void* v_cache, const float* kv_scale,
                     const int* seg_slot, const int* seg_pos0, const int* seg_nrows, const int* block_table, int max_blocks,
                     int kv_block, int nseg, int max_kvlen, int nkv, int hd, int scratch_tokens_per_slot, int bits,
                     cudaStream_t s);
// tcgen05 / TMEM form (attn_prefill_tc.cu): hd 64/128/256 and kv_block a multiple of 64, else returns -20
int fb_attn_prefill_tc(void* out, const void* q, const void* k_cache, const void* v_cache, const void* proj,
                       long proj_stride, const int* seg_slot, const int* seg_row0, const int* seg_nrows,
                       const int* seg_pos0, const int* block_table, int max_blocks, int kv_block, int nseg, int max_rows,
                       long q_rows, long cache_rows, int nq, int nkv, int hd, int gated, int* status, cudaStream_t s);

// ---- gdn.cu ----
int fb_gdn_conv(void* out, const void* proj, long proj_stride, const void* conv_w, const void* conv_state,
                const int* seg_slot, const int* seg_row0, const int* seg_nrows, int nseg, int max_rows, int conv_dim,
                cudaStream_t s);
// verify trees: windows / states follow `row_parent` (parent row inside the segment, -1 = root); see gdn.cu
long fb_gdn_tree_scratch_bytes(int rows, int nv, int dk, int dv);
int fb_gdn_conv_tree(void* out, const void* proj, long proj_stride, const void* conv_w, const void* conv_state,
                     const int* seg_slot, const int* seg_row0, const int* seg_nrows, const int* row_parent, int nseg,
                     int conv_dim, cudaStream_t s);
int fb_gdn_rec_tree(float* y, float* rec_state, const void* qkv, const void* proj, long proj_stride, const float* A_log,
                    const float* dt_bias, const int* seg_slot, const int* seg_row0, const int* seg_nrows,
                    const int* row_parent, const int* row_flags, float* node_state, int nseg, int nk, int nv, int dk,
                    int dv, float eps, cudaStream_t s);
int fb_gdn_rec(float* y, float* rec_state, void* conv_state, const void* qkv, const void* proj, long proj_stride,
               const float* A_log, const float* dt_bias, const int* seg_slot, const int* seg_row0,
               const int* seg_nrows, int nseg, int nk, int nv, int dk, int dv, float eps, int commit, cudaStream_t s);
// decode rows: conv + recurrence + gated norm of a layer in one launch (bf16 out [rows][nv * dv])
int fb_gdn_step(void* out, float* rec_state, void* conv_state, const void* proj, long proj_stride, const void* conv_w,
                const float* A_log, const float* dt_bias, const void* gnorm_w, const int* seg_slot, const int* seg_row0,
                const int* seg_nrows, int nseg, int nk, int nv, int dk, int dv, float eps, int commit, cudaStream_t s);
// chunked scan for prompt-sized segments; `scratch` holds fb_gdn_chunk_scratch_bytes(rows, nseg, nv, dk) bytes
long fb_gdn_chunk_scratch_bytes(int rows, int nseg, int nv, int dk);
int fb_gdn_chunk(float* y, float* rec_state, void* conv_state, float* scratch, const void* qkv, const void* proj,
                 long proj_stride, const float* A_log, const float* dt_bias, const int* seg_slot, const int* seg_row0,
                 const int* seg_nrows, int nseg, int max_rows, int nk, int nv, int dk, int dv, float eps, int commit,
                 cudaStream_t s);

// ---- sample.cu ----
int fb_argmax(int* ids, float* vals, int* finite, const void* logits, long stride, int rows, int vocab, int is_f32,
              cudaStream_t s);
int fb_argmax2(int* ids, float* vals, int* finite, const void* logits, long stride, int rows, int vocab, int is_f32,
               void* scratch, cudaStream_t s);
int fb_sample(int* ids, const void* logits, long stride, int rows, int vocab, const void* params, const int* counts,
              float* work, int is_f32, cudaStream_t s);
// accepted tree path: cache rows src[i] -> dst[i] (flat row = page * kv_block + offset), moves grouped per segment
int fb_kv_move_rows(void* k, long k_row_bytes, void* v, long v_row_bytes, void* sc, long sc_row_bytes, const int* src,
                    const int* dst, const int* seg_off, int nseg, cudaStream_t s);
int fb_chain_accept(int* n_accept, int* out_tokens, const int* target, const int* draft, const int* seg_row0,
                    const int* seg_ndraft, int nseg, int max_draft, cudaStream_t s);

#ifdef __cplusplus
}
#endif
