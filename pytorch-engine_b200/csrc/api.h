// Every entry point of the library, as C prototypes.  Each launcher takes raw device pointers and a stream,
// checks its sizes on the host and returns 0, a negative PE_ERR_* code for a size or argument it refuses
// (common.cuh), or a positive CUDA runtime error number.  kernels/lib.py declares the same signatures for
// ctypes; every .cu file includes this header, so a definition that drifts from it does not compile.
// pe_attention_decode_noalloc is described in attention_noalloc.h.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif


// attention_generic.cu
long long pe_attention_generic_scratch_floats(int n_seqs, int n_heads, int head_dim, int max_splits);
int pe_attention_generic(int dtype, int decode, const void* q, long long q_ld, void* out, long long out_ld,
    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart,
    const int* seq_past, const int* seq_slot, const int* page_table, int table_stride, int num_pages,
    const void* k_pages, const void* v_pages, float* scratch, int split_keys, int max_splits, int* status,
    cudaStream_t stream);
int pe_attention_generic_ex(int dtype, int decode, const void* q, long long q_ld, void* out, long long out_ld,
    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale, int window, int sink,
    const float* out_cos, const float* out_sin, int out_rot, int out_rows, int out_inter, const int* seq_qstart,
    const int* seq_past, const int* seq_slot, const int* page_table, int table_stride, int num_pages,
    const void* k_pages, const void* v_pages, float* scratch, int split_keys, int max_splits, int* status,
    cudaStream_t stream);
int pe_attention_generic_masked(int dtype, int decode, const void* q, long long q_ld, void* out, long long out_ld,
    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale, int window, int chunk,
    int keep_first, int v_ld, int v_heads, int out_f32, int sink, const float* out_cos, const float* out_sin, int out_rot, int out_rows, int out_inter,
    const int* seq_qstart, const int* seq_past, const int* seq_slot, const int* page_table, int table_stride,
    int num_pages, const void* k_pages, const void* v_pages, float* scratch, int split_keys, int max_splits, int* status,
    cudaStream_t stream);
int pe_attention_decode_noalloc(int dtype, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs,
    int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart, const int* seq_past,
    const int* seq_slot, const int* page_table, int table_stride, int num_pages, const void* k_pages,
    const void* v_pages, int split_keys, int max_splits, int* status, cudaStream_t stream);

// attention_mma.cu
int pe_attention_mma_decode_blocks_per_sm(int head_dim);
int pe_attention_mma_supported(int head_dim, int n_heads, int n_kv_heads);
int pe_attention_mma(int decode, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs, int max_q,
    int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart, const int* seq_past,
    const int* seq_slot, const int* page_table, int table_stride, int num_pages, const void* k_pages,
    const void* v_pages, float* scratch, int split_keys, int max_splits, int min_range_keys, int* status,
    cudaStream_t stream);
int pe_attention_mma_ex(int decode, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs, int max_q,
    int n_heads, int n_kv_heads, int head_dim, float scale, int window, int sink, const float* out_cos,
    const float* out_sin, int out_rows, const int* seq_qstart, const int* seq_past, const int* seq_slot,
    const int* page_table, int table_stride, int num_pages, const void* k_pages, const void* v_pages, float* scratch,
    int split_keys, int max_splits, int min_range_keys, int* status, cudaStream_t stream);
int pe_attention_mma_masked(int decode, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs, int max_q,
    int n_heads, int n_kv_heads, int head_dim, float scale, int window, int chunk, int keep_first, int v_heads, int out_f32,
    int split_p, int sink,
    const float* out_cos, const float* out_sin, int out_rows, const int* seq_qstart, const int* seq_past,
    const int* seq_slot, const int* page_table, int table_stride, int num_pages, const void* k_pages,
    const void* v_pages, float* scratch, int split_keys, int max_splits, int min_range_keys, int* status,
    cudaStream_t stream);

// attention_latent.cu
int pe_attention_latent_supported(int row, int rank);
int pe_attention_latent(int decode, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs, int max_q,
    int n_heads, int row, int rank, float scale, const int* seq_qstart, const int* seq_past, const int* seq_slot,
    const int* page_table, int table_stride, int num_pages, const void* pages, float* scratch, int split_keys,
    int max_splits, int min_range_keys, int* status, cudaStream_t stream);

// attention_umma.cu
int pe_attention_umma_supported(int head_dim, int n_heads, int n_kv_heads);
int pe_attention_umma_prefill(const void* q, long long q_ld, long long n_tokens, void* out, long long out_ld,
    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart,
    const int* seq_past, const int* seq_slot, const int* page_table, int table_stride, int num_pages,
    const void* k_pages, const void* v_pages, int n_sms, int* work_counter, int* status, cudaStream_t stream);
int pe_attention_umma_prefill_ex(const void* q, long long q_ld, long long n_tokens, void* out, long long out_ld,
    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, float scale, int window, int sink,
    const float* out_cos, const float* out_sin, int out_rows, const int* seq_qstart, const int* seq_past,
    const int* seq_slot, const int* page_table, int table_stride, int num_pages, const void* k_pages,
    const void* v_pages, int n_sms, int* work_counter, int* status, cudaStream_t stream);

// stream_parts.cu
int pe_norm_token_shift(int out_dtype, const float* x, const float* w, float eps, const float* mix, float* state,
    const int* token_seq, const int* seq_slot, const int* seq_qstart, void* out, int n_tokens, int width, int n_slots,
    int* status, cudaStream_t stream);
int pe_depth_average(const float* results, long long layer_stride, const float* coeff, int n_terms, float* out,
    float* copy, long long n, cudaStream_t stream);
int pe_polynorm(int dtype, const void* z, const float* coeff, float eps, void* out, int n_rows, int width,
    cudaStream_t stream);
int pe_sigmoid_gate(int dtype, const void* x, long long x_head_stride, long long x_token_stride, const void* g,
    long long g_ld, void* out, long long out_ld, int n_tokens, int heads, int dv, int per_head, cudaStream_t stream);
int pe_diff_combine(int dtype, const float* a, void* out, int n_tokens, int heads, int dv, float lambda, float eps,
    float post, cudaStream_t stream);
int pe_rows_to_pages(int dtype, const void* src, long long src_ld, int col0, int heads, int dim, int n_tokens,
    const int* token_seq, const int* token_pos, const int* seq_slot, const int* page_table, int table_stride,
    int num_pages, void* pages, int* status, cudaStream_t stream);
int pe_rows_to_pages_pair(int dtype, const void* src, long long src_ld, int col0, int heads, int dim, int col0_b, int heads_b,
    int dim_b, int n_tokens, const int* token_seq, const int* token_pos, const int* seq_slot, const int* page_table,
    int table_stride, int num_pages, void* pages, void* pages_b, int* status, cudaStream_t stream);
int pe_latent_prepare(int dtype, const void* x, long long x_ld, int q_col0, int low_col0, int heads, int d, int dr,
    int rank, const float* norm_w, float eps, const float* cos_t, const float* sin_t, int rot, int table_rows,
    int n_tokens, const int* token_seq, const int* token_pos, const int* seq_slot, const int* page_table,
    int table_stride, int num_pages, void* pages, void* qfull, const void* absorbed, int write_cache, int* status,
    cudaStream_t stream);

// embedding.cu
int pe_embed_gather(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden, int vocab,
    int* status, cudaStream_t stream);
int pe_embed_gather_scaled(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden, int vocab,
    float scale, float* copy, int* status, cudaStream_t stream);

// gemm_smallm.cu
int pe_gemm_smallm_supported(int M, int N, int K);
int pe_gemm_smallm(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
    int out_f32, int pair_offset, int n_sms, cudaStream_t stream);
int pe_gemm_smallm_grouped(const void* x, long long ldx, long long x_group_stride, int groups, int group_rows,
    const void* w, void* y, long long ldy, int M, int K, int out_f32, int n_sms, cudaStream_t stream);

// gemm_umma.cu
int pe_gemm_umma_supported(int M, int N, int K, int pair_offset);
int pe_gemm_umma(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
    int out_f32, int pair_offset, int n_sms, int* status, cudaStream_t stream);

// gemm_umma2.cu
int pe_gemm_umma2_supported(int M, int N, int K, int pair_offset);
int pe_gemm_umma2(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
    int out_f32, int pair_offset, int n_sms, int* status, cudaStream_t stream);
int pe_gemm_umma2_qkv_rope_supported(int M, int K, int n_heads, int n_kv_heads, int head_dim, int rotary_dim);
int pe_gemm_umma2_qkv_rope(const void* x, long long ldx, const void* w, void* qkv, long long ld, int M, int K,
    int n_heads, int n_kv_heads, int head_dim, const float* q_norm_w, const float* k_norm_w, float eps,
    const float* cos_table, const float* sin_table, int rotary_dim, int table_rows, const int* token_seq,
    const int* token_pos, const int* seq_slot, const int* seq_qstart, const int* page_table, int table_stride,
    int num_pages, void* k_pages, void* v_pages, int write_cache, int n_sms, int* status, cudaStream_t stream);

// rmsnorm.cu
int pe_rmsnorm_residual(int dtype, float* residual, const void* delta, const float* weight, void* out,
    const int* rows, int n_rows, int dim, float eps, cudaStream_t stream);
int pe_rmsnorm(int dtype, const void* x, const float* weight, void* out, int n_rows, int dim, float eps,
    cudaStream_t stream);
int pe_rmsnorm_add(int dtype, float* stream, const void* delta, const float* weight, void* cast, int n_rows, int dim,
    float eps, cudaStream_t stream_);

// rope_append.cu
int pe_batch_expand(const int* seq_qstart, const int* seq_past, int n_seqs, int* token_seq, int* token_pos,
    cudaStream_t stream);
int pe_qk_norm_rope_append(int dtype, void* qkv, long long ld, int n_tokens, int n_heads, int n_kv_heads,
    int head_dim, const float* q_norm_w, const float* k_norm_w, float eps, const float* cos_table,
    const float* sin_table, int rotary_dim, int table_rows, const int* token_seq, const int* token_pos,
    const int* seq_slot, const int* seq_qstart, const int* page_table, int table_stride, int num_pages,
    void* k_pages, void* v_pages, int write_cache, int* status, cudaStream_t stream);
int pe_qkv_rotate_append(int dtype, void* qkv, long long ld, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
    int v_dim, const float* q_norm_w, const float* k_norm_w, float eps, const float* cos_table, const float* sin_table,
    int rotary_dim, int table_rows, int interleaved, int v_unit_norm, const float* v_cos, const float* v_sin,
    int v_rotary_dim, int v_table_rows, int v_interleaved, const int* token_seq, const int* token_pos,
    const int* seq_slot, const int* seq_qstart, const int* page_table, int table_stride, int num_pages, void* k_pages,
    void* v_pages, int write_cache, const float* bias, int* status, cudaStream_t stream);

// sampling.cu
long long pe_sample_scratch_bytes(int n_rows, int vocab, float temperature, int top_k, float top_p, float min_p);
int pe_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k, float top_p,
    float min_p, unsigned long long seed, const int* row_request, const int* row_step, int* out_tokens,
    void* scratch, long long scratch_bytes, cudaStream_t stream);
int pe_repetition_penalty(float* logits, long long ld, int n_rows, int vocab, const int* recent, int recent_stride,
    const int* recent_count, float penalty, cudaStream_t stream);

// swiglu.cu
int pe_silu_mul(int dtype, const void* gate_up, void* out, int n_rows, int inter, cudaStream_t stream);

// token_gate.cu
int pe_token_gate(int dtype, const void* gx, const void* table, long long table_ld, int col0, const int* tokens,
    void* out, int n_tokens, int dim, int vocab, int* status, cudaStream_t stream);

// wkv.cu
int pe_token_shift_mix(int dtype, const void* x, const float* mu, int n_mix, const float* prev_state,
    const int* token_seq, const int* seq_slot, const int* seq_qstart, void* out, int n_tokens, int width, int n_slots,
    int* status, cudaStream_t stream);
int pe_tanh_inplace(int dtype, void* y, long long n, cudaStream_t stream);
long long pe_wkv_scratch_floats(int n_seqs, int heads, int d, int max_chunks);
int pe_wkv_recurrence(int dtype, const void* r, const void* k, const void* v, const void* g, long long ld,
    const float* wlin, const float* w0, const float* u, const float* gnorm, float eps, void* out, float* state,
    float* prev_state, const void* x, int width, const int* seq_slot, const int* seq_qstart, int n_seqs, int max_q,
    int heads, int d, int n_slots, int chunk, int max_chunks, float* scratch, int* status, cudaStream_t stream);

// embedding.cu (pair embedding), rmsnorm.cu (sum of scaled deltas)
int pe_embed_pair_gather(int dtype, const void* table, const void* pairs, const int* ids, const int* token_seq,
    const int* token_pos, const int* seq_slot, const int* seq_qstart, int* last, float* out, int n_tokens, int hidden,
    int vocab, int buckets, int mul_prev, int mul_cur, int n_slots, int* status, cudaStream_t stream);
int pe_rmsnorm_residual_sum(int dtype, float* residual, const void* const* deltas, const float* scales, int n_deltas,
    const float* weight, void* out, const int* rows, int n_rows, int dim, float eps, cudaStream_t stream);

// mlstm.cu
int pe_mlstm_recurrence(int dtype, const void* q, const void* k, const void* v, const void* g, long long ld,
    const float* gates, const float* gate_bias, const float* norm_w, float cap, float eps, float q_scale, void* out,
    float* S, float* n, float* m, const int* seq_slot, const int* seq_qstart, int n_seqs, int max_q, int heads, int d,
    int dv, int n_slots, int chunk, int max_chunks, float* scratch, int* status, cudaStream_t stream);
long long pe_mlstm_scratch_floats(int n_seqs, int heads, int d, int dv, int max_chunks);

// delta_rule.cu
int pe_short_conv_silu(int dtype, const void* x, long long ld, int col0, const float* w, const float* bias, int taps, float* tail,
    const int* token_seq, const int* seq_slot, const int* seq_qstart, void* out, int n_tokens, int n_seqs, int channels,
    int n_slots, int* status, cudaStream_t stream);
int pe_delta_rule_recurrence(int dtype, const void* qkv, const float* a, const float* dt_bias, const float* A_log,
    const float* b, const void* gate, long long gate_ld, const float* norm_w, float eps, float q_scale, void* out, float* S,
    const int* seq_slot, const int* seq_qstart, int n_seqs, int max_q, int heads, int kv_heads, int d, int dv, int n_slots,
    int chunk, int max_chunks, float* scratch, int head_decay, int gate_silu, long long a_ld, long long b_ld, int* status,
    cudaStream_t stream);
long long pe_delta_rule_scratch_floats(int n_seqs, int heads, int d, int dv, int max_chunks);

// moe.cu
int pe_moe_route(const float* logits, const float* correction, int n_tokens, int n_all, int top, int* chosen,
    float* weight, int* dense_rows, int n_real, cudaStream_t stream);
int pe_moe_route_logits(const float* logits, const float* bias, int n_tokens, int n_all, int top, int* chosen,
    float* weight, int* dense_rows, int n_real, cudaStream_t stream);
int pe_moe_route_sigmoid_groups(const float* logits, int n_tokens, int n_all, int top, int n_groups, int keep, int* chosen,
    float* weight, int* dense_rows, int n_real, cudaStream_t stream);
int pe_moe_group(const int* chosen, int n_tokens, int top, int n_real, int* offsets, int* row_token, int* pair_row,
    cudaStream_t stream);
int pe_moe_rows_gemm(int dtype, int out_dtype, const void* x, long long x_ld, const int* row_map, const int* offsets,
    int n_groups, int max_rows, const void* w, long long w_group_stride, void* out, long long out_ld, int n_out, int k_dim,
    int glu, float limit, float alpha, cudaStream_t stream);
int pe_moe_gather_rows(int dtype, const void* x, const int* row_token, const int* offsets, int n_groups, void* xs,
    int max_rows, int width, cudaStream_t stream);
int pe_moe_combine(int dtype, const void* rows, const void* x, const void* shared, const int* pair_row,
    const float* weight, int top, void* out, int n_tokens, int width, cudaStream_t stream);
int pe_glu_act(int dtype, const void* gate_up, void* out, int n_rows, int inter, int kind, float limit, float alpha,
    cudaStream_t stream);

// ssd.cu
int pe_ssd_recurrence(int dtype, const void* xbc, long long xbc_ld, const void* dt, long long dt_ld, const float* dt_bias,
    const float* A_log, const float* D, float* y, float* S, const int* seq_slot, const int* seq_qstart, int n_seqs, int max_q,
    int heads, int groups, int n, int dv, int n_slots, int chunk, int max_chunks, float* scratch, int* status,
    cudaStream_t stream);
long long pe_ssd_scratch_floats(int n_seqs, int heads, int n, int dv, int max_chunks);
int pe_gated_part_norm(int dtype, const float* y, const void* z, long long z_ld, const float* w, float eps, void* out,
    int n_tokens, int width, int parts, cudaStream_t stream);

// dyt.cu
int pe_dyt(int dtype, int in_f32, const void* x, const int* rows, const float* w, const float* b, float alpha, void* out,
    int n_rows, int dim, cudaStream_t stream);
int pe_dyt_add(int dtype, float* stream_rows, const void* delta, const float* w1, const float* b1, float alpha1,
    const float* w2, const float* b2, float alpha2, void* out, int n_rows, int dim, cudaStream_t stream);
int pe_rmsnorm_pair_mix(int dtype, const void* a, const void* b, const float* wa, const float* wb, float eps, float sa,
    float sb, void* out, int n_rows, int dim, cudaStream_t stream);

int pe_rmsnorm_pair_mix_dyt_add(int dtype, const void* a, const void* b, const float* wa, const float* wb, float eps, float sa,
    float sb, float* stream_rows, const float* w1, const float* b1, float alpha1, const float* w2, const float* b2, float alpha2,
    void* out, int n_rows, int dim, cudaStream_t stream);
int pe_concat_split(int dtype, const float* a, const float* b, void* hi, void* lo, int n_rows, int dim, cudaStream_t stream);

// wait_probe.cu
int pe_wait_probe(unsigned long long* out, int polls, cudaStream_t stream);
long long pe_wait_limit_polls();

#ifdef __cplusplus
}
#endif
