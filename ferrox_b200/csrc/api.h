// C entry points of the kernel library (libferrox_b200.so).  Every function
// enqueues work on `stream` (a cudaStream_t passed as void*) and returns 0, a
// cudaError_t (> 0) from the launch, or one of the negative FX_ERR_* codes of
// common.cuh when it refuses its arguments.  Nothing here allocates or synchronises.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int fx_gemm(const void* A, int a_dtype, long lda, const int* a_rows, const void* W, int w_dtype, long ldw,
            const void* bias, int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int M, int N, int K,
            const int* group_offsets, int n_groups, long w_group_stride, void* stream);

// Streaming multiprocessors of the current device (asked once).
int fx_sm_count();

// Programmatic dependent launch of the short kernels on (1, default) or off (0); returns the old setting.
int fx_set_pdl(int on);

int fx_embed(const void* table, int dtype, const int* ids, float* out, int n_tokens, int hidden, int vocab,
             int* status, void* stream);
int fx_rmsnorm(const float* x, const int* rows, const void* w, int w_dtype, float eps, void* out, int out_dtype,
               int n_rows, int hidden, void* stream);
int fx_silu_mul(const void* gu, long ld_in, void* out, long ld_out, int dtype, const int* n_rows_dev, int rows, int n,
                void* stream);
int fx_rope_kv_write(void* qkv, int dtype, long ld, const int* positions, const int* token_seq, const int* seq_slot,
                     const float* inv_freq, const float* cos_sin, int rotary_dim, int pairing, void* k_pages, void* v_pages, const int* block_table,
                     int table_width, int page_size, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                     int write_cache, int* status, void* stream);
int fx_moe_combine(float* h, const void* y, int dtype, const int* inv_perm, const float* topk_w, int top_k,
                   const void* shared, const float* shared_gate_logit, long gate_ld, int n_tokens, int hidden,
                   void* stream);
int fx_residual_add(float* h, const void* y, int dtype, long n, void* stream);

int fx_paged_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, int dtype,
                       const int* block_table, int table_width, int page_size, const int* positions,
                       const int* token_seq, const int* seq_slot, void* out, long ldo, int n_tokens, int n_heads,
                       int n_kv_heads, int head_dim, int window, float scale, void* stream);

int fx_prefill_attention_tc(const void* q, long ldq, int n_tokens, const void* k_pages, const void* v_pages, int n_pages,
                            const int* block_table, int table_width, int page_size, const int* items, int n_items,
                            const int* seq_slot, void* out, long ldo, int n_heads, int n_kv_heads, int head_dim,
                            int window, float scale, int* status, float* part_o, float* part_ml, const int* merges,
                            int n_merges, void* stream);
int fx_prefill_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, const int* block_table,
                         int table_width, int page_size, const int* tiles, int n_tiles, const int* seq_slot, void* out,
                         long ldo, int n_heads, int n_kv_heads, int head_dim, int window, float scale, void* stream);

int fx_router_topk(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids,
                   float* weights, void* stream);
int fx_moe_align(const int* ids, int n_tokens, int top_k, int n_experts, int* scratch, int* offsets, int* src_token,
                 int* inv_perm, int* active, int n_slots, void* stream);

int fx_gemm_tc(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows, const void* bias,
               int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int M, int N, int K, int gated,
               int gate_up_offset, const int* group_offsets, int n_groups, int* status, void* stream);
int fx_gemm_tc_swap(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows, const void* bias,
                    int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int M, int N, int K, int gated,
                    int gate_up_offset, const int* group_offsets, int n_groups, int tokens_per_tile, int weights_first,
                    int k_splits, float* partials, int* status, void* stream);
int fx_gemm_tc2(const void* X, long ldx, const void* W, long ldw, int w_rows, const void* bias, int bias_dtype, void* C,
                int c_dtype, long ldc, int accumulate, int M, int N, int K, int gated, int gate_up_offset, int* status,
                void* stream);
int fx_moe_combine_norm(float* h, const void* y, int dtype, const int* inv_perm, const float* topk_w, int top_k,
                        const void* shared, const float* shared_gate_logit, long gate_ld, int n_tokens, int hidden,
                        const void* norm_w, int norm_w_dtype, float eps, void* x_out, void* stream);
int fx_gather_rows(const void* x, long ldx, const int* rows, void* out, long ldo, int dtype, int n_rows, int width,
                   void* stream);
int fx_route(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids, float* weights,
             int* scratch, int* offsets, int* src_token, int* inv_perm, int* active, int n_slots, void* stream);
int fx_route_small(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids, float* weights,
                   int* offsets, int* src_token, int* inv_perm, int* active, int n_slots, void* stream);
int fx_route_fused(const void* X, long ldx, const void* W, long ldw, int n_tokens, int n_route, int n_experts, int hidden,
                   int top_k, int renorm, float* logits, long ldl, int* ids, float* weights, int* offsets, int* src_token,
                   int* inv_perm, int* active, int n_slots, void* xp_out, long ldxp, void* stream);
int fx_rope_table(const int* positions, const float* inv_freq, int n_tokens, int half, float* cos_sin, void* stream);
// A few tokens against a plain matrix that fits the shared memory of all SMs together (gemm_slab.cu): every block asks
// for its whole slab of W before it waits for the kernel before it on the stream, which therefore must not have written W.
// C[t, n] (+)= sum_k X[t, k] W[n, k] (+ bias[n]); bfloat16 X and W, K a multiple of 128, C bfloat16 or float32.
int fx_gemm_slab_ok(int N, int K, int n_tokens);
int fx_gemm_slab(const void* X, long ldx, const void* W, long ldw, const void* bias, int bias_dtype, void* C,
                 int c_dtype, long ldc, int accumulate, int n_tokens, int N, int K, int* status, void* stream);

int fx_gemm_skinny(const void* X, long ldx, const int* x_rows, const void* W, long ldw, long w_group_stride,
                   const void* bias, int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int n_tokens,
                   int N, int K, int gated, int gate_up_offset, const int* group_offsets, const int* active_groups,
                   int n_slots, int tokens_hint, int c_transposed, void* stream);
int fx_decode_split_mma(const void* q, long ldq, const void* k_pages, const void* v_pages, const int* block_table,
                        int table_width, int page_size, const int* positions, const int* token_seq, const int* seq_slot,
                        float* part_acc, float* part_ml, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                        int window, float scale, int split_len, int n_splits, int fresh_positions, void* stream);
int fx_decode_split_tma(const void* q, long ldq, const void* k_pages, const void* v_pages, int n_pages,
                        const int* block_table, int table_width, int page_size, const int* positions,
                        const int* token_seq, const int* seq_slot, float* part_acc, float* part_ml, int n_tokens,
                        int n_heads, int n_kv_heads, int head_dim, int window, float scale, int split_len,
                        int n_splits, int* status, void* out, long ldo, int* counters, int fresh_positions,
                        int store_new, int write_pages, const float* cos_sin, void* stream);
// n_pages > 0 (the number of pages behind k_pages / v_pages) lets bfloat16 take the TMA kernel; status: the step's
// status word (may be null).
// fresh_positions: 0 makes no assumption about the kernel launched before this one on the stream: nothing is read until
// it has finished.  N > 0 is the caller's promise that that kernel wrote, of everything this call reads, only the
// queries and the keys and values of at most the last N positions of each request (positions, token_seq, seq_slot and
// the block table are older); the bfloat16 kernels then fetch tiles of older keys while that kernel still runs.  A
// promise that does not hold gives stale keys without any error.
// store_new = 1 (bfloat16, head sizes in steps of 64, pages of a multiple of 64 positions, one token a request; else
// refused): `q` is the step's fused [q | k | v] rows as projected, and the kernel does the rotary kernel's work
// itself: it rotates the queries (split-half pairs over the whole head; cos_sin [tokens][head_dim / 2][2] from
// fx_rope_table, or null for no rotation), and rotates and stores each token's own key and value (into the pages only
// if write_pages).  The kernel before it must then not write the pages at all.
int fx_decode_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, int n_pages, int dtype,
                        const int* block_table, int table_width, int page_size, const int* positions,
                        const int* token_seq, const int* seq_slot, void* out, long ldo, float* part_acc,
                        float* part_ml, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int window,
                        float scale, int split_len, int n_splits, int* status, int* counters, int fresh_positions,
                        int store_new, int write_pages, const float* cos_sin, void* stream);

// out[i] = mean + stdev * z_i, z the standard normal stream of `key` (random_init.cu; the host restates the rule
// bit for bit).  dtype: FX_F32 or FX_BF16.
int fx_random_normal(void* out, int dtype, long n, unsigned long long key, double mean, double stdev, void* stream);

int fx_argmax(const float* logits, long ld, int n_rows, int vocab, int* out, void* stream);
int fx_sample_or(const float* scores, long lds, float* work, long ld, int n_rows, int vocab, const float* temperature,
                 const int* top_k, const float* top_p, const float* draw, const int* use_sample, const int* instead,
                 int* out, void* stream);
int fx_repetition_penalty(float* work, long ld, int n_rows, int vocab, const int* history, const int* hist_offsets,
                          const float* penalty, void* stream);
int fx_sample(float* work, long ld, int n_rows, int vocab, const float* temperature, const int* top_k,
              const float* top_p, const float* draw, int* out, void* stream);

#ifdef __cplusplus
}
#endif
