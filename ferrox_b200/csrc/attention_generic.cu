// Attention of every query token over its own request's cache pages: one kernel
// for whole prompts, portions of prompts and single decoded tokens alike.
//
// The query at absolute position p of a request sees the keys at positions
// max(0, p - W + 1) .. p of that request (W = window, 0 = all), found through
// the request's block table: position t lives in page table[t / page_size] at
// offset t % page_size.  K and V of the tokens of this step were written to the
// pages before this kernel runs, so earlier steps' keys and this portion's keys
// are read the same way, and the mask is a function of absolute positions only.
//
// One warp per (token, head).  Keys are taken in blocks of 32 aligned to absolute
// positions; lane j scores key j of the block with the full 32-bit dot product,
// the block's maximum and sum update a running (m, l) pair, and the 32 lanes then
// share out the head dimension for the sum of p * V.  The order of every sum is
// fixed by (p, W) alone: the result does not depend on how the tokens were cut
// into steps, on the batch, or on which pages hold the keys.
//
// Reference: online softmax crates/ferrox-core/src/attention.rs:146-175; head h
// reads kv head h / (n_heads / n_kv_heads), scale 1/sqrt(head_dim) :432-449; window
// = the last W positions, the query's own included :484-524; pages :572-610.
// CUDA-core arithmetic throughout: this is the 32-bit path and the fallback of the
// bfloat16 path.  head_dim <= 256.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_kernel(
    const T* __restrict__ q, long ldq, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    const int* __restrict__ block_table, int table_width, int page_size,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
    T* __restrict__ out, long ldo, int n_heads, int n_kv_heads, int head_dim, int window, float scale)
{
    __shared__ float q_s[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= n_heads) return;  // whole warp leaves; no block-wide barrier below
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (long)seq_slot[token_seq[t]] * table_width;
    const T* qh = q + (long)t * ldq + (long)h * head_dim;
    for (int i = lane; i < head_dim; i += 32) q_s[warp][i] = to_f32(qh[i]) ;
    __syncwarp();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;
    const long head_stride = (long)page_size * head_dim;

    for (int kb = (lo / 32) * 32; kb <= pos; kb += 32) {
        const int key = kb + lane;
        bool valid = key >= lo && key <= pos;
        long base = -1;
        float s = -INFINITY;
        const int page = valid ? table[key / page_size] : -1;
        valid = valid && page >= 0;  // a position without a page is skipped, never dereferenced
        if (valid) {
            base = ((long)page * n_kv_heads + kvh) * head_stride + (long)(key % page_size) * head_dim;
            const T* kr = k_pages + base;
            float dot = 0.f;
            for (int i = 0; i < head_dim; ++i) dot = fmaf(q_s[warp][i], to_f32(kr[i]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;  // no key of this block is readable (uniform across the warp)
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long bj = __shfl_sync(0xffffffffu, base, j);
            if (bj < 0) continue;  // uniform across the warp
            const T* vr = v_pages + bj;
#pragma unroll
            for (int i = 0; i < MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (long)t * ldo + (long)h * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) o[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace

extern "C" int fx_paged_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, int dtype,
                                  const int* block_table, int table_width, int page_size, const int* positions,
                                  const int* token_seq, const int* seq_slot, void* out, long ldo, int n_tokens,
                                  int n_heads, int n_kv_heads, int head_dim, int window, float scale, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (head_dim > MAX_D || head_dim <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, (unsigned)fx_cdiv(n_heads, WARPS));
    if (dtype == FX_F32)
        paged_attention_kernel<float><<<grid, WARPS * 32, 0, s>>>((const float*)q, ldq, (const float*)k_pages,
            (const float*)v_pages, block_table, table_width, page_size, positions, token_seq, seq_slot, (float*)out,
            ldo, n_heads, n_kv_heads, head_dim, window, scale);
    else if (dtype == FX_BF16)
        paged_attention_kernel<bf16><<<grid, WARPS * 32, 0, s>>>((const bf16*)q, ldq, (const bf16*)k_pages,
            (const bf16*)v_pages, block_table, table_width, page_size, positions, token_seq, seq_slot, (bf16*)out,
            ldo, n_heads, n_kv_heads, head_dim, window, scale);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}
