// Split-key attention for decoding in bfloat16 on the tensor cores.
//
// Same contract and same partial results as decode_split_kernel (attention_decode.cu):
//   grid = (kv head [x block of 16 query heads], query token, key range),
//   partial (max, sum, acc) per (token, head, range) to scratch, merged by merge_kernel.
// The CUDA-core kernel spends about a hundred instructions per key on conversions, dot
// products and shuffles and is bound by instruction issue; here the query heads that
// share a kv head form the 16 rows of an mma.sync.m16n8k16 tile (rows beyond the group
// are zero), so a warp scores 16 keys with 16 instructions and adds them to the output
// with 16 more.  With one head per kv head most of the tile is idle, which costs
// nothing: the kernel is bound by the bytes of K and V.
//
// A block has 4 warps.  Tiles of 64 keys arrive in shared memory by cp.async (two
// buffers, rows padded by 16 bytes against bank conflicts); warp w takes keys
// 16w..16w+15 of every tile and keeps its own running (m, l, O); the four are merged
// in warp order at the end.  Scores, softmax and sums are 32-bit; P is rounded to
// bfloat16 for the second product, as in the prompt kernel.
//
// Launched as a dependent of the kernel that wrote the step's queries and newest keys, a block fetches its
// first tile of older keys before it waits for that kernel; the caller must not have more than 64 new positions
// of a request written by the kernel directly before this one (the engine sends at most 8 this way).
//
// Reference: crates/ferrox-core/src/attention.rs:146-175 (online softmax), :484-524
// (window), :572-610 (pages).
#include "common.cuh"
#include "api.h"

namespace {

constexpr int NTHREADS = 128, TK = 64, STAGES = 2, MAXQ = 16;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int DMAX>
__global__ void __launch_bounds__(NTHREADS) decode_mma_kernel(
    const bf16* __restrict__ q, long ldq, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
    const int* __restrict__ block_table, int table_width, int page_size,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
    float* __restrict__ part_acc, float* __restrict__ part_ml,
    int n_heads, int n_kv_heads, int head_dim, int window, float scale_log2e, float scale, int split_len, int n_splits,
    int fresh)
{
    // fresh <= 0: nothing is known about the kernel before this one, so nothing is read before it has finished.
    if (fresh <= 0) fx_pdl_wait();
    const int group_size = n_heads / n_kv_heads;
    const int chunks = (group_size + MAXQ - 1) / MAXQ;
    const int kvh = blockIdx.x / chunks;
    const int h0 = kvh * group_size + (blockIdx.x % chunks) * MAXQ;   // first query head of this block
    const int nq = min(MAXQ, kvh * group_size + group_size - h0);
    const int tkn = blockIdx.y, split = blockIdx.z;
    const int pos = positions[tkn];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    int k_begin, k_end;
    fx_split_range(pos, lo, split, n_splits, split_len, k_begin, k_end);
    if (k_begin >= k_end) return;   // nothing of this range is visible: `merge` skips it by the same rule

    extern __shared__ __align__(16) uint8_t smem[];
    const int pitch = head_dim * 2 + 16;
    uint8_t* q_s = smem;                                   // [16][pitch]
    uint8_t* kv_s = q_s + 16 * pitch;                      // [STAGES][2][TK][pitch]
    uint8_t* flag_s = kv_s + STAGES * 2 * TK * pitch;      // [STAGES][TK]
    const uint32_t q_u = (uint32_t)__cvta_generic_to_shared(q_s);
    const uint32_t kv_u = (uint32_t)__cvta_generic_to_shared(kv_s);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int chunks_row = head_dim / 8;                   // 16-byte chunks per row
    const int* table = block_table + (long)seq_slot[token_seq[tkn]] * table_width;
    const long head_stride = (long)page_size * head_dim;
    const int n_tiles = (k_end - k_begin + TK - 1) / TK;

    // query rows of this block (zero beyond the group)
    auto load_q = [&]() {
        for (int c = threadIdx.x; c < 16 * chunks_row; c += NTHREADS) {
            const int r = c / chunks_row, ch = c - r * chunks_row;
            const bf16* src = q + (long)tkn * ldq + (long)(h0 + min(r, nq - 1)) * head_dim + ch * 8;
            cp_async16(q_u + r * pitch + ch * 16, src, r < nq ? 16 : 0);
        }
    };
    const bool lanes_fit = chunks_row <= NTHREADS && NTHREADS % chunks_row == 0;
    const int my_ch = lanes_fit ? threadIdx.x % chunks_row : 0;
    const int my_r0 = lanes_fit ? threadIdx.x / chunks_row : 0;
    const int rows_per_pass = lanes_fit ? NTHREADS / chunks_row : 1;
    auto load_tile = [&](int tile, int buf) {
        const int key0 = k_begin + tile * TK;
        const uint32_t ku = kv_u + buf * 2 * TK * pitch, vu = ku + TK * pitch;
        uint8_t* fl = flag_s + buf * TK;
        if (lanes_fit && page_size % TK == 0 && key0 % TK == 0) {
            // the tile lies in one page: one table lookup
            const int page = table[key0 / page_size];
            const long tile_base = page >= 0 ? ((long)page * n_kv_heads + kvh) * head_stride + (long)(key0 % page_size) * head_dim : 0;
            for (int r = my_r0; r < TK; r += rows_per_pass) {
                const bool ok = page >= 0 && key0 + r < k_end;
                const long off = tile_base + (ok ? (long)r * head_dim : 0) + my_ch * 8;
                cp_async16(ku + r * pitch + my_ch * 16, k_pages + off, ok ? 16 : 0);
                cp_async16(vu + r * pitch + my_ch * 16, v_pages + off, ok ? 16 : 0);
                if (my_ch == 0) fl[r] = ok ? 1 : 0;
            }
            return;
        }
        for (int c = threadIdx.x; c < TK * chunks_row; c += NTHREADS) {
            const int r = c / chunks_row, ch = c - r * chunks_row;
            const int key = key0 + r;
            int page = -1;
            if (key < k_end) page = table[key / page_size];
            const bool ok = page >= 0;   // a position without a page is skipped, never dereferenced
            const long off = ok ? ((long)page * n_kv_heads + kvh) * head_stride + (long)(key % page_size) * head_dim + ch * 8 : 0;
            cp_async16(ku + r * pitch + ch * 16, k_pages + off, ok ? 16 : 0);
            cp_async16(vu + r * pitch + ch * 16, v_pages + off, ok ? 16 : 0);
            if (ch == 0) fl[r] = ok ? 1 : 0;
        }
    };
    // fresh > 0 is the caller's promise: the kernel before this one on the stream wrote the queries and the keys and
    // values of at most the last `fresh` positions of each request, and nothing else that this kernel reads
    // (positions, slots and block table are older).  A block whose first tile ends before those positions then asks
    // for it before it waits for that kernel.
    const bool early = fresh > 0 && k_begin + TK <= pos + 1 - fresh;
    if (early) load_tile(0, 0);
    fx_pdl_wait();
    load_q();
    if (!early) load_tile(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the ring: STAGES - 1 tiles are in flight beside the one being worked on
#pragma unroll
    for (int i = 1; i < STAGES - 1; ++i) {
        if (i < n_tiles) load_tile(i, i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    constexpr int KS = DMAX / 16, ON = DMAX / 8;
    const int ks_n = head_dim / 16;
    uint32_t qa[KS][4];
    float o[ON][4];
#pragma unroll
    for (int i = 0; i < ON; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8

    for (int tile = 0; tile < n_tiles; ++tile) {
        const int buf = tile % STAGES;
        if (tile + STAGES - 1 < n_tiles) load_tile(tile + STAGES - 1, (tile + STAGES - 1) % STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
        __syncthreads();
        if (tile == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                if (ks < ks_n)
                    ldsm4(q_u + (lane & 15) * pitch + (ks * 16 + (lane >> 4) * 8) * 2, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
        }
        const uint32_t ku = kv_u + buf * 2 * TK * pitch, vu = ku + TK * pitch;
        const uint8_t* fl = flag_s + buf * TK;
        const int kw = warp * 16;                  // this warp's keys inside the tile
        if (k_begin + tile * TK + kw < k_end) {    // same for the whole warp
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                if (ks < ks_n) {
                    uint32_t b0, b1, b2, b3;
                    const int krow = kw + (lane & 7) + (lane >> 4) * 8;
                    ldsm4(ku + krow * pitch + (ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
                    mma16816(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                    mma16816(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                }
            }
            // keys past the range or without a page do not count
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const bool ok = fl[kw + j * 8 + 2 * t4 + e] != 0;
                    if (!ok) { s[j][e] = -INFINITY; s[j][2 + e] = -INFINITY; }
                    mx0 = fmaxf(mx0, s[j][e]);
                    mx1 = fmaxf(mx1, s[j][2 + e]);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ref0 = mn0 == -INFINITY ? 0.f : mn0 * scale_log2e, ref1 = mn1 == -INFINITY ? 0.f : mn1 * scale_log2e;
            const float al0 = m0 == -INFINITY ? 0.f : exp2f(m0 * scale_log2e - ref0);
            const float al1 = m1 == -INFINITY ? 0.f : exp2f(m1 * scale_log2e - ref1);
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t p[2][2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float e0 = exp2f(s[j][0] * scale_log2e - ref0), e1 = exp2f(s[j][1] * scale_log2e - ref0);
                const float e2 = exp2f(s[j][2] * scale_log2e - ref1), e3 = exp2f(s[j][3] * scale_log2e - ref1);
                sum0 += e0 + e1; sum1 += e2 + e3;
                p[j][0] = pack_bf16(e0, e1);
                p[j][1] = pack_bf16(e2, e3);
            }
            sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
            sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
            l0 = l0 * al0 + sum0; l1 = l1 * al1 + sum1;
            m0 = mn0; m1 = mn1;
#pragma unroll
            for (int i = 0; i < ON; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
            // O += P V over this warp's 16 keys
#pragma unroll
            for (int i = 0; i < ON / 2; ++i) {
                if (i * 16 < head_dim) {
                    uint32_t b0, b1, b2, b3;
                    const int vrow = kw + (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldsm4t(vu + vrow * pitch + (i * 16 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
                    mma16816(o[2 * i], p[0][0], p[0][1], p[1][0], p[1][1], b0, b1);
                    mma16816(o[2 * i + 1], p[0][0], p[0][1], p[1][0], p[1][1], b2, b3);
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before it is loaded again
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- merge the four warps, in warp order, and write the partial result ------------
    float* acc_s = reinterpret_cast<float*>(kv_s);          // [4][16][head_dim] (the ring is free now)
    __shared__ float m_s[4][16], l_s[4][16];
    if (t4 == 0) { m_s[warp][g] = m0; m_s[warp][g + 8] = m1; l_s[warp][g] = l0; l_s[warp][g + 8] = l1; }
#pragma unroll
    for (int i = 0; i < ON; ++i) {
        const int col = i * 8 + 2 * t4;
        if (col < head_dim) {
            float* a0 = acc_s + ((long)warp * 16 + g) * head_dim + col;
            float* a1 = acc_s + ((long)warp * 16 + g + 8) * head_dim + col;
            a0[0] = o[i][0]; a0[1] = o[i][1]; a1[0] = o[i][2]; a1[1] = o[i][3];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nq * head_dim; idx += NTHREADS) {
        const int h = idx / head_dim, e = idx - h * head_dim;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, m_s[w][h]);
        float ll = 0.f, a = 0.f;
        if (mm > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float wgt = m_s[w][h] == -INFINITY ? 0.f : exp2f((m_s[w][h] - mm) * scale_log2e);
                ll += l_s[w][h] * wgt;
                a += acc_s[((long)w * 16 + h) * head_dim + e] * wgt;
            }
        }
        const long slot = ((long)tkn * n_heads + (h0 + h)) * n_splits + split;
        part_acc[slot * head_dim + e] = a;
        // merge_kernel works with natural-log maxima of the scaled scores
        if (e == 0) { part_ml[slot * 2] = mm == -INFINITY ? -INFINITY : mm * scale; part_ml[slot * 2 + 1] = ll; }
    }
}

template <int DMAX>
int launch(dim3 grid, size_t smem, cudaStream_t s, const bf16* q, long ldq, const bf16* k, const bf16* v, const int* bt,
           int tw, int ps, const int* pos, const int* tseq, const int* sslot, float* pa, float* pm, int nh, int nkv, int d,
           int window, float scale, int split_len, int n_splits, int fresh)
{
    auto kern = decode_mma_kernel<DMAX>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    fx_launch_pdl(kern, grid, NTHREADS, smem, s, q, ldq, k, v, bt, tw, ps, pos, tseq, sslot, pa, pm, nh, nkv, d, window,
                  scale * 1.4426950408889634f, scale, split_len, n_splits, fresh);
    return fx_launch_status();
}

}  // namespace

// The first half of fx_decode_attention for bfloat16 (partials only; the caller runs the merge).
// Returns FX_ERR_SIZE for shapes it does not take; the caller then uses the CUDA-core kernel.
extern "C" int fx_decode_split_mma(const void* q, long ldq, const void* k_pages, const void* v_pages,
                                   const int* block_table, int table_width, int page_size, const int* positions,
                                   const int* token_seq, const int* seq_slot, float* part_acc, float* part_ml,
                                   int n_tokens, int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                   int split_len, int n_splits, int fresh_positions, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (head_dim % 16 || head_dim <= 0 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads) return FX_ERR_SIZE;
    if (ldq % 8 || (uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16) return FX_ERR_ALIGN;
    const int group = n_heads / n_kv_heads;
    const int chunks = (group + MAXQ - 1) / MAXQ;
    dim3 grid(n_kv_heads * chunks, n_tokens, n_splits);
    if (grid.y > 65535u || grid.z > 65535u) return FX_ERR_SIZE;
    const int pitch = head_dim * 2 + 16;
    size_t smem = (size_t)16 * pitch + (size_t)STAGES * 2 * TK * pitch + STAGES * TK;
    const size_t merge = (size_t)4 * 16 * head_dim * sizeof(float);
    if ((size_t)STAGES * 2 * TK * pitch < merge) smem += merge;   // never with these tile sizes; kept for safety
    cudaStream_t s = (cudaStream_t)stream;
    const bf16* Q = (const bf16*)q; const bf16* K = (const bf16*)k_pages; const bf16* V = (const bf16*)v_pages;
    if (head_dim <= 64)
        return launch<64>(grid, smem, s, Q, ldq, K, V, block_table, table_width, page_size, positions, token_seq, seq_slot,
                          part_acc, part_ml, n_heads, n_kv_heads, head_dim, window, scale, split_len, n_splits, fresh_positions);
    if (head_dim <= 128)
        return launch<128>(grid, smem, s, Q, ldq, K, V, block_table, table_width, page_size, positions, token_seq, seq_slot,
                           part_acc, part_ml, n_heads, n_kv_heads, head_dim, window, scale, split_len, n_splits, fresh_positions);
    return launch<256>(grid, smem, s, Q, ldq, K, V, block_table, table_width, page_size, positions, token_seq, seq_slot,
                       part_acc, part_ml, n_heads, n_kv_heads, head_dim, window, scale, split_len, n_splits, fresh_positions);
}
