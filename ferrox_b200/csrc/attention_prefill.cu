// Attention for prompt portions in bfloat16: tiles of 64 query tokens of one request
// against that request's cache pages, keys in blocks of 64, online softmax in 32 bits
// (flash attention).  Earlier steps' keys and the portion's own keys are read the
// same way from the pages; the mask is a function of absolute positions:
// query at p sees keys max(0, p - W + 1) .. p.
//
//   grid = (query tile, head); a tile = up to 64 consecutive tokens of one entry,
//   listed by the host in `tiles` = (first flat token, rows, entry, first position).
//   4 warps, 16 query rows each.  K and V blocks arrive in shared memory by cp.async
//   (two buffers), each key row found through the block table, so any page size
//   works; rows past the visible range are zero-filled.
//   S = Q K^T and O += P V run on the tensor cores (mma.sync.m16n8k16, bf16 in,
//   f32 out), P is rounded to bfloat16 for the second product, everything else
//   (scores, max, sum, rescaling, output) is 32-bit.
//
// mma.sync is used here because attention is a few per cent of a prompt's
// arithmetic; the matrix products, which are the rest, run on tcgen05 (gemm_tc.cu).
//
// Reference: causal prefill = query t over keys 0..=t
// (crates/ferrox-core/src/attention.rs:531-563), online softmax :146-175, window
// :484-524, pages :572-610, grouped heads :432-449.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int BQ = 64, BKEY = 32, NWARPS = 4, NTHREADS = NWARPS * 32;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
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

// DMAX: largest head_dim of this instantiation (head_dim itself is a run-time multiple of 16)
template <int DMAX>
__global__ void __launch_bounds__(NTHREADS) prefill_attention_kernel(
    const bf16* __restrict__ q, long ldq, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
    const int* __restrict__ block_table, int table_width, int page_size, const int* __restrict__ tiles,
    const int* __restrict__ seq_slot, bf16* __restrict__ out, long ldo, int n_heads, int n_kv_heads, int head_dim,
    int window, float scale_log2e)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const int pitch = head_dim * 2 + 16;                 // bytes per row: 16 bytes of padding spread the banks
    uint8_t* q_s = smem;                                  // [BQ][pitch]
    uint8_t* k_s = q_s + BQ * pitch;                      // [2][BKEY][pitch]
    uint8_t* v_s = k_s + 2 * BKEY * pitch;                // [2][BKEY][pitch]
    const uint32_t q_u = (uint32_t)__cvta_generic_to_shared(q_s);
    const uint32_t k_u = (uint32_t)__cvta_generic_to_shared(k_s);
    const uint32_t v_u = (uint32_t)__cvta_generic_to_shared(v_s);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    // heavy tiles (late in their request) first
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int tok0 = tiles[tile * 4], rows = tiles[tile * 4 + 1], entry = tiles[tile * 4 + 2], pos0 = tiles[tile * 4 + 3];
    const int head = blockIdx.y;
    const int kvh = head / (n_heads / n_kv_heads);
    const int* table = block_table + (long)seq_slot[entry] * table_width;
    const int chunks = head_dim / 8;                      // 16-byte chunks per row
    const long head_stride = (long)page_size * head_dim;

    const int last_pos = pos0 + rows - 1;
    const int key_lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;   // first key any row may see
    const int kb_begin = (key_lo / BKEY) * BKEY;
    const int n_blocks = (last_pos - kb_begin) / BKEY + 1;

    // ---- Q tile -> shared memory (rows past the tile's end are zero) -------------
    for (int c = threadIdx.x; c < BQ * chunks; c += NTHREADS) {
        const int r = c / chunks, ch = c - r * chunks;
        const bf16* src = q + (long)(tok0 + min(r, rows - 1)) * ldq + (long)head * head_dim + ch * 8;
        cp_async16(q_u + r * pitch + ch * 16, src, r < rows ? 16 : 0);
    }
    // A thread always copies the same 16-byte column of several rows: (row, column) is found once.  When a
    // block of keys lies inside one page (page_size a multiple of 64), one table lookup serves the block.
    const bool lanes_fit = chunks <= NTHREADS && NTHREADS % chunks == 0;
    const int my_ch = lanes_fit ? threadIdx.x % chunks : 0;
    const int my_r0 = lanes_fit ? threadIdx.x / chunks : 0;
    const int rows_per_pass = lanes_fit ? NTHREADS / chunks : 1;
    const bool block_in_page = page_size % BKEY == 0;
    auto load_kv = [&](int blk, int buf) {
        const int kb = kb_begin + blk * BKEY;
        if (lanes_fit) {
            int page_blk = -1;
            if (block_in_page) page_blk = table[kb / page_size];
            const int off_blk = kb % page_size;
            for (int r = my_r0; r < BKEY; r += rows_per_pass) {
                const int key = kb + r;
                int page = -1, off = 0;
                if (key <= last_pos && key >= key_lo) {
                    if (block_in_page) { page = page_blk; off = off_blk + r; }
                    else { page = table[key / page_size]; off = key % page_size; }
                }
                const bool ok = page >= 0;
                const long base = ok ? ((long)page * n_kv_heads + kvh) * head_stride + (long)off * head_dim + my_ch * 8 : 0;
                const uint32_t dst = (buf * BKEY + r) * pitch + my_ch * 16;
                cp_async16(k_u + dst, k_pages + base, ok ? 16 : 0);
                cp_async16(v_u + dst, v_pages + base, ok ? 16 : 0);
            }
            return;
        }
        for (int c = threadIdx.x; c < BKEY * chunks; c += NTHREADS) {
            const int r = c / chunks, ch = c - r * chunks;
            const int key = kb + r;
            int page = -1;
            if (key <= last_pos && key >= key_lo) page = table[key / page_size];
            const bool ok = page >= 0;
            const long base = ok ? ((long)page * n_kv_heads + kvh) * head_stride + (long)(key % page_size) * head_dim + ch * 8 : 0;
            const uint32_t off = (buf * BKEY + r) * pitch + ch * 16;
            cp_async16(k_u + off, k_pages + base, ok ? 16 : 0);
            cp_async16(v_u + off, v_pages + base, ok ? 16 : 0);
        }
    };
    load_kv(0, 0);
    cp_commit();

    constexpr int KS = DMAX / 16;     // k-steps over the head dimension
    constexpr int ON = DMAX / 8;      // n-tiles of the output
    const int ks_n = head_dim / 16;
    float o[ON][4];
#pragma unroll
    for (int i = 0; i < ON; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8 of this warp's 16
    const int qrow0 = warp * 16;
    const int p_row0 = pos0 + qrow0 + g, p_row1 = p_row0 + 8;    // absolute positions of this thread's two rows

    for (int blk = 0; blk < n_blocks; ++blk) {
        const int buf = blk & 1;
        if (blk + 1 < n_blocks) load_kv(blk + 1, buf ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();

        const int kb = kb_begin + blk * BKEY;
        // does this warp see anything in this block?  (its rows qrow0 .. qrow0+15)
        const int w_last = pos0 + qrow0 + 15, w_first = pos0 + qrow0;
        const int w_lo = (window > 0 && w_first - window + 1 > 0) ? w_first - window + 1 : 0;
        const bool warp_active = qrow0 < rows && kb <= w_last && kb + BKEY - 1 >= w_lo;
        if (warp_active) {
            // ---- S = Q K^T : 16 x 64 per warp ---------------------------------------
            float s[BKEY / 8][4];
#pragma unroll
            for (int j = 0; j < BKEY / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                if (ks < ks_n) {
                    uint32_t a0, a1, a2, a3;
                    ldsm4(q_u + (qrow0 + (lane & 15)) * pitch + (ks * 16 + (lane >> 4) * 8) * 2, a0, a1, a2, a3);
#pragma unroll
                    for (int j = 0; j < BKEY / 16; ++j) {
                        uint32_t b0, b1, b2, b3;
                        const int krow = j * 16 + (lane & 7) + (lane >> 4) * 8;
                        ldsm4(k_u + (buf * BKEY + krow) * pitch + (ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
                        mma16816(s[2 * j], a0, a1, a2, a3, b0, b1);
                        mma16816(s[2 * j + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
            // ---- mask by absolute position, online softmax ---------------------------
            const int lo0 = window > 0 ? p_row0 - window + 1 : 0, lo1 = window > 0 ? p_row1 - window + 1 : 0;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < BKEY / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = kb + j * 8 + 2 * t4 + e;
                    if (key > p_row0 || key < lo0) s[j][e] = -INFINITY;
                    if (key > p_row1 || key < lo1) s[j][2 + e] = -INFINITY;
                    mx0 = fmaxf(mx0, s[j][e]);
                    mx1 = fmaxf(mx1, s[j][2 + e]);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            // a row that sees no key yet keeps m = -inf: use 0 as the reference so that exp2 stays finite
            const float ref0 = mn0 == -INFINITY ? 0.f : mn0 * scale_log2e, ref1 = mn1 == -INFINITY ? 0.f : mn1 * scale_log2e;
            const float al0 = m0 == -INFINITY ? 0.f : exp2f(m0 * scale_log2e - ref0);
            const float al1 = m1 == -INFINITY ? 0.f : exp2f(m1 * scale_log2e - ref1);
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t p[BKEY / 8][2];
#pragma unroll
            for (int j = 0; j < BKEY / 8; ++j) {
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
            // ---- O += P V ------------------------------------------------------------
#pragma unroll
            for (int kk = 0; kk < BKEY / 16; ++kk) {
                const uint32_t a0 = p[2 * kk][0], a1 = p[2 * kk][1], a2 = p[2 * kk + 1][0], a3 = p[2 * kk + 1][1];
#pragma unroll
                for (int i = 0; i < ON / 2; ++i) {
                    if (i * 16 < head_dim) {
                        uint32_t b0, b1, b2, b3;
                        const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                        ldsm4t(v_u + (buf * BKEY + vrow) * pitch + (i * 16 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
                        mma16816(o[2 * i], a0, a1, a2, a3, b0, b1);
                        mma16816(o[2 * i + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before it is loaded again
    }
    cp_wait<0>();

    // ---- normalise and store ---------------------------------------------------------
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int r0 = qrow0 + g, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < ON; ++i) {
        const int col = i * 8 + 2 * t4;
        if (col < head_dim) {
            if (r0 < rows)
                *reinterpret_cast<uint32_t*>(out + (long)(tok0 + r0) * ldo + (long)head * head_dim + col) =
                    pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
            if (r1 < rows)
                *reinterpret_cast<uint32_t*>(out + (long)(tok0 + r1) * ldo + (long)head * head_dim + col) =
                    pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
        }
    }
}

template <int DMAX>
int launch(dim3 grid, size_t smem, cudaStream_t s, const bf16* q, long ldq, const bf16* k, const bf16* v, const int* bt,
           int tw, int ps, const int* tiles, const int* seq_slot, bf16* out, long ldo, int nh, int nkv, int d, int window,
           float scale_log2e)
{
    auto kern = prefill_attention_kernel<DMAX>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kern<<<grid, NTHREADS, smem, s>>>(q, ldq, k, v, bt, tw, ps, tiles, seq_slot, out, ldo, nh, nkv, d, window, scale_log2e);
    return fx_launch_status();
}

}  // namespace

// tiles: int32 [n_tiles, 4] = (first flat token, rows <= 64, entry index, absolute position of the first row).
extern "C" int fx_prefill_attention(const void* q, long ldq, const void* k_pages, const void* v_pages,
                                    const int* block_table, int table_width, int page_size, const int* tiles,
                                    int n_tiles, const int* seq_slot, void* out, long ldo, int n_heads, int n_kv_heads,
                                    int head_dim, int window, float scale, void* stream)
{
    if (n_tiles <= 0) return FX_OK;
    if (head_dim % 16 || head_dim <= 0 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads) return FX_ERR_SIZE;
    if (ldq % 8 || ldo % 2 || (uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)out % 4)
        return FX_ERR_ALIGN;
    if (n_heads > 65535) return FX_ERR_SIZE;
    const size_t smem = (size_t)(BQ + 4 * BKEY) * (head_dim * 2 + 16);
    dim3 grid(n_tiles, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
    const float sl = scale * 1.4426950408889634f;
    const bf16* Q = (const bf16*)q; const bf16* K = (const bf16*)k_pages; const bf16* V = (const bf16*)v_pages;
    if (head_dim <= 64)
        return launch<64>(grid, smem, s, Q, ldq, K, V, block_table, table_width, page_size, tiles, seq_slot, (bf16*)out,
                          ldo, n_heads, n_kv_heads, head_dim, window, sl);
    if (head_dim <= 128)
        return launch<128>(grid, smem, s, Q, ldq, K, V, block_table, table_width, page_size, tiles, seq_slot, (bf16*)out,
                           ldo, n_heads, n_kv_heads, head_dim, window, sl);
    return launch<256>(grid, smem, s, Q, ldq, K, V, block_table, table_width, page_size, tiles, seq_slot, (bf16*)out, ldo,
                       n_heads, n_kv_heads, head_dim, window, sl);
}
