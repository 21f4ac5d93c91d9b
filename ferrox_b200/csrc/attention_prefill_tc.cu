// Attention for prompt portions on the 5th-generation tensor cores (bfloat16, head_dim 64 or 128,
// pages of 64 positions or a multiple).
//
// One CTA takes a tile of 128 query tokens of one request and one head, and walks that request's keys in
// blocks of 128 positions (earlier steps' keys and the portion's own alike, found through the block table):
//
//   S = Q K^T        tcgen05.mma 128 x 128 x head_dim, Q and K tiles in shared memory (TMA, 128-byte swizzle),
//                    S in tensor memory (32-bit)
//   P = exp2(...)    each of the 128 softmax threads owns one query row: tcgen05.ld of its row of S, mask by
//                    absolute position (query p sees keys max(0, p - W + 1) .. p), running max and sum in
//                    32 bits, P rounded to bfloat16 and stored, swizzled, as the A operand of the next product
//   O_blk = P V      tcgen05.mma 128 x head_dim x 128 with V as an N-major B operand, exactly as TMA lays the
//                    [key][head_dim] rows down; O_blk in tensor memory
//   O = O * alpha + O_blk   in the softmax threads' registers (a row of O per thread), no read-modify-write
//                    of tensor memory
//
// Warp 0 issues the TMA loads (K and V blocks double-buffered), warp 1 issues the tensor-core instructions
// and owns the tensor-memory allocation, warps 2-5 are the softmax threads.  The product S of block i+1 is
// issued as soon as P of block i is written, so it overlaps the accumulation of O.  Every wait is bounded
// (status code 3 on time-out, then the roles leave, tensor memory is freed and the kernel returns).
// Keys that are masked for every row are still multiplied (with weight 0); the half of a block that lies
// beyond the request's pages is read from page 0, which always holds finite values.
//
// Reference: crates/ferrox-core/src/attention.rs:531-563 (query t over keys 0..=t), :146-175 (online
// softmax), :484-524 (window), :572-610 (pages), :432-449 (grouped heads).  The mma.sync kernel of
// attention_prefill.cu remains for other head sizes and page sizes.
#include "tc_common.cuh"
#include "api.h"

namespace {

using namespace fxtc;

constexpr int BQ = 128, BKEY = 128, NTHREADS = 192;

__device__ __forceinline__ float fast_exp2(float x) {   // 2^x, approximate; -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct AttnArgs {
    const int* block_table; int table_width; int page_size;
    const int* tiles; const int* seq_slot;
    bf16* out; long ldo;
    int n_heads, n_kv_heads, window;
    float scale_log2e;
    int* status;
};

template <int D>
struct Smem {
    static constexpr int HALVES = D / 64;                  // 64-element (128-byte) slices of the head dimension
    static constexpr int SUB = 128 * 128;                  // bytes of a [128 rows x 128 bytes] sub-tile
    static constexpr int Q_BYTES = HALVES * SUB, KV_BYTES = HALVES * SUB, P_BYTES = 2 * SUB;
    static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = K_OFF + 2 * KV_BYTES, P_OFF = V_OFF + 2 * KV_BYTES;
    static constexpr int BAR_OFF = P_OFF + P_BYTES;
    static constexpr int TOTAL = BAR_OFF + 128 + 1024;     // barriers, alignment slack
};

template <int D>
__global__ void __launch_bounds__(NTHREADS, 1) prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                           const __grid_constant__ CUtensorMap map_k,
                                                                           const __grid_constant__ CUtensorMap map_v,
                                                                           AttnArgs a)
{
    using L = Smem<D>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag_s;
    __shared__ uint32_t tmem_base_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // heavy tiles (late in their request) first
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int tok0 = a.tiles[tile * 4], rows = a.tiles[tile * 4 + 1], entry = a.tiles[tile * 4 + 2], pos0 = a.tiles[tile * 4 + 3];
    const int head = blockIdx.y;
    const int kvh = head / (a.n_heads / a.n_kv_heads);
    const int last_pos = pos0 + rows - 1;
    const int key_lo = (a.window > 0 && pos0 - a.window + 1 > 0) ? pos0 - a.window + 1 : 0;
    const int kb_begin = (key_lo / BKEY) * BKEY;
    const int n_blocks = (last_pos - kb_begin) / BKEY + 1;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar0 = base + L::BAR_OFF;
    const uint32_t q_full = bar0, s_full = bar0 + 8, p_full = bar0 + 16, o_full = bar0 + 24;
    auto k_full = [&](int b) { return bar0 + 32 + 8u * b; };
    auto v_full = [&](int b) { return bar0 + 48 + 8u * b; };
    auto kv_empty = [&](int b) { return bar0 + 64 + 8u * b; };
    volatile int* abort_flag = &abort_flag_s;

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        mbar_init(q_full, 1); mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(o_full, 1);
        for (int b = 0; b < 2; ++b) { mbar_init(k_full(b), 1); mbar_init(v_full(b), 1); mbar_init(kv_empty(b), 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {   // tensor memory: S (128 columns) and O_blk (D columns)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

    if (warp == 0) {
        // ---------------- producer: Q once, then K and V blocks ----------------
        if (lane == 0) {
            mbar_expect_tx(q_full, L::Q_BYTES);
            for (int h = 0; h < L::HALVES; ++h)
                tma_load_2d(base + L::Q_OFF + h * L::SUB, &map_q, head * D + h * 64, tok0, q_full);
            const int* table = a.block_table + (long)a.seq_slot[entry] * a.table_width;
            int issued = 0;
            for (int i = 0; i < n_blocks; ++i) {
                const int b = i & 1;
                if (!mbar_wait(kv_empty(b), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag)) break;
                const int kb = kb_begin + i * BKEY;
                int page[2], off[2];
                for (int hk = 0; hk < 2; ++hk) {   // the two runs of 64 keys of the block
                    const int key = kb + hk * 64;
                    int p = key <= last_pos ? table[key / a.page_size] : -1;
                    page[hk] = p >= 0 ? p : 0;      // beyond the request's pages: any finite data will do (masked)
                    off[hk] = p >= 0 ? key % a.page_size : 0;
                }
                mbar_expect_tx(k_full(b), L::KV_BYTES);
                for (int h = 0; h < L::HALVES; ++h)
                    for (int hk = 0; hk < 2; ++hk)
                        tma_load_4d(base + L::K_OFF + b * L::KV_BYTES + h * L::SUB + hk * 8192, &map_k, h * 64, off[hk], kvh,
                                    page[hk], k_full(b));
                mbar_expect_tx(v_full(b), L::KV_BYTES);
                for (int h = 0; h < L::HALVES; ++h)
                    for (int hk = 0; hk < 2; ++hk)
                        tma_load_4d(base + L::V_OFF + b * L::KV_BYTES + h * L::SUB + hk * 8192, &map_v, h * 64, off[hk], kvh,
                                    page[hk], v_full(b));
                issued = i + 1;
            }
            if (*abort_flag) {   // loads already issued must land before the shared memory is released
                for (int i = max(0, issued - 2); i < issued; ++i)
                    for (uint32_t w = 0; w < WAIT_LIMIT; ++w)
                        if (mbar_try_wait(k_full(i & 1), (uint32_t)((i >> 1) & 1)) && mbar_try_wait(v_full(i & 1), (uint32_t)((i >> 1) & 1))) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issue ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc_ex(BQ, BKEY, 0);   // S: B = K tile, K-major
            constexpr uint32_t idesc_o = instr_desc_ex(BQ, D, 1);      // O: B = V tile, N-major
            auto issue_s = [&](int i) {
                const int b = i & 1;
                if (!mbar_wait(k_full(b), (uint32_t)((i >> 1) & 1), abort_flag)) return false;
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < L::HALVES; ++h) {
                    const uint64_t dq = smem_desc(base + L::Q_OFF + h * L::SUB);
                    const uint64_t dk = smem_desc(base + L::K_OFF + b * L::KV_BYTES + h * L::SUB);
#pragma unroll
                    for (int k = 0; k < 4; ++k) tc_mma(tmem_s, dq + 2u * k, dk + 2u * k, idesc_s, (h | k) != 0);
                }
                tc_commit(s_full);
                return true;
            };
            bool ok = mbar_wait(q_full, 0, abort_flag);
            if (ok) ok = issue_s(0);
            for (int i = 0; i < n_blocks && ok; ++i) {
                const int b = i & 1;
                ok = mbar_wait(p_full, (uint32_t)(i & 1), abort_flag) && mbar_wait(v_full(b), (uint32_t)((i >> 1) & 1), abort_flag);
                if (!ok) break;
                tc_fence_after();
                // O_blk = P V: 8 steps of 16 keys.  A = P, K-major (keys contiguous), two sub-tiles of 64 keys.
                // B = V, N-major: a step covers two 8-key groups (1024 bytes each, stride operand); the two
                // 64-element slices of the head dimension lie SUB bytes apart (leading operand).
#pragma unroll
                for (int ks = 0; ks < BKEY / 16; ++ks) {
                    const uint64_t dp = smem_desc(base + L::P_OFF + (ks >> 2) * L::SUB) + 2u * (ks & 3);
                    const uint64_t dv = smem_desc_lbo_sbo(base + L::V_OFF + b * L::KV_BYTES + ks * 2048, L::SUB, 1024);
                    tc_mma(tmem_o, dp, dv, idesc_o, ks != 0);
                }
                tc_commit(o_full);
                tc_commit(kv_empty(b));
                if (i + 1 < n_blocks) ok = issue_s(i + 1);
            }
        }
    } else {
        // ---------------- softmax and accumulation: one query row per thread ----------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const int p_r = pos0 + r;                                   // absolute position of this row
        const int lo_r = a.window > 0 ? p_r - a.window + 1 : 0;
        const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
        float o[D];
#pragma unroll
        for (int j = 0; j < D; ++j) o[j] = 0.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_blocks; ++i) {
            ok = __all_sync(0xffffffffu, mbar_wait(s_full, (uint32_t)(i & 1), abort_flag));
            if (!ok) break;
            tc_fence_after();
            const int kb = kb_begin + i * BKEY;
            // every key of the block visible to every row of the tile: no masking (most blocks)
            const bool interior = kb + BKEY - 1 <= pos0 && (a.window <= 0 || kb >= pos0 + BQ - 1 - a.window + 1);
            // pass 1: the row's maximum
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < BKEY / 32; ++c) {
                uint32_t s[32];
                tc_ld32(tmem_s + lane_off + c * 32, s);
                tc_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int key = kb + c * 32 + j;
                    const bool vis = interior || (key <= p_r && key >= lo_r);
                    if (vis) mx = fmaxf(mx, __uint_as_float(s[j]));
                }
            }
            const float mn = fmaxf(m, mx);
            const float ref = mn == -INFINITY ? 0.f : mn * a.scale_log2e;
            const float alpha = m == -INFINITY ? 0.f : fast_exp2(m * a.scale_log2e - ref);
            // pass 2: P = exp2(S * scale - ref), rounded to bfloat16, into shared memory (128-byte swizzle)
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < BKEY / 32; ++c) {
                uint32_t s[32];
                tc_ld32(tmem_s + lane_off + c * 32, s);
                tc_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int key = kb + c * 32 + j;
                    const bool v0 = interior || (key <= p_r && key >= lo_r);
                    const bool v1 = interior || (key + 1 <= p_r && key + 1 >= lo_r);
                    const float e0 = v0 ? fast_exp2(__uint_as_float(s[j]) * a.scale_log2e - ref) : 0.f;
                    const float e1 = v1 ? fast_exp2(__uint_as_float(s[j + 1]) * a.scale_log2e - ref) : 0.f;
                    sum += e0 + e1;
                    __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
                    pk[j >> 1] = *reinterpret_cast<uint32_t*>(&pr);
                }
                // keys c*32 .. c*32+31 of row r: sub-tile c/2, 16-byte chunks (c%2)*4 .. +3, swizzled by the row
                uint8_t* prow = base_ptr + L::P_OFF + (c >> 1) * L::SUB + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int ch = ((c & 1) * 4 + q4) ^ (r & 7);
                    *reinterpret_cast<uint4*>(prow + ch * 16) = make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
                }
            }
            l = l * alpha + sum;
            m = mn;
            // P is written with ordinary stores and read by the tensor cores: make it visible to that proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            // O = O * alpha + O_blk
            ok = __all_sync(0xffffffffu, mbar_wait(o_full, (uint32_t)(i & 1), abort_flag));
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t ob[32];
                tc_ld32(tmem_o + lane_off + c * 32, ob);
                tc_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) o[c * 32 + j] = o[c * 32 + j] * alpha + __uint_as_float(ob[j]);
            }
        }
        if (ok && r < rows) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = a.out + (long)(tok0 + r) * a.ldo + (long)head * D;
#pragma unroll
            for (int j = 0; j < D; j += 8) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(o[j] * inv, o[j + 1] * inv), p1 = __floats2bfloat162_rn(o[j + 2] * inv, o[j + 3] * inv);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(o[j + 4] * inv, o[j + 5] * inv), p3 = __floats2bfloat162_rn(o[j + 6] * inv, o[j + 7] * inv);
                v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j) = v;
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag_s && a.status) atomicExch(a.status, STATUS_TC_TIMEOUT);
}

bool encode(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a, dim3 grid, cudaStream_t s)
{
    auto kern = prefill_attention_tc_kernel<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    kern<<<grid, NTHREADS, Smem<D>::TOTAL, s>>>(mq, mk, mv, a);
    return fx_launch_status();
}

}  // namespace

// tiles: int32 [n_tiles, 4] = (first flat token, rows <= 128, entry index, absolute position of the first row).
// q is the fused [tokens, ldq] buffer whose rows start with the query heads; n_tokens its number of rows.
// Refuses (FX_ERR_SIZE / FX_ERR_ALIGN) what it does not take; the caller then uses the mma.sync kernel.
extern "C" int fx_prefill_attention_tc(const void* q, long ldq, int n_tokens, const void* k_pages, const void* v_pages,
                                       int n_pages, const int* block_table, int table_width, int page_size,
                                       const int* tiles, int n_tiles, const int* seq_slot, void* out, long ldo,
                                       int n_heads, int n_kv_heads, int head_dim, int window, float scale, int* status,
                                       void* stream)
{
    if (n_tiles <= 0) return FX_OK;
    if ((head_dim != 64 && head_dim != 128) || page_size < 64 || page_size % 64 || n_kv_heads <= 0 || n_heads % n_kv_heads)
        return FX_ERR_SIZE;
    if (ldq % 8 || ldo % 8 || (uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)out % 16)
        return FX_ERR_ALIGN;
    if (n_heads > 65535) return FX_ERR_SIZE;
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[2] = {(cuuint64_t)n_heads * head_dim, (cuuint64_t)n_tokens};
        cuuint64_t strides[1] = {(cuuint64_t)ldq * 2};
        cuuint32_t box[2] = {64, 128};
        if (!encode(&mq, q, 2, dims, strides, box)) return FX_ERR_SIZE;
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads, (cuuint64_t)n_pages};
        cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)page_size * head_dim * 2,
                                 (cuuint64_t)n_kv_heads * page_size * head_dim * 2};
        cuuint32_t box[4] = {64, 64, 1, 1};
        if (!encode(&mk, k_pages, 4, dims, strides, box) || !encode(&mv, v_pages, 4, dims, strides, box)) return FX_ERR_SIZE;
    }
    AttnArgs a;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size;
    a.tiles = tiles; a.seq_slot = seq_slot; a.out = (bf16*)out; a.ldo = ldo;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.window = window;
    a.scale_log2e = scale * 1.4426950408889634f; a.status = status;
    dim3 grid(n_tiles, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
    return head_dim == 64 ? launch<64>(mq, mk, mv, a, grid, s) : launch<128>(mq, mk, mv, a, grid, s);
}
