// Attention for prompt portions on the 5th-generation tensor cores (bfloat16, head_dim 64 or 128,
// pages of 64 positions or a multiple).
//
// One CTA takes up to 256 query tokens of one request and one head, as two sub-tiles of 128 rows, and
// walks that request's keys in blocks of 128 positions (earlier steps' keys and the portion's own alike,
// found through the block table).  For each sub-tile t and key block j:
//
//   S_t = Q_t K_j^T    tcgen05.mma 128 x 128 x head_dim; Q and K tiles in shared memory (TMA, 128-byte
//                      swizzle), S_t in tensor memory (32-bit)
//   P_t = exp2(...)    each of the sub-tile's 128 softmax threads owns one query row: tcgen05.ld of its
//                      row of S, mask by absolute position (query p sees keys max(0, p - W + 1) .. p),
//                      running max and sum in 32 bits; P rounded to bfloat16 and written back over the
//                      first columns of S_t (tcgen05.st), where the next product reads it as its A operand
//   O_t += P_t V_j     tcgen05.mma 128 x head_dim x 128, A from tensor memory, V as an N-major B operand,
//                      exactly as TMA lays the [key][head_dim] rows down; O_t stays in tensor memory
//
// The running maximum of a row is only raised when it grows by more than 2^8 (the weights then stay
// below 2^8 and the final division by the row sum makes the result the same); when it is raised, the
// row's thread scales its row of O_t in tensor memory.  This takes the accumulator out of the softmax
// threads' registers and off their critical path.
//
// Warp 0 issues the TMA loads (K and V blocks double-buffered), warp 1 issues the tensor-core
// instructions and owns the tensor-memory allocation (512 columns: S_0, S_1, O_0, O_1), warps 2-5 are
// sub-tile 0's softmax threads and warps 6-9 sub-tile 1's.  The products are issued in the order
// PV_0(j), S_0(j+1), PV_1(j), S_1(j+1): while one sub-tile's threads work on their block the tensor
// cores work for the other.  Every wait is bounded (status code 3 on time-out, then the roles leave,
// tensor memory is freed and the kernel returns).  Keys that are masked for every row are still
// multiplied (with weight 0); the half of a block that lies beyond the request's pages is read from
// page 0, which always holds finite values.
//
// A work item is a tile of queries, a head and a run of key blocks [kb_begin, kb_end).  The host cuts the
// key blocks of long tiles into runs (the last 256 queries of a long prompt see many times the keys the
// first see, and a portion behind a long cached prefix is a single tile with all of them), so that the
// items are of similar length and there are enough of them for every SM; the heavy ones come first in the
// table.  An item that holds all of its tile's key blocks writes the tile's output.  Any other writes what
// it has (the unnormalised sums in 32 bits, and each row's reference maximum and sum of weights) into
// scratch memory, and a second kernel (prefill_merge_kernel) adds a tile's runs up in their order.
//
// Reference: crates/ferrox-core/src/attention.rs:531-563 (query t over keys 0..=t), :146-175 (online
// softmax), :484-524 (window), :572-610 (pages), :432-449 (grouped heads).  The mma.sync kernel of
// attention_prefill.cu remains for other head sizes and page sizes.
#include "tc_common.cuh"
#include "api.h"

namespace {

using namespace fxtc;

constexpr int BQ = 128, BKEY = 128, NTHREADS = 320, TMEM_COLS = 512;
constexpr float RAISE_MAX_BY = 8.f;   // in powers of two

__device__ __forceinline__ float fast_exp2(float x) {   // 2^x, approximate; -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int ITEM_INTS = 8;   // a work item: first flat token, rows, entry, first position, kb_begin, kb_end, part, -

struct AttnArgs {
    const int* block_table; int table_width; int page_size;
    const int* tiles; const int* seq_slot;
    bf16* out; long ldo;
    float* part_o; float* part_ml;   // partial results of items that hold a run of their tile's key blocks only
    int n_heads, n_kv_heads, window;
    float scale_log2e;
    int* status;
};

template <int D>
struct Smem {
    static constexpr int HALVES = D / 64;                  // 64-element (128-byte) slices of the head dimension
    static constexpr int SUB = 128 * 128;                  // bytes of a [128 rows x 128 bytes] piece
    static constexpr int Q_BYTES = HALVES * SUB, KV_BYTES = HALVES * SUB;
    static constexpr int Q_OFF = 0, K_OFF = 2 * Q_BYTES, V_OFF = K_OFF + 2 * KV_BYTES;
    static constexpr int BAR_OFF = V_OFF + 2 * KV_BYTES;
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

    // The host lists heavy items first, and blocks are handed out with blockIdx.x running fastest: every head's
    // heaviest item, then every head's next one, so that the light items fill the gaps at the end.
    const int* item = a.tiles + (long)blockIdx.y * ITEM_INTS;
    const int tok0 = item[0], rows = item[1], entry = item[2], pos0 = item[3];
    const int kb_begin = item[4], kb_end = item[5], part = item[6];
    const int head = blockIdx.x;
    const int kvh = head / (a.n_heads / a.n_kv_heads);
    const int last_pos = pos0 + rows - 1;
    // sub-tile t: rows_of(t) rows from position pos0 + 128 t; it needs the key blocks blk_lo(t) .. blk_hi(t)
    const int nt = rows > BQ ? 2 : 1;
    auto rows_of = [&](int t) { return min(BQ, rows - t * BQ); };
    auto blk_lo = [&](int t) {
        const int p = pos0 + t * BQ;
        return (a.window > 0 && p - a.window + 1 > 0 ? p - a.window + 1 : 0) / BKEY;
    };
    auto blk_hi = [&](int t) { return (pos0 + t * BQ + rows_of(t) - 1) / BKEY; };
    // the key blocks of sub-tile t inside this item's run: lo_t[t] .. hi_t[t] (none if lo > hi)
    const int lo0 = max(blk_lo(0), kb_begin), hi0 = min(blk_hi(0), kb_end - 1);
    const int lo1 = nt > 1 ? max(blk_lo(1), kb_begin) : 1, hi1 = nt > 1 ? min(blk_hi(1), kb_end - 1) : 0;
    auto lo_of = [&](int t) { return t ? lo1 : lo0; };
    auto hi_of = [&](int t) { return t ? hi1 : hi0; };
    const bool act0 = lo0 <= hi0, act1 = lo1 <= hi1;
    const int first_blk = act0 && act1 ? min(lo0, lo1) : act0 ? lo0 : lo1;
    const int last_blk = act0 && act1 ? max(hi0, hi1) : act0 ? hi0 : hi1;
    auto active = [&](int t, int j) { return t < 2 && j >= lo_of(t) && j <= hi_of(t); };

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = base + L::BAR_OFF;
    const uint32_t q_full = bar0;
    auto s_full = [&](int t) { return bar0 + 8 + 8u * t; };
    auto p_full = [&](int t) { return bar0 + 24 + 8u * t; };
    auto o_done = [&](int t) { return bar0 + 40 + 8u * t; };
    auto k_full = [&](int b) { return bar0 + 56 + 8u * b; };
    auto v_full = [&](int b) { return bar0 + 72 + 8u * b; };
    auto kv_empty = [&](int b) { return bar0 + 88 + 8u * b; };
    volatile int* abort_flag = &abort_flag_s;

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full(b), 1); mbar_init(p_full(b), 4); mbar_init(o_done(b), 1);
            mbar_init(k_full(b), 1); mbar_init(v_full(b), 1); mbar_init(kv_empty(b), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    fx_pdl_wait();   // set up while the kernel before this one drains; its results (q, the pages) from here on
    auto tmem_s = [&](int t) { return tmem_base + 128u * t; };        // S_t, and P_t over its first 64 columns
    auto tmem_o = [&](int t) { return tmem_base + 256u + 128u * t; };

    if (warp == 0) {
        // ---------------- producer: Q once, then K and V blocks ----------------
        if (lane == 0) {
            mbar_expect_tx(q_full, nt * L::Q_BYTES);
            for (int t = 0; t < nt; ++t)
                for (int h = 0; h < L::HALVES; ++h)
                    tma_load_2d(base + L::Q_OFF + t * L::Q_BYTES + h * L::SUB, &map_q, head * D + h * 64, tok0 + t * BQ, q_full);
            const int* table = a.block_table + (long)a.seq_slot[entry] * a.table_width;
            int issued = 0;
            for (int j = first_blk; j <= last_blk; ++j) {
                const int i = j - first_blk, b = i & 1;
                if (!mbar_wait(kv_empty(b), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag)) break;
                int page[2], off[2];
                for (int hk = 0; hk < 2; ++hk) {   // the two runs of 64 keys of the block
                    const int key = j * BKEY + hk * 64;
                    const int p = key <= last_pos ? table[key / a.page_size] : -1;
                    page[hk] = p >= 0 ? p : 0;      // no page (beyond the request, or before its window): masked anyway
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
            int k_ready = first_blk - 1;   // the last block whose K is known to have landed
            bool ok = mbar_wait(q_full, 0, abort_flag);
            auto issue_s = [&](int t, int j) {
                const int i = j - first_blk, b = i & 1;
                if (k_ready < j) {
                    if (!mbar_wait(k_full(b), (uint32_t)((i >> 1) & 1), abort_flag)) return false;
                    k_ready = j;
                    tc_fence_after();
                }
#pragma unroll
                for (int h = 0; h < L::HALVES; ++h) {
                    const uint64_t dq = smem_desc(base + L::Q_OFF + t * L::Q_BYTES + h * L::SUB);
                    const uint64_t dk = smem_desc(base + L::K_OFF + b * L::KV_BYTES + h * L::SUB);
#pragma unroll
                    for (int k = 0; k < 4; ++k) tc_mma(tmem_s(t), dq + 2u * k, dk + 2u * k, idesc_s, (h | k) != 0);
                }
                tc_commit(s_full(t));
                return true;
            };
            for (int t = 0; t < nt && ok; ++t)
                if (active(t, first_blk)) ok = issue_s(t, first_blk);
            int n_p[2] = {0, 0};   // blocks of each sub-tile whose P has been taken
            for (int j = first_blk; j <= last_blk && ok; ++j) {
                const int i = j - first_blk, b = i & 1;
                bool v_ready = false;
                for (int t = 0; t < nt && ok; ++t) {
                    if (active(t, j)) {
                        ok = mbar_wait(p_full(t), (uint32_t)(n_p[t] & 1), abort_flag);
                        if (ok && !v_ready) { ok = mbar_wait(v_full(b), (uint32_t)((i >> 1) & 1), abort_flag); v_ready = true; }
                        if (!ok) break;
                        tc_fence_after();
                        // O_t += P V: 8 steps of 16 keys.  A = P from tensor memory, 8 columns a step.  B = V,
                        // N-major: a step covers two 8-key groups (1024 bytes each, the stride operand); the two
                        // 64-element slices of the head dimension lie SUB bytes apart (the leading operand).
#pragma unroll
                        for (int ks = 0; ks < BKEY / 16; ++ks) {
                            const uint64_t dv = smem_desc_lbo_sbo(base + L::V_OFF + b * L::KV_BYTES + ks * 2048, L::SUB, 1024);
                            tc_mma_ts(tmem_o(t), tmem_s(t) + 8u * ks, dv, idesc_o, (n_p[t] | ks) != 0);
                        }
                        ++n_p[t];
                        if (j == hi_of(t)) tc_commit(o_done(t));
                    }
                    if (t == nt - 1) tc_commit(kv_empty(b));   // every product that reads this stage has been issued
                    if (active(t, j + 1)) ok = issue_s(t, j + 1);
                }
            }
        }
    } else {
        // ---------------- softmax: one query row per thread ----------------
        const int t = (warp - 2) >> 2;
        const int quad = warp & 3;                       // the lanes of tensor memory this warp may touch
        const int r = quad * 32 + lane;
        if (t < nt) {
            const int rows_t = rows_of(t);
            const int pos0_t = pos0 + t * BQ;
            const int p_r = pos0_t + r;                  // absolute position of this row
            const int lo_r = a.window > 0 ? p_r - a.window + 1 : 0;
            const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
            const uint32_t ts = tmem_s(t) + lane_off, to = tmem_o(t) + lane_off;
            const float sl2 = a.scale_log2e;
            float m = -INFINITY, l = 0.f;
            bool ok = true;
            int cnt = 0;
            const int hi = hi_of(t);
            for (int j = lo_of(t); j <= hi; ++j, ++cnt) {
                ok = __all_sync(0xffffffffu, mbar_wait(s_full(t), (uint32_t)(cnt & 1), abort_flag));
                if (!ok) break;
                tc_fence_after();
                const int kb = j * BKEY;
                // every key of the block visible to every row of the sub-tile: no masking (most blocks)
                const bool interior = kb + BKEY - 1 <= pos0_t && (a.window <= 0 || kb >= pos0_t + BQ - a.window);
                // The row of S is read in chunks of 32 columns into two register buffers in turn: the load of the
                // next chunk is in flight while the current one is worked on.
                uint32_t ca[32], cb[32], pk[32];
                auto mask = [&](uint32_t* c, int chunk) {
                    if (interior) return;
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        const int key = kb + chunk * 32 + k;
                        if (key > p_r || key < lo_r) c[k] = 0xff800000u;   // -inf
                    }
                };
                // first pass: the row's maximum
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
                auto take_max = [&](uint32_t* c, int chunk) {
                    mask(c, chunk);
#pragma unroll
                    for (int k = 0; k < 32; k += 4) {
                        mx0 = fmaxf(mx0, __uint_as_float(c[k])); mx1 = fmaxf(mx1, __uint_as_float(c[k + 1]));
                        mx2 = fmaxf(mx2, __uint_as_float(c[k + 2])); mx3 = fmaxf(mx3, __uint_as_float(c[k + 3]));
                    }
                };
                tc_ld32(ts, ca);
                tc_ld_wait_for(ca);
                tc_ld32(ts + 32, cb); take_max(ca, 0); tc_ld_wait_for(cb);
                tc_ld32(ts + 64, ca); take_max(cb, 1); tc_ld_wait_for(ca);
                tc_ld32(ts + 96, cb); take_max(ca, 2); tc_ld_wait_for(cb);
                tc_ld32(ts, ca);      take_max(cb, 3);   // chunk 0 again, for the second pass
                const float mn = fmaxf(fmaxf(m, fmaxf(mx0, mx1)), fmaxf(mx2, mx3));
                const bool raise = mn > m && (m == -INFINITY || (mn - m) * sl2 > RAISE_MAX_BY);
                if (__any_sync(0xffffffffu, raise)) {
                    const float alpha = m == -INFINITY ? 0.f : fast_exp2((m - mn) * sl2);
                    l *= alpha;
                    m = mn;
                    if (cnt > 0) {   // the sums so far of this row, in tensor memory, take the new reference too
#pragma unroll
                        for (int c = 0; c < D / 32; ++c) {
                            tc_ld32(to + c * 32, cb);
                            tc_ld_wait_for(cb);
#pragma unroll
                            for (int k = 0; k < 32; ++k) cb[k] = __float_as_uint(__uint_as_float(cb[k]) * alpha);
                            tc_st32(to + c * 32, cb);
                        }
                    }
                }
                // second pass: P = exp2(S * scale - reference), as bfloat16 pairs over the first 64 columns of S
                // (columns 0-31 are written after columns 0-63 were read, columns 32-63 after all were)
                const float ref = m == -INFINITY ? 0.f : m * sl2;
                float sum0 = 0.f, sum1 = 0.f;
                auto take_exp = [&](uint32_t* c, int chunk, uint32_t* out) {
                    mask(c, chunk);
#pragma unroll
                    for (int k = 0; k < 32; k += 2) {
                        const float e0 = fast_exp2(fmaf(__uint_as_float(c[k]), sl2, -ref));
                        const float e1 = fast_exp2(fmaf(__uint_as_float(c[k + 1]), sl2, -ref));
                        sum0 += e0; sum1 += e1;
                        __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
                        out[k >> 1] = *reinterpret_cast<uint32_t*>(&pr);
                    }
                };
                tc_ld_wait_for(ca);
                tc_ld32(ts + 32, cb); take_exp(ca, 0, pk);      tc_ld_wait_for(cb);
                tc_ld32(ts + 64, ca); take_exp(cb, 1, pk + 16); tc_ld_wait_for(ca);
                tc_ld32(ts + 96, cb);
                tc_st32(ts, pk);                                 // the loads of columns 0-63 have completed
                take_exp(ca, 2, pk);
                tc_ld_wait_for(cb);
                take_exp(cb, 3, pk + 16);
                tc_st32(ts + 32, pk);
                l += sum0 + sum1;
                tc_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full(t));
            }
            const bool has_blocks = lo_of(t) <= hi_of(t);
            if (ok && has_blocks) ok = __all_sync(0xffffffffu, mbar_wait(o_done(t), 0, abort_flag));
            if (ok && part >= 0) {
                // a run of the tile's key blocks: the sums as they are, each row's reference and sum of weights
                tc_fence_after();
                const long slot = ((long)part * a.n_heads + head) * (2 * BQ) + t * BQ + r;
                if (r < rows_t) { a.part_ml[slot * 2] = has_blocks ? m : -INFINITY; a.part_ml[slot * 2 + 1] = has_blocks ? l : 0.f; }
                if (has_blocks) {
                    float* dst = a.part_o + slot * D;
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t ob[32];
                        tc_ld32(to + c * 32, ob);
                        tc_ld_wait();
                        if (r < rows_t) {
#pragma unroll
                            for (int k = 0; k < 32; k += 4)
                                *reinterpret_cast<uint4*>(dst + c * 32 + k) = make_uint4(ob[k], ob[k + 1], ob[k + 2], ob[k + 3]);
                        }
                    }
                }
            } else if (ok && has_blocks) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.f / l : 0.f;
                bf16* dst = a.out + (long)(tok0 + t * BQ + r) * a.ldo + (long)head * D;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t ob[32];
                    tc_ld32(to + c * 32, ob);
                    tc_ld_wait();
                    if (r < rows_t) {
#pragma unroll
                        for (int k = 0; k < 32; k += 8) {
                            uint4 v;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(ob[k]) * inv, __uint_as_float(ob[k + 1]) * inv);
                            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(ob[k + 2]) * inv, __uint_as_float(ob[k + 3]) * inv);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(ob[k + 4]) * inv, __uint_as_float(ob[k + 5]) * inv);
                            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(ob[k + 6]) * inv, __uint_as_float(ob[k + 7]) * inv);
                            v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                            v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                            *reinterpret_cast<uint4*>(dst + c * 32 + k) = v;
                        }
                    }
                }
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag_s && a.status) atomicExch(a.status, STATUS_TC_TIMEOUT);
}

// Adds up the runs of key blocks of the tiles that were cut: row r of a tile has, from run c, the sums o_c (32-bit,
// relative to the reference m_c) and the sum of weights l_c; with M = max m_c the result is
// sum_c o_c 2^((m_c - M) s) / sum_c l_c 2^((m_c - M) s), the runs taken in their order.  A run without visible keys
// for the row has m_c = -inf and is skipped.  merges: int32 [n, 4] = (first flat token, rows, first part, runs).
template <int D>
__global__ void __launch_bounds__(128) prefill_merge_kernel(const int* __restrict__ merges, const float* __restrict__ part_o,
                                                            const float* __restrict__ part_ml, bf16* __restrict__ out, long ldo,
                                                            int n_heads, float scale_log2e)
{
    fx_pdl_wait();
    const int* mg = merges + (long)blockIdx.x * 4;
    const int tok0 = mg[0], rows = mg[1], part0 = mg[2], runs = mg[3];
    const int head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int PER = D / 32;   // elements of a row per lane
    const int r = blockIdx.z * 4 + warp;   // a warp a row: all of a row's loads are on their way together
    if (r >= rows) return;
    const long slot0 = ((long)part0 * n_heads + head) * (2 * BQ) + r;
    const long run_stride = (long)n_heads * (2 * BQ);          // slots from one run to the next
    // lane c holds run c's reference and sum (runs <= 32)
    float m_c = -INFINITY, l_c = 0.f;
    if (lane < runs) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (slot0 + lane * run_stride) * 2);
        m_c = ml.x; l_c = ml.y;
    }
    const float mx = warp_max(m_c);
    const float w_c = m_c == -INFINITY ? 0.f : fast_exp2((m_c - mx) * scale_log2e);
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    float l = 0.f;
#pragma unroll 4
    for (int c = 0; c < runs; ++c) {
        const float w = __shfl_sync(0xffffffffu, w_c, c);
        l = fmaf(__shfl_sync(0xffffffffu, l_c, c), w, l);
        if (w == 0.f) continue;    // a run without visible keys for this row wrote no sums
        const float* src = part_o + (slot0 + c * run_stride) * D + lane * PER;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = fmaf(src[i], w, acc[i]);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    bf16* dst = out + (long)(tok0 + r) * ldo + (long)head * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) dst[i] = __float2bfloat16_rn(acc[i] * inv);
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
    fx_launch_pdl(kern, grid, NTHREADS, Smem<D>::TOTAL, s, mq, mk, mv, a);
    return fx_launch_status();
}

}  // namespace

// items: int32 [n_items, 8] = (first flat token, rows <= 256, entry index, absolute position of the first row, first
// key block of 128 positions, end of the key blocks, part or -1, unused), the heavy ones first.  An item with part -1
// holds every key block its tile sees and writes the tile's output; the items of a tile that was cut write their
// partial results to part_o [parts, n_heads, 256, head_dim] and part_ml [parts, n_heads, 256, 2] (32-bit), and
// merges: int32 [n_merges, 4] = (first flat token, rows, first part, runs) tells the second kernel which to add up
// (a tile's runs have consecutive parts, in the order of their keys).
// q is the fused [tokens, ldq] buffer whose rows start with the query heads; n_tokens its number of rows.
// Refuses (FX_ERR_SIZE / FX_ERR_ALIGN) what it does not take; the caller then uses the mma.sync kernel.
extern "C" int fx_prefill_attention_tc(const void* q, long ldq, int n_tokens, const void* k_pages, const void* v_pages,
                                       int n_pages, const int* block_table, int table_width, int page_size,
                                       const int* tiles, int n_tiles, const int* seq_slot, void* out, long ldo,
                                       int n_heads, int n_kv_heads, int head_dim, int window, float scale, int* status,
                                       float* part_o, float* part_ml, const int* merges, int n_merges, void* stream)
{
    if (n_tiles <= 0) return FX_OK;
    if (n_merges > 0 && (!part_o || !part_ml || !merges || (uintptr_t)part_o % 16)) return FX_ERR_ALIGN;
    if ((head_dim != 64 && head_dim != 128) || page_size < 64 || page_size % 64 || n_kv_heads <= 0 || n_heads % n_kv_heads)
        return FX_ERR_SIZE;
    if (ldq % 8 || ldo % 8 || (uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)out % 16)
        return FX_ERR_ALIGN;
    if (n_tiles > 65535) return FX_ERR_SIZE;
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
    a.part_o = part_o; a.part_ml = part_ml;
    dim3 grid(n_heads, n_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    const int rc = head_dim == 64 ? launch<64>(mq, mk, mv, a, grid, s) : launch<128>(mq, mk, mv, a, grid, s);
    if (rc != FX_OK || n_merges <= 0) return rc;
    dim3 mgrid(n_merges, n_heads, 2 * BQ / 4);
    if (head_dim == 64)
        fx_launch_pdl(prefill_merge_kernel<64>, mgrid, 128, 0, s, merges, (const float*)part_o, (const float*)part_ml, (bf16*)out,
                      ldo, n_heads, a.scale_log2e);
    else
        fx_launch_pdl(prefill_merge_kernel<128>, mgrid, 128, 0, s, merges, (const float*)part_o, (const float*)part_ml,
                      (bf16*)out, ldo, n_heads, a.scale_log2e);
    return fx_launch_status();
}
