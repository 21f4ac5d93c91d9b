// Split-key attention for decoding in bfloat16: keys and values stream through a ring of
// shared-memory stages filled by TMA, the tensor cores score them.
//
// Same contract and same partial results as decode_mma_kernel (attention_decode_mma.cu):
//   grid = (kv head [x block of 16 query heads], query token, key range),
//   partial (max, sum, acc) per (token, head, range) to scratch, merged by merge_kernel.
// That kernel's threads copy every tile themselves (cp.async, one tile in flight beside
// the one in work) and meet at two block-wide barriers a tile; a decode step is bound by
// the bytes of K and V, and a block that has one tile in flight cannot keep its share of
// the memory system busy.  Here a fifth warp does nothing but ask for tiles: a tile of 64
// keys is one page-aligned box of the cache ([64 keys][64 dims] pieces with the 128-byte
// swizzle), every stage of the ring that the four scoring warps have let go is in flight,
// and a stage changes hands through a pair of mbarriers (filled / free), so no warp waits
// for another.  Two blocks an SM with three stages of 32 KB each (head size 128) keep
// some 190 KB on their way to every SM.
//
// Warp w of the scoring warps takes keys 16w..16w+15 of every tile and keeps its own
// running (m, l, O); the four are merged in warp order at the end.  Scores, softmax and
// sums are 32-bit; P is rounded to bfloat16 for the second product, as in the prompt
// kernel.  Positions of a tile outside the block's range of keys are masked by their
// index; the bytes that arrive for them (pages hold finite values from the start) meet a
// probability of exactly zero.
//
// Launched as a dependent of the kernel that wrote the step's queries and newest keys:
// tiles that end before the step's own positions are requested before the wait for that
// kernel.  The caller must not have more than 64 new positions of a request written by
// the kernel directly before this one (the engine sends at most 8 this way).
//
// Every wait on a barrier is bounded; a block that gives up raises the status word.
//
// Reference: crates/ferrox-core/src/attention.rs:146-175 (online softmax), :484-524
// (window), :572-610 (pages).
#include "tc_common.cuh"
#include "api.h"

namespace {
using namespace fxtc;

constexpr int NCONSUMERS = 128, NTHREADS = 160, TK = 64, MAXQ = 16, MAX_STAGES = 8;
constexpr int PIECE = TK * 128;        // bytes of a [64 keys][64 dims] piece

struct DecArgs {
    const bf16* q; long ldq;
    const int* block_table; int table_width, page_size;
    const int* positions; const int* token_seq; const int* seq_slot;
    float* part_acc; float* part_ml;
    int n_heads, n_kv_heads, head_dim, window;
    float scale_log2e, scale;
    int split_len, n_splits, stages;
    // fresh > 0 is the caller's promise: the kernel before this one on the stream wrote the queries and the keys and
    // values of at most the last `fresh` positions of each request and nothing else that this kernel reads; tiles of
    // older keys are then asked for before that kernel has finished.  fresh <= 0: nothing is read before it has.
    int fresh;
    int* status;
    // With `counters` (one zeroed int per (token, block of heads), left zeroed again) the block that finishes a token's
    // last key range merges all of them into `out`; without, the caller runs the merge kernel.  A single key range a
    // token is written to `out` at once if that is given.
    bf16* out; long ldo; int* counters;
    // store_new: the rows of q are the fused [q | k | v] rows of the step as the projection left them, one token a
    // request.  The kernel then rotates the queries itself (split-half pairs over the whole head, cos and sin from
    // cos_sin [tokens][head_dim / 2][2]; null: no rotation), and the block that holds a token's own position rotates
    // that token's key, puts it and the value into its copy of their tile, and (one block per kv head, if
    // write_pages) into the cache pages: the work of the rotary kernel without its launch.
    int store_new, write_pages;
    const float* cos_sin;
    bf16* k_pages; bf16* v_pages;
};

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
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCONSUMERS) : "memory"); }
// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a [rows][128 bytes] piece stored with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

template <int DMAX>
// (two blocks an SM up to head size 128: the compiler may use the registers that leaves, which the loop's speed needs)
__global__ void __launch_bounds__(NTHREADS, DMAX <= 128 ? 2 : 1) decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                              const __grid_constant__ CUtensorMap map_v, DecArgs a)
{
    if (a.fresh <= 0) fx_pdl_wait();
    const int head_dim = a.head_dim, n_heads = a.n_heads, n_kv_heads = a.n_kv_heads;
    const int group_size = n_heads / n_kv_heads;
    const int chunks = (group_size + MAXQ - 1) / MAXQ;
    const int kvh = blockIdx.x / chunks;
    const int h0 = kvh * group_size + (blockIdx.x % chunks) * MAXQ;   // first query head of this block
    const int nq = min(MAXQ, kvh * group_size + group_size - h0);
    const int tkn = blockIdx.y, split = blockIdx.z;
    const int pos = a.positions[tkn];
    const int seq = a.token_seq[tkn];                 // (asked for beside the position: the table row hangs on it)
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    int k_begin, k_end;
    fx_split_range(pos, lo, split, a.n_splits, a.split_len, k_begin, k_end);
    if (k_begin >= k_end) return;   // nothing of this range is visible: `merge` skips it by the same rule

    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag_s, last_block_s, complete_s;
    __shared__ uint32_t ranges_with_keys_s;
    __shared__ int page_ok_s[MAX_STAGES];
    __shared__ float m_s[4][16], l_s[4][16];
    __shared__ __align__(8) uint64_t bars_s[2 * MAX_STAGES];
    volatile int* abort_flag = &abort_flag_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int halves = head_dim / 64;
    const int stage_bytes = 2 * halves * PIECE;             // K pieces, then V pieces
    const int stages = a.stages;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int pitch = head_dim * 2 + 16;
    const uint32_t q_u = ring + stages * stage_bytes;       // [16][pitch]
    auto full = [&](int s) { return smem_u32(&bars_s[s]); };
    auto empty = [&](int s) { return smem_u32(&bars_s[MAX_STAGES + s]); };

    // tiles are the 64-key blocks of the request's positions that meet [k_begin, k_end)
    const int first_tile = k_begin / TK;
    const int n_tiles = (k_end - 1) / TK - first_tile + 1;

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        for (int s = 0; s < stages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == 4) {
        // ---------------- producer: one thread asks for every tile ----------------
        if (lane == 0) {
            const int* table = a.block_table + (long)a.seq_slot[seq] * a.table_width;
            bool waited = false;
            // table entries are read one tile ahead, so that a stage that comes free is asked for at once
            int page_next = table[first_tile * TK / a.page_size];
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % stages;
                const int key0 = (first_tile + j) * TK;
                const int page = page_next;
                if (j + 1 < n_tiles) page_next = table[(key0 + TK) / a.page_size];
                // The kernel before this one wrote the keys and values of the step's own positions (the last
                // a.fresh of a request at most); a tile that ends before them may be asked for at once.  With
                // store_new it wrote no key at all: this kernel puts the token's own row into its copy of the tile
                // after the tile has arrived, whatever the page held.
                if (!waited && !a.store_new && key0 + TK > pos + 1 - a.fresh) { fx_pdl_wait(); waited = true; }
                if (j >= stages && !mbar_wait(empty(s), ((j / stages) - 1) & 1, abort_flag)) break;
                page_ok_s[s] = page >= 0;
                if (page >= 0) {
                    // a position without a page is never dereferenced; its tile is skipped by the scoring warps
                    mbar_expect_tx(full(s), (uint32_t)stage_bytes);
                    const uint32_t dst = ring + s * stage_bytes;
                    const int in_page = key0 % a.page_size;
                    for (int hf = 0; hf < halves; ++hf) {
                        tma_load_4d(dst + hf * PIECE, &map_k, hf * 64, in_page, kvh, page, full(s));
                        tma_load_4d(dst + (halves + hf) * PIECE, &map_v, hf * 64, in_page, kvh, page, full(s));
                    }
                } else {
                    mbar_arrive(full(s));
                }
            }
            if (!waited) fx_pdl_wait();
        }
    } else {
        // ---------------- four scoring warps ----------------
        const int g = lane >> 2, t4 = lane & 3;
        const int chunks_row = head_dim / 8;                   // 16-byte chunks per row
        const int half_d = head_dim >> 1;
        // store_new: the warp whose 16 keys of the last tile hold the token's own position prepares that key and value
        const bool owns_new = a.store_new && pos >= k_begin && pos < k_end && warp == ((pos % TK) >> 4);
        const bool writes_page = owns_new && a.write_pages && blockIdx.x % chunks == 0;
        // (the table is not the work of the kernel before this one: the page is looked up before the wait for it)
        const int new_page = writes_page ? a.block_table[(long)a.seq_slot[seq] * a.table_width + pos / a.page_size] : -1;
        fx_pdl_wait();
        // query rows of this block (zero beyond the group): on their way while the new key is prepared
        for (int c = threadIdx.x; c < 16 * chunks_row; c += NCONSUMERS) {
            const int r = c / chunks_row, ch = c - r * chunks_row;
            const bf16* src = a.q + (long)tkn * a.ldq + (long)(h0 + min(r, nq - 1)) * head_dim + ch * 8;
            cp_async16(q_u + r * pitch + ch * 16, src, r < nq ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        // cos and sin of this thread's first pair of the queries' rotation, asked for beside the queries
        const bool rotates_q = a.store_new && a.cos_sin;
        float2 cs_first = make_float2(1.f, 0.f);
        if (rotates_q && (int)threadIdx.x < nq * half_d)
            cs_first = *reinterpret_cast<const float2*>(a.cos_sin + ((long)tkn * half_d + (int)threadIdx.x % half_d) * 2);
        bf16 new_k[DMAX / 32], new_v[DMAX / 32];   // elements lane + 32 u of the row
        if (owns_new) {
            const bf16* krow = a.q + (long)tkn * a.ldq + (long)(n_heads + kvh) * head_dim;
            const bf16* vrow = krow + (long)n_kv_heads * head_dim;
#pragma unroll
            for (int u = 0; u < DMAX / 32; ++u) {
                const int e = lane + 32 * u;
                if (e < head_dim) {
                    new_v[u] = vrow[e];
                    float x = __bfloat162float(krow[e]);
                    if (a.cos_sin) {
                        // element e pairs with e +- head_dim / 2; the same arithmetic as the rotary kernel's
                        const int i = e < half_d ? e : e - half_d;
                        const float2 cs = *reinterpret_cast<const float2*>(a.cos_sin + ((long)tkn * half_d + i) * 2);
                        const float other = __bfloat162float(krow[e < half_d ? e + half_d : e - half_d]);
                        x = e < half_d ? x * cs.x - other * cs.y : other * cs.y + x * cs.x;
                    }
                    new_k[u] = __float2bfloat16_rn(x);
                }
            }
            if (writes_page) {
                if (new_page < 0) { if (lane == 0 && a.status) atomicExch(a.status, 2); }
                else {
                    const long at = (((long)new_page * n_kv_heads + kvh) * a.page_size + pos % a.page_size) * head_dim;
#pragma unroll
                    for (int u = 0; u < DMAX / 32; ++u) {
                        const int e = lane + 32 * u;
                        if (e < head_dim) { a.k_pages[at + e] = new_k[u]; a.v_pages[at + e] = new_v[u]; }
                    }
                }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        consumers_sync();
        if (rotates_q) {
            // the queries as projected: rotate them where they lie (pairs i, i + head_dim / 2 of every head)
            bf16* q_s = reinterpret_cast<bf16*>(smem_raw + (q_u - smem_u32(smem_raw)));
            for (int idx = threadIdx.x; idx < nq * half_d; idx += NCONSUMERS) {
                const int r = idx / half_d, i = idx - r * half_d;
                const float2 cs = idx == (int)threadIdx.x ? cs_first
                                                          : *reinterpret_cast<const float2*>(a.cos_sin + ((long)tkn * half_d + i) * 2);
                bf16* row = q_s + (long)r * (pitch / 2);
                const float x = __bfloat162float(row[i]), y = __bfloat162float(row[i + half_d]);
                row[i] = __float2bfloat16_rn(x * cs.x - y * cs.y);
                row[i + half_d] = __float2bfloat16_rn(x * cs.y + y * cs.x);
            }
            consumers_sync();
        }

        constexpr int KS = DMAX / 16, ON = DMAX / 8;
        const int ks_n = head_dim / 16;
        uint32_t qa[KS][4];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
            if (ks < ks_n)
                ldsm4(q_u + (lane & 15) * pitch + (ks * 16 + (lane >> 4) * 8) * 2, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
        float o[ON][4];
#pragma unroll
        for (int i = 0; i < ON; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8
        const int kw = warp * 16;                                   // this warp's keys inside a tile

        for (int j = 0; j < n_tiles; ++j) {
            const int s = j % stages;
            if (!mbar_wait(full(s), (j / stages) & 1, abort_flag)) break;
            if (owns_new && j == n_tiles - 1) {
                // the token's own key and value into this block's copy of their tile (only this warp reads the row)
                const int r = pos % TK;
                const uint32_t ku = ring + s * stage_bytes, vu = ku + halves * PIECE;
#pragma unroll
                for (int u = 0; u < DMAX / 32; ++u) {
                    const int e = lane + 32 * u;
                    if (e < head_dim) {
                        const uint32_t off = (uint32_t)((e >> 6) * PIECE) + swz(r, (e & 63) >> 3) + (uint32_t)((e & 7) * 2);
                        asm volatile("st.shared.b16 [%0], %1;" ::"r"(ku + off), "h"(*reinterpret_cast<const uint16_t*>(&new_k[u])) : "memory");
                        asm volatile("st.shared.b16 [%0], %1;" ::"r"(vu + off), "h"(*reinterpret_cast<const uint16_t*>(&new_v[u])) : "memory");
                    }
                }
                __syncwarp();
            }
            const int key0 = (first_tile + j) * TK + kw;            // this warp's first key
            if (page_ok_s[s] && key0 < k_end && key0 + 16 > k_begin) {
                const uint32_t ku = ring + s * stage_bytes, vu = ku + halves * PIECE;
                float sc[2][4];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) { sc[jj][0] = sc[jj][1] = sc[jj][2] = sc[jj][3] = 0.f; }
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    if (ks < ks_n) {
                        uint32_t b0, b1, b2, b3;
                        const int krow = kw + (lane & 7) + (lane >> 4) * 8;
                        ldsm4(ku + (ks >> 2) * PIECE + swz(krow, (ks & 3) * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
                        mma16816(sc[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                        mma16816(sc[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                    }
                }
                // keys outside the block's range do not count
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + jj * 8 + 2 * t4 + e;
                        const bool ok = key >= k_begin && key < k_end;
                        if (!ok) { sc[jj][e] = -INFINITY; sc[jj][2 + e] = -INFINITY; }
                        mx0 = fmaxf(mx0, sc[jj][e]);
                        mx1 = fmaxf(mx1, sc[jj][2 + e]);
                    }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                const float ref0 = mn0 == -INFINITY ? 0.f : mn0 * a.scale_log2e, ref1 = mn1 == -INFINITY ? 0.f : mn1 * a.scale_log2e;
                const float al0 = m0 == -INFINITY ? 0.f : exp2f(m0 * a.scale_log2e - ref0);
                const float al1 = m1 == -INFINITY ? 0.f : exp2f(m1 * a.scale_log2e - ref1);
                float sum0 = 0.f, sum1 = 0.f;
                uint32_t p[2][2];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const float e0 = exp2f(sc[jj][0] * a.scale_log2e - ref0), e1 = exp2f(sc[jj][1] * a.scale_log2e - ref0);
                    const float e2 = exp2f(sc[jj][2] * a.scale_log2e - ref1), e3 = exp2f(sc[jj][3] * a.scale_log2e - ref1);
                    sum0 += e0 + e1; sum1 += e2 + e3;
                    p[jj][0] = pack_bf16(e0, e1);
                    p[jj][1] = pack_bf16(e2, e3);
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
                        ldsm4t(vu + (i >> 2) * PIECE + swz(vrow, (i & 3) * 2 + (lane >> 4)), b0, b1, b2, b3);
                        mma16816(o[2 * i], p[0][0], p[0][1], p[1][0], p[1][1], b0, b1);
                        mma16816(o[2 * i + 1], p[0][0], p[0][1], p[1][0], p[1][1], b2, b3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));   // this warp is done with the stage
        }

        // ---- merge the four warps, in warp order, and write the partial result ------------
        consumers_sync();                            // every warp has left the ring (all its tiles have arrived)
        // [4][16][head_dim + 8]: rows 8 floats longer than a head, so that the 8-byte stores of a quarter warp
        // (rows g, columns 2 t4) fall into different banks; only the rows of real heads are written
        float* acc_s = reinterpret_cast<float*>(smem_raw + (ring - smem_u32(smem_raw)));
        const int acc_pitch = head_dim + 8;
        if (t4 == 0) { m_s[warp][g] = m0; m_s[warp][g + 8] = m1; l_s[warp][g] = l0; l_s[warp][g + 8] = l1; }
        if (threadIdx.x == 0) complete_s = !abort_flag_s;   // one reading for all: the barriers below are taken by all or none
#pragma unroll
        for (int i = 0; i < ON; ++i) {
            const int col = i * 8 + 2 * t4;
            if (col < head_dim) {
                if (g < nq) *reinterpret_cast<float2*>(acc_s + ((long)warp * 16 + g) * acc_pitch + col) = make_float2(o[i][0], o[i][1]);
                if (g + 8 < nq) *reinterpret_cast<float2*>(acc_s + ((long)warp * 16 + g + 8) * acc_pitch + col) = make_float2(o[i][2], o[i][3]);
            }
        }
        consumers_sync();
        if (complete_s) {
            for (int idx = threadIdx.x; idx < nq * head_dim; idx += NCONSUMERS) {
                const int h = idx / head_dim, e = idx - h * head_dim;
                float mm = -INFINITY;
#pragma unroll
                for (int w = 0; w < 4; ++w) mm = fmaxf(mm, m_s[w][h]);
                float ll = 0.f, acc = 0.f;
                if (mm > -INFINITY) {
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float wgt = m_s[w][h] == -INFINITY ? 0.f : exp2f((m_s[w][h] - mm) * a.scale_log2e);
                        ll += l_s[w][h] * wgt;
                        acc += acc_s[((long)w * 16 + h) * acc_pitch + e] * wgt;
                    }
                }
                if (a.n_splits == 1 && a.out) {
                    // the only key range of its token: this is the result
                    a.out[(long)tkn * a.ldo + (long)(h0 + h) * head_dim + e] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
                    continue;
                }
                const long slot = ((long)tkn * n_heads + (h0 + h)) * a.n_splits + split;
                a.part_acc[slot * head_dim + e] = acc;
                // merge_kernel works with natural-log maxima of the scaled scores
                if (e == 0) { a.part_ml[slot * 2] = mm == -INFINITY ? -INFINITY : mm * a.scale; a.part_ml[slot * 2 + 1] = ll; }
            }
            if (a.counters && a.n_splits > 1) {
                // ---- the block that finishes a token's last key range merges them, in range order ----
                // Every thread's partial sums are written before the barrier; the one thread that counts does so with
                // release and acquire at the scope of the GPU, which orders the block's writes (cumulative through the
                // barrier) before the count and the count before what the last block reads: no fence in every thread.
                consumers_sync();
                if (warp == 0) {
                    // ranges without visible keys never ran (n_splits <= 32 here): lane s2 looks at range s2
                    int b = 0, e = 0;
                    if (lane < a.n_splits) fx_split_range(pos, lo, lane, a.n_splits, a.split_len, b, e);
                    const uint32_t with_keys = __ballot_sync(0xffffffffu, b < e);
                    if (lane == 0) {
                        ranges_with_keys_s = with_keys;
                        int* counter = a.counters + (long)tkn * gridDim.x + blockIdx.x;
                        int before;
                        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(before) : "l"(counter) : "memory");
                        last_block_s = before == __popc(with_keys) - 1;
                        if (last_block_s) *counter = 0;    // every other block of this token has counted: ready for the next launch
                    }
                }
                consumers_sync();
                if (last_block_s) {
                    const uint32_t with_keys = ranges_with_keys_s;
                    const int n_splits = a.n_splits;
                    // The partial sums of this thread's first element and every range's (max, sum) of the block's heads
                    // are asked for together: one trip to the L2 instead of three.  (The ring is free: every thread
                    // has read its part of acc_s before the barriers above.)  A range without keys was never
                    // written and counts as one whose maximum is -inf.
                    constexpr int MERGE_AHEAD = 16;    // partial sums asked for together; added up in range order
                    float part[MERGE_AHEAD];
                    auto load_parts = [&](int idx, int s0) {
                        const int h = idx / head_dim, e = idx - h * head_dim;
                        const long base = ((long)tkn * n_heads + (h0 + h)) * n_splits;
#pragma unroll
                        for (int u = 0; u < MERGE_AHEAD; ++u) {
                            const int s2 = s0 + u;
                            part[u] = (s2 < n_splits && (with_keys >> s2 & 1)) ? __ldcg(a.part_acc + (base + s2) * head_dim + e) : 0.f;
                        }
                    };
                    if ((int)threadIdx.x < nq * head_dim) load_parts(threadIdx.x, 0);
                    float* ml2 = acc_s;                // [nq][n_splits][2]
                    for (int i = threadIdx.x; i < nq * n_splits; i += NCONSUMERS) {
                        const int h = i / n_splits, s2 = i - h * n_splits;
                        float2 v = make_float2(-INFINITY, 0.f);
                        if (with_keys >> s2 & 1)
                            v = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (((long)tkn * n_heads + (h0 + h)) * n_splits + s2) * 2));
                        ml2[2 * i] = v.x; ml2[2 * i + 1] = v.y;
                    }
                    consumers_sync();
                    for (int idx = threadIdx.x; idx < nq * head_dim; idx += NCONSUMERS) {
                        const int h = idx / head_dim, e = idx - h * head_dim;
                        const float* ml_h = ml2 + (long)h * n_splits * 2;
                        float mm = -INFINITY;
                        for (int s2 = 0; s2 < n_splits; ++s2) mm = fmaxf(mm, ml_h[s2 * 2]);
                        float ll = 0.f, acc = 0.f;
                        for (int s0 = 0; s0 < n_splits; s0 += MERGE_AHEAD) {
                            if (idx != (int)threadIdx.x || s0 != 0) load_parts(idx, s0);
#pragma unroll
                            for (int u = 0; u < MERGE_AHEAD; ++u) {
                                const float ms = s0 + u < n_splits ? ml_h[(s0 + u) * 2] : -INFINITY;
                                if (ms == -INFINITY) continue;
                                const float wgt = __expf(ms - mm);
                                ll += ml_h[(s0 + u) * 2 + 1] * wgt;
                                acc += part[u] * wgt;
                            }
                        }
                        a.out[(long)tkn * a.ldo + (long)(h0 + h) * head_dim + e] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
                    }
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag_s && a.status) atomicExch(a.status, STATUS_TC_TIMEOUT);
}

bool encode(CUtensorMap* map, const void* ptr, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int DMAX>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const DecArgs& a, dim3 grid, size_t smem, cudaStream_t s)
{
    auto kern = decode_tma_kernel<DMAX>;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    fx_launch_pdl(kern, grid, NTHREADS, smem, s, mk, mv, a);
    return fx_launch_status();
}

}  // namespace

// Stages of the ring and bytes of dynamic shared memory for a head size (0 stages: not taken).
static int tma_ring(int head_dim, size_t* smem)
{
    if (head_dim <= 0 || head_dim % 64 || head_dim > 256) return 0;
    const int stage_bytes = 2 * (head_dim / 64) * PIECE;
    int stages = (96 * 1024) / stage_bytes;             // two blocks an SM up to head size 128
    if (stages < 3) stages = 3;                         // head size 192, 256: one block an SM
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    const size_t merge = (size_t)4 * 16 * (head_dim + 8) * sizeof(float);
    size_t ring = (size_t)stages * stage_bytes;
    if (ring < merge) ring = merge;
    *smem = 1024 + ring + (size_t)16 * (head_dim * 2 + 16);
    return stages;
}

// As fx_decode_split_mma (partials; the caller runs the merge), or with `counters` the whole attention: the last block of
// a token merges its key ranges into `out`.  Returns FX_ERR_SIZE for shapes it does not take.
extern "C" int fx_decode_split_tma(const void* q, long ldq, const void* k_pages, const void* v_pages, int n_pages,
                                   const int* block_table, int table_width, int page_size, const int* positions,
                                   const int* token_seq, const int* seq_slot, float* part_acc, float* part_ml,
                                   int n_tokens, int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                   int split_len, int n_splits, int* status, void* out, long ldo, int* counters,
                                   int fresh_positions, int store_new, int write_pages, const float* cos_sin, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (counters && (n_splits > 32 || !out || ldo % 2)) return FX_ERR_SIZE;
    if (head_dim <= 0 || n_pages <= 0 || page_size < TK || page_size % TK || n_kv_heads <= 0 || n_heads % n_kv_heads)
        return FX_ERR_SIZE;
    if (ldq % 8 || (uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16) return FX_ERR_ALIGN;
    const int group = n_heads / n_kv_heads;
    const int chunks = (group + MAXQ - 1) / MAXQ;
    size_t smem = 0;
    const int stages = tma_ring(head_dim, &smem);
    if (stages == 0) return FX_ERR_SIZE;
    dim3 grid(n_kv_heads * chunks, n_tokens, n_splits);
    if (grid.y > 65535u || grid.z > 65535u) return FX_ERR_SIZE;
    CUtensorMap mk, mv;
    {
        cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads, (cuuint64_t)n_pages};
        cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)page_size * head_dim * 2,
                                 (cuuint64_t)n_kv_heads * page_size * head_dim * 2};
        cuuint32_t box[4] = {64, TK, 1, 1};
        if (!encode(&mk, k_pages, dims, strides, box) || !encode(&mv, v_pages, dims, strides, box)) return FX_ERR_SIZE;
    }
    DecArgs a;
    a.q = (const bf16*)q; a.ldq = ldq;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size;
    a.positions = positions; a.token_seq = token_seq; a.seq_slot = seq_slot;
    a.part_acc = part_acc; a.part_ml = part_ml;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.window = window;
    a.scale_log2e = scale * 1.4426950408889634f; a.scale = scale;
    a.split_len = split_len; a.n_splits = n_splits; a.stages = stages; a.status = status;
    a.fresh = fresh_positions;
    a.store_new = store_new; a.write_pages = write_pages; a.cos_sin = cos_sin;
    a.k_pages = (bf16*)const_cast<void*>(k_pages); a.v_pages = (bf16*)const_cast<void*>(v_pages);
    a.out = (bf16*)out; a.ldo = ldo; a.counters = counters;
    if (n_splits > 1 && !counters) a.out = nullptr;   // partial results only
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim <= 64) return launch<64>(mk, mv, a, grid, smem, s);
    if (head_dim <= 128) return launch<128>(mk, mv, a, grid, smem, s);
    return launch<256>(mk, mv, a, grid, smem, s);
}
