// Attention for steps with few query tokens (decoding, short portions): the keys of
// each request are split into ranges that separate blocks read, so that one long
// context keeps many SMs busy; a second kernel merges the ranges.
//
//   grid = (kv head [x head chunk], query token, split)
//   split s covers the token's visible keys [max(0, p - W + 1), p] cut into n_splits runs of equal length
//   (split_len 0), or the absolute key positions [s * split_len, (s+1) * split_len) clipped to the
//   visible range (split_len > 0): fx_split_range in common.cuh.
//
// A block reads each key and value of its range once for all query heads that
// share the kv head (up to 8; more are handled by further head chunks).  Threads
// form groups of LPK lanes; a group takes every (128/LPK)-th key, each lane
// holding 8 (bfloat16) or 4 (float) consecutive elements of the head dimension,
// scores it with a group-wide sum and keeps a running (m, l, acc) per query head.
// The groups are merged in fixed order through shared memory, the block writes
// (m, l, acc) for its split to scratch memory, and `merge` combines the splits in
// order.  All sums are 32-bit.  The number of runs depends on the step's size and the
// context limit; where a token's runs are cut depends on its own position only.
//
// Reference: one warp per head over a contiguous cache
// (crates/ferrox-cuda/src/attn.rs:22-79); online softmax
// crates/ferrox-core/src/attention.rs:146-175; window :484-524; pages :572-610.
#include "common.cuh"
#include "api.h"
#include "no_alloc.h"

namespace {

constexpr int NTHREADS = 128;
constexpr int STAGES = 4;    // buffers of the key/value ring
constexpr int MAXQ = 8;      // query heads per block
constexpr int MAX_D = 256;

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* o) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
};
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16* p, float* o) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// exp in full precision on the 32-bit path, the fast approximation on the bfloat16 path
template <typename T> __device__ __forceinline__ float fx_exp(float x);
template <> __device__ __forceinline__ float fx_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float fx_exp<bf16>(float x) { return __expf(x); }

// LPK lanes per key; each lane owns VPL vectors of Vec<T>::N elements: element
// index of vector v of lane ln is (v * LPK + ln) * N.
template <typename T, int LPK, int VPL, int GQ>
__global__ void __launch_bounds__(NTHREADS) decode_split_kernel(
    const T* __restrict__ q, long ldq, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    const int* __restrict__ block_table, int table_width, int page_size,
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
    float* __restrict__ part_acc, float* __restrict__ part_ml,
    int n_heads, int n_kv_heads, int head_dim, int window, float scale, int split_len, int n_splits)
{
    constexpr int N = Vec<T>::N;
    constexpr int GROUPS = NTHREADS / LPK;
    fx_pdl_wait();
    const int group_size = n_heads / n_kv_heads;
    const int chunks = (group_size + GQ - 1) / GQ;
    const int kvh = blockIdx.x / chunks;
    const int h0 = kvh * group_size + (blockIdx.x % chunks) * GQ;   // first query head of this block
    const int nq = min(GQ, kvh * group_size + group_size - h0);
    const int tkn = blockIdx.y, split = blockIdx.z;
    const int pos = positions[tkn];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    int k_begin, k_end;
    fx_split_range(pos, lo, split, n_splits, split_len, k_begin, k_end);
    if (k_begin >= k_end) return;   // nothing of this range is visible: `merge` skips it by the same rule
    const int grp = threadIdx.x / LPK, ln = threadIdx.x % LPK;

    float qr[GQ][VPL][N], acc[GQ][VPL][N], m[GQ], l[GQ];
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int e = (v * LPK + ln) * N;
#pragma unroll
            for (int i = 0; i < N; ++i) { acc[h][v][i] = 0.f; qr[h][v][i] = 0.f; }
            if (h < nq && e < head_dim) Vec<T>::load(q + (long)tkn * ldq + (long)(h0 + h) * head_dim + e, qr[h][v]);
        }
    }

    // ---- stream the keys and values of this range through shared memory ------------
    // Tiles of TK keys arrive by cp.async into a ring of STAGES buffers, so that the
    // bytes in flight do not depend on registers; a position without a page, or past
    // the range, is zero-filled and flagged.  Group g then takes keys g, g + GROUPS, ...
    // of each tile, in key order.
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    const int row_bytes = head_dim * (int)sizeof(T);
    const int TK = row_bytes <= 256 ? 32 : (row_bytes <= 512 ? 16 : 8);   // keys per tile (multiple of GROUPS)
    const int stage_bytes = 2 * TK * row_bytes + 128;                     // K rows, V rows, validity flags
    const int n_tiles = k_begin < k_end ? (k_end - k_begin + TK - 1) / TK : 0;
    constexpr int KB = (GQ * VPL <= 2) ? 4 : (GQ * VPL <= 4 ? 2 : 1);    // keys of a group scored together
    if (n_tiles > 0) {
        const int* table = block_table + (long)seq_slot[token_seq[tkn]] * table_width;
        const long head_stride = (long)page_size * head_dim;
        const int cpk = row_bytes / 16;                                   // 16-byte chunks per key row
        const uint32_t smem_u = (uint32_t)__cvta_generic_to_shared(dyn_smem);
        auto issue = [&](int tile) {
            if (tile < n_tiles) {
                uint8_t* st = dyn_smem + (tile % STAGES) * stage_bytes;
                const uint32_t su = smem_u + (tile % STAGES) * stage_bytes;
                for (int c = threadIdx.x; c < TK * cpk; c += NTHREADS) {
                    const int r = c / cpk, ch = c - r * cpk;
                    const int key = k_begin + tile * TK + r;
                    int page = -1;
                    if (key < k_end) page = table[key / page_size];
                    const bool ok = page >= 0;
                    const long base = ok ? ((long)page * n_kv_heads + kvh) * head_stride + (long)(key % page_size) * head_dim : 0;
                    const uint32_t dst = su + r * row_bytes + ch * 16;
                    const uint8_t* ksrc = reinterpret_cast<const uint8_t*>(k_pages + base) + ch * 16;
                    const uint8_t* vsrc = reinterpret_cast<const uint8_t*>(v_pages + base) + ch * 16;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(ksrc), "r"(ok ? 16 : 0) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + TK * row_bytes), "l"(vsrc), "r"(ok ? 16 : 0) : "memory");
                    if (ch == 0) st[2 * TK * row_bytes + r] = ok ? 1 : 0;
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        for (int s = 0; s < STAGES - 1; ++s) issue(s);
        for (int tile = 0; tile < n_tiles; ++tile) {
            asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
            __syncthreads();                 // tile `tile` has landed; everyone is done with tile - 1
            issue(tile + STAGES - 1);        // refills the buffer that tile - 1 used
            const uint8_t* st = dyn_smem + (tile % STAGES) * stage_bytes;
            const T* ks = reinterpret_cast<const T*>(st);
            const T* vs = reinterpret_cast<const T*>(st + TK * row_bytes);
            const uint8_t* flags = st + 2 * TK * row_bytes;
            // A group takes KPG = TK / GROUPS keys of the tile (same count for every thread, so
            // the group-wide shuffles are executed by whole warps).  Their scores are
            // independent, so they are computed together; then ONE update of (m, l, acc)
            // takes them in key order.
            for (int r0 = 0; r0 < TK; r0 += GROUPS * KB) {
                float sc[KB][GQ];
                bool valid[KB];
#pragma unroll
                for (int u = 0; u < KB; ++u) {
                    const int r = r0 + u * GROUPS + grp;
                    valid[u] = r < TK && flags[r] != 0;
                    float kv[VPL][N];
#pragma unroll
                    for (int h = 0; h < GQ; ++h) sc[u][h] = 0.f;
#pragma unroll
                    for (int v = 0; v < VPL; ++v) {
                        const int e = (v * LPK + ln) * N;
                        if (r < TK && e < head_dim) {
                            Vec<T>::load(ks + (long)r * head_dim + e, kv[v]);
#pragma unroll
                            for (int h = 0; h < GQ; ++h)
#pragma unroll
                                for (int i = 0; i < N; ++i) sc[u][h] = fmaf(qr[h][v][i], kv[v][i], sc[u][h]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < KB; ++u)
#pragma unroll
                    for (int h = 0; h < GQ; ++h) {
#pragma unroll
                        for (int o = LPK / 2; o > 0; o >>= 1) sc[u][h] += __shfl_xor_sync(0xffffffffu, sc[u][h], o);
                        sc[u][h] = valid[u] ? sc[u][h] * scale : -INFINITY;
                    }
#pragma unroll
                for (int h = 0; h < GQ; ++h) {
                    float m_new = m[h];
#pragma unroll
                    for (int u = 0; u < KB; ++u) m_new = fmaxf(m_new, sc[u][h]);
                    if (m_new == -INFINITY) continue;              // nothing visible yet for this head
                    const float alpha = fx_exp<T>(m[h] - m_new);  // m = -inf at first: exp(-inf) = 0
                    float p[KB];
                    float psum = 0.f;
#pragma unroll
                    for (int u = 0; u < KB; ++u) { p[u] = fx_exp<T>(sc[u][h] - m_new); psum += p[u]; }
                    l[h] = l[h] * alpha + psum;
                    m[h] = m_new;
#pragma unroll
                    for (int v = 0; v < VPL; ++v)
#pragma unroll
                        for (int i = 0; i < N; ++i) acc[h][v][i] *= alpha;
#pragma unroll
                    for (int u = 0; u < KB; ++u) {
                        const int r = r0 + u * GROUPS + grp;
                        if (!valid[u]) continue;
#pragma unroll
                        for (int v = 0; v < VPL; ++v) {
                            const int e = (v * LPK + ln) * N;
                            if (e < head_dim) {
                                float vv[N];
                                Vec<T>::load(vs + (long)r * head_dim + e, vv);
#pragma unroll
                                for (int i = 0; i < N; ++i) acc[h][v][i] = fmaf(p[u], vv[i], acc[h][v][i]);
                            }
                        }
                    }
                }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();   // the ring is reused below for the merge
    }

    // merge the groups of this block, in group order
    __shared__ float sm_m[GROUPS][GQ], sm_l[GROUPS][GQ];
    float* sm_acc = reinterpret_cast<float*>(dyn_smem);   // [GROUPS][GQ][head_dim_padded]
    const int dpad = VPL * LPK * N;
    if (ln == 0) {
#pragma unroll
        for (int h = 0; h < GQ; ++h) { sm_m[grp][h] = m[h]; sm_l[grp][h] = l[h]; }
    }
#pragma unroll
    for (int h = 0; h < GQ; ++h)
#pragma unroll
        for (int v = 0; v < VPL; ++v)
#pragma unroll
            for (int i = 0; i < N; ++i)
                sm_acc[((long)grp * GQ + h) * dpad + (v * LPK + ln) * N + i] = acc[h][v][i];
    __syncthreads();
    for (int o = threadIdx.x; o < nq * head_dim; o += NTHREADS) {
        const int h = o / head_dim, e = o - h * head_dim;
        float mm = -INFINITY;
        for (int gI = 0; gI < GROUPS; ++gI) mm = fmaxf(mm, sm_m[gI][h]);
        float ll = 0.f, a = 0.f;
        if (mm > -INFINITY) {
            for (int gI = 0; gI < GROUPS; ++gI) {
                const float w = fx_exp<T>(sm_m[gI][h] - mm);
                ll += sm_l[gI][h] * w;
                a += sm_acc[((long)gI * GQ + h) * dpad + e] * w;
            }
        }
        const long slot = ((long)tkn * n_heads + (h0 + h)) * n_splits + split;
        part_acc[slot * head_dim + e] = a;
        if (e == 0) { part_ml[slot * 2] = mm; part_ml[slot * 2 + 1] = ll; }
    }
}

template <typename T>
__global__ void merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                             const int* __restrict__ positions, T* __restrict__ out, long ldo, int n_heads,
                             int head_dim, int n_splits, int split_len, int window)
{
    fx_pdl_wait();
    const int tkn = blockIdx.x, h = blockIdx.y;
    const long base = ((long)tkn * n_heads + h) * n_splits;
    // the splits that hold visible keys of this token (the others were not written)
    const int pos = positions[tkn];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    auto has_keys = [&](int s) { int b, e; fx_split_range(pos, lo, s, n_splits, split_len, b, e); return b < e; };
    float mm = -INFINITY;
    for (int s = 0; s < n_splits; ++s)
        if (has_keys(s)) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    for (int e = threadIdx.x; e < head_dim; e += blockDim.x) {
        float ll = 0.f, a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            if (!has_keys(s)) continue;
            const float ms = part_ml[(base + s) * 2];
            if (ms == -INFINITY) continue;
            const float w = fx_exp<T>(ms - mm);
            ll += part_ml[(base + s) * 2 + 1] * w;
            a += part_acc[(base + s) * head_dim + e] * w;
        }
        out[(long)tkn * ldo + (long)h * head_dim + e] = from_f32<T>(ll > 0.f ? a / ll : 0.f);
    }
}

template <typename T, int LPK, int VPL, int GQ>
int launch_one(dim3 grid, cudaStream_t s, const T* q, long ldq, const T* k, const T* v, const int* bt, int tw, int ps,
               const int* pos, const int* tseq, const int* sslot, float* pa, float* pm, int nh, int nkv, int d,
               int window, float scale, int split_len, int n_splits)
{
    auto kern = decode_split_kernel<T, LPK, VPL, GQ>;
    const size_t merge_bytes = sizeof(float) * (NTHREADS / LPK) * GQ * (VPL * LPK * Vec<T>::N);
    const int row_bytes = d * (int)sizeof(T);
    const int tk = row_bytes <= 256 ? 32 : (row_bytes <= 512 ? 16 : 8);
    const size_t ring_bytes = (size_t)STAGES * (2 * tk * row_bytes + 128);
    const size_t smem = merge_bytes > ring_bytes ? merge_bytes : ring_bytes;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    fx_launch_pdl(kern, grid, NTHREADS, smem, s, q, ldq, k, v, bt, tw, ps, pos, tseq, sslot, pa, pm, nh, nkv, d, window, scale,
                                      split_len, n_splits);
    return fx_launch_status();
}

template <typename T, int LPK, int VPL, typename... A>
int launch_split(int gq, A... args)
{
    switch (gq) {
        case 1: return launch_one<T, LPK, VPL, 1>(args...);
        case 2: return launch_one<T, LPK, VPL, 2>(args...);
        case 4: return launch_one<T, LPK, VPL, 4>(args...);
        default: return launch_one<T, LPK, VPL, 8>(args...);
    }
}

template <typename T>
int run(const void* q, long ldq, const void* k_pages, const void* v_pages, int n_pages, const int* block_table,
        int table_width, int page_size, const int* positions, const int* token_seq, const int* seq_slot, void* out,
        long ldo, float* part_acc, float* part_ml, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int window,
        float scale, int split_len, int n_splits, int* status, int* counters, int fresh, int store_new, int write_pages,
        const float* cos_sin, cudaStream_t s)
{
    constexpr int N = Vec<T>::N;
    if (head_dim % N || head_dim > MAX_D || head_dim <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return FX_ERR_SIZE;
    if (ldq % N || (uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16) return FX_ERR_ALIGN;
    if (sizeof(T) == 2) {
        // bfloat16: the tensor-core kernels write the same partial results; the merge below is shared.  The one
        // that streams whole pages by TMA first (head sizes in steps of 64, pages of a multiple of 64 positions).
        int rc_mma = FX_ERR_SIZE;
        if (n_pages > 0) {
            if (n_splits > 32) counters = nullptr;
            rc_mma = fx_decode_split_tma(q, ldq, k_pages, v_pages, n_pages, block_table, table_width, page_size,
                                         positions, token_seq, seq_slot, part_acc, part_ml, n_tokens, n_heads,
                                         n_kv_heads, head_dim, window, scale, split_len, n_splits, status, out, ldo,
                                         counters, fresh, store_new, write_pages, cos_sin, (void*)s);
            if (rc_mma == FX_OK && (counters || n_splits == 1)) return FX_OK;   // merged by the kernel's last blocks
        }
        // only the kernel above rotates and stores the step's own keys and values itself
        if (store_new && rc_mma != FX_OK) return rc_mma;
        if (rc_mma < 0)
            rc_mma = fx_decode_split_mma(q, ldq, k_pages, v_pages, block_table, table_width, page_size, positions,
                                         token_seq, seq_slot, part_acc, part_ml, n_tokens, n_heads, n_kv_heads,
                                         head_dim, window, scale, split_len, n_splits, fresh, (void*)s);
        if (rc_mma == FX_OK) {
            fx_launch_pdl(merge_kernel<T>, dim3(n_tokens, n_heads), 64, 0, s, part_acc, part_ml, positions, (T*)out, ldo,
                          n_heads, head_dim, n_splits, split_len, window);
            return fx_launch_status();
        }
        if (rc_mma > 0) return rc_mma;   // a CUDA error; a refusal (< 0) falls through to the CUDA-core kernel
    }
    if (store_new) return FX_ERR_DTYPE;
    const int group = n_heads / n_kv_heads;
    int gq = 1;
    while (gq < group && gq < MAXQ) gq <<= 1;
    const int chunks = (group + gq - 1) / gq;
    dim3 grid(n_kv_heads * chunks, n_tokens, n_splits);
    if (grid.y > 65535u || grid.z > 65535u) return FX_ERR_SIZE;
    const int vecs = head_dim / N;   // vectors per key
    const T* Q = (const T*)q; const T* K = (const T*)k_pages; const T* V = (const T*)v_pages;
    int rc;
#define FX_GO(LPK, VPL)                                                                                       \
    rc = launch_split<T, LPK, VPL>(gq, grid, s, Q, ldq, K, V, block_table, table_width, page_size, positions, \
                                   token_seq, seq_slot, part_acc, part_ml, n_heads, n_kv_heads, head_dim,    \
                                   window, scale, split_len, n_splits)
    if (vecs <= 4) { FX_GO(4, 1); }
    else if (vecs <= 8) { FX_GO(8, 1); }
    else if (vecs <= 16) { FX_GO(16, 1); }
    else if (vecs <= 32) { FX_GO(16, 2); }
    else { FX_GO(16, 4); }
#undef FX_GO
    if (rc != FX_OK) return rc;
    fx_launch_pdl(merge_kernel<T>, dim3(n_tokens, n_heads), 64, 0, s, part_acc, part_ml, positions, (T*)out, ldo, n_heads, head_dim,
                                                          n_splits, split_len, window);
    return fx_launch_status();
}

}  // namespace

// Scratch: part_acc [n_tokens, n_heads, n_splits, head_dim] and part_ml [n_tokens, n_heads, n_splits, 2], float32.
extern "C" int fx_decode_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, int n_pages,
                                   int dtype, const int* block_table, int table_width, int page_size,
                                   const int* positions, const int* token_seq, const int* seq_slot, void* out, long ldo,
                                   float* part_acc, float* part_ml, int n_tokens, int n_heads, int n_kv_heads,
                                   int head_dim, int window, float scale, int split_len, int n_splits, int* status,
                                   int* counters, int fresh_positions, int store_new, int write_pages,
                                   const float* cos_sin, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (split_len < 0 || n_splits <= 0) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FX_F32)
        return run<float>(q, ldq, k_pages, v_pages, n_pages, block_table, table_width, page_size, positions, token_seq,
                          seq_slot, out, ldo, part_acc, part_ml, n_tokens, n_heads, n_kv_heads, head_dim, window, scale,
                          split_len, n_splits, status, counters, fresh_positions, store_new, write_pages, cos_sin, s);
    if (dtype == FX_BF16)
        return run<bf16>(q, ldq, k_pages, v_pages, n_pages, block_table, table_width, page_size, positions, token_seq,
                         seq_slot, out, ldo, part_acc, part_ml, n_tokens, n_heads, n_kv_heads, head_dim, window, scale,
                         split_len, n_splits, status, counters, fresh_positions, store_new, write_pages, cos_sin, s);
    return FX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Entry point that allocates nothing (declared in no_alloc.h; no counterpart in the
// reference).  Same computation as fx_decode_attention, but the per-split partial
// results live in the fixed array below instead of caller-provided scratch memory.
//
// The array is part of the library's image: every GPU on which the library is used
// holds FX_NOALLOC_SCRATCH_FLOATS * 4 bytes from the moment the library is loaded
// there until the process exits.  Host code cannot use the array's name as a
// pointer (on the host it names a stand-in, not device memory), so the device
// address is asked for once per device with cudaGetSymbolAddress and kept.
static __device__ __align__(256) float fx_noalloc_scratch[FX_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int FX_MAX_DEVICES = 64;
float* g_noalloc_ptr[FX_MAX_DEVICES] = {nullptr};
}  // namespace

extern "C" int fx_decode_attention_noalloc(const void* q, long ldq, const void* k_pages, const void* v_pages, int dtype,
                                           const int* block_table, int table_width, int page_size,
                                           const int* positions, const int* token_seq, const int* seq_slot, void* out,
                                           long ldo, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                           int window, float scale, int split_len, int n_splits, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (split_len < 0 || n_splits <= 0 || n_heads <= 0 || head_dim <= 0) return FX_ERR_SIZE;
    // partial sums [tokens, heads, splits, head_dim] followed by (max, sum) pairs [tokens, heads, splits, 2]
    const long slots = (long)n_tokens * n_heads * n_splits;
    const long need = slots * head_dim + slots * 2;
    if (need > (long)FX_NOALLOC_SCRATCH_FLOATS) return FX_ERR_SCRATCH;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= FX_MAX_DEVICES) return FX_ERR_SIZE;
    if (g_noalloc_ptr[dev] == nullptr) {
        // first call on this device (it is the current one): resolve the array's device address
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, fx_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return FX_ERR_SIZE;
        g_noalloc_ptr[dev] = p;
    }
    float* part_acc = g_noalloc_ptr[dev];
    float* part_ml = part_acc + slots * head_dim;   // offset is a multiple of head_dim floats; only 4-byte access
    cudaStream_t s = (cudaStream_t)stream;
    // Every slot that the merge reads is written by the split kernel of the same call (a split
    // without visible keys writes nothing and the merge skips it by the same rule), so nothing
    // has to be cleared first.  No promise is made about the kernel before this call: the
    // attention kernels read nothing before it has finished.
    if (dtype == FX_F32)
        return run<float>(q, ldq, k_pages, v_pages, 0, block_table, table_width, page_size, positions, token_seq, seq_slot,
                          out, ldo, part_acc, part_ml, n_tokens, n_heads, n_kv_heads, head_dim, window, scale,
                          split_len, n_splits, nullptr, nullptr, 0, 0, 0, nullptr, s);
    if (dtype == FX_BF16)
        return run<bf16>(q, ldq, k_pages, v_pages, 0, block_table, table_width, page_size, positions, token_seq, seq_slot,
                         out, ldo, part_acc, part_ml, n_tokens, n_heads, n_kv_heads, head_dim, window, scale,
                         split_len, n_splits, nullptr, nullptr, 0, 0, 0, nullptr, s);
    return FX_ERR_DTYPE;
}
