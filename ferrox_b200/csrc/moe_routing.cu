// Routing of tokens to experts: softmax over all experts, top-k, optional
// renormalisation; then the bookkeeping that sorts (token, rank) pairs by expert so
// that each expert's rows are contiguous for the grouped matrix products.
#include "common.cuh"
#include "api.h"

namespace {

// One warp per token.  p = softmax(logits) over ALL experts (max-subtracted), the k
// largest p are kept in descending order, on equal p the lowest expert index wins,
// and the weights are the kept p, divided by their sum when `renorm` is set
// (reference: crates/ferrox-moe/src/lib.rs:333-355; lowest-index tie-break as in
// its GPU kernel, crates/ferrox-metal/src/gpu.rs:686-699).
// In shared memory a probability is kept as its bit pattern plus one (probabilities are >= 0, so the patterns
// order like the values) and 0 once taken: the warp's maximum and the lowest index that holds it are two integer
// warp reductions instead of two chains of shuffles.  `counts` (optional): counts[e] += 1 for each kept expert.
__device__ __forceinline__ void route_token(const float* __restrict__ lg, float* p, int lane, int t, int n_experts,
                                            int top_k, int renorm, int* __restrict__ ids, float* __restrict__ weights,
                                            int* __restrict__ counts = nullptr, int* ids_shared = nullptr)
{
    uint32_t* pb = reinterpret_cast<uint32_t*>(p);
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, lg[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) { const float v = expf(lg[e] - mx); pb[e] = __float_as_uint(v) + 1u; sum += v; }
    sum = warp_sum(sum);
    __syncwarp();
    // up to 32 kept experts stay in registers (lane k holds the k-th) and are written once, side by side
    const bool in_regs = top_k <= 32;
    float kept = 0.f, mine_w = 0.f;
    int mine_e = 0;
    for (int k = 0; k < top_k; ++k) {
        uint32_t best = 0u; int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const uint32_t v = pb[e];
            if (v > best) { best = v; best_e = e; }  // ascending e: the first maximum stays
        }
        const uint32_t top = __reduce_max_sync(0xffffffffu, best);
        const int win = __reduce_min_sync(0xffffffffu, best == top ? best_e : 0x7fffffff);
        const float w = __uint_as_float(top - 1u) / sum;
        if (lane == 0) {
            pb[win] = 0u;
            if (!in_regs) {
                ids[(long)t * top_k + k] = win; weights[(long)t * top_k + k] = w;
                if (ids_shared) ids_shared[t * top_k + k] = win;
                if (counts) atomicAdd(&counts[win], 1);
            }
        }
        if (lane == k) { mine_w = w; mine_e = win; }
        kept += w;
        __syncwarp();
    }
    if (in_regs) {
        if (lane < top_k) {
            ids[(long)t * top_k + lane] = mine_e;
            weights[(long)t * top_k + lane] = renorm ? mine_w / kept : mine_w;
            if (ids_shared) ids_shared[t * top_k + lane] = mine_e;
            if (counts) atomicAdd(&counts[mine_e], 1);
        }
    } else if (renorm) {
        __syncwarp();
        for (int k = lane; k < top_k; k += 32) weights[(long)t * top_k + k] /= kept;
    }
}

__global__ void router_topk_kernel(const float* __restrict__ logits, long ld, int n_tokens, int n_experts, int top_k,
                                   int renorm, int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ counts)
{
    extern __shared__ float smem[];  // [warps][n_experts]
    fx_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    route_token(logits + (long)t * ld, smem + (long)warp * n_experts, lane, t, n_experts, top_k, renorm, ids,
                weights, counts);
}

// Routing and bookkeeping of a small step in ONE block: top-k per token (a warp
// each), then counts, offsets, the list of experts that got rows, and the placement
// of every (token, rank) pair, all in shared memory.  `p_scratch`: [warps][n_experts]
// floats, `counts`: 2 * n_experts + 1 ints, both in shared memory.
__device__ __forceinline__ void route_in_block(const float* lg, long ld, float* p_scratch, int* counts, int n_warps,
                                               int n_tokens, int n_experts, int top_k, int renorm,
                                               int* __restrict__ ids, float* __restrict__ weights,
                                               int* __restrict__ offsets, int* __restrict__ src_token,
                                               int* __restrict__ inv_perm, int* __restrict__ active, int n_slots,
                                               int* ids_s = nullptr, int* src_s = nullptr)
{
    // ids_s, src_s (optional, shared memory, n_tokens * top_k ints each): the block keeps what it chose and where it
    // put it beside the copies in global memory, so that it (and its caller) need not read those back
    int* offs = counts + n_experts;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int t = warp; t < n_tokens; t += n_warps) {
        route_token(lg + (long)t * ld, p_scratch + (long)warp * n_experts, lane, t, n_experts, top_k, renorm, ids,
                    weights, counts, ids_s);
        __syncwarp();
    }
    __syncthreads();  // ids written by this block are visible to it after the barrier
    const int* ids_r = ids_s ? ids_s : ids;
    const int n = n_tokens * top_k;
    if (warp == 0) {
        // offsets = running sum of the counts, 32 experts a pass; the experts with rows, in ascending order
        int run = 0, n_active = 0;
        for (int e0 = 0; e0 < n_experts; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < n_experts ? counts[e] : 0;
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
            const int off = run + incl - c;
            if (e < n_experts) { offs[e] = off; offsets[e] = off; counts[e] = 0; }  // the count becomes the cursor
            const unsigned has = __ballot_sync(0xffffffffu, c > 0);
            if (active && c > 0) {
                const int slot = n_active + __popc(has & ((1u << lane) - 1u));
                if (slot < n_slots) active[slot] = e;
            }
            n_active += __popc(has);
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) offsets[n_experts] = run;
        if (active) for (int i = min(n_active, n_slots) + lane; i < n_slots; i += 32) active[i] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids_r[i];
        const int r = offs[e] + atomicAdd(&counts[e], 1);
        src_token[r] = i / top_k;
        if (src_s) src_s[r] = i / top_k;
        inv_perm[i] = r;
    }
}

constexpr int SMALL_WARPS = 32;
__global__ void __launch_bounds__(SMALL_WARPS * 32) route_small_kernel(
    const float* __restrict__ logits, long ld, int n_tokens, int n_experts, int top_k, int renorm,
    int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ offsets, int* __restrict__ src_token, int* __restrict__ inv_perm,
    int* __restrict__ active, int n_slots)
{
    extern __shared__ float smem[];  // [SMALL_WARPS][n_experts] floats, then 2 * n_experts + 1 ints
    fx_pdl_wait();
    int* counts = reinterpret_cast<int*>(smem + (long)SMALL_WARPS * n_experts);
    route_in_block(logits, ld, smem, counts, SMALL_WARPS, n_tokens, n_experts, top_k, renorm, ids, weights, offsets,
                   src_token, inv_perm, active, n_slots);
}

// What stands between the norm and the experts in a decode step of a few tokens, in ONE launch of one cluster of
// FUSED_CTAS blocks instead of three dependent launches (each costs a few microseconds of waiting for the one before):
//   1. the router's product: the blocks share the rows of W (a warp a row: its dot products with every token, 32-bit
//      sums); every warp puts its logits into the first block's shared memory (DSMEM) and into logits_out, which
//      later kernels read for rows beyond the experts' (a gate's logit);
//   2. after the cluster's barrier the first block routes as route_small_kernel does;
//   3. (optional) and copies each (token, rank) pair's row of x into expert order (xp_out), for kernels that want
//      an expert's rows side by side.
// n_route >= n_experts rows of W; the first n_experts are routed over.  (The norm before it was taken in as well,
// measured and left out: the shared expert, which needs only the normed rows, would wait for the whole kernel.)
struct FusedArgs {
    const bf16* X; long ldx;                 // the tokens' rows
    const bf16* W; long ldw;
    int n_tokens, n_route, n_experts, hidden, top_k, renorm;
    float* logits_out; long ldl;
    int* ids; float* weights; int* offsets; int* src_token; int* inv_perm; int* active; int n_slots;
    bf16* xp_out; long ldxp;                 // rows in expert order (may be null)
};

constexpr int FUSED_CTAS = 8, FUSED_WARPS = 8, FUSED_PASS = 8;   // a pass: 8 x 16 bytes a lane = 2,048 elements a warp
template <int NT>
__global__ void __launch_bounds__(FUSED_WARPS * 32) route_fused_kernel(FusedArgs a)
{
    // every block: the tokens' rows [NT][hidden] bfloat16; the first block behind them: logits [NT][n_route],
    // p [FUSED_WARPS][n_experts], 2 n_experts + 1 ints
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* x_s = reinterpret_cast<bf16*>(smem_raw);
    float* lg_s = reinterpret_cast<float*>(smem_raw + (size_t)NT * a.hidden * sizeof(bf16));
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hidden = a.hidden, n_route = a.n_route, n_tokens = a.n_tokens;
    const int rows_per_cta = (n_route + FUSED_CTAS - 1) / FUSED_CTAS;
    const int row_begin = rank * rows_per_cta, row_end = min(n_route, row_begin + rows_per_cta);
    const int n_vec = hidden >> 3;                       // 16-byte pieces of a row
    // the first block's logits as every block of the cluster addresses them
    uint32_t lg_remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(lg_remote) : "r"((uint32_t)__cvta_generic_to_shared(lg_s)), "r"(0));

    uint4 wv[FUSED_PASS];
    auto load_w = [&](int row, int v0) {
#pragma unroll
        for (int u = 0; u < FUSED_PASS; ++u) {
            const int v = v0 + u * 32 + lane;
            wv[u] = v < n_vec ? *reinterpret_cast<const uint4*>(a.W + (long)row * a.ldw + (long)v * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    // the weights do not depend on the kernel before this one: the first pass is on its way before the wait
    if (row_begin + warp < row_end) load_w(row_begin + warp, 0);
    fx_pdl_wait();
    // the tokens' rows into shared memory, all loads of a thread in flight together (rows beyond the step's: zeros)
    for (int i = threadIdx.x; i < NT * n_vec; i += FUSED_WARPS * 32) {
        const int t = i / n_vec, v = i - t * n_vec;
        reinterpret_cast<uint4*>(x_s)[i] = t < n_tokens ? *reinterpret_cast<const uint4*>(a.X + (long)t * a.ldx + (long)v * 8)
                                                        : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    for (int row = row_begin + warp; row < row_end; row += FUSED_WARPS) {
        float acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.f;
        for (int v0 = 0; v0 < n_vec; v0 += FUSED_PASS * 32) {
            if (!(row == row_begin + warp && v0 == 0)) load_w(row, v0);
#pragma unroll
            for (int u = 0; u < FUSED_PASS; ++u) {
                const int v = min(v0 + u * 32 + lane, n_vec - 1);   // (beyond the row the weights are zeros)
                const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
                float2 wf[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) wf[i] = __bfloat1622float2(w2[i]);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const uint4 xv = reinterpret_cast<const uint4*>(x_s)[t * n_vec + v];
                    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 b = __bfloat1622float2(x2[i]);
                        acc[t] = fmaf(wf[i].x, b.x, acc[t]);
                        acc[t] = fmaf(wf[i].y, b.y, acc[t]);
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == 0 && t < n_tokens) {
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(lg_remote + 4u * (uint32_t)(t * n_route + row)), "f"(v) : "memory");
                a.logits_out[(long)t * a.ldl + row] = v;
            }
        }
    }
    // every block's logits are in the first block's shared memory after the cluster's barrier
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank != 0) return;
    float* p_scratch = lg_s + (long)NT * n_route;
    int* counts = reinterpret_cast<int*>(p_scratch + (long)FUSED_WARPS * a.n_experts);
    int* ids_s = counts + 2 * a.n_experts + 1;      // [NT * top_k], then src_s [NT * top_k]
    int* src_s = ids_s + NT * a.top_k;
    route_in_block(lg_s, n_route, p_scratch, counts, FUSED_WARPS, n_tokens, a.n_experts, a.top_k, a.renorm, a.ids, a.weights,
                   a.offsets, a.src_token, a.inv_perm, a.active, a.n_slots, ids_s, src_s);
    if (a.xp_out) {
        // the rows in expert order, out of shared memory: a warp a row, 16 bytes a lane and pass
        __syncthreads();
        const int n = n_tokens * a.top_k;
        for (int r = warp; r < n; r += FUSED_WARPS) {
            const uint4* src = reinterpret_cast<const uint4*>(x_s) + (long)src_s[r] * n_vec;
            uint4* dst = reinterpret_cast<uint4*>(a.xp_out + (long)r * a.ldxp);
#pragma unroll 4
            for (int v = lane; v < n_vec; v += 32) dst[v] = src[v];
        }
    }
}

// counts[e] = number of (token, rank) pairs routed to e.
__global__ void count_kernel(const int* __restrict__ ids, int n, int n_experts, int* __restrict__ counts)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
}

// offsets = exclusive prefix sum of counts ([E+1]); cursors reset to 0.
// active[slot] lists the experts that got at least one row, then -1 up to n_slots.
__global__ void scan_kernel(const int* __restrict__ counts, int n_experts, int* __restrict__ offsets,
                            int* __restrict__ cursors, int* __restrict__ active, int n_slots)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int run = 0, n_active = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = run; run += counts[e]; cursors[e] = 0;
            if (active && counts[e] > 0 && n_active < n_slots) active[n_active++] = e;
        }
        offsets[n_experts] = run;
        if (active) for (int i = n_active; i < n_slots; ++i) active[i] = -1;
    }
}

// Place pair i in its expert's segment.  The place inside the segment follows the
// order in which threads arrive; every row is computed alone and read back through
// inv_perm, so results do not depend on it.
__global__ void place_kernel(const int* __restrict__ ids, int n, int n_experts, int top_k,
                             const int* __restrict__ offsets, int* __restrict__ cursors,
                             int* __restrict__ src_token, int* __restrict__ inv_perm)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int e = ids[i];
        if (e < 0 || e >= n_experts) { inv_perm[i] = 0; continue; }
        const int r = offsets[e] + atomicAdd(&cursors[e], 1);
        src_token[r] = i / top_k;
        inv_perm[i] = r;
    }
}

// scan_kernel and place_kernel in one: every block sums the counts before its experts itself (one warp, a run of
// experts per lane), block 0 also writes the offsets (and the list of experts with rows); cursors start at zero.
constexpr int SCAN_MAX_EXPERTS = 4096;
__global__ void scan_place_kernel(const int* __restrict__ ids, int n, int n_experts, int top_k,
                                  const int* __restrict__ counts, int* __restrict__ cursors, int* __restrict__ offsets,
                                  int* __restrict__ src_token, int* __restrict__ inv_perm, int* __restrict__ active, int n_slots)
{
    __shared__ int offs[SCAN_MAX_EXPERTS + 1];
    fx_pdl_wait();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x, per = (n_experts + 31) / 32;
        const int e0 = min(lane * per, n_experts), e1 = min(e0 + per, n_experts);
        int mine = 0;
        for (int e = e0; e < e1; ++e) mine += counts[e];
        int before = mine;                         // inclusive scan over the lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, before, o); if (lane >= o) before += v; }
        int run = before - mine;
        for (int e = e0; e < e1; ++e) { offs[e] = run; run += counts[e]; }
        if (lane == 31) offs[n_experts] = before;
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) offsets[e] = offs[e];
        if (active && threadIdx.x == 0) {
            int n_active = 0;
            for (int e = 0; e < n_experts; ++e)
                if (offs[e + 1] > offs[e] && n_active < n_slots) active[n_active++] = e;
            for (int i = n_active; i < n_slots; ++i) active[i] = -1;
        }
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int e = ids[i];
        if (e < 0 || e >= n_experts) { inv_perm[i] = 0; continue; }
        const int r = offs[e] + atomicAdd(&cursors[e], 1);
        src_token[r] = i / top_k;
        inv_perm[i] = r;
    }
}

}  // namespace

extern "C" int fx_router_topk(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids,
                              float* weights, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (top_k <= 0 || top_k > n_experts || n_experts > 4096) return FX_ERR_SIZE;
    const int warps = 4;
    const size_t smem = (size_t)warps * n_experts * sizeof(float);
    if (smem > 48 * 1024) return FX_ERR_SIZE;
    router_topk_kernel<<<(unsigned)fx_cdiv(n_tokens, warps), warps * 32, smem, (cudaStream_t)stream>>>(
        logits, ld, n_tokens, n_experts, top_k, renorm, ids, weights, nullptr);
    return fx_launch_status();
}

// fx_router_topk and fx_moe_align of a step of any size in two kernels (and a memset): the top-k kernel counts the
// rows of every expert as it chooses them, the placing kernel sums the counts itself.  scratch: 2 * n_experts ints.
extern "C" int fx_route(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids,
                        float* weights, int* scratch, int* offsets, int* src_token, int* inv_perm, int* active,
                        int n_slots, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (top_k <= 0 || top_k > n_experts || n_experts > SCAN_MAX_EXPERTS) return FX_ERR_SIZE;
    const int warps = 4;
    const size_t smem = (size_t)warps * n_experts * sizeof(float);
    if (smem > 48 * 1024) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int) * 2 * n_experts, s);
    if (e != cudaSuccess) return (int)e;
    fx_launch_pdl(router_topk_kernel, (unsigned)fx_cdiv(n_tokens, warps), warps * 32, smem, s,
                  logits, ld, n_tokens, n_experts, top_k, renorm, ids, weights, scratch);
    const int n = n_tokens * top_k;
    int blocks = (int)fx_cdiv(n, 256);
    if (blocks > fx_sm_count() * 4L) blocks = fx_sm_count() * 4L;
    fx_launch_pdl(scan_place_kernel, blocks, 256, 0, s, ids, n, n_experts, top_k, scratch, scratch + n_experts, offsets,
                  src_token, inv_perm, active, n_slots);
    return fx_launch_status();
}

// Routing of at most 1024 tokens in one launch (see route_small_kernel).
extern "C" int fx_route_small(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids,
                              float* weights, int* offsets, int* src_token, int* inv_perm, int* active, int n_slots,
                              void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (top_k <= 0 || top_k > n_experts || n_tokens > 1024) return FX_ERR_SIZE;
    const size_t smem = (size_t)SMALL_WARPS * n_experts * sizeof(float) + (2 * (size_t)n_experts + 1) * sizeof(int);
    if (smem > 48 * 1024) return FX_ERR_SIZE;
    fx_launch_pdl(route_small_kernel, 1, SMALL_WARPS * 32, smem, (cudaStream_t)stream,
        logits, ld, n_tokens, n_experts, top_k, renorm, ids, weights, offsets, src_token, inv_perm, active, n_slots);
    return fx_launch_status();
}

template <int NT>
static int launch_route_fused(size_t smem, cudaStream_t s, const FusedArgs& a)
{
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(route_fused_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(FUSED_CTAS);
    cfg.blockDim = dim3(FUSED_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = FUSED_CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_fx_pdl_enabled ? 2 : 1;
    cudaLaunchKernelEx(&cfg, route_fused_kernel<NT>, a);
    return fx_launch_status();
}

// One launch for what stands between the norm and the experts in a step of at most 8 tokens (see route_fused_kernel).
// X [n_tokens, hidden] and W [n_route, hidden] bfloat16; logits [n_tokens, n_route] 32-bit; the routing outputs as
// fx_route_small; xp_out (optional) [n_tokens * top_k, hidden] the rows in expert order.  Rows of a multiple of 8
// elements, 16-byte aligned.  Refuses other sizes (FX_ERR_SIZE / FX_ERR_ALIGN): the caller then runs the separate kernels.
extern "C" int fx_route_fused(const void* X, long ldx, const void* W, long ldw, int n_tokens, int n_route,
                              int n_experts, int hidden, int top_k, int renorm, float* logits, long ldl, int* ids,
                              float* weights, int* offsets, int* src_token, int* inv_perm, int* active, int n_slots,
                              void* xp_out, long ldxp, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (n_tokens > 8 || top_k <= 0 || top_k > n_experts || top_k > 64 || n_experts > n_route || n_route > 1024 || hidden <= 0)
        return FX_ERR_SIZE;
    if (hidden % 8 || ldw % 8 || (uintptr_t)W % 16 || ldx % 8 || (uintptr_t)X % 16) return FX_ERR_ALIGN;
    if (xp_out && (ldxp % 8 || (uintptr_t)xp_out % 16)) return FX_ERR_ALIGN;
    const int nt = n_tokens <= 1 ? 1 : n_tokens <= 2 ? 2 : n_tokens <= 4 ? 4 : 8;
    const size_t smem = (size_t)nt * hidden * sizeof(bf16) + ((size_t)nt * n_route + (size_t)FUSED_WARPS * n_experts) * sizeof(float) +
                        (2 * (size_t)n_experts + 1 + 2 * (size_t)nt * top_k) * sizeof(int);
    if (smem > 200 * 1024) return FX_ERR_SIZE;
    FusedArgs a;
    a.X = (const bf16*)X; a.ldx = ldx; a.W = (const bf16*)W; a.ldw = ldw;
    a.n_tokens = n_tokens; a.n_route = n_route; a.n_experts = n_experts; a.hidden = hidden; a.top_k = top_k; a.renorm = renorm;
    a.logits_out = logits; a.ldl = ldl; a.ids = ids; a.weights = weights; a.offsets = offsets; a.src_token = src_token;
    a.inv_perm = inv_perm; a.active = active; a.n_slots = n_slots; a.xp_out = (bf16*)xp_out; a.ldxp = ldxp;
    cudaStream_t s = (cudaStream_t)stream;
    switch (nt) {
        case 1: return launch_route_fused<1>(smem, s, a);
        case 2: return launch_route_fused<2>(smem, s, a);
        case 4: return launch_route_fused<4>(smem, s, a);
        default: return launch_route_fused<8>(smem, s, a);
    }
}

// scratch: 2 * n_experts ints (counts, cursors).  Outputs: offsets [E+1],
// src_token [n_tokens * top_k] (row of the sorted order -> token it reads),
// inv_perm [n_tokens * top_k] (pair -> its row in the sorted order); optionally
// active [n_slots]: the experts with rows, then -1 (n_slots >= min(n_experts, n_tokens * top_k)).
extern "C" int fx_moe_align(const int* ids, int n_tokens, int top_k, int n_experts, int* scratch, int* offsets,
                            int* src_token, int* inv_perm, int* active, int n_slots, void* stream)
{
    const int n = n_tokens * top_k;
    if (n <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int) * 2 * n_experts, s);
    if (e != cudaSuccess) return (int)e;
    int blocks = (int)fx_cdiv(n, 256);
    if (blocks > fx_sm_count() * 4L) blocks = fx_sm_count() * 4L;
    count_kernel<<<blocks, 256, 0, s>>>(ids, n, n_experts, scratch);
    scan_kernel<<<1, 32, 0, s>>>(scratch, n_experts, offsets, scratch + n_experts, active, n_slots);
    place_kernel<<<blocks, 256, 0, s>>>(ids, n, n_experts, top_k, offsets, scratch + n_experts, src_token, inv_perm);
    return fx_launch_status();
}
