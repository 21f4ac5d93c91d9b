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
                                            int* __restrict__ counts = nullptr)
{
    uint32_t* pb = reinterpret_cast<uint32_t*>(p);
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, lg[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) { const float v = expf(lg[e] - mx); pb[e] = __float_as_uint(v) + 1u; sum += v; }
    sum = warp_sum(sum);
    __syncwarp();
    float kept = 0.f;
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
            ids[(long)t * top_k + k] = win; weights[(long)t * top_k + k] = w; pb[win] = 0u;
            if (counts) atomicAdd(&counts[win], 1);
        }
        kept += w;
        __syncwarp();
    }
    if (renorm) {
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
// of every (token, rank) pair, all in shared memory.
constexpr int SMALL_WARPS = 32;
__global__ void __launch_bounds__(SMALL_WARPS * 32) route_small_kernel(
    const float* __restrict__ logits, long ld, int n_tokens, int n_experts, int top_k, int renorm,
    int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ offsets, int* __restrict__ src_token, int* __restrict__ inv_perm,
    int* __restrict__ active, int n_slots)
{
    extern __shared__ float smem[];  // [SMALL_WARPS][n_experts] floats, then 2 * n_experts + 1 ints
    fx_pdl_wait();
    int* counts = reinterpret_cast<int*>(smem + (long)SMALL_WARPS * n_experts);
    int* offs = counts + n_experts;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    for (int t = warp; t < n_tokens; t += SMALL_WARPS) {
        route_token(logits + (long)t * ld, smem + (long)warp * n_experts, lane, t, n_experts, top_k, renorm, ids,
                    weights);
        __syncwarp();
    }
    __syncthreads();  // ids written by this block are visible to it after the barrier
    const int n = n_tokens * top_k;
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, n_active = 0;
        for (int e = 0; e < n_experts; ++e) {
            offs[e] = run; offsets[e] = run; run += counts[e];
            if (active && counts[e] > 0 && n_active < n_slots) active[n_active++] = e;
            counts[e] = 0;  // becomes the cursor
        }
        offsets[n_experts] = run;
        if (active) for (int i = n_active; i < n_slots; ++i) active[i] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids[i];
        const int r = offs[e] + atomicAdd(&counts[e], 1);
        src_token[r] = i / top_k;
        inv_perm[i] = r;
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
