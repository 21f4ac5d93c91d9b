// Skinny matrix products for decoding: a few tokens against a whole weight matrix,
//   C[tokens, N] (+)= X[tokens, K] . W[N, K]^T (+ bias),       bfloat16 in, 32-bit sums,
// where the time is the time to stream W from HBM once.  Also the grouped form for
// experts (rows sorted by expert, each expert's matrix streamed once for its few
// tokens) and the gated form that computes silu(gate) * up in the epilogue, so the
// [gate | up] intermediate never reaches memory.
//
// Layout of the work: a block owns 16 output features (one m16 tile of W; in the
// gated form the 16 gate rows and the matching 16 up rows) and all tokens; its 8
// warps split K in chunks of 32, each lane fetching 16 contiguous bytes of a row
// (ld.global.nc, no L1 allocation: every weight byte is used once).  The tensor
// core instruction is mma.sync.m16n8k16 with W as the A operand and 8 tokens as
// the n dimension: at these sizes the kernel is bound by memory, and one warp's
// registers hold its whole working set.  (The 128-row tcgen05 tiles serve the
// prompt-sized products.)  Inside a chunk the k index is permuted the same way for
// W and X, so that each lane's 16 bytes feed two instructions directly.
// The 8 partial sums of a block are added in warp order through shared memory:
// the result does not depend on timing, on the other tokens, or on the grid.
//
// Reference: the reference's CUDA matvec streams quantized rows with one block per
// row (crates/ferrox-cuda/src/gpu.rs:132-189) and fuses the FFN chain for one
// host-chosen expert (gpu.rs:1174-1195); here experts are chosen on the device.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int WARPS = 8;
constexpr int NTHREADS = WARPS * 32;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyArgs {
    const bf16* W; long ldw; long w_group_stride;
    const bf16* X; long ldx; const int* x_rows;
    const void* bias; int bias_dtype;
    void* C; long ldc; int c_dtype; int accumulate;
    int c_transposed;              // store C[n][r] instead of C[r][n] (ldc is then the pitch of a feature's row)
    int n_tokens; int N; int K;
    int gate_up_offset;            // gated form: row of `up` matching gate row i is i + gate_up_offset
    const int* group_offsets;      // grouped form: rows [off[e], off[e+1]) belong to expert e
    const int* active_groups;      // grouped form: the experts that got rows, then -1
    int n_slots;                   // length of active_groups
};

// MODE 0: 16 features per block.  MODE 1 (gated): 16 gate rows and their 16 up rows, out = silu(gate) * up.
// MODE 2: 32 features per block (two tiles of rows), for wide matrices: half as many, fatter blocks.
//
// Grouped form: blockIdx.y walks the list of experts that got rows in steps of gridDim.y, so that a block pays
// its start-up once for several experts.  The weight loads of a pass are issued before the token rows are
// looked up, and in the plain form even before the wait on the kernel that produced X: the weights do not
// depend on it.
template <int NT, int MODE>
__global__ void __launch_bounds__(NTHREADS) skinny_kernel(SkinnyArgs a)
{
    constexpr bool GATED = MODE != 0;   // a second set of 16 rows is streamed beside the first
    constexpr int UNROLL = (GATED ? 4 : 8) / (NT > 2 ? 2 : 1);
    constexpr int RPB = MODE == 2 ? 32 : 16;   // output features per tile
    __shared__ float red[WARPS][GATED ? 2 : 1][NT][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_chunks = a.K >> 5;
    const bool grouped = a.group_offsets != nullptr;
    const int tiles_n = (a.N + RPB - 1) / RPB;
    const int total = tiles_n * (grouped ? a.n_slots : 1);

    // One pass = UNROLL chunks of this warp, of the 16 (+16) rows of a tile, into registers.
    uint4 wa[UNROLL], wb[UNROLL], ua[UNROLL], ub[UNROLL];
    auto load_pass = [&](const bf16* W, int n0, int i0) {
        // rows of W this lane reads: g and g+8 of the tile (clamped; masked at the store)
        const long o0 = (long)min(n0 + g, a.N - 1) * a.ldw + t * 8;
        const long o1 = (long)min(n0 + g + 8, a.N - 1) * a.ldw + t * 8;
        long p0 = 0, p1 = 0;   // the second set of rows
        if (MODE == 1) { p0 = o0 + (long)a.gate_up_offset * a.ldw; p1 = o1 + (long)a.gate_up_offset * a.ldw; }
        if (MODE == 2) {
            p0 = (long)min(n0 + 16 + g, a.N - 1) * a.ldw + t * 8;
            p1 = (long)min(n0 + 24 + g, a.N - 1) * a.ldw + t * 8;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int c = warp + WARPS * (i0 + u);
            if (c < n_chunks) {
                wa[u] = ldg_stream(W + o0 + c * 32);
                wb[u] = ldg_stream(W + o1 + c * 32);
                if (GATED) { ua[u] = ldg_stream(W + p0 + c * 32); ub[u] = ldg_stream(W + p1 + c * 32); }
            }
        }
    };
    // the matrix a tile reads (nullptr: no such tile)
    auto tile_matrix = [&](int idx) -> const bf16* {
        if (idx >= total) return nullptr;
        if (!grouped) return a.W;
        const int e = a.active_groups[idx / tiles_n];
        return e < 0 ? nullptr : a.W + (long)e * a.w_group_stride;
    };

    // The first pass of the first tile: in the plain form W is a weight matrix and does not depend on the
    // kernel before this one.  (With transposed output the roles are swapped and W holds activations.)
    bool have_first = false;
    if (!grouped && !a.c_transposed && (int)blockIdx.x < total) { load_pass(a.W, (blockIdx.x % tiles_n) * RPB, 0); have_first = true; }
    fx_pdl_wait();

    for (int idx = blockIdx.x; idx < total; idx += gridDim.x) {
        const int slot = idx / tiles_n, n0 = (idx - slot * tiles_n) * RPB;
        int row_begin = 0, row_end = a.n_tokens;
        const bf16* W = a.W;
        if (grouped) {
            const int e = a.active_groups[slot];
            if (e < 0) break;   // the list is compact: nothing after the first -1
            W += (long)e * a.w_group_stride;
            if (!have_first) { load_pass(W, n0, 0); have_first = true; }
            row_begin = a.group_offsets[e];
            row_end = a.group_offsets[e + 1];
        } else if (!have_first) {
            load_pass(W, n0, 0);
            have_first = true;
        }
        for (int tok0 = row_begin; tok0 < row_end; tok0 += 8 * NT) {
            const bool last_tokens = tok0 + 8 * NT >= row_end;
            // token rows this lane reads for the B operand: token g of each n-tile
            const bf16* xp[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int r = tok0 + j * 8 + g;
                xp[j] = r < row_end ? a.X + (long)(a.x_rows ? a.x_rows[r] : r) * a.ldx + t * 8 : nullptr;
            }
            float acc[GATED ? 2 : 1][NT][4];
#pragma unroll
            for (int s = 0; s < (GATED ? 2 : 1); ++s)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[s][j][i] = 0.f;

            // Chunk c of K belongs to warp c % 8, so that the 8 warps read 512 contiguous bytes of a row
            // together and share the chunks evenly whatever K is; a warp issues the loads of UNROLL of its
            // chunks before it uses the first.
            for (int i0 = 0; warp + WARPS * i0 < n_chunks; i0 += UNROLL) {
                if (!(have_first && i0 == 0)) load_pass(W, n0, i0);
                have_first = false;
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int c = warp + WARPS * (i0 + u);
                    if (c >= n_chunks) break;
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                        if (xp[j]) xv = *reinterpret_cast<const uint4*>(xp[j] + c * 32);
                        mma16816(acc[0][j], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
                        mma16816(acc[0][j], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
                        if (GATED) {
                            mma16816(acc[1][j], ua[u].x, ub[u].x, ua[u].y, ub[u].y, xv.x, xv.y);
                            mma16816(acc[1][j], ua[u].z, ub[u].z, ua[u].w, ub[u].w, xv.z, xv.w);
                        }
                    }
                }
            }
            have_first = false;
            if (last_tokens) {
                // the weights of this block's next tile start to arrive while this tile is reduced and stored
                const int nidx = idx + gridDim.x;
                const bf16* Wn = tile_matrix(nidx);
                if (Wn) { load_pass(Wn, (nidx % tiles_n) * RPB, 0); have_first = true; }
            }
            // partial sums of this warp -> shared memory: [row g | g+8][token 2t | 2t+1]
            __syncthreads();  // the previous reduction has been read
#pragma unroll
            for (int s = 0; s < (GATED ? 2 : 1); ++s)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    red[warp][s][j][g][2 * t] = acc[s][j][0];
                    red[warp][s][j][g][2 * t + 1] = acc[s][j][1];
                    red[warp][s][j][g + 8][2 * t] = acc[s][j][2];
                    red[warp][s][j][g + 8][2 * t + 1] = acc[s][j][3];
                }
            __syncthreads();
            // 16 features x 8*NT tokens: consecutive threads take consecutive features of one token
            for (int o = threadIdx.x; o < 16 * 8 * NT; o += NTHREADS) {
                const int f = o & 15, tk = o >> 4;
                const int j = tk >> 3, tn = tk & 7;
                const int r = tok0 + tk, n = n0 + f;
                if (r >= row_end || n >= a.N) continue;
                float v = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    v += red[w][0][j][f][tn];
                    if (GATED) up += red[w][1][j][f][tn];
                }
                if (a.bias) v += load_any(a.bias, a.bias_dtype, n);
                if (MODE == 1) v = v / (1.0f + expf(-v)) * up;
                auto store = [&](int col, float val) {
                    const long at = a.c_transposed ? (long)col * a.ldc + r : (long)r * a.ldc + col;
                    if (a.c_dtype == FX_F32) {
                        float* c = reinterpret_cast<float*>(a.C) + at;
                        *c = a.accumulate ? *c + val : val;
                    } else {
                        bf16* c = reinterpret_cast<bf16*>(a.C) + at;
                        *c = __float2bfloat16_rn(a.accumulate ? __bfloat162float(*c) + val : val);
                    }
                };
                store(n, v);
                if (MODE == 2 && n + 16 < a.N) {
                    if (a.bias) up += load_any(a.bias, a.bias_dtype, n + 16);
                    store(n + 16, up);
                }
            }
        }
    }
}

template <int MODE>
int launch_nt(const SkinnyArgs& a, int max_tokens_per_group, dim3 grid, cudaStream_t s)
{
    if (max_tokens_per_group <= 8) fx_launch_pdl(skinny_kernel<1, MODE>, grid, NTHREADS, 0, s, a);
    else if (max_tokens_per_group <= 16) fx_launch_pdl(skinny_kernel<2, MODE>, grid, NTHREADS, 0, s, a);
    else fx_launch_pdl(skinny_kernel<4, MODE>, grid, NTHREADS, 0, s, a);
    return fx_launch_status();
}

}  // namespace

// Plain / grouped, optionally gated.  bfloat16 X and W; C bfloat16 or float32.
//   gated: W holds gate rows [0, N) and up rows [gate_up_offset, gate_up_offset + N); C gets silu(gate) * up.
//   grouped: group_offsets [G+1] and active_groups [n_slots] (expert per slot, -1 = unused) on the device;
//            tokens_hint = most rows one group can have (chooses how many tokens a pass covers).
// Refuses (FX_ERR_SIZE / FX_ERR_ALIGN) K not a multiple of 32 and rows not 16-byte aligned.
extern "C" int fx_gemm_skinny(const void* X, long ldx, const int* x_rows, const void* W, long ldw, long w_group_stride,
                              const void* bias, int bias_dtype, void* C, int c_dtype, long ldc, int accumulate,
                              int n_tokens, int N, int K, int gated, int gate_up_offset,
                              const int* group_offsets, const int* active_groups, int n_slots, int tokens_hint,
                              int c_transposed, void* stream)
{
    if (n_tokens <= 0 || N <= 0) return FX_OK;
    if (K % 32 != 0 || K <= 0) return FX_ERR_SIZE;
    if (ldw % 8 || ldx % 8 || w_group_stride % 8 || (uintptr_t)W % 16 || (uintptr_t)X % 16) return FX_ERR_ALIGN;
    if (c_dtype != FX_F32 && c_dtype != FX_BF16) return FX_ERR_DTYPE;
    SkinnyArgs a;
    a.W = (const bf16*)W; a.ldw = ldw; a.w_group_stride = w_group_stride;
    a.X = (const bf16*)X; a.ldx = ldx; a.x_rows = x_rows;
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.C = C; a.ldc = ldc; a.c_dtype = c_dtype; a.accumulate = accumulate; a.c_transposed = c_transposed;
    a.n_tokens = n_tokens; a.N = N; a.K = K; a.gate_up_offset = gate_up_offset;
    a.group_offsets = group_offsets; a.active_groups = active_groups; a.n_slots = n_slots;
    // grouped: one block row per expert slot (many short blocks hide each other's start-up better than
    // few long ones; measured)
    const int slots = group_offsets ? n_slots : 1;
    // wide matrices: 32 features per block, so that half as many blocks pay the start-up latency
    // (also where 16-feature tiles would be a little more than one round of resident blocks: one round of fat
    // blocks beats a round and a bit of thin ones)
    const long resident = 2L * fx_sm_count();   // two blocks an SM
    const bool two_tiles = !gated && (fx_cdiv(N, 32) * slots >= resident || fx_cdiv(N, 16) * slots > resident);
    // Two resident blocks per SM walk the tiles (expert slot major, then feature tile); a block fetches its
    // next tile's weights while it finishes the current one.
    long tiles = fx_cdiv(N, two_tiles ? 32 : 16) * (long)slots;
    dim3 grid((unsigned)(tiles < resident ? tiles : resident), 1);
    const int hint = group_offsets ? tokens_hint : n_tokens;
    cudaStream_t s = (cudaStream_t)stream;
    if (gated) return launch_nt<1>(a, hint, grid, s);
    return two_tiles ? launch_nt<2>(a, hint, grid, s) : launch_nt<0>(a, hint, grid, s);
}
