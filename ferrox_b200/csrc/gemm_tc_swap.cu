// Matrix products with few rows of X per weight matrix, on the 5th-generation tensor cores, with the
// operands' roles swapped:
//   C[r, n] (+)= sum_k X[r, k] W[n, k] (+ bias[n])        bfloat16 in, 32-bit sums in tensor memory
// The 128 lanes of a tcgen05 tile are 128 output features (rows of W), its columns are the tokens (rows
// of X): any multiple of 16 up to TNB.  A product of 136 tokens with an expert's matrix thus costs 144
// columns, where the 128-row tiles of gemm_tc.cu would cost 256 rows; a decode step of 40 tokens costs
// 48 columns.  Plain, gated (two accumulators: the gate rows and the up rows of the same features;
// silu(gate) * up in the epilogue) and grouped by expert (rows of X sorted by expert, tile (expert,
// token tile) found on the device), as in gemm_tc.cu.
//
// One CTA takes one tile of 128 features x up to TNB tokens at a time (persistent, one CTA per SM).
// Warp 0: TMA loads of 128 x 64 slices of W (two of them when gated) and a TNB x 64 slice of X per
// stage.  Warp 1: tcgen05.mma, accumulators double-buffered in tensor memory where two sets fit.  Warps 2-5: epilogue;
// a thread owns one feature and walks the tokens, so that a warp's store of one token is 32
// consecutive features.  Every wait is bounded (status code 3 on time-out).
//
// Shapes: any M, N; K a multiple of 8; 16-byte aligned pointers and row pitches.
//
// Reference: the product is crates/ferrox-core/src/matmul.rs:18-58, experts
// crates/ferrox-moe/src/lib.rs:619-659; the reference has no counterpart of the tiling.
#include "tc_common.cuh"
#include "api.h"

namespace {

using namespace fxtc;

constexpr int BF = 128;          // features per tile = TMEM lanes
constexpr int BK = 64;           // bfloat16 elements per stage along K = one 128-byte swizzle row
constexpr int NTHREADS = 192;
constexpr int MAX_GROUPS = 512;

constexpr int pow2_at_least(int x) { int p = 32; while (p < x) p *= 2; return p; }

template <int TNB, bool GATED> struct Cfg {
    static constexpr int NA = GATED ? 2 : 1;
    static constexpr int A_BYTES = BF * BK * 2;
    static constexpr int B_BYTES = TNB * BK * 2;
    static constexpr int STAGE_BYTES = NA * A_BYTES + B_BYTES;
    // Tiles of up to 32 tokens: two CTAs an SM (their tiles then spread over 296 CTAs instead of 148, and one CTA's
    // epilogue and tile change hide behind the other's stream); wider tiles: one CTA with the whole ring.
    static constexpr int CTAS_PER_SM = TNB <= 32 ? 2 : 1;
    static constexpr int RING_BYTES = CTAS_PER_SM == 2 ? 108 * 1024 : 200 * 1024;
    static constexpr int STAGES = RING_BYTES / STAGE_BYTES < 8 ? RING_BYTES / STAGE_BYTES : 8;
    static constexpr int ACC_COLS = NA * TNB;                   // one accumulator set
    static constexpr int NBUF = 2 * ACC_COLS <= 512 ? 2 : 1;    // accumulator sets: two when they fit tensor memory
    static constexpr int TMEM_COLS = pow2_at_least(NBUF * ACC_COLS);
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(TMEM_COLS <= 512, "the accumulators must fit tensor memory");
};

struct SwArgs {
    void* C; long ldc; int c_dtype; int accumulate;
    const void* bias; int bias_dtype;
    int M, N, K;
    int gate_up_offset;
    const int* group_offsets;
    int n_groups;
    int weights_first;
    int k_splits;          // > 1 (dense only): K is cut into this many runs, each tile and run writes 32-bit partial sums
    float* partials;       // [k_splits, M, N], summed by splitk_reduce_kernel
    int* status;
};

struct Tile { int group, r0, row_end, n0, split, kb0, kb1; };

template <int TNB>
__device__ __forceinline__ Tile tile_of(int id, const SwArgs& a, int t_tiles, int n_tiles, const int* cum) {
    Tile t;
    const int k_blocks = (a.K + BK - 1) / BK;
    t.split = 0; t.kb0 = 0; t.kb1 = k_blocks;
    if (!a.group_offsets) {
        // the runs of K of one tile are neighbours, then the token tiles of one feature tile: CTAs working at the same
        // time share a slice of W
        if (a.k_splits > 1) {
            const int per = (k_blocks + a.k_splits - 1) / a.k_splits;
            t.split = id % a.k_splits;
            id /= a.k_splits;
            t.kb0 = t.split * per;
            t.kb1 = t.kb0 + per < k_blocks ? t.kb0 + per : k_blocks;
        }
        t.group = 0;
        t.n0 = (id / t_tiles) * BF;
        t.r0 = (id % t_tiles) * TNB;
        t.row_end = a.M;
    } else {
        const int ti = id / n_tiles;
        t.n0 = (id % n_tiles) * BF;
        int lo = 0, hi = a.n_groups;            // largest e with cum[e] <= ti
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cum[mid] <= ti) lo = mid; else hi = mid; }
        t.group = lo;
        t.r0 = a.group_offsets[lo] + (ti - cum[lo]) * TNB;
        t.row_end = a.group_offsets[lo + 1];
    }
    return t;
}

template <int TNB>
__device__ __forceinline__ int cols_of(const Tile& t) {   // columns of the tile's products: tokens rounded up to 16
    const int rows = t.row_end - t.r0;
    return rows >= TNB ? TNB : (rows + 15) & ~15;
}

template <int TNB, bool GATED>
__global__ void __launch_bounds__(NTHREADS, (TNB <= 32 ? 2 : 1)) gemm_tc_swap_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                   const __grid_constant__ CUtensorMap map_x, SwArgs a)
{
    using C = Cfg<TNB, GATED>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int cum_s[MAX_GROUPS + 1];        // grouped: token tiles before each group
    __shared__ int abort_flag_s;
    __shared__ uint32_t tmem_base_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (a.N + BF - 1) / BF;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = base + STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    volatile int* abort_flag = &abort_flag_s;

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b2 = 0; b2 < 2; ++b2) { mbar_init(acc_full_bar(b2), 1); mbar_init(acc_empty_bar(b2), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    // Everything above touched nothing that the kernel before this one on the stream writes.  What follows reads the
    // experts' row offsets and the rows.  weights_first: the caller says that only the rows (X, and the rows of C that
    // are added to) come from the kernel directly before this one; the offsets are older.  Then the thread that
    // issues the loads asks for the weights of its first stages before it waits for that kernel: they stream while
    // it drains.
    const bool early = a.weights_first != 0;
    if (!early) fx_pdl_wait();
    int t_tiles = (a.M + TNB - 1) / TNB;
    if (a.group_offsets) {
        for (int e = threadIdx.x; e < a.n_groups; e += NTHREADS)
            cum_s[e + 1] = (a.group_offsets[e + 1] - a.group_offsets[e] + TNB - 1) / TNB;
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = 0;
            for (int e = 0; e < a.n_groups; ++e) { const int n = cum_s[e + 1]; cum_s[e] = run; run += n; }
            cum_s[a.n_groups] = run;
        }
        __syncthreads();
        t_tiles = cum_s[a.n_groups];
    }
    // a CTA beyond the tiles has nothing to do and goes straight to the end
    const int total = t_tiles * n_tiles * (a.group_offsets || a.k_splits < 1 ? 1 : a.k_splits);
    if (early && threadIdx.x != 0) fx_pdl_wait();

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            long issued = 0;
            bool ok = true;
            int pre = 0;   // stages of the first tile whose weights were asked for before the dependency wait
            if (early) {
                if ((int)blockIdx.x < total) {
                    const Tile t = tile_of<TNB>(blockIdx.x, a, t_tiles, n_tiles, cum_s);
                    pre = t.kb1 - t.kb0 < STAGES ? t.kb1 - t.kb0 : STAGES;
                    for (int i = 0; i < pre; ++i) {   // fresh barriers: every stage is free
                        const int kb = t.kb0 + i;
                        const uint32_t sw = base + i * C::STAGE_BYTES;
                        mbar_expect_tx(full_bar(i), C::STAGE_BYTES);
                        tma_load_3d(sw, &map_w, kb * BK, t.n0, t.group, full_bar(i));
                        if (GATED) tma_load_3d(sw + C::A_BYTES, &map_w, kb * BK, a.gate_up_offset + t.n0, t.group, full_bar(i));
                    }
                }
                fx_pdl_wait();
                if ((int)blockIdx.x < total) {
                    const Tile t = tile_of<TNB>(blockIdx.x, a, t_tiles, n_tiles, cum_s);
                    for (int i = 0; i < pre; ++i)
                        tma_load_2d(base + i * C::STAGE_BYTES + C::NA * C::A_BYTES, &map_x, (t.kb0 + i) * BK, t.r0, full_bar(i));
                }
                issued = pre;
            }
            for (int id = blockIdx.x; id < total && ok; id += gridDim.x) {
                const Tile t = tile_of<TNB>(id, a, t_tiles, n_tiles, cum_s);
                for (int kb = t.kb0 + (id == (int)blockIdx.x ? pre : 0); kb < t.kb1; ++kb, ++issued) {
                    const int s = (int)(issued % STAGES);
                    const uint32_t parity = (uint32_t)((issued / STAGES) & 1) ^ 1u;
                    if (!mbar_wait(empty_bar(s), parity, abort_flag)) { ok = false; break; }
                    const uint32_t sw = base + s * C::STAGE_BYTES, sx = sw + C::NA * C::A_BYTES;
                    mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
                    tma_load_3d(sw, &map_w, kb * BK, t.n0, t.group, full_bar(s));
                    if (GATED) tma_load_3d(sw + C::A_BYTES, &map_w, kb * BK, a.gate_up_offset + t.n0, t.group, full_bar(s));
                    tma_load_2d(sx, &map_x, kb * BK, t.r0, full_bar(s));
                }
            }
            if (*abort_flag) {
                for (long kb = issued > STAGES ? issued - STAGES : 0; kb < issued; ++kb) {
                    const int s = (int)(kb % STAGES);
                    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                        if (mbar_try_wait(full_bar(s), (uint32_t)((kb / STAGES) & 1))) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issue ----------------
        if (lane == 0) {
            long used = 0;
            bool ok = true;
            int it = 0;
            for (int id = blockIdx.x; id < total && ok; id += gridDim.x, ++it) {
                const Tile t = tile_of<TNB>(id, a, t_tiles, n_tiles, cum_s);
                const uint32_t idesc = instr_desc_ex(BF, cols_of<TNB>(t), 0);
                const int buf = it % C::NBUF;
                ok = mbar_wait(acc_empty_bar(buf), (uint32_t)((it / C::NBUF) & 1) ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * C::ACC_COLS);
                for (int kb = t.kb0; kb < t.kb1; ++kb, ++used) {
                    const int s = (int)(used % STAGES);
                    ok = mbar_wait(full_bar(s), (uint32_t)((used / STAGES) & 1), abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sw = base + s * C::STAGE_BYTES, sx = sw + C::NA * C::A_BYTES;
                    const uint64_t dw = smem_desc(sw), du = smem_desc(sw + C::A_BYTES), dx = smem_desc(sx);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        tc_mma(acc, dw + 2u * k, dx + 2u * k, idesc, kb > t.kb0 || k > 0);
                        if (GATED) tc_mma(acc + TNB, du + 2u * k, dx + 2u * k, idesc, kb > t.kb0 || k > 0);
                    }
                    tc_commit(empty_bar(s));
                }
                if (ok) tc_commit(acc_full_bar(buf));
            }
        }
    } else {
        // ---------------- epilogue: a thread owns one feature ----------------
        const int quad = warp & 3;
        int it = 0;
        for (int id = blockIdx.x; id < total; id += gridDim.x, ++it) {
            const Tile t = tile_of<TNB>(id, a, t_tiles, n_tiles, cum_s);
            const int buf = it % C::NBUF;
            const int f = t.n0 + quad * 32 + lane;
            const bool f_ok = f < a.N;
            const float bias = (a.bias && f_ok && a.k_splits <= 1) ? load_any(a.bias, a.bias_dtype, f) : 0.f;
            const int n_chunks = (cols_of<TNB>(t) + 31) / 32;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_full_bar(buf), (uint32_t)((it / C::NBUF) & 1), abort_flag));
            if (!ok) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * C::ACC_COLS);
#pragma unroll 1
            for (int c = 0; c < n_chunks; ++c) {
                uint32_t r[32], u[32];
                tc_ld32(lane_addr + c * 32, r);
                if (GATED) tc_ld32(lane_addr + TNB + c * 32, u);
                tc_ld_wait();
                if (c == n_chunks - 1) {   // the accumulators are in registers: hand them back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
                if (!f_ok) continue;
                const int row0 = t.r0 + c * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (row0 + j >= t.row_end) break;
                    float x = __uint_as_float(r[j]) + bias;
                    if (GATED) x = x / (1.0f + __expf(-x)) * __uint_as_float(u[j]);
                    if (a.k_splits > 1) {   // a run of K: the plain partial sum
                        a.partials[((long)t.split * a.M + row0 + j) * a.N + f] = __uint_as_float(r[j]);
                        continue;
                    }
                    const long at = (long)(row0 + j) * a.ldc + f;
                    if (a.c_dtype == FX_F32) {
                        float* cp = reinterpret_cast<float*>(a.C) + at;
                        *cp = a.accumulate ? *cp + x : x;
                    } else {
                        bf16* cp = reinterpret_cast<bf16*>(a.C) + at;
                        *cp = __float2bfloat16_rn(a.accumulate ? __bfloat162float(*cp) + x : x);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag_s && a.status) atomicExch(a.status, STATUS_TC_TIMEOUT);
}

// C[r, n] (+)= sum over the runs of K, in run order (+ bias[n])
__global__ void splitk_reduce_kernel(const float* __restrict__ partials, int k_splits, int M, int N, void* C, long ldc,
                                     int c_dtype, int accumulate, const void* bias, int bias_dtype)
{
    fx_pdl_wait();
    const long total = (long)M * N;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / N; const int n = (int)(i - r * N);
        float v = 0.f;
        for (int s2 = 0; s2 < k_splits; ++s2) v += partials[(long)s2 * total + i];
        if (bias) v += load_any(bias, bias_dtype, n);
        if (c_dtype == FX_F32) {
            float* cp = reinterpret_cast<float*>(C) + r * ldc + n;
            *cp = accumulate ? *cp + v : v;
        } else {
            bf16* cp = reinterpret_cast<bf16*>(C) + r * ldc + n;
            *cp = __float2bfloat16_rn(accumulate ? __bfloat162float(*cp) + v : v);
        }
    }
}

// bf16 tensor [d2][d1][K] (row pitch ld1 elements, matrix pitch ld2 elements), box {64, box1, 1}
bool make_map(CUtensorMap* map, const void* ptr, uint64_t K, uint64_t d1, uint64_t d2, uint64_t ld1, uint64_t ld2,
              uint32_t box1, int rank)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {K, d1, d2};
    cuuint64_t strides[2] = {ld1 * 2, ld2 * 2};
    cuuint32_t box[3] = {(cuuint32_t)BK, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int TNB, bool GATED>
int launch(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows, const SwArgs& a, cudaStream_t s)
{
    CUtensorMap mw, mx;
    const int G = a.group_offsets ? a.n_groups : 1;
    if (!make_map(&mw, W, (uint64_t)a.K, (uint64_t)w_rows, (uint64_t)G, (uint64_t)ldw,
                  (uint64_t)(G > 1 ? w_group_stride : (long)w_rows * ldw), BF, 3))
        return FX_ERR_SIZE;
    if (!make_map(&mx, X, (uint64_t)a.K, (uint64_t)a.M, 1, (uint64_t)ldx, 0, TNB, 2)) return FX_ERR_SIZE;
    auto kern = gemm_tc_swap_kernel<TNB, GATED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<TNB, GATED>::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long t_tiles = a.group_offsets ? fx_cdiv(a.M, TNB) + a.n_groups : fx_cdiv(a.M, TNB);   // an upper bound when grouped
    const long max_tiles = t_tiles * fx_cdiv(a.N, BF) * (a.k_splits > 1 ? a.k_splits : 1);
    const long slots = (long)fx_sm_count() * Cfg<TNB, GATED>::CTAS_PER_SM;
    const unsigned grid = (unsigned)(max_tiles < slots ? max_tiles : slots);
    fx_launch_pdl(kern, grid, NTHREADS, Cfg<TNB, GATED>::SMEM, s, mw, mx, a);
    if (a.k_splits > 1) {
        long blocks = fx_cdiv((long)a.M * a.N, 256);
        if (blocks > fx_sm_count() * 8L) blocks = fx_sm_count() * 8L;
        fx_launch_pdl(splitk_reduce_kernel, (unsigned)blocks, 256, 0, s, (const float*)a.partials, a.k_splits, a.M, a.N, a.C,
                      a.ldc, a.c_dtype, a.accumulate, a.bias, a.bias_dtype);
    }
    return fx_launch_status();
}

template <int TNB>
int run_tnb(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows, const SwArgs& a, int gated,
            cudaStream_t s)
{
    return gated ? launch<TNB, true>(X, ldx, W, ldw, w_group_stride, w_rows, a, s)
                 : launch<TNB, false>(X, ldx, W, ldw, w_group_stride, w_rows, a, s);
}

}  // namespace

// k_splits > 1 (plain dense products only): K is cut into runs that separate CTAs take, partial sums [k_splits, M, N]
// (float32, caller's scratch) are added up in run order by a second kernel: for matrices with too few rows to fill the
// machine with tiles.
// Same operands as fx_gemm_tc.  weights_first: group_offsets (if any) were NOT written by the kernel directly before
// this one on the stream, so that the weights may be fetched before that kernel has finished.  tokens_per_tile: 32, 64, 128 or 256 columns of a tile (0: chosen from M; grouped: 128).
// With 256 columns the gated form has room for one set of accumulators only: its epilogue and the next tile's
// products do not overlap.
extern "C" int fx_gemm_tc_swap(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows,
                               const void* bias, int bias_dtype, void* C, int c_dtype, long ldc, int accumulate,
                               int M, int N, int K, int gated, int gate_up_offset, const int* group_offsets, int n_groups,
                               int tokens_per_tile, int weights_first, int k_splits, float* partials, int* status,
                               void* stream)
{
    if (M <= 0 || N <= 0) return FX_OK;
    if (K <= 0 || K % 8) return FX_ERR_SIZE;
    if (ldx % 8 || ldw % 8 || w_group_stride % 8 || (uintptr_t)X % 16 || (uintptr_t)W % 16) return FX_ERR_ALIGN;
    if (c_dtype != FX_F32 && c_dtype != FX_BF16) return FX_ERR_DTYPE;
    if (group_offsets && n_groups > MAX_GROUPS) return FX_ERR_SIZE;
    SwArgs a;
    a.C = C; a.ldc = ldc; a.c_dtype = c_dtype; a.accumulate = accumulate;
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.M = M; a.N = N; a.K = K; a.gate_up_offset = gate_up_offset;
    a.group_offsets = group_offsets; a.n_groups = n_groups; a.status = status; a.weights_first = weights_first;
    a.k_splits = k_splits > 1 ? k_splits : 1; a.partials = partials;
    if (a.k_splits > 1 && (group_offsets || gated || !partials || a.k_splits > (K + BK - 1) / BK)) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    int tnb = tokens_per_tile;
    if (tnb == 0) tnb = group_offsets ? 128 : (M <= 32 ? 32 : M <= 64 ? 64 : 128);
    if (tnb == 32) return run_tnb<32>(X, ldx, W, ldw, w_group_stride, w_rows, a, gated, s);
    if (tnb == 64) return run_tnb<64>(X, ldx, W, ldw, w_group_stride, w_rows, a, gated, s);
    if (tnb == 128) return run_tnb<128>(X, ldx, W, ldw, w_group_stride, w_rows, a, gated, s);
    if (tnb == 256) return run_tnb<256>(X, ldx, W, ldw, w_group_stride, w_rows, a, gated, s);
    return FX_ERR_SIZE;
}
