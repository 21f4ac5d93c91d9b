// Prompt-sized matrix products on the 5th-generation tensor cores:
//   C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias)          bfloat16 in, 32-bit sums in TMEM
// plus the gated form (silu(gate) * up in the epilogue) and the grouped form for
// experts (rows sorted by expert; tile (expert, m) found on the device).
//
// One CTA computes one 128 x BN tile.  Warp 0 is the producer: one thread issues
// TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a 128 x 64 slice of X and a
// BN x 64 slice of W per stage into a ring of shared-memory stages guarded by
// mbarriers.  Warp 1 issues tcgen05.mma (one thread, cta_group::1, kind::f16 with
// bfloat16 operands): four K=16 instructions per stage, accumulating into BN
// columns of tensor memory, and releases each stage with tcgen05.commit.  Warps 2-5
// are the epilogue: each reads its quadrant of 32 TMEM lanes (= 32 rows of the tile)
// with tcgen05.ld, applies bias / SiLU gate / accumulation and stores rows.
// No cluster launch and no multicast: every CTA fetches its own tiles.
//
// Every wait is bounded: a wait that runs out raises `status` (code 3), the roles
// leave their loops, the producer waits (bounded) for loads it has in flight, tensor
// memory is freed and the kernel returns.
//
// Shapes: any M, N; K a multiple of 8 (16-byte row pitch for TMA), pointers 16-byte
// aligned; rows and columns beyond the edges are zero-filled by TMA and masked at
// the store.  Other shapes are refused (the caller falls back to the CUDA-core
// kernel).
//
// Reference: none on the GPU (the reference's prefill loops a mat-vec per token,
// crates/ferrox-core/src/weight_matrix.rs:1115-1122); the product itself is
// crates/ferrox-core/src/matmul.rs:18-58, experts crates/ferrox-moe/src/lib.rs:619-659.
#include "tc_common.cuh"
#include "tc_epilogue.cuh"
#include "api.h"

namespace {

constexpr int BM = 128;          // rows of X per tile = TMEM lanes
constexpr int BK = 64;           // bfloat16 elements per stage along K = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NTHREADS = 192;    // producer warp, mma warp, four epilogue warps

template <int BN> struct Cfg {
    static constexpr int STAGES = BN <= 128 ? 6 : 4;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ +
                                4 * fxtc::EPI_WARP_BYTES /* the epilogue warps' staging tiles */;
    static_assert(2 * BN <= 512, "two accumulators must fit the 512 columns of tensor memory");
};

struct TcArgs {
    void* C; long ldc; int c_dtype; int accumulate;
    const void* bias; int bias_dtype;
    int M, N, K;
    int gate_up_offset;             // gated: W row of `up` feature j is gate_up_offset + j
    const int* group_offsets;       // grouped: rows [off[e], off[e+1]) use matrix e
    int n_groups;
    int* status;
};

using namespace fxtc;

// Instruction descriptor: D = f32, A = B = bf16, both K-major, N / 8 and M / 16.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Where a tile lies.  Dense: ids run over the row tiles first, so that CTAs working at the same time share
// a slice of W.  Grouped: ids run over the feature tiles first, so that they share an expert's rows of X.
struct TileCoord { int group, m0, row_end, n0; };

template <int OUT_N>
__device__ __forceinline__ TileCoord tile_coord(int id, const TcArgs& a, int m_tiles, int n_tiles, const int* cum) {
    TileCoord t;
    if (!a.group_offsets) {
        t.group = 0;
        t.n0 = (id / m_tiles) * OUT_N;
        t.m0 = (id % m_tiles) * BM;
        t.row_end = a.M;
    } else {
        const int mi = id / n_tiles;
        t.n0 = (id % n_tiles) * OUT_N;
        int lo = 0, hi = a.n_groups;            // largest e with cum[e] <= mi
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cum[mid] <= mi) lo = mid; else hi = mid; }
        t.group = lo;
        t.m0 = a.group_offsets[lo] + (mi - cum[lo]) * BM;
        t.row_end = a.group_offsets[lo + 1];
    }
    return t;
}

constexpr int MAX_GROUPS = 1024;

// Persistent: gridDim.x CTAs (at most one per SM) take tiles id = blockIdx.x, + gridDim.x, ...  The
// accumulator is double-buffered in tensor memory (2 x BN columns), so the epilogue of one tile runs while
// the tensor cores work on the next.
template <int BN, bool GATED>
__global__ void __launch_bounds__(NTHREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                              const __grid_constant__ CUtensorMap map_b, TcArgs a)
{
    using C = Cfg<BN>;
    constexpr int STAGES = C::STAGES;
    constexpr int OUT_N = GATED ? BN / 2 : BN;   // output features per tile
    extern __shared__ uint8_t smem_raw[];
    __shared__ int cum_s[MAX_GROUPS + 1];        // grouped: row tiles before each group
    __shared__ int abort_flag_s;
    __shared__ uint32_t tmem_base_s;
    __shared__ __align__(16) float bias_s[4][OUT_N];   // each epilogue warp keeps the tile's bias for itself

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (a.N + OUT_N - 1) / OUT_N;
    int m_tiles = (a.M + BM - 1) / BM;
    if (a.group_offsets) fx_pdl_wait();   // the offsets come from the kernel before this one
    if (a.group_offsets) {
        for (int e = threadIdx.x; e < a.n_groups; e += NTHREADS)     // row tiles of each group, loaded in parallel
            cum_s[e + 1] = (a.group_offsets[e + 1] - a.group_offsets[e] + BM - 1) / BM;
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = 0;
            for (int e = 0; e < a.n_groups; ++e) { const int n = cum_s[e + 1]; cum_s[e] = run; run += n; }
            cum_s[a.n_groups] = run;
        }
        __syncthreads();
        m_tiles = cum_s[a.n_groups];
    }
    const int total = m_tiles * n_tiles;
    if ((int)blockIdx.x >= total) return;
    const int k_blocks = (a.K + BK - 1) / BK;

    // ---- shared memory: stages (1024-byte aligned), then barriers ---------------
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
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
    if (warp == 1) {   // tensor memory: two accumulators of BN columns (128 lanes x 32 bit each)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)(2 * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    if (!a.group_offsets) fx_pdl_wait();   // set up while the kernel before this one drains; its results from here on

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            long issued = 0;   // k-blocks issued so far, over all tiles of this CTA
            bool ok = true;
            for (int id = blockIdx.x; id < total && ok; id += gridDim.x) {
                const TileCoord tc = tile_coord<OUT_N>(id, a, m_tiles, n_tiles, cum_s);
                for (int kb = 0; kb < k_blocks; ++kb, ++issued) {
                    const int s = (int)(issued % STAGES);
                    const uint32_t parity = (uint32_t)((issued / STAGES) & 1) ^ 1u;
                    if (!mbar_wait(empty_bar(s), parity, abort_flag)) { ok = false; break; }
                    const uint32_t sa = base + s * C::STAGE_BYTES, sb = sa + C::A_BYTES;
                    mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
                    tma_load_2d(sa, &map_a, kb * BK, tc.m0, full_bar(s));
                    if (GATED) {
                        tma_load_3d(sb, &map_b, kb * BK, tc.n0, tc.group, full_bar(s));
                        tma_load_3d(sb + C::B_BYTES / 2, &map_b, kb * BK, a.gate_up_offset + tc.n0, tc.group, full_bar(s));
                    } else {
                        tma_load_3d(sb, &map_b, kb * BK, tc.n0, tc.group, full_bar(s));
                    }
                }
            }
            if (*abort_flag) {
                // loads already issued must land before the CTA's shared memory is released
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
            constexpr uint32_t idesc = instr_desc(BM, BN);
            long used = 0;
            bool ok = true;
            int it = 0;
            for (int id = blockIdx.x; id < total && ok; id += gridDim.x, ++it) {
                const int buf = it & 1;
                // the epilogue has drained this accumulator (first use of each passes at once)
                ok = mbar_wait(acc_empty_bar(buf), (uint32_t)((it >> 1) & 1) ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++used) {
                    const int s = (int)(used % STAGES);
                    ok = mbar_wait(full_bar(s), (uint32_t)((used / STAGES) & 1), abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = base + s * C::STAGE_BYTES, sb = sa + C::A_BYTES;
                    const uint64_t da = smem_desc(sa), db = smem_desc(sb);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements = 32 bytes further along K inside the swizzled row: +2 in units of 16 bytes
                        tc_mma(acc, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                    }
                    tc_commit(empty_bar(s));   // the stage is free once these instructions have read it
                }
                if (ok) tc_commit(acc_full_bar(buf));  // complete once all instructions so far have retired
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quad = warp & 3;                       // TMEM lanes 32*quad .. 32*quad+31
        int it = 0;
        for (int id = blockIdx.x; id < total; id += gridDim.x, ++it) {
            const TileCoord tc = tile_coord<OUT_N>(id, a, m_tiles, n_tiles, cum_s);
            const int buf = it & 1;
            const int row = tc.m0 + quad * 32 + lane;
            // tcgen05.ld needs whole warps: agree on the outcome of the wait
            if (a.bias) {   // the bias of this tile's columns, once per warp (no barrier between warps)
                __syncwarp();
                for (int j = lane; j < OUT_N; j += 32)
                    bias_s[quad][j] = tc.n0 + j < a.N ? load_any(a.bias, a.bias_dtype, tc.n0 + j) : 0.f;
                __syncwarp();
            }
            // Accumulating into 32-bit rows: the values already there are fetched one chunk ahead, the first chunk
            // before the wait for the accumulator, so that their latency hides behind the products.
            const bool row_ok = row < tc.row_end;
            // whole tiles of aligned rows go out through the warp's staging tile in whole 128-byte lines (tc_epilogue.cuh)
            const bool fast = tc.n0 + OUT_N <= a.N && (uintptr_t)a.C % 16 == 0 &&
                              (a.c_dtype == FX_F32 ? a.ldc % 4 == 0 : (a.ldc % 8 == 0 && !a.accumulate));
            uint8_t* stage = smem_raw + (bar_base + 256u - smem_u32(smem_raw)) + quad * EPI_WARP_BYTES;
            const int rows_ok = min(32, max(0, tc.row_end - (tc.m0 + quad * 32)));
            const bool acc_ahead = !fast && !GATED && a.accumulate && a.c_dtype == FX_F32 && a.ldc % 4 == 0 && row_ok;
            float4 pre[8], nxt[8];
            auto fetch_c = [&](int c, float4* buf4) {
                const int nb = tc.n0 + c * 32;
                if (acc_ahead && c < OUT_N / 32 && nb + 32 <= a.N) {
                    const float4* cp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.C) + (long)row * a.ldc + nb);
#pragma unroll
                    for (int j = 0; j < 8; ++j) buf4[j] = cp[j];
                }
            };
            if (acc_ahead) fetch_c(0, pre);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_full_bar(buf), (uint32_t)((it >> 1) & 1), abort_flag));
            if (!ok) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
            for (int c = 0; c < OUT_N / 32; ++c) {
                uint32_t r[32], u[32];
                tc_ld32(lane_addr + c * 32, r);
                if (GATED) tc_ld32(lane_addr + BN / 2 + c * 32, u);
                if (acc_ahead) fetch_c(c + 1, nxt);
                tc_ld_wait();
                if (c == OUT_N / 32 - 1) {
                    // everything of this accumulator is in registers: hand it back to the tensor cores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
                const int nb = tc.n0 + c * 32;
                if (!fast && (!row_ok || nb >= a.N)) continue;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float x = __uint_as_float(r[j]);
                    if (a.bias) x += bias_s[quad][c * 32 + j];
                    if (GATED) x = __fdividef(x, 1.0f + __expf(-x)) * __uint_as_float(u[j]);
                    v[j] = x;
                }
                if (fast) {
                    const long row0 = tc.m0 + quad * 32;
                    if (a.c_dtype == FX_F32) {
                        epi_stage_f32(stage, lane, v);
                        __syncwarp();
                        epi_flush(stage, lane, reinterpret_cast<uint8_t*>(a.C) + (row0 * a.ldc + nb) * 4, a.ldc * 4, rows_ok, a.accumulate != 0);
                        __syncwarp();
                    } else {
                        epi_stage_bf16(stage, lane, c & 1, v);
                        if (c & 1) {
                            __syncwarp();
                            epi_flush(stage, lane, reinterpret_cast<uint8_t*>(a.C) + (row0 * a.ldc + nb - 32) * 2, a.ldc * 2, rows_ok, false);
                            __syncwarp();
                        }
                    }
                    continue;
                }
                const bool full = nb + 32 <= a.N;
                if (a.c_dtype == FX_F32) {
                    float* cp = reinterpret_cast<float*>(a.C) + (long)row * a.ldc + nb;
                    if (full && (a.ldc % 4 == 0)) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            if (a.accumulate) {
                                const float4 p = acc_ahead ? pre[j >> 2] : *reinterpret_cast<const float4*>(cp + j);
                                o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                            }
                            *reinterpret_cast<float4*>(cp + j) = o;
                        }
                    } else {
                        for (int j = 0; j < 32 && nb + j < a.N; ++j) cp[j] = a.accumulate ? cp[j] + v[j] : v[j];
                    }
                } else {
                    bf16* cp = reinterpret_cast<bf16*>(a.C) + (long)row * a.ldc + nb;
                    if (full && (a.ldc % 8 == 0) && !a.accumulate) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 o;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]);
                            __nv_bfloat162 p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
                            __nv_bfloat162 p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                            o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                            o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                            *reinterpret_cast<uint4*>(cp + j) = o;
                        }
                    } else {
                        for (int j = 0; j < 32 && nb + j < a.N; ++j)
                            cp[j] = __float2bfloat16_rn(a.accumulate ? __bfloat162float(cp[j]) + v[j] : v[j]);
                    }
                }
                if (acc_ahead) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) pre[j] = nxt[j];
                }
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag_s && a.status) atomicExch(a.status, STATUS_TC_TIMEOUT);
}

// ---- host side ----------------------------------------------------------------
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

template <int BN, bool GATED>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, long max_tiles, cudaStream_t s)
{
    auto kern = gemm_tc_kernel<BN, GATED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const unsigned grid = (unsigned)(max_tiles < fx_sm_count() ? max_tiles : fx_sm_count());
    fx_launch_pdl(kern, grid, NTHREADS, Cfg<BN>::SMEM, s, ma, mb, a);
    return fx_launch_status();
}

template <int BN>
int run_bn(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows, TcArgs& a, int gated,
           cudaStream_t s)
{
    const int out_n = gated ? BN / 2 : BN;
    CUtensorMap ma, mb;
    if (!make_map(&ma, X, (uint64_t)a.K, (uint64_t)a.M, 1, (uint64_t)ldx, 0, BM, 2)) return FX_ERR_SIZE;
    const int G = a.group_offsets ? a.n_groups : 1;
    if (!make_map(&mb, W, (uint64_t)a.K, (uint64_t)w_rows, (uint64_t)G, (uint64_t)ldw,
                  (uint64_t)(G > 1 ? w_group_stride : (long)w_rows * ldw), gated ? BN / 2 : BN, 3))
        return FX_ERR_SIZE;
    const long m_tiles = a.group_offsets ? fx_cdiv(a.M, BM) + a.n_groups : fx_cdiv(a.M, BM);   // an upper bound when grouped
    const long max_tiles = m_tiles * fx_cdiv(a.N, out_n);
    return gated ? launch<BN, true>(ma, mb, a, max_tiles, s) : launch<BN, false>(ma, mb, a, max_tiles, s);
}

}  // namespace

// X [M, K] and W [G, w_rows, K] bfloat16; C bfloat16 or float32.  gated: W holds gate rows [0, N) and up rows
// [gate_up_offset, gate_up_offset + N), C = silu(gate) * up.  grouped: group_offsets [n_groups + 1] on the device,
// rows of X (and of C) sorted by group; M is then the total number of rows.
extern "C" int fx_gemm_tc(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows,
                          const void* bias, int bias_dtype, void* C, int c_dtype, long ldc, int accumulate,
                          int M, int N, int K, int gated, int gate_up_offset, const int* group_offsets, int n_groups,
                          int* status, void* stream)
{
    if (M <= 0 || N <= 0) return FX_OK;
    if (K <= 0 || K % 8) return FX_ERR_SIZE;
    if (ldx % 8 || ldw % 8 || w_group_stride % 8 || (uintptr_t)X % 16 || (uintptr_t)W % 16) return FX_ERR_ALIGN;
    if (c_dtype != FX_F32 && c_dtype != FX_BF16) return FX_ERR_DTYPE;
    if (group_offsets && n_groups > MAX_GROUPS) return FX_ERR_SIZE;
    TcArgs a;
    a.C = C; a.ldc = ldc; a.c_dtype = c_dtype; a.accumulate = accumulate;
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.M = M; a.N = N; a.K = K; a.gate_up_offset = gate_up_offset;
    a.group_offsets = group_offsets; a.n_groups = n_groups; a.status = status;
    cudaStream_t s = (cudaStream_t)stream;
    // wide outputs take 128 x 256 tiles (fewer bytes fetched per flop; measured faster even when they give
    // every SM a single tile); narrow ones 128 x 128
    const int wide = gated ? N >= 256 : N >= 512;
    if (wide) return run_bn<256>(X, ldx, W, ldw, w_group_stride, w_rows, a, gated, s);
    return run_bn<128>(X, ldx, W, ldw, w_group_stride, w_rows, a, gated, s);
}
