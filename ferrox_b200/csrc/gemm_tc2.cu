// Large dense matrix products on pairs of SMs (tcgen05 with cta_group::2):
//   C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias)          bfloat16 in, 32-bit sums in tensor memory
// and the gated form (silu(gate) * up in the epilogue).
//
// Two CTAs of a cluster share one 256 x 256 tile: each loads 128 rows of X and 128 rows of W per stage (its half
// of the tile's rows and its half of the tile's columns) into its own shared memory, one thread of the first CTA
// issues tcgen05.mma.cta_group::2 (M = 256: both SMs' tensor cores, each reading its own rows of X and both halves
// of W), and each CTA's tensor memory receives its 128 rows of the result.  Per SM and k-block this moves 32 KB
// from L2 for 128 x 256 x 64 products, where the single-CTA kernel of gemm_tc.cu moves 48 KB: that kernel is
// bound by exactly this traffic.  No multicast loads: each CTA fetches what it keeps.
//
// Roles per CTA: warp 0 producer (TMA; both CTAs signal the first CTA's "full" barrier), warp 1 tensor-core issue
// (first CTA only; tcgen05.commit with a cluster mask releases a stage, or hands over an accumulator, in both
// CTAs), warps 2-5 epilogue (each CTA its own rows; they give the accumulator back with a remote arrive on the
// first CTA's barrier).  Accumulators are double-buffered (2 x 256 columns).  Every mbarrier wait is bounded
// (status code 3 on time-out; the roles leave their loops and both CTAs meet at the final cluster barrier).
//
// Reference: none (see gemm_tc.cu).
#include <cooperative_groups.h>

#include "tc_common.cuh"
#include "tc_epilogue.cuh"
#include "api.h"

namespace {

using namespace fxtc;

constexpr int BM = 128;          // rows of X per CTA (256 per pair)
constexpr int BNH = 128;         // rows of W per CTA (256 per pair)
constexpr int BK = 64;
constexpr int NTHREADS = 192;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256 + 4 * EPI_WARP_BYTES;   // ring, alignment slack, barriers, the epilogue warps' staging tiles
constexpr int ACC_COLS = 2 * BNH;            // columns of one accumulator: both halves of W
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // a shared::cluster address with this bit cleared names the pair's first CTA

struct Tc2Args {
    void* C; long ldc; int c_dtype; int accumulate;
    const void* bias; int bias_dtype;
    int M, N, K;
    int gate_up_offset;
    int gated;
    int* status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA loads whose bytes are counted on the barrier of the pair's first CTA
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar & PEER_MASK), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc2_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
// arrives (once all tensor-core instructions issued so far have finished) on the barrier at this address in both CTAs
__device__ __forceinline__ void tc2_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void arrive_on_first_cta(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_MASK) : "memory");
}

// GATED as a template argument: with a run-time flag the compiler evaluates the gate's exponential and division for
// every element of plain products too (a select instead of a branch).
template <bool GATED>
__global__ void __launch_bounds__(NTHREADS, 1) gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b, Tc2Args a)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag_s;
    __shared__ uint32_t tmem_base_s;
    __shared__ __align__(16) float bias_s[4][ACC_COLS];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();            // 0: the CTA that issues the tensor-core instructions
    const int out_n = GATED ? BNH : 2 * BNH;       // output features of a pair's tile
    const int n_tiles = (a.N + out_n - 1) / out_n;
    const int m_tiles = (a.M + 2 * BM - 1) / (2 * BM);
    const int total = m_tiles * n_tiles;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int k_blocks = (a.K + BK - 1) / BK;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // first CTA's is used
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };           // each CTA its own
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };    // each CTA its own
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };   // first CTA's is used
    volatile int* abort_flag = &abort_flag_s;

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b2 = 0; b2 < 2; ++b2) { mbar_init(acc_full_bar(b2), 1); mbar_init(acc_empty_bar(b2), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {   // the same warp in both CTAs, the same destination
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)(2 * ACC_COLS)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();   // the peer's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    fx_pdl_wait();    // set up while the kernel before this one drains; its results from here on

    if (warp == 0) {
        // ---------------- producer (both CTAs) ----------------
        if (lane == 0) {
            long issued = 0;
            bool ok = true;
            for (int id = pair; id < total && ok; id += n_pairs) {
                const int m0 = (id % m_tiles) * 2 * BM + (int)rank * BM;
                const int n0 = (id / m_tiles) * out_n;
                // this CTA's rows of W: plain: its half of the tile's features; gated: the gate rows (first CTA) or
                // the up rows (second CTA) of the tile's features
                const int w0 = GATED ? (rank ? a.gate_up_offset + n0 : n0) : n0 + (int)rank * BNH;
                for (int kb = 0; kb < k_blocks; ++kb, ++issued) {
                    const int s = (int)(issued % STAGES);
                    const uint32_t parity = (uint32_t)((issued / STAGES) & 1) ^ 1u;
                    if (!mbar_wait(empty_bar(s), parity, abort_flag)) { ok = false; break; }
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);   // both CTAs' bytes
                    tma2_load_2d(sa, &map_a, kb * BK, m0, full_bar(s));
                    tma2_load_2d(sb, &map_b, kb * BK, w0, full_bar(s));
                }
            }
            if (*abort_flag && rank == 0) {
                // loads already issued (by either CTA: all are counted here) must land before shared memory is released;
                // the second CTA stays at the cluster barrier below until this CTA gets there
                for (long kb = issued > STAGES ? issued - STAGES : 0; kb < issued; ++kb) {
                    const int s = (int)(kb % STAGES);
                    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
                        if (mbar_try_wait(full_bar(s), (uint32_t)((kb / STAGES) & 1))) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issue (first CTA) ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc_ex(2 * BM, 2 * BNH, 0);
            long used = 0;
            bool ok = true;
            int it = 0;
            for (int id = pair; id < total && ok; id += n_pairs, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(acc_empty_bar(buf), (uint32_t)((it >> 1) & 1) ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * ACC_COLS);
                for (int kb = 0; kb < k_blocks; ++kb, ++used) {
                    const int s = (int)(used % STAGES);
                    ok = mbar_wait(full_bar(s), (uint32_t)((used / STAGES) & 1), abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
                    const uint64_t da = smem_desc(sa), db = smem_desc(sb);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) tc2_mma(acc, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0);
                    tc2_commit_both(empty_bar(s));
                }
                if (ok) tc2_commit_both(acc_full_bar(buf));
            }
        }
    } else {
        // ---------------- epilogue (both CTAs, each its 128 rows) ----------------
        const int quad = warp & 3;
        int it = 0;
        for (int id = pair; id < total; id += n_pairs, ++it) {
            const int m0 = (id % m_tiles) * 2 * BM + (int)rank * BM;
            const int n0 = (id / m_tiles) * out_n;
            const int buf = it & 1;
            const int row = m0 + quad * 32 + lane;
            if (a.bias) {
                __syncwarp();
                for (int j = lane; j < out_n; j += 32)
                    bias_s[quad][j] = n0 + j < a.N ? load_any(a.bias, a.bias_dtype, n0 + j) : 0.f;
                __syncwarp();
            }
            // Accumulating into 32-bit rows: the values already there are fetched one chunk ahead, the first chunk
            // before the wait for the accumulator (as in gemm_tc.cu).
            const bool row_ok = row < a.M;
            const int chunks = out_n / 32;
            // whole tiles of aligned rows go out through the warp's staging tile in whole 128-byte lines (tc_epilogue.cuh)
            const bool fast = n0 + out_n <= a.N && (uintptr_t)a.C % 16 == 0 &&
                              (a.c_dtype == FX_F32 ? a.ldc % 4 == 0 : (a.ldc % 8 == 0 && !a.accumulate));
            uint8_t* stage = smem_raw + (bar_base + 256u - smem_u32(smem_raw)) + quad * EPI_WARP_BYTES;
            const int rows_ok = min(32, max(0, a.M - (m0 + quad * 32)));
            const bool acc_ahead = !fast && !GATED && a.accumulate && a.c_dtype == FX_F32 && a.ldc % 4 == 0 && row_ok;
            float4 pre[8], nxt[8];
            auto fetch_c = [&](int c, float4* buf4) {
                const int nb = n0 + c * 32;
                if (acc_ahead && c < chunks && nb + 32 <= a.N) {
                    const float4* cp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.C) + (long)row * a.ldc + nb);
#pragma unroll
                    for (int j = 0; j < 8; ++j) buf4[j] = cp[j];
                }
            };
            fetch_c(0, pre);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_full_bar(buf), (uint32_t)((it >> 1) & 1), abort_flag));
            if (!ok) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * ACC_COLS);
#pragma unroll 1
            for (int c = 0; c < chunks; ++c) {
                uint32_t r[32], u[32];
                tc_ld32(lane_addr + c * 32, r);
                if (GATED) tc_ld32(lane_addr + BNH + c * 32, u);
                fetch_c(c + 1, nxt);
                tc_ld_wait();
                if (c == chunks - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) arrive_on_first_cta(acc_empty_bar(buf));
                }
                const int nb = n0 + c * 32;
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
                    const long row0 = m0 + quad * 32;
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
#pragma unroll
                for (int j = 0; j < 8; ++j) pre[j] = nxt[j];
            }
        }
    }

    // ---- teardown: nobody leaves while the peer may still signal its barriers or read its shared memory ----
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * ACC_COLS)) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag_s && a.status) atomicExch(a.status, STATUS_TC_TIMEOUT);
}

bool make_map(CUtensorMap* map, const void* ptr, uint64_t K, uint64_t rows, uint64_t ld, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// X [M, K] and W [w_rows, K] bfloat16; C bfloat16 or float32.  gated: W holds gate rows [0, N) and up rows
// [gate_up_offset, gate_up_offset + N), C = silu(gate) * up.  Dense products only (no groups).
extern "C" int fx_gemm_tc2(const void* X, long ldx, const void* W, long ldw, int w_rows, const void* bias, int bias_dtype,
                           void* C, int c_dtype, long ldc, int accumulate, int M, int N, int K, int gated,
                           int gate_up_offset, int* status, void* stream)
{
    if (M <= 0 || N <= 0) return FX_OK;
    if (K <= 0 || K % 8) return FX_ERR_SIZE;
    if (ldx % 8 || ldw % 8 || (uintptr_t)X % 16 || (uintptr_t)W % 16) return FX_ERR_ALIGN;
    if (c_dtype != FX_F32 && c_dtype != FX_BF16) return FX_ERR_DTYPE;
    Tc2Args a;
    a.C = C; a.ldc = ldc; a.c_dtype = c_dtype; a.accumulate = accumulate;
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.M = M; a.N = N; a.K = K; a.gate_up_offset = gate_up_offset; a.gated = gated; a.status = status;
    CUtensorMap ma, mb;
    if (!make_map(&ma, X, (uint64_t)K, (uint64_t)M, (uint64_t)ldx, BM)) return FX_ERR_SIZE;
    if (!make_map(&mb, W, (uint64_t)K, (uint64_t)w_rows, (uint64_t)ldw, BNH)) return FX_ERR_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int sms = fx_sm_count();
    const int out_n = gated ? BNH : 2 * BNH;
    const long tiles = fx_cdiv(M, 2 * BM) * fx_cdiv(N, out_n);
    long pairs = tiles < sms / 2 ? tiles : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_fx_pdl_enabled ? 2 : 1;
    cudaError_t e = gated ? cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<true>, ma, mb, a) : cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<false>, ma, mb, a);
    if (e != cudaSuccess) return (int)e;
    return fx_launch_status();
}
