// C (+)= X . W^T (+ bias) for a few tokens against a matrix that fits the shared memory of all SMs together.
//
// The weight-streaming kernel (gemm_skinny.cu) has one batch of loads per thread in flight before it may look at
// its tokens; what it streams after the wait for the kernel before it is most of the matrix.  Here every block owns
// a slab of rows of W, N / SMs of them, and asks for the WHOLE slab at its start: one bulk copy (TMA, untiled) per
// row into shared memory, all signalling one mbarrier, before the wait for the kernel before.  If that kernel is
// short and leaves the memory system idle (the combination of the experts before the Q/K/V product), the matrix
// travels while it runs, and after the wait there is little left to do: the tokens' rows into shared memory, a
// few mma.sync per warp, the sum over the warps.
//
// Warp w takes the w-th eighth of K for all rows of the slab (tiles of 16 rows: A = W rows by ldmatrix from rows
// padded by 16 bytes, B = the tokens' rows, 8 tokens a pass) and leaves its partial sums in shared memory; they are
// added in warp order, so a token's result does not depend on the other tokens, on the grid or on timing.
//
// bfloat16 X and W, 32-bit sums; C bfloat16 or 32-bit, optionally added to.  K a multiple of 128.
#include "tc_common.cuh"
#include "api.h"

namespace {
using namespace fxtc;

constexpr int WARPS = 8, NTHREADS = WARPS * 32, TOKENS = 8;

struct SlabArgs {
    const bf16* W; long ldw;
    const bf16* X; long ldx;
    const void* bias; int bias_dtype;
    void* C; long ldc; int c_dtype, accumulate;
    int n_tokens, N, K, rows_per_block, rows_pad;
    int* status;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// KSTEPS: the 16-wide steps of a warp's eighth of K (K / 128), as a bound the compiler can unroll by
template <int KSTEPS_MAX>
__global__ void __launch_bounds__(NTHREADS, 1) slab_kernel(SlabArgs a)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_s;
    __shared__ int abort_s;
    const int K = a.K, pitch = K * 2 + 16;                      // bytes of a row in shared memory
    const uint32_t w_u = smem_u32(smem_raw);                          // [rows_per_block][pitch]
    const uint32_t x_u = w_u + (uint32_t)a.rows_per_block * pitch;    // [TOKENS][pitch]
    // the warps' partial sums take the tokens' place once every warp holds its part of them in registers
    float* part = reinterpret_cast<float*>(smem_raw + (size_t)a.rows_per_block * pitch);   // [WARPS][rows_pad][TOKENS]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * a.rows_per_block;
    const int rows = min(a.rows_per_block, a.N - row0);
    const uint32_t bar = smem_u32(&bar_s);

    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, (uint32_t)rows * (uint32_t)K * 2u);
    }
    __syncthreads();
    // the slab: a bulk copy a row, asked for before anything is known of the tokens
    for (int r = threadIdx.x; r < rows; r += NTHREADS)
        bulk_load(w_u + (uint32_t)r * pitch, a.W + (long)(row0 + r) * a.ldw, (uint32_t)K * 2u, bar);
    fx_pdl_wait();

    const int g = lane >> 2, t4 = lane & 3;
    const int ksteps = K / (16 * WARPS);                        // this warp's steps of 16 along K
    const int k_begin = warp * ksteps * 16;
    const int row_tiles = a.rows_pad / 16;
    bool have_w = false;
    for (int t0 = 0; t0 < a.n_tokens; t0 += TOKENS) {
        // this pass's tokens; a step of fewer than 8 keeps only its own rows (the tensor cores read the last of them
        // again in place of the missing ones, and those columns of the result are not used)
        const int kept = min(TOKENS, a.n_tokens);
        for (int i = threadIdx.x; i < kept * (K / 8); i += NTHREADS) {
            const int t = i / (K / 8), c = i - t * (K / 8);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (t0 + t < a.n_tokens) v = *reinterpret_cast<const uint4*>(a.X + (long)(t0 + t) * a.ldx + c * 8);
            *reinterpret_cast<uint4*>(smem_raw + (size_t)(a.rows_per_block + t) * pitch + c * 16) = v;
        }
        __syncthreads();
        if (!have_w) {
            if (!mbar_wait(bar, 0, &abort_s)) abort_s = 1;
            have_w = true;
            __syncthreads();
        }
        if (abort_s) break;
        // B fragments of this warp's part of K: tokens in the columns
        uint32_t xb[KSTEPS_MAX][2];
#pragma unroll
        for (int ks = 0; ks < KSTEPS_MAX; ++ks)
            if (ks < ksteps)
                ldsm2(x_u + (uint32_t)min(lane & 7, kept - 1) * pitch + (uint32_t)(k_begin + ks * 16 + ((lane >> 3) & 1) * 8) * 2, xb[ks][0], xb[ks][1]);
        __syncthreads();                   // the tokens' rows are in registers: their place is free for the sums
        for (int rt = 0; rt < row_tiles; ++rt) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            // (the last tile's rows beyond the slab read its last row again; their results are not used)
            const uint32_t a_row = w_u + (uint32_t)min(rt * 16 + (lane & 15), rows - 1) * pitch + (uint32_t)(k_begin + (lane >> 4) * 8) * 2;
#pragma unroll
            for (int ks = 0; ks < KSTEPS_MAX; ++ks) {
                if (ks < ksteps) {
                    uint32_t a0, a1, a2, a3;
                    ldsm4(a_row + ks * 32, a0, a1, a2, a3);
                    mma16816(acc, a0, a1, a2, a3, xb[ks][0], xb[ks][1]);
                }
            }
            // acc: rows g and g + 8 of the tile, tokens 2 t4 and 2 t4 + 1
            float* p = part + ((long)warp * a.rows_pad + rt * 16) * TOKENS;
            *reinterpret_cast<float2*>(p + g * TOKENS + 2 * t4) = make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(p + (g + 8) * TOKENS + 2 * t4) = make_float2(acc[2], acc[3]);
        }
        __syncthreads();
        // the eighths of K added in warp order; rows fastest, so that a token's results are written side by side
        for (int i = threadIdx.x; i < rows * TOKENS; i += NTHREADS) {
            const int t = i / rows, r = i - t * rows;
            if (t0 + t >= a.n_tokens) break;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += part[((long)w * a.rows_pad + r) * TOKENS + t];
            const int n = row0 + r;
            if (a.bias) v += a.bias_dtype == FX_F32 ? reinterpret_cast<const float*>(a.bias)[n]
                                                    : __bfloat162float(reinterpret_cast<const bf16*>(a.bias)[n]);
            const long at = (long)(t0 + t) * a.ldc + n;
            if (a.c_dtype == FX_F32) {
                float* c = reinterpret_cast<float*>(a.C);
                c[at] = a.accumulate ? c[at] + v : v;
            } else {
                bf16* c = reinterpret_cast<bf16*>(a.C);
                c[at] = __float2bfloat16(a.accumulate ? __bfloat162float(c[at]) + v : v);
            }
        }
        __syncthreads();
    }
    if (!have_w) mbar_wait(bar, 0, &abort_s);     // (no tokens: the copies still have to land before the block ends)
    if (threadIdx.x == 0 && abort_s && a.status) atomicExch(a.status, STATUS_TC_TIMEOUT);
}

constexpr size_t SLAB_SMEM_MAX = 220 * 1024;

// rows a block and bytes of shared memory; false where the matrix does not fit
bool slab_plan(int N, int K, int n_tokens, int* rows_per_block, int* rows_pad, size_t* smem)
{
    if (N <= 0 || K <= 0 || K % 128 || K / 128 > 64) return false;
    const int sms = fx_sm_count();
    const int r = (int)fx_cdiv(N, sms);
    const int pad = (r + 15) & ~15;
    const size_t pitch = (size_t)K * 2 + 16;
    const size_t tokens = (size_t)(n_tokens < TOKENS ? n_tokens : TOKENS) * pitch, sums = (size_t)WARPS * pad * TOKENS * sizeof(float);
    const size_t bytes = (size_t)r * pitch + (tokens > sums ? tokens : sums);
    if (bytes > SLAB_SMEM_MAX) return false;
    *rows_per_block = r; *rows_pad = pad; *smem = bytes;
    return true;
}

template <int KSTEPS_MAX>
int launch(const SlabArgs& a, unsigned blocks, size_t smem, cudaStream_t s)
{
    auto kern = slab_kernel<KSTEPS_MAX>;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    fx_launch_pdl(kern, dim3(blocks), dim3(NTHREADS), smem, s, a);
    return fx_launch_status();
}

}  // namespace

// 1 where fx_gemm_slab takes the sizes (the whole matrix fits the SMs' shared memory, one slab of rows a block).
extern "C" int fx_gemm_slab_ok(int N, int K, int n_tokens)
{
    int r, pad; size_t smem;
    return slab_plan(N, K, n_tokens, &r, &pad, &smem) ? 1 : 0;
}

// C[t, n] (+)= sum_k X[t, k] W[n, k] (+ bias[n]).  X [n_tokens, K] and W [N, K] bfloat16 (rows 16-byte aligned);
// C bfloat16 or float32.  The weights are fetched before the kernel waits for the one before it on the stream:
// they must not be that kernel's work.  Refuses (FX_ERR_SIZE / FX_ERR_ALIGN) what does not fit.
extern "C" int fx_gemm_slab(const void* X, long ldx, const void* W, long ldw, const void* bias, int bias_dtype, void* C,
                            int c_dtype, long ldc, int accumulate, int n_tokens, int N, int K, int* status, void* stream)
{
    if (n_tokens <= 0 || N <= 0) return FX_OK;
    SlabArgs a;
    size_t smem = 0;
    if (!slab_plan(N, K, n_tokens, &a.rows_per_block, &a.rows_pad, &smem)) return FX_ERR_SIZE;
    if (ldw % 8 || ldx % 8 || (uintptr_t)W % 16 || (uintptr_t)X % 16) return FX_ERR_ALIGN;
    if (c_dtype != FX_F32 && c_dtype != FX_BF16) return FX_ERR_DTYPE;
    if (bias && bias_dtype != FX_F32 && bias_dtype != FX_BF16) return FX_ERR_DTYPE;
    a.W = (const bf16*)W; a.ldw = ldw; a.X = (const bf16*)X; a.ldx = ldx;
    a.bias = bias; a.bias_dtype = bias_dtype; a.C = C; a.ldc = ldc; a.c_dtype = c_dtype; a.accumulate = accumulate;
    a.n_tokens = n_tokens; a.N = N; a.K = K; a.status = status;
    const unsigned blocks = (unsigned)fx_cdiv(N, a.rows_per_block);
    cudaStream_t s = (cudaStream_t)stream;
    const int ksteps = K / (16 * WARPS);
    if (ksteps <= 8) return launch<8>(a, blocks, smem, s);
    if (ksteps <= 16) return launch<16>(a, blocks, smem, s);
    if (ksteps <= 32) return launch<32>(a, blocks, smem, s);
    return launch<64>(a, blocks, smem, s);
}
