// C[M,N] (+)= A[M,K] . W[N,K]^T (+ bias): the matrix product every projection is.
//
// CUDA-core kernel (FFMA, 32-bit accumulate, no tensor-core or reduced-precision
// mode): it is the whole 32-bit path and the fallback of the bfloat16 path for
// shapes the tensor-core kernels refuse.  Takes any M, N, K.
//
//  * rows of A may be gathered through `a_rows` (row r of the product reads row
//    a_rows[r] of A), which is how expert inputs are picked without a copy;
//  * grouped mode (`group_offsets` != null): rows [off[g], off[g+1]) use matrix g of
//    W (stride `w_group_stride` elements); gridDim.z walks the groups and blocks
//    whose tile lies outside their group return at once;
//  * each output element is one thread's sequential sum over k, so a row's result
//    does not depend on M, on which other rows share the launch, or on its place.
//
// Reference: the reference has no GEMM on CUDA (prefill loops a mat-vec per
// position, crates/ferrox-core/src/weight_matrix.rs:1115-1122); the CPU product
// is crates/ferrox-core/src/matmul.rs:18-58 ([m,k].[n,k]^T, sequential f32 sum).
#include "common.cuh"
#include "api.h"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

template <typename T> __device__ __forceinline__ void load4(const T* p, float* o);
template <> __device__ __forceinline__ void load4<float>(const float* p, float* o) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float* o) {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v.y);
    o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
}

template <typename AT, typename WT, typename CT, bool VEC>
__global__ void __launch_bounds__(NT) gemm_kernel(
    const AT* __restrict__ A, long lda, const int* __restrict__ a_rows,
    const WT* __restrict__ W, long ldw,
    const void* __restrict__ bias, int bias_dtype,
    CT* __restrict__ C, long ldc, int accumulate,
    int M, int N, int K,
    const int* __restrict__ group_offsets, long w_group_stride)
{
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Ws[BK][BN + 4];

    int row_begin = 0, row_end = M;
    if (group_offsets) {
        row_begin = group_offsets[blockIdx.z];
        row_end = group_offsets[blockIdx.z + 1];
        W += (long)blockIdx.z * w_group_stride;
    }
    const int m0 = row_begin + blockIdx.y * BM;
    if (m0 >= row_end) return;
    const int n0 = blockIdx.x * BN;

    const int tid = threadIdx.x;
    const int lr = tid >> 2;        // 0..63: row of the tile this thread loads
    const int lk = (tid & 3) * 4;   // 0,4,8,12: first k of its four
    const int tx = tid & 15, ty = tid >> 4;

    // Source rows for this thread's loads.
    const int am = m0 + lr;
    const AT* a_ptr = nullptr;
    if (am < row_end) a_ptr = A + (long)(a_rows ? a_rows[am] : am) * lda;
    const int wn = n0 + lr;
    const WT* w_ptr = wn < N ? W + (long)wn * ldw : nullptr;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float av[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        const int k = k0 + lk;
        if (VEC) {
            if (a_ptr && k < K) load4<AT>(a_ptr + k, av);
            if (w_ptr && k < K) load4<WT>(w_ptr + k, wv);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (a_ptr && k + i < K) av[i] = to_f32(a_ptr[k + i]);
                if (w_ptr && k + i < K) wv[i] = to_f32(w_ptr[k + i]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lr] = av[i];
            Ws[lk + i][lr] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float ar[4] = {a.x, a.y, a.z, a.w};
            const float br[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_any(bias, bias_dtype, n);
            CT* c = C + (long)m * ldc + n;
            if (accumulate) v += to_f32(*c);
            *c = from_f32<CT>(v);
        }
    }
}

template <typename AT, typename WT, typename CT>
int launch(const void* A, long lda, const int* a_rows, const void* W, long ldw, const void* bias, int bias_dtype,
           void* C, long ldc, int accumulate, int M, int N, int K, const int* group_offsets, int n_groups,
           long w_group_stride, cudaStream_t stream)
{
    if (M <= 0 || N <= 0) return FX_OK;
    dim3 grid((unsigned)fx_cdiv(N, BN), (unsigned)fx_cdiv(M, BM), group_offsets ? n_groups : 1);
    if (grid.y > 65535u || grid.z > 65535u) return FX_ERR_SIZE;
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && (w_group_stride % 4 == 0) &&
                     ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
    if (vec)
        gemm_kernel<AT, WT, CT, true><<<grid, NT, 0, stream>>>(
            (const AT*)A, lda, a_rows, (const WT*)W, ldw, bias, bias_dtype, (CT*)C, ldc, accumulate, M, N, K,
            group_offsets, w_group_stride);
    else
        gemm_kernel<AT, WT, CT, false><<<grid, NT, 0, stream>>>(
            (const AT*)A, lda, a_rows, (const WT*)W, ldw, bias, bias_dtype, (CT*)C, ldc, accumulate, M, N, K,
            group_offsets, w_group_stride);
    return fx_launch_status();
}

}  // namespace

extern "C" int fx_gemm(const void* A, int a_dtype, long lda, const int* a_rows,
                       const void* W, int w_dtype, long ldw,
                       const void* bias, int bias_dtype,
                       void* C, int c_dtype, long ldc, int accumulate,
                       int M, int N, int K,
                       const int* group_offsets, int n_groups, long w_group_stride,
                       void* stream)
{
    cudaStream_t s = (cudaStream_t)stream;
#define FX_GEMM_CASE(AC, WC, CC, AT, WT, CT)                                                            \
    if (a_dtype == AC && w_dtype == WC && c_dtype == CC)                                                  \
        return launch<AT, WT, CT>(A, lda, a_rows, W, ldw, bias, bias_dtype, C, ldc, accumulate, M, N, K, \
                                  group_offsets, n_groups, w_group_stride, s);
    FX_GEMM_CASE(FX_F32, FX_F32, FX_F32, float, float, float)
    FX_GEMM_CASE(FX_BF16, FX_BF16, FX_BF16, bf16, bf16, bf16)
    FX_GEMM_CASE(FX_BF16, FX_BF16, FX_F32, bf16, bf16, float)
    FX_GEMM_CASE(FX_BF16, FX_F32, FX_BF16, bf16, float, bf16)
    FX_GEMM_CASE(FX_BF16, FX_F32, FX_F32, bf16, float, float)
#undef FX_GEMM_CASE
    return FX_ERR_DTYPE;
}
