// Shared helpers of the sm_100a kernels: element types, conversions, reductions,
// the status codes that the C entry points return.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Element type codes of the C ABI (ferrox_b200/kernels/lib.py mirrors them).
#define FX_F32 0
#define FX_BF16 1

// Status codes returned by every entry point. 0 = launched; positive values are
// cudaError_t from the launch; negative values are refusals of this library.
#define FX_OK 0
#define FX_ERR_DTYPE -1     // combination of element types not built
#define FX_ERR_SIZE -2      // a size outside what the kernel handles
#define FX_ERR_ALIGN -3     // pointer or stride not aligned as required
#define FX_ERR_TIMEOUT -4   // a bounded wait inside a kernel ran out

typedef __nv_bfloat16 bf16;

template <typename T> struct fx_code;
template <> struct fx_code<float> { static constexpr int value = FX_F32; };
template <> struct fx_code<bf16> { static constexpr int value = FX_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Read element i of an array whose element type is only known at run time
// (small tensors that keep their stored precision: norm weights, biases).
__device__ __forceinline__ float load_any(const void* p, int dtype, long i) {
    return dtype == FX_F32 ? reinterpret_cast<const float*>(p)[i]
                           : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. The order
// of additions is fixed by the thread layout alone.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Key range [k_begin, k_end) of run `split` of a decoding token at position pos whose first visible key is lo.
// split_len > 0: runs of split_len keys counted from position 0.  split_len == 0: the token's own visible keys,
// counted from the multiple of 64 at or below lo, cut into n_splits runs of equal length (a multiple of 64), so
// that every run has work whatever the context length is.  An empty range (k_begin >= k_end) has no block
// result and is skipped when the runs are merged.
__device__ __forceinline__ void fx_split_range(int pos, int lo, int split, int n_splits, int split_len, int& k_begin,
                                               int& k_end) {
    int base = 0, len = split_len;
    if (split_len <= 0) {
        base = lo & ~63;
        len = (((pos + 1 - base) + n_splits - 1) / n_splits + 63) & ~63;
    }
    k_begin = max(lo, base + split * len);
    k_end = min(pos + 1, base + (split + 1) * len);
}

// Programmatic dependent launch.  A kernel launched with fx_launch_pdl may be set up
// on the GPU while the kernel before it on the stream is still running; it must
// call fx_pdl_wait() before it touches anything that kernel wrote (here: first
// thing), which also lets the kernel after it start its own set-up.  Launch
// latencies of a chain of short kernels then overlap instead of adding up.
__device__ __forceinline__ void fx_pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// fx_set_pdl(0) (elementwise.cu) makes fx_launch_pdl launch without the attribute; for measurements.
extern int g_fx_pdl_enabled;

template <typename... KArgs, typename... Args>
static inline void fx_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_fx_pdl_enabled ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface through cudaGetLastError
}

static inline int fx_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FX_OK : (int)e;
}

static inline long fx_cdiv(long a, long b) { return (a + b - 1) / b; }

// Streaming multiprocessors of the current device, asked once (elementwise.cu); grids are sized by it.
extern "C" int fx_sm_count();
