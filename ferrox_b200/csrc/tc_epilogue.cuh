// The way from an epilogue warp's registers to global memory, shared by the tcgen05 product kernels.
//
// A warp reads 32 lanes of tensor memory: lane = row of the tile, 32 columns a chunk.  Stored from there, one store
// instruction touches 32 rows 16 bytes each: 32 partial sectors, and the epilogue of a 128 x 256 tile takes 6 us (time
// stamps inside the kernel; the products of the next tile slow down beside it, and the last tile's epilogue is not
// hidden at all).  Instead the warp puts its chunk into a tile of its own in shared memory, rows of 128 bytes (two
// chunks of bfloat16 or one of 32-bit values), and writes it out with eight lanes a row: every store instruction is
// four whole 128-byte lines.
#pragma once
#include "common.cuh"

namespace fxtc {

constexpr int EPI_PITCH = 144;                    // bytes from one staged row to the next: 128 + 16, so that the
                                                  // 16-byte stores of eight lanes (a row each) meet different banks
constexpr int EPI_WARP_BYTES = 32 * EPI_PITCH;    // a warp's staging tile

// this lane's row: 32 values as bfloat16 into bytes [64 half, 64 half + 64) of its staged row
__device__ __forceinline__ void epi_stage_bf16(uint8_t* stage, int lane, int half, const float* v)
{
    uint4* dst = reinterpret_cast<uint4*>(stage + lane * EPI_PITCH + half * 64);
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]);
        __nv_bfloat162 p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
        __nv_bfloat162 p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        uint4 o;
        o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
        o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
        dst[j >> 3] = o;
    }
}

// this lane's row: 32 values of 32 bits, the whole staged row
__device__ __forceinline__ void epi_stage_f32(uint8_t* stage, int lane, const float* v)
{
    float4* dst = reinterpret_cast<float4*>(stage + lane * EPI_PITCH);
#pragma unroll
    for (int j = 0; j < 32; j += 4) dst[j >> 2] = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
}

// The staged 32 rows x 128 bytes to global memory: `c` points at the first staged byte of the warp's first row,
// rows `pitch` bytes apart, the first `rows_ok` of them exist.  add_f32: the staged values are 32-bit and are added
// to what is there.  The caller puts __syncwarp() between staging and this, and after it before staging again.
__device__ __forceinline__ void epi_flush(const uint8_t* stage, int lane, uint8_t* c, long pitch, int rows_ok, bool add_f32)
{
    const int piece = lane & 7;
    if (add_f32) {
        float4 old[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int r = k * 4 + (lane >> 3);
            if (r < rows_ok) old[k] = *reinterpret_cast<const float4*>(c + (long)r * pitch + piece * 16);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int r = k * 4 + (lane >> 3);
            if (r < rows_ok) {
                const float4 s = *reinterpret_cast<const float4*>(stage + r * EPI_PITCH + piece * 16);
                *reinterpret_cast<float4*>(c + (long)r * pitch + piece * 16) =
                    make_float4(old[k].x + s.x, old[k].y + s.y, old[k].z + s.z, old[k].w + s.w);
            }
        }
        return;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int r = k * 4 + (lane >> 3);
        if (r < rows_ok)
            *reinterpret_cast<uint4*>(c + (long)r * pitch + piece * 16) = *reinterpret_cast<const uint4*>(stage + r * EPI_PITCH + piece * 16);
    }
}

}  // namespace fxtc
