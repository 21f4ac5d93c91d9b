// Memory-bound kernels around the matrix products: embedding rows, RMSNorm,
// rotary encoding fused with the write of K and V into cache pages, SiLU*up.
// All arithmetic is 32-bit; only loads and stores use the tensor's element type.
#include "common.cuh"
#include "api.h"

int g_fx_pdl_enabled = 1;

extern "C" int fx_set_pdl(int on)
{
    const int was = g_fx_pdl_enabled;
    g_fx_pdl_enabled = on ? 1 : 0;
    return was;
}

extern "C" int fx_sm_count()
{
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) n = v;
        else return 148;   // no answer (no device yet): the B200's count, not remembered
    }
    return n;
}

namespace {

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = table[ids[t], :] widened to 32-bit (the residual stream
// is 32-bit in both engines).  Reference: decoder.rs:1279, 3032-3035.
// A token id outside [0, vocab) writes zeros and raises *status.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int hidden, int vocab, int* __restrict__ status)
{
    fx_pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0 && status) atomicExch(status, 1);
    const T* row = table + (long)(ok ? id : 0) * hidden;
    float* o = out + (long)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.f;
}

// ---------------------------------------------------------------------------
// RMSNorm: out = x * (1/sqrt(mean(x^2) + eps)) * w, multiplied in that order
// (reference: crates/ferrox-core/src/matmul.rs:62-69,121-123).  x is the 32-bit
// residual stream; `rows` (optional) picks the rows to normalise, which is how the
// final norm runs only at the positions whose logits are wanted.
template <typename OT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const void* __restrict__ w, int w_dtype, float eps,
                               OT* __restrict__ out, int hidden)
{
    __shared__ float scratch[33];
    fx_pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (long)(rows ? rows[r] : r) * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    OT* o = out + (long)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = from_f32<OT>(xr[i] * scale * load_any(w, w_dtype, i));
}

// ---------------------------------------------------------------------------
// SiLU(gate) * up over rows of [gate | up] (two halves of width n side by side).
// silu(x) = x / (1 + exp(-x)) (reference: matmul.rs:268-280).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, long ld_in, T* __restrict__ out, long ld_out,
                                const int* __restrict__ n_rows_dev, int rows, int n)
{
    const long total = (long)(n_rows_dev ? *n_rows_dev : rows) * n;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / n; const int c = (int)(i - r * n);
        const float g = to_f32(gu[r * ld_in + c]);
        const float u = to_f32(gu[r * ld_in + n + c]);
        out[r * ld_out + c] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// ---------------------------------------------------------------------------
// Rotary encoding of q and k, and the write of k and v into their cache pages, in
// one pass over the fused q|k|v rows.
//   angle = pos * inv_freq[i];  (a, b) <- (a cos - b sin, a sin + b cos)
// where pair i is (x_i, x_{i+r/2}) for pairing 0 (split halves; reference:
// crates/ferrox-core/src/attention.rs:20-32) and (x_2i, x_2i+1) for pairing 1
// (adjacent elements; attention.rs:340-352); the table inv_freq carries whatever
// per-band frequencies the position part wants (attention.rs:319-337 divides them
// by factors).  Applied per head at the token's absolute position
// (decoder.rs:2106-2111, 3489-3507); K/V append decoder.rs:2123-2125, paged
// cache.rs:382-404.  Elements beyond `rotary_dim` pass through.  `inv_freq == nullptr` means no rotation (position encoding none).
// `cos_sin` (optional, [tokens, rotary_dim/2, 2]) holds cos and sin of exactly these
// angles, made once per step by rope_table_kernel for all layers that share them.
// Page layout: [page][kv_head][token_in_page][head_dim].
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, long ld, const int* __restrict__ positions,
                                     const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                     const float* __restrict__ inv_freq, const float* __restrict__ cos_sin,
                                     int rotary_dim, int pairing, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const int* __restrict__ block_table, int table_width, int page_size,
                                     int n_heads, int n_kv_heads, int head_dim, int write_cache,
                                     int* __restrict__ status)
{
    fx_pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    T* row = qkv + (long)t * ld;
    const int half = rotary_dim >> 1;
    long page_base = -1;
    if (write_cache) {
        const int slot = seq_slot[token_seq[t]];
        const int page = block_table[(long)slot * table_width + pos / page_size];
        if (page < 0) { if (threadIdx.x == 0 && status) atomicExch(status, 2); }
        else page_base = ((long)page * n_kv_heads * page_size + (pos % page_size)) * head_dim;
    }
    const int n_rot_heads = n_heads + n_kv_heads;
    // rotate q and k heads in place
    if (inv_freq) {
        for (int idx = threadIdx.x; idx < n_rot_heads * half; idx += blockDim.x) {
            const int h = idx / half, i = idx - h * half;
            float s, c;
            if (cos_sin) {
                const float2 cs = *reinterpret_cast<const float2*>(cos_sin + ((long)t * half + i) * 2);
                c = cs.x; s = cs.y;
            } else {
                sincosf((float)pos * inv_freq[i], &s, &c);
            }
            T* x = row + (long)h * head_dim;
            const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
            const float a = to_f32(x[ia]), b = to_f32(x[ib]);
            x[ia] = from_f32<T>(a * c - b * s);
            x[ib] = from_f32<T>(a * s + b * c);
        }
    }
    if (page_base < 0) return;
    __syncthreads();
    const T* k = row + (long)n_heads * head_dim;
    const T* v = k + (long)n_kv_heads * head_dim;
    for (int idx = threadIdx.x; idx < n_kv_heads * head_dim; idx += blockDim.x) {
        const int h = idx / head_dim, i = idx - h * head_dim;
        const long dst = page_base + (long)h * page_size * head_dim + i;
        k_pages[dst] = k[idx];
        v_pages[dst] = v[idx];
    }
}

// cos_sin[t, i] = (cos, sin)(pos_t * inv_freq[i]), 32-bit angle and functions.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int n_tokens,
                                  int half, float* __restrict__ cos_sin)
{
    fx_pdl_wait();
    const long n = (long)n_tokens * half;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < n; idx += (long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / half), i = (int)(idx - (long)t * half);
        float s, c;
        sincosf((float)positions[t] * inv_freq[i], &s, &c);
        cos_sin[idx * 2] = c;
        cos_sin[idx * 2 + 1] = s;
    }
}

// ---------------------------------------------------------------------------
// h[t,:] += sum_k w[t,k] * y[inv_perm[t*K+k], :]  (rank order k = 0..K-1)
//          + (gate ? sigmoid(gate[t]) : 1) * shared[t,:]
// (reference: crates/ferrox-moe/src/lib.rs:735-752; sigmoid gate on the shared
// expert decoder.rs:2660-2681).  The sum per token has a fixed order, so it does
// not depend on what else is in the batch.
template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ h, const T* __restrict__ y, const int* __restrict__ inv_perm,
                                   const float* __restrict__ topk_w, int top_k,
                                   const T* __restrict__ shared, const float* __restrict__ shared_gate_logit,
                                   long gate_ld, int hidden)
{
    fx_pdl_wait();
    const int t = blockIdx.x;
    float g = 1.f;
    if (shared && shared_gate_logit) g = 1.0f / (1.0f + expf(-shared_gate_logit[(long)t * gate_ld]));
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top_k; ++k) {
            const long r = inv_perm[(long)t * top_k + k];
            acc = fmaf(topk_w[(long)t * top_k + k], to_f32(y[r * hidden + i]), acc);
        }
        if (shared) acc = fmaf(g, to_f32(shared[(long)t * hidden + i]), acc);
        h[(long)t * hidden + i] += acc;
    }
}

// out[r, :] = x[rows[r], :]  (tokens brought into expert order for the grouped products)
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, long ldx, const int* __restrict__ rows,
                                   T* __restrict__ out, long ldo, int width, int vec_ok)
{
    fx_pdl_wait();
    const int r = blockIdx.x;
    const T* src = x + (long)rows[r] * ldx;
    T* dst = out + (long)r * ldo;
    if (vec_ok) {
        constexpr int V = 16 / sizeof(T);
        for (int i = threadIdx.x; i < width / V; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

// h[t,:] += y[t,:]
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ h, const T* __restrict__ y, long n)
{
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        h[i] += to_f32(y[i]);
}

// ---------------------------------------------------------------------------
// 16-byte vector forms of the kernels above, used when widths and addresses allow.
template <typename T> struct Pack;
template <> struct Pack<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* o) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* o) {
        *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
    }
};
template <> struct Pack<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16* p, float* o) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(bf16* p, const float* o) {
        uint4 v;
        __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
        __nv_bfloat162 c = __floats2bfloat162_rn(o[4], o[5]), d = __floats2bfloat162_rn(o[6], o[7]);
        v.x = *reinterpret_cast<uint32_t*>(&a); v.y = *reinterpret_cast<uint32_t*>(&b);
        v.z = *reinterpret_cast<uint32_t*>(&c); v.w = *reinterpret_cast<uint32_t*>(&d);
        *reinterpret_cast<uint4*>(p) = v;
    }
};

// RMSNorm, 4 elements per thread and pass (hidden % 4 == 0, rows 16-byte aligned).
template <typename OT>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   const void* __restrict__ w, int w_dtype, float eps,
                                   OT* __restrict__ out, int hidden)
{
    __shared__ float scratch[33];
    fx_pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (long)(rows ? rows[r] : r) * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    OT* o = out + (long)r * hidden;
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        float wv[4];
        if (w_dtype == FX_F32) {
            const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i);
            wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
        } else {
            const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(w) + i);
            wv[0] = __uint_as_float(t.x << 16); wv[1] = __uint_as_float(t.x & 0xffff0000u);
            wv[2] = __uint_as_float(t.y << 16); wv[3] = __uint_as_float(t.y & 0xffff0000u);
        }
        const float y0 = v.x * scale * wv[0], y1 = v.y * scale * wv[1], y2 = v.z * scale * wv[2], y3 = v.w * scale * wv[3];
        if (sizeof(OT) == 4) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + i) = make_float4(y0, y1, y2, y3);
        } else {
            __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
            uint2 pk; pk.x = *reinterpret_cast<uint32_t*>(&a); pk.y = *reinterpret_cast<uint32_t*>(&b);
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(o) + i) = pk;
        }
    }
}

// Rotary + cache write, 16 bytes per thread and pass.  Needs rotary_dim == head_dim, (head_dim / 2) a
// multiple of the vector width and 16-byte aligned rows; same arithmetic as the scalar kernel.
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, long ld, const int* __restrict__ positions,
                                         const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                         const float* __restrict__ inv_freq, const float* __restrict__ cos_sin,
                                         T* __restrict__ k_pages, T* __restrict__ v_pages,
                                         const int* __restrict__ block_table, int table_width, int page_size,
                                         int n_heads, int n_kv_heads, int head_dim, int write_cache,
                                         int* __restrict__ status)
{
    constexpr int V = Pack<T>::N;
    fx_pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    T* row = qkv + (long)t * ld;
    const int half = head_dim >> 1;
    long page_base = -1;
    if (write_cache) {
        const int slot = seq_slot[token_seq[t]];
        const int page = block_table[(long)slot * table_width + pos / page_size];
        if (page < 0) { if (threadIdx.x == 0 && status) atomicExch(status, 2); }
        else page_base = ((long)page * n_kv_heads * page_size + (pos % page_size)) * head_dim;
    }
    const int cph = half / V;                       // vector chunks per half head
    const int n_rot = (n_heads + n_kv_heads) * cph; // q and k heads: one item = a chunk of each half
    const int n_v = n_kv_heads * (head_dim / V);    // v heads: plain copies into the pages
    for (int idx = threadIdx.x; idx < n_rot + n_v; idx += blockDim.x) {
        if (idx < n_rot) {
            const int h = idx / cph, i = (idx - h * cph) * V;
            T* x = row + (long)h * head_dim;
            float a[V], b[V], ra[V], rb[V];
            Pack<T>::load(x + i, a);
            Pack<T>::load(x + i + half, b);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                float s, c;
                if (inv_freq == nullptr) { s = 0.f; c = 1.f; }
                else if (cos_sin) {
                    const float2 cs = *reinterpret_cast<const float2*>(cos_sin + ((long)t * half + i + e) * 2);
                    c = cs.x; s = cs.y;
                } else {
                    sincosf((float)pos * inv_freq[i + e], &s, &c);
                }
                ra[e] = a[e] * c - b[e] * s;
                rb[e] = a[e] * s + b[e] * c;
            }
            if (inv_freq) { Pack<T>::store(x + i, ra); Pack<T>::store(x + i + half, rb); }
            if (h >= n_heads && page_base >= 0) {
                T* dst = k_pages + page_base + (long)(h - n_heads) * page_size * head_dim;
                Pack<T>::store(dst + i, ra);
                Pack<T>::store(dst + i + half, rb);
            }
        } else if (page_base >= 0) {
            const int j = idx - n_rot;
            const int h = j / (head_dim / V), i = (j - h * (head_dim / V)) * V;
            const T* src = row + (long)(n_heads + n_kv_heads + h) * head_dim + i;
            T* dst = v_pages + page_base + (long)h * page_size * head_dim + i;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        }
    }
}

// Expert combine, 16 bytes of y per thread and pass (hidden a multiple of the vector width).
template <typename T>
__global__ void moe_combine_vec_kernel(float* __restrict__ h, const T* __restrict__ y, const int* __restrict__ inv_perm,
                                       const float* __restrict__ topk_w, int top_k,
                                       const T* __restrict__ shared, const float* __restrict__ shared_gate_logit,
                                       long gate_ld, int hidden)
{
    constexpr int V = Pack<T>::N;
    fx_pdl_wait();
    const int t = blockIdx.x;
    float g = 1.f;
    if (shared && shared_gate_logit) g = 1.0f / (1.0f + expf(-shared_gate_logit[(long)t * gate_ld]));
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * V; i < hidden; i += gridDim.y * blockDim.x * V) {
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
        for (int k = 0; k < top_k; ++k) {
            const long r = inv_perm[(long)t * top_k + k];
            const float w = topk_w[(long)t * top_k + k];
            float v[V];
            Pack<T>::load(y + r * hidden + i, v);
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = fmaf(w, v[e], acc[e]);
        }
        if (shared) {
            float v[V];
            Pack<T>::load(shared + (long)t * hidden + i, v);
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = fmaf(g, v[e], acc[e]);
        }
        float* hp = h + (long)t * hidden + i;
#pragma unroll
        for (int e = 0; e < V; e += 4) {
            float4 o = *reinterpret_cast<float4*>(hp + e);
            o.x += acc[e]; o.y += acc[e + 1]; o.z += acc[e + 2]; o.w += acc[e + 3];
            *reinterpret_cast<float4*>(hp + e) = o;
        }
    }
}

// The same combine with the RMSNorm that follows it (the next layer's first norm): one block takes a whole row,
// keeps the new residual values in registers, sums their squares and writes the normed row beside the residual
// stream.  Saves the norm's launch and its reading of the row.  A thread holds up to CH vectors of the row.
template <typename T, int CH>
__global__ void moe_combine_norm_kernel(float* __restrict__ h, const T* __restrict__ y, const int* __restrict__ inv_perm,
                                        const float* __restrict__ topk_w, int top_k,
                                        const T* __restrict__ shared, const float* __restrict__ shared_gate_logit,
                                        long gate_ld, int hidden, const void* __restrict__ norm_w, int norm_w_dtype,
                                        float eps, T* __restrict__ x_out)
{
    constexpr int V = Pack<T>::N;
    __shared__ float scratch[33];
    fx_pdl_wait();
    const int t = blockIdx.x;
    float g = 1.f;
    if (shared && shared_gate_logit) g = 1.0f / (1.0f + expf(-shared_gate_logit[(long)t * gate_ld]));
    float hv[CH][V];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * V;
        if (i >= hidden) continue;
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
        for (int k = 0; k < top_k; ++k) {
            const long r = inv_perm[(long)t * top_k + k];
            const float w = topk_w[(long)t * top_k + k];
            float v[V];
            Pack<T>::load(y + r * hidden + i, v);
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = fmaf(w, v[e], acc[e]);
        }
        if (shared) {
            float v[V];
            Pack<T>::load(shared + (long)t * hidden + i, v);
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = fmaf(g, v[e], acc[e]);
        }
        float* hp = h + (long)t * hidden + i;
#pragma unroll
        for (int e = 0; e < V; e += 4) {
            float4 o = *reinterpret_cast<float4*>(hp + e);
            o.x += acc[e]; o.y += acc[e + 1]; o.z += acc[e + 2]; o.w += acc[e + 3];
            *reinterpret_cast<float4*>(hp + e) = o;
            hv[c][e] = o.x; hv[c][e + 1] = o.y; hv[c][e + 2] = o.z; hv[c][e + 3] = o.w;
            ss = fmaf(o.x, o.x, ss); ss = fmaf(o.y, o.y, ss); ss = fmaf(o.z, o.z, ss); ss = fmaf(o.w, o.w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * V;
        if (i >= hidden) continue;
        float o[V];
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] = hv[c][e] * scale * load_any(norm_w, norm_w_dtype, i + e);
        Pack<T>::store(x_out + (long)t * hidden + i, o);
    }
}

inline int threads_for(int n) { int t = 32; while (t < n && t < 1024) t <<= 1; return t; }

}  // namespace

extern "C" int fx_embed(const void* table, int dtype, const int* ids, float* out, int n_tokens, int hidden,
                        int vocab, int* status, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = threads_for(hidden > 256 ? 256 : hidden);
    if (dtype == FX_F32) fx_launch_pdl(embed_kernel<float>, n_tokens, nt, 0, s, (const float*)table, ids, out, hidden, vocab, status);
    else if (dtype == FX_BF16) fx_launch_pdl(embed_kernel<bf16>, n_tokens, nt, 0, s, (const bf16*)table, ids, out, hidden, vocab, status);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_rmsnorm(const float* x, const int* rows, const void* w, int w_dtype, float eps, void* out,
                          int out_dtype, int n_rows, int hidden, void* stream)
{
    if (n_rows <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = threads_for(hidden / 4 > 32 ? hidden / 4 : 32);
    const bool vec = hidden % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)w % 16 == 0;
    if (vec) {
        const int vt = nt > 512 ? 512 : nt;
        if (out_dtype == FX_F32) fx_launch_pdl(rmsnorm_vec_kernel<float>, n_rows, vt, 0, s, x, rows, w, w_dtype, eps, (float*)out, hidden);
        else if (out_dtype == FX_BF16) fx_launch_pdl(rmsnorm_vec_kernel<bf16>, n_rows, vt, 0, s, x, rows, w, w_dtype, eps, (bf16*)out, hidden);
        else return FX_ERR_DTYPE;
        return fx_launch_status();
    }
    if (out_dtype == FX_F32) fx_launch_pdl(rmsnorm_kernel<float>, n_rows, nt, 0, s, x, rows, w, w_dtype, eps, (float*)out, hidden);
    else if (out_dtype == FX_BF16) fx_launch_pdl(rmsnorm_kernel<bf16>, n_rows, nt, 0, s, x, rows, w, w_dtype, eps, (bf16*)out, hidden);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_silu_mul(const void* gu, long ld_in, void* out, long ld_out, int dtype, const int* n_rows_dev,
                           int rows, int n, void* stream)
{
    if (rows <= 0 || n <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    long blocks = fx_cdiv((long)rows * n, 256);
    if (blocks > fx_sm_count() * 16L) blocks = fx_sm_count() * 16L;
    if (dtype == FX_F32) silu_mul_kernel<float><<<(unsigned)blocks, 256, 0, s>>>((const float*)gu, ld_in, (float*)out, ld_out, n_rows_dev, rows, n);
    else if (dtype == FX_BF16) silu_mul_kernel<bf16><<<(unsigned)blocks, 256, 0, s>>>((const bf16*)gu, ld_in, (bf16*)out, ld_out, n_rows_dev, rows, n);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_rope_kv_write(void* qkv, int dtype, long ld, const int* positions, const int* token_seq,
                                const int* seq_slot, const float* inv_freq, const float* cos_sin, int rotary_dim,
                                int pairing, void* k_pages,
                                void* v_pages, const int* block_table, int table_width, int page_size, int n_tokens,
                                int n_heads, int n_kv_heads, int head_dim, int write_cache, int* status, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (rotary_dim % 2 || rotary_dim > head_dim || page_size <= 0 || pairing < 0 || pairing > 1) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int work = (n_heads + n_kv_heads) * (head_dim / 2);
    const int nt = threads_for(work > 256 ? 256 : work);
    const int vw = dtype == FX_F32 ? 4 : 8;
    const int es = dtype == FX_F32 ? 4 : 2;
    const bool vec = ((rotary_dim == head_dim && pairing == 0) || inv_freq == nullptr) && (head_dim / 2) % vw == 0 && (ld * es) % 16 == 0 &&
                     (uintptr_t)qkv % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0;
    if (vec && (dtype == FX_F32 || dtype == FX_BF16)) {
        const int items = ((n_heads + n_kv_heads) * (head_dim / 2) + n_kv_heads * head_dim) / vw;
        const int vt = threads_for(items > 256 ? 256 : items);
        if (dtype == FX_F32)
            fx_launch_pdl(rope_kv_write_vec_kernel<float>, n_tokens, vt, 0, s, (float*)qkv, ld, positions, token_seq, seq_slot,
                          inv_freq, cos_sin, (float*)k_pages, (float*)v_pages, block_table, table_width, page_size, n_heads,
                          n_kv_heads, head_dim, write_cache, status);
        else
            fx_launch_pdl(rope_kv_write_vec_kernel<bf16>, n_tokens, vt, 0, s, (bf16*)qkv, ld, positions, token_seq, seq_slot,
                          inv_freq, cos_sin, (bf16*)k_pages, (bf16*)v_pages, block_table, table_width, page_size, n_heads,
                          n_kv_heads, head_dim, write_cache, status);
        return fx_launch_status();
    }
    if (dtype == FX_F32)
        fx_launch_pdl(rope_kv_write_kernel<float>, n_tokens, nt, 0, s, (float*)qkv, ld, positions, token_seq, seq_slot, inv_freq,
            cos_sin, rotary_dim, pairing, (float*)k_pages, (float*)v_pages, block_table, table_width, page_size, n_heads, n_kv_heads,
            head_dim, write_cache, status);
    else if (dtype == FX_BF16)
        fx_launch_pdl(rope_kv_write_kernel<bf16>, n_tokens, nt, 0, s, (bf16*)qkv, ld, positions, token_seq, seq_slot, inv_freq,
            cos_sin, rotary_dim, pairing, (bf16*)k_pages, (bf16*)v_pages, block_table, table_width, page_size, n_heads, n_kv_heads,
            head_dim, write_cache, status);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_rope_table(const int* positions, const float* inv_freq, int n_tokens, int half, float* cos_sin,
                             void* stream)
{
    if (n_tokens <= 0 || half <= 0) return FX_OK;
    long blocks = fx_cdiv((long)n_tokens * half, 128);
    if (blocks > fx_sm_count() * 8L) blocks = fx_sm_count() * 8L;
    fx_launch_pdl(rope_table_kernel, (unsigned)blocks, 128, 0, (cudaStream_t)stream, positions, inv_freq, n_tokens, half, cos_sin);
    return fx_launch_status();
}

extern "C" int fx_moe_combine(float* h, const void* y, int dtype, const int* inv_perm, const float* topk_w, int top_k,
                              const void* shared, const float* shared_gate_logit, long gate_ld, int n_tokens,
                              int hidden, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = threads_for(hidden > 128 ? 128 : hidden);
    const dim3 grid(n_tokens, (unsigned)fx_cdiv(hidden, nt));
    const int vw = dtype == FX_F32 ? 4 : 8;
    if (hidden % vw == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)shared % 16 == 0 &&
        (dtype == FX_F32 || dtype == FX_BF16)) {
        const int vt = threads_for(hidden / vw > 128 ? 128 : hidden / vw);
        const dim3 vgrid(n_tokens, (unsigned)fx_cdiv(hidden / vw, vt));
        if (dtype == FX_F32)
            fx_launch_pdl(moe_combine_vec_kernel<float>, vgrid, vt, 0, s, h, (const float*)y, inv_perm, topk_w, top_k,
                          (const float*)shared, shared_gate_logit, gate_ld, hidden);
        else
            fx_launch_pdl(moe_combine_vec_kernel<bf16>, vgrid, vt, 0, s, h, (const bf16*)y, inv_perm, topk_w, top_k,
                          (const bf16*)shared, shared_gate_logit, gate_ld, hidden);
        return fx_launch_status();
    }
    if (dtype == FX_F32)
        fx_launch_pdl(moe_combine_kernel<float>, grid, nt, 0, s, h, (const float*)y, inv_perm, topk_w, top_k,
                                                      (const float*)shared, shared_gate_logit, gate_ld, hidden);
    else if (dtype == FX_BF16)
        fx_launch_pdl(moe_combine_kernel<bf16>, grid, nt, 0, s, h, (const bf16*)y, inv_perm, topk_w, top_k,
                                                     (const bf16*)shared, shared_gate_logit, gate_ld, hidden);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

// fx_moe_combine and, on the new residual rows, the RMSNorm with weight `norm_w` into x_out (element type of y).
// Refuses (FX_ERR_SIZE / FX_ERR_ALIGN) rows it cannot keep in registers; the caller then runs the two kernels.
extern "C" int fx_moe_combine_norm(float* h, const void* y, int dtype, const int* inv_perm, const float* topk_w,
                                   int top_k, const void* shared, const float* shared_gate_logit, long gate_ld,
                                   int n_tokens, int hidden, const void* norm_w, int norm_w_dtype, float eps,
                                   void* x_out, void* stream)
{
    if (n_tokens <= 0) return FX_OK;
    if (dtype != FX_F32 && dtype != FX_BF16) return FX_ERR_DTYPE;
    const int vw = dtype == FX_F32 ? 4 : 8;
    if (hidden % vw) return FX_ERR_SIZE;
    if ((uintptr_t)y % 16 || (uintptr_t)h % 16 || (uintptr_t)shared % 16 || (uintptr_t)x_out % 16) return FX_ERR_ALIGN;
    const int vecs = hidden / vw;
    const int nt = threads_for(vecs > 256 ? 256 : vecs);
    const int ch = (int)fx_cdiv(vecs, nt);
    if (ch > 4) return FX_ERR_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
#define FX_GO(T, CH)                                                                                                \
    fx_launch_pdl(moe_combine_norm_kernel<T, CH>, n_tokens, nt, 0, s, h, (const T*)y, inv_perm, topk_w, top_k,       \
                  (const T*)shared, shared_gate_logit, gate_ld, hidden, norm_w, norm_w_dtype, eps, (T*)x_out)
    if (dtype == FX_F32) { if (ch <= 1) FX_GO(float, 1); else if (ch == 2) FX_GO(float, 2); else FX_GO(float, 4); }
    else { if (ch <= 1) FX_GO(bf16, 1); else if (ch == 2) FX_GO(bf16, 2); else FX_GO(bf16, 4); }
#undef FX_GO
    return fx_launch_status();
}

extern "C" int fx_gather_rows(const void* x, long ldx, const int* rows, void* out, long ldo, int dtype, int n_rows,
                              int width, void* stream)
{
    if (n_rows <= 0 || width <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int es = dtype == FX_F32 ? 4 : 2;
    const int vec_ok = (width * es) % 16 == 0 && (ldx * es) % 16 == 0 && (ldo * es) % 16 == 0 &&
                       (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0;
    if (dtype == FX_F32)
        fx_launch_pdl(gather_rows_kernel<float>, n_rows, 128, 0, s, (const float*)x, ldx, rows, (float*)out, ldo, width, vec_ok);
    else if (dtype == FX_BF16)
        fx_launch_pdl(gather_rows_kernel<bf16>, n_rows, 128, 0, s, (const bf16*)x, ldx, rows, (bf16*)out, ldo, width, vec_ok);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}

extern "C" int fx_residual_add(float* h, const void* y, int dtype, long n, void* stream)
{
    if (n <= 0) return FX_OK;
    cudaStream_t s = (cudaStream_t)stream;
    long blocks = fx_cdiv(n, 256);
    if (blocks > fx_sm_count() * 16L) blocks = fx_sm_count() * 16L;
    if (dtype == FX_F32) residual_add_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(h, (const float*)y, n);
    else if (dtype == FX_BF16) residual_add_kernel<bf16><<<(unsigned)blocks, 256, 0, s>>>(h, (const bf16*)y, n);
    else return FX_ERR_DTYPE;
    return fx_launch_status();
}
