// Choice of the next token from 32-bit logits: greedy argmax, or temperature
// softmax with optional top-k / top-p filters and an inverse-CDF draw, after the
// repetition penalty.  One block per row of logits.
//
// Reference: crates/ferrox-models/src/sampling.rs:93-189 (order of operations:
// penalties, /temperature, softmax, top-k, top-p, renormalise, draw; the first
// index whose running sum exceeds the draw is taken) and :191-202 (penalty:
// positive logits are divided, negative ones multiplied, once per occurrence in
// the history of generated tokens).
// Differences, all on exact ties only: argmax takes the lowest index among equal
// maxima (the reference's `max_by` takes the last); top-k keeps every probability
// equal to the k-th largest; top-p keeps every probability equal to the one that
// crosses the threshold.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int NT = 1024;

__global__ void __launch_bounds__(NT) argmax_kernel(const float* __restrict__ logits, long ld, int vocab,
                                                    int* __restrict__ out)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    fx_pdl_wait();
    const float* row = logits + (long)blockIdx.x * ld;
    float best = -INFINITY; int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += NT) {
        const float v = row[i];
        if (v > best || best_i == 0x7fffffff) { best = v; best_i = i; }
    }
    // NaN never wins a '>' comparison; a row of NaNs yields its first visited index.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = sv[lane]; best_i = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
        }
        if (lane == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

// work[row, tok] is penalised once per occurrence of tok in the row's history.
__global__ void penalty_kernel(float* __restrict__ work, long ld, int vocab, const int* __restrict__ history,
                               const int* __restrict__ hist_offsets, const float* __restrict__ penalty)
{
    const int r = blockIdx.x;
    if (threadIdx.x != 0) return;
    const float p = penalty[r];
    if (p == 1.0f) return;
    float* row = work + (long)r * ld;
    for (int i = hist_offsets[r]; i < hist_offsets[r + 1]; ++i) {
        const int tok = history[i];
        if (tok < 0 || tok >= vocab) continue;
        const float s = row[tok];
        row[tok] = s > 0.f ? s / p : s * p;
    }
}

__device__ __forceinline__ float block_max(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) { float t = warp_max(scratch[lane]); if (lane == 0) scratch[32] = t; }
    __syncthreads();
    return scratch[32];
}

// Sum of the probabilities whose bit pattern is >= bits (probabilities are >= 0,
// so the unsigned order of the patterns is the numeric order), and their count.
__device__ __forceinline__ void mass_at_least(const float* p, int vocab, unsigned bits, float* scratch,
                                              float* mass, float* count)
{
    float s = 0.f, c = 0.f;
    for (int i = threadIdx.x; i < vocab; i += NT) {
        const float v = p[i];
        if (__float_as_uint(v) >= bits && v > 0.f) { s += v; c += 1.f; }
    }
    *mass = block_sum(s, scratch);
    *count = block_sum(c, scratch);
}

// work: scores in, probabilities out (in place).  temperature > 0.
// With `scores` the scores are read from there and `work` is written only.  With `use_sample` and `instead` a row
// whose flag is 0, or whose candidates were all filtered away, gets instead[r] (the arg max of its untouched scores):
// the whole choice of a step in one launch, for steps replayed from a CUDA graph.
__global__ void __launch_bounds__(NT) sample_kernel(float* __restrict__ work, long ld, int vocab,
                                                    const float* __restrict__ temperature,
                                                    const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                    const float* __restrict__ draw, int* __restrict__ out,
                                                    const float* __restrict__ scores, long lds,
                                                    const int* __restrict__ use_sample, const int* __restrict__ instead)
{
    __shared__ float scratch[33];
    __shared__ float chunk_sum[NT];
    __shared__ int chosen;
    fx_pdl_wait();
    const int r = blockIdx.x;
    if (use_sample && !use_sample[r]) {
        if (threadIdx.x == 0) out[r] = instead[r];
        return;
    }
    float* p = work + (long)r * ld;
    const float* src = scores ? scores + (long)r * lds : p;
    const float inv_t = 1.0f / temperature[r];

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += NT) mx = fmaxf(mx, src[i] * inv_t);
    mx = block_max(mx, scratch);
    float sum = 0.f;
    for (int i = threadIdx.x; i < vocab; i += NT) { const float e = expf(src[i] * inv_t - mx); p[i] = e; sum += e; }
    sum = block_sum(sum, scratch);
    for (int i = threadIdx.x; i < vocab; i += NT) p[i] = sum > 0.f ? p[i] / sum : 1.0f / (float)vocab;
    __syncthreads();

    // threshold below which probabilities are dropped (bit pattern; 0 keeps all)
    unsigned keep_bits = 0u;
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
        // largest pattern b with count(p >= b) >= k, by bisection over the 31 value bits
        unsigned lo = 0u, hi = 0x7f800000u;  // invariant: count(lo) >= k, count(hi) < k (no p is +inf)
        while (hi - lo > 1u) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            float mass, cnt;
            mass_at_least(p, vocab, mid, scratch, &mass, &cnt);
            if (cnt >= (float)k) lo = mid; else hi = mid;
        }
        keep_bits = lo;
    }
    const float tp = top_p[r];
    if (tp < 1.0f) {
        // largest pattern b >= keep_bits with mass(p >= b) >= top_p; if even the whole
        // kept mass stays below top_p nothing more is dropped.
        float mass, cnt;
        mass_at_least(p, vocab, keep_bits, scratch, &mass, &cnt);
        if (mass >= tp) {
            unsigned lo = keep_bits, hi = 0x7f800000u;
            while (hi - lo > 1u) {
                const unsigned mid = lo + ((hi - lo) >> 1);
                mass_at_least(p, vocab, mid, scratch, &mass, &cnt);
                if (mass >= tp) lo = mid; else hi = mid;
            }
            keep_bits = lo;
        }
    }

    // inverse CDF over the kept probabilities, in index order
    const int per = (vocab + NT - 1) / NT;
    const int c0 = threadIdx.x * per, c1 = min(vocab, c0 + per);
    float local = 0.f;
    for (int i = c0; i < c1; ++i) { const float v = p[i]; if (__float_as_uint(v) >= keep_bits && v > 0.f) local += v; }
    chunk_sum[threadIdx.x] = local;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int i = 0; i < NT; ++i) total += chunk_sum[i];
        if (total <= 0.f) {
            chosen = -2;  // degenerate filters: the caller falls back to argmax of the logits
        } else {
            const float target = draw[r] * total;
            float run = 0.f; int c = NT - 1;
            for (int i = 0; i < NT; ++i) { if (target < run + chunk_sum[i]) { c = i; break; } run += chunk_sum[i]; }
            // walk the chunk; if rounding leaves the draw above the last sum, the last kept token stands
            int pick = -1, last = -1;
            for (int cc = c; cc < NT && pick < 0; ++cc) {
                const int b0 = cc * per, b1 = min(vocab, b0 + per);
                for (int i = b0; i < b1; ++i) {
                    const float v = p[i];
                    if (!(__float_as_uint(v) >= keep_bits && v > 0.f)) continue;
                    last = i; run += v;
                    if (target < run) { pick = i; break; }
                }
            }
            if (pick < 0) {
                if (last < 0) for (int i = vocab - 1; i >= 0; --i) { const float v = p[i]; if (__float_as_uint(v) >= keep_bits && v > 0.f) { last = i; break; } }
                pick = last < 0 ? 0 : last;
            }
            chosen = pick;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out[r] = (instead && chosen < 0) ? instead[r] : chosen;
}

}  // namespace

extern "C" int fx_argmax(const float* logits, long ld, int n_rows, int vocab, int* out, void* stream)
{
    if (n_rows <= 0) return FX_OK;
    fx_launch_pdl(argmax_kernel, n_rows, NT, 0, (cudaStream_t)stream, logits, ld, vocab, out);
    return fx_launch_status();
}

extern "C" int fx_repetition_penalty(float* work, long ld, int n_rows, int vocab, const int* history,
                                     const int* hist_offsets, const float* penalty, void* stream)
{
    if (n_rows <= 0) return FX_OK;
    penalty_kernel<<<n_rows, 32, 0, (cudaStream_t)stream>>>(work, ld, vocab, history, hist_offsets, penalty);
    return fx_launch_status();
}

// out[r] = sampled index, or -2 when every candidate was filtered away.
extern "C" int fx_sample(float* work, long ld, int n_rows, int vocab, const float* temperature, const int* top_k,
                         const float* top_p, const float* draw, int* out, void* stream)
{
    if (n_rows <= 0) return FX_OK;
    sample_kernel<<<n_rows, NT, 0, (cudaStream_t)stream>>>(work, ld, vocab, temperature, top_k, top_p, draw, out,
                                                           nullptr, 0, nullptr, nullptr);
    return fx_launch_status();
}

// The choice of a whole step: row r gets a sample of scores[r] (temperature, top-k, top-p, draw as in fx_sample) if
// use_sample[r], else instead[r]; also instead[r] when every candidate of the row was filtered away.  `scores` is
// left untouched, `work` ([n_rows, vocab] floats) is scratch.
extern "C" int fx_sample_or(const float* scores, long lds, float* work, long ld, int n_rows, int vocab,
                            const float* temperature, const int* top_k, const float* top_p, const float* draw,
                            const int* use_sample, const int* instead, int* out, void* stream)
{
    if (n_rows <= 0) return FX_OK;
    if (!scores || !use_sample || !instead) return FX_ERR_SIZE;
    fx_launch_pdl(sample_kernel, n_rows, NT, 0, (cudaStream_t)stream, work, ld, vocab, temperature, top_k, top_p, draw, out,
                  scores, lds, use_sample, instead);
    return fx_launch_status();
}
