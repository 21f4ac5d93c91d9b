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
    __shared__ int digit_count[256], digit_found, digit_above;
    __shared__ int walk_chunk, walk_last;
    __shared__ float walk_run, walk_target, group_sum[32];
    constexpr int LIST = 8;                      // probabilities a thread keeps after a top-k
    __shared__ float kept_list[NT][LIST];
    fx_pdl_wait();
    const int r = blockIdx.x;
    if (use_sample && !use_sample[r]) {
        if (threadIdx.x == 0) out[r] = instead[r];
        return;
    }
    float* p = work + (long)r * ld;
    const float* src = scores ? scores + (long)r * lds : p;
    const float temp = temperature[r];   // the scores are divided by it, as the reference does (sampling.rs:129-131)

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += NT) mx = fmaxf(mx, src[i] / temp);
    mx = block_max(mx, scratch);
    float sum = 0.f;
    for (int i = threadIdx.x; i < vocab; i += NT) { const float e = expf(src[i] / temp - mx); p[i] = e; sum += e; }
    sum = block_sum(sum, scratch);
    for (int i = threadIdx.x; i < vocab; i += NT) p[i] = sum > 0.f ? p[i] / sum : 1.0f / (float)vocab;
    __syncthreads();

    // threshold below which probabilities are dropped (bit pattern; 0 keeps all)
    unsigned keep_bits = 0u;
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
        // The pattern of the k-th largest probability = the largest pattern b with count(p >= b) >= k, found digit
        // by digit from the top (8, 8, 8 and 7 bits): a histogram of the digit over the probabilities that share the
        // digits found so far, then the digit in which the k-th largest lies.  Integer counts: the same answer in
        // every run.  Fewer than k probabilities above zero: nothing is dropped.
        unsigned prefix = 0u, prefix_mask = 0u;
        int remaining = k;
        for (int level = 0; level < 4 && remaining > 0; ++level) {
            const int shift = level == 0 ? 23 : (level == 1 ? 15 : (level == 2 ? 7 : 0));
            const unsigned digit_mask = level == 3 ? 0x7fu : 0xffu;
            for (int i = threadIdx.x; i < 256; i += NT) digit_count[i] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < vocab; i += NT) {
                const unsigned b = __float_as_uint(p[i]);
                if (b != 0u && (b & prefix_mask) == prefix) atomicAdd(&digit_count[(b >> shift) & digit_mask], 1);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int above = 0, d = (int)digit_mask;
                for (; d >= 0; --d) { if (above + digit_count[d] >= remaining) break; above += digit_count[d]; }
                digit_found = d;           // -1: fewer than `remaining` candidates in all
                digit_above = above;
            }
            __syncthreads();
            if (digit_found < 0) { prefix = 0u; remaining = 0; break; }
            prefix |= (unsigned)digit_found << shift;
            prefix_mask |= digit_mask << shift;
            remaining -= digit_above;
        }
        keep_bits = prefix;
    }
    const float tp = top_p[r];
    if (tp < 1.0f) {
        // largest pattern b >= keep_bits with mass(p >= b) >= top_p; if even the whole
        // kept mass stays below top_p nothing more is dropped.
        // After a top-k the few probabilities still kept are copied to shared memory, every thread its own (those it
        // meets in the loops above and below, in the same order), and the bisection sums those: the same sums as over
        // the whole row, bit for bit, without reading the row 31 times.
        int mine = 0;
        bool listed = false;
        if (keep_bits != 0u) {
            int overflow = 0;
            for (int i = threadIdx.x; i < vocab; i += NT) {
                const float v = p[i];
                if (__float_as_uint(v) >= keep_bits && v > 0.f) {
                    if (mine < LIST) kept_list[threadIdx.x][mine++] = v; else overflow = 1;
                }
            }
            listed = !__syncthreads_or(overflow);
        }
        auto mass_of = [&](unsigned bits, float* mass, float* cnt) {
            if (!listed) { mass_at_least(p, vocab, bits, scratch, mass, cnt); return; }
            float s2 = 0.f, c2 = 0.f;
            for (int j = 0; j < mine; ++j) {
                const float v = kept_list[threadIdx.x][j];
                if (__float_as_uint(v) >= bits) { s2 += v; c2 += 1.f; }
            }
            *mass = block_sum(s2, scratch);
            *cnt = block_sum(c2, scratch);
        };
        float mass, cnt;
        mass_of(keep_bits, &mass, &cnt);
        if (mass >= tp) {
            unsigned lo = keep_bits, hi = 0x7f800000u;
            while (hi - lo > 1u) {
                const unsigned mid = lo + ((hi - lo) >> 1);
                mass_of(mid, &mass, &cnt);
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
    // sums of 32 chunks each (32 threads side by side), then one thread: the group, then the chunk inside it
    static_assert(NT == 32 * 32, "two levels of 32");
    if (threadIdx.x < 32) {
        float g = 0.f;
        for (int i = 0; i < 32; ++i) g += chunk_sum[threadIdx.x * 32 + i];
        group_sum[threadIdx.x] = g;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int i = 0; i < 32; ++i) total += group_sum[i];
        if (total <= 0.f) {
            chosen = -2;  // degenerate filters: the caller falls back to argmax of the logits
        } else {
            const float target = draw[r] * total;
            float run = 0.f; int g = 31;
            for (int i = 0; i < 32; ++i) { if (target < run + group_sum[i]) { g = i; break; } run += group_sum[i]; }
            int c = g * 32 + 31;
            for (int i = g * 32; i < g * 32 + 32; ++i) { if (target < run + chunk_sum[i]) { c = i; break; } run += chunk_sum[i]; }
            walk_chunk = c; walk_run = run; walk_target = target; walk_last = -1;
        }
    }
    __syncthreads();
    if (chosen != -2) {
        // Walk the chunk in index order; if rounding leaves the draw above the last sum, the last kept token stands.
        // All threads bring the chunk to shared memory (one thread reading it element by element from global
        // memory takes ten times as long as the rest of the kernel), one thread walks it.
        float* stage = &kept_list[0][0];
        for (int cc = walk_chunk; cc < NT; ++cc) {
            const int b0 = cc * per, b1 = min(vocab, b0 + per);
            const bool staged = per <= NT * LIST;
            if (staged) for (int i = b0 + threadIdx.x; i < b1; i += NT) stage[i - b0] = p[i];
            __syncthreads();
            if (threadIdx.x == 0) {
                float run = walk_run;
                int last = walk_last;
                for (int i = b0; i < b1; ++i) {
                    const float v = staged ? stage[i - b0] : p[i];
                    if (!(__float_as_uint(v) >= keep_bits && v > 0.f)) continue;
                    last = i; run += v;
                    if (walk_target < run) { chosen = i; break; }
                }
                walk_run = run; walk_last = last;
            }
            __syncthreads();
            if (chosen >= 0) break;
        }
        if (threadIdx.x == 0 && chosen < 0) {
            int last = walk_last;
            if (last < 0) for (int i = vocab - 1; i >= 0; --i) { const float v = p[i]; if (__float_as_uint(v) >= keep_bits && v > 0.f) { last = i; break; } }
            chosen = last < 0 ? 0 : last;
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
