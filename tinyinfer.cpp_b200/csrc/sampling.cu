// Temperature / top-k / top-p sampling of one token per row of logits, one block per row.
//
// With z = logits / T and e = exp(z - max z):
//   top-k keeps the k largest logits (all logits equal to the k-th largest are kept);
//   top-p then keeps, of those, the shortest run of largest logits whose share of the kept
//         mass reaches p (the one that crosses p included; equal logits stay together);
//   the token is the first index, in vocabulary order, at which the running sum of the kept
//   e exceeds u times their total, u in [0, 1) being supplied by the caller per row.
// Both filters are thresholds on the logit's order-preserving integer key, found bit by
// bit with one pass over the row per bit; sums run in a fixed order, so a row's result
// does not depend on the other rows.  Rows with T <= 0 take the argmax (lowest index wins).
// The reference samples on the host after sorting (src/main.cpp:30-84).
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned order_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_sum_all(float v, float* scratch) { return block_sum(v, scratch); }

__device__ __forceinline__ unsigned block_count(unsigned v, unsigned* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    unsigned r = lane < (THREADS >> 5) ? scratch[lane] : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float fs[32];
    __shared__ unsigned us[32];
    __shared__ int chosen;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * vocab;
    const float temp = temperature[row];

    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += THREADS) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, fs);

    if (!(temp > 0.0f)) {                       // greedy: lowest index among the maxima
        int best = 0x7fffffff;
        for (int i = tid; i < vocab; i += THREADS)
            if (x[i] == mx) { best = i; break; }
        if (tid == 0) chosen = 0x7fffffff;
        __syncthreads();
        atomicMin(&chosen, best);
        __syncthreads();
        if (tid == 0) out[row] = chosen == 0x7fffffff ? 0 : chosen;
        return;
    }
    const float inv_t = 1.0f / temp;

    // threshold from top-k: the k-th largest key
    unsigned thr = 0u;
    const int k = top_k[row];
    if (k > 0 && k < vocab) {
        for (int b = 31; b >= 0; --b) {
            const unsigned trial = thr | (1u << b);
            unsigned c = 0;
            for (int i = tid; i < vocab; i += THREADS) c += order_key(x[i]) >= trial;
            if (block_count(c, us) >= (unsigned)k) thr = trial;
        }
    }
    // mass of what top-k kept
    float s = 0.0f;
    for (int i = tid; i < vocab; i += THREADS)
        if (order_key(x[i]) >= thr) s += expf((x[i] - mx) * inv_t);
    float total = block_sum_all(s, fs);

    // threshold from top-p: the largest key c with mass(key >= c) >= p * total
    const float p = top_p[row];
    if (p < 1.0f) {
        const float want = p * total;
        unsigned thr_p = 0u;                      // built bit by bit; the top-k cut stays in force
        for (int b = 31; b >= 0; --b) {
            const unsigned trial = thr_p | (1u << b);
            const unsigned cut = trial > thr ? trial : thr;
            float ms = 0.0f;
            for (int i = tid; i < vocab; i += THREADS)
                if (order_key(x[i]) >= cut) ms += expf((x[i] - mx) * inv_t);
            if (block_sum_all(ms, fs) >= want) thr_p = trial;
        }
        if (thr_p < thr) thr_p = thr;
        if (thr_p != thr) {
            thr = thr_p;
            s = 0.0f;
            for (int i = tid; i < vocab; i += THREADS)
                if (order_key(x[i]) >= thr) s += expf((x[i] - mx) * inv_t);
            total = block_sum_all(s, fs);
        }
    }

    // first index whose running sum exceeds u * total, in vocabulary order
    const float target = uniform[row] * total;
    __shared__ int last;
    if (tid == 0) { chosen = 0x7fffffff; last = -1; }
    float running = 0.0f;
    int last_kept = -1;
    const int lane = tid & 31, warp = tid >> 5;
    for (int base = 0; base < vocab; base += THREADS) {
        const int i = base + tid;
        const bool kept = i < vocab && order_key(x[i]) >= thr;
        const float e = kept ? expf((x[i] - mx) * inv_t) : 0.0f;
        float incl = e;                          // inclusive scan inside the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        __syncthreads();                         // fs is free again
        if (lane == 31) fs[warp] = incl;
        __syncthreads();
        float before = running, tile_total = 0.0f;
        for (int w = 0; w < (THREADS >> 5); ++w) {
            if (w == warp) before += tile_total;
            tile_total += fs[w];
        }
        if (kept && before + incl > target) atomicMin(&chosen, i);
        const unsigned ballot = __ballot_sync(0xffffffffu, kept);
        if (ballot) last_kept = base + warp * 32 + 31 - __clz(ballot);
        running += tile_total;
        __syncthreads();
        if (chosen != 0x7fffffff) break;
    }
    if (chosen == 0x7fffffff) {                  // rounding left the target unreached: last kept
        atomicMax(&last, last_kept);
        __syncthreads();
        if (tid == 0) out[row] = max(last, 0);
    } else if (tid == 0) {
        out[row] = chosen;
    }
}

}  // namespace

extern "C" int ti_sample(const float* logits, int rows, int vocab, const float* temperature,
                         const int* top_k, const float* top_p, const float* uniform, int* out,
                         void* stream) {
    if (rows == 0) return 0;
    TI_REQUIRE(vocab > 0, "sample: vocabulary size %d", vocab);
    sample_kernel<<<rows, THREADS, 0, (cudaStream_t)stream>>>(logits, vocab, temperature, top_k,
                                                              top_p, uniform, out);
    return ti_check_launch("sample");
}
