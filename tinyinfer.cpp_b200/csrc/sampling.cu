// Temperature / top-k / top-p sampling of one token per row of logits, one block per row.
//
// With z = logits / T and e = exp(z - max z):
//   top-k keeps the k largest logits (all logits equal to the k-th largest are kept);
//   top-p then keeps, of those, the shortest run of largest logits whose share of the kept
//         mass reaches p (the one that crosses p included; equal logits stay together);
//   the token is the first index, in vocabulary order, at which the running sum of the kept
//   e exceeds u times their total, u in [0, 1) being supplied by the caller per row.
// Both filters are thresholds on the logit's order-preserving integer key.  All sums run in an
// order that depends on the row alone, so a row's result does not depend on the other rows.
// Rows with T <= 0 take the argmax (lowest index wins).
//
// How the thresholds are found: the k-th largest key by a radix select, four passes over the row
// with a 256-bin histogram each.  The few logits that survive (at most CANDIDATES; with top-p but
// no top-k the CANDIDATES largest are tried, which hold the wanted mass unless the distribution
// is very flat) are then gathered into shared memory, put into vocabulary order, and top-p and
// the draw are settled among them without another pass over the row.  Whatever does not fit that
// scheme (more survivors than CANDIDATES) takes the general way: thresholds found bit by bit
// with one pass over the row per bit.  Without either filter the draw is one pass in which every
// warp scans a contiguous part of the row.
// The reference samples on the host after sorting (src/main.cpp:30-84).
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;
constexpr int WARPS = THREADS / 32;
constexpr int CANDIDATES = 1024;

__device__ __forceinline__ unsigned order_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned block_max_u(unsigned v, unsigned* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    unsigned r = lane < WARPS ? scratch[lane] : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = max(r, __shfl_xor_sync(0xffffffffu, r, o));
    return r;
}

// f(i, x[i]) for every element of the row, dealt to the block's threads; 16 bytes a load and four
// loads in flight where the row allows it (a pass over a row of 150,000 logits is bound by what
// a single SM has in flight: 22 microseconds with 4-byte loads).
template <class F>
__device__ __forceinline__ void for_row(const float* __restrict__ x, int vocab, F f) {
    if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const int n4 = vocab >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x);
#pragma unroll 4
        for (int i = threadIdx.x; i < n4; i += THREADS) {
            const float4 v = x4[i];
            f(4 * i, v.x); f(4 * i + 1, v.y); f(4 * i + 2, v.z); f(4 * i + 3, v.w);
        }
        for (int i = (n4 << 2) + threadIdx.x; i < vocab; i += THREADS) f(i, x[i]);
    } else {
#pragma unroll 4
        for (int i = threadIdx.x; i < vocab; i += THREADS) f(i, x[i]);
    }
}

// The key of the k-th largest element of the row (1 <= k <= vocab): the histogram of one byte of
// the keys that agree with the bytes found so far, from the most significant byte down.
__device__ unsigned kth_largest_key(const float* __restrict__ x, int vocab, unsigned k, unsigned* hist,
                                    unsigned* shared_word) {
    unsigned prefix = 0u, mask = 0u, remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += THREADS) hist[i] = 0u;
        __syncthreads();
        for_row(x, vocab, [&](int, float v) {
            const unsigned key = order_key(v);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        });
        __syncthreads();
        if (threadIdx.x < 32) {
            // lane l looks at bins 255 - 8l .. 248 - 8l; the bin in which the count from the top
            // reaches `remaining` holds the wanted key
            const int lane = threadIdx.x;
            unsigned mine = 0u;
#pragma unroll
            for (int j = 0; j < 8; ++j) mine += hist[255 - (lane * 8 + j)];
            unsigned above = mine;                       // inclusive scan over the lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned up = __shfl_up_sync(0xffffffffu, above, o);
                if (lane >= o) above += up;
            }
            above -= mine;                               // keys in the bins above this lane's
            if (above < remaining && remaining <= above + mine) {
                unsigned cum = above;
                for (int j = 0; j < 8; ++j) {
                    const unsigned bin = 255u - (unsigned)(lane * 8 + j);
                    if (remaining <= cum + hist[bin]) {
                        shared_word[0] = bin;
                        shared_word[1] = remaining - cum;
                        break;
                    }
                    cum += hist[bin];
                }
            }
        }
        __syncthreads();
        prefix |= shared_word[0] << shift;
        mask |= 255u << shift;
        remaining = shared_word[1];
        __syncthreads();
    }
    return prefix;
}

// Exclusive prefix sums of vals[0 .. n) (n <= CANDIDATES) into pre[0 .. n], pre[n] the total, by
// warp 0: a lane adds its 32 consecutive values in order, the lanes' sums are scanned in order.
__device__ void ordered_prefix(const float* vals, int n, float* pre) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        constexpr int PER = CANDIDATES / 32;
        float local = 0.0f;
        for (int j = 0; j < PER; ++j) {
            const int i = lane * PER + j;
            if (i < n) local += vals[i];
        }
        float incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        float run = incl - local;
        for (int j = 0; j < PER; ++j) {
            const int i = lane * PER + j;
            if (i < n) {
                pre[i] = run;
                run += vals[i];
            }
        }
        if (lane == 31) pre[n] = incl;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float fs[32];
    __shared__ unsigned us[32];
    __shared__ unsigned hist[256];
    __shared__ unsigned word[2];
    __shared__ int chosen, last;
    __shared__ unsigned found;
    __shared__ int c_idx[CANDIDATES], s_idx[CANDIDATES];
    __shared__ float c_val[CANDIDATES], s_val[CANDIDATES], s_e[CANDIDATES], pre[CANDIDATES + 1];
    const int row = blockIdx.x, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * vocab;
    const float temp = temperature[row];

    float mx = -INFINITY;
    for_row(x, vocab, [&](int, float v) { mx = fmaxf(mx, v); });
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
    const int k = top_k[row];
    const float p = top_p[row];
    const bool has_k = k > 0 && k < vocab;
    const bool has_p = p < 1.0f;
    unsigned thr = 0u;                          // keys below it are out

    if (has_k || has_p) {
        // ---- the survivors as a short list -------------------------------------------------
        const unsigned want_k = has_k ? (unsigned)k : (unsigned)min(vocab, CANDIDATES);
        thr = kth_largest_key(x, vocab, want_k, hist, word);
        if (tid == 0) found = 0u;
        __syncthreads();
        for_row(x, vocab, [&](int i, float v) {
            if (order_key(v) >= thr) {
                const unsigned slot = atomicAdd(&found, 1u);
                if (slot < CANDIDATES) { c_idx[slot] = i; c_val[slot] = v; }
            }
        });
        __syncthreads();
        const int n = (int)found;
        bool listed = n <= CANDIDATES;
        float all_mass = 0.0f;
        if (listed && !has_k) {
            // top-p alone: the list is the CANDIDATES largest; it decides only if it holds the
            // wanted share of the whole row's mass
            float s = 0.0f;
            for_row(x, vocab, [&](int, float v) { s += expf((v - mx) * inv_t); });
            all_mass = block_sum(s, fs);
        }
        if (listed) {
            // into vocabulary order: an entry's place is the number of entries with a smaller index
            for (int t = tid; t < n; t += THREADS) {
                const int mine = c_idx[t];
                int place = 0;
                for (int j = 0; j < n; ++j) place += c_idx[j] < mine;
                s_idx[place] = mine;
                s_val[place] = c_val[t];
                s_e[place] = expf((c_val[t] - mx) * inv_t);
            }
            __syncthreads();
            ordered_prefix(s_e, n, pre);
            float total = pre[n];
            if (!has_k && !(total >= p * all_mass)) listed = false;       // too flat for the list
            unsigned cut = 0u;                   // top-p's threshold (everything listed passes top-k)
            if (listed && has_p) {
                // the largest key c whose share mass(key >= c) reaches p of the total (of the whole
                // row's mass when there is no top-k: the list holds all larger keys)
                const float want = p * (has_k ? total : all_mass);
                unsigned best = 0u;
                for (int t = tid; t < n; t += THREADS) {
                    const unsigned mine = order_key(s_val[t]);
                    float mass = 0.0f;
                    for (int j = 0; j < n; ++j)
                        if (order_key(s_val[j]) >= mine) mass += s_e[j];
                    if (mass >= want) best = max(best, mine);
                }
                cut = block_max_u(best, us);
                __syncthreads();
                for (int t = tid; t < n; t += THREADS)
                    if (order_key(s_val[t]) < cut) s_e[t] = 0.0f;
                __syncthreads();
                ordered_prefix(s_e, n, pre);
                total = pre[n];
            }
            if (listed) {
                // first entry, in vocabulary order, at which the running sum exceeds u * total
                const float target = uniform[row] * total;
                if (tid == 0) { chosen = 0x7fffffff; last = -1; }
                __syncthreads();
                for (int t = tid; t < n; t += THREADS) {
                    if (order_key(s_val[t]) < cut) continue;
                    if (pre[t] + s_e[t] > target) atomicMin(&chosen, t);
                    atomicMax(&last, t);
                }
                __syncthreads();
                if (tid == 0) out[row] = s_idx[chosen != 0x7fffffff ? chosen : max(last, 0)];
                return;
            }
        }
        if (!has_k) thr = 0u;                   // the general way starts from the whole row
        __syncthreads();
    }

    // ---- the general way: one pass over the row per decision ------------------------------------
    float s = 0.0f;
    for_row(x, vocab, [&](int, float v) { if (order_key(v) >= thr) s += expf((v - mx) * inv_t); });
    float total = block_sum(s, fs);

    if (has_p) {
        // threshold from top-p: the largest key c with mass(key >= c) >= p * total, bit by bit
        const float want = p * total;
        unsigned thr_p = 0u;                      // the top-k cut stays in force
        for (int b = 31; b >= 0; --b) {
            const unsigned trial = thr_p | (1u << b);
            const unsigned cut = trial > thr ? trial : thr;
            float ms = 0.0f;
            for (int i = tid; i < vocab; i += THREADS)
                if (order_key(x[i]) >= cut) ms += expf((x[i] - mx) * inv_t);
            if (block_sum(ms, fs) >= want) thr_p = trial;
        }
        if (thr_p < thr) thr_p = thr;
        if (thr_p != thr) {
            thr = thr_p;
            s = 0.0f;
            for (int i = tid; i < vocab; i += THREADS)
                if (order_key(x[i]) >= thr) s += expf((x[i] - mx) * inv_t);
            total = block_sum(s, fs);
        }
    }

    // First index whose running sum exceeds u * total, in vocabulary order.  Every warp owns a
    // contiguous part of the row and adds it up in groups of 256 elements (a lane adds eight,
    // the lanes' sums are added once per group); the parts' sums are then added in order, and the
    // warp in whose part the target falls walks its groups again, the group that crosses the
    // target 32 elements at a time.
    const float target = uniform[row] * total;
    constexpr int GROUP = 256;
    const int part = ((vocab + WARPS - 1) / WARPS + GROUP - 1) / GROUP * GROUP;
    const int lo = min(vocab, warp * part), hi = min(vocab, lo + part);
    auto weight = [&](int i) {
        return i < hi && order_key(x[i]) >= thr ? expf((x[i] - mx) * inv_t) : 0.0f;
    };
    auto group_sum = [&](int base) {             // the same value in every lane
        float e = 0.0f;
#pragma unroll
        for (int j = 0; j < GROUP / 32; ++j) e += weight(base + j * 32 + lane);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
        return e;
    };
    float mine = 0.0f;
    for (int base = lo; base < hi; base += GROUP) mine += group_sum(base);
    if (tid == 0) { chosen = 0x7fffffff; last = -1; }
    __syncthreads();
    if (lane == 0) fs[warp] = mine;
    __syncthreads();
    float before = 0.0f;
    for (int w = 0; w < warp; ++w) before += fs[w];
    if (before <= target && target < before + mine) {
        float running = before;
        int found_at = -1, last_kept = -1;
        for (int base = lo; base < hi && found_at < 0; base += GROUP) {
            const float g = group_sum(base);
            if (!(running + g > target) && base + GROUP < hi) { running += g; continue; }
            for (int b2 = base; b2 < min(hi, base + GROUP); b2 += 32) {      // the group that crosses (or the last)
                const int i = b2 + lane;
                const float e = weight(i);
                const bool kept = i < hi && order_key(x[i]) >= thr;
                float incl = e;                  // inclusive scan inside the warp
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                const unsigned hit = __ballot_sync(0xffffffffu, kept && running + incl > target);
                const unsigned any = __ballot_sync(0xffffffffu, kept);
                if (hit) { found_at = b2 + __ffs(hit) - 1; break; }
                if (any) last_kept = b2 + 31 - __clz(any);
                running += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        // (rounding: the part's sum said the target lies here, the running sums did not reach it)
        if (lane == 0) atomicMin(&chosen, found_at >= 0 ? found_at : last_kept >= 0 ? last_kept : 0x7fffffff);
    }
    // the last kept index of the row, should rounding leave the target unreached altogether
    if (hi > lo) {
        int lk = -1;
        for (int base = ((hi - lo - 1) / 32) * 32 + lo; base >= lo && lk < 0; base -= 32) {
            const int i = base + lane;
            const unsigned any = __ballot_sync(0xffffffffu, i < hi && order_key(x[i]) >= thr);
            if (any) lk = base + 31 - __clz(any);
        }
        if (lane == 0 && lk >= 0) atomicMax(&last, lk);
    }
    __syncthreads();
    if (tid == 0) out[row] = chosen != 0x7fffffff ? chosen : max(last, 0);   // rounding left the target unreached: last kept
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
