// The work of one flash-decoding item: a warp, one split of the keys of one (row, kv head).
//
// Used by the flash-decoding kernels of attn_decode.cu (a block of one warp per item), with the
// queries ready in memory or prepared by the item itself.  See attn_decode.cu for the algorithm.
#pragma once

#include "common.cuh"

namespace attn_decode_core {


constexpr int TILE = 32;       // keys per tile
constexpr int STAGES = 3;
constexpr int MAX_SPLITS = 256;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;               // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                         unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {           // 2^x, 2 ulp, 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// out[:] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M = max_s m_s, by one warp, over the splits
// in ascending order, for H heads at once (1 or 2).  Other blocks of the same launch wrote the
// partial results, so every load is a round trip to L2, and the merge is the exposed tail of the
// kernel: all (m, l) pairs and the first sixteen partial outputs of every head are requested
// together, before anything is computed, and further splits sixteen at a time for all heads at
// once (a round trip per sixteen splits, not per eight and head: 64 splits of two heads took 14
// round trips after the first, now 3).  `wbuf` holds H * MAX_SPLITS floats of shared memory.
template <int H>
__device__ __forceinline__ void merge_heads(const float* part_o, const float* part_ml, const size_t (&base)[H],
                                            int num_splits, int head_dim, bf16* const (&out)[H], int lane,
                                            float* wbuf) {
    constexpr int PER_LANE = MAX_SPLITS / 32;                 // (m, l) pairs a lane holds per head
    const int d0 = lane * 4;                                  // dims lane*4 .. lane*4 + 3
    const bool has_dims = d0 < head_dim;
    constexpr int W = 16;                                     // splits per round
    float4 v[H][W];
    float2 ml[H][PER_LANE];
#pragma unroll
    for (int h = 0; h < H; ++h) {
#pragma unroll
        for (int u = 0; u < W; ++u)
            if (has_dims && u < num_splits)
                v[h][u] = __ldcg(reinterpret_cast<const float4*>(part_o + (base[h] + u) * head_dim + d0));
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int s = lane + 32 * i;
            ml[h][i] = s < num_splits ? __ldcg(reinterpret_cast<const float2*>(part_ml + (base[h] + s) * 2))
                                      : make_float2(-INFINITY, 0.0f);
        }
    }
    float total[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
        float mmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) mmax = fmaxf(mmax, ml[h][i].x);
        mmax = warp_max(mmax);
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int s = lane + 32 * i;
            if (s >= num_splits) break;
            const float wgt = ml[h][i].x == -INFINITY ? 0.0f : exp2f(ml[h][i].x - mmax);
            wbuf[h * MAX_SPLITS + s] = wgt;
            sum += ml[h][i].y * wgt;                              // lanes hold disjoint splits
        }
        // a fixed order of the additions: lane partial sums, then the shuffle tree
        total[h] = warp_sum(sum);
    }
    __syncwarp();
    if (has_dims) {
        float acc[H][4];
#pragma unroll
        for (int h = 0; h < H; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.0f;
        for (int s = 0; s < num_splits; s += W) {
            if (s > 0) {                                          // the next sixteen of every head, all at once
#pragma unroll
                for (int h = 0; h < H; ++h) {
                    const float* src = part_o + base[h] * head_dim + d0;
#pragma unroll
                    for (int u = 0; u < W; ++u)
                        if (s + u < num_splits)
                            v[h][u] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(s + u) * head_dim));
                }
            }
#pragma unroll
            for (int h = 0; h < H; ++h) {
                const float* wgts = wbuf + h * MAX_SPLITS;
#pragma unroll
                for (int u = 0; u < W; ++u) {
                    if (s + u >= num_splits) break;
                    const float wgt = wgts[s + u];
                    acc[h][0] = fmaf(v[h][u].x, wgt, acc[h][0]); acc[h][1] = fmaf(v[h][u].y, wgt, acc[h][1]);
                    acc[h][2] = fmaf(v[h][u].z, wgt, acc[h][2]); acc[h][3] = fmaf(v[h][u].w, wgt, acc[h][3]);
                }
            }
        }
#pragma unroll
        for (int h = 0; h < H; ++h) {
            const float inv = 1.0f / total[h];
            *reinterpret_cast<__nv_bfloat162*>(out[h] + d0) = __floats2bfloat162_rn(acc[h][0] * inv, acc[h][1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(out[h] + d0 + 2) = __floats2bfloat162_rn(acc[h][2] * inv, acc[h][3] * inv);
        }
    }
    __syncwarp();                                             // wbuf may be reused for the next heads
}


// Which tiles of 32 keys a split of a row at position `pos` takes.  The cut depends only on the
// row's own length and on `num_splits`.
struct SplitRange {
    int lo;                 // first visible key (> 0 only with a window)
    int tile_hi;            // past the last tile with keys
    int active;             // splits that have keys at all
    int my_lo, my_hi;       // this split's tiles
    // the split whose tiles hold the row's own, newest key
    __device__ bool owns_newest() const { return my_lo < my_hi && my_hi == tile_hi; }
};

__device__ __forceinline__ SplitRange split_range(int pos, int window, int num_splits, int split) {
    SplitRange r;
    const int ctx = pos + 1;
    r.lo = window > 0 ? max(0, ctx - window) : 0;
    const int tile_lo = r.lo / TILE;
    r.tile_hi = (ctx + TILE - 1) / TILE;
    // Tiles per split: all splits busy for long rows; for rows of up to 128 tiles no more than 32
    // splits (beyond that, starting and merging more one-warp blocks costs more than their shorter
    // loops save: 12.4 against 15.0 µs for one row of 4,096 keys).
    const int n_tiles = r.tile_hi - tile_lo;
    const int per_split = max(max((n_tiles + num_splits - 1) / num_splits, min(4, (n_tiles + 31) / 32)), 1);
    r.active = max((n_tiles + per_split - 1) / per_split, 1);
    r.my_lo = tile_lo + split * per_split;
    r.my_hi = min(r.tile_hi, r.my_lo + per_split);
    return r;
}

// Shared memory one item needs: STAGES stages of a key tile and a value tile.
template <int HD> constexpr int item_smem_bytes() { return STAGES * 2 * TILE * (HD * 2 + 16); }

// PDL: the item runs as a kernel of its own in a chain of programmatic dependent launches (it
// requests the tiles that earlier steps wrote before it waits for the kernel before it).
// `qbase`: the bfloat16 queries of the kv head's group, [group, HD] (global or shared memory).
// `new_k`, `new_v` (shared memory, HD bfloat16 each, or null): the key and value of the row's own
// token when the caller has not stored them through global memory before the item reads the
// tile that holds them; the item that owns that tile puts them in place.
struct NoPrologue {
    __device__ __forceinline__ void operator()() const {}
};

// `prologue()` runs once, by the whole warp, right after the wait for the kernel before and before
// the queries (and `new_k`, `new_v`) are read: a caller whose queries come out of that kernel
// unnormed prepares them there.
// SINGLE: the caller knows that the row's keys are not split (num_splits == 1 and counters given):
// the code of the merge is then left out, and its registers do not weigh on the key loop.
template <int HD, bool PDL, class Prologue = NoPrologue, bool SINGLE = false, bool LATE_WAIT = false>
__device__ __forceinline__ void decode_item(
        unsigned char* smem, const bf16* qbase, const bf16* new_k, const bf16* new_v,
        int split, int num_splits, int kvh, int row, int t, int pos,
        const int* __restrict__ table, const bf16* __restrict__ pages, int num_pages, int page_size,
        int num_heads, int num_kv_heads, int window, float scale_log2,
        float* __restrict__ part_o, float* __restrict__ part_ml, unsigned* __restrict__ counters,
        bf16* __restrict__ out, int* __restrict__ status, Prologue prologue = Prologue()) {
    constexpr int ROW_BYTES = HD * 2 + 16;          // padded: ldmatrix rows fall in distinct banks
    constexpr int CHUNKS = HD / 8;                  // 16-byte chunks per key
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;
    const int lane = threadIdx.x & 31;
    const int group = num_heads / num_kv_heads;
    const SplitRange range = split_range(pos, window, num_splits, split);
    const int ctx = pos + 1, lo = range.lo;
    const int active = range.active, my_lo = range.my_lo, my_hi = range.my_hi;

    const int g = lane >> 2, tq = lane & 3;
    const size_t kv_stride = (size_t)num_kv_heads * page_size * HD;   // keys -> values of a page
    // partial results of this block: heads kvh*group + r, r < group
    const size_t part_base = ((size_t)row * num_heads + (size_t)kvh * group) * num_splits + split;

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    if (PDL) pdl_launch();
    if (my_lo < my_hi) {
        auto issue = [&](int tile, int stage) {
            unsigned char* kdst = smem + (size_t)stage * 2 * TILE * ROW_BYTES;
            unsigned char* vdst = kdst + TILE * ROW_BYTES;
            // a tile is two runs of 16 keys; a run lies inside one page and is contiguous there
            // (16 * HD elements), so a lane's source addresses advance by 512 bytes per copy
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int key0 = tile * TILE + r * 16;
                int pg = -1;
                if (key0 < ctx && key0 + 16 > lo) {
                    pg = table[key0 / page_size];
                    if (pg < 0 || pg >= num_pages) {
                        if (lane == 0) atomicCAS(status, 0, 1);
                        pg = -1;
                    }
                }
                const bool valid = pg >= 0;
                const bf16* ksrc = pages;
                if (valid)
                    ksrc = pages + (((size_t)pg * 2 * num_kv_heads + kvh) * page_size +
                                    key0 % page_size) * HD + lane * 8;
                const bf16* vsrc = valid ? ksrc + kv_stride : pages;
#pragma unroll
                for (int i = 0; i < 16 * CHUNKS / 32; ++i) {
                    const int c = i * 32 + lane;                 // 16-byte chunk of the run
                    const int off = (r * 16 + c / CHUNKS) * ROW_BYTES + (c % CHUNKS) * 16;
                    cp_async16(kdst + off, ksrc + (valid ? i * 256 : 0), valid);
                    cp_async16(vdst + off, vsrc + (valid ? i * 256 : 0), valid);
                }
            }
        };

        // Keys of earlier steps do not depend on the kernel before this one; the new token's own
        // key and value (in the tile that holds `pos`) and the queries do.  So the first tiles
        // are requested before waiting for that kernel.
        const int new_tile = pos / TILE;
        int early = 0;
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (PDL && early == s && my_lo + s < my_hi && my_lo + s < new_tile) {
                issue(my_lo + s, s);
                cp_async_commit();
                ++early;
            }
        }
        if (PDL && !LATE_WAIT) pdl_wait();
        prologue();
        // queries of the group as the A operand: row r of the tile is head kvh*group + r
        unsigned qa[KSTEPS][4];
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int k0 = ks * 16 + tq * 2;
            // (with LATE_WAIT they lie in global memory and are read from L2: this block has not
            // itself waited for the kernel that wrote them; otherwise they may lie in shared memory)
            auto ld = [&](const bf16* p) {
                const unsigned* u = reinterpret_cast<const unsigned*>(p);
                if constexpr (LATE_WAIT) return __ldcg(u);
                else return *u;
            };
            qa[ks][0] = g < group ? ld(qbase + (size_t)g * HD + k0) : 0u;
            qa[ks][1] = g + 8 < group ? ld(qbase + (size_t)(g + 8) * HD + k0) : 0u;
            qa[ks][2] = g < group ? ld(qbase + (size_t)g * HD + k0 + 8) : 0u;
            qa[ks][3] = g + 8 < group ? ld(qbase + (size_t)(g + 8) * HD + k0 + 8) : 0u;
        }

#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < early) continue;
            if (my_lo + s < my_hi) issue(my_lo + s, s);
            cp_async_commit();
        }
        for (int tile = my_lo; tile < my_hi; ++tile) {
            const int stage = (tile - my_lo) % STAGES;
            if (tile + STAGES - 1 < my_hi) issue(tile + STAGES - 1, (tile - my_lo + STAGES - 1) % STAGES);
            cp_async_commit();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            unsigned char* ks = smem + (size_t)stage * 2 * TILE * ROW_BYTES;
            unsigned char* vs = ks + TILE * ROW_BYTES;
            if (new_k != nullptr && tile == new_tile) {
                // the row's own key and value have not gone through global memory: put them in place
                const int key = pos - tile * TILE;
                for (int c = lane; c < CHUNKS; c += 32) {
                    *reinterpret_cast<uint4*>(ks + key * ROW_BYTES + c * 16) =
                        *reinterpret_cast<const uint4*>(new_k + c * 8);
                    *reinterpret_cast<uint4*>(vs + key * ROW_BYTES + c * 16) =
                        *reinterpret_cast<const uint4*>(new_v + c * 8);
                }
                __syncwarp();
            }

            // scores of 16 heads x 32 keys
            float s_acc[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    unsigned b[4];
                    // lanes 0-15: keys of tile 2jp, dims kk*16 (+8); lanes 16-31: keys of tile 2jp+1
                    const int key = jp * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, ks + key * ROW_BYTES + dim * 2);
                    mma_bf16(s_acc[2 * jp], qa[kk], b[0], b[1]);
                    mma_bf16(s_acc[2 * jp + 1], qa[kk], b[2], b[3]);
                }
            }
            // mask, scale, online softmax (rows g and g + 8 of the head tile)
            const bool edge = tile * TILE < lo || tile * TILE + TILE > ctx;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s_acc[j][e] * scale_log2;
                    if (edge) {
                        const int key = tile * TILE + j * 8 + tq * 2 + (e & 1);
                        if (key < lo || key >= ctx) v = -INFINITY;
                    }
                    s_acc[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                alpha[r] = m_new == -INFINITY ? 1.0f : fast_exp2(m_run[r] - m_new);
                m_run[r] = m_new;
            }
            // a tile always holds at least one visible key, so the running maxima are finite
            float sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = fast_exp2(s_acc[j][e] - m_run[e >> 1]);
                    s_acc[j][e] = p;
                    sum[e >> 1] += p;
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + sum[r];
            if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
                for (int i = 0; i < NT_O; ++i) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                    o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
            // probabilities (bfloat16) times values
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                unsigned pa[4];
                pa[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
                pa[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
                pa[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
                pa[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < NT_O / 2; ++dp) {
                    unsigned b[4];
                    // lanes 0-7: keys kk*16.., dims dp*16; 8-15: keys +8; 16-31: dims dp*16 + 8
                    const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int dim = dp * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b, vs + key * ROW_BYTES + dim * 2);
                    mma_bf16(o[2 * dp], pa, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
                }
            }
            __syncwarp();                         // the stage may be refilled
        }
        cp_async_wait<0>();
    } else {
        if (PDL && !LATE_WAIT) pdl_wait();
        prologue();
    }
    // the sums of a row live in the four lanes of a quad
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (SINGLE || (num_splits == 1 && counters != nullptr)) {
        // One block has all keys of the row: what the merge would make of its single partial
        // result (weight 2^0, the sum's reciprocal) is computed here, without the round trip
        // through global memory, the fence and the ticket.
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int head = g + 8 * r;
            if (head >= group) continue;
            const float inv = 1.0f / l_run[r];
            bf16* dst = out + ((size_t)t * num_heads + (size_t)kvh * group + head) * HD;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + tq * 2) =
                    __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
        }
        return;
    }
    if constexpr (!SINGLE) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int head = g + 8 * r;
        if (head >= group) continue;
        const size_t idx = part_base + (size_t)head * num_splits;
        float* po = part_o + idx * HD;
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            *reinterpret_cast<float2*>(po + i * 8 + tq * 2) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
        }
        if (tq == 0) {
            part_ml[idx * 2] = m_run[r];
            part_ml[idx * 2 + 1] = l_run[r];
        }
    }
    if (counters == nullptr) return;                 // a separate launch merges
    // The block that finishes last for this (row, kv head) merges the splits of the group's heads.
    // The counter returns to zero, so the next launch finds it ready.
    __threadfence();
    __syncwarp();                                    // every lane's stores and fence come before the ticket
    unsigned ticket = 0;
    unsigned* counter = counters + (size_t)row * num_kv_heads + kvh;
    if (lane == 0) ticket = atomicAdd(counter, 1u);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != (unsigned)num_splits - 1) return;
    __threadfence();
    if (lane == 0) *counter = 0u;
    float* wbuf = reinterpret_cast<float*>(smem);
    int r = 0;
    for (; r + 2 <= group; r += 2) {                        // two heads at a time: their loads overlap
        const int h = kvh * group + r;
        const size_t base[2] = {((size_t)row * num_heads + h) * num_splits,
                                ((size_t)row * num_heads + h + 1) * num_splits};
        bf16* const dst[2] = {out + ((size_t)t * num_heads + h) * HD, out + ((size_t)t * num_heads + h + 1) * HD};
        merge_heads<2>(part_o, part_ml, base, active, HD, dst, lane, wbuf);
    }
    if (r < group) {
        const int h = kvh * group + r;
        const size_t base[1] = {((size_t)row * num_heads + h) * num_splits};
        bf16* const dst[1] = {out + ((size_t)t * num_heads + h) * HD};
        merge_heads<1>(part_o, part_ml, base, active, HD, dst, lane, wbuf);
    }
    }   // not SINGLE
}

}  // namespace attn_decode_core
