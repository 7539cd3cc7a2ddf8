// Paged flash attention for prompt portions on the 5th-generation tensor cores (bfloat16,
// head_dim 128, pages of a multiple of 16 tokens).
//
// A block takes 128 consecutive query tokens of one request and one query head and walks the
// request's keys in tiles of 128, from the first key any of its rows may see to its last row's own
// position (keys of earlier steps and of this portion alike).  Roles:
//   warp 0     TMA: the query tile once, then key and value tiles into two-stage rings.  A tile is
//              128 / run runs of tokens that lie in one page, each run one box of the page pool
//              seen as a 2-D tensor (rows = token slots, 128-byte swizzle); runs nobody may see are
//              fetched from outside the tensor, which TMA fills with zeros.
//   warp 1     tcgen05.mma: S = Q K^T (128 x 128 x 128, both operands K-major) into one of two
//              score accumulators in tensor memory, one tile ahead of the softmax; then O += P V
//              (P K-major from shared memory, V with its rows along N) into the output accumulator.
//   warps 2-5  softmax, one thread per query row: read the scores with tcgen05.ld, mask at the
//              edges, keep a running maximum and sum in float32, write P = 2^(s - m) as bfloat16 into
//              shared memory in the swizzled layout the MMA reads.  The output accumulator is
//              rescaled in tensor memory only when a row's maximum has grown by more than 2^8
//              since the last rescale (exact arithmetic: the reference maximum may lag behind).
// When a step has fewer (tile, head) pairs than the GPU has SMs (a portion of a long prompt: few
// tiles with long rows of keys), the keys of every tile are cut into `gridDim.z` equal runs of
// key tiles, one block each: a block then leaves its output unnormalised in a float32 workspace
// with its rows' reference maxima and sums, and a second kernel adds the runs.
// Every wait on an mbarrier is bounded; on a timeout the block records status 2, frees its tensor
// memory and returns.
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int SUB = 128 * 64 * 2;                     // a [128 rows][64 elements] swizzled sub-tile
constexpr int SMEM_Q = 0, SMEM_K = 2 * SUB, SMEM_V = SMEM_K + 4 * SUB, SMEM_P = SMEM_V + 4 * SUB;
constexpr int SMEM_BARS = SMEM_P + 2 * SUB;
constexpr int SMEM_BYTES = SMEM_BARS + 256 + 1024;
constexpr int THREADS = 192;
constexpr unsigned TMEM_COLS = 512;                   // scores 0..127 and 128..255, output 256..383
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;                  // in log2 units

enum { TI_ERR_TIMEOUT = 2 };

__device__ __forceinline__ float fast_exp2(float x) {           // 2^x, 2 ulp, 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// tiles[i] = {request row, first flat token, number of query rows (<= 128)}
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                       const int* __restrict__ tiles, const int* __restrict__ positions,
                       const int* __restrict__ block_table, int bt_stride, int num_pages, int page_size,
                       int num_heads, int num_kv_heads, int window, int run, float scale_log2,
                       bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                       int* __restrict__ status, int hold_dependents) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = (unsigned long long*)(smem + SMEM_BARS);
    unsigned long long* q_full = bars;
    unsigned long long* k_full = bars + 1;            // [2]
    unsigned long long* k_empty = bars + 3;           // [2]
    unsigned long long* v_full = bars + 5;            // [2]
    unsigned long long* v_empty = bars + 7;           // [2]
    unsigned long long* s_full = bars + 9;            // [2] scores ready in TMEM
    unsigned long long* s_empty = bars + 11;          // [2] scores read by the softmax
    unsigned long long* p_full = bars + 13;           // P written to shared memory
    unsigned long long* p_empty = bars + 14;          // P V done: P may be rewritten, O is up to date
    unsigned* tmem_slot = (unsigned*)(bars + 15);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heads run fastest in the grid, tiles are sorted by length: blocks start longest first
    const int h = blockIdx.x, tile_id = blockIdx.y;
    const int kvh = h / (num_heads / num_kv_heads);
    const int req = tiles[tile_id * 3], tok0 = tiles[tile_id * 3 + 1];
    const int nrows = tiles[tile_id * 3 + 2];
    const int pos_first = positions[tok0], pos_last = pos_first + nrows - 1;
    const int kv_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    // this block's run of the tile's key tiles (all of them without a split; none if there are
    // more blocks than key tiles)
    const int splits = gridDim.z, split = blockIdx.z;
    const int kt_first = kv_lo / BN, kt_all = pos_last / BN + 1 - kt_first;
    const int kt_lo = kt_first + (int)((long long)kt_all * split / splits);
    const int num_kt = kt_first + (int)((long long)kt_all * (split + 1) / splits) - kt_lo;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
        }
        mbar_init(p_full, 4);
        mbar_init(p_empty, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    // `hold_dependents`: the next kernel is released only when this block's wait has returned, so
    // that it may run beside this one on what this one waited for, without a wait of its own
    if (!hold_dependents) pdl_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();        // queries, keys and values come from the kernel before
    if (hold_dependents) pdl_launch();
    const unsigned tmem_o = tmem_base + 256;

    bool ok = true;
    if (warp == 0) {
        // A tile is cut into runs of `run` keys that lie in one page (16 to 128, the largest power of
        // two that divides the page size: the fewer and larger the boxes, the less the TMA unit's
        // issue rate of about one box per 64 cycles paces the tile).  Each of the first 128 / run
        // lanes owns one run: it looks up its page and issues its four boxes (two halves of the
        // head dimension, keys and values); lane 0 also does the waiting.
        const int* table = block_table + (size_t)req * bt_stride;
        const int oob_row = num_pages * 2 * num_kv_heads * page_size;          // outside the tensor: zeros
        const int to_v = num_kv_heads * page_size;                             // keys -> values of a page
        if (lane == 0 && num_kt > 0) {
            mbar_expect_tx(q_full, 2 * SUB);
            tma_load_2d(smem + SMEM_Q, &map_q, q_full, h * HD, tok0);
            tma_load_2d(smem + SMEM_Q + SUB, &map_q, q_full, h * HD + 64, tok0);
        }
        // the row of the pool's 2-D view where this lane's run of 16 keys of tile j begins
        auto lookup = [&](int j) {
            int krow = oob_row;
            if (lane < BN / run) {
                const int key0 = (kt_lo + j) * BN + lane * run;
                if (key0 <= pos_last && key0 + run > kv_lo) {
                    const int pg = table[key0 / page_size];
                    if (pg >= 0 && pg < num_pages)
                        krow = (pg * 2 * num_kv_heads + kvh) * page_size + key0 % page_size;
                    else
                        atomicCAS(status, 0, 1);
                }
            }
            return krow;
        };
        int krow_next = num_kt > 0 ? lookup(0) : oob_row;
        for (int j = 0; j < num_kt && ok; ++j) {
            const int st = j & 1;
            const int krow = krow_next;
            // the next tile's block-table entries are on their way while this tile is issued
            if (j + 1 < num_kt) krow_next = lookup(j + 1);
            if (lane == 0) {
                ok = mbar_wait(&k_empty[st], ((j >> 1) & 1) ^ 1);
                if (ok) mbar_expect_tx(&k_full[st], 2 * SUB);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < BN / run) {
                unsigned char* kdst = smem + SMEM_K + st * 2 * SUB + lane * run * 128;
                tma_load_2d(kdst, &map_kv, &k_full[st], 0, krow);
                tma_load_2d(kdst + SUB, &map_kv, &k_full[st], 64, krow);
            }
            if (lane == 0) {
                ok = mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1);
                if (ok) mbar_expect_tx(&v_full[st], 2 * SUB);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < BN / run) {
                const int vrow = krow == oob_row ? oob_row : krow + to_v;
                unsigned char* vdst = smem + SMEM_V + st * 2 * SUB + lane * run * 128;
                tma_load_2d(vdst, &map_kv, &v_full[st], 0, vrow);
                tma_load_2d(vdst + SUB, &map_kv, &v_full[st], 64, vrow);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && num_kt > 0) {
            const unsigned idesc_s = umma_idesc(BM, BN);
            const unsigned idesc_o = umma_idesc(BM, HD, /*b_mn_major=*/true);
            auto issue_scores = [&](int buf, int st) {
                const unsigned char* kbuf = smem + SMEM_K + st * 2 * SUB;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const int sub = ks >> 2, kk = ks & 3;
                    umma_bf16(tmem_base + buf * BN,
                              umma_desc(smem + SMEM_Q + sub * SUB) + (unsigned long long)(kk * 2),
                              umma_desc(kbuf + sub * SUB) + (unsigned long long)(kk * 2), idesc_s, ks != 0);
                }
            };
            ok = mbar_wait(q_full, 0);
            if (ok) ok = mbar_wait(&k_full[0], 0);
            if (ok) {
                tc_fence_after();
                issue_scores(0, 0);
                umma_commit(&k_empty[0]);
                umma_commit(&s_full[0]);
            }
            for (int j = 0; j < num_kt && ok; ++j) {
                if (j + 1 < num_kt) {                 // the next tile's scores, one tile ahead
                    const int n = j + 1, b = n & 1;
                    ok = mbar_wait(&k_full[b], (n >> 1) & 1);
                    if (ok) ok = mbar_wait(&s_empty[b], ((n >> 1) & 1) ^ 1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_scores(b, b);
                    umma_commit(&k_empty[b]);
                    umma_commit(&s_full[b]);
                }
                const int st = j & 1;
                ok = mbar_wait(p_full, j & 1);
                if (ok) ok = mbar_wait(&v_full[st], (j >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const unsigned char* vbuf = smem + SMEM_V + st * 2 * SUB;
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    const int sub = ks >> 2, kk = ks & 3;
                    // V: rows (keys) of 128 bytes along N; 16 keys further = 2048 bytes; the second
                    // half of the head dimension is one sub-tile further (leading byte offset)
                    umma_bf16(tmem_o, umma_desc(smem + SMEM_P + sub * SUB) + (unsigned long long)(kk * 2),
                              umma_desc(vbuf + ks * 2048, SUB, 1024), idesc_o, (j | ks) != 0);
                }
                umma_commit(&v_empty[st]);
                umma_commit(p_empty);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int pos_row = row < nrows ? pos_first + row : -1;               // -1: sees nothing
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        float m_ref = -INFINITY, l_run = 0.0f;
        for (int j = 0; j < num_kt && ok; ++j) {
            const int b = j & 1;
            const int key_lo = (kt_lo + j) * BN;
            const bool edge = key_lo + BN - 1 > pos_first || (window > 0 && key_lo <= pos_last - window);
            ok = mbar_wait(&s_full[b], (j >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            // the row's 128 scores into registers; the score buffer is free again at once
            float v[BN];
#pragma unroll
            for (int c = 0; c < 4; ++c)
                tmem_load32(tmem_base + lane_addr + b * BN + c * 32, *reinterpret_cast<float(*)[32]>(&v[c * 32]));
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[b]);
            if (edge) {
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    const int key = key_lo + i;
                    if (key > pos_row || (window > 0 && key <= pos_row - window)) v[i] = -INFINITY;
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < BN; ++i) mx = fmaxf(mx, v[i]);
            mx *= scale_log2;                                    // the scale is positive
            const float m_new = fmaxf(m_ref, mx);
            const bool grow = m_new > m_ref + RESCALE_STEP;      // also true when m_ref is still -inf
            bool waited = false;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // the output so far was built against m_ref: bring it to the new reference
                ok = mbar_wait(p_empty, (j - 1) & 1);
                if (!ok) break;
                waited = true;
                tc_fence_after();
                const float factor = grow ? exp2f(m_ref - m_new) : 1.0f;      // 0 if m_ref was -inf
                l_run *= factor;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_load32(tmem_o + lane_addr + c * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= factor;
                    tmem_store32(tmem_o + lane_addr + c * 32, o);
                }
            }
            if (grow) m_ref = m_new;
            const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
            // P = 2^(s * scale - m) and its sum; two values per register as bfloat16
            float sum = 0.0f;
            unsigned packed[BN / 2];
#pragma unroll
            for (int i = 0; i < BN; i += 2) {
                const float p0 = fast_exp2(fmaf(v[i], scale_log2, neg_m));
                const float p1 = fast_exp2(fmaf(v[i + 1], scale_log2, neg_m));
                sum += p0 + p1;
                __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                packed[i >> 1] = *reinterpret_cast<unsigned*>(&pk);
            }
            l_run += sum;
            if (j > 0 && !waited) {
                ok = mbar_wait(p_empty, (j - 1) & 1);            // the last P V has read the tile
                if (!ok) break;
            }
            // keys 8q .. 8q+7 of this row: sub-tile q / 8, 16-byte chunk q % 8 (swizzled by the row)
            unsigned char* prow = smem + SMEM_P + row * 128;
#pragma unroll
            for (int q8 = 0; q8 < BN / 8; ++q8) {
                const int chunk = (q8 & 7) ^ (row & 7);
                *reinterpret_cast<uint4*>(prow + (q8 >> 3) * SUB + chunk * 16) =
                    make_uint4(packed[q8 * 4], packed[q8 * 4 + 1], packed[q8 * 4 + 2], packed[q8 * 4 + 3]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (ok && num_kt > 0) ok = mbar_wait(p_empty, (num_kt - 1) & 1);
        if (ok && splits > 1) {
            // this run's share: the output as it stands against m_ref, with m_ref and the sum
            tc_fence_after();
            const size_t slot = ((size_t)tile_id * num_heads + h) * splits + split;
            float* prow = part_o + (slot * BM + row) * HD;
            if (row < nrows) {
                part_ml[(slot * BM + row) * 2] = m_ref;
                part_ml[(slot * BM + row) * 2 + 1] = l_run;
            }
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float v[32];
                if (num_kt > 0) {
                    tmem_load32(tmem_o + lane_addr + c * 32, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                }
                if (row >= nrows) continue;
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(prow + c * 32 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            }
        } else if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l_run;
            bf16* orow = out + ((size_t)(tok0 + row) * num_heads + h) * HD;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float v[32];
                tmem_load32(tmem_o + lane_addr + c * 32, v);
                if (row >= nrows) continue;
                unsigned packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    __nv_bfloat162 pk = __floats2bfloat162_rn(v[i] * inv, v[i + 1] * inv);
                    packed[i >> 1] = *reinterpret_cast<unsigned*>(&pk);
                }
                // a thread's stores are a row each: whole 32-byte sectors (the row is 256 bytes, aligned)
#pragma unroll
                for (int q8 = 0; q8 < 2; ++q8)
                    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(orow + c * 32 + q8 * 16),
                                 "r"(packed[q8 * 8]), "r"(packed[q8 * 8 + 1]), "r"(packed[q8 * 8 + 2]),
                                 "r"(packed[q8 * 8 + 3]), "r"(packed[q8 * 8 + 4]), "r"(packed[q8 * 8 + 5]),
                                 "r"(packed[q8 * 8 + 6]), "r"(packed[q8 * 8 + 7]) : "memory");
            }
        }
    }
    if (!ok) atomicCAS(status, 0, TI_ERR_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Adds the runs of a split tile: out = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s, M the largest
// m_s.  A warp per query row, a lane per four elements of the head.
constexpr int MERGE_ROWS = 16;
__global__ void __launch_bounds__(MERGE_ROWS * 32)
attn_prefill_merge_kernel(const int* __restrict__ tiles, const float* part_o,
                          const float* part_ml, int num_heads, int splits,
                          bf16* __restrict__ out) {
    pdl_launch();
    const int h = blockIdx.x, tile_id = blockIdx.y;
    const int row = blockIdx.z * MERGE_ROWS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int tok0 = tiles[tile_id * 3 + 1], nrows = tiles[tile_id * 3 + 2];
    pdl_wait();
    if (row >= nrows) return;
    const size_t first = ((size_t)tile_id * num_heads + h) * splits;
    float big = -INFINITY;
    for (int s = 0; s < splits; ++s) big = fmaxf(big, part_ml[((first + s) * BM + row) * 2]);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float sum = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float m = part_ml[((first + s) * BM + row) * 2];
        if (m == -INFINITY) continue;                     // this run saw no key of the row
        const float w = exp2f(m - big);
        sum += w * part_ml[((first + s) * BM + row) * 2 + 1];
        const float4 o = *reinterpret_cast<const float4*>(part_o + ((first + s) * BM + row) * HD + lane * 4);
        acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
    }
    const float inv = 1.0f / sum;
    bf16* dst = out + ((size_t)(tok0 + row) * num_heads + h) * HD + lane * 4;
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
}

}  // namespace

extern "C" int ti_attn_prefill_tc_tile_rows() { return BM; }

extern "C" int ti_attn_prefill_tc_supported(int head_dim, int page_size, int num_heads, int num_kv_heads) {
    return head_dim == HD && page_size >= 16 && page_size % 16 == 0 && num_kv_heads > 0 &&
           num_heads % num_kv_heads == 0;
}

// In how many runs the keys of every tile are cut: so many that the blocks fill the SMs once, and
// none when there are as many (tile, head) pairs as SMs already.
constexpr int MAX_SPLITS = 8;
extern "C" int ti_attn_prefill_tc_splits(int num_tiles, int num_heads) {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long pairs = (long long)num_tiles * num_heads;
    if (pairs <= 0 || sms <= 0) return 1;
    const long long s = sms / pairs;
    return (int)(s < 1 ? 1 : s > MAX_SPLITS ? MAX_SPLITS : s);
}

// q, out: [tokens, num_heads * 128] bfloat16, contiguous.  pages: the cache slot's pool
// [num_pages, 2, kv_heads, page_size, 128] bfloat16, contiguous.  tiles: int32 [num_tiles, 3] =
// {request row, first flat token, query rows (<= 128)}.  splits: 1, or ti_attn_prefill_tc_splits
// with part_o [num_tiles, num_heads, splits, 128, 128] and part_ml [num_tiles, num_heads, splits,
// 128, 2] float32 as scratch; the runs are then added by a second launch, which comes after
// `between` (may be null: a launch the caller wants between the two, on the same stream; with
// `hold_dependents` a kernel that runs beside this one and waits for it at its end).
extern "C" int ti_attn_prefill_tc(const void* q, int num_tokens, const int* tiles, int num_tiles,
                                  const int* positions, const int* block_table, int bt_stride,
                                  const void* pages, int num_pages, int page_size, int num_heads,
                                  int num_kv_heads, int head_dim, int window, float scale, void* out,
                                  int splits, float* part_o, float* part_ml,
                                  int* status, int hold_dependents, void* stream) {
    if (num_tiles == 0) return 0;
    TI_REQUIRE(ti_attn_prefill_tc_supported(head_dim, page_size, num_heads, num_kv_heads),
               "attn_prefill_tc: head_dim %d (128), page size %d (multiple of 16) or heads %d/%d "
               "are not supported", head_dim, page_size, num_heads, num_kv_heads);
    TI_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)pages % 16 == 0 && (uintptr_t)out % 32 == 0,
               "attn_prefill_tc: tensors must be 16-byte aligned, the output 32-byte");
    TI_REQUIRE(num_tiles <= 65535, "attn_prefill_tc: %d tiles exceed the grid limit", num_tiles);
    TI_REQUIRE(splits >= 1 && splits <= MAX_SPLITS &&
               (splits == 1 || (part_o != nullptr && part_ml != nullptr && (uintptr_t)part_o % 16 == 0)),
               "attn_prefill_tc: %d runs per tile (1..%d) need their 16-byte aligned scratch", splits, MAX_SPLITS);
    const long long pool_rows = (long long)num_pages * 2 * num_kv_heads * page_size;
    TI_REQUIRE(pool_rows < (1LL << 31) - 1, "attn_prefill_tc: the page pool has too many token slots");
    CUtensorMap map_q, map_kv;
    if (int rc = make_map_bf16(&map_q, q, num_tokens, num_heads * HD, (long long)num_heads * HD, BM,
                               "attn_prefill_tc"))
        return rc;
    int run = 128;
    while (page_size % run) run /= 2;
    if (int rc = make_map_bf16(&map_kv, pages, pool_rows, HD, HD, run, "attn_prefill_tc")) return rc;
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return ti_fail("attn_prefill_tc: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid(num_heads, num_tiles, splits);
    ti_launch_pdl(attn_prefill_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, (cudaStream_t)stream, map_q, map_kv,
                  tiles, positions, block_table, bt_stride, num_pages, page_size, num_heads, num_kv_heads,
                  window, run, scale * LOG2E, (bf16*)out, part_o, part_ml, status, hold_dependents);
    return ti_check_launch("attn_prefill_tc");
}

// The second launch of a split ti_attn_prefill_tc (same tiles, scratch and output).
extern "C" int ti_attn_prefill_tc_merge(const int* tiles, int num_tiles, int num_heads, int splits,
                                        const float* part_o, const float* part_ml, void* out, void* stream) {
    if (num_tiles == 0 || splits <= 1) return 0;
    dim3 grid(num_heads, num_tiles, BM / MERGE_ROWS);
    ti_launch_pdl(attn_prefill_merge_kernel, grid, dim3(MERGE_ROWS * 32), 0, (cudaStream_t)stream, tiles, part_o,
                  part_ml, num_heads, splits, (bf16*)out);
    return ti_check_launch("attn_prefill_tc_merge");
}
