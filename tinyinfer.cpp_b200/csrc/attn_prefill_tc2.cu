// Paged flash attention for long prompt portions on the 5th-generation tensor cores (bfloat16,
// head_dim 128, pages of a multiple of 16 tokens, an even number of query heads per kv head).
//
// A block takes 128 consecutive query tokens of one request and TWO query heads that share a kv
// head, and walks the request's keys in tiles of 128 once for both: a key tile is fetched into
// shared memory once for two score products, a value tile once for two output products.  Why:
// a 128 x 128 x 16 product with both operands in shared memory reads 8 KB in its 64 cycles, all an
// SM's shared memory delivers, so what else goes through shared memory per product (the TMA's
// writes, P) is what bounds a tile; here that is 32 KB of writes per product pair instead of 64,
// and P never touches it.  Roles:
//   warp 0     TMA: the two query tiles once, then key and value tiles into two-stage rings (runs
//              of tokens that lie in one page, as in attn_prefill_tc.cu).
//   warp 1     tcgen05.mma, one issuing thread: S_g = Q_g K^T (128 x 128 x 128, operands K-major
//              from shared memory) into head g's score buffer and O_g += P_g V (P as the A operand
//              from tensor memory, where the softmax left it over the scores it was made from; V
//              from shared memory with its rows along N), a head's next scores right behind its
//              P V.
//   warps 4-7  softmax of head 0, warps 8-11 of head 1, one thread per query row: while one head's
//              threads wait on the exponential unit or write P, the other head's products and
//              softmax run.  A thread reads its row's 128 scores with tcgen05.ld into registers
//              (the control warps give theirs up: setmaxnreg), masks at the edges, keeps a
//              running maximum and sum in float32 and writes P = 2^(s - m) as bfloat16 pairs with
//              tcgen05.st into the first 64 columns of its score buffer (a row's P lies in the
//              row's own lane, behind the scores already read).  The output accumulator is
//              rescaled in tensor memory only when a row's maximum has grown by more than 2^8
//              since the last rescale (exact arithmetic: the reference maximum may lag behind).
// A query tile's own chain per key tile is longer than in attn_prefill_tc.cu (softmax, P V and
// the next scores follow one another, because P lies where the next scores go), so this kernel
// is for prompts with several tiles per SM, where two tiles in that time count; the caller chooses.
// Every wait on an mbarrier is bounded; on a timeout the block records status 2, frees its tensor
// memory and returns.
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int SUB = 128 * 64 * 2;                     // a [128 rows][64 elements] swizzled sub-tile
constexpr int SMEM_Q = 0, SMEM_K = 4 * SUB, SMEM_V = SMEM_K + 4 * SUB;      // two query tiles
constexpr int SMEM_BARS = SMEM_V + 4 * SUB;           // (P lives in tensor memory)
constexpr int SMEM_BYTES = SMEM_BARS + 256 + 1024;
constexpr int THREADS = 384;                          // three warpgroups: control, softmax of head 0, of head 1
constexpr int CONTROL_REGS = 40, SOFTMAX_REGS = 224;  // (4 * 40 + 8 * 224) * 32 <= 65,536
constexpr unsigned TMEM_COLS = 512;                   // scores of head 0, head 1; outputs of head 0, head 1
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of a block");
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;                  // in log2 units

enum { TI_ERR_TIMEOUT = 2 };

__device__ __forceinline__ float fast_exp2(float x) {           // 2^x, 2 ulp, 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// D (+)= A B with A from tensor memory (rows in lanes, two bfloat16 of K per 32-bit column).
__device__ __forceinline__ void umma_bf16_tmem_a(unsigned tmem_d, unsigned tmem_a, unsigned long long db,
                                                 unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive 32-bit columns of this thread's lane; completion is awaited by the caller.
__device__ __forceinline__ void tmem_store16(unsigned taddr, const unsigned (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

// tiles[i] = {request row, first flat token, number of query rows (<= 128)}
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
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
    unsigned long long* p_full = bars + 13;           // [2] P written over the scores in tensor memory
    unsigned long long* p_empty = bars + 15;          // [2] P V done: P may be rewritten, O is up to date
    unsigned* tmem_slot = (unsigned*)(bars + 17);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // pairs of heads run fastest in the grid, tiles are sorted by length: blocks start longest first
    const int h = 2 * blockIdx.x, tile_id = blockIdx.y;     // heads h and h + 1: the same kv head
    const int kvh = h / (num_heads / num_kv_heads);
    const int req = tiles[tile_id * 3], tok0 = tiles[tile_id * 3 + 1];
    const int nrows = tiles[tile_id * 3 + 2];
    const int pos_first = positions[tok0], pos_last = pos_first + nrows - 1;
    const int kv_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    // this block's run of the tile's key tiles (see attn_prefill_tc.cu: all of them without a
    // split; none if there are more blocks than key tiles)
    const int splits = gridDim.z, split = blockIdx.z;
    const int kt_first = kv_lo / BN, kt_all = pos_last / BN + 1 - kt_first;
    const int kt_lo = kt_first + (int)((long long)kt_all * split / splits);
    const int num_kt = kt_first + (int)((long long)kt_all * (split + 1) / splits) - kt_lo;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 4); mbar_init(&p_empty[i], 1);
        }
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

    // The softmax threads hold a row's 128 scores in registers; the warps that only issue copies
    // and products give their registers up for that (each warpgroup as a whole).
    bool ok = true;
    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(CONTROL_REGS));
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
            mbar_expect_tx(q_full, 4 * SUB);
            for (int g = 0; g < 2; ++g) {
                tma_load_2d(smem + SMEM_Q + g * 2 * SUB, &map_q, q_full, (h + g) * HD, tok0);
                tma_load_2d(smem + SMEM_Q + g * 2 * SUB + SUB, &map_q, q_full, (h + g) * HD + 64, tok0);
            }
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
        // One thread issues all products, per key tile in the order P V of head 0, next scores of
        // head 0, P V of head 1, next scores of head 1.  A head's next scores follow its P V at
        // once (the tensor core runs a thread's products in the order of issue, so they cannot
        // overtake the P V that still reads P from the same columns), and because head 0 is served
        // first, head 1 falls half a period behind and stays there: one head's softmax runs while
        // the other's products do.  (Issued as P V 0, P V 1, scores 0, scores 1 both heads'
        // softmaxes ended together and each waited for three products: 4,770 cycles a tile.)
        if (lane == 0 && num_kt > 0) {
            const unsigned idesc_s = umma_idesc(BM, BN);
            const unsigned idesc_o = umma_idesc(BM, HD, /*b_mn_major=*/true);
            auto issue_scores = [&](int g, int st) {
                const unsigned char* kbuf = smem + SMEM_K + st * 2 * SUB;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const int sub = ks >> 2, kk = ks & 3;
                    umma_bf16(tmem_base + g * BN,
                              umma_desc(smem + SMEM_Q + g * 2 * SUB + sub * SUB) + (unsigned long long)(kk * 2),
                              umma_desc(kbuf + sub * SUB) + (unsigned long long)(kk * 2), idesc_s, ks != 0);
                }
                umma_commit(&s_full[g]);
            };
            ok = mbar_wait(q_full, 0);
            if (ok) ok = mbar_wait(&k_full[0], 0);
            if (ok) {
                tc_fence_after();
                issue_scores(0, 0);
                issue_scores(1, 0);
                umma_commit(&k_empty[0]);
            }
            for (int j = 0; j < num_kt && ok; ++j) {
                const int st = j & 1, nst = (j + 1) & 1;
                ok = mbar_wait(&v_full[st], (j >> 1) & 1);
                const unsigned char* vbuf = smem + SMEM_V + st * 2 * SUB;
                for (int g = 0; g < 2 && ok; ++g) {
                    ok = mbar_wait(&p_full[g], j & 1);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < BN / 16; ++ks) {
                        // P: 16 keys = 8 columns of bfloat16 pairs in the score buffer.  V: rows (keys) of
                        // 128 bytes along N; 16 keys further = 2048 bytes; the second half of the head
                        // dimension is one sub-tile further (leading byte offset)
                        umma_bf16_tmem_a(tmem_o + g * HD, tmem_base + g * BN + ks * 8,
                                         umma_desc(vbuf + ks * 2048, SUB, 1024), idesc_o, j >= 1 || ks != 0);
                    }
                    umma_commit(&p_empty[g]);
                    if (g == 1) umma_commit(&v_empty[st]);
                    if (j + 1 < num_kt) {
                        if (g == 0) ok = mbar_wait(&k_full[nst], ((j + 1) >> 1) & 1);
                        if (!ok) break;
                        tc_fence_after();
                        issue_scores(g, nst);
                        if (g == 1) umma_commit(&k_empty[nst]);
                    }
                }
            }
        }
    } else if (warp >= 4) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(SOFTMAX_REGS));
        const int quarter = warp & 3;                                         // tensor-memory lanes
        const int group = (warp - 4) >> 2;                                    // the head of the pair
        const int row = quarter * 32 + lane;
        const int pos_row = row < nrows ? pos_first + row : -1;               // -1: sees nothing
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned tmem_s = tmem_base + lane_addr + group * BN;
        const unsigned tmem_mine = tmem_o + lane_addr + group * HD;
        float m_ref = -INFINITY, l_run = 0.0f;
        int use = 0;                                                          // tiles this group has done
        for (int j = 0; j < num_kt && ok; ++j, ++use) {
            const int key_lo = (kt_lo + j) * BN;
            const bool edge = key_lo + BN - 1 > pos_first || (window > 0 && key_lo <= pos_last - window);
            auto masked = [&](float x, int i) {
                const int key = key_lo + i;
                return (key > pos_row || (window > 0 && key <= pos_row - window)) ? -INFINITY : x;
            };
            ok = mbar_wait(&s_full[group], use & 1);
            if (!ok) break;
            tc_fence_after();
            // the row's 128 scores into registers (the buffer is then free for P)
            float v[BN];
#pragma unroll
            for (int c = 0; c < 4; ++c)
                tmem_load32(tmem_s + c * 32, *reinterpret_cast<float(*)[32]>(&v[c * 32]));
            if (edge) {
#pragma unroll
                for (int i = 0; i < BN; ++i) v[i] = masked(v[i], i);
            }
            float m4[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
            for (int i = 4; i < BN; i += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) m4[u] = fmaxf(m4[u], v[i + u]);
            }
            const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale_log2;   // the scale is positive
            const float m_new = fmaxf(m_ref, mx);
            const bool grow = m_new > m_ref + RESCALE_STEP;      // also true when m_ref is still -inf
            // the last P V of this head has read P and brought the output up to date
            if (use > 0) {
                ok = mbar_wait(&p_empty[group], (use - 1) & 1);
                if (!ok) break;
            }
            if (use > 0 && __any_sync(0xffffffffu, grow)) {
                // the output so far was built against m_ref: bring it to the new reference
                tc_fence_after();
                const float factor = grow ? exp2f(m_ref - m_new) : 1.0f;      // 0 if m_ref was -inf
                l_run *= factor;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_load32(tmem_mine + c * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= factor;
                    tmem_store32(tmem_mine + c * 32, o);
                }
            }
            if (grow) m_ref = m_new;
            const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
            // P = 2^(s * scale - m) as bfloat16 pairs, 32 keys = 16 columns at a time, and its sum
            float s2[2] = {0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                unsigned packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = fast_exp2(fmaf(v[c * 32 + i], scale_log2, neg_m));
                    const float p1 = fast_exp2(fmaf(v[c * 32 + i + 1], scale_log2, neg_m));
                    s2[(i >> 1) & 1] += p0 + p1;
                    __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                    packed[i >> 1] = *reinterpret_cast<unsigned*>(&pk);
                }
                tmem_store16(tmem_s + c * 16, packed);
            }
            const float sum = s2[0] + s2[1];
            l_run += sum;
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[group]);
        }
        if (ok && use > 0) ok = mbar_wait(&p_empty[group], (use - 1) & 1);
        if (ok && splits > 1) {
            // this run's share: the output as it stands against m_ref, with m_ref and the sum
            tc_fence_after();
            const size_t slot = ((size_t)tile_id * num_heads + h + group) * splits + split;
            float* prow = part_o + (slot * BM + row) * HD;
            if (row < nrows) {
                part_ml[(slot * BM + row) * 2] = m_ref;
                part_ml[(slot * BM + row) * 2 + 1] = l_run;
            }
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float v[32];
                if (use > 0) {
                    tmem_load32(tmem_mine + c * 32, v);
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
            bf16* orow = out + ((size_t)(tok0 + row) * num_heads + h + group) * HD;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float v[32];
                tmem_load32(tmem_mine + c * 32, v);
                if (row >= nrows) continue;
                unsigned packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    __nv_bfloat162 pk = __floats2bfloat162_rn(v[i] * inv, v[i + 1] * inv);
                    packed[i >> 1] = *reinterpret_cast<unsigned*>(&pk);
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) =
                        make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
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

}  // namespace

extern "C" int ti_attn_prefill_tc2_supported(int head_dim, int page_size, int num_heads, int num_kv_heads) {
    return head_dim == HD && page_size >= 16 && page_size % 16 == 0 && num_kv_heads > 0 &&
           num_heads % num_kv_heads == 0 && (num_heads / num_kv_heads) % 2 == 0;
}

// As ti_attn_prefill_tc (attn_prefill_tc.cu), for an even number of query heads per kv head; the
// runs of a split are added by ti_attn_prefill_tc_merge as well (the same scratch layout).
extern "C" int ti_attn_prefill_tc2(const void* q, int num_tokens, const int* tiles, int num_tiles,
                                   const int* positions, const int* block_table, int bt_stride,
                                   const void* pages, int num_pages, int page_size, int num_heads,
                                   int num_kv_heads, int head_dim, int window, float scale, void* out,
                                   int splits, float* part_o, float* part_ml,
                                   int* status, int hold_dependents, void* stream) {
    if (num_tiles == 0) return 0;
    TI_REQUIRE(splits >= 1 && splits <= 8 &&
               (splits == 1 || (part_o != nullptr && part_ml != nullptr && (uintptr_t)part_o % 16 == 0)),
               "attn_prefill_tc2: %d runs per tile (1..8) need their 16-byte aligned scratch", splits);
    TI_REQUIRE(ti_attn_prefill_tc2_supported(head_dim, page_size, num_heads, num_kv_heads),
               "attn_prefill_tc2: head_dim %d (128), page size %d (multiple of 16) or heads %d/%d (an even "
               "number per kv head) are not supported", head_dim, page_size, num_heads, num_kv_heads);
    TI_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)pages % 16 == 0 && (uintptr_t)out % 16 == 0,
               "attn_prefill_tc2: tensors must be 16-byte aligned");
    TI_REQUIRE(num_tiles <= 65535, "attn_prefill_tc2: %d tiles exceed the grid limit", num_tiles);
    const long long pool_rows = (long long)num_pages * 2 * num_kv_heads * page_size;
    TI_REQUIRE(pool_rows < (1LL << 31) - 1, "attn_prefill_tc2: the page pool has too many token slots");
    CUtensorMap map_q, map_kv;
    if (int rc = make_map_bf16(&map_q, q, num_tokens, num_heads * HD, (long long)num_heads * HD, BM,
                               "attn_prefill_tc2"))
        return rc;
    int run = 128;
    while (page_size % run) run /= 2;
    if (int rc = make_map_bf16(&map_kv, pages, pool_rows, HD, HD, run, "attn_prefill_tc2")) return rc;
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc2_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return ti_fail("attn_prefill_tc2: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid(num_heads / 2, num_tiles, splits);
    ti_launch_pdl(attn_prefill_tc2_kernel, grid, dim3(THREADS), SMEM_BYTES, (cudaStream_t)stream, map_q, map_kv,
                  tiles, positions, block_table, bt_stride, num_pages, page_size, num_heads, num_kv_heads,
                  window, run, scale * LOG2E, (bf16*)out, part_o, part_ml, status, hold_dependents);
    return ti_check_launch("attn_prefill_tc2");
}
