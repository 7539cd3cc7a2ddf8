// The prefill product on pairs of SMs: C[M,N] (+)= A[M,K] * W[N,K]^T with tcgen05 cta_group::2.
//
// Two blocks of a cluster (two SMs of one TPC) compute one 256 x 256 tile of C together.  Each block
// fetches its own 128 rows of A and its own 128 rows of W per k-block (32 KB, half of what a block
// of the one-SM kernel fetches for half the tile), so the tile does twice as many flop per byte that
// crosses from L2 to an SM; the one-SM kernel is bound by that path.  The leader (rank 0) issues
// tcgen05.mma.cta_group::2 (256 x 256 x 16): the tensor cores of both SMs read both blocks' shared
// memory at the same offsets, and each SM accumulates its 128 rows x 256 columns in its own tensor
// memory.  Both blocks run the same epilogue on their own rows (store, accumulate, SwiGLU, or the
// QKV epilogue of qkv_epilogue.cuh: head norm, rotation and the store into the paged cache).
//
// Barriers: a stage's "full" barrier lives in the leader and counts the bytes of both blocks' TMA
// loads (loads of the peer name the leader's barrier); "empty" and "accumulator full" are signalled
// in both blocks at once by tcgen05.commit with a cluster multicast of the barrier arrival (no data
// is multicast); "accumulator empty" collects arrivals of both blocks' epilogue warps at the
// leader.  Every wait is bounded; on a timeout the block records status 2 and both blocks leave
// through the cluster barrier at the end, freeing their tensor memory.
#include "qkv_epilogue.cuh"

namespace {

using namespace sm100;

constexpr int BM = 256, BK = 64, UMMA_K = 16;
constexpr int THREADS = 320;       // TMA warp, MMA warp, eight epilogue warps
constexpr int STAGE_A = 128 * BK * 2;                                  // per block

// (Tried for narrow outputs and dropped: 256 x 128 tiles (twice the tiles, no faster than the one-SM
// kernel) and cutting K over pairs with an ordered accumulation into C (slower: 6.4 ms against 5.6 ms
// for the 2,048-token step).)
template <int BN> struct Pair {
    static constexpr int STAGES = BN == 256 ? 6 : 8;
    static constexpr int STAGE_B = (BN / 2) * BK * 2;                  // per block
    static constexpr int SMEM = STAGES * (STAGE_A + STAGE_B) + 1024 + 256;
    static constexpr unsigned TMEM_COLS = 2 * BN;
};

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SWIGLU = 2, MODE_QKV = 3 };
enum { TI_ERR_TIMEOUT = 2 };

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of the same variable in the block of rank `rank`.
__device__ __forceinline__ unsigned map_to_rank(const void* p, unsigned rank) {
    unsigned out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// A TMA tile load of a block of a pair: the data goes to this block's shared memory, the bytes are
// counted by the barrier at `bar_cluster_addr` (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, unsigned bar_cluster_addr,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long da, unsigned long long db,
                                               unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// One arrival, on the barrier at this offset in both blocks of the pair, when the MMAs issued so far
// have completed.
__device__ __forceinline__ void umma_commit_pair(void* bar) {
    const unsigned short mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
        ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tcgen05_2sm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const __grid_constant__ qkv::Epilogue qkv_e, float* __restrict__ c,
                        bf16* __restrict__ out_act, int m, int n, int k, int ldc, int ld_act, int mode,
                        int* __restrict__ status) {
    constexpr int STAGES = Pair<BN>::STAGES, STAGE_B = Pair<BN>::STAGE_B;
    constexpr unsigned TMEM_COLS = Pair<BN>::TMEM_COLS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_a = smem;
    unsigned char* stage_b = smem + STAGES * STAGE_A;
    unsigned long long* bars = (unsigned long long*)(smem + STAGES * (STAGE_A + STAGE_B));
    unsigned long long* full = bars;                     // [STAGES] used in the leader only
    unsigned long long* empty = bars + STAGES;           // [STAGES] in both blocks
    unsigned long long* acc_full = bars + 2 * STAGES;    // [2] in both blocks
    unsigned long long* acc_empty = bars + 2 * STAGES + 2;   // [2] used in the leader only
    unsigned* tmem_slot = (unsigned*)(bars + 2 * STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (k + BK - 1) / BK;
    const int tiles_m = (m + BM - 1) / BM, tiles_n = (n + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 16); }
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    __shared__ float qkv_norm_w[2 * qkv::HEAD_DIM];
    if (mode == MODE_QKV) qkv::load_norm_weights(qkv_e, qkv_norm_w, threadIdx.x, THREADS);
    pdl_launch();
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                      // both blocks' barriers exist before any use
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    bool ok = true;
    if (warp == 0) {
        if (lane == 0) {
            // The weights do not depend on the kernel before this one: the first ring-full of W
            // tiles is requested before waiting for it; its results (A) follow after the wait.
            int primed = 0;
            for (int tile = pair; tile < num_tiles && primed < STAGES; tile += num_pairs) {
                const int n0 = (tile / tiles_m) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < num_kb && primed < STAGES; ++kb, ++primed) {
                    if (leader) mbar_expect_tx(&full[primed], 2 * (STAGE_A + STAGE_B));   // both blocks' bytes
                    tma_load_2d_pair(stage_b + primed * STAGE_B, &map_w, map_to_rank(&full[primed], 0), kb * BK, n0);
                }
            }
            pdl_wait();
            int it = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int m0 = (tile % tiles_m) * BM + (int)rank * 128;
                const int n0 = (tile / tiles_m) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const unsigned bar = map_to_rank(&full[s], 0);
                    if (it >= primed) {
                        ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1);
                        if (!ok) break;
                        if (leader) mbar_expect_tx(&full[s], 2 * (STAGE_A + STAGE_B));   // both blocks' bytes
                        tma_load_2d_pair(stage_b + s * STAGE_B, &map_w, bar, kb * BK, n0);
                    }
                    tma_load_2d_pair(stage_a + s * STAGE_A, &map_a, bar, kb * BK, m0);
                }
            }
        }
    } else if (warp == 1) {
        if (leader && lane == 0) {
            const unsigned idesc = umma_idesc(BM, BN);
            int it = 0, local = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
                const int buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1);
                if (!ok) break;
                tc_fence_after();
                const unsigned tmem_acc = tmem_base + (unsigned)(buf * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const unsigned long long da = umma_desc(stage_a + s * STAGE_A);
                    const unsigned long long db = umma_desc(stage_b + s * STAGE_B);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)
                        umma_bf16_pair(tmem_acc, da + (unsigned long long)(kk * UMMA_K * 2 >> 4),
                                       db + (unsigned long long)(kk * UMMA_K * 2 >> 4), idesc, (kb | kk) != 0);
                    umma_commit_pair(&empty[s]);
                }
                umma_commit_pair(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;                 // the TMEM lanes this warp may read
        const int col_half = (warp - 2) >> 2;         // two warps share a quarter: half of the columns each
        pdl_wait();                                   // C and what the QKV epilogue reads belong to the chain
        int local = 0;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
            const int buf = local & 1;
            const int m0 = (tile % tiles_m) * BM + (int)rank * 128, n0 = (tile / tiles_m) * BN;
            const int row = m0 + quarter * 32 + lane;
            // where the tile's two heads go, and this warp's half of the token's sines and cosines:
            // requested while the products still run
            bf16 *qkv_dst0 = nullptr, *qkv_dst1 = nullptr;
            qkv::Angles angles;
            if (mode == MODE_QKV) {
                const int item0 = n0 / qkv::HEAD_DIM, items = qkv_e.num_heads + 2 * qkv_e.num_kv_heads;
                qkv_dst0 = qkv::destination(qkv_e, row, item0, row < m && item0 < items, status);
                qkv_dst1 = qkv::destination(qkv_e, row, item0 + 1, row < m && item0 + 1 < items, status);
                qkv::load_angles(qkv_e, row, col_half, row < m, angles);
            }
            ok = mbar_wait(&acc_full[buf], (local >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            if (mode == MODE_QKV)
                qkv::two_heads(qkv_e, qkv_norm_w, tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN),
                               n0 / qkv::HEAD_DIM, col_half, qkv_dst0, qkv_dst1, angles);
#pragma unroll 1
            for (int c0 = col_half * (BN / 2); c0 < (col_half + 1) * (BN / 2) && mode != MODE_QKV; c0 += 32) {
                float v[32];
                tmem_load32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN + c0), v);
                const int col = n0 + c0;
                if (row >= m || col >= n) continue;
                if (mode == MODE_SWIGLU) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (col + half * 16 >= n) break;
                        unsigned packed[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float g0 = v[half * 16 + 2 * i], g1 = v[half * 16 + 2 * i + 1];
                            const float u0 = v[half * 16 + 8 + 2 * i], u1 = v[half * 16 + 9 + 2 * i];
                            __nv_bfloat162 y = __floats2bfloat162_rn(silu_mul(g0, u0), silu_mul(g1, u1));
                            packed[i] = *reinterpret_cast<unsigned*>(&y);
                        }
                        *reinterpret_cast<uint4*>(out_act + (size_t)row * ld_act + (col + half * 16) / 2) =
                            make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                } else {
                    float* dst = c + (size_t)row * ldc + col;
                    // whole 32-byte sectors where the rows allow it: a thread's stores are a row each
                    const bool by8 = ((uintptr_t)c % 32 == 0) && ldc % 8 == 0 && n % 8 == 0;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (col + i >= n) break;
                        float4 x = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        float4 y = make_float4(v[i + 4], v[i + 5], v[i + 6], v[i + 7]);
                        const bool second = col + i + 4 < n;
                        if (mode == MODE_ACCUMULATE) {
                            const float4 old = *reinterpret_cast<const float4*>(dst + i);
                            x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
                            if (second) {
                                const float4 old2 = *reinterpret_cast<const float4*>(dst + i + 4);
                                y.x += old2.x; y.y += old2.y; y.z += old2.z; y.w += old2.w;
                            }
                        }
                        if (by8) {
                            store_f32x8(dst + i, x, y);
                        } else {
                            *reinterpret_cast<float4*>(dst + i) = x;
                            if (second) *reinterpret_cast<float4*>(dst + i + 4) = y;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(&acc_empty[buf], 0));
        }
    }
    if (!ok) atomicCAS(status, 0, TI_ERR_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                      // nobody leaves while its pair may still signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

extern "C" int ti_gemm_tcgen05_2sm_supported(int m, int n, int k, int lda, int ldw, int ldc, int mode) {
    if (m < 1 || n < 1 || k < 8 || k % 8 || lda % 8 || ldw % 8) return 0;
    if (mode == MODE_SWIGLU) return n % 16 == 0;
    return n % 4 == 0 && ldc % 4 == 0;
}

namespace {

int launch_pairs(const void* a, const void* w, const qkv::Epilogue& e, float* c, void* out_act, int m, int n,
                 int k, int lda, int ldw, int ldc, int ld_act, int mode, int* status, void* stream) {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    CUtensorMap map_a, map_w;
    if (int rc = make_map_bf16(&map_a, a, m, k, lda, 128, "gemm_tcgen05_2sm")) return rc;
    if (int rc = make_map_bf16(&map_w, w, n, k, ldw, 128, "gemm_tcgen05_2sm")) return rc;
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e2 = cudaFuncSetAttribute(gemm_tcgen05_2sm_kernel<256>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, Pair<256>::SMEM);
        if (e2 != cudaSuccess) return ti_fail("gemm_tcgen05_2sm: %s", cudaGetErrorString(e2));
        configured.mark();
    }
    const int tiles = ((m + BM - 1) / BM) * ((n + 255) / 256);
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    ti_launch_pdl(gemm_tcgen05_2sm_kernel<256>, 2 * pairs, THREADS, Pair<256>::SMEM, (cudaStream_t)stream,
                  map_a, map_w, e, c, (bf16*)out_act, m, n, k, ldc, ld_act, mode, status);
    return ti_check_launch("gemm_tcgen05_2sm");
}

}  // namespace

// Same contract as ti_gemm_tcgen05; meant for outputs with at least as many 256 x 256 tiles as the GPU
// has pairs of SMs.
extern "C" int ti_gemm_tcgen05_2sm(const void* a, const void* w, float* c, void* out_act, int m, int n,
                                   int k, int lda, int ldw, int ldc, int ld_act, int mode, int* status,
                                   void* stream) {
    if (m == 0 || n == 0) return 0;
    TI_REQUIRE(mode >= MODE_STORE && mode <= MODE_SWIGLU, "gemm_tcgen05_2sm: mode %d", mode);
    TI_REQUIRE(ti_gemm_tcgen05_2sm_supported(m, n, k, lda, ldw, ldc, mode),
               "gemm_tcgen05_2sm: K=%d and the row strides %d, %d must be multiples of 8, N=%d a multiple "
               "of 4 (16 with SwiGLU)", k, lda, ldw, n);
    TI_REQUIRE((uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0, "gemm_tcgen05_2sm: operands must be 16-byte aligned");
    TI_REQUIRE(mode == MODE_SWIGLU ? ((uintptr_t)out_act % 16 == 0 && ld_act % 8 == 0) : (uintptr_t)c % 16 == 0,
               "gemm_tcgen05_2sm: the output must be 16-byte aligned");
    return launch_pairs(a, w, qkv::Epilogue{}, c, out_act, m, n, k, lda, ldw, ldc, ld_act, mode, status, stream);
}

// The QKV product of a prompt portion with the epilogue of qkv_epilogue.cuh (head size 128):
// w is [(heads + 2 kv_heads) * 128, k]; nothing but q_out and the pages is written.
extern "C" int ti_gemm_tcgen05_2sm_qkv(const void* a, const void* w, int m, int k, int lda, int ldw,
                                       const float* q_weight, const float* k_weight, float eps,
                                       const float* table, const int* positions, const int* req_of_tok,
                                       const int* block_table, int bt_stride, void* pages, int num_pages,
                                       int page_size, int write_kv, int num_heads, int num_kv_heads,
                                       void* q_out, int* status, void* stream) {
    if (m == 0) return 0;
    const int n = (num_heads + 2 * num_kv_heads) * qkv::HEAD_DIM;
    TI_REQUIRE(k >= 8 && k % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tcgen05_2sm_qkv: K=%d and the row strides %d, %d must be multiples of 8", k, lda, ldw);
    TI_REQUIRE((uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)q_out % 32 == 0 &&
               (uintptr_t)pages % 32 == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)q_weight % 16 == 0 &&
               (uintptr_t)k_weight % 16 == 0, "gemm_tcgen05_2sm_qkv: operands must be 16-byte aligned, q_out and the pages 32-byte");
    const qkv::Epilogue e{q_weight, k_weight, eps, table, positions, req_of_tok, block_table, bt_stride,
                          (bf16*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads, (bf16*)q_out};
    return launch_pairs(a, w, e, nullptr, nullptr, m, n, k, lda, ldw, 0, 0, MODE_QKV, status, stream);
}
