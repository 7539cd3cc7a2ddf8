// Matrix product for few rows on the 5th-generation tensor cores, for matrices large enough that
// the product is bound by streaming W from HBM (the decode step of big models, the LM head):
// C[M,N] (+)= A[M,K] * W[N,K]^T, M <= 64, bfloat16 operands, float32 accumulation in tensor memory.
//
// The roles of the operands are swapped: 128 rows of W are the MMA's M side, the (padded) rows of
// A its N side (16, 32 or 64), so a tile of W is read once for all rows of A and the activations
// re-read per tile are an eighth of the weights at most.  W arrives by TMA in 16 KB boxes (128
// rows x 64 of K, 128-byte swizzle) into a ring that holds 160-190 KB per SM in flight; no
// register takes part in the transfer.  Because N / 128 tiles are too few for 148 SMs, K is split:
// a work unit is (tile, split), the persistent blocks take units in turn, and the splits of a
// tile put their partial sums into a workspace; the block that finishes a tile last (an atomic
// ticket) adds the partial sums in ascending order of the split and runs the epilogue (store,
// accumulate into C, or SwiGLU over 8 gate + 8 up rows of W).  The number of splits depends on N,
// K and the number of SMs only, so an output's sum does not depend on M or on the batch around it.
//
// Warp 0 issues TMA (the weights of the first stages before the kernel waits for its
// predecessor), warp 1 issues tcgen05.mma into one of two accumulators, warps 2-5 read
// accumulators with tcgen05.ld.  Every wait on an mbarrier is bounded: on a timeout the block
// records status 2, frees its tensor memory and returns.
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BW = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;       // TMA warp, MMA warp, four epilogue warps
constexpr int MAX_SPLITS = 16;
constexpr int BLOCKS_PER_SM = 2;   // two half-size rings: one block's epilogue overlaps the other's stream

template <int NTOK> struct Few {
    static constexpr int STAGES = NTOK == 64 ? 4 : 5;
    static constexpr int STAGE_W = BW * BK * 2, STAGE_X = NTOK * BK * 2;
    static constexpr int SMEM = STAGES * (STAGE_W + STAGE_X) + 1024 /* alignment */ + 256 /* barriers */;
    static constexpr unsigned TMEM_COLS = 2 * NTOK < 32 ? 32 : 2 * NTOK;     // two accumulators
};

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SWIGLU = 2 };
enum { TI_ERR_TIMEOUT = 2 };

__device__ __forceinline__ void epilogue_sync() {     // the four epilogue warps only
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
}

// The work units of one block in the order it takes them: unit = tile * splits + split, k blocks
// [kb, kb_end) of the split.
struct Units {
    int unit, num_units, splits, num_kb, step;
    __device__ Units(int first, int step_, int num_units_, int splits_, int num_kb_)
        : unit(first), num_units(num_units_), splits(splits_), num_kb(num_kb_), step(step_) {}
    __device__ bool done() const { return unit >= num_units; }
    __device__ int tile() const { return unit / splits; }
    __device__ int split() const { return unit % splits; }
    __device__ int kb_begin() const { return (int)((long long)split() * num_kb / splits); }
    __device__ int kb_end() const { return (int)((long long)(split() + 1) * num_kb / splits); }
    __device__ void next() { unit += step; }
};

// 16 tokens' values of W row `n_row` (this thread's), tokens tok0 .. tok0 + 15.
__device__ __forceinline__ void finish16(const float (&v)[16], int tok0, int n_row, int lane, float* c,
                                         bf16* out_act, int m, int n, int ldc, int ld_act, int mode) {
    if (mode == MODE_SWIGLU) {
        // rows of W: 8 gate, their 8 up, ...; lane l (l % 16 < 8) holds a gate row, lane l + 8 its up row
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float up = __shfl_down_sync(0xffffffffu, v[i], 8);
            const int tok = tok0 + i;
            if ((lane & 8) == 0 && tok < m && n_row + 8 < n) {
                const int col = (n_row - (lane & 7)) / 2 + (lane & 7);
                out_act[(size_t)tok * ld_act + col] = __float2bfloat16_rn(v[i] / (1.0f + expf(-v[i])) * up);
            }
        }
    } else if (n_row < n) {
        // When adding to C, all old values are requested before the first sum is stored: written
        // one after the other, every read would wait behind the store before it (the compiler
        // cannot tell that the addresses differ), a round trip to L2 per row (the down projection
        // of the 8B shape at 64 rows: 55 -> 34 microseconds).
        float old[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
            old[i] = mode == MODE_ACCUMULATE && tok0 + i < m ? __ldcg(c + (size_t)(tok0 + i) * ldc + n_row) : 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int tok = tok0 + i;
            if (tok >= m) break;
            c[(size_t)tok * ldc + n_row] = old[i] + v[i];
        }
    }
}

template <int NTOK>
__global__ void __launch_bounds__(THREADS, BLOCKS_PER_SM)
gemm_few_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                float* __restrict__ c, bf16* __restrict__ out_act, float* __restrict__ ws,
                int* __restrict__ tickets, int m, int n, int k, int ldc, int ld_act, int mode, int splits,
                int* __restrict__ status) {
    using T = Few<NTOK>;
    constexpr int STAGES = T::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_w = smem;
    unsigned char* stage_x = smem + STAGES * T::STAGE_W;
    unsigned long long* bars = (unsigned long long*)(smem + STAGES * (T::STAGE_W + T::STAGE_X));
    unsigned long long* full = bars;                     // [STAGES] TMA -> MMA
    unsigned long long* empty = bars + STAGES;           // [STAGES] MMA -> TMA
    unsigned long long* acc_full = bars + 2 * STAGES;    // [2] MMA -> epilogue
    unsigned long long* acc_empty = bars + 2 * STAGES + 2;   // [2] epilogue -> MMA
    unsigned* tmem_slot = (unsigned*)(bars + 2 * STAGES + 4);
    int* ticket_slot = (int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (k + BK - 1) / BK;
    const int num_units = ((n + BW - 1) / BW) * splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, T::TMEM_COLS);
    pdl_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    bool ok = true;
    if (warp == 0) {
        if (lane == 0) {
            // the weights of the first ring-full of stages do not depend on the kernel before this one
            Units ahead(blockIdx.x, gridDim.x, num_units, splits, num_kb);
            int primed = 0;
            for (; !ahead.done() && primed < STAGES; ahead.next()) {
                const int n0 = ahead.tile() * BW;
                int kb = ahead.kb_begin();
                const int kb_end = ahead.kb_end();
                for (; kb < kb_end && primed < STAGES; ++kb, ++primed) {
                    mbar_expect_tx(&full[primed], T::STAGE_W + T::STAGE_X);
                    tma_load_2d(stage_w + primed * T::STAGE_W, &map_w, &full[primed], kb * BK, n0);
                }
                if (kb < kb_end) break;
            }
            pdl_wait();
            int it = 0;
            for (Units u(blockIdx.x, gridDim.x, num_units, splits, num_kb); !u.done() && ok; u.next()) {
                const int n0 = u.tile() * BW;
                const int kb_end = u.kb_end();
                for (int kb = u.kb_begin(); kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= primed) {
                        ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1);
                        if (!ok) break;
                        mbar_expect_tx(&full[s], T::STAGE_W + T::STAGE_X);
                        tma_load_2d(stage_w + s * T::STAGE_W, &map_w, &full[s], kb * BK, n0);
                    }
                    tma_load_2d(stage_x + s * T::STAGE_X, &map_x, &full[s], kb * BK, 0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = umma_idesc(BW, NTOK);
            int it = 0, local = 0;
            for (Units u(blockIdx.x, gridDim.x, num_units, splits, num_kb); !u.done() && ok; u.next(), ++local) {
                const int buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1);   // the epilogue has read it
                if (!ok) break;
                tc_fence_after();
                const unsigned tmem_acc = tmem_base + (unsigned)(buf * NTOK);
                const int kb_begin = u.kb_begin(), kb_end = u.kb_end();
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const unsigned long long dw = umma_desc(stage_w + s * T::STAGE_W);
                    const unsigned long long dx = umma_desc(stage_x + s * T::STAGE_X);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk)
                        umma_bf16(tmem_acc, dw + (unsigned long long)(kk * UMMA_K * 2 >> 4),
                                  dx + (unsigned long long)(kk * UMMA_K * 2 >> 4), idesc,
                                  (kb != kb_begin) || kk != 0);
                    umma_commit(&empty[s]);
                }
                umma_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;                 // the TMEM lanes this warp may read
        const int row_in_tile = quarter * 32 + lane;
        pdl_wait();                                   // C, the workspace and the tickets belong to the chain
        int local = 0;
        for (Units u(blockIdx.x, gridDim.x, num_units, splits, num_kb); !u.done() && ok; u.next(), ++local) {
            const int buf = local & 1;
            const int tile = u.tile();
            const int n_row = tile * BW + row_in_tile;
            ok = mbar_wait(&acc_full[buf], (local >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            float* part = ws + (size_t)u.unit * NTOK * BW;     // [NTOK][128]
#pragma unroll 1
            for (int t0 = 0; t0 < NTOK; t0 += 16) {
                float v[16];
                tmem_load16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * NTOK + t0), v);
                if (splits == 1) {
                    finish16(v, t0, n_row, lane, c, out_act, m, n, ldc, ld_act, mode);
                } else if (t0 < m) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) part[(size_t)(t0 + i) * BW + row_in_tile] = v[i];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (splits == 1) continue;
            // the tile is complete when all its splits have stored their sums; the last one adds them
            __threadfence();
            epilogue_sync();
            if (warp == 2 && lane == 0) *ticket_slot = atomicAdd(&tickets[tile], 1);
            epilogue_sync();
            if (*ticket_slot != splits - 1) continue;
            __threadfence();
            // Other blocks wrote the partial sums, so every load is a round trip to L2 of most of
            // a microsecond, and this merge is the exposed tail of the tile: the loads of several
            // splits (as many as the registers hold) are all requested before any is added, and
            // the additions then follow in ascending order of the split.
            const float* first = ws + (size_t)tile * splits * NTOK * BW + row_in_tile;
            constexpr int AT_ONCE = NTOK == 16 ? 8 : NTOK == 32 ? 3 : 1;
            float acc[NTOK];
#pragma unroll
            for (int i = 0; i < NTOK; ++i) acc[i] = 0.0f;
            for (int s0 = 0; s0 < splits; s0 += AT_ONCE) {
                float got[AT_ONCE][NTOK];
#pragma unroll
                for (int j = 0; j < AT_ONCE; ++j) {
                    // a split past the last one is read from the last one and counts as zero
                    const int sj = s0 + j < splits ? s0 + j : splits - 1;
                    const float* p = first + (size_t)sj * NTOK * BW;
#pragma unroll
                    for (int i = 0; i < NTOK; ++i) got[j][i] = __ldcg(p + (size_t)i * BW);
                }
#pragma unroll
                for (int j = 0; j < AT_ONCE; ++j) {
                    const bool live = s0 + j < splits;
#pragma unroll
                    for (int i = 0; i < NTOK; ++i) acc[i] += live ? got[j][i] : 0.0f;
                }
            }
#pragma unroll
            for (int t0 = 0; t0 < NTOK; t0 += 16) {
                if (t0 < m)
                    finish16(*reinterpret_cast<const float(*)[16]>(&acc[t0]), t0, n_row, lane, c, out_act, m, n,
                             ldc, ld_act, mode);
            }
            if (warp == 2 && lane == 0) tickets[tile] = 0;
        }
    }
    if (!ok) atomicCAS(status, 0, TI_ERR_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, T::TMEM_COLS);
    }
}

int padded_rows(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : 64; }

// The number of splits of K: the one that lets the busiest block stream the fewest blocks of K
// (each unit costs one more for its epilogue, a split tile two for the merge); smallest on a tie.
int choose_splits(int n, int k, int sms) {
    const int tiles = (n + BW - 1) / BW, num_kb = (k + BK - 1) / BK;
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= MAX_SPLITS && s * 2 <= num_kb || s == 1; ++s) {
        const long long units = (long long)tiles * s;
        const long long grid = units < sms ? units : sms;
        const long long cost = ((units + grid - 1) / grid) * ((num_kb + s - 1) / s + 1) + (s > 1 ? 2 : 0);
        if (best_cost < 0 || cost < best_cost) { best = s; best_cost = cost; }
    }
    return best;
}

int device_sms() {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms;
}

template <int NTOK>
int launch_few(const CUtensorMap& map_w, const CUtensorMap& map_x, float* c, bf16* out_act, float* ws,
               int* tickets, int m, int n, int k, int ldc, int ld_act, int mode, int splits, int sms,
               int* status, cudaStream_t stream) {
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_few_kernel<NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Few<NTOK>::SMEM);
        if (e != cudaSuccess) return ti_fail("gemm_tcgen05_few: %s", cudaGetErrorString(e));
        configured.mark();
    }
    const int units = ((n + BW - 1) / BW) * splits;
    const int slots = sms * BLOCKS_PER_SM;
    cudaError_t e = ti_launch_pdl(gemm_few_kernel<NTOK>, dim3(units < slots ? units : slots), dim3(THREADS),
                                  Few<NTOK>::SMEM, stream, map_w, map_x, c, out_act, ws, tickets, m, n, k, ldc,
                                  ld_act, mode, splits, status);
    if (e != cudaSuccess) return ti_fail("gemm_tcgen05_few: %s", cudaGetErrorString(e));
    return ti_check_launch("gemm_tcgen05_few");
}

}  // namespace

extern "C" int ti_gemm_tcgen05_few_supported(int m, int n, int k, int lda, int ldw, int mode) {
    if (m < 1 || m > 64 || n < 1 || k < 8 || k % 8 || lda % 8 || ldw % 8) return 0;
    return mode != MODE_SWIGLU || n % 16 == 0;
}

// What a call needs besides its operands: `*ws_floats` float32 values of workspace (0 if K is not
// split) and `*num_tickets` int32 counters that are zero before the first call and are left zero.
extern "C" int ti_gemm_tcgen05_few_scratch(int m, int n, int k, long long* ws_floats, int* num_tickets) {
    const int tiles = (n + BW - 1) / BW;
    const int splits = choose_splits(n, k, device_sms());
    *ws_floats = splits > 1 ? (long long)tiles * splits * padded_rows(m) * BW : 0;
    *num_tickets = tiles;
    return 0;
}

// mode 0: c = a w^T; 1: c += a w^T; 2: out_act[m, n/2] = SwiGLU over groups of 8 gate + 8 up rows of w.
extern "C" int ti_gemm_tcgen05_few(const void* a, const void* w, float* c, void* out_act, int m, int n,
                                   int k, int lda, int ldw, int ldc, int ld_act, int mode, float* ws,
                                   int* tickets, int* status, void* stream) {
    if (m == 0 || n == 0) return 0;
    TI_REQUIRE(ti_gemm_tcgen05_few_supported(m, n, k, lda, ldw, mode),
               "gemm_tcgen05_few: M=%d (1..64), K=%d and the row strides %d, %d (multiples of 8) or N=%d "
               "(a multiple of 16 with SwiGLU) are not supported", m, k, lda, ldw, n);
    TI_REQUIRE((uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0, "gemm_tcgen05_few: operands must be 16-byte aligned");
    const int sms = device_sms();
    const int splits = choose_splits(n, k, sms);
    TI_REQUIRE(tickets != nullptr && (splits == 1 || ws != nullptr), "gemm_tcgen05_few: scratch is missing");
    const int ntok = padded_rows(m);
    CUtensorMap map_w, map_x;
    if (int rc = make_map_bf16(&map_w, w, n, k, ldw, BW, "gemm_tcgen05_few")) return rc;
    if (int rc = make_map_bf16(&map_x, a, m, k, lda, ntok, "gemm_tcgen05_few")) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (ntok == 16)
        return launch_few<16>(map_w, map_x, c, (bf16*)out_act, ws, tickets, m, n, k, ldc, ld_act, mode, splits, sms, status, s);
    if (ntok == 32)
        return launch_few<32>(map_w, map_x, c, (bf16*)out_act, ws, tickets, m, n, k, ldc, ld_act, mode, splits, sms, status, s);
    return launch_few<64>(map_w, map_x, c, (bf16*)out_act, ws, tickets, m, n, k, ldc, ld_act, mode, splits, sms, status, s);
}
