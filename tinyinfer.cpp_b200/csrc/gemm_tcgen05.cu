// Matrix product on the 5th-generation tensor cores: C[M,N] (+)= A[M,K] * W[N,K]^T, bfloat16
// operands, float32 accumulation in tensor memory.  This is the prefill product (M > 64).
//
// The kernel is persistent: one block per SM walks over 128 x BN tiles of C (BN = 256; 128 when
// the output is too narrow to give every SM a wide tile; 64 when even those leave more than half
// of the SMs without one: a portion of 128 rows and N = 1,024 then has 16 tiles instead of 8; a
// prefill of 100 to 256 tokens at the 0.6B sizes is 1 to 5 % shorter for it).  Warp 0 feeds a ring of
// shared-memory stages with TMA tile loads (64 elements of K = one 128-byte swizzled row per
// matrix row); warp 1 issues tcgen05.mma (128 x BN x 16, both operands K-major from shared
// memory) into one of two accumulators in TMEM and hands each stage back with tcgen05.commit;
// warps 2-9 read a finished accumulator with tcgen05.ld (a warp reads the 32 TMEM lanes = rows
// that its position in the warpgroup allows) and run the epilogue while the next tile's
// products already fill the other accumulator.  Epilogues: store, accumulate into C (the
// residual stream), SwiGLU over 8 gate + 8 up columns into bfloat16, or (BN = 256) the QKV
// epilogue of qkv_epilogue.cuh: head norm, rotation and the store into the paged cache.  Rows and columns past
// M, N and K are zero-filled by TMA on the way in and skipped on the way out.
//
// The k order of the accumulation is fixed (ascending blocks of 64, 16 at a time), so an
// output element does not depend on the tile around it, nor on M as long as K is not cut:
// an output of so few tiles that most SMs would idle (a short prompt portion into a narrow
// output: 512 rows x 1,024 columns are 32 tiles of 128 x 128) has its K cut into equal runs, a
// work unit per (tile, run); a unit stores its sums into its run's slab of a float32 workspace,
// and a second launch adds the slabs in ascending order of K into C.  Every wait on an mbarrier
// is bounded: on a timeout the block records status 2, frees its tensor memory and returns.
#include "qkv_epilogue.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 320;       // TMA warp, MMA warp, eight epilogue warps

template <int BN> struct Tile {
    static constexpr int STAGES = BN == 256 ? 4 : BN == 128 ? 6 : 8;
    static constexpr int STAGE_A = BM * BK * 2, STAGE_B = BN * BK * 2;
    static constexpr int SMEM = STAGES * (STAGE_A + STAGE_B) + 1024 /* alignment */ + 256 /* barriers */;
    static constexpr unsigned TMEM_COLS = 2 * BN;     // two accumulators
};

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SWIGLU = 2, MODE_QKV = 3 };
enum { TI_ERR_TIMEOUT = 2 };

// Work unit `unit` of a product whose K is cut into `splits` runs: its tile and its k blocks.
struct Unit { int tile, run, kb_begin, kb_end; };
__device__ __forceinline__ Unit unit_of(int unit, int splits, int num_kb) {
    if (splits == 1) return {unit, 0, 0, num_kb};
    const int tile = unit / splits, run = unit - tile * splits;
    return {tile, run, num_kb * run / splits, num_kb * (run + 1) / splits};
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ qkv::Epilogue qkv_e, float* __restrict__ c,
                    bf16* __restrict__ out_act, int m, int n, int k, int ldc, int ld_act, int mode,
                    float* __restrict__ ws, int splits, int* __restrict__ status) {
    using T = Tile<BN>;
    constexpr int STAGES = T::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stage_a = smem;
    unsigned char* stage_b = smem + STAGES * T::STAGE_A;
    unsigned long long* bars = (unsigned long long*)(smem + STAGES * (T::STAGE_A + T::STAGE_B));
    unsigned long long* full = bars;                     // [STAGES] TMA -> MMA
    unsigned long long* empty = bars + STAGES;           // [STAGES] MMA -> TMA
    unsigned long long* acc_full = bars + 2 * STAGES;    // [2] MMA -> epilogue
    unsigned long long* acc_empty = bars + 2 * STAGES + 2;   // [2] epilogue -> MMA
    unsigned* tmem_slot = (unsigned*)(bars + 2 * STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (k + BK - 1) / BK;
    const int tiles_m = (m + BM - 1) / BM, tiles_n = (n + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    // a work unit: tile unit / splits, k blocks [num_kb * r / splits, num_kb * (r + 1) / splits) for r = unit % splits
    const int num_units = num_tiles * splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, T::TMEM_COLS);
    }
    __shared__ float qkv_norm_w[2 * qkv::HEAD_DIM];
    if (mode == MODE_QKV) qkv::load_norm_weights(qkv_e, qkv_norm_w, threadIdx.x, THREADS);
    pdl_launch();
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    // tiles in order of m fastest, so that blocks running together share few panels of W
    bool ok = true;
    if (warp == 0) {
        if (lane == 0) {
            // The weights do not depend on the kernel before this one: the first ring-full of W
            // tiles is requested before waiting for it; its results (A) follow after the wait.
            int primed = 0;
            for (int unit = blockIdx.x; unit < num_units && primed < STAGES; unit += gridDim.x) {
                const Unit u = unit_of(unit, splits, num_kb);
                const int n0 = (u.tile / tiles_m) * BN;
                for (int kb = u.kb_begin; kb < u.kb_end && primed < STAGES; ++kb, ++primed) {
                    mbar_expect_tx(&full[primed], T::STAGE_A + T::STAGE_B);
                    tma_load_2d(stage_b + primed * T::STAGE_B, &map_w, &full[primed], kb * BK, n0);
                }
            }
            pdl_wait();
            int it = 0;
            for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
                const Unit u = unit_of(unit, splits, num_kb);
                const int m0 = (u.tile % tiles_m) * BM, n0 = (u.tile / tiles_m) * BN;
                for (int kb = u.kb_begin; kb < u.kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= primed) {
                        ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1);
                        if (!ok) break;
                        mbar_expect_tx(&full[s], T::STAGE_A + T::STAGE_B);
                        tma_load_2d(stage_b + s * T::STAGE_B, &map_w, &full[s], kb * BK, n0);
                    }
                    tma_load_2d(stage_a + s * T::STAGE_A, &map_a, &full[s], kb * BK, m0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // bf16 x bf16 -> f32, both K-major, N at bit 17 (/8), M at bit 24 (/16)
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                   ((unsigned)(BM >> 4) << 24);
            int it = 0, local = 0;
            for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++local) {
                const Unit u = unit_of(unit, splits, num_kb);
                const int kb_begin = u.kb_begin, kb_end = u.kb_end;
                const int buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1);   // the epilogue has read it
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned tmem_acc = tmem_base + (unsigned)(buf * BN);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned long long da = umma_desc(stage_a + s * T::STAGE_A);
                    const unsigned long long db = umma_desc(stage_b + s * T::STAGE_B);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // 16 elements of K = 32 bytes further inside the swizzled row
                        umma_bf16(tmem_acc, da + (unsigned long long)(kk * UMMA_K * 2 >> 4),
                                  db + (unsigned long long)(kk * UMMA_K * 2 >> 4), idesc, kb != kb_begin || kk != 0);
                    }
                    umma_commit(&empty[s]);           // the stage is free once these MMAs have read it
                }
                umma_commit(&acc_full[buf]);          // the tile's accumulator is complete
            }
        }
    } else {
        const int quarter = warp & 3;                 // the TMEM lanes this warp may read
        const int col_half = (warp - 2) >> 2;         // two warps share a quarter: half of the columns each
        pdl_wait();                                   // C and what the QKV epilogue reads belong to the chain
        int local = 0;
        for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++local) {
            const Unit u = unit_of(unit, splits, num_kb);
            const int tile = u.tile;
            if (splits > 1) {                     // this run's sums go to its slab of the workspace as they are
                c = ws + (size_t)u.run * m * n;
                ldc = n;
                mode = MODE_STORE;
            }
            const int buf = local & 1;
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            const int row = m0 + quarter * 32 + lane;
            // narrow tiles that add to C fetch C's old values while the products still run
            constexpr int OLD = BN <= 128 ? BN / 8 : 1;
            float4 old[OLD];
            if constexpr (BN <= 128) {
                if (mode == MODE_ACCUMULATE) {
                    const float* src = c + (size_t)row * ldc + n0 + col_half * (BN / 2);
#pragma unroll
                    for (int i = 0; i < OLD; ++i)
                        old[i] = row < m && n0 + col_half * (BN / 2) + 4 * i < n
                                     ? __ldcg(reinterpret_cast<const float4*>(src + 4 * i))
                                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
            // where the tile's two heads go, and this warp's half of the token's sines and cosines:
            // requested while the products still run
            bf16 *qkv_dst0 = nullptr, *qkv_dst1 = nullptr;
            qkv::Angles angles;
            if constexpr (BN == 256) {
                if (mode == MODE_QKV) {
                    const int item0 = n0 / qkv::HEAD_DIM, items = qkv_e.num_heads + 2 * qkv_e.num_kv_heads;
                    qkv_dst0 = qkv::destination(qkv_e, row, item0, row < m && item0 < items, status);
                    qkv_dst1 = qkv::destination(qkv_e, row, item0 + 1, row < m && item0 + 1 < items, status);
                    qkv::load_angles(qkv_e, row, col_half, row < m, angles);
                }
            }
            ok = mbar_wait(&acc_full[buf], (local >> 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if constexpr (BN == 256) {
                if (mode == MODE_QKV)
                    qkv::two_heads(qkv_e, qkv_norm_w, tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN),
                                   n0 / qkv::HEAD_DIM, col_half, qkv_dst0, qkv_dst1, angles);
            }
#pragma unroll
            for (int cc = 0; cc < BN / 64; ++cc) {
                if (mode == MODE_QKV) break;
                const int c0 = col_half * (BN / 2) + cc * 32;
                float v[32];
                tmem_load32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN + c0), v);
                const int col = n0 + c0;
                if (row >= m || col >= n) continue;
                if (mode == MODE_SWIGLU) {
                    // columns: 8 gate, their 8 up, 8 gate, their 8 up
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
                            float4 was, was2 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            if constexpr (BN <= 128) {
                                was = old[cc * 8 + i / 4];
                                was2 = old[cc * 8 + i / 4 + 1];
                            } else {
                                was = *reinterpret_cast<const float4*>(dst + i);
                                if (second) was2 = *reinterpret_cast<const float4*>(dst + i + 4);
                            }
                            x.x += was.x; x.y += was.y; x.z += was.z; x.w += was.w;
                            y.x += was2.x; y.y += was2.y; y.z += was2.z; y.w += was2.w;
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
            // all of this warp's reads of the accumulator are done: hand it back
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    if (!ok) atomicCAS(status, 0, TI_ERR_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        tmem_dealloc(tmem_base, T::TMEM_COLS);
    }
}

// table[t] = {cos(pos_t * inv_freq[0 .. half)), sin(...)}: the rotation of every token of a step.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  int num_tokens, int half, float* __restrict__ table) {
    pdl_launch();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_tokens * half) return;
    const int t = i / half, k = i % half;
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[k], &sn, &cs);
    table[(size_t)t * 2 * half + k] = cs;
    table[(size_t)t * 2 * half + half + k] = sn;
}

// c (+)= the sum of the runs' slabs ws[run][m][n], in ascending order of the run (of K).
__global__ void __launch_bounds__(256)
gemm_split_merge_kernel(const float* ws, float* __restrict__ c, int m, int n, int ldc, int splits,
                        int accumulate) {
    pdl_launch();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // a float4 of the output
    const int n4 = n / 4;
    pdl_wait();
    if (i >= (long long)m * n4) return;
    const int row = (int)(i / n4), col = (int)(i % n4) * 4;
    const size_t slab = (size_t)m * n;
    const float* src = ws + (size_t)row * n + col;
    float4 was = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (accumulate) was = __ldcg(reinterpret_cast<const float4*>(c + (size_t)row * ldc + col));
    float4 sum = __ldcg(reinterpret_cast<const float4*>(src));
    for (int r = 1; r < splits; ++r) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + r * slab));
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    *reinterpret_cast<float4*>(c + (size_t)row * ldc + col) =
        make_float4(was.x + sum.x, was.y + sum.y, was.z + sum.z, was.w + sum.w);
}

constexpr int MAX_SPLITS = 8, MIN_RUN_KB = 4;

// In how many runs K is cut (1 = not at all): the count with the shortest estimated time, if that
// is a twentieth shorter than the uncut product's.  The estimate, in microseconds, from timings of
// this kernel on a B200: the (tile, run) units go over the SMs in waves; a wave costs 1.5 plus
// 0.3 per k block of a run (a 128 x 128 tile takes in 32 KB per k block); the launch that adds
// the runs costs 2.5 plus the reading of the runs' slabs and of C and the writing of C at 4 TB/s.
// It depends on the product's sizes and the number of SMs alone.
int choose_splits(int m, int n, int k, int mode, int sms) {
    if (mode != MODE_STORE && mode != MODE_ACCUMULATE) return 1;
    if (n % 4) return 1;
    const int tiles = ((m + BM - 1) / BM) * ((n + 127) / 128), num_kb = (k + BK - 1) / BK;
    const double slab_us = (double)m * n * 4.0 / 4.0e6;
    int best = 1;
    double best_us = 0.0, uncut_us = 0.0;
    for (int s = 1; s <= MAX_SPLITS && (s == 1 || s * MIN_RUN_KB <= num_kb); ++s) {
        const int waves = (tiles * s + sms - 1) / sms;
        double us = waves * (1.5 + 0.3 * ((num_kb + s - 1) / s));
        if (s > 1) us += 2.5 + (s + 2) * slab_us;
        if (s == 1) uncut_us = us;
        if (s == 1 || us < best_us) { best = s; best_us = us; }
    }
    return best_us <= 0.95 * uncut_us ? best : 1;
}

// width: the tiles' columns, 256, 128 or 64
int launch_tiles(const void* a, const void* w, const qkv::Epilogue& e, float* c, void* out_act, int m, int n,
                 int k, int lda, int ldw, int ldc, int ld_act, int mode, int width, float* ws, int splits,
                 int* status, void* stream, bool add_runs = true) {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int tiles_m = (m + BM - 1) / BM;
    CUtensorMap map_a, map_w;
    if (int rc = make_map_bf16(&map_a, a, m, k, lda, BM, "gemm_tcgen05")) return rc;
    if (int rc = make_map_bf16(&map_w, w, n, k, ldw, width, "gemm_tcgen05")) return rc;
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e2 = cudaFuncSetAttribute(gemm_tcgen05_kernel<256>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, Tile<256>::SMEM);
        if (e2 == cudaSuccess)
            e2 = cudaFuncSetAttribute(gemm_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Tile<128>::SMEM);
        if (e2 == cudaSuccess)
            e2 = cudaFuncSetAttribute(gemm_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Tile<64>::SMEM);
        if (e2 != cudaSuccess) return ti_fail("gemm_tcgen05: %s", cudaGetErrorString(e2));
        configured.mark();
    }
    if (width == 256) {
        const int tiles = tiles_m * ((n + 255) / 256) * splits;
        ti_launch_pdl(gemm_tcgen05_kernel<256>, tiles < sms ? tiles : sms, THREADS, Tile<256>::SMEM,
                      (cudaStream_t)stream, map_a, map_w, e, c, (bf16*)out_act, m, n, k, ldc, ld_act, mode, ws,
                      splits, status);
    } else if (width == 128) {
        const int tiles = tiles_m * ((n + 127) / 128) * splits;
        ti_launch_pdl(gemm_tcgen05_kernel<128>, tiles < sms ? tiles : sms, THREADS, Tile<128>::SMEM,
                      (cudaStream_t)stream, map_a, map_w, e, c, (bf16*)out_act, m, n, k, ldc, ld_act, mode, ws,
                      splits, status);
    } else {
        const int tiles = tiles_m * ((n + 63) / 64) * splits;
        ti_launch_pdl(gemm_tcgen05_kernel<64>, tiles < sms ? tiles : sms, THREADS, Tile<64>::SMEM,
                      (cudaStream_t)stream, map_a, map_w, e, c, (bf16*)out_act, m, n, k, ldc, ld_act, mode, ws,
                      splits, status);
    }
    if (int rc = ti_check_launch("gemm_tcgen05")) return rc;
    if (splits > 1 && add_runs) {
        const long long quads = (long long)m * (n / 4);
        ti_launch_pdl(gemm_split_merge_kernel, (unsigned)((quads + 255) / 256), 256, 0, (cudaStream_t)stream,
                      (const float*)ws, c, m, n, ldc, splits, mode == MODE_ACCUMULATE ? 1 : 0);
        return ti_check_launch("gemm_split_merge");
    }
    return 0;
}

}  // namespace

extern "C" int ti_gemm_tcgen05_supported(int m, int n, int k, int lda, int ldw, int ldc, int mode) {
    if (m < 1 || n < 1 || k < 8 || k % 8 || lda % 8 || ldw % 8) return 0;
    if (mode == MODE_SWIGLU) return n % 16 == 0;
    return n % 4 == 0 && ldc % 4 == 0;
}

// The runs of K that ti_gemm_tcgen05 would like for these sizes (1: K is not cut); with more than
// one it wants runs * m * n float32 values of scratch.
extern "C" int ti_gemm_tcgen05_splits(int m, int n, int k, int mode) {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms > 0 && m > 0 && n > 0 ? choose_splits(m, n, k, mode, sms) : 1;
}

// c (+)= the runs' slabs ws[run][m][n] of a product that was launched with `leave_runs`.
extern "C" int ti_gemm_tcgen05_add_runs(const float* ws, float* c, int m, int n, int ldc, int runs,
                                        int accumulate, void* stream) {
    if (m == 0 || n == 0 || runs < 1) return 0;
    TI_REQUIRE(n % 4 == 0 && ldc % 4 == 0 && (uintptr_t)ws % 16 == 0 && (uintptr_t)c % 16 == 0,
               "gemm_tcgen05_add_runs: N=%d and the row stride %d must be multiples of 4", n, ldc);
    const long long quads = (long long)m * (n / 4);
    ti_launch_pdl(gemm_split_merge_kernel, (unsigned)((quads + 255) / 256), 256, 0, (cudaStream_t)stream, ws, c, m,
                  n, ldc, runs, accumulate ? 1 : 0);
    return ti_check_launch("gemm_split_merge");
}

// mode 0: c = a w^T; 1: c += a w^T; 2: out_act[m, n/2] = SwiGLU over groups of 8 gate + 8 up columns.
// ws: null, or the scratch for ti_gemm_tcgen05_splits(m, n, k, mode) runs of K (16-byte aligned).
// leave_runs: with K cut, do not add the runs into c; the caller does (ti_gemm_tcgen05_add_runs, or
// a norm that completes its rows from the slabs).
extern "C" int ti_gemm_tcgen05(const void* a, const void* w, float* c, void* out_act, int m, int n,
                               int k, int lda, int ldw, int ldc, int ld_act, int mode, float* ws,
                               int leave_runs, int* status, void* stream) {
    if (m == 0 || n == 0) return 0;
    TI_REQUIRE(mode >= MODE_STORE && mode <= MODE_SWIGLU, "gemm_tcgen05: mode %d", mode);
    TI_REQUIRE(ti_gemm_tcgen05_supported(m, n, k, lda, ldw, ldc, mode),
               "gemm_tcgen05: K=%d and the row strides %d, %d must be multiples of 8, N=%d a multiple "
               "of 4 (16 with SwiGLU)", k, lda, ldw, n);
    TI_REQUIRE((uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0, "gemm_tcgen05: operands must be 16-byte aligned");
    TI_REQUIRE(mode == MODE_SWIGLU ? ((uintptr_t)out_act % 16 == 0 && ld_act % 8 == 0)
                                   : (uintptr_t)c % 16 == 0,
               "gemm_tcgen05: the output must be 16-byte aligned");
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    // wide tiles when they still give every SM one; else twice as many narrow ones; else, when
    // those still leave more than half of the SMs idle, four times as many of 64 columns
    const int tiles_m = (m + BM - 1) / BM;
    const int splits = ws != nullptr ? choose_splits(m, n, k, mode, sms) : 1;
    if (splits > 1) {
        TI_REQUIRE((uintptr_t)ws % 16 == 0, "gemm_tcgen05: the scratch must be 16-byte aligned");
        return launch_tiles(a, w, qkv::Epilogue{}, c, out_act, m, n, k, lda, ldw, ldc, ld_act, mode, 128, ws,
                            splits, status, stream, !leave_runs);
    }
    const int width = tiles_m * ((n + 255) / 256) >= sms ? 256 : tiles_m * ((n + 127) / 128) * 2 >= sms ? 128 : 64;
    return launch_tiles(a, w, qkv::Epilogue{}, c, out_act, m, n, k, lda, ldw, ldc, ld_act, mode, width, nullptr, 1,
                        status, stream);
}

// The QKV product of a prompt portion with the epilogue of qkv_epilogue.cuh (head size 128), on
// 128 x 256 tiles: w is [(heads + 2 kv_heads) * 128, k]; nothing but q_out and the pages is written.
extern "C" int ti_gemm_tcgen05_qkv(const void* a, const void* w, int m, int k, int lda, int ldw,
                                   const float* q_weight, const float* k_weight, float eps,
                                   const float* table, const int* positions, const int* req_of_tok,
                                   const int* block_table, int bt_stride, void* pages, int num_pages,
                                   int page_size, int write_kv, int num_heads, int num_kv_heads,
                                   void* q_out, int* status, void* stream) {
    if (m == 0) return 0;
    const int n = (num_heads + 2 * num_kv_heads) * qkv::HEAD_DIM;
    TI_REQUIRE(k >= 8 && k % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tcgen05_qkv: K=%d and the row strides %d, %d must be multiples of 8", k, lda, ldw);
    TI_REQUIRE((uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)q_out % 32 == 0 &&
               (uintptr_t)pages % 32 == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)q_weight % 16 == 0 &&
               (uintptr_t)k_weight % 16 == 0, "gemm_tcgen05_qkv: operands must be 16-byte aligned, q_out and the pages 32-byte");
    const qkv::Epilogue e{q_weight, k_weight, eps, table, positions, req_of_tok, block_table, bt_stride,
                          (bf16*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads, (bf16*)q_out};
    return launch_tiles(a, w, e, nullptr, nullptr, m, n, k, lda, ldw, 0, 0, MODE_QKV, 256, nullptr, 1, status, stream);
}

// table [num_tokens][2][half] float32: cosines then sines of positions[t] * inv_freq[k].
extern "C" int ti_rope_table(const int* positions, const float* inv_freq, int num_tokens, int half,
                             float* table, void* stream) {
    if (num_tokens == 0 || half == 0) return 0;
    const int total = num_tokens * half;
    ti_launch_pdl(rope_table_kernel, (total + 255) / 256, 256, 0, (cudaStream_t)stream, positions, inv_freq,
                  num_tokens, half, table);
    return ti_check_launch("rope_table");
}
