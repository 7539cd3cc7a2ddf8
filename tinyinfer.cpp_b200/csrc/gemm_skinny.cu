// Matrix product for few rows (M <= 64, the decode step): C[M,N] (+)= A[M,K] * W[N,K]^T, bfloat16
// operands, float32 accumulation.  The work is bound by reading W once from HBM.
//
// A block owns a strip of 16 rows of W (16 outputs per token).  Its 8 warps split K in chunks
// of 32 that they take in turn, so the block reads each W row in contiguous 512-byte pieces.
// Operands go straight from global memory into tensor-core fragments (mma.sync m16n8k16, W as
// the 16-row A operand, tokens as the 8-column B operand): a thread loads 16 bytes = 8
// consecutive k of one W row and of one token, and the contraction index inside a chunk is
// permuted identically for both operands, which a sum over k allows.  The 8 partial sums of a
// block are added in a fixed order in shared memory, so an output does not depend on M, on the
// other rows or on the launch.
//
// Epilogues: store, accumulate into C (the residual stream), or SwiGLU: W holds, in every strip,
// 8 gate rows followed by their 8 up rows, and out[m, j] = silu(gate_j) * up_j in bfloat16.
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int STRIP = 16;
constexpr int CHUNK = 32;

enum { MODE_STORE = 0, MODE_ACCUMULATE = 1, MODE_SWIGLU = 2 };

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ROWS = 16: a block owns 16 rows of W.  ROWS = 8: it owns 8 (the upper half of the MMA's A
// operand is zero), which doubles the number of blocks for narrow outputs.
constexpr int SHORT_K = WARPS * CHUNK * 4;     // what four chunks per warp cover: 1,024
// BATCH: chunks of W a warp has in flight.  4 covers K <= 1,024 in one round and leaves registers
// for three blocks per SM (384 blocks of a 6,144-row weight then run as one wave instead of 1.3).
// STORE_ONLY: the kernel without its other two epilogues (the QKV product of a small model's
// decode step, which waits for this kernel once a layer: the shorter the kernel the better).
template <int NT, int ROWS, int BATCH, bool STORE_ONLY = false>
__global__ void __launch_bounds__(WARPS * 32, BATCH == 4 && NT == 1 ? 3 : 2)
gemm_skinny_kernel(const bf16* a, const bf16* __restrict__ w, float* __restrict__ c,
                   bf16* __restrict__ out_act, int m, int n, int k, int lda, int ldw, int ldc,
                   int ld_act, int mode) {
    constexpr int MP = NT * 8;                                  // padded token count
    __shared__ float part[WARPS][ROWS][MP + 1];
    if (STORE_ONLY) mode = MODE_STORE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    // rows past N are read from the last row and never stored
    const bf16* w_lo = w + (size_t)min(n0 + g, n - 1) * ldw + tq * 8;
    const bf16* w_hi = w + (size_t)min(n0 + g + 8, n - 1) * ldw + tq * 8;
    const bf16* a_row[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) a_row[j] = a + (size_t)min(j * 8 + g, m - 1) * lda + tq * 8;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    const int chunks = k / CHUNK;
    pdl_launch();
    for (int c0 = warp; c0 < chunks; c0 += WARPS * BATCH) {
        // all loads of the batch first: the product is bound by memory latency, not by arithmetic
        uint4 wl[BATCH], wh[BATCH];
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            const int ch = c0 + u * WARPS;
            if (ch < chunks) {
                wl[u] = ld_stream(w_lo + (size_t)ch * CHUNK);
                if (ROWS == 16) wh[u] = ld_stream(w_hi + (size_t)ch * CHUNK);
            }
        }
        // the weights do not depend on the kernel before this one; the activations do
        if (c0 == warp) pdl_wait();
        if constexpr (NT * BATCH <= 16) {
            // few tokens: all activations of the batch are requested at once (one round trip to
            // L2 behind the wait instead of one per chunk)
            uint4 xr[BATCH][NT];
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const int ch = c0 + u * WARPS;
                if (ch < chunks) {
#pragma unroll
                    for (int j = 0; j < NT; ++j)
                        xr[u][j] = *reinterpret_cast<const uint4*>(a_row[j] + (size_t)ch * CHUNK);
                }
            }
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const int ch = c0 + u * WARPS;
                if (ch >= chunks) break;
                if (ROWS == 8) wh[u] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mma_bf16(acc[j], wl[u].x, wh[u].x, wl[u].y, wh[u].y, xr[u][j].x, xr[u][j].y);
                    mma_bf16(acc[j], wl[u].z, wh[u].z, wl[u].w, wh[u].w, xr[u][j].z, xr[u][j].w);
                }
            }
        } else {
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const int ch = c0 + u * WARPS;
                if (ch >= chunks) break;
                if (ROWS == 8) wh[u] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint4 x = *reinterpret_cast<const uint4*>(a_row[j] + (size_t)ch * CHUNK);
                    mma_bf16(acc[j], wl[u].x, wh[u].x, wl[u].y, wh[u].y, x.x, x.y);
                    mma_bf16(acc[j], wl[u].z, wh[u].z, wl[u].w, wh[u].w, x.z, x.w);
                }
            }
        }
    }
    // What this thread will add to, requested now: the reads return while the partial sums are
    // exchanged (read one by one between the stores below, each would wait a round trip to L2).
    constexpr int OUT_STEP = WARPS * 32 / ROWS;                 // tokens a pass of the block covers
    float old_c[8 * NT / OUT_STEP > 0 ? 8 * NT / OUT_STEP : 1];
    if (mode == MODE_ACCUMULATE) {
        if (chunks <= warp) pdl_wait();
        const int i = threadIdx.x % ROWS;
#pragma unroll
        for (int it = 0; it < (int)(sizeof(old_c) / sizeof(float)); ++it) {
            const int tok = threadIdx.x / ROWS + it * OUT_STEP;
            old_c[it] = tok < m && n0 + i < n ? __ldcg(c + (size_t)tok * ldc + n0 + i) : 0.0f;
        }
    }
    // acc[j]: [0],[1] = W row g, tokens 8j + 2tq (+1); [2],[3] = W row g + 8
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        part[warp][g][j * 8 + tq * 2] = acc[j][0];
        part[warp][g][j * 8 + tq * 2 + 1] = acc[j][1];
        if (ROWS == 16) {
            part[warp][g + 8][j * 8 + tq * 2] = acc[j][2];
            part[warp][g + 8][j * 8 + tq * 2 + 1] = acc[j][3];
        }
    }
    if (chunks <= warp) pdl_wait();                   // a warp without chunks still orders its writes
    __syncthreads();
    if (mode == MODE_SWIGLU) {
        if (ROWS == 16) {
            const int i = threadIdx.x & 7;                      // gate row i, up row i + 8
            const int col = blockIdx.x * 8 + i;
            for (int tok = threadIdx.x >> 3; tok < m; tok += WARPS * 4) {
                float gate = 0.0f, up = 0.0f;
#pragma unroll
                for (int wp = 0; wp < WARPS; ++wp) {
                    gate += part[wp][i][tok];
                    up += part[wp][(i + 8) % ROWS][tok];
                }
                if (n0 + i + 8 < n)
                    out_act[(size_t)tok * ld_act + col] =
                        __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
            }
        }
    } else {
        const int i = threadIdx.x % ROWS;
#pragma unroll
        for (int it = 0; it < (int)(sizeof(old_c) / sizeof(float)); ++it) {
            const int tok = threadIdx.x / ROWS + it * OUT_STEP;
            if (tok >= m) break;
            float sum = 0.0f;
#pragma unroll
            for (int wp = 0; wp < WARPS; ++wp) sum += part[wp][i][tok];
            if (n0 + i < n) c[(size_t)tok * ldc + n0 + i] = mode == MODE_ACCUMULATE ? old_c[it] + sum : sum;
        }
    }
}

}  // namespace

extern "C" int ti_gemm_skinny_supported(int m, int n, int k, int lda, int ldw) {
    return m >= 1 && m <= 64 && n >= 1 && k >= CHUNK && k % CHUNK == 0 && lda % 8 == 0 && ldw % 8 == 0;
}

// mode 0: c = a w^T; 1: c += a w^T; 2: out_act[m, n/2] = swiglu over strips of 8 gate + 8 up rows.
extern "C" int ti_gemm_skinny(const void* a, const void* w, float* c, void* out_act, int m, int n,
                              int k, int lda, int ldw, int ldc, int ld_act, int mode, void* stream) {
    if (m == 0 || n == 0) return 0;
    TI_REQUIRE(ti_gemm_skinny_supported(m, n, k, lda, ldw),
               "gemm_skinny: M=%d (1..64), K=%d (multiple of 32) or row strides %d, %d (multiples of 8) "
               "are not supported", m, k, lda, ldw);
    TI_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0),
               "gemm_skinny: operands must be 16-byte aligned");
    TI_REQUIRE(mode != MODE_SWIGLU || n % 16 == 0, "gemm_skinny: SwiGLU needs N %% 16 == 0, got %d", n);
    cudaStream_t s = (cudaStream_t)stream;
    // narrow outputs get blocks of 8 rows, so that at least about 128 blocks share the reading
    const bool narrow = mode != MODE_SWIGLU && (n + STRIP - 1) / STRIP < 128;
#define LAUNCH(NT)                                                                                  \
    if (narrow)                                                                                     \
        ti_launch_pdl(gemm_skinny_kernel<NT, 8, 8>, (unsigned)((n + 7) / 8), WARPS * 32, 0, s,      \
                      (const bf16*)a, (const bf16*)w, c, (bf16*)out_act, m, n, k, lda, ldw, ldc,    \
                      ld_act, mode);                                                                \
    else if (k <= SHORT_K && mode == MODE_STORE && NT <= 2)                                         \
        ti_launch_pdl((gemm_skinny_kernel<NT <= 2 ? NT : 1, 16, 4, true>), (unsigned)((n + STRIP - 1) / STRIP), \
                      WARPS * 32, 0, s, (const bf16*)a, (const bf16*)w, c, (bf16*)out_act, m, n, k, \
                      lda, ldw, ldc, ld_act, mode);                                                 \
    else if (k <= SHORT_K)                                                                          \
        ti_launch_pdl(gemm_skinny_kernel<NT, 16, 4>, (unsigned)((n + STRIP - 1) / STRIP),           \
                      WARPS * 32, 0, s, (const bf16*)a, (const bf16*)w, c, (bf16*)out_act, m, n, k, \
                      lda, ldw, ldc, ld_act, mode);                                                 \
    else                                                                                            \
        ti_launch_pdl(gemm_skinny_kernel<NT, 16, 8>, (unsigned)((n + STRIP - 1) / STRIP),           \
                      WARPS * 32, 0, s, (const bf16*)a, (const bf16*)w, c, (bf16*)out_act, m, n, k, \
                      lda, ldw, ldc, ld_act, mode)
    if (m <= 8) { LAUNCH(1); }
    else if (m <= 16) { LAUNCH(2); }
    else if (m <= 32) { LAUNCH(4); }
    else { LAUNCH(8); }
#undef LAUNCH
    return ti_check_launch("gemm_skinny");
}
