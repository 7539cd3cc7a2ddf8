// Paged flash attention for prompt portions (bfloat16, head_dim a multiple of 16 up to 128).
//
// A block takes 64 consecutive query tokens of one request and one query head (4 warps x 16
// rows).  It walks the request's keys in tiles of 64, from the first key any of its rows may see
// (0, or the window's edge) to its last row's own position: keys that earlier steps left in the
// pages and the keys of this portion alike, since the portion's keys are stored before this
// kernel runs.  Tiles come through a two-stage cp.async ring; scores and the product with the
// values run on the tensor cores (mma.sync m16n8k16), the softmax is online and float32.
// The causal and window masks are applied only in tiles that touch an edge.
#include "common.cuh"

namespace {

constexpr int BM = 64;         // query rows per block (must match the host's tile list)
constexpr int BN = 64;         // keys per tile
constexpr int STAGES = 2;
constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
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
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// tiles[i] = {request row, first flat token, number of query rows (<= 64)}
template <int HD>
__global__ void __launch_bounds__(WARPS * 32, HD > 64 ? 3 : 4)
attn_prefill_kernel(const bf16* __restrict__ q, const int* __restrict__ tiles,
                    const int* __restrict__ positions, const int* __restrict__ block_table,
                    int bt_stride, const bf16* __restrict__ pages, int num_pages, int page_size,
                    int num_heads, int num_kv_heads, int window, float scale_log2,
                    bf16* __restrict__ out, int* __restrict__ status) {
    constexpr int ROW_BYTES = HD * 2 + 16;
    constexpr int CHUNKS = HD / 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;
    constexpr int STAGE_BYTES = 2 * BN * ROW_BYTES;
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    // heads run fastest in the grid, tiles are sorted by length: blocks start longest first
    const int h = blockIdx.x, tile_id = blockIdx.y;
    const int kvh = h / (num_heads / num_kv_heads);
    const int req = tiles[tile_id * 3], tok0 = tiles[tile_id * 3 + 1];
    const int nrows = tiles[tile_id * 3 + 2];
    const int* table = block_table + (size_t)req * bt_stride;
    const size_t kv_stride = (size_t)num_kv_heads * page_size * HD;

    const int pos_first = positions[tok0], pos_last = pos_first + nrows - 1;
    const int kv_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int kt_lo = kv_lo / BN, kt_hi = pos_last / BN + 1;

    // this thread's two rows: warp * 16 + g and + 8; a row past the tile sees nothing
    int row_pos[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = warp * 16 + g + 8 * r;
        row_pos[r] = i < nrows ? pos_first + i : -1;
    }
    const int warp_pos_lo = pos_first + warp * 16;                       // first row of the warp
    const int warp_pos_hi = min(pos_last, pos_first + warp * 16 + 15);   // its last real row

    unsigned qa[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const int k0 = ks * 16 + tq * 2;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int i = warp * 16 + g + 8 * r;
            const bf16* qp = q + ((size_t)(tok0 + i) * num_heads + h) * HD + k0;
            qa[ks][r] = i < nrows ? *reinterpret_cast<const unsigned*>(qp) : 0u;
            qa[ks][r + 2] = i < nrows ? *reinterpret_cast<const unsigned*>(qp + 8) : 0u;
        }
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    auto issue = [&](int kt, int stage) {
        unsigned char* kdst = smem + (size_t)stage * STAGE_BYTES;
        unsigned char* vdst = kdst + BN * ROW_BYTES;
        // four runs of 16 keys; a run is contiguous inside its page
#pragma unroll
        for (int r = 0; r < BN / 16; ++r) {
            const int key0 = kt * BN + r * 16;
            int pg = -1;
            if (key0 <= pos_last && key0 + 16 > kv_lo) {
                pg = table[key0 / page_size];
                if (pg < 0 || pg >= num_pages) {
                    if (threadIdx.x == 0) atomicCAS(status, 0, 1);
                    pg = -1;
                }
            }
            const bool valid = pg >= 0;
            const bf16* ksrc = pages;
            if (valid)
                ksrc = pages + (((size_t)pg * 2 * num_kv_heads + kvh) * page_size + key0 % page_size) * HD;
            const bf16* vsrc = valid ? ksrc + kv_stride : pages;
            for (int c = threadIdx.x; c < 16 * CHUNKS; c += WARPS * 32) {
                const int off = (r * 16 + c / CHUNKS) * ROW_BYTES + (c % CHUNKS) * 16;
                cp_async16(kdst + off, ksrc + (valid ? c * 8 : 0), valid);
                cp_async16(vdst + off, vsrc + (valid ? c * 8 : 0), valid);
            }
        }
    };

    issue(kt_lo, 0);
    cp_async_commit();
    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int stage = (kt - kt_lo) % STAGES;
        if (kt + 1 < kt_hi) issue(kt + 1, (kt + 1 - kt_lo) % STAGES);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key_lo = kt * BN, key_hi = key_lo + BN - 1;
        // the warp skips tiles none of its rows can see
        const bool visible = key_lo <= warp_pos_hi &&
                             (window <= 0 || key_hi > warp_pos_lo - window);
        if (visible) {
            const unsigned char* ks = smem + (size_t)stage * STAGE_BYTES;
            const unsigned char* vs = ks + BN * ROW_BYTES;
            float s_acc[BN / 8][4];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int jp = 0; jp < BN / 16; ++jp) {
                    unsigned b[4];
                    const int key = jp * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, ks + key * ROW_BYTES + dim * 2);
                    mma_bf16(s_acc[2 * jp], qa[kk], b[0], b[1]);
                    mma_bf16(s_acc[2 * jp + 1], qa[kk], b[2], b[3]);
                }
            }
            const bool edge = key_hi > warp_pos_lo ||
                              (window > 0 && key_lo <= warp_pos_hi - window);
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s_acc[j][e] * scale_log2;
                    if (edge) {
                        const int key = key_lo + j * 8 + tq * 2 + (e & 1);
                        const int p = row_pos[e >> 1];
                        if (key > p || (window > 0 && key <= p - window)) v = -INFINITY;
                    }
                    s_acc[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
            float alpha[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                alpha[r] = m_new == -INFINITY ? 1.0f : exp2f(m_run[r] - m_new);
                m_run[r] = m_new;
                m_use[r] = m_new == -INFINITY ? 0.0f : m_new;     // a row that sees nothing yet
            }
            float sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2f(s_acc[j][e] - m_use[e >> 1]);
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
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                unsigned pa[4];
                pa[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
                pa[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
                pa[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
                pa[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < NT_O / 2; ++dp) {
                    unsigned b[4];
                    const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int dim = dp * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b, vs + key * ROW_BYTES + dim * 2);
                    mma_bf16(o[2 * dp], pa, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();                              // the stage may be refilled
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = warp * 16 + g + 8 * r;
        if (i >= nrows) continue;
        const float inv = 1.0f / l_run[r];
        bf16* op = out + ((size_t)(tok0 + i) * num_heads + h) * HD + tq * 2;
#pragma unroll
        for (int t = 0; t < NT_O; ++t) {
            *reinterpret_cast<__nv_bfloat162*>(op + t * 8) =
                __floats2bfloat162_rn(o[t][2 * r] * inv, o[t][2 * r + 1] * inv);
        }
    }
}

template <int HD>
int launch_prefill(const bf16* q, const int* tiles, int num_tiles, const int* positions,
                   const int* block_table, int bt_stride, const bf16* pages, int num_pages,
                   int page_size, int num_heads, int num_kv_heads, int window, float scale,
                   bf16* out, int* status, cudaStream_t s) {
    constexpr int SMEM = STAGES * 2 * BN * (HD * 2 + 16);
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return ti_fail("attn_prefill: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid(num_heads, num_tiles);
    attn_prefill_kernel<HD><<<grid, WARPS * 32, SMEM, s>>>(q, tiles, positions, block_table, bt_stride,
                                                          pages, num_pages, page_size, num_heads,
                                                          num_kv_heads, window, scale * LOG2E, out,
                                                          status);
    return ti_check_launch("attn_prefill");
}

}  // namespace

extern "C" int ti_attn_prefill_tile_rows() { return BM; }

extern "C" int ti_attn_prefill_supported(int head_dim, int page_size) {
    return head_dim >= 16 && head_dim <= 128 && head_dim % 16 == 0 && page_size >= 16 &&
           page_size % 16 == 0;
}

// tiles: int32 [num_tiles, 3] = {request row, first flat token, query rows}; rows of a tile are
// consecutive tokens of one request.
extern "C" int ti_attn_prefill(const void* q, const int* tiles, int num_tiles, const int* positions,
                               const int* block_table, int bt_stride, const void* pages,
                               int num_pages, int page_size, int num_heads, int num_kv_heads,
                               int head_dim, int window, float scale, void* out, int* status,
                               void* stream) {
    if (num_tiles == 0) return 0;
    TI_REQUIRE(num_heads % num_kv_heads == 0, "attn_prefill: %d heads over %d kv heads", num_heads,
               num_kv_heads);
    TI_REQUIRE(ti_attn_prefill_supported(head_dim, page_size),
               "attn_prefill: head_dim %d (multiple of 16 up to 128) or page size %d (multiple of 16) "
               "is not supported", head_dim, page_size);
    TI_REQUIRE(num_tiles <= 65535, "attn_prefill: %d tiles exceed the grid limit", num_tiles);
#define CASE(HD)                                                                                     \
    case HD:                                                                                         \
        return launch_prefill<HD>((const bf16*)q, tiles, num_tiles, positions, block_table, bt_stride, \
                                  (const bf16*)pages, num_pages, page_size, num_heads, num_kv_heads, \
                                  window, scale, (bf16*)out, status, (cudaStream_t)stream)
    switch (head_dim) {
        CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
    }
#undef CASE
    return ti_fail("attn_prefill: head_dim %d", head_dim);
}
