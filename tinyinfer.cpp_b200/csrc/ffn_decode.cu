// SwiGLU feed-forward of a decode step in one launch, for models whose feed-forward weights of
// one layer fit into the shared memory of the whole GPU:
//     act = silu(x Wgate^T) * (x Wup^T)  (bfloat16),   C += act Wdown^T  (float32 residual).
//
// Why: as separate launches the down projection's blocks cannot become resident, and so cannot
// ask for their weights, before the gate/up blocks have left, and the step then waits for two
// rounds of weights from HBM behind that boundary.  Here one block per SM copies all weight rows
// it will need (its strips of gate/up rows and its strip of down rows) into shared memory with
// bulk copies BEFORE it waits for the kernel before it, so the copy runs while the attention's tail,
// the output projection and the norm still execute.  After the wait only activations move: x from
// L2, the SwiGLU outputs to L2 and back.
//
// Arithmetic and its order are those of gemm_skinny.cu (mma.sync m16n8k16, the 8 warps take the
// 32-element chunks of K in turn, the warps' partial sums are added in warp order), so the result
// has the same bits as the two launches it replaces.
//
// Between the two products all blocks meet once: every block adds one to a 64-bit counter when
// its SwiGLU outputs are written (fence, then atomic), and a block with down rows polls the
// counter with acquire loads until all blocks of this launch have arrived.  The counter is never
// reset (a reset would put one more round trip to L2 on the step's critical path): a launch waits
// for the next multiple of the grid size.  The wait is bounded; when it runs out the block
// records status 2 and returns.  All blocks are resident at once by construction: the grid has
// one block per SM, and a block's shared memory admits one block per SM.  (Two launches of this
// kernel that run at the same time on different streams could each hold a part of the SMs and
// wait for the rest; their waits then run out and both report status 2.  An engine launches on
// one stream; who steps several engines concurrently on one GPU turns this kernel off.)
#include "sm100.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int CHUNK = 32;
constexpr int PAD = 64;                 // bytes after each weight row in shared memory: a quarter
                                        // warp's 16-byte reads of two rows then cover all 32 banks
constexpr int SMEM_LIMIT = 227 * 1024 - 1024;
enum { TI_ERR_TIMEOUT = 2 };

// One row of weights into shared memory as a bulk copy (no multicast) that reports its bytes to
// an mbarrier.  Both addresses are 16-byte aligned and the size is a multiple of 16.
__device__ __forceinline__ void bulk_row(void* dst, const void* src, unsigned bytes, void* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(sm100::smem_u32(dst)), "l"(src), "r"(bytes), "r"(sm100::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Args {
    // the front (optional): residual += attn w_o^T, then x = rmsnorm(residual) * norm_w
    const bf16* attn; const bf16* w_o; const float* norm_w; float eps; int nq, ld_attn, ld_o;
    // the feed-forward
    const bf16* x; const bf16* w_gu; const bf16* w_dn; bf16* act; float* c;
    int m, hidden, inter, ldx, ld_gu, ld_dn, ld_act, ldc;
    unsigned long long* counters;       // [0]: after the front's product, [1]: after SwiGLU
    int* status;
};

struct Layout {
    int gu_strips, dn_strips;           // strips of 16 gate/up rows (8 + 8) and of 8 down (and O) rows
    int max_gu, max_dn;                 // the most a block owns
    int gu_row, dn_row, o_row;          // bytes of a weight row in shared memory
    int part_floats;                    // per strip: [WARPS][16][MP + 1]
    long long o_bytes, scratch_bytes, bytes;
};

__host__ __device__ inline Layout make_layout(int hidden, int inter, int nq, int blocks, int mp, bool front) {
    Layout l;
    l.gu_strips = inter / 8;
    l.dn_strips = hidden / 8;
    l.max_gu = (l.gu_strips + blocks - 1) / blocks;
    l.max_dn = (l.dn_strips + blocks - 1) / blocks;
    l.gu_row = hidden * 2 + PAD;
    l.dn_row = inter * 2 + PAD;
    l.o_row = nq * 2 + PAD;
    l.part_floats = WARPS * 16 * (mp + 1);
    const int part_strips = l.max_gu > l.max_dn ? l.max_gu : l.max_dn;
    l.scratch_bytes = (long long)part_strips * l.part_floats * 4;
    const long long norm_bytes = front ? (long long)(mp * 256 + mp) * 4 : 0;   // sums of squares, factors
    if (norm_bytes > l.scratch_bytes) l.scratch_bytes = norm_bytes;
    l.o_bytes = front ? (long long)l.max_dn * 8 * l.o_row : 0;
    l.bytes = (long long)l.max_gu * 16 * l.gu_row + (long long)l.max_dn * 8 * l.dn_row + l.o_bytes +
              l.scratch_bytes;
    return l;
}

// Thread 0 of a block: arrive at the counter (everything the block wrote before the barrier in
// front of this call is visible to who sees the arrival) and, if `wait`, poll until all blocks
// of this launch have arrived.  `before`: the counter as read before this block arrived.
__device__ __forceinline__ bool arrive_and_wait(unsigned long long* counter, unsigned long long before,
                                                int blocks, bool wait, int* status) {
    __threadfence();
    atomicAdd(counter, 1ull);
    if (!wait) return true;
    const unsigned long long target = (before / (unsigned)blocks + 1ull) * (unsigned)blocks;
    const unsigned long long start = global_timer();
    unsigned polls = 0;
    while (ld_acquire(counter) < target) {
        if ((++polls & 255u) == 0 && global_timer() - start > 1000000000ull) {   // one second
            atomicCAS(status, 0, TI_ERR_TIMEOUT);
            return false;
        }
    }
    return true;
}

// The partial sums of one strip of 8 weight rows (rows `g` of the MMA's A operand, its upper half
// zero) against the tokens' rows `a_row`, chunks of K taken by the warps in turn.
template <int NT, int XB, bool THROUGH_L2>
__device__ __forceinline__ void strip8(const unsigned char* w_lo, const bf16* const (&a_row)[NT], int chunks,
                                       int warp, float (&acc)[NT][4]) {
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    for (int c0 = warp; c0 < chunks; c0 += WARPS * XB) {
        uint4 xr[XB][NT];
#pragma unroll
        for (int u = 0; u < XB; ++u) {
            const int ch = c0 + u * WARPS;
            if (ch < chunks) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint4* src = reinterpret_cast<const uint4*>(a_row[j] + (size_t)ch * CHUNK);
                    xr[u][j] = THROUGH_L2 ? __ldcg(src) : *src;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < XB; ++u) {
            const int ch = c0 + u * WARPS;
            if (ch >= chunks) break;
            const uint4 wl = *reinterpret_cast<const uint4*>(w_lo + (size_t)ch * (CHUNK * 2));
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                mma_bf16(acc[j], wl.x, 0u, wl.y, 0u, xr[u][j].x, xr[u][j].y);
                mma_bf16(acc[j], wl.z, 0u, wl.w, 0u, xr[u][j].z, xr[u][j].w);
            }
        }
    }
}

// NT: token columns of 8 (M <= 8 NT).  XB: chunks of activations a warp requests at once in the
// products with 8-row strips.  FRONT: the output projection and the norm run here too.
template <int NT, int XB, bool FRONT>
__global__ void __launch_bounds__(THREADS, 1) ffn_decode_kernel(const Args p) {
    constexpr int MP = NT * 8;
    constexpr int XU = 4;                       // chunks of x per warp: hidden <= 1,024 with FRONT
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int blocks = gridDim.x, b = blockIdx.x;
    const int m = p.m, hidden = p.hidden, inter = p.inter;
    const Layout l = make_layout(hidden, inter, p.nq, blocks, MP, FRONT);
    unsigned char* gu_smem = smem;
    unsigned char* dn_smem = gu_smem + (size_t)l.max_gu * 16 * l.gu_row;
    unsigned char* o_smem = dn_smem + (size_t)l.max_dn * 8 * l.dn_row;
    float* part = reinterpret_cast<float*>(o_smem + l.o_bytes);
    // gate/up strips b, b + blocks, ...; down strips from the other end of the grid, so that the
    // blocks with one gate/up strip fewer take the down strips first; O strips like down strips
    const int my_gu = b < l.gu_strips ? (l.gu_strips - 1 - b) / blocks + 1 : 0;
    const int d0 = blocks - 1 - b;
    const int my_dn = d0 < l.dn_strips ? (l.dn_strips - 1 - d0) / blocks + 1 : 0;

    pdl_launch();
    // ---- all weights of this block, requested before anything else is known -------------------
    // Row by row as bulk copies issued by the lanes of warp 0 (a few dozen instructions in all: a
    // block that starts late, when the attention before it has only just left its SM, has its
    // first rows within a microsecond).  One mbarrier per group: O rows, gate/up rows, down rows.
    __shared__ __align__(8) unsigned long long bars[3];
    if (tid == 0) {
        for (int i = 0; i < 3; ++i) sm100::mbar_init(&bars[i], 1);
        sm100::mbar_fence_init();
    }
    __syncthreads();
    if (warp == 0) {
        const unsigned o_bytes = (unsigned)p.nq * 2, gu_bytes = (unsigned)hidden * 2, dn_bytes = (unsigned)inter * 2;
        if (lane == 0) {
            sm100::mbar_expect_tx(&bars[0], FRONT ? (unsigned)my_dn * 8 * o_bytes : 0u);
            sm100::mbar_expect_tx(&bars[1], (unsigned)my_gu * 16 * gu_bytes);
            sm100::mbar_expect_tx(&bars[2], (unsigned)my_dn * 8 * dn_bytes);
        }
        __syncwarp();
        if (FRONT) {
            for (int i = lane; i < my_dn * 8; i += 32)
                bulk_row(o_smem + (size_t)i * l.o_row,
                         p.w_o + ((size_t)(d0 + (i >> 3) * blocks) * 8 + (i & 7)) * p.ld_o, o_bytes, &bars[0]);
        }
        for (int i = lane; i < my_gu * 16; i += 32)
            bulk_row(gu_smem + (size_t)i * l.gu_row,
                     p.w_gu + ((size_t)(b + (i >> 4) * blocks) * 16 + (i & 15)) * p.ld_gu, gu_bytes, &bars[1]);
        for (int i = lane; i < my_dn * 8; i += 32)
            bulk_row(dn_smem + (size_t)i * l.dn_row,
                     p.w_dn + ((size_t)(d0 + (i >> 3) * blocks) * 8 + (i & 7)) * p.ld_dn, dn_bytes, &bars[2]);
    }
    pdl_wait();                            // activations, residual and counters belong to the chain
    // The counters only grow: launch after launch adds one per block.  What one holds now, before
    // this block has arrived, tells the round (not all blocks of this launch can have arrived
    // yet), and with it the count to wait for.  The latency hides behind the first product.
    unsigned long long before_a = 0, before_b = 0;
    if (tid == 0) {
        if (FRONT) before_a = ld_relaxed(p.counters);
        before_b = ld_relaxed(p.counters + 1);
    }
    __shared__ int proceed;
    const int out_i = tid & 7, out_tok = tid >> 3;              // 32 tokens' worth of threads >= MP
    // the residual values this thread will add to, requested before the products
    float old_c[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        old_c[s] = 0.0f;
        if (s < my_dn && out_tok < m)
            old_c[s] = __ldcg(p.c + (size_t)out_tok * p.ldc + (d0 + s * blocks) * 8 + out_i);
    }

    // the norm's weights at the columns whose activations this thread will hold (asked for after
    // the wait: the wait does not return while loads of this block are outstanding)
    float gw[XU][8];
    if (FRONT) {
#pragma unroll
        for (int u = 0; u < XU; ++u) {
            const int ch = warp + u * WARPS;
            if (ch * CHUNK < hidden) {
                const float4 lo = *reinterpret_cast<const float4*>(p.norm_w + ch * CHUNK + tq * 8);
                const float4 hi = *reinterpret_cast<const float4*>(p.norm_w + ch * CHUNK + tq * 8 + 4);
                gw[u][0] = lo.x; gw[u][1] = lo.y; gw[u][2] = lo.z; gw[u][3] = lo.w;
                gw[u][4] = hi.x; gw[u][5] = hi.y; gw[u][6] = hi.z; gw[u][7] = hi.w;
            }
        }
    }
    uint4 xn[XU][NT];                      // FRONT: the normed activations, as the MMA's B fragments
    if (FRONT) {
        // ---- output projection into the residual ---------------------------------------------
        const bf16* a_row[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) a_row[j] = p.attn + (size_t)min(j * 8 + g, m - 1) * p.ld_attn + tq * 8;
        bool landed = sm100::mbar_wait(&bars[0], 0);
        for (int s = 0; s < my_dn; ++s) {
            float acc[NT][4];
            strip8<NT, XB, false>(o_smem + (size_t)(s * 8 + g) * l.o_row + tq * 16, a_row, p.nq / CHUNK, warp, acc);
            if (s > 0) __syncthreads();
            float* ps = part + (size_t)warp * 16 * (MP + 1);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                ps[g * (MP + 1) + j * 8 + tq * 2] = acc[j][0];
                ps[g * (MP + 1) + j * 8 + tq * 2 + 1] = acc[j][1];
            }
            __syncthreads();
            if (out_tok < m) {
                float sum = 0.0f;
#pragma unroll
                for (int wp = 0; wp < WARPS; ++wp) sum += part[(wp * 16 + out_i) * (MP + 1) + out_tok];
                float old = old_c[0];
                if (s == 1) old = old_c[1];
                if (s == 2) old = old_c[2];
                if (s == 3) old = old_c[3];
                p.c[(size_t)out_tok * p.ldc + (d0 + s * blocks) * 8 + out_i] = old + sum;
            }
        }
        __syncthreads();
        if (tid == 0) proceed = arrive_and_wait(p.counters, before_a, blocks, true, p.status) && landed;
        __syncthreads();
        if (!proceed) {                    // leave only when no copy into this block is in flight
            if (!(sm100::mbar_wait(&bars[1], 0) && sm100::mbar_wait(&bars[2], 0) && landed))
                atomicCAS(p.status, 0, TI_ERR_TIMEOUT);
            return;
        }
        // ---- the norm of the residual rows, in the order of the block-per-row kernel -----------
        // (rowwise.cu: thread t of 256 adds the squares of elements 4t .. 4t+3 with fused
        // multiply-adds, a butterfly over the 32 lanes of each warp, then over the 8 warps' sums)
        float* ssbuf = part;               // [MP][256]
        float* inv_s = part + MP * 256;    // [MP]
        float rv[XU][NT][8];
#pragma unroll
        for (int u = 0; u < XU; ++u) {
            const int ch = warp + u * WARPS;
            if (ch * CHUNK < hidden) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const float* src = p.c + (size_t)min(j * 8 + g, m - 1) * p.ldc + ch * CHUNK + tq * 8;
                    const float4 lo = __ldcg(reinterpret_cast<const float4*>(src));
                    const float4 hi = __ldcg(reinterpret_cast<const float4*>(src + 4));
                    rv[u][j][0] = lo.x; rv[u][j][1] = lo.y; rv[u][j][2] = lo.z; rv[u][j][3] = lo.w;
                    rv[u][j][4] = hi.x; rv[u][j][5] = hi.y; rv[u][j][6] = hi.z; rv[u][j][7] = hi.w;
                }
            }
        }
#pragma unroll
        for (int s = 0; s < 4; ++s)        // what the down projection will add to (the O product changed it)
            if (s < my_dn && out_tok < m)
                old_c[s] = __ldcg(p.c + (size_t)out_tok * p.ldc + (d0 + s * blocks) * 8 + out_i);
#pragma unroll
        for (int u = 0; u < XU; ++u) {
            const int ch = warp + u * WARPS;
            if (ch * CHUNK < hidden) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    if (j * 8 + g < m) {
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            float ss = 0.0f;
#pragma unroll
                            for (int e = 0; e < 4; ++e) ss = fmaf(rv[u][j][half * 4 + e], rv[u][j][half * 4 + e], ss);
                            ssbuf[(j * 8 + g) * 256 + ch * 8 + tq * 2 + half] = ss;
                        }
                    }
                }
            }
        }
        __syncthreads();
        const int n4 = hidden / 4;
        for (int row = warp; row < m; row += WARPS) {
            float r = 0.0f;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                const int idx = v * 32 + lane;
                const float tot = warp_sum(idx < n4 ? ssbuf[row * 256 + idx] : 0.0f);
                if (lane == v) r = tot;
            }
            const float total = warp_sum(r);
            if (lane == 0) inv_s[row] = 1.0f / sqrtf(total / (float)hidden + p.eps);
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < XU; ++u) {
            const int ch = warp + u * WARPS;
            if (ch * CHUNK < hidden) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const float inv = inv_s[min(j * 8 + g, m - 1)];
                    unsigned pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(rv[u][j][2 * e] * inv * gw[u][2 * e],
                                                                  rv[u][j][2 * e + 1] * inv * gw[u][2 * e + 1]);
                        pk[e] = *reinterpret_cast<unsigned*>(&h2);
                    }
                    xn[u][j] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
        }
        __syncthreads();                   // the scratch is free for the partial sums
    }

    // ---- gate/up and SwiGLU --------------------------------------------------------------------
    const bf16* x_row[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j)
        x_row[j] = FRONT ? nullptr : p.x + (size_t)min(j * 8 + g, m - 1) * p.ldx + tq * 8;
    const bool gu_landed = sm100::mbar_wait(&bars[1], 0);
    {
        const int chunks = hidden / CHUNK;
        for (int s = 0; s < my_gu; ++s) {
            const unsigned char* w_lo = gu_smem + (size_t)(s * 16 + g) * l.gu_row + tq * 16;
            const unsigned char* w_hi = w_lo + (size_t)8 * l.gu_row;
            float acc[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
            for (int c0 = warp; c0 < chunks; c0 += WARPS * XU) {
                uint4 xr[XU][NT];
#pragma unroll
                for (int u = 0; u < XU; ++u) {
                    const int ch = c0 + u * WARPS;
                    if (ch < chunks) {
#pragma unroll
                        for (int j = 0; j < NT; ++j)
                            xr[u][j] = FRONT ? xn[u][j]
                                             : *reinterpret_cast<const uint4*>(x_row[j] + (size_t)ch * CHUNK);
                    }
                }
#pragma unroll
                for (int u = 0; u < XU; ++u) {
                    const int ch = c0 + u * WARPS;
                    if (ch >= chunks) break;
                    const uint4 wl = *reinterpret_cast<const uint4*>(w_lo + (size_t)ch * (CHUNK * 2));
                    const uint4 wh = *reinterpret_cast<const uint4*>(w_hi + (size_t)ch * (CHUNK * 2));
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        mma_bf16(acc[j], wl.x, wh.x, wl.y, wh.y, xr[u][j].x, xr[u][j].y);
                        mma_bf16(acc[j], wl.z, wh.z, wl.w, wh.w, xr[u][j].z, xr[u][j].w);
                    }
                }
            }
            float* ps = part + (size_t)s * l.part_floats + (size_t)warp * 16 * (MP + 1);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                ps[g * (MP + 1) + j * 8 + tq * 2] = acc[j][0];
                ps[g * (MP + 1) + j * 8 + tq * 2 + 1] = acc[j][1];
                ps[(g + 8) * (MP + 1) + j * 8 + tq * 2] = acc[j][2];
                ps[(g + 8) * (MP + 1) + j * 8 + tq * 2 + 1] = acc[j][3];
            }
        }
        __syncthreads();
        for (int s = 0; s < my_gu; ++s) {
            const float* ps = part + (size_t)s * l.part_floats;
            const int col = (b + s * blocks) * 8 + out_i;               // gate row i, up row i + 8
            for (int tok = out_tok; tok < m; tok += THREADS / 8) {
                float gate = 0.0f, up = 0.0f;
#pragma unroll
                for (int wp = 0; wp < WARPS; ++wp) {
                    gate += ps[(wp * 16 + out_i) * (MP + 1) + tok];
                    up += ps[(wp * 16 + out_i + 8) * (MP + 1) + tok];
                }
                p.act[(size_t)tok * p.ld_act + col] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
            }
        }
    }
    // ---- every block's outputs are written: arrive, and wait if there are down rows to do -------
    __syncthreads();
    if (tid == 0) proceed = arrive_and_wait(p.counters + 1, before_b, blocks, my_dn > 0, p.status);
    const bool dn_landed = sm100::mbar_wait(&bars[2], 0);
    __syncthreads();
    if (!(gu_landed && dn_landed)) atomicCAS(p.status, 0, TI_ERR_TIMEOUT);
    if (!proceed || my_dn == 0) return;

    // ---- down projection into the residual ---------------------------------------------------
    const bf16* a_row[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) a_row[j] = p.act + (size_t)min(j * 8 + g, m - 1) * p.ld_act + tq * 8;
    for (int s = 0; s < my_dn; ++s) {
        float acc[NT][4];
        strip8<NT, XB, true>(dn_smem + (size_t)(s * 8 + g) * l.dn_row + tq * 16, a_row, inter / CHUNK, warp, acc);
        if (s > 0) __syncthreads();                 // the sums of the strip before have been read
        float* ps = part + (size_t)warp * 16 * (MP + 1);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            ps[g * (MP + 1) + j * 8 + tq * 2] = acc[j][0];
            ps[g * (MP + 1) + j * 8 + tq * 2 + 1] = acc[j][1];
        }
        __syncthreads();
        if (out_tok < m) {
            float sum = 0.0f;
#pragma unroll
            for (int wp = 0; wp < WARPS; ++wp) sum += part[(wp * 16 + out_i) * (MP + 1) + out_tok];
            float old = old_c[0];                   // (a block owns at most four down strips)
            if (s == 1) old = old_c[1];
            if (s == 2) old = old_c[2];
            if (s == 3) old = old_c[3];
            p.c[(size_t)out_tok * p.ldc + (d0 + s * blocks) * 8 + out_i] = old + sum;
        }
    }
}

int num_sms() {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 0;
    if (sms[dev] == 0) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev];
}

bool sizes_ok(int m, int hidden, int inter, int nq, bool front) {
    const int sms = num_sms();
    if (sms <= 0 || m < 1 || m > 16 || hidden < CHUNK || inter < CHUNK || hidden % CHUNK || inter % CHUNK) return false;
    if (front && (nq < CHUNK || nq % CHUNK || hidden > 1024)) return false;
    const Layout l = make_layout(hidden, inter, nq, sms, m <= 8 ? 8 : 16, front);
    return l.bytes <= SMEM_LIMIT && l.max_dn <= 4;
}

template <int NT, int XB, bool FRONT> int launch(const Args& a, cudaStream_t s) {
    const int sms = num_sms();
    const Layout l = make_layout(a.hidden, a.inter, a.nq, sms, NT * 8, FRONT);
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(ffn_decode_kernel<NT, XB, FRONT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        if (e != cudaSuccess) return ti_fail("ffn_decode: %s", cudaGetErrorString(e));
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ffn_decode_kernel<NT, XB, FRONT>, THREADS,
                                                          (size_t)l.bytes);
        if (e != cudaSuccess || per_sm < 1)
            return ti_fail("ffn_decode: a block of %lld bytes does not fit on an SM", l.bytes);
        configured.mark();
    }
    ti_launch_pdl(ffn_decode_kernel<NT, XB, FRONT>, dim3(sms), dim3(THREADS), (size_t)l.bytes, s, a);
    return ti_check_launch("ffn_decode");
}

}  // namespace

// Whether the fused kernel takes these sizes on this GPU: at most 16 rows, rows of whole chunks,
// and all weight strips of a block in its shared memory.
extern "C" int ti_ffn_decode_supported(int m, int hidden, int inter, int ldx, int ld_gu, int ld_dn,
                                       int ld_act, int ldc) {
    if (ldx % 8 || ld_gu % 8 || ld_dn % 8 || ld_act % 8 || ldc < hidden) return 0;
    return sizes_ok(m, hidden, inter, 0, false) ? 1 : 0;
}

// x: [m, hidden] bfloat16; w_gu: [2 inter, hidden] bfloat16 in strips of 8 gate rows followed by
// their 8 up rows; w_dn: [hidden, inter] bfloat16; act: [m, inter] bfloat16 scratch; c: [m, hidden]
// float32, added to.  counters: two 64-bit counters, 8-byte aligned, zero before the first call,
// used by no other grid size.
extern "C" int ti_ffn_decode(const void* x, const void* w_gu, const void* w_dn, void* act, float* c,
                             int m, int hidden, int inter, int ldx, int ld_gu, int ld_dn, int ld_act,
                             int ldc, unsigned long long* counters, int* status, void* stream) {
    if (m == 0) return 0;
    TI_REQUIRE(ti_ffn_decode_supported(m, hidden, inter, ldx, ld_gu, ld_dn, ld_act, ldc),
               "ffn_decode: M=%d (1..16), hidden %d, intermediate %d (multiples of 32 whose strips fit "
               "into shared memory) or the row strides are not supported", m, hidden, inter);
    TI_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w_gu % 16 == 0 && (uintptr_t)w_dn % 16 == 0 &&
               (uintptr_t)act % 16 == 0 && (uintptr_t)counters % 8 == 0,
               "ffn_decode: operands must be 16-byte aligned, the counters 8-byte");
    Args a = {};
    a.x = (const bf16*)x; a.w_gu = (const bf16*)w_gu; a.w_dn = (const bf16*)w_dn; a.act = (bf16*)act; a.c = c;
    a.m = m; a.hidden = hidden; a.inter = inter; a.ldx = ldx; a.ld_gu = ld_gu; a.ld_dn = ld_dn;
    a.ld_act = ld_act; a.ldc = ldc; a.counters = counters; a.status = status;
    return m <= 8 ? launch<1, 12, false>(a, (cudaStream_t)stream) : launch<2, 6, false>(a, (cudaStream_t)stream);
}

// The same with the front: c += attn w_o^T, then x = rmsnorm(c, norm_w, eps) (bfloat16, never
// written to memory), then the feed-forward of x into c.
extern "C" int ti_attn_out_ffn_decode_supported(int m, int hidden, int inter, int nq, int ld_attn, int ld_o,
                                                int ld_gu, int ld_dn, int ld_act, int ldc) {
    if (ld_attn % 8 || ld_o % 8 || ld_gu % 8 || ld_dn % 8 || ld_act % 8 || ldc < hidden || ldc % 4) return 0;
    return sizes_ok(m, hidden, inter, nq, true) ? 1 : 0;
}

extern "C" int ti_attn_out_ffn_decode(const void* attn, const void* w_o, const float* norm_w, float eps,
                                      const void* w_gu, const void* w_dn, void* act, float* c, int m, int hidden,
                                      int inter, int nq, int ld_attn, int ld_o, int ld_gu, int ld_dn, int ld_act,
                                      int ldc, unsigned long long* counters, int* status, void* stream) {
    if (m == 0) return 0;
    TI_REQUIRE(ti_attn_out_ffn_decode_supported(m, hidden, inter, nq, ld_attn, ld_o, ld_gu, ld_dn, ld_act, ldc),
               "attn_out_ffn_decode: M=%d (1..16), hidden %d (to 1,024), intermediate %d, attention width %d "
               "(multiples of 32 whose strips fit into shared memory) or the row strides are not supported",
               m, hidden, inter, nq);
    TI_REQUIRE((uintptr_t)attn % 16 == 0 && (uintptr_t)w_o % 16 == 0 && (uintptr_t)norm_w % 16 == 0 &&
               (uintptr_t)w_gu % 16 == 0 && (uintptr_t)w_dn % 16 == 0 && (uintptr_t)act % 16 == 0 &&
               (uintptr_t)c % 16 == 0 && (uintptr_t)counters % 8 == 0,
               "attn_out_ffn_decode: operands must be 16-byte aligned, the counters 8-byte");
    Args a = {};
    a.attn = (const bf16*)attn; a.w_o = (const bf16*)w_o; a.norm_w = norm_w; a.eps = eps; a.nq = nq;
    a.ld_attn = ld_attn; a.ld_o = ld_o;
    a.w_gu = (const bf16*)w_gu; a.w_dn = (const bf16*)w_dn; a.act = (bf16*)act; a.c = c;
    a.m = m; a.hidden = hidden; a.inter = inter; a.ld_gu = ld_gu; a.ld_dn = ld_dn;
    a.ld_act = ld_act; a.ldc = ldc; a.counters = counters; a.status = status;
    return m <= 8 ? launch<1, 12, true>(a, (cudaStream_t)stream) : launch<2, 6, true>(a, (cudaStream_t)stream);
}
