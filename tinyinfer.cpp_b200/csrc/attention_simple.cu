// Attention on the CUDA cores, for every head size and both cache types.
//
//  * qk_norm_rope_store: per-head RMSNorm of q and k, NeoX rotation at the token's position,
//    k and v written once per kv head into the token's page, q written for the attention kernel.
//  * paged_attention_simple: one block per (token, query head); its warps share the keys of the
//    token's context [lo, pos] (lo > 0 only for a window) and merge their online softmaxes.
//
// These are the true 32-bit kernels and the fallback of the bfloat16 path for shapes that
// the tensor-core kernels refuse.  Cache layout: pages[page][0 = keys, 1 = values][kv head]
// [slot][head_dim]; a token at position p of request r lies in page block_table[r][p / page_size],
// slot p % page_size.
#include "common.cuh"

namespace {

constexpr int MAX_HEAD_DIM = 256;
constexpr int WARPS = 4;

enum { TI_ERR_BAD_PAGE = 1 };

template <typename TQ, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_kernel(const float* qkv, int qkv_stride,
                          const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                          float eps, const float* __restrict__ inv_freq,
                          const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                          const int* __restrict__ block_table, int bt_stride,
                          TC* __restrict__ pages, int num_pages, int page_size, int write_kv,
                          int num_heads, int num_kv_heads, int head_dim, int rotary_dim,
                          TQ* __restrict__ q_out, int* __restrict__ status) {
    __shared__ float vec[WARPS][MAX_HEAD_DIM];
    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int item = blockIdx.y * WARPS + warp;
    const int items = num_heads + 2 * num_kv_heads;
    if (item >= items) return;
    const int half = rotary_dim >> 1;                 // pairs (k, k + half), k < half, are rotated
    const int nq = num_heads * head_dim, nk = num_kv_heads * head_dim;
    const int pos = positions[t];

    // which vector: a query head, a key head or a value head
    int kind, head;
    if (item < num_heads) { kind = 0; head = item; }
    else if (item < num_heads + num_kv_heads) { kind = 1; head = item - num_heads; }
    else { kind = 2; head = item - num_heads - num_kv_heads; }
    if (kind != 0 && !write_kv) return;
    const float* src = qkv + (size_t)t * qkv_stride +
                       (kind == 0 ? head * head_dim : kind == 1 ? nq + head * head_dim
                                                                : nq + nk + head * head_dim);
    TC* dst = nullptr;
    if (kind != 0) {
        const int r = req_of_tok[t];
        const int page = block_table[(size_t)r * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
            return;
        }
        dst = pages + ((((size_t)page * 2 + (kind - 1)) * num_kv_heads + head) * page_size +
                       pos % page_size) * head_dim;
    }
    if (kind == 2) {                                   // values are stored as they are
        for (int d = lane; d < head_dim; d += 32) dst[d] = from_f32<TC>(src[d]);
        return;
    }
    const float* w = kind == 0 ? q_weight : k_weight;
    float ss = 0.0f;
    for (int d = lane; d < head_dim; d += 32) {
        const float v = src[d];
        vec[warp][d] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
    __syncwarp();
    for (int k = lane; k < half; k += 32) {
        const float x0 = vec[warp][k] * inv * w[k];
        const float x1 = vec[warp][k + half] * inv * w[k + half];
        const float angle = (float)pos * inv_freq[k];
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const float y0 = x0 * cs - x1 * sn;
        const float y1 = x0 * sn + x1 * cs;
        if (kind == 0) {
            TQ* q = q_out + (size_t)t * nq + head * head_dim;
            q[k] = from_f32<TQ>(y0);
            q[k + half] = from_f32<TQ>(y1);
        } else {
            dst[k] = from_f32<TC>(y0);
            dst[k + half] = from_f32<TC>(y1);
        }
    }
    // what lies beyond the rotated width is normed only
    for (int d = rotary_dim + lane; d < head_dim; d += 32) {
        const float y = vec[warp][d] * inv * w[d];
        if (kind == 0) q_out[(size_t)t * nq + head * head_dim + d] = from_f32<TQ>(y);
        else dst[d] = from_f32<TC>(y);
    }
}

// The same work for head sizes up to 64 * VEC with head_dim / 2 a multiple of VEC: a lane keeps
// VEC consecutive elements of each half of the vector in registers (the rotation pairs element
// k with k + head_dim / 2, so a lane owns whole pairs); no shared memory.
template <typename TQ, typename TC, int VEC>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_vec_kernel(const float* qkv, int qkv_stride,
                              const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                              float eps, const float* __restrict__ inv_freq,
                              const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                              const int* __restrict__ block_table, int bt_stride,
                              TC* __restrict__ pages, int num_pages, int page_size, int write_kv,
                              int num_heads, int num_kv_heads, int head_dim, int items_per_warp,
                              TQ* __restrict__ q_out, int* __restrict__ status) {
    __shared__ float cs_tab[MAX_HEAD_DIM / 2], sn_tab[MAX_HEAD_DIM / 2];
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const int nq = num_heads * head_dim, nk = num_kv_heads * head_dim;
    const int pos = positions[t];
    // the rotation of a token is the same for all its heads: its sines and cosines once per block
    for (int k = threadIdx.x; k < half; k += WARPS * 32)
        sincosf((float)pos * inv_freq[k], &sn_tab[k], &cs_tab[k]);
    pdl_wait();
    __syncthreads();
    // With many tokens a warp takes up to MAX_TURNS vectors, so that blocks are not tiny; all of
    // their loads are issued before any of them is used.  (Few tokens take
    // qk_norm_rope_store_one_kernel below.)
    constexpr int MAX_TURNS = 8;
    const int items = num_heads + 2 * num_kv_heads;
    const int k0 = lane * VEC;
    const bool active = k0 < half;
    float lo[MAX_TURNS][VEC], hi[MAX_TURNS][VEC];
#pragma unroll
    for (int turn = 0; turn < MAX_TURNS; ++turn) {
        const int item = (blockIdx.y * items_per_warp + turn) * WARPS + warp;
        const bool live = turn < items_per_warp && item < items && active;
        const float* src = qkv + (size_t)t * qkv_stride + (size_t)(live ? item : 0) * head_dim;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            lo[turn][i] = live ? src[k0 + i] : 0.0f;
            hi[turn][i] = live ? src[half + k0 + i] : 0.0f;
        }
    }
    int page = -1;
    if (write_kv) {
        page = block_table[(size_t)req_of_tok[t] * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
            page = -1;
        }
    }
#pragma unroll
    for (int turn = 0; turn < MAX_TURNS; ++turn) {
        const int item = (blockIdx.y * items_per_warp + turn) * WARPS + warp;
        if (turn >= items_per_warp || item >= items) break;
        // the vectors of a token lie one after the other: query heads, key heads, value heads
        const int kind = item < num_heads ? 0 : item < num_heads + num_kv_heads ? 1 : 2;
        const int head = kind == 0 ? item : kind == 1 ? item - num_heads : item - num_heads - num_kv_heads;
        if (kind != 0 && page < 0) continue;
        TC* dst = nullptr;
        if (kind != 0)
            dst = pages + ((((size_t)page * 2 + (kind - 1)) * num_kv_heads + head) * page_size +
                           pos % page_size) * head_dim;
        if (kind == 2) {
            if (active) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    dst[k0 + i] = from_f32<TC>(lo[turn][i]);
                    dst[half + k0 + i] = from_f32<TC>(hi[turn][i]);
                }
            }
            continue;
        }
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            ss = fmaf(lo[turn][i], lo[turn][i], ss);
            ss = fmaf(hi[turn][i], hi[turn][i], ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
        if (!active) continue;
        const float* w = kind == 0 ? q_weight : k_weight;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float x0 = lo[turn][i] * inv * w[k0 + i];
            const float x1 = hi[turn][i] * inv * w[half + k0 + i];
            const float sn = sn_tab[k0 + i], cs = cs_tab[k0 + i];
            const float y0 = x0 * cs - x1 * sn;
            const float y1 = x0 * sn + x1 * cs;
            if (kind == 0) {
                TQ* q = q_out + (size_t)t * nq + head * head_dim;
                q[k0 + i] = from_f32<TQ>(y0);
                q[half + k0 + i] = from_f32<TQ>(y1);
            } else {
                dst[k0 + i] = from_f32<TC>(y0);
                dst[half + k0 + i] = from_f32<TC>(y1);
            }
        }
    }
}

// The same work for the few tokens of a decode step, one vector per warp: everything that does
// not come from the kernel before (the token's position and page, its sines and cosines, the norm
// weights) is in registers before the wait for that kernel returns, so that behind the wait
// there is one round of loads, the norm, the rotation and the stores.  Arithmetic and order are
// those of qk_norm_rope_store_vec_kernel.
template <typename TQ, typename TC, int VEC>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_one_kernel(const float* qkv, int qkv_stride,
                              const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                              float eps, const float* __restrict__ inv_freq,
                              const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                              const int* __restrict__ block_table, int bt_stride,
                              TC* __restrict__ pages, int num_pages, int page_size, int write_kv,
                              int num_heads, int num_kv_heads, int head_dim,
                              TQ* __restrict__ q_out, int* __restrict__ status) {
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const int items = num_heads + 2 * num_kv_heads;
    const int item = blockIdx.y * WARPS + warp;
    const int k0 = lane * VEC;
    const bool active = k0 < half, live = item < items;
    // the vectors of a token lie one after the other: query heads, key heads, value heads
    const int kind = item < num_heads ? 0 : item < num_heads + num_kv_heads ? 1 : 2;
    const int head = kind == 0 ? item : kind == 1 ? item - num_heads : item - num_heads - num_kv_heads;
    const int pos = positions[t];
    int page = -1;
    if (write_kv && kind != 0 && live) {
        page = block_table[(size_t)req_of_tok[t] * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
            page = -1;
        }
    }
    float sn[VEC], cs[VEC], w0[VEC], w1[VEC];
    if (live && active && kind != 2) {
        const float* w = kind == 0 ? q_weight : k_weight;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            sincosf((float)pos * inv_freq[k0 + i], &sn[i], &cs[i]);
            w0[i] = w[k0 + i];
            w1[i] = w[half + k0 + i];
        }
    }
    pdl_wait();
    if (!live) return;
    float lo[VEC], hi[VEC];
    const float* src = qkv + (size_t)t * qkv_stride + (size_t)item * head_dim;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        lo[i] = active ? src[k0 + i] : 0.0f;
        hi[i] = active ? src[half + k0 + i] : 0.0f;
    }
    if (kind != 0 && page < 0) return;
    TC* dst = nullptr;
    if (kind != 0)
        dst = pages + ((((size_t)page * 2 + (kind - 1)) * num_kv_heads + head) * page_size +
                       pos % page_size) * head_dim;
    if (kind == 2) {
        if (active) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                dst[k0 + i] = from_f32<TC>(lo[i]);
                dst[half + k0 + i] = from_f32<TC>(hi[i]);
            }
        }
        return;
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        ss = fmaf(lo[i], lo[i], ss);
        ss = fmaf(hi[i], hi[i], ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
    if (!active) return;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const float x0 = lo[i] * inv * w0[i];
        const float x1 = hi[i] * inv * w1[i];
        const float y0 = x0 * cs[i] - x1 * sn[i];
        const float y1 = x0 * sn[i] + x1 * cs[i];
        if (kind == 0) {
            TQ* q = q_out + ((size_t)t * num_heads + head) * head_dim;
            q[k0 + i] = from_f32<TQ>(y0);
            q[half + k0 + i] = from_f32<TQ>(y1);
        } else {
            dst[k0 + i] = from_f32<TC>(y0);
            dst[half + k0 + i] = from_f32<TC>(y1);
        }
    }
}

template <typename TQ, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simple_kernel(const TQ* __restrict__ q, const int* __restrict__ rows,
                              const int* __restrict__ positions,
                              const int* __restrict__ req_of_tok,
                              const int* __restrict__ block_table, int bt_stride,
                              const TC* __restrict__ pages, int num_pages, int page_size,
                              int num_heads, int num_kv_heads, int head_dim, int window,
                              float scale, TQ* __restrict__ out, int* __restrict__ status) {
    constexpr int PER_LANE = MAX_HEAD_DIM / 32;
    __shared__ float so[WARPS][MAX_HEAD_DIM];
    __shared__ float sm[WARPS], sl[WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, t = rows ? rows[blockIdx.x] : blockIdx.x;
    const int kvh = h / (num_heads / num_kv_heads);
    const int pos = positions[t];
    const int r = req_of_tok[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)r * bt_stride;

    float qv[PER_LANE], o[PER_LANE];
    const TQ* qh = q + ((size_t)t * num_heads + h) * head_dim;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < head_dim ? to_f32(qh[d]) : 0.0f;
        o[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    bool bad = false;
    for (int p = lo + warp; p <= pos; p += WARPS) {
        const int page = table[p / page_size];
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const TC* kp = pages + (((size_t)page * 2 * num_kv_heads + kvh) * page_size +
                                p % page_size) * head_dim;
        const TC* vp = kp + (size_t)num_kv_heads * page_size * head_dim;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) s = fmaf(qv[i], to_f32(kp[d]), s);
        }
        s = warp_sum(s) * scale;
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);          // exp(-inf) = 0 on the first key
        const float pr = expf(s - m_new);
        l = l * alpha + pr;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) o[i] = fmaf(pr, to_f32(vp[d]), o[i] * alpha);
        }
        m = m_new;
    }
    if (bad && lane == 0) atomicCAS(status, 0, TI_ERR_BAD_PAGE);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) so[warp][d] = o[i];
    }
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
    __syncthreads();
    if (warp == 0) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sm[w]);
        float ltot = 0.0f, wt[WARPS];
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            wt[w] = sl[w] > 0.0f ? expf(sm[w] - mm) : 0.0f;
            ltot += sl[w] * wt[w];
        }
        const float inv = 1.0f / ltot;
        TQ* oh = out + ((size_t)t * num_heads + h) * head_dim;
        for (int d = lane; d < head_dim; d += 32) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) acc = fmaf(so[w][d], wt[w], acc);
            oh[d] = from_f32<TQ>(acc * inv);
        }
    }
}

}  // namespace

#define TI_DISPATCH_QC(qd, cd, CALL)                                               \
    if (qd == TI_F32 && cd == TI_F32) { CALL(float, float); }                      \
    else if (qd == TI_BF16 && cd == TI_BF16) { CALL(bf16, bf16); }                 \
    else if (qd == TI_F32 && cd == TI_BF16) { CALL(float, bf16); }                 \
    else return ti_fail("attention: dtype codes q=%d cache=%d are not supported", qd, cd);

extern "C" int ti_qk_norm_rope_store(const float* qkv, int qkv_stride, const float* q_weight,
                                     const float* k_weight, float eps, const float* inv_freq,
                                     const int* positions, const int* req_of_tok,
                                     const int* block_table, int bt_stride, void* pages,
                                     int cache_dtype, int num_pages, int page_size, int write_kv,
                                     int num_tokens, int num_heads, int num_kv_heads, int head_dim,
                                     int rotary_dim, void* q_out, int q_dtype, int* status,
                                     void* stream) {
    if (num_tokens == 0) return 0;
    TI_REQUIRE(head_dim >= 1 && head_dim <= MAX_HEAD_DIM,
               "qk_norm_rope_store: head_dim %d must be at most %d", head_dim, MAX_HEAD_DIM);
    TI_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
               "qk_norm_rope_store: the rotated width %d must be even and at most head_dim %d",
               rotary_dim, head_dim);
    TI_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "qk_norm_rope_store: no rotation table");
    const int items = num_heads + 2 * num_kv_heads;
    dim3 grid(num_tokens, (items + WARPS - 1) / WARPS);
    cudaStream_t s = (cudaStream_t)stream;
    const int half = head_dim / 2;
    int ipw = num_tokens >= 512 ? (items + WARPS - 1) / WARPS : 1;            // vectors per warp
    if (ipw > 8) ipw = 8;
    dim3 vgrid(num_tokens, (items + WARPS * ipw - 1) / (WARPS * ipw));
    // the register kernel pairs element k with k + head_dim / 2: for a rotation over the whole head only
    const int vec = rotary_dim != head_dim ? 0
                    : (half % 4 == 0 && half > 64) ? 4 : (half % 2 == 0 && half <= 64) ? 2 : 0;
#define CALL(TQ, TC)                                                                          \
    if (vec == 2 && ipw == 1)                                                                 \
        ti_launch_pdl((qk_norm_rope_store_one_kernel<TQ, TC, 2>), vgrid, WARPS * 32, 0, s,     \
            qkv, qkv_stride, q_weight, k_weight, eps, inv_freq, positions, req_of_tok, block_table, \
            bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads,     \
            head_dim, (TQ*)q_out, status);                                                     \
    else if (vec == 4 && ipw == 1)                                                            \
        ti_launch_pdl((qk_norm_rope_store_one_kernel<TQ, TC, 4>), vgrid, WARPS * 32, 0, s,     \
            qkv, qkv_stride, q_weight, k_weight, eps, inv_freq, positions, req_of_tok, block_table, \
            bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads,     \
            head_dim, (TQ*)q_out, status);                                                     \
    else if (vec == 2)                                                                        \
        ti_launch_pdl(qk_norm_rope_store_vec_kernel<TQ, TC, 2>, vgrid, WARPS * 32, 0, s,       \
            qkv, qkv_stride, q_weight, k_weight, eps, inv_freq, positions, req_of_tok, block_table, \
            bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads,     \
            head_dim, ipw, (TQ*)q_out, status);                                                \
    else if (vec == 4)                                                                        \
        ti_launch_pdl(qk_norm_rope_store_vec_kernel<TQ, TC, 4>, vgrid, WARPS * 32, 0, s,       \
            qkv, qkv_stride, q_weight, k_weight, eps, inv_freq, positions, req_of_tok, block_table, \
            bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads,     \
            head_dim, ipw, (TQ*)q_out, status);                                                \
    else                                                                                      \
        ti_launch_pdl(qk_norm_rope_store_kernel<TQ, TC>, grid, WARPS * 32, 0, s,               \
            qkv, qkv_stride, q_weight, k_weight, eps, inv_freq, positions, req_of_tok, block_table, \
            bt_stride, (TC*)pages, num_pages, page_size, write_kv, num_heads, num_kv_heads,     \
            head_dim, rotary_dim, (TQ*)q_out, status)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
    return ti_check_launch("qk_norm_rope_store");
}

// `rows` (may be null) lists the tokens to compute; without it all `num_rows` tokens are computed.
extern "C" int ti_paged_attention_simple(const void* q, int q_dtype, const int* rows,
                                         const int* positions,
                                         const int* req_of_tok, const int* block_table,
                                         int bt_stride, const void* pages, int cache_dtype,
                                         int num_pages, int page_size, int num_rows,
                                         int num_heads, int num_kv_heads, int head_dim, int window,
                                         float scale, void* out, int* status, void* stream) {
    if (num_rows == 0) return 0;
    TI_REQUIRE(head_dim >= 1 && head_dim <= MAX_HEAD_DIM,
               "paged_attention: head_dim %d must be at most %d", head_dim, MAX_HEAD_DIM);
    TI_REQUIRE(num_heads % num_kv_heads == 0, "paged_attention: %d heads over %d kv heads",
               num_heads, num_kv_heads);
    dim3 grid(num_rows, num_heads);
    cudaStream_t s = (cudaStream_t)stream;
#define CALL(TQ, TC)                                                                           \
    paged_attention_simple_kernel<TQ, TC><<<grid, WARPS * 32, 0, s>>>(                          \
        (const TQ*)q, rows, positions, req_of_tok, block_table, bt_stride, (const TC*)pages,     \
        num_pages,                                                                              \
        page_size, num_heads, num_kv_heads, head_dim, window, scale, (TQ*)out, status)
    TI_DISPATCH_QC(q_dtype, cache_dtype, CALL)
#undef CALL
    return ti_check_launch("paged_attention_simple");
}
