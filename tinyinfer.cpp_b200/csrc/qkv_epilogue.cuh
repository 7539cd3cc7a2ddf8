// Epilogue of the QKV product of a prompt portion, run by the tcgen05 kernels in place of storing
// the product: the threads that own a token's accumulator columns of a head (head size 128)
// apply the head's RMSNorm (queries and keys), rotate it (NeoX pairs k, k + 64) by the token's
// position, and write bfloat16: queries to q_out, keys and values into the token's slot of its
// request's page.  The float32 product never reaches memory, and the separate norm / rotation /
// store launch and its read of the product are saved.
//
// The sines and cosines of a step's positions are the same for all layers: rope_table_kernel makes
// them once per step, table[t] = {cos(pos_t * inv_freq[0..63]), sin(...)} in float32 with the
// precise sincosf.
#pragma once

#include "sm100.cuh"

namespace qkv {

constexpr int HEAD_DIM = 128, HALF = 64;

struct Epilogue {
    const float* q_weight;       // [128] norm weights
    const float* k_weight;
    float eps;
    const float* table;          // [T][2][64]
    const int* positions;        // [T]
    const int* req_of_tok;       // [T]
    const int* block_table;      // [requests][bt_stride]
    int bt_stride;
    bf16* pages;                 // [page][2][kv_heads][page_size][128]
    int num_pages, page_size, write_kv;
    int num_heads, num_kv_heads;
    bf16* q_out;                 // [T][num_heads * 128]
};

__device__ __forceinline__ uint4 pack8(const float* y) {
    __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(y[4], y[5]), d = __floats2bfloat162_rn(y[6], y[7]);
    return make_uint4(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b),
                      *reinterpret_cast<unsigned*>(&c), *reinterpret_cast<unsigned*>(&d));
}

// Where the head `item` (among [queries, keys, values]) of token `t` goes: a row of q_out or the
// token's slot in its request's page; null if the row or head does not exist (`live`) or nothing
// is to be written.  The look-ups (position, request, block table) depend on nothing the product
// computes, so the caller does them before it waits for the accumulator.
__device__ __forceinline__ bf16* destination(const Epilogue& e, int t, int item, bool live, int* status) {
    const int kind = item < e.num_heads ? 0 : item < e.num_heads + e.num_kv_heads ? 1 : 2;
    bf16* dst = nullptr;
    if (live) {
        if (kind == 0) {
            dst = e.q_out + ((size_t)t * e.num_heads + item) * HEAD_DIM;
        } else if (e.write_kv) {
            const int pos = e.positions[t];
            const int page = e.block_table[(size_t)e.req_of_tok[t] * e.bt_stride + pos / e.page_size];
            if (page < 0 || page >= e.num_pages) {
                atomicCAS(status, 0, 1);
            } else {
                const int h = kind == 1 ? item - e.num_heads : item - e.num_heads - e.num_kv_heads;
                dst = e.pages + ((((size_t)page * 2 + (kind - 1)) * e.num_kv_heads + h) * e.page_size +
                                 pos % e.page_size) * HEAD_DIM;
            }
        }
    }
    return dst;
}

// A 256-column tile holds two heads of 128 tokens.  A warp of the epilogue has 32 of the tokens
// (its lanes of tensor memory) and, of both heads, the rotation pairs 32 h .. 32 h + 31 (columns k
// and k + 64), h = 0 or 1: so a thread needs half of its token's sines and cosines and uses them
// for both heads.  It requests them, like the destinations, before it waits for the accumulator;
// after the wait only tensor memory, arithmetic and 32-byte stores remain.
struct Angles {
    float4 cs[8], sn[8];         // of pairs 32 h .. 32 h + 31
};

__device__ __forceinline__ void load_angles(const Epilogue& e, int t, int h, bool live, Angles& a) {
    const float* tab = e.table + (size_t)(live ? t : 0) * HEAD_DIM + h * 32;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        a.cs[j] = __ldg(reinterpret_cast<const float4*>(tab + j * 4));
        a.sn[j] = __ldg(reinterpret_cast<const float4*>(tab + HALF + j * 4));
    }
}

// The q and k norm weights, [2][128], copied once into shared memory by the block.
__device__ __forceinline__ void load_norm_weights(const Epilogue& e, float* norm_w, int tid, int threads) {
    for (int i = tid; i < 2 * HEAD_DIM; i += threads)
        norm_w[i] = i < HEAD_DIM ? e.q_weight[i] : e.k_weight[i - HEAD_DIM];
}

__device__ __forceinline__ void store16(bf16* dst, const float* y) {      // 32 bytes, 32-byte aligned
    const uint4 a = pack8(y), b = pack8(y + 8);
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(a.x), "r"(a.y),
                 "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}

// `taddr`: tensor-memory address of this thread's lane at the tile's first column; `item0`: the
// tile's first head; `h`: which half of the pairs; `dst0`, `dst1` from destination() for the two
// heads; `norm_w`: shared memory filled by load_norm_weights.  All 32 lanes of the warp call this
// (tcgen05.ld is warp-wide).
__device__ __forceinline__ void two_heads(const Epilogue& e, const float* norm_w, unsigned taddr, int item0,
                                          int h, bf16* dst0, bf16* dst1, const Angles& a) {
    const float* cs = reinterpret_cast<const float*>(a.cs);
    const float* sn = reinterpret_cast<const float*>(a.sn);
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
        const int item = item0 + which;
        if (item >= e.num_heads + 2 * e.num_kv_heads) break;           // the same for the whole warp
        const int kind = item < e.num_heads ? 0 : item < e.num_heads + e.num_kv_heads ? 1 : 2;
        bf16* dst = which ? dst1 : dst0;
        const unsigned base = taddr + (unsigned)(which * HEAD_DIM);
        float inv = 1.0f;
        if (kind != 2) {
            float ss4[4] = {0.0f, 0.0f, 0.0f, 0.0f};          // four chains: one warp has little else to issue
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float v[32];
                sm100::tmem_load32(base + (unsigned)(c * 32), v);
#pragma unroll
                for (int i = 0; i < 32; ++i) ss4[i & 3] = fmaf(v[i], v[i], ss4[i & 3]);
            }
            const float ss = (ss4[0] + ss4[1]) + (ss4[2] + ss4[3]);
            inv = 1.0f / sqrtf(ss / (float)HEAD_DIM + e.eps);
        }
        const float* w = norm_w + (kind == 1 ? HEAD_DIM : 0);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float lo[16], hi[16];
            sm100::tmem_load16(base + (unsigned)(h * 32 + c * 16), lo);
            sm100::tmem_load16(base + (unsigned)(HALF + h * 32 + c * 16), hi);
            if (dst == nullptr) continue;
            if (kind != 2) {                                   // values are rounded and stored as they are
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int k = h * 32 + c * 16 + i;
                    const float x0 = lo[i] * inv * w[k], x1 = hi[i] * inv * w[HALF + k];
                    lo[i] = x0 * cs[c * 16 + i] - x1 * sn[c * 16 + i];
                    hi[i] = x0 * sn[c * 16 + i] + x1 * cs[c * 16 + i];
                }
            }
            store16(dst + h * 32 + c * 16, lo);
            store16(dst + HALF + h * 32 + c * 16, hi);
        }
    }
}

}  // namespace qkv
