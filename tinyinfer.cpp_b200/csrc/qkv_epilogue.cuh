// Epilogue of the QKV product of a prompt portion, run by the tcgen05 kernels in place of storing
// the product: a thread that owns one token's 128 accumulator columns of one head (head size 128)
// applies the head's RMSNorm (queries and keys), rotates it (NeoX pairs k, k + 64) by the token's
// position, and writes bfloat16: queries to q_out, keys and values into the token's slot of its
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

// `taddr`: tensor-memory address of this thread's lane at the first of the head's 128 columns.
// `t`: the token (row of the product), `item`: the head, `dst` from destination().  All 32 lanes of
// the warp call this (tcgen05.ld is warp-wide).
__device__ __forceinline__ void head(const Epilogue& e, unsigned taddr, int t, int item, bf16* dst) {
    const int kind = item < e.num_heads ? 0 : item < e.num_heads + e.num_kv_heads ? 1 : 2;
    float v[32];
    if (kind == 2) {                                   // values: rounded and stored as they are
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            sm100::tmem_load32(taddr + (unsigned)(c * 32), v);
            if (dst != nullptr) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = pack8(v + j * 8);
            }
        }
        return;
    }
    float ss4[4] = {0.0f, 0.0f, 0.0f, 0.0f};              // four chains: one warp has little else to issue
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
        sm100::tmem_load32(taddr + (unsigned)(c * 32), v);
#pragma unroll
        for (int i = 0; i < 32; ++i) ss4[i & 3] = fmaf(v[i], v[i], ss4[i & 3]);
    }
    const float ss = (ss4[0] + ss4[1]) + (ss4[2] + ss4[3]);
    const float inv = 1.0f / sqrtf(ss / (float)HEAD_DIM + e.eps);
    const float* w = kind == 0 ? e.q_weight : e.k_weight;
    const float* tab = e.table + (size_t)(dst != nullptr ? t : 0) * HEAD_DIM;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
        // the sines and cosines come from L2: all of this half's loads are in flight together
        float4 cs[8], sn[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            cs[j] = __ldg(reinterpret_cast<const float4*>(tab + c * 32 + j * 4));
            sn[j] = __ldg(reinterpret_cast<const float4*>(tab + HALF + c * 32 + j * 4));
        }
        float hi[32];
        sm100::tmem_load32(taddr + (unsigned)(c * 32), v);
        sm100::tmem_load32(taddr + (unsigned)(HALF + c * 32), hi);
        if (dst == nullptr) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float y0[8], y1[8];
#pragma unroll
            for (int i = 0; i < 8; i += 4) {
                const int k = c * 32 + j * 8 + i;
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + k));
                const float4 w1 = __ldg(reinterpret_cast<const float4*>(w + HALF + k));
                const float4 c4 = cs[j * 2 + i / 4], s4 = sn[j * 2 + i / 4];
                const float cs_[4] = {c4.x, c4.y, c4.z, c4.w}, sn_[4] = {s4.x, s4.y, s4.z, s4.w};
                const float w0_[4] = {w0.x, w0.y, w0.z, w0.w}, w1_[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float x0 = v[j * 8 + i + u] * inv * w0_[u];
                    const float x1 = hi[j * 8 + i + u] * inv * w1_[u];
                    y0[i + u] = x0 * cs_[u] - x1 * sn_[u];
                    y1[i + u] = x0 * sn_[u] + x1 * cs_[u];
                }
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = pack8(y0);
            *reinterpret_cast<uint4*>(dst + HALF + c * 32 + j * 8) = pack8(y1);
        }
    }
}

}  // namespace qkv
