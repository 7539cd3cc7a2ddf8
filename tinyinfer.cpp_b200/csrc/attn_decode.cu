// Paged flash-decoding for single-token rows (bfloat16 cache, head_dim a multiple of 16 up to 128).
//
// A row is one new token of a request; it attends to the keys [lo, pos] of its request's
// pages (lo > 0 only with a window).  The keys are cut into tiles of 32; the tiles of a row
// are dealt to `num_splits` blocks per kv head.  A block is ONE warp: it streams its tiles
// through a ring of shared-memory stages with cp.async, computes the scores of all query
// heads of the kv group at once on the tensor cores (mma.sync m16n8k16, the group's heads
// are the 16 rows of the A operand), keeps a float32 online softmax per head, multiplies the
// probabilities with the values, and writes an unnormalised partial result with its running
// maximum and sum.  The block that finishes a (row, kv head) last merges the partial results
// (or a second kernel does, if the caller gives no counters); a short row leaves some splits
// without keys, and the merge in the same launch skips them.
// The work is bound by the bytes of keys and values; the tensor cores only keep the arithmetic
// out of the way.
//
// Everything that changes from step to step (positions, block tables) is read from device
// memory, and the cut into splits depends only on the row's own length and on `num_splits`,
// so a launch can be replayed from a CUDA graph.
#include "attn_decode_core.cuh"

namespace {

using namespace attn_decode_core;

// LATE_WAIT: the kernel before this one needs none of this kernel's results and this kernel none
// of its, and that kernel released its dependents only after its own wait had returned, so
// everything a block reads here was complete when the block started.  The blocks run beside that
// kernel without waiting for it; one block waits for it at its end (the others leave their SMs to
// blocks still to come), so that whoever waits for this kernel has waited for both.
template <int HD, bool SINGLE, bool LATE_WAIT = false>
__global__ void __launch_bounds__(32)
attn_decode_kernel(const bf16* q, const int* __restrict__ rows,
                   const int* __restrict__ positions, const int* __restrict__ req_of_tok,
                   const int* __restrict__ block_table, int bt_stride,
                   const bf16* __restrict__ pages, int num_pages, int page_size,
                   int num_heads, int num_kv_heads, int window, float scale_log2,
                   float* __restrict__ part_o, float* __restrict__ part_ml,
                   unsigned* __restrict__ counters, bf16* __restrict__ out,
                   int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int kvh = blockIdx.y, row = blockIdx.z;
    const int t = rows ? rows[row] : row;
    const int group = num_heads / num_kv_heads;
    decode_item<HD, true, NoPrologue, SINGLE, LATE_WAIT>(
        smem, q + ((size_t)t * num_heads + (size_t)kvh * group) * HD, nullptr, nullptr,
        blockIdx.x, gridDim.x, kvh, row, t, positions[t],
        block_table + (size_t)req_of_tok[t] * bt_stride, pages, num_pages, page_size,
        num_heads, num_kv_heads, window, scale_log2, part_o, part_ml, counters, out, status);
    if constexpr (LATE_WAIT) {
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) pdl_wait();
    }
}

// Head norm and NeoX rotation of a head vector of which a lane holds the elements k0, k0 + 1 of both
// halves (lo, hi); sn/cs: sine and cosine of the position's angles for these two pairs.  The
// arithmetic and its order are those of qk_norm_rope_store_vec_kernel with two elements per lane.
template <int HD>
__device__ __forceinline__ void norm_rotate(float2 lo, float2 hi, const float* __restrict__ weight, float eps,
                                            const float (&sn)[2], const float (&cs)[2], bool active,
                                            bf16* dst, bf16* dst2) {
    constexpr int HALF = HD / 2;
    const int k0 = (threadIdx.x & 31) * 2;
    float ss = 0.0f;
    ss = fmaf(lo.x, lo.x, ss); ss = fmaf(hi.x, hi.x, ss);
    ss = fmaf(lo.y, lo.y, ss); ss = fmaf(hi.y, hi.y, ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
    if (!active) return;
    const float l[2] = {lo.x, lo.y}, h[2] = {hi.x, hi.y};
    float y0[2], y1[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float x0 = l[i] * inv * weight[k0 + i];
        const float x1 = h[i] * inv * weight[HALF + k0 + i];
        y0[i] = x0 * cs[i] - x1 * sn[i];
        y1[i] = x0 * sn[i] + x1 * cs[i];
    }
    const __nv_bfloat162 a = __floats2bfloat162_rn(y0[0], y0[1]), b = __floats2bfloat162_rn(y1[0], y1[1]);
    *reinterpret_cast<__nv_bfloat162*>(dst + k0) = a;
    *reinterpret_cast<__nv_bfloat162*>(dst + HALF + k0) = b;
    if (dst2) {
        *reinterpret_cast<__nv_bfloat162*>(dst2 + k0) = a;
        *reinterpret_cast<__nv_bfloat162*>(dst2 + HALF + k0) = b;
    }
}

constexpr int QKV_MAX_GROUP = 8;           // query heads per kv head that the kernel below stages

// Flash-decoding straight from the float32 QKV product: what qk_norm_rope_store does for a
// single-token row happens in the attention kernel itself, so the step has one launch less per
// layer.  Every item norms and rotates the queries of its kv head's group (a few hundred
// flops); the split that holds the row's own position also norms and rotates the new key,
// rounds the new value, writes both into the page for later steps and uses them from shared
// memory itself.  No other item reads that key: it lies in the last tile, which one split owns.
template <int HD>
__global__ void __launch_bounds__(32)
attn_decode_qkv_kernel(const float* qkv, int width, const float* __restrict__ q_weight,
                       const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
                       const int* __restrict__ rows, const int* __restrict__ positions,
                       const int* __restrict__ req_of_tok, const int* __restrict__ block_table, int bt_stride,
                       bf16* __restrict__ pages, int num_pages, int page_size, int write_kv,
                       int num_heads, int num_kv_heads, int window, float scale_log2,
                       float* __restrict__ part_o, float* __restrict__ part_ml,
                       unsigned* __restrict__ counters, bf16* __restrict__ out, int* __restrict__ status) {
    constexpr int HALF = HD / 2;
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* q_stage = reinterpret_cast<bf16*>(smem + item_smem_bytes<HD>());
    bf16* new_k = q_stage + QKV_MAX_GROUP * HD;
    bf16* new_v = new_k + HD;
    const int lane = threadIdx.x;
    const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const int t = rows ? rows[row] : row;
    const int group = num_heads / num_kv_heads;
    const int nq = num_heads * HD, nk = num_kv_heads * HD;
    const int pos = positions[t];
    const int* table = block_table + (size_t)req_of_tok[t] * bt_stride;
    const SplitRange range = split_range(pos, window, gridDim.x, split);
    const bool owner = range.owns_newest();
    const bool has_tiles = range.my_lo < range.my_hi;
    const int k0 = lane * 2;
    const bool active = k0 < HALF;
    // what does not depend on the kernel before: the norm weights, the angles, the new key's place
    float sn[2] = {0.0f, 0.0f}, cs[2] = {1.0f, 1.0f};
    if (active && has_tiles) {
        sincosf((float)pos * inv_freq[k0], &sn[0], &cs[0]);
        sincosf((float)pos * inv_freq[k0 + 1], &sn[1], &cs[1]);
    }
    bf16* kdst = nullptr;
    bf16* vdst = nullptr;
    if (owner && write_kv) {
        const int page = table[pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicCAS(status, 0, 1);
        } else {
            kdst = pages + ((((size_t)page * 2) * num_kv_heads + kvh) * page_size + pos % page_size) * HD;
            vdst = kdst + (size_t)num_kv_heads * page_size * HD;
        }
    }
    auto prologue = [&]() {
        if (!has_tiles) return;
        const float* src = qkv + (size_t)t * width;
        // all of the item's vectors are requested before any is used
        float2 qlo[QKV_MAX_GROUP], qhi[QKV_MAX_GROUP];
        float2 klo = make_float2(0.f, 0.f), khi = klo, v0 = klo, v1 = klo;
#pragma unroll
        for (int h = 0; h < QKV_MAX_GROUP; ++h) {
            qlo[h] = qhi[h] = make_float2(0.f, 0.f);
            if (h < group && active) {
                const float* q = src + (size_t)(kvh * group + h) * HD;
                qlo[h] = *reinterpret_cast<const float2*>(q + k0);
                qhi[h] = *reinterpret_cast<const float2*>(q + HALF + k0);
            }
        }
        if (owner && active) {
            const float* k = src + nq + (size_t)kvh * HD;
            const float* v = k + nk;
            klo = *reinterpret_cast<const float2*>(k + k0);
            khi = *reinterpret_cast<const float2*>(k + HALF + k0);
            v0 = *reinterpret_cast<const float2*>(v + k0);
            v1 = *reinterpret_cast<const float2*>(v + HALF + k0);
        }
#pragma unroll
        for (int h = 0; h < QKV_MAX_GROUP; ++h)
            if (h < group) norm_rotate<HD>(qlo[h], qhi[h], q_weight, eps, sn, cs, active, q_stage + h * HD, nullptr);
        if (owner) {
            norm_rotate<HD>(klo, khi, k_weight, eps, sn, cs, active, new_k, kdst);
            if (active) {
                const __nv_bfloat162 a = __floats2bfloat162_rn(v0.x, v0.y), b = __floats2bfloat162_rn(v1.x, v1.y);
                *reinterpret_cast<__nv_bfloat162*>(new_v + k0) = a;
                *reinterpret_cast<__nv_bfloat162*>(new_v + HALF + k0) = b;
                if (vdst) {
                    *reinterpret_cast<__nv_bfloat162*>(vdst + k0) = a;
                    *reinterpret_cast<__nv_bfloat162*>(vdst + HALF + k0) = b;
                }
            }
        }
        __syncwarp();
    };
    // an entry that only reads the cache finds the key and value that another entry stored
    const bool patch = owner && write_kv;
    decode_item<HD, true>(smem, q_stage, patch ? new_k : nullptr, patch ? new_v : nullptr, split, gridDim.x,
                          kvh, row, t, pos, table, pages, num_pages, page_size, num_heads, num_kv_heads, window,
                          scale_log2, part_o, part_ml, counters, out, status, prologue);
}

// The merge as a launch of its own (used when no counters are given): one warp per (row, head).
__global__ void __launch_bounds__(128)
attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         const int* __restrict__ rows, int num_rows, int num_heads, int num_splits,
                         int head_dim, bf16* __restrict__ out) {
    __shared__ float wbuf[4][MAX_SPLITS];
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= num_rows * num_heads) return;
    const int row = item / num_heads, h = item % num_heads;
    const int t = rows ? rows[row] : row;
    const size_t base[1] = {(size_t)item * num_splits};
    bf16* const dst[1] = {out + ((size_t)t * num_heads + h) * head_dim};
    merge_heads<1>(part_o, part_ml, base, num_splits, head_dim, dst, lane, wbuf[threadIdx.x >> 5]);
}

template <int HD>
int launch_decode(const bf16* q, const int* rows, int num_rows, const int* positions,
                  const int* req_of_tok, const int* block_table, int bt_stride, const bf16* pages,
                  int num_pages, int page_size, int num_heads, int num_kv_heads, int window,
                  float scale, int num_splits, float* part_o, float* part_ml, unsigned* counters,
                  bf16* out, int* status, int late_wait, cudaStream_t s) {
    constexpr int SMEM = STAGES * 2 * TILE * (HD * 2 + 16);
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, false>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_decode_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return ti_fail("attn_decode: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid(num_splits, num_kv_heads, num_rows);
    const bool single = num_splits == 1 && counters != nullptr;     // nothing to merge: the kernel without that code
#define LAUNCH(KERNEL)                                                                                   \
    ti_launch_pdl(KERNEL, grid, 32, SMEM, s, q, rows, positions, req_of_tok, block_table, bt_stride, pages, \
                  num_pages, page_size, num_heads, num_kv_heads, window, scale * LOG2E, part_o, part_ml,    \
                  counters, out, status)
    if (late_wait) {
        if constexpr (HD == 128) {
            static TiPerDevice late_configured;
            if (late_configured.first_use()) {
                cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, false, true>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
                if (e == cudaSuccess)
                    e = cudaFuncSetAttribute(attn_decode_kernel<HD, true, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
                if (e != cudaSuccess) return ti_fail("attn_decode: %s", cudaGetErrorString(e));
                late_configured.mark();
            }
            if (single) LAUNCH((attn_decode_kernel<HD, true, true>));
            else LAUNCH((attn_decode_kernel<HD, false, true>));
        } else {
            return ti_fail("attn_decode: a late wait is built for head_dim 128 only, not %d", HD);
        }
    } else if (single) {
        LAUNCH((attn_decode_kernel<HD, true>));
    } else {
        LAUNCH((attn_decode_kernel<HD, false>));
    }
#undef LAUNCH
    if (int rc = ti_check_launch("attn_decode")) return rc;
    if (counters) return 0;
    attn_decode_merge_kernel<<<(num_rows * num_heads + 3) / 4, 128, 0, s>>>(
        part_o, part_ml, rows, num_rows, num_heads, num_splits, HD, out);
    return ti_check_launch("attn_decode_merge");
}

}  // namespace

template <int HD>
int launch_decode_qkv(const float* qkv, int width, const float* q_weight, const float* k_weight, float eps,
                      const float* inv_freq, const int* rows, int num_rows, const int* positions,
                      const int* req_of_tok, const int* block_table, int bt_stride, bf16* pages, int num_pages,
                      int page_size, int write_kv, int num_heads, int num_kv_heads, int window, float scale,
                      int num_splits, float* part_o, float* part_ml, unsigned* counters, bf16* out,
                      int* status, cudaStream_t s) {
    constexpr int SMEM = item_smem_bytes<HD>() + QKV_MAX_GROUP * HD * 2 + 2 * HD * 2;
    static TiPerDevice configured;
    if (configured.first_use()) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_qkv_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return ti_fail("attn_decode_qkv: %s", cudaGetErrorString(e));
        configured.mark();
    }
    dim3 grid(num_splits, num_kv_heads, num_rows);
    ti_launch_pdl(attn_decode_qkv_kernel<HD>, grid, 32, SMEM, s, qkv, width, q_weight, k_weight, eps, inv_freq,
                  rows, positions, req_of_tok, block_table, bt_stride, pages, num_pages, page_size, write_kv,
                  num_heads, num_kv_heads, window, scale * LOG2E, part_o, part_ml, counters, out, status);
    return ti_check_launch("attn_decode_qkv");
}

// How many of the kernel's one-warp blocks fit on an SM (by shared memory), for sizing the grid.
extern "C" int ti_attn_decode_blocks_per_sm(int head_dim) {
    const int smem = STAGES * 2 * TILE * (head_dim * 2 + 16) + 1024;
    const int fit = (227 * 1024) / smem;
    return fit > 16 ? 16 : fit;
}

// 1 if (head_dim, heads per kv head, page_size) can run on this kernel, else 0.
extern "C" int ti_attn_decode_supported(int head_dim, int group, int page_size) {
    return head_dim >= 16 && head_dim <= 128 && head_dim % 16 == 0 && group >= 1 && group <= 16 &&
           page_size >= 16 && page_size % 16 == 0;
}

// Scratch the caller provides: part_o [num_rows, num_heads, num_splits, head_dim] float32 and
// part_ml [num_rows, num_heads, num_splits, 2] float32.  `counters` is either null (the splits are
// then merged by a second launch) or num_rows * num_kv_heads unsigned integers that are zero
// before the first launch: the last block of a (row, kv head) merges in the same launch and
// leaves its counter at zero again.
extern "C" int ti_attn_decode_fused(const void* q, const int* rows, int num_rows, const int* positions,
                                    const int* req_of_tok, const int* block_table, int bt_stride,
                                    const void* pages, int num_pages, int page_size, int num_heads,
                                    int num_kv_heads, int head_dim, int window, float scale,
                                    int num_splits, float* part_o, float* part_ml,
                                    unsigned* counters, void* out, int* status, int late_wait, void* stream);

extern "C" int ti_attn_decode(const void* q, const int* rows, int num_rows, const int* positions,
                              const int* req_of_tok, const int* block_table, int bt_stride,
                              const void* pages, int num_pages, int page_size, int num_heads,
                              int num_kv_heads, int head_dim, int window, float scale,
                              int num_splits, float* part_o, float* part_ml, void* out,
                              int* status, void* stream) {
    return ti_attn_decode_fused(q, rows, num_rows, positions, req_of_tok, block_table, bt_stride,
                                pages, num_pages, page_size, num_heads, num_kv_heads, head_dim,
                                window, scale, num_splits, part_o, part_ml, nullptr, out, status, 0,
                                stream);
}

extern "C" int ti_attn_decode_fused(const void* q, const int* rows, int num_rows, const int* positions,
                                    const int* req_of_tok, const int* block_table, int bt_stride,
                                    const void* pages, int num_pages, int page_size, int num_heads,
                                    int num_kv_heads, int head_dim, int window, float scale,
                                    int num_splits, float* part_o, float* part_ml,
                                    unsigned* counters, void* out, int* status, int late_wait, void* stream) {
    if (num_rows == 0) return 0;
    TI_REQUIRE(!late_wait || counters != nullptr, "attn_decode: a late wait needs the merge in the same launch");
    TI_REQUIRE(num_heads % num_kv_heads == 0, "attn_decode: %d heads over %d kv heads", num_heads,
               num_kv_heads);
    TI_REQUIRE(ti_attn_decode_supported(head_dim, num_heads / num_kv_heads, page_size),
               "attn_decode: head_dim %d (multiple of 16 up to 128), %d heads per kv head (up to 16) "
               "or page size %d (multiple of 16) is not supported",
               head_dim, num_heads / num_kv_heads, page_size);
    TI_REQUIRE(num_splits >= 1 && num_splits <= MAX_SPLITS && num_rows <= 65535 && num_kv_heads <= 65535,
               "attn_decode: grid out of range (at most %d splits)", MAX_SPLITS);
#define CASE(HD)                                                                                   \
    case HD:                                                                                       \
        return launch_decode<HD>((const bf16*)q, rows, num_rows, positions, req_of_tok,            \
                                 block_table, bt_stride, (const bf16*)pages, num_pages, page_size, \
                                 num_heads, num_kv_heads, window, scale, num_splits, part_o,       \
                                 part_ml, counters, (bf16*)out, status, late_wait, (cudaStream_t)stream)
    switch (head_dim) {
        CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
    }
#undef CASE
    return ti_fail("attn_decode: head_dim %d", head_dim);
}

// 1 if flash-decoding can start from the float32 QKV product for these sizes.
extern "C" int ti_attn_decode_qkv_supported(int head_dim, int group, int page_size) {
    return (head_dim == 64 || head_dim == 128) && group >= 1 && group <= QKV_MAX_GROUP && page_size >= 16 &&
           page_size % 16 == 0;
}

// Flash-decoding of single-token rows from their float32 QKV product `qkv` [tokens, width] (query
// heads, key heads, value heads): head norm, NeoX rotation over the whole head, the store of the
// new key and value (if `write_kv`) and the attention in one launch.  Scratch and counters as
// for ti_attn_decode_fused (the counters are required).
extern "C" int ti_attn_decode_qkv(const float* qkv, int width, const float* q_weight, const float* k_weight,
                                  float eps, const float* inv_freq, const int* rows, int num_rows,
                                  const int* positions, const int* req_of_tok, const int* block_table,
                                  int bt_stride, void* pages, int num_pages, int page_size, int write_kv,
                                  int num_heads, int num_kv_heads, int head_dim, int window, float scale,
                                  int num_splits, float* part_o, float* part_ml, unsigned* counters, void* out,
                                  int* status, void* stream) {
    if (num_rows == 0) return 0;
    TI_REQUIRE(num_kv_heads >= 1 && num_heads % num_kv_heads == 0, "attn_decode_qkv: %d heads over %d kv heads",
               num_heads, num_kv_heads);
    TI_REQUIRE(ti_attn_decode_qkv_supported(head_dim, num_heads / num_kv_heads, page_size),
               "attn_decode_qkv: head_dim %d (64 or 128), %d heads per kv head (up to %d) or page size %d "
               "(multiple of 16) is not supported", head_dim, num_heads / num_kv_heads, QKV_MAX_GROUP, page_size);
    TI_REQUIRE(width == (num_heads + 2 * num_kv_heads) * head_dim, "attn_decode_qkv: width %d", width);
    TI_REQUIRE(counters != nullptr, "attn_decode_qkv: the merge needs its counters");
    TI_REQUIRE(num_splits >= 1 && num_splits <= MAX_SPLITS && num_rows <= 65535 && num_kv_heads <= 65535,
               "attn_decode_qkv: grid out of range (at most %d splits)", MAX_SPLITS);
#define CASE(HD)                                                                                             \
    case HD:                                                                                                 \
        return launch_decode_qkv<HD>(qkv, width, q_weight, k_weight, eps, inv_freq, rows, num_rows, positions, \
                                     req_of_tok, block_table, bt_stride, (bf16*)pages, num_pages, page_size, \
                                     write_kv, num_heads, num_kv_heads, window, scale, num_splits, part_o,   \
                                     part_ml, counters, (bf16*)out, status, (cudaStream_t)stream)
    switch (head_dim) {
        CASE(64); CASE(128);
    }
#undef CASE
    return ti_fail("attn_decode_qkv: head_dim %d", head_dim);
}

// ---- the variant that allocates nothing (declared and described in attn_decode_noalloc.h) ----
#include "attn_decode_noalloc.h"

#include <mutex>

namespace {

// The partial results of the key splits live here instead of in caller-provided buffers.
static __device__ __align__(256) unsigned char g_noalloc_scratch[TI_DECODE_NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
void* g_noalloc_ptr[MAX_DEVICES] = {};        // device address of the array, per device
std::mutex g_noalloc_mutex;

// In host code the array's name is only a handle: the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device while that device is current.
int noalloc_scratch(void** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return ti_fail("attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return ti_fail("attn_decode_noalloc: device %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return ti_fail("attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_noalloc_ptr[dev] = p;
    }
    *ptr = g_noalloc_ptr[dev];
    return 0;
}

}  // namespace

extern "C" int ti_attn_decode_noalloc(const void* q, const int* rows, int num_rows,
                                      const int* positions, const int* req_of_tok,
                                      const int* block_table, int bt_stride, const void* pages,
                                      int num_pages, int page_size, int num_heads, int num_kv_heads,
                                      int head_dim, int window, float scale, int num_splits,
                                      void* out, int* status, void* stream) {
    if (num_rows == 0) return 0;
    TI_REQUIRE(num_rows > 0 && num_heads > 0 && num_splits > 0 && head_dim > 0,
               "attn_decode_noalloc: sizes must be positive");
    const unsigned long long slots = (unsigned long long)num_rows * num_heads * num_splits;
    const unsigned long long need = slots * (unsigned long long)(head_dim + 2) * sizeof(float);
    TI_REQUIRE(need <= TI_DECODE_NOALLOC_SCRATCH_BYTES,
               "attn_decode_noalloc: %d rows x %d heads x %d splits x head_dim %d need %llu bytes of "
               "scratch; the built-in array holds %u",
               num_rows, num_heads, num_splits, head_dim, need, TI_DECODE_NOALLOC_SCRATCH_BYTES);
    void* base = nullptr;
    if (int rc = noalloc_scratch(&base)) return rc;
    float* part_o = (float*)base;                                   // [slots, head_dim]
    float* part_ml = part_o + slots * (unsigned long long)head_dim; // [slots, 2]
    return ti_attn_decode(q, rows, num_rows, positions, req_of_tok, block_table, bt_stride, pages,
                          num_pages, page_size, num_heads, num_kv_heads, head_dim, window, scale,
                          num_splits, part_o, part_ml, out, status, stream);
}
