// Row-wise kernels: token embedding, RMSNorm (optionally of gathered rows), SwiGLU, argmax.
// All arithmetic is float32; results are rounded once to the output type.
#include "common.cuh"

namespace {

// x[t, :] = float32(table[token[t], :])
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             int hidden, float* __restrict__ out) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const TW* row = table + (size_t)tokens[t] * hidden;
    float* o = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
}

// out[r, :] = x[src(r), :] * (1 / sqrt(mean(x^2) + eps)) * w, src(r) = rows ? rows[r] : r
template <typename TO>
__global__ void rmsnorm_kernel(const float* x, const float* __restrict__ w,
                               const int* __restrict__ rows, float eps, int n,
                               TO* __restrict__ out) {
    __shared__ float scratch[32];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * n;
    TO* o = out + (size_t)r * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    const float mean = block_sum(ss, scratch) / (float)n;
    const float inv = 1.0f / sqrtf(mean + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_f32<TO>(xr[i] * inv * w[i]);
}

// The same norm with one warp per row and 16-byte accesses, for row lengths that are multiples
// of 4: no shared memory, no block barrier; the second pass reads the row from L1.
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const float* x, const float* __restrict__ w,
                    const int* __restrict__ rows, float eps, int n, int num_rows,
                    TO* __restrict__ out) {
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= num_rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * n);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const int n4 = n >> 2;
    float ss = 0.0f;
    for (int i = lane; i < n4; i += 32) {
        const float4 v = xr[i];
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
        ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
    TO* o = out + (size_t)r * n;
    for (int i = lane; i < n4; i += 32) {
        const float4 v = xr[i], g = w4[i];
        if constexpr (sizeof(TO) == 2) {
            __nv_bfloat162 a = __floats2bfloat162_rn(v.x * inv * g.x, v.y * inv * g.y);
            __nv_bfloat162 b = __floats2bfloat162_rn(v.z * inv * g.z, v.w * inv * g.w);
            uint2 pk = make_uint2(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b));
            *reinterpret_cast<uint2*>(o + 4 * i) = pk;
        } else {
            *reinterpret_cast<float4*>(o + 4 * i) =
                make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
        }
    }
}

// The warp-per-row norm for rows of at most 2,048 elements: a lane keeps its up to sixteen 16-byte
// pieces in registers, so the row is read once and all its loads are in flight together.  The sum
// of squares runs in the same order as in rmsnorm_warp_kernel.
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_warp_reg_kernel(const float* x, const float* __restrict__ w,
                        const int* __restrict__ rows, float eps, int n, int num_rows,
                        TO* __restrict__ out) {
    constexpr int MAXV = 16;
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= num_rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * n);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const int n4 = n >> 2;
    float4 v[MAXV];
#pragma unroll
    for (int j = 0; j < MAXV; ++j)
        if (lane + 32 * j < n4) v[j] = xr[lane + 32 * j];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        if (lane + 32 * j < n4) {
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
    TO* o = out + (size_t)r * n;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = lane + 32 * j;
        if (i >= n4) continue;
        const float4 g = w4[i];
        const float4 y = make_float4(v[j].x * inv * g.x, v[j].y * inv * g.y, v[j].z * inv * g.z,
                                     v[j].w * inv * g.w);
        if constexpr (sizeof(TO) == 2) {
            __nv_bfloat162 a = __floats2bfloat162_rn(y.x, y.y), b = __floats2bfloat162_rn(y.z, y.w);
            *reinterpret_cast<uint2*>(o + 4 * i) =
                make_uint2(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b));
        } else {
            *reinterpret_cast<float4*>(o + 4 * i) = y;
        }
    }
}

// The same norm with one block per row for few rows whose length is a multiple of 4 and at most
// 16 * THREADS: a thread keeps its up to four 16-byte pieces of the row in registers, so the row
// is read once and all loads are in flight together; the weights are fetched before the wait on
// the previous kernel.
//
// With `ws` (rows == null): the row is first completed from the slabs of a product whose K was cut
// into `runs` (gemm_tcgen05.cu): x[r] = (accumulate ? x[r] : 0) + (ws[0][r] + ws[1][r] + ...), the
// slabs added in ascending order as that product's own adding launch does, and written back; the
// norm is then of the completed row (one launch and one pass over the rows less).
template <typename TO, int THREADS, bool ADD_RUNS = false, int PIECES = 4>
__global__ void __launch_bounds__(THREADS)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows,
                   float eps, int n, TO* __restrict__ out, const float* ws, int runs,
                   size_t slab, int accumulate) {
    __shared__ float scratch[32];
    pdl_launch();
    const int n4 = n >> 2;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4 g[PIECES], v[PIECES];
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i < n4) g[j] = w4[i];
    }
    pdl_wait();
    const int r = blockIdx.x;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)(rows ? rows[r] : r) * n);
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i < n4) v[j] = !ADD_RUNS || accumulate ? xr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if constexpr (ADD_RUNS) {
        const float4* part = reinterpret_cast<const float4*>(ws + (size_t)r * n);
#pragma unroll
        for (int j = 0; j < PIECES; ++j) {
            const int i = threadIdx.x + j * THREADS;
            if (i >= n4) continue;
            float4 sum = __ldcg(part + i);
            for (int k = 1; k < runs; ++k) {
                const float4 p = __ldcg(reinterpret_cast<const float4*>(ws + k * slab + (size_t)r * n) + i);
                sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
            }
            v[j] = make_float4(v[j].x + sum.x, v[j].y + sum.y, v[j].z + sum.z, v[j].w + sum.w);
            xr[i] = v[j];
        }
    }
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        if (threadIdx.x + j * THREADS < n4) {
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    TO* o = out + (size_t)r * n;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i >= n4) continue;
        const float4 y = make_float4(v[j].x * inv * g[j].x, v[j].y * inv * g[j].y, v[j].z * inv * g[j].z,
                                     v[j].w * inv * g[j].w);
        if constexpr (sizeof(TO) == 2) {
            __nv_bfloat162 a = __floats2bfloat162_rn(y.x, y.y), b = __floats2bfloat162_rn(y.z, y.w);
            *reinterpret_cast<uint2*>(o + 4 * i) =
                make_uint2(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b));
        } else {
            *reinterpret_cast<float4*>(o + 4 * i) = y;
        }
    }
}

// y[t, j] = silu(gate_j) * up_j, silu(g) = g / (1 + exp(-g)).  Stacked layout: gate_j = gu[t, j],
// up_j = gu[t, inter + j].  Interleaved layout (groups of 8 gate columns followed by their 8 up
// columns): gate_j = gu[t, 16 (j / 8) + j % 8], up_j eight columns further.
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, int inter, size_t total,
                              int interleaved, TO* __restrict__ y) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / inter, j = i % inter;
    const size_t gcol = interleaved ? (j / 8) * 16 + j % 8 : j;
    const float g = gu[t * 2 * inter + gcol];
    const float u = gu[t * 2 * inter + gcol + (interleaved ? 8 : inter)];
    y[i] = from_f32<TO>(g / (1.0f + expf(-g)) * u);
}

__device__ __forceinline__ void keep_best(float v, int i, float& bv, int& bi) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

// Row argmax; among equal maxima the lowest index wins.
__global__ void argmax_kernel(const float* logits, int vocab, int* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) keep_best(row[i], i, bv, bi);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        keep_best(ov, oi, bv, bi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            keep_best(ov, oi, bv, bi);
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// Argmax in two steps for wide rows: blocks take slices of a row and leave their best (value,
// index); one more small launch picks among the slices.  Ties still go to the lowest index.
constexpr int ARGMAX_SLICES = 64;

__global__ void __launch_bounds__(256)
argmax_slice_kernel(const float* logits, int vocab, float* __restrict__ part_v,
                    int* __restrict__ part_i) {
    __shared__ float sv[8];
    __shared__ int si[8];
    const int row = blockIdx.y, slice = blockIdx.x;
    const int per = (vocab + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int lo = slice * per, hi = min(vocab, lo + per);
    const float* x = logits + (size_t)row * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += 256) keep_best(x[i], i, bv, bi);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        keep_best(ov, oi, bv, bi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) keep_best(sv[w], si[w], bv, bi);
        part_v[row * ARGMAX_SLICES + slice] = bv;
        part_i[row * ARGMAX_SLICES + slice] = bi;
    }
}

__global__ void __launch_bounds__(ARGMAX_SLICES)
argmax_pick_kernel(const float* part_v, const int* part_i,
                   int* __restrict__ out) {
    __shared__ float sv[2];
    __shared__ int si[2];
    const int row = blockIdx.x;
    float bv = part_v[row * ARGMAX_SLICES + threadIdx.x];
    int bi = part_i[row * ARGMAX_SLICES + threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        keep_best(ov, oi, bv, bi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        keep_best(sv[1], si[1], bv, bi);
        out[row] = bi == 0x7fffffff ? 0 : bi;
    }
}

}  // namespace

// Scratch for the two-step argmax: rows * 64 floats and rows * 64 ints.
extern "C" int ti_argmax_sliced(const float* logits, int rows, int vocab, float* part_v, int* part_i,
                                int* out, void* stream) {
    if (rows == 0) return 0;
    TI_REQUIRE(vocab > 0 && rows <= 65535, "argmax: %d rows of %d", rows, vocab);
    cudaStream_t s = (cudaStream_t)stream;
    argmax_slice_kernel<<<dim3(ARGMAX_SLICES, rows), 256, 0, s>>>(logits, vocab, part_v, part_i);
    if (int rc = ti_check_launch("argmax")) return rc;
    argmax_pick_kernel<<<rows, ARGMAX_SLICES, 0, s>>>(part_v, part_i, out);
    return ti_check_launch("argmax");
}

extern "C" int ti_embed(const void* table, int table_dtype, const int* tokens, int num_tokens,
                        int hidden, float* out, void* stream) {
    if (num_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == TI_BF16)
        ti_launch_pdl(embed_kernel<bf16>, num_tokens, 256, 0, s, (const bf16*)table, tokens, hidden, out);
    else if (table_dtype == TI_F32)
        ti_launch_pdl(embed_kernel<float>, num_tokens, 256, 0, s, (const float*)table, tokens, hidden, out);
    else
        return ti_fail("embed: table dtype code %d is not float32 or bfloat16", table_dtype);
    return ti_check_launch("embed");
}

extern "C" int ti_rmsnorm(const float* x, const float* weight, const int* rows, int num_rows,
                          int n, float eps, void* out, int out_dtype, void* stream) {
    if (num_rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    // A float32 result is the 32-bit path: there the kernel, and with it the order in which a
    // row's squares are added, must not depend on how many rows the step happens to bring, so
    // that a token's bits are the same however the tokens are cut into steps.  Only the
    // bfloat16 path picks the warp-per-row kernels for many rows.
    // (A warp per row pays from about a thousand rows on: 64 rows as 8 blocks of 8 warps left
    // most of the GPU idle, 21 against 2 microseconds at a row length of 5,120.)
    if (n % 4 == 0 && num_rows >= 1024 && out_dtype == TI_BF16 &&
        (uintptr_t)x % 16 == 0 && (uintptr_t)weight % 16 == 0 && (uintptr_t)out % 16 == 0) {
        // many rows: a warp per row.  (Fewer rows keep a block per row: more threads per row.)
        const unsigned grid = (unsigned)((num_rows + 7) / 8);
        if (n <= 2048)
            ti_launch_pdl(rmsnorm_warp_reg_kernel<bf16>, grid, 256, 0, s, x, weight, rows, eps, n, num_rows, (bf16*)out);
        else
            ti_launch_pdl(rmsnorm_warp_kernel<bf16>, grid, 256, 0, s, x, weight, rows, eps, n, num_rows, (bf16*)out);
        return ti_check_launch("rmsnorm");
    }
    if (n % 4 == 0 && n <= 16 * 1024 && (out_dtype == TI_BF16 || out_dtype == TI_F32) &&
        (uintptr_t)x % 16 == 0 && (uintptr_t)weight % 16 == 0 && (uintptr_t)out % 16 == 0) {
        // few rows: a block per row that keeps the row in registers
        const bool small = n <= 16 * 256;
        if (out_dtype == TI_BF16 && n <= 4 * 256)
            // one piece of the row per thread (the same sums in the same order: the other pieces
            // are empty): the short kernel a small model's decode step waits for twice a layer
            ti_launch_pdl(rmsnorm_vec_kernel<bf16, 256, false, 1>, num_rows, 256, 0, s, (float*)x, weight, rows, eps, n,
                          (bf16*)out, (const float*)nullptr, 0, (size_t)0, 0);
        else if (out_dtype == TI_BF16 && small)
            ti_launch_pdl(rmsnorm_vec_kernel<bf16, 256>, num_rows, 256, 0, s, (float*)x, weight, rows, eps, n, (bf16*)out,
                          (const float*)nullptr, 0, (size_t)0, 0);
        else if (out_dtype == TI_BF16)
            ti_launch_pdl(rmsnorm_vec_kernel<bf16, 1024>, num_rows, 1024, 0, s, (float*)x, weight, rows, eps, n, (bf16*)out,
                          (const float*)nullptr, 0, (size_t)0, 0);
        else if (small)
            ti_launch_pdl(rmsnorm_vec_kernel<float, 256>, num_rows, 256, 0, s, (float*)x, weight, rows, eps, n, (float*)out,
                          (const float*)nullptr, 0, (size_t)0, 0);
        else
            ti_launch_pdl(rmsnorm_vec_kernel<float, 1024>, num_rows, 1024, 0, s, (float*)x, weight, rows, eps, n, (float*)out,
                          (const float*)nullptr, 0, (size_t)0, 0);
        return ti_check_launch("rmsnorm");
    }
    const int threads = n >= 1024 ? 256 : 128;
    if (out_dtype == TI_BF16)
        ti_launch_pdl(rmsnorm_kernel<bf16>, num_rows, threads, 0, s, x, weight, rows, eps, n, (bf16*)out);
    else if (out_dtype == TI_F32)
        ti_launch_pdl(rmsnorm_kernel<float>, num_rows, threads, 0, s, x, weight, rows, eps, n, (float*)out);
    else
        return ti_fail("rmsnorm: output dtype code %d is not float32 or bfloat16", out_dtype);
    return ti_check_launch("rmsnorm");
}

// rmsnorm of rows that are first completed from the `runs` slabs ws[run][num_rows][n] of a
// product whose K was cut (see rmsnorm_vec_kernel); x is written.  Returns -1, launching nothing,
// for sizes this form does not take (the caller then adds and norms in turn).
extern "C" int ti_rmsnorm_merge(float* x, const float* ws, int runs, int accumulate, const float* weight,
                                int num_rows, int n, float eps, void* out, int out_dtype, void* stream) {
    if (num_rows == 0) return 0;
    if (!(n % 4 == 0 && n <= 16 * 1024 && out_dtype == TI_BF16 && num_rows < 1024 && runs >= 1 &&
          (uintptr_t)x % 16 == 0 && (uintptr_t)ws % 16 == 0 && (uintptr_t)weight % 16 == 0 &&
          (uintptr_t)out % 16 == 0))
        return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t slab = (size_t)num_rows * n;
    if (n <= 16 * 256)
        ti_launch_pdl(rmsnorm_vec_kernel<bf16, 256, true>, num_rows, 256, 0, s, x, weight, (const int*)nullptr, eps, n,
                      (bf16*)out, ws, runs, slab, accumulate);
    else
        ti_launch_pdl(rmsnorm_vec_kernel<bf16, 1024, true>, num_rows, 1024, 0, s, x, weight, (const int*)nullptr, eps, n,
                      (bf16*)out, ws, runs, slab, accumulate);
    return ti_check_launch("rmsnorm_merge");
}

extern "C" int ti_swiglu(const float* gu, int num_tokens, int inter, int interleaved, void* out,
                         int out_dtype, void* stream) {
    TI_REQUIRE(!interleaved || inter % 8 == 0, "swiglu: interleaved layout needs inter %% 8 == 0");
    const size_t total = (size_t)num_tokens * inter;
    if (total == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == TI_BF16)
        swiglu_kernel<bf16><<<blocks, 256, 0, s>>>(gu, inter, total, interleaved, (bf16*)out);
    else if (out_dtype == TI_F32)
        swiglu_kernel<float><<<blocks, 256, 0, s>>>(gu, inter, total, interleaved, (float*)out);
    else
        return ti_fail("swiglu: output dtype code %d is not float32 or bfloat16", out_dtype);
    return ti_check_launch("swiglu");
}

extern "C" int ti_argmax(const float* logits, int rows, int vocab, int* out, void* stream) {
    if (rows == 0) return 0;
    TI_REQUIRE(vocab > 0, "argmax: vocabulary size %d", vocab);
    argmax_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>(logits, vocab, out);
    return ti_check_launch("argmax");
}
