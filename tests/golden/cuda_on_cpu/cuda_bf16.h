// A stand-in for <cuda_bf16.h>: bfloat16 as 16 stored bits, converted with round-to-nearest-even.
#pragma once

#include <cstdint>
#include <cstring>

struct __nv_bfloat16 {
    uint16_t bits;
};

static inline __nv_bfloat16 __float2bfloat16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    __nv_bfloat16 r;
    if ((u & 0x7fffffffu) > 0x7f800000u) {          // NaN stays NaN
        r.bits = 0x7fff;
        return r;
    }
    u += 0x7fffu + ((u >> 16) & 1u);                // to nearest, ties to even
    r.bits = (uint16_t)(u >> 16);
    return r;
}
static inline float __bfloat162float(__nv_bfloat16 v) {
    const uint32_t u = (uint32_t)v.bits << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static inline unsigned short __bfloat16_as_ushort(__nv_bfloat16 v) { return v.bits; }
