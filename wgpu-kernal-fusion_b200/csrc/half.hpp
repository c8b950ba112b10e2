// Host-side f16 / bf16 conversions (round to nearest even), used for immediates of 16-bit
// chains and for `arange` on 16-bit tensors.
#pragma once
#include <cstdint>
#include <cstring>

namespace wgf {

inline uint32_t f32_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
inline float bits_f32(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

inline uint16_t f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | (ax > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to >= 65520 -> inf
    if (ax < 0x38800000u) {                                    // subnormal or zero in f16
        if (ax < 0x33000000u) return (uint16_t)sign;           // < 2^-25 -> 0
        uint32_t exp = ax >> 23;
        uint32_t man = (ax & 0x7fffffu) | 0x800000u;
        uint32_t shift = 126 - exp;  // 14..24
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((ax - 0x38000000u) >> 13);
    uint32_t rem = ax & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}

inline float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        int e = -1;
        do {
            man <<= 1;
            e++;
        } while (!(man & 0x400u));
        return bits_f32(sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3ffu) << 13));
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112) << 23) | (man << 13));
}

inline uint16_t f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}
inline float bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

}  // namespace wgf
