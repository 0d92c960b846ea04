// Host-side scalar conversions between the 13 element types and double / int64. bf16 and f16 round to
// nearest even (the reference's buffer packing does the same for bf16:
// Sources/MetalHLOCore/Runtime/BufferStorage.swift:332-346).
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>

#include "ir.h"

namespace mhlo {

inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
inline float bf16_bits_to_f32(uint16_t h) {
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_f16_bits(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return static_cast<uint16_t>(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
    if (x >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return static_cast<uint16_t>(sign | 0x7c00u);
    }
    if (x < 0x38800000u) {  // subnormal half or zero
        if (x < 0x33000000u) return static_cast<uint16_t>(sign);
        const int shift = 113 - static_cast<int>(x >> 23);
        uint32_t mant = (x & 0x7fffffu) | 0x800000u;
        uint32_t half = mant >> (shift + 13);
        const uint32_t rem = mant & ((1u << (shift + 13)) - 1);
        const uint32_t halfway = 1u << (shift + 12);
        if (rem > halfway || (rem == halfway && (half & 1))) ++half;
        return static_cast<uint16_t>(sign | half);
    }
    uint32_t half = ((x - 0x38000000u) >> 13);
    const uint32_t rem = x & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
}
inline float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (static_cast<uint32_t>(h) & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, mant = h & 0x3ffu, u;
    if (exp == 0) {
        if (mant == 0) u = sign;
        else {
            int e = -1;
            do { ++e; mant <<= 1; } while (!(mant & 0x400u));
            u = sign | ((112 - e) << 23) | ((mant & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (mant << 13);
    } else {
        u = sign | ((exp + 112) << 23) | (mant << 13);
    }
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// Writes `v` as one element of floating type t.
inline void encode_float(DType t, double v, uint8_t* dst) {
    switch (t) {
        case DType::F64: std::memcpy(dst, &v, 8); break;
        case DType::F32: { float f = static_cast<float>(v); std::memcpy(dst, &f, 4); break; }
        case DType::F16: { uint16_t h = f32_to_f16_bits(static_cast<float>(v)); std::memcpy(dst, &h, 2); break; }
        case DType::BF16: { uint16_t h = f32_to_bf16_bits(static_cast<float>(v)); std::memcpy(dst, &h, 2); break; }
        default: break;
    }
}

// Reads one element of any type as a double (exact for every type except 64-bit integers above 2^53).
inline double decode_as_double(DType t, const uint8_t* src) {
    switch (t) {
        case DType::F64: { double v; std::memcpy(&v, src, 8); return v; }
        case DType::F32: { float v; std::memcpy(&v, src, 4); return v; }
        case DType::F16: { uint16_t h; std::memcpy(&h, src, 2); return f16_bits_to_f32(h); }
        case DType::BF16: { uint16_t h; std::memcpy(&h, src, 2); return bf16_bits_to_f32(h); }
        case DType::I1: return src[0] ? 1.0 : 0.0;
        case DType::I8: return static_cast<int8_t>(src[0]);
        case DType::UI8: return src[0];
        case DType::I16: { int16_t v; std::memcpy(&v, src, 2); return v; }
        case DType::UI16: { uint16_t v; std::memcpy(&v, src, 2); return v; }
        case DType::I32: { int32_t v; std::memcpy(&v, src, 4); return v; }
        case DType::UI32: { uint32_t v; std::memcpy(&v, src, 4); return v; }
        case DType::I64: { int64_t v; std::memcpy(&v, src, 8); return static_cast<double>(v); }
        case DType::UI64: { uint64_t v; std::memcpy(&v, src, 8); return static_cast<double>(v); }
    }
    return 0;
}

inline int64_t decode_as_int(DType t, const uint8_t* src) {
    switch (t) {
        case DType::I64: case DType::UI64: { int64_t v; std::memcpy(&v, src, 8); return v; }
        default: return static_cast<int64_t>(decode_as_double(t, src));
    }
}

// Writes a scalar given as double (floats) or int64 (integers) in element type t.
inline void encode_scalar(DType t, double f, int64_t i, uint8_t* dst) {
    if (is_float(t)) { encode_float(t, f, dst); return; }
    if (t == DType::I1) { dst[0] = i != 0; return; }
    std::memcpy(dst, &i, dtype_size(t));
}

}  // namespace mhlo
