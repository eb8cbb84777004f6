// TEST INFRASTRUCTURE ONLY — part of the CPU oracle, never linked into the product library.
//
// Software bf16 / f16 with the semantics of the `half` crate (version 2.6.x, the
// dependency the reference pins in Cargo.toml:19 and which is not vendored in the
// reference tree): every arithmetic operator converts both operands to f32,
// operates in f32 and rounds the result back with round-to-nearest-even; comparisons
// follow IEEE-754 (NaN unordered, +0 == -0); negation flips the sign bit.
// Call sites this stands in for: every `bf16` / `f16` lambda in
// crates/maidenx_cpu/src/ops/binary.rs:372-373, ops/unary.rs:131-132,
// ops/reduction.rs:555-556, ops/matmul.rs:281-282, nn/conv.rs:156-157.
#pragma once
#include <cstdint>
#include <cstring>

namespace mxo {

static inline uint32_t f32_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}
static inline float bits_f32(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

struct bf16 {
    uint16_t bits;
    bf16() : bits(0) {}
    static bf16 from_bits(uint16_t b) {
        bf16 r;
        r.bits = b;
        return r;
    }
    // Round-to-nearest-even on the upper 16 bits; a NaN keeps its sign and upper
    // payload and gets the quiet bit so it cannot collapse to infinity.
    static bf16 from_f32(float f) {
        uint32_t x = f32_bits(f);
        if ((x & 0x7FFFFFFFu) > 0x7F800000u) return from_bits((uint16_t)((x >> 16) | 0x0040u));
        uint32_t round_bit = 0x00008000u;
        if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return from_bits((uint16_t)((x >> 16) + 1));
        return from_bits((uint16_t)(x >> 16));
    }
    float to_f32() const { return bits_f32((uint32_t)bits << 16); }
};

struct f16 {
    uint16_t bits;
    f16() : bits(0) {}
    static f16 from_bits(uint16_t b) {
        f16 r;
        r.bits = b;
        return r;
    }
    static f16 from_f32(float f) {
        uint32_t x = f32_bits(f);
        uint32_t sign = x & 0x80000000u;
        uint32_t exp = x & 0x7F800000u;
        uint32_t man = x & 0x007FFFFFu;
        if (exp == 0x7F800000u) {
            uint32_t nan_bit = man == 0 ? 0 : 0x0200u;
            return from_bits((uint16_t)((sign >> 16) | 0x7C00u | nan_bit | (man >> 13)));
        }
        uint32_t half_sign = sign >> 16;
        int32_t unbiased = (int32_t)(exp >> 23) - 127;
        int32_t half_exp = unbiased + 15;
        if (half_exp >= 0x1F) return from_bits((uint16_t)(half_sign | 0x7C00u));
        if (half_exp <= 0) {
            if (14 - half_exp > 24) return from_bits((uint16_t)half_sign);
            man |= 0x00800000u;
            uint32_t half_man = man >> (14 - half_exp);
            uint32_t round_bit = 1u << (13 - half_exp);
            if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0) half_man += 1;
            return from_bits((uint16_t)(half_sign | half_man));
        }
        uint32_t he = (uint32_t)half_exp << 10;
        uint32_t half_man = man >> 13;
        uint32_t round_bit = 0x00001000u;
        if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0)
            return from_bits((uint16_t)((half_sign | he | half_man) + 1));
        return from_bits((uint16_t)(half_sign | he | half_man));
    }
    float to_f32() const {
        uint32_t h = bits;
        uint32_t sign = (h & 0x8000u) << 16;
        uint32_t exp = (h >> 10) & 0x1Fu;
        uint32_t man = h & 0x03FFu;
        if (exp == 0) {
            if (man == 0) return bits_f32(sign);
            // subnormal: normalise
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x0400u) == 0);
            man &= 0x03FFu;
            return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13));
        }
        if (exp == 0x1F) return bits_f32(sign | 0x7F800000u | (man << 13));
        return bits_f32(sign | ((exp + 127 - 15) << 23) | (man << 13));
    }
};

#define MXO_HALF_OPS(H)                                                                    \
    static inline H operator+(H a, H b) { return H::from_f32(a.to_f32() + b.to_f32()); }   \
    static inline H operator-(H a, H b) { return H::from_f32(a.to_f32() - b.to_f32()); }   \
    static inline H operator*(H a, H b) { return H::from_f32(a.to_f32() * b.to_f32()); }   \
    static inline H operator/(H a, H b) { return H::from_f32(a.to_f32() / b.to_f32()); }   \
    static inline H operator-(H a) { return H::from_bits((uint16_t)(a.bits ^ 0x8000u)); }  \
    static inline bool operator==(H a, H b) { return a.to_f32() == b.to_f32(); }           \
    static inline bool operator!=(H a, H b) { return a.to_f32() != b.to_f32(); }           \
    static inline bool operator<(H a, H b) { return a.to_f32() < b.to_f32(); }             \
    static inline bool operator<=(H a, H b) { return a.to_f32() <= b.to_f32(); }           \
    static inline bool operator>(H a, H b) { return a.to_f32() > b.to_f32(); }             \
    static inline bool operator>=(H a, H b) { return a.to_f32() >= b.to_f32(); }           \
    static inline H& operator+=(H& a, H b) {                                               \
        a = a + b;                                                                         \
        return a;                                                                          \
    }
MXO_HALF_OPS(bf16)
MXO_HALF_OPS(f16)
#undef MXO_HALF_OPS

}  // namespace mxo
