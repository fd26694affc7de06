// Seeded synthetic inputs, one definition for host and device: element `index` of tensor
// `tensor_id` under `seed` is a pure function of the three, so any slice of a 1 GiB operand can
// be regenerated anywhere. Arithmetic is integer up to at most one fp32 multiply, and the
// conversions to fp16 / bf16 are round-to-nearest-even written out on the bits, so host and
// device agree exactly. The reference seeds rand() from the clock (matmul_test.h:239, :328-339)
// and cannot be reproduced; this replaces it.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200 {
namespace synth {

B200_HD uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

B200_HD uint64_t key_of(uint64_t seed, uint64_t tensor_id) {
    return splitmix64(seed ^ (tensor_id * 0xD1B54A32D192ED03ull));
}

B200_HD uint64_t hash_of(uint64_t key, uint64_t index, uint64_t lane) {
    return splitmix64(key + index * 0x9E3779B97F4A7C15ull + lane * 0xC2B2AE3D27D4EB4Full);
}

B200_HD uint32_t float_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
#endif
}

// uniform in [-1, 1): 24 random bits b -> b * 2^-23 - 1; both steps are exact in fp32.
B200_HD float uniform(uint64_t key, uint64_t index) {
    const uint32_t b = static_cast<uint32_t>(hash_of(key, index, 0) >> 40);
#if defined(__CUDA_ARCH__)
    return __fadd_rn(__fmul_rn(static_cast<float>(b), 1.1920928955078125e-7f), -1.0f);
#else
    return static_cast<float>(b) * 1.1920928955078125e-7f - 1.0f;
#endif
}

// approximately normal(0, sigma): sum of twelve 16-bit uniforms, centred and scaled exactly,
// then one fp32 multiply by sigma. Support is +-6 sigma.
B200_HD float normal(uint64_t key, uint64_t index, float sigma) {
    int32_t s = 0;
    for (uint64_t lane = 1; lane <= 3; ++lane) {
        const uint64_t h = hash_of(key, index, lane);
        s += static_cast<int32_t>(h & 0xFFFF) + static_cast<int32_t>((h >> 16) & 0xFFFF) +
             static_cast<int32_t>((h >> 32) & 0xFFFF) + static_cast<int32_t>(h >> 48);
    }
#if defined(__CUDA_ARCH__)
    return __fmul_rn(__fmul_rn(static_cast<float>(s - 393210), 1.52587890625e-5f), sigma);
#else
    const float z = static_cast<float>(s - 393210) * 1.52587890625e-5f;
    return z * sigma;
#endif
}

B200_HD uint16_t to_half_bits(float f) {
    const uint32_t x = float_bits(f);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return static_cast<uint16_t>(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u : 0u));
    if (ax >= 0x477FF000u) return static_cast<uint16_t>(sign | 0x7C00u);
    if (ax < 0x33000001u) return static_cast<uint16_t>(sign);
    const int32_t e = static_cast<int32_t>(ax >> 23) - 127;
    const uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    const uint32_t shift = e < -14 ? static_cast<uint32_t>(13 + (-14 - e)) : 13u;
    const uint32_t hexp = e < -14 ? 0u : static_cast<uint32_t>(e + 15);
    uint32_t qv = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (qv & 1u))) ++qv;
    const uint32_t out = hexp == 0 ? qv : (((hexp - 1u) << 10) + qv);
    return static_cast<uint16_t>(sign | out);
}

B200_HD uint16_t to_bf16_bits(float f) {
    uint32_t x = float_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((x >> 16) | 0x40u);
    x += 0x7FFFu + ((x >> 16) & 1u);
    return static_cast<uint16_t>(x >> 16);
}

B200_HD float value(uint64_t key, uint64_t index, int dist, float sigma) {
    return dist ? normal(key, index, sigma) : uniform(key, index);
}

B200_HD uint16_t value_u16(uint64_t key, uint64_t index, int dist, float sigma, int dtype) {
    const float v = value(key, index, dist, sigma);
    return dtype ? to_bf16_bits(v) : to_half_bits(v);
}

}  // namespace synth
}  // namespace b200
