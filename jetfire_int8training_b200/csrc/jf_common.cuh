// Shared device helpers for the Jetfire INT8 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jetfire_b200.h"

namespace jf {

constexpr int QB = 32;  // quantisation block edge

// ---------------------------------------------------------------------------------------------------------
// host-side status plumbing
// ---------------------------------------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return JF_ERR_LAUNCH;
    }
    return JF_OK;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool mult32(int64_t v) { return v > 0 && (v % 32) == 0; }

// ---------------------------------------------------------------------------------------------------------
// Philox4x32-10 (Random123) and the stochastic-rounding noise
// ---------------------------------------------------------------------------------------------------------
// Noise mapping.  One Philox call (four 32-bit words) serves the 8 consecutive elements of group g = e / 8; element e uses the
// 16-bit half (e & 1) of word (e >> 1) & 3:  noise = h * 2^-16 - 0.5, a multiple of 2^-16 in [-0.5, 0.5) like the reference's
// uniform_(-0.5, 0.5).  Built without an int->float conversion: the half is placed in the low mantissa bits of 2^23, and one
// FMA rescales it: (2^23 + h) * 2^-16 - 128.5 = h * 2^-16 - 0.5, exact in fp32.
__device__ __forceinline__ float half_to_noise(uint32_t w, int hi) {
    const uint32_t bits = __byte_perm(w, 0x4B000000u, hi ? 0x7432 : 0x7410);   // {h.lo, h.hi, 0x00, 0x4B}
    return __fmaf_rn(__uint_as_float(bits), 1.52587890625e-05f, -128.5f);
}

// The ten round keys of Philox4x32-10 for one seed (key schedule: k + r * (0x9E3779B9, 0xBB67AE85)), computed on the host and
// passed with the kernel parameters: in the kernel they are constant-bank operands of the round's XOR, which saves the 18
// additions of the schedule per call (a call serves only 8 elements, so the generator is a large part of every stochastic kernel).
struct PhiloxKeys {
    uint32_t k[20];
};
inline PhiloxKeys make_philox_keys(uint64_t seed) {
    PhiloxKeys ks;
    uint32_t kx = (uint32_t)seed, ky = (uint32_t)(seed >> 32);
    for (int r = 0; r < 10; ++r) {
        ks.k[2 * r] = kx;
        ks.k[2 * r + 1] = ky;
        kx += 0x9E3779B9u;
        ky += 0xBB67AE85u;
    }
    return ks;
}
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, const PhiloxKeys& ks) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ ks.k[2 * r], lo1, hi0 ^ c.w ^ ks.k[2 * r + 1], lo0);
    }
    return c;
}

// Noise for the 8 consecutive elements starting at linear index e (e % 8 == 0).
__device__ __forceinline__ void philox_noise8(uint64_t e, const PhiloxKeys& keys, uint64_t offset, float out[8]) {
    const uint64_t g = e >> 3;
    const uint4 w = philox4x32_10(make_uint4((uint32_t)g, (uint32_t)(g >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)), keys);
    out[0] = half_to_noise(w.x, 0); out[1] = half_to_noise(w.x, 1);
    out[2] = half_to_noise(w.y, 0); out[3] = half_to_noise(w.y, 1);
    out[4] = half_to_noise(w.z, 0); out[5] = half_to_noise(w.z, 1);
    out[6] = half_to_noise(w.w, 0); out[7] = half_to_noise(w.w, 1);
}

// ---------------------------------------------------------------------------------------------------------
// Exact IEEE division by a value shared across many elements.
// With y = RN(1/b) (correctly rounded reciprocal), q0 = RN(a*y), r = a - b*q0 (exact in one FMA) and
// q = RN(q0 + r*y) is the correctly rounded quotient RN(a/b) (Markstein's correction step), provided nothing
// under/overflows.  The fast path is taken only for b in [2^-60, 2^60]; otherwise div.rn is used.
// ---------------------------------------------------------------------------------------------------------
struct Divisor {
    float b;     // divisor
    float inv;   // RN(1/b)
    bool fast;   // fast path is valid
};
__device__ __forceinline__ Divisor make_divisor(float b) {
    Divisor d;
    d.b = b;
    d.inv = __frcp_rn(b);
    const float ab = fabsf(b);
    d.fast = (ab >= 8.673617379884035e-19f) && (ab <= 1.152921504606847e18f);
    return d;
}
// use: q0 = a * d.inv;  q = fma(fma(-d.b, q0, a), d.inv, q0)   (d.fast)      or      q = a / d.b   (otherwise)

// Two fp32 values in one 64-bit register and the two-wide IEEE operations on them (each half is rounded exactly like the scalar
// mul.rn / add.rn / fma.rn; subnormals are kept): one issue slot for two elements in the kernels that are bound by instruction issue.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// the exact quotients a / d.b of two values (d.fast)
__device__ __forceinline__ uint64_t f2_div_fast(uint64_t a2, uint64_t inv2, uint64_t negb2) {
    const uint64_t q0 = f2_mul(a2, inv2);
    return f2_fma(f2_fma(negb2, q0, a2), inv2, q0);
}

// fp16 product of an int8 payload value and its fp16 scale, as the reference's "int8 * fp16" does
// (the int8 is converted to fp16 exactly, the product is rounded to fp16 once).  q*s is exact in fp32.
__device__ __forceinline__ __half deq16(int q, float s_as_float) { return __float2half_rn(__fmul_rn((float)q, s_as_float)); }

__device__ __forceinline__ int sbyte(uint32_t w, int i) { return (int)(int8_t)(w >> (8 * i)); }

// Exact int8 -> fp32 without the conversion unit: byte k of w (two's complement), with its sign bit flipped, goes into the low
// mantissa byte of 2^23; (2^23 + u) - (2^23 + 128) = q exactly.  `wx` must be w ^ 0x80808080.
__device__ __forceinline__ float byte_to_float(uint32_t wx, int k) {
    const uint32_t sel = k == 0 ? 0x7440u : k == 1 ? 0x7441u : k == 2 ? 0x7442u : 0x7443u;   // {byte k, 0x00, 0x00, 0x4B}
    return __fadd_rn(__uint_as_float(__byte_perm(wx, 0x4B000000u, sel)), -8388736.0f);
}

// dtype-generic 16-element row chunk loads -> fp32
template <typename T>
struct Load16;
template <>
struct Load16<float> {
    static __device__ __forceinline__ void load(const float* p, float v[16]) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 t = __ldg(p4 + i);
            v[4 * i + 0] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    }
};
template <>
struct Load16<__half> {
    static __device__ __forceinline__ void load(const __half* p, float v[16]) {
        const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 t = __ldg(p4 + i);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                const float2 f = __half22float2(h);
                v[8 * i + 2 * j] = f.x; v[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
};
template <>
struct Load16<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float v[16]) {
        const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 t = __ldg(p4 + i);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            }
        }
    }
};

}  // namespace jf
