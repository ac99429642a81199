// oz_common.cuh -- small device helpers shared by the kernels.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "oz_tables.cuh"

namespace ozk {

// A kernel attribute (or anything else that belongs to a device's context) has to be set once on EVERY device a process
// uses, not once per process: run `f` the first time the calling site is reached with each device current.
struct PerDevice {
    unsigned long long seen = 0;   // one bit per device ordinal (0..63)
    template <class F> cudaError_t once(F &&f) {
        int dev = 0;
        if (cudaError_t e = cudaGetDevice(&dev)) return e;
        if (dev < 0 || dev > 63) return cudaErrorInvalidDevice;
        if (seen >> dev & 1ull) return cudaSuccess;
        if (cudaError_t e = f()) return e;
        seen |= 1ull << dev;       // callers hold the library's mutex or tolerate a repeated, idempotent call
        return cudaSuccess;
    }
};

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {   // signed bytes x signed bytes
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // unsigned bytes of a x signed bytes of b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// byte 0 of four registers into one word
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
// u mod m for 0 <= u below the bound checked by magic_ok(): one multiply-high, one multiply-add
template <int L>
__device__ __forceinline__ uint32_t mod_magic(uint32_t u) {
    return u - __umulhi(u, magic_of(L)) * (uint32_t)modulus(L);
}
// Balanced residue of a lifted sum: `a` is a non-negative representative of the class that is already shifted down by
// floor(m/2), i.e. a = S + (multiple of m) with S the signed sum; bal(S) = (a + floor(m/2)) mod m - floor(m/2). One add, one
// multiply-high, one multiply-add, one subtract. (Folding the add into the quotient with a 64-bit multiply-add and a
// constant addend is exact too, but measured on B200 it executes MORE instructions: 86.0 M against 78.1 M warp instructions
// for the residues of a 4096 x 4096 matrix -- the 64-bit constant costs more than the add it saves. -DOZ_FOLD_BALANCE keeps
// that form for comparison.) Exact while a + floor(m/2) is below the bound checked by magic_ok(). Returns the residue as a
// 32-bit two's-complement value (its low byte is the int8).
template <int L>
__device__ __forceinline__ uint32_t balanced_magic(uint32_t a) {
#ifdef OZ_FOLD_BALANCE
    constexpr unsigned long long add = (unsigned long long)half_of(L) * magic_of(L);
    unsigned long long prod;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(prod) : "r"(a), "r"(magic_of(L)), "l"(add));
    return a - (uint32_t)(prod >> 32) * (uint32_t)modulus(L);
#else
    const uint32_t u = a + (uint32_t)half_of(L);
    return u - __umulhi(u, magic_of(L)) * (uint32_t)modulus(L) - (uint32_t)half_of(L);
#endif
}
// The same balanced residue on the FP32 pipes. `biased` is the signed sum S on top of the bit pattern of 1.5 * 2^23
// (FLOAT_BIAS: seed the dp4a chain with it and the sum lands in the mantissa, so the word read as a float IS 1.5 * 2^23 + S).
// q = rint(S / m) by the add-and-subtract of 1.5 * 2^23, then 1.5 * 2^23 + S - q m in one fused multiply-add; the low
// byte of that float's bit pattern is the int8 residue. Exact for odd m and |S| < 2^22: S / m computed as S * fl(1/m) is
// off by less than |S| 2^-24 / m, and S / m is never closer than 1/(2m) to a half-integer; every other step is exact integer
// arithmetic below 2^24. Four FP32 instructions, which run on either FMA pipe; the multiply-high form keeps two of its four on
// the one pipe that also runs dp4a.
constexpr int FLOAT_BIAS = 0x4B400000;   // 1.5 * 2^23 = 12582912.0f
template <int L>
__device__ __forceinline__ uint32_t balanced_float(int biased) {
    static_assert(modulus(L) % 2 == 1, "an even modulus has ties");
    constexpr float C = 12582912.0f, inv = 1.0f / (float)modulus(L), m = (float)modulus(L);
    const float A = __int_as_float(biased);
    const float q = __fadd_rn(__fmaf_rn(__fadd_rn(A, -C), inv, C), -C);
    return (uint32_t)__float_as_int(__fmaf_rn(q, -m, A));
}
// Two sums at once with the packed FP32 instructions of sm_100 (add.f32x2 / fma.rn.f32x2: one instruction, two lanes, each
// lane rounded like the scalar form -- same bits, half the instruction slots; these kernels are bound by instruction issue).
template <int L>
__device__ __forceinline__ void balanced_float_x2(int biased0, int biased1, uint32_t &x0, uint32_t &x1) {
#ifdef OZ_NO_F32X2
    x0 = balanced_float<L>(biased0);
    x1 = balanced_float<L>(biased1);
#else
    static_assert(modulus(L) % 2 == 1, "an even modulus has ties");
    constexpr float C = 12582912.0f, inv = 1.0f / (float)modulus(L), m = (float)modulus(L);
    const float2 A = make_float2(__int_as_float(biased0), __int_as_float(biased1));
    const float2 q = __fadd2_rn(__ffma2_rn(__fadd2_rn(A, make_float2(-C, -C)), make_float2(inv, inv), make_float2(C, C)), make_float2(-C, -C));
    const float2 X = __ffma2_rn(q, make_float2(-m, -m), A);
    x0 = (uint32_t)__float_as_int(X.x);
    x1 = (uint32_t)__float_as_int(X.y);
#endif
}
// 2^s as a double for -1022 <= s <= 1023
__device__ __forceinline__ double pow2_normal(int s) { return __hiloint2double((s + 1023) << 20, 0); }
// llrint(ldexp(x, s)) as the reference computes it (src/ozaki2.cuh:76). For s in the normal exponent range the scaling
// is a multiplication by 2^s: exact whenever the result is a normal number, and any result below 2^-1022 rounds to the
// integer 0 either way. Outside that range (rows whose largest entry is subnormal or above 2^1000) ldexp itself is used.
__device__ __forceinline__ long long scaled_int(double x, int s, double p2, bool fast) {
    return __double2ll_rn(fast ? x * p2 : ldexp(x, s));
}
// the reference's scale: bits - 1 - ilogb(max |x|), 0 for an all-zero row (src/ozaki2.cuh:66)
__device__ __forceinline__ int scale_from_max(double mx, int bits) { return mx == 0 ? 0 : bits - 1 - ilogb(mx); }

}  // namespace ozk
