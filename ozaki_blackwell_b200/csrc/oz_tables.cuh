// oz_tables.cuh -- the moduli and every constant derived from them, evaluated at compile time.
//
// The modulus set is the reference's (src/ozaki2.cuh:21-23: pairwise coprime, largest first); everything else here is
// derived from it so that the device kernels can reduce with multiplies instead of divisions and run Garner's algorithm
// with one modular reduction per digit instead of one per step.
#pragma once
#include <cstdint>
#include <type_traits>

#if defined(__CUDACC__)
#define OZ_HD __host__ __device__
#else
#define OZ_HD
#endif

namespace ozk {

constexpr int MAXM = 49;      // size of the table (the triple-double path of the reference uses all 49)
constexpr int MAX_NM64 = 16;  // the FP64 product takes 8..16 of them

OZ_HD constexpr int modulus(int l) {
    constexpr int T[MAXM] = {256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193,
                             191, 181, 179, 173, 167, 163, 157, 151, 149, 139, 137, 131, 127, 113, 109, 107,
                             103, 101, 97,  89,  83,  79,  73,  71,  67,  61,  59,  53,  47,  43,  41,  37,  29};
    return T[l];
}

// x mod m folded into the reference's balanced range [-(m/2), (m+1)/2)  (src/ozaki2.cuh:38-42)
OZ_HD constexpr int bal_c(long long x, int m) {
    int r = (int)(x % m);
    if (r < 0) r += m;
    return r >= (m + 1) / 2 ? r - m : r;
}
OZ_HD constexpr int posmod_c(long long x, int m) {
    int r = (int)(x % m);
    return r < 0 ? r + m : r;
}
// a^-1 mod m by search (src/ozaki2.cuh:99); only ever evaluated by the compiler
OZ_HD constexpr int inv_mod_c(int a, int m) {
    for (int x = 1; x < m; x++)
        if (a * x % m == 1) return x;
    return 0;
}
// c_inv[t][l] of the reference: m_t^-1 mod m_l for t < l  (src/ozaki2.cuh:112)
OZ_HD constexpr int garner_inv(int t, int l) { return inv_mod_c(modulus(t) % modulus(l), modulus(l)); }

// Garner's recurrence  v <- (v - x_t) * inv[t][l]  (t = 0..l-1, starting from the residue r_l) unrolls to
//     x_l = r_l * P_l - sum_{t<l} x_t * Q_{t,l}   (mod m_l),   P_l = prod_{t<l} inv[t][l],  Q_{t,l} = prod_{s=t}^{l-1} inv[s][l].
// The digit is the balanced representative of that class, so one reduction of the whole sum gives the same digit as
// the reference's l reductions. Both coefficient sets are stored balanced so that they fit int8 (dp4a operands):
//     garner_p(l)   = bal(P_l),     garner_q(t,l) = bal(-Q_{t,l}),     x_l = bal(garner_p(l) r_l + sum_t garner_q(t,l) x_t).
OZ_HD constexpr int garner_p(int l) {
    const int m = modulus(l);
    long long p = 1;
    for (int t = 0; t < l; t++) p = p * garner_inv(t, l) % m;
    return bal_c(p, m);
}
OZ_HD constexpr int garner_q(int t, int l) {
    const int m = modulus(l);
    long long q = 1;
    for (int s = t; s < l; s++) q = q * garner_inv(s, l) % m;
    return bal_c(-q, m);
}

// floor(m/2): subtracting it from a residue in [0, m) gives the balanced residue
OZ_HD constexpr int half_of(int l) { return modulus(l) / 2; }
// ceil(2^32 / m): for 0 <= u with u * (magic*m - 2^32) < 2^32, floor(u / m) = umulhi(u, magic) exactly
OZ_HD constexpr uint32_t magic_of(int l) { return (uint32_t)(((1ull << 32) + modulus(l) - 1) / modulus(l)); }
OZ_HD constexpr uint32_t magic_err(int l) { return (uint32_t)((uint64_t)magic_of(l) * modulus(l) - (1ull << 32)); }

// bal(256^i mod m_l): weight of byte i of a 64-bit integer
OZ_HD constexpr int byte_weight(int i, int l) {
    const int m = modulus(l);
    long long w = 1;
    for (int s = 0; s < i; s++) w = w * 256 % m;
    return bal_c(w, m);
}
OZ_HD constexpr uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 255) | ((uint32_t)(b & 255) << 8) | ((uint32_t)(c & 255) << 16) | ((uint32_t)(d & 255) << 24);
}
// 2^e mod m
OZ_HD constexpr int pow2_mod(int e, int m) {
    long long w = 1;
    for (int s = 0; s < e; s++) w = w * 2 % m;
    return (int)w;
}

// A multiple of m_l that exceeds `bound`, plus floor(m/2): added to a sum S with |S| <= bound it makes S non-negative
// and shifts the residue so that (S' mod m) - floor(m/2) is balanced.
OZ_HD constexpr int lift_of(int l, int bound) {
    const int m = modulus(l);
    return ((bound + m - 1) / m + 1) * m + half_of(l);
}

// Largest |sum| the two uses of dp4a produce: 16 terms of at most 128 * 128 (Garner), 8 bytes of at most 255 * 128 (residues)
constexpr int GARNER_BOUND = 16 * 128 * 128;
constexpr int BYTES_BOUND = 8 * 255 * 128;

// the exactness condition of the multiply-high division for everything that goes through it
OZ_HD constexpr bool magic_ok(int l, uint64_t umax) { return umax * magic_err(l) < (1ull << 32); }

// Per-modulus constants for kernels that take the modulus index at run time (the GEMM epilogue).
struct ModConsts {
    uint32_t m, magic, c16, adj;  // modulus; ceil(2^32/m); 2^16 mod m; (floor(m/2) - 2^31) mod m
    int half;                     // floor(m/2)
};
OZ_HD constexpr ModConsts mod_consts(int l) {
    const int m = modulus(l);
    return ModConsts{(uint32_t)m, magic_of(l), (uint32_t)pow2_mod(16, m), (uint32_t)posmod_c(half_of(l) - (long long)pow2_mod(31, m), m),
                     half_of(l)};
}
// largest value the epilogue's reduction feeds to the multiply-high: hi16 * c16 + lo16 + adj
OZ_HD constexpr uint64_t epi_umax(int l) {
    const ModConsts c = mod_consts(l);
    return 65535ull * c.c16 + 65535ull + c.adj;
}

// Tables of the double-double path's direct-sum CRT (reference: src/ozaki_dd.cuh:73-91, crt_consts): for the first NM
// moduli with product P, W[l] = (P/m_l) * ((P/m_l)^-1 mod m_l) and P as eight 32-bit limbs, F[l] = round(2^40 w_l / m_l).
template <int NM>
struct DdTables {
    unsigned W[NM][8];
    unsigned P[8];
    long long F[NM];
};
OZ_HD constexpr void mul_small(unsigned (&a)[8], unsigned m) {
    unsigned long long c = 0;
    for (int k = 0; k < 8; k++) { c += (unsigned long long)a[k] * m; a[k] = (unsigned)c; c >>= 32; }
}
template <int NM>
OZ_HD constexpr DdTables<NM> make_dd_tables() {
    DdTables<NM> t{};
    t.P[0] = 1;
    for (int l = 0; l < NM; l++) mul_small(t.P, (unsigned)modulus(l));
    for (int l = 0; l < NM; l++) {
        const int ml = modulus(l);
        int r = 1;
        t.W[l][0] = 1;
        for (int s = 0; s < NM; s++)
            if (s != l) { mul_small(t.W[l], (unsigned)modulus(s)); r = r * (modulus(s) % ml) % ml; }
        const int w = inv_mod_c(r, ml);
        mul_small(t.W[l], (unsigned)w);
        // llround(ldexp((double)w / m, 40)): the quotient has 13 spare bits below 2^40, so adding 0.5 is exact
        t.F[l] = (long long)((double)w / ml * 1099511627776.0 + 0.5);
    }
    return t;
}
template <int L, int N, class F>
OZ_HD inline void static_for(F &&f) {
    if constexpr (L < N) {
        f(std::integral_constant<int, L>{});
        static_for<L + 1, N>(f);
    }
}

}  // namespace ozk
