// host_tables_check.cpp -- CPU check of the integer identities the device kernels rely on (compiled and run by
// tests/test_host_tables.py with g++; no GPU involved). Uses the same constexpr tables as the kernels
// (ozaki_blackwell_b200/csrc/oz_tables.cuh) and emulates dp4a / umulhi in plain C++.
//   1. residues of a 64-bit integer from its bytes          (scale_residue.cu: residues_of_4)
//   2. balanced residue of an int32 product by 16-bit split  (gemm_i8_sm100.cu: fused epilogue)
//   3. Garner digits with one reduction per digit            (crt.cu: garner_horner)
//   6. the same reductions done in FP32 (oz_common.cuh: balanced_float), which is what the kernels run: every sum in
//      (-2^22, 2^22) for every odd modulus of the table, and the byte-sum / Garner / double-double forms built on it
// Each is compared with the reference's definition: bal(x, m) and the step-by-step Garner recurrence
// (src/ozaki2.cuh:38-42, 86-92 of the reference).
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include "oz_tables.cuh"
using namespace ozk;

static int dp4a(uint32_t a, uint32_t b, int c, bool a_signed) {
    for (int i = 0; i < 4; i++) {
        const int x = a_signed ? (int)(int8_t)(a >> (8 * i)) : (int)(uint8_t)(a >> (8 * i));
        c += x * (int)(int8_t)(b >> (8 * i));
    }
    return c;
}
static uint32_t umulhi(uint32_t a, uint32_t b) { return (uint32_t)(((uint64_t)a * b) >> 32); }
// oz_common.cuh: balanced_magic<L> -- the quotient of (a + floor(m/2)) / m from one wide multiply-add with a constant addend
template <int L> static uint32_t balanced_magic(uint32_t a) {
    const uint32_t u = a + (uint32_t)half_of(L);
    const uint32_t plain = u - umulhi(u, magic_of(L)) * (uint32_t)modulus(L) - (uint32_t)half_of(L);
    const uint64_t prod = (uint64_t)a * magic_of(L) + (uint64_t)half_of(L) * magic_of(L);   // the folded form (-DOZ_FOLD_BALANCE)
    const uint32_t folded = a - (uint32_t)(prod >> 32) * (uint32_t)modulus(L);
    return plain == folded ? plain : 0x7fffffffu;   // both forms must agree; a disagreement shows up as a wrong residue
}
static int bal(long long x, int m) { return bal_c(x, m); }
// oz_common.cuh: balanced_float<L> -- the sum rides on the bit pattern of 1.5 * 2^23; IEEE single arithmetic, fused multiply-adds
constexpr int FLOAT_BIAS = 0x4B400000;
static float as_float(int32_t b) { float f; memcpy(&f, &b, 4); return f; }
static int32_t as_int(float f) { int32_t b; memcpy(&b, &f, 4); return b; }
template <int L> static uint32_t balanced_float(int biased) {
    const float C = 12582912.0f, inv = 1.0f / (float)modulus(L), m = (float)modulus(L);
    const volatile float A = as_float(biased);            // volatile: every step is rounded to single, nothing is re-associated
    const volatile float f = A - C;
    const volatile float t = std::fmaf(f, inv, C);
    const volatile float q = t - C;
    const volatile float x = std::fmaf(q, -m, A);
    return (uint32_t)as_int(x);
}
template <int L> static long check_float_reduction() {
    if (modulus(L) % 2 == 0) return 0;                    // 256 is never reduced this way
    long bad = 0;
    for (int S = -(1 << 22) + 1; S < (1 << 22); S++) bad += (int)(int8_t)(balanced_float<L>(FLOAT_BIAS + S) & 255) != bal(S, modulus(L));
    return bad;
}

template <int L> struct PerMod {
    static int residue_from_bytes(long long v) {
        constexpr int l = L, m = modulus(l);
        if (l == 0) return (int)(int8_t)(v & 255);
        constexpr uint32_t wlo = pack4(byte_weight(0, l), byte_weight(1, l), byte_weight(2, l), byte_weight(3, l));
        constexpr uint32_t whi = pack4(byte_weight(4, l), byte_weight(5, l), byte_weight(6, l), byte_weight(7, l));
        constexpr int init = lift_of(l, BYTES_BOUND) - half_of(l) - pow2_mod(62, m);
        static_assert(init > BYTES_BOUND && magic_ok(l, (uint64_t)init + half_of(l) + BYTES_BOUND), "range");
        const uint64_t w = (uint64_t)v + (1ull << 62);
        const uint32_t u = (uint32_t)dp4a((uint32_t)(w >> 32), whi, dp4a((uint32_t)w, wlo, init, false), false);
        const int viaint = (int)(int8_t)(balanced_magic<l>(u) & 255);
        const int seed = FLOAT_BIAS - pow2_mod(62, m);     // scale_residue.cu, exact_f8.cu: the chain seeded for the FP32 form
        const int viafloat = (int)(int8_t)(balanced_float<l>(dp4a((uint32_t)(w >> 32), whi, dp4a((uint32_t)w, wlo, seed, false), false)) & 255);
        return viaint == viafloat ? viaint : 0x7fff;
    }
    static int residue_of_product(int32_t x) {
        constexpr ModConsts mc = mod_consts(L);
        const uint32_t u = (uint32_t)x ^ 0x80000000u;
        const uint32_t t = (u >> 16) * mc.c16 + (u & 0xFFFFu) + mc.adj;
        return (int)(int8_t)((t - umulhi(t, mc.magic) * mc.m - (uint32_t)mc.half) & 255);
    }
};

template <int NM> static void garner_fast(const int *r, int *x) {   // r: balanced residues
    uint32_t X[(NM + 3) / 4] = {};
    for (int l = 0; l < NM; l++) X[l / 4] |= (uint32_t)(r[l] & 255) << (8 * (l % 4));
    x[0] = (int)(int8_t)(X[0] & 255);
    static_for<1, NM>([&](auto Lc) {
        constexpr int l = decltype(Lc)::value, m = modulus(l);
        int acc = lift_of(l, GARNER_BOUND) - half_of(l);
        for (int g = 0; g <= l / 4; g++) {
            int c[4];
            for (int q = 0; q < 4; q++) { const int idx = 4 * g + q; c[q] = idx < l ? garner_q(idx, l) : (idx == l ? garner_p(l) : 0); }
            acc = dp4a(X[g], pack4(c[0], c[1], c[2], c[3]), acc, true);
        }
        int accf = FLOAT_BIAS;                              // crt.cu: the same dot product seeded for the FP32 form
        for (int g = 0; g <= l / 4; g++) {
            int c[4];
            for (int q = 0; q < 4; q++) { const int idx = 4 * g + q; c[q] = idx < l ? garner_q(idx, l) : (idx == l ? garner_p(l) : 0); }
            accf = dp4a(X[g], pack4(c[0], c[1], c[2], c[3]), accf, true);
        }
        const int xi = (int)(int8_t)(balanced_magic<l>((uint32_t)acc) & 255), xf = (int)(int8_t)(balanced_float<l>(accf) & 255);
        const int xl = xi == xf ? xi : 0x7fff;
        (void)m;
        X[l / 4] = (X[l / 4] & ~(255u << (8 * (l % 4)))) | ((uint32_t)(xl & 255) << (8 * (l % 4)));
        x[l] = xl;
    });
}
template <int NM> static void garner_ref(const int *r, int *x) {   // src/ozaki2.cuh:86-92
    for (int l = 0; l < NM; l++) {
        const int m = modulus(l);
        int v = bal(r[l], m);
        for (int t = 0; t < l; t++) v = bal((long long)(v - x[t]) * garner_inv(t, l), m);
        x[l] = v;
    }
}

template <int L> static long check_mod(std::mt19937_64 &g) {
    long bad = 0;
    constexpr int m = modulus(L);
    const long long edge[] = {0, 1, -1, 127, 128, -128, -129, 255, 256, (1ll << 61), -(1ll << 61), (1ll << 62) - 1, -(1ll << 62) + 1,
                              (1ll << 57) - 1, -(1ll << 57)};
    for (long long v : edge) bad += PerMod<L>::residue_from_bytes(v) != bal(v, m);
    for (int i = 0; i < 50000; i++) {
        const long long v = (long long)(g() >> 1) - (1ll << 62);
        bad += PerMod<L>::residue_from_bytes(v) != bal(v, m);
        const long long small = (long long)(g() % 100001) - 50000;
        bad += PerMod<L>::residue_from_bytes(small) != bal(small, m);
    }
    const int32_t pedge[] = {0, 1, -1, INT32_MAX, INT32_MIN, INT32_MIN + 1, 65535, 65536, -65536, -65537, 128 * 128 * 131071, -128 * 127 * 131071};
    for (int32_t x : pedge) bad += PerMod<L>::residue_of_product(x) != bal(x, m);
    for (int i = 0; i < 100000; i++) { const int32_t x = (int32_t)g(); bad += PerMod<L>::residue_of_product(x) != bal(x, m); }
    // every value of the high half with the extreme low halves (the bound of the multiply-high is tight for m = 255)
    for (uint32_t hi = 0; hi < 65536; hi++)
        for (uint32_t lo : {0u, 1u, 65534u, 65535u}) { const int32_t x = (int32_t)((hi << 16) | lo); bad += PerMod<L>::residue_of_product(x) != bal(x, m); }
    return bad;
}
template <int NM> static long check_garner(std::mt19937_64 &g) {
    long bad = 0;
    for (int i = 0; i < 6000; i++) {
        int r[NM], a[NM], b[NM];
        for (int l = 0; l < NM; l++) {
            const int m = modulus(l);
            r[l] = i < 4 ? (i == 0 ? -(m / 2) : i == 1 ? (m + 1) / 2 - 1 : i == 2 ? 0 : ((l & 1) ? -(m / 2) : (m + 1) / 2 - 1))
                         : bal((long long)(g() % m), m);
        }
        garner_fast<NM>(r, a);
        garner_ref<NM>(r, b);
        for (int l = 0; l < NM; l++) bad += a[l] != b[l];
    }
    return bad;
}

// ---- double-double path ----
//   4. residue of V = u 2^53 + t from the sixteen bytes of (u + 2^62, t + 2^62)   (dd.cu: residues_of_4_dd)
//   5. the direct-sum CRT tables: known signed integers of up to 192 bits come back from their residues
//      (the reference's own known-answer test, bench/crt_check.cpp:18-35)
template <int L> static int dd_residue(long long u, long long t) {
    constexpr int l = L, m = modulus(l), p53 = pow2_mod(53, m);
    if (l == 0) return (int)(int8_t)(t & 255);
    int wt[8], wu[8];
    for (int i = 0; i < 8; i++) { wt[i] = byte_weight(i, l); wu[i] = bal_c((long long)posmod_c(byte_weight(i, l), m) * p53, m); }
    constexpr int bound = 16 * 255 * 128;
    constexpr int off = posmod_c((long long)pow2_mod(62, m) * p53 + pow2_mod(62, m), m);
    constexpr int init = lift_of(l, bound) - off;
    static_assert(init > bound && magic_ok(l, (uint64_t)init + bound), "range");
    const uint64_t a = (uint64_t)u + (1ull << 62), b = (uint64_t)t + (1ull << 62);
    int acc = init;
    acc = dp4a((uint32_t)b, pack4(wt[0], wt[1], wt[2], wt[3]), acc, false);
    acc = dp4a((uint32_t)(b >> 32), pack4(wt[4], wt[5], wt[6], wt[7]), acc, false);
    acc = dp4a((uint32_t)a, pack4(wu[0], wu[1], wu[2], wu[3]), acc, false);
    acc = dp4a((uint32_t)(a >> 32), pack4(wu[4], wu[5], wu[6], wu[7]), acc, false);
    const uint32_t uu = (uint32_t)acc;
    const int viaint = (int)(int8_t)((uu - umulhi(uu, magic_of(l)) * (uint32_t)m - (uint32_t)half_of(l)) & 255);
    int accf = FLOAT_BIAS - off;                           // dd.cu: the chain seeded for the FP32 form
    accf = dp4a((uint32_t)b, pack4(wt[0], wt[1], wt[2], wt[3]), accf, false);
    accf = dp4a((uint32_t)(b >> 32), pack4(wt[4], wt[5], wt[6], wt[7]), accf, false);
    accf = dp4a((uint32_t)a, pack4(wu[0], wu[1], wu[2], wu[3]), accf, false);
    accf = dp4a((uint32_t)(a >> 32), pack4(wu[4], wu[5], wu[6], wu[7]), accf, false);
    const int viafloat = (int)(int8_t)(balanced_float<l>(accf) & 255);
    return viaint == viafloat ? viaint : 0x7fff;
}
template <int L> static long check_dd_mod(std::mt19937_64 &g) {
    long bad = 0;
    constexpr int m = modulus(L);
    for (int i = 0; i < 20000; i++) {
        long long u = (long long)(g() >> 11) - (1ll << 52), t = (long long)(g() >> 9) - (1ll << 54);
        if (i < 4) { u = i & 1 ? (1ll << 53) - 1 : -(1ll << 53) + 1; t = i & 2 ? (1ll << 55) : -(1ll << 55); }
        const __int128 V = (__int128)u * ((__int128)1 << 53) + t;
        int r = (int)(V % m); if (r < 0) r += m; if (r >= (m + 1) / 2) r -= m;
        bad += dd_residue<L>(u, t) != r;
    }
    return bad;
}
template <int NM> static long check_dd_crt(std::mt19937_64 &g) {
    constexpr DdTables<NM> T = make_dd_tables<NM>();
    long bad = 0;
    const int maxlimbs = NM >= 32 ? 6 : NM >= 28 ? 5 : 4;   // stay below P/2
    for (int it = 0; it < 20000; it++) {
        unsigned V[8] = {}; const int nl = 1 + g() % maxlimbs; for (int k = 0; k < nl; k++) V[k] = (unsigned)g();
        const bool sgn = g() & 1;
        if (sgn) { unsigned long long b = 1; for (int k = 0; k < 8; k++) { b += (unsigned)~V[k]; V[k] = (unsigned)b; b >>= 32; } }
        unsigned long long acc[8] = {}; long long qf = 0;
        for (int l = 0; l < NM; l++) {
            const int m = modulus(l);
            long long x = 0; for (int k = 7; k >= 0; k--) x = ((x << 32) + V[k]) % m;
            if (sgn) { long long p = 1; for (int t = 0; t < 256; t++) p = p * 2 % m; x = ((x - p) % m + m) % m; }
            qf += x * T.F[l]; for (int k = 0; k < 8; k++) acc[k] += (unsigned long long)x * T.W[l][k];
        }
        long long q = (qf + (1ll << 39)) >> 40, c = 0; bool same = true;
        for (int k = 0; k < 8; k++) { c += (long long)acc[k] - q * (long long)T.P[k]; same &= (unsigned)c == V[k]; c >>= 32; }
        bad += !same;
    }
    return bad;
}

int main() {
    std::mt19937_64 g(12345);
    long bad = 0;
    static_for<0, 32>([&](auto L) { bad += check_dd_mod<decltype(L)::value>(g); });
    bad += check_dd_crt<24>(g) + check_dd_crt<28>(g) + check_dd_crt<32>(g);
    static_for<0, MAXM>([&](auto L) { bad += check_mod<decltype(L)::value>(g); });
    static_for<8, 17>([&](auto N) { bad += check_garner<decltype(N)::value>(g); });
    static_for<1, MAXM>([&](auto L) { bad += check_float_reduction<decltype(L)::value>(); });
    printf("%ld wrong\n", bad);
    return bad != 0;
}
