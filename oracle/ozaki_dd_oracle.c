/* ozaki_dd_oracle.c -- CPU restatement of the reference's double-double (~106-bit) product, stage by stage.
 *
 * TEST INFRASTRUCTURE ONLY, like ozaki2_oracle.c: the checker for the CUDA double-double path, never linked into the
 * library. Paths are relative to the reference project:
 *   src/ozaki_dd.cuh:11        pow2mod                                   -> pow2mod
 *   src/ozaki_dd.cuh:13-20     dd, two_sum, quick_two_sum                -> two_sum, quick_two_sum
 *   src/ozaki_dd.cuh:23-35     scales_dd (the FP64 scales on the hi parts) -> oz_oracle_scales (ozaki2_oracle.c)
 *   src/ozaki_dd.cuh:39-44     C16, cut16, res16                         -> cut16, res16
 *   src/ozaki_dd.cuh:46-64     residues_dd<NM>                           -> oz_oracle_residues_dd
 *   src/ozaki_dd.cuh:73-91     crt_consts (W, M, F tables)               -> oz_oracle_dd_consts
 *   src/ozaki_dd.cuh:93-140    crt_dd<NM> (direct sum over 8 limbs, modes 0/1/2) -> oz_oracle_crt_dd
 *   src/ozaki_dd.cuh:145-155   ddgemm_t<NM>                              -> oz_oracle_ddgemm
 *   bench/ref_quad.cpp:6-16    the __float128 reference product          -> oz_oracle_ref_quad
 *   bench/crt_check.cpp:18-35  known-answer test of the direct-sum CRT   -> oz_oracle_dd_crt_kat
 *   bench/dd_test.cu:56-57     error in units of 2^-106                  -> oz_oracle_dd_err_units
 * Compile with -O2 -ffp-contract=off: the only fused operation is the explicit fma() of crt_dd.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int oz_oracle_modulus(int l);
int oz_oracle_inv_mod(int a, int m);
int oz_oracle_bits_for(int nm, int K, int maxbits);
void oz_oracle_scales(const double *X, int rows, int len, long long sRow, long long sCol, int bits, int *s);
void oz_oracle_gemm_i8(const int8_t *A, const int8_t *Bt, int32_t *C, int M, int N, int K, int lda, int ldb, int ldc);

#define OZ_MAXM 49

static int bal(long long x, int m) { int r = (int)(x % m); if (r < 0) r += m; return r >= (m + 1) / 2 ? r - m : r; }
static int pow2mod(int e, int m) { int r = 1 % m; for (int i = 0; i < e; i++) r = r * 2 % m; return r; }

typedef struct { double hi, lo; } dd;
static dd two_sum(double a, double b) { double s = a + b, v = s - a; dd r = {s, (a - (s - v)) + (b - v)}; return r; }
static dd quick_two_sum(double a, double b) { double s = a + b; dd r = {s, b - (s - a)}; return r; }

/* src/ozaki_dd.cuh:39-44 */
typedef struct { int c3, c2, c1, c0; } C16;
static C16 cut16(long long S) { C16 c = {(int)(S >> 48), (int)((S >> 32) & 0xffff), (int)((S >> 16) & 0xffff), (int)(S & 0xffff)}; return c; }
static int res16(C16 c, int m) { return bal((long long)(c.c3 * pow2mod(48, m) + c.c2 * pow2mod(32, m) + c.c1 * pow2mod(16, m) + c.c0), m); }

/* src/ozaki_dd.cuh:46-64 */
void oz_oracle_residues_dd(const double *Xh, const double *Xl, int rows, int len, long long sRow, long long sCol, const int *s, int nm,
                           int8_t *R, int ld, size_t plane) {
    int p53[OZ_MAXM];
    for (int l = 0; l < nm; l++) p53[l] = pow2mod(53, oz_oracle_modulus(l));
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        for (int k = 0; k < len; k++) {
            const size_t at = (size_t)(r * sRow + k * sCol);
            const double a = ldexp(Xh[at], s[r]), b = ldexp(Xl[at], s[r]);
            const double ai = trunc(a), bi = trunc(b);
            const double f = rint((a - ai) + (b - bi));
            const long long u = (long long)trunc(ldexp(ai, -53)), w = (long long)(ai - ldexp((double)u, 53)), bb = (long long)bi;
            const C16 c1 = cut16(u), c0 = cut16(w + bb + (long long)f);
            for (int l = 0; l < nm; l++) {
                const int m = oz_oracle_modulus(l);
                const int v = res16(c1, m) * p53[l] + res16(c0, m);
                R[l * plane + (size_t)r * ld + k] = (int8_t)bal(v, m);
            }
        }
}

/* src/ozaki_dd.cuh:73-91 -- W[l] = (P/m_l) * ((P/m_l)^-1 mod m_l) as 8 limbs of 32 bits, P = product of the nm moduli
 * (limbs in Mm), F[l] = round(2^40 * w_l / m_l) */
static void mul_small(unsigned *a, unsigned m) {
    unsigned long long c = 0;
    for (int k = 0; k < 8; k++) { c += (unsigned long long)a[k] * m; a[k] = (unsigned)c; c >>= 32; }
}
void oz_oracle_dd_consts(int nm, unsigned W[][8], unsigned *Mm, long long *F) {
    memset(Mm, 0, 8 * sizeof(unsigned));
    Mm[0] = 1;
    for (int l = 0; l < nm; l++) mul_small(Mm, (unsigned)oz_oracle_modulus(l));
    for (int l = 0; l < nm; l++) {
        const int ml = oz_oracle_modulus(l);
        int r = 1;
        memset(W[l], 0, 8 * sizeof(unsigned));
        W[l][0] = 1;
        for (int t = 0; t < nm; t++)
            if (t != l) { mul_small(W[l], (unsigned)oz_oracle_modulus(t)); r = r * (oz_oracle_modulus(t) % ml) % ml; }
        const int w = oz_oracle_inv_mod(r, ml);
        mul_small(W[l], (unsigned)w);
        F[l] = llround(ldexp((double)w / ml, 40));
    }
}

/* one element of src/ozaki_dd.cuh:97-139: residues r[l] of the exact product (any representative; reduced here as
 * the reference does, C remainder made non-negative) -> (hi, lo), sign and exponent handling included */
static dd crt_dd_one(const int32_t *res, size_t stride, int nm, unsigned W[][8], const unsigned *Mm, const long long *F, int sab, int mode,
                     double ch, double cl, int *is_zero) {
    unsigned long long acc[8] = {0};
    long long qf = 0;
    for (int l = 0; l < nm; l++) {
        const int m = oz_oracle_modulus(l);
        int r = res[l * stride] % m;
        if (r < 0) r += m;
        qf += (long long)r * F[l];
        for (int k = 0; k < 8; k++) acc[k] += (unsigned long long)r * W[l][k];
    }
    long long q = (qf + (1ll << 39)) >> 40, c = 0;
    unsigned v[8];
    for (int k = 0; k < 8; k++) { c += (long long)acc[k] - q * (long long)Mm[k]; v[k] = (unsigned)c; c >>= 32; }
    const int neg = (int)v[7] < 0;
    if (neg) {
        unsigned long long b = 1;
        for (int k = 0; k < 8; k++) { b += (unsigned)~v[k]; v[k] = (unsigned)b; b >>= 32; }
    }
    int top = -1;
    for (int k = 0; k < 8; k++) if (v[k]) top = k;
    *is_zero = top < 0;
    dd y = {0, 0};
    if (top < 0) return y;
    const unsigned t4 = v[top], t3 = top >= 1 ? v[top - 1] : 0, t2 = top >= 2 ? v[top - 2] : 0, t1 = top >= 3 ? v[top - 3] : 0,
                   t0 = top >= 4 ? v[top - 4] : 0;
    const int z = __builtin_clz(t4);
    unsigned long long H = (unsigned long long)t4 << 32 | t3, Lw = (unsigned long long)t2 << 32 | t1;
    if (z) { H = H << z | Lw >> (64 - z); Lw = Lw << z | t0 >> (32 - z); }
    const double dh = (double)(H & ~0x7FFull);            /* __ull2double_rd: H >= 2^63, so rounding down drops the low 11 bits */
    const double lo = fma((double)(H - (unsigned long long)dh), 18446744073709551616.0, (double)Lw);
    const int e = 32 * (top - 3) - z - sab;
    y = quick_two_sum(ldexp(dh, e + 64), ldexp(lo, e));
    if (neg != (mode != 0)) { y.hi = -y.hi; y.lo = -y.lo; }
    if (mode == 1) {
        dd s = two_sum(ch, y.hi), t = two_sum(cl, y.lo);
        s = quick_two_sum(s.hi, s.lo + t.hi);
        y = quick_two_sum(s.hi, s.lo + t.lo);
    }
    return y;
}

/* src/ozaki_dd.cuh:93-140 -- Cl: nm int32 planes (pitch ldc, plane pitch `plane`); outputs with pitch ldo; mode 0: C = AB,
 * 1: C -= AB, 2: C = -AB */
void oz_oracle_crt_dd(const int32_t *Cl, size_t plane, int M, int N, int ldc, const int *sa, const int *sb, int nm, double *Ch,
                      double *Cl_, int ldo, int mode) {
    unsigned W[OZ_MAXM][8], Mm[8];
    long long F[OZ_MAXM];
    oz_oracle_dd_consts(nm, W, Mm, F);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            const size_t o = (size_t)i * ldo + j;
            int zero;
            const dd y = crt_dd_one(Cl + (size_t)i * ldc + j, plane, nm, W, Mm, F, sa[i] + sb[j], mode, Ch[o], Cl_[o], &zero);
            if (zero) { if (mode != 1) { Ch[o] = 0; Cl_[o] = 0; } continue; }
            Ch[o] = y.hi; Cl_[o] = y.lo;
        }
}

/* src/ozaki_dd.cuh:145-155 with plan(M, N, K, nm, 106) (src/ozaki2.cuh:122-131). Dense operands (lda = K, ldb = N, ldo = N). */
int oz_oracle_ddgemm(int M, int N, int K, const double *Ah, const double *Al, const double *Bh, const double *Bl, double *Ch, double *Cl,
                     int nm, int mode) {
    if (M <= 0 || N <= 0 || K <= 0 || nm < 1 || nm > OZ_MAXM) return -2;
    const int bits = oz_oracle_bits_for(nm, K, 106);
    if (bits < 0) return -1;
    const size_t pa = (size_t)M * K, pb = (size_t)N * K, pc = (size_t)M * N;
    int8_t *Ar = calloc((size_t)nm * pa, 1), *Br = calloc((size_t)nm * pb, 1);
    int32_t *C32 = malloc((size_t)nm * pc * 4);
    int *sa = malloc((size_t)M * 4), *sb = malloc((size_t)N * 4);
    int rc = 0;
    if (!Ar || !Br || !C32 || !sa || !sb) rc = -3;
    else {
        oz_oracle_scales(Ah, M, K, K, 1, bits, sa);
        oz_oracle_scales(Bh, N, K, 1, N, bits, sb);
        oz_oracle_residues_dd(Ah, Al, M, K, K, 1, sa, nm, Ar, K, pa);
        oz_oracle_residues_dd(Bh, Bl, N, K, 1, N, sb, nm, Br, K, pb);
        for (int l = 0; l < nm; l++) oz_oracle_gemm_i8(Ar + l * pa, Br + l * pb, C32 + l * pc, M, N, K, K, K, N);
        oz_oracle_crt_dd(C32, pc, M, N, N, sa, sb, nm, Ch, Cl, N, mode);
    }
    free(Ar); free(Br); free(C32); free(sa); free(sb);
    return rc;
}

/* bench/ref_quad.cpp:6-16 -- every product and sum in __float128 (113-bit significand); |x| by comparison instead of fabsq */
void oz_oracle_ref_quad(const double *Ah, const double *Al, const double *Bh, const double *Bl, int M, int N, int K, double *Rh, double *Rl,
                        double *absAB) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            __float128 s = 0, a = 0;
            for (int k = 0; k < K; k++) {
                const __float128 p = ((__float128)Ah[(size_t)i * K + k] + Al[(size_t)i * K + k]) * ((__float128)Bh[(size_t)k * N + j] + Bl[(size_t)k * N + j]);
                s += p;
                a += p < 0 ? -p : p;
            }
            Rh[(size_t)i * N + j] = (double)s;
            Rl[(size_t)i * N + j] = (double)(s - (__float128)Rh[(size_t)i * N + j]);
            absAB[(size_t)i * N + j] = (double)a;
        }
}

/* bench/dd_test.cu:56-57 with the __float128 reference in place of the MPFR one: max |(Ch - Rh) + (Cl - Rl)| / (|A||B| 2^-106) */
double oz_oracle_dd_err_units(const double *Ch, const double *Cl, const double *Rh, const double *Rl, const double *absAB, size_t count) {
    double worst = 0;
    for (size_t t = 0; t < count; t++) {
        const double e = fabs((Ch[t] - Rh[t]) + (Cl[t] - Rl[t])) / (absAB[t] * 0x1p-106);
        if (e > worst) worst = e;
    }
    return worst;
}

/* bench/crt_check.cpp:18-35 -- the direct-sum CRT recovers known signed integers of up to 192 bits from their residues.
 * The reference draws them from std::mt19937_64(3); here the caller supplies `count` integers as 8 limbs each (two's
 * complement), so the test can use any generator. Returns how many come back wrong (the reference prints "0 of 100000"). */
int oz_oracle_dd_crt_kat(const unsigned *V, int count, int nm) {
    unsigned W[OZ_MAXM][8], Mm[8];
    long long F[OZ_MAXM];
    oz_oracle_dd_consts(nm, W, Mm, F);
    int bad = 0;
    for (int it = 0; it < count; it++) {
        const unsigned *v0 = V + 8 * (size_t)it;
        const int sgn = (int)v0[7] < 0;
        unsigned long long acc[8] = {0};
        long long qf = 0;
        for (int l = 0; l < nm; l++) {
            const int m = oz_oracle_modulus(l);
            long long x = 0;
            for (int k = 7; k >= 0; k--) x = ((x << 32) + v0[k]) % m;
            if (sgn) { long long p = 1; for (int t = 0; t < 256; t++) p = p * 2 % m; x = ((x - p) % m + m) % m; }
            qf += x * F[l];
            for (int k = 0; k < 8; k++) acc[k] += (unsigned long long)x * W[l][k];
        }
        long long q = (qf + (1ll << 39)) >> 40, c = 0;
        int same = 1;
        for (int k = 0; k < 8; k++) { c += (long long)acc[k] - q * (long long)Mm[k]; same &= (unsigned)c == v0[k]; c >>= 32; }
        bad += !same;
    }
    return bad;
}
