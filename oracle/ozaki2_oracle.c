/* ozaki2_oracle.c -- CPU restatement of the reference's Ozaki scheme II FP64 GEMM, stage by stage.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA path is compared against (tests, the smoke check and the
 * CPU-baseline leg of the benchmark). Nothing in the shipped library links, loads or calls it.
 *
 * Every function restates, in plain C, one piece of the reference (paths are relative to the reference project):
 *   src/ozaki2.cuh:18-34   moduli table                      -> oz_oracle_modulus
 *   src/ozaki2.cuh:38-50   bal / balc  (balanced residue)    -> bal
 *   src/ozaki2.cuh:56-68   scales                            -> oz_oracle_scales
 *   src/ozaki2.cuh:71-78   residues<NM>                      -> oz_oracle_residues
 *   src/gemm_i8.cuh:1      C = A * Bt^T, exact in int32      -> oz_oracle_gemm_i8   (bench/gemm_i8_test.cu:23-28 is the
 *                                                               reference's own CPU statement of it)
 *   src/ozaki2.cuh:82-97   crt<NM>  (Garner, FP64 fma Horner)-> oz_oracle_crt
 *   src/ozaki2.cuh:99      inv_mod                           -> oz_oracle_inv_mod
 *   src/ozaki2.cuh:101-108 bits_for                          -> oz_oracle_bits_for
 *   src/ozaki2.cuh:116-164 plan / dgemm_t / dgemm            -> oz_oracle_dgemm
 *   bench/ozaki_test.cu:42-63  80-bit sum, Dot2 sum, |A||B|, error in units of 2^-53 -> oz_oracle_err_units
 *   bench/gemm_i8_test.cu:11-13 srand/rand inputs of the INT8 known-answer test      -> oz_oracle_fill_i8
 *
 * Compile with -O2 -ffp-contract=off (the only fused multiply-adds are the explicit fma() calls of the Horner loop, which
 * are part of the arithmetic contract: the reference's result depends on that exact sequence of roundings).
 *
 * Pinning: tests/test_oracle_golden.py runs this file on the reference's own accuracy-test inputs (same generator, same
 * seeds) and requires the published error table; on a GPU machine tests/test_reference_parity.py compares it bit for bit
 * with the reference's own kernels built from the reference sources.
 */
#ifdef _OPENMP
#include <omp.h>
#endif
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define OZ_MAXM 49

/* src/ozaki2.cuh:21-23 -- pairwise coprime, largest first */
static const int MODULI[OZ_MAXM] = {256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193,
                                    191, 181, 179, 173, 167, 163, 157, 151, 149, 139, 137, 131, 127, 113, 109, 107,
                                    103, 101, 97,  89,  83,  79,  73,  71,  67,  61,  59,  53,  47,  43,  41,  37,  29};

/* Number of OpenMP threads of the checker's loops (0: leave as is). Launchers such as torch.distributed.run export
 * OMP_NUM_THREADS=1 to their children; a caller that wants every host core back says so here. Returns the count in use. */
int oz_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

int oz_oracle_modulus(int l) { return (l >= 0 && l < OZ_MAXM) ? MODULI[l] : 0; }

/* src/ozaki2.cuh:38-42 (bal) and :46-50 (balc): C remainder, made non-negative, then folded into [-(m/2), (m+1)/2) */
static inline int bal(long long x, int m) {
    int r = (int)(x % m);
    if (r < 0) r += m;
    return r >= (m + 1) / 2 ? r - m : r;
}

/* src/ozaki2.cuh:99 -- brute-force modular inverse */
int oz_oracle_inv_mod(int a, int m) {
    for (int x = 1; x < m; x++)
        if (a * x % m == 1) return x;
    return 0;
}

/* src/ozaki2.cuh:101-108 -- bits = floor((log2 P - 2 - log2 K) / 2), capped at maxbits. The reference aborts for
 * K >= 131072; the oracle returns -1 there (the C ABI turns the same condition into an error code, python/capi.cu:25). */
int oz_oracle_bits_for(int nm, int K, int maxbits) {
    double log2P = 0;
    for (int l = 0; l < nm; l++) log2P += log2((double)MODULI[l]);
    if (K >= 131072) return -1;
    const int b = (int)floor((log2P - 2 - log2((double)K)) / 2);
    return b > maxbits ? maxbits : b;
}

/* src/ozaki2.cuh:56-68 -- s[r] = bits - 1 - ilogb(max_k |X[r,k]|), 0 for an all-zero row; X read with strides */
void oz_oracle_scales(const double *X, int rows, int len, long long sRow, long long sCol, int bits, int *s) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        double mx = 0;
        for (int k = 0; k < len; k++) mx = fmax(mx, fabs(X[r * sRow + k * sCol]));
        s[r] = mx == 0 ? 0 : bits - 1 - ilogb(mx);
    }
}

/* src/ozaki2.cuh:71-78 -- R[l][r][k] = int8(bal(llrint(ldexp(X[r,k], s[r])), m_l)); row pitch ld, plane pitch `plane`.
 * Only the M x K (or N x K) payload is written: the caller zeroes the buffer first, as plan() does (:128). */
void oz_oracle_residues(const double *X, int rows, int len, long long sRow, long long sCol, const int *s, int nm,
                        int8_t *R, int ld, size_t plane) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        for (int k = 0; k < len; k++) {
            const long long v = llrint(ldexp(X[r * sRow + k * sCol], s[r]));
            for (int l = 0; l < nm; l++) R[l * plane + (size_t)r * ld + k] = (int8_t)bal(v, MODULI[l]);
        }
}

/* src/gemm_i8.cuh:1 / bench/gemm_i8_test.cu:23-28 -- C[i,j] = sum_k A[i,k] * Bt[j,k], exact in int32 */
void oz_oracle_gemm_i8(const int8_t *A, const int8_t *Bt, int32_t *C, int M, int N, int K, int lda, int ldb, int ldc) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            const int8_t *a = A + (size_t)i * lda, *b = Bt + (size_t)j * ldb;
            int32_t acc = 0;
            for (int k = 0; k < K; k++) acc += (int32_t)a[k] * (int32_t)b[k];
            C[(size_t)i * ldc + j] = acc;
        }
}

/* src/ozaki2.cuh:82-97 -- per output element: balanced residues, Garner's mixed-radix digits (one balanced reduction per
 * step, exactly the reference's order), Horner from the top digit with FP64 fma, then ldexp by -(sa[i] + sb[j]).
 * Cl holds nm planes of pitch `plane` with row pitch ldc; C has row pitch ldC (the reference uses ldC = N). */
void oz_oracle_crt(const int32_t *Cl, size_t plane, int M, int N, int ldc, const int *sa, const int *sb, int nm,
                   double *C, int ldC) {
    int inv[OZ_MAXM][OZ_MAXM];
    memset(inv, 0, sizeof inv);
    for (int t = 0; t < nm; t++) /* src/ozaki2.cuh:112 */
        for (int l = t + 1; l < nm; l++) inv[t][l] = oz_oracle_inv_mod(MODULI[t] % MODULI[l], MODULI[l]);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            int x[OZ_MAXM];
            for (int l = 0; l < nm; l++) {
                const int m = MODULI[l];
                int v = bal(Cl[l * plane + (size_t)i * ldc + j], m);
                for (int t = 0; t < l; t++) v = bal((long long)((v - x[t]) * inv[t][l]), m);
                x[l] = v;
            }
            double y = x[nm - 1];
            for (int l = nm - 2; l >= 0; l--) y = fma(y, (double)MODULI[l], (double)x[l]);
            C[(size_t)i * ldC + j] = ldexp(y, -(sa[i] + sb[j]));
        }
}

/* The mixed-radix digits alone (no Horner), for tests of the device CRT's integer phase. x has nm ints per element. */
void oz_oracle_garner_digits(const int32_t *res, int nm, int *x) {
    for (int l = 0; l < nm; l++) {
        const int m = MODULI[l];
        int v = bal(res[l], m);
        for (int t = 0; t < l; t++) v = bal((long long)((v - x[t]) * oz_oracle_inv_mod(MODULI[t] % m, m)), m);
        x[l] = v;
    }
}

/* src/ozaki2.cuh:122-164 -- the whole product: plan (pads, zeroed residue planes), scales x2, residues x2, nm exact
 * GEMMs, CRT. A is M x K, B is K x N, C is M x N, all dense row-major. nm outside 8..16 behaves as the reference's
 * switch does (default -> 16) only through the C ABI's argument check, so the oracle simply requires 1 <= nm <= 49 and
 * callers pass 8..16. Returns 0, or -1 for K >= 131072, -2 for bad arguments, -3 when out of memory. */
int oz_oracle_dgemm(int M, int N, int K, const double *A, const double *B, double *C, int nm) {
    if (M <= 0 || N <= 0 || K <= 0 || nm < 1 || nm > OZ_MAXM) return -2;
    const int bits = oz_oracle_bits_for(nm, K, 62);
    if (bits < 0) return -1;
    const size_t pa = (size_t)M * K, pb = (size_t)N * K, pc = (size_t)M * N;
    int8_t *Ar = calloc((size_t)nm * pa, 1), *Br = calloc((size_t)nm * pb, 1);
    int32_t *Cl = malloc((size_t)nm * pc * 4);
    int *sa = malloc((size_t)M * 4), *sb = malloc((size_t)N * 4);
    int rc = 0;
    if (!Ar || !Br || !Cl || !sa || !sb) rc = -3;
    else {
        oz_oracle_scales(A, M, K, K, 1, bits, sa);
        oz_oracle_scales(B, N, K, 1, N, bits, sb); /* column j of B: element k at k*N + j (:140) */
        oz_oracle_residues(A, M, K, K, 1, sa, nm, Ar, K, pa);
        oz_oracle_residues(B, N, K, 1, N, sb, nm, Br, K, pb);
        for (int l = 0; l < nm; l++) oz_oracle_gemm_i8(Ar + l * pa, Br + l * pb, Cl + l * pc, M, N, K, K, K, N);
        oz_oracle_crt(Cl, pc, M, N, N, sa, sb, nm, C, N);
    }
    free(Ar); free(Br); free(Cl); free(sa); free(sb);
    return rc;
}

/* bench/ozaki_test.cu:42-63 -- the accuracy references and the error measure.
 * For every output: the 80-bit (long double) i-k-j sum, the exact-product double-double sum (TwoProd by fma, TwoSum,
 * kept unrounded as hi + lo), and |A||B| in long double. Returns max |C - ref| / (|A||B|) in units of 2^-53:
 * which = 0 against the Dot2 sum (the reference's err()), which = 1 against the 80-bit sum, which = 2 the distance
 * between the two references ("ref80 off by"). rows0/rows limits the check to rows [rows0, rows0 + rows). */
double oz_oracle_err_units(int M, int N, int K, const double *A, const double *B, const double *C, int which, int rows0,
                           int rows) {
    (void)M;
    long double worst = 0;
#pragma omp parallel
    {
        long double *ref = malloc((size_t)N * sizeof(long double)), *ab = malloc((size_t)N * sizeof(long double));
        double *rs = malloc((size_t)N * 8), *rc = malloc((size_t)N * 8);
        long double mine = 0;
#pragma omp for schedule(dynamic, 4)
        for (int i = rows0; i < rows0 + rows; i++) {
            for (int j = 0; j < N; j++) { ref[j] = 0; ab[j] = 0; rs[j] = 0; rc[j] = 0; }
            for (int k = 0; k < K; k++) {
                const long double a = A[(size_t)i * K + k];
                for (int j = 0; j < N; j++) {
                    const double y = B[(size_t)k * N + j];
                    ref[j] += a * y;
                    const double x = (double)a, p = x * y, e = fma(x, y, -p), s = rs[j], t = s + p, bp = t - s;
                    rs[j] = t;
                    rc[j] += ((s - (t - bp)) + (p - bp)) + e;
                    ab[j] += fabsl(a * y);
                }
            }
            for (int j = 0; j < N; j++) {
                long double d;
                if (which == 0) d = fabsl(((long double)C[(size_t)i * N + j] - rs[j]) - rc[j]);
                else if (which == 1) d = fabsl((long double)C[(size_t)i * N + j] - ref[j]);
                else d = fabsl((ref[j] - rs[j]) - rc[j]);
                d /= ab[j];
                if (d > mine) mine = d;
            }
        }
#pragma omp critical
        if (mine > worst) worst = mine;
        free(ref); free(ab); free(rs); free(rc);
    }
    return (double)(worst / 0x1p-53L);
}

/* The same measure on a list of sampled entries (for sizes where the full check takes too long): idx holds `count`
 * flattened positions i*N + j. */
double oz_oracle_err_units_sampled(int M, int N, int K, const double *A, const double *B, const double *C,
                                   const long long *idx, int count) {
    (void)M;
    long double worst = 0;
#pragma omp parallel for schedule(dynamic, 16)
    for (int q = 0; q < count; q++) {
        const long long i = idx[q] / N, j = idx[q] % N;
        double rs = 0, rc = 0;
        long double ab = 0;
        for (int k = 0; k < K; k++) {
            const double x = A[(size_t)i * K + k], y = B[(size_t)k * N + j];
            const double p = x * y, e = fma(x, y, -p), s = rs, t = s + p, bp = t - s;
            rs = t;
            rc += ((s - (t - bp)) + (p - bp)) + e;
            ab += fabsl((long double)x * y);
        }
        const long double d = fabsl(((long double)C[(size_t)i * N + j] - rs) - rc) / ab;
#pragma omp critical
        if (d > worst) worst = d;
    }
    return (double)(worst / 0x1p-53L);
}

/* bench/gemm_i8_test.cu:11-13 -- the INT8 known-answer inputs: srand(M*7 + N*3 + K), then A (M*K values) and Bt (N*K
 * values) drawn in that order as rand() % 255 - 127 (glibc's rand). */
void oz_oracle_fill_i8(int M, int N, int K, int8_t *A, int8_t *Bt) {
    srand((unsigned)(M * 7 + N * 3 + K));
    for (size_t t = 0; t < (size_t)M * K; t++) A[t] = (int8_t)(rand() % 255 - 127);
    for (size_t t = 0; t < (size_t)N * K; t++) Bt[t] = (int8_t)(rand() % 255 - 127);
}

/* bench/oz_strassen.cu:74-97 (scales_norm) -- the optional scale from the 2-norm: s = beta - 1 - (e + ilogb(sqrt(ss)(1 + 2^-30)))
 * with e = ilogb(max |x|) and ss = sum (x 2^-e)^2. The sum is accumulated exactly in the reference's order, because its last
 * bits can move the result across a power of two: 256 threads, thread t takes k = t, t + 256, ... with fma; a butterfly of
 * additions inside each warp of 32 (offsets 16, 8, 4, 2, 1); then the eight warp sums added in order. X read with strides. */
void oz_oracle_scales_norm(const double *X, int rows, int len, long long sRow, long long sCol, int beta, int *s) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        double mx = 0;
        for (int k = 0; k < len; k++) mx = fmax(mx, fabs(X[r * sRow + k * sCol]));
        if (mx == 0) { s[r] = 0; continue; }
        const int e = ilogb(mx);
        double part[256];
        for (int t = 0; t < 256; t++) {
            double ss = 0;
            for (int k = t; k < len; k += 256) { const double v = ldexp(X[r * sRow + k * sCol], -e); ss = fma(v, v, ss); }
            part[t] = ss;
        }
        double w[8];
        for (int wp = 0; wp < 8; wp++) {
            double v[32], u[32];
            for (int l = 0; l < 32; l++) v[l] = part[32 * wp + l];
            for (int o = 16; o; o >>= 1) {
                for (int l = 0; l < 32; l++) u[l] = v[l ^ o];
                for (int l = 0; l < 32; l++) v[l] = v[l] + u[l];
            }
            w[wp] = v[0];
        }
        double ss = w[0];
        for (int i = 1; i < 8; i++) ss = ss + w[i];
        s[r] = beta - 1 - (e + ilogb(sqrt(ss) * (1 + 0x1p-30)));
    }
}

/* bench/oz_strassen.cu:247 -- the bits of the 2-norm mode: floor((log2 P - 1.001) / 2), at most 62 */
int oz_oracle_bits_for_norm(int nm) {
    double l2 = 0;
    for (int l = 0; l < nm; l++) l2 += log2((double)MODULI[l]);
    const int b = (int)floor((l2 - 1.001) / 2);
    return b > 62 ? 62 : b;
}

/* the product with the 2-norm scales in place of the max-based ones (everything else as oz_oracle_dgemm) */
int oz_oracle_dgemm_norm(int M, int N, int K, const double *A, const double *B, double *C, int nm) {
    if (M <= 0 || N <= 0 || K <= 0 || nm < 1 || nm > OZ_MAXM || K >= 131072) return -2;
    const int bits = oz_oracle_bits_for_norm(nm);
    const size_t pa = (size_t)M * K, pb = (size_t)N * K, pc = (size_t)M * N;
    int8_t *Ar = calloc((size_t)nm * pa, 1), *Br = calloc((size_t)nm * pb, 1);
    int32_t *Cl = malloc((size_t)nm * pc * 4);
    int *sa = malloc((size_t)M * 4), *sb = malloc((size_t)N * 4);
    int rc = 0;
    if (!Ar || !Br || !Cl || !sa || !sb) rc = -3;
    else {
        oz_oracle_scales_norm(A, M, K, K, 1, bits, sa);
        oz_oracle_scales_norm(B, N, K, 1, N, bits, sb);
        oz_oracle_residues(A, M, K, K, 1, sa, nm, Ar, K, pa);
        oz_oracle_residues(B, N, K, 1, N, sb, nm, Br, K, pb);
        for (int l = 0; l < nm; l++) oz_oracle_gemm_i8(Ar + l * pa, Br + l * pb, Cl + l * pc, M, N, K, K, K, N);
        oz_oracle_crt(Cl, pc, M, N, N, sa, sb, nm, C, N);
    }
    free(Ar); free(Br); free(Cl); free(sa); free(sb);
    return rc;
}
