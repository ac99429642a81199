// dd.cu -- the double-double (~106-bit) product: the two memory-bound stages that differ from the FP64 path.
//
// What they compute is the reference's residues_dd<NM> and crt_dd<NM> (src/ozaki_dd.cuh:46-64, 93-140):
//   residues: with a = hi 2^s, b = lo 2^s (s from the hi parts, as in the FP64 path), the integer
//             V = trunc(a) + trunc(b) + rint(frac(a) + frac(b)), |V| < 2^106, and its balanced residue mod every modulus;
//   CRT:      x = sum_l r_l W_l - q P over eight 32-bit limbs (W_l = (P/m_l)((P/m_l)^-1 mod m_l), q from 40-bit fixed-point
//             fractions), the top 128 bits normalised into a double-double, scaled by 2^-(sa+sb); modes C = AB, C -= AB, C = -AB.
// The INT8 GEMMs in between are the FP64 path's kernel with 24..32 planes.
//
// How: V is kept as u 2^53 + t with two int64 (the reference's split, so the floating-point steps are the same
// operations in the same order); its residue is one signed dot product over the sixteen bytes of (u + 2^62, t + 2^62)
// -- four dp4a and one multiply-high reduction per modulus instead of the reference's eight multiplies and three
// reductions. The CRT is the reference's integer algorithm with the tables in constant memory and four outputs per thread.
#include <mutex>
#include "oz_common.cuh"

namespace ozk {

// ---------------------------------------------------------------------------------------------------------------
// tables of the direct-sum CRT (src/ozaki_dd.cuh:73-91), evaluated by the compiler
// ---------------------------------------------------------------------------------------------------------------
__constant__ DdTables<24> c_dd24 = make_dd_tables<24>();
__constant__ DdTables<28> c_dd28 = make_dd_tables<28>();
__constant__ DdTables<32> c_dd32 = make_dd_tables<32>();
template <int NM> __device__ __forceinline__ const DdTables<NM> &dd_tables();
template <> __device__ __forceinline__ const DdTables<24> &dd_tables<24>() { return c_dd24; }
template <> __device__ __forceinline__ const DdTables<28> &dd_tables<28>() { return c_dd28; }
template <> __device__ __forceinline__ const DdTables<32> &dd_tables<32>() { return c_dd32; }

// ---------------------------------------------------------------------------------------------------------------
// residues
// ---------------------------------------------------------------------------------------------------------------
constexpr int DD_BYTES_BOUND = 16 * 255 * 128;

// the reference's split of one scaled value (src/ozaki_dd.cuh:52-58): V = u 2^53 + t
__device__ __forceinline__ void dd_split(double xh, double xl, int s, double p2, bool fast, long long &u, long long &t) {
    const double a = fast ? xh * p2 : ldexp(xh, s), b = fast ? xl * p2 : ldexp(xl, s);
    const double ai = trunc(a), bi = trunc(b);
    const double f = rint((a - ai) + (b - bi));                  // |f| <= 2
    u = __double2ll_rz(ai * 0x1p-53);                            // exact scaling of an integer below 2^106
    const long long w = __double2ll_rz(ai - (double)u * 0x1p53); // exact
    t = w + __double2ll_rz(bi) + __double2ll_rz(f);
}

// residues of four consecutive values for every modulus: put(l, word of four int8)
template <int NM, class Put>
__device__ __forceinline__ void residues_of_4_dd(const long long (&u)[4], const long long (&t)[4], Put &&put) {
    uint32_t ul[4], uh[4], tl[4], th[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const unsigned long long a = (unsigned long long)u[e] + (1ull << 62), b = (unsigned long long)t[e] + (1ull << 62);
        ul[e] = (uint32_t)a; uh[e] = (uint32_t)(a >> 32); tl[e] = (uint32_t)b; th[e] = (uint32_t)(b >> 32);
    }
    put(std::integral_constant<int, 0>{}, pack_low_bytes(tl[0], tl[1], tl[2], tl[3]));   // mod 256 only t's low byte counts
    static_for<1, NM>([&](auto L) {
        constexpr int l = decltype(L)::value, m = modulus(l), p53 = pow2_mod(53, m);
        constexpr auto wu = [](int i) constexpr { return bal_c((long long)posmod_c(byte_weight(i, l), m) * p53, m); };
        constexpr uint32_t wtl = pack4(byte_weight(0, l), byte_weight(1, l), byte_weight(2, l), byte_weight(3, l));
        constexpr uint32_t wth = pack4(byte_weight(4, l), byte_weight(5, l), byte_weight(6, l), byte_weight(7, l));
        constexpr uint32_t wul = pack4(wu(0), wu(1), wu(2), wu(3)), wuh = pack4(wu(4), wu(5), wu(6), wu(7));
        // the two 2^62 offsets are taken out again: -(2^62 2^53 + 2^62) mod m, folded into the starting value
        constexpr int off = posmod_c((long long)pow2_mod(62, m) * p53 + pow2_mod(62, m), m);
        constexpr int init = lift_of(l, DD_BYTES_BOUND) - off;
        static_assert(init > DD_BYTES_BOUND && magic_ok(l, (uint64_t)init + DD_BYTES_BOUND), "multiply-high reduction out of range");
        uint32_t x[4];
#ifndef OZ_INT_REDUCE   // the reduction on the FP32 pipes (balanced_float): the sum sits on the bit pattern of 1.5 * 2^23
        constexpr int seed = FLOAT_BIAS - off;
        static_assert(DD_BYTES_BOUND + 256 < (1 << 22), "the byte sum must fit the float's mantissa");
#pragma unroll
        for (int e = 0; e < 4; e++)
            x[e] = balanced_float<l>(dp4a_us(uh[e], wuh, dp4a_us(ul[e], wul, dp4a_us(th[e], wth, dp4a_us(tl[e], wtl, seed)))));
#else
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int acc = dp4a_us(tl[e], wtl, init);
            acc = dp4a_us(th[e], wth, acc);
            acc = dp4a_us(ul[e], wul, acc);
            acc = dp4a_us(uh[e], wuh, acc);
            x[e] = mod_magic<l>((uint32_t)acc) - (uint32_t)half_of(l);
        }
#endif
        put(L, pack_low_bytes(x[0], x[1], x[2], x[3]));
    });
}

// A side: one block per row; the hi and lo rows stay in registers between the max reduction (on hi) and the split
template <int NM, int R, int MAXT>
__global__ void __launch_bounds__(MAXT) row_scale_residues_dd(const double *__restrict__ Xh, const double *__restrict__ Xl, int len,
                                                              long long ldx, int bits, int *__restrict__ s_out, int8_t *__restrict__ Rp,
                                                              int ld, size_t plane) {
    const int r = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const double *rh = Xh + (size_t)r * ldx, *rl = Xl + (size_t)r * ldx;
    const int chunks = (len + 3) >> 2;
    const bool cached = chunks <= R * nt;
    double xh[R][4], xl[R][4];
    double mx = 0;
    auto load4 = [&](const double *row, int c, double (&d)[4]) {
        const int k = c << 2;
#pragma unroll
        for (int e = 0; e < 4; e++) d[e] = k + e < len ? row[k + e] : 0.0;
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int c = i * nt + tid;
            if (c < chunks) { load4(rh, c, xh[i]); load4(rl, c, xl[i]); }
            else {
#pragma unroll
                for (int e = 0; e < 4; e++) xh[i][e] = xl[i][e] = 0.0;
            }
#pragma unroll
            for (int e = 0; e < 4; e++) mx = fmax(mx, fabs(xh[i][e]));
        }
    } else {
        for (int c = tid; c < chunks; c += nt) {
            double d[4];
            load4(rh, c, d);
#pragma unroll
            for (int e = 0; e < 4; e++) mx = fmax(mx, fabs(d[e]));
        }
    }
    __shared__ double wmax[32];
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmax(mx, __shfl_xor_sync(~0u, mx, o));
    if ((tid & 31) == 0) wmax[tid >> 5] = mx;
    __syncthreads();
    mx = wmax[0];
    for (int w = 1; w < (nt >> 5); w++) mx = fmax(mx, wmax[w]);
    const int s = scale_from_max(mx, bits);
    if (tid == 0) s_out[r] = s;
    const bool fast = s >= -1022 && s <= 1023;
    const double p2 = pow2_normal(fast ? s : 0);
    int8_t *out = Rp + (size_t)r * ld;
    auto emit = [&](int c, const double (&dh)[4], const double (&dl)[4]) {
        long long u[4], t[4];
#pragma unroll
        for (int e = 0; e < 4; e++) dd_split(dh[e], dl[e], s, p2, fast, u[e], t[e]);
        residues_of_4_dd<NM>(u, t, [&](auto L, uint32_t word) {
            *reinterpret_cast<uint32_t *>(out + decltype(L)::value * plane + ((size_t)c << 2)) = word;
        });
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int c = i * nt + tid;
            if (c < chunks) emit(c, xh[i], xl[i]);
        }
    } else {
        for (int c = tid; c < chunks; c += nt) {
            double dh[4], dl[4];
            load4(rh, c, dh);
            load4(rl, c, dl);
            emit(c, dh, dl);
        }
    }
}

// B side, pass 1: column maxima of the hi parts (same kernel idea as the FP64 path, scalar loads: any alignment)
__global__ void __launch_bounds__(256) col_absmax_dd(const double *__restrict__ X, int rows, int cols, long long ldx,
                                                     unsigned long long *__restrict__ colmax) {
    const int j = blockIdx.x * 256 + threadIdx.x;
    const int k0 = blockIdx.y * 64, k1 = min(rows, k0 + 64);
    if (j >= cols) return;
    double m0 = 0;
#pragma unroll 8
    for (int k = k0; k < k1; k++) m0 = fmax(m0, fabs(X[(size_t)k * ldx + j]));
    if (m0 != 0) atomicMax(colmax + j, (unsigned long long)__double_as_longlong(m0));
}

// B side, pass 2: residues written transposed through shared memory: tile of 32 columns x 64 k, 8 k per thread
constexpr int DT_COLS = 32, DT_K = 64, DT_PITCH = DT_K + 16;
template <int NM> constexpr int dd_tile_smem() { return NM * DT_COLS * DT_PITCH; }
template <int NM>
__global__ void __launch_bounds__(256) col_residues_t_dd(const double *__restrict__ Xh, const double *__restrict__ Xl, int rows, int cols,
                                                         long long ldx, const unsigned long long *__restrict__ colmax, int bits,
                                                         int *__restrict__ s_out, int8_t *__restrict__ Rp, int ld, size_t plane) {
    extern __shared__ __align__(16) uint8_t tile[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j0 = blockIdx.x * DT_COLS, kb = blockIdx.y * DT_K;
    {
        const int j = j0 + lane, k0 = kb + warp * 8;
        if (j < cols) {   // k beyond the matrix contributes zeros, so that every byte of a valid column's tile row is defined
            const int s = scale_from_max(__longlong_as_double((long long)colmax[j]), bits);
            if (blockIdx.y == 0 && warp == 0) s_out[j] = s;
            const bool fast = s >= -1022 && s <= 1023;
            const double p2 = pow2_normal(fast ? s : 0);
#pragma unroll
            for (int q = 0; q < 2; q++) {
                long long u[4], t[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int k = k0 + 4 * q + e;
                    const double h = k < rows ? Xh[(size_t)k * ldx + j] : 0.0, l = k < rows ? Xl[(size_t)k * ldx + j] : 0.0;
                    dd_split(h, l, s, p2, fast, u[e], t[e]);
                }
                residues_of_4_dd<NM>(u, t, [&](auto L, uint32_t word) {
                    *reinterpret_cast<uint32_t *>(tile + (decltype(L)::value * DT_COLS + lane) * DT_PITCH + warp * 8 + 4 * q) = word;
                });
            }
        }
    }
    __syncthreads();
    const int c = threadIdx.x & 3;                  // 16-byte piece of the 64-byte row
    const int kpos = kb + c * 16;
    if (kpos >= rows) return;
    for (int i = threadIdx.x >> 2; i < NM * DT_COLS; i += 64) {   // rows of the tile: (l, j)
        const int l = i / DT_COLS, j = i % DT_COLS;
        if (j0 + j < cols) {
            const uint4 v = *reinterpret_cast<const uint4 *>(tile + (l * DT_COLS + j) * DT_PITCH + c * 16);
            *reinterpret_cast<uint4 *>(Rp + (size_t)l * plane + (size_t)(j0 + j) * ld + kpos) = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// CRT: direct sum over 8 limbs (src/ozaki_dd.cuh:93-140), from the GEMM epilogue's int8 balanced residues
// ---------------------------------------------------------------------------------------------------------------
struct dd2 { double hi, lo; };
__device__ __forceinline__ dd2 two_sum(double a, double b) { const double s = a + b, v = s - a; return {s, (a - (s - v)) + (b - v)}; }
__device__ __forceinline__ dd2 quick_two_sum(double a, double b) { const double s = a + b; return {s, b - (s - a)}; }

template <int NM>
__global__ void __launch_bounds__(128) crt_dd_kernel(const int8_t *__restrict__ Cr, size_t plane, int M, int N, long long ldr,
                                                     const int *__restrict__ sa, const int *__restrict__ sb, double *__restrict__ Ch,
                                                     double *__restrict__ Cl, long long ldo, int mode) {
    const DdTables<NM> &T = dd_tables<NM>();
    const int i = blockIdx.x;
    const int j0 = (blockIdx.y * 128 + threadIdx.x) * 4;
    if (j0 >= N) return;
    uint32_t w[NM];
    const int8_t *base = Cr + (size_t)i * ldr + j0;
#pragma unroll
    for (int l = 0; l < NM; l++) w[l] = __ldg(reinterpret_cast<const uint32_t *>(base + (size_t)l * plane));
    const int si = sa[i];
#pragma unroll 1
    for (int e = 0; e < 4; e++) {
        const int j = j0 + e;
        if (j >= N) break;
        unsigned long long acc[8] = {};
        long long qf = 0;
#pragma unroll
        for (int l = 0; l < NM; l++) {
            int r = (int)(int8_t)(w[l] & 255);
            w[l] >>= 8;
            if (r < 0) r += modulus(l);                        // the reference's r in [0, m)
            qf += (long long)r * T.F[l];
#pragma unroll
            for (int k = 0; k < 8; k++) acc[k] += (unsigned long long)(unsigned)r * T.W[l][k];
        }
        const long long q = (qf + (1ll << 39)) >> 40;
        long long c = 0;
        unsigned v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) { c += (long long)acc[k] - q * (long long)T.P[k]; v[k] = (unsigned)c; c >>= 32; }
        const bool neg = (int)v[7] < 0;
        if (neg) {
            unsigned long long b = 1;
#pragma unroll
            for (int k = 0; k < 8; k++) { b += (unsigned)~v[k]; v[k] = (unsigned)b; b >>= 32; }
        }
        int top = -1;
#pragma unroll
        for (int k = 0; k < 8; k++) if (v[k]) top = k;
        const size_t o = (size_t)i * ldo + j;
        if (top < 0) { if (mode != 1) { Ch[o] = 0; Cl[o] = 0; } continue; }
        unsigned t4 = 0, t3 = 0, t2 = 0, t1 = 0, t0 = 0;
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (k == top) { t4 = v[k]; t3 = k >= 1 ? v[k - 1] : 0; t2 = k >= 2 ? v[k - 2] : 0; t1 = k >= 3 ? v[k - 3] : 0; t0 = k >= 4 ? v[k - 4] : 0; }
        const int z = __clz(t4);
        unsigned long long H = (unsigned long long)t4 << 32 | t3, Lw = (unsigned long long)t2 << 32 | t1;
        if (z) { H = H << z | Lw >> (64 - z); Lw = Lw << z | t0 >> (32 - z); }
        const double dh = __ull2double_rd(H);
        const double lo = fma((double)(H - (unsigned long long)dh), 18446744073709551616.0, (double)Lw);
        const int ex = 32 * (top - 3) - z - (si + sb[j]);
        dd2 y = quick_two_sum(ldexp(dh, ex + 64), ldexp(lo, ex));
        if (neg != (mode != 0)) y = {-y.hi, -y.lo};
        if (mode == 1) {
            dd2 s = two_sum(Ch[o], y.hi), t = two_sum(Cl[o], y.lo);
            s = quick_two_sum(s.hi, s.lo + t.hi);
            y = quick_two_sum(s.hi, s.lo + t.lo);
        }
        Ch[o] = y.hi;
        Cl[o] = y.lo;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------
#define OZ_DISPATCH_DD(nm, CALL)                                                                       \
    switch (nm) {                                                                                      \
    case 24: { constexpr int NM = 24; return CALL; }                                                   \
    case 28: { constexpr int NM = 28; return CALL; }                                                   \
    case 32: { constexpr int NM = 32; return CALL; }                                                   \
    default: return cudaErrorInvalidValue;                                                             \
    }

template <int NM>
static cudaError_t rows_dd_t(const double *Xh, const double *Xl, int rows, int len, long long ldx, int bits, int *s, int8_t *R, int ld,
                             size_t plane, cudaStream_t st) {
    constexpr int RR = 4, MAXT = 512;
    int nt = ((len + 3) / 4 + RR - 1) / RR;
    nt = (nt + 31) / 32 * 32;
    if (nt < 32) nt = 32;
    if (nt > MAXT) nt = MAXT;
    row_scale_residues_dd<NM, RR, MAXT><<<rows, nt, 0, st>>>(Xh, Xl, len, ldx, bits, s, R, ld, plane);
    return cudaGetLastError();
}
template <int NM>
static cudaError_t cols_dd_t(const double *Xh, const double *Xl, int rows, int cols, long long ldx, int bits, unsigned long long *colmax,
                             int *s, int8_t *R, int ld, size_t plane, cudaStream_t st) {
    static PerDevice pd;
    if (cudaError_t a = pd.once([] { return cudaFuncSetAttribute(col_residues_t_dd<NM>, cudaFuncAttributeMaxDynamicSharedMemorySize, dd_tile_smem<NM>()); })) return a;
    cudaError_t e = cudaMemsetAsync(colmax, 0, (size_t)cols * 8, st);
    if (e) return e;
    col_absmax_dd<<<dim3((cols + 255) / 256, (rows + 63) / 64), 256, 0, st>>>(Xh, rows, cols, ldx, colmax);
    col_residues_t_dd<NM><<<dim3((cols + DT_COLS - 1) / DT_COLS, (rows + DT_K - 1) / DT_K), 256, dd_tile_smem<NM>(), st>>>(
        Xh, Xl, rows, cols, ldx, colmax, bits, s, R, ld, plane);
    return cudaGetLastError();
}
template <int NM>
static cudaError_t crt_dd_t(const int8_t *Cr, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb, double *Ch,
                            double *Cl, long long ldo, int mode, cudaStream_t st) {
    crt_dd_kernel<NM><<<dim3(M, (N + 511) / 512), 128, 0, st>>>(Cr, plane, M, N, ldr, sa, sb, Ch, Cl, ldo, mode);
    return cudaGetLastError();
}

cudaError_t dd_scale_residues_rows(int nm, const double *Xh, const double *Xl, int rows, int len, long long ldx, int bits, int *s,
                                   int8_t *R, int ld, size_t plane, cudaStream_t st) {
    OZ_DISPATCH_DD(nm, (rows_dd_t<NM>(Xh, Xl, rows, len, ldx, bits, s, R, ld, plane, st)));
}
cudaError_t dd_scale_residues_cols(int nm, const double *Xh, const double *Xl, int rows, int cols, long long ldx, int bits,
                                   unsigned long long *colmax, int *s, int8_t *R, int ld, size_t plane, cudaStream_t st) {
    OZ_DISPATCH_DD(nm, (cols_dd_t<NM>(Xh, Xl, rows, cols, ldx, bits, colmax, s, R, ld, plane, st)));
}
cudaError_t dd_crt_from_i8(int nm, const int8_t *Cr, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb, double *Ch,
                           double *Cl, long long ldo, int mode, cudaStream_t st) {
    OZ_DISPATCH_DD(nm, (crt_dd_t<NM>(Cr, plane, M, N, ldr, sa, sb, Ch, Cl, ldo, mode, st)));
}

}  // namespace ozk
