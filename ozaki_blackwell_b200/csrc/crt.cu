// crt.cu -- kernel 4 of the FP64 product: Chinese-remainder reconstruction back to FP64.
//
// What it computes is the reference's `crt<NM>` (src/ozaki2.cuh:82-97): per output element the balanced residues of the
// nm exact products, Garner's balanced mixed-radix digits x_0..x_{nm-1}, then
//     y = x_{nm-1};  y = fma(y, m_l, x_l) for l = nm-2 .. 0   (IEEE double: the sequence of roundings is part of the result)
//     C[i][j] = ldexp(y, -(sa[i] + sb[j])).
//
// How: the reference spends l modular reductions on digit l (120 at 16 moduli). Here the recurrence is unrolled into one
// signed dot product per digit (see garner_p / garner_q in oz_tables.cuh), evaluated with dp4a on digits packed four to
// a register, and reduced once: 39 dp4a and 15 multiply-high reductions per element; a thread runs its four elements in
// lockstep so that they share the coefficient words. The digits are the same integers
// (a balanced digit is unique in its residue class), so the FP64 Horner loop sees the same operands in the same order.
// Input is either the GEMM epilogue's int8 planes of already balanced residues (16 bytes per element at 16 moduli
// instead of 64) or, for the reference's layout, int32 planes of raw products.
#include "oz_common.cuh"
#include "oz_bounds.cuh"

namespace ozk {

// 4 x 4 byte transpose: in[p] holds plane p of elements 0..3; out[e] holds planes 0..3 of element e
__device__ __forceinline__ void transpose4x4(const uint32_t (&in)[4], uint32_t (&out)[4]) {
    const uint32_t a = __byte_perm(in[0], in[1], 0x5140), b = __byte_perm(in[0], in[1], 0x7362);   // (p0e0 p1e0 p0e1 p1e1), (.. e2 e3)
    const uint32_t c = __byte_perm(in[2], in[3], 0x5140), d = __byte_perm(in[2], in[3], 0x7362);
    out[0] = __byte_perm(a, c, 0x5410);
    out[1] = __byte_perm(a, c, 0x7632);
    out[2] = __byte_perm(b, d, 0x5410);
    out[3] = __byte_perm(b, d, 0x7632);
}

// Garner digits of E elements in lockstep, in place: on entry X[e][g] holds the balanced residues r_{4g}..r_{4g+3} of
// element e as int8 (unused bytes zero), on exit the balanced mixed-radix digits x_{4g}..x_{4g+3}. Running the elements
// side by side lets them share every coefficient word and keeps the state to (NM+3)/4 registers per element.
template <int NM, int E>
__device__ __forceinline__ void garner_digits(uint32_t (&X)[E][(NM + 3) / 4]) {
    static_for<1, NM>([&](auto L) {   // digit 0 is the residue mod 256 itself
        constexpr int l = decltype(L)::value;
        constexpr int lift = lift_of(l, GARNER_BOUND) - half_of(l);   // a multiple of m_l; the balancing shift is folded into balanced_magic
        static_assert(lift > GARNER_BOUND && magic_ok(l, (uint64_t)lift + half_of(l) + GARNER_BOUND), "multiply-high reduction out of range");
        int acc[E];
#ifndef OZ_INT_REDUCE
        static_assert(GARNER_BOUND < (1 << 22), "the dot product must fit the float's mantissa");
#pragma unroll
        for (int e = 0; e < E; e++) acc[e] = FLOAT_BIAS;
#else
#pragma unroll
        for (int e = 0; e < E; e++) acc[e] = lift;
#endif
        // digits x_0..x_{l-1} have already replaced the residues in the low bytes; byte l still holds r_l
        static_for<0, l / 4 + 1>([&](auto G) {
            constexpr int g = decltype(G)::value;
            constexpr auto coef = [](int idx) constexpr { return idx < l ? garner_q(idx, l) : (idx == l ? garner_p(l) : 0); };
            constexpr uint32_t cw = pack4(coef(4 * g), coef(4 * g + 1), coef(4 * g + 2), coef(4 * g + 3));
#pragma unroll
            for (int e = 0; e < E; e++) acc[e] = dp4a_ss(X[e][g], cw, acc[e]);
        });
        constexpr uint32_t sel = l % 4 == 0 ? 0x3214u : l % 4 == 1 ? 0x3240u : l % 4 == 2 ? 0x3410u : 0x4210u;
        uint32_t xl[E];                                                                  // balanced digits, low bytes
#ifndef OZ_INT_REDUCE
        static_assert(E % 2 == 0, "the elements are reduced in pairs");
#pragma unroll
        for (int e = 0; e < E; e += 2) balanced_float_x2<l>(acc[e], acc[e + 1], xl[e], xl[e + 1]);
#else
#pragma unroll
        for (int e = 0; e < E; e++) xl[e] = balanced_magic<l>((uint32_t)acc[e]);
#endif
#pragma unroll
        for (int e = 0; e < E; e++) X[e][l / 4] = __byte_perm(X[e][l / 4], xl[e], sel);     // byte l%4 <- xl
    });
}

// digit l of a packed word of BIASED digits (x + 128, an unsigned byte) as a double: the byte moved into the low word of
// 2^52 (one permute), minus 2^52 + 128 (one add)
template <int B>
__device__ __forceinline__ double digit_to_double(uint32_t biased) {
#ifdef OZ_OLD_DIGIT_CONV   // the earlier form, on the unbiased word: sign-extend the byte, flip the top bit, subtract 2^52 + 2^31
    constexpr uint32_t sel = B == 0 ? 0x8880u : B == 1 ? 0x9991u : B == 2 ? 0xAAA2u : 0xBBB3u;
    uint32_t v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(biased ^ 0x80808080u), "r"(0u), "r"(sel));
    return __hiloint2double(0x43300000, (int)(v ^ 0x80000000u)) - 4503601774854144.0;
#else
    return __hiloint2double(0x43300000, (int)__byte_perm(biased, 0u, 0x4440u + B)) - 4503599627370624.0;   // 2^52 + 128
#endif
}

// the reference's Horner loop (src/ozaki2.cuh:93-95) on the packed digits of one element
template <int NM>
__device__ __forceinline__ double horner(const uint32_t (&X)[(NM + 3) / 4]) {
    uint32_t Bx[(NM + 3) / 4];
#pragma unroll
    for (int g = 0; g < (NM + 3) / 4; g++) Bx[g] = X[g] ^ 0x80808080u;   // int8 digits -> biased bytes, four at a time
    double y = digit_to_double<(NM - 1) % 4>(Bx[(NM - 1) / 4]);
    static_for<1, NM>([&](auto I) {
        constexpr int l = NM - 1 - decltype(I)::value;
        y = fma(y, (double)modulus(l), digit_to_double<l % 4>(Bx[l / 4]));
    });
    return y;
}

// ldexp(y, e) as the reference applies it (src/ozaki2.cuh:96). For e in the normal exponent range 2^e is a double and the
// product y * 2^e is a single correctly rounded operation, which is what ldexp returns (exact unless the result is
// subnormal, rounded once if it is, infinite on overflow); other exponents take ldexp itself.
__device__ __forceinline__ double unscale(double y, int e) {
    return (e >= -1022 && e <= 1023) ? y * pow2_normal(e) : ldexp(y, e);
}

// balanced residue of a raw int32 product (reference layout of the planes)
template <int L>
__device__ __forceinline__ int balanced_of_i32(int32_t x) {
    constexpr int m = modulus(L);
    int r = x % m;
    if (r < 0) r += m;
    return r >= (m + 1) / 2 ? r - m : r;
}

// Each thread reconstructs four consecutive columns of one row.
// In = int8_t: planes of balanced residues, row pitch ldr bytes (multiple of 4), plane pitch `plane` bytes.
// In = int32_t: planes of raw products, row pitch ldr elements, plane pitch `plane` elements.
template <int NM, class In>
__global__ void __launch_bounds__(256) crt_kernel(const In *__restrict__ Cp, size_t plane, int M, int N, long long ldr,
                                                  const int *__restrict__ sa, const int *__restrict__ sb,
                                                  double *__restrict__ C, long long ldc) {
    constexpr int G = (NM + 3) / 4;
    const int i = blockIdx.x;
    const int j0 = (blockIdx.y * 256 + threadIdx.x) * 4;
    if (j0 >= N) return;
    uint32_t E[4][G];   // E[e][g]: residues 4g..4g+3 of element j0 + e
    if constexpr (sizeof(In) == 1) {
        const int8_t *base = reinterpret_cast<const int8_t *>(Cp) + (size_t)i * ldr + j0;
#pragma unroll
        for (int g = 0; g < G; g++) {
            uint32_t w[4], t[4];
#pragma unroll
            for (int p = 0; p < 4; p++)
                w[p] = 4 * g + p < NM ? oz_load(reinterpret_cast<const uint32_t *>(base + (size_t)(4 * g + p) * plane)) : 0u;
            transpose4x4(w, t);
#pragma unroll
            for (int e = 0; e < 4; e++) E[e][g] = t[e];
        }
    } else {
        const int32_t *base = reinterpret_cast<const int32_t *>(Cp) + (size_t)i * ldr + j0;
#pragma unroll
        for (int e = 0; e < 4; e++) {
#pragma unroll
            for (int g = 0; g < G; g++) E[e][g] = 0;
            if (j0 + e < N) {
                static_for<0, NM>([&](auto L) {
                    constexpr int l = decltype(L)::value;
                    const int r = balanced_of_i32<l>(oz_load(base + (size_t)l * plane + e));
                    E[e][l / 4] |= (uint32_t)(r & 255) << (8 * (l % 4));
                });
            }
        }
    }
    garner_digits<NM, 4>(E);
    const int si = oz_load(sa + i);
    double out[4];
#pragma unroll
    for (int e = 0; e < 4; e++) out[e] = j0 + e < N ? unscale(horner<NM>(E[e]), -(si + oz_load(sb + j0 + e))) : 0.0;
    double *dst = C + (size_t)i * ldc + j0;
    if (j0 + 3 < N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        oz_store(reinterpret_cast<double2 *>(dst), make_double2(out[0], out[1]));
        oz_store(reinterpret_cast<double2 *>(dst) + 1, make_double2(out[2], out[3]));
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (j0 + e < N) oz_store(dst + e, out[e]);
    }
}

template <int NM, class In>
static cudaError_t launch_crt_t(const In *Cp, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb, double *C,
                                long long ldc, cudaStream_t st) {
    // the int8 planes are read a 4-byte word at a time (rows readable up to the next multiple of 4 columns)
    OZ_WINDOWS(st, OZK_CRT, window3d(Cp, NM, plane * sizeof(In), M, (size_t)ldr * sizeof(In), sizeof(In) == 1 ? (size_t)(N + 3) / 4 * 4 : (size_t)N * 4),
               window1d(sa, (size_t)M * 4), window1d(sb, (size_t)N * 4), window2d(C, M, (size_t)ldc * 8, (size_t)N * 8));
    crt_kernel<NM, In><<<dim3(M, (N + 1023) / 1024), 256, 0, st>>>(Cp, plane, M, N, ldr, sa, sb, C, ldc);
    return cudaGetLastError();
}

#define OZ_DISPATCH_NM(nm, CALL)                                                                                  \
    switch (nm) {                                                                                                 \
    case 8: { constexpr int NM = 8; return CALL; }    case 9: { constexpr int NM = 9; return CALL; }              \
    case 10: { constexpr int NM = 10; return CALL; }  case 11: { constexpr int NM = 11; return CALL; }            \
    case 12: { constexpr int NM = 12; return CALL; }  case 13: { constexpr int NM = 13; return CALL; }            \
    case 14: { constexpr int NM = 14; return CALL; }  case 15: { constexpr int NM = 15; return CALL; }            \
    case 16: { constexpr int NM = 16; return CALL; }                                                              \
    default: return cudaErrorInvalidValue;                                                                        \
    }

// planes of balanced int8 residues [nm][M][ldr] (ldr a multiple of 4, rows readable up to the next multiple of 4 columns)
cudaError_t crt_from_i8(int nm, const int8_t *Cr, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
                        double *C, long long ldc, cudaStream_t st) {
    OZ_DISPATCH_NM(nm, (launch_crt_t<NM, int8_t>(Cr, plane, M, N, ldr, sa, sb, C, ldc, st)));
}
// planes of raw int32 products [nm][M][ldr], the reference's layout (src/ozaki2.cuh:146)
cudaError_t crt_from_i32(int nm, const int32_t *Cl, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
                         double *C, long long ldc, cudaStream_t st) {
    OZ_DISPATCH_NM(nm, (launch_crt_t<NM, int32_t>(Cl, plane, M, N, ldr, sa, sb, C, ldc, st)));
}

// violations the checked accesses of this file recorded since the last call (debug build; zeros otherwise)
cudaError_t crt_violations(unsigned long long out[4]) { return oz_read_violations(out); }

}  // namespace ozk
