// exact_f8.cu -- correctly rounded product of BF16 activations and block-scaled FP8 (E4M3) weights:
//     Y[i][j] = RN_fp32( sum_k X[i][k] * W[k][j] * S[k / 128][j / 128] )        X: M x K bf16, W: K x N e4m3, S: FP32 per 128 x 128 block
// every output the round-to-nearest-even FP32 value of the EXACT sum. This is the contract of the reference's tiled exact
// products (llm/tgemm.cu:61-162, F8 mode: FP8 weights with one scale per 128 x 128 block, BF16 activations) checked
// against its host superaccumulator (llm/ultra.cu:336-369); the operand decodings are those of llm/ultra.cu:45-62.
//
// How it is computed here differs from the reference (digit planes, 128-bit windows, certificates on every output): all
// three operands are dyadic, so after one power-of-two scale per row of X and per column block of W*S every term is an
// integer, and the product is an integer GEMM done exactly by the same machinery as the FP64 path:
//   1. x_stats: per row of X the exponent range of its non-zero entries -> a row scale that makes X' = X 2^-base an
//      int64 (window of 62 bits; entries below the window are truncated and counted);
//   2. on the host, from the few thousand block scales: per column block a scale and an integer multiplier per block,
//      W' = (E4M3 * 2^9) * multiplier, int64 as well;
//   3. the modulus count nm (8..19) is chosen so that the product of the moduli exceeds twice the largest possible
//      |sum X' W'|; residues of X' and W' (W' transposed to K-contiguous), the tcgen05 INT8 GEMMs with their fused
//      reduction, as in the FP64 product;
//   4. crt_round: the exact integer by the direct-sum CRT over six 32-bit limbs, then one rounding to FP32 (subnormals
//      and overflow included). Where entries were truncated in step 1 or 2, the rounding is certified against the bound
//      on what was dropped: an output whose rounding the bound leaves open is returned as NaN and counted.
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "oz_common.cuh"
#include "oz_kernels.h"

namespace ozk {
namespace xf8 {

constexpr int NMAX = 19, NL = 6, WINDOW = 62, SCALE_WINDOW = 44;

// direct-sum CRT tables for nm = 8..NMAX moduli, six limbs (the product of 19 moduli has 148 bits)
struct Tables {
    unsigned W[NMAX][NL];
    unsigned P[NL];
    long long F[NMAX];
};
constexpr void mul_small6(unsigned (&a)[NL], unsigned m) {
    unsigned long long c = 0;
    for (int k = 0; k < NL; k++) { c += (unsigned long long)a[k] * m; a[k] = (unsigned)c; c >>= 32; }
}
constexpr Tables make_tables(int nm) {
    Tables t{};
    t.P[0] = 1;
    for (int l = 0; l < nm; l++) mul_small6(t.P, (unsigned)modulus(l));
    for (int l = 0; l < nm; l++) {
        const int ml = modulus(l);
        int r = 1;
        t.W[l][0] = 1;
        for (int s = 0; s < nm; s++)
            if (s != l) { mul_small6(t.W[l], (unsigned)modulus(s)); r = r * (modulus(s) % ml) % ml; }
        const int w = inv_mod_c(r, ml);
        mul_small6(t.W[l], (unsigned)w);
        t.F[l] = (long long)((double)w / ml * 1099511627776.0 + 0.5);
    }
    return t;
}
__constant__ Tables c_tab[NMAX - 7] = {make_tables(8),  make_tables(9),  make_tables(10), make_tables(11), make_tables(12), make_tables(13),
                                       make_tables(14), make_tables(15), make_tables(16), make_tables(17), make_tables(18), make_tables(19)};

struct RowInfo { int base, bits, ndrop, pad; };   // X'[i][k] = X[i][k] * 2^-base; largest |X'| < 2^bits; entries truncated
struct ColInfo { int base, bits, ndrop, pad; };   // per column block: W'[k][j] = v * mult, (W S)[k][j] = W' * 2^(base - 9)

__device__ __forceinline__ void decode_bf16(unsigned u, int &m, int &e) {   // value = m 2^e (llm/ultra.cu:48-50)
    const int ex = (u >> 7) & 255, f = u & 127;
    m = ex ? 128 + f : f;
    e = ex ? ex - 134 : -133;
    if (u >> 15) m = -m;
}
__device__ __forceinline__ int decode_e4m3(unsigned b) {   // E4M3 * 2^9 as an integer (llm/tgemm.cu:38)
    const int ex = (b >> 3) & 15, f = b & 7;
    const int v = ex ? (8 + f) << (ex - 1) : f;
    return (b & 0x80) ? -v : v;
}

// ---- 1. row statistics ----
__global__ void __launch_bounds__(256) x_stats(const uint16_t *__restrict__ X, int K, long long ldx, RowInfo *__restrict__ info,
                                               int *__restrict__ global) {   // global[0] = max bits, global[1] = non-finite count
    const int i = blockIdx.x;
    const uint16_t *row = X + (size_t)i * ldx;
    int lo = INT_MAX, hi = INT_MIN, bad = 0;
    for (int k = threadIdx.x; k < K; k += 256) {
        const unsigned u = row[k];
        if (((u >> 7) & 255) == 255) { bad++; continue; }
        int m, e;
        decode_bf16(u, m, e);
        if (m) { lo = min(lo, e); hi = max(hi, e + 32 - __clz(abs(m))); }
    }
    __shared__ int slo[8], shi[8], sbad[8], sbase;
    for (int o = 16; o; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(~0u, lo, o));
        hi = max(hi, __shfl_xor_sync(~0u, hi, o));
        bad += __shfl_xor_sync(~0u, bad, o);
    }
    if ((threadIdx.x & 31) == 0) { slo[threadIdx.x >> 5] = lo; shi[threadIdx.x >> 5] = hi; sbad[threadIdx.x >> 5] = bad; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) { lo = min(lo, slo[w]); hi = max(hi, shi[w]); bad += sbad[w]; }
        int base = 0, bits = 0;
        if (hi != INT_MIN) { base = hi - lo <= WINDOW ? lo : hi - WINDOW; bits = hi - base; }
        sbase = (hi != INT_MIN && hi - lo > WINDOW) ? base : INT_MIN;
        info[i].base = base; info[i].bits = bits; info[i].ndrop = 0; info[i].pad = 0;
        atomicMax(&global[0], bits);
        if (bad) atomicAdd(&global[1], bad);
    }
    __syncthreads();
    if (sbase != INT_MIN) {   // rare: the row spans more than the window; count what will be truncated
        int n = 0;
        for (int k = threadIdx.x; k < K; k += 256) {
            int m, e;
            decode_bf16(row[k], m, e);
            if (m && e < sbase && ((row[k] >> 7) & 255) != 255) n++;
        }
        for (int o = 16; o; o >>= 1) n += __shfl_xor_sync(~0u, n, o);
        if ((threadIdx.x & 31) == 0 && n) atomicAdd(&info[i].ndrop, n);
    }
}

// residues of four int64 for the first nm (<= NMAX) moduli
template <class Put>
__device__ __forceinline__ void residues_of_4_n(const long long (&v)[4], int nm, Put &&put) {
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const unsigned long long w = (unsigned long long)v[e] + (1ull << 62);
        lo[e] = (uint32_t)w;
        hi[e] = (uint32_t)(w >> 32);
    }
    put(0, pack_low_bytes(lo[0], lo[1], lo[2], lo[3]));
    static_for<1, NMAX>([&](auto L) {
        constexpr int l = decltype(L)::value, m = modulus(l);
        if (l < nm) {
            constexpr uint32_t wlo = pack4(byte_weight(0, l), byte_weight(1, l), byte_weight(2, l), byte_weight(3, l));
            constexpr uint32_t whi = pack4(byte_weight(4, l), byte_weight(5, l), byte_weight(6, l), byte_weight(7, l));
            constexpr int init = lift_of(l, BYTES_BOUND) - pow2_mod(62, m);
            static_assert(init > BYTES_BOUND && magic_ok(l, (uint64_t)init + BYTES_BOUND), "multiply-high reduction out of range");
            uint32_t x[4];
#ifndef OZ_INT_REDUCE   // the reduction on the FP32 pipes (balanced_float)
            constexpr int seed = FLOAT_BIAS - pow2_mod(62, m);
            static_assert(BYTES_BOUND + 256 < (1 << 22), "the byte sum must fit the float's mantissa");
#pragma unroll
            for (int e = 0; e < 4; e++) x[e] = balanced_float<l>(dp4a_us(hi[e], whi, dp4a_us(lo[e], wlo, seed)));
#else
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const uint32_t u = (uint32_t)dp4a_us(hi[e], whi, dp4a_us(lo[e], wlo, init));
                x[e] = mod_magic<l>(u) - (uint32_t)half_of(l);
            }
#endif
            put(l, pack_low_bytes(x[0], x[1], x[2], x[3]));
        }
    });
}

__device__ __forceinline__ long long scaled_bf16(unsigned u, int base) {   // X * 2^-base as an integer, truncated toward zero
    int m, e;
    decode_bf16(u, m, e);
    const int sh = e - base;
    if (sh >= 0) return (long long)m << sh;
    if (sh <= -9) return 0;
    const int a = abs(m) >> (-sh);
    return m < 0 ? -a : a;
}

// ---- 3a. residues of X', one block per row, four k per thread and step ----
__global__ void __launch_bounds__(256) x_residues(const uint16_t *__restrict__ X, int K, long long ldx, const RowInfo *__restrict__ info, int nm,
                                                  int8_t *__restrict__ Rp, int ld, size_t plane) {
    const int i = blockIdx.x;
    const uint16_t *row = X + (size_t)i * ldx;
    const int base = info[i].base;
    int8_t *out = Rp + (size_t)i * ld;
    for (int c = threadIdx.x; 4 * c < K; c += 256) {
        long long v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = 4 * c + e < K ? scaled_bf16(row[4 * c + e], base) : 0;
        residues_of_4_n(v, nm, [&](int l, uint32_t word) { *reinterpret_cast<uint32_t *>(out + (size_t)l * plane + 4 * (size_t)c) = word; });
    }
}

// ---- 3b. residues of W' = (E4M3 2^9) * multiplier, written transposed (K contiguous) through shared memory ----
// Block: 256 threads, tile of 128 columns x 32 k (inside one 128 x 128 scale block). Phase 1: lane = columns lane, lane +
// 32, lane + 64, lane + 96 of the tile (every load instruction of a warp reads one 32-byte sector), warp w owns k in
// [4w, 4w + 4): each thread forms four W' per column and parks their residues, four k to a word, in S[l][j][k], rows of
// nine words (an odd pitch: neighbouring columns fall into different banks). Phase 2: eight threads per 32-byte row
// write the tile out, a full sector per row.
constexpr int WT_COLS = 128, WT_K = 32, WT_PITCH = WT_K + 4;
__global__ void __launch_bounds__(256) w_residues_t(const uint8_t *__restrict__ W, int K, int N, long long ldw, const long long *__restrict__ mult,
                                                    int nbj, int nm, int8_t *__restrict__ Rp, int ld, size_t plane) {
    extern __shared__ __align__(16) uint8_t tile[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j0 = blockIdx.x * WT_COLS, kb = blockIdx.y * WT_K, k0 = kb + warp * 4;
    const long long mu = mult[(size_t)(kb / 128) * nbj + j0 / 128];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const int jj = lane + 32 * c, j = j0 + jj;
        if (j < N) {
            long long v[4];
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] = k0 + e < K ? (long long)decode_e4m3(W[(size_t)(k0 + e) * ldw + j]) * mu : 0;
            residues_of_4_n(v, nm, [&](int l, uint32_t word) {
                *reinterpret_cast<uint32_t *>(tile + (l * WT_COLS + jj) * WT_PITCH + warp * 4) = word;
            });
        }
    }
    __syncthreads();
    const int c = threadIdx.x & 7, kpos = kb + c * 4;
    if (kpos >= K) return;
    for (int i = threadIdx.x >> 3; i < nm * WT_COLS; i += 32) {   // rows of the tile: (l, j)
        const int l = i / WT_COLS, jj = i % WT_COLS;
        if (j0 + jj < N)
            *reinterpret_cast<uint32_t *>(Rp + (size_t)l * plane + (size_t)(j0 + jj) * ld + kpos) =
                *reinterpret_cast<const uint32_t *>(tile + (l * WT_COLS + jj) * WT_PITCH + c * 4);
    }
}

// ---- 4. exact integer, one rounding ----
// |value| = mag * 2^E (mag as six limbs, least significant first) rounded to FP32, nearest even, subnormals and overflow included
__device__ __forceinline__ float round_limbs(const unsigned (&v)[NL], int E) {
    int top = -1;
#pragma unroll
    for (int k = 0; k < NL; k++) if (v[k]) top = k;
    if (top < 0) return 0.f;
    unsigned t4 = 0, t3 = 0, t2 = 0, t1 = 0, t0 = 0, lower = 0;
#pragma unroll
    for (int k = 0; k < NL; k++) {
        if (k == top) { t4 = v[k]; t3 = k >= 1 ? v[k - 1] : 0; t2 = k >= 2 ? v[k - 2] : 0; t1 = k >= 3 ? v[k - 3] : 0; t0 = k >= 4 ? v[k - 4] : 0; }
        if (k + 5 <= top) lower |= v[k];
    }
    const int z = __clz(t4);
    unsigned long long H = (unsigned long long)t4 << 32 | t3, Lw = (unsigned long long)t2 << 32 | t1;
    unsigned rest = t0;
    if (z) { H = H << z | Lw >> (64 - z); Lw = Lw << z | t0 >> (32 - z); rest = t0 << z; }
    const int msb = 32 * top + 31 - z + E;                      // exponent of the leading bit
    const int lsb = max(msb - 23, -149);                        // exponent of the last bit FP32 keeps
    const int keep = msb - lsb + 1;                             // 24 for normal results, fewer (possibly <= 0) below 2^-126
    if (keep < 0) return 0.f;
    unsigned q = keep > 0 ? (unsigned)(H >> (64 - keep)) : 0u;
    const unsigned half = (unsigned)(H >> (63 - keep)) & 1u;
    const bool sticky = (H & ((1ull << (63 - keep)) - 1)) != 0 || Lw != 0 || rest != 0 || lower != 0;
    if (half && (sticky || (q & 1u))) q++;
    return ldexpf((float)q, lsb);                                // q <= 2^24: exact; overflow gives infinity
}
// mag +- 2^d (d < 190); returns false if the difference would be <= 0
__device__ __forceinline__ void add_pow2(unsigned (&v)[NL], int d) {
    unsigned long long c = 0;
#pragma unroll
    for (int k = 0; k < NL; k++) { c += (unsigned long long)v[k] + (k == (d >> 5) ? 1ull << (d & 31) : 0ull); v[k] = (unsigned)c; c >>= 32; }
}
__device__ __forceinline__ bool sub_pow2(unsigned (&v)[NL], int d) {
    long long c = 0;
#pragma unroll
    for (int k = 0; k < NL; k++) { c += (long long)v[k] - (k == (d >> 5) ? (long long)(1ull << (d & 31)) : 0ll); v[k] = (unsigned)c; c >>= 32; }
    return c >= 0;
}

template <int LIMBS>   // limbs the product of the nm moduli needs: 4 up to 15 moduli (118 bits), 5 up to 19 (148 bits)
__global__ void __launch_bounds__(128) crt_round(const int8_t *__restrict__ Cr, size_t plane, int M, int N, long long ldr, int nm,
                                                 const RowInfo *__restrict__ rinfo, const ColInfo *__restrict__ cinfo, float *__restrict__ Y,
                                                 long long ldy, int *__restrict__ open) {
    const Tables &T = c_tab[nm - 8];
    const int i = blockIdx.x;
    const int j0 = (blockIdx.y * 128 + threadIdx.x) * 4;
    if (j0 >= N) return;
    uint32_t w[NMAX];
    const int8_t *base = Cr + (size_t)i * ldr + j0;
#pragma unroll
    for (int l = 0; l < NMAX; l++) w[l] = l < nm ? __ldg(reinterpret_cast<const uint32_t *>(base + (size_t)l * plane)) : 0u;
    const RowInfo ri = rinfo[i];
    const ColInfo ci = cinfo[j0 / 128];                 // four consecutive columns starting at a multiple of 4: one block
    const int E = ri.base + ci.base - 9;
    // bound on what truncation dropped, in units of 2^E, as a power of two (0: nothing was truncated)
    int d = -1;
    {   // truncated X entries matter only against non-zero W', truncated multipliers only against a non-zero row of X'
        const int dx = (ri.ndrop && ci.bits) ? 32 - __clz(ri.ndrop) + ci.bits : -1;
        const int dw = (ci.ndrop && ri.bits) ? 32 - __clz(ci.ndrop) + 25 + ri.bits : -1;
        if (dx >= 0 || dw >= 0) d = max(dx, dw) + 2;
    }
    float out[4];
#pragma unroll 1
    for (int e = 0; e < 4; e++) {
        unsigned long long acc[LIMBS] = {};
        long long qf = 0;
#pragma unroll
        for (int l = 0; l < NMAX; l++) {
            if (l < nm) {
                int r = (int)(int8_t)(w[l] & 255);
                w[l] >>= 8;
                if (r < 0) r += modulus(l);
                qf += (long long)r * T.F[l];
#pragma unroll
                for (int k = 0; k < LIMBS; k++) acc[k] += (unsigned long long)(unsigned)r * T.W[l][k];
            }
        }
        const long long q = (qf + (1ll << 39)) >> 40;
        long long c = 0;
        unsigned v[NL];   // two's complement over LIMBS limbs, then sign-extended to NL for the shared rounding code
#pragma unroll
        for (int k = 0; k < LIMBS; k++) { c += (long long)acc[k] - q * (long long)T.P[k]; v[k] = (unsigned)c; c >>= 32; }
#pragma unroll
        for (int k = LIMBS; k < NL; k++) v[k] = (int)v[LIMBS - 1] < 0 ? 0xFFFFFFFFu : 0u;
        const bool neg = (int)v[NL - 1] < 0;
        if (neg) {
            unsigned long long b = 1;
#pragma unroll
            for (int k = 0; k < NL; k++) { b += (unsigned)~v[k]; v[k] = (unsigned)b; b >>= 32; }
        }
        float y = round_limbs(v, E);
        if (d >= 0) {   // certify: both ends of [mag - 2^d, mag + 2^d] must round to the same value
            unsigned lo[NL], hi[NL];
#pragma unroll
            for (int k = 0; k < NL; k++) { lo[k] = v[k]; hi[k] = v[k]; }
            add_pow2(hi, d);
            const bool pos = sub_pow2(lo, d);
            if (!pos || round_limbs(lo, E) != round_limbs(hi, E)) { y = __int_as_float(0x7fc00000); atomicAdd(open, 1); }
        }
        out[e] = neg ? -y : y;
    }
    float *dst = Y + (size_t)i * ldy + j0;
#pragma unroll
    for (int e = 0; e < 4; e++)
        if (j0 + e < N) dst[e] = out[e];
}

// workspace kept between calls of the same shape
struct Work {
    int M = 0, N = 0, K = 0, nm = 0, Kp = 0, Np = 0, dev = -1;
    int8_t *Xr = nullptr, *Wr = nullptr, *Cr = nullptr;
    RowInfo *rinfo = nullptr;
    ColInfo *cinfo = nullptr;
    long long *mult = nullptr;
    int *global = nullptr, *status = nullptr;   // global: max bits, non-finite count, open count
    void release() {
        cudaFree(Xr); cudaFree(Wr); cudaFree(Cr); cudaFree(rinfo); cudaFree(cinfo); cudaFree(mult); cudaFree(global); cudaFree(status);
        *this = Work();
    }
};
static Work work;

}  // namespace xf8

void exact_f8_release() { xf8::work.release(); }

// Device pointers; synchronous (the modulus count depends on the data). Returns 0 or a cudaError_t / OZB_E* value;
// *open = outputs returned as NaN because truncation left their rounding undecided; *moduli = planes used.
int exact_bf16_fp8_gemm(int M, int N, int K, const uint16_t *X, long long ldx, const uint8_t *W, long long ldw, const float *S, float *Y,
                        long long ldy, int *open, int *moduli, cudaStream_t st) {
    using namespace xf8;
    const int nbk = (K + 127) / 128, nbj = (N + 127) / 128;
    // 2. block scales on the host
    std::vector<float> hs((size_t)nbk * nbj);
    cudaError_t e = cudaMemcpyAsync(hs.data(), S, hs.size() * 4, cudaMemcpyDeviceToHost, st);
    if (!e) e = cudaStreamSynchronize(st);
    if (e) return (int)e;
    std::vector<long long> hmult((size_t)nbk * nbj, 0);
    std::vector<ColInfo> hc(nbj);
    int maxbitsW = 0;
    for (int jb = 0; jb < nbj; jb++) {
        int lo = INT_MAX, hi = INT_MIN;
        for (int kb = 0; kb < nbk; kb++) {
            uint32_t u; memcpy(&u, &hs[(size_t)kb * nbj + jb], 4);
            const int ex = (u >> 23) & 255, f = u & 0x7FFFFF;
            if (ex == 255) return 10001;   // OZB_EARG: non-finite scale
            const int sig = ex ? (1 << 23) + f : f, es = ex ? ex - 150 : -149;
            if (sig) { lo = std::min(lo, es); hi = std::max(hi, es + 32 - __builtin_clz((unsigned)sig)); }
        }
        ColInfo ci{0, 0, 0, 0};
        if (hi != INT_MIN) {
            ci.base = hi - lo <= SCALE_WINDOW ? lo : hi - SCALE_WINDOW;
            ci.bits = 18 + hi - ci.base;
            for (int kb = 0; kb < nbk; kb++) {
                uint32_t u; memcpy(&u, &hs[(size_t)kb * nbj + jb], 4);
                const int ex = (u >> 23) & 255, f = u & 0x7FFFFF;
                const long long sig = ex ? (1 << 23) + f : f;
                const int es = ex ? ex - 150 : -149, sh = es - ci.base;
                long long mu = 0;
                if (sig) {
                    if (sh >= 0) mu = sig << sh;
                    else { mu = sh > -25 ? sig >> (-sh) : 0; ci.ndrop++; }   // truncated toward zero: error below one unit
                }
                hmult[(size_t)kb * nbj + jb] = (u >> 31) ? -mu : mu;
            }
        }
        hc[jb] = ci;
        maxbitsW = std::max(maxbitsW, ci.bits);
    }
    // workspace
    Work &wk = work;
    const int Kp = (K + 127) / 128 * 128, Np = (N + 15) / 16 * 16;
    int dev = -1;
    cudaGetDevice(&dev);
    if (wk.M != M || wk.N != N || wk.K != K || wk.dev != dev) {
        wk.release();
        wk.M = M; wk.N = N; wk.K = K; wk.Kp = Kp; wk.Np = Np; wk.dev = dev;
        e = cudaMalloc(&wk.rinfo, (size_t)M * sizeof(RowInfo));
        if (!e) e = cudaMalloc(&wk.cinfo, (size_t)nbj * sizeof(ColInfo));
        if (!e) e = cudaMalloc(&wk.mult, (size_t)nbk * nbj * 8);
        if (!e) e = cudaMalloc(&wk.global, 16);
        if (!e) e = cudaMalloc(&wk.status, 256);
        if (!e) e = cudaMemset(wk.status, 0, 256);
        if (e) { wk.release(); return (int)e; }
    }
    e = cudaMemsetAsync(wk.global, 0, 16, st);
    if (!e) e = cudaMemcpyAsync(wk.cinfo, hc.data(), (size_t)nbj * sizeof(ColInfo), cudaMemcpyHostToDevice, st);
    if (!e) e = cudaMemcpyAsync(wk.mult, hmult.data(), hmult.size() * 8, cudaMemcpyHostToDevice, st);
    if (e) return (int)e;
    // 1. row statistics, then the modulus count
    x_stats<<<M, 256, 0, st>>>(X, K, ldx, wk.rinfo, wk.global);
    int hg[4] = {};
    e = cudaMemcpyAsync(hg, wk.global, 16, cudaMemcpyDeviceToHost, st);
    if (!e) e = cudaStreamSynchronize(st);
    if (e) return (int)e;
    if (hg[1]) return 10001;   // OZB_EARG: non-finite activations
    int kbits = 0;
    while ((1 << kbits) < K) kbits++;
    const double need = hg[0] + maxbitsW + kbits + 2;
    int nm = 8;
    double log2P = 0;
    for (int l = 0; l < 8; l++) log2P += log2((double)modulus(l));
    while (log2P < need && nm < NMAX) { log2P += log2((double)modulus(nm)); nm++; }
    if (log2P < need) return 10006;   // OZB_ESIZE: cannot happen with the two windows (62 + 62 + 17 + 2 bits < 147)
    if (wk.nm != nm || !wk.Xr) {
        cudaFree(wk.Xr); cudaFree(wk.Wr); cudaFree(wk.Cr);
        wk.Xr = wk.Wr = wk.Cr = nullptr;
        e = cudaMalloc(&wk.Xr, (size_t)nm * M * Kp);
        if (!e) e = cudaMalloc(&wk.Wr, (size_t)nm * N * Kp);
        if (!e) e = cudaMalloc(&wk.Cr, (size_t)nm * M * Np);
        if (e) { wk.release(); return (int)e; }
        wk.nm = nm;
    }
    static PerDevice pd;
    if (cudaError_t a = pd.once([] { return cudaFuncSetAttribute(w_residues_t, cudaFuncAttributeMaxDynamicSharedMemorySize, NMAX * WT_COLS * WT_PITCH); }))
        return (int)a;
    // 3. residues, GEMMs; 4. reconstruction and rounding
    x_residues<<<M, 256, 0, st>>>(X, K, ldx, wk.rinfo, nm, wk.Xr, Kp, (size_t)M * Kp);
    w_residues_t<<<dim3((N + WT_COLS - 1) / WT_COLS, (K + WT_K - 1) / WT_K), 256, nm * WT_COLS * WT_PITCH, st>>>(W, K, N, ldw, wk.mult, nbj, nm, wk.Wr,
                                                                                                          Kp, (size_t)N * Kp);
    e = cudaGetLastError();
    {   // long K in chunks of about 8192, as in the FP64 product (later chunks add to the stored residues)
        const int chunks = K > 12288 ? (K + 8191) / 8192 : 1, kc = ((K + chunks - 1) / chunks + 127) / 128 * 128;
        for (int k0 = 0, c = 0; k0 < K && !e; k0 += kc, c++)
            e = gemm_i8_planes(wk.Xr + k0, wk.Wr + k0, wk.Cr, M, N, K - k0 < kc ? K - k0 : kc, nm, Kp, Kp, Np, (size_t)M * Kp, (size_t)N * Kp,
                               (size_t)M * Np, 1, 0, wk.status, 0, st, c > 0);
    }
    if (e) return (int)e;
    if (nm <= 15) crt_round<4><<<dim3(M, (N + 511) / 512), 128, 0, st>>>(wk.Cr, (size_t)M * Np, M, N, Np, nm, wk.rinfo, wk.cinfo, Y, ldy, wk.global + 2);
    else crt_round<5><<<dim3(M, (N + 511) / 512), 128, 0, st>>>(wk.Cr, (size_t)M * Np, M, N, Np, nm, wk.rinfo, wk.cinfo, Y, ldy, wk.global + 2);
    e = cudaGetLastError();
    int hst[64] = {};
    if (!e) e = cudaMemcpyAsync(hg, wk.global, 16, cudaMemcpyDeviceToHost, st);
    if (!e) e = cudaMemcpyAsync(hst, wk.status, 256, cudaMemcpyDeviceToHost, st);
    if (!e) e = cudaStreamSynchronize(st);
    if (e) return (int)e;
    if (hst[0]) { cudaMemset(wk.status, 0, 256); return 10004; }   // OZB_ETIMEOUT
    if (open) *open = hg[2];
    if (moduli) *moduli = nm;
    return 0;
}

}  // namespace ozk
