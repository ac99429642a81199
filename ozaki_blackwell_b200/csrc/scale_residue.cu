// scale_residue.cu -- kernels 1 and 2 of the FP64 product: exponent scaling and the int8 residue split.
//
// What they compute is the reference's `scales` and `residues<NM>` (src/ozaki2.cuh:56-78):
//     s[r]       = bits - 1 - ilogb(max_k |X[r,k]|)           (0 for an all-zero row / column)
//     R[l][r][k] = int8( balanced (llrint(ldexp(X[r,k], s[r])) mod m_l) )    for every modulus l < NM
// with R stored K-contiguous for both operands (B comes out transposed: Bt[l][j][k]).
//
// How: both are HBM-bound, so each input is read as few times as its access pattern allows and the 64-bit "% m" is
// replaced by byte arithmetic. A row of A is read once: the block keeps it in registers between the max reduction
// and the residue split. B is scaled per column, which needs a pass over whole columns first (col_absmax, coalesced
// along rows) and a second, transposing pass. The residue of a 64-bit integer is taken from its eight bytes:
// v + 2^62 = sum b_i 256^i with b_i unsigned, so v mod m = sum b_i (256^i mod m) - (2^62 mod m): two dp4a per modulus
// and one multiply-high reduction of a 19-bit sum, instead of a 64-bit division by a constant.
#include <mutex>
#include "oz_common.cuh"
#include "oz_bounds.cuh"

namespace ozk {

// ---------------------------------------------------------------------------------------------------------------
// residues of four consecutive integers for every modulus: calls put(l, word) with the four int8 packed little-endian
// ---------------------------------------------------------------------------------------------------------------
template <int NM, class Put>
__device__ __forceinline__ void residues_of_4(const long long (&v)[4], Put &&put) {
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const unsigned long long w = (unsigned long long)v[e] + (1ull << 62);   // |v| < 2^62: w is positive
        lo[e] = (uint32_t)w;
        hi[e] = (uint32_t)(w >> 32);
    }
    // modulus 256: the balanced residue is the low byte read as int8
    put(std::integral_constant<int, 0>{}, pack_low_bytes(lo[0], lo[1], lo[2], lo[3]));
    static_for<1, NM>([&](auto L) {
        constexpr int l = decltype(L)::value, m = modulus(l);
        constexpr uint32_t wlo = pack4(byte_weight(0, l), byte_weight(1, l), byte_weight(2, l), byte_weight(3, l));
        constexpr uint32_t whi = pack4(byte_weight(4, l), byte_weight(5, l), byte_weight(6, l), byte_weight(7, l));
        // a multiple of m that lifts the byte sum above zero, minus 2^62 mod m (the offset added above); the +floor(m/2)
        // that balances the residue is folded into the quotient (balanced_magic)
        constexpr int init = lift_of(l, BYTES_BOUND) - half_of(l) - pow2_mod(62, m);
        static_assert(init > BYTES_BOUND && magic_ok(l, (uint64_t)init + half_of(l) + BYTES_BOUND), "multiply-high reduction out of range");
        uint32_t x[4];
#ifndef OZ_INT_REDUCE
        constexpr int seed = FLOAT_BIAS - pow2_mod(62, m);
        static_assert(BYTES_BOUND + 256 < (1 << 22), "the byte sum must fit the float's mantissa");
#pragma unroll
        for (int e = 0; e < 4; e += 2)
            balanced_float_x2<l>(dp4a_us(hi[e], whi, dp4a_us(lo[e], wlo, seed)), dp4a_us(hi[e + 1], whi, dp4a_us(lo[e + 1], wlo, seed)), x[e], x[e + 1]);
#else
#pragma unroll
        for (int e = 0; e < 4; e++) x[e] = balanced_magic<l>((uint32_t)dp4a_us(hi[e], whi, dp4a_us(lo[e], wlo, init)));
#endif
        put(L, pack_low_bytes(x[0], x[1], x[2], x[3]));
    });
}

// ---------------------------------------------------------------------------------------------------------------
// A side: one block per row. R chunks of four doubles per thread stay in registers between the two phases.
// ---------------------------------------------------------------------------------------------------------------
#ifndef OZ_ROW_R
#define OZ_ROW_R 4      // chunks of four doubles a thread keeps in registers
#define OZ_ROW_T 256    // largest block
#define OZ_ROW_MINB 4   // blocks per SM the register allocation must allow
#endif
template <int NM, int R, int MAXT, bool GIVEN = false>   // GIVEN: the scales are already in s_out (2-norm mode), no max pass
__global__ void __launch_bounds__(MAXT, OZ_ROW_MINB) row_scale_residues(const double *__restrict__ X, int len, long long ldx, int bits,
                                                           int *__restrict__ s_out, int8_t *__restrict__ Rp, int ld,
                                                           size_t plane) {
    const int r = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const double *row = X + (size_t)r * ldx;
    const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
    const int chunks = (len + 3) >> 2;                // chunks of four
    const bool cached = chunks <= R * nt;             // does the whole row fit the block's registers?
    double x[R][4];
    double mx = 0;
    auto load4 = [&](int c, double (&d)[4]) {
        const int k = c << 2;
        if (vec && k + 3 < len) {
            const double2 a = oz_load(reinterpret_cast<const double2 *>(row + k)), b = oz_load(reinterpret_cast<const double2 *>(row + k + 2));
            d[0] = a.x; d[1] = a.y; d[2] = b.x; d[3] = b.y;
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) d[e] = k + e < len ? oz_load(row + k + e) : 0.0;
        }
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int c = i * nt + tid;
            if (c < chunks) load4(c, x[i]);
            else { x[i][0] = x[i][1] = x[i][2] = x[i][3] = 0.0; }
#pragma unroll
            for (int e = 0; e < 4; e++) mx = fmax(mx, fabs(x[i][e]));
        }
    } else if (!GIVEN) {
        for (int c = tid; c < chunks; c += nt) {
            double d[4];
            load4(c, d);
#pragma unroll
            for (int e = 0; e < 4; e++) mx = fmax(mx, fabs(d[e]));
        }
    }
    int s;
    if constexpr (GIVEN) {
        s = oz_load(s_out + r);
    } else {
        // block max: shuffles inside the warp, shared memory across warps
        __shared__ double wmax[32];
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmax(mx, __shfl_xor_sync(~0u, mx, o));
        if ((tid & 31) == 0) wmax[tid >> 5] = mx;
        __syncthreads();
        mx = wmax[0];
        for (int w = 1; w < (nt >> 5); w++) mx = fmax(mx, wmax[w]);
        s = scale_from_max(mx, bits);
        if (tid == 0) oz_store(s_out + r, s);
    }

    const bool fast = s >= -1022 && s <= 1023;
    const double p2 = pow2_normal(fast ? s : 0);
    int8_t *out = Rp + (size_t)r * ld;
    auto emit = [&](int c, const double (&d)[4]) {
        long long v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = scaled_int(d[e], s, p2, fast);
        residues_of_4<NM>(v, [&](auto L, uint32_t word) {
            oz_store(reinterpret_cast<uint32_t *>(out + decltype(L)::value * plane + ((size_t)c << 2)), word);
        });
    };
    if (cached) {
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int c = i * nt + tid;
            if (c < chunks) emit(c, x[i]);
        }
    } else {
        for (int c = tid; c < chunks; c += nt) {
            double d[4];
            load4(c, d);
            emit(c, d);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// B side, pass 1: per-column max |x| of a row-major K x N matrix, as the bit pattern of a non-negative double
// (for those the integer order is the numeric order; NaNs are dropped by fmax as in the reference's loop).
// Block: 256 threads x 2 adjacent columns, ROWS rows; one atomicMax per column per block.
// ---------------------------------------------------------------------------------------------------------------
constexpr int CM_ROWS = 64;
__global__ void __launch_bounds__(256) col_absmax(const double *__restrict__ X, int rows, int cols, long long ldx,
                                                  unsigned long long *__restrict__ colmax) {
    const int j = (blockIdx.x * 256 + threadIdx.x) * 2;
    const int k0 = blockIdx.y * CM_ROWS, k1 = min(rows, k0 + CM_ROWS);
    if (j >= cols) return;
    const bool pair = j + 1 < cols && ((reinterpret_cast<uintptr_t>(X) & 15) == 0) && (ldx & 1) == 0;
    double m0 = 0, m1 = 0;
    if (pair) {
#pragma unroll 8
        for (int k = k0; k < k1; k++) {
            const double2 d = oz_load(reinterpret_cast<const double2 *>(X + (size_t)k * ldx + j));
            m0 = fmax(m0, fabs(d.x));
            m1 = fmax(m1, fabs(d.y));
        }
    } else {
        for (int k = k0; k < k1; k++) {
            m0 = fmax(m0, fabs(oz_load(X + (size_t)k * ldx + j)));
            if (j + 1 < cols) m1 = fmax(m1, fabs(oz_load(X + (size_t)k * ldx + j + 1)));
        }
    }
    if (m0 != 0) oz_atomic_max(colmax + j, (unsigned long long)__double_as_longlong(m0));
    if (j + 1 < cols && m1 != 0) oz_atomic_max(colmax + j + 1, (unsigned long long)__double_as_longlong(m1));
}

// ---------------------------------------------------------------------------------------------------------------
// B side, pass 2: residues of a row-major K x N matrix written transposed, Rt[l][j][k].
// Block: 256 threads, tile of 32 columns x 128 k. Phase 1: lane = column, warp w owns k in [16w, 16w + 16): reads are
// 256-byte row segments, each thread produces 16 bytes per plane and parks them in shared memory, S[l][j][k] with rows
// padded to 144 bytes (conflict-free for 16-byte accesses both ways). Phase 2: the tile is written out row by row,
// eight threads per 128-byte row, so every store instruction writes four full 128-byte lines.
// ---------------------------------------------------------------------------------------------------------------
constexpr int CT_COLS = 32, CT_K = 128, CT_PITCH = CT_K + 16;
template <int NM> constexpr int col_tile_smem() { return NM * CT_COLS * CT_PITCH; }

#ifndef OZ_COL_MINB
#define OZ_COL_MINB 3   // measured on B200: 3 blocks per SM (80 registers, a 40-byte spill) 0.511 ms, 2 blocks 0.545 ms, 4 blocks 0.530 ms at n = 8192
#endif
template <int NM>
__global__ void __launch_bounds__(256, OZ_COL_MINB) col_residues_t(const double *__restrict__ X, int rows, int cols, long long ldx,
                                                      const unsigned long long *__restrict__ colmax, int bits,
                                                      int *__restrict__ s_out, int8_t *__restrict__ Rp, int ld, size_t plane) {
    extern __shared__ __align__(16) uint8_t tile[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j0 = blockIdx.x * CT_COLS, kb = blockIdx.y * CT_K;
    {
        const int j = j0 + lane, k0 = kb + warp * 16;
        if (j < cols && k0 < rows) {
            // colmax == nullptr: the scales are already in s_out (2-norm mode)
            const int s = colmax ? scale_from_max(__longlong_as_double((long long)oz_load(colmax + j)), bits) : oz_load(s_out + j);
            if (colmax && blockIdx.y == 0 && warp == 0) oz_store(s_out + j, s);
            const bool fast = s >= -1022 && s <= 1023;
            const double p2 = pow2_normal(fast ? s : 0);
            double d[16];
#pragma unroll
            for (int e = 0; e < 16; e++) d[e] = k0 + e < rows ? oz_load(X + (size_t)(k0 + e) * ldx + j) : 0.0;
            uint32_t w[NM][4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                long long v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) v[e] = scaled_int(d[4 * q + e], s, p2, fast);
                residues_of_4<NM>(v, [&](auto L, uint32_t word) { w[decltype(L)::value][q] = word; });
            }
#pragma unroll
            for (int l = 0; l < NM; l++)
                *reinterpret_cast<uint4 *>(tile + (l * CT_COLS + lane) * CT_PITCH + warp * 16) = make_uint4(w[l][0], w[l][1], w[l][2], w[l][3]);
        }
    }
    __syncthreads();
    const int c = threadIdx.x & 7;                 // 16-byte piece of the 128-byte row
    const int kpos = kb + c * 16;
    if (kpos >= rows) return;                      // pieces wholly beyond K are never read by the GEMM (TMA extent = K)
#pragma unroll 4
    for (int i = 0; i < NM; i++) {                 // rows of the tile: (l, j), 32 per pass
        const int j = threadIdx.x >> 3, l = i;
        if (j0 + j < cols) {
            const uint4 v = *reinterpret_cast<const uint4 *>(tile + (l * CT_COLS + j) * CT_PITCH + c * 16);
            oz_store(reinterpret_cast<uint4 *>(Rp + (size_t)l * plane + (size_t)(j0 + j) * ld + kpos), v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Optional scale from the 2-norm (the reference's scales_norm, bench/oz_strassen.cu:74-97): s = beta - 1 - (e + ilogb(
// sqrt(ss) (1 + 2^-30))), e = ilogb(max |x|), ss = sum (x 2^-e)^2. The last bits of ss can move s across a power of two,
// so the sum is taken in the reference's order: 256 threads, thread t accumulates k = t, t + 256, ... with fma, a
// butterfly of additions inside each warp, then the eight warp sums in order. `vecs` vectors per block (1 for rows, 4
// adjacent columns for a row-major matrix so that each thread reads whole 32-byte sectors).
// ---------------------------------------------------------------------------------------------------------------
template <int VECS>
__global__ void __launch_bounds__(256) scales_norm_kernel(const double *__restrict__ X, int nvec, int len, long long sVec, long long sElem,
                                                          int beta, int *__restrict__ s) {
    const int v0 = blockIdx.x * VECS, tid = threadIdx.x;
    __shared__ double w[VECS][8];
    __shared__ int se[VECS];
    __shared__ bool zero[VECS];
    double acc[VECS];
#pragma unroll
    for (int q = 0; q < VECS; q++) acc[q] = 0;
    for (int k = tid; k < len; k += 256)
#pragma unroll
        for (int q = 0; q < VECS; q++)
            if (v0 + q < nvec) acc[q] = fmax(acc[q], fabs(oz_load(X + (size_t)(v0 + q) * sVec + (size_t)k * sElem)));
#pragma unroll
    for (int q = 0; q < VECS; q++) {
        for (int o = 16; o; o >>= 1) acc[q] = fmax(acc[q], __shfl_xor_sync(~0u, acc[q], o));
        if ((tid & 31) == 0) w[q][tid >> 5] = acc[q];
    }
    __syncthreads();
    if (tid < VECS) {
        double m = w[tid][0];
        for (int i = 1; i < 8; i++) m = fmax(m, w[tid][i]);
        zero[tid] = m == 0;
        se[tid] = m == 0 ? 0 : ilogb(m);
    }
    __syncthreads();
    int e[VECS];
#pragma unroll
    for (int q = 0; q < VECS; q++) { e[q] = se[q]; acc[q] = 0; }
    for (int k = tid; k < len; k += 256)
#pragma unroll
        for (int q = 0; q < VECS; q++)
            if (v0 + q < nvec) { const double v = ldexp(oz_load(X + (size_t)(v0 + q) * sVec + (size_t)k * sElem), -e[q]); acc[q] = fma(v, v, acc[q]); }
    __syncthreads();   // w is reused
#pragma unroll
    for (int q = 0; q < VECS; q++) {
        for (int o = 16; o; o >>= 1) acc[q] = acc[q] + __shfl_xor_sync(~0u, acc[q], o);
        if ((tid & 31) == 0) w[q][tid >> 5] = acc[q];
    }
    __syncthreads();
    if (tid < VECS && v0 + tid < nvec) {
        double t = w[tid][0];
        for (int i = 1; i < 8; i++) t = t + w[tid][i];
        oz_store(s + v0 + tid, zero[tid] ? 0 : beta - 1 - (se[tid] + ilogb(sqrt(t) * (1 + 0x1p-30))));
    }
}

// ---------------------------------------------------------------------------------------------------------------
// launchers (nm is a run-time value in the API, a template parameter in the kernels)
// ---------------------------------------------------------------------------------------------------------------
template <int NM>
static cudaError_t launch_rows_t(const double *X, int rows, int len, long long ldx, int bits, int *s, int8_t *R, int ld,
                                 size_t plane, cudaStream_t st) {
    // Rows of up to 4096 entries stay in registers (4 chunks x 256 threads); longer ones are read a second time, from L2.
    // Measured on B200 at K = 8192: this shape (64 registers, 4 blocks per SM) takes 0.427 ms, keeping the whole row in
    // registers (8 chunks, 100 registers, 2 blocks per SM) 0.456 ms: occupancy matters more than the second read.
    constexpr int RR = OZ_ROW_R, MAXT = OZ_ROW_T;
    int nt = ((len + 3) / 4 + RR - 1) / RR;     // threads that hold the row in registers
    nt = (nt + 31) / 32 * 32;
    if (nt < 32) nt = 32;
    if (nt > MAXT) nt = MAXT;
    OZ_WINDOWS(st, OZK_ROW_RESIDUES, window2d(X, rows, (size_t)ldx * 8, (size_t)len * 8), window1d(s, (size_t)rows * 4),
               window3d(R, NM, plane, rows, ld, (size_t)(len + 3) / 4 * 4));
    row_scale_residues<NM, RR, MAXT><<<rows, nt, 0, st>>>(X, len, ldx, bits, s, R, ld, plane);
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

cudaError_t cols_residues_from_max(int nm, const double *X, int rows, int cols, long long ldx, int bits, const unsigned long long *colmax,
                                   int *s, int8_t *R, int ld, size_t plane, cudaStream_t st);
template <int NM>
static cudaError_t launch_rows_given_t(const double *X, int rows, int len, long long ldx, int *s, int8_t *R, int ld, size_t plane,
                                       cudaStream_t st) {
    constexpr int RR = OZ_ROW_R, MAXT = OZ_ROW_T;
    int nt = ((len + 3) / 4 + RR - 1) / RR;
    nt = (nt + 31) / 32 * 32;
    if (nt < 32) nt = 32;
    if (nt > MAXT) nt = MAXT;
    OZ_WINDOWS(st, OZK_ROW_RESIDUES, window2d(X, rows, (size_t)ldx * 8, (size_t)len * 8), window1d(s, (size_t)rows * 4),
               window3d(R, NM, plane, rows, ld, (size_t)(len + 3) / 4 * 4));
    row_scale_residues<NM, RR, MAXT, true><<<rows, nt, 0, st>>>(X, len, ldx, 0, s, R, ld, plane);
    return cudaGetLastError();
}
// The 2-norm scales alone: of `nvec` rows of a row-major matrix (by_rows) or of its `nvec` columns
cudaError_t scales_norm_only(const double *X, int nvec, int len, long long ldx, int by_rows, int beta, int *s, cudaStream_t st) {
    if (by_rows) OZ_WINDOWS(st, OZK_SCALES_NORM, window2d(X, nvec, (size_t)ldx * 8, (size_t)len * 8), window1d(s, (size_t)nvec * 4));
    else OZ_WINDOWS(st, OZK_SCALES_NORM, window2d(X, len, (size_t)ldx * 8, (size_t)nvec * 8), window1d(s, (size_t)nvec * 4));
    if (by_rows) scales_norm_kernel<1><<<nvec, 256, 0, st>>>(X, nvec, len, ldx, 1, beta, s);
    else scales_norm_kernel<4><<<(nvec + 3) / 4, 256, 0, st>>>(X, nvec, len, 1, ldx, beta, s);
    return cudaGetLastError();
}
// The 2-norm mode of both operands: scales first (reference order of summation), then the residue passes with those scales
cudaError_t norm_scale_residues_rows(int nm, const double *X, int rows, int len, long long ldx, int beta, int *s, int8_t *R, int ld,
                                     size_t plane, cudaStream_t st) {
    if (cudaError_t e = scales_norm_only(X, rows, len, ldx, 1, beta, s, st)) return e;
    OZ_DISPATCH_NM(nm, (launch_rows_given_t<NM>(X, rows, len, ldx, s, R, ld, plane, st)));
}
cudaError_t norm_scale_residues_cols(int nm, const double *X, int rows, int cols, long long ldx, int beta, int *s, int8_t *R, int ld,
                                     size_t plane, cudaStream_t st) {
    if (cudaError_t e = scales_norm_only(X, cols, rows, ldx, 0, beta, s, st)) return e;
    return cols_residues_from_max(nm, X, rows, cols, ldx, 0, nullptr, s, R, ld, plane, st);
}
// A-like operand: `rows` rows of `len` contiguous doubles, row pitch ldx; writes s[rows] and R[nm][rows][ld]
cudaError_t scale_residues_rows(int nm, const double *X, int rows, int len, long long ldx, int bits, int *s, int8_t *R, int ld,
                                size_t plane, cudaStream_t st) {
    OZ_DISPATCH_NM(nm, (launch_rows_t<NM>(X, rows, len, ldx, bits, s, R, ld, plane, st)));
}
// The two passes of the B-like operand separately, for callers that receive the matrix in row chunks: the column maxima
// of rows [0, rows) of X accumulate into colmax (which the caller cleared once), the residue pass runs when all chunks
// have been seen.
cudaError_t cols_absmax_accumulate(const double *X, int rows, int cols, long long ldx, unsigned long long *colmax, cudaStream_t st) {
    OZ_WINDOWS(st, OZK_COL_ABSMAX, window2d(X, rows, (size_t)ldx * 8, (size_t)cols * 8), window1d(colmax, (size_t)cols * 8));
    col_absmax<<<dim3((cols + 511) / 512, (rows + CM_ROWS - 1) / CM_ROWS), 256, 0, st>>>(X, rows, cols, ldx, colmax);
    return cudaGetLastError();
}
template <int NM>
static cudaError_t launch_cols_residues_t(const double *X, int rows, int cols, long long ldx, int bits, const unsigned long long *colmax,
                                          int *s, int8_t *R, int ld, size_t plane, cudaStream_t st) {
    static PerDevice pd;
    if (cudaError_t a = pd.once([] { return cudaFuncSetAttribute(col_residues_t<NM>, cudaFuncAttributeMaxDynamicSharedMemorySize, col_tile_smem<NM>()); })) return a;
    OZ_WINDOWS(st, OZK_COL_RESIDUES, window2d(X, rows, (size_t)ldx * 8, (size_t)cols * 8), window1d(colmax, colmax ? (size_t)cols * 8 : 0),
               window1d(s, (size_t)cols * 4), window3d(R, NM, plane, cols, ld, (size_t)(rows + 15) / 16 * 16));
    col_residues_t<NM><<<dim3((cols + CT_COLS - 1) / CT_COLS, (rows + CT_K - 1) / CT_K), 256, col_tile_smem<NM>(), st>>>(
        X, rows, cols, ldx, colmax, bits, s, R, ld, plane);
    return cudaGetLastError();
}
cudaError_t cols_residues_from_max(int nm, const double *X, int rows, int cols, long long ldx, int bits, const unsigned long long *colmax,
                                   int *s, int8_t *R, int ld, size_t plane, cudaStream_t st) {
    OZ_DISPATCH_NM(nm, (launch_cols_residues_t<NM>(X, rows, cols, ldx, bits, colmax, s, R, ld, plane, st)));
}
// B-like operand: row-major `rows` x `cols` (rows = K), scaled per column; writes s[cols] and Rt[nm][cols][ld]
cudaError_t scale_residues_cols(int nm, const double *X, int rows, int cols, long long ldx, int bits, unsigned long long *colmax,
                                int *s, int8_t *R, int ld, size_t plane, cudaStream_t st) {
    cudaError_t e = cudaMemsetAsync(colmax, 0, (size_t)cols * 8, st);
    if (!e) e = cols_absmax_accumulate(X, rows, cols, ldx, colmax, st);
    if (e) return e;
    return cols_residues_from_max(nm, X, rows, cols, ldx, bits, colmax, s, R, ld, plane, st);
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the column pass (C ABI: ozb_scale_residues_cols_static)
// ---------------------------------------------------------------------------------------------------------------
// For callers that must not allocate device memory at the point of the call: processes that have handed all of the
// GPU's memory to an allocator of their own (a serving engine or a framework's caching pool that reserved the HBM up
// front, where a cudaMalloc from a library would fail or fragment the pool), and latency-critical loops that cannot
// afford cudaMalloc / cudaFree because both synchronise the whole device. The column pass needs one 64-bit word of
// scratch per column (the running column maxima). Here that scratch is a fixed array in the library's own device image:
// every GPU that loads the library holds these OZB_STATIC_MAX_COLS * 8 bytes (512 KiB) until the process exits.
//
// The array's name is only a host-side handle. Its device address is fetched with cudaGetSymbolAddress, once per device,
// with that device current, on the first call made on that device -- so the first call on each device should come
// before any stream capture begins. All calls on one device share the array: it keeps the previous call's maxima, so
// every call clears the part it uses first (on the caller's stream), and two calls that overlap on the GPU (different
// streams, no ordering between them) would race on it.
constexpr int OZB_STATIC_MAX_COLS = 65536;
static __device__ __align__(256) unsigned long long g_colmax_scratch[OZB_STATIC_MAX_COLS];

static unsigned long long *static_scratch_for_current_device(cudaError_t *err) {
    static unsigned long long *ptrs[64] = {};
    static std::mutex mu;
    int dev = -1;
    if ((*err = cudaGetDevice(&dev)) != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
    std::lock_guard<std::mutex> g(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        if ((*err = cudaGetSymbolAddress(&p, g_colmax_scratch)) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<unsigned long long *>(p);
    }
    *err = cudaSuccess;
    return ptrs[dev];
}

// violations the checked accesses of this file recorded since the last call (debug build; zeros otherwise)
cudaError_t scale_residue_violations(unsigned long long out[4]) { return oz_read_violations(out); }

}  // namespace ozk

// Same contract as ozb_scale_residues_cols (scales per column of a row-major rows x cols matrix, residues written
// transposed), without the caller-provided scratch and without any allocation: no cudaMalloc, cudaFree or allocating
// library routine is called. cols above OZB_STATIC_MAX_COLS (65536) is rejected with OZB_ESIZE (10006).
extern "C" __attribute__((visibility("default"))) int ozb_scale_residues_cols_static(int moduli, const double *X, int rows, int cols,
                                                                                    long long ldx, int bits, int *s, int8_t *R, int ld,
                                                                                    size_t plane, void *stream) {
    if (rows <= 0 || cols <= 0) return 10001;                       // OZB_EARG
    if (rows >= 131072) return 10002;                               // OZB_EK
    if (cols > ozk::OZB_STATIC_MAX_COLS) return 10006;              // OZB_ESIZE: beyond the fixed scratch
    if (moduli < 8 || moduli > 16 || !X || !s || !R || ldx < cols || ld < (rows + 15) / 16 * 16 || (ld & 15) || (plane & 15) ||
        (reinterpret_cast<uintptr_t>(R) & 15))
        return 10001;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) return (int)cudaGetLastError();
    if (major != 10) return 10003;                                  // OZB_EARCH
    cudaError_t e;
    unsigned long long *scratch = ozk::static_scratch_for_current_device(&e);
    if (!scratch) return (int)e;
    // scale_residues_cols clears colmax[0, cols) on the stream before the maxima pass, then runs the two kernels
    return (int)ozk::scale_residues_cols(moduli, X, rows, cols, ldx, bits, scratch, s, R, ld, plane, (cudaStream_t)stream);
}
