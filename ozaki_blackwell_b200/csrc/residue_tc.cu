// residue_tc.cu -- the residue split of a row-contiguous operand with the byte sums on the tensor core.
//
// Same results as row_scale_residues (scale_residue.cu): s[r] = bits - 1 - ilogb(max |x|), R[l][r][k] = the balanced
// residue of v = llrint(ldexp(x, s[r])) mod m_l. There the sum  sum_i b_i (256^i mod m_l)  over the eight bytes of
// v + 2^62 costs two dp4a per element and modulus on the integer pipe, which bounds the kernel; here it is one small
// matrix product on the otherwise idle tensor pipe:
//   left operand   128 x 32 bytes per instruction: tile row g holds the 8 bytes of 4 consecutive elements of the matrix
//                  row (written by thread g itself, in the 128-byte-swizzle layout tcgen05 reads);
//   right operand  64 x 32 bytes, block diagonal: column 4 l + e carries 256^i mod m_l in the byte slots of element e;
//   result         D[g][4 l + e] = the byte sum of element e of row g for modulus l, in tensor memory, lane g.
// Thread g reads its own lane back (tcgen05.ld), reduces each sum once (multiply-high), packs the four elements of a
// modulus into a word and subtracts floor(m/2) from the four bytes at once. Two instructions (eight elements per thread)
// make a tile. A CTA works on one tile at a time (the loads of the next tile are in flight meanwhile); four CTAs share an
// SM and its 512 columns of tensor memory, so that one CTA's product runs while the others convert or reduce.
#include "oz_common.cuh"
#include "oz_tcgen05.cuh"

namespace ozk {
namespace rtc {

constexpr int TR = 128;                    // tile rows = tensor-memory lanes = threads of the CTA
constexpr int TE = 8;                      // elements per tile row: 64 bytes of K, two instructions of K = 32
constexpr int TILE_ELEMS = TR * TE;
constexpr int A_TILE = TR * 128;           // 16 KB (the first 64 bytes of each 128-byte row are used)
constexpr int W_TILE = 64 * 128;           // 8 KB (the first 32 bytes of each row)
constexpr int TM_COLS = 128;                // per CTA: 64 columns per instruction
constexpr int CTAS_PER_SM = 4;             // 4 x 128 columns of tensor memory
constexpr int SMEM = 48 * 1024;            // more than the 25 KB in use: keeps a fifth CTA (and its tensor-memory request) off the SM
constexpr uint32_t IDESC = tc::idesc_i8(128, 64, 0, 0);   // unsigned bytes times unsigned weights

// 256^i mod m_l as an unsigned byte
struct WeightTable { uint8_t w[16][8]; };
constexpr WeightTable make_weights() {
    WeightTable t{};
    for (int l = 0; l < 16; l++) {
        const int m = modulus(l);
        int w = 1 % m;
        for (int i = 0; i < 8; i++) { t.w[l][i] = (uint8_t)w; w = w * 256 % m; }
    }
    return t;
}
__constant__ WeightTable c_weights = make_weights();

// added to a byte sum d (d = v + 2^62 mod m, 0 <= d <= 8 * 255 * (m - 1)) so that (d + c) mod m - floor(m/2) is the balanced residue
constexpr uint32_t shift_of(int l) {
    const int m = modulus(l);
    return (uint32_t)(((half_of(l) - pow2_mod(62, m)) % m + m) % m);
}
constexpr bool sums_reduce_exactly() {
    for (int l = 1; l < 16; l++)
        if (!magic_ok(l, 8ull * 255 * (modulus(l) - 1) + shift_of(l))) return false;
    return true;
}
static_assert(sums_reduce_exactly(), "multiply-high reduction out of range");

// bytes r (0 <= r < 255) of a word minus h (h <= 127) each, modulo 256, without borrows between the bytes
__device__ __forceinline__ uint32_t sub_bytes(uint32_t r, uint32_t h4) {
    const uint32_t t = (r | 0x80808080u) - h4;
    return t ^ (~r & 0x80808080u);
}

template <int NM, bool GIVEN>
__global__ void __launch_bounds__(TR) row_residues_tc(const double *__restrict__ X, int rows, int len, long long ldx, int bits,
                                                      int *__restrict__ s_out, int8_t *__restrict__ Rp, int ld, size_t plane,
                                                      int *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tileA = base, tileW = base + A_TILE;
    __shared__ __align__(8) unsigned long long bars[1];
    __shared__ uint32_t tmem_slot;
    __shared__ double wmax[4];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar0 = tc::smem_u32(&bars[0]);

    // once per CTA: barriers, tensor memory, the weight operand
    if (tid == 0) {
        tc::mbar_init(bar0, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), TM_COLS);
    for (int i = tid; i < W_TILE / 16; i += TR)
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(tileW + 16u * i), "r"(0u) : "memory");
    __syncthreads();
    if (tid < 64) {                         // column n = 4 l + e: the weights of modulus l in the byte slots of element e
        const int l = tid >> 2, e = tid & 3;
        uint32_t lo = 0, hi = 0;
        for (int i = 0; i < 4; i++) { lo |= (uint32_t)c_weights.w[l][i] << (8 * i); hi |= (uint32_t)c_weights.w[l][4 + i] << (8 * i); }
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(tileW + tc::sw128_offset(tid, 8u * e)), "r"(lo), "r"(hi) : "memory");
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    const uint64_t descW = tc::smem_desc_sw128(tileW);

    uint32_t used = 0;                      // how often the barrier has completed
    bool alive = true;
    for (int r = blockIdx.x; r < rows && alive; r += gridDim.x) {
        const double *row = X + (size_t)r * ldx;
        const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
        int s;
        if constexpr (GIVEN) {
            s = s_out[r];
        } else {
            double mx = 0;
            if (vec) {
                const int pairs = len >> 1;
                for (int c = tid; c < pairs; c += TR) {
                    const double2 d = reinterpret_cast<const double2 *>(row)[c];
                    mx = fmax(mx, fmax(fabs(d.x), fabs(d.y)));
                }
                if ((len & 1) && tid == 0) mx = fmax(mx, fabs(row[len - 1]));
            } else {
                for (int k = tid; k < len; k += TR) mx = fmax(mx, fabs(row[k]));
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) mx = fmax(mx, __shfl_xor_sync(~0u, mx, o));
            __syncthreads();                // the previous row's readers of wmax are done
            if (lane == 0) wmax[warp] = mx;
            __syncthreads();
            mx = fmax(fmax(wmax[0], wmax[1]), fmax(wmax[2], wmax[3]));
            s = scale_from_max(mx, bits);
            if (tid == 0) s_out[r] = s;
        }
        const bool fast = s >= -1022 && s <= 1023;
        const double p2 = pow2_normal(fast ? s : 0);
        int8_t *out = Rp + (size_t)r * ld;
        const int words = (len + 3) >> 2;   // 4-byte words of residues this row gets
        const int tiles = (len + TILE_ELEMS - 1) / TILE_ELEMS;

        // the eight doubles of tile t that this thread converts
        auto load = [&](int t, double (&d)[TE]) {
            const int k0 = t * TILE_ELEMS + tid * TE;
            if (vec && k0 + TE <= len) {
#pragma unroll
                for (int j = 0; j < TE; j += 2) {
                    const double2 q = *reinterpret_cast<const double2 *>(row + k0 + j);
                    d[j] = q.x; d[j + 1] = q.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < TE; j++) d[j] = k0 + j < len ? row[k0 + j] : 0.0;
            }
        };
        // their 64 bytes into row `tid` of the left operand, then the two products
        auto feed = [&](const double (&d)[TE]) {
#pragma unroll
            for (int j = 0; j < TE; j += 2) {
                const unsigned long long a = (unsigned long long)scaled_int(d[j], s, p2, fast) + (1ull << 62);
                const unsigned long long b = (unsigned long long)scaled_int(d[j + 1], s, p2, fast) + (1ull << 62);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                             ::"r"(tileA + tc::sw128_offset(tid, 8u * j)), "r"((uint32_t)a), "r"((uint32_t)(a >> 32)), "r"((uint32_t)b),
                               "r"((uint32_t)(b >> 32)) : "memory");
            }
            tc::fence_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            if (tid == 0) {
                tc::fence_after_sync();
                const uint64_t descA = tc::smem_desc_sw128(tileA);
                tc::mma_i8(tmem_base, descA, descW, IDESC, 0u);             // elements 0..3 of every tile row
                tc::mma_i8(tmem_base + 64, descA + 2u, descW, IDESC, 0u);   // elements 4..7 (the next 32 bytes of K)
                tc::mma_commit(bar0);
            }
        };
        // tile t: sums out of tensor memory, one reduction each, 4-byte words of residues to every plane
        auto drain = [&](int t) -> bool {
            const bool ok = tc::mbar_wait(bar0, used & 1u);
            if (!__syncthreads_and(ok)) return false;
            used++;
            tc::fence_after_sync();
            const int w0 = (t * TILE_ELEMS + tid * TE) >> 2;   // first of this thread's two words
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll
            for (int half = 0; half < 2; half++) {              // moduli 8 half .. 8 half + 7
                if (8 * half >= NM) break;
                uint32_t v0[32], v1[32];
                tc::tmem_ld32(taddr + 32 * half, v0);           // elements 0..3
                tc::tmem_ld32(taddr + 64 + 32 * half, v1);      // elements 4..7
                tc::tmem_ld_wait();
                static_for<0, 8>([&](auto I) {
                    constexpr int i = decltype(I)::value;
                    auto emit = [&](auto L) {
                        constexpr int l = decltype(L)::value;
                        if constexpr (l < NM) {
                            uint32_t a, b;
                            if constexpr (l == 0) {             // modulus 256: the low byte itself
                                a = pack_low_bytes(v0[4 * i], v0[4 * i + 1], v0[4 * i + 2], v0[4 * i + 3]);
                                b = pack_low_bytes(v1[4 * i], v1[4 * i + 1], v1[4 * i + 2], v1[4 * i + 3]);
                            } else {
                                constexpr uint32_t c = shift_of(l), h4 = (uint32_t)half_of(l) * 0x01010101u;
                                a = sub_bytes(pack_low_bytes(mod_magic<l>(v0[4 * i] + c), mod_magic<l>(v0[4 * i + 1] + c),
                                                             mod_magic<l>(v0[4 * i + 2] + c), mod_magic<l>(v0[4 * i + 3] + c)), h4);
                                b = sub_bytes(pack_low_bytes(mod_magic<l>(v1[4 * i] + c), mod_magic<l>(v1[4 * i + 1] + c),
                                                             mod_magic<l>(v1[4 * i + 2] + c), mod_magic<l>(v1[4 * i + 3] + c)), h4);
                            }
                            uint32_t *dst = reinterpret_cast<uint32_t *>(out + (size_t)l * plane) + w0;
                            if (w0 < words) dst[0] = a;
                            if (w0 + 1 < words) dst[1] = b;
                        }
                    };
                    if (half == 0) emit(std::integral_constant<int, i>{});
                    else emit(std::integral_constant<int, 8 + i>{});
                });
            }
            tc::fence_before_sync();
            return true;
        };

        double cur[TE], nxt[TE];
        load(0, cur);
        for (int t = 0; t < tiles; t++) {
            feed(cur);
            if (t + 1 < tiles) load(t + 1, nxt);   // in flight while the products run
            if (!drain(t)) { alive = false; break; }
            __syncthreads();                       // tensor memory and the operand tile are free again
#pragma unroll
            for (int j = 0; j < TE; j++) cur[j] = nxt[j];
        }
    }
    if (!alive && tid == 0 && status) atomicCAS(status, 0, 0x80);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    if (warp == 0) tc::tmem_dealloc(tmem_base, TM_COLS);
}

template <int NM, bool GIVEN>
static cudaError_t launch(const double *X, int rows, int len, long long ldx, int bits, int *s, int8_t *R, int ld, size_t plane,
                          int *status, cudaStream_t st) {
    static PerDevice pd;
    if (cudaError_t a = pd.once([] { return cudaFuncSetAttribute(row_residues_tc<NM, GIVEN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); })) return a;
    int dev = 0, sms = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return e;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) return e;
    const int grid = rows < CTAS_PER_SM * sms ? rows : CTAS_PER_SM * sms;
    row_residues_tc<NM, GIVEN><<<grid, TR, SMEM, st>>>(X, rows, len, ldx, bits, s, R, ld, plane, status);
    return cudaGetLastError();
}

}  // namespace rtc

#define OZ_DISPATCH_NM_TC(nm, CALL)                                                                               \
    switch (nm) {                                                                                                 \
    case 8: { constexpr int NM = 8; return CALL; }    case 9: { constexpr int NM = 9; return CALL; }              \
    case 10: { constexpr int NM = 10; return CALL; }  case 11: { constexpr int NM = 11; return CALL; }            \
    case 12: { constexpr int NM = 12; return CALL; }  case 13: { constexpr int NM = 13; return CALL; }            \
    case 14: { constexpr int NM = 14; return CALL; }  case 15: { constexpr int NM = 15; return CALL; }            \
    case 16: { constexpr int NM = 16; return CALL; }                                                              \
    default: return cudaErrorInvalidValue;                                                                        \
    }

cudaError_t scale_residues_rows_tc(int nm, const double *X, int rows, int len, long long ldx, int bits, int *s, int8_t *R, int ld,
                                   size_t plane, int *status, cudaStream_t st) {
    OZ_DISPATCH_NM_TC(nm, (rtc::launch<NM, false>(X, rows, len, ldx, bits, s, R, ld, plane, status, st)));
}

}  // namespace ozk
