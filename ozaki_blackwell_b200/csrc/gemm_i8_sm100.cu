// gemm_i8_sm100.cu -- kernel 3 of the FP64 product: the exact INT8 GEMMs, one per modulus, on 5th-generation tensor cores.
//
// What it computes is the reference's gemm_i8_run (src/gemm_i8.cuh:148-160): for every plane z < Z
//     C[z][i][j] = sum_k A[z][i][k] * Bt[z][j][k]       int8 x int8 -> exact int32, both operands K-contiguous
// and, in the fused mode, what the first line of the reference's crt kernel does to it (src/ozaki2.cuh:88): the balanced
// residue mod m_z, stored as int8 (one byte per product instead of four).
//
// How (sm_100a only): a persistent, warp-specialised kernel, one CTA per SM.
//   warp 0   producer: TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) fills a ring of shared-memory stages,
//            each one 128-byte K-slab of a 128-row A tile and a 256-row B tile, straight from the K-major residue planes
//            (a 3-D tensor map {k, row, plane}; rows and k beyond the matrix are zero-filled by the hardware).
//   warp 1   issuer: one thread issues tcgen05.mma kind::i8 (M 128, N 256, K 32 per instruction) from shared-memory
//            descriptors into one of two 128 x 256 int32 accumulators in tensor memory, and commits each stage back to
//            the producer and each finished tile to the epilogue through mbarriers.
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (one row per thread), reduce mod m_z (or keep int32) and
//            store, while the issuer is already accumulating the next tile into the other buffer.
// Work items are (plane, tile) pairs walked plane by plane and, inside a plane, in bands of tile rows so that the A
// band and the B panels in flight stay in L2. The two-CTA kernel hands them out dynamically (a device-wide counter read
// by one otherwise idle warp per pair, a few items ahead), so pairs that run faster, or start earlier because the SMs of
// others are still held by another kernel, take more of them. Every mbarrier wait is bounded: on expiry the CTA raises a status word,
// stops issuing, releases its tensor memory and returns.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include "oz_common.cuh"
#include "oz_bounds.cuh"

namespace ozk {

namespace g8 {
constexpr int BM = 128, BN = 256, BKB = 128;       // tile: rows of A, rows of Bt, bytes (= int8 elements) of K per stage
constexpr int UK = 32;                             // K of one tcgen05.mma kind::i8
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES;   // 16 KB + 32 KB
constexpr int ACC_COLS = BN, TMEM_COLS = 512;      // two accumulators of 256 columns
constexpr int THREADS = 192;                       // producer warp, issuer warp, four epilogue warps
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr unsigned long long WAIT_NS = 4000000000ull;   // give up on a barrier after 4 s

// instruction descriptor of tcgen05.mma kind::i8: D = S32, A = B = signed 8-bit, both K-major, N = 256, M = 128
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: each wait has its own budget, started the first time the spin loop looks at the clock. Returns false
// when the budget ran out or another role of this CTA already gave up (*abort_flag != 0).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int who = 1,
                                          unsigned long long budget_ns = WAIT_NS) {
    unsigned long long deadline = 0;
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 1023u) == 1023u) {
            if (*abort_flag) return false;
            const unsigned long long t = now_ns();
            if (!deadline) deadline = t + budget_ns;
            else if (t > deadline) { *abort_flag = who; return false; }   // who: which wait gave up (diagnostics)
        }
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle; rows are 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}

struct Params {
    int M, N, K, Z;               // rows of A, rows of Bt, inner length, planes
    int tiles_m, tiles_n, band;   // tile grid of one plane and the band height (tile rows)
    int first_modulus;            // plane z reduces mod modulus(first_modulus + z) in the fused mode
    int accumulate;               // fused mode: add the residues already stored in C (a previous K chunk) before reducing
    void *C;                      // int32 [Z][M][ldc] or int8 [Z][M][ldc]
    long long ldc;                // row pitch of C in elements
    int wcols;                    // fused mode: columns of this launch's C that may be written, N rounded up to 16 (whole 16-byte pieces)
    size_t plane_c;               // plane pitch of C in elements
    int *status;                  // device word: set to 1 when a wait timed out
    int *counter;                 // two-CTA kernel: next work item, zeroed before the launch
    const int *yield_flag;        // two-CTA kernel: pairs from `keep_pairs` on leave at once while this word is non-zero (nullptr: nobody leaves)
    int keep_pairs;               // pairs that always work; the first item of pair i < keep_pairs is item i
};

struct ModTable { ModConsts v[MAXM]; };
constexpr ModTable make_mod_table() {
    ModTable t{};
    for (int l = 0; l < MAXM; l++) t.v[l] = mod_consts(l);
    return t;
}
__constant__ ModTable c_modt = make_mod_table();   // part of the device image: present on every device that loads the library
constexpr bool epilogue_reduction_exact() {
    for (int l = 0; l < MAXM; l++)
        if (!magic_ok(l, epi_umax(l))) return false;
    return true;
}
static_assert(epilogue_reduction_exact(), "multiply-high reduction out of range for some modulus");

// work item w -> (plane, tile row, tile column): planes outermost, then bands of `band` tile rows walked column by column
__device__ __forceinline__ void decode_work(const Params &p, int w, int &z, int &tm, int &tn) {
    const int per_plane = p.tiles_m * p.tiles_n;
    z = w / per_plane;
    const int idx = w - z * per_plane, span = p.band * p.tiles_n, first = idx / span * p.band;
    const int rows = min(p.band, p.tiles_m - first), within = idx - (idx / span) * span;
    tm = first + within % rows;
    tn = within / rows;
}

// the epilogue of one 32-column piece of one accumulator row: shared by both kernels
template <bool FUSED_MOD>
__device__ __forceinline__ void store_piece(const Params &p, const ModConsts &mc, const uint32_t (&v)[32], int z, int row, int col) {
    if (row >= p.M || col >= p.N) return;
    if constexpr (FUSED_MOD) {
        int8_t *dst = reinterpret_cast<int8_t *>(p.C) + (size_t)z * p.plane_c + (size_t)row * p.ldc + col;
        uint32_t prev[8] = {};
        if (p.accumulate) {   // residues of the K chunks before this one: residues add, |sum| stays far below 2^31
            if (col + 16 <= p.wcols) { const uint4 q = oz_load(reinterpret_cast<const uint4 *>(dst)); prev[0] = q.x; prev[1] = q.y; prev[2] = q.z; prev[3] = q.w; }
            if (col + 32 <= p.wcols) { const uint4 q = oz_load(reinterpret_cast<const uint4 *>(dst + 16)); prev[4] = q.x; prev[5] = q.y; prev[6] = q.z; prev[7] = q.w; }
        }
        uint32_t o[8];
#pragma unroll
        for (int g = 0; g < 8; g++) {
            uint32_t x[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int add = (int)(int8_t)(prev[g] >> (8 * e));
                const uint32_t u = (v[4 * g + e] + (uint32_t)add) ^ 0x80000000u;   // product (+ earlier chunks) + 2^31, non-negative
                const uint32_t t = (u >> 16) * mc.c16 + (u & 0xFFFFu) + mc.adj;  // same class mod m, below 2^24 + 2^16
                x[e] = t - __umulhi(t, mc.magic) * mc.m - (uint32_t)mc.half;     // balanced residue
            }
            o[g] = pack_low_bytes(x[0], x[1], x[2], x[3]);
        }
        if (col + 16 <= p.wcols) oz_store(reinterpret_cast<uint4 *>(dst), make_uint4(o[0], o[1], o[2], o[3]));
        if (col + 32 <= p.wcols) oz_store(reinterpret_cast<uint4 *>(dst + 16), make_uint4(o[4], o[5], o[6], o[7]));
    } else {
        int32_t *dst = reinterpret_cast<int32_t *>(p.C) + (size_t)z * p.plane_c + (size_t)row * p.ldc + col;
        if (col + 32 <= p.N && ((p.ldc | p.plane_c) & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) {
#pragma unroll
            for (int g = 0; g < 8; g++)
                oz_store(reinterpret_cast<uint4 *>(dst) + g, make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]));
        } else {
#pragma unroll
            for (int e = 0; e < 32; e++)
                if (col + e < p.N) oz_store(dst + e, (int32_t)v[e]);
        }
    }
}

template <bool FUSED_MOD>
__global__ void __launch_bounds__(THREADS, 1) gemm_i8_tc(const __grid_constant__ CUtensorMap mapA,
                                                         const __grid_constant__ CUtensorMap mapB, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto accfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto accempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // the issuer warp owns the tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    const int total = p.tiles_m * p.tiles_n * p.Z;
    const int kblocks = (p.K + BKB - 1) / BKB;
    volatile int *abortp = &abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;   // running stage counter
            for (int w = blockIdx.x; w < total && !*abortp; w += gridDim.x) {
                int z, tm, tn;
                decode_work(p, w, z, tm, tn);
                for (int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, abortp)) break;
                    mbar_expect_tx(full_bar(s), STAGE_BYTES);
                    const uint32_t sa = base + s * STAGE_BYTES;
                    tma_load_3d(sa, &mapA, kb * BKB, tm * BM, z, full_bar(s));
                    tma_load_3d(sa + A_BYTES, &mapB, kb * BKB, tn * BN, z, full_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, n = 0;   // stage counter, tile counter of this CTA
            for (int w = blockIdx.x; w < total && !*abortp; w += gridDim.x, n++) {
                const uint32_t acc = n & 1u;
                if (!mbar_wait(accempty_bar(acc), ((n >> 1) & 1u) ^ 1u, abortp)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
                bool ok = true;
                for (int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, abortp)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = base + s * STAGE_BYTES;
                    const uint64_t da = smem_desc(sa), db = smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BKB / UK; k++)   // +32 bytes of K inside the swizzled row = +2 in the address field
                        mma_i8(d_tmem, da + 2u * k, db + 2u * k, (kb | k) != 0);
                    mma_commit(empty_bar(s));            // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                mma_commit(accfull_bar(acc));            // the accumulator is complete once all MMAs above retire
            }
        }
    } else {
        const int q = warp & 3;                          // a warp may only touch TMEM lanes 32 (warp % 4) .. +31
        ModConsts mc{};
        uint32_t n = 0;
        for (int w = blockIdx.x; w < total && !*abortp; w += gridDim.x, n++) {
            int z, tm, tn;
            decode_work(p, w, z, tm, tn);
            const uint32_t acc = n & 1u;
            if constexpr (FUSED_MOD) mc = c_modt.v[p.first_modulus + z];
            // every lane waits (each needs the barrier's acquire); the vote keeps the warp together if one gave up
            if (!__all_sync(~0u, mbar_wait(accfull_bar(acc), (n >> 1) & 1u, abortp))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = tm * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t v[32];
                tmem_ld32(taddr + c * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                store_piece<FUSED_MOD>(p, mc, v, z, row, tn * BN + c * 32);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accempty_bar(acc));
        }
    }

    // teardown: everyone meets, then the owning warp releases the tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag) {   // word 0: the first code of the launch; words 1..63: per-CTA codes (diagnostics)
        atomicCAS(p.status, 0, abort_flag);
        if (blockIdx.x < 63) p.status[1 + blockIdx.x] = abort_flag;
    }
}


// ---------------------------------------------------------------------------------------------------------------
// Two-CTA variant (cta_group::2): a cluster of two CTAs on one TPC works on one 256 x 256 tile.
// Each CTA loads its own 128 rows of A and its own 128 of the 256 rows of Bt (half the shared-memory fill and read
// traffic per tensor operation of the one-CTA kernel, so 7 stages of 32 KB fit instead of 4 of 48 KB); the leader CTA
// (cluster rank 0) issues tcgen05.mma.cta_group::2 with M = 256, and every CTA finds its 128 rows of the accumulator in
// its own tensor memory. Signals cross the pair like this:
//   full[s]      lives in the leader: its producer expects the bytes of both CTAs, and both producers point their TMA
//                loads at it (cp.async.bulk.tensor with .cta_group::2 may complete on the peer's barrier; no multicast);
//   empty[s]     one per CTA. The issuer commits to the leader's; the leader's producer, once it has seen its own
//                stage free, passes that on to the peer's barrier with a plain remote mbarrier.arrive;
//   accfull[a]   one per CTA, same relay (by the leader's first epilogue warp);
//   accempty[a]  lives in the leader; the 8 epilogue warps of the pair arrive on it.
// Only mbarrier.arrive crosses the pair; tcgen05.commit always targets the issuing CTA's own barriers.
// ---------------------------------------------------------------------------------------------------------------
namespace two {
constexpr int BM2 = 256;                            // rows of A per pair (128 per CTA)
constexpr int STAGES2 = 7;
constexpr int HALF_B = (BN / 2) * BKB;              // this CTA's 128 rows of Bt per stage
constexpr int STAGE2_BYTES = A_BYTES + HALF_B;      // 16 KB + 16 KB
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 1024 + 256;
constexpr int WORK_SLOTS = 4;                       // work items handed out ahead of their use
constexpr int WORK_READERS = 11;                    // per pair: two producers, one issuer, eight epilogue warps
static_assert(8 * (2 * STAGES2 + 5 + 2 * WORK_SLOTS) + 4 * WORK_SLOTS <= 256, "barrier area");
constexpr uint32_t IDESC2 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM2 >> 4) << 24);
}  // namespace two

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {   // the same shared-memory offset in CTA `rank`
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    // default semantics (release at CTA scope): a cluster-scope release here stalled the arriving thread for ~1400 cycles
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t bar) {   // orders this thread's earlier writes, remote ones included
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_acquire_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_acquire_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag, int who) {
    unsigned long long deadline = 0;
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try_acquire_cluster(bar, parity)) return true;
        if ((spin & 1023u) == 1023u) {
            if (*abort_flag) return false;
            const unsigned long long t = now_ns();
            if (!deadline) deadline = t + WAIT_NS;
            else if (t > deadline) { *abort_flag = who; return false; }
        }
    }
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(two::IDESC2), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {   // bar: a barrier of the issuing (leader) CTA
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <bool FUSED_MOD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_i8_tc2(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const Params p) {
    using namespace two;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES2 * STAGE2_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES2 + s); };
    auto accfull_bar = [&](int a) { return bars + 8u * (2 * STAGES2 + a); };
    auto accempty_bar = [&](int a) { return bars + 8u * (2 * STAGES2 + 2 + a); };
    const uint32_t tmem_slot = bars + 8u * (2 * STAGES2 + 4);
    auto work_bar = [&](int s) { return bars + 8u * (2 * STAGES2 + 5 + s); };            // "slot s of the work ring is filled"
    auto taken_bar = [&](int s) { return bars + 8u * (2 * STAGES2 + 5 + WORK_SLOTS + s); };  // "every role has read slot s" (CTA 1's is used)
    const uint32_t work_ring = bars + 8u * (2 * STAGES2 + 5 + 2 * WORK_SLOTS);
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();          // 0 = leader
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES2; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), 8); }
        for (int s = 0; s < WORK_SLOTS; s++) { mbar_init(work_bar(s), 1); mbar_init(taken_bar(s), WORK_READERS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // warp 1 of both CTAs allocates together
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                             // the peer's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    const int tiles_m2 = (p.M + BM2 - 1) / BM2;
    Params pp = p;                                  // decode_work over 256-row tiles
    pp.tiles_m = tiles_m2;
    const int total = tiles_m2 * p.tiles_n * p.Z;
    const int kblocks = (p.K + BKB - 1) / BKB;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    volatile int *abortp = &abort_flag;
    (void)pair; (void)npairs;
    // next work item of this pair, -1 when there is none left: read from the ring the scheduler fills (below)
    auto next_work = [&](uint32_t n, int who) -> int {
        const int s = n % WORK_SLOTS;
        if (!mbar_wait_acquire_cluster(work_bar(s), (n / WORK_SLOTS) & 1u, abortp, who)) return -1;
        int w;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w) : "r"(work_ring + 4u * s) : "memory");
        return w;
    };
    // "this role has read slot n": a plain remote arrive whose address depends on the value read (w >= -1 always, which
    // the compiler cannot know), so it cannot be issued before the load has returned. The scheduler refills the slot only
    // after all eleven arrivals and an atomic round trip; a cluster-scope release on every arrive would stall the issuer
    // for about a microsecond per tile.
    auto work_taken = [&](uint32_t n, int w) {
        const uint32_t never = w < -1 ? 8u : 0u;
        mbar_arrive_cluster(map_to_cta(taken_bar(n % WORK_SLOTS) + never, 1));
    };
#ifdef OZ_TIMING
    long long t_wait = 0, t_all = clock64();
#define OZ_T0 const long long t0_ = clock64();
#define OZ_T1 t_wait += clock64() - t0_;
#else
#define OZ_T0
#define OZ_T1
#endif

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t n = 0; !*abortp; n++) {
                const int w = next_work(n, 0x60 + (int)rank);
                work_taken(n, w);
                if (w < 0) break;
                int z, tm, tn;
                decode_work(pp, w, z, tm, tn);
                for (int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES2;
                    OZ_T0
                    if (!mbar_wait(empty_bar(s), ((it / STAGES2) & 1u) ^ 1u, abortp, 0x10 + (int)rank + ((int)(it & 0xfff) << 8))) break;
                    OZ_T1
                    const uint32_t lead_full = map_to_cta(full_bar(s), 0);
                    if (rank == 0) {
                        if (it >= STAGES2) mbar_arrive_cluster(map_to_cta(empty_bar(s), 1));   // the stage is free in the peer too
                        mbar_expect_tx(full_bar(s), 2 * STAGE2_BYTES);                          // both CTAs' bytes land here
                    }
                    const uint32_t sa = base + s * STAGE2_BYTES;
                    tma_load_3d_pair(sa, &mapA, kb * BKB, tm * BM2 + (int)rank * BM, z, lead_full);
                    tma_load_3d_pair(sa + A_BYTES, &mapB, kb * BKB, tn * BN + (int)rank * (BN / 2), z, lead_full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t it = 0;
            for (uint32_t n = 0; !*abortp; n++) {
                const int w = next_work(n, 0x62);
                work_taken(n, w);
                if (w < 0) break;
                const uint32_t acc = n & 1u;
                if (!mbar_wait(accempty_bar(acc), ((n >> 1) & 1u) ^ 1u, abortp, 0x20 + ((int)(n & 0xfff) << 8))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
                bool ok = true;
                for (int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES2;
                    OZ_T0
                    if (!mbar_wait(full_bar(s), (it / STAGES2) & 1u, abortp, 0x30 + ((int)(it & 0xfff) << 8))) { ok = false; break; }
                    OZ_T1
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = base + s * STAGE2_BYTES;
                    const uint64_t da = smem_desc(sa), db = smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BKB / UK; k++) mma_i8_pair(d_tmem, da + 2u * k, db + 2u * k, (kb | k) != 0);
                    mma_commit_pair(empty_bar(s));
                }
                if (!ok) break;
                mma_commit_pair(accfull_bar(acc));
            }
        } else if (lane == 0) {
            // The peer's otherwise idle warp hands out the work: item n of this pair is whatever the device-wide counter
            // says when the ring has room for it, so a pair that starts late (its SMs still busy with another kernel)
            // or runs slowly simply takes fewer items. The first item needs no round trip to memory.
            for (uint32_t n = 0; !*abortp; n++) {
                const int s = n % WORK_SLOTS;
                if (!mbar_wait(taken_bar(s), ((n / WORK_SLOTS) & 1u) ^ 1u, abortp, 0x70)) break;
                // a pair beyond keep_pairs gives its SMs up when it starts while transfers are outstanding: the kernels that
                // carry them need SMs, and a persistent pair would hold these until the launch ends
                int w;
                if (n == 0 && pair < p.keep_pairs) w = pair;
                else if (n == 0 && p.yield_flag && *(const volatile int *)p.yield_flag != 0) w = -1;
                else w = p.keep_pairs + atomicAdd(p.counter, 1);
                if (w >= total) w = -1;
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(work_ring + 4u * s), "r"(w) : "memory");
                asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(map_to_cta(work_ring + 4u * s, 0)), "r"(w) : "memory");
                mbar_arrive_release_cluster(map_to_cta(work_bar(s), 0));
                mbar_arrive(work_bar(s));
                if (w < 0) break;
            }
        }
    } else {
        const int q = warp & 3;
        ModConsts mc{};
        for (uint32_t n = 0; !*abortp; n++) {
            const int w = next_work(n, 0x64 + (int)rank);
            __syncwarp();
            if (lane == 0) work_taken(n, w);
            if (__any_sync(~0u, w < 0)) break;
            int z, tm, tn;
            decode_work(pp, w, z, tm, tn);
            const uint32_t acc = n & 1u;
            if constexpr (FUSED_MOD) mc = c_modt.v[p.first_modulus + z];
            if (!__all_sync(~0u, mbar_wait(accfull_bar(acc), (n >> 1) & 1u, abortp, 0x40 + (int)rank + ((int)(n & 0xfff) << 8)))) break;
            if (rank == 0 && warp == 2 && lane == 0) mbar_arrive_cluster(map_to_cta(accfull_bar(acc), 1));   // tell the peer's epilogue
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = tm * BM2 + (int)rank * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t v[32];
                tmem_ld32(taddr + c * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                store_piece<FUSED_MOD>(p, mc, v, z, row, tn * BN + c * 32);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(accempty_bar(acc), 0));
        }
    }

#ifdef OZ_TIMING
    if (blockIdx.x < 2 && lane == 0 && warp < 2) {   // words 8..: [cta][warp] = (wait cycles, total cycles) in units of 1024 cycles
        p.status[8 + (blockIdx.x * 2 + warp) * 2] = (int)(t_wait >> 10);
        p.status[9 + (blockIdx.x * 2 + warp) * 2] = (int)((clock64() - t_all) >> 10);
    }
#endif
    // teardown: nobody may leave while the peer can still signal into this CTA's shared memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag) {   // word 0: the first code of the launch; words 1..63: per-CTA codes (diagnostics)
        atomicCAS(p.status, 0, abort_flag);
        if (blockIdx.x < 63) p.status[1 + blockIdx.x] = abort_flag;
    }
}


// ---------------------------------------------------------------------------------------------------------------
// Tensor-pipe probe: the INT8 rate this GPU sustains when nothing but tcgen05.mma runs (the counterpart of the
// reference's register-only mma.sync peak, bench/peak.cu:20-58). Every CTA (or CTA pair) fills one shared-memory stage
// with pseudo-random bytes once and then issues the GEMM kernel's own instruction shape back to back on it, alternating
// between the two accumulators; there is no TMA and no epilogue inside the timed loop. The result is the roofline the
// GEMM kernel is measured against: it includes whatever the power limit does to the clock under full tensor load.
// ---------------------------------------------------------------------------------------------------------------
template <bool PAIR>
__global__ void __launch_bounds__(THREADS, 1) tensor_peak_probe(int iters, int *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar = base + STAGE_BYTES, tmem_slot = bar + 16;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank = 0;
    if constexpr (PAIR) rank = cluster_rank();
    if (threadIdx.x == 0) { abort_flag = 0; mbar_init(bar, 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    {   // fill the stage: 48 KB of hashed bytes (random data draws the power real residues draw)
        uint32_t x = 0x9E3779B9u * (blockIdx.x * THREADS + threadIdx.x + 1);
        uint32_t *w = reinterpret_cast<uint32_t *>(smem_raw + (base - smem_u32(smem_raw)));
        for (int i = threadIdx.x; i < STAGE_BYTES / 4; i += THREADS) { x ^= x << 13; x ^= x >> 17; x ^= x << 5; w[i] = x; }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core's reads
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
    if (warp == 1 && lane == 0 && rank == 0) {
        const uint64_t da = smem_desc(base), db = smem_desc(base + A_BYTES);
        uint32_t phase = 0;
        for (int it = 0; it < iters && !abort_flag; it++) {
#pragma unroll
            for (int a = 0; a < 2; a++)
#pragma unroll
                for (int k = 0; k < BKB / UK; k++) {
                    if constexpr (PAIR) mma_i8_pair(tmem_base + a * ACC_COLS, da + 2u * k, db + 2u * k, 1u);
                    else mma_i8(tmem_base + a * ACC_COLS, da + 2u * k, db + 2u * k, 1u);
                }
            if ((it & 15) == 15 || it == iters - 1) {   // bound the work in flight: wait for everything issued so far
                if constexpr (PAIR) mma_commit_pair(bar); else mma_commit(bar);
                if (!mbar_wait(bar, phase, &abort_flag, 0x50)) break;
                phase ^= 1u;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1) {
        __syncwarp();
        if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag) atomicCAS(status, 0, abort_flag);
}


// Self-test of the bounded wait: one CTA waits on a barrier that nothing will ever complete, with a short budget, and
// must come back with the status word set instead of spinning. Nothing faults and nothing hangs.
__global__ void wait_expiry_selftest(unsigned long long budget_ns, int *status) {
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ int abort_flag;
    const uint32_t bar = smem_u32(&bar_storage);
    if (threadIdx.x == 0) { abort_flag = 0; mbar_init(bar, 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    __syncthreads();
    const bool ok = mbar_wait(bar, 0, &abort_flag, 0x60, budget_ns);   // phase 0 never completes: nobody arrives
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || abort_flag)) atomicCAS(status, 0, abort_flag ? abort_flag : 0x60);
}

}  // namespace g8

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeTiledFn)f;
    }();
    return fn;
}

// 3-D map {k, row, plane} over K-contiguous int8 planes: row pitch ld bytes (multiple of 16), plane pitch `plane` bytes
static cudaError_t make_map(CUtensorMap *map, const int8_t *ptr, int K, int rows, int Z, long long ld, size_t plane, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld & 15) || (plane & 15)) return cudaErrorMisalignedAddress;
    const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)Z};
    const cuuint64_t strides[2] = {(cuuint64_t)ld, (cuuint64_t)plane};
    const cuuint32_t box[3] = {(cuuint32_t)g8::BKB, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

static cudaError_t gemm_setup() {   // the kernels' shared-memory opt-in, on every device the process uses
    static PerDevice pd;
    return pd.once([] {
        cudaError_t e = cudaFuncSetAttribute(g8::gemm_i8_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, g8::SMEM_BYTES);
        if (!e) e = cudaFuncSetAttribute(g8::gemm_i8_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, g8::SMEM_BYTES);
        if (!e) e = cudaFuncSetAttribute(g8::gemm_i8_tc2<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, g8::two::SMEM2_BYTES);
        if (!e) e = cudaFuncSetAttribute(g8::gemm_i8_tc2<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, g8::two::SMEM2_BYTES);
        if (!e) e = cudaFuncSetAttribute(g8::tensor_peak_probe<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, g8::SMEM_BYTES);
        if (!e) e = cudaFuncSetAttribute(g8::tensor_peak_probe<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, g8::SMEM_BYTES);
        return e;
    });
}

// Work counters of the two-CTA kernel. Every launch gets its own, zeroed on the launch's stream just before the kernel, so
// launches that run at the same time on different streams never share one. They come round-robin from a fixed array in
// the device image (nothing is allocated); one is handed out again after WORK_COUNTERS further launches on the device.
constexpr int WORK_COUNTERS = 4096;
static __device__ int g_work_counters[WORK_COUNTERS];
static int *next_work_counter() {
    static int *base[64] = {};
    static unsigned next[64] = {};
    static std::mutex m;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> g(m);
    if (!base[dev]) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_work_counters) != cudaSuccess || !ptr) { cudaGetLastError(); return nullptr; }
        base[dev] = static_cast<int *>(ptr);
    }
    return base[dev] + (next[dev]++ % WORK_COUNTERS);
}

// C[z] = A[z] * Bt[z]^T for z < Z. A: [Z][M][lda] int8, Bt: [Z][N][ldb] int8 (pitches in bytes, multiples of 16; plane
// pitches pa, pb). fused = 0: C is int32 [Z][M][ldc]. fused = 1: C is int8 [Z][M][ldc] holding the balanced residue of
// plane z mod modulus(first_modulus + z); ldc must then be a multiple of 16 with the padding columns writable.
// `status` is a device int the kernel sets if a barrier wait expired. `sms` = 0 uses every SM. accumulate = 1 (fused mode only)
// adds the residues already in C before reducing: the caller splits a long K into chunks whose panels stay in L2.
// `reserve_sms` SMs are left free: a persistent grid never gives an SM back before the launch ends, so a kernel that must
// start while this one runs (the next transfer of a broadcast in flight) needs SMs that this launch does not take.
// With `yield_flag` (a device word) the two-CTA kernel decides that on the device instead: every pair is launched, and the
// pairs that would have been left out leave at once if the word is non-zero when they start, and work otherwise.
cudaError_t gemm_i8_planes(const int8_t *A, const int8_t *Bt, void *C, int M, int N, int K, int Z, long long lda, long long ldb,
                           long long ldc, size_t pa, size_t pb, size_t pc, int fused, int first_modulus, int *status, int sms,
                           cudaStream_t st, int accumulate, int reserve_sms, const int *yield_flag) {
    if (M <= 0 || N <= 0 || K <= 0 || Z <= 0 || (accumulate && !fused)) return cudaErrorInvalidValue;
    if (fused && ((ldc & 15) || first_modulus < 0 || first_modulus + Z > MAXM)) return cudaErrorInvalidValue;
    cudaError_t e = gemm_setup();
    if (e) return e;
    // OZ_GEMM_CTAS=1 selects the one-CTA kernel; the default pairs CTAs (cta_group::2) once there are two tile rows
    static const int want_pair = [] { const char *env = getenv("OZ_GEMM_CTAS"); return !(env && *env == '1'); }();
    const bool pair = want_pair && M > g8::BM;
    CUtensorMap mapA, mapB;
    if ((e = make_map(&mapA, A, K, M, Z, lda, pa, g8::BM))) return e;
    // the TMA box must match the stage layout: a whole 256-row B tile per CTA, or this CTA's 128-row half in a pair
    if ((e = make_map(&mapB, Bt, K, N, Z, ldb, pb, pair ? g8::BN / 2 : g8::BN))) return e;
    g8::Params p{};
    p.M = M; p.N = N; p.K = K; p.Z = Z;
    p.tiles_m = (M + g8::BM - 1) / g8::BM;
    p.tiles_n = (N + g8::BN - 1) / g8::BN;
    // band height in tile rows (OZ_BAND overrides, as in the reference, src/gemm_i8.cuh:149). Measured on B200 with the
    // two-CTA kernel: 16 beats 8 by 5-8 % at n = 16384 and 32768 (B is re-read from HBM once per band) and is no worse at
    // n = 8192; 32 is slower again (the working set of one wave of tiles grows past what L2 serves best).
    {
        static const int env_band = [] { const char *e = getenv("OZ_BAND"); return e && *e ? atoi(e) : 0; }();
        p.band = env_band > 0 ? env_band : 16;
    }
    p.first_modulus = first_modulus;
    p.accumulate = accumulate;
    p.C = C; p.ldc = ldc; p.plane_c = pc; p.status = status;
    p.wcols = (N + 15) / 16 * 16;   // C may be a column window of wider planes: nothing beyond this launch's own pieces is touched
    if (sms <= 0) {
        int dev;
        if ((e = cudaGetDevice(&dev))) return e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev))) return e;
    }
    const long long total = (long long)p.tiles_m * p.tiles_n * Z;
    if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
    // the epilogue's entitlement: rows [0, M) of every plane, whole 16-byte pieces up to wcols (fused) or N int32 (plain)
    OZ_WINDOWS(st, OZK_GEMM_EPILOGUE, fused ? window3d(C, Z, pc, M, (size_t)ldc, (size_t)p.wcols) : window3d(C, Z, pc * 4, M, (size_t)ldc * 4, (size_t)N * 4));
    if (pair) {
        // A persistent grid must be fully resident: ask how many 2-CTA clusters of this kernel the device can hold at once
        static int max_pairs[64][2] = {};   // per device
        int dev_ = 0;
        cudaGetDevice(&dev_);
        int (&mp)[2] = max_pairs[dev_ & 63];
        if (!mp[fused ? 1 : 0]) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(sms & ~1); cfg.blockDim = dim3(g8::THREADS); cfg.dynamicSmemBytes = g8::two::SMEM2_BYTES;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            int n = 0;
            cudaError_t q = fused ? cudaOccupancyMaxActiveClusters(&n, g8::gemm_i8_tc2<true>, &cfg)
                                  : cudaOccupancyMaxActiveClusters(&n, g8::gemm_i8_tc2<false>, &cfg);
            if (q != cudaSuccess || n <= 0) { cudaGetLastError(); n = sms / 2; }
            if (n > sms / 2) n = sms / 2;
            mp[fused ? 1 : 0] = n;
            if (getenv("OZ_DEBUG")) fprintf(stderr, "ozb: %d SMs, at most %d resident CTA pairs\n", sms, n);
        }
        const long long pairs_total = (long long)((M + g8::two::BM2 - 1) / g8::two::BM2) * p.tiles_n * Z;
        int limit = mp[fused ? 1 : 0] - (reserve_sms > 0 ? (reserve_sms + 1) / 2 : 0);
        if (limit < 1) limit = 1;
        const int all = mp[fused ? 1 : 0];
        const int keep = (int)(pairs_total < limit ? pairs_total : limit);
        const int pairs = yield_flag ? (int)(pairs_total < all ? pairs_total : all) : keep;
        p.keep_pairs = keep;
        p.yield_flag = pairs > keep ? yield_flag : nullptr;
        if (!(p.counter = next_work_counter())) return cudaErrorInvalidDevice;
        if ((e = cudaMemsetAsync(p.counter, 0, sizeof(int), st))) return e;
        if (fused) g8::gemm_i8_tc2<true><<<2 * pairs, g8::THREADS, g8::two::SMEM2_BYTES, st>>>(mapA, mapB, p);
        else g8::gemm_i8_tc2<false><<<2 * pairs, g8::THREADS, g8::two::SMEM2_BYTES, st>>>(mapA, mapB, p);
        return cudaGetLastError();
    }
    if (reserve_sms > 0 && sms - reserve_sms >= 1) sms -= reserve_sms;
    const int grid = (int)(total < sms ? total : sms);
    if (fused) g8::gemm_i8_tc<true><<<grid, g8::THREADS, g8::SMEM_BYTES, st>>>(mapA, mapB, p);
    else g8::gemm_i8_tc<false><<<grid, g8::THREADS, g8::SMEM_BYTES, st>>>(mapA, mapB, p);
    return cudaGetLastError();
}


// Runs the tensor-pipe probe on every SM for `iters` rounds of 8 MMAs per CTA (pair = 1: cta_group::2, 8 M-256 MMAs
// per pair) and reports the time and the INT8 rate. `status` as for gemm_i8_planes.
cudaError_t int8_peak_probe(int iters, int pair, float *ms, double *tops, int *status, cudaStream_t st) {
    if (iters <= 0 || iters > (1 << 22)) return cudaErrorInvalidValue;
    cudaError_t e = gemm_setup();
    if (e) return e;
    int dev, sms;
    if ((e = cudaGetDevice(&dev))) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev))) return e;
    cudaEvent_t e0, e1;
    if ((e = cudaEventCreate(&e0))) return e;
    if ((e = cudaEventCreate(&e1))) { cudaEventDestroy(e0); return e; }
    const int grid = sms & ~1;
    cudaEventRecord(e0, st);
    if (pair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid); cfg.blockDim = dim3(g8::THREADS); cfg.dynamicSmemBytes = g8::SMEM_BYTES; cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, g8::tensor_peak_probe<true>, iters, status);
    } else {
        g8::tensor_peak_probe<false><<<grid, g8::THREADS, g8::SMEM_BYTES, st>>>(iters, status);
        e = cudaGetLastError();
    }
    cudaEventRecord(e1, st);
    if (!e) e = cudaEventSynchronize(e1);
    float t = 0;
    if (!e) e = cudaEventElapsedTime(&t, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (e) return e;
    const double per_mma = 2.0 * g8::BM * g8::BN * g8::UK * (pair ? 2 : 1);
    const double units = pair ? grid / 2 : grid;
    if (ms) *ms = t;
    if (tops) *tops = units * (double)iters * 8.0 * per_mma / (t * 1e-3) / 1e12;
    return cudaSuccess;
}

// launches the self-test above; the caller then reads the status word (expected: set)
cudaError_t wait_expiry_selftest(unsigned budget_ms, int *status, cudaStream_t st) {
    if (budget_ms == 0 || budget_ms > 2000) return cudaErrorInvalidValue;
    g8::wait_expiry_selftest<<<1, 32, 0, st>>>((unsigned long long)budget_ms * 1000000ull, status);
    return cudaGetLastError();
}

// violations the checked accesses of this file recorded since the last call (debug build; zeros otherwise)
cudaError_t gemm_violations(unsigned long long out[4]) { return oz_read_violations(out); }

#ifdef OZ_BOUNDS
// Self-test of the checker itself: a checked store one element past a registered window of four ints. The store is not
// performed and the violation is recorded; nothing touches memory it should not.
__global__ void bounds_selftest_kernel(int *buf) { oz_store(buf + threadIdx.x, (int)threadIdx.x); }
cudaError_t bounds_selftest(int *buf5, cudaStream_t st) {
    OZ_WINDOWS(st, OZK_SELFTEST, window1d(buf5, 4 * sizeof(int)));
    bounds_selftest_kernel<<<1, 5, 0, st>>>(buf5);   // thread 4 is the one outside
    return cudaGetLastError();
}
#else
cudaError_t bounds_selftest(int *, cudaStream_t) { return cudaErrorNotSupported; }
#endif

}  // namespace ozk
