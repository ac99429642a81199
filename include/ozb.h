/* ozb.h -- C ABI of libozaki_blackwell.so, the B200 (sm_100a) build of the Ozaki scheme II matrix products.
 *
 * The first eight functions are the reference's C ABI, symbol for symbol (reference file python/capi.cu, lines cited at
 * each declaration): same names, argument order, meaning and error convention, so that the reference's ctypes wrapper
 * (python/ozaki_blackwell/__init__.py:26-36) binds to this library unchanged. All matrices are row-major float64,
 * A is M x K, B is K x N, C is M x N. Every function returns 0 or an error code (a cudaError_t value or one of the
 * OZB_E* codes below); ozb_error() turns a code into text. Nothing aborts the process or throws across this boundary.
 * Calls are serialised by one process-wide mutex, as in the reference (python/capi.cu:19).
 *
 * The functions after them are additions with the same conventions: leading dimensions and streams, the plan-level
 * interface that C++ callers of the reference get from src/ozaki2.cuh (oz::plan / oz::dgemm / oz::release), and the
 * four stages as separate calls, which the reference's phase benchmark launches directly (bench/phases.cu:21-30).
 */
#ifndef OZB_H
#define OZB_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    OZB_EARG = 10001,     /* python/capi.cu:17 -- M, N, K not positive, or moduli outside 8..16 */
    OZB_EK = 10002,       /* python/capi.cu:17 -- K >= 131072: the int32 accumulators of the INT8 GEMMs would overflow */
    OZB_EARCH = 10003,    /* python/capi.cu:17 -- unsupported GPU; here: anything that is not compute capability 10.x */
    OZB_ETIMEOUT = 10004, /* addition: a bounded wait inside the GEMM kernel expired; the result is not valid */
    OZB_ENOTBUILT = 10005,/* addition: the entry point exists for ABI compatibility but this build has no kernel for it */
    OZB_ESIZE = 10006,    /* addition: a size exceeds a stated fixed limit of the entry point */
    OZB_ECOMM = 10007,    /* addition: the exchange between GPUs failed or did not finish in time; the communicator was aborted */
    OZB_ENCCL = 10008     /* addition: the NCCL library (libnccl.so.2) could not be loaded */
};

/* ---- the reference's ABI ------------------------------------------------------------------------------------- */

/* python/capi.cu:52 -- version string of the library */
const char *ozb_version(void);

/* python/capi.cu:54-62 -- text for a return code (0 -> "ok") */
const char *ozb_error(int code);

/* python/capi.cu:65-74 -- current device: name (NUL-terminated, truncated to len), 10*major+minor, L2 size in KiB,
 * SM count. Any of the out pointers may be NULL. */
int ozb_device(char *name, int len, int *sm, int *l2_kib, int *sms);

/* python/capi.cu:77-89 -- C = A B in FP64 with `moduli` moduli (8..16). on_host = 0: A, B, C are device pointers valid
 * on the current device; on_host = 1: host pointers, staged by the library. Synchronous: returns after the device is
 * idle. Dense operands (lda = K, ldb = N, ldc = N). */
int ozb_dgemm(int M, int N, int K, const double *A, const double *B, double *C, int moduli, int on_host);

/* python/capi.cu:92-105 -- (Ch + Cl) = (Ah + Al)(Bh + Bl) in double-double, 32 moduli. */
int ozb_ddgemm(int M, int N, int K, const double *Ah, const double *Al, const double *Bh, const double *Bl, double *Ch,
               double *Cl, int on_host);

/* python/capi.cu:108-121 -- triple-double product, 49 moduli. Exported for ABI compatibility; this build returns
 * OZB_ENOTBUILT after the argument checks. */
int ozb_tdgemm(int M, int N, int K, const double *A0, const double *A1, const double *A2, const double *B0,
               const double *B1, const double *B2, double *C0, double *C1, double *C2, int on_host);

/* python/capi.cu:124-127 -- free the cached plans (device memory); the next call plans again. Also frees what
 * ozb_dgemm_mg keeps between calls (ozb_mg_release). */
void ozb_release(void);

/* python/capi.cu:130-164 -- GPU time of `reps` (1..101) products of fixed pseudo-random n x n matrices resident on the
 * device, through the public entry point; the median in ms. kind 0 FP64 (16 moduli), 1 double-double, 2 triple-double. */
int ozb_bench(int n, int kind, int reps, double *median_ms);

/* ---- additions ----------------------------------------------------------------------------------------------- */

/* src/ozaki2.cuh:101-108 (oz::bits_for) -- scaling bits for nm moduli at inner dimension K; -1 if K >= 131072 */
int ozb_bits_for(int nm, int K, int maxbits);
/* src/ozaki2.cuh:24-34 (oz::modulus) -- the l-th modulus, 0 <= l < 49 (0 otherwise) */
int ozb_modulus(int l);

/* The reference's oz::Plan (src/ozaki2.cuh:116-132) as an opaque handle: workspaces for one (M, N, K, moduli) shape on
 * the device that is current at creation. */
typedef struct ozb_plan ozb_plan;
/* src/ozaki2.cuh:122-131 (oz::plan). The plan's workspaces live on the device that is current at this call; the
 * computing ozb_plan_* calls return cudaErrorInvalidDevice (101) when made with another device current. */
int ozb_plan_create(int M, int N, int K, int moduli, int maxbits, ozb_plan **out);
/* src/ozaki2.cuh:132 (oz::release) */
void ozb_plan_destroy(ozb_plan *p);
/* src/ozaki2.cuh:134-164 (oz::dgemm) with leading dimensions (in elements) and a stream (a cudaStream_t passed as
 * void*; NULL = the legacy default stream, which the reference uses). Asynchronous: it only enqueues work. */
int ozb_plan_dgemm(ozb_plan *p, const double *A, long long lda, const double *B, long long ldb, double *C, long long ldc,
                   void *stream);
/* Split form for callers that stream B in column panels (multi-GPU row-block sharding, host staging): residues of A
 * once, then any number of column panels [j0, j0 + ncols) of B and C; j0 must be a multiple of 256. B and C point at
 * the panel's first column. */
int ozb_plan_set_a(ozb_plan *p, const double *A, long long lda, void *stream);
int ozb_plan_panel(ozb_plan *p, const double *B, long long ldb, double *C, long long ldc, int j0, int ncols, void *stream);
/* The same product with B delivered in chunks of rows (a broadcast or a host transfer in flight): ozb_plan_b_begin once,
 * ozb_plan_b_rows for every chunk in any order (it only accumulates the column maxima of those rows), ozb_plan_b_finish
 * with the complete B (forms the residues), then ozb_plan_multiply with the A given to ozb_plan_set_a. The prepared
 * operands stay valid, so one B can be multiplied by several A (call ozb_plan_set_a and ozb_plan_multiply again). */
int ozb_plan_b_begin(ozb_plan *p, void *stream);
int ozb_plan_b_rows(ozb_plan *p, const double *Brows, long long ldb, int rows, void *stream);
int ozb_plan_b_finish(ozb_plan *p, const double *B, long long ldb, void *stream);
int ozb_plan_multiply(ozb_plan *p, double *C, long long ldc, void *stream);
/* The same when the column maxima of B are known before B itself is complete (the holder of B computed them and sent
 * them ahead): ozb_cols_absmax accumulates max |x| of every column of a row-major block into `colmax` (cols 64-bit words,
 * the bit patterns of non-negative doubles; the caller clears them once), and ozb_plan_b_rows_residues forms the scales
 * and the residues of rows [k0, k0 + rows) of B from such maxima as soon as those rows are there (k0 a multiple of 128).
 * When all rows have been given, ozb_plan_multiply. */
int ozb_cols_absmax(const double *X, int rows, int cols, long long ldx, void *colmax, void *stream);
int ozb_plan_b_rows_residues(ozb_plan *p, const double *Brows, long long ldb, int k0, int rows, const void *colmax, void *stream);
/* Workspace view, for stage-by-stage checks against the reference's Plan fields (src/ozaki2.cuh:117-119):
 * Ar [nm][M][Kp] int8, Br [nm][N][Kp] int8, Cr [nm][M][Np] int8 (balanced residues of the products, where the
 * reference keeps int32 Cl), sa [M], sb [N]. */
int ozb_plan_view(ozb_plan *p, int *bits, int *Kp, int *Np, int8_t **Ar, int8_t **Br, int8_t **Cr, int **sa, int **sb);
/* Device status word of the plan: 0, or OZB_ETIMEOUT if a bounded wait expired in a kernel launched through it.
 * Synchronises the stream the last call used. */
int ozb_plan_status(ozb_plan *p);
/* Phase timing (src/ozaki2.cuh:135-153, the reference's OZ_PROF): with `slots` > 0 every ozb_plan_dgemm records
 * events on its stream (no host synchronisation) into slot (call number mod slots); slots = 0 turns it off. A plan
 * created while the environment variable OZ_PROF is set starts with one slot and prints the reference's line on stderr
 * after every product (which synchronises). */
int ozb_plan_profile(ozb_plan *p, int slots);
/* Milliseconds of the product recorded in `slot`: ms[0] start of the product to the start of the first GEMM (exposed
 * scaling + residues), ms[1] sum of the GEMM kernels' own durations, ms[2] end of the last GEMM to the end of the
 * product (exposed CRT), ms[3] the whole product. By default a product is one column panel on the caller's stream and
 * the three parts add up to ms[3]. A plan made while the environment variable OZ_PANELS is 2..8 cuts the columns into
 * that many panels whose B-residue, GEMM and CRT stages overlap on internal streams (measured slower on B200, hence not
 * the default); ms[1] is then the sum over the panels. Waits for that product to finish. */
int ozb_plan_phase_ms(ozb_plan *p, int slot, float ms[4]);
/* The same product kernel by kernel (one-panel plans only, OZB_EARG otherwise) -- what the reference's OZ_PROF line and its
 * phase benchmark report (src/ozaki2.cuh:147-152, bench/phases.cu:21-30): ms[0] scales + residues of A, ms[1] column maxima
 * of B, ms[2] residues of B, ms[3] the INT8 GEMM launches, ms[4] the reconstruction. */
int ozb_plan_kernel_ms(ozb_plan *p, int slot, float ms[5]);

/* ozb_dgemm with leading dimensions, on device pointers, on a stream, without the final synchronisation. Uses the same
 * cached plan as ozb_dgemm (one per precision, replaced when the shape changes). ozb_dgemm_ex, ozb_dgemm_norm and
 * ozb_ddgemm_ex share that plan's workspaces: the library orders each such product after the previous one (an event
 * per plan), so calls on different streams are safe but do not overlap; use ozb_plan_create for independent plans.
 * A bounded wait that expired in one of these products is reported by ozb_status. */
int ozb_dgemm_ex(int M, int N, int K, const double *A, long long lda, const double *B, long long ldb, double *C,
                 long long ldc, int moduli, void *stream);

/* ---- several GPUs of one machine --------------------------------------------------------------------------------
 * No counterpart in the reference, which is single-GPU; the entry shape extended is ozb_dgemm (python/capi.cu:77-89).
 * The product is partitioned by output row blocks: every rank (one per GPU) owns a block of rows of A and produces the
 * same rows of C; B is held by one rank and broadcast once per product over NVLink by NCCL (loaded at run time), nothing
 * else is exchanged, and the rows every rank returns are bit-identical to the same rows of the single-GPU product. */

/* One process, `ndev` GPUs (devices 0 .. ndev-1): C = A B as ozb_dgemm computes it. on_host = 1: A, B, C are host
 * pointers (pinned memory lets every GPU stream its rows while it computes). on_host = 0: device pointers on the calling
 * thread's current device, which must be one of the ndev; the other GPUs get their rows by peer copies. Synchronous.
 * The communicators and workspaces are cached until ozb_mg_release or a call with another ndev. */
int ozb_dgemm_mg(int M, int N, int K, const double *A, const double *B, double *C, int moduli, int on_host, int ndev);
void ozb_mg_release(void);

/* One rank per process (or thread). Rendezvous: one rank fills a 128-byte id with ozb_mg_unique_id and hands it to the
 * others by any means; every rank then calls ozb_mg_create with its device current. timeout_ms (0: 30 s) bounds every
 * host-side wait of the handle: setting up, queueing a transfer, waiting for a product. When it runs out -- a peer never
 * joined or is gone -- the communicator is aborted and the call returns OZB_ECOMM, as does every later call on the
 * handle; the CUDA context stays usable. */
#define OZB_MG_ID_BYTES 128
typedef struct ozb_mg ozb_mg;
int ozb_mg_unique_id(void *id);
int ozb_mg_create(int world, int rank, const void *id, int timeout_ms, ozb_mg **out);
void ozb_mg_destroy(ozb_mg *g);
/* This rank's rows: C_local (m_local x N) = A_local (m_local x K) B (K x N). B is read on rank `root` only (others may
 * pass NULL). on_host = 0: device pointers with leading dimensions, asynchronous on `stream` and on a communication
 * stream of the handle; ozb_mg_wait tells how the product ended. on_host = 1: dense host pointers (lda = K, ldb = N,
 * ldc = N), copies pipelined with the broadcast and the computation, synchronous. Every rank must make the same
 * sequence of calls with the same N, K, moduli and root. */
int ozb_mg_dgemm(ozb_mg *g, int m_local, int N, int K, const double *A, long long lda, const double *B, long long ldb, double *C,
                 long long ldc, int moduli, int root, int on_host, void *stream);
/* Waits (within the handle's budget) for the last product queued on the handle: 0, OZB_ETIMEOUT (a bounded wait inside a
 * GEMM kernel expired) or OZB_ECOMM. */
int ozb_mg_wait(ozb_mg *g);
/* What a device-operand product of this shape would do, without doing it (plain arithmetic, no device needed): *layout as
 * in ozb_mg_info, *pieces = transfers of B, *ranges = K ranges whose GEMMs are launched as their pieces land (1: one launch
 * after the last piece). Any pointer may be NULL. */
int ozb_mg_schedule(int m_local, int N, int K, int moduli, int *layout, int *pieces, int *ranges);
/* The pieces themselves: piece i carries rows [k0[i], k0[i] + len[i]) of B; range_len[i] > 0 says that the GEMMs of the K
 * range [range_k0[i], range_k0[i] + range_len[i]) are launched behind it. `layout` 0 / 1 as above, -1: as the library would
 * choose. Fills at most `cap` entries of each array (NULL arrays are skipped) and returns the number of pieces, or a
 * negative error code (-OZB_EARG, -OZB_EK). Plain arithmetic, no device needed. */
int ozb_mg_schedule_pieces(int m_local, int N, int K, int moduli, int layout, int cap, int *k0, int *len, int *range_k0,
                           int *range_len);
/* How the last device-operand product moved B: *layout 0 = in one transfer, 1 = column maxima first, then pieces of rows
 * consumed as they land; *pieces = number of transfers of B; *kernels = kernels of this library it launched on this rank
 * (NCCL's own are not counted). Any pointer may be NULL. */
int ozb_mg_info(ozb_mg *g, int *layout, int *pieces, int *kernels);

/* bench/oz_strassen.cu:74-97,247 (scales_norm) -- C = A B with the reference's optional scaling from the 2-norm of each row
 * of A and column of B instead of its largest entry (Cauchy-Schwarz bounds the integer products without K, so more bits
 * survive: at large K one modulus fewer gives the same error). Opt-in: the result is NOT bit-identical to ozb_dgemm, it is
 * bit-identical to the reference's pipeline run with scales_norm. Device pointers, leading dimensions, asynchronous. */
int ozb_dgemm_norm(int M, int N, int K, const double *A, long long lda, const double *B, long long ldb, double *C, long long ldc,
                   int moduli, void *stream);

/* bench/oz_strassen.cu:78-97 (scales_norm) alone, as a stage: the 2-norm scales of the `nvec` rows (by_rows = 1: rows of
 * `len` contiguous doubles, pitch ldx) or of the `nvec` columns (by_rows = 0: a row-major len x nvec matrix, pitch ldx) for
 * `moduli` moduli, beta = floor((log2 P - 1.001) / 2) as bench/oz_strassen.cu:247 sets it. Asynchronous. */
int ozb_scales_norm(const double *X, int nvec, int len, long long ldx, int by_rows, int moduli, int *s, void *stream);

/* src/ozaki_dd.cuh:143-148 (oz::ddgemm_t) -- the double-double product with leading dimensions (elements), the
 * reference's mode (0: C = AB, 1: C -= AB, 2: C = -AB, used by its LU solvers to update blocks in place), a modulus
 * count in {24, 28, 32} and a stream; device pointers, no final synchronisation. */
int ozb_ddgemm_ex(int M, int N, int K, const double *Ah, const double *Al, long long lda, const double *Bh, const double *Bl,
                  long long ldb, double *Ch, double *Cl, long long ldo, int moduli, int mode, void *stream);

/* llm/tgemm.cu:61-162 (the reference's tiled exact product, F8 mode) checked as the reference checks it, against the
 * exact sum rounded once (llm/ultra.cu:336-369) -- Y = RN_fp32(X (W o S)): X is M x K bf16 (uint16 bit patterns), W is
 * K x N FP8 E4M3 bytes, S holds one FP32 scale per 128 x 128 block of W ([ceil(K/128)][ceil(N/128)]), Y is M x N FP32;
 * all dense row-major device pointers. Every output is the round-to-nearest-even FP32 value of the exact sum. Operands
 * whose exponents span more than the 62-bit windows are truncated; an output whose rounding that leaves undecided is
 * returned as NaN and counted in *open (0 for ordinary data). *moduli receives the number of INT8 GEMM planes used
 * (8..19, chosen from the data). Synchronous. Non-finite inputs give OZB_EARG. */
int ozb_bf16_fp8_gemm(int M, int N, int K, const void *X, const void *W, const float *S, float *Y, int *open, int *moduli,
                      void *stream);

/* The four stages on caller-owned device buffers (what bench/phases.cu launches one by one). Asynchronous.
 * Pitches: ld of int8 planes in bytes and a multiple of 16; `plane` = distance between planes in elements. */
/* src/ozaki2.cuh:56-78 -- scales + residues of an A-like operand (rows of `len` contiguous doubles, pitch ldx) */
int ozb_scale_residues_rows(int moduli, const double *X, int rows, int len, long long ldx, int bits, int *s, int8_t *R,
                            int ld, size_t plane, void *stream);
/* src/ozaki2.cuh:56-78 -- the same for a B-like operand (row-major rows x cols, scaled per column, written transposed
 * as R[l][col][row]); colmax is scratch of `cols` 64-bit words */
int ozb_scale_residues_cols(int moduli, const double *X, int rows, int cols, long long ldx, int bits, void *colmax, int *s,
                            int8_t *R, int ld, size_t plane, void *stream);
/* No counterpart in the reference. The column pass of ozb_scale_residues_cols for callers that cannot allocate device
 * memory when they call: programs whose GPU memory is wholly owned by another allocator (a serving engine or framework
 * pool that reserved the HBM at start-up), and latency-critical loops that cannot take the device-wide synchronisation
 * of cudaMalloc / cudaFree. Same arguments minus the scratch: the per-column scratch lives in a fixed array inside the
 * library (512 KiB on every GPU that loads it, for the life of the process), so `cols` may not exceed 65536
 * (OZB_ESIZE otherwise). The call allocates nothing. The first call on each device looks up the array's device address
 * and should therefore be made before any stream capture; all calls on a device share the array (each clears what it
 * uses, on its stream), so calls that may overlap on the GPU must be ordered by the caller. */
int ozb_scale_residues_cols_static(int moduli, const double *X, int rows, int cols, long long ldx, int bits, int *s,
                                   int8_t *R, int ld, size_t plane, void *stream);
/* src/gemm_i8.cuh:148-160 (oz::gemm_i8_run) -- C[z] = A[z] Bt[z]^T, Z planes, int32 out [Z][M][ldc]. No padding
 * requirement on M, N, K; lda/ldb in bytes, multiples of 16, base pointers 16-byte aligned. */
int ozb_gemm_i8(const int8_t *A, const int8_t *Bt, int32_t *C, int M, int N, int K, int Z, long long lda, long long ldb,
                long long ldc, size_t plane_a, size_t plane_b, size_t plane_c, void *stream);
/* The same with the reduction of src/ozaki2.cuh:88 fused in: plane z comes out as int8 balanced residues mod
 * ozb_modulus(first_modulus + z); ldc a multiple of 16 */
int ozb_gemm_i8_mod(const int8_t *A, const int8_t *Bt, int8_t *C, int M, int N, int K, int Z, long long lda, long long ldb,
                    long long ldc, size_t plane_a, size_t plane_b, size_t plane_c, int first_modulus, void *stream);
/* The same beside other kernels that need SMs while it runs (the transfer kernels of a broadcast in flight): the
 * persistent grid leaves `reserve_sms` SMs free. With `busy` (a device word, may be NULL) that is decided on the device:
 * every CTA pair is launched, and the pairs that would have been left out leave at once if *busy is non-zero when they
 * start and work otherwise. No counterpart in the reference (it has no multi-GPU path). */
int ozb_gemm_i8_mod_beside(const int8_t *A, const int8_t *Bt, int8_t *C, int M, int N, int K, int Z, long long lda,
                           long long ldb, long long ldc, size_t plane_a, size_t plane_b, size_t plane_c, int first_modulus,
                           int reserve_sms, const int *busy, void *stream);
/* src/ozaki2.cuh:82-97 (oz::crt) -- from int32 planes of raw products (the reference's layout) */
int ozb_crt_i32(int moduli, const int32_t *Cl, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
                double *C, long long ldc, void *stream);
/* the same from int8 planes of balanced residues (ldr a multiple of 4) */
int ozb_crt_i8(int moduli, const int8_t *Cr, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
               double *C, long long ldc, void *stream);
/* bench/peak.cu:20-58 (the reference's register-only mma.sync peak) -- the INT8 rate of this GPU's tensor cores with
 * nothing else running: every SM issues the GEMM kernel's tcgen05.mma shape back to back on one shared-memory stage of
 * pseudo-random bytes, `iters` (1..2^22) rounds of 8 instructions per CTA (pair = 0) or per CTA pair (pair = 1,
 * cta_group::2). Synchronous. Returns the elapsed ms and tera-operations per second (2 ops per multiply-add). */
int ozb_int8_peak(int iters, int pair, float *ms, double *tops);
/* No counterpart in the reference (its kernels have no waits that could expire). Self-test of the failure path: one CTA
 * waits, with a budget of budget_ms (1..2000), on a barrier that nothing completes. The expected return value is
 * OZB_ETIMEOUT: the wait gave up, raised the status word and the kernel returned normally; the context stays usable. */
int ozb_selftest_wait_expiry(int budget_ms);
/* No counterpart in the reference (its debugging aid is a poison fill of the workspaces, src/ozaki_hol.cuh:498). The
 * checked-access debug build of this library (libozaki_blackwell_bounds.so, compiled with -DOZ_BOUNDS) tests every global
 * load and store of the scale / residue / reconstruction kernels and of the GEMM epilogue against the exact bytes the
 * launch is entitled to; an access outside is skipped and recorded. ozb_bounds_report synchronises the device, returns
 * out[0] = violations since the last call, out[1] = address, out[2] = kernel id, out[3] = size of the first one, and clears
 * the record. ozb_selftest_bounds makes one checked store just outside a registered window and expects it to be skipped;
 * the following ozb_bounds_report then shows exactly one violation. Both return OZB_ENOTBUILT in the normal build. */
int ozb_bounds_report(unsigned long long out[4]);
int ozb_selftest_bounds(void);
/* Status of the stage calls above (they share one status word per device) and of the cached plans behind ozb_dgemm_ex,
 * ozb_dgemm_norm and ozb_ddgemm_ex on the current device: 0 or OZB_ETIMEOUT. Synchronises the device. */
int ozb_status(void);

#ifdef __cplusplus
}
#endif
#endif /* OZB_H */
