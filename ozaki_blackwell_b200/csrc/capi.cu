// capi.cu -- the C ABI (include/ozb.h) and the plan/driver layer behind it.
//
// Mirrors the reference's python/capi.cu (argument checks, error codes, one mutex, one cached plan per precision, host
// staging, the built-in benchmark) and src/ozaki2.cuh:116-164 (Plan, plan, release, dgemm), over this library's own
// kernels. There is no CPU path: every entry point that computes needs a compute-capability-10 device and fails with
// OZB_EARCH otherwise.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include "../../include/ozb.h"
#include "oz_common.cuh"
#include "oz_kernels.h"
#include "oz_plan.h"

#define OZB_API extern "C" __attribute__((visibility("default")))
#ifndef OZB_VERSION
#define OZB_VERSION "0.1.0-b200"
#endif

using namespace ozk;

// ---------------------------------------------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------------------------------------------
static int round_up(int x, int to) { return (x + to - 1) / to * to; }
static int plan_make(int M, int N, int K, int nm, int maxbits, ozb_plan **out);
static void plan_free(ozb_plan *p);
static int read_status(int *dev_words);
int ozb_plan_make_internal(int M, int N, int K, int nm, int maxbits, ozb_plan **out) { return plan_make(M, N, K, nm, maxbits, out); }
void ozb_plan_free_internal(ozb_plan *p) { plan_free(p); }
int ozb_read_status_words(int *dev_words) { return read_status(dev_words); }

static int bits_for_impl(int nm, int K, int maxbits) {   // src/ozaki2.cuh:101-108, with the abort turned into -1
    double log2P = 0;
    for (int l = 0; l < nm; l++) log2P += log2((double)modulus(l));
    if (K >= 131072) return -1;
    const int b = (int)floor((log2P - 2 - log2((double)K)) / 2);
    return b > maxbits ? maxbits : b;
}

static void plan_free(ozb_plan *p) {
    if (!p) return;
    cudaFree(p->Ar); cudaFree(p->Br); cudaFree(p->Cr); cudaFree(p->sa); cudaFree(p->sb); cudaFree(p->status); cudaFree(p->colmax);
    for (int i = 0; i < EV_PER_SLOT * p->slots; i++) cudaEventDestroy(p->ev[i]);
    delete[] p->ev;
    if (p->s1) cudaStreamDestroy(p->s1);
    if (p->s2) cudaStreamDestroy(p->s2);
    if (p->evFork) cudaEventDestroy(p->evFork);
    if (p->evJoin) cudaEventDestroy(p->evJoin);
    for (int i = 0; i < MAXP; i++) { if (p->evB[i]) cudaEventDestroy(p->evB[i]); if (p->evG[i]) cudaEventDestroy(p->evG[i]); }
    cudaFree(p->hA); cudaFree(p->hB); cudaFree(p->hC);
    if (p->sIn) cudaStreamDestroy(p->sIn);
    if (p->sRun) cudaStreamDestroy(p->sRun);
    if (p->sOut) cudaStreamDestroy(p->sOut);
    for (auto &e : p->evIn) if (e) cudaEventDestroy(e);
    for (auto &e : p->evRun) if (e) cudaEventDestroy(e);
    if (p->evDone) cudaEventDestroy(p->evDone);
    delete p;
}

static int plan_profile(ozb_plan *p, int slots) {
    for (int i = 0; i < EV_PER_SLOT * p->slots; i++) cudaEventDestroy(p->ev[i]);
    delete[] p->ev;
    p->ev = nullptr; p->slots = 0; p->calls = 0;
    if (slots <= 0) return 0;
    p->ev = new cudaEvent_t[EV_PER_SLOT * slots];
    for (int i = 0; i < EV_PER_SLOT * slots; i++)
        if (cudaError_t e = cudaEventCreate(&p->ev[i])) { for (int j = 0; j < i; j++) cudaEventDestroy(p->ev[j]); delete[] p->ev; p->ev = nullptr; return (int)e; }
    p->slots = slots;
    return 0;
}
// ms[0]: start of the product to the start of the first GEMM (exposed scaling + residues); ms[1]: sum of the GEMM
// kernels' durations; ms[2]: end of the last GEMM to the end of the product (exposed CRT); ms[3]: the whole product
static int plan_phase_ms(ozb_plan *p, int slot, float ms[4]) {
    if (slot < 0 || slot >= p->slots || slot >= p->calls) return OZB_EARG;
    cudaEvent_t *ev = p->ev + EV_PER_SLOT * slot;
    if (cudaError_t e = cudaEventSynchronize(ev[1])) return (int)e;
    cudaError_t e = cudaEventElapsedTime(&ms[0], ev[0], ev[2]);
    ms[1] = 0;
    for (int q = 0; q < p->panels && !e; q++) { float t; e = cudaEventElapsedTime(&t, ev[2 + 2 * q], ev[3 + 2 * q]); ms[1] += t; }
    if (!e) e = cudaEventElapsedTime(&ms[2], ev[3 + 2 * (p->panels - 1)], ev[1]);
    if (!e) e = cudaEventElapsedTime(&ms[3], ev[0], ev[1]);
    return (int)e;
}

// the kernels of a one-panel product, one by one: ms[0] residues of A (row_scale_residues), ms[1] column maxima of B
// (memset + col_absmax), ms[2] residues of B (col_residues_t), ms[3] the GEMM launches, ms[4] the reconstruction (crt_kernel)
static int plan_kernel_ms(ozb_plan *p, int slot, float ms[5]) {
    if (slot < 0 || slot >= p->slots || slot >= p->calls || p->panels != 1) return OZB_EARG;
    cudaEvent_t *ev = p->ev + EV_PER_SLOT * slot;
    if (cudaError_t e = cudaEventSynchronize(ev[1])) return (int)e;
    cudaError_t e = cudaEventElapsedTime(&ms[0], ev[0], ev[EV_ROWS]);
    if (!e) e = cudaEventElapsedTime(&ms[1], ev[EV_ROWS], ev[EV_ABSMAX]);
    if (!e) e = cudaEventElapsedTime(&ms[2], ev[EV_ABSMAX], ev[2]);
    if (!e) e = cudaEventElapsedTime(&ms[3], ev[2], ev[3]);
    if (!e) e = cudaEventElapsedTime(&ms[4], ev[3], ev[1]);
    return (int)e;
}

static int plan_make(int M, int N, int K, int nm, int maxbits, ozb_plan **out) {
    ozb_plan *p = new ozb_plan();
    memset(p, 0, sizeof *p);
    p->M = M; p->N = N; p->K = K; p->nm = nm; p->maxbits = maxbits;
    cudaGetDevice(&p->dev);
    p->bits = bits_for_impl(nm, K, maxbits);
    p->Kp = round_up(K, 128);   // rows start on 128-byte lines; the TMA extent is K itself, so the padding is never read
    p->Np = round_up(N, 16);
    p->planeA = (size_t)M * p->Kp; p->planeB = (size_t)N * p->Kp; p->planeC = (size_t)M * p->Np;
    cudaError_t e = cudaMalloc(&p->Ar, nm * p->planeA);
    if (!e) e = cudaMalloc(&p->Br, nm * p->planeB);
    if (!e) e = cudaMalloc(&p->Cr, nm * p->planeC);
    if (!e) e = cudaMalloc(&p->sa, (size_t)M * 4);
    if (!e) e = cudaMalloc(&p->sb, (size_t)N * 4);
    if (!e) e = cudaMalloc(&p->colmax, (size_t)N * 8);
    if (!e) e = cudaMalloc(&p->status, 256);
    if (!e) e = cudaMemset(p->status, 0, 256);
    if (!e) e = cudaEventCreateWithFlags(&p->evDone, cudaEventDisableTiming);
#ifdef OZ_BOUNDS
    // debug build: the workspaces start out poisoned (as the reference does, src/ozaki_hol.cuh:498), so a byte that is read
    // without having been written shows up in the result
    if (!e) e = cudaMemset(p->Ar, 0x7B, nm * p->planeA);
    if (!e) e = cudaMemset(p->Br, 0x7B, nm * p->planeB);
    if (!e) e = cudaMemset(p->Cr, 0x7B, nm * p->planeC);
#endif
    // panels: one by default; OZ_PANELS = 2..8 splits the columns and overlaps the stages of different panels
    p->panel_width = round_up(N, 256); p->panels = 1;
    {
        const char *env = getenv("OZ_PANELS");
        int want = env && *env ? atoi(env) : 1;   // measured on B200: overlapping the stages slows the GEMMs by more than it hides
        if (want > MAXP) want = MAXP;
        if (want > 1) { p->panel_width = round_up((N + want - 1) / want, 256); p->panels = (N + p->panel_width - 1) / p->panel_width; }
    }
    if (!e && p->panels > 1) {
        e = cudaStreamCreateWithFlags(&p->s1, cudaStreamNonBlocking);
        if (!e) e = cudaStreamCreateWithFlags(&p->s2, cudaStreamNonBlocking);
        if (!e) e = cudaEventCreateWithFlags(&p->evFork, cudaEventDisableTiming);
        if (!e) e = cudaEventCreateWithFlags(&p->evJoin, cudaEventDisableTiming);
        for (int i = 0; i < MAXP && !e; i++) { e = cudaEventCreateWithFlags(&p->evB[i], cudaEventDisableTiming); if (!e) e = cudaEventCreateWithFlags(&p->evG[i], cudaEventDisableTiming); }
    }
    p->env_prof = getenv("OZ_PROF") != nullptr;
    if (!e && p->env_prof) e = (cudaError_t)plan_profile(p, 1);
    if (e) { cudaGetLastError(); plan_free(p); return (int)e; }
    *out = p;
    return 0;
}

// The fused GEMMs of one column panel over the inner range [k0, k0 + klen). A long range is cut into chunks of about 8192:
// within one chunk the A band and the B panels that the resident CTAs share fit the L2 cache, whereas at K = 32768 they do
// not (measured: 1.8 instead of 3.2 POP/s, the kernel turns HBM-bound); later chunks add to the residues the earlier ones
// stored. `accumulate` says whether the first chunk already finds residues of an earlier part of K in Cr.
static cudaError_t gemm_range(ozb_plan *p, const int8_t *Br, int8_t *Cr, int n, cudaStream_t st, int i0, int m, int k0, int klen,
                              int accumulate, int *launches = nullptr, int reserve_sms = 0, const int *yield_flag = nullptr) {
    if (m < 0) m = p->M;   // rows [i0, i0 + m) of A and C
    static const int target = [] { const char *env = getenv("OZ_KCHUNK"); const int v = env && *env ? atoi(env) : 0; return v >= 1024 ? v : 8192; }();
    const int chunks = klen > target + target / 2 ? (klen + target - 1) / target : 1;
    const int kc = round_up((klen + chunks - 1) / chunks, 128);
    for (int k = k0, i = 0; k < k0 + klen; k += kc, i++) {
        const int len = k0 + klen - k < kc ? k0 + klen - k : kc;
        cudaError_t e = gemm_i8_planes(p->Ar + (size_t)i0 * p->Kp + k, Br + k, Cr + (size_t)i0 * p->Np, m, n, len, p->nm, p->Kp, p->Kp,
                                       p->Np, p->planeA, p->planeB, p->planeC, 1, 0, p->status, 0, st, accumulate || i > 0, reserve_sms, yield_flag);
        if (e) return e;
        if (launches) ++*launches;
    }
    return cudaSuccess;
}
static cudaError_t gemm_chunks(ozb_plan *p, const int8_t *Br, int8_t *Cr, int n, cudaStream_t st, int i0 = 0, int m = -1) {
    return gemm_range(p, Br, Cr, n, st, i0, m, 0, p->K, 0);
}
cudaError_t ozb_plan_gemm_range(ozb_plan *p, int n, int k0, int klen, int accumulate, cudaStream_t st, int i0, int m, int *launches,
                                int reserve_sms, const int *yield_flag) {
    return gemm_range(p, p->Br, p->Cr, n, st, i0, m, k0, klen, accumulate, launches, reserve_sms, yield_flag);
}

// a plan's workspaces live on the device that was current when it was made: launching from another one would read them
// through peer mappings at best
static bool on_plan_device(const ozb_plan *p) {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess && dev == p->dev;
}
static int plan_set_a(ozb_plan *p, const double *A, long long lda, cudaStream_t st) {
    p->last = st;
    return (int)scale_residues_rows(p->nm, A, p->M, p->K, lda, p->bits, p->sa, p->Ar, p->Kp, p->planeA, st);
}
// columns [j0, j0 + n) of B and C; B and C point at column j0
static int plan_panel(ozb_plan *p, const double *B, long long ldb, double *C, long long ldc, int j0, int n, cudaStream_t st,
                      cudaEvent_t *ev) {
    p->last = st;
    int8_t *Br = p->Br + (size_t)j0 * p->Kp, *Cr = p->Cr + j0;
    cudaError_t e = scale_residues_cols(p->nm, B, p->K, n, ldb, p->bits, p->colmax + j0, p->sb + j0, Br, p->Kp, p->planeB, st);
    if (e) return (int)e;
    if (ev) cudaEventRecord(ev[1], st);
    // the epilogue writes whole 16-byte pieces: the panel's pitch view must allow n rounded up to 16 inside Np
    e = gemm_chunks(p, Br, Cr, n, st);
    if (e) return (int)e;
    if (ev) cudaEventRecord(ev[2], st);
    e = crt_from_i8(p->nm, Cr, p->planeC, p->M, n, p->Np, p->sa, p->sb + j0, C, ldc, st);
    return (int)e;
}
static int plan_dgemm(ozb_plan *p, const double *A, long long lda, const double *B, long long ldb, double *C, long long ldc,
                      cudaStream_t st) {
    cudaEvent_t *ev = p->slots ? p->ev + EV_PER_SLOT * (p->calls % p->slots) : nullptr;
    const bool multi = p->panels > 1;
    cudaStream_t s1 = multi ? p->s1 : st, s2 = multi ? p->s2 : st;
    p->last = st;
    if (ev) cudaEventRecord(ev[0], st);
    if (multi) { cudaEventRecord(p->evFork, st); cudaStreamWaitEvent(s1, p->evFork, 0); }
    cudaError_t e = scale_residues_rows(p->nm, A, p->M, p->K, lda, p->bits, p->sa, p->Ar, p->Kp, p->planeA, st);
    if (ev && !multi) cudaEventRecord(ev[EV_ROWS], st);
    if (!multi && !e) {   // one panel: the two passes over B as separate calls, with a timing mark between them
        e = cudaMemsetAsync(p->colmax, 0, (size_t)p->N * 8, st);
        if (!e) e = cols_absmax_accumulate(B, p->K, p->N, ldb, p->colmax, st);
        if (ev) cudaEventRecord(ev[EV_ABSMAX], st);
        if (!e) e = cols_residues_from_max(p->nm, B, p->K, p->N, ldb, p->bits, p->colmax, p->sb, p->Br, p->Kp, p->planeB, st);
    }
    for (int q = 0; multi && q < p->panels && !e; q++) {   // B: maxima + residues of every panel, queued on s1 ahead of the GEMMs
        const int j0 = q * p->panel_width, n = (p->N - j0 < p->panel_width) ? p->N - j0 : p->panel_width;
        e = scale_residues_cols(p->nm, B + j0, p->K, n, ldb, p->bits, p->colmax + j0, p->sb + j0, p->Br + (size_t)j0 * p->Kp, p->Kp,
                                p->planeB, s1);
        if (!e) e = cudaEventRecord(p->evB[q], s1);
    }
    for (int q = 0; q < p->panels && !e; q++) {
        const int j0 = q * p->panel_width, n = (p->N - j0 < p->panel_width) ? p->N - j0 : p->panel_width;
        if (multi) cudaStreamWaitEvent(st, p->evB[q], 0);
        if (ev) cudaEventRecord(ev[2 + 2 * q], st);
        e = gemm_chunks(p, p->Br + (size_t)j0 * p->Kp, p->Cr + j0, n, st);
        if (ev) cudaEventRecord(ev[3 + 2 * q], st);
        if (e) break;
        if (multi) { cudaEventRecord(p->evG[q], st); cudaStreamWaitEvent(s2, p->evG[q], 0); }
        e = crt_from_i8(p->nm, p->Cr + j0, p->planeC, p->M, n, p->Np, p->sa, p->sb + j0, C + j0, ldc, s2);
    }
    if (multi) { cudaEventRecord(p->evJoin, s2); cudaStreamWaitEvent(st, p->evJoin, 0); }
    if (e) return (int)e;
    if (ev) {
        cudaEventRecord(ev[1], st);
        const int slot = p->calls % p->slots;
        p->calls++;
        if (p->calls >= 0x40000000) p->calls = p->slots;   // keep the counter bounded; every slot stays readable
        if (p->env_prof) {   // src/ozaki2.cuh:147-152: one line per product on stderr (this synchronises, like the reference)
            float ms[4];
            if (!plan_phase_ms(p, slot, ms))
                fprintf(stderr, "oz%d %dx%dx%d: scale+residues %.3f  INT8 GEMMs %.3f (%.0f TOPS)  CRT %.3f ms  (total %.3f, %d panels)\n",
                        p->nm, p->M, p->N, p->K, ms[0], ms[1], 2.0 * p->nm * p->M * (double)p->N * p->K / (ms[1] * 1e9), ms[2], ms[3],
                        p->panels);
        }
    }
    return 0;
}
// src/ozaki_dd.cuh:145-155 (ddgemm_t): scales from the hi parts, residues of hi + lo, the same INT8 GEMMs, direct-sum CRT.
// lda, ldb, ldo in elements; mode 0: C = AB, 1: C -= AB, 2: C = -AB.
static int plan_ddgemm(ozb_plan *p, const double *Ah, const double *Al, long long lda, const double *Bh, const double *Bl, long long ldb,
                       double *Ch, double *Cl, long long ldo, int mode, cudaStream_t st) {
    p->last = st;
    cudaError_t e = dd_scale_residues_rows(p->nm, Ah, Al, p->M, p->K, lda, p->bits, p->sa, p->Ar, p->Kp, p->planeA, st);
    if (!e) e = dd_scale_residues_cols(p->nm, Bh, Bl, p->K, p->N, ldb, p->bits, p->colmax, p->sb, p->Br, p->Kp, p->planeB, st);
    if (!e) e = gemm_chunks(p, p->Br, p->Cr, p->N, st);
    if (!e) e = dd_crt_from_i8(p->nm, p->Cr, p->planeC, p->M, p->N, p->Np, p->sa, p->sb, Ch, Cl, ldo, mode, st);
    return (int)e;
}

// device copies of host operands, kept with the plan: all three or none
static cudaError_t host_buffers(ozb_plan *p) {
    if (p->hA && p->hB && p->hC) return cudaSuccess;
    const size_t M = p->M, N = p->N, K = p->K;
    cudaFree(p->hA); cudaFree(p->hB); cudaFree(p->hC);
    p->hA = p->hB = p->hC = nullptr;
    cudaError_t e = cudaMalloc(&p->hA, M * K * 8);
    if (!e) e = cudaMalloc(&p->hB, K * N * 8);
    if (!e) e = cudaMalloc(&p->hC, M * N * 8);
    if (e) { cudaFree(p->hA); cudaFree(p->hB); cudaFree(p->hC); p->hA = p->hB = p->hC = nullptr; cudaGetLastError(); }
    return e;
}

// Host operands (python/capi.cu:37-48,82-88 stage everything, compute, copy back). Here the three phases overlap and every
// copy is contiguous: B goes first, in chunks of rows whose column maxima are taken as they land; once B is complete its
// residues are formed, and A follows in blocks of rows. A block of rows of C needs only its rows of A (row scales are
// local), so each block is scaled, multiplied and reconstructed as soon as it has landed, and its rows of C travel back
// while the next block is in flight. With pinned host memory the copies are asynchronous and the whole product hides
// behind the transfers; with pageable memory the calls below block in issue order and the result is the same.
// The device copies stay with the plan (freed by ozb_release).
static int plan_dgemm_host(ozb_plan *p, const double *A, const double *B, double *C) {
    const size_t M = p->M, N = p->N, K = p->K;
    cudaError_t e = cudaSuccess;
    if ((e = host_buffers(p))) return (int)e;
    if (!p->host_streams) {   // all or nothing: a partial set-up is torn down, so the next call starts from scratch
        e = cudaStreamCreateWithFlags(&p->sIn, cudaStreamNonBlocking);
        if (!e) e = cudaStreamCreateWithFlags(&p->sRun, cudaStreamNonBlocking);
        if (!e) e = cudaStreamCreateWithFlags(&p->sOut, cudaStreamNonBlocking);
        for (auto &ev : p->evIn) if (!e) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        for (auto &ev : p->evRun) if (!e) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e) {
            if (p->sIn) cudaStreamDestroy(p->sIn);
            if (p->sRun) cudaStreamDestroy(p->sRun);
            if (p->sOut) cudaStreamDestroy(p->sOut);
            p->sIn = p->sRun = p->sOut = nullptr;
            for (auto &ev : p->evIn) if (ev) { cudaEventDestroy(ev); ev = nullptr; }
            for (auto &ev : p->evRun) if (ev) { cudaEventDestroy(ev); ev = nullptr; }
            cudaGetLastError();
            return (int)e;
        }
        p->host_streams = true;
    }
    static const int want = [] { const char *env = getenv("OZ_HOST_PANELS"); return env && *env ? atoi(env) : 0; }();
    auto pieces = [&](size_t extent) {   // about 512 rows per piece, at most 16 (measured on B200: 16 beats 8 and 4 at n = 8192)
        int n = want > 0 ? want : (int)(extent / 512);
        if (n > 16) n = 16;
        if (n > HOST_PANELS) n = HOST_PANELS;
        return n < 1 ? 1 : n;
    };
    const int blocks = pieces(M) > pieces(K) ? pieces(M) : pieces(K);
    const int kchunk = (int)((K + pieces(K) - 1) / pieces(K)), mblock = (int)((M + pieces(M) - 1) / pieces(M));
    p->last = p->sRun;
    e = cudaMemsetAsync(p->colmax, 0, N * 8, p->sRun);
    for (int q = 0; q < blocks && !e; q++) {   // B, chunk of rows by chunk
        const size_t k0 = (size_t)q * kchunk;
        if (k0 >= K) break;
        const int rows = (int)(K - k0 < (size_t)kchunk ? K - k0 : kchunk);
        e = cudaMemcpyAsync(p->hB + k0 * N, B + k0 * N, (size_t)rows * N * 8, cudaMemcpyHostToDevice, p->sIn);
        if (!e) e = cudaEventRecord(p->evIn[q], p->sIn);
        if (!e) e = cudaStreamWaitEvent(p->sRun, p->evIn[q], 0);
        if (!e) e = cols_absmax_accumulate(p->hB + k0 * N, rows, (int)N, (long long)N, p->colmax, p->sRun);
    }
    if (!e) e = cols_residues_from_max(p->nm, p->hB, (int)K, (int)N, (long long)N, p->bits, p->colmax, p->sb, p->Br, p->Kp, p->planeB, p->sRun);
    // A, block of rows by block; C goes back block by block. What remains after the last block has landed (its residues,
    // GEMMs, reconstruction and the copy of its rows of C) is exposed, so the last blocks are small: the final mblock rows
    // go as halves of halves down to 128 rows.
    size_t i0 = 0;
    for (int q = 0; i0 < M && !e; q++) {
        const size_t left = M - i0;
        size_t m_ = left > (size_t)mblock ? (size_t)mblock : (left > 128 ? (left / 2 + 127) / 128 * 128 : left);
        if (q >= HOST_PANELS - 1 || m_ > left) m_ = left;   // the event arrays are finite
        const int m = (int)m_;
        e = cudaMemcpyAsync(p->hA + i0 * K, A + i0 * K, (size_t)m * K * 8, cudaMemcpyHostToDevice, p->sIn);
        if (!e) e = cudaEventRecord(p->evIn[q], p->sIn);
        if (!e) e = cudaStreamWaitEvent(p->sRun, p->evIn[q], 0);
        if (!e) e = scale_residues_rows(p->nm, p->hA + i0 * K, m, (int)K, (long long)K, p->bits, p->sa + i0, p->Ar + i0 * p->Kp, p->Kp, p->planeA, p->sRun);
        if (!e) e = gemm_chunks(p, p->Br, p->Cr, (int)N, p->sRun, (int)i0, m);
        if (!e) e = crt_from_i8(p->nm, p->Cr + i0 * p->Np, p->planeC, m, (int)N, p->Np, p->sa + i0, p->sb, p->hC + i0 * N, (long long)N, p->sRun);
        if (!e) e = cudaEventRecord(p->evRun[q], p->sRun);
        if (!e) e = cudaStreamWaitEvent(p->sOut, p->evRun[q], 0);
        if (!e) e = cudaMemcpyAsync(C + i0 * N, p->hC + i0 * N, (size_t)m * N * 8, cudaMemcpyDeviceToHost, p->sOut);
        i0 += m_;
    }
    if (!e) e = cudaStreamSynchronize(p->sOut);
    cudaError_t e2 = cudaStreamSynchronize(p->sRun), e3 = cudaStreamSynchronize(p->sIn);
    if (e) return (int)e;
    if (e2) return (int)e2;
    return (int)e3;
}

// status words: [0] the first wait code of a launch that gave up (0 = none), [1..63] per-CTA codes for diagnostics
static int read_status(int *dev_words) {
    int h[64] = {};
    if (cudaError_t e = cudaMemcpy(h, dev_words, sizeof h, cudaMemcpyDeviceToHost)) return (int)e;
    if (getenv("OZ_DEBUG") && (h[8] | h[9] | h[10] | h[11]))   // timing build of the pair kernel: (wait, total) in 1024-cycle units
        fprintf(stderr, "ozb: cta0 producer %d/%d issuer %d/%d | cta1 producer %d/%d issuer %d/%d\n", h[8], h[9], h[10], h[11], h[12], h[13],
                h[14], h[15]);
    if (!h[0]) return 0;
    cudaMemset(dev_words, 0, sizeof h);
    if (getenv("OZ_DEBUG")) {
        fprintf(stderr, "ozb: a wait expired, first code 0x%x; per CTA:", h[0]);
        for (int i = 1; i < 64; i++) if (h[i]) fprintf(stderr, " [%d]=0x%x", i - 1, h[i]);
        fprintf(stderr, "\n");
    }
    return OZB_ETIMEOUT;
}
static int plan_status(ozb_plan *p) {
    cudaError_t e = cudaStreamSynchronize(p->last);
    if (e) return (int)e;
    return read_status(p->status);
}

// ---------------------------------------------------------------------------------------------------------------
// the reference's ABI
// ---------------------------------------------------------------------------------------------------------------
namespace {
std::mutex mu;
struct Cache { ozb_plan *p = nullptr; };
Cache cache[3];   // 0 FP64, 1 double-double, 2 triple-double (python/capi.cu:21)
int *stage_status[64] = {};   // one status word per device for the stage calls

int check_args(int M, int N, int K) {   // python/capi.cu:23-29
    if (M <= 0 || N <= 0 || K <= 0) return OZB_EARG;
    if (K >= 131072) return OZB_EK;
    int dev, major;
    if (cudaGetDevice(&dev) || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) return (int)cudaGetLastError();
    return major != 10 ? OZB_EARCH : 0;   // tcgen05 / tensor memory: this binary holds sm_100a code only
}
int plan_for(int which, int M, int N, int K, int nm, int maxbits, ozb_plan **out) {   // python/capi.cu:30-35
    Cache &c = cache[which];
    int dev = -1;
    cudaGetDevice(&dev);   // a cached plan is only good on the device it was made on
    if (c.p && (c.p->M != M || c.p->N != N || c.p->K != K || c.p->nm != nm || c.p->maxbits != maxbits || c.p->dev != dev)) { plan_free(c.p); c.p = nullptr; }
    if (!c.p) if (int e = plan_make(M, N, K, nm, maxbits, &c.p)) { c.p = nullptr; return e; }
    *out = c.p;
    return 0;
}
// The asynchronous entry points that use a cached plan share its workspaces: a product queued on one stream must not
// start before the previous one, possibly queued on another stream, has finished with them.
template <class F> int ordered_on_cached_plan(ozb_plan *p, cudaStream_t st, F &&enqueue) {
    if (cudaError_t e = cudaStreamWaitEvent(st, p->evDone, 0)) return (int)e;
    if (int e = enqueue()) return e;
    return (int)cudaEventRecord(p->evDone, st);
}
int finish() { const int e = (int)cudaDeviceSynchronize(); return e ? e : (int)cudaGetLastError(); }   // python/capi.cu:49
int *status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) || dev < 0 || dev >= 64) return nullptr;
    if (!stage_status[dev]) {
        if (cudaMalloc(&stage_status[dev], 256) || cudaMemset(stage_status[dev], 0, 256)) { cudaGetLastError(); stage_status[dev] = nullptr; }
    }
    return stage_status[dev];
}
}  // namespace

OZB_API const char *ozb_version(void) { return OZB_VERSION; }

OZB_API const char *ozb_error(int e) {
    switch (e) {
    case 0: return "ok";
    case OZB_EARG: return "M, N and K must be positive";
    case OZB_EK: return "K must be below 131072 (the int32 accumulators of the INT8 GEMMs)";
    case OZB_EARCH: return "this build runs on compute capability 10.x GPUs (B200, sm_100a: tcgen05 tensor cores) only";
    case OZB_ETIMEOUT: return "a bounded wait inside the INT8 GEMM kernel expired; the result is not valid";
    case OZB_ENOTBUILT: return "this entry point is exported for ABI compatibility but not built in this library";
    case OZB_ESIZE: return "a size exceeds the fixed limit of this entry point";
    case OZB_ECOMM: return "the exchange between GPUs failed or did not finish in time; the communicator was aborted";
    case OZB_ENCCL: return "the NCCL library (libnccl.so.2) could not be loaded";
    default: return cudaGetErrorString((cudaError_t)e);
    }
}

OZB_API int ozb_device(char *name, int len, int *sm, int *l2_kib, int *sms) {
    int dev; cudaDeviceProp p;
    if (int e = cudaGetDevice(&dev)) return e;
    if (int e = cudaGetDeviceProperties(&p, dev)) return e;
    if (name && len > 0) { strncpy(name, p.name, len - 1); name[len - 1] = 0; }
    if (sm) *sm = 10 * p.major + p.minor;
    if (l2_kib) *l2_kib = p.l2CacheSize >> 10;
    if (sms) *sms = p.multiProcessorCount;
    return 0;
}

OZB_API int ozb_dgemm(int M, int N, int K, const double *A, const double *B, double *C, int moduli, int on_host) {
    if (int e = check_args(M, N, K)) return e;
    if (moduli < 8 || moduli > 16) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    ozb_plan *p;
    if (int e = plan_for(0, M, N, K, moduli, 62, &p)) return e;
    if (!on_host) {
        if (int e = plan_dgemm(p, A, K, B, N, C, N, 0)) return e;
        if (int e = finish()) return e;
        return plan_status(p);
    }
    // Pinned (page-locked) host memory takes the overlapped path. Pageable memory cannot be copied asynchronously -- every
    // piece would be staged by the driver in issue order -- so it is moved with three plain copies, as the reference does
    // (python/capi.cu:37-48); OZ_HOST_PIPELINE=1 / 0 forces one or the other.
    static const int force = [] { const char *env = getenv("OZ_HOST_PIPELINE"); return env && *env ? atoi(env) : -1; }();
    bool pinned = false;
    {
        cudaPointerAttributes pa, pb, pc;
        if (!cudaPointerGetAttributes(&pa, A) && !cudaPointerGetAttributes(&pb, B) && !cudaPointerGetAttributes(&pc, C))
            pinned = pa.type == cudaMemoryTypeHost && pb.type == cudaMemoryTypeHost && pc.type == cudaMemoryTypeHost;
        cudaGetLastError();
    }
    if (force == 1 || (force != 0 && pinned)) {
        if (int e = plan_dgemm_host(p, A, B, C)) return e;
        if (int e = finish()) return e;
        return plan_status(p);
    }
    const size_t la = (size_t)M * K * 8, lb = (size_t)K * N * 8, lc = (size_t)M * N * 8;
    int e = (int)host_buffers(p);
    if (e) return e;
    e = (int)cudaMemcpy(p->hA, A, la, cudaMemcpyHostToDevice);
    if (!e) e = (int)cudaMemcpy(p->hB, B, lb, cudaMemcpyHostToDevice);
    if (!e) e = plan_dgemm(p, p->hA, K, p->hB, N, p->hC, N, 0);
    if (!e) e = finish();
    if (!e) e = plan_status(p);
    if (!e) e = (int)cudaMemcpy(C, p->hC, lc, cudaMemcpyDeviceToHost);
    return e;
}

OZB_API int ozb_ddgemm(int M, int N, int K, const double *Ah, const double *Al, const double *Bh, const double *Bl, double *Ch,
                       double *Cl, int on_host) {   // python/capi.cu:92-105
    if (int e = check_args(M, N, K)) return e;
    std::lock_guard<std::mutex> g(mu);
    ozb_plan *p;
    if (int e = plan_for(1, M, N, K, 32, 106, &p)) return e;
    if (!on_host) {
        if (int e = plan_ddgemm(p, Ah, Al, K, Bh, Bl, N, Ch, Cl, N, 0, 0)) return e;
        if (int e = finish()) return e;
        return plan_status(p);
    }
    // host operands: staged through device buffers (python/capi.cu:37-48,98-104)
    const double *in[4] = {Ah, Al, Bh, Bl};
    const size_t len[4] = {(size_t)M * K, (size_t)M * K, (size_t)K * N, (size_t)K * N}, lo = (size_t)M * N;
    double *d[6] = {};
    int e = 0;
    for (int i = 0; i < 6 && !e; i++) e = (int)cudaMalloc(&d[i], (i < 4 ? len[i] : lo) * 8);
    for (int i = 0; i < 4 && !e; i++) e = (int)cudaMemcpy(d[i], in[i], len[i] * 8, cudaMemcpyHostToDevice);
    if (!e) e = plan_ddgemm(p, d[0], d[1], K, d[2], d[3], N, d[4], d[5], N, 0, 0);
    if (!e) e = finish();
    if (!e) e = plan_status(p);
    if (!e) e = (int)cudaMemcpy(Ch, d[4], lo * 8, cudaMemcpyDeviceToHost);
    if (!e) e = (int)cudaMemcpy(Cl, d[5], lo * 8, cudaMemcpyDeviceToHost);
    for (double *x : d) if (x) cudaFree(x);
    return e;
}

// src/ozaki_dd.cuh:143-148 -- the double-double product with leading dimensions, a mode and a stream, on device pointers,
// without the final synchronisation. moduli in {24, 28, 32}; mode 0: C = AB, 1: C -= AB, 2: C = -AB.
OZB_API int ozb_ddgemm_ex(int M, int N, int K, const double *Ah, const double *Al, long long lda, const double *Bh, const double *Bl,
                          long long ldb, double *Ch, double *Cl, long long ldo, int moduli, int mode, void *stream) {
    if (int e = check_args(M, N, K)) return e;
    if ((moduli != 24 && moduli != 28 && moduli != 32) || mode < 0 || mode > 2 || !Ah || !Al || !Bh || !Bl || !Ch || !Cl || lda < K ||
        ldb < N || ldo < N)
        return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    ozb_plan *p;
    if (int e = plan_for(1, M, N, K, moduli, 106, &p)) return e;
    return ordered_on_cached_plan(p, (cudaStream_t)stream, [&] { return plan_ddgemm(p, Ah, Al, lda, Bh, Bl, ldb, Ch, Cl, ldo, mode, (cudaStream_t)stream); });
}

OZB_API int ozb_tdgemm(int M, int N, int K, const double *, const double *, const double *, const double *, const double *,
                       const double *, double *, double *, double *, int) {
    if (int e = check_args(M, N, K)) return e;
    return OZB_ENOTBUILT;
}

OZB_API void ozb_release(void) {
    std::lock_guard<std::mutex> g(mu);
    for (Cache &c : cache) if (c.p) { plan_free(c.p); c.p = nullptr; }
    exact_f8_release();
    ozb_mg_release();   // the communicators and workspaces ozb_dgemm_mg keeps between calls
}

static int bench_dd(int n, int reps, double *median_ms) {   // python/capi.cu:130-164, kind 1: lower parts 2^-53 below
    const size_t len = (size_t)n * n;
    double *d[6] = {};   // Ah, Al, Ch, Cl, Bh, Bl
    int err = 0;
    for (int i = 0; i < 6 && !err; i++) err = (int)cudaMalloc(&d[i], len * sizeof(double));
    if (!err) {
        double *h = (double *)malloc(len * sizeof(double));
        if (!h) err = (int)cudaErrorMemoryAllocation;
        for (int i = 0; i < 4 && !err; i++) {
            const double sc = i % 2 == 0 ? 1.0 : 0x1p-53;
            uint64_t x = 0x9E3779B97F4A7C15ull * (i + 1);
            for (size_t j = 0; j < len; j++) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; h[j] = sc * ((double)(x >> 11) * 0x1p-52 - 1.0); }
            err = (int)cudaMemcpy(d[i < 2 ? i : 2 + i], h, len * sizeof(double), cudaMemcpyHostToDevice);
        }
        free(h);
    }
    float t[101]; int nt = 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (!err) { cudaEventCreate(&e0); cudaEventCreate(&e1); }
    for (int r = -1; r < reps && !err; r++) {
        cudaEventRecord(e0);
        err = ozb_ddgemm(n, n, n, d[0], d[1], d[4], d[5], d[2], d[3], 0);
        cudaEventRecord(e1); cudaEventSynchronize(e1);
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        if (r >= 0) t[nt++] = ms;
    }
    if (nt) {
        for (int i = 1; i < nt; i++) for (int j = i; j > 0 && t[j - 1] > t[j]; j--) { const float x = t[j]; t[j] = t[j - 1]; t[j - 1] = x; }
        *median_ms = t[nt / 2];
    }
    if (e0) { cudaEventDestroy(e0); cudaEventDestroy(e1); }
    for (double *p : d) if (p) cudaFree(p);
    return err;
}

OZB_API int ozb_bench(int n, int kind, int reps, double *median_ms) {   // python/capi.cu:130-164
    if (int e = check_args(n, n, n)) return e;
    if (kind < 0 || kind > 2 || reps < 1 || reps > 101 || !median_ms) return OZB_EARG;
    if (kind == 2) return OZB_ENOTBUILT;
    if (kind == 1) return bench_dd(n, reps, median_ms);
    const size_t len = (size_t)n * n;
    double *d[3] = {};
    int err = 0;
    for (int i = 0; i < 3 && !err; i++) err = (int)cudaMalloc(&d[i], len * sizeof(double));
    if (!err) {   // values in [-1, 1) from the fixed xorshift hash of the reference (python/capi.cu:140-145)
        double *h = (double *)malloc(len * sizeof(double));
        if (!h) err = (int)cudaErrorMemoryAllocation;
        for (int i = 0; i < 2 && !err; i++) {
            uint64_t x = 0x9E3779B97F4A7C15ull * (i + 1);
            for (size_t j = 0; j < len; j++) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; h[j] = (double)(x >> 11) * 0x1p-52 - 1.0; }
            err = (int)cudaMemcpy(d[i == 0 ? 0 : 2], h, len * sizeof(double), cudaMemcpyHostToDevice);
        }
        free(h);
    }
    float t[101]; int nt = 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (!err) { cudaEventCreate(&e0); cudaEventCreate(&e1); }
    for (int r = -1; r < reps && !err; r++) {   // r = -1: warm-up (plan, first launches)
        cudaEventRecord(e0);
        err = ozb_dgemm(n, n, n, d[0], d[2], d[1], 16, 0);
        cudaEventRecord(e1); cudaEventSynchronize(e1);
        float ms; cudaEventElapsedTime(&ms, e0, e1);
        if (r >= 0) t[nt++] = ms;
    }
    if (nt) {
        for (int i = 1; i < nt; i++) for (int j = i; j > 0 && t[j - 1] > t[j]; j--) { const float x = t[j]; t[j] = t[j - 1]; t[j - 1] = x; }
        *median_ms = t[nt / 2];
    }
    if (e0) { cudaEventDestroy(e0); cudaEventDestroy(e1); }
    for (double *p : d) if (p) cudaFree(p);
    return err;
}

// ---------------------------------------------------------------------------------------------------------------
// additions
// ---------------------------------------------------------------------------------------------------------------
OZB_API int ozb_bits_for(int nm, int K, int maxbits) { return (nm < 1 || nm > MAXM || K <= 0) ? -1 : bits_for_impl(nm, K, maxbits); }
OZB_API int ozb_modulus(int l) { return (l >= 0 && l < MAXM) ? modulus(l) : 0; }

OZB_API int ozb_plan_create(int M, int N, int K, int moduli, int maxbits, ozb_plan **out) {
    if (!out) return OZB_EARG;
    if (int e = check_args(M, N, K)) return e;
    if (moduli < 8 || moduli > 16) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    return plan_make(M, N, K, moduli, maxbits, out);
}
OZB_API void ozb_plan_destroy(ozb_plan *p) {
    std::lock_guard<std::mutex> g(mu);
    plan_free(p);
}
OZB_API int ozb_plan_dgemm(ozb_plan *p, const double *A, long long lda, const double *B, long long ldb, double *C, long long ldc,
                           void *stream) {
    if (!p || !A || !B || !C || lda < p->K || ldb < p->N || ldc < p->N) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    return plan_dgemm(p, A, lda, B, ldb, C, ldc, (cudaStream_t)stream);
}
OZB_API int ozb_plan_set_a(ozb_plan *p, const double *A, long long lda, void *stream) {
    if (!p || !A || lda < p->K) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    return plan_set_a(p, A, lda, (cudaStream_t)stream);
}
OZB_API int ozb_plan_panel(ozb_plan *p, const double *B, long long ldb, double *C, long long ldc, int j0, int ncols, void *stream) {
    if (!p || !B || !C || j0 < 0 || (j0 & 255) || ncols <= 0 || j0 + ncols > p->N || ldb < ncols || ldc < ncols) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    return plan_panel(p, B, ldb, C, ldc, j0, ncols, (cudaStream_t)stream, nullptr);
}
// B in chunks of rows (as it arrives from a broadcast or from the host), then the product with the prepared operands
OZB_API int ozb_plan_b_begin(ozb_plan *p, void *stream) {
    if (!p) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    p->last = (cudaStream_t)stream;
    return (int)cudaMemsetAsync(p->colmax, 0, (size_t)p->N * 8, (cudaStream_t)stream);
}
OZB_API int ozb_plan_b_rows(ozb_plan *p, const double *Brows, long long ldb, int rows, void *stream) {
    if (!p || !Brows || rows <= 0 || rows > p->K || ldb < p->N) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    return (int)cols_absmax_accumulate(Brows, rows, p->N, ldb, p->colmax, (cudaStream_t)stream);
}
OZB_API int ozb_plan_b_finish(ozb_plan *p, const double *B, long long ldb, void *stream) {
    if (!p || !B || ldb < p->N) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    return (int)cols_residues_from_max(p->nm, B, p->K, p->N, ldb, p->bits, p->colmax, p->sb, p->Br, p->Kp, p->planeB, (cudaStream_t)stream);
}
// rows [k0, k0 + rows) of B with column maxima the caller holds (computed where the whole of B is, e.g. on another GPU)
OZB_API int ozb_plan_b_rows_residues(ozb_plan *p, const double *Brows, long long ldb, int k0, int rows, const void *colmax, void *stream) {
    if (!p || !Brows || !colmax || rows <= 0 || k0 < 0 || (k0 & 127) || k0 + rows > p->K || ldb < p->N) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    p->last = (cudaStream_t)stream;
    return (int)cols_residues_from_max(p->nm, Brows, rows, p->N, ldb, p->bits, (const unsigned long long *)colmax, p->sb, p->Br + k0, p->Kp,
                                       p->planeB, (cudaStream_t)stream);
}
OZB_API int ozb_cols_absmax(const double *X, int rows, int cols, long long ldx, void *colmax, void *stream) {
    if (int e = check_args(rows, cols, 1)) return e;
    if (!X || !colmax || ldx < cols) return OZB_EARG;
    return (int)cols_absmax_accumulate(X, rows, cols, ldx, (unsigned long long *)colmax, (cudaStream_t)stream);
}
OZB_API int ozb_plan_multiply(ozb_plan *p, double *C, long long ldc, void *stream) {
    if (!p || !C || ldc < p->N) return OZB_EARG;
    if (!on_plan_device(p)) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    cudaStream_t st = (cudaStream_t)stream;
    p->last = st;
    cudaError_t e = gemm_chunks(p, p->Br, p->Cr, p->N, st);
    if (!e) e = crt_from_i8(p->nm, p->Cr, p->planeC, p->M, p->N, p->Np, p->sa, p->sb, C, ldc, st);
    return (int)e;
}
OZB_API int ozb_plan_view(ozb_plan *p, int *bits, int *Kp, int *Np, int8_t **Ar, int8_t **Br, int8_t **Cr, int **sa, int **sb) {
    if (!p) return OZB_EARG;
    if (bits) *bits = p->bits;
    if (Kp) *Kp = p->Kp;
    if (Np) *Np = p->Np;
    if (Ar) *Ar = p->Ar;
    if (Br) *Br = p->Br;
    if (Cr) *Cr = p->Cr;
    if (sa) *sa = p->sa;
    if (sb) *sb = p->sb;
    return 0;
}
OZB_API int ozb_plan_status(ozb_plan *p) {
    if (!p) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    return plan_status(p);
}
OZB_API int ozb_plan_profile(ozb_plan *p, int slots) {
    if (!p || slots < 0 || slots > 4096) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    return plan_profile(p, slots);
}
OZB_API int ozb_plan_phase_ms(ozb_plan *p, int slot, float ms[4]) {
    if (!p || !ms) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    return plan_phase_ms(p, slot, ms);
}
OZB_API int ozb_plan_kernel_ms(ozb_plan *p, int slot, float ms[5]) {
    if (!p || !ms) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    return plan_kernel_ms(p, slot, ms);
}

OZB_API int ozb_dgemm_ex(int M, int N, int K, const double *A, long long lda, const double *B, long long ldb, double *C,
                         long long ldc, int moduli, void *stream) {
    if (int e = check_args(M, N, K)) return e;
    if (moduli < 8 || moduli > 16 || !A || !B || !C || lda < K || ldb < N || ldc < N) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    ozb_plan *p;
    if (int e = plan_for(0, M, N, K, moduli, 62, &p)) return e;
    return ordered_on_cached_plan(p, (cudaStream_t)stream, [&] { return plan_dgemm(p, A, lda, B, ldb, C, ldc, (cudaStream_t)stream); });
}

// bench/oz_strassen.cu:74-97,247 -- the product with the reference's optional 2-norm scales: beta = floor((log2 P - 1.001) / 2)
OZB_API int ozb_dgemm_norm(int M, int N, int K, const double *A, long long lda, const double *B, long long ldb, double *C, long long ldc,
                           int moduli, void *stream) {
    if (int e = check_args(M, N, K)) return e;
    if (moduli < 8 || moduli > 16 || !A || !B || !C || lda < K || ldb < N || ldc < N) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    ozb_plan *p;
    if (int e = plan_for(0, M, N, K, moduli, 62, &p)) return e;
    double l2 = 0;
    for (int l = 0; l < moduli; l++) l2 += log2((double)modulus(l));
    int beta = (int)floor((l2 - 1.001) / 2);
    if (beta > 62) beta = 62;
    cudaStream_t st = (cudaStream_t)stream;
    p->last = st;
    return ordered_on_cached_plan(p, st, [&] {
        cudaError_t e = norm_scale_residues_rows(p->nm, A, M, K, lda, beta, p->sa, p->Ar, p->Kp, p->planeA, st);
        if (!e) e = norm_scale_residues_cols(p->nm, B, K, N, ldb, beta, p->sb, p->Br, p->Kp, p->planeB, st);
        if (!e) e = gemm_chunks(p, p->Br, p->Cr, N, st);
        if (!e) e = crt_from_i8(p->nm, p->Cr, p->planeC, M, N, p->Np, p->sa, p->sb, C, ldc, st);
        return (int)e;
    });
}
OZB_API int ozb_scales_norm(const double *X, int nvec, int len, long long ldx, int by_rows, int moduli, int *s, void *stream) {
    if (int e = check_args(nvec, 1, len)) return e;
    if (moduli < 8 || moduli > 16 || !X || !s || ldx < (by_rows ? len : nvec)) return OZB_EARG;
    double l2 = 0;
    for (int l = 0; l < moduli; l++) l2 += log2((double)modulus(l));
    int beta = (int)floor((l2 - 1.001) / 2);
    if (beta > 62) beta = 62;
    return (int)scales_norm_only(X, nvec, len, ldx, by_rows ? 1 : 0, beta, s, (cudaStream_t)stream);
}
OZB_API int ozb_scale_residues_rows(int moduli, const double *X, int rows, int len, long long ldx, int bits, int *s, int8_t *R,
                                    int ld, size_t plane, void *stream) {
    if (int e = check_args(rows, 1, len)) return e;
    if (moduli < 8 || moduli > 16 || !X || !s || !R || ldx < len || ld < round_up(len, 4) || (ld & 3) || (plane & 3)) return OZB_EARG;
    return (int)scale_residues_rows(moduli, X, rows, len, ldx, bits, s, R, ld, plane, (cudaStream_t)stream);
}
OZB_API int ozb_scale_residues_cols(int moduli, const double *X, int rows, int cols, long long ldx, int bits, void *colmax, int *s,
                                    int8_t *R, int ld, size_t plane, void *stream) {
    if (int e = check_args(1, cols, rows)) return e;
    if (moduli < 8 || moduli > 16 || !X || !s || !R || !colmax || ldx < cols || ld < round_up(rows, 16) || (ld & 15) || (plane & 15) ||
        (reinterpret_cast<uintptr_t>(R) & 15))
        return OZB_EARG;
    return (int)scale_residues_cols(moduli, X, rows, cols, ldx, bits, (unsigned long long *)colmax, s, R, ld, plane, (cudaStream_t)stream);
}
OZB_API int ozb_gemm_i8(const int8_t *A, const int8_t *Bt, int32_t *C, int M, int N, int K, int Z, long long lda, long long ldb,
                        long long ldc, size_t plane_a, size_t plane_b, size_t plane_c, void *stream) {
    if (int e = check_args(M, N, K)) return e;
    if (!A || !Bt || !C || Z <= 0 || lda < K || ldb < K || ldc < N) return OZB_EARG;
    int *st = status_word();
    if (!st) return (int)cudaErrorMemoryAllocation;
    return (int)gemm_i8_planes(A, Bt, C, M, N, K, Z, lda, ldb, ldc, plane_a, plane_b, plane_c, 0, 0, st, 0, (cudaStream_t)stream);
}
OZB_API int ozb_gemm_i8_mod(const int8_t *A, const int8_t *Bt, int8_t *C, int M, int N, int K, int Z, long long lda, long long ldb,
                            long long ldc, size_t plane_a, size_t plane_b, size_t plane_c, int first_modulus, void *stream) {
    if (int e = check_args(M, N, K)) return e;
    if (!A || !Bt || !C || Z <= 0 || lda < K || ldb < K || ldc < round_up(N, 16) || (plane_c & 15) ||
        (reinterpret_cast<uintptr_t>(C) & 15))
        return OZB_EARG;
    int *st = status_word();
    if (!st) return (int)cudaErrorMemoryAllocation;
    return (int)gemm_i8_planes(A, Bt, C, M, N, K, Z, lda, ldb, ldc, plane_a, plane_b, plane_c, 1, first_modulus, st, 0,
                               (cudaStream_t)stream);
}
OZB_API int ozb_gemm_i8_mod_beside(const int8_t *A, const int8_t *Bt, int8_t *C, int M, int N, int K, int Z, long long lda,
                                   long long ldb, long long ldc, size_t plane_a, size_t plane_b, size_t plane_c, int first_modulus,
                                   int reserve_sms, const int *busy, void *stream) {
    if (int e = check_args(M, N, K)) return e;
    if (!A || !Bt || !C || Z <= 0 || lda < K || ldb < K || ldc < round_up(N, 16) || (plane_c & 15) ||
        (reinterpret_cast<uintptr_t>(C) & 15) || reserve_sms < 0)
        return OZB_EARG;
    int *st = status_word();
    if (!st) return (int)cudaErrorMemoryAllocation;
    return (int)gemm_i8_planes(A, Bt, C, M, N, K, Z, lda, ldb, ldc, plane_a, plane_b, plane_c, 1, first_modulus, st, 0,
                               (cudaStream_t)stream, 0, reserve_sms, busy);
}
OZB_API int ozb_crt_i32(int moduli, const int32_t *Cl, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
                        double *C, long long ldc, void *stream) {
    if (int e = check_args(M, N, 1)) return e;
    if (moduli < 8 || moduli > 16 || !Cl || !sa || !sb || !C || ldr < N || ldc < N) return OZB_EARG;
    return (int)crt_from_i32(moduli, Cl, plane, M, N, ldr, sa, sb, C, ldc, (cudaStream_t)stream);
}
OZB_API int ozb_crt_i8(int moduli, const int8_t *Cr, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
                       double *C, long long ldc, void *stream) {
    if (int e = check_args(M, N, 1)) return e;
    if (moduli < 8 || moduli > 16 || !Cr || !sa || !sb || !C || ldr < round_up(N, 4) || (ldr & 3) || (plane & 3) ||
        (reinterpret_cast<uintptr_t>(Cr) & 3) || ldc < N)
        return OZB_EARG;
    return (int)crt_from_i8(moduli, Cr, plane, M, N, ldr, sa, sb, C, ldc, (cudaStream_t)stream);
}
OZB_API int ozb_bf16_fp8_gemm(int M, int N, int K, const void *X, const void *W, const float *S, float *Y, int *open, int *moduli, void *stream) {
    if (int e = check_args(M, N, K)) return e;
    if (!X || !W || !S || !Y) return OZB_EARG;
    std::lock_guard<std::mutex> g(mu);
    return exact_bf16_fp8_gemm(M, N, K, (const uint16_t *)X, K, (const uint8_t *)W, N, S, Y, N, open, moduli, (cudaStream_t)stream);
}
OZB_API int ozb_int8_peak(int iters, int pair, float *ms, double *tops) {
    if (int e = check_args(1, 1, 1)) return e;
    int *st = status_word();
    if (!st) return (int)cudaErrorMemoryAllocation;
    if (int e = (int)int8_peak_probe(iters, pair, ms, tops, st, 0)) return e == (int)cudaErrorInvalidValue ? OZB_EARG : e;
    return read_status(st);
}
OZB_API int ozb_selftest_wait_expiry(int budget_ms) {
    if (int e = check_args(1, 1, 1)) return e;
    int *st = status_word();
    if (!st) return (int)cudaErrorMemoryAllocation;
    if (int e = (int)wait_expiry_selftest((unsigned)budget_ms, st, 0)) return e == (int)cudaErrorInvalidValue ? OZB_EARG : e;
    if (int e = (int)cudaDeviceSynchronize()) return e;
    return read_status(st);
}
OZB_API int ozb_bounds_report(unsigned long long out[4]) {
#ifdef OZ_BOUNDS
    if (!out) return OZB_EARG;
    if (int e = (int)cudaDeviceSynchronize()) return e;
    std::lock_guard<std::mutex> g(mu);
    unsigned long long v[3][4] = {};
    cudaError_t e = scale_residue_violations(v[0]);
    if (!e) e = crt_violations(v[1]);
    if (!e) e = gemm_violations(v[2]);
    if (e) return (int)e;
    out[0] = out[1] = out[2] = out[3] = 0;
    for (auto &w : v) {
        if (w[0] && !out[0]) { out[1] = w[1]; out[2] = w[2]; out[3] = w[3]; }
        out[0] += w[0];
    }
    return 0;
#else
    (void)out;
    return OZB_ENOTBUILT;
#endif
}
OZB_API int ozb_selftest_bounds(void) {
#ifdef OZ_BOUNDS
    if (int e = check_args(1, 1, 1)) return e;
    int *buf = nullptr;
    if (cudaError_t e = cudaMalloc(&buf, 8 * sizeof(int))) return (int)e;   // eight ints allocated, four registered
    cudaError_t e = cudaMemset(buf, 0xFF, 8 * sizeof(int));
    if (!e) e = bounds_selftest(buf, 0);
    if (!e) e = cudaDeviceSynchronize();
    int h[8] = {};
    if (!e) e = cudaMemcpy(h, buf, sizeof h, cudaMemcpyDeviceToHost);
    cudaFree(buf);
    if (e) return (int)e;
    for (int i = 0; i < 4; i++) if (h[i] != i) return OZB_EARG;            // the stores inside the window happened
    return h[4] == -1 ? 0 : OZB_EARG;                                     // the one outside did not
#else
    return OZB_ENOTBUILT;
#endif
}
OZB_API int ozb_status(void) {
    if (int e = (int)cudaDeviceSynchronize()) return e;
    std::lock_guard<std::mutex> g(mu);
    int *st = status_word();
    if (!st) return (int)cudaErrorMemoryAllocation;
    int r = read_status(st);
    int dev = -1;
    cudaGetDevice(&dev);
    for (Cache &c : cache)   // the cached plans of ozb_dgemm_ex / ozb_dgemm_norm / ozb_ddgemm_ex have status words of their own
        if (c.p && c.p->dev == dev) { const int q = read_status(c.p->status); if (!r) r = q; }
    return r;
}
