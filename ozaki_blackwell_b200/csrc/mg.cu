// mg.cu -- the FP64 product over several GPUs of one machine, behind the C ABI (ozb_mg_*, ozb_dgemm_mg).
//
// The reference is single-GPU (no NCCL, MPI, peer copy or cudaSetDevice anywhere in it); this is the one distributed
// strategy that does not change a bit of the result. Rank g owns a block of rows of A and produces the same rows of C
// (the reference's entry point python/capi.cu:77-89, with a row count per rank). Row scales belong to those rows; column
// scales and residues of B are formed identically on every rank, so the only exchange is one broadcast of B from the rank
// that holds it: ncclBroadcast over NVLink / NVSwitch on a communication stream of the library's own. Nothing else is
// exchanged, no kernel of the library reads another GPU's memory, and B is in the GPU's own HBM before any kernel or TMA
// load touches it.
//
// How B travels depends on how long the transfer is against this rank's share of the product:
//   whole   (B up to 1 GiB, or a short transfer) one transfer straight out of the holder's matrix, beside the residues of A; then the column
//           maxima, the residues of B, the GEMMs and the reconstruction, each once at full width.
//   stream  the holder first reduces the column maxima of its B (one pass at HBM speed) and sends those 8 N bytes ahead;
//           B follows in pieces of whole rows (contiguous, nothing is packed; four to nine pieces). Every rank turns a
//           piece into residues the moment it has landed. A K the single-GPU product runs in one launch then gets its one
//           full-width GEMM launch after the last piece; a longer K gets the INT8 GEMMs of a K range of about 8192 as soon
//           as the pieces of that range are there, adding to the residues of the ranges before it (the same cut of a long
//           K the single-GPU product makes to keep its panels in L2). The reconstruction runs once at the end.
//
//           The pieces travel over a second communicator whose kernels are capped to a few CTAs, and the GEMMs -- persistent
//           grids that give no SM back before they end -- leave that many SMs alone while pieces are still to come: every
//           CTA pair is launched, and the pairs beyond the kept ones read a device word when they start (set before the
//           first piece, cleared behind the last, both on the communication stream) and leave at once if it is set.
//
// NCCL is loaded at run time (dlopen of libnccl.so.2: the library itself links against nothing but the driver), the
// communicators are non-blocking, and every host-side wait is bounded: when a call does not settle or a product does not
// finish within the handle's time budget -- a peer that never joined -- the communicators are aborted (ncclCommAbort, each
// in a thread of its own, bounded too), the handle is marked broken and the call returns OZB_ECOMM; the CUDA context
// stays usable.
#include <nccl.h>
#include <dlfcn.h>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <thread>
#include "../../include/ozb.h"
#include "oz_common.cuh"
#include "oz_kernels.h"
#include "oz_plan.h"

#define OZB_API extern "C" __attribute__((visibility("default")))
using namespace ozk;

namespace {

// ---------------------------------------------------------------------------------------------------------------
// NCCL, loaded on first use
// ---------------------------------------------------------------------------------------------------------------
struct Nccl {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    bool ok = false;
};
const Nccl &nccl() {
    static Nccl n = [] {
        Nccl n;
        // a process that already holds NCCL (a framework's bundled copy) gets that one back: dlopen matches the soname
        const char *env = getenv("OZB_NCCL_LIBRARY");
        n.handle = dlopen(env && *env ? env : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!n.handle) return n;
        auto sym = [&](const char *name) { return dlsym(n.handle, name); };
        n.GetUniqueId = (decltype(n.GetUniqueId))sym("ncclGetUniqueId");
        n.CommInitRankConfig = (decltype(n.CommInitRankConfig))sym("ncclCommInitRankConfig");
        n.CommGetAsyncError = (decltype(n.CommGetAsyncError))sym("ncclCommGetAsyncError");
        n.CommAbort = (decltype(n.CommAbort))sym("ncclCommAbort");
        n.CommDestroy = (decltype(n.CommDestroy))sym("ncclCommDestroy");
        n.Broadcast = (decltype(n.Broadcast))sym("ncclBroadcast");
        n.GroupStart = (decltype(n.GroupStart))sym("ncclGroupStart");
        n.GroupEnd = (decltype(n.GroupEnd))sym("ncclGroupEnd");
        n.ok = n.GetUniqueId && n.CommInitRankConfig && n.CommGetAsyncError && n.CommAbort && n.CommDestroy && n.Broadcast && n.GroupStart &&
               n.GroupEnd;
        return n;
    }();
    return n;
}

using Clock = std::chrono::steady_clock;
double ms_since(Clock::time_point t0) { return std::chrono::duration<double, std::milli>(Clock::now() - t0).count(); }

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// the handle: one per rank (process or thread) and device
// ---------------------------------------------------------------------------------------------------------------
constexpr int MG_MAX_PIECES = 64, MG_MAX_BLOCKS = 32;
struct ozb_mg {
    int world, rank, dev, timeout_ms;
    int reserve_sms;                   // SMs the GEMMs leave to NCCL's kernels while transfers are outstanding (its CTA cap)
    int *pending;                      // device word: non-zero while pieces of B are still to come (set and cleared on sComm)
    ncclComm_t comm;                   // every transfer that is waited for: as many CTAs as NCCL likes
    ncclComm_t comm_beside;            // transfers that run beside the GEMMs (the stream layout): CTAs capped, SMs reserved for them
    bool broken;                       // the communicator was aborted: every later call answers OZB_ECOMM
    cudaStream_t sComm, sIn, sRun, sOut;
    cudaEvent_t evStart, evDone, evPiece[MG_MAX_PIECES], evIn[MG_MAX_PIECES], evRun[MG_MAX_BLOCKS];
    ozb_plan *plan;
    double *stageB; size_t stageB_elems;   // this rank's copy of B (receivers; a holder whose B is strided or comes from the host)
    double *dA, *dC; size_t dA_elems, dC_elems;   // host-operand and single-process paths: this rank's rows on its device
    cudaEvent_t mark[96]; char mark_name[96][20]; int marks;   // OZ_MG_TRACE: a timeline of the last product on this rank
    cudaEvent_t landed[MG_MAX_PIECES]; int landings;           // OZ_MG_TRACE: when each piece of B had arrived (communication stream)
    int last_layout, last_pieces, last_kernels;   // what the last product did (0 whole, 1 stream; transfers of B; kernels of this library), for reports
};

namespace {

// ncclCommAbort of the handle's communicators, side by side and bounded: each runs in a thread of its own, and a thread
// that has not come back within the budget (a tear-down that waits for a peer that is gone) is left behind rather than
// waited for -- the call that noticed the failure must return.
void abort_comms(ncclComm_t a, ncclComm_t b, int budget_ms) {
    std::shared_ptr<std::atomic<int>> left = std::make_shared<std::atomic<int>>(0);
    for (ncclComm_t c : {a, b}) {
        if (!c) continue;
        left->fetch_add(1);
        std::thread([c, left] { nccl().CommAbort(c); left->fetch_sub(1); }).detach();
    }
    const auto t0 = Clock::now();
    while (left->load() > 0 && ms_since(t0) < budget_ms) std::this_thread::sleep_for(std::chrono::microseconds(200));
}
void mg_abort(ozb_mg *g) {
    if (!g->broken) abort_comms(g->comm, g->comm_beside != g->comm ? g->comm_beside : nullptr, g->timeout_ms);
    g->comm = g->comm_beside = nullptr;
    g->broken = true;
}
// waits, within the handle's budget, until the communicator has settled the call that returned `r`
int mg_settle(ozb_mg *g, ncclResult_t r, ncclComm_t comm = nullptr) {
    if (!comm) comm = g->comm;
    const auto t0 = Clock::now();
    while (r == ncclInProgress) {
        if (ms_since(t0) > g->timeout_ms) { mg_abort(g); return OZB_ECOMM; }
        std::this_thread::sleep_for(std::chrono::microseconds(20));
        if (nccl().CommGetAsyncError(comm, &r) != ncclSuccess) { mg_abort(g); return OZB_ECOMM; }
    }
    if (r != ncclSuccess) { mg_abort(g); return OZB_ECOMM; }
    return 0;
}
int mg_bcast(ozb_mg *g, void *buf, size_t bytes, int root, bool beside = false) {
    if (g->world == 1) return 0;   // a single rank holds B already; the rest of the schedule is the same
    if (g->broken) return OZB_ECOMM;
    static const bool trace = getenv("OZ_MG_TRACE") != nullptr;   // host time of every enqueue, on stderr
    const auto t0 = Clock::now();
    ncclComm_t comm = beside ? g->comm_beside : g->comm;
    const int rc = mg_settle(g, nccl().Broadcast(buf, buf, bytes, ncclChar, root, comm, g->sComm), comm);
    if (trace) fprintf(stderr, "ozb mg rank %d: broadcast of %zu bytes queued in %.3f ms (rc %d)\n", g->rank, bytes, ms_since(t0), rc);
    return rc;
}
// after an abort the collective's kernel leaves and the stream drains; the wait for that is bounded all the same
void drain(cudaEvent_t ev, int budget_ms) {
    const auto t0 = Clock::now();
    while (cudaEventQuery(ev) == cudaErrorNotReady && ms_since(t0) < budget_ms) std::this_thread::sleep_for(std::chrono::microseconds(200));
}
// waits for an event on the host, within the budget, watching the communicator: a product whose broadcast never completes
// (a peer is gone) ends here with the communicator aborted instead of blocking in a synchronise call for ever
int mg_wait_event(ozb_mg *g, cudaEvent_t ev) {
    const auto t0 = Clock::now();
    for (unsigned spin = 0;; spin++) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) return 0;
        if (q != cudaErrorNotReady) return (int)q;
        if ((spin & 63) == 63 && g->comm) {
            ncclResult_t r = ncclSuccess;
            ncclResult_t r2 = ncclSuccess;
            const bool bad2 = g->comm_beside && g->comm_beside != g->comm &&
                              (nccl().CommGetAsyncError(g->comm_beside, &r2) != ncclSuccess || (r2 != ncclSuccess && r2 != ncclInProgress));
            if (bad2 || nccl().CommGetAsyncError(g->comm, &r) != ncclSuccess || (r != ncclSuccess && r != ncclInProgress)) {
                mg_abort(g);
                drain(ev, g->timeout_ms);
                return OZB_ECOMM;
            }
        }
        if (ms_since(t0) > g->timeout_ms) {
            if (g->world > 1) mg_abort(g);
            drain(ev, g->timeout_ms);
            return g->world > 1 ? OZB_ECOMM : OZB_ETIMEOUT;
        }
        if (spin > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

cudaError_t grow(double **buf, size_t *have, size_t want) {
    if (*have >= want) return cudaSuccess;
    cudaFree(*buf);
    *buf = nullptr; *have = 0;
    cudaError_t e = cudaMalloc(buf, want * sizeof(double));
    if (e) { cudaGetLastError(); return e; }
    *have = want;
    return cudaSuccess;
}
int mg_plan(ozb_mg *g, int m, int N, int K, int nm) {
    ozb_plan *p = g->plan;
    if (p && (p->M != m || p->N != N || p->K != K || p->nm != nm)) { ozb_plan_free_internal(p); g->plan = nullptr; }
    if (!g->plan) if (int e = ozb_plan_make_internal(m, N, K, nm, 62, &g->plan)) { g->plan = nullptr; return e; }
    return 0;
}

// rows per piece of a K x N matrix sent in pieces of about `target` bytes: a multiple of 128 rows, fewer than MG_MAX_PIECES pieces
int piece_rows(int K, int N, size_t target) {
    long long rows = (long long)(target / ((size_t)N * 8)) / 128 * 128;
    if (rows < 128) rows = 128;
    while ((K + rows - 1) / rows > MG_MAX_PIECES - 1) rows += 128;   /* one more piece may be split off the front */
    return (int)rows;
}

enum { LAYOUT_WHOLE = 0, LAYOUT_STREAM = 1 };
// One transfer, or pieces consumed as they land? Streaming costs a pass over B on the holder before anything can be sent
// (the column maxima) and NCCL's kernels beside the compute kernels; it pays when the transfer is long against this
// rank's share of the product. Measured on B200s with n = 32768: two ranks (16384 rows each, 8 GiB of B) 216.1 ms in one
// transfer against 222.9 - 225.1 ms in 4 - 8 pieces; with 4096 rows per rank the transfer is a quarter of the step. A B of
// 512 MiB (n = 8192) is always sent whole: two ranks 7.32 ms per product against 7.62 - 7.67 ms in 4 - 8 pieces (one GPU
// 7.09 ms) -- NCCL's kernels beside the residue kernels cost more than the 0.25 ms of transfer they would hide. The
// estimate uses 600 GB/s for the broadcast and 3 POP/s for the GEMMs.
int choose_layout(int m, int K, int N, int nm) {
    static const int forced = [] {
        const char *env = getenv("OZ_MG_LAYOUT");
        return !env ? -1 : !strcmp(env, "whole") ? LAYOUT_WHOLE : !strcmp(env, "stream") ? LAYOUT_STREAM : -1;
    }();
    if (forced >= 0) return forced;
    const double bytes = 8.0 * K * N, transfer = bytes / 600e9, compute = 2.0 * nm * m * (double)N * K / 3.0e15;
    return bytes > (double)((size_t)1 << 30) && transfer > 0.08 * compute ? LAYOUT_STREAM : LAYOUT_WHOLE;
}
// bytes per piece of the stream layout: about 1 GiB, but at least four pieces (a B of 512 MiB travels in four pieces of
// 128 MiB); many more outstanding transfers than eight were measured to cost more than they hide
size_t piece_target(int K, int N) {
    static const size_t forced = [] { const char *env = getenv("OZ_MG_PIECE_MB"); const int v = env && *env ? atoi(env) : 0; return (size_t)(v > 0 ? v : 0) << 20; }();
    if (forced) return forced;
    const size_t bytes = (size_t)K * N * 8, quarter = bytes / 4;
    return quarter > ((size_t)1 << 30) ? (size_t)1 << 30 : quarter;
}

// The stream layout's schedule, as plain arithmetic: the pieces B travels in and, for each, whether the GEMMs of a K range
// are launched behind it. A K the single-GPU product runs in one launch (up to 1.5 chunks) stays one launch, after the last
// piece: only the residues of B are formed piece by piece. A longer K is cut as the single-GPU product cuts it: a first
// short range of about 2048 (one piece of half the usual size: the GEMMs start early), a second of about 4096, then about
// 8192 each; arrival (about 400 GB/s with NCCL's kernels capped to 32 CTAs, measured beside the GEMMs on four B200s) stays
// ahead of the GEMMs from there on.
struct Piece { int k0, len, range_k0, range_len; };   // range_len > 0: the GEMMs of [range_k0, range_k0 + range_len) follow this piece
int stream_schedule(int K, int N, Piece *out) {
    static const int kchunk = [] { const char *env = getenv("OZ_KCHUNK"); const int v = env && *env ? atoi(env) : 0; return v >= 1024 ? v : 8192; }();
    const bool one_range = K <= kchunk + kchunk / 2;
    const int rows = piece_rows(K, N, piece_target(K, N));
    const int first = !one_range && rows >= 512 && K > rows ? rows / 2 / 128 * 128 : rows;
    const int pieces = K <= first ? 1 : 1 + (K - first + rows - 1) / rows;
    int range_k0 = 0, ranges = 0;
    for (int i = 0; i < pieces; i++) {
        const int k0 = i == 0 ? 0 : first + (i - 1) * rows, full = i == 0 ? first : rows;
        const int len = K - k0 < full ? K - k0 : full, done = k0 + len;
        const int want = ranges == 0 ? kchunk / 4 : ranges == 1 ? kchunk / 2 : kchunk;
        // close the range when it is long enough, unless what would remain is too short to be a range of its own (a short K
        // leaves the accumulating epilogue, which re-reads the residues of the ranges before, longer than the MMAs of a tile)
        const bool close = i == pieces - 1 || (!one_range && done - range_k0 >= want && K - done >= kchunk * 3 / 4);
        out[i] = Piece{k0, len, range_k0, close ? done - range_k0 : 0};
        if (close) { range_k0 = done; ranges++; }
    }
    return pieces;
}

// OZ_MG_TRACE: a timing mark on the compute stream (events are created on first use and kept with the handle)
void mg_mark(ozb_mg *g, cudaStream_t st, const char *name, int i = -1) {
    static const bool trace = getenv("OZ_MG_TRACE") != nullptr;
    if (!trace || g->marks >= 96) return;
    cudaEvent_t &ev = g->mark[g->marks];
    if (!ev && cudaEventCreate(&ev) != cudaSuccess) return;
    if (i >= 0) snprintf(g->mark_name[g->marks], sizeof g->mark_name[0], "%s%d", name, i);
    else snprintf(g->mark_name[g->marks], sizeof g->mark_name[0], "%s", name);
    cudaEventRecord(ev, st);
    g->marks++;
}
void mg_landed(ozb_mg *g, int i) {
    static const bool trace = getenv("OZ_MG_TRACE") != nullptr;
    if (!trace || i >= MG_MAX_PIECES) return;
    if (!g->landed[i] && cudaEventCreate(&g->landed[i]) != cudaSuccess) return;
    cudaEventRecord(g->landed[i], g->sComm);
    g->landings = i + 1;
}
void mg_print_marks(ozb_mg *g) {
    if (g->marks < 2) return;
    char line[4096];   // one write per rank: the ranks of a job share the terminal
    int at = snprintf(line, sizeof line, "ozb mg rank %d timeline (ms):", g->rank);
    for (int i = 1; i < g->marks && at < (int)sizeof line - 64; i++) {
        float t = 0;
        if (cudaEventElapsedTime(&t, g->mark[i - 1], g->mark[i]) == cudaSuccess) at += snprintf(line + at, sizeof line - at, " %s %.2f", g->mark_name[i], t);
    }
    float all = 0;
    cudaEventElapsedTime(&all, g->mark[0], g->mark[g->marks - 1]);
    at += snprintf(line + at, sizeof line - at, " | total %.2f", all);
    if (g->landings) at += snprintf(line + at, sizeof line - at, " | pieces landed at");
    for (int i = 0; i < g->landings && at < (int)sizeof line - 32; i++) {
        float t = 0;
        if (cudaEventElapsedTime(&t, g->mark[0], g->landed[i]) == cudaSuccess) at += snprintf(line + at, sizeof line - at, " %.1f", t);
    }
    snprintf(line + at, sizeof line - at, "\n");
    fputs(line, stderr);
}

// C_local = A_local B on device operands; B is read on `root` only. Asynchronous on `st` (and the handle's own
// communication stream); ozb_mg_wait reports how it ended.
int mg_dgemm_dev(ozb_mg *g, int m, int N, int K, const double *A, long long lda, const double *B, long long ldb, double *C,
                 long long ldc, int nm, int root, cudaStream_t st) {
    if (g->broken) return OZB_ECOMM;
    if (int e = mg_plan(g, m, N, K, nm)) return e;
    ozb_plan *p = g->plan;
    p->last = st;
    cudaError_t e = cudaSuccess;
    const bool src = g->rank == root;
    const bool in_place = src && ldb == N;            // a dense B is sent from where it lies
    if (!in_place) if ((e = grow(&g->stageB, &g->stageB_elems, (size_t)K * N))) return (int)e;
    double *whole = in_place ? const_cast<double *>(B) : g->stageB;
    const int layout = choose_layout(m, K, N, nm);
    // order: after the caller's writes of A and B (stream st), and after the previous product's reads of the staging copy
    if (src && !in_place) e = cudaMemcpy2DAsync(g->stageB, (size_t)N * 8, B, (size_t)ldb * 8, (size_t)N * 8, K, cudaMemcpyDeviceToDevice, st);
    if (!e) e = cudaMemsetAsync(p->colmax, 0, (size_t)N * 8, st);
    g->marks = 0; g->landings = 0;
    mg_mark(g, st, "start");
    int kernels = 2;   // the residues of A and the reconstruction; counted below: maxima, residues of B, GEMM launches
    if (!e && layout == LAYOUT_STREAM && src) { e = cols_absmax_accumulate(whole, K, N, N, p->colmax, st); kernels++; }
    if (!e) e = cudaEventRecord(g->evStart, st);
    if (!e) e = cudaStreamWaitEvent(g->sComm, g->evStart, 0);
    if (!e) e = cudaStreamWaitEvent(g->sComm, g->evDone, 0);
    if (e) return (int)e;

    // The host queues the residues of A first and then, piece by piece, the transfer and right behind it the work that
    // consumes the piece (the compute stream waits for the arrival on the device). Queueing every transfer before any
    // computation would leave the GPU without work while the host is still inside NCCL's enqueue calls, which take
    // milliseconds each when several transfers are outstanding.
    mg_mark(g, st, "maxima");
    e = scale_residues_rows(nm, A, m, K, lda, p->bits, p->sa, p->Ar, p->Kp, p->planeA, st);
    if (e) return (int)e;
    mg_mark(g, st, "rowsA");
    int pieces = 1;
    if (layout == LAYOUT_WHOLE) {
        if (int c = mg_bcast(g, whole, (size_t)K * N * 8, root)) return c;
        if ((e = cudaEventRecord(g->evPiece[0], g->sComm))) return (int)e;
        if (!src) e = cudaStreamWaitEvent(st, g->evPiece[0], 0);
        mg_mark(g, st, "wait");
        if (!e) e = cols_absmax_accumulate(whole, K, N, N, p->colmax, st);
        if (!e) e = cols_residues_from_max(nm, whole, K, N, N, p->bits, p->colmax, p->sb, p->Br, p->Kp, p->planeB, st);
        mg_mark(g, st, "colsB");
        if (!e) e = ozb_plan_gemm_range(p, N, 0, K, 0, st, 0, -1, &kernels);
        mg_mark(g, st, "gemm");
        kernels += 2;
    } else {
        Piece sched[MG_MAX_PIECES];
        pieces = stream_schedule(K, N, sched);
        // OZ_MG_YIELD=0: the GEMMs of every range but the last leave NCCL's SMs free whatever the transfers do
        static const bool yield = [] { const char *env = getenv("OZ_MG_YIELD"); return !(env && *env == '0'); }();
        const bool beside = g->world > 1 && g->reserve_sms > 0;
        if (beside) if ((e = cudaMemsetAsync(g->pending, 1, sizeof(int), g->sComm))) return (int)e;
        if (int c = mg_bcast(g, p->colmax, (size_t)N * 8, root, true)) return c;   // the column maxima, ahead of B on the same stream
        for (int i = 0, ranges = 0; i < pieces && !e; i++) {
            const Piece &pc = sched[i];
            if (int c = mg_bcast(g, whole + (size_t)pc.k0 * N, (size_t)pc.len * N * 8, root, true)) return c;
            if (beside && i == pieces - 1) if ((e = cudaMemsetAsync(g->pending, 0, sizeof(int), g->sComm))) break;
            if ((e = cudaEventRecord(g->evPiece[i], g->sComm))) break;
            mg_landed(g, i);
            if (!src) e = cudaStreamWaitEvent(st, g->evPiece[i], 0);
            mg_mark(g, st, "wait", i);
            if (!e) e = cols_residues_from_max(nm, whole + (size_t)pc.k0 * N, pc.len, N, N, p->bits, p->colmax, p->sb, p->Br + pc.k0, p->Kp, p->planeB, st);
            kernels++;
            mg_mark(g, st, "res", i);
            if (!e && pc.range_len) {
                // A persistent GEMM gives no SM back before it ends, and the transfer of the next piece is a kernel of its
                // own that starts when the one before it has finished: while pieces are still to come, the GEMMs leave
                // NCCL's SMs free. Whether pieces are still to come is read on the device when a CTA pair starts (the word
                // `pending`, cleared on the communication stream behind the last piece): the host queues the launches long
                // before they run and cannot know. The last range starts after the last piece and takes every SM.
                const int reserve = beside && i < pieces - 1 ? g->reserve_sms : 0;
                e = ozb_plan_gemm_range(p, N, pc.range_k0, pc.range_len, ranges++ > 0, st, 0, -1, &kernels, reserve, yield ? g->pending : nullptr);
                mg_mark(g, st, "gemm", ranges - 1);
            }
        }
    }
    g->last_layout = layout; g->last_pieces = pieces; g->last_kernels = kernels;
    if (!e) e = crt_from_i8(nm, p->Cr, p->planeC, m, N, p->Np, p->sa, p->sb, C, ldc, st);
    mg_mark(g, st, "crt");
    // the holder's stream also waits for the sends: the caller may overwrite B (or the next call the staging copy) after this call
    if (!e && src) e = cudaStreamWaitEvent(st, g->evPiece[pieces - 1], 0);
    if (!e) e = cudaEventRecord(g->evDone, st);
    return (int)e;
}

// The same product on host operands (pinned memory makes the copies asynchronous): B goes to the holder's GPU in pieces
// of rows, each piece is broadcast as it lands and its column maxima are taken on every rank as it arrives; once B is
// complete its residues are formed, while this rank's rows of A follow in blocks. A block of rows of C needs only its
// rows of A, so each block is scaled, multiplied and reconstructed as soon as it has landed and travels back while the
// next one is in flight (the block pipeline of the single-GPU host path). Synchronous.
int mg_dgemm_host(ozb_mg *g, int m, int N, int K, const double *A, const double *B, double *C, int nm, int root) {
    if (g->broken) return OZB_ECOMM;
    if (int e = mg_plan(g, m, N, K, nm)) return e;
    ozb_plan *p = g->plan;
    cudaError_t e = grow(&g->stageB, &g->stageB_elems, (size_t)K * N);
    if (!e) e = grow(&g->dA, &g->dA_elems, (size_t)m * K);
    if (!e) e = grow(&g->dC, &g->dC_elems, (size_t)m * N);
    if (e) return (int)e;
    const bool src = g->rank == root;
    p->last = g->sRun;
    int pieces = K / 512;
    if (pieces > 16) pieces = 16;
    if (pieces < 1) pieces = 1;
    const int rows = (K + pieces - 1) / pieces;
    pieces = (K + rows - 1) / rows;
    e = cudaMemsetAsync(p->colmax, 0, (size_t)N * 8, g->sRun);
    for (int i = 0; i < pieces && !e; i++) {
        const size_t k0 = (size_t)i * rows;
        const int len = (int)(K - k0 < (size_t)rows ? K - k0 : rows);
        if (src) {
            e = cudaMemcpyAsync(g->stageB + k0 * N, B + k0 * N, (size_t)len * N * 8, cudaMemcpyHostToDevice, g->sIn);
            if (!e) e = cudaEventRecord(g->evIn[i], g->sIn);
            if (!e) e = cudaStreamWaitEvent(g->sComm, g->evIn[i], 0);
        }
        if (e) break;
        if (g->world > 1) {
            if (int c = mg_bcast(g, g->stageB + k0 * N, (size_t)len * N * 8, root)) return c;
            e = cudaEventRecord(g->evPiece[i], g->sComm);
            if (!e) e = cudaStreamWaitEvent(g->sRun, g->evPiece[i], 0);
        } else {
            e = cudaStreamWaitEvent(g->sRun, g->evIn[i], 0);
        }
        if (!e) e = cols_absmax_accumulate(g->stageB + k0 * N, len, N, N, p->colmax, g->sRun);
    }
    if (!e) e = cols_residues_from_max(nm, g->stageB, K, N, N, p->bits, p->colmax, p->sb, p->Br, p->Kp, p->planeB, g->sRun);
    int blocks = m / 512;
    if (blocks > 16) blocks = 16;
    if (blocks < 1) blocks = 1;
    const int mblock = (m + blocks - 1) / blocks;
    size_t i0 = 0;
    for (int q = 0; i0 < (size_t)m && !e; q++) {   // the last blocks are halved down to 128 rows: what follows the last copy is exposed
        const size_t left = m - i0;
        size_t m_ = left > (size_t)mblock ? (size_t)mblock : (left > 128 ? (left / 2 + 127) / 128 * 128 : left);
        if (q >= MG_MAX_BLOCKS - 1 || m_ > left) m_ = left;
        const int mb = (int)m_;
        static_assert(16 + MG_MAX_BLOCKS <= MG_MAX_PIECES, "evIn holds the pieces of B and the blocks of A");
        e = cudaMemcpyAsync(g->dA + i0 * K, A + i0 * K, (size_t)mb * K * 8, cudaMemcpyHostToDevice, g->sIn);
        if (!e) e = cudaEventRecord(g->evIn[pieces + q], g->sIn);
        if (!e) e = cudaStreamWaitEvent(g->sRun, g->evIn[pieces + q], 0);
        if (!e) e = scale_residues_rows(nm, g->dA + i0 * K, mb, K, K, p->bits, p->sa + i0, p->Ar + i0 * p->Kp, p->Kp, p->planeA, g->sRun);
        if (!e) e = ozb_plan_gemm_range(p, N, 0, K, 0, g->sRun, (int)i0, mb);
        if (!e) e = crt_from_i8(nm, p->Cr + i0 * p->Np, p->planeC, mb, N, p->Np, p->sa + i0, p->sb, g->dC + i0 * N, N, g->sRun);
        if (!e) e = cudaEventRecord(g->evRun[q], g->sRun);
        if (!e) e = cudaStreamWaitEvent(g->sOut, g->evRun[q], 0);
        if (!e) e = cudaMemcpyAsync(C + i0 * N, g->dC + i0 * N, (size_t)mb * N * 8, cudaMemcpyDeviceToHost, g->sOut);
        i0 += m_;
    }
    if (e) return (int)e;
    if ((e = cudaEventRecord(g->evDone, g->sOut))) return (int)e;
    if (int c = mg_wait_event(g, g->evDone)) return c;
    if ((e = cudaStreamSynchronize(g->sRun))) return (int)e;
    if ((e = cudaStreamSynchronize(g->sIn))) return (int)e;
    if (g->world > 1 && !g->broken) if ((e = cudaStreamSynchronize(g->sComm))) return (int)e;
    g->last_layout = LAYOUT_WHOLE; g->last_pieces = pieces;
    return ozb_read_status_words(p->status);
}

int check_device() {
    int dev, major;
    if (cudaGetDevice(&dev) || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) return (int)cudaGetLastError();
    return major != 10 ? OZB_EARCH : 0;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------------
OZB_API int ozb_mg_unique_id(void *id) {
    if (!id) return OZB_EARG;
    if (!nccl().ok) return OZB_ENCCL;
    static_assert(sizeof(ncclUniqueId) == OZB_MG_ID_BYTES, "rendezvous id size");
    ncclUniqueId u;
    if (nccl().GetUniqueId(&u) != ncclSuccess) return OZB_ECOMM;
    memcpy(id, &u, sizeof u);
    return 0;
}

OZB_API int ozb_mg_create(int world, int rank, const void *id, int timeout_ms, ozb_mg **out) {
    if (!out || world < 1 || rank < 0 || rank >= world || (world > 1 && !id) || timeout_ms < 0) return OZB_EARG;
    if (int e = check_device()) return e;
    if (world > 1 && !nccl().ok) return OZB_ENCCL;
    ozb_mg *g = new ozb_mg();
    memset(g, 0, sizeof *g);
    g->world = world; g->rank = rank; g->timeout_ms = timeout_ms ? timeout_ms : 30000;
    cudaGetDevice(&g->dev);
    int lo = 0, hi = 0;
    cudaError_t e = cudaDeviceGetStreamPriorityRange(&lo, &hi);
    // the communication stream has the highest priority: a transfer kernel queued behind a compute kernel's block dispatch waits otherwise
    if (!e) e = cudaStreamCreateWithPriority(&g->sComm, cudaStreamNonBlocking, hi);
    if (!e) e = cudaStreamCreateWithFlags(&g->sIn, cudaStreamNonBlocking);
    if (!e) e = cudaStreamCreateWithFlags(&g->sRun, cudaStreamNonBlocking);
    if (!e) e = cudaStreamCreateWithFlags(&g->sOut, cudaStreamNonBlocking);
    if (!e) e = cudaEventCreateWithFlags(&g->evStart, cudaEventDisableTiming);
    if (!e) e = cudaEventCreateWithFlags(&g->evDone, cudaEventDisableTiming);
    for (auto &ev : g->evPiece) if (!e) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    for (auto &ev : g->evIn) if (!e) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    for (auto &ev : g->evRun) if (!e) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (!e) e = cudaMalloc(&g->pending, sizeof(int));
    if (!e) e = cudaMemset(g->pending, 0, sizeof(int));
    int rc = (int)e;
    if (!rc && world > 1) {
        ncclUniqueId u;
        memcpy(&u, id, sizeof u);
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.blocking = 0;
        rc = mg_settle(g, nccl().CommInitRankConfig(&g->comm, world, u, rank, &cfg));
        if (!rc) {   // initialisation itself proceeds in the background: wait for it within the budget
            ncclResult_t r = ncclInProgress;
            if (nccl().CommGetAsyncError(g->comm, &r) != ncclSuccess) r = ncclInternalError;
            rc = mg_settle(g, r);
        }
        // A second communicator over the same ranks for the transfers that run beside the GEMMs: its kernels are capped to a
        // few CTAs (OZ_MG_MAX_CTAS; default 32, 16 between two ranks) and the GEMMs leave as many SMs free (OZ_MG_RESERVE_SMS)
        // while pieces are still to come. Measured beside the GEMMs, 1 GiB pieces: among four B200s (every rank receives and
        // forwards) 16 CTAs deliver 114 GB/s (the 8 GiB of B at n = 32768 take 62 ms -- longer than an eighth of that
        // product), 24 CTAs 330 GB/s, 32 CTAs 405 GB/s; between two B200s 16 CTAs deliver 350 GB/s and 32 CTAs 580 GB/s, and a
        // 4096-row share of that product takes 60.7 ms with 16, 61.9 with 32, 63.3 with 48 (58.1 with no transfer at all).
        // Transfers that are
        // waited for keep the first communicator and all the CTAs NCCL wants: capped, a 512 MiB broadcast between four
        // B200s took 0.9 ms longer.
        g->comm_beside = g->comm;
        g->reserve_sms = 0;
        static const bool two = [] { const char *env = getenv("OZ_MG_ONE_COMM"); return !(env && *env == '1'); }();
        if (!rc && two) {
            // its rendezvous id is made by rank 0 and travels over the first communicator
            ncclUniqueId u2;
            void *dbuf = nullptr;
            cudaError_t ce = cudaMalloc(&dbuf, sizeof u2);
            if (!ce && rank == 0) {
                if (nccl().GetUniqueId(&u2) != ncclSuccess) ce = cudaErrorUnknown;
                if (!ce) ce = cudaMemcpyAsync(dbuf, &u2, sizeof u2, cudaMemcpyHostToDevice, g->sComm);
            }
            if (ce) rc = (int)ce;
            if (!rc) rc = mg_bcast(g, dbuf, sizeof u2, 0);
            if (!rc) rc = (int)cudaEventRecord(g->evStart, g->sComm);
            if (!rc) rc = mg_wait_event(g, g->evStart);
            if (!rc) rc = (int)cudaMemcpy(&u2, dbuf, sizeof u2, cudaMemcpyDeviceToHost);
            cudaFree(dbuf);
            if (!rc) {
                ncclConfig_t cap = NCCL_CONFIG_INITIALIZER;
                cap.blocking = 0;
                const char *env = getenv("OZ_MG_MAX_CTAS");
                cap.maxCTAs = env && atoi(env) > 0 ? atoi(env) : world <= 2 ? 16 : 32;
                ncclComm_t second = nullptr;
                ncclResult_t r = nccl().CommInitRankConfig(&second, world, u2, rank, &cap);
                if (second) g->comm_beside = second;          // from here on an abort takes it along
                if (r == ncclInProgress || r == ncclSuccess) {
                    ncclResult_t st2 = ncclInProgress;
                    if (!second || nccl().CommGetAsyncError(second, &st2) != ncclSuccess) st2 = ncclInternalError;
                    rc = mg_settle(g, st2, second);
                } else {
                    rc = mg_settle(g, r, second);
                }
                if (!rc) {
                    const char *res = getenv("OZ_MG_RESERVE_SMS");
                    g->reserve_sms = res && *res ? atoi(res) : cap.maxCTAs;
                }
            }
        }
    }
    if (rc) { ozb_mg_destroy(g); return rc; }
    *out = g;
    return 0;
}

OZB_API void ozb_mg_destroy(ozb_mg *g) {
    if (!g) return;
    int cur = -1;
    const int dev = g->dev;
    cudaGetDevice(&cur);
    if (cur != dev) cudaSetDevice(dev);
    if (g->comm && !g->broken) {
        // Tear-down must not depend on the peers: ncclCommDestroy of a live communicator may wait for them (a rank that
        // leaves on its own would block there), ncclCommAbort releases the local resources whatever the others do. The
        // handle's own transfers have been waited for by then (every product ends with ozb_mg_wait or a synchronous call).
        cudaEvent_t idle = g->evStart;
        if (cudaEventRecord(idle, g->sComm) == cudaSuccess) drain(idle, g->timeout_ms);
        abort_comms(g->comm, g->comm_beside != g->comm ? g->comm_beside : nullptr, g->timeout_ms);
    }
    if (g->plan) ozb_plan_free_internal(g->plan);
    cudaFree(g->stageB); cudaFree(g->dA); cudaFree(g->dC); cudaFree(g->pending);
    for (cudaStream_t s : {g->sComm, g->sIn, g->sRun, g->sOut}) if (s) cudaStreamDestroy(s);
    for (cudaEvent_t ev : {g->evStart, g->evDone}) if (ev) cudaEventDestroy(ev);
    for (auto ev : g->evPiece) if (ev) cudaEventDestroy(ev);
    for (auto ev : g->evIn) if (ev) cudaEventDestroy(ev);
    for (auto ev : g->evRun) if (ev) cudaEventDestroy(ev);
    for (auto ev : g->mark) if (ev) cudaEventDestroy(ev);
    for (auto ev : g->landed) if (ev) cudaEventDestroy(ev);
    delete g;
    if (cur >= 0 && cur != dev) cudaSetDevice(cur);
}

OZB_API int ozb_mg_dgemm(ozb_mg *g, int m_local, int N, int K, const double *A, long long lda, const double *B, long long ldb, double *C,
                         long long ldc, int moduli, int root, int on_host, void *stream) {
    if (!g || m_local <= 0 || N <= 0 || K <= 0 || moduli < 8 || moduli > 16 || root < 0 || root >= g->world || !A || !C) return OZB_EARG;
    if (K >= 131072) return OZB_EK;
    if (g->rank == root && !B) return OZB_EARG;
    int dev = -1;
    if (cudaGetDevice(&dev) || dev != g->dev) return (int)cudaErrorInvalidDevice;
    if (on_host) {
        if (lda != K || ldc != N || (g->rank == root && ldb != N)) return OZB_EARG;   // host operands are dense, as in ozb_dgemm
        return mg_dgemm_host(g, m_local, N, K, A, B, C, moduli, root);
    }
    if (lda < K || ldc < N || (g->rank == root && ldb < N)) return OZB_EARG;
    return mg_dgemm_dev(g, m_local, N, K, A, lda, B, ldb, C, ldc, moduli, root, (cudaStream_t)stream);
}

OZB_API int ozb_mg_wait(ozb_mg *g) {
    if (!g) return OZB_EARG;
    if (g->broken) return OZB_ECOMM;
    if (!g->plan) return 0;
    if (int c = mg_wait_event(g, g->evDone)) return c;
    mg_print_marks(g);
    return ozb_read_status_words(g->plan->status);
}

OZB_API int ozb_mg_schedule(int m_local, int N, int K, int moduli, int *layout, int *pieces, int *ranges) {
    if (m_local <= 0 || N <= 0 || K <= 0 || moduli < 8 || moduli > 16) return OZB_EARG;
    if (K >= 131072) return OZB_EK;
    const int lay = choose_layout(m_local, K, N, moduli);
    int np = 1, nr = 1;
    if (lay == LAYOUT_STREAM) {
        Piece sched[MG_MAX_PIECES];
        np = stream_schedule(K, N, sched);
        nr = 0;
        for (int i = 0; i < np; i++) nr += sched[i].range_len > 0;
    }
    if (layout) *layout = lay;
    if (pieces) *pieces = np;
    if (ranges) *ranges = nr;
    return 0;
}

OZB_API int ozb_mg_schedule_pieces(int m_local, int N, int K, int moduli, int layout, int cap, int *k0, int *len, int *range_k0,
                                   int *range_len) {
    if (m_local <= 0 || N <= 0 || K <= 0 || moduli < 8 || moduli > 16 || layout < -1 || layout > 1 || cap < 0) return -OZB_EARG;
    if (K >= 131072) return -OZB_EK;
    const int lay = layout < 0 ? choose_layout(m_local, K, N, moduli) : layout;
    Piece sched[MG_MAX_PIECES];
    int np = 1;
    if (lay == LAYOUT_STREAM) np = stream_schedule(K, N, sched);
    else sched[0] = Piece{0, K, 0, K};
    for (int i = 0; i < np && i < cap; i++) {
        if (k0) k0[i] = sched[i].k0;
        if (len) len[i] = sched[i].len;
        if (range_k0) range_k0[i] = sched[i].range_k0;
        if (range_len) range_len[i] = sched[i].range_len;
    }
    return np;
}

OZB_API int ozb_mg_info(ozb_mg *g, int *layout, int *pieces, int *kernels) {
    if (!g) return OZB_EARG;
    if (layout) *layout = g->last_layout;
    if (pieces) *pieces = g->last_pieces;
    if (kernels) *kernels = g->last_kernels;
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// one process, several devices: the reference's ozb_dgemm with a device count
// ---------------------------------------------------------------------------------------------------------------
namespace {
std::mutex mg_mu;
ozb_mg *mg_handles[16] = {};
int mg_ndev = 0;

void mg_release_all() {
    for (int d = 0; d < mg_ndev; d++) { ozb_mg_destroy(mg_handles[d]); mg_handles[d] = nullptr; }
    mg_ndev = 0;
}
void row_block(int M, int r, int world, int *lo, int *hi) {   // blocks differ by at most one row, earlier ranks get the longer ones
    const int base = M / world, extra = M % world;
    *lo = r * base + (r < extra ? r : extra);
    *hi = *lo + base + (r < extra ? 1 : 0);
}
}  // namespace

OZB_API int ozb_dgemm_mg(int M, int N, int K, const double *A, const double *B, double *C, int moduli, int on_host, int ndev) {
    if (M <= 0 || N <= 0 || K <= 0 || moduli < 8 || moduli > 16 || ndev < 1 || ndev > 16 || !A || !B || !C) return OZB_EARG;
    if (K >= 131072) return OZB_EK;
    int have = 0, cur = 0;
    if (cudaGetDeviceCount(&have) || cudaGetDevice(&cur)) return (int)cudaGetLastError();
    if (ndev > have) return OZB_EARG;
    if (ndev > M) ndev = M;
    std::lock_guard<std::mutex> lock(mg_mu);
    int rcs[16] = {};
    if (mg_ndev != ndev) {   // one handle per device 0 .. ndev-1, made by one thread per device as separate processes would
        mg_release_all();
        char id[OZB_MG_ID_BYTES] = {};
        if (ndev > 1) if (int e = ozb_mg_unique_id(id)) return e;
        std::thread th[16];
        for (int d = 0; d < ndev; d++)
            th[d] = std::thread([&, d] { rcs[d] = (int)cudaSetDevice(d); if (!rcs[d]) rcs[d] = ozb_mg_create(ndev, d, id, 0, &mg_handles[d]); });
        for (int d = 0; d < ndev; d++) th[d].join();
        mg_ndev = ndev;
        for (int d = 0; d < ndev; d++) if (rcs[d]) { const int e = rcs[d]; mg_release_all(); cudaSetDevice(cur); return e; }
    }
    // device operands live on the calling thread's current device, which also holds B: that device is the root and works
    // in place, the others get their rows of A and return their rows of C with peer copies
    const int root = on_host ? 0 : (cur < ndev ? cur : 0);
    if (!on_host && cur >= ndev) return OZB_EARG;
    if (!on_host) if (cudaError_t e = cudaDeviceSynchronize()) return (int)e;   // the operands' pending writes, whatever stream made them
    std::thread th[16];
    for (int d = 0; d < ndev; d++)
        th[d] = std::thread([&, d] {
            int &rc = rcs[d];
            rc = (int)cudaSetDevice(d);
            if (rc) return;
            ozb_mg *g = mg_handles[d];
            int lo, hi;
            row_block(M, d, ndev, &lo, &hi);
            const int m = hi - lo;
            if (on_host) { rc = mg_dgemm_host(g, m, N, K, A + (size_t)lo * K, d == root ? B : nullptr, C + (size_t)lo * N, moduli, root); return; }
            if (d == cur) {
                rc = mg_dgemm_dev(g, m, N, K, A + (size_t)lo * K, K, B, N, C + (size_t)lo * N, N, moduli, root, g->sRun);
            } else {
                cudaError_t e = grow(&g->dA, &g->dA_elems, (size_t)m * K);
                if (!e) e = grow(&g->dC, &g->dC_elems, (size_t)m * N);
                if (!e) e = cudaMemcpyPeerAsync(g->dA, d, A + (size_t)lo * K, cur, (size_t)m * K * 8, g->sRun);
                rc = (int)e;
                if (!rc) rc = mg_dgemm_dev(g, m, N, K, g->dA, K, nullptr, N, g->dC, N, moduli, root, g->sRun);
                if (!rc) rc = (int)cudaMemcpyPeerAsync(C + (size_t)lo * N, cur, g->dC, d, (size_t)m * N * 8, g->sRun);
                if (!rc) rc = (int)cudaEventRecord(g->evDone, g->sRun);
            }
            if (!rc) rc = ozb_mg_wait(g);
        });
    for (int d = 0; d < ndev; d++) th[d].join();
    cudaSetDevice(cur);
    int rc = 0;
    for (int d = 0; d < ndev; d++) if (rcs[d] && !rc) rc = rcs[d];
    if (rc == OZB_ECOMM) mg_release_all();   // an aborted communicator cannot be used again: the next call starts afresh
    return rc;
}

OZB_API void ozb_mg_release(void) {
    std::lock_guard<std::mutex> lock(mg_mu);
    mg_release_all();
}
