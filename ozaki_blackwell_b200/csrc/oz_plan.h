// oz_plan.h -- the plan behind the C ABI (the reference's oz::Plan, src/ozaki2.cuh:116-132, plus what the overlapped paths
// need), shared by the translation units of the host layer: capi.cu (the ABI itself) and mg.cu (row blocks over several GPUs).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

constexpr int HOST_PANELS = 32;
struct ozb_plan {
    int M, N, K, nm, bits, maxbits, dev;   // dev: the device the workspaces live on
    int Kp, Np;                      // pitch of the residue planes of A and B (bytes); pitch of the product planes (bytes)
    size_t planeA, planeB, planeC;   // plane pitches in bytes
    int8_t *Ar, *Br, *Cr;
    int *sa, *sb, *status;
    unsigned long long *colmax;
    cudaStream_t last;
    bool env_prof;                   // OZ_PROF set: one line per product on stderr, as the reference does
    int slots, calls;                // event ring: EV_PER_SLOT events per slot, slot = call number mod slots
    cudaEvent_t *ev;
    // column panels of one product: B's residues (stream s1), the GEMMs (caller's stream) and the CRT (stream s2) of
    // different panels run side by side; panels = 1 keeps everything on the caller's stream
    int panels, panel_width;
    cudaStream_t s1, s2;
    cudaEvent_t evFork, evJoin, evB[8], evG[8];
    // host operands (on_host = 1): device copies kept with the plan, three streams, one event pair per column panel
    double *hA, *hB, *hC;
    cudaStream_t sIn, sRun, sOut;
    bool host_streams;               // sIn, sRun, sOut and their events are all there
    cudaEvent_t evDone;              // end of the last asynchronous product queued on a cached plan (orders the next one after it)
    cudaEvent_t evIn[HOST_PANELS + 1], evRun[HOST_PANELS];
};
constexpr int MAXP = 8, EV_PER_SLOT = 2 + 2 * MAXP + 2;   // start, end, (start, end) of each panel's GEMM, and two marks inside
                                                            // the one-panel product: after the rows of A, after B's column maxima
constexpr int EV_ROWS = 2 + 2 * MAXP, EV_ABSMAX = EV_ROWS + 1;

// host-layer functions of capi.cu that mg.cu builds on (none of them takes the library's mutex)
int ozb_plan_make_internal(int M, int N, int K, int nm, int maxbits, ozb_plan **out);
void ozb_plan_free_internal(ozb_plan *p);
// the fused INT8 GEMMs of all planes over the inner range [k0, k0 + klen) of rows [i0, i0 + m) (m < 0: all rows) and the
// first n columns; accumulate != 0 adds to the residues already in Cr (an earlier part of K)
cudaError_t ozb_plan_gemm_range(ozb_plan *p, int n, int k0, int klen, int accumulate, cudaStream_t st, int i0 = 0, int m = -1,
                                int *launches = nullptr,    // *launches is incremented per GEMM kernel launched
                                int reserve_sms = 0,        // SMs the launches leave free for kernels that must start beside them
                                const int *yield_flag = nullptr);   // device word: leave them free only while it is non-zero
int ozb_read_status_words(int *dev_words);
