// ozaki2.hpp -- the reference's C++ entry points (src/ozaki2.cuh:101-164: oz::bits_for, oz::Plan, oz::plan, oz::release,
// oz::dgemm) as a thin inline layer over the C ABI of libozaki_blackwell.so (include/ozb.h), for C++ callers that
// `#include "ozaki2.cuh"` in the reference (every bench/*.cu does, e.g. bench/ozaki_test.cu:69-72). Same names, same
// call shapes; link with -lozaki_blackwell. Differences a caller can see:
//   * Plan holds a handle; the residue planes of the products are int8 (Cr) where the reference keeps int32 (Cl), so Cl
//     stays null. Mp, Np, Kp report this library's pitches (no row padding is needed: M and N are not rounded up).
//   * bits_for returns -1 for K >= 131072 where the reference aborts (src/ozaki2.cuh:105); plan() then yields a Plan
//     whose handle is null and whose `error` holds the code.
//   * dgemm takes optional leading dimensions and a stream; the defaults are the reference's (dense, legacy stream).
#pragma once
#include <cstdint>
#include "ozb.h"

namespace oz {

constexpr int MAXM = 49;
inline int modulus(int l) { return ozb_modulus(l); }
inline int bits_for(int nm, int K, int maxbits = 62) { return ozb_bits_for(nm, K, maxbits); }

struct Plan {
    int M, N, K, Mp, Np, Kp, nm, bits;
    int8_t *Ar, *Br;
    int32_t *Cl;        // always null here: the products are kept as int8 residues in Cr
    int *sa, *sb;
    int8_t *Cr;
    ozb_plan *handle;
    int error;          // 0, or the code ozb_plan_create returned
};

inline Plan plan(int M, int N, int K, int nm, int maxbits = 62) {
    Plan p{M, N, K, M, 0, 0, nm, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0};
    p.error = ozb_plan_create(M, N, K, nm, maxbits, &p.handle);
    if (!p.error) ozb_plan_view(p.handle, &p.bits, &p.Kp, &p.Np, &p.Ar, &p.Br, &p.Cr, &p.sa, &p.sb);
    return p;
}
inline void release(Plan &p) {
    if (p.handle) ozb_plan_destroy(p.handle);
    p.handle = nullptr;
}
// A: M x K, B: K x N, C: M x N, device FP64, row-major. Asynchronous on `stream` like the reference's launches.
inline int dgemm(Plan &p, const double *A, const double *B, double *C, long long lda = 0, long long ldb = 0, long long ldc = 0,
                 void *stream = nullptr) {
    if (!p.handle) return p.error ? p.error : OZB_EARG;
    return ozb_plan_dgemm(p.handle, A, lda ? lda : p.K, B, ldb ? ldb : p.N, C, ldc ? ldc : p.N, stream);
}

}  // namespace oz
