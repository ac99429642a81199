// oz_bounds.cuh -- checked global-memory accesses of the debug build (compile with -DOZ_BOUNDS).
//
// The memory checker of the CUDA toolkit cannot always be run where this library is tested, so the library can check
// itself: in a build with OZ_BOUNDS every global load and store of the scale / residue / reconstruction kernels and of
// the GEMM epilogue goes through oz_load / oz_store, which test the address against the windows the launcher registered
// for that launch -- the exact bytes the kernel is entitled to: row r of a pitched matrix is a window of `len` elements,
// not of `ld`, so an access into the padding between rows, or into the neighbouring column panel, counts as a violation.
// A violating access is NOT performed (a load returns zero); the first one is recorded (address, kernel, size) in a
// device word the host reads with ozb_bounds_report. Nothing traps and nothing faults.
// (The reference fills its workspaces with a poison value for the same purpose: src/ozaki_hol.cuh:498.)
// The GEMM's operand loads need no such check: they are TMA loads, bounded by the extents in their tensor maps.
//
// In a normal build oz_load / oz_store are plain accesses and OZ_WINDOWS expands to nothing.
// The registered windows are one set per translation unit, written on the launch's stream just before the kernel; the
// debug build drains the device before every such write, so checked kernels never overlap (it tests addresses, not timing).
#pragma once
#include <cuda_runtime.h>

namespace ozk {

#ifdef OZ_BOUNDS
// bytes [base + i2 * pitch2 + i1 * pitch1, ... + bytes0) for i2 < n2, i1 < n1
struct Window { unsigned long long base, n2, pitch2, n1, pitch1, bytes0; };
constexpr int MAX_WINDOWS = 8;
struct Windows { Window w[MAX_WINDOWS]; int n, kernel; };
static __device__ Windows g_windows;
static __device__ unsigned long long g_violation[4];   // count, first address, kernel id, bytes of the access

__device__ __forceinline__ bool oz_inside(const void *p, unsigned bytes) {
    const unsigned long long a = (unsigned long long)p;
    for (int i = 0; i < g_windows.n; i++) {
        const Window &w = g_windows.w[i];
        if (a < w.base) continue;
        unsigned long long off = a - w.base;
        const unsigned long long i2 = off / w.pitch2;
        if (i2 >= w.n2) continue;
        off -= i2 * w.pitch2;
        const unsigned long long i1 = off / w.pitch1;
        if (i1 >= w.n1) continue;
        off -= i1 * w.pitch1;
        if (off + bytes <= w.bytes0) return true;
    }
    if (atomicAdd(&g_violation[0], 1ull) == 0) { g_violation[1] = a; g_violation[2] = (unsigned long long)g_windows.kernel; g_violation[3] = bytes; }
    return false;
}
template <class T> __device__ __forceinline__ T oz_load(const T *p) { return oz_inside(p, sizeof(T)) ? *p : T{}; }
template <class T> __device__ __forceinline__ void oz_store(T *p, const T &v) { if (oz_inside(p, sizeof(T))) *p = v; }
__device__ __forceinline__ void oz_atomic_max(unsigned long long *p, unsigned long long v) { if (oz_inside(p, 8)) atomicMax(p, v); }

inline Window window1d(const void *base, size_t bytes) { return Window{(unsigned long long)base, 1, ~0ull >> 1, 1, ~0ull >> 1, bytes}; }
inline Window window2d(const void *base, size_t rows, size_t pitch, size_t row_bytes) {
    return Window{(unsigned long long)base, 1, ~0ull >> 1, rows, pitch ? pitch : 1, row_bytes};
}
inline Window window3d(const void *base, size_t planes, size_t plane_pitch, size_t rows, size_t pitch, size_t row_bytes) {
    return Window{(unsigned long long)base, planes, plane_pitch ? plane_pitch : 1, rows, pitch ? pitch : 1, row_bytes};
}
inline cudaError_t oz_set_windows(cudaStream_t st, int kernel, std::initializer_list<Window> ws) {
    Windows h{};
    for (const Window &w : ws) if (h.n < MAX_WINDOWS) h.w[h.n++] = w;
    h.kernel = kernel;
    // every checked kernel runs alone: the windows are one set per file, and kernels of one file may be queued on several
    // streams (the multi-panel path), so the device is drained before the set is replaced
    if (cudaError_t e = cudaDeviceSynchronize()) return e;
    return cudaMemcpyToSymbolAsync(g_windows, &h, sizeof h, 0, cudaMemcpyHostToDevice, st);   // pageable source: staged before the call returns
}
// count of violations in this translation unit since the last call (and the first one's details), then cleared
inline cudaError_t oz_read_violations(unsigned long long out[4]) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_violation, 4 * sizeof(unsigned long long));
    const unsigned long long zero[4] = {};
    if (!e && out[0]) e = cudaMemcpyToSymbol(g_violation, zero, sizeof zero);
    return e;
}
#define OZ_WINDOWS(st, id, ...) do { if (cudaError_t e_ = ::ozk::oz_set_windows(st, id, {__VA_ARGS__})) return e_; } while (0)
#else
template <class T> __device__ __forceinline__ T oz_load(const T *p) { return *p; }
template <class T> __device__ __forceinline__ void oz_store(T *p, const T &v) { *p = v; }
__device__ __forceinline__ void oz_atomic_max(unsigned long long *p, unsigned long long v) { atomicMax(p, v); }
inline cudaError_t oz_read_violations(unsigned long long out[4]) { out[0] = out[1] = out[2] = out[3] = 0; return cudaSuccess; }
#define OZ_WINDOWS(st, id, ...) do { } while (0)
#endif

// kernel ids in the violation report
enum { OZK_ROW_RESIDUES = 1, OZK_COL_ABSMAX = 2, OZK_COL_RESIDUES = 3, OZK_SCALES_NORM = 4, OZK_CRT = 5, OZK_GEMM_EPILOGUE = 6, OZK_SELFTEST = 7 };

}  // namespace ozk
