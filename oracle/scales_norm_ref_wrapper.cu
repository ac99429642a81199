// scales_norm_ref_wrapper.cu -- TEST INFRASTRUCTURE ONLY: the reference's optional 2-norm scaling kernel for the tests.
//
// Compiles the reference's bench/oz_strassen.cu where it lies (REF, never copied), with its main() renamed, and exports one
// C function that launches its scales_norm kernel (bench/oz_strassen.cu:78-97) the way the reference does
// (bench/oz_strassen.cu:258: one block of 256 threads per row of a row-contiguous matrix). Built by oracle/Makefile into
// oracle/_ref/; used on a GPU machine to pin the CPU checker's restatement of that kernel.
#define main ozref_strassen_main_unused
#include "bench/oz_strassen.cu"
#undef main

// s[r] for r < rows of the row-contiguous device matrix X (rows x len); returns a cudaError_t value
extern "C" __attribute__((visibility("default"))) int ozref_scales_norm(const double *X, int rows, int len, int beta, int *s) {
    scales_norm<<<rows, 256>>>(X, len, beta, s);
    const cudaError_t e = cudaGetLastError();
    return (int)(e ? e : cudaDeviceSynchronize());
}
