// oz_kernels.h -- host-callable launchers of the four stages (definitions in scale_residue.cu, gemm_i8_sm100.cu, crt.cu)
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace ozk {

cudaError_t scale_residues_rows(int nm, const double *X, int rows, int len, long long ldx, int bits, int *s, int8_t *R, int ld,
                                size_t plane, cudaStream_t st);
cudaError_t scale_residues_cols(int nm, const double *X, int rows, int cols, long long ldx, int bits, unsigned long long *colmax,
                                int *s, int8_t *R, int ld, size_t plane, cudaStream_t st);
cudaError_t cols_absmax_accumulate(const double *X, int rows, int cols, long long ldx, unsigned long long *colmax, cudaStream_t st);
cudaError_t cols_residues_from_max(int nm, const double *X, int rows, int cols, long long ldx, int bits, const unsigned long long *colmax,
                                   int *s, int8_t *R, int ld, size_t plane, cudaStream_t st);
cudaError_t scales_norm_only(const double *X, int nvec, int len, long long ldx, int by_rows, int beta, int *s, cudaStream_t st);
cudaError_t norm_scale_residues_rows(int nm, const double *X, int rows, int len, long long ldx, int beta, int *s, int8_t *R, int ld,
                                     size_t plane, cudaStream_t st);
cudaError_t norm_scale_residues_cols(int nm, const double *X, int rows, int cols, long long ldx, int beta, int *s, int8_t *R, int ld,
                                     size_t plane, cudaStream_t st);
cudaError_t gemm_i8_planes(const int8_t *A, const int8_t *Bt, void *C, int M, int N, int K, int Z, long long lda, long long ldb,
                           long long ldc, size_t pa, size_t pb, size_t pc, int fused, int first_modulus, int *status, int sms,
                           cudaStream_t st, int accumulate = 0, int reserve_sms = 0, const int *yield_flag = nullptr);
cudaError_t int8_peak_probe(int iters, int pair, float *ms, double *tops, int *status, cudaStream_t st);
cudaError_t wait_expiry_selftest(unsigned budget_ms, int *status, cudaStream_t st);
cudaError_t crt_from_i8(int nm, const int8_t *Cr, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
                        double *C, long long ldc, cudaStream_t st);
cudaError_t crt_from_i32(int nm, const int32_t *Cl, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb,
                         double *C, long long ldc, cudaStream_t st);

// checked-access debug build (oz_bounds.cuh): per-file violation words and the checker's self-test
cudaError_t scale_residue_violations(unsigned long long out[4]);
cudaError_t crt_violations(unsigned long long out[4]);
cudaError_t gemm_violations(unsigned long long out[4]);
cudaError_t bounds_selftest(int *buf5, cudaStream_t st);

// double-double path (dd.cu); nm in {24, 28, 32}
cudaError_t dd_scale_residues_rows(int nm, const double *Xh, const double *Xl, int rows, int len, long long ldx, int bits, int *s,
                                   int8_t *R, int ld, size_t plane, cudaStream_t st);
cudaError_t dd_scale_residues_cols(int nm, const double *Xh, const double *Xl, int rows, int cols, long long ldx, int bits,
                                   unsigned long long *colmax, int *s, int8_t *R, int ld, size_t plane, cudaStream_t st);
cudaError_t dd_crt_from_i8(int nm, const int8_t *Cr, size_t plane, int M, int N, long long ldr, const int *sa, const int *sb, double *Ch,
                           double *Cl, long long ldo, int mode, cudaStream_t st);

// correctly rounded BF16 x block-scaled FP8 product (exact_f8.cu)
int exact_bf16_fp8_gemm(int M, int N, int K, const uint16_t *X, long long ldx, const uint8_t *W, long long ldw, const float *S, float *Y,
                        long long ldy, int *open, int *moduli, cudaStream_t st);
void exact_f8_release();

}  // namespace ozk
