/*
 * TEST INFRASTRUCTURE (oracle build only).  Minimal CBLAS declarations for the one routine the
 * reference's CPU matmul calls (ormi-core/csrc/backend/cpu/kernels/blas/matmul.cpp:70-73).  The image
 * ships an OpenBLAS shared library but no cblas.h; these are the standard CBLAS enum values and the
 * standard cblas_sgemm prototype.
 */
#ifndef ORMI_ORACLE_CBLAS_H
#define ORMI_ORACLE_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif

typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
typedef CBLAS_ORDER CBLAS_LAYOUT;

void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE trans_a, CBLAS_TRANSPOSE trans_b,
                 int m, int n, int k, float alpha, const float* a, int lda,
                 const float* b, int ldb, float beta, float* c, int ldc);

#ifdef __cplusplus
}
#endif
#endif
