// Declarations of the three standard CBLAS entry points the reference's blas
// backend calls; resolved at link time against an OpenBLAS shared object.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
                 float alpha, const float* a, int lda, const float* b, int ldb, float beta,
                 float* c, int ldc);
void cblas_sgemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int m, int n, float alpha, const float* a,
                 int lda, const float* x, int incx, float beta, float* y, int incy);
float cblas_sdot(int n, const float* x, int incx, const float* y, int incy);
#ifdef __cplusplus
}
#endif
