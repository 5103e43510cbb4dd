/* Minimal CBLAS prototypes for linking the reference build against an
 * OpenBLAS shared object that ships without headers. TEST INFRASTRUCTURE
 * ONLY: used when compiling the unmodified reference into oracle/_ref. */
#ifndef ORACLE_CBLAS_H
#define ORACLE_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
typedef CBLAS_ORDER CBLAS_LAYOUT;
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
                 float alpha, const float *a, int lda, const float *b, int ldb, float beta,
                 float *c, int ldc);
void cblas_sgemv(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, int m, int n, float alpha,
                 const float *a, int lda, const float *x, int incx, float beta, float *y,
                 int incy);
#ifdef __cplusplus
}
#endif
#endif
