// Shim: prototypes of the few CBLAS entry points the reference's MatMul/Syrk/Gemv kernels call, mapped onto the
// OpenBLAS that ships inside the scipy wheel (its symbols carry a scipy_ prefix).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
typedef enum CBLAS_UPLO { CblasUpper = 121, CblasLower = 122 } CBLAS_UPLO;
typedef CBLAS_ORDER CBLAS_LAYOUT;
double scipy_cblas_ddot(int n, const double *x, int incx, const double *y, int incy);
float scipy_cblas_sdot(int n, const float *x, int incx, const float *y, int incy);
void scipy_cblas_dgemv(CBLAS_ORDER o, CBLAS_TRANSPOSE t, int m, int n, double alpha, const double *a, int lda,
                       const double *x, int incx, double beta, double *y, int incy);
void scipy_cblas_sgemv(CBLAS_ORDER o, CBLAS_TRANSPOSE t, int m, int n, float alpha, const float *a, int lda,
                       const float *x, int incx, float beta, float *y, int incy);
void scipy_cblas_dgemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, double alpha,
                       const double *a, int lda, const double *b, int ldb, double beta, double *c, int ldc);
void scipy_cblas_sgemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                       const float *a, int lda, const float *b, int ldb, float beta, float *c, int ldc);
void scipy_cblas_dsyrk(CBLAS_ORDER o, CBLAS_UPLO u, CBLAS_TRANSPOSE t, int n, int k, double alpha, const double *a,
                       int lda, double beta, double *c, int ldc);
void scipy_cblas_ssyrk(CBLAS_ORDER o, CBLAS_UPLO u, CBLAS_TRANSPOSE t, int n, int k, float alpha, const float *a,
                       int lda, float beta, float *c, int ldc);
void scipy_openblas_set_num_threads(int n);
#ifdef __cplusplus
}
#endif
#define cblas_ddot scipy_cblas_ddot
#define cblas_sdot scipy_cblas_sdot
#define cblas_dgemv scipy_cblas_dgemv
#define cblas_sgemv scipy_cblas_sgemv
#define cblas_dgemm scipy_cblas_dgemm
#define cblas_sgemm scipy_cblas_sgemm
#define cblas_dsyrk scipy_cblas_dsyrk
#define cblas_ssyrk scipy_cblas_ssyrk
