// Shim: the one LAPACKE routine the reference's Solve kernel calls, from scipy's bundled OpenBLAS.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
#define LAPACK_ROW_MAJOR 101
#define LAPACK_COL_MAJOR 102
typedef int lapack_int;
lapack_int scipy_LAPACKE_dgesv(int layout, lapack_int n, lapack_int nrhs, double *a, lapack_int lda, lapack_int *ipiv,
                               double *b, lapack_int ldb);
lapack_int scipy_LAPACKE_sgesv(int layout, lapack_int n, lapack_int nrhs, float *a, lapack_int lda, lapack_int *ipiv,
                               float *b, lapack_int ldb);
#ifdef __cplusplus
}
#endif
#define LAPACKE_dgesv scipy_LAPACKE_dgesv
#define LAPACKE_sgesv scipy_LAPACKE_sgesv
