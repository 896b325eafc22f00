/* Minimal CBLAS declarations for building the reference's src/kernel/cblas.cc
 * against the OpenBLAS that ships inside SciPy, whose symbols carry a
 * `scipy_` prefix (LP64 build: blasint is int).  TEST INFRASTRUCTURE ONLY. */
#ifndef ORACLE_SHIM_CBLAS_H
#define ORACLE_SHIM_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 }
    CBLAS_TRANSPOSE;
void scipy_cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb,
        int m, int n, int k, float alpha, const float *a, int lda,
        const float *b, int ldb, float beta, float *c, int ldc);
void scipy_cblas_dgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb,
        int m, int n, int k, double alpha, const double *a, int lda,
        const double *b, int ldb, double beta, double *c, int ldc);
void scipy_openblas_set_num_threads(int n);
#define cblas_sgemm scipy_cblas_sgemm
#define cblas_dgemm scipy_cblas_dgemm
#ifdef __cplusplus
}
#endif
#endif
