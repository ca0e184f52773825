/* Minimal CBLAS declarations, written for building the reference's
 * ops_matrix_openblas.c against an OpenBLAS shared object that ships without
 * headers.  Only what that file uses.  TEST INFRASTRUCTURE. */
#ifndef HODU_ORACLE_CBLAS_H
#define HODU_ORACLE_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb, int m, int n,
                 int k, float alpha, const float *a, int lda, const float *b, int ldb, float beta,
                 float *c, int ldc);
void cblas_dgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb, int m, int n,
                 int k, double alpha, const double *a, int lda, const double *b, int ldb, double beta,
                 double *c, int ldc);
void openblas_set_num_threads(int n);
int openblas_get_num_threads(void);
#ifdef __cplusplus
}
#endif
#endif
