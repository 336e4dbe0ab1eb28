/* TEST INFRASTRUCTURE. Minimal prototype of the one CBLAS routine the
 * reference's BLAS build calls on this path (cblas_sgemm), so that the
 * reference sources compile against an OpenBLAS binary that ships without
 * headers. Enumerator values follow the published CBLAS interface. */
#ifndef ORACLE_CBLAS_SHIM_H
#define ORACLE_CBLAS_SHIM_H
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb,
                 int m, int n, int k, float alpha, const float *a, int lda,
                 const float *b, int ldb, float beta, float *c, int ldc);
void openblas_set_num_threads(int n);
int openblas_get_num_threads(void);
#endif
