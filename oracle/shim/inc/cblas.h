/* Test infrastructure (oracle build only): a minimal CBLAS declaration set so the reference's CPU driver
 * can be compiled without a system BLAS.  The symbols are bound to the LP64 OpenBLAS that ships inside
 * the scipy wheel, whose exports carry a "scipy_" prefix.  Only the routines the reference driver calls
 * are declared. */
#ifndef CCT_ORACLE_SHIM_CBLAS_H
#define CCT_ORACLE_SHIM_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
#define cblas_sgemm scipy_cblas_sgemm
#define cblas_sgemv scipy_cblas_sgemv
#define cblas_saxpy scipy_cblas_saxpy
#define cblas_saxpby scipy_cblas_saxpby
#define cblas_sscal scipy_cblas_sscal
#define cblas_scopy scipy_cblas_scopy
#define cblas_sdot scipy_cblas_sdot
#define openblas_set_num_threads scipy_openblas_set_num_threads
#define openblas_get_config scipy_openblas_get_config
void cblas_sgemm(enum CBLAS_ORDER, enum CBLAS_TRANSPOSE, enum CBLAS_TRANSPOSE, int m, int n, int k, float alpha,
                 const float* a, int lda, const float* b, int ldb, float beta, float* c, int ldc);
void cblas_sgemv(enum CBLAS_ORDER, enum CBLAS_TRANSPOSE, int m, int n, float alpha, const float* a, int lda,
                 const float* x, int incx, float beta, float* y, int incy);
void cblas_saxpy(int n, float alpha, const float* x, int incx, float* y, int incy);
void cblas_saxpby(int n, float alpha, const float* x, int incx, float beta, float* y, int incy);
void cblas_sscal(int n, float alpha, float* x, int incx);
void cblas_scopy(int n, const float* x, int incx, float* y, int incy);
float cblas_sdot(int n, const float* x, int incx, const float* y, int incy);
void openblas_set_num_threads(int n);
char* openblas_get_config(void);
#ifdef __cplusplus
}
#endif
#endif
