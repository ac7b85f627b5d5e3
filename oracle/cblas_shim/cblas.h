/*
 * Minimal <cblas.h> stand-in used only to compile the reference's CPU sources
 * (test infrastructure).  OpenBLAS headers are not installed in this image;
 * the OpenBLAS binary that ships inside scipy is, with its symbols prefixed
 * "scipy_".  cblas_shim.c forwards these entry points to that binary, which is
 * opened at run time by pxref_blas_init().
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
typedef CBLAS_ORDER CBLAS_LAYOUT;

void cblas_sscal(int n, float alpha, float* x, int incx);
void cblas_saxpy(int n, float alpha, const float* x, int incx, float* y, int incy);
void cblas_scopy(int n, const float* x, int incx, float* y, int incy);
float cblas_sdot(int n, const float* x, int incx, const float* y, int incy);
float cblas_snrm2(int n, const float* x, int incx);
float cblas_sasum(int n, const float* x, int incx);
void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
                 float alpha, const float* a, int lda, const float* b, int ldb, float beta,
                 float* c, int ldc);

/* Opens the OpenBLAS shared object at `path` (symbols scipy_cblas_*); returns 0 on success. */
int pxref_blas_init(const char* path);
/* Sets the OpenBLAS thread count; returns the value now in effect (or -1). */
int pxref_blas_set_threads(int n);
/* Address of the resolved sgemm, for callers that take a function pointer. */
void* pxref_blas_sgemm_ptr(void);

#ifdef __cplusplus
}
#endif
