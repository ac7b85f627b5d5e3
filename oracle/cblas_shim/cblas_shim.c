/* Forwards the CBLAS entry points the reference CPU sources use to the
 * OpenBLAS build bundled with scipy (test infrastructure only). */
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include "cblas.h"

#define API __attribute__((visibility("default")))

static void* g_lib;
static void (*p_sscal)(int, float, float*, int);
static void (*p_saxpy)(int, float, const float*, int, float*, int);
static void (*p_scopy)(int, const float*, int, float*, int);
static float (*p_sdot)(int, const float*, int, const float*, int);
static float (*p_snrm2)(int, const float*, int);
static float (*p_sasum)(int, const float*, int);
static void (*p_sgemm)(int, int, int, int, int, int, float, const float*, int, const float*, int,
                       float, float*, int);
static void (*p_set_threads)(int);
static int (*p_get_threads)(void);

static void need(void)
{
    if (!g_lib) { fprintf(stderr, "pxref: pxref_blas_init() was not called\n"); abort(); }
}

API int pxref_blas_init(const char* path)
{
    if (g_lib) return 0;
    void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) { fprintf(stderr, "pxref: dlopen(%s): %s\n", path, dlerror()); return 1; }
    *(void**)&p_sscal = dlsym(h, "scipy_cblas_sscal");
    *(void**)&p_saxpy = dlsym(h, "scipy_cblas_saxpy");
    *(void**)&p_scopy = dlsym(h, "scipy_cblas_scopy");
    *(void**)&p_sdot = dlsym(h, "scipy_cblas_sdot");
    *(void**)&p_snrm2 = dlsym(h, "scipy_cblas_snrm2");
    *(void**)&p_sasum = dlsym(h, "scipy_cblas_sasum");
    *(void**)&p_sgemm = dlsym(h, "scipy_cblas_sgemm");
    *(void**)&p_set_threads = dlsym(h, "scipy_openblas_set_num_threads");
    *(void**)&p_get_threads = dlsym(h, "scipy_openblas_get_num_threads");
    if (!p_sscal || !p_saxpy || !p_scopy || !p_sdot || !p_snrm2 || !p_sgemm) return 2;
    g_lib = h;
    return 0;
}

API int pxref_blas_set_threads(int n)
{
    need();
    if (p_set_threads && n > 0) p_set_threads(n);
    return p_get_threads ? p_get_threads() : -1;
}

API void* pxref_blas_sgemm_ptr(void) { need(); return *(void**)&p_sgemm; }

void cblas_sscal(int n, float a, float* x, int ix) { need(); p_sscal(n, a, x, ix); }
void cblas_saxpy(int n, float a, const float* x, int ix, float* y, int iy) { need(); p_saxpy(n, a, x, ix, y, iy); }
void cblas_scopy(int n, const float* x, int ix, float* y, int iy) { need(); p_scopy(n, x, ix, y, iy); }
float cblas_sdot(int n, const float* x, int ix, const float* y, int iy) { need(); return p_sdot(n, x, ix, y, iy); }
float cblas_snrm2(int n, const float* x, int ix) { need(); return p_snrm2(n, x, ix); }
float cblas_sasum(int n, const float* x, int ix) { need(); return p_sasum ? p_sasum(n, x, ix) : 0.0f; }
void cblas_sgemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                 const float* a, int lda, const float* b, int ldb, float beta, float* c, int ldc)
{
    need();
    p_sgemm((int)o, (int)ta, (int)tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}
