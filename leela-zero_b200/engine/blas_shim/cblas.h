/*
 * CBLAS declarations (ABI only) for building the engine's sources where no
 * cblas.h is installed: the engine calls cblas_sgemm / cblas_sgemv
 * (src/Network.cpp:609-637) and two OpenBLAS set-up routines
 * (src/Network.cpp:496-507).
 */
#ifndef LZB_ENGINE_CBLAS_H
#define LZB_ENGINE_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb, int m,
                 int n, int k, float alpha, const float* a, int lda, const float* b, int ldb,
                 float beta, float* c, int ldc);
void cblas_sgemv(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, int m, int n, float alpha,
                 const float* a, int lda, const float* x, int incx, float beta, float* y, int incy);
void openblas_set_num_threads(int n);
char* openblas_get_corename(void);
#ifdef __cplusplus
}
#endif
#endif
