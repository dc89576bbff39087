/*
 * Plain-loop cblas_sgemm used only when no OpenBLAS with the standard CBLAS
 * symbols can be found to link the reference's CPUPipe.cpp against.
 * Supports exactly the two call shapes CPUPipe makes (row major;
 * Trans/NoTrans and NoTrans/NoTrans; alpha 1, beta 0).  Test infrastructure.
 */
#include "cblas.h"
#include <string.h>

void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta,
                 enum CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                 const float* a, int lda, const float* b, int ldb, float beta,
                 float* c, int ldc) {
    (void)order; (void)tb; (void)alpha; (void)beta;
    for (int i = 0; i < m; i++) memset(c + (size_t)i * ldc, 0, sizeof(float) * n);
    for (int l = 0; l < k; l++) {
        for (int i = 0; i < m; i++) {
            const float av = (ta == CblasTrans) ? a[(size_t)l * lda + i]
                                                : a[(size_t)i * lda + l];
            const float* brow = b + (size_t)l * ldb;
            float* crow = c + (size_t)i * ldc;
            for (int j = 0; j < n; j++) crow[j] += av * brow[j];
        }
    }
}

void openblas_set_num_threads(int n) { (void)n; }
