/*
 * CPU restatement of Leela Zero's network forward path (TEST INFRASTRUCTURE,
 * see lz_oracle.h).  Plain C99, single thread, no BLAS: the GEMMs are written
 * as loops, so sums are accumulated in a different order than OpenBLAS does
 * (differences are of the order of 1e-6 relative).
 *
 * The arithmetic follows the reference's factored forms operation by
 * operation so that, compiled without -ffast-math, it reproduces CPUPipe's
 * transform values exactly.
 */
#include "lz_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define SQ2 1.4142135623730951f

/* ---- weight preparation ------------------------------------------------ */

void lzo_process_bn_var(float* w, int n) {
    /* src/Network.cpp:151-157 */
    const float epsilon = 1e-5f;
    for (int i = 0; i < n; i++) {
        w[i] = 1.0f / sqrtf(w[i] + epsilon);
    }
}

void lzo_winograd_transform_f(const float* f, int outputs, int channels,
                              float* U) {
    /* src/Network.cpp:159-223.  G is 6x3; U[xi*6+nu][c][o] = (G f G^T)[xi][nu].
     * The reference accumulates "acc += G*f" left to right starting from 0. */
    static const float G[6][3] = {
        {1.0f, 0.0f, 0.0f},
        {-2.0f / 3.0f, -SQ2 / 3.0f, -1.0f / 3.0f},
        {-2.0f / 3.0f, SQ2 / 3.0f, -1.0f / 3.0f},
        {1.0f / 6.0f, SQ2 / 6.0f, 1.0f / 3.0f},
        {1.0f / 6.0f, -SQ2 / 6.0f, 1.0f / 3.0f},
        {0.0f, 0.0f, 1.0f}};
    for (int c = 0; c < channels; c++) {
        for (int o = 0; o < outputs; o++) {
            const float* flt = f + ((size_t)o * channels + c) * 9;
            float gf[6][3];
            for (int i = 0; i < 6; i++) {
                for (int j = 0; j < 3; j++) {
                    float acc = 0.0f;
                    for (int k = 0; k < 3; k++) {
                        acc += G[i][k] * flt[k * 3 + j];
                    }
                    gf[i][j] = acc;
                }
            }
            for (int xi = 0; xi < 6; xi++) {
                for (int nu = 0; nu < 6; nu++) {
                    float acc = 0.0f;
                    for (int k = 0; k < 3; k++) {
                        acc += gf[xi][k] * G[nu][k];
                    }
                    U[((size_t)(xi * 6 + nu) * channels + c) * outputs + o] = acc;
                }
            }
        }
    }
}

/* ---- Winograd input transform ----------------------------------------- */

/* One application of B^T to a 6-vector, in the reference's factored order
 * (src/CPUPipe.cpp:88-106). */
static void apply_bt(float o[6], const float i[6]) {
    float a = i[1] * -SQ2 + i[3] * (SQ2 / 2.0f);
    float b = i[2] * -2.0f + i[4] * 1.0f;
    o[0] = i[0] + i[2] * (-5.0f / 2.0f) + i[4];
    o[1] = a + b;
    o[2] = -a + b;
    float a2 = i[3] * (SQ2) + i[1] * (-SQ2 / 2.0f);
    float b2 = i[2] * (-1.0f / 2.0f) + i[4];
    o[3] = a2 + b2;
    o[4] = -a2 + b2;
    o[5] = i[1] + i[3] * (-5.0f / 2.0f) + i[5];
}

void lzo_transform_in(const float* in, float* V, int C) {
    /* src/CPUPipe.cpp:63-183.  Board padded by one zero ring (22x22 covers the
     * 25 overlapping 6x6 tiles with stride 4). */
    enum { PAD = 2 + 4 * LZO_WTILES };
    float pad[PAD][PAD];
    for (int ch = 0; ch < C; ch++) {
        memset(pad, 0, sizeof(pad));
        for (int y = 0; y < LZO_BOARD; y++) {
            for (int x = 0; x < LZO_BOARD; x++) {
                pad[y + 1][x + 1] = in[(size_t)ch * LZO_SQ + y * LZO_BOARD + x];
            }
        }
        for (int by = 0; by < LZO_WTILES; by++) {
            for (int bx = 0; bx < LZO_WTILES; bx++) {
                const int y0 = 4 * by, x0 = 4 * bx;
                /* T1[.][col] = B^T * column col of the patch */
                float t1[6][6];
                for (int col = 0; col < 6; col++) {
                    float vin[6], vout[6];
                    for (int r = 0; r < 6; r++) vin[r] = pad[y0 + r][x0 + col];
                    apply_bt(vout, vin);
                    for (int r = 0; r < 6; r++) t1[r][col] = vout[r];
                }
                /* V[xi][.] = B^T * row xi of T1 (i.e. T1 * B) */
                const int tile = by * LZO_WTILES + bx;
                for (int xi = 0; xi < 6; xi++) {
                    float vout[6];
                    apply_bt(vout, t1[xi]);
                    for (int nu = 0; nu < 6; nu++) {
                        V[((size_t)(xi * 6 + nu) * C + ch) * LZO_P + tile] = vout[nu];
                    }
                }
            }
        }
    }
}

/* ---- 36 channel contractions ------------------------------------------ */

void lzo_sgemm36(const float* U, const float* V, float* M, int C, int K) {
    /* src/CPUPipe.cpp:185-210 : row-major sgemm(Trans, NoTrans, K, P, C,
     * U[t] with lda = K, V[t] with ldb = P) -> M[t] (K x P). */
    for (int t = 0; t < LZO_TILE; t++) {
        const float* u = U + (size_t)t * C * K;
        const float* v = V + (size_t)t * C * LZO_P;
        float* m = M + (size_t)t * K * LZO_P;
        memset(m, 0, sizeof(float) * (size_t)K * LZO_P);
        for (int c = 0; c < C; c++) {
            const float* vrow = v + (size_t)c * LZO_P;
            const float* urow = u + (size_t)c * K;
            for (int k = 0; k < K; k++) {
                const float uk = urow[k];
                float* mrow = m + (size_t)k * LZO_P;
                for (int p = 0; p < LZO_P; p++) {
                    mrow[p] += uk * vrow[p];
                }
            }
        }
    }
}

/* ---- Winograd output transform ---------------------------------------- */

/* One application of A^T to a 6-vector (src/CPUPipe.cpp:225-238). */
static void apply_at(float o[4], const float i[6]) {
    float t1p2 = (i[1] + i[2]) * (1.0f / 2.0f);
    float t1m2 = (i[1] - i[2]) * (SQ2 / 4.0f);
    float t3p4 = i[3] + i[4];
    float t3m4 = (i[3] - i[4]) * (SQ2);
    o[0] = i[0] + t1p2 + t1p2 + t3p4;
    o[1] = t1m2 + t1m2 + t3m4;
    o[2] = t1p2 + t3p4 + t3p4;
    o[3] = t1m2 + t3m4 + t3m4 + i[5];
}

void lzo_transform_out(const float* M, float* Y, int K) {
    /* src/CPUPipe.cpp:212-284 */
    for (int k = 0; k < K; k++) {
        for (int by = 0; by < LZO_WTILES; by++) {
            for (int bx = 0; bx < LZO_WTILES; bx++) {
                const int tile = by * LZO_WTILES + bx;
                float m[6][6];
                for (int xi = 0; xi < 6; xi++) {
                    for (int nu = 0; nu < 6; nu++) {
                        m[xi][nu] =
                            M[((size_t)(xi * 6 + nu) * K + k) * LZO_P + tile];
                    }
                }
                /* temp[i][j] = sum_xi At[i][xi] m[xi][j] */
                float temp[4][6];
                for (int j = 0; j < 6; j++) {
                    float colv[6], o4[4];
                    for (int xi = 0; xi < 6; xi++) colv[xi] = m[xi][j];
                    apply_at(o4, colv);
                    for (int i = 0; i < 4; i++) temp[i][j] = o4[i];
                }
                for (int i = 0; i < 4; i++) {
                    float o4[4];
                    apply_at(o4, temp[i]);
                    const int y = 4 * by + i;
                    if (y >= LZO_BOARD) continue;
                    for (int j = 0; j < 4; j++) {
                        const int x = 4 * bx + j;
                        if (x < LZO_BOARD) {
                            Y[(size_t)k * LZO_SQ + y * LZO_BOARD + x] = o4[j];
                        }
                    }
                }
            }
        }
    }
}

/* ---- batch norm, 1x1 convolution -------------------------------------- */

void lzo_batchnorm(int channels, int spatial, float* data, const float* means,
                   const float* invstd, const float* residual) {
    /* src/CPUPipe.cpp:352-377 (same code as src/Network.cpp:639-664) */
    for (int c = 0; c < channels; c++) {
        float* arr = data + (size_t)c * spatial;
        const float mean = means[c], s = invstd[c];
        if (!residual) {
            for (int b = 0; b < spatial; b++) {
                float v = s * (arr[b] - mean);
                arr[b] = v > 0.0f ? v : 0.0f;
            }
        } else {
            const float* res = residual + (size_t)c * spatial;
            for (int b = 0; b < spatial; b++) {
                float v = (s * (arr[b] - mean)) + res[b];
                arr[b] = v > 0.0f ? v : 0.0f;
            }
        }
    }
}

void lzo_conv1x1(int outputs, int channels, const float* in, const float* w,
                 float* out) {
    /* src/CPUPipe.cpp:301-350 with filter_size 1: im2col is a copy
     * (src/Im2Col.h:82-88); the biases the pipe adds are all zero
     * (src/CPUPipe.cpp:437-441). */
    for (int o = 0; o < outputs; o++) {
        float* dst = out + (size_t)o * LZO_SQ;
        for (int s = 0; s < LZO_SQ; s++) dst[s] = 0.0f;
        for (int c = 0; c < channels; c++) {
            const float wc = w[(size_t)o * channels + c];
            const float* src = in + (size_t)c * LZO_SQ;
            for (int s = 0; s < LZO_SQ; s++) dst[s] += wc * src[s];
        }
    }
}

/* ---- the tower -------------------------------------------------------- */

static void conv3(const float* in, const float* U, float* V, float* M,
                  float* out, int C, int K) {
    /* src/CPUPipe.cpp:286-299 */
    lzo_transform_in(in, V, C);
    lzo_sgemm36(U, V, M, C, K);
    lzo_transform_out(M, out, K);
}

void lzo_forward(const lzo_tower* net, const float* input, float* pol,
                 float* val) {
    /* src/CPUPipe.cpp:379-428 */
    const int C = net->channels;
    const int maxc = C > LZO_INPUT_PLANES ? C : LZO_INPUT_PLANES;
    float* V = (float*)malloc(sizeof(float) * LZO_TILE * maxc * LZO_P);
    float* M = (float*)malloc(sizeof(float) * LZO_TILE * C * LZO_P);
    float* x = (float*)malloc(sizeof(float) * C * LZO_SQ);   /* block input  */
    float* h = (float*)malloc(sizeof(float) * C * LZO_SQ);   /* first conv   */
    float* y = (float*)malloc(sizeof(float) * C * LZO_SQ);   /* block output */

    conv3(input, net->U[0], V, M, x, LZO_INPUT_PLANES, C);
    lzo_batchnorm(C, LZO_SQ, x, net->bn_mean[0], net->bn_invstd[0], NULL);

    for (int b = 0; b < net->blocks; b++) {
        const int l1 = 1 + 2 * b, l2 = l1 + 1;
        conv3(x, net->U[l1], V, M, h, C, C);
        lzo_batchnorm(C, LZO_SQ, h, net->bn_mean[l1], net->bn_invstd[l1], NULL);
        conv3(h, net->U[l2], V, M, y, C, C);
        lzo_batchnorm(C, LZO_SQ, y, net->bn_mean[l2], net->bn_invstd[l2], x);
        float* tmp = x; x = y; y = tmp;
    }
    lzo_conv1x1(LZO_POLICY_PLANES, C, x, net->pol_w, pol);
    lzo_conv1x1(LZO_VALUE_PLANES, C, x, net->val_w, val);

    free(V); free(M); free(x); free(h); free(y);
}

/* ---- heads ------------------------------------------------------------ */

static void innerproduct(int inputs, int outputs, int relu, const float* in,
                         const float* w, const float* b, float* out) {
    /* src/Network.cpp:609-637 : row-major sgemv then bias (+ReLU). */
    for (int o = 0; o < outputs; o++) {
        float acc = 0.0f;
        const float* row = w + (size_t)o * inputs;
        for (int i = 0; i < inputs; i++) acc += row[i] * in[i];
        float v = b[o] + acc;
        if (relu && v < 0.0f) v = 0.0f;
        out[o] = v;
    }
}

void lzo_heads(const lzo_heads_w* h, float* pol, float* val, float* policy_out,
               float* winrate_out) {
    /* src/Network.cpp:833-851 */
    lzo_batchnorm(LZO_POLICY_PLANES, LZO_SQ, pol, h->bn_pol_mean,
                  h->bn_pol_invstd, NULL);
    float logits[LZO_MOVES];
    innerproduct(LZO_POLICY_PLANES * LZO_SQ, LZO_MOVES, 0, pol, h->ip_pol_w,
                 h->ip_pol_b, logits);
    /* softmax, src/Network.cpp:693-712 */
    float alpha = logits[0];
    for (int i = 1; i < LZO_MOVES; i++) if (logits[i] > alpha) alpha = logits[i];
    float denom = 0.0f;
    for (int i = 0; i < LZO_MOVES; i++) {
        float e = expf((logits[i] - alpha) / h->softmax_temp);
        denom += e;
        policy_out[i] = e;
    }
    for (int i = 0; i < LZO_MOVES; i++) policy_out[i] /= denom;

    lzo_batchnorm(LZO_VALUE_PLANES, LZO_SQ, val, h->bn_val_mean,
                  h->bn_val_invstd, NULL);
    float hidden[LZO_VALUE_HIDDEN];
    innerproduct(LZO_SQ, LZO_VALUE_HIDDEN, 1, val, h->ip1_val_w, h->ip1_val_b,
                 hidden);
    float out1;
    innerproduct(LZO_VALUE_HIDDEN, 1, 0, hidden, h->ip2_val_w, h->ip2_val_b,
                 &out1);
    *winrate_out = (1.0f + tanhf(out1)) / 2.0f;
}

float lzo_selfcheck_l2(const float* policy_a, float winrate_a,
                       const float* policy_b, float winrate_b) {
    /* src/Network.cpp:667-690 : policy[361], then pass, then winrate. */
    float error = 0.0f;
    for (int i = 0; i < LZO_MOVES; i++) {
        float d = policy_a[i] - policy_b[i];
        error += d * d;
    }
    float dw = winrate_a - winrate_b;
    error += dw * dw;
    return sqrtf(error);
}
