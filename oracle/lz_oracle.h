/*
 * CPU restatement of Leela Zero's network forward path (TEST INFRASTRUCTURE).
 *
 * This is the checker the CUDA pipe is compared against.  It is never linked
 * into, imported by, or called from the product library; only the test-suite,
 * the smoke check and the CPU-baseline leg of the benchmark load it.
 *
 * Parity pin: the reference ships no golden vectors for this path.  The port
 * is pinned against the reference's own CPUPipe.cpp compiled unchanged (the
 * "_ref" build next to this file) and against committed fixtures that build
 * produced.
 *
 * Each function names the reference file:line it restates.
 */
#ifndef LZ_ORACLE_H
#define LZ_ORACLE_H

#ifdef __cplusplus
extern "C" {
#endif

enum {
    LZO_BOARD = 19,
    LZO_SQ = 361,
    LZO_INPUT_PLANES = 18,
    LZO_WTILES = 5,      /* ceil(19 / 4)            */
    LZO_P = 25,          /* tiles per position      */
    LZO_ALPHA = 6,       /* 4 + 3 - 1               */
    LZO_TILE = 36,       /* alpha * alpha           */
    LZO_POLICY_PLANES = 2,
    LZO_VALUE_PLANES = 1,
    LZO_MOVES = 362,     /* 361 intersections + pass */
    LZO_VALUE_HIDDEN = 256
};

/* src/Network.cpp:151-157 : variance -> 1/sqrt(var + 1e-5), in place. */
void lzo_process_bn_var(float* w, int n);

/* src/Network.cpp:159-223 : f[K][C][3][3] -> U[36][C][K] = (G f G^T)^T-layout. */
void lzo_winograd_transform_f(const float* f, int outputs, int channels, float* U);

/* src/CPUPipe.cpp:63-183 : in[C][19][19] -> V[36][C][25] = B^T d B per tile. */
void lzo_transform_in(const float* in, float* V, int C);

/* src/CPUPipe.cpp:185-210 : M[t][K][25] = U[t]^T (K x C) * V[t] (C x 25). */
void lzo_sgemm36(const float* U, const float* V, float* M, int C, int K);

/* src/CPUPipe.cpp:212-284 : M[36][K][25] -> Y[K][19][19] = A^T m A, clipped. */
void lzo_transform_out(const float* M, float* Y, int K);

/* src/CPUPipe.cpp:352-377 : y = max(0, s*(x-mean) [+ residual]) in place. */
void lzo_batchnorm(int channels, int spatial, float* data, const float* means,
                   const float* invstd, const float* residual);

/* src/CPUPipe.cpp:301-350 with filter_size 1 : out[o][s] = sum_c w[o][c] x[c][s]. */
void lzo_conv1x1(int outputs, int channels, const float* in, const float* w,
                 float* out);

/*
 * Weights as the reference hands them to a pipe
 * (src/ForwardPipe.h:40-54 after src/Network.cpp:540-576).
 */
typedef struct {
    int channels;         /* filters in the tower                           */
    int blocks;           /* residual blocks; conv layers = 1 + 2*blocks    */
    const float* const* U;       /* [1+2B] each [36][C_in][channels]        */
    const float* const* bn_mean; /* [1+2B] each [channels] (bias folded)    */
    const float* const* bn_invstd;
    const float* pol_w;   /* [2][channels] */
    const float* val_w;   /* [1][channels] */
} lzo_tower;

/* src/CPUPipe.cpp:379-428 : one position, in[18*361] -> pol[2*361], val[361]. */
void lzo_forward(const lzo_tower* net, const float* input, float* pol, float* val);

/* Head parameters private to Network (src/Network.h:166-183). */
typedef struct {
    const float* bn_pol_mean;   /* [2]   (bias folded)   */
    const float* bn_pol_invstd; /* [2]                   */
    const float* ip_pol_w;      /* [362][722]            */
    const float* ip_pol_b;      /* [362]                 */
    const float* bn_val_mean;   /* [1]                   */
    const float* bn_val_invstd; /* [1]                   */
    const float* ip1_val_w;     /* [256][361]            */
    const float* ip1_val_b;     /* [256]                 */
    const float* ip2_val_w;     /* [256]                 */
    const float* ip2_val_b;     /* [1]                   */
    float softmax_temp;
} lzo_heads_w;

/*
 * src/Network.cpp:833-851 : raw head planes -> policy[362] (softmax) and
 * winrate = (1 + tanh(v)) / 2.  pol/val are modified in place like the
 * reference does (batchnorm is in place).
 */
void lzo_heads(const lzo_heads_w* h, float* pol, float* val, float* policy_out,
               float* winrate_out);

/* src/Network.cpp:667-690 : L2 distance over policy[361] + pass + winrate. */
float lzo_selfcheck_l2(const float* policy_a, float winrate_a,
                       const float* policy_b, float winrate_b);

#ifdef __cplusplus
}
#endif
#endif
