// The network heads after the two 1x1 convolutions, finished on the device:
//   policy: batch-norm + ReLU on 2 planes -> FC 722 -> 362 -> softmax
//   value : batch-norm + ReLU on 1 plane  -> FC 361 -> 256 ReLU -> FC 256 -> 1
//           -> (1 + tanh) / 2
// This is the arithmetic Network::get_output_internal runs on the CPU for every
// evaluation (src/Network.cpp:833-851, innerproduct :609-637, softmax :693-712).
// FC matrices are kept transposed ([in][out]) so that neighbouring threads read
// neighbouring weights.  One CTA per position.
#pragma once
#include "winograd_math.cuh"

namespace lzb {

constexpr int kMoves = 362;
constexpr int kValueHidden = 256;

__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, off);
        v = is_max ? fmaxf(v, o) : v + o;
    }
    __syncthreads();               // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
    for (int i = 1; i < nw; i++) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
    return r;
}

// grid n, block 384.  pol[n][2][361] raw planes -> policy[n][362].
__global__ void __launch_bounds__(384) policy_head_kernel(
    const float* __restrict__ pol, const float* __restrict__ bn_mean,
    const float* __restrict__ bn_invstd, const float* __restrict__ wT /*[722][362]*/,
    const float* __restrict__ bias, float inv_temp, float* __restrict__ policy) {
    __shared__ float x[2 * kSq];
    __shared__ float scratch[12];
    const int n = blockIdx.x;
    for (int i = threadIdx.x; i < 2 * kSq; i += blockDim.x) {
        const int c = i / kSq;
        const float v = nf_mul(bn_invstd[c], nf_add(pol[(size_t)n * 2 * kSq + i], -bn_mean[c]));
        x[i] = fmaxf(v, 0.f);
    }
    __syncthreads();
    const int o = threadIdx.x;
    float logit = -INFINITY;
    if (o < kMoves) {
        float acc = 0.f;
        for (int i = 0; i < 2 * kSq; i++) acc = fmaf(wT[(size_t)i * kMoves + o], x[i], acc);
        logit = bias[o] + acc;
    }
    const float mx = block_reduce(logit, scratch, true);
    const float e = (o < kMoves) ? expf((logit - mx) * inv_temp) : 0.f;
    const float denom = block_reduce(e, scratch, false);
    if (o < kMoves) policy[(size_t)n * kMoves + o] = e / denom;
}

// grid n, block 256.  val[n][361] raw plane -> winrate[n].
__global__ void __launch_bounds__(256) value_head_kernel(
    const float* __restrict__ val, const float* __restrict__ bn_mean,
    const float* __restrict__ bn_invstd, const float* __restrict__ w1T /*[361][256]*/,
    const float* __restrict__ b1, const float* __restrict__ w2, const float* __restrict__ b2,
    float* __restrict__ winrate) {
    __shared__ float x[kSq];
    __shared__ float scratch[8];
    const int n = blockIdx.x;
    for (int i = threadIdx.x; i < kSq; i += blockDim.x) {
        const float v = nf_mul(bn_invstd[0], nf_add(val[(size_t)n * kSq + i], -bn_mean[0]));
        x[i] = fmaxf(v, 0.f);
    }
    __syncthreads();
    const int j = threadIdx.x;
    float acc = 0.f;
    for (int i = 0; i < kSq; i++) acc = fmaf(w1T[(size_t)i * kValueHidden + j], x[i], acc);
    const float h = fmaxf(b1[j] + acc, 0.f);
    const float s = block_reduce(w2[j] * h, scratch, false);
    if (j == 0) winrate[n] = (1.0f + tanhf(b2[0] + s)) / 2.0f;
}

}  // namespace lzb
