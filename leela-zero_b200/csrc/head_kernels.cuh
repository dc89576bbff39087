// The network heads after the two 1x1 convolutions, finished on the device:
//   policy: batch-norm + ReLU on 2 planes -> FC 722 -> 362 -> softmax
//   value : batch-norm + ReLU on 1 plane  -> FC 361 -> 256 ReLU -> FC 256 -> 1
//           -> (1 + tanh) / 2
// This is the arithmetic Network::get_output_internal runs on the CPU for every
// evaluation (src/Network.cpp:833-851, innerproduct :609-637, softmax :693-712).
// FC matrices are kept transposed ([in][out]) so that neighbouring threads read
// neighbouring weights.  One CLUSTER per position: the inputs of the first
// fully connected layer are cut into one slice per CTA (a single CTA walking
// all 722 rows of the 1 MB policy matrix took 34 us whatever the batch size);
// the partial sums are written into the first CTA's shared memory
// (st.shared::cluster), which adds them in slice order and finishes the head.
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

constexpr int kPolicySlices = 8;     // CTAs per position in policy_head_kernel
constexpr int kValueSlices = 4;      // ... in value_head_kernel

__device__ __forceinline__ uint32_t head_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// store into the shared memory of CTA 0 of the cluster, at the offset `local` has here
__device__ __forceinline__ void store_to_first_cta(float* local, float v) {
    uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(local)), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(0u));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void head_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// grid kPolicySlices * n (clusters of kPolicySlices), block 384.
// pol[n][2][361] raw planes -> policy[n][362].
__global__ void __cluster_dims__(kPolicySlices, 1, 1) __launch_bounds__(384) policy_head_kernel(
    const float* __restrict__ pol, const float* __restrict__ bn_mean,
    const float* __restrict__ bn_invstd, const float* __restrict__ wT /*[722][362]*/,
    const float* __restrict__ bias, float inv_temp, float* __restrict__ policy) {
    constexpr int kRows = (2 * kSq + kPolicySlices - 1) / kPolicySlices;   // FC inputs per slice
    __shared__ float x[kRows];
    __shared__ float part[kPolicySlices][kMoves];       // used in the first CTA of the cluster
    __shared__ float scratch[12];
    const int n = blockIdx.x / kPolicySlices;
    const int slice = static_cast<int>(head_cluster_rank());
    const int i0 = slice * kRows;
    const int rows = (2 * kSq - i0) < kRows ? (2 * kSq - i0) : kRows;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const int i = i0 + r, c = i / kSq;
        const float v = nf_mul(bn_invstd[c], nf_add(pol[(size_t)n * 2 * kSq + i], -bn_mean[c]));
        x[r] = fmaxf(v, 0.f);
    }
    __syncthreads();
    const int o = threadIdx.x;
    if (o < kMoves) {
        float acc = 0.f;
        const float* w = wT + (size_t)i0 * kMoves + o;
#pragma unroll 4
        for (int r = 0; r < rows; r++) acc = fmaf(w[(size_t)r * kMoves], x[r], acc);
        store_to_first_cta(&part[slice][o], acc);
    }
    __syncthreads();                  // every warp whole again before the aligned cluster barrier
    head_cluster_sync();              // all partial sums are in the first CTA
    if (slice != 0) return;
    float logit = -INFINITY;
    if (o < kMoves) {
        float acc = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < kPolicySlices; s2++) acc += part[s2][o];
        logit = bias[o] + acc;
    }
    const float mx = block_reduce(logit, scratch, true);
    const float e = (o < kMoves) ? expf((logit - mx) * inv_temp) : 0.f;
    const float denom = block_reduce(e, scratch, false);
    if (o < kMoves) policy[(size_t)n * kMoves + o] = e / denom;
}

// grid kValueSlices * n (clusters of kValueSlices), block 256.
// val[n][361] raw plane -> winrate[n].
__global__ void __cluster_dims__(kValueSlices, 1, 1) __launch_bounds__(256) value_head_kernel(
    const float* __restrict__ val, const float* __restrict__ bn_mean,
    const float* __restrict__ bn_invstd, const float* __restrict__ w1T /*[361][256]*/,
    const float* __restrict__ b1, const float* __restrict__ w2, const float* __restrict__ b2,
    float* __restrict__ winrate) {
    constexpr int kRows = (kSq + kValueSlices - 1) / kValueSlices;
    __shared__ float x[kRows];
    __shared__ float part[kValueSlices][kValueHidden];  // used in the first CTA of the cluster
    __shared__ float scratch[8];
    const int n = blockIdx.x / kValueSlices;
    const int slice = static_cast<int>(head_cluster_rank());
    const int i0 = slice * kRows;
    const int rows = (kSq - i0) < kRows ? (kSq - i0) : kRows;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const float v = nf_mul(bn_invstd[0], nf_add(val[(size_t)n * kSq + i0 + r], -bn_mean[0]));
        x[r] = fmaxf(v, 0.f);
    }
    __syncthreads();
    const int j = threadIdx.x;
    {
        float acc = 0.f;
        const float* w = w1T + (size_t)i0 * kValueHidden + j;
#pragma unroll 4
        for (int r = 0; r < rows; r++) acc = fmaf(w[(size_t)r * kValueHidden], x[r], acc);
        store_to_first_cta(&part[slice][j], acc);
    }
    head_cluster_sync();
    if (slice != 0) return;
    float acc = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < kValueSlices; s2++) acc += part[s2][j];
    const float h = fmaxf(b1[j] + acc, 0.f);
    const float s = block_reduce(w2[j] * h, scratch, false);
    if (j == 0) winrate[n] = (1.0f + tanhf(b2[0] + s)) / 2.0f;
}

}  // namespace lzb
