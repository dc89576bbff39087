// fp32 form of the 36 channel contractions (FFMA on the CUDA cores):
//   M[t][p][k] = sum_c V[t][p][c] * U[t][k][c],   t = 0..35
// Both operands have the reduction axis innermost.  64x64 output tile per CTA,
// 16-wide reduction steps staged through shared memory, 4x4 outputs per thread.
// This is the arithmetic of CPUPipe::winograd_sgemm (src/CPUPipe.cpp:185-210)
// and stands where the reference launches XgemmBatched in single precision
// (src/OpenCL.cpp:404-426); it is the path held to the 1e-4 bound.
#pragma once

namespace lzb {

constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;

// grid (Pa/64, Kp/64, 36), block 256.  Pa, Kp multiples of 64; Cp of 16.
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ V,
                                                       const float* __restrict__ U,
                                                       float* __restrict__ M, int Pa, int Cp,
                                                       int Kp) {
    __shared__ float As[kSimtK][kSimtTile + 4];
    __shared__ float Bs[kSimtK][kSimtTile + 4];
    const int t = blockIdx.z;
    const int p0 = blockIdx.x * kSimtTile, k0 = blockIdx.y * kSimtTile;
    const float* Vt = V + ((size_t)t * Pa + p0) * Cp;
    const float* Ut = U + ((size_t)t * Kp + k0) * Cp;
    const int tid = threadIdx.x;
    const int lrow = tid >> 2, lc4 = (tid & 3) * 4;   // loader: 64 rows x 4 float4
    const int ty = tid >> 4, tx = tid & 15;           // compute: 16 x 16 threads
    float acc[4][4] = {};
    for (int c0 = 0; c0 < Cp; c0 += kSimtK) {
        const float4 a = *reinterpret_cast<const float4*>(Vt + (size_t)lrow * Cp + c0 + lc4);
        const float4 b = *reinterpret_cast<const float4*>(Ut + (size_t)lrow * Cp + c0 + lc4);
        As[lc4 + 0][lrow] = a.x; As[lc4 + 1][lrow] = a.y;
        As[lc4 + 2][lrow] = a.z; As[lc4 + 3][lrow] = a.w;
        Bs[lc4 + 0][lrow] = b.x; Bs[lc4 + 1][lrow] = b.y;
        Bs[lc4 + 2][lrow] = b.z; Bs[lc4 + 3][lrow] = b.w;
        __syncthreads();
#pragma unroll
        for (int c = 0; c < kSimtK; c++) {
            const float4 av = *reinterpret_cast<const float4*>(&As[c][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[c][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* Mt = M + ((size_t)t * Pa + p0 + ty * 4) * Kp + k0 + tx * 4;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        *reinterpret_cast<float4*>(Mt + (size_t)i * Kp) =
            make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
}

}  // namespace lzb
