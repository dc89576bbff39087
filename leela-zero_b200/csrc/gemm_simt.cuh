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

namespace lzb {

// The same contraction with larger tiles, for the whole-network path: 128 rows
// p by BN (128 or 64) output channels per CTA, 8 x (BN / 16) outputs per
// thread held as 4 x 4 blocks, 16-wide reduction steps.  The next step's
// operands travel from global memory into registers while the current step is
// computed from shared memory, and land in the other of two shared-memory
// buffers: one __syncthreads per step.  Per reduction element a thread issues
// 2 + BN / 64 128-bit shared-memory loads for 8 * BN / 16 FFMAs (the 64 x 64
// kernel above: 2 for 16), which is what lifts it from 45 % towards the FFMA
// peak.  Every output still sums its products in ascending channel order.
constexpr int kSimtBigM = 128;

// Persistent: grid = CTAs resident at once (two per SM); a CTA walks tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... of the row_tiles x Kp / BN x 36 tiles
// (channel tile fastest, then rows, then the Winograd point), and the operand
// pipeline runs on across tile boundaries: the first step of the next tile is
// fetched while the last step of the current one is computed, so the 16 steps
// of a tile (Cp = 256) are not followed by an empty pipeline.
// Pa multiple of 128, Kp of BN, Cp of 16.
template <int BN>
__global__ void __launch_bounds__(256, 2) gemm_f32_big_kernel(const float* __restrict__ V,
                                                              const float* __restrict__ U,
                                                              float* __restrict__ M, int Pa, int Cp,
                                                              int Kp, int row_tiles) {
    constexpr int BM = kSimtBigM, BK = kSimtK;
    constexpr int NB = BN / 64;                 // 4-column blocks per thread along the channels
    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN + 4];
    const int col_tiles = Kp / BN;
    const int ntiles = row_tiles * col_tiles * 36;
    const int tid = threadIdx.x;
    const int lrow = tid >> 2, lc4 = (tid & 3) * 4;   // loader: 64 rows x 4 float4 per pass
    const int ty = tid >> 4, tx = tid & 15;           // compute: 16 x 16 threads
    float acc[2][NB][4][4] = {};
    float4 a_next[2], b_next[NB];

    auto fetch = [&](int tile, int c0) {
        const int kb = tile % col_tiles, rest = tile / col_tiles;
        const int pb = rest % row_tiles, t = rest / row_tiles;
        const float* Vt = V + ((size_t)t * Pa + pb * BM) * Cp;
        const float* Ut = U + ((size_t)t * Kp + kb * BN) * Cp;
#pragma unroll
        for (int h = 0; h < 2; h++)
            a_next[h] = *reinterpret_cast<const float4*>(Vt + (size_t)(lrow + 64 * h) * Cp + c0 + lc4);
#pragma unroll
        for (int h = 0; h < NB; h++)
            b_next[h] = *reinterpret_cast<const float4*>(Ut + (size_t)(lrow + 64 * h) * Cp + c0 + lc4);
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            As[buf][lc4 + 0][lrow + 64 * h] = a_next[h].x;
            As[buf][lc4 + 1][lrow + 64 * h] = a_next[h].y;
            As[buf][lc4 + 2][lrow + 64 * h] = a_next[h].z;
            As[buf][lc4 + 3][lrow + 64 * h] = a_next[h].w;
        }
#pragma unroll
        for (int h = 0; h < NB; h++) {
            Bs[buf][lc4 + 0][lrow + 64 * h] = b_next[h].x;
            Bs[buf][lc4 + 1][lrow + 64 * h] = b_next[h].y;
            Bs[buf][lc4 + 2][lrow + 64 * h] = b_next[h].z;
            Bs[buf][lc4 + 3][lrow + 64 * h] = b_next[h].w;
        }
    };

    int tile = blockIdx.x;
    if (tile >= ntiles) return;
    fetch(tile, 0);
    stash(0);
    __syncthreads();
    int buf = 0;
    while (true) {
        const int next_tile = tile + gridDim.x;
        for (int c0 = 0; c0 < Cp; c0 += BK) {
            const bool last_step = c0 + BK >= Cp;
            const bool more = !last_step || next_tile < ntiles;
            if (!last_step) fetch(tile, c0 + BK);
            else if (next_tile < ntiles) fetch(next_tile, 0);
#pragma unroll
            for (int c = 0; c < BK; c++) {
                float ar[2][4], br[NB][4];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float4 v = *reinterpret_cast<const float4*>(&As[buf][c][ty * 4 + 64 * h]);
                    ar[h][0] = v.x; ar[h][1] = v.y; ar[h][2] = v.z; ar[h][3] = v.w;
                }
#pragma unroll
                for (int h = 0; h < NB; h++) {
                    const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][c][tx * 4 + 64 * h]);
                    br[h][0] = v.x; br[h][1] = v.y; br[h][2] = v.z; br[h][3] = v.w;
                }
#pragma unroll
                for (int hi = 0; hi < 2; hi++)
#pragma unroll
                    for (int hj = 0; hj < NB; hj++)
#pragma unroll
                        for (int i = 0; i < 4; i++)
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                acc[hi][hj][i][j] = fmaf(ar[hi][i], br[hj][j], acc[hi][hj][i][j]);
            }
            if (more) {
                stash(buf ^ 1);       // nobody reads that buffer: its readers passed the last barrier
                __syncthreads();
                buf ^= 1;
            }
        }
        {
            const int kb = tile % col_tiles, rest = tile / col_tiles;
            const int pb = rest % row_tiles, t = rest / row_tiles;
#pragma unroll
            for (int hi = 0; hi < 2; hi++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float* row = M + ((size_t)t * Pa + pb * BM + ty * 4 + 64 * hi + i) * Kp + kb * BN + tx * 4;
#pragma unroll
                    for (int hj = 0; hj < NB; hj++) {
                        *reinterpret_cast<float4*>(row + 64 * hj) = make_float4(
                            acc[hi][hj][i][0], acc[hi][hj][i][1], acc[hi][hj][i][2], acc[hi][hj][i][3]);
#pragma unroll
                        for (int j = 0; j < 4; j++) acc[hi][hj][i][j] = 0.f;
                    }
                }
        }
        if (next_tile >= ntiles) break;
        tile = next_tile;
    }
}

}  // namespace lzb
