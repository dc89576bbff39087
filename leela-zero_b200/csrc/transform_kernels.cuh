// Transform kernels of the residual tower (everything except the 36 channel
// contractions).  All of them are bandwidth work: coalesced along the channel
// axis, which is innermost in every device tensor.
//
// Device layouts (T = float, __half or __nv_bfloat16; Cp = channels rounded up
// to a multiple of 64, extra channels are zero):
//   activations  X[n][361][Cp]        (board cell major, channel minor)
//   V[36][Pa][Cp]   transformed input tiles,  row p = position * 25 + tile
//   M[36][Pa][Cp]   contraction results, same row index
// Pa = rows allocated (a multiple of 128).
//
// They replace the reference's in_transform / out_transform_fused_bn /
// out_transform_fused_bn_in OpenCL kernels (src/kernels/convolve3.opencl:109-452)
// and follow the arithmetic of src/CPUPipe.cpp:63-183, 212-284, 352-377.
#pragma once
#include "winograd_math.cuh"

namespace lzb {

constexpr int kBoardPad = 22;                 // 2 + 4 * 5 : cells -1 .. 20
constexpr int kBoardCells = kBoardPad * kBoardPad;
constexpr int kXformWarps = 8;
constexpr int kXformThreads = kXformWarps * 32;
// The fused transform runs one warp per tile in the 16-bit modes (25 warps: all
// 25 tiles of a position have their loads in flight at once; the kernel is
// bound by L2 latency, not by arithmetic) and 8 warps in fp32, whose 124 KB
// board leaves room for one CTA per SM anyway.
template <typename T> struct XformShape { static constexpr int warps = 25; static constexpr int ctas = 1; };
template <> struct XformShape<float> { static constexpr int warps = 8; static constexpr int ctas = 1; };
constexpr int kChanPerCta = 64;               // one warp covers 32 channel pairs

// B^T d B of the 6x6 patch of tile (by, bx), read from a zero-haloed board in
// shared memory, written to V rows of point t = xi*6 + nu.
template <typename T>
__device__ __forceinline__ void tile_in_transform(const float2* board,
                                                  int lane, int by, int bx,
                                                  T* V, size_t v_row_stride_pts,
                                                  size_t v_off) {
    using P2 = Pair<T>;
    float2 t1[6][6];
#pragma unroll
    for (int col = 0; col < 6; col++) {
        float2 vin[6], vout[6];
#pragma unroll
        for (int r = 0; r < 6; r++) {
            vin[r] = board[((4 * by + r) * kBoardPad + 4 * bx + col) * 32 + lane];
        }
        apply_bt<Pair<T>::exact>(vout, vin);
#pragma unroll
        for (int r = 0; r < 6; r++) t1[r][col] = vout[r];
    }
#pragma unroll
    for (int xi = 0; xi < 6; xi++) {
        float2 vout[6];
        apply_bt<Pair<T>::exact>(vout, t1[xi]);
#pragma unroll
        for (int nu = 0; nu < 6; nu++) {
            auto* dst = reinterpret_cast<typename P2::type*>(
                V + (size_t)(xi * 6 + nu) * v_row_stride_pts + v_off);
            *dst = P2::from_f2(vout[nu]);
        }
    }
}

__device__ __forceinline__ void zero_halo(float2* board, int warp, int lane, int nwarps) {
    for (int cell = warp; cell < kBoardCells; cell += nwarps) {
        const int r = cell / kBoardPad, c = cell % kBoardPad;
        if (r == 0 || r > kBoard || c == 0 || c > kBoard) {
            board[cell * 32 + lane] = make_float2(0.f, 0.f);
        }
    }
}

// ---------------------------------------------------------------------------
// Input planes of the network: in[n][18][361] fp32 (as the engine builds them,
// src/Network.cpp:935-966) -> V[36][Pa][64], channels 18..63 zero.
// One warp per tile, one lane per channel pair.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) first_in_transform_kernel(
    const float* __restrict__ in, T* __restrict__ V, int Pa, int P) {
    using P2 = Pair<T>;
    const int lane = threadIdx.x & 31;
    const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (p >= P) return;
    const int n = p / kTilesPerPos, tile = p % kTilesPerPos;
    const int by = tile / kTilesPerSide, bx = tile % kTilesPerSide;
    const int c0 = 2 * lane;
    const bool live = c0 < kInputPlanes;   // 18 is even: pairs never straddle
    const float* pl0 = in + ((size_t)n * kInputPlanes + (live ? c0 : 0)) * kSq;
    const float* pl1 = pl0 + kSq;

    float2 t1[6][6];
#pragma unroll
    for (int col = 0; col < 6; col++) {
        float2 vin[6], vout[6];
        const int x = 4 * bx - 1 + col;
#pragma unroll
        for (int r = 0; r < 6; r++) {
            const int y = 4 * by - 1 + r;
            const bool inside = live && x >= 0 && x < kBoard && y >= 0 && y < kBoard;
            vin[r] = inside ? make_float2(pl0[y * kBoard + x], pl1[y * kBoard + x])
                            : make_float2(0.f, 0.f);
        }
        apply_bt<Pair<T>::exact>(vout, vin);
#pragma unroll
        for (int r = 0; r < 6; r++) t1[r][col] = vout[r];
    }
#pragma unroll
    for (int xi = 0; xi < 6; xi++) {
        float2 vout[6];
        apply_bt<Pair<T>::exact>(vout, t1[xi]);
#pragma unroll
        for (int nu = 0; nu < 6; nu++) {
            auto* dst = reinterpret_cast<typename P2::type*>(
                V + ((size_t)(xi * 6 + nu) * Pa + p) * 64 + c0);
            *dst = P2::from_f2(vout[nu]);
        }
    }
}

// ---------------------------------------------------------------------------
// Input transform of activations already on the device:
// X[n][361][Cp] -> V[36][Pa][Cp].  Used by the single-layer diagnostics; in
// the tower this step is the tail of xform_kernel.
// grid (Cp/64, n), block 256.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kXformThreads) in_transform_kernel(
    const T* __restrict__ X, T* __restrict__ V, int Pa, int Cp) {
    using P2 = Pair<T>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto* board = reinterpret_cast<float2*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.y, k = blockIdx.x * kChanPerCta + 2 * lane;
    zero_halo(board, warp, lane, kXformWarps);
    for (int s = warp; s < kSq; s += kXformWarps) {
        const int y = s / kBoard, x = s % kBoard;
        board[((y + 1) * kBoardPad + x + 1) * 32 + lane] =
            P2::to_f2(*reinterpret_cast<const typename P2::type*>(X + ((size_t)n * kSq + s) * Cp + k));
    }
    __syncthreads();
    for (int tile = warp; tile < kTilesPerPos; tile += kXformWarps) {
        const int p = n * kTilesPerPos + tile;
        tile_in_transform<T>(board, lane, tile / kTilesPerSide, tile % kTilesPerSide, V,
                             (size_t)Pa * Cp, (size_t)p * Cp + k);
    }
}

// ---------------------------------------------------------------------------
// The fused step between two contractions:
//   M of layer l  --A^T m A-->  4x4 outputs  --batch-norm [+ residual], ReLU-->
//   activations (optionally stored to X_out)  --B^T d B-->  V of layer l+1.
// One CTA owns one position and 64 channels, so the whole 19x19 plane of those
// channels is assembled in shared memory between the two transforms and the
// activations never travel through global memory unless they are needed later
// as a residual.  R and X_out may be the same buffer: every element is read
// and written by the same thread.
// grid (Cp/64, n), block XformShape<T>::warps * 32, dynamic smem = 484 * 32 * 8 bytes (fp32 board).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(XformShape<T>::warps * 32, XformShape<T>::ctas) xform_kernel(
    const T* M, int Pa, int Cp,
    const float* __restrict__ bn_mean, const float* __restrict__ bn_invstd,
    const T* R, T* X_out, T* __restrict__ V) {
    using P2 = Pair<T>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto* board = reinterpret_cast<float2*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.y, k = blockIdx.x * kChanPerCta + 2 * lane;
    const size_t pt_stride = (size_t)Pa * Cp;

    // launched with programmatic stream serialization: let the next kernel set
    // up, prepare what does not depend on the previous one, then wait for it
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (V != nullptr) zero_halo(board, warp, lane, XformShape<T>::warps);
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const float2 mean = *reinterpret_cast<const float2*>(bn_mean + k);
    const float2 scale = *reinterpret_cast<const float2*>(bn_invstd + k);

    for (int tile = warp; tile < kTilesPerPos; tile += XformShape<T>::warps) {
        const int by = tile / kTilesPerSide, bx = tile % kTilesPerSide;
        const T* msrc = M + (size_t)(n * kTilesPerPos + tile) * Cp + k;
        // temp[i][nu] = sum_xi At[i][xi] m[xi][nu]
        float2 temp[4][6];
#pragma unroll
        for (int nu = 0; nu < 6; nu++) {
            float2 colv[6], o4[4];
#pragma unroll
            for (int xi = 0; xi < 6; xi++) {
                // M is still being written when this kernel starts, so it is
                // not read-only for the kernel's lifetime: no ld.global.nc
                colv[xi] = P2::to_f2(__ldcg(reinterpret_cast<const typename P2::type*>(
                    msrc + (size_t)(xi * 6 + nu) * pt_stride)));
            }
            apply_at<Pair<T>::exact>(o4, colv);
#pragma unroll
            for (int i = 0; i < 4; i++) temp[i][nu] = o4[i];
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 o4[4];
            apply_at<Pair<T>::exact>(o4, temp[i]);
            const int y = 4 * by + i;
            if (y >= kBoard) continue;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int x = 4 * bx + j;
                if (x >= kBoard) continue;
                // max(0, invstd * (v - mean) [+ residual]), src/CPUPipe.cpp:352-377
                constexpr bool kE = Pair<T>::exact;
                float2 v = make_float2(op_mul<kE>(scale.x, op_add<kE>(o4[j].x, -mean.x)),
                                       op_mul<kE>(scale.y, op_add<kE>(o4[j].y, -mean.y)));
                const size_t xoff = ((size_t)n * kSq + y * kBoard + x) * Cp + k;
                if (R != nullptr) {
                    const float2 r = P2::to_f2(*reinterpret_cast<const typename P2::type*>(R + xoff));
                    v = add2<Pair<T>::exact>(v, r);
                }
                v.x = fmaxf(v.x, 0.f);
                v.y = fmaxf(v.y, 0.f);
                const typename P2::type packed = P2::from_f2(v);
                if (X_out != nullptr) {
                    *reinterpret_cast<typename P2::type*>(X_out + xoff) = packed;
                }
                if (V != nullptr) {
                    board[((y + 1) * kBoardPad + x + 1) * 32 + lane] = v;
                }
            }
        }
    }
    if (V == nullptr) return;
    __syncthreads();
    for (int tile = warp; tile < kTilesPerPos; tile += XformShape<T>::warps) {
        const int p = n * kTilesPerPos + tile;
        tile_in_transform<T>(board, lane, tile / kTilesPerSide, tile % kTilesPerSide, V,
                             pt_stride, (size_t)p * Cp + k);
    }
}

// ---------------------------------------------------------------------------
// The two 1x1 head convolutions (policy: 2 outputs, value: 1 output):
//   out[o][s] = sum_c w[o][c] * X[n][s][c]          (src/CPUPipe.cpp:301-350)
// One warp per board cell, lanes stride over channel pairs.  w is [3][Cp]
// fp32: rows 0,1 policy, row 2 value.  Outputs are fp32 planes in the layout
// ForwardPipe::forward returns: pol[n][2][361], val[n][361].
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) head_conv_kernel(
    const T* __restrict__ X, const float* __restrict__ w, int Cp, int cells,
    float* __restrict__ pol, float* __restrict__ val) {
    using P2 = Pair<T>;
    const int lane = threadIdx.x & 31;
    const int cell = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (cell >= cells) return;
    const T* x = X + (size_t)cell * Cp;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;
    for (int c = 2 * lane; c < Cp; c += 64) {
        const float2 v = P2::to_f2(*reinterpret_cast<const typename P2::type*>(x + c));
        const float2 w0 = *reinterpret_cast<const float2*>(w + c);
        const float2 w1 = *reinterpret_cast<const float2*>(w + Cp + c);
        const float2 w2 = *reinterpret_cast<const float2*>(w + 2 * Cp + c);
        a0 += w0.x * v.x + w0.y * v.y;
        a1 += w1.x * v.x + w1.y * v.y;
        a2 += w2.x * v.x + w2.y * v.y;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        a0 += __shfl_xor_sync(0xffffffffu, a0, off);
        a1 += __shfl_xor_sync(0xffffffffu, a1, off);
        a2 += __shfl_xor_sync(0xffffffffu, a2, off);
    }
    if (lane == 0) {
        const int n = cell / kSq, s = cell % kSq;
        pol[((size_t)n * 2 + 0) * kSq + s] = a0;
        pol[((size_t)n * 2 + 1) * kSq + s] = a1;
        val[(size_t)n * kSq + s] = a2;
    }
}

// ---------------------------------------------------------------------------
// Weight repack at upload time: U32[36][c_in][K] fp32 (engine layout,
// src/Network.cpp:215) -> U[36][Kp][Cin_p] of type T, zero padded, input
// channel innermost so that both contraction operands are K-major.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void repack_u_kernel(const float* __restrict__ U32, T* __restrict__ U, int c_in,
                                int K, int Cin_p, int Kp) {
    const size_t total = (size_t)kPoints * Kp * Cin_p;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int c = i % Cin_p;
        const int k = (i / Cin_p) % Kp;
        const int t = i / ((size_t)Cin_p * Kp);
        float v = 0.f;
        if (c < c_in && k < K) v = U32[((size_t)t * c_in + c) * K + k];
        U[i] = (T)v;
    }
}

// Filter transform on the device: f[K][c_in][3][3] -> U32[36][c_in][K] with
// U[xi*6+nu] = (G f G^T)[xi][nu], accumulating like the reference does
// (src/Network.cpp:159-223: acc = 0; acc += G[i][k] * f[k][j] for k = 0..2).
__global__ void transform_f_kernel(const float* __restrict__ f, float* __restrict__ U32, int c_in,
                                   int K) {
    const float G[6][3] = {{1.0f, 0.0f, 0.0f},
                           {-2.0f / 3.0f, -kSq2 / 3.0f, -1.0f / 3.0f},
                           {-2.0f / 3.0f, kSq2 / 3.0f, -1.0f / 3.0f},
                           {1.0f / 6.0f, kSq2 / 6.0f, 1.0f / 3.0f},
                           {1.0f / 6.0f, -kSq2 / 6.0f, 1.0f / 3.0f},
                           {0.0f, 0.0f, 1.0f}};
    const int total = c_in * K;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i % K, c = i / K;
        const float* flt = f + ((size_t)k * c_in + c) * 9;
        float gf[6][3];
        for (int a = 0; a < 6; a++)
            for (int j = 0; j < 3; j++) {
                float acc = 0.0f;
                for (int m = 0; m < 3; m++) acc = nf_add(acc, nf_mul(G[a][m], flt[m * 3 + j]));
                gf[a][j] = acc;
            }
        for (int xi = 0; xi < 6; xi++)
            for (int nu = 0; nu < 6; nu++) {
                float acc = 0.0f;
                for (int m = 0; m < 3; m++) acc = nf_add(acc, nf_mul(gf[xi][m], G[nu][m]));
                U32[((size_t)(xi * 6 + nu) * c_in + c) * K + k] = acc;
            }
    }
}

// Bit-packed planes [n][18][12] words -> fp32 planes [n][18][361] of 0 / 1.
__global__ void unpack_planes_kernel(const unsigned int* __restrict__ packed, float* __restrict__ out,
                                     int n) {
    const size_t total = (size_t)n * kInputPlanes * kSq;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int s = i % kSq;
        const size_t plane = i / kSq;
        out[i] = (packed[plane * 12 + (s >> 5)] >> (s & 31)) & 1u ? 1.0f : 0.0f;
    }
}

// fp32 NCHW [n][C][361] <-> T NHWC [n][361][Cp] (diagnostics only).
template <typename T>
__global__ void nchw_to_nhwc_kernel(const float* __restrict__ src, T* __restrict__ dst, int n,
                                    int C, int Cp) {
    const size_t total = (size_t)n * kSq * Cp;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int c = i % Cp;
        const int s = (i / Cp) % kSq;
        const int b = i / ((size_t)Cp * kSq);
        dst[i] = (T)(c < C ? src[((size_t)b * C + c) * kSq + s] : 0.f);
    }
}

template <typename T>
__global__ void nhwc_to_nchw_kernel(const T* __restrict__ src, float* __restrict__ dst, int n,
                                    int C, int Cp) {
    const size_t total = (size_t)n * C * kSq;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int s = i % kSq;
        const int c = (i / kSq) % C;
        const int b = i / ((size_t)C * kSq);
        dst[i] = (float)src[((size_t)b * kSq + s) * Cp + c];
    }
}

}  // namespace lzb
