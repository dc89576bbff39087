// 3x3 convolution + batch-norm + residual + ReLU as ONE implicit GEMM on the
// Blackwell tensor cores (tcgen05, accumulators in tensor memory, operands
// brought in by TMA), fp16 or bf16 operands with fp32 accumulation.
//
// Activation layout ("padded cell-major"): a position is stored as 20 rows of
// 20 cells, row 0 and column 0 being zero halo; because rows and positions
// follow each other without gaps, the halo of one row/position doubles as the
// opposite halo of its neighbour:
//     cell(n, y, x) = (n * 20 + y + 1) * 20 + (x + 1),  y, x in [0, 19)
//     X[cell][Cp], channels innermost; Q = (20 * n + 1) * 20 cells in all.
// With that layout the input of filter tap (dy, dx) for the 128 consecutive
// output cells m0 .. m0+127 is simply rows m0 + 20*dy + dx .. of X, i.e. one
// TMA box load at a shifted row coordinate (rows outside [0, Qa) read as zero).
// The nine shifted inputs of a tile overlap almost entirely, so the kernel
// loads ONE window of 176 rows per 64-channel chunk and points the nine MMA
// groups at row offsets inside it: under the 128-byte swizzle a K-major tile
// is a linear array of 128-byte rows whose swizzle phase comes from the
// address bits, so a descriptor may start at any row.
// Halo cells are computed like any other row and forced to zero on store, so
// the output is again a valid input.
//
// GEMM view per output tile:  D[128 cells][Kp] = sum over 9 taps and Cin/64
// chunks of A[128][64] * W[tap][Kp][64]^T.  Weights are stored
// Wd[9][Kp][Cin] (input channel innermost), so both operands are K-major.
//
// Per tile and chunk the producer brings one window (22 KB) and nine weight
// tiles (32 KB each, 5-deep ring): 1.24 MB per tile instead of 1.73 MB with one
// activation tile per tap.
//
// Roles in the CTA (10 warps, one CTA per SM, persistent over a contiguous
// range of tiles): warp 0 TMA producer, warp 1 MMA issuer and tensor-memory
// owner, warps 2-9 epilogue (two warps per tensor-memory lane quadrant, each
// converting half of the output channels, with the tensor-memory and residual
// loads of the next 32-column chunk in flight while the current one is
// processed).  Two 256-column accumulators alternate, so the epilogue of tile i
// (tcgen05.ld, batch-norm, residual, ReLU, fp16 store) overlaps the MMAs of
// tile i+1.  All waits are bounded (see mbar_wait).
//
// The arithmetic is that of CPUPipe's convolve3 + batchnorm
// (src/CPUPipe.cpp:286-299, 352-377) evaluated directly instead of through
// the Winograd transforms; it replaces the reference's three launches per
// layer (src/OpenCL.cpp:332-494) with one.
#pragma once
#include "gemm_tcgen05.cuh"
#include "winograd_math.cuh"

namespace lzb {
namespace dc {

using namespace tc;   // PTX helpers, descriptor builders

constexpr int kCellsPerRow = 20;
constexpr int kCellsPerPos = 400;
constexpr int kTileM = 128;
constexpr int kDcThreads = 320;            // producer warp, MMA warp, 8 epilogue warps
// Activation window: the 128 output cells of a tile plus the cells the 9 taps
// reach (+-21 rows), padded to +-24 so that it starts on an 8-row swizzle atom.
constexpr int kWinPad = 24;
constexpr int kWinRows = kTileM + 2 * kWinPad;             // 176
constexpr uint32_t kWinBytes = kWinRows * 128;             // 22 KB per 64-channel chunk
constexpr int kWinBufs = 2;
constexpr int kBStages = 5;                                // weight-tile ring
constexpr uint32_t kBStageBytes = kMaxN * 128;             // 32 KB
constexpr uint32_t kOperandBytes = kWinBufs * kWinBytes + kBStages * kBStageBytes;
constexpr uint32_t kStageOutBytes = 32 * 64;               // one epilogue warp: 32 cells x 32 channels
constexpr uint32_t kDSmemBytes =
    kOperandBytes + 8 * kStageOutBytes + 2 * kMaxN * 4 /* bn */ + kBarBytes + 1024;

constexpr int kErrDcProducer = 201;
constexpr int kErrDcMmaAcc = 202;
constexpr int kErrDcMmaFull = 203;
constexpr int kErrDcEpilogue = 204;

__host__ __device__ inline long long cells_for(int n) { return (20LL * n + 1) * kCellsPerRow; }
__host__ __device__ inline int cell_of(int n, int y, int x) {
    return (n * 20 + y + 1) * kCellsPerRow + x + 1;
}
__device__ __forceinline__ bool cell_is_interior(int q, int Q) {
    const int c = q % kCellsPerRow, r = (q / kCellsPerRow) % 20;
    return q < Q && c != 0 && r != 0;
}

template <typename T> struct Vec2;
template <> struct Vec2<__half> {
    static __device__ __forceinline__ float2 unpack(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2*>(&u));
    }
};
template <> struct Vec2<__nv_bfloat16> {
    static __device__ __forceinline__ float2 unpack(uint32_t u) {
        return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
    }
};

// 64 bytes (32 channels) of the residual row, or zeros.
template <typename T>
__device__ __forceinline__ void load_residual(uint4 (&v)[4], const T* src, bool use) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = use ? reinterpret_cast<const uint4*>(src)[i] : make_uint4(0u, 0u, 0u, 0u);
    }
}

// One 32-channel chunk of one output cell: max(0, x * invstd - mean * invstd
// [+ residual]) (src/CPUPipe.cpp:352-377), halo cells forced to zero, packed
// to 16 bits and written to this warp's staging tile (32 cells x 64 bytes,
// 64-byte swizzle: 16-byte word v of row r sits at slot v ^ ((r >> 1) & 3),
// which is both bank-conflict free and the layout the TMA store expects).
template <typename T>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], const uint4 (&rv)[4],
                                               const float* s_scale, const float* s_bias,
                                               bool use_res, bool interior, unsigned char* stg_row,
                                               int lane) {
    const T tag = T();
    const float4* sc4 = reinterpret_cast<const float4*>(s_scale);
    const float4* bi4 = reinterpret_cast<const float4*>(s_bias);
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const float4 s0 = sc4[2 * v], s1 = sc4[2 * v + 1];
        const float4 b0 = bi4[2 * v], b1 = bi4[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float bi[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const uint32_t rr[4] = {rv[v].x, rv[v].y, rv[v].z, rv[v].w};
        uint32_t o[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            float a = fmaf(__uint_as_float(r[8 * v + 2 * h]), sc[2 * h], bi[2 * h]);
            float b = fmaf(__uint_as_float(r[8 * v + 2 * h + 1]), sc[2 * h + 1], bi[2 * h + 1]);
            if (use_res) {
                const float2 f = Vec2<T>::unpack(rr[h]);
                a += f.x;
                b += f.y;
            }
            a = interior ? fmaxf(a, 0.f) : 0.f;
            b = interior ? fmaxf(b, 0.f) : 0.f;
            o[h] = pack2(tag, a, b);
        }
        *reinterpret_cast<uint4*>(stg_row + ((v ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// The same for activations carried as two 16-bit planes, x = hi + lo: the
// residual is the sum of its two planes, the result is split again.  The high
// plane goes to the staging tile, the low plane is returned packed (word
// 4 * v + h holds channels 8 * v + 2 * h, + 1) for a second store.
template <typename T>
__device__ __forceinline__ void epilogue_chunk_x2(const uint32_t (&r)[32], const uint4 (&rv)[4],
                                                  const uint4 (&rl)[4], const float* s_scale,
                                                  const float* s_bias, bool use_res, bool interior,
                                                  unsigned char* stg_row, int lane,
                                                  uint32_t (&lo)[16]) {
    const T tag = T();
    const float4* sc4 = reinterpret_cast<const float4*>(s_scale);
    const float4* bi4 = reinterpret_cast<const float4*>(s_bias);
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const float4 s0 = sc4[2 * v], s1 = sc4[2 * v + 1];
        const float4 b0 = bi4[2 * v], b1 = bi4[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float bi[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const uint32_t rr[4] = {rv[v].x, rv[v].y, rv[v].z, rv[v].w};
        const uint32_t ll[4] = {rl[v].x, rl[v].y, rl[v].z, rl[v].w};
        uint32_t o[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            float a = fmaf(__uint_as_float(r[8 * v + 2 * h]), sc[2 * h], bi[2 * h]);
            float b = fmaf(__uint_as_float(r[8 * v + 2 * h + 1]), sc[2 * h + 1], bi[2 * h + 1]);
            if (use_res) {
                const float2 f = Vec2<T>::unpack(rr[h]);
                const float2 g = Vec2<T>::unpack(ll[h]);
                a += f.x + g.x;
                b += f.y + g.y;
            }
            a = interior ? fmaxf(a, 0.f) : 0.f;
            b = interior ? fmaxf(b, 0.f) : 0.f;
            o[h] = pack2(tag, a, b);
            const float2 hi = Vec2<T>::unpack(o[h]);
            lo[4 * v + h] = pack2(tag, a - hi.x, b - hi.y);
        }
        *reinterpret_cast<uint4*>(stg_row + ((v ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}
// Put a packed low plane (see epilogue_chunk_x2) into the staging tile.
__device__ __forceinline__ void stage_low_plane(const uint32_t (&lo)[16], unsigned char* stg_row, int lane) {
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        *reinterpret_cast<uint4*>(stg_row + ((v ^ sw) << 4)) =
            make_uint4(lo[4 * v], lo[4 * v + 1], lo[4 * v + 2], lo[4 * v + 3]);
    }
}

// ---- activations as an fp16 plane plus an e5m2 plane, x = hi + lo ----------
// e5m2 (1-5-2) is the upper byte of an fp16 number, so both conversions are
// byte moves around one rounding.
__device__ __forceinline__ uint32_t e5m2_from_float(float v) {
    const uint32_t h = __half_as_ushort(__float2half_rn(v));
    return (h + 0x7Fu + ((h >> 8) & 1u)) >> 8;            // round to nearest even on the dropped byte
}
__device__ __forceinline__ float e5m2_to_float(uint32_t byte) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>((byte & 0xFFu) << 8)));
}
// Two at a time with the hardware conversions (one rounding, saturating):
// byte 0 of the result is `even`, byte 1 is `odd`.
__device__ __forceinline__ uint32_t e5m2x2_from_floats(float even, float odd) {
    unsigned short d;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(d) : "f"(odd), "f"(even));
    return d;
}
__device__ __forceinline__ float2 e5m2x2_to_float2(uint32_t two_bytes) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(static_cast<unsigned short>(two_bytes)));
    return __half22float2(*reinterpret_cast<__half2*>(&h2));
}
// fp16 x2 -> e5m2 x2 and back, and fp32 arithmetic that takes an fp16 operand
// as it is (sm_100 mixed-precision add / fma): the conversion unit runs at a
// quarter of the arithmetic rate, and the two epilogue warps of a scheduler
// share it, so the epilogue converts as little as it can.
__device__ __forceinline__ uint32_t e5m2x2_from_half2(uint32_t h2) {
    unsigned short d;
    asm("cvt.rn.satfinite.e5m2x2.f16x2 %0, %1;" : "=h"(d) : "r"(h2));
    return d;
}
__device__ __forceinline__ uint32_t half2_from_e5m2x2(uint32_t two_bytes) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(static_cast<unsigned short>(two_bytes)));
    return h2;
}
// c + h, h the low (or high) half of a packed fp16 pair
__device__ __forceinline__ float add_half_lo(uint32_t h2, float c) {
    float d;
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(static_cast<unsigned short>(h2)), "f"(c));
    return d;
}
__device__ __forceinline__ float add_half_hi(uint32_t h2, float c) {
    float d;
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(static_cast<unsigned short>(h2 >> 16)), "f"(c));
    return d;
}
// c - h
__device__ __forceinline__ float minus_half_lo(uint32_t h2, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(static_cast<unsigned short>(h2)),
        "h"(static_cast<unsigned short>(0xBC00)), "f"(c));
    return d;
}
__device__ __forceinline__ float minus_half_hi(uint32_t h2, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(static_cast<unsigned short>(h2 >> 16)),
        "h"(static_cast<unsigned short>(0xBC00)), "f"(c));
    return d;
}
// 32 bytes (32 channels) of an e5m2 residual row, or zeros.
__device__ __forceinline__ void load_residual8(uint4 (&v)[2], const unsigned char* src, bool use) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        v[i] = use ? reinterpret_cast<const uint4*>(src)[i] : make_uint4(0u, 0u, 0u, 0u);
    }
}
// Scale between the fp16 plane and its e5m2 copy "hi8" (and, inversely, on the
// e5m2 plane of the weight remainders it is multiplied with): w - fp16(w) is
// around 2^-12 |w|, below the e5m2 range for typical filters, so the remainder
// is stored times 256 and the activations divided by 256.
constexpr float kHi8Scale = 1.0f / 256.0f;
constexpr float kWLoScale = 256.0f;
// epilogue_chunk for that form: the residual is fp16 + e5m2, the result is
// split into an fp16 tile (written to the staging tile like epilogue_chunk
// does) and 32 e5m2 bytes returned in lo[8] (byte c of the row = channel c);
// with want_h8, h8[8] receives the fp16 values scaled by kHi8Scale in e5m2.
template <typename T>
__device__ __forceinline__ void epilogue_chunk_e5m2(const uint32_t (&r)[32], const uint4 (&rv)[4],
                                                    const uint4 (&rl)[2], const float* s_scale,
                                                    const float* s_bias, bool use_res, bool interior,
                                                    unsigned char* stg_row, int lane,
                                                    uint32_t (&lo)[8], uint32_t (&h8)[8], bool want_h8) {
    const T tag = T();
    const float4* sc4 = reinterpret_cast<const float4*>(s_scale);
    const float4* bi4 = reinterpret_cast<const float4*>(s_bias);
    const int sw = (lane >> 1) & 3;
    const uint32_t lw[8] = {rl[0].x, rl[0].y, rl[0].z, rl[0].w, rl[1].x, rl[1].y, rl[1].z, rl[1].w};
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const float4 s0 = sc4[2 * v], s1 = sc4[2 * v + 1];
        const float4 b0 = bi4[2 * v], b1 = bi4[2 * v + 1];
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float bi[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const uint32_t rr[4] = {rv[v].x, rv[v].y, rv[v].z, rv[v].w};
        uint32_t o[4];
        uint32_t packed[2] = {0u, 0u}, packed8[2] = {0u, 0u};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            float a = fmaf(__uint_as_float(r[8 * v + 2 * h]), sc[2 * h], bi[2 * h]);
            float b = fmaf(__uint_as_float(r[8 * v + 2 * h + 1]), sc[2 * h + 1], bi[2 * h + 1]);
            if (use_res) {
                // channels 8v + 2h, +1 are bytes (2h, 2h + 1) & 3 of word 2v + h / 2
                const uint32_t g = half2_from_e5m2x2(lw[2 * v + (h >> 1)] >> (16 * (h & 1)));
                a = add_half_lo(g, add_half_lo(rr[h], a));
                b = add_half_hi(g, add_half_hi(rr[h], b));
            }
            a = interior ? fmaxf(a, 0.f) : 0.f;
            b = interior ? fmaxf(b, 0.f) : 0.f;
            o[h] = pack2(tag, a, b);
            packed[h >> 1] |= e5m2x2_from_floats(minus_half_lo(o[h], a), minus_half_hi(o[h], b)) << (16 * (h & 1));
            if (want_h8) {
                const __half2 scaled = __hmul2(*reinterpret_cast<const __half2*>(&o[h]), __float2half2_rn(kHi8Scale));
                packed8[h >> 1] |= e5m2x2_from_half2(*reinterpret_cast<const uint32_t*>(&scaled)) << (16 * (h & 1));
            }
        }
        lo[2 * v] = packed[0];
        lo[2 * v + 1] = packed[1];
        h8[2 * v] = packed8[0];
        h8[2 * v + 1] = packed8[1];
        *reinterpret_cast<uint4*>(stg_row + ((v ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Hand the warp's staging tile to the TMA engine: rows m .. m+31, channels
// col .. col+31 of the output.  Every lane fences its shared-memory writes
// towards the async proxy, one lane issues the store.
__device__ __forceinline__ void store_staged_tile(const CUtensorMap* map, uint32_t stg, int col,
                                                  int row, int lane) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        asm volatile(
            "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                reinterpret_cast<uint64_t>(map)),
            "r"(col), "r"(row), "r"(stg)
            : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}
// Before the staging tile is overwritten: the previous store must have read it.
__device__ __forceinline__ void wait_staged_tile_read(int lane) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
}

// tmX : 2-D map over the input activations [Qa rows][Cin], box 64 x kWinRows.
// tmW : 2-D map over this layer's weights  [9*Kp rows][Cin], box 64 x Kp.
// tmO : 2-D map over the output activations [Qa rows][Kp], box 32 x 32, 64-byte swizzle.
// res : residual [Qa][Kp] or nullptr (may be the output buffer: a warp reads the
//       residual of a chunk before it stores that chunk).
template <typename T>
__global__ void __launch_bounds__(kDcThreads, 1) conv_direct_kernel(
    const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
    const __grid_constant__ CUtensorMap tmO, const T* res, const float* __restrict__ bn_mean, const float* __restrict__ bn_invstd,
    int Q, int Kp, int kchunks, int ntiles, int* err) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (base - raw);
    const uint32_t win_base = base;
    const uint32_t b_base = base + kWinBufs * kWinBytes;
    unsigned char* stage_out = smem + kOperandBytes;            // 8 x 2 KB, 1024-byte aligned
    float* s_scale = reinterpret_cast<float*>(stage_out + 8 * kStageOutBytes);
    float* s_bias = s_scale + kMaxN;
    unsigned char* bar_mem = stage_out + 8 * kStageOutBytes + 2 * kMaxN * 4;
    const uint32_t bars = smem_u32(bar_mem);
    auto bfull_bar = [&](int s) { return bars + 8u * (0 + s); };
    auto bempty_bar = [&](int s) { return bars + 8u * (8 + s); };
    auto wfull_bar = [&](int w) { return bars + 8u * (16 + w); };
    auto wempty_bar = [&](int w) { return bars + 8u * (18 + w); };
    auto tfull_bar = [&](int a) { return bars + 8u * (20 + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (22 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * 24);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * 24 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kBStages; i++) {
            mbar_init(bfull_bar(i), 1);
            mbar_init(bempty_bar(i), 1);
        }
        for (int i = 0; i < kWinBufs; i++) {
            mbar_init(wfull_bar(i), 1);
            mbar_init(wempty_bar(i), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);     // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // batch norm as one FMA per element: y = x * invstd + (-mean * invstd)
    for (int i = threadIdx.x; i < Kp; i += blockDim.x) {
        s_scale[i] = bn_invstd[i];
        s_bias[i] = -bn_mean[i] * bn_invstd[i];
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tile_begin = static_cast<int>(static_cast<long long>(blockIdx.x) * ntiles / gridDim.x);
    const int tile_end = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * ntiles / gridDim.x);

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0, wb = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            const uint32_t btx = static_cast<uint32_t>(Kp) * 128u;
            for (int tile = tile_begin; tile < tile_end && ok; ++tile) {
                const int m0 = tile * kTileM;
                for (int c = 0; c < kchunks && ok; ++c) {
                    ok = mbar_wait(wempty_bar(wb), wphase ^ 1u, abort_flag, err, kErrDcProducer);
                    if (!ok) break;
                    mbar_expect_tx(wfull_bar(wb), kWinBytes);
                    tma_load_2d(win_base + wb * kWinBytes, &tmX, c * kChunkK, m0 - kWinPad, wfull_bar(wb));
                    if (++wb == kWinBufs) { wb = 0; wphase ^= 1u; }
                    for (int tap = 0; tap < 9; ++tap) {
                        ok = mbar_wait(bempty_bar(stage), phase ^ 1u, abort_flag, err, kErrDcProducer);
                        if (!ok) break;
                        mbar_expect_tx(bfull_bar(stage), btx);
                        tma_load_2d(b_base + stage * kBStageBytes, &tmW, c * kChunkK, tap * Kp,
                                    bfull_bar(stage));
                        if (++stage == kBStages) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (OperandFormat<T>::value << 7) |
                                   (OperandFormat<T>::value << 10) |
                                   (static_cast<uint32_t>(Kp >> 3) << 17) |
                                   (static_cast<uint32_t>(kTileM >> 4) << 24);
            int stage = 0, wb = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            int local = 0;
            for (int tile = tile_begin; tile < tile_end && ok; ++tile, ++local) {
                const int acc = local & 1;
                const uint32_t accphase = (local >> 1) & 1u;
                ok = mbar_wait(tempty_bar(acc), accphase ^ 1u, abort_flag, err, kErrDcMmaAcc);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kMaxN);
                for (int c = 0; c < kchunks && ok; ++c) {
                    ok = mbar_wait(wfull_bar(wb), wphase, abort_flag, err, kErrDcMmaFull);
                    if (!ok) break;
                    const uint32_t win = win_base + wb * kWinBytes;
                    for (int tap = 0; tap < 9; ++tap) {
                        ok = mbar_wait(bfull_bar(stage), phase, abort_flag, err, kErrDcMmaFull);
                        if (!ok) break;
                        tcgen05_fence_after();
                        // rows of the window this tap reads: (24 + 20*dy + dx) .. +127
                        const int row0 = kWinPad + (tap / 3 - 1) * kCellsPerRow + (tap % 3 - 1);
                        const uint64_t a_desc = umma_desc_sw128(win + static_cast<uint32_t>(row0) * 128u);
                        const uint64_t b_desc = umma_desc_sw128(b_base + stage * kBStageBytes);
#pragma unroll
                        for (int k = 0; k < kChunkK / 16; ++k) {
                            tcgen05_mma_f16(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                                            (c > 0 || tap > 0 || k > 0) ? 1u : 0u);
                        }
                        tcgen05_commit(bempty_bar(stage));
                        if (++stage == kBStages) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    tcgen05_commit(wempty_bar(wb));      // window free once these MMAs retire
                    if (++wb == kWinBufs) { wb = 0; wphase ^= 1u; }
                }
                if (!ok) break;
                tcgen05_commit(tfull_bar(acc));
            }
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..9)
        const int qd = warp & 3;                 // tensor-memory lane quadrant of this warp
        const int ncols = Kp >> 1;               // this warp converts half of the channels
        const int col0 = ((warp - 2) >> 2) * ncols;
        unsigned char* stg_ptr = stage_out + (warp - 2) * kStageOutBytes;
        const uint32_t stg = smem_u32(stg_ptr);
        unsigned char* stg_row = stg_ptr + lane * 64;
        int local = 0;
        for (int tile = tile_begin; tile < tile_end; ++tile, ++local) {
            const int acc = local & 1;
            const uint32_t accphase = (local >> 1) & 1u;
            const int q = tile * kTileM + qd * 32 + lane;
            const bool interior = cell_is_interior(q, Q);
            bool ok = mbar_wait(tfull_bar(acc), accphase, abort_flag, err, kErrDcEpilogue);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const bool use_res = (res != nullptr) && interior;
            const T* rrow = res + static_cast<size_t>(q) * Kp + col0;
            const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(qd * 32) << 16) +
                                    static_cast<uint32_t>(acc * kMaxN + col0);
            const int row0 = tile * kTileM + qd * 32;     // first cell of this warp's 32 rows
            uint32_t ra[32], rb[32];
            uint4 va[4], vb[4];
            load_residual(va, rrow, use_res);
            LZB_TMEM_LD32(ra, taddr0);
            for (int j = 0; j < ncols; j += 64) {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const bool more = j + 32 < ncols;
                if (more) {
                    load_residual(vb, rrow + j + 32, use_res);
                    LZB_TMEM_LD32(rb, taddr0 + j + 32);
                }
                wait_staged_tile_read(lane);
                epilogue_chunk<T>(ra, va, s_scale + col0 + j, s_bias + col0 + j, use_res, interior,
                                  stg_row, lane);
                store_staged_tile(&tmO, stg, col0 + j, row0, lane);
                if (more) {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (j + 64 < ncols) {
                        load_residual(va, rrow + j + 64, use_res);
                        LZB_TMEM_LD32(ra, taddr0 + j + 64);
                    }
                    wait_staged_tile_read(lane);
                    epilogue_chunk<T>(rb, vb, s_scale + col0 + j + 32, s_bias + col0 + j + 32, use_res,
                                      interior, stg_row, lane);
                    store_staged_tile(&tmO, stg, col0 + j + 32, row0, lane);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        // the bulk stores of this warp must be complete before the CTA retires
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// Helper kernels of the direct path (all bandwidth-trivial).
// ---------------------------------------------------------------------------

// Network input planes in[n][18][361] fp32 -> padded cell-major X0[Qa][64],
// channels 18..63 and halo cells zero.  One thread per (cell, channel pair).
template <typename T>
__global__ void __launch_bounds__(256) input_to_cells_kernel(const float* __restrict__ in,
                                                             T* __restrict__ X0, int n) {
    using P2 = Pair<T>;
    const long long total = cells_for(n) * 32;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int pair = static_cast<int>(i & 31);
        const int q = static_cast<int>(i >> 5);
        const int c = q % kCellsPerRow, r = q / kCellsPerRow;
        float2 v = make_float2(0.f, 0.f);
        if (c != 0 && (r % 20) != 0 && 2 * pair < kInputPlanes) {
            const int pos = r / 20, y = r % 20 - 1, x = c - 1;
            const float* src = in + ((size_t)pos * kInputPlanes + 2 * pair) * kSq + y * kBoard + x;
            v = make_float2(src[0], src[kSq]);
        }
        *reinterpret_cast<typename P2::type*>(X0 + (size_t)q * 64 + 2 * pair) = P2::from_f2(v);
    }
}

// Recover the 3x3 filters from their Winograd transform and lay them out for
// the implicit GEMM:  U32[36][c_in][K] (U = G f G^T, src/Network.cpp:159-223)
// -> Wd[9][Kp][Cin_p], zero padded.  f = P U P^T with P a left inverse of G:
// rows 0 and 5 of G are unit vectors, and rows 1,2 differ only in the sign of
// the middle coefficient, so f_0 = u_0, f_2 = u_5, f_1 = (u_2 - u_1) * 3/(2 sqrt 2).
template <typename T>
__global__ void untransform_u_kernel(const float* __restrict__ U32, T* __restrict__ Wd, int c_in,
                                     int K, int Cin_p, int Kp) {
    const int total = c_in * K;
    const float mid = 3.0f / (2.0f * kSq2);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i % K, c = i / K;
        auto u = [&](int xi, int nu) { return U32[((size_t)(xi * 6 + nu) * c_in + c) * K + k]; };
        float g[3][6];   // rows of P U
        for (int nu = 0; nu < 6; nu++) {
            g[0][nu] = u(0, nu);
            g[1][nu] = (u(2, nu) - u(1, nu)) * mid;
            g[2][nu] = u(5, nu);
        }
        for (int a = 0; a < 3; a++) {
            const float f[3] = {g[a][0], (g[a][2] - g[a][1]) * mid, g[a][5]};
            for (int b = 0; b < 3; b++) {
                Wd[((size_t)(a * 3 + b) * Kp + k) * Cin_p + c] = (T)f[b];
            }
        }
    }
}

// Untransformed filters f[K][c_in][3][3] -> Wd[9][Kp][Cin_p] (Wd zeroed beforehand).
template <typename T>
__global__ void filters_to_wd_kernel(const float* __restrict__ f, T* __restrict__ Wd, int c_in, int K,
                                     int Cin_p, int Kp) {
    const int total = c_in * K * 9;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int tap = i % 9, c = (i / 9) % c_in, k = i / (9 * c_in);
        Wd[((size_t)tap * Kp + k) * Cin_p + c] = (T)f[i];
    }
}

// Weights for activations carried as two 16-bit planes (and, optionally,
// weights carried as two planes as well): Wd32[9][Kp][Cin_p] fp32 ->
// Wd[9][Kp][planes * Cin_p], plane j holding the 16-bit rounding of w
// ("high") or, where bit j of lo_mask is set, the rounding of what that left
// over ("low").  The convolution over the widened input-channel axis is then
// x_hi*w + x_lo*w [+ x_hi*w_lo].
template <typename T>
__global__ void widen_weights_kernel(const float* __restrict__ Wd32, T* __restrict__ Wd, int Cin_p,
                                     int Kp, int planes, unsigned lo_mask) {
    const size_t rows = (size_t)9 * Kp;
    const size_t total = rows * planes * Cin_p;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int c = i % Cin_p;
        const int j = (i / Cin_p) % planes;
        const size_t row = i / ((size_t)Cin_p * planes);
        const float w = Wd32[row * Cin_p + c];
        const T hi = (T)w;
        Wd[i] = ((lo_mask >> j) & 1u) ? (T)(w - (float)hi) : hi;
    }
}

// The weights once more in e5m2, for the MMAs of the e5m2 activation planes:
// Wd32[9][Kp][Cin_p] fp32 -> W8[9][Kp][Cin8] bytes, zero padded (Cin8 a multiple
// of 128, one 128-byte swizzle row).  Bytes [0, Cin_p): e5m2(w), the partner of
// the activations' low plane.  With with_remainder, bytes [Cin_p, 2 Cin_p):
// e5m2(kWLoScale (w - fp16(w))), the partner of the activations' hi8 plane.
__global__ void weights_to_e5m2_kernel(const float* __restrict__ Wd32, unsigned char* __restrict__ W8,
                                       int Cin_p, int Cin8, int Kp, int with_remainder) {
    const size_t total = (size_t)9 * Kp * Cin8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int c = i % Cin8;
        const size_t row = i / Cin8;
        uint32_t b = 0;
        if (c < Cin_p) {
            b = e5m2_from_float(Wd32[row * Cin_p + c]);
        } else if (with_remainder && c < 2 * Cin_p) {
            const float w = Wd32[row * Cin_p + c - Cin_p];
            b = e5m2_from_float(kWLoScale * (w - __half2float(__float2half_rn(w))));
        }
        W8[i] = static_cast<unsigned char>(b);
    }
}

// 1x1 head convolutions reading the padded cell-major layout (see
// head_conv_kernel for the arithmetic).  One warp per board cell.
// ldx: elements (of T) per cell row of X; lo_off > 0: activations are two
// planes, the low one lo_off elements after the high one, stored as T or,
// with lo_e5m2, as one e5m2 byte per channel.
template <typename T>
__global__ void __launch_bounds__(256) head_conv_cells_kernel(
    const T* __restrict__ X, const float* __restrict__ w, int Cp, int cells,
    float* __restrict__ pol, float* __restrict__ val, int ldx, int lo_off, int lo_e5m2) {
    using P2 = Pair<T>;
    const int lane = threadIdx.x & 31;
    const int cell = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (cell >= cells) return;
    const int n = cell / kSq, s = cell % kSq;
    const T* x = X + (size_t)cell_of(n, s / kBoard, s % kBoard) * ldx;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;
    for (int c = 2 * lane; c < Cp; c += 64) {
        float2 v = P2::to_f2(*reinterpret_cast<const typename P2::type*>(x + c));
        if (lo_off > 0 && lo_e5m2) {
            const unsigned short two =
                *reinterpret_cast<const unsigned short*>(reinterpret_cast<const unsigned char*>(x + lo_off) + c);
            v.x += e5m2_to_float(two);
            v.y += e5m2_to_float(two >> 8);
        } else if (lo_off > 0) {
            const float2 l = P2::to_f2(*reinterpret_cast<const typename P2::type*>(x + lo_off + c));
            v.x += l.x;
            v.y += l.y;
        }
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
        pol[((size_t)n * 2 + 0) * kSq + s] = a0;
        pol[((size_t)n * 2 + 1) * kSq + s] = a1;
        val[(size_t)n * kSq + s] = a2;
    }
}

// padded cell-major <-> fp32 NCHW (diagnostics)
template <typename T>
__global__ void nchw_to_cells_kernel(const float* __restrict__ src, T* __restrict__ dst, int n, int C,
                                     int Cp) {
    const long long total = cells_for(n) * Cp;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int ch = static_cast<int>(i % Cp);
        const int q = static_cast<int>(i / Cp);
        const int c = q % kCellsPerRow, r = q / kCellsPerRow;
        float v = 0.f;
        if (c != 0 && (r % 20) != 0 && ch < C) {
            v = src[((size_t)(r / 20) * C + ch) * kSq + (r % 20 - 1) * kBoard + c - 1];
        }
        dst[i] = (T)v;
    }
}

template <typename T>
__global__ void cells_to_nchw_kernel(const T* __restrict__ src, float* __restrict__ dst, int n, int C,
                                     int Cp) {
    const size_t total = (size_t)n * C * kSq;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int s = i % kSq;
        const int c = (i / kSq) % C;
        const int b = i / ((size_t)C * kSq);
        dst[i] = (float)src[(size_t)cell_of(b, s / kBoard, s % kBoard) * Cp + c];
    }
}

}  // namespace dc
}  // namespace lzb
