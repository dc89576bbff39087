// Winograd F(4x4, 3x3) arithmetic shared by the transform kernels.
//
// The interpolation points are 0, +-sqrt(2)/2, +-sqrt(2) and infinity, the set
// Leela Zero uses (B^T: src/CPUPipe.cpp:81-87, A^T: src/CPUPipe.cpp:220-224),
// and the factored evaluation order is the reference's, so that in fp32 the
// transforms produce the same values as the CPU pipe.
//
// Every routine works on a pair of channels at once (float2), because the
// kernels give each thread two adjacent channels of one tile.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace lzb {

constexpr int kBoard = 19;
constexpr int kSq = 361;
constexpr int kInputPlanes = 18;
constexpr int kTilesPerSide = 5;
constexpr int kTilesPerPos = 25;   // P
constexpr int kPoints = 36;        // alpha^2
constexpr float kSq2 = 1.4142135623730951f;

__device__ __forceinline__ float2 operator-(float2 a) { return make_float2(-a.x, -a.y); }

// Two flavours of every operation: kExact keeps multiplies and adds apart
// (__fmul_rn/__fadd_rn are never contracted into FMAs), so that the fp32 path
// reproduces the CPU pipe's transform values bit for bit; the other flavour
// lets the compiler fuse, which halves the instruction count and is used where
// the result is rounded to 16 bits anyway.
template <bool kExact> __device__ __forceinline__ float op_mul(float a, float b) {
    return kExact ? __fmul_rn(a, b) : a * b;
}
template <bool kExact> __device__ __forceinline__ float op_add(float a, float b) {
    return kExact ? __fadd_rn(a, b) : a + b;
}
__device__ __forceinline__ float nf_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float nf_add(float a, float b) { return __fadd_rn(a, b); }
template <bool kExact> __device__ __forceinline__ float2 mul2(float2 a, float s) {
    return make_float2(op_mul<kExact>(a.x, s), op_mul<kExact>(a.y, s));
}
template <bool kExact> __device__ __forceinline__ float2 add2(float2 a, float2 b) {
    return make_float2(op_add<kExact>(a.x, b.x), op_add<kExact>(a.y, b.y));
}
template <bool kExact> __device__ __forceinline__ float2 sub2(float2 a, float2 b) {
    return make_float2(op_add<kExact>(a.x, -b.x), op_add<kExact>(a.y, -b.y));
}

// o = B^T i, factored as in src/CPUPipe.cpp:88-106.
template <bool kExact>
__device__ __forceinline__ void apply_bt(float2 (&o)[6], const float2 (&i)[6]) {
    float2 a = add2<kExact>(mul2<kExact>(i[1], -kSq2), mul2<kExact>(i[3], kSq2 / 2.0f));
    float2 b = add2<kExact>(mul2<kExact>(i[2], -2.0f), i[4]);
    o[0] = add2<kExact>(add2<kExact>(i[0], mul2<kExact>(i[2], -5.0f / 2.0f)), i[4]);
    o[1] = add2<kExact>(a, b);
    o[2] = add2<kExact>(-a, b);
    float2 a2 = add2<kExact>(mul2<kExact>(i[3], kSq2), mul2<kExact>(i[1], -kSq2 / 2.0f));
    float2 b2 = add2<kExact>(mul2<kExact>(i[2], -1.0f / 2.0f), i[4]);
    o[3] = add2<kExact>(a2, b2);
    o[4] = add2<kExact>(-a2, b2);
    o[5] = add2<kExact>(add2<kExact>(i[1], mul2<kExact>(i[3], -5.0f / 2.0f)), i[5]);
}

// o = A^T i, factored as in src/CPUPipe.cpp:225-238.
template <bool kExact>
__device__ __forceinline__ void apply_at(float2 (&o)[4], const float2 (&i)[6]) {
    float2 t1p2 = mul2<kExact>(add2<kExact>(i[1], i[2]), 1.0f / 2.0f);
    float2 t1m2 = mul2<kExact>(sub2<kExact>(i[1], i[2]), kSq2 / 4.0f);
    float2 t3p4 = add2<kExact>(i[3], i[4]);
    float2 t3m4 = mul2<kExact>(sub2<kExact>(i[3], i[4]), kSq2);
    o[0] = add2<kExact>(add2<kExact>(add2<kExact>(i[0], t1p2), t1p2), t3p4);
    o[1] = add2<kExact>(add2<kExact>(t1m2, t1m2), t3m4);
    o[2] = add2<kExact>(add2<kExact>(t1p2, t3p4), t3p4);
    o[3] = add2<kExact>(add2<kExact>(add2<kExact>(t1m2, t3m4), t3m4), i[5]);
}

// ---- two adjacent channels of storage type T <-> float2 -------------------

template <typename T> struct Pair;
template <> struct Pair<float> {
    static constexpr bool exact = true;      // fp32 storage: keep the CPU pipe's operation order
    using type = float2;
    static __device__ __forceinline__ float2 to_f2(float2 v) { return v; }
    static __device__ __forceinline__ float2 from_f2(float2 v) { return v; }
    static __device__ __forceinline__ float2 zero() { return make_float2(0.f, 0.f); }
};
template <> struct Pair<__half> {
    static constexpr bool exact = false;
    using type = __half2;
    static __device__ __forceinline__ float2 to_f2(__half2 v) { return __half22float2(v); }
    static __device__ __forceinline__ __half2 from_f2(float2 v) { return __float22half2_rn(v); }
    static __device__ __forceinline__ __half2 zero() { return __float2half2_rn(0.f); }
};
template <> struct Pair<__nv_bfloat16> {
    static constexpr bool exact = false;
    using type = __nv_bfloat162;
    static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
    static __device__ __forceinline__ __nv_bfloat162 from_f2(float2 v) { return __float22bfloat162_rn(v); }
    static __device__ __forceinline__ __nv_bfloat162 zero() { return __float2bfloat162_rn(0.f); }
};

}  // namespace lzb
