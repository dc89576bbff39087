// The 36 channel contractions on the Blackwell tensor cores (sm_100a):
//   M[t][p][k] = sum_c V[t][p][c] * U[t][k][c],   t = 0..35
// fp16 or bf16 operands, fp32 accumulation in tensor memory.
//
// Shape of the work.  V is [36][Pa][Cin] and U is [36][Kp][Cin] with the
// reduction axis c innermost on both (K-major operands).  One work item is a
// (t, block of 128 rows p) pair: a 128 x Kp x Cin product, Kp <= 256,
// Cin = 64 * kchunks <= 256.  Items are numbered t-major and each persistent
// CTA (one per SM) takes a contiguous range, so that the weights U[t] it holds
// in shared memory (128 KB at 256 x 256) are reloaded only when t changes and
// only the V rows stream through the 4-stage ring.
//
// Roles inside a CTA (6 warps):
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma and commits
//   warps 2-5 epilogue: tcgen05.ld the 128 x Kp fp32 accumulator, convert to
//            the storage type and write M rows; two accumulators (2 x 256
//            columns) alternate so the epilogue of item i overlaps the MMAs of
//            item i+1.
// Synchronisation is by mbarriers only.  Every wait is bounded: after
// kWaitLimitNs without progress the waiting thread records a code in *err,
// raises a CTA-wide abort flag and all roles leave their loops, the tensor
// memory is released and the kernel returns; the host reports
// LZB_ERR_DEVICE_WAIT.
//
// This kernel stands where the reference launches XgemmBatched / the wmma
// HGEMM (src/OpenCL.cpp:404-426, src/kernels/clblast/hgemm_tensorcore.opencl);
// it needs no tuner because the shape family is closed.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace lzb {
namespace tc {

constexpr int kBlockM = 128;        // rows p per work item (tensor-memory lanes)
constexpr int kChunkK = 64;         // reduction elements per smem tile row (128 bytes)
constexpr int kMaxN = 256;          // output channels per MMA (tensor-memory columns)
constexpr int kMaxChunks = 4;       // Cin <= 256
constexpr int kStages = 4;          // V ring depth
constexpr int kThreads = 192;
constexpr uint32_t kVStageBytes = kBlockM * 128;   // 16 KB
constexpr uint32_t kUChunkBytes = kMaxN * 128;     // 32 KB
constexpr uint32_t kBarBytes = 1024;
constexpr uint32_t kSmemBytes =
    kMaxChunks * kUChunkBytes + kStages * kVStageBytes + kBarBytes + 1024 /* alignment slack */;
constexpr uint32_t kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s

// error codes written to *err (first one wins)
constexpr int kErrProducerUEmpty = 101;
constexpr int kErrProducerVEmpty = 102;
constexpr int kErrMmaAccEmpty = 103;
constexpr int kErrMmaUFull = 104;
constexpr int kErrMmaVFull = 105;
constexpr int kErrEpilogueFull = 106;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the CTA is aborting or the limit ran out.
// The limit must be exceeded on two independent counters, the global
// nanosecond timer and the SM cycle counter (>= 1 cycle per ns at any clock the
// part runs kernels at), so that a step in either of them cannot end a wait
// early.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            int* err, int code,
                                            unsigned long long limit_ns = kWaitLimitNs) {
    const unsigned long long t0 = globaltimer_ns();
    const long long c0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 31u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns &&
                static_cast<unsigned long long>(clock64() - c0) > limit_ns) {
                *abort_flag = 1;
                atomicCAS(err, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* err, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, err, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, one 128 x N x 16 step.
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes
// (64 16-bit elements) under the 128-byte swizzle TMA writes: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused for
// swizzled K-major tiles and set to 1 unit, descriptor version 1 (sm_100).
// The swizzle phase is taken from the address bits, so the start address may
// be any 128-byte row of a 1024-byte-aligned tile (base-offset field 0), and
// +32 bytes steps 16 elements along K.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset
    d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                       // version
    d |= static_cast<uint64_t>(2) << 61;                       // SWIZZLE_128B
    return d;
}

#define LZB_TMEM_LD32(r, taddr)                                                                  \
    asm volatile(                                                                                \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "      \
        "[%32];"                                                                                 \
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),    \
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),             \
          "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),          \
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),          \
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),          \
          "=r"(r[31])                                                                            \
        : "r"(taddr)                                                                             \
        : "memory")

template <typename T> struct OperandFormat;
template <> struct OperandFormat<__half> { static constexpr uint32_t value = 0; };
template <> struct OperandFormat<__nv_bfloat16> { static constexpr uint32_t value = 1; };

__device__ __forceinline__ uint32_t pack2(__half, float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(__nv_bfloat16, float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// tmV: 2-D map over V seen as [36*Pa rows][Cin], box 64 x 128, swizzle 128B.
// tmU: 2-D map over U seen as [36*Kp rows][Cin], box 64 x Kp,  swizzle 128B.
// nblk = 128-row blocks per point (covering P rows); grid = persistent CTAs.
template <typename T>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(
    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU,
    T* __restrict__ M, int Pa, int P, int Kp, int kchunks, int nblk, int* err) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
    unsigned char* smem = smem_raw + (base - raw);
    const uint32_t u_base = base;
    const uint32_t v_base = base + kMaxChunks * kUChunkBytes;
    unsigned char* bar_mem = smem + kMaxChunks * kUChunkBytes + kStages * kVStageBytes;
    const uint32_t bars = smem_u32(bar_mem);
    // barrier slots (8 bytes each)
    auto full_bar = [&](int s) { return bars + 8u * (0 + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (4 + s); };
    auto ufull_bar = [&](int c) { return bars + 8u * (8 + c); };
    auto uempty_bar = [&](int c) { return bars + 8u * (12 + c); };
    auto tfull_bar = [&](int a) { return bars + 8u * (16 + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (18 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * 20 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; i++) {
            mbar_init(full_bar(i), 1);
            mbar_init(empty_bar(i), 1);
            mbar_init(ufull_bar(i), 1);
            mbar_init(uempty_bar(i), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);     // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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
    // launched with programmatic stream serialization: the set-up above overlaps
    // the tail of the previous kernel, V is only read after it has finished
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // V was written with ordinary stores and is read here by TMA (async proxy)
    asm volatile("fence.proxy.async;" ::: "memory");

    const int items = 36 * nblk;   // 36 Winograd points
    const int item_begin = static_cast<int>(static_cast<long long>(blockIdx.x) * items / gridDim.x);
    const int item_end = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * items / gridDim.x);

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, uphase = 0;
            int cur_t = -1;
            bool ok = true;
            for (int item = item_begin; item < item_end && ok; ++item) {
                const int t = item / nblk, pb = item - t * nblk;
                const bool new_t = (t != cur_t);
                for (int c = 0; c < kchunks && ok; ++c) {
                    if (new_t) {
                        ok = mbar_wait(uempty_bar(c), uphase ^ 1u, abort_flag, err, kErrProducerUEmpty);
                        if (!ok) break;
                        mbar_expect_tx(ufull_bar(c), static_cast<uint32_t>(Kp) * 128u);
                        tma_load_2d(u_base + c * kUChunkBytes, &tmU, c * kChunkK, t * Kp, ufull_bar(c));
                    }
                    ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, err, kErrProducerVEmpty);
                    if (!ok) break;
                    mbar_expect_tx(full_bar(stage), kVStageBytes);
                    tma_load_2d(v_base + stage * kVStageBytes, &tmV, c * kChunkK,
                                t * Pa + pb * kBlockM, full_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (new_t) { uphase ^= 1u; cur_t = t; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4)                                   // D is fp32
                                   | (OperandFormat<T>::value << 7)            // A format
                                   | (OperandFormat<T>::value << 10)           // B format
                                   | (static_cast<uint32_t>(Kp >> 3) << 17)    // N
                                   | (static_cast<uint32_t>(kBlockM >> 4) << 24);  // M
            int stage = 0;
            uint32_t phase = 0, ufphase = 0;
            int cur_t = -1;
            bool ok = true;
            int local = 0;
            for (int item = item_begin; item < item_end && ok; ++item, ++local) {
                const int t = item / nblk;
                const bool new_t = (t != cur_t);
                const bool last_of_t = (item + 1 == item_end) || ((item + 1) / nblk != t);
                const int acc = local & 1;
                const uint32_t accphase = (local >> 1) & 1u;
                ok = mbar_wait(tempty_bar(acc), accphase ^ 1u, abort_flag, err, kErrMmaAccEmpty);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kMaxN);
                for (int c = 0; c < kchunks && ok; ++c) {
                    if (new_t) {
                        ok = mbar_wait(ufull_bar(c), ufphase, abort_flag, err, kErrMmaUFull);
                        if (!ok) break;
                    }
                    ok = mbar_wait(full_bar(stage), phase, abort_flag, err, kErrMmaVFull);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint64_t a_desc = umma_desc_sw128(v_base + stage * kVStageBytes);
                    const uint64_t b_desc = umma_desc_sw128(u_base + c * kUChunkBytes);
#pragma unroll
                    for (int k = 0; k < kChunkK / 16; ++k) {
                        // advancing 16 elements (32 bytes) along K inside the swizzle row:
                        // +2 in the 16-byte-unit start address field
                        tcgen05_mma_f16(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                                        (c > 0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(empty_bar(stage));          // V stage free when these MMAs retire
                    if (last_of_t) tcgen05_commit(uempty_bar(c));   // and this U chunk too
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tcgen05_commit(tfull_bar(acc));                // accumulator complete
                if (new_t) { ufphase ^= 1u; cur_t = t; }
            }
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                 // tensor-memory lane quadrant this warp may read
        const T tag = T();
        int local = 0;
        for (int item = item_begin; item < item_end; ++item, ++local) {
            const int t = item / nblk, pb = item - t * nblk;
            const int acc = local & 1;
            const uint32_t accphase = (local >> 1) & 1u;
            bool ok = mbar_wait(tfull_bar(acc), accphase, abort_flag, err, kErrEpilogueFull);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const int p = pb * kBlockM + q * 32 + lane;
            T* mrow = M + (static_cast<size_t>(t) * Pa + p) * Kp;
            const uint32_t taddr0 =
                tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * kMaxN);
            for (int j = 0; j < Kp; j += 32) {
                uint32_t r[32];
                LZB_TMEM_LD32(r, taddr0 + j);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p < P) {
                    uint4* dst = reinterpret_cast<uint4*>(mrow + j);
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 o;
                        o.x = pack2(tag, __uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                        o.y = pack2(tag, __uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                        o.z = pack2(tag, __uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                        o.w = pack2(tag, __uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                        dst[v] = o;
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
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

}  // namespace tc
}  // namespace lzb
