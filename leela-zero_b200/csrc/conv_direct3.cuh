// The implicit-GEMM convolution for SMALL batches: the input channels of one
// 256-cell tile are split over the CTA pairs of one cluster.
//
// Why.  With few positions there are few 256-cell tiles (13 for 8 positions),
// and one tile is 144 dependent MMAs (9 taps x 4 channel chunks x 4) of about
// 128 cycles each on its CTA pair.  Cutting the OUTPUT channels of a tile into
// slices (conv_direct2.cuh) spreads the tile over more SMs but does not make
// it faster: measured on B200, a tcgen05.mma of 256 x 64 x 16 takes as long as
// one of 256 x 256 x 16 (the unit streams the M rows, N rides along), so every
// slice still spends 144 full MMA times.  Cutting the REDUCTION does: here pair
// p of the cluster takes input-channel chunk p (64 channels, all 9 taps, all
// output channels: 36 MMAs of 256 x 256 x 16), and the partial sums meet
// through distributed shared memory.
//
// Cluster = 2 * kchunks CTAs (kchunks = input channels / 64, 2..4).  Rank r:
// pair p = r / 2 works on chunk p; h = r % 2 is the half (128 cells) of the
// tile, as in conv_direct2.cuh.  One tile per cluster, nothing is reused, so
// every mbarrier completes exactly one phase.
//
//   1. every CTA loads its activation window (176 x 64) and its half of the 9
//      weight tiles of chunk p (9 x 16 KB), all at once;
//   2. the pair's leader issues 36 MMAs into tensor memory and commits;
//   3. output channels are cut into kchunks groups of 64; CTA (p, h) will
//      finish group p of its 128 cells.  Each epilogue warp reads the partial
//      sums of the groups its CTA does not own from tensor memory into a send
//      area in its own shared memory, 32 cells x 32 channels (4 KB) per block;
//   4. cluster barrier: every pair's MMAs have retired, so the operand area of
//      every CTA is dead and becomes its receive area; one thread then sends
//      each owner its eight blocks (32 KB, contiguous on both sides) with a bulk
//      shared-to-shared::cluster copy that completes on the owner's mbarrier.  (Scattered st.shared::cluster
//      from the tensor-memory register layout was measured first: 16-byte
//      packets, 5 us for the 96 KB a CTA sends.)
//   5. the owner waits for its incoming bytes, adds its own partial and the
//      received ones in chunk order, applies batch-norm / residual / ReLU and
//      stores the tile by TMA exactly like the other kernels.
//
// Two-plane activations (kPlanes == 3, LZB_FP16_X2): the e5m2 planes of a cell
// row are cut into 128-byte chunks exactly as conv_direct2.cuh cuts them, and
// there are never more of them than fp16 chunks.  Pair p < nlow runs e5m2 chunk
// p as a second pass into the same accumulator: its window has a buffer of its
// own (the operand area is sized for the exchange and has 26 KB to spare while
// the MMAs run), and its nine weight tiles reuse the nine fp16 slots one by
// one, each as soon as the fp16 MMAs of that tap have retired (one commit and
// one "slot free" barrier per tap), so that the second pass's loads trail the
// first pass's MMAs by one tap.  The epilogue is the two-plane one of the other
// kernels (fp16 tile by TMA, byte planes by direct stores).
//
// All waits on mbarriers are bounded; a thread that gives up still arrives at
// every cluster barrier, so its peers are never left waiting.
#pragma once
#include "conv_direct2.cuh"

namespace lzb {
namespace dc3 {

using namespace tc;
using namespace dc;
using dc2::cluster_ctarank;
using dc2::map_to_cta;
using dc2::cluster_sync_all;
using dc2::mbar_expect_tx_cluster;
using dc2::tma_load_2d_pair;
using dc2::tcgen05_mma_f16_pair;
using dc2::tcgen05_mma_f8_pair;
using dc2::kPairM;

constexpr int kTaps = 9;
constexpr uint32_t kWStageBytes = (kMaxN / 2) * 128;           // 16 KB: one tap, half the output channels
constexpr uint32_t kWAreaBytes = kTaps * kWStageBytes;        // 144 KB
constexpr int kGroupCols = 64;                                 // output channels finished per CTA
constexpr uint32_t kBlockBytes = 32 * 32 * 4;                  // 32 cells x 32 channels of fp32 partial sums
constexpr uint32_t kSlotBytes = 8 * kBlockBytes;               // one sender's 128 x 64: a block per epilogue warp
constexpr int kMaxSplit = 4;
constexpr uint32_t kExchangeBytes = (kMaxSplit - 1) * kSlotBytes;      // 96 KB received, 96 KB sent
// After the MMAs the operand area is reused: [receive area][send area].
constexpr uint32_t kOperand3Bytes =
    2 * kExchangeBytes > kWinBytes + kWAreaBytes ? 2 * kExchangeBytes : kWinBytes + kWAreaBytes;
constexpr uint32_t kD3SmemBytes =
    kOperand3Bytes + 8 * kStageOutBytes + 2 * kMaxN * 4 + kBarBytes + 1024;
static_assert(kD3SmemBytes <= 227 * 1024, "shared memory of one CTA");
static_assert(kOperand3Bytes >= 2 * kWinBytes + kWAreaBytes, "room for the second pass's window");
constexpr uint32_t kTmemCols3 = 256;

constexpr int kErrD3MmaFull = 401;
constexpr int kErrD3Epilogue = 402;
constexpr int kErrD3Producer = 403;

// Arrive on the barrier at this offset in the two CTAs `first`, `first + 1` of
// the cluster once the pair's MMAs issued so far have retired.
__device__ __forceinline__ void tcgen05_commit_to_pair(uint32_t bar, uint32_t first) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(bar),
        "h"(static_cast<uint16_t>(3u << first))
        : "memory");
}
// Copy `bytes` of this CTA's shared memory into another CTA of the cluster; the
// bytes are counted on a barrier of the receiving CTA.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes,
                                                 uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(dst_cluster),
        "r"(src_cta), "r"(bytes), "r"(bar_cluster)
        : "memory");
}
// 16-byte word v of row `row` inside a 32 x 128-byte block sits at slot
// v ^ (row & 7): conflict-free for threads that own a row each, on both sides.
__device__ __forceinline__ uint32_t block_word(int row, int v) {
    return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(v ^ (row & 7)) << 4);
}

// tmX : activations [Qa][Cin], box 64 x kWinRows.
// tmW : weights [9*Kp][Cin], box 64 x Kp/2.
// tmO : outputs [Qa][Kp], box 32 x 32, 64-byte swizzle.
// Launched with cluster dimension 2 * kchunks and grid = tiles * 2 * kchunks;
// requires Kp == 64 * kchunks (a tower layer: as many output groups as chunks).
// achunks : 64-channel chunks the activation tensor has; weight chunk c >= achunks
// is paired with activation chunk c - achunks (a second set of weight planes
// against the same activations, as in conv_direct2_kernel).
// tmXl, tmWl : byte maps over the e5m2 planes of the activations and over the
// e5m2 weights (box 128 x kWinRows, box 128 x Kp/2); nlow : e5m2 chunks of
// this layer (0 .. kchunks); ldr : elements of T per cell row of the residual
// tensor; out_lo, out_hi8, out_pitch, q_rows as in conv_direct2_kernel.  All
// ignored when kPlanes == 1 except ldr.
template <typename T, int kPlanes>
__global__ void __launch_bounds__(kDcThreads, 1) conv_ksplit_kernel(
    const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
    const __grid_constant__ CUtensorMap tmO, const T* res, const float* __restrict__ bn_mean,
    const float* __restrict__ bn_invstd, int Q, int Kp, int kchunks, int* err,
    const __grid_constant__ CUtensorMap tmXl, const __grid_constant__ CUtensorMap tmWl, int nlow,
    int ldr, unsigned char* out_lo, unsigned char* out_hi8, int out_pitch, int q_rows, int achunks) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (base - raw);
    const uint32_t win_base = base;
    const uint32_t w_base = base + kWinBytes;
    const uint32_t win2_base = base + kWinBytes + kWAreaBytes;   // second pass's window
    unsigned char* recv = smem;                               // the operand area after step 4:
    unsigned char* send = smem + kExchangeBytes;              // [receive area][send area]
    unsigned char* stage_out = smem + kOperand3Bytes;
    float* s_scale = reinterpret_cast<float*>(stage_out + 8 * kStageOutBytes);
    float* s_bias = s_scale + kMaxN;
    unsigned char* bar_mem = stage_out + 8 * kStageOutBytes + 2 * kMaxN * 4;
    const uint32_t bars = smem_u32(bar_mem);
    auto bfull_bar = [&](int t) { return bars + 8u * (0 + t); };      // the pair leader's are used
    const uint32_t wfull_bar = bars + 8u * 9;                          // leader's
    const uint32_t tfull_bar = bars + 8u * 10;                         // both CTAs of the pair
    const uint32_t rfull_bar = bars + 8u * 11;                         // every CTA: incoming partial sums
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * 12 + 8);
    auto bempty_bar = [&](int t) { return bars + 8u * (16 + t); };    // both CTAs of the pair: slot t is free
    const uint32_t wfull2_bar = bars + 8u * 25;                        // leader's: second pass's window

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t p = rank >> 1, h = rank & 1u;       // chunk of this pair, half of the tile
    const uint32_t lead = rank & ~1u;                  // cluster rank of the pair's leader
    const int csize = 2 * kchunks;
    const int tile = blockIdx.x / csize;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kTaps; i++) mbar_init(bfull_bar(i), 2);   // one arrive.expect_tx per CTA
        mbar_init(wfull_bar, 2);
        mbar_init(tfull_bar, 1);
        mbar_init(rfull_bar, 1);
        for (int i = 0; i < kTaps; i++) mbar_init(bempty_bar(i), 1);
        mbar_init(wfull2_bar, 2);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i = threadIdx.x; i < Kp; i += blockDim.x) {
        s_scale[i] = bn_invstd[i];
        s_bias[i] = -bn_mean[i] * bn_invstd[i];
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(kTmemCols3)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();          // every CTA's barriers exist before anyone signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // (kchunks - 1) senders x 8 blocks will arrive here
    if (threadIdx.x == 0) mbar_expect_tx(rfull_bar, static_cast<uint32_t>(kchunks - 1) * kSlotBytes);
    const int half_n = Kp >> 1;                        // weight rows each CTA stages per tap
    const int m0 = tile * kPairM + static_cast<int>(h) * kTileM;
    // this pair's second pass: e5m2 chunk p of the activation planes
    const bool pass2 = kPlanes == 3 && static_cast<int>(p) < nlow;

    // ------------------------------------------------ TMA producer (warp 0 of every CTA)
    // The weights are constant, so their tiles are requested before this kernel
    // waits for its predecessor: where the CTA got an SM early (a small layer
    // leaves most of them free) they arrive while the previous layer still runs.
    if (warp == 0 && lane == 0) {
        const uint32_t btx = static_cast<uint32_t>(half_n) * 128u;
        for (int tap = 0; tap < kTaps; ++tap) {
            const uint32_t bf = map_to_cta(bfull_bar(tap), lead);
            mbar_expect_tx_cluster(bf, btx);
            tma_load_2d_pair(w_base + tap * kWStageBytes, &tmW, static_cast<int>(p) * kChunkK,
                             tap * Kp + static_cast<int>(h) * half_n, bf);
        }
    }
    // inputs, residuals and outputs belong to the chain of kernels in the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t wf = map_to_cta(wfull_bar, lead);
            mbar_expect_tx_cluster(wf, kWinBytes);
            const int achunk = static_cast<int>(p) < achunks ? static_cast<int>(p) : static_cast<int>(p) - achunks;
            tma_load_2d_pair(win_base, &tmX, achunk * kChunkK, m0 - kWinPad, wf);
            if (pass2) {
                const uint32_t wf2 = map_to_cta(wfull2_bar, lead);
                mbar_expect_tx_cluster(wf2, kWinBytes);
                tma_load_2d_pair(win2_base, &tmXl, static_cast<int>(p) * 128, m0 - kWinPad, wf2);
                const uint32_t btx = static_cast<uint32_t>(half_n) * 128u;
                for (int tap = 0; tap < kTaps; ++tap) {
                    // slot `tap` is free once the first pass's MMAs of that tap have retired
                    if (!mbar_wait(bempty_bar(tap), 0u, abort_flag, err, kErrD3Producer)) break;
                    const uint32_t bf = map_to_cta(bfull_bar(tap), lead);
                    mbar_expect_tx_cluster(bf, btx);
                    tma_load_2d_pair(w_base + tap * kWStageBytes, &tmWl, static_cast<int>(p) * 128,
                                     tap * Kp + static_cast<int>(h) * half_n, bf);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (pair leaders)
        if (lane == 0 && h == 0) {
            const uint32_t idesc = (1u << 4) | (OperandFormat<T>::value << 7) |
                                   (OperandFormat<T>::value << 10) |
                                   (static_cast<uint32_t>(Kp >> 3) << 17) |
                                   (static_cast<uint32_t>(kPairM >> 4) << 24);
            bool ok = mbar_wait(wfull_bar, 0u, abort_flag, err, kErrD3MmaFull);
            for (int tap = 0; tap < kTaps && ok; ++tap) {
                ok = mbar_wait(bfull_bar(tap), 0u, abort_flag, err, kErrD3MmaFull);
                if (!ok) break;
                tcgen05_fence_after();
                const int row0 = kWinPad + (tap / 3 - 1) * kCellsPerRow + (tap % 3 - 1);
                const uint64_t a_desc = umma_desc_sw128(win_base + static_cast<uint32_t>(row0) * 128u);
                const uint64_t b_desc = umma_desc_sw128(w_base + tap * kWStageBytes);
#pragma unroll
                for (int k = 0; k < kChunkK / 16; ++k) {
                    tcgen05_mma_f16_pair(tmem_base, a_desc + 2u * k, b_desc + 2u * k, idesc,
                                         (tap > 0 || k > 0) ? 1u : 0u);
                }
                if (pass2) tcgen05_commit_to_pair(bempty_bar(tap), lead);
            }
            if (pass2 && ok) {
                // e5m2 x e5m2 -> fp32, K = 32 per instruction: again 32 bytes of every row
                const uint32_t idesc8 = (1u << 4) | (1u << 7) | (1u << 10) |
                                        (static_cast<uint32_t>(Kp >> 3) << 17) |
                                        (static_cast<uint32_t>(kPairM >> 4) << 24);
                ok = mbar_wait(wfull2_bar, 0u, abort_flag, err, kErrD3MmaFull);
                for (int tap = 0; tap < kTaps && ok; ++tap) {
                    ok = mbar_wait(bfull_bar(tap), 1u, abort_flag, err, kErrD3MmaFull);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const int row0 = kWinPad + (tap / 3 - 1) * kCellsPerRow + (tap % 3 - 1);
                    const uint64_t a_desc = umma_desc_sw128(win2_base + static_cast<uint32_t>(row0) * 128u);
                    const uint64_t b_desc = umma_desc_sw128(w_base + tap * kWStageBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tcgen05_mma_f8_pair(tmem_base, a_desc + 2u * k, b_desc + 2u * k, idesc8, 1u);
                    }
                }
            }
            // also after a failed wait: the epilogue warps of both CTAs must not
            // sit out their own limit on a barrier nobody will complete
            tcgen05_commit_to_pair(tfull_bar, lead);
        }
    }

    // ---------------------------------------------------- epilogue warps 2..9
    const bool epi = warp >= 2;
    const int qd = warp & 3;                                   // tensor-memory lane quadrant
    const int side = epi ? (warp - 2) >> 2 : 0;                // which half of a 64-column group
    const uint32_t tlane = static_cast<uint32_t>(qd * 32) << 16;
    bool ok = true;
    if (epi) {
        if (lane == 0) ok = mbar_wait(tfull_bar, 0u, abort_flag, err, kErrD3Epilogue);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        tcgen05_fence_after();
    }
    const int blk = epi ? qd * 2 + side : 0;                   // this warp's block inside a slot
    if (epi && ok) {
        // step 3: the groups this CTA does not own, from tensor memory to the
        // send area (this CTA's own weight tiles: its pair's MMAs have retired)
        int gi = 0;
        for (int g = 0; g < kchunks; ++g) {
            if (g == static_cast<int>(p)) continue;
            uint32_t r[32];
            LZB_TMEM_LD32(r, tmem_base + tlane + static_cast<uint32_t>(g * kGroupCols + side * 32));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            unsigned char* dst = send + static_cast<size_t>(gi) * kSlotBytes + blk * kBlockBytes;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                *reinterpret_cast<uint4*>(dst + block_word(lane, v)) =
                    make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            }
            ++gi;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    cluster_sync_all();          // step 4: every pair's MMAs have retired; operands are dead
    // one copy per owner: the eight blocks of a slot are contiguous on both sides
    if (warp == 2 && lane == 0 && ok) {
        int gi = 0;
        for (int g = 0; g < kchunks; ++g) {
            if (g == static_cast<int>(p)) continue;
            const int slot = static_cast<int>(p) < g ? static_cast<int>(p) : static_cast<int>(p) - 1;
            const uint32_t owner = static_cast<uint32_t>(2 * g) + h;
            bulk_copy_to_cta(map_to_cta(smem_u32(recv) + static_cast<uint32_t>(slot) * kSlotBytes, owner),
                             smem_u32(send) + static_cast<uint32_t>(gi) * kSlotBytes, kSlotBytes,
                             map_to_cta(rfull_bar, owner));
            ++gi;
        }
    }
    __syncwarp();

    if (epi && ok) {
        // step 5
        const int col0 = static_cast<int>(p) * kGroupCols + side * 32;     // output channels of this warp
        const int row0 = m0 + qd * 32;
        const int q = row0 + lane;
        const bool interior = cell_is_interior(q, Q);
        const bool use_res = (res != nullptr) && interior;
        uint4 rv[4], re[2];
        load_residual(rv, res + static_cast<size_t>(q) * ldr + col0, use_res);
        if constexpr (kPlanes == 3) {
            // e5m2 plane of the same row: Kp bytes after the Kp 16-bit channels
            load_residual8(re, reinterpret_cast<const unsigned char*>(res + static_cast<size_t>(q) * ldr + Kp) + col0,
                           use_res);
        }
        uint32_t own[32];
        LZB_TMEM_LD32(own, tmem_base + tlane + static_cast<uint32_t>(col0));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (lane == 0) ok = mbar_wait(rfull_bar, 0u, abort_flag, err, kErrD3Epilogue);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
            // add in chunk order, whichever chunk is this CTA's own
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.f;
            for (int c = 0; c < kchunks; ++c) {
                if (c == static_cast<int>(p)) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] += __uint_as_float(own[i]);
                } else {
                    const int slot = c < static_cast<int>(p) ? c : c - 1;
                    const unsigned char* src = recv + static_cast<size_t>(slot) * kSlotBytes + blk * kBlockBytes;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 f = *reinterpret_cast<const float4*>(src + block_word(lane, v));
                        acc[4 * v] += f.x;
                        acc[4 * v + 1] += f.y;
                        acc[4 * v + 2] += f.z;
                        acc[4 * v + 3] += f.w;
                    }
                }
            }
            uint32_t r[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(acc[i]);
            unsigned char* stg_ptr = stage_out + (warp - 2) * kStageOutBytes;
            if constexpr (kPlanes == 3) {
                uint32_t lo[8], h8[8];
                epilogue_chunk_e5m2<T>(r, rv, re, s_scale + col0, s_bias + col0, use_res, interior,
                                       stg_ptr + lane * 64, lane, lo, h8, out_hi8 != nullptr);
                store_staged_tile(&tmO, smem_u32(stg_ptr), col0, row0, lane);
                if (q < q_rows) {
                    const size_t off = static_cast<size_t>(q) * out_pitch + col0;
                    if (out_lo != nullptr) {
                        uint4* dst = reinterpret_cast<uint4*>(out_lo + off);
                        dst[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        dst[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                    }
                    if (out_hi8 != nullptr) {
                        uint4* dst = reinterpret_cast<uint4*>(out_hi8 + off);
                        dst[0] = make_uint4(h8[0], h8[1], h8[2], h8[3]);
                        dst[1] = make_uint4(h8[4], h8[5], h8[6], h8[7]);
                    }
                }
            } else {
                epilogue_chunk<T>(r, rv, s_scale + col0, s_bias + col0, use_res, interior,
                                  stg_ptr + lane * 64, lane);
                store_staged_tile(&tmO, smem_u32(stg_ptr), col0, row0, lane);
            }
            if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();          // nobody retires while a peer may still touch it
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(kTmemCols3)
                     : "memory");
    }
}

}  // namespace dc3
}  // namespace lzb
