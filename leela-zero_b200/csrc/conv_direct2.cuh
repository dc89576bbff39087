// The implicit-GEMM convolution of conv_direct.cuh on CTA PAIRS
// (tcgen05 cta_group::2): two CTAs of a 2-CTA cluster work on 256 consecutive
// output cells, 128 each.  Each CTA stages its own activation window and only
// HALF of every weight tile (128 of the 256 output channels); one
// tcgen05.mma.cta_group::2 of shape 256 x 256 x 16, issued by the leader CTA,
// reads both halves, and each CTA's tensor memory receives the accumulators of
// its own 128 cells.  Compared with one CTA per tile this halves the weight
// bytes every SM pulls from L2 and writes to shared memory (16 KB instead of
// 32 KB per k-step), which is what caps the single-CTA kernel.
//
// Protocol (leader = cluster rank 0):
//  * "full" barriers (weight stage, activation window) live in the leader and
//    expect one arrive.expect_tx from each CTA's producer; both CTAs' TMA loads
//    complete their bytes on the leader's barrier (cp.async.bulk.tensor
//    .cta_group::2).  Only the leader's MMA lane waits on them.
//  * "empty" barriers and the accumulator-full barriers exist in both CTAs at
//    the same shared-memory offset; the leader's tcgen05.commit arrives on both.
//  * accumulator-empty barriers live in the leader and collect the 8 epilogue
//    warps of each CTA (the follower's arrive remotely).
// Everything else (window addressing, epilogue, bounded waits) is shared with
// the single-CTA kernel.
#pragma once
#include "conv_direct.cuh"

namespace lzb {
namespace dc2 {

using namespace tc;
using namespace dc;

constexpr int kPairM = 2 * kTileM;                         // 256 cells per CTA pair
constexpr int kB2Stages = 10;                              // ring of half weight tiles
constexpr uint32_t kB2StageBytes = (kMaxN / 2) * 128;      // 16 KB
constexpr uint32_t kOperand2Bytes = kWinBufs * kWinBytes + kB2Stages * kB2StageBytes;
// The same shared memory cut differently when the output channels are sliced
// (small batches, a chain of short launches bound by load latency): all four
// activation windows of a unit in flight at once and fewer, fuller weight
// stages, each carrying the slices of up to three taps.
constexpr int kWinBufsSliced = 4;
constexpr int kB2StagesSliced = 7;
constexpr int kMaxTapsPerStage = 3;
static_assert(kWinBufsSliced * kWinBytes + kB2StagesSliced * kB2StageBytes <= kOperand2Bytes,
              "the sliced layout must fit the operand area");
constexpr uint32_t kD2SmemBytes =
    kOperand2Bytes + 8 * kStageOutBytes + 2 * kMaxN * 4 + kBarBytes + 1024;

constexpr int kErrD2Producer = 301;
constexpr int kErrD2MmaAcc = 302;
constexpr int kErrD2MmaFull = 303;
constexpr int kErrD2Epilogue = 304;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t d;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(d) : "r"(smem_addr), "r"(rank));
    return d;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load into THIS CTA's shared memory whose bytes complete on a barrier of the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                     uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with e5m2 / e4m3 operands (K = 32 per instruction: again 32 bytes of every row).
__device__ __forceinline__ void tcgen05_mma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                    uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive, once the pair's MMAs issued so far have retired, on the barrier at
// this shared-memory offset in BOTH CTAs of the pair.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(bar),
        "h"(static_cast<uint16_t>(3))
        : "memory");
}

// ---- per-tile dependencies between consecutive layers (whole-tile launches) ----
// A tile of one layer reads, through its window, only tiles i-1, i, i+1 of the
// layer before.  When the host passes flag arrays, a launch does not wait for
// the whole previous launch (griddepcontrol.wait): its producers wait for the
// flags of those three tiles instead, and its epilogue warps raise their own
// tile's flag once their stores have completed.  A dependent launch starts only
// after every CTA of its predecessor has started (both call
// griddepcontrol.launch_dependents first thing), so a flag that is waited for
// always has a running or finished writer.  Per tile there are two words: a
// counter of arrivals, 16 per evaluation of the tile (8 epilogue warps in each
// CTA of the pair; its value is always a multiple of 16 between evaluations,
// whatever batch sizes came before), and the number of the tower run that
// completed the tile last, stored by the sixteenth arrival.  Neither is reset.
constexpr uint32_t kFlagArrivals = 16;
constexpr unsigned long long kFlagWaitLimitNs = 250000000ull;   // a layer takes about 0.1 ms
constexpr int kErrD2Flags = 305;
constexpr int kMaxOrder = 16;          // tiles per CTA pair the visiting order is kept for

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t atom_acq_rel_gpu_add(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded like every other wait of this library.
__device__ __noinline__ bool flag_wait(const uint32_t* flag, uint32_t target, volatile int* abort_flag,
                                       int* err) {
    if (static_cast<int32_t>(ld_acquire_gpu(flag) - target) >= 0) return true;
    const unsigned long long t0 = globaltimer_ns();
    const long long c0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (static_cast<int32_t>(ld_acquire_gpu(flag) - target) >= 0) return true;
        __nanosleep(64);
        if ((spin & 31u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > kFlagWaitLimitNs &&
                static_cast<unsigned long long>(clock64() - c0) > kFlagWaitLimitNs) {
                *abort_flag = 1;
                atomicCAS(err, 0, kErrD2Flags);
                return false;
            }
        }
    }
}
// The k-th tile a pair visits in its range [begin, begin + n): from the middle
// outwards, the two ends last.  The first tile of a layer then depends on tiles
// this pair finished early in the layer before, and the end tiles, which depend
// on the neighbours' end tiles, come when those are long done.
__device__ __forceinline__ int middle_out(int k, int n) {
    const int m = n / 2;
    // distances 1, 1, 2, 2, ... alternate left and right of m until one side runs out
    const int left = m, right = n - 1 - m;           // tiles on either side of m
    const int paired = left < right ? left : right;  // distances with both sides present
    if (k == 0) return m;
    if (k <= 2 * paired) {
        const int d = (k + 1) / 2;
        return (k & 1) ? m - d : m + d;
    }
    const int d = k - paired;                        // beyond: only the longer side is left
    return left > right ? m - d : m + d;
}

// tmX : activations [Qa][Cin], box 64 x kWinRows.
// tmW : weights [9*Kp][Cin], box 64 x Kp/(2*nsplit) (one tap's rows of one CTA's
//       half slice; a stage of the ring takes up to three such boxes when sliced).
// tmO : outputs [Qa][Kp], box 32 x 32, 64-byte swizzle.
// npairs : 256-cell tiles covering Q.  nsplit : the output channels of a tile are
// cut into nsplit slices of N = Kp/nsplit (a multiple of 64), each slice a work
// unit of its own; used when there are fewer tiles than CTA pairs, so that a
// small batch spreads over more SMs.
//
// achunks : 64-channel chunks the activation tensor has; weight chunk c >= achunks
// is paired with activation chunk c - achunks (the weights may repeat the activations
// against a second, "low" set of weight planes).  kPlanes : 1, or 2 when the
// activations are carried as two 16-bit planes (high in channels [0, Kp), low in
// [Kp, 2 Kp) of tmO and res, see epilogue_chunk_x2), or 3 when low planes are
// e5m2: a cell row is [Kp x 16 bits | Kp bytes lo | (Kp bytes hi8)]; chunks
// c >= fchunks then come from tmXl / tmWl (byte maps, 128 channels per 128-byte
// chunk) and are multiplied by kind::f8f6f4 MMAs.  The byte planes of the
// output are written with plain 32-byte stores, one sector per cell and chunk,
// straight from the registers: out_lo (x - fp16(x) in e5m2, the residual reads it
// back) and, where the next layer corrects its weights as well, out_hi8
// (fp16(x) / 256 in e5m2, the operand of that layer's e5m2(256 (w - fp16(w)))
// plane); either may be null; out_pitch bytes per cell row, rows below q_rows
// exist.  tmXl, tmWl, out_lo, out_hi8 are ignored for the other kPlanes.
// ldr : elements of T per cell row of the residual tensor (its rows may be
// wider than Kp when the tensor also holds a low plane).
// flags_in, flags_out, counts_out, flag_target : per-tile dependencies (above);
// whole-tile launches only.  flags_out non-null: tiles are visited middle-out,
// arrivals are counted in counts_out and the tile's flag is set to flag_target
// (the number of this tower run) by the last one; flags_in non-null: the flags
// of the previous layer's tiles are waited for instead of the previous launch
// as a whole.
//
// The kernel is launched with programmatic stream serialization: it lets its
// successor start at once (griddepcontrol.launch_dependents) and itself waits
// for its predecessor's results only after its own set-up (barriers, tensor
// memory, batch-norm constants), which takes that set-up off the critical path
// of a chain of small layers.
template <typename T, int kPlanes, bool kSliced>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kDcThreads, 1) conv_direct2_kernel(
    const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
    const __grid_constant__ CUtensorMap tmO, const T* res, const float* __restrict__ bn_mean,
    const float* __restrict__ bn_invstd, int Q, int Kp, int kchunks, int npairs, int nsplit,
    int* err, int achunks, const __grid_constant__ CUtensorMap tmXl,
    const __grid_constant__ CUtensorMap tmWl, int ldr, unsigned char* out_lo, int out_pitch,
    int q_rows, int fchunks, unsigned char* out_hi8, const uint32_t* flags_in, uint32_t* flags_out,
    uint32_t* counts_out, uint32_t flag_target) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (base - raw);
    // kSliced (nsplit > 1) selects the shared-memory layout at compile time, so
    // that the loops of the whole-tile case keep constant bounds
    constexpr int nwin = kSliced ? kWinBufsSliced : kWinBufs;
    constexpr int nstages = kSliced ? kB2StagesSliced : kB2Stages;
    const uint32_t win_base = base;
    const uint32_t b_base = base + static_cast<uint32_t>(nwin) * kWinBytes;
    unsigned char* stage_out = smem + kOperand2Bytes;
    float* s_scale = reinterpret_cast<float*>(stage_out + 8 * kStageOutBytes);
    float* s_bias = s_scale + kMaxN;
    unsigned char* bar_mem = stage_out + 8 * kStageOutBytes + 2 * kMaxN * 4;
    const uint32_t bars = smem_u32(bar_mem);
    auto bfull_bar = [&](int s) { return bars + 8u * (0 + s); };      // leader's are used
    auto bempty_bar = [&](int s) { return bars + 8u * (16 + s); };    // both CTAs
    auto wfull_bar = [&](int w) { return bars + 8u * (32 + w); };     // leader's
    auto wempty_bar = [&](int w) { return bars + 8u * (36 + w); };    // both
    auto tfull_bar = [&](int a) { return bars + 8u * (40 + a); };     // both
    auto tempty_bar = [&](int a) { return bars + 8u * (42 + a); };    // leader's
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * 44);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * 44 + 8);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kB2Stages; i++) {
            mbar_init(bfull_bar(i), 2);      // one arrive.expect_tx per CTA of the pair
            mbar_init(bempty_bar(i), 1);
        }
        for (int i = 0; i < kWinBufsSliced; i++) {
            mbar_init(wfull_bar(i), 2);
            mbar_init(wempty_bar(i), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 16);    // 8 epilogue warps in each CTA
        }
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
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers are initialised before anyone signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // work units: (tile, channel slice), numbered tile-major
    const int nclusters = gridDim.x >> 1, cid = blockIdx.x >> 1;
    const int units = npairs * nsplit;
    const int unit_begin = static_cast<int>(static_cast<long long>(cid) * units / nclusters);
    const int unit_end = static_cast<int>(static_cast<long long>(cid + 1) * units / nclusters);
    const int n_slice = Kp / nsplit;          // MMA N
    const int half_n = n_slice >> 1;          // weight rows each CTA stages
    // taps whose weight slices share one stage of the ring (1 for whole tiles)
    const int taps_per_stage =
        kSliced ? ((kMaxN / 2) / half_n < kMaxTapsPerStage ? (kMaxN / 2) / half_n : kMaxTapsPerStage) : 1;

    // Activations, residuals and outputs belong to the chain of kernels in the
    // stream: nobody touches them before the previous kernel has finished.
    // (Starting the constant weight tiles ahead of this wait was tried and made
    // no measurable difference.)
    const bool tile_flags = !kSliced && flags_in != nullptr;    // wait per tile, not per launch
    if (!tile_flags) asm volatile("griddepcontrol.wait;" ::: "memory");
    // visiting order of this pair's tiles (whole-tile launches that raise flags)
    const bool reorder = !kSliced && flags_out != nullptr && unit_end - unit_begin <= kMaxOrder;
    auto tile_of = [&](int unit) {
        return reorder ? unit_begin + middle_out(unit - unit_begin, unit_end - unit_begin) : unit / nsplit;
    };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0, wb = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            const uint32_t btx = static_cast<uint32_t>(half_n) * 128u;
            for (int unit = unit_begin; unit < unit_end && ok; ++unit) {
                const int pair = tile_of(unit), slice = kSliced ? unit - pair * nsplit : 0;
                const int m0 = pair * kPairM + static_cast<int>(rank) * kTileM;
                const int wrow0 = slice * n_slice + static_cast<int>(rank) * half_n;
                if (tile_flags) {
                    // the window of this tile reaches into the tiles on either side
                    for (int t = pair - 1; t <= pair + 1 && ok; ++t) {
                        if (t >= 0 && t < npairs) ok = flag_wait(flags_in + t, flag_target, abort_flag, err);
                    }
                    if (!ok) break;
                    // what those tiles' epilogues stored is read below by TMA (async proxy)
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
                for (int c = 0; c < kchunks && ok; ++c) {
                    ok = mbar_wait(wempty_bar(wb), wphase ^ 1u, abort_flag, err, kErrD2Producer);
                    if (!ok) break;
                    const uint32_t wf = map_to_cta(wfull_bar(wb), 0);
                    mbar_expect_tx_cluster(wf, kWinBytes);
                    const bool low8 = kPlanes == 3 && c >= fchunks;     // e5m2 chunk: byte coordinates
                    const int wcol = low8 ? (c - fchunks) * 128 : c * kChunkK;
                    tma_load_2d_pair(win_base + wb * kWinBytes, low8 ? &tmXl : &tmX,
                                     low8 ? wcol : (c < achunks ? c : c - achunks) * kChunkK,
                                     m0 - kWinPad, wf);
                    if (++wb == nwin) { wb = 0; wphase ^= 1u; }
                    for (int tap = 0; tap < 9; tap += taps_per_stage) {
                        const int g = 9 - tap < taps_per_stage ? 9 - tap : taps_per_stage;
                        ok = mbar_wait(bempty_bar(stage), phase ^ 1u, abort_flag, err, kErrD2Producer);
                        if (!ok) break;
                        const uint32_t bf = map_to_cta(bfull_bar(stage), 0);
                        mbar_expect_tx_cluster(bf, btx * static_cast<uint32_t>(g));
                        for (int j = 0; j < g; ++j) {
                            tma_load_2d_pair(b_base + stage * kB2StageBytes + j * btx, low8 ? &tmWl : &tmW,
                                             wcol, (tap + j) * Kp + wrow0, bf);
                        }
                        if (++stage == nstages) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            const uint32_t idesc = (1u << 4) | (OperandFormat<T>::value << 7) |
                                   (OperandFormat<T>::value << 10) |
                                   (static_cast<uint32_t>(n_slice >> 3) << 17) |
                                   (static_cast<uint32_t>(kPairM >> 4) << 24);
            // e5m2 x e5m2 -> fp32 for the chunks of an e5m2 activation plane
            const uint32_t idesc8 = (1u << 4) | (1u << 7) | (1u << 10) |
                                    (static_cast<uint32_t>(n_slice >> 3) << 17) |
                                    (static_cast<uint32_t>(kPairM >> 4) << 24);
            int stage = 0, wb = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            int local = 0;
            if constexpr (!kSliced) {
                // Whole tiles, one tap per stage.  This lane's instruction stream is what
                // paces the tensor pipe (a 256 x 256 x 16 MMA lasts ~128 cycles, so a stage
                // leaves ~500 cycles for everything between two waits): descriptors are a
                // constant plus an address in 16-byte units, the nine row offsets of the
                // window are immediates, and the two operand formats have a loop each.
                const uint64_t dbase = umma_desc_sw128(0);
                const uint32_t win16 = (win_base & 0x3FFFFu) >> 4, b16 = (b_base & 0x3FFFFu) >> 4;
                for (int unit = unit_begin; unit < unit_end && ok; ++unit, ++local) {
                    const int acc = local & 1;
                    const uint32_t accphase = (local >> 1) & 1u;
                    ok = mbar_wait(tempty_bar(acc), accphase ^ 1u, abort_flag, err, kErrD2MmaAcc);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kMaxN);
                    uint32_t accum = 0u;
                    for (int c = 0; c < kchunks && ok; ++c) {
                        ok = mbar_wait(wfull_bar(wb), wphase, abort_flag, err, kErrD2MmaFull);
                        if (!ok) break;
                        const uint64_t a_win = dbase + (win16 + static_cast<uint32_t>(wb) * (kWinBytes >> 4));
                        const bool f8 = kPlanes == 3 && c >= fchunks;
#pragma unroll
                        for (int tap = 0; tap < 9; ++tap) {
                            ok = mbar_wait(bfull_bar(stage), phase, abort_flag, err, kErrD2MmaFull);
                            if (!ok) break;
                            // rows (24 + 20 dy + dx) .. of the window, 8 sixteen-byte units each
                            const uint64_t a_desc =
                                a_win + static_cast<uint32_t>((kWinPad + (tap / 3 - 1) * kCellsPerRow + (tap % 3 - 1)) * 8);
                            const uint64_t b_desc = dbase + (b16 + static_cast<uint32_t>(stage) * (kB2StageBytes >> 4));
                            if (f8) {
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    tcgen05_mma_f8_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc8, 1u);
                                }
                            } else {
                                tcgen05_mma_f16_pair(d_tmem, a_desc, b_desc, idesc, accum);
                                accum = 1u;
#pragma unroll
                                for (int k = 1; k < kChunkK / 16; ++k) {
                                    tcgen05_mma_f16_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, 1u);
                                }
                            }
                            tcgen05_commit_pair(bempty_bar(stage));
                            if (++stage == nstages) { stage = 0; phase ^= 1u; }
                        }
                        if (!ok) break;
                        tcgen05_commit_pair(wempty_bar(wb));
                        if (++wb == nwin) { wb = 0; wphase ^= 1u; }
                    }
                    if (!ok) break;
                    tcgen05_commit_pair(tfull_bar(acc));
                }
            } else {
                for (int unit = unit_begin; unit < unit_end && ok; ++unit, ++local) {
                    const int acc = local & 1;
                    const uint32_t accphase = (local >> 1) & 1u;
                    ok = mbar_wait(tempty_bar(acc), accphase ^ 1u, abort_flag, err, kErrD2MmaAcc);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kMaxN);
                    for (int c = 0; c < kchunks && ok; ++c) {
                        ok = mbar_wait(wfull_bar(wb), wphase, abort_flag, err, kErrD2MmaFull);
                        if (!ok) break;
                        const uint32_t win = win_base + wb * kWinBytes;
                        const uint32_t btx = static_cast<uint32_t>(half_n) * 128u;
                        for (int tap0 = 0; tap0 < 9; tap0 += taps_per_stage) {
                            const int g = 9 - tap0 < taps_per_stage ? 9 - tap0 : taps_per_stage;
                            ok = mbar_wait(bfull_bar(stage), phase, abort_flag, err, kErrD2MmaFull);
                            if (!ok) break;
                            tcgen05_fence_after();
                            for (int j = 0; j < g; ++j) {
                                const int tap = tap0 + j;
                                const int row0 = kWinPad + (tap / 3 - 1) * kCellsPerRow + (tap % 3 - 1);
                                const uint64_t a_desc =
                                    umma_desc_sw128(win + static_cast<uint32_t>(row0) * 128u);
                                const uint64_t b_desc =
                                    umma_desc_sw128(b_base + stage * kB2StageBytes + j * btx);
                                if (kPlanes == 3 && c >= fchunks) {
#pragma unroll
                                    for (int k = 0; k < 4; ++k) {
                                        tcgen05_mma_f8_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc8, 1u);
                                    }
                                } else {
#pragma unroll
                                    for (int k = 0; k < kChunkK / 16; ++k) {
                                        tcgen05_mma_f16_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                                                             (c > 0 || tap > 0 || k > 0) ? 1u : 0u);
                                    }
                                }
                            }
                            tcgen05_commit_pair(bempty_bar(stage));
                            if (++stage == nstages) { stage = 0; phase ^= 1u; }
                        }
                        if (!ok) break;
                        tcgen05_commit_pair(wempty_bar(wb));
                        if (++wb == nwin) { wb = 0; wphase ^= 1u; }
                    }
                    if (!ok) break;
                    tcgen05_commit_pair(tfull_bar(acc));
                }
            }
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..9, both CTAs)
        const int qd = warp & 3;
        const int ncols = n_slice >> 1;          // channels this warp converts per unit
        const int wcol = ((warp - 2) >> 2) * ncols;
        unsigned char* stg_ptr = stage_out + (warp - 2) * kStageOutBytes;
        const uint32_t stg = smem_u32(stg_ptr);
        unsigned char* stg_row = stg_ptr + lane * 64;
        int local = 0;
        for (int unit = unit_begin; unit < unit_end; ++unit, ++local) {
            const int pair = tile_of(unit), slice = kSliced ? unit - pair * nsplit : 0;
            const int col0 = slice * n_slice + wcol;   // first output channel of this warp
            const int acc = local & 1;
            const uint32_t accphase = (local >> 1) & 1u;
            const int row0 = pair * kPairM + static_cast<int>(rank) * kTileM + qd * 32;
            const int q = row0 + lane;
            const bool interior = cell_is_interior(q, Q);
            // one lane polls, the others sleep at the warp barrier
            bool ok = true;
            if (lane == 0) ok = mbar_wait(tfull_bar(acc), accphase, abort_flag, err, kErrD2Epilogue);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tcgen05_fence_after();
            const bool use_res = (res != nullptr) && interior;
            constexpr bool two = kPlanes == 2;
            constexpr bool e5 = kPlanes == 3;
            const T* rrow = res + static_cast<size_t>(q) * ldr + col0;
            // e5m2 plane of the same row: Kp bytes after the Kp 16-bit channels
            const unsigned char* erow =
                reinterpret_cast<const unsigned char*>(res + static_cast<size_t>(q) * ldr + Kp) + col0;
            // accumulator columns are numbered within the slice
            const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(qd * 32) << 16) +
                                    static_cast<uint32_t>(acc * kMaxN + wcol);
            uint32_t ra[32], rb[32];
            uint4 va[4], vb[4], la[4], lb[4], ea[2], eb[2];
            // batch-norm etc. of one 32-channel chunk and its store(s)
            auto emit = [&](const uint32_t (&r)[32], const uint4 (&v)[4], const uint4 (&l)[4],
                            const uint4 (&e)[2], int col) {
                wait_staged_tile_read(lane);
                if constexpr (e5) {
                    uint32_t lo[8], h8[8];
                    epilogue_chunk_e5m2<T>(r, v, e, s_scale + col, s_bias + col, use_res, interior, stg_row,
                                           lane, lo, h8, out_hi8 != nullptr);
                    store_staged_tile(&tmO, stg, col, row0, lane);
                    if (q < q_rows) {
                        const size_t off = static_cast<size_t>(q) * out_pitch + col;
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
                } else if constexpr (!two) {
                    epilogue_chunk<T>(r, v, s_scale + col, s_bias + col, use_res, interior, stg_row, lane);
                    store_staged_tile(&tmO, stg, col, row0, lane);
                } else {
                    uint32_t lo[16];
                    epilogue_chunk_x2<T>(r, v, l, s_scale + col, s_bias + col, use_res, interior, stg_row,
                                         lane, lo);
                    store_staged_tile(&tmO, stg, col, row0, lane);
                    wait_staged_tile_read(lane);
                    stage_low_plane(lo, stg_row, lane);
                    store_staged_tile(&tmO, stg, Kp + col, row0, lane);
                }
            };
            load_residual(va, rrow, use_res);
            if constexpr (two) load_residual(la, rrow + Kp, use_res);
            if constexpr (e5) load_residual8(ea, erow, use_res);
            LZB_TMEM_LD32(ra, taddr0);
            for (int j = 0; j < ncols; j += 64) {
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const bool more = j + 32 < ncols;
                if (more) {
                    load_residual(vb, rrow + j + 32, use_res);
                    if constexpr (two) load_residual(lb, rrow + Kp + j + 32, use_res);
                    if constexpr (e5) load_residual8(eb, erow + j + 32, use_res);
                    LZB_TMEM_LD32(rb, taddr0 + j + 32);
                }
                emit(ra, va, la, ea, col0 + j);
                if (more) {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (j + 64 < ncols) {
                        load_residual(va, rrow + j + 64, use_res);
                        if constexpr (two) load_residual(la, rrow + Kp + j + 64, use_res);
                        if constexpr (e5) load_residual8(ea, erow + j + 64, use_res);
                        LZB_TMEM_LD32(ra, taddr0 + j + 64);
                    }
                    emit(rb, vb, lb, eb, col0 + j + 32);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
            if (!kSliced && flags_out != nullptr) {
                // this warp's part of the tile is in memory: its TMA stores have
                // completed, its lanes' direct stores are fenced; then count it
                if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    asm volatile("fence.proxy.async;" ::: "memory");
                    // the read-modify-write chain carries every earlier arrival's writes
                    const uint32_t before = atom_acq_rel_gpu_add(counts_out + pair, 1u);
                    if ((before & (kFlagArrivals - 1u)) == kFlagArrivals - 1u) {
                        st_release_gpu(flags_out + pair, flag_target);
                    }
                }
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();      // neither CTA may retire while its peer can still touch it
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(kTmemCols)
                     : "memory");
    }
}

}  // namespace dc2
}  // namespace lzb
