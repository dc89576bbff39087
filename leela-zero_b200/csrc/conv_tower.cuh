// The whole residual tower of a large batch in ONE launch.
//
// conv_direct2.cuh runs a layer per launch; what a launch pays once (turnover
// of the CTAs on the SMs, barrier and tensor-memory set-up, the first operands'
// round trip, the last tile's epilogue, which nothing overlaps) is about 6 us
// of an 87 us layer.  Here the CTA pairs stay: every pair owns the same range
// of 256-cell tiles in every layer and walks the layers in one loop, its TMA
// ring, its two accumulators and its epilogue pipeline running on across layer
// boundaries.  Layers depend on each other tile by tile through the flags of
// conv_direct2.cuh (a tile of layer l+1 reads tiles i-1, i, i+1 of layer l);
// since the tiles that are waited for belong to other pairs of the SAME launch,
// all pairs must be resident at once: the kernel is launched cooperatively,
// and the host falls back to the launch-per-layer path where that is refused.
//
// Per layer the kernel reads a TowerLayer record from global memory: the weight
// tensor maps (used in place by the TMA unit), batch-norm vectors, which of the
// two activation buffers it reads and writes, chunk counts and plane switches.
// Everything else (window addressing, descriptors, epilogue arithmetic, bounded
// waits) is that of conv_direct2_kernel's whole-tile path.
#pragma once
#include "conv_direct2.cuh"

namespace lzb {
namespace dct {

using namespace tc;
using namespace dc;
using namespace dc2;

struct alignas(64) TowerLayer {
    CUtensorMap tmW;            // weights [9*Kp][Cin'], box 64 x Kp/2
    CUtensorMap tmWl;           // e5m2 weights (byte map), box 128 x Kp/2; any valid map if unused
    const float* mean;          // batch norm, Kp entries each
    const float* invstd;
    int in_sel;                 // 0: network input cells, 1: X, 2: H
    int out_sel;                // 1: X, 2: H
    int kchunks;                // chunks of the reduction in total (fp16 ones first, then e5m2 ones)
    int fchunks;                // fp16 chunks among them
    int achunks;                // 64-channel chunks the activation tensor has
    int has_res;                // add X (the block's input) before the ReLU
    int res_lo;                 // the residual carries an e5m2 plane to add as well
    int out_lo;                 // write the e5m2 plane of the result
    int out_hi8;                // write the scaled high plane in e5m2 as well
    int pad;
};

constexpr int kErrTowerProducer = 501;
constexpr int kErrTowerMmaAcc = 502;
constexpr int kErrTowerMmaFull = 503;
constexpr int kErrTowerEpilogue = 504;
constexpr uint32_t kTowerSmemBytes = kD2SmemBytes + 2 * kMaxN * 4;   // a second set of batch-norm constants

// tmIN, tmX, tmH : activation windows (box 64 x kWinRows); tmXl, tmHl : their
// e5m2 planes (byte maps, box 128 x kWinRows); tmXo, tmHo : output tiles (box
// 32 x 32, 64-byte swizzle).  X, H : the two activation tensors (residual reads,
// byte-plane stores), ldr elements of T / out_pitch bytes per cell row, q_rows
// rows.  flags, counts : [n_layers][tile_cap] words each (conv_direct2.cuh),
// run : the number of this tower run.
template <typename T, int kPlanes>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kDcThreads, 1) conv_tower_kernel(
    const __grid_constant__ CUtensorMap tmIN, const __grid_constant__ CUtensorMap tmX,
    const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmXl,
    const __grid_constant__ CUtensorMap tmHl, const __grid_constant__ CUtensorMap tmXo,
    const __grid_constant__ CUtensorMap tmHo, const TowerLayer* __restrict__ layers, int n_layers,
    T* X, T* H, int Q, int Kp, int npairs, int ldr, int out_pitch, int q_rows, uint32_t* flags,
    uint32_t* counts, int tile_cap, uint32_t run, int* err) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (base - raw);
    constexpr int nwin = kWinBufs;
    constexpr int nstages = kB2Stages;
    const uint32_t win_base = base;
    const uint32_t b_base = base + static_cast<uint32_t>(nwin) * kWinBytes;
    unsigned char* stage_out = smem + kOperand2Bytes;
    // batch-norm constants of two layers: the epilogue may still be in layer l
    // while nothing else is, and each warp refills the half it reads itself
    float* s_const = reinterpret_cast<float*>(stage_out + 8 * kStageOutBytes);   // [2][scale | bias][kMaxN]
    unsigned char* bar_mem = stage_out + 8 * kStageOutBytes + 4 * kMaxN * 4;
    const uint32_t bars = smem_u32(bar_mem);
    auto bfull_bar = [&](int s) { return bars + 8u * (0 + s); };      // leader's are used
    auto bempty_bar = [&](int s) { return bars + 8u * (16 + s); };    // both CTAs
    auto wfull_bar = [&](int w) { return bars + 8u * (32 + w); };     // leader's
    auto wempty_bar = [&](int w) { return bars + 8u * (36 + w); };    // both
    auto tfull_bar = [&](int a) { return bars + 8u * (40 + a); };     // both
    auto tempty_bar = [&](int a) { return bars + 8u * (42 + a); };    // leader's
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * 44);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * 44 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kB2Stages; i++) {
            mbar_init(bfull_bar(i), 2);      // one arrive.expect_tx per CTA of the pair
            mbar_init(bempty_bar(i), 1);
        }
        for (int i = 0; i < nwin; i++) {
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
    const int nclusters = gridDim.x >> 1, cid = blockIdx.x >> 1;
    const int tile_begin = static_cast<int>(static_cast<long long>(cid) * npairs / nclusters);
    const int tile_end = static_cast<int>(static_cast<long long>(cid + 1) * npairs / nclusters);
    const int ntiles = tile_end - tile_begin;
    const bool reorder = ntiles <= kMaxOrder;
    auto tile_of = [&](int k) { return tile_begin + (reorder ? middle_out(k, ntiles) : k); };
    const int half_n = Kp >> 1;               // weight rows each CTA stages per tap

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0, wb = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            const uint32_t btx = static_cast<uint32_t>(half_n) * 128u;
            for (int li = 0; li < n_layers && ok; ++li) {
                const TowerLayer* tl = layers + li;
                const int kchunks = tl->kchunks, fchunks = tl->fchunks, achunks = tl->achunks;
                const CUtensorMap* in_map = tl->in_sel == 0 ? &tmIN : (tl->in_sel == 1 ? &tmX : &tmH);
                const CUtensorMap* in_lo = tl->in_sel == 2 ? &tmHl : &tmXl;
                const uint32_t* flags_in = li > 0 ? flags + static_cast<size_t>(li - 1) * tile_cap : nullptr;
                for (int k = 0; k < ntiles && ok; ++k) {
                    const int pair = tile_of(k);
                    const int m0 = pair * kPairM + static_cast<int>(rank) * kTileM;
                    const int wrow0 = static_cast<int>(rank) * half_n;
                    if (flags_in != nullptr) {
                        // the window of this tile reaches into the tiles on either side
                        for (int t = pair - 1; t <= pair + 1 && ok; ++t) {
                            if (t >= 0 && t < npairs) ok = flag_wait(flags_in + t, run, abort_flag, err);
                        }
                        if (!ok) break;
                        // what those tiles' epilogues stored is read below by TMA (async proxy)
                        asm volatile("fence.proxy.async;" ::: "memory");
                    }
                    for (int c = 0; c < kchunks && ok; ++c) {
                        ok = mbar_wait(wempty_bar(wb), wphase ^ 1u, abort_flag, err, kErrTowerProducer);
                        if (!ok) break;
                        const uint32_t wf = map_to_cta(wfull_bar(wb), 0);
                        mbar_expect_tx_cluster(wf, kWinBytes);
                        const bool low8 = kPlanes == 3 && c >= fchunks;     // e5m2 chunk: byte coordinates
                        const int wcol = low8 ? (c - fchunks) * 128 : c * kChunkK;
                        tma_load_2d_pair(win_base + wb * kWinBytes, low8 ? in_lo : in_map,
                                         low8 ? wcol : (c < achunks ? c : c - achunks) * kChunkK,
                                         m0 - kWinPad, wf);
                        if (++wb == nwin) { wb = 0; wphase ^= 1u; }
                        for (int tap = 0; tap < 9; ++tap) {
                            ok = mbar_wait(bempty_bar(stage), phase ^ 1u, abort_flag, err, kErrTowerProducer);
                            if (!ok) break;
                            const uint32_t bf = map_to_cta(bfull_bar(stage), 0);
                            mbar_expect_tx_cluster(bf, btx);
                            tma_load_2d_pair(b_base + stage * kB2StageBytes, low8 ? &tl->tmWl : &tl->tmW, wcol,
                                             tap * Kp + wrow0, bf);
                            if (++stage == nstages) { stage = 0; phase ^= 1u; }
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            const uint32_t idesc = (1u << 4) | (OperandFormat<T>::value << 7) |
                                   (OperandFormat<T>::value << 10) |
                                   (static_cast<uint32_t>(Kp >> 3) << 17) |
                                   (static_cast<uint32_t>(kPairM >> 4) << 24);
            // e5m2 x e5m2 -> fp32 for the chunks of an e5m2 activation plane
            const uint32_t idesc8 = (1u << 4) | (1u << 7) | (1u << 10) |
                                    (static_cast<uint32_t>(Kp >> 3) << 17) |
                                    (static_cast<uint32_t>(kPairM >> 4) << 24);
            int stage = 0, wb = 0;
            uint32_t phase = 0, wphase = 0;
            bool ok = true;
            int local = 0;
            const uint64_t dbase = umma_desc_sw128(0);
            const uint32_t win16 = (win_base & 0x3FFFFu) >> 4, b16 = (b_base & 0x3FFFFu) >> 4;
            for (int li = 0; li < n_layers && ok; ++li) {
                const int kchunks = layers[li].kchunks, fchunks = layers[li].fchunks;
                for (int k = 0; k < ntiles && ok; ++k, ++local) {
                    const int acc = local & 1;
                    const uint32_t accphase = (local >> 1) & 1u;
                    ok = mbar_wait(tempty_bar(acc), accphase ^ 1u, abort_flag, err, kErrTowerMmaAcc);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kMaxN);
                    uint32_t accum = 0u;
                    for (int c = 0; c < kchunks && ok; ++c) {
                        ok = mbar_wait(wfull_bar(wb), wphase, abort_flag, err, kErrTowerMmaFull);
                        if (!ok) break;
                        const uint64_t a_win = dbase + (win16 + static_cast<uint32_t>(wb) * (kWinBytes >> 4));
                        const bool f8 = kPlanes == 3 && c >= fchunks;
#pragma unroll
                        for (int tap = 0; tap < 9; ++tap) {
                            ok = mbar_wait(bfull_bar(stage), phase, abort_flag, err, kErrTowerMmaFull);
                            if (!ok) break;
                            // rows (24 + 20 dy + dx) .. of the window, 8 sixteen-byte units each
                            const uint64_t a_desc =
                                a_win + static_cast<uint32_t>((kWinPad + (tap / 3 - 1) * kCellsPerRow + (tap % 3 - 1)) * 8);
                            const uint64_t b_desc = dbase + (b16 + static_cast<uint32_t>(stage) * (kB2StageBytes >> 4));
                            if (f8) {
#pragma unroll
                                for (int kk = 0; kk < 4; ++kk) {
                                    tcgen05_mma_f8_pair(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc8, 1u);
                                }
                            } else {
                                tcgen05_mma_f16_pair(d_tmem, a_desc, b_desc, idesc, accum);
                                accum = 1u;
#pragma unroll
                                for (int kk = 1; kk < kChunkK / 16; ++kk) {
                                    tcgen05_mma_f16_pair(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, 1u);
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
        const int ncols = Kp >> 1;               // channels this warp converts per tile
        const int wcol = ((warp - 2) >> 2) * ncols;
        unsigned char* stg_ptr = stage_out + (warp - 2) * kStageOutBytes;
        const uint32_t stg = smem_u32(stg_ptr);
        unsigned char* stg_row = stg_ptr + lane * 64;
        int local = 0;
        bool alive = true;
        for (int li = 0; li < n_layers && alive; ++li) {
            const TowerLayer* tl = layers + li;
            // this warp's half of the layer's batch-norm constants (four warps write
            // the same values into the same half; each reads back what it wrote)
            float* s_scale = s_const + (li & 1) * 2 * kMaxN;
            float* s_bias = s_scale + kMaxN;
            for (int i = wcol + lane; i < wcol + ncols; i += 32) {
                const float is = tl->invstd[i];
                s_scale[i] = is;
                s_bias[i] = -tl->mean[i] * is;
            }
            __syncwarp();
            const CUtensorMap* out_map = tl->out_sel == 1 ? &tmXo : &tmHo;
            T* out_base = tl->out_sel == 1 ? X : H;
            const T* res = tl->has_res ? X : nullptr;
            const bool res_lo = tl->res_lo != 0;
            unsigned char* out_lo =
                tl->out_lo ? reinterpret_cast<unsigned char*>(out_base) + static_cast<size_t>(Kp) * sizeof(T) : nullptr;
            unsigned char* out_hi8 = tl->out_hi8 ? reinterpret_cast<unsigned char*>(out_base) +
                                                       static_cast<size_t>(Kp) * (sizeof(T) + 1)
                                                 : nullptr;
            uint32_t* flags_out = flags + static_cast<size_t>(li) * tile_cap;
            uint32_t* counts_out = counts + static_cast<size_t>(li) * tile_cap;
            for (int k = 0; k < ntiles; ++k, ++local) {
                const int pair = tile_of(k);
                const int col0 = wcol;                      // first output channel of this warp
                const int acc = local & 1;
                const uint32_t accphase = (local >> 1) & 1u;
                const int row0 = pair * kPairM + static_cast<int>(rank) * kTileM + qd * 32;
                const int q = row0 + lane;
                const bool interior = cell_is_interior(q, Q);
                // one lane polls, the others sleep at the warp barrier
                bool ok = true;
                if (lane == 0) ok = mbar_wait(tfull_bar(acc), accphase, abort_flag, err, kErrTowerEpilogue);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
                tcgen05_fence_after();
                const bool use_res = (res != nullptr) && interior;
                constexpr bool e5 = kPlanes == 3;
                const T* rrow = res + static_cast<size_t>(q) * ldr + col0;
                // e5m2 plane of the same row: Kp bytes after the Kp 16-bit channels
                const unsigned char* erow =
                    reinterpret_cast<const unsigned char*>(res + static_cast<size_t>(q) * ldr + Kp) + col0;
                const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(qd * 32) << 16) +
                                        static_cast<uint32_t>(acc * kMaxN + wcol);
                uint32_t ra[32], rb[32];
                uint4 va[4], vb[4], ea[2], eb[2];
                auto emit = [&](const uint32_t (&r)[32], const uint4 (&v)[4], const uint4 (&e)[2], int col) {
                    wait_staged_tile_read(lane);
                    if constexpr (e5) {
                        uint32_t lo[8], h8[8];
                        epilogue_chunk_e5m2<T>(r, v, e, s_scale + col, s_bias + col, use_res, interior, stg_row,
                                               lane, lo, h8, out_hi8 != nullptr);
                        store_staged_tile(out_map, stg, col, row0, lane);
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
                    } else {
                        epilogue_chunk<T>(r, v, s_scale + col, s_bias + col, use_res, interior, stg_row, lane);
                        store_staged_tile(out_map, stg, col, row0, lane);
                    }
                };
                load_residual(va, rrow, use_res);
                if constexpr (e5) load_residual8(ea, erow, use_res && res_lo);
                LZB_TMEM_LD32(ra, taddr0);
                for (int j = 0; j < ncols; j += 64) {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const bool more = j + 32 < ncols;
                    if (more) {
                        load_residual(vb, rrow + j + 32, use_res);
                        if constexpr (e5) load_residual8(eb, erow + j + 32, use_res && res_lo);
                        LZB_TMEM_LD32(rb, taddr0 + j + 32);
                    }
                    emit(ra, va, ea, col0 + j);
                    if (more) {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (j + 64 < ncols) {
                            load_residual(va, rrow + j + 64, use_res);
                            if constexpr (e5) load_residual8(ea, erow + j + 64, use_res && res_lo);
                            LZB_TMEM_LD32(ra, taddr0 + j + 64);
                        }
                        emit(rb, vb, eb, col0 + j + 32);
                    }
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
                // this warp's part of the tile is in memory: its TMA stores have
                // completed, its lanes' direct stores are fenced; then count it
                if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    asm volatile("fence.proxy.async;" ::: "memory");
                    const uint32_t before = atom_acq_rel_gpu_add(counts_out + pair, 1u);
                    if ((before & (kFlagArrivals - 1u)) == kFlagArrivals - 1u) st_release_gpu(flags_out + pair, run);
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

}  // namespace dct
}  // namespace lzb
