// C-ABI implementation of the B200 forward pipe (see include/lzb200.h).
//
// A pipe holds the network on one GPU: per 3x3 layer the Winograd-transformed
// filters U[36][Kp][Cin_p] in the tower's storage type plus fp32 batch-norm
// vectors, and the two 1x1 head filters.  A context holds a stream and the
// activation buffers (V, M, X) sized for one micro-batch; a batch is pushed
// through the whole tower one micro-batch at a time so that V and M, the two
// large tensors every layer writes and reads once, stay resident in L2.
//
// Per 3x3 layer two kernels run: the channel contractions (tcgen05 or FFMA)
// and the fused output-transform / batch-norm / residual / ReLU / next input
// transform.  The sequence mirrors OpenCL_Network::forward
// (src/OpenCL.cpp:143-329) and CPUPipe::forward (src/CPUPipe.cpp:379-428).
#include "../../include/lzb200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>
#include <vector>

#include "conv_direct.cuh"
#include "conv_direct2.cuh"
#include "conv_direct3.cuh"
#include "conv_tower.cuh"
#include "gemm_simt.cuh"
#include "gemm_tcgen05.cuh"
#include "head_kernels.cuh"
#include "transform_kernels.cuh"

namespace {

thread_local std::string g_error;

int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}

#define LZB_CUDA(expr)                                                                     \
    do {                                                                                   \
        cudaError_t e_ = (expr);                                                           \
        if (e_ != cudaSuccess) {                                                           \
            (void)cudaGetLastError(); /* reported here: do not leave it for a later check */ \
            return fail(LZB_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_)); \
        }                                                                                  \
    } while (0)

// Select the device and drop any error an earlier call (of this library or of
// another one in the process) left behind, so that the cudaGetLastError() after
// a kernel launch reports that launch and nothing older.
inline cudaError_t enter_device(int device) {
    const cudaError_t e = cudaSetDevice(device);
    (void)cudaGetLastError();
    return e;
}

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

constexpr int kXformSmem = lzb::kBoardCells * 32 * 8;   // fp32 board of one position x 64 channels
constexpr int kMaxMicroBatch = 256;      // rows of V/M allocated: 25 * 256 = 6400
constexpr int kDefaultMicroBatch = 64;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library loads
// (and its symbols can be listed) on a machine without a CUDA driver.
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

// 2-D map over a row-major [rows][cols] matrix of 16-bit elements.  Operand
// maps use boxes of 64 columns (128 bytes) x box_rows under the 128-byte swizzle
// the UMMA descriptors expect; the output maps of the convolution kernel use
// 32 x 32 boxes under the 64-byte swizzle.
// precision < 0: a byte tensor (e5m2 planes).  pitch_bytes 0: rows are dense.
int make_map_2d(CUtensorMap* map, int precision, void* base, uint64_t rows, uint64_t cols,
                uint32_t box_rows, uint32_t box_cols = 64,
                CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, uint64_t pitch_bytes = 0) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(LZB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const uint64_t elt = precision < 0 ? 1 : 2;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch_bytes ? pitch_bytes : cols * elt};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt =
        precision < 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                      : (precision == LZB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    CUresult r = fn(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(LZB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    }
    return LZB_OK;
}

struct Layer {
    void* U = nullptr;          // [36][Kp][cin_p] storage type
    float* mean = nullptr;      // [Kp]
    float* invstd = nullptr;    // [Kp]
    int cin_p = 0;
    bool present = false;
    CUtensorMap tmU;
    void* Wd = nullptr;         // direct path: [9][Kp][cinw] storage type
    int cinw = 0;               // input-channel extent of Wd: cin_p x weight planes
    int achunks = 0;            // 64-channel chunks of the activation tensor this layer reads
    unsigned char* Wd8 = nullptr;   // e5m2 copy of the weights [9][Kp][cin8] (LZB_FP16_X2), or null
    int lchunks = 0;            // 128-channel e5m2 chunks that follow the fp16 chunks
    bool out_lo = false;        // this layer writes an e5m2 low plane beside its fp16 output
    bool out_hi8 = false;       // ... and an e5m2 copy of the fp16 plane (the next layer corrects its weights)
    CUtensorMap tmW8[5];        // byte maps over Wd8, box 128 x Kp/(2*ns)
    CUtensorMap tmW;            // box 64 x Kp   (one CTA per tile)
    CUtensorMap tmW2[5];        // CTA pairs: [ns] has box 64 x Kp/(2*ns), ns = 1..4 where valid
    bool split_ok[5] = {false, false, false, false, false};
};

struct Heads {
    bool present = false;
    float *bn_pol_mean = nullptr, *bn_pol_invstd = nullptr, *ip_pol_wT = nullptr,
          *ip_pol_b = nullptr, *bn_val_mean = nullptr, *bn_val_invstd = nullptr,
          *ip1_val_wT = nullptr, *ip1_val_b = nullptr, *ip2_val_w = nullptr, *ip2_val_b = nullptr;
};

}  // namespace

struct lzb_pipe {
    int device = 0;
    int channels = 0;   // C
    int Cp = 0;         // C rounded up to 64
    int blocks = 0;
    int precision = LZB_FP16;   // storage type: LZB_FP32, LZB_FP16 or LZB_BF16
    bool direct = false;        // true: implicit-GEMM convolution; false: Winograd pipeline
    bool pairs = false;         // direct path on CTA pairs (tcgen05 cta_group::2)
    int aplanes = 1;            // activations carried as hi + lo: 2 = two 16-bit planes (LZB_FP16_X3),
                                // 3 = a 16-bit plane and an e5m2 plane (LZB_FP16_X2)
    // bytes of one cell row of the activation tensors
    int row_bytes() const { return aplanes == 3 ? (wlo_layers > 1 ? 4 : 3) * Cp : aplanes * Cp * elt; }
    // LZB_FP16_X2: layers 0 .. lo_layers-1 write the e5m2 plane and layers
    // 1 .. lo_layers-1 read it; the layers after them run on the fp16 plane alone
    // (same buffers, the low bytes of a row are then neither written nor read).
    int lo_layers = 0;
    // Layers 0 .. wlo_layers-1 (a prefix of those) also correct the rounding of
    // their weights: they read a third plane, e5m2(fp16(x) / 256), against
    // e5m2(256 (w - fp16(w))); a cell row is then [Cp x fp16 | Cp lo | Cp hi8].
    // The input convolution does the same with a second fp16 weight plane.
    int wlo_layers = 0;
    bool wsplit = false;        // weights carried as hi + lo planes as well (LZB_FP16_X3)
    int elt = 2;        // bytes per stored element
    int sm_count = 0;
    // Reduction-split kernel (conv_direct3.cuh): most tiles one launch may have
    // (clusters of 2 * chunks CTAs that can be resident at once), per chunk
    // count 2..4; 0 = not used.
    int ksplit_max_tiles[5] = {0, 0, 0, 0, 0};
    std::vector<Layer> layers;
    // per-layer records of the one-launch tower kernel (conv_tower.cuh), on the
    // device; null where that kernel does not apply
    lzb::dct::TowerLayer* tower_table = nullptr;
    bool tower_refused = false;         // a cooperative launch of it failed once: not tried again
    // contexts on this pipe (their streams are asked whether they are busy)
    std::mutex ctx_mutex;
    std::vector<lzb_ctx*> contexts;
    float* head_w = nullptr;   // [3][Cp] fp32
    bool head_convs = false;
    bool finalized = false;
    Heads heads;
};

struct lzb_ctx {
    lzb_pipe* pipe = nullptr;
    int max_batch = 0;
    int micro_cap = 0;     // positions V/M/X can hold
    int micro = 0;         // positions per pass through the tower
    int Pa = 0;            // rows of V and M (multiple of 128)
    cudaStream_t stream = nullptr;
    void *V = nullptr, *M = nullptr, *X = nullptr;
    float *d_in = nullptr, *d_pol = nullptr, *d_val = nullptr;
    float *d_policy = nullptr, *d_winrate = nullptr;
    unsigned int* d_packed = nullptr;   // bit-packed input planes [max_batch][18][12]
    // per-tile completion words of the direct path, [2][layers][tile_cap] (the run
    // that completed a tile last, then the arrival counters), and the number of
    // tower runs so far (see conv_direct2.cuh); null: not used
    uint32_t* tile_flags = nullptr;
    int tile_cap = 0;
    uint32_t tower_runs = 0;
    bool tile_flags_always = false;     // asked for by LZB_TILE_FLAGS=1: also while other contexts are busy
    bool tower_kernel = false;          // LZB_TOWER_KERNEL=1: all layers of a large batch in one launch
    std::atomic<long long> last_tower_ns{0};   // when this context last enqueued a tower (steady clock)
    int* d_err = nullptr;
    int* h_err = nullptr;  // pinned
    CUtensorMap tmV_first, tmV;
    // direct path: padded cell-major activations
    int Qa = 0;            // rows allocated in IN / X / H
    void *IN = nullptr, *H = nullptr;
    CUtensorMap tmIN, tmX, tmH;      // window loads
    CUtensorMap tmXo, tmHo;          // 32 x 32 output stores
    CUtensorMap tmXl, tmHl;          // e5m2 planes of X and H: 128-byte windows (LZB_FP16_X2)
    long long launches = 0;
    // per-launch timing (diagnostics): event pairs tagged with a kernel class
    bool profiling = false;
    std::vector<cudaEvent_t> prof_events;   // 2 per launch
    std::vector<int> prof_class;
    std::vector<int> prof_layers;           // layers a launch covers (1, or the whole tower)
};

namespace {

using namespace lzb;

template <typename T>
int upload_layer_t(lzb_pipe* p, Layer& L, const float* U32_dev, int c_in) {
    const size_t n = (size_t)kPoints * p->Cp * L.cin_p;
    LZB_CUDA(cudaMalloc(&L.U, n * sizeof(T)));
    repack_u_kernel<T><<<1024, 256>>>(U32_dev, static_cast<T*>(L.U), c_in, p->channels, L.cin_p, p->Cp);
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

template <typename T>
int upload_layer_direct_t(lzb_pipe* p, Layer& L, const float* U32_dev, int c_in) {
    const size_t n = (size_t)9 * p->Cp * L.cin_p;
    LZB_CUDA(cudaMalloc(&L.Wd, n * sizeof(T)));
    LZB_CUDA(cudaMemset(L.Wd, 0, n * sizeof(T)));
    dc::untransform_u_kernel<T><<<256, 256>>>(U32_dev, static_cast<T*>(L.Wd), c_in, p->channels,
                                              L.cin_p, p->Cp);
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

int upload_padded(float** dst, const float* src, int n, int n_pad) {
    std::vector<float> tmp(n_pad, 0.0f);
    std::memcpy(tmp.data(), src, sizeof(float) * n);
    LZB_CUDA(cudaMalloc(dst, sizeof(float) * n_pad));
    LZB_CUDA(cudaMemcpy(*dst, tmp.data(), sizeof(float) * n_pad, cudaMemcpyHostToDevice));
    return LZB_OK;
}

int upload_plain(float** dst, const float* src, size_t n) {
    LZB_CUDA(cudaMalloc(dst, sizeof(float) * n));
    LZB_CUDA(cudaMemcpy(*dst, src, sizeof(float) * n, cudaMemcpyHostToDevice));
    return LZB_OK;
}

int upload_transposed(float** dst, const float* src, int rows, int cols) {
    std::vector<float> t((size_t)rows * cols);
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < cols; c++) t[(size_t)c * rows + r] = src[(size_t)r * cols + c];
    return upload_plain(dst, t.data(), t.size());
}

// ---- launches -------------------------------------------------------------

enum KernelClass { kClassContraction = 0, kClassTransform = 1, kClassInput = 2, kClassHead = 3 };

// Counts a launch and, while profiling, brackets it with two events.
struct LaunchScope {
    lzb_ctx* c;
    LaunchScope(lzb_ctx* ctx, int cls, int layers = 1) : c(ctx) {
        c->launches++;
        if (c->profiling) {
            cudaEvent_t a, b;
            cudaEventCreate(&a);
            cudaEventCreate(&b);
            c->prof_events.push_back(a);
            c->prof_events.push_back(b);
            c->prof_class.push_back(cls);
            c->prof_layers.push_back(layers);
            cudaEventRecord(a, c->stream);
        }
    }
    ~LaunchScope() {
        if (c->profiling) cudaEventRecord(c->prof_events.back(), c->stream);
    }
};

// fp32: FFMA contraction.
int launch_gemm_f32(lzb_ctx* c, const Layer& L, int P) {
    lzb_pipe* p = c->pipe;
    {
        LaunchScope scope(c, kClassContraction);
        // 128-row tiles (V and M have Pa rows, a multiple of 128; rows beyond P
        // are scratch), 128 output channels per tile where they divide evenly;
        // persistent CTAs, two per SM
        const int bn = p->Cp % 128 == 0 ? 128 : 64;
        const int row_tiles = round_up(P, kSimtBigM) / kSimtBigM;
        const int tiles = row_tiles * (p->Cp / bn) * kPoints;
        const int grid = tiles < 2 * p->sm_count ? tiles : 2 * p->sm_count;
        if (bn == 128) {
            gemm_f32_big_kernel<128><<<grid, 256, 0, c->stream>>>(
                static_cast<const float*>(c->V), static_cast<const float*>(L.U),
                static_cast<float*>(c->M), c->Pa, L.cin_p, p->Cp, row_tiles);
        } else {
            gemm_f32_big_kernel<64><<<grid, 256, 0, c->stream>>>(
                static_cast<const float*>(c->V), static_cast<const float*>(L.U),
                static_cast<float*>(c->M), c->Pa, L.cin_p, p->Cp, row_tiles);
        }
    }
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

// 16-bit: tcgen05 contraction, persistent CTAs.
template <typename T>
int launch_gemm_tc(lzb_ctx* c, const Layer& L, int P, bool first) {
    lzb_pipe* p = c->pipe;
    const int nblk = (P + tc::kBlockM - 1) / tc::kBlockM;
    const int items = kPoints * nblk;
    const int grid = items < p->sm_count ? items : p->sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(tc::kThreads);
    cfg.dynamicSmemBytes = tc::kSmemBytes;
    cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le;
    {
        LaunchScope scope(c, kClassContraction);
        le = cudaLaunchKernelEx(&cfg, tc::gemm_tc_kernel<T>, first ? c->tmV_first : c->tmV, L.tmU,
                                static_cast<T*>(c->M), c->Pa, P, p->Cp, L.cin_p / tc::kChunkK, nblk,
                                c->d_err);
    }
    LZB_CUDA(le);
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

// The 36 channel contractions of one layer in the storage type T.
template <typename T>
int contraction(lzb_ctx* c, const Layer& L, int P, bool first) {
    return launch_gemm_tc<T>(c, L, P, first);
}
template <>
int contraction<float>(lzb_ctx* c, const Layer& L, int P, bool) {
    return launch_gemm_f32(c, L, P);
}

template <typename T>
int launch_xform(lzb_ctx* c, const Layer& L, int nb, const T* R, T* X_out, T* V) {
    lzb_pipe* p = c->pipe;
    const dim3 grid(p->Cp / kChanPerCta, nb);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(XformShape<T>::warps * 32);
    cfg.dynamicSmemBytes = kXformSmem;
    cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le;
    {
        LaunchScope scope(c, kClassTransform);
        le = cudaLaunchKernelEx(&cfg, xform_kernel<T>, static_cast<const T*>(c->M), c->Pa, p->Cp,
                                (const float*)L.mean, (const float*)L.invstd, R, X_out, V);
    }
    LZB_CUDA(le);
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

// One micro-batch (nb positions, device pointers) through the whole tower.
template <typename T>
int run_tower(lzb_ctx* c, const float* in_dev, int nb, float* pol_dev, float* val_dev) {
    lzb_pipe* p = c->pipe;
    const int P = nb * kTilesPerPos;
    T* V = static_cast<T*>(c->V);
    T* X = static_cast<T*>(c->X);
    int rc;
    {
        LaunchScope scope(c, kClassInput);
        first_in_transform_kernel<T><<<(P + 7) / 8, 256, 0, c->stream>>>(in_dev, V, c->Pa, P);
    }
    LZB_CUDA(cudaGetLastError());
    if ((rc = contraction<T>(c, p->layers[0], P, true))) return rc;
    if ((rc = launch_xform<T>(c, p->layers[0], nb, nullptr, X, p->blocks ? V : nullptr))) return rc;
    for (int b = 0; b < p->blocks; b++) {
        const Layer& l1 = p->layers[1 + 2 * b];
        const Layer& l2 = p->layers[2 + 2 * b];
        if ((rc = contraction<T>(c, l1, P, false))) return rc;
        if ((rc = launch_xform<T>(c, l1, nb, nullptr, nullptr, V))) return rc;
        if ((rc = contraction<T>(c, l2, P, false))) return rc;
        const bool last = (b + 1 == p->blocks);
        if ((rc = launch_xform<T>(c, l2, nb, X, X, last ? nullptr : V))) return rc;
    }
    const int cells = nb * kSq;
    {
        LaunchScope scope(c, kClassHead);
        head_conv_kernel<T><<<(cells + 7) / 8, 256, 0, c->stream>>>(X, p->head_w, p->Cp, cells,
                                                                     pol_dev, val_dev);
    }
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

template <typename T>
int launch_conv_direct(lzb_ctx* c, const Layer& L, int nb, const CUtensorMap& tm_in,
                       const CUtensorMap& tm_out, const T* res, const CUtensorMap* tm_in_lo = nullptr,
                       void* out = nullptr, const uint32_t* flags_in = nullptr,
                       uint32_t* flags_out = nullptr, uint32_t* counts_out = nullptr,
                       uint32_t flag_target = 0) {
    lzb_pipe* p = c->pipe;
    const int Q = static_cast<int>(dc::cells_for(nb));
    if (p->pairs) {
        const int npairs = (Q + dc2::kPairM - 1) / dc2::kPairM;
        const int max_clusters = p->sm_count / 2;
        // Few tiles (small batches) and a tower layer: split the reduction of
        // each tile over the pairs of one cluster.
        const int kchunks = L.cinw / tc::kChunkK;
        if ((p->aplanes == 1 || p->aplanes == 3) && kchunks >= 2 && kchunks <= dc3::kMaxSplit &&
            p->Cp == kchunks * dc3::kGroupCols && L.lchunks <= kchunks && npairs <= p->ksplit_max_tiles[kchunks]) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(npairs * 2 * kchunks);
            cfg.blockDim = dim3(dc::kDcThreads);
            cfg.dynamicSmemBytes = dc3::kD3SmemBytes;
            cfg.stream = c->stream;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            attr[1].id = cudaLaunchAttributeClusterDimension;
            attr[1].val.clusterDim.x = 2 * kchunks;
            attr[1].val.clusterDim.y = 1;
            attr[1].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 2;
            cudaError_t le;
            {
                LaunchScope scope(c, kClassContraction);
                auto kernel = dc3::conv_ksplit_kernel<T, 1>;
                if constexpr (std::is_same<T, __half>::value) {     // the two-plane mode is fp16 only
                    if (p->aplanes == 3 && (L.out_lo || L.lchunks > 0)) kernel = dc3::conv_ksplit_kernel<T, 3>;
                }
                const CUtensorMap& in_lo = tm_in_lo ? *tm_in_lo : tm_in;
                const CUtensorMap& w_lo = L.Wd8 ? L.tmW8[1] : L.tmW2[1];
                unsigned char* out_lo =
                    (L.out_lo && out) ? static_cast<unsigned char*>(out) + (size_t)p->Cp * p->elt : nullptr;
                unsigned char* out_hi8 =
                    (L.out_hi8 && out) ? static_cast<unsigned char*>(out) + (size_t)p->Cp * (p->elt + 1) : nullptr;
                le = cudaLaunchKernelEx(&cfg, kernel, tm_in, L.tmW2[1], tm_out, res,
                                        (const float*)L.mean, (const float*)L.invstd, Q, p->Cp, kchunks,
                                        c->d_err, in_lo, w_lo, L.lchunks, p->row_bytes() / p->elt, out_lo,
                                        out_hi8, p->row_bytes(), c->Qa, L.achunks);
            }
            LZB_CUDA(le);
            LZB_CUDA(cudaGetLastError());
            return LZB_OK;
        }
        // Small batches: cut the output channels of each tile into slices so that
        // the layer spreads over more SMs (one slice per CTA pair).
        int nsplit = 1;
        for (int ns = 4; ns > 1; ns--) {
            if (L.split_ok[ns] && npairs * ns <= max_clusters) {
                nsplit = ns;
                break;
            }
        }
        // Every CTA pair runs `rounds` units; use just enough pairs for that many
        // rounds (400 tiles on 74 pairs need 6 rounds, which 67 pairs also do:
        // the idle SMs leave their power budget to the busy ones).
        const int units = npairs * nsplit;
        const int rounds = (units + max_clusters - 1) / max_clusters;
        const int clusters = (units + rounds - 1) / rounds;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * clusters);
        cfg.blockDim = dim3(dc::kDcThreads);
        cfg.dynamicSmemBytes = dc2::kD2SmemBytes;
        cfg.stream = c->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t le;
        {
            LaunchScope scope(c, kClassContraction);
            auto kernel = nsplit > 1 ? dc2::conv_direct2_kernel<T, 1, true> : dc2::conv_direct2_kernel<T, 1, false>;
            if (p->aplanes == 2) {
                kernel = nsplit > 1 ? dc2::conv_direct2_kernel<T, 2, true> : dc2::conv_direct2_kernel<T, 2, false>;
            }
            if constexpr (std::is_same<T, __half>::value) {     // the e5m2 planes accompany fp16 only
                if (p->aplanes == 3 && (L.out_lo || L.lchunks > 0)) {
                    kernel = nsplit > 1 ? dc2::conv_direct2_kernel<T, 3, true> : dc2::conv_direct2_kernel<T, 3, false>;
                }
            }
            // the byte maps only matter to the e5m2 variant; any valid map serves the others
            const CUtensorMap& in_lo = tm_in_lo ? *tm_in_lo : tm_in;
            const CUtensorMap& w_lo = L.Wd8 ? L.tmW8[nsplit] : L.tmW2[nsplit];
            const int ldr = p->row_bytes() / p->elt;
            unsigned char* out_lo =
                (L.out_lo && out) ? static_cast<unsigned char*>(out) + (size_t)p->Cp * p->elt : nullptr;
            unsigned char* out_hi8 =
                (L.out_hi8 && out) ? static_cast<unsigned char*>(out) + (size_t)p->Cp * (p->elt + 1) : nullptr;
            le = cudaLaunchKernelEx(&cfg, kernel, tm_in, L.tmW2[nsplit], tm_out, res,
                                    (const float*)L.mean, (const float*)L.invstd, Q, p->Cp,
                                    kchunks + L.lchunks, npairs, nsplit, c->d_err, L.achunks, in_lo, w_lo,
                                    ldr, out_lo, p->row_bytes(), c->Qa, kchunks, out_hi8,
                                    nsplit == 1 ? flags_in : nullptr, nsplit == 1 ? flags_out : nullptr,
                                    counts_out, flag_target);
        }
        LZB_CUDA(le);
        LZB_CUDA(cudaGetLastError());
        return LZB_OK;
    }
    const int ntiles = (Q + dc::kTileM - 1) / dc::kTileM;
    const int tile_rounds = (ntiles + p->sm_count - 1) / p->sm_count;
    const int grid = (ntiles + tile_rounds - 1) / tile_rounds;
    {
        LaunchScope scope(c, kClassContraction);
        dc::conv_direct_kernel<T><<<grid, dc::kDcThreads, dc::kDSmemBytes, c->stream>>>(
            tm_in, L.tmW, tm_out, res, L.mean, L.invstd, Q, p->Cp, L.cin_p / tc::kChunkK, ntiles,
            c->d_err);
    }
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

// One micro-batch through the tower, direct (implicit GEMM) path: one launch
// per 3x3 layer, batch-norm / residual / ReLU in its epilogue.
template <typename T>
int run_tower_direct(lzb_ctx* c, const float* in_dev, int nb, float* pol_dev, float* val_dev) {
    lzb_pipe* p = c->pipe;
    T* X = static_cast<T*>(c->X);
    int rc;
    {
        LaunchScope scope(c, kClassInput);
        dc::input_to_cells_kernel<T><<<p->sm_count * 4, 256, 0, c->stream>>>(
            in_dev, static_cast<T*>(c->IN), nb);
    }
    LZB_CUDA(cudaGetLastError());
    // Per-tile dependencies between the layers (conv_direct2.cuh) where every
    // layer of this batch runs whole tiles on CTA pairs: more tiles than half the
    // pairs, so that neither the channel slices nor the reduction-split kernel apply.
    const int npairs = (static_cast<int>(dc::cells_for(nb)) + dc2::kPairM - 1) / dc2::kPairM;
    bool flags = c->tile_flags != nullptr && p->pairs && npairs <= c->tile_cap &&
                 2 * npairs > p->sm_count / 2;
    const long long now_ns = std::chrono::duration_cast<std::chrono::nanoseconds>(
                                 std::chrono::steady_clock::now().time_since_epoch()).count();
    if (flags && !c->tile_flags_always) {
        // A launch that waits tile by tile holds its SMs while it waits.  Alone on
        // the GPU that hides the turnover between layers (-4 % per step); beside
        // another context's tower, whose launches would have filled those gaps
        // anyway, it costs 4 %.  So: only while no other context of this pipe is at
        // work, i.e. none has work in flight or has enqueued a tower in the last 100 ms.
        std::lock_guard<std::mutex> lk(p->ctx_mutex);
        for (lzb_ctx* other : p->contexts) {
            if (other == c || other->stream == nullptr) continue;
            if (now_ns - other->last_tower_ns.load(std::memory_order_relaxed) < 100000000ll ||
                cudaStreamQuery(other->stream) == cudaErrorNotReady) {
                flags = false;
                break;
            }
        }
        (void)cudaGetLastError();       // "not ready" is an answer, not an error
    }
    c->last_tower_ns.store(now_ns, std::memory_order_relaxed);
    const uint32_t target = flags ? ++c->tower_runs : 0u;     // the number of this run
    const size_t words = (size_t)(1 + 2 * p->blocks) * c->tile_cap;
    auto layer_flags = [&](int layer) { return flags ? c->tile_flags + (size_t)layer * c->tile_cap : nullptr; };
    auto layer_counts = [&](int layer) { return flags ? c->tile_flags + words + (size_t)layer * c->tile_cap : nullptr; };
    if (flags && c->tower_kernel && p->tower_table != nullptr && !p->tower_refused) {
        // every layer in one cooperative launch (conv_tower.cuh)
        const int max_clusters = p->sm_count / 2;
        const int rounds = (npairs + max_clusters - 1) / max_clusters;
        const int clusters = (npairs + rounds - 1) / rounds;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * clusters);
        cfg.blockDim = dim3(dc::kDcThreads);
        cfg.dynamicSmemBytes = dct::kTowerSmemBytes;
        cfg.stream = c->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        auto kernel = dct::conv_tower_kernel<T, 1>;
        if constexpr (std::is_same<T, __half>::value) {
            if (p->aplanes == 3) kernel = dct::conv_tower_kernel<T, 3>;
        }
        const int n_layers = static_cast<int>(p->layers.size());
        cudaError_t le;
        {
            LaunchScope scope(c, kClassContraction, n_layers);
            le = cudaLaunchKernelEx(&cfg, kernel, c->tmIN, c->tmX, c->tmH, p->aplanes == 3 ? c->tmXl : c->tmX,
                                    p->aplanes == 3 ? c->tmHl : c->tmH, c->tmXo, c->tmHo,
                                    (const dct::TowerLayer*)p->tower_table, n_layers, X, static_cast<T*>(c->H),
                                    static_cast<int>(dc::cells_for(nb)), p->Cp, npairs, p->row_bytes() / p->elt,
                                    p->row_bytes(), c->Qa, c->tile_flags, c->tile_flags + words, c->tile_cap,
                                    target, c->d_err);
        }
        if (le == cudaSuccess) le = cudaGetLastError();
        if (le != cudaSuccess) {
            // e.g. cooperative launches with clusters not available: keep to a launch per layer
            (void)cudaGetLastError();
            p->tower_refused = true;
        } else {
            const int cells = nb * kSq;
            {
                LaunchScope scope(c, kClassHead);
                dc::head_conv_cells_kernel<T><<<(cells + 7) / 8, 256, 0, c->stream>>>(
                    X, p->head_w, p->Cp, cells, pol_dev, val_dev, p->row_bytes() / p->elt,
                    (p->aplanes == 2 || (p->aplanes == 3 && p->layers.back().out_lo)) ? p->Cp : 0,
                    p->aplanes == 3 ? 1 : 0);
            }
            LZB_CUDA(cudaGetLastError());
            return LZB_OK;
        }
    }
    if ((rc = launch_conv_direct<T>(c, p->layers[0], nb, c->tmIN, c->tmXo, nullptr, nullptr, c->X, nullptr,
                                    layer_flags(0), layer_counts(0), target))) {
        return rc;
    }
    for (int b = 0; b < p->blocks; b++) {
        if ((rc = launch_conv_direct<T>(c, p->layers[1 + 2 * b], nb, c->tmX, c->tmHo, nullptr, &c->tmXl,
                                        c->H, layer_flags(2 * b), layer_flags(1 + 2 * b),
                                        layer_counts(1 + 2 * b), target))) {
            return rc;
        }
        if ((rc = launch_conv_direct<T>(c, p->layers[2 + 2 * b], nb, c->tmH, c->tmXo, X, &c->tmHl,
                                        c->X, layer_flags(1 + 2 * b), layer_flags(2 + 2 * b),
                                        layer_counts(2 + 2 * b), target))) {
            return rc;
        }
    }
    const int cells = nb * kSq;
    {
        LaunchScope scope(c, kClassHead);
        dc::head_conv_cells_kernel<T><<<(cells + 7) / 8, 256, 0, c->stream>>>(
            X, p->head_w, p->Cp, cells, pol_dev, val_dev, p->row_bytes() / p->elt,
            (p->aplanes == 2 || (p->aplanes == 3 && p->layers.back().out_lo)) ? p->Cp : 0,
            p->aplanes == 3 ? 1 : 0);
    }
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

int run_tower_any(lzb_ctx* c, const float* in_dev, int nb, float* pol_dev, float* val_dev) {
    if (c->pipe->direct) {
        return c->pipe->precision == LZB_FP16
                   ? run_tower_direct<__half>(c, in_dev, nb, pol_dev, val_dev)
                   : run_tower_direct<__nv_bfloat16>(c, in_dev, nb, pol_dev, val_dev);
    }
    switch (c->pipe->precision) {
        case LZB_FP32: return run_tower<float>(c, in_dev, nb, pol_dev, val_dev);
        case LZB_FP16: return run_tower<__half>(c, in_dev, nb, pol_dev, val_dev);
        default: return run_tower<__nv_bfloat16>(c, in_dev, nb, pol_dev, val_dev);
    }
}

int check_ctx(lzb_ctx* c, int n) {
    if (!c || !c->pipe) return fail(LZB_ERR_ARG, "null context");
    if (!c->pipe->finalized) return fail(LZB_ERR_ARG, "pipe not finalized");
    if (n < 1 || n > c->max_batch) {
        return fail(LZB_ERR_ARG, "batch " + std::to_string(n) + " outside 1.." +
                                     std::to_string(c->max_batch));
    }
    return LZB_OK;
}

int set_smem_attrs() {
    LZB_CUDA(cudaFuncSetAttribute(xform_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kXformSmem));
    LZB_CUDA(cudaFuncSetAttribute(in_transform_kernel<float>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kXformSmem));
    LZB_CUDA(cudaFuncSetAttribute(xform_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kXformSmem));
    LZB_CUDA(cudaFuncSetAttribute(xform_kernel<__nv_bfloat16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kXformSmem));
    LZB_CUDA(cudaFuncSetAttribute(in_transform_kernel<__half>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kXformSmem));
    LZB_CUDA(cudaFuncSetAttribute(in_transform_kernel<__nv_bfloat16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kXformSmem));
    LZB_CUDA(cudaFuncSetAttribute(tc::gemm_tc_kernel<__half>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, tc::kSmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(tc::gemm_tc_kernel<__nv_bfloat16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, tc::kSmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(dc::conv_direct_kernel<__half>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dc::kDSmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(dc::conv_direct_kernel<__nv_bfloat16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dc::kDSmemBytes));
    {
        const void* variants[] = {
            (const void*)dc2::conv_direct2_kernel<__half, 1, false>, (const void*)dc2::conv_direct2_kernel<__half, 1, true>,
            (const void*)dc2::conv_direct2_kernel<__half, 2, false>, (const void*)dc2::conv_direct2_kernel<__half, 2, true>,
            (const void*)dc2::conv_direct2_kernel<__half, 3, false>, (const void*)dc2::conv_direct2_kernel<__half, 3, true>,
            (const void*)dc2::conv_direct2_kernel<__nv_bfloat16, 1, false>,
            (const void*)dc2::conv_direct2_kernel<__nv_bfloat16, 1, true>,
            (const void*)dc2::conv_direct2_kernel<__nv_bfloat16, 2, false>,
            (const void*)dc2::conv_direct2_kernel<__nv_bfloat16, 2, true>};
        for (const void* k : variants) {
            LZB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, dc2::kD2SmemBytes));
        }
    }
    LZB_CUDA(cudaFuncSetAttribute(dct::conv_tower_kernel<__half, 1>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dct::kTowerSmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(dct::conv_tower_kernel<__half, 3>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dct::kTowerSmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(dct::conv_tower_kernel<__nv_bfloat16, 1>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dct::kTowerSmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(dc3::conv_ksplit_kernel<__half, 1>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dc3::kD3SmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(dc3::conv_ksplit_kernel<__half, 3>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dc3::kD3SmemBytes));
    LZB_CUDA(cudaFuncSetAttribute(dc3::conv_ksplit_kernel<__nv_bfloat16, 1>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, dc3::kD3SmemBytes));
    return LZB_OK;
}

// How many clusters of `csize` CTAs of the reduction-split kernel fit the
// device at once (0 if the question fails: the kernel is then not used).
template <typename T>
int ksplit_resident_clusters(int csize) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize);
    cfg.blockDim = dim3(dc::kDcThreads);
    cfg.dynamicSmemBytes = dc3::kD3SmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, dc3::conv_ksplit_kernel<T, 1>, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

}  // namespace

namespace {
using namespace lzb;

template <typename T>
int debug_conv_direct_t(lzb_ctx* c, int layer, const float* in, int n, const float* residual,
                        float* out) {
    lzb_pipe* p = c->pipe;
    const Layer& L = p->layers[layer];
    const int C = p->channels;
    const size_t plane_floats = (size_t)n * C * kSq;
    const size_t in_floats = layer == 0 ? (size_t)n * LZB_IN_FLOATS : plane_floats;
    float* stage = nullptr;
    LZB_CUDA(cudaMalloc(&stage, sizeof(float) * (plane_floats > in_floats ? plane_floats : in_floats)));
    int rc = LZB_OK;
    auto guard = [&](cudaError_t e, const char* what) {
        if (rc == LZB_OK && e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    };
    T* X = static_cast<T*>(c->X);
    T* H = static_cast<T*>(c->H);
    guard(cudaMemcpyAsync(stage, in, sizeof(float) * in_floats, cudaMemcpyHostToDevice, c->stream), "copy in");
    if (layer == 0) {
        dc::input_to_cells_kernel<T><<<512, 256, 0, c->stream>>>(stage, static_cast<T*>(c->IN), n);
    } else {
        dc::nchw_to_cells_kernel<T><<<512, 256, 0, c->stream>>>(stage, H, n, C, p->Cp);
    }
    const T* R = nullptr;
    if (residual) {
        guard(cudaMemcpyAsync(stage, residual, sizeof(float) * plane_floats, cudaMemcpyHostToDevice, c->stream), "copy residual");
        dc::nchw_to_cells_kernel<T><<<512, 256, 0, c->stream>>>(stage, X, n, C, p->Cp);
        R = X;
    }
    guard(cudaGetLastError(), "layout conversion");
    if (rc == LZB_OK) rc = launch_conv_direct<T>(c, L, n, layer == 0 ? c->tmIN : c->tmH, c->tmXo, R);
    if (rc == LZB_OK) {
        dc::cells_to_nchw_kernel<T><<<512, 256, 0, c->stream>>>(X, stage, n, C, p->Cp);
        guard(cudaGetLastError(), "layout conversion");
        guard(cudaMemcpyAsync(out, stage, sizeof(float) * plane_floats, cudaMemcpyDeviceToHost, c->stream), "copy out");
    }
    int rc2 = lzb_ctx_sync(c);
    cudaFree(stage);
    return rc ? rc : rc2;
}

template <typename T>
int debug_conv_t(lzb_ctx* c, int layer, const float* in, int n, const float* residual, float* out) {
    lzb_pipe* p = c->pipe;
    const Layer& L = p->layers[layer];
    const int P = n * kTilesPerPos;
    const int C = p->channels;
    const size_t plane_floats = (size_t)n * C * kSq;
    T* V = static_cast<T*>(c->V);
    T* X = static_cast<T*>(c->X);
    float* stage = nullptr;    // fp32 NCHW staging on the device
    LZB_CUDA(cudaMalloc(&stage, sizeof(float) * (plane_floats > (size_t)n * LZB_IN_FLOATS
                                                     ? plane_floats
                                                     : (size_t)n * LZB_IN_FLOATS)));
    int rc = LZB_OK;
    auto guard = [&](cudaError_t e, const char* what) {
        if (rc == LZB_OK && e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    };
    if (layer == 0) {
        guard(cudaMemcpyAsync(stage, in, sizeof(float) * n * LZB_IN_FLOATS, cudaMemcpyHostToDevice, c->stream), "copy in");
        first_in_transform_kernel<T><<<(P + 7) / 8, 256, 0, c->stream>>>(stage, V, c->Pa, P);
    } else {
        guard(cudaMemcpyAsync(stage, in, sizeof(float) * plane_floats, cudaMemcpyHostToDevice, c->stream), "copy in");
        nchw_to_nhwc_kernel<T><<<512, 256, 0, c->stream>>>(stage, X, n, C, p->Cp);
        const dim3 grid(p->Cp / kChanPerCta, n);
        in_transform_kernel<T><<<grid, kXformThreads, kXformSmem, c->stream>>>(
            X, V, c->Pa, p->Cp);
    }
    guard(cudaGetLastError(), "input transform");
    if (rc == LZB_OK) rc = contraction<T>(c, L, P, layer == 0);
    const T* R = nullptr;
    if (rc == LZB_OK && residual) {
        guard(cudaMemcpyAsync(stage, residual, sizeof(float) * plane_floats, cudaMemcpyHostToDevice, c->stream), "copy residual");
        nchw_to_nhwc_kernel<T><<<512, 256, 0, c->stream>>>(stage, X, n, C, p->Cp);
        R = X;
    }
    if (rc == LZB_OK) rc = launch_xform<T>(c, L, n, R, X, nullptr);
    if (rc == LZB_OK) {
        nhwc_to_nchw_kernel<T><<<512, 256, 0, c->stream>>>(X, stage, n, C, p->Cp);
        guard(cudaGetLastError(), "layout conversion");
        guard(cudaMemcpyAsync(out, stage, sizeof(float) * plane_floats, cudaMemcpyDeviceToHost, c->stream), "copy out");
    }
    int rc2 = lzb_ctx_sync(c);
    cudaFree(stage);
    return rc ? rc : rc2;
}
}  // namespace

// A wait that nothing will ever satisfy, bounded like every wait in the
// tensor-core kernels: the barrier expects one arrival and nobody arrives, so
// the wait runs out after limit_ns, records its code and the kernel returns
// normally.  Used to check, without hanging anything, that a kernel giving up
// a wait reaches the host as LZB_ERR_DEVICE_WAIT and leaves the context usable.
namespace {
constexpr int kErrWaitProbe = 900;
__global__ void wait_probe_kernel(int* err, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = lzb::tc::smem_u32(&bar);
    if (threadIdx.x == 0) {
        lzb::tc::mbar_init(b, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0 && !lzb::tc::mbar_try_wait(b, 0)) {
        lzb::tc::mbar_wait_slow(b, 0, &abort_flag, err, kErrWaitProbe, limit_ns);
    }
}
}  // namespace

namespace {
// Upload one 3x3 layer from either the Winograd-transformed U[36][c_in][K] or
// the plain filters f[K][c_in][3][3] and bring it into the layout of the
// pipe's mode.
int install_conv(lzb_pipe* p, int layer, const float* src, int c_in, const float* bn_mean,
                 const float* bn_invstd, bool src_is_filters) {
    if (!p || !src || !bn_mean || !bn_invstd) return fail(LZB_ERR_ARG, "null argument");
    if (p->finalized) return fail(LZB_ERR_ARG, "pipe already finalized");
    if (layer < 0 || layer >= (int)p->layers.size()) return fail(LZB_ERR_ARG, "layer out of range");
    const int want = layer == 0 ? kInputPlanes : p->channels;
    if (c_in != want) return fail(LZB_ERR_ARG, "c_in does not match the layer");
    LZB_CUDA(enter_device(p->device));
    Layer& L = p->layers[layer];
    if (L.present) return fail(LZB_ERR_ARG, "layer pushed twice");
    L.cin_p = round_up(c_in, 64);
    const int K = p->channels;
    const size_t n_src = (size_t)(src_is_filters ? 9 : kPoints) * c_in * K;
    const size_t n_u32 = (size_t)kPoints * c_in * K;
    float* src_dev = nullptr;
    float* U32 = nullptr;            // transformed filters on the device (Winograd modes)
    LZB_CUDA(cudaMalloc(&src_dev, n_src * sizeof(float)));
    cudaError_t e = cudaMemcpy(src_dev, src, n_src * sizeof(float), cudaMemcpyHostToDevice);
    int rc = LZB_OK;
    if (e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string("weight upload: ") + cudaGetErrorString(e));
    // Direct path: the weight planes along the input-channel axis.  One plane
    // normally; with two activation planes the weights repeat for the low plane,
    // and a low weight plane (against the high activations) follows if asked for.
    // The network input (layer 0) is exact in 16 bits and has no low plane.
    int wplanes = 1;
    unsigned lo_mask = 0;
    bool remainder8 = false;         // this layer's e5m2 weights carry the remainder plane too
    if (p->direct) {
        const int act_planes = (p->aplanes == 2 && layer > 0) ? 2 : 1;
        // the network input is exact in 16 bits: a layer-0 weight remainder is a second fp16 plane
        const bool wsplit = p->wsplit || (p->aplanes == 3 && layer == 0 && p->wlo_layers > 0);
        wplanes = act_planes + (wsplit ? 1 : 0);
        if (wsplit) lo_mask = 1u << (wplanes - 1);
        L.cinw = L.cin_p * wplanes;
        L.achunks = L.cin_p * act_planes / 64;
        // e5m2 planes of the activations: 128 channels per chunk, none for the network
        // input and none beyond the layers that carry them; lo alone, or lo and hi8
        // (2 cin_p bytes, always whole chunks)
        remainder8 = p->aplanes == 3 && layer > 0 && layer < p->wlo_layers;
        if (p->aplanes == 3 && layer > 0 && layer < p->lo_layers) {
            L.lchunks = remainder8 ? L.cin_p / 64 : (L.cin_p + 127) / 128;
        }
        L.out_lo = p->aplanes == 3 && layer < p->lo_layers;
        L.out_hi8 = p->aplanes == 3 && layer + 1 < p->wlo_layers;
    }
    float* Wd32 = nullptr;           // fp32 filters in the implicit-GEMM layout (widened modes)
    if (rc == LZB_OK && p->direct && src_is_filters) {
        // plain filters into the implicit-GEMM layout, no transform involved
        const size_t n = (size_t)9 * p->Cp * L.cinw * p->elt;
        e = cudaMalloc(&L.Wd, n);
        if (e == cudaSuccess) e = cudaMemset(L.Wd, 0, n);
        if (e == cudaSuccess && p->aplanes >= 2) {
            const size_t n32 = (size_t)9 * p->Cp * L.cin_p * sizeof(float);
            e = cudaMalloc(&Wd32, n32);
            if (e == cudaSuccess) e = cudaMemset(Wd32, 0, n32);
            if (e == cudaSuccess) {
                dc::filters_to_wd_kernel<float><<<256, 256>>>(src_dev, Wd32, c_in, K, L.cin_p, p->Cp);
                e = cudaGetLastError();
            }
        } else if (e == cudaSuccess) {
            if (p->precision == LZB_FP16) {
                dc::filters_to_wd_kernel<__half><<<256, 256>>>(src_dev, static_cast<__half*>(L.Wd), c_in, K,
                                                               L.cin_p, p->Cp);
            } else {
                dc::filters_to_wd_kernel<__nv_bfloat16><<<256, 256>>>(
                    src_dev, static_cast<__nv_bfloat16*>(L.Wd), c_in, K, L.cin_p, p->Cp);
            }
            e = cudaGetLastError();
        }
        if (e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string("filter upload: ") + cudaGetErrorString(e));
    } else if (rc == LZB_OK) {
        const float* u_dev = src_dev;
        if (src_is_filters) {
            e = cudaMalloc(&U32, n_u32 * sizeof(float));
            if (e == cudaSuccess) {
                transform_f_kernel<<<256, 256>>>(src_dev, U32, c_in, K);
                e = cudaGetLastError();
            }
            if (e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string("filter transform: ") + cudaGetErrorString(e));
            u_dev = U32;
        }
        if (rc == LZB_OK) {
            if (p->direct && p->aplanes >= 2) {
                const size_t n32 = (size_t)9 * p->Cp * L.cin_p * sizeof(float);
                e = cudaMalloc(&Wd32, n32);
                if (e == cudaSuccess) e = cudaMemset(Wd32, 0, n32);
                if (e == cudaSuccess) e = cudaMalloc(&L.Wd, (size_t)9 * p->Cp * L.cinw * p->elt);
                if (e == cudaSuccess) {
                    dc::untransform_u_kernel<float><<<256, 256>>>(u_dev, Wd32, c_in, p->channels, L.cin_p,
                                                                  p->Cp);
                    e = cudaGetLastError();
                }
                if (e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string("filter upload: ") + cudaGetErrorString(e));
            } else if (p->direct) {
                rc = p->precision == LZB_FP16 ? upload_layer_direct_t<__half>(p, L, u_dev, c_in)
                                              : upload_layer_direct_t<__nv_bfloat16>(p, L, u_dev, c_in);
            } else if (p->precision == LZB_FP32) {
                rc = upload_layer_t<float>(p, L, u_dev, c_in);
            } else if (p->precision == LZB_FP16) {
                rc = upload_layer_t<__half>(p, L, u_dev, c_in);
            } else {
                rc = upload_layer_t<__nv_bfloat16>(p, L, u_dev, c_in);
            }
        }
    }
    if (rc == LZB_OK && Wd32 != nullptr) {
        if (p->precision == LZB_FP16) {
            dc::widen_weights_kernel<__half><<<512, 256>>>(Wd32, static_cast<__half*>(L.Wd), L.cin_p, p->Cp,
                                                           wplanes, lo_mask);
        } else {
            dc::widen_weights_kernel<__nv_bfloat16><<<512, 256>>>(
                Wd32, static_cast<__nv_bfloat16*>(L.Wd), L.cin_p, p->Cp, wplanes, lo_mask);
        }
        e = cudaGetLastError();
        if (e == cudaSuccess && L.lchunks > 0) {
            const int cin8 = L.lchunks * 128;
            e = cudaMalloc(&L.Wd8, (size_t)9 * p->Cp * cin8);
            if (e == cudaSuccess) {
                dc::weights_to_e5m2_kernel<<<512, 256>>>(Wd32, L.Wd8, L.cin_p, cin8, p->Cp, remainder8 ? 1 : 0);
                e = cudaGetLastError();
            }
        }
        if (e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string("weight planes: ") + cudaGetErrorString(e));
    }
    if (rc == LZB_OK) {
        e = cudaDeviceSynchronize();
        if (e != cudaSuccess) rc = fail(LZB_ERR_CUDA, std::string("weight repack: ") + cudaGetErrorString(e));
    }
    cudaFree(src_dev);
    cudaFree(U32);
    cudaFree(Wd32);
    if (rc) return rc;
    if ((rc = upload_padded(&L.mean, bn_mean, p->channels, p->Cp))) return rc;
    if ((rc = upload_padded(&L.invstd, bn_invstd, p->channels, p->Cp))) return rc;
    if (p->direct) {
        rc = make_map_2d(&L.tmW, p->precision, L.Wd, (uint64_t)9 * p->Cp, L.cinw, p->Cp);
        for (int ns = 1; ns <= 4 && !rc; ns++) {
            // a channel slice must be a multiple of 64 (two epilogue warps x 32 columns)
            if (p->Cp % ns != 0 || (p->Cp / ns) % 64 != 0) continue;
            rc = make_map_2d(&L.tmW2[ns], p->precision, L.Wd, (uint64_t)9 * p->Cp, L.cinw,
                             p->Cp / (2 * ns));
            if (!rc && L.Wd8) {
                rc = make_map_2d(&L.tmW8[ns], -1, L.Wd8, (uint64_t)9 * p->Cp, (uint64_t)L.lchunks * 128,
                                 p->Cp / (2 * ns), 128);
            }
            L.split_ok[ns] = (rc == LZB_OK);
        }
        if (rc) return rc;
    } else if (p->precision != LZB_FP32) {
        rc = make_map_2d(&L.tmU, p->precision, L.U, (uint64_t)kPoints * p->Cp, L.cin_p, p->Cp);
        if (rc) return rc;
    }
    L.present = true;
    return LZB_OK;
}
}  // namespace

// ===========================================================================
// C ABI
// ===========================================================================

namespace {
// LZB_FP16_X2: how many residual blocks, counted from the input, carry the e5m2
// low plane of the activations and how many also correct the rounding of
// their weights.  A rounding error made in block b is amplified by the blocks
// after it, and most by the early ones, where the residual stream is still
// small next to what a block adds to it.  Measured on a 40-block network
// (exact-accumulation emulation, 128 positions, winrate max-abs): fp16 weights
// everywhere cost 5.1e-3, exact weights in the first 4 blocks alone bring that
// to 1.6e-3; the activations' low plane stops paying somewhere after block 16.
// So the first half of a deep tower carries the low plane (shallow towers
// throughout) and the first 4 blocks correct their weights.
void default_x2_blocks(int blocks, int* activation_blocks, int* weight_blocks) {
    *activation_blocks = blocks <= 24 ? blocks : (blocks + 1) / 2;
    *weight_blocks = blocks < 4 ? blocks : 4;
}
}  // namespace

extern "C" {

const char* lzb_last_error(void) { return g_error.c_str(); }

int lzb_device_count(int* count) {
    if (!count) return fail(LZB_ERR_ARG, "null count");
    *count = 0;
    LZB_CUDA(cudaGetDeviceCount(count));
    return LZB_OK;
}

int lzb_host_alloc(void** out, size_t bytes) {
    if (!out || bytes == 0) return fail(LZB_ERR_ARG, "bad host allocation request");
    *out = nullptr;
    cudaError_t e = cudaMallocHost(out, bytes);
    if (e != cudaSuccess) {
        return fail(e == cudaErrorMemoryAllocation ? LZB_ERR_NOMEM : LZB_ERR_CUDA,
                    std::string("cudaMallocHost: ") + cudaGetErrorString(e));
    }
    return LZB_OK;
}

void lzb_host_free(void* p) {
    if (p) cudaFreeHost(p);
}

int lzb_pipe_create(lzb_pipe** out, int device, int channels, int blocks, int precision) {
    if (!out) return fail(LZB_ERR_ARG, "null out");
    *out = nullptr;
    if (channels < 1 || blocks < 0) return fail(LZB_ERR_ARG, "bad channels/blocks");
    bool direct = false, wsplit = false;
    int aplanes = 1;
    switch (precision) {
        case LZB_FP32: break;
        case LZB_FP16: case LZB_BF16: direct = true; break;
        case LZB_FP16_X2: case LZB_FP16_X3:
            aplanes = precision == LZB_FP16_X3 ? 2 : 3;
            wsplit = (precision == LZB_FP16_X3);
            precision = LZB_FP16;
            direct = true;
            break;
        case LZB_BF16_X3:
            aplanes = 2;
            wsplit = true;
            precision = LZB_BF16;
            direct = true;
            break;
        case LZB_FP16_WINOGRAD: precision = LZB_FP16; break;
        case LZB_BF16_WINOGRAD: precision = LZB_BF16; break;
        default: return fail(LZB_ERR_ARG, "unknown precision");
    }
    const int Cp = round_up(channels, 64);
    if (precision != LZB_FP32 && Cp > tc::kMaxN) {
        return fail(LZB_ERR_ARG, "tensor-core path supports at most 256 filters; use LZB_FP32");
    }
    LZB_CUDA(enter_device(device));
    cudaDeviceProp prop;
    LZB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        return fail(LZB_ERR_CUDA, std::string("device ") + prop.name +
                                      " is not compute capability 10.x; this library is sm_100a only");
    }
    int rc = set_smem_attrs();
    if (rc) return rc;
    lzb_pipe* p = new lzb_pipe;
    p->device = device;
    p->channels = channels;
    p->Cp = Cp;
    p->blocks = blocks;
    p->precision = precision;
    p->direct = direct;
    p->aplanes = aplanes;
    p->wsplit = wsplit;
    if (aplanes == 3) {
        int b0, b1;
        default_x2_blocks(blocks, &b0, &b1);
        p->lo_layers = 1 + 2 * b0;
        p->wlo_layers = b1 > 0 ? 1 + 2 * b1 : 0;
    }
    // CTA pairs are the default; LZB_CONV_PAIRS=0 selects the one-CTA-per-tile
    // kernel (kept as a cross-check and for diagnostics).
    p->pairs = direct && (aplanes >= 2 ||
                          !(getenv("LZB_CONV_PAIRS") != nullptr && atoi(getenv("LZB_CONV_PAIRS")) == 0));
    p->elt = precision == LZB_FP32 ? 4 : 2;
    p->sm_count = prop.multiProcessorCount;
    // LZB_CONV_KSPLIT=0 keeps small batches on the sliced CTA-pair kernel
    // (cross-check and diagnostics).
    if (p->pairs && (aplanes == 1 || aplanes == 3) && !(getenv("LZB_CONV_KSPLIT") != nullptr && atoi(getenv("LZB_CONV_KSPLIT")) == 0)) {
        for (int k = 2; k <= dc3::kMaxSplit; k++) {
            p->ksplit_max_tiles[k] = precision == LZB_FP16 ? ksplit_resident_clusters<__half>(2 * k)
                                                            : ksplit_resident_clusters<__nv_bfloat16>(2 * k);
        }
    }
    p->layers.resize(1 + 2 * blocks);
    *out = p;
    return LZB_OK;
}

int lzb_pipe_set_low_plane_blocks(lzb_pipe* p, int activation_blocks, int weight_blocks) {
    if (!p) return fail(LZB_ERR_ARG, "null pipe");
    if (p->aplanes != 3) return fail(LZB_ERR_ARG, "only LZB_FP16_X2 pipes carry low planes");
    for (const Layer& L : p->layers) {
        if (L.present) return fail(LZB_ERR_ARG, "set the low-plane blocks before the first layer is pushed");
    }
    int b0 = activation_blocks, b1 = weight_blocks;
    if (b0 < 0 || b0 > p->blocks) b0 = p->blocks;
    if (b1 < 0 || b1 > b0) b1 = b0;
    p->lo_layers = 1 + 2 * b0;
    // no weight correction at all: not even the input convolution's
    p->wlo_layers = weight_blocks == 0 ? 0 : 1 + 2 * b1;
    return LZB_OK;
}

void lzb_pipe_destroy(lzb_pipe* p) {
    if (!p) return;
    cudaSetDevice(p->device);
    for (auto& L : p->layers) {
        cudaFree(L.U);
        cudaFree(L.Wd);
        cudaFree(L.Wd8);
        cudaFree(L.mean);
        cudaFree(L.invstd);
    }
    cudaFree(p->head_w);
    cudaFree(p->tower_table);
    Heads& h = p->heads;
    float* hs[] = {h.bn_pol_mean, h.bn_pol_invstd, h.ip_pol_wT, h.ip_pol_b, h.bn_val_mean,
                   h.bn_val_invstd, h.ip1_val_wT, h.ip1_val_b, h.ip2_val_w, h.ip2_val_b};
    for (float* q : hs) cudaFree(q);
    delete p;
}

int lzb_pipe_push_conv(lzb_pipe* p, int layer, const float* U, int c_in, const float* bn_mean,
                       const float* bn_invstd) {
    return install_conv(p, layer, U, c_in, bn_mean, bn_invstd, false);
}

int lzb_pipe_push_conv_filters(lzb_pipe* p, int layer, const float* f, int c_in,
                               const float* bn_mean, const float* bn_invstd) {
    return install_conv(p, layer, f, c_in, bn_mean, bn_invstd, true);
}

int lzb_pipe_push_head_convs(lzb_pipe* p, const float* pol_w, const float* val_w) {
    if (!p || !pol_w || !val_w) return fail(LZB_ERR_ARG, "null argument");
    if (p->finalized) return fail(LZB_ERR_ARG, "pipe already finalized");
    LZB_CUDA(enter_device(p->device));
    std::vector<float> w((size_t)3 * p->Cp, 0.0f);
    for (int c = 0; c < p->channels; c++) {
        w[c] = pol_w[c];
        w[p->Cp + c] = pol_w[p->channels + c];
        w[2 * p->Cp + c] = val_w[c];
    }
    if (p->head_w) cudaFree(p->head_w);
    int rc = upload_plain(&p->head_w, w.data(), w.size());
    if (rc) return rc;
    p->head_convs = true;
    return LZB_OK;
}

int lzb_pipe_push_heads(lzb_pipe* p, const float* bn_pol_mean, const float* bn_pol_invstd,
                        const float* ip_pol_w, const float* ip_pol_b, const float* bn_val_mean,
                        const float* bn_val_invstd, const float* ip1_val_w, const float* ip1_val_b,
                        const float* ip2_val_w, const float* ip2_val_b) {
    if (!p || !bn_pol_mean || !bn_pol_invstd || !ip_pol_w || !ip_pol_b || !bn_val_mean ||
        !bn_val_invstd || !ip1_val_w || !ip1_val_b || !ip2_val_w || !ip2_val_b) {
        return fail(LZB_ERR_ARG, "null argument");
    }
    if (p->heads.present) return fail(LZB_ERR_ARG, "heads pushed twice");
    LZB_CUDA(enter_device(p->device));
    Heads& h = p->heads;
    int rc;
    if ((rc = upload_plain(&h.bn_pol_mean, bn_pol_mean, 2))) return rc;
    if ((rc = upload_plain(&h.bn_pol_invstd, bn_pol_invstd, 2))) return rc;
    if ((rc = upload_transposed(&h.ip_pol_wT, ip_pol_w, kMoves, 2 * kSq))) return rc;
    if ((rc = upload_plain(&h.ip_pol_b, ip_pol_b, kMoves))) return rc;
    if ((rc = upload_plain(&h.bn_val_mean, bn_val_mean, 1))) return rc;
    if ((rc = upload_plain(&h.bn_val_invstd, bn_val_invstd, 1))) return rc;
    if ((rc = upload_transposed(&h.ip1_val_wT, ip1_val_w, kValueHidden, kSq))) return rc;
    if ((rc = upload_plain(&h.ip1_val_b, ip1_val_b, kValueHidden))) return rc;
    if ((rc = upload_plain(&h.ip2_val_w, ip2_val_w, kValueHidden))) return rc;
    if ((rc = upload_plain(&h.ip2_val_b, ip2_val_b, 1))) return rc;
    h.present = true;
    return LZB_OK;
}

int lzb_pipe_finalize(lzb_pipe* p) {
    if (!p) return fail(LZB_ERR_ARG, "null pipe");
    for (size_t l = 0; l < p->layers.size(); l++) {
        if (!p->layers[l].present) return fail(LZB_ERR_ARG, "layer " + std::to_string(l) + " missing");
    }
    if (!p->head_convs) return fail(LZB_ERR_ARG, "head convolutions missing");
    // the one-launch tower (conv_tower.cuh): CTA pairs, one or the e5m2 two-plane form
    if (p->direct && p->pairs && (p->aplanes == 1 || p->aplanes == 3) && p->blocks > 0) {
        LZB_CUDA(enter_device(p->device));
        std::vector<dct::TowerLayer> table(p->layers.size());
        for (size_t l = 0; l < p->layers.size(); l++) {
            const Layer& L = p->layers[l];
            dct::TowerLayer& t = table[l];
            std::memset(&t, 0, sizeof(t));
            t.tmW = L.tmW2[1];
            t.tmWl = L.Wd8 ? L.tmW8[1] : L.tmW2[1];
            t.mean = L.mean;
            t.invstd = L.invstd;
            const bool second = l > 0 && l % 2 == 0;          // second convolution of a block
            t.in_sel = l == 0 ? 0 : (second ? 2 : 1);
            t.out_sel = (l == 0 || second) ? 1 : 2;
            t.fchunks = L.cinw / tc::kChunkK;
            t.kchunks = t.fchunks + L.lchunks;
            t.achunks = L.achunks;
            t.has_res = second ? 1 : 0;
            // the planes a layer reads and writes, as the launch-per-layer path decides them
            const bool planes = p->aplanes == 3 && (L.out_lo || L.lchunks > 0);
            t.res_lo = (second && planes) ? 1 : 0;
            t.out_lo = (planes && L.out_lo) ? 1 : 0;
            t.out_hi8 = (planes && L.out_hi8) ? 1 : 0;
        }
        LZB_CUDA(cudaMalloc(&p->tower_table, table.size() * sizeof(dct::TowerLayer)));
        LZB_CUDA(cudaMemcpy(p->tower_table, table.data(), table.size() * sizeof(dct::TowerLayer),
                            cudaMemcpyHostToDevice));
    }
    p->finalized = true;
    return LZB_OK;
}

// Positions per pass through the tower.  Direct convolution: the whole batch.
// Winograd pipeline: V and M of one micro-batch should stay in L2 (64 positions
// x 256 channels = 2 x 29 MB in 16 bits); in the 16-bit modes the fused
// transform runs one CTA per SM (25 warps), so the count is raised to the next
// one that makes its grid, (channels / 64) x positions, whole waves of the SMs
// (74 for 256 channels on 148 SMs: +10 % measured against 64).
static int default_micro_batch(const lzb_pipe* p, int cap) {
    if (p->direct) return cap;
    int n = kDefaultMicroBatch;
    if (p->elt == 2) {
        const int groups = p->Cp / kChanPerCta;
        for (int cand = kDefaultMicroBatch; cand <= 2 * p->sm_count && cand <= kMaxMicroBatch; cand++) {
            if ((groups * cand) % p->sm_count == 0) { n = cand; break; }
        }
    } else {
        // fp32: the FFMA contraction runs tiles of 128 rows x 128 (or 64) channels,
        // two CTAs per SM; take the count, from 64 down to 48, whose tiles fill
        // their last wave best (61 positions at 256 channels: 864 tiles = 2.9 waves
        // of 296, where 64 positions make 936 = 3.2)
        const int col_tiles = p->Cp / (p->Cp % 128 == 0 ? 128 : 64);
        const int slots = 2 * p->sm_count;
        double best = 0.0;
        for (int cand = kDefaultMicroBatch; cand >= 48; cand--) {
            const int tiles = round_up(cand * kTilesPerPos, kSimtBigM) / kSimtBigM * col_tiles * kPoints;
            const int waves = (tiles + slots - 1) / slots;
            const double rate = static_cast<double>(cand) / waves;     // positions per wave
            if (rate > best * 1.02) { best = rate; n = cand; }
        }
    }
    return n < cap ? n : cap;
}

int lzb_ctx_create(lzb_ctx** out, lzb_pipe* p, int max_batch) {
    if (!out) return fail(LZB_ERR_ARG, "null out");
    *out = nullptr;
    if (!p || !p->finalized) return fail(LZB_ERR_ARG, "pipe not finalized");
    if (max_batch < 1 || max_batch > (1 << 16)) return fail(LZB_ERR_ARG, "bad max_batch");
    LZB_CUDA(enter_device(p->device));
    lzb_ctx* c = new lzb_ctx;
    c->pipe = p;
    c->max_batch = max_batch;
    c->micro_cap = max_batch < kMaxMicroBatch ? max_batch : kMaxMicroBatch;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** ptr, size_t bytes) {
        if (e == cudaSuccess) e = cudaMalloc(ptr, bytes);
        if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
    };
    if (p->direct) {
        // activations are small here (no transformed tensors): the whole batch
        // goes through the tower in one piece by default
        c->micro = c->micro_cap;
        c->Qa = round_up(static_cast<int>(dc::cells_for(c->micro_cap)), dc::kTileM);
        alloc(&c->IN, (size_t)c->Qa * 64 * p->elt);
        alloc(&c->X, (size_t)c->Qa * p->row_bytes());
        alloc(&c->H, (size_t)c->Qa * p->row_bytes());
        // Layers of large batches depend on each other tile by tile instead of
        // launch by launch (conv_direct2.cuh).  Measured gain: 3-4 % per step with
        // the e5m2 planes (LZB_FP16_X2), none without them, so that mode has it by
        // default, used while the context is alone on the GPU (run_tower_direct);
        // LZB_TILE_FLAGS=0 / 1, read here, switches it off / always on for any mode.
        const char* tf = getenv("LZB_TILE_FLAGS");
        const bool tile_flags = tf != nullptr ? atoi(tf) == 1 : p->aplanes == 3;
        c->tile_flags_always = tf != nullptr && atoi(tf) == 1;
        const char* tk = getenv("LZB_TOWER_KERNEL");
        c->tower_kernel = tk != nullptr && atoi(tk) == 1;
        if (p->pairs && tile_flags) {
            c->tile_cap = (c->Qa + dc2::kPairM - 1) / dc2::kPairM;
            // two words per layer and tile: the run that completed it last, and the arrival counter
            alloc((void**)&c->tile_flags, (size_t)2 * (1 + 2 * p->blocks) * c->tile_cap * sizeof(uint32_t));
        }
    } else {
        c->micro = default_micro_batch(p, c->micro_cap);
        c->Pa = round_up(c->micro_cap * kTilesPerPos, 128);
        const size_t vm = (size_t)kPoints * c->Pa * p->Cp * p->elt;
        alloc(&c->V, vm);
        alloc(&c->M, vm);
        alloc(&c->X, (size_t)c->micro_cap * kSq * p->Cp * p->elt);
    }
    alloc((void**)&c->d_in, (size_t)max_batch * LZB_IN_FLOATS * sizeof(float));
    alloc((void**)&c->d_pol, (size_t)max_batch * LZB_POL_FLOATS * sizeof(float));
    alloc((void**)&c->d_val, (size_t)max_batch * LZB_VAL_FLOATS * sizeof(float));
    alloc((void**)&c->d_policy, (size_t)max_batch * LZB_MOVES * sizeof(float));
    alloc((void**)&c->d_winrate, (size_t)max_batch * sizeof(float));
    alloc((void**)&c->d_packed, (size_t)max_batch * LZB_PACKED_WORDS * sizeof(unsigned int));
    alloc((void**)&c->d_err, sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost((void**)&c->h_err, sizeof(int));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        const int code = (e == cudaErrorMemoryAllocation) ? LZB_ERR_NOMEM : LZB_ERR_CUDA;
        fail(code, std::string("context allocation: ") + cudaGetErrorString(e));
        lzb_ctx_destroy(c);
        return code;
    }
    *c->h_err = 0;
    {
        std::lock_guard<std::mutex> lk(p->ctx_mutex);
        p->contexts.push_back(c);
    }
    if (p->direct) {
        int rc = make_map_2d(&c->tmIN, p->precision, c->IN, (uint64_t)c->Qa, 64, dc::kWinRows);
        // 16-bit channels of a cell row (hi [+ 16-bit lo] plane) and the row pitch
        const uint64_t xp = (uint64_t)p->Cp * (p->aplanes == 2 ? 2 : 1);
        const uint64_t pitch = p->row_bytes();
        const CUtensorMapSwizzle sw128 = CU_TENSOR_MAP_SWIZZLE_128B, sw64 = CU_TENSOR_MAP_SWIZZLE_64B;
        if (!rc) rc = make_map_2d(&c->tmX, p->precision, c->X, (uint64_t)c->Qa, xp, dc::kWinRows, 64, sw128, pitch);
        if (!rc) rc = make_map_2d(&c->tmH, p->precision, c->H, (uint64_t)c->Qa, xp, dc::kWinRows, 64, sw128, pitch);
        if (!rc) rc = make_map_2d(&c->tmXo, p->precision, c->X, (uint64_t)c->Qa, xp, 32, 32, sw64, pitch);
        if (!rc) rc = make_map_2d(&c->tmHo, p->precision, c->H, (uint64_t)c->Qa, xp, 32, 32, sw64, pitch);
        if (p->aplanes == 3) {
            // the e5m2 planes: Cp bytes per row, after the 16-bit channels
            unsigned char* xl = static_cast<unsigned char*>(c->X) + 2 * p->Cp;
            unsigned char* hl = static_cast<unsigned char*>(c->H) + 2 * p->Cp;
            // ... and, where weights are corrected too, the Cp bytes of the hi8 plane behind them
            const uint64_t lb = (uint64_t)p->Cp * (p->wlo_layers > 1 ? 2 : 1);
            if (!rc) rc = make_map_2d(&c->tmXl, -1, xl, (uint64_t)c->Qa, lb, dc::kWinRows, 128, sw128, pitch);
            if (!rc) rc = make_map_2d(&c->tmHl, -1, hl, (uint64_t)c->Qa, lb, dc::kWinRows, 128, sw128, pitch);
        }
        if (rc) {
            lzb_ctx_destroy(c);
            return rc;
        }
    } else if (p->precision != LZB_FP32) {
        int rc = make_map_2d(&c->tmV_first, p->precision, c->V, (uint64_t)kPoints * c->Pa, 64, tc::kBlockM);
        if (!rc) rc = make_map_2d(&c->tmV, p->precision, c->V, (uint64_t)kPoints * c->Pa, p->Cp, tc::kBlockM);
        if (rc) {
            lzb_ctx_destroy(c);
            return rc;
        }
    }
    *out = c;
    return LZB_OK;
}

void lzb_ctx_destroy(lzb_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->pipe->device);
    {
        std::lock_guard<std::mutex> lk(c->pipe->ctx_mutex);
        auto& v = c->pipe->contexts;
        for (size_t i = 0; i < v.size(); i++) {
            if (v[i] == c) {
                v.erase(v.begin() + i);
                break;
            }
        }
    }
    if (c->stream) {
        cudaStreamSynchronize(c->stream);
        cudaStreamDestroy(c->stream);
    }
    void* ptrs[] = {c->V, c->M, c->X, c->IN, c->H, c->d_in, c->d_pol, c->d_val, c->d_policy, c->d_winrate, c->d_packed, c->d_err, c->tile_flags};
    for (void* q : ptrs) cudaFree(q);
    if (c->h_err) cudaFreeHost(c->h_err);
    delete c;
}

int lzb_ctx_micro_batch(const lzb_ctx* c) { return c ? c->micro : 0; }

int lzb_ctx_set_micro_batch(lzb_ctx* c, int positions) {
    if (!c) return fail(LZB_ERR_ARG, "null context");
    if (positions == 0) positions = default_micro_batch(c->pipe, c->micro_cap);
    if (positions < 1) return fail(LZB_ERR_ARG, "bad micro-batch");
    c->micro = positions < c->micro_cap ? positions : c->micro_cap;
    return LZB_OK;
}

long long lzb_ctx_launch_count(const lzb_ctx* c) { return c ? c->launches : 0; }

void* lzb_ctx_stream(lzb_ctx* c) { return c ? (void*)c->stream : nullptr; }

int lzb_ctx_forward_device(lzb_ctx* c, const float* in_dev, int n, float* pol_dev, float* val_dev) {
    int rc = check_ctx(c, n);
    if (rc) return rc;
    if (!in_dev || !pol_dev || !val_dev) return fail(LZB_ERR_ARG, "null buffer");
    LZB_CUDA(enter_device(c->pipe->device));
    for (int off = 0; off < n; off += c->micro) {
        const int nb = (n - off) < c->micro ? (n - off) : c->micro;
        rc = run_tower_any(c, in_dev + (size_t)off * LZB_IN_FLOATS, nb,
                           pol_dev + (size_t)off * LZB_POL_FLOATS,
                           val_dev + (size_t)off * LZB_VAL_FLOATS);
        if (rc) return rc;
    }
    return LZB_OK;
}

int lzb_ctx_sync(lzb_ctx* c) {
    if (!c) return fail(LZB_ERR_ARG, "null context");
    LZB_CUDA(enter_device(c->pipe->device));
    LZB_CUDA(cudaMemcpyAsync(c->h_err, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    LZB_CUDA(cudaStreamSynchronize(c->stream));
    if (*c->h_err != 0) {
        const int code = *c->h_err;
        *c->h_err = 0;
        cudaMemsetAsync(c->d_err, 0, sizeof(int), c->stream);
        if (c->tile_flags != nullptr) {
            // an abandoned run may have left a tile's arrivals short of sixteen
            cudaMemsetAsync(c->tile_flags, 0,
                            (size_t)2 * (1 + 2 * c->pipe->blocks) * c->tile_cap * sizeof(uint32_t), c->stream);
            c->tower_runs = 0;
        }
        return fail(LZB_ERR_DEVICE_WAIT,
                    "a kernel gave up a bounded wait (code " + std::to_string(code) + ")");
    }
    return LZB_OK;
}

int lzb_ctx_forward(lzb_ctx* c, const float* in, int n, float* pol, float* val) {
    int rc = check_ctx(c, n);
    if (rc) return rc;
    if (!in || !pol || !val) return fail(LZB_ERR_ARG, "null buffer");
    LZB_CUDA(enter_device(c->pipe->device));
    LZB_CUDA(cudaMemcpyAsync(c->d_in, in, (size_t)n * LZB_IN_FLOATS * sizeof(float),
                             cudaMemcpyHostToDevice, c->stream));
    if ((rc = lzb_ctx_forward_device(c, c->d_in, n, c->d_pol, c->d_val))) return rc;
    LZB_CUDA(cudaMemcpyAsync(pol, c->d_pol, (size_t)n * LZB_POL_FLOATS * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    LZB_CUDA(cudaMemcpyAsync(val, c->d_val, (size_t)n * LZB_VAL_FLOATS * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    return lzb_ctx_sync(c);
}

int lzb_ctx_forward_heads_device(lzb_ctx* c, const float* in_dev, int n, float softmax_temp,
                                 float* policy_dev, float* winrate_dev) {
    int rc = check_ctx(c, n);
    if (rc) return rc;
    if (!c->pipe->heads.present) return fail(LZB_ERR_ARG, "head weights were not pushed");
    if (!(softmax_temp > 0.f)) return fail(LZB_ERR_ARG, "softmax temperature must be positive");
    if (!policy_dev || !winrate_dev) return fail(LZB_ERR_ARG, "null buffer");
    if ((rc = lzb_ctx_forward_device(c, in_dev, n, c->d_pol, c->d_val))) return rc;
    const Heads& h = c->pipe->heads;
    {
        LaunchScope scope(c, kClassHead);
        policy_head_kernel<<<n * kPolicySlices, 384, 0, c->stream>>>(c->d_pol, h.bn_pol_mean, h.bn_pol_invstd,
                                                     h.ip_pol_wT, h.ip_pol_b, 1.0f / softmax_temp,
                                                     policy_dev);
    }
    {
        LaunchScope scope(c, kClassHead);
        value_head_kernel<<<n * kValueSlices, 256, 0, c->stream>>>(c->d_val, h.bn_val_mean, h.bn_val_invstd,
                                                    h.ip1_val_wT, h.ip1_val_b, h.ip2_val_w,
                                                    h.ip2_val_b, winrate_dev);
    }
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

int lzb_ctx_forward_heads(lzb_ctx* c, const float* in, int n, float softmax_temp, float* policy,
                          float* winrate) {
    int rc = check_ctx(c, n);
    if (rc) return rc;
    if (!in || !policy || !winrate) return fail(LZB_ERR_ARG, "null buffer");
    LZB_CUDA(enter_device(c->pipe->device));
    LZB_CUDA(cudaMemcpyAsync(c->d_in, in, (size_t)n * LZB_IN_FLOATS * sizeof(float),
                             cudaMemcpyHostToDevice, c->stream));
    if ((rc = lzb_ctx_forward_heads_device(c, c->d_in, n, softmax_temp, c->d_policy, c->d_winrate))) {
        return rc;
    }
    LZB_CUDA(cudaMemcpyAsync(policy, c->d_policy, (size_t)n * LZB_MOVES * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    LZB_CUDA(cudaMemcpyAsync(winrate, c->d_winrate, (size_t)n * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    return lzb_ctx_sync(c);
}

// ---------------------------------------------------------------------------
// One 3x3 layer without any allocation (lzb_conv3x3_static).
//
// All working memory of this entry point lives in the array below, which is
// part of the library image: every GPU that loads the library holds these
// bytes until the process exits.  Limits: 8 positions, 64 input and 64 output
// channels (fp32).  Layout of the array (offsets are multiples of 256 bytes):
//   U   repacked filters   [36][64][64] fp32
//   V   transformed input  [36][256][64] fp32
//   M   contraction result [36][256][64] fp32
//   X   activations        [8][361][64] fp32
//   BN  mean[64], invstd[64]
// ---------------------------------------------------------------------------
constexpr int kStaticMaxBatch = 8;
constexpr int kStaticMaxChannels = 64;
constexpr int kStaticRows = 256;   // 8 * 25 = 200 tiles, rounded up to the contraction tile
constexpr size_t kStaticU = 0;
constexpr size_t kStaticV = kStaticU + (size_t)36 * 64 * 64 * 4;
constexpr size_t kStaticM = kStaticV + (size_t)36 * kStaticRows * 64 * 4;
constexpr size_t kStaticX = kStaticM + (size_t)36 * kStaticRows * 64 * 4;
constexpr size_t kStaticBN = kStaticX + (size_t)kStaticMaxBatch * 361 * 64 * 4;
constexpr size_t kStaticScratchBytes = kStaticBN + 2 * 64 * 4 + 256;
static_assert(kStaticV % 256 == 0 && kStaticM % 256 == 0 && kStaticX % 256 == 0 && kStaticBN % 256 == 0,
              "sub-buffers must keep the 256-byte alignment of the array");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kStaticMaxDevices = 64;
std::mutex g_static_mutex;
unsigned char* g_static_ptr[kStaticMaxDevices] = {};   // device address of the array, per device

// Once per device, with that device current: ask the runtime where the array
// lives on this GPU.  In host code the name g_static_scratch is only a handle
// for the symbol, not an address a kernel could use.
int static_scratch_for(int device, unsigned char** out) {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[device]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            return fail(LZB_ERR_CUDA, std::string("cudaGetSymbolAddress(g_static_scratch): ") +
                                          cudaGetErrorString(e));
        }
        e = cudaFuncSetAttribute(lzb::xform_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kXformSmem);
        if (e == cudaSuccess) {
            e = cudaFuncSetAttribute(lzb::in_transform_kernel<float>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kXformSmem);
        }
        if (e != cudaSuccess) {
            return fail(LZB_ERR_CUDA, std::string("kernel attribute set-up: ") + cudaGetErrorString(e));
        }
        g_static_ptr[device] = static_cast<unsigned char*>(ptr);
    }
    *out = g_static_ptr[device];
    return LZB_OK;
}
}  // namespace

int lzb_conv3x3_static(int device, const float* in_dev, int n, int c_in, int channels,
                       const float* U_dev, const float* bn_mean_dev, const float* bn_invstd_dev,
                       const float* residual_dev, float* out_dev, void* stream_handle) {
    using namespace lzb;
    if (!in_dev || !U_dev || !bn_mean_dev || !bn_invstd_dev || !out_dev) {
        return fail(LZB_ERR_ARG, "null device pointer");
    }
    if (device < 0 || device >= kStaticMaxDevices) return fail(LZB_ERR_ARG, "device ordinal out of range");
    if (n < 1 || n > kStaticMaxBatch) {
        return fail(LZB_ERR_ARG, "lzb_conv3x3_static handles 1.." + std::to_string(kStaticMaxBatch) +
                                     " positions, got " + std::to_string(n));
    }
    if (c_in < 1 || c_in > kStaticMaxChannels || channels < 1 || channels > kStaticMaxChannels) {
        return fail(LZB_ERR_ARG, "lzb_conv3x3_static handles at most " +
                                     std::to_string(kStaticMaxChannels) + " input and output channels, got " +
                                     std::to_string(c_in) + " and " + std::to_string(channels));
    }
    LZB_CUDA(enter_device(device));
    unsigned char* scratch = nullptr;
    int rc = static_scratch_for(device, &scratch);
    if (rc) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    float* U = reinterpret_cast<float*>(scratch + kStaticU);
    float* V = reinterpret_cast<float*>(scratch + kStaticV);
    float* M = reinterpret_cast<float*>(scratch + kStaticM);
    float* X = reinterpret_cast<float*>(scratch + kStaticX);
    float* bn = reinterpret_cast<float*>(scratch + kStaticBN);
    const int Cp = 64, P = n * kTilesPerPos;
    // The array keeps whatever the previous call left.  Everything read below
    // is rewritten first; the padded batch-norm entries are the one part a
    // kernel does not rewrite, so they are cleared here.
    LZB_CUDA(cudaMemsetAsync(bn, 0, 2 * 64 * sizeof(float), stream));
    LZB_CUDA(cudaMemcpyAsync(bn, bn_mean_dev, channels * sizeof(float), cudaMemcpyDeviceToDevice, stream));
    LZB_CUDA(cudaMemcpyAsync(bn + 64, bn_invstd_dev, channels * sizeof(float), cudaMemcpyDeviceToDevice,
                             stream));
    repack_u_kernel<float><<<144, 256, 0, stream>>>(U_dev, U, c_in, channels, Cp, Cp);
    nchw_to_nhwc_kernel<float><<<128, 256, 0, stream>>>(in_dev, X, n, c_in, Cp);
    const dim3 tgrid(Cp / kChanPerCta, n);
    const size_t tsmem = kXformSmem;
    in_transform_kernel<float><<<tgrid, kXformThreads, tsmem, stream>>>(X, V, kStaticRows, Cp);
    const dim3 ggrid(round_up(P, kSimtTile) / kSimtTile, Cp / kSimtTile, kPoints);
    gemm_f32_kernel<<<ggrid, 256, 0, stream>>>(V, U, M, kStaticRows, Cp, Cp);
    const float* R = nullptr;
    if (residual_dev) {
        nchw_to_nhwc_kernel<float><<<128, 256, 0, stream>>>(residual_dev, X, n, channels, Cp);
        R = X;
    }
    xform_kernel<float><<<tgrid, XformShape<float>::warps * 32, tsmem, stream>>>(M, kStaticRows, Cp, bn, bn + 64, R, X,
                                                                  nullptr);
    nhwc_to_nchw_kernel<float><<<128, 256, 0, stream>>>(X, out_dev, n, channels, Cp);
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

namespace {
// Copy n bit-packed positions to the device and expand them into c->d_in.
int stage_packed(lzb_ctx* c, const unsigned int* planes, int n) {
    LZB_CUDA(cudaMemcpyAsync(c->d_packed, planes, (size_t)n * LZB_PACKED_WORDS * sizeof(unsigned int),
                             cudaMemcpyHostToDevice, c->stream));
    {
        LaunchScope scope(c, kClassInput);
        lzb::unpack_planes_kernel<<<c->pipe->sm_count * 2, 256, 0, c->stream>>>(c->d_packed, c->d_in, n);
    }
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}
}  // namespace

int lzb_ctx_forward_packed(lzb_ctx* c, const unsigned int* planes, int n, float* pol, float* val) {
    int rc = check_ctx(c, n);
    if (rc) return rc;
    if (!planes || !pol || !val) return fail(LZB_ERR_ARG, "null buffer");
    LZB_CUDA(enter_device(c->pipe->device));
    if ((rc = stage_packed(c, planes, n))) return rc;
    if ((rc = lzb_ctx_forward_device(c, c->d_in, n, c->d_pol, c->d_val))) return rc;
    LZB_CUDA(cudaMemcpyAsync(pol, c->d_pol, (size_t)n * LZB_POL_FLOATS * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    LZB_CUDA(cudaMemcpyAsync(val, c->d_val, (size_t)n * LZB_VAL_FLOATS * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    return lzb_ctx_sync(c);
}

int lzb_ctx_forward_heads_packed(lzb_ctx* c, const unsigned int* planes, int n, float softmax_temp,
                                 float* policy, float* winrate) {
    int rc = check_ctx(c, n);
    if (rc) return rc;
    if (!planes || !policy || !winrate) return fail(LZB_ERR_ARG, "null buffer");
    LZB_CUDA(enter_device(c->pipe->device));
    if ((rc = stage_packed(c, planes, n))) return rc;
    if ((rc = lzb_ctx_forward_heads_device(c, c->d_in, n, softmax_temp, c->d_policy, c->d_winrate))) {
        return rc;
    }
    LZB_CUDA(cudaMemcpyAsync(policy, c->d_policy, (size_t)n * LZB_MOVES * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    LZB_CUDA(cudaMemcpyAsync(winrate, c->d_winrate, (size_t)n * sizeof(float),
                             cudaMemcpyDeviceToHost, c->stream));
    return lzb_ctx_sync(c);
}

int lzb_ctx_debug_wait_probe(lzb_ctx* c, int limit_ms) {
    if (!c) return fail(LZB_ERR_ARG, "null context");
    if (limit_ms < 1 || limit_ms > 1000) return fail(LZB_ERR_ARG, "limit must be 1..1000 ms");
    LZB_CUDA(enter_device(c->pipe->device));
    wait_probe_kernel<<<1, 32, 0, c->stream>>>(c->d_err, (unsigned long long)limit_ms * 1000000ull);
    c->launches++;
    LZB_CUDA(cudaGetLastError());
    return LZB_OK;
}

int lzb_ctx_profile_begin(lzb_ctx* c) {
    if (!c) return fail(LZB_ERR_ARG, "null context");
    if (c->profiling) return fail(LZB_ERR_ARG, "profiling already on");
    c->profiling = true;
    return LZB_OK;
}

int lzb_ctx_profile_end(lzb_ctx* c, double* ms_by_class, long long* launches_by_class) {
    if (!c || !ms_by_class || !launches_by_class) return fail(LZB_ERR_ARG, "null argument");
    if (!c->profiling) return fail(LZB_ERR_ARG, "profiling is off");
    c->profiling = false;
    int rc = lzb_ctx_sync(c);
    for (int k = 0; k < 4; k++) {
        ms_by_class[k] = 0.0;
        launches_by_class[k] = 0;
    }
    for (size_t i = 0; i < c->prof_class.size(); i++) {
        float ms = 0.f;
        if (rc == LZB_OK && cudaEventElapsedTime(&ms, c->prof_events[2 * i], c->prof_events[2 * i + 1]) == cudaSuccess) {
            ms_by_class[c->prof_class[i]] += ms;
            launches_by_class[c->prof_class[i]] += c->prof_layers[i];
        }
        cudaEventDestroy(c->prof_events[2 * i]);
        cudaEventDestroy(c->prof_events[2 * i + 1]);
    }
    c->prof_events.clear();
    c->prof_class.clear();
    c->prof_layers.clear();
    return rc;
}

int lzb_ctx_debug_conv(lzb_ctx* c, int layer, const float* in, int n, const float* residual,
                       float* out) {
    if (!c || !c->pipe || !c->pipe->finalized) return fail(LZB_ERR_ARG, "context not ready");
    if (n < 1 || n > c->micro_cap) return fail(LZB_ERR_ARG, "batch outside the micro-batch capacity");
    if (layer < 0 || layer >= (int)c->pipe->layers.size()) return fail(LZB_ERR_ARG, "layer out of range");
    if (!in || !out) return fail(LZB_ERR_ARG, "null buffer");
    LZB_CUDA(enter_device(c->pipe->device));
    if (c->pipe->aplanes >= 2) {
        return fail(LZB_ERR_ARG, "single-layer diagnostics are not available in the two-plane modes");
    }
    if (c->pipe->direct) {
        return c->pipe->precision == LZB_FP16
                   ? debug_conv_direct_t<__half>(c, layer, in, n, residual, out)
                   : debug_conv_direct_t<__nv_bfloat16>(c, layer, in, n, residual, out);
    }
    switch (c->pipe->precision) {
        case LZB_FP32: return debug_conv_t<float>(c, layer, in, n, residual, out);
        case LZB_FP16: return debug_conv_t<__half>(c, layer, in, n, residual, out);
        default: return debug_conv_t<__nv_bfloat16>(c, layer, in, n, residual, out);
    }
}

}  // extern "C"
