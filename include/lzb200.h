/*
 * lzb200 - C ABI of the B200 forward pipe for Leela Zero networks.
 *
 * This is the boundary a host program binds to.  It stands where the
 * reference engine reaches its GPU backend: a C++ ForwardPipe implementation
 * (CUDAPipe, shipped beside this library) calls these functions the way
 * OpenCLScheduler calls OpenCL_Network.  Plain pointers and sizes only; every
 * function returns a status code; no exceptions cross the boundary.
 *
 * Threading: a pipe is immutable after lzb_pipe_finalize().  Each lzb_ctx owns
 * a stream and private activation buffers, so different contexts may be
 * driven from different host threads at the same time.  One context must not
 * be used by two threads at once.
 *
 * Current device: every entry point that touches a GPU makes the device of its
 * pipe (or its `device` argument) the calling thread's current CUDA device and
 * leaves it current on return (cudaSetDevice); a host that relies on its own
 * current device sets it again after calling in.
 *
 * There is no CPU fallback: every entry point that computes needs a CUDA
 * device of compute capability 10.0 and fails with LZB_ERR_CUDA otherwise.
 */
#ifndef LZB200_H
#define LZB200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LZB_OK 0
#define LZB_ERR_ARG 1       /* bad argument, wrong call order, unsupported shape */
#define LZB_ERR_CUDA 2      /* a CUDA runtime / driver call failed               */
#define LZB_ERR_DEVICE_WAIT 3 /* a kernel gave up a bounded wait (see error text) */
#define LZB_ERR_NOMEM 4

/*
 * Arithmetic of the residual tower.
 *  LZB_FP32            Winograd F(4x4,3x3), fp32 storage, FFMA contractions: the
 *                      mode that reproduces CPUPipe to 1e-4.
 *  LZB_FP16, LZB_BF16  16-bit operands on the tensor cores (tcgen05), fp32
 *                      accumulation; each 3x3 layer is one implicit-GEMM
 *                      convolution with batch-norm/residual/ReLU in its epilogue.
 *                      LZB_FP16 is the fast mode: on 20 and 40 block networks
 *                      its winrate error reaches 6-7e-3 on a few per cent of
 *                      positions (policy within 2e-3).  The bf16 modes
 *                      (3 fewer mantissa bits) are an order of magnitude
 *                      coarser and hold only the engine's self-check (L2 of
 *                      policy and winrate differences <= 0.2,
 *                      src/Network.cpp:667-690); use LZB_FP16_X2 where the
 *                      half-precision bounds must hold for every position.
 *                      (Runs on CTA pairs; the environment variable
 *                      LZB_CONV_PAIRS=0, read at lzb_pipe_create, selects the
 *                      bit-identical single-CTA kernel for diagnostics.)
 *  LZB_*_WINOGRAD      16-bit operands on the tensor cores through the Winograd
 *                      pipeline (transform, 36 batched contractions, fused
 *                      output/input transform).  3.6x fewer multiply-adds, about
 *                      4x the rounding error of the direct form.
 *  LZB_FP16_X2         the direct convolution with activations carried as
 *                      x = hi + lo, hi in fp16 and lo in e5m2 (one byte); the
 *                      fp16 plane is multiplied with the fp16 weights, the e5m2
 *                      plane with an e5m2 copy of them (kind::f8f6f4 MMAs, half
 *                      the time of the fp16 ones): 1.5x the cost of LZB_FP16
 *                      for a layer that carries the plane.  Removes the
 *                      rounding of the activations, which is what limits
 *                      LZB_FP16 on deep networks.  Rounding errors made in the
 *                      first blocks are the ones the rest of the tower
 *                      amplifies, so by default only the first half of a tower
 *                      deeper than 24 blocks carries the low plane, and the
 *                      first 4 blocks also correct the rounding of their
 *                      weights with a third pair of e5m2 planes
 *                      (lzb_pipe_set_low_plane_blocks).  With these counts the
 *                      half-precision bounds (policy 2e-3, winrate 5e-3)
 *                      hold for every position of the 40-block benchmark
 *                      network with a factor of two to spare; a network with
 *                      sharper outputs may need more blocks (30 and 8 held
 *                      them on the hardest random network tried), which is
 *                      what the counts are adjustable for.  (For batches of
 *                      more than 23 positions the layers of this mode wait for
 *                      each other tile by tile rather than launch by launch;
 *                      the environment variable LZB_TILE_FLAGS=0 / 1, read at
 *                      lzb_ctx_create, switches that off / on for any of the
 *                      direct-convolution modes; LZB_TOWER_KERNEL=1 on top
 *                      of it runs all layers of such a batch in one
 *                      cooperative launch; results are bit-identical.)
 *  LZB_FP16_X3         activations and weights both carried as two fp16 planes
 *                      (three MMAs: hi*hi + lo*hi + hi*lo): ten times closer
 *                      to fp32 than LZB_FP16 (what remains is the accumulation
 *                      inside the tensor cores).
 *  LZB_BF16_X3         the same scheme on bf16 planes (two 8-bit mantissas per
 *                      operand): the bf16 mode that holds the half-precision
 *                      bounds, at the cost of LZB_FP16_X3.
 */
#define LZB_FP32 0
#define LZB_FP16 1
#define LZB_BF16 2
#define LZB_FP16_WINOGRAD 3
#define LZB_BF16_WINOGRAD 4
#define LZB_FP16_X2 5
#define LZB_FP16_X3 6
#define LZB_BF16_X3 7

#define LZB_INPUT_PLANES 18
#define LZB_SQ 361
#define LZB_IN_FLOATS (18 * 361)   /* one position, as Network::gather_features makes it */
#define LZB_POL_FLOATS (2 * 361)   /* policy head 1x1 conv planes                          */
#define LZB_VAL_FLOATS 361         /* value head 1x1 conv plane                            */
#define LZB_MOVES 362

typedef struct lzb_pipe lzb_pipe;  /* weights of one network on one GPU      */
typedef struct lzb_ctx lzb_ctx;    /* stream + activation buffers on a pipe  */

/* Text of the last error raised on the calling thread ("" if none). */
const char* lzb_last_error(void);

/* Number of CUDA devices visible.  Replaces the platform/device scan of
 * OpenCL::OpenCL (src/OpenCL.cpp:708-858). */
int lzb_device_count(int* count);

/*
 * Create a pipe on CUDA device `device` for a tower of `blocks` residual
 * blocks with `channels` filters.  `precision` is LZB_FP32/FP16/BF16.
 * Replaces OpenCL::initialize + OpenCL_Network construction
 * (src/OpenCL.cpp:860-930, src/OpenCLScheduler.cpp:85-106); there is no
 * tuner run, kernel shapes are fixed.
 */
int lzb_pipe_create(lzb_pipe** out, int device, int channels, int blocks,
                    int precision);
void lzb_pipe_destroy(lzb_pipe* p);

/*
 * LZB_FP16_X2 pipes only, before the first layer is pushed: which part of the
 * tower carries the correction planes.  The first `activation_blocks` residual
 * blocks (and the input convolution) carry the e5m2 low plane of the
 * activations; the first `weight_blocks` of them (at most activation_blocks)
 * also correct the rounding of their weights (a third e5m2 plane pair); the
 * blocks after them run on the fp16 plane alone.  A negative or too large count
 * means "as many as possible"; weight_blocks 0 switches the weight correction
 * off altogether.  Defaults: every block for towers of up to 24 blocks and the
 * first half of deeper ones; weights corrected in the first 4 blocks.
 * Precision selection has no finer grain than half/single in the reference
 * (cfg_precision, src/Network.cpp:417-493); this knob has no counterpart there.
 */
int lzb_pipe_set_low_plane_blocks(lzb_pipe* p, int activation_blocks, int weight_blocks);

/*
 * Upload one 3x3 convolution layer.  `layer` 0 is the input convolution
 * (c_in = 18), layers 1..2*blocks are the tower (c_in = channels).
 * U is the Winograd-transformed filter exactly as the engine hands it to a
 * ForwardPipe: fp32 [36][c_in][channels] (src/Network.cpp:215,
 * src/ForwardPipe.h:43).  bn_mean has the conv bias folded in and bn_invstd is
 * 1/sqrt(var + 1e-5) (src/Network.cpp:151-157, 554-576).
 * Replaces OpenCLScheduler::push_input_convolution / push_residual
 * (src/OpenCLScheduler.cpp:157-210).
 */
int lzb_pipe_push_conv(lzb_pipe* p, int layer, const float* U, int c_in,
                       const float* bn_mean, const float* bn_invstd);

/*
 * Same as lzb_pipe_push_conv, but from the UNTRANSFORMED filters as they stand
 * in a weights file: f fp32 [channels][c_in][3][3].  The Winograd modes compute
 * U = G f G^T on the GPU (the arithmetic of Network::winograd_transform_f,
 * src/Network.cpp:159-223); the direct-convolution modes use f as it is, which
 * spares them the recovery of f from U.  For hosts that own the weights file
 * rather than the engine's already transformed ForwardPipeWeights.
 */
int lzb_pipe_push_conv_filters(lzb_pipe* p, int layer, const float* f, int c_in,
                               const float* bn_mean, const float* bn_invstd);

/*
 * Upload the two 1x1 head convolutions: pol_w fp32 [2][channels], val_w fp32
 * [1][channels] (biases are folded away by the engine).  Replaces
 * OpenCLScheduler::push_convolve (src/OpenCLScheduler.cpp:212-221).
 */
int lzb_pipe_push_head_convs(lzb_pipe* p, const float* pol_w, const float* val_w);

/*
 * Optional: upload what Network keeps private for the heads
 * (src/Network.h:166-183) so that lzb_ctx_forward_heads can finish the
 * evaluation on the GPU.  Means have the 1x1 conv biases folded in and
 * *_invstd are 1/sqrt(var + 1e-5).  ip_pol_w [362][722], ip1_val_w [256][361],
 * ip2_val_w [256].
 */
int lzb_pipe_push_heads(lzb_pipe* p, const float* bn_pol_mean,
                        const float* bn_pol_invstd, const float* ip_pol_w,
                        const float* ip_pol_b, const float* bn_val_mean,
                        const float* bn_val_invstd, const float* ip1_val_w,
                        const float* ip1_val_b, const float* ip2_val_w,
                        const float* ip2_val_b);

/* Check that every layer arrived; after this the pipe is read-only. */
int lzb_pipe_finalize(lzb_pipe* p);

/*
 * Create an execution context able to run up to `max_batch` positions per
 * call.  Replaces the per-thread OpenCLContext with its buffers
 * (src/OpenCL.h:64-84, src/OpenCL.cpp:156-202).
 */
int lzb_ctx_create(lzb_ctx** out, lzb_pipe* p, int max_batch);
void lzb_ctx_destroy(lzb_ctx* c);

/*
 * Evaluate n positions held in HOST memory.  in: [n][18][361] fp32; pol:
 * [n][2][361]; val: [n][361] - the raw 1x1 head planes, exactly what
 * ForwardPipe::forward returns per position (src/ForwardPipe.h:62-64).
 * Copies in, runs the tower, copies out and returns when the results are in
 * pol/val.  Replaces OpenCL_Network::forward (src/OpenCL.cpp:143-329).
 */
int lzb_ctx_forward(lzb_ctx* c, const float* in, int n, float* pol, float* val);

/*
 * Same computation with DEVICE pointers, enqueued on the context's stream
 * without waiting; call lzb_ctx_sync to wait and collect the status.
 */
int lzb_ctx_forward_device(lzb_ctx* c, const float* in_dev, int n, float* pol_dev,
                           float* val_dev);

/*
 * Host buffers in, finished evaluation out: policy [n][362] after softmax
 * (temperature softmax_temp) and winrate [n] = (1 + tanh(v)) / 2, i.e. the
 * values Network::get_output_internal computes on the CPU
 * (src/Network.cpp:833-851), before the symmetry un-rotation.  Needs
 * lzb_pipe_push_heads.
 */
int lzb_ctx_forward_heads(lzb_ctx* c, const float* in, int n, float softmax_temp,
                          float* policy, float* winrate);
int lzb_ctx_forward_heads_device(lzb_ctx* c, const float* in_dev, int n,
                                 float softmax_temp, float* policy_dev,
                                 float* winrate_dev);

/*
 * Bit-packed positions.  The 18 input planes hold only zeros and ones
 * (src/Network.cpp:935-966), so a position can travel as 18 x 12 32-bit words
 * (bit i of word w of a plane = board cell 32 w + i; 864 bytes instead of the
 * 25,992 the fp32 planes take: 30x less host-to-device traffic).  planes is
 * HOST memory [n][18][12]; outputs as lzb_ctx_forward / lzb_ctx_forward_heads.
 * The planes are expanded on the GPU and then take the normal path, so results
 * are identical to the fp32 entry points.
 */
#define LZB_PACKED_WORDS (18 * 12)
int lzb_ctx_forward_packed(lzb_ctx* c, const unsigned int* planes, int n, float* pol, float* val);
int lzb_ctx_forward_heads_packed(lzb_ctx* c, const unsigned int* planes, int n, float softmax_temp,
                                 float* policy, float* winrate);

/*
 * Page-locked host memory for batch staging.  Host buffers handed to
 * lzb_ctx_forward may be any memory, but copies from and to page-locked memory
 * run at full PCIe speed and asynchronously.  Replaces the pinned output
 * buffers of the reference (CL_MEM_ALLOC_HOST_PTR, src/OpenCL.cpp:192-199).
 */
int lzb_host_alloc(void** out, size_t bytes);
void lzb_host_free(void* p);

/* Wait for everything enqueued on the context; reports device-side errors. */
int lzb_ctx_sync(lzb_ctx* c);

/* The context's cudaStream_t, for callers that time or order work on it. */
void* lzb_ctx_stream(lzb_ctx* c);

/*
 * Positions pushed through the tower together (the batch is cut into pieces
 * of this size so that the transformed tiles stay in L2).  0 restores the
 * default.
 */
int lzb_ctx_set_micro_batch(lzb_ctx* c, int positions);
/* The count in force (the library's own choice unless set). */
int lzb_ctx_micro_batch(const lzb_ctx* c);

/* Kernel launches issued by this context since it was created. */
long long lzb_ctx_launch_count(const lzb_ctx* c);

/*
 * Per-kernel timing (diagnostics; adds two CUDA events per launch while on).
 * Between begin and end every launch of this context is timed on its stream;
 * end waits for the stream and returns, per kernel class, the summed
 * durations in milliseconds and the launch counts.  Classes: 0 channel
 * contractions, 1 fused transforms, 2 input-plane transform, 3 head kernels.
 * The reference has this only inside its tuner (OpenCL event profiling,
 * src/Tuner.cpp:452-453, 542-546).
 */
int lzb_ctx_profile_begin(lzb_ctx* c);
int lzb_ctx_profile_end(lzb_ctx* c, double ms_by_class[4], long long launches_by_class[4]);

/*
 * Diagnostics for tests: run one 3x3 layer (input transform, contraction,
 * output transform + batch-norm [+ residual] + ReLU) on n positions given as
 * fp32 NCHW host arrays and return the fp32 NCHW result.  layer 0 takes
 * [n][18][361]; other layers take [n][channels][361]; residual may be NULL.
 */
int lzb_ctx_debug_conv(lzb_ctx* c, int layer, const float* in, int n,
                       const float* residual, float* out);

/*
 * Diagnostics for tests: enqueue a kernel whose only wait can never be
 * satisfied.  Like every device-side wait of this library it is bounded: after
 * limit_ms (1..1000) it records an error code and returns, and the next
 * lzb_ctx_sync reports LZB_ERR_DEVICE_WAIT.  The context stays usable.  No
 * counterpart in the reference (its kernels have no inter-thread waits).
 */
int lzb_ctx_debug_wait_probe(lzb_ctx* c, int limit_ms);

/*
 * One 3x3 layer (Winograd F(4x4,3x3) in fp32, then batch-norm, optional
 * residual, ReLU) that allocates nothing.  This entry point has no counterpart
 * in the reference.
 *
 * Who needs it: a host that has given all device memory to its own pool at
 * start-up, so that a later cudaMalloc inside this library would fail; and a
 * thread that must not stall the rest of the process, since cudaMalloc and
 * cudaFree synchronise the whole device.  Such callers cannot create a pipe
 * or a context (both allocate), but they can still run a layer through this
 * function: its working memory is a fixed array inside the library image
 * (about 6 MB, held by every GPU that loads the library until the process
 * ends), and inputs, weights and outputs are the caller's own DEVICE buffers.
 *
 * Limits: n <= 8 positions, c_in <= 64, channels <= 64; larger sizes are
 * refused with LZB_ERR_ARG and an explanatory lzb_last_error().
 * Arguments (all fp32, all on `device`): in [n][c_in][361]; U [36][c_in][channels]
 * as for lzb_pipe_push_conv; bn_mean, bn_invstd [channels]; residual
 * [n][channels][361] or NULL; out [n][channels][361].  The work is enqueued on
 * `stream` (a cudaStream_t, NULL for the default stream) and not waited for.
 *
 * The first call on each device looks up the array's device address and sets
 * kernel attributes; make that first call outside any stream capture.  It is
 * also the moment at which the CUDA driver loads this library's code onto that
 * device and with it sets the array aside (CUDA loads modules lazily, at first
 * use), which takes device memory once: a host that hands all device memory to
 * its own pool must make this first call BEFORE the pool takes the memory;
 * later calls take nothing.  All
 * calls share the one array: it is rewritten (and cleared where needed) at the
 * start of each call, and two calls whose kernels overlap on the GPU, from
 * different streams or threads, race on it.  Serialise them.
 */
int lzb_conv3x3_static(int device, const float* in, int n, int c_in, int channels,
                       const float* U, const float* bn_mean, const float* bn_invstd,
                       const float* residual, float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif
