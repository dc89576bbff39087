/*
 * lzb200_sched - C view of CUDAPipe, the batching scheduler in front of the
 * lzb200 library, for hosts that are not C++ (ctypes, cgo, JNI).
 *
 * CUDAPipe itself is the C++ class the engine uses (a ForwardPipe, see
 * leela-zero_b200/host/CUDAPipe.h): callers block with their positions, worker
 * threads per GPU gather them into batches and run them through lzb200.h.
 * These functions wrap one CUDAPipe object; they take the role the methods of
 * OpenCLScheduler have for the engine (src/OpenCLScheduler.h:50-118).  Every
 * function returns a status; no exception crosses the boundary.
 */
#ifndef LZB200_SCHED_H
#define LZB200_SCHED_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LZB_SCHED_OK 0
#define LZB_SCHED_ERROR 1    /* see lzb_sched_last_error()                                  */
#define LZB_SCHED_HALTED 2   /* the pipe is draining: NetworkHaltException in the C++ class */

typedef struct lzb_sched lzb_sched;

/* Text of the last error raised on the calling thread. */
const char* lzb_sched_last_error(void);

/*
 * A scheduler over the CUDA devices gpus[0..n_gpus) (n_gpus 0: device 0), with
 * batches of up to batch_size positions and worker threads sized for
 * num_threads callers, as OpenCLScheduler sizes them from cfg_batch_size and
 * cfg_num_threads (src/OpenCLScheduler.cpp:85-125).  precision is one of the
 * LZB_* modes of lzb200.h.  eager != 0 selects the batch-forming rule for
 * callers that do not come from one search tree (take what is waiting as soon
 * as the GPU has room) instead of the reference's full-batch-or-time-out rule
 * (src/OpenCLScheduler.cpp:293-353).
 */
int lzb_sched_create(lzb_sched** out, const int* gpus, int n_gpus, int batch_size, int num_threads,
                     int precision, int eager);
void lzb_sched_destroy(lzb_sched* s);

/*
 * The weights, in the order the engine holds them in ForwardPipeWeights
 * (src/ForwardPipe.h:40-54): one call per 3x3 layer (the input convolution
 * first) with U fp32 [36][c_in][channels], the batch-norm mean with the bias
 * folded in and 1/sqrt(var + 1e-5); then lzb_sched_start with the two 1x1 head
 * convolutions, which uploads everything to every GPU and starts the workers
 * (ForwardPipe::initialize + push_weights, src/Network.cpp:407-414).
 */
int lzb_sched_add_conv(lzb_sched* s, const float* U, int c_in, int channels, const float* bn_mean,
                       const float* bn_invstd);
int lzb_sched_start(lzb_sched* s, int channels, const float* pol_w, const float* val_w);

/*
 * Evaluate n positions (any host memory): in [n][18][361], pol [n][2][361],
 * val [n][361], the raw head planes of ForwardPipe::forward
 * (src/ForwardPipe.h:62-64).  Blocks until all are done; callable from any
 * number of threads at once.  n = 1 is ForwardPipe::forward.
 */
int lzb_sched_forward(lzb_sched* s, const float* in, int n, float* pol, float* val);

/* ForwardPipe::drain / resume (src/OpenCLScheduler.cpp:412-441). */
int lzb_sched_drain(lzb_sched* s);
int lzb_sched_resume(lzb_sched* s);

/*
 * Counters since start: out[0] backend calls (batches), [1] positions, [2]
 * full batches, [3] batches sent because the wait ran out, [4] batches whose
 * input went to the GPU as bit planes, [5] callers sent away while draining,
 * [6] GPUs still in service, [7] current wait for a full batch in ms.
 */
int lzb_sched_stats(const lzb_sched* s, unsigned long long out[8]);

#ifdef __cplusplus
}
#endif
#endif
