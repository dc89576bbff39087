// CUDAPipe: the engine-facing ForwardPipe implementation for B200.
//
// It takes the place of OpenCLScheduler<net_t> (src/OpenCLScheduler.h:50-118,
// src/OpenCLScheduler.cpp:85-441): callers block in forward() with one
// position each; worker threads, some per GPU, gather the waiting positions
// into batches, run them through the lzb200 C ABI (a full network replica per
// GPU, no data moves between GPUs) and wake the callers.  drain() makes every
// queued caller throw NetworkHaltException; resume() re-opens the pipe.
//
// Differences from the OpenCL scheduler, on purpose:
//  * a batch that did not fill within the wait time is sent as it is (all
//    waiting positions, not one): the CUDA kernels take any batch size;
//  * callers wait on a completion flag, so spurious wake-ups are harmless
//    (the reference waits on the condition variable without a predicate,
//    src/OpenCLScheduler.cpp:272);
//  * a GPU whose backend call fails is taken out of rotation, the callers of
//    that batch get std::runtime_error, the other GPUs keep serving;
//  * the adaptive wait for a full batch is capped at 100 ms (the reference lets it
//    grow by 2 ms per arriving request without bound);
//  * nothing here calls exit();
//  * a second batch-forming rule, Batching::EAGER, for callers that do not come
//    from one search tree (many games in one process): a worker takes whatever
//    is waiting as soon as its GPU has room for another batch, after a short
//    gathering window, instead of waiting for a full batch.  Batch sizes then
//    follow the arrival rate: small while the GPU keeps up, full when it is the
//    limit.  The reference's rule stays the default.
#ifndef LZB_CUDAPIPE_H
#define LZB_CUDAPIPE_H

#ifdef LZ_REFERENCE_TREE
#include "ForwardPipe.h"
#include "Network.h"   // NetworkHaltException
#else
#include "forward_pipe_iface.h"
#endif

#include <atomic>
#include <condition_variable>
#include <cstddef>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

class CUDAPipe : public ForwardPipe {
public:
    enum class Precision { FP32 = 0, FP16 = 1, BF16 = 2, FP16_WINOGRAD = 3, BF16_WINOGRAD = 4,
                           FP16_X2 = 5, FP16_X3 = 6, BF16_X3 = 7 };

    // What runs a batch.  The production backend calls the lzb200 C ABI; tests
    // substitute their own to exercise the scheduler without a GPU.
    class Backend {
    public:
        virtual ~Backend() = default;
        // Called once, from push_weights.  `gpus` are device ordinals.
        virtual void load(const std::vector<int>& gpus, int channels, int blocks, int max_batch,
                          int workers_per_gpu, Precision precision,
                          const ForwardPipeWeights& weights) = 0;
        // Evaluate n positions on (gpu index, worker slot).  in [n][18*361],
        // pol [n][2*361], val [n][361].  Returns 0 or an error code and text.
        virtual int forward(int gpu_index, int worker, const float* in, int n, float* pol,
                            float* val, std::string* error) = 0;
        // Optional second form of the input: the 18 planes of a position as
        // bits ([18][12] 32-bit words, bit i of word w = cell 32 w + i), which
        // is what the engine's planes are (zeros and ones only,
        // src/Network.cpp:935-966) and 30 times less to send to the GPU.  A
        // backend that returns true from takes_bit_planes() gets a batch this
        // way whenever every value of the batch is exactly 0 or 1.
        virtual bool takes_bit_planes() const { return false; }
        virtual int forward_bit_planes(int /*gpu_index*/, int /*worker*/, const unsigned int* /*planes*/,
                                       int /*n*/, float* /*pol*/, float* /*val*/, std::string* /*error*/) {
            return -1;
        }
        // Staging memory for a worker's batches (page-locked in the production
        // backend); the default is ordinary memory.
        virtual float* alloc_staging(std::size_t floats) { return new float[floats]; }
        virtual void free_staging(float* p) { delete[] p; }
    };

    // How a worker decides that a batch is ready (see the header comment).
    enum class Batching { REFERENCE_WAIT = 0, EAGER = 1 };

    struct Stats {
        std::size_t batches = 0;        // backend calls
        std::size_t positions = 0;      // positions evaluated
        std::size_t full_batches = 0;   // calls that carried batch_size positions
        std::size_t timeouts = 0;       // calls sent because the wait ran out
        std::size_t bit_plane_batches = 0;   // calls whose input went to the GPU as bit planes
        std::size_t halted = 0;         // callers sent away with NetworkHaltException (drain)
        int wait_ms = 0;                // current wait for a full batch
    };

    // gpus: CUDA ordinals (empty = device 0), batch_size = cfg_batch_size,
    // num_threads = cfg_num_threads (sizes the worker pool like the reference).
    CUDAPipe(std::vector<int> gpus, int batch_size, int num_threads,
             Precision precision = Precision::FP16);
    // backend: what runs the batches; null selects the production backend.
    CUDAPipe(std::vector<int> gpus, int batch_size, int num_threads, Precision precision,
             std::unique_ptr<Backend> backend);
    ~CUDAPipe() override;

    void initialize(int channels) override;
    void forward(const std::vector<float>& input, std::vector<float>& output_pol,
                 std::vector<float>& output_val) override;
    void push_weights(unsigned int filter_size, unsigned int channels, unsigned int outputs,
                      std::shared_ptr<const ForwardPipeWeights> weights) override;
    void drain() override;
    void resume() override;

    // Batched form of forward() for callers that hold several positions at
    // once (many games in one process, benchmark drivers): n positions,
    // in [n][18*361], pol [n][2*361], val [n][361], any host memory.  Blocks
    // until all n are evaluated; the positions join the same queue as single
    // requests and may be spread over several batches and GPUs.  Throws like
    // forward().  Not part of ForwardPipe: the engine's interface carries one
    // position per call (src/ForwardPipe.h:62-64).
    void forward_many(const float* in, int n, float* pol, float* val);

    Stats stats() const;
    int live_gpus() const;
    Precision precision() const { return m_precision; }
    // Call before push_weights.  gather_us: how long an EAGER worker lets
    // further requests join once the first one is there.
    void set_batching(Batching mode, int gather_us = 100);

    static constexpr int kPlaneWords = 12;            // 361 cells as bits
    static constexpr int kPackedWords = 18 * kPlaneWords;
    static constexpr int kInputFloats = 18 * 361;
    static constexpr int kPolicyFloats = 2 * 361;
    static constexpr int kValueFloats = 361;
    static constexpr int kMaxWaitMs = 100;

private:
    // One blocked caller: `count` positions in the caller's own memory.  The
    // entry lives on the caller's stack; a worker touches it for the last time
    // when it sets `done` (and notifies) under the entry's mutex.
    struct Entry {
        const float* in;
        const unsigned int* bits = nullptr;   // the same positions as bit planes, if all values are 0 or 1
        float* out_p;
        float* out_v;
        int count;
        std::mutex mutex;
        std::condition_variable cv;
        bool done = false;
        bool halted = false;
        std::string error;
        Entry(const float* i, int n, float* p, float* v) : in(i), out_p(p), out_v(v), count(n) {}
    };

    void submit_and_wait(Entry* const* entries, int n_entries);
    void worker(int gpu_index, int slot);
    void serve(int gpu_index, int slot);
    void retire_gpu(int gpu_index, const std::string& error);
    std::vector<Entry*> pickup(bool* timed_out, int gpu_index);
    std::vector<Entry*> take(std::size_t positions);
    static void finish(Entry* e, bool halted, const std::string& error);

    std::vector<int> m_gpus;
    int m_batch_size;
    int m_num_threads;
    Precision m_precision;
    std::unique_ptr<Backend> m_backend;
    int m_channels = 0;
    int m_workers_per_gpu = 1;
    bool m_bit_planes = false;          // the backend takes positions as bit planes

    mutable std::mutex m_mutex;
    std::condition_variable m_cv;
    std::deque<Entry*> m_queue;
    std::size_t m_queued = 0;            // positions in m_queue
    bool m_running = true;
    std::atomic<bool> m_draining{false};
    std::atomic<bool> m_partial_in_progress{false};
    int m_wait_ms = 10;                 // start with 10 ms, adapted like the reference
    Batching m_batching = Batching::REFERENCE_WAIT;
    int m_gather_us = 100;
    std::vector<int> m_in_flight;       // EAGER: per GPU, batches picked up and not yet finished
    bool m_gathering = false;           // EAGER: a worker is inside its gathering window
    std::size_t m_last_batch = 0;       // EAGER: positions in the batch picked up last
    std::atomic<int> m_live_gpus{0};
    std::vector<char> m_gpu_failed;     // per GPU, guarded by m_mutex
    std::vector<std::thread> m_threads;
    Stats m_stats;
};

#endif
