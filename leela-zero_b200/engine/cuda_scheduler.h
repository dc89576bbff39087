// CUDAPipe in the place of OpenCLScheduler, with the engine's sources unchanged.
//
// The engine constructs its GPU backend as OpenCLScheduler<float> or
// OpenCLScheduler<half_float::half> (src/Network.cpp:426, 437, 448, 465, 472,
// 481, 488, 596) and afterwards talks to it through ForwardPipe only.  This
// header is force-included (g++ -include) in front of every engine source of
// the CUDA build.  It claims the include guard of src/OpenCLScheduler.h, so the
// engine's own `#include "OpenCLScheduler.h"` lines bring in nothing, and it
// declares a class template of the same name that IS a CUDAPipe.  The engine is
// then compiled as a normal GPU build (no USE_CPU_ONLY), which keeps everything
// the reference ties to its GPU backend:
//   * Network::select_precision (src/Network.cpp:417-493), including the
//     fall-back to single precision when the half-precision pipe fails to
//     initialise or fails its first checked evaluation (:426-441);
//   * the CPU reference pipe m_forward_cpu and the built-in self-check
//     (src/Network.cpp:583-587, 667-690, 781-791), forced once by
//     benchmark_time (:102-105) and drawn with probability 1/2000 in play;
//   * Network::drain_evals / resume_evals reaching the scheduler's drain and
//     resume (src/Network.cpp:1052-1058, src/UCTSearch.cpp:829-832);
//   * --cpu-only (cfg_cpu_only) selecting the reference's own CPUPipe.
// A maintainer who edits the engine instead adds a USE_CUDA branch at the same
// places; see the integration notes shipped with this library.
#ifndef LZB_CUDA_SCHEDULER_H
#define LZB_CUDA_SCHEDULER_H
#ifdef __cplusplus

#define OPENCLSCHEDULER_H_INCLUDED   // the guard of src/OpenCLScheduler.h:30-31

#include "config.h"

#include <atomic>
#include <memory>
#include <stdexcept>
#include <vector>

#include "CUDAPipe.h"
#include "GTP.h"

namespace lzb_engine {
// Which arithmetic stands behind the engine's two precisions.
extern CUDAPipe::Precision single_mode;   // OpenCLScheduler<float>: LZB_FP32
extern CUDAPipe::Precision half_mode;     // OpenCLScheduler<half>: LZB_FP16_X2 unless chosen otherwise
extern bool eager;                        // CUDAPipe::Batching::EAGER instead of the reference's rule
extern int callers;                       // threads that will call forward(); 0: cfg_num_threads
extern int fail_half_init;                // test hook: the next N half-precision pipes refuse to initialise
extern CUDAPipe* last_pipe;               // the pipe constructed last (statistics)
// Test hook: when set, makes the backend of every pipe constructed (a fake one,
// to drive the engine's precision selection and stop protocol without a GPU).
extern std::unique_ptr<CUDAPipe::Backend> (*backend_factory)();
extern std::atomic<unsigned long long> evals;   // forward() calls on GPU pipes
CUDAPipe::Precision precision_from_name(const char* name, bool* ok);
void note_pipe(CUDAPipe* pipe, bool alive);
}  // namespace lzb_engine

// src/OpenCLScheduler.h:44-48; UCTSearch prints it in debug builds.
struct batch_stats_t {
    std::atomic<size_t> single_evals{0};
    std::atomic<size_t> batch_evals{0};
};
extern batch_stats_t batch_stats;

template <typename net_t>
class OpenCLScheduler : public CUDAPipe {
    static constexpr bool is_half = sizeof(net_t) == 2;

public:
    // cfg_gpus, cfg_batch_size and cfg_num_threads are read where the
    // reference reads them (src/OpenCLScheduler.cpp:85-125).
    OpenCLScheduler()
        : CUDAPipe(cfg_gpus, static_cast<int>(cfg_batch_size),
                   lzb_engine::callers > 0 ? lzb_engine::callers : static_cast<int>(cfg_num_threads),
                   is_half ? lzb_engine::half_mode : lzb_engine::single_mode,
                   lzb_engine::backend_factory ? lzb_engine::backend_factory()
                                               : std::unique_ptr<CUDAPipe::Backend>()) {
        if (lzb_engine::eager) set_batching(Batching::EAGER);
        lzb_engine::note_pipe(this, true);
    }
    ~OpenCLScheduler() override { lzb_engine::note_pipe(this, false); }

    // Every B200 has the tensor cores the half-precision modes run on, so the
    // timing comparison of select_precision is skipped, as the reference does
    // for devices with native fp16 or tensor cores (src/OpenCLScheduler.cpp:146-155).
    bool needs_autodetect() override { return false; }

    void initialize(int channels) override {
        if (is_half && lzb_engine::fail_half_init > 0) {
            lzb_engine::fail_half_init--;
            throw std::runtime_error("CUDAPipe: half-precision initialisation refused (injected)");
        }
        CUDAPipe::initialize(channels);
    }

    void forward(const std::vector<float>& input, std::vector<float>& output_pol,
                 std::vector<float>& output_val) override {
        lzb_engine::evals++;
        CUDAPipe::forward(input, output_pol, output_val);
    }
};

#endif  // __cplusplus
#endif
