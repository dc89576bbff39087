// Puts CUDAPipe behind the leela-zero engine WITHOUT touching the engine's
// sources.  A CPU-only build of the engine constructs its network backend as
// std::make_unique<CPUPipe>() (src/Network.cpp:598-601) and talks to it through
// the ForwardPipe interface only.  This file is linked INSTEAD of the engine's
// CPUPipe.cpp: it defines the three virtual methods the class declares
// (src/CPUPipe.h:41-49) and forwards them to a CUDAPipe kept beside the object.
// The engine then runs its search, cache and head math unchanged on top of the
// B200 pipe.  (Network::drain_evals reaches only the base-class no-op this
// way: at the end of a search the worker threads return when their current
// batch does, at most one batch-forming wait later.)
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "CPUPipe.h"
#include "CUDAPipe.h"
#include "GTP.h"

namespace lzb_engine {
std::vector<int> gpus{0};
CUDAPipe::Precision precision = CUDAPipe::Precision::FP16;
std::atomic<unsigned long long> evals{0};
CUDAPipe* last_pipe = nullptr;
int callers = 0;     // threads that will call forward(); 0: cfg_num_threads
bool eager = true;   // CUDAPipe::Batching::EAGER (measured faster under the engine); false: the reference's wait rule
}  // namespace lzb_engine

namespace {
std::mutex g_mutex;
std::map<const CPUPipe*, std::unique_ptr<CUDAPipe>> g_pipes;

CUDAPipe* pipe_of(const CPUPipe* self) {
    std::lock_guard<std::mutex> lk(g_mutex);
    return g_pipes.at(self).get();
}
}  // namespace

void CPUPipe::initialize(const int channels) {
    m_input_channels = channels;
    std::unique_ptr<CUDAPipe> pipe(new CUDAPipe(lzb_engine::gpus, static_cast<int>(cfg_batch_size),
                                                lzb_engine::callers > 0
                                                    ? lzb_engine::callers
                                                    : static_cast<int>(cfg_num_threads),
                                                lzb_engine::precision));
    if (lzb_engine::eager) pipe->set_batching(CUDAPipe::Batching::EAGER);
    pipe->initialize(channels);
    std::lock_guard<std::mutex> lk(g_mutex);
    lzb_engine::last_pipe = pipe.get();
    g_pipes[this] = std::move(pipe);
}

void CPUPipe::forward(const std::vector<float>& input, std::vector<float>& output_pol,
                      std::vector<float>& output_val) {
    lzb_engine::evals++;
    pipe_of(this)->forward(input, output_pol, output_val);
}

void CPUPipe::push_weights(const unsigned int filter_size, const unsigned int channels,
                           const unsigned int outputs,
                           std::shared_ptr<const ForwardPipeWeights> weights) {
    pipe_of(this)->push_weights(filter_size, channels, outputs, weights);
}
