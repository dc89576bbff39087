// Checker for the engine-level comparison: a CUDAPipe backend that evaluates
// every batch with the reference's own CPUPipe (src/CPUPipe.cpp), linked into
// the test binary engine_check only.  The engine then runs exactly as in a GPU
// build (same scheduler, same self-check draws from the random generator, same
// precision selection), with the reference arithmetic behind the queue, so a
// game played by engine_check and a game played by engine_bench on the GPU can
// be compared move by move.  Test infrastructure: the library and engine_bench
// contain no CPU evaluation path.
#include <algorithm>
#include <memory>
#include <string>
#include <vector>

#include "CPUPipe.h"
#include "cuda_scheduler.h"

namespace {
class CPUPipeBackend : public CUDAPipe::Backend {
public:
    void load(const std::vector<int>&, int channels, int, int, int, CUDAPipe::Precision,
              const ForwardPipe::ForwardPipeWeights& w) override {
        m_pipe.initialize(channels);
        m_pipe.push_weights(6, 18, channels, std::make_shared<ForwardPipe::ForwardPipeWeights>(w));
    }
    int forward(int, int, const float* in, int n, float* pol, float* val, std::string*) override {
        std::vector<float> x(CUDAPipe::kInputFloats), p(CUDAPipe::kPolicyFloats), v(CUDAPipe::kValueFloats);
        for (int i = 0; i < n; i++) {
            std::copy(in + static_cast<size_t>(i) * x.size(), in + static_cast<size_t>(i + 1) * x.size(),
                      x.begin());
            m_pipe.forward(x, p, v);   // re-entrant: all scratch is local (src/CPUPipe.cpp:392-405)
            std::copy(p.begin(), p.end(), pol + static_cast<size_t>(i) * p.size());
            std::copy(v.begin(), v.end(), val + static_cast<size_t>(i) * v.size());
        }
        return 0;
    }

private:
    CPUPipe m_pipe;
};

std::unique_ptr<CUDAPipe::Backend> make_backend() {
    return std::unique_ptr<CUDAPipe::Backend>(new CPUPipeBackend);
}
const struct Install {
    Install() { lzb_engine::backend_factory = &make_backend; }
} install;
}  // namespace
