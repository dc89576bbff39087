// C view of CUDAPipe (include/lzb200_sched.h): one object per handle,
// exceptions turned into status codes.
#include "lzb200_sched.h"

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "CUDAPipe.h"

struct lzb_sched {
    std::unique_ptr<CUDAPipe> pipe;
    std::shared_ptr<ForwardPipe::ForwardPipeWeights> weights;
    bool started = false;
};

namespace {
thread_local std::string g_error;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return LZB_SCHED_OK;
    } catch (const NetworkHaltException&) {
        g_error = "the pipe is draining";
        return LZB_SCHED_HALTED;
    } catch (const std::exception& e) {
        g_error = e.what();
        return LZB_SCHED_ERROR;
    } catch (...) {
        g_error = "unknown exception";
        return LZB_SCHED_ERROR;
    }
}

int bad(const char* what) {
    g_error = what;
    return LZB_SCHED_ERROR;
}
}  // namespace

extern "C" {

const char* lzb_sched_last_error(void) { return g_error.c_str(); }

int lzb_sched_create(lzb_sched** out, const int* gpus, int n_gpus, int batch_size, int num_threads,
                     int precision, int eager) {
    if (!out || n_gpus < 0 || (n_gpus > 0 && !gpus) || batch_size < 1 || num_threads < 1 ||
        precision < 0 || precision > static_cast<int>(CUDAPipe::Precision::BF16_X3)) {
        return bad("lzb_sched_create: bad arguments");
    }
    return guarded([&] {
        std::unique_ptr<lzb_sched> s(new lzb_sched);
        s->pipe.reset(new CUDAPipe(std::vector<int>(gpus, gpus + n_gpus), batch_size, num_threads,
                                   static_cast<CUDAPipe::Precision>(precision)));
        if (eager) s->pipe->set_batching(CUDAPipe::Batching::EAGER);
        s->weights = std::make_shared<ForwardPipe::ForwardPipeWeights>();
        *out = s.release();
    });
}

void lzb_sched_destroy(lzb_sched* s) { delete s; }

int lzb_sched_add_conv(lzb_sched* s, const float* U, int c_in, int channels, const float* bn_mean,
                       const float* bn_invstd) {
    if (!s || !U || !bn_mean || !bn_invstd || c_in < 1 || channels < 1) return bad("lzb_sched_add_conv: bad arguments");
    if (s->started) return bad("lzb_sched_add_conv: the scheduler is already started");
    return guarded([&] {
        auto& w = *s->weights;
        w.m_conv_weights.emplace_back(U, U + static_cast<size_t>(36) * c_in * channels);
        w.m_conv_biases.emplace_back(channels, 0.0f);
        w.m_batchnorm_means.emplace_back(bn_mean, bn_mean + channels);
        w.m_batchnorm_stddevs.emplace_back(bn_invstd, bn_invstd + channels);
    });
}

int lzb_sched_start(lzb_sched* s, int channels, const float* pol_w, const float* val_w) {
    if (!s || !pol_w || !val_w || channels < 1) return bad("lzb_sched_start: bad arguments");
    if (s->started) return bad("lzb_sched_start: called twice");
    return guarded([&] {
        auto& w = *s->weights;
        w.m_conv_pol_w.assign(pol_w, pol_w + 2 * static_cast<size_t>(channels));
        w.m_conv_val_w.assign(val_w, val_w + static_cast<size_t>(channels));
        w.m_conv_pol_b.assign(2, 0.0f);
        w.m_conv_val_b.assign(1, 0.0f);
        s->pipe->initialize(channels);
        s->pipe->push_weights(6, 18, static_cast<unsigned int>(channels), s->weights);
        s->started = true;
        s->weights.reset();   // the pipe has uploaded its copies (src/Network.cpp:604-606 drops them too)
    });
}

int lzb_sched_forward(lzb_sched* s, const float* in, int n, float* pol, float* val) {
    if (!s || !s->started) return bad("lzb_sched_forward: the scheduler is not started");
    return guarded([&] { s->pipe->forward_many(in, n, pol, val); });
}

int lzb_sched_drain(lzb_sched* s) {
    if (!s || !s->started) return bad("lzb_sched_drain: the scheduler is not started");
    return guarded([&] { s->pipe->drain(); });
}

int lzb_sched_resume(lzb_sched* s) {
    if (!s || !s->started) return bad("lzb_sched_resume: the scheduler is not started");
    return guarded([&] { s->pipe->resume(); });
}

int lzb_sched_stats(const lzb_sched* s, unsigned long long out[8]) {
    if (!s || !out) return bad("lzb_sched_stats: bad arguments");
    const auto st = s->pipe->stats();
    out[0] = st.batches;
    out[1] = st.positions;
    out[2] = st.full_batches;
    out[3] = st.timeouts;
    out[4] = st.bit_plane_batches;
    out[5] = st.halted;
    out[6] = static_cast<unsigned long long>(s->pipe->live_gpus());
    out[7] = static_cast<unsigned long long>(st.wait_ms);
    return LZB_SCHED_OK;
}

}  // extern "C"
