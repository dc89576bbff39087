/*
 * C-ABI wrapper around the reference's own CPUPipe (TEST INFRASTRUCTURE).
 *
 * Compiled together with the reference's src/CPUPipe.cpp, taken unchanged
 * from where the reference tree lies, into _ref/libref_cpupipe.so by the
 * Makefile beside this file.  It lets Python drive the real CPUPipe through
 * the reference's ForwardPipe interface (src/ForwardPipe.h:38-71):
 * initialize -> push_weights -> forward.
 */
#include <cstddef>
#include <memory>
#include <vector>

#include "CPUPipe.h"
#include "Network.h"

extern "C" void openblas_set_num_threads(int);

namespace {
struct RefPipe {
    CPUPipe pipe;
    std::shared_ptr<ForwardPipe::ForwardPipeWeights> weights;
    int channels;
};
}  // namespace

extern "C" {

/* U_all, mean_all, invstd_all are the per-layer arrays concatenated in layer
 * order: U[0] is [36][18][C], the others [36][C][C]; means/invstd [C] each. */
void* ref_pipe_create(int channels, int blocks, const float* U_all,
                      const float* mean_all, const float* invstd_all,
                      const float* pol_w, const float* val_w) {
    auto* rp = new RefPipe;
    rp->channels = channels;
    auto w = std::make_shared<ForwardPipe::ForwardPipeWeights>();
    const int layers = 1 + 2 * blocks;
    size_t uoff = 0;
    for (int l = 0; l < layers; l++) {
        const size_t cin = (l == 0) ? Network::INPUT_CHANNELS : channels;
        const size_t n = size_t(WINOGRAD_TILE) * cin * channels;
        w->m_conv_weights.emplace_back(U_all + uoff, U_all + uoff + n);
        uoff += n;
        w->m_conv_biases.emplace_back(channels, 0.0f);
        w->m_batchnorm_means.emplace_back(mean_all + size_t(l) * channels,
                                          mean_all + size_t(l + 1) * channels);
        w->m_batchnorm_stddevs.emplace_back(invstd_all + size_t(l) * channels,
                                            invstd_all + size_t(l + 1) * channels);
    }
    w->m_conv_pol_w.assign(pol_w, pol_w + size_t(Network::OUTPUTS_POLICY) * channels);
    w->m_conv_pol_b.assign(Network::OUTPUTS_POLICY, 0.0f);
    w->m_conv_val_w.assign(val_w, val_w + size_t(Network::OUTPUTS_VALUE) * channels);
    w->m_conv_val_b.assign(Network::OUTPUTS_VALUE, 0.0f);
    rp->weights = w;
    rp->pipe.initialize(channels);
    rp->pipe.push_weights(WINOGRAD_ALPHA, Network::INPUT_CHANNELS, channels, w);
    return rp;
}

/* One position: in[18*361] -> pol[2*361], val[361].  Re-entrant. */
void ref_pipe_forward(void* h, const float* in, float* pol, float* val) {
    auto* rp = static_cast<RefPipe*>(h);
    const size_t sq = NUM_INTERSECTIONS;
    std::vector<float> input(in, in + Network::INPUT_CHANNELS * sq);
    std::vector<float> p(Network::OUTPUTS_POLICY * sq), v(Network::OUTPUTS_VALUE * sq);
    rp->pipe.forward(input, p, v);
    std::copy(p.begin(), p.end(), pol);
    std::copy(v.begin(), v.end(), val);
}

void ref_pipe_destroy(void* h) { delete static_cast<RefPipe*>(h); }

/* The reference pins BLAS to one thread per caller (src/Network.cpp:498-499). */
void ref_set_blas_threads(int n) { openblas_set_num_threads(n); }

}  // extern "C"
