// Stand-alone mirror of the engine's network-backend interface, used when
// CUDAPipe is built outside the leela-zero source tree (this repository's
// tests and tools).  Inside the engine, define LZ_REFERENCE_TREE and the
// engine's own ForwardPipe.h / Network.h are used instead.
//
// It restates the contract of src/ForwardPipe.h:38-71: a backend is
// initialised with the tower width, receives the (already Winograd-transformed,
// bias-folded) weights once, then evaluates one position per forward() call
// from many threads; drain()/resume() bracket the end of a search.
#ifndef LZB_FORWARD_PIPE_IFACE_H
#define LZB_FORWARD_PIPE_IFACE_H

#include <exception>
#include <memory>
#include <vector>

// Thrown out of forward() while the pipe is draining (src/Network.h:66-67).
class NetworkHaltException : public std::exception {};

class ForwardPipe {
public:
    // What Network hands over in push_weights (src/ForwardPipe.h:40-54).
    class ForwardPipeWeights {
    public:
        std::vector<std::vector<float>> m_conv_weights;       // U[36][c_in][K] per 3x3 layer
        std::vector<std::vector<float>> m_conv_biases;        // all zero after the fold
        std::vector<std::vector<float>> m_batchnorm_means;    // mean - bias
        std::vector<std::vector<float>> m_batchnorm_stddevs;  // 1 / sqrt(var + 1e-5)
        std::vector<float> m_conv_pol_w;                      // [2][K]
        std::vector<float> m_conv_pol_b;
        std::vector<float> m_conv_val_w;                      // [1][K]
        std::vector<float> m_conv_val_b;
    };

    virtual ~ForwardPipe() = default;
    virtual void initialize(int channels) = 0;
    virtual bool needs_autodetect() { return false; }
    virtual void forward(const std::vector<float>& input, std::vector<float>& output_pol,
                         std::vector<float>& output_val) = 0;
    virtual void push_weights(unsigned int filter_size, unsigned int channels, unsigned int outputs,
                              std::shared_ptr<const ForwardPipeWeights> weights) = 0;
    virtual void drain() {}
    virtual void resume() {}
};

#endif
