// Drives the real CUDAPipe (lzb200 backend) the way the engine does: many
// threads, one position per forward() call.  Reads a network and positions
// from a binary blob written by tests/test_scheduler.py, writes the raw head
// planes of every position to the output file.
//   blob: int32 channels, blocks, n, threads, batch, gpus, precision; then per
//   layer U, mean, invstd; pol_w, val_w; n * 18*361 inputs (all fp32).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "CUDAPipe.h"

static std::vector<float> read_floats(FILE* f, size_t n) {
    std::vector<float> v(n);
    if (std::fread(v.data(), sizeof(float), n, f) != n) {
        std::fprintf(stderr, "short read\n");
        std::exit(2);
    }
    return v;
}

int main(int argc, char** argv) {
    if (argc != 3) return 2;
    FILE* f = std::fopen(argv[1], "rb");
    if (!f) return 2;
    int hdr[7];
    if (std::fread(hdr, sizeof(int), 7, f) != 7) return 2;
    const int C = hdr[0], blocks = hdr[1], n = hdr[2], threads = hdr[3], batch = hdr[4], ngpu = hdr[5];
    auto w = std::make_shared<ForwardPipe::ForwardPipeWeights>();
    for (int l = 0; l < 1 + 2 * blocks; l++) {
        const size_t cin = l == 0 ? 18 : C;
        w->m_conv_weights.push_back(read_floats(f, 36 * cin * C));
        w->m_batchnorm_means.push_back(read_floats(f, C));
        w->m_batchnorm_stddevs.push_back(read_floats(f, C));
        w->m_conv_biases.emplace_back(C, 0.0f);
    }
    w->m_conv_pol_w = read_floats(f, 2 * C);
    w->m_conv_val_w = read_floats(f, C);
    w->m_conv_pol_b.assign(2, 0.0f);
    w->m_conv_val_b.assign(1, 0.0f);
    std::vector<float> in = read_floats(f, (size_t)n * CUDAPipe::kInputFloats);
    std::fclose(f);

    std::vector<int> gpus;
    for (int g = 0; g < ngpu; g++) gpus.push_back(g);
    int failures = 0;
    std::vector<float> out((size_t)n * (CUDAPipe::kPolicyFloats + CUDAPipe::kValueFloats));
    try {
        CUDAPipe pipe(gpus, batch, threads, static_cast<CUDAPipe::Precision>(hdr[6]));
        pipe.initialize(C);
        pipe.push_weights(6, 18, C, w);
        std::atomic<int> next{0};
        std::vector<std::thread> ts;
        for (int t = 0; t < threads; t++) {
            ts.emplace_back([&] {
                std::vector<float> x(CUDAPipe::kInputFloats), p(CUDAPipe::kPolicyFloats), v(CUDAPipe::kValueFloats);
                for (int i = next++; i < n; i = next++) {
                    std::copy(in.begin() + (size_t)i * x.size(), in.begin() + (size_t)(i + 1) * x.size(), x.begin());
                    pipe.forward(x, p, v);
                    float* o = &out[(size_t)i * (p.size() + v.size())];
                    std::copy(p.begin(), p.end(), o);
                    std::copy(v.begin(), v.end(), o + p.size());
                }
            });
        }
        for (auto& t : ts) t.join();
        // drain with nothing queued, then resume: the pipe must keep working
        pipe.drain();
        pipe.resume();
        std::vector<float> x(in.begin(), in.begin() + CUDAPipe::kInputFloats), p(CUDAPipe::kPolicyFloats), v(CUDAPipe::kValueFloats);
        pipe.forward(x, p, v);
        for (size_t j = 0; j < p.size(); j++) failures += (p[j] != out[j]);
        auto s = pipe.stats();
        std::printf("batches %zu positions %zu full %zu timeouts %zu\n", s.batches, s.positions, s.full_batches, s.timeouts);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "exception: %s\n", e.what());
        return 3;
    }
    FILE* g = std::fopen(argv[2], "wb");
    std::fwrite(out.data(), sizeof(float), out.size(), g);
    std::fclose(g);
    return failures ? 1 : 0;
}
