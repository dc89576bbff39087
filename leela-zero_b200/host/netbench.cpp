// netbench: evaluations per second through the engine-facing interface.
//
// The counterpart of the engine's `netbench` command (Network::benchmark,
// src/Network.cpp:128-149; GTP side src/GTP.cpp:1055-1069): T caller threads
// loop over ForwardPipe::forward, one position per call, until N evaluations
// are done; the pipe batches them across its GPUs.  Random-init weights of the
// requested shape (throughput does not depend on their values).
//
//   netbench [--blocks B] [--filters C] [--threads T] [--batch S] [--gpus G]
//            [--iterations N] [--precision fp32|fp16|bf16|fp16x2] [--batching wait|eager]
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "CUDAPipe.h"

int main(int argc, char** argv) {
    int blocks = 15, filters = 192, threads = 64, batch = 8, gpus = 1, iterations = 16000;
    CUDAPipe::Precision precision = CUDAPipe::Precision::FP16;
    bool eager = false;
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string k = argv[i], v = argv[i + 1];
        if (k == "--blocks") blocks = std::atoi(v.c_str());
        else if (k == "--filters") filters = std::atoi(v.c_str());
        else if (k == "--threads") threads = std::atoi(v.c_str());
        else if (k == "--batch") batch = std::atoi(v.c_str());
        else if (k == "--gpus") gpus = std::atoi(v.c_str());
        else if (k == "--iterations") iterations = std::atoi(v.c_str());
        else if (k == "--precision") {
            precision = v == "fp32" ? CUDAPipe::Precision::FP32
                        : v == "bf16" ? CUDAPipe::Precision::BF16
                        : v == "fp16x2" ? CUDAPipe::Precision::FP16_X2 : CUDAPipe::Precision::FP16;
        } else if (k == "--batching") {
            eager = (v == "eager");
        } else {
            std::fprintf(stderr, "unknown option %s\n", k.c_str());
            return 2;
        }
    }
    std::mt19937 rng(1);
    auto w = std::make_shared<ForwardPipe::ForwardPipeWeights>();
    for (int l = 0; l < 1 + 2 * blocks; l++) {
        const int cin = l == 0 ? 18 : filters;
        std::normal_distribution<float> dist(0.0f, 0.5f / std::sqrt(9.0f * cin));
        std::vector<float> U(static_cast<size_t>(36) * cin * filters);
        for (auto& u : U) u = dist(rng);
        w->m_conv_weights.push_back(std::move(U));
        w->m_conv_biases.emplace_back(filters, 0.0f);
        w->m_batchnorm_means.emplace_back(filters, 0.0f);
        w->m_batchnorm_stddevs.emplace_back(filters, 1.0f);
    }
    std::normal_distribution<float> hd(0.0f, 0.05f);
    w->m_conv_pol_w.resize(2 * filters);
    w->m_conv_val_w.resize(filters);
    for (auto& v : w->m_conv_pol_w) v = hd(rng);
    for (auto& v : w->m_conv_val_w) v = hd(rng);
    w->m_conv_pol_b.assign(2, 0.0f);
    w->m_conv_val_b.assign(1, 0.0f);

    std::vector<int> ids;
    for (int g = 0; g < gpus; g++) ids.push_back(g);
    try {
        CUDAPipe pipe(ids, batch, threads, precision);
        if (eager) pipe.set_batching(CUDAPipe::Batching::EAGER);
        pipe.initialize(filters);
        pipe.push_weights(6, 18, filters, w);
        std::atomic<int> runcount{0};
        auto body = [&](int t, int limit) {
            std::vector<float> in(CUDAPipe::kInputFloats, 0.0f), pol(CUDAPipe::kPolicyFloats),
                val(CUDAPipe::kValueFloats);
            std::mt19937 r(100 + t);
            for (auto& x : in) x = (r() % 10) < 3 ? 1.0f : 0.0f;
            while (runcount < limit) {
                runcount++;
                pipe.forward(in, pol, val);
            }
        };
        auto run = [&](int limit) {
            runcount = 0;
            std::vector<std::thread> ts;
            for (int t = 0; t < threads; t++) ts.emplace_back(body, t, limit);
            for (auto& t : ts) t.join();
        };
        run(threads * 4);   // warm-up
        const auto t0 = std::chrono::steady_clock::now();
        run(iterations);
        const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        const auto s = pipe.stats();
        std::printf("%5d evaluations in %5.2f seconds -> %d n/s\n", runcount.load(), sec,
                    static_cast<int>(runcount.load() / sec));
        std::printf("{\"evals_per_s\": %.1f, \"blocks\": %d, \"filters\": %d, \"threads\": %d, "
                    "\"batch\": %d, \"batching\": \"%s\", \"gpus\": %d, \"batches\": %zu, \"mean_batch\": %.2f, "
                    "\"full_batches\": %zu, \"timeouts\": %zu, \"wait_ms\": %d}\n",
                    runcount.load() / sec, blocks, filters, threads, batch, eager ? "eager" : "wait", gpus, s.batches,
                    s.batches ? double(s.positions) / s.batches : 0.0, s.full_batches, s.timeouts,
                    s.wait_ms);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "netbench: %s\n", e.what());
        return 1;
    }
    return 0;
}
