// Host-side tests of CUDAPipe with a fake backend (no GPU): batch forming,
// adaptive wait, partial batches, drain/resume, error propagation, removal of a
// failing GPU.  Behaviour under test is that of src/OpenCLScheduler.cpp:257-441.
// Exit code 0 = all checks passed; each failure prints a line.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <functional>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>

#include "CUDAPipe.h"

static int g_failures = 0;
#define CHECK(cond)                                                      \
    do {                                                                 \
        if (!(cond)) {                                                   \
            std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond);  \
            g_failures++;                                                \
        }                                                                \
    } while (0)

using Weights = ForwardPipe::ForwardPipeWeights;

// pol[j] = in[j] * 2 + in[0], val[j] = in[j] + 3: lets every caller check that
// it got the answer to its own question.
class FakeBackend : public CUDAPipe::Backend {
public:
    std::atomic<int> calls{0};
    std::atomic<int> max_n{0};
    std::atomic<int> loaded_gpus{0};
    std::atomic<int> fail_gpu{-1};       // gpu index whose calls fail
    std::atomic<int> throw_gpu{-1};      // gpu index whose calls throw
    std::atomic<int> calls_on[4] = {{0}, {0}, {0}, {0}};
    std::atomic<bool> bit_planes{false};  // accept positions as bit planes
    std::atomic<int> bit_plane_calls{0};
    std::atomic<int> delay_ms{0};
    std::atomic<bool> gate_closed{false};  // while true, forward() blocks
    std::atomic<int> running[4] = {{0}, {0}, {0}, {0}};   // calls inside forward(), per gpu
    std::atomic<int> max_running{0};
    std::mutex m;
    std::multiset<int> batch_sizes;
    std::set<int> gpus_used;

    void load(const std::vector<int>& gpus, int channels, int blocks, int max_batch, int workers,
              CUDAPipe::Precision, const Weights& w) override {
        loaded_gpus = static_cast<int>(gpus.size());
        CHECK(channels == 8 && blocks == 1 && max_batch >= 1 && workers >= 1);
        CHECK(w.m_conv_weights.size() == 3);
    }
    int forward(int gpu, int, const float* in, int n, float* pol, float* val,
                std::string* error) override {
        calls++;
        struct Count {
            std::atomic<int>& c;
            explicit Count(std::atomic<int>& x, std::atomic<int>& mx) : c(x) {
                const int now = ++c;
                int prev = mx.load();
                while (now > prev && !mx.compare_exchange_weak(prev, now)) {}
            }
            ~Count() { --c; }
        } count(running[gpu & 3], max_running);
        while (gate_closed) std::this_thread::sleep_for(std::chrono::milliseconds(1));
        if (delay_ms > 0) std::this_thread::sleep_for(std::chrono::milliseconds(delay_ms));
        {
            std::lock_guard<std::mutex> lk(m);
            batch_sizes.insert(n);
            gpus_used.insert(gpu);
        }
        int prev = max_n.load();
        while (n > prev && !max_n.compare_exchange_weak(prev, n)) {}
        calls_on[gpu & 3]++;
        if (gpu == throw_gpu) throw std::runtime_error("injected exception");
        if (gpu == fail_gpu) {
            *error = "injected failure";
            return 2;
        }
        for (int i = 0; i < n; i++) {
            const float* x = in + (size_t)i * CUDAPipe::kInputFloats;
            for (int j = 0; j < CUDAPipe::kPolicyFloats; j++) pol[(size_t)i * CUDAPipe::kPolicyFloats + j] = x[j] * 2 + x[0];
            for (int j = 0; j < CUDAPipe::kValueFloats; j++) val[(size_t)i * CUDAPipe::kValueFloats + j] = x[j] + 3;
        }
        return 0;
    }
    bool takes_bit_planes() const override { return bit_planes; }
    int forward_bit_planes(int gpu, int worker, const unsigned int* planes, int n, float* pol, float* val,
                           std::string* error) override {
        bit_plane_calls++;
        std::vector<float> x((size_t)n * CUDAPipe::kInputFloats);
        for (int i = 0; i < n; i++)
            for (int p = 0; p < 18; p++)
                for (int c = 0; c < 361; c++)
                    x[(size_t)i * CUDAPipe::kInputFloats + p * 361 + c] =
                        (planes[(size_t)i * CUDAPipe::kPackedWords + p * 12 + c / 32] >> (c % 32)) & 1u ? 1.0f : 0.0f;
        return forward(gpu, worker, x.data(), n, pol, val, error);
    }
};

static std::shared_ptr<const Weights> tiny_weights() {
    auto w = std::make_shared<Weights>();
    w->m_conv_weights = {std::vector<float>(36 * 18 * 8), std::vector<float>(36 * 8 * 8), std::vector<float>(36 * 8 * 8)};
    w->m_batchnorm_means.assign(3, std::vector<float>(8));
    w->m_batchnorm_stddevs.assign(3, std::vector<float>(8, 1.0f));
    w->m_conv_biases.assign(3, std::vector<float>(8));
    w->m_conv_pol_w.assign(16, 0.f);
    w->m_conv_val_w.assign(8, 0.f);
    return w;
}

struct Caller {
    std::vector<float> in, pol, val;
    explicit Caller(float tag) : in(CUDAPipe::kInputFloats), pol(CUDAPipe::kPolicyFloats), val(CUDAPipe::kValueFloats) {
        for (size_t j = 0; j < in.size(); j++) in[j] = tag + 0.001f * (j % 97);
    }
    bool answer_is_mine() const {
        for (int j = 0; j < CUDAPipe::kPolicyFloats; j++)
            if (pol[j] != in[j] * 2 + in[0]) return false;
        for (int j = 0; j < CUDAPipe::kValueFloats; j++)
            if (val[j] != in[j] + 3) return false;
        return true;
    }
};

static std::unique_ptr<CUDAPipe> make_pipe(FakeBackend** fb, std::vector<int> gpus, int batch, int threads,
                                           bool eager = false) {
    auto backend = std::unique_ptr<FakeBackend>(new FakeBackend);
    *fb = backend.get();
    std::unique_ptr<CUDAPipe> pipe(new CUDAPipe(std::move(gpus), batch, threads, CUDAPipe::Precision::FP16, std::move(backend)));
    if (eager) pipe->set_batching(CUDAPipe::Batching::EAGER, 100);
    pipe->initialize(8);
    pipe->push_weights(6, 18, 8, tiny_weights());
    return pipe;
}

static void test_many_callers_two_gpus() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0, 1}, 8, 32);
    CHECK(fb->loaded_gpus == 2 && pipe->live_gpus() == 2);
    fb->delay_ms = 1;
    std::atomic<int> good{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < 32; t++) {
        ts.emplace_back([&, t] {
            for (int r = 0; r < 20; r++) {
                Caller c(t * 100.0f + r);
                pipe->forward(c.in, c.pol, c.val);
                if (c.answer_is_mine()) good++;
            }
        });
    }
    for (auto& t : ts) t.join();
    CHECK(good == 32 * 20);                       // nothing lost, duplicated or crossed
    auto s = pipe->stats();
    CHECK(s.positions == 32 * 20);
    CHECK(fb->max_n <= 8 && fb->max_n >= 2);      // batches formed, never above batch_size
    CHECK(s.batches < 32 * 20);
    CHECK(fb->gpus_used.size() == 2);             // both replicas served
    std::printf("many callers: %zu batches for %zu positions, %zu full, %zu on timeout, wait %d ms\n",
                s.batches, s.positions, s.full_batches, s.timeouts, s.wait_ms);
}

static void test_single_caller_does_not_deadlock() {
    // Fewer callers than batch_size can never fill a batch: the wait must run
    // out and the partial batch must go (src/OpenCLScheduler.cpp:293-345).
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0}, 8, 2);
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < 5; r++) {
        Caller c(r);
        pipe->forward(c.in, c.pol, c.val);
        CHECK(c.answer_is_mine());
    }
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    auto s = pipe->stats();
    CHECK(s.timeouts == 5 && s.full_batches == 0);
    CHECK(s.wait_ms < 10);                        // shortened after every timeout
    CHECK(sec < 2.0);
}

static void test_partial_batch_takes_all_waiting() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0}, 16, 4);
    std::vector<std::thread> ts;
    std::atomic<int> good{0};
    for (int t = 0; t < 5; t++) {
        ts.emplace_back([&, t] {
            Caller c(t);
            pipe->forward(c.in, c.pol, c.val);
            if (c.answer_is_mine()) good++;
        });
    }
    for (auto& t : ts) t.join();
    CHECK(good == 5);
    CHECK(pipe->stats().batches <= 3);            // not five single evaluations
}

static void test_drain_and_resume() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0}, 4, 8);
    fb->gate_closed = true;                       // the first batch sticks in the backend
    std::atomic<int> halted{0}, answered{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < 12; t++) {
        ts.emplace_back([&, t] {
            Caller c(t);
            try {
                pipe->forward(c.in, c.pol, c.val);
                if (c.answer_is_mine()) answered++;
            } catch (const NetworkHaltException&) {
                halted++;
            }
        });
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    pipe->drain();                                // queued callers must wake and throw
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
    CHECK(halted >= 4);                           // at least those still queued
    {   // while draining, new requests are refused the same way
        Caller c(99);
        bool threw = false;
        try { pipe->forward(c.in, c.pol, c.val); } catch (const NetworkHaltException&) { threw = true; }
        CHECK(threw);
    }
    fb->gate_closed = false;                      // batches already on the device finish normally
    for (auto& t : ts) t.join();
    CHECK(halted + answered == 12 && answered >= 1);
    pipe->resume();
    Caller c(7);
    pipe->forward(c.in, c.pol, c.val);
    CHECK(c.answer_is_mine());
}

static void test_failing_gpu_is_removed() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0, 1}, 2, 4);
    fb->fail_gpu = 1;
    int errors = 0, ok = 0;
    for (int r = 0; r < 40; r++) {
        Caller c(r);
        try {
            pipe->forward(c.in, c.pol, c.val);
            if (c.answer_is_mine()) ok++;
        } catch (const std::runtime_error& e) {
            errors++;
            CHECK(std::string(e.what()).find("injected failure") != std::string::npos);
        }
    }
    CHECK(errors >= 1 && errors <= 2);            // only the batch(es) that hit the bad GPU
    CHECK(ok == 40 - errors);
    CHECK(pipe->live_gpus() == 1);                // the other replica keeps serving
    fb->fail_gpu = 0;                             // now the last one fails too
    int late_errors = 0;
    for (int r = 0; r < 3; r++) {
        Caller c(r);
        try { pipe->forward(c.in, c.pol, c.val); } catch (const std::runtime_error&) { late_errors++; }
    }
    CHECK(late_errors == 3 && pipe->live_gpus() == 0);
}

static void test_bad_arguments() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {}, 4, 4);         // empty GPU list = device 0
    CHECK(fb->loaded_gpus == 1);
    std::vector<float> in(10), pol(CUDAPipe::kPolicyFloats), val(CUDAPipe::kValueFloats);
    bool threw = false;
    try { pipe->forward(in, pol, val); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);
    threw = false;
    try { pipe->push_weights(6, 18, 8, tiny_weights()); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);                                 // weights pushed twice
    CHECK(!pipe->needs_autodetect());
}

static void test_destructor_releases_waiters() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0}, 64, 2);
    fb->gate_closed = true;
    std::atomic<int> released{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < 3; t++) {
        ts.emplace_back([&, t] {
            Caller c(t);
            try { pipe->forward(c.in, c.pol, c.val); released++; }
            catch (const NetworkHaltException&) { released++; }
        });
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(60));
    fb->gate_closed = false;
    for (auto& t : ts) t.join();
    pipe.reset();
    CHECK(released == 3);
}

// Batching::EAGER: as many callers as a batch holds, so full batches hardly
// ever form by themselves.  Batches must go as soon as the GPU has room, grow
// while it is busy, stay within batch_size and within two calls per GPU.
static void test_eager_batches_follow_the_load() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0, 1}, 64, 64, true);
    fb->delay_ms = 2;
    std::atomic<int> good{0};
    std::vector<std::thread> ts;
    const auto t0 = std::chrono::steady_clock::now();
    for (int t = 0; t < 64; t++) {
        ts.emplace_back([&, t] {
            for (int r = 0; r < 25; r++) {
                Caller c(t * 100.0f + r);
                pipe->forward(c.in, c.pol, c.val);
                if (c.answer_is_mine()) good++;
            }
        });
    }
    for (auto& t : ts) t.join();
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    auto s = pipe->stats();
    CHECK(good == 64 * 25 && s.positions == 64 * 25);
    CHECK(fb->max_n <= 64);
    CHECK(fb->max_running <= 2);                              // per GPU: one computing, one staged
    CHECK(double(s.positions) / s.batches >= 4.0);            // requests gathered while the GPUs were busy
    CHECK(sec < 1.5);                                         // 25 rounds of 2 ms calls, not 25 waits of 10 ms
    CHECK(fb->gpus_used.size() == 2);
    std::printf("eager: %zu batches for %zu positions (mean %.1f), %.3f s\n", s.batches, s.positions,
                double(s.positions) / s.batches, sec);
}

static void test_eager_single_caller_is_served_at_once() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0}, 16, 16, true);
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < 20; r++) {
        Caller c(r);
        pipe->forward(c.in, c.pol, c.val);
        CHECK(c.answer_is_mine());
    }
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    CHECK(pipe->stats().batches == 20);
    CHECK(sec < 0.15);                                        // twenty 10 ms waits would take 0.2 s; a lone caller also skips the window
}

static void test_eager_drain_failure_and_shutdown() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0, 1}, 4, 8, true);
    fb->gate_closed = true;
    std::atomic<int> halted{0}, answered{0}, failed{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < 24; t++) {
        ts.emplace_back([&, t] {
            Caller c(t);
            try {
                pipe->forward(c.in, c.pol, c.val);
                if (c.answer_is_mine()) answered++;
            } catch (const NetworkHaltException&) {
                halted++;
            }
        });
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    pipe->drain();                                // 2 GPUs x 2 calls x 4 positions are in the backend, 8 wait
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
    CHECK(halted >= 8);
    fb->gate_closed = false;
    for (auto& t : ts) t.join();
    CHECK(halted + answered == 24 && answered >= 4);
    pipe->resume();
    fb->fail_gpu = 1;
    for (int r = 0; r < 30; r++) {
        Caller c(r);
        try { pipe->forward(c.in, c.pol, c.val); CHECK(c.answer_is_mine()); }
        catch (const std::runtime_error&) { failed++; }
    }
    if (!(failed <= 2 && pipe->live_gpus() == (failed ? 1 : 2))) std::printf("failed %d live %d\n", failed.load(), pipe->live_gpus());
    CHECK(failed <= 2 && pipe->live_gpus() == (failed ? 1 : 2));   // GPU 1 may never have been picked
    bool threw = false;
    try { pipe->set_batching(CUDAPipe::Batching::REFERENCE_WAIT); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);                                 // the rule is fixed once the workers run
    pipe.reset();                                 // workers idle in the eager wait must leave
}

// Blocks of positions from several threads: every position gets its own
// answer, blocks larger than a batch are cut, none is split inside a batch.
static void test_forward_many() {
    for (int eager = 0; eager < 2; eager++) {
        FakeBackend* fb;
        auto pipe = make_pipe(&fb, {0, 1}, 8, 16, eager != 0);
        std::atomic<int> bad{0};
        std::vector<std::thread> ts;
        for (int t = 0; t < 6; t++) {
            ts.emplace_back([&, t] {
                const int sizes[] = {5, 8, 20, 1, 3};
                for (int r = 0; r < 10; r++) {
                    const int n = sizes[(t + r) % 5];
                    std::vector<float> in((size_t)n * CUDAPipe::kInputFloats), pol((size_t)n * CUDAPipe::kPolicyFloats),
                        val((size_t)n * CUDAPipe::kValueFloats);
                    for (int i = 0; i < n; i++)
                        for (int j = 0; j < CUDAPipe::kInputFloats; j++)
                            in[(size_t)i * CUDAPipe::kInputFloats + j] = 100.f * t + 10.f * r + i + 0.001f * (j % 97);
                    pipe->forward_many(in.data(), n, pol.data(), val.data());
                    for (int i = 0; i < n; i++) {
                        const float* x = &in[(size_t)i * CUDAPipe::kInputFloats];
                        for (int j = 0; j < CUDAPipe::kPolicyFloats; j++)
                            if (pol[(size_t)i * CUDAPipe::kPolicyFloats + j] != x[j] * 2 + x[0]) bad++;
                        for (int j = 0; j < CUDAPipe::kValueFloats; j++)
                            if (val[(size_t)i * CUDAPipe::kValueFloats + j] != x[j] + 3) bad++;
                    }
                }
            });
        }
        for (auto& t : ts) t.join();
        CHECK(bad == 0);
        CHECK(fb->max_n <= 8);
        CHECK(pipe->stats().positions == 6u * 2u * (5 + 8 + 20 + 1 + 3));
        bool threw = false;
        std::vector<float> x(CUDAPipe::kInputFloats), p(CUDAPipe::kPolicyFloats), v(CUDAPipe::kValueFloats);
        try { pipe->forward_many(x.data(), 0, p.data(), v.data()); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
        pipe->drain();
        threw = false;
        try { pipe->forward_many(x.data(), 1, p.data(), v.data()); } catch (const NetworkHaltException&) { threw = true; }
        CHECK(threw);
        pipe->resume();
    }
}

// Zero/one planes travel as bits, anything else as fp32, with the same answers.
static void test_bit_planes() {
    auto backend = std::unique_ptr<FakeBackend>(new FakeBackend);
    FakeBackend* fb = backend.get();
    fb->bit_planes = true;
    CUDAPipe pipe({0}, 4, 4, CUDAPipe::Precision::FP16, std::move(backend));
    pipe.initialize(8);
    pipe.push_weights(6, 18, 8, tiny_weights());
    std::vector<float> in(3 * CUDAPipe::kInputFloats), pol(3 * CUDAPipe::kPolicyFloats), val(3 * CUDAPipe::kValueFloats);
    for (size_t j = 0; j < in.size(); j++) in[j] = ((j * 2654435761u) >> 7) % 3 == 0 ? 1.0f : 0.0f;
    pipe.forward_many(in.data(), 3, pol.data(), val.data());
    int bad = 0;
    for (int i = 0; i < 3; i++) {
        const float* x = &in[(size_t)i * CUDAPipe::kInputFloats];
        for (int j = 0; j < CUDAPipe::kPolicyFloats; j++) bad += pol[(size_t)i * CUDAPipe::kPolicyFloats + j] != x[j] * 2 + x[0];
        for (int j = 0; j < CUDAPipe::kValueFloats; j++) bad += val[(size_t)i * CUDAPipe::kValueFloats + j] != x[j] + 3;
    }
    CHECK(bad == 0 && fb->bit_plane_calls == 1 && pipe.stats().bit_plane_batches == 1);
    in[CUDAPipe::kInputFloats + 5] = 0.5f;            // not a stone plane any more
    pipe.forward_many(in.data(), 3, pol.data(), val.data());
    CHECK(fb->bit_plane_calls == 1 && pipe.stats().bit_plane_batches == 1);
    CHECK(pol[CUDAPipe::kPolicyFloats + 5] == 0.5f * 2 + in[CUDAPipe::kInputFloats]);
    Caller c(0.25f);                                  // Caller's inputs are not binary either
    pipe.forward(c.in, c.pol, c.val);
    CHECK(c.answer_is_mine() && fb->bit_plane_calls == 1);
}

static void test_failed_gpu_gets_no_further_batches() {
    // Two GPUs with two workers each.  After GPU 0 fails once, its second
    // worker, asleep in the queue wait at that moment, must leave without
    // taking a batch: one failing backend call, one failed caller.
    for (int eager = 0; eager < 2; eager++) {
        FakeBackend* fb;
        auto pipe = make_pipe(&fb, {0, 1}, 2, 8, eager != 0);
        fb->fail_gpu = 0;
        int errors = 0, ok = 0;
        for (int r = 0; r < 60; r++) {
            Caller c(r);
            try {
                pipe->forward(c.in, c.pol, c.val);
                if (c.answer_is_mine()) ok++;
            } catch (const std::runtime_error&) {
                errors++;
            }
        }
        CHECK(fb->calls_on[0] <= 1 && errors == fb->calls_on[0] && ok == 60 - errors);
        CHECK(pipe->live_gpus() == (errors ? 1 : 2));
    }
}

static void test_backend_exception_is_an_error_not_a_crash() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0, 1}, 2, 4);
    fb->throw_gpu = 1;
    int errors = 0, ok = 0;
    for (int r = 0; r < 40; r++) {
        Caller c(r);
        try {
            pipe->forward(c.in, c.pol, c.val);
            if (c.answer_is_mine()) ok++;
        } catch (const std::runtime_error& e) {
            errors++;
            CHECK(std::string(e.what()).find("injected exception") != std::string::npos);
        }
    }
    CHECK(errors <= 1 && ok == 40 - errors && pipe->live_gpus() == (errors ? 1 : 2));
}

static void test_halted_callers_are_counted() {
    FakeBackend* fb;
    auto pipe = make_pipe(&fb, {0}, 4, 8);
    fb->gate_closed = true;
    std::atomic<int> halted{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < 12; t++) {
        ts.emplace_back([&, t] {
            Caller c(t);
            try { pipe->forward(c.in, c.pol, c.val); } catch (const NetworkHaltException&) { halted++; }
        });
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    pipe->drain();
    fb->gate_closed = false;
    for (auto& t : ts) t.join();
    CHECK(halted >= 4 && pipe->stats().halted == static_cast<size_t>(halted.load()));
    pipe->resume();
}

int main() {
    test_forward_many();
    test_bit_planes();
    test_failed_gpu_gets_no_further_batches();
    test_backend_exception_is_an_error_not_a_crash();
    test_halted_callers_are_counted();
    test_many_callers_two_gpus();
    test_single_caller_does_not_deadlock();
    test_partial_batch_takes_all_waiting();
    test_drain_and_resume();
    test_failing_gpu_is_removed();
    test_bad_arguments();
    test_destructor_releases_waiters();
    test_eager_batches_follow_the_load();
    test_eager_single_caller_is_served_at_once();
    test_eager_drain_failure_and_shutdown();
    if (g_failures == 0) std::printf("ALL OK\n");
    return g_failures == 0 ? 0 : 1;
}
