// CUDAPipe implementation: request queue, batch forming, per-GPU workers,
// drain/resume.  See CUDAPipe.h for the contract and the reference lines.
#include "CUDAPipe.h"

#include <algorithm>
#include <chrono>
#include <cstring>
#include <stdexcept>

#include "lzb200.h"

namespace {

// Production backend: one lzb_pipe per GPU, one lzb_ctx per worker slot.
class LzbBackend : public CUDAPipe::Backend {
public:
    ~LzbBackend() override {
        for (auto& per_gpu : m_ctx)
            for (auto* c : per_gpu) lzb_ctx_destroy(c);
        for (auto* p : m_pipes) lzb_pipe_destroy(p);
    }

    void load(const std::vector<int>& gpus, int channels, int blocks, int max_batch,
              int workers_per_gpu, CUDAPipe::Precision precision,
              const ForwardPipe::ForwardPipeWeights& w) override {
        for (int gpu : gpus) {
            lzb_pipe* p = nullptr;
            check(lzb_pipe_create(&p, gpu, channels, blocks, static_cast<int>(precision)));
            m_pipes.push_back(p);
            for (size_t l = 0; l < w.m_conv_weights.size(); l++) {
                const int c_in = l == 0 ? LZB_INPUT_PLANES : channels;
                check(lzb_pipe_push_conv(p, static_cast<int>(l), w.m_conv_weights[l].data(), c_in,
                                         w.m_batchnorm_means[l].data(),
                                         w.m_batchnorm_stddevs[l].data()));
            }
            check(lzb_pipe_push_head_convs(p, w.m_conv_pol_w.data(), w.m_conv_val_w.data()));
            check(lzb_pipe_finalize(p));
            m_ctx.emplace_back();
            for (int s = 0; s < workers_per_gpu; s++) {
                lzb_ctx* c = nullptr;
                check(lzb_ctx_create(&c, p, max_batch));
                m_ctx.back().push_back(c);
            }
        }
    }

    int forward(int gpu_index, int worker, const float* in, int n, float* pol, float* val,
                std::string* error) override {
        const int rc = lzb_ctx_forward(m_ctx[gpu_index][worker], in, n, pol, val);
        if (rc != LZB_OK && error) *error = lzb_last_error();
        return rc;
    }

    bool takes_bit_planes() const override { return true; }
    int forward_bit_planes(int gpu_index, int worker, const unsigned int* planes, int n, float* pol,
                           float* val, std::string* error) override {
        const int rc = lzb_ctx_forward_packed(m_ctx[gpu_index][worker], planes, n, pol, val);
        if (rc != LZB_OK && error) *error = lzb_last_error();
        return rc;
    }

    float* alloc_staging(std::size_t floats) override {
        void* p = nullptr;
        check(lzb_host_alloc(&p, floats * sizeof(float)));
        return static_cast<float*>(p);
    }
    void free_staging(float* p) override { lzb_host_free(p); }

private:
    static void check(int rc) {
        // Initialisation failures surface as std::runtime_error, as in the
        // reference (src/OpenCL.cpp:809, 823, 871, 905).
        if (rc != LZB_OK) throw std::runtime_error(std::string("CUDAPipe: ") + lzb_last_error());
    }
    std::vector<lzb_pipe*> m_pipes;
    std::vector<std::vector<lzb_ctx*>> m_ctx;
};

}  // namespace

CUDAPipe::CUDAPipe(std::vector<int> gpus, int batch_size, int num_threads, Precision precision)
    : CUDAPipe(std::move(gpus), batch_size, num_threads, precision,
               std::unique_ptr<Backend>(new LzbBackend)) {}

CUDAPipe::CUDAPipe(std::vector<int> gpus, int batch_size, int num_threads, Precision precision,
                   std::unique_ptr<Backend> backend)
    : m_gpus(std::move(gpus)),
      m_batch_size(std::max(1, batch_size)),
      m_num_threads(std::max(1, num_threads)),
      m_precision(precision),
      m_backend(backend ? std::move(backend) : std::unique_ptr<Backend>(new LzbBackend)) {
    // An empty list means "pick one" in the engine (src/OpenCLScheduler.cpp:90-94).
    if (m_gpus.empty()) m_gpus.push_back(0);
}

CUDAPipe::~CUDAPipe() {
    {
        std::lock_guard<std::mutex> lk(m_mutex);
        m_running = false;
    }
    m_cv.notify_all();
    for (auto& t : m_threads) t.join();
    // Anyone still queued is released rather than left asleep.
    std::deque<Entry*> left;
    {
        std::lock_guard<std::mutex> lk(m_mutex);
        left.swap(m_queue);
        m_queued = 0;
    }
    for (auto* e : left) finish(e, true, "");
}

void CUDAPipe::initialize(int channels) {
    // The tower depth is only known when the weights arrive, so the device
    // side is built in push_weights; the call order is fixed by
    // Network::init_net (src/Network.cpp:407-414).
    m_channels = channels;
}

void CUDAPipe::push_weights(unsigned int /*filter_size*/, unsigned int /*channels*/,
                            unsigned int outputs,
                            std::shared_ptr<const ForwardPipeWeights> weights) {
    if (!weights || weights->m_conv_weights.empty() || weights->m_conv_weights.size() % 2 == 0) {
        throw std::runtime_error("CUDAPipe: malformed weights (expected 1 + 2*blocks layers)");
    }
    if (m_channels == 0) m_channels = static_cast<int>(outputs);
    if (static_cast<int>(outputs) != m_channels) {
        throw std::runtime_error("CUDAPipe: push_weights does not match initialize(channels)");
    }
    if (!m_threads.empty()) throw std::runtime_error("CUDAPipe: weights pushed twice");
    const int blocks = static_cast<int>(weights->m_conv_weights.size() - 1) / 2;
    // Same sizing rule as the reference: at least one worker per GPU, more when
    // many search threads share few GPUs (src/OpenCLScheduler.cpp:113-114).
    m_workers_per_gpu = m_num_threads / m_batch_size / (static_cast<int>(m_gpus.size()) + 1) + 1;
    // EAGER keeps two batches per GPU in flight (one computing, one being staged)
    if (m_batching == Batching::EAGER && m_workers_per_gpu < 2) m_workers_per_gpu = 2;
    m_backend->load(m_gpus, m_channels, blocks, m_batch_size, m_workers_per_gpu, m_precision,
                    *weights);
    m_bit_planes = m_backend->takes_bit_planes();
    m_live_gpus = static_cast<int>(m_gpus.size());
    m_gpu_failed.assign(m_gpus.size(), 0);
    m_in_flight.assign(m_gpus.size(), 0);
    for (size_t g = 0; g < m_gpus.size(); g++) {
        for (int s = 0; s < m_workers_per_gpu; s++) {
            m_threads.emplace_back(&CUDAPipe::worker, this, static_cast<int>(g), s);
        }
    }
}

// The last thing a worker does with an entry.  The notification happens under
// the entry's mutex: the caller cannot leave its wait (and let the entry, which
// lives on its stack, go out of scope) before this function has released it.
void CUDAPipe::finish(Entry* e, bool halted, const std::string& error) {
    std::lock_guard<std::mutex> lk(e->mutex);
    e->halted = halted;
    e->error = error;
    e->done = true;
    e->cv.notify_all();
}

void CUDAPipe::submit_and_wait(Entry* const* entries, int n_entries) {
    {
        std::lock_guard<std::mutex> lk(m_mutex);
        if (m_draining) {
            m_stats.halted++;
            throw NetworkHaltException();
        }
        if (m_live_gpus.load() == 0) throw std::runtime_error("CUDAPipe: no GPU left in service");
        for (int i = 0; i < n_entries; i++) {
            m_queue.push_back(entries[i]);
            m_queued += static_cast<size_t>(entries[i]->count);
        }
        // Requests arriving while a partial batch is in flight mean the wait
        // was too short (src/OpenCLScheduler.cpp:267-269).
        if (m_partial_in_progress.load() && m_wait_ms < kMaxWaitMs) m_wait_ms += 2;
    }
    // EAGER waiters have different wake conditions (room on their own GPU, the
    // gathering window, a full batch), so one wake-up could land on a worker
    // that goes back to sleep while an idle GPU's worker sleeps on.
    if (m_batching == Batching::EAGER || n_entries > 1) m_cv.notify_all();
    else m_cv.notify_one();
    // Every entry is waited for before anything is thrown: the entries are the
    // caller's, and a worker may still hold a pointer to one that is not done.
    bool halted = false;
    std::string error;
    for (int i = 0; i < n_entries; i++) {
        Entry& e = *entries[i];
        std::unique_lock<std::mutex> lk(e.mutex);
        e.cv.wait(lk, [&] { return e.done; });
        halted = halted || e.halted;
        if (error.empty()) error = e.error;
    }
    if (halted) throw NetworkHaltException();
    if (!error.empty()) throw std::runtime_error("CUDAPipe: " + error);
}

namespace {
// Writes the 18 planes of one position as bits; false if a value is neither 0
// nor 1 (then the batch travels as fp32).
bool pack_position(const float* in, unsigned int* words) {
    bool binary = true;
    for (int plane = 0; plane < 18; plane++) {
        const float* p = in + plane * 361;
        for (int w = 0; w < CUDAPipe::kPlaneWords; w++) {
            const int cells = w == CUDAPipe::kPlaneWords - 1 ? 361 - 32 * w : 32;
            unsigned int bits = 0, odd = 0;
            for (int i = 0; i < cells; i++) {
                const float v = p[32 * w + i];
                bits |= static_cast<unsigned int>(v != 0.0f) << i;
                odd |= static_cast<unsigned int>((v != 0.0f) & (v != 1.0f));
            }
            binary &= odd == 0;
            words[plane * CUDAPipe::kPlaneWords + w] = bits;
        }
    }
    return binary;
}
}  // namespace

void CUDAPipe::forward(const std::vector<float>& input, std::vector<float>& output_pol,
                       std::vector<float>& output_val) {
    if (input.size() != static_cast<size_t>(kInputFloats) ||
        output_pol.size() != static_cast<size_t>(kPolicyFloats) ||
        output_val.size() != static_cast<size_t>(kValueFloats)) {
        throw std::runtime_error("CUDAPipe::forward: wrong buffer sizes");
    }
    Entry entry(input.data(), 1, output_pol.data(), output_val.data());
    unsigned int words[kPackedWords];
    if (m_bit_planes && pack_position(input.data(), words)) entry.bits = words;
    Entry* one = &entry;
    submit_and_wait(&one, 1);
}

void CUDAPipe::forward_many(const float* in, int n, float* pol, float* val) {
    if (!in || !pol || !val || n < 1) throw std::runtime_error("CUDAPipe::forward_many: bad arguments");
    // Pieces of at most one batch; a piece is never split over two batches.
    const int pieces = (n + m_batch_size - 1) / m_batch_size;
    // The planes are packed into bits here, on the caller's thread, so that the
    // workers, which are few, only move bytes.
    std::vector<unsigned int> words;
    bool binary = m_bit_planes;
    if (binary) {
        words.resize(static_cast<size_t>(n) * kPackedWords);
        for (int i = 0; i < n && binary; i++) {
            binary = pack_position(in + static_cast<size_t>(i) * kInputFloats,
                                   words.data() + static_cast<size_t>(i) * kPackedWords);
        }
    }
    std::deque<Entry> entries;    // Entry is neither copyable nor movable
    for (int i = 0; i < pieces; i++) {
        const int first = i * m_batch_size;
        const int count = std::min(m_batch_size, n - first);
        entries.emplace_back(in + static_cast<size_t>(first) * kInputFloats, count,
                             pol + static_cast<size_t>(first) * kPolicyFloats,
                             val + static_cast<size_t>(first) * kValueFloats);
        if (binary) entries.back().bits = words.data() + static_cast<size_t>(first) * kPackedWords;
    }
    std::vector<Entry*> order;
    for (auto& e : entries) order.push_back(&e);
    submit_and_wait(order.data(), pieces);
}

// Removes entries from the front of the queue until `positions` positions are
// taken or the next entry would not fit any more.  m_mutex is held.
std::vector<CUDAPipe::Entry*> CUDAPipe::take(std::size_t positions) {
    std::vector<Entry*> batch;
    std::size_t taken = 0;
    while (!m_queue.empty() && taken + static_cast<size_t>(m_queue.front()->count) <= positions) {
        taken += static_cast<size_t>(m_queue.front()->count);
        batch.push_back(m_queue.front());
        m_queue.pop_front();
    }
    m_queued -= taken;
    return batch;
}

// Batch-forming heuristic of the reference (src/OpenCLScheduler.cpp:293-353):
// wait up to m_wait_ms for a full batch; if it does not fill and no other
// partial batch is in flight, send what is there and wait 1 ms less next time.
//
// Batching::EAGER instead: take what is waiting as soon as there is room for
// another batch on the worker's GPU (two per GPU), after a gathering window in which the
// callers released together by the previous batch come back.
std::vector<CUDAPipe::Entry*> CUDAPipe::pickup(bool* timed_out, int gpu_index) {
    std::vector<Entry*> batch;
    *timed_out = false;
    std::unique_lock<std::mutex> lk(m_mutex);
    const size_t full = static_cast<size_t>(m_batch_size);
    while (m_batching == Batching::EAGER) {
        m_cv.wait(lk, [&] {
            return !m_running || m_gpu_failed[gpu_index] ||
                   (m_queued > 0 && !m_gathering && (m_queued >= full || m_in_flight[gpu_index] < 2));
        });
        if (!m_running || m_gpu_failed[gpu_index]) return batch;
        // A lone caller (one request now, one in the previous batch) gains
        // nothing from the window; everybody else does.
        if (m_queued < full && m_gather_us > 0 && (m_queued > 1 || m_last_batch > 1)) {
            m_gathering = true;
            m_cv.wait_for(lk, std::chrono::microseconds(m_gather_us),
                          [&] { return !m_running || m_queued >= full; });
            m_gathering = false;
            if (!m_running || m_gpu_failed[gpu_index]) {
                lk.unlock();
                m_cv.notify_all();         // the window is closed: somebody else gathers
                return batch;
            }
        }
        batch = take(full);
        if (batch.empty()) continue;       // drained while gathering
        size_t count = 0;
        for (auto* e : batch) count += static_cast<size_t>(e->count);
        *timed_out = count < full && m_queued == 0;
        m_last_batch = count;
        m_in_flight[gpu_index]++;
        lk.unlock();
        m_cv.notify_all();                 // others may take what is left
        return batch;
    }
    while (true) {
        if (!m_running || m_gpu_failed[gpu_index]) return batch;
        if (m_queued >= full) break;
        const bool filled = m_cv.wait_for(lk, std::chrono::milliseconds(m_wait_ms), [&] {
            return !m_running || m_gpu_failed[gpu_index] || m_queued >= full;
        });
        if (!m_running || m_gpu_failed[gpu_index]) return batch;
        if (!filled && m_queued > 0 && !m_partial_in_progress.exchange(true)) {
            if (m_wait_ms > 1) m_wait_ms--;
            *timed_out = true;
            break;
        }
    }
    return take(full);
}

// Takes a GPU out of rotation: its workers leave at their next look at the
// queue (pickup wakes on the flag), and when it was the last GPU everybody
// still queued is released with an error.
void CUDAPipe::retire_gpu(int gpu_index, const std::string& error) {
    std::deque<Entry*> orphans;
    {
        std::lock_guard<std::mutex> lk(m_mutex);
        if (!m_gpu_failed[gpu_index]) {
            m_gpu_failed[gpu_index] = 1;
            if (--m_live_gpus <= 0) {
                m_live_gpus = 0;
                orphans.swap(m_queue);
                m_queued = 0;
            }
        }
    }
    m_cv.notify_all();
    for (auto* e : orphans) finish(e, false, "no GPU left in service (" + error + ")");
}

void CUDAPipe::worker(int gpu_index, int slot) {
    // Nothing may leave a thread body as an exception (that would end the
    // process): a worker that cannot get its staging memory retires its GPU.
    try {
        serve(gpu_index, slot);
    } catch (const std::exception& e) {
        retire_gpu(gpu_index, e.what());
    } catch (...) {
        retire_gpu(gpu_index, "unknown exception in a worker");
    }
}

void CUDAPipe::serve(int gpu_index, int slot) {
    // Staging buffers of this worker, released when it leaves.
    struct Staging {
        Backend* b;
        float* p;
        Staging(Backend* backend, size_t n) : b(backend), p(n ? backend->alloc_staging(n) : nullptr) {}
        ~Staging() { if (p) b->free_staging(p); }
        float* data() { return p; }
        float& operator[](size_t i) { return p[i]; }
    };
    const bool bit_planes = m_bit_planes;
    Staging in(m_backend.get(), static_cast<size_t>(m_batch_size) * kInputFloats);
    Staging bits(m_backend.get(), bit_planes ? static_cast<size_t>(m_batch_size) * kPackedWords : 0);
    Staging pol(m_backend.get(), static_cast<size_t>(m_batch_size) * kPolicyFloats);
    Staging val(m_backend.get(), static_cast<size_t>(m_batch_size) * kValueFloats);
    unsigned int* words = reinterpret_cast<unsigned int*>(bits.data());
    while (true) {
        bool timed_out = false;
        auto batch = pickup(&timed_out, gpu_index);
        if (batch.empty()) return;   // shutting down, or a sibling worker saw this GPU fail
        int n = 0;
        bool binary = bit_planes;
        for (auto* e : batch) {
            binary = binary && e->bits != nullptr;
            n += e->count;
        }
        int at = 0;
        for (auto* e : batch) {
            if (binary) {
                std::memcpy(words + static_cast<size_t>(at) * kPackedWords, e->bits,
                            sizeof(unsigned int) * kPackedWords * static_cast<size_t>(e->count));
            } else {
                std::memcpy(&in[static_cast<size_t>(at) * kInputFloats], e->in,
                            sizeof(float) * kInputFloats * static_cast<size_t>(e->count));
            }
            at += e->count;
        }
        std::string error;
        int rc;
        try {
            rc = binary ? m_backend->forward_bit_planes(gpu_index, slot, words, n, pol.data(), val.data(), &error)
                        : m_backend->forward(gpu_index, slot, in.data(), n, pol.data(), val.data(), &error);
        } catch (const std::exception& e) {
            rc = -1;
            error = e.what();
        }
        if (rc == 0) {
            int at = 0;
            for (auto* e : batch) {
                std::memcpy(e->out_p, &pol[static_cast<size_t>(at) * kPolicyFloats],
                            sizeof(float) * kPolicyFloats * static_cast<size_t>(e->count));
                std::memcpy(e->out_v, &val[static_cast<size_t>(at) * kValueFloats],
                            sizeof(float) * kValueFloats * static_cast<size_t>(e->count));
                at += e->count;
            }
        } else if (error.empty()) {
            error = "backend error " + std::to_string(rc);
        }
        {
            std::lock_guard<std::mutex> lk(m_mutex);
            m_stats.batches++;
            m_stats.positions += static_cast<size_t>(n);
            if (n == m_batch_size) m_stats.full_batches++;
            if (timed_out) m_stats.timeouts++;
            if (binary) m_stats.bit_plane_batches++;
            if (m_batching == Batching::EAGER) m_in_flight[gpu_index]--;
        }
        for (auto* e : batch) finish(e, false, rc == 0 ? std::string() : error);
        if (m_batching == Batching::EAGER) m_cv.notify_all();   // room for another batch
        else if (timed_out) m_partial_in_progress = false;
        if (rc != 0) {
            retire_gpu(gpu_index, error);
            return;
        }
    }
}

void CUDAPipe::set_batching(Batching mode, int gather_us) {
    std::lock_guard<std::mutex> lk(m_mutex);
    if (!m_threads.empty()) throw std::runtime_error("CUDAPipe: set_batching after push_weights");
    m_batching = mode;
    m_gather_us = gather_us < 0 ? 0 : gather_us;
}

void CUDAPipe::drain() {
    // Wake every queued caller; each throws NetworkHaltException out of
    // forward() (src/OpenCLScheduler.cpp:412-433).  Batches already on a GPU
    // complete normally.
    std::deque<Entry*> queued;
    {
        std::lock_guard<std::mutex> lk(m_mutex);
        m_draining = true;
        queued.swap(m_queue);
        m_queued = 0;
        m_stats.halted += queued.size();
    }
    for (auto* e : queued) finish(e, true, "");
}

void CUDAPipe::resume() {
    // Called after all search threads returned (src/OpenCLScheduler.cpp:436-441).
    std::lock_guard<std::mutex> lk(m_mutex);
    m_draining = false;
}

CUDAPipe::Stats CUDAPipe::stats() const {
    std::lock_guard<std::mutex> lk(m_mutex);
    Stats s = m_stats;
    s.wait_ms = m_wait_ms;
    return s;
}

int CUDAPipe::live_gpus() const { return m_live_gpus.load(); }
