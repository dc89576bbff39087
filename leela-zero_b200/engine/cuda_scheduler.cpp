// State shared between the OpenCLScheduler stand-in (cuda_scheduler.h) and
// engine_bench: which arithmetic the engine's two precisions map to, the batch
// forming rule, counters.
#include <cstring>
#include <mutex>

#include "cuda_scheduler.h"

batch_stats_t batch_stats;

namespace lzb_engine {
CUDAPipe::Precision single_mode = CUDAPipe::Precision::FP32;
CUDAPipe::Precision half_mode = CUDAPipe::Precision::FP16_X2;
bool eager = true;
int callers = 0;
int fail_half_init = 0;
CUDAPipe* last_pipe = nullptr;
std::unique_ptr<CUDAPipe::Backend> (*backend_factory)() = nullptr;
std::atomic<unsigned long long> evals{0};

namespace {
std::mutex g_mutex;
}

void note_pipe(CUDAPipe* pipe, bool alive) {
    std::lock_guard<std::mutex> lk(g_mutex);
    if (alive) last_pipe = pipe;
    else if (last_pipe == pipe) last_pipe = nullptr;
}

CUDAPipe::Precision precision_from_name(const char* name, bool* ok) {
    static const struct { const char* name; CUDAPipe::Precision p; } table[] = {
        {"fp32", CUDAPipe::Precision::FP32},
        {"fp16", CUDAPipe::Precision::FP16},
        {"bf16", CUDAPipe::Precision::BF16},
        {"fp16-winograd", CUDAPipe::Precision::FP16_WINOGRAD},
        {"bf16-winograd", CUDAPipe::Precision::BF16_WINOGRAD},
        {"fp16x2", CUDAPipe::Precision::FP16_X2},
        {"fp16x3", CUDAPipe::Precision::FP16_X3},
        {"bf16x3", CUDAPipe::Precision::BF16_X3},
    };
    for (const auto& row : table) {
        if (std::strcmp(row.name, name) == 0) {
            if (ok) *ok = true;
            return row.p;
        }
    }
    if (ok) *ok = false;
    return CUDAPipe::Precision::FP16_X2;
}
}  // namespace lzb_engine
