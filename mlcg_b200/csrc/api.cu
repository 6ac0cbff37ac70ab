// Library-level entry points: error text, version, last CUDA error.
#include "common.cuh"

#include <cstring>
#include <vector>

namespace mlcgb {
thread_local int g_last_cuda_error = 0;

namespace {
struct TimelineRecord {
    const char *name;
    cudaEvent_t start, stop;
};
struct TimelineTotal {
    const char *name;
    int64_t calls;
    double ms;
};
struct Timeline {
    bool on = false;
    int depth = 0;
    std::vector<TimelineRecord> records;
    std::vector<cudaEvent_t> spare;          // events of earlier recordings, reused
    std::vector<TimelineTotal> totals;
    cudaEvent_t take() {
        if (!spare.empty()) {
            cudaEvent_t e = spare.back();
            spare.pop_back();
            return e;
        }
        cudaEvent_t e = nullptr;
        cudaEventCreate(&e);
        return e;
    }
};
thread_local Timeline g_timeline;
}  // namespace

TimelineScope::TimelineScope(const char *name, void *stream) : slot(-1), st((cudaStream_t)stream) {
    Timeline &t = g_timeline;
    if (!t.on) return;
    if (t.depth++ > 0) return;
    TimelineRecord r{name, t.take(), t.take()};
    if (!r.start || !r.stop) return;
    cudaEventRecord(r.start, st);
    slot = (int)t.records.size();
    t.records.push_back(r);
}

TimelineScope::~TimelineScope() {
    Timeline &t = g_timeline;
    if (!t.on) return;
    --t.depth;
    if (slot >= 0) cudaEventRecord(t.records[slot].stop, st);
}
}  // namespace mlcgb

extern "C" {

const char *mlcgb_strerror(int code) {
    switch (code) {
        case MLCGB_OK: return "ok";
        case MLCGB_E_ARG: return "invalid argument (null pointer, negative size or unsupported option)";
        case MLCGB_E_WORKSPACE: return "workspace too small";
        case MLCGB_E_LAUNCH: return "CUDA launch failed";
        case MLCGB_E_LIMIT: return "size beyond the supported limit";
        default: return "unknown error code";
    }
}

int mlcgb_last_cuda_error(void) { return mlcgb::g_last_cuda_error; }

int mlcgb_version(void) { return 101; }

int mlcgb_timeline_begin(void) {
    mlcgb::Timeline &t = mlcgb::g_timeline;
    for (auto &r : t.records) {
        t.spare.push_back(r.start);
        t.spare.push_back(r.stop);
    }
    t.records.clear();
    t.totals.clear();
    t.depth = 0;
    t.on = true;
    return MLCGB_OK;
}

int mlcgb_timeline_end(void) {
    mlcgb::Timeline &t = mlcgb::g_timeline;
    t.on = false;
    t.totals.clear();
    for (auto &r : t.records) {
        if (cudaEventSynchronize(r.stop) != cudaSuccess) {
            mlcgb::g_last_cuda_error = (int)cudaGetLastError();
            return MLCGB_E_LAUNCH;
        }
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess) {
            mlcgb::g_last_cuda_error = (int)cudaGetLastError();
            return MLCGB_E_LAUNCH;
        }
        bool found = false;
        for (auto &tt : t.totals)
            if (tt.name == r.name || std::strcmp(tt.name, r.name) == 0) {
                tt.calls++;
                tt.ms += ms;
                found = true;
                break;
            }
        if (!found) t.totals.push_back({r.name, 1, (double)ms});
    }
    return (int)t.totals.size();
}

int mlcgb_timeline_entry(int index, const char **name, int64_t *calls, double *ms) {
    mlcgb::Timeline &t = mlcgb::g_timeline;
    if (index < 0 || index >= (int)t.totals.size() || !name || !calls || !ms) return MLCGB_E_ARG;
    *name = t.totals[index].name;
    *calls = t.totals[index].calls;
    *ms = t.totals[index].ms;
    return MLCGB_OK;
}

}  // extern "C"
