// Error reporting and device probes of the C ABI.

#include <stdarg.h>
#include <stdlib.h>

#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <mutex>
#include <new>
#include <utility>
#include <vector>

#include "common.cuh"

namespace pb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail_arg(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return PB_ERR_ARG;
}

int fail_cuda(cudaError_t e, const char* what) {
    snprintf(g_error, sizeof(g_error), "CUDA error: %s (%s) in %s", cudaGetErrorString(e), cudaGetErrorName(e), what);
    return PB_ERR_CUDA;
}

// Timing hooks.  A profile object (pb_profile_create) hangs off a training state; while it is
// there, a pair of events brackets each launch of a kernel family on the launching stream and
// pb_profile_collect* (after the caller synchronised) reads the elapsed times.  Every state has
// its own object, so concurrent trainers do not see each other's launches.
struct Profile {
    std::mutex mu;
    std::vector<cudaEvent_t> pool;
    std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> used;
    cudaEvent_t open[kProfKinds] = {};
    ~Profile() {
        for (auto e : pool) cudaEventDestroy(e);
        for (auto& u : used) { cudaEventDestroy(u.second.first); cudaEventDestroy(u.second.second); }
    }
    cudaEvent_t take() {
        if (!pool.empty()) {
            cudaEvent_t e = pool.back();
            pool.pop_back();
            return e;
        }
        cudaEvent_t e = nullptr;
        cudaEventCreate(&e);
        return e;
    }
};
static std::atomic<long long> g_launches{0};

// (no timing inside a stream capture: the events would become graph dependencies)
static bool capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    return cudaStreamIsCapturing(stream, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone;
}

void prof_begin(void* prof, int kind, cudaStream_t stream) {
    if (!prof || capturing(stream)) return;
    Profile* p = static_cast<Profile*>(prof);
    std::lock_guard<std::mutex> lk(p->mu);
    cudaEvent_t e = p->take();
    cudaEventRecord(e, stream);
    p->open[kind] = e;
}

void prof_end(void* prof, int kind, cudaStream_t stream) {
    if (!prof || capturing(stream)) return;
    Profile* p = static_cast<Profile*>(prof);
    std::lock_guard<std::mutex> lk(p->mu);
    if (!p->open[kind]) return;
    cudaEvent_t e = p->take();
    cudaEventRecord(e, stream);
    p->used.push_back({kind, {p->open[kind], e}});
    p->open[kind] = nullptr;
}

// NVTX ranges around the phases of a round (PACKBOOST_NVTX=1): visible on the timeline of a tool
// that attaches to the process, free otherwise.
static bool nvtx_on() {
    static const bool on = [] {
        const char* e = getenv("PACKBOOST_NVTX");
        return e && e[0] == '1';
    }();
    return on;
}
void nvtx_push(const char* fmt, long long a) {
    if (!nvtx_on()) return;
    char buf[64];
    snprintf(buf, sizeof(buf), fmt, a);
    nvtxRangePushA(buf);
}
void nvtx_pop() {
    if (nvtx_on()) nvtxRangePop();
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

}  // namespace pb

extern "C" void* pb_profile_create(void) { return new (std::nothrow) pb::Profile(); }

extern "C" void pb_profile_destroy(void* prof) { delete static_cast<pb::Profile*>(prof); }

static int collect(void* prof, double* ms_by_kind, int64_t* launches_by_kind, int32_t* kinds, float* ms_each, int64_t cap,
                   int64_t* n_out) {
    PB_REQUIRE(prof != nullptr, "profile is null");
    pb::Profile* p = static_cast<pb::Profile*>(prof);
    std::lock_guard<std::mutex> lk(p->mu);
    if (ms_by_kind)
        for (int k = 0; k < pb::kProfKinds; ++k) { ms_by_kind[k] = 0.0; launches_by_kind[k] = 0; }
    int64_t n = 0;
    size_t taken = 0;
    for (auto& u : p->used) {
        // launches come back in issue order; the first one that has not finished yet ends the batch
        // (the caller may be enqueuing ahead of the device) and stays for the next collection
        if (cudaEventQuery(u.second.second) == cudaErrorNotReady) break;
        float ms = 0.f;
        cudaError_t e = cudaEventElapsedTime(&ms, u.second.first, u.second.second);
        if (e != cudaSuccess) return pb::fail_cuda(e, "cudaEventElapsedTime");
        ++taken;
        if (ms_by_kind) {
            ms_by_kind[u.first] += ms;
            launches_by_kind[u.first] += 1;
        }
        if (kinds && n < cap) {
            kinds[n] = u.first;
            ms_each[n] = ms;
        }
        ++n;
        p->pool.push_back(u.second.first);
        p->pool.push_back(u.second.second);
    }
    p->used.erase(p->used.begin(), p->used.begin() + (long)taken);
    if (n_out) *n_out = n;
    return PB_OK;
}

extern "C" int pb_profile_collect(void* prof, double* ms_by_kind, int64_t* launches_by_kind) {
    PB_REQUIRE(ms_by_kind && launches_by_kind, "null argument");
    return collect(prof, ms_by_kind, launches_by_kind, nullptr, nullptr, 0, nullptr);
}

extern "C" int pb_profile_collect_launches(void* prof, int32_t* kinds, float* ms, int64_t cap, int64_t* n_out) {
    PB_REQUIRE(kinds && ms && n_out && cap >= 0, "null argument");
    return collect(prof, nullptr, nullptr, kinds, ms, cap, n_out);
}

extern "C" int64_t pb_launch_count(void) { return (int64_t)pb::g_launches.load(); }

extern "C" const char* pb_last_error(void) { return pb::g_error; }

extern "C" int pb_abi_version(void) { return 1; }

extern "C" int pb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int ok = 0;
    for (int i = 0; i < n; ++i) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ++ok;
    }
    return ok;
}

extern "C" int64_t pb_train_state_bytes(void) { return (int64_t)sizeof(pb_train_state); }
