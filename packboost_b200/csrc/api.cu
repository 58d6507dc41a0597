// Error reporting and device probes of the C ABI.

#include <stdarg.h>

#include <atomic>
#include <mutex>
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

// Timing hooks: when enabled, a pair of events brackets each launch of a kernel family on the
// launching stream; pb_profile_collect (after the caller synchronised) sums the elapsed times.
static bool g_prof_on = false;
static std::vector<cudaEvent_t> g_ev_pool;
static std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> g_ev_used;
static cudaEvent_t g_open[kProfKinds];
static std::atomic<long long> g_launches{0};
static std::mutex g_prof_mu;

static cudaEvent_t take_event() {
    if (!g_ev_pool.empty()) {
        cudaEvent_t e = g_ev_pool.back();
        g_ev_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

// (no timing inside a stream capture: the events would become graph dependencies)
static bool capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    return cudaStreamIsCapturing(stream, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone;
}

void prof_begin(int kind, cudaStream_t stream) {
    if (!g_prof_on || capturing(stream)) return;
    std::lock_guard<std::mutex> lk(g_prof_mu);
    cudaEvent_t e = take_event();
    cudaEventRecord(e, stream);
    g_open[kind] = e;
}

void prof_end(int kind, cudaStream_t stream) {
    if (!g_prof_on || capturing(stream)) return;
    std::lock_guard<std::mutex> lk(g_prof_mu);
    cudaEvent_t e = take_event();
    cudaEventRecord(e, stream);
    g_ev_used.push_back({kind, {g_open[kind], e}});
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

}  // namespace pb

extern "C" int pb_profile_enable(int on) {
    std::lock_guard<std::mutex> lk(pb::g_prof_mu);
    pb::g_prof_on = (on != 0);
    return PB_OK;
}

extern "C" int pb_profile_collect(double* ms_by_kind, int64_t* launches_by_kind) {
    PB_REQUIRE(ms_by_kind && launches_by_kind, "null argument");
    std::lock_guard<std::mutex> lk(pb::g_prof_mu);
    for (int k = 0; k < pb::kProfKinds; ++k) { ms_by_kind[k] = 0.0; launches_by_kind[k] = 0; }
    for (auto& u : pb::g_ev_used) {
        float ms = 0.f;
        cudaError_t e = cudaEventElapsedTime(&ms, u.second.first, u.second.second);
        if (e != cudaSuccess) return pb::fail_cuda(e, "cudaEventElapsedTime (synchronise the stream first)");
        ms_by_kind[u.first] += ms;
        launches_by_kind[u.first] += 1;
        pb::g_ev_pool.push_back(u.second.first);
        pb::g_ev_pool.push_back(u.second.second);
    }
    pb::g_ev_used.clear();
    return PB_OK;
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
