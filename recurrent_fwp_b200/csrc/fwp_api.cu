// Host-side plumbing shared by every entry point: argument validation, status
// strings, the per-thread CUDA error slot, the launch counter and the tuning table.
#include <atomic>
#include <climits>
#include <cstring>
#include "fwp_core.cuh"

namespace fwp {

static thread_local int g_last_cuda_error = 0;
static std::atomic<unsigned long long> g_launches{0};
static thread_local const char* g_last_kernel = "";

// Process-wide execution-plan switches: one atomic per key, INT_MIN = not set.
static const char* const kTuneNames[T_COUNT] = {
    "delta.blocked", "delta.chunk64", "delta.tc64",
    "delta_fwd.16.split", "delta_fwd.32.split", "delta_fwd.64.split",
    "sum_fwd.16.split", "sum_fwd.32.split", "sum_fwd.64.split",
    "delta_bwd.16.split", "delta_bwd.32.split", "delta_bwd.64.split",
    "delta_bwd.bulk", "delta_bwd.16.chunk",
    "lstm_fwd.32.split", "lstm_bwd.32.split", "rnn_fwd.32.split", "rnn_bwd.32.split", "rec_fwd.32.split", "rec_bwd.32.split",
    "rec_fwd.32.warp", "rnn_bwd.32.roles", "lstm_bwd.32.roles", "lstm_fwd.32.gates", "delta.pipe64", "rec_bwd.32.roles", "sum_bwd.roles", "launch.dependent", "step.spread",
};
struct TuneTable {
    std::atomic<int> v[T_COUNT];
    TuneTable() { for (auto& x : v) x.store(INT_MIN, std::memory_order_relaxed); }
};
static TuneTable g_tune;

int set_cuda_error(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return FWP_ERR_CUDA;
}

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

void note_kernel(const char* name) { g_last_kernel = name; }

// SMs of the current device (asked once per device)
int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

int tune_get(TuneKey key, int fallback) {
    const int v = g_tune.v[key].load(std::memory_order_relaxed);
    return v == INT_MIN ? fallback : v;
}

int check_tensor(const fwp_tensor* t, int elem_bytes, bool required) {
    if (!t) return required ? FWP_ERR_NULL : FWP_OK;
    if (!t->data) return required ? FWP_ERR_NULL : FWP_OK;
    if (t->stride[3] != 1) return FWP_ERR_STRIDE;
    if (t->stride[0] < 0 || t->stride[1] < 0 || t->stride[2] < 0) return FWP_ERR_STRIDE;
    if (reinterpret_cast<uintptr_t>(t->data) % (uintptr_t)elem_bytes) return FWP_ERR_ALIGN;
    return FWP_OK;
}

}  // namespace fwp

FWP_API const char* fwp_status_string(int status) {
    switch (status) {
        case FWP_OK: return "ok";
        case FWP_ERR_NULL: return "a required tensor or pointer is NULL";
        case FWP_ERR_SHAPE: return "a size is <= 0 or inconsistent";
        case FWP_ERR_STRIDE: return "unsupported strides (innermost stride must be 1, none negative)";
        case FWP_ERR_ALIGN: return "pointer not aligned to its element size";
        case FWP_ERR_DTYPE: return "unknown io_dtype";
        case FWP_ERR_UNSUPPORTED: return "head dimension beyond what the kernels cover";
        case FWP_ERR_CUDA: return "a CUDA runtime call failed (see fwp_last_cuda_error)";
        case FWP_ERR_VARIANT: return "unknown LSTM variant (must be 1..4)";
        case FWP_ERR_SCRATCH: return "scratch buffer missing, misaligned or too small";
        case FWP_ERR_NOALLOC_TOO_LARGE: return "problem too large for the built-in scratch of the no-allocation entry point (N*H*(3*D*D+D) > FWP_NOALLOC_SCRATCH_FLOATS)";
    }
    return "unknown status";
}

FWP_API int fwp_last_cuda_error(void) { return fwp::g_last_cuda_error; }
FWP_API int fwp_version(void) { return 100; }
FWP_API int fwp_max_head_dim(void) { return 64; }
FWP_API unsigned long long fwp_launch_count(void) { return fwp::g_launches.load(); }

FWP_API const char* fwp_last_kernel(void) { return fwp::g_last_kernel; }

FWP_API int fwp_tune(const char* key, int value) {
    if (!key) return FWP_ERR_NULL;
    if (value == INT_MIN) return FWP_ERR_SHAPE;
    for (int i = 0; i < fwp::T_COUNT; i++)
        if (std::strcmp(key, fwp::kTuneNames[i]) == 0) {
            fwp::g_tune.v[i].store(value, std::memory_order_relaxed);
            return FWP_OK;
        }
    return FWP_ERR_UNSUPPORTED;     // not a switch of this library
}
