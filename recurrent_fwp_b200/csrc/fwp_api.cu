// Host-side plumbing shared by every entry point: argument validation, status
// strings, the per-thread CUDA error slot, the launch counter and the tuning table.
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include "fwp_core.cuh"

namespace fwp {

static thread_local int g_last_cuda_error = 0;
static std::atomic<unsigned long long> g_launches{0};
static std::mutex g_tune_mu;
static std::map<std::string, int>& tune_table() {
    static std::map<std::string, int> t;
    return t;
}

int set_cuda_error(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return FWP_ERR_CUDA;
}

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int tune_get(const char* key, int fallback) {
    std::lock_guard<std::mutex> lk(g_tune_mu);
    auto it = tune_table().find(key);
    return it == tune_table().end() ? fallback : it->second;
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

FWP_API int fwp_tune(const char* key, int value) {
    if (!key || std::strlen(key) > 40) return FWP_ERR_NULL;
    std::lock_guard<std::mutex> lk(fwp::g_tune_mu);
    fwp::tune_table()[key] = value;
    return FWP_OK;
}
