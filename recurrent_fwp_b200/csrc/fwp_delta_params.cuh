// Kernel parameter blocks of the delta rule and the launch helper, shared by the translation
// units that hold the recurrent plans and the chunkwise plan.
#pragma once
#include "fwp_core.cuh"

namespace fwp {

struct DeltaFwdParams {
    Row4 q, k, v, beta, v_old, v_ins, out;
    float* W; long long wN, wH, wE;
    int H, L, E, M;
    int NH;     // number of sequences (N*H)
};

struct DeltaBwdParams {
    Row4 q, k, v, beta, v_old, gy, gq, gk, gv, gb;
    float* W; long long wN, wH, wE;
    int H, L, E, M;
    int NH;     // number of sequences (N*H)
    int bulk = 1;           // stage contiguous chunks with bulk copies where the kernel supports it
};

template <typename K>
static int set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return set_cuda_error(e);
    }
    return FWP_OK;
}

// `name` (a string literal) is what fwp_last_kernel() reports for the calling thread afterwards.
template <typename K, typename P>
static int launch(K kern, const P& p, int grid, int threads, size_t bytes, cudaStream_t st, const char* name) {
    if (int rc = set_smem(kern, bytes)) return rc;
    kern<<<grid, threads, bytes, st>>>(p);
    count_launch();
    note_kernel(name);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

// Same, for kernels that call griddep_wait() before their first access to global memory: launched so that they
// may be scheduled while the kernel before them in the stream drains ("launch.dependent" = 0: a plain launch).
template <typename K, typename P>
static int launch_dependent(K kern, const P& p, int grid, int threads, size_t bytes, cudaStream_t st, const char* name) {
    if (!tune_get(T_LAUNCH_DEPENDENT, 1)) return launch(kern, p, grid, threads, bytes, st, name);
    if (int rc = set_smem(kern, bytes)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    count_launch();
    note_kernel(name);
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

// chunkwise plan for bf16 streams with E = M = 64 (fwp_delta_chunk_bf16.cuh): applies when every row is 16-byte aligned
bool chunk_bf16_applies(const DeltaFwdParams& p);
int launch_fwd_chunk_bf16(const DeltaFwdParams& p, int nseq, cudaStream_t st);
bool chunk_bf16_applies(const DeltaBwdParams& p);
int launch_bwd_chunk_bf16(const DeltaBwdParams& p, int nseq, cudaStream_t st);
int tc_fault_read_clear();
int launch_wait_probe(int polls, cudaStream_t st);

}  // namespace fwp
