// Chunkwise plan of the delta rule for bf16 streams with E = M = 64: kernels in fwp_delta_chunk_bf16.cuh,
// applicability test and launches here.  One fused launch per direction, no workspace.
#include <atomic>
#include "fwp_delta_chunk_bf16.cuh"
#include "fwp_delta_tc.cuh"

namespace fwp {

static bool rows_ok(const Row4& r, int elem_bytes) {
    const long long per16 = 16 / elem_bytes;
    return (reinterpret_cast<uintptr_t>(r.p) & 15) == 0 && r.sN % per16 == 0 && r.sH % per16 == 0 && r.sL % per16 == 0;
}

bool chunk_bf16_applies(const DeltaFwdParams& p) {
    return p.E == cb::D && p.M == cb::D && rows_ok(p.q, 2) && rows_ok(p.k, 2) && rows_ok(p.v, 2) && rows_ok(p.out, 2) &&
           rows_ok(p.v_old, 4) && (!p.v_ins.p || rows_ok(p.v_ins, 4));
}

// tcgen05 forward: needs 16-byte aligned rows for the TMA maps, an 8-byte aligned state with even strides for
// its two-float accesses, and a caller that does not ask for u_t (v_insert)
static bool tc_applies(const DeltaFwdParams& p) {
    return !p.v_ins.p && (reinterpret_cast<uintptr_t>(p.W) & 7) == 0 && p.wN % 2 == 0 && p.wH % 2 == 0 && p.wE % 2 == 0 &&
           (unsigned long long)p.q.sN * 2 < (1ull << 40) && (unsigned long long)p.k.sN * 2 < (1ull << 40) &&
           (unsigned long long)p.v.sN * 2 < (1ull << 40);
}

static int launch_fwd_tc(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    CUtensorMap tq, tk, tv;
    const int N = p.NH / p.H;
    if (!tc_make_map(&tq, p.q, N, p.H, p.L) || !tc_make_map(&tk, p.k, N, p.H, p.L) || !tc_make_map(&tv, p.v, N, p.H, p.L))
        return -1;      // the driver refused the layout: the caller takes the warp-level kernel
    const size_t bytes = sizeof(tcd::Smem) + 1024;
    if (int rc = set_smem(delta_fwd_tc_kernel, bytes)) return rc;
    delta_fwd_tc_kernel<<<nseq, tcd::NTH, bytes, st>>>(p, tq, tk, tv);
    count_launch();
    note_kernel("delta_fwd_tc_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

// 1 if a bounded wait of the tcgen05 kernel ran out on the current device since the last call (reading clears it)
int tc_fault_read_clear() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_fault, sizeof v) != cudaSuccess) return -1;
    if (v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tc_fault, &zero, sizeof zero);
    }
    return v;
}


// Test hook for the bounded waits: one CTA waits, with the given poll limit, on an mbarrier that nothing ever
// completes.  The wait runs out, the kernel returns and the device flag is raised, exactly what a kernel of this file
// does when a copy or a product it waits for never arrives.
__global__ void tc_wait_probe_kernel(unsigned limit) {
    __shared__ uint64_t bar;
    __shared__ int failed;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        failed = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    tc::mbar_wait(&bar, 0, &failed, limit);
    __syncthreads();
    if (failed && threadIdx.x == 0) atomicExch(&g_tc_fault, 1);
}

int launch_wait_probe(int polls, cudaStream_t st) {
    tc_wait_probe_kernel<<<1, 32, 0, st>>>((unsigned)polls);
    count_launch();
    note_kernel("tc_wait_probe_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

int launch_fwd_chunk_bf16(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    // "delta.tc64": the tcgen05 / TMA forward (64-step chunks, one sequence per SM) or the warp-level mma forward
    // (16-step chunks, four sequences per SM).  -1 (default) picks by the measured crossover: with no more sequences
    // than SMs every sequence has an SM to itself either way and the tcgen05 kernel is 1.1x (L = 128) to 1.6x
    // (L = 4096) faster; beyond that the warp-level kernel's four resident sequences per SM win.  1 / 0 force one.
    const int tc = tune_get(T_DELTA_TC64, -1);
    if ((tc == 1 || (tc == -1 && p.L >= 128 && nseq <= sm_count())) && tc_applies(p)) {
        const int rc = launch_fwd_tc(p, nseq, st);
        if (rc >= 0) return rc;
    }
    // "delta.pipe64" = 1 (default): the state-independent part of every chunk is prepared one chunk ahead by a fifth warp
    if (tune_get(T_DELTA_PIPE64, 1) >= 1)
        return launch(delta_fwd_chunk_bf16_pipe_kernel, p, nseq, cb::NTP, sizeof(cb::SmemP), st, "delta_fwd_chunk_bf16_pipe_kernel");
    return launch(delta_fwd_chunk_bf16_inv_kernel, p, nseq, cb::NT, sizeof(cb::SmemI), st, "delta_fwd_chunk_bf16_inv_kernel");
}

bool chunk_bf16_applies(const DeltaBwdParams& p) {
    return p.E == cb::D && p.M == cb::D && rows_ok(p.q, 2) && rows_ok(p.k, 2) && rows_ok(p.v, 2) && rows_ok(p.gy, 2) &&
           rows_ok(p.v_old, 4) && rows_ok(p.gq, 2) && rows_ok(p.gk, 2) && rows_ok(p.gv, 2) &&
           (reinterpret_cast<uintptr_t>(p.W) & 7) == 0 && p.wN % 2 == 0 && p.wH % 2 == 0 && p.wE % 2 == 0;
}

int launch_bwd_chunk_bf16(const DeltaBwdParams& p, int nseq, cudaStream_t st) {
    // "delta.pipe64": 1 both directions with a preparing warp, 2 the forward only, 0 neither
    if (tune_get(T_DELTA_PIPE64, 1) == 1)
        return launch(delta_bwd_chunk_bf16_pipe_kernel, p, nseq, cb::NTP, sizeof(cb::SmemBP), st, "delta_bwd_chunk_bf16_pipe_kernel");
    return launch(delta_bwd_chunk_bf16_inv_kernel, p, nseq, cb::NT, sizeof(cb::SmemB2), st, "delta_bwd_chunk_bf16_inv_kernel");
}

}  // namespace fwp
