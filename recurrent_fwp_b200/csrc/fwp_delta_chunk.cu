// Chunkwise plan of the delta rule: kernels in fwp_delta_chunk.cuh, launch sequence here.
#include "fwp_delta_chunk.cuh"
#include "fwp_delta_chunk_bf16.cuh"

namespace fwp {

size_t chunk_ws_floats(long long nseq, int L, int E, int M, int io_dtype, bool backward) {
    if (io_dtype != FWP_F32 || E > 16 || M > 16 || L < 1 || nseq < 1) return 0;
    return (size_t)nseq * ((L + 15) / 16) * (backward ? CkWs::kBwd : CkWs::kFwd);
}

static int chunk_grid(int nseq, int L) {
    const long long chunks = (long long)nseq * ((L + 15) / 16);
    return (int)((chunks + kCkWarps - 1) / kCkWarps);
}

int launch_fwd_chunk(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    const int grid = chunk_grid(nseq, p.L);
    if (int rc = launch(delta_fwd_chunk_prep_kernel, p, grid, kCkWarps * 32, kCkWarps * CkFwdPrep::kWarp * sizeof(float), st)) return rc;
    if (int rc = launch(delta_fwd_chunk_scan_kernel, p, nseq, 32, kCkScanDepth * 2 * 256 * sizeof(float), st)) return rc;
    return launch(delta_fwd_chunk_post_kernel, p, grid, kCkWarps * 32, kCkWarps * CkFwdPost::kWarp * sizeof(float), st);
}

int launch_bwd_chunk(const DeltaBwdParams& p, int nseq, cudaStream_t st) {
    const int grid = chunk_grid(nseq, p.L);
    if (int rc = launch(delta_bwd_chunk_prep_kernel, p, grid, kCkWarps * 32, kCkWarps * CkBwdPrep::kWarp * sizeof(float), st)) return rc;
    if (int rc = launch(delta_bwd_chunk_scan_kernel, p, nseq, 32, kCkScanDepth * 3 * 256 * sizeof(float), st)) return rc;
    return launch(delta_bwd_chunk_post_kernel, p, grid, kCkWarps * 32, kCkWarps * CkBwdPost::kWarp * sizeof(float), st);
}

// ---- bf16 streams, E = M = 64: one fused launch per direction, no workspace
static bool rows_ok(const Row4& r, int elem_bytes) {
    const long long per16 = 16 / elem_bytes;
    return (reinterpret_cast<uintptr_t>(r.p) & 15) == 0 && r.sN % per16 == 0 && r.sH % per16 == 0 && r.sL % per16 == 0;
}

bool chunk_bf16_applies(const DeltaFwdParams& p) {
    return p.E == cb::D && p.M == cb::D && rows_ok(p.q, 2) && rows_ok(p.k, 2) && rows_ok(p.v, 2) && rows_ok(p.out, 2) &&
           rows_ok(p.v_old, 4) && (!p.v_ins.p || rows_ok(p.v_ins, 4));
}

int launch_fwd_chunk_bf16(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    // "delta_fwd.chunk64.solve" = 1: per-thread substitution through shared memory (0.93 ms at 512 sequences of 4096
    // steps); 0, the default: explicit inverse in registers (0.86 ms; 1.43 against 1.75 ms at 4096 sequences of 1024)
    if (tune_get("delta_fwd.chunk64.solve", 0) == 0)
    {
        const int ctas = tune_get("delta_fwd.chunk64.ctas", 4);     // resident CTAs per SM the kernel is compiled for
        if (ctas == 5) return launch(delta_fwd_chunk_bf16_inv_kernel<5>, p, nseq, cb::NT, sizeof(cb::SmemI), st);
        if (ctas == 6) return launch(delta_fwd_chunk_bf16_inv_kernel<6>, p, nseq, cb::NT, sizeof(cb::SmemI), st);
        return launch(delta_fwd_chunk_bf16_inv_kernel<4>, p, nseq, cb::NT, sizeof(cb::SmemI), st);
    }
    return launch(delta_fwd_chunk_bf16_kernel, p, nseq, cb::NT, sizeof(cb::Smem), st);
}

bool chunk_bf16_applies(const DeltaBwdParams& p) {
    return p.E == cb::D && p.M == cb::D && rows_ok(p.q, 2) && rows_ok(p.k, 2) && rows_ok(p.v, 2) && rows_ok(p.gy, 2) &&
           rows_ok(p.v_old, 4) && rows_ok(p.gq, 2) && rows_ok(p.gk, 2) && rows_ok(p.gv, 2) &&
           (reinterpret_cast<uintptr_t>(p.W) & 7) == 0 && p.wN % 2 == 0 && p.wH % 2 == 0 && p.wE % 2 == 0;
}

int launch_bwd_chunk_bf16(const DeltaBwdParams& p, int nseq, cudaStream_t st) {
    // "delta_bwd.chunk64.solve" = 1: per-thread substitution through shared memory (2.55 ms at 512 sequences of 4096
    // steps); 0, the default: explicit inverse in registers (1.82 ms; 2.69 against 3.80 ms at 4096 sequences of 1024)
    if (tune_get("delta_bwd.chunk64.solve", 0) == 0)
        return tune_get("delta_bwd.chunk64.ctas", 3) == 4
                   ? launch(delta_bwd_chunk_bf16_inv_kernel<4>, p, nseq, cb::NT, sizeof(cb::SmemB2), st)
                   : launch(delta_bwd_chunk_bf16_inv_kernel<3>, p, nseq, cb::NT, sizeof(cb::SmemB2), st);
    return launch(delta_bwd_chunk_bf16_kernel, p, nseq, cb::NT, sizeof(cb::SmemB), st);
}

}  // namespace fwp
