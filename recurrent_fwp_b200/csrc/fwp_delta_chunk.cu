// Chunkwise plan of the delta rule: kernels in fwp_delta_chunk.cuh, launch sequence here.
#include "fwp_delta_chunk.cuh"

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

}  // namespace fwp
