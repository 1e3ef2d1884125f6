// Chunkwise plan of the delta rule for bf16 streams with E = M = 64: kernels in fwp_delta_chunk_bf16.cuh,
// applicability test and launches here.  One fused launch per direction, no workspace.
#include "fwp_delta_chunk_bf16.cuh"

namespace fwp {

static bool rows_ok(const Row4& r, int elem_bytes) {
    const long long per16 = 16 / elem_bytes;
    return (reinterpret_cast<uintptr_t>(r.p) & 15) == 0 && r.sN % per16 == 0 && r.sH % per16 == 0 && r.sL % per16 == 0;
}

bool chunk_bf16_applies(const DeltaFwdParams& p) {
    return p.E == cb::D && p.M == cb::D && rows_ok(p.q, 2) && rows_ok(p.k, 2) && rows_ok(p.v, 2) && rows_ok(p.out, 2) &&
           rows_ok(p.v_old, 4) && (!p.v_ins.p || rows_ok(p.v_ins, 4));
}

int launch_fwd_chunk_bf16(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    return launch(delta_fwd_chunk_bf16_inv_kernel, p, nseq, cb::NT, sizeof(cb::SmemI), st, "delta_fwd_chunk_bf16_inv_kernel");
}

bool chunk_bf16_applies(const DeltaBwdParams& p) {
    return p.E == cb::D && p.M == cb::D && rows_ok(p.q, 2) && rows_ok(p.k, 2) && rows_ok(p.v, 2) && rows_ok(p.gy, 2) &&
           rows_ok(p.v_old, 4) && rows_ok(p.gq, 2) && rows_ok(p.gk, 2) && rows_ok(p.gv, 2) &&
           (reinterpret_cast<uintptr_t>(p.W) & 7) == 0 && p.wN % 2 == 0 && p.wH % 2 == 0 && p.wE % 2 == 0;
}

int launch_bwd_chunk_bf16(const DeltaBwdParams& p, int nseq, cudaStream_t st) {
    return launch(delta_bwd_chunk_bf16_inv_kernel, p, nseq, cb::NT, sizeof(cb::SmemB2), st, "delta_bwd_chunk_bf16_inv_kernel");
}

}  // namespace fwp
