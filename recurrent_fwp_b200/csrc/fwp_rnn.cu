// Delta RNN v2 and v1 (fast-weight RNN whose recurrent matrix is written by the delta rule), sm_100a.
//
//   both : S_t = S_{t-1} + k_t (x) beta_t (v_t - S_{t-1}^T k_t)
//   v2   : s_t = exp(h_{t-1} - max) / (sum + 1e-6) ;  h_t = S_t^T s_t + z_t
//   v1   : h_t = softmax(S_t^T h_{t-1} + z_t)
//
// Restates algorithmic/fast_weight_rnn_v2/fast_rnn_cuda.cu (forward kernel :25-229,
// backward kernel :297-588) and language_modeling/src/utils/fast_weight_rnn/fast_rnn_cuda.cu
// with the register-resident plan of fwp_core.cuh.  These are per-step latency
// kernels: the hidden state feeds back through a softmax every step.
#include "fwp_core.cuh"

namespace fwp {

constexpr float kSoftmaxEps = 1e-6f;

struct RnnFwdParams {
    Row4 z, k, v, beta, v_old, out, out_nmz;
    float* W; long long wN, wH, wE;
    float* h; long long hN, hH;
    int H, L, D;
};

template <int D, int TC>
struct RnnFwdStage {
    Tile<D, TC, float> z, k, v;
    Tile<1, TC, float> b;
    static constexpr int kFloats = 3 * r4(TC * D) + r4(TC);
    __device__ __forceinline__ void bind(float* mem) {
        z.bind(mem); mem += r4(TC * D);
        k.bind(mem); mem += r4(TC * D);
        v.bind(mem); mem += r4(TC * D);
        b.bind(mem);
    }
};

template <int D, int SPLIT, int TC, bool V1>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) rnn_fwd_kernel(const RnnFwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = RnnFwdStage<D, TC>;
    constexpr int kX = 2 * (D + 16);      // per parity: vector[D], reduction slots[2][8]
    for (int i = g.tid; i < 2 * Stage::kFloats + kX; i += G::NT) smem[i] = 0.f;
    float* xch = smem + 2 * Stage::kFloats;

    Src<float> sz, sk, sv, sb;
    sz.init(p.z, n, h, p.D);
    sk.init(p.k, n, h, p.D);
    sv.init(p.v, n, h, p.D);
    sb.init(p.beta, n, h, 1);

    float* W = p.W + n * p.wN + h * p.wH;
    float* hp = p.h + n * p.hN + h * p.hH;
    f2 S[G::NP];
    load_cols(g, S, W, p.wE, p.D, p.D);
    const bool ok = g.idx < p.D;
    float hv = ok ? hp[g.idx] : 0.f;
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int c) {
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.z.template load<G::NT>(sz, t0, nt, g.tid);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        s.b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    issue(0);
    // running output pointers of this thread's column (threads that store nothing keep a valid address)
    const bool writer = ok && g.s == 0;
    const int col = writer ? g.idx : 0;
    float* po = reinterpret_cast<float*>(p.out.p) + n * p.out.sN + h * p.out.sH + col;
    float* pvo = reinterpret_cast<float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH + col;
    float* pnm = V1 ? po : reinterpret_cast<float*>(p.out_nmz.p) + n * p.out_nmz.sN + h * p.out_nmz.sH + col;
    const long long so = p.out.sL, svo = p.v_old.sL, snm = V1 ? 0 : p.out_nmz.sL;
    int par = 0;
    for (int c = 0; c < nchunks; c++) {
        if (c + 1 < nchunks) { issue(c + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int nt = min(TC, p.L - c * TC);
        const float* krow = s.k.f + g.off;
        const float* vcol = s.v.f + g.idx;
        const float* zcol = s.z.f + g.idx;
        const float* brow = s.b.f;
#pragma unroll 1
        for (int t = 0; t < nt; t++, krow += D, vcol += D, zcol += D, brow++) {
            float* xv = xch + par * (D + 16);
            float* slot = xv + D;
            par ^= 1;
            // delta update of the recurrent matrix: independent of the hidden state, so in the v2 step it is placed
            // between the start of the softmax (max, exp, sum: long fixed latencies) and its use
            f2 kk[G::NP];
            lds_slice<G::NR>(kk, krow);
            const float zz = zcol[0];
            float hn, vo;
            if constexpr (!V1) {
                const float mx = cta_allreduce_idx<G, true>(g, ok ? hv : -INFINITY, slot);
                const float ex = ok ? exp_neg(hv - mx) : 0.f;
                if (g.s == 0) xv[g.idx] = ex;
                const float den = softmax_den(g, ex, slot + 8);
                vo = reduce_split<SPLIT>(dot2<G::NP>(S, kk));
                const float u = brow[0] * (vcol[0] - vo);
                axpy2<G::NP>(S, kk, u);
                cta_sync<G::WPS>();
                const float inv = rcp_approx(den + kSoftmaxEps);
                f2 ss[G::NP];
                lds_slice<G::NR>(ss, xv + g.off);
                hn = reduce_split<SPLIT>(dot2<G::NP>(S, ss)) * inv + zz;
                if (writer) *pnm = ex * inv;
            } else {
                vo = reduce_split<SPLIT>(dot2<G::NP>(S, kk));
                const float u = brow[0] * (vcol[0] - vo);
                axpy2<G::NP>(S, kk, u);
                if (g.s == 0) xv[g.idx] = hv;
                cta_sync<G::WPS>();
                f2 ss[G::NP];
                lds_slice<G::NR>(ss, xv + g.off);
                const float pre = reduce_split<SPLIT>(dot2<G::NP>(S, ss)) + zz;
                const float mx = cta_allreduce_idx<G, true>(g, ok ? pre : -INFINITY, slot);
                const float ex = ok ? exp_neg(pre - mx) : 0.f;
                hn = ex * rcp_approx(softmax_den(g, ex, slot + 8));
            }
            hv = hn;
            if (writer) {
                *po = hn;
                *pvo = vo;
            }
            po += so; pvo += svo; pnm += snm;
        }
        __syncthreads();
    }
    store_cols(g, S, W, p.wE, p.D, p.D);
    if (ok && g.s == 0) hp[g.idx] = hv;
}

// ------------------------------------------------------------------ backward
struct RnnBwdParams {
    Row4 k, v, beta, v_old, gy, out, od, gz, gk, gv, gb;
    float* W; long long wN, wH, wE;
    int H, L, D;
};

template <int D, int TC, bool V1>
struct RnnBwdStage {
    Tile<D, TC, float> k, v, gy, vo, od, out;
    Tile<1, TC, float> b;
    static constexpr int kFloats = (V1 ? 6 : 5) * r4(TC * D) + r4(TC);
    __device__ __forceinline__ void bind(float* mem) {
        k.bind(mem); mem += r4(TC * D);
        v.bind(mem); mem += r4(TC * D);
        gy.bind(mem); mem += r4(TC * D);
        vo.bind(mem); mem += r4(TC * D);
        od.bind(mem); mem += r4(TC * D);
        if (V1) { out.bind(mem); mem += r4(TC * D); }
        b.bind(mem);
    }
};

// v2 step (time reversed): g = gy + g_h ; dz = g ; G += s (x) g ; gs = S_t g ; delta block ; g_h = s .* (gs - <s, gs>)
// v1 step:                 g = gy + g_h ; dz = h_t .* (g - <h_t, g>) ; G += h_{t-1} (x) dz ; g_h = S_t dz ; delta block
template <int D, int SPLIT, int TC, bool V1>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) rnn_bwd_kernel(const RnnBwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = RnnBwdStage<D, TC, V1>;
    constexpr int kXs = 3 * D + 24;       // per parity: g[D], u[D], br[D], slots[3][8]
    for (int i = g.tid; i < 2 * Stage::kFloats + 2 * kXs; i += G::NT) smem[i] = 0.f;
    float* xch = smem + 2 * Stage::kFloats;

    Src<float> sk, sv, sg, so, sd, sb, sout;
    sk.init(p.k, n, h, p.D);
    sv.init(p.v, n, h, p.D);
    sg.init(p.gy, n, h, p.D);
    so.init(p.v_old, n, h, p.D);
    sd.init(p.od, n, h, p.D);
    sb.init(p.beta, n, h, 1);
    if (V1) sout.init(p.out, n, h, p.D);

    float* W = p.W + n * p.wN + h * p.wH;
    f2 Sr[G::NP], Gr[G::NP], Gc[G::NP];
    load_rows(g, Sr, W, p.wE, p.D, p.D);
#pragma unroll
    for (int i = 0; i < G::NP; i++) { Gr[i] = 0ull; Gc[i] = 0ull; }
    float gh = 0.f;
    const bool ok = g.idx < p.D;
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {
        Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        s.gy.template load<G::NT>(sg, t0, nt, g.tid);
        s.vo.template load<G::NT>(so, t0, nt, g.tid);
        s.od.template load<G::NT>(sd, t0, nt, g.tid);
        if (V1) s.out.template load<G::NT>(sout, t0, nt, g.tid);
        s.b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    issue(0);
    int par = 0;
    for (int j = 0; j < nchunks; j++) {
        if (j + 1 < nchunks) { issue(j + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        for (int t = nt - 1; t >= 0; t--) {
            float* xg = xch + par * kXs;
            float* xu = xg + D;
            float* xbr = xu + D;
            float* slot = xbr + D;
            par ^= 1;
            const float beta = s.b.f[t];
            // ---- column role
            float gcol = s.gy.f[t * D + g.idx] + gh;     // g[m]
            if constexpr (V1) {
                const float hm = s.out.f[t * D + g.idx];
                const float dotp = cta_allreduce_idx<G, false>(g, hm * gcol, slot);
                gcol = hm * (gcol - dotp);               // dz[m]
            }
            {
                f2 xs[G::NP], kk[G::NP];
                lds_slice<G::NR>(xs, s.od.f + t * D + g.off);
                lds_slice<G::NR>(kk, s.k.f + t * D + g.off);
                const float w = s.v.f[t * D + g.idx] - s.vo.f[t * D + g.idx];
                axpy2<G::NP>(Gc, xs, gcol);
                const float r = reduce_split<SPLIT>(dot2<G::NP>(Gc, kk));
                const float br = beta * r;
                axpy2<G::NP>(Gc, kk, -br);
                const float db = cta_allreduce_idx<G, false>(g, r * w, slot + 8);
                if (g.s == 0) {
                    xg[g.idx] = gcol;
                    xu[g.idx] = beta * w;
                    xbr[g.idx] = br;
                    if (ok) {
                        put<float>(p.gz, n, h, t0 + t, g.idx, gcol);
                        put<float>(p.gv, n, h, t0 + t, g.idx, br);
                    }
                }
                if (g.tid == 0) put<float>(p.gb, n, h, t0 + t, 0, db);
            }
            cta_sync<G::WPS>();
            // ---- row role
            {
                f2 gr[G::NP], ur[G::NP], brr[G::NP];
                lds_slice<G::NR>(gr, xg + g.off);
                lds_slice<G::NR>(ur, xu + g.off);
                lds_slice<G::NR>(brr, xbr + g.off);
                const float se = s.od.f[t * D + g.idx], ke = s.k.f[t * D + g.idx];
                float gs = dot2<G::NP>(Sr, gr);
                axpy2<G::NP>(Gr, gr, se);
                float dk = dot2<G::NP>(Gr, ur);
                axpy2<G::NP>(Sr, ur, -ke);
                dk -= dot2<G::NP>(Sr, brr);
                axpy2<G::NP>(Gr, brr, -ke);
                gs = reduce_split<SPLIT>(gs);
                dk = reduce_split<SPLIT>(dk);
                if (ok && g.s == 0) put<float>(p.gk, n, h, t0 + t, g.idx, dk);
                if constexpr (V1) {
                    gh = gs;
                } else {
                    const float dotp = cta_allreduce_idx<G, false>(g, se * gs, slot + 16);
                    gh = se * (gs - dotp);
                }
            }
        }
        __syncthreads();
    }
    store_rows(g, Sr, W, p.wE, p.D, p.D);
}

}  // namespace fwp
#include "fwp_rnn_roles.cuh"
namespace fwp {

// ------------------------------------------------------------------ launchers
template <typename K>
static int smem_optin(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return set_cuda_error(e);
    }
    return FWP_OK;
}

template <int D, int SPLIT, int TC, bool V1>
static int launch_rnn_fwd(const RnnFwdParams& p, int nseq, cudaStream_t st) {
    auto kern = rnn_fwd_kernel<D, SPLIT, TC, V1>;
    const size_t bytes = (2 * RnnFwdStage<D, TC>::kFloats + 2 * (D + 16)) * sizeof(float);
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    if (int rc = smem_optin(kern, bytes * slots)) return rc;
    kern<<<nseq / slots, D * SPLIT * slots, bytes * slots, st>>>(p);
    count_launch();
    note_kernel("rnn_fwd_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int D, int SPLIT, int TC, bool V1>
static int launch_rnn_bwd(const RnnBwdParams& p, int nseq, cudaStream_t st) {
    auto kern = rnn_bwd_kernel<D, SPLIT, TC, V1>;
    const size_t bytes = (2 * RnnBwdStage<D, TC, V1>::kFloats + 2 * (3 * D + 24)) * sizeof(float);
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    if (int rc = smem_optin(kern, bytes * slots)) return rc;
    kern<<<nseq / slots, D * SPLIT * slots, bytes * slots, st>>>(p);
    count_launch();
    note_kernel("rnn_bwd_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int TC, bool V1>
static int launch_rnn_bwd_roles32(const RnnBwdParams& p, int nseq, cudaStream_t st) {
    auto kern = rnn_bwd_roles32_kernel<TC, V1>;
    int slots = 4;
    while (nseq % slots) slots >>= 1;
    const size_t bytes = (size_t)RnnRolesSmem<TC, V1>::kFloats * sizeof(float) * slots;
    if (int rc = smem_optin(kern, bytes)) return rc;
    kern<<<nseq / slots, 64 * slots, bytes, st>>>(p);
    count_launch();
    note_kernel("rnn_bwd_roles32_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <bool V1>
static int rnn_forward(int N, int H, int L, int D,
                       const fwp_tensor* Z, const fwp_tensor* K, const fwp_tensor* V,
                       const fwp_tensor* beta, const fwp_tensor* v_old,
                       const fwp_tensor* states, const fwp_tensor* kv,
                       const fwp_tensor* out, const fwp_tensor* out_nmz,
                       int io_dtype, void* stream, int device) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32) return FWP_ERR_DTYPE;
    const int DP = pad_dim(D);
    if (!DP) return FWP_ERR_UNSUPPORTED;
    int rc;
    if ((rc = check_tensor(Z, 4, true)) || (rc = check_tensor(K, 4, true)) || (rc = check_tensor(V, 4, true)) ||
        (rc = check_tensor(beta, 4, true)) || (rc = check_tensor(v_old, 4, true)) ||
        (rc = check_tensor(states, 4, true)) || (rc = check_tensor(kv, 4, true)) ||
        (rc = check_tensor(out, 4, true)) || (rc = check_tensor(out_nmz, 4, !V1)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    RnnFwdParams p;
    p.z = row4(Z); p.k = row4(K); p.v = row4(V); p.beta = row4(beta); p.v_old = row4(v_old);
    p.out = row4(out); p.out_nmz = row4(out_nmz);
    p.W = (float*)kv->data; p.wN = kv->stride[0]; p.wH = kv->stride[1]; p.wE = kv->stride[2];
    p.h = (float*)states->data; p.hN = states->stride[0]; p.hH = states->stride[1];
    p.H = H; p.L = L; p.D = D;
    cudaStream_t st = (cudaStream_t)stream;
    switch (DP) {
        case 16: return launch_rnn_fwd<16, 2, 32, V1>(p, N * H, st);
        case 32: {
            const int sp = tune_get(T_RNN_FWD_SPLIT32, 1);
            if (sp == 2) return launch_rnn_fwd<32, 2, 16, V1>(p, N * H, st);
            return launch_rnn_fwd<32, 1, 16, V1>(p, N * H, st);
        }
        case 64: return launch_rnn_fwd<64, 2, 8, V1>(p, N * H, st);
    }
    return FWP_ERR_UNSUPPORTED;
}

template <bool V1>
static int rnn_backward(int N, int H, int L, int D,
                        const fwp_tensor* K, const fwp_tensor* V, const fwp_tensor* beta,
                        const fwp_tensor* v_old, const fwp_tensor* grad_out,
                        const fwp_tensor* out, const fwp_tensor* out_delayed,
                        const fwp_tensor* fw_mem,
                        const fwp_tensor* grad_Z, const fwp_tensor* grad_K,
                        const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                        int io_dtype, void* stream, int device) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32) return FWP_ERR_DTYPE;
    const int DP = pad_dim(D);
    if (!DP) return FWP_ERR_UNSUPPORTED;
    int rc;
    if ((rc = check_tensor(K, 4, true)) || (rc = check_tensor(V, 4, true)) || (rc = check_tensor(beta, 4, true)) ||
        (rc = check_tensor(v_old, 4, true)) || (rc = check_tensor(grad_out, 4, true)) ||
        (rc = check_tensor(out, 4, V1)) || (rc = check_tensor(out_delayed, 4, true)) ||
        (rc = check_tensor(fw_mem, 4, true)) || (rc = check_tensor(grad_Z, 4, true)) ||
        (rc = check_tensor(grad_K, 4, true)) || (rc = check_tensor(grad_V, 4, true)) ||
        (rc = check_tensor(grad_beta, 4, true)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    RnnBwdParams p;
    p.k = row4(K); p.v = row4(V); p.beta = row4(beta); p.v_old = row4(v_old); p.gy = row4(grad_out);
    p.out = row4(out); p.od = row4(out_delayed);
    p.gz = row4(grad_Z); p.gk = row4(grad_K); p.gv = row4(grad_V); p.gb = row4(grad_beta);
    p.W = (float*)fw_mem->data; p.wN = fw_mem->stride[0]; p.wH = fw_mem->stride[1]; p.wE = fw_mem->stride[2];
    p.H = H; p.L = L; p.D = D;
    cudaStream_t st = (cudaStream_t)stream;
    switch (DP) {
        case 16: return launch_rnn_bwd<16, 2, 16, V1>(p, N * H, st);
        case 32: {
            int roles = tune_get(T_RNN_BWD_ROLES32, 1);
            if (p.D != 32 || !rows_16B_aligned(p.k) || !rows_16B_aligned(p.v) || !rows_16B_aligned(p.gy) ||
                !rows_16B_aligned(p.v_old) || !rows_16B_aligned(p.od) || (V1 && !rows_16B_aligned(p.out)))
                roles = 0;              // the two-warp kernel wants full width and 16-byte aligned rows
            if (roles == 1) return launch_rnn_bwd_roles32<16, V1>(p, N * H, st);
            if (roles == 2) return launch_rnn_bwd_roles32<8, V1>(p, N * H, st);
            const int sp = tune_get(T_RNN_BWD_SPLIT32, 1);
            // measured (512 sequences x 512 steps): 1 -> 0.34 ms, 2 -> 0.39 ms, 4 -> 0.42 ms
            if (sp == 2) return launch_rnn_bwd<32, 2, 8, V1>(p, N * H, st);
            if (sp == 4) return launch_rnn_bwd<32, 4, 8, V1>(p, N * H, st);
            return launch_rnn_bwd<32, 1, 8, V1>(p, N * H, st);
        }
        case 64: return launch_rnn_bwd<64, 4, 4, V1>(p, N * H, st);
    }
    return FWP_ERR_UNSUPPORTED;
}

}  // namespace fwp

using namespace fwp;

FWP_API int fwp_fast_rnn_v2_forward(int N, int H, int L, int D,
                                    const fwp_tensor* Z, const fwp_tensor* K, const fwp_tensor* V,
                                    const fwp_tensor* beta, const fwp_tensor* v_old,
                                    const fwp_tensor* states, const fwp_tensor* kv,
                                    const fwp_tensor* out, const fwp_tensor* out_nmz,
                                    int io_dtype, void* stream, int device) {
    return rnn_forward<false>(N, H, L, D, Z, K, V, beta, v_old, states, kv, out, out_nmz, io_dtype, stream, device);
}

FWP_API int fwp_fast_rnn_v2_backward(int N, int H, int L, int D,
                                     const fwp_tensor* K, const fwp_tensor* V, const fwp_tensor* beta,
                                     const fwp_tensor* v_old, const fwp_tensor* grad_out,
                                     const fwp_tensor* out, const fwp_tensor* out_delayed,
                                     const fwp_tensor* fw_mem,
                                     const fwp_tensor* grad_Z, const fwp_tensor* grad_K,
                                     const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                                     int io_dtype, void* stream, int device) {
    return rnn_backward<false>(N, H, L, D, K, V, beta, v_old, grad_out, out, out_delayed, fw_mem,
                               grad_Z, grad_K, grad_V, grad_beta, io_dtype, stream, device);
}

FWP_API int fwp_fast_rnn_forward(int N, int H, int L, int D,
                                 const fwp_tensor* Z, const fwp_tensor* K, const fwp_tensor* V,
                                 const fwp_tensor* beta, const fwp_tensor* v_old,
                                 const fwp_tensor* states, const fwp_tensor* kv,
                                 const fwp_tensor* out,
                                 int io_dtype, void* stream, int device) {
    return rnn_forward<true>(N, H, L, D, Z, K, V, beta, v_old, states, kv, out, nullptr, io_dtype, stream, device);
}

FWP_API int fwp_fast_rnn_backward(int N, int H, int L, int D,
                                  const fwp_tensor* K, const fwp_tensor* V, const fwp_tensor* beta,
                                  const fwp_tensor* v_old, const fwp_tensor* grad_out,
                                  const fwp_tensor* out, const fwp_tensor* out_delayed,
                                  const fwp_tensor* fw_mem,
                                  const fwp_tensor* grad_Z, const fwp_tensor* grad_K,
                                  const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                                  int io_dtype, void* stream, int device) {
    return rnn_backward<true>(N, H, L, D, K, V, beta, v_old, grad_out, out, out_delayed, fw_mem,
                              grad_Z, grad_K, grad_V, grad_beta, io_dtype, stream, device);
}
