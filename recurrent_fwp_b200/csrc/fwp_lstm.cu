// Delta LSTM v1..v4: an LSTM-like cell whose three recurrent matrices (input gate,
// update, output gate) are fast weights written by the delta rule.  sm_100a.
//
//   S^g_t = S^g_{t-1} + k^g_t (x) beta^g_t (v^g_t - S^g_{t-1}^T k^g_t)          g in {i, u, o}
//   x_t = h_{t-1} (v1) | exp(h_{t-1}-max)/(sum+1e-6) (v2-4)
//   i = sigmoid(S^i_t^T x + z^i) ; uh = S^u_t^T x + z^u ; u = sigmoid(uh) (v1-3) | uh (v4)
//   o = sigmoid(S^o_t^T x + z^o) ; c_t = i u + (1-i) c_{t-1}
//   h_t = softmax(o c_t) (v1) | o c_t (v2, v4) | o c_t + z^u (v3)
//
// Restates language_modeling/src/utils/fast_lstm/fast_lstm_cuda.cu (forward kernel :28-360,
// backward kernel :484-1056) and the v2/v3/v4 files' variant lines, with the
// register-resident plan of fwp_core.cuh.  Gate order in every array: 0 = i, 1 = u, 2 = o.
#include "fwp_core.cuh"

namespace fwp {

constexpr float kLstmEps = 1e-6f;

struct LstmFwdParams {
    Row4 z[3], k[3], v[3], beta[3], v_old[3], gate[3];
    Row4 out, nmz, cell;
    float* W[3]; long long wN[3], wH[3], wE[3];
    float* h; long long hN, hH;
    float* c; long long cN, cH;
    int H, L, D;
};

template <int D, int TC>
struct LstmFwdStage {
    Tile<D, TC, float> z[3], k[3], v[3];
    Tile<1, TC, float> b[3];
    static constexpr int kFloats = 9 * r4(TC * D) + 3 * r4(TC);
    __device__ __forceinline__ void bind(float* mem) {
#pragma unroll
        for (int g = 0; g < 3; g++) {
            z[g].bind(mem); mem += r4(TC * D);
            k[g].bind(mem); mem += r4(TC * D);
            v[g].bind(mem); mem += r4(TC * D);
        }
#pragma unroll
        for (int g = 0; g < 3; g++) { b[g].bind(mem); mem += r4(TC); }
    }
};

template <int D, int SPLIT, int TC, int VAR>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) lstm_fwd_kernel(const LstmFwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = LstmFwdStage<D, TC>;
    constexpr int kX = D + 16;
    for (int i = g.tid; i < 2 * Stage::kFloats + 2 * kX; i += G::NT) smem[i] = 0.f;
    float* xch = smem + 2 * Stage::kFloats;

    Src<float> sz[3], sk[3], sv[3], sb[3];
#pragma unroll
    for (int a = 0; a < 3; a++) {
        sz[a].init(p.z[a], n, h, p.D);
        sk[a].init(p.k[a], n, h, p.D);
        sv[a].init(p.v[a], n, h, p.D);
        sb[a].init(p.beta[a], n, h, 1);
    }
    f2 S[3][G::NP];
#pragma unroll
    for (int a = 0; a < 3; a++) load_cols(g, S[a], p.W[a] + n * p.wN[a] + h * p.wH[a], p.wE[a], p.D, p.D);
    const bool ok = g.idx < p.D;
    float* hp = p.h + n * p.hN + h * p.hH;
    float* cp = p.c + n * p.cN + h * p.cH;
    float hv = ok ? hp[g.idx] : 0.f;
    float cv = ok ? cp[g.idx] : 0.f;
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int c) {
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
#pragma unroll
        for (int a = 0; a < 3; a++) {
            s.z[a].template load<G::NT>(sz[a], t0, nt, g.tid);
            s.k[a].template load<G::NT>(sk[a], t0, nt, g.tid);
            s.v[a].template load<G::NT>(sv[a], t0, nt, g.tid);
            s.b[a].template load<G::NT>(sb[a], t0, nt, g.tid);
        }
        cp_async_commit();
    };
    issue(0);
    // running output pointers of this thread's column (threads that store nothing keep a valid address)
    const bool writer = ok && g.s == 0;
    const int col = writer ? g.idx : 0;
    auto colptr = [&](const Row4& r) { return reinterpret_cast<float*>(r.p) + n * r.sN + h * r.sH + col; };
    float* po = colptr(p.out);
    float* pc = colptr(p.cell);
    float* pg[3] = {colptr(p.gate[0]), colptr(p.gate[1]), colptr(p.gate[2])};
    float* pvo[3] = {colptr(p.v_old[0]), colptr(p.v_old[1]), colptr(p.v_old[2])};
    float* pnm = VAR == 1 ? po : colptr(p.nmz);
    const long long snm = VAR == 1 ? 0 : p.nmz.sL;
    int par = 0;
    for (int c = 0; c < nchunks; c++) {
        if (c + 1 < nchunks) { issue(c + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int nt = min(TC, p.L - c * TC);
        // the nine tiles of a stage lie r4(TC * D) floats apart (z, k, v of gate 0, then gate 1, gate 2)
        constexpr int kTile = r4(TC * D);
        const float* zcol = s.z[0].f + g.idx;          // + (3 a + 0) kTile: z of gate a ; + (3 a + 2) kTile: v
        const float* krow = s.k[0].f + g.off;          // + 3 a kTile: k of gate a
        const float* brow = s.b[0].f;                  // + a r4(TC): beta of gate a
#pragma unroll 1
        for (int t = 0; t < nt; t++, zcol += D, krow += D, brow++) {
            float* xv = xch + par * kX;
            float* slot = xv + D;
            par ^= 1;
            // the fed-back vector x_t, published for the slice reads below
            float xe, inv = 1.f;
            if constexpr (VAR == 1) {
                xe = hv;
            } else {
                const float mx = cta_allreduce_idx<G, true>(g, ok ? hv : -INFINITY, slot);
                xe = ok ? exp_neg(hv - mx) : 0.f;
                const float den = softmax_den(g, xe, slot + 8);
                inv = rcp_approx(den + kLstmEps);
                xe *= inv;
            }
            if (g.s == 0) xv[g.idx] = xe;
            cta_sync<G::WPS>();
            f2 xs[G::NP];
            lds_slice<G::NR>(xs, xv + g.off);
            float pre[3], vo[3];
#pragma unroll
            for (int a = 0; a < 3; a++) {
                f2 kk[G::NP];
                lds_slice<G::NR>(kk, krow + 3 * a * kTile);
                vo[a] = reduce_split<SPLIT>(dot2<G::NP>(S[a], kk));
                const float u = brow[a * r4(TC)] * (zcol[(3 * a + 2) * kTile] - vo[a]);
                axpy2<G::NP>(S[a], kk, u);
                pre[a] = reduce_split<SPLIT>(dot2<G::NP>(S[a], xs)) + zcol[3 * a * kTile];
            }
            const float gi = sigmoidf_(pre[0]);
            const float uu = (VAR == 4) ? pre[1] : sigmoidf_(pre[1]);
            const float go = sigmoidf_(pre[2]);
            cv = gi * uu + (1.f - gi) * cv;
            float hn = go * cv;
            if constexpr (VAR == 1) {
                const float mx = cta_allreduce_idx<G, true>(g, ok ? hn : -INFINITY, slot);
                const float ex = ok ? exp_neg(hn - mx) : 0.f;
                hn = ex * rcp_approx(softmax_den(g, ex, slot + 8));
            } else if constexpr (VAR == 3) {
                hn += zcol[3 * kTile];
            }
            hv = hn;
            if (writer) {
                *po = hn;
                *pc = cv;
                *pg[0] = gi;
                *pg[1] = uu;
                *pg[2] = go;
#pragma unroll
                for (int a = 0; a < 3; a++) *pvo[a] = vo[a];
                if constexpr (VAR != 1) *pnm = xe;
            }
            po += p.out.sL; pc += p.cell.sL; pnm += snm;
#pragma unroll
            for (int a = 0; a < 3; a++) { pg[a] += p.gate[a].sL; pvo[a] += p.v_old[a].sL; }
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 3; a++) store_cols(g, S[a], p.W[a] + n * p.wN[a] + h * p.wH[a], p.wE[a], p.D, p.D);
    if (ok && g.s == 0) { hp[g.idx] = hv; cp[g.idx] = cv; }
}

// ------------------------------------------------------------------ backward
struct LstmBwdParams {
    Row4 k[3], v[3], beta[3], v_old[3], gate[3];
    Row4 gy, out, od, cell, umc;
    Row4 gz[3], gk[3], gv[3], gb[3];
    float* W[3]; long long wN[3], wH[3], wE[3];
    int H, L, D;
};

template <int D, int TC>
struct LstmBwdStage {
    Tile<D, TC, float> k[3], v[3], vo[3], gate[3], gy, out, od, cell, umc;
    Tile<1, TC, float> b[3];
    static constexpr int kFloats = 17 * r4(TC * D) + 3 * r4(TC);
    __device__ __forceinline__ void bind(float* mem) {
#pragma unroll
        for (int g = 0; g < 3; g++) {
            k[g].bind(mem); mem += r4(TC * D);
            v[g].bind(mem); mem += r4(TC * D);
            vo[g].bind(mem); mem += r4(TC * D);
            gate[g].bind(mem); mem += r4(TC * D);
        }
        gy.bind(mem); mem += r4(TC * D);
        out.bind(mem); mem += r4(TC * D);
        od.bind(mem); mem += r4(TC * D);
        cell.bind(mem); mem += r4(TC * D);
        umc.bind(mem); mem += r4(TC * D);
#pragma unroll
        for (int g = 0; g < 3; g++) { b[g].bind(mem); mem += r4(TC); }
    }
};

template <int D, int SPLIT, int TC, int VAR>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) lstm_bwd_kernel(const LstmBwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = LstmBwdStage<D, TC>;
    constexpr int kXs = 9 * D + 48;      // per parity: dz[3][D], u[3][D], br[3][D], slots
    for (int i = g.tid; i < 2 * Stage::kFloats + 2 * kXs; i += G::NT) smem[i] = 0.f;
    float* xch = smem + 2 * Stage::kFloats;

    Src<float> sk[3], sv[3], so[3], sgt[3], sb[3], sgy, sout, sod, sc, sumc;
#pragma unroll
    for (int a = 0; a < 3; a++) {
        sk[a].init(p.k[a], n, h, p.D);
        sv[a].init(p.v[a], n, h, p.D);
        so[a].init(p.v_old[a], n, h, p.D);
        sgt[a].init(p.gate[a], n, h, p.D);
        sb[a].init(p.beta[a], n, h, 1);
    }
    sgy.init(p.gy, n, h, p.D);
    sout.init(p.out, n, h, p.D);
    sod.init(p.od, n, h, p.D);
    sc.init(p.cell, n, h, p.D);
    sumc.init(p.umc, n, h, p.D);

    f2 Sr[3][G::NP], Gr[3][G::NP], Gc[3][G::NP];
#pragma unroll
    for (int a = 0; a < 3; a++) {
        load_rows(g, Sr[a], p.W[a] + n * p.wN[a] + h * p.wH[a], p.wE[a], p.D, p.D);
#pragma unroll
        for (int i = 0; i < G::NP; i++) { Gr[a][i] = 0ull; Gc[a][i] = 0ull; }
    }
    float gh = 0.f, gc = 0.f;
    const bool ok = g.idx < p.D;
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {
        Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
#pragma unroll
        for (int a = 0; a < 3; a++) {
            s.k[a].template load<G::NT>(sk[a], t0, nt, g.tid);
            s.v[a].template load<G::NT>(sv[a], t0, nt, g.tid);
            s.vo[a].template load<G::NT>(so[a], t0, nt, g.tid);
            s.gate[a].template load<G::NT>(sgt[a], t0, nt, g.tid);
            s.b[a].template load<G::NT>(sb[a], t0, nt, g.tid);
        }
        s.gy.template load<G::NT>(sgy, t0, nt, g.tid);
        if (VAR == 1) s.out.template load<G::NT>(sout, t0, nt, g.tid);
        s.od.template load<G::NT>(sod, t0, nt, g.tid);
        s.cell.template load<G::NT>(sc, t0, nt, g.tid);
        s.umc.template load<G::NT>(sumc, t0, nt, g.tid);
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
            float* xdz = xch + par * kXs;       // [3][D]
            float* xu = xdz + 3 * D;            // [3][D]
            float* xbr = xu + 3 * D;            // [3][D]
            float* slot = xbr + 3 * D;          // [6][8]
            par ^= 1;
            const int o = t * D + g.idx;
            // ---- element-wise part (idx = m)
            const float gsum = s.gy.f[o] + gh;
            float a = gsum;
            if constexpr (VAR == 1) {
                const float hm = s.out.f[o];
                const float dotp = cta_allreduce_idx<G, false>(g, hm * gsum, slot);
                a = hm * (gsum - dotp);
            }
            const float gi = s.gate[0].f[o], uu = s.gate[1].f[o], go = s.gate[2].f[o];
            float dz[3];
            dz[2] = (s.cell.f[o] * a) * (1.f - go) * go;
            gc += go * a;
            dz[0] = (gc * s.umc.f[o]) * (1.f - gi) * gi;
            dz[1] = gc * gi;
            if constexpr (VAR != 4) dz[1] = dz[1] * (1.f - uu) * uu;
            gc *= (1.f - gi);
            // ---- column role, one delta block per gate
            f2 xs[G::NP];
            lds_slice<G::NR>(xs, s.od.f + t * D + g.off);
#pragma unroll
            for (int q = 0; q < 3; q++) {
                f2 kk[G::NP];
                lds_slice<G::NR>(kk, s.k[q].f + t * D + g.off);
                const float beta = s.b[q].f[t];
                const float w = s.v[q].f[o] - s.vo[q].f[o];
                axpy2<G::NP>(Gc[q], xs, dz[q]);
                const float r = reduce_split<SPLIT>(dot2<G::NP>(Gc[q], kk));
                const float br = beta * r;
                axpy2<G::NP>(Gc[q], kk, -br);
                const float pw = warp_sum_idx<SPLIT>(r * w);
                if (g.s == 0) {
                    xdz[q * D + g.idx] = dz[q];
                    xu[q * D + g.idx] = beta * w;
                    xbr[q * D + g.idx] = br;
                    if (ok) {
                        put<float>(p.gv[q], n, h, t0 + t, g.idx, br);
                        put<float>(p.gz[q], n, h, t0 + t, g.idx, (VAR == 3 && q == 1) ? dz[q] + gsum : dz[q]);
                    }
                }
                if (g.lane == 0) slot[8 + q * 8 + g.warp] = pw;
            }
            cta_sync<G::WPS>();
            // ---- row role
            {
                const float xe = s.od.f[o];
                float ghn = 0.f;
#pragma unroll
                for (int q = 0; q < 3; q++) {
                    f2 dr[G::NP], ur[G::NP], brr[G::NP];
                    lds_slice<G::NR>(dr, xdz + q * D + g.off);
                    lds_slice<G::NR>(ur, xu + q * D + g.off);
                    lds_slice<G::NR>(brr, xbr + q * D + g.off);
                    const float ke = s.k[q].f[o];
                    ghn += dot2<G::NP>(Sr[q], dr);
                    axpy2<G::NP>(Gr[q], dr, xe);
                    float dk = dot2<G::NP>(Gr[q], ur);
                    axpy2<G::NP>(Sr[q], ur, -ke);
                    dk -= dot2<G::NP>(Sr[q], brr);
                    axpy2<G::NP>(Gr[q], brr, -ke);
                    dk = reduce_split<SPLIT>(dk);
                    if (ok && g.s == 0) put<float>(p.gk[q], n, h, t0 + t, g.idx, dk);
                    if (g.tid == 0) {
                        float db = slot[8 + q * 8];
#pragma unroll
                        for (int w2 = 1; w2 < G::WPS; w2++) db += slot[8 + q * 8 + w2];
                        put<float>(p.gb[q], n, h, t0 + t, 0, db);
                    }
                }
                ghn = reduce_split<SPLIT>(ghn);
                if constexpr (VAR != 1) {
                    const float dotp = cta_allreduce_idx<G, false>(g, xe * ghn, slot + 32);
                    ghn = xe * (ghn - dotp);
                }
                gh = ghn;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 3; a++) store_rows(g, Sr[a], p.W[a] + n * p.wN[a] + h * p.wH[a], p.wE[a], p.D, p.D);
}

}  // namespace fwp
#include "fwp_lstm_roles.cuh"
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

template <int D, int SPLIT, int TC, int VAR>
static int launch_lstm_fwd(const LstmFwdParams& p, int nseq, cudaStream_t st) {
    auto kern = lstm_fwd_kernel<D, SPLIT, TC, VAR>;
    const size_t bytes = (2 * LstmFwdStage<D, TC>::kFloats + 2 * (D + 16)) * sizeof(float);
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    if (int rc = smem_optin(kern, bytes * slots)) return rc;
    kern<<<nseq / slots, D * SPLIT * slots, bytes * slots, st>>>(p);
    count_launch();
    note_kernel("lstm_fwd_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int D, int SPLIT, int TC, int VAR>
static int launch_lstm_bwd(const LstmBwdParams& p, int nseq, cudaStream_t st) {
    auto kern = lstm_bwd_kernel<D, SPLIT, TC, VAR>;
    const size_t bytes = (2 * LstmBwdStage<D, TC>::kFloats + 2 * (9 * D + 48)) * sizeof(float);
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    if (int rc = smem_optin(kern, bytes * slots)) return rc;
    kern<<<nseq / slots, D * SPLIT * slots, bytes * slots, st>>>(p);
    count_launch();
    note_kernel("lstm_bwd_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int VAR>
static int launch_lstm_bwd_roles32(const LstmBwdParams& p, int nseq, cudaStream_t st) {
    constexpr int TC = 8;
    auto kern = lstm_bwd_roles32_kernel<TC, VAR>;
    const int slots = nseq % 2 ? 1 : 2;
    const size_t bytes = (size_t)LstmRolesSmem<TC>::kFloats * sizeof(float) * slots;
    if (int rc = smem_optin(kern, bytes)) return rc;
    kern<<<nseq / slots, 128 * slots, bytes, st>>>(p);
    count_launch();
    note_kernel("lstm_bwd_roles32_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int VAR>
static int launch_lstm_fwd_gates32(const LstmFwdParams& p, int nseq, cudaStream_t st) {
    constexpr int TC = 16;
    auto kern = lstm_fwd_gates32_kernel<TC, VAR>;
    int slots = 4;
    while (nseq % slots) slots >>= 1;
    const size_t bytes = (size_t)LstmGatesSmem<TC>::kFloats * sizeof(float) * slots;
    if (int rc = smem_optin(kern, bytes)) return rc;
    kern<<<nseq / slots, 96 * slots, bytes, st>>>(p);
    count_launch();
    note_kernel("lstm_fwd_gates32_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int VAR>
static int dispatch_lstm_fwd(const LstmFwdParams& p, int nseq, cudaStream_t st) {
    switch (pad_dim(p.D)) {
        case 16: return launch_lstm_fwd<16, 2, 16, VAR>(p, nseq, st);
        case 32: {
            bool fast = p.D == 32 && tune_get(T_LSTM_FWD_GATES32, 1);       // full width, 16-byte aligned rows
            for (int a = 0; a < 3 && fast; a++)
                fast = rows_16B_aligned(p.z[a]) && rows_16B_aligned(p.k[a]) && rows_16B_aligned(p.v[a]);
            if (fast) return launch_lstm_fwd_gates32<VAR>(p, nseq, st);
            const int sp = tune_get(T_LSTM_FWD_SPLIT32, 1);
            // measured (512 sequences x 512 steps): 1 -> 0.78 ms, 4 -> 0.83 ms, 2 -> 0.85 ms
            if (sp == 2) return launch_lstm_fwd<32, 2, 8, VAR>(p, nseq, st);
            if (sp == 4) return launch_lstm_fwd<32, 4, 8, VAR>(p, nseq, st);
            return launch_lstm_fwd<32, 1, 8, VAR>(p, nseq, st);
        }
        case 64: return launch_lstm_fwd<64, 4, 4, VAR>(p, nseq, st);
    }
    return FWP_ERR_UNSUPPORTED;
}

template <int VAR>
static int dispatch_lstm_bwd(const LstmBwdParams& p, int nseq, cudaStream_t st) {
    switch (pad_dim(p.D)) {
        case 16: return launch_lstm_bwd<16, 2, 8, VAR>(p, nseq, st);
        case 32: {
            bool fast = p.D == 32 && tune_get(T_LSTM_BWD_ROLES32, 1);      // full width, 16-byte aligned rows
            for (int a = 0; a < 3 && fast; a++)
                fast = rows_16B_aligned(p.k[a]) && rows_16B_aligned(p.v[a]) && rows_16B_aligned(p.v_old[a]) &&
                       rows_16B_aligned(p.gate[a]);
            fast = fast && rows_16B_aligned(p.gy) && rows_16B_aligned(p.od) && rows_16B_aligned(p.cell) &&
                   rows_16B_aligned(p.umc) && (VAR != 1 || rows_16B_aligned(p.out));
            if (fast) return launch_lstm_bwd_roles32<VAR>(p, nseq, st);
            const int sp = tune_get(T_LSTM_BWD_SPLIT32, 2);
            // measured: 2 -> 1.37 ms, 4 -> 2.14 ms
            if (sp == 4) return launch_lstm_bwd<32, 4, 4, VAR>(p, nseq, st);
            return launch_lstm_bwd<32, 2, 4, VAR>(p, nseq, st);
        }
        case 64: return launch_lstm_bwd<64, 4, 2, VAR>(p, nseq, st);
    }
    return FWP_ERR_UNSUPPORTED;
}

static int check3(const fwp_tensor* t, bool required = true) {
    if (!t) return FWP_ERR_NULL;
    for (int a = 0; a < 3; a++)
        if (int rc = check_tensor(t + a, 4, required)) return rc;
    return FWP_OK;
}

static void set_w(float** W, long long* wN, long long* wH, long long* wE, const fwp_tensor* kv) {
    for (int a = 0; a < 3; a++) {
        W[a] = (float*)kv[a].data;
        wN[a] = kv[a].stride[0]; wH[a] = kv[a].stride[1]; wE[a] = kv[a].stride[2];
    }
}

}  // namespace fwp

using namespace fwp;

FWP_API int fwp_fast_lstm_forward(int variant, int N, int H, int L, int D,
                                  const fwp_tensor Z[3], const fwp_tensor K[3],
                                  const fwp_tensor V[3], const fwp_tensor beta[3],
                                  const fwp_tensor* states, const fwp_tensor* cells,
                                  const fwp_tensor kv[3],
                                  const fwp_tensor* out, const fwp_tensor* out_del_nmz,
                                  const fwp_tensor* cell_out,
                                  const fwp_tensor gates[3], const fwp_tensor v_old[3],
                                  int io_dtype, void* stream, int device) {
    if (variant < 1 || variant > 4) return FWP_ERR_VARIANT;
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32) return FWP_ERR_DTYPE;
    if (!pad_dim(D)) return FWP_ERR_UNSUPPORTED;
    int rc;
    if ((rc = check3(Z)) || (rc = check3(K)) || (rc = check3(V)) || (rc = check3(beta)) || (rc = check3(kv)) ||
        (rc = check3(gates)) || (rc = check3(v_old)) || (rc = check_tensor(states, 4, true)) ||
        (rc = check_tensor(cells, 4, true)) || (rc = check_tensor(out, 4, true)) ||
        (rc = check_tensor(cell_out, 4, true)) || (rc = check_tensor(out_del_nmz, 4, variant != 1)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    LstmFwdParams p;
    for (int a = 0; a < 3; a++) {
        p.z[a] = row4(Z + a); p.k[a] = row4(K + a); p.v[a] = row4(V + a); p.beta[a] = row4(beta + a);
        p.v_old[a] = row4(v_old + a); p.gate[a] = row4(gates + a);
    }
    p.out = row4(out); p.nmz = row4(out_del_nmz); p.cell = row4(cell_out);
    set_w(p.W, p.wN, p.wH, p.wE, kv);
    p.h = (float*)states->data; p.hN = states->stride[0]; p.hH = states->stride[1];
    p.c = (float*)cells->data; p.cN = cells->stride[0]; p.cH = cells->stride[1];
    p.H = H; p.L = L; p.D = D;
    cudaStream_t st = (cudaStream_t)stream;
    switch (variant) {
        case 1: return dispatch_lstm_fwd<1>(p, N * H, st);
        case 2: return dispatch_lstm_fwd<2>(p, N * H, st);
        case 3: return dispatch_lstm_fwd<3>(p, N * H, st);
        default: return dispatch_lstm_fwd<4>(p, N * H, st);
    }
}

FWP_API int fwp_fast_lstm_backward(int variant, int N, int H, int L, int D,
                                   const fwp_tensor* grad_out,
                                   const fwp_tensor K[3], const fwp_tensor V[3], const fwp_tensor beta[3],
                                   const fwp_tensor v_old[3],
                                   const fwp_tensor* out, const fwp_tensor* out_delayed,
                                   const fwp_tensor* cell_out, const fwp_tensor* u_minus_c,
                                   const fwp_tensor gates[3], const fwp_tensor kv[3],
                                   const fwp_tensor grad_Z[3], const fwp_tensor grad_K[3],
                                   const fwp_tensor grad_V[3], const fwp_tensor grad_beta[3],
                                   int io_dtype, void* stream, int device) {
    if (variant < 1 || variant > 4) return FWP_ERR_VARIANT;
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32) return FWP_ERR_DTYPE;
    if (!pad_dim(D)) return FWP_ERR_UNSUPPORTED;
    int rc;
    if ((rc = check3(K)) || (rc = check3(V)) || (rc = check3(beta)) || (rc = check3(v_old)) || (rc = check3(gates)) ||
        (rc = check3(kv)) || (rc = check3(grad_Z)) || (rc = check3(grad_K)) || (rc = check3(grad_V)) ||
        (rc = check3(grad_beta)) || (rc = check_tensor(grad_out, 4, true)) ||
        (rc = check_tensor(out, 4, variant == 1)) || (rc = check_tensor(out_delayed, 4, true)) ||
        (rc = check_tensor(cell_out, 4, true)) || (rc = check_tensor(u_minus_c, 4, true)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    LstmBwdParams p;
    for (int a = 0; a < 3; a++) {
        p.k[a] = row4(K + a); p.v[a] = row4(V + a); p.beta[a] = row4(beta + a); p.v_old[a] = row4(v_old + a);
        p.gate[a] = row4(gates + a);
        p.gz[a] = row4(grad_Z + a); p.gk[a] = row4(grad_K + a); p.gv[a] = row4(grad_V + a); p.gb[a] = row4(grad_beta + a);
    }
    p.gy = row4(grad_out); p.out = row4(out); p.od = row4(out_delayed); p.cell = row4(cell_out); p.umc = row4(u_minus_c);
    set_w(p.W, p.wN, p.wH, p.wE, kv);
    p.H = H; p.L = L; p.D = D;
    cudaStream_t st = (cudaStream_t)stream;
    switch (variant) {
        case 1: return dispatch_lstm_bwd<1>(p, N * H, st);
        case 2: return dispatch_lstm_bwd<2>(p, N * H, st);
        case 3: return dispatch_lstm_bwd<3>(p, N * H, st);
        default: return dispatch_lstm_bwd<4>(p, N * H, st);
    }
}
