// Delta-rule fast weight memory, forward and fused backward (sm_100a).
//
//   v_old_t = S_{t-1}^T k_t ; u_t = beta_t (v_t - v_old_t) ; S_t = S_{t-1} + k_t (x) u_t ; y_t = S_t^T q_t
//
// Restates the math of the reference's algorithmic/fast_weight/fast_weight_cuda.cu
// (forward kernel :17-178, backward kernels :244-560) with a different execution
// plan: the matrix never leaves registers, every reduction is thread-local plus
// at most two shuffles, outputs are plain stores, and the backward is one pass.
// The same file holds the sum rule (causal_product_cuda.cu), which is the delta
// rule without beta and v_old.
#include "fwp_delta_params.cuh"

namespace fwp {


template <int D, int TC, typename T>
struct FwdStage {
    Tile<D, TC, T> q, k, v;
    Tile<1, TC, T> b;
    static constexpr int kFloats = 3 * r4(Tile<D, TC, T>::kFloats) + r4(Tile<1, TC, T>::kFloats);
    __device__ __forceinline__ void bind(float* mem) {
        q.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        k.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        v.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        b.bind(mem);
    }
};

// SUM = true drops beta / v_old (sum rule): S_t = S_{t-1} + k_t (x) v_t.
template <int D, int SPLIT, int TC, typename T, bool SUM>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT), D == 64 ? 4 : 1)
delta_fwd_step_kernel(const DeltaFwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = FwdStage<D, TC, T>;
    for (int i = g.tid; i < 2 * Stage::kFloats; i += G::NT) smem[i] = 0.f;
    griddep_wait();               // launched as a dependent: global memory is touched from here on
    griddep_launch_dependents();

    Src<T> sq, sk, sv, sb;
    sq.init(p.q, n, h, p.E);
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    if (!SUM) sb.init(p.beta, n, h, 1);

    float* W = p.W + n * p.wN + h * p.wH;
    f2 S[G::NP];
    load_cols(g, S, W, p.wE, p.E, p.M);
    __syncthreads();   // zero-fill done before any copy lands

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int c) {
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.q.template load<G::NT>(sq, t0, nt, g.tid);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        if (!SUM) s.b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    issue(0);
    const bool col_ok = g.idx < p.M;
    for (int c = 0; c < nchunks; c++) {
        if (c + 1 < nchunks) { issue(c + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        if constexpr (sizeof(T) != 4) {
            s.q.widen(nt, p.E, g.tid, G::NT);
            s.k.widen(nt, p.E, g.tid, G::NT);
            s.v.widen(nt, p.M, g.tid, G::NT);
            if (!SUM) s.b.widen(nt, 1, g.tid, G::NT);
            __syncthreads();
        }
#pragma unroll 2
        for (int t = 0; t < nt; t++) {
            f2 kk[G::NP], qq[G::NP];
            lds_slice<G::NR>(kk, s.k.f + t * D + g.off);
            lds_slice<G::NR>(qq, s.q.f + t * D + g.off);
            const float vv = s.v.f[t * D + g.idx];
            float u, vo = 0.f;
            if constexpr (SUM) {
                u = vv;
            } else {
                vo = reduce_split<SPLIT>(dot2<G::NP>(S, kk));
                u = s.b.f[t] * (vv - vo);
            }
            axpy2<G::NP>(S, kk, u);
            const float y = reduce_split<SPLIT>(dot2<G::NP>(S, qq));
            if (col_ok && g.s == 0) {
                put<T>(p.out, n, h, t0 + t, g.idx, y);
                if constexpr (!SUM) {
                    put<float>(p.v_old, n, h, t0 + t, g.idx, vo);
                    if (p.v_ins.p) put<float>(p.v_ins, n, h, t0 + t, g.idx, u);
                }
            }
        }
        __syncthreads();   // stage may be refilled by the next iteration's issue
    }
    store_cols(g, S, W, p.wE, p.E, p.M);
}

// ------------------------------------------------------------------ backward

template <int D, int TC, typename T>
struct BwdStage {
    Tile<D, TC, T> q, k, v, gy;
    Tile<D, TC, float> vo;
    Tile<1, TC, T> b;
    static constexpr int kFloats = 4 * r4(Tile<D, TC, T>::kFloats) + r4(Tile<D, TC, float>::kFloats) +
                                   r4(Tile<1, TC, T>::kFloats);
    __device__ __forceinline__ void bind(float* mem) {
        q.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        k.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        v.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        gy.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        vo.bind(mem); mem += r4(Tile<D, TC, float>::kFloats);
        b.bind(mem);
    }
};

// Per step, walking time backwards with S = S_t (row role) and G = dL/dS_t kept
// twice (column role Gc for the reduction over e that sits on the dependency
// chain, row role Gr for the reductions over m that feed dk):
//   Gc += q (x) gy ; r = Gc^T k ; dv = beta r ; dbeta = r . (v - v_old) ; Gc -= k (x) beta r
//   dq = S gy ; Gr += q (x) gy ; dk = Gr u ; S -= k (x) u ; dk -= S (beta r) ; Gr -= k (x) beta r
template <int D, int SPLIT, int TC, typename T>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) delta_bwd_step_kernel(const DeltaBwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = BwdStage<D, TC, T>;
    constexpr int kXch = 2 * (2 * D + 8);   // per parity: u[D], br[D], dbeta partials[WPS<=8]
    for (int i = g.tid; i < 2 * Stage::kFloats + kXch; i += G::NT) smem[i] = 0.f;
    float* xch = smem + 2 * Stage::kFloats;
    griddep_wait();               // launched as a dependent: global memory is touched from here on
    griddep_launch_dependents();

    Src<T> sq, sk, sv, sg, sb;
    Src<float> so;
    sq.init(p.q, n, h, p.E);
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    sg.init(p.gy, n, h, p.M);
    so.init(p.v_old, n, h, p.M);
    sb.init(p.beta, n, h, 1);

    float* W = p.W + n * p.wN + h * p.wH;
    f2 Sr[G::NP], Gr[G::NP], Gc[G::NP];
    load_rows(g, Sr, W, p.wE, p.E, p.M);
#pragma unroll
    for (int i = 0; i < G::NP; i++) { Gr[i] = 0ull; Gc[i] = 0ull; }
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {   // j-th chunk counted from the end of the sequence
        Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.q.template load<G::NT>(sq, t0, nt, g.tid);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        s.gy.template load<G::NT>(sg, t0, nt, g.tid);
        s.vo.template load<G::NT>(so, t0, nt, g.tid);
        s.b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    issue(0);
    const bool col_ok = g.idx < p.M, row_ok = g.idx < p.E;
    int par = 0;
    for (int j = 0; j < nchunks; j++) {
        if (j + 1 < nchunks) { issue(j + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        if constexpr (sizeof(T) != 4) {
            s.q.widen(nt, p.E, g.tid, G::NT);
            s.k.widen(nt, p.E, g.tid, G::NT);
            s.v.widen(nt, p.M, g.tid, G::NT);
            s.gy.widen(nt, p.M, g.tid, G::NT);
            s.b.widen(nt, 1, g.tid, G::NT);
            __syncthreads();
        }
        for (int t = nt - 1; t >= 0; t--) {
            float* xu = xch + par * (2 * D + 8);
            float* xbr = xu + D;
            float* xdb = xbr + D;
            par ^= 1;
            const float beta = s.b.f[t];
            // ---- column role
            {
                f2 kk[G::NP], qq[G::NP];
                lds_slice<G::NR>(qq, s.q.f + t * D + g.off);
                lds_slice<G::NR>(kk, s.k.f + t * D + g.off);
                const float gym = s.gy.f[t * D + g.idx];
                const float w = s.v.f[t * D + g.idx] - s.vo.f[t * D + g.idx];
                axpy2<G::NP>(Gc, qq, gym);
                const float r = reduce_split<SPLIT>(dot2<G::NP>(Gc, kk));
                const float br = beta * r;
                axpy2<G::NP>(Gc, kk, -br);
                float pw = warp_sum_idx<SPLIT>(r * w);
                if (g.s == 0) {
                    xu[g.idx] = beta * w;
                    xbr[g.idx] = br;
                    if (col_ok) put<T>(p.gv, n, h, t0 + t, g.idx, br);
                }
                if (G::WPS > 1 && g.lane == 0) xdb[g.warp] = pw;
                if (G::WPS == 1 && g.tid == 0) put<T>(p.gb, n, h, t0 + t, 0, pw);
            }
            cta_sync<G::WPS>();
            // ---- row role
            {
                f2 gr[G::NP], ur[G::NP], brr[G::NP];
                lds_slice<G::NR>(gr, s.gy.f + t * D + g.off);
                lds_slice<G::NR>(ur, xu + g.off);
                lds_slice<G::NR>(brr, xbr + g.off);
                const float qe = s.q.f[t * D + g.idx], ke = s.k.f[t * D + g.idx];
                float dq = dot2<G::NP>(Sr, gr);
                axpy2<G::NP>(Gr, gr, qe);
                float dk = dot2<G::NP>(Gr, ur);
                axpy2<G::NP>(Sr, ur, -ke);
                dk -= dot2<G::NP>(Sr, brr);
                axpy2<G::NP>(Gr, brr, -ke);
                dq = reduce_split<SPLIT>(dq);
                dk = reduce_split<SPLIT>(dk);
                if (row_ok && g.s == 0) {
                    put<T>(p.gq, n, h, t0 + t, g.idx, dq);
                    put<T>(p.gk, n, h, t0 + t, g.idx, dk);
                }
                if (G::WPS > 1 && g.tid == 0) {
                    float db = xdb[0];
#pragma unroll
                    for (int w2 = 1; w2 < G::WPS; w2++) db += xdb[w2];
                    put<T>(p.gb, n, h, t0 + t, 0, db);
                }
            }
        }
        __syncthreads();
    }
    store_rows(g, Sr, W, p.wE, p.E, p.M);
}

// sum-rule backward: dq_t = S_t gy_t with S accumulated forwards from zero,
// dk_t = G_t v_t, dv_t = G_t^T k_t with G accumulated backwards (causal_product_cuda.cu:369-445).
struct SumBwdParams {
    Row4 q, k, v, gy, gq, gk, gv;
    int H, L, E, M;
    int NH;     // number of sequences (N*H)
};

template <int D, int TC, typename T>
struct SumStage {
    Tile<D, TC, T> q, k, v, gy;
    static constexpr int kFloats = 4 * r4(Tile<D, TC, T>::kFloats);
    __device__ __forceinline__ void bind(float* mem) {
        q.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        k.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        v.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        gy.bind(mem);
    }
};

template <int D, int SPLIT, int TC, typename T>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) sum_bwd_kernel(const SumBwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = SumStage<D, TC, T>;
    for (int i = g.tid; i < 2 * Stage::kFloats; i += G::NT) smem[i] = 0.f;
    Src<T> sq, sk, sv, sg;
    sq.init(p.q, n, h, p.E);
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    sg.init(p.gy, n, h, p.M);
    __syncthreads();
    const int nchunks = (p.L + TC - 1) / TC;
    const bool col_ok = g.idx < p.M, row_ok = g.idx < p.E;
    // phase 0: forwards, S row role, dq.  phase 1: backwards, G in both roles, dk and dv.
    for (int phase = 0; phase < 2; phase++) {
        f2 A[G::NP], B[G::NP];
#pragma unroll
        for (int i = 0; i < G::NP; i++) { A[i] = 0ull; B[i] = 0ull; }
        auto issue = [&](int j) {
            Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
            const int c = phase ? nchunks - 1 - j : j;
            const int t0 = c * TC, nt = min(TC, p.L - t0);
            s.q.template load<G::NT>(sq, t0, nt, g.tid);
            s.k.template load<G::NT>(sk, t0, nt, g.tid);
            s.v.template load<G::NT>(sv, t0, nt, g.tid);
            s.gy.template load<G::NT>(sg, t0, nt, g.tid);
            cp_async_commit();
        };
        issue(0);
        for (int j = 0; j < nchunks; j++) {
            if (j + 1 < nchunks) { issue(j + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
            __syncthreads();
            Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
            const int c = phase ? nchunks - 1 - j : j;
            const int t0 = c * TC, nt = min(TC, p.L - t0);
            if constexpr (sizeof(T) != 4) {
                s.q.widen(nt, p.E, g.tid, G::NT);
                s.k.widen(nt, p.E, g.tid, G::NT);
                s.v.widen(nt, p.M, g.tid, G::NT);
                s.gy.widen(nt, p.M, g.tid, G::NT);
                __syncthreads();
            }
            for (int i = 0; i < nt; i++) {
                const int t = phase ? nt - 1 - i : i;
                if (phase == 0) {
                    f2 vr[G::NP], gr[G::NP];
                    lds_slice<G::NR>(vr, s.v.f + t * D + g.off);
                    lds_slice<G::NR>(gr, s.gy.f + t * D + g.off);
                    axpy2<G::NP>(A, vr, s.k.f[t * D + g.idx]);
                    const float dq = reduce_split<SPLIT>(dot2<G::NP>(A, gr));
                    if (row_ok && g.s == 0) put<T>(p.gq, n, h, t0 + t, g.idx, dq);
                } else {
                    f2 vr[G::NP], gr[G::NP], kk[G::NP], qq[G::NP];
                    lds_slice<G::NR>(vr, s.v.f + t * D + g.off);
                    lds_slice<G::NR>(gr, s.gy.f + t * D + g.off);
                    lds_slice<G::NR>(kk, s.k.f + t * D + g.off);
                    lds_slice<G::NR>(qq, s.q.f + t * D + g.off);
                    axpy2<G::NP>(A, gr, s.q.f[t * D + g.idx]);        // row role G
                    axpy2<G::NP>(B, qq, s.gy.f[t * D + g.idx]);       // column role G
                    const float dk = reduce_split<SPLIT>(dot2<G::NP>(A, vr));
                    const float dv = reduce_split<SPLIT>(dot2<G::NP>(B, kk));
                    if (g.s == 0) {
                        if (row_ok) put<T>(p.gk, n, h, t0 + t, g.idx, dk);
                        if (col_ok) put<T>(p.gv, n, h, t0 + t, g.idx, dv);
                    }
                }
            }
            __syncthreads();
        }
    }
}


// The three gradients of the sum rule are independent prefix sums, so each gets warps of its own and the
// three run side by side: dq forwards over S (rows), dk backwards over G (rows), dv backwards over G (columns).
// Per step a role adds x[idx] * a[slice] to its matrix slice and writes the dot product with b[slice]:
//   dq: x = k, a = v,  b = gy;    dk: x = q, a = gy, b = v;    dv: x = gy, a = q, b = k.
// Threads of the CTA: [role][sequence slot][D * SPLIT]; every role stages its own three streams, three or four chunks deep
// (a chunk is 1 KB per stream and its arithmetic a few hundred cycles, so the copies have to run several chunks
// ahead to cover the memory latency), and all roles pass the same number of CTA-wide barriers per chunk.
template <typename T> __host__ __device__ constexpr int sum_stages() { return sizeof(T) == 4 ? 4 : 3; }
template <int D, int TC, typename T>
__host__ __device__ constexpr int sum_roles_floats() { return sum_stages<T>() * 3 * r4(Tile<D, TC, T>::kFloats) + 2 * TC * D; }   // per role and sequence
template <int D, int SPLIT, int TC, typename T>
__global__ void __launch_bounds__(3 * D * SPLIT * slots_for(D * SPLIT)) sum_bwd_roles_kernel(const SumBwdParams p) {
    using G = Geo<D, SPLIT>;
    using Tl = Tile<D, TC, T>;
    constexpr int TT = r4(Tl::kFloats), NST = sum_stages<T>(), PER = sum_roles_floats<D, TC, T>();
    const int per_role = blockDim.x / 3;
    const int role = threadIdx.x / per_role;
    const G g(threadIdx.x - role * per_role);
    const int nslots = per_role / G::NT;
    const int seq = blockIdx.x * nslots + g.slot;
    const int n = seq / p.H, h = seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = smem_all + (size_t)(g.slot * 3 + role) * PER;
    float* const otile = smem + NST * 3 * TT;      // two output tiles [TC][D], flushed a chunk at a time
    for (int i = g.tid; i < PER; i += G::NT) smem[i] = 0.f;
    // copies by value: a reference picked at run time would turn every later field access into an indexed
    // load from the parameter bank
    const Row4 rx = role == 0 ? p.k : role == 1 ? p.q : p.gy;
    const Row4 ra = role == 0 ? p.v : role == 1 ? p.gy : p.q;
    const Row4 rb = role == 0 ? p.gy : role == 1 ? p.v : p.k;
    const Row4 ro = role == 0 ? p.gq : role == 1 ? p.gk : p.gv;
    const int xw = role < 2 ? p.E : p.M, sw = role < 2 ? p.M : p.E;
    Src<T> sx, sa, sb;
    sx.init(rx, n, h, xw);
    sa.init(ra, n, h, sw);
    sb.init(rb, n, h, sw);
    __syncthreads();
    const int nchunks = (p.L + TC - 1) / TC;
    const bool rev = role != 0;
    const bool writes = g.s == 0;
    f2 A[G::NP];
#pragma unroll
    for (int i = 0; i < G::NP; i++) A[i] = 0ull;
    auto issue = [&](int j) {
        float* st = smem + (j % NST) * 3 * TT;
        Tl x, a, b;
        x.bind(st); a.bind(st + TT); b.bind(st + 2 * TT);
        const int c = rev ? nchunks - 1 - j : j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        x.template load<G::NT>(sx, t0, nt, g.tid);
        a.template load<G::NT>(sa, t0, nt, g.tid);
        b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    for (int j = 0; j < NST - 1; j++) {
        if (j < nchunks) issue(j); else cp_async_commit();
    }
    for (int j = 0; j < nchunks; j++) {
        // one group per iteration, empty past the end: chunk j is the NST-th youngest after this commit
        if (j + NST - 1 < nchunks) issue(j + NST - 1); else cp_async_commit();
        cp_async_wait<NST - 1>();
        __syncthreads();
        float* st = smem + (j % NST) * 3 * TT;
        Tl x, a, b;
        x.bind(st); a.bind(st + TT); b.bind(st + 2 * TT);
        const int c = rev ? nchunks - 1 - j : j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        if constexpr (sizeof(T) != 4) {
            x.widen(nt, xw, g.tid, G::NT);
            a.widen(nt, sw, g.tid, G::NT);
            b.widen(nt, sw, g.tid, G::NT);
            __syncthreads();
        }
        float* const ot = otile + (j & 1) * TC * D + g.idx;
        auto step = [&](int t) {
            f2 ar[G::NP], br[G::NP];
            lds_slice<G::NR>(ar, a.f + t * D + g.off);
            lds_slice<G::NR>(br, b.f + t * D + g.off);
            axpy2<G::NP>(A, ar, x.f[t * D + g.idx]);
            const float o = reduce_split<SPLIT>(dot2<G::NP>(A, br));
            if (writes) ot[t * D] = o;
        };
        if (nt == TC) {         // unrolled, so that the loads, shuffles and stores of neighbouring steps overlap
#pragma unroll
            for (int i = 0; i < TC; i++) step(rev ? TC - 1 - i : i);
        } else {
            for (int i = 0; i < nt; i++) step(rev ? nt - 1 - i : i);
        }
        __syncthreads();
        // this tile is written again two chunks on, behind the barriers of the next chunk
        flush_rows<D, G::NT, T, TC>(otile + (j & 1) * TC * D, ro, n, h, t0, nt, xw, g.tid);
    }
}

}  // namespace fwp

#include "fwp_delta_blocked.cuh"
#include "fwp_delta_generic.cuh"

namespace fwp {

// ------------------------------------------------------------------ launchers
template <int D, int SPLIT, int TC, typename T, bool SUM>
static int launch_fwd(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    constexpr int NSL = slots_for(D * SPLIT);
    return launch_dependent(delta_fwd_kernel<D, SPLIT, TC, T, SUM>, p, (nseq + NSL - 1) / NSL, NSL * (D * SPLIT + 32),
                  NSL * WsFwdSmem<D, TC, T>::kFloats * sizeof(float), st, "delta_fwd_kernel");
}
template <int D, int SPLIT, int TC, typename T, int PF = 2>
static int launch_bwd(const DeltaBwdParams& p, int nseq, cudaStream_t st) {
    constexpr int NSL = slots_for(D * SPLIT);
    return launch_dependent(delta_bwd_kernel<D, SPLIT, TC, T, PF>, p, (nseq + NSL - 1) / NSL, NSL * (2 * D * SPLIT + 32),
                  NSL * WsBwdSmem<D, TC, T, PF>::kFloats * sizeof(float), st, "delta_bwd_kernel");
}
template <int D, int SPLIT, int TC, typename T, bool SUM>
static int launch_fwd_step(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    // few sequences: rather one or two per CTA on twice or four times the SMs than four per CTA on a part of them
    if (tune_get(T_STEP_SPREAD, 1))
        while (slots > 1 && nseq / slots < sm_count()) slots >>= 1;
    return launch_dependent(delta_fwd_step_kernel<D, SPLIT, TC, T, SUM>, p, nseq / slots, D * SPLIT * slots,
                  slots * 2 * FwdStage<D, TC, T>::kFloats * sizeof(float), st, "delta_fwd_step_kernel");
}
template <int D, int SPLIT, int TC, typename T>
static int launch_bwd_step(const DeltaBwdParams& p, int nseq, cudaStream_t st) {
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    return launch_dependent(delta_bwd_step_kernel<D, SPLIT, TC, T>, p, nseq / slots, D * SPLIT * slots,
                  slots * (2 * BwdStage<D, TC, T>::kFloats + 2 * (2 * D + 8)) * sizeof(float), st, "delta_bwd_step_kernel");
}
template <int D, int SPLIT, int TC, typename T>
static int launch_sum_bwd(const SumBwdParams& p, int nseq, cudaStream_t st) {
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    if (tune_get(T_SUM_BWD_ROLES, 1))
        return launch(sum_bwd_roles_kernel<D, SPLIT, TC, T>, p, nseq / slots, 3 * D * SPLIT * slots,
                      slots * 3 * sum_roles_floats<D, TC, T>() * sizeof(float), st, "sum_bwd_roles_kernel");
    return launch(sum_bwd_kernel<D, SPLIT, TC, T>, p, nseq / slots, D * SPLIT * slots,
                  slots * 2 * SumStage<D, TC, T>::kFloats * sizeof(float), st, "sum_bwd_kernel");
}

// Shapes beyond the register-resident kernels: one CTA per sequence, matrices in shared memory.
static const size_t kGenericSmemLimit = 227 * 1024;
template <typename T, bool SUM>
static int launch_fwd_generic(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    const size_t bytes = gen_fwd_floats(p.E, p.M) * sizeof(float);
    if (bytes > kGenericSmemLimit) return FWP_ERR_UNSUPPORTED;
    return launch(delta_fwd_generic_kernel<T, SUM>, p, nseq, kGenThreads, bytes, st, "delta_fwd_generic_kernel");
}
template <typename T>
static int launch_bwd_generic(const DeltaBwdParams& p, int nseq, cudaStream_t st) {
    const size_t bytes = gen_bwd_floats(p.E, p.M) * sizeof(float);
    if (bytes > kGenericSmemLimit) return FWP_ERR_UNSUPPORTED;
    return launch(delta_bwd_generic_kernel<T>, p, nseq, kGenThreads, bytes, st, "delta_bwd_generic_kernel");
}
template <typename T>
static int launch_sum_bwd_generic(const SumBwdParams& p, int nseq, cudaStream_t st) {
    const size_t bytes = gen_sum_bwd_floats(p.E, p.M) * sizeof(float);
    if (bytes > kGenericSmemLimit) return FWP_ERR_UNSUPPORTED;
    return launch(sum_bwd_generic_kernel<T>, p, nseq, kGenThreads, bytes, st, "sum_bwd_generic_kernel");
}

// Which execution plan runs by default was picked per head dimension from measurements on B200
// (forward / backward device time, 512 sequences):
//   D=16: blocked + warp-specialised wins both ways (28.3 / 48.5 us vs 41.7 / 103.7 us per-step);
//   D=32: forward per-step 55 us vs blocked 56-71 us, backward blocked 138 us vs per-step 175 us;
//   D=64: forward per-step 161 us vs blocked 208 us; backward fp32 blocked 479 us vs per-step 584 us,
//         bf16 streams (1024 steps) per-step 2.35 ms vs blocked 3.12 ms (the producer warp's widening pass).
// Short segments (the reinforcement-learning callers step the op with L = 1, reinforcement_learning/torchbeast/
// layer.py:143-186) take the per-step plan, whose CTAs start faster: at L <= 16 it measures 10-12 us against
// 12-15 us per launch (32 x 8 sequences), and the d=64 fp32 backward only pays off beyond 64 steps.
// "delta.blocked" = 0 / 1 forces the per-step / blocked plan (tests cross-check one against the other).
constexpr int kShortSeq = 16;
template <typename T, bool SUM>
static int dispatch_fwd(const DeltaFwdParams& p, int nseq, cudaStream_t st) {
    const int D = pad_dim(p.E > p.M ? p.E : p.M);
    const int force = tune_get(T_DELTA_BLOCKED, -1);
    if (D == 0) return launch_fwd_generic<T, SUM>(p, nseq, st);
    switch (D) {
        case 16: {
            if (force == 0 || (force == -1 && p.L <= kShortSeq)) return launch_fwd_step<16, 2, 32, T, SUM>(p, nseq, st);
            if (tune_get(SUM ? T_SUM_FWD_SPLIT16 : T_DELTA_FWD_SPLIT16, 2) == 4) return launch_fwd<16, 4, 32, T, SUM>(p, nseq, st);
            return launch_fwd<16, 2, 32, T, SUM>(p, nseq, st);
        }
        case 32: {
            // fp32 streams: per-step 55 us vs blocked 56 us; bf16 streams: blocked 80 us vs per-step 87 us
            if (force == 0 || (force == -1 && (sizeof(T) == 4 || p.L <= kShortSeq))) return launch_fwd_step<32, 1, 16, T, SUM>(p, nseq, st);
            const int sp = tune_get(SUM ? T_SUM_FWD_SPLIT32 : T_DELTA_FWD_SPLIT32, 1);
            if (sp == 2) return launch_fwd<32, 2, 16, T, SUM>(p, nseq, st);
            if (sp == 4) return launch_fwd<32, 4, 16, T, SUM>(p, nseq, st);
            return launch_fwd<32, 1, 16, T, SUM>(p, nseq, st);
        }
        case 64: {
            if constexpr (!SUM && sizeof(T) == 2) {
                // chunkwise tensor-core form for bf16 streams ("delta.chunk64" = 0 switches it off)
                if (force == -1 && p.L > kShortSeq && tune_get(T_DELTA_CHUNK64, 1) == 1 && chunk_bf16_applies(p))
                    return launch_fwd_chunk_bf16(p, nseq, st);
            }
            if (force != 1) return launch_fwd_step<64, 2, 8, T, SUM>(p, nseq, st);
            if (tune_get(SUM ? T_SUM_FWD_SPLIT64 : T_DELTA_FWD_SPLIT64, 2) == 4) return launch_fwd<64, 4, 8, T, SUM>(p, nseq, st);
            return launch_fwd<64, 2, 8, T, SUM>(p, nseq, st);
        }
    }
    return FWP_ERR_UNSUPPORTED;
}

template <typename T>
static int dispatch_bwd(const DeltaBwdParams& p0, int nseq, cudaStream_t st) {
    DeltaBwdParams p = p0;
    p.bulk = tune_get(T_DELTA_BWD_BULK, 1);
    const int D = pad_dim(p.E > p.M ? p.E : p.M);
    const int force = tune_get(T_DELTA_BLOCKED, -1);
    if (D == 0) return launch_bwd_generic<T>(p, nseq, st);
    switch (D) {
        case 16: {
            if (force == 0 || (force == -1 && p.L <= kShortSeq)) return launch_bwd_step<16, 2, 16, T>(p, nseq, st);
            if (tune_get(T_DELTA_BWD_SPLIT16, 2) == 4) return launch_bwd<16, 4, 16, T>(p, nseq, st);
            // 32-step chunks staged one chunk ahead (three stages; 203 KB of shared memory for four sequences) against
            // 16-step chunks staged two ahead: 45.3 vs 46.3 us at 256 steps, 149.8 vs 155.4 us at 1024
            // (fp32 streams only: the 16-bit staging copies of bf16 streams do not fit next to 32-step chunks)
            if (sizeof(T) != 4 || tune_get(T_DELTA_BWD_CHUNK16, 32) == 16) return launch_bwd<16, 2, 16, T>(p, nseq, st);
            return launch_bwd<16, 2, 32, float, 1>(p, nseq, st);
        }
        case 32: {
            // fp32 streams: blocked 138 us vs per-step 175 us; bf16 streams: per-step 201 us vs blocked 207 us
            if (force == 0 || (force == -1 && (p.L <= kShortSeq || sizeof(T) != 4))) return launch_bwd_step<32, 2, 8, T>(p, nseq, st);
            if (tune_get(T_DELTA_BWD_SPLIT32, 2) == 4) return launch_bwd<32, 4, 8, T>(p, nseq, st);
            return launch_bwd<32, 2, 8, T>(p, nseq, st);
        }
        case 64: {
            if constexpr (sizeof(T) == 2) {
                // chunkwise tensor-core form for bf16 streams ("delta.chunk64" = 0 switches it off)
                if (force == -1 && p.L > kShortSeq && tune_get(T_DELTA_CHUNK64, 1) == 1 && chunk_bf16_applies(p))
                    return launch_bwd_chunk_bf16(p, nseq, st);
            }
            const bool blocked = force == 1 || (force == -1 && sizeof(T) == 4 && p.L > 4 * kShortSeq);
            if (!blocked) return launch_bwd_step<64, 4, 4, T>(p, nseq, st);
            if (tune_get(T_DELTA_BWD_SPLIT64, 2) == 4) return launch_bwd<64, 4, 4, T>(p, nseq, st);
            return launch_bwd<64, 2, 4, T>(p, nseq, st);
        }
    }
    return FWP_ERR_UNSUPPORTED;
}

template <typename T>
static int dispatch_sum_bwd(const SumBwdParams& p, int nseq, cudaStream_t st) {
    const int D = pad_dim(p.E > p.M ? p.E : p.M);
    if (D == 0) return launch_sum_bwd_generic<T>(p, nseq, st);
    switch (D) {
        case 16: return launch_sum_bwd<16, 2, 16, T>(p, nseq, st);
        case 32: return launch_sum_bwd<32, 2, 8, T>(p, nseq, st);
        case 64: return launch_sum_bwd<64, 4, 4, T>(p, nseq, st);
    }
    return FWP_ERR_UNSUPPORTED;
}

static int check_common(int N, int H, int L, int E, int M, int io_dtype) {
    if (N <= 0 || H <= 0 || L <= 0 || E <= 0 || M <= 0) return FWP_ERR_SHAPE;
    if ((long long)N * H > 0x7fffffffLL) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32 && io_dtype != FWP_BF16) return FWP_ERR_DTYPE;
    if (pad_dim(E > M ? E : M) == 0 && gen_bwd_floats(E, M) * sizeof(float) > kGenericSmemLimit)
        return FWP_ERR_UNSUPPORTED;     // beyond both the register-resident and the shared-memory kernels
    return FWP_OK;
}

}  // namespace fwp

using namespace fwp;

static int fast_weight_forward_impl(int N, int H, int L, int E, int M,
                                    const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                                    const fwp_tensor* beta, const fwp_tensor* v_old,
                                    const fwp_tensor* v_insert, const fwp_tensor* kv,
                                    const fwp_tensor* out, int io_dtype, void* stream, int device) {
    if (int rc = check_common(N, H, L, E, M, io_dtype)) return rc;
    const int eb = io_dtype == FWP_F32 ? 4 : 2;
    int rc;
    if ((rc = check_tensor(Q, eb, true)) || (rc = check_tensor(K, eb, true)) || (rc = check_tensor(V, eb, true)) ||
        (rc = check_tensor(beta, eb, true)) || (rc = check_tensor(v_old, 4, true)) ||
        (rc = check_tensor(v_insert, 4, false)) || (rc = check_tensor(kv, 4, true)) ||
        (rc = check_tensor(out, eb, true)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    DeltaFwdParams p;
    p.q = row4(Q); p.k = row4(K); p.v = row4(V); p.beta = row4(beta);
    p.v_old = row4(v_old); p.v_ins = row4(v_insert); p.out = row4(out);
    p.W = (float*)kv->data; p.wN = kv->stride[0]; p.wH = kv->stride[1]; p.wE = kv->stride[2];
    p.H = H; p.L = L; p.E = E; p.M = M; p.NH = N * H;
    cudaStream_t st = (cudaStream_t)stream;
    if (io_dtype == FWP_F32) return dispatch_fwd<float, false>(p, N * H, st);
    return dispatch_fwd<__nv_bfloat16, false>(p, N * H, st);
}

FWP_API int fwp_fast_weight_forward(int N, int H, int L, int E, int M,
                                       const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                                       const fwp_tensor* beta, const fwp_tensor* v_old,
                                       const fwp_tensor* v_insert, const fwp_tensor* kv,
                                       const fwp_tensor* out, int io_dtype, void* stream, int device) {
    return fast_weight_forward_impl(N, H, L, E, M, Q, K, V, beta, v_old, v_insert, kv, out, io_dtype, stream, device);
}

static int fast_weight_backward_impl(int N, int H, int L, int E, int M,
                                        const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                                        const fwp_tensor* beta, const fwp_tensor* v_old,
                                        const fwp_tensor* v_insert, const fwp_tensor* grad_out,
                                        const fwp_tensor* fw_mem,
                                        const fwp_tensor* grad_Q, const fwp_tensor* grad_K,
                                        const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                                        int io_dtype, void* stream, int device) {
    (void)v_insert;
    if (int rc = check_common(N, H, L, E, M, io_dtype)) return rc;
    const int eb = io_dtype == FWP_F32 ? 4 : 2;
    int rc;
    if ((rc = check_tensor(Q, eb, true)) || (rc = check_tensor(K, eb, true)) || (rc = check_tensor(V, eb, true)) ||
        (rc = check_tensor(beta, eb, true)) || (rc = check_tensor(v_old, 4, true)) ||
        (rc = check_tensor(grad_out, eb, true)) || (rc = check_tensor(fw_mem, 4, true)) ||
        (rc = check_tensor(grad_Q, eb, true)) || (rc = check_tensor(grad_K, eb, true)) ||
        (rc = check_tensor(grad_V, eb, true)) || (rc = check_tensor(grad_beta, eb, true)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    DeltaBwdParams p;
    p.q = row4(Q); p.k = row4(K); p.v = row4(V); p.beta = row4(beta); p.v_old = row4(v_old);
    p.gy = row4(grad_out); p.gq = row4(grad_Q); p.gk = row4(grad_K); p.gv = row4(grad_V); p.gb = row4(grad_beta);
    p.W = (float*)fw_mem->data; p.wN = fw_mem->stride[0]; p.wH = fw_mem->stride[1]; p.wE = fw_mem->stride[2];
    p.H = H; p.L = L; p.E = E; p.M = M; p.NH = N * H;
    cudaStream_t st = (cudaStream_t)stream;
    if (io_dtype == FWP_F32) return dispatch_bwd<float>(p, N * H, st);
    return dispatch_bwd<__nv_bfloat16>(p, N * H, st);
}

FWP_API int fwp_fast_weight_backward(int N, int H, int L, int E, int M,
                                        const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                                        const fwp_tensor* beta, const fwp_tensor* v_old,
                                        const fwp_tensor* v_insert, const fwp_tensor* grad_out,
                                        const fwp_tensor* fw_mem,
                                        const fwp_tensor* grad_Q, const fwp_tensor* grad_K,
                                        const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                                        int io_dtype, void* stream, int device) {
    return fast_weight_backward_impl(N, H, L, E, M, Q, K, V, beta, v_old, v_insert, grad_out, fw_mem, grad_Q, grad_K, grad_V,
                                     grad_beta, io_dtype, stream, device);
}

FWP_API int fwp_causal_dot_product(int N, int H, int L, int E, int M,
                                      const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                                      const fwp_tensor* kv, const fwp_tensor* out,
                                      int io_dtype, void* stream, int device) {
    if (int rc = check_common(N, H, L, E, M, io_dtype)) return rc;
    const int eb = io_dtype == FWP_F32 ? 4 : 2;
    int rc;
    if ((rc = check_tensor(Q, eb, true)) || (rc = check_tensor(K, eb, true)) || (rc = check_tensor(V, eb, true)) ||
        (rc = check_tensor(kv, 4, true)) || (rc = check_tensor(out, eb, true)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    DeltaFwdParams p;
    p.q = row4(Q); p.k = row4(K); p.v = row4(V); p.beta = row4(nullptr);
    p.v_old = row4(nullptr); p.v_ins = row4(nullptr); p.out = row4(out);
    p.W = (float*)kv->data; p.wN = kv->stride[0]; p.wH = kv->stride[1]; p.wE = kv->stride[2];
    p.H = H; p.L = L; p.E = E; p.M = M; p.NH = N * H;
    cudaStream_t st = (cudaStream_t)stream;
    if (io_dtype == FWP_F32) return dispatch_fwd<float, true>(p, N * H, st);
    return dispatch_fwd<__nv_bfloat16, true>(p, N * H, st);
}

FWP_API int fwp_causal_dot_backward(int N, int H, int L, int E, int M,
                                       const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                                       const fwp_tensor* grad_out,
                                       const fwp_tensor* grad_Q, const fwp_tensor* grad_K,
                                       const fwp_tensor* grad_V,
                                       int io_dtype, void* stream, int device) {
    if (int rc = check_common(N, H, L, E, M, io_dtype)) return rc;
    const int eb = io_dtype == FWP_F32 ? 4 : 2;
    int rc;
    if ((rc = check_tensor(Q, eb, true)) || (rc = check_tensor(K, eb, true)) || (rc = check_tensor(V, eb, true)) ||
        (rc = check_tensor(grad_out, eb, true)) || (rc = check_tensor(grad_Q, eb, true)) ||
        (rc = check_tensor(grad_K, eb, true)) || (rc = check_tensor(grad_V, eb, true)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    SumBwdParams p;
    p.q = row4(Q); p.k = row4(K); p.v = row4(V); p.gy = row4(grad_out);
    p.gq = row4(grad_Q); p.gk = row4(grad_K); p.gv = row4(grad_V);
    p.H = H; p.L = L; p.E = E; p.M = M; p.NH = N * H;
    cudaStream_t st = (cudaStream_t)stream;
    if (io_dtype == FWP_F32) return dispatch_sum_bwd<float>(p, N * H, st);
    return dispatch_sum_bwd<__nv_bfloat16>(p, N * H, st);
}

// Test hook: launches a kernel whose only wait can never be satisfied, with a limit of `polls` (1..65536) polls;
// afterwards fwp_delta_device_fault() must read 1.  Bounded by construction: nothing hangs, the context stays usable.
FWP_API int fwp_debug_bounded_wait_probe(int polls, void* stream, int device) {
    if (polls < 1 || polls > 65536) return FWP_ERR_SHAPE;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    return fwp::launch_wait_probe(polls, (cudaStream_t)stream);
}

// 1 if a bounded wait on a bulk copy ever ran out on the current device since the last call
// (the affected launch produced wrong numbers instead of hanging), 0 if not, -1 on a CUDA error.
// Synchronises the device; reading clears the flag.
FWP_API int fwp_delta_device_fault(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, fwp::g_delta_fault, sizeof v) != cudaSuccess) return -1;
    if (v) {
        const int zero = 0;
        cudaMemcpyToSymbol(fwp::g_delta_fault, &zero, sizeof zero);
    }
    const int t = fwp::tc_fault_read_clear();
    if (t < 0) return -1;
    return (v || t) ? 1 : 0;
}
