// Recurrent delta net (rec_update_fwm_tanh): delta-rule fast weight memory whose
// query, key, value and beta receive additive feedback R . tanh(y_{t-1}).  sm_100a.
//
//   ht = tanh(y_{t-1}) ; q = softmax(qx_t + Rq^T ht) ; k = softmax(kx_t + Rk^T ht)
//   v = vx_t + Rv^T ht ; beta = sigmoid(bx_t + rb . ht) ; delta-rule step ; y_t = S_t^T q
//
// Restates algorithmic/rec_update_fwm_tanh/rec_update_fwm_tanh.cu (forward kernel :25-345,
// backward kernel :448-876) with the register-resident plan of fwp_core.cuh.  The
// parameter gradients dRq, dRk, dRv, drb are accumulated per (n, h) in registers,
// written once to a scratch buffer and summed over n by a second kernel in a fixed
// order (the reference adds them with global atomics every step).
#include <mutex>
#include "fwp_core.cuh"

namespace fwp {

struct RecFwdParams {
    Row4 qx, kx, vx, bx, q_out, k_out, v_out, b_out, v_old, out;
    const float *Rq, *Rk, *Rv, *rb;
    long long rH, rE;       // strides of R over head and first matrix index
    long long rbH;          // stride of rb over head
    float* W; long long wN, wH, wE;
    float* h; long long hN, hH;
    int H, L, D;
};

template <int D, int TC>
struct RecFwdStage {
    Tile<D, TC, float> q, k, v;
    Tile<1, TC, float> b;
    static constexpr int kFloats = 3 * r4(TC * D) + r4(TC);
    __device__ __forceinline__ void bind(float* mem) {
        q.bind(mem); mem += r4(TC * D);
        k.bind(mem); mem += r4(TC * D);
        v.bind(mem); mem += r4(TC * D);
        b.bind(mem);
    }
};

template <int D, int SPLIT, int TC>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) rec_fwd_kernel(const RecFwdParams p) {
    using G = Geo<D, SPLIT>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = RecFwdStage<D, TC>;
    constexpr int kX = 3 * D + 32;        // per parity: ht[D], eq[D], ek[D], slots[4][8]
    for (int i = g.tid; i < 2 * Stage::kFloats + 2 * kX; i += G::NT) smem[i] = 0.f;
    float* xch = smem + 2 * Stage::kFloats;

    Src<float> sq, sk, sv, sb;
    sq.init(p.qx, n, h, p.D);
    sk.init(p.kx, n, h, p.D);
    sv.init(p.vx, n, h, p.D);
    sb.init(p.bx, n, h, 1);

    f2 S[G::NP], Rq[G::NP], Rk[G::NP], Rv[G::NP], rb[G::NP];
    load_cols(g, S, p.W + n * p.wN + h * p.wH, p.wE, p.D, p.D);
    load_cols(g, Rq, p.Rq + h * p.rH, p.rE, p.D, p.D);
    load_cols(g, Rk, p.Rk + h * p.rH, p.rE, p.D, p.D);
    load_cols(g, Rv, p.Rv + h * p.rH, p.rE, p.D, p.D);
    {
        float pr[2];
#pragma unroll
        for (int i = 0; i < G::NR; i++) {
            const int e = g.off + i;
            pr[i & 1] = e < p.D ? p.rb[h * p.rbH + e] : 0.f;
            if (i & 1) rb[i >> 1] = f2_pack(pr[0], pr[1]);
        }
    }
    const bool ok = g.idx < p.D;
    float* hp = p.h + n * p.hN + h * p.hH;
    float hv = ok ? hp[g.idx] : 0.f;
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int c) {
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.q.template load<G::NT>(sq, t0, nt, g.tid);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        s.b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    issue(0);
    int par = 0;
    for (int c = 0; c < nchunks; c++) {
        if (c + 1 < nchunks) { issue(c + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        for (int t = 0; t < nt; t++) {
            float* xh = xch + par * kX;
            float* xq = xh + D;
            float* xk = xq + D;
            float* slot = xk + D;
            par ^= 1;
            const int o = t * D + g.idx;
            if (g.s == 0) xh[g.idx] = ok ? tanh_fast(hv) : 0.f;
            cta_sync<G::WPS>();
            f2 hs[G::NP];
            lds_slice<G::NR>(hs, xh + g.off);
            const float qh = s.q.f[o] + reduce_split<SPLIT>(dot2<G::NP>(Rq, hs));
            const float kh = s.k.f[o] + reduce_split<SPLIT>(dot2<G::NP>(Rk, hs));
            const float vv = s.v.f[o] + reduce_split<SPLIT>(dot2<G::NP>(Rv, hs));
            const float beta = sigmoidf_(s.b.f[t] + reduce_split<SPLIT>(dot2<G::NP>(rb, hs)));
            const float mq = cta_allreduce_idx<G, true>(g, ok ? qh : -INFINITY, slot);
            const float mk = cta_allreduce_idx<G, true>(g, ok ? kh : -INFINITY, slot + 8);
            const float eq = ok ? exp_neg(qh - mq) : 0.f;
            const float ek = ok ? exp_neg(kh - mk) : 0.f;
            if (g.s == 0) { xq[g.idx] = eq; xk[g.idx] = ek; }
            const float invq = rcp_approx(softmax_den(g, eq, slot + 16));
            const float invk = rcp_approx(softmax_den(g, ek, slot + 24));
            cta_sync<G::WPS>();
            f2 ks[G::NP], qs[G::NP];
            lds_slice<G::NR>(ks, xk + g.off);
            lds_slice<G::NR>(qs, xq + g.off);
            const float vo = reduce_split<SPLIT>(dot2<G::NP>(S, ks)) * invk;
            const float u = beta * (vv - vo);
            axpy2<G::NP>(S, ks, u * invk);
            const float y = reduce_split<SPLIT>(dot2<G::NP>(S, qs)) * invq;
            hv = y;
            if (ok && g.s == 0) {
                const int tt = t0 + t;
                put<float>(p.out, n, h, tt, g.idx, y);
                put<float>(p.q_out, n, h, tt, g.idx, eq * invq);
                put<float>(p.k_out, n, h, tt, g.idx, ek * invk);
                put<float>(p.v_out, n, h, tt, g.idx, vv);
                put<float>(p.v_old, n, h, tt, g.idx, vo);
                if (g.idx == 0) put<float>(p.b_out, n, h, tt, 0, beta);
            }
        }
        __syncthreads();
    }
    store_cols(g, S, p.W + n * p.wN + h * p.wH, p.wE, p.D, p.D);
    if (ok && g.s == 0) hp[g.idx] = hv;
}

// ------------------------------------------------- forward, one warp per sequence, d <= 32
// The per-step chain of the kernel above at d = 32 is one warp's latency: every instruction waits for the one
// before it.  This form keeps the arithmetic and shortens the chain:
//   * the two maxima of the softmaxes are one warp-wide reduction instruction each (redux.sync.max.f32);
//   * the softmax denominators are summed by every lane from the exchanged vectors it reads anyway (no shuffle tree);
//   * y_t = S_t^T q is taken from the matrix *before* the update, y = (S^T q + (k.q) c) with c the update's scale, so
//     the three dot products of a step run side by side and the rank-one update leaves the chain;
//   * beta's feedback term r_b . tanh(h) is a lane-local product summed by shuffles beside the matrix products;
//   * tanh by exp2 / reciprocal (a short polynomial near zero), outputs through running pointers.
// FULL: the head dimension is exactly 32 (no padding lanes, no predicates in the step).
template <int TC, bool FULL>
__global__ void __launch_bounds__(128) rec_fwd_warp32_kernel(const RecFwdParams p) {
    constexpr int D = 32;
    using G = Geo<D, 1>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = RecFwdStage<D, TC>;
    constexpr int kTile = r4(TC * D);     // distance between the q, k and v tiles of a stage
    constexpr int kX = 3 * D;             // ht[D], eq[D], ek[D]
    for (int i = g.tid; i < 2 * Stage::kFloats + kX; i += G::NT) smem[i] = 0.f;
    float* xh = smem + 2 * Stage::kFloats;
    float* xq = xh + D;
    float* xk = xq + D;

    Src<float> sq, sk, sv, sb;
    sq.init(p.qx, n, h, p.D);
    sk.init(p.kx, n, h, p.D);
    sv.init(p.vx, n, h, p.D);
    sb.init(p.bx, n, h, 1);

    f2 S[G::NP], Rq[G::NP], Rk[G::NP], Rv[G::NP];
    load_cols(g, S, p.W + n * p.wN + h * p.wH, p.wE, p.D, p.D);
    load_cols(g, Rq, p.Rq + h * p.rH, p.rE, p.D, p.D);
    load_cols(g, Rk, p.Rk + h * p.rH, p.rE, p.D, p.D);
    load_cols(g, Rv, p.Rv + h * p.rH, p.rE, p.D, p.D);
    const bool ok = FULL || g.idx < p.D;
    // beta's feedback r_b . tanh(h): lane products in fixed point (24 bits below the largest |r_b|), integer warp sum
    float rbl = ok ? p.rb[h * p.rbH + g.idx] : 0.f;
    const float rbmax = warp_max_f32(fabsf(rbl));
    const float rb_unscale = rbmax * (1.f / 8388608.f);         // 2^-23 of the largest entry
    rbl = rbmax > 0.f ? rbl * (8388608.f / rbmax) : 0.f;
    float* hp = p.h + n * p.hN + h * p.hH;
    float hv = ok ? hp[g.idx] : 0.f;
    const int col = ok ? g.idx : 0;
    float* po = reinterpret_cast<float*>(p.out.p) + n * p.out.sN + h * p.out.sH + col;
    float* pq = reinterpret_cast<float*>(p.q_out.p) + n * p.q_out.sN + h * p.q_out.sH + col;
    float* pk = reinterpret_cast<float*>(p.k_out.p) + n * p.k_out.sN + h * p.k_out.sH + col;
    float* pv = reinterpret_cast<float*>(p.v_out.p) + n * p.v_out.sN + h * p.v_out.sH + col;
    float* pvo = reinterpret_cast<float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH + col;
    float* pb = reinterpret_cast<float*>(p.b_out.p) + n * p.b_out.sN + h * p.b_out.sH;
    __syncwarp();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int c) {
        Stage s; s.bind(smem + (c & 1) * Stage::kFloats);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.q.template load<G::NT>(sq, t0, nt, g.tid);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        s.b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    issue(0);
    // tanh of the fed-back vector is the head of the next step's chain: it is taken as soon as y is known, and
    // the matrix update and the stores of the step follow it and fill its latency
    float th = tanh_fast(hv);                               // padding lanes hold hv = 0
    for (int c = 0; c < nchunks; c++) {
        if (c + 1 < nchunks) { issue(c + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncwarp();
        const float* row = smem + (c & 1) * Stage::kFloats + g.idx;     // this lane's column of the q tile
        const float* brow = smem + (c & 1) * Stage::kFloats + 3 * kTile;
        const int nt = min(TC, p.L - c * TC);
#pragma unroll 1
        for (int t = 0; t < nt; t++, row += D, brow++) {
            const float qin = row[0], kin = row[kTile], vin = row[2 * kTile], bin = brow[0];
            xh[g.idx] = th;
            __syncwarp();
            const float bsum = warp_sum_scaled(th * rbl);
            f2 hs[G::NP];
            lds_slice<G::NR>(hs, xh);
            const float qh = qin + dot2<G::NP>(Rq, hs);
            const float kh = kin + dot2<G::NP>(Rk, hs);
            const float vv = vin + dot2<G::NP>(Rv, hs);
            const float mk = warp_max_f32(ok ? kh : -INFINITY);
            const float mq = warp_max_f32(ok ? qh : -INFINITY);
            const float ek = ok ? ex2_approx((kh - mk) * kLog2e) : 0.f;
            const float eq = ok ? ex2_approx((qh - mq) * kLog2e) : 0.f;
            xk[g.idx] = ek;
            xq[g.idx] = eq;
            __syncwarp();
            const float invk = rcp_approx(warp_sum_unit_scaled(ek)) * 67108864.f;
            const float invq = rcp_approx(warp_sum_unit_scaled(eq)) * 67108864.f;
            const float beta = rcp_approx(1.f + ex2_approx(-kLog2e * fmaf(bsum, rb_unscale, bin)));
            f2 ks[G::NP], qs[G::NP];
            lds_slice<G::NR>(ks, xk);
            lds_slice<G::NR>(qs, xq);
            const float vo_un = dot2<G::NP>(S, ks);
            const float y_un = dot2<G::NP>(S, qs);
            const float kq_un = dot2<G::NP>(ks, qs);
            const float vo = vo_un * invk;
            const float cc = beta * (vv - vo) * invk;       // S += ek (x) cc
            const float y = fmaf(kq_un, cc, y_un) * invq;
            hv = ok ? y : 0.f;
            th = tanh_fast(hv);
            axpy2<G::NP>(S, ks, cc);
            if (ok) {
                *po = y;
                *pq = eq * invq;
                *pk = ek * invk;
                *pv = vv;
                *pvo = vo;
                if (g.idx == 0) *pb = beta;
            }
            po += p.out.sL; pq += p.q_out.sL; pk += p.k_out.sL; pv += p.v_out.sL; pvo += p.v_old.sL; pb += p.b_out.sL;
        }
        __syncwarp();
    }
    store_cols(g, S, p.W + n * p.wN + h * p.wH, p.wE, p.D, p.D);
    if (ok) hp[g.idx] = hv;
}

// Barrier among the warps of one sequence (the sequences that share a CTA do not wait for each other).
template <class G>
__device__ __forceinline__ void seq_sync(const G& g) {
    if constexpr (G::WPS == 1) __syncwarp(); else slot_barrier(g.slot, G::NT);
}

// ------------------------------------------------------------------ backward
struct RecBwdParams {
    Row4 q, k, v, beta, v_old, od, gy, gq, gk, gv, gb;
    const float *Rq, *Rk, *Rv, *rb;
    long long rH, rE, rbH;
    float* W; long long wN, wH, wE;
    float* scratch;          // [N*H][3*d*d + d] partial parameter gradients
    int H, L, D;
};

template <int D, int TC>
struct RecBwdStage {
    Tile<D, TC, float> q, k, v, vo, od, gy;
    Tile<1, TC, float> b;
    static constexpr int kFloats = 6 * r4(TC * D) + r4(TC);
    __device__ __forceinline__ void bind(float* mem) {
        q.bind(mem); mem += r4(TC * D);
        k.bind(mem); mem += r4(TC * D);
        v.bind(mem); mem += r4(TC * D);
        vo.bind(mem); mem += r4(TC * D);
        od.bind(mem); mem += r4(TC * D);
        gy.bind(mem); mem += r4(TC * D);
        b.bind(mem);
    }
};

template <int D>
struct RecBwdSmem {
    static constexpr int kRS = D + 4;                    // padded row stride of the R copies
    static constexpr int kR = 3 * D * kRS + D;           // Rq, Rk, Rv rows + rb
    static constexpr int kXs = 5 * D + 40;               // per parity: g, u, br, dq, dk [D] + slots[5][8]
};

template <int D, int SPLIT, int TC>
__global__ void __launch_bounds__(D * SPLIT * slots_for(D * SPLIT)) rec_bwd_kernel(const RecBwdParams p) {
    using G = Geo<D, SPLIT>;
    using SM = RecBwdSmem<D>;
    const G g;
    const int n = g.seq / p.H, h = g.seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = slot_smem(smem_all, g);
    using Stage = RecBwdStage<D, TC>;
    for (int i = g.tid; i < 2 * Stage::kFloats + 2 * SM::kXs + SM::kR; i += G::NT) smem[i] = 0.f;
    float* xch = smem + 2 * Stage::kFloats;
    float* rmem = xch + 2 * SM::kXs;       // R rows: [3][D][kRS], then rb[D]
    __syncthreads();
    for (int i = g.tid; i < p.D * p.D; i += G::NT) {
        const int e = i / p.D, m = i - e * p.D;
        const long long src = h * p.rH + (long long)e * p.rE + m;
        rmem[0 * D * SM::kRS + e * SM::kRS + m] = p.Rq[src];
        rmem[1 * D * SM::kRS + e * SM::kRS + m] = p.Rk[src];
        rmem[2 * D * SM::kRS + e * SM::kRS + m] = p.Rv[src];
    }
    for (int i = g.tid; i < p.D; i += G::NT) rmem[3 * D * SM::kRS + i] = p.rb[h * p.rbH + i];

    Src<float> sq, sk, sv, so, sd, sg, sb;
    sq.init(p.q, n, h, p.D);
    sk.init(p.k, n, h, p.D);
    sv.init(p.v, n, h, p.D);
    so.init(p.v_old, n, h, p.D);
    sd.init(p.od, n, h, p.D);
    sg.init(p.gy, n, h, p.D);
    sb.init(p.beta, n, h, 1);

    f2 Sr[G::NP], Gr[G::NP], Gc[G::NP], aq[G::NP], ak[G::NP], av[G::NP];
    load_rows(g, Sr, p.W + n * p.wN + h * p.wH, p.wE, p.D, p.D);
#pragma unroll
    for (int i = 0; i < G::NP; i++) {
        Gr[i] = Gc[i] = aq[i] = ak[i] = av[i] = 0ull;
    }
    float gh = 0.f, arb = 0.f;
    const bool ok = g.idx < p.D;
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {
        Stage s; s.bind(smem + (j & 1) * Stage::kFloats);
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.q.template load<G::NT>(sq, t0, nt, g.tid);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        s.vo.template load<G::NT>(so, t0, nt, g.tid);
        s.od.template load<G::NT>(sd, t0, nt, g.tid);
        s.gy.template load<G::NT>(sg, t0, nt, g.tid);
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
            float* xg = xch + par * SM::kXs;
            float* xu = xg + D;
            float* xbr = xu + D;
            float* xdq = xbr + D;
            float* xdk = xdq + D;
            float* slot = xdk + D;
            par ^= 1;
            const int o = t * D + g.idx;
            const float beta = s.b.f[t];
            const float gcol = s.gy.f[o] + gh;
            float dv, dbh;
            // ---- column role
            {
                f2 qq[G::NP], kk[G::NP];
                lds_slice<G::NR>(qq, s.q.f + t * D + g.off);
                lds_slice<G::NR>(kk, s.k.f + t * D + g.off);
                const float w = s.v.f[o] - s.vo.f[o];
                axpy2<G::NP>(Gc, qq, gcol);
                const float r = reduce_split<SPLIT>(dot2<G::NP>(Gc, kk));
                dv = beta * r;
                axpy2<G::NP>(Gc, kk, -dv);
                if (g.s == 0) { xg[g.idx] = gcol; xu[g.idx] = beta * w; xbr[g.idx] = dv; }
                // db = sum over idx of r w: the warps' partial sums cross with the exchange below (no barrier of their own)
                const float dbp = warp_sum_idx<SPLIT>(r * w);
                if (G::WPS > 1 && g.lane == 0) slot[g.warp] = dbp;
                seq_sync<G>(g);
                float db = dbp;
                if constexpr (G::WPS > 1) {
                    db = slot[0];
#pragma unroll
                    for (int w2 = 1; w2 < G::WPS; w2++) db += slot[w2];
                }
                dbh = db * beta * (1.f - beta);
            }
            // ---- row role: the delta block, then the two softmax backward maps
            float dqh, dkh;
            const float qe = s.q.f[o], ke = s.k.f[o], hte = s.od.f[o];
            {
                f2 gr[G::NP], ur[G::NP], brr[G::NP];
                lds_slice<G::NR>(gr, xg + g.off);
                lds_slice<G::NR>(ur, xu + g.off);
                lds_slice<G::NR>(brr, xbr + g.off);
                float dq = dot2<G::NP>(Sr, gr);
                axpy2<G::NP>(Gr, gr, qe);
                float dk = dot2<G::NP>(Gr, ur);
                axpy2<G::NP>(Sr, ur, -ke);
                dk -= dot2<G::NP>(Sr, brr);
                axpy2<G::NP>(Gr, brr, -ke);
                dq = reduce_split<SPLIT>(dq);
                dk = reduce_split<SPLIT>(dk);
                // the two softmax backward sums cross the warps behind one barrier
                float cq = warp_sum_idx<SPLIT>(qe * dq), ck = warp_sum_idx<SPLIT>(ke * dk);
                if constexpr (G::WPS > 1) {
                    if (g.lane == 0) { slot[8 + g.warp] = cq; slot[16 + g.warp] = ck; }
                    seq_sync<G>(g);
                    cq = slot[8]; ck = slot[16];
#pragma unroll
                    for (int w2 = 1; w2 < G::WPS; w2++) { cq += slot[8 + w2]; ck += slot[16 + w2]; }
                }
                dqh = qe * (dq - cq);
                dkh = ke * (dk - ck);
            }
            if (g.s == 0) {
                xdq[g.idx] = dqh;
                xdk[g.idx] = dkh;
                if (ok) {
                    const int tt = t0 + t;
                    put<float>(p.gq, n, h, tt, g.idx, dqh);
                    put<float>(p.gk, n, h, tt, g.idx, dkh);
                    put<float>(p.gv, n, h, tt, g.idx, dv);
                    if (g.idx == 0) put<float>(p.gb, n, h, tt, 0, dbh);
                }
            }
            seq_sync<G>(g);
            // ---- feedback gradient (row role over R) and parameter gradients (column role)
            {
                f2 dqs[G::NP], dks[G::NP], dvs[G::NP], rr[G::NP];
                lds_slice<G::NR>(dqs, xdq + g.off);
                lds_slice<G::NR>(dks, xdk + g.off);
                lds_slice<G::NR>(dvs, xbr + g.off);
                const float* rrow = rmem + g.idx * SM::kRS + g.off;
                lds_slice<G::NR>(rr, rrow);
                float back = dot2<G::NP>(rr, dqs);
                lds_slice<G::NR>(rr, rrow + D * SM::kRS);
                back += dot2<G::NP>(rr, dks);
                lds_slice<G::NR>(rr, rrow + 2 * D * SM::kRS);
                back += dot2<G::NP>(rr, dvs);
                back = reduce_split<SPLIT>(back) + rmem[3 * D * SM::kRS + g.idx] * dbh;
                gh = (1.f - hte * hte) * back;
                f2 hs[G::NP];
                lds_slice<G::NR>(hs, s.od.f + t * D + g.off);
                axpy2<G::NP>(aq, hs, dqh);
                axpy2<G::NP>(ak, hs, dkh);
                axpy2<G::NP>(av, hs, dv);
                arb += hte * dbh;
            }
        }
        __syncthreads();
    }
    store_rows(g, Sr, p.W + n * p.wN + h * p.wH, p.wE, p.D, p.D);
    // partial parameter gradients of this (n, h): [3][d][d] then [d]
    float* out = p.scratch + (long long)g.seq * (3 * p.D * p.D + p.D);
    store_cols(g, aq, out, p.D, p.D, p.D);
    store_cols(g, ak, out + p.D * p.D, p.D, p.D, p.D);
    store_cols(g, av, out + 2 * p.D * p.D, p.D, p.D, p.D);
    if (ok && g.s == 0) out[3 * p.D * p.D + g.idx] = arb;
}

// sum the per-(n,h) partials over n in index order: one thread per (h, element)
__global__ void rec_param_reduce_kernel(const float* __restrict__ scratch, int N, int H, int D,
                                        float* gRq, float* gRk, float* gRv, float* grb,
                                        long long rH, long long rE, long long rbH) {
    const int per = 3 * D * D + D;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H * per) return;
    const int h = i / per, j = i - h * per;
    float acc = 0.f;
    for (int n = 0; n < N; n++) acc += scratch[((long long)n * H + h) * per + j];
    if (j < 3 * D * D) {
        const int which = j / (D * D), r = j - which * D * D, e = r / D, m = r - e * D;
        float* dst = which == 0 ? gRq : (which == 1 ? gRk : gRv);
        dst[h * rH + (long long)e * rE + m] = acc;
    } else {
        grb[h * rbH + (j - 3 * D * D)] = acc;
    }
}

}  // namespace fwp
#include "fwp_recdelta_roles.cuh"
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

template <int D, int SPLIT, int TC>
static int launch_rec_fwd(const RecFwdParams& p, int nseq, cudaStream_t st) {
    auto kern = rec_fwd_kernel<D, SPLIT, TC>;
    const size_t bytes = (2 * RecFwdStage<D, TC>::kFloats + 2 * (3 * D + 32)) * sizeof(float);
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    if (int rc = smem_optin(kern, bytes * slots)) return rc;
    kern<<<nseq / slots, D * SPLIT * slots, bytes * slots, st>>>(p);
    count_launch();
    note_kernel("rec_fwd_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int TC>
static int launch_rec_fwd_warp32(const RecFwdParams& p, int nseq, cudaStream_t st) {
    auto kern = p.D == 32 ? rec_fwd_warp32_kernel<TC, true> : rec_fwd_warp32_kernel<TC, false>;
    const size_t bytes = (2 * RecFwdStage<32, TC>::kFloats + 3 * 32) * sizeof(float);
    int slots = 4;
    while (nseq % slots) slots >>= 1;
    if (int rc = smem_optin(kern, bytes * slots)) return rc;
    kern<<<nseq / slots, 32 * slots, bytes * slots, st>>>(p);
    count_launch();
    note_kernel("rec_fwd_warp32_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

template <int D, int SPLIT, int TC>
static int launch_rec_bwd(const RecBwdParams& p, int nseq, cudaStream_t st) {
    auto kern = rec_bwd_kernel<D, SPLIT, TC>;
    const size_t bytes = (2 * RecBwdStage<D, TC>::kFloats + 2 * RecBwdSmem<D>::kXs + RecBwdSmem<D>::kR) * sizeof(float);
    int slots = slots_for(D * SPLIT);
    while (nseq % slots) slots >>= 1;          // sequences per CTA must divide the sequence count
    if (int rc = smem_optin(kern, bytes * slots)) return rc;
    kern<<<nseq / slots, D * SPLIT * slots, bytes * slots, st>>>(p);
    count_launch();
    note_kernel("rec_bwd_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

static int launch_rec_bwd_roles32(const RecBwdParams& p, int nseq, cudaStream_t st) {
    constexpr int TC = 8;
    auto kern = rec_bwd_roles32_kernel<TC>;
    int slots = 4;
    while (nseq % slots) slots >>= 1;
    const size_t bytes = (size_t)RecRolesSmem<TC>::kFloats * sizeof(float) * slots;
    if (int rc = smem_optin(kern, bytes)) return rc;
    kern<<<nseq / slots, 64 * slots, bytes, st>>>(p);
    count_launch();
    note_kernel("rec_bwd_roles32_kernel");
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

static int check_params(const fwp_tensor* Rq, const fwp_tensor* Rk, const fwp_tensor* Rv, const fwp_tensor* rb) {
    int rc;
    if ((rc = check_tensor(Rq, 4, true)) || (rc = check_tensor(Rk, 4, true)) || (rc = check_tensor(Rv, 4, true)) ||
        (rc = check_tensor(rb, 4, true)))
        return rc;
    // one kernel-side stride set serves the three matrices
    for (int i = 1; i < 3; i++)
        if (Rk->stride[i] != Rq->stride[i] || Rv->stride[i] != Rq->stride[i]) return FWP_ERR_STRIDE;
    return FWP_OK;
}

}  // namespace fwp

using namespace fwp;

FWP_API int64_t fwp_rec_update_fwm_tanh_scratch_floats(int N, int H, int D) {
    if (N <= 0 || H <= 0 || D <= 0) return 0;
    return (int64_t)N * H * (3LL * D * D + D);
}

FWP_API int fwp_rec_update_fwm_tanh_forward(int N, int H, int L, int D,
                                            const fwp_tensor* qx, const fwp_tensor* kx,
                                            const fwp_tensor* vx, const fwp_tensor* bx,
                                            const fwp_tensor* Rq, const fwp_tensor* Rk,
                                            const fwp_tensor* Rv, const fwp_tensor* rb,
                                            const fwp_tensor* q_out, const fwp_tensor* k_out,
                                            const fwp_tensor* v_out, const fwp_tensor* beta_out,
                                            const fwp_tensor* v_old, const fwp_tensor* states,
                                            const fwp_tensor* kv, const fwp_tensor* out,
                                            int io_dtype, void* stream, int device) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32) return FWP_ERR_DTYPE;
    const int DP = pad_dim(D);
    if (!DP) return FWP_ERR_UNSUPPORTED;
    int rc;
    if ((rc = check_tensor(qx, 4, true)) || (rc = check_tensor(kx, 4, true)) || (rc = check_tensor(vx, 4, true)) ||
        (rc = check_tensor(bx, 4, true)) || (rc = check_params(Rq, Rk, Rv, rb)) ||
        (rc = check_tensor(q_out, 4, true)) || (rc = check_tensor(k_out, 4, true)) ||
        (rc = check_tensor(v_out, 4, true)) || (rc = check_tensor(beta_out, 4, true)) ||
        (rc = check_tensor(v_old, 4, true)) || (rc = check_tensor(states, 4, true)) ||
        (rc = check_tensor(kv, 4, true)) || (rc = check_tensor(out, 4, true)))
        return rc;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    RecFwdParams p;
    p.qx = row4(qx); p.kx = row4(kx); p.vx = row4(vx); p.bx = row4(bx);
    p.q_out = row4(q_out); p.k_out = row4(k_out); p.v_out = row4(v_out); p.b_out = row4(beta_out);
    p.v_old = row4(v_old); p.out = row4(out);
    p.Rq = (const float*)Rq->data; p.Rk = (const float*)Rk->data; p.Rv = (const float*)Rv->data;
    p.rb = (const float*)rb->data;
    p.rH = Rq->stride[1]; p.rE = Rq->stride[2]; p.rbH = rb->stride[1];
    p.W = (float*)kv->data; p.wN = kv->stride[0]; p.wH = kv->stride[1]; p.wE = kv->stride[2];
    p.h = (float*)states->data; p.hN = states->stride[0]; p.hH = states->stride[1];
    p.H = H; p.L = L; p.D = D;
    cudaStream_t st = (cudaStream_t)stream;
    switch (DP) {
        case 16: return launch_rec_fwd<16, 2, 32>(p, N * H, st);
        case 32: {
            const int sp = tune_get(T_REC_FWD_SPLIT32, 1);
            // measured on B200 (512 sequences x 256 steps): 1 -> 0.36 ms, 2 -> 0.38 ms, 4 -> 0.41 ms
            if (sp == 1 && tune_get(T_REC_FWD_WARP32, 1)) return launch_rec_fwd_warp32<16>(p, N * H, st);
            if (sp == 2) return launch_rec_fwd<32, 2, 16>(p, N * H, st);
            if (sp == 4) return launch_rec_fwd<32, 4, 16>(p, N * H, st);
            return launch_rec_fwd<32, 1, 16>(p, N * H, st);
        }
        case 64: return launch_rec_fwd<64, 4, 8>(p, N * H, st);
    }
    return FWP_ERR_UNSUPPORTED;
}

FWP_API int fwp_rec_update_fwm_tanh_backward(int N, int H, int L, int D,
                                             const fwp_tensor* q, const fwp_tensor* k,
                                             const fwp_tensor* v, const fwp_tensor* beta,
                                             const fwp_tensor* v_old, const fwp_tensor* o_delayed,
                                             const fwp_tensor* grad_out,
                                             const fwp_tensor* Rq, const fwp_tensor* Rk,
                                             const fwp_tensor* Rv, const fwp_tensor* rb,
                                             const fwp_tensor* fw_mem,
                                             const fwp_tensor* grad_q, const fwp_tensor* grad_k,
                                             const fwp_tensor* grad_v, const fwp_tensor* grad_beta,
                                             const fwp_tensor* grad_Rq, const fwp_tensor* grad_Rk,
                                             const fwp_tensor* grad_Rv, const fwp_tensor* grad_rb,
                                             float* scratch, int64_t scratch_floats,
                                             int io_dtype, void* stream, int device) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32) return FWP_ERR_DTYPE;
    const int DP = pad_dim(D);
    if (!DP) return FWP_ERR_UNSUPPORTED;
    int rc;
    if ((rc = check_tensor(q, 4, true)) || (rc = check_tensor(k, 4, true)) || (rc = check_tensor(v, 4, true)) ||
        (rc = check_tensor(beta, 4, true)) || (rc = check_tensor(v_old, 4, true)) ||
        (rc = check_tensor(o_delayed, 4, true)) || (rc = check_tensor(grad_out, 4, true)) ||
        (rc = check_params(Rq, Rk, Rv, rb)) || (rc = check_tensor(fw_mem, 4, true)) ||
        (rc = check_tensor(grad_q, 4, true)) || (rc = check_tensor(grad_k, 4, true)) ||
        (rc = check_tensor(grad_v, 4, true)) || (rc = check_tensor(grad_beta, 4, true)) ||
        (rc = check_params(grad_Rq, grad_Rk, grad_Rv, grad_rb)))
        return rc;
    if (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 15) ||
        scratch_floats < fwp_rec_update_fwm_tanh_scratch_floats(N, H, D))
        return FWP_ERR_SCRATCH;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    RecBwdParams p;
    p.q = row4(q); p.k = row4(k); p.v = row4(v); p.beta = row4(beta); p.v_old = row4(v_old);
    p.od = row4(o_delayed); p.gy = row4(grad_out);
    p.gq = row4(grad_q); p.gk = row4(grad_k); p.gv = row4(grad_v); p.gb = row4(grad_beta);
    p.Rq = (const float*)Rq->data; p.Rk = (const float*)Rk->data; p.Rv = (const float*)Rv->data;
    p.rb = (const float*)rb->data;
    p.rH = Rq->stride[1]; p.rE = Rq->stride[2]; p.rbH = rb->stride[1];
    p.W = (float*)fw_mem->data; p.wN = fw_mem->stride[0]; p.wH = fw_mem->stride[1]; p.wE = fw_mem->stride[2];
    p.scratch = scratch;
    p.H = H; p.L = L; p.D = D;
    cudaStream_t st = (cudaStream_t)stream;
    switch (DP) {
        case 16: rc = launch_rec_bwd<16, 2, 16>(p, N * H, st); break;
        case 32: {
            if (p.D == 32 && tune_get(T_REC_BWD_ROLES32, 1) && rows_16B_aligned(p.q) && rows_16B_aligned(p.k) &&
                rows_16B_aligned(p.v) && rows_16B_aligned(p.v_old) && rows_16B_aligned(p.od) && rows_16B_aligned(p.gy)) {
                rc = launch_rec_bwd_roles32(p, N * H, st);
                break;
            }
            const int sp = tune_get(T_REC_BWD_SPLIT32, 2);
            // measured: 2 -> 0.32 ms, 4 -> 0.37 ms, 1 -> 0.43 ms (spills); the chain-warp kernel above 0.27 ms
            // (0.42 ms in a first version that spilled 80 registers: it now fetches its vectors where it uses them)
            if (sp == 4) rc = launch_rec_bwd<32, 4, 8>(p, N * H, st);
            else if (sp == 1) rc = launch_rec_bwd<32, 1, 8>(p, N * H, st);
            else rc = launch_rec_bwd<32, 2, 8>(p, N * H, st);
            break;
        }
        case 64: rc = launch_rec_bwd<64, 4, 4>(p, N * H, st); break;
        default: rc = FWP_ERR_UNSUPPORTED;
    }
    if (rc) return rc;
    const int total = H * (3 * D * D + D);
    rec_param_reduce_kernel<<<(total + 255) / 256, 256, 0, st>>>(
        scratch, N, H, D, (float*)grad_Rq->data, (float*)grad_Rk->data, (float*)grad_Rv->data,
        (float*)grad_rb->data, grad_Rq->stride[1], grad_Rq->stride[2], grad_rb->stride[1]);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}


// ---------------------------------------------------------------------------
// Backward of the recurrent delta net for callers that cannot allocate.
//
// The regular entry point above takes a caller-allocated scratch buffer.  Some
// hosts have nothing to allocate it with at the moment of the call: a plain C
// or Fortran program bound to this ABI without a device memory pool, or a
// process that has handed all device memory to another owner at start-up and
// may not call cudaMalloc afterwards.  For them this variant keeps the scratch
// in a fixed array inside the library image, FWP_NOALLOC_SCRATCH_FLOATS floats
// (8 MiB) on every GPU that loads the library, held until the process exits.
//
// The array's name is only a host-side handle; its device address is looked up
// once per device with cudaGetSymbolAddress, with that device current, on the
// first call that targets the device.  Make that first call outside any stream
// capture.  Every call on a device uses the same array, so two calls that can
// overlap on the GPU (different streams, no ordering between them) race; calls
// ordered on one stream are fine.  Nothing in the array has to start at zero:
// each (batch, head) block overwrites its whole region before the reduction
// kernel reads it.  This function calls no cudaMalloc, cudaFree or any other
// allocating routine.
namespace {
static __device__ __align__(256) float g_noalloc_scratch[FWP_NOALLOC_SCRATCH_FLOATS];
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_ptr[kMaxDevices] = {};
}  // namespace

FWP_API int fwp_rec_update_fwm_tanh_backward_noalloc(int N, int H, int L, int D,
                                                     const fwp_tensor* q, const fwp_tensor* k,
                                                     const fwp_tensor* v, const fwp_tensor* beta,
                                                     const fwp_tensor* v_old, const fwp_tensor* o_delayed,
                                                     const fwp_tensor* grad_out,
                                                     const fwp_tensor* Rq, const fwp_tensor* Rk,
                                                     const fwp_tensor* Rv, const fwp_tensor* rb,
                                                     const fwp_tensor* fw_mem,
                                                     const fwp_tensor* grad_q, const fwp_tensor* grad_k,
                                                     const fwp_tensor* grad_v, const fwp_tensor* grad_beta,
                                                     const fwp_tensor* grad_Rq, const fwp_tensor* grad_Rk,
                                                     const fwp_tensor* grad_Rv, const fwp_tensor* grad_rb,
                                                     int io_dtype, void* stream, int device) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (io_dtype != FWP_F32) return FWP_ERR_DTYPE;          // the same order of checks as the regular entry point,
    if (!pad_dim(D)) return FWP_ERR_UNSUPPORTED;            // so an unsupported call reports the same status from both
    if (fwp_rec_update_fwm_tanh_scratch_floats(N, H, D) > (int64_t)FWP_NOALLOC_SCRATCH_FLOATS)
        return FWP_ERR_NOALLOC_TOO_LARGE;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    int dev = device;
    if (dev < 0) {
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return set_cuda_error(e);
    }
    if (dev >= kMaxDevices) return FWP_ERR_SHAPE;
    float* scratch;
    {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!g_noalloc_ptr[dev]) {      // first call on this device: resolve the array's device address
            void* ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
            if (e != cudaSuccess) return set_cuda_error(e);
            g_noalloc_ptr[dev] = static_cast<float*>(ptr);
        }
        scratch = g_noalloc_ptr[dev];
    }
    return fwp_rec_update_fwm_tanh_backward(N, H, L, D, q, k, v, beta, v_old, o_delayed, grad_out, Rq, Rk, Rv, rb,
                                            fw_mem, grad_q, grad_k, grad_v, grad_beta, grad_Rq, grad_Rk, grad_Rv,
                                            grad_rb, scratch, (int64_t)FWP_NOALLOC_SCRATCH_FLOATS, io_dtype, stream,
                                            device);
}
