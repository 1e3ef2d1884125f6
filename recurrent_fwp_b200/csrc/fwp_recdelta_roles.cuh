// Backward of the recurrent delta net at d = 32: a chain warp and a trailing warp per sequence.
//
// Everything but the parameter gradients sits on the chain here: the gradient handed back through tanh(y_{t-1})
// needs dq, dk (both matrices G and S), their softmax backward and the three products with the rows of R.  A
// hand-off between warps costs about 140 cycles against 33 for an exchange inside a warp, so one warp X runs the
// whole chain with G by columns, G by rows and S by rows in registers (R by rows in shared memory), and prepares
// whatever does not wait for the chain one step early:
//   S is rewound first (that needs inputs only), so  dq = S_{t-1} g + k (u.g)  and  dk = G u + q (u.g) - S_{t-1} dv
//   with G u, G^T k and q.k taken before g is known; r = G^T k + (q.k) g.
// Vectors are fetched from shared memory where they are used instead of being kept across the step, so that the
// three matrices and at most three vectors are live at a time (no spills).  The second warp Y trails one chunk of
// steps behind, reads dq~, dk~, dv, db~ from a ring and does the three outer-product accumulations of the parameter
// gradients and the four stores.
#pragma once

namespace fwp {

template <int TC>
struct RecRolesSmem {
    static constexpr int D = 32;
    using Stage = RecBwdStage<D, TC>;
    static constexpr int kStages = 3;                 // X on chunk j, Y on chunk j - 1, chunk j + 1 in flight
    static constexpr int kStep = 4 * D;               // per step: dq~, dk~, dv, db~ (lane 0)
    static constexpr int kRing = TC * kStep;
    static constexpr int kRS = D + 4;                 // padded row stride of the R copies
    static constexpr int kR = 3 * D * kRS + D;        // Rq, Rk, Rv rows + rb
    static constexpr int kX = 2 * D;                  // X's exchange vectors: g, u
    static constexpr int kTable = (sizeof(StageTable) + 15) / 16 * 4;
    static constexpr int kFloats = kStages * Stage::kFloats + 2 * kRing + kR + kX + kTable;
};

template <int TC>
__global__ void __launch_bounds__(256, 1) rec_bwd_roles32_kernel(const RecBwdParams p) {
    constexpr int D = 32, NP = 16, NT = 64;
    using SM = RecRolesSmem<TC>;
    using Stage = typename SM::Stage;
    const int nslots = blockDim.x / NT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = warp % nslots, role = warp / nslots;
    const int stid = role * 32 + lane;
    const int seq = blockIdx.x * nslots + slot;
    const int n = seq / p.H, h = seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = smem_all + (size_t)slot * SM::kFloats;
    for (int i = stid; i < SM::kFloats - SM::kTable; i += NT) smem[i] = 0.f;
    float* ring = smem + SM::kStages * Stage::kFloats;
    float* rmem = ring + 2 * SM::kRing;             // R rows: [3][D][kRS], then rb[D]
    float* xg = rmem + SM::kR;
    float* xu = xg + D;
    StageTable* tb = reinterpret_cast<StageTable*>(xu + D);
    if (stid == 0) {                // tile order of RecBwdStage: q, k, v, v_old, od, gy
        stage_table_set(tb, 0, p.q, n, h);
        stage_table_set(tb, 1, p.k, n, h);
        stage_table_set(tb, 2, p.v, n, h);
        stage_table_set(tb, 3, p.v_old, n, h);
        stage_table_set(tb, 4, p.od, n, h);
        stage_table_set(tb, 5, p.gy, n, h);
        stage_table_set_col(tb, 0, p.beta, n, h);
    }
    slot_barrier(slot, NT);         // the zero fill is complete
    for (int i = stid; i < D * D; i += NT) {
        const int e = i / D, m = i - e * D;
        const long long src = h * p.rH + (long long)e * p.rE + m;
        rmem[0 * D * SM::kRS + e * SM::kRS + m] = p.Rq[src];
        rmem[1 * D * SM::kRS + e * SM::kRS + m] = p.Rk[src];
        rmem[2 * D * SM::kRS + e * SM::kRS + m] = p.Rv[src];
    }
    if (stid < D) rmem[3 * D * SM::kRS + stid] = p.rb[h * p.rbH + stid];

    float* W = p.W + n * p.wN + h * p.wH;
    // X: A = G by columns, B = S by rows, C = G by rows.  Y: A, B, C = the partial gradients of Rq, Rk, Rv by columns.
    f2 A[NP], B[NP], C[NP];
#pragma unroll
    for (int i = 0; i < NP; i++) { A[i] = 0ull; B[i] = 0ull; C[i] = 0ull; }
    if (role == 0) {
        float v[2];
#pragma unroll
        for (int i = 0; i < D; i++) {
            v[i & 1] = W[(long long)lane * p.wE + i];
            if (i & 1) B[i >> 1] = f2_pack(v[0], v[1]);
        }
    }
    float arb = 0.f;

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        stage_table_issue<TC, NT>(smem + (j % SM::kStages) * Stage::kFloats, tb, 6, 1, t0, nt, stid);
    };
    issue(0);
    float gh = 0.f;
    for (int j = 0; j <= nchunks; j++) {
        cp_async_wait<0>();
        slot_barrier(slot, NT);     // chunk j's tiles (and, first time, the R rows) are in place
        if (j + 1 < nchunks) issue(j + 1);
        if (role == 0 && j < nchunks) {
            // ------------------------------------------------------------ X: the chain
            Stage s; s.bind(smem + (j % SM::kStages) * Stage::kFloats);
            const int c = nchunks - 1 - j;
            const int nt = min(TC, p.L - c * TC);
            float* rg = ring + (j & 1) * SM::kRing;
            const float* rrow = rmem + lane * SM::kRS;
            const float rbl = rmem[3 * D * SM::kRS + lane];
            float r0, qk, dk0, w, beta, qe, ke, ul;
            // Everything of step t that does not wait for g_h, in two parts.  The scalars and the vector u go out
            // first (u through shared memory, with whatever exchange comes next); the products follow a barrier:
            // r0 = (G k) and q.k for the head of the step, the early rewind of S and dk0 = G u.  The step loop runs
            // them for step t - 1 inside step t, without a branch: at t = 0 they repeat step 0 with `live` = 0 (the
            // rewind then adds zero), so that the compiler may schedule them beside the end of the step.
            auto prep_scalars = [&](int t) {
                const int o = t * D + lane;
                beta = s.b.f[t];
                w = s.v.f[o] - s.vo.f[o];
                qe = s.q.f[o];
                ke = s.k.f[o];
                ul = beta * w;
                xu[lane] = ul;
            };
            auto prep_products = [&](int t, float live) {
                f2 va[NP], vb[NP];
                lds_slice<D>(va, s.q.f + t * D);
                lds_slice<D>(vb, s.k.f + t * D);
                r0 = dot2<NP>(A, vb);
                qk = dot2<NP>(va, vb);
                lds_slice<D>(va, xu);
                axpy2<NP>(B, va, -ke * live);       // S_{t-1}
                dk0 = dot2<NP>(C, va);
            };
            prep_scalars(nt - 1);
            __syncwarp();
            prep_products(nt - 1, 1.f);
#pragma unroll 1
            for (int t = nt - 1; t >= 0; t--) {
                const int o = t * D + lane;
                float* e = rg + t * SM::kStep;
                const float hte = s.od.f[o];
                const float gcol = s.gy.f[o] + gh;
                const float r = fmaf(qk, gcol, r0);
                const float dv = beta * r;
                xg[lane] = gcol;
                e[2 * D + lane] = dv;
                // u.g and db from lane products, in one shuffle sequence beside the exchange
                float pgu = gcol * ul, pdb = r * w;
#pragma unroll
                for (int sft = 16; sft >= 1; sft >>= 1) {
                    pgu += __shfl_xor_sync(0xffffffffu, pgu, sft);
                    pdb += __shfl_xor_sync(0xffffffffu, pdb, sft);
                }
                const float dbh = pdb * beta * (1.f - beta);
                f2 gv[NP], dvv[NP];
                // G by columns takes this step's own vectors: += q (x) g, -= k (x) dv (the vectors come back from the tiles)
                lds_slice<D>(gv, s.q.f + t * D);
                axpy2<NP>(A, gv, gcol);
                lds_slice<D>(dvv, s.k.f + t * D);
                axpy2<NP>(A, dvv, -dv);
                __syncwarp();
                lds_slice<D>(gv, xg);
                lds_slice<D>(dvv, e + 2 * D);
                const float sg = dot2<NP>(B, gv);
                const float sdv = dot2<NP>(B, dvv);
                const float dq = fmaf(ke, pgu, sg);
                const float dk = fmaf(qe, pgu, dk0) - sdv;
                // the two softmax backward maps: both sums in one shuffle sequence
                float pq = qe * dq, pk = ke * dk;
#pragma unroll
                for (int sft = 16; sft >= 1; sft >>= 1) {
                    pq += __shfl_xor_sync(0xffffffffu, pq, sft);
                    pk += __shfl_xor_sync(0xffffffffu, pk, sft);
                }
                // the part of the feedback that needs dv only, and the two updates of G by rows: placed ahead of the
                // stores below so that they may be scheduled inside the shuffle sequence above
                f2 rr[NP];
                lds_slice<D>(rr, rrow + 2 * D * SM::kRS);
                float back = fmaf(rbl, dbh, dot2<NP>(rr, dvv));
                axpy2<NP>(C, gv, qe);               // G by rows: += q (x) g, -= k (x) dv
                axpy2<NP>(C, dvv, -ke);
                const float dqh = qe * (dq - pq), dkh = ke * (dk - pk);
                e[lane] = dqh;
                e[D + lane] = dkh;
                if (lane == 0) e[3 * D] = dbh;
                const int tn = t > 0 ? t - 1 : 0;
                prep_scalars(tn);                   // the next step's u travels with this exchange
                __syncwarp();
                lds_slice<D>(gv, e);                // dq~
                lds_slice<D>(rr, rrow);
                back += dot2<NP>(rr, gv);
                lds_slice<D>(dvv, e + D);           // dk~
                lds_slice<D>(rr, rrow + D * SM::kRS);
                back += dot2<NP>(rr, dvv);
                gh = (1.f - hte * hte) * back;
                prep_products(tn, t > 0 ? 1.f : 0.f);
            }
        } else if (role == 1 && j > 0) {
            // ------------------------------------------------------------ Y: one chunk behind
            const int jj = j - 1;
            Stage s; s.bind(smem + (jj % SM::kStages) * Stage::kFloats);
            const int c = nchunks - 1 - jj;
            const int t0 = c * TC, nt = min(TC, p.L - t0);
            const float* rg = ring + (jj & 1) * SM::kRing;
            const long long tl = t0 + nt - 1;
            float* pgq = reinterpret_cast<float*>(p.gq.p) + n * p.gq.sN + h * p.gq.sH + tl * p.gq.sL + lane;
            float* pgk = reinterpret_cast<float*>(p.gk.p) + n * p.gk.sN + h * p.gk.sH + tl * p.gk.sL + lane;
            float* pgv = reinterpret_cast<float*>(p.gv.p) + n * p.gv.sN + h * p.gv.sH + tl * p.gv.sL + lane;
            float* pgb = reinterpret_cast<float*>(p.gb.p) + n * p.gb.sN + h * p.gb.sH + tl * p.gb.sL;
#pragma unroll 1
            for (int t = nt - 1; t >= 0; t--) {
                const float* e = rg + t * SM::kStep;
                const float dqh = e[lane], dkh = e[D + lane], dv = e[2 * D + lane], dbh = e[3 * D];
                const float hte = s.od.f[t * D + lane];
                f2 hs[NP];
                lds_slice<D>(hs, s.od.f + t * D);
                axpy2<NP>(A, hs, dqh);
                axpy2<NP>(B, hs, dkh);
                axpy2<NP>(C, hs, dv);
                arb += hte * dbh;
                *pgq = dqh; *pgk = dkh; *pgv = dv;
                if (lane == 0) *pgb = dbh;
                pgq -= p.gq.sL; pgk -= p.gk.sL; pgv -= p.gv.sL; pgb -= p.gb.sL;
            }
        }
    }
    if (role == 0) {
#pragma unroll
        for (int i = 0; i < D; i++) {
            float lo, hi;
            f2_unpack(B[i >> 1], lo, hi);
            W[(long long)lane * p.wE + i] = (i & 1) ? hi : lo;
        }
    } else {
        // partial parameter gradients of this (n, h): [3][d][d] then [d]; lane = column m, element (e, m) at e d + m
        float* out = p.scratch + (long long)seq * (3 * D * D + D);
#pragma unroll
        for (int i = 0; i < D; i++) {
            float lo, hi;
            f2_unpack(A[i >> 1], lo, hi);
            out[i * D + lane] = (i & 1) ? hi : lo;
            f2_unpack(B[i >> 1], lo, hi);
            out[D * D + i * D + lane] = (i & 1) ? hi : lo;
            f2_unpack(C[i >> 1], lo, hi);
            out[2 * D * D + i * D + lane] = (i & 1) ? hi : lo;
        }
        out[3 * D * D + lane] = arb;
    }
}

}  // namespace fwp
