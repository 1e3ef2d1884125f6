// Backward of the delta LSTM (v1..v4) at d <= 32: a chain warp and one trailing warp per gate.
//
// Time reversed, the only quantities one step hands to the next are the gradient of the fed-back output g_h and
// the cell gradient g_c.  The chain is  g_h, g_c -> dz[3] (element-wise) -> sum over the gates of S^q_t dz^q ->
// (softmax backward) -> g_h;  the value, key and beta gradients of the three delta rules hang off dz but feed
// nothing back.  So per sequence
//   warp X      holds S^i, S^u, S^o by rows, runs the chain, rewinds the matrices (that needs inputs only) and
//               leaves dz[3], u[3] = beta (v - v_old) and the z-gradient of the update gate in a ring;
//   warp H_q    (q = i, u, o) holds G^q by columns, G^q by rows and its own copy of S^q, runs one chunk of steps
//               behind X, and produces the gate's value, key, beta and z gradients and their stores.
// The four warps of a sequence meet once per chunk on a named barrier (that is also where staged input tiles
// change hands); nothing else crosses warps, because a hand-off costs about 140 cycles on this machine against 33
// for an exchange inside a warp.  Twelve matrices per sequence do not fit the register file for 512 sequences at
// once, so a CTA carries two sequences and the grid runs in two waves of a much shorter step.
#pragma once

namespace fwp {

template <int TC>
struct LstmRolesSmem {
    static constexpr int D = 32;
    using Stage = LstmBwdStage<D, TC>;
    static constexpr int kStages = 3;                 // X on chunk j, the H warps on chunk j - 1, chunk j + 1 in flight
    static constexpr int kStep = 7 * D;               // per step: dz[3], u[3], z-gradient of gate u (variant 3)
    static constexpr int kRing = TC * kStep;
    static constexpr int kTable = (sizeof(StageTable) + 15) / 16 * 4;
    static constexpr int kFloats = kStages * Stage::kFloats + 2 * kRing + 3 * D + kTable;
};

template <int TC, int VAR>
__global__ void __launch_bounds__(256, 1) lstm_bwd_roles32_kernel(const LstmBwdParams p) {
    constexpr int D = 32, NP = 16, NT = 128;
    using SM = LstmRolesSmem<TC>;
    using Stage = typename SM::Stage;
    const int nslots = blockDim.x / NT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = warp % nslots, role = warp / nslots;       // role 0: X, 1..3: H of gate role - 1
    const int stid = role * 32 + lane;
    const int seq = blockIdx.x * nslots + slot;
    const int n = seq / p.H, h = seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = smem_all + (size_t)slot * SM::kFloats;
    for (int i = stid; i < SM::kFloats - SM::kTable; i += NT) smem[i] = 0.f;
    float* ring = smem + SM::kStages * Stage::kFloats;
    float* hbuf = ring + 2 * SM::kRing;

    StageTable* tb = reinterpret_cast<StageTable*>(hbuf + 3 * D);
    if (stid == 0) {                // tile order of LstmBwdStage: k, v, v_old, gate of each gate, then gy, out, od, cell, umc
        for (int a = 0; a < 3; a++) {
            stage_table_set(tb, 4 * a + 0, p.k[a], n, h);
            stage_table_set(tb, 4 * a + 1, p.v[a], n, h);
            stage_table_set(tb, 4 * a + 2, p.v_old[a], n, h);
            stage_table_set(tb, 4 * a + 3, p.gate[a], n, h);
            stage_table_set_col(tb, a, p.beta[a], n, h);
        }
        stage_table_set(tb, 12, p.gy, n, h);
        stage_table_set(tb, 13, p.out, n, h);
        if (VAR != 1) tb->src[13] = nullptr;
        stage_table_set(tb, 14, p.od, n, h);
        stage_table_set(tb, 15, p.cell, n, h);
        stage_table_set(tb, 16, p.umc, n, h);
    }

    const int col = lane;           // the head dimension is exactly 32 (the launcher sends other sizes elsewhere)
    auto load_w_rows = [&](f2 (&S)[NP], int q) {
        const float* W = p.W[q] + n * p.wN[q] + h * p.wH[q];
        float v[2];
#pragma unroll
        for (int i = 0; i < D; i++) {
            v[i & 1] = W[(long long)lane * p.wE[q] + i];
            if (i & 1) S[i >> 1] = f2_pack(v[0], v[1]);
        }
    };
    // X: M0, M1, M2 = S^i, S^u, S^o by rows.  H_q: M0 = G^q by columns, M1 = G^q by rows, M2 = S^q by rows.
    f2 M0[NP], M1[NP], M2[NP];
    if (role == 0) {
        load_w_rows(M0, 0);
        load_w_rows(M1, 1);
        load_w_rows(M2, 2);
    } else {
#pragma unroll
        for (int i = 0; i < NP; i++) { M0[i] = 0ull; M1[i] = 0ull; }
        if (role == 1) load_w_rows(M2, 0);
        else if (role == 2) load_w_rows(M2, 1);
        else load_w_rows(M2, 2);
    }
    slot_barrier(slot, NT);      // the zero fill is complete before the first copies land

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        stage_table_issue<TC, NT>(smem + (j % SM::kStages) * Stage::kFloats, tb, 17, 3, t0, nt, stid);
    };
    issue(0);
    float gh = 0.f, gc = 0.f;       // X: gradients handed back through the output and the cell
    // H_q: this gate's gradient streams, picked once (by value: a reference chosen at run time would make every
    // later field access an indexed load from the parameter bank)
    const int gq = role > 0 ? role - 1 : 0;
    const Row4 rk = gq == 0 ? p.gk[0] : (gq == 1 ? p.gk[1] : p.gk[2]);
    const Row4 rz = gq == 0 ? p.gz[0] : (gq == 1 ? p.gz[1] : p.gz[2]);
    const Row4 rv = gq == 0 ? p.gv[0] : (gq == 1 ? p.gv[1] : p.gv[2]);
    const Row4 rb = gq == 0 ? p.gb[0] : (gq == 1 ? p.gb[1] : p.gb[2]);
    float* const bgk = reinterpret_cast<float*>(rk.p) + n * rk.sN + h * rk.sH + col;
    float* const bgz = reinterpret_cast<float*>(rz.p) + n * rz.sN + h * rz.sH + col;
    float* const bgv = reinterpret_cast<float*>(rv.p) + n * rv.sN + h * rv.sH + col;
    float* const bgb = reinterpret_cast<float*>(rb.p) + n * rb.sN + h * rb.sH;
    const long long sgk = rk.sL, sgz = rz.sL, sgv = rv.sL, sgb = rb.sL;
    for (int j = 0; j <= nchunks; j++) {
        cp_async_wait<0>();
        slot_barrier(slot, NT);  // chunk j's tiles have landed; X is through chunk j - 1, the H warps through j - 2
        if (j + 1 < nchunks) issue(j + 1);      // into the stage the H warps have just left
        if (role == 0 && j < nchunks) {
            // ------------------------------------------------------------ X: the chain
            Stage s; s.bind(smem + (j % SM::kStages) * Stage::kFloats);
            const int c = nchunks - 1 - j;
            const int nt = min(TC, p.L - c * TC);
            float* rg = ring + (j & 1) * SM::kRing;
#pragma unroll 1
            for (int t = nt - 1; t >= 0; t--) {
                const int o = t * D + lane;
                float* e = rg + t * SM::kStep;
                // what the rewind and the trailing warps need and the chain does not
#pragma unroll
                for (int q = 0; q < 3; q++) e[(3 + q) * D + lane] = s.b[q].f[t] * (s.v[q].f[o] - s.vo[q].f[o]);
                const float gsum = s.gy.f[o] + gh;
                float a = gsum;
                if constexpr (VAR == 1) {
                    const float hm = s.out.f[o];
                    const float dotp = warp_sum_idx<1>(hm * gsum);
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
#pragma unroll
                for (int q = 0; q < 3; q++) e[q * D + lane] = dz[q];
                if constexpr (VAR == 3) e[6 * D + lane] = dz[1] + gsum;
                __syncwarp();
                // three vectors in three register sets: the loads go out together and the products overlap
                f2 va[NP], vb[NP], vc[NP];
                lds_slice<D>(va, e);
                lds_slice<D>(vb, e + D);
                lds_slice<D>(vc, e + 2 * D);
                const float k0 = s.k[0].f[o], k1 = s.k[1].f[o], k2 = s.k[2].f[o];
                float ghn = dot2<NP>(M0, va) + dot2<NP>(M1, vb) + dot2<NP>(M2, vc);
                lds_slice<D>(va, e + 3 * D);        // u[3] for the rewind: in flight during the reduction below
                lds_slice<D>(vb, e + 4 * D);
                lds_slice<D>(vc, e + 5 * D);
                if constexpr (VAR != 1) {
                    const float xe = s.od.f[o];
                    const float dotp = warp_sum_idx<1>(xe * ghn);
                    gh = xe * (ghn - dotp);
                } else {
                    gh = ghn;
                }
                axpy2<NP>(M0, va, -k0);             // S^q_{t-1}
                axpy2<NP>(M1, vb, -k1);
                axpy2<NP>(M2, vc, -k2);
            }
        } else if (role > 0 && j > 0) {
            // ------------------------------------------------------------ H_q: one chunk behind
            const int q = role - 1;
            const int jj = j - 1;
            Stage s; s.bind(smem + (jj % SM::kStages) * Stage::kFloats);
            const int c = nchunks - 1 - jj;
            const int t0 = c * TC, nt = min(TC, p.L - t0);
            const float* rg = ring + (jj & 1) * SM::kRing;
            float* hb = hbuf + q * D;
            const float* ktile = q == 0 ? s.k[0].f : (q == 1 ? s.k[1].f : s.k[2].f);
            const float* vtile = q == 0 ? s.v[0].f : (q == 1 ? s.v[1].f : s.v[2].f);
            const float* votile = q == 0 ? s.vo[0].f : (q == 1 ? s.vo[1].f : s.vo[2].f);
            const float* btile = q == 0 ? s.b[0].f : (q == 1 ? s.b[1].f : s.b[2].f);
            const long long tl = t0 + nt - 1;
            float* pgk = bgk + tl * sgk;
            float* pgz = bgz + tl * sgz;
            float* pgv = bgv + tl * sgv;
            float* pgb = bgb + tl * sgb;
#pragma unroll 1
            for (int t = nt - 1; t >= 0; t--) {
                const int o = t * D + lane;
                const float* e = rg + t * SM::kStep;
                const float dzl = e[q * D + lane];
                const float gzl = (VAR == 3 && q == 1) ? e[6 * D + lane] : dzl;
                const float beta = btile[t];
                const float w = vtile[o] - votile[o];
                const float xe = s.od.f[o], ke = ktile[o];
                // the four vectors that do not wait for this step's br, in four register sets
                f2 xs[NP], kk[NP], dr[NP], ur[NP];
                lds_slice<D>(xs, s.od.f + t * D);
                lds_slice<D>(kk, ktile + t * D);
                lds_slice<D>(dr, e + q * D);
                lds_slice<D>(ur, e + (3 + q) * D);
                // column role
                axpy2<NP>(M0, xs, dzl);
                const float r = dot2<NP>(M0, kk);
                const float br = beta * r;
                hb[lane] = br;
                // row role, the part before br
                axpy2<NP>(M1, dr, xe);
                float dk = dot2<NP>(M1, ur);
                axpy2<NP>(M2, ur, -ke);             // S^q_{t-1}
                axpy2<NP>(M0, kk, -br);
                const float db = warp_sum_idx<1>(r * w);
                __syncwarp();
                lds_slice<D>(xs, hb);
                dk -= dot2<NP>(M2, xs);
                axpy2<NP>(M1, xs, -ke);
                __syncwarp();                       // everyone has read hb before the next step rewrites it
                *pgk = dk; *pgz = gzl; *pgv = br;
                if (lane == 0) *pgb = db;
                pgk -= sgk; pgz -= sgz; pgv -= sgv; pgb -= sgb;
            }
        }
    }
    if (role == 0) {
        auto store_w_rows = [&](const f2 (&S)[NP], int q) {
            float* W = p.W[q] + n * p.wN[q] + h * p.wH[q];
#pragma unroll
            for (int i = 0; i < D; i++) {
                float lo, hi;
                f2_unpack(S[i >> 1], lo, hi);
                W[(long long)lane * p.wE[q] + i] = (i & 1) ? hi : lo;
            }
        };
        store_w_rows(M0, 0);
        store_w_rows(M1, 1);
        store_w_rows(M2, 2);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Forward of the delta LSTM at d = 32 with one warp per gate.
//
// A step has three delta-rule updates and three read-outs, one per gate, and they meet only in the element-wise
// cell update.  Warp q of a sequence holds S^q, applies its update (inputs only, so it runs beside the chain),
// forms its pre-activation S^q_t^T x + z^q, applies its gate's nonlinearity and posts the gate; after the one
// barrier of the step every warp reads the three gates and computes the cell, the output and the next fed-back
// vector for itself (the same instructions on the same numbers in all three warps, so they agree bit for bit).  One barrier per step
// (about 110 cycles) buys a chain warp of about 150 instead of 400 instructions per step.
template <int TC>
struct LstmGatesSmem {
    static constexpr int D = 32;
    using Stage = LstmFwdStage<D, TC>;
    static constexpr int kStages = 2;
    static constexpr int kX = 3 * D;                  // the fed-back vector, one private copy per warp
    static constexpr int kP = 2 * 3 * D;              // posted pre-activations, two step parities
    static constexpr int kTable = (sizeof(StageTable) + 15) / 16 * 4;
    static constexpr int kFloats = kStages * Stage::kFloats + kX + kP + kTable;
};

template <int TC, int VAR>
__global__ void __launch_bounds__(384, 1) lstm_fwd_gates32_kernel(const LstmFwdParams p) {
    constexpr int D = 32, NP = 16, NT = 96;
    using SM = LstmGatesSmem<TC>;
    using Stage = typename SM::Stage;
    constexpr int kTile = r4(TC * D);
    const int nslots = blockDim.x / NT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = warp % nslots, q = warp / nslots;          // q: the gate this warp serves (0 = i, 1 = u, 2 = o)
    const int stid = q * 32 + lane;
    const int seq = blockIdx.x * nslots + slot;
    const int n = seq / p.H, h = seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = smem_all + (size_t)slot * SM::kFloats;
    for (int i = stid; i < SM::kFloats - SM::kTable; i += NT) smem[i] = 0.f;
    float* xv = smem + SM::kStages * Stage::kFloats + q * D;
    float* post = smem + SM::kStages * Stage::kFloats + SM::kX;
    StageTable* tb = reinterpret_cast<StageTable*>(post + SM::kP);
    if (stid == 0) {                // tile order of LstmFwdStage: z, k, v of each gate
        for (int a = 0; a < 3; a++) {
            stage_table_set(tb, 3 * a + 0, p.z[a], n, h);
            stage_table_set(tb, 3 * a + 1, p.k[a], n, h);
            stage_table_set(tb, 3 * a + 2, p.v[a], n, h);
            stage_table_set_col(tb, a, p.beta[a], n, h);
        }
    }
    // this warp's matrix and its three output streams
    // selected with compares, not with a run-time index (that would put the parameter block in local memory)
    float* const Wb = q == 0 ? p.W[0] : (q == 1 ? p.W[1] : p.W[2]);
    const long long wN = q == 0 ? p.wN[0] : (q == 1 ? p.wN[1] : p.wN[2]);
    const long long wH = q == 0 ? p.wH[0] : (q == 1 ? p.wH[1] : p.wH[2]);
    const long long wE = q == 0 ? p.wE[0] : (q == 1 ? p.wE[1] : p.wE[2]);
    const Row4& rgate = q == 0 ? p.gate[0] : (q == 1 ? p.gate[1] : p.gate[2]);
    const Row4& rvold = q == 0 ? p.v_old[0] : (q == 1 ? p.v_old[1] : p.v_old[2]);
    float* W = Wb + n * wN + h * wH;
    f2 S[NP];
    {
        float v[2];
#pragma unroll
        for (int i = 0; i < D; i++) {       // column m = lane: element (e, m)
            v[i & 1] = W[(long long)i * wE + lane];
            if (i & 1) S[i >> 1] = f2_pack(v[0], v[1]);
        }
    }
    auto colptr = [&](const Row4& r) { return reinterpret_cast<float*>(r.p) + n * r.sN + h * r.sH + lane; };
    // stores are shared out: every warp writes its gate and its v_old, and one of out / cell / fed-back vector
    float* pg = colptr(rgate);
    float* pvo = colptr(rvold);
    const Row4& third = q == 0 ? p.out : (q == 1 ? p.cell : p.nmz);
    const bool has_third = q < 2 || VAR != 1;
    float* p3 = has_third ? colptr(third) : pg;
    const long long sg = rgate.sL, svo = rvold.sL, s3 = has_third ? third.sL : 0;
    float* hp = p.h + n * p.hN + h * p.hH;
    float* cp = p.c + n * p.cN + h * p.cH;
    float hv = hp[lane], cv = cp[lane];
    slot_barrier(slot, NT);         // the zero fill is complete before the first copies land

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int c) {
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        stage_table_issue<TC, NT>(smem + (c & 1) * Stage::kFloats, tb, 9, 3, t0, nt, stid);
    };
    issue(0);
    int par = 0;
    for (int c = 0; c < nchunks; c++) {
        cp_async_wait<0>();
        slot_barrier(slot, NT);     // chunk c has landed; everyone is through chunk c - 1
        if (c + 1 < nchunks) issue(c + 1);
        const float* base = smem + (c & 1) * Stage::kFloats;
        const float* zcol = base + (3 * q) * kTile + lane;          // z of this gate
        const float* krow = base + (3 * q + 1) * kTile;             // k of this gate
        const float* vcol = base + (3 * q + 2) * kTile + lane;      // v of this gate
        const float* zu = base + 3 * kTile + lane;                  // z of the update gate (variant 3)
        const float* brow = base + 9 * kTile + q * r4(TC);
        const int nt = min(TC, p.L - c * TC);
#pragma unroll 1
        for (int t = 0; t < nt; t++, zcol += D, krow += D, vcol += D, zu += D, brow++) {
            float* pp = post + par * (3 * D);
            par ^= 1;
            // this gate's delta update (inputs only)
            f2 kk[NP];
            lds_slice<D>(kk, krow);
            const float vo = dot2<NP>(S, kk);
            const float u = brow[0] * (vcol[0] - vo);
            axpy2<NP>(S, kk, u);
            // the fed-back vector, computed by every warp for itself
            float xe;
            if constexpr (VAR == 1) {
                xe = hv;
            } else {
                const float mx = warp_max_f32(hv);
                xe = exp_neg(hv - mx);
                xe *= rcp_approx(warp_sum_unit_scaled(xe) * (1.f / 67108864.f) + kLstmEps);
            }
            xv[lane] = xe;
            __syncwarp();
            f2 xs[NP];
            lds_slice<D>(xs, xv);
            // each warp posts its gate already activated: one sigmoid per warp and step instead of three
            const float pre = dot2<NP>(S, xs) + zcol[0];
            pp[q * D + lane] = (VAR == 4 && q == 1) ? pre : sigmoidf_(pre);
            slot_barrier(slot, NT);
            const float gi = pp[lane], uu = pp[D + lane], go = pp[2 * D + lane];
            cv = gi * uu + (1.f - gi) * cv;
            float hn = go * cv;
            if constexpr (VAR == 1) {
                const float mx = warp_max_f32(hn);
                const float ex = exp_neg(hn - mx);
                hn = ex * rcp_approx(warp_sum_unit_scaled(ex) * (1.f / 67108864.f));
            } else if constexpr (VAR == 3) {
                hn += zu[0];
            }
            hv = hn;
            *pg = q == 0 ? gi : (q == 1 ? uu : go);
            *pvo = vo;
            if (has_third) *p3 = q == 0 ? hn : (q == 1 ? cv : xe);
            pg += sg; pvo += svo; p3 += s3;
        }
    }
#pragma unroll
    for (int i = 0; i < D; i++) {
        float lo, hi;
        f2_unpack(S[i >> 1], lo, hi);
        W[(long long)i * wE + lane] = (i & 1) ? hi : lo;
    }
    if (q == 0) { hp[lane] = hv; cp[lane] = cv; }
}

}  // namespace fwp
