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
            const Row4& rk = q == 0 ? p.gk[0] : (q == 1 ? p.gk[1] : p.gk[2]);
            const Row4& rz = q == 0 ? p.gz[0] : (q == 1 ? p.gz[1] : p.gz[2]);
            const Row4& rv = q == 0 ? p.gv[0] : (q == 1 ? p.gv[1] : p.gv[2]);
            const Row4& rb = q == 0 ? p.gb[0] : (q == 1 ? p.gb[1] : p.gb[2]);
            const long long tl = t0 + nt - 1;
            float* pgk = reinterpret_cast<float*>(rk.p) + n * rk.sN + h * rk.sH + tl * rk.sL + col;
            float* pgz = reinterpret_cast<float*>(rz.p) + n * rz.sN + h * rz.sH + tl * rz.sL + col;
            float* pgv = reinterpret_cast<float*>(rv.p) + n * rv.sN + h * rv.sH + tl * rv.sL + col;
            float* pgb = reinterpret_cast<float*>(rb.p) + n * rb.sN + h * rb.sH + tl * rb.sL;
            const long long sgk = rk.sL, sgz = rz.sL, sgv = rv.sL, sgb = rb.sL;
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

}  // namespace fwp
