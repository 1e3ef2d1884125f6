// Backward of the delta RNN (v2 and v1) at d <= 32: a chain warp and a trailing warp per sequence.
//
// The backward of one step (time reversed) is a chain  g_h -> g = gy + g_h -> r = G^T k -> br = beta r ->
// gs = S_t g -> softmax backward -> g_h  plus work that nothing on the chain waits for: the key gradient
// (G by rows and the rewound S_{t-1}), the beta gradient and the stores.  A hand-off between two warps costs about
// 140 cycles on this machine (named barrier or flag, measured), four times a round trip through shared memory
// inside one warp, so the chain stays inside one warp and only one-way traffic crosses warps:
//   warp X (chain)    holds G by columns and S by rows; r is taken as r0 + (x.k) g with r0 = G^T k and x.k prepared
//                     before g_h is known; it leaves g, u = beta (v - v_old), br and r w of every step in a ring;
//   warp Y (trailing) holds G by rows and its own copy of S (rewinding S needs only inputs), runs one chunk of
//                     steps behind X, reads the ring and produces the key and beta gradients and all four stores.
// The two warps meet once per chunk on a named barrier; that is also where staged input tiles change hands.
#pragma once

namespace fwp {

template <int TC, bool V1>
struct RnnRolesSmem {
    static constexpr int D = 32;
    using Stage = RnnBwdStage<D, TC, V1>;
    static constexpr int kStages = 3;                 // X on chunk j, Y on chunk j - 1, chunk j + 1 in flight
    static constexpr int kStep = 4 * D;               // per step: g, u, br, r w
    static constexpr int kRing = TC * kStep;
    static constexpr int kTable = (sizeof(StageTable) + 15) / 16 * 4;
    static constexpr int kFloats = kStages * Stage::kFloats + 2 * kRing + kTable;
};

template <int TC, bool V1>
__global__ void __launch_bounds__(256, 1) rnn_bwd_roles32_kernel(const RnnBwdParams p) {
    constexpr int D = 32, NP = 16, NT = 64;
    using SM = RnnRolesSmem<TC, V1>;
    using Stage = typename SM::Stage;
    const int nslots = blockDim.x / NT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = warp % nslots, role = warp / nslots;       // the two warps of a sequence share a scheduler
    const int stid = role * 32 + lane;
    const int seq = blockIdx.x * nslots + slot;
    const int n = seq / p.H, h = seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = smem_all + (size_t)slot * SM::kFloats;
    for (int i = stid; i < SM::kFloats - SM::kTable; i += NT) smem[i] = 0.f;
    float* ring = smem + SM::kStages * Stage::kFloats;

    StageTable* tb = reinterpret_cast<StageTable*>(ring + 2 * SM::kRing);
    if (stid == 0) {                // tile order of RnnBwdStage: k, v, gy, v_old, od, (out)
        stage_table_set(tb, 0, p.k, n, h);
        stage_table_set(tb, 1, p.v, n, h);
        stage_table_set(tb, 2, p.gy, n, h);
        stage_table_set(tb, 3, p.v_old, n, h);
        stage_table_set(tb, 4, p.od, n, h);
        if (V1) stage_table_set(tb, 5, p.out, n, h);
        stage_table_set_col(tb, 0, p.beta, n, h);
    }

    const int col = lane;           // the head dimension is exactly 32 (the launcher sends other sizes elsewhere)
    float* W = p.W + n * p.wN + h * p.wH;
    f2 Sr[NP], Gm[NP];              // S by rows (both warps); X: G by columns, Y: G by rows
    {
        float v[2];
#pragma unroll
        for (int i = 0; i < D; i++) {
            v[i & 1] = W[(long long)lane * p.wE + i];
            if (i & 1) Sr[i >> 1] = f2_pack(v[0], v[1]);
        }
#pragma unroll
        for (int i = 0; i < NP; i++) Gm[i] = 0ull;
    }
    slot_barrier(slot, NT);      // the zero fill is complete before the first copies land

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        stage_table_issue<TC, NT>(smem + (j % SM::kStages) * Stage::kFloats, tb, V1 ? 6 : 5, 1, t0, nt, stid);
    };
    issue(0);
    float gh = 0.f;                 // X: the gradient handed back through the recurrence (lane = feature index)
    for (int j = 0; j <= nchunks; j++) {
        cp_async_wait<0>();
        slot_barrier(slot, NT);  // chunk j's tiles have landed; X is through chunk j - 1, Y through j - 2
        if (j + 1 < nchunks) issue(j + 1);      // into the stage Y has just left
        if (role == 0 && j < nchunks) {
            // ------------------------------------------------------------ X: the chain
            Stage s; s.bind(smem + (j % SM::kStages) * Stage::kFloats);
            const int c = nchunks - 1 - j;
            const int nt = min(TC, p.L - c * TC);
            float* rg = ring + (j & 1) * SM::kRing;
            f2 xs[NP], kk[NP];
            float r0, xk, w, beta;
            auto prep = [&](int t) {                // everything of step t that does not wait for g_h
                lds_slice<D>(xs, s.od.f + t * D);
                lds_slice<D>(kk, s.k.f + t * D);
                r0 = dot2<NP>(Gm, kk);
                xk = dot2<NP>(xs, kk);
                beta = s.b.f[t];
                w = s.v.f[t * D + lane] - s.vo.f[t * D + lane];
                rg[t * SM::kStep + D + lane] = beta * w;
            };
            prep(nt - 1);
#pragma unroll 1
            for (int t = nt - 1; t >= 0; t--) {
                const float se = s.od.f[t * D + lane], ke = s.k.f[t * D + lane];
                float gcol = s.gy.f[t * D + lane] + gh;
                if constexpr (V1) {
                    const float hm = s.out.f[t * D + lane];
                    const float dotp = warp_sum_idx<1>(hm * gcol);
                    gcol = hm * (gcol - dotp);
                }
                const float r = fmaf(xk, gcol, r0);
                const float br = beta * r;
                rg[t * SM::kStep + lane] = gcol;
                rg[t * SM::kStep + 2 * D + lane] = br;
                rg[t * SM::kStep + 3 * D + lane] = r * w;
                // G takes this step's own vectors, so it is brought to G_{t-1} here, and the next step is prepared
                // (without a branch: the last call of a chunk repeats step 0, which rewrites the same ring entry)
                // beside the exchange and the reduction below: once g_h is known the next step starts at once
                axpy2<NP>(Gm, xs, gcol);
                axpy2<NP>(Gm, kk, -br);
                __syncwarp();
                f2 vg[NP], vu[NP];                  // two register sets: u is in flight during the product and the reduction
                lds_slice<D>(vg, rg + t * SM::kStep);
                lds_slice<D>(vu, rg + t * SM::kStep + D);
                const float gs = dot2<NP>(Sr, vg);
                prep(t > 0 ? t - 1 : 0);
                if constexpr (V1) {
                    gh = gs;
                } else {
                    const float dotp = warp_sum_idx<1>(se * gs);
                    gh = se * (gs - dotp);
                }
                axpy2<NP>(Sr, vu, -ke);             // S_{t-1}
            }
        } else if (role == 1 && j > 0) {
            // ------------------------------------------------------------ Y: one chunk behind
            const int jj = j - 1;
            Stage s; s.bind(smem + (jj % SM::kStages) * Stage::kFloats);
            const int c = nchunks - 1 - jj;
            const int t0 = c * TC, nt = min(TC, p.L - t0);
            const float* rg = ring + (jj & 1) * SM::kRing;
            const long long tl = t0 + nt - 1;
            float* pgk = reinterpret_cast<float*>(p.gk.p) + n * p.gk.sN + h * p.gk.sH + tl * p.gk.sL + col;
            float* pgz = reinterpret_cast<float*>(p.gz.p) + n * p.gz.sN + h * p.gz.sH + tl * p.gz.sL + col;
            float* pgv = reinterpret_cast<float*>(p.gv.p) + n * p.gv.sN + h * p.gv.sH + tl * p.gv.sL + col;
            float* pgb = reinterpret_cast<float*>(p.gb.p) + n * p.gb.sN + h * p.gb.sH + tl * p.gb.sL;
#pragma unroll 1
            for (int t = nt - 1; t >= 0; t--) {
                const float se = s.od.f[t * D + lane], ke = s.k.f[t * D + lane];
                const float* e = rg + t * SM::kStep;
                const float gl = e[lane], bl = e[2 * D + lane];
                const float db = warp_sum_idx<1>(e[3 * D + lane]);
                f2 vg[NP], vu[NP], vb[NP];          // three register sets: the loads go out together
                lds_slice<D>(vg, e);
                lds_slice<D>(vu, e + D);
                lds_slice<D>(vb, e + 2 * D);
                axpy2<NP>(Gm, vg, se);
                const float dkg = dot2<NP>(Gm, vu);
                axpy2<NP>(Sr, vu, -ke);             // S_{t-1}
                const float dk = dkg - dot2<NP>(Sr, vb);
                axpy2<NP>(Gm, vb, -ke);
                *pgk = dk; *pgz = gl; *pgv = bl;
                if (lane == 0) *pgb = db;
                pgk -= p.gk.sL; pgz -= p.gz.sL; pgv -= p.gv.sL; pgb -= p.gb.sL;
            }
        }
    }
    if (role == 0) {
#pragma unroll
        for (int i = 0; i < D; i++) {
            float lo, hi;
            f2_unpack(Sr[i >> 1], lo, hi);
            W[(long long)lane * p.wE + i] = (i & 1) ? hi : lo;
        }
    }
}

}  // namespace fwp
