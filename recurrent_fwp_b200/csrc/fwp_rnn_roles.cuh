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

__device__ __forceinline__ void named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

template <int TC, bool V1>
struct RnnRolesSmem {
    static constexpr int D = 32;
    using Stage = RnnBwdStage<D, TC, V1>;
    static constexpr int kStages = 3;                 // X on chunk j, Y on chunk j - 1, chunk j + 1 in flight
    static constexpr int kStep = 4 * D;               // per step: g, u, br, r w
    static constexpr int kRing = TC * kStep;
    static constexpr int kFloats = kStages * Stage::kFloats + 2 * kRing;
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
    const int bar_chunk = 1 + slot;
    extern __shared__ __align__(16) float smem_all[];
    float* smem = smem_all + (size_t)slot * SM::kFloats;
    for (int i = stid; i < SM::kFloats; i += NT) smem[i] = 0.f;
    float* ring = smem + SM::kStages * Stage::kFloats;

    Src<float> sk, sv, sg, so, sd, sb, sout;
    sk.init(p.k, n, h, p.D);
    sv.init(p.v, n, h, p.D);
    sg.init(p.gy, n, h, p.D);
    so.init(p.v_old, n, h, p.D);
    sd.init(p.od, n, h, p.D);
    sb.init(p.beta, n, h, 1);
    if (V1) sout.init(p.out, n, h, p.D);

    const bool ok = lane < p.D;
    const int col = ok ? lane : 0;
    float* W = p.W + n * p.wN + h * p.wH;
    f2 Sr[NP], Gm[NP];              // S by rows (both warps); X: G by columns, Y: G by rows
    {
        float v[2];
#pragma unroll
        for (int i = 0; i < D; i++) {
            v[i & 1] = (lane < p.D && i < p.D) ? W[(long long)lane * p.wE + i] : 0.f;
            if (i & 1) Sr[i >> 1] = f2_pack(v[0], v[1]);
        }
#pragma unroll
        for (int i = 0; i < NP; i++) Gm[i] = 0ull;
    }
    named_sync(bar_chunk, NT);      // the zero fill is complete before the first copies land

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int j) {
        Stage s; s.bind(smem + (j % SM::kStages) * Stage::kFloats);
        const int c = nchunks - 1 - j;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.k.template load<NT>(sk, t0, nt, stid);
        s.v.template load<NT>(sv, t0, nt, stid);
        s.gy.template load<NT>(sg, t0, nt, stid);
        s.vo.template load<NT>(so, t0, nt, stid);
        s.od.template load<NT>(sd, t0, nt, stid);
        if (V1) s.out.template load<NT>(sout, t0, nt, stid);
        s.b.template load<NT>(sb, t0, nt, stid);
        cp_async_commit();
    };
    issue(0);
    float gh = 0.f;                 // X: the gradient handed back through the recurrence (lane = feature index)
    for (int j = 0; j <= nchunks; j++) {
        cp_async_wait<0>();
        named_sync(bar_chunk, NT);  // chunk j's tiles have landed; X is through chunk j - 1, Y through j - 2
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
                __syncwarp();
                f2 vec[NP];
                lds_slice<D>(vec, rg + t * SM::kStep);
                const float gs = dot2<NP>(Sr, vec);
                if constexpr (V1) {
                    gh = gs;
                } else {
                    const float dotp = warp_sum_idx<1>(se * gs);
                    gh = se * (gs - dotp);
                }
                axpy2<NP>(Gm, xs, gcol);
                axpy2<NP>(Gm, kk, -br);
                lds_slice<D>(vec, rg + t * SM::kStep + D);
                axpy2<NP>(Sr, vec, -ke);            // S_{t-1}
                if (t > 0) prep(t - 1);
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
                f2 vec[NP];
                lds_slice<D>(vec, e);
                axpy2<NP>(Gm, vec, se);
                lds_slice<D>(vec, e + D);
                const float dkg = dot2<NP>(Gm, vec);
                axpy2<NP>(Sr, vec, -ke);            // S_{t-1}
                lds_slice<D>(vec, e + 2 * D);
                const float dk = dkg - dot2<NP>(Sr, vec);
                axpy2<NP>(Gm, vec, -ke);
                if (ok) { *pgk = dk; *pgz = gl; *pgv = bl; }
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
            if (lane < p.D && i < p.D) W[(long long)lane * p.wE + i] = (i & 1) ? hi : lo;
        }
    }
}

}  // namespace fwp
