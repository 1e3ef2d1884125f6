// Delta rule, four-step blocked form (sm_100a).
//
// The per-step kernels put one reduction round (dot, shuffle, scalar update) on
// the dependency chain of every time step.  Here four consecutive steps share one
// round: all eight matrix-vector products of a group are taken with the state at
// the *start* of the group and corrected with Gram scalars of the group's keys
// and queries, which do not depend on the state and are computed per chunk off
// the chain:
//
//   a_j = S^T k_j,  b_j = S^T q_j                      (S = state before the group)
//   v_old_j = a_j + sum_{i<j}  u_i (k_i . k_j) ;  u_j = beta_j (v_j - v_old_j)
//   y_j     = b_j + sum_{i<=j} u_i (k_i . q_j) ;  S += sum_j k_j (x) u_j
//
// Backward (time reversed inside a group), with G = dL/dS before the group:
//   a_j = G^T k_j
//   r_j = a_j + gy_j (q_j . k_j) + sum_{i later than j} ( gy_i (q_i . k_j) - beta_i r_i (k_i . k_j) )
//   G  += sum_j ( q_j (x) gy_j - k_j (x) beta_j r_j )
// and the row-role part (dq, dk, rewind of S) runs per step from the published u_j, beta_j r_j.
// The algebra is exact; only the fp32 summation order differs from the per-step form.
// Outputs are staged in shared memory and written per chunk with 16-byte stores.
#pragma once
#include "fwp_core.cuh"

namespace fwp {

template <int D, int TC, typename T>
struct BlkFwdStage {
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

template <int D, int TC, typename T>
struct BlkFwdSmem {
    static constexpr int kStage = BlkFwdStage<D, TC, T>::kFloats;
    static constexpr int kGram = (TC / 4) * 16;
    static constexpr int kOut = TC * D;
    static constexpr int kFloats = 2 * kStage + kGram + 3 * kOut;
};

// zero rows [r0, r1) of an fp32 tile with row length RL
template <int RL>
__device__ __forceinline__ void zero_rows(float* tile, int r0, int r1, int tid, int nthreads) {
    for (int i = r0 * RL + tid; i < r1 * RL; i += nthreads) tile[i] = 0.f;
}

template <int D, int SPLIT, int TC, typename T, bool SUM>
__global__ void __launch_bounds__(D * SPLIT) delta_fwd_kernel(const DeltaFwdParams p) {
    using G = Geo<D, SPLIT>;
    using SM = BlkFwdSmem<D, TC, T>;
    using Stage = BlkFwdStage<D, TC, T>;
    static_assert(TC % 4 == 0, "chunk must hold whole groups");
    constexpr bool KEEP = G::NR <= 16;     // keep the four key slices in registers between dot and update
    const G g;
    FWP_PROF_BEGIN
    const int n = blockIdx.x / p.H, h = blockIdx.x - n * p.H;
    extern __shared__ __align__(16) float smem[];
    for (int i = g.tid; i < SM::kFloats; i += G::NT) smem[i] = 0.f;
    float* gram = smem + 2 * SM::kStage;
    float* oy = gram + SM::kGram;
    float* ovo = oy + SM::kOut;
    float* ou = ovo + SM::kOut;

    Src<T> sq, sk, sv, sb;
    sq.init(p.q, n, h, p.E);
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    if (!SUM) sb.init(p.beta, n, h, 1);

    float* W = p.W + n * p.wN + h * p.wH;
    f2 S[G::NP];
    load_cols(g, S, W, p.wE, p.E, p.M);
    __syncthreads();

    const int nchunks = (p.L + TC - 1) / TC;
    auto issue = [&](int c) {
        Stage s; s.bind(smem + (c & 1) * SM::kStage);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        s.q.template load<G::NT>(sq, t0, nt, g.tid);
        s.k.template load<G::NT>(sk, t0, nt, g.tid);
        s.v.template load<G::NT>(sv, t0, nt, g.tid);
        if (!SUM) s.b.template load<G::NT>(sb, t0, nt, g.tid);
        cp_async_commit();
    };
    issue(0);
    FWP_PROF(0)
    for (int c = 0; c < nchunks; c++) {
        if (c + 1 < nchunks) { issue(c + 1); FWP_PROF(1) cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        FWP_PROF(2)
        Stage s; s.bind(smem + (c & 1) * SM::kStage);
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        const int ng = (nt + 3) >> 2;
        if constexpr (sizeof(T) != 4) {
            s.q.widen(nt, p.E, g.tid, G::NT);
            s.k.widen(nt, p.E, g.tid, G::NT);
            s.v.widen(nt, p.M, g.tid, G::NT);
            if (!SUM) s.b.widen(nt, 1, g.tid, G::NT);
        }
        if (nt & 3) {   // pad the last group with inert steps (k = q = v = beta = 0)
            zero_rows<D>(s.q.f, nt, 4 * ng, g.tid, G::NT);
            zero_rows<D>(s.k.f, nt, 4 * ng, g.tid, G::NT);
            zero_rows<D>(s.v.f, nt, 4 * ng, g.tid, G::NT);
            if (!SUM) zero_rows<1>(s.b.f, nt, 4 * ng, g.tid, G::NT);
        }
        if ((sizeof(T) != 4) || (nt & 3)) __syncthreads();
        gram_phase<D>(s.k.f, s.q.f, gram, ng, g.tid, G::NT);
        __syncthreads();
        FWP_PROF(3)

        for (int gi = 0; gi < ng; gi++) {
            const int tb = 4 * gi;
            float a[4], b[4];
            f2 kk[KEEP ? 4 : 1][G::NP];
            if constexpr (G::NR <= 8) {
                // small slices: fetch all eight operand slices first, then run the eight
                // dot-product chains interleaved so that no FMA waits on its predecessor
                f2 qq[4][G::NP];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    lds_slice<G::NR>(kk[j], s.k.f + (tb + j) * D + g.off);
                    lds_slice<G::NR>(qq[j], s.q.f + (tb + j) * D + g.off);
                }
                FWP_PROF(8)
                f2 aa[4] = {0ull, 0ull, 0ull, 0ull}, bb[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                for (int i = 0; i < G::NP; i++) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if constexpr (!SUM) aa[j] = ffma2(S[i], kk[j][i], aa[j]);
                        bb[j] = ffma2(S[i], qq[j][i], bb[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) { a[j] = SUM ? 0.f : f2_hsum(aa[j]); b[j] = f2_hsum(bb[j]); }
                FWP_PROF(9)
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    f2 (&kj)[G::NP] = kk[KEEP ? j : 0];
                    lds_slice<G::NR>(kj, s.k.f + (tb + j) * D + g.off);
                    if constexpr (!SUM) a[j] = dot2_chain<G::NP>(S, kj); else a[j] = 0.f;
                    f2 qq[G::NP];
                    lds_slice<G::NR>(qq, s.q.f + (tb + j) * D + g.off);
                    b[j] = dot2_chain<G::NP>(S, qq);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if constexpr (!SUM) a[j] = reduce_split<SPLIT>(a[j]);
                b[j] = reduce_split<SPLIT>(b[j]);
            }
            FWP_PROF(10)
            float gs[16];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float4 t4 = *reinterpret_cast<const float4*>(gram + gi * 16 + 4 * i);
                gs[4 * i] = t4.x; gs[4 * i + 1] = t4.y; gs[4 * i + 2] = t4.z; gs[4 * i + 3] = t4.w;
            }
            float be[4] = {1.f, 1.f, 1.f, 1.f};
            if constexpr (!SUM) {
                const float4 b4 = *reinterpret_cast<const float4*>(s.b.f + tb);
                be[0] = b4.x; be[1] = b4.y; be[2] = b4.z; be[3] = b4.w;
            }
            float u[4], vo[4], y[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float vv = s.v.f[(tb + j) * D + g.idx];
                if constexpr (SUM) {
                    vo[j] = 0.f;
                    u[j] = vv;
                } else {
                    float acc = a[j];
#pragma unroll
                    for (int i = 0; i < j; i++) acc = fmaf(u[i], gs[gram_kk(i, j)], acc);
                    vo[j] = acc;
                    u[j] = be[j] * (vv - acc);
                }
                float yy = b[j];
#pragma unroll
                for (int i = 0; i <= j; i++) yy = fmaf(u[i], gs[gram_kq(i, j)], yy);
                y[j] = yy;
            }
            FWP_PROF(11)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if constexpr (KEEP) {
                    axpy2<G::NP>(S, kk[j], u[j]);
                } else {
                    lds_slice<G::NR>(kk[0], s.k.f + (tb + j) * D + g.off);
                    axpy2<G::NP>(S, kk[0], u[j]);
                }
            }
            FWP_PROF(12)
            if (g.s == 0) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    oy[(tb + j) * D + g.idx] = y[j];
                    if constexpr (!SUM) {
                        ovo[(tb + j) * D + g.idx] = vo[j];
                        ou[(tb + j) * D + g.idx] = u[j];
                    }
                }
            }
            FWP_PROF(13)
        }
        __syncthreads();
        FWP_PROF(4)
        flush_rows<D, G::NT, T>(oy, p.out, n, h, t0, nt, p.M, g.tid);
        if constexpr (!SUM) {
            flush_rows<D, G::NT, float>(ovo, p.v_old, n, h, t0, nt, p.M, g.tid);
            if (p.v_ins.p) flush_rows<D, G::NT, float>(ou, p.v_ins, n, h, t0, nt, p.M, g.tid);
        }
        FWP_PROF(5)
    }
    store_cols(g, S, W, p.wE, p.E, p.M);
    FWP_PROF(6)
    FWP_PROF_END
}

// ------------------------------------------------------------------ backward
template <int D, int TC, typename T>
struct BlkBwdStage {
    Tile<D, TC, T> q, k, v, gy;
    Tile<D, TC, float> vo;
    Tile<1, TC, T> b;
    static constexpr int kFloats = 4 * r4(Tile<D, TC, T>::kFloats) + r4(TC * D) + r4(Tile<1, TC, T>::kFloats);
    __device__ __forceinline__ void bind(float* mem) {
        q.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        k.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        v.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        gy.bind(mem); mem += r4(Tile<D, TC, T>::kFloats);
        vo.bind(mem); mem += r4(TC * D);
        b.bind(mem);
    }
};

template <int D, int TC, typename T>
struct BlkBwdSmem {
    static constexpr int kStage = BlkBwdStage<D, TC, T>::kFloats;
    static constexpr int kGram = (TC / 4) * 16;
    static constexpr int kOut = TC * D;
    static constexpr int kXg = 8 * D + 32;          // per group parity: u[4][D], br[4][D], dbeta partials[4][8]
    static constexpr int kFloats = 2 * kStage + kGram + 3 * kOut + r4(TC) + 2 * kXg;
};

template <int D, int SPLIT, int TC, typename T>
__global__ void __launch_bounds__(D * SPLIT) delta_bwd_kernel(const DeltaBwdParams p) {
    using G = Geo<D, SPLIT>;
    using SM = BlkBwdSmem<D, TC, T>;
    using Stage = BlkBwdStage<D, TC, T>;
    static_assert(TC % 4 == 0, "chunk must hold whole groups");
    constexpr bool KEEP = G::NR <= 8;
    constexpr int HS = sum4_stride<SPLIT>();
    const G g;
    const int n = blockIdx.x / p.H, h = blockIdx.x - n * p.H;
    extern __shared__ __align__(16) float smem[];
    for (int i = g.tid; i < SM::kFloats; i += G::NT) smem[i] = 0.f;
    float* gram = smem + 2 * SM::kStage;
    float* odq = gram + SM::kGram;
    float* odk = odq + SM::kOut;
    float* odv = odk + SM::kOut;
    float* odb = odv + SM::kOut;
    float* xch = odb + r4(TC);

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
    auto issue = [&](int jc) {   // jc-th chunk counted from the end of the sequence
        Stage s; s.bind(smem + (jc & 1) * SM::kStage);
        const int c = nchunks - 1 - jc;
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
    int par = 0;
    for (int jc = 0; jc < nchunks; jc++) {
        if (jc + 1 < nchunks) { issue(jc + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        Stage s; s.bind(smem + (jc & 1) * SM::kStage);
        const int c = nchunks - 1 - jc;
        const int t0 = c * TC, nt = min(TC, p.L - t0);
        const int ng = (nt + 3) >> 2;
        if constexpr (sizeof(T) != 4) {
            s.q.widen(nt, p.E, g.tid, G::NT);
            s.k.widen(nt, p.E, g.tid, G::NT);
            s.v.widen(nt, p.M, g.tid, G::NT);
            s.gy.widen(nt, p.M, g.tid, G::NT);
            s.b.widen(nt, 1, g.tid, G::NT);
        }
        if (nt & 3) {
            zero_rows<D>(s.q.f, nt, 4 * ng, g.tid, G::NT);
            zero_rows<D>(s.k.f, nt, 4 * ng, g.tid, G::NT);
            zero_rows<D>(s.v.f, nt, 4 * ng, g.tid, G::NT);
            zero_rows<D>(s.gy.f, nt, 4 * ng, g.tid, G::NT);
            zero_rows<D>(s.vo.f, nt, 4 * ng, g.tid, G::NT);
            zero_rows<1>(s.b.f, nt, 4 * ng, g.tid, G::NT);
        }
        if ((sizeof(T) != 4) || (nt & 3)) __syncthreads();
        gram_phase<D>(s.k.f, s.q.f, gram, ng, g.tid, G::NT);
        __syncthreads();

        for (int gi = ng - 1; gi >= 0; gi--) {
            const int tb = 4 * gi;
            const int nv = min(4, nt - tb);            // valid steps in this group
            float* xu = xch + par * SM::kXg;           // [4][D]
            float* xbr = xu + 4 * D;                   // [4][D]
            float* xdb = xbr + 4 * D;                  // [4][8]
            par ^= 1;
            // ---------------- column role: one reduction round for the four steps
            {
                float a[4];
                f2 kk[KEEP ? 4 : 1][G::NP];
                if constexpr (KEEP) {
#pragma unroll
                    for (int j = 0; j < 4; j++) lds_slice<G::NR>(kk[j], s.k.f + (tb + j) * D + g.off);
                    f2 aa[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                    for (int i = 0; i < G::NP; i++) {
#pragma unroll
                        for (int j = 0; j < 4; j++) aa[j] = ffma2(Gc[i], kk[j][i], aa[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) a[j] = f2_hsum(aa[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        lds_slice<G::NR>(kk[0], s.k.f + (tb + j) * D + g.off);
                        a[j] = dot2_chain<G::NP>(Gc, kk[0]);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) a[j] = reduce_split<SPLIT>(a[j]);
                float gs[16];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 t4 = *reinterpret_cast<const float4*>(gram + gi * 16 + 4 * i);
                    gs[4 * i] = t4.x; gs[4 * i + 1] = t4.y; gs[4 * i + 2] = t4.z; gs[4 * i + 3] = t4.w;
                }
                const float4 b4 = *reinterpret_cast<const float4*>(s.b.f + tb);
                const float be[4] = {b4.x, b4.y, b4.z, b4.w};
                float gy[4], w[4], r[4], br[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    gy[j] = s.gy.f[(tb + j) * D + g.idx];
                    w[j] = s.v.f[(tb + j) * D + g.idx] - s.vo.f[(tb + j) * D + g.idx];
                }
#pragma unroll
                for (int j = 3; j >= 0; j--) {          // time reversed
                    float acc = fmaf(gy[j], gs[gram_kq(j, j)], a[j]);
#pragma unroll
                    for (int i = 3; i > j; i--) {
                        acc = fmaf(gy[i], gs[gram_kq(j, i)], acc);
                        acc = fmaf(-br[i], gs[gram_kk(j, i)], acc);
                    }
                    r[j] = acc;
                    br[j] = be[j] * acc;
                }
#pragma unroll
                for (int j = 3; j >= 0; j--) {
                    f2 qq[G::NP];
                    lds_slice<G::NR>(qq, s.q.f + (tb + j) * D + g.off);
                    axpy2<G::NP>(Gc, qq, gy[j]);
                    if constexpr (KEEP) {
                        axpy2<G::NP>(Gc, kk[j], -br[j]);
                    } else {
                        lds_slice<G::NR>(kk[0], s.k.f + (tb + j) * D + g.off);
                        axpy2<G::NP>(Gc, kk[0], -br[j]);
                    }
                }
                const float tot = warp_sum4_idx<SPLIT>(r[0] * w[0], r[1] * w[1], r[2] * w[2], r[3] * w[3], g.lane);
                if (g.s == 0) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        xu[j * D + g.idx] = be[j] * w[j];
                        xbr[j * D + g.idx] = br[j];
                        odv[(tb + j) * D + g.idx] = br[j];
                    }
                    const int lm = g.lane % G::MC;
                    if ((lm % HS) == 0 && lm / HS < 4) {
                        if (G::WPS == 1) odb[tb + lm / HS] = tot; else xdb[(lm / HS) * 8 + g.warp] = tot;
                    }
                }
            }
            cta_sync<G::WPS>();
            // ---------------- row role: per step, time reversed
            for (int j = nv - 1; j >= 0; j--) {
                const int t = tb + j;
                f2 gr[G::NP], ur[G::NP], brr[G::NP];
                lds_slice<G::NR>(gr, s.gy.f + t * D + g.off);
                lds_slice<G::NR>(ur, xu + j * D + g.off);
                lds_slice<G::NR>(brr, xbr + j * D + g.off);
                const float qe = s.q.f[t * D + g.idx], ke = s.k.f[t * D + g.idx];
                float dq = dot2<G::NP>(Sr, gr);
                axpy2<G::NP>(Gr, gr, qe);
                float dk = dot2<G::NP>(Gr, ur);
                axpy2<G::NP>(Sr, ur, -ke);
                dk -= dot2<G::NP>(Sr, brr);
                axpy2<G::NP>(Gr, brr, -ke);
                dq = reduce_split<SPLIT>(dq);
                dk = reduce_split<SPLIT>(dk);
                if (g.s == 0) {
                    odq[t * D + g.idx] = dq;
                    odk[t * D + g.idx] = dk;
                }
                if (G::WPS > 1 && g.tid == 0) {
                    float db = xdb[j * 8];
#pragma unroll
                    for (int w2 = 1; w2 < G::WPS; w2++) db += xdb[j * 8 + w2];
                    odb[t] = db;
                }
            }
        }
        __syncthreads();
        flush_rows<D, G::NT, T>(odq, p.gq, n, h, t0, nt, p.E, g.tid);
        flush_rows<D, G::NT, T>(odk, p.gk, n, h, t0, nt, p.E, g.tid);
        flush_rows<D, G::NT, T>(odv, p.gv, n, h, t0, nt, p.M, g.tid);
        flush_rows<1, G::NT, T>(odb, p.gb, n, h, t0, nt, 1, g.tid);
    }
    store_rows(g, Sr, W, p.wE, p.E, p.M);
}

}  // namespace fwp
