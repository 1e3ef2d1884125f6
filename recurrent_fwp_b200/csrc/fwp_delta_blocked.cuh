// Delta rule, four-step blocked and warp-specialised (sm_100a).
//
// Blocking.  The per-step kernels put one reduction round (dot, shuffle, scalar
// update) on the dependency chain of every time step.  Here four consecutive
// steps share one round: all matrix-vector products of a group are taken with the
// state at the *start* of the group and corrected with Gram scalars of the
// group's keys and queries, which do not depend on the state:
//
//   a_j = S^T k_j,  b_j = S^T q_j                      (S = state before the group)
//   v_old_j = a_j + sum_{i<j}  u_i (k_i . k_j) ;  u_j = beta_j (v_j - v_old_j)
//   y_j     = b_j + sum_{i<=j} u_i (k_i . q_j) ;  S += sum_j k_j (x) u_j
//
// Backward (time reversed inside a group), with G = dL/dS before the group:
//   a_j = G^T k_j
//   r_j = a_j + gy_j (q_j . k_j) + sum_{i later than j} ( gy_i (q_i . k_j) - beta_i r_i (k_i . k_j) )
//   G  += sum_j ( q_j (x) gy_j - k_j (x) beta_j r_j )
// The algebra is exact; only the fp32 summation order differs from the per-step form.
//
// Warp specialisation.  With a few hundred sequences there is about one warp per
// SM sub-partition, so anything a warp does besides the dependency chain is
// exposed latency.  Each sequence is therefore served by separate warps that meet
// at a named barrier of their own once per chunk (several sequences share a CTA
// without waiting for each other):
//   * a producer warp: staging two chunks ahead (forward: cp.async; backward: one
//     1-D bulk copy per tensor and chunk completing on an mbarrier whose wait is
//     bounded, cp.async for rows that are strided or unaligned), Gram scalars one
//     chunk ahead, and the 16-byte flush of the previous chunk's outputs;
//   * forward: the consumer warps own the state columns and only run the group loop;
//   * backward: "column" warps run the blocked chain on G and publish u_t, beta_t r_t
//     for a whole chunk; "row" warps follow one chunk behind with the per-step part
//     (dq, dk, in-place rewind of S).
#pragma once
#include "fwp_core.cuh"

namespace fwp {

// raised (and left raised) when a bounded wait on a bulk copy ran out; read by fwp_delta_device_fault()
static __device__ int g_delta_fault;

template <int RL>
__device__ __forceinline__ void zero_rows(float* tile, int r0, int r1, int tid, int nthreads) {
    for (int i = r0 * RL + tid; i < r1 * RL; i += nthreads) tile[i] = 0.f;
}

__device__ __forceinline__ void load16(float (&gs)[16], const float* p) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 t4 = *reinterpret_cast<const float4*>(p + 4 * i);
        gs[4 * i] = t4.x; gs[4 * i + 1] = t4.y; gs[4 * i + 2] = t4.z; gs[4 * i + 3] = t4.w;
    }
}

// ------------------------------------------------------------------ forward
template <int D, int TC, typename T>
struct WsFwdStage {
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
struct WsFwdSmem {
    static constexpr int NS = 3;                       // stages: in flight, prepared, consumed
    static constexpr int kStage = WsFwdStage<D, TC, T>::kFloats;
    static constexpr int kGram = (TC / 4) * 16;
    static constexpr int kOut = 3 * TC * D;            // y, v_old, u
    static constexpr int kFloats = NS * kStage + 2 * kGram + 2 * kOut;
};

template <int D, int SPLIT, int TC, typename T, bool SUM>
__global__ void __launch_bounds__(slots_for(D * SPLIT) * (D * SPLIT + 32)) delta_fwd_kernel(const DeltaFwdParams p) {
    using G = Geo<D, SPLIT>;
    using SM = WsFwdSmem<D, TC, T>;
    using Stage = WsFwdStage<D, TC, T>;
    static_assert(TC % 4 == 0, "chunk must hold whole groups");
    constexpr bool KEEP = G::NR <= 16;
    constexpr int NSL = slots_for(G::NT);          // sequences per CTA
    constexpr int NCONS = NSL * G::NT;             // consumer threads come first, then one producer warp per slot
    const int tid = threadIdx.x;
    const bool producer = tid >= NCONS;
    const int slot = producer ? (tid - NCONS) >> 5 : tid / G::NT;
    const int ptid = (tid - NCONS) & 31;
    const int seq = blockIdx.x * NSL + slot;
    const int n = seq / p.H, h = seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    static_assert(SM::kFloats % 4 == 0, "the zero fill goes by 16-byte stores");
    for (int i = tid; i < NSL * SM::kFloats / 4; i += NSL * (G::NT + 32))
        reinterpret_cast<float4*>(smem_all)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    float* smem = smem_all + slot * SM::kFloats;
    float* gram0 = smem + SM::NS * SM::kStage;
    float* out0 = gram0 + 2 * SM::kGram;
    const int nchunks = (p.L + TC - 1) / TC;
    __syncthreads();
    griddep_wait();               // global memory is touched from here on
    griddep_launch_dependents();
    if (seq >= p.NH) return;      // an empty slot of the last CTA: nobody waits on its barrier

    if (producer) {
        // ===================================================== producer warp
        Src<T> sq, sk, sv, sb;
        sq.init(p.q, n, h, p.E);
        sk.init(p.k, n, h, p.E);
        sv.init(p.v, n, h, p.M);
        if (!SUM) sb.init(p.beta, n, h, 1);
        auto issue = [&](int c) {
            Stage s; s.bind(smem + (c % SM::NS) * SM::kStage);
            const int t0 = c * TC, nt = min(TC, p.L - t0);
            s.q.template load<32>(sq, t0, nt, ptid);
            s.k.template load<32>(sk, t0, nt, ptid);
            s.v.template load<32>(sv, t0, nt, ptid);
            if (!SUM) s.b.template load<32>(sb, t0, nt, ptid);
            cp_async_commit();
        };
        auto prepare = [&](int c) {     // chunk c has landed: widen, pad, Gram scalars
            Stage s; s.bind(smem + (c % SM::NS) * SM::kStage);
            const int nt = min(TC, p.L - c * TC), ng = (nt + 3) >> 2;
            __syncwarp();
            if constexpr (sizeof(T) != 4) {
                s.q.widen(nt, p.E, ptid, 32);
                s.k.widen(nt, p.E, ptid, 32);
                s.v.widen(nt, p.M, ptid, 32);
                if (!SUM) s.b.widen(nt, 1, ptid, 32);
            }
            if (nt & 3) {   // pad the last group with inert steps (k = q = v = beta = 0)
                zero_rows<D>(s.q.f, nt, 4 * ng, ptid, 32);
                zero_rows<D>(s.k.f, nt, 4 * ng, ptid, 32);
                zero_rows<D>(s.v.f, nt, 4 * ng, ptid, 32);
                if (!SUM) zero_rows<1>(s.b.f, nt, 4 * ng, ptid, 32);
            }
            if ((sizeof(T) != 4) || (nt & 3)) __syncwarp();
            gram_phase<D, 32, TC>(s.k.f, s.q.f, gram0 + (c & 1) * SM::kGram, ng, ptid);
        };
        auto flush = [&](int c) {
            const float* o = out0 + (c & 1) * SM::kOut;
            const int t0 = c * TC, nt = min(TC, p.L - t0);
            flush_rows<D, 32, T, TC>(o, p.out, n, h, t0, nt, p.M, ptid);
            if constexpr (!SUM) {
                flush_rows<D, 32, float, TC>(o + TC * D, p.v_old, n, h, t0, nt, p.M, ptid);
                if (p.v_ins.p) flush_rows<D, 32, float, TC>(o + 2 * TC * D, p.v_ins, n, h, t0, nt, p.M, ptid);
            }
        };
        issue(0);
        if (nchunks > 1) { issue(1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        prepare(0);
        slot_barrier(slot, G::NT + 32);
        for (int c = 0; c <= nchunks; c++) {
            if (c + 2 < nchunks) issue(c + 2);      // lands while this iteration's other work runs
            if (c >= 1) flush(c - 1);
            if (c + 1 < nchunks) {
                if (c + 2 < nchunks) cp_async_wait<1>(); else cp_async_wait<0>();
                prepare(c + 1);
            }
            slot_barrier(slot, G::NT + 32);
        }
    } else {
        // ===================================================== consumer warps: the group loop
        const G g(tid);
        float* W = p.W + n * p.wN + h * p.wH;
        f2 S[G::NP];
        load_cols(g, S, W, p.wE, p.E, p.M);
        slot_barrier(slot, G::NT + 32);
        for (int c = 0; c <= nchunks; c++) {
            if (c < nchunks) {
                Stage s; s.bind(smem + (c % SM::NS) * SM::kStage);
                const float* gram = gram0 + (c & 1) * SM::kGram;
                float* oy = out0 + (c & 1) * SM::kOut;
                float* ovo = oy + TC * D;
                float* ou = ovo + TC * D;
                const int nt = min(TC, p.L - c * TC), ng = (nt + 3) >> 2;
                // One group: dots with the pre-group state, scalar recurrences, rank-4 update, staged outputs.
                // `cur` holds this group's operand slices (already in registers); `nxt` receives the next
                // group's slices, whose loads are issued before this group's arithmetic.
                auto tail = [&](int tb, float (&a)[4], float (&b)[4], auto&& update) {
                    float gs[16], vv[4];
                    load16(gs, gram + (tb >> 2) * 16);
                    float be[4] = {1.f, 1.f, 1.f, 1.f};
                    if constexpr (!SUM) {
                        const float4 b4 = *reinterpret_cast<const float4*>(s.b.f + tb);
                        be[0] = b4.x; be[1] = b4.y; be[2] = b4.z; be[3] = b4.w;
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) vv[j] = s.v.f[(tb + j) * D + g.idx];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if constexpr (!SUM) a[j] = reduce_split<SPLIT>(a[j]);
                        b[j] = reduce_split<SPLIT>(b[j]);
                    }
                    float u[4], vo[4], y[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if constexpr (SUM) {
                            vo[j] = 0.f;
                            u[j] = vv[j];
                        } else {
                            float acc = a[j];
#pragma unroll
                            for (int i = 0; i < j; i++) acc = fmaf(u[i], gs[gram_kk(i, j)], acc);
                            vo[j] = acc;
                            u[j] = be[j] * (vv[j] - acc);
                        }
                        float yy = b[j];
#pragma unroll
                        for (int i = 0; i <= j; i++) yy = fmaf(u[i], gs[gram_kq(i, j)], yy);
                        y[j] = yy;
                    }
                    update(u);
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
                };
                if constexpr (G::NR <= 8) {
                    // small slices: fetch all eight operand slices first, then run the eight dot-product
                    // chains interleaved so that no FMA waits on its predecessor
#pragma unroll 1
                    for (int gi = 0; gi < ng; gi++) {
                        const int tb = 4 * gi;
                        f2 kk[4][G::NP], qq[4][G::NP];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            lds_slice<G::NR>(kk[j], s.k.f + (tb + j) * D + g.off);
                            lds_slice<G::NR>(qq[j], s.q.f + (tb + j) * D + g.off);
                        }
                        f2 aa[4] = {0ull, 0ull, 0ull, 0ull}, bb[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                        for (int i = 0; i < G::NP; i++) {
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                if constexpr (!SUM) aa[j] = ffma2(S[i], kk[j][i], aa[j]);
                                bb[j] = ffma2(S[i], qq[j][i], bb[j]);
                            }
                        }
                        float a[4], b[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) { a[j] = SUM ? 0.f : f2_hsum(aa[j]); b[j] = f2_hsum(bb[j]); }
                        tail(tb, a, b, [&](const float (&u)[4]) {
#pragma unroll
                            for (int j = 0; j < 4; j++) axpy2<G::NP>(S, kk[j], u[j]);
                        });
                    }
                } else {
                    for (int gi = 0; gi < ng; gi++) {
                        const int tb = 4 * gi;
                        float a[4], b[4];
                        f2 kk[KEEP ? 4 : 1][G::NP];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            f2 (&kj)[G::NP] = kk[KEEP ? j : 0];
                            lds_slice<G::NR>(kj, s.k.f + (tb + j) * D + g.off);
                            if constexpr (!SUM) a[j] = dot2_chain<G::NP>(S, kj); else a[j] = 0.f;
                            f2 qq[G::NP];
                            lds_slice<G::NR>(qq, s.q.f + (tb + j) * D + g.off);
                            b[j] = dot2_chain<G::NP>(S, qq);
                        }
                        tail(tb, a, b, [&](const float (&u)[4]) {
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                if constexpr (KEEP) {
                                    axpy2<G::NP>(S, kk[j], u[j]);
                                } else {
                                    lds_slice<G::NR>(kk[0], s.k.f + (tb + j) * D + g.off);
                                    axpy2<G::NP>(S, kk[0], u[j]);
                                }
                            }
                        });
                    }
                }
            }
            slot_barrier(slot, G::NT + 32);
        }
        store_cols(g, S, W, p.wE, p.E, p.M);
    }
}

// ------------------------------------------------------------------ backward
template <int D, int TC, typename T>
struct WsBwdStage {
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

template <int D, int TC, typename T, int PF = 2>
struct WsBwdSmem {
    static constexpr int NS = PF + 2;                  // PF chunks ahead (in flight / prepared), column role, row role
    static constexpr int kStage = WsBwdStage<D, TC, T>::kFloats;
    static constexpr int kGram = (TC / 4) * 16;
    static constexpr int kX = 2 * TC * D + TC * 8;     // u[TC][D], beta*r[TC][D] (= dv), dbeta partials[TC][8]
    static constexpr int kO = 2 * TC * D;              // dq[TC][D], dk[TC][D]
    static constexpr int kBars = r4(2 * NS);           // one 8-byte mbarrier per stage
    static constexpr int kFloats = NS * kStage + 2 * kGram + 2 * kX + 2 * kO + r4(TC) + kBars;
};

// PF = how many chunks ahead the producer stages: 2 hides the memory latency behind a whole iteration; 1 needs one
// stage less, which is what lets a chunk of 32 steps fit four sequences into the shared memory of an SM.
template <int D, int SPLIT, int TC, typename T, int PF = 2>
__global__ void __launch_bounds__(slots_for(D * SPLIT) * (2 * D * SPLIT + 32)) delta_bwd_kernel(const DeltaBwdParams p) {
    using G = Geo<D, SPLIT>;
    using SM = WsBwdSmem<D, TC, T, PF>;
    static_assert(PF == 1 || PF == 2, "prefetch distance");
    using Stage = WsBwdStage<D, TC, T>;
    static_assert(TC % 4 == 0, "chunk must hold whole groups");
    constexpr bool KEEP = G::NR <= 8;
    constexpr int HS = sum4_stride<SPLIT>();
    constexpr int NSL = slots_for(G::NT);          // sequences per CTA
    constexpr int NCONS = NSL * G::NT;             // column-role threads, then row-role threads, then producers
    // Gradients leave by 16-byte stores of the producer warp.  Bulk stores from shared memory are implemented
    // (set to true) but need a generic-to-async proxy fence in the compute roles before every chunk's barrier,
    // which measured about 1900 cycles per chunk on the column role's critical path.
    constexpr bool kBulkStores = false;
    const int tid = threadIdx.x;
    const int role = tid < NCONS ? 0 : (tid < 2 * NCONS ? 1 : 2);     // 0 column, 1 row, 2 producer
    const int rtid = tid - role * NCONS;                               // index within the role
    const int slot = role == 2 ? rtid >> 5 : rtid / G::NT;
    const int seq = blockIdx.x * NSL + slot;
    const int n = seq / p.H, h = seq - n * p.H;
    extern __shared__ __align__(16) float smem_all[];
    static_assert(SM::kFloats % 4 == 0, "the zero fill goes by 16-byte stores");
    for (int i = tid; i < NSL * SM::kFloats / 4; i += NSL * (2 * G::NT + 32))
        reinterpret_cast<float4*>(smem_all)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    fence_async_smem();     // the zero fill is ordered before any bulk copy into the same tiles
    float* smem = smem_all + slot * SM::kFloats;
    float* gram0 = smem + SM::NS * SM::kStage;
    float* x0 = gram0 + 2 * SM::kGram;
    float* o0 = x0 + 2 * SM::kX;
    float* dbt = o0 + 2 * SM::kO;       // dbeta of one chunk, assembled by the producer before its flush
    const int nchunks = (p.L + TC - 1) / TC;
    __syncthreads();
    griddep_wait();               // global memory is touched from here on
    griddep_launch_dependents();
    if (seq >= p.NH) return;      // an empty slot of the last CTA: nobody waits on its barrier
    // chunk index jc counts from the end of the sequence; nchunks-1-jc is the time-order chunk
    if (role == 2) {
        // ===================================================== producer warp
        const int ptid = rtid & 31;
        Src<T> sq, sk, sv, sg, sb;
        Src<float> so;
        sq.init(p.q, n, h, p.E);
        sk.init(p.k, n, h, p.E);
        sv.init(p.v, n, h, p.M);
        sg.init(p.gy, n, h, p.M);
        so.init(p.v_old, n, h, p.M);
        sb.init(p.beta, n, h, 1);
        unsigned long long* bars = reinterpret_cast<unsigned long long*>(dbt + r4(TC));
        if (ptid == 0) {
            for (int i = 0; i < SM::NS; i++) mbar_init(&bars[i], 1);
            mbar_fence_init();
        }
        __syncwarp();
        // One bulk copy per tensor and chunk pays off only when a chunk is long: at d = 32 / 64 a chunk is 8 / 4
        // steps, six copies per chunk cost more to issue than the cp.async pieces they replace (measured 159 vs
        // 138 us at d = 32 and 588 vs 479 us at d = 64 for 512 sequences of 256 steps), so those sizes keep cp.async.
        // Issuing the six copies from six lanes of one instruction instead of one lane in turn was slower (50 us).
        const bool kBulkLoads = D <= 16 && p.bulk;      // "delta_bwd.bulk" = 0 keeps cp.async (48.4 vs 46.3 us at d = 16)
        const bool eq = kBulkLoads && bulk_rows_ok<D, T>(sq.base, sq.sL, sq.width), ek = kBulkLoads && bulk_rows_ok<D, T>(sk.base, sk.sL, sk.width),
                   ev = kBulkLoads && bulk_rows_ok<D, T>(sv.base, sv.sL, sv.width), eg = kBulkLoads && bulk_rows_ok<D, T>(sg.base, sg.sL, sg.width),
                   eo = kBulkLoads && bulk_rows_ok<D, float>(so.base, so.sL, so.width);
        unsigned phase = 0;
        bool failed = false;
        auto issue = [&](int jc) {
            Stage s; s.bind(smem + (jc % SM::NS) * SM::kStage);
            const int t0 = (nchunks - 1 - jc) * TC, nt = min(TC, p.L - t0);
            const bool eb = kBulkLoads && bulk_col_ok<T>(sb.base, sb.sL, t0, nt);
            if (ptid == 0 && (eq || ek || ev || eg || eo || eb)) {
                unsigned long long* bar = &bars[jc % SM::NS];
                const unsigned rows = nt * D * sizeof(T), rowsf = nt * D * sizeof(float), col = nt * sizeof(T);
                mbar_arrive_expect_tx(bar, (eq ? rows : 0) + (ek ? rows : 0) + (ev ? rows : 0) + (eg ? rows : 0) +
                                               (eo ? rowsf : 0) + (eb ? col : 0));
                if (eq) bulk_g2s(s.q.raw, sq.base + (long long)t0 * D, rows, bar);
                if (ek) bulk_g2s(s.k.raw, sk.base + (long long)t0 * D, rows, bar);
                if (ev) bulk_g2s(s.v.raw, sv.base + (long long)t0 * D, rows, bar);
                if (eg) bulk_g2s(s.gy.raw, sg.base + (long long)t0 * D, rows, bar);
                if (eo) bulk_g2s(s.vo.raw, so.base + (long long)t0 * D, rowsf, bar);
                if (eb) bulk_g2s(s.b.raw, sb.base + t0, col, bar);
            }
            if (!eq) s.q.template load<32>(sq, t0, nt, ptid);
            if (!ek) s.k.template load<32>(sk, t0, nt, ptid);
            if (!ev) s.v.template load<32>(sv, t0, nt, ptid);
            if (!eg) s.gy.template load<32>(sg, t0, nt, ptid);
            if (!eo) s.vo.template load<32>(so, t0, nt, ptid);
            if (!eb) s.b.template load<32>(sb, t0, nt, ptid);
            cp_async_commit();
        };
        auto landed = [&](int jc) {
            const int t0 = (nchunks - 1 - jc) * TC, nt = min(TC, p.L - t0);
            if (eq || ek || ev || eg || eo || (kBulkLoads && bulk_col_ok<T>(sb.base, sb.sL, t0, nt))) {
                const int st = jc % SM::NS;
                if (!failed && !mbar_wait_bounded(&bars[st], (phase >> st) & 1)) {
                    failed = true;
                    atomicExch(&g_delta_fault, 1);
                }
                phase ^= 1u << st;
            }
        };
        auto prepare = [&](int jc) {
            Stage s; s.bind(smem + (jc % SM::NS) * SM::kStage);
            const int nt = min(TC, p.L - (nchunks - 1 - jc) * TC), ng = (nt + 3) >> 2;
            __syncwarp();
            if constexpr (sizeof(T) != 4) {
                s.q.widen(nt, p.E, ptid, 32);
                s.k.widen(nt, p.E, ptid, 32);
                s.v.widen(nt, p.M, ptid, 32);
                s.gy.widen(nt, p.M, ptid, 32);
                s.b.widen(nt, 1, ptid, 32);
            }
            if (nt & 3) {
                zero_rows<D>(s.q.f, nt, 4 * ng, ptid, 32);
                zero_rows<D>(s.k.f, nt, 4 * ng, ptid, 32);
                zero_rows<D>(s.v.f, nt, 4 * ng, ptid, 32);
                zero_rows<D>(s.gy.f, nt, 4 * ng, ptid, 32);
                zero_rows<D>(s.vo.f, nt, 4 * ng, ptid, 32);
                zero_rows<1>(s.b.f, nt, 4 * ng, ptid, 32);
            }
            if ((sizeof(T) != 4) || (nt & 3)) __syncwarp();
            gram_phase<D, 32, TC>(s.k.f, s.q.f, gram0 + (jc & 1) * SM::kGram, ng, ptid);
        };
        // gradients: fp32 tiles whose destination rows are contiguous leave by one bulk store each
        const Row4 rg[3] = {p.gv, p.gq, p.gk};
        bool es[3];
        float* gbase[3];
#pragma unroll
        for (int i = 0; i < 3; i++) {
            gbase[i] = reinterpret_cast<float*>(rg[i].p) + n * rg[i].sN + h * rg[i].sH;
            es[i] = kBulkStores && sizeof(T) == 4 && bulk_rows_ok<D, float>(gbase[i], rg[i].sL, i == 0 ? p.M : p.E);
        }
        auto flush_col = [&](int jc) {      // dv = beta*r and dbeta of the chunk the column role just finished
            const float* x = x0 + (jc & 1) * SM::kX;
            const int t0 = (nchunks - 1 - jc) * TC, nt = min(TC, p.L - t0);
            if (es[0]) {
                if (ptid == 0) { bulk_s2g(gbase[0] + (long long)t0 * D, x + TC * D, nt * D * sizeof(float)); bulk_commit(); }
            } else {
                flush_rows<D, 32, T, TC>(x + TC * D, p.gv, n, h, t0, nt, p.M, ptid);
            }
            const float* part = x + 2 * TC * D;
            for (int t = ptid; t < nt; t += 32) {
                float db = part[t * 8];
#pragma unroll
                for (int w = 1; w < G::WPS; w++) db += part[t * 8 + w];
                dbt[t] = db;
            }
            __syncwarp();
            flush_rows<1, 32, T, 0>(dbt, p.gb, n, h, t0, nt, 1, ptid);
            __syncwarp();
        };
        auto flush_row = [&](int jc) {
            const float* o = o0 + (jc & 1) * SM::kO;
            const int t0 = (nchunks - 1 - jc) * TC, nt = min(TC, p.L - t0);
            if (ptid == 0 && (es[1] || es[2])) {
                if (es[1]) bulk_s2g(gbase[1] + (long long)t0 * D, o, nt * D * sizeof(float));
                if (es[2]) bulk_s2g(gbase[2] + (long long)t0 * D, o + TC * D, nt * D * sizeof(float));
                bulk_commit();
            }
            if (!es[1]) flush_rows<D, 32, T, TC>(o, p.gq, n, h, t0, nt, p.E, ptid);
            if (!es[2]) flush_rows<D, 32, T, TC>(o + TC * D, p.gk, n, h, t0, nt, p.E, ptid);
        };
        issue(0);
        if (PF == 2 && nchunks > 1) { issue(1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        landed(0);
        prepare(0);
        slot_barrier(slot, 2 * G::NT + 32);
        for (int i = 0; i <= nchunks + 1; i++) {
            if (i + PF < nchunks) issue(i + PF);    // lands while this iteration's other work runs
            if (i >= 1 && i - 1 < nchunks) flush_col(i - 1);
            if (i >= 2) flush_row(i - 2);
            if (i + 1 < nchunks) {
                if (PF == 2 && i + 2 < nchunks) cp_async_wait<1>(); else cp_async_wait<0>();
                landed(i + 1);
                prepare(i + 1);
            }
            if (ptid == 0) bulk_wait_read_all();     // the flushed tiles may be rewritten after the barrier
            slot_barrier(slot, 2 * G::NT + 32);
        }
        if (ptid == 0) bulk_wait_all();
    } else if (role == 0) {
        // ===================================================== column role: blocked chain on G
        const G g(rtid);
        f2 Gc[G::NP];
#pragma unroll
        for (int i = 0; i < G::NP; i++) Gc[i] = 0ull;
        slot_barrier(slot, 2 * G::NT + 32);
        for (int i = 0; i <= nchunks + 1; i++) {
            if (i < nchunks) {
                const int jc = i;
                Stage s; s.bind(smem + (jc % SM::NS) * SM::kStage);
                const float* gram = gram0 + (jc & 1) * SM::kGram;
                float* xu = x0 + (jc & 1) * SM::kX;
                float* xbr = xu + TC * D;
                float* xdb = xbr + TC * D;
                const int nt = min(TC, p.L - (nchunks - 1 - jc) * TC), ng = (nt + 3) >> 2;
                for (int gi = ng - 1; gi >= 0; gi--) {
                    const int tb = 4 * gi;
                    float a[4];
                    f2 kk[KEEP ? 4 : 1][G::NP];
                    f2 qk[KEEP ? 4 : 1][G::NP];     // query slices, fetched with the keys so their latency overlaps the chain
                    if constexpr (KEEP) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            lds_slice<G::NR>(kk[j], s.k.f + (tb + j) * D + g.off);
                            lds_slice<G::NR>(qk[j], s.q.f + (tb + j) * D + g.off);
                        }
                        f2 aa[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                        for (int q = 0; q < G::NP; q++) {
#pragma unroll
                            for (int j = 0; j < 4; j++) aa[j] = ffma2(Gc[q], kk[j][q], aa[j]);
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
                    float gs[16];
                    load16(gs, gram + gi * 16);
                    const float4 b4 = *reinterpret_cast<const float4*>(s.b.f + tb);
                    const float be[4] = {b4.x, b4.y, b4.z, b4.w};
                    float gy[4], w[4], r[4], br[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        gy[j] = s.gy.f[(tb + j) * D + g.idx];
                        w[j] = s.v.f[(tb + j) * D + g.idx] - s.vo.f[(tb + j) * D + g.idx];
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) a[j] = reduce_split<SPLIT>(a[j]);
#pragma unroll
                    for (int j = 3; j >= 0; j--) {          // time reversed
                        float acc = fmaf(gy[j], gs[gram_kq(j, j)], a[j]);
#pragma unroll
                        for (int q = 3; q > j; q--) {
                            acc = fmaf(gy[q], gs[gram_kq(j, q)], acc);
                            acc = fmaf(-br[q], gs[gram_kk(j, q)], acc);
                        }
                        r[j] = acc;
                        br[j] = be[j] * acc;
                    }
#pragma unroll
                    for (int j = 3; j >= 0; j--) {
                        if constexpr (KEEP) {
                            axpy2<G::NP>(Gc, qk[j], gy[j]);
                            axpy2<G::NP>(Gc, kk[j], -br[j]);
                        } else {
                            lds_slice<G::NR>(qk[0], s.q.f + (tb + j) * D + g.off);
                            axpy2<G::NP>(Gc, qk[0], gy[j]);
                            lds_slice<G::NR>(kk[0], s.k.f + (tb + j) * D + g.off);
                            axpy2<G::NP>(Gc, kk[0], -br[j]);
                        }
                    }
                    const float tot = warp_sum4_idx<SPLIT>(r[0] * w[0], r[1] * w[1], r[2] * w[2], r[3] * w[3], g.lane);
                    if (g.s == 0) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            xu[(tb + j) * D + g.idx] = be[j] * w[j];
                            xbr[(tb + j) * D + g.idx] = br[j];
                        }
                        const int lm = g.lane % G::MC;
                        if ((lm % HS) == 0 && lm / HS < 4) xdb[(tb + lm / HS) * 8 + g.warp] = tot;
                    }
                }
                if (kBulkStores) fence_async_smem();      // beta*r (= dv) is read by a bulk store
            }
            slot_barrier(slot, 2 * G::NT + 32);
        }
    } else {
        // ===================================================== row role: per step, one chunk behind
        const G g(rtid);
        float* W = p.W + n * p.wN + h * p.wH;
        f2 Sr[G::NP], Gr[G::NP];
        load_rows(g, Sr, W, p.wE, p.E, p.M);
#pragma unroll
        for (int i = 0; i < G::NP; i++) Gr[i] = 0ull;
        slot_barrier(slot, 2 * G::NT + 32);
        for (int i = 0; i <= nchunks + 1; i++) {
            if (i >= 1 && i - 1 < nchunks) {
                const int jc = i - 1;
                Stage s; s.bind(smem + (jc % SM::NS) * SM::kStage);
                const float* xu = x0 + (jc & 1) * SM::kX;
                const float* xbr = xu + TC * D;
                float* odq = o0 + (jc & 1) * SM::kO;
                float* odk = odq + TC * D;
                const int nt = min(TC, p.L - (nchunks - 1 - jc) * TC);
#pragma unroll 2
                for (int t = nt - 1; t >= 0; t--) {
                    f2 gr[G::NP], ur[G::NP], brr[G::NP];
                    lds_slice<G::NR>(gr, s.gy.f + t * D + g.off);
                    lds_slice<G::NR>(ur, xu + t * D + g.off);
                    lds_slice<G::NR>(brr, xbr + t * D + g.off);
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
                }
                if (kBulkStores) fence_async_smem();
            }
            slot_barrier(slot, 2 * G::NT + 32);
        }
        store_rows(g, Sr, W, p.wE, p.E, p.M);
    }
}

}  // namespace fwp
