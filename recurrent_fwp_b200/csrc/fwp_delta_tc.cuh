// Delta rule, chunkwise (WY / UT transform) forward on the fifth-generation tensor cores (sm_100a):
// bf16 streams, E = M = 64, 64 steps per chunk, fp32 state.
//
// With S0 the state before a chunk, K, Q, V its rows (64 x 64 each), b = beta:
//   Akk = K K^T, Aqk = lower(Q K^T)                    N = strict_lower(Akk) diag(b),  T = (I + N)^-1
//   Ck = T K,  Cv = T V                                 (the unit triangular solve as an explicit inverse)
//   w = Cv - Ck S0 (= v - v_old),  u = b w,  v_old = V - w
//   y = Q S0 + Aqk u,   S1 = S0 + K^T u
// (the recurrence of algorithmic/fast_weight/fast_weight_cuda.cu:101-169, regrouped over 64 steps).
//
// Every 64-deep contraction is a tcgen05.mma (M = N = 64, K = 16, four instructions per product), operands in
// 128-byte-swizzled shared-memory tiles, fp32 accumulators in tensor memory:
//   S (the fp32 master copy of the state, updated in place by S += K^T u), w (Cv, then Cv - Ck S0 accumulated into
//   it with the negated-A form), y, Akk, Aqk, Ck.
// K, Q, V tiles arrive by TMA tile loads (three stages, one mbarrier each).  The tiles the kernel produces itself
// (Aqk, T, Ck, u, the bf16 copy of S) are written from registers in the same swizzled layout (stmatrix); T and u
// are kept as two bf16 parts (hi + lo) so that the products they enter carry 16 mantissa bits.
// The inverse is blocked 16 x 16: warp w of the preparing group owns rows 16w..16w+15 of the chunk (the quarter of
// the tensor-memory lanes it can read), inverts its diagonal block in registers by the nilpotent product
// (I - D)(I + D^2)(I + D^4)(I + D^8) and obtains the blocks left of it by block forward substitution,
//   T[w][c] = -(I + Y_ww) (N[w][c] + sum_{c <= l < w} N[w][l] X[l][c]),   X = T - I,
// with the blocks of the warps above exchanged through shared memory (three rounds); these 16-wide products run on
// warp-level mma, everything 64 wide on tcgen05.
//
// One CTA per sequence, three roles that meet only at mbarriers:
//   * chain warps 0-3   per chunk c: w(c) -> u (two parts) and v_old;  S(c+1) -> bf16 copy;  y(c) -> global
//   * preparing warps 4-7, one chunk ahead: Gram tiles -> masked Aqk and T;  Ck -> bf16
//   * warp 8, one thread: every TMA load and every tcgen05.mma, in the order
//       Gram(c+1) | S += K^T u(c), y(c) | Ck, Cv(c+1) | w(c+1) = Cv - Ck S(c+1) | refill of the stage chunk c used
//     each product waiting for the mbarrier on which the producers of its operands (128 threads) arrive after
//     their proxy fence, each batch followed by a tcgen05.commit onto the mbarrier its consumers wait for.
// The state-dependent chain per chunk is: w product -> u -> state product -> bf16 copy; everything else runs beside it.
// Every mbarrier wait is bounded; a wait that runs out marks the CTA as failed, after which nobody waits any more,
// all roles finish their (fixed-length) loops, the CTA frees its tensor memory and raises the device flag that
// fwp_delta_device_fault() reads.
#pragma once
#include <cuda.h>
#include "fwp_delta_params.cuh"
#include "fwp_tc.cuh"

namespace fwp {

static __device__ int g_tc_fault;
#ifdef FWP_TC_PROF
static __device__ long long g_tc_prof[48];
#define TCP(i) { const long long _n = clock64(); _pt[i] += _n - _pc; _pc = _n; }
#define TCP_BEGIN long long _pt[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}, _pc = clock64();
#define TCP_END(base) if (blockIdx.x == 0 && lane == 0 && gw == 0) { for (int _i = 0; _i < 16; _i++) g_tc_prof[(base) + _i] = _pt[_i]; }
#else
#define TCP(i)
#define TCP_BEGIN
#define TCP_END(base)
#endif

namespace tcd {

using namespace cb;     // warp-level mma helpers of the 16-step kernels (pack_bf16, split_bf16, a_of, b_of, mm, ldb_kn)

constexpr int CH = 64;                  // steps per chunk
constexpr int NTH = 288;                // chain warps 0-3, preparing warps 4-7, issuing warp 8
constexpr int NG = 128;                 // threads per compute group
constexpr int NSTAGE = 3;
constexpr int LDX = 72;                 // row stride (bf16) of the row-major exchange and output tiles: 144 B, 16-byte aligned
constexpr uint32_t COL_S = 0, COL_W = 64, COL_Y = 128, COL_AKK = 192, COL_AQK = 256, COL_CK = 320, TMEM_COLS = 512;

struct Smem {
    alignas(1024) unsigned char k[NSTAGE][tc::kTileBytes];
    unsigned char q[NSTAGE][tc::kTileBytes];
    unsigned char v[NSTAGE][tc::kTileBytes];
    unsigned char aq[2][tc::kTileBytes];        // Aqk, [t][i], zero above the diagonal (K-major left operand)
    unsigned char th[tc::kTileBytes];           // T hi, [t][i] (K-major left operand)
    unsigned char tl[tc::kTileBytes];           // T lo
    unsigned char ck[tc::kTileBytes];           // Ck, [t][e] (K-major left operand)
    unsigned char uh[tc::kTileBytes];           // u hi, [i][m] (MN-major right operand)
    unsigned char ul[tc::kTileBytes];           // u lo
    unsigned char sb[tc::kTileBytes];           // bf16 copy of the state, [e][m] (MN-major right operand)
    __nv_bfloat16 x[CH * LDX];                  // X = T - I, lower blocks, row-major (exchange between preparing warps)
    __nv_bfloat16 ys[CH * LDX];                 // y, [t][m] row-major (staging for 16-byte stores)
    float b[2][CH];
    // completion of asynchronous work (one arrival each): TMA stages, tcgen05.commit of the five product batches
    uint64_t bar_full[NSTAGE], bar_gram, bar_ckcv, bar_p, bar_s, bar_y;
    // operands written / accumulators read by a compute group (128 arrivals each)
    uint64_t bar_t_ready, bar_ck_ready, bar_u_ready, bar_s_ready, bar_y_read;
    uint32_t tmem_base;
    int failed;
};
// Tensor memory is taken whole (512 columns); that is only safe while a second CTA cannot become resident on the
// SM and wait for columns forever, which the shared-memory footprint guarantees.
static_assert(sizeof(Smem) > 116 * 1024, "two CTAs per SM would deadlock on the tensor-memory allocation");
static_assert(sizeof(Smem) + 1024 <= 227 * 1024, "shared memory budget");

// the four tcgen05.mma of one 64 x 64 x 64 product, from prebuilt descriptors
template <bool A_MN, bool B_MN, bool NEG_A>
__device__ __forceinline__ void product(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, bool accumulate) {
    constexpr uint32_t id = tc::idesc(A_MN, B_MN, NEG_A);
#pragma unroll
    for (int k = 0; k < 4; k++)
        tc::mma_issue(d_tmem, a_desc + (uint64_t)(k * (A_MN ? 128 : 2)), b_desc + (uint64_t)(k * (B_MN ? 128 : 2)), id,
                      (accumulate || k > 0) ? 1u : 0u);
}

}  // namespace tcd

__global__ void __launch_bounds__(tcd::NTH, 1)
delta_fwd_tc_kernel(const DeltaFwdParams p, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    using namespace tcd;
    using bf16 = __nv_bfloat16;
    extern __shared__ unsigned char tc_smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int role = warp >> 2;                         // 0 chain, 1 preparing, 2 issuing
    const int gw = warp & 3, gtid = tid & (NG - 1);     // warp and thread inside a compute group
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const bf16* bb = reinterpret_cast<const bf16*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    bf16* yb = reinterpret_cast<bf16*>(p.out.p) + n * p.out.sN + h * p.out.sH;
    float* vob = reinterpret_cast<float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH;
    float* W = p.W + n * p.wN + h * p.wH;
    const int nchunks = (p.L + CH - 1) / CH;
    const int row0 = 16 * gw, r0 = row0 + g, r1 = r0 + 8;      // the chunk rows (and state rows) this thread holds
    volatile int* failed = &s.failed;

    if (tid == 0) {
        for (int i = 0; i < NSTAGE; i++) tc::mbar_init(&s.bar_full[i], 1);
        tc::mbar_init(&s.bar_gram, 1);
        tc::mbar_init(&s.bar_ckcv, 1);
        tc::mbar_init(&s.bar_p, 1);
        tc::mbar_init(&s.bar_s, 1);
        tc::mbar_init(&s.bar_y, 1);
        tc::mbar_init(&s.bar_t_ready, NG);
        tc::mbar_init(&s.bar_ck_ready, NG);
        tc::mbar_init(&s.bar_u_ready, NG);
        tc::mbar_init(&s.bar_s_ready, NG);
        tc::mbar_init(&s.bar_y_read, NG);
        s.failed = 0;
        tc::fence_barrier_init();
    }
    if (warp == 8) tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t tlane = tmem + ((uint32_t)(gw * 32) << 16);      // this warp's quarter of the lanes

    if (role == 0) {
        // ---- the state: global -> registers -> tensor memory (fp32) and shared memory (bf16)
        float S[32];
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float2 a = *reinterpret_cast<const float2*>(W + (long long)r0 * p.wE + 8 * j + 2 * t4);
            const float2 c = *reinterpret_cast<const float2*>(W + (long long)r1 * p.wE + 8 * j + 2 * t4);
            S[4 * j] = a.x; S[4 * j + 1] = a.y; S[4 * j + 2] = c.x; S[4 * j + 3] = c.y;
            pk[2 * j] = pack_bf16(a.x, a.y);
            pk[2 * j + 1] = pack_bf16(c.x, c.y);
        }
        tc::st_frag_swz(s.sb, row0, pk, lane);
        tc::tmem_st_16x64(tlane + COL_S, S);
        tc::tmem_wait_st();
        tc::fence_proxy_async();
        tc::tc_fence_before();
    }
    __syncthreads();

    if (role == 2) {
        // =============================================================== issuing thread
        if (lane == 0) {
            tc::tc_fence_after();
            tc::tma_prefetch_desc(&tm_q);
            tc::tma_prefetch_desc(&tm_k);
            tc::tma_prefetch_desc(&tm_v);
            auto issue_tma = [&](int c) {
                if (c < nchunks) {
                    const int st = c % NSTAGE;
                    tc::mbar_expect_tx(&s.bar_full[st], 3 * tc::kTileBytes);
                    tc::tma_load_4d(s.k[st], &tm_k, &s.bar_full[st], 0, c * CH, h, n);
                    tc::tma_load_4d(s.q[st], &tm_q, &s.bar_full[st], 0, c * CH, h, n);
                    tc::tma_load_4d(s.v[st], &tm_v, &s.bar_full[st], 0, c * CH, h, n);
                }
            };
            issue_tma(0); issue_tma(1); issue_tma(2);
            uint64_t dk[NSTAGE], dq[NSTAGE], dv[NSTAGE];
#pragma unroll
            for (int i = 0; i < NSTAGE; i++) {
                dk[i] = tc::smem_desc(tc::smem_addr(s.k[i]));
                dq[i] = tc::smem_desc(tc::smem_addr(s.q[i]));
                dv[i] = tc::smem_desc(tc::smem_addr(s.v[i]));
            }
            const uint64_t daq[2] = {tc::smem_desc(tc::smem_addr(s.aq[0])), tc::smem_desc(tc::smem_addr(s.aq[1]))};
            const uint64_t dth = tc::smem_desc(tc::smem_addr(s.th)), dtl = tc::smem_desc(tc::smem_addr(s.tl));
            const uint64_t dck = tc::smem_desc(tc::smem_addr(s.ck)), dsb = tc::smem_desc(tc::smem_addr(s.sb));
            const uint64_t duh = tc::smem_desc(tc::smem_addr(s.uh)), dul = tc::smem_desc(tc::smem_addr(s.ul));
            auto sel = [&](const uint64_t (&d)[NSTAGE], int st) { return st == 0 ? d[0] : (st == 1 ? d[1] : d[2]); };

            TCP_BEGIN
            auto gram = [&](int c) {
                const int st = c % NSTAGE;
                tc::mbar_wait(&s.bar_full[st], (c / NSTAGE) & 1, failed);
                TCP(9)
                tc::tc_fence_after();
                product<false, false, false>(tmem + COL_AKK, sel(dk, st), sel(dk, st), false);
                product<false, false, false>(tmem + COL_AQK, sel(dq, st), sel(dk, st), false);
                tc::mma_commit(&s.bar_gram);
            };
            auto ckcv = [&](int c) {
                const int st = c % NSTAGE;
                tc::mbar_wait(&s.bar_t_ready, c & 1, failed);
                TCP(10)
                tc::tc_fence_after();
                product<false, true, false>(tmem + COL_CK, dth, sel(dk, st), false);
                product<false, true, false>(tmem + COL_CK, dtl, sel(dk, st), true);
                product<false, true, false>(tmem + COL_W, dth, sel(dv, st), false);
                product<false, true, false>(tmem + COL_W, dtl, sel(dv, st), true);
                tc::mma_commit(&s.bar_ckcv);
            };
            auto wprod = [&](int c) {       // w(c) = Cv(c) - Ck(c) S(c): needs Ck(c) as an operand and the bf16 copy of S(c)
                tc::mbar_wait(&s.bar_ck_ready, c & 1, failed);
                TCP(11)
                tc::tc_fence_after();
                product<false, true, true>(tmem + COL_W, dck, dsb, true);
                tc::mma_commit(&s.bar_p);
            };
            gram(0);
            ckcv(0);
            wprod(0);
#ifdef FWP_TC_PROF
            for (int i = 0; i < 16; i++) _pt[i] = 0;
            _pc = clock64();
#endif
            for (int c = 0; c < nchunks; c++) {
                const int st = c % NSTAGE;
                const bool has_next = c + 1 < nchunks;
                if (has_next) gram(c + 1);
                TCP(0)
                // the state first (it is on the chain), then y
                tc::mbar_wait(&s.bar_u_ready, c & 1, failed);
                TCP(1)
                tc::tc_fence_after();
                product<true, true, false>(tmem + COL_S, sel(dk, st), duh, true);
                product<true, true, false>(tmem + COL_S, sel(dk, st), dul, true);
                tc::mma_commit(&s.bar_s);
                TCP(2)
                if (c > 0) { tc::mbar_wait(&s.bar_y_read, (c - 1) & 1, failed); tc::tc_fence_after(); }
                TCP(3)
                product<false, true, false>(tmem + COL_Y, sel(dq, st), dsb, false);
                product<false, true, false>(tmem + COL_Y, c & 1 ? daq[1] : daq[0], duh, true);
                tc::mma_commit(&s.bar_y);
                TCP(4)
                if (has_next) ckcv(c + 1);
                TCP(5)
                tc::mbar_wait(&s.bar_s_ready, c & 1, failed);      // bf16 copy of S(c+1) written
                TCP(6)
                if (has_next) wprod(c + 1);
                TCP(7)
                // y(c) read by the chain warps: its products (the last readers of this stage) are complete
                if (c + NSTAGE < nchunks) {
                    tc::mbar_wait(&s.bar_y_read, c & 1, failed);
                    TCP(12)
                    issue_tma(c + NSTAGE);
                }
                TCP(8)
            }
            TCP_END(32)
        }
    } else if (role == 1) {
        // =============================================================== preparing warps (one chunk ahead of the chain)
        auto load_beta = [&](int c) -> float {      // threads 0..63 of the group: beta of step c * 64 + gtid, zero past the end
            const int t = c * CH + gtid;
            return (gtid < CH && t < p.L) ? __bfloat162float(bb[(long long)t * p.beta.sL]) : 0.f;
        };
        float bnext = load_beta(0);
        TCP_BEGIN
        for (int c = 0; c < nchunks; c++) {
            float* bs = s.b[c & 1];
            if (gtid < CH) bs[gtid] = bnext;
            bnext = load_beta(c + 1);
            tc::group_sync(2, NG);
            TCP(0)
            tc::mbar_wait(&s.bar_gram, c & 1, failed);
            TCP(1)
            tc::tc_fence_after();
            float nn[32];
            {
                float aqk[32];
                tc::tmem_ld_16x64(nn, tlane + COL_AKK);
                tc::tmem_ld_16x64(aqk, tlane + COL_AQK);
                tc::tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c0 = 8 * j + 2 * t4;
                    const float b0 = bs[c0], b1 = bs[c0 + 1];
                    pk[2 * j] = pack_bf16(c0 <= r0 ? aqk[4 * j] : 0.f, c0 + 1 <= r0 ? aqk[4 * j + 1] : 0.f);
                    pk[2 * j + 1] = pack_bf16(c0 <= r1 ? aqk[4 * j + 2] : 0.f, c0 + 1 <= r1 ? aqk[4 * j + 3] : 0.f);
                    nn[4 * j] = c0 < r0 ? nn[4 * j] * b0 : 0.f;
                    nn[4 * j + 1] = c0 + 1 < r0 ? nn[4 * j + 1] * b1 : 0.f;
                    nn[4 * j + 2] = c0 < r1 ? nn[4 * j + 2] * b0 : 0.f;
                    nn[4 * j + 3] = c0 + 1 < r1 ? nn[4 * j + 3] * b1 : 0.f;
                }
                tc::st_frag_swz(s.aq[c & 1], row0, pk, lane);
            }
            TCP(2)
            // N as four 16 x 16 blocks of this warp's rows, in the [2][4] fragment form of the warp-level mma helpers
            float N[4][2][4], X[4][2][4];
#pragma unroll
            for (int cbk = 0; cbk < 4; cbk++)
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) { N[cbk][j][i] = nn[4 * (2 * cbk + j) + i]; X[cbk][j][i] = 0.f; }
            float Y[2][4];      // T - I of the diagonal block
            {
                // diagonal block D = N[gw][gw]: Y = (I - D)(I + D^2)(I + D^4)(I + D^8) - I
                float D1[2][4];
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float d = 0.f;
#pragma unroll
                        for (int cbk = 0; cbk < 4; cbk++) d = cbk == gw ? N[cbk][j][i] : d;
                        D1[j][i] = d;
                        Y[j][i] = -d;
                    }
                unsigned a[4], bN[4], b2[4];
                float N2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, D1);
                b_of(bN, D1);
                mm(N2, a, bN);
                b_of(b2, N2);
                {
                    float N3[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    mm(N3, a, b2);
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int i = 0; i < 4; i++) Y[j][i] += N2[j][i] - N3[j][i];
                }
                float N4[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, N2);
                mm(N4, a, b2);
                unsigned b4[4];
                b_of(b4, N4);
                {
                    float Z1[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    a_of(a, Y);
                    mm(Z1, a, b4);
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int i = 0; i < 4; i++) Y[j][i] += N4[j][i] + Z1[j][i];
                }
                float N8[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, N4);
                mm(N8, a, b4);
                {
                    unsigned b8[4];
                    b_of(b8, N8);
                    float Z2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    a_of(a, Y);
                    mm(Z2, a, b8);
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int i = 0; i < 4; i++) Y[j][i] += N8[j][i] + Z2[j][i];
                }
            }
            // store a 16 x 16 block of X (rows 16 gw.., columns 16 cbk..) row-major for the warps below
            auto put_x = [&](int cbk, const float (&blk)[2][4]) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    *reinterpret_cast<unsigned*>(s.x + r0 * LDX + 16 * cbk + 8 * j + 2 * t4) = pack_bf16(blk[j][0], blk[j][1]);
                    *reinterpret_cast<unsigned*>(s.x + r1 * LDX + 16 * cbk + 8 * j + 2 * t4) = pack_bf16(blk[j][2], blk[j][3]);
                }
            };
            put_x(gw, Y);
            unsigned ya[4];
            a_of(ya, Y);
            // block forward substitution, one block diagonal per round: round d gives X[gw][gw - d]
#pragma unroll
            for (int d = 1; d < 4; d++) {
                tc::group_sync(2, NG);
                if (gw >= d) {
                    const int cbk = gw - d;
                    float R[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    for (int l = cbk; l < gw; l++) {      // sum_l N[gw][l] X[l][cbk]
                        float Nl[2][4];
#pragma unroll
                        for (int j = 0; j < 2; j++)
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                float v = 0.f;
#pragma unroll
                                for (int q4 = 0; q4 < 4; q4++) v = q4 == l ? N[q4][j][i] : v;
                                Nl[j][i] = v;
                            }
                        unsigned na[4], xb[4];
                        a_of(na, Nl);
                        ldb_kn(xb, s.x + (16 * l) * LDX + 16 * cbk, LDX, lane);
                        mm(R, na, xb);
                    }
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            float v = 0.f;
#pragma unroll
                            for (int q4 = 0; q4 < 4; q4++) v = q4 == cbk ? N[q4][j][i] : v;
                            R[j][i] += v;       // N[gw][cbk] enters in fp32: the first-order term of T stays exact
                        }
                    unsigned rb[4];
                    b_of(rb, R);
                    float P2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    mm(P2, ya, rb);
                    float Xn[2][4];
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int i = 0; i < 4; i++) Xn[j][i] = -(R[j][i] + P2[j][i]);
                    if (d < 3 || gw < 3) put_x(cbk, Xn);
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++)
                        if (q4 == cbk) {
#pragma unroll
                            for (int j = 0; j < 2; j++)
#pragma unroll
                                for (int i = 0; i < 4; i++) X[q4][j][i] = Xn[j][i];
                        }
                }
            }
            TCP(3)
            // T = I + X in two bf16 parts, rows r0, r1 of the K-major tiles.  The previous chunk's Ck, Cv products, which
            // read these tiles, completed before this warp passed its wait for them at the end of the last iteration.
            {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int cbk = 0; cbk < 4; cbk++)
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        const int c0 = 16 * cbk + 8 * j + 2 * t4;
                        float x0 = X[cbk][j][0], x1 = X[cbk][j][1], x2 = X[cbk][j][2], x3 = X[cbk][j][3];
                        if (cbk == gw) { x0 = Y[j][0]; x1 = Y[j][1]; x2 = Y[j][2]; x3 = Y[j][3]; }
                        x0 += c0 == r0 ? 1.f : 0.f; x1 += c0 + 1 == r0 ? 1.f : 0.f;
                        x2 += c0 == r1 ? 1.f : 0.f; x3 += c0 + 1 == r1 ? 1.f : 0.f;
                        split_bf16(x0, x1, hi[2 * (2 * cbk + j)], lo[2 * (2 * cbk + j)]);
                        split_bf16(x2, x3, hi[2 * (2 * cbk + j) + 1], lo[2 * (2 * cbk + j) + 1]);
                    }
                tc::st_frag_swz(s.th, row0, hi, lane);
                tc::st_frag_swz(s.tl, row0, lo, lane);
            }
            tc::fence_proxy_async();
            tc::tc_fence_before();
            tc::mbar_arrive(&s.bar_t_ready);
            TCP(4)

            // Ck -> bf16 left operand of the w product
            tc::mbar_wait(&s.bar_ckcv, c & 1, failed);
            TCP(5)
            tc::tc_fence_after();
            {
                float ckr[32];
                tc::tmem_ld_16x64(ckr, tlane + COL_CK);
                tc::tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    pk[2 * j] = pack_bf16(ckr[4 * j], ckr[4 * j + 1]);
                    pk[2 * j + 1] = pack_bf16(ckr[4 * j + 2], ckr[4 * j + 3]);
                }
                tc::st_frag_swz(s.ck, row0, pk, lane);
            }
            tc::fence_proxy_async();
            tc::tc_fence_before();
            tc::mbar_arrive(&s.bar_ck_ready);
            TCP(6)
        }
        TCP_END(16)
    } else {
        // =============================================================== chain warps
        TCP_BEGIN
        for (int c = 0; c < nchunks; c++) {
            const int st = c % NSTAGE, t0 = c * CH, nt = min(CH, p.L - t0);
            const float* bs = s.b[c & 1];
            // w -> u (two bf16 parts) and v_old
            tc::mbar_wait(&s.bar_full[st], (c / NSTAGE) & 1, failed);      // the V tile read below (long complete)
            tc::mbar_wait(&s.bar_p, c & 1, failed);
            TCP(0)
            tc::tc_fence_after();
            {
                float w[32];
                tc::tmem_ld_16x64(w, tlane + COL_W);
                uint32_t vp[16];
                tc::ld_frag_swz(vp, s.v[st], row0, lane);
                const float br0 = bs[r0], br1 = bs[r1];
                tc::tmem_wait_ld();
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    split_bf16(br0 * w[4 * j], br0 * w[4 * j + 1], hi[2 * j], lo[2 * j]);
                    split_bf16(br1 * w[4 * j + 2], br1 * w[4 * j + 3], hi[2 * j + 1], lo[2 * j + 1]);
                }
                tc::st_frag_swz(s.uh, row0, hi, lane);
                tc::st_frag_swz(s.ul, row0, lo, lane);
                tc::fence_proxy_async();
                tc::tc_fence_before();
                tc::mbar_arrive(&s.bar_u_ready);
                TCP(1)
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c0 = 8 * j + 2 * t4;
                    const __nv_bfloat162 v0 = *reinterpret_cast<const __nv_bfloat162*>(&vp[2 * j]);
                    const __nv_bfloat162 v1 = *reinterpret_cast<const __nv_bfloat162*>(&vp[2 * j + 1]);
                    if (r0 < nt)
                        *reinterpret_cast<float2*>(vob + (long long)(t0 + r0) * p.v_old.sL + c0) =
                            make_float2(__low2float(v0) - w[4 * j], __high2float(v0) - w[4 * j + 1]);
                    if (r1 < nt)
                        *reinterpret_cast<float2*>(vob + (long long)(t0 + r1) * p.v_old.sL + c0) =
                            make_float2(__low2float(v1) - w[4 * j + 2], __high2float(v1) - w[4 * j + 3]);
                }
            }
            TCP(2)
            // the new state -> bf16 copy (and, after the last chunk, back to global memory)
            tc::mbar_wait(&s.bar_s, c & 1, failed);
            TCP(3)
            tc::tc_fence_after();
            {
                float S[32];
                tc::tmem_ld_16x64(S, tlane + COL_S);
                tc::tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    pk[2 * j] = pack_bf16(S[4 * j], S[4 * j + 1]);
                    pk[2 * j + 1] = pack_bf16(S[4 * j + 2], S[4 * j + 3]);
                }
                // the y product of this chunk still reads the old copy: wait for it before overwriting
                TCP(4)
                tc::mbar_wait(&s.bar_y, c & 1, failed);
                TCP(5)
                tc::st_frag_swz(s.sb, row0, pk, lane);
                tc::fence_proxy_async();
                tc::tc_fence_before();
                tc::mbar_arrive(&s.bar_s_ready);
                TCP(6)
                if (c + 1 == nchunks) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int c0 = 8 * j + 2 * t4;
                        *reinterpret_cast<float2*>(W + (long long)r0 * p.wE + c0) = make_float2(S[4 * j], S[4 * j + 1]);
                        *reinterpret_cast<float2*>(W + (long long)r1 * p.wE + c0) = make_float2(S[4 * j + 2], S[4 * j + 3]);
                    }
                }
            }
            // y -> global memory through a row-major staging tile (16-byte stores)
            tc::tc_fence_after();
            {
                float y[32];
                tc::tmem_ld_16x64(y, tlane + COL_Y);
                tc::tmem_wait_ld();
                tc::tc_fence_before();
                tc::mbar_arrive(&s.bar_y_read);
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    pk[2 * j] = pack_bf16(y[4 * j], y[4 * j + 1]);
                    pk[2 * j + 1] = pack_bf16(y[4 * j + 2], y[4 * j + 3]);
                }
                tc::st_frag_rowmajor(s.ys, LDX, row0, pk, lane);
            }
            tc::group_sync(1, NG);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int idx = gtid + NG * i, row = idx >> 3, part = (idx & 7) * 8;
                if (row < nt)
                    *reinterpret_cast<uint4*>(yb + (long long)(t0 + row) * p.out.sL + part) =
                        *reinterpret_cast<const uint4*>(s.ys + row * LDX + part);
            }
            tc::group_sync(1, NG);
            TCP(7)
        }
        TCP_END(0)
    }

    tc::tc_fence_before();
    __syncthreads();
    if (*failed) {
        // copies or products may still be in flight into this CTA's memory: give them time before the CTA ends
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        if (tid == 0) atomicExch(&g_tc_fault, 1);
        __syncthreads();
    }
    if (warp == 8) tc::tmem_free(tmem, TMEM_COLS);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point query (the library does not link libcuda)
static TcEncodeFn tc_encode_fn() {
    static TcEncodeFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<TcEncodeFn>(ptr);
    }();
    return fn;
}

// (N, H, L, 64) bf16 tensor with a unit inner stride as a 4-D map, boxes of 64 steps x 64 elements, 128-byte swizzle,
// rows past L read as zero
static bool tc_make_map(CUtensorMap* m, const Row4& r, int N, int H, int L) {
    TcEncodeFn enc = tc_encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[4] = {64, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)r.sL * 2, (cuuint64_t)r.sH * 2, (cuuint64_t)r.sN * 2};
    const cuuint32_t box[4] = {64, 64, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, r.p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace fwp
