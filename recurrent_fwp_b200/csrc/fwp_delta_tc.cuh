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
// Every 64-deep contraction is a tcgen05.mma (M = N = 64, K = 16, four instructions per product) issued by one
// thread, operands in 128-byte-swizzled shared-memory tiles, fp32 accumulators in tensor memory:
//   S (the fp32 master copy of the state, updated in place by S += K^T u), w (Cv, then Cv - Ck S0 accumulated into
//   it with the negated-A form), y, Akk, Aqk, Ck.
// K, Q, V tiles arrive by TMA tile loads (three stages, one mbarrier each).  The tiles the kernel produces itself
// (Aqk, T, Ck, u, the bf16 copy of S) are written from registers in the same swizzled layout; T and u are kept
// as two bf16 parts (hi + lo) so that the products they enter carry 16 mantissa bits.
// The inverse is blocked 16 x 16: warp w owns rows 16w..16w+15 of the chunk (the quarter of the tensor-memory
// lanes it can read), inverts its diagonal block in registers by the nilpotent product
// (I - D)(I + D^2)(I + D^4)(I + D^8) and obtains the blocks left of it by block forward substitution,
//   T[w][c] = -(I + Y_ww) (N[w][c] + sum_{c <= l < w} N[w][l] X[l][c]),   X = T - I,
// with the blocks of the warps above exchanged through shared memory (three rounds); these 16-wide products run on
// warp-level mma, everything 64 wide on tcgen05.
//
// One CTA of four warps per sequence; the work of two consecutive chunks is interleaved so that the tensor
// pipe and the TMA run while the warps move accumulators between tensor memory and shared memory:
//   1  issue Gram(c+1)                      4  wait; y(c) out, S -> bf16 copy; refill the freed stage by TMA
//   2  wait w(c); u, v_old; issue y, S += K^T u     5  wait; Ck(c+1) -> bf16; issue w(c+1) = Cv - Ck S
//   3  wait Gram(c+1); inverse; issue Ck, Cv(c+1)
// Every mbarrier wait is bounded; a wait that runs out marks the CTA as failed, after which it stops waiting,
// finishes its barrier sequence, frees its tensor memory and raises the device flag fwp_delta_device_fault() reads.
#pragma once
#include <cuda.h>
#include "fwp_delta_params.cuh"
#include "fwp_tc.cuh"

namespace fwp {

static __device__ int g_tc_fault;
#ifdef FWP_TC_PROF
static __device__ long long g_tc_prof[16];
#define TCP(i) { const long long _n = clock64(); if (tid == 0 && blockIdx.x == 0) { _pt[i] += _n - _pc; } _pc = _n; }
#else
#define TCP(i)
#endif

namespace tcd {

using namespace cb;     // warp-level mma helpers of the 16-step kernels (pack_bf16, split_bf16, a_of, b_of, mm, ldb_kn)

constexpr int CH = 64;                  // steps per chunk
constexpr int NTH = 128;                // four warps
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
    __nv_bfloat16 x[CH * LDX];                  // X = T - I, lower blocks, row-major (exchange between warps)
    __nv_bfloat16 ys[CH * LDX];                 // y, [t][m] row-major (staging for 16-byte stores)
    float b[2][CH];
    uint64_t bar_full[NSTAGE], bar_gram, bar_ckcv, bar_p, bar_b2;
    uint32_t tmem_base;
    int failed;
};
// Tensor memory is taken whole (512 columns); that is only safe while a second CTA cannot become resident on the
// SM and wait for columns forever, which the shared-memory footprint guarantees.
static_assert(sizeof(Smem) > 116 * 1024, "two CTAs per SM would deadlock on the tensor-memory allocation");
static_assert(sizeof(Smem) + 1024 <= 227 * 1024, "shared memory budget");

}  // namespace tcd

__global__ void __launch_bounds__(tcd::NTH, 1)
delta_fwd_tc_kernel(const DeltaFwdParams p, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    using namespace tcd;
    using bf16 = __nv_bfloat16;
    extern __shared__ unsigned char tc_smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const bf16* bb = reinterpret_cast<const bf16*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    bf16* yb = reinterpret_cast<bf16*>(p.out.p) + n * p.out.sN + h * p.out.sH;
    float* vob = reinterpret_cast<float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH;
    float* W = p.W + n * p.wN + h * p.wH;
    const int nchunks = (p.L + CH - 1) / CH;
    const int r0 = 16 * warp + g, r1 = r0 + 8;          // the two chunk rows (and state rows) this thread holds
    volatile int* failed = &s.failed;
#ifdef FWP_TC_PROF
    long long _pt[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}, _pc = clock64();
#endif

    if (tid == 0) {
        for (int i = 0; i < NSTAGE; i++) tc::mbar_init(&s.bar_full[i], 1);
        tc::mbar_init(&s.bar_gram, 1);
        tc::mbar_init(&s.bar_ckcv, 1);
        tc::mbar_init(&s.bar_p, 1);
        tc::mbar_init(&s.bar_b2, 1);
        s.failed = 0;
        tc::fence_barrier_init();
        tc::tma_prefetch_desc(&tm_q);
        tc::tma_prefetch_desc(&tm_k);
        tc::tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);      // this warp's quarter of the lanes

    auto issue_tma = [&](int c) {      // thread 0 only
        if (c < nchunks) {
            const int st = c % NSTAGE;
            tc::mbar_expect_tx(&s.bar_full[st], 3 * tc::kTileBytes);
            tc::tma_load_4d(s.k[st], &tm_k, &s.bar_full[st], 0, c * CH, h, n);
            tc::tma_load_4d(s.q[st], &tm_q, &s.bar_full[st], 0, c * CH, h, n);
            tc::tma_load_4d(s.v[st], &tm_v, &s.bar_full[st], 0, c * CH, h, n);
        }
    };
    auto load_beta = [&](int c) -> float {      // threads 0..63: beta of step c * 64 + tid, zero past the end
        const int t = c * CH + tid;
        return (tid < CH && t < p.L) ? __bfloat162float(bb[(long long)t * p.beta.sL]) : 0.f;
    };
    if (tid == 0) { issue_tma(0); issue_tma(1); issue_tma(2); }

    // ---- the state: global -> registers -> tensor memory (fp32) and shared memory (bf16)
    {
        float S[32];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float2 a = *reinterpret_cast<const float2*>(W + (long long)r0 * p.wE + 8 * j + 2 * t4);
            const float2 c = *reinterpret_cast<const float2*>(W + (long long)r1 * p.wE + 8 * j + 2 * t4);
            S[4 * j] = a.x; S[4 * j + 1] = a.y; S[4 * j + 2] = c.x; S[4 * j + 3] = c.y;
            *reinterpret_cast<unsigned*>(s.sb + tc::swz(r0, 8 * j + 2 * t4)) = pack_bf16(a.x, a.y);
            *reinterpret_cast<unsigned*>(s.sb + tc::swz(r1, 8 * j + 2 * t4)) = pack_bf16(c.x, c.y);
        }
        tc::tmem_st_16x64(tlane + COL_S, S);
        tc::tmem_wait_st();
    }
    if (tid < CH) s.b[0][tid] = load_beta(0);
    float bnext = load_beta(1);
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();

    // ---- pieces of the schedule (every thread runs them; thread 0 issues)
    auto issue_gram = [&](int c) {
        const int st = c % NSTAGE;
        tc::mbar_wait(&s.bar_full[st], (c / NSTAGE) & 1, failed);
        TCP(1)
        if (tid == 0) {
            tc::tc_fence_after();
            const uint32_t ka = tc::smem_addr(s.k[st]), qa = tc::smem_addr(s.q[st]);
            tc::mma_64x64x64<false, false, false>(tmem + COL_AKK, ka, ka, false);
            tc::mma_64x64x64<false, false, false>(tmem + COL_AQK, qa, ka, false);
            tc::mma_commit(&s.bar_gram);
        }
        __syncwarp();
        TCP(2)
    };

    // Gram tiles -> masked Aqk, T = (I + N)^-1 in two bf16 parts; then Ck = T K and Cv = T V are issued
    auto prep_mid = [&](int c) {
        const int st = c % NSTAGE;
        const float* bs = s.b[c & 1];
        tc::mbar_wait(&s.bar_gram, c & 1, failed);
        TCP(6)
        tc::tc_fence_after();
        float nn[32];
        {
            float aqk[32];
            tc::tmem_ld_16x64(nn, tlane + COL_AKK);
            tc::tmem_ld_16x64(aqk, tlane + COL_AQK);
            tc::tmem_wait_ld();
            unsigned char* aq = s.aq[c & 1];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c0 = 8 * j + 2 * t4;
                const float b0 = bs[c0], b1 = bs[c0 + 1];
                *reinterpret_cast<unsigned*>(aq + tc::swz(r0, c0)) =
                    pack_bf16(c0 <= r0 ? aqk[4 * j] : 0.f, c0 + 1 <= r0 ? aqk[4 * j + 1] : 0.f);
                *reinterpret_cast<unsigned*>(aq + tc::swz(r1, c0)) =
                    pack_bf16(c0 <= r1 ? aqk[4 * j + 2] : 0.f, c0 + 1 <= r1 ? aqk[4 * j + 3] : 0.f);
                nn[4 * j] = c0 < r0 ? nn[4 * j] * b0 : 0.f;
                nn[4 * j + 1] = c0 + 1 < r0 ? nn[4 * j + 1] * b1 : 0.f;
                nn[4 * j + 2] = c0 < r1 ? nn[4 * j + 2] * b0 : 0.f;
                nn[4 * j + 3] = c0 + 1 < r1 ? nn[4 * j + 3] * b1 : 0.f;
            }
        }
        TCP(7)
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
            // diagonal block D = N[warp][warp]: Y = (I - D)(I + D^2)(I + D^4)(I + D^8) - I
            float D1[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float d = 0.f;
#pragma unroll
                    for (int cbk = 0; cbk < 4; cbk++) d = cbk == warp ? N[cbk][j][i] : d;
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
        // store a 16 x 16 block of X (rows 16 warp.., columns 16 cbk..) row-major for the warps below
        auto put_x = [&](int cbk, const float (&blk)[2][4]) {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                *reinterpret_cast<unsigned*>(s.x + r0 * LDX + 16 * cbk + 8 * j + 2 * t4) = pack_bf16(blk[j][0], blk[j][1]);
                *reinterpret_cast<unsigned*>(s.x + r1 * LDX + 16 * cbk + 8 * j + 2 * t4) = pack_bf16(blk[j][2], blk[j][3]);
            }
        };
        put_x(warp, Y);
        unsigned ya[4];
        a_of(ya, Y);
        // block forward substitution, one block diagonal per round: round d gives X[warp][warp - d]
#pragma unroll
        for (int d = 1; d < 4; d++) {
            __syncthreads();
            if (warp >= d) {
                const int cbk = warp - d;
                float R[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                for (int l = cbk; l < warp; l++) {      // sum_l N[warp][l] X[l][cbk]
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
                        R[j][i] += v;       // N[warp][cbk] enters in fp32: the first-order term of T stays exact
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
                if (d < 3 || warp < 3) put_x(cbk, Xn);
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
        TCP(8)
        // T = I + X in two bf16 parts, rows r0, r1 of the K-major tiles
#pragma unroll
        for (int cbk = 0; cbk < 4; cbk++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int c0 = 16 * cbk + 8 * j + 2 * t4;
                float x0 = X[cbk][j][0], x1 = X[cbk][j][1], x2 = X[cbk][j][2], x3 = X[cbk][j][3];
                if (cbk == warp) { x0 = Y[j][0]; x1 = Y[j][1]; x2 = Y[j][2]; x3 = Y[j][3]; }
                x0 += c0 == r0 ? 1.f : 0.f; x1 += c0 + 1 == r0 ? 1.f : 0.f;
                x2 += c0 == r1 ? 1.f : 0.f; x3 += c0 + 1 == r1 ? 1.f : 0.f;
                unsigned hi, lo;
                split_bf16(x0, x1, hi, lo);
                *reinterpret_cast<unsigned*>(s.th + tc::swz(r0, c0)) = hi;
                *reinterpret_cast<unsigned*>(s.tl + tc::swz(r0, c0)) = lo;
                split_bf16(x2, x3, hi, lo);
                *reinterpret_cast<unsigned*>(s.th + tc::swz(r1, c0)) = hi;
                *reinterpret_cast<unsigned*>(s.tl + tc::swz(r1, c0)) = lo;
            }
        tc::fence_proxy_async();
        tc::tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc::tc_fence_after();
            const uint32_t tha = tc::smem_addr(s.th), tla = tc::smem_addr(s.tl);
            const uint32_t ka = tc::smem_addr(s.k[st]), va = tc::smem_addr(s.v[st]);
            tc::mma_64x64x64<false, true, false>(tmem + COL_CK, tha, ka, false);
            tc::mma_64x64x64<false, true, false>(tmem + COL_CK, tla, ka, true);
            tc::mma_64x64x64<false, true, false>(tmem + COL_W, tha, va, false);
            tc::mma_64x64x64<false, true, false>(tmem + COL_W, tla, va, true);
            tc::mma_commit(&s.bar_ckcv);
        }
        __syncwarp();
        TCP(9)
    };

    // Ck -> bf16 left operand; then w = Cv - Ck S0 accumulates into the Cv columns
    auto ck_out = [&](int c) {
        tc::mbar_wait(&s.bar_ckcv, c & 1, failed);
        TCP(12)
        tc::tc_fence_after();
        float ckr[32];
        tc::tmem_ld_16x64(ckr, tlane + COL_CK);
        tc::tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c0 = 8 * j + 2 * t4;
            *reinterpret_cast<unsigned*>(s.ck + tc::swz(r0, c0)) = pack_bf16(ckr[4 * j], ckr[4 * j + 1]);
            *reinterpret_cast<unsigned*>(s.ck + tc::swz(r1, c0)) = pack_bf16(ckr[4 * j + 2], ckr[4 * j + 3]);
        }
        tc::fence_proxy_async();
        tc::tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc::tc_fence_after();
            tc::mma_64x64x64<false, true, true>(tmem + COL_W, tc::smem_addr(s.ck), tc::smem_addr(s.sb), true);
            tc::mma_commit(&s.bar_p);
        }
        __syncwarp();
        TCP(13)
    };

    // w -> u (two bf16 parts) and v_old; then y = Q S0 + Aqk u and S += K^T u
    auto chain_mid = [&](int c) {
        const int st = c % NSTAGE, t0 = c * CH, nt = min(CH, p.L - t0);
        const float* bs = s.b[c & 1];
        tc::mbar_wait(&s.bar_p, c & 1, failed);
        TCP(3)
        tc::tc_fence_after();
        float w[32];
        tc::tmem_ld_16x64(w, tlane + COL_W);
        tc::tmem_wait_ld();
        const float br0 = bs[r0], br1 = bs[r1];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c0 = 8 * j + 2 * t4;
            const __nv_bfloat162 v0 = *reinterpret_cast<const __nv_bfloat162*>(s.v[st] + tc::swz(r0, c0));
            const __nv_bfloat162 v1 = *reinterpret_cast<const __nv_bfloat162*>(s.v[st] + tc::swz(r1, c0));
            if (r0 < nt)
                *reinterpret_cast<float2*>(vob + (long long)(t0 + r0) * p.v_old.sL + c0) =
                    make_float2(__low2float(v0) - w[4 * j], __high2float(v0) - w[4 * j + 1]);
            if (r1 < nt)
                *reinterpret_cast<float2*>(vob + (long long)(t0 + r1) * p.v_old.sL + c0) =
                    make_float2(__low2float(v1) - w[4 * j + 2], __high2float(v1) - w[4 * j + 3]);
            unsigned hi, lo;
            split_bf16(br0 * w[4 * j], br0 * w[4 * j + 1], hi, lo);
            *reinterpret_cast<unsigned*>(s.uh + tc::swz(r0, c0)) = hi;
            *reinterpret_cast<unsigned*>(s.ul + tc::swz(r0, c0)) = lo;
            split_bf16(br1 * w[4 * j + 2], br1 * w[4 * j + 3], hi, lo);
            *reinterpret_cast<unsigned*>(s.uh + tc::swz(r1, c0)) = hi;
            *reinterpret_cast<unsigned*>(s.ul + tc::swz(r1, c0)) = lo;
        }
        TCP(4)
        tc::fence_proxy_async();
        tc::tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc::tc_fence_after();
            const uint32_t ka = tc::smem_addr(s.k[st]), qa = tc::smem_addr(s.q[st]);
            const uint32_t uha = tc::smem_addr(s.uh), ula = tc::smem_addr(s.ul);
            tc::mma_64x64x64<false, true, false>(tmem + COL_Y, qa, tc::smem_addr(s.sb), false);
            tc::mma_64x64x64<false, true, false>(tmem + COL_Y, tc::smem_addr(s.aq[c & 1]), uha, true);
            tc::mma_64x64x64<true, true, false>(tmem + COL_S, ka, uha, true);
            tc::mma_64x64x64<true, true, false>(tmem + COL_S, ka, ula, true);
            tc::mma_commit(&s.bar_b2);
        }
        __syncwarp();
        TCP(5)
    };

    // y out; the new state -> bf16 copy (and, after the last chunk, back to global memory)
    auto chain_out = [&](int c) {
        const int t0 = c * CH, nt = min(CH, p.L - t0);
        tc::mbar_wait(&s.bar_b2, c & 1, failed);
        TCP(10)
        tc::tc_fence_after();
        {
            float y[32];
            tc::tmem_ld_16x64(y, tlane + COL_Y);
            tc::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c0 = 8 * j + 2 * t4;
                *reinterpret_cast<unsigned*>(s.ys + r0 * LDX + c0) = pack_bf16(y[4 * j], y[4 * j + 1]);
                *reinterpret_cast<unsigned*>(s.ys + r1 * LDX + c0) = pack_bf16(y[4 * j + 2], y[4 * j + 3]);
            }
        }
        {
            float S[32];
            tc::tmem_ld_16x64(S, tlane + COL_S);
            tc::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c0 = 8 * j + 2 * t4;
                *reinterpret_cast<unsigned*>(s.sb + tc::swz(r0, c0)) = pack_bf16(S[4 * j], S[4 * j + 1]);
                *reinterpret_cast<unsigned*>(s.sb + tc::swz(r1, c0)) = pack_bf16(S[4 * j + 2], S[4 * j + 3]);
                if (c + 1 == nchunks) {
                    *reinterpret_cast<float2*>(W + (long long)r0 * p.wE + c0) = make_float2(S[4 * j], S[4 * j + 1]);
                    *reinterpret_cast<float2*>(W + (long long)r1 * p.wE + c0) = make_float2(S[4 * j + 2], S[4 * j + 3]);
                }
            }
        }
        tc::fence_proxy_async();
        tc::tc_fence_before();
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int idx = tid + NTH * i, row = idx >> 3, part = (idx & 7) * 8;
            if (row < nt)
                *reinterpret_cast<uint4*>(yb + (long long)(t0 + row) * p.out.sL + part) =
                    *reinterpret_cast<const uint4*>(s.ys + row * LDX + part);
        }
        if (tid == 0) issue_tma(c + NSTAGE);        // the stage of chunk c is free: K, Q, V of chunk c + 3
        __syncwarp();
        TCP(11)
    };

    // ---- chunk 0 is prepared alone, then the interleaved schedule
    TCP(0)
    issue_gram(0);
    prep_mid(0);
    ck_out(0);
#ifdef FWP_TC_PROF
    for (int i = 1; i < 16; i++) _pt[i] = 0;
    _pc = clock64();
#endif
    for (int c = 0; c < nchunks; c++) {
        const bool has_next = c + 1 < nchunks;
        if (tid < CH) s.b[(c + 1) & 1][tid] = bnext;
        if (has_next) issue_gram(c + 1);
        chain_mid(c);
        if (has_next) prep_mid(c + 1);
        chain_out(c);
        bnext = load_beta(c + 2);
        if (has_next) ck_out(c + 1);
    }

#ifdef FWP_TC_PROF
    if (tid == 0 && blockIdx.x == 0)
        for (int i = 0; i < 16; i++) g_tc_prof[i] = _pt[i];
#endif
    tc::tc_fence_before();
    __syncthreads();
    if (*failed) {
        // copies or products may still be in flight into this CTA's memory: give them time before the CTA ends
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        if (tid == 0) atomicExch(&g_tc_fault, 1);
        __syncthreads();
    }
    if (warp == 0) tc::tmem_free(tmem, TMEM_COLS);
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
