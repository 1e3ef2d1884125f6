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
// Every 64-deep contraction is a tcgen05.mma with M = 64, K = 16 (four instructions per product), operands in
// 128-byte-swizzled shared-memory tiles, fp32 accumulators in tensor memory.  Products that share their left
// operand are issued 128 columns wide over two adjacent right-hand tiles:
//   [Akk | Aqk^T] = K [K ; Q]^T     [Ck | Cv] = T [K | V]     [K^T u_hi | K^T u_lo] = K^T [u_hi | u_lo]
//   w = Cv - Ck S0 (accumulated into the Cv columns with the negated-A form),   y = Q S0 + Aqk u_hi
// K, Q, V tiles arrive by TMA tile loads (three stages, one mbarrier each).  The tiles the kernel produces itself
// (Aqk^T, T, Ck, u, the bf16 copy of S) are written from registers in the same swizzled layout (stmatrix); T and u
// are kept as two bf16 parts (hi + lo) so that the products they enter carry 16 mantissa bits.  The fp32 master copy
// of the state lives in the registers of the chain warps, which add the two halves of K^T [u_hi | u_lo] each chunk.
// The inverse is blocked 16 x 16: warp w of the preparing group owns rows 16w..16w+15 of the chunk (the quarter of
// the tensor-memory lanes it can read), inverts its diagonal block in registers by the nilpotent product
// (I - D)(I + D^2)(I + D^4)(I + D^8) and obtains the blocks left of it by block forward substitution,
//   T[w][c] = -(I + Y_ww) (N[w][c] + sum_{c <= l < w} N[w][l] X[l][c]),   X = T - I,
// with the blocks of the warps above exchanged through shared memory (three rounds); these 16-wide products run on
// warp-level mma, everything 64 wide on tcgen05.
//
// One CTA per sequence; five roles that meet only at mbarriers:
//   * chain warps 0-3       per chunk c: w(c) -> u (two parts);  K^T u -> S(c+1) (registers) -> bf16 copy
//   * preparing warps 4-7   one chunk ahead: Akk -> N -> T
//   * helper warps 8-11     Aqk^T -> masked operand, Ck -> bf16 operand (one chunk ahead); v_old(c), y(c) -> global
//   * warp 12, one thread   the products on the chain: Q S(c) | K^T u(c) | Aqk u(c) | w(c+1) = Cv - Ck S(c+1)
//   * warp 13, one thread   the TMA loads and the products beside the chain: Gram(c+1) | [Ck | Cv](c+1)
// Each product waits for the mbarriers on which the producers of its operands (128 threads) arrive after their
// proxy fence, and each batch is followed by a tcgen05.commit onto the mbarrier its consumers wait for.
// The state-dependent chain per chunk is: w product -> u -> K^T u product -> add, round, store.
// Every mbarrier wait is bounded; a wait that runs out marks the CTA as failed, after which nobody waits any more,
// all roles finish their (fixed-length) loops, the CTA frees its tensor memory and raises the device flag that
// fwp_delta_device_fault() reads.
#pragma once
#include <cuda.h>
#include "fwp_delta_params.cuh"
#include "fwp_tc.cuh"

namespace fwp {

static __device__ int g_tc_fault;

namespace tcd {

using namespace cb;     // warp-level mma helpers of the 16-step kernels (pack_bf16, split_bf16, a_of, b_of, mm, ldb_kn)

constexpr int CH = 64;                  // steps per chunk
constexpr int NTH = 480;                // chain 0-3, preparing 4-7, helper 8-11, issuing warps 12 and 13, loading warp 14
constexpr int NG = 128;                 // threads per compute group
constexpr int NSTAGE = 3;
constexpr int LDX = 72;                 // row stride (bf16) of the row-major exchange and output tiles: 144 B, 16-byte aligned
// Tensor memory.  An M = 64 accumulator occupies lanes 0-15 of each quarter of the 128 lanes; a second one can sit in
// lanes 16-31 of the same columns.  Lower lanes: K^T [u_hi | u_lo] (columns 0-127), y (128-191) and two buffers of
// [Ck | w] (192-319, 320-447) for consecutive chunks; upper lanes of columns 0-127: [Akk | Aqk^T].
constexpr uint32_t COL_D = 0, COL_Y = 128, COL_CKW = 192, TMEM_COLS = 512;
constexpr uint32_t COL_AKK = 0, COL_AQK = 64, LANE_G = 16u << 16;
__device__ __forceinline__ uint32_t col_ck(int c) { return COL_CKW + 128u * (uint32_t)(c & 1); }
__device__ __forceinline__ uint32_t col_w(int c) { return col_ck(c) + 64u; }

struct Stage {                          // one chunk's rows; q follows k and v follows q so that [K ; Q] and [K | V] are one operand
    unsigned char k[tc::kTileBytes], q[tc::kTileBytes], v[tc::kTileBytes];
};
struct Smem {
    alignas(1024) Stage st[NSTAGE];
    unsigned char aq[2][tc::kTileBytes];        // Aqk^T, [i][t], zero below the diagonal (MN-major left operand)
    unsigned char th[tc::kTileBytes];           // T hi, [t][i] (K-major left operand)
    unsigned char tl[tc::kTileBytes];           // T lo
    unsigned char ck[2][tc::kTileBytes];        // Ck of two consecutive chunks, [t][e] (K-major left operand)
    unsigned char uh[tc::kTileBytes];           // u hi, [i][m] (MN-major right operand); ul follows it: [u_hi | u_lo] is one operand
    unsigned char ul[tc::kTileBytes];           // u lo
    unsigned char sb[tc::kTileBytes];           // bf16 copy of the state, [e][m] (MN-major right operand)
    __nv_bfloat16 x[CH * LDX];                  // X = T - I, lower blocks, row-major (exchange between preparing warps)
    __nv_bfloat16 ys[CH * LDX];                 // y, [t][m] row-major (staging for 16-byte stores)
    float b[4][CH];                             // beta of four consecutive chunks (the preparing warps run up to two ahead)
    // completion of asynchronous work (one arrival each): TMA stages, tcgen05.commit of the product batches
    uint64_t bar_full[NSTAGE], bar_gram, bar_ckcv[2], bar_p, bar_d, bar_y;
    // operands written / accumulators read by a compute group (128 arrivals each)
    uint64_t bar_t_ready, bar_aq_ready[2], bar_ck_ready[2], bar_u_ready[2], bar_s_ready, bar_w_read[2], bar_y_read, bar_free[2];
    uint32_t tmem_base;
    int failed;
};
// Tensor memory is taken whole (512 columns); that is only safe while a second CTA cannot become resident on the
// SM and wait for columns forever, which the shared-memory footprint guarantees.
static_assert(sizeof(Smem) > 116 * 1024, "two CTAs per SM would deadlock on the tensor-memory allocation");
static_assert(sizeof(Smem) + 1024 <= 227 * 1024, "shared memory budget");

// The four tcgen05.mma of one 64-deep product (M = 64, N columns), from prebuilt descriptors.  Called by a whole
// (converged) warp: every lane carries the same descriptors, which lets them live in uniform registers, and one
// elected lane issues.
template <bool A_MN, bool B_MN, bool NEG_A, int N>
__device__ __forceinline__ void product(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, bool accumulate) {
    constexpr uint32_t id = tc::idesc(A_MN, B_MN, NEG_A, N);
    if (tc::elect_one()) {
#pragma unroll
        for (int k = 0; k < 4; k++)
            tc::mma_issue(d_tmem, a_desc + (uint64_t)(k * (A_MN ? 128 : 2)), b_desc + (uint64_t)(k * (B_MN ? 128 : 2)), id,
                          (accumulate || k > 0) ? 1u : 0u);
    }
    __syncwarp();
}

// fp32 fragment -> bf16 pairs in the order the tile stores take
__device__ __forceinline__ void pack_frag(uint32_t (&pk)[16], const float (&r)[32]) {
#pragma unroll
    for (int j = 0; j < 8; j++) {
        pk[2 * j] = pack_bf16(r[4 * j], r[4 * j + 1]);
        pk[2 * j + 1] = pack_bf16(r[4 * j + 2], r[4 * j + 3]);
    }
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
    const int role = warp >> 2;                         // 0 chain, 1 preparing, 2 helper, 3 issuing
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
        tc::mbar_init(&s.bar_ckcv[0], 1);
        tc::mbar_init(&s.bar_ckcv[1], 1);
        tc::mbar_init(&s.bar_p, 1);
        tc::mbar_init(&s.bar_d, 1);
        tc::mbar_init(&s.bar_y, 1);
        tc::mbar_init(&s.bar_t_ready, NG);
        tc::mbar_init(&s.bar_aq_ready[0], NG);
        tc::mbar_init(&s.bar_aq_ready[1], NG);
        tc::mbar_init(&s.bar_ck_ready[0], NG);
        tc::mbar_init(&s.bar_ck_ready[1], NG);
        tc::mbar_init(&s.bar_u_ready[0], NG);
        tc::mbar_init(&s.bar_u_ready[1], NG);
        tc::mbar_init(&s.bar_s_ready, NG);
        tc::mbar_init(&s.bar_w_read[0], NG);
        tc::mbar_init(&s.bar_w_read[1], NG);
        tc::mbar_init(&s.bar_y_read, NG);
        tc::mbar_init(&s.bar_free[0], NG);
        tc::mbar_init(&s.bar_free[1], NG);
        s.failed = 0;
        tc::fence_barrier_init();
    }
    if (warp == 12) tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = s.tmem_base;
    const uint32_t tlane = tmem + ((uint32_t)(gw * 32) << 16);      // this warp's quarter of the lanes

    float S[32];        // chain warps: the fp32 state, rows r0, r1 in fragment form
    if (role == 0) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float2 a = *reinterpret_cast<const float2*>(W + (long long)r0 * p.wE + 8 * j + 2 * t4);
            const float2 c = *reinterpret_cast<const float2*>(W + (long long)r1 * p.wE + 8 * j + 2 * t4);
            S[4 * j] = a.x; S[4 * j + 1] = a.y; S[4 * j + 2] = c.x; S[4 * j + 3] = c.y;
        }
        pack_frag(pk, S);
        tc::st_frag_swz(s.sb, row0, pk, lane);
        tc::fence_proxy_async();
    }
    __syncthreads();

    if (role == 3) {
        if (warp == 12) {
            // =========================================================== issuing thread A: the products on the chain
            tc::tc_fence_after();
            const uint64_t dsb = tc::smem_desc(tc::smem_addr(s.sb));
            const uint64_t dck[2] = {tc::smem_desc(tc::smem_addr(s.ck[0])), tc::smem_desc(tc::smem_addr(s.ck[1]))};
            const uint64_t duh = tc::smem_desc(tc::smem_addr(s.uh));
            const uint64_t du2 = tc::smem_desc_mn128(tc::smem_addr(s.uh), tc::kTileBytes);
            // w(0) = Cv(0) - Ck(0) S(0)
            tc::mbar_wait(&s.bar_ck_ready[0], 0, failed);
            tc::tc_fence_after();
            product<false, true, true, 64>(tmem + col_w(0), dck[0], dsb, true);
            if (tc::elect_one()) tc::mma_commit(&s.bar_p);
            __syncwarp();
#pragma unroll 1
    #pragma unroll 1
        for (int c = 0; c < nchunks; c++) {
                const int st = c % NSTAGE;
                const uint64_t dk = tc::smem_desc(tc::smem_addr(s.st[st].k)), dq = tc::smem_desc(tc::smem_addr(s.st[st].q));
                // y(c) = Q S(c): needs the y columns read (chunk c - 1); the bf16 copy of S(c) was waited for before w(c)
                tc::mbar_wait(&s.bar_full[st], (c / NSTAGE) & 1, failed);
                if (c > 0) tc::mbar_wait(&s.bar_y_read, (c - 1) & 1, failed);
                tc::tc_fence_after();
                product<false, true, false, 64>(tmem + COL_Y, dq, dsb, false);
                // [K^T u_hi | K^T u_lo]
                tc::mbar_wait(&s.bar_u_ready[c & 1], (c >> 1) & 1, failed);
                tc::tc_fence_after();
                product<true, true, false, 128>(tmem + COL_D, dk, du2, false);
                if (tc::elect_one()) tc::mma_commit(&s.bar_d);
                __syncwarp();
                // y(c) += Aqk u_hi
                tc::mbar_wait(&s.bar_aq_ready[c & 1], (c >> 1) & 1, failed);
                tc::tc_fence_after();
                product<true, true, false, 64>(tmem + COL_Y, tc::smem_desc(tc::smem_addr(s.aq[c & 1])), duh, true);
                if (tc::elect_one()) tc::mma_commit(&s.bar_y);
                __syncwarp();
                // w(c+1) = Cv(c+1) - Ck(c+1) S(c+1)
                tc::mbar_wait(&s.bar_s_ready, c & 1, failed);
                if (c + 1 < nchunks) {
                    tc::mbar_wait(&s.bar_ck_ready[(c + 1) & 1], ((c + 1) >> 1) & 1, failed);
                    tc::tc_fence_after();
                    product<false, true, true, 64>(tmem + col_w(c + 1), (c + 1) & 1 ? dck[1] : dck[0], dsb, true);
                    if (tc::elect_one()) tc::mma_commit(&s.bar_p);
            __syncwarp();
                }
            }
        } else if (warp == 13) {
            // =========================================================== issuing thread B: Gram, [Ck | Cv]
            tc::tc_fence_after();
            const uint64_t dth = tc::smem_desc(tc::smem_addr(s.th)), dtl = tc::smem_desc(tc::smem_addr(s.tl));
            auto gram = [&](int c) {        // [Akk | Aqk^T](c) = K [K ; Q]^T
                const int st = c % NSTAGE;
                tc::mbar_wait(&s.bar_full[st], (c / NSTAGE) & 1, failed);
                tc::tc_fence_after();
                const uint64_t dk = tc::smem_desc(tc::smem_addr(s.st[st].k));
                product<false, false, false, 128>(tmem + LANE_G + COL_AKK, dk, dk, false);
                if (tc::elect_one()) tc::mma_commit(&s.bar_gram);
                __syncwarp();
            };
            // Order: Gram(c+1) as soon as the preparing and helper warps have read Gram(c) (it overwrites those
            // columns), so that the inverse of chunk c+1 starts while [Ck | Cv](c) still waits for the chain.
            gram(0);
#pragma unroll 1
    #pragma unroll 1
        for (int c = 0; c < nchunks; c++) {
                // T(c) written (so Akk(c) is read); Aqk^T(c) read
                tc::mbar_wait(&s.bar_t_ready, c & 1, failed);
                if (c + 1 < nchunks) {
                    tc::mbar_wait(&s.bar_aq_ready[c & 1], (c >> 1) & 1, failed);
                    gram(c + 1);
                }
                // [Ck | Cv](c) goes to the buffer chunk c - 2 used: Ck(c-2) read (ck_ready), w(c-2) read by the chain (u_ready)
                // and by the helper warps (w_read).  Each of these barriers exists twice, one per buffer, so the phase
                // waited for here is the one right before the phase this very product makes possible.
                if (c > 1) {
                    const uint32_t ph = ((c - 2) >> 1) & 1;
                    tc::mbar_wait(&s.bar_ck_ready[c & 1], ph, failed);
                    tc::mbar_wait(&s.bar_u_ready[c & 1], ph, failed);
                    tc::mbar_wait(&s.bar_w_read[c & 1], ph, failed);
                }
                {
                    const int st = c % NSTAGE;
                    tc::tc_fence_after();
                    const uint64_t dkv = tc::smem_desc_mn128(tc::smem_addr(s.st[st].k), 2 * tc::kTileBytes);
                    product<false, true, false, 128>(tmem + col_ck(c), dth, dkv, false);
                    product<false, true, false, 128>(tmem + col_ck(c), dtl, dkv, true);
                    if (tc::elect_one()) tc::mma_commit(&s.bar_ckcv[c & 1]);
                    __syncwarp();
                }
            }
        }
        else if (warp == 14) {
            // =========================================================== loading thread: K, Q, V tiles by TMA
            tc::tma_prefetch_desc(&tm_q);
            tc::tma_prefetch_desc(&tm_k);
            tc::tma_prefetch_desc(&tm_v);
            auto issue_tma = [&](int c) {
                const int st = c % NSTAGE;
                if (tc::elect_one()) {
                    tc::mbar_expect_tx(&s.bar_full[st], 3 * tc::kTileBytes);
                    tc::tma_load_4d(s.st[st].k, &tm_k, &s.bar_full[st], 0, c * CH, h, n);
                    tc::tma_load_4d(s.st[st].q, &tm_q, &s.bar_full[st], 0, c * CH, h, n);
                    tc::tma_load_4d(s.st[st].v, &tm_v, &s.bar_full[st], 0, c * CH, h, n);
                }
                __syncwarp();
            };
            for (int c = 0; c < NSTAGE && c < nchunks; c++) issue_tma(c);
            for (int c = 0; c + NSTAGE < nchunks; c++) {
                // the stage of chunk c is free once the helper warps have read y(c): they read V for v_old before, and
                // the products that read Q and K completed before y(c) was readable
                tc::mbar_wait(&s.bar_free[c & 1], (c >> 1) & 1, failed);
                issue_tma(c + NSTAGE);
            }
        }
    } else if (role == 1) {
        // =============================================================== preparing warps (one chunk ahead of the chain)
        auto load_beta = [&](int c) -> float {      // threads 0..63 of the group: beta of step c * 64 + gtid, zero past the end
            const int t = c * CH + gtid;
            return (gtid < CH && t < p.L) ? __bfloat162float(bb[(long long)t * p.beta.sL]) : 0.f;
        };
        float bnext = load_beta(0);
#pragma unroll 1
        for (int c = 0; c < nchunks; c++) {
            float* bs = s.b[c & 3];
            if (gtid < CH) bs[gtid] = bnext;
            bnext = load_beta(c + 1);
            tc::group_sync(2, NG);
            tc::mbar_wait(&s.bar_gram, c & 1, failed);
            tc::tc_fence_after();
            float nn[32];
            tc::tmem_ld_16x64(nn, tlane + LANE_G + COL_AKK);
            tc::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c0 = 8 * j + 2 * t4;
                const float b0 = bs[c0], b1 = bs[c0 + 1];
                nn[4 * j] = c0 < r0 ? nn[4 * j] * b0 : 0.f;
                nn[4 * j + 1] = c0 + 1 < r0 ? nn[4 * j + 1] * b1 : 0.f;
                nn[4 * j + 2] = c0 < r1 ? nn[4 * j + 2] * b0 : 0.f;
                nn[4 * j + 3] = c0 + 1 < r1 ? nn[4 * j + 3] * b1 : 0.f;
            }
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
#pragma unroll 1
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
            // T = I + X in two bf16 parts, rows r0, r1 of the K-major tiles; the previous chunk's [Ck | Cv] product,
            // which reads these tiles, must have completed
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
                if (c > 0) tc::mbar_wait(&s.bar_ckcv[(c - 1) & 1], ((c - 1) >> 1) & 1, failed);
                tc::st_frag_swz(s.th, row0, hi, lane);
                tc::st_frag_swz(s.tl, row0, lo, lane);
            }
            tc::fence_proxy_async();
            tc::tc_fence_before();
            tc::mbar_arrive(&s.bar_t_ready);
        }
    } else if (role == 2) {
        // =============================================================== helper warps
        auto aq_out = [&](int c) {      // Aqk^T(c): rows are key steps i, columns query steps t; keep t >= i
            tc::mbar_wait(&s.bar_gram, c & 1, failed);
            tc::tc_fence_after();
            float a[32];
            tc::tmem_ld_16x64(a, tlane + LANE_G + COL_AQK);
            tc::tmem_wait_ld();
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c0 = 8 * j + 2 * t4;
                pk[2 * j] = pack_bf16(c0 >= r0 ? a[4 * j] : 0.f, c0 + 1 >= r0 ? a[4 * j + 1] : 0.f);
                pk[2 * j + 1] = pack_bf16(c0 >= r1 ? a[4 * j + 2] : 0.f, c0 + 1 >= r1 ? a[4 * j + 3] : 0.f);
            }
            tc::st_frag_swz(s.aq[c & 1], row0, pk, lane);
            tc::fence_proxy_async();
            tc::tc_fence_before();
            tc::mbar_arrive(&s.bar_aq_ready[c & 1]);
        };
        auto ck_out = [&](int c) {      // Ck(c) -> bf16 left operand of the w product
            tc::mbar_wait(&s.bar_ckcv[c & 1], (c >> 1) & 1, failed);
            tc::tc_fence_after();
            float a[32];
            tc::tmem_ld_16x64(a, tlane + col_ck(c));
            tc::tmem_wait_ld();
            uint32_t pk[16];
            pack_frag(pk, a);
            tc::st_frag_swz(s.ck[c & 1], row0, pk, lane);
            tc::fence_proxy_async();
            tc::tc_fence_before();
            tc::mbar_arrive(&s.bar_ck_ready[c & 1]);
        };
        // iteration c = -1 only prepares chunk 0
#pragma unroll 1
        for (int c = -1; c < nchunks; c++) {
            const int st = (c + NSTAGE) % NSTAGE, t0 = c * CH, nt = min(CH, p.L - t0);
            if (c + 1 < nchunks) aq_out(c + 1);
            if (c < 0) { ck_out(0); continue; }
            // v_old(c) = V - w
            tc::mbar_wait(&s.bar_full[st], (c / NSTAGE) & 1, failed);
            tc::mbar_wait(&s.bar_p, c & 1, failed);
            tc::tc_fence_after();
            {
                float w[32];
                tc::tmem_ld_16x64(w, tlane + col_w(c));
                uint32_t vp[16];
                tc::ld_frag_swz(vp, s.st[st].v, row0, lane);
                tc::tmem_wait_ld();
                tc::tc_fence_before();
                tc::mbar_arrive(&s.bar_w_read[c & 1]);
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
            if (c + 1 < nchunks) ck_out(c + 1);     // before y: the w product of the next chunk waits for it
            // y(c) -> global memory through a row-major staging tile (16-byte stores)
            tc::mbar_wait(&s.bar_y, c & 1, failed);
            tc::tc_fence_after();
            {
                float y[32];
                tc::tmem_ld_16x64(y, tlane + COL_Y);
                tc::tmem_wait_ld();
                tc::tc_fence_before();
                tc::mbar_arrive(&s.bar_y_read);
                tc::mbar_arrive(&s.bar_free[c & 1]);        // this chunk's K, Q, V tiles have no reader left
                uint32_t pk[16];
                pack_frag(pk, y);
                tc::st_frag_rowmajor(s.ys, LDX, row0, pk, lane);
            }
            tc::group_sync(3, NG);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int idx = gtid + NG * i, row = idx >> 3, part = (idx & 7) * 8;
                if (row < nt)
                    *reinterpret_cast<uint4*>(yb + (long long)(t0 + row) * p.out.sL + part) =
                        *reinterpret_cast<const uint4*>(s.ys + row * LDX + part);
            }
            tc::group_sync(3, NG);
        }
    } else {
        // =============================================================== chain warps
#pragma unroll 1
        for (int c = 0; c < nchunks; c++) {
            const float* bs = s.b[c & 3];
            // w -> u (two bf16 parts)
            tc::mbar_wait(&s.bar_p, c & 1, failed);
            tc::tc_fence_after();
            {
                float w[32];
                tc::tmem_ld_16x64(w, tlane + col_w(c));
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
                tc::mbar_arrive(&s.bar_u_ready[c & 1]);
            }
            // S += K^T u_hi + K^T u_lo; the bf16 copy for the next chunk's products
            tc::mbar_wait(&s.bar_d, c & 1, failed);
            tc::tc_fence_after();
            {
                float dh[32], dl[32];
                tc::tmem_ld_16x64(dh, tlane + COL_D);
                tc::tmem_ld_16x64(dl, tlane + COL_D + 64);
                tc::tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) S[i] += dh[i] + dl[i];
                uint32_t pk[16];
                pack_frag(pk, S);
                tc::st_frag_swz(s.sb, row0, pk, lane);
                tc::fence_proxy_async();
                tc::tc_fence_before();
                tc::mbar_arrive(&s.bar_s_ready);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c0 = 8 * j + 2 * t4;
            *reinterpret_cast<float2*>(W + (long long)r0 * p.wE + c0) = make_float2(S[4 * j], S[4 * j + 1]);
            *reinterpret_cast<float2*>(W + (long long)r1 * p.wE + c0) = make_float2(S[4 * j + 2], S[4 * j + 3]);
        }
    }

    tc::tc_fence_before();
    __syncthreads();
    if (*failed) {
        // copies or products may still be in flight into this CTA's memory: give them time before the CTA ends
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        if (tid == 0) atomicExch(&g_tc_fault, 1);
        __syncthreads();
    }
    if (warp == 12) tc::tmem_free(tmem, TMEM_COLS);
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
