// Delta rule in chunkwise (WY / UT-transform) form for 16-bit streams and head dimension 64 (sm_100a).
//
// At d = 64 the per-step kernels are bound by fp32 FMA issue and by the delivery of every operand
// vector to all columns (12 d^2 FMAs per step forward).  Here one CTA of four warps walks a sequence
// in chunks of 16 steps, and every d-sized contraction is a warp-level bf16 tensor-core product
// (mma.sync.m16n8k16, fp32 accumulation).  With S0 the state before the chunk, K, Q, V the chunk's
// rows and b = beta:
//
//   Akk = strict_lower(K K^T), Aqk = lower(Q K^T)                          (bf16 products)
//   [Cv | Ck] = T [V | K],  T = (I + Akk diag(b))^-1   (the unit triangular solve
//               c_t = rhs_t - sum_{i<t} Akk[t,i] b_i c_i as an explicit inverse, see the forward kernel)
//   w = Cv - Ck S0  (= v - v_old),  u = b w,  v_old = (V - Cv) + Ck S0
//   y = Q S0 + Aqk u,   S1 = S0 + K^T u
//
// (the same recurrence as algorithmic/fast_weight/fast_weight_cuda.cu:107-180, regrouped).
// The state is kept transposed, S^T (value index m by key index e): warp w owns the 16 rows
// m in [16w, 16w+16) as a 16 x 64 fp32 accumulator.  That choice keeps the chain in registers:
// the accumulator fragments of S^T, rounded to bf16, are the left operand of S^T Ck^T and S^T Q^T,
// the accumulator fragment of u^T is the left operand of u^T Aqk^T and of the update u^T K, and
// every right operand is a row-major shared-memory tile read with ldmatrix (transposed for K in
// the update).  y leaves through a shared-memory tile as 16-byte row pieces, v_old and u straight from the fragments.
//
// Rounding: the streams are bf16 already; S, Ck and u are rounded to bf16 only as product
// operands, the state itself and all sums stay fp32, and the state update takes u as two bf16 parts.
#pragma once
#include "fwp_delta_params.cuh"

namespace fwp {

namespace cb {

constexpr int D = 64;                   // E = M = 64
constexpr int C = 16;                   // steps per chunk
constexpr int NT = 128;                 // threads: four warps, and one thread per column of [V | K]
constexpr int LDT = 72;                 // row stride of the 16 x 64 bf16 tiles (144 B: ldmatrix rows hit distinct banks)
constexpr int LDQ = 24;                 // row stride of Aqk (bf16; 48 B)
constexpr int LDO = 68;                 // row stride of the fp32 output tiles [t][m]

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)) : "memory");
}
__device__ __forceinline__ void ldsm4t(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)) : "memory");
}
// d += a b, a: 16 x 16 (row), b: 16 x 8 (col), bf16 operands, fp32 accumulation
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&h);
}

// Left-operand fragments of a 16 x 16 row-major bf16 block at `tile` (row stride ld elements):
// lane l supplies the address of row (l & 15), column 8 (l >> 4).
__device__ __forceinline__ void lda_rowmajor(unsigned (&a)[4], const __nv_bfloat16* tile, int ld, int lane) {
    ldsm4(a, tile + (lane & 15) * ld + 8 * (lane >> 4));
}
// Right-operand fragments B[k][n] = X[n][k] from a row-major X (rows n, k contiguous), 16 (n) x 16 (k) block:
// r[0], r[1] = b0, b1 of the n-tile 0..7, r[2], r[3] of the n-tile 8..15.
__device__ __forceinline__ void ldb_nk(unsigned (&r)[4], const __nv_bfloat16* tile, int ld, int lane) {
    ldsm4(r, tile + ((lane & 7) + 8 * (lane >> 4)) * ld + 8 * ((lane >> 3) & 1));
}
// Right-operand fragments B[k][n] = X[k][n] from a row-major X (rows k, n contiguous), 16 (k) x 16 (n) block:
// r[0], r[1] = b0, b1 of the n-tile 0..7, r[2], r[3] of the n-tile 8..15.
__device__ __forceinline__ void ldb_kn(unsigned (&r)[4], const __nv_bfloat16* tile, int ld, int lane) {
    ldsm4t(r, tile + ((lane & 7) + 8 * ((lane >> 3) & 1)) * ld + 8 * (lane >> 4));
}

// rows [t0, t0 + nt) of a (N,H,L,64) bf16 tensor into a tile, one 16-byte piece per thread; rows past nt become zero
__device__ __forceinline__ void load_tile(__nv_bfloat16* tile, const __nv_bfloat16* base, long long sL, int t0, int nt, int tid) {
    const int row = tid >> 3, part = (tid & 7) * 8;
    __nv_bfloat16* dst = tile + row * LDT + part;
    if (row < nt) cp_async16(dst, base + (long long)(t0 + row) * sL + part);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace cb

// ------------------------------------------------------------------ backward
// Chunks are walked from the last to the first.  With S1, G1 = dL/dS1 at the end of the chunk, the saved
// v_old (w = V - v_old, U = b w) and gY = dL/dy:
//   S0 = S1 - K^T U
//   lambda_t = rhs_t - sum_{j>t} Akk[j,t] b_j lambda_j  for rhs = Aqk^T gY + K G1, solved as
//       lambda = Lt + Kt G1 with [Lt | Kt] the solutions for rhs = [Aqk^T gY | K]
//   dv = b lambda,  dbeta = rowsum(lambda w),  G0 = G1 + Q^T gY - K^T (b lambda)
//   dQ = gY S0^T + B K,  B = lower(gY U^T)
//   dK = U G1^T - (b lambda) S0^T + B^T Q - (strict_lower(Z) + strict_lower(Z)^T) K,  Z = (b lambda) U^T
// (the chunk form of reversing the rank-1 updates, algorithmic/fast_weight/fast_weight_cuda.cu:244-560).
// Here the matrices are kept untransposed, S[e][m] and G[e][m], warp w owning the rows e in [16w, 16w+16):
// an accumulator fragment in this layout is directly the right operand of a product that contracts over m
// (gY S0^T, U G1^T, (b lambda) S0^T), each warp producing its own 16 columns of dQ and dK.  The one product
// that contracts over e (Kt G1) reads a bf16 copy of G that the warps leave in shared memory once per chunk.
namespace cb {

// Left-operand fragments A[r][k] = X[k][r] from a row-major X (rows k, r contiguous), 16 (k) x 16 (r) block
__device__ __forceinline__ void lda_trans(unsigned (&a)[4], const __nv_bfloat16* tile, int ld, int lane) {
    ldsm4t(a, tile + ((lane & 7) + 8 * (lane >> 4)) * ld + 8 * ((lane >> 3) & 1));
}
// (x0, x1) as two packed bf16 pairs hi + lo
__device__ __forceinline__ void split_bf16(float x0, float x1, unsigned& hi, unsigned& lo) {
    hi = pack_bf16(x0, x1);
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&hi);
    lo = pack_bf16(x0 - __low2float(h), x1 - __high2float(h));
}
__device__ __forceinline__ void neg4(unsigned (&d)[4], const unsigned (&a)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) d[i] = a[i] ^ 0x80008000u;
}
// one 16 x 8 tile (columns 8j..8j+7) of X Y^T for 16 x 64 row-major tiles X, Y
__device__ __forceinline__ void gram_tile(float (&acc)[4], const __nv_bfloat16* X, const __nv_bfloat16* Y, int j, int lane) {
#pragma unroll
    for (int kp = 0; kp < 2; kp++) {
        unsigned bfr[4];
        ldsm4(bfr, Y + (8 * j + (lane & 7)) * LDT + 8 * (lane >> 3) + 32 * kp);
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            unsigned a[4];
            lda_rowmajor(a, X + 16 * (2 * kp + kk), LDT, lane);
            mma_bf16(acc, a, bfr[2 * kk], bfr[2 * kk + 1]);
        }
    }
}
__device__ __forceinline__ void load_tile_f32(float* tile, const float* base, long long sL, int t0, int nt, int tid) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int idx = tid + NT * i, row = idx >> 4, part = (idx & 15) * 4;
        float* dst = tile + row * LDO + part;
        if (row < nt) cp_async16(dst, base + (long long)(t0 + row) * sL + part);
        else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

}  // namespace cb

// ------------------------------------------------------------------ forward
// One CTA per sequence, four warps; the input tiles of the next chunk are in flight (cp.async) while a chunk
// is computed.  The triangular solve is taken as the explicit inverse
// T = (I + N)^-1, N = Akk diag(b) strictly lower and therefore nilpotent:
//   T = (I - N)(I + N^2)(I + N^4)(I + N^8)
// Every warp builds Akk, Aqk and T for itself in accumulator fragments (six 16 x 16 x 16 products whose right
// operands are transposed in registers with movmatrix), so the Gram tiles, the solve and Cv never touch shared
// memory: Cv^T = V^T T^T and (V - Cv)^T = -V^T (T - I)^T are two products of the chain warp with T taken from
// its own fragments, and only Ck = T K (16 columns per warp) is exchanged through shared memory.
namespace cb {

struct SmemI {
    __nv_bfloat16 k[2][C * LDT], v[2][C * LDT], q[2][C * LDT];    // input stages
    __nv_bfloat16 ck[C * LDT];          // Ck, [t][e]
    __nv_bfloat16 ys[C * LDT];          // y, [t][m]
    float b[2][C];
};

__device__ __forceinline__ unsigned movm(unsigned x) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}
// a 16 x 16 matrix held as an accumulator fragment, as the left operand of a product
__device__ __forceinline__ void a_of(unsigned (&a)[4], const float (&x)[2][4]) {
    a[0] = pack_bf16(x[0][0], x[0][1]); a[1] = pack_bf16(x[0][2], x[0][3]);
    a[2] = pack_bf16(x[1][0], x[1][1]); a[3] = pack_bf16(x[1][2], x[1][3]);
}
// ... as the right operand B[k][n] = X[k][n]: b[2j], b[2j+1] for the column tile j
__device__ __forceinline__ void b_of(unsigned (&b)[4], const float (&x)[2][4]) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        b[2 * j] = movm(pack_bf16(x[j][0], x[j][1]));
        b[2 * j + 1] = movm(pack_bf16(x[j][2], x[j][3]));
    }
}
// ... as the right operand B[k][n] = X[n][k] (the transposed matrix), in two bf16 parts: no data movement
__device__ __forceinline__ void bt_of(unsigned (&hi)[4], unsigned (&lo)[4], const float (&x)[2][4]) {
    split_bf16(x[0][0], x[0][1], hi[0], lo[0]);   // column tile 0 (n = g): k = 2 t4, +1
    split_bf16(x[1][0], x[1][1], hi[1], lo[1]);   //                        k = 8 + 2 t4, +1
    split_bf16(x[0][2], x[0][3], hi[2], lo[2]);   // column tile 1 (n = 8 + g)
    split_bf16(x[1][2], x[1][3], hi[3], lo[3]);
}
// out += A B for 16 x 16 fragments
__device__ __forceinline__ void mm(float (&out)[2][4], const unsigned (&a)[4], const unsigned (&b)[4]) {
    mma_bf16(out[0], a, b[0], b[1]);
    mma_bf16(out[1], a, b[2], b[3]);
}

}  // namespace cb

__global__ void __launch_bounds__(cb::NT, 4) delta_fwd_chunk_bf16_inv_kernel(const DeltaFwdParams p) {
    using namespace cb;
    using bf16 = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char cb_smem[];
    SmemI& s = *reinterpret_cast<SmemI*>(cb_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const bf16* qb = reinterpret_cast<const bf16*>(p.q.p) + n * p.q.sN + h * p.q.sH;
    const bf16* kb = reinterpret_cast<const bf16*>(p.k.p) + n * p.k.sN + h * p.k.sH;
    const bf16* vb = reinterpret_cast<const bf16*>(p.v.p) + n * p.v.sN + h * p.v.sH;
    const bf16* bb = reinterpret_cast<const bf16*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    bf16* yb = reinterpret_cast<bf16*>(p.out.p) + n * p.out.sN + h * p.out.sH;
    float* vob = reinterpret_cast<float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH;
    float* uib = p.v_ins.p ? reinterpret_cast<float*>(p.v_ins.p) + n * p.v_ins.sN + h * p.v_ins.sH : nullptr;
    float* W = p.W + n * p.wN + h * p.wH;
    const int m0 = 16 * warp;

    float S[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) S[j][i] = W[(long long)(8 * j + 2 * t4 + (i & 1)) * p.wE + m0 + g + 8 * (i >> 1)];

    const int nchunks = (p.L + C - 1) / C;
    {
        const int nt = min(C, p.L);
        load_tile(s.k[0], kb, p.k.sL, 0, nt, tid);
        load_tile(s.v[0], vb, p.v.sL, 0, nt, tid);
        load_tile(s.q[0], qb, p.q.sL, 0, nt, tid);
        cp_async_commit();
        if (tid < C) s.b[0][tid] = tid < nt ? __bfloat162float(bb[(long long)tid * p.beta.sL]) : 0.f;
    }
    for (int c = 0; c < nchunks; c++) {
        const int cur = c & 1, t0 = c * C, nt = min(C, p.L - t0);
        float bnext = 0.f;
        if (c + 1 < nchunks) {
            const int t1 = t0 + C, nt1 = min(C, p.L - t1);
            load_tile(s.k[cur ^ 1], kb, p.k.sL, t1, nt1, tid);
            load_tile(s.v[cur ^ 1], vb, p.v.sL, t1, nt1, tid);
            load_tile(s.q[cur ^ 1], qb, p.q.sL, t1, nt1, tid);
            cp_async_commit();
            if (tid < nt1) bnext = __bfloat162float(bb[(long long)(t1 + tid) * p.beta.sL]);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* Ks = s.k[cur];
        const bf16* Qs = s.q[cur];
        const float* bs = s.b[cur];

        // (1) per warp: Akk, Aqk, T; the warp's 16 columns of Ck = T K
        unsigned th[4], tl[4], yh[4], yl[4], qk[4];     // right operands T^T, (T - I)^T (two parts each), Aqk^T
        {
            float akk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float aqk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kp = 0; kp < 2; kp++) {
                unsigned b0[4], b1[4];
                ldsm4(b0, Ks + (lane & 7) * LDT + 8 * (lane >> 3) + 32 * kp);
                ldsm4(b1, Ks + (8 + (lane & 7)) * LDT + 8 * (lane >> 3) + 32 * kp);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    unsigned ak[4], aq[4];
                    lda_rowmajor(ak, Ks + 16 * (2 * kp + kk), LDT, lane);
                    lda_rowmajor(aq, Qs + 16 * (2 * kp + kk), LDT, lane);
                    mma_bf16(akk[0], ak, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(akk[1], ak, b1[2 * kk], b1[2 * kk + 1]);
                    mma_bf16(aqk[0], aq, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(aqk[1], aq, b1[2 * kk], b1[2 * kk + 1]);
                }
            }
            float N1[2][4], Y[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t4 + (i & 1);
                    N1[j][i] = cc < r ? akk[j][i] * bs[cc] : 0.f;
                    aqk[j][i] = cc <= r ? aqk[j][i] : 0.f;
                    Y[j][i] = -N1[j][i];
                }
            {
                unsigned lo[4];
                bt_of(qk, lo, aqk);
            }
            unsigned a[4], bN[4], b2[4];
            float N2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N1);
            b_of(bN, N1);
            mm(N2, a, bN);                                  // N^2
            b_of(b2, N2);
            {
                float N3[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                mm(N3, a, b2);                              // N^3
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) Y[j][i] += N2[j][i] - N3[j][i];
            }
            float N4[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N2);
            mm(N4, a, b2);                                  // N^4
            unsigned b4[4];
            b_of(b4, N4);
            {
                float Z1[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, Y);
                mm(Z1, a, b4);                              // Y N^4
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) Y[j][i] += N4[j][i] + Z1[j][i];
            }
            float N8[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N4);
            mm(N8, a, b4);                                  // N^8
            {
                unsigned b8[4];
                b_of(b8, N8);
                float Z2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, Y);
                mm(Z2, a, b8);                              // Y N^8
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) Y[j][i] += N8[j][i] + Z2[j][i];
            }
            // Y = T - I (strictly lower).  Ck[:, 16w..16w+15] = T K
            float T[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) T[j][i] = Y[j][i] + ((8 * j + 2 * t4 + (i & 1)) == (g + 8 * (i >> 1)) ? 1.f : 0.f);
            bt_of(th, tl, T);
            bt_of(yh, yl, Y);
            unsigned ah[4], al[4], bK[4];
            split_bf16(T[0][0], T[0][1], ah[0], al[0]); split_bf16(T[0][2], T[0][3], ah[1], al[1]);
            split_bf16(T[1][0], T[1][1], ah[2], al[2]); split_bf16(T[1][2], T[1][3], ah[3], al[3]);
            ldb_kn(bK, Ks + m0, LDT, lane);
            float ck[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            mm(ck, ah, bK);
            mm(ck, al, bK);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                *reinterpret_cast<unsigned*>(s.ck + g * LDT + m0 + 8 * j + 2 * t4) = pack_bf16(ck[j][0], ck[j][1]);
                *reinterpret_cast<unsigned*>(s.ck + (g + 8) * LDT + m0 + 8 * j + 2 * t4) = pack_bf16(ck[j][2], ck[j][3]);
            }
        }
        __syncthreads();

        {   // (2) chain
            unsigned sa[4][4];
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                sa[ks][0] = pack_bf16(S[2 * ks][0], S[2 * ks][1]);
                sa[ks][1] = pack_bf16(S[2 * ks][2], S[2 * ks][3]);
                sa[ks][2] = pack_bf16(S[2 * ks + 1][0], S[2 * ks + 1][1]);
                sa[ks][3] = pack_bf16(S[2 * ks + 1][2], S[2 * ks + 1][3]);
            }
            float P[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float Yo[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                unsigned bc[4], bq[4];
                ldb_nk(bc, s.ck + 16 * ks, LDT, lane);
                ldb_nk(bq, Qs + 16 * ks, LDT, lane);
                mm(P, sa[ks], bc);
                mm(Yo, sa[ks], bq);
            }
            float cv[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float py[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            {
                unsigned va[4];
                lda_trans(va, s.v[cur] + m0, LDT, lane);
                mm(cv, va, th);
                mm(cv, va, tl);
                mm(py, va, yh);
                mm(py, va, yl);
            }
            float u[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int m = m0 + g + 8 * (i >> 1), t = 8 * j + 2 * t4 + (i & 1);
                    u[j][i] = bs[t] * (cv[j][i] - P[j][i]);
                    if (t < nt) {
                        vob[(long long)(t0 + t) * p.v_old.sL + m] = P[j][i] - py[j][i];
                        if (uib) uib[(long long)(t0 + t) * p.v_ins.sL + m] = u[j][i];
                    }
                }
            unsigned ua[4], ul[4];
            split_bf16(u[0][0], u[0][1], ua[0], ul[0]); split_bf16(u[0][2], u[0][3], ua[1], ul[1]);
            split_bf16(u[1][0], u[1][1], ua[2], ul[2]); split_bf16(u[1][2], u[1][3], ua[3], ul[3]);
            mm(Yo, ua, qk);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                unsigned bk[4];
                ldb_kn(bk, Ks + 16 * jp, LDT, lane);
                mma_bf16(S[2 * jp], ua, bk[0], bk[1]);
                mma_bf16(S[2 * jp + 1], ua, bk[2], bk[3]);
                mma_bf16(S[2 * jp], ul, bk[0], bk[1]);
                mma_bf16(S[2 * jp + 1], ul, bk[2], bk[3]);
            }
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    s.ys[(8 * j + 2 * t4 + (i & 1)) * LDT + m0 + g + 8 * (i >> 1)] = __float2bfloat16_rn(Yo[j][i]);
        }
        __syncthreads();

        {   // (3) y: 16-byte row pieces
            const int row = tid >> 3, part = (tid & 7) * 8;
            if (row < nt)
                *reinterpret_cast<uint4*>(yb + (long long)(t0 + row) * p.out.sL + part) =
                    *reinterpret_cast<const uint4*>(s.ys + row * LDT + part);
            if (tid < C && c + 1 < nchunks) s.b[cur ^ 1][tid] = bnext;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) W[(long long)(8 * j + 2 * t4 + (i & 1)) * p.wE + m0 + g + 8 * (i >> 1)] = S[j][i];
}


// ------------------------------------------------------------------ forward, state-independent part one chunk ahead
// Everything of a chunk that does not involve the state -- the Gram tiles, the inverse T, Aqk^T and Ck = T K -- is
// the same for the four chain warps and does not wait for the previous chunk.  In the kernel above every warp
// computes it for itself, between two CTA-wide barriers, on the critical path of the chunk.  Here a fifth warp
// prepares it one chunk ahead (and issues all the copies): it leaves the five right-operand fragment sets
// (T^T and (T - I)^T as two bf16 parts each, Aqk^T) in shared memory in fragment order, one 16-byte piece per lane,
// and Ck as a row-major tile.  The chain warps wait for that package, run the state-dependent products and hand the
// buffers back.  Two named barriers per package buffer: FULL (the preparing warp arrives, the chain warps wait) and
// EMPTY (the chain warps arrive after their last read of the package and of the input stage, the preparing warp
// waits before it refills either); in this order neither side can arrive twice on a barrier before the other has
// waited on it.  Input stages are a ring of three, packages a ring of two.
namespace cb {

constexpr int NTP = 160;                // four chain warps and the preparing warp

struct SmemP {
    __nv_bfloat16 k[3][C * LDT], v[3][C * LDT], q[3][C * LDT];    // input stages
    uint4 frag[2][5][32];               // per package: T^T hi, lo; (T - I)^T hi, lo; Aqk^T -- in fragment order
    __nv_bfloat16 ck[2][C * LDT];       // per package: Ck, [t][e]
    __nv_bfloat16 ys[2][C * LDT];       // y, [t][m]
    float b[3][C];
};

enum { BAR_FULL = 1, BAR_EMPTY = 3, BAR_CHAIN = 5 };     // FULL, EMPTY: + (chunk & 1)

__device__ __forceinline__ void nbar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void nbar_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }

}  // namespace cb

__global__ void __launch_bounds__(cb::NTP, 4) delta_fwd_chunk_bf16_pipe_kernel(const DeltaFwdParams p) {
    using namespace cb;
    using bf16 = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char cb_smem[];
    SmemP& s = *reinterpret_cast<SmemP*>(cb_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const int nchunks = (p.L + C - 1) / C;

    if (warp == 4) {
        // ------------------------------------------------------------ the preparing warp
        const bf16* qb = reinterpret_cast<const bf16*>(p.q.p) + n * p.q.sN + h * p.q.sH;
        const bf16* kb = reinterpret_cast<const bf16*>(p.k.p) + n * p.k.sN + h * p.k.sH;
        const bf16* vb = reinterpret_cast<const bf16*>(p.v.p) + n * p.v.sN + h * p.v.sH;
        const bf16* bb = reinterpret_cast<const bf16*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
        auto stage_in = [&](int c) {        // all copies of chunk c by this warp: 3 tiles x 16 rows x 8 pieces
            const int st = c % 3, t0 = c * C, nt = min(C, p.L - t0);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int idx = lane + 32 * i, row = idx >> 3, part = (idx & 7) * 8;
                bf16* dk = s.k[st] + row * LDT + part;
                bf16* dv = s.v[st] + row * LDT + part;
                bf16* dq = s.q[st] + row * LDT + part;
                if (row < nt) {
                    cp_async16(dk, kb + (long long)(t0 + row) * p.k.sL + part);
                    cp_async16(dv, vb + (long long)(t0 + row) * p.v.sL + part);
                    cp_async16(dq, qb + (long long)(t0 + row) * p.q.sL + part);
                } else {
                    *reinterpret_cast<uint4*>(dk) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(dv) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(dq) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            cp_async_commit();
            if (lane < C) s.b[st][lane] = lane < nt ? __bfloat162float(bb[(long long)(t0 + lane) * p.beta.sL]) : 0.f;
        };
        stage_in(0);
        for (int c = 0; c < nchunks; c++) {
            const int pk = c & 1;
            if (c >= 2) nbar_sync(BAR_EMPTY + pk, NTP);      // the chain warps are through chunk c - 2
            if (c + 1 < nchunks) { stage_in(c + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
            __syncwarp();
            const bf16* Ks = s.k[c % 3];
            const bf16* Qs = s.q[c % 3];
            const float* bs = s.b[c % 3];
            float akk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float aqk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kp = 0; kp < 2; kp++) {
                unsigned b0[4], b1[4];
                ldsm4(b0, Ks + (lane & 7) * LDT + 8 * (lane >> 3) + 32 * kp);
                ldsm4(b1, Ks + (8 + (lane & 7)) * LDT + 8 * (lane >> 3) + 32 * kp);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    unsigned ak[4], aq[4];
                    lda_rowmajor(ak, Ks + 16 * (2 * kp + kk), LDT, lane);
                    lda_rowmajor(aq, Qs + 16 * (2 * kp + kk), LDT, lane);
                    mma_bf16(akk[0], ak, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(akk[1], ak, b1[2 * kk], b1[2 * kk + 1]);
                    mma_bf16(aqk[0], aq, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(aqk[1], aq, b1[2 * kk], b1[2 * kk + 1]);
                }
            }
            float N1[2][4], Y[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t4 + (i & 1);
                    N1[j][i] = cc < r ? akk[j][i] * bs[cc] : 0.f;
                    aqk[j][i] = cc <= r ? aqk[j][i] : 0.f;
                    Y[j][i] = -N1[j][i];
                }
            unsigned th[4], tl[4], yh[4], yl[4], qk[4];
            {
                unsigned lo[4];
                bt_of(qk, lo, aqk);
            }
            unsigned a[4], bN[4], b2[4];
            float N2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N1);
            b_of(bN, N1);
            mm(N2, a, bN);                                  // N^2
            b_of(b2, N2);
            {
                float N3[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                mm(N3, a, b2);                              // N^3
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) Y[j][i] += N2[j][i] - N3[j][i];
            }
            float N4[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N2);
            mm(N4, a, b2);                                  // N^4
            unsigned b4[4];
            b_of(b4, N4);
            {
                float Z1[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, Y);
                mm(Z1, a, b4);                              // Y N^4
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) Y[j][i] += N4[j][i] + Z1[j][i];
            }
            float N8[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N4);
            mm(N8, a, b4);                                  // N^8
            {
                unsigned b8[4];
                b_of(b8, N8);
                float Z2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, Y);
                mm(Z2, a, b8);                              // Y N^8
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) Y[j][i] += N8[j][i] + Z2[j][i];
            }
            float T[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) T[j][i] = Y[j][i] + ((8 * j + 2 * t4 + (i & 1)) == (g + 8 * (i >> 1)) ? 1.f : 0.f);
            bt_of(th, tl, T);
            bt_of(yh, yl, Y);
            s.frag[pk][0][lane] = make_uint4(th[0], th[1], th[2], th[3]);
            s.frag[pk][1][lane] = make_uint4(tl[0], tl[1], tl[2], tl[3]);
            s.frag[pk][2][lane] = make_uint4(yh[0], yh[1], yh[2], yh[3]);
            s.frag[pk][3][lane] = make_uint4(yl[0], yl[1], yl[2], yl[3]);
            s.frag[pk][4][lane] = make_uint4(qk[0], qk[1], qk[2], qk[3]);
            unsigned ah[4], al[4];
            split_bf16(T[0][0], T[0][1], ah[0], al[0]); split_bf16(T[0][2], T[0][3], ah[1], al[1]);
            split_bf16(T[1][0], T[1][1], ah[2], al[2]); split_bf16(T[1][2], T[1][3], ah[3], al[3]);
#pragma unroll
            for (int w = 0; w < 4; w++) {                   // Ck = T K, sixteen columns at a time
                unsigned bK[4];
                ldb_kn(bK, Ks + 16 * w, LDT, lane);
                float ck[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                mm(ck, ah, bK);
                mm(ck, al, bK);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    *reinterpret_cast<unsigned*>(s.ck[pk] + g * LDT + 16 * w + 8 * j + 2 * t4) = pack_bf16(ck[j][0], ck[j][1]);
                    *reinterpret_cast<unsigned*>(s.ck[pk] + (g + 8) * LDT + 16 * w + 8 * j + 2 * t4) = pack_bf16(ck[j][2], ck[j][3]);
                }
            }
            nbar_arrive(BAR_FULL + pk, NTP);
        }
        return;
    }

    // ---------------------------------------------------------------- the chain warps
    bf16* yb = reinterpret_cast<bf16*>(p.out.p) + n * p.out.sN + h * p.out.sH;
    float* vob = reinterpret_cast<float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH;
    float* uib = p.v_ins.p ? reinterpret_cast<float*>(p.v_ins.p) + n * p.v_ins.sN + h * p.v_ins.sH : nullptr;
    float* W = p.W + n * p.wN + h * p.wH;
    const int m0 = 16 * warp;
    float S[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) S[j][i] = W[(long long)(8 * j + 2 * t4 + (i & 1)) * p.wE + m0 + g + 8 * (i >> 1)];

    for (int c = 0; c < nchunks; c++) {
        const int pk = c & 1, st = c % 3, t0 = c * C, nt = min(C, p.L - t0);
        nbar_sync(BAR_FULL + pk, NTP);
        const bf16* Ks = s.k[st];
        const bf16* Qs = s.q[st];
        const float* bs = s.b[st];
        const bf16* cks = s.ck[pk];
        unsigned th[4], tl[4], yh[4], yl[4], qk[4];
        {
            const uint4 f0 = s.frag[pk][0][lane], f1 = s.frag[pk][1][lane], f2 = s.frag[pk][2][lane],
                        f3 = s.frag[pk][3][lane], f4 = s.frag[pk][4][lane];
            th[0] = f0.x; th[1] = f0.y; th[2] = f0.z; th[3] = f0.w;
            tl[0] = f1.x; tl[1] = f1.y; tl[2] = f1.z; tl[3] = f1.w;
            yh[0] = f2.x; yh[1] = f2.y; yh[2] = f2.z; yh[3] = f2.w;
            yl[0] = f3.x; yl[1] = f3.y; yl[2] = f3.z; yl[3] = f3.w;
            qk[0] = f4.x; qk[1] = f4.y; qk[2] = f4.z; qk[3] = f4.w;
        }
        unsigned sa[4][4];
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            sa[ks][0] = pack_bf16(S[2 * ks][0], S[2 * ks][1]);
            sa[ks][1] = pack_bf16(S[2 * ks][2], S[2 * ks][3]);
            sa[ks][2] = pack_bf16(S[2 * ks + 1][0], S[2 * ks + 1][1]);
            sa[ks][3] = pack_bf16(S[2 * ks + 1][2], S[2 * ks + 1][3]);
        }
        float P[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float Yo[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            unsigned bc[4], bq[4];
            ldb_nk(bc, cks + 16 * ks, LDT, lane);
            ldb_nk(bq, Qs + 16 * ks, LDT, lane);
            mm(P, sa[ks], bc);
            mm(Yo, sa[ks], bq);
        }
        float cv[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float py[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            unsigned va[4];
            lda_trans(va, s.v[st] + m0, LDT, lane);
            mm(cv, va, th);
            mm(cv, va, tl);
            mm(py, va, yh);
            mm(py, va, yl);
        }
        float u[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int m = m0 + g + 8 * (i >> 1), t = 8 * j + 2 * t4 + (i & 1);
                u[j][i] = bs[t] * (cv[j][i] - P[j][i]);
                if (t < nt) {
                    vob[(long long)(t0 + t) * p.v_old.sL + m] = P[j][i] - py[j][i];
                    if (uib) uib[(long long)(t0 + t) * p.v_ins.sL + m] = u[j][i];
                }
            }
        unsigned ua[4], ul[4];
        split_bf16(u[0][0], u[0][1], ua[0], ul[0]); split_bf16(u[0][2], u[0][3], ua[1], ul[1]);
        split_bf16(u[1][0], u[1][1], ua[2], ul[2]); split_bf16(u[1][2], u[1][3], ua[3], ul[3]);
        mm(Yo, ua, qk);
#pragma unroll
        for (int jp = 0; jp < 4; jp++) {
            unsigned bk[4];
            ldb_kn(bk, Ks + 16 * jp, LDT, lane);
            mma_bf16(S[2 * jp], ua, bk[0], bk[1]);
            mma_bf16(S[2 * jp + 1], ua, bk[2], bk[3]);
            mma_bf16(S[2 * jp], ul, bk[0], bk[1]);
            mma_bf16(S[2 * jp + 1], ul, bk[2], bk[3]);
        }
        if (c + 2 < nchunks) nbar_arrive(BAR_EMPTY + pk, NTP);      // last read of the package and of the stage is behind us
        bf16* ys = s.ys[pk];
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                ys[(8 * j + 2 * t4 + (i & 1)) * LDT + m0 + g + 8 * (i >> 1)] = __float2bfloat16_rn(Yo[j][i]);
        nbar_sync(BAR_CHAIN, NT);
        {   // y: 16-byte row pieces
            const int row = tid >> 3, part = (tid & 7) * 8;
            if (row < nt)
                *reinterpret_cast<uint4*>(yb + (long long)(t0 + row) * p.out.sL + part) =
                    *reinterpret_cast<const uint4*>(ys + row * LDT + part);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) W[(long long)(8 * j + 2 * t4 + (i & 1)) * p.wE + m0 + g + 8 * (i >> 1)] = S[j][i];
}


// ------------------------------------------------------------------ backward kernel
// The backward substitution is the transposed system: with
// T' = (I + diag(b) Akk)^-1 (built per warp in registers like T of the forward), [Lt | Kt] = T'^T [Aqk^T gY | K],
// so Lt^T = gY^T (Aqk T') is one product of the chain warp and Kt = T'^T K is exchanged through shared memory,
// 16 columns per warp.  The Gram tiles, Aqk^T gY and Lt never touch shared memory.
namespace cb {
struct SmemB2 {
    __nv_bfloat16 k[2][C * LDT], q[2][C * LDT], v[2][C * LDT], gy[2][C * LDT];   // input stages
    float vo[2][C * LDO];               // v_old stages, [t][m]; the current one becomes w = v - v_old in place
    __nv_bfloat16 uh[C * LDT], ul[C * LDT];   // U = b w as two bf16 parts, [t][m]
    __nv_bfloat16 bl[C * LDT];          // b lambda = dv, [t][m]
    __nv_bfloat16 kt[C * LDT];          // Kt, [t][e]
    __nv_bfloat16 gs[D * LDT];          // G1 rounded to bf16, [e][m]
    __nv_bfloat16 bm[C * LDQ];          // B = lower(gY U^T), [t][i]
    alignas(16) __nv_bfloat16 dqdk[2 * C * LDT];   // dQ, dK, [t][e]
    float dbp[4][C];                    // per-warp partial sums of dbeta
    float b[2][C];
};
}  // namespace cb

__global__ void __launch_bounds__(cb::NT, 3) delta_bwd_chunk_bf16_inv_kernel(const DeltaBwdParams p) {
    using namespace cb;
    using bf16 = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char cb_smem[];
    SmemB2& s = *reinterpret_cast<SmemB2*>(cb_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const bf16* qb = reinterpret_cast<const bf16*>(p.q.p) + n * p.q.sN + h * p.q.sH;
    const bf16* kb = reinterpret_cast<const bf16*>(p.k.p) + n * p.k.sN + h * p.k.sH;
    const bf16* vb = reinterpret_cast<const bf16*>(p.v.p) + n * p.v.sN + h * p.v.sH;
    const bf16* bb = reinterpret_cast<const bf16*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    const bf16* gyb = reinterpret_cast<const bf16*>(p.gy.p) + n * p.gy.sN + h * p.gy.sH;
    const float* vob = reinterpret_cast<const float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH;
    bf16* gqb = reinterpret_cast<bf16*>(p.gq.p) + n * p.gq.sN + h * p.gq.sH;
    bf16* gkb = reinterpret_cast<bf16*>(p.gk.p) + n * p.gk.sN + h * p.gk.sH;
    bf16* gvb = reinterpret_cast<bf16*>(p.gv.p) + n * p.gv.sN + h * p.gv.sH;
    bf16* gbb = reinterpret_cast<bf16*>(p.gb.p) + n * p.gb.sN + h * p.gb.sH;
    float* W = p.W + n * p.wN + h * p.wH;
    const int e0 = 16 * warp;           // rows of S and G this warp owns; also its rows m of lambda^T

    // S, G rows e0+g, e0+g+8; tile j holds the value indices 8j + 2 t4, +1
    float S[8][4], G[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
            const float2 x = *reinterpret_cast<const float2*>(W + (long long)(e0 + g + 8 * hr) * p.wE + 8 * j + 2 * t4);
            S[j][2 * hr] = x.x; S[j][2 * hr + 1] = x.y;
            G[j][2 * hr] = 0.f; G[j][2 * hr + 1] = 0.f;
        }

    const int nchunks = (p.L + C - 1) / C;
    auto issue = [&](int c, int st) {
        const int t0 = c * C, nt = min(C, p.L - t0);
        load_tile(s.k[st], kb, p.k.sL, t0, nt, tid);
        load_tile(s.q[st], qb, p.q.sL, t0, nt, tid);
        load_tile(s.v[st], vb, p.v.sL, t0, nt, tid);
        load_tile(s.gy[st], gyb, p.gy.sL, t0, nt, tid);
        load_tile_f32(s.vo[st], vob, p.v_old.sL, t0, nt, tid);
        cp_async_commit();
    };
    issue(nchunks - 1, 0);
    {
        const int t0 = (nchunks - 1) * C;
        if (tid < C) s.b[0][tid] = t0 + tid < p.L ? __bfloat162float(bb[(long long)(t0 + tid) * p.beta.sL]) : 0.f;
    }
    for (int it = 0; it < nchunks; it++) {
        const int c = nchunks - 1 - it, cur = it & 1, t0 = c * C, nt = min(C, p.L - t0);
        float bnext = 0.f;
        if (c > 0) {
            issue(c - 1, cur ^ 1);
            if (tid < C) bnext = __bfloat162float(bb[(long long)(t0 - C + tid) * p.beta.sL]);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* Ks = s.k[cur];
        const bf16* Qs = s.q[cur];
        const bf16* Ys = s.gy[cur];
        float* Ws = s.vo[cur];
        const float* bs = s.b[cur];
        bf16* dqs = s.dqdk;
        bf16* dks = s.dqdk + C * LDT;

        unsigned bX[4];     // right operand X = Aqk T' of the product that gives Lt^T
        {   // (1) per warp: Akk, Aqk, T' = (I + diag(b) Akk)^-1, X, the warp's 16 columns of Kt = T'^T K; w and U; bf16 copy of G1
            float akk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float aqk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kp = 0; kp < 2; kp++) {
                unsigned b0[4], b1[4];
                ldsm4(b0, Ks + (lane & 7) * LDT + 8 * (lane >> 3) + 32 * kp);
                ldsm4(b1, Ks + (8 + (lane & 7)) * LDT + 8 * (lane >> 3) + 32 * kp);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    unsigned ak[4], aq[4];
                    lda_rowmajor(ak, Ks + 16 * (2 * kp + kk), LDT, lane);
                    lda_rowmajor(aq, Qs + 16 * (2 * kp + kk), LDT, lane);
                    mma_bf16(akk[0], ak, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(akk[1], ak, b1[2 * kk], b1[2 * kk + 1]);
                    mma_bf16(aqk[0], aq, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(aqk[1], aq, b1[2 * kk], b1[2 * kk + 1]);
                }
            }
            float N1[2][4], Y[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t4 + (i & 1);
                    N1[j][i] = cc < r ? akk[j][i] * bs[r] : 0.f;
                    aqk[j][i] = cc <= r ? aqk[j][i] : 0.f;
                    Y[j][i] = -N1[j][i];
                }
            unsigned a[4], bN[4], b2[4], b4[4];
            float N2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N1);
            b_of(bN, N1);
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
            {
                float N8[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, N4);
                mm(N8, a, b4);
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
            {   // X = Aqk T' = Aqk + Aqk (T' - I)
                unsigned by[4];
                b_of(by, Y);
                a_of(a, aqk);
                mm(aqk, a, by);
                b_of(bX, aqk);
            }
            {   // Kt[:, e0..e0+15] = T'^T K: the left operand is the transposed fragment, in two bf16 parts
                float T[2][4];
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) T[j][i] = Y[j][i] + ((8 * j + 2 * t4 + (i & 1)) == (g + 8 * (i >> 1)) ? 1.f : 0.f);
                unsigned ah[4], al[4], th2[4], tl2[4], bK[4];
                split_bf16(T[0][0], T[0][1], ah[0], al[0]); split_bf16(T[0][2], T[0][3], ah[1], al[1]);
                split_bf16(T[1][0], T[1][1], ah[2], al[2]); split_bf16(T[1][2], T[1][3], ah[3], al[3]);
                th2[0] = movm(ah[0]); th2[1] = movm(ah[2]); th2[2] = movm(ah[1]); th2[3] = movm(ah[3]);
                tl2[0] = movm(al[0]); tl2[1] = movm(al[2]); tl2[2] = movm(al[1]); tl2[3] = movm(al[3]);
                ldb_kn(bK, Ks + e0, LDT, lane);
                float kt[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                mm(kt, th2, bK);
                mm(kt, tl2, bK);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    *reinterpret_cast<unsigned*>(s.kt + g * LDT + e0 + 8 * j + 2 * t4) = pack_bf16(kt[j][0], kt[j][1]);
                    *reinterpret_cast<unsigned*>(s.kt + (g + 8) * LDT + e0 + 8 * j + 2 * t4) = pack_bf16(kt[j][2], kt[j][3]);
                }
            }
            const int row = tid >> 3, part = (tid & 7) * 8;
            const uint4 vraw = *reinterpret_cast<const uint4*>(s.v[cur] + row * LDT + part);
            const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vraw);
            float* wp = Ws + row * LDO + part;
            const float4 o0 = *reinterpret_cast<const float4*>(wp), o1 = *reinterpret_cast<const float4*>(wp + 4);
            const float vo8[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
            float w8[8];
            unsigned hi[4], lo[4];
            const float br = bs[row];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                w8[2 * i] = __low2float(v2[i]) - vo8[2 * i];
                w8[2 * i + 1] = __high2float(v2[i]) - vo8[2 * i + 1];
                const float u0 = br * w8[2 * i], u1 = br * w8[2 * i + 1];
                hi[i] = pack_bf16(u0, u1);
                const __nv_bfloat162 hh = *reinterpret_cast<const __nv_bfloat162*>(&hi[i]);
                lo[i] = pack_bf16(u0 - __low2float(hh), u1 - __high2float(hh));
            }
            *reinterpret_cast<float4*>(wp) = make_float4(w8[0], w8[1], w8[2], w8[3]);
            *reinterpret_cast<float4*>(wp + 4) = make_float4(w8[4], w8[5], w8[6], w8[7]);
            *reinterpret_cast<uint4*>(s.uh + row * LDT + part) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(s.ul + row * LDT + part) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
#pragma unroll
            for (int jj = 0; jj < 8; jj++) {
                *reinterpret_cast<unsigned*>(s.gs + (e0 + g) * LDT + 8 * jj + 2 * t4) = pack_bf16(G[jj][0], G[jj][1]);
                *reinterpret_cast<unsigned*>(s.gs + (e0 + g + 8) * LDT + 8 * jj + 2 * t4) = pack_bf16(G[jj][2], G[jj][3]);
            }
        }
        __syncthreads();

        if (warp < 2) {   // B = lower(gY U^T), one column tile on each of warps 0 and 1 (read after the next barrier)
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const int col = 8 * warp + 2 * t4;
            gram_tile(acc, Ys, s.uh, warp, lane);
            *reinterpret_cast<unsigned*>(s.bm + g * LDQ + col) =
                pack_bf16(col <= g ? acc[0] : 0.f, col + 1 <= g ? acc[1] : 0.f);
            *reinterpret_cast<unsigned*>(s.bm + (g + 8) * LDQ + col) =
                pack_bf16(col <= g + 8 ? acc[2] : 0.f, col + 1 <= g + 8 ? acc[3] : 0.f);
        }

        {   // (4a) lambda^T rows m in [e0, e0+16): Lt^T + G1^T Kt^T with Lt^T = gY^T X; dv = b lambda; partial sums of dbeta
            float lm[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            {
                unsigned ya[4];
                lda_trans(ya, Ys + e0, LDT, lane);
                mm(lm, ya, bX);
            }
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                unsigned a[4], bk[4];
                lda_trans(a, s.gs + 16 * ks * LDT + e0, LDT, lane);
                ldb_nk(bk, s.kt + 16 * ks, LDT, lane);
                mma_bf16(lm[0], a, bk[0], bk[1]);
                mma_bf16(lm[1], a, bk[2], bk[3]);
            }
            float db[2][2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                db[j][0] = 0.f; db[j][1] = 0.f;
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    const int m = e0 + g + 8 * hr, t = 8 * j + 2 * t4;
                    const float l0 = lm[j][2 * hr], l1 = lm[j][2 * hr + 1];
                    db[j][0] = fmaf(l0, Ws[t * LDO + m], db[j][0]);
                    db[j][1] = fmaf(l1, Ws[(t + 1) * LDO + m], db[j][1]);
                    s.bl[t * LDT + m] = __float2bfloat16_rn(bs[t] * l0);
                    s.bl[(t + 1) * LDT + m] = __float2bfloat16_rn(bs[t + 1] * l1);
                }
            }
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int par = 0; par < 2; par++) {
                    float x = db[j][par];
                    x += __shfl_xor_sync(0xffffffffu, x, 4);
                    x += __shfl_xor_sync(0xffffffffu, x, 8);
                    x += __shfl_xor_sync(0xffffffffu, x, 16);
                    if (g == 0) s.dbp[warp][8 * j + 2 * t4 + par] = x;
                }
        }
        __syncthreads();

        {   // (4b) rewind S, the warp's 16 columns of dQ and dK, then G
            unsigned ka[4], kan[4];
            lda_trans(ka, Ks + e0, LDT, lane);          // K^T rows e0.., contraction over the 16 steps
            neg4(kan, ka);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                unsigned bh[4], bl2[4];
                ldb_kn(bh, s.uh + 16 * jp, LDT, lane);
                ldb_kn(bl2, s.ul + 16 * jp, LDT, lane);
                mma_bf16(S[2 * jp], kan, bh[0], bh[1]);
                mma_bf16(S[2 * jp + 1], kan, bh[2], bh[3]);
                mma_bf16(S[2 * jp], kan, bl2[0], bl2[1]);
                mma_bf16(S[2 * jp + 1], kan, bl2[2], bl2[3]);
            }
            float dq[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float dk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float Z[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float ZT[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                // right operands from the accumulators, each as two bf16 parts: contraction over m in
                // [16ks, 16ks+16), columns e0+g (first index 0) and e0+8+g (first index 1)
                unsigned sh[2][2], sl[2][2], gh[2][2], gl[2][2];
#pragma unroll
                for (int hr = 0; hr < 2; hr++)
#pragma unroll
                    for (int kk = 0; kk < 2; kk++) {
                        split_bf16(S[2 * ks + kk][2 * hr], S[2 * ks + kk][2 * hr + 1], sh[hr][kk], sl[hr][kk]);
                        split_bf16(G[2 * ks + kk][2 * hr], G[2 * ks + kk][2 * hr + 1], gh[hr][kk], gl[hr][kk]);
                    }
                unsigned ya[4], ua[4], ula[4], la[4], lan[4], bu[4], bb2[4];
                lda_rowmajor(ya, Ys + 16 * ks, LDT, lane);
                lda_rowmajor(ua, s.uh + 16 * ks, LDT, lane);
                lda_rowmajor(ula, s.ul + 16 * ks, LDT, lane);
                lda_rowmajor(la, s.bl + 16 * ks, LDT, lane);
                neg4(lan, la);
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    mma_bf16(dq[hr], ya, sh[hr][0], sh[hr][1]);
                    mma_bf16(dq[hr], ya, sl[hr][0], sl[hr][1]);
                    mma_bf16(dk[hr], ua, gh[hr][0], gh[hr][1]);
                    mma_bf16(dk[hr], ua, gl[hr][0], gl[hr][1]);
                    mma_bf16(dk[hr], ula, gh[hr][0], gh[hr][1]);
                    mma_bf16(dk[hr], lan, sh[hr][0], sh[hr][1]);
                    mma_bf16(dk[hr], lan, sl[hr][0], sl[hr][1]);
                }
                ldb_nk(bu, s.uh + 16 * ks, LDT, lane);
                ldb_nk(bb2, s.bl + 16 * ks, LDT, lane);
                mma_bf16(Z[0], la, bu[0], bu[1]);
                mma_bf16(Z[1], la, bu[2], bu[3]);
                mma_bf16(ZT[0], ua, bb2[0], bb2[1]);
                mma_bf16(ZT[1], ua, bb2[2], bb2[3]);
            }
            unsigned bK[4], bQ[4], ba[4], bta[4], za[4], qa[4];
            ldb_kn(bK, Ks + e0, LDT, lane);
            ldb_kn(bQ, Qs + e0, LDT, lane);
            lda_rowmajor(ba, s.bm, LDQ, lane);
            lda_trans(bta, s.bm, LDQ, lane);
            mma_bf16(dq[0], ba, bK[0], bK[1]);
            mma_bf16(dq[1], ba, bK[2], bK[3]);
            mma_bf16(dk[0], bta, bQ[0], bQ[1]);
            mma_bf16(dk[1], bta, bQ[2], bQ[3]);
            {
                float z[2][4];
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t4 + (i & 1);
                        z[j][i] = -((cc < r ? Z[j][i] : 0.f) + (cc > r ? ZT[j][i] : 0.f));
                    }
                za[0] = pack_bf16(z[0][0], z[0][1]); za[1] = pack_bf16(z[0][2], z[0][3]);
                za[2] = pack_bf16(z[1][0], z[1][1]); za[3] = pack_bf16(z[1][2], z[1][3]);
            }
            mma_bf16(dk[0], za, bK[0], bK[1]);
            mma_bf16(dk[1], za, bK[2], bK[3]);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int col = e0 + 8 * j + 2 * t4;
                *reinterpret_cast<unsigned*>(dqs + g * LDT + col) = pack_bf16(dq[j][0], dq[j][1]);
                *reinterpret_cast<unsigned*>(dqs + (g + 8) * LDT + col) = pack_bf16(dq[j][2], dq[j][3]);
                *reinterpret_cast<unsigned*>(dks + g * LDT + col) = pack_bf16(dk[j][0], dk[j][1]);
                *reinterpret_cast<unsigned*>(dks + (g + 8) * LDT + col) = pack_bf16(dk[j][2], dk[j][3]);
            }
            // G0 = G1 + Q^T gY - K^T (b lambda)
            lda_trans(qa, Qs + e0, LDT, lane);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                unsigned bg[4], bd[4];
                ldb_kn(bg, Ys + 16 * jp, LDT, lane);
                ldb_kn(bd, s.bl + 16 * jp, LDT, lane);
                mma_bf16(G[2 * jp], qa, bg[0], bg[1]);
                mma_bf16(G[2 * jp + 1], qa, bg[2], bg[3]);
                mma_bf16(G[2 * jp], kan, bd[0], bd[1]);
                mma_bf16(G[2 * jp + 1], kan, bd[2], bd[3]);
            }
        }
        __syncthreads();

        {   // (5) stores: 16-byte row pieces of dQ, dK, dv; dbeta
            const int row = tid >> 3, part = (tid & 7) * 8;
            if (row < nt) {
                *reinterpret_cast<uint4*>(gqb + (long long)(t0 + row) * p.gq.sL + part) =
                    *reinterpret_cast<const uint4*>(dqs + row * LDT + part);
                *reinterpret_cast<uint4*>(gkb + (long long)(t0 + row) * p.gk.sL + part) =
                    *reinterpret_cast<const uint4*>(dks + row * LDT + part);
                *reinterpret_cast<uint4*>(gvb + (long long)(t0 + row) * p.gv.sL + part) =
                    *reinterpret_cast<const uint4*>(s.bl + row * LDT + part);
            }
            if (tid < nt)
                gbb[(long long)(t0 + tid) * p.gb.sL] =
                    __float2bfloat16_rn(s.dbp[0][tid] + s.dbp[1][tid] + s.dbp[2][tid] + s.dbp[3][tid]);
            if (tid < C && c > 0) s.b[cur ^ 1][tid] = bnext;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int hr = 0; hr < 2; hr++)
            *reinterpret_cast<float2*>(W + (long long)(e0 + g + 8 * hr) * p.wE + 8 * j + 2 * t4) =
                make_float2(S[j][2 * hr], S[j][2 * hr + 1]);
}

// ------------------------------------------------------------------ backward, state-independent part one chunk ahead
// The same split as in the forward: a fifth warp issues the copies and prepares, one chunk ahead, everything of a
// chunk that involves neither S nor G -- the Gram tiles, T' = (I + diag(b) Akk)^-1, X = Aqk T' (a fragment set),
// Kt = T'^T K, w = v - v_old and U = b w in two bf16 parts, B = lower(gY U^T) -- and the four chain warps keep the
// products with S and G.  FULL / EMPTY named barriers per package buffer as in the forward; input stages and
// packages are rings of two (the preparing warp refills a stage as soon as the chain warps have left it, a whole
// chunk of chain work before it is needed).
namespace cb {

struct SmemBP {
    __nv_bfloat16 k[2][C * LDT], q[2][C * LDT], v[2][C * LDT], gy[2][C * LDT];   // input stages
    float vo[2][C * LDO];               // v_old stages, [t][m]; becomes w = v - v_old in place
    float b[2][C];
    uint4 fx[2][32];                    // per package: X = Aqk T' as right-operand fragments
    __nv_bfloat16 kt[2][C * LDT];       // per package: Kt, [t][e]
    __nv_bfloat16 uh[2][C * LDT], ul[2][C * LDT];   // per package: U = b w as two bf16 parts, [t][m]
    __nv_bfloat16 bm[2][C * LDQ];       // per package: B = lower(gY U^T), [t][i]
    __nv_bfloat16 bl[2][C * LDT];       // b lambda = dv, [t][m]; two chunk parities (the stores of a chunk may still read it
                                        // while the next chunk writes)
    __nv_bfloat16 gs[D * LDT];          // G1 rounded to bf16, [e][m]
    alignas(16) __nv_bfloat16 dqdk[2 * C * LDT];   // dQ, dK, [t][e]
    float dbp[2][4][C];                 // per-warp partial sums of dbeta, two chunk parities
};

}  // namespace cb

__global__ void __launch_bounds__(cb::NTP, 3) delta_bwd_chunk_bf16_pipe_kernel(const DeltaBwdParams p) {
    using namespace cb;
    using bf16 = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char cb_smem[];
    SmemBP& s = *reinterpret_cast<SmemBP*>(cb_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const int nchunks = (p.L + C - 1) / C;

    if (warp == 4) {
        // ------------------------------------------------------------ the preparing warp
        const bf16* qb = reinterpret_cast<const bf16*>(p.q.p) + n * p.q.sN + h * p.q.sH;
        const bf16* kb = reinterpret_cast<const bf16*>(p.k.p) + n * p.k.sN + h * p.k.sH;
        const bf16* vb = reinterpret_cast<const bf16*>(p.v.p) + n * p.v.sN + h * p.v.sH;
        const bf16* bb = reinterpret_cast<const bf16*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
        const bf16* gyb = reinterpret_cast<const bf16*>(p.gy.p) + n * p.gy.sN + h * p.gy.sH;
        const float* vob = reinterpret_cast<const float*>(p.v_old.p) + n * p.v_old.sN + h * p.v_old.sH;
        auto stage_in = [&](int it) {       // all copies of the chunk processed it-th, by this warp
            const int st = it & 1, c = nchunks - 1 - it, t0 = c * C, nt = min(C, p.L - t0);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int idx = lane + 32 * i, row = idx >> 3, part = (idx & 7) * 8;
                const int o = row * LDT + part;
                if (row < nt) {
                    cp_async16(s.k[st] + o, kb + (long long)(t0 + row) * p.k.sL + part);
                    cp_async16(s.q[st] + o, qb + (long long)(t0 + row) * p.q.sL + part);
                    cp_async16(s.v[st] + o, vb + (long long)(t0 + row) * p.v.sL + part);
                    cp_async16(s.gy[st] + o, gyb + (long long)(t0 + row) * p.gy.sL + part);
                } else {
                    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(s.k[st] + o) = z;
                    *reinterpret_cast<uint4*>(s.q[st] + o) = z;
                    *reinterpret_cast<uint4*>(s.v[st] + o) = z;
                    *reinterpret_cast<uint4*>(s.gy[st] + o) = z;
                }
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int idx = lane + 32 * i, row = idx >> 4, part = (idx & 15) * 4;
                float* dst = s.vo[st] + row * LDO + part;
                if (row < nt) cp_async16(dst, vob + (long long)(t0 + row) * p.v_old.sL + part);
                else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            cp_async_commit();
            if (lane < C) s.b[st][lane] = lane < nt ? __bfloat162float(bb[(long long)(t0 + lane) * p.beta.sL]) : 0.f;
        };
        stage_in(0);
        for (int it = 0; it < nchunks; it++) {
            const int pk = it & 1;
            cp_async_wait<0>();
            __syncwarp();
            const bf16* Ks = s.k[pk];
            const bf16* Qs = s.q[pk];
            const bf16* Ys = s.gy[pk];
            float* Ws = s.vo[pk];
            const float* bs = s.b[pk];
            unsigned bX[4];
            float Y[2][4];
            {
            float akk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float aqk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kp = 0; kp < 2; kp++) {
                unsigned b0[4], b1[4];
                ldsm4(b0, Ks + (lane & 7) * LDT + 8 * (lane >> 3) + 32 * kp);
                ldsm4(b1, Ks + (8 + (lane & 7)) * LDT + 8 * (lane >> 3) + 32 * kp);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    unsigned ak[4], aq[4];
                    lda_rowmajor(ak, Ks + 16 * (2 * kp + kk), LDT, lane);
                    lda_rowmajor(aq, Qs + 16 * (2 * kp + kk), LDT, lane);
                    mma_bf16(akk[0], ak, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(akk[1], ak, b1[2 * kk], b1[2 * kk + 1]);
                    mma_bf16(aqk[0], aq, b0[2 * kk], b0[2 * kk + 1]);
                    mma_bf16(aqk[1], aq, b1[2 * kk], b1[2 * kk + 1]);
                }
            }
            float N1[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t4 + (i & 1);
                    N1[j][i] = cc < r ? akk[j][i] * bs[r] : 0.f;
                    aqk[j][i] = cc <= r ? aqk[j][i] : 0.f;
                    Y[j][i] = -N1[j][i];
                }
            unsigned a[4], bN[4], b2[4], b4[4];
            float N2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            a_of(a, N1);
            b_of(bN, N1);
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
            {
                float N8[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                a_of(a, N4);
                mm(N8, a, b4);
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
            {   // X = Aqk T' = Aqk + Aqk (T' - I)
                unsigned by[4];
                b_of(by, Y);
                a_of(a, aqk);
                mm(aqk, a, by);
                b_of(bX, aqk);
            }
            }
            s.fx[pk][lane] = make_uint4(bX[0], bX[1], bX[2], bX[3]);
            {   // Kt = T'^T K, sixteen columns at a time: the left operand is the transposed fragment, in two bf16 parts
                float T[2][4];
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) T[j][i] = Y[j][i] + ((8 * j + 2 * t4 + (i & 1)) == (g + 8 * (i >> 1)) ? 1.f : 0.f);
                unsigned ah[4], al[4], th2[4], tl2[4];
                split_bf16(T[0][0], T[0][1], ah[0], al[0]); split_bf16(T[0][2], T[0][3], ah[1], al[1]);
                split_bf16(T[1][0], T[1][1], ah[2], al[2]); split_bf16(T[1][2], T[1][3], ah[3], al[3]);
                th2[0] = movm(ah[0]); th2[1] = movm(ah[2]); th2[2] = movm(ah[1]); th2[3] = movm(ah[3]);
                tl2[0] = movm(al[0]); tl2[1] = movm(al[2]); tl2[2] = movm(al[1]); tl2[3] = movm(al[3]);
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    unsigned bK[4];
                    ldb_kn(bK, Ks + 16 * w, LDT, lane);
                    float kt[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    mm(kt, th2, bK);
                    mm(kt, tl2, bK);
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        *reinterpret_cast<unsigned*>(s.kt[pk] + g * LDT + 16 * w + 8 * j + 2 * t4) = pack_bf16(kt[j][0], kt[j][1]);
                        *reinterpret_cast<unsigned*>(s.kt[pk] + (g + 8) * LDT + 16 * w + 8 * j + 2 * t4) = pack_bf16(kt[j][2], kt[j][3]);
                    }
                }
            }
            // w = v - v_old in place, U = b w in two bf16 parts: sixteen rows of eight 8-element pieces
#pragma unroll
            for (int ii = 0; ii < 4; ii++) {
                const int idx = lane + 32 * ii, row = idx >> 3, part = (idx & 7) * 8;
                const uint4 vraw = *reinterpret_cast<const uint4*>(s.v[pk] + row * LDT + part);
                const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vraw);
                float* wp = Ws + row * LDO + part;
                const float4 o0 = *reinterpret_cast<const float4*>(wp), o1 = *reinterpret_cast<const float4*>(wp + 4);
                const float vo8[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
                float w8[8];
                unsigned hi[4], lo[4];
                const float br = bs[row];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    w8[2 * i] = __low2float(v2[i]) - vo8[2 * i];
                    w8[2 * i + 1] = __high2float(v2[i]) - vo8[2 * i + 1];
                    const float u0 = br * w8[2 * i], u1 = br * w8[2 * i + 1];
                    hi[i] = pack_bf16(u0, u1);
                    const __nv_bfloat162 hh = *reinterpret_cast<const __nv_bfloat162*>(&hi[i]);
                    lo[i] = pack_bf16(u0 - __low2float(hh), u1 - __high2float(hh));
                }
                *reinterpret_cast<float4*>(wp) = make_float4(w8[0], w8[1], w8[2], w8[3]);
                *reinterpret_cast<float4*>(wp + 4) = make_float4(w8[4], w8[5], w8[6], w8[7]);
                *reinterpret_cast<uint4*>(s.uh[pk] + row * LDT + part) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(s.ul[pk] + row * LDT + part) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
            __syncwarp();
#pragma unroll
            for (int w = 0; w < 2; w++) {   // B = lower(gY U^T), two column tiles
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const int col = 8 * w + 2 * t4;
                gram_tile(acc, Ys, s.uh[pk], w, lane);
                *reinterpret_cast<unsigned*>(s.bm[pk] + g * LDQ + col) =
                    pack_bf16(col <= g ? acc[0] : 0.f, col + 1 <= g ? acc[1] : 0.f);
                *reinterpret_cast<unsigned*>(s.bm[pk] + (g + 8) * LDQ + col) =
                    pack_bf16(col <= g + 8 ? acc[2] : 0.f, col + 1 <= g + 8 ? acc[3] : 0.f);
            }
            nbar_arrive(BAR_FULL + pk, NTP);
            if (it + 1 < nchunks) {
                if (it >= 1) nbar_sync(BAR_EMPTY + (pk ^ 1), NTP);     // the chain warps have left the other stage and package
                stage_in(it + 1);
            }
        }
        return;
    }

    // ---------------------------------------------------------------- the chain warps
    bf16* gqb = reinterpret_cast<bf16*>(p.gq.p) + n * p.gq.sN + h * p.gq.sH;
    bf16* gkb = reinterpret_cast<bf16*>(p.gk.p) + n * p.gk.sN + h * p.gk.sH;
    bf16* gvb = reinterpret_cast<bf16*>(p.gv.p) + n * p.gv.sN + h * p.gv.sH;
    bf16* gbb = reinterpret_cast<bf16*>(p.gb.p) + n * p.gb.sN + h * p.gb.sH;
    float* W = p.W + n * p.wN + h * p.wH;
    const int e0 = 16 * warp;
    float S[8][4], G[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
            const float2 x = *reinterpret_cast<const float2*>(W + (long long)(e0 + g + 8 * hr) * p.wE + 8 * j + 2 * t4);
            S[j][2 * hr] = x.x; S[j][2 * hr + 1] = x.y;
            G[j][2 * hr] = 0.f; G[j][2 * hr + 1] = 0.f;
        }
    // the bf16 copy of G that the products contracting over e read: written by every warp for its rows at the end of a
    // chunk (behind the barrier that chunk has anyway), zero before the first
#pragma unroll
    for (int jj = 0; jj < 8; jj++) {
        *reinterpret_cast<unsigned*>(s.gs + (e0 + g) * LDT + 8 * jj + 2 * t4) = 0u;
        *reinterpret_cast<unsigned*>(s.gs + (e0 + g + 8) * LDT + 8 * jj + 2 * t4) = 0u;
    }
    nbar_sync(BAR_CHAIN, NT);
    for (int it = 0; it < nchunks; it++) {
        const int c = nchunks - 1 - it, pk = it & 1, t0 = c * C, nt = min(C, p.L - t0);
        nbar_sync(BAR_FULL + pk, NTP);
        const bf16* Ks = s.k[pk];
        const bf16* Qs = s.q[pk];
        const bf16* Ys = s.gy[pk];
        const float* Ws = s.vo[pk];
        const float* bs = s.b[pk];
        const bf16* s_kt = s.kt[pk];
        const bf16* s_uh = s.uh[pk];
        const bf16* s_ul = s.ul[pk];
        const bf16* s_bm = s.bm[pk];
        bf16* dqs = s.dqdk;
        bf16* dks = s.dqdk + C * LDT;
        bf16* s_bl = s.bl[pk];
        float (*s_dbp)[C] = s.dbp[pk];
        unsigned bX[4];
        {
            const uint4 f = s.fx[pk][lane];
            bX[0] = f.x; bX[1] = f.y; bX[2] = f.z; bX[3] = f.w;
        }

        {   // (4a) lambda^T rows m in [e0, e0+16): Lt^T + G1^T Kt^T with Lt^T = gY^T X; dv = b lambda; partial sums of dbeta
            float lm[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            {
                unsigned ya[4];
                lda_trans(ya, Ys + e0, LDT, lane);
                mm(lm, ya, bX);
            }
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                unsigned a[4], bk[4];
                lda_trans(a, s.gs + 16 * ks * LDT + e0, LDT, lane);
                ldb_nk(bk, s_kt + 16 * ks, LDT, lane);
                mma_bf16(lm[0], a, bk[0], bk[1]);
                mma_bf16(lm[1], a, bk[2], bk[3]);
            }
            float db[2][2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                db[j][0] = 0.f; db[j][1] = 0.f;
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    const int m = e0 + g + 8 * hr, t = 8 * j + 2 * t4;
                    const float l0 = lm[j][2 * hr], l1 = lm[j][2 * hr + 1];
                    db[j][0] = fmaf(l0, Ws[t * LDO + m], db[j][0]);
                    db[j][1] = fmaf(l1, Ws[(t + 1) * LDO + m], db[j][1]);
                    s_bl[t * LDT + m] = __float2bfloat16_rn(bs[t] * l0);
                    s_bl[(t + 1) * LDT + m] = __float2bfloat16_rn(bs[t + 1] * l1);
                }
            }
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int par = 0; par < 2; par++) {
                    float x = db[j][par];
                    x += __shfl_xor_sync(0xffffffffu, x, 4);
                    x += __shfl_xor_sync(0xffffffffu, x, 8);
                    x += __shfl_xor_sync(0xffffffffu, x, 16);
                    if (g == 0) s_dbp[warp][8 * j + 2 * t4 + par] = x;
                }
        }
        nbar_sync(BAR_CHAIN, NT);

        {   // (4b) rewind S, the warp's 16 columns of dQ and dK, then G
            unsigned ka[4], kan[4];
            lda_trans(ka, Ks + e0, LDT, lane);          // K^T rows e0.., contraction over the 16 steps
            neg4(kan, ka);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                unsigned bh[4], bl2[4];
                ldb_kn(bh, s_uh + 16 * jp, LDT, lane);
                ldb_kn(bl2, s_ul + 16 * jp, LDT, lane);
                mma_bf16(S[2 * jp], kan, bh[0], bh[1]);
                mma_bf16(S[2 * jp + 1], kan, bh[2], bh[3]);
                mma_bf16(S[2 * jp], kan, bl2[0], bl2[1]);
                mma_bf16(S[2 * jp + 1], kan, bl2[2], bl2[3]);
            }
            float dq[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float dk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float Z[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float ZT[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                // right operands from the accumulators, each as two bf16 parts: contraction over m in
                // [16ks, 16ks+16), columns e0+g (first index 0) and e0+8+g (first index 1)
                unsigned sh[2][2], sl[2][2], gh[2][2], gl[2][2];
#pragma unroll
                for (int hr = 0; hr < 2; hr++)
#pragma unroll
                    for (int kk = 0; kk < 2; kk++) {
                        split_bf16(S[2 * ks + kk][2 * hr], S[2 * ks + kk][2 * hr + 1], sh[hr][kk], sl[hr][kk]);
                        split_bf16(G[2 * ks + kk][2 * hr], G[2 * ks + kk][2 * hr + 1], gh[hr][kk], gl[hr][kk]);
                    }
                unsigned ya[4], ua[4], ula[4], la[4], lan[4];
                lda_rowmajor(ya, Ys + 16 * ks, LDT, lane);
                lda_rowmajor(ua, s_uh + 16 * ks, LDT, lane);
                lda_rowmajor(ula, s_ul + 16 * ks, LDT, lane);
                lda_rowmajor(la, s_bl + 16 * ks, LDT, lane);
                neg4(lan, la);
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    mma_bf16(dq[hr], ya, sh[hr][0], sh[hr][1]);
                    mma_bf16(dq[hr], ya, sl[hr][0], sl[hr][1]);
                    mma_bf16(dk[hr], ua, gh[hr][0], gh[hr][1]);
                    mma_bf16(dk[hr], ua, gl[hr][0], gl[hr][1]);
                    mma_bf16(dk[hr], ula, gh[hr][0], gh[hr][1]);
                    mma_bf16(dk[hr], lan, sh[hr][0], sh[hr][1]);
                    mma_bf16(dk[hr], lan, sl[hr][0], sl[hr][1]);
                }
            }
            // Z = (b lambda) U^T and its transpose in a loop of their own: fewer accumulators live at once
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                unsigned ua[4], la[4], bu[4], bb2[4];
                lda_rowmajor(ua, s_uh + 16 * ks, LDT, lane);
                lda_rowmajor(la, s_bl + 16 * ks, LDT, lane);
                ldb_nk(bu, s_uh + 16 * ks, LDT, lane);
                ldb_nk(bb2, s_bl + 16 * ks, LDT, lane);
                mma_bf16(Z[0], la, bu[0], bu[1]);
                mma_bf16(Z[1], la, bu[2], bu[3]);
                mma_bf16(ZT[0], ua, bb2[0], bb2[1]);
                mma_bf16(ZT[1], ua, bb2[2], bb2[3]);
            }
            unsigned bK[4], bQ[4], ba[4], bta[4], za[4], qa[4];
            ldb_kn(bK, Ks + e0, LDT, lane);
            ldb_kn(bQ, Qs + e0, LDT, lane);
            lda_rowmajor(ba, s_bm, LDQ, lane);
            lda_trans(bta, s_bm, LDQ, lane);
            mma_bf16(dq[0], ba, bK[0], bK[1]);
            mma_bf16(dq[1], ba, bK[2], bK[3]);
            mma_bf16(dk[0], bta, bQ[0], bQ[1]);
            mma_bf16(dk[1], bta, bQ[2], bQ[3]);
            {
                float z[2][4];
#pragma unroll
                for (int j = 0; j < 2; j++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t4 + (i & 1);
                        z[j][i] = -((cc < r ? Z[j][i] : 0.f) + (cc > r ? ZT[j][i] : 0.f));
                    }
                za[0] = pack_bf16(z[0][0], z[0][1]); za[1] = pack_bf16(z[0][2], z[0][3]);
                za[2] = pack_bf16(z[1][0], z[1][1]); za[3] = pack_bf16(z[1][2], z[1][3]);
            }
            mma_bf16(dk[0], za, bK[0], bK[1]);
            mma_bf16(dk[1], za, bK[2], bK[3]);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int col = e0 + 8 * j + 2 * t4;
                *reinterpret_cast<unsigned*>(dqs + g * LDT + col) = pack_bf16(dq[j][0], dq[j][1]);
                *reinterpret_cast<unsigned*>(dqs + (g + 8) * LDT + col) = pack_bf16(dq[j][2], dq[j][3]);
                *reinterpret_cast<unsigned*>(dks + g * LDT + col) = pack_bf16(dk[j][0], dk[j][1]);
                *reinterpret_cast<unsigned*>(dks + (g + 8) * LDT + col) = pack_bf16(dk[j][2], dk[j][3]);
            }
            // G0 = G1 + Q^T gY - K^T (b lambda)
            lda_trans(qa, Qs + e0, LDT, lane);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                unsigned bg[4], bd[4];
                ldb_kn(bg, Ys + 16 * jp, LDT, lane);
                ldb_kn(bd, s_bl + 16 * jp, LDT, lane);
                mma_bf16(G[2 * jp], qa, bg[0], bg[1]);
                mma_bf16(G[2 * jp + 1], qa, bg[2], bg[3]);
                mma_bf16(G[2 * jp], kan, bd[0], bd[1]);
                mma_bf16(G[2 * jp + 1], kan, bd[2], bd[3]);
            }
            // the bf16 copy of G0 for the next chunk's products (nobody reads the tile between here and the barrier below)
#pragma unroll
            for (int jj = 0; jj < 8; jj++) {
                *reinterpret_cast<unsigned*>(s.gs + (e0 + g) * LDT + 8 * jj + 2 * t4) = pack_bf16(G[jj][0], G[jj][1]);
                *reinterpret_cast<unsigned*>(s.gs + (e0 + g + 8) * LDT + 8 * jj + 2 * t4) = pack_bf16(G[jj][2], G[jj][3]);
            }
        }
        if (it + 2 < nchunks) nbar_arrive(BAR_EMPTY + pk, NTP);      // last read of the stage and of the package is behind us
        nbar_sync(BAR_CHAIN, NT);

        {   // (5) stores: 16-byte row pieces of dQ, dK, dv; dbeta
            const int row = tid >> 3, part = (tid & 7) * 8;
            if (row < nt) {
                *reinterpret_cast<uint4*>(gqb + (long long)(t0 + row) * p.gq.sL + part) =
                    *reinterpret_cast<const uint4*>(dqs + row * LDT + part);
                *reinterpret_cast<uint4*>(gkb + (long long)(t0 + row) * p.gk.sL + part) =
                    *reinterpret_cast<const uint4*>(dks + row * LDT + part);
                *reinterpret_cast<uint4*>(gvb + (long long)(t0 + row) * p.gv.sL + part) =
                    *reinterpret_cast<const uint4*>(s_bl + row * LDT + part);
            }
            if (tid < nt)
                gbb[(long long)(t0 + tid) * p.gb.sL] =
                    __float2bfloat16_rn(s_dbp[0][tid] + s_dbp[1][tid] + s_dbp[2][tid] + s_dbp[3][tid]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int hr = 0; hr < 2; hr++)
            *reinterpret_cast<float2*>(W + (long long)(e0 + g + 8 * hr) * p.wE + 8 * j + 2 * t4) =
                make_float2(S[j][2 * hr], S[j][2 * hr + 1]);
}

}  // namespace fwp
