// Delta rule in chunkwise (WY / UT-transform) form for head dimensions up to 16, fp32 (sm_100a).
//
// The per-step and four-step-blocked kernels walk one dependency chain per sequence, and with a
// few hundred sequences the machine is mostly idle.  Here 16 consecutive steps form a chunk whose
// work is dense 16x16 matrix algebra; only two small products per chunk stay on the chain.
// With S0 the state before the chunk, K, Q (16 x E), V (16 x M), b = beta (16):
//
//   Akk = strict_lower(K K^T), Aqk = lower(Q K^T)                     (state independent)
//   u = b (V - K S0 - Akk u)   <=>   u = Ut - Wt S0, where [Ut | Wt] solves the unit lower
//       triangular system  x_t = b_t (rhs_t - sum_{i<t} Akk[t,i] x_i)  for rhs = [V | K]
//   v_old = K S0 + Akk u,   y = Q S0 + Aqk u,   S1 = S0 + K^T u
//
// Backward, with S1, G1 = dL/dS1 at the end of the chunk and the saved v_old (w = V - v_old, U = b w):
//   S0 = S1 - K^T U
//   lambda = Lt + Kt G1, where [Lt | Kt] solves  x_i = rhs_i - sum_{t>i} Akk[t,i] b_t x_t
//       for rhs = [Aqk^T gY | K];   dv = b lambda,  dbeta = rowsum(lambda w)
//   G0 = G1 + Q^T gY - K^T (b lambda)
//   dQ = gY S0^T + lower(gY U^T) K
//   dK = U G1^T - (b lambda) S0^T + lower(gY U^T)^T Q - sym_strict((b lambda) U^T) K
// (same result as reversing the rank-1 updates step by step, algorithmic/fast_weight/
// fast_weight_cuda.cu:244-560; only the fp32 summation order differs).
//
// Execution.  Three launches per direction over a caller-provided workspace (it stays in L2 at the
// usual sizes): every chunk of every sequence is prepared by its own warp, one warp per sequence
// then walks the chunks with a single product per chunk, and every chunk is finished by its own
// warp, storing straight from the accumulator fragments.  Every product is a warp-level
// 16x16x16 tensor-core contraction, mma.sync m16n8k8 TF32 with error compensation: operands are
// split x = hi + lo and hi*hi + hi*lo + lo*hi is accumulated in fp32, which keeps the result
// within a few ulp of an fp32 FMA chain.  The triangular solves stay in fp32 FMAs, one right-hand
// column per lane.  (tcgen05 needs M >= 64 rows per instruction and a CTA-wide issue; a 16-row
// chunk of one sequence does not fill it.)
#pragma once
#include "fwp_delta_params.cuh"
#include "fwp_mma.cuh"

namespace fwp {

constexpr int kCkLd = 20;                 // tile row stride in floats: rows stay 16-byte aligned, row-fragment loads hit 32 banks
constexpr int kCkTile = 16 * kCkLd;       // one 16x16 tile
constexpr int kCkWarps = 4;               // warps per CTA = chunks per super-chunk

// acc += A B for 16x16 operands given as element functors a(m, k) and b(k, n)
template <class FA, class FB>
__device__ __forceinline__ void mm16(Frag& acc, FA a, FB b, int g, int t) {
    Frag lo;
    frag_zero(lo);
#pragma unroll
    for (int ks = 0; ks < 2; ks++) {
        const int k0 = ks * 8 + t;
        const float af[4] = {a(g, k0), a(g + 8, k0), a(g, k0 + 4), a(g + 8, k0 + 4)};
        unsigned ah[4], al[4];
#pragma unroll
        for (int i = 0; i < 4; i++) tf32_split(af[i], ah[i], al[i]);
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float bf[2] = {b(k0, 8 * j + g), b(k0 + 4, 8 * j + g)};
            unsigned bh[2], bl[2];
#pragma unroll
            for (int i = 0; i < 2; i++) tf32_split(bf[i], bh[i], bl[i]);
            mma_tf32(lo.c[j], al, bh);
            mma_tf32(lo.c[j], ah, bl);
            mma_tf32(acc.c[j], ah, bh);
        }
    }
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc.c[j][i] += lo.c[j][i];
}

template <class FA>
__device__ __forceinline__ void load_a(AFr& f, FA a, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < 2; ks++) {
        const int k0 = ks * 8 + t;
        tf32_split(a(g, k0), f.h[ks][0], f.l[ks][0]);
        tf32_split(a(g + 8, k0), f.h[ks][1], f.l[ks][1]);
        tf32_split(a(g, k0 + 4), f.h[ks][2], f.l[ks][2]);
        tf32_split(a(g + 8, k0 + 4), f.h[ks][3], f.l[ks][3]);
    }
}
template <class FB>
__device__ __forceinline__ void load_b(BFr& f, FB b, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < 2; ks++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
            tf32_split(b(ks * 8 + t, 8 * j + g), f.h[ks][j][0], f.l[ks][j][0]);
            tf32_split(b(ks * 8 + t + 4, 8 * j + g), f.h[ks][j][1], f.l[ks][j][1]);
        }
}
template <class FB>
__device__ __forceinline__ void load_b_relabelled(BFr& f, FB b, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < 2; ks++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
            tf32_split(b(ks * 8 + 2 * t, 8 * j + g), f.h[ks][j][0], f.l[ks][j][0]);
            tf32_split(b(ks * 8 + 2 * t + 1, 8 * j + g), f.h[ks][j][1], f.l[ks][j][1]);
        }
}
// acc += A B
__device__ __forceinline__ void mma16(Frag& acc, const AFr& a, const BFr& b) {
    Frag lo;
    frag_zero(lo);
#pragma unroll
    for (int ks = 0; ks < 2; ks++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
            mma_tf32(lo.c[j], a.l[ks], b.h[ks][j]);
            mma_tf32(lo.c[j], a.h[ks], b.l[ks][j]);
            mma_tf32(acc.c[j], a.h[ks], b.h[ks][j]);
        }
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc.c[j][i] += lo.c[j][i];
}

// fragment <-> tile; f(r, c, x) maps the value before the store
template <class F>
__device__ __forceinline__ void frag_store(float* tile, const Frag& a, int g, int t, F f) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int c = 8 * j + 2 * t;
        *reinterpret_cast<float2*>(tile + g * kCkLd + c) = make_float2(f(g, c, a.c[j][0]), f(g, c + 1, a.c[j][1]));
        *reinterpret_cast<float2*>(tile + (g + 8) * kCkLd + c) = make_float2(f(g + 8, c, a.c[j][2]), f(g + 8, c + 1, a.c[j][3]));
    }
}
__device__ __forceinline__ void frag_store(float* tile, const Frag& a, int g, int t) {
    frag_store(tile, a, g, t, [](int, int, float x) { return x; });
}
__device__ __forceinline__ void frag_load(Frag& a, const float* tile, int g, int t) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int c = 8 * j + 2 * t;
        const float2 lo = *reinterpret_cast<const float2*>(tile + g * kCkLd + c);
        const float2 hi = *reinterpret_cast<const float2*>(tile + (g + 8) * kCkLd + c);
        a.c[j][0] = lo.x; a.c[j][1] = lo.y; a.c[j][2] = hi.x; a.c[j][3] = hi.y;
    }
}

// rows [t0, t0+nt) of one (N,H,L,width) fp32 tensor into a tile; rows past nt and columns past width become zero
struct CkSrc {
    const float* base;
    long long sL;
    int width;
    bool vec;
    __device__ __forceinline__ void init(const Row4& r, int n, int h, int w) {
        base = reinterpret_cast<const float*>(r.p) + n * r.sN + h * r.sH;
        sL = r.sL;
        width = w;
        vec = w == 16 && (reinterpret_cast<uintptr_t>(base) & 15) == 0 && (sL & 3) == 0;
    }
};
__device__ __forceinline__ void ck_load_tile(float* tile, const CkSrc& s, int t0, int nt, int lane) {
    if (s.vec) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int seg = lane + 32 * i, row = seg >> 2, part = (seg & 3) * 4;
            float* dst = tile + row * kCkLd + part;
            if (row < nt) cp_async16(dst, s.base + (long long)(t0 + row) * s.sL + part);
            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int idx = lane + 32 * i, row = idx >> 4, col = idx & 15;
            tile[row * kCkLd + col] = (row < nt && col < s.width) ? s.base[(long long)(t0 + row) * s.sL + col] : 0.f;
        }
    }
}

// rows [t0, t0+nt) of an output tensor straight from an accumulator fragment
struct CkDst {
    float* base;
    long long sL;
    int width;
    bool vec2;
    __device__ __forceinline__ void init(const Row4& r, int n, int h, int w) {
        base = reinterpret_cast<float*>(r.p) + n * r.sN + h * r.sH;
        sL = r.sL;
        width = w;
        vec2 = (w & 1) == 0 && (reinterpret_cast<uintptr_t>(base) & 7) == 0 && (sL & 1) == 0;
    }
};
__device__ __forceinline__ void ck_store_frag(const CkDst& d, const Frag& a, int t0, int nt, int g, int t) {
#pragma unroll
    for (int hrow = 0; hrow < 2; hrow++) {
        const int row = g + 8 * hrow;
        if (row >= nt) continue;
        float* p = d.base + (long long)(t0 + row) * d.sL;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int c = 8 * j + 2 * t;
            const float x0 = a.c[j][2 * hrow], x1 = a.c[j][2 * hrow + 1];
            if (d.vec2) {
                if (c < d.width) *reinterpret_cast<float2*>(p + c) = make_float2(x0, x1);
            } else {
                if (c < d.width) p[c] = x0;
                if (c + 1 < d.width) p[c + 1] = x1;
            }
        }
    }
}

// ------------------------------------------------------------------ workspace layout
// Per chunk, in floats; every piece is a 16x16 tile stored without padding.
struct CkWs {
    static constexpr int kCk = 0;         // Ck = Wt / beta (the solve before the scaling by beta), row-major [t][e]
    static constexpr int kCv = 256;       // Cv = Ut / beta, row-major [t][m]
    static constexpr int kT = 512;        // chain operator T = Wt^T K, in the B-fragment order of the scan
    static constexpr int kR = 768;        // chain offset R = Ut^T K, in accumulator-fragment order
    static constexpr int kS0 = 1024;      // S0^T, row-major [m][e], written by the scan
    static constexpr int kFwd = 1280;
    // backward
    static constexpr int kLt = 0;         // Lt, row-major [t][m]
    static constexpr int kKt = 256;       // Kt, row-major [t][e]
    static constexpr int kTg = 512;       // chain operator T = Kt^T b K, B-fragment order
    static constexpr int kRg = 768;       // chain offset R = gY^T Q - Lt^T b K, accumulator order
    static constexpr int kD = 1024;       // state decrement D = U^T K, accumulator order
    static constexpr int kS0b = 1280;     // S0^T, row-major [m][e], written by the scan
    static constexpr int kG1 = 1536;      // G1^T, row-major [m][e], written by the scan
    static constexpr int kBwd = 1792;
};

// a 16x16 tile that sits in the workspace as 256 consecutive floats
__device__ __forceinline__ void ck_load_ws_tile(float* tile, const float* src, int lane) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int seg = lane + 32 * i, row = seg >> 2, part = (seg & 3) * 4;
        cp_async16(tile + row * kCkLd + part, src + row * 16 + part);
    }
}
__device__ __forceinline__ void ck_store_ws_frag(float* dst, const Frag& a, int g, int t) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int c = 8 * j + 2 * t;
        *reinterpret_cast<float2*>(dst + g * 16 + c) = make_float2(a.c[j][0], a.c[j][1]);
        *reinterpret_cast<float2*>(dst + (g + 8) * 16 + c) = make_float2(a.c[j][2], a.c[j][3]);
    }
}

// ------------------------------------------------------------------ forward
// Three launches.  (1) one warp per chunk, all chunks of all sequences in parallel: Akk, the
// triangular solve (kept before its scaling by beta: Ut = beta Cv, Wt = beta Ck), and the chunk's transition in
// the form  S1^T = S0^T + R - S0^T T  with T = Wt^T K and R = Ut^T K (the identity part of the transition stays
// an exact fp32 add).  (2) one warp per sequence walks its chunks: one product per
// chunk, with the state kept in the accumulator fragment, which is also the A-operand fragment
// of the next product once the contraction index is relabelled (slot t <-> column 2t, slot
// t+4 <-> column 2t+1), so nothing on the chain goes through shared memory.  (3) one warp per
// chunk again: u, v_old and y from S0 (four products, see the kernel).
struct CkFwdPrep { static constexpr int kTiles = 5; static constexpr int kWarp = kTiles * kCkTile + 16; };   // K, V, Akk (-> T), Cv, Ck
struct CkFwdPost { static constexpr int kTiles = 6; static constexpr int kWarp = kTiles * kCkTile + 16; };   // Q, K, V, Cv (-> u), Ck, S0^T

__global__ void __launch_bounds__(kCkWarps * 32) delta_fwd_chunk_prep_kernel(const DeltaFwdParams p) {
    constexpr int LD = kCkLd;
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nchunks = (p.L + 15) >> 4;
    const long long cid = (long long)blockIdx.x * kCkWarps + warp;
    if (cid >= (long long)p.NH * nchunks) return;
    const int seq = (int)(cid / nchunks), c = (int)(cid - (long long)seq * nchunks);
    const int n = seq / p.H, h = seq - n * p.H, t0 = c * 16, nt = min(16, p.L - t0);
    float* base = smem + warp * CkFwdPrep::kWarp;
    float* Ks = base; float* Vs = base + kCkTile; float* AK = base + 2 * kCkTile; float* CV = base + 3 * kCkTile;
    float* CK = base + 4 * kCkTile; float* bs = base + 5 * kCkTile;
    float* ws = p.ws + cid * CkWs::kFwd;
    CkSrc sk, sv;
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    const float* bsrc = reinterpret_cast<const float*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    ck_load_tile(Ks, sk, t0, nt, lane);
    ck_load_tile(Vs, sv, t0, nt, lane);
    cp_async_commit();
    if (lane < 16) bs[lane] = lane < nt ? bsrc[(long long)(t0 + lane) * p.beta.sL] : 0.f;
    cp_async_wait<0>();
    __syncwarp();
    Frag a;
    {
        AFr ka;
        BFr kt;
        load_a(ka, [&](int m, int k) { return Ks[m * LD + k]; }, g, t);
        load_b(kt, [&](int k, int nn) { return Ks[nn * LD + k]; }, g, t);
        frag_zero(a);
        mma16(a, ka, kt);
    }
    frag_store(AK, a, g, t, [](int r, int cc, float x) { return cc < r ? x : 0.f; });
    __syncwarp();
    {   // unit lower triangular solve, one right-hand column per lane: lanes 0-15 the columns of V, 16-31 of K.
        // c_t = rhs_t - sum_{i<t} Akk[t,i] beta_i c_i ; [Cv | Ck] keeps c, and Ut = beta Cv, Wt = beta Ck.
        const int col = lane & 15;
        const float* rhs = (lane < 16 ? Vs : Ks) + col;
        float* dst = (lane < 16 ? CV : CK) + col;
        float* gdst = ws + (lane < 16 ? CkWs::kCv : CkWs::kCk) + col;
        float x[16];
#pragma unroll
        for (int tt = 0; tt < 16; tt++) {
            float acc = rhs[tt * LD];
#pragma unroll
            for (int i4 = 0; i4 * 4 < tt; i4++) {
                const float4 a4 = *reinterpret_cast<const float4*>(AK + tt * LD + 4 * i4);
                acc = fmaf(-a4.x, x[4 * i4], acc);
                if (4 * i4 + 1 < tt) acc = fmaf(-a4.y, x[4 * i4 + 1], acc);
                if (4 * i4 + 2 < tt) acc = fmaf(-a4.z, x[4 * i4 + 2], acc);
                if (4 * i4 + 3 < tt) acc = fmaf(-a4.w, x[4 * i4 + 3], acc);
            }
            x[tt] = bs[tt] * acc;
            dst[tt * LD] = acc;
            gdst[tt * 16] = acc;
        }
    }
    __syncwarp();
    BFr kb;
    load_b(kb, [&](int k, int nn) { return Ks[k * LD + nn]; }, g, t);
    AFr lhs;
    // R = Ut^T K, already in the order the scan's accumulator wants
    load_a(lhs, [&](int m, int k) { return bs[k] * CV[k * LD + m]; }, g, t);
    frag_zero(a);
    mma16(a, lhs, kb);
    *reinterpret_cast<float4*>(ws + CkWs::kR + lane * 8) = make_float4(a.c[0][0], a.c[0][1], a.c[0][2], a.c[0][3]);
    *reinterpret_cast<float4*>(ws + CkWs::kR + lane * 8 + 4) = make_float4(a.c[1][0], a.c[1][1], a.c[1][2], a.c[1][3]);
    // T = Wt^T K, re-ordered through shared memory (the Akk tile is free) into the scan's B fragments
    load_a(lhs, [&](int m, int k) { return bs[k] * CK[k * LD + m]; }, g, t);
    frag_zero(a);
    mma16(a, lhs, kb);
    frag_store(AK, a, g, t);
    __syncwarp();
    float tf[8];
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int jn = 0; jn < 2; jn++) {
            tf[(j * 2 + jn) * 2] = AK[(8 * j + 2 * t) * LD + 8 * jn + g];
            tf[(j * 2 + jn) * 2 + 1] = AK[(8 * j + 2 * t + 1) * LD + 8 * jn + g];
        }
    *reinterpret_cast<float4*>(ws + CkWs::kT + lane * 8) = make_float4(tf[0], tf[1], tf[2], tf[3]);
    *reinterpret_cast<float4*>(ws + CkWs::kT + lane * 8 + 4) = make_float4(tf[4], tf[5], tf[6], tf[7]);
}

// X <- X + R - X T for the transposed state X = S^T held as an accumulator fragment; tf / rf are one lane's
// eight floats of T (B-fragment order) and R (accumulator order)
__device__ __forceinline__ void ck_scan_step(Frag& X, const float (&tf)[8], const float (&rf)[8]) {
    unsigned ah[2][4], al[2][4];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        tf32_split(X.c[j][0], ah[j][0], al[j][0]);      // (row g,   slot t)
        tf32_split(X.c[j][2], ah[j][1], al[j][1]);      // (row g+8, slot t)
        tf32_split(X.c[j][1], ah[j][2], al[j][2]);      // (row g,   slot t+4)
        tf32_split(X.c[j][3], ah[j][3], al[j][3]);      // (row g+8, slot t+4)
    }
    Frag hi[2], lo[2];
#pragma unroll
    for (int j = 0; j < 2; j++) { frag_zero(hi[j]); frag_zero(lo[j]); }
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int jn = 0; jn < 2; jn++) {
            unsigned bh[2], bl[2];
            tf32_split(tf[(j * 2 + jn) * 2], bh[0], bl[0]);
            tf32_split(tf[(j * 2 + jn) * 2 + 1], bh[1], bl[1]);
            mma_tf32(lo[j].c[jn], al[j], bh);
            mma_tf32(lo[j].c[jn], ah[j], bl);
            mma_tf32(hi[j].c[jn], ah[j], bh);
        }
#pragma unroll
    for (int jn = 0; jn < 2; jn++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            X.c[jn][i] = (X.c[jn][i] + rf[jn * 4 + i]) - ((lo[0].c[jn][i] + lo[1].c[jn][i]) + (hi[0].c[jn][i] + hi[1].c[jn][i]));
}

__device__ __forceinline__ void ck_load8(float (&d)[8], const float* src) {
    const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
    d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w; d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
}

// The scan reads each chunk's operators exactly once; they are fetched kCkScanDepth chunks ahead with
// cp.async into a ring in shared memory (every lane copies and later reads only its own 32 bytes per
// tile, so waiting for the copy group is the only synchronisation).
constexpr int kCkScanDepth = 8;

template <int NTILES>
__device__ __forceinline__ void ck_scan_fetch(float* ring, int slot, const float* chunk, const int (&offs)[NTILES], int lane, bool valid) {
    if (valid) {
#pragma unroll
        for (int i = 0; i < NTILES; i++) {
            float* d = ring + (slot * NTILES + i) * 256 + lane * 8;
            const float* src = chunk + offs[i] + lane * 8;
            cp_async16(d, src);
            cp_async16(d + 4, src + 4);
        }
    }
    cp_async_commit();      // also when nothing was issued: the group count per iteration stays fixed
}

__global__ void __launch_bounds__(32) delta_fwd_chunk_scan_kernel(const DeltaFwdParams p) {
    extern __shared__ __align__(16) float ring[];       // [kCkScanDepth][2][256]
    const int lane = threadIdx.x, g = lane >> 2, t = lane & 3;
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const int nchunks = (p.L + 15) >> 4;
    float* W = p.W + n * p.wN + h * p.wH;
    float* ws = p.ws + (long long)seq * nchunks * CkWs::kFwd;
    const int offs[2] = {CkWs::kT, CkWs::kR};
    for (int c = 0; c < kCkScanDepth - 1; c++) ck_scan_fetch<2>(ring, c, ws + (long long)c * CkWs::kFwd, offs, lane, c < nchunks);
    Frag X;
    ck_load_state_t(X, W, p.wE, p.E, p.M, g, t);
    for (int c = 0; c < nchunks; c++) {
        const int cn = c + kCkScanDepth - 1;
        ck_scan_fetch<2>(ring, cn % kCkScanDepth, ws + (long long)cn * CkWs::kFwd, offs, lane, cn < nchunks);
        cp_async_wait<kCkScanDepth - 1>();
        float tf[8], rf[8];
        const float* slot = ring + (c % kCkScanDepth) * 512 + lane * 8;
        ck_load8(tf, slot);
        ck_load8(rf, slot + 256);
        ck_store_ws_frag(ws + (long long)c * CkWs::kFwd + CkWs::kS0, X, g, t);
        ck_scan_step(X, tf, rf);
    }
    ck_store_state_t(X, W, p.wE, p.E, p.M, g, t);
}

// With c = [Cv | Ck] from the solve and P = Ck S0:  u = beta (Cv - P),  v_old = V - Cv + P  (the identity
// K S0 + Akk u = V - u / beta, taken before the scaling by beta so that nothing is divided), and
// y = Q S0 + lower(Q K^T) u.  Four products; Q and S0 are split once and used twice.
__global__ void __launch_bounds__(kCkWarps * 32) delta_fwd_chunk_post_kernel(const DeltaFwdParams p) {
    constexpr int LD = kCkLd;
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nchunks = (p.L + 15) >> 4;
    const long long cid = (long long)blockIdx.x * kCkWarps + warp;
    if (cid >= (long long)p.NH * nchunks) return;
    const int seq = (int)(cid / nchunks), c = (int)(cid - (long long)seq * nchunks);
    const int n = seq / p.H, h = seq - n * p.H, t0 = c * 16, nt = min(16, p.L - t0);
    float* base = smem + warp * CkFwdPost::kWarp;
    float* Qs = base; float* Ks = base + kCkTile; float* Vs = base + 2 * kCkTile; float* CV = base + 3 * kCkTile;
    float* CK = base + 4 * kCkTile; float* XT = base + 5 * kCkTile; float* bs = base + 6 * kCkTile;
    const float* ws = p.ws + cid * CkWs::kFwd;
    CkSrc sq, sk, sv;
    sq.init(p.q, n, h, p.E);
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    const float* bsrc = reinterpret_cast<const float*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    CkDst dy, dvo, dvi;
    dy.init(p.out, n, h, p.M);
    dvo.init(p.v_old, n, h, p.M);
    dvi.init(p.v_ins, n, h, p.M);
    ck_load_tile(Qs, sq, t0, nt, lane);
    ck_load_tile(Ks, sk, t0, nt, lane);
    ck_load_tile(Vs, sv, t0, nt, lane);
    ck_load_ws_tile(CV, ws + CkWs::kCv, lane);
    ck_load_ws_tile(CK, ws + CkWs::kCk, lane);
    ck_load_ws_tile(XT, ws + CkWs::kS0, lane);
    cp_async_commit();
    if (lane < 16) bs[lane] = lane < nt ? bsrc[(long long)(t0 + lane) * p.beta.sL] : 0.f;
    cp_async_wait<0>();
    __syncwarp();
    BFr s0;
    load_b(s0, [&](int k, int nn) { return XT[nn * LD + k]; }, g, t);       // S0[e][m] from the transposed tile
    Frag pf;
    {
        AFr ck;
        load_a(ck, [&](int m, int k) { return CK[m * LD + k]; }, g, t);
        frag_zero(pf);
        mma16(pf, ck, s0);
    }
    Frag u, vo;
    frag_load(u, CV, g, t);
    frag_load(vo, Vs, g, t);
    const float b0 = bs[g], b1 = bs[g + 8];
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float d = u.c[j][i] - pf.c[j][i];
            vo.c[j][i] -= d;
            u.c[j][i] = (i < 2 ? b0 : b1) * d;
        }
    __syncwarp();       // every lane has read Cv before u replaces it
    frag_store(CV, u, g, t);
    ck_store_frag(dvo, vo, t0, nt, g, t);
    if (p.v_ins.p) ck_store_frag(dvi, u, t0, nt, g, t);
    AFr qa;
    load_a(qa, [&](int m, int k) { return Qs[m * LD + k]; }, g, t);
    Frag aqk;
    {
        BFr kt;
        load_b(kt, [&](int k, int nn) { return Ks[nn * LD + k]; }, g, t);
        frag_zero(aqk);
        mma16(aqk, qa, kt);
    }
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t + (i & 1);
            if (cc > r) aqk.c[j][i] = 0.f;
        }
    Frag y;
    frag_zero(y);
    mma16(y, qa, s0);
    __syncwarp();       // u is visible
    {
        AFr am;
        BFr ub;
        a_from_acc(am, aqk);
        load_b_relabelled(ub, [&](int k, int nn) { return CV[k * LD + nn]; }, g, t);
        mma16(y, am, ub);
    }
    ck_store_frag(dy, y, t0, nt, g, t);
}

// ------------------------------------------------------------------ backward
// Same three launches.  (1) per chunk: w = V - v_old, Akk, Aqk, the transposed triangular solve for
// [Lt | Kt], and the chunk's transitions  S0^T = S1^T - D  with D = U^T K, and
// G0^T = G1^T + R - G1^T T  with T = Kt^T b K, R = gY^T Q - Lt^T b K.  (2) per sequence, newest chunk
// first: publish G1 and S0 of every chunk; one product per chunk on the chain.  (3) per chunk:
// lambda = Lt + Kt G1 and the four gradients.
struct CkBwdPrep { static constexpr int kTiles = 8; static constexpr int kWarp = kTiles * kCkTile + 16; };    // Q, K, w, gY, Aqk (-> T staging), Akk^T b, Lt (first v_old), Kt
struct CkBwdPost { static constexpr int kTiles = 10; static constexpr int kWarp = kTiles * kCkTile + 16; };   // Q, K, w, gY, Lt (-> lambda), Kt, S0^T, G1^T, lower(gY U^T), sym (first v_old)

__global__ void __launch_bounds__(kCkWarps * 32) delta_bwd_chunk_prep_kernel(const DeltaBwdParams p) {
    constexpr int LD = kCkLd;
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nchunks = (p.L + 15) >> 4;
    const long long cid = (long long)blockIdx.x * kCkWarps + warp;
    if (cid >= (long long)p.NH * nchunks) return;
    const int seq = (int)(cid / nchunks), c = (int)(cid - (long long)seq * nchunks);
    const int n = seq / p.H, h = seq - n * p.H, t0 = c * 16, nt = min(16, p.L - t0);
    float* base = smem + warp * CkBwdPrep::kWarp;
    float* Qs = base; float* Ks = base + kCkTile; float* Ws = base + 2 * kCkTile; float* Gs = base + 3 * kCkTile;
    float* AQ = base + 4 * kCkTile; float* AT = base + 5 * kCkTile; float* LT = base + 6 * kCkTile; float* KT = base + 7 * kCkTile;
    float* bs = base + 8 * kCkTile;
    float* ws = p.ws + cid * CkWs::kBwd;
    CkSrc sq, sk, sv, so, sg;
    sq.init(p.q, n, h, p.E);
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    so.init(p.v_old, n, h, p.M);
    sg.init(p.gy, n, h, p.M);
    const float* bsrc = reinterpret_cast<const float*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    ck_load_tile(Qs, sq, t0, nt, lane);
    ck_load_tile(Ks, sk, t0, nt, lane);
    ck_load_tile(Ws, sv, t0, nt, lane);
    ck_load_tile(LT, so, t0, nt, lane);
    ck_load_tile(Gs, sg, t0, nt, lane);
    cp_async_commit();
    if (lane < 16) bs[lane] = lane < nt ? bsrc[(long long)(t0 + lane) * p.beta.sL] : 0.f;
    cp_async_wait<0>();
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int idx = lane + 32 * i, o = (idx >> 4) * LD + (idx & 15);
        Ws[o] -= LT[o];
    }
    auto kT = [&](int k, int nn) { return Ks[nn * LD + k]; };
    Frag a;
    frag_zero(a);
    mm16(a, [&](int m, int k) { return Ks[m * LD + k]; }, kT, g, t);
    // transposed and scaled: AT[i][tt] = Akk[tt][i] * beta[tt] for tt > i, else 0
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t + (i & 1);
            AT[cc * LD + r] = cc < r ? a.c[j][i] * bs[r] : 0.f;
        }
    frag_zero(a);
    mm16(a, [&](int m, int k) { return Qs[m * LD + k]; }, kT, g, t);
    frag_store(AQ, a, g, t, [](int r, int cc, float x) { return cc <= r ? x : 0.f; });
    __syncwarp();       // w is complete (v_old no longer needed), Aqk and the scaled Akk^T are visible
    frag_zero(a);
    mm16(a, [&](int m, int k) { return AQ[k * LD + m]; }, [&](int k, int nn) { return Gs[k * LD + nn]; }, g, t);
    frag_store(LT, a, g, t);
    __syncwarp();
    {   // unit upper triangular solve, one right-hand column per lane: lanes 0-15 the columns of Aqk^T gY, 16-31 of K
        const int col = lane & 15;
        const float* rhs = (lane < 16 ? LT : Ks) + col;
        float* dst = (lane < 16 ? LT : KT) + col;
        float* gdst = ws + (lane < 16 ? CkWs::kLt : CkWs::kKt) + col;
        float x[16];
#pragma unroll
        for (int i = 15; i >= 0; i--) {
            float acc = rhs[i * LD];
#pragma unroll
            for (int i4 = 3; i4 * 4 + 3 > i; i4--) {
                const float4 a4 = *reinterpret_cast<const float4*>(AT + i * LD + 4 * i4);
                if (4 * i4 + 3 > i) acc = fmaf(-a4.w, x[4 * i4 + 3], acc);
                if (4 * i4 + 2 > i) acc = fmaf(-a4.z, x[4 * i4 + 2], acc);
                if (4 * i4 + 1 > i) acc = fmaf(-a4.y, x[4 * i4 + 1], acc);
                if (4 * i4 > i) acc = fmaf(-a4.x, x[4 * i4], acc);
            }
            x[i] = acc;
            dst[i * LD] = acc;
            gdst[i * 16] = acc;
        }
    }
    __syncwarp();
    auto kB = [&](int k, int nn) { return Ks[k * LD + nn]; };
    auto bkB = [&](int k, int nn) { return bs[k] * Ks[k * LD + nn]; };
    // D = U^T K
    frag_zero(a);
    mm16(a, [&](int m, int k) { return bs[k] * Ws[k * LD + m]; }, kB, g, t);
    *reinterpret_cast<float4*>(ws + CkWs::kD + lane * 8) = make_float4(a.c[0][0], a.c[0][1], a.c[0][2], a.c[0][3]);
    *reinterpret_cast<float4*>(ws + CkWs::kD + lane * 8 + 4) = make_float4(a.c[1][0], a.c[1][1], a.c[1][2], a.c[1][3]);
    // R = gY^T Q - Lt^T b K
    frag_zero(a);
    mm16(a, [&](int m, int k) { return Gs[k * LD + m]; }, [&](int k, int nn) { return Qs[k * LD + nn]; }, g, t);
    mm16(a, [&](int m, int k) { return -LT[k * LD + m]; }, bkB, g, t);
    *reinterpret_cast<float4*>(ws + CkWs::kRg + lane * 8) = make_float4(a.c[0][0], a.c[0][1], a.c[0][2], a.c[0][3]);
    *reinterpret_cast<float4*>(ws + CkWs::kRg + lane * 8 + 4) = make_float4(a.c[1][0], a.c[1][1], a.c[1][2], a.c[1][3]);
    // T = Kt^T b K, re-ordered through shared memory (the Aqk tile is free) into the scan's B fragments
    frag_zero(a);
    mm16(a, [&](int m, int k) { return KT[k * LD + m]; }, bkB, g, t);
    frag_store(AQ, a, g, t);
    __syncwarp();
    float tf[8];
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int jn = 0; jn < 2; jn++) {
            tf[(j * 2 + jn) * 2] = AQ[(8 * j + 2 * t) * LD + 8 * jn + g];
            tf[(j * 2 + jn) * 2 + 1] = AQ[(8 * j + 2 * t + 1) * LD + 8 * jn + g];
        }
    *reinterpret_cast<float4*>(ws + CkWs::kTg + lane * 8) = make_float4(tf[0], tf[1], tf[2], tf[3]);
    *reinterpret_cast<float4*>(ws + CkWs::kTg + lane * 8 + 4) = make_float4(tf[4], tf[5], tf[6], tf[7]);
}

__global__ void __launch_bounds__(32) delta_bwd_chunk_scan_kernel(const DeltaBwdParams p) {
    extern __shared__ __align__(16) float ring[];       // [kCkScanDepth][3][256]
    const int lane = threadIdx.x, g = lane >> 2, t = lane & 3;
    const int seq = blockIdx.x, n = seq / p.H, h = seq - n * p.H;
    const int nchunks = (p.L + 15) >> 4;
    float* W = p.W + n * p.wN + h * p.wH;
    float* ws = p.ws + (long long)seq * nchunks * CkWs::kBwd;
    const int offs[3] = {CkWs::kTg, CkWs::kRg, CkWs::kD};
    // i counts chunks from the end of the sequence: chunk c = nchunks - 1 - i
    for (int i = 0; i < kCkScanDepth - 1; i++)
        ck_scan_fetch<3>(ring, i, ws + (long long)(nchunks - 1 - i) * CkWs::kBwd, offs, lane, i < nchunks);
    Frag X, Y;
    ck_load_state_t(X, W, p.wE, p.E, p.M, g, t);
    frag_zero(Y);
    for (int i = 0; i < nchunks; i++) {
        const int in = i + kCkScanDepth - 1;
        ck_scan_fetch<3>(ring, in % kCkScanDepth, ws + (long long)(nchunks - 1 - in) * CkWs::kBwd, offs, lane, in < nchunks);
        cp_async_wait<kCkScanDepth - 1>();
        float tf[8], rf[8], df[8];
        const float* slot = ring + (i % kCkScanDepth) * 768 + lane * 8;
        ck_load8(tf, slot);
        ck_load8(rf, slot + 256);
        ck_load8(df, slot + 512);
        float* out = ws + (long long)(nchunks - 1 - i) * CkWs::kBwd;
        ck_store_ws_frag(out + CkWs::kG1, Y, g, t);
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) X.c[j][q] -= df[j * 4 + q];
        ck_store_ws_frag(out + CkWs::kS0b, X, g, t);
        ck_scan_step(Y, tf, rf);
    }
    ck_store_state_t(X, W, p.wE, p.E, p.M, g, t);
}

__global__ void __launch_bounds__(kCkWarps * 32) delta_bwd_chunk_post_kernel(const DeltaBwdParams p) {
    constexpr int LD = kCkLd;
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nchunks = (p.L + 15) >> 4;
    const long long cid = (long long)blockIdx.x * kCkWarps + warp;
    if (cid >= (long long)p.NH * nchunks) return;
    const int seq = (int)(cid / nchunks), c = (int)(cid - (long long)seq * nchunks);
    const int n = seq / p.H, h = seq - n * p.H, t0 = c * 16, nt = min(16, p.L - t0);
    float* base = smem + warp * CkBwdPost::kWarp;
    float* Qs = base; float* Ks = base + kCkTile; float* Ws = base + 2 * kCkTile; float* Gs = base + 3 * kCkTile;
    float* LT = base + 4 * kCkTile; float* KT = base + 5 * kCkTile; float* XT = base + 6 * kCkTile; float* YT = base + 7 * kCkTile;
    float* BM = base + 8 * kCkTile; float* MK = base + 9 * kCkTile; float* bs = base + 10 * kCkTile;
    const float* ws = p.ws + cid * CkWs::kBwd;
    CkSrc sq, sk, sv, so, sg;
    sq.init(p.q, n, h, p.E);
    sk.init(p.k, n, h, p.E);
    sv.init(p.v, n, h, p.M);
    so.init(p.v_old, n, h, p.M);
    sg.init(p.gy, n, h, p.M);
    const float* bsrc = reinterpret_cast<const float*>(p.beta.p) + n * p.beta.sN + h * p.beta.sH;
    CkDst dq, dk, dv;
    dq.init(p.gq, n, h, p.E);
    dk.init(p.gk, n, h, p.E);
    dv.init(p.gv, n, h, p.M);
    float* dbeta = reinterpret_cast<float*>(p.gb.p) + n * p.gb.sN + h * p.gb.sH;
    ck_load_tile(Qs, sq, t0, nt, lane);
    ck_load_tile(Ks, sk, t0, nt, lane);
    ck_load_tile(Ws, sv, t0, nt, lane);
    ck_load_tile(MK, so, t0, nt, lane);
    ck_load_tile(Gs, sg, t0, nt, lane);
    ck_load_ws_tile(LT, ws + CkWs::kLt, lane);
    ck_load_ws_tile(KT, ws + CkWs::kKt, lane);
    ck_load_ws_tile(XT, ws + CkWs::kS0b, lane);
    ck_load_ws_tile(YT, ws + CkWs::kG1, lane);
    cp_async_commit();
    if (lane < 16) bs[lane] = lane < nt ? bsrc[(long long)(t0 + lane) * p.beta.sL] : 0.f;
    cp_async_wait<0>();
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int idx = lane + 32 * i, o = (idx >> 4) * LD + (idx & 15);
        Ws[o] -= MK[o];
    }
    // lambda = Lt + Kt G1, in place (each lane owns the same elements on both sides)
    Frag lam;
    frag_load(lam, LT, g, t);
    mm16(lam, [&](int m, int k) { return KT[m * LD + k]; }, [&](int k, int nn) { return YT[nn * LD + k]; }, g, t);
    __syncwarp();       // w complete; every lane is done with Lt
    frag_store(LT, lam, g, t);
    Frag a;
    frag_zero(a);
    mm16(a, [&](int m, int k) { return Gs[m * LD + k]; }, [&](int k, int nn) { return bs[nn] * Ws[nn * LD + k]; }, g, t);
    frag_store(BM, a, g, t, [](int r, int cc, float x) { return cc <= r ? x : 0.f; });
    __syncwarp();
    // dQ = gY S0^T + lower(gY U^T) K
    frag_zero(a);
    mm16(a, [&](int m, int k) { return Gs[m * LD + k]; }, [&](int k, int nn) { return XT[k * LD + nn]; }, g, t);
    mm16(a, [&](int m, int k) { return BM[m * LD + k]; }, [&](int k, int nn) { return Ks[k * LD + nn]; }, g, t);
    ck_store_frag(dq, a, t0, nt, g, t);
    // sym_strict((b lambda) U^T)
    frag_zero(a);
    mm16(a, [&](int m, int k) { return bs[m] * LT[m * LD + k]; }, [&](int k, int nn) { return bs[nn] * Ws[nn * LD + k]; }, g, t);
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = g + 8 * (i >> 1), cc = 8 * j + 2 * t + (i & 1);
            if (cc < r) { MK[r * LD + cc] = a.c[j][i]; MK[cc * LD + r] = a.c[j][i]; }
            if (cc == r) MK[r * LD + cc] = 0.f;
        }
    __syncwarp();
    // dK = U G1^T - (b lambda) S0^T + lower(gY U^T)^T Q - sym K
    frag_zero(a);
    mm16(a, [&](int m, int k) { return bs[m] * Ws[m * LD + k]; }, [&](int k, int nn) { return YT[k * LD + nn]; }, g, t);
    mm16(a, [&](int m, int k) { return -bs[m] * LT[m * LD + k]; }, [&](int k, int nn) { return XT[k * LD + nn]; }, g, t);
    mm16(a, [&](int m, int k) { return BM[k * LD + m]; }, [&](int k, int nn) { return Qs[k * LD + nn]; }, g, t);
    mm16(a, [&](int m, int k) { return -MK[m * LD + k]; }, [&](int k, int nn) { return Ks[k * LD + nn]; }, g, t);
    ck_store_frag(dk, a, t0, nt, g, t);
    // dv = beta lambda, dbeta = rowsum(lambda w)
    Frag w;
    frag_load(w, Ws, g, t);
    float db0 = 0.f, db1 = 0.f;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        db0 = fmaf(lam.c[j][0], w.c[j][0], fmaf(lam.c[j][1], w.c[j][1], db0));
        db1 = fmaf(lam.c[j][2], w.c[j][2], fmaf(lam.c[j][3], w.c[j][3], db1));
        lam.c[j][0] *= bs[g]; lam.c[j][1] *= bs[g];
        lam.c[j][2] *= bs[g + 8]; lam.c[j][3] *= bs[g + 8];
    }
    ck_store_frag(dv, lam, t0, nt, g, t);
    db0 += __shfl_xor_sync(0xffffffffu, db0, 1); db0 += __shfl_xor_sync(0xffffffffu, db0, 2);
    db1 += __shfl_xor_sync(0xffffffffu, db1, 1); db1 += __shfl_xor_sync(0xffffffffu, db1, 2);
    if (t == 0) {
        if (g < nt) dbeta[(long long)(t0 + g) * p.gb.sL] = db0;
        if (g + 8 < nt) dbeta[(long long)(t0 + g + 8) * p.gb.sL] = db1;
    }
}

}  // namespace fwp
