// Delta rule for shapes outside the register-resident kernels (E or M above 64):
// the callers' Performer / DPFP feature maps give E = 2*proj_dim or 2*n_roll*d with a
// small M, and the "delta-delta" layers give M = 3d+1.  One CTA per sequence, the
// E x M matrices live in shared memory, every reduction is "thread-local partial
// over a strided subset, partials in shared memory, barrier, final sum".  This is
// the coverage path (same math, same outputs, deterministic), not a tuned one; the
// reference's single kernel covers these shapes with shared-memory atomics
// (algorithmic/fast_weight/fast_weight_cuda.cu:17-178, 244-560).
#pragma once
#include "fwp_core.cuh"

namespace fwp {

constexpr int kGenThreads = 256;

__host__ __device__ inline int gen_pow2_at_least(int x) {
    int p = 1;
    while (p < x && p < kGenThreads) p <<= 1;
    return p;
}
__host__ __device__ inline int gen_max3(int a, int b, int c) { return a > b ? (a > c ? a : c) : (b > c ? b : c); }

// floats of dynamic shared memory
static inline size_t gen_fwd_floats(int E, int M) {
    return (size_t)E * (M + 1) + 2 * E + 2 * M + 4 + gen_max3(kGenThreads, E, M);
}
static inline size_t gen_bwd_floats(int E, int M) {
    return 2 * (size_t)E * (M + 1) + 3 * E + 6 * M + 4 + 2 * (size_t)gen_max3(kGenThreads, E, M);
}

static inline size_t gen_sum_bwd_floats(int E, int M) {
    return (size_t)E * (M + 1) + 2 * E + 2 * M + 2 * (size_t)gen_max3(kGenThreads, E, M);
}

template <typename T>
__device__ __forceinline__ float gen_ld(const Row4& r, int n, int h, int t, int c) {
    return to_f32(reinterpret_cast<const T*>(r.p)[n * r.sN + h * r.sH + (long long)t * r.sL + c]);
}

template <typename T, bool SUM>
__global__ void __launch_bounds__(kGenThreads) delta_fwd_generic_kernel(const DeltaFwdParams p) {
    const int tid = threadIdx.x, NT = kGenThreads;
    const int n = blockIdx.x / p.H, h = blockIdx.x - n * p.H;
    const int E = p.E, M = p.M, LD = M + 1;
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                    // [E][LD]
    float* ks = S + (size_t)E * LD;   // [E]
    float* qs = ks + E;               // [E]
    float* vs = qs + E;               // [M]
    float* us = vs + M;               // [M]
    float* sc = us + M;               // [4] scalars
    float* part = sc + 4;             // partial sums
    // column mapping: thread (eg, m0) walks m = m0, m0+MT, ... and e = eg, eg+EG, ...
    const int MT = gen_pow2_at_least(M), EG = NT / MT;
    const int m0 = tid % MT, eg = tid / MT;
    float* W = p.W + n * p.wN + h * p.wH;
    for (int i = tid; i < E * M; i += NT) S[(i / M) * LD + (i % M)] = W[(long long)(i / M) * p.wE + (i % M)];
    __syncthreads();
    for (int t = 0; t < p.L; t++) {
        for (int e = tid; e < E; e += NT) { ks[e] = gen_ld<T>(p.k, n, h, t, e); qs[e] = gen_ld<T>(p.q, n, h, t, e); }
        for (int m = tid; m < M; m += NT) vs[m] = gen_ld<T>(p.v, n, h, t, m);
        if (tid == 0) sc[0] = SUM ? 1.f : gen_ld<T>(p.beta, n, h, t, 0);
        __syncthreads();
        if (!SUM) {
            for (int m = m0; m < M; m += MT) {
                float acc = 0.f;
                for (int e = eg; e < E; e += EG) acc = fmaf(S[e * LD + m], ks[e], acc);
                part[eg * M + m] = acc;
            }
            __syncthreads();
        }
        for (int m = tid; m < M; m += NT) {
            float vo = 0.f;
            if (!SUM) for (int g2 = 0; g2 < EG; g2++) vo += part[g2 * M + m];
            const float u = SUM ? vs[m] : sc[0] * (vs[m] - vo);
            us[m] = u;
            if (!SUM) {
                put<float>(p.v_old, n, h, t, m, vo);
                if (p.v_ins.p) put<float>(p.v_ins, n, h, t, m, u);
            }
        }
        __syncthreads();
        for (int m = m0; m < M; m += MT) {
            float acc = 0.f;
            const float u = us[m];
            for (int e = eg; e < E; e += EG) {
                const float s = fmaf(ks[e], u, S[e * LD + m]);
                S[e * LD + m] = s;
                acc = fmaf(s, qs[e], acc);
            }
            part[eg * M + m] = acc;
        }
        __syncthreads();
        for (int m = tid; m < M; m += NT) {
            float y = 0.f;
            for (int g2 = 0; g2 < EG; g2++) y += part[g2 * M + m];
            put<T>(p.out, n, h, t, m, y);
        }
        __syncthreads();
    }
    for (int i = tid; i < E * M; i += NT) W[(long long)(i / M) * p.wE + (i % M)] = S[(i / M) * LD + (i % M)];
}

template <typename T>
__global__ void __launch_bounds__(kGenThreads) delta_bwd_generic_kernel(const DeltaBwdParams p) {
    const int tid = threadIdx.x, NT = kGenThreads;
    const int n = blockIdx.x / p.H, h = blockIdx.x - n * p.H;
    const int E = p.E, M = p.M, LD = M + 1;
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                        // [E][LD]  state, rewound step by step
    float* G = S + (size_t)E * LD;        // [E][LD]  dL/dS
    float* ks = G + (size_t)E * LD;       // [E]
    float* qs = ks + E;                   // [E]
    float* dk1 = qs + E;                  // [E]
    float* gys = dk1 + E;                 // [M]
    float* ws = gys + M;                  // [M] v - v_old
    float* us = ws + M;                   // [M] beta * w
    float* brs = us + M;                  // [M] beta * r
    float* pws = brs + M;                 // [M] r * w
    float* sc = pws + M;                  // [4]
    const int PS = gen_max3(NT, E, M);
    float* part = sc + 4 + M;             // [PS]
    float* part2 = part + PS;             // [PS]
    const int MT = gen_pow2_at_least(M), EG = NT / MT, m0 = tid % MT, eg = tid / MT;   // column mapping
    const int ET = gen_pow2_at_least(E), MG = NT / ET, e0 = tid % ET, mg = tid / ET;   // row mapping
    float* W = p.W + n * p.wN + h * p.wH;
    for (int i = tid; i < E * M; i += NT) {
        S[(i / M) * LD + (i % M)] = W[(long long)(i / M) * p.wE + (i % M)];
        G[(i / M) * LD + (i % M)] = 0.f;
    }
    __syncthreads();
    for (int t = p.L - 1; t >= 0; t--) {
        if (tid == 0) sc[0] = gen_ld<T>(p.beta, n, h, t, 0);
        for (int e = tid; e < E; e += NT) { ks[e] = gen_ld<T>(p.k, n, h, t, e); qs[e] = gen_ld<T>(p.q, n, h, t, e); }
        __syncthreads();
        const float beta = sc[0];
        for (int m = tid; m < M; m += NT) {
            gys[m] = gen_ld<T>(p.gy, n, h, t, m);
            const float w = gen_ld<T>(p.v, n, h, t, m) - gen_ld<float>(p.v_old, n, h, t, m);
            ws[m] = w;
            us[m] = beta * w;
        }
        __syncthreads();
        // G += q (x) gy ; r = G^T k  (column mapping)
        for (int m = m0; m < M; m += MT) {
            float acc = 0.f;
            const float gy = gys[m];
            for (int e = eg; e < E; e += EG) {
                const float g2 = fmaf(qs[e], gy, G[e * LD + m]);
                G[e * LD + m] = g2;
                acc = fmaf(g2, ks[e], acc);
            }
            part[eg * M + m] = acc;
        }
        __syncthreads();
        for (int m = tid; m < M; m += NT) {
            float r = 0.f;
            for (int g2 = 0; g2 < EG; g2++) r += part[g2 * M + m];
            const float br = beta * r;
            brs[m] = br;
            pws[m] = r * ws[m];
            put<T>(p.gv, n, h, t, m, br);
        }
        __syncthreads();
        if (tid == 0) {
            float db = 0.f;
            for (int m = 0; m < M; m++) db += pws[m];
            put<T>(p.gb, n, h, t, 0, db);
        }
        // dq = S gy ; dk1 = G u  (row mapping)
        for (int e = e0; e < E; e += ET) {
            float a1 = 0.f, a2 = 0.f;
            for (int m = mg; m < M; m += MG) {
                a1 = fmaf(S[e * LD + m], gys[m], a1);
                a2 = fmaf(G[e * LD + m], us[m], a2);
            }
            part[mg * E + e] = a1;
            part2[mg * E + e] = a2;
        }
        __syncthreads();
        for (int e = tid; e < E; e += NT) {
            float dq = 0.f, d1 = 0.f;
            for (int g2 = 0; g2 < MG; g2++) { dq += part[g2 * E + e]; d1 += part2[g2 * E + e]; }
            put<T>(p.gq, n, h, t, e, dq);
            dk1[e] = d1;
        }
        __syncthreads();
        // S -= k (x) u ; dk = dk1 - S (beta r) ; G -= k (x) beta r  (row mapping)
        for (int e = e0; e < E; e += ET) {
            float a1 = 0.f;
            const float ke = ks[e];
            for (int m = mg; m < M; m += MG) {
                const float s = fmaf(-ke, us[m], S[e * LD + m]);
                S[e * LD + m] = s;
                a1 = fmaf(s, brs[m], a1);
                G[e * LD + m] = fmaf(-ke, brs[m], G[e * LD + m]);
            }
            part[mg * E + e] = a1;
        }
        __syncthreads();
        for (int e = tid; e < E; e += NT) {
            float d2 = 0.f;
            for (int g2 = 0; g2 < MG; g2++) d2 += part[g2 * E + e];
            put<T>(p.gk, n, h, t, e, dk1[e] - d2);
        }
        __syncthreads();
    }
    for (int i = tid; i < E * M; i += NT) W[(long long)(i / M) * p.wE + (i % M)] = S[(i / M) * LD + (i % M)];
}

// Sum-rule backward for the same shapes (algorithmic/fast_transformers/causal_product_cuda.cu:369-445 takes any
// E, M): a forward sweep with S accumulated from zero gives dq_t = S_t gy_t, a backward sweep with
// G = sum_{s>=t} q_s (x) gy_s gives dk_t = G_t v_t and dv_t = G_t^T k_t.  One E x M matrix in shared memory serves
// both sweeps.
template <typename T>
__global__ void __launch_bounds__(kGenThreads) sum_bwd_generic_kernel(const SumBwdParams p) {
    const int tid = threadIdx.x, NT = kGenThreads;
    const int n = blockIdx.x / p.H, h = blockIdx.x - n * p.H;
    const int E = p.E, M = p.M, LD = M + 1;
    extern __shared__ __align__(16) float sm[];
    float* A = sm;                        // [E][LD]  S in the first sweep, G in the second
    float* ks = A + (size_t)E * LD;       // [E]
    float* qs = ks + E;                   // [E]
    float* vs = qs + E;                   // [M]
    float* gys = vs + M;                  // [M]
    const int PS = gen_max3(NT, E, M);
    float* part = gys + M;                // [PS]
    float* part2 = part + PS;             // [PS]
    const int MT = gen_pow2_at_least(M), EG = NT / MT, m0 = tid % MT, eg = tid / MT;   // column mapping
    const int ET = gen_pow2_at_least(E), MG = NT / ET, e0 = tid % ET, mg = tid / ET;   // row mapping
    for (int sweep = 0; sweep < 2; sweep++) {
        for (int i = tid; i < E * LD; i += NT) A[i] = 0.f;
        __syncthreads();
        for (int i = 0; i < p.L; i++) {
            const int t = sweep ? p.L - 1 - i : i;
            for (int e = tid; e < E; e += NT) { ks[e] = gen_ld<T>(p.k, n, h, t, e); qs[e] = gen_ld<T>(p.q, n, h, t, e); }
            for (int m = tid; m < M; m += NT) { vs[m] = gen_ld<T>(p.v, n, h, t, m); gys[m] = gen_ld<T>(p.gy, n, h, t, m); }
            __syncthreads();
            if (sweep == 0) {
                // S += k (x) v ; dq = S gy  (row mapping)
                for (int e = e0; e < E; e += ET) {
                    float a1 = 0.f;
                    const float ke = ks[e];
                    for (int m = mg; m < M; m += MG) {
                        const float s = fmaf(ke, vs[m], A[e * LD + m]);
                        A[e * LD + m] = s;
                        a1 = fmaf(s, gys[m], a1);
                    }
                    part[mg * E + e] = a1;
                }
                __syncthreads();
                for (int e = tid; e < E; e += NT) {
                    float dq = 0.f;
                    for (int g2 = 0; g2 < MG; g2++) dq += part[g2 * E + e];
                    put<T>(p.gq, n, h, t, e, dq);
                }
            } else {
                // G += q (x) gy ; dk = G v  (row mapping)
                for (int e = e0; e < E; e += ET) {
                    float a1 = 0.f;
                    const float qe = qs[e];
                    for (int m = mg; m < M; m += MG) {
                        const float g2 = fmaf(qe, gys[m], A[e * LD + m]);
                        A[e * LD + m] = g2;
                        a1 = fmaf(g2, vs[m], a1);
                    }
                    part[mg * E + e] = a1;
                }
                __syncthreads();
                for (int e = tid; e < E; e += NT) {
                    float dk = 0.f;
                    for (int g2 = 0; g2 < MG; g2++) dk += part[g2 * E + e];
                    put<T>(p.gk, n, h, t, e, dk);
                }
                // dv = G^T k  (column mapping)
                for (int m = m0; m < M; m += MT) {
                    float acc = 0.f;
                    for (int e = eg; e < E; e += EG) acc = fmaf(A[e * LD + m], ks[e], acc);
                    part2[eg * M + m] = acc;
                }
                __syncthreads();
                for (int m = tid; m < M; m += NT) {
                    float dv = 0.f;
                    for (int g2 = 0; g2 < EG; g2++) dv += part2[g2 * M + m];
                    put<T>(p.gv, n, h, t, m, dv);
                }
            }
            __syncthreads();
        }
    }
}

}  // namespace fwp
