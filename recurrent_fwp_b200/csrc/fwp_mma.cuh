// Warp-level tensor-core building blocks shared by the delta-rule kernels (sm_100a): the 16x16 fp32 accumulator
// fragment of mma.sync.m16n8k8 / m16n8k4 TF32, the hi/lo operand split that keeps fp32 accuracy (three MMAs per
// tile: hi*hi + lo*hi + hi*lo), and the use of an accumulator fragment as the left operand of the next product.
#pragma once
#include "fwp_core.cuh"

namespace fwp {

struct Frag {                             // 16x16 fp32 accumulator of one warp: lane (g = lane/4, t = lane%4) holds
    float c[2][4];                        // c[j][0..1] = (row g, cols 8j+2t, +1), c[j][2..3] = (row g+8, same cols)
};

__device__ __forceinline__ void frag_zero(Frag& f) {
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) f.c[j][i] = 0.f;
}

// x = hi + lo with hi and lo valid TF32 bit patterns (10 explicit mantissa bits, the low 13 bits zero).  Both
// parts are taken by truncation: hi is within one TF32 ulp of x, lo carries the next 11 bits, and what is
// dropped is below 2^-20 |x|.  Two logic operations and one subtraction; the rounding conversion of the ISA
// costs several times that on this part and the products are issue-bound.
__device__ __forceinline__ void tf32_split(float x, unsigned& hi, unsigned& lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi)) & 0xffffe000u;
}

__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void mma_tf32_k4(float (&d)[4], const unsigned (&a)[2], unsigned b) {
    asm("mma.sync.aligned.m16n8k4.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(b));
}

// Operand fragments of a 16x16 matrix, split once into TF32 hi/lo parts, so that a matrix that feeds several
// products is loaded and split a single time.
struct AFr { unsigned h[2][4], l[2][4]; };            // [k-step][m16n8k8 A registers]
struct BFr { unsigned h[2][2][2], l[2][2][2]; };      // [k-step][n-tile][B registers]

// An accumulator fragment used as the left operand of the next product: k-step j takes the accumulator's
// column tile j with the contraction index relabelled (slot t <-> column 8j+2t, slot t+4 <-> column 8j+2t+1);
// the right operand must then be loaded with load_b_relabelled.
__device__ __forceinline__ void a_from_acc(AFr& f, const Frag& c) {
#pragma unroll
    for (int j = 0; j < 2; j++) {
        tf32_split(c.c[j][0], f.h[j][0], f.l[j][0]);
        tf32_split(c.c[j][2], f.h[j][1], f.l[j][1]);
        tf32_split(c.c[j][1], f.h[j][2], f.l[j][2]);
        tf32_split(c.c[j][3], f.h[j][3], f.l[j][3]);
    }
}
// transposed state fragment <-> the E x M state in global memory
__device__ __forceinline__ void ck_load_state_t(Frag& X, const float* W, long long wE, int E, int M, int g, int t) {
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int m = g + 8 * (i >> 1), e = 8 * j + 2 * t + (i & 1);
            X.c[j][i] = (e < E && m < M) ? W[e * wE + m] : 0.f;
        }
}
__device__ __forceinline__ void ck_store_state_t(const Frag& X, float* W, long long wE, int E, int M, int g, int t) {
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int m = g + 8 * (i >> 1), e = 8 * j + 2 * t + (i & 1);
            if (e < E && m < M) W[e * wE + m] = X.c[j][i];
        }
}
}  // namespace fwp
