// Input prologue and output epilogue of the delta-rule attention layer (sm_100a).
//
// Between the fused q/k/v/beta projection and the fast-weight op the reference's layers run a chain of
// separate elementwise and permute launches (language_modeling/src/utils/cuda_fast_weight_layer.py:106-125,
// algorithmic/layers.py:110-137):
//   qkvb (len, B, H, 3d+1) -> split -> sigmoid(beta) -> permute to (B, H, len, .) -> elu+1 -> sum-normalise q, k
// and after the op a scale, transpose and reshape back to (len, B, H*d) (cuda_fast_weight_layer.py:152-163).
// Here each direction is one pass: a projected row is read once and q, k, v, beta leave in the (B, H, len, .)
// layout with aligned, contiguous rows (which is also what lets the op stage them with 16-byte and bulk
// copies); the backward pass recomputes the normalisation from the same row and writes the gradient row once.
// All kernels are plain streaming kernels.  The prologue kernels give 8, 16 or 32 lanes to a (len, batch, head) row,
// visit rows in the order of the projected tensor so that reads are fully contiguous and writes are whole aligned
// rows, and issue every load before the first use; the transpose moves 16-byte pieces, four per thread.
#include "fwp_core.cuh"

namespace fwp {

constexpr int kLayerWarps = 8;          // warps per CTA
constexpr int kLayerRows = 4;           // pieces per thread of the transpose, all loads issued before the first use
constexpr int kLayerMaxD = 128;

struct LayerDims {
    int L, B, H, D;
    long long rows;     // L * B * H
};

// elu(x) + 1 = x + 1 for x > 0, exp(x) otherwise
__device__ __forceinline__ float elu_p1(float x) { return x > 0.f ? x + 1.f : expf(x); }

// row r of the projected (len, B, H, .) tensor -> row of the (B, H, len, .) tensors (rows fit 31 bits: 32-bit divisions)
__device__ __forceinline__ long long bhl_row(const LayerDims& d, long long r) {
    const unsigned r32 = (unsigned)r;
    const unsigned lb = r32 / (unsigned)d.H, h = r32 - lb * (unsigned)d.H;
    const unsigned l = lb / (unsigned)d.B, b = lb - l * (unsigned)d.B;
    return ((long long)b * d.H + h) * d.L + l;
}

// sum over the LPR consecutive lanes that share a row
template <int LPR>
__device__ __forceinline__ float row_sum(float x) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// LPR lanes share a row (8, 16 or 32 for D up to 32, 64, 128); lane `sub` of a row holds elements sub + LPR*j,
// j < 4, of each of q, k, v, so that one load instruction covers 32/LPR rows with contiguous 4*LPR-byte pieces.
constexpr int kLayerPer = 4;

template <int LPR, int PASSES>
__global__ void __launch_bounds__(kLayerWarps * 32) layer_prologue_fwd_kernel(const float* __restrict__ qkvb, float* __restrict__ q,
                                                                               float* __restrict__ k, float* __restrict__ v,
                                                                               float* __restrict__ beta, const LayerDims d) {
    constexpr int RPW = 32 / LPR;       // rows per warp and pass
    const int lane = threadIdx.x & 31, sub = lane % LPR, D = d.D;
    const long long r0 = ((long long)blockIdx.x * kLayerWarps + (threadIdx.x >> 5)) * (RPW * PASSES) + lane / LPR;
    float xq[PASSES][kLayerPer], xk[PASSES][kLayerPer], xv[PASSES][kLayerPer], xb[PASSES];
#pragma unroll
    for (int a = 0; a < PASSES; a++) {
        const long long r = r0 + a * RPW;
        const float* x = qkvb + r * (3 * D + 1);
        const bool live = r < d.rows;
#pragma unroll
        for (int j = 0; j < kLayerPer; j++) {
            const int i = sub + LPR * j;
            const bool ok = live && i < D;
            xq[a][j] = ok ? x[i] : 0.f;
            xk[a][j] = ok ? x[D + i] : 0.f;
            xv[a][j] = ok ? x[2 * D + i] : 0.f;
        }
        xb[a] = (live && sub == 0) ? x[3 * D] : 0.f;
    }
#pragma unroll
    for (int a = 0; a < PASSES; a++) {
        const long long r = r0 + a * RPW;
        const bool live = r < d.rows;
        const long long o = live ? bhl_row(d, r) : 0;
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int j = 0; j < kLayerPer; j++) {
            const bool ok = sub + LPR * j < D;
            xq[a][j] = ok ? elu_p1(xq[a][j]) : 0.f;
            xk[a][j] = ok ? elu_p1(xk[a][j]) : 0.f;
            sq += xq[a][j];
            sk += xk[a][j];
        }
        const float iq = 1.f / row_sum<LPR>(sq), ik = 1.f / row_sum<LPR>(sk);
        if (!live) continue;
#pragma unroll
        for (int j = 0; j < kLayerPer; j++) {
            const int i = sub + LPR * j;
            if (i < D) {
                q[o * D + i] = xq[a][j] * iq;
                k[o * D + i] = xk[a][j] * ik;
                v[o * D + i] = xv[a][j];
            }
        }
        if (sub == 0) beta[o] = 1.f / (1.f + expf(-xb[a]));
    }
}

// y = p / s with p = elu(x)+1:  dL/dx_i = (g_i - sum_j g_j y_j) / s * (x_i > 0 ? 1 : p_i);  sigmoid: g * b * (1 - b)
template <int LPR>
__global__ void __launch_bounds__(kLayerWarps * 32) layer_prologue_bwd_kernel(const float* __restrict__ qkvb, const float* __restrict__ gq,
                                                                               const float* __restrict__ gk, const float* __restrict__ gv,
                                                                               const float* __restrict__ gbeta, float* __restrict__ gx,
                                                                               const LayerDims d) {
    constexpr int RPW = 32 / LPR;
    const int lane = threadIdx.x & 31, sub = lane % LPR, D = d.D;
    const long long r = ((long long)blockIdx.x * kLayerWarps + (threadIdx.x >> 5)) * RPW + lane / LPR;
    const bool live = r < d.rows;
    const long long o = live ? bhl_row(d, r) : 0;
    const float* x = qkvb + r * (3 * D + 1);
    float xq[kLayerPer], xk[kLayerPer], aq[kLayerPer], ak[kLayerPer], av[kLayerPer];
#pragma unroll
    for (int j = 0; j < kLayerPer; j++) {
        const int i = sub + LPR * j;
        const bool ok = live && i < D;
        xq[j] = ok ? x[i] : 0.f;
        xk[j] = ok ? x[D + i] : 0.f;
        aq[j] = ok ? gq[o * D + i] : 0.f;
        ak[j] = ok ? gk[o * D + i] : 0.f;
        av[j] = ok ? gv[o * D + i] : 0.f;
    }
    const float xb = (live && sub == 0) ? x[3 * D] : 0.f;
    const float ab = (live && sub == 0) ? gbeta[o] : 0.f;
    float pq[kLayerPer], pk[kLayerPer];
    float sq = 0.f, sk = 0.f, dq = 0.f, dk = 0.f;
#pragma unroll
    for (int j = 0; j < kLayerPer; j++) {
        const bool ok = sub + LPR * j < D;
        pq[j] = ok ? elu_p1(xq[j]) : 0.f;
        pk[j] = ok ? elu_p1(xk[j]) : 0.f;
        sq += pq[j];
        sk += pk[j];
        dq = fmaf(aq[j], pq[j], dq);
        dk = fmaf(ak[j], pk[j], dk);
    }
    const float iq = 1.f / row_sum<LPR>(sq), ik = 1.f / row_sum<LPR>(sk);
    dq = row_sum<LPR>(dq) * iq;     // sum_j g_j y_j
    dk = row_sum<LPR>(dk) * ik;
    if (!live) return;
    float* y = gx + r * (3 * D + 1);
#pragma unroll
    for (int j = 0; j < kLayerPer; j++) {
        const int i = sub + LPR * j;
        if (i < D) {
            y[i] = (aq[j] - dq) * iq * (xq[j] > 0.f ? 1.f : pq[j]);
            y[D + i] = (ak[j] - dk) * ik * (xk[j] > 0.f ? 1.f : pk[j]);
            y[2 * D + i] = av[j];
        }
    }
    if (sub == 0) {
        const float sg = 1.f / (1.f + expf(-xb));
        y[3 * D] = ab * sg * (1.f - sg);
    }
}

// (B, H, len, D) <-> (len, B, H, D) with a scale: dst row of one side = scale * src row of the other.
// One thread per 16-byte piece (4-byte piece when D is not a multiple of 4), kLayerRows pieces per thread.
template <typename V>
__global__ void __launch_bounds__(kLayerWarps * 32) layer_transpose_kernel(const V* __restrict__ src, V* __restrict__ dst,
                                                                            const LayerDims d, int per_row, float scale, int to_len_major) {
    const long long total = d.rows * per_row;
    const long long i0 = ((long long)blockIdx.x * kLayerRows) * (kLayerWarps * 32) + threadIdx.x;
    V x[kLayerRows];
    long long to[kLayerRows];
#pragma unroll
    for (int a = 0; a < kLayerRows; a++) {
        const long long i = i0 + (long long)a * (kLayerWarps * 32);      // piece index in (len, B, H, .) order
        to[a] = -1;
        if (i < total) {
            long long r;
            int c;
            if (total <= 0x7fffffffLL) {
                const unsigned q32 = (unsigned)i / (unsigned)per_row;
                r = q32;
                c = (int)((unsigned)i - q32 * (unsigned)per_row);
            } else {
                r = i / per_row;
                c = (int)(i - r * per_row);
            }
            const long long j = bhl_row(d, r) * per_row + c;
            x[a] = src[to_len_major ? j : i];
            to[a] = to_len_major ? i : j;
        }
    }
#pragma unroll
    for (int a = 0; a < kLayerRows; a++) {
        if (to[a] < 0) continue;
        if constexpr (sizeof(V) == 16) {
            x[a].x *= scale; x[a].y *= scale; x[a].z *= scale; x[a].w *= scale;
        } else {
            x[a] *= scale;
        }
        dst[to[a]] = x[a];
    }
}

// dst[n,h,t,:] = f(t == 0 ? first[n,h,0,:] : src[n,h,t-1,:]), f = identity or tanh; with a minuend, minuend - that.
// V = float4 when rows are 16-byte aligned and D % 4 == 0.
struct DelayedParams {
    const float* src; long long sN, sH, sL;
    const float* first; long long fN, fH;
    const float* minuend; long long mN, mH, mL;
    float* dst; long long dN, dH, dL;
    int H, L, per_row, op;
    long long total;
};
template <typename V>
__global__ void __launch_bounds__(256) delayed_kernel(const DelayedParams p) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= p.total) return;
    constexpr int W = sizeof(V) / 4;
    const int c = (int)(i % p.per_row) * W;
    const long long row = i / p.per_row;
    const int t = (int)(row % p.L);
    const long long nh = row / p.L;
    const int h = (int)(nh % p.H);
    const long long n = nh / p.H;
    const float* sp = t == 0 ? p.first + n * p.fN + h * p.fH + c : p.src + n * p.sN + h * p.sH + (long long)(t - 1) * p.sL + c;
    V x = *reinterpret_cast<const V*>(sp);
    float* xf = reinterpret_cast<float*>(&x);
    if (p.op == 1) {
#pragma unroll
        for (int j = 0; j < W; j++) xf[j] = tanhf(xf[j]);
    }
    if (p.minuend) {
        const V m = *reinterpret_cast<const V*>(p.minuend + n * p.mN + h * p.mH + (long long)t * p.mL + c);
        const float* mf = reinterpret_cast<const float*>(&m);
#pragma unroll
        for (int j = 0; j < W; j++) xf[j] = mf[j] - xf[j];
    }
    *reinterpret_cast<V*>(p.dst + n * p.dN + h * p.dH + (long long)t * p.dL + c) = x;
}

static int layer_dims(int L, int B, int H, int D, LayerDims& d) {
    if (L <= 0 || B <= 0 || H <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (D > kLayerMaxD) return FWP_ERR_UNSUPPORTED;
    d.L = L; d.B = B; d.H = H; d.D = D;
    d.rows = (long long)L * B * H;
    if (d.rows > 0x7fffffffLL) return FWP_ERR_SHAPE;
    return FWP_OK;
}

static int finish_launch() {
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FWP_OK : set_cuda_error(e);
}

}  // namespace fwp

using namespace fwp;

FWP_API int fwp_delta_layer_prologue_forward(int L, int B, int H, int D, const float* qkvb,
                                             float* q, float* k, float* v, float* beta, void* stream, int device) {
    LayerDims d;
    if (int rc = layer_dims(L, B, H, D, d)) return rc;
    if (!qkvb || !q || !k || !v || !beta) return FWP_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(qkvb) | reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
         reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(beta)) & 3) return FWP_ERR_ALIGN;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    cudaStream_t st = (cudaStream_t)stream;
    auto grid = [&](int rows_per_warp) { return (int)((d.rows + kLayerWarps * rows_per_warp - 1) / (kLayerWarps * rows_per_warp)); };
    if (D <= 32) layer_prologue_fwd_kernel<8, 2><<<grid(8), kLayerWarps * 32, 0, st>>>(qkvb, q, k, v, beta, d);
    else if (D <= 64) layer_prologue_fwd_kernel<16, 2><<<grid(4), kLayerWarps * 32, 0, st>>>(qkvb, q, k, v, beta, d);
    else layer_prologue_fwd_kernel<32, 2><<<grid(2), kLayerWarps * 32, 0, st>>>(qkvb, q, k, v, beta, d);
    return finish_launch();
}

FWP_API int fwp_delta_layer_prologue_backward(int L, int B, int H, int D, const float* qkvb,
                                              const float* grad_q, const float* grad_k, const float* grad_v,
                                              const float* grad_beta, float* grad_qkvb, void* stream, int device) {
    LayerDims d;
    if (int rc = layer_dims(L, B, H, D, d)) return rc;
    if (!qkvb || !grad_q || !grad_k || !grad_v || !grad_beta || !grad_qkvb) return FWP_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(qkvb) | reinterpret_cast<uintptr_t>(grad_q) | reinterpret_cast<uintptr_t>(grad_k) |
         reinterpret_cast<uintptr_t>(grad_v) | reinterpret_cast<uintptr_t>(grad_beta) | reinterpret_cast<uintptr_t>(grad_qkvb)) & 3)
        return FWP_ERR_ALIGN;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    cudaStream_t st = (cudaStream_t)stream;
    auto grid = [&](int rows_per_warp) { return (int)((d.rows + kLayerWarps * rows_per_warp - 1) / (kLayerWarps * rows_per_warp)); };
    if (D <= 32) layer_prologue_bwd_kernel<8><<<grid(4), kLayerWarps * 32, 0, st>>>(qkvb, grad_q, grad_k, grad_v, grad_beta, grad_qkvb, d);
    else if (D <= 64) layer_prologue_bwd_kernel<16><<<grid(2), kLayerWarps * 32, 0, st>>>(qkvb, grad_q, grad_k, grad_v, grad_beta, grad_qkvb, d);
    else layer_prologue_bwd_kernel<32><<<grid(1), kLayerWarps * 32, 0, st>>>(qkvb, grad_q, grad_k, grad_v, grad_beta, grad_qkvb, d);
    return finish_launch();
}

FWP_API int fwp_delta_layer_transpose(int L, int B, int H, int D, const float* src, float* dst, float scale,
                                      int to_len_major, void* stream, int device) {
    LayerDims d;
    if (int rc = layer_dims(L, B, H, D, d)) return rc;
    if (!src || !dst) return FWP_ERR_NULL;
    const uintptr_t mask = (D & 3) == 0 ? 15 : 3;
    if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & mask) return FWP_ERR_ALIGN;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    const int per_row = (D & 3) == 0 ? D / 4 : D;
    const long long per_cta = (long long)kLayerWarps * 32 * kLayerRows;
    const long long ctas = (d.rows * per_row + per_cta - 1) / per_cta;
    if (ctas > 0x7fffffffLL) return FWP_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if ((D & 3) == 0)
        layer_transpose_kernel<float4><<<(int)ctas, kLayerWarps * 32, 0, st>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst),
                                                                              d, per_row, scale, to_len_major ? 1 : 0);
    else
        layer_transpose_kernel<float><<<(int)ctas, kLayerWarps * 32, 0, st>>>(src, dst, d, per_row, scale, to_len_major ? 1 : 0);
    return finish_launch();
}

FWP_API int fwp_delayed(int N, int H, int L, int D, const fwp_tensor* src, const fwp_tensor* first,
                        const fwp_tensor* minuend, const fwp_tensor* dst, int op, void* stream, int device) {
    if (N <= 0 || H <= 0 || L <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (op != 0 && op != 1) return FWP_ERR_UNSUPPORTED;
    int rc;
    if ((rc = check_tensor(src, 4, true)) || (rc = check_tensor(first, 4, true)) || (rc = check_tensor(dst, 4, true)) ||
        (rc = check_tensor(minuend, 4, false)))
        return rc;
    const bool sub = minuend && minuend->data;
    DeviceGuard guard(device);
    if (guard.status) return guard.status;
    DelayedParams p;
    p.src = (const float*)src->data; p.sN = src->stride[0]; p.sH = src->stride[1]; p.sL = src->stride[2];
    p.first = (const float*)first->data; p.fN = first->stride[0]; p.fH = first->stride[1];
    p.minuend = sub ? (const float*)minuend->data : nullptr;
    p.mN = sub ? minuend->stride[0] : 0; p.mH = sub ? minuend->stride[1] : 0; p.mL = sub ? minuend->stride[2] : 0;
    p.dst = (float*)dst->data; p.dN = dst->stride[0]; p.dH = dst->stride[1]; p.dL = dst->stride[2];
    p.H = H; p.L = L; p.op = op;
    auto al = [](const void* q, long long a, long long b, long long c) {
        return (reinterpret_cast<uintptr_t>(q) & 15) == 0 && a % 4 == 0 && b % 4 == 0 && c % 4 == 0;
    };
    const bool vec = D % 4 == 0 && al(p.src, p.sN, p.sH, p.sL) && al(p.first, p.fN, p.fH, 0) &&
                     al(p.dst, p.dN, p.dH, p.dL) && (!sub || al(p.minuend, p.mN, p.mH, p.mL));
    p.per_row = vec ? D / 4 : D;
    p.total = (long long)N * H * L * p.per_row;
    const long long ctas = (p.total + 255) / 256;
    if (ctas > 0x7fffffffLL) return FWP_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (vec) delayed_kernel<float4><<<(int)ctas, 256, 0, st>>>(p);
    else delayed_kernel<float><<<(int)ctas, 256, 0, st>>>(p);
    return finish_launch();
}
