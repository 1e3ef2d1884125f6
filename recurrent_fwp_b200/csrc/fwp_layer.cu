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
// All four kernels are plain streaming kernels: one warp per (len, batch, head) row, rows visited in the order
// of the projected tensor so that reads are fully contiguous and writes are whole aligned rows.
#include "fwp_core.cuh"

namespace fwp {

constexpr int kLayerWarps = 8;          // rows per CTA
constexpr int kLayerMaxPerLane = 4;     // head dimension up to 128

struct LayerDims {
    int L, B, H, D;
    long long rows;     // L * B * H
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// phi(x) = (elu(x) + 1) / sum: returns the un-normalised p and accumulates nothing; elu(x)+1 = x+1 for x > 0, exp(x) otherwise
__device__ __forceinline__ float elu_p1(float x) { return x > 0.f ? x + 1.f : expf(x); }

__global__ void __launch_bounds__(kLayerWarps * 32) layer_prologue_fwd_kernel(const float* __restrict__ qkvb, float* __restrict__ q,
                                                                               float* __restrict__ k, float* __restrict__ v,
                                                                               float* __restrict__ beta, const LayerDims d) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * kLayerWarps + (threadIdx.x >> 5);     // row of the projected tensor
    if (r >= d.rows) return;
    const int h = (int)(r % d.H);
    const long long lb = r / d.H;
    const int b = (int)(lb % d.B), l = (int)(lb / d.B);
    const int D = d.D;
    const float* x = qkvb + r * (3 * D + 1);
    const long long o = (((long long)b * d.H + h) * d.L + l);      // row of the (B, H, len, .) tensors
    float pq[kLayerMaxPerLane], pk[kLayerMaxPerLane];
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int j = 0; j < kLayerMaxPerLane; j++) {
        const int i = lane + 32 * j;
        pq[j] = pk[j] = 0.f;
        if (i < D) {
            pq[j] = elu_p1(x[i]);
            pk[j] = elu_p1(x[D + i]);
            v[o * D + i] = x[2 * D + i];
        }
        sq += pq[j];
        sk += pk[j];
    }
    const float iq = 1.f / warp_sum(sq), ik = 1.f / warp_sum(sk);
#pragma unroll
    for (int j = 0; j < kLayerMaxPerLane; j++) {
        const int i = lane + 32 * j;
        if (i < D) {
            q[o * D + i] = pq[j] * iq;
            k[o * D + i] = pk[j] * ik;
        }
    }
    if (lane == 0) beta[o] = 1.f / (1.f + expf(-x[3 * D]));
}

// y = p / s with p = elu(x)+1:  dL/dx_i = (g_i - sum_j g_j y_j) / s * (x_i > 0 ? 1 : p_i);  sigmoid: g * b * (1 - b)
__global__ void __launch_bounds__(kLayerWarps * 32) layer_prologue_bwd_kernel(const float* __restrict__ qkvb, const float* __restrict__ gq,
                                                                               const float* __restrict__ gk, const float* __restrict__ gv,
                                                                               const float* __restrict__ gbeta, float* __restrict__ gx,
                                                                               const LayerDims d) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * kLayerWarps + (threadIdx.x >> 5);
    if (r >= d.rows) return;
    const int h = (int)(r % d.H);
    const long long lb = r / d.H;
    const int b = (int)(lb % d.B), l = (int)(lb / d.B);
    const int D = d.D;
    const float* x = qkvb + r * (3 * D + 1);
    float* y = gx + r * (3 * D + 1);
    const long long o = (((long long)b * d.H + h) * d.L + l);
    float xq[kLayerMaxPerLane], xk[kLayerMaxPerLane], pq[kLayerMaxPerLane], pk[kLayerMaxPerLane], aq[kLayerMaxPerLane], ak[kLayerMaxPerLane];
    float sq = 0.f, sk = 0.f, dq = 0.f, dk = 0.f;
#pragma unroll
    for (int j = 0; j < kLayerMaxPerLane; j++) {
        const int i = lane + 32 * j;
        xq[j] = xk[j] = pq[j] = pk[j] = aq[j] = ak[j] = 0.f;
        if (i < D) {
            xq[j] = x[i];
            xk[j] = x[D + i];
            pq[j] = elu_p1(xq[j]);
            pk[j] = elu_p1(xk[j]);
            aq[j] = gq[o * D + i];
            ak[j] = gk[o * D + i];
            y[2 * D + i] = gv[o * D + i];
        }
        sq += pq[j];
        sk += pk[j];
        dq = fmaf(aq[j], pq[j], dq);
        dk = fmaf(ak[j], pk[j], dk);
    }
    const float iq = 1.f / warp_sum(sq), ik = 1.f / warp_sum(sk);
    dq = warp_sum(dq) * iq;     // sum_j g_j y_j
    dk = warp_sum(dk) * ik;
#pragma unroll
    for (int j = 0; j < kLayerMaxPerLane; j++) {
        const int i = lane + 32 * j;
        if (i < D) {
            y[i] = (aq[j] - dq) * iq * (xq[j] > 0.f ? 1.f : pq[j]);
            y[D + i] = (ak[j] - dk) * ik * (xk[j] > 0.f ? 1.f : pk[j]);
        }
    }
    if (lane == 0) {
        const float s = 1.f / (1.f + expf(-x[3 * D]));
        y[3 * D] = gbeta[o] * s * (1.f - s);
    }
}

// (B, H, len, D) <-> (len, B, H, D) with a scale: dst row of one side = scale * src row of the other
__global__ void __launch_bounds__(kLayerWarps * 32) layer_transpose_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                                            const LayerDims d, float scale, int to_len_major) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * kLayerWarps + (threadIdx.x >> 5);     // row in (len, B, H) order
    if (r >= d.rows) return;
    const int h = (int)(r % d.H);
    const long long lb = r / d.H;
    const int b = (int)(lb % d.B), l = (int)(lb / d.B);
    const long long o = (((long long)b * d.H + h) * d.L + l);
    const float* s = src + (to_len_major ? o : r) * d.D;
    float* t = dst + (to_len_major ? r : o) * d.D;
    if ((d.D & 3) == 0) {
        for (int i = lane * 4; i < d.D; i += 128) {
            float4 x = *reinterpret_cast<const float4*>(s + i);
            x.x *= scale; x.y *= scale; x.z *= scale; x.w *= scale;
            *reinterpret_cast<float4*>(t + i) = x;
        }
    } else {
        for (int i = lane; i < d.D; i += 32) t[i] = scale * s[i];
    }
}

static int layer_dims(int L, int B, int H, int D, LayerDims& d) {
    if (L <= 0 || B <= 0 || H <= 0 || D <= 0) return FWP_ERR_SHAPE;
    if (D > 32 * kLayerMaxPerLane) return FWP_ERR_UNSUPPORTED;
    d.L = L; d.B = B; d.H = H; d.D = D;
    d.rows = (long long)L * B * H;
    if ((d.rows + kLayerWarps - 1) / kLayerWarps > 0x7fffffffLL) return FWP_ERR_SHAPE;
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
    const int grid = (int)((d.rows + kLayerWarps - 1) / kLayerWarps);
    layer_prologue_fwd_kernel<<<grid, kLayerWarps * 32, 0, (cudaStream_t)stream>>>(qkvb, q, k, v, beta, d);
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
    const int grid = (int)((d.rows + kLayerWarps - 1) / kLayerWarps);
    layer_prologue_bwd_kernel<<<grid, kLayerWarps * 32, 0, (cudaStream_t)stream>>>(qkvb, grad_q, grad_k, grad_v, grad_beta, grad_qkvb, d);
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
    const int grid = (int)((d.rows + kLayerWarps - 1) / kLayerWarps);
    layer_transpose_kernel<<<grid, kLayerWarps * 32, 0, (cudaStream_t)stream>>>(src, dst, d, scale, to_len_major ? 1 : 0);
    return finish_launch();
}
