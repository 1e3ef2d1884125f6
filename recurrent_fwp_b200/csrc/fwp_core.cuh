// Shared device/host building blocks of the fast-weight kernels (sm_100a only).
//
// Execution model used by every kernel in this library:
//   * one CTA per (batch, head) sequence; the d x d fast-weight matrices live in
//     registers for the whole sequence;
//   * a thread is identified by (s, idx): `idx` in [0, D) is the column it owns
//     in the "column role" (reductions over the key index e are thread-local)
//     and, at the same time, the row it owns in the "row role" (reductions over
//     the value index m are thread-local); `s` in [0, SPLIT) selects which
//     D/SPLIT-long slice of that column / row the thread holds.  The SPLIT
//     threads of one idx sit in one warp, so a slice reduction is 0-2 shuffles;
//   * inputs stream through a two-stage shared-memory ring filled with
//     cp.async (16-byte copies when rows are aligned, 4-byte otherwise), so any
//     outer strides are accepted and padding columns read as zero;
//   * fp32 arithmetic uses the packed two-wide FMA of sm_100 (fma.rn.f32x2).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/fwp.h"

// every entry point declared in include/fwp.h is defined with this
#define FWP_API extern "C" __attribute__((visibility("default")))

namespace fwp {

// ------------------------------------------------------------------ host side
struct Row4 {            // one (N,H,L,width) tensor with unit inner stride
    void* p;
    long long sN, sH, sL;
};

static inline Row4 row4(const fwp_tensor* t) {
    Row4 r;
    r.p = t ? t->data : nullptr;
    r.sN = t ? t->stride[0] : 0;
    r.sH = t ? t->stride[1] : 0;
    r.sL = t ? t->stride[2] : 0;
    return r;
}

int check_tensor(const fwp_tensor* t, int elem_bytes, bool required);
int set_cuda_error(cudaError_t e);
void count_launch(int n = 1);
void note_kernel(const char* name);     // remembers, per host thread, the kernel launched last (fwp_last_kernel)

// Execution-plan switches (fwp_tune).  Each is one atomic integer looked up by index, so the dispatch of a
// call reads a few relaxed atomics: no string handling, no lock.
enum TuneKey {
    T_DELTA_BLOCKED,        // "delta.blocked": -1 automatic, 0 per-step kernels, 1 four-step blocked kernels
    T_DELTA_CHUNK64,        // "delta.chunk64": 1 chunkwise tensor-core plan for bf16 streams at E = M = 64, 0 off
    T_DELTA_TC64,           // "delta.tc64": -1 automatic (tcgen05 forward when the call has no more sequences than the device has SMs and at least 128 steps), 1 tcgen05 forward of that plan, 0 the warp-level mma forward
    T_DELTA_FWD_SPLIT16, T_DELTA_FWD_SPLIT32, T_DELTA_FWD_SPLIT64,      // "delta_fwd.<D>.split"
    T_SUM_FWD_SPLIT16, T_SUM_FWD_SPLIT32, T_SUM_FWD_SPLIT64,            // "sum_fwd.<D>.split"
    T_DELTA_BWD_SPLIT16, T_DELTA_BWD_SPLIT32, T_DELTA_BWD_SPLIT64,      // "delta_bwd.<D>.split"
    T_DELTA_BWD_BULK,       // "delta_bwd.bulk": 1 bulk-copy staging in the d = 16 backward, 0 cp.async
    T_DELTA_BWD_CHUNK16,    // "delta_bwd.16.chunk": 32 or 16 steps per staged chunk
    T_LSTM_FWD_SPLIT32, T_LSTM_BWD_SPLIT32, T_RNN_FWD_SPLIT32, T_RNN_BWD_SPLIT32, T_REC_FWD_SPLIT32, T_REC_BWD_SPLIT32,
    T_REC_FWD_WARP32,       // "rec_fwd.32.warp": 1 short-chain one-warp forward of the recurrent delta net at d <= 32, 0 the general kernel
    T_RNN_BWD_ROLES32,      // "rnn_bwd.32.roles": 1 / 2 chain-warp + trailing-warp backward of the delta RNN at d <= 32 (16 / 8 steps per chunk), 0 the general kernel
    T_LSTM_BWD_ROLES32,     // "lstm_bwd.32.roles": 1 chain-warp + three trailing-warp backward of the delta LSTM at d <= 32, 0 the general kernel
    T_LSTM_FWD_GATES32,     // "lstm_fwd.32.gates": 1 one-warp-per-gate forward of the delta LSTM at d = 32, 0 the general kernel
    T_DELTA_PIPE64,         // "delta.pipe64": 1 chunkwise bf16 forward with a preparing warp one chunk ahead, 0 every warp prepares for itself
    T_REC_BWD_ROLES32,      // "rec_bwd.32.roles": 1 chain-warp + trailing-warp backward of the recurrent delta net at d = 32, 0 the general kernel
    T_SUM_BWD_ROLES,        // "sum_bwd.roles": 1 the three gradients of the sum rule in warps of their own, side by side; 0 one after the other
    T_LAUNCH_DEPENDENT,     // "launch.dependent": 1 the register-resident delta-rule kernels (blocked and per-step) are launched with programmatic stream serialisation (their prologue overlaps the tail of the kernel before), 0 plain launches
    T_STEP_SPREAD,          // "step.spread": 1 the per-step forward packs fewer sequences into a CTA while that puts CTAs on more SMs, 0 always four warps per CTA
    T_COUNT
};
int tune_get(TuneKey key, int fallback);
int sm_count();             // SMs of the current device

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    int status = FWP_OK;
    explicit DeviceGuard(int device) {
        if (device < 0) return;
        cudaError_t e = cudaGetDevice(&prev);
        if (e != cudaSuccess) { status = set_cuda_error(e); return; }
        if (prev != device) {
            e = cudaSetDevice(device);
            if (e != cudaSuccess) { status = set_cuda_error(e); return; }
            switched = true;
        }
    }
    ~DeviceGuard() { if (switched) cudaSetDevice(prev); }
};

#ifdef __CUDACC__
__host__ __device__
#endif
constexpr int r4(int x) { return (x + 3) & ~3; }   // round a float count up to 16 bytes

// every row of every (n, h) slice of a float stream starts on a 16-byte boundary
static inline bool rows_16B_aligned(const Row4& r) {
    return (reinterpret_cast<uintptr_t>(r.p) & 15) == 0 && r.sN % 4 == 0 && r.sH % 4 == 0 && r.sL % 4 == 0;
}

static inline int pad_dim(int d) { return d <= 16 ? 16 : (d <= 32 ? 32 : (d <= 64 ? 64 : 0)); }

// ---------------------------------------------------------------- device side
#ifdef __CUDACC__

// Two fp32 values packed in one 64-bit register.  Everything that lives across
// time steps (the matrices, operand slices, dot-product accumulators) stays in
// this form, so the packed FMA needs no pack/unpack moves around it.
typedef unsigned long long f2;

__device__ __forceinline__ f2 f2_pack(float lo, float hi) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(f2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ float f2_hsum(f2 v) {
    float lo, hi;
    f2_unpack(v, lo, hi);
    return lo + hi;
}
__device__ __forceinline__ f2 ffma2(f2 a, f2 b, f2 c) {
    f2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f2 fadd2(f2 a, f2 b) {
    f2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// ---- short-latency forms of the transcendental steps on the recurrent chains (one MUFU each, no range split) ----
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// e^x for x <= 0 (softmax numerators after the shift): relative error about 2e-7 + 1e-7 |x|
__device__ __forceinline__ float exp_neg(float x) { return ex2_approx(x * kLog2e); }
__device__ __forceinline__ float sigmoidf_(float x) { return rcp_approx(1.f + ex2_approx(-kLog2e * x)); }
// |error| below 2e-7 over the whole range: odd polynomial to x^9 under 0.25, 1 - 2 / (e^{2|x|} + 1) above
__device__ __forceinline__ float tanh_fast(float x) {
    const float ax = fabsf(x), x2 = x * x;
    const float e = ex2_approx(ax * 2.885390082f);              // e^{2|x|}; inf above 44 gives exactly 1
    const float big = copysignf(fmaf(-2.f, rcp_approx(e + 1.f), 1.f), x);
    float pl = fmaf(x2, 2.1869488e-2f, -5.3968254e-2f);
    pl = fmaf(pl, x2, 1.3333334e-1f);
    pl = fmaf(pl, x2, -3.3333334e-1f);
    const float small = fmaf(x * x2, pl, x);
    return ax < 0.25f ? small : big;
}
// Warp-wide maximum in one instruction (sm_100a).
__device__ __forceinline__ float warp_max_f32(float x) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
    return r;
}
// Sum over the warp of values in [0, 1] whose total is at least 1 (softmax numerators after the shift by the
// maximum): fixed point with 26 fractional bits and the integer warp reduction.  The total is below 2^31, each
// addend is off by at most 2^-27, so the sum is good to 32 * 2^-27 relative -- two ulp -- and does not depend on
// any order of addition.  Returns 2^26 times the sum.
__device__ __forceinline__ float warp_sum_unit_scaled(float x) {
    return (float)__reduce_add_sync(0xffffffffu, __float2uint_rn(x * 67108864.f));
}
// Sum over the warp of signed values bounded by 2^24 in magnitude after the caller's scaling.
__device__ __forceinline__ float warp_sum_scaled(float x) {
    return (float)__reduce_add_sync(0xffffffffu, __float2int_rn(x));
}

template <int D_, int SPLIT_>
struct Geo {
    static constexpr int D = D_;
    static constexpr int SPLIT = SPLIT_;
    static constexpr int NT = D * SPLIT;     // threads per CTA
    static constexpr int NR = D / SPLIT;     // slice length held by one thread
    static constexpr int NP = NR / 2;        // ... in packed pairs
    static constexpr int MC = 32 / SPLIT;    // idx values per warp
    static constexpr int WPS = NT / 32;      // warps per sequence
    static_assert(NT % 32 == 0 && NR % 4 == 0 && SPLIT <= 4, "unsupported geometry");
    int tid, lane, warp, s, idx, off;        // off = first element of the slice
    int slot, seq;                           // several sequences may share a CTA: slot in the CTA, global sequence
    // Warps are spread over the four SM sub-partitions by their index in the CTA, so a CTA
    // should hold at least four warps: CTAs of fewer warps are packed with several sequences.
    __device__ __forceinline__ Geo() {
        init(threadIdx.x);
        seq = blockIdx.x * (blockDim.x / NT) + slot;
    }
    // t = index of the thread among the threads that play this role in the CTA
    __device__ __forceinline__ explicit Geo(int t) {
        init(t);
        seq = -1;
    }
    __device__ __forceinline__ void init(int t) {
        slot = t / NT;
        tid = t - slot * NT;
        lane = tid & 31;
        warp = tid >> 5;
        s = lane / MC;
        idx = warp * MC + (lane % MC);
        off = s * NR;
    }
};

// A kernel launched with programmatic stream serialisation may start while the kernel before it in the stream
// is still draining: everything up to this wait (index arithmetic, the shared-memory zero fill, barrier set-up)
// overlaps that tail; nothing of global memory is read or written before it.  A no-op for a plain launch.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets a dependent kernel behind this one be scheduled from now on (once every CTA of this grid has said so or
// left): its CTAs take the SMs this grid leaves free, run their prologue and park in griddep_wait() until this
// grid has completed.  Without a dependent launch behind it, nothing happens.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Barrier among the warps that serve one sequence slot of a CTA (named barriers 1..15; 0 is __syncthreads).
__device__ __forceinline__ void slot_barrier(int slot, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(slot + 1), "r"(nthreads) : "memory");
}

// sequences per CTA that fill four warps
__host__ __device__ constexpr int slots_for(int threads_per_seq) { return threads_per_seq >= 128 ? 1 : 128 / threads_per_seq; }

// the slice of dynamic shared memory that belongs to one sequence slot
template <class G>
__device__ __forceinline__ float* slot_smem(float* smem_all, const G& g) {
    unsigned dsz;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dsz));
    return smem_all + (size_t)g.slot * (dsz / (blockDim.x / G::NT) / 4);
}

// sum over the SPLIT threads that share one idx (all of them get the result)
template <int SPLIT>
__device__ __forceinline__ float reduce_split(float x) {
#pragma unroll
    for (int o = 16; o >= 32 / SPLIT; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// sum / max over the idx values of one warp (threads with equal s)
template <int SPLIT>
__device__ __forceinline__ float warp_sum_idx(float x) {
#pragma unroll
    for (int o = (32 / SPLIT) / 2; o >= 1; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
template <int SPLIT>
__device__ __forceinline__ float warp_max_idx(float x) {
#pragma unroll
    for (int o = (32 / SPLIT) / 2; o >= 1; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

template <int WPS>
__device__ __forceinline__ void cta_sync() {
    if constexpr (WPS == 1) __syncwarp(); else __syncthreads();
}

// All-reduce over idx across the whole CTA.  `slot` points at WPS floats of
// shared memory that no other reduction uses until the *next* cta_sync after
// this call (callers rotate slots).  Contains one cta_sync when WPS > 1.
template <class G, bool IS_MAX>
__device__ __forceinline__ float cta_allreduce_idx(const G& g, float x, float* slot) {
    if constexpr (IS_MAX && G::WPS == 1) return warp_max_f32(x);      // every idx sits in this warp (SPLIT times)
    x = IS_MAX ? warp_max_idx<G::SPLIT>(x) : warp_sum_idx<G::SPLIT>(x);
    if constexpr (G::WPS > 1) {
        if (g.lane == 0) slot[g.warp] = x;
        __syncthreads();
        float r = slot[0];
#pragma unroll
        for (int w = 1; w < G::WPS; w++) r = IS_MAX ? fmaxf(r, slot[w]) : r + slot[w];
        x = r;
    }
    return x;
}

// Denominator of a softmax over idx whose numerators were shifted by the maximum (each in [0, 1], the largest
// exactly 1; padding lanes pass 0).  One warp per sequence: the integer warp reduction, exact to two ulp.
template <class G>
__device__ __forceinline__ float softmax_den(const G& g, float ex, float* slot) {
    if constexpr (G::WPS == 1) return warp_sum_unit_scaled(ex) * (1.f / (67108864.f * G::SPLIT));
    else return cta_allreduce_idx<G, false>(g, ex, slot);
}

// slice of a shared-memory row -> packed registers (row must be 16-byte aligned)
template <int NR>
__device__ __forceinline__ void lds_slice(f2 (&d)[NR / 2], const float* p) {
#pragma unroll
    for (int i = 0; i < NR / 4; i++) {
        const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(p + 4 * i);
        d[2 * i] = t.x;
        d[2 * i + 1] = t.y;
    }
}

// Same load, but pinned in program order (volatile): used for operand prefetch, where the
// point is that the loads issue *before* the arithmetic of the current group, not next to
// their first use.
template <int NR>
__device__ __forceinline__ void lds_slice_early(f2 (&d)[NR / 2], const float* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
#pragma unroll
    for (int i = 0; i < NR / 4; i++)
        asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(d[2 * i]), "=l"(d[2 * i + 1]) : "r"(a + 16 * i));
}

template <int NP>
__device__ __forceinline__ float dot2(const f2 (&a)[NP], const f2 (&b)[NP]) {
    f2 acc0 = 0ull, acc1 = 0ull;
#pragma unroll
    for (int i = 0; i < NP; i += 2) {
        acc0 = ffma2(a[i], b[i], acc0);
        if (i + 1 < NP) acc1 = ffma2(a[i + 1], b[i + 1], acc1);
    }
    return f2_hsum(NP > 1 ? fadd2(acc0, acc1) : acc0);
}
// same with one accumulator chain: fewer instructions, for places with many independent dots
template <int NP>
__device__ __forceinline__ float dot2_chain(const f2 (&a)[NP], const f2 (&b)[NP]) {
    f2 acc = 0ull;
#pragma unroll
    for (int i = 0; i < NP; i++) acc = ffma2(a[i], b[i], acc);
    return f2_hsum(acc);
}

// A += x * a  (a scalar)
template <int NP>
__device__ __forceinline__ void axpy2(f2 (&A)[NP], const f2 (&x)[NP], float a) {
    const f2 aa = f2_pack(a, a);
#pragma unroll
    for (int i = 0; i < NP; i++) A[i] = ffma2(x[i], aa, A[i]);
}

// ---- fast-weight matrix <-> registers.  Column role: thread holds
// S[off..off+NR, idx]; row role: thread holds S[idx, off..off+NR].
template <class G>
__device__ __forceinline__ void load_cols(const G& g, f2 (&S)[G::NP], const float* W, long long sE, int E, int M) {
    float v[2];
#pragma unroll
    for (int i = 0; i < G::NR; i++) {
        int e = g.off + i;
        float x = (e < E && g.idx < M) ? W[(long long)e * sE + g.idx] : 0.f;
        v[i & 1] = x;
        if (i & 1) S[i >> 1] = f2_pack(v[0], v[1]);
    }
}
template <class G>
__device__ __forceinline__ void store_cols(const G& g, const f2 (&S)[G::NP], float* W, long long sE, int E, int M) {
#pragma unroll
    for (int i = 0; i < G::NR; i++) {
        int e = g.off + i;
        float lo, hi;
        f2_unpack(S[i >> 1], lo, hi);
        if (e < E && g.idx < M) W[(long long)e * sE + g.idx] = (i & 1) ? hi : lo;
    }
}
template <class G>
__device__ __forceinline__ void load_rows(const G& g, f2 (&S)[G::NP], const float* W, long long sE, int E, int M) {
    float v[2];
#pragma unroll
    for (int i = 0; i < G::NR; i++) {
        int m = g.off + i;
        float x = (g.idx < E && m < M) ? W[(long long)g.idx * sE + m] : 0.f;
        v[i & 1] = x;
        if (i & 1) S[i >> 1] = f2_pack(v[0], v[1]);
    }
}
template <class G>
__device__ __forceinline__ void store_rows(const G& g, const f2 (&S)[G::NP], float* W, long long sE, int E, int M) {
#pragma unroll
    for (int i = 0; i < G::NR; i++) {
        int m = g.off + i;
        float lo, hi;
        f2_unpack(S[i >> 1], lo, hi);
        if (g.idx < E && m < M) W[(long long)g.idx * sE + m] = (i & 1) ? hi : lo;
    }
}

// ---- cp.async staging -------------------------------------------------------
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }


// ---- bulk asynchronous copies (TMA, one instruction per contiguous chunk) ------------
// A producer warp moves whole [rows x D] chunks between global and shared memory with
// cp.async.bulk when the rows are contiguous and 16-byte aligned; loads complete on an
// mbarrier (complete_tx), stores are tracked by bulk groups.  Every wait is bounded: after
// kTmaSpinLimit failed polls the waiter records a fault and carries on, so a copy that never
// completes yields wrong numbers and a raised flag, never a hung GPU.
constexpr int kTmaSpinLimit = 1 << 16;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%1], %0;" ::"r"(count), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%1], %0;" ::"r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P1;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// returns false when the limit ran out
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity) {
    for (int i = 0; i < kTmaSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (before a bulk store / after zero fill)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// whole rows of a chunk can go by one bulk copy: full-width, contiguous, 16-byte aligned
template <int D, typename T>
__device__ __forceinline__ bool bulk_rows_ok(const T* base, long long sL, int width) {
    return width == D && sL == D && (reinterpret_cast<uintptr_t>(base) & 15) == 0 && (D * sizeof(T)) % 16 == 0;
}
template <typename T>
__device__ __forceinline__ bool bulk_col_ok(const T* base, long long sL, int t0, int nt) {   // [L,1] tensors
    return sL == 1 && (reinterpret_cast<uintptr_t>(base + t0) & 15) == 0 && (nt * sizeof(T)) % 16 == 0;
}

// One streamed tensor of one sequence: rows of `width` elements, row stride sL.
template <typename T>
struct Src {
    const T* base;      // element (n, h, 0, 0)
    long long sL;
    int width;          // valid elements per row (<= D)
    bool vec;           // rows can be copied in 16-byte pieces
    __device__ __forceinline__ void init(const Row4& r, int n, int h, int w) {
        base = reinterpret_cast<const T*>(r.p) + n * r.sN + h * r.sH;
        sL = r.sL;
        width = w;
        constexpr int per16 = 16 / (int)sizeof(T);
        vec = (w % per16 == 0) && ((reinterpret_cast<uintptr_t>(base) & 15) == 0) && (sL % per16 == 0);
    }
};

// Copy rows [t0, t0+nt) into a tile whose rows are D elements of T (row r of the
// tile = time step t0+r).  Elements beyond `width` are never written (the tile
// is zeroed once at kernel start).  NT = threads of the CTA.  The common case
// (full-width rows) walks rows with a fixed per-thread column, so each copy costs
// one address add; only padded widths pay for an integer division.
template <int D, int NT, int TC, typename T>
__device__ __forceinline__ void stage_rows(T* tile, const Src<T>& src, int t0, int nt, int tid) {
    constexpr int per16 = 16 / (int)sizeof(T);
    if (src.vec && src.width == D && D >= per16) {
        constexpr int PPR = (D >= per16) ? D / per16 : 1;    // 16-byte pieces per row
        constexpr int RSTEP = (NT >= PPR) ? NT / PPR : 1;    // rows covered per sweep of the CTA
        static_assert(D < per16 || NT % PPR == 0, "thread count must be a multiple of the pieces per row");
        int r = tid / PPR;
        const int c = (tid % PPR) * per16;
        const T* gp = src.base + (long long)(t0 + r) * src.sL + c;
        T* sp = tile + r * D + c;
        const long long gstep = (long long)RSTEP * src.sL;
        if (nt == TC && TC % RSTEP == 0) {      // full chunk: fixed trip count, copies issue back to back
#pragma unroll
            for (int it = 0; it < TC / RSTEP; it++) cp_async16(sp + it * RSTEP * D, gp + it * gstep);
        } else {
            for (; r < nt; r += RSTEP, gp += gstep, sp += RSTEP * D) cp_async16(sp, gp);
        }
    } else if (src.vec) {
        const int ppr = src.width / per16;
        const int total = nt * ppr;
        for (int i = tid; i < total; i += NT) {
            int r = i / ppr, c = (i - r * ppr) * per16;
            cp_async16(tile + r * D + c, src.base + (long long)(t0 + r) * src.sL + c);
        }
    } else if (src.width == D) {
        for (int i = tid; i < nt * D; i += NT) {
            const int r = i / D, c = i % D;
            const T* gp = src.base + (long long)(t0 + r) * src.sL + c;
            if constexpr (sizeof(T) == 4) cp_async4(tile + i, gp); else tile[i] = *gp;
        }
    } else {
        const int total = nt * src.width;
        for (int i = tid; i < total; i += NT) {
            int r = i / src.width, c = i - r * src.width;
            const T* gp = src.base + (long long)(t0 + r) * src.sL + c;
            if constexpr (sizeof(T) == 4) cp_async4(tile + r * D + c, gp); else tile[r * D + c] = *gp;
        }
    }
}

// ---- table-driven staging for the kernels whose stages hold many tiles ----------------------------------------
// A stage is `ntile` tiles of TC rows x 32 floats laid one after the other, followed by `ncol` columns of r4(TC)
// floats ([L,1] streams).  The sources sit in a small table in shared memory, so one short loop issues every copy of
// a chunk: a few instructions per 16-byte piece instead of one inlined copy routine per tile.  Requires full-width
// rows that start on 16-byte boundaries (the host checks with rows_16B_aligned before choosing such a kernel).
struct StageTable {
    static constexpr int kMaxTiles = 20, kMaxCols = 4;
    const float* src[kMaxTiles];        // element (n, h, 0, 0) of each tile's stream; nullptr = tile not used
    long long sL[kMaxTiles];
    const float* csrc[kMaxCols];
    long long csL[kMaxCols];
};
__device__ __forceinline__ void stage_table_set(StageTable* tb, int i, const Row4& r, int n, int h) {
    tb->src[i] = r.p ? reinterpret_cast<const float*>(r.p) + n * r.sN + h * r.sH : nullptr;
    tb->sL[i] = r.sL;
}
__device__ __forceinline__ void stage_table_set_col(StageTable* tb, int i, const Row4& r, int n, int h) {
    tb->csrc[i] = reinterpret_cast<const float*>(r.p) + n * r.sN + h * r.sH;
    tb->csL[i] = r.sL;
}
template <int TC, int NT>
__device__ __forceinline__ void stage_table_issue(float* stage, const StageTable* tb, int ntile, int ncol,
                                                  int t0, int nt, int tid) {
    static_assert((TC & (TC - 1)) == 0 && TC >= 4, "rows per chunk: a power of two");
    constexpr int D = 32;
    const int total = ntile * TC * 8;
#pragma unroll 1
    for (int i = tid; i < total; i += NT) {
        const int piece = i & 7, r = (i >> 3) & (TC - 1), tile = i / (8 * TC);
        const float* sp = tb->src[tile];
        if (r < nt && sp) cp_async16(stage + i * 4, sp + (long long)(t0 + r) * tb->sL[tile] + piece * 4);
    }
    float* cols = stage + ntile * TC * D;
    if (tid < ncol * TC) {
        const int c = tid / TC, r = tid - c * TC;
        if (r < nt) cp_async4(cols + c * r4(TC) + r, tb->csrc[c] + (long long)(t0 + r) * tb->csL[c]);
    }
    cp_async_commit();
}

// shared-memory tile of one streamed tensor: fp32 rows the compute loop reads,
// plus (for 16-bit inputs) the raw rows cp.async lands in.
template <int D, int TC, typename T>
struct Tile {
    static constexpr bool kRaw = sizeof(T) != 4;
    static constexpr int kFloats = TC * D + (kRaw ? TC * D / 2 : 0);
    float* f;     // [TC][D] fp32
    T* raw;       // [TC][D] T   (aliases f when T is float)
    __device__ __forceinline__ void bind(float* mem) {
        f = mem;
        raw = kRaw ? reinterpret_cast<T*>(mem + TC * D) : reinterpret_cast<T*>(mem);
    }
    template <int NT>
    __device__ __forceinline__ void load(const Src<T>& src, int t0, int nt, int tid) {
        stage_rows<D, NT, TC, T>(raw, src, t0, nt, tid);
    }
    // after the copies have landed and a barrier: widen 16-bit rows to fp32
    __device__ __forceinline__ void widen(int nt, int width, int tid, int nthreads) {
        if constexpr (kRaw) {
            for (int i = tid; i < nt * D; i += nthreads) {
                int c = i % D;
                f[i] = (c < width) ? to_f32(raw[i]) : 0.f;
            }
        }
    }
};

// write one element of a streamed output
template <typename T>
__device__ __forceinline__ void put(const Row4& r, int n, int h, int t, int c, float x) {
    reinterpret_cast<T*>(r.p)[n * r.sN + h * r.sH + (long long)t * r.sL + c] = from_f32<T>(x);
}


// Flush rows [0, nt) of an fp32 shared-memory tile (row length D, first `width`
// columns valid) to rows [t0, t0+nt) of a streamed output of element type T.
// 16-byte stores with a fixed per-thread column when the destination rows allow
// it, element stores otherwise.
template <int D, int NT, typename T>
__device__ __forceinline__ void flush_piece(T* dst, const float* src) {
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
    } else {
        const float4 a = *reinterpret_cast<const float4*>(src);
        const float4 b = *reinterpret_cast<const float4*>(src + 4);
        __nv_bfloat162 o[4];
        o[0] = __floats2bfloat162_rn(a.x, a.y);
        o[1] = __floats2bfloat162_rn(a.z, a.w);
        o[2] = __floats2bfloat162_rn(b.x, b.y);
        o[3] = __floats2bfloat162_rn(b.z, b.w);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
    }
}

template <int D, int NT, typename T, int TC = 0>
__device__ __forceinline__ void flush_rows(const float* tile, const Row4& r, int n, int h, int t0, int nt,
                                           int width, int tid) {
    T* base = reinterpret_cast<T*>(r.p) + n * r.sN + h * r.sH + (long long)t0 * r.sL;
    constexpr int per16 = 16 / (int)sizeof(T);
    const bool vec = (width % per16 == 0) && ((reinterpret_cast<uintptr_t>(base) & 15) == 0) && (r.sL % per16 == 0);
    if (vec && width == D && D >= per16) {
        constexpr int PPR = (D >= per16) ? D / per16 : 1;
        constexpr int RSTEP = (NT >= PPR) ? NT / PPR : 1;
        int row = tid / PPR;
        const int c = (tid % PPR) * per16;
        const float* src = tile + row * D + c;
        T* dst = base + (long long)row * r.sL + c;
        const long long dstep = (long long)RSTEP * r.sL;
        if (TC > 0 && nt == TC && TC % RSTEP == 0) {
#pragma unroll
            for (int it = 0; it < (TC > 0 ? TC / RSTEP : 1); it++)
                flush_piece<D, NT, T>(dst + it * dstep, src + it * RSTEP * D);
        } else {
            for (; row < nt; row += RSTEP, src += RSTEP * D, dst += dstep) flush_piece<D, NT, T>(dst, src);
        }
    } else if (width == D) {
        for (int i = tid; i < nt * D; i += NT) {
            const int row = i / D, c = i % D;
            base[(long long)row * r.sL + c] = from_f32<T>(tile[i]);
        }
    } else {
        for (int i = tid; i < nt * width; i += NT) {
            const int row = i / width, c = i - row * width;
            base[(long long)row * r.sL + c] = from_f32<T>(tile[row * D + c]);
        }
    }
}

// Gram scalars of one group of four consecutive steps, in time order within the group:
//   slot b(b-1)/2 + a      : k_a . k_b   for a <  b   (6 values)
//   slot 6 + b(b+1)/2 + a  : k_a . q_b   for a <= b   (10 values)
__host__ __device__ constexpr int gram_kk(int a, int b) { return b * (b - 1) / 2 + a; }
__host__ __device__ constexpr int gram_kq(int a, int b) { return 6 + b * (b + 1) / 2 + a; }

// Fill gram[g][16] for groups g < ng from the fp32 k and q tiles (rows 4g..4g+3).
template <int D, int NT, int TC>
__device__ __forceinline__ void gram_phase(const float* ktile, const float* qtile, float* gram, int ng, int tid) {
    constexpr unsigned IA = 0u | (0u << 2) | (1u << 4) | (0u << 6) | (1u << 8) | (2u << 10) |
                            (0u << 12) | (0u << 14) | (1u << 16) | (0u << 18) | (1u << 20) | (2u << 22) |
                            (0u << 24) | (1u << 26) | (2u << 28) | (3u << 30);
    constexpr unsigned IB = 1u | (2u << 2) | (2u << 4) | (3u << 6) | (3u << 8) | (3u << 10) |
                            (0u << 12) | (1u << 14) | (1u << 16) | (2u << 18) | (2u << 20) | (2u << 22) |
                            (3u << 24) | (3u << 26) | (3u << 28) | (3u << 30);
    constexpr int ITER = ((TC / 4) * 16 + NT - 1) / NT;
#pragma unroll
    for (int it = 0; it < ITER; it++) {
        const int w = tid + it * NT;
        if (w >= ng * 16) break;
        const int gi = w >> 4, pidx = w & 15;
        const int a = (IA >> (2 * pidx)) & 3, b = (IB >> (2 * pidx)) & 3;
        const float* x = ktile + (4 * gi + a) * D;
        const float* y = (pidx < 6 ? ktile : qtile) + (4 * gi + b) * D;
        // rows two apart start in the same bank: each lane walks its rows from a different 16-byte piece
        const int rot = ((4 * gi + a) >> 1) + ((4 * gi + b) >> 1);
        f2 acc0 = 0ull, acc1 = 0ull;
#pragma unroll
        for (int ii = 0; ii < D / 4; ii++) {
            const int i = (ii + rot) & (D / 4 - 1);
            const ulonglong2 xa = *reinterpret_cast<const ulonglong2*>(x + 4 * i);
            const ulonglong2 ya = *reinterpret_cast<const ulonglong2*>(y + 4 * i);
            acc0 = ffma2(xa.x, ya.x, acc0);
            acc1 = ffma2(xa.y, ya.y, acc1);
        }
        gram[w] = f2_hsum(fadd2(acc0, acc1));
    }
}

// Sum four per-thread values over the idx lanes of a warp with a halving butterfly
// (5-6 shuffles instead of 16-20).  Afterwards, within each group of MC lanes, the
// lane whose (lane % MC) == j * sum4_stride<SPLIT>() holds the total of value j.
template <int SPLIT>
__host__ __device__ constexpr int sum4_stride() { return ((32 / SPLIT) >= 16 ? 16 : (32 / SPLIT)) / 4; }
template <int SPLIT>
__device__ __forceinline__ float warp_sum4_idx(float p0, float p1, float p2, float p3, int lane) {
    constexpr int MC = 32 / SPLIT;
    if constexpr (MC == 32) {   // fold the top level first so that 16 lanes remain
        p0 += __shfl_xor_sync(0xffffffffu, p0, 16);
        p1 += __shfl_xor_sync(0xffffffffu, p1, 16);
        p2 += __shfl_xor_sync(0xffffffffu, p2, 16);
        p3 += __shfl_xor_sync(0xffffffffu, p3, 16);
    }
    constexpr int H1 = (MC >= 16 ? 16 : MC) / 2;   // 8 (or 4 when MC == 8)
    constexpr int H2 = H1 / 2;
    const bool hi1 = lane & H1;
    float k0 = hi1 ? p2 : p0, s0 = hi1 ? p0 : p2;
    float k1 = hi1 ? p3 : p1, s1 = hi1 ? p1 : p3;
    k0 += __shfl_xor_sync(0xffffffffu, s0, H1);
    k1 += __shfl_xor_sync(0xffffffffu, s1, H1);
    const bool hi2 = lane & H2;
    float k = hi2 ? k1 : k0, sx = hi2 ? k0 : k1;
    k += __shfl_xor_sync(0xffffffffu, sx, H2);
#pragma unroll
    for (int o = H2 / 2; o >= 1; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
    return k;
}

#endif  // __CUDACC__
}  // namespace fwp
