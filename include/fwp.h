/*
 * fwp.h -- C ABI of the B200 (sm_100a) fast-weight update kernels.
 *
 * One entry point per native function of the reference project's JIT-compiled
 * CUDA extensions (the pybind functions its torch.autograd.Function wrappers
 * call).  Each declaration cites the reference function it replaces, by the
 * file's path inside the reference project.  Argument order follows the
 * reference function; the differences are the ones a C ABI needs:
 *
 *   - tensors are passed as `fwp_tensor` (device pointer + 4 element strides
 *     of the logical (N, H, L, D) view) instead of torch::Tensor;
 *   - sizes are explicit; the CUDA stream and the device ordinal are explicit
 *     (the reference launches on the legacy default stream of device 0);
 *   - every function returns a status code (0 = ok) instead of void, validates
 *     on the host before any launch, and never throws;
 *   - `io_dtype` selects the element type of the *streamed* tensors
 *     (q, k, v, beta, z, outputs, gradients).  Fast-weight states (kv, states,
 *     cells), the tensors saved for the backward pass (v_old, v_insert, gates,
 *     post-activation copies) and parameter gradients are always fp32.
 *
 * Layout contract (same as the reference's PackedTensorAccessor32 view):
 * 4-D logical shape, arbitrary strides for the three outer dimensions,
 * innermost stride must be 1.  Strides are in elements and 64-bit.
 * Output buffers are overwritten (the reference accumulates into zeros).
 * State tensors are in/out: the forward leaves the end-of-segment state in
 * them, the backward rewinds them in place to the start-of-segment state.
 *
 * Ownership: the caller allocates everything, including scratch; the library
 * allocates nothing and keeps no pointer after a call returns.  Calls may be made
 * from several host threads and on several devices at once.  Three pieces of
 * process-wide state exist and are shared by all of them: the execution-plan
 * switches set by fwp_tune (atomic integers), the built-in scratch array of the
 * no-allocation entry point (one per GPU), and the per-GPU flag that
 * fwp_delta_device_fault reads.
 */
#ifndef FWP_H_
#define FWP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fwp_tensor {
    void*   data;       /* device pointer to element (0,0,0,0) */
    int64_t stride[4];  /* element strides of (N, H, L, D); stride[3] must be 1 */
} fwp_tensor;

enum fwp_dtype { FWP_F32 = 0, FWP_BF16 = 1 };

enum fwp_status {
    FWP_OK = 0,
    FWP_ERR_NULL = 1,         /* a required pointer is NULL */
    FWP_ERR_SHAPE = 2,        /* a size is <= 0 or inconsistent */
    FWP_ERR_STRIDE = 3,       /* innermost stride != 1, or a negative stride */
    FWP_ERR_ALIGN = 4,        /* pointer not aligned to its element size */
    FWP_ERR_DTYPE = 5,        /* unknown io_dtype */
    FWP_ERR_UNSUPPORTED = 6,  /* head dimension beyond what the kernels cover */
    FWP_ERR_CUDA = 7,         /* a CUDA runtime call failed; see fwp_last_cuda_error */
    FWP_ERR_VARIANT = 8,      /* unknown LSTM variant */
    FWP_ERR_SCRATCH = 9,      /* scratch buffer missing or too small */
    FWP_ERR_NOALLOC_TOO_LARGE = 10 /* problem needs more than FWP_NOALLOC_SCRATCH_FLOATS of built-in scratch */
};

/* Human-readable text for a status code.  Never NULL. */
const char* fwp_status_string(int status);
/* cudaError_t of the last failing CUDA call made by this thread (0 if none). */
int fwp_last_cuda_error(void);
/* Library version, major*10000 + minor*100 + patch. */
int fwp_version(void);
/* Largest head dimension the register-resident kernels cover (E, M <= this). */
int fwp_max_head_dim(void);
/* Number of kernels this library has launched in this process (all threads). */
unsigned long long fwp_launch_count(void);
/* Execution-plan switch for experiments and cross-checks (process-wide, atomic):
 * "delta.blocked" (-1 automatic, 0 per-step kernels, 1 four-step blocked kernels),
 * "delta.chunk64" (1 / 0: chunkwise tensor-core plan for bf16 streams at E = M = 64),
 * "delta.tc64" (-1 / 1 / 0: tcgen05 forward of that plan when the call has no more sequences than the device has SMs
 * and at least 128 steps, always, or never), "<op>.<D>.split", "delta_bwd.bulk",
 * "delta_bwd.16.chunk", "rec_fwd.32.warp" (1 / 0: short-chain forward of the recurrent delta net),
 * "rnn_bwd.32.roles" (1 / 2 / 0: chain-warp + trailing-warp backward of the delta RNN, 16 or 8 steps per chunk, or off),
 * "lstm_bwd.32.roles" (1 / 0: chain-warp + per-gate trailing-warp backward of the delta LSTM),
 * "lstm_fwd.32.gates" (1 / 0: one-warp-per-gate forward of the delta LSTM),
 * "rec_bwd.32.roles" (1 / 0: chain-warp + trailing-warp backward of the recurrent delta net),
 * "sum_bwd.roles" (1 / 0: the three gradients of the sum rule computed side by side by warps of their own, or one
 * after the other by the same warps),
 * "step.spread" (1 / 0: the per-step forward packs fewer sequences into a CTA while that puts CTAs on more SMs, or
 * always four warps per CTA),
 * "launch.dependent" (1 / 0: the register-resident delta-rule kernels are launched with programmatic stream serialisation, so that
 * their prologue overlaps the tail of the kernel before them in the stream, or plainly),
 * "delta.pipe64" (1 / 2 / 0: chunkwise bf16 kernels with a preparing warp one chunk ahead in both directions,
 * in the forward only, or not at all).  Returns 0 if accepted, FWP_ERR_UNSUPPORTED for an unknown key. */
int fwp_tune(const char* key, int value);
/* Name of the kernel this host thread launched last through the library ("" before the
 * first launch): lets a benchmark label its numbers with the plan the dispatch picked. */
const char* fwp_last_kernel(void);

/* ---- delta rule --------------------------------------------------------
 * replaces fast_weight_forward(Q,K,V,beta,v_old,v_insert,kv,out),
 *   algorithmic/fast_weight/fast_weight_cuda.cu:182-240
 * Q,K [N,H,L,E]; V,v_old,v_insert,out [N,H,L,M]; beta [N,H,L,1]; kv [N,H,E,M].
 * v_insert may have data == NULL (the backward recomputes it). */
int fwp_fast_weight_forward(int N, int H, int L, int E, int M,
                            const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                            const fwp_tensor* beta, const fwp_tensor* v_old,
                            const fwp_tensor* v_insert, const fwp_tensor* kv,
                            const fwp_tensor* out, int io_dtype, void* stream, int device);

/* replaces fast_weight_backward(Q,K,V,beta,v_old,v_insert,grad_out,fw_mem,gQ,gK,gV,gbeta),
 *   algorithmic/fast_weight/fast_weight_cuda.cu:564-664
 * One fused pass (the reference runs two).  v_insert is accepted for
 * signature parity and ignored (data may be NULL). */
int fwp_fast_weight_backward(int N, int H, int L, int E, int M,
                             const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                             const fwp_tensor* beta, const fwp_tensor* v_old,
                             const fwp_tensor* v_insert, const fwp_tensor* grad_out,
                             const fwp_tensor* fw_mem,
                             const fwp_tensor* grad_Q, const fwp_tensor* grad_K,
                             const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                             int io_dtype, void* stream, int device);

/* The delta-rule kernels move contiguous chunks with bulk asynchronous copies (in the tcgen05 plan also TMA
 * tile loads and tensor-core products) whose completion waits are bounded.  Returns 1 if such a wait ever ran out on the current device since the last
 * call (that launch then produced wrong numbers instead of hanging the GPU), 0 if not, -1 on a
 * CUDA error.  Synchronises the device; reading clears the flag.  No counterpart in the reference. */
int fwp_delta_device_fault(void);
/* Test hook for that mechanism: launches one CTA that waits, with a limit of `polls` (1..65536) polls, on a
 * barrier nothing completes; the wait runs out, the kernel returns, and the next fwp_delta_device_fault() reads 1.
 * Nothing hangs and the context stays usable.  No counterpart in the reference. */
int fwp_debug_bounded_wait_probe(int polls, void* stream, int device);

/* ---- input prologue / output epilogue of the delta-rule attention layer ----
 * One pass each for what the reference's layers do with a chain of elementwise and permute launches around the
 * op (language_modeling/src/utils/cuda_fast_weight_layer.py:106-125 and :152-163, algorithmic/layers.py:110-137).
 * All tensors fp32 and contiguous; D <= 128.
 *   prologue_forward:  qkvb (L,B,H,3D+1) -> q, k (elu+1, normalised to sum 1 over D), v, beta = sigmoid, each (B,H,L,.)
 *   prologue_backward: gradients of q, k, v, beta (B,H,L,.) and the same qkvb -> gradient of qkvb (L,B,H,3D+1)
 *   transpose:         to_len_major != 0: dst (L,B,H,D) = scale * src (B,H,L,D)  (the layer's output path);
 *                      to_len_major == 0: dst (B,H,L,D) = scale * src (L,B,H,D)  (its gradient) */
/* The delayed copies the recurrent families' wrappers hand to the backward kernels, in one pass:
 *   dst[n,h,t,:] = f(t == 0 ? first[n,h,0,:] : src[n,h,t-1,:]),  op 0: f = identity, op 1: f = tanh;
 * with minuend->data != NULL, dst = minuend[n,h,t,:] - that value.  src, minuend, dst [N,H,L,D]; first [N,H,1,D];
 * float32, unit inner stride.  Replaces the torch.cat / tanh / subtraction chains of
 * algorithmic/rec_update_fwm_tanh/__init__.py:108 and language_modeling/src/utils/fast_lstm/__init__.py:142-148. */
int fwp_delayed(int N, int H, int L, int D, const fwp_tensor* src, const fwp_tensor* first,
                const fwp_tensor* minuend, const fwp_tensor* dst, int op, void* stream, int device);

int fwp_delta_layer_prologue_forward(int L, int B, int H, int D, const float* qkvb,
                                     float* q, float* k, float* v, float* beta, void* stream, int device);
int fwp_delta_layer_prologue_backward(int L, int B, int H, int D, const float* qkvb,
                                      const float* grad_q, const float* grad_k, const float* grad_v,
                                      const float* grad_beta, float* grad_qkvb, void* stream, int device);
int fwp_delta_layer_transpose(int L, int B, int H, int D, const float* src, float* dst, float scale,
                              int to_len_major, void* stream, int device);

/* ---- sum rule (linear-transformer causal product with carried state) ----
 * replaces causal_dot_product(Q,K,V,kv,out),
 *   algorithmic/fast_transformers/causal_product_cuda.cu:98-140 */
int fwp_causal_dot_product(int N, int H, int L, int E, int M,
                           const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                           const fwp_tensor* kv, const fwp_tensor* out,
                           int io_dtype, void* stream, int device);

/* replaces causal_dot_backward(Q,K,V,grad_out,gQ,gK,gV),
 *   algorithmic/fast_transformers/causal_product_cuda.cu:369-445
 * Like the reference it takes no state: the prefix sums restart from zero. */
int fwp_causal_dot_backward(int N, int H, int L, int E, int M,
                            const fwp_tensor* Q, const fwp_tensor* K, const fwp_tensor* V,
                            const fwp_tensor* grad_out,
                            const fwp_tensor* grad_Q, const fwp_tensor* grad_K,
                            const fwp_tensor* grad_V,
                            int io_dtype, void* stream, int device);

/* ---- recurrent delta net -------------------------------------------------
 * replaces rec_update_fwm_tanh_forward(qx,kx,vx,bx,Rq,Rk,Rv,rb,q,k,v,beta,v_old,states,kv,out),
 *   algorithmic/rec_update_fwm_tanh/rec_update_fwm_tanh.cu:349-444
 * qx,kx,vx,q,k,v,v_old,out [N,H,L,D]; bx,beta_out [N,H,L,1]; Rq,Rk,Rv [1,H,D,D];
 * rb [1,H,1,D]; states [N,H,1,D] in/out; kv [N,H,D,D] in/out. */
int fwp_rec_update_fwm_tanh_forward(int N, int H, int L, int D,
                                    const fwp_tensor* qx, const fwp_tensor* kx,
                                    const fwp_tensor* vx, const fwp_tensor* bx,
                                    const fwp_tensor* Rq, const fwp_tensor* Rk,
                                    const fwp_tensor* Rv, const fwp_tensor* rb,
                                    const fwp_tensor* q_out, const fwp_tensor* k_out,
                                    const fwp_tensor* v_out, const fwp_tensor* beta_out,
                                    const fwp_tensor* v_old, const fwp_tensor* states,
                                    const fwp_tensor* kv, const fwp_tensor* out,
                                    int io_dtype, void* stream, int device);

/* replaces rec_update_fwm_tanh_backward(q,k,v,beta,v_old,o_delayed,grad_out,Rq,Rk,Rv,rb,fw_mem,
 *                                       gq,gk,gv,gbeta,gRq,gRk,gRv,grb),
 *   algorithmic/rec_update_fwm_tanh/rec_update_fwm_tanh.cu:880-986
 * The reference adds every sequence's parameter gradient into gR* with global
 * atomics; here each (n,h) writes its partial sums into `scratch` and a second
 * kernel adds them over n in a fixed order.  scratch: fp32, at least
 * fwp_rec_update_fwm_tanh_scratch_floats(N,H,D) elements, 16-byte aligned. */
int fwp_rec_update_fwm_tanh_backward(int N, int H, int L, int D,
                                     const fwp_tensor* q, const fwp_tensor* k,
                                     const fwp_tensor* v, const fwp_tensor* beta,
                                     const fwp_tensor* v_old, const fwp_tensor* o_delayed,
                                     const fwp_tensor* grad_out,
                                     const fwp_tensor* Rq, const fwp_tensor* Rk,
                                     const fwp_tensor* Rv, const fwp_tensor* rb,
                                     const fwp_tensor* fw_mem,
                                     const fwp_tensor* grad_q, const fwp_tensor* grad_k,
                                     const fwp_tensor* grad_v, const fwp_tensor* grad_beta,
                                     const fwp_tensor* grad_Rq, const fwp_tensor* grad_Rk,
                                     const fwp_tensor* grad_Rv, const fwp_tensor* grad_rb,
                                     float* scratch, int64_t scratch_floats,
                                     int io_dtype, void* stream, int device);
int64_t fwp_rec_update_fwm_tanh_scratch_floats(int N, int H, int D);

/* Same backward for callers that cannot allocate device memory when they call it
 * (a host bound to this ABI without a memory pool, or a process whose device memory
 * was handed out completely at start-up).  No counterpart in the reference, whose
 * wrapper always allocates with torch.  The scratch lives in a fixed array inside the
 * library, FWP_NOALLOC_SCRATCH_FLOATS floats per GPU (held by every GPU that loads
 * the library until the process exits), so N*H*(3*D*D+D) must not exceed it; larger
 * problems return FWP_ERR_NOALLOC_TOO_LARGE and launch nothing.  The first call on a
 * device looks up the array's device address (cudaGetSymbolAddress, that device
 * current): make it before any stream capture.  With lazy module loading the CUDA
 * runtime creates the array (and the kernels' local-memory pool) when this module is
 * first used on a device, so make the first recurrent-delta-net call of a process
 * (forward or backward) on each device before the device memory is handed out
 * completely; from then on the function itself allocates nothing (no cudaMalloc /
 * cudaFree / allocating library call).  All calls on a device share the array:
 * calls that may overlap on the GPU race, calls ordered on one stream do not. */
#define FWP_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
int fwp_rec_update_fwm_tanh_backward_noalloc(int N, int H, int L, int D,
                                             const fwp_tensor* q, const fwp_tensor* k,
                                             const fwp_tensor* v, const fwp_tensor* beta,
                                             const fwp_tensor* v_old, const fwp_tensor* o_delayed,
                                             const fwp_tensor* grad_out,
                                             const fwp_tensor* Rq, const fwp_tensor* Rk,
                                             const fwp_tensor* Rv, const fwp_tensor* rb,
                                             const fwp_tensor* fw_mem,
                                             const fwp_tensor* grad_q, const fwp_tensor* grad_k,
                                             const fwp_tensor* grad_v, const fwp_tensor* grad_beta,
                                             const fwp_tensor* grad_Rq, const fwp_tensor* grad_Rk,
                                             const fwp_tensor* grad_Rv, const fwp_tensor* grad_rb,
                                             int io_dtype, void* stream, int device);

/* ---- delta RNN v2 and v1 ---------------------------------------------------
 * replaces fast_rnn_v2_forward(Z,K,V,beta,v_old,states,kv,out,out_nmz),
 *   algorithmic/fast_weight_rnn_v2/fast_rnn_cuda.cu:233-293 */
int fwp_fast_rnn_v2_forward(int N, int H, int L, int D,
                            const fwp_tensor* Z, const fwp_tensor* K, const fwp_tensor* V,
                            const fwp_tensor* beta, const fwp_tensor* v_old,
                            const fwp_tensor* states, const fwp_tensor* kv,
                            const fwp_tensor* out, const fwp_tensor* out_nmz,
                            int io_dtype, void* stream, int device);
/* replaces fast_rnn_v2_backward(K,V,beta,v_old,grad_out,out,out_delayed,fw_mem,gZ,gK,gV,gbeta),
 *   algorithmic/fast_weight_rnn_v2/fast_rnn_cuda.cu:592-659.  `out` is unused (may have data NULL). */
int fwp_fast_rnn_v2_backward(int N, int H, int L, int D,
                             const fwp_tensor* K, const fwp_tensor* V, const fwp_tensor* beta,
                             const fwp_tensor* v_old, const fwp_tensor* grad_out,
                             const fwp_tensor* out, const fwp_tensor* out_delayed,
                             const fwp_tensor* fw_mem,
                             const fwp_tensor* grad_Z, const fwp_tensor* grad_K,
                             const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                             int io_dtype, void* stream, int device);
/* replaces fast_rnn_forward(Z,K,V,beta,v_old,states,kv,out),
 *   language_modeling/src/utils/fast_weight_rnn/fast_rnn_cuda.cu (forward host function) */
int fwp_fast_rnn_forward(int N, int H, int L, int D,
                         const fwp_tensor* Z, const fwp_tensor* K, const fwp_tensor* V,
                         const fwp_tensor* beta, const fwp_tensor* v_old,
                         const fwp_tensor* states, const fwp_tensor* kv,
                         const fwp_tensor* out,
                         int io_dtype, void* stream, int device);
/* replaces fast_rnn_backward(K,V,beta,v_old,grad_out,out,out_delayed,fw_mem,gZ,gK,gV,gbeta),
 *   language_modeling/src/utils/fast_weight_rnn/fast_rnn_cuda.cu (backward host function) */
int fwp_fast_rnn_backward(int N, int H, int L, int D,
                          const fwp_tensor* K, const fwp_tensor* V, const fwp_tensor* beta,
                          const fwp_tensor* v_old, const fwp_tensor* grad_out,
                          const fwp_tensor* out, const fwp_tensor* out_delayed,
                          const fwp_tensor* fw_mem,
                          const fwp_tensor* grad_Z, const fwp_tensor* grad_K,
                          const fwp_tensor* grad_V, const fwp_tensor* grad_beta,
                          int io_dtype, void* stream, int device);

/* ---- delta LSTM v1..v4 -----------------------------------------------------
 * One entry point for the four variants (variant = 1..4).  The twelve streamed
 * inputs are passed as arrays ordered by gate: index 0 = input gate (i),
 * 1 = update (u), 2 = output gate (o).
 * replaces fast_lstm_forward / fast_lstm_v2_forward / _v3_ / _v4_
 *   (Zi,Ki,Vi,bi, Zu,Ku,Vu,bu, Zo,Ko,Vo,bo, states, cells, kv_i,kv_u,kv_o,
 *    out, [out_del_nmz,] cell_out, gate_i, update_u, gate_o, v_old_i, v_old_u, v_old_o),
 *   language_modeling/src/utils/fast_lstm/fast_lstm_cuda.cu:364-480 and
 *   language_modeling/src/utils/fast_lstm_v{2,3,4}/fast_lstm_v{2,3,4}_cuda.cu (forward host functions).
 * out_del_nmz is required for variants 2-4 and ignored for variant 1. */
int fwp_fast_lstm_forward(int variant, int N, int H, int L, int D,
                          const fwp_tensor Z[3], const fwp_tensor K[3],
                          const fwp_tensor V[3], const fwp_tensor beta[3],
                          const fwp_tensor* states, const fwp_tensor* cells,
                          const fwp_tensor kv[3],
                          const fwp_tensor* out, const fwp_tensor* out_del_nmz,
                          const fwp_tensor* cell_out,
                          const fwp_tensor gates[3], /* gate_i, update_u, gate_o */
                          const fwp_tensor v_old[3],
                          int io_dtype, void* stream, int device);
/* replaces fast_lstm*_backward(grad_out, Ki,Vi,bi, Ku,Vu,bu, Ko,Vo,bo, v_old_i,v_old_u,v_old_o,
 *    out, out_delayed, cell_out, u_minus_c, gate_i, update_u, gate_o, kv_i,kv_u,kv_o,
 *    gZi,gKi,gVi,gbi, gZu,gKu,gVu,gbu, gZo,gKo,gVo,gbo),
 *   language_modeling/src/utils/fast_lstm/fast_lstm_cuda.cu:1061-1205 and the v2-v4 files. */
int fwp_fast_lstm_backward(int variant, int N, int H, int L, int D,
                           const fwp_tensor* grad_out,
                           const fwp_tensor K[3], const fwp_tensor V[3], const fwp_tensor beta[3],
                           const fwp_tensor v_old[3],
                           const fwp_tensor* out, const fwp_tensor* out_delayed,
                           const fwp_tensor* cell_out, const fwp_tensor* u_minus_c,
                           const fwp_tensor gates[3], const fwp_tensor kv[3],
                           const fwp_tensor grad_Z[3], const fwp_tensor grad_K[3],
                           const fwp_tensor grad_V[3], const fwp_tensor grad_beta[3],
                           int io_dtype, void* stream, int device);

#ifdef __cplusplus
}
#endif
#endif /* FWP_H_ */
