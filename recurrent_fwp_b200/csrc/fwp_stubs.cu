// Temporary: entry points whose kernels are not written yet.
#include "fwp_core.cuh"
#define T const fwp_tensor*
FWP_API int fwp_rec_update_fwm_tanh_forward(int, int, int, int, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
FWP_API int fwp_rec_update_fwm_tanh_backward(int, int, int, int, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, float*, int64_t, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
FWP_API int64_t fwp_rec_update_fwm_tanh_scratch_floats(int, int, int) { return 0; }
FWP_API int fwp_fast_rnn_v2_forward(int, int, int, int, T, T, T, T, T, T, T, T, T, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
FWP_API int fwp_fast_rnn_v2_backward(int, int, int, int, T, T, T, T, T, T, T, T, T, T, T, T, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
FWP_API int fwp_fast_rnn_forward(int, int, int, int, T, T, T, T, T, T, T, T, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
FWP_API int fwp_fast_rnn_backward(int, int, int, int, T, T, T, T, T, T, T, T, T, T, T, T, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
FWP_API int fwp_fast_lstm_forward(int, int, int, int, int, T, T, T, T, T, T, T, T, T, T, T, T, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
FWP_API int fwp_fast_lstm_backward(int, int, int, int, int, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, int, void*, int) { return FWP_ERR_UNSUPPORTED; }
