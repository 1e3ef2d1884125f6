"""ctypes binding of ``libfwp.so`` (the C ABI declared in ``include/fwp.h``).

There is no CPU path and no fallback: if the shared library is missing this
module raises at import, and every call raises ``RuntimeError`` with the decoded
status when the library rejects its arguments or a CUDA call fails.
"""
import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, 'libfwp.so')

F32, BF16 = 0, 1


class FwpTensor(ctypes.Structure):
    _fields_ = [('data', ctypes.c_void_p), ('stride', ctypes.c_int64 * 4)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            'recurrent_fwp_b200: %s not found. Build it with `python recurrent_fwp_b200/build.py` '
            '(nvcc, sm_100a). There is no CPU or PyTorch fallback.' % LIB_PATH)
    return ctypes.CDLL(LIB_PATH)


lib = _load()
_T = ctypes.POINTER(FwpTensor)
_T3 = ctypes.POINTER(FwpTensor)   # arrays of three descriptors are passed as pointers
_i, _vp, _i64 = ctypes.c_int, ctypes.c_void_p, ctypes.c_int64

# name -> argument types, exactly as declared in include/fwp.h
SIGNATURES = {
    'fwp_fast_weight_forward': [_i] * 5 + [_T] * 8 + [_i, _vp, _i],
    'fwp_fast_weight_backward': [_i] * 5 + [_T] * 12 + [_i, _vp, _i],
    'fwp_causal_dot_product': [_i] * 5 + [_T] * 5 + [_i, _vp, _i],
    'fwp_causal_dot_backward': [_i] * 5 + [_T] * 7 + [_i, _vp, _i],
    'fwp_rec_update_fwm_tanh_forward': [_i] * 4 + [_T] * 16 + [_i, _vp, _i],
    'fwp_rec_update_fwm_tanh_backward': [_i] * 4 + [_T] * 20 + [ctypes.POINTER(ctypes.c_float), _i64, _i, _vp, _i],
    'fwp_rec_update_fwm_tanh_backward_noalloc': [_i] * 4 + [_T] * 20 + [_i, _vp, _i],
    'fwp_fast_rnn_v2_forward': [_i] * 4 + [_T] * 9 + [_i, _vp, _i],
    'fwp_fast_rnn_v2_backward': [_i] * 4 + [_T] * 12 + [_i, _vp, _i],
    'fwp_fast_rnn_forward': [_i] * 4 + [_T] * 8 + [_i, _vp, _i],
    'fwp_fast_rnn_backward': [_i] * 4 + [_T] * 12 + [_i, _vp, _i],
    'fwp_fast_lstm_forward': [_i] * 5 + [_T3] * 4 + [_T, _T, _T3, _T, _T, _T, _T3, _T3] + [_i, _vp, _i],
    'fwp_delta_layer_prologue_forward': [_i] * 4 + [ctypes.c_void_p] * 5 + [_vp, _i],
    'fwp_delta_layer_prologue_backward': [_i] * 4 + [ctypes.c_void_p] * 6 + [_vp, _i],
    'fwp_delta_layer_transpose': [_i] * 4 + [ctypes.c_void_p] * 2 + [ctypes.c_float, _i, _vp, _i],
    'fwp_debug_bounded_wait_probe': [_i, _vp, _i],
    'fwp_delayed': [_i] * 4 + [_T] * 4 + [_i, _vp, _i],
    'fwp_fast_lstm_backward': [_i] * 5 + [_T] + [_T3] * 4 + [_T] * 4 + [_T3] * 6 + [_i, _vp, _i],
}
OTHER_SYMBOLS = ['fwp_status_string', 'fwp_last_cuda_error', 'fwp_version', 'fwp_max_head_dim',
                 'fwp_launch_count', 'fwp_tune', 'fwp_rec_update_fwm_tanh_scratch_floats', 'fwp_delta_device_fault',
                 'fwp_last_kernel']

for _name, _args in SIGNATURES.items():
    _f = getattr(lib, _name)
    _f.argtypes = _args
    _f.restype = ctypes.c_int
lib.fwp_status_string.argtypes = [_i]
lib.fwp_status_string.restype = ctypes.c_char_p
lib.fwp_launch_count.restype = ctypes.c_ulonglong
lib.fwp_tune.argtypes = [ctypes.c_char_p, _i]
lib.fwp_rec_update_fwm_tanh_scratch_floats.argtypes = [_i, _i, _i]
lib.fwp_rec_update_fwm_tanh_scratch_floats.restype = _i64
lib.fwp_last_kernel.restype = ctypes.c_char_p


def io_dtype(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError('fast-weight kernels take float32 or bfloat16 streams, got %s' % t.dtype)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError('fast-weight kernels run on CUDA tensors only (got a %s tensor); '
                               'there is no CPU path' % t.device.type)


def require_streams(ref, shape_by_name):
    """Every stream handed to a kernel is read with the element type of the first one and with the sizes
    (N, H, L, D) passed beside the pointers, so a stream of another dtype, device or shape would be read out of
    bounds.  ``shape_by_name`` maps an argument name to ``(tensor, expected shape)``; raises ``TypeError`` for a
    dtype mismatch (the reference raises from ``data_ptr<float>()``) and ``RuntimeError`` otherwise."""
    for name, (t, shape) in shape_by_name.items():
        if t is None:
            continue
        if t.dtype != ref.dtype:
            raise TypeError('%s is %s but the first stream is %s: all streams of one call share a dtype'
                            % (name, t.dtype, ref.dtype))
        if t.device != ref.device:
            raise RuntimeError('%s is on %s but the first stream is on %s' % (name, t.device, ref.device))
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError('%s has shape %s, expected %s' % (name, tuple(t.shape), tuple(shape)))


def require_f32(ref, shape_by_name):
    """States, recurrent parameters and initial hidden vectors are float32 on the streams' device."""
    for name, (t, shape) in shape_by_name.items():
        if t.dtype != torch.float32:
            raise TypeError('%s must be float32, got %s' % (name, t.dtype))
        if t.device != ref.device:
            raise RuntimeError('%s is on %s but the streams are on %s' % (name, t.device, ref.device))
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError('%s has shape %s, expected %s' % (name, tuple(t.shape), tuple(shape)))


def grad_like(grad_out, ref, shape):
    """The incoming gradient in the streams' dtype with a unit inner stride; its device and shape are checked."""
    if grad_out.device != ref.device or tuple(grad_out.shape) != tuple(shape):
        raise RuntimeError('grad_out is %s on %s, expected %s on %s'
                           % (tuple(grad_out.shape), grad_out.device, tuple(shape), ref.device))
    if grad_out.dtype != ref.dtype:
        grad_out = grad_out.to(ref.dtype)
    return unit_inner(grad_out)


def desc(t):
    """Descriptor of a CUDA tensor viewed as 4-D (N, H, L, D); ``None`` -> NULL data."""
    d = FwpTensor()
    if t is None:
        d.data = None
        return d
    if not t.is_cuda:
        raise RuntimeError('fast-weight kernels run on CUDA tensors only (got a %s tensor); there is no CPU path'
                           % t.device.type)
    assert t.dim() == 4, 'expected a 4-D tensor'
    d.data = t.data_ptr()
    for i in range(4):
        d.stride[i] = 1 if (i == 3 and t.shape[3] == 1) else t.stride(i)
    return d


def delayed(src, first, op=0, minuend=None):
    """``f(cat([first, src[:, :, :-1]], dim=2))`` in one pass (op 0: identity, 1: tanh); with ``minuend``,
    ``minuend - that``.  The delayed copies the recurrent families' backward kernels take."""
    N, H, L, M = src.shape
    out = torch.empty((N, H, L, M), device=src.device, dtype=torch.float32)
    stream, dev = stream_and_device(src)
    check(lib.fwp_delayed(N, H, L, M, desc(unit_inner(src)), desc(unit_inner(first)),
                          desc(None if minuend is None else unit_inner(minuend)), desc(out), op, stream, dev),
          'delayed')
    return out


def desc3(ts):
    arr = (FwpTensor * 3)()
    for i, t in enumerate(ts):
        arr[i] = desc(t)
    return arr


def unit_inner(t):
    """Streams need a unit innermost stride; anything else is made contiguous."""
    if t.shape[-1] == 1 or t.stride(-1) == 1:
        return t
    return t.contiguous()


def stream_and_device(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream), t.device.index


def check(rc, what):
    if rc != 0:
        msg = lib.fwp_status_string(rc).decode()
        if rc == 7:
            msg += ' [cudaError %d]' % lib.fwp_last_cuda_error()
        raise RuntimeError('%s failed: %s' % (what, msg))


def device_fault():
    """1 if a bounded wait inside a delta-rule kernel ran out since the last call (synchronises the device)."""
    return int(lib.fwp_delta_device_fault())


def raise_on_device_fault(what):
    """With FWP_CHECK_DEVICE_FAULT=1 in the environment the delta-rule wrappers call this after every launch: it
    synchronises the device and raises if a bounded wait inside a kernel ran out (the launch then produced wrong
    numbers instead of hanging).  Off by default because of the synchronisation; a trainer can instead poll
    ``device_fault()`` at step or epoch boundaries."""
    if _CHECK_FAULT and device_fault() != 0:
        raise RuntimeError('%s: a bounded wait inside the kernel ran out; its results are invalid' % what)


_CHECK_FAULT = os.environ.get('FWP_CHECK_DEVICE_FAULT', '0') == '1'


def launch_count():
    return int(lib.fwp_launch_count())


def last_kernel():
    """Name of the kernel the calling thread launched last through the library."""
    return lib.fwp_last_kernel().decode()


def tune(key, value):
    check(lib.fwp_tune(key.encode(), int(value)), 'fwp_tune(%r)' % key)
