"""ctypes binding of libgonngpu_cuda.so, used by the tests and by bench.py.

It is deliberately thin: every function below is one call through the C ABI
declared in include/gonngpu.h, with numpy arrays as the host buffers.  There is
no fallback: if the library is missing, or no B200 is visible, calls fail.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GONNGPU_LIB", os.path.join(HERE, "libgonngpu_cuda.so"))

FP32_3XTF32, FP16_RN, FP16_TRUNC = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_LEAKY, ACT_SIGMOID, ACT_TANH, ACT_GELU = -1, 0, 1, 2, 3, 4


class CError(ctypes.Structure):
    _fields_ = [("message", ctypes.c_void_p)]


class GonnError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


_lib = None

_c_long, _c_int, _c_float, _vp = ctypes.c_long, ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_errp = ctypes.POINTER(CError)

# name -> (restype, argtypes); the list mirrors include/gonngpu.h one to one.
SIGNATURES = {
    "create_gpu_buffer": (_c_int, [_vp, _c_long, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _errp]),
    "retrieve_gpu_buffer_data": (_c_int, [_vp, _vp, _c_long, _errp]),
    "release_gpu_buffer": (_c_int, [_vp]),
    "free_c_error_message": (None, [_vp]),
    "perform_mps_matrix_multiplication": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _errp]),
    "perform_mps_matrix_transpose": (_c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _errp]),
    "perform_mps_matrix_add_broadcast": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _errp]),
    "perform_activation_relu_forward": (_c_int, [_vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_relu_backward": (_c_int, [_vp, _vp, _c_long, _vp, _vp, _errp]),
    "perform_mps_matrix_add": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _errp]),
    "perform_mps_matrix_subtract": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _errp]),
    "perform_mps_matrix_element_multiply": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _errp]),
    "perform_mps_matrix_element_divide": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _errp]),
    "perform_mps_matrix_scalar_add": (_c_int, [_vp, _c_long, _c_long, _c_float, _vp, _vp, _errp]),
    "perform_mps_matrix_scalar_multiply": (_c_int, [_vp, _c_long, _c_long, _c_float, _vp, _vp, _errp]),
    "perform_activation_sigmoid_forward": (_c_int, [_vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_sigmoid_backward": (_c_int, [_vp, _vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_tanh_forward": (_c_int, [_vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_tanh_backward": (_c_int, [_vp, _vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_leaky_relu_forward": (_c_int, [_vp, _c_long, _c_float, _vp, _vp, _errp]),
    "perform_activation_leaky_relu_backward": (_c_int, [_vp, _vp, _c_long, _c_float, _vp, _vp, _errp]),
    "perform_activation_softmax_1d_forward": (_c_int, [_vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_softmax_1d_backward": (_c_int, [_vp, _vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_softmax_2d_forward": (_c_int, [_vp, _c_long, _c_long, _vp, _vp, _errp]),
    "perform_activation_softmax_2d_backward": (_c_int, [_vp, _vp, _c_long, _c_long, _vp, _vp, _errp]),
    "perform_activation_elu_forward": (_c_int, [_vp, _c_long, _c_float, _vp, _vp, _errp]),
    "perform_activation_elu_backward": (_c_int, [_vp, _vp, _c_long, _c_float, _vp, _vp, _errp]),
    "perform_activation_swish_forward": (_c_int, [_vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_swish_backward": (_c_int, [_vp, _vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_gelu_forward": (_c_int, [_vp, _c_long, _vp, _vp, _errp]),
    "perform_activation_gelu_backward": (_c_int, [_vp, _vp, _c_long, _vp, _vp, _errp]),
    "perform_fused_linear_activation": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _vp, _c_int, _c_float, _vp, _vp, _errp]),
    "perform_optimized_gemm": (
        _c_int, [_vp, _vp, _vp, _c_long, _c_long, _c_long, _c_float, _c_float, _vp, _errp]),
    "perform_batch_matmul_optimized": (
        _c_int, [_vp, _vp, _vp, _c_long, _c_long, _c_long, _c_long, _vp, _errp]),
    "allocateSharedMemory": (_vp, [_c_long]),
    "createGPUBufferFromSharedMemory": (_vp, [_vp, _vp, _c_long]),
    "gonngpu_matmul_ex": (
        _c_int, [_vp, _c_long, _c_long, _c_int, _vp, _c_long, _c_long, _c_int, _vp, _c_long, _c_long,
                 _c_int, _c_float, _c_float, _vp, _c_int, _c_float, _errp]),
    "gonngpu_gemm_f16_device": (
        _c_int, [_vp, _c_long, _c_long, _c_long, _c_int, _vp, _c_long, _c_long, _c_long, _c_int, _vp,
                 _c_long, _c_float, _c_float, _vp, _c_int, _c_float, _errp]),
    "gonngpu_convert_f16_device": (_c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_int, _errp]),
    "gonngpu_matmul_f16_static_scratch": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _vp, _errp]),
    "gonngpu_replicate_send": (
        _c_int, [_vp, _vp, _c_long, _vp, _c_int, _c_int, _c_long, _c_int, ctypes.c_uint, ctypes.c_uint,
                 _c_int, _vp, _errp]),
    "gonngpu_replicate_wait": (
        _c_int, [_vp, _c_int, _c_int, _c_int, _c_long, _c_int, ctypes.c_uint, ctypes.c_uint, _errp]),
    "gonngpu_gemm_f16_sharded": (
        _c_int, [_vp, _c_long, _c_long, _c_long, _vp, _c_long, _vp, _vp, _vp, _c_int, _c_int, _c_int,
                 _c_long, _c_long, ctypes.c_uint, _vp, _c_long, _c_int, _errp]),
    "gonngpu_matmul_sharded": (
        _c_int, [_vp, _c_long, _c_long, _vp, _c_long, _c_long, _vp, _c_int, _c_int, _errp]),
    "gonngpu_shard_plan": (_c_int, [_c_long, _c_int, _c_int, ctypes.POINTER(_c_long), ctypes.POINTER(_c_long)]),
    "gonngpu_linear_backward": (
        _c_int, [_vp, _vp, _vp, _vp, _c_long, _c_long, _c_long, _vp, _vp, _vp, _errp]),
    "gonngpu_column_sum": (_c_int, [_vp, _c_long, _c_long, _vp, _errp]),
    "gonngpu_alloc_device_buffer": (_c_int, [_c_long, ctypes.POINTER(_vp), _errp]),
    "gonngpu_wrap_device_memory": (_c_int, [_vp, _c_long, ctypes.POINTER(_vp), _errp]),
    "gonngpu_device_address": (_vp, [_vp]),
    "gonngpu_upload": (_c_int, [_vp, _vp, _c_long, _errp]),
    "gonngpu_upload_f64": (_c_int, [_vp, _vp, _c_long, _errp]),
    "gonngpu_retrieve_f64": (_c_int, [_vp, _vp, _c_long, _errp]),
    "gonngpu_mark_modified": (_c_int, [_vp]),
    "gonngpu_host_alloc": (_vp, [_c_long]),
    "gonngpu_host_free": (None, [_vp]),
    "gonngpu_inject_fault": (_c_int, [ctypes.c_char_p, _c_int]),
    "gonngpu_device_count": (_c_int, []),
    "gonngpu_set_device": (_c_int, [_c_int]),
    "gonngpu_get_device": (_c_int, []),
    "gonngpu_stream": (_vp, []),
    "gonngpu_set_blocking": (_c_int, [_c_int]),
    "gonngpu_synchronize": (_c_int, [_errp]),
    "gonngpu_set_plane_cache": (_c_int, [_c_int]),
    "gonngpu_set_gemm_tuning": (_c_int, [_c_int, _c_int]),
    "gonngpu_set_gemm_pair_mode": (_c_int, [_c_int]),
    "gonngpu_set_gemm_split_k": (_c_int, [_c_int]),
    "gonngpu_set_sharded_tuning": (_c_int, [_c_int, _c_int]),
    "gonngpu_set_sharded_trace": (_c_int, [_vp]),
    "gonngpu_trim_cache": (_c_long, []),
    "gonngpu_get_stats": (None, [ctypes.POINTER(_c_long)]),
    "gonngpu_last_kernel_status": (None, [ctypes.POINTER(ctypes.c_uint)]),
    "gonngpu_version": (ctypes.c_char_p, []),
}


def lib():
    """Loads the shared library once and types every exported function."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is not built; run python go-nngpu_b200/build.py")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def _check(code, err):
    if code != 0:
        msg = ""
        if err.message:
            msg = ctypes.string_at(err.message).decode("utf-8", "replace")
            lib().free_c_error_message(err.message)
        raise GonnError(code, msg)


def _np_ptr(a):
    return a.ctypes.data_as(_vp)


class Buffer:
    """A GPUPtr handle.  `host` keeps the registered numpy array alive."""

    def __init__(self, handle, nbytes, host=None):
        self.handle = handle
        self.nbytes = nbytes
        self.host = host

    @classmethod
    def from_host(cls, array):
        """create_gpu_buffer over a C-contiguous float32 array (lazy upload)."""
        a = np.ascontiguousarray(array, dtype=np.float32)
        h, dev, err = _vp(), _vp(), CError()
        _check(lib().create_gpu_buffer(_np_ptr(a), a.nbytes, ctypes.byref(h), ctypes.byref(dev),
                                       ctypes.byref(err)), err)
        return cls(h, a.nbytes, a)

    @classmethod
    def empty(cls, nbytes):
        h, err = _vp(), CError()
        _check(lib().gonngpu_alloc_device_buffer(int(nbytes), ctypes.byref(h), ctypes.byref(err)), err)
        return cls(h, int(nbytes))

    @classmethod
    def wrap(cls, device_ptr, nbytes, keepalive=None):
        h, err = _vp(), CError()
        _check(lib().gonngpu_wrap_device_memory(_vp(device_ptr), int(nbytes), ctypes.byref(h),
                                                ctypes.byref(err)), err)
        return cls(h, int(nbytes), keepalive)

    def upload(self, array):
        a = np.ascontiguousarray(array, dtype=np.float32)
        err = CError()
        _check(lib().gonngpu_upload(self.handle, _np_ptr(a), a.nbytes, ctypes.byref(err)), err)

    def upload_f64(self, array):
        """float64 host data, narrowed to float32 on the device."""
        a = np.ascontiguousarray(array, dtype=np.float64)
        err = CError()
        _check(lib().gonngpu_upload_f64(self.handle, _np_ptr(a), a.size, ctypes.byref(err)), err)

    def retrieve_f64(self, shape, out=None):
        """The float32 contents widened to float64 on the device."""
        if out is None:
            out = np.empty(shape, dtype=np.float64)
        err = CError()
        _check(lib().gonngpu_retrieve_f64(self.handle, _np_ptr(out), out.size, ctypes.byref(err)), err)
        return out

    def retrieve(self, shape):
        out = np.empty(shape, dtype=np.float32)
        self.retrieve_into(out)
        return out

    def retrieve_into(self, out):
        err = CError()
        _check(lib().retrieve_gpu_buffer_data(self.handle, _np_ptr(out), out.nbytes, ctypes.byref(err)), err)

    def device_address(self):
        return lib().gonngpu_device_address(self.handle)

    def release(self):
        if self.handle:
            lib().release_gpu_buffer(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def matmul(a, a_shape, b, b_shape, c, c_shape):
    err = CError()
    _check(lib().perform_mps_matrix_multiplication(
        a.handle, a_shape[0], a_shape[1], b.handle, b_shape[0], b_shape[1], c.handle, c_shape[0],
        c_shape[1], None, ctypes.byref(err)), err)


def matmul_ex(a, a_shape, trans_a, b, b_shape, trans_b, c, c_shape, precision=FP32_3XTF32,
              alpha=1.0, beta=0.0, bias=None, act=ACT_NONE, act_param=0.0):
    err = CError()
    _check(lib().gonngpu_matmul_ex(
        a.handle, a_shape[0], a_shape[1], int(trans_a), b.handle, b_shape[0], b_shape[1],
        int(trans_b), c.handle, c_shape[0], c_shape[1], precision, alpha, beta,
        bias.handle if bias is not None else None, act, act_param, ctypes.byref(err)), err)


def transpose(inp, in_shape, out):
    err = CError()
    _check(lib().perform_mps_matrix_transpose(inp.handle, in_shape[0], in_shape[1], out.handle,
                                              in_shape[1], in_shape[0], None, ctypes.byref(err)), err)


def add_broadcast(a, a_shape, b, b_shape, c, c_shape):
    err = CError()
    _check(lib().perform_mps_matrix_add_broadcast(
        a.handle, a_shape[0], a_shape[1], b.handle, b_shape[0], b_shape[1], c.handle, c_shape[0],
        c_shape[1], None, ctypes.byref(err)), err)


def relu_forward(inp, size, out):
    err = CError()
    _check(lib().perform_activation_relu_forward(inp.handle, size, out.handle, None, ctypes.byref(err)), err)


def relu_backward(grad_out, act_out, size, grad_in):
    err = CError()
    _check(lib().perform_activation_relu_backward(grad_out.handle, act_out.handle, size,
                                                  grad_in.handle, None, ctypes.byref(err)), err)


def fused_linear_activation(x, batch, in_size, w, out_size, bias, act, alpha, y):
    err = CError()
    _check(lib().perform_fused_linear_activation(
        x.handle, batch, in_size, w.handle, out_size, bias.handle if bias is not None else None,
        act, alpha, y.handle, None, ctypes.byref(err)), err)


def optimized_gemm(a, b, c, m, n, k, alpha, beta):
    err = CError()
    _check(lib().perform_optimized_gemm(a.handle, b.handle, c.handle, m, n, k, alpha, beta, None,
                                        ctypes.byref(err)), err)


def gemm_f16_device(a_ptr, a_shape, a_pitch, trans_a, b_ptr, b_shape, b_pitch, trans_b, c_ptr, ldc,
                    alpha=1.0, beta=0.0, bias_ptr=None, act=ACT_NONE, act_param=0.0):
    """Raw device pointers (ints): fp16 operands as stored, float32 result."""
    err = CError()
    _check(lib().gonngpu_gemm_f16_device(
        _vp(a_ptr), a_shape[0], a_shape[1], a_pitch, int(trans_a), _vp(b_ptr), b_shape[0], b_shape[1],
        b_pitch, int(trans_b), _vp(c_ptr), ldc, alpha, beta, _vp(bias_ptr) if bias_ptr else None, act,
        act_param, ctypes.byref(err)), err)


def convert_f16_device(src_ptr, rows, cols, dst_ptr, dst_pitch, mode=FP16_RN):
    err = CError()
    _check(lib().gonngpu_convert_f16_device(_vp(src_ptr), rows, cols, _vp(dst_ptr), dst_pitch, mode,
                                            ctypes.byref(err)), err)


def replicate_send(src_ptr, dst_multicast_ptr, nbytes, bases_dev_ptr, world, rank, ctrl_offset, slot,
                   epoch, ack_needed, ctas=0, stream=None):
    """Owner of B: pushes `nbytes` from src to the multicast address of the slot (one copy per
    GPU of the group through NVSwitch) and publishes `epoch` on every rank.  `stream`: a
    cudaStream_t as an int, None = the library's stream."""
    err = CError()
    _check(lib().gonngpu_replicate_send(_vp(src_ptr), _vp(dst_multicast_ptr), nbytes, _vp(bases_dev_ptr),
                                        world, rank, ctrl_offset, slot, epoch, ack_needed, ctas,
                                        _vp(stream) if stream else None, ctypes.byref(err)), err)


def replicate_wait(bases_dev_ptr, world, owner, rank, ctrl_offset, slot, epoch, ack_value):
    """Every rank: acknowledges `ack_value` to the owner, then holds the stream until the slot
    holds `epoch`."""
    err = CError()
    _check(lib().gonngpu_replicate_wait(_vp(bases_dev_ptr), world, owner, rank, ctrl_offset, slot, epoch,
                                        ack_value, ctypes.byref(err)), err)


def gemm_f16_sharded(a_ptr, a_shape, a_pitch, b_src_ptr, b_cols, local_base, bases_dev_ptr, multicast_base,
                     world, owner, rank, slots_offset, ctrl_offset, epoch, c_ptr, ldc, first_group=0):
    """One rank's share of the row-sharded product; B travels inside the kernel."""
    err = CError()
    _check(lib().gonngpu_gemm_f16_sharded(
        _vp(a_ptr), a_shape[0], a_shape[1], a_pitch, _vp(b_src_ptr) if b_src_ptr else None, b_cols,
        _vp(local_base), _vp(bases_dev_ptr), _vp(multicast_base) if multicast_base else None, world, owner,
        rank, slots_offset, ctrl_offset, epoch, _vp(c_ptr), ldc, first_group, ctypes.byref(err)), err)


def matmul_sharded(A, B, C, precision=FP16_RN, n_devices=0):
    """Host float32 arrays in and out: A's rows split over the process's GPUs."""
    err = CError()
    _check(lib().gonngpu_matmul_sharded(_np_ptr(A), A.shape[0], A.shape[1], _np_ptr(B), B.shape[0], B.shape[1],
                                        _np_ptr(C), precision, n_devices, ctypes.byref(err)), err)


def shard_plan(rows, n_devices, device):
    lo, hi = _c_long(), _c_long()
    rc = lib().gonngpu_shard_plan(rows, n_devices, device, ctypes.byref(lo), ctypes.byref(hi))
    if rc != 0:
        raise GonnError(rc, "bad shard plan arguments")
    return lo.value, hi.value


def matmul_f16_static_scratch(a_ptr, a_shape, b_ptr, b_shape, c_ptr, stream=None):
    """float32 device pointers in, float32 device pointer out; allocates nothing."""
    err = CError()
    _check(lib().gonngpu_matmul_f16_static_scratch(
        _vp(a_ptr), a_shape[0], a_shape[1], _vp(b_ptr), b_shape[0], b_shape[1], _vp(c_ptr),
        _vp(stream) if stream else None, ctypes.byref(err)), err)


def linear_backward(x, w, dy, act_out, batch, in_size, out_size, dx=None, dw=None, db=None):
    err = CError()
    h = lambda b: b.handle if b is not None else None  # noqa: E731
    _check(lib().gonngpu_linear_backward(h(x), h(w), h(dy), h(act_out), batch, in_size, out_size,
                                         h(dx), h(dw), h(db), ctypes.byref(err)), err)


def elementwise(name, a, b, c, shape):
    """name in {add, subtract, element_multiply, element_divide}; equal shapes."""
    err = CError()
    fn = getattr(lib(), "perform_mps_matrix_" + name)
    _check(fn(a.handle, shape[0], shape[1], b.handle, shape[0], shape[1], c.handle, shape[0], shape[1],
              None, ctypes.byref(err)), err)


def scalar_op(name, a, shape, scalar, c):
    """name in {scalar_add, scalar_multiply}."""
    err = CError()
    fn = getattr(lib(), "perform_mps_matrix_" + name)
    _check(fn(a.handle, shape[0], shape[1], scalar, c.handle, None, ctypes.byref(err)), err)


def activation_forward(name, inp, size, out, alpha=None):
    """name in {sigmoid, tanh, swish, gelu, softmax_1d} or, with alpha, {leaky_relu, elu}."""
    err = CError()
    fn = getattr(lib(), f"perform_activation_{name}_forward")
    if alpha is None:
        _check(fn(inp.handle, size, out.handle, None, ctypes.byref(err)), err)
    else:
        _check(fn(inp.handle, size, alpha, out.handle, None, ctypes.byref(err)), err)


def activation_backward(name, grad_out, act_out, size, grad_in, alpha=None):
    err = CError()
    fn = getattr(lib(), f"perform_activation_{name}_backward")
    if alpha is None:
        _check(fn(grad_out.handle, act_out.handle, size, grad_in.handle, None, ctypes.byref(err)), err)
    else:
        _check(fn(grad_out.handle, act_out.handle, size, alpha, grad_in.handle, None, ctypes.byref(err)), err)


def softmax_2d(inp, batch, features, out):
    err = CError()
    _check(lib().perform_activation_softmax_2d_forward(inp.handle, batch, features, out.handle, None,
                                                       ctypes.byref(err)), err)


def softmax_2d_backward(grad_out, act_out, batch, features, grad_in):
    err = CError()
    _check(lib().perform_activation_softmax_2d_backward(grad_out.handle, act_out.handle, batch, features,
                                                        grad_in.handle, None, ctypes.byref(err)), err)


def batch_matmul(a, b, c, batch, m, n, k):
    err = CError()
    _check(lib().perform_batch_matmul_optimized(a.handle, b.handle, c.handle, batch, m, n, k, None,
                                                ctypes.byref(err)), err)


def column_sum(inp, rows, cols, out):
    err = CError()
    _check(lib().gonngpu_column_sum(inp.handle, rows, cols, out.handle, ctypes.byref(err)), err)


def synchronize():
    err = CError()
    _check(lib().gonngpu_synchronize(ctypes.byref(err)), err)


def stats():
    out = (_c_long * 8)()
    lib().gonngpu_get_stats(out)
    keys = ["hbm_bytes", "h2d_bytes", "d2h_bytes", "kernel_launches", "gemm_launches", "buffers",
            "plane_bytes", "cached_bytes"]
    return dict(zip(keys, list(out)))


def last_kernel_status():
    out = (ctypes.c_uint * 4)()
    lib().gonngpu_last_kernel_status(out)
    return list(out)


def pinned_array(shape, dtype=np.float32):
    """numpy array over page-locked memory from gonngpu_host_alloc."""
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = lib().gonngpu_host_alloc(max(n, 1))
    if not p:
        raise MemoryError("gonngpu_host_alloc failed")
    buf = (ctypes.c_char * max(n, 1)).from_address(p)
    arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
    return arr, p
