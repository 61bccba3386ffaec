"""ctypes binding of the C ABI in include/catlass_b200.h.

Used by the tests and the benchmark to call the library exactly as a C caller would: PODs, raw device
pointers, a stream handle.  Loading fails loudly when the shared object is missing; nothing here computes.
"""
import ctypes
import os

from . import build as _build

SUCCESS, INVALID, CUDA_ERROR, DEVICE_TIMEOUT, SCRATCH_TOO_SMALL = 0, 1, 2, 3, 4
ROW_MAJOR, COLUMN_MAJOR, ZN = 0, 1, 2
GROUP_LIST_INT64, GROUP_LIST_INT32 = 0, 1
DTYPE_F32, DTYPE_BF16, DTYPE_F16, DTYPE_F32_IN_U64 = 0, 1, 2, 3
FLAG_STATIC_WEIGHTS = 2
QUANT_PER_TENSOR, QUANT_PER_CHANNEL = 0, 1

_u32, _u64, _vp = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p


class QuantMatmulArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("layout_a", _u32), ("layout_b", _u32),
        ("a", _vp), ("b", _vp), ("scale", _vp), ("per_token_scale", _vp), ("d", _vp), ("acc", _vp),
        ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("flags", _u32),
        ("scale_type", _u32), ("d_type", _u32),
    ]


class GroupedQuantMatmulArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_count", _u32), ("layout_b", _u32),
        ("group_list_type", _u32),
        ("a", _vp), ("b", _vp), ("group_list", _vp), ("scale", _vp), ("per_token_scale", _vp), ("d", _vp),
        ("acc", _vp), ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("flags", _u32),
        ("scale_type", _u32), ("d_type", _u32),
    ]


class GroupedSliceKArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_count", _u32), ("group_list_type", _u32), ("scale_type", _u32),
        ("a", _vp), ("b", _vp), ("group_list", _vp), ("scale", _vp), ("per_token_scale", _vp), ("d", _vp),
        ("acc", _vp), ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("d_type", _u32),
    ]


class GroupedFixpipeDequantArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_count", _u32), ("layout_b", _u32),
        ("group_list_type", _u32), ("quant_mode", _u32), ("scale_per_tensor", ctypes.c_float),
        ("a", _vp), ("b", _vp), ("group_list", _vp), ("per_channel_scale", _vp), ("d", _vp), ("acc", _vp),
        ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("per_channel_scale_type", _u32),
        ("d_type", _u32), ("flags", _u32),
    ]


class GroupedQuantMatmulHostArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_count", _u32), ("layout_b", _u32), ("chunks", _u32),
        ("a_host", _vp), ("group_list_host", _vp), ("per_token_host", _vp), ("d_host", _vp),
        ("b", _vp), ("scale", _vp), ("workspace", _vp), ("workspace_bytes", _u64),
    ]


class W4A8MatmulArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_size", _u32),
        ("a", _vp), ("w_packed", _vp), ("weight_scale", _vp), ("per_token_scale", _vp), ("d", _vp),
        ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("flags", _u32),
        ("d_type", _u32), ("pack_axis", _u32),
    ]


class MxMatmulArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("format", _u32), ("layout_a", _u32), ("layout_b", _u32),
        ("a", _vp), ("b", _vp), ("scale_a", _vp), ("scale_b", _vp), ("d", _vp),
        ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("flags", _u32),
    ]


class MxGroupedMatmulArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_count", _u32), ("format", _u32), ("layout_b", _u32),
        ("group_list_type", _u32), ("group_list_kind", _u32),
        ("a", _vp), ("b", _vp), ("group_list", _vp), ("scale_a", _vp), ("scale_b", _vp), ("d", _vp),
        ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("flags", _u32),
    ]


GROUP_LIST_SIZES, GROUP_LIST_PREFIX_SUMS = 0, 1


class MxGroupedSwigluQuantArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_count", _u32), ("layout_b", _u32),
        ("group_list_type", _u32), ("group_list_kind", _u32), ("flags", _u32),
        ("a", _vp), ("b", _vp), ("group_list", _vp), ("scale_a", _vp), ("scale_b", _vp), ("q", _vp), ("q_scale", _vp),
        ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("reserved", _u32),
    ]


class QuantizeInt8Args(ctypes.Structure):
    _fields_ = [("rows", _u32), ("k", _u32), ("x_type", _u32), ("reserved", _u32), ("x_pitch", _u64), ("x", _vp),
                ("q", _vp), ("scale", _vp)]


class MxQuantizeArgs(ctypes.Structure):
    _fields_ = [
        ("rows", _u32), ("k", _u32), ("format", _u32), ("x_type", _u32), ("x_pitch", _u64),
        ("x", _vp), ("q", _vp), ("scale", _vp),
    ]


class MxGroupedFinalizeRoutingArgs(ctypes.Structure):
    _fields_ = [
        ("m", _u32), ("n", _u32), ("k", _u32), ("group_count", _u32), ("layout_b", _u32),
        ("group_list_type", _u32), ("group_list_kind", _u32), ("row_index_type", _u32), ("batch", _u32),
        ("shared_rows", _u32), ("shared_offset", _u32), ("shared_weight", ctypes.c_float),
        ("a", _vp), ("b", _vp), ("group_list", _vp), ("scale_a", _vp), ("scale_b", _vp), ("logit", _vp),
        ("row_index", _vp), ("bias", _vp), ("shared_input", _vp), ("out", _vp),
        ("workspace", _vp), ("workspace_bytes", _u64), ("block_num", _u32), ("flags", _u32),
    ]


MX_E4M3, MX_E2M1 = 0, 1
MX_OUT_F32 = 1
W4_PACKED_ALONG_K, W4_PACKED_ALONG_N = 0, 1

_lib = None


def library_path():
    return _build.LIB_PATH


def load():
    """The loaded shared library. Raises if it has not been built (python -m catlass_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m catlass_b200.build` (needs nvcc). "
            "There is no fallback path.")
    lib = ctypes.CDLL(path)
    for name, args_t in (("cb200_quant_matmul", QuantMatmulArgs),
                         ("cb200_grouped_quant_matmul_slice_m", GroupedQuantMatmulArgs),
                         ("cb200_grouped_matmul_slice_m_fixpipe_dequant", GroupedFixpipeDequantArgs),
                         ("cb200_grouped_quant_matmul_slice_k", GroupedSliceKArgs),
                         ("cb200_w4a8_matmul", W4A8MatmulArgs),
                         ("cb200_mx_matmul", MxMatmulArgs),
                         ("cb200_mx_grouped_matmul_slice_m", MxGroupedMatmulArgs),
                         ("cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant", MxGroupedSwigluQuantArgs),
                         ("cb200_mx_grouped_matmul_finalize_routing", MxGroupedFinalizeRoutingArgs)):
        getattr(lib, name + "_can_implement").argtypes = [ctypes.POINTER(args_t)]
        getattr(lib, name + "_can_implement").restype = ctypes.c_int
        getattr(lib, name + "_workspace_size").argtypes = [ctypes.POINTER(args_t)]
        getattr(lib, name + "_workspace_size").restype = _u64
        getattr(lib, name).argtypes = [ctypes.POINTER(args_t), _vp]
        getattr(lib, name).restype = ctypes.c_int
    lib.cb200_grouped_quant_matmul_slice_m_host.argtypes = [ctypes.POINTER(GroupedQuantMatmulHostArgs), _vp]
    lib.cb200_grouped_quant_matmul_slice_m_host.restype = ctypes.c_int
    lib.cb200_grouped_quant_matmul_slice_m_host_workspace_size.argtypes = [ctypes.POINTER(GroupedQuantMatmulHostArgs)]
    lib.cb200_grouped_quant_matmul_slice_m_host_workspace_size.restype = _u64
    lib.cb200_mx_quantize.argtypes = [ctypes.POINTER(MxQuantizeArgs), _vp]
    lib.cb200_mx_quantize.restype = ctypes.c_int
    lib.cb200_mx_quantize_can_implement.argtypes = [ctypes.POINTER(MxQuantizeArgs)]
    lib.cb200_mx_quantize_can_implement.restype = ctypes.c_int
    lib.cb200_quantize_per_token_int8.argtypes = [ctypes.POINTER(QuantizeInt8Args), _vp]
    lib.cb200_quantize_per_token_int8.restype = ctypes.c_int
    lib.cb200_quantize_per_token_int8_can_implement.argtypes = [ctypes.POINTER(QuantizeInt8Args)]
    lib.cb200_quantize_per_token_int8_can_implement.restype = ctypes.c_int
    lib.cb200_mx_matmul_static.argtypes = [ctypes.POINTER(MxMatmulArgs), _vp]
    lib.cb200_mx_matmul_static.restype = ctypes.c_int
    lib.cb200_mx_matmul_static_scratch_bytes.restype = _u64
    lib.cb200_selftest_wait_timeout.argtypes = [_u32, _vp]
    lib.cb200_selftest_wait_timeout.restype = ctypes.c_int
    lib.cb200_device_status.argtypes = [ctypes.POINTER(_u32)]
    lib.cb200_device_status.restype = ctypes.c_int
    lib.cb200_last_cuda_error.restype = ctypes.c_int
    lib.cb200_launch_count.restype = _u64
    lib.cb200_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


class CallError(RuntimeError):
    def __init__(self, what, status):
        super().__init__(f"{what} returned status {status} (cuda error {load().cb200_last_cuda_error()})")
        self.status = status


def _check(what, status):
    if status != SUCCESS:
        raise CallError(what, status)


def device_status():
    """(status, code): synchronises the device and reads the kernels' status word."""
    code = _u32(0)
    st = load().cb200_device_status(ctypes.byref(code))
    return st, code.value


def launch_count():
    return int(load().cb200_launch_count())


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(stream):
    if stream is None:
        import torch
        stream = torch.cuda.current_stream()
    return ctypes.c_void_p(stream.cuda_stream)


def quant_matmul(a, b, scale, per_token, d, m, n, k, layout_b=COLUMN_MAJOR, acc=None, stream=None,
                 block_num=0, layout_a=ROW_MAJOR, scale_type=DTYPE_F32, d_type=DTYPE_BF16, static_weights=False):
    """Enqueue the dense W8A8 dequant matmul. Arguments are torch CUDA tensors used as raw buffers."""
    args = QuantMatmulArgs(m=m, n=n, k=k, layout_a=layout_a, layout_b=layout_b, a=_p(a), b=_p(b),
                           scale=_p(scale), per_token_scale=_p(per_token), d=_p(d), acc=_p(acc),
                           workspace=None, workspace_bytes=0, block_num=block_num,
                           flags=FLAG_STATIC_WEIGHTS if static_weights else 0, scale_type=scale_type, d_type=d_type)
    _check("cb200_quant_matmul", load().cb200_quant_matmul(ctypes.byref(args), _stream(stream)))


def grouped_quant_matmul(a, b, group_list, scale, per_token, d, m, n, k, group_count, layout_b=ROW_MAJOR,
                         acc=None, stream=None, block_num=0, group_list_type=GROUP_LIST_INT64,
                         scale_type=DTYPE_F32, d_type=DTYPE_BF16):
    args = GroupedQuantMatmulArgs(m=m, n=n, k=k, group_count=group_count, layout_b=layout_b,
                                  group_list_type=group_list_type, a=_p(a), b=_p(b),
                                  group_list=_p(group_list), scale=_p(scale), per_token_scale=_p(per_token),
                                  d=_p(d), acc=_p(acc), workspace=None, workspace_bytes=0,
                                  block_num=block_num, flags=0, scale_type=scale_type, d_type=d_type)
    _check("cb200_grouped_quant_matmul_slice_m",
           load().cb200_grouped_quant_matmul_slice_m(ctypes.byref(args), _stream(stream)))


def grouped_fixpipe_dequant(a, b, group_list, d, m, n, k, group_count, quant_mode, scale_per_tensor=1.0,
                            per_channel_scale=None, per_channel_scale_type=DTYPE_F32, layout_b=ROW_MAJOR,
                            d_type=DTYPE_F16, acc=None, stream=None, group_list_type=GROUP_LIST_INT64):
    """Grouped slice-M W8A8 with per-tensor (quant_mode 0) or per-channel (1) dequant, no per-token factor."""
    args = GroupedFixpipeDequantArgs(m=m, n=n, k=k, group_count=group_count, layout_b=layout_b,
                                     group_list_type=group_list_type, quant_mode=quant_mode,
                                     scale_per_tensor=scale_per_tensor, a=_p(a), b=_p(b), group_list=_p(group_list),
                                     per_channel_scale=_p(per_channel_scale), d=_p(d), acc=_p(acc), workspace=None,
                                     workspace_bytes=0, block_num=0, per_channel_scale_type=per_channel_scale_type,
                                     d_type=d_type, flags=0)
    _check("cb200_grouped_matmul_slice_m_fixpipe_dequant",
           load().cb200_grouped_matmul_slice_m_fixpipe_dequant(ctypes.byref(args), _stream(stream)))


def grouped_quant_matmul_slice_k_workspace_size(m, n, k, group_count):
    args = GroupedSliceKArgs(m=m, n=n, k=k, group_count=group_count, a=256, b=256, group_list=256, scale=256,
                             per_token_scale=256, d=256)
    return int(load().cb200_grouped_quant_matmul_slice_k_workspace_size(ctypes.byref(args)))


def grouped_quant_matmul_slice_k(a, b, group_list, scale, per_token, d, m, n, k, group_count, workspace, acc=None,
                                 stream=None, group_list_type=GROUP_LIST_INT64, scale_type=DTYPE_F32,
                                 d_type=DTYPE_BF16, block_num=0):
    """Grouped slice-K W8A8: a [k][m] (A column-major), b [k][n], group_list prefix sums over K, scale [G][n],
    per_token [G][m], d [G][m][n]."""
    args = GroupedSliceKArgs(m=m, n=n, k=k, group_count=group_count, group_list_type=group_list_type,
                             scale_type=scale_type, a=_p(a), b=_p(b), group_list=_p(group_list), scale=_p(scale),
                             per_token_scale=_p(per_token), d=_p(d), acc=_p(acc), workspace=_p(workspace),
                             workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size(),
                             block_num=block_num, d_type=d_type)
    _check("cb200_grouped_quant_matmul_slice_k",
           load().cb200_grouped_quant_matmul_slice_k(ctypes.byref(args), _stream(stream)))


W4A8_SPLIT_K = 1  # flags: split the K range over a CTA cluster (faster, fp32 sums reassociated)


def _w4a8_args(a, w_packed, weight_scale, per_token, d, m, n, k, group_size, flags, d_type, pack_axis, workspace):
    return W4A8MatmulArgs(m=m, n=n, k=k, group_size=group_size, a=_p(a), w_packed=_p(w_packed),
                          weight_scale=_p(weight_scale), per_token_scale=_p(per_token), d=_p(d),
                          workspace=_p(workspace),
                          workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size(),
                          block_num=0, flags=flags, d_type=d_type, pack_axis=pack_axis)


def w4a8_matmul_workspace_size(m, n, k, group_size, pack_axis=W4_PACKED_ALONG_K, aligned=True):
    """Bytes the call needs (0 on the fast path). `aligned`: the operand pointers are 16-byte aligned."""
    ptr = 256 if aligned else 257
    args = W4A8MatmulArgs(m=m, n=n, k=k, group_size=group_size, a=ptr, w_packed=ptr, weight_scale=256,
                          per_token_scale=256, d=256, pack_axis=pack_axis)
    return int(load().cb200_w4a8_matmul_workspace_size(ctypes.byref(args)))


def w4a8_matmul(a, w_packed, weight_scale, per_token, d, m, n, k, group_size, stream=None, split_k=False,
                static_weights=False, d_type=DTYPE_BF16, pack_axis=W4_PACKED_ALONG_K, workspace=None):
    flags = (W4A8_SPLIT_K if split_k else 0) | (FLAG_STATIC_WEIGHTS if static_weights else 0)
    args = _w4a8_args(a, w_packed, weight_scale, per_token, d, m, n, k, group_size, flags, d_type, pack_axis, workspace)
    _check("cb200_w4a8_matmul", load().cb200_w4a8_matmul(ctypes.byref(args), _stream(stream)))


def _mx_args(a, b, scale_a, scale_b, d, m, n, k, fmt, workspace, layout_a, layout_b, out_f32):
    return MxMatmulArgs(m=m, n=n, k=k, format=fmt, layout_a=layout_a, layout_b=layout_b, a=_p(a), b=_p(b),
                        scale_a=_p(scale_a), scale_b=_p(scale_b), d=_p(d), workspace=_p(workspace),
                        workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size(),
                        block_num=0, flags=MX_OUT_F32 if out_f32 else 0)


def mx_matmul_workspace_size(m, n, k, fmt, layout_a=ROW_MAJOR, layout_b=COLUMN_MAJOR):
    args = MxMatmulArgs(m=m, n=n, k=k, format=fmt, layout_a=layout_a, layout_b=layout_b, a=256, b=256,
                        scale_a=256, scale_b=256, d=256)
    return int(load().cb200_mx_matmul_workspace_size(ctypes.byref(args)))


def mx_matmul(a, b, scale_a, scale_b, d, m, n, k, fmt, workspace, stream=None, layout_a=ROW_MAJOR,
              layout_b=COLUMN_MAJOR, out_f32=False):
    """a: [m][k] elements, or [k][m] with layout_a = COLUMN_MAJOR; b: [n][k] (column-major B), or [k][n] with
    layout_b = ROW_MAJOR; E2M1: two elements per byte along the contiguous axis.  Scales follow the operand:
    [rows][KS] bytes, or [KS/2][rows][2] for an operand stored with k first (KS = even number of 32-blocks).
    workspace: a CUDA byte tensor of at least mx_matmul_workspace_size bytes."""
    args = _mx_args(a, b, scale_a, scale_b, d, m, n, k, fmt, workspace, layout_a, layout_b, out_f32)
    _check("cb200_mx_matmul", load().cb200_mx_matmul(ctypes.byref(args), _stream(stream)))


def mx_matmul_static(a, b, scale_a, scale_b, d, m, n, k, fmt, stream=None, layout_a=ROW_MAJOR,
                     layout_b=COLUMN_MAJOR, out_f32=False):
    """cb200_mx_matmul_static: as mx_matmul, scratch inside the library image, no workspace argument."""
    args = _mx_args(a, b, scale_a, scale_b, d, m, n, k, fmt, None, layout_a, layout_b, out_f32)
    _check("cb200_mx_matmul_static", load().cb200_mx_matmul_static(ctypes.byref(args), _stream(stream)))


def _mx_grouped_args(a, b, group_list, scale_a, scale_b, d, m, n, k, group_count, fmt, workspace, layout_b,
                     group_list_type, group_list_kind, out_f32):
    return MxGroupedMatmulArgs(m=m, n=n, k=k, group_count=group_count, format=fmt, layout_b=layout_b,
                               group_list_type=group_list_type, group_list_kind=group_list_kind, a=_p(a), b=_p(b),
                               group_list=_p(group_list), scale_a=_p(scale_a), scale_b=_p(scale_b), d=_p(d),
                               workspace=_p(workspace),
                               workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size(),
                               block_num=0, flags=MX_OUT_F32 if out_f32 else 0)


def mx_grouped_matmul_workspace_size(m, n, k, group_count, fmt, layout_b=COLUMN_MAJOR):
    args = MxGroupedMatmulArgs(m=m, n=n, k=k, group_count=group_count, format=fmt, layout_b=layout_b, a=256, b=256,
                               group_list=256, scale_a=256, scale_b=256, d=256)
    return int(load().cb200_mx_grouped_matmul_slice_m_workspace_size(ctypes.byref(args)))


def mx_grouped_matmul(a, b, group_list, scale_a, scale_b, d, m, n, k, group_count, fmt, workspace, stream=None,
                      layout_b=COLUMN_MAJOR, group_list_type=GROUP_LIST_INT64, group_list_kind=GROUP_LIST_SIZES,
                      out_f32=False):
    """Grouped slice-M MX matmul: a [m][k], b [G][n][k] (or [G][k][n] with layout_b = ROW_MAJOR), group_list the
    groups' row counts (or prefix sums), scales as for mx_matmul with a leading group axis on scale_b."""
    args = _mx_grouped_args(a, b, group_list, scale_a, scale_b, d, m, n, k, group_count, fmt, workspace, layout_b,
                            group_list_type, group_list_kind, out_f32)
    _check("cb200_mx_grouped_matmul_slice_m",
           load().cb200_mx_grouped_matmul_slice_m(ctypes.byref(args), _stream(stream)))


def mx_grouped_swiglu_quant_workspace_size(m, n, k, group_count, layout_b=COLUMN_MAJOR):
    args = MxGroupedSwigluQuantArgs(m=m, n=n, k=k, group_count=group_count, layout_b=layout_b, a=256, b=256,
                                    group_list=256, scale_a=256, scale_b=256, q=256, q_scale=256)
    return int(load().cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_workspace_size(ctypes.byref(args)))


def mx_grouped_swiglu_quant(a, b, group_list, scale_a, scale_b, q, q_scale, m, n, k, group_count, workspace,
                            stream=None, layout_b=COLUMN_MAJOR, group_list_type=GROUP_LIST_INT64,
                            group_list_kind=GROUP_LIST_SIZES):
    """Grouped slice-M MXFP8 matmul + SwiGLU + MX quantisation: q [m][n/2] E4M3 bytes, q_scale [m][n/64] E8M0."""
    args = MxGroupedSwigluQuantArgs(
        m=m, n=n, k=k, group_count=group_count, layout_b=layout_b, group_list_type=group_list_type,
        group_list_kind=group_list_kind, flags=0, a=_p(a), b=_p(b), group_list=_p(group_list), scale_a=_p(scale_a),
        scale_b=_p(scale_b), q=_p(q), q_scale=_p(q_scale), workspace=_p(workspace),
        workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size(), block_num=0)
    _check("cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant",
           load().cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant(ctypes.byref(args), _stream(stream)))


ROUTING_DETERMINISTIC = 1


def mx_grouped_finalize_routing_workspace_size(m, n, k, group_count, batch, layout_b=COLUMN_MAJOR, deterministic=False):
    args = MxGroupedFinalizeRoutingArgs(m=m, n=n, k=k, group_count=group_count, layout_b=layout_b, batch=batch, a=256,
                                        b=256, group_list=256, scale_a=256, scale_b=256, logit=256, row_index=256,
                                        out=256, flags=ROUTING_DETERMINISTIC if deterministic else 0)
    return int(load().cb200_mx_grouped_matmul_finalize_routing_workspace_size(ctypes.byref(args)))


def mx_grouped_finalize_routing(a, b, group_list, scale_a, scale_b, logit, row_index, out, m, n, k, group_count, batch,
                                workspace, bias=None, shared_input=None, shared_rows=0, shared_offset=0,
                                shared_weight=0.0, stream=None, layout_b=COLUMN_MAJOR,
                                group_list_type=GROUP_LIST_INT64, group_list_kind=GROUP_LIST_SIZES,
                                row_index_type=GROUP_LIST_INT64, deterministic=False):
    """Grouped slice-M MXFP8 matmul + finalize routing: out [batch][n] fp32 = shared contribution +
    sum over rows p of logit[p] * (C[p] + bias[group]) at row row_index[p]."""
    args = MxGroupedFinalizeRoutingArgs(
        m=m, n=n, k=k, group_count=group_count, layout_b=layout_b, group_list_type=group_list_type,
        group_list_kind=group_list_kind, row_index_type=row_index_type, batch=batch, shared_rows=shared_rows,
        shared_offset=shared_offset, shared_weight=shared_weight, a=_p(a), b=_p(b), group_list=_p(group_list),
        scale_a=_p(scale_a), scale_b=_p(scale_b), logit=_p(logit), row_index=_p(row_index), bias=_p(bias),
        shared_input=_p(shared_input), out=_p(out), workspace=_p(workspace),
        workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size(), block_num=0,
        flags=ROUTING_DETERMINISTIC if deterministic else 0)
    _check("cb200_mx_grouped_matmul_finalize_routing",
           load().cb200_mx_grouped_matmul_finalize_routing(ctypes.byref(args), _stream(stream)))


def mx_quantize(x, q, scale, rows, k, fmt, x_type=DTYPE_F32, x_pitch=0, stream=None):
    """x: fp32 / bf16 [rows][k] -> q codes ([rows][k] bytes, E2M1 [rows][ceil(k/2)]) and scale [rows][KS] bytes."""
    args = MxQuantizeArgs(rows=rows, k=k, format=fmt, x_type=x_type, x_pitch=x_pitch, x=_p(x), q=_p(q), scale=_p(scale))
    _check("cb200_mx_quantize", load().cb200_mx_quantize(ctypes.byref(args), _stream(stream)))


def _host_args(a_host, group_list_host, per_token_host, d_host, b, scale, m, n, k, group_count, layout_b, chunks,
               workspace):
    return GroupedQuantMatmulHostArgs(
        m=m, n=n, k=k, group_count=group_count, layout_b=layout_b, chunks=chunks, a_host=_p(a_host),
        group_list_host=_p(group_list_host), per_token_host=_p(per_token_host), d_host=_p(d_host), b=_p(b),
        scale=_p(scale), workspace=_p(workspace),
        workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size())


def grouped_quant_matmul_host_workspace_size(m, n, k, group_count, chunks=0):
    args = GroupedQuantMatmulHostArgs(m=m, n=n, k=k, group_count=group_count, layout_b=ROW_MAJOR, chunks=chunks)
    return int(load().cb200_grouped_quant_matmul_slice_m_host_workspace_size(ctypes.byref(args)))


def grouped_quant_matmul_host(a_host, group_list_host, per_token_host, d_host, b, scale, m, n, k, group_count,
                              workspace, layout_b=ROW_MAJOR, chunks=0, stream=None):
    """Host-resident A / per-token scales / int64 group list / D (CPU tensors, pinned for overlap); b, scale and
    workspace are CUDA tensors."""
    args = _host_args(a_host, group_list_host, per_token_host, d_host, b, scale, m, n, k, group_count, layout_b,
                      chunks, workspace)
    _check("cb200_grouped_quant_matmul_slice_m_host",
           load().cb200_grouped_quant_matmul_slice_m_host(ctypes.byref(args), _stream(stream)))


def quantize_per_token_int8(x, q, scale, rows, k, x_type=DTYPE_F32, x_pitch=0, stream=None):
    """x: fp32 / bf16 [rows][k] -> q int8 [rows][k] and scale fp32 [rows] (amax / 127), the A operand and the
    per-token scale of the W8A8 entry points."""
    args = QuantizeInt8Args(rows=rows, k=k, x_type=x_type, reserved=0, x_pitch=x_pitch, x=_p(x), q=_p(q), scale=_p(scale))
    _check("cb200_quantize_per_token_int8", load().cb200_quantize_per_token_int8(ctypes.byref(args), _stream(stream)))

