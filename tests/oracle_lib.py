"""ctypes bindings of the CPU oracle (oracle/liboracle.so) and, when it was built, of the reference's own
golden (oracle/_ref/libref.so).  Test infrastructure: imported by the tests, the smoke check and the CPU
baseline leg of the bench only."""
import ctypes
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ORACLE_DIR = os.path.join(_ROOT, "oracle")

ROW_MAJOR = 0
COL_MAJOR = 1
MX_E4M3 = 0
MX_E2M1 = 1

_c_u32 = ctypes.c_uint32
_p = ctypes.c_void_p


def _ptr(a):
    return a.ctypes.data_as(_p) if a is not None else None


def build_oracle():
    """Compile the oracle (and the reference golden when the reference tree is present)."""
    subprocess.run(["make", "-s", "-C", _ORACLE_DIR], check=True, stdout=subprocess.DEVNULL)


def _load(path):
    return ctypes.CDLL(path)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_ORACLE_DIR, "liboracle.so")
        if not os.path.exists(path):
            build_oracle()
        _lib = _load(path)
        _lib.orc_bf16_rne.restype = ctypes.c_uint16
        _lib.orc_bf16_rne.argtypes = [ctypes.c_float]
        _lib.orc_f16_rne.restype = ctypes.c_uint16
        _lib.orc_f16_rne.argtypes = [ctypes.c_float]
        for name in ("orc_e4m3_to_float", "orc_e2m1_to_float", "orc_e8m0_to_float"):
            getattr(_lib, name).restype = ctypes.c_float
            getattr(_lib, name).argtypes = [ctypes.c_uint8]
        _lib.orc_e4m3_rne_sat.restype = ctypes.c_uint8
        _lib.orc_e4m3_rne_sat.argtypes = [ctypes.c_float]
    return _lib


def ref():
    """The reference's own golden, or None when it was not built (no reference tree at build time)."""
    global _ref
    if _ref is None:
        path = os.path.join(_ORACLE_DIR, "_ref", "libref.so")
        if not os.path.exists(path):
            return None
        _ref = _load(path)
        _ref.ref_layout_offset.restype = ctypes.c_int64
        _ref.ref_layout_capacity.restype = ctypes.c_int64
    return _ref


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def quant_matmul(a, b, scale, per_token, m, n, k, layout_a=ROW_MAJOR, layout_b=COL_MAJOR, want_acc=False):
    """a, b: flat int8 buffers in the stated layouts. Returns fp32 out [m,n] (and int32 acc [m,n])."""
    a, b = _c(a, np.int8), _c(b, np.int8)
    scale, per_token = _c(scale, np.float32), _c(per_token, np.float32)
    out = np.empty((m, n), np.float32)
    acc = np.empty((m, n), np.int32) if want_acc else None
    lib().orc_quant_matmul(_c_u32(m), _c_u32(n), _c_u32(k), _ptr(a), layout_a, _ptr(b), layout_b,
                           _ptr(scale), _ptr(per_token), _ptr(out), _ptr(acc))
    return (out, acc) if want_acc else out


def grouped_quant_matmul(a, b, group_list, scale, per_token, m, n, k, layout_b=ROW_MAJOR, want_acc=False,
                         out_init=None):
    a, b = _c(a, np.int8), _c(b, np.int8)
    gl = _c(group_list, np.int64)
    scale, per_token = _c(scale, np.float32), _c(per_token, np.float32)
    out = np.zeros((m, n), np.float32) if out_init is None else _c(out_init, np.float32).copy()
    acc = np.zeros((m, n), np.int32) if want_acc else None
    lib().orc_grouped_quant_matmul_slice_m(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(len(gl)), _ptr(gl),
                                           _ptr(a), _ptr(b), layout_b, _ptr(scale), _ptr(per_token),
                                           _ptr(out), _ptr(acc))
    return (out, acc) if want_acc else out


def grouped_fixpipe_dequant(a, b, group_list, quant_mode, scale_per_tensor, per_channel_scale, m, n, k,
                            layout_b=ROW_MAJOR, want_acc=False, out_init=None):
    """Per-tensor (quant_mode 0) / per-channel (1) grouped dequant golden. Returns fp32 out [m, n]."""
    a, b = _c(a, np.int8), _c(b, np.int8)
    gl = _c(group_list, np.int64)
    pcs = _c(per_channel_scale, np.float32) if per_channel_scale is not None else None
    out = np.zeros((m, n), np.float32) if out_init is None else _c(out_init, np.float32).copy()
    acc = np.zeros((m, n), np.int32) if want_acc else None
    lib().orc_grouped_matmul_fixpipe_dequant(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(len(gl)), _ptr(gl), _ptr(a),
                                             _ptr(b), layout_b, int(quant_mode), ctypes.c_float(scale_per_tensor),
                                             _ptr(pcs), _ptr(out), _ptr(acc))
    return (out, acc) if want_acc else out


def grouped_quant_matmul_slice_k(a, b, group_list, scale, per_token, m, n, k, want_acc=False):
    """a: column-major m x k ([k][m] bytes), b: row-major k x n; groups along K. Returns fp32 [G, m, n]."""
    a, b = _c(a, np.int8), _c(b, np.int8)
    gl = _c(group_list, np.int64)
    scale, per_token = _c(scale, np.float32), _c(per_token, np.float32)
    out = np.zeros((len(gl), m, n), np.float32)
    acc = np.zeros((len(gl), m, n), np.int32) if want_acc else None
    lib().orc_grouped_quant_matmul_slice_k(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(len(gl)), _ptr(gl), _ptr(a),
                                           _ptr(b), _ptr(scale), _ptr(per_token), _ptr(out), _ptr(acc))
    return (out, acc) if want_acc else out


def w4a8_per_group_readings(a, w_packed, sw, sa, m, n, k, group_size):
    """(unfused fp32 result, exact result in float64, sum of |group terms| * |sa|) of the per-group formula."""
    a, w_packed = _c(a, np.int8), _c(w_packed, np.uint8)
    sw, sa = _c(sw, np.float32), _c(sa, np.float32)
    unfused = np.empty((m, n), np.float32)
    exact = np.empty((m, n), np.float64)
    mag = np.empty((m, n), np.float64)
    lib().orc_w4a8_matmul_per_group_readings(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(group_size), _ptr(a),
                                             _ptr(w_packed), _ptr(sw), _ptr(sa), _ptr(unfused), _ptr(exact),
                                             _ptr(mag))
    return unfused, exact, mag


def w4a8_per_group(a, w_packed, sw, sa, m, n, k, group_size):
    a, w_packed = _c(a, np.int8), _c(w_packed, np.uint8)
    sw, sa = _c(sw, np.float32), _c(sa, np.float32)
    out = np.empty((m, n), np.float32)
    lib().orc_w4a8_matmul_per_group(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(group_size), _ptr(a),
                                    _ptr(w_packed), _ptr(sw), _ptr(sa), _ptr(out))
    return out


def w4a8_per_tensor(a, w_packed, scalar, m, n, k):
    a, w_packed = _c(a, np.int8), _c(w_packed, np.uint8)
    out = np.empty((m, n), np.float32)
    lib().orc_w4a8_matmul_per_tensor(_c_u32(m), _c_u32(n), _c_u32(k), _ptr(a), _ptr(w_packed),
                                     ctypes.c_float(scalar), _ptr(out))
    return out


def quantize_per_token_int8(x):
    """x: fp32 [rows, cols] -> (q int8 [rows, cols], scale fp32 [rows])."""
    x = _c(x, np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), np.int8)
    scale = np.empty(rows, np.float32)
    lib().orc_quantize_per_token_int8(_c_u32(rows), _c_u32(cols), _ptr(x), _ptr(q), _ptr(scale))
    return q, scale


def mx_quantize(x, fmt, want_deq=False):
    """x: fp32 [rows, cols], blocks of 32 along cols. Returns (codes u8 [rows,cols], sf u8 [rows,ceil(cols/32)])."""
    x = _c(x, np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), np.uint8)
    sf = np.empty((rows, (cols + 31) // 32), np.uint8)
    deq = np.empty((rows, cols), np.float32) if want_deq else None
    lib().orc_mx_quantize(_c_u32(rows), _c_u32(cols), fmt, _ptr(x), _ptr(q), _ptr(sf), _ptr(deq))
    return (q, sf, deq) if want_deq else (q, sf)


def mx_matmul(aq, sfa, bq, sfb, m, n, k, fmt):
    aq, sfa, bq, sfb = _c(aq, np.uint8), _c(sfa, np.uint8), _c(bq, np.uint8), _c(sfb, np.uint8)
    out = np.empty((m, n), np.float32)
    lib().orc_mx_matmul(_c_u32(m), _c_u32(n), _c_u32(k), fmt, _ptr(aq), _ptr(sfa), _ptr(bq), _ptr(sfb),
                        _ptr(out))
    return out


def swiglu_bf16(c):
    """c: fp32 [m, n] (act | gate) -> bf16 bit patterns [m, n/2] of act / (1 + exp(-act)) * gate."""
    c = _c(c, np.float32)
    m, n = c.shape
    out = np.empty((m, n // 2), np.uint16)
    lib().orc_swiglu_bf16(_ptr(c), ctypes.c_uint64(m), ctypes.c_uint64(n), _ptr(out))
    return out


def mx_quant_bf16_e4m3(s_bits):
    """s_bits: bf16 bit patterns [rows, cols], cols % 32 == 0 -> (E4M3 codes [rows, cols], E8M0 [rows, cols/32])."""
    s_bits = _c(s_bits, np.uint16)
    rows, cols = s_bits.shape
    q = np.empty((rows, cols), np.uint8)
    scale = np.empty((rows, cols // 32), np.uint8)
    lib().orc_mx_quant_bf16_e4m3(_ptr(s_bits), ctypes.c_uint64(rows), ctypes.c_uint64(cols), _ptr(q), _ptr(scale))
    return q, scale


def bf16_bits(x):
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_bf16_rne_array(_ptr(x), _ptr(y), ctypes.c_size_t(x.size))
    return y


def f16_bits(x):
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_f16_rne_array(_ptr(x), _ptr(y), ctypes.c_size_t(x.size))
    return y


def out_bits(x, f16=False):
    """fp32 golden values rounded to the output element type (bf16, or fp16)."""
    return f16_bits(x) if f16 else bf16_bits(x)


def bf16_to_float(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack_int4_along_k(w):
    """w: int8 [k, n] with values in [-8, 7] -> uint8 [n, ceil(k/2)]; low nibble = even k, high nibble = odd k
    (an odd k leaves the last high nibble zero)."""
    k, n = w.shape
    wt = np.ascontiguousarray(w.T).astype(np.uint8) & 0xF  # [n, k]
    if k & 1:
        wt = np.concatenate([wt, np.zeros((n, 1), np.uint8)], axis=1)
    return (wt[:, 0::2] | (wt[:, 1::2] << 4)).astype(np.uint8)


# --- the reference's own golden (only where oracle/_ref was built) ------------------------------------

def ref_quant_matmul(a, b, scale, per_token, m, n, k, layout_a=ROW_MAJOR, layout_b=COL_MAJOR):
    a, b = _c(a, np.int8), _c(b, np.int8)
    scale, per_token = _c(scale, np.float32), _c(per_token, np.float32)
    out = np.empty((m, n), np.float32)
    ref().ref_quant_matmul(_c_u32(m), _c_u32(n), _c_u32(k), _ptr(a), layout_a, _ptr(b), layout_b,
                           _ptr(scale), _ptr(per_token), _ptr(out))
    return out


def ref_grouped_quant_matmul(a, b, group_list, scale, per_token, m, n, k, layout_b=ROW_MAJOR):
    a, b = _c(a, np.int8), _c(b, np.int8)
    gl = _c(group_list, np.int64)
    scale, per_token = _c(scale, np.float32), _c(per_token, np.float32)
    out = np.zeros((m, n), np.float32)
    ref().ref_grouped_quant_matmul_slice_m(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(len(gl)), _ptr(gl),
                                           _ptr(a), _ptr(b), layout_b, _ptr(scale), _ptr(per_token),
                                           _ptr(out))
    return out


def ref_grouped_fixpipe_dequant(a, b, group_list, quant_mode, scale_per_tensor, per_channel_scale, m, n, k,
                                layout_b=ROW_MAJOR):
    a, b = _c(a, np.int8), _c(b, np.int8)
    gl = _c(group_list, np.int64)
    pcs = _c(per_channel_scale, np.float32) if per_channel_scale is not None else None
    out = np.zeros((m, n), np.float32)
    ref().ref_grouped_fixpipe_dequant(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(len(gl)), _ptr(gl), _ptr(a), _ptr(b),
                                      layout_b, int(quant_mode), ctypes.c_float(scale_per_tensor), _ptr(pcs),
                                      _ptr(out))
    return out


def ref_grouped_quant_matmul_slice_k(a, b, group_list, scale, per_token, m, n, k):
    a, b = _c(a, np.int8), _c(b, np.int8)
    gl = _c(group_list, np.int64)
    scale, per_token = _c(scale, np.float32), _c(per_token, np.float32)
    out = np.zeros((len(gl), m, n), np.float32)
    ref().ref_grouped_quant_matmul_slice_k(_c_u32(m), _c_u32(n), _c_u32(k), _c_u32(len(gl)), _ptr(gl), _ptr(a),
                                           _ptr(b), _ptr(scale), _ptr(per_token), _ptr(out))
    return out


def ref_generate_group_list(m, g):
    out = np.empty(g, np.int64)
    ref().ref_generate_group_list(_c_u32(m), _c_u32(g), _ptr(out))
    return out
