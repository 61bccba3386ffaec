"""Caller-side binding with the function names, argument order and defaults of the reference's `torch_catlass`
package (tests/optest/torch_catlass/ops/*.py), over the C ABI of this library: the reference's pytest files for
the quantized-matmul path can be run against CUDA tensors by importing this module under that name.

    from catlass_b200 import torch_catlass
    d = torch_catlass.quant_matmul(a, b, scale, per_token_scale)           # tests/optest/tests/test_12_quant_matmul.py

Covered: quant_matmul (example 12), quant_optimized_matmul_tla (42), grouped_matmul_slice_m_per_token_dequant (07),
grouped_matmul_slice_m_per_token_dequant_multistage (10), grouped_matmul_slice_k_per_token_dequant (11),
ascend950_grouped_matmul_slice_m_per_token_dequant (47),
ascend950_grouped_matmul_slice_m_per_tensor_per_channel_dequant (48), w4a8_matmul (32),
ascend950_fp8_mx_matmul[_aswt] (53), ascend950_fp4_mx_matmul[_aswt] (54), ascend950_mx_grouped_matmul_slice_m (55).

Tensors are CUDA tensors; outputs are allocated with torch (this module is the binding, not the library: the
library itself never allocates).  Every call enqueues on the current stream and returns without synchronising.
"""
import torch

from . import capi

_SCALE_TYPES = {torch.float32: capi.DTYPE_F32, torch.bfloat16: capi.DTYPE_BF16, torch.float16: capi.DTYPE_F16}
_OUT_TYPES = {torch.bfloat16: capi.DTYPE_BF16, torch.float16: capi.DTYPE_F16}


def _dtype(out_dtype):
    if isinstance(out_dtype, str):
        out_dtype = getattr(torch, out_dtype.lower(), None)
    if out_dtype is None:
        raise ValueError(f"{out_dtype} is not a data type of torch")
    return out_dtype


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("catlass_b200 runs on CUDA tensors only (there is no CPU path)")


def _scales(scale, per_token):
    if scale.dtype != per_token.dtype or scale.dtype not in _SCALE_TYPES:
        raise ValueError("scale and perTokenScale must share one of float32 / bfloat16 / float16")
    return scale.contiguous().reshape(-1), per_token.contiguous().reshape(-1), _SCALE_TYPES[scale.dtype]


def _out(m, n, out_dtype, like):
    out_dtype = _dtype(out_dtype)
    if out_dtype not in _OUT_TYPES:
        raise ValueError("outDType must be float16 or bfloat16")
    return torch.empty((m, n), dtype=out_dtype, device=like.device), _OUT_TYPES[out_dtype]


def _b_layout(trans_b, use_nz_b):
    if use_nz_b:
        if trans_b:
            raise ValueError("fractal (zN) weights are taken untransposed")
        return capi.ZN
    return capi.COLUMN_MAJOR if trans_b else capi.ROW_MAJOR


def quant_matmul(mat1, mat2, scale, perTokenScale, outDType=torch.float16, transA=False, transB=False,
                 useNzA=False, useNzB=False):
    """tests/optest/torch_catlass/ops/quant_matmul.py: D = (int32(A @ B) * scale[n]) * perTokenScale[m].
    mat1 is (M, K), or (K, M) with transA; mat2 is (K, N), or (N, K) with transB, or zN fractals with useNzB."""
    _require_cuda(mat1, mat2, scale, perTokenScale)
    if useNzA:
        raise ValueError("fractal (zN) activations are not supported")
    mat1, mat2 = mat1.contiguous(), mat2.contiguous()
    k, m = (mat1.shape[0], mat1.shape[1]) if transA else (mat1.shape[1], mat1.shape[0])
    n = scale.numel()
    s, p, st = _scales(scale, perTokenScale)
    d, dt = _out(m, n, outDType, mat1)
    capi.quant_matmul(mat1, mat2, s, p, d, m, n, k, layout_a=capi.COLUMN_MAJOR if transA else capi.ROW_MAJOR,
                      layout_b=_b_layout(transB, useNzB), scale_type=st, d_type=dt)
    return d


def quant_optimized_matmul_tla(mat1, mat2, scale, per_token_scale, outDType=torch.bfloat16, transA=False, transB=True,
                               formatA=False, formatB=False):
    """tests/optest/torch_catlass/ops/quant_optimized_matmul_tla.py (example 42): scales are (1, N) and (1, M)."""
    return quant_matmul(mat1, mat2, scale, per_token_scale, outDType, transA, transB, formatA, formatB)


def _grouped(mat1, mat2, groupList, scale, perTokenScale, outDType, transA, transB, useNzA, useNzB):
    _require_cuda(mat1, mat2, groupList, scale, perTokenScale)
    if transA or useNzA:
        raise ValueError("slice-M groups cut A by rows: A is row-major (M, K)")
    mat1, mat2, groupList = mat1.contiguous(), mat2.contiguous(), groupList.contiguous()
    m, k = mat1.shape
    g = groupList.numel()
    n = scale.numel() // g
    if groupList.dtype == torch.int32:
        glt = capi.GROUP_LIST_INT32
    elif groupList.dtype == torch.int64:
        glt = capi.GROUP_LIST_INT64
    else:
        raise ValueError("groupList must be int32 or int64 prefix sums")
    s, p, st = _scales(scale, perTokenScale)
    d, dt = _out(m, n, outDType, mat1)
    capi.grouped_quant_matmul(mat1, mat2, groupList, s, p, d, m, n, k, g, layout_b=_b_layout(transB, useNzB),
                              group_list_type=glt, scale_type=st, d_type=dt)
    return d


def grouped_matmul_slice_m_per_token_dequant(mat1, mat2, groupList, scale, perTokenScale, outDType=torch.float16,
                                             transA=False, transB=False, useNzA=False, useNzB=False):
    """Example 07 (MoE): int8 (M, K) x int8 (G, K, N), prefix-sum groupList, float scales, half output."""
    return _grouped(mat1, mat2, groupList, scale, perTokenScale, outDType, transA, transB, useNzA, useNzB)


def grouped_matmul_slice_m_per_token_dequant_multistage(mat1, mat2, groupList, scale, perTokenScale,
                                                        outDType=torch.bfloat16, transA=False, transB=False,
                                                        useNzA=False, useNzB=False):
    """Example 10: int64 groupList, bf16 scales, bf16 output."""
    return _grouped(mat1, mat2, groupList, scale, perTokenScale, outDType, transA, transB, useNzA, useNzB)


def grouped_matmul_slice_k_per_token_dequant(mat1, mat2, groupList, scale, perTokenScale, outDType=torch.bfloat16,
                                             transA=False, transB=False, useNzA=False, useNzB=False):
    """Example 11: the groups cut K.  mat1 is A column-major, passed as (K, M) with transA=True; mat2 (K, N);
    groupList int64 prefix sums over K; scale (G, N), perTokenScale (G, M); output (G, M, N)."""
    _require_cuda(mat1, mat2, groupList, scale, perTokenScale)
    if not transA or transB or useNzA or useNzB:
        raise ValueError("slice-K takes A as (K, M) with transA=True and B as (K, N)")
    mat1, mat2, groupList = mat1.contiguous(), mat2.contiguous(), groupList.contiguous()
    k, m = mat1.shape
    n = mat2.shape[1]
    g = groupList.numel()
    s, p, st = _scales(scale, perTokenScale)
    out_dtype = _dtype(outDType)
    if out_dtype not in _OUT_TYPES:
        raise ValueError("outDType must be float16 or bfloat16")
    d = torch.empty((g, m, n), dtype=out_dtype, device=mat1.device)
    ws = torch.empty(max(capi.grouped_quant_matmul_slice_k_workspace_size(m, n, k, g), 1), dtype=torch.uint8,
                     device=mat1.device)
    capi.grouped_quant_matmul_slice_k(mat1, mat2, groupList, s, p, d, m, n, k, g, ws,
                                      group_list_type=capi.GROUP_LIST_INT32 if groupList.dtype == torch.int32
                                      else capi.GROUP_LIST_INT64, scale_type=st, d_type=_OUT_TYPES[out_dtype])
    return d


def ascend950_grouped_matmul_slice_m_per_token_dequant(mat1, mat2, groupList, scale, perTokenScale,
                                                       outDType=torch.bfloat16, transA=False, transB=False,
                                                       useNzA=False, useNzB=False):
    """Example 47."""
    return _grouped(mat1, mat2, groupList, scale, perTokenScale, outDType, transA, transB, useNzA, useNzB)


def ascend950_grouped_matmul_slice_m_per_tensor_per_channel_dequant(mat1, mat2, groupList, perChannelScale,
                                                                    scalePerTensor=1.0, quantMode=0,
                                                                    outDType=torch.float16, transA=False, transB=False,
                                                                    useNzA=False, useNzB=False):
    """Example 48: perChannelScale holds fp32 bit patterns in 64-bit words (shape (N,)), quantMode 0 = per tensor,
    1 = per channel."""
    _require_cuda(mat1, mat2, groupList, perChannelScale)
    if transA or useNzA:
        raise ValueError("slice-M groups cut A by rows: A is row-major (M, K)")
    mat1, mat2, groupList = mat1.contiguous(), mat2.contiguous(), groupList.contiguous()
    m, k = mat1.shape
    g = groupList.numel()
    n = mat2.shape[1] if transB else mat2.shape[2]
    if perChannelScale.dtype in (torch.int64, torch.uint64):
        pct = capi.DTYPE_F32_IN_U64
    elif perChannelScale.dtype == torch.float32:
        pct = capi.DTYPE_F32
    else:
        raise ValueError("perChannelScale must be 64-bit words holding fp32 bits, or float32")
    d, dt = _out(m, n, outDType, mat1)
    capi.grouped_fixpipe_dequant(mat1, mat2, groupList, d, m, n, k, g, int(quantMode),
                                 scale_per_tensor=float(scalePerTensor), per_channel_scale=perChannelScale.contiguous(),
                                 per_channel_scale_type=pct, layout_b=_b_layout(transB, useNzB), d_type=dt,
                                 group_list_type=capi.GROUP_LIST_INT32 if groupList.dtype == torch.int32
                                 else capi.GROUP_LIST_INT64)
    return d


W4A8_REFERENCE_SCALAR = 1.5  # the per-tensor dequant scalar of the reference's example 32 (gen_data.py:111-131)


def w4a8_matmul(mat1, mat2, outDType=torch.float16, transA=False, transB=False, formatA=False, formatB=False):
    """Example 32: C = 1.5 * (A_int8 @ B_int4).  mat2 is the packed weight: (K, ceil(N/2)) bytes packed along N, or
    with transB (N, ceil(K/2)) bytes packed along K; low nibble = even index."""
    _require_cuda(mat1, mat2)
    if transA or formatA or formatB:
        raise ValueError("w4a8_matmul takes row-major A and unformatted operands")
    mat1, mat2 = mat1.contiguous(), mat2.contiguous()
    m, k = mat1.shape
    if transB:
        n = mat2.shape[0]
        pack_axis = capi.W4_PACKED_ALONG_K
    else:
        # the reference's wrapper is given the packed array only: its width is ceil(n/2) bytes and n is even
        n = mat2.shape[1] * 2
        pack_axis = capi.W4_PACKED_ALONG_N
    d, dt = _out(m, n, outDType, mat1)
    ones = torch.ones((1, n), dtype=torch.float32, device=mat1.device)
    scalar = torch.full((m,), W4A8_REFERENCE_SCALAR, dtype=torch.float32, device=mat1.device)
    ws_bytes = capi.w4a8_matmul_workspace_size(m, n, k, k, pack_axis)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=mat1.device)
    capi.w4a8_matmul(mat1, mat2, ones, scalar, d, m, n, k, k, d_type=dt, pack_axis=pack_axis, workspace=ws)
    return d


def _mx(mat1, mat2, mx_scale_a, mx_scale_b, transA, transB, fmt):
    _require_cuda(mat1, mat2, mx_scale_a, mx_scale_b)
    mat1, mat2 = mat1.contiguous(), mat2.contiguous()
    a_bytes, b_bytes = mat1.view(torch.uint8), mat2.view(torch.uint8)
    per_byte = 2 if fmt == capi.MX_E2M1 else 1
    # shapes in elements: mat1 (M, K) or (K, M); mat2 (N, K) with transB (the reference's default) or (K, N)
    if per_byte == 2 and a_bytes.shape == tuple(mat1.shape):
        # a float4_e2m1fn_x2 tensor reports its logical element shape; a plain byte tensor its packed one
        raise ValueError("pass packed E2M1 operands as float4_e2m1fn_x2 tensors")
    sa, sb = tuple(mat1.shape), tuple(mat2.shape)
    k, m = (sa[0], sa[1]) if transA else (sa[1], sa[0])
    n = sb[0] if transB else sb[1]
    d = torch.empty((m, n), dtype=torch.float32, device=mat1.device)
    la = capi.COLUMN_MAJOR if transA else capi.ROW_MAJOR
    lb = capi.COLUMN_MAJOR if transB else capi.ROW_MAJOR
    ws = torch.empty(max(capi.mx_matmul_workspace_size(m, n, k, fmt, la, lb), 1), dtype=torch.uint8, device=mat1.device)
    capi.mx_matmul(a_bytes, b_bytes, mx_scale_a.contiguous().view(torch.uint8), mx_scale_b.contiguous().view(torch.uint8),
                   d, m, n, k, fmt, ws, layout_a=la, layout_b=lb, out_f32=True)
    return d


def ascend950_mx_grouped_matmul_slice_m(mat1, mat2, groupList, mx_scale_a, mx_scale_b, transA=False, transB=False,
                                        enable_aswt=False, enable_preload=False):
    """Example 55: mat1 (M, K), mat2 (G, K, N) or with transB (G, N, K), groupList the groups' row counts (int64,
    not prefix sums), block scales per group for mat2; fp32 output.  The two scheduler switches of the reference
    select variants of its kernel and change no result: they are accepted and ignored."""
    _require_cuda(mat1, mat2, groupList, mx_scale_a, mx_scale_b)
    if transA:
        raise ValueError("slice-M groups cut A by rows: A is (M, K)")
    mat1, mat2, groupList = mat1.contiguous(), mat2.contiguous(), groupList.contiguous()
    fmt = capi.MX_E2M1 if mat1.dtype == getattr(torch, "float4_e2m1fn_x2", None) else capi.MX_E4M3
    m, k = tuple(mat1.shape)
    g = groupList.numel()
    n = mat2.shape[1] if transB else mat2.shape[2]
    lb = capi.COLUMN_MAJOR if transB else capi.ROW_MAJOR
    d = torch.zeros((m, n), dtype=torch.float32, device=mat1.device)
    ws = torch.empty(max(capi.mx_grouped_matmul_workspace_size(m, n, k, g, fmt, lb), 1), dtype=torch.uint8,
                     device=mat1.device)
    capi.mx_grouped_matmul(mat1.view(torch.uint8), mat2.view(torch.uint8), groupList,
                           mx_scale_a.contiguous().view(torch.uint8), mx_scale_b.contiguous().view(torch.uint8), d, m, n,
                           k, g, fmt, ws, layout_b=lb,
                           group_list_type=capi.GROUP_LIST_INT32 if groupList.dtype == torch.int32
                           else capi.GROUP_LIST_INT64, group_list_kind=capi.GROUP_LIST_SIZES, out_f32=True)
    return d


def ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant(mat1, mat2, mx_scale_a, mx_scale_b, group_list,
                                                            transB=True):
    """Example 65 (tests/optest/torch_catlass/ops/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant.py): grouped
    MXFP8 matmul, SwiGLU over the two halves of its columns, MX quantisation of the result.  mat1 (M, K)
    float8_e4m3fn, mat2 (G, N, K) with transB else (G, K, N), group_list the groups' row counts (int64).
    Returns [Q (M, N/2) float8_e4m3fn, Q_scale (M, N/64) float8_e8m0fnu]; rows past the last group are zero."""
    _require_cuda(mat1, mat2, mx_scale_a, mx_scale_b, group_list)
    mat1, mat2, group_list = mat1.contiguous(), mat2.contiguous(), group_list.contiguous()
    m, k = tuple(mat1.shape)
    g = group_list.numel()
    n = mat2.shape[1] if transB else mat2.shape[2]
    lb = capi.COLUMN_MAJOR if transB else capi.ROW_MAJOR
    q = torch.zeros((m, n // 2), dtype=torch.uint8, device=mat1.device)
    q_scale = torch.zeros((m, n // 64), dtype=torch.uint8, device=mat1.device)
    ws = torch.empty(max(capi.mx_grouped_swiglu_quant_workspace_size(m, n, k, g, lb), 1), dtype=torch.uint8,
                     device=mat1.device)
    capi.mx_grouped_swiglu_quant(mat1.view(torch.uint8), mat2.view(torch.uint8), group_list,
                                 mx_scale_a.contiguous().view(torch.uint8), mx_scale_b.contiguous().view(torch.uint8),
                                 q, q_scale, m, n, k, g, ws, layout_b=lb,
                                 group_list_type=capi.GROUP_LIST_INT32 if group_list.dtype == torch.int32
                                 else capi.GROUP_LIST_INT64, group_list_kind=capi.GROUP_LIST_SIZES)
    e8m0 = getattr(torch, "float8_e8m0fnu", None)
    return [q.view(torch.float8_e4m3fn), q_scale.view(e8m0) if e8m0 is not None else q_scale]


def ascend950_fp8_mx_grouped_matmul_finalize_routing(mat1, mat2, mx_scale_a, mx_scale_b, group_list, logit, row_index,
                                                     bias, shared_input, batch, data_parallel_size=1,
                                                     shared_input_weight=0.0, shared_input_offset=0, group_list_type=0,
                                                     trans_a=False, trans_b=False):
    """Example 71, deterministic variant (tests/optest/torch_catlass/ops/
    ascend950_fp8_mx_grouped_matmul_finalize_routing.py): the same bits on every run."""
    return ascend950_fp8_mx_grouped_matmul_finalize_routing_no_deter(
        mat1, mat2, mx_scale_a, mx_scale_b, group_list, logit, row_index, bias, shared_input, batch,
        data_parallel_size, shared_input_weight, shared_input_offset, group_list_type, trans_a, trans_b,
        _deterministic=True)


def ascend950_fp8_mx_grouped_matmul_finalize_routing_no_deter(mat1, mat2, mx_scale_a, mx_scale_b, group_list, logit,
                                                              row_index, bias, shared_input, batch,
                                                              data_parallel_size=1, shared_input_weight=0.0,
                                                              shared_input_offset=0, group_list_type=0, trans_a=False,
                                                              trans_b=False, _deterministic=False):
    """Example 71, non-deterministic variant (tests/optest/torch_catlass/ops/
    ascend950_fp8_mx_grouped_matmul_finalize_routing_no_deter.py): grouped MXFP8 matmul whose rows are weighted
    with `logit` and added into rows `row_index` of an fp32 (batch, N) output, with an optional bf16 bias per group
    and an optional shared-expert input added at `shared_input_offset`.  group_list_type 0 = prefix sums, 1 = sizes.
    Empty tensors stand for "no bias" / "no shared input", as in the reference."""
    _require_cuda(mat1, mat2, mx_scale_a, mx_scale_b, group_list, logit, row_index)
    if trans_a:
        raise ValueError("slice-M groups cut A by rows: A is (M, K)")
    mat1, mat2, group_list = mat1.contiguous(), mat2.contiguous(), group_list.contiguous()
    m, k = tuple(mat1.shape)
    g = group_list.numel()
    n = mat2.shape[1] if trans_b else mat2.shape[2]
    lb = capi.COLUMN_MAJOR if trans_b else capi.ROW_MAJOR
    has_bias = bias is not None and bias.numel() != 0
    has_shared = shared_input is not None and shared_input.numel() != 0
    bsdp = batch // max(int(data_parallel_size), 1)
    out = torch.empty((batch, n), dtype=torch.float32, device=mat1.device)
    ws = torch.empty(max(capi.mx_grouped_finalize_routing_workspace_size(m, n, k, g, batch, lb, _deterministic), 1),
                     dtype=torch.uint8, device=mat1.device)
    row_index = row_index.contiguous()
    capi.mx_grouped_finalize_routing(
        mat1.view(torch.uint8), mat2.view(torch.uint8), group_list, mx_scale_a.contiguous().view(torch.uint8),
        mx_scale_b.contiguous().view(torch.uint8), logit.contiguous().float(), row_index, out, m, n, k, g, batch, ws,
        bias=bias.contiguous().to(torch.bfloat16) if has_bias else None,
        shared_input=shared_input.contiguous().to(torch.bfloat16) if has_shared else None,
        shared_rows=bsdp if has_shared else 0, shared_offset=int(shared_input_offset),
        shared_weight=float(shared_input_weight), layout_b=lb,
        group_list_type=capi.GROUP_LIST_INT32 if group_list.dtype == torch.int32 else capi.GROUP_LIST_INT64,
        group_list_kind=capi.GROUP_LIST_PREFIX_SUMS if group_list_type == 0 else capi.GROUP_LIST_SIZES,
        row_index_type=capi.GROUP_LIST_INT32 if row_index.dtype == torch.int32 else capi.GROUP_LIST_INT64,
        deterministic=_deterministic)
    return out


def ascend950_fp8_mx_matmul_aswt(mat1, mat2, mx_scale_a, mx_scale_b, transA=False, transB=True):
    """Example 53: float8_e4m3fn operands, float8_e8m0fnu block scales, fp32 output."""
    return _mx(mat1, mat2, mx_scale_a, mx_scale_b, transA, transB, capi.MX_E4M3)


ascend950_fp8_mx_matmul = ascend950_fp8_mx_matmul_aswt


def ascend950_fp4_mx_matmul_aswt(mat1, mat2, mx_scale_a, mx_scale_b, transA=False, transB=True):
    """Example 54: float4_e2m1fn_x2 operands (two per byte), float8_e8m0fnu block scales, fp32 output."""
    return _mx(mat1, mat2, mx_scale_a, mx_scale_b, transA, transB, capi.MX_E2M1)


ascend950_fp4_mx_matmul = ascend950_fp4_mx_matmul_aswt
