"""Shapes and layouts off the kernels' fast paths, as the reference's own tests run them: MX operands in all four
transpose pairs and with K that is not a multiple of the K block, even K = 2 (tests/optest/tests/
test_53_ascend950_fp8_mx_matmul_aswt.py:21-30, test_54_ascend950_fp4_mx_matmul_aswt.py:37-54), fp32 output; W4A8
with the runner's m=860 n=5712 k=4535 (tests/test_example.py:141-152), weights packed along N
(tests/optest/tests/test_32_w4a8_matmul.py:11-28), a shorter last scale group, unaligned operands.  All through
the C ABI, against the CPU oracle."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


def _dev(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


# ------------------------------------------------------------------------------------------------ MX

def _pack_last_axis(codes):
    """E2M1 codes (one per byte) -> two per byte along the last axis, even index in the low nibble."""
    if codes.shape[-1] & 1:
        codes = np.concatenate([codes, np.zeros(codes.shape[:-1] + (1,), np.uint8)], axis=-1)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def _stored_operand(codes_rows_k, fmt, k_first):
    """codes [rows][k] -> the caller's array: rows along K, or [k][rows] when k_first; E2M1 packed along the
    contiguous axis."""
    arr = np.ascontiguousarray(codes_rows_k.T) if k_first else codes_rows_k
    return _pack_last_axis(arr) if fmt == O.MX_E2M1 else arr


def _stored_scales(sf_rows_blocks, k_first):
    """sf [rows][ceil(k/32)] -> [rows][KS] (KS even, padding 2^0), or [KS/2][rows][2] when k_first."""
    rows, blocks = sf_rows_blocks.shape
    ks = (blocks + 1) // 2 * 2
    padded = np.full((rows, ks), 127, np.uint8)
    padded[:, :blocks] = sf_rows_blocks
    if not k_first:
        return padded
    return np.ascontiguousarray(padded.reshape(rows, ks // 2, 2).transpose(1, 0, 2))


def _mx_case(cuda, m, n, k, fmt, trans_a, trans_b, out_f32, seed, static=False):
    import torch
    from catlass_b200 import capi
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal((m, k)) * 10.0 - 5.0).astype(np.float32)   # the law of the reference's MX tests
    bt = (rng.standard_normal((n, k)) * 10.0 - 5.0).astype(np.float32)
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb = O.mx_quantize(bt, fmt)
    want = O.mx_matmul(aq, sfa, bq, sfb, m, n, k, fmt)
    # the reference's transB=True stores B as [n][k]: this library's CB200_COLUMN_MAJOR
    la = capi.COLUMN_MAJOR if trans_a else capi.ROW_MAJOR
    lb = capi.COLUMN_MAJOR if trans_b else capi.ROW_MAJOR
    d = torch.full((m, n), -3.0, dtype=torch.float32 if out_f32 else torch.bfloat16, device=cuda)
    args = (_dev(_stored_operand(aq, fmt, trans_a)), _dev(_stored_operand(bq, fmt, not trans_b)),
            _dev(_stored_scales(sfa, trans_a)), _dev(_stored_scales(sfb, not trans_b)), d, m, n, k, fmt)
    if static:
        capi.mx_matmul_static(*args, layout_a=la, layout_b=lb, out_f32=out_f32)
    else:
        ws = torch.empty(max(capi.mx_matmul_workspace_size(m, n, k, fmt, la, lb), 256), dtype=torch.uint8, device=cuda)
        capi.mx_matmul(*args, ws, layout_a=la, layout_b=lb, out_f32=out_f32)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    got = d.float().cpu().numpy()
    assert np.isfinite(got).all()
    err = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    tol = 1e-2 if not out_f32 else 1e-3   # fp32 output carries no bf16 rounding: only the accumulation order differs
    assert err.max() <= tol, f"max rel err {err.max():.5f} at {np.unravel_index(err.argmax(), err.shape)}"


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)],
                         ids=["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_mx_all_transpose_pairs(cuda, fmt, trans_a, trans_b):
    _mx_case(cuda, 256, 512, 1024, fmt, trans_a, trans_b, out_f32=True, seed=53)


@pytest.mark.parametrize("m,n,k,trans_a,trans_b", [
    (4097, 4, 2, False, False), (1024, 17, 129, False, False), (513, 1280, 33, False, False),
    (768, 1025, 63, True, False), (8193, 257, 63, False, False), (513, 1280, 33, False, True),
    (130, 264, 192, False, True), (64, 72, 1000, True, True),
])
@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_mx_ragged_k_and_odd_shapes(cuda, fmt, m, n, k, trans_a, trans_b):
    """The reference's FP4 test shapes (rows scaled down where the oracle would take minutes): K = 2, 33, 63, 129,
    odd N, odd M, mixed transposes."""
    _mx_case(cuda, m, n, k, fmt, trans_a, trans_b, out_f32=True, seed=m + n + k)


@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_mx_bf16_output_off_the_fast_path(cuda, fmt):
    _mx_case(cuda, 300, 264, 520, fmt, True, False, out_f32=False, seed=9)


@pytest.mark.parametrize("fmt,out_f32,m,n,k", [
    (O.MX_E4M3, False, 1100, 7700, 384), (O.MX_E2M1, True, 1100, 7700, 512), (O.MX_E4M3, True, 530, 19200, 160),
])
def test_mx_on_cta_pairs(cuda, fmt, out_f32, m, n, k):
    """Dense shapes with at least two waves of 256 x 256 tiles run on CTA pairs: ragged last tile row (the second
    CTA of a pair past the end of A), ragged last tile column, both output types, a ragged K through the ingestion
    pre-pass."""
    assert ((m + 255) // 256) * ((n + 255) // 256) >= 148
    _mx_case(cuda, m, n, k, fmt, False, True, out_f32=out_f32, seed=m + n)


def test_mx_static_scratch_entry_takes_the_same_layouts(cuda):
    _mx_case(cuda, 200, 136, 330, O.MX_E4M3, True, False, out_f32=True, seed=11, static=True)
    _mx_case(cuda, 130, 520, 190, O.MX_E2M1, False, False, out_f32=False, seed=12, static=True)


# ------------------------------------------------------------------------------------------------ W4A8

def _pack_along_n(w):
    """w: int8 [k, n] in [-8, 7] -> uint8 [k, ceil(n/2)], even n in the low nibble (the reference's row-major B)."""
    k, n = w.shape
    u = w.astype(np.uint8) & 0xF
    if n & 1:
        u = np.concatenate([u, np.zeros((k, 1), np.uint8)], axis=1)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)


def _w4_case(cuda, m, n, k, gs, along_n, seed, f16=False, misalign=False, cols=None):
    import torch
    from catlass_b200 import capi
    rng = np.random.default_rng(seed)
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    groups = 1 if gs >= k else (k + gs - 1) // gs
    sw = rng.uniform(1e-3, 1e-2, (groups, n)).astype(np.float32)
    sa = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    packed_k = O.pack_int4_along_k(w)
    stored = _pack_along_n(w) if along_n else packed_k
    axis = capi.W4_PACKED_ALONG_N if along_n else capi.W4_PACKED_ALONG_K
    a_dev, w_dev = _dev(a), _dev(stored)
    if misalign:   # operands one byte off a 16-byte boundary
        a_buf = torch.zeros(a.size + 32, dtype=torch.int8, device=cuda)
        w_buf = torch.zeros(stored.size + 32, dtype=torch.uint8, device=cuda)
        a_buf[1:1 + a.size].copy_(a_dev.reshape(-1))
        w_buf[1:1 + stored.size].copy_(w_dev.reshape(-1))
        a_dev, w_dev = a_buf[1:], w_buf[1:]
    d = torch.full((m, n), -3.0, dtype=torch.float16 if f16 else torch.bfloat16, device=cuda)
    ws_bytes = capi.w4a8_matmul_workspace_size(m, n, k, gs, axis, aligned=not misalign)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=cuda)
    capi.w4a8_matmul(a_dev, w_dev, _dev(sw), _dev(sa), d, m, n, k, gs, pack_axis=axis, workspace=ws,
                     d_type=capi.DTYPE_F16 if f16 else capi.DTYPE_BF16)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    got = d.view(torch.int16).cpu().numpy().view(np.uint16)
    if cols is None:
        cols = np.arange(n)
    want = O.w4a8_per_group(a, packed_k[cols], np.ascontiguousarray(sw[:, cols]), sa, m, len(cols), k, max(gs, 1))
    want_bits = O.out_bits(want, f16)
    assert np.array_equal(got[:, cols], want_bits), f"{(got[:, cols] != want_bits).sum()} of {want_bits.size} differ"


@pytest.mark.parametrize("m,n,k,gs,along_n", [
    (16, 128, 300, 128, False),     # last scale group of 44 elements
    (70, 200, 293, 128, False),     # odd k
    (33, 136, 1000, 256, False),    # group 256, last group 232
    (64, 256, 256, 256, True),      # the reference's torch test: 256^3, packed along N, one group
    (40, 130, 520, 128, True),      # packed along N, n/2 odd
    (24, 77, 333, 333, True),       # odd n, odd k, one group
    (128, 512, 1024, 128, False),   # fast path beside them (no workspace use)
])
def test_w4a8_off_the_fast_path(cuda, m, n, k, gs, along_n):
    _w4_case(cuda, m, n, k, gs, along_n, seed=m + n + k)


def test_w4a8_reference_runner_shape(cuda):
    """m=860 n=5712 k=4535, one scale for the tensor (group = k), half output: the shape tests/test_example.py runs
    example 32 with.  The oracle checks 160 columns over the full K."""
    rng = np.random.default_rng(4535)
    cols = np.unique(np.concatenate([[0, 127, 128, 5711], rng.integers(0, 5712, 156)]))
    _w4_case(cuda, 860, 5712, 4535, 4535, False, seed=32, f16=True, cols=cols)


def test_w4a8_unaligned_operands_and_half_output(cuda):
    _w4_case(cuda, 48, 256, 512, 128, False, seed=5, f16=True, misalign=True)


def test_w4a8_weights_written_on_the_stream_right_before_the_call(cuda):
    """Plain stream order under programmatic dependent launch: the kernel must see weights and weight scales that
    a copy earlier on the same stream produced."""
    import torch
    from catlass_b200 import capi
    m, n, k, gs = 64, 4096, 4096, 128
    rng = np.random.default_rng(8)
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    sw = rng.uniform(1e-3, 1e-2, (k // gs, n)).astype(np.float32)
    sa = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    packed = O.pack_int4_along_k(w)
    cols = np.arange(0, n, 37)
    want = O.bf16_bits(O.w4a8_per_group(a, packed[cols], np.ascontiguousarray(sw[:, cols]), sa, m, len(cols), k, gs))
    src_w, src_s, a_d, sa_d = _dev(packed), _dev(sw), _dev(a), _dev(sa)
    big = torch.zeros(64 << 20, dtype=torch.int8, device=cuda)
    for _ in range(4):
        wd = torch.zeros_like(src_w)
        sd = torch.zeros_like(src_s)
        d = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
        torch.cuda.synchronize()
        big.add_(1)
        wd.copy_(src_w)
        sd.copy_(src_s)
        capi.w4a8_matmul(a_d, wd, sd, sa_d, d, m, n, k, gs)
        assert capi.device_status()[0] == 0
        got = d.view(torch.int16).cpu().numpy().view(np.uint16)[:, cols]
        assert np.array_equal(got, want)


# ------------------------------------------------------------------------------------------------ grouped MX

@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
@pytest.mark.parametrize("sizes,n,k,trans_b,prefix", [
    ((128, 128), 128, 256, False, False),           # the reference's optest shape
    ((130, 0, 64, 257, 1, 300), 264, 512, True, False),
    ((5, 200, 0, 129), 520, 330, False, True),      # ragged K, prefix-sum list
    ((1000, 24), 1025, 96, True, True),
    ((700, 37, 600), 19200, 128, True, False),      # large enough for the CTA-pair kernel: 256-row tiles of one group
])
def test_mx_grouped_slice_m(cuda, fmt, sizes, n, k, trans_b, prefix):
    """Example 55: per-group weights and weight scales, the group list given as row counts (the reference's
    convention) or prefix sums; every group checked against the oracle's dequantised matmul of its own rows; rows
    past the last group keep the caller's bytes."""
    import torch
    from catlass_b200 import capi
    rng = np.random.default_rng(sum(sizes) + n + k)
    g = len(sizes)
    rows = sum(sizes)
    m = rows + 37
    a = (rng.standard_normal((m, k)) * 10.0 - 5.0).astype(np.float32)
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb, want = [], [], np.zeros((m, n), np.float32)
    start = 0
    for e in range(g):
        bt = (rng.standard_normal((n, k)) * 10.0 - 5.0).astype(np.float32)
        q_e, s_e = O.mx_quantize(bt, fmt)
        bq.append(q_e)
        sfb.append(s_e)
        if sizes[e]:
            want[start:start + sizes[e]] = O.mx_matmul(aq[start:start + sizes[e]], sfa[start:start + sizes[e]], q_e, s_e,
                                                       sizes[e], n, k, fmt)
        start += sizes[e]
    lb = capi.COLUMN_MAJOR if trans_b else capi.ROW_MAJOR
    b_dev = _dev(np.stack([_stored_operand(q_e, fmt, not trans_b) for q_e in bq]))
    sb_dev = _dev(np.stack([_stored_scales(s_e, not trans_b) for s_e in sfb]))
    gl = np.cumsum(sizes) if prefix else np.array(sizes)
    canary = -7.0
    d = torch.full((m, n), canary, dtype=torch.float32, device=cuda)
    ws = torch.empty(max(capi.mx_grouped_matmul_workspace_size(m, n, k, g, fmt, lb), 256), dtype=torch.uint8, device=cuda)
    capi.mx_grouped_matmul(_dev(_stored_operand(aq, fmt, False)), b_dev, _dev(gl.astype(np.int64)),
                           _dev(_stored_scales(sfa, False)), sb_dev, d, m, n, k, g, fmt, ws, layout_b=lb,
                           group_list_kind=capi.GROUP_LIST_PREFIX_SUMS if prefix else capi.GROUP_LIST_SIZES, out_f32=True)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    got = d.cpu().numpy()
    assert (got[rows:] == canary).all(), "rows past the last group were written"
    err = np.abs(got[:rows] - want[:rows]) / np.maximum(1.0, np.abs(want[:rows]))
    assert np.isfinite(got[:rows]).all() and err.max() <= 1e-3, f"max rel err {err.max():.5f}"
