"""Grouped MXFP8 matmul with the SwiGLU + MX quantisation epilogue fused in (the reference's
experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant example), through the C ABI.

Two checks per case:
  * against the library's own unfused result: the same grouped matmul with fp32 output (same accumulators), pushed
    through the CPU oracle's swiglu + quantiser.  Only exp() can differ (device expf against the host's), which the
    rounding to bf16 hides almost always: scales must agree on all but a handful of blocks, codes on all but a
    handful of elements, and a disagreeing code must be the neighbouring E4M3 code;
  * the reference's own acceptance rule (compare.py:236-287 of that example): relative error of the dequantised
    output against the high-precision result (fp32 operands, no quantisation of the inputs' product) at most twice
    max(2^-4, the golden's own error)."""
import numpy as np
import pytest

import oracle_lib as O
from test_ingest_gpu import _dev, _stored_operand, _stored_scales

pytestmark = pytest.mark.gpu


def _e4m3_values(codes):
    lut = np.array([O.lib().orc_e4m3_to_float(c) for c in range(256)], np.float32)
    return lut[codes]


@pytest.mark.parametrize("sizes,n,k,trans_b,prefix,scale", [
    ((128, 128), 512, 1024, True, False, 1.0),        # the example's own run: 2 x 128 rows, n = 512, k = 1024
    ((130, 0, 64, 257, 1), 256, 512, True, False, 1.0),
    ((5, 200, 129), 768, 330, False, True, 1.0),      # B stored [G][k][n], ragged K, prefix sums
    ((300, 77), 1024, 256, True, False, 0.02),        # small products: blocks below the exponent floor
    ((700, 600), 19456, 128, True, False, 1.0),       # large enough for the CTA-pair kernel (leader: act, peer: gate)
])
def test_mx_grouped_swiglu_mx_quant(cuda, sizes, n, k, trans_b, prefix, scale):
    import torch
    from catlass_b200 import capi
    fmt = O.MX_E4M3
    rng = np.random.default_rng(sum(sizes) + n + k)
    g, rows = len(sizes), sum(sizes)
    m = rows + 19
    h = n // 2
    a = (rng.standard_normal((m, k)) * scale).astype(np.float32)
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb, bts = [], [], []
    for e in range(g):
        bt = (rng.standard_normal((n, k)) * scale).astype(np.float32)
        q_e, s_e = O.mx_quantize(bt, fmt)
        bq.append(q_e)
        sfb.append(s_e)
        bts.append(bt)
    lb = capi.COLUMN_MAJOR if trans_b else capi.ROW_MAJOR
    a_dev = _dev(_stored_operand(aq, fmt, False))
    b_dev = _dev(np.stack([_stored_operand(q_e, fmt, not trans_b) for q_e in bq]))
    sa_dev = _dev(_stored_scales(sfa, False))
    sb_dev = _dev(np.stack([_stored_scales(s_e, not trans_b) for s_e in sfb]))
    gl = np.cumsum(sizes) if prefix else np.array(sizes)
    gl_dev = _dev(gl.astype(np.int64))
    kind = capi.GROUP_LIST_PREFIX_SUMS if prefix else capi.GROUP_LIST_SIZES

    # unfused: C in fp32 from the same kernel family, then the oracle's epilogue on the host
    c = torch.zeros((m, n), dtype=torch.float32, device=cuda)
    ws = torch.empty(max(capi.mx_grouped_matmul_workspace_size(m, n, k, g, fmt, lb), 256), dtype=torch.uint8, device=cuda)
    capi.mx_grouped_matmul(a_dev, b_dev, gl_dev, sa_dev, sb_dev, c, m, n, k, g, fmt, ws, layout_b=lb,
                           group_list_kind=kind, out_f32=True)
    c_host = c.cpu().numpy()[:rows]
    want_q, want_s = O.mx_quant_bf16_e4m3(O.swiglu_bf16(c_host))

    # fused
    q = torch.full((m, h), 0x55, dtype=torch.uint8, device=cuda)
    qs = torch.full((m, h // 32), 0x55, dtype=torch.uint8, device=cuda)
    ws2 = torch.empty(max(capi.mx_grouped_swiglu_quant_workspace_size(m, n, k, g, lb), 256), dtype=torch.uint8,
                      device=cuda)
    capi.mx_grouped_swiglu_quant(a_dev, b_dev, gl_dev, sa_dev, sb_dev, q, qs, m, n, k, g, ws2, layout_b=lb,
                                 group_list_kind=kind)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    got_q, got_s = q.cpu().numpy(), qs.cpu().numpy()
    assert (got_q[rows:] == 0x55).all() and (got_s[rows:] == 0x55).all(), "rows past the last group were written"
    got_q, got_s = got_q[:rows], got_s[:rows]

    scale_mismatch = got_s != want_s
    assert scale_mismatch.mean() <= 1e-3, f"{scale_mismatch.sum()} of {scale_mismatch.size} block scales differ"
    same_scale = np.repeat(~scale_mismatch, 32, axis=1)
    code_mismatch = (got_q != want_q) & same_scale
    assert code_mismatch.mean() <= 1e-3, f"{code_mismatch.sum()} of {code_mismatch.size} codes differ"
    step = np.abs(got_q[code_mismatch].astype(np.int32) - want_q[code_mismatch].astype(np.int32))
    assert (step <= 1).all() or ((got_q[code_mismatch] ^ want_q[code_mismatch]) == 0x80).all()

    # the reference's acceptance rule against the high-precision result
    start = 0
    hp_q, hp_s = np.zeros_like(got_q), np.zeros_like(got_s)
    for e in range(g):
        if sizes[e]:
            rows_e = slice(start, start + sizes[e])
            hp = a[rows_e].astype(np.float32) @ bts[e].T.astype(np.float32)
            hp_q[rows_e], hp_s[rows_e] = O.mx_quant_bf16_e4m3(O.swiglu_bf16(hp))
        start += sizes[e]
    err = 2.0 ** -4
    vals = lambda codes: _e4m3_values(codes).astype(np.float64)
    e_ex = np.abs(vals(hp_q) - vals(got_q)) / np.maximum(np.abs(vals(hp_q)), 1.0)
    e_gold = np.abs(vals(hp_q) - vals(want_q)) / np.maximum(np.abs(vals(hp_q)), 1.0)
    assert not (e_ex > np.maximum(e_gold, err) * 2).any()
    s_ex = np.abs(hp_s.astype(np.float64) - got_s) / np.maximum(hp_s.astype(np.float64), 1.0)
    s_gold = np.abs(hp_s.astype(np.float64) - want_s) / np.maximum(hp_s.astype(np.float64), 1.0)
    assert not (s_ex > np.maximum(s_gold, err) * 2).any()


def test_mx_grouped_swiglu_mx_quant_rejects(cuda):
    """Statuses of the argument checks: n not a multiple of 256, missing scale output, misaligned Q."""
    import torch
    from catlass_b200 import capi
    import ctypes
    lib = capi.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device=cuda)
    base = dict(m=128, n=512, k=256, group_count=2, layout_b=capi.COLUMN_MAJOR, group_list_type=capi.GROUP_LIST_INT64,
                group_list_kind=capi.GROUP_LIST_SIZES, flags=0, a=buf.data_ptr(), b=buf.data_ptr(),
                group_list=buf.data_ptr(), scale_a=buf.data_ptr(), scale_b=buf.data_ptr(), q=buf.data_ptr(),
                q_scale=buf.data_ptr(), workspace=buf.data_ptr(), workspace_bytes=1 << 20)
    ok = capi.MxGroupedSwigluQuantArgs(**base)
    assert lib.cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_can_implement(ctypes.byref(ok)) == 0
    for change in (dict(n=384), dict(q_scale=None), dict(q=buf.data_ptr() + 8), dict(group_count=0), dict(flags=1)):
        bad = capi.MxGroupedSwigluQuantArgs(**{**base, **change})
        assert lib.cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_can_implement(ctypes.byref(bad)) != 0, change
