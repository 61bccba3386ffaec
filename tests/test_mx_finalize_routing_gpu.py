"""Grouped MXFP8 matmul with the finalize-routing epilogue fused in (the reference's
experimental/gmm/ascend950_fp8_mx_grouped_matmul_finalize_routing example, non-deterministic variant), through the
C ABI, against the golden's definition (gen_data_compare.py:718-757 of that example):

    out = 0;  out[offset:offset+bsdp] += weight * shared;  out.index_add_(0, row_index, logit[:, None] * (C + bias))

with C from the CPU oracle's dequantised matmul of each group's rows.  The additions into one output row happen in
any order on the device, so the comparison is relative (1e-3 of max(1, |expected|) scaled by the number of terms
that meet in a row), as for the other fp32 MX outputs."""
import numpy as np
import pytest

import oracle_lib as O
from test_ingest_gpu import _dev, _stored_operand, _stored_scales

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("sizes,n,k,trans_b,prefix,batch,bias,shared,i32", [
    ((10, 21, 32, 65), 128, 128, False, True, 16, False, False, False),   # the example's own run (4 128 128 128 ... 16 2)
    ((130, 0, 64, 257, 1), 264, 512, True, False, 64, True, True, False),
    ((5, 200, 129), 520, 330, False, True, 400, True, False, True),
    ((300, 77), 1024, 256, True, False, 48, False, True, True),
])
def test_mx_grouped_finalize_routing(cuda, sizes, n, k, trans_b, prefix, batch, bias, shared, i32):
    import torch
    from catlass_b200 import capi
    fmt = O.MX_E4M3
    rng = np.random.default_rng(sum(sizes) + n + k + batch)
    g, rows = len(sizes), sum(sizes)
    m = rows + 11
    a = (rng.standard_normal((m, k)) * 2.0).astype(np.float32)
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb = [], []
    c = np.zeros((m, n), np.float32)
    bias_h = rng.standard_normal((g, n)).astype(np.float32)
    bias_bits = O.bf16_bits(bias_h)
    bias_f = O.bf16_to_float(bias_bits)
    start = 0
    for e in range(g):
        bt = (rng.standard_normal((n, k)) * 2.0).astype(np.float32)
        q_e, s_e = O.mx_quantize(bt, fmt)
        bq.append(q_e)
        sfb.append(s_e)
        if sizes[e]:
            sl = slice(start, start + sizes[e])
            c[sl] = O.mx_matmul(aq[sl], sfa[sl], q_e, s_e, sizes[e], n, k, fmt)
            if bias:
                c[sl] += bias_f[e][None, :]
        start += sizes[e]
    logit = rng.standard_normal(m).astype(np.float32)
    row_index = (np.arange(m) % batch).astype(np.int64)        # the example's mapping
    row_index[3] = batch + 5                                   # out of range: dropped
    row_index[7] = -1
    dp = 2
    bsdp = batch // dp
    offset = batch - bsdp - 1 if shared else 0
    weight = np.float32(0.75)
    shared_bits = O.bf16_bits(rng.standard_normal((bsdp, n)).astype(np.float32))
    want = np.zeros((batch, n), np.float64)
    terms = np.zeros(batch, np.int64)
    if shared:
        want[offset:offset + bsdp] += (weight * O.bf16_to_float(shared_bits)).astype(np.float64)
    for p in range(rows):
        t = int(row_index[p])
        if 0 <= t < batch:
            want[t] += (logit[p] * c[p]).astype(np.float64)
            terms[t] += 1

    lb = capi.COLUMN_MAJOR if trans_b else capi.ROW_MAJOR
    gl = np.cumsum(sizes) if prefix else np.array(sizes)
    out = torch.full((batch, n), 123.0, dtype=torch.float32, device=cuda)   # stale contents must be overwritten
    ws = torch.empty(max(capi.mx_grouped_finalize_routing_workspace_size(m, n, k, g, batch, lb), 256),
                     dtype=torch.uint8, device=cuda)
    ri = row_index.astype(np.int32) if i32 else row_index
    capi.mx_grouped_finalize_routing(
        _dev(_stored_operand(aq, fmt, False)), _dev(np.stack([_stored_operand(q_e, fmt, not trans_b) for q_e in bq])),
        _dev(gl.astype(np.int64)), _dev(_stored_scales(sfa, False)),
        _dev(np.stack([_stored_scales(s_e, not trans_b) for s_e in sfb])), _dev(logit), _dev(ri), out, m, n, k, g, batch,
        ws, bias=_dev(bias_bits) if bias else None, shared_input=_dev(shared_bits) if shared else None,
        shared_rows=bsdp if shared else 0, shared_offset=offset, shared_weight=float(weight), layout_b=lb,
        group_list_kind=capi.GROUP_LIST_PREFIX_SUMS if prefix else capi.GROUP_LIST_SIZES,
        row_index_type=capi.GROUP_LIST_INT32 if i32 else capi.GROUP_LIST_INT64)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    got = out.cpu().numpy().astype(np.float64)
    tol = 1e-3 * np.maximum(1.0, np.abs(want)) * np.maximum(terms, 1)[:, None]
    assert np.isfinite(got).all() and (np.abs(got - want) <= tol).all(), \
        f"max excess {(np.abs(got - want) / tol).max():.3f}"
    untouched = (terms == 0) & ~((np.arange(batch) >= offset) & (np.arange(batch) < offset + bsdp) & shared)
    assert (got[untouched] == 0).all()


@pytest.mark.parametrize("sizes,n,k,batch,bias,shared,i32,top", [
    ((130, 0, 64, 257, 1), 264, 512, 64, True, True, False, 8),
    ((700, 37, 600), 1024, 128, 1, False, False, True, 600),     # more rows per token than the in-block sort holds
    ((5, 200, 129), 520, 330, 400, True, False, True, 1),
])
def test_mx_grouped_finalize_routing_deterministic(cuda, sizes, n, k, batch, bias, shared, i32, top):
    """CB200_ROUTING_DETERMINISTIC: the same bits on every run, and exactly the golden's arithmetic on the library's
    own C: out = 0 + weight * shared, then += logit[p] * (C[p] + bias) for the rows of a token in ascending p
    (gen_data_compare.py:744-757), with C taken from the grouped matmul's fp32 output."""
    import torch
    from catlass_b200 import capi
    fmt = O.MX_E4M3
    rng = np.random.default_rng(sum(sizes) + n + batch)
    g, rows = len(sizes), sum(sizes)
    m = rows + 7
    aq, sfa = O.mx_quantize((rng.standard_normal((m, k)) * 2.0).astype(np.float32), fmt)
    bq, sfb = zip(*[O.mx_quantize((rng.standard_normal((n, k)) * 2.0).astype(np.float32), fmt) for _ in range(g)])
    a_dev = _dev(_stored_operand(aq, fmt, False))
    b_dev = _dev(np.stack([_stored_operand(q_e, fmt, False) for q_e in bq]))
    sa_dev = _dev(_stored_scales(sfa, False))
    sb_dev = _dev(np.stack([_stored_scales(s_e, False) for s_e in sfb]))
    gl_dev = _dev(np.array(sizes, np.int64))
    logit = rng.standard_normal(m).astype(np.float32)
    row_index = rng.integers(0, batch, m).astype(np.int64)
    row_index[1] = -3
    row_index[2] = batch
    bias_bits = O.bf16_bits(rng.standard_normal((g, n)).astype(np.float32))
    bsdp = max(batch // 2, 1)
    offset = batch - bsdp
    shared_bits = O.bf16_bits(rng.standard_normal((bsdp, n)).astype(np.float32))
    weight = np.float32(-1.25)

    c = torch.zeros((m, n), dtype=torch.float32, device=cuda)
    ws = torch.empty(max(capi.mx_grouped_matmul_workspace_size(m, n, k, g, fmt), 256), dtype=torch.uint8, device=cuda)
    capi.mx_grouped_matmul(a_dev, b_dev, gl_dev, sa_dev, sb_dev, c, m, n, k, g, fmt, ws, out_f32=True)
    c_host = c.cpu().numpy()
    want = np.zeros((batch, n), np.float32)
    if shared:
        want[offset:offset + bsdp] += weight * O.bf16_to_float(shared_bits)
    group_of = np.repeat(np.arange(g), sizes)
    bias_f = O.bf16_to_float(bias_bits)
    for p in range(rows):
        t = int(row_index[p])
        if 0 <= t < batch:
            y = c_host[p] + bias_f[group_of[p]] if bias else c_host[p]
            want[t] = want[t] + logit[p] * y

    outs = []
    ws2 = torch.empty(max(capi.mx_grouped_finalize_routing_workspace_size(m, n, k, g, batch, deterministic=True), 256),
                      dtype=torch.uint8, device=cuda)
    ri = row_index.astype(np.int32) if i32 else row_index
    for _ in range(2):
        out = torch.full((batch, n), 5.0, dtype=torch.float32, device=cuda)
        capi.mx_grouped_finalize_routing(
            a_dev, b_dev, gl_dev, sa_dev, sb_dev, _dev(logit), _dev(ri), out, m, n, k, g, batch, ws2,
            bias=_dev(bias_bits) if bias else None, shared_input=_dev(shared_bits) if shared else None,
            shared_rows=bsdp if shared else 0, shared_offset=offset, shared_weight=float(weight),
            row_index_type=capi.GROUP_LIST_INT32 if i32 else capi.GROUP_LIST_INT64, deterministic=True)
        st, code = capi.device_status()
        assert st == 0, f"device status {st} code {code:#x}"
        outs.append(out.cpu().numpy())
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32)), "two runs differ"
    assert np.array_equal(outs[0].view(np.uint32), want.view(np.uint32)), \
        f"{(outs[0].view(np.uint32) != want.view(np.uint32)).sum()} values differ from the golden's order"


def test_mx_grouped_finalize_routing_rejects(cuda):
    import ctypes
    import torch
    from catlass_b200 import capi
    lib = capi.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device=cuda)
    base = dict(m=128, n=512, k=256, group_count=2, layout_b=capi.COLUMN_MAJOR, group_list_type=capi.GROUP_LIST_INT64,
                group_list_kind=capi.GROUP_LIST_SIZES, row_index_type=capi.GROUP_LIST_INT64, batch=32, shared_rows=16,
                shared_offset=8, shared_weight=1.0, a=buf.data_ptr(), b=buf.data_ptr(), group_list=buf.data_ptr(),
                scale_a=buf.data_ptr(), scale_b=buf.data_ptr(), logit=buf.data_ptr(), row_index=buf.data_ptr(),
                bias=buf.data_ptr(), shared_input=buf.data_ptr(), out=buf.data_ptr(), workspace=buf.data_ptr(),
                workspace_bytes=1 << 20)
    ok = capi.MxGroupedFinalizeRoutingArgs(**base)
    assert lib.cb200_mx_grouped_matmul_finalize_routing_can_implement(ctypes.byref(ok)) == 0
    for change in (dict(batch=0), dict(logit=None), dict(row_index=None), dict(shared_offset=20), dict(flags=2),
                   dict(row_index_type=7), dict(out=buf.data_ptr() + 4), dict(row_index=buf.data_ptr() + 4)):
        bad = capi.MxGroupedFinalizeRoutingArgs(**{**base, **change})
        assert lib.cb200_mx_grouped_matmul_finalize_routing_can_implement(ctypes.byref(bad)) != 0, change
