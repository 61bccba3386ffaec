"""GPU parity of the MXFP8 / MXFP4 block-scaled matmul against the CPU oracle (fp32 dequantised matmul, the
reference's golden), called through the C ABI.  Bar: |got - want| <= 1e-2 * max(1, |want|) for every output."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2


def _quantized(m, n, k, fmt, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    bt = rng.standard_normal((n, k)).astype(np.float32)  # column-major B: one row of bt per column of B
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb = O.mx_quantize(bt, fmt)
    return aq, sfa, bq, sfb


def _device_operand(codes, fmt):
    if fmt == O.MX_E2M1:
        return (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return codes


def _run(cuda, aq, sfa, bq, sfb, m, n, k, fmt):
    import torch
    from catlass_b200 import capi
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()  # noqa: E731
    d = torch.full((m, n), -3.0, dtype=torch.bfloat16, device=cuda)
    ws = torch.empty(max(capi.mx_matmul_workspace_size(m, n, k, fmt), 256), dtype=torch.uint8, device=cuda)
    capi.mx_matmul(dev(_device_operand(aq, fmt)), dev(_device_operand(bq, fmt)), dev(sfa), dev(sfb), d, m, n, k,
                   fmt, ws)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    return d.float().cpu().numpy()


def _check(got, want, what):
    err = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    assert np.isfinite(got).all(), f"{what}: non-finite outputs"
    assert err.max() <= REL_TOL, f"{what}: max rel err {err.max():.4f} at {np.unravel_index(err.argmax(), err.shape)}"


@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (256, 512, 1024), (300, 264, 512), (1, 8, 256),
                                   (129, 136, 1792)])
def test_mx_matmul_matches_oracle(cuda, fmt, m, n, k):
    aq, sfa, bq, sfb = _quantized(m, n, k, fmt, seed=m + n + k + fmt)
    got = _run(cuda, aq, sfa, bq, sfb, m, n, k, fmt)
    want = O.mx_matmul(aq, sfa, bq, sfb, m, n, k, fmt)
    _check(got, want, f"mx fmt={fmt} {m}x{n}x{k}")


@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_mx_scales_are_applied_per_block(cuda, fmt):
    """Every 32-wide K block gets its own exponent: scales spanning 2^-10 .. 2^10 along K and across rows."""
    m, n, k = 128, 128, 512
    rng = np.random.default_rng(5)
    a = rng.standard_normal((m, k)).astype(np.float32)
    bt = rng.standard_normal((n, k)).astype(np.float32)
    a *= np.repeat(2.0 ** rng.integers(-10, 11, (m, k // 32)), 32, axis=1).astype(np.float32)
    bt *= np.repeat(2.0 ** rng.integers(-10, 11, (n, k // 32)), 32, axis=1).astype(np.float32)
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb = O.mx_quantize(bt, fmt)
    assert len(np.unique(sfa)) > 10
    got = _run(cuda, aq, sfa, bq, sfb, m, n, k, fmt)
    want = O.mx_matmul(aq, sfa, bq, sfb, m, n, k, fmt)
    err = np.abs(got - want) / np.maximum(np.abs(want).max() * 1e-3, np.abs(want))
    assert err.max() <= REL_TOL, err.max()


@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_mx_full_size_sampled(cuda, fmt):
    """M=N=K=8192 on the GPU; the oracle checks a 96 x 96 sample of rows and columns that includes tile
    edges (dequantised fp32 matmul over the full K)."""
    m = n = k = 8192
    aq, sfa, bq, sfb = _quantized(m, n, k, fmt, seed=81 + fmt)
    got = _run(cuda, aq, sfa, bq, sfb, m, n, k, fmt)
    rng = np.random.default_rng(2)
    rows = np.unique(np.concatenate([[0, 127, 128, 4095, 4096, 8191], rng.integers(0, m, 90)]))
    cols = np.unique(np.concatenate([[0, 127, 128, 255, 4096, 8191], rng.integers(0, n, 90)]))
    want = O.mx_matmul(aq[rows], sfa[rows], bq[cols], sfb[cols], len(rows), len(cols), k, fmt)
    _check(got[np.ix_(rows, cols)], want, f"mx full fmt={fmt}")


def test_mx_invalid_arguments(cuda):
    import torch
    from catlass_b200 import capi
    z = torch.zeros(1 << 16, dtype=torch.uint8, device=cuda)
    d = torch.empty((128, 128), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(capi.CallError) as e:
        capi.mx_matmul(z, z, z, z, d, 128, 128, 256, 7, z)   # unknown element format
    assert e.value.status == capi.INVALID
    with pytest.raises(capi.CallError):
        capi.mx_matmul(z, z, z, z, d, 128, 128, 256, capi.MX_E2M1, z, layout_a=5)
    with pytest.raises(capi.CallError):
        capi.mx_matmul(z, z, z, z, d, 128, 128, 256, capi.MX_E4M3, None)  # no workspace
    with pytest.raises(capi.CallError):
        capi.mx_matmul(z, z, z, z, d, 128, 128, 192, capi.MX_E4M3, z[:4096])  # ragged k: workspace too small
