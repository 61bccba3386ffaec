"""GPU parity of the W4A8 per-group kernel against the CPU oracle, called through the C ABI.

With one CTA per channel tile (CB200_W4A8_SPLITS=1) the kernel performs the oracle's operations in the
oracle's order and must be bit-exact.  With the K range split over a cluster (the default for shapes that
would otherwise leave SMs idle) the fp32 partial sums are added in another order: outputs must then agree
to 1 bf16 ulp, and nearly all of them exactly."""
import os

import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


def _problem(m, n, k, gs, seed):
    rng = np.random.default_rng(seed)
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    sw = rng.uniform(1e-3, 1e-2, (k // gs, n)).astype(np.float32)
    sa = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    return a, w, O.pack_int4_along_k(w), sw, sa


def _ordered(bits):
    """bf16 bit patterns -> integers whose difference is the distance in ulps."""
    b = bits.astype(np.int32)
    return np.where(b & 0x8000, -(b & 0x7FFF), b)


def _check(got, want, exact):
    if exact:
        assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} outputs differ"
        return
    dist = np.abs(_ordered(got) - _ordered(want))
    assert dist.max() <= 1, f"max distance {dist.max()} bf16 ulp"   # tolerance: 1 bf16 ulp
    assert (dist != 0).mean() <= 0.01, f"{(dist != 0).mean():.4f} of the outputs are off by one ulp"


@pytest.fixture(params=["split", "single"])
def exact(request):
    """Runs a test twice: with the default K split (1-ulp tolerance) and with one CTA per tile (bit-exact)."""
    old = os.environ.get("CB200_W4A8_SPLITS")
    if request.param == "single":
        os.environ["CB200_W4A8_SPLITS"] = "1"
    else:
        os.environ.pop("CB200_W4A8_SPLITS", None)
    yield request.param == "single"
    if old is None:
        os.environ.pop("CB200_W4A8_SPLITS", None)
    else:
        os.environ["CB200_W4A8_SPLITS"] = old


def _run(cuda, a, packed, sw, sa, m, n, k, gs):
    import torch
    from catlass_b200 import capi
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()  # noqa: E731
    d = torch.full((m, n), -3.0, dtype=torch.bfloat16, device=cuda)
    capi.w4a8_matmul(dev(a), dev(packed), dev(sw), dev(sa), d, m, n, k, gs)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    return d.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("m,n,k,gs", [
    (128, 512, 1024, 128), (16, 256, 256, 128), (77, 200, 384, 128), (64, 128, 2048, 256),
    (130, 136, 512, 128), (1, 128, 128, 128), (128, 4096, 2048, 128), (128, 256, 1024, 1024), (300, 384, 1280, 256), (33, 1000, 4096, 128), (40, 192, 1536, 512), (16, 64, 384, 128), (24, 128, 768, 384),
])
def test_w4a8_per_group_matches_oracle(cuda, exact, m, n, k, gs):
    a, w, packed, sw, sa = _problem(m, n, k, gs, seed=m + n + k)
    got = _run(cuda, a, packed, sw, sa, m, n, k, gs)
    want = O.bf16_bits(O.w4a8_per_group(a, packed, sw, sa, m, n, k, gs))
    _check(got, want, exact)


def test_w4a8_extreme_values(cuda, exact):
    m, n, k, gs = 64, 128, 1024, 128
    a = np.full((m, k), -128, np.int8)
    w = np.full((k, n), -8, np.int8)
    w[:, ::2] = 7
    a[::2] = 127
    sw = np.ones((k // gs, n), np.float32)
    sa = np.ones(m, np.float32)
    packed = O.pack_int4_along_k(w)
    got = _run(cuda, a, packed, sw, sa, m, n, k, gs)
    _check(got, O.bf16_bits(O.w4a8_per_group(a, packed, sw, sa, m, n, k, gs)), exact)


def test_w4a8_per_tensor_mode_matches_reference_formula(cuda):
    """The reference's example 32: out = 1.5 * (A @ W), one scalar for the whole tensor."""
    m, n, k = 40, 256, 1024
    a, w, packed, _, _ = _problem(m, n, k, k, seed=32)
    got = _run(cuda, a, packed, np.ones((1, n), np.float32), np.full(m, 1.5, np.float32), m, n, k, k)
    want = O.bf16_bits(O.w4a8_per_tensor(a, packed, 1.5, m, n, k))
    assert np.array_equal(got, want)


def test_w4a8_full_config_sampled_columns(cuda, exact):
    """M=128, N=8192, K=8192, group 128 at full size; the oracle checks 192 columns spread over the tiles,
    including both edges of several 128-column tiles."""
    m, n, k, gs = 128, 8192, 8192, 128
    a, w, packed, sw, sa = _problem(m, n, k, gs, seed=7)
    got = _run(cuda, a, packed, sw, sa, m, n, k, gs)
    rng = np.random.default_rng(1)
    cols = np.unique(np.concatenate([[0, 127, 128, 255, 4095, 4096, 8191], rng.integers(0, n, 185)]))
    want = O.bf16_bits(O.w4a8_per_group(a, packed[cols], np.ascontiguousarray(sw[:, cols]), sa, m, len(cols), k, gs))
    _check(got[:, cols], want, exact)


def test_w4a8_invalid_arguments(cuda):
    import torch
    from catlass_b200 import capi
    z = torch.zeros(1 << 16, dtype=torch.int8, device=cuda)
    f = torch.ones(1 << 12, device=cuda)
    d = torch.empty((16, 128), dtype=torch.bfloat16, device=cuda)
    for k, gs in ((192, 128), (256, 64), (256, 192), (0, 128), (32768, 32768)):
        with pytest.raises(capi.CallError) as e:
            capi.w4a8_matmul(z, z, f, f, d, 16, 128, k, gs)
        assert e.value.status == capi.INVALID
