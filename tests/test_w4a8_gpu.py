"""GPU parity of the W4A8 per-group kernel against the CPU oracle, called through the C ABI.

Default call: every CTA sums the scale groups in ascending order, exactly like the oracle: outputs must be
bit-identical.  With the CB200_W4A8_SPLIT_K flag the K range is split over a CTA cluster and fp32 partial sums
are added at the end: the sum is reassociated, so the bar is |got - want| <= max(1 bf16 ulp of want,
2^-20 x sa[m] x sum_g |acc_g| x sw[g,n]) -- one ulp wherever the terms do not cancel, the fp32 reassociation
bound where they do -- and at most 1 % of the outputs may differ at all.

So that parity does not hang on the oracle's choice of a fused multiply-add alone, every case (both modes) is
also compared with two references that do not share it: the exact sum in float64 and the unfused fp32 reading
(round the product, then the sum).  Bar for both: |got - ref| <= max(1 bf16 ulp of ref,
2^-20 x sa[m] x sum_g |acc_g x sw[g,n]|)."""
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


def _abs_terms(a, w, sw, sa, gs):
    """sa[m] * sum_g |acc_g[m,n]| * sw[g,n] in float64: the scale of the terms an output is summed from."""
    m, k = a.shape
    n = w.shape[1]
    total = np.zeros((m, n), np.float64)
    for g in range(k // gs):
        acc = a[:, g * gs:(g + 1) * gs].astype(np.int64) @ w[g * gs:(g + 1) * gs].astype(np.int64)
        total += np.abs(acc) * sw[g].astype(np.float64)
    return total * sa.astype(np.float64)[:, None]


def _check(got, want, exact, terms=None):
    if exact:
        assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} outputs differ"
        return
    dist = np.abs(_ordered(got) - _ordered(want))
    assert (dist != 0).mean() <= 0.01, f"{(dist != 0).mean():.4f} of the outputs differ"
    bad = dist > 1
    if bad.any():
        diff = np.abs(O.bf16_to_float(got).astype(np.float64) - O.bf16_to_float(want).astype(np.float64))
        assert terms is not None
        over = bad & (diff > terms * 2.0 ** -20)
        assert not over.any(), f"{over.sum()} outputs beyond both bounds (max {dist[over].max()} bf16 ulp)"


def _check_order_independent(got, a, packed, sw, sa, m, n, k, gs):
    unfused, exact64, mag = O.w4a8_per_group_readings(a, packed, sw, sa, m, n, k, gs)
    got64 = O.bf16_to_float(got).astype(np.float64)
    for name, ref in (("exact float64 sum", exact64), ("unfused fp32 reading", unfused.astype(np.float64))):
        ulp = np.spacing(np.abs(ref).astype(np.float32)).astype(np.float64) * 65536.0  # one bf16 step at ref
        bound = np.maximum(ulp, mag * 2.0 ** -20)
        over = np.abs(got64 - ref) > bound
        assert not over.any(), f"{over.sum()} of {over.size} outputs beyond the bound against the {name}"


@pytest.fixture(params=["default", "split_k"])
def exact(request):
    """Runs a test twice: default call (bit-exact) and with the split-K flag (reassociation bound)."""
    return request.param == "default"


def _run(cuda, a, packed, sw, sa, m, n, k, gs, split_k=False):
    import torch
    from catlass_b200 import capi
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()  # noqa: E731
    d = torch.full((m, n), -3.0, dtype=torch.bfloat16, device=cuda)
    capi.w4a8_matmul(dev(a), dev(packed), dev(sw), dev(sa), d, m, n, k, gs, split_k=split_k)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    return d.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("m,n,k,gs", [
    (128, 512, 1024, 128), (16, 256, 256, 128), (77, 200, 384, 128), (64, 128, 2048, 256),
    (130, 136, 512, 128), (1, 128, 128, 128), (257, 392, 8192, 1024), (130, 136, 2048, 256), (257, 64, 256, 128), (128, 4096, 2048, 128), (128, 256, 1024, 1024), (300, 384, 1280, 256), (33, 1000, 4096, 128), (40, 192, 1536, 512), (16, 64, 384, 128), (24, 128, 768, 384),
    # scale groups of several K blocks: odd block counts, a single group, an odd number of groups
    (48, 256, 1152, 1152), (128, 128, 640, 640), (20, 128, 1280, 640), (64, 256, 768, 256), (200, 256, 3840, 768),
])
def test_w4a8_per_group_matches_oracle(cuda, exact, m, n, k, gs):
    a, w, packed, sw, sa = _problem(m, n, k, gs, seed=m + n + k)
    got = _run(cuda, a, packed, sw, sa, m, n, k, gs, split_k=not exact)
    want = O.bf16_bits(O.w4a8_per_group(a, packed, sw, sa, m, n, k, gs))
    _check(got, want, exact, None if exact else _abs_terms(a, w, sw, sa, gs))
    _check_order_independent(got, a, packed, sw, sa, m, n, k, gs)


def test_w4a8_cancelling_groups_against_order_independent_references(cuda, exact):
    """Scales of both signs: group terms that nearly cancel are where the fused and the unfused reading, and
    any reordering, differ most."""
    m, n, k, gs = 96, 384, 4096, 128
    a, w, packed, sw, sa = _problem(m, n, k, gs, seed=99)
    rng = np.random.default_rng(100)
    sw = (sw * rng.choice([-1.0, 1.0], sw.shape)).astype(np.float32)
    got = _run(cuda, a, packed, sw, sa, m, n, k, gs, split_k=not exact)
    if exact:
        _check(got, O.bf16_bits(O.w4a8_per_group(a, packed, sw, sa, m, n, k, gs)), True)
    _check_order_independent(got, a, packed, sw, sa, m, n, k, gs)


def test_w4a8_extreme_values(cuda, exact):
    m, n, k, gs = 64, 128, 1024, 128
    a = np.full((m, k), -128, np.int8)
    w = np.full((k, n), -8, np.int8)
    w[:, ::2] = 7
    a[::2] = 127
    sw = np.ones((k // gs, n), np.float32)
    sa = np.ones(m, np.float32)
    packed = O.pack_int4_along_k(w)
    got = _run(cuda, a, packed, sw, sa, m, n, k, gs, split_k=not exact)
    _check(got, O.bf16_bits(O.w4a8_per_group(a, packed, sw, sa, m, n, k, gs)), exact,
           None if exact else _abs_terms(a, w, sw, sa, gs))


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
    got = _run(cuda, a, packed, sw, sa, m, n, k, gs, split_k=not exact)
    rng = np.random.default_rng(1)
    cols = np.unique(np.concatenate([[0, 127, 128, 255, 4095, 4096, 8191], rng.integers(0, n, 185)]))
    want = O.bf16_bits(O.w4a8_per_group(a, packed[cols], np.ascontiguousarray(sw[:, cols]), sa, m, len(cols), k, gs))
    _check(got[:, cols], want, exact, None if exact else _abs_terms(a, w[:, cols], sw[:, cols], sa, gs))
    _check_order_independent(np.ascontiguousarray(got[:, cols]), a, packed[cols], np.ascontiguousarray(sw[:, cols]), sa,
                             m, len(cols), k, gs)


def test_w4a8_invalid_arguments(cuda):
    import torch
    from catlass_b200 import capi
    z = torch.zeros(1 << 16, dtype=torch.int8, device=cuda)
    f = torch.ones(1 << 12, device=cuda)
    d = torch.empty((16, 128), dtype=torch.bfloat16, device=cuda)
    for k, gs in ((256, 64), (512, 192), (0, 128), (32768, 32768), (192, 128)):   # (192, 128): no workspace given
        with pytest.raises(capi.CallError) as e:
            capi.w4a8_matmul(z, z, f, f, d, 16, 128, k, gs)
        assert e.value.status == capi.INVALID
