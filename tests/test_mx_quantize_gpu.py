"""cb200_mx_quantize on the GPU against the CPU oracle's quantiser (itself pinned to the reference's generators):
element codes and scale bytes must be identical, for E4M3 and E2M1, fp32 and bf16 inputs, ragged K, zero blocks,
saturating and tiny values; and its output must feed cb200_mx_matmul unchanged."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


def _inputs(rows, k, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    x *= np.float32(2.0) ** rng.integers(-12, 13, (rows, 1)).astype(np.float32)   # a spread of row magnitudes
    if rows > 4 and k >= 64:
        x[1, :32] = 0.0                       # an all-zero block
        x[2, 5] = 3.0e4                       # saturates its block's grid
        x[3, 32:64] *= np.float32(1.0e-20)    # tiny values (exponent clamp)
        x[4, :] = np.float32(448.0)           # exactly the largest E4M3 value
    # exact grid ties: halves between neighbouring codes
    x[0, :min(k, 8)] = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], np.float32)[:min(k, 8)]
    if rows > 8 and k >= 128:
        # negative ties, and with a block maximum of 256 (E4M3 exponent 0) / 4 (E2M1 exponent 0): ties on the normal
        # E4M3 grid (half way between neighbours 1/8 apart per octave), values in the subnormal E4M3 range
        # (multiples and half-multiples of 2^-9), negative values that round to zero
        x[5, :32] = 0.0
        x[5, 0] = 256.0
        x[5, 1:17] = np.array([1.0625, -1.0625, 1.1875, -1.1875, 2.125, 2.375, 0.5625, 432.0, 440.0, 232.0,
                               2.5 / 512, -2.5 / 512, 3.5 / 512, 0.5 / 512, -0.5 / 512, -0.2 / 512], np.float32)
        x[5, 17:21] = np.array([7.5 / 512, 8.5 / 512, 1.0 / 64 + 1.0 / 1024, 1.0 / 64 + 3.0 / 1024], np.float32)
        x[6, 32:64] = 0.0
        x[6, 32] = 4.0
        x[6, 33:47] = np.array([-0.25, -0.75, -1.25, -1.75, -2.5, -3.5, 0.1, -0.1, -0.26, 0.74, 0.76, 3.49, 3.51,
                                -5.0], np.float32)
        # fp32 neighbours of half-way points (one unit in the last place either side): block maximum 256 (E4M3
        # exponent 0) in the first block, 4 (E2M1 exponent 0) in the second
        mids8 = np.array([1.0625, 1.1875, 17.0, 440.0, 2.5 / 512, 7.5 / 512, 0.5 / 512, 1.0 / 64 + 1.0 / 1024, 120.0],
                         np.float32)
        mids4 = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
        x[7, :64] = 0.0
        x[7, 0] = 256.0
        x[7, 1:10] = np.nextafter(mids8, np.float32(np.inf))
        x[7, 10:19] = -np.nextafter(mids8, np.float32(0.0))
        x[7, 19:28] = np.nextafter(mids8, np.float32(0.0))
        x[7, 32] = 4.0
        x[7, 33:40] = np.nextafter(mids4, np.float32(np.inf))
        x[7, 40:47] = np.nextafter(mids4, np.float32(0.0))
        x[7, 47:54] = -np.nextafter(mids4, np.float32(np.inf))
    return x


def _run(cuda, x, fmt, bf16):
    import torch
    from catlass_b200 import capi
    rows, k = x.shape
    xt = torch.from_numpy(x).cuda()
    if bf16:
        xt = xt.to(torch.bfloat16)
    ks = ((k + 31) // 32 + 1) // 2 * 2
    q_cols = (k + 1) // 2 if fmt == O.MX_E2M1 else k
    q = torch.full((rows, q_cols), 0xAA, dtype=torch.uint8, device=cuda)
    sf = torch.full((rows, ks), 0xAA, dtype=torch.uint8, device=cuda)
    capi.mx_quantize(xt, q, sf, rows, k, fmt, x_type=capi.DTYPE_BF16 if bf16 else capi.DTYPE_F32)
    assert capi.device_status()[0] == 0
    ref_in = xt.float().cpu().numpy() if bf16 else x
    return q.cpu().numpy(), sf.cpu().numpy(), ref_in


@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("rows,k", [(64, 1024), (7, 129), (33, 63), (5, 2), (300, 4096), (16, 96), (1200, 7168),
                                     (9, 14400), (40, 64), (3, 16384), (10, 7200)])
def test_mx_quantize_matches_the_oracle_bit_for_bit(cuda, fmt, bf16, rows, k):
    x = _inputs(rows, k, seed=rows + k)
    q, sf, ref_in = _run(cuda, x, fmt, bf16)
    want_q, want_sf = O.mx_quantize(ref_in, fmt)
    blocks = want_sf.shape[1]
    assert np.array_equal(sf[:, :blocks], want_sf)
    assert (sf[:, blocks:] == 127).all()
    if fmt == O.MX_E2M1:
        kk = want_q.shape[1]
        padded = np.concatenate([want_q, np.zeros((rows, kk & 1), np.uint8)], axis=1)
        want_q = (padded[:, 0::2] | (padded[:, 1::2] << 4)).astype(np.uint8)
    assert np.array_equal(q, want_q), f"{(q != want_q).sum()} of {q.size} codes differ"


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_mx_quantize_values_around_every_half_way_point(cuda, fmt, bf16):
    """fp32 inputs a few units in the last place either side of (and exactly on) every half-way point and every
    code of the format, both signs, with the block's exponent pinned to 0 by its first element: the kernel's cut to
    12 bits and its shift towards zero must not move a value across a half-way point.  (With bf16 inputs the
    neighbours collapse onto bf16 values: the points themselves and their bf16 neighbourhood.)"""
    if fmt == O.MX_E4M3:
        codes = np.array(sorted({O.lib().orc_e4m3_to_float(c) for c in range(0x7F)}), np.float64)
        top = 256.0
    else:
        codes = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float64)
        top = 4.0
    mids = (codes[:-1] + codes[1:]) / 2
    points = np.concatenate([codes, mids]).astype(np.float32)
    vals = []
    for j in (-3, -1, 0, 1, 2):
        v = points.copy()
        for _ in range(abs(j)):
            v = np.nextafter(v, np.float32(np.inf if j > 0 else -np.inf)).astype(np.float32)
        vals.append(v)
    vals = np.concatenate(vals)
    vals = np.concatenate([vals, -vals]).astype(np.float32)
    per_block = 31
    blocks = (len(vals) + per_block - 1) // per_block
    blocks = (blocks + 1) // 2 * 2                      # k a multiple of 64
    x = np.zeros((blocks * 32,), np.float32)
    x[0::32] = top
    body = np.zeros((blocks * per_block,), np.float32)
    body[:len(vals)] = vals
    x.reshape(blocks, 32)[:, 1:] = body.reshape(blocks, per_block)
    x = np.tile(x[None, :], (3, 1))
    if bf16:
        # bf16 neighbours of the points as well: one bf16 unit in the last place is 2^16 fp32 units
        bits = x.view(np.uint32)
        sizable = np.abs(x) > 1e-6   # (zeros and the denormal neighbours of zero stay as they are)
        up = np.where(sizable, bits + np.uint32(0x10000), bits).view(np.float32)
        down = np.where(sizable, bits - np.uint32(0x10000), bits).view(np.float32)
        x = np.concatenate([x, up, down], axis=0)
        x[:, 0::32] = top
    q, sf, ref_in = _run(cuda, x, fmt, bf16)
    want_q, want_sf = O.mx_quantize(ref_in, fmt)
    assert np.array_equal(sf[:, :want_sf.shape[1]], want_sf)
    if fmt == O.MX_E2M1:
        want_q = (want_q[:, 0::2] | (want_q[:, 1::2] << 4)).astype(np.uint8)
    bad = np.argwhere(q != want_q)
    assert len(bad) == 0, (f"{len(bad)} of {q.size} codes differ, first at {bad[:4].tolist()}: inputs "
                           f"{[float(ref_in[r, c if fmt != O.MX_E2M1 else 2 * c]) for r, c in bad[:4]]}, got "
                           f"{[int(q[r, c]) for r, c in bad[:4]]}, want {[int(want_q[r, c]) for r, c in bad[:4]]}")


@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_quantize_then_matmul(cuda, fmt):
    """Activations quantised on the device go straight into the MX matmul (same layouts, no host step)."""
    import torch
    from catlass_b200 import capi
    m, n, k = 200, 264, 1024
    rng = np.random.default_rng(3)
    a = rng.standard_normal((m, k)).astype(np.float32)
    bt = rng.standard_normal((n, k)).astype(np.float32)
    ks = k // 32
    q_cols = k // 2 if fmt == O.MX_E2M1 else k
    dev = lambda z: torch.from_numpy(np.ascontiguousarray(z)).cuda()  # noqa: E731
    qa = torch.empty((m, q_cols), dtype=torch.uint8, device=cuda)
    qb = torch.empty((n, q_cols), dtype=torch.uint8, device=cuda)
    sa = torch.empty((m, ks), dtype=torch.uint8, device=cuda)
    sb = torch.empty((n, ks), dtype=torch.uint8, device=cuda)
    capi.mx_quantize(dev(a), qa, sa, m, k, fmt)
    capi.mx_quantize(dev(bt), qb, sb, n, k, fmt)
    d = torch.empty((m, n), dtype=torch.float32, device=cuda)
    ws = torch.empty(capi.mx_matmul_workspace_size(m, n, k, fmt), dtype=torch.uint8, device=cuda)
    capi.mx_matmul(qa, qb, sa, sb, d, m, n, k, fmt, ws, out_f32=True)
    assert capi.device_status()[0] == 0
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb = O.mx_quantize(bt, fmt)
    want = O.mx_matmul(aq, sfa, bq, sfb, m, n, k, fmt)
    err = np.abs(d.cpu().numpy() - want) / np.maximum(1.0, np.abs(want))
    assert err.max() <= 1e-3, err.max()
