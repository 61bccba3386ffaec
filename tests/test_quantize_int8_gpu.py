"""Per-token int8 quantisation of activations on the device (cb200_quantize_per_token_int8) against the CPU oracle:
codes and scales bit-exact, fp32 and bf16 inputs, padded row pitch, all-zero rows, rows whose largest element is
negative; then the quantised operand is fed to cb200_quant_matmul and the product compared with the oracle's
matmul on the same codes (the two entry points compose without a conversion in between)."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


def _bf16_round(x):
    return O.bf16_to_float(O.bf16_bits(x))


@pytest.mark.parametrize("rows,k,pitch,bf16", [
    (1, 16, 0, False), (7, 48, 0, False), (33, 512, 0, True), (130, 7168, 0, True), (64, 1040, 1056, False),
    (19, 2064, 2080, True), (300, 4096, 0, False),
    (5, 8192, 0, False), (9, 16400, 16416, True),   # rows of 28 to 112 KB: one CTA per row, a segment per warp
    (400, 16384, 0, True), (2, 28672, 0, False),    # ... more rows than CTAs; the longest such row
    (3, 65536, 0, True),                            # beyond that: the plain-load kernel
    (1500, 256, 0, True),                            # more rows than warps in the grid: several rows per warp
])
def test_quantize_per_token_int8_matches_the_oracle(cuda, rows, k, pitch, bf16):
    import torch
    from catlass_b200 import capi
    rng = np.random.default_rng(rows * 31 + k)
    x = (rng.standard_normal((rows, k)) * rng.uniform(1e-3, 50.0, (rows, 1))).astype(np.float32)
    if rows > 2:
        x[1] = 0.0                       # an all-zero row
        x[2, 5] = -np.abs(x[2]).max() * 3  # the largest magnitude is negative
    if k >= 48:
        x[0, :32] = np.float32(0.5) * np.abs(x[0]).max() / 127 * np.arange(-16, 16)  # products on .5 grid points
    if bf16:
        x = _bf16_round(x)
    want_q, want_s = O.quantize_per_token_int8(x)
    p = pitch or k
    host = np.zeros((rows, p), np.float32)
    host[:, :k] = x
    xd = torch.from_numpy(host).to(cuda)
    if bf16:
        xd = xd.to(torch.bfloat16)
    q = torch.full((rows, k), 0x55, dtype=torch.int8, device=cuda)
    s = torch.full((rows,), -1.0, dtype=torch.float32, device=cuda)
    capi.quantize_per_token_int8(xd, q, s, rows, k, x_type=capi.DTYPE_BF16 if bf16 else capi.DTYPE_F32, x_pitch=pitch)
    torch.cuda.synchronize()
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32)), "scales differ"
    got_q = q.cpu().numpy()
    assert np.array_equal(got_q, want_q), f"{(got_q != want_q).sum()} of {got_q.size} codes differ"


def test_quantized_activations_feed_the_w8a8_matmul(cuda):
    import torch
    from catlass_b200 import capi
    rng = np.random.default_rng(5)
    m, n, k = 200, 384, 1024
    x = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.integers(-127, 128, (n, k), dtype=np.int8)          # column-major B: [n][k]
    scale = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    xd = torch.from_numpy(x).to(cuda)
    q = torch.empty((m, k), dtype=torch.int8, device=cuda)
    pt = torch.empty((m,), dtype=torch.float32, device=cuda)
    capi.quantize_per_token_int8(xd, q, pt, m, k)
    d = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
    capi.quant_matmul(q, torch.from_numpy(b).to(cuda), torch.from_numpy(scale).to(cuda), pt, d, m, n, k)
    torch.cuda.synchronize()
    want_q, want_s = O.quantize_per_token_int8(x)
    want = O.bf16_bits(O.quant_matmul(want_q, b, scale, want_s, m, n, k))
    got = d.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, want)


def test_quantize_per_token_int8_rejects(cuda):
    import torch
    from catlass_b200 import capi
    x = torch.zeros((4, 64), dtype=torch.float32, device=cuda)
    q = torch.zeros((4, 64), dtype=torch.int8, device=cuda)
    s = torch.zeros((4,), dtype=torch.float32, device=cuda)
    for rows, k, pitch in ((4, 24, 0), (4, 32, 16), (4, 32, 34)):  # k % 16, pitch < k, rows off 16-byte boundaries
        with pytest.raises(capi.CallError):
            capi.quantize_per_token_int8(x, q, s, rows, k, x_pitch=pitch)
