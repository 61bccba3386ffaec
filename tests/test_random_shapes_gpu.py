"""Seeded sweep of random shapes over every entry point against the CPU oracle (same bars as the per-op
tests: int32 bit-exact and bf16 <= 1 ulp for W8A8, bit-exact for the default W4A8 call, the reassociation
bound for W4A8 with the split-K flag, rel-err <= 1e-2 for MX).  Shapes mix tile-aligned and ragged sizes,
few-token and multi-tile problems, empty and tiny groups."""
import numpy as np
import pytest

import oracle_lib as O
import test_mx_gpu as TM
import test_w4a8_gpu as T4
import test_w8a8_gpu as T8

pytestmark = pytest.mark.gpu


def _case(cuda, rng):
    pick = lambda xs: int(rng.choice(xs))  # noqa: E731
    kind = pick([0, 1, 2, 3, 4])
    seed = int(rng.integers(1 << 30))
    if kind == 0:    # dense W8A8: few-token, single-tile and pair kernels by shape
        m = pick([1, 7, 16, 33, 100, 128, 129, 200, 256, 300, 513])
        n = pick([8, 24, 128, 136, 264, 520, 1000])
        k = 16 * pick([1, 3, 8, 9, 32, 61, 128])
        col = bool(pick([0, 1]))
        if not col and n % 16:
            n = (n + 15) // 16 * 16
        T8.run_dense(cuda, m, n, k, col, seed=seed)
    elif kind == 1:  # grouped W8A8
        g = pick([1, 2, 5, 17])
        n = 16 * pick([1, 8, 17, 33])
        k = 16 * pick([2, 8, 24, 65])
        col = bool(pick([0, 1]))
        sizes = rng.integers(0, 400, size=g)
        sizes[rng.integers(0, g)] = pick([0, 1, 255, 256, 257, 700])
        T8.run_grouped(cuda, sizes, n, k, col, seed=seed, m_capacity=int(sizes.sum()) + pick([0, 5, 130]),
                       list_i32=bool(pick([0, 1])))
    elif kind == 2:  # W4A8, default (bit-exact) or split-K
        m = pick([1, 15, 16, 17, 64, 100, 128, 130, 257])
        n = pick([8, 64, 128, 136, 392, 1024])
        gs = 128 * pick([1, 1, 2, 3, 8])
        k = gs * pick([1, 2, 3, 5, 8])
        exact = bool(pick([0, 1]))
        a, w, packed, sw, sa = T4._problem(m, n, k, gs, seed=seed)
        got = T4._run(cuda, a, packed, sw, sa, m, n, k, gs, split_k=not exact)
        T4._check(got, O.bf16_bits(O.w4a8_per_group(a, packed, sw, sa, m, n, k, gs)), exact,
                  None if exact else T4._abs_terms(a, w, sw, sa, gs))
    else:            # MXFP8 / MXFP4
        fmt = O.MX_E4M3 if kind == 3 else O.MX_E2M1
        m = pick([1, 100, 128, 129, 300, 640])
        n = pick([8, 136, 256, 264, 520, 1032])
        k = (128 if fmt == O.MX_E4M3 else 256) * pick([1, 2, 3, 7])
        aq, sfa, bq, sfb = TM._quantized(m, n, k, fmt, seed=seed)
        got = TM._run(cuda, aq, sfa, bq, sfb, m, n, k, fmt)
        TM._check(got, O.mx_matmul(aq, sfa, bq, sfb, m, n, k, fmt), f"mx fmt={fmt} m={m} n={n} k={k}")


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes(cuda, seed):
    rng = np.random.default_rng(seed)
    for _ in range(120):
        _case(cuda, rng)
