"""cb200_mx_matmul_static: the MX matmul for hosts that cannot allocate device memory (an inference server
whose arena owns all of HBM, a loop that cannot afford cudaMalloc's device synchronisation).  Its scale
scratch is an array inside the library image, so the call takes no workspace.

The test calls it through the C ABI twice in a row with different problems and compares every output with
cb200_mx_matmul's (same kernels, so the comparison is exact; the MX tolerance of the other tests would
also hold).  The second call is smaller than the first and uses other data: stale bytes that the first call
left in the shared array must not leak into it.  Collected last on purpose."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


def _inputs(m, n, k, fmt, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    bt = rng.standard_normal((n, k)).astype(np.float32)
    aq, sfa = O.mx_quantize(a, fmt)
    bq, sfb = O.mx_quantize(bt, fmt)
    if fmt == O.MX_E2M1:
        aq = (aq[:, 0::2] | (aq[:, 1::2] << 4)).astype(np.uint8)
        bq = (bq[:, 0::2] | (bq[:, 1::2] << 4)).astype(np.uint8)
    return aq, sfa, bq, sfb


@pytest.mark.parametrize("fmt", [O.MX_E4M3, O.MX_E2M1])
def test_static_scratch_entry_matches_workspace_entry_twice(cuda, fmt):
    import torch
    from catlass_b200 import capi
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()  # noqa: E731
    for call, (m, n, k) in enumerate([(384, 520, 1024), (130, 136, 512)]):
        aq, sfa, bq, sfb = (dev(x) for x in _inputs(m, n, k, fmt, seed=100 + call + fmt))
        want = torch.full((m, n), -1.0, dtype=torch.bfloat16, device=cuda)
        got = torch.full((m, n), -2.0, dtype=torch.bfloat16, device=cuda)
        ws = torch.empty(capi.mx_matmul_workspace_size(m, n, k, fmt), dtype=torch.uint8, device=cuda)
        capi.mx_matmul(aq, bq, sfa, sfb, want, m, n, k, fmt, ws)
        capi.mx_matmul_static(aq, bq, sfa, sfb, got, m, n, k, fmt)
        st, code = capi.device_status()
        assert st == 0, f"device status {st} code {code:#x}"
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: outputs differ"


def test_static_scratch_entry_rejects_oversized_problems(cuda):
    import torch
    from catlass_b200 import capi
    limit = int(capi.load().cb200_mx_matmul_static_scratch_bytes())
    assert limit == 8 << 20
    m = n = 8192
    k = 32768  # (64 + 64) * 256 * 512 bytes = 16 MiB of re-tiled scales
    assert capi.mx_matmul_workspace_size(m, n, k, capi.MX_E4M3) > limit
    z = torch.zeros(1 << 12, dtype=torch.uint8, device=cuda)  # never dereferenced: the call must launch nothing
    before = capi.launch_count()
    with pytest.raises(capi.CallError) as e:
        capi.mx_matmul_static(z, z, z, z, z, m, n, k, capi.MX_E4M3)
    assert e.value.status == capi.SCRATCH_TOO_SMALL
    assert capi.launch_count() == before
