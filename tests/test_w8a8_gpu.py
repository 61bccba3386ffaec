"""GPU parity of the W8A8 kernels against the CPU oracle, called through the C ABI.

Bars: int32 accumulators bit-exact; bf16 outputs within 1 bf16 ulp of the fp32 golden rounded to bf16
(the kernels reproduce the golden's operation order, so the observed difference is 0 ulp and the tests
also report the count of non-identical outputs).
"""
import numpy as np
import pytest

import oracle_lib as O
import problems as P

pytestmark = pytest.mark.gpu

BF16_ULP_TOL = 1  # units in the last place of bf16


def _torch():
    import torch
    return torch


def _dev(x):
    torch = _torch()
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf16_ulp_diff(got_bits, want_bits):
    """Distance in bf16 representable steps (sign-magnitude mapped to a line)."""
    def lin(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    return np.abs(lin(got_bits) - lin(want_bits))


def check_bf16(got_bits, want_f32, what):
    want_bits = O.bf16_bits(want_f32)
    diff = bf16_ulp_diff(got_bits, want_bits)
    worst = int(diff.max()) if diff.size else 0
    assert worst <= BF16_ULP_TOL, f"{what}: max bf16 ulp diff {worst}, {(diff > 0).sum()} of {diff.size} differ"
    return int((diff > 0).sum())


def run_dense(cuda, m, n, k, b_col_major, seed, want_acc=True):
    from catlass_b200 import capi
    torch = _torch()
    a, b, scale, pt = P.w8a8_dense(m, n, k, seed)
    b_flat = P.b_storage(b, b_col_major)
    layout_b = capi.COLUMN_MAJOR if b_col_major else capi.ROW_MAJOR
    d = torch.full((m, n), -1.0, dtype=torch.bfloat16, device=cuda)
    acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda) if want_acc else None
    capi.quant_matmul(_dev(a), _dev(b_flat), _dev(scale), _dev(pt), d, m, n, k, layout_b=layout_b, acc=acc)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    want, want_acc_np = O.quant_matmul(a, b_flat, scale, pt, m, n, k, O.ROW_MAJOR,
                                       O.COL_MAJOR if b_col_major else O.ROW_MAJOR, want_acc=True)
    if want_acc:
        got_acc = acc.cpu().numpy()
        assert np.array_equal(got_acc, want_acc_np), \
            f"int32 accumulators differ in {(got_acc != want_acc_np).sum()} of {got_acc.size} places"
    got_bits = d.view(torch.int16).cpu().numpy().view(np.uint16)
    return check_bf16(got_bits, want, f"dense {m}x{n}x{k} colB={b_col_major}")


DENSE_CASES = [
    # (m, n, k) : the reference runner's shape first, then ragged edges
    (256, 512, 1024),
    (128, 256, 128),
    (1, 256, 64),
    (129, 264, 1040),
    (300, 100, 48),
    (77, 130, 16),
    (512, 1024, 4096),
]


@pytest.mark.parametrize("m,n,k", DENSE_CASES)
def test_dense_column_major_b(cuda, m, n, k):
    run_dense(cuda, m, n, k, True, seed=m * 7 + n + k)


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (128, 256, 128), (129, 272, 1040), (300, 112, 48),
                                   (1, 16, 16), (512, 1024, 4096)])
def test_dense_row_major_b(cuda, m, n, k):
    run_dense(cuda, m, n, k, False, seed=m * 5 + n + k)


# few-token (decode) shapes: the transposed split-K kernel, 1/2/4/8-way clusters, token padding
SMALL_M_CASES = [
    (16, 14336, 4096, True), (16, 4096, 14336, True), (16, 1024, 4096, False), (1, 384, 2048, True),
    (33, 640, 2048, False), (64, 512, 8192, True), (128, 256, 16384, False), (17, 200, 1040, True),
    (5, 128, 640, True),
]


@pytest.mark.parametrize("m,n,k,col", SMALL_M_CASES)
def test_dense_few_tokens(cuda, m, n, k, col):
    run_dense(cuda, m, n, k, col, seed=m + n + k)


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (300, 264, 1040), (16, 384, 256), (129, 96, 48),
                                   (1000, 1024, 2048)])
def test_dense_zn_weights(cuda, m, n, k):
    """B in the reference's zN fractal format (16-row x 32-byte fractals, k padded to 16, n to 32)."""
    from catlass_b200 import capi
    torch = _torch()
    a, b, scale, pt = P.w8a8_dense(m, n, k, seed=m + n + k)
    d = torch.full((m, n), -1.0, dtype=torch.bfloat16, device=cuda)
    acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda)
    capi.quant_matmul(_dev(a), _dev(P.zn_storage(b)), _dev(scale), _dev(pt), d, m, n, k, layout_b=capi.ZN, acc=acc)
    assert capi.device_status()[0] == 0
    want, want_acc = O.quant_matmul(a, b, scale, pt, m, n, k, O.ROW_MAJOR, O.ROW_MAJOR, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    check_bf16(d.view(torch.int16).cpu().numpy().view(np.uint16), want, f"zN {m}x{n}x{k}")


def test_grouped_zn_weights(cuda):
    from catlass_b200 import capi
    torch = _torch()
    sizes = [200, 0, 129, 700, 31]
    n, k = 544, 528
    a, b, scale, pt, gl = P.w8a8_grouped(sizes, n, k, seed=8)
    m, g = a.shape[0], len(sizes)
    b_zn = np.stack([P.zn_storage(b[e]) for e in range(g)])
    d = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
    capi.grouped_quant_matmul(_dev(a), _dev(b_zn), _dev(gl), _dev(scale), _dev(pt), d, m, n, k, g, layout_b=capi.ZN)
    assert capi.device_status()[0] == 0
    want = O.grouped_quant_matmul(a, b, gl, scale, pt, m, n, k, O.ROW_MAJOR)
    check_bf16(d.view(torch.int16).cpu().numpy().view(np.uint16), want, "grouped zN")


def test_dense_extreme_values(cuda):
    """All operands at +-127/-128: the largest accumulator magnitudes the int8 path can produce."""
    from catlass_b200 import capi
    torch = _torch()
    m, n, k = 128, 256, 8192
    a = np.full((m, k), -128, np.int8)
    b = np.full((k, n), -128, np.int8)
    b[:, ::2] = 127
    scale = np.full(n, 1.0, np.float32)
    pt = np.full(m, 1.0, np.float32)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=cuda)
    acc = torch.empty((m, n), dtype=torch.int32, device=cuda)
    capi.quant_matmul(_dev(a), _dev(P.b_storage(b, True)), _dev(scale), _dev(pt), d, m, n, k, acc=acc)
    assert capi.device_status()[0] == 0
    want, want_acc = O.quant_matmul(a, P.b_storage(b, True), scale, pt, m, n, k, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    check_bf16(d.view(torch.int16).cpu().numpy().view(np.uint16), want, "extreme")


def run_grouped(cuda, sizes, n, k, b_col_major, seed, m_capacity=None, list_i32=False):
    from catlass_b200 import capi
    torch = _torch()
    a, b, scale, pt, gl = P.w8a8_grouped(sizes, n, k, seed, m_capacity)
    m = a.shape[0]
    g = len(sizes)
    b_flat = np.ascontiguousarray(b.transpose(0, 2, 1)) if b_col_major else b
    canary = 12345.0
    d = torch.full((m, n), canary, dtype=torch.bfloat16, device=cuda)
    acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda)
    gl_dev = _dev(gl.astype(np.int32)) if list_i32 else _dev(gl)
    capi.grouped_quant_matmul(_dev(a), _dev(b_flat), gl_dev, _dev(scale), _dev(pt), d, m, n, k, g,
                              layout_b=capi.COLUMN_MAJOR if b_col_major else capi.ROW_MAJOR, acc=acc,
                              group_list_type=capi.GROUP_LIST_INT32 if list_i32 else capi.GROUP_LIST_INT64)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    init = np.full((m, n), canary, np.float32)
    want, want_acc = O.grouped_quant_matmul(a, b_flat, gl, scale, pt, m, n, k,
                                            O.COL_MAJOR if b_col_major else O.ROW_MAJOR, want_acc=True,
                                            out_init=init)
    rows = int(gl[-1])
    got_acc = acc.cpu().numpy()
    assert np.array_equal(got_acc[:rows], want_acc[:rows])
    assert (got_acc[rows:] == -7).all(), "accumulator rows past the last group were written"
    got_bits = d.view(torch.int16).cpu().numpy().view(np.uint16)
    check_bf16(got_bits, want, f"grouped G={g} n={n} k={k}")
    # rows past the last group keep the caller's bytes
    assert np.array_equal(got_bits[rows:], O.bf16_bits(init)[rows:])


def test_grouped_reference_runner_shape(cuda):
    """tests/test_example.py runs examples 07/10 with `128 512 1024 2048` (groups m n k) and the group
    list of golden::GenerateGroupList; the same list law (sorted uniform cut points, repeats allowed)."""
    rng = np.random.default_rng(0)
    cuts = np.sort(rng.integers(0, 513, size=128))
    sizes = np.diff(np.concatenate([[0], cuts]))
    run_grouped(cuda, sizes, 1024, 2048, False, seed=1, m_capacity=512)


@pytest.mark.parametrize("b_col_major", [False, True])
def test_grouped_ragged(cuda, b_col_major):
    sizes = [0, 1, 127, 128, 129, 0, 0, 300, 5, 256, 0]
    run_grouped(cuda, sizes, 384, 272, b_col_major, seed=3, m_capacity=sum(sizes) + 40)


def test_grouped_int32_list_and_narrow_n(cuda):
    run_grouped(cuda, [64, 0, 200, 31], 128, 512, False, seed=4, list_i32=True)
    run_grouped(cuda, [5, 3], 48, 64, True, seed=5)


def test_grouped_all_empty(cuda):
    run_grouped(cuda, [0, 0, 0], 256, 128, False, seed=6, m_capacity=64)


def test_grouped_zipf_moe_slice(cuda):
    """A scaled-down cut of the MoE configuration: 64 experts, Zipf(1.1) loads, K=7168."""
    sizes = P.zipf_group_sizes(4096, 64, seed=11)
    run_grouped(cuda, sizes, 512, 7168, False, seed=12)


def test_grouped_full_moe_config_sampled_rows(cuda):
    """The benchmark configuration at full size (64 experts, K=7168, N=4096, 131072 rows, Zipf loads) on the
    GPU; the oracle recomputes sampled rows of every expert: its first and last row, the rows on either side
    of its first 128-row tile boundary, and a random one."""
    import torch
    from catlass_b200 import capi
    g, n, k, rows = 64, 4096, 7168, 131072
    sizes = P.zipf_group_sizes(rows, g, seed=20240)
    gl = np.cumsum(sizes).astype(np.int64)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    a = torch.randint(-127, 128, (rows, k), dtype=torch.int8, device=cuda, generator=gen)
    b = torch.randint(-127, 128, (g, k, n), dtype=torch.int8, device=cuda, generator=gen)
    scale = torch.empty((g, n), device=cuda).uniform_(1e-3, 1e-2, generator=gen)
    pt = torch.empty(rows, device=cuda).uniform_(1e-3, 1e-2, generator=gen)
    d = torch.zeros((rows, n), dtype=torch.bfloat16, device=cuda)
    capi.grouped_quant_matmul(a, b, _dev(gl), scale, pt, d, rows, n, k, g, layout_b=capi.ROW_MAJOR)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    rng = np.random.default_rng(3)
    starts = np.concatenate([[0], gl[:-1]])
    bad = 0
    checked = 0
    for e in range(g):
        if sizes[e] == 0:
            continue
        local = {0, int(sizes[e]) - 1, int(rng.integers(0, sizes[e]))}
        if sizes[e] > 128:
            local |= {127, 128}
        idx = np.array(sorted(local)) + starts[e]
        a_rows = a[torch.from_numpy(idx).cuda()].cpu().numpy()
        want = O.quant_matmul(a_rows, b[e].cpu().numpy(), scale[e].cpu().numpy(), pt[torch.from_numpy(idx).cuda()].cpu().numpy(),
                              len(idx), n, k, O.ROW_MAJOR, O.ROW_MAJOR)
        got = d[torch.from_numpy(idx).cuda()].view(torch.int16).cpu().numpy().view(np.uint16)
        bad += int((got != O.bf16_bits(want)).sum())
        checked += got.size
    assert bad == 0, f"{bad} of {checked} sampled outputs differ"
    # every routed row was written: a row of exact zeros would need an all-zero accumulator row
    assert int((d.view(torch.int16) != 0).any(dim=1).sum()) == rows


@pytest.mark.parametrize("chunks", [0, 1, 3])
def test_grouped_host_buffers_entry(cuda, chunks):
    """Host-resident activations and output through the chunked copy/compute pipeline: same bits as the oracle,
    rows past the last group untouched in the caller's host buffer."""
    import torch
    from catlass_b200 import capi
    sizes = [0, 300, 1, 127, 700, 0, 129, 64]
    n, k = 512, 272
    a, b, scale, pt, gl = P.w8a8_grouped(sizes, n, k, seed=21, m_capacity=sum(sizes) + 33)
    m, g = a.shape[0], len(sizes)
    a_h = torch.from_numpy(a).pin_memory()
    pt_h = torch.from_numpy(pt).pin_memory()
    gl_h = torch.from_numpy(gl).pin_memory()
    d_h = torch.full((m, n), 777.0, dtype=torch.bfloat16).pin_memory()
    ws = torch.empty(capi.grouped_quant_matmul_host_workspace_size(m, n, k, g, chunks), dtype=torch.uint8, device=cuda)
    for _ in range(2):  # twice: the pipeline's events and pinned list buffer are reused
        capi.grouped_quant_matmul_host(a_h, gl_h, pt_h, d_h, _dev(b), _dev(scale), m, n, k, g, ws, chunks=chunks)
        torch.cuda.current_stream().synchronize()
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    init = np.full((m, n), 777.0, np.float32)
    want = O.grouped_quant_matmul(a, b, gl, scale, pt, m, n, k, O.ROW_MAJOR, out_init=init)
    got = d_h.view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, O.bf16_bits(want))


def test_k_zero_writes_zeros(cuda):
    from catlass_b200 import capi
    torch = _torch()
    m, n = 130, 264
    d = torch.full((m, n), 3.0, dtype=torch.bfloat16, device=cuda)
    dummy = torch.zeros(max(m, n) * 16, dtype=torch.int8, device=cuda)
    scale = torch.ones(n, device=cuda)
    pt = torch.ones(m, device=cuda)
    capi.quant_matmul(dummy, dummy, scale, pt, d, m, n, 0)
    assert capi.device_status()[0] == 0
    assert (d == 0).all()


def test_invalid_arguments_are_rejected(cuda):
    from catlass_b200 import capi
    torch = _torch()
    m, n, k = 128, 256, 128
    a = torch.zeros(m * k + 64, dtype=torch.int8, device=cuda)
    b = torch.zeros(k * n, dtype=torch.int8, device=cuda)
    s = torch.ones(n, device=cuda)
    p = torch.ones(m, device=cuda)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(capi.CallError) as e:
        capi.quant_matmul(a, b, s, p, d, m, n, 100)  # k not a multiple of 16
    assert e.value.status == capi.INVALID
    with pytest.raises(capi.CallError):
        capi.quant_matmul(a[1:], b, s, p, d, m, n, k)  # misaligned A
    with pytest.raises(capi.CallError):
        capi.quant_matmul(a, b, s, p, d, m, n, k, layout_a=7)
    with pytest.raises(capi.CallError):
        capi.quant_matmul(a, b, s, p, d, 120, n, k, layout_a=capi.COLUMN_MAJOR)  # column-major A: m % 16
    with pytest.raises(capi.CallError):
        capi.quant_matmul(a, b, s, p, d, m, n, k, d_type=5)
    with pytest.raises(capi.CallError):
        capi.quant_matmul(a, b, s, p, d, m, n, k, layout_b=7)
    with pytest.raises(capi.CallError):
        capi.quant_matmul(None, b, s, p, d, m, n, k)


def test_bounded_wait_gives_up_and_reports(cuda):
    """The give-up path of the kernels' waits: a wait that nothing will ever satisfy ends after its limit,
    the status word carries the code, reading it clears it, and the device keeps working."""
    import time
    import torch
    from catlass_b200 import capi
    lib = capi.load()
    assert capi.device_status() == (0, 0)
    t0 = time.perf_counter()
    assert lib.cb200_selftest_wait_timeout(2000, ctypes_stream()) == 0   # 2 ms limit
    st, code = capi.device_status()
    assert time.perf_counter() - t0 < 5.0
    assert (st, code) == (capi.DEVICE_TIMEOUT, 0x1F0)
    assert capi.device_status() == (0, 0)            # cleared by the read
    run_dense(cuda, 256, 512, 1024, True, seed=1)    # the context is still healthy


def ctypes_stream():
    import ctypes
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
