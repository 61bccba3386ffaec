"""GPU parity of the W8A8 operator variants against the CPU oracle, through the C ABI: column-major A (the four
layout pairs of the reference's example 103), half / bf16 scale vectors and half output (examples 12 / 07 / 10
instantiate those), the per-tensor / per-channel grouped dequant of example 48, the output staging of tiles with
an odd number of column chunks, and stream ordering against a kernel that writes the weights right before."""
import numpy as np
import pytest

import oracle_lib as O
import problems as P
from test_w8a8_gpu import _dev, _torch, bf16_ulp_diff

pytestmark = pytest.mark.gpu


def check_out(got_bits, want_f32, f16, what):
    want_bits = O.out_bits(want_f32, f16)
    if f16:
        bad = int((got_bits != want_bits).sum())
        assert bad == 0, f"{what}: {bad} of {got_bits.size} fp16 outputs differ"
    else:
        diff = bf16_ulp_diff(got_bits, want_bits)
        assert int(diff.max(initial=0)) == 0, f"{what}: {(diff > 0).sum()} of {diff.size} bf16 outputs differ"


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (128, 256, 128), (16, 384, 256), (304, 272, 1040),
                                   (48, 96, 64), (1024, 1024, 2048)])
@pytest.mark.parametrize("b_layout", ["row", "col", "zn"])
def test_dense_column_major_a(cuda, m, n, k, b_layout):
    from catlass_b200 import capi
    torch = _torch()
    if b_layout == "row" and n % 16:
        pytest.skip("row-major B needs n % 16 == 0")
    a, b, scale, pt = P.w8a8_dense(m, n, k, seed=m + 3 * n + k)
    a_cm = np.ascontiguousarray(a.T)  # [k][m]
    b_flat = {"row": P.b_storage(b, False), "col": P.b_storage(b, True), "zn": P.zn_storage(b)}[b_layout]
    lb = {"row": capi.ROW_MAJOR, "col": capi.COLUMN_MAJOR, "zn": capi.ZN}[b_layout]
    d = torch.full((m, n), -1.0, dtype=torch.bfloat16, device=cuda)
    acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda)
    capi.quant_matmul(_dev(a_cm), _dev(b_flat), _dev(scale), _dev(pt), d, m, n, k, layout_a=capi.COLUMN_MAJOR,
                      layout_b=lb, acc=acc)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    want, want_acc = O.quant_matmul(a_cm, P.b_storage(b, False), scale, pt, m, n, k, O.COL_MAJOR, O.ROW_MAJOR,
                                    want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    check_out(d.view(torch.int16).cpu().numpy().view(np.uint16), want, False, f"A col-major, B {b_layout}")


def _as_type(x, kind):
    """(device tensor in the scale element type, the fp32 values those elements hold)."""
    torch = _torch()
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda()
    if kind == "f32":
        return t, x.astype(np.float32)
    tt = t.to(torch.bfloat16 if kind == "bf16" else torch.float16)
    return tt, tt.float().cpu().numpy()


SCALE_TYPES = {"f32": 0, "bf16": 1, "f16": 2}


@pytest.mark.parametrize("scale_kind,f16_out", [("f16", True), ("f32", True), ("bf16", False), ("f16", False)])
@pytest.mark.parametrize("m,n,k,col", [(256, 512, 1024, True), (16, 640, 512, True), (300, 120, 272, False),
                                       (130, 264, 1040, True)])
def test_dense_scale_and_output_types(cuda, m, n, k, col, scale_kind, f16_out):
    """Example 12 runs half scales and half D, example 10 bf16 scales and bf16 D: the golden converts the scales
    to float and multiplies in fp32 (examples/common/golden/matmul.hpp:320-321), D is rounded once."""
    from catlass_b200 import capi
    torch = _torch()
    a, b, scale, pt = P.w8a8_dense(m, n, k, seed=m + n + k + 1)
    if not col and n % 16:
        pytest.skip("row-major B needs n % 16 == 0")
    scale_t, scale_v = _as_type(scale * (30.0 if f16_out else 1.0), scale_kind)  # keep halves out of the subnormals
    pt_t, pt_v = _as_type(pt * (30.0 if f16_out else 1.0), scale_kind)
    b_flat = P.b_storage(b, col)
    d = torch.zeros((m, n), dtype=torch.float16 if f16_out else torch.bfloat16, device=cuda)
    capi.quant_matmul(_dev(a), _dev(b_flat), scale_t, pt_t, d, m, n, k,
                      layout_b=capi.COLUMN_MAJOR if col else capi.ROW_MAJOR, scale_type=SCALE_TYPES[scale_kind],
                      d_type=capi.DTYPE_F16 if f16_out else capi.DTYPE_BF16)
    assert capi.device_status()[0] == 0
    want = O.quant_matmul(a, b_flat, scale_v, pt_v, m, n, k, O.ROW_MAJOR, O.COL_MAJOR if col else O.ROW_MAJOR)
    check_out(d.view(torch.int16).cpu().numpy().view(np.uint16), want, f16_out, f"{scale_kind} scales")


@pytest.mark.parametrize("scale_kind,f16_out", [("f32", True), ("bf16", False)])
def test_grouped_scale_and_output_types(cuda, scale_kind, f16_out):
    """Example 07 (float scales, half D) and example 10 (bf16 scales, bf16 D)."""
    from catlass_b200 import capi
    torch = _torch()
    sizes = [130, 0, 64, 257, 1, 300]
    n, k = 512, 1024
    a, b, scale, pt, gl = P.w8a8_grouped(sizes, n, k, seed=77)
    m, g = a.shape[0], len(sizes)
    scale_t, scale_v = _as_type(scale * 20.0, scale_kind)
    pt_t, pt_v = _as_type(pt * 20.0, scale_kind)
    d = torch.zeros((m, n), dtype=torch.float16 if f16_out else torch.bfloat16, device=cuda)
    capi.grouped_quant_matmul(_dev(a), _dev(b), _dev(gl), scale_t, pt_t, d, m, n, k, g,
                              scale_type=SCALE_TYPES[scale_kind],
                              d_type=capi.DTYPE_F16 if f16_out else capi.DTYPE_BF16)
    assert capi.device_status()[0] == 0
    want = O.grouped_quant_matmul(a, b, gl, scale_v, pt_v, m, n, k, O.ROW_MAJOR)
    check_out(d.view(torch.int16).cpu().numpy().view(np.uint16), want, f16_out, f"grouped {scale_kind}")


@pytest.mark.parametrize("quant_mode", [0, 1])
@pytest.mark.parametrize("u64_scales,f16_out,col", [(True, True, False), (False, False, True), (False, True, False)])
def test_grouped_per_tensor_per_channel_dequant(cuda, quant_mode, u64_scales, f16_out, col):
    """Example 48: values in [-16, 16], scales in [0, 1), evenly cut groups, half output; plus ragged groups."""
    from catlass_b200 import capi
    torch = _torch()
    for sizes, n, k in (([64] * 8, 256, 512), ([0, 200, 1, 127, 300, 0, 129], 384, 272)):
        a, b, _, _, gl = P.w8a8_grouped(sizes, n, k, seed=48 + quant_mode, m_capacity=sum(sizes) + 9, lo=-16, hi=16)
        m, g = a.shape[0], len(sizes)
        rng = np.random.default_rng(quant_mode)
        pcs = rng.uniform(0, 1, n).astype(np.float32)
        scalar = float(np.float32(rng.uniform(0, 1)))
        b_flat = np.ascontiguousarray(b.transpose(0, 2, 1)) if col else b
        if u64_scales:  # the reference's hand-over: fp32 bits in the low half of a 64-bit word
            pcs_dev = _dev(pcs.view(np.uint32).astype(np.uint64).view(np.int64))
        else:
            pcs_dev = _dev(pcs)
        canary = 3.0
        d = torch.full((m, n), canary, dtype=torch.float16 if f16_out else torch.bfloat16, device=cuda)
        acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda)
        capi.grouped_fixpipe_dequant(_dev(a), _dev(b_flat), _dev(gl), d, m, n, k, g, quant_mode,
                                     scale_per_tensor=scalar, per_channel_scale=pcs_dev if quant_mode == 1 else None,
                                     per_channel_scale_type=capi.DTYPE_F32_IN_U64 if u64_scales else capi.DTYPE_F32,
                                     layout_b=capi.COLUMN_MAJOR if col else capi.ROW_MAJOR,
                                     d_type=capi.DTYPE_F16 if f16_out else capi.DTYPE_BF16, acc=acc)
        assert capi.device_status()[0] == 0
        init = np.full((m, n), canary, np.float32)
        want, want_acc = O.grouped_fixpipe_dequant(a, b_flat, gl, quant_mode, scalar, pcs, m, n, k,
                                                   O.COL_MAJOR if col else O.ROW_MAJOR, want_acc=True, out_init=init)
        rows = int(gl[-1])
        assert np.array_equal(acc.cpu().numpy()[:rows], want_acc[:rows])
        check_out(d.view(torch.int16).cpu().numpy().view(np.uint16), want, f16_out, f"fixpipe mode {quant_mode}")


@pytest.mark.parametrize("n", [352, 288, 160, 4096 + 32])
def test_grouped_odd_number_of_column_chunks(cuda, n):
    """Tiles whose last column tile holds an odd number of 32-column chunks, many tiles per CTA pair and K short
    enough that a pair reaches its next tile while the previous tile's output stores are still in flight."""
    from catlass_b200 import capi
    torch = _torch()
    scale_rows = 1 if n < 1024 else 8   # keeps the oracle's work near 1.5 G multiply-adds
    sizes = [256 * 40 // scale_rows, (256 * 37 + 64) // scale_rows, 0, 256 * 50 // scale_rows]
    k = 128
    a, b, scale, pt, gl = P.w8a8_grouped(sizes, n, k, seed=n)
    m, g = a.shape[0], len(sizes)
    a_d, b_d, gl_d, s_d, p_d = _dev(a), _dev(b), _dev(gl), _dev(scale), _dev(pt)
    want = O.out_bits(O.grouped_quant_matmul(a, b, gl, scale, pt, m, n, k, O.ROW_MAJOR))
    for block_num in (0, 8):  # 8 CTAs = 4 pairs: hundreds of tiles per pair
        d = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
        capi.grouped_quant_matmul(a_d, b_d, gl_d, s_d, p_d, d, m, n, k, g, block_num=block_num)
        assert capi.device_status()[0] == 0
        got = d.view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got, want), f"n={n} block_num={block_num}: {(got != want).sum()} outputs differ"


@pytest.mark.parametrize("static_weights", [False])
def test_weights_written_on_the_stream_right_before_the_call(cuda, static_weights):
    """Plain stream order: the few-token kernel (launched with programmatic dependent launch) must see weights
    and channel scales that a kernel earlier on the same stream produced."""
    from catlass_b200 import capi
    torch = _torch()
    m, n, k = 16, 4096, 4096
    a, b, scale, pt = P.w8a8_dense(m, n, k, seed=5)
    b_new = P.b_storage(b, True)
    want = O.out_bits(O.quant_matmul(a, b_new, scale, pt, m, n, k))
    a_d, pt_d = _dev(a), _dev(pt)
    src_b, src_s = _dev(b_new), _dev(scale)
    big = torch.zeros(64 << 20, dtype=torch.int8, device=cuda)
    for _ in range(5):
        w = torch.zeros((n, k), dtype=torch.int8, device=cuda)
        s = torch.zeros(n, device=cuda)
        d = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
        torch.cuda.synchronize()
        big.add_(1)          # keeps the GPU busy so that the copies below are still running at the launch
        w.copy_(src_b)
        s.copy_(src_s)
        capi.quant_matmul(a_d, w, s, pt_d, d, m, n, k, static_weights=static_weights)
        assert capi.device_status()[0] == 0
        got = d.view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got, want), f"{(got != want).sum()} outputs differ"


def test_static_weights_flag_gives_the_same_result(cuda):
    from catlass_b200 import capi
    torch = _torch()
    for m, n, k in ((16, 14336, 4096), (33, 640, 2048)):
        a, b, scale, pt = P.w8a8_dense(m, n, k, seed=6)
        b_flat = P.b_storage(b, True)
        want = O.out_bits(O.quant_matmul(a, b_flat, scale, pt, m, n, k))
        d = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
        args = (_dev(a), _dev(b_flat), _dev(scale), _dev(pt), d, m, n, k)
        for _ in range(3):
            capi.quant_matmul(*args, static_weights=True)
        assert capi.device_status()[0] == 0
        assert np.array_equal(d.view(torch.int16).cpu().numpy().view(np.uint16), want)


@pytest.mark.parametrize("layout", ["row", "col", "zn"])
def test_grouped_partial_row_tiles_of_every_width(cuda, layout):
    """Groups whose last row tile holds 1 ... 255 rows, beside full tiles and alone, with column tiles cut by n:
    rows past a group's end belong to the next group and must keep its results."""
    from catlass_b200 import capi
    torch = _torch()
    rems = [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 96, 127, 128, 129, 160, 191, 192, 193, 224, 255]
    sizes = []
    for i, r in enumerate(rems):
        sizes.append(r + 256 * (i % 3))   # alone, after one full tile, after two
    sizes.insert(5, 0)
    n, k = (392 if layout != "row" else 400), 272
    a, b, scale, pt, gl = P.w8a8_grouped(sizes, n, k, seed=7, m_capacity=sum(sizes) + 70)
    m, g = a.shape[0], len(sizes)
    if layout == "row":
        b_flat, lb, olb = b, capi.ROW_MAJOR, O.ROW_MAJOR
    elif layout == "col":
        b_flat, lb, olb = np.ascontiguousarray(b.transpose(0, 2, 1)), capi.COLUMN_MAJOR, O.COL_MAJOR
    else:
        b_flat, lb, olb = np.stack([P.zn_storage(b[e]) for e in range(g)]), capi.ZN, O.ROW_MAJOR
    canary = 5.0
    d = torch.full((m, n), canary, dtype=torch.bfloat16, device=cuda)
    acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda)
    capi.grouped_quant_matmul(_dev(a), _dev(b_flat), _dev(gl), _dev(scale), _dev(pt), d, m, n, k, g, layout_b=lb,
                              acc=acc)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    init = np.full((m, n), canary, np.float32)
    want, want_acc = O.grouped_quant_matmul(a, b if layout == "zn" else b_flat, gl, scale, pt, m, n, k, olb,
                                            want_acc=True, out_init=init)
    rows = int(gl[-1])
    got_acc = acc.cpu().numpy()
    assert np.array_equal(got_acc[:rows], want_acc[:rows])
    assert (got_acc[rows:] == -7).all()
    got = d.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, O.out_bits(want)), f"{(got != O.out_bits(want)).sum()} outputs differ"


@pytest.mark.parametrize("m", [44, 129, 192, 300, 448, 512 + 33])
def test_dense_partial_last_row_tile(cuda, m):
    """Dense problems are one group: a partial last row tile, alone and after full tiles."""
    from catlass_b200 import capi
    torch = _torch()
    n, k = 520, 1040
    a, b, scale, pt = P.w8a8_dense(m, n, k, seed=m)
    b_flat = P.b_storage(b, True)
    d = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
    acc = torch.zeros((m, n), dtype=torch.int32, device=cuda)
    capi.quant_matmul(_dev(a), _dev(b_flat), _dev(scale), _dev(pt), d, m, n, k, acc=acc)
    assert capi.device_status()[0] == 0
    want, want_acc = O.quant_matmul(a, b_flat, scale, pt, m, n, k, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    assert np.array_equal(d.view(torch.int16).cpu().numpy().view(np.uint16), O.out_bits(want))


@pytest.mark.parametrize("cuts,m,n,k", [
    ((64, 128, 192, 256), 128, 128, 256),               # the reference's optest shape (example 11)
    ((5, 5, 133, 300, 300, 1000), 272, 392 + 8, 1000),  # ragged cuts, empty groups, rows and columns cut by tiles
    ((0, 0), 64, 64, 128),                              # nothing but empty groups
    ((700, 2048), 512, 1024, 2048),
])
@pytest.mark.parametrize("f16_out", [False, True])
def test_grouped_slice_k(cuda, cuts, m, n, k, f16_out):
    """Groups along K (example 11): A column-major, B row-major, one m x n output block per group."""
    from catlass_b200 import capi
    torch = _torch()
    rng = np.random.default_rng(k + m)
    g = len(cuts)
    a = rng.integers(-127, 128, (k, m), dtype=np.int8)     # [k][m]: A column-major
    b = rng.integers(-127, 128, (k, n), dtype=np.int8)
    scale = rng.uniform(1e-3, 1e-2, (g, n)).astype(np.float32)
    pt = rng.uniform(1e-3, 1e-2, (g, m)).astype(np.float32)
    gl = np.array(cuts, np.int64)
    d = torch.full((g, m, n), -1.0, dtype=torch.float16 if f16_out else torch.bfloat16, device=cuda)
    acc = torch.full((g, m, n), -7, dtype=torch.int32, device=cuda)
    ws = torch.empty(capi.grouped_quant_matmul_slice_k_workspace_size(m, n, k, g), dtype=torch.uint8, device=cuda)
    capi.grouped_quant_matmul_slice_k(_dev(a), _dev(b), _dev(gl), _dev(scale), _dev(pt), d, m, n, k, g, ws, acc=acc,
                                      d_type=capi.DTYPE_F16 if f16_out else capi.DTYPE_BF16)
    st, code = capi.device_status()
    assert st == 0, f"device status {st} code {code:#x}"
    want, want_acc = O.grouped_quant_matmul_slice_k(a, b, gl, scale, pt, m, n, k, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    check_out(d.view(torch.int16).cpu().numpy().view(np.uint16), want, f16_out, "slice-K")
