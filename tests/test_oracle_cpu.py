"""The CPU oracle against the reference: committed golden vectors (produced by the reference's own C++
golden and Python generators, see tests/golden/make_golden.py) and, where oracle/_ref was built, the
reference golden itself on fresh random inputs."""
import ctypes
import os

import numpy as np
import pytest

import oracle_lib as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bits(x):
    return np.ascontiguousarray(x, np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def w8a8_golden():
    return np.load(os.path.join(GOLDEN, "w8a8_ref_golden.npz"))


def test_dense_matches_reference_golden_vectors(w8a8_golden):
    g = w8a8_golden
    m, n, k = (int(x) for x in g["dense_shape"])
    for la in (0, 1):
        for lb in (0, 1):
            out = O.quant_matmul(g["dense_a"], g["dense_b"], g["dense_scale"], g["dense_pt"], m, n, k, la, lb)
            assert np.array_equal(bits(out), bits(g[f"dense_out_{la}{lb}"])), (la, lb)


def test_grouped_matches_reference_golden_vectors(w8a8_golden):
    g = w8a8_golden
    m, n, k, groups = (int(x) for x in g["grp_shape"])
    assert len(g["grp_list"]) == groups
    for lb in (0, 1):
        out = O.grouped_quant_matmul(g["grp_a"], g["grp_b"], g["grp_list"], g["grp_scale"], g["grp_pt"],
                                     m, n, k, lb)
        assert np.array_equal(bits(out), bits(g[f"grp_out_{lb}"])), lb


def test_fixpipe_dequant_matches_reference_golden_vectors(w8a8_golden):
    g = w8a8_golden
    m, n, k, groups = (int(x) for x in g["grp_shape"])
    for mode in (0, 1):
        for lb in (0, 1):
            out = O.grouped_fixpipe_dequant(g["grp_a"], g["grp_b"], g["grp_list"], mode, float(g["fix_scalar"]),
                                            g["fix_pcs"], m, n, k, lb)
            assert np.array_equal(bits(out), bits(g[f"fix_out_{mode}{lb}"])), (mode, lb)


def test_slice_k_matches_reference_golden_vectors(w8a8_golden):
    g = w8a8_golden
    m, n, k, groups = (int(x) for x in g["slk_shape"])
    out = O.grouped_quant_matmul_slice_k(g["slk_a"], g["slk_b"], g["slk_list"], g["slk_scale"], g["slk_pt"], m, n, k)
    assert out.shape == (groups, m, n)
    assert np.array_equal(bits(out), bits(g["slk_out"]))


@pytest.mark.skipif(O.ref() is None, reason="reference golden (oracle/_ref) not built")
def test_siblings_against_live_reference_golden():
    rng = np.random.default_rng(48)
    m, n, k, g = 70, 36, 64, 6
    gl = O.ref_generate_group_list(m, g)
    a = rng.integers(-128, 128, m * k, dtype=np.int8)
    b = rng.integers(-128, 128, g * k * n, dtype=np.int8)
    pcs = rng.uniform(0, 1, n).astype(np.float32)
    for mode in (0, 1):
        for lb in (0, 1):
            assert np.array_equal(bits(O.grouped_fixpipe_dequant(a, b, gl, mode, 0.8125, pcs, m, n, k, lb)),
                                  bits(O.ref_grouped_fixpipe_dequant(a, b, gl, mode, 0.8125, pcs, m, n, k, lb)))
    kk = 150
    glk = O.ref_generate_group_list(kk, g)
    a2 = rng.integers(-128, 128, 24 * kk, dtype=np.int8)
    b2 = rng.integers(-128, 128, kk * n, dtype=np.int8)
    s2 = rng.uniform(1e-3, 1e-2, g * n).astype(np.float32)
    p2 = rng.uniform(1e-3, 1e-2, g * 24).astype(np.float32)
    assert np.array_equal(bits(O.grouped_quant_matmul_slice_k(a2, b2, glk, s2, p2, 24, n, kk)),
                          bits(O.ref_grouped_quant_matmul_slice_k(a2, b2, glk, s2, p2, 24, n, kk)))


def test_reference_group_list_fixture_is_a_prefix_sum_list(w8a8_golden):
    gl = w8a8_golden["group_list_512_128"]
    assert len(gl) == 128 and (np.diff(gl) >= 0).all() and 0 <= gl[0] and gl[-1] <= 512
    assert (np.diff(gl) == 0).any(), "the runner's list contains empty groups"


@pytest.mark.skipif(O.ref() is None, reason="reference golden (oracle/_ref) not built")
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (7, 33, 65), (64, 48, 256)])
def test_dense_against_live_reference_golden(m, n, k):
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(-128, 128, m * k, dtype=np.int8)
    b = rng.integers(-128, 128, k * n, dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    p = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    for la in (0, 1):
        for lb in (0, 1):
            assert np.array_equal(bits(O.quant_matmul(a, b, s, p, m, n, k, la, lb)),
                                  bits(O.ref_quant_matmul(a, b, s, p, m, n, k, la, lb)))


@pytest.mark.skipif(O.ref() is None, reason="reference golden (oracle/_ref) not built")
def test_grouped_against_live_reference_golden():
    rng = np.random.default_rng(5)
    m, n, k, g = 96, 40, 48, 17
    gl = O.ref_generate_group_list(m, g)
    a = rng.integers(-128, 128, m * k, dtype=np.int8)
    b = rng.integers(-128, 128, g * k * n, dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, g * n).astype(np.float32)
    p = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    for lb in (0, 1):
        assert np.array_equal(bits(O.grouped_quant_matmul(a, b, gl, s, p, m, n, k, lb)),
                              bits(O.ref_grouped_quant_matmul(a, b, gl, s, p, m, n, k, lb)))


def test_accumulators_are_the_integer_products():
    rng = np.random.default_rng(9)
    m, n, k = 9, 11, 40
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    _, acc = O.quant_matmul(a, b, np.ones(n), np.ones(m), m, n, k, 0, 0, want_acc=True)
    assert np.array_equal(acc, a.astype(np.int64) @ b.astype(np.int64))


def test_bf16_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.4e38, 0.0, -0.0], np.float32)
    # 1 + 2^-8 is a tie between 1.0 (even) and 1 + 2^-7; 1 + 3*2^-8 ties up to 1 + 2^-6
    want = np.array([0x3F80, 0x3F80, 0x3F82, 0xBF80, 0x7F80, 0x0000, 0x8000], np.uint16)
    assert np.array_equal(O.bf16_bits(x), want)
    import torch
    y = np.random.default_rng(1).standard_normal(4096).astype(np.float32) * 1e-3
    t = torch.from_numpy(y).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.bf16_bits(y), t)


def test_f16_round_to_nearest_even():
    rng = np.random.default_rng(16)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 1.5 * 2.0 ** -25,
                  2.0 ** -14, 2.0 ** -14 - 2.0 ** -25, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11], np.float32)])
    x = x.astype(np.float32)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(O.f16_bits(x), want)


# ------------------------------------------------------------------ MX

@pytest.fixture(scope="module")
def mx_golden():
    return np.load(os.path.join(GOLDEN, "mx_ref_golden.npz"))


@pytest.mark.parametrize("name,fmt", [("fp8", O.MX_E4M3), ("fp4", O.MX_E2M1)])
def test_mx_quantize_matches_reference_generators(mx_golden, name, fmt):
    g = mx_golden
    a = g[f"{name}_a"]
    q, sf, deq = O.mx_quantize(a, fmt, want_deq=True)
    blocks = sf.shape[1]
    assert np.array_equal(q, g[f"{name}_a_code"])
    assert np.array_equal(sf, g[f"{name}_a_sf"][:, :blocks])
    assert np.array_equal(bits(deq), bits(g[f"{name}_a_deq"]))
    # B is quantised along K too: blocks run down the columns of the k x n matrix
    bt = np.ascontiguousarray(g[f"{name}_b"].T)
    qb, sfb, deqb = O.mx_quantize(bt, fmt, want_deq=True)
    assert np.array_equal(qb.T, g[f"{name}_b_code"])
    assert np.array_equal(sfb.T, g[f"{name}_b_sf"][:sfb.shape[1], :])
    assert np.array_equal(bits(deqb.T), bits(g[f"{name}_b_deq"]))


@pytest.mark.parametrize("name,fmt", [("fp8", O.MX_E4M3), ("fp4", O.MX_E2M1)])
def test_mx_matmul_matches_reference_golden(mx_golden, name, fmt):
    g = mx_golden
    a, b = g[f"{name}_a"], g[f"{name}_b"]
    m, k = a.shape
    n = b.shape[1]
    qa, sfa = O.mx_quantize(a, fmt)
    qb, sfb = O.mx_quantize(np.ascontiguousarray(b.T), fmt)
    out = O.mx_matmul(qa, sfa, qb, sfb, m, n, k, fmt)
    gold = g[f"{name}_golden"]
    # the reference accumulates in fp32 (torch matmul); the oracle in double: equal to fp32 rounding noise
    err = np.abs(out - gold) / np.maximum(1.0, np.abs(gold))
    assert err.max() < 1e-5


def test_mx_fp4_nibble_packing_matches_reference(mx_golden):
    codes = mx_golden["fp4_a_code"]
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    assert np.array_equal(packed, mx_golden["fp4_packed_a"])


def test_mx_element_decoders():
    lib = O.lib()
    assert lib.orc_e4m3_to_float(0x7E) == 448.0 and lib.orc_e4m3_to_float(0x01) == 2.0 ** -9
    assert lib.orc_e4m3_to_float(0xB8) == -1.0
    assert [lib.orc_e2m1_to_float(i) for i in range(8)] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert lib.orc_e2m1_to_float(0xF) == -6.0
    assert lib.orc_e8m0_to_float(127) == 1.0 and lib.orc_e8m0_to_float(130) == 8.0


# ------------------------------------------------------------------ W4A8

def test_swiglu_mx_quant_matches_reference_golden():
    """Pins the epilogue restatement to the reference's own swiglu() and quant()
    (experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant/compare.py:31-121)."""
    g = np.load(os.path.join(GOLDEN, "swiglu_quant_ref_golden.npz"))
    # the quantiser is integer arithmetic on bf16 fields plus exact products: bit for bit, fed the reference's S
    q, scale = O.mx_quant_bf16_e4m3(g["s_bits"])
    nan_blocks = np.repeat(g["scale"] == 0xFF, 32, axis=1)
    assert np.array_equal(scale, g["scale"])
    assert np.array_equal(q[~nan_blocks], g["q"][~nan_blocks])
    assert np.all((q[nan_blocks] & 0x7F) == 0x7F) and nan_blocks.any()  # a block holding Inf: all NaN codes
    # the swish goes through exp(): another libm may differ in the last place, which the rounding to bf16 hides
    # almost always; demand equality up to one bf16 step on a handful of values at most
    s = O.swiglu_bf16(g["c"])
    diff = np.abs(s.astype(np.int32) - g["s_bits"].astype(np.int32))
    finite = (g["s_bits"] & 0x7F80) != 0x7F80
    assert diff[finite].max() <= 1 and (diff[finite] != 0).mean() < 2e-3
    assert np.array_equal(s[~finite] & 0x7F80, g["s_bits"][~finite] & 0x7F80)


def test_e4m3_rne_encoder_against_decoder():
    """Every E4M3 code decodes and re-encodes to itself; midpoints go to the even code; 448 saturates."""
    for code in range(256):
        if (code & 0x7F) == 0x7F:
            continue
        v = O.lib().orc_e4m3_to_float(code)
        assert O.lib().orc_e4m3_rne_sat(ctypes.c_float(v)) == (code if v != 0 or code == 0 else code), code
    lib = O.lib()
    for code in range(0, 0x7E):
        lo, hi = lib.orc_e4m3_to_float(code), lib.orc_e4m3_to_float(code + 1)
        mid = np.float32((np.float64(lo) + np.float64(hi)) / 2)
        want = code if code % 2 == 0 else code + 1
        assert lib.orc_e4m3_rne_sat(ctypes.c_float(mid)) == want, (code, mid)
    assert lib.orc_e4m3_rne_sat(ctypes.c_float(1e9)) == 0x7E and lib.orc_e4m3_rne_sat(ctypes.c_float(-500.0)) == 0xFE


def test_w4a8_per_tensor_matches_reference_generator():
    g = np.load(os.path.join(GOLDEN, "w4a8_ref_golden.npz"))
    m, n, k = (int(x) for x in g["shape"])
    # nibble order of the reference's packer: even k in bits 0-3, odd k in bits 4-7
    assert np.array_equal(O.pack_int4_along_k(g["b_int8"]).ravel(), g["b_packed"])
    out = O.w4a8_per_tensor(g["a"], g["b_packed"], 1.5, m, n, k)
    assert np.array_equal(bits(out), bits(g["expected"]))


def test_w4a8_per_group_formula():
    rng = np.random.default_rng(3)
    m, n, k, gs = 5, 12, 256, 128
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    sw = rng.uniform(1e-3, 1e-2, (k // gs, n)).astype(np.float32)
    sa = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    out = O.w4a8_per_group(a, O.pack_int4_along_k(w), sw, sa, m, n, k, gs)
    y = np.zeros((m, n), np.float32)
    for g in range(k // gs):
        acc = a[:, g * gs:(g + 1) * gs].astype(np.int32) @ w[g * gs:(g + 1) * gs].astype(np.int32)
        # fused multiply-add: the product of two fp32 values is exact in fp64, one rounding at the end
        y = (acc.astype(np.float64) * sw[g][None, :].astype(np.float64) + y.astype(np.float64)).astype(np.float32)
    want = (y * sa[:, None]).astype(np.float32)
    assert np.array_equal(bits(out), bits(want))
    # one group and unit scales reduce to the per-tensor reference formula with scalar 1
    one = O.w4a8_per_group(a, O.pack_int4_along_k(w), np.ones((1, n), np.float32), np.ones(m, np.float32),
                           m, n, k, k)
    assert np.array_equal(bits(one), bits(O.w4a8_per_tensor(a, O.pack_int4_along_k(w), 1.0, m, n, k)))


def test_w4a8_per_group_readings_bracket_the_definition():
    """The fused definition, the unfused fp32 reading and the exact sum agree within the stated bound, and the
    ragged forms (odd k, a shorter last group) reduce to the same integer sums."""
    rng = np.random.default_rng(36)
    m, n, k, gs = 7, 10, 640, 128
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w = rng.integers(-8, 8, (k, n), dtype=np.int8)
    sw = (rng.uniform(1e-3, 1e-2, (k // gs, n)) * rng.choice([-1.0, 1.0], (k // gs, n))).astype(np.float32)
    sa = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    wp = O.pack_int4_along_k(w)
    fused = O.w4a8_per_group(a, wp, sw, sa, m, n, k, gs)
    unfused, exact, mag = O.w4a8_per_group_readings(a, wp, sw, sa, m, n, k, gs)
    groups = k // gs
    bound = (groups + 2) * 2.0 ** -24 * mag + 2.0 ** -149
    assert (np.abs(fused.astype(np.float64) - exact) <= bound).all()
    assert (np.abs(unfused.astype(np.float64) - exact) <= bound).all()
    want = (a.astype(np.int64) @ w.astype(np.int64)).astype(np.float64)
    one = O.w4a8_per_group_readings(a, wp, np.ones((1, n), np.float32), np.ones(m, np.float32), m, n, k, k)[1]
    assert np.array_equal(one, want)
    # odd k and a last group of 37 elements
    k2 = 293
    a2, w2 = a[:, :k2], w[:k2]
    exact2 = O.w4a8_per_group_readings(a2, O.pack_int4_along_k(w2), sw[:3], sa, m, n, k2, 128)[1]
    ref2 = np.zeros((m, n))
    for g in range(3):
        ref2 += (a2[:, g * 128:(g + 1) * 128].astype(np.int64) @ w2[g * 128:(g + 1) * 128].astype(np.int64)) \
            * sw[g].astype(np.float64)
    assert np.allclose(exact2, ref2 * sa[:, None].astype(np.float64), rtol=1e-12, atol=0)


def test_zn_storage_helper_matches_the_reference_layout(w8a8_golden):
    """The zN packing used by the GPU tests places every element where the reference's layout::zN says."""
    import problems as P
    g = w8a8_golden
    coords = g["layout_coords"]
    for row in g["layout_table"]:
        tag, eb, rows, cols = (int(x) for x in row[:4])
        if tag == 2 and eb == 1:
            assert [P.zn_offset(rows, cols, int(r), int(c)) for r, c in coords] == [int(x) for x in row[5:]]
            b = np.arange(rows * cols, dtype=np.int64).reshape(rows, cols).astype(np.int8)
            flat = P.zn_storage(b).ravel()
            assert flat.size == int(row[4])   # Capacity()
            for r, c in coords:
                assert flat[P.zn_offset(rows, cols, int(r), int(c))] == b[int(r), int(c)]


def test_quantize_per_token_int8_definition():
    """The int8 activation quantiser's oracle against its definition written with numpy (round half to even, one
    fp32 multiply per element, scale = amax / 127, all-zero rows)."""
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((37, 96)) * rng.uniform(1e-4, 30.0, (37, 1))).astype(np.float32)
    x[3] = 0.0
    x[4, :8] = np.float32(0.5) * np.abs(x[4]).max() / 127 * np.arange(-4, 4)
    q, s = O.quantize_per_token_int8(x)
    amax = np.abs(x).max(axis=1)
    assert np.array_equal(s, (amax / np.float32(127.0)).astype(np.float32))
    with np.errstate(divide="ignore"):
        inv = np.where(amax > 0, np.float32(127.0) / amax, np.float32(0.0)).astype(np.float32)
    want = np.clip(np.rint((x * inv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    assert np.array_equal(q, want)
    assert (q[3] == 0).all() and s[3] == 0.0
    assert np.abs(q).max(axis=1)[np.arange(37) != 3].min() == 127

