"""Generates the golden fixtures in this directory from the REFERENCE itself.

Run where the reference tree is present (it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/reference

It uses (a) the reference's C++ CPU golden, compiled from the reference tree into oracle/_ref/libref.so by
oracle/Makefile, and (b) the reference's Python data generators and goldens for MX, W4A8 and the SwiGLU +
MX quantisation epilogue, imported as modules.
Only small arrays (inputs and the reference's outputs for them) are stored; no reference code is copied.
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle_lib as O  # noqa: E402


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def w8a8(ref_lib):
    rng = np.random.default_rng(2024)
    out = {}
    # dense, the four layout combinations
    m, n, k = 24, 40, 64
    a = rng.integers(-127, 128, m * k, dtype=np.int8)
    b = rng.integers(-127, 128, k * n, dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    p = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    out.update(dense_shape=np.array([m, n, k]), dense_a=a, dense_b=b, dense_scale=s, dense_pt=p)
    for la in (0, 1):
        for lb in (0, 1):
            out[f"dense_out_{la}{lb}"] = O.ref_quant_matmul(a, b, s, p, m, n, k, la, lb)
    # grouped, group list from the reference's generator (srand(0); repeats = empty groups)
    gm, gn, gk, gg = 40, 24, 32, 9
    gl = O.ref_generate_group_list(gm, gg)
    ga = rng.integers(-16, 17, gm * gk, dtype=np.int8)
    gb = rng.integers(-16, 17, gg * gk * gn, dtype=np.int8)
    gs = rng.uniform(0, 1, gg * gn).astype(np.float32)
    gp = rng.uniform(0, 1, gm).astype(np.float32)
    out.update(grp_shape=np.array([gm, gn, gk, gg]), grp_list=gl, grp_a=ga, grp_b=gb, grp_scale=gs, grp_pt=gp)
    for lb in (0, 1):
        out[f"grp_out_{lb}"] = O.ref_grouped_quant_matmul(ga, gb, gl, gs, gp, gm, gn, gk, lb)
    # per-tensor / per-channel grouped dequant (example 48's golden) on the grouped inputs above, and slice-K
    # (example 11's golden: A column-major, groups along K) on inputs of its own
    pcs = rng.uniform(0, 1, gn).astype(np.float32)
    out.update(fix_pcs=pcs, fix_scalar=np.float32(0.37))
    for mode in (0, 1):
        for lb in (0, 1):
            out[f"fix_out_{mode}{lb}"] = O.ref_grouped_fixpipe_dequant(ga, gb, gl, mode, 0.37, pcs, gm, gn, gk, lb)
    sm, sn, sk, sg = 16, 24, 80, 5
    sgl = O.ref_generate_group_list(sk, sg)
    sa_ = rng.integers(-16, 17, sm * sk, dtype=np.int8)
    sb_ = rng.integers(-16, 17, sk * sn, dtype=np.int8)
    ss_ = rng.uniform(0, 1, sg * sn).astype(np.float32)
    sp_ = rng.uniform(0, 1, sg * sm).astype(np.float32)
    out.update(slk_shape=np.array([sm, sn, sk, sg]), slk_list=sgl, slk_a=sa_, slk_b=sb_, slk_scale=ss_, slk_pt=sp_,
               slk_out=O.ref_grouped_quant_matmul_slice_k(sa_, sb_, sgl, ss_, sp_, sm, sn, sk))
    # the runner's group list: examples 07/10/47 are run with 128 groups over m = 512
    out["group_list_512_128"] = O.ref_generate_group_list(512, 128)
    # layout offsets: (tag, elem_bytes, rows, cols) -> offsets of a fixed coordinate walk
    coords = [(r, c) for r in (0, 1, 15, 16, 17, 33) for c in (0, 1, 31, 32, 33, 63)]
    lay = []
    for tag in (0, 1, 2):
        for eb in (1, 4):
            rows, cols = 34, 64
            offs = [ref_lib.ref_layout_offset(tag, eb, rows, cols, r, c) for r, c in coords]
            lay.append([tag, eb, rows, cols, ref_lib.ref_layout_capacity(tag, eb, rows, cols)] + offs)
    out["layout_coords"] = np.array(coords)
    out["layout_table"] = np.array(lay, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "w8a8_ref_golden.npz"), **out)


def mx(reference):
    import torch
    g53 = _load(os.path.join(reference, "examples/53_ascend950_fp8_mx_matmul/gen_data.py"), "g53")
    g54 = _load(os.path.join(reference, "examples/54_ascend950_fp4_mx_matmul/gen_data.py"), "g54")
    out = {}
    torch.manual_seed(53)
    m, n, k = 16, 24, 96
    for name, gen, fmt in (("fp8", g53, "E4M3"), ("fp4", g54, "E2M1")):
        a = torch.randn(m, k)
        b = torch.randn(k, n)
        a[2, :32] = 0.0          # an all-zero block
        a[3, 40] = 3.0e4         # a value that saturates
        a[5, 64:96] *= 1.0e-5    # a block of tiny values
        qa, sa, da = gen._quantize(a, fmt, 1)
        qb, sb, db = gen._quantize(b, fmt, 0)
        if name == "fp8":
            qa_code = qa.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
            qb_code = qb.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        else:
            qa_code = gen._quantize_to_fp4_lut(qa, fmt)[1].numpy()
            qb_code = gen._quantize_to_fp4_lut(qb, fmt)[1].numpy()
            out["fp4_packed_a"] = gen._pack_fp4_nibbles(torch.from_numpy(qa_code)).numpy()
        out[f"{name}_a"] = a.numpy()
        out[f"{name}_b"] = b.numpy()
        out[f"{name}_a_code"] = qa_code
        out[f"{name}_b_code"] = qb_code                      # [k, n]
        out[f"{name}_a_sf"] = sa.to(torch.float8_e8m0fnu).view(torch.uint8).numpy()   # [m, blocks(+pad)]
        out[f"{name}_b_sf"] = sb.to(torch.float8_e8m0fnu).view(torch.uint8).numpy()   # [blocks(+pad), n]
        out[f"{name}_a_deq"] = da.numpy()
        out[f"{name}_b_deq"] = db.numpy()
        out[f"{name}_golden"] = (da @ db).numpy()
    np.savez_compressed(os.path.join(HERE, "mx_ref_golden.npz"), **out)


def w4a8(reference):
    g32 = _load(os.path.join(reference, "examples/32_w4a8_matmul/gen_data.py"), "g32")
    np.random.seed(32)
    m, n, k = 12, 20, 48
    a = g32.gen_data_int8(m, k)
    # trans=True is the reference's column-major B: values packed along K
    b_int8, b_int4 = g32.gen_data_int4(k, n, True)
    expected = np.float32(1.5) * np.dot(a.astype(np.float32), b_int8.astype(np.float32))
    np.savez_compressed(os.path.join(HERE, "w4a8_ref_golden.npz"), shape=np.array([m, n, k]), a=a,
                        b_int8=b_int8, b_packed=b_int4.view(np.uint8), expected=expected.astype(np.float32))


def swiglu_quant(reference):
    """SwiGLU + MX quantisation epilogue: the golden functions of the reference's example, on a small fp32 matrix
    that covers ordinary values, saturation of the swish, all-zero blocks, blocks below E4M3's exponent floor,
    values that round up across a binade, and a block holding Inf."""
    import types

    import torch
    # the script imports two dtype packages for its file I/O only; its swiglu() and quant() are pure torch
    for name, attrs in (("en_dtypes", ["float8_e8m0"]), ("ml_dtypes", ["float8_e4m3fn", "float8_e5m2"])):
        if name not in sys.modules:
            stub = types.ModuleType(name)
            for attr in attrs:
                setattr(stub, attr, np.uint8)
            sys.modules[name] = stub
    cmp_mod = _load(os.path.join(
        reference, "experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant/compare.py"), "swq")
    rng = np.random.default_rng(65)
    m, n = 24, 256
    c = (rng.standard_normal((m, n)) * 3.0).astype(np.float32)
    h = n // 2
    c[1, :] *= 40.0                      # swish saturates, products reach the E4M3 clamp after scaling
    c[2, :32] = 0.0                      # an all-zero block (act = 0)
    c[3, :] *= 1e-4                      # blocks whose largest exponent is below the floor
    c[4, :] *= 1e-30
    c[5, 0:32] = 1.9999                  # rounds up across a binade in bf16
    c[5, h:h + 32] = 1.0
    c[6, 3] = np.inf                     # Inf in act: swish(inf) = inf
    c[6, h + 3] = 2.0
    c[7, :h] = np.linspace(-30, 30, h, dtype=np.float32)
    c[7, h:] = 448.0
    c[8, :h] = rng.uniform(-1, 1, h).astype(np.float32) * np.float32(2.0) ** rng.integers(-20, 20, h)
    t = torch.from_numpy(c)
    s = cmp_mod.swiglu(t).to(torch.bfloat16)
    s_bits = s.view(torch.int16).numpy().view(np.uint16)
    q, sc = cmp_mod.quant(s.to(torch.float32), 36)
    np.savez_compressed(os.path.join(HERE, "swiglu_quant_ref_golden.npz"), c=c, s_bits=s_bits,
                        q=q.view(np.uint8), scale=sc.astype(np.uint8))


if __name__ == "__main__":
    reference = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CATLASS_REFERENCE", "")
    if not os.path.isdir(reference):
        raise SystemExit("usage: make_golden.py /path/to/reference")
    O.build_oracle()
    ref_lib = O.ref()
    if ref_lib is None:
        raise SystemExit("oracle/_ref/libref.so was not built (make -C oracle REF=/path/to/reference)")
    w8a8(ref_lib)
    mx(reference)
    w4a8(reference)
    swiglu_quant(reference)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
