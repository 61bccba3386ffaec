"""The C-ABI shared library loads without a GPU and exports every symbol the public header declares.
No compute entry point is called here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from catlass_b200 import build, capi
    build.build()
    return capi.load()


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            names |= set(re.findall(r"CB200_API\s+[\w\s\*]+?\b(cb200_\w+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_operator_triples():
    names = declared_symbols()
    for op in ("cb200_quant_matmul", "cb200_grouped_quant_matmul_slice_m"):
        for suffix in ("", "_can_implement", "_workspace_size"):
            assert op + suffix in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_version_and_counters(lib):
    assert b"sm_100a" in lib.cb200_version()
    assert lib.cb200_launch_count() >= 0


def test_can_implement_validates_without_a_device(lib):
    from catlass_b200 import capi
    args = capi.QuantMatmulArgs(m=128, n=256, k=100, layout_a=0, layout_b=1, a=16, b=32, scale=64,
                                per_token_scale=128, d=256)
    assert lib.cb200_quant_matmul_can_implement(ctypes.byref(args)) == capi.INVALID  # k % 16
    args.k = 128
    assert lib.cb200_quant_matmul_can_implement(ctypes.byref(args)) == capi.SUCCESS
    args.a = 17
    assert lib.cb200_quant_matmul_can_implement(ctypes.byref(args)) == capi.INVALID  # alignment
    assert lib.cb200_quant_matmul_workspace_size(ctypes.byref(args)) == 0


def test_struct_layout_matches_the_header(lib):
    """Size and every field offset of the ctypes mirrors equal what a C compiler gives the header's structs."""
    import subprocess
    import tempfile
    from catlass_b200 import capi
    pairs = [
        ("cb200_quant_matmul_args", capi.QuantMatmulArgs),
        ("cb200_grouped_quant_matmul_args", capi.GroupedQuantMatmulArgs),
        ("cb200_grouped_fixpipe_dequant_args", capi.GroupedFixpipeDequantArgs),
        ("cb200_grouped_quant_matmul_slice_k_args", capi.GroupedSliceKArgs),
        ("cb200_grouped_quant_matmul_host_args", capi.GroupedQuantMatmulHostArgs),
        ("cb200_w4a8_matmul_args", capi.W4A8MatmulArgs),
        ("cb200_mx_matmul_args", capi.MxMatmulArgs),
        ("cb200_mx_grouped_matmul_args", capi.MxGroupedMatmulArgs),
        ("cb200_mx_grouped_swiglu_quant_args", capi.MxGroupedSwigluQuantArgs),
        ("cb200_mx_grouped_finalize_routing_args", capi.MxGroupedFinalizeRoutingArgs),
        ("cb200_mx_quantize_args", capi.MxQuantizeArgs),
        ("cb200_quantize_int8_args", capi.QuantizeInt8Args),
    ]
    lines = []
    for cname, ctype in pairs:
        offs = ", ".join(f"offsetof({cname}, {f[0]})" for f in ctype._fields_)
        fmt = " ".join(["%zu"] * (len(ctype._fields_) + 1))
        lines.append(f'  printf("{fmt}\\n", sizeof({cname}), {offs});')
    src = "#include <stdio.h>\n#include <stddef.h>\n#include \"catlass_b200.h\"\nint main(void) {\n" + \
        "\n".join(lines) + "\n  return 0; }\n"
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(td, "t")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.strip().splitlines()
    for (cname, ctype), line in zip(pairs, out):
        want = [ctypes.sizeof(ctype)] + [getattr(ctype, f[0]).offset for f in ctype._fields_]
        assert [int(x) for x in line.split()] == want, cname
