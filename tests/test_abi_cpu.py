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
    """Field offsets of the ctypes mirrors equal those a C compiler gives the header's structs."""
    import subprocess
    import tempfile
    from catlass_b200 import capi
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "catlass_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu\n", sizeof(cb200_quant_matmul_args), offsetof(cb200_quant_matmul_args, a),
         offsetof(cb200_quant_matmul_args, acc), offsetof(cb200_quant_matmul_args, block_num));
  printf("%zu %zu %zu %zu\n", sizeof(cb200_grouped_quant_matmul_args),
         offsetof(cb200_grouped_quant_matmul_args, a), offsetof(cb200_grouped_quant_matmul_args, group_list),
         offsetof(cb200_grouped_quant_matmul_args, block_num));
  return 0; }'''
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(td, "t")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()
    q, g = capi.QuantMatmulArgs, capi.GroupedQuantMatmulArgs
    assert [int(x) for x in out[:4]] == [ctypes.sizeof(q), q.a.offset, q.acc.offset, q.block_num.offset]
    assert [int(x) for x in out[4:]] == [ctypes.sizeof(g), g.a.offset, g.group_list.offset, g.block_num.offset]
