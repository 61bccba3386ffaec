"""Compiles the example programs (test infrastructure: they link the CPU oracle for their self-check)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
BIN = os.path.join(HERE, "bin")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
EXAMPLES = ["12_quant_matmul", "07_grouped_matmul_slice_m_per_token_dequant"]


def build():
    from catlass_b200 import build as libbuild
    lib = libbuild.build()
    subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "liboracle.so"], check=True)
    os.makedirs(BIN, exist_ok=True)
    libdir = os.path.dirname(lib)
    oracledir = os.path.join(ROOT, "oracle")
    out = []
    for name in EXAMPLES:
        exe = os.path.join(BIN, name)
        src = os.path.join(HERE, name + ".cpp")
        if not os.path.exists(exe) or os.path.getmtime(exe) < max(os.path.getmtime(src), os.path.getmtime(lib)):
            cmd = ["nvcc", "-std=c++17", "-O2", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a",
                   "-I", os.path.join(ROOT, "include"), "-I", oracledir, "-I", HERE, src, "-o", exe,
                   "-L", libdir, "-lcatlass_b200", "-L", oracledir, "-loracle",
                   "-Xlinker", f"-rpath={libdir}", "-Xlinker", f"-rpath={oracledir}"]
            subprocess.run(cmd, check=True)
        out.append(exe)
    return out


if __name__ == "__main__":
    print(build())
