"""The example programs (ports of the reference's examples 12 and 07 onto the C++ surface) run on the GPU with
the reference runner's arguments (tests/test_example.py: `12_quant_matmul 256 512 1024`,
`07/10 ... 128 512 1024 2048`) and must print "Compare success."."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def exes(cuda):
    sys.path.insert(0, os.path.join(ROOT, "tests", "examples"))
    import build as example_build
    return {os.path.basename(e): e for e in example_build.build()}


@pytest.mark.parametrize("argv", [["256", "512", "1024"], ["16", "4096", "2048"], ["300", "264", "1040"]])
def test_example_12_quant_matmul(exes, argv):
    r = subprocess.run([exes["12_quant_matmul"]] + argv + ["0"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "Compare success." in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("argv", [["128", "512", "1024", "2048"], ["7", "1000", "256", "512"]])
def test_example_07_grouped(exes, argv):
    r = subprocess.run([exes["07_grouped_matmul_slice_m_per_token_dequant"]] + argv + ["0"], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "Compare success." in r.stdout, r.stdout + r.stderr


def test_example_rejects_unsupported_shape(exes):
    r = subprocess.run([exes["12_quant_matmul"], "64", "64", "100"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 1 and "not supported" in r.stderr
