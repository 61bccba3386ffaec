"""The C++ operator surface (include/catlass_b200/*.hpp) on the host: layouts against the reference's own
offsets (golden fixture produced from the reference's layout classes), descriptor accessors, and that the
example programs compile against the surface and the C ABI."""
import os
import subprocess
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "w8a8_ref_golden.npz")

PROGRAM = r'''
#include <cstdio>
#include <cstdlib>
#include "catlass_b200/gemm_coord.hpp"
#include "catlass_b200/layout.hpp"
#include "catlass_b200/status.hpp"
using namespace Catlass;
template <class L> void dump(L const& l, int argc, char** argv) {
    std::printf("%lld", (long long)l.Capacity());
    for (int i = 5; i + 1 < argc; i += 2)
        std::printf(" %lld", (long long)l.GetOffset(MatrixCoord(std::atoi(argv[i]), std::atoi(argv[i + 1]))));
    std::printf("\n");
}
int main(int argc, char** argv) {
    // argv: tag elemBytes rows cols (r c)*
    int tag = std::atoi(argv[1]), eb = std::atoi(argv[2]);
    uint32_t rows = std::atoi(argv[3]), cols = std::atoi(argv[4]);
    if (tag == 0) dump(layout::RowMajor::MakeLayout<int8_t>(rows, cols), argc, argv);
    else if (tag == 1) dump(layout::ColumnMajor::MakeLayout<int8_t>(rows, cols), argc, argv);
    else if (eb == 1) dump(layout::zN::MakeLayout<int8_t>(rows, cols), argc, argv);
    else dump(layout::zN::MakeLayout<int32_t>(rows, cols), argc, argv);
    GemmCoord g{3, 5, 7};
    static_assert(GemmShape<128, 256, 64>::MN == 128 * 256, "tile shape");
    if (g.m() != 3 || g.n() != 5 || g.k() != 7 || g.GetCoordMN()[1] != 5 || CeilDiv(10u, 4u) != 3 ||
        RoundUp(10u, 4u) != 12 || int(Status::kSuccess) != 0 || int(Status::kInvalid) != 1) return 3;
    auto tile = layout::RowMajor(100, 200).GetTileLayout(MatrixCoord(16, 32));
    if (tile.shape(0) != 16 || tile.shape(1) != 32 || tile.stride(0) != 200) return 4;
    return 0;
}
'''


def test_layouts_match_the_reference_offsets():
    g = np.load(GOLDEN)
    coords = g["layout_coords"]
    table = g["layout_table"]
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "t.cpp")
        open(src, "w").write(PROGRAM)
        exe = os.path.join(td, "t")
        subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), src, "-o", exe],
                       check=True)
        flat = [str(int(v)) for rc in coords for v in rc]
        for row in table:
            tag, eb, rows, cols, capacity = (int(x) for x in row[:5])
            out = subprocess.run([exe, str(tag), str(eb), str(rows), str(cols)] + flat, capture_output=True,
                                 text=True, check=True).stdout.split()
            got = [int(x) for x in out]
            assert got[0] == capacity, (tag, eb, "capacity", got[0], capacity)
            assert got[1:] == [int(x) for x in row[5:]], (tag, eb)


def test_example_programs_compile_against_the_surface():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests", "examples"))
    import build as example_build
    exes = example_build.build()
    assert len(exes) == 2 and all(os.path.exists(e) for e in exes)
    # without arguments they print the reference's usage line and exit non-zero, touching no GPU
    r = subprocess.run([exes[0]], capture_output=True, text=True)
    assert r.returncode == 64 and "usage: 12_quant_matmul m n k" in r.stderr


DESCRIPTORS = r"""
#include <cstdio>
#include "catlass_b200/catlass_kernel.hpp"
using namespace Catlass;
template <class K> int probe(typename K::Arguments const& a) {
    // null operands: every descriptor must map onto its C-ABI struct and be refused by the argument check
    return Gemm::Device::DeviceGemm<K>::CanImplement(a) == Status::kSuccess ? 1 : 0;
}
int main() {
    int accepted = 0;
    { using K = Gemm::Kernel::GroupedMatmulSliceKPerTokenDequant<>; K::Arguments a{}; a.problemShape = GemmCoord{128, 128, 256}; a.problemCount = 2; accepted += probe<K>(a); }
    { using K = Gemm::Kernel::GroupedMxMatmulSliceM<false>; K::Arguments a{}; a.problemShape = GemmCoord{128, 128, 256}; a.problemCount = 2; accepted += probe<K>(a); }
    { using K = Gemm::Kernel::GroupedMxMatmulSliceM<true, layout::RowMajor, int32_t>; K::Arguments a{}; a.problemShape = GemmCoord{128, 128, 256}; a.problemCount = 2; accepted += probe<K>(a); }
    { using K = Gemm::Kernel::GroupedMxMatmulSliceMSwigluMxQuant<>; K::Arguments a{}; a.problemShape = GemmCoord{128, 512, 256}; a.problemCount = 2; accepted += probe<K>(a); }
    { using K = Gemm::Kernel::GroupedMxMatmulFinalizeRouting<>; K::Arguments a{}; a.problemShape = GemmCoord{128, 512, 256}; a.problemCount = 2; a.batch = 16; accepted += probe<K>(a); }
    std::printf("%d\n", accepted);
    return accepted;
}
"""


def test_grouped_and_fused_descriptors_map_onto_the_c_abi():
    """The C++ descriptors of the grouped siblings and the fused MoE epilogues compile, link against the library and
    reach its argument checks (which refuse the null operands without touching a device)."""
    import sys
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from catlass_b200 import build as libbuild
    lib = libbuild.build()
    libdir = os.path.dirname(lib)
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "d.cpp")
        open(src, "w").write(DESCRIPTORS)
        exe = os.path.join(td, "d")
        subprocess.run(["nvcc", "-std=c++17", "-x", "cu", "-I", os.path.join(ROOT, "include"), src, "-o", exe, "-L", libdir,
                        "-lcatlass_b200", "-Xlinker", f"-rpath={libdir}"], check=True)
        r = subprocess.run([exe], capture_output=True, text=True)
        assert r.returncode == 0 and r.stdout.strip() == "0", (r.returncode, r.stdout, r.stderr)
