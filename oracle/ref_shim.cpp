// Builds the reference's OWN CPU golden (its header-only C++ templates) into a small shared library so
// that the plain-C restatement in oracle.c can be checked against it and so that it can be timed as the
// CPU baseline.  TEST INFRASTRUCTURE ONLY.
//
// The reference headers are included from the reference tree at build time (see the Makefile's REF
// variable); no reference source is copied into this repository.  Only host-side headers are used:
// examples/common/golden/{matmul,fill_data}.hpp and include/catlass/{gemm_coord,layout/layout}.hpp.
#include <cmath>   // the golden header uses std::exp without including <cmath> itself
#include <cstdint>
#include <cstring>
#include <stack>
#include <vector>

#include "golden/fill_data.hpp"
#include "golden/matmul.hpp"

using namespace Catlass;

namespace {
template <class LayoutB>
void RunQuant(uint32_t m, uint32_t n, uint32_t k, const int8_t *a, bool aColMajor, const int8_t *b,
              const float *scale, const float *perToken, float *out)
{
    std::vector<int8_t> va(a, a + size_t(m) * k), vb(b, b + size_t(k) * n);
    std::vector<float> vs(scale, scale + n), vp(perToken, perToken + m), vo(size_t(m) * n);
    GemmCoord shape{m, n, k};
    layout::VectorLayout ls{n}, lp{m};
    layout::RowMajor lo{m, n};
    LayoutB lb{k, n};
    if (aColMajor) {
        layout::ColumnMajor la{m, k};
        golden::QuantMatmul(shape, va, la, vb, lb, vs, ls, vp, lp, vo, lo);
    } else {
        layout::RowMajor la{m, k};
        golden::QuantMatmul(shape, va, la, vb, lb, vs, ls, vp, lp, vo, lo);
    }
    std::memcpy(out, vo.data(), vo.size() * sizeof(float));
}

template <class LayoutB>
void RunGrouped(uint32_t m, uint32_t n, uint32_t k, uint32_t g, const int64_t *groupList, const int8_t *a,
                const int8_t *b, const float *scale, const float *perToken, float *out)
{
    std::vector<int64_t> gl(groupList, groupList + g);
    std::vector<int8_t> va(a, a + size_t(m) * k), vb(b, b + size_t(g) * k * n);
    std::vector<float> vs(scale, scale + size_t(g) * n), vp(perToken, perToken + m);
    std::vector<float> vo(out, out + size_t(m) * n); // rows past the last group keep the caller's bytes
    GemmCoord shape{m, n, k};
    layout::VectorLayout ls{n}, lp{m};
    layout::RowMajor la{m, k}, lo{m, n};
    LayoutB lb{k, n};
    golden::ComputeGroupedMatmulPerTokenDequant(shape, g, gl, va, la, vb, lb, vs, ls, vp, lp, vo, lo);
    std::memcpy(out, vo.data(), vo.size() * sizeof(float));
}

template <class LayoutB>
void RunFixpipe(uint32_t m, uint32_t n, uint32_t k, uint32_t g, const int64_t *groupList, const int8_t *a,
                const int8_t *b, int quantMode, float scalePerTensor, const float *perChannel, float *out)
{
    std::vector<int64_t> gl(groupList, groupList + g);
    std::vector<int8_t> va(a, a + size_t(m) * k), vb(b, b + size_t(g) * k * n);
    std::vector<float> vc(perChannel ? perChannel : nullptr, perChannel ? perChannel + n : nullptr);
    std::vector<float> vo(out, out + size_t(m) * n);
    GemmCoord shape{m, n, k};
    layout::RowMajor la{m, k}, lo{m, n};
    LayoutB lb{k, n};
    golden::ComputeGroupedMatmulFixpipeDequant(shape, g, gl, va, la, vb, lb, vo, lo, quantMode, scalePerTensor, vc);
    std::memcpy(out, vo.data(), vo.size() * sizeof(float));
}
} // namespace

extern "C" {

// golden::ComputeGroupedMatmulFixpipeDequant, examples/common/golden/matmul.hpp:234-269
void ref_grouped_fixpipe_dequant(uint32_t m, uint32_t n, uint32_t k, uint32_t g, const int64_t *groupList,
                                 const int8_t *a, const int8_t *b, int layoutB, int quantMode, float scalePerTensor,
                                 const float *perChannel, float *out)
{
    if (layoutB == 1) {
        RunFixpipe<layout::ColumnMajor>(m, n, k, g, groupList, a, b, quantMode, scalePerTensor, perChannel, out);
    } else {
        RunFixpipe<layout::RowMajor>(m, n, k, g, groupList, a, b, quantMode, scalePerTensor, perChannel, out);
    }
}

// golden::ComputeGroupedMatmulSliceKPerTokenDequant, examples/common/golden/matmul.hpp:326-359
// (A column-major m x k, B row-major k x n, groups along K, one m x n output block per group)
void ref_grouped_quant_matmul_slice_k(uint32_t m, uint32_t n, uint32_t k, uint32_t g, const int64_t *groupList,
                                      const int8_t *a, const int8_t *b, const float *scale, const float *perToken,
                                      float *out)
{
    std::vector<int64_t> gl(groupList, groupList + g);
    std::vector<int8_t> va(a, a + size_t(m) * k), vb(b, b + size_t(k) * n);
    std::vector<float> vs(scale, scale + size_t(g) * n), vp(perToken, perToken + size_t(g) * m);
    std::vector<float> vo(out, out + size_t(g) * m * n);
    GemmCoord shape{m, n, k};
    layout::VectorLayout ls{n}, lp{m};
    layout::ColumnMajor la{m, k};
    layout::RowMajor lb{k, n}, lo{m, n};
    golden::ComputeGroupedMatmulSliceKPerTokenDequant(shape, g, gl, va, la, vb, lb, vs, ls, vp, lp, vo, lo);
    std::memcpy(out, vo.data(), vo.size() * sizeof(float));
}

// golden::QuantMatmul, examples/common/golden/matmul.hpp:303-324
void ref_quant_matmul(uint32_t m, uint32_t n, uint32_t k, const int8_t *a, int layoutA, const int8_t *b,
                      int layoutB, const float *scale, const float *perToken, float *out)
{
    if (layoutB == 1) {
        RunQuant<layout::ColumnMajor>(m, n, k, a, layoutA == 1, b, scale, perToken, out);
    } else {
        RunQuant<layout::RowMajor>(m, n, k, a, layoutA == 1, b, scale, perToken, out);
    }
}

// golden::ComputeGroupedMatmulPerTokenDequant, examples/common/golden/matmul.hpp:271-301
void ref_grouped_quant_matmul_slice_m(uint32_t m, uint32_t n, uint32_t k, uint32_t g,
                                      const int64_t *groupList, const int8_t *a, const int8_t *b, int layoutB,
                                      const float *scale, const float *perToken, float *out)
{
    if (layoutB == 1) {
        RunGrouped<layout::ColumnMajor>(m, n, k, g, groupList, a, b, scale, perToken, out);
    } else {
        RunGrouped<layout::RowMajor>(m, n, k, g, groupList, a, b, scale, perToken, out);
    }
}

// golden::GenerateGroupList, examples/common/golden/fill_data.hpp:134-151 (srand(0), sorted rand()%(m+1))
void ref_generate_group_list(uint32_t m, uint32_t g, int64_t *out)
{
    auto gl = golden::GenerateGroupList<int64_t>(m, g);
    std::memcpy(out, gl.data(), g * sizeof(int64_t));
}

// golden::FillRandomData<int8_t,int>, examples/common/golden/fill_data.hpp:43-49 (uses rand())
void ref_fill_int8(int8_t *out, uint64_t count, int low, int high, unsigned seed)
{
    std::srand(seed);
    std::vector<int8_t> v(count);
    golden::FillRandomData<int8_t, int>(v, low, high);
    std::memcpy(out, v.data(), count);
}

// Layout offset functions of the kept surface: include/catlass/layout/matrix.hpp:24-165 (RowMajor),
// :168-304 (ColumnMajor), :475-649 (zN); tag 0/1/2.  elemBytes selects MakeLayout<int8_t|int32_t>.
int64_t ref_layout_offset(int tag, int elemBytes, uint32_t rows, uint32_t cols, uint32_t r, uint32_t c)
{
    MatrixCoord coord{r, c};
    if (tag == 0) {
        return layout::RowMajor{rows, cols}.GetOffset(coord);
    }
    if (tag == 1) {
        return layout::ColumnMajor{rows, cols}.GetOffset(coord);
    }
    if (elemBytes == 1) {
        return layout::zN::MakeLayout<int8_t>(rows, cols).GetOffset(coord);
    }
    return layout::zN::MakeLayout<int32_t>(rows, cols).GetOffset(coord);
}

int64_t ref_layout_capacity(int tag, int elemBytes, uint32_t rows, uint32_t cols)
{
    if (tag == 0) {
        return layout::RowMajor{rows, cols}.Capacity();
    }
    if (tag == 1) {
        return layout::ColumnMajor{rows, cols}.Capacity();
    }
    if (elemBytes == 1) {
        return layout::zN::MakeLayout<int8_t>(rows, cols).Capacity();
    }
    return layout::zN::MakeLayout<int32_t>(rows, cols).Capacity();
}

} // extern "C"
