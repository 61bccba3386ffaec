// Problem and tile descriptors of the operator surface (host-side PODs).
// Same names and accessors as the reference's Coord (include/catlass/coord.hpp:24-407), GemmShape / GemmCoord
// (include/catlass/gemm_coord.hpp:26-160) and MatrixShape / MatrixCoord (include/catlass/matrix_coord.hpp:19-116),
// reduced to what the quantized-matmul path uses.
#pragma once

#include <cstdint>
#include <type_traits>

namespace Catlass {

template <int RANK_, class Index_ = uint32_t, class LongIndex_ = int64_t>
struct Coord {
    static constexpr int RANK = RANK_;
    using Index = Index_;
    using LongIndex = LongIndex_;

    Index idx[RANK_] = {};

    constexpr Coord() = default;
    constexpr explicit Coord(Index value)
    {
        for (int i = 0; i < RANK_; ++i) {
            idx[i] = value;
        }
    }
    constexpr Index& operator[](int dim) { return idx[dim]; }
    constexpr Index const& operator[](int dim) const { return idx[dim]; }
    template <int DIM>
    constexpr Index& At() { return idx[DIM]; }
    template <int DIM>
    constexpr Index const& At() const { return idx[DIM]; }
    constexpr bool operator==(Coord const& other) const
    {
        for (int i = 0; i < RANK_; ++i) {
            if (idx[i] != other.idx[i]) {
                return false;
            }
        }
        return true;
    }
    constexpr bool operator!=(Coord const& other) const { return !(*this == other); }
};

template <class... Ts>
constexpr auto MakeCoord(Ts... values)
{
    using Index = typename std::common_type<Ts...>::type;
    Coord<sizeof...(Ts), Index> c;
    Index tmp[] = {static_cast<Index>(values)...};
    for (int i = 0; i < static_cast<int>(sizeof...(Ts)); ++i) {
        c[i] = tmp[i];
    }
    return c;
}

/// Compile-time tile shape.
template <uint32_t M_ = 1, uint32_t N_ = 1, uint32_t K_ = 1>
struct GemmShape {
    static constexpr uint32_t M = M_;
    static constexpr uint32_t N = N_;
    static constexpr uint32_t K = K_;
    static constexpr int64_t MN = int64_t(M_) * N_;
    static constexpr int64_t MK = int64_t(M_) * K_;
    static constexpr int64_t KN = int64_t(N_) * K_;
    static constexpr int64_t COUNT = MN * K_;
};

/// Run-time (m, n, k) coordinate / problem size.
struct GemmCoord : public Coord<3, uint32_t> {
    using Base = Coord<3, uint32_t>;
    static constexpr int M_INDEX = 0;
    static constexpr int N_INDEX = 1;
    static constexpr int K_INDEX = 2;

    constexpr GemmCoord() = default;
    constexpr GemmCoord(uint32_t m, uint32_t n, uint32_t k)
    {
        idx[0] = m;
        idx[1] = n;
        idx[2] = k;
    }
    constexpr uint32_t const& m() const { return idx[M_INDEX]; }
    constexpr uint32_t& m() { return idx[M_INDEX]; }
    constexpr uint32_t const& n() const { return idx[N_INDEX]; }
    constexpr uint32_t& n() { return idx[N_INDEX]; }
    constexpr uint32_t const& k() const { return idx[K_INDEX]; }
    constexpr uint32_t& k() { return idx[K_INDEX]; }
    constexpr Coord<2, uint32_t> GetCoordMN() const { return MakeCoord(m(), n()); }
    constexpr Coord<2, uint32_t> GetCoordMK() const { return MakeCoord(m(), k()); }
    constexpr Coord<2, uint32_t> GetCoordKN() const { return MakeCoord(k(), n()); }
};

template <uint32_t ROW_ = 1, uint32_t COLUMN_ = 1>
struct MatrixShape {
    static constexpr uint32_t ROW = ROW_;
    static constexpr uint32_t COLUMN = COLUMN_;
    static constexpr int64_t COUNT = int64_t(ROW_) * COLUMN_;
};

/// (row, column) coordinate.
struct MatrixCoord : public Coord<2, uint32_t> {
    static constexpr int ROW_INDEX = 0;
    static constexpr int COLUMN_INDEX = 1;

    constexpr MatrixCoord() = default;
    constexpr MatrixCoord(uint32_t row, uint32_t column)
    {
        idx[0] = row;
        idx[1] = column;
    }
    constexpr MatrixCoord(Coord<2, uint32_t> const& c)
    {
        idx[0] = c[0];
        idx[1] = c[1];
    }
    constexpr uint32_t const& row() const { return idx[ROW_INDEX]; }
    constexpr uint32_t& row() { return idx[ROW_INDEX]; }
    constexpr uint32_t const& column() const { return idx[COLUMN_INDEX]; }
    constexpr uint32_t& column() { return idx[COLUMN_INDEX]; }
};

/// ceil(a / b) and the next multiple of b (include/catlass/detail/alignment.hpp:17-81).
template <class T>
constexpr T CeilDiv(T a, T b)
{
    return (a + b - 1) / b;
}
template <class T>
constexpr T RoundUp(T a, T b)
{
    return CeilDiv(a, b) * b;
}

}  // namespace Catlass
