// Matrix layouts of the operator surface: offset maps from a (row, column) coordinate to linear memory.
// Same public interface as the reference's layout::RowMajor (include/catlass/layout/matrix.hpp:24-165),
// ColumnMajor (:168-304), zN (:475-649) and VectorLayout (include/catlass/layout/vector.hpp:20): constructors,
// MakeLayout<Element>, GetOffset, GetTileLayout, shape / stride accessors, Capacity.
#pragma once

#include <cstdint>

#include "gemm_coord.hpp"

namespace Catlass::layout {

/// Rows are contiguous: offset = row * ldm + column.
struct RowMajor {
    static constexpr int RANK = 2;
    using Index = uint32_t;
    using LongIndex = int64_t;
    using Shape = Coord<RANK, Index>;
    using Stride = Coord<RANK, LongIndex>;

    RowMajor(Index rows = 0, Index cols = 0) : RowMajor(rows, cols, LongIndex(cols)) {}
    RowMajor(Index rows, Index cols, LongIndex ldm)
    {
        shape_[0] = rows;
        shape_[1] = cols;
        stride_[0] = ldm;
        stride_[1] = 1;
    }
    RowMajor(Shape shape, Stride stride) : shape_(shape), stride_(stride) {}

    template <class Element>
    static RowMajor MakeLayout(Index rows, Index cols)
    {
        return RowMajor(rows, cols);
    }
    LongIndex GetOffset(MatrixCoord const& c) const { return LongIndex(c.row()) * stride_[0] + LongIndex(c.column()); }
    RowMajor GetTileLayout(MatrixCoord const& tileShape) const { return RowMajor(Shape(tileShape), stride_); }
    Shape shape() const { return shape_; }
    Index shape(int i) const { return shape_[i]; }
    Stride stride() const { return stride_; }
    LongIndex stride(int i) const { return stride_[i]; }
    LongIndex Capacity() const { return LongIndex(shape_[0]) * stride_[0]; }

private:
    Shape shape_;
    Stride stride_;
};

/// Columns are contiguous: offset = column * ldm + row.
struct ColumnMajor {
    static constexpr int RANK = 2;
    using Index = uint32_t;
    using LongIndex = int64_t;
    using Shape = Coord<RANK, Index>;
    using Stride = Coord<RANK, LongIndex>;

    ColumnMajor(Index rows = 0, Index cols = 0) : ColumnMajor(rows, cols, LongIndex(rows)) {}
    ColumnMajor(Index rows, Index cols, LongIndex ldm)
    {
        shape_[0] = rows;
        shape_[1] = cols;
        stride_[0] = 1;
        stride_[1] = ldm;
    }
    ColumnMajor(Shape shape, Stride stride) : shape_(shape), stride_(stride) {}

    template <class Element>
    static ColumnMajor MakeLayout(Index rows, Index cols)
    {
        return ColumnMajor(rows, cols);
    }
    LongIndex GetOffset(MatrixCoord const& c) const { return LongIndex(c.row()) + LongIndex(c.column()) * stride_[1]; }
    ColumnMajor GetTileLayout(MatrixCoord const& tileShape) const { return ColumnMajor(Shape(tileShape), stride_); }
    Shape shape() const { return shape_; }
    Index shape(int i) const { return shape_[i]; }
    Stride stride() const { return stride_; }
    LongIndex stride(int i) const { return stride_[i]; }
    LongIndex Capacity() const { return LongIndex(shape_[1]) * stride_[1]; }

private:
    Shape shape_;
    Stride stride_;
};

/// The "zN" fractal layout: the matrix is cut into fractals of 16 rows x 32 bytes; inside a fractal rows are
/// contiguous ("z"), fractals follow each other down a column of fractals first ("N").  Rows are padded to a
/// multiple of 16 and columns to a multiple of the 32-byte element count.
struct zN {
    static constexpr int RANK = 4;
    static constexpr int ORG_SHAPE_RANK = 2;
    using Index = uint32_t;
    using LongIndex = int64_t;
    using OrgShape = Coord<ORG_SHAPE_RANK, Index>;
    using Shape = Coord<RANK, Index>;     // rows in fractal, fractal rows, cols in fractal, fractal cols
    using Stride = Coord<RANK, LongIndex>;

    static constexpr Index kRowsPerFractal = 16;
    static constexpr Index kBytesPerFractalRow = 32;

    zN() = default;
    zN(OrgShape org, Shape shape, Stride stride) : org_(org), shape_(shape), stride_(stride) {}

    template <class Element>
    static zN MakeLayout(Index rows, Index cols)
    {
        const Index colsInFractal = kBytesPerFractalRow / Index(sizeof(Element));
        const Index rowsRound = RoundUp(rows, kRowsPerFractal);
        const Index colsRound = RoundUp(cols, colsInFractal);
        OrgShape org;
        org[0] = rows;
        org[1] = cols;
        Shape shape;
        shape[0] = kRowsPerFractal;
        shape[1] = rowsRound / kRowsPerFractal;
        shape[2] = colsInFractal;
        shape[3] = colsRound / colsInFractal;
        Stride stride;
        stride[0] = colsInFractal;                       // next row inside a fractal
        stride[1] = LongIndex(kRowsPerFractal) * colsInFractal;  // next fractal down
        stride[2] = 1;                                   // next column inside a fractal
        stride[3] = LongIndex(rowsRound) * colsInFractal;        // next column of fractals
        return zN(org, shape, stride);
    }
    LongIndex GetOffset(MatrixCoord const& c) const
    {
        const LongIndex r = c.row(), col = c.column();
        return (r / shape_[0]) * stride_[1] + (r % shape_[0]) * stride_[0] + (col / shape_[2]) * stride_[3] +
               (col % shape_[2]) * stride_[2];
    }
    zN GetTileLayout(MatrixCoord const& tileShape) const
    {
        OrgShape org;
        org[0] = tileShape.row();
        org[1] = tileShape.column();
        Shape shape = shape_;
        shape[1] = CeilDiv(tileShape.row(), shape_[0]);
        shape[3] = CeilDiv(tileShape.column(), shape_[2]);
        return zN(org, shape, stride_);
    }
    Index orgShape(int i) const { return org_[i]; }
    Shape shape() const { return shape_; }
    Index shape(int i) const { return shape_[i]; }
    Stride stride() const { return stride_; }
    LongIndex stride(int i) const { return stride_[i]; }
    LongIndex Capacity() const { return stride_[3] * LongIndex(shape_[3]); }

private:
    OrgShape org_;
    Shape shape_;
    Stride stride_;
};

/// One-dimensional layout of scale vectors.
struct VectorLayout {
    static constexpr int RANK = 1;
    using Index = uint32_t;
    using LongIndex = int64_t;
    using Shape = Coord<RANK, Index>;
    using Stride = Coord<RANK, LongIndex>;

    VectorLayout(Index size = 0) : shape_(size), stride_(LongIndex(1)) {}
    template <class Element>
    static VectorLayout MakeLayout(Index size)
    {
        return VectorLayout(size);
    }
    LongIndex GetOffset(Coord<1, Index> const& c) const { return LongIndex(c[0]) * stride_[0]; }
    VectorLayout GetTileLayout(Coord<1, Index> const& tileShape) const { return VectorLayout(tileShape[0]); }
    Shape shape() const { return shape_; }
    Index shape(int i) const { return shape_[i]; }
    Stride stride() const { return stride_; }
    LongIndex Capacity() const { return LongIndex(shape_[0]) * stride_[0]; }

private:
    Shape shape_;
    Stride stride_;
};

}  // namespace Catlass::layout
