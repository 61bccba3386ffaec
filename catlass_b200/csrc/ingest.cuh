// Ingestion pre-passes: bring operands the tensor-core kernels cannot read in place into their canonical form,
// in the caller's workspace.  They run only for shapes and layouts off the fast path and are plain HBM-bound
// copies: one pass over the operand, coalesced on the side that is written.
//
// The tensor-core kernels stream their operands with TMA, which needs 16-byte aligned row pitches, and (for the
// packed 4-bit formats) rows that run along K.  The reference's own tests also run
//   - K that is not a multiple of the kernels' K block, even odd K (W4A8: tests/test_example.py:141-152 runs
//     m=860 n=5712 k=4535; MXFP4: tests/optest/tests/test_54_ascend950_fp4_mx_matmul_aswt.py:37-54 runs
//     k = 2, 33, 63, 129),
//   - operands stored the other way round (MX: all four transpose pairs,
//     tests/optest/tests/test_53_ascend950_fp8_mx_matmul_aswt.py:21-30; W4A8: weights packed along N,
//     tests/optest/tests/test_32_w4a8_matmul.py:11-28).
// The reference pads K on chip (include/catlass/gemm/block/block_mmad_mx_tla.hpp:357,389 pads to 64); here the
// pre-pass writes rows padded with zeros to a whole number of K blocks, which adds nothing to any sum.
#pragma once

#include <stdint.h>

namespace cb200 {

// dst[r][0 .. dst_pitch) = src[r][0 .. valid) followed by zeros; when `clear_last_high_nibble` the upper four bits
// of byte valid-1 are cleared too (packed 4-bit rows with an odd element count).
// (All three kernels: blockIdx.y walks a batch of matrices, src_batch / dst_batch bytes apart.)
__global__ void pad_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint32_t rows,
                                uint64_t src_pitch, uint32_t dst_pitch, uint32_t valid, uint32_t clear_last_high_nibble,
                                uint64_t src_batch = 0, uint64_t dst_batch = 0)
{
    src += blockIdx.y * src_batch;
    dst += blockIdx.y * dst_batch;
    const uint64_t words_per_row = dst_pitch / 16;  // dst_pitch is a multiple of 16
    const uint64_t total = static_cast<uint64_t>(rows) * words_per_row;
    for (uint64_t w = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; w < total;
         w += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t r = w / words_per_row;
        const uint32_t c0 = static_cast<uint32_t>(w - r * words_per_row) * 16u;
        const uint8_t* s = src + r * src_pitch;
        uint8_t v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t c = c0 + i;
            uint8_t x = c < valid ? s[c] : 0;
            if (clear_last_high_nibble && c + 1 == valid) {
                x &= 0x0F;
            }
            v[i] = x;
        }
        *reinterpret_cast<uint4*>(dst + r * dst_pitch + c0) = *reinterpret_cast<const uint4*>(v);
    }
}

// Transposes a byte matrix: src is [k][rows] (pitch src_pitch), dst is [rows][dst_pitch] with columns >= k zero.
// 32 x 32 tiles through shared memory: reads and writes are both coalesced.
__global__ void transpose_bytes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint32_t rows,
                                       uint32_t k, uint64_t src_pitch, uint32_t dst_pitch, uint64_t src_batch = 0,
                                       uint64_t dst_batch = 0)
{
    src += blockIdx.y * src_batch;
    dst += blockIdx.y * dst_batch;
    __shared__ uint8_t tile[32][33];
    const uint32_t tiles_r = (rows + 31) / 32, tiles_k = dst_pitch / 32;  // dst_pitch is a multiple of 32
    const uint64_t total = static_cast<uint64_t>(tiles_r) * tiles_k;
    for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t tr = static_cast<uint32_t>(t % tiles_r), tk = static_cast<uint32_t>(t / tiles_r);
        for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
            const uint32_t kk = tk * 32 + i, r = tr * 32 + threadIdx.x;
            tile[i][threadIdx.x] = (kk < k && r < rows) ? src[kk * src_pitch + r] : 0;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
            const uint32_t r = tr * 32 + i, kk = tk * 32 + threadIdx.x;
            if (r < rows) {
                dst[static_cast<uint64_t>(r) * dst_pitch + kk] = tile[threadIdx.x][i];
            }
        }
        __syncthreads();
    }
}

// Transposes a matrix of 4-bit values: src holds [k][rows] values, two per byte along `rows` (even index in bits
// 0-3, pitch src_pitch bytes); dst holds [rows][k] values, two per byte along k (pitch dst_pitch bytes, columns
// >= k zero).  One thread builds one 32-bit word of dst (eight k values of one row).
__global__ void transpose_nibbles_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint32_t rows,
                                         uint32_t k, uint64_t src_pitch, uint32_t dst_pitch, uint64_t src_batch = 0,
                                         uint64_t dst_batch = 0)
{
    src += blockIdx.y * src_batch;
    dst += blockIdx.y * dst_batch;
    const uint32_t words_per_row = dst_pitch / 4;
    const uint64_t total = static_cast<uint64_t>(rows) * words_per_row;
    // consecutive threads take consecutive rows of one word column: they read neighbouring source bytes
    for (uint64_t w = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; w < total;
         w += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t r = static_cast<uint32_t>(w % rows);
        const uint32_t wc = static_cast<uint32_t>(w / rows);
        uint32_t out = 0;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t kk = wc * 8 + i;
            uint32_t nib = 0;
            if (kk < k) {
                nib = (src[kk * src_pitch + (r >> 1)] >> ((r & 1u) * 4u)) & 0xFu;
            }
            out |= nib << (i * 4u);
        }
        *reinterpret_cast<uint32_t*>(dst + static_cast<uint64_t>(r) * dst_pitch + wc * 4u) = out;
    }
}

// ---- grouped slice-K: pad every group's K range to whole 128-row blocks ----
// One block.  group_list holds ascending prefix sums over K (clamped to k).  Per group: src[g] = (first source row,
// rows, first destination block, destination blocks); blocks[g] = (first destination block, destination blocks),
// the table the matmul kernel reads.  *total_blocks = destination blocks in all.
__global__ void slice_k_plan_kernel(const void* group_list, uint32_t is_i32, uint32_t groups, uint32_t k, int4* src,
                                    int2* blocks, uint32_t* total_blocks)
{
    if (threadIdx.x == 0) {
        long long prev = 0;
        uint32_t blk = 0;
        for (uint32_t g = 0; g < groups; ++g) {
            long long e = is_i32 ? static_cast<long long>(static_cast<const int32_t*>(group_list)[g])
                                 : static_cast<const long long*>(group_list)[g];
            e = e > static_cast<long long>(k) ? static_cast<long long>(k) : e;
            const uint32_t len = e > prev ? static_cast<uint32_t>(e - prev) : 0u;
            const uint32_t nb = (len + 127u) / 128u;
            src[g] = make_int4(static_cast<int>(prev), static_cast<int>(len), static_cast<int>(blk), static_cast<int>(nb));
            blocks[g] = make_int2(static_cast<int>(blk), static_cast<int>(nb));
            blk += nb;
            prev = e > prev ? e : prev;  // the golden restarts at the previous entry (also when the list is not ascending)
        }
        *total_blocks = blk;
    }
}

// dst row r (of the padded layout) = the source row of its group, or zeros in a group's padding.  One warp per row,
// 16-byte chunks; `width` (bytes per row, a multiple of 16) is m for A ([k][m]) and n for B ([k][n]).
__global__ void slice_k_scatter_kernel(const uint8_t* __restrict__ src_rows, uint8_t* __restrict__ dst_rows,
                                       uint32_t width, const int4* __restrict__ table, uint32_t groups,
                                       const uint32_t* __restrict__ total_blocks)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t rows = *total_blocks * 128u;
    for (uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const uint32_t blk = r >> 7;
        // first group whose block range ends beyond blk (skips empty groups)
        uint32_t lo = 0, hi = groups - 1;
        while (lo < hi) {
            const uint32_t mid = (lo + hi) >> 1;
            const int4 e = table[mid];
            if (static_cast<uint32_t>(e.z + e.w) > blk) {
                hi = mid;
            } else {
                lo = mid + 1;
            }
        }
        const int4 e = table[lo];
        const uint32_t local = r - static_cast<uint32_t>(e.z) * 128u;
        const bool real = local < static_cast<uint32_t>(e.y);
        const uint4* s = reinterpret_cast<const uint4*>(src_rows + (static_cast<uint64_t>(e.x) + local) * width);
        uint4* d = reinterpret_cast<uint4*>(dst_rows + static_cast<uint64_t>(r) * width);
        for (uint32_t c = lane; c < width / 16u; c += 32) {
            d[c] = real ? s[c] : make_uint4(0, 0, 0, 0);
        }
    }
}

}  // namespace cb200
