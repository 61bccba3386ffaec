// MXFP8 (E4M3) and MXFP4 (E2M1) block-scaled matmul for sm_100a:
//     D[m,n] = bf16_rne( sum_k (a[m,k] * 2^(ea[m,k/32]-127)) * (b[k,n] * 2^(eb[n,k/32]-127)) ),  fp32 accumulate
// with one E8M0 scale per 32 contiguous K elements of every row of A and every column of B.
//
// What the reference's MxMatmulTla / BlockMmadTla<MmadMx> compute
// (include/catlass/gemm/kernel/mx_matmul_tla.hpp:29-393, include/catlass/gemm/block/block_mmad_mx_tla.hpp:291-647):
// there too the scaling happens inside the matrix unit; here it is tcgen05.mma.kind::mxf8f6f4 / kind::mxf4 with
// .block_scale, the scale factors sitting in TMEM next to the accumulator.
//
// Two kernels:
//   mx_pack_scales_kernel  rewrites the caller's scale arrays ([rows][K/32] bytes, the reference's layout:
//                          include/tla/layout.hpp:609-660, examples/53_ascend950_fp8_mx_matmul/gen_data.py:390-401)
//                          into the tile order the tensor core's scale copy wants: per 128 rows x 4 scale
//                          blocks a 512-byte block [row % 32][row / 32][4 bytes].  Output goes to the
//                          caller-provided workspace; B's blocks are padded to a whole number of 256-wide tiles.
//   mx_gemm_kernel         persistent, warp-specialised like the W8A8 kernel, twelve warps: TMA producer (operand
//                          tiles + packed scale blocks), MMA issuer (the block-scaled MMAs), two scale copier
//                          threads (tcgen05.cp scale blocks smem -> TMEM, off the MMA thread), eight epilogue warps
//                          (two per TMEM lane quarter; fp32 -> bf16, or fp32 as it is).  Tile 128 x 256 with ONE
//                          accumulator: a 128 x 128 MMA would run shorter than issuing it takes (~70 ns), which
//                          capped 128-wide tiles at half the tensor rate; 256 columns plus the scale columns do
//                          not leave room for a second accumulator, so the epilogue pulls its columns out of TMEM
//                          first, hands the accumulator back, and stores afterwards.
//
// kSwiglu (grouped E4M3 problems): the reference's GroupedMxMatmulSliceMSwigluMxQuantTla with its
// BlockEpilogueSwigluMxQuant (include/catlass/gemm/kernel/grouped_mx_matmul_slice_m_swiglu_mx_quant_tla.hpp:29-408,
// include/catlass/epilogue/tile/tile_swiglu_mx_quant.hpp:27-286).  The matmul result C [m][n] is never written:
// a tile pairs 128 columns of its left half ("act") with the same 128 columns of its right half ("gate") as one
// 128 x 256 accumulator, and the epilogue computes S = act / (1 + exp(-act)) * gate in fp32, rounds S to bf16
// and MX-quantises it along N, 32 columns per E8M0 scale, into E4M3 bytes Q [m][n/2] and scales [m][n/64].  A
// thread owns one row of the accumulator, so a block of 32 columns is 32 registers of one thread: the block's
// largest exponent needs no exchange between threads.
//
// kMxEpiRouting (grouped E4M3 problems): the reference's GroupedMxMatmulFinalizeRoutingNoDeterTla with
// BlockEpilogueFinalizeRoutingNoDeter (include/catlass/gemm/kernel/grouped_mx_matmul_finalize_routing_no_deter_tla.hpp,
// include/catlass/epilogue/block/block_epilogue_finalize_routing_no_deter.hpp): the second half of an MoE expert MLP.
// Row p of C, plus its group's bias, is weighted with logit[p] and added into row row_index[p] of the fp32 output
// with vector reductions (red.global.add.v4.f32) straight from the accumulator's registers; C is never written.
// Rows of different tiles that meet in one output row are added in the order the tiles finish: like the reference's
// kernel of that name the result is not bit-reproducible from run to run.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "w8a8_gemm.cuh"

namespace cb200 {

constexpr int kMxBlockN = 256;  // one tcgen05.mma of 128 x 256 runs about as long as issuing it costs its thread
constexpr int kMxAccs = 1;      // one accumulator: 256 columns + the scale columns leave no room for a second
constexpr int kMxStages = 4;
// warps: 0 TMA producer, 1 MMA issuer, 2 and 3 scale copiers, then the epilogue warps: sixteen (four per TMEM lane
// quarter, 64 columns each), or eight with 128 columns each for the SwiGLU epilogue, whose threads need the registers
__host__ __device__ constexpr int mx_epilogue_warps(int epi) { return epi == 1 ? 8 : 16; }
__host__ __device__ constexpr int mx_threads(int epi) { return (4 + mx_epilogue_warps(epi)) * 32; }

struct MxParams {
    uint32_t m, n, k;
    uint32_t fp4;              // 0: E4M3 bytes, 1: E2M1 packed two per byte
    uint32_t num_k_blocks;     // K bytes per row / 128
    uint32_t words_per_stage;  // scale words (4 scale blocks = 128 K elements) per 128-byte stage: 1 (fp8), 2 (fp4)
    uint32_t kq_total;         // scale words per row = K / 128
    uint32_t band_rows;        // tile rows per band of the tile order (see mx_tile_coords)
    const uint8_t* sfa;        // packed scales of A: [ceil(m/128)][kq_total][512]
    const uint8_t* sfb;        // packed scales of B: [ceil(n/128)][kq_total][512]
    void* d;                   // [m][n] bf16, or fp32 when out_f32
    unsigned* status;
    uint32_t out_f32;
    // grouped (slice-M) problems: the row tiles come from a table a planning kernel wrote (see mx_group_plan_kernel)
    const int4* tile_table;           // [row tile] = (first row, one past the group's last row, group, 0)
    const uint32_t* num_row_tiles;    // number of table entries
    uint32_t sfb_blocks_per_group;    // 128-row scale blocks of B per group: 2 * ceil(n / 256)
    // SwiGLU + MX quantisation epilogue (kMxEpiSwiglu): d holds E4M3 bytes [m][n/2], q_scale E8M0 bytes [m][n/64]
    uint8_t* q_scale;
    // finalize-routing epilogue (kMxEpiRouting): d is the fp32 output [batch][n] that rows are added into
    const float* logit;          // [m] weight of row p
    const void* row_index;       // [m] output row of row p (int64, or int32 when row_index_i32)
    const __nv_bfloat16* bias;   // [groups][n] or nullptr
    uint32_t row_index_i32;
    uint32_t batch;
};

constexpr int kMxEpiPlain = 0;    // D = C as bf16 or fp32
constexpr int kMxEpiSwiglu = 1;   // Q, scales = MX quantisation of SwiGLU(C)
constexpr int kMxEpiRouting = 2;  // out[row_index[p]] += logit[p] * (C[p] + bias[group])

// One block: turns the group list of a grouped slice-M problem into the row-tile table the matmul and the scale
// re-tiling walk.  Group g owns rows [start_g, start_g + size_g) of A and D, clamped to m; its row tiles are 128
// rows each (the last one partial); empty groups add nothing.  The list holds sizes (the reference's example 55:
// examples/55_ascend950_mx_grouped_matmul_slice_m/mx_grouped_matmul_slice_m.cpp:265, non-cumsum) or prefix sums.
// tile_rows: 128, or 256 for the CTA-pair kernel (a pair's tile is 256 rows of one group).
__global__ void mx_group_plan_kernel(const void* group_list, uint32_t is_i32, uint32_t is_prefix_sum, uint32_t groups,
                                     uint32_t m, int4* table, uint32_t* num_row_tiles, uint32_t tile_rows)
{
    __shared__ uint32_t s_begin[kMaxGroups + 1];
    __shared__ uint32_t s_tile[kMaxGroups + 1];
    if (threadIdx.x == 0) {
        long long prev = 0;
        uint32_t tiles = 0;
        for (uint32_t g = 0; g < groups; ++g) {
            long long v = is_i32 ? static_cast<long long>(static_cast<const int32_t*>(group_list)[g])
                                 : static_cast<const long long*>(group_list)[g];
            long long end = is_prefix_sum ? v : prev + (v < 0 ? 0 : v);
            end = end < prev ? prev : (end > static_cast<long long>(m) ? static_cast<long long>(m) : end);
            s_begin[g] = static_cast<uint32_t>(prev);
            s_tile[g] = tiles;
            tiles += static_cast<uint32_t>((end - prev + tile_rows - 1) / tile_rows);
            prev = end;
        }
        s_begin[groups] = static_cast<uint32_t>(prev);
        s_tile[groups] = tiles;
        *num_row_tiles = tiles;
    }
    __syncthreads();
    for (uint32_t g = threadIdx.x; g < groups; g += blockDim.x) {
        const uint32_t begin = s_begin[g], end = s_begin[g + 1];
        for (uint32_t t = s_tile[g]; t < s_tile[g + 1]; ++t) {
            table[t] = make_int4(static_cast<int>(begin + (t - s_tile[g]) * tile_rows), static_cast<int>(end),
                                 static_cast<int>(g), 0);
        }
    }
}

struct MxSmem {
    static constexpr int kABytes = kBlockM * kBlockKBytes;      // 16 KB
    static constexpr int kBBytes = kMxBlockN * kBlockKBytes;    // 32 KB
    // scale blocks: A up to two words (1 KB) at +0, B two 128-row blocks x up to two words (2 KB) at +1024
    static constexpr int kSfBytes = 4096;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;  // 52 KB
    static constexpr int kRingBytes = kMxStages * kStageBytes;
    static constexpr int kBarrierBytes = (3 * kMxStages + 4) * 8 + 16;
    static constexpr int kTotalBytes = 1024 + kRingBytes + kBarrierBytes;
};

// Re-tiles one operand's scale bytes: out is [row_blocks][kq_total][512], one 512-byte block per 128 rows x 4 scale
// blocks, laid out [row % 32][row / 32][4 bytes].  The input is either
//   rows-major  [rows][ks_pitch] bytes (the operand's rows run along K: A row-major, B column-major), or
//   k-major     [ks_pitch / 2][rows][2] bytes (the operand is stored the other way round),
// the reference's two scale layouts (tests/optest/tests/mx_golden.py:253-266), with ks_pitch = the even number of
// scale blocks per row the caller's array holds.  Blocks at or beyond `kblocks_valid` = ceil(K / 32), and rows
// past the end, get the neutral scale 2^0 (their elements are zero).
// blockIdx.y walks a batch (the weight matrices of a grouped problem): input and output advance by in_batch /
// out_batch bytes.  With a row-tile table (grouped A) output block t holds the 128 rows that start at the table's
// row for tile t, which need not be a multiple of 128.
__global__ void mx_pack_scales_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, uint32_t rows,
                                      uint32_t kblocks_valid, uint32_t ks_pitch, uint32_t kq_total,
                                      uint32_t row_blocks, uint32_t k_major, uint64_t in_batch, uint64_t out_batch,
                                      const int4* tile_table, const uint32_t* num_row_tiles,
                                      uint32_t table_tile_rows = 128)
{
    in += blockIdx.y * in_batch;
    out += blockIdx.y * out_batch;
    if (tile_table != nullptr) {  // (a 256-row table tile fills two consecutive 128-row output blocks)
        const uint32_t blocks = *num_row_tiles * (table_tile_rows / 128u);
        row_blocks = blocks < row_blocks ? blocks : row_blocks;
    }
    const size_t words = static_cast<size_t>(row_blocks) * kq_total * 128;
    const bool word_loads = !k_major && (ks_pitch & 3u) == 0 && (reinterpret_cast<uintptr_t>(in) & 3u) == 0;
    for (size_t w = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; w < words;
         w += static_cast<size_t>(gridDim.x) * blockDim.x) {
        // consecutive threads walk consecutive scale words of one row: coalesced reads
        const uint32_t kq = static_cast<uint32_t>(w % kq_total);
        const uint32_t prow = static_cast<uint32_t>(w / kq_total);  // row index inside the padded output
        const uint32_t row = tile_table == nullptr
                                 ? prow
                                 : static_cast<uint32_t>(tile_table[prow / table_tile_rows].x) + prow % table_tile_rows;
        uint32_t v = 0x7F7F7F7Fu;
        if (row < rows) {
            if (word_loads && kq * 4 + 4 <= kblocks_valid) {
                v = *reinterpret_cast<const uint32_t*>(in + static_cast<size_t>(row) * ks_pitch + kq * 4);
            } else {
                v = 0;
#pragma unroll
                for (uint32_t b = 0; b < 4; ++b) {
                    const uint32_t kb = kq * 4 + b;
                    uint32_t byte = 0x7Fu;
                    if (kb < kblocks_valid) {
                        byte = k_major ? in[(static_cast<size_t>(kb >> 1) * rows + row) * 2 + (kb & 1u)]
                                       : in[static_cast<size_t>(row) * ks_pitch + kb];
                    }
                    v |= byte << (8 * b);
                }
            }
        }
        const uint32_t rb = prow / 128, r = prow % 128;
        uint8_t* dst = out + (static_cast<size_t>(rb) * kq_total + kq) * 512 + (r % 32) * 16 + (r / 32) * 4;
        *reinterpret_cast<uint32_t*>(dst) = v;
    }
}

// MX quantisation of 32 bf16 values (their bit patterns in `bits`) to E4M3 with one E8M0 scale, the arithmetic of
// the reference's epilogue on bf16 exponent fields (include/catlass/epilogue/tile/tile_swiglu_mx_quant.hpp:167-215;
// restated for the CPU in experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant/compare.py:41-121):
//   max_exp = largest exponent field of the block, raised to 8 + 127 at least (E4M3's largest exponent is 8)
//   scale   = max_exp - 8 as an E8M0 byte (0 for an all-zero block, 0xFF if the block holds Inf or NaN)
//   q       = e4m3_rne_saturating(bf16(x * 2^-(max_exp - 8 - 127)))
// Returns the scale byte; out[8] receives the 32 E4M3 bytes, column order.
__device__ __forceinline__ uint32_t mx_quant_block_bf16_e4m3(const uint32_t (&bits)[32], uint32_t (&out)[8])
{
    uint32_t max_exp = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const uint32_t e = bits[i] & 0x7f80u;
        max_exp = e > max_exp ? e : max_exp;
    }
    const bool finite = max_exp != 0x7f80u;
    const bool nonzero = max_exp != 0u;
    const uint32_t clamped = max_exp <= 0x0400u ? 0x0400u : max_exp;
    const uint32_t shared = clamped - 0x0400u;
    uint32_t scale = shared >> 7;
    scale = finite ? scale : 0xffu;
    scale = nonzero ? scale : 0u;
    uint32_t inv = 0x7f00u - shared;  // bf16 bits of 2^-(shared exponent)
    inv = finite ? inv : 0x7f81u;     // NaN: the whole block becomes NaN
    inv = nonzero ? inv : 0u;
    inv = shared == 0x7f00u ? 0x0040u : inv;  // 2^-127 is a bf16 denormal
    const float inv_f = __uint_as_float(inv << 16);
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float x = __uint_as_float(bits[4 * w + b] << 16);
            // the product of two bf16 values is exact in fp32; the reference multiplies in bf16 (one rounding)
            const float scaled = __bfloat162float(__float2bfloat16_rn(__fmul_rn(x, inv_f)));
            const uint32_t code = __nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3);
            word |= (code & 0xffu) << (8 * b);
        }
        out[w] = word;
    }
    return scale;
}

// Prepares the output of the finalize-routing epilogue: zeros, plus weight * shared_input in rows
// [offset, offset + shared_rows) (the shared expert's contribution, bf16 -> fp32 before the multiplication:
// experimental/gmm/ascend950_fp8_mx_grouped_matmul_finalize_routing/gen_data_compare.py:744-751).
__global__ void finalize_routing_init_kernel(float* __restrict__ out, uint32_t batch, uint32_t n,
                                             const __nv_bfloat16* __restrict__ shared, float weight, uint32_t offset,
                                             uint32_t shared_rows)
{
    const uint64_t total = static_cast<uint64_t>(batch) * n;
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t r = static_cast<uint32_t>(i / n);
        const uint32_t c = static_cast<uint32_t>(i - static_cast<uint64_t>(r) * n);
        float v = 0.0f;
        if (shared != nullptr && r >= offset && r - offset < shared_rows) {
            v = __fmul_rn(weight, __bfloat162float(shared[static_cast<size_t>(r - offset) * n + c]));
        }
        out[i] = v;
    }
}

// Tile order: bands of `band_rows` tile rows, walked column by column inside a band.  The 148 tiles in flight at
// any time then share the band's row panels of A (the host sizes a band to ~32 MB of A) and a few column panels
// of B, which stay in L2; with a plain row-major order every wave streamed all of B from HBM again (measured at
// 8192^3 fp8: 7x the operand bytes).
__device__ __forceinline__ void mx_tile_coords(uint32_t idx, uint32_t m_tiles, uint32_t n_tiles, uint32_t band_rows,
                                               uint32_t& mt, uint32_t& nt)
{
    const uint32_t per_band = band_rows * n_tiles;
    const uint32_t band = idx / per_band;
    const uint32_t r = idx - band * per_band;
    const uint32_t rows = m_tiles - band * band_rows < band_rows ? m_tiles - band * band_rows : band_rows;
    nt = r / rows;
    mt = band * band_rows + (r - nt * rows);
}

// Finalize routing for one epilogue thread: its accumulator row's 64 columns r (fp32 bit patterns) starting at column
// col_base are added into row `target` of the fp32 output as weight * (C + bias[group]).  Every lane of the warp
// calls this (lanes without a valid target take part in the exchange only).
__device__ __forceinline__ void mx_route_row(const MxParams& p, const uint32_t (&r)[2][32], uint32_t lane,
                                             uint32_t col_base, int32_t group, long long target, float weight)
{
    const bool mine = target >= 0 && target < static_cast<long long>(p.batch);
    float* orow = static_cast<float*>(p.d) + static_cast<size_t>(mine ? target : 0) * p.n;
    const __nv_bfloat16* brow = p.bias != nullptr ? p.bias + static_cast<size_t>(group) * p.n : nullptr;
    if ((p.n & 7u) == 0 && col_base + 64 <= p.n) {
        // Two neighbouring lanes (two rows of C) work together so that every reduction instruction
        // carries 32 contiguous bytes per output row, a whole L2 sector, instead of 16: of each 8
        // columns the even lane keeps its columns 0-3 and hands its columns 4-7 to the odd lane, which
        // hands over its columns 0-3 in return; instruction A then adds the even lane's row (columns
        // 0-3 from the even lane, 4-7 from the odd lane), instruction B the odd lane's row.  With one
        // lane per row every instruction touched 32 sectors half-way: twice the sector operations on
        // the way to L2 (ncu: the L1-to-crossbar request path two thirds busy); worth 3 % here.
        const bool odd = (lane & 1u) != 0;
        const unsigned long long mine_ptr = reinterpret_cast<unsigned long long>(orow);
        const unsigned long long peer_ptr = __shfl_xor_sync(0xffffffffu, mine_ptr, 1);
        const bool peer_ok = __shfl_xor_sync(0xffffffffu, mine ? 1 : 0, 1) != 0;
        float* row_a = reinterpret_cast<float*>(odd ? peer_ptr : mine_ptr);   // the even lane's row
        float* row_b = reinterpret_cast<float*>(odd ? mine_ptr : peer_ptr);   // the odd lane's row
        const bool ok_a = odd ? peer_ok : mine, ok_b = odd ? mine : peer_ok;
        const uint32_t off = odd ? 4u : 0u;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {   // 8 columns at a time
                const uint32_t col = col_base + c * 32 + v * 8;
                float x[8];
                if (brow != nullptr) {
                    const uint4 braw = __ldg(reinterpret_cast<const uint4*>(brow + col));
                    const uint32_t bw[4] = {braw.x, braw.y, braw.z, braw.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        x[2 * e] = __fadd_rn(__uint_as_float(r[c][8 * v + 2 * e]),
                                             __uint_as_float(bw[e] << 16));
                        x[2 * e + 1] = __fadd_rn(__uint_as_float(r[c][8 * v + 2 * e + 1]),
                                                 __uint_as_float(bw[e] & 0xFFFF0000u));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        x[e] = __uint_as_float(r[c][8 * v + e]);
                    }
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    x[e] = __fmul_rn(x[e], weight);
                }
                float keep[4], got[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    keep[e] = odd ? x[4 + e] : x[e];           // stays: the lane's own half of its own row
                    const float send = odd ? x[e] : x[4 + e];  // goes: the other half, to the neighbour
                    got[e] = __shfl_xor_sync(0xffffffffu, send, 1);
                }
                // even lane: A = own row, own columns 0-3;   B = odd's row, its columns 0-3 (received)
                // odd lane:  A = even's row, columns 4-7 (received);   B = own row, own columns 4-7
                const float* va = odd ? got : keep;
                const float* vb = odd ? keep : got;
                if (ok_a) {
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(row_a + col + off),
                                 "f"(va[0]), "f"(va[1]), "f"(va[2]), "f"(va[3])
                                 : "memory");
                }
                if (ok_b) {
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(row_b + col + off),
                                 "f"(vb[0]), "f"(vb[1]), "f"(vb[2]), "f"(vb[3])
                                 : "memory");
                }
            }
        }
        return;
    }
    if (!mine) {
        return;
    }
    const bool vec4 = (p.n & 3u) == 0;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int v = 0; v < 8; ++v) {
            float x[4];
            const uint32_t col = col_base + c * 32 + v * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float y = __uint_as_float(r[c][4 * v + e]);
                if (brow != nullptr && col + e < p.n) {
                    y = __fadd_rn(y, __bfloat162float(brow[col + e]));
                }
                x[e] = __fmul_rn(y, weight);
            }
            if (vec4 && col + 4 <= p.n) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(orow + col), "f"(x[0]),
                             "f"(x[1]), "f"(x[2]), "f"(x[3])
                             : "memory");
            } else {
                for (int e = 0; e < 4; ++e) {
                    if (col + e < p.n) {
                        atomicAdd(orow + col + e, x[e]);
                    }
                }
            }
        }
    }
}

// kGrouped: slice-M groups (the reference's GroupedMxMatmulSliceMTla, example 55): row tiles come from the tile
// table, every group has its own weight matrix (third coordinate of B's tensor map) and B scales.
template <bool kFp4, bool kGrouped, int kEpi = kMxEpiPlain>
__global__ void __launch_bounds__(mx_threads(kEpi), 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const MxParams p)
{
    using S = MxSmem;
    constexpr uint32_t kAccCols = kMxAccs * kMxBlockN;  // fp32 accumulator(s)
    constexpr uint32_t kSfSlot = 24;                    // one scale slot: A up to 8 columns, B up to 16
    constexpr uint32_t kSfCols = kMxStages * kSfSlot;   // one slot per shared-memory stage
    constexpr uint32_t kTmemCols = 512;                 // power of two >= kAccCols + kSfCols
    constexpr uint32_t kWords = kFp4 ? 2 : 1;
    static_assert(kAccCols + kSfCols <= kTmemCols, "TMEM budget");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t ring = raw_addr + pad;
    uint64_t* s_bars = reinterpret_cast<uint64_t*>(smem + S::kRingBytes);
    const uint32_t bar_full = smem_u32(s_bars);
    const uint32_t bar_empty = bar_full + kMxStages * 8;
    const uint32_t bar_tmem_full = bar_empty + kMxStages * 8;
    const uint32_t bar_tmem_empty = bar_tmem_full + 2 * 8;  // (slots for two accumulators are reserved)
    const uint32_t bar_sf_full = bar_tmem_empty + 2 * 8;    // the stage's scale blocks have been copied into TMEM
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + 3 * kMxStages + 4);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t m_tiles = kGrouped ? *p.num_row_tiles : (p.m + kBlockM - 1) / kBlockM;
    constexpr bool kSwiglu = kEpi == kMxEpiSwiglu;
    static_assert(kEpi == kMxEpiPlain || (kGrouped && !kFp4), "the fused epilogues serve grouped E4M3 problems");
    // kSwiglu: a tile is 128 columns of the left half of C next to the same 128 columns of the right half
    const uint32_t n_tiles = kSwiglu ? (p.n / 2 + 127) / 128 : (p.n + kMxBlockN - 1) / kMxBlockN;
    const uint32_t total_tiles = m_tiles * n_tiles;
    // first row, end of the rows that may be stored, group of row tile mt
    auto row_tile = [&](uint32_t mt, int32_t& row0, int32_t& row_end, int32_t& group) {
        if constexpr (kGrouped) {
            const int4 e = __ldg(p.tile_table + mt);
            row0 = e.x;
            row_end = e.y;
            group = e.z;
        } else {
            row0 = static_cast<int32_t>(mt) * kBlockM;
            row_end = static_cast<int32_t>(p.m);
            group = 0;
        }
    };
    const uint32_t num_kb = p.num_k_blocks;

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int s = 0; s < kMxStages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
            mbar_init(bar_sf_full + s * 8, kFp4 ? 2 : 1);  // one arrival per scale copier at work
        }
        for (int a = 0; a < kMxAccs; ++a) {
            mbar_init(bar_tmem_full + a * 8, 1);
            mbar_init(bar_tmem_empty + a * 8, mx_epilogue_warps(kEpi));  // one arrival per epilogue warp
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(s_tmem_ptr), kTmemCols);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem_ptr;
    constexpr uint32_t kStageTx = S::kABytes + S::kBBytes + 3 * kWords * 512;  // A scales + two B scale blocks

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t idx = blockIdx.x; ok && idx < total_tiles; idx += gridDim.x) {
                uint32_t mt, nt;
                mx_tile_coords(idx, m_tiles, n_tiles, p.band_rows, mt, nt);
                int32_t row0, row_end, group;
                row_tile(mt, row0, row_end, group);
                // the tile's two 128-row scale blocks of B (the workspace pads every matrix to a pair)
                const size_t sfb_first = static_cast<size_t>(group) * p.sfb_blocks_per_group;
                const size_t sfb_block0 = sfb_first + (kSwiglu ? nt : 2 * nt);
                const size_t sfb_block1 = sfb_first + (kSwiglu ? p.n / 256 + nt : 2 * nt + 1);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar_empty + stage * 8, phase ^ 1, s_abort, p.status, kDevTimeoutProducer);
                    if (!ok) {
                        break;
                    }
                    const uint32_t full = bar_full + stage * 8;
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    const uint32_t ssf = sb + S::kBBytes;
                    const int32_t k0 = static_cast<int32_t>(kb) * kBlockKBytes;
                    const size_t kq = static_cast<size_t>(kb) * kWords;
                    mbar_expect_tx(full, kStageTx);
                    tma_load_2d(sa, &tmap_a, full, k0, row0);
                    if constexpr (kSwiglu) {  // (B's tensor map then has boxes of 128 rows)
                        tma_load_3d(sb, &tmap_b, full, k0, static_cast<int32_t>(nt) * 128, group);
                        tma_load_3d(sb + S::kBBytes / 2, &tmap_b, full, k0, static_cast<int32_t>(p.n / 2 + nt * 128),
                                    group);
                    } else {
                        tma_load_3d(sb, &tmap_b, full, k0, static_cast<int32_t>(nt) * kMxBlockN, group);
                    }
                    bulk_load(ssf, p.sfa + (static_cast<size_t>(mt) * p.kq_total + kq) * 512, kWords * 512, full);
                    bulk_load(ssf + 1024, p.sfb + (sfb_block0 * p.kq_total + kq) * 512, kWords * 512, full);
                    bulk_load(ssf + 1024 + kWords * 512, p.sfb + (sfb_block1 * p.kq_total + kq) * 512, kWords * 512,
                              full);
                    if (++stage == kMxStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t fmt = kFp4 ? kFmtMxf4E2M1 : kFmtE4M3;
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t idx = blockIdx.x; ok && idx < total_tiles; idx += gridDim.x) {
                ok = mbar_wait(bar_tmem_empty + acc * 8, acc_phase ^ 1, s_abort, p.status, kDevTimeoutMmaTmem);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * kMxBlockN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    // The stage's scale blocks are copied into TMEM slot `stage` by the copier threads, which wait
                    // for the stage's "full" barrier first and whose commit arrives (release) when the copies are
                    // done: acquiring "sf_full" therefore orders this thread after the operand tiles' arrival too,
                    // and one probe per stage less on the thread whose instruction issue sets the kernel's pace.
                    ok = mbar_wait(bar_sf_full + stage * 8, phase, s_abort, p.status, kDevTimeoutMma);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t t_sfa = tmem_base + kAccCols + stage * kSfSlot;
                    const uint32_t t_sfb = t_sfa + 8;
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        const uint64_t da = make_smem_desc_sw128(sa + j * 32, 16, 1024);
                        const uint64_t db = make_smem_desc_sw128(sb + j * 32, 16, 1024);
                        // fp8: MMA j covers scale block j of the stage's single word (byte j)
                        // fp4: MMA j covers 64 elements = scale blocks 2j, 2j+1: word j/2, bytes (j%2)*2..+1
                        const uint32_t word = kFp4 ? (j >> 1) : 0;
                        const uint32_t sf_id = kFp4 ? ((j & 1) * 2) : j;
                        const uint32_t idesc = make_idesc_mx(fmt, fmt, kBlockM, kMxBlockN, sf_id, sf_id);
                        umma_mx<kFp4>(tmem_d, da, db, idesc, (kb | j) != 0 ? 1u : 0u, t_sfa + word * 4,
                                      t_sfb + word * 8);
                    }
                    umma_commit<1>(bar_empty + stage * 8);
                    if (++stage == kMxStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) {
                    break;
                }
                umma_commit<1>(bar_tmem_full + acc * 8);
                if (++acc == kMxAccs) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else if (warp == 2 || warp == 3) {
        // ---- scale copier: smem -> TMEM, one thread.  Issuing a tcgen05 instruction costs its thread ~70 ns
        // whatever it does; three copies on top of four MMAs and a commit per stage made the MMA thread the
        // limit of the kernel, so the copies have a thread of their own.  TMEM slot `stage` is free when the
        // stage's "full" barrier fires: the MMAs that read its previous contents completed before the producer
        // was allowed to refill the stage.
        // (fp4 has two scale words per stage, six copies: warp 2 takes word 0, warp 3 word 1)
        const uint32_t my_word = warp == 2 ? 0u : 1u;
        if (lane == 0 && my_word < kWords) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t idx = blockIdx.x; ok && idx < total_tiles; idx += gridDim.x) {
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar_full + stage * 8, phase, s_abort, p.status, kDevTimeoutConvert);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t ssf = ring + stage * S::kStageBytes + S::kABytes + S::kBBytes;
                    // TMEM layout of a slot: A word w at columns [4w, 4w+4); B word w at [8 + 8w, 8 + 8w + 8):
                    // columns 0-3 of it for the tile's first 128 columns, 4-7 for the second.  Each copy moves
                    // 32 rows x 16 bytes, replicated to the four lane quarters.
                    const uint32_t t_sfa = tmem_base + kAccCols + stage * kSfSlot;
                    const uint32_t t_sfb = t_sfa + 8;
                    {
                        const uint32_t w = my_word;
                        tmem_cp_32x128b_warpx4(t_sfa + w * 4, make_smem_desc_noswizzle(ssf + w * 512, 16, 128));
#pragma unroll
                        for (uint32_t nb = 0; nb < 2; ++nb) {
                            tmem_cp_32x128b_warpx4(
                                t_sfb + w * 8 + nb * 4,
                                make_smem_desc_noswizzle(ssf + 1024 + (nb * kWords + w) * 512, 16, 128));
                        }
                    }
                    umma_commit<1>(bar_sf_full + stage * 8);  // arrives when this thread's copies have completed
                    if (++stage == kMxStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue.  There is room for one accumulator only (256 columns + the scale slots fill TMEM), so between
        // two tiles the tensor core waits for the epilogue to pull the accumulator out: with eight warps reading
        // four 32-column pieces one after the other that took ~2.5 us, against 8.8 us of MMAs per fp8 tile at K = 8192.
        // Sixteen warps (four per lane quarter, 64 columns each) issue their two reads together, wait once and hand
        // their share back before they round or store anything.  (The SwiGLU epilogue keeps eight warps: its
        // threads hold four pieces, 128 registers, and hand back before their arithmetic as well.)
        const uint32_t quad = warp & 3;
        const uint32_t part = (warp - 4) >> 2;   // 0..3: which 64 columns; SwiGLU: 0..1 = `half`
        const uint32_t half = part;
        const bool vec_ok = (p.n & 7u) == 0;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t idx = blockIdx.x; ok && idx < total_tiles; idx += gridDim.x) {
            uint32_t mt, nt;
            mx_tile_coords(idx, m_tiles, n_tiles, p.band_rows, mt, nt);
            int32_t row0, row_end, group;
            row_tile(mt, row0, row_end, group);
            const uint32_t row = static_cast<uint32_t>(row0) + quad * 32 + lane;
            const bool row_ok = static_cast<int32_t>(row) < row_end;
            // finalize routing: this row's target and weight are fetched while the tile's MMAs still run (after the
            // accumulator's hand-over they were a trip to L2 on every tile's critical path)
            long long route_target = -1;
            float route_weight = 0.0f;
            if constexpr (kEpi == kMxEpiRouting) {
                if (row_ok) {
                    route_target = p.row_index_i32
                                       ? static_cast<long long>(static_cast<const int32_t*>(p.row_index)[row])
                                       : static_cast<const long long*>(p.row_index)[row];
                    route_weight = __ldg(p.logit + row);
                }
            }
            ok = mbar_wait(bar_tmem_full + acc * 8, acc_phase, s_abort, p.status, kDevTimeoutEpilogue);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            tcgen05_fence_after();
            if constexpr (kSwiglu) {
                // This warp: output columns [half * 64, half * 64 + 64) of the tile's 128, as two blocks of 32; "act"
                // sits in accumulator columns 0..127, "gate" in 128..255.
                const uint32_t tcols = tmem_base + acc * kMxBlockN + ((quad * 32u) << 16);
                const uint32_t half_n = p.n / 2;
                uint8_t* qrow = static_cast<uint8_t*>(p.d) + static_cast<size_t>(row_ok ? row : 0) * half_n;
                uint8_t* srow = p.q_scale + static_cast<size_t>(row_ok ? row : 0) * (half_n / 32);
                // all four pieces (2 x 32 columns of act and of gate) come out of TMEM first and the accumulator goes
                // back to the MMA issuer before any arithmetic: the next tile's MMAs wait for reads only
                uint32_t ra[2][32], rg[2][32];
#pragma unroll
                for (uint32_t blk = 0; blk < 2; ++blk) {
                    tmem_ld_32x32b_x32(tcols + half * 64 + blk * 32, ra[blk]);
                    tmem_ld_32x32b_x32(tcols + 128 + half * 64 + blk * 32, rg[blk]);
                }
                tmem_ld_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_tmem_empty + acc * 8);
                }
#pragma unroll
                for (uint32_t blk = 0; blk < 2; ++blk) {
                    const uint32_t c0 = half * 64 + blk * 32;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        // S = act / (1 + exp(-act)) * gate, step by step in fp32 as the reference's epilogue does
                        // (tile_swiglu_mx_quant.hpp:96-103), rounded to bf16 (RNE)
                        const float a = __uint_as_float(ra[blk][i]);
                        const float g = __uint_as_float(rg[blk][i]);
                        const float t = __fadd_rn(expf(-a), 1.0f);
                        const float sw = __fmul_rn(__fdiv_rn(a, t), g);
                        ra[blk][i] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(sw)));
                    }
                    uint32_t q[8];
                    const uint32_t scale = mx_quant_block_bf16_e4m3(ra[blk], q);
                    const uint32_t col0 = nt * 128 + c0;
                    if (row_ok && col0 < half_n) {  // (n is a multiple of 256: whole blocks)
                        *reinterpret_cast<uint4*>(qrow + col0) = make_uint4(q[0], q[1], q[2], q[3]);
                        *reinterpret_cast<uint4*>(qrow + col0 + 16) = make_uint4(q[4], q[5], q[6], q[7]);
                        srow[col0 / 32] = static_cast<uint8_t>(scale);
                    }
                }
                if (++acc == kMxAccs) {
                    acc = 0;
                    acc_phase ^= 1;
                }
                continue;
            }
            // ---- the other epilogues: this warp's 64 columns come out of TMEM at once, then the hand-back
            const uint32_t taddr = tmem_base + acc * kMxBlockN + part * 64 + ((quad * 32u) << 16);
            uint32_t r[2][32];
            tmem_ld_32x32b_x32(taddr, r[0]);
            tmem_ld_32x32b_x32(taddr + 32, r[1]);
            tmem_ld_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_tmem_empty + acc * 8);
            }
            if (++acc == kMxAccs) {
                acc = 0;
                acc_phase ^= 1;
            }
            const uint32_t col_base = nt * kMxBlockN + part * 64;
            if (col_base >= p.n) {
                continue;
            }
            if constexpr (kEpi == kMxEpiRouting) {
                mx_route_row(p, r, lane, col_base, group, route_target, route_weight);
                continue;
            }
            if (!row_ok) {
                continue;
            }
            if (p.out_f32) {
                // fp32 output (what the reference's MX kernels write): the accumulator goes out as it is
                float* frow = static_cast<float*>(p.d) + static_cast<size_t>(row) * p.n;
                if ((p.n & 3u) == 0 && col_base + 64 <= p.n) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            *reinterpret_cast<uint4*>(frow + col_base + c * 32 + v * 4) =
                                make_uint4(r[c][4 * v], r[c][4 * v + 1], r[c][4 * v + 2], r[c][4 * v + 3]);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col_base + c * 32 + j < p.n) {
                                frow[col_base + c * 32 + j] = __uint_as_float(r[c][j]);
                            }
                        }
                    }
                }
                continue;
            }
            __nv_bfloat16* drow = static_cast<__nv_bfloat16*>(p.d) + static_cast<size_t>(row) * p.n;
            uint32_t packed[32];  // bf16 pairs: columns 2i, 2i+1 of this warp's 64
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const __nv_bfloat162 h =
                        __floats2bfloat162_rn(__uint_as_float(r[c][2 * e]), __uint_as_float(r[c][2 * e + 1]));
                    packed[c * 16 + e] = *reinterpret_cast<const uint32_t*>(&h);
                }
            }
            if (vec_ok && col_base + 64 <= p.n) {
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    *reinterpret_cast<uint4*>(drow + col_base + v * 8) =
                        make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&packed[i]);
                    if (col_base + 2 * i < p.n) {
                        drow[col_base + 2 * i] = h.x;
                    }
                    if (col_base + 2 * i + 1 < p.n) {
                        drow[col_base + 2 * i + 1] = h.y;
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

}  // namespace cb200
