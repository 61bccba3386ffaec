// W8A8 GEMM with fused per-token / per-channel dequant for sm_100a: dense and grouped (slice-M) problems.
//
// One persistent CTA per SM, 6 warps, warp-specialised:
//   warp 0      TMA producer   - one thread streams 128x128-byte A tiles and BNx128-byte B tiles into a
//                                kStages-deep ring of 128B-swizzled shared memory
//   warp 1      MMA issuer     - one thread issues tcgen05.mma.kind::i8 (128 x BN x 32 per instruction) into one
//                                of two int32 accumulators held in TMEM; owns the TMEM allocation
//   warps 2-5   epilogue       - tcgen05.ld the finished accumulator (one row per thread), apply
//                                (float(acc) * scale[n]) * per_token[m] with two separate fp32 multiplies,
//                                round to bf16 (nearest even) and store; runs under the next tile's mainloop
// The roles hand tiles over through mbarriers only; every wait is bounded (ptx.cuh: mbar_wait).
//
// What it computes is what the reference's kernels QuantMatmulMultiStageWorkspace
// (include/catlass/gemm/kernel/quant_matmul_multistage_workspace.hpp:147-268) and
// GroupedMatmulSliceMPerTokenDequant (include/catlass/gemm/kernel/grouped_matmul_slice_m_per_token_dequant.hpp:
// 181-321) compute with BlockMmad + BlockEpilogue<EpilogueAtlasA2PerTokenDequant>
// (include/catlass/epilogue/block/block_epilogue_per_token_dequant.hpp:483-614); the int32 accumulator never
// leaves the SM here, where the reference hands it from cube to vector cores through a global workspace.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace cb200 {

constexpr int kBlockM = 128;        // rows of A per tile = TMEM lanes
constexpr int kBlockKBytes = 128;   // K bytes per pipeline stage = one 128B swizzle row
constexpr int kUmmaK = 32;          // K per tcgen05.mma.kind::i8
constexpr int kMaxGroups = 1024;

// How the weight matrices B[k][n] lie in memory
enum class BLayout : int {
    kColumnMajor = 0,  // [n][k]: K contiguous           -> K-major operand tiles, 128-byte swizzle
    kRowMajor = 1,     // [k][n]: N contiguous           -> MN-major tiles, 128-byte-wide panels
    kZN = 2,           // [n/32][round16(k)][32]: the reference's zN fractal format -> MN-major, 32-byte panels
};
constexpr int kGemmThreads = 192;
constexpr int kEpilogueThreads = 128;

// Element types of the scale vectors (converted to fp32 when loaded, which is what the goldens do with
// static_cast<float>) and of D.
constexpr uint32_t kTypeF32 = 0;
constexpr uint32_t kTypeBf16 = 1;
constexpr uint32_t kTypeF16 = 2;
constexpr uint32_t kTypeF32InU64 = 3;  // fp32 bit pattern in the low half of a 64-bit word (the reference's
                                       // fixpipe scale format, example 48)

struct W8A8Params {
    uint32_t m;                // row capacity of A / D (dense: M)
    uint32_t n;
    uint32_t k;
    uint32_t group_count;      // 0 = dense problem
    uint32_t group_list_is_i32;
    uint32_t num_k_blocks;     // ceil(k / 128)
    const void* group_list;    // device: ascending prefix sums of rows
    const void* scale;         // channel scales, scale_type elements; group g uses scale + g * scale_stride
    const void* per_token;     // [m] scale_type elements, or null: no per-token factor
    uint16_t* d;               // [m][n] bf16 or fp16 bit patterns
    int32_t* acc;              // optional raw accumulators [m][n]
    unsigned* status;          // device status word
    uint32_t tma_store;        // pair kernel: D has a tensor map, full 32-row slabs leave through TMA stores
    uint32_t scale_type;       // kTypeF32 / kTypeBf16 / kTypeF16 / kTypeF32InU64
    uint32_t scale_stride;     // elements between the scale vectors of two groups (0: one vector for all groups)
    uint32_t scalar_mode;      // 1: every channel uses scalar_scale (per-tensor dequant), `scale` is not read
    float scalar_scale;
    uint32_t out_f16;          // D holds fp16 instead of bf16
    uint32_t static_weights;   // weights and channel scales may be read before the stream dependency resolves
};

// One element of a scale vector as fp32.
__device__ __forceinline__ float load_scale(const void* base, size_t i, uint32_t type)
{
    if (type == kTypeF32) {
        return __ldg(static_cast<const float*>(base) + i);
    }
    if (type == kTypeF32InU64) {
        return __ldg(static_cast<const float*>(base) + 2 * i);
    }
    const uint32_t v = __ldg(static_cast<const unsigned short*>(base) + i);
    if (type == kTypeBf16) {
        return __uint_as_float(v << 16);
    }
    return __half2float(__ushort_as_half(static_cast<unsigned short>(v)));
}

// The dequant step of the goldens: (float(acc) * scale) * per_token, two separately rounded fp32 multiplies
// (examples/common/golden/matmul.hpp:320-321); per_token = 1 where the operator has no per-token factor.
__device__ __forceinline__ float dequant(uint32_t acc, float scale, float per_token)
{
    return __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(acc)), scale), per_token);
}

// Two / one fp32 values rounded to nearest even into bf16 or fp16 bit patterns.
__device__ __forceinline__ uint32_t pack_out2(float x0, float x1, bool f16)
{
    if (f16) {
        const __half2 h = __floats2half2_rn(x0, x1);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ uint16_t pack_out1(float x, bool f16)
{
    if (f16) {
        return __half_as_ushort(__float2half_rn(x));
    }
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

// This warp's private copy of a tile's channel scales (columns n0 .. n0 + count), zero past column n.
__device__ __forceinline__ void stage_tile_scales(float* sc, const W8A8Params& p, uint32_t group, uint32_t n0,
                                                  uint32_t count, uint32_t lane)
{
    const size_t base = static_cast<size_t>(p.group_count == 0 ? 0 : group) * p.scale_stride;
    for (uint32_t i = lane; i < count; i += 32) {
        const uint32_t col = n0 + i;
        float v = 0.0f;
        if (col < p.n) {
            v = p.scalar_mode ? p.scalar_scale : load_scale(p.scale, base + col, p.scale_type);
        }
        sc[i] = v;
    }
}

template <int BN>
struct W8A8Smem {
    static constexpr int kStageABytes = kBlockM * kBlockKBytes;
    static constexpr int kStageBBytes = BN * kBlockKBytes;
    static constexpr int kStageBytes = kStageABytes + kStageBBytes;
    static constexpr int kStages = (BN == 256) ? 4 : 6;
    static constexpr int kRingBytes = kStages * kStageBytes;
    static constexpr int kScaleBytes = 4 * BN * 4;  // one private copy of the tile's scales per epilogue warp
    static constexpr int kTableEntries = kMaxGroups + 2;  // even, so the barriers behind the tables stay 8-byte aligned
    static constexpr int kTableBytes = 3 * kTableEntries * 4;
    static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
    // + 1024 so the ring can be aligned to the swizzle atom whatever the dynamic smem base is
    static constexpr int kTotalBytes = 1024 + kRingBytes + kScaleBytes + kTableBytes + kBarrierBytes;
};

// Maps a linear tile index to (group, row range, column offset).  A dense problem is one group.
// Tiles of a group are numbered with the column tile fastest, so the CTAs working at the same time
// share a handful of A row panels and all of the group's B.
struct TileScheduler {
    const int32_t* row_begin;    // [G]   first row of group g
    const int32_t* row_end;      // [G]   one past its last row
    const uint32_t* tile_begin;  // [G+1] first tile index of group g; [G] = number of tiles
    uint32_t n_tiles;
    uint32_t group;

    struct Tile {
        int32_t row0;
        int32_t row_end;
        int32_t n0;
        uint32_t group;
    };

    template <int BN, int TM = 128>
    __device__ __forceinline__ void get(uint32_t idx, Tile& t)
    {
        while (idx >= tile_begin[group + 1]) {
            ++group;
        }
        const uint32_t local = idx - tile_begin[group];
        const uint32_t mt = local / n_tiles;
        const uint32_t nt = local - mt * n_tiles;
        t.row0 = row_begin[group] + static_cast<int32_t>(mt) * TM;
        t.row_end = row_end[group];
        t.n0 = static_cast<int32_t>(nt) * BN;
        t.group = group;
    }
};

template <int BN, bool kBMnMajor>
__global__ void __launch_bounds__(kGemmThreads, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const W8A8Params p)
{
    using S = W8A8Smem<BN>;
    constexpr int kStages = S::kStages;
    constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators of BN int32 columns
    static_assert(kTmemCols == 512 || kTmemCols == 256 || kTmemCols == 128 || kTmemCols == 64, "TMEM columns");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t ring = raw_addr + pad;

    float* s_scale = reinterpret_cast<float*>(smem + S::kRingBytes);
    int32_t* s_row_begin = reinterpret_cast<int32_t*>(smem + S::kRingBytes + S::kScaleBytes);
    int32_t* s_row_end = s_row_begin + S::kTableEntries;
    uint32_t* s_tile_begin = reinterpret_cast<uint32_t*>(s_row_end + S::kTableEntries);
    uint64_t* s_bars = reinterpret_cast<uint64_t*>(smem + S::kRingBytes + S::kScaleBytes + S::kTableBytes);
    // barrier slots: [0,kStages) full, [kStages,2kStages) empty, then tmem_full[2], tmem_empty[2]
    const uint32_t bar_full = smem_u32(s_bars);
    const uint32_t bar_empty = bar_full + kStages * 8;
    const uint32_t bar_tmem_full = bar_empty + kStages * 8;
    const uint32_t bar_tmem_empty = bar_tmem_full + 2 * 8;
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + 2 * kStages + 4);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t n_tiles = (p.n + BN - 1) / BN;
    const uint32_t groups = p.group_count == 0 ? 1u : p.group_count;

    // ------------------------------------------------------------------ set-up
    // 1) group boundaries into smem (clamped to [0, m]); a dense problem is the single group [0, m)
    if (p.group_count == 0) {
        if (threadIdx.x == 0) {
            s_row_end[0] = static_cast<int32_t>(p.m);
        }
    } else {
        for (uint32_t g = threadIdx.x; g < groups; g += blockDim.x) {
            long long e = p.group_list_is_i32 ? static_cast<long long>(static_cast<const int32_t*>(p.group_list)[g])
                                              : static_cast<const long long*>(p.group_list)[g];
            e = e < 0 ? 0 : (e > static_cast<long long>(p.m) ? static_cast<long long>(p.m) : e);
            s_row_end[g] = static_cast<int32_t>(e);
        }
    }
    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tmem_full + a * 8, 1);
            mbar_init(bar_tmem_empty + a * 8, kEpilogueThreads / 32);
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    __syncthreads();
    // 2) per-group first row and first tile index (serial scan, at most kMaxGroups short steps)
    if (threadIdx.x == 0) {
        int32_t prev = 0;
        uint32_t tiles = 0;
        for (uint32_t g = 0; g < groups; ++g) {
            const int32_t e = s_row_end[g];
            s_row_begin[g] = prev;
            s_tile_begin[g] = tiles;
            if (e > prev) {
                tiles += static_cast<uint32_t>((e - prev + kBlockM - 1) / kBlockM) * n_tiles;
            }
            prev = e;  // the golden restarts at the previous entry also when the list is not ascending
        }
        s_tile_begin[groups] = tiles;
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(s_tmem_ptr), kTmemCols);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();

    const uint32_t tmem_base = *s_tmem_ptr;
    const uint32_t total_tiles = s_tile_begin[groups];
    const uint32_t num_kb = p.num_k_blocks;

    // ------------------------------------------------------------------ roles
    if (warp == 0) {
        if (lane == 0) {
            TileScheduler sched{s_row_begin, s_row_end, s_tile_begin, n_tiles, 0};
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t idx = blockIdx.x; ok && idx < total_tiles; idx += gridDim.x) {
                TileScheduler::Tile t;
                sched.get<BN>(idx, t);
                const int32_t bz = (p.group_count == 0) ? 0 : static_cast<int32_t>(t.group);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar_empty + stage * 8, phase ^ 1, s_abort, p.status, kDevTimeoutProducer);
                    if (!ok) {
                        break;
                    }
                    const uint32_t full = bar_full + stage * 8;
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kStageABytes;
                    const int32_t k0 = static_cast<int32_t>(kb) * kBlockKBytes;
                    mbar_expect_tx(full, S::kStageBytes);
                    tma_load_2d(sa, &tmap_a, full, k0, t.row0);
                    if constexpr (kBMnMajor) {
                        // B rows are K, 128 columns of N per panel: BN/128 panels of 128(k) x 128 bytes
#pragma unroll
                        for (int pn = 0; pn < BN / 128; ++pn) {
                            tma_load_3d(sb + pn * (kBlockKBytes * 128), &tmap_b, full, t.n0 + pn * 128, k0, bz);
                        }
                    } else {
                        tma_load_3d(sb, &tmap_b, full, k0, t.n0, bz);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, false, kBMnMajor, kBlockM, BN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t idx = blockIdx.x; ok && idx < total_tiles; idx += gridDim.x) {
                ok = mbar_wait(bar_tmem_empty + acc * 8, acc_phase ^ 1, s_abort, p.status, kDevTimeoutMmaTmem);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar_full + stage * 8, phase, s_abort, p.status, kDevTimeoutMma);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kStageABytes;
#pragma unroll
                    for (int j = 0; j < kBlockKBytes / kUmmaK; ++j) {
                        const uint64_t da = make_smem_desc_sw128(sa + j * kUmmaK, 16, 1024);
                        uint64_t db;
                        if constexpr (kBMnMajor) {
                            // 32 rows of K further down each panel; panels 16 KB apart, 8-row groups 1 KB apart
                            db = make_smem_desc_sw128(sb + j * (kUmmaK * 128), kBlockKBytes * 128, 1024);
                        } else {
                            db = make_smem_desc_sw128(sb + j * kUmmaK, 16, 1024);
                        }
                        umma_i8<1>(tmem_d, da, db, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    umma_commit<1>(bar_empty + stage * 8);  // stage is free once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) {
                    break;
                }
                umma_commit<1>(bar_tmem_full + acc * 8);  // accumulator complete
                acc ^= 1;
                if (acc == 0) {
                    acc_phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue warps 2..5
        const uint32_t quad = warp & 3;             // the 32-lane quarter of TMEM this warp can read
        const bool vec_ok = (p.n & 7u) == 0;
        const bool f16 = p.out_f16 != 0;
        TileScheduler sched{s_row_begin, s_row_end, s_tile_begin, n_tiles, 0};
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t idx = blockIdx.x; ok && idx < total_tiles; idx += gridDim.x) {
            TileScheduler::Tile t;
            sched.get<BN>(idx, t);
            // channel scales of this tile -> this warp's private smem copy (no cross-warp barrier needed)
            float* sc = s_scale + (warp - 2) * BN;
            __syncwarp();
            stage_tile_scales(sc, p, t.group, static_cast<uint32_t>(t.n0), BN, lane);
            __syncwarp();

            ok = mbar_wait(bar_tmem_full + acc * 8, acc_phase, s_abort, p.status, kDevTimeoutEpilogue);
            ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .aligned TMEM loads
            if (!ok) {
                break;
            }
            tcgen05_fence_after();

            const int32_t row = t.row0 + static_cast<int32_t>(quad * 32 + lane);
            const bool row_ok = row < t.row_end;
            const float pt = !row_ok ? 0.0f : (p.per_token ? load_scale(p.per_token, row, p.scale_type) : 1.0f);
            const uint32_t taddr = tmem_base + acc * BN + ((quad * 32u) << 16);
            uint16_t* drow = p.d + static_cast<size_t>(row_ok ? row : 0) * p.n;
            int32_t* arow = p.acc ? p.acc + static_cast<size_t>(row_ok ? row : 0) * p.n : nullptr;

#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + c * 32, r);
                tmem_ld_wait();
                const uint32_t col0 = t.n0 + c * 32;
                if (row_ok && col0 < p.n) {
                    const float* scc = sc + c * 32;
                    if (vec_ok && col0 + 32 <= p.n) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint32_t packed[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int j = v * 8 + e * 2;
                                packed[e] = pack_out2(dequant(r[j], scc[j], pt), dequant(r[j + 1], scc[j + 1], pt), f16);
                            }
                            *reinterpret_cast<uint4*>(drow + col0 + v * 8) =
                                make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        }
                    } else {
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < p.n) {
                                drow[col0 + j] = pack_out1(dequant(r[j], scc[j], pt), f16);
                            }
                        }
                    }
                    if (arow != nullptr) {
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < p.n) {
                                arow[col0 + j] = static_cast<int32_t>(r[j]);
                            }
                        }
                    }
                }
            }
            // accumulator drained: hand it back to the MMA issuer
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_tmem_empty + acc * 8);
            }
            acc ^= 1;
            if (acc == 0) {
                acc_phase ^= 1;
            }
        }
    }

    // ------------------------------------------------------------------ common exit
    // Reached by every thread, also after a timed-out wait.  The wait limit is far beyond the lifetime of
    // any copy or MMA in flight, so the TMEM columns and shared memory are idle here.
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

// D rows [0, rows) := 0 for a problem with k == 0 (the reference epilogue writes zeros then:
// include/catlass/epilogue/block/block_epilogue_per_token_dequant.hpp:500-527).
__global__ void zero_rows_kernel(uint16_t* d, const void* group_list, uint32_t group_list_is_i32,
                                 uint32_t group_count, uint32_t m, uint32_t n)
{
    long long rows = m;
    if (group_count != 0) {
        rows = group_list_is_i32 ? static_cast<long long>(static_cast<const int32_t*>(group_list)[group_count - 1])
                                 : static_cast<const long long*>(group_list)[group_count - 1];
        rows = rows < 0 ? 0 : (rows > static_cast<long long>(m) ? static_cast<long long>(m) : rows);
    }
    const size_t total = static_cast<size_t>(rows) * n;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        d[i] = 0;  // +0.0 in bf16 and in fp16
    }
}

}  // namespace cb200
