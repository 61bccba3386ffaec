// MXFP8 / MXFP4 block-scaled GEMM on CTA pairs (tcgen05.mma.cta_group::2): pair tile 256 x 256; dense problems,
// grouped slice-M problems (a pair's tile is 256 rows of one group) and the SwiGLU + MX quantisation epilogue.
//
// Same arithmetic, operand formats, scale re-tiling and TMEM scale layout as mx_gemm_kernel (mx_gemm.cuh), with the
// pairing of w8a8_pair_kernel: CTA r of a cluster of two owns rows [128 r, 128 r + 128) of the tile (its A tile,
// its 128 x 256 accumulator in its own TMEM) and loads only half of the tile's 256 columns of B.  The single-CTA
// kernel is bound by shared-memory bandwidth (per stage 52 KB written by TMA and 48 KB read back by the MMAs for
// 8.4 MFLOP); the pair reads the same A share but half the B share per CTA.
//
// Per CTA and stage: A 16 KB, B half 16 KB, scale blocks (own rows of A: kWords x 512 B; both 128-column blocks
// of B: 2 x kWords x 512 B; each CTA needs the B scales of all 256 columns, because its tensor core computes all
// 256 columns for its rows).  The scales travel WITH the operands: they are fetched by tensor-map loads from the
// packed scale arrays (a 512-byte block is two 256-byte rows of a byte tensor), which like the operand loads count
// their bytes on the LEADER's "full" barrier (cp.async.bulk.tensor.cta_group::2), so one barrier per stage says
// "both CTAs hold operands and scales".  A first version moved the scales through a ring and barriers of their
// own (plain bulk copies can only signal a barrier of the CTA they land in, so the peer's arrival had to be
// forwarded) with one thread requesting, forwarding and copying: that thread's ~10 instructions per stage set
// the pace at 0.9-1.5 PFLOP/s.  Now every single-thread role issues at most five instructions per stage:
//   warp 0   operand producer (both CTAs): wait empty, expect (leader), A, B half
//   warp 2   scale producer (both CTAs): wait empty, A scales, the two B scale blocks
//   warps 3, 4  scale copiers (leader): wait full, smem -> TMEM copies for the pair (tcgen05.cp.cta_group::2: each
//            CTA copies from its own shared memory into its own TMEM), commit to "sf_full" (two arrivals)
//   warp 1   MMA issuer (leader): wait sf_full, four MMAs, one multicast commit that frees the stage in both CTAs
//   warps 5-20  epilogue (both CTAs): sixteen warps, four per TMEM lane quarter with 64 columns each.  There is one
//            accumulator (256 columns + the scale slots fill TMEM), so between two tiles the tensor core waits for
//            the epilogue to pull the accumulator out: ~2.5 us with eight warps reading four 32-column pieces one
//            after the other, against 8.8 us (fp4) or 17.7 us (fp8) of MMAs per tile.  A warp here issues its two
//            reads together, waits once and hands its share back before it rounds or stores anything.
#pragma once

#include "mx_gemm.cuh"
#include "w8a8_gemm_pair.cuh"

namespace cb200 {

constexpr int kMxPairStages = 6;
constexpr int kMxPairThreads = 672;  // 21 warps, see above
constexpr int kMxPairEpiWarps = 16;  // per CTA: four per TMEM lane quarter, 64 columns each

struct MxPairSmem {
    static constexpr int kABytes = kBlockM * kBlockKBytes;          // 16 KB: this CTA's 128 rows of A
    static constexpr int kBBytes = (kMxBlockN / 2) * kBlockKBytes;  // 16 KB: this CTA's half of B
    static constexpr int kSfBytes = 3072;  // A scales at +0 (<= 1 KB), the two B blocks at +1024 (<= 2 KB)
    static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;  // 35 KB
    static constexpr int kRingBytes = kMxPairStages * kStageBytes;
    // full, empty, sf_full [stages]; tmem_full, tmem_empty
    static constexpr int kBarriers = 3 * kMxPairStages + 2;
    static constexpr int kBarrierBytes = kBarriers * 8 + 16;
    static constexpr int kTotalBytes = 1024 + kRingBytes + kBarrierBytes;
};
static_assert(MxPairSmem::kTotalBytes <= 227 * 1024, "shared memory budget");
static_assert(MxPairSmem::kStageBytes % 1024 == 0, "swizzled tiles start on 1 KB boundaries");

template <bool kFp4>
__device__ __forceinline__ void umma_mx_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate, uint32_t sfa, uint32_t sfb)
{
    if constexpr (kFp4) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
            : "memory");
    }
}

__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// tmap_b: {row bytes, n, weight matrices} with boxes of 128 rows; tmap_sfa: the packed A scales as a byte tensor
// {256, 2 * kq_total * row blocks}; tmap_sfb: the packed B scales as {256, 2 * kq_total, column blocks} with boxes of
// one block (see the host side).
// kGrouped: row tiles (256 rows of one group) come from the table of mx_group_plan_kernel; the packed A scales hold
// two 128-row blocks per table tile.  kEpi: kMxEpiPlain or kMxEpiSwiglu (see mx_gemm.cuh; the pair's leader then loads
// the tile's 128 "act" columns of B and its peer the 128 "gate" columns).
template <bool kFp4, bool kGrouped = false, int kEpi = kMxEpiPlain>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMxPairThreads, 1)
mx_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
               const MxParams p)
{
    using S = MxPairSmem;
    constexpr int kStages = kMxPairStages;
    constexpr uint32_t kAccCols = kMxBlockN;           // one fp32 accumulator: 128 lanes x 256 columns per CTA
    constexpr uint32_t kSfSlot = 24;                   // one scale slot: A up to 8 columns, B up to 16
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kWords = kFp4 ? 2 : 1;
    constexpr uint32_t kSfTx = 3 * kWords * 512;       // scale bytes per CTA and stage
    static_assert(kAccCols + kStages * kSfSlot <= kTmemCols, "TMEM budget");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t ring = raw_addr + pad;
    uint64_t* s_bars = reinterpret_cast<uint64_t*>(smem + S::kRingBytes);
    const uint32_t bar_full = smem_u32(s_bars);               // leader: operands and scales of both CTAs landed
    const uint32_t bar_empty = bar_full + kStages * 8;        // both: the stage's MMAs completed
    const uint32_t bar_sf_full = bar_empty + kStages * 8;     // leader: scales copied into both TMEMs
    const uint32_t bar_tmem_full = bar_sf_full + kStages * 8; // both: accumulator complete
    const uint32_t bar_tmem_empty = bar_tmem_full + 8;        // leader: accumulator read by both epilogues
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + S::kBarriers);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;
    constexpr bool kSwiglu = kEpi == kMxEpiSwiglu;
    static_assert(kEpi == kMxEpiPlain || (kSwiglu && kGrouped && !kFp4), "epilogues of the pair kernel");
    const uint32_t m_tiles = kGrouped ? *p.num_row_tiles : (p.m + 2 * kBlockM - 1) / (2 * kBlockM);
    const uint32_t n_tiles = kSwiglu ? (p.n / 2 + 127) / 128 : (p.n + kMxBlockN - 1) / kMxBlockN;
    const uint32_t total_tiles = m_tiles * n_tiles;
    const uint32_t num_kb = p.num_k_blocks;
    // first row of the pair's tile, end of the rows that may be stored, group
    auto row_tile = [&](uint32_t mt, int32_t& row0, int32_t& row_end, int32_t& group) {
        if constexpr (kGrouped) {
            const int4 e = __ldg(p.tile_table + mt);
            row0 = e.x;
            row_end = e.y;
            group = e.z;
        } else {
            row0 = static_cast<int32_t>(mt) * 2 * kBlockM;
            row_end = static_cast<int32_t>(p.m);
            group = 0;
        }
    };

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
            mbar_init(bar_sf_full + s * 8, 2);  // one arrival per copier thread
        }
        mbar_init(bar_tmem_full, 1);
        mbar_init(bar_tmem_empty, 2 * kMxPairEpiWarps);  // the epilogue warps of both CTAs
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        prefetch_tmap(&tmap_sfa);
        prefetch_tmap(&tmap_sfb);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(s_tmem_ptr), kTmemCols);
        tmem_relinquish<2>();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers are initialised and their TMEM allocated before any cross-CTA signal
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem_ptr;

    if (warp == 0) {
        // ---------------------------------------------------------------- operand producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
                uint32_t mt, nt;
                mx_tile_coords(idx, m_tiles, n_tiles, p.band_rows, mt, nt);
                int32_t tile_row0, row_end, group;
                row_tile(mt, tile_row0, row_end, group);
                const int32_t row0 = tile_row0 + static_cast<int32_t>(cta_rank * kBlockM);
                const int32_t col0 = kSwiglu ? static_cast<int32_t>(cta_rank == 0 ? nt * 128 : p.n / 2 + nt * 128)
                                             : static_cast<int32_t>(nt * kMxBlockN + cta_rank * (kMxBlockN / 2));
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar_empty + stage * 8, phase ^ 1, s_abort, p.status, kDevTimeoutProducer);
                    if (!ok) {
                        break;
                    }
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    const int32_t k0 = static_cast<int32_t>(kb) * kBlockKBytes;
                    if (cta_rank == 0) {  // both CTAs' tiles and scale blocks
                        mbar_expect_tx(bar_full + stage * 8, 2 * (S::kABytes + S::kBBytes + kSfTx));
                    }
                    const uint32_t full = map_to_cta(bar_full + stage * 8, 0);  // the leader's barrier
                    tma_load_2d_pair(sa, &tmap_a, full, k0, row0);
                    tma_load_3d_pair(sb, &tmap_b, full, k0, col0, group);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ---------------------------------------------------------------- scale producer (both CTAs)
        // (waits on the same "empty" barrier as the operand producer; the bytes are expected by the leader's
        // operand producer, in whatever order the loads and the expectation reach the barrier)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
                uint32_t mt, nt;
                mx_tile_coords(idx, m_tiles, n_tiles, p.band_rows, mt, nt);
                // rows of the scale tensors: 256 bytes each, two per 512-byte block; this CTA's 128-row block of A
                // (past the end of A the box reads zeros: those rows are never stored) and the tile's two blocks of B
                const int32_t a_row0 = static_cast<int32_t>((2 * mt + cta_rank) * p.kq_total * 2);
                int32_t tile_row0, row_end, group;
                row_tile(mt, tile_row0, row_end, group);
                const int32_t sfb_first = group * static_cast<int32_t>(p.sfb_blocks_per_group);
                const int32_t sfb0 = sfb_first + static_cast<int32_t>(kSwiglu ? nt : 2 * nt);
                const int32_t sfb1 = sfb_first + static_cast<int32_t>(kSwiglu ? p.n / 256 + nt : 2 * nt + 1);
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar_empty + stage * 8, phase ^ 1, s_abort, p.status, kDevTimeoutProducer);
                    if (!ok) {
                        break;
                    }
                    const uint32_t ssf = ring + stage * S::kStageBytes + S::kABytes + S::kBBytes;
                    const uint32_t full = map_to_cta(bar_full + stage * 8, 0);
                    const int32_t kq2 = static_cast<int32_t>(kb * kWords * 2);
                    tma_load_2d_pair(ssf, &tmap_sfa, full, 0, a_row0 + kq2);
                    tma_load_3d_pair(ssf + 1024, &tmap_sfb, full, 0, kq2, sfb0);
                    tma_load_3d_pair(ssf + 1024 + kWords * 512, &tmap_sfb, full, 0, kq2, sfb1);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t fmt = kFp4 ? kFmtMxf4E2M1 : kFmtE4M3;
            uint32_t stage = 0, phase = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
                ok = mbar_wait(bar_tmem_empty, acc_phase ^ 1, s_abort, p.status, kDevTimeoutMmaTmem);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    // (the copiers waited for "full" before they copied: see mx_gemm_kernel)
                    ok = mbar_wait(bar_sf_full + stage * 8, phase, s_abort, p.status, kDevTimeoutMma);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    const uint32_t t_sfa = tmem_base + kAccCols + stage * kSfSlot;
                    const uint32_t t_sfb = t_sfa + 8;
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        // the descriptors name this CTA's tiles; the peer's tiles sit at the same offsets
                        const uint64_t da = make_smem_desc_sw128(sa + j * 32, 16, 1024);
                        const uint64_t db = make_smem_desc_sw128(sb + j * 32, 16, 1024);
                        const uint32_t word = kFp4 ? (j >> 1) : 0;
                        const uint32_t sf_id = kFp4 ? ((j & 1) * 2) : j;
                        const uint32_t idesc = make_idesc_mx(fmt, fmt, 2 * kBlockM, kMxBlockN, sf_id, sf_id);
                        umma_mx_pair<kFp4>(tmem_base, da, db, idesc, (kb | j) != 0 ? 1u : 0u, t_sfa + word * 4,
                                           t_sfb + word * 8);
                    }
                    umma_commit_pair(bar_empty + stage * 8, 0x3);  // frees the stage (and its TMEM scale slot) in both CTAs
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) {
                    break;
                }
                umma_commit_pair(bar_tmem_full, 0x3);  // both CTAs' halves of the accumulator are complete
                acc_phase ^= 1;
            }
        }
        __syncwarp();
    } else if (warp == 3 || warp == 4) {
        // ---------------------------------------------------------------- scale copiers (leader CTA only)
        // TMEM slot `stage` is free when the stage's "full" barrier fires: the MMAs that read its previous contents
        // completed before the producers were allowed to refill the stage.
        // fp8 (three copies per stage): warp 3 copies A's block and B's first, warp 4 B's second;
        // fp4 (six): warp 3 takes scale word 0 of all three blocks, warp 4 word 1.
        const uint32_t me = warp == 3 ? 0u : 1u;
        if (lane == 0 && cta_rank == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar_full + stage * 8, phase, s_abort, p.status, kDevTimeoutConvert);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t ssf = ring + stage * S::kStageBytes + S::kABytes + S::kBBytes;
                    const uint32_t t_sfa = tmem_base + kAccCols + stage * kSfSlot;
                    const uint32_t t_sfb = t_sfa + 8;
                    auto copy_a = [&](uint32_t w) {
                        tmem_cp_32x128b_warpx4_pair(t_sfa + w * 4, make_smem_desc_noswizzle(ssf + w * 512, 16, 128));
                    };
                    auto copy_b = [&](uint32_t w, uint32_t nb) {
                        tmem_cp_32x128b_warpx4_pair(t_sfb + w * 8 + nb * 4,
                                                    make_smem_desc_noswizzle(ssf + 1024 + (nb * kWords + w) * 512, 16, 128));
                    };
                    if constexpr (kFp4) {
                        copy_a(me);
                        copy_b(me, 0);
                        copy_b(me, 1);
                    } else {
                        if (me == 0) {
                            copy_a(0);
                            copy_b(0, 0);
                        } else {
                            copy_b(0, 1);
                        }
                    }
                    umma_commit<2>(bar_sf_full + stage * 8);  // arrives when this thread's copies have completed
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue: sixteen warps per CTA
        const uint32_t quad = warp & 3;           // TMEM lane quarter this warp may read
        const uint32_t part = (warp - 5) >> 2;    // which 64 columns of the tile's 256
        const bool vec_ok = (p.n & 7u) == 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
            uint32_t mt, nt;
            mx_tile_coords(idx, m_tiles, n_tiles, p.band_rows, mt, nt);
            ok = mbar_wait(bar_tmem_full, acc_phase, s_abort, p.status, kDevTimeoutEpilogue);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            tcgen05_fence_after();
            int32_t tile_row0, row_end, group;
            row_tile(mt, tile_row0, row_end, group);
            const uint32_t row = static_cast<uint32_t>(tile_row0) + cta_rank * kBlockM + quad * 32 + lane;
            const bool row_ok = static_cast<int32_t>(row) < row_end;
            if constexpr (kSwiglu) {
                // This warp: output columns [32 * part, 32 * part + 32) of the tile's 128; "act" sits in accumulator
                // columns 0..127, "gate" in 128..255.  Both pieces leave TMEM, the share goes back, then the arithmetic.
                const uint32_t tcols = tmem_base + part * 32 + ((quad * 32u) << 16);
                uint32_t ra[32], rg[32];
                tmem_ld_32x32b_x32(tcols, ra);
                tmem_ld_32x32b_x32(tcols + 128, rg);
                tmem_ld_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(bar_tmem_empty, 0);
                }
                acc_phase ^= 1;
                const uint32_t half_n = p.n / 2;
                const uint32_t col0 = nt * 128 + part * 32;
                if (!row_ok || col0 >= half_n) {
                    continue;
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float a = __uint_as_float(ra[i]);
                    const float g = __uint_as_float(rg[i]);
                    const float t = __fadd_rn(expf(-a), 1.0f);
                    const float sw = __fmul_rn(__fdiv_rn(a, t), g);
                    ra[i] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(sw)));
                }
                uint32_t q[8];
                const uint32_t scale = mx_quant_block_bf16_e4m3(ra, q);
                uint8_t* qrow = static_cast<uint8_t*>(p.d) + static_cast<size_t>(row) * half_n;
                *reinterpret_cast<uint4*>(qrow + col0) = make_uint4(q[0], q[1], q[2], q[3]);
                *reinterpret_cast<uint4*>(qrow + col0 + 16) = make_uint4(q[4], q[5], q[6], q[7]);
                p.q_scale[static_cast<size_t>(row) * (half_n / 32) + col0 / 32] = static_cast<uint8_t>(scale);
                continue;
            }
            const uint32_t taddr = tmem_base + part * 64 + ((quad * 32u) << 16);
            uint32_t r[2][32];
            tmem_ld_32x32b_x32(taddr, r[0]);
            tmem_ld_32x32b_x32(taddr + 32, r[1]);
            tmem_ld_wait();
            // this warp's share of the accumulator is in registers: hand it back (remote arrive from the peer CTA)
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(bar_tmem_empty, 0);
            }
            acc_phase ^= 1;
            const uint32_t col_base = nt * kMxBlockN + part * 64;
            if (!row_ok || col_base >= p.n) {
                continue;
            }
            if (p.out_f32) {
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

    // Every thread of both CTAs gets here (all waits are bounded).  The cluster barrier keeps either CTA's shared
    // memory and barriers alive until its peer has stopped signalling them.
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

}  // namespace cb200
