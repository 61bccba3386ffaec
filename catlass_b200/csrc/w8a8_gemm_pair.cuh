// W8A8 GEMM (dense and grouped) on CTA pairs: the tcgen05.mma.cta_group::2 variant of w8a8_gemm_kernel.
//
// Two CTAs of a cluster (two neighbouring SMs) compute one 256 x 256 tile.  CTA r of the pair owns rows
// [r*128, r*128+128) of the tile (its A tile and its 128 x 256 int32 accumulators in its own TMEM) and loads
// only ONE HALF of the B tile (columns [r*128, r*128+128)); the pair's tensor cores read both halves.  Per
// 128-byte K step a CTA therefore fills 32 KB of shared memory instead of 48 KB and reads 8 KB instead of
// 12 KB per MMA: a third less L2->SM traffic, shared-memory bandwidth and power for the same math, and six
// ring stages instead of four in the same 192 KB.  No multicast load is involved: each CTA fetches its own
// operands with plain TMA loads whose completion bytes are counted on the leader CTA's barrier.
//
// Roles per CTA (6 warps) are those of w8a8_gemm_kernel; only the leader CTA (cluster rank 0) issues MMAs.
//   full[s]        lives in the leader: 1 arrival (its producer's expect_tx for both CTAs' bytes)
//   empty[s]       one per CTA: the MMA commit is multicast to both
//   tmem_full[a]   one per CTA: commit multicast to both, each CTA's epilogue waits on its own
//   tmem_empty[a]  lives in the leader: 8 arrivals (4 epilogue warps x 2 CTAs, the peer's arrive remotely)
#pragma once

#include <cuda_bf16.h>

#include "ptx.cuh"
#include "w8a8_gemm.cuh"

namespace cb200 {

constexpr int kPairTileM = 256;  // rows of the pair's tile
constexpr int kPairBN = 256;     // columns of the pair's tile

struct W8A8PairSmem {
    static constexpr int kStageABytes = kBlockM * kBlockKBytes;         // 16 KB: this CTA's 128 rows
    static constexpr int kStageBBytes = (kPairBN / 2) * kBlockKBytes;   // 16 KB: this CTA's half of B
    static constexpr int kStageBytes = kStageABytes + kStageBBytes;
    static constexpr int kStages = 6;
    static constexpr int kRingBytes = kStages * kStageBytes;
    // output staging: per epilogue warp two slabs of 32 rows x 32 bf16 (64 B rows, 64-byte swizzle) for TMA stores
    static constexpr int kStoreSlabBytes = 32 * 64;
    static constexpr int kStoreBytes = 4 * 2 * kStoreSlabBytes;
    static constexpr int kScaleBytes = 4 * kPairBN * 4;
    static constexpr int kTableEntries = kMaxGroups + 2;
    static constexpr int kTableBytes = 3 * kTableEntries * 4;
    static constexpr int kBarrierBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kTotalBytes = 1024 + kRingBytes + kStoreBytes + kScaleBytes + kTableBytes + kBarrierBytes;
};

// address of `local` (a shared::cta address of this CTA) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}

// kAMn: A is column-major ([k][m], m contiguous; dense problems only): its tiles are loaded as MN-major
// operand panels, 128 rows of K x 128 bytes of M, exactly as a row-major B is.
// kSliceK: grouped slice-K (the reference's GroupedMatmulSliceKPerTokenDequant,
// include/catlass/gemm/kernel/grouped_matmul_slice_k_per_token_dequant.hpp:125-134, example 11): the groups cut K, not
// M; group g multiplies A[:, K_g] with B[K_g, :] into its own m x n output block (row g*m + i of D) with its own scale
// and per-token vectors.  A is column-major and B row-major there, so both operands are MN-major tiles whose rows run
// along K: a group's K range starts at any row.  An ingestion pre-pass has padded every group to whole 128-row K blocks
// (zeros); p.group_list then points to its table of (first K block, number of K blocks) per group.
template <BLayout kB, bool kAMn, bool kSliceK = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
w8a8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_d, const W8A8Params p)
{
    using S = W8A8PairSmem;
    constexpr int kStages = S::kStages;
    constexpr int BN = kPairBN;
    constexpr uint32_t kTmemCols = 2 * BN;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t ring = raw_addr + pad;

    uint8_t* s_store = smem + S::kRingBytes;
    float* s_scale = reinterpret_cast<float*>(smem + S::kRingBytes + S::kStoreBytes);
    int32_t* s_row_begin = reinterpret_cast<int32_t*>(smem + S::kRingBytes + S::kStoreBytes + S::kScaleBytes);
    int32_t* s_row_end = s_row_begin + S::kTableEntries;
    uint32_t* s_tile_begin = reinterpret_cast<uint32_t*>(s_row_end + S::kTableEntries);
    uint64_t* s_bars =
        reinterpret_cast<uint64_t*>(smem + S::kRingBytes + S::kStoreBytes + S::kScaleBytes + S::kTableBytes);
    const uint32_t bar_full = smem_u32(s_bars);
    const uint32_t bar_empty = bar_full + kStages * 8;
    const uint32_t bar_tmem_full = bar_empty + kStages * 8;
    const uint32_t bar_tmem_empty = bar_tmem_full + 2 * 8;
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + 2 * kStages + 4);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();  // 0 = leader: issues the MMAs, hosts full / tmem_empty
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;
    const uint32_t n_tiles = (p.n + BN - 1) / BN;
    const uint32_t groups = p.group_count == 0 ? 1u : p.group_count;

    // ------------------------------------------------------------------ set-up (as in w8a8_gemm_kernel)
    if constexpr (kSliceK) {
        // per group: first K block and number of K blocks of its padded K range
        for (uint32_t g = threadIdx.x; g < groups; g += blockDim.x) {
            const int2 e = static_cast<const int2*>(p.group_list)[g];
            s_row_begin[g] = e.x;
            s_row_end[g] = e.y;
        }
    } else if (p.group_count == 0) {
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
            mbar_init(bar_tmem_empty + a * 8, 2 * (kEpilogueThreads / 32));
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    __syncthreads();
    // slice-K: every group has the same m x n grid of tiles
    const uint32_t tiles_per_group = ((p.m + kPairTileM - 1) / kPairTileM) * n_tiles;
    if (threadIdx.x == 0) {
        if constexpr (kSliceK) {
            s_tile_begin[groups] = groups * tiles_per_group;
        } else {
            int32_t prev = 0;
            uint32_t tiles = 0;
            for (uint32_t g = 0; g < groups; ++g) {
                const int32_t e = s_row_end[g];
                s_row_begin[g] = prev;
                s_tile_begin[g] = tiles;
                if (e > prev) {
                    tiles += static_cast<uint32_t>((e - prev + kPairTileM - 1) / kPairTileM) * n_tiles;
                }
                prev = e;
            }
            s_tile_begin[groups] = tiles;
        }
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
    const uint32_t total_tiles = s_tile_begin[groups];
    const uint32_t num_kb = p.num_k_blocks;
    // tile idx -> rows, columns, group; K blocks [kb0, kb0 + nkb) of the tile
    auto get_tile = [&](TileScheduler& sched, uint32_t idx, TileScheduler::Tile& t, uint32_t& kb0, uint32_t& nkb) {
        if constexpr (kSliceK) {
            t.group = idx / tiles_per_group;
            const uint32_t local = idx - t.group * tiles_per_group;
            const uint32_t mt = local / n_tiles;
            t.row0 = static_cast<int32_t>(mt) * kPairTileM;
            t.row_end = static_cast<int32_t>(p.m);
            t.n0 = static_cast<int32_t>(local - mt * n_tiles) * BN;
            kb0 = static_cast<uint32_t>(s_row_begin[t.group]);
            nkb = static_cast<uint32_t>(s_row_end[t.group]);
        } else {
            sched.get<BN, kPairTileM>(idx, t);
            kb0 = 0;
            nkb = num_kb;
        }
    };

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            TileScheduler sched{s_row_begin, s_row_end, s_tile_begin, n_tiles, 0};
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
                TileScheduler::Tile t;
                uint32_t kb0, nkb;
                get_tile(sched, idx, t, kb0, nkb);
                const int32_t bz = (kSliceK || p.group_count == 0) ? 0 : static_cast<int32_t>(t.group);
                const int32_t row0 = t.row0 + static_cast<int32_t>(cta_rank) * kBlockM;
                const int32_t ncol0 = t.n0 + static_cast<int32_t>(cta_rank) * (BN / 2);
                for (uint32_t kb = kb0; kb < kb0 + nkb; ++kb) {
                    ok = mbar_wait(bar_empty + stage * 8, phase ^ 1, s_abort, p.status, kDevTimeoutProducer);
                    if (!ok) {
                        break;
                    }
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kStageABytes;
                    const int32_t k0 = static_cast<int32_t>(kb) * kBlockKBytes;
                    if (cta_rank == 0) {
                        mbar_expect_tx(bar_full + stage * 8, 2 * S::kStageBytes);  // both CTAs' operands
                    }
                    const uint32_t full = map_to_cta(bar_full + stage * 8, 0);    // the leader's barrier
                    if constexpr (kAMn) {
                        tma_load_2d_pair(sa, &tmap_a, full, row0, k0);  // 128 rows of K x 128 bytes of M
                    } else {
                        tma_load_2d_pair(sa, &tmap_a, full, k0, row0);  // 128 rows of M x 128 bytes of K
                    }
                    if constexpr (kB == BLayout::kRowMajor) {
                        tma_load_3d_pair(sb, &tmap_b, full, ncol0, k0, bz);  // 128 rows of K x 128 bytes of N
                    } else if constexpr (kB == BLayout::kZN) {
                        // four 32-byte-wide panels of 128 K rows each: coordinates (byte in panel, k, panel, group)
                        tma_load_4d_pair(sb, &tmap_b, full, 0, k0, ncol0 / 32, bz);
                    } else {
                        tma_load_3d_pair(sb, &tmap_b, full, k0, ncol0, bz);  // 128 rows of N x 128 bytes of K
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
        // ---------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc =
                make_idesc(kAccS32, kFmtS8, kFmtS8, kAMn, kB != BLayout::kColumnMajor, kPairTileM, BN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
                uint32_t nkb = num_kb;
                if constexpr (kSliceK) {
                    nkb = static_cast<uint32_t>(s_row_end[idx / tiles_per_group]);  // none for an empty group
                }
                ok = mbar_wait(bar_tmem_empty + acc * 8, acc_phase ^ 1, s_abort, p.status, kDevTimeoutMmaTmem);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    ok = mbar_wait(bar_full + stage * 8, phase, s_abort, p.status, kDevTimeoutMma);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sa = ring + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kStageABytes;
#pragma unroll
                    for (int j = 0; j < kBlockKBytes / kUmmaK; ++j) {
                        // the descriptors name this CTA's tiles; the peer's tiles sit at the same offsets
                        uint64_t da, db;
                        if constexpr (kAMn) {
                            // one 128-byte panel of M per CTA; 32 rows of K further down per MMA
                            da = make_smem_desc_sw128(sa + j * (kUmmaK * 128), kBlockKBytes * 128, 1024);
                        } else {
                            da = make_smem_desc_sw128(sa + j * kUmmaK, 16, 1024);
                        }
                        if constexpr (kB == BLayout::kRowMajor) {
                            db = make_smem_desc_sw128(sb + j * (kUmmaK * 128), kBlockKBytes * 128, 1024);
                        } else if constexpr (kB == BLayout::kZN) {
                            // panels of 128 rows x 32 bytes (4 KB apart), 8-row groups 256 bytes apart;
                            // 32 rows of K further down per MMA
                            db = make_smem_desc_sw32(sb + j * (kUmmaK * 32), kBlockKBytes * 32, 256);
                        } else {
                            db = make_smem_desc_sw128(sb + j * kUmmaK, 16, 1024);
                        }
                        umma_i8<2>(tmem_d, da, db, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(bar_empty + stage * 8, 0x3);  // frees the stage in both CTAs
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) {
                    break;
                }
                umma_commit_pair(bar_tmem_full + acc * 8, 0x3);  // both CTAs' halves of the accumulator are done
                acc ^= 1;
                if (acc == 0) {
                    acc_phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue warps 2..5 (both CTAs)
        const uint32_t quad = warp & 3;
        const bool vec_ok = (p.n & 7u) == 0;
        const bool f16 = p.out_f16 != 0;
        TileScheduler sched{s_row_begin, s_row_end, s_tile_begin, n_tiles, 0};
        uint32_t acc = 0, acc_phase = 0;
        uint32_t slab_stores = 0;  // TMA stores this warp has issued: picks the staging slab, across tiles too
        bool ok = true;
        for (uint32_t idx = pair; ok && idx < total_tiles; idx += num_pairs) {
            TileScheduler::Tile t;
            uint32_t kb0_unused, nkb;
            get_tile(sched, idx, t, kb0_unused, nkb);
            // slice-K: group g writes rows [g*m, g*m + m) of D and reads that range of the per-token scales
            const int32_t out_row_offset = kSliceK ? static_cast<int32_t>(t.group * p.m) : 0;
            const bool no_k = kSliceK && nkb == 0;  // an empty group: the accumulator was not written, the sums are 0
            float* sc = s_scale + (warp - 2) * BN;
            __syncwarp();
            stage_tile_scales(sc, p, t.group, static_cast<uint32_t>(t.n0), BN, lane);
            __syncwarp();

            ok = mbar_wait(bar_tmem_full + acc * 8, acc_phase, s_abort, p.status, kDevTimeoutEpilogue);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            tcgen05_fence_after();

            const int32_t row = t.row0 + static_cast<int32_t>(cta_rank * kBlockM + quad * 32 + lane);
            const bool row_ok = row < t.row_end;
            const int32_t out_row = row + out_row_offset;
            const float pt = !row_ok ? 0.0f : (p.per_token ? load_scale(p.per_token, out_row, p.scale_type) : 1.0f);
            const uint32_t taddr = tmem_base + acc * BN + ((quad * 32u) << 16);
            uint16_t* drow = p.d + static_cast<size_t>(row_ok ? out_row : 0) * p.n;
            int32_t* arow = p.acc ? p.acc + static_cast<size_t>(row_ok ? out_row : 0) * p.n : nullptr;
            // a whole warp without valid rows (ragged tail of a group) skips the drain
            const int32_t warp_row0 = t.row0 + static_cast<int32_t>(cta_rank * kBlockM + quad * 32);
            const bool warp_rows = warp_row0 < t.row_end;
            // A warp whose 32 rows all belong to the group stages 32 x 32 outputs in shared memory and hands
            // them to a TMA store (columns past N are clipped by the tensor map); a ragged warp must not write
            // the rows below the group's end, which belong to the next group, and stores row by row.
            const bool slab_store = p.tma_store != 0 && warp_row0 + 32 <= t.row_end;

#pragma unroll 1
            for (int c = 0; c < BN / 32 && warp_rows; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + c * 32, r);
                tmem_ld_wait();
                if constexpr (kSliceK) {
                    if (no_k) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            r[j] = 0;
                        }
                    }
                }
                const uint32_t col0 = t.n0 + c * 32;
                if (slab_store && col0 < p.n) {
                    const float* scc = sc + c * 32;
                    // the two slabs strictly alternate over the warp's stores (a tile may issue an odd number), so
                    // "at most one store still reading" means the store that last read THIS slab has finished
                    uint8_t* slab = s_store + ((warp - 2) * 2 + (slab_stores & 1)) * S::kStoreSlabBytes;
                    ++slab_stores;
                    if (lane == 0) {
                        tma_store_wait_read<1>();
                    }
                    __syncwarp();
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint32_t packed[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = v * 8 + e * 2;
                            packed[e] = pack_out2(dequant(r[j], scc[j], pt), dequant(r[j + 1], scc[j + 1], pt), f16);
                        }
                        // row = lane, 16-byte chunk v at v ^ ((row >> 1) & 3): the 64-byte swizzle of the map
                        *reinterpret_cast<uint4*>(slab + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) =
                            make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                    fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA engine
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmap_d, smem_u32(slab), static_cast<int32_t>(col0 * 2), warp_row0 + out_row_offset);
                        tma_store_commit();
                    }
                    if (arow != nullptr) {
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < p.n) {
                                arow[col0 + j] = static_cast<int32_t>(r[j]);
                            }
                        }
                    }
                } else if (row_ok && col0 < p.n) {
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
            // drained: tell the leader's MMA issuer (remote arrive from the peer CTA)
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(bar_tmem_empty + acc * 8, 0);
            }
            acc ^= 1;
            if (acc == 0) {
                acc_phase ^= 1;
            }
        }
        if (lane == 0) {
            tma_store_wait_all<0>();  // this thread's TMA stores have been written
        }
        __syncwarp();
    }

    // ------------------------------------------------------------------ common exit
    // Every thread of both CTAs gets here (all waits are bounded).  The cluster barrier keeps either CTA's
    // shared memory and barriers alive until its peer has stopped signalling them.
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

}  // namespace cb200
