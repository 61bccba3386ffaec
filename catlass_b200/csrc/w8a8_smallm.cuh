// W8A8 dequant GEMM for few tokens (M <= 128): the decode-shaped, HBM-bound case.
//
// The problem is transposed onto the tensor core: a tile is 128 WEIGHT rows (output channels n) on the
// UMMA M axis / TMEM lanes and all MT = round_up(M, 16) tokens on the UMMA N axis, so a token panel as small
// as 16 wastes nothing of the 128-lane datapath and every weight byte is read from HBM exactly once.
// K is split over the `splits` CTAs of a thread-block cluster; each streams its slice of the weight panel
// through a deep TMA ring, accumulates int32 in TMEM, and the partial sums are added - still as int32, so
// the result stays bit-exact - in the shared memory of the cluster's first CTA (distributed shared memory,
// no global workspace, no atomics).  That CTA applies (float(acc) * scale[n]) * per_token[m] and writes bf16.
//
// Covers what the reference's decode-oriented variants are for: the A-resident kernel
// (include/catlass/gemm/kernel/quant_matmul_full_loadA_tla.hpp) and multi-core split-K
// (examples/52_quant_multi_core_splitk_matmul_tla), with the reduction kept on chip.
#pragma once

#include <cuda_bf16.h>

#include "ptx.cuh"
#include "w8a8_gemm.cuh"

namespace cb200 {

constexpr int kSmallMThreads = 192;
constexpr int kSmallMTileN = 128;     // weight rows per tile
constexpr int kSmallMMaxStages = 8;
constexpr int kSmallMMaxSplits = 8;   // portable cluster size

struct SmallMParams {
    uint32_t m, n, k;
    uint32_t mt;            // tokens padded to a multiple of 16 (<= 128)
    uint32_t splits;        // cluster size along K (1, 2, 4 or 8)
    uint32_t num_k_blocks;  // ceil(k / 128)
    uint32_t stages;        // ring depth (fits the dynamic smem given at launch)
    uint32_t kbs;           // 128-byte K blocks per ring stage: one stage = kbs*128 contiguous bytes per weight row
    uint32_t tile_rows;     // weight rows a CTA owns (<= 128, multiple of 8): chosen so the tiles fill the SMs
    const void* scale;      // [n] scale_type elements (not read in scalar mode)
    const void* per_token;  // [m] scale_type elements, or null: no per-token factor
    uint16_t* d;            // [m][n] bf16 or fp16 bit patterns
    int32_t* acc;           // optional [m][n]
    unsigned* status;
    uint32_t scale_type;
    uint32_t scalar_mode;
    float scalar_scale;
    uint32_t out_f16;
    uint32_t static_weights;  // weights and channel scales may be read before the stream dependency resolves
    uint32_t own_partials;    // the partial-sum buffer has shared memory of its own (see smallm_smem_bytes)
};

// dynamic smem: [1024 align pad][stages x (16 KB W + mt*128 B X)][(splits-1) x 128 x mt x 4 B partials][barriers]
// The partial sums of the other CTAs of a cluster land in the first CTA.  When they are small (few tokens: 24 KB for
// 16 tokens and a 4-way split) they get memory of their own behind the ring, and a CTA pushes its sums the moment
// its own K slice is done, then arrives on a barrier in the first CTA: no cluster-wide barrier on the critical path.
// Large ones (up to 192 KB) are aliased onto the first CTA's ring and need a cluster barrier before (the ring must be
// idle) and after the pushes.
constexpr uint32_t kSmallMOwnPartialsMax = 32u * 1024u;
__host__ __device__ inline bool smallm_own_partials(uint32_t mt, uint32_t splits)
{
    return splits > 1 && (splits - 1) * kSmallMTileN * mt * 4 <= kSmallMOwnPartialsMax;
}
__host__ __device__ inline uint32_t smallm_block_bytes(uint32_t mt)
{
    return kSmallMTileN * kBlockKBytes + mt * kBlockKBytes;
}
__host__ __device__ inline uint32_t smallm_stage_bytes(uint32_t mt, uint32_t kbs)
{
    return kbs * smallm_block_bytes(mt);
}
__host__ __device__ inline uint32_t smallm_body_bytes(uint32_t mt, uint32_t stages, uint32_t splits, uint32_t kbs,
                                                      bool own_partials)
{
    uint32_t ring = stages * smallm_stage_bytes(mt, kbs);
    uint32_t partials = (splits - 1) * kSmallMTileN * mt * 4;
    if (own_partials) {
        return ring + partials;
    }
    return ring > partials ? ring : partials;
}
__host__ __device__ inline uint32_t smallm_smem_bytes(uint32_t mt, uint32_t stages, uint32_t splits, uint32_t kbs,
                                                      bool own_partials)
{
    return 1024 + smallm_body_bytes(mt, stages, splits, kbs, own_partials) + (2 * kSmallMMaxStages + 2) * 8 + 16;
}

template <bool kWMnMajor>
__global__ void __launch_bounds__(kSmallMThreads)
w8a8_smallm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const SmallMParams p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t ring = raw_addr + pad;

    const uint32_t block_bytes = smallm_block_bytes(p.mt);
    const uint32_t stage_bytes = smallm_stage_bytes(p.mt, p.kbs);
    const uint32_t ring_bytes = p.stages * stage_bytes;
    const bool own_partials = p.own_partials != 0;
    const uint32_t body = smallm_body_bytes(p.mt, p.stages, p.splits, p.kbs, own_partials);
    uint64_t* s_bars = reinterpret_cast<uint64_t*>(smem + body);
    const uint32_t bar_full = smem_u32(s_bars);
    const uint32_t bar_empty = bar_full + kSmallMMaxStages * 8;
    const uint32_t bar_tmem_full = bar_empty + kSmallMMaxStages * 8;
    const uint32_t bar_partials = bar_tmem_full + 8;  // first CTA: the other CTAs' sums have landed
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + 2 * kSmallMMaxStages + 2);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;
    // [(splits-1)][128][mt], first CTA only: behind the ring, or aliased onto it
    int32_t* s_partials = reinterpret_cast<int32_t*>(smem + (own_partials ? ring_bytes : 0));

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t split = p.splits > 1 ? cluster_ctarank() : 0;
    const uint32_t tile = blockIdx.x / p.splits;
    const int32_t n0 = static_cast<int32_t>(tile * p.tile_rows);

    // this CTA's slice of K, in 128-byte blocks
    const uint32_t kb_per = (p.num_k_blocks + p.splits - 1) / p.splits;
    const uint32_t kb_begin = split * kb_per < p.num_k_blocks ? split * kb_per : p.num_k_blocks;
    const uint32_t kb_end = kb_begin + kb_per < p.num_k_blocks ? kb_begin + kb_per : p.num_k_blocks;
    const uint32_t my_kb = kb_end - kb_begin;

    uint32_t tmem_cols = 32;
    while (tmem_cols < p.mt) {
        tmem_cols <<= 1;
    }

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        mbar_init(bar_tmem_full, 1);
        mbar_init(bar_partials, (p.splits - 1) * kEpilogueThreads);  // one arrival per pushing thread
        fence_mbar_init();
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(s_tmem_ptr), tmem_cols);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem_ptr;
    if (own_partials) {
        cluster_sync();  // the first CTA's barrier exists before any other CTA can arrive on it (off the critical path)
    }
    grid_launch_dependents();  // a dependent launch may start its own set-up and weight prefetch from here on

    if (warp == 0) {
        if (lane == 0) {
            // The kernel is launched with programmatic dependent launch: its set-up overlaps the tail of the kernel
            // before it on the stream.  By default nothing is read from global memory before griddepcontrol.wait
            // (plain stream order).  When the caller declares the weights static (not written by earlier work on
            // this stream), the first ring fill of WEIGHT tiles is issued before the wait; the activation tiles
            // (and, transitively, every store to D) always come after it.
            auto load_w = [&](uint32_t stage, uint32_t kb, uint32_t nsub) {
                const uint32_t full = bar_full + stage * 8;
                // the W box holds tile_rows rows; the UMMA still reads 128: the rows behind are never stored
                mbar_expect_tx(full, nsub * (p.tile_rows + p.mt) * kBlockKBytes);
                // the sub-blocks of a stage are neighbours in K: each weight row is read in runs of
                // nsub*128 contiguous bytes issued together
                for (uint32_t sub = 0; sub < nsub; ++sub) {
                    const uint32_t sw = ring + stage * stage_bytes + sub * block_bytes;
                    const int32_t k0 = static_cast<int32_t>(kb + sub) * kBlockKBytes;
                    if constexpr (kWMnMajor) {
                        tma_load_2d(sw, &tmap_w, full, n0, k0);  // rows = k, 128 bytes of n
                    } else {
                        tma_load_2d(sw, &tmap_w, full, k0, n0);  // rows = n, 128 bytes of k
                    }
                }
            };
            auto load_x = [&](uint32_t stage, uint32_t kb, uint32_t nsub) {
                const uint32_t full = bar_full + stage * 8;
                for (uint32_t sub = 0; sub < nsub; ++sub) {
                    const uint32_t sx = ring + stage * stage_bytes + sub * block_bytes + kSmallMTileN * kBlockKBytes;
                    tma_load_2d(sx, &tmap_x, full, static_cast<int32_t>(kb + sub) * kBlockKBytes, 0);
                }
            };
            const uint32_t iters = (my_kb + p.kbs - 1) / p.kbs;
            const uint32_t pre = iters < p.stages ? iters : p.stages;  // the ring is empty: no waits needed
            if (!p.static_weights) {
                grid_dependency_wait();
            }
            for (uint32_t i = 0; i < pre; ++i) {
                const uint32_t kb = kb_begin + i * p.kbs;
                load_w(i, kb, kb_end - kb < p.kbs ? kb_end - kb : p.kbs);
            }
            grid_dependency_wait();
            for (uint32_t i = 0; i < pre; ++i) {
                const uint32_t kb = kb_begin + i * p.kbs;
                load_x(i, kb, kb_end - kb < p.kbs ? kb_end - kb : p.kbs);
            }
            uint32_t stage = pre == p.stages ? 0 : pre;
            uint32_t phase = pre == p.stages ? 1 : 0;
            for (uint32_t i = pre; i < iters; ++i) {
                if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, s_abort, p.status, kDevTimeoutProducer)) {
                    break;
                }
                const uint32_t kb = kb_begin + i * p.kbs;
                const uint32_t nsub = kb_end - kb < p.kbs ? kb_end - kb : p.kbs;
                load_w(stage, kb, nsub);
                load_x(stage, kb, nsub);
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && my_kb != 0) {
            const uint32_t idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, kWMnMajor, false, kSmallMTileN, p.mt);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t kb = 0; kb < my_kb; kb += p.kbs) {
                ok = mbar_wait(bar_full + stage * 8, phase, s_abort, p.status, kDevTimeoutMma);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const uint32_t nsub = my_kb - kb < p.kbs ? my_kb - kb : p.kbs;
                for (uint32_t sub = 0; sub < nsub; ++sub) {
                    const uint32_t sw = ring + stage * stage_bytes + sub * block_bytes;
                    const uint32_t sx = sw + kSmallMTileN * kBlockKBytes;
#pragma unroll
                    for (int j = 0; j < kBlockKBytes / kUmmaK; ++j) {
                        uint64_t dw;
                        if constexpr (kWMnMajor) {
                            dw = make_smem_desc_sw128(sw + j * (kUmmaK * 128), kBlockKBytes * 128, 1024);
                        } else {
                            dw = make_smem_desc_sw128(sw + j * kUmmaK, 16, 1024);
                        }
                        const uint64_t dx = make_smem_desc_sw128(sx + j * kUmmaK, 16, 1024);
                        umma_i8<1>(tmem_base, dw, dx, idesc, (kb | sub | j) != 0 ? 1u : 0u);
                    }
                }
                umma_commit<1>(bar_empty + stage * 8);
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) {
                umma_commit<1>(bar_tmem_full);
            }
        }
        __syncwarp();
    }

    // ---- epilogue: warps 2..5 own the accumulator rows; every thread of the cluster passes both cluster
    // barriers, whatever happened before, so no CTA can be left waiting for a peer
    const bool epi = warp >= 2;
    const uint32_t quad = warp & 3;
    const uint32_t row = quad * 32 + lane;  // weight row inside the tile = TMEM lane
    bool have = false;                      // this thread's accumulator row is valid
    // The scales are fetched while the K loop runs, not after it: channel scale of this thread's row, and the
    // per-token scales four to a lane (token t in lane t % 32, register t / 32), handed out by shuffles later.
    // Loads issued after the accumulator is ready would each cost an L2 round trip on the kernel's tail.
    float sc = 0.0f;
    float tok[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (epi && split == 0) {
        const uint32_t ncol_early = static_cast<uint32_t>(n0) + row;
        if (!p.static_weights) {
            grid_dependency_wait();
        }
        if (ncol_early < p.n && row < p.tile_rows) {
            sc = p.scalar_mode ? p.scalar_scale : load_scale(p.scale, ncol_early, p.scale_type);
        }
        grid_dependency_wait();                // the per-token scales may depend on the previous kernel
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t t = q * 32 + lane;
            tok[q] = t >= p.m ? 0.0f : (p.per_token ? load_scale(p.per_token, t, p.scale_type) : 1.0f);
        }
    }
    if (epi && my_kb != 0) {
        bool ok = mbar_wait(bar_tmem_full, 0, s_abort, p.status, kDevTimeoutEpilogue);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tcgen05_fence_after();
            have = true;
        }
    }
    const uint32_t taddr = tmem_base + ((quad * 32u) << 16);
    const uint32_t chunks = p.mt / 16;

    if (p.splits > 1) {
        if (!own_partials) {
            cluster_sync();  // the first CTA's ring is idle from here on: it becomes the partial-sum buffer
        }
        if (split != 0 && epi) {
            // remote address of slot (split-1), this thread's row
            const uint32_t local = smem_u32(s_partials) + ((split - 1) * kSmallMTileN + row) * p.mt * 4;
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0u));
            for (uint32_t c = 0; c < chunks; ++c) {
                uint32_t r[16];
                if (have) {
                    tmem_ld_32x32b_x16(taddr + c * 16, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        r[i] = 0;
                    }
                }
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(remote + c * 64 + v * 16),
                                 "r"(r[v * 4]), "r"(r[v * 4 + 1]), "r"(r[v * 4 + 2]), "r"(r[v * 4 + 3])
                                 : "memory");
                }
            }
            if (own_partials) {
                mbar_arrive_cluster(bar_partials, 0);  // release: this thread's stores are visible to the waiter
            }
        }
        if (!own_partials) {
            cluster_sync();  // partial sums have landed in the first CTA's smem
        } else if (split == 0 && epi) {
            // (a CTA that timed out still arrives, with zeros: every thread of the cluster passes this point)
            bool ok = mbar_wait_cluster(bar_partials, 0, s_abort, p.status, kDevTimeoutPeerCta);
            ok = __all_sync(0xffffffffu, ok);
            (void)ok;
        }
    }

    if (split == 0 && epi) {
        const uint32_t ncol = static_cast<uint32_t>(n0) + row;
        const bool n_ok = ncol < p.n && row < p.tile_rows;
        for (uint32_t c = 0; c < chunks; ++c) {
            uint32_t r[16];
            if (have) {
                tmem_ld_32x32b_x16(taddr + c * 16, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    r[i] = 0;
                }
            }
            for (uint32_t s = 1; s < p.splits; ++s) {
                const uint4* src =
                    reinterpret_cast<const uint4*>(s_partials + ((s - 1) * kSmallMTileN + row) * p.mt + c * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const uint4 q = src[v];
                    r[v * 4] += q.x;
                    r[v * 4 + 1] += q.y;
                    r[v * 4 + 2] += q.z;
                    r[v * 4 + 3] += q.w;
                }
            }
            // tokens c*16 .. c*16+15 sit in register c/2 of lanes (c%2)*16 .. +15 (all lanes take part in the
            // shuffles, whether or not their own row is stored)
            const float tq = (c >> 1) == 0 ? tok[0] : ((c >> 1) == 1 ? tok[1] : ((c >> 1) == 2 ? tok[2] : tok[3]));
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t mrow = c * 16 + i;
                const float st = __shfl_sync(0xffffffffu, tq, (c & 1) * 16 + i);
                if (n_ok && mrow < p.m) {
                    p.d[static_cast<size_t>(mrow) * p.n + ncol] = pack_out1(dequant(r[i], sc, st), p.out_f16 != 0);
                    if (p.acc != nullptr) {
                        p.acc[static_cast<size_t>(mrow) * p.n + ncol] = static_cast<int32_t>(r[i]);
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, tmem_cols);
    }
}

}  // namespace cb200
