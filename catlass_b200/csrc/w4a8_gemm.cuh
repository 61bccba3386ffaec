// W4A8 matmul with per-group weight scales for sm_100a.
//
//   acc_g[m,n] = sum_{k in group g} A[m,k] * W[k,n]              int32, exact
//   y[m,n]     = fma(float(acc_g), sw[g,n], y)   for g = 0,1,..   fp32, groups in ascending order
//   D[m,n]     = bf16_rne(y * sa[m])
//
// Weights are signed 4-bit, two per byte along K (even k in bits 0-3), one column of K/2 bytes after
// another: the reference's column-major ("trans") packing of example 32
// (examples/32_w4a8_matmul/gen_data.py:77-105).  The reference unpacks int4 -> int8 on its vector cores into
// a global staging ring and runs an int8 GEMM on top (include/catlass/gemm/kernel/w4a8_matmul.hpp:167-197,
// include/catlass/gemm/tile/atlasa2/cast_int4_to_int8.hpp:136-146); here the unpack happens between two
// shared-memory buffers of the same CTA and nothing is staged through global memory.
//
// Decomposition.  A CTA owns 128 output channels and up to 128 tokens.  The channels sit on the TMEM lanes
// (UMMA M = 128, A operand = unpacked weights) and the tokens on the UMMA N axis (N = token rows rounded up to
// 16), so a thread of the epilogue owns ONE channel: the group's weight scale is a scalar in a register.
// Every CTA has to read the whole token matrix once per pass over K, from L2; with 128 channels per CTA that
// is 2 token bytes per packed weight byte (64 channels per CTA would double it and made the token stream the
// limit).  To fill the machine when N/128 tiles are fewer than the SMs, the K range (whole scale groups) can be
// split over the 2 or 4 CTAs of a cluster; each keeps fp32 partial sums y and at the end every CTA reduces
// and stores one slice of the token columns, the partials travelling through distributed shared memory.
// With a split the fp32 sums are added in a different order than the sequential definition above: results are
// then no longer bit-identical, and an output whose partial sums nearly cancel can differ by many bf16 ulps of
// its (tiny) value.  The split is therefore opt-in (CB200_W4A8_SPLIT_K in the arguments).  By default every CTA
// runs the whole K range, which is bit-exact; to fill the machine then, the token rows are cut into tiles of 64
// instead of 128 when that still fits one wave of CTAs (each weight tile is then unpacked by two CTAs).
//
// Warp roles (16 warps):
//   warps 0,15  TMA producers: packed weight tiles (128 x 64 B, 12 in flight: they come from HBM) and token
//               tiles (mt x 128 B, as many as fit 64 KB: 8 for 64 tokens; they come from L2), one thread and one
//               ring each, two consecutive K blocks per load (3-D boxes).  Scale groups longer than one K block:
//               the token tile of a K block shares the tile slot (and both barriers) of the block's unpacked
//               weight tile instead, one block per load
//   warps 1,14  MMA issuers (tcgen05.mma.kind::i8, 128 x mt x 32; issuing an MMA costs its thread ~70 ns).
//               One-block scale groups alternate between them, each group into one of four int32 accumulators in
//               TMEM.  The K blocks of a longer group alternate between them as well: each issuer sums its
//               blocks into an accumulator of its own and the epilogue adds the two, still as int32, so the
//               group's sum stays exact.  Per K block one commit frees the unpacked tile and one its half of
//               the token load; per group one more hands the accumulator to the epilogue.
//   warps 2-5   unpack: nibble -> int8 holding 16*w (the nibble moved to the high half of the byte: no sign
//               fix-up needed), written in the 128B-swizzled K-major operand layout, then handed to the MMA
//               through a proxy fence + mbarrier.  The factor 16 is removed again, exactly, when the epilogue
//               turns the accumulator into fp32.
//   warps 6-13  epilogue (two warps per TMEM lane quarter, 64 or 32 token columns each): per group tcgen05.ld in
//               16-column pieces (the next piece is in flight while the current one is processed), int->float,
//               packed fma with the group's scale into the running sums y held in registers; after the last
//               group: reduction over the cluster, * sa[m], bf16 stores
#pragma once

#include <cuda_bf16.h>

#include "ptx.cuh"
#include "w8a8_gemm.cuh"

namespace cb200 {

constexpr int kW4Threads = 512;     // 16 warps: weight producer, MMA issuer A, 4 unpack, 8 epilogue, MMA issuer B,
                                    // token producer
constexpr int kW4Channels = 128;    // output channels per CTA (UMMA M)
constexpr int kW4Tokens = 128;      // tokens per CTA at most (UMMA N)
constexpr int kW4Accs = 4;          // int32 accumulators in TMEM (128 columns each)
constexpr int kW4AccPairs = 2;      // accumulators are handed over two at a time (halves the hand-shakes per group)
constexpr int kW4Tiles = 4;         // unpacked weight tiles in flight (= unpack warps, see there); 6 in one mode
constexpr int kW4MaxTiles = 6;
constexpr int kW4MaxPackedSlots = 12;  // packed-weight tiles in flight at most (8 KB each): covers HBM latency
constexpr int kW4MaxSplits = 4;     // CTAs of a cluster sharing one channel tile along K
#ifndef CB200_W4_LOAD
#define CB200_W4_LOAD 2
#endif
constexpr int kW4Load = CB200_W4_LOAD;  // K blocks per TMA load (3-D boxes): half the loads and barrier round trips
constexpr int kW4MaxPackedLoads = kW4MaxPackedSlots / kW4Load;  // load slots of the packed-weight ring at most
constexpr int kW4MaxTokenLoads = 8;                       // load slots of the token ring at most (see x_loads)

#ifdef CB200_DEVELOPER_KNOBS
// Developer builds only: per-role cycle counters of CTA 0 (where each role of the pipeline spends its time).
__device__ unsigned long long g_w4a8_probe[64];
#define W4_PROBE_BEGIN() const long long probe_t0__ = clock64()
#define W4_PROBE_END(slot)                                                                    \
    do {                                                                                      \
        if (blockIdx.x == 0 && blockIdx.y == 0) {                                             \
            atomicAdd(&g_w4a8_probe[slot], static_cast<unsigned long long>(clock64() - probe_t0__)); \
        }                                                                                     \
    } while (0)
#define W4_STAMP(slot)                                                                        \
    do {                                                                                      \
        if (blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0) {                  \
            atomicAdd(&g_w4a8_probe[slot], static_cast<unsigned long long>(clock64() - kernel_t0__)); \
        }                                                                                     \
    } while (0)
#define W4_STAMP_INIT() const long long kernel_t0__ = clock64()
#else
#define W4_PROBE_BEGIN() do { } while (0)
#define W4_PROBE_END(slot) do { } while (0)
#define W4_STAMP(slot) do { } while (0)
#define W4_STAMP_INIT() do { } while (0)
#endif

struct W4A8Params {
    uint32_t m, n, k;
    uint32_t tile_m;            // token rows per CTA tile: 128, or 64 (twice the CTAs for the same channel tiles)
    uint32_t mt;                // token rows loaded per tile: min(tile_m, round_up(m, 16)); also the UMMA N
    uint32_t blocks_per_group;  // group_size / 128
    uint32_t num_groups;        // k / group_size
    uint32_t splits;            // cluster size along K: 1, 2 or 4
    const float* sw;            // [k / group_size][n]
    const float* sa;            // [m]
    uint16_t* d;                // [m][n] bf16 or fp16 bit patterns
    unsigned* status;
    uint32_t out_f16;
    uint32_t static_weights;    // weights and their scales may be read before the stream dependency resolves
    uint32_t token_loads_max;   // cap on the token ring's load slots (<= kW4MaxTokenLoads)
};

// How the 224 KB of ring space are split.  kTiles = 4: four 16 KB token slots (token tiles of up to 128 rows), four
// unpacked weight tiles, twelve packed tiles.  kTiles = 6 (scale groups of several K blocks, token tiles of at most
// 64 rows): six 8 KB token slots, six unpacked tiles, ten packed tiles.  There a K block's unpacked tile stays
// in its slot from the start of the unpack to the end of its MMAs, about as long as unpacking a tile takes
// again: with four slots for four unpack warps every warp waited that long for "its" slot.
template <int kTiles>
struct W4A8Smem {
    static_assert(kTiles == 4 || kTiles == 6, "tile slots");
    static constexpr int kTokenSlotBytes = (kTiles == 6 ? 64 : kW4Tokens) * 128;  // UMMA B operand
    static constexpr int kTokenRingBytes = kTiles * kTokenSlotBytes;
    static constexpr int kCookedBytes = kW4Channels * 128;  // 16 KB: unpacked int8 weights, UMMA A operand
    static constexpr int kPackedBytes = kW4Channels * 64;   //  8 KB: packed weights as loaded
    static constexpr int kPackedSlots = kTiles == 6 ? 10 : 12;
    static constexpr int kPackedLoads = kPackedSlots / kW4Load;
    static constexpr int kTokenRing = 0;
    static constexpr int kCookedRing = kTokenRing + kTokenRingBytes;
    static constexpr int kPackedRing = kCookedRing + kTiles * kCookedBytes;
    static constexpr int kRingBytes = kPackedRing + kPackedSlots * kPackedBytes;
    // after the K loop the ring is idle and holds this CTA's fp32 sums (64 KB) followed by the other CTAs'
    // partial sums: (splits - 1) x (128 / splits) token columns x 128 channels x fp32 <= 48 KB
    static constexpr int kLandingBytes =
        kW4Tokens * kW4Channels * 4 + (kW4MaxSplits - 1) * (kW4Tokens / kW4MaxSplits) * kW4Channels * 4;
    // p_full, p_empty [packed loads]; x_full, x_free [token loads]; c_full, tiles_free [tiles]; acc_full,
    // acc_empty [accumulator pairs]
    static constexpr int kBarriers =
        2 * kW4MaxPackedLoads + 2 * kW4MaxTokenLoads + 2 * kW4MaxTiles + 2 * kW4AccPairs;
    static constexpr int kBarrierBytes = kBarriers * 8 + 16 + kW4Tokens * 4;  // + the tile's per-token scales
    static constexpr int kTotalBytes = 1024 + kRingBytes + kBarrierBytes;
    static_assert(kPackedSlots % kW4Load == 0 && kPackedSlots <= kW4MaxPackedSlots && kTiles <= kW4MaxTiles, "rings");
    static_assert(kTotalBytes <= 227 * 1024, "shared memory budget");
    static_assert(kLandingBytes <= kRingBytes, "the landing buffer aliases the ring");
};
static_assert(kW4Accs * kW4Tokens <= 512, "TMEM budget");

// The running sums y are kept as pairs of fp32 in 64-bit registers so that the per-group update is exactly four
// instructions per two outputs (two integer adds, one packed subtract, one packed fused multiply-add) with no
// register shuffling in between.
//
// scaled_accumulate_pair: y += (x/16) * s for two (x, s, y) triples, x an int32 with |x| < 2^22.
//   x/16 exactly, without the conversion unit: 0x49400000 is the bit pattern of 1.5 * 2^19, whose unit in the
//   last place is 1/16; adding x to the pattern yields the float 1.5 * 2^19 + x/16, and subtracting 1.5 * 2^19
//   again is exact.  (The accumulators hold 16 times the true sums: see the unpack warps.)
__device__ __forceinline__ void scaled_accumulate_pair(unsigned long long& y2, uint32_t x0, uint32_t x1,
                                                       unsigned long long s2)
{
    // (volatile: keeps the arithmetic where the source puts it, between the issue of the next TMEM read and the
    // wait for it; left to itself the compiler gathers it behind the wait and the read's latency is exposed)
    asm volatile("{\n\t"
        ".reg .b32 lo, hi;\n\t"
        ".reg .b64 t, c;\n\t"
        "add.u32 lo, %1, 0x49400000;\n\t"
        "add.u32 hi, %2, 0x49400000;\n\t"
        "mov.b64 t, {lo, hi};\n\t"
        "mov.b64 c, 0xC9400000C9400000;\n\t"   // (-1.5 * 2^19, -1.5 * 2^19)
        "add.rn.f32x2 t, t, c;\n\t"
        "fma.rn.f32x2 %0, t, %3, %0;\n\t"
        "}\n"
        : "+l"(y2)
        : "r"(x0), "r"(x1), "l"(s2));
}

// y += a * s for two lanes, a given as two floats
__device__ __forceinline__ void fma_pair(unsigned long long& y2, float a0, float a1, unsigned long long s2)
{
    asm("{\n\t"
        ".reg .b64 t;\n\t"
        "mov.b64 t, {%1, %2};\n\t"
        "fma.rn.f32x2 %0, t, %3, %0;\n\t"
        "}\n"
        : "+l"(y2)
        : "f"(a0), "f"(a1), "l"(s2));
}

__device__ __forceinline__ void unpack_pair(unsigned long long v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ unsigned long long pack_pair(float lo, float hi)
{
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}

// y2[kOff .. kOff+7] (16 token columns) += group sums r[0..15] * s.
// kMagic: |r| < 2^22 (one 128-wide K block per group).
template <bool kMagic, int kOff, int kSums>
__device__ __forceinline__ void accumulate16(unsigned long long (&y2)[kSums], const uint32_t (&r)[16], float s)
{
    static_assert(kOff + 8 <= kSums, "running sums of this thread");
    const unsigned long long s2 = pack_pair(s, s);
#pragma unroll
    for (int v = 0; v < 8; ++v) {
        if constexpr (kMagic) {
            scaled_accumulate_pair(y2[kOff + v], r[2 * v], r[2 * v + 1], s2);
        } else {
            // the sums are multiples of 16 below 2^28: the conversion and the scaling by 1/16 are exact
            fma_pair(y2[kOff + v], __int2float_rn(static_cast<int32_t>(r[2 * v])) * 0.0625f,
                     __int2float_rn(static_cast<int32_t>(r[2 * v + 1])) * 0.0625f, s2);
        }
    }
}

// kOneBlockGroups: the scale group is exactly one 128-wide K block (the common case): the int->float step can
// then use the add-a-constant form.
// kTiles: tile slots of the ring (see W4A8Smem); 6 only with scale groups of several K blocks and token tiles of at
// most 64 rows.
template <bool kOneBlockGroups, int kTiles = kW4Tiles>
__global__ void __launch_bounds__(kW4Threads, 1)
w4a8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const W4A8Params p)
{
    using S = W4A8Smem<kTiles>;
    static_assert(kTiles == kW4Tiles || !kOneBlockGroups, "one-block groups: one tile slot per unpack warp");
    constexpr uint32_t kPackedSlots = S::kPackedSlots, kPackedLoads = S::kPackedLoads;
    extern __shared__ uint8_t smem_raw[];
    W4_STAMP_INIT();
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t ring = raw_addr + pad;

    uint64_t* s_bars = reinterpret_cast<uint64_t*>(smem + S::kRingBytes);
    const uint32_t bar_p_full = smem_u32(s_bars);                    // packed tile landed (TMA bytes)
    const uint32_t bar_p_empty = bar_p_full + kW4MaxPackedLoads * 8;    // the unpack warps have read both tiles
    const uint32_t bar_x_full = bar_p_empty + kW4MaxPackedLoads * 8;    // a pair of token tiles landed
    const uint32_t bar_x_free = bar_x_full + kW4MaxTokenLoads * 8;   // the MMAs that read the pair completed
    const uint32_t bar_c_full = bar_x_free + kW4MaxTokenLoads * 8;   // unpacked tile written
    const uint32_t bar_tiles_free = bar_c_full + kW4MaxTiles * 8;    // the MMAs that read the unpacked tile completed
    const uint32_t bar_acc_full = bar_tiles_free + kW4MaxTiles * 8;     // all MMAs of a pair of scale groups completed
    const uint32_t bar_acc_empty = bar_acc_full + kW4AccPairs * 8;   // the epilogue has read the pair's accumulators
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + S::kBarriers);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;
    float* s_sa = reinterpret_cast<float*>(s_tmem_ptr + 4);  // per-token scales of this tile's rows (see the epilogue)

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t splits = p.splits;
    const uint32_t rank = splits > 1 ? cluster_ctarank() : 0;  // position along K inside the cluster
    const int32_t n0 = static_cast<int32_t>(blockIdx.x / splits) * kW4Channels;
    const int32_t m0 = static_cast<int32_t>(blockIdx.y * p.tile_m);
    const uint32_t bpg = p.blocks_per_group;
    // this CTA's scale groups [g_begin, g_begin + my_groups) and K blocks [kb_begin, kb_begin + my_kb)
    const uint32_t groups_per_rank = (p.num_groups + splits - 1) / splits;
    const uint32_t g_begin = rank * groups_per_rank < p.num_groups ? rank * groups_per_rank : p.num_groups;
    const uint32_t my_groups =
        g_begin + groups_per_rank <= p.num_groups ? groups_per_rank : p.num_groups - g_begin;
    const uint32_t kb_begin = g_begin * bpg;
    const uint32_t my_kb = my_groups * bpg;
    // One scale group for the whole K range of this CTA: the epilogue has nothing to do until the last MMA, and what
    // sets the pace is the unpacking (one warp needs ~1350 cycles per tile).  Four of the epilogue warps then take
    // the lower half of every tile's rows off the unpack warps.
    const bool unpack_helpers = !kOneBlockGroups && my_groups == 1;
    constexpr uint32_t kTmemCols = 512;
    // The token ring (64 KB) holds as many K blocks of mt x 128 bytes as fit: 4 blocks of 128 tokens, 8 of 64, 16 of
    // fewer.  Token tiles come from L2 with ~1-2 us of latency while every CTA of the grid asks for the same lines,
    // so the bytes in flight decide the rate; the ring is independent of the four unpacked-tile slots.
    const uint32_t x_load_bytes = kW4Load * p.mt * 128;
    const uint32_t x_loads_fit = S::kTokenRingBytes / x_load_bytes;
    const uint32_t x_loads = x_loads_fit < p.token_loads_max ? x_loads_fit : p.token_loads_max;

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int i = 0; i < kW4MaxPackedLoads; ++i) {
            mbar_init(bar_p_full + i * 8, 1);
            mbar_init(bar_p_empty + i * 8, kW4Load * (unpack_helpers ? 2 : 1));  // one arrival per tile (half)
        }
        for (int i = 0; i < kW4MaxTokenLoads; ++i) {
            mbar_init(bar_x_full + i * 8, 1);
            mbar_init(bar_x_free + i * 8, kW4Load);  // one commit per K block of the load
        }
        for (int i = 0; i < kW4MaxTiles; ++i) {
            // longer groups: the slot's token tile lands on the same barrier (the producer's expect_tx arrival)
            mbar_init(bar_c_full + i * 8, kOneBlockGroups ? 1 : (unpack_helpers ? 3 : 2));
            mbar_init(bar_tiles_free + i * 8, 1);
        }
        for (int i = 0; i < kW4AccPairs; ++i) {
            mbar_init(bar_acc_full + i * 8, 2);   // one arrival per group of the pair
            mbar_init(bar_acc_empty + i * 8, 8);  // one per epilogue warp
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(s_tmem_ptr), kTmemCols);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem_ptr;
    grid_launch_dependents();  // a dependent launch may start its own set-up and weight prefetch from here on
    if (warp == 6) {
        W4_STAMP(20);  // set-up done
    }

    // running sums of this thread's channel over its 64 token columns, two fp32 per register (epilogue warps)
    // (six tile slots: token tiles of at most 64 rows, 32 columns per epilogue thread)
    constexpr int kSums = kTiles == 6 ? 16 : 32;
    unsigned long long y2[kSums];
#pragma unroll
    for (int i = 0; i < kSums; ++i) {
        y2[i] = 0ull;
    }

    // Ring discipline: local K block i uses packed slot i % kPackedSlots and tile slot i % kTiles; local
    // group j uses accumulator j % kW4Accs.  "The previous user of this slot is done" = wait with the inverted
    // parity of the use count (passes at once for the first use).

    // ------------------------------------------------------- unpacking (warps 2..5; with helpers: also warps 6..9)
    // Unpack warp u handles the local K blocks i = u, u+4, ... : sixteen 16-byte chunks per lane (rounds 0..3 of four
    // chunks), one fence and one arrival per block; with helpers it does rounds 0..1 and epilogue warp 6+u rounds
    // 2..3 of the same blocks.  A block's tile slot was last used kTiles blocks earlier; the warps that wait for it
    // walk the same blocks one after the other: a parity wait can tell "the previous use is over" from "not yet"
    // only if the waiter is never two uses ahead (kTiles = 6: the MMAs of block i-10, which this warp waited for
    // at block i-4, were committed by the issuer of block i-12 after that block's).
    // Lane l, step s works on row = s*8 + l/4, packed chunk c = l%4.
    auto unpack_loop = [&](const uint32_t u, const uint32_t round_begin, const uint32_t round_end) {
        // the packed tile was loaded with the 64-byte TMA swizzle: 16-byte chunk c of row r sits at
        // chunk c ^ ((r >> 1) & 3); the operand tile uses the 128-byte swizzle: chunk j at j ^ (r & 7)
        const uint32_t c = lane & 3;
        const uint32_t rsub = lane >> 2;  // 0..7: row inside a group of eight (= row & 7)
        for (uint32_t i = u; i < my_kb; i += 4) {
            const uint32_t pl = (i / kW4Load) % kPackedLoads;          // load slot of this block's packed tile
            const uint32_t pph = ((i / kW4Load) / kPackedLoads) & 1;
            const uint32_t ps = i % kPackedSlots;                      // tile slot inside the ring
            const uint32_t cs = i % kTiles;
            bool ok;
            {
                W4_PROBE_BEGIN();
                ok = mbar_wait(bar_p_full + pl * 8, pph, s_abort, p.status, kDevTimeoutConvert);
                if (lane == 0 && u == 0 && round_begin == 0) {
                    W4_PROBE_END(10);
                }
            }
            {
                W4_PROBE_BEGIN();
                ok = ok && mbar_wait(bar_tiles_free + cs * 8, ((i / kTiles) & 1) ^ 1, s_abort, p.status,
                                     kDevTimeoutConvert);
                if (lane == 0 && u == 0 && round_begin == 0) {
                    W4_PROBE_END(11);
                }
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                return;
            }
            W4_PROBE_BEGIN();
            const uint8_t* packed = smem + S::kPackedRing + ps * S::kPackedBytes;
            uint8_t* cooked = smem + S::kCookedRing + cs * S::kCookedBytes;
            // (four rounds of four chunks, deliberately not unrolled across rounds: the loop body has to stay
            // small, the warps of this CTA run five different loops and share one instruction cache)
#pragma unroll 1
            for (uint32_t round = round_begin; round < round_end; ++round) {
                uint4 q[4];
#pragma unroll
                for (uint32_t s = 0; s < 4; ++s) {
                    const uint32_t row = (round * 4 + s) * 8 + rsub;
                    q[s] = *reinterpret_cast<const uint4*>(packed + row * 64 + ((c ^ ((row >> 1) & 3)) << 4));
                }
                if (round + 1 == round_end) {
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(bar_p_empty + pl * 8);  // this tile is in registers (the slot refills after both)
                    }
                }
#pragma unroll
                for (uint32_t s = 0; s < 4; ++s) {
                    const uint32_t row = (round * 4 + s) * 8 + rsub;
                    const uint32_t w[4] = {q[s].x, q[s].y, q[s].z, q[s].w};
                    uint32_t o[8];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t lo = (w[j] << 4) & 0xF0F0F0F0u;  // even k: low nibbles, moved up
                        const uint32_t hi = w[j] & 0xF0F0F0F0u;         // odd k: high nibbles, in place
                        o[2 * j] = __byte_perm(lo, hi, 0x5140);
                        o[2 * j + 1] = __byte_perm(lo, hi, 0x7362);
                    }
                    uint8_t* crow = cooked + row * 128;
                    *reinterpret_cast<uint4*>(crow + (((2 * c) ^ rsub) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(crow + (((2 * c + 1) ^ rsub) << 4)) =
                        make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_c_full + cs * 8);
            }
            if (lane == 0 && u == 0 && round_begin == 0) {
                W4_PROBE_END(12);
            }
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------- packed-weight producer
        // (Weights and tokens each have a producer thread of their own: the deep weight ring keeps running ahead
        // while the token thread waits for a tile slot.)
        if (lane == 0) {
            if (!p.static_weights) {
                grid_dependency_wait();  // plain stream order: the weights may come from the kernel before this one
            }
            bool ok = true;
            const uint32_t loads = (my_kb + kW4Load - 1) / kW4Load;
            for (uint32_t l = 0; ok && l < loads; ++l) {
                const uint32_t slot = l % kPackedLoads;
                W4_PROBE_BEGIN();
                ok = mbar_wait(bar_p_empty + slot * 8, ((l / kPackedLoads) & 1) ^ 1, s_abort, p.status,
                               kDevTimeoutProducer);
                W4_PROBE_END(0);
                if (ok) {
                    // kW4Load consecutive K blocks, one 128 x 64 B tile each (a last, odd block brings the
                    // neighbouring block or zeros along: the transaction count is always that of a full box)
                    const uint32_t full = bar_p_full + slot * 8;
                    mbar_expect_tx(full, kW4Load * S::kPackedBytes);
                    tma_load_3d(ring + S::kPackedRing + slot * (kW4Load * S::kPackedBytes), &tmap_w, full, 0, n0,
                                static_cast<int32_t>(kb_begin + l * kW4Load));
                }
            }
        }
        __syncwarp();
    } else if (warp == 15) {
        // ------------------------------------------------------- token producer
        // The tokens may depend on the kernel launched before this one on the stream: under programmatic
        // dependent launch this thread waits for that kernel before its first load.  (When the caller declares
        // the weights static, the weight ring is already filling meanwhile.)  Everything that reads
        // token-dependent data or writes the output happens after a token tile has landed.
        if (lane == 0) {
            grid_dependency_wait();
            bool ok = true;
            if constexpr (!kOneBlockGroups) {
                // Longer groups: K block i's token tile shares tile slot i % kTiles with its unpacked weight tile:
                // it is loaded once the MMAs of the slot's previous block are done (the barrier the unpack warp
                // waits on, too) and lands on the slot's "full" barrier, so an MMA issuer probes one barrier and
                // commits one per K block.  (The tensor map's box is one K block deep in this mode.)
                for (uint32_t i = 0; ok && i < my_kb; ++i) {
                    const uint32_t slot = i % kTiles;
                    W4_PROBE_BEGIN();
                    ok = mbar_wait(bar_tiles_free + slot * 8, ((i / kTiles) & 1) ^ 1, s_abort, p.status,
                                   kDevTimeoutProducer);
                    W4_PROBE_END(1);
                    if (ok) {
                        const uint32_t full = bar_c_full + slot * 8;
                        mbar_expect_tx(full, p.mt * 128);
                        tma_load_3d(ring + S::kTokenRing + slot * S::kTokenSlotBytes, &tmap_x, full, 0, m0,
                                    static_cast<int32_t>(kb_begin + i));
                    }
                }
            }
            const uint32_t loads = (my_kb + kW4Load - 1) / kW4Load;
            for (uint32_t l = 0; kOneBlockGroups && ok && l < loads; ++l) {
                const uint32_t slot = l % x_loads;
                const uint32_t parity = ((l / x_loads) & 1) ^ 1;
                W4_PROBE_BEGIN();
                ok = mbar_wait(bar_x_free + slot * 8, parity, s_abort, p.status, kDevTimeoutProducer);
                W4_PROBE_END(1);
                if (ok) {
                    // kW4Load consecutive K blocks of the mt token rows (rows past m read as zeros): the tiles of
                    // a load land back to back, mt * 128 bytes apart
                    const uint32_t full = bar_x_full + slot * 8;
                    mbar_expect_tx(full, x_load_bytes);
                    tma_load_3d(ring + S::kTokenRing + slot * x_load_bytes, &tmap_x, full, 0, m0,
                                static_cast<int32_t>(kb_begin + l * kW4Load));
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 14) {
        // ------------------------------------------------------- MMA issuers
        // Even K blocks (tile slots 0,2) belong to the first issuer, odd ones (slots 1,3) to the second: each waits
        // on its tile barriers one use after the other.  A one-block group is one block = one issuer = one
        // accumulator (0,2 the first issuer's, 1,3 the second's), handed to the epilogue in pairs of groups.  A
        // longer group owns an accumulator PAIR: each issuer sums its blocks of the group into its own
        // accumulator of the pair (its MMAs into that accumulator are issued in order), both commit the pair's
        // "full" barrier after their last block, and the epilogue adds the two int32 sums.
        static_assert(kTiles % 2 == 0 && kW4Accs % 2 == 0, "slot ownership of the two issuers");
        if (lane == 0) {
            const uint32_t idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, false, false, kW4Channels, p.mt);
            const uint32_t w = warp == 1 ? 0u : 1u;
            bool ok = true;
            // one K block: wait for its token tile and its unpacked tile, four MMAs, free both
            auto issue_block = [&](uint32_t i, uint32_t tmem_d, bool first) -> bool {
                const uint32_t slot = i % kTiles;
                const uint32_t ph = (i / kTiles) & 1;
                if constexpr (!kOneBlockGroups) {
                    // token tile and unpacked tile share the slot and its barriers (see the token producer)
                    bool got;
                    {
                        W4_PROBE_BEGIN();
                        got = mbar_wait(bar_c_full + slot * 8, ph, s_abort, p.status, kDevTimeoutMma);
                        W4_PROBE_END(warp == 1 ? 6 : 7);
                    }
                    if (!got) {
                        return false;
                    }
                    W4_PROBE_BEGIN();
                    tcgen05_fence_after();
                    const uint32_t sw_tile = ring + S::kCookedRing + slot * S::kCookedBytes;  // UMMA A operand
                    const uint32_t sx_tile = ring + S::kTokenRing + slot * S::kTokenSlotBytes;    // UMMA B operand
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint64_t da = make_smem_desc_sw128(sw_tile + q * kUmmaK, 16, 1024);
                        const uint64_t db = make_smem_desc_sw128(sx_tile + q * kUmmaK, 16, 1024);
                        umma_i8<1>(tmem_d, da, db, idesc, (!first || q != 0) ? 1u : 0u);
                    }
                    umma_commit<1>(bar_tiles_free + slot * 8);  // both tiles of the slot may be overwritten
                    W4_PROBE_END(warp == 1 ? 8 : 9);
                    return true;
                }
                const uint32_t xl = i / kW4Load;        // token load this block came with
                const uint32_t xslot = xl % x_loads;
                bool got;
                {
                    W4_PROBE_BEGIN();
                    got = mbar_wait(bar_x_full + xslot * 8, (xl / x_loads) & 1, s_abort, p.status, kDevTimeoutMma);
                    W4_PROBE_END(warp == 1 ? 4 : 5);
                }
                {
                    W4_PROBE_BEGIN();
                    got = got && mbar_wait(bar_c_full + slot * 8, ph, s_abort, p.status, kDevTimeoutMma);
                    W4_PROBE_END(warp == 1 ? 6 : 7);
                }
                if (!got) {
                    return false;
                }
                W4_PROBE_BEGIN();
                tcgen05_fence_after();
                const uint32_t sw_tile = ring + S::kCookedRing + slot * S::kCookedBytes;  // UMMA A operand
                const uint32_t sx_tile =
                    ring + S::kTokenRing + xslot * x_load_bytes + (i % kW4Load) * p.mt * 128;  // UMMA B operand
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint64_t da = make_smem_desc_sw128(sw_tile + q * kUmmaK, 16, 1024);
                    const uint64_t db = make_smem_desc_sw128(sx_tile + q * kUmmaK, 16, 1024);
                    umma_i8<1>(tmem_d, da, db, idesc, (!first || q != 0) ? 1u : 0u);
                }
                umma_commit<1>(bar_tiles_free + slot * 8);  // the unpacked tile may be overwritten
                umma_commit<1>(bar_x_free + xslot * 8);     // ... and this block's half of the token load
                W4_PROBE_END(warp == 1 ? 8 : 9);
                return true;
            };
            if constexpr (kOneBlockGroups) {
                for (uint32_t j = w; ok && j < my_groups; j += 2) {
                    const uint32_t pair = j >> 1, pslot = pair % kW4AccPairs;
                    {
                        W4_PROBE_BEGIN();
                        ok = mbar_wait(bar_acc_empty + pslot * 8, ((pair / kW4AccPairs) & 1) ^ 1, s_abort, p.status,
                                       kDevTimeoutMmaTmem);
                        W4_PROBE_END(warp == 1 ? 2 : 3);
                    }
                    ok = ok && issue_block(j, tmem_base + (j % kW4Accs) * kW4Tokens, true);
                    if (!ok) {
                        break;
                    }
                    umma_commit<1>(bar_acc_full + pslot * 8);  // the group's accumulator is complete
                    if (j + 1 == my_groups && (j & 1) == 0) {
                        mbar_arrive(bar_acc_full + pslot * 8);  // an odd last group: the pair has no second member
                    }
                }
            } else {
                for (uint32_t j = 0; ok && j < my_groups; ++j) {
                    const uint32_t pslot = j % kW4AccPairs;
                    {
                        W4_PROBE_BEGIN();
                        ok = mbar_wait(bar_acc_empty + pslot * 8, ((j / kW4AccPairs) & 1) ^ 1, s_abort, p.status,
                                       kDevTimeoutMmaTmem);
                        W4_PROBE_END(warp == 1 ? 2 : 3);
                    }
                    const uint32_t tmem_d = tmem_base + (2 * pslot + w) * kW4Tokens;
                    const uint32_t i0 = j * bpg;
                    bool first = true;
                    for (uint32_t i = i0 + ((i0 & 1) != w ? 1u : 0u); ok && i < i0 + bpg; i += 2) {
                        ok = issue_block(i, tmem_d, first);
                        first = false;
                    }
                    if (!ok) {
                        break;
                    }
                    umma_commit<1>(bar_acc_full + pslot * 8);  // this issuer's share of the group is complete
                }
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        unpack_loop(warp - 2, 0, unpack_helpers ? 2u : 4u);
    } else {
        // ------------------------------------------------------- epilogue warps 6..13
        const uint32_t ew = warp - 6;     // 0..7
        if (unpack_helpers && ew < 4) {
            unpack_loop(ew, 2, 4);  // the lower halves of unpack warp ew's tiles, then the epilogue of the one group
        }
        const uint32_t quad = warp & 3;   // TMEM lane quarter this warp may read: channels quad*32 .. +31
        const uint32_t half = ew >> 2;    // which part of the token columns (see hcols)
        // the two warps of a lane quarter split the token columns: 64 each, or 32 each when the tile has <= 64
        const uint32_t hcols = p.mt > 64 ? 64u : 32u;
        const uint32_t cols_mine = p.mt > half * hcols ? (p.mt - half * hcols < hcols ? p.mt - half * hcols : hcols) : 0;
        const uint32_t np = (cols_mine + 31) / 32;  // 32-column halves of this warp's range that hold tokens
        // This lane's channel scale of every group: plain loads issued three groups ahead of their use and
        // held in registers, so that the latency never sits on the per-group critical path.
        const uint32_t scol = static_cast<uint32_t>(n0) + quad * 32 + lane;
        const float* sw_col = p.sw + static_cast<size_t>(g_begin) * p.n + (scol < p.n ? scol : 0);
        if (!p.static_weights) {
            grid_dependency_wait();  // the weight scales may come from the kernel before this one
        }
        auto load_sw = [&](uint32_t j) -> float {
            return j < my_groups ? __ldg(sw_col + static_cast<size_t>(j) * p.n) : 0.0f;
        };
        float s_now = load_sw(0), s_next1 = load_sw(1), s_next2 = load_sw(2);
        if (ew >= 4) {
            // The per-token scales of this tile's rows, fetched now for the output loop at the end: there a load
            // from global memory per step of the loop was 0.35 us each time, on the kernel's tail.  (They may depend
            // on the kernel before this one on the stream; the barrier before the output loop orders the stores.)
            grid_dependency_wait();
            const uint32_t t = (ew - 4) * 32 + lane;
            s_sa[t] = static_cast<uint32_t>(m0) + t < p.m ? __ldg(p.sa + m0 + t) : 0.0f;
        }
        auto scale_of = [&](uint32_t j) -> float {
            const float s = s_now;
            s_now = s_next1;
            s_next1 = s_next2;
            s_next2 = load_sw(j + 3);
            return s;
        };
        auto acquire = [&](uint32_t pair) -> bool {
            W4_PROBE_BEGIN();
            bool got = mbar_wait(bar_acc_full + (pair % kW4AccPairs) * 8, (pair / kW4AccPairs) & 1, s_abort, p.status,
                                 kDevTimeoutEpilogue);
            if (lane == 0 && ew == 0) {
                W4_PROBE_END(13);
            }
            got = __all_sync(0xffffffffu, got);
            if (got) {
                tcgen05_fence_after();
            }
            return got;
        };
        auto release = [&](uint32_t pair) {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_acc_empty + (pair % kW4AccPairs) * 8);
            }
        };
        const uint32_t tmem_mine = tmem_base + half * hcols + ((quad * 32u) << 16);
        auto issue = [&](uint32_t j, uint32_t piece, uint32_t(&r)[16]) {
            tmem_ld_32x32b_x16(tmem_mine + (j % kW4Accs) * kW4Tokens + piece * 16, r);
        };
        // one-block groups are handed over two at a time; a longer group is a hand-over of its own
        const uint32_t handovers = kOneBlockGroups ? (my_groups + 1) / 2 : my_groups;
        if (np == 0) {
            // no token columns here (few tokens): only keep the accumulator hand-shake going
            for (uint32_t pair = 0; pair < handovers; ++pair) {
                if (!acquire(pair)) {
                    break;
                }
                release(pair);
            }
        } else if constexpr (!kOneBlockGroups) {
            // Longer groups: the two issuers' int32 sums of the group (accumulators 2*slot and 2*slot+1) are read
            // together, 16 token columns at a time, and added before the int->float step.  These hand-overs are
            // bpg K blocks apart, and the other accumulator pair is being filled meanwhile.
            uint32_t ra[16], rb[16];
            bool ok = true;
            for (uint32_t j = 0; ok && j < my_groups; ++j) {
                const float s = scale_of(j);
                ok = acquire(j);
                if (!ok) {
                    break;
                }
                const uint32_t t0 = tmem_mine + 2 * (j % kW4AccPairs) * kW4Tokens;
                auto piece = [&](uint32_t c) {
                    tmem_ld_32x32b_x16(t0 + c * 16, ra);
                    tmem_ld_32x32b_x16(t0 + kW4Tokens + c * 16, rb);
                    tmem_ld_wait_x16(ra);
                    tmem_ld_wait_x16(rb);
#pragma unroll
                    for (int v = 0; v < 16; ++v) {
                        ra[v] += rb[v];
                    }
                };
                piece(0);
                accumulate16<false, 0>(y2, ra, s);
                piece(1);
                if constexpr (kSums == 32) {
                    if (np == 2) {
                        accumulate16<false, 8>(y2, ra, s);
                        piece(2);
                        accumulate16<false, 16>(y2, ra, s);
                        piece(3);
                        release(j);
                        accumulate16<false, 24>(y2, ra, s);
                        continue;
                    }
                }
                release(j);
                accumulate16<false, 8>(y2, ra, s);
            }
        } else if constexpr (kSums == 32) {
            // Two register sets alternate over the 16-column pieces of a group; the read of the next piece (of
            // the next group, at the end) is in flight while the sums of the current one are updated.
            uint32_t ra[16], rb[16];
            bool ok = my_groups == 0 || acquire(0);
            if (ok && my_groups != 0) {
                issue(0, 0, ra);
            }
#ifdef CB200_DEVELOPER_KNOBS
            const long long epi_t0 = clock64();
#endif
            for (uint32_t j = 0; ok && j < my_groups; ++j) {
                const float s = scale_of(j);
                tmem_ld_wait_x16(ra);
                issue(j, 1, rb);
                accumulate16<kOneBlockGroups, 0>(y2, ra, s);
                tmem_ld_wait_x16(rb);
                if (np == 2) {
                    issue(j, 2, ra);
                    accumulate16<kOneBlockGroups, 8>(y2, rb, s);
                    tmem_ld_wait_x16(ra);
                    issue(j, 3, rb);
                    accumulate16<kOneBlockGroups, 16>(y2, ra, s);
                    tmem_ld_wait_x16(rb);
                }
                const bool pair_ends = (j & 1) != 0 || j + 1 == my_groups;
                if (pair_ends) {
                    release(j >> 1);  // every read of the pair's accumulators has completed
                }
                if (j + 1 < my_groups) {
                    if (pair_ends) {
                        ok = acquire((j + 1) >> 1);
                    }
                    if (ok) {
                        issue(j + 1, 0, ra);
                    }
                }
                if (np == 2) {
                    accumulate16<kOneBlockGroups, 24>(y2, rb, s);
                } else {
                    accumulate16<kOneBlockGroups, 8>(y2, rb, s);
                }
            }
#ifdef CB200_DEVELOPER_KNOBS
            if (lane == 0 && ew == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
                atomicAdd(&g_w4a8_probe[14], static_cast<unsigned long long>(clock64() - epi_t0));  // whole epilogue loop
            }
#endif
        }
    }

    // ----------------------------------------------------------- reduction over the cluster, output
    // This part runs once per CTA, from a cold instruction cache: it is written as short rolled loops over
    // shared memory instead of unrolled code over the register array (every 128 bytes of straight-line code
    // cost a trip to L2).  The ring is idle by now: the epilogue saw the last accumulator complete, so every
    // MMA and with it every TMA load and unpack of this CTA is over.
    //   ytile   [128 token columns][128 channels] fp32: this CTA's sums
    //   landing [splits - 1][128 / splits columns][128 channels] fp32: the other CTAs' sums for the columns
    //           this CTA reduces and stores
    const bool is_epi = warp >= 6 && warp < 14;
    if (warp == 6) {
        W4_STAMP(21);  // K loop and the last group's sums done
    }
    float* ytile = reinterpret_cast<float*>(smem);
    float* landing = ytile + kW4Tokens * kW4Channels;
    const uint32_t split_log2 = splits == 4 ? 2u : (splits == 2 ? 1u : 0u);
    const uint32_t cps_log2 = 7u - split_log2;  // log2 of the columns per CTA (shifts: no integer division here)
    const uint32_t cps_mask = (1u << cps_log2) - 1u;
    const uint32_t et = threadIdx.x - 6 * 32;   // 0..255 among the epilogue threads
    if (is_epi) {
        const uint32_t ch = (warp & 3) * 32 + lane;
        const uint32_t hcols = p.mt > 64 ? 64u : 32u;  // token columns per warp, as in the epilogue loop
        float* dst = ytile + ((warp - 6) >> 2) * hcols * kW4Channels + ch;
#pragma unroll
        for (int i = 0; i < kSums; ++i) {
            if (2u * i < hcols) {
                float lo, hi;
                unpack_pair(y2[i], lo, hi);
                dst[(2 * i) * kW4Channels] = lo;
                dst[(2 * i + 1) * kW4Channels] = hi;
            }
        }
    }
    if (splits > 1) {
        cluster_sync();  // every CTA of the cluster is past its K loop and has written its ytile
        if (is_epi) {
            // push the columns other CTAs own into their landing buffers, 16 bytes at a time
            for (uint32_t v = et; v < kW4Tokens * (kW4Channels / 4); v += 256) {
                const uint32_t col = v >> 5, c4 = v & 31;
                const uint32_t owner = col >> cps_log2;
                if (owner != rank && col < p.mt) {
                    const uint32_t slot = rank < owner ? rank : rank - 1;
                    const float4 val = *reinterpret_cast<const float4*>(ytile + col * kW4Channels + c4 * 4);
                    const uint32_t local =
                        smem_u32(landing + ((slot << cps_log2) + (col & cps_mask)) * kW4Channels + c4 * 4);
                    uint32_t remote;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(owner));
                    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(val.x),
                                 "f"(val.y), "f"(val.z), "f"(val.w)
                                 : "memory");
                }
            }
        }
        cluster_sync();  // the partial sums have landed
    } else if (is_epi) {
        asm volatile("bar.sync 1, 256;" ::: "memory");  // ytile complete (epilogue warps only)
    }
    if (warp == 6) {
        W4_STAMP(22);  // sums in shared memory
    }
    if (is_epi && *s_abort == 0) {
        // each thread: one token row, eight channels -> one 16-byte store
        const bool vec_ok = (p.n & 7u) == 0;
        for (uint32_t v = et; v < (kW4Channels / 8) << cps_log2; v += 256) {
            const uint32_t col = (rank << cps_log2) + (v >> 4), c8 = v & 15;
            const uint32_t mrow = static_cast<uint32_t>(m0) + col;
            const uint32_t ncol = static_cast<uint32_t>(n0) + c8 * 8;
            if (col >= p.mt || mrow >= p.m || ncol >= p.n) {  // (columns past mt belong to the next token tile)
                continue;
            }
            const float* src = ytile + col * kW4Channels + c8 * 8;
            float4 a = *reinterpret_cast<const float4*>(src);
            float4 b = *reinterpret_cast<const float4*>(src + 4);
            for (uint32_t s = 0; s + 1 < splits; ++s) {  // the other CTAs' sums, in ascending rank order
                const float* other = landing + ((s << cps_log2) + (col & cps_mask)) * kW4Channels + c8 * 8;
                const float4 oa = *reinterpret_cast<const float4*>(other);
                const float4 ob = *reinterpret_cast<const float4*>(other + 4);
                a.x += oa.x; a.y += oa.y; a.z += oa.z; a.w += oa.w;
                b.x += ob.x; b.y += ob.y; b.z += ob.z; b.w += ob.w;
            }
            const float sa = s_sa[col];
            const float y[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            uint16_t* drow = p.d + static_cast<size_t>(mrow) * p.n + ncol;
            const bool f16 = p.out_f16 != 0;
            if (vec_ok && ncol + 8 <= p.n) {
                uint32_t packed[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    packed[e] = pack_out2(__fmul_rn(y[2 * e], sa), __fmul_rn(y[2 * e + 1], sa), f16);
                }
                *reinterpret_cast<uint4*>(drow) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
                for (uint32_t e = 0; e < 8 && ncol + e < p.n; ++e) {
                    drow[e] = pack_out1(__fmul_rn(y[e], sa), f16);
                }
            }
        }
    }

    if (warp == 6) {
        W4_STAMP(23);  // output stored
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
        W4_STAMP(24);  // TMEM released
    }
}

}  // namespace cb200
