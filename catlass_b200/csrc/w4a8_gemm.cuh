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
// A CTA owns 64 output channels (so each weight byte is unpacked exactly once per 128-token row tile) and up
// to 128 tokens: tokens on the TMEM lanes (UMMA M = 128), channels on the UMMA N axis (N = 64).
//
// Warp roles (15 warps):
//   warp 0      TMA producer: packed weight tiles (64 x 64 B, 12 in flight: they come from HBM) and token tiles
//               (mt x 128 B, 6 in flight: they come from L2) into two rings fed by one non-blocking loop
//   warps 1,14  MMA issuers (tcgen05.mma.kind::i8, 128 x 64 x 32), alternate K blocks.  Every K block gets its
//               own int32 accumulator in TMEM and ONE tcgen05.commit: the same barrier tells the producer and
//               the unpack warps that the block's shared-memory tiles are free and the epilogue that its
//               accumulator is complete.  Six blocks in flight (token tiles, unpacked tiles, accumulators).
//               Issuing an MMA costs its thread ~70 ns, more than an MMA this small runs: hence two issuers.
//   warps 2-5   unpack: nibble -> int8 holding 16*w (the nibble moved to the high half of the byte: no sign
//               fix-up needed), written in the 128B-swizzled K-major operand layout, then handed to the MMA
//               through a proxy fence + mbarrier.  The factor 16 is removed again, exactly, when the epilogue
//               turns the accumulator into fp32.
//   warps 6-13  epilogue (two warps per TMEM lane quarter, 32 channels each): per group tcgen05.ld,
//               int->float, packed fma with the group's channel scales into the running sum y held in
//               registers; after the last group: * sa[m], bf16, 16-byte stores
#pragma once

#include <cuda_bf16.h>

#include "ptx.cuh"
#include "w8a8_gemm.cuh"

namespace cb200 {

constexpr int kW4Threads = 480;      // 15 warps: producer, MMA issuer A, 4 unpack, 8 epilogue, MMA issuer B
constexpr int kW4TileN = 64;        // output channels per CTA (UMMA N)
constexpr int kW4TileM = 128;       // tokens per CTA (UMMA M)
constexpr int kW4Batch = 1;         // K blocks per batch (one commit per batch)
constexpr int kW4InFlight = 6;      // batches whose tiles / accumulators exist at the same time
constexpr int kW4Issuers = 2;       // MMA-issuing threads (batches alternate between them)
constexpr int kW4TokenSlots = kW4Batch * kW4InFlight;
constexpr int kW4CookedSlots = kW4Batch * kW4InFlight;
constexpr int kW4Accs = kW4Batch * kW4InFlight;
constexpr int kW4PackedSlots = 12;  // packed-weight tiles in flight (4 KB each): covers HBM latency

struct W4A8Params {
    uint32_t m, n, k;
    uint32_t mt;                // token rows loaded per tile: min(128, round_up(m, 16))
    uint32_t blocks_per_group;  // group_size / 128
    uint32_t num_k_blocks;      // k / 128
    const float* sw;            // [k / group_size][n]
    const float* sa;            // [m]
    __nv_bfloat16* d;           // [m][n]
    unsigned* status;
};

struct W4A8Smem {
    static constexpr int kTokenBytes = kW4TileM * 128;   // 16 KB: UMMA A operand
    static constexpr int kCookedBytes = kW4TileN * 128;  //  8 KB: unpacked int8 weights, UMMA B operand
    static constexpr int kPackedBytes = kW4TileN * 64;   //  4 KB: packed weights as loaded
    static constexpr int kTokenRing = 0;
    static constexpr int kCookedRing = kTokenRing + kW4TokenSlots * kTokenBytes;
    static constexpr int kPackedRing = kCookedRing + kW4CookedSlots * kCookedBytes;
    static constexpr int kRingBytes = kPackedRing + kW4PackedSlots * kPackedBytes;
    static constexpr int kScaleSlots = 8;                // per epilogue warp: ring of 32-channel scale rows
    static constexpr int kScaleBytes = 8 * kScaleSlots * 32 * 4;
    // p_full, p_empty [packed]; x_full [token]; c_full [cooked]; batch_done, tmem_empty [in flight]
    static constexpr int kBarriers = 2 * kW4PackedSlots + kW4TokenSlots + kW4CookedSlots + 2 * kW4InFlight;
    static constexpr int kBarrierBytes = kBarriers * 8 + 16;
    static constexpr int kTotalBytes = 1024 + kRingBytes + kScaleBytes + kBarrierBytes;
};

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
    asm("{\n\t"
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

// kOneBlockGroups: the scale group is exactly one 128-wide K block (the common case).  The epilogue then needs no
// int32 group sums and reads the next accumulator from TMEM while it does the arithmetic of the current one.
template <bool kOneBlockGroups>
__global__ void __launch_bounds__(kW4Threads, 1)
w4a8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const W4A8Params p)
{
    using S = W4A8Smem;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    const uint32_t ring = raw_addr + pad;

    float* s_scales = reinterpret_cast<float*>(smem + S::kRingBytes);
    uint64_t* s_bars = reinterpret_cast<uint64_t*>(smem + S::kRingBytes + S::kScaleBytes);
    const uint32_t bar_p_full = smem_u32(s_bars);                   // packed tile landed (TMA bytes)
    const uint32_t bar_p_empty = bar_p_full + kW4PackedSlots * 8;    // an unpack warp has read it
    const uint32_t bar_x_full = bar_p_empty + kW4PackedSlots * 8;    // token tile landed
    const uint32_t bar_c_full = bar_x_full + kW4TokenSlots * 8;      // unpacked tile written
    const uint32_t bar_batch_done = bar_c_full + kW4CookedSlots * 8; // all MMAs of a batch completed
    const uint32_t bar_tmem_empty = bar_batch_done + kW4InFlight * 8;  // epilogue drained a batch's accumulators
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + S::kBarriers);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const int32_t n0 = static_cast<int32_t>(blockIdx.x) * kW4TileN;
    const int32_t m0 = static_cast<int32_t>(blockIdx.y) * kW4TileM;
    const uint32_t num_kb = p.num_k_blocks;
    const uint32_t bpg = p.blocks_per_group;
    const uint32_t unit = bpg < static_cast<uint32_t>(kW4Batch) ? bpg : kW4Batch;  // K blocks per accumulator
    const uint32_t num_batches = (num_kb + kW4Batch - 1) / kW4Batch;
    constexpr uint32_t kTmemCols = 512;  // power of two >= kW4Accs * 64
    static_assert(kW4Accs * kW4TileN <= 512, "TMEM budget");

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int i = 0; i < kW4PackedSlots; ++i) {
            mbar_init(bar_p_full + i * 8, 1);
            mbar_init(bar_p_empty + i * 8, 1);
        }
        for (int i = 0; i < kW4TokenSlots; ++i) {
            mbar_init(bar_x_full + i * 8, 1);
        }
        for (int i = 0; i < kW4CookedSlots; ++i) {
            mbar_init(bar_c_full + i * 8, 1);
        }
        for (int i = 0; i < kW4InFlight; ++i) {
            mbar_init(bar_batch_done + i * 8, 1);
            mbar_init(bar_tmem_empty + i * 8, 8);
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

    // Batch B uses barrier slot B % kW4InFlight; it is the (B / kW4InFlight)-th use of that slot.
    // "the previous user of this slot is done" = wait with the inverted parity (passes at once for the first use).

    if (warp == 0) {
        if (lane == 0) {
            // One thread feeds two rings of different depth: it polls both "slot free" conditions without
            // blocking on either, so the deep packed-weight ring keeps running ahead of the token ring.
            uint32_t kw = 0, kx = 0, idle = 0;
            bool dep_ok = false;
            unsigned long long t0 = 0;
            while (kw < num_kb || kx < num_kb) {
                bool progressed = false;
                if (kw < num_kb) {
                    const uint32_t slot = kw % kW4PackedSlots;
                    if (mbar_test_wait(bar_p_empty + slot * 8, ((kw / kW4PackedSlots) & 1) ^ 1)) {
                        const uint32_t full = bar_p_full + slot * 8;
                        mbar_expect_tx(full, S::kPackedBytes);
                        tma_load_2d(ring + S::kPackedRing + slot * S::kPackedBytes, &tmap_w, full,
                                    static_cast<int32_t>(kw) * 64, n0);
                        ++kw;
                        progressed = true;
                    }
                }
                // Weights and their scales never depend on the kernel launched before this one on the stream; the
                // tokens may.  Under programmatic dependent launch the first token tile therefore waits for that
                // kernel, after the packed-weight ring has been filled.  Everything that reads token-dependent
                // data or writes the output happens after a token tile has landed.
                if (kx == 0 && kw >= (num_kb < kW4PackedSlots ? num_kb : kW4PackedSlots)) {
                    grid_dependency_wait();
                    dep_ok = true;
                }
                if (dep_ok && kx < num_kb) {
                    const uint32_t batch = kx / kW4Batch;
                    const uint32_t bslot = batch % kW4InFlight;
                    if (mbar_test_wait(bar_batch_done + bslot * 8, ((batch / kW4InFlight) & 1) ^ 1)) {
                        const uint32_t slot = kx % kW4TokenSlots;
                        const uint32_t full = bar_x_full + slot * 8;
                        mbar_expect_tx(full, p.mt * 128);
                        tma_load_2d(ring + S::kTokenRing + slot * S::kTokenBytes, &tmap_x, full,
                                    static_cast<int32_t>(kx) * 128, m0);
                        ++kx;
                        progressed = true;
                    }
                }
                if (progressed) {
                    idle = 0;
                    t0 = 0;
                } else if ((++idle & 0x3f) == 0) {
                    if (t0 == 0) {
                        t0 = globaltimer_ns();
                    }
                    if (*s_abort != 0) {
                        break;
                    }
                    if (globaltimer_ns() - t0 > kWaitLimitNs) {
                        *s_abort = 1;
                        atomicMax(p.status, kDevTimeoutProducer);
                        break;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 14) {
        // Two issuing threads take alternate batches: issuing a tcgen05.mma costs its thread ~70 ns, more than
        // an MMA of this small shape runs, so one issuer alone would leave the tensor core idle.
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, false, false, kW4TileM, kW4TileN);
            bool ok = true;
            for (uint32_t batch = (warp == 1 ? 0 : 1); ok && batch < num_batches; batch += kW4Issuers) {
                const uint32_t bslot = batch % kW4InFlight;
                const uint32_t use = batch / kW4InFlight;
                ok = mbar_wait(bar_tmem_empty + bslot * 8, (use & 1) ^ 1, s_abort, p.status, kDevTimeoutMmaTmem);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const uint32_t kb_end = (batch + 1) * kW4Batch < num_kb ? (batch + 1) * kW4Batch : num_kb;
                for (uint32_t kb = batch * kW4Batch; kb < kb_end; ++kb) {
                    const uint32_t slot = kb % kW4TokenSlots;  // token and unpacked rings have the same depth
                    const uint32_t ph = (kb / kW4TokenSlots) & 1;
                    ok = mbar_wait(bar_x_full + slot * 8, ph, s_abort, p.status, kDevTimeoutMma) &&
                         mbar_wait(bar_c_full + slot * 8, ph, s_abort, p.status, kDevTimeoutMma);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t sx_tile = ring + S::kTokenRing + slot * S::kTokenBytes;    // UMMA A operand
                    const uint32_t sw_tile = ring + S::kCookedRing + slot * S::kCookedBytes;  // UMMA B operand
                    const uint32_t in_batch = kb - batch * kW4Batch;
                    const uint32_t acc = bslot * kW4Batch + in_batch / unit;
                    const uint32_t tmem_d = tmem_base + acc * kW4TileN;
                    const uint32_t first = in_batch % unit;  // 0: this K block starts a new accumulator
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t da = make_smem_desc_sw128(sx_tile + j * kUmmaK, 16, 1024);
                        const uint64_t db = make_smem_desc_sw128(sw_tile + j * kUmmaK, 16, 1024);
                        umma_i8<1>(tmem_d, da, db, idesc, (first | j) != 0 ? 1u : 0u);
                    }
                }
                if (!ok) {
                    break;
                }
                umma_commit<1>(bar_batch_done + bslot * 8);  // tiles free + accumulators complete, one signal
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ------------------------------------------------------- unpack warps (2..5)
        // Warp u of the four handles the K blocks kb = u, u+4, ... on its own (eight independent 16-byte
        // chunks per lane: plenty of instruction-level parallelism, one fence and one arrival per block).
        // Lane l, step i works on row = i*8 + l/4, packed chunk c = l%4.
        const uint32_t u = warp - 2;
        // the packed tile was loaded with the 64-byte TMA swizzle: 16-byte chunk c of row r sits at
        // chunk c ^ ((r >> 1) & 3); the operand tile uses the 128-byte swizzle: chunk j at j ^ (r & 7)
        const uint32_t c = lane & 3;
        const uint32_t rsub = lane >> 2;  // 0..7: row inside a group of eight (= row & 7)
        for (uint32_t kb = u; kb < num_kb; kb += 4) {
            const uint32_t ps = kb % kW4PackedSlots, pph = (kb / kW4PackedSlots) & 1;
            const uint32_t cs = kb % kW4CookedSlots;
            const uint32_t batch = kb / kW4Batch;
            const uint32_t bslot = batch % kW4InFlight, buse = batch / kW4InFlight;
            bool ok = mbar_wait(bar_p_full + ps * 8, pph, s_abort, p.status, kDevTimeoutConvert) &&
                      mbar_wait(bar_batch_done + bslot * 8, (buse & 1) ^ 1, s_abort, p.status, kDevTimeoutConvert);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            const uint8_t* packed = smem + S::kPackedRing + ps * S::kPackedBytes;
            uint8_t* cooked = smem + S::kCookedRing + cs * S::kCookedBytes;
            uint4 q[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) {
                const uint32_t row = i * 8 + rsub;
                q[i] = *reinterpret_cast<const uint4*>(packed + row * 64 + ((c ^ ((row >> 1) & 3)) << 4));
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_p_empty + ps * 8);  // the packed tile is in registers: its slot can be refilled
            }
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) {
                const uint32_t row = i * 8 + rsub;
                const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
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
                *reinterpret_cast<uint4*>(crow + (((2 * c + 1) ^ rsub) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
            }
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_c_full + cs * 8);
            }
        }
    } else {
        // ------------------------------------------------------- epilogue warps 6..13
        const uint32_t ew = warp - 6;          // 0..7
        const uint32_t quad = warp & 3;        // TMEM lane quarter this warp may read
        const uint32_t half = ew >> 2;         // which 32 of the 64 channels
        const uint32_t row = quad * 32 + lane;
        const uint32_t mrow = static_cast<uint32_t>(m0) + row;
        const uint32_t col0 = static_cast<uint32_t>(n0) + half * 32;
        const uint32_t groups = num_kb / bpg;
        const bool warp_has_rows = static_cast<uint32_t>(m0) + quad * 32 < p.m;  // else: only hand buffers back
        float* sbuf = s_scales + ew * (S::kScaleSlots * 32);  // ring of scale rows, one float per lane
        unsigned long long y2[16];  // running sums of this thread's 32 channels, two fp32 per register
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            y2[i] = 0ull;
        }
        // Channel scales stream from global memory into the ring with cp.async, kAhead groups ahead of their
        // use, so that their latency never sits on the per-group critical path.
        constexpr uint32_t kAhead = 6;
        const uint32_t scol = col0 + lane;
        const bool scol_ok = scol < p.n;
        for (uint32_t i = 0; i < static_cast<uint32_t>(S::kScaleSlots); ++i) {
            sbuf[i * 32 + lane] = 0.0f;
        }
        __syncwarp();
        auto fetch_scale = [&](uint32_t g) {
            if (g < groups && scol_ok) {
                const uint32_t dst = smem_u32(sbuf + (g % S::kScaleSlots) * 32 + lane);
                const float* src = p.sw + static_cast<size_t>(g) * p.n + scol;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        for (uint32_t g = 0; g < kAhead; ++g) {
            fetch_scale(g);
        }
        bool ok = true;
        if constexpr (kOneBlockGroups) {
            static_assert(kW4Batch == 1, "one accumulator per batch");
            // Batch b is K block b is scale group b.  Two register sets alternate: while the sums of batch b are
            // updated from one set, the TMEM read of batch b+1 into the other set is in flight.
            uint32_t ra[32], rb[32];
            auto acquire = [&](uint32_t batch, uint32_t(&r)[32]) -> bool {
                const uint32_t bslot = batch % kW4InFlight, buse = batch / kW4InFlight;
                bool got = mbar_wait(bar_batch_done + bslot * 8, buse & 1, s_abort, p.status, kDevTimeoutEpilogue);
                got = __all_sync(0xffffffffu, got);
                if (got) {
                    tcgen05_fence_after();
                    if (warp_has_rows) {
                        tmem_ld_32x32b_x32(tmem_base + bslot * kW4TileN + half * 32 + ((quad * 32u) << 16), r);
                    }
                }
                return got;
            };
            // the read into r has been issued: wait for it, hand the accumulator back, return with r valid
            auto settle = [&](uint32_t batch, uint32_t(&r)[32]) {
                tmem_ld_wait_x32(r);
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_tmem_empty + (batch % kW4InFlight) * 8);
                }
            };
            auto consume = [&](uint32_t batch, const uint32_t(&r)[32]) {
                fetch_scale(batch + kAhead);
                asm volatile("cp.async.wait_group %0;" ::"n"(kAhead) : "memory");  // this group's scales landed
                __syncwarp();
                if (warp_has_rows) {
                    // |16 * acc| <= 16 * 128 * 128 * 8 = 2^21
                    const ulonglong2* sc = reinterpret_cast<const ulonglong2*>(sbuf + (batch % S::kScaleSlots) * 32);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const ulonglong2 s4 = sc[v];  // scales of channels 4v .. 4v+3
                        scaled_accumulate_pair(y2[2 * v], r[4 * v], r[4 * v + 1], s4.x);
                        scaled_accumulate_pair(y2[2 * v + 1], r[4 * v + 2], r[4 * v + 3], s4.y);
                    }
                }
            };
            ok = num_batches == 0 || acquire(0, ra);
            for (uint32_t batch = 0; ok && batch < num_batches; batch += 2) {
                settle(batch, ra);
                if (batch + 1 < num_batches) {
                    ok = acquire(batch + 1, rb);
                    if (!ok) {
                        break;
                    }
                }
                consume(batch, ra);
                if (batch + 1 >= num_batches) {
                    break;
                }
                settle(batch + 1, rb);
                if (batch + 2 < num_batches) {
                    ok = acquire(batch + 2, ra);
                    if (!ok) {
                        break;
                    }
                }
                consume(batch + 1, rb);
            }
        } else {
            int32_t isum[32];  // int32 sum of a group that spans several K blocks (exact)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                isum[i] = 0;
            }
            const uint32_t accs_per_batch = kW4Batch / unit;
            uint32_t g = 0;             // group whose scale the next finished accumulator needs
            uint32_t kb_in_group = 0;   // K blocks of group g already summed
            for (uint32_t batch = 0; ok && batch < num_batches; ++batch) {
                const uint32_t bslot = batch % kW4InFlight, buse = batch / kW4InFlight;
                ok = mbar_wait(bar_batch_done + bslot * 8, buse & 1, s_abort, p.status, kDevTimeoutEpilogue);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const uint32_t kb0 = batch * kW4Batch;
                const uint32_t kbs_here = kb0 + kW4Batch <= num_kb ? kW4Batch : num_kb - kb0;
                for (uint32_t a = 0; a < accs_per_batch && a * unit < kbs_here; ++a) {
                    const uint32_t kb_acc = (a + 1) * unit <= kbs_here ? unit : kbs_here - a * unit;
                    const bool group_ends = kb_in_group + kb_acc == bpg;
                    if (group_ends) {
                        fetch_scale(g + kAhead);
                        asm volatile("cp.async.wait_group %0;" ::"n"(kAhead) : "memory");  // group g's scales landed
                        __syncwarp();
                    }
                    if (warp_has_rows) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(
                            tmem_base + (bslot * kW4Batch + a) * kW4TileN + half * 32 + ((quad * 32u) << 16), r);
                        tmem_ld_wait();
                        if (bpg == 1) {
                            // one 128-wide K block per group: |16 * acc| <= 16 * 128 * 128 * 8 = 2^21
                            const ulonglong2* sc = reinterpret_cast<const ulonglong2*>(sbuf + (g % S::kScaleSlots) * 32);
    #pragma unroll
                            for (int v = 0; v < 8; ++v) {
                                const ulonglong2 s4 = sc[v];  // scales of channels 4v .. 4v+3
                                scaled_accumulate_pair(y2[2 * v], r[4 * v], r[4 * v + 1], s4.x);
                                scaled_accumulate_pair(y2[2 * v + 1], r[4 * v + 2], r[4 * v + 3], s4.y);
                            }
                        } else {
    #pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                isum[i] += static_cast<int32_t>(r[i]);
                            }
                            if (group_ends) {
                                const ulonglong2* sc = reinterpret_cast<const ulonglong2*>(sbuf + (g % S::kScaleSlots) * 32);
    #pragma unroll
                                for (int v = 0; v < 8; ++v) {
                                    const ulonglong2 s4 = sc[v];
                                    // the sums are multiples of 16: the conversion and the scaling by 1/16 are exact
                                    fma_pair(y2[2 * v], __int2float_rn(isum[4 * v]) * 0.0625f,
                                             __int2float_rn(isum[4 * v + 1]) * 0.0625f, s4.x);
                                    fma_pair(y2[2 * v + 1], __int2float_rn(isum[4 * v + 2]) * 0.0625f,
                                             __int2float_rn(isum[4 * v + 3]) * 0.0625f, s4.y);
                                    isum[4 * v] = isum[4 * v + 1] = isum[4 * v + 2] = isum[4 * v + 3] = 0;
                                }
                            }
                        }
                    }
                    kb_in_group += kb_acc;
                    if (group_ends) {
                        kb_in_group = 0;
                        ++g;
                    }
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_tmem_empty + bslot * 8);
                }
            }
        }
        if (ok && mrow < p.m) {
            float y[32];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                unpack_pair(y2[i], y[2 * i], y[2 * i + 1]);
            }
            const float sa = __ldg(p.sa + mrow);
            __nv_bfloat16* drow = p.d + static_cast<size_t>(mrow) * p.n + col0;
            if ((p.n & 7u) == 0 && col0 + 32 <= p.n) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint32_t packed[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(__fmul_rn(y[v * 8 + e * 2], sa),
                                                                       __fmul_rn(y[v * 8 + e * 2 + 1], sa));
                        packed[e] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(drow + v * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (col0 + i < p.n) {
                        drow[i] = __float2bfloat16_rn(__fmul_rn(y[i], sa));
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
