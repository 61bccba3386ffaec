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
// Warp roles (14 warps):
//   warp 0      TMA producer: packed weight tile (64 x 64 B) + token tile (mt x 128 B) per 128-wide K block
//   warp 1      MMA issuer (tcgen05.mma.kind::i8, 128 x 64 x 32); eight int32 accumulators in TMEM, one per group
//               in flight, so the issuer never waits for the epilogue's hand-back
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

constexpr int kW4Threads = 448;
constexpr int kW4TileN = 64;       // output channels per CTA (UMMA N)
constexpr int kW4TileM = 128;      // tokens per CTA (UMMA M)
constexpr int kW4Stages = 7;
constexpr int kW4Accs = 8;        // group accumulators in TMEM (8 x 64 columns): hides the MMA<->epilogue hand-off latency

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
    static constexpr int kStageBytes = kTokenBytes + kCookedBytes + kPackedBytes;  // 28 KB
    static constexpr int kRingBytes = kW4Stages * kStageBytes;
    static constexpr int kScaleSlots = 8;                // per epilogue warp: ring of 32-channel scale rows
    static constexpr int kScaleBytes = 8 * kScaleSlots * 32 * 4;
    static constexpr int kBarrierBytes = (3 * kW4Stages + 2 * kW4Accs) * 8 + 16;
    static constexpr int kTotalBytes = 1024 + kRingBytes + kScaleBytes + kBarrierBytes;
};

// Exact fp32 value of x/16 for an int32 x with |x| < 2^22, without the conversion unit:
// 0x49400000 is 1.5 * 2^19, whose unit in the last place is 1/16; adding x to the bit pattern yields the
// float 1.5 * 2^19 + x/16, and subtracting 1.5 * 2^19 again is exact.  Two values per packed subtract.
// (The accumulators hold 16 times the true sums: see the unpack warps.)
__device__ __forceinline__ void int2float_pair(uint32_t x0, uint32_t x1, float& f0, float& f1)
{
    const float t0 = __uint_as_float(x0 + 0x49400000u);
    const float t1 = __uint_as_float(x1 + 0x49400000u);
    asm("{\n\t"
        ".reg .b64 rt, rc;\n\t"
        "mov.b64 rt, {%2, %3};\n\t"
        "mov.b64 rc, {%4, %4};\n\t"
        "add.rn.f32x2 rt, rt, rc;\n\t"
        "mov.b64 {%0, %1}, rt;\n\t"
        "}\n"
        : "=f"(f0), "=f"(f1)
        : "f"(t0), "f"(t1), "f"(-786432.0f));
}

// y += a * s on two independent lanes: one packed IEEE fused multiply-add
__device__ __forceinline__ void fma2(float& y0, float& y1, float a0, float a1, float s0, float s1)
{
    asm("{\n\t"
        ".reg .b64 ra, rs, ry;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rs, {%4, %5};\n\t"
        "mov.b64 ry, {%0, %1};\n\t"
        "fma.rn.f32x2 ry, ra, rs, ry;\n\t"
        "mov.b64 {%0, %1}, ry;\n\t"
        "}\n"
        : "+f"(y0), "+f"(y1)
        : "f"(a0), "f"(a1), "f"(s0), "f"(s1));
}

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
    const uint32_t bar_full = smem_u32(s_bars);               // TMA landed (tx bytes)
    const uint32_t bar_cooked = bar_full + kW4Stages * 8;     // an unpack warp finished the stage
    const uint32_t bar_empty = bar_cooked + kW4Stages * 8;    // MMAs that read the stage completed
    const uint32_t bar_tmem_full = bar_empty + kW4Stages * 8;
    const uint32_t bar_tmem_empty = bar_tmem_full + kW4Accs * 8;
    uint32_t* s_tmem_ptr = reinterpret_cast<uint32_t*>(s_bars + 3 * kW4Stages + 2 * kW4Accs);
    volatile uint32_t* s_abort = s_tmem_ptr + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const int32_t n0 = static_cast<int32_t>(blockIdx.x) * kW4TileN;
    const int32_t m0 = static_cast<int32_t>(blockIdx.y) * kW4TileM;
    const uint32_t num_kb = p.num_k_blocks;
    const uint32_t bpg = p.blocks_per_group;
    constexpr uint32_t kTmemCols = kW4Accs * kW4TileN;

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int s = 0; s < kW4Stages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_cooked + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < kW4Accs; ++a) {
            mbar_init(bar_tmem_full + a * 8, 1);
            mbar_init(bar_tmem_empty + a * 8, 8);
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
    const uint32_t stage_tx = S::kPackedBytes + p.mt * 128;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, s_abort, p.status, kDevTimeoutProducer)) {
                    break;
                }
                const uint32_t base = ring + stage * S::kStageBytes;
                const uint32_t full = bar_full + stage * 8;
                mbar_expect_tx(full, stage_tx);
                tma_load_2d(base, &tmap_x, full, static_cast<int32_t>(kb) * 128, m0);
                tma_load_2d(base + S::kTokenBytes + S::kCookedBytes, &tmap_w, full, static_cast<int32_t>(kb) * 64, n0);
                if (++stage == kW4Stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kAccS32, kFmtS8, kFmtS8, false, false, kW4TileM, kW4TileN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t kb = 0; ok && kb < num_kb; ++kb) {
                const uint32_t in_group = kb % bpg;
                if (in_group == 0) {
                    ok = mbar_wait(bar_tmem_empty + acc * 8, acc_phase ^ 1, s_abort, p.status, kDevTimeoutMmaTmem);
                    if (!ok) {
                        break;
                    }
                }
                ok = mbar_wait(bar_full + stage * 8, phase, s_abort, p.status, kDevTimeoutMma) &&
                     mbar_wait(bar_cooked + stage * 8, phase, s_abort, p.status, kDevTimeoutMma);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const uint32_t sx_tile = ring + stage * S::kStageBytes;  // tokens: UMMA A operand
                const uint32_t sw_tile = sx_tile + S::kTokenBytes;       // unpacked weights: UMMA B operand
                const uint32_t tmem_d = tmem_base + acc * kW4TileN;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint64_t da = make_smem_desc_sw128(sx_tile + j * kUmmaK, 16, 1024);
                    const uint64_t db = make_smem_desc_sw128(sw_tile + j * kUmmaK, 16, 1024);
                    umma_i8<1>(tmem_d, da, db, idesc, (in_group | j) != 0 ? 1u : 0u);
                }
                umma_commit<1>(bar_empty + stage * 8);
                if (in_group == bpg - 1) {
                    umma_commit<1>(bar_tmem_full + acc * 8);  // this group's accumulator is complete
                    if (++acc == kW4Accs) {
                        acc = 0;
                        acc_phase ^= 1;
                    }
                }
                if (++stage == kW4Stages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ------------------------------------------------------- unpack warps
        // Warp u of the four handles the K blocks kb = u, u+4, ... on its own (eight independent 16-byte
        // chunks per lane: plenty of instruction-level parallelism, one fence and one arrival per block).
        // Lane l, step i works on row = i*8 + l/4, packed chunk c = l%4.
        const uint32_t u = warp - 2;
        // the packed tile was loaded with the 64-byte TMA swizzle: 16-byte chunk c of row r sits at
        // chunk c ^ ((r >> 1) & 3); the operand tile uses the 128-byte swizzle: chunk j at j ^ (r & 7)
        const uint32_t c = lane & 3;
        const uint32_t rsub = lane >> 2;  // 0..7: row inside a group of eight (= row & 7)
        for (uint32_t kb = u; kb < num_kb; kb += 4) {
            const uint32_t stage = kb % kW4Stages;
            const uint32_t phase = (kb / kW4Stages) & 1;
            bool ok = mbar_wait(bar_full + stage * 8, phase, s_abort, p.status, kDevTimeoutConvert);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            uint8_t* base = smem + stage * S::kStageBytes;
            const uint8_t* packed = base + S::kTokenBytes + S::kCookedBytes;
            uint8_t* cooked = base + S::kTokenBytes;
            uint4 q[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) {
                const uint32_t row = i * 8 + rsub;
                q[i] = *reinterpret_cast<const uint4*>(packed + row * 64 + ((c ^ ((row >> 1) & 3)) << 4));
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
                mbar_arrive(bar_cooked + stage * 8);
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
        float y[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            y[i] = 0.0f;
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
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t g = 0; g < groups; ++g) {
            fetch_scale(g + kAhead);
            ok = mbar_wait(bar_tmem_full + acc * 8, acc_phase, s_abort, p.status, kDevTimeoutEpilogue);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                break;
            }
            tcgen05_fence_after();
            asm volatile("cp.async.wait_group %0;" ::"n"(kAhead) : "memory");  // this group's scales landed
            __syncwarp();
            if (warp_has_rows) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_base + acc * kW4TileN + half * 32 + ((quad * 32u) << 16), r);
                tmem_ld_wait();
                const float4* sc4 = reinterpret_cast<const float4*>(sbuf + (g % S::kScaleSlots) * 32);
                if (bpg == 1) {
                    // one 128-wide K block per group: |16 * acc| <= 16 * 128 * 128 * 8 = 2^21
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 s4 = sc4[v];
                        float f0, f1, f2, f3;
                        int2float_pair(r[4 * v], r[4 * v + 1], f0, f1);
                        int2float_pair(r[4 * v + 2], r[4 * v + 3], f2, f3);
                        fma2(y[4 * v], y[4 * v + 1], f0, f1, s4.x, s4.y);
                        fma2(y[4 * v + 2], y[4 * v + 3], f2, f3, s4.z, s4.w);
                    }
                } else {
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 s4 = sc4[v];
                        fma2(y[4 * v], y[4 * v + 1], __int2float_rn(static_cast<int>(r[4 * v])) * 0.0625f,
                             __int2float_rn(static_cast<int>(r[4 * v + 1])) * 0.0625f, s4.x, s4.y);
                        fma2(y[4 * v + 2], y[4 * v + 3], __int2float_rn(static_cast<int>(r[4 * v + 2])) * 0.0625f,
                             __int2float_rn(static_cast<int>(r[4 * v + 3])) * 0.0625f, s4.z, s4.w);
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_tmem_empty + acc * 8);
            }
            if (++acc == kW4Accs) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (ok && mrow < p.m) {
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
