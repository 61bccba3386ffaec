// Per-token int8 quantisation of activations: the step in front of the W8A8 matmuls (HBM-bound).
//
//   amax[r]  = max_k |x[r,k]|
//   scale[r] = amax[r] / 127                          (fp32, round to nearest)  -> the matmul's per-token scale
//   q[r,k]   = clamp(rint(x[r,k] * (127 / amax[r])), -127, 127)   (one fp32 multiply, round half to even)
//   an all-zero row: scale 0, codes 0
//
// The reference has no device kernel for this step (its examples start from int8 data made on the host:
// examples/12_quant_matmul/gen_data.py); the outputs are exactly what cb200_quant_matmul and the grouped entry
// points read: q [rows][k] int8 with row pitch k, scale [rows] fp32.
//
// One warp per row, rows strided over the grid.  A lane works on 16 consecutive elements per step (fp32: four
// 16-byte loads, bf16: two) and stores their 16 codes with one 16-byte store.
//   quant_int8_staged_kernel  rows of at most 28 KB: the whole row comes into the warp's own shared-memory slot
//                             with ONE bulk copy (two slots per warp when a row is at most 14 KB: the next row is
//                             in flight while this one is worked on), both passes read shared memory.  Eight
//                             warps keep up to 224 KB of loads outstanding per SM; with plain loads a warp had
//                             1 KB outstanding and the kernel ran at 0.6 of the HBM copy rate.
//   quant_int8_wide_kernel    rows of 28 to 112 KB: one CTA per row, a segment per warp staged the same way.
//   quant_int8_kernel         any row length: the row is read twice with plain loads, the second time from L2
//                             where the first pass left it.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace cb200 {

constexpr int kQuantInt8Threads = 256;
constexpr uint32_t kQuantInt8StageBytes = 28u * 1024u;  // shared memory per warp

template <bool kBf16In>
__device__ __forceinline__ void quant_int8_load16(const void* row, uint32_t c0, float (&v)[16])
{
    if constexpr (kBf16In) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(row) + c0);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 raw = src[h];
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[h * 8 + 2 * i] = __uint_as_float(w[i] << 16);
                v[h * 8 + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
        }
    } else {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(row) + c0);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const float4 raw = src[h];
            v[h * 4] = raw.x;
            v[h * 4 + 1] = raw.y;
            v[h * 4 + 2] = raw.z;
            v[h * 4 + 3] = raw.w;
        }
    }
}

// amax of 16 values, and their 16 codes
__device__ __forceinline__ float quant_int8_amax16(const float (&v)[16], float amax)
{
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        amax = fmaxf(amax, fabsf(v[i]));
    }
    return amax;
}

// (c << 16) | (sat8(a) << 8) | sat8(b): two int32 packed as saturated int8 below the low half of c
__device__ __forceinline__ uint32_t pack_sat_s8(int a, int b, uint32_t c)
{
    uint32_t d;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint4 quant_int8_codes16(const float (&v)[16], float inv)
{
    uint32_t out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        int code[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            code[b] = __float2int_rn(__fmul_rn(v[w * 4 + b], inv));
        }
        // |x * inv| <= 127 (1 + 2^-23): the rounded value never leaves [-127, 127]; the saturating pack is the clamp
        // for anything that is not a number
        out[w] = pack_sat_s8(code[1], code[0], pack_sat_s8(code[3], code[2], 0u));
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// Rows of at most kQuantInt8StageBytes bytes.  Dynamic shared memory: 8 warps x kQuantInt8StageBytes + barriers.
template <bool kBf16In>
__global__ void __launch_bounds__(kQuantInt8Threads, 1)
quant_int8_staged_kernel(const void* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, uint32_t rows,
                         uint32_t k, uint64_t x_pitch, unsigned* status)
{
    extern __shared__ __align__(128) uint8_t quant_smem[];
    constexpr uint32_t kWarps = kQuantInt8Threads / 32;
    constexpr uint32_t kElemBytes = kBf16In ? 2 : 4;
    uint64_t* bars = reinterpret_cast<uint64_t*>(quant_smem + kWarps * kQuantInt8StageBytes);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(bars + 2 * kWarps);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_bytes = k * kElemBytes;
    const uint32_t slots = 2 * row_bytes <= kQuantInt8StageBytes ? 2u : 1u;
    const uint32_t slot_bytes = kQuantInt8StageBytes / slots;
    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (uint32_t i = 0; i < 2 * kWarps; ++i) {
            mbar_init(smem_u32(bars + i), 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    const uint32_t warps_per_grid = gridDim.x * kWarps;
    const uint32_t stage = smem_u32(quant_smem) + warp * kQuantInt8StageBytes;
    const uint8_t* stage_ptr = quant_smem + warp * kQuantInt8StageBytes;
    const uint32_t bar0 = smem_u32(bars + 2 * warp);
    auto fetch = [&](uint32_t r, uint32_t slot) {  // lane 0 only
        const uint8_t* src = static_cast<const uint8_t*>(x) + static_cast<uint64_t>(r) * x_pitch * kElemBytes;
        mbar_expect_tx(bar0 + slot * 8, row_bytes);
        bulk_load(stage + slot * slot_bytes, src, row_bytes, bar0 + slot * 8);
    };
    uint32_t r = blockIdx.x * kWarps + warp;
    if (r < rows && lane == 0) {
        fetch(r, 0);
    }
    uint32_t slot = 0, phase[2] = {0, 0};
    for (; r < rows; r += warps_per_grid) {
        const uint32_t next = r + warps_per_grid;
        if (slots == 2 && next < rows && lane == 0) {
            fetch(next, slot ^ 1);  // (that slot's previous row was worked off before the __syncwarp below)
        }
        bool ok = mbar_wait(bar0 + slot * 8, phase[slot], s_abort, status, kDevTimeoutProducer);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            break;
        }
        phase[slot] ^= 1;
        const uint8_t* row = stage_ptr + slot * slot_bytes;
        float amax = 0.0f;
        for (uint32_t c0 = lane * 16; c0 < k; c0 += 32 * 16) {
            float v[16];
            quant_int8_load16<kBf16In>(row, c0, v);
            amax = quant_int8_amax16(v, amax);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        }
        const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        if (lane == 0) {
            scale[r] = __fdiv_rn(amax, 127.0f);
        }
        int8_t* qr = q + static_cast<uint64_t>(r) * k;
        for (uint32_t c0 = lane * 16; c0 < k; c0 += 32 * 16) {
            float v[16];
            quant_int8_load16<kBf16In>(row, c0, v);
            *reinterpret_cast<uint4*>(qr + c0) = quant_int8_codes16(v, inv);
        }
        __syncwarp();  // every lane is done with this slot
        if (slots == 2) {
            slot ^= 1;
        } else if (next < rows && lane == 0) {
            fetch(next, 0);
        }
    }
}

// Rows of 28 KB to 112 KB: one CTA per row, the row cut into eight segments of `seg` elements (a multiple of 16, at
// most half a warp's slot), one per warp; every warp keeps the next row's segment in flight in its second slot.
// The row's maximum goes through shared memory (one CTA-wide barrier per row).  Same dynamic shared memory.
template <bool kBf16In>
__global__ void __launch_bounds__(kQuantInt8Threads, 1)
quant_int8_wide_kernel(const void* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, uint32_t rows,
                       uint32_t k, uint64_t x_pitch, uint32_t seg, unsigned* status)
{
    extern __shared__ __align__(128) uint8_t quant_smem[];
    constexpr uint32_t kWarps = kQuantInt8Threads / 32;
    constexpr uint32_t kElemBytes = kBf16In ? 2 : 4;
    constexpr uint32_t kSlotBytes = kQuantInt8StageBytes / 2;
    uint64_t* bars = reinterpret_cast<uint64_t*>(quant_smem + kWarps * kQuantInt8StageBytes);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(bars + 2 * kWarps);
    __shared__ float s_part[2][kWarps];  // the warps' partial maxima, one set per slot
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (uint32_t i = 0; i < 2 * kWarps; ++i) {
            mbar_init(smem_u32(bars + i), 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    const uint32_t c_begin = warp * seg;                                   // this warp's elements of every row
    const uint32_t len = c_begin < k ? (k - c_begin < seg ? k - c_begin : seg) : 0u;
    const uint32_t stage = smem_u32(quant_smem) + warp * kQuantInt8StageBytes;
    const uint8_t* stage_ptr = quant_smem + warp * kQuantInt8StageBytes;
    const uint32_t bar0 = smem_u32(bars + 2 * warp);
    auto fetch = [&](uint32_t r, uint32_t slot) {  // lane 0 only, len != 0
        const uint8_t* src =
            static_cast<const uint8_t*>(x) + (static_cast<uint64_t>(r) * x_pitch + c_begin) * kElemBytes;
        mbar_expect_tx(bar0 + slot * 8, len * kElemBytes);
        bulk_load(stage + slot * kSlotBytes, src, len * kElemBytes, bar0 + slot * 8);
    };
    uint32_t r = blockIdx.x;
    if (r < rows && lane == 0 && len != 0) {
        fetch(r, 0);
    }
    uint32_t slot = 0, phase0 = 0, phase1 = 0;
    // (every thread of the CTA makes the same number of trips and meets the barrier in each of them)
    for (; r < rows; r += gridDim.x) {
        const uint32_t next = r + gridDim.x;
        if (next < rows && lane == 0 && len != 0) {
            fetch(next, slot ^ 1);  // (that slot's previous row was worked off before the __syncwarp below)
        }
        const uint8_t* row = stage_ptr + slot * kSlotBytes;
        float amax = 0.0f;
        bool failed = false;
        if (len != 0) {
            const bool got = mbar_wait(bar0 + slot * 8, slot == 0 ? phase0 : phase1, s_abort, status, kDevTimeoutProducer);
            failed = !got;
            if (slot == 0) {
                phase0 ^= 1;
            } else {
                phase1 ^= 1;
            }
            if (got) {
                for (uint32_t c0 = lane * 16; c0 < len; c0 += 32 * 16) {
                    float v[16];
                    quant_int8_load16<kBf16In>(row, c0, v);
                    amax = quant_int8_amax16(v, amax);
                }
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        }
        if (lane == 0) {
            s_part[slot][warp] = amax;
        }
        if (__syncthreads_or(failed ? 1 : 0) != 0) {
            break;  // (the barrier hands every thread the same answer: all leave in the same trip)
        }
#pragma unroll
        for (uint32_t w = 0; w < kWarps; ++w) {
            amax = fmaxf(amax, s_part[slot][w]);
        }
        const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        if (threadIdx.x == 0) {
            scale[r] = __fdiv_rn(amax, 127.0f);
        }
        int8_t* qr = q + static_cast<uint64_t>(r) * k + c_begin;
        for (uint32_t c0 = lane * 16; c0 < len; c0 += 32 * 16) {
            float v[16];
            quant_int8_load16<kBf16In>(row, c0, v);
            *reinterpret_cast<uint4*>(qr + c0) = quant_int8_codes16(v, inv);
        }
        __syncwarp();  // every lane is done with this slot
        slot ^= 1;
    }
}

// k is a multiple of 16; x rows start on 16-byte boundaries (base and pitch), q likewise.
template <bool kBf16In>
__global__ void __launch_bounds__(kQuantInt8Threads)
quant_int8_kernel(const void* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, uint32_t rows,
                  uint32_t k, uint64_t x_pitch)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const uint32_t warp_id = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    constexpr uint32_t kElemBytes = kBf16In ? 2 : 4;
    for (uint32_t r = warp_id; r < rows; r += warps_per_grid) {
        const uint8_t* xr = static_cast<const uint8_t*>(x) + static_cast<uint64_t>(r) * x_pitch * kElemBytes;
        float amax = 0.0f;
        for (uint32_t c0 = lane * 16; c0 < k; c0 += 32 * 16) {
            float v[16];
            quant_int8_load16<kBf16In>(xr, c0, v);
            amax = quant_int8_amax16(v, amax);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        }
        const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        if (lane == 0) {
            scale[r] = __fdiv_rn(amax, 127.0f);
        }
        int8_t* qr = q + static_cast<uint64_t>(r) * k;
        for (uint32_t c0 = lane * 16; c0 < k; c0 += 32 * 16) {
            float v[16];
            quant_int8_load16<kBf16In>(xr, c0, v);
            *reinterpret_cast<uint4*>(qr + c0) = quant_int8_codes16(v, inv);
        }
    }
}

}  // namespace cb200
