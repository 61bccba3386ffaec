// MX (OCP microscaling) quantisation on the device: fp32 or bf16 rows -> E4M3 / E2M1 element codes plus one E8M0
// scale byte per 32 contiguous elements, written in the layout cb200_mx_matmul reads (elements [rows][k], E2M1 two
// per byte with the even index in bits 0-3; scales [rows][KS], KS = ceil(k/32) rounded up to even, padding 2^0).
//
// The rule is the reference's (examples/53_ascend950_fp8_mx_matmul/gen_data.py:186-265,
// examples/54_ascend950_fp4_mx_matmul/gen_data.py:46-95, tests/optest/tests/mx_golden.py:177-221):
//   shared exponent = floor(log2(max |x| of the block)) - emax   (emax 8 / 2), clamped to [-128, 127], 0 for a block
//                     whose maximum is below 1e-12;
//   element         = x / 2^exponent, clamped to +-448 / +-6, snapped to the nearest representable value, a tie
//                     going to the smaller magnitude.
// The reference quantises on the host; on the device it does so inside its experimental fused MoE epilogue
// (experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant).  HBM-bound: 4 (or 2) bytes read and
// about one byte written per element; a warp handles 128 consecutive elements (four blocks) per step with 16-byte
// loads and 4-byte stores.
//
// mx_quantize_staged_kernel serves the aligned case (k a multiple of 32, rows on 16-byte boundaries):
// one warp per row, the whole row brought into the warp's shared-memory slot by ONE bulk copy (the next row in
// flight meanwhile when two fit), a lane working on 16 consecutive elements (half a block) per step, the codes made
// by the conversion instructions (cvt.rn.satfinite.e4m3x2 / e2m1x2) from values shifted towards zero by one part in
// 4096, which turns the instructions' nearest-even into the reference's tie rule (see the kernel).
// mx_quantize_kernel (plain loads, 4 elements per lane and step, any k and pitch) had 256 bytes of loads outstanding
// per warp and ran at 0.2 of the HBM copy rate on 32768 x 7168 bf16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "ptx.cuh"

namespace cb200 {

// |v| (finite, <= 448) -> E4M3 magnitude code, nearest with ties to the smaller magnitude.
__device__ __forceinline__ uint32_t e4m3_code_of(float mag)
{
    // normal codes: (1 + m/8) * 2^(e-7), e = 1..15 (0x7E = 448 is the largest); subnormal: m/8 * 2^-6
    if (mag < 0.015625f) {  // below 2^-6: the grid is multiples of 2^-9
        const float t = mag * 512.0f;               // exact
        float lower = floorf(t);
        if (t - lower > 0.5f) {
            lower += 1.0f;                          // (a carry to 8 is the smallest normal, code 0x08)
        }
        return static_cast<uint32_t>(lower);
    }
    const uint32_t bits = __float_as_uint(mag);
    const uint32_t low = bits & 0xFFF00000u;        // mantissa cut to 3 bits: the grid point at or below
    const float lower = __uint_as_float(low);
    const float ulp = __uint_as_float((bits & 0x7F800000u) - (3u << 23));  // 2^(exponent - 3)
    uint32_t code = ((low >> 23) - 120u) << 3 | ((low >> 20) & 7u);        // exponent bias 127 -> 7
    if (mag - lower > 0.5f * ulp) {
        code += 1;                                  // next grid point (mantissa carry runs into the exponent)
    }
    return code > 0x7Eu ? 0x7Eu : code;
}

// |v| (<= 6) -> E2M1 magnitude code: grid 0, .5, 1, 1.5, 2, 3, 4, 6; a tie goes to the smaller magnitude.
__device__ __forceinline__ uint32_t e2m1_code_of(float mag)
{
    return (mag > 0.25f) + (mag > 0.75f) + (mag > 1.25f) + (mag > 1.75f) + (mag > 2.5f) + (mag > 3.5f) + (mag > 5.0f);
}

template <bool kFp4, bool kBf16In>
__global__ void mx_quantize_kernel(const void* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                   uint32_t rows, uint32_t k, uint64_t x_pitch, uint32_t q_pitch, uint32_t sf_pitch)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const uint32_t warp_id = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t steps_per_row = (sf_pitch * 32u + 127u) / 128u;  // covers the padding scale byte too
    const uint64_t total = static_cast<uint64_t>(rows) * steps_per_row;
    constexpr float kMaxValue = kFp4 ? 6.0f : 448.0f;
    constexpr int kEmax = kFp4 ? 2 : 8;
    for (uint64_t w = warp_id; w < total; w += warps_per_grid) {
        const uint32_t row = static_cast<uint32_t>(w / steps_per_row);
        const uint32_t c0 = static_cast<uint32_t>(w - static_cast<uint64_t>(row) * steps_per_row) * 128u + lane * 4u;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (kBf16In) {
            const __nv_bfloat16* xr = static_cast<const __nv_bfloat16*>(x) + row * x_pitch;
            if (c0 + 4 <= k && ((x_pitch | c0) & 3u) == 0) {
                const uint2 raw = *reinterpret_cast<const uint2*>(xr + c0);
                v[0] = __uint_as_float(raw.x << 16);
                v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
                v[2] = __uint_as_float(raw.y << 16);
                v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
            } else {
                for (int i = 0; i < 4; ++i) {
                    v[i] = c0 + i < k ? __bfloat162float(xr[c0 + i]) : 0.0f;
                }
            }
        } else {
            const float* xr = static_cast<const float*>(x) + row * x_pitch;
            if (c0 + 4 <= k && ((x_pitch | c0) & 3u) == 0) {
                const float4 raw = *reinterpret_cast<const float4*>(xr + c0);
                v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
            } else {
                for (int i = 0; i < 4; ++i) {
                    v[i] = c0 + i < k ? xr[c0 + i] : 0.0f;
                }
            }
        }
        // block maximum: eight lanes hold one block of 32
        float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        int exp = 0;
        if (!(mx < 1e-12f)) {
            exp = static_cast<int>((__float_as_uint(mx) >> 23) & 0xFFu) - 127 - kEmax;
            exp = exp < -128 ? -128 : (exp > 127 ? 127 : exp);
        }
        // 2^exp as a float (2^-127 and 2^-128 are subnormals: bit patterns 0x00400000 and 0x00200000)
        const float scale = exp >= -126 ? __uint_as_float(static_cast<uint32_t>(exp + 127) << 23)
                                        : __uint_as_float(0x00400000u >> (-127 - exp));
        uint32_t codes[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float t = __fdiv_rn(v[i], scale);
            t = fminf(fmaxf(t, -kMaxValue), kMaxValue);
            const float mag = fabsf(t);
            const uint32_t c = kFp4 ? e2m1_code_of(mag) : e4m3_code_of(mag);
            codes[i] = (t < 0.0f && c != 0) ? (c | (kFp4 ? 0x8u : 0x80u)) : c;
        }
        const uint32_t block = c0 >> 5;
        if ((lane & 7u) == 0 && block < sf_pitch) {
            const uint32_t valid_blocks = (k + 31u) >> 5;
            int code = exp + 127;
            code = code < 0 ? 0 : code;
            sf[static_cast<uint64_t>(row) * sf_pitch + block] = block < valid_blocks ? static_cast<uint8_t>(code) : 127;
        }
        if (c0 < k) {
            if (kFp4) {
                uint8_t* qr = q + static_cast<uint64_t>(row) * q_pitch + (c0 >> 1);
                const uint32_t lo = codes[0] | (c0 + 1 < k ? codes[1] << 4 : 0u);
                const uint32_t hi = codes[2] | (c0 + 3 < k ? codes[3] << 4 : 0u);
                if (c0 + 2 < k && (q_pitch & 1u) == 0) {
                    *reinterpret_cast<uint16_t*>(qr) = static_cast<uint16_t>(lo | hi << 8);
                } else {
                    qr[0] = static_cast<uint8_t>(lo);
                    if (c0 + 2 < k) {
                        qr[1] = static_cast<uint8_t>(hi);
                    }
                }
            } else {
                uint8_t* qr = q + static_cast<uint64_t>(row) * q_pitch + c0;
                if (c0 + 4 <= k && (q_pitch & 3u) == 0) {
                    *reinterpret_cast<uint32_t*>(qr) = codes[0] | codes[1] << 8 | codes[2] << 16 | codes[3] << 24;
                } else {
                    for (int i = 0; i < 4 && c0 + i < k; ++i) {
                        qr[i] = static_cast<uint8_t>(codes[i]);
                    }
                }
            }
        }
    }
}

constexpr int kMxQuantThreads = 256;
constexpr uint32_t kMxQuantStageBytes = 28u * 1024u;  // shared memory per warp

// Two scaled values -> two element codes (a in bits 0-7 / 0-3, b above).  The values were moved towards zero by one
// part in 4096 beforehand (see the kernel): the conversion instruction's nearest-even then IS the reference's rule
// (nearest, a tie to the smaller magnitude, saturating), and only -0 is left to put right (zero is always +0).
template <bool kFp4>
__device__ __forceinline__ uint32_t mx_codes2_nudged(float a, float b)
{
    if constexpr (kFp4) {
        uint32_t c = __nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest);
        c = (c & 0x07u) == 0 ? (c & 0xF0u) : c;
        c = (c & 0x70u) == 0 ? (c & 0x0Fu) : c;
        return c;
    } else {
        uint32_t c = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        c = (c & 0x007Fu) == 0 ? (c & 0xFF00u) : c;
        c = (c & 0x7F00u) == 0 ? (c & 0x00FFu) : c;
        return c;
    }
}

// k a multiple of 32; rows of x on 16-byte boundaries; q rows 16-byte aligned.  A row is worked off in segments of
// `seg` elements (a multiple of 512, or k itself when the whole row fits a warp's kMxQuantStageBytes; blocks of 32
// are independent of each other, so a long row is simply several work items).
// Dynamic shared memory: 8 warps x kMxQuantStageBytes + barriers.
template <bool kFp4, bool kBf16In>
__global__ void __launch_bounds__(kMxQuantThreads, 1)
mx_quantize_staged_kernel(const void* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, uint32_t rows,
                          uint32_t k, uint64_t x_pitch, uint32_t seg, unsigned* status)
{
    extern __shared__ __align__(128) uint8_t mxq_smem[];
    constexpr uint32_t kWarps = kMxQuantThreads / 32;
    constexpr uint32_t kElemBytes = kBf16In ? 2 : 4;
    constexpr int kEmax = kFp4 ? 2 : 8;
    uint64_t* bars = reinterpret_cast<uint64_t*>(mxq_smem + kWarps * kMxQuantStageBytes);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(bars + 2 * kWarps);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t slots = 2 * seg * kElemBytes <= kMxQuantStageBytes ? 2u : 1u;
    const uint32_t slot_bytes = kMxQuantStageBytes / slots;
    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (uint32_t i = 0; i < 2 * kWarps; ++i) {
            mbar_init(smem_u32(bars + i), 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    const uint32_t warps_per_grid = gridDim.x * kWarps;
    const uint32_t stage = smem_u32(mxq_smem) + warp * kMxQuantStageBytes;
    const uint8_t* stage_ptr = mxq_smem + warp * kMxQuantStageBytes;
    const uint32_t bar0 = smem_u32(bars + 2 * warp);
    const uint32_t q_pitch = kFp4 ? k / 2 : k;
    const uint32_t sf_pitch = (k / 32 + 1u) & ~1u;  // an even number of scale columns; the odd one out holds 2^0
    const uint32_t segs = (k + seg - 1) / seg;
    const uint32_t items = rows * segs;  // (row, segment) pairs, a row's segments adjacent (the host checks the range)
    auto fetch = [&](uint32_t item, uint32_t slot) {  // lane 0 only
        const uint32_t r = segs == 1 ? item : item / segs;
        const uint32_t c_begin = (item - r * segs) * seg;
        const uint32_t bytes = (k - c_begin < seg ? k - c_begin : seg) * kElemBytes;
        const uint8_t* src =
            static_cast<const uint8_t*>(x) + (static_cast<uint64_t>(r) * x_pitch + c_begin) * kElemBytes;
        mbar_expect_tx(bar0 + slot * 8, bytes);
        bulk_load(stage + slot * slot_bytes, src, bytes, bar0 + slot * 8);
    };
    uint32_t item = blockIdx.x * kWarps + warp;
    if (item < items && lane == 0) {
        fetch(item, 0);
    }
    uint32_t slot = 0, phase0 = 0, phase1 = 0;
    for (; item < items; item += warps_per_grid) {
        const uint32_t next = item + warps_per_grid;  // (items + warps_per_grid < 2^32: checked by the host)
        if (slots == 2 && next < items && lane == 0) {
            fetch(next, slot ^ 1);  // (that slot's previous segment was worked off before the __syncwarp below)
        }
        bool ok = mbar_wait(bar0 + slot * 8, slot == 0 ? phase0 : phase1, s_abort, status, kDevTimeoutProducer);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            break;
        }
        if (slot == 0) {
            phase0 ^= 1;
        } else {
            phase1 ^= 1;
        }
        const uint32_t r = segs == 1 ? item : item / segs;
        const uint32_t c_begin = (item - r * segs) * seg;
        const uint32_t len = k - c_begin < seg ? k - c_begin : seg;
        const uint8_t* row = stage_ptr + slot * slot_bytes;
        uint8_t* qr = q + static_cast<uint64_t>(r) * q_pitch + (kFp4 ? c_begin / 2 : c_begin);
        uint8_t* sr = sf + static_cast<uint64_t>(r) * sf_pitch + c_begin / 32;
        // (the trip count is the same for every lane: the block maximum below is a full-warp shuffle; the length is
        // a multiple of 32, so the two lanes of a block are in range together)
        for (uint32_t base = 0; base < len; base += 32 * 16) {
            const uint32_t c0 = base + lane * 16;
            const bool active = c0 < len;
            float v[16];
            if (!active) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    v[i] = 0.0f;
                }
            } else if constexpr (kBf16In) {
                const uint4* src = reinterpret_cast<const uint4*>(row + c0 * 2);
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
                const float4* src = reinterpret_cast<const float4*>(row + c0 * 4);
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float4 raw = src[h];
                    v[h * 4] = raw.x;
                    v[h * 4 + 1] = raw.y;
                    v[h * 4 + 2] = raw.z;
                    v[h * 4 + 3] = raw.w;
                }
            }
            float mx = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                mx = fmaxf(mx, fabsf(v[i]));
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));  // the block's other half
            int exp = 0;
            if (!(mx < 1e-12f)) {
                exp = static_cast<int>((__float_as_uint(mx) >> 23) & 0xFFu) - 127 - kEmax;
                exp = exp < -128 ? -128 : (exp > 127 ? 127 : exp);
            }
            // x / 2^exp as a multiplication by 2^-exp: exact either way.  exp lies in [-48, 125] (a block's maximum
            // is at least 1e-12 or the exponent is 0; at most 2^128), so 2^-exp is a normal number.
            // bf16 inputs: the factor is (1 - 2^-12) * 2^-exp instead.  A bf16 value has 8 significant bits and the
            // factor 12, so the product is still exact; it lies below x / 2^exp by one part in 4096, which moves
            // an exact tie (and nothing else: any other value is at least one part in 256 away from the nearest
            // half-way point, in the subnormal range at least 2^-10 against a shift below 2^-18) to the side of
            // the smaller magnitude, where the reference's rule sends it.  The conversion instruction's nearest-
            // even result is then the rule's result, for normal and subnormal codes alike.
            // fp32 inputs get there in two steps: the value is first cut to 11 significant bits plus a twelfth that
            // says whether anything was cut off (every code and every half-way point has at most 6 significant
            // bits, so the cut changes neither on which side of a half-way point the value lies nor whether it
            // sits exactly on one), then multiplied by the same factor (12 + 12 bits: exact).  A value off a
            // half-way point is now at least half a unit of the 11-bit grid away from it, more than the shift.
            const float inv = __uint_as_float((static_cast<uint32_t>(126 - exp) << 23) | 0x007FF000u);
            if constexpr (!kBf16In) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t bits = __float_as_uint(v[i]);
                    v[i] = __uint_as_float((bits & 0xFFFFE000u) | ((bits & 0x00001FFFu) != 0 ? 0x00001000u : 0u));
                }
            }
            uint32_t words[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                uint32_t word = 0;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const float t0 = v[w * 4 + 2 * b] * inv, t1 = v[w * 4 + 2 * b + 1] * inv;
                    const uint32_t pair = mx_codes2_nudged<kFp4>(t0, t1);
                    word |= pair << ((kFp4 ? 8 : 16) * b);
                }
                words[w] = word;
            }
            if (!active) {
                continue;
            }
            if constexpr (kFp4) {
                // 16 elements = 8 bytes
                *reinterpret_cast<uint2*>(qr + (c0 >> 1)) =
                    make_uint2(words[0] | words[1] << 16, words[2] | words[3] << 16);
            } else {
                *reinterpret_cast<uint4*>(qr + c0) = make_uint4(words[0], words[1], words[2], words[3]);
            }
            if ((lane & 1u) == 0) {
                sr[c0 >> 5] = static_cast<uint8_t>(exp + 127);
                if (c_begin + c0 + 32 == k && ((k >> 5) & 1u) != 0) {
                    sr[(c0 >> 5) + 1] = 127;  // the padding column behind the row's last block
                }
            }
        }
        __syncwarp();  // every lane is done with this slot
        if (slots == 2) {
            slot ^= 1;
        } else if (next < items && lane == 0) {
            fetch(next, 0);
        }
    }
}

}  // namespace cb200
