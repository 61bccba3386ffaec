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
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

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

}  // namespace cb200
