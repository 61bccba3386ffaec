// Shared helpers of the example programs: argv parsing in the reference's positional style
// (examples/common/options.hpp:34-150), seeded data, device buffers, comparison against the CPU oracle.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <random>
#include <vector>

#include "oracle.h"

#define CUDA_CHECK(expr)                                                                             \
    do {                                                                                             \
        cudaError_t e__ = (expr);                                                                    \
        if (e__ != cudaSuccess) {                                                                    \
            std::cerr << "cudaError " << cudaGetErrorString(e__) << " at " << __FILE__ << ":" << __LINE__ << "\n"; \
            std::exit(2);                                                                            \
        }                                                                                            \
    } while (0)

namespace example {

inline void FillInt8(std::vector<int8_t>& v, int low, int high, uint64_t seed)
{
    std::mt19937_64 gen(seed);
    std::uniform_int_distribution<int> dist(low, high);
    for (auto& x : v) {
        x = static_cast<int8_t>(dist(gen));
    }
}

inline void FillFloat(std::vector<float>& v, float low, float high, uint64_t seed)
{
    std::mt19937_64 gen(seed);
    std::uniform_real_distribution<float> dist(low, high);
    for (auto& x : v) {
        x = dist(gen);
    }
}

template <class T>
uint8_t* ToDevice(std::vector<T> const& host)
{
    void* p = nullptr;
    CUDA_CHECK(cudaMalloc(&p, host.size() * sizeof(T) + 16));
    CUDA_CHECK(cudaMemcpy(p, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice));
    return static_cast<uint8_t*>(p);
}

/// Counts outputs whose bf16 bits differ from the oracle's fp32 result rounded to bf16.
inline size_t CountMismatches(std::vector<uint16_t> const& got, std::vector<float> const& want, size_t count)
{
    size_t bad = 0;
    for (size_t i = 0; i < count; ++i) {
        if (got[i] != orc_bf16_rne(want[i])) {
            ++bad;
        }
    }
    return bad;
}

inline int Report(size_t bad)
{
    if (bad == 0) {
        std::cout << "Compare success." << std::endl;
        return 0;
    }
    std::cerr << "Compare failed. Error count: " << bad << std::endl;
    return 1;
}

}  // namespace example
