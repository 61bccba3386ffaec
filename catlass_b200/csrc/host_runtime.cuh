// Host-side plumbing shared by the C-ABI entry points: per-device state (SM count, status word address),
// tensor-map encoding through the driver entry point, error bookkeeping and launch counting.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

#include "../../include/catlass_b200.h"

namespace cb200 {

// Device status word: kernels that give up on a bounded wait atomicMax their code into it.
__device__ unsigned g_device_status = 0;

namespace host {

inline thread_local int t_last_cuda_error = 0;
inline std::atomic<uint64_t> g_launches{0};

inline int cuda_fail(int code)
{
    t_last_cuda_error = code;
    return CB200_CUDA_ERROR;
}

#define CB200_CUDA_TRY(expr)                                   \
    do {                                                       \
        cudaError_t e__ = (expr);                              \
        if (e__ != cudaSuccess) {                              \
            return ::cb200::host::cuda_fail(static_cast<int>(e__)); \
        }                                                      \
    } while (0)

constexpr int kMaxDevices = 64;

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    unsigned* status = nullptr;
};

// State of the current device, set up on the first call made with that device current.
inline int device_state(DeviceState** out)
{
    static DeviceState states[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    CB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        return CB200_INVALID;
    }
    DeviceState& st = states[dev];
    if (!st.ready) {
        std::lock_guard<std::mutex> lock(mu);
        if (!st.ready) {
            int major = 0;
            CB200_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
            if (major != 10) {
                return CB200_INVALID;  // the kernels are sm_100a only
            }
            CB200_CUDA_TRY(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
            void* p = nullptr;
            CB200_CUDA_TRY(cudaGetSymbolAddress(&p, g_device_status));
            st.status = static_cast<unsigned*>(p);
            st.ready = true;
        }
    }
    *out = &st;
    return CB200_SUCCESS;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Byte tensor (uint8 elements) of `rank` dims, dims[0] contiguous; strides[i] = byte stride of dim i+1.
// Out-of-range parts of a box read as zero.
inline int encode_tmap_u8(CUtensorMap* map, const void* base, uint32_t rank, const uint64_t* dims,
                          const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        return cuda_fail(-1);
    }
    cuuint64_t gdim[5];
    cuuint64_t gstr[4];
    cuuint32_t bdim[5];
    cuuint32_t estr[5];
    for (uint32_t i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) {
            gstr[i] = strides[i];
        }
    }
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return cuda_fail(static_cast<int>(r));
    }
    return CB200_SUCCESS;
}

inline bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

}  // namespace host
}  // namespace cb200
