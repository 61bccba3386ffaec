// Library-style entry points with the reference's shared_lib signature
// (examples/shared_lib/include/catlass_kernel.h:19-65): Op(blockNum, stream, KernelInfo).
// As in the reference's RunAdapter (examples/shared_lib/src/common/common.hpp:33-47) a call obtains its own
// workspace, launches, synchronises the stream and releases the workspace.  Operand order follows the
// reference's optest kernels: dense [A, B, scale, perTokenScale], grouped [A, B, groupList, scale,
// perTokenScale] (groupList on the device), W4A8 [A, packedB, weightScale, perTokenScale],
// MX [A, B, scaleA, scaleB]; outputAddr = [D].
//
// Differences from the reference header, all deliberate:
//  - the functions return an int status (0 = success; the reference returns void and only prints ACL errors,
//    examples/shared_lib/src/common/common.hpp:22-28), so that a caller can tell an unsupported problem from a run;
//  - KernelInfo has no aclDataType members (there is no ACL here): `outputDataType` / `scaleDataType` are the
//    DataType enum below, and the quantized operators add `groupSize` (W4A8), `fp4` (MX), `quantMode` and
//    `scalePerTensor` (per-tensor / per-channel grouped dequant), which the reference's fp16 operators do not need.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "device_gemm.hpp"

namespace CatlassKernel {

using ElementGroupList = int64_t;

enum class DataType : uint32_t { FLOAT = CB200_DTYPE_F32, BF16 = CB200_DTYPE_BF16, FLOAT16 = CB200_DTYPE_F16 };

struct KernelInfo {
    enum class GMMSplit : uint32_t { SPLIT_M = 0, SPLIT_K = 1, SPLIT_N = 2 };
    DataType scaleDataType = DataType::FLOAT;   // W8A8: element type of scale and perTokenScale
    DataType outputDataType = DataType::BF16;   // element type of D (BF16 or FLOAT16)
    uint32_t g = 1;
    uint32_t b = 1;
    uint32_t m = 1;
    uint32_t n = 1;
    uint32_t k = 1;
    uint32_t M = 1;
    uint32_t K = 1;
    bool transA = false;
    bool transB = false;          // true: B is column-major (each column K-contiguous)
    uint32_t groupSize = 128;     // W4A8 weight-scale group along K
    bool fp4 = false;             // MX: E2M1 elements instead of E4M3
    int32_t quantMode = 0;        // per-tensor (0) / per-channel (1) grouped dequant
    float scalePerTensor = 1.0f;
    std::vector<ElementGroupList> groupList;  // unused: the grouped op takes the device list in inputAddr[2]
    GMMSplit split = GMMSplit::SPLIT_M;
    std::vector<uint8_t*> inputAddr;
    std::vector<uint8_t*> outputAddr;
};

namespace detail {
template <class Kernel>
inline int RunAdapter(typename Kernel::Arguments const& args, cudaStream_t stream, uint32_t blockNum)
{
    using Op = Catlass::Gemm::Device::DeviceGemm<Kernel>;
    if (Op::CanImplement(args) != Catlass::Status::kSuccess) {
        return CB200_INVALID;
    }
    Op op;
    const size_t wsBytes = Op::GetWorkspaceSize(args);
    uint8_t* ws = nullptr;
    if (wsBytes != 0 && cudaMalloc(reinterpret_cast<void**>(&ws), wsBytes) != cudaSuccess) {
        return CB200_CUDA_ERROR;
    }
    op.Initialize(args, ws);
    op(stream, blockNum);
    const int code = op.LastCode();
    const cudaError_t sync = cudaStreamSynchronize(stream);
    if (ws != nullptr) {
        cudaFree(ws);
    }
    return code != CB200_SUCCESS ? code : (sync == cudaSuccess ? CB200_SUCCESS : CB200_CUDA_ERROR);
}
}  // namespace detail

/// D = round((int32(A*B) * scale[n]) * perToken[m]); A per info.transA, B per info.transB (true = column-major).
inline int QuantMatmul(const uint32_t blockNum, cudaStream_t stream, const KernelInfo& info)
{
    if (info.inputAddr.size() < 4 || info.outputAddr.empty()) {
        return CB200_INVALID;
    }
    using namespace Catlass;
    auto run = [&](auto kernel_tag) {
        using K = decltype(kernel_tag);
        typename K::Arguments a{GemmCoord{info.m, info.n, info.k}, blockNum, info.inputAddr[0], info.inputAddr[1],
                                info.inputAddr[2], info.inputAddr[3], info.outputAddr[0],
                                static_cast<uint32_t>(info.scaleDataType), static_cast<uint32_t>(info.outputDataType)};
        return detail::RunAdapter<K>(a, stream, blockNum);
    };
    if (info.transA) {
        return info.transB ? run(Gemm::Kernel::QuantMatmul<layout::ColumnMajor, layout::ColumnMajor>{})
                           : run(Gemm::Kernel::QuantMatmul<layout::ColumnMajor, layout::RowMajor>{});
    }
    return info.transB ? run(Gemm::Kernel::QuantMatmul<layout::RowMajor, layout::ColumnMajor>{})
                       : run(Gemm::Kernel::QuantMatmul<layout::RowMajor, layout::RowMajor>{});
}

/// Grouped slice-M W8A8: info.g groups, inputAddr = [A, B, groupList(int64, device), scale, perTokenScale].
inline int GroupedMatmulSliceMPerTokenDequant(const uint32_t blockNum, cudaStream_t stream, const KernelInfo& info)
{
    if (info.transA || info.inputAddr.size() < 5 || info.outputAddr.empty() ||
        info.split != KernelInfo::GMMSplit::SPLIT_M) {
        return CB200_INVALID;
    }
    using namespace Catlass;
    if (info.transB) {
        using K = Gemm::Kernel::GroupedMatmulSliceMPerTokenDequant<layout::ColumnMajor, ElementGroupList>;
        K::Arguments a{GemmCoord{info.m, info.n, info.k}, info.g, info.inputAddr[2], info.inputAddr[0],
                       info.inputAddr[1], info.inputAddr[3], info.inputAddr[4], info.outputAddr[0], blockNum,
                       static_cast<uint32_t>(info.scaleDataType), static_cast<uint32_t>(info.outputDataType)};
        return detail::RunAdapter<K>(a, stream, blockNum);
    }
    using K = Gemm::Kernel::GroupedMatmulSliceMPerTokenDequant<layout::RowMajor, ElementGroupList>;
    K::Arguments a{GemmCoord{info.m, info.n, info.k}, info.g, info.inputAddr[2], info.inputAddr[0], info.inputAddr[1],
                   info.inputAddr[3], info.inputAddr[4], info.outputAddr[0], blockNum,
                   static_cast<uint32_t>(info.scaleDataType), static_cast<uint32_t>(info.outputDataType)};
    return detail::RunAdapter<K>(a, stream, blockNum);
}

/// Grouped slice-M W8A8 with per-tensor (info.quantMode 0, info.scalePerTensor) or per-channel (1) dequant:
/// inputAddr = [A, B (row-major), groupList(int64, device), perChannelScale (64-bit words, fp32 bits low)].
inline int GroupedMatmulSliceMFixpipeDequant(const uint32_t blockNum, cudaStream_t stream, const KernelInfo& info)
{
    if (info.transA || info.transB || info.inputAddr.size() < 4 || info.outputAddr.empty() ||
        (info.quantMode != 0 && info.quantMode != 1)) {
        return CB200_INVALID;
    }
    using namespace Catlass;
    auto run = [&](auto kernel_tag) {
        using K = decltype(kernel_tag);
        typename K::Arguments a{GemmCoord{info.m, info.n, info.k}, info.g, info.inputAddr[2], info.inputAddr[0],
                                info.inputAddr[1], info.outputAddr[0], info.scalePerTensor, info.inputAddr[3],
                                CB200_DTYPE_F32_IN_U64, static_cast<uint32_t>(info.outputDataType)};
        return detail::RunAdapter<K>(a, stream, blockNum);
    };
    return info.quantMode == 1 ? run(Gemm::Kernel::GroupedMatmulSliceMFixpipeDequant<true>{})
                               : run(Gemm::Kernel::GroupedMatmulSliceMFixpipeDequant<false>{});
}

/// W4A8 per-group: inputAddr = [A, packedB (column-major, packed along K), weightScale, perTokenScale].
inline int W4A8Matmul(const uint32_t blockNum, cudaStream_t stream, const KernelInfo& info)
{
    if (info.transA || !info.transB || info.inputAddr.size() < 4 || info.outputAddr.empty()) {
        return CB200_INVALID;
    }
    using K = Catlass::Gemm::Kernel::W4A8Matmul;
    K::Arguments a{Catlass::GemmCoord{info.m, info.n, info.k}, info.groupSize, info.inputAddr[0], info.inputAddr[1],
                   info.inputAddr[2], info.inputAddr[3], info.outputAddr[0],
                   static_cast<uint32_t>(info.outputDataType)};
    return detail::RunAdapter<K>(a, stream, blockNum);
}

/// MX block-scaled matmul: inputAddr = [A, B (column-major), scaleA, scaleB]; info.fp4 selects E2M1.
inline int MxMatmul(const uint32_t blockNum, cudaStream_t stream, const KernelInfo& info)
{
    if (info.transA || !info.transB || info.inputAddr.size() < 4 || info.outputAddr.empty()) {
        return CB200_INVALID;
    }
    using namespace Catlass;
    if (info.fp4) {
        using K = Gemm::Kernel::MxMatmul<true>;
        K::Arguments a{GemmCoord{info.m, info.n, info.k}, info.inputAddr[0], info.inputAddr[1], info.inputAddr[2],
                       info.inputAddr[3], info.outputAddr[0]};
        return detail::RunAdapter<K>(a, stream, blockNum);
    }
    using K = Gemm::Kernel::MxMatmul<false>;
    K::Arguments a{GemmCoord{info.m, info.n, info.k}, info.inputAddr[0], info.inputAddr[1], info.inputAddr[2],
                   info.inputAddr[3], info.outputAddr[0]};
    return detail::RunAdapter<K>(a, stream, blockNum);
}

}  // namespace CatlassKernel
