// Examples 07 / 10 of the reference (examples/07_grouped_matmul_slice_m_per_token_dequant_moe/...) on the B200
// library:
//     07_grouped_matmul_slice_m_per_token_dequant problem_count m n k [deviceId]
// Ascending random group list over m rows (repeats = empty groups), B row-major per group, bf16 out;
// self-checks the rows below groupList[problem_count-1] against the CPU oracle.
#include <algorithm>

#include "catlass_b200/device_gemm.hpp"
#include "common.hpp"

using namespace Catlass;

int main(int argc, const char** argv)
{
    if (argc < 5) {
        std::cerr << "usage: 07_grouped_matmul_slice_m_per_token_dequant problem_count m n k [deviceId]" << std::endl;
        return 64;
    }
    const uint32_t problemCount = std::atoi(argv[1]);
    const uint32_t m = std::atoi(argv[2]), n = std::atoi(argv[3]), k = std::atoi(argv[4]);
    const int device = argc > 5 ? std::atoi(argv[5]) : 0;
    CUDA_CHECK(cudaSetDevice(device));
    cudaStream_t stream;
    CUDA_CHECK(cudaStreamCreate(&stream));

    // group list: sorted uniform cut points in [0, m], as golden::GenerateGroupList draws them
    std::vector<int64_t> groupList(problemCount);
    {
        std::mt19937_64 gen(0);
        std::uniform_int_distribution<int64_t> dist(0, m);
        for (auto& g : groupList) {
            g = dist(gen);
        }
        std::sort(groupList.begin(), groupList.end());
    }
    std::vector<int8_t> hostA(size_t(m) * k), hostB(size_t(problemCount) * k * n);
    std::vector<float> hostScale(size_t(problemCount) * n), hostPerToken(m);
    example::FillInt8(hostA, -16, 16, 1);
    example::FillInt8(hostB, -16, 16, 2);
    example::FillFloat(hostScale, 0.0f, 1.0f, 3);
    example::FillFloat(hostPerToken, 0.0f, 1.0f, 4);

    uint8_t* deviceA = example::ToDevice(hostA);
    uint8_t* deviceB = example::ToDevice(hostB);
    uint8_t* deviceScale = example::ToDevice(hostScale);
    uint8_t* devicePerToken = example::ToDevice(hostPerToken);
    uint8_t* deviceGroupList = example::ToDevice(groupList);
    std::vector<uint16_t> hostD(size_t(m) * n, 0);
    uint8_t* deviceD = example::ToDevice(hostD);

    using Kernel = Gemm::Kernel::GroupedMatmulSliceMPerTokenDequant<layout::RowMajor, int64_t>;
    using MatmulAdapter = Gemm::Device::DeviceGemm<Kernel>;
    Kernel::Arguments arguments{GemmCoord{m, n, k}, problemCount, deviceGroupList, deviceA, deviceB,
                                deviceScale,        devicePerToken, deviceD};
    if (MatmulAdapter::CanImplement(arguments) != Status::kSuccess) {
        std::cerr << "problem not supported (k and n must be multiples of 16, at most 1024 groups)" << std::endl;
        return 1;
    }
    MatmulAdapter matmulOp;
    matmulOp.Initialize(arguments, nullptr);
    if (matmulOp(stream) != Status::kSuccess) {
        std::cerr << "launch failed, status " << matmulOp.LastCode() << std::endl;
        return 1;
    }
    CUDA_CHECK(cudaStreamSynchronize(stream));
    CUDA_CHECK(cudaMemcpy(hostD.data(), deviceD, hostD.size() * 2, cudaMemcpyDeviceToHost));

    std::vector<float> golden(size_t(m) * n, 0.0f);
    orc_grouped_quant_matmul_slice_m(m, n, k, problemCount, groupList.data(), hostA.data(), hostB.data(),
                                     ORC_ROW_MAJOR, hostScale.data(), hostPerToken.data(), golden.data(), nullptr);
    const size_t validNum = problemCount ? size_t(groupList[problemCount - 1]) * n : 0;
    return example::Report(example::CountMismatches(hostD, golden, validNum));
}
