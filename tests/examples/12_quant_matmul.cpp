// Example 12 of the reference (examples/12_quant_matmul/quant_matmul.cpp) on the B200 library:
//     12_quant_matmul m n k [deviceId]
// A int8 row-major, B int8 column-major, fp32 scales, bf16 out; self-checks against the CPU oracle and prints
// "Compare success." like the reference's examples do.
#include "catlass_b200/device_gemm.hpp"
#include "common.hpp"

using namespace Catlass;

int main(int argc, const char** argv)
{
    if (argc < 4) {
        std::cerr << "usage: 12_quant_matmul m n k [deviceId]" << std::endl;
        return 64;
    }
    const uint32_t m = std::atoi(argv[1]), n = std::atoi(argv[2]), k = std::atoi(argv[3]);
    const int device = argc > 4 ? std::atoi(argv[4]) : 0;
    CUDA_CHECK(cudaSetDevice(device));
    cudaStream_t stream;
    CUDA_CHECK(cudaStreamCreate(&stream));

    GemmCoord problemShape{m, n, k};
    layout::RowMajor layoutA{m, k};
    layout::ColumnMajor layoutB{k, n};
    std::vector<int8_t> hostA(layoutA.Capacity()), hostB(layoutB.Capacity());
    std::vector<float> hostScale(n), hostPerToken(m);
    example::FillInt8(hostA, -16, 16, 1);
    example::FillInt8(hostB, -16, 16, 2);
    example::FillFloat(hostScale, 0.0f, 1.0f, 3);
    example::FillFloat(hostPerToken, 0.0f, 1.0f, 4);

    uint8_t* deviceA = example::ToDevice(hostA);
    uint8_t* deviceB = example::ToDevice(hostB);
    uint8_t* deviceScale = example::ToDevice(hostScale);
    uint8_t* devicePerToken = example::ToDevice(hostPerToken);
    std::vector<uint16_t> hostD(size_t(m) * n, 0);
    uint8_t* deviceD = example::ToDevice(hostD);

    using Kernel = Gemm::Kernel::QuantMatmul<layout::RowMajor, layout::ColumnMajor>;
    using MatmulAdapter = Gemm::Device::DeviceGemm<Kernel>;
    Kernel::Arguments arguments{problemShape, 0, deviceA, deviceB, deviceScale, devicePerToken, deviceD};
    if (MatmulAdapter::CanImplement(arguments) != Status::kSuccess) {
        std::cerr << "problem not supported (k must be a multiple of 16)" << std::endl;
        return 1;
    }
    MatmulAdapter matmulOp;
    uint8_t* deviceWorkspace = nullptr;
    const size_t sizeWorkspace = MatmulAdapter::GetWorkspaceSize(arguments);
    if (sizeWorkspace > 0) {
        CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&deviceWorkspace), sizeWorkspace));
    }
    matmulOp.Initialize(arguments, deviceWorkspace);
    if (matmulOp(stream) != Status::kSuccess) {
        std::cerr << "launch failed, status " << matmulOp.LastCode() << std::endl;
        return 1;
    }
    CUDA_CHECK(cudaStreamSynchronize(stream));
    CUDA_CHECK(cudaMemcpy(hostD.data(), deviceD, hostD.size() * 2, cudaMemcpyDeviceToHost));

    std::vector<float> golden(size_t(m) * n);
    orc_quant_matmul(m, n, k, hostA.data(), ORC_ROW_MAJOR, hostB.data(), ORC_COL_MAJOR, hostScale.data(),
                     hostPerToken.data(), golden.data(), nullptr);
    return example::Report(example::CountMismatches(hostD, golden, golden.size()));
}
