// C-ABI entry points of libcatlass_b200.so (declared in include/catlass_b200.h).
// Host code only validates arguments, encodes tensor maps and launches; it never touches matrix data and
// has no CPU compute path: without a sm_100 device every launch entry returns an error.
#include <cuda_bf16.h>

#include "host_runtime.cuh"
#include "w8a8_gemm.cuh"

using namespace cb200;
using namespace cb200::host;

namespace {

struct W8A8Problem {
    uint32_t m, n, k;
    uint32_t group_count;  // 0 = dense
    uint32_t group_list_type;
    uint32_t layout_b;
    const void* a;
    const void* b;
    const void* group_list;
    const float* scale;
    const float* per_token;
    void* d;
    int32_t* acc;
    uint32_t block_num;
};

int check_w8a8(const W8A8Problem& q, uint32_t layout_a)
{
    if (q.a == nullptr || q.b == nullptr || q.scale == nullptr || q.per_token == nullptr || q.d == nullptr) {
        return (q.m == 0 || q.n == 0) ? CB200_SUCCESS : CB200_INVALID;
    }
    if (layout_a != CB200_ROW_MAJOR) {
        return CB200_INVALID;
    }
    if (q.layout_b != CB200_ROW_MAJOR && q.layout_b != CB200_COLUMN_MAJOR) {
        return CB200_INVALID;
    }
    if (q.group_count > static_cast<uint32_t>(kMaxGroups)) {
        return CB200_INVALID;
    }
    if (q.group_count != 0 && q.group_list == nullptr) {
        return CB200_INVALID;
    }
    if (q.group_list_type != CB200_GROUP_LIST_INT64 && q.group_list_type != CB200_GROUP_LIST_INT32) {
        return CB200_INVALID;
    }
    if (q.m > 0x7fffff00u || q.n > 0x7fffff00u || q.k > 0x7fffff00u) {
        return CB200_INVALID;
    }
    // TMA: base addresses 16-byte aligned, row pitches multiples of 16 bytes.
    if (!aligned16(q.a) || !aligned16(q.b)) {
        return CB200_INVALID;
    }
    if (q.k != 0) {
        if ((q.k & 15u) != 0) {
            return CB200_INVALID;  // A rows (and column-major B columns) are k bytes apart
        }
        if (q.layout_b == CB200_ROW_MAJOR && (q.n & 15u) != 0) {
            return CB200_INVALID;  // row-major B rows are n bytes apart
        }
    }
    if ((reinterpret_cast<uintptr_t>(q.d) & 1u) != 0 || (reinterpret_cast<uintptr_t>(q.scale) & 3u) != 0 ||
        (reinterpret_cast<uintptr_t>(q.per_token) & 3u) != 0) {
        return CB200_INVALID;
    }
    if ((q.n & 7u) == 0 && !aligned16(q.d)) {
        return CB200_INVALID;  // vector stores of 8 bf16
    }
    return CB200_SUCCESS;
}

template <int BN, bool kBMn>
int launch_w8a8(const W8A8Problem& q, const DeviceState& dev, cudaStream_t stream)
{
    using S = W8A8Smem<BN>;
    static_assert(S::kTotalBytes <= 232448, "shared memory budget of one CTA");
    CUtensorMap tmap_a, tmap_b;
    const uint32_t groups = q.group_count == 0 ? 1u : q.group_count;
    {
        const uint64_t dims[2] = {q.k, q.m};
        const uint64_t strides[1] = {q.k};
        const uint32_t box[2] = {kBlockKBytes, kBlockM};
        int rc = encode_tmap_u8(&tmap_a, q.a, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    if (kBMn) {  // each weight matrix is k rows of n contiguous bytes
        const uint64_t dims[3] = {q.n, q.k, groups};
        const uint64_t strides[2] = {q.n, static_cast<uint64_t>(q.n) * q.k};
        const uint32_t box[3] = {128, kBlockKBytes, 1};
        int rc = encode_tmap_u8(&tmap_b, q.b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    } else {  // each weight matrix is n columns of k contiguous bytes
        const uint64_t dims[3] = {q.k, q.n, groups};
        const uint64_t strides[2] = {q.k, static_cast<uint64_t>(q.n) * q.k};
        const uint32_t box[3] = {kBlockKBytes, BN, 1};
        int rc = encode_tmap_u8(&tmap_b, q.b, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }

    W8A8Params p;
    p.m = q.m;
    p.n = q.n;
    p.k = q.k;
    p.group_count = q.group_count;
    p.group_list_is_i32 = q.group_list_type == CB200_GROUP_LIST_INT32 ? 1u : 0u;
    p.num_k_blocks = (q.k + kBlockKBytes - 1) / kBlockKBytes;
    p.group_list = q.group_list;
    p.scale = q.scale;
    p.per_token = q.per_token;
    p.d = static_cast<__nv_bfloat16*>(q.d);
    p.acc = q.acc;
    p.status = dev.status;

    auto kernel = w8a8_gemm_kernel<BN, kBMn>;
    static bool attr_set[kMaxDevices] = {};
    int devid = 0;
    CB200_CUDA_TRY(cudaGetDevice(&devid));
    if (!attr_set[devid]) {
        CB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotalBytes));
        attr_set[devid] = true;
    }
    // upper bound of the tile count: every group may add one partial row tile
    const uint64_t n_tiles = (q.n + BN - 1) / BN;
    const uint64_t max_tiles = (static_cast<uint64_t>((q.m + kBlockM - 1) / kBlockM) + groups) * n_tiles;
    uint32_t grid = static_cast<uint32_t>(dev.sm_count);
    if (q.block_num != 0 && q.block_num < grid) {
        grid = q.block_num;
    }
    if (max_tiles < grid) {
        grid = static_cast<uint32_t>(max_tiles);
    }
    if (grid == 0) {
        return CB200_SUCCESS;
    }
    kernel<<<grid, kGemmThreads, S::kTotalBytes, stream>>>(tmap_a, tmap_b, p);
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

int run_w8a8(const W8A8Problem& q, uint32_t layout_a, void* stream_v)
{
    int rc = check_w8a8(q, layout_a);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    if (q.m == 0 || q.n == 0) {
        return CB200_SUCCESS;
    }
    DeviceState* dev = nullptr;
    rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (q.k == 0) {
        zero_rows_kernel<<<dev->sm_count * 4, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(q.d), q.group_list,
                                                                q.group_list_type == CB200_GROUP_LIST_INT32,
                                                                q.group_count, q.m, q.n);
        CB200_CUDA_TRY(cudaGetLastError());
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return CB200_SUCCESS;
    }
    const bool b_mn = q.layout_b == CB200_ROW_MAJOR;
    if (q.n > 128) {
        return b_mn ? launch_w8a8<256, true>(q, *dev, stream) : launch_w8a8<256, false>(q, *dev, stream);
    }
    return b_mn ? launch_w8a8<128, true>(q, *dev, stream) : launch_w8a8<128, false>(q, *dev, stream);
}

}  // namespace

extern "C" {

int cb200_quant_matmul_can_implement(const cb200_quant_matmul_args* args)
{
    if (args == nullptr) {
        return CB200_INVALID;
    }
    W8A8Problem q{args->m, args->n, args->k, 0, CB200_GROUP_LIST_INT64, args->layout_b, args->a, args->b, nullptr,
                  args->scale, args->per_token_scale, args->d, args->acc, args->block_num};
    return check_w8a8(q, args->layout_a);
}

uint64_t cb200_quant_matmul_workspace_size(const cb200_quant_matmul_args* args)
{
    (void)args;
    return 0;  // the accumulator stays in TMEM; nothing is staged through global memory
}

int cb200_quant_matmul(const cb200_quant_matmul_args* args, void* stream)
{
    if (args == nullptr) {
        return CB200_INVALID;
    }
    W8A8Problem q{args->m, args->n, args->k, 0, CB200_GROUP_LIST_INT64, args->layout_b, args->a, args->b, nullptr,
                  args->scale, args->per_token_scale, args->d, args->acc, args->block_num};
    return run_w8a8(q, args->layout_a, stream);
}

int cb200_grouped_quant_matmul_slice_m_can_implement(const cb200_grouped_quant_matmul_args* args)
{
    if (args == nullptr || args->group_count == 0) {
        return CB200_INVALID;
    }
    W8A8Problem q{args->m, args->n, args->k, args->group_count, args->group_list_type, args->layout_b, args->a,
                  args->b, args->group_list, args->scale, args->per_token_scale, args->d, args->acc,
                  args->block_num};
    return check_w8a8(q, CB200_ROW_MAJOR);
}

uint64_t cb200_grouped_quant_matmul_slice_m_workspace_size(const cb200_grouped_quant_matmul_args* args)
{
    (void)args;
    return 0;
}

int cb200_grouped_quant_matmul_slice_m(const cb200_grouped_quant_matmul_args* args, void* stream)
{
    if (args == nullptr || args->group_count == 0) {
        return CB200_INVALID;
    }
    W8A8Problem q{args->m, args->n, args->k, args->group_count, args->group_list_type, args->layout_b, args->a,
                  args->b, args->group_list, args->scale, args->per_token_scale, args->d, args->acc,
                  args->block_num};
    return run_w8a8(q, CB200_ROW_MAJOR, stream);
}

int cb200_device_status(uint32_t* code)
{
    if (code == nullptr) {
        return CB200_INVALID;
    }
    DeviceState* dev = nullptr;
    int rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    CB200_CUDA_TRY(cudaDeviceSynchronize());
    unsigned v = 0;
    CB200_CUDA_TRY(cudaMemcpy(&v, dev->status, sizeof(v), cudaMemcpyDeviceToHost));
    if (v != 0) {
        unsigned zero = 0;
        CB200_CUDA_TRY(cudaMemcpy(dev->status, &zero, sizeof(zero), cudaMemcpyHostToDevice));
    }
    *code = v;
    return v == 0 ? CB200_SUCCESS : CB200_DEVICE_TIMEOUT;
}

int cb200_last_cuda_error(void)
{
    return t_last_cuda_error;
}

uint64_t cb200_launch_count(void)
{
    return g_launches.load(std::memory_order_relaxed);
}

const char* cb200_version(void)
{
    return "catlass_b200 0.1 (sm_100a)";
}

}  // extern "C"
