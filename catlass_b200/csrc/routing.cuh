// Deterministic finalize routing: out[t] = shared-expert term + the weighted rows routed to token t, added in ascending
// row order: the order of the golden's index_add_
// (experimental/gmm/ascend950_fp8_mx_grouped_matmul_finalize_routing/gen_data_compare.py:744-757), so that the
// result does not depend on which tile finished first.  The reference serves this with a second kernel
// (GroupedMxMatmulFinalizeRoutingTla + BlockEpilogueFinalizeRouting with a column-block scheduler,
// include/catlass/gemm/kernel/grouped_mx_matmul_finalize_routing_tla.hpp,
// include/catlass/epilogue/block/block_epilogue_finalize_routing.hpp); here the grouped matmul writes C in fp32 and
// four small kernels invert row_index (count, scan, fill) and gather.  All HBM-bound: one pass over C.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace cb200 {

struct RoutingLists {
    int32_t* group_end;   // [groups]: one past the last row of group g (clamped to m, never decreasing)
    int32_t* total_rows;  // [1]: rows that belong to a group
    int32_t* count;       // [batch]: rows routed to token t; after the scan: fill cursor
    int32_t* start;       // [batch + 1]: first entry of token t in `order`
    int32_t* order;       // [m]: rows grouped by token (unordered inside a token until the gather sorts them)
};

__device__ __forceinline__ long long routing_target(const void* row_index, uint32_t is_i32, uint32_t p)
{
    return is_i32 ? static_cast<long long>(static_cast<const int32_t*>(row_index)[p])
                  : static_cast<const long long*>(row_index)[p];
}

// One block: group ends from the group list (sizes or prefix sums, int32 or int64), total rows; clears the counts.
__global__ void routing_prepare_kernel(const void* group_list, uint32_t is_i32, uint32_t is_prefix_sum, uint32_t groups,
                                       uint32_t m, uint32_t batch, RoutingLists l)
{
    if (threadIdx.x == 0) {
        long long prev = 0;
        for (uint32_t g = 0; g < groups; ++g) {
            const long long v = is_i32 ? static_cast<long long>(static_cast<const int32_t*>(group_list)[g])
                                       : static_cast<const long long*>(group_list)[g];
            long long end = is_prefix_sum ? v : prev + (v < 0 ? 0 : v);
            end = end < prev ? prev : (end > static_cast<long long>(m) ? static_cast<long long>(m) : end);
            l.group_end[g] = static_cast<int32_t>(end);
            prev = end;
        }
        *l.total_rows = static_cast<int32_t>(prev);
    }
    for (uint32_t t = threadIdx.x; t < batch; t += blockDim.x) {
        l.count[t] = 0;
    }
}

__global__ void routing_count_kernel(const void* row_index, uint32_t is_i32, uint32_t batch, RoutingLists l)
{
    const uint32_t total = static_cast<uint32_t>(*l.total_rows);
    for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < total; p += gridDim.x * blockDim.x) {
        const long long t = routing_target(row_index, is_i32, p);
        if (t >= 0 && t < static_cast<long long>(batch)) {
            atomicAdd(l.count + t, 1);
        }
    }
}

// One block of 1024 threads: start = exclusive prefix sums of count; count becomes the fill cursor (= start).
__global__ void routing_scan_kernel(uint32_t batch, RoutingLists l)
{
    __shared__ int32_t s_part[1024];
    const uint32_t per = (batch + blockDim.x - 1) / blockDim.x;
    const uint32_t lo = threadIdx.x * per, hi = lo + per < batch ? lo + per : batch;
    int32_t sum = 0;
    for (uint32_t t = lo; t < hi; ++t) {
        sum += l.count[t];
    }
    s_part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t run = 0;
        for (uint32_t i = 0; i < blockDim.x; ++i) {
            const int32_t v = s_part[i];
            s_part[i] = run;
            run += v;
        }
        l.start[batch] = run;
    }
    __syncthreads();
    int32_t run = s_part[threadIdx.x];
    for (uint32_t t = lo; t < hi; ++t) {
        const int32_t c = l.count[t];
        l.start[t] = run;
        l.count[t] = run;
        run += c;
    }
}

__global__ void routing_fill_kernel(const void* row_index, uint32_t is_i32, uint32_t batch, RoutingLists l)
{
    const uint32_t total = static_cast<uint32_t>(*l.total_rows);
    for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < total; p += gridDim.x * blockDim.x) {
        const long long t = routing_target(row_index, is_i32, p);
        if (t >= 0 && t < static_cast<long long>(batch)) {
            l.order[atomicAdd(l.count + t, 1)] = static_cast<int32_t>(p);
        }
    }
}

constexpr int kRoutingMaxSorted = 1024;  // rows of one token sorted in shared memory (more: sorted in place, serially)

// One block per token.  c [m][n] fp32 (the grouped matmul's result), out [batch][n].
__global__ void routing_gather_kernel(const float* __restrict__ c, float* __restrict__ out, uint32_t n, uint32_t groups,
                                      const float* __restrict__ logit, const __nv_bfloat16* __restrict__ bias,
                                      const __nv_bfloat16* __restrict__ shared_input, float shared_weight,
                                      uint32_t shared_offset, uint32_t shared_rows, RoutingLists l)
{
    __shared__ int32_t s_rows[kRoutingMaxSorted];
    __shared__ int32_t s_group[kRoutingMaxSorted];
    __shared__ float s_logit[kRoutingMaxSorted];
    const uint32_t t = blockIdx.x;
    const int32_t lo = l.start[t], hi = l.start[t + 1];
    const uint32_t k = static_cast<uint32_t>(hi - lo);
    const bool in_smem = k <= kRoutingMaxSorted;
    if (in_smem) {
        // rank sort: the rows of a token are distinct, so the number of smaller rows is the position
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
            const int32_t v = l.order[lo + i];
            uint32_t rank = 0;
            for (uint32_t j = 0; j < k; ++j) {
                rank += l.order[lo + j] < v ? 1u : 0u;
            }
            s_rows[rank] = v;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
            const int32_t p = s_rows[i];
            uint32_t a = 0, b = groups - 1;  // first group whose end lies beyond p
            while (a < b) {
                const uint32_t mid = (a + b) >> 1;
                if (l.group_end[mid] > p) {
                    b = mid;
                } else {
                    a = mid + 1;
                }
            }
            s_group[i] = static_cast<int32_t>(a);
            s_logit[i] = logit[p];
        }
    } else if (threadIdx.x == 0) {
        for (int32_t i = lo + 1; i < hi; ++i) {  // insertion sort in place (only this block touches the range)
            const int32_t v = l.order[i];
            int32_t j = i - 1;
            while (j >= lo && l.order[j] > v) {
                l.order[j + 1] = l.order[j];
                --j;
            }
            l.order[j + 1] = v;
        }
    }
    __syncthreads();
    const bool has_shared = shared_input != nullptr && t >= shared_offset && t - shared_offset < shared_rows;
    const __nv_bfloat16* srow = has_shared ? shared_input + static_cast<size_t>(t - shared_offset) * n : nullptr;
    float* orow = out + static_cast<size_t>(t) * n;
    for (uint32_t col = threadIdx.x; col < n; col += blockDim.x) {
        float acc = 0.0f;
        if (has_shared) {
            acc = __fadd_rn(acc, __fmul_rn(shared_weight, __bfloat162float(srow[col])));
        }
        for (uint32_t i = 0; i < k; ++i) {
            int32_t p, g;
            float w;
            if (in_smem) {
                p = s_rows[i];
                g = s_group[i];
                w = s_logit[i];
            } else {
                p = l.order[lo + i];
                uint32_t a = 0, b = groups - 1;
                while (a < b) {
                    const uint32_t mid = (a + b) >> 1;
                    if (l.group_end[mid] > p) {
                        b = mid;
                    } else {
                        a = mid + 1;
                    }
                }
                g = static_cast<int32_t>(a);
                w = logit[p];
            }
            float y = c[static_cast<size_t>(p) * n + col];
            if (bias != nullptr) {
                y = __fadd_rn(y, __bfloat162float(bias[static_cast<size_t>(g) * n + col]));
            }
            acc = __fadd_rn(acc, __fmul_rn(w, y));
        }
        orow[col] = acc;
    }
}

}  // namespace cb200
