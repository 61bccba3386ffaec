// C-ABI entry points of libcatlass_b200.so (declared in include/catlass_b200.h).
// Host code only validates arguments, encodes tensor maps and launches; it never touches matrix data and
// has no CPU compute path: without a sm_100 device every launch entry returns an error.
#include <cstring>
#include <cuda_bf16.h>

#include <cmath>
#include <cstdlib>

#include "host_runtime.cuh"
#include "w8a8_gemm.cuh"
#include "w8a8_gemm_pair.cuh"
#include "w8a8_smallm.cuh"
#include "w4a8_gemm.cuh"
#include "quant_int8.cuh"
#include "mx_gemm.cuh"
#include "mx_gemm_pair.cuh"
#include "routing.cuh"
#include "ingest.cuh"
#include "mx_quantize.cuh"

using namespace cb200;
using namespace cb200::host;

namespace {

// Tuning hooks for sweeps.  They exist only in builds made with -DCB200_DEVELOPER_KNOBS (never the shipped
// library): there `dev_knob` reads an environment variable, here it is the constant default, so nothing in the
// environment can change what the library does.
#ifdef CB200_DEVELOPER_KNOBS
inline long dev_knob(const char* name, long dflt)
{
    const char* e = getenv(name);
    return e == nullptr ? dflt : atol(e);
}
#else
constexpr long dev_knob(const char*, long dflt)
{
    return dflt;
}
#endif

// One-time per-device set-up of a launcher (function attributes, occupancy queries), safe from several host
// threads: the flag is published after the set-up ran, under the mutex.
struct PerDeviceOnce {
    std::mutex mu;
    std::atomic<bool> done[kMaxDevices];
    PerDeviceOnce()
    {
        for (auto& d : done) {
            d.store(false, std::memory_order_relaxed);
        }
    }
    template <class F>
    int run(int dev, F&& f)
    {
        if (done[dev].load(std::memory_order_acquire)) {
            return CB200_SUCCESS;
        }
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev].load(std::memory_order_relaxed)) {
            const int rc = f();
            if (rc != CB200_SUCCESS) {
                return rc;
            }
            done[dev].store(true, std::memory_order_release);
        }
        return CB200_SUCCESS;
    }
};

int current_device(int* dev)
{
    CB200_CUDA_TRY(cudaGetDevice(dev));
    return (*dev < 0 || *dev >= kMaxDevices) ? CB200_INVALID : CB200_SUCCESS;
}

struct W8A8Problem {
    uint32_t m, n, k;
    uint32_t group_count;  // 0 = dense
    uint32_t group_list_type;
    uint32_t layout_a;
    uint32_t layout_b;
    const void* a;
    const void* b;
    const void* group_list;
    const void* scale;      // null in scalar mode
    const void* per_token;  // null when the operator has no per-token factor
    void* d;
    int32_t* acc;
    uint32_t block_num;
    uint32_t scale_type = CB200_DTYPE_F32;
    uint32_t d_type = CB200_DTYPE_BF16;
    uint32_t scale_stride = 0;   // elements between the channel-scale vectors of two groups
    bool has_per_token = true;
    bool scalar_mode = false;
    float scalar_scale = 0.0f;
    bool static_weights = false;
};

uint32_t scale_elem_bytes(uint32_t type)
{
    return type == CB200_DTYPE_F32 ? 4u : (type == CB200_DTYPE_F32_IN_U64 ? 8u : 2u);
}

int check_w8a8(const W8A8Problem& q)
{
    if (q.scale_type > CB200_DTYPE_F32_IN_U64 || (q.d_type != 0 && q.d_type != CB200_DTYPE_BF16 &&
                                                  q.d_type != CB200_DTYPE_F16)) {
        return CB200_INVALID;
    }
    if (q.a == nullptr || q.b == nullptr || (!q.scalar_mode && q.scale == nullptr) ||
        (q.has_per_token && q.per_token == nullptr) || q.d == nullptr) {
        return (q.m == 0 || q.n == 0) ? CB200_SUCCESS : CB200_INVALID;
    }
    if (q.layout_a != CB200_ROW_MAJOR && q.layout_a != CB200_COLUMN_MAJOR) {
        return CB200_INVALID;
    }
    if (q.layout_a == CB200_COLUMN_MAJOR && q.group_count != 0) {
        return CB200_INVALID;  // slice-M groups cut A by rows: the reference's grouped kernels take row-major A
    }
    if (q.layout_b != CB200_ROW_MAJOR && q.layout_b != CB200_COLUMN_MAJOR && q.layout_b != CB200_ZN) {
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
        if (q.layout_a == CB200_ROW_MAJOR && (q.k & 15u) != 0) {
            return CB200_INVALID;  // A rows are k bytes apart
        }
        if (q.layout_a == CB200_COLUMN_MAJOR && (q.m & 15u) != 0) {
            return CB200_INVALID;  // A columns are m bytes apart
        }
        if (q.layout_b == CB200_COLUMN_MAJOR && (q.k & 15u) != 0) {
            return CB200_INVALID;  // B columns are k bytes apart
        }
        if (q.layout_b == CB200_ROW_MAJOR && (q.n & 15u) != 0) {
            return CB200_INVALID;  // row-major B rows are n bytes apart
        }
    }
    const uintptr_t scale_mask = scale_elem_bytes(q.scale_type) - 1u;
    if ((reinterpret_cast<uintptr_t>(q.d) & 1u) != 0 || (reinterpret_cast<uintptr_t>(q.scale) & scale_mask) != 0 ||
        (reinterpret_cast<uintptr_t>(q.per_token) & scale_mask) != 0) {
        return CB200_INVALID;
    }
    if ((q.n & 7u) == 0 && !aligned16(q.d)) {
        return CB200_INVALID;  // vector stores of 8 outputs
    }
    return CB200_SUCCESS;
}

void fill_params(W8A8Params& p, const W8A8Problem& q, const DeviceState& dev)
{
    p.tma_store = 0;
    p.m = q.m;
    p.n = q.n;
    p.k = q.k;
    p.group_count = q.group_count;
    p.group_list_is_i32 = q.group_list_type == CB200_GROUP_LIST_INT32 ? 1u : 0u;
    p.num_k_blocks = (q.k + kBlockKBytes - 1) / kBlockKBytes;
    p.group_list = q.group_list;
    p.scale = q.scale;
    p.per_token = q.has_per_token ? q.per_token : nullptr;
    p.d = static_cast<uint16_t*>(q.d);
    p.acc = q.acc;
    p.status = dev.status;
    p.scale_type = q.scale_type;
    p.scale_stride = q.scale_stride;
    p.scalar_mode = q.scalar_mode ? 1u : 0u;
    p.scalar_scale = q.scalar_scale;
    p.out_f16 = q.d_type == CB200_DTYPE_F16 ? 1u : 0u;
    p.static_weights = q.static_weights ? 1u : 0u;
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
    fill_params(p, q, dev);

    auto kernel = w8a8_gemm_kernel<BN, kBMn>;
    static PerDeviceOnce once;
    int devid = 0;
    int rc_dev = current_device(&devid);
    if (rc_dev != CB200_SUCCESS) {
        return rc_dev;
    }
    rc_dev = once.run(devid, [&]() -> int {
        CB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotalBytes));
        return CB200_SUCCESS;
    });
    if (rc_dev != CB200_SUCCESS) {
        return rc_dev;
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

// 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2): the default for problems with more than 128 columns.
template <BLayout kB, bool kAMn>
int launch_w8a8_pair(const W8A8Problem& q, const DeviceState& dev, cudaStream_t stream)
{
    constexpr bool kBMn = kB == BLayout::kRowMajor;
    using S = W8A8PairSmem;
    static_assert(S::kTotalBytes <= 232448, "shared memory budget of one CTA");
    CUtensorMap tmap_a, tmap_b;
    const uint32_t groups = q.group_count == 0 ? 1u : q.group_count;
    {
        // row-major A: rows of k bytes; column-major A: k rows of m bytes (a tile is 128 bytes of M x 128 rows of K)
        const uint64_t dims_k[2] = {q.k, q.m};
        const uint64_t dims_m[2] = {q.m, q.k};
        const uint64_t strides[1] = {kAMn ? q.m : q.k};
        const uint32_t box[2] = {128, 128};
        int rc = encode_tmap_u8(&tmap_a, q.a, 2, kAMn ? dims_m : dims_k, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    if constexpr (kB == BLayout::kZN) {
        // zN: [group][n/32 panels][round16(k) rows][32 bytes]; a CTA loads four panels x 128 rows
        const uint64_t k_round = (static_cast<uint64_t>(q.k) + 15u) / 16u * 16u;
        const uint64_t panels = (static_cast<uint64_t>(q.n) + 31u) / 32u;
        const uint64_t dims[4] = {32, q.k, panels, groups};
        const uint64_t strides[3] = {32, k_round * 32u, panels * k_round * 32u};
        const uint32_t box[4] = {32, 128, 4, 1};
        int rc = encode_tmap_u8(&tmap_b, q.b, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    } else {
        // each CTA of a pair loads 128 of the tile's 256 columns
        const uint64_t dims_mn[3] = {q.n, q.k, groups};
        const uint64_t dims_k[3] = {q.k, q.n, groups};
        const uint64_t strides[2] = {kBMn ? q.n : q.k, static_cast<uint64_t>(q.n) * q.k};
        const uint32_t box[3] = {128, 128, 1};
        int rc = encode_tmap_u8(&tmap_b, q.b, 3, kBMn ? dims_mn : dims_k, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    W8A8Params p;
    fill_params(p, q, dev);
    // D as a byte tensor [m][2n] for the epilogue's TMA stores (32 rows x 64 bytes per store): possible when the
    // row pitch is a multiple of 16 bytes; otherwise every row is stored by its thread
    CUtensorMap tmap_d;
    memset(&tmap_d, 0, sizeof(tmap_d));
    if (dev_knob("CB200_W8A8_TMA_STORE", 1) != 0 && (q.n & 7u) == 0 && aligned16(q.d)) {
        const uint64_t dims[2] = {static_cast<uint64_t>(q.n) * 2u, q.m};
        const uint64_t strides[1] = {static_cast<uint64_t>(q.n) * 2u};
        const uint32_t box[2] = {64, 32};
        int rc = encode_tmap_u8(&tmap_d, q.d, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        p.tma_store = 1;
    }

    auto kernel = w8a8_pair_kernel<kB, kAMn>;
    static PerDeviceOnce once;
    int devid = 0;
    int rc = current_device(&devid);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    rc = once.run(devid, [&]() -> int {
        CB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotalBytes));
        return CB200_SUCCESS;
    });
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    const uint64_t n_tiles = (q.n + kPairBN - 1) / kPairBN;
    const uint64_t max_tiles = (static_cast<uint64_t>((q.m + kPairTileM - 1) / kPairTileM) + groups) * n_tiles;
    uint32_t pairs = static_cast<uint32_t>(dev.sm_count) / 2u;
    if (q.block_num != 0 && q.block_num / 2u < pairs) {
        pairs = q.block_num / 2u == 0 ? 1u : q.block_num / 2u;
    }
    if (max_tiles < pairs) {
        pairs = static_cast<uint32_t>(max_tiles);
    }
    if (pairs == 0) {
        return CB200_SUCCESS;
    }
    kernel<<<2 * pairs, kGemmThreads, S::kTotalBytes, stream>>>(tmap_a, tmap_b, tmap_d, p);
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

// Few-token (m <= 128) dense problems: weights on the UMMA M axis, K split over a cluster.
template <bool kWMn>
int launch_smallm(const W8A8Problem& q, const DeviceState& dev, cudaStream_t stream)
{
    SmallMParams p;
    p.m = q.m;
    p.n = q.n;
    p.k = q.k;
    p.mt = (q.m + 15u) & ~15u;
    p.num_k_blocks = (q.k + kBlockKBytes - 1) / kBlockKBytes;
    // Tile height R (weight rows per CTA) and K split S: one CTA per SM, so the grid should be a whole
    // number of waves of sm_count CTAs with as little padding as possible.  Cost of a candidate, in
    // "bytes": every wave pays a fixed start-up/drain equivalent plus its share of the weight stream;
    // a split adds the cluster reduction.
    const uint32_t max_by_partials = 1u + (96u * 1024u) / (kSmallMTileN * p.mt * 4u);
    uint32_t splits = 1, tile_rows = kSmallMTileN;
    auto kernel = w8a8_smallm_kernel<kWMn>;
    static PerDeviceOnce once;
    static int resident_ctas[kMaxDevices][4] = {};  // co-resident CTAs for cluster sizes 1, 2, 4, 8
    int devid = 0;
    int rc_dev = current_device(&devid);
    if (rc_dev != CB200_SUCCESS) {
        return rc_dev;
    }
    rc_dev = once.run(devid, [&]() -> int {
        CB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        // clusters must sit inside one GPC, so fewer CTAs than SMs may be resident at once: ask the runtime
        for (int i = 0; i < 4; ++i) {
            cudaLaunchConfig_t oc = {};
            oc.gridDim = dim3(static_cast<unsigned>(dev.sm_count) * 8u, 1, 1);
            oc.blockDim = dim3(kSmallMThreads, 1, 1);
            oc.dynamicSmemBytes = 200 * 1024;  // one CTA per SM, as launched below
            cudaLaunchAttribute oa[1];
            oa[0].id = cudaLaunchAttributeClusterDimension;
            oa[0].val.clusterDim.x = 1u << i;
            oa[0].val.clusterDim.y = 1;
            oa[0].val.clusterDim.z = 1;
            oc.attrs = oa;
            oc.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &oc) != cudaSuccess || clusters <= 0) {
                clusters = dev.sm_count >> i;
                (void)cudaGetLastError();
            }
            resident_ctas[devid][i] = clusters << i;
        }
        return CB200_SUCCESS;
    });
    if (rc_dev != CB200_SUCCESS) {
        return rc_dev;
    }
    {
        // Time of a candidate split: every wave pays a fixed start-up / epilogue (a split adds the cluster reduction),
        // and the weight stream is bounded both by what one CTA's pipeline moves (~70 GB/s: measured, 128 rows x
        // 14336 bytes in 7.7 us) and by what HBM delivers to all of them.  The tile is always 128 weight rows:
        // shorter tiles make more CTAs but each K block takes a CTA as long as before (the MMA reads 128 rows
        // anyway), and measured they never won (16 x 14336 x 4096: 112 CTAs of 128 rows beat 138 of 104 by 2 %;
        // 16 x 4096 x 14336, 2-way split: 64 CTAs of 128 rows 15.2 us, 114 of 72 rows 15.7 us).
        const double fixed = 3.5e-6, reduce = 2.0e-6, per_cta_rate = 70.0e9, hbm_rate = 6.0e12;
        const double total_bytes = static_cast<double>(q.n) * q.k;
        const uint32_t tiles = (q.n + kSmallMTileN - 1) / kSmallMTileN;
        double best = 1e300;
        int si = 0;
        for (uint32_t s = 1; s <= static_cast<uint32_t>(kSmallMMaxSplits); s *= 2, ++si) {
            if (s > max_by_partials || s > p.num_k_blocks) {
                break;
            }
            const double sm = static_cast<double>(resident_ctas[devid][si]);
            const double waves = ceil(static_cast<double>(tiles) * s / sm);
            const double kb_per = ceil(static_cast<double>(p.num_k_blocks) / s);
            const double cta_bytes = static_cast<double>(kSmallMTileN + p.mt) * kb_per * kBlockKBytes;
            const double stream = waves * cta_bytes / per_cta_rate;
            const double cost = waves * (fixed + (s > 1 ? reduce : 0.0)) +
                                (stream > total_bytes / hbm_rate ? stream : total_bytes / hbm_rate);
            if (cost < best) {
                best = cost;
                splits = s;
            }
        }
    }
    p.tile_rows = tile_rows;
    // a ring stage holds 4 neighbouring K blocks: 512 contiguous bytes per weight row are requested together
    uint32_t kbs = static_cast<uint32_t>(dev_knob("CB200_SMALLM_KBS", 0));
    kbs = (kbs >= 1 && kbs <= 8) ? kbs : 4;
    uint32_t ring_budget = static_cast<uint32_t>(dev_knob("CB200_SMALLM_RING_KB", 216));
    ring_budget = (ring_budget >= 36 && ring_budget <= 216 ? ring_budget : 216u) * 1024u;
    while (kbs > 1 && 2 * smallm_stage_bytes(p.mt, kbs) > ring_budget) {
        kbs /= 2;  // wide token panels: keep at least two stages
    }
    p.kbs = kbs;
    const uint32_t stage_bytes = smallm_stage_bytes(p.mt, kbs);
    uint32_t stages = ring_budget / stage_bytes;
    {
        const uint32_t v = static_cast<uint32_t>(dev_knob("CB200_SMALLM_SPLITS", 0));
        if ((v == 1 || v == 2 || v == 4 || v == 8) && v <= max_by_partials && v <= p.num_k_blocks) {
            splits = v;
        }
        const uint32_t r = static_cast<uint32_t>(dev_knob("CB200_SMALLM_ROWS", 0));
        if (!kWMn && r >= 8 && r <= 128 && r % 8 == 0) {
            p.tile_rows = r;
        }
        const uint32_t st = static_cast<uint32_t>(dev_knob("CB200_SMALLM_STAGES", 0));
        if (st >= 2 && st * stage_bytes <= 216u * 1024u) {
            stages = st;
        }
    }
    p.splits = splits;
    p.own_partials = (smallm_own_partials(p.mt, splits) && dev_knob("CB200_SMALLM_OWN_PARTIALS", 1) != 0) ? 1u : 0u;
    if (p.own_partials) {
        // the partial sums take their memory out of the ring's budget; K blocks per stage are re-chosen so that
        // whole stages fill what is left (4 blocks = 72 KB stages would leave 48 of 192 KB unused)
        const uint32_t budget = ring_budget - (splits - 1) * kSmallMTileN * p.mt * 4u;
        uint32_t best_kbs = p.kbs, best_fill = (budget / smallm_stage_bytes(p.mt, p.kbs)) * smallm_stage_bytes(p.mt, p.kbs);
        for (uint32_t cand = p.kbs / 2; cand >= 1; cand /= 2) {
            const uint32_t sb = smallm_stage_bytes(p.mt, cand);
            if ((budget / sb) * sb > best_fill) {
                best_fill = (budget / sb) * sb;
                best_kbs = cand;
            }
        }
        if (dev_knob("CB200_SMALLM_KBS", 0) == 0) {
            p.kbs = best_kbs;
        }
        stages = budget / smallm_stage_bytes(p.mt, p.kbs);
    }
    stages = stages > static_cast<uint32_t>(kSmallMMaxStages) ? kSmallMMaxStages : (stages < 2 ? 2 : stages);
    p.stages = stages;
    p.scale = q.scale;
    p.per_token = q.has_per_token ? q.per_token : nullptr;
    p.d = static_cast<uint16_t*>(q.d);
    p.acc = q.acc;
    p.status = dev.status;
    p.scale_type = q.scale_type;
    p.scalar_mode = q.scalar_mode ? 1u : 0u;
    p.scalar_scale = q.scalar_scale;
    p.out_f16 = q.d_type == CB200_DTYPE_F16 ? 1u : 0u;
    p.static_weights = q.static_weights ? 1u : 0u;

    CUtensorMap tmap_w, tmap_x;
    {
        const uint64_t dims_k[2] = {q.k, q.n};
        const uint64_t dims_n[2] = {q.n, q.k};
        const uint64_t strides[1] = {kWMn ? q.n : q.k};
        const uint32_t box[2] = {128, kWMn ? 128u : p.tile_rows};
        int rc = encode_tmap_u8(&tmap_w, q.b, 2, kWMn ? dims_n : dims_k, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    {
        const uint64_t dims[2] = {q.k, q.m};
        const uint64_t strides[1] = {q.k};
        const uint32_t box[2] = {kBlockKBytes, p.mt};
        int rc = encode_tmap_u8(&tmap_x, q.a, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    const uint32_t smem = smallm_smem_bytes(p.mt, p.stages, p.splits, p.kbs, p.own_partials != 0);
    const uint32_t n_tiles = (q.n + p.tile_rows - 1) / p.tile_rows;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles * p.splits, 1, 1);
    cfg.blockDim = dim3(kSmallMThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this kernel's set-up (and, for static weights, its first weight loads) may
    // overlap the tail of the kernel before it on the stream; it waits (griddepcontrol.wait) before it reads
    // anything else from global memory or writes D
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dev_knob("CB200_SMALLM_PDL", 1) != 0 ? 2 : 1;
    CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmap_w, tmap_x, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

int run_w8a8(const W8A8Problem& q, void* stream_v)
{
    int rc = check_w8a8(q);
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
        zero_rows_kernel<<<dev->sm_count * 4, 256, 0, stream>>>(static_cast<uint16_t*>(q.d), q.group_list,
                                                                q.group_list_type == CB200_GROUP_LIST_INT32,
                                                                q.group_count, q.m, q.n);
        CB200_CUDA_TRY(cudaGetLastError());
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return CB200_SUCCESS;
    }
    if (q.layout_a == CB200_COLUMN_MAJOR) {  // MN-major A tiles: the pair kernel, whatever the shape
        switch (q.layout_b) {
            case CB200_ZN: return launch_w8a8_pair<BLayout::kZN, true>(q, *dev, stream);
            case CB200_ROW_MAJOR: return launch_w8a8_pair<BLayout::kRowMajor, true>(q, *dev, stream);
            default: return launch_w8a8_pair<BLayout::kColumnMajor, true>(q, *dev, stream);
        }
    }
    if (q.layout_b == CB200_ZN) {
        return launch_w8a8_pair<BLayout::kZN, false>(q, *dev, stream);  // fractal weights: always the pair kernel
    }
    const bool b_mn = q.layout_b == CB200_ROW_MAJOR;
    if (q.group_count == 0 && q.m <= 128) {
        return b_mn ? launch_smallm<true>(q, *dev, stream) : launch_smallm<false>(q, *dev, stream);
    }
    if (q.n > 128) {
        if (dev_knob("CB200_W8A8_PAIR", 1) != 0) {  // 0: the single-CTA 128 x 256 kernel, for comparisons
            return b_mn ? launch_w8a8_pair<BLayout::kRowMajor, false>(q, *dev, stream)
                        : launch_w8a8_pair<BLayout::kColumnMajor, false>(q, *dev, stream);
        }
        return b_mn ? launch_w8a8<256, true>(q, *dev, stream) : launch_w8a8<256, false>(q, *dev, stream);
    }
    return b_mn ? launch_w8a8<128, true>(q, *dev, stream) : launch_w8a8<128, false>(q, *dev, stream);
}

inline uint64_t align256(uint64_t v)
{
    return (v + 255u) & ~static_cast<uint64_t>(255u);
}

// How a W4A8 call is served: in place (fast path), or through the ingestion pre-pass that writes K-padded,
// K-packed copies of both operands into the workspace.
struct W4Plan {
    bool ingest;
    uint32_t k_padded;    // K the kernel runs on: a whole number of scale groups of 128-element blocks
    uint32_t group_size;  // scale group the kernel runs with
    uint64_t a_bytes, w_bytes;
};

int plan_w4a8(const cb200_w4a8_matmul_args* a, W4Plan* plan)
{
    if (a == nullptr) {
        return CB200_INVALID;
    }
    if (a->m == 0 || a->n == 0) {
        plan->ingest = false;
        return CB200_SUCCESS;
    }
    if (a->a == nullptr || a->w_packed == nullptr || a->weight_scale == nullptr || a->per_token_scale == nullptr ||
        a->d == nullptr) {
        return CB200_INVALID;
    }
    if (a->k == 0 || a->group_size == 0 || a->pack_axis > CB200_W4_PACKED_ALONG_N) {
        return CB200_INVALID;
    }
    const bool one_group = a->group_size >= a->k;
    if (!one_group && (a->group_size % 128u) != 0) {
        return CB200_INVALID;
    }
    // 16 x the int32 sum of a group must stay exactly convertible to fp32: at most 16384 elements per group
    if ((one_group ? a->k : a->group_size) > 16384u) {
        return CB200_INVALID;
    }
    if (a->m > 0x7fffff00u || a->n > 0x7fffff00u || a->k > 0x7fffff00u) {
        return CB200_INVALID;
    }
    if (a->d_type != 0 && a->d_type != CB200_DTYPE_BF16 && a->d_type != CB200_DTYPE_F16) {
        return CB200_INVALID;
    }
    if ((reinterpret_cast<uintptr_t>(a->d) & 1u) != 0 || (reinterpret_cast<uintptr_t>(a->weight_scale) & 3u) != 0 ||
        (reinterpret_cast<uintptr_t>(a->per_token_scale) & 3u) != 0) {
        return CB200_INVALID;
    }
    if ((a->n & 7u) == 0 && !aligned16(a->d)) {
        return CB200_INVALID;  // vector stores of 8 outputs
    }
    const uint32_t unit = one_group ? 128u : a->group_size;
    plan->k_padded = (a->k + unit - 1u) / unit * unit;
    plan->group_size = one_group ? plan->k_padded : a->group_size;
    plan->ingest = a->pack_axis != CB200_W4_PACKED_ALONG_K || plan->k_padded != a->k || !aligned16(a->a) ||
                   !aligned16(a->w_packed);
    plan->a_bytes = align256(static_cast<uint64_t>(a->m) * plan->k_padded);
    plan->w_bytes = align256(static_cast<uint64_t>(a->n) * (plan->k_padded / 2u));
    return CB200_SUCCESS;
}

// An MX problem as the launcher sees it: the dense call is one group whose rows are all of A.
struct MxProblem {
    uint32_t m, n, k;
    uint32_t group_count;      // 0 = dense
    uint32_t format;
    uint32_t layout_a, layout_b;
    uint32_t group_list_type, group_list_is_prefix_sum;
    const void* a;
    const void* b;
    const void* group_list;
    const void* scale_a;
    const void* scale_b;
    void* d;
    void* workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t flags;
    // SwiGLU + MX quantisation instead of the plain output: d = Q (E4M3 [m][n/2]), q_scale = E8M0 [m][n/64]
    bool swiglu_quant;
    void* q_scale;
    // finalize routing instead of the plain output: d = out (fp32 [batch][n]), rows added with weights
    bool routing;
    const void* logit;
    const void* row_index;
    const void* bias;
    const void* shared_input;
    uint32_t row_index_i32, batch, shared_rows, shared_offset;
    float shared_weight;
};

// How an MX call is served.  The kernel wants both operands with rows along K, padded to whole K stages
// (128 E4M3 / 256 E2M1 elements) and 16-byte aligned; an operand that is not is rewritten by the ingestion
// pre-pass into the workspace, behind the re-tiled scales (and, for a grouped problem, the row-tile table).
struct MxPlan {
    uint32_t k_padded;
    uint32_t row_bytes;       // bytes of one padded operand row
    uint32_t max_row_tiles;   // 128-row tiles of A at most: ceil(m/128), plus one partial tile per group
    uint32_t b_matrices;      // weight matrices: 1, or the group count
    bool ingest_a, ingest_b;
    uint64_t table_bytes, sfa_bytes, sfb_bytes, a_bytes, b_bytes;
    uint64_t total() const
    {
        return table_bytes + sfa_bytes + sfb_bytes + (ingest_a ? a_bytes : 0) + (ingest_b ? b_bytes : 0);
    }
};

int plan_mx(const MxProblem& q, MxPlan* plan)
{
    *plan = MxPlan{};
    if (q.m == 0 || q.n == 0) {
        return CB200_SUCCESS;
    }
    if (q.a == nullptr || q.b == nullptr || q.scale_a == nullptr || q.scale_b == nullptr || q.d == nullptr) {
        return CB200_INVALID;
    }
    if (q.format != CB200_MX_E4M3 && q.format != CB200_MX_E2M1) {
        return CB200_INVALID;
    }
    if ((q.layout_a != CB200_ROW_MAJOR && q.layout_a != CB200_COLUMN_MAJOR) ||
        (q.layout_b != CB200_ROW_MAJOR && q.layout_b != CB200_COLUMN_MAJOR)) {
        return CB200_INVALID;
    }
    if (q.group_count != 0) {
        if (q.group_count > static_cast<uint32_t>(kMaxGroups) || q.group_list == nullptr ||
            q.layout_a != CB200_ROW_MAJOR ||  // slice-M groups cut A by rows
            (q.group_list_type != CB200_GROUP_LIST_INT64 && q.group_list_type != CB200_GROUP_LIST_INT32)) {
            return CB200_INVALID;
        }
    }
    if ((q.flags & ~CB200_MX_OUT_F32) != 0) {
        return CB200_INVALID;
    }
    if (q.k == 0 || q.m > 0x7fffff00u || q.n > 0x7fffff00u || q.k > 0x7fffff00u) {
        return CB200_INVALID;
    }
    const bool f32 = (q.flags & CB200_MX_OUT_F32) != 0;
    if (q.swiglu_quant) {
        // tiles pair 128 columns of either half of C, and the halves' scale blocks start on 128-row boundaries
        if (q.group_count == 0 || q.format != CB200_MX_E4M3 || q.flags != 0 || (q.n % 256u) != 0 ||
            q.q_scale == nullptr || !aligned16(q.d)) {
            return CB200_INVALID;
        }
    } else if (q.routing) {
        if (q.group_count == 0 || q.format != CB200_MX_E4M3 || q.flags != 0 || q.logit == nullptr ||
            q.row_index == nullptr || q.batch == 0 || (reinterpret_cast<uintptr_t>(q.d) & 3u) != 0 ||
            ((q.n & 3u) == 0 && !aligned16(q.d)) || (reinterpret_cast<uintptr_t>(q.logit) & 3u) != 0 ||
            (reinterpret_cast<uintptr_t>(q.row_index) & (q.row_index_i32 ? 3u : 7u)) != 0 ||
            (reinterpret_cast<uintptr_t>(q.bias) & 1u) != 0 || (reinterpret_cast<uintptr_t>(q.shared_input) & 1u) != 0) {
            return CB200_INVALID;
        }
        if (q.shared_input != nullptr &&
            (q.shared_offset > q.batch || q.shared_rows > q.batch - q.shared_offset)) {
            return CB200_INVALID;
        }
    } else {
        if ((reinterpret_cast<uintptr_t>(q.d) & (f32 ? 3u : 1u)) != 0) {
            return CB200_INVALID;
        }
        if (((q.n & (f32 ? 3u : 7u)) == 0) && !aligned16(q.d)) {
            return CB200_INVALID;  // 16-byte vector stores
        }
    }
    const bool fp4 = q.format == CB200_MX_E2M1;
    const uint32_t kmul = fp4 ? 256u : 128u;
    plan->k_padded = (q.k + kmul - 1u) / kmul * kmul;
    plan->row_bytes = fp4 ? plan->k_padded / 2u : plan->k_padded;
    plan->ingest_a = q.layout_a != CB200_ROW_MAJOR || plan->k_padded != q.k || !aligned16(q.a);
    plan->ingest_b = q.layout_b != CB200_COLUMN_MAJOR || plan->k_padded != q.k || !aligned16(q.b);
    plan->b_matrices = q.group_count == 0 ? 1u : q.group_count;
    // 128-row blocks at most: ceil(m/128), plus one partial 128-row tile per group, or (CTA pairs: 256-row tiles of two
    // blocks each) up to two blocks per group
    plan->max_row_tiles = (q.m + 127u) / 128u + 2u * q.group_count;
    const uint64_t kq = plan->k_padded / 128u;
    plan->table_bytes = q.group_count == 0 ? 0 : align256(static_cast<uint64_t>(plan->max_row_tiles) * 16u + 16u);
    // scale blocks of 128 rows; B's are padded to whole 256-column tiles
    plan->sfa_bytes = static_cast<uint64_t>(plan->max_row_tiles) * kq * 512u;
    plan->sfb_bytes = static_cast<uint64_t>(plan->b_matrices) * 2u * ((q.n + 255u) / 256u) * kq * 512u;
    plan->a_bytes = align256(static_cast<uint64_t>(q.m) * plan->row_bytes);
    plan->b_bytes = align256(static_cast<uint64_t>(plan->b_matrices) * q.n * plan->row_bytes);
    return CB200_SUCCESS;
}

// `batch` operands into their canonical form: `rows` rows of row_bytes bytes along K each.
// stored_k_major: the caller's arrays are [k][rows] (elements, packed two per byte along `rows` for E2M1).
void ingest_mx_operand(const void* src, uint8_t* dst, uint32_t rows, uint32_t k, bool fp4, bool stored_k_major,
                       uint32_t row_bytes, uint32_t batch, int sm_count, cudaStream_t stream)
{
    const uint8_t* s = static_cast<const uint8_t*>(src);
    const uint32_t per_batch = static_cast<uint32_t>(sm_count) * 8u / (batch > 8u ? 8u : batch);
    const dim3 grid(per_batch == 0 ? 1u : per_batch, batch, 1);
    const uint64_t dst_batch = static_cast<uint64_t>(rows) * row_bytes;
    if (!stored_k_major) {
        const uint32_t valid = fp4 ? (k + 1u) / 2u : k;
        pad_rows_kernel<<<grid, 256, 0, stream>>>(s, dst, rows, valid, row_bytes, valid, fp4 ? (k & 1u) : 0u,
                                                  static_cast<uint64_t>(rows) * valid, dst_batch);
    } else if (fp4) {
        const uint64_t pitch = (rows + 1u) / 2u;
        transpose_nibbles_kernel<<<grid, 256, 0, stream>>>(s, dst, rows, k, pitch, row_bytes, pitch * k, dst_batch);
    } else {
        transpose_bytes_kernel<<<grid, dim3(32, 8), 0, stream>>>(s, dst, rows, k, rows, row_bytes,
                                                                 static_cast<uint64_t>(rows) * k, dst_batch);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
}

template <bool kFp4, bool kGrouped, int kEpi = kMxEpiPlain>
int launch_mx(const MxProblem& q, const MxPlan& plan, const DeviceState& dev, cudaStream_t stream)
{
    constexpr bool kSwiglu = kEpi == kMxEpiSwiglu;
    // Large problems run on CTA pairs (256 x 256 tiles, half the B traffic per SM): dense ones with at least two waves
    // of pair tiles, grouped ones (plain and SwiGLU epilogues) whose groups average at least 512 rows.
    constexpr bool kPairCapable = kEpi == kMxEpiPlain || kSwiglu;
    const uint32_t pairs = static_cast<uint32_t>(dev.sm_count) / 2u;
    const uint32_t pair_n_tiles = kSwiglu ? q.n / 256u : (q.n + 255u) / 256u;
    bool use_pair = false;
    if constexpr (kPairCapable) {
        const uint64_t pair_tiles = static_cast<uint64_t>((q.m + 255u) / 256u) * pair_n_tiles;
        use_pair = q.m >= 512u && pair_tiles >= 2ull * pairs && (q.block_num == 0 || q.block_num >= 2u * pairs) &&
                   (!kGrouped || q.m / q.group_count >= 512u);
        const long v = dev_knob("CB200_MX_PAIR", -1);
        if (v == 0) {
            use_pair = false;
        } else if (v == 1) {
            use_pair = pairs != 0;
        }
    }
    const uint32_t tile_rows = use_pair ? 256u : 128u;
    uint8_t* ws = static_cast<uint8_t*>(q.workspace);
    int4* table = reinterpret_cast<int4*>(ws);
    uint32_t* num_row_tiles = reinterpret_cast<uint32_t*>(ws + static_cast<uint64_t>(plan.max_row_tiles) * 16u);
    uint8_t* sfa = ws + plan.table_bytes;
    uint8_t* sfb = sfa + plan.sfa_bytes;
    const void* a_ptr = q.a;
    const void* b_ptr = q.b;
    {
        uint8_t* next = sfb + plan.sfb_bytes;
        if (plan.ingest_a) {
            ingest_mx_operand(q.a, next, q.m, q.k, kFp4, q.layout_a == CB200_COLUMN_MAJOR, plan.row_bytes, 1,
                              dev.sm_count, stream);
            a_ptr = next;
            next += plan.a_bytes;
        }
        if (plan.ingest_b) {
            ingest_mx_operand(q.b, next, q.n, q.k, kFp4, q.layout_b == CB200_ROW_MAJOR, plan.row_bytes, plan.b_matrices,
                              dev.sm_count, stream);
            b_ptr = next;
        }
    }
    if constexpr (kGrouped) {
        mx_group_plan_kernel<<<1, 1024, 0, stream>>>(q.group_list, q.group_list_type == CB200_GROUP_LIST_INT32 ? 1u : 0u,
                                                     q.group_list_is_prefix_sum, q.group_count, q.m, table, num_row_tiles,
                                                     tile_rows);
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    const uint32_t row_bytes = plan.row_bytes;
    const uint32_t sfb_blocks = 2u * ((q.n + 255u) / 256u);
    MxParams p;
    p.m = q.m;
    p.n = q.n;
    p.k = plan.k_padded;
    p.fp4 = kFp4 ? 1u : 0u;
    p.num_k_blocks = row_bytes / 128u;
    p.words_per_stage = kFp4 ? 2u : 1u;
    p.kq_total = plan.k_padded / 128u;
    // a band of the tile order holds ~32 MB of A (measured best at 8192^3: 32 row panels for fp8): its row panels
    // stay in L2 while the band's columns go by
    p.band_rows = (32u << 20) / (128u * (row_bytes > 0 ? row_bytes : 1u));
    p.band_rows = p.band_rows < 4u ? 4u : (p.band_rows > 64u ? 64u : p.band_rows);
    {
        const uint32_t v = static_cast<uint32_t>(dev_knob("CB200_MX_BAND", 0));
        if (v >= 1 && v <= 4096) {
            p.band_rows = v;
        }
    }
    p.sfa = sfa;
    p.sfb = sfb;
    p.d = q.d;
    p.status = dev.status;
    p.out_f32 = (q.flags & CB200_MX_OUT_F32) ? 1u : 0u;
    p.tile_table = kGrouped ? table : nullptr;
    p.num_row_tiles = kGrouped ? num_row_tiles : nullptr;
    p.sfb_blocks_per_group = sfb_blocks;
    p.q_scale = static_cast<uint8_t*>(q.q_scale);
    p.logit = static_cast<const float*>(q.logit);
    p.row_index = q.row_index;
    p.bias = static_cast<const __nv_bfloat16*>(q.bias);
    p.row_index_i32 = q.row_index_i32;
    p.batch = q.batch;
    if constexpr (kEpi == kMxEpiRouting) {
        finalize_routing_init_kernel<<<dev.sm_count * 4, 256, 0, stream>>>(
            static_cast<float*>(q.d), q.batch, q.n, static_cast<const __nv_bfloat16*>(q.shared_input), q.shared_weight,
            q.shared_offset, q.shared_input != nullptr ? q.shared_rows : 0u);
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }

    // the caller's scale arrays: ceil(k/32) blocks per row, held in an even number of columns; stored along the
    // operand's rows, or K-major when the operand itself is stored K-major
    const uint32_t kblocks = (q.k + 31u) / 32u;
    const uint32_t ks_pitch = (kblocks + 1u) & ~1u;
    mx_pack_scales_kernel<<<dim3(dev.sm_count * 2, 1, 1), 256, 0, stream>>>(
        static_cast<const uint8_t*>(q.scale_a), sfa, q.m, kblocks, ks_pitch, p.kq_total, plan.max_row_tiles,
        q.layout_a == CB200_COLUMN_MAJOR ? 1u : 0u, 0, 0, p.tile_table, p.num_row_tiles, tile_rows);
    {
        const uint32_t gx = plan.b_matrices > 8u ? static_cast<uint32_t>(dev.sm_count) / 4u : dev.sm_count * 2u;
        mx_pack_scales_kernel<<<dim3(gx, plan.b_matrices, 1), 256, 0, stream>>>(
            static_cast<const uint8_t*>(q.scale_b), sfb, q.n, kblocks, ks_pitch, p.kq_total, sfb_blocks,
            q.layout_b == CB200_ROW_MAJOR ? 1u : 0u, static_cast<uint64_t>(q.n) * ks_pitch,
            static_cast<uint64_t>(sfb_blocks) * p.kq_total * 512u, nullptr, nullptr);
    }
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(2, std::memory_order_relaxed);

    CUtensorMap tmap_a, tmap_b;
    {
        const uint64_t dims[2] = {row_bytes, q.m};
        const uint64_t strides[1] = {row_bytes};
        const uint32_t box[2] = {kBlockKBytes, kBlockM};
        int rc = encode_tmap_u8(&tmap_a, a_ptr, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    {
        const uint64_t dims[3] = {row_bytes, q.n, plan.b_matrices};
        const uint64_t strides[2] = {row_bytes, static_cast<uint64_t>(q.n) * row_bytes};
        // (the SwiGLU epilogue's tiles take 128 rows from either half of B: two loads per stage)
        const uint32_t box[3] = {kBlockKBytes, kSwiglu ? 128u : static_cast<uint32_t>(kMxBlockN), 1};
        int rc = encode_tmap_u8(&tmap_b, b_ptr, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    if constexpr (kPairCapable) {
        if (use_pair) {
            CUtensorMap tmap_bh, tmap_sfa, tmap_sfb;
            {
                const uint64_t dims[3] = {row_bytes, q.n, plan.b_matrices};
                const uint64_t strides[2] = {row_bytes, static_cast<uint64_t>(q.n) * row_bytes};
                const uint32_t box[3] = {kBlockKBytes, kMxBlockN / 2, 1};  // a CTA loads half of the tile's columns
                int rc = encode_tmap_u8(&tmap_bh, b_ptr, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
                if (rc != CB200_SUCCESS) {
                    return rc;
                }
            }
            const uint32_t words = kFp4 ? 2u : 1u;
            {
                // packed A scales [row block][kq_total][512 bytes] as rows of 256 bytes
                const uint64_t dims[2] = {256, 2ull * p.kq_total * plan.max_row_tiles};
                const uint64_t strides[1] = {256};
                const uint32_t box[2] = {256, 2u * words};
                int rc = encode_tmap_u8(&tmap_sfa, sfa, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
                if (rc != CB200_SUCCESS) {
                    return rc;
                }
            }
            {
                // packed B scales [column block][kq_total][512 bytes], all weight matrices one after the other
                const uint64_t dims[3] = {256, 2ull * p.kq_total, static_cast<uint64_t>(sfb_blocks) * plan.b_matrices};
                const uint64_t strides[2] = {256, 512ull * p.kq_total};
                const uint32_t box[3] = {256, 2u * words, 1};
                int rc = encode_tmap_u8(&tmap_sfb, sfb, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
                if (rc != CB200_SUCCESS) {
                    return rc;
                }
            }
            auto pair_kernel = mx_pair_kernel<kFp4, kGrouped, kEpi>;
            static PerDeviceOnce once_pair;
            int devid_pair = 0;
            int rc_pair = current_device(&devid_pair);
            if (rc_pair != CB200_SUCCESS) {
                return rc_pair;
            }
            rc_pair = once_pair.run(devid_pair, [&]() -> int {
                CB200_CUDA_TRY(cudaFuncSetAttribute(pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    MxPairSmem::kTotalBytes));
                return CB200_SUCCESS;
            });
            if (rc_pair != CB200_SUCCESS) {
                return rc_pair;
            }
            const uint64_t pair_tiles_max =
                static_cast<uint64_t>((q.m + 255u) / 256u + (kGrouped ? q.group_count : 0u)) * pair_n_tiles;
            const uint32_t launch_pairs = pair_tiles_max < pairs ? static_cast<uint32_t>(pair_tiles_max) : pairs;
            MxParams pp = p;
            pp.band_rows = p.band_rows / 2u < 2u ? 2u : p.band_rows / 2u;  // tile rows are 256 rows here: same bytes of A per band
            pair_kernel<<<2 * launch_pairs, kMxPairThreads, MxPairSmem::kTotalBytes, stream>>>(tmap_a, tmap_bh, tmap_sfa,
                                                                                           tmap_sfb, pp);
            CB200_CUDA_TRY(cudaGetLastError());
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return CB200_SUCCESS;
        }
    }
    auto kernel = mx_gemm_kernel<kFp4, kGrouped, kEpi>;
    static PerDeviceOnce once;
    int devid = 0;
    int rc_dev = current_device(&devid);
    if (rc_dev != CB200_SUCCESS) {
        return rc_dev;
    }
    rc_dev = once.run(devid, [&]() -> int {
        CB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem::kTotalBytes));
        return CB200_SUCCESS;
    });
    if (rc_dev != CB200_SUCCESS) {
        return rc_dev;
    }
    const uint64_t tiles =
        static_cast<uint64_t>(plan.max_row_tiles) * (kSwiglu ? q.n / 256u : (q.n + kMxBlockN - 1) / kMxBlockN);
    uint32_t grid = static_cast<uint32_t>(dev.sm_count);
    if (q.block_num != 0 && q.block_num < grid) {
        grid = q.block_num;
    }
    if (tiles < grid) {
        grid = static_cast<uint32_t>(tiles);
    }
    kernel<<<grid, mx_threads(kEpi), MxSmem::kTotalBytes, stream>>>(tmap_a, tmap_b, p);
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

MxProblem mx_dense_problem(const cb200_mx_matmul_args* a)
{
    MxProblem q{};
    q.m = a->m;
    q.n = a->n;
    q.k = a->k;
    q.group_count = 0;
    q.format = a->format;
    q.layout_a = a->layout_a;
    q.layout_b = a->layout_b;
    q.a = a->a;
    q.b = a->b;
    q.scale_a = a->scale_a;
    q.scale_b = a->scale_b;
    q.d = a->d;
    q.workspace = a->workspace;
    q.workspace_bytes = a->workspace_bytes;
    q.block_num = a->block_num;
    q.flags = a->flags;
    return q;
}

MxProblem mx_grouped_problem(const cb200_mx_grouped_matmul_args* a)
{
    MxProblem q{};
    q.m = a->m;
    q.n = a->n;
    q.k = a->k;
    q.group_count = a->group_count;
    q.format = a->format;
    q.layout_a = CB200_ROW_MAJOR;
    q.layout_b = a->layout_b;
    q.group_list_type = a->group_list_type;
    q.group_list_is_prefix_sum = a->group_list_kind == CB200_GROUP_LIST_PREFIX_SUMS ? 1u : 0u;
    q.a = a->a;
    q.b = a->b;
    q.group_list = a->group_list;
    q.scale_a = a->scale_a;
    q.scale_b = a->scale_b;
    q.d = a->d;
    q.workspace = a->workspace;
    q.workspace_bytes = a->workspace_bytes;
    q.block_num = a->block_num;
    q.flags = a->flags;
    return q;
}

MxProblem mx_swiglu_problem(const cb200_mx_grouped_swiglu_quant_args* a)
{
    MxProblem q{};
    q.m = a->m;
    q.n = a->n;
    q.k = a->k;
    q.group_count = a->group_count;
    q.format = CB200_MX_E4M3;
    q.layout_a = CB200_ROW_MAJOR;
    q.layout_b = a->layout_b;
    q.group_list_type = a->group_list_type;
    q.group_list_is_prefix_sum = a->group_list_kind == CB200_GROUP_LIST_PREFIX_SUMS ? 1u : 0u;
    q.a = a->a;
    q.b = a->b;
    q.group_list = a->group_list;
    q.scale_a = a->scale_a;
    q.scale_b = a->scale_b;
    q.d = a->q;
    q.q_scale = a->q_scale;
    q.swiglu_quant = true;
    q.workspace = a->workspace;
    q.workspace_bytes = a->workspace_bytes;
    q.block_num = a->block_num;
    q.flags = a->flags;
    return q;
}

MxProblem mx_routing_problem(const cb200_mx_grouped_finalize_routing_args* a)
{
    MxProblem q{};
    q.m = a->m;
    q.n = a->n;
    q.k = a->k;
    q.group_count = a->group_count;
    q.format = CB200_MX_E4M3;
    q.layout_a = CB200_ROW_MAJOR;
    q.layout_b = a->layout_b;
    q.group_list_type = a->group_list_type;
    q.group_list_is_prefix_sum = a->group_list_kind == CB200_GROUP_LIST_PREFIX_SUMS ? 1u : 0u;
    q.a = a->a;
    q.b = a->b;
    q.group_list = a->group_list;
    q.scale_a = a->scale_a;
    q.scale_b = a->scale_b;
    q.d = a->out;
    q.routing = true;
    q.logit = a->logit;
    q.row_index = a->row_index;
    q.bias = a->bias;
    q.shared_input = a->shared_input;
    q.row_index_i32 = a->row_index_type == CB200_GROUP_LIST_INT32 ? 1u : 0u;
    q.batch = a->batch;
    q.shared_rows = a->shared_rows;
    q.shared_offset = a->shared_offset;
    q.shared_weight = a->shared_weight;
    q.workspace = a->workspace;
    q.workspace_bytes = a->workspace_bytes;
    q.block_num = a->block_num;
    q.flags = a->flags & ~CB200_ROUTING_DETERMINISTIC;
    return q;
}

int run_mx(const MxProblem& q, void* stream_v);

// Deterministic finalize routing: the grouped matmul writes C (fp32) into the workspace, then the rows of every
// token are gathered in ascending row order (routing.cuh).  Workspace: C | lists | the matmul's own workspace.
struct RoutingDetPlan {
    uint64_t c_bytes, lists_bytes;
    MxPlan mx;
    uint64_t total() const { return c_bytes + lists_bytes + mx.total(); }
};

MxProblem routing_matmul_problem(const cb200_mx_grouped_finalize_routing_args* a, void* c, void* ws, uint64_t ws_bytes)
{
    MxProblem q = mx_routing_problem(a);
    q.routing = false;
    q.d = c;
    q.flags = CB200_MX_OUT_F32;
    q.workspace = ws;
    q.workspace_bytes = ws_bytes;
    return q;
}

int plan_routing_det(const cb200_mx_grouped_finalize_routing_args* a, RoutingDetPlan* plan)
{
    MxPlan check;
    MxProblem as_fused = mx_routing_problem(a);
    as_fused.flags = 0;
    int rc = plan_mx(as_fused, &check);  // the operands, lists and output as for the fused variant
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    plan->c_bytes = align256(static_cast<uint64_t>(a->m) * a->n * 4u);
    plan->lists_bytes = align256((static_cast<uint64_t>(a->group_count) + 1u + a->batch + a->batch + 1u + a->m) * 4u);
    // (an aligned non-null value stands in for C while planning: it is not dereferenced)
    return plan_mx(routing_matmul_problem(a, reinterpret_cast<void*>(uintptr_t{256}), nullptr, 0), &plan->mx);
}

int run_routing_det(const cb200_mx_grouped_finalize_routing_args* a, void* stream_v)
{
    RoutingDetPlan plan;
    int rc = plan_routing_det(a, &plan);
    if (rc != CB200_SUCCESS || a->m == 0 || a->n == 0) {
        return rc;
    }
    if (a->workspace == nullptr || a->workspace_bytes < plan.total() ||
        (reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0) {
        return CB200_INVALID;
    }
    DeviceState* dev = nullptr;
    rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    float* c = reinterpret_cast<float*>(ws);
    int32_t* lists = reinterpret_cast<int32_t*>(ws + plan.c_bytes);
    RoutingLists l;
    l.group_end = lists;
    l.total_rows = l.group_end + a->group_count;
    l.count = l.total_rows + 1;
    l.start = l.count + a->batch;
    l.order = l.start + a->batch + 1;
    rc = run_mx(routing_matmul_problem(a, c, ws + plan.c_bytes + plan.lists_bytes, plan.mx.total()), stream_v);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    const uint32_t idx_i32 = a->row_index_type == CB200_GROUP_LIST_INT32 ? 1u : 0u;
    routing_prepare_kernel<<<1, 1024, 0, stream>>>(a->group_list, a->group_list_type == CB200_GROUP_LIST_INT32 ? 1u : 0u,
                                                   a->group_list_kind == CB200_GROUP_LIST_PREFIX_SUMS ? 1u : 0u,
                                                   a->group_count, a->m, a->batch, l);
    const uint32_t row_blocks = (a->m + 255u) / 256u;
    const uint32_t grid = row_blocks < static_cast<uint32_t>(dev->sm_count) * 4u ? row_blocks : dev->sm_count * 4u;
    routing_count_kernel<<<grid, 256, 0, stream>>>(a->row_index, idx_i32, a->batch, l);
    routing_scan_kernel<<<1, 1024, 0, stream>>>(a->batch, l);
    routing_fill_kernel<<<grid, 256, 0, stream>>>(a->row_index, idx_i32, a->batch, l);
    routing_gather_kernel<<<a->batch, 256, 0, stream>>>(
        c, static_cast<float*>(a->out), a->n, a->group_count, static_cast<const float*>(a->logit),
        static_cast<const __nv_bfloat16*>(a->bias), static_cast<const __nv_bfloat16*>(a->shared_input), a->shared_weight,
        a->shared_offset, a->shared_input != nullptr ? a->shared_rows : 0u, l);
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(5, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

int run_mx(const MxProblem& q, void* stream_v)
{
    MxPlan plan;
    int rc = plan_mx(q, &plan);
    if (rc != CB200_SUCCESS || q.m == 0 || q.n == 0) {
        return rc;
    }
    if (q.workspace == nullptr || q.workspace_bytes < plan.total() ||
        (reinterpret_cast<uintptr_t>(q.workspace) & 255u) != 0) {
        return CB200_INVALID;
    }
    DeviceState* dev = nullptr;
    rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const bool fp4 = q.format == CB200_MX_E2M1;
    if (q.swiglu_quant) {
        return launch_mx<false, true, kMxEpiSwiglu>(q, plan, *dev, stream);
    }
    if (q.routing) {
        return launch_mx<false, true, kMxEpiRouting>(q, plan, *dev, stream);
    }
    if (q.group_count != 0) {
        return fp4 ? launch_mx<true, true>(q, plan, *dev, stream) : launch_mx<false, true>(q, plan, *dev, stream);
    }
    return fp4 ? launch_mx<true, false>(q, plan, *dev, stream) : launch_mx<false, false>(q, plan, *dev, stream);
}

}  // namespace

extern "C" {

int cb200_mx_matmul_can_implement(const cb200_mx_matmul_args* args)
{
    MxPlan plan;
    return args == nullptr ? CB200_INVALID : plan_mx(mx_dense_problem(args), &plan);
}

uint64_t cb200_mx_matmul_workspace_size(const cb200_mx_matmul_args* args)
{
    MxPlan plan;
    if (args == nullptr || plan_mx(mx_dense_problem(args), &plan) != CB200_SUCCESS) {
        return 0;
    }
    return plan.total();
}

int cb200_mx_matmul(const cb200_mx_matmul_args* args, void* stream)
{
    return args == nullptr ? CB200_INVALID : run_mx(mx_dense_problem(args), stream);
}

int cb200_mx_grouped_matmul_slice_m_can_implement(const cb200_mx_grouped_matmul_args* args)
{
    MxPlan plan;
    if (args == nullptr || args->group_count == 0 || args->group_list_kind > CB200_GROUP_LIST_PREFIX_SUMS) {
        return CB200_INVALID;
    }
    return plan_mx(mx_grouped_problem(args), &plan);
}

uint64_t cb200_mx_grouped_matmul_slice_m_workspace_size(const cb200_mx_grouped_matmul_args* args)
{
    MxPlan plan;
    if (cb200_mx_grouped_matmul_slice_m_can_implement(args) != CB200_SUCCESS ||
        plan_mx(mx_grouped_problem(args), &plan) != CB200_SUCCESS) {
        return 0;
    }
    return plan.total();
}

int cb200_mx_grouped_matmul_slice_m(const cb200_mx_grouped_matmul_args* args, void* stream)
{
    const int rc = cb200_mx_grouped_matmul_slice_m_can_implement(args);
    return rc != CB200_SUCCESS ? rc : run_mx(mx_grouped_problem(args), stream);
}

int cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_can_implement(const cb200_mx_grouped_swiglu_quant_args* args)
{
    MxPlan plan;
    if (args == nullptr || args->group_count == 0 || args->group_list_kind > CB200_GROUP_LIST_PREFIX_SUMS) {
        return CB200_INVALID;
    }
    return plan_mx(mx_swiglu_problem(args), &plan);
}

uint64_t cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_workspace_size(const cb200_mx_grouped_swiglu_quant_args* args)
{
    MxPlan plan;
    if (cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_can_implement(args) != CB200_SUCCESS ||
        plan_mx(mx_swiglu_problem(args), &plan) != CB200_SUCCESS) {
        return 0;
    }
    return plan.total();
}

int cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant(const cb200_mx_grouped_swiglu_quant_args* args, void* stream)
{
    const int rc = cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_can_implement(args);
    return rc != CB200_SUCCESS ? rc : run_mx(mx_swiglu_problem(args), stream);
}

int cb200_mx_grouped_matmul_finalize_routing_can_implement(const cb200_mx_grouped_finalize_routing_args* args)
{
    MxPlan plan;
    if (args == nullptr || args->group_count == 0 || args->group_list_kind > CB200_GROUP_LIST_PREFIX_SUMS ||
        (args->row_index_type != CB200_GROUP_LIST_INT64 && args->row_index_type != CB200_GROUP_LIST_INT32) ||
        (args->flags & ~CB200_ROUTING_DETERMINISTIC) != 0) {
        return CB200_INVALID;
    }
    if (args->flags & CB200_ROUTING_DETERMINISTIC) {
        RoutingDetPlan det;
        return plan_routing_det(args, &det);
    }
    return plan_mx(mx_routing_problem(args), &plan);
}

uint64_t cb200_mx_grouped_matmul_finalize_routing_workspace_size(const cb200_mx_grouped_finalize_routing_args* args)
{
    MxPlan plan;
    if (cb200_mx_grouped_matmul_finalize_routing_can_implement(args) != CB200_SUCCESS) {
        return 0;
    }
    if (args->flags & CB200_ROUTING_DETERMINISTIC) {
        RoutingDetPlan det;
        return plan_routing_det(args, &det) == CB200_SUCCESS ? det.total() : 0;
    }
    if (plan_mx(mx_routing_problem(args), &plan) != CB200_SUCCESS) {
        return 0;
    }
    return plan.total();
}

int cb200_mx_grouped_matmul_finalize_routing(const cb200_mx_grouped_finalize_routing_args* args, void* stream)
{
    const int rc = cb200_mx_grouped_matmul_finalize_routing_can_implement(args);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    if (args->flags & CB200_ROUTING_DETERMINISTIC) {
        return run_routing_det(args, stream);
    }
    return run_mx(mx_routing_problem(args), stream);
}

int cb200_w4a8_matmul_can_implement(const cb200_w4a8_matmul_args* args)
{
    W4Plan plan;
    return plan_w4a8(args, &plan);
}

uint64_t cb200_w4a8_matmul_workspace_size(const cb200_w4a8_matmul_args* args)
{
    // Fast path (weights packed along K, K a whole number of 128-element blocks, 16-byte aligned operands): the
    // weights are unpacked between two shared-memory buffers and nothing goes through global memory.  Otherwise
    // the ingestion pre-pass needs room for the K-padded copies of A and W.
    W4Plan plan;
    if (plan_w4a8(args, &plan) != CB200_SUCCESS || args->m == 0 || args->n == 0 || !plan.ingest) {
        return 0;
    }
    return plan.a_bytes + plan.w_bytes;
}

int cb200_w4a8_matmul(const cb200_w4a8_matmul_args* args_in, void* stream_v)
{
    W4Plan plan;
    int rc = plan_w4a8(args_in, &plan);
    if (rc != CB200_SUCCESS || args_in->m == 0 || args_in->n == 0) {
        return rc;
    }
    DeviceState* dev = nullptr;
    rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    cb200_w4a8_matmul_args local = *args_in;
    const cb200_w4a8_matmul_args* args = &local;
    if (plan.ingest) {
        if (args_in->workspace == nullptr || args_in->workspace_bytes < plan.a_bytes + plan.w_bytes ||
            (reinterpret_cast<uintptr_t>(args_in->workspace) & 255u) != 0) {
            return CB200_INVALID;
        }
        uint8_t* a_pad = static_cast<uint8_t*>(args_in->workspace);
        uint8_t* w_pad = a_pad + plan.a_bytes;
        const uint32_t blocks = static_cast<uint32_t>(dev->sm_count) * 8u;
        pad_rows_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(args_in->a), a_pad, args_in->m,
                                                    args_in->k, plan.k_padded, args_in->k, 0);
        if (args_in->pack_axis == CB200_W4_PACKED_ALONG_K) {
            pad_rows_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(args_in->w_packed), w_pad,
                                                        args_in->n, (args_in->k + 1u) / 2u, plan.k_padded / 2u,
                                                        (args_in->k + 1u) / 2u, args_in->k & 1u);
        } else {
            transpose_nibbles_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(args_in->w_packed), w_pad,
                                                                 args_in->n, args_in->k, (args_in->n + 1u) / 2u,
                                                                 plan.k_padded / 2u);
        }
        CB200_CUDA_TRY(cudaGetLastError());
        g_launches.fetch_add(2, std::memory_order_relaxed);
        local.a = a_pad;
        local.w_packed = w_pad;
        local.k = plan.k_padded;
        local.flags &= ~CB200_FLAG_STATIC_WEIGHTS;  // the kernel's weights now come from the pre-pass on this stream
    }
    local.group_size = plan.group_size;
    W4A8Params p;
    p.m = args->m;
    p.n = args->n;
    p.k = args->k;
    p.blocks_per_group = args->group_size / 128u;
    p.num_groups = args->k / args->group_size;
    const uint32_t tiles_n = (args->n + kW4Channels - 1) / kW4Channels;
    // Default: every CTA runs the whole K range (the sequential fp32 order of the definition: bit-exact).  Token
    // tiles of 64 rows instead of 128 double the CTAs when the result still fits one wave.
    p.splits = 1;
    p.tile_m = kW4Tokens;
    if (args->m > 64u && tiles_n * ((args->m + 63u) / 64u) <= static_cast<uint32_t>(dev->sm_count)) {
        p.tile_m = 64;
    }
    // Opt-in (flags bit 0): the K range split over the CTAs of a cluster, as many as still fit the SMs in one
    // wave; fp32 partial sums are then added at the end.
    const uint32_t want_splits = (args->flags & CB200_W4A8_SPLIT_K) ? static_cast<uint32_t>(kW4MaxSplits) : 1u;
    if (want_splits > 1) {
        const uint32_t tiles = tiles_n * ((args->m + kW4Tokens - 1) / kW4Tokens);
        while (p.splits < want_splits && tiles * p.splits * 2 <= static_cast<uint32_t>(dev->sm_count) &&
               p.splits * 2 <= p.num_groups) {
            p.splits *= 2;
        }
        if (p.splits > 1) {
            p.tile_m = kW4Tokens;
        }
    }
    {
        const uint32_t v = static_cast<uint32_t>(dev_knob("CB200_W4A8_TILE_M", 0));
        if ((v == 64 || v == 128) && p.splits == 1) {
            p.tile_m = v;
        }
    }
    p.mt = args->m >= p.tile_m ? p.tile_m : ((args->m + 15u) & ~15u);
    p.sw = args->weight_scale;
    p.sa = args->per_token_scale;
    p.d = static_cast<uint16_t*>(args->d);
    p.status = dev->status;
    p.out_f16 = args->d_type == CB200_DTYPE_F16 ? 1u : 0u;
    p.static_weights = (args->flags & CB200_FLAG_STATIC_WEIGHTS) ? 1u : 0u;
    {
        const long v = dev_knob("CB200_W4A8_TOKEN_LOADS", kW4MaxTokenLoads);
        p.token_loads_max = (v >= 1 && v <= kW4MaxTokenLoads) ? static_cast<uint32_t>(v) : kW4MaxTokenLoads;
    }
    CUtensorMap tmap_w, tmap_x;
    {
        // packed weights as (64 bytes of a K block, channel, K block): a box is kW4Load consecutive blocks
        const uint64_t dims[3] = {64, args->n, args->k / 128u};
        const uint64_t strides[2] = {args->k / 2u, 64};
        const uint32_t box[3] = {64, kW4Channels, kW4Load};
        rc = encode_tmap_u8(&tmap_w, args->w_packed, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    {
        // tokens as (128 bytes of a K block, token, K block); groups longer than one block load block by block
        const uint64_t dims[3] = {128, args->m, args->k / 128u};
        const uint64_t strides[2] = {args->k, 128};
        const uint32_t box[3] = {128, p.mt, args->group_size == 128 ? static_cast<uint32_t>(kW4Load) : 1u};
        rc = encode_tmap_u8(&tmap_x, args->a, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    static PerDeviceOnce once;
    int devid = 0;
    rc = current_device(&devid);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    rc = once.run(devid, [&]() -> int {
        CB200_CUDA_TRY(cudaFuncSetAttribute(w4a8_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            W4A8Smem<4>::kTotalBytes));
        CB200_CUDA_TRY(cudaFuncSetAttribute(w4a8_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            W4A8Smem<4>::kTotalBytes));
        CB200_CUDA_TRY(cudaFuncSetAttribute(w4a8_gemm_kernel<false, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            W4A8Smem<6>::kTotalBytes));
        return CB200_SUCCESS;
    });
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    const dim3 grid(tiles_n * p.splits, (args->m + p.tile_m - 1) / p.tile_m, 1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kW4Threads, 1, 1);
    // scale groups of several K blocks and token tiles of at most 64 rows: six tile slots (see W4A8Smem)
    const bool six_slots = args->group_size != 128 && p.mt <= 64 && dev_knob("CB200_W4A8_SIX_SLOTS", 1) != 0;
    cfg.dynamicSmemBytes = six_slots ? W4A8Smem<6>::kTotalBytes : W4A8Smem<4>::kTotalBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: set-up (and, for static weights, the first weight loads) may overlap the
    // tail of the kernel before this one on the stream; the kernel waits (griddepcontrol.wait) before it reads
    // anything else from global memory or writes D
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dev_knob("CB200_W4A8_PDL", 1) != 0 ? 2 : 1;
    if (args->group_size == 128) {
        CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4a8_gemm_kernel<true>, tmap_w, tmap_x, p));
    } else if (six_slots) {
        CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4a8_gemm_kernel<false, 6>, tmap_w, tmap_x, p));
    } else {
        CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, w4a8_gemm_kernel<false>, tmap_w, tmap_x, p));
    }
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

}  // extern "C"

namespace {

W8A8Problem dense_problem(const cb200_quant_matmul_args* args)
{
    W8A8Problem q{};
    q.m = args->m;
    q.n = args->n;
    q.k = args->k;
    q.group_count = 0;
    q.group_list_type = CB200_GROUP_LIST_INT64;
    q.layout_a = args->layout_a;
    q.layout_b = args->layout_b;
    q.a = args->a;
    q.b = args->b;
    q.group_list = nullptr;
    q.scale = args->scale;
    q.per_token = args->per_token_scale;
    q.d = args->d;
    q.acc = args->acc;
    q.block_num = args->block_num;
    q.scale_type = args->scale_type;
    q.d_type = args->d_type;
    q.scale_stride = 0;
    q.static_weights = (args->flags & CB200_FLAG_STATIC_WEIGHTS) != 0;
    return q;
}

W8A8Problem grouped_problem(const cb200_grouped_quant_matmul_args* args)
{
    W8A8Problem q{};
    q.m = args->m;
    q.n = args->n;
    q.k = args->k;
    q.group_count = args->group_count;
    q.group_list_type = args->group_list_type;
    q.layout_a = CB200_ROW_MAJOR;
    q.layout_b = args->layout_b;
    q.a = args->a;
    q.b = args->b;
    q.group_list = args->group_list;
    q.scale = args->scale;
    q.per_token = args->per_token_scale;
    q.d = args->d;
    q.acc = args->acc;
    q.block_num = args->block_num;
    q.scale_type = args->scale_type;
    q.d_type = args->d_type;
    q.scale_stride = args->n;
    return q;
}

// Per-tensor / per-channel dequant: the grouped kernel with one scale vector (or one scalar) for all groups and no
// per-token factor.  (x * 1.0f is exact, so the epilogue's second multiply changes nothing.)
W8A8Problem fixpipe_problem(const cb200_grouped_fixpipe_dequant_args* args)
{
    W8A8Problem q{};
    q.m = args->m;
    q.n = args->n;
    q.k = args->k;
    q.group_count = args->group_count;
    q.group_list_type = args->group_list_type;
    q.layout_a = CB200_ROW_MAJOR;
    q.layout_b = args->layout_b;
    q.a = args->a;
    q.b = args->b;
    q.group_list = args->group_list;
    q.scale = args->per_channel_scale;
    q.per_token = nullptr;
    q.has_per_token = false;
    q.d = args->d;
    q.acc = args->acc;
    q.block_num = args->block_num;
    q.scale_type = args->per_channel_scale_type;
    q.d_type = args->d_type;
    q.scale_stride = 0;
    q.scalar_mode = args->quant_mode == CB200_QUANT_PER_TENSOR;
    q.scalar_scale = args->scale_per_tensor;
    return q;
}

bool fixpipe_args_ok(const cb200_grouped_fixpipe_dequant_args* args)
{
    return args != nullptr && args->group_count != 0 &&
           (args->quant_mode == CB200_QUANT_PER_TENSOR || args->quant_mode == CB200_QUANT_PER_CHANNEL) &&
           (args->per_channel_scale_type == CB200_DTYPE_F32 || args->per_channel_scale_type == CB200_DTYPE_F32_IN_U64);
}

}  // namespace

extern "C" {

int cb200_quant_matmul_can_implement(const cb200_quant_matmul_args* args)
{
    if (args == nullptr) {
        return CB200_INVALID;
    }
    return check_w8a8(dense_problem(args));
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
    return run_w8a8(dense_problem(args), stream);
}

int cb200_grouped_quant_matmul_slice_m_can_implement(const cb200_grouped_quant_matmul_args* args)
{
    if (args == nullptr || args->group_count == 0) {
        return CB200_INVALID;
    }
    return check_w8a8(grouped_problem(args));
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
    return run_w8a8(grouped_problem(args), stream);
}

}  // extern "C"

namespace {

struct SliceKPlan {
    uint32_t rows_max;  // padded K rows at most
    uint64_t table_bytes, blocks_bytes, a_bytes, b_bytes;
    uint64_t total() const { return table_bytes + blocks_bytes + a_bytes + b_bytes; }
};

int plan_slice_k(const cb200_grouped_quant_matmul_slice_k_args* a, SliceKPlan* plan)
{
    if (a == nullptr || a->group_count == 0 || a->group_count > static_cast<uint32_t>(kMaxGroups)) {
        return CB200_INVALID;
    }
    *plan = SliceKPlan{};
    if (a->m == 0 || a->n == 0) {
        return CB200_SUCCESS;
    }
    if (a->a == nullptr || a->b == nullptr || a->group_list == nullptr || a->scale == nullptr ||
        a->per_token_scale == nullptr || a->d == nullptr) {
        return CB200_INVALID;
    }
    if ((a->group_list_type != CB200_GROUP_LIST_INT64 && a->group_list_type != CB200_GROUP_LIST_INT32) ||
        a->scale_type > CB200_DTYPE_F16 || (a->d_type != 0 && a->d_type != CB200_DTYPE_BF16 && a->d_type != CB200_DTYPE_F16)) {
        return CB200_INVALID;
    }
    if ((a->m & 15u) != 0 || (a->n & 15u) != 0 || !aligned16(a->a) || !aligned16(a->b) || !aligned16(a->d)) {
        return CB200_INVALID;
    }
    const uintptr_t scale_mask = scale_elem_bytes(a->scale_type) - 1u;
    if ((reinterpret_cast<uintptr_t>(a->scale) & scale_mask) != 0 ||
        (reinterpret_cast<uintptr_t>(a->per_token_scale) & scale_mask) != 0) {
        return CB200_INVALID;
    }
    const uint64_t out_rows = static_cast<uint64_t>(a->group_count) * a->m;
    if (a->m > 0x7fffff00u || a->n > 0x7fffff00u || a->k > 0x7fffff00u || out_rows > 0x7fffff00u) {
        return CB200_INVALID;
    }
    plan->rows_max = ((a->k + 127u) / 128u + a->group_count) * 128u;
    plan->table_bytes = align256(static_cast<uint64_t>(a->group_count) * 16u + 16u);
    plan->blocks_bytes = align256(static_cast<uint64_t>(a->group_count) * 8u);
    plan->a_bytes = align256(static_cast<uint64_t>(plan->rows_max) * a->m);
    plan->b_bytes = align256(static_cast<uint64_t>(plan->rows_max) * a->n);
    return CB200_SUCCESS;
}

}  // namespace

extern "C" {

int cb200_grouped_quant_matmul_slice_k_can_implement(const cb200_grouped_quant_matmul_slice_k_args* args)
{
    SliceKPlan plan;
    return plan_slice_k(args, &plan);
}

uint64_t cb200_grouped_quant_matmul_slice_k_workspace_size(const cb200_grouped_quant_matmul_slice_k_args* args)
{
    SliceKPlan plan;
    if (plan_slice_k(args, &plan) != CB200_SUCCESS) {
        return 0;
    }
    return plan.total();
}

int cb200_grouped_quant_matmul_slice_k(const cb200_grouped_quant_matmul_slice_k_args* args, void* stream_v)
{
    SliceKPlan plan;
    int rc = plan_slice_k(args, &plan);
    if (rc != CB200_SUCCESS || args->m == 0 || args->n == 0) {
        return rc;
    }
    if (args->workspace == nullptr || args->workspace_bytes < plan.total() ||
        (reinterpret_cast<uintptr_t>(args->workspace) & 255u) != 0) {
        return CB200_INVALID;
    }
    DeviceState* dev = nullptr;
    rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    uint8_t* ws = static_cast<uint8_t*>(args->workspace);
    int4* table = reinterpret_cast<int4*>(ws);
    uint32_t* total_blocks = reinterpret_cast<uint32_t*>(ws + static_cast<uint64_t>(args->group_count) * 16u);
    int2* blocks = reinterpret_cast<int2*>(ws + plan.table_bytes);
    uint8_t* a_pad = ws + plan.table_bytes + plan.blocks_bytes;
    uint8_t* b_pad = a_pad + plan.a_bytes;
    // 1) where every group's padded K range lies; 2) A and B copied there, padding rows zeroed
    slice_k_plan_kernel<<<1, 32, 0, stream>>>(args->group_list, args->group_list_type == CB200_GROUP_LIST_INT32 ? 1u : 0u,
                                              args->group_count, args->k, table, blocks, total_blocks);
    const uint32_t copy_blocks = static_cast<uint32_t>(dev->sm_count) * 4u;
    slice_k_scatter_kernel<<<copy_blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(args->a), a_pad, args->m, table,
                                                            args->group_count, total_blocks);
    slice_k_scatter_kernel<<<copy_blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(args->b), b_pad, args->n, table,
                                                            args->group_count, total_blocks);
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(3, std::memory_order_relaxed);

    // 3) the pair kernel over (group, row tile, column tile), each tile running its group's K blocks
    using S = W8A8PairSmem;
    CUtensorMap tmap_a, tmap_b, tmap_d;
    {
        const uint64_t dims[2] = {args->m, plan.rows_max};
        const uint64_t strides[1] = {args->m};
        const uint32_t box[2] = {128, 128};
        rc = encode_tmap_u8(&tmap_a, a_pad, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    {
        const uint64_t dims[3] = {args->n, plan.rows_max, 1};
        const uint64_t strides[2] = {args->n, static_cast<uint64_t>(args->n) * plan.rows_max};
        const uint32_t box[3] = {128, 128, 1};
        rc = encode_tmap_u8(&tmap_b, b_pad, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
    }
    W8A8Problem q{};
    q.m = args->m;
    q.n = args->n;
    q.k = args->k;
    q.group_count = args->group_count;
    q.group_list_type = CB200_GROUP_LIST_INT64;
    q.group_list = blocks;
    q.scale = args->scale;
    q.per_token = args->per_token_scale;
    q.d = args->d;
    q.acc = args->acc;
    q.scale_type = args->scale_type;
    q.d_type = args->d_type;
    q.scale_stride = args->n;
    W8A8Params p;
    fill_params(p, q, *dev);
    memset(&tmap_d, 0, sizeof(tmap_d));
    if ((args->n & 7u) == 0) {
        const uint64_t dims[2] = {static_cast<uint64_t>(args->n) * 2u, static_cast<uint64_t>(args->group_count) * args->m};
        const uint64_t strides[1] = {static_cast<uint64_t>(args->n) * 2u};
        const uint32_t box[2] = {64, 32};
        rc = encode_tmap_u8(&tmap_d, args->d, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        p.tma_store = 1;
    }
    auto kernel = w8a8_pair_kernel<BLayout::kRowMajor, true, true>;
    static PerDeviceOnce once;
    int devid = 0;
    rc = current_device(&devid);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    rc = once.run(devid, [&]() -> int {
        CB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotalBytes));
        return CB200_SUCCESS;
    });
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    const uint64_t tiles = static_cast<uint64_t>(args->group_count) * ((args->m + kPairTileM - 1) / kPairTileM) *
                           ((args->n + kPairBN - 1) / kPairBN);
    uint32_t pairs = static_cast<uint32_t>(dev->sm_count) / 2u;
    if (args->block_num != 0 && args->block_num / 2u < pairs) {
        pairs = args->block_num / 2u == 0 ? 1u : args->block_num / 2u;
    }
    if (tiles < pairs) {
        pairs = static_cast<uint32_t>(tiles);
    }
    kernel<<<2 * pairs, kGemmThreads, S::kTotalBytes, stream>>>(tmap_a, tmap_b, tmap_d, p);
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

int cb200_grouped_matmul_slice_m_fixpipe_dequant_can_implement(const cb200_grouped_fixpipe_dequant_args* args)
{
    if (!fixpipe_args_ok(args)) {
        return CB200_INVALID;
    }
    return check_w8a8(fixpipe_problem(args));
}

uint64_t cb200_grouped_matmul_slice_m_fixpipe_dequant_workspace_size(const cb200_grouped_fixpipe_dequant_args* args)
{
    (void)args;
    return 0;
}

int cb200_grouped_matmul_slice_m_fixpipe_dequant(const cb200_grouped_fixpipe_dequant_args* args, void* stream)
{
    if (!fixpipe_args_ok(args)) {
        return CB200_INVALID;
    }
    return run_w8a8(fixpipe_problem(args), stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Host-buffer grouped matmul: chunked copy-in / compute / copy-out overlap (see the header).
namespace {

constexpr uint32_t kHostDefaultChunks = 16;  // measured on the MoE workload: 4: 25.2 ms, 8: 23.2, 16: 22.3, 32: 22.9
constexpr uint32_t kHostMaxChunks = 64;

struct HostPipe {
    std::mutex mu;  // held for the whole of a host-buffer call: the streams, events and lists_host are shared
    bool ready = false;
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t start = nullptr, lists_copied = nullptr, all_out = nullptr;
    cudaEvent_t chunk_in[kHostMaxChunks] = {}, chunk_done[kHostMaxChunks] = {};
    int64_t* lists_host = nullptr;  // pinned: [chunks][group_count] chunk-local prefix sums
    size_t lists_capacity = 0;
};

struct HostLayout {
    uint64_t a, pt, d, lists, total;
};

HostLayout host_layout(const cb200_grouped_quant_matmul_host_args* a, uint32_t chunks)
{
    HostLayout l;
    l.a = 0;
    l.pt = align256(static_cast<uint64_t>(a->m) * a->k);
    l.d = l.pt + align256(static_cast<uint64_t>(a->m) * 4u);
    l.lists = l.d + align256(static_cast<uint64_t>(a->m) * a->n * 2u);
    l.total = l.lists + align256(static_cast<uint64_t>(chunks) * a->group_count * 8u);
    return l;
}

uint32_t host_chunks(const cb200_grouped_quant_matmul_host_args* a)
{
    uint32_t c = a->chunks == 0 ? kHostDefaultChunks : a->chunks;
    c = c > kHostMaxChunks ? kHostMaxChunks : c;
    const uint32_t tiles = (a->m + 127u) / 128u;
    return c > tiles ? (tiles == 0 ? 1u : tiles) : c;
}

// The pipe of the current device, created on first use.
int host_pipe(HostPipe** out)
{
    static HostPipe pipes[kMaxDevices];
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    HostPipe& hp = pipes[dev];
    std::lock_guard<std::mutex> lock(hp.mu);
    if (!hp.ready) {
        CB200_CUDA_TRY(cudaStreamCreateWithFlags(&hp.in, cudaStreamNonBlocking));
        CB200_CUDA_TRY(cudaStreamCreateWithFlags(&hp.out, cudaStreamNonBlocking));
        CB200_CUDA_TRY(cudaEventCreateWithFlags(&hp.start, cudaEventDisableTiming));
        CB200_CUDA_TRY(cudaEventCreateWithFlags(&hp.lists_copied, cudaEventDisableTiming));
        CB200_CUDA_TRY(cudaEventCreateWithFlags(&hp.all_out, cudaEventDisableTiming));
        for (uint32_t c = 0; c < kHostMaxChunks; ++c) {
            CB200_CUDA_TRY(cudaEventCreateWithFlags(&hp.chunk_in[c], cudaEventDisableTiming));
            CB200_CUDA_TRY(cudaEventCreateWithFlags(&hp.chunk_done[c], cudaEventDisableTiming));
        }
        hp.ready = true;
    }
    *out = &hp;
    return CB200_SUCCESS;
}

// Grows the pinned staging buffer of the group lists; the caller holds the pipe's mutex.
int host_pipe_lists(HostPipe* hp, size_t lists_needed)
{
    if (hp->lists_capacity < lists_needed) {
        if (hp->lists_host != nullptr) {
            CB200_CUDA_TRY(cudaEventSynchronize(hp->lists_copied));
            CB200_CUDA_TRY(cudaFreeHost(hp->lists_host));
            hp->lists_host = nullptr;
            hp->lists_capacity = 0;
        }
        CB200_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&hp->lists_host), lists_needed, cudaHostAllocDefault));
        hp->lists_capacity = lists_needed;
    }
    return CB200_SUCCESS;
}

}  // namespace

extern "C" {

uint64_t cb200_grouped_quant_matmul_slice_m_host_workspace_size(const cb200_grouped_quant_matmul_host_args* args)
{
    if (args == nullptr || args->group_count == 0) {
        return 0;
    }
    return host_layout(args, host_chunks(args)).total;
}

int cb200_grouped_quant_matmul_slice_m_host(const cb200_grouped_quant_matmul_host_args* args, void* stream_v)
{
    if (args == nullptr || args->group_count == 0 || args->group_count > static_cast<uint32_t>(kMaxGroups) ||
        args->a_host == nullptr || args->group_list_host == nullptr || args->per_token_host == nullptr ||
        args->d_host == nullptr || args->workspace == nullptr ||
        (reinterpret_cast<uintptr_t>(args->workspace) & 255u) != 0) {
        return CB200_INVALID;
    }
    if (args->m == 0 || args->n == 0) {
        return CB200_SUCCESS;
    }
    const uint32_t chunks = host_chunks(args);
    const HostLayout lay = host_layout(args, chunks);
    if (args->workspace_bytes < lay.total) {
        return CB200_INVALID;
    }
    uint8_t* ws = static_cast<uint8_t*>(args->workspace);
    int8_t* a_dev = reinterpret_cast<int8_t*>(ws + lay.a);
    float* pt_dev = reinterpret_cast<float*>(ws + lay.pt);
    uint16_t* d_dev = reinterpret_cast<uint16_t*>(ws + lay.d);
    int64_t* lists_dev = reinterpret_cast<int64_t*>(ws + lay.lists);
    const uint32_t G = args->group_count;
    // the chunk launches differ only in their row range
    auto chunk_problem = [&](uint32_t rows, int64_t r0, uint32_t c) {
        W8A8Problem q{};
        q.m = rows;
        q.n = args->n;
        q.k = args->k;
        q.group_count = G;
        q.group_list_type = CB200_GROUP_LIST_INT64;
        q.layout_a = CB200_ROW_MAJOR;
        q.layout_b = args->layout_b;
        q.a = a_dev + r0 * args->k;
        q.b = args->b;
        q.group_list = lists_dev + static_cast<size_t>(c) * G;
        q.scale = args->scale;
        q.per_token = pt_dev + r0;
        q.d = d_dev + r0 * args->n;
        q.acc = nullptr;
        q.block_num = 0;
        q.scale_stride = args->n;
        return q;
    };
    // validate once with the whole problem (alignment, layouts, sizes)
    int rc = check_w8a8(chunk_problem(args->m, 0, 0));
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    HostPipe* hp = nullptr;
    rc = host_pipe(&hp);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    std::lock_guard<std::mutex> pipe_lock(hp->mu);
    rc = host_pipe_lists(hp, static_cast<size_t>(chunks) * G * 8u);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    // rows that take part: [0, last list entry); chunk boundaries on multiples of 128 rows
    int64_t rows = args->group_list_host[G - 1];
    rows = rows < 0 ? 0 : (rows > static_cast<int64_t>(args->m) ? static_cast<int64_t>(args->m) : rows);
    const int64_t per = ((rows + chunks - 1) / chunks + 127) / 128 * 128;

    // chunk-local group lists: entry g of chunk c = rows of groups 0..g that fall inside the chunk
    CB200_CUDA_TRY(cudaEventSynchronize(hp->lists_copied));  // the previous call's copy has left the buffer
    for (uint32_t c = 0; c < chunks; ++c) {
        const int64_t r0 = static_cast<int64_t>(c) * per < rows ? static_cast<int64_t>(c) * per : rows;
        const int64_t r1 = r0 + per < rows ? r0 + per : rows;
        for (uint32_t g = 0; g < G; ++g) {
            int64_t e = args->group_list_host[g];
            e = e < r0 ? r0 : (e > r1 ? r1 : e);
            hp->lists_host[static_cast<size_t>(c) * G + g] = e - r0;
        }
    }
    // order the copy-in stream behind whatever the caller has enqueued so far
    CB200_CUDA_TRY(cudaEventRecord(hp->start, stream));
    CB200_CUDA_TRY(cudaStreamWaitEvent(hp->in, hp->start, 0));
    CB200_CUDA_TRY(cudaStreamWaitEvent(hp->out, hp->start, 0));
    CB200_CUDA_TRY(cudaMemcpyAsync(lists_dev, hp->lists_host, static_cast<size_t>(chunks) * G * 8u,
                                   cudaMemcpyHostToDevice, hp->in));
    CB200_CUDA_TRY(cudaEventRecord(hp->lists_copied, hp->in));

    for (uint32_t c = 0; c < chunks; ++c) {
        const int64_t r0 = static_cast<int64_t>(c) * per < rows ? static_cast<int64_t>(c) * per : rows;
        const int64_t r1 = r0 + per < rows ? r0 + per : rows;
        const int64_t cr = r1 - r0;
        if (cr <= 0) {
            continue;
        }
        CB200_CUDA_TRY(cudaMemcpyAsync(a_dev + r0 * args->k, static_cast<const int8_t*>(args->a_host) + r0 * args->k,
                                       static_cast<size_t>(cr) * args->k, cudaMemcpyHostToDevice, hp->in));
        CB200_CUDA_TRY(cudaMemcpyAsync(pt_dev + r0, args->per_token_host + r0, static_cast<size_t>(cr) * 4u,
                                       cudaMemcpyHostToDevice, hp->in));
        CB200_CUDA_TRY(cudaEventRecord(hp->chunk_in[c], hp->in));
        CB200_CUDA_TRY(cudaStreamWaitEvent(stream, hp->chunk_in[c], 0));
        rc = run_w8a8(chunk_problem(static_cast<uint32_t>(cr), r0, c), stream);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        CB200_CUDA_TRY(cudaEventRecord(hp->chunk_done[c], stream));
        CB200_CUDA_TRY(cudaStreamWaitEvent(hp->out, hp->chunk_done[c], 0));
        CB200_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(args->d_host) + static_cast<size_t>(r0) * args->n * 2u,
                                       d_dev + r0 * args->n, static_cast<size_t>(cr) * args->n * 2u,
                                       cudaMemcpyDeviceToHost, hp->out));
    }
    // the caller's stream completes only after the last copy-out
    CB200_CUDA_TRY(cudaEventRecord(hp->all_out, hp->out));
    CB200_CUDA_TRY(cudaStreamWaitEvent(stream, hp->all_out, 0));
    return CB200_SUCCESS;
}

}  // extern "C"

extern "C" {

int cb200_quantize_per_token_int8_can_implement(const cb200_quantize_int8_args* args)
{
    if (args == nullptr || args->reserved != 0) {
        return CB200_INVALID;
    }
    if (args->rows == 0 || args->k == 0) {
        return CB200_SUCCESS;
    }
    if (args->x == nullptr || args->q == nullptr || args->scale == nullptr ||
        (args->x_type != CB200_DTYPE_F32 && args->x_type != CB200_DTYPE_BF16) || args->k % 16u != 0) {
        return CB200_INVALID;
    }
    const uint64_t pitch = args->x_pitch != 0 ? args->x_pitch : args->k;
    const uint64_t elem = args->x_type == CB200_DTYPE_F32 ? 4u : 2u;
    if (pitch < args->k || (pitch * elem) % 16u != 0 || (reinterpret_cast<uintptr_t>(args->x) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(args->q) & 15u) != 0 || (reinterpret_cast<uintptr_t>(args->scale) & 3u) != 0) {
        return CB200_INVALID;
    }
    return CB200_SUCCESS;
}

int cb200_quantize_per_token_int8(const cb200_quantize_int8_args* args, void* stream_v)
{
    int rc = cb200_quantize_per_token_int8_can_implement(args);
    if (rc != CB200_SUCCESS || args->rows == 0 || args->k == 0) {
        return rc;
    }
    DeviceState* dev = nullptr;
    rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const uint64_t pitch = args->x_pitch != 0 ? args->x_pitch : args->k;
    // one warp per row, eight warps per CTA, eight CTAs per SM at most
    const uint32_t want = (args->rows + 7u) / 8u;
    const uint32_t cap = static_cast<uint32_t>(dev->sm_count) * 8u;
    const uint32_t blocks = want < cap ? want : cap;
    int8_t* q = static_cast<int8_t*>(args->q);
    float* scale = static_cast<float*>(args->scale);
    const bool bf16 = args->x_type == CB200_DTYPE_BF16;
    const uint64_t row_bytes = static_cast<uint64_t>(args->k) * (bf16 ? 2u : 4u);
    if (row_bytes <= kQuantInt8StageBytes) {
        // rows staged through shared memory, one CTA of eight warps per SM
        constexpr uint32_t kSmem = 8u * kQuantInt8StageBytes + 2u * 8u * 8u + 16u;
        static PerDeviceOnce once;
        int devid = 0;
        rc = current_device(&devid);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        rc = once.run(devid, [&]() -> int {
            CB200_CUDA_TRY(cudaFuncSetAttribute(quant_int8_staged_kernel<true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            CB200_CUDA_TRY(cudaFuncSetAttribute(quant_int8_staged_kernel<false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            return CB200_SUCCESS;
        });
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        const uint32_t sms = static_cast<uint32_t>(dev->sm_count);
        const uint32_t grid = want < sms ? want : sms;
        if (bf16) {
            quant_int8_staged_kernel<true><<<grid, kQuantInt8Threads, kSmem, stream>>>(args->x, q, scale, args->rows,
                                                                                        args->k, pitch, dev->status);
        } else {
            quant_int8_staged_kernel<false><<<grid, kQuantInt8Threads, kSmem, stream>>>(args->x, q, scale, args->rows,
                                                                                         args->k, pitch, dev->status);
        }
    } else if (row_bytes <= 4ull * kQuantInt8StageBytes) {
        // one CTA per row, eight segments of at most half a slot
        constexpr uint32_t kSmem = 8u * kQuantInt8StageBytes + 2u * 8u * 8u + 16u;
        static PerDeviceOnce once_wide;
        int devid = 0;
        rc = current_device(&devid);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        rc = once_wide.run(devid, [&]() -> int {
            CB200_CUDA_TRY(cudaFuncSetAttribute(quant_int8_wide_kernel<true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            CB200_CUDA_TRY(cudaFuncSetAttribute(quant_int8_wide_kernel<false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            return CB200_SUCCESS;
        });
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        const uint32_t seg = ((args->k + 7u) / 8u + 15u) & ~15u;
        const uint32_t sms = static_cast<uint32_t>(dev->sm_count);
        const uint32_t grid = args->rows < sms ? args->rows : sms;
        if (bf16) {
            quant_int8_wide_kernel<true><<<grid, kQuantInt8Threads, kSmem, stream>>>(args->x, q, scale, args->rows,
                                                                                      args->k, pitch, seg, dev->status);
        } else {
            quant_int8_wide_kernel<false><<<grid, kQuantInt8Threads, kSmem, stream>>>(args->x, q, scale, args->rows,
                                                                                       args->k, pitch, seg, dev->status);
        }
    } else if (bf16) {
        quant_int8_kernel<true><<<blocks, kQuantInt8Threads, 0, stream>>>(args->x, q, scale, args->rows, args->k, pitch);
    } else {
        quant_int8_kernel<false><<<blocks, kQuantInt8Threads, 0, stream>>>(args->x, q, scale, args->rows, args->k, pitch);
    }
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Fixed-scratch variant of the MX matmul for callers that may not allocate device memory (a server that owns
// all of HBM through its own arena, a loop that cannot take cudaMalloc's device-wide synchronisation).
// The scratch is part of the library image: every GPU that loads the library holds these bytes until exit.
namespace {

constexpr uint64_t kMxStaticScratchBytes = 8ull << 20;
static __device__ __align__(256) uint8_t g_mx_static_scratch[kMxStaticScratchBytes];

// In host code the name g_mx_static_scratch is only a handle for the runtime, not a device address: the
// address a kernel may use is looked up once per device, with that device current.
int mx_static_scratch(uint8_t** out)
{
    static uint8_t* ptrs[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    CB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        return CB200_INVALID;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        uint8_t* p = nullptr;
        CB200_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_mx_static_scratch));
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return CB200_SUCCESS;
}

}  // namespace

extern "C" {

uint64_t cb200_mx_matmul_static_scratch_bytes(void)
{
    return kMxStaticScratchBytes;
}

// Same kernels and same results as cb200_mx_matmul; the re-tiled scales go to the library's own array.
// Allocates nothing.  The first call on a device performs the address look-up above.
int cb200_mx_matmul_static(const cb200_mx_matmul_args* args, void* stream_v)
{
    if (args == nullptr) {
        return CB200_INVALID;
    }
    MxProblem q = mx_dense_problem(args);
    MxPlan plan;
    int rc = plan_mx(q, &plan);
    if (rc != CB200_SUCCESS || args->m == 0 || args->n == 0) {
        return rc;
    }
    if (plan.total() > kMxStaticScratchBytes) {
        return CB200_SCRATCH_TOO_SMALL;
    }
    uint8_t* scratch = nullptr;
    rc = mx_static_scratch(&scratch);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    q.workspace = scratch;
    q.workspace_bytes = kMxStaticScratchBytes;
    return run_mx(q, stream_v);
}

}  // extern "C"

extern "C" {

int cb200_mx_quantize_can_implement(const cb200_mx_quantize_args* args)
{
    if (args == nullptr) {
        return CB200_INVALID;
    }
    if (args->rows == 0 || args->k == 0) {
        return CB200_SUCCESS;
    }
    if (args->x == nullptr || args->q == nullptr || args->scale == nullptr) {
        return CB200_INVALID;
    }
    if ((args->format != CB200_MX_E4M3 && args->format != CB200_MX_E2M1) ||
        (args->x_type != CB200_DTYPE_F32 && args->x_type != CB200_DTYPE_BF16)) {
        return CB200_INVALID;
    }
    if (args->x_pitch != 0 && args->x_pitch < args->k) {
        return CB200_INVALID;
    }
    const uintptr_t x_mask = args->x_type == CB200_DTYPE_F32 ? 3u : 1u;
    if ((reinterpret_cast<uintptr_t>(args->x) & x_mask) != 0) {
        return CB200_INVALID;
    }
    return CB200_SUCCESS;
}

int cb200_mx_quantize(const cb200_mx_quantize_args* args, void* stream_v)
{
    int rc = cb200_mx_quantize_can_implement(args);
    if (rc != CB200_SUCCESS || args->rows == 0 || args->k == 0) {
        return rc;
    }
    DeviceState* dev = nullptr;
    rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const bool fp4 = args->format == CB200_MX_E2M1;
    const bool bf16 = args->x_type == CB200_DTYPE_BF16;
    const uint64_t x_pitch = args->x_pitch != 0 ? args->x_pitch : args->k;
    const uint32_t q_pitch = fp4 ? (args->k + 1u) / 2u : args->k;
    const uint32_t sf_pitch = (((args->k + 31u) / 32u) + 1u) & ~1u;
    // vector accesses need aligned bases; the kernel falls back to element accesses on odd pitches by itself
    const bool x_vec = (reinterpret_cast<uintptr_t>(args->x) & 15u) == 0;
    const bool q_vec = (reinterpret_cast<uintptr_t>(args->q) & 3u) == 0;
    if (!x_vec || !q_vec) {
        return CB200_INVALID;  // torch / cudaMalloc buffers are 256-byte aligned; unaligned views are not taken
    }
    const uint32_t blocks = static_cast<uint32_t>(dev->sm_count) * 8u;
    uint8_t* q = static_cast<uint8_t*>(args->q);
    uint8_t* sf = static_cast<uint8_t*>(args->scale);
    const uint64_t row_bytes = static_cast<uint64_t>(args->k) * (bf16 ? 2u : 4u);
    const uint64_t segs_if_cut = (args->k + kMxQuantStageBytes / 2u / (bf16 ? 2u : 4u) - 1u) /
                                 (kMxQuantStageBytes / 2u / (bf16 ? 2u : 4u));
    if (args->k % 32u == 0 && (x_pitch * (bf16 ? 2u : 4u)) % 16u == 0 &&
        (reinterpret_cast<uintptr_t>(args->q) & 15u) == 0 &&
        static_cast<uint64_t>(args->rows) * segs_if_cut < (1ull << 31)) {
        // whole rows when they fit a warp's slot, else segments of half a slot (a multiple of 512 elements)
        const uint32_t seg = row_bytes <= kMxQuantStageBytes ? args->k : kMxQuantStageBytes / 2u / (bf16 ? 2u : 4u);
        static_assert((kMxQuantStageBytes / 2u / 2u) % 512u == 0 && (kMxQuantStageBytes / 2u / 4u) % 512u == 0,
                      "segment length");
        // the aligned case: rows staged through shared memory, one CTA of eight warps per SM
        constexpr uint32_t kSmem = 8u * kMxQuantStageBytes + 2u * 8u * 8u + 16u;
        static PerDeviceOnce once;
        int devid = 0;
        rc = current_device(&devid);
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        rc = once.run(devid, [&]() -> int {
            CB200_CUDA_TRY(cudaFuncSetAttribute(mx_quantize_staged_kernel<false, false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            CB200_CUDA_TRY(cudaFuncSetAttribute(mx_quantize_staged_kernel<false, true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            CB200_CUDA_TRY(cudaFuncSetAttribute(mx_quantize_staged_kernel<true, false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            CB200_CUDA_TRY(cudaFuncSetAttribute(mx_quantize_staged_kernel<true, true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
            return CB200_SUCCESS;
        });
        if (rc != CB200_SUCCESS) {
            return rc;
        }
        const uint64_t items = static_cast<uint64_t>(args->rows) * ((args->k + seg - 1u) / seg);
        const uint64_t want = (items + 7u) / 8u;
        const uint32_t sms = static_cast<uint32_t>(dev->sm_count);
        const uint32_t grid = want < sms ? static_cast<uint32_t>(want) : sms;
        if (fp4) {
            if (bf16) {
                mx_quantize_staged_kernel<true, true><<<grid, kMxQuantThreads, kSmem, stream>>>(
                    args->x, q, sf, args->rows, args->k, x_pitch, seg, dev->status);
            } else {
                mx_quantize_staged_kernel<true, false><<<grid, kMxQuantThreads, kSmem, stream>>>(
                    args->x, q, sf, args->rows, args->k, x_pitch, seg, dev->status);
            }
        } else if (bf16) {
            mx_quantize_staged_kernel<false, true><<<grid, kMxQuantThreads, kSmem, stream>>>(
                args->x, q, sf, args->rows, args->k, x_pitch, seg, dev->status);
        } else {
            mx_quantize_staged_kernel<false, false><<<grid, kMxQuantThreads, kSmem, stream>>>(
                args->x, q, sf, args->rows, args->k, x_pitch, seg, dev->status);
        }
    } else if (fp4) {
        if (bf16) {
            mx_quantize_kernel<true, true><<<blocks, 256, 0, stream>>>(args->x, q, sf, args->rows, args->k, x_pitch, q_pitch, sf_pitch);
        } else {
            mx_quantize_kernel<true, false><<<blocks, 256, 0, stream>>>(args->x, q, sf, args->rows, args->k, x_pitch, q_pitch, sf_pitch);
        }
    } else if (bf16) {
        mx_quantize_kernel<false, true><<<blocks, 256, 0, stream>>>(args->x, q, sf, args->rows, args->k, x_pitch, q_pitch, sf_pitch);
    } else {
        mx_quantize_kernel<false, false><<<blocks, 256, 0, stream>>>(args->x, q, sf, args->rows, args->k, x_pitch, q_pitch, sf_pitch);
    }
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
}

}  // extern "C"

#ifdef CB200_DEVELOPER_KNOBS
// Developer builds only: reads and clears the W4A8 kernel's per-role cycle counters.
extern "C" CB200_API int cb200_dev_w4a8_probe(unsigned long long* out)
{
    CB200_CUDA_TRY(cudaDeviceSynchronize());
    CB200_CUDA_TRY(cudaMemcpyFromSymbol(out, cb200::g_w4a8_probe, 64 * sizeof(unsigned long long)));
    unsigned long long zero[64] = {};
    CB200_CUDA_TRY(cudaMemcpyToSymbol(cb200::g_w4a8_probe, zero, sizeof(zero)));
    return CB200_SUCCESS;
}
#endif

namespace {
// One thread waits on an mbarrier that nobody will ever arrive on, with a short limit: exercises exactly the
// give-up path of the production kernels (status word, abort flag, orderly exit) without hanging anything.
__global__ void wait_selftest_kernel(unsigned* status, unsigned long long limit_ns)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_wait(smem_u32(&bar), 0, &abort_flag, status, kDevTimeoutSelfTest, limit_ns);
    }
    __syncthreads();
}
}  // namespace

extern "C" {

int cb200_selftest_wait_timeout(uint32_t limit_us, void* stream_v)
{
    DeviceState* dev = nullptr;
    int rc = device_state(&dev);
    if (rc != CB200_SUCCESS) {
        return rc;
    }
    if (limit_us == 0 || limit_us > 1000000u) {
        return CB200_INVALID;
    }
    wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_v)>>>(dev->status, limit_us * 1000ull);
    CB200_CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return CB200_SUCCESS;
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
