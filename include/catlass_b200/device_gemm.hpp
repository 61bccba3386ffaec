// Host-side operator adapter over the C ABI, with the reference's calling sequence
// (include/catlass/gemm/device/device_gemm.hpp:21-98):
//     Kernel::Arguments args{...};
//     DeviceGemm<Kernel> op;
//     op.CanImplement(args); size_t ws = op.GetWorkspaceSize(args); op.Initialize(args, workspace);
//     op(stream, blockNum);
// The kernel classes below carry the reference's Arguments members for the quantized-matmul path.
#pragma once

#include <cstddef>
#include <cstdint>

#include "../catlass_b200.h"
#include "gemm_coord.hpp"
#include "layout.hpp"
#include "status.hpp"

namespace Catlass::Gemm {

namespace detail {
template <class Layout>
struct LayoutTag;
template <>
struct LayoutTag<layout::RowMajor> {
    static constexpr uint32_t value = CB200_ROW_MAJOR;
};
template <>
struct LayoutTag<layout::ColumnMajor> {
    static constexpr uint32_t value = CB200_COLUMN_MAJOR;
};
template <>
struct LayoutTag<layout::zN> {
    static constexpr uint32_t value = CB200_ZN;  // weights (B) only
};
inline Status ToStatus(int rc)
{
    return rc == CB200_SUCCESS ? Status::kSuccess : Status::kInvalid;
}
}  // namespace detail

namespace Kernel {

/// Dense W8A8 with per-token / per-channel dequant. Arguments as
/// Gemm::Kernel::QuantMatmulMultiStageWorkspace::Arguments (quant_matmul_multistage_workspace.hpp:92-100).
template <class LayoutA = layout::RowMajor, class LayoutB = layout::ColumnMajor>
struct QuantMatmul {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t aicCoreNum = 0;  // upper bound on CTAs (0 = one per SM)
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrScale = nullptr;
        uint8_t* ptrPerTokenScale = nullptr;
        uint8_t* ptrD = nullptr;
        uint32_t scaleType = CB200_DTYPE_F32;  // element type of both scale vectors (the reference's ElementScale)
        uint32_t dType = CB200_DTYPE_BF16;     // element type of D (the reference's ElementD: bf16 or half)
        uint32_t flags = 0;                    // CB200_FLAG_STATIC_WEIGHTS
    };
    using CArgs = cb200_quant_matmul_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.layout_a = detail::LayoutTag<LayoutA>::value;
        c.layout_b = detail::LayoutTag<LayoutB>::value;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.scale = a.ptrScale;
        c.per_token_scale = a.ptrPerTokenScale;
        c.d = a.ptrD;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        c.block_num = a.aicCoreNum;
        c.flags = a.flags;
        c.scale_type = a.scaleType;
        c.d_type = a.dType;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_quant_matmul_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c) { return cb200_quant_matmul_workspace_size(c); }
    static int Run(CArgs const* c, void* stream) { return cb200_quant_matmul(c, stream); }
};

/// Grouped slice-M W8A8 with per-token dequant. Arguments as
/// GroupedMatmulSliceMPerTokenDequant::Arguments (grouped_matmul_slice_m_per_token_dequant.hpp:125-137).
template <class LayoutB = layout::RowMajor, class ElementGroupList = int64_t>
struct GroupedMatmulSliceMPerTokenDequant {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t problemCount = 0;
        uint8_t* ptrGroupList = nullptr;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrScale = nullptr;
        uint8_t* ptrPerTokenScale = nullptr;
        uint8_t* ptrD = nullptr;
        uint32_t aicCoreNum = 0;
        uint32_t scaleType = CB200_DTYPE_F32;
        uint32_t dType = CB200_DTYPE_BF16;
    };
    using CArgs = cb200_grouped_quant_matmul_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        static_assert(sizeof(ElementGroupList) == 8 || sizeof(ElementGroupList) == 4, "int64 or int32 group list");
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.group_count = a.problemCount;
        c.layout_b = detail::LayoutTag<LayoutB>::value;
        c.group_list_type = sizeof(ElementGroupList) == 8 ? CB200_GROUP_LIST_INT64 : CB200_GROUP_LIST_INT32;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.group_list = a.ptrGroupList;
        c.scale = a.ptrScale;
        c.per_token_scale = a.ptrPerTokenScale;
        c.d = a.ptrD;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        c.block_num = a.aicCoreNum;
        c.scale_type = a.scaleType;
        c.d_type = a.dType;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_grouped_quant_matmul_slice_m_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c) { return cb200_grouped_quant_matmul_slice_m_workspace_size(c); }
    static int Run(CArgs const* c, void* stream) { return cb200_grouped_quant_matmul_slice_m(c, stream); }
};

/// Grouped slice-M W8A8 with per-tensor or per-channel dequant (no per-token factor).  Arguments as
/// GroupedMatmulSliceMFixpipeDequantTla::Arguments (example 48: problemShape, problemCount, ptrGroupList, ptrA,
/// ptrB, ptrC, scalePerTensor, ptrPerChannelScale).  kPerChannel is the reference's ScaleGranularity template
/// argument; the per-channel scales are the reference's 64-bit words (fp32 bits in the low half).
template <bool kPerChannel, class LayoutB = layout::RowMajor, class ElementGroupList = int64_t>
struct GroupedMatmulSliceMFixpipeDequant {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t problemCount = 0;
        uint8_t* ptrGroupList = nullptr;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrC = nullptr;
        float scalePerTensor = 1.0f;
        uint8_t* ptrPerChannelScale = nullptr;
        uint32_t perChannelScaleType = CB200_DTYPE_F32_IN_U64;
        uint32_t dType = CB200_DTYPE_F16;  // the reference writes half
    };
    using CArgs = cb200_grouped_fixpipe_dequant_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.group_count = a.problemCount;
        c.layout_b = detail::LayoutTag<LayoutB>::value;
        c.group_list_type = sizeof(ElementGroupList) == 8 ? CB200_GROUP_LIST_INT64 : CB200_GROUP_LIST_INT32;
        c.quant_mode = kPerChannel ? CB200_QUANT_PER_CHANNEL : CB200_QUANT_PER_TENSOR;
        c.scale_per_tensor = a.scalePerTensor;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.group_list = a.ptrGroupList;
        c.per_channel_scale = a.ptrPerChannelScale;
        c.d = a.ptrC;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        c.per_channel_scale_type = a.perChannelScaleType;
        c.d_type = a.dType;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_grouped_matmul_slice_m_fixpipe_dequant_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c)
    {
        return cb200_grouped_matmul_slice_m_fixpipe_dequant_workspace_size(c);
    }
    static int Run(CArgs const* c, void* stream) { return cb200_grouped_matmul_slice_m_fixpipe_dequant(c, stream); }
};

/// W4A8 with per-group weight scales (W4A8Matmul::Arguments, w4a8_matmul.hpp:83-93, plus the scale arrays).
struct W4A8Matmul {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t groupSize = 128;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrPackedB = nullptr;
        uint8_t* ptrWeightScale = nullptr;
        uint8_t* ptrPerTokenScale = nullptr;
        uint8_t* ptrC = nullptr;
        uint32_t dType = CB200_DTYPE_BF16;
        uint32_t flags = 0;  // CB200_W4A8_SPLIT_K, CB200_FLAG_STATIC_WEIGHTS
    };
    using CArgs = cb200_w4a8_matmul_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.group_size = a.groupSize;
        c.a = a.ptrA;
        c.w_packed = a.ptrPackedB;
        c.weight_scale = reinterpret_cast<const float*>(a.ptrWeightScale);
        c.per_token_scale = reinterpret_cast<const float*>(a.ptrPerTokenScale);
        c.d = a.ptrC;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        c.flags = a.flags;
        c.d_type = a.dType;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_w4a8_matmul_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c) { return cb200_w4a8_matmul_workspace_size(c); }
    static int Run(CArgs const* c, void* stream) { return cb200_w4a8_matmul(c, stream); }
};

/// MX block-scaled matmul (MxMatmulTla::Arguments, mx_matmul_tla.hpp:95-108).  kFp4 selects E2M1 elements.
template <bool kFp4>
struct MxMatmul {
    struct Arguments {
        GemmCoord problemShape;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrMxScaleA = nullptr;
        uint8_t* ptrMxScaleB = nullptr;
        uint8_t* ptrC = nullptr;
    };
    using CArgs = cb200_mx_matmul_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.format = kFp4 ? CB200_MX_E2M1 : CB200_MX_E4M3;
        c.layout_a = CB200_ROW_MAJOR;
        c.layout_b = CB200_COLUMN_MAJOR;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.scale_a = a.ptrMxScaleA;
        c.scale_b = a.ptrMxScaleB;
        c.d = a.ptrC;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_mx_matmul_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c) { return cb200_mx_matmul_workspace_size(c); }
    static int Run(CArgs const* c, void* stream) { return cb200_mx_matmul(c, stream); }
};

/// Grouped slice-K W8A8 with per-token dequant: GroupedMatmulSliceKPerTokenDequant::Arguments of the reference
/// (include/catlass/gemm/kernel/grouped_matmul_slice_k_per_token_dequant.hpp:125-134: problemShape, problemCount,
/// ptrGroupList, ptrA [k][m], ptrB [k][n], ptrScale [G][n], ptrPerTokenScale [G][m], ptrD [G][m][n]).
template <class ElementGroupList = int64_t>
struct GroupedMatmulSliceKPerTokenDequant {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t problemCount = 0;
        uint8_t* ptrGroupList = nullptr;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrScale = nullptr;
        uint8_t* ptrPerTokenScale = nullptr;
        uint8_t* ptrD = nullptr;
        uint32_t scaleType = CB200_DTYPE_F32;
        uint32_t dType = CB200_DTYPE_BF16;
    };
    using CArgs = cb200_grouped_quant_matmul_slice_k_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.group_count = a.problemCount;
        c.group_list_type = sizeof(ElementGroupList) == 8 ? CB200_GROUP_LIST_INT64 : CB200_GROUP_LIST_INT32;
        c.scale_type = a.scaleType;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.group_list = a.ptrGroupList;
        c.scale = a.ptrScale;
        c.per_token_scale = a.ptrPerTokenScale;
        c.d = a.ptrD;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        c.d_type = a.dType;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_grouped_quant_matmul_slice_k_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c) { return cb200_grouped_quant_matmul_slice_k_workspace_size(c); }
    static int Run(CArgs const* c, void* stream) { return cb200_grouped_quant_matmul_slice_k(c, stream); }
};

/// Grouped slice-M MX matmul: GroupedMxMatmulSliceMTla::Arguments of the reference (example 55:
/// examples/55_ascend950_mx_grouped_matmul_slice_m/mx_grouped_matmul_slice_m.cpp:325-357).  The group list holds
/// the groups' row counts, as there.  LayoutB: ColumnMajor = [G][n][k] (the example's "trans" case), RowMajor = [G][k][n].
template <bool kFp4, class LayoutB = layout::ColumnMajor, class ElementGroupList = int64_t>
struct GroupedMxMatmulSliceM {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t problemCount = 0;
        uint8_t* ptrGroupList = nullptr;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrMxScaleA = nullptr;
        uint8_t* ptrMxScaleB = nullptr;
        uint8_t* ptrC = nullptr;       // fp32 [m][n], what the reference's kernel writes
    };
    using CArgs = cb200_mx_grouped_matmul_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.group_count = a.problemCount;
        c.format = kFp4 ? CB200_MX_E2M1 : CB200_MX_E4M3;
        c.layout_b = detail::LayoutTag<LayoutB>::value;
        c.group_list_type = sizeof(ElementGroupList) == 8 ? CB200_GROUP_LIST_INT64 : CB200_GROUP_LIST_INT32;
        c.group_list_kind = CB200_GROUP_LIST_SIZES;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.group_list = a.ptrGroupList;
        c.scale_a = a.ptrMxScaleA;
        c.scale_b = a.ptrMxScaleB;
        c.d = a.ptrC;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        c.flags = CB200_MX_OUT_F32;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_mx_grouped_matmul_slice_m_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c) { return cb200_mx_grouped_matmul_slice_m_workspace_size(c); }
    static int Run(CArgs const* c, void* stream) { return cb200_mx_grouped_matmul_slice_m(c, stream); }
};

/// Grouped MXFP8 matmul + SwiGLU + MX quantisation: GroupedMxMatmulSliceMSwigluMxQuantTla::Arguments of the reference
/// (include/catlass/gemm/kernel/grouped_mx_matmul_slice_m_swiglu_mx_quant_tla.hpp:72-118: problemShape, problemCount,
/// ptrGroupList, ptrA, ptrB, ptrMxScaleA, ptrMxScaleB, ptrQ, ptrQScale).
template <class LayoutB = layout::ColumnMajor, class ElementGroupList = int64_t>
struct GroupedMxMatmulSliceMSwigluMxQuant {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t problemCount = 0;
        uint8_t* ptrGroupList = nullptr;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrMxScaleA = nullptr;
        uint8_t* ptrMxScaleB = nullptr;
        uint8_t* ptrQ = nullptr;       // E4M3 [m][n/2]
        uint8_t* ptrQScale = nullptr;  // E8M0 [m][n/64]
    };
    using CArgs = cb200_mx_grouped_swiglu_quant_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.group_count = a.problemCount;
        c.layout_b = detail::LayoutTag<LayoutB>::value;
        c.group_list_type = sizeof(ElementGroupList) == 8 ? CB200_GROUP_LIST_INT64 : CB200_GROUP_LIST_INT32;
        c.group_list_kind = CB200_GROUP_LIST_SIZES;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.group_list = a.ptrGroupList;
        c.scale_a = a.ptrMxScaleA;
        c.scale_b = a.ptrMxScaleB;
        c.q = a.ptrQ;
        c.q_scale = a.ptrQScale;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c)
    {
        return cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_workspace_size(c);
    }
    static int Run(CArgs const* c, void* stream) { return cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant(c, stream); }
};

/// Grouped MXFP8 matmul + finalize routing (the reference's GroupedMxMatmulFinalizeRoutingNoDeterTla; parameters as
/// GroupedMxFinalizeRoutingParams, tests/optest/include/catlass_kernel_jit.h:489-495): out [batch][n] fp32.
template <class LayoutB = layout::ColumnMajor, class ElementGroupList = int64_t>
struct GroupedMxMatmulFinalizeRouting {
    struct Arguments {
        GemmCoord problemShape;
        uint32_t problemCount = 0;
        uint32_t groupListType = 0;    // 0: prefix sums, 1: row counts (the reference's convention)
        uint8_t* ptrGroupList = nullptr;
        uint8_t* ptrA = nullptr;
        uint8_t* ptrB = nullptr;
        uint8_t* ptrMxScaleA = nullptr;
        uint8_t* ptrMxScaleB = nullptr;
        uint8_t* ptrLogit = nullptr;        // fp32 [m]
        uint8_t* ptrRowIndex = nullptr;     // int64 [m]
        uint8_t* ptrBias = nullptr;         // bf16 [problemCount][n] or null
        uint8_t* ptrSharedInput = nullptr;  // bf16 [bsdp][n] or null
        uint8_t* ptrOut = nullptr;          // fp32 [batch][n]
        uint32_t batch = 0;
        uint32_t bsdp = 0;
        float sharedInputWeight = 0.0f;
        uint32_t sharedInputOffset = 0;
    };
    using CArgs = cb200_mx_grouped_finalize_routing_args;
    static CArgs ToUnderlyingArguments(Arguments const& a, void* workspace, size_t workspaceBytes)
    {
        CArgs c{};
        c.m = a.problemShape.m();
        c.n = a.problemShape.n();
        c.k = a.problemShape.k();
        c.group_count = a.problemCount;
        c.layout_b = detail::LayoutTag<LayoutB>::value;
        c.group_list_type = sizeof(ElementGroupList) == 8 ? CB200_GROUP_LIST_INT64 : CB200_GROUP_LIST_INT32;
        c.group_list_kind = a.groupListType == 0 ? CB200_GROUP_LIST_PREFIX_SUMS : CB200_GROUP_LIST_SIZES;
        c.row_index_type = CB200_GROUP_LIST_INT64;
        c.batch = a.batch;
        c.shared_rows = a.bsdp;
        c.shared_offset = a.sharedInputOffset;
        c.shared_weight = a.sharedInputWeight;
        c.a = a.ptrA;
        c.b = a.ptrB;
        c.group_list = a.ptrGroupList;
        c.scale_a = a.ptrMxScaleA;
        c.scale_b = a.ptrMxScaleB;
        c.logit = a.ptrLogit;
        c.row_index = a.ptrRowIndex;
        c.bias = a.ptrBias;
        c.shared_input = a.ptrSharedInput;
        c.out = a.ptrOut;
        c.workspace = workspace;
        c.workspace_bytes = workspaceBytes;
        return c;
    }
    static int CanImplement(CArgs const* c) { return cb200_mx_grouped_matmul_finalize_routing_can_implement(c); }
    static uint64_t WorkspaceSize(CArgs const* c) { return cb200_mx_grouped_matmul_finalize_routing_workspace_size(c); }
    static int Run(CArgs const* c, void* stream) { return cb200_mx_grouped_matmul_finalize_routing(c, stream); }
};

}  // namespace Kernel

namespace Device {

template <class Kernel_>
class DeviceGemm {
public:
    using Kernel = Kernel_;
    using Arguments = typename Kernel::Arguments;

    /// Checks alignment, layouts and ranges (the reference's kernels always answer true).
    static Status CanImplement(Arguments const& args)
    {
        auto c = Kernel::ToUnderlyingArguments(args, nullptr, 0);
        return detail::ToStatus(Kernel::CanImplement(&c));
    }
    static size_t GetWorkspaceSize(Arguments const& args)
    {
        auto c = Kernel::ToUnderlyingArguments(args, nullptr, 0);
        return static_cast<size_t>(Kernel::WorkspaceSize(&c));
    }
    /// Keeps the arguments and the caller's workspace (device memory of at least GetWorkspaceSize bytes).
    Status Initialize(Arguments const& args, uint8_t* workspace = nullptr)
    {
        cargs_ = Kernel::ToUnderlyingArguments(args, workspace, GetWorkspaceSize(args));
        initialized_ = true;
        return detail::ToStatus(Kernel::CanImplement(&cargs_));
    }
    /// Enqueues the kernel(s) on `stream`; does not synchronise. blockNum bounds the number of CTAs (0 = auto).
    Status operator()(void* stream, uint32_t blockNum = 0)
    {
        if (!initialized_) {
            return Status::kInvalid;
        }
        if (blockNum != 0) {
            cargs_.block_num = blockNum;
        }
        lastCode_ = Kernel::Run(&cargs_, stream);
        return detail::ToStatus(lastCode_);
    }
    int LastCode() const { return lastCode_; }

private:
    typename Kernel::CArgs cargs_{};
    bool initialized_ = false;
    int lastCode_ = 0;
};

}  // namespace Device
}  // namespace Catlass::Gemm
