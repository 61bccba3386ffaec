/*
 * catlass_b200 - C ABI of the B200 (sm_100a) quantized-matmul library.
 *
 * Plain C: PODs, raw device pointers and sizes only.  Every operator comes as a triple that mirrors the
 * reference's device adapter (include/catlass/gemm/device/device_gemm.hpp:47-97):
 *     <op>_can_implement(args)   -> status            (DeviceGemm::CanImplement)
 *     <op>_workspace_size(args)  -> bytes             (DeviceGemm::GetWorkspaceSize)
 *     <op>(args, stream)         -> status, async     (DeviceGemm::Initialize + operator())
 * The caller owns all buffers, including the workspace (args->workspace, at least _workspace_size bytes,
 * 256-byte aligned).  Calls enqueue work on `stream` (a cudaStream_t passed as void*) and return without
 * synchronising.  All pointers are device pointers unless stated otherwise.
 *
 * Status: 0 = success (Catlass::Status::kSuccess, include/catlass/status.hpp:16-20), 1 = invalid
 * arguments / unsupported problem (Status::kInvalid), >= 2 = runtime failures listed below.
 */
#ifndef CATLASS_B200_H
#define CATLASS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define CB200_API
#else
#define CB200_API __attribute__((visibility("default")))
#endif

/* ---- status ---- */
#define CB200_SUCCESS 0
#define CB200_INVALID 1        /* bad descriptor: null pointer, misaligned buffer, unsupported layout */
#define CB200_CUDA_ERROR 2     /* a CUDA runtime/driver call failed (see cb200_last_cuda_error) */
#define CB200_DEVICE_TIMEOUT 3 /* a kernel gave up on a bounded wait (see cb200_device_status) */
#define CB200_SCRATCH_TOO_SMALL 4 /* the problem needs more scratch than a fixed-scratch entry point owns */

/* ---- matrix layouts (include/catlass/layout/matrix.hpp: RowMajor :24, ColumnMajor :168, zN :475) ---- */
#define CB200_ROW_MAJOR 0
#define CB200_COLUMN_MAJOR 1
#define CB200_ZN 2 /* weights only: 16-row x 32-byte fractals, layout::zN::MakeLayout<int8_t>(k, n) */

/* ---- group list element type (the reference accepts int32 or int64 prefix sums) ---- */
#define CB200_GROUP_LIST_INT64 0
#define CB200_GROUP_LIST_INT32 1

/* ---- element types of scale vectors and of the output D ----
 * The reference instantiates its W8A8 kernels with fp32, bf16 or half scales and bf16 or half outputs
 * (examples 12: half/half, 07: float/half, 10: bf16/bf16); the goldens convert a scale to float before they
 * use it (examples/common/golden/matmul.hpp:296-298), so do the kernels here. */
#define CB200_DTYPE_F32 0
#define CB200_DTYPE_BF16 1
#define CB200_DTYPE_F16 2
#define CB200_DTYPE_F32_IN_U64 3 /* fp32 bit pattern in the low half of a uint64: the reference's fixpipe scales */

/* ---- flags ----
 * CB200_FLAG_STATIC_WEIGHTS: the weight matrix and the weight/channel scales of this call are not written by
 * any work enqueued earlier on the same stream (the usual case: parameters loaded once).  The few-token (m <= 128)
 * W8A8 kernel and the W4A8 kernel are launched with programmatic dependent launch; with this flag they start
 * streaming weights while the kernel before them on the stream is still finishing.  Without it every read of
 * global memory waits for that kernel (plain stream order).  Activations, per-token scales and the output are
 * always ordered after it. */
#define CB200_FLAG_STATIC_WEIGHTS 2u

/*
 * Dense W8A8 matmul with per-token / per-channel dequant:
 *     D[i,j] = bf16_rne( (float(sum_k A[i,k]*B[k,j]) * scale[j]) * per_token_scale[i] )
 * Replaces the kernels behind examples 12 / 42 / 103:
 *     Gemm::Kernel::QuantMatmulMultiStageWorkspace::Arguments
 *         (include/catlass/gemm/kernel/quant_matmul_multistage_workspace.hpp:92-100),
 *     operand order of tests/optest/kernels/12_quant_matmul/quant_matmul_impl.cpp:103-105
 *         (inputs A, B, scale, perTokenScale; output D).
 * A: int8 m x k row-major or column-major (the four layout pairs of example 103,
 * examples/103_dynamic_optimized_quant_matmul_per_token_basic/include/do_tiling_b8.h:24,62,117,166; column-major A
 * needs m % 16 == 0); B: int8 k x n row-major, column-major (densely packed) or in the reference's zN
 * fractal format (k padded to 16, n to 32: layout::zN::MakeLayout<int8_t>(k, n)); D: m x n row-major.
 * Thread safety: any number of host threads may call concurrently, on any streams.
 */
typedef struct cb200_quant_matmul_args {
    uint32_t m, n, k;
    uint32_t layout_a;            /* CB200_ROW_MAJOR or CB200_COLUMN_MAJOR */
    uint32_t layout_b;            /* CB200_ROW_MAJOR, CB200_COLUMN_MAJOR or CB200_ZN */
    const void *a;                /* int8 */
    const void *b;                /* int8 */
    const void *scale;            /* n per-channel scales, scale_type elements */
    const void *per_token_scale;  /* m per-token scales, scale_type elements */
    void *d;                      /* out, d_type elements */
    int32_t *acc;                 /* optional: raw int32 accumulators, m x n row-major (NULL = off) */
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;           /* upper bound on the CTAs launched; 0 = one per SM */
    uint32_t flags;               /* 0, or CB200_FLAG_STATIC_WEIGHTS */
    uint32_t scale_type;          /* CB200_DTYPE_F32 (0, default), _BF16 or _F16: type of both scale vectors */
    uint32_t d_type;              /* CB200_DTYPE_BF16 (default; 0 is accepted as bf16) or CB200_DTYPE_F16 */
} cb200_quant_matmul_args;

CB200_API int cb200_quant_matmul_can_implement(const cb200_quant_matmul_args *args);
CB200_API uint64_t cb200_quant_matmul_workspace_size(const cb200_quant_matmul_args *args);
CB200_API int cb200_quant_matmul(const cb200_quant_matmul_args *args, void *stream);

/*
 * Grouped (MoE) slice-M W8A8 matmul with per-token dequant.  group_list holds `group_count` ascending
 * prefix sums of rows; group g owns rows [group_list[g-1], group_list[g]) of A and D, weight matrix
 * B + g*k*n and channel scales scale + g*n.  Rows at or beyond group_list[group_count-1] are not written.
 * Replaces the kernels behind examples 07 / 10 / 47:
 *     Gemm::Kernel::GroupedMatmulSliceMPerTokenDequant::Arguments
 *         (include/catlass/gemm/kernel/grouped_matmul_slice_m_per_token_dequant.hpp:125-137),
 *     operand order of tests/optest/kernels/07_grouped_matmul_slice_m_per_token_dequant_moe/
 *         grouped_matmul_slice_m_per_token_dequant_moe_impl.cpp:98-102
 *         (inputs A, B, groupList, scale, perTokenScale; batch = group count).
 * m is the row capacity of A / D / per_token_scale (group_list entries are clamped to it).
 * Thread safety: any number of host threads may call concurrently, on any streams.
 */
typedef struct cb200_grouped_quant_matmul_args {
    uint32_t m, n, k;
    uint32_t group_count;         /* 1 .. 1024 */
    uint32_t layout_b;            /* layout of each k x n weight matrix (row-major, column-major or zN;
                                     zN matrices follow each other Capacity() bytes apart) */
    uint32_t group_list_type;     /* CB200_GROUP_LIST_INT64 / _INT32 */
    const void *a;                /* int8 m x k row-major */
    const void *b;                /* int8 [group_count][k x n] */
    const void *group_list;       /* device pointer */
    const void *scale;            /* [group_count][n], scale_type elements */
    const void *per_token_scale;  /* [m], scale_type elements */
    void *d;                      /* m x n row-major, d_type elements */
    int32_t *acc;                 /* optional raw accumulators */
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t flags;               /* 0 */
    uint32_t scale_type;          /* CB200_DTYPE_F32 (0, default), _BF16 or _F16 */
    uint32_t d_type;              /* CB200_DTYPE_BF16 (default; 0 is accepted as bf16) or CB200_DTYPE_F16 */
} cb200_grouped_quant_matmul_args;

CB200_API int cb200_grouped_quant_matmul_slice_m_can_implement(const cb200_grouped_quant_matmul_args *args);
CB200_API uint64_t cb200_grouped_quant_matmul_slice_m_workspace_size(const cb200_grouped_quant_matmul_args *args);
CB200_API int cb200_grouped_quant_matmul_slice_m(const cb200_grouped_quant_matmul_args *args, void *stream);

/*
 * Grouped slice-M W8A8 matmul with per-tensor or per-channel dequant and no per-token factor:
 *     quant_mode 0:  D[i,j] = round( float(acc[i,j]) * scale_per_tensor )
 *     quant_mode 1:  D[i,j] = round( float(acc[i,j]) * per_channel_scale[j] )     one [n] vector for all groups
 * Groups, group_list and B as in cb200_grouped_quant_matmul_slice_m.  Replaces the kernel behind example 48:
 *     Gemm::Kernel::GroupedMatmulSliceMFixpipeDequantTla::Arguments (problemShape, problemCount, ptrGroupList,
 *     ptrA, layoutA, ptrB, layoutB, ptrC, layoutC, scalePerTensor, ptrPerChannelScale:
 *     examples/48_ascend950_grouped_matmul_slice_m_per_tensor_per_channel_dequant/
 *     grouped_matmul_slice_m_per_tensor_per_channel_dequant.cpp:173-185), golden
 *     golden::ComputeGroupedMatmulFixpipeDequant (examples/common/golden/matmul.hpp:234-269).
 * The reference hands the per-channel scales over as 64-bit words with the fp32 bits in the low half
 * (same file :103-107): pass them unchanged with per_channel_scale_type = CB200_DTYPE_F32_IN_U64, or a plain
 * float array with CB200_DTYPE_F32.  The reference writes half: d_type = CB200_DTYPE_F16.
 */
#define CB200_QUANT_PER_TENSOR 0
#define CB200_QUANT_PER_CHANNEL 1
typedef struct cb200_grouped_fixpipe_dequant_args {
    uint32_t m, n, k;
    uint32_t group_count;
    uint32_t layout_b;
    uint32_t group_list_type;
    uint32_t quant_mode;              /* CB200_QUANT_PER_TENSOR / CB200_QUANT_PER_CHANNEL */
    float scale_per_tensor;
    const void *a;                    /* int8 m x k row-major */
    const void *b;                    /* int8 [group_count][k x n] */
    const void *group_list;
    const void *per_channel_scale;    /* [n]; read in per-channel mode only */
    void *d;                          /* m x n row-major, d_type elements */
    int32_t *acc;                     /* optional raw accumulators */
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t per_channel_scale_type;  /* CB200_DTYPE_F32 or CB200_DTYPE_F32_IN_U64 */
    uint32_t d_type;                  /* CB200_DTYPE_BF16 (0 accepted) or CB200_DTYPE_F16 */
    uint32_t flags;                   /* 0 */
} cb200_grouped_fixpipe_dequant_args;

CB200_API int cb200_grouped_matmul_slice_m_fixpipe_dequant_can_implement(
    const cb200_grouped_fixpipe_dequant_args *args);
CB200_API uint64_t cb200_grouped_matmul_slice_m_fixpipe_dequant_workspace_size(
    const cb200_grouped_fixpipe_dequant_args *args);
CB200_API int cb200_grouped_matmul_slice_m_fixpipe_dequant(const cb200_grouped_fixpipe_dequant_args *args,
                                                           void *stream);

/*
 * Grouped slice-K W8A8 matmul with per-token dequant: the groups cut K.  group_list holds `group_count` ascending
 * prefix sums over K; group g multiplies A[:, K_g] with B[K_g, :] into its own m x n block of D:
 *     D[g][i][j] = round( (float(sum_{kk in K_g} A[i,kk] * B[kk,j]) * scale[g][j]) * per_token_scale[g][i] )
 * (an empty group gives zeros).  Replaces Gemm::Kernel::GroupedMatmulSliceKPerTokenDequant::Arguments
 * (include/catlass/gemm/kernel/grouped_matmul_slice_k_per_token_dequant.hpp:125-134: problemShape, problemCount,
 * ptrGroupList, ptrA, ptrB, ptrScale, ptrPerTokenScale, ptrD; example 11), golden
 * golden::ComputeGroupedMatmulSliceKPerTokenDequant (examples/common/golden/matmul.hpp:326-359).
 * Layouts are the reference's for this operator: A column-major (stored [k][m]), B row-major ([k][n]).
 * Requirements: m % 16 == 0, n % 16 == 0, a and b 16-byte aligned.  The groups' K ranges start at arbitrary rows;
 * an ingestion pre-pass copies A and B into the workspace with every group padded to whole 128-row K blocks
 * (cb200_grouped_quant_matmul_slice_k_workspace_size bytes: about (k + 128 * group_count) * (m + n)).
 */
typedef struct cb200_grouped_quant_matmul_slice_k_args {
    uint32_t m, n, k;
    uint32_t group_count;         /* 1 .. 1024 */
    uint32_t group_list_type;     /* CB200_GROUP_LIST_INT64 / _INT32 */
    uint32_t scale_type;          /* CB200_DTYPE_F32 (0, default), _BF16 or _F16 */
    const void *a;                /* int8 [k][m] */
    const void *b;                /* int8 [k][n] */
    const void *group_list;       /* device pointer */
    const void *scale;            /* [group_count][n] */
    const void *per_token_scale;  /* [group_count][m] */
    void *d;                      /* [group_count][m][n], d_type elements */
    int32_t *acc;                 /* optional raw accumulators [group_count][m][n] */
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t d_type;              /* CB200_DTYPE_BF16 (default; 0 accepted) or CB200_DTYPE_F16 */
} cb200_grouped_quant_matmul_slice_k_args;

CB200_API int cb200_grouped_quant_matmul_slice_k_can_implement(const cb200_grouped_quant_matmul_slice_k_args *args);
CB200_API uint64_t cb200_grouped_quant_matmul_slice_k_workspace_size(
    const cb200_grouped_quant_matmul_slice_k_args *args);
CB200_API int cb200_grouped_quant_matmul_slice_k(const cb200_grouped_quant_matmul_slice_k_args *args, void *stream);

/*
 * The grouped matmul for HOST-resident activations and output: what the reference's example mains do around
 * the kernel (aclrtMemcpy host->device, launch, aclrtMemcpy device->host:
 * examples/07_grouped_matmul_slice_m_per_token_dequant_moe/grouped_matmul_slice_m_per_token_dequant_moe.cpp:
 * 78-110, 176-184), folded into one call that overlaps the three phases.  The routed rows are cut into
 * `chunks` row ranges; chunk c+1 is copied in (PCIe down) while chunk c is computed and chunk c-1 is copied
 * out (PCIe up), on two library-owned copy streams ordered against `stream` with events.
 * a_host, per_token_host, group_list_host, d_host are host pointers (pinned memory for real overlap);
 * b and scale (the expert weights) stay on the device.  The device workspace
 * (cb200_grouped_quant_matmul_slice_m_host_workspace_size bytes) stages A, the per-token scales, D and the
 * per-chunk group lists.  On return all work is enqueued; d_host is complete once `stream` has caught up.
 * Thread safety: calls on one device are serialised inside the library (they share its copy streams and a
 * pinned staging buffer for the group lists); calls on different devices run concurrently.
 */
typedef struct cb200_grouped_quant_matmul_host_args {
    uint32_t m, n, k;
    uint32_t group_count;
    uint32_t layout_b;
    uint32_t chunks;                  /* 0 = library default (16) */
    const void *a_host;               /* int8 m x k */
    const int64_t *group_list_host;   /* prefix sums */
    const float *per_token_host;      /* [m] */
    void *d_host;                     /* bf16 m x n */
    const void *b;                    /* device: int8 [group_count][k x n] */
    const float *scale;               /* device: [group_count][n] */
    void *workspace;                  /* device */
    uint64_t workspace_bytes;
} cb200_grouped_quant_matmul_host_args;

CB200_API uint64_t cb200_grouped_quant_matmul_slice_m_host_workspace_size(
    const cb200_grouped_quant_matmul_host_args *args);
CB200_API int cb200_grouped_quant_matmul_slice_m_host(const cb200_grouped_quant_matmul_host_args *args,
                                                      void *stream);

/*
 * W4A8 matmul with per-group weight scales:
 *     acc_g[i,j] = sum_{k in group g} A[i,k] * W[k,j]                       (int32)
 *     y[i,j]     = fma(float(acc_g), weight_scale[g,j], y), g ascending     (fp32, y starts at 0)
 *     D[i,j]     = round(y * per_token_scale[i])
 * W holds signed 4-bit values, two per byte along K (even k in bits 0-3, odd k in bits 4-7), column after
 * column (ceil(k/2) bytes each): the packing of the reference's example 32 for a column-major B
 * (examples/32_w4a8_matmul/gen_data.py:77-105).  Replaces Gemm::Kernel::W4A8Matmul::Arguments
 * (include/catlass/gemm/kernel/w4a8_matmul.hpp:83-93; operand order A, packed B of
 * tests/optest/kernels/32_w4a8_matmul/w4a8_matmul_impl.cpp:101-103).  The reference's own kernel applies one
 * per-tensor scalar and writes half; that case is group_size = k with weight_scale all ones,
 * per_token_scale = the scalar and d_type = CB200_DTYPE_F16.
 *
 * Which fp32 reading of "rescale each group and sum in fp32" this is: ONE rounding per group (a fused
 * multiply-add), groups in ascending order.  The reference holds no per-group golden to settle the choice; the
 * fused form is the more accurate of the two natural readings (the unfused one rounds the product first) and
 * is what the hardware does at full rate.  Both readings, and any other summation order, agree with the exact
 * sum to within 2^-22 x sum_g |acc_g * weight_scale[g,j]| x per_token_scale[i] (64 groups, one ulp of the
 * running sum each at most), plus the final rounding of D; the GPU tests check the output against the exact
 * (float64) sum with that bound, and bit for bit against the fused definition.
 *
 * Requirements: group_size a multiple of 128 (the last group may be shorter), or group_size >= k (one group over
 * any k, also odd: the reference's runner case m=860 n=5712 k=4535); at most 16384 elements per group.
 * Fast path: weights packed along K, k a multiple of 128 (and of group_size), a and w_packed 16-byte aligned: the
 * operands are streamed in place and the workspace is not used.  Everything else (k not a whole number of blocks,
 * weights packed along N as in tests/optest/tests/test_32_w4a8_matmul.py:11-28, unaligned operands) first goes
 * through an ingestion pre-pass that writes zero-padded, K-packed copies of both operands into the workspace
 * (cb200_w4a8_matmul_workspace_size bytes): one extra pass over A and W; keep weights in the fast-path form
 * where speed matters.
 * Summation order: by default the groups are summed in ascending order, exactly as written above (D is
 * bit-exact against that definition).  With CB200_W4A8_SPLIT_K in `flags`, shapes with few 128-channel tiles
 * split the groups over the 2 or 4 CTAs of a cluster and add the fp32 partial sums at the end: faster, but an
 * output whose partial sums nearly cancel can then differ from the definition by more than one ulp of its small
 * value; the absolute difference stays inside the bound above.
 * Thread safety: any number of host threads may call concurrently, on any streams.
 */
#define CB200_W4A8_SPLIT_K 1u
#define CB200_W4_PACKED_ALONG_K 0 /* w_packed: n columns of ceil(k/2) bytes (the reference's column-major B) */
#define CB200_W4_PACKED_ALONG_N 1 /* w_packed: k rows of ceil(n/2) bytes (the reference's row-major B) */
typedef struct cb200_w4a8_matmul_args {
    uint32_t m, n, k;
    uint32_t group_size;
    const void *a;                /* int8 m x k row-major */
    const void *w_packed;         /* n columns of k/2 bytes */
    const float *weight_scale;    /* [ceil(k / group_size)][n] */
    const float *per_token_scale; /* [m] */
    void *d;                      /* m x n row-major, d_type elements */
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t flags;               /* 0, CB200_W4A8_SPLIT_K and/or CB200_FLAG_STATIC_WEIGHTS */
    uint32_t d_type;              /* CB200_DTYPE_BF16 (0 accepted) or CB200_DTYPE_F16 */
    uint32_t pack_axis;           /* CB200_W4_PACKED_ALONG_K (0, default) or CB200_W4_PACKED_ALONG_N */
} cb200_w4a8_matmul_args;

CB200_API int cb200_w4a8_matmul_can_implement(const cb200_w4a8_matmul_args *args);
CB200_API uint64_t cb200_w4a8_matmul_workspace_size(const cb200_w4a8_matmul_args *args);
CB200_API int cb200_w4a8_matmul(const cb200_w4a8_matmul_args *args, void *stream);

/*
 * MX block-scaled matmul (OCP microscaling): elements E4M3 (one byte) or E2M1 (two per byte, even index in bits
 * 0-3), one E8M0 scale byte per 32 contiguous K elements of every row of A and every column of B:
 *     D[i,j] = round( sum_k (A[i,k] * 2^(scale_a[i,k/32]-127)) * (B[k,j] * 2^(scale_b[j,k/32]-127)) )
 * accumulated in fp32 inside the tensor core.  Replaces Gemm::Kernel::MxMatmulTla::Arguments
 * (include/catlass/gemm/kernel/mx_matmul_tla.hpp:95-108; operand order A, B, scaleA, scaleB of
 * tests/optest/kernels/53_ascend950_fp8_mx_matmul/fp8_mx_matmul_impl.cpp:80-84).
 *
 * Layouts (the four transpose pairs of tests/optest/tests/test_53_ascend950_fp8_mx_matmul_aswt.py:21-30):
 *   layout_a = CB200_ROW_MAJOR: A is [m][k];  CB200_COLUMN_MAJOR: A is stored [k][m] (the reference's transA)
 *   layout_b = CB200_COLUMN_MAJOR: B is stored [n][k] (the reference's transB, its default);  CB200_ROW_MAJOR: [k][n]
 *   E2M1 arrays pack two elements per byte along their contiguous axis (an odd count leaves the last high nibble
 *   unused).
 * Scales follow the operand, as the reference's do (tests/optest/tests/mx_golden.py:253-266), with
 * KS = ceil(k/32) rounded up to even:
 *   operand stored with rows along K ([m][k] / [n][k]):  scale array [rows][KS] bytes (the reference's [rows, KS/2, 2])
 *   operand stored the other way ([k][m] / [k][n]):      scale array [KS/2][rows][2] bytes
 * k is arbitrary (the reference's tests run k = 2, 33, 63, 129).
 * Fast path: A [m][k] and B [n][k], k a multiple of 128 (E4M3) / 256 (E2M1), 16-byte aligned: the operands are
 * streamed in place.  Anything else is first rewritten by an ingestion pre-pass (one extra pass over that operand)
 * into zero-padded rows along K in the workspace.
 * The workspace (cb200_mx_matmul_workspace_size bytes, 256-byte aligned) receives the scales re-tiled for the tensor
 * core and the ingested operands.
 * Output: bf16 by default; fp32 (what the reference's kernels write) with CB200_MX_OUT_F32 in `flags`.
 */
#define CB200_MX_E4M3 0
#define CB200_MX_E2M1 1
#define CB200_MX_OUT_F32 1u

typedef struct cb200_mx_matmul_args {
    uint32_t m, n, k;
    uint32_t format;              /* CB200_MX_E4M3 / CB200_MX_E2M1 */
    uint32_t layout_a;            /* CB200_ROW_MAJOR ([m][k]) or CB200_COLUMN_MAJOR ([k][m]) */
    uint32_t layout_b;            /* CB200_COLUMN_MAJOR ([n][k]) or CB200_ROW_MAJOR ([k][n]) */
    const void *a;
    const void *b;
    const void *scale_a;          /* E8M0 bytes */
    const void *scale_b;
    void *d;                      /* m x n row-major: bf16, or fp32 with CB200_MX_OUT_F32 */
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t flags;               /* 0 or CB200_MX_OUT_F32 */
} cb200_mx_matmul_args;

CB200_API int cb200_mx_matmul_can_implement(const cb200_mx_matmul_args *args);
CB200_API uint64_t cb200_mx_matmul_workspace_size(const cb200_mx_matmul_args *args);
CB200_API int cb200_mx_matmul(const cb200_mx_matmul_args *args, void *stream);

/*
 * Grouped (slice-M) MX block-scaled matmul: group g owns a run of rows of A and D, its own weight matrix B[g] and
 * that matrix's scales.  Replaces Gemm::Kernel::GroupedMxMatmulSliceMTla::Arguments (example 55:
 * examples/55_ascend950_mx_grouped_matmul_slice_m/mx_grouped_matmul_slice_m.cpp:168-176, 325-357: problemShape,
 * problemCount, ptrGroupList, ptrA, ptrB, ptrMxScaleA, ptrMxScaleB, ptrC), golden
 * tests/optest/tests/mx_golden.py:325-378.
 *   a        [m][k] elements, rows along K (E2M1 two per byte)          scale_a [m][KS]
 *   b        CB200_COLUMN_MAJOR: [G][n][k];  CB200_ROW_MAJOR: [G][k][n]   scale_b [G][n][KS] / [G][KS/2][n][2]
 *   group_list  `group_count` entries on the device, int64 or int32: the groups' row counts (the reference's
 *            example passes sizes, not prefix sums) or ascending prefix sums, as group_list_kind says; rows past
 *            the last group are not written, entries are clamped to m
 * Arbitrary k, ingestion and output type as for cb200_mx_matmul; the workspace also holds the row-tile table a
 * small planning kernel derives from the group list.
 */
#define CB200_GROUP_LIST_SIZES 0
#define CB200_GROUP_LIST_PREFIX_SUMS 1
typedef struct cb200_mx_grouped_matmul_args {
    uint32_t m, n, k;
    uint32_t group_count;         /* 1 .. 1024 */
    uint32_t format;              /* CB200_MX_E4M3 / CB200_MX_E2M1 */
    uint32_t layout_b;            /* CB200_COLUMN_MAJOR ([G][n][k]) or CB200_ROW_MAJOR ([G][k][n]) */
    uint32_t group_list_type;     /* CB200_GROUP_LIST_INT64 / _INT32 */
    uint32_t group_list_kind;     /* CB200_GROUP_LIST_SIZES / CB200_GROUP_LIST_PREFIX_SUMS */
    const void *a;
    const void *b;
    const void *group_list;
    const void *scale_a;
    const void *scale_b;
    void *d;                      /* m x n row-major: bf16, or fp32 with CB200_MX_OUT_F32 */
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t flags;               /* 0 or CB200_MX_OUT_F32 */
} cb200_mx_grouped_matmul_args;

CB200_API int cb200_mx_grouped_matmul_slice_m_can_implement(const cb200_mx_grouped_matmul_args *args);
CB200_API uint64_t cb200_mx_grouped_matmul_slice_m_workspace_size(const cb200_mx_grouped_matmul_args *args);
CB200_API int cb200_mx_grouped_matmul_slice_m(const cb200_mx_grouped_matmul_args *args, void *stream);

/*
 * Grouped (slice-M) MXFP8 matmul with the SwiGLU + MX quantisation epilogue fused in: the first half of an MoE
 * expert MLP that feeds the second half's MX matmul directly.  Replaces
 * Gemm::Kernel::GroupedMxMatmulSliceMSwigluMxQuantTla::Arguments with Epilogue::BlockEpilogueSwigluMxQuant
 * (include/catlass/gemm/kernel/grouped_mx_matmul_slice_m_swiglu_mx_quant_tla.hpp:72-162,
 * experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant/fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant.cpp:196-227;
 * reserved optest entry tests/optest/include/catlass_kernel_jit.h:477), golden compare.py:31-121 of that example:
 *     C          = (scale_a * A) @ (scale_b * B[g])          fp32, never written
 *     act, gate  = C[:, :n/2], C[:, n/2:]
 *     S          = bf16_rne( act / (1 + exp(-act)) * gate )   each step in fp32
 *     Q, q_scale = MX quantisation of S along n: per 32 columns scale = 2^(largest bf16 exponent of the block - 8)
 *                  (at least 2^-127 ... the block's exponent floor is 8), Q = e4m3_rne_sat(bf16(S / scale));
 *                  scale byte 0 for an all-zero block, 0xFF (and NaN codes) for a block holding Inf or NaN
 *   a, b, scales, group_list: as for cb200_mx_grouped_matmul_slice_m with format E4M3
 *   q        [m][n/2] E4M3 bytes, 16-byte aligned            q_scale  [m][n/64] E8M0 bytes
 * n must be a multiple of 256 here (the reference asks for 128): a tile pairs 128 columns of either half of C.
 * Rows past the last group are not written.
 */
typedef struct cb200_mx_grouped_swiglu_quant_args {
    uint32_t m, n, k;
    uint32_t group_count;         /* 1 .. 1024 */
    uint32_t layout_b;            /* CB200_COLUMN_MAJOR ([G][n][k]) or CB200_ROW_MAJOR ([G][k][n]) */
    uint32_t group_list_type;     /* CB200_GROUP_LIST_INT64 / _INT32 */
    uint32_t group_list_kind;     /* CB200_GROUP_LIST_SIZES / CB200_GROUP_LIST_PREFIX_SUMS */
    uint32_t flags;               /* 0 */
    const void *a;
    const void *b;
    const void *group_list;
    const void *scale_a;
    const void *scale_b;
    void *q;
    void *q_scale;
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t reserved;
} cb200_mx_grouped_swiglu_quant_args;

CB200_API int cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_can_implement(
    const cb200_mx_grouped_swiglu_quant_args *args);
CB200_API uint64_t cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant_workspace_size(
    const cb200_mx_grouped_swiglu_quant_args *args);
CB200_API int cb200_mx_grouped_matmul_slice_m_swiglu_mx_quant(const cb200_mx_grouped_swiglu_quant_args *args,
                                                              void *stream);

/*
 * Grouped (slice-M) MXFP8 matmul with the MoE finalize-routing epilogue fused in: the second half of an expert
 * MLP, which adds every routed row, weighted, into its token's output row.  Replaces
 * Gemm::Kernel::GroupedMxMatmulFinalizeRoutingNoDeterTla::Arguments with
 * Epilogue::BlockEpilogueFinalizeRoutingNoDeter
 * (include/catlass/gemm/kernel/grouped_mx_matmul_finalize_routing_no_deter_tla.hpp,
 * experimental/gmm/ascend950_fp8_mx_grouped_matmul_finalize_routing/fp8_mx_grouped_matmul_finalize_routing_no_deter.cpp;
 * optest parameters tests/optest/include/catlass_kernel_jit.h:489-495), golden gen_data_compare.py:718-757 of
 * that example:
 *     out                          = 0                                        [batch][n] fp32
 *     out[offset : offset+rows]   += shared_weight * float(shared_input)      (when shared_input != NULL)
 *     out[row_index[p]]           += logit[p] * (C[p] + float(bias[group of p]))     for every row p of a group
 * with C = (scale_a * A) @ (scale_b * B[g]) in fp32, never written.  Rows whose row_index is outside [0, batch)
 * are dropped.  By default the additions into an output row happen in the order tiles finish (vector atomics): as
 * in the reference's kernel of this name, results are not bit-reproducible from run to run.  With
 * CB200_ROUTING_DETERMINISTIC in flags (the reference's GroupedMxMatmulFinalizeRoutingTla,
 * include/catlass/gemm/kernel/grouped_mx_matmul_finalize_routing_tla.hpp) C goes to the workspace in fp32 (m x n x 4
 * more bytes) and every output row is summed in ascending row order, the order of the golden's index_add_: the same
 * bits on every run.  The call overwrites all of out.
 *   logit [m] fp32; row_index [m] int64 or int32 (row_index_type: CB200_GROUP_LIST_INT64 / _INT32);
 *   bias [group_count][n] bf16 or NULL; shared_input [shared_rows][n] bf16 or NULL.
 */
#define CB200_ROUTING_DETERMINISTIC 1u
typedef struct cb200_mx_grouped_finalize_routing_args {
    uint32_t m, n, k;
    uint32_t group_count;         /* 1 .. 1024 */
    uint32_t layout_b;            /* CB200_COLUMN_MAJOR ([G][n][k]) or CB200_ROW_MAJOR ([G][k][n]) */
    uint32_t group_list_type;     /* CB200_GROUP_LIST_INT64 / _INT32 */
    uint32_t group_list_kind;     /* CB200_GROUP_LIST_SIZES / CB200_GROUP_LIST_PREFIX_SUMS */
    uint32_t row_index_type;      /* CB200_GROUP_LIST_INT64 / _INT32 */
    uint32_t batch;               /* rows of out */
    uint32_t shared_rows;         /* rows of shared_input (the reference's bsdp) */
    uint32_t shared_offset;       /* first row of out the shared input is added to */
    float shared_weight;
    const void *a;
    const void *b;
    const void *group_list;
    const void *scale_a;
    const void *scale_b;
    const void *logit;
    const void *row_index;
    const void *bias;
    const void *shared_input;
    void *out;
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t block_num;
    uint32_t flags;               /* 0 or CB200_ROUTING_DETERMINISTIC */
} cb200_mx_grouped_finalize_routing_args;

CB200_API int cb200_mx_grouped_matmul_finalize_routing_can_implement(
    const cb200_mx_grouped_finalize_routing_args *args);
CB200_API uint64_t cb200_mx_grouped_matmul_finalize_routing_workspace_size(
    const cb200_mx_grouped_finalize_routing_args *args);
CB200_API int cb200_mx_grouped_matmul_finalize_routing(const cb200_mx_grouped_finalize_routing_args *args,
                                                       void *stream);

/*
 * cb200_mx_matmul_static: the MX matmul above for callers that cannot give it a workspace.
 * (No counterpart in the reference: every reference kernel takes its workspace from the caller or allocates
 * it per call, examples/shared_lib/src/common/common.hpp:36-46.)
 *
 * Some hosts of this library never get to call cudaMalloc: an inference server that hands all of HBM to its
 * own arena at start-up and forbids plug-ins to allocate behind its back, or a latency-critical loop that
 * cannot afford the device-wide synchronisation an allocation implies.  For them the re-tiled scale factors
 * go into a buffer that is part of the library image itself: a file-scope __device__ array of
 * cb200_mx_matmul_static_scratch_bytes() bytes (8 MiB), resident on every GPU that loads the library until
 * the process exits.  args->workspace and args->workspace_bytes are ignored; inputs and output are passed
 * as usual.  The call allocates nothing and calls no allocating routine.
 *
 *  - Limit: cb200_mx_matmul_workspace_size(args) bytes must fit the array: (ceil(m/128) + 2*ceil(n/256)) *
 *    (k/128) * 512 bytes on the fast path (m = n = k = 8192 needs 4 MiB), plus the ingested operands off it.
 *    Larger problems return CB200_SCRATCH_TOO_SMALL and launch nothing.
 *  - The first call on a device looks up the array's device address (with that device current) and keeps it;
 *    make that first call outside any stream capture.
 *  - All calls on a device share the one array.  Each call rewrites every byte of it that it later reads, so
 *    nothing has to be cleared between calls, but two calls that overlap on the GPU (different streams)
 *    race on it: serialise them.
 */
CB200_API int cb200_mx_matmul_static(const cb200_mx_matmul_args *args, void *stream);
CB200_API uint64_t cb200_mx_matmul_static_scratch_bytes(void);

/*
 * MX quantisation of activations on the device: x (fp32 or bf16, rows x k, row pitch x_pitch elements) ->
 * element codes q and E8M0 scales in exactly the form cb200_mx_matmul takes for an operand whose rows run along K:
 *     q      [rows][k] bytes (E4M3), or [rows][ceil(k/2)] bytes (E2M1, even index in bits 0-3)
 *     scale  [rows][KS] bytes, KS = ceil(k/32) rounded up to even (padding = 2^0)
 * Rule (the reference's host-side generators, examples/53_ascend950_fp8_mx_matmul/gen_data.py:186-265 and
 * examples/54_ascend950_fp4_mx_matmul/gen_data.py:46-95): per block of 32, exponent = floor(log2(max|x|)) - emax
 * (emax 8 / 2; 0 for an all-zero block), element = x / 2^exponent clamped and snapped to the nearest code, ties to
 * the smaller magnitude.  On the device the reference does this only inside its experimental fused MoE epilogue
 * (experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant); this entry is the stand-alone step
 * in front of the MX matmul.  No workspace.
 */
typedef struct cb200_mx_quantize_args {
    uint32_t rows, k;
    uint32_t format;      /* CB200_MX_E4M3 / CB200_MX_E2M1 */
    uint32_t x_type;      /* CB200_DTYPE_F32 or CB200_DTYPE_BF16 */
    uint64_t x_pitch;     /* elements between rows of x; 0 = k */
    const void *x;
    void *q;
    void *scale;
} cb200_mx_quantize_args;

CB200_API int cb200_mx_quantize_can_implement(const cb200_mx_quantize_args *args);
CB200_API int cb200_mx_quantize(const cb200_mx_quantize_args *args, void *stream);

/*
 * Per-token int8 quantisation of activations on the device: x (fp32 or bf16, rows x k, row pitch x_pitch elements)
 * -> the A operand and the per-token scale of cb200_quant_matmul and the grouped W8A8 entry points:
 *     q      [rows][k] int8 (row pitch k)
 *     scale  [rows] fp32
 * Rule: amax = max |x| over the row; scale = amax / 127; q = clamp(rint(x * (127 / amax)), -127, 127) with one fp32
 * multiply per element and round-half-to-even; an all-zero row gives scale 0 and codes 0.  Inputs are expected to
 * be finite.  The reference has no device kernel for this step (its quantised examples start from int8 data made
 * on the host, examples/12_quant_matmul/gen_data.py); the entry is the stand-alone step in front of the W8A8
 * matmuls, as cb200_mx_quantize is in front of the MX ones.  No workspace.
 * Requirements: k a multiple of 16; x, q and the rows of x (x_pitch) 16-byte aligned.
 */
typedef struct cb200_quantize_int8_args {
    uint32_t rows, k;
    uint32_t x_type;      /* CB200_DTYPE_F32 or CB200_DTYPE_BF16 */
    uint32_t reserved;    /* 0 */
    uint64_t x_pitch;     /* elements between rows of x; 0 = k */
    const void *x;
    void *q;
    void *scale;
} cb200_quantize_int8_args;

CB200_API int cb200_quantize_per_token_int8_can_implement(const cb200_quantize_int8_args *args);
CB200_API int cb200_quantize_per_token_int8(const cb200_quantize_int8_args *args, void *stream);

/* ---- library / device state ---- */

/* Reads and clears the status word kernels of this library write on the current device when a bounded
 * wait expires.  Synchronises the device.  *code = 0 when every kernel ran to completion.  Returns
 * CB200_SUCCESS, CB200_DEVICE_TIMEOUT (when *code != 0) or CB200_CUDA_ERROR. */
CB200_API int cb200_device_status(uint32_t *code);

/* Self-test of the bounded-wait path every kernel of the library uses: launches one tiny kernel in which a
 * thread waits, for at most limit_us microseconds (1 .. 1000000), on a barrier that nothing signals.  The wait
 * gives up, leaves code 0x1F0 in the device status word and the kernel exits normally; cb200_device_status()
 * then returns CB200_DEVICE_TIMEOUT once.  Nothing hangs or faults; the context stays usable. */
CB200_API int cb200_selftest_wait_timeout(uint32_t limit_us, void *stream);

/* Last CUDA error code (cudaError_t / CUresult as int) seen by this thread inside the library. */
CB200_API int cb200_last_cuda_error(void);

/* Number of kernels this library has launched from the calling process (all threads). */
CB200_API uint64_t cb200_launch_count(void);

CB200_API const char *cb200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CATLASS_B200_H */
