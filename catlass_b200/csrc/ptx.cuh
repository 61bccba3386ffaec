// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA (cp.async.bulk.tensor),
// tcgen05 (UMMA issue, TMEM allocation and loads) and the proxy/thread-sync fences between them.
// Every wait on an mbarrier is bounded: see mbar_wait().
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cb200 {

// ---- status codes written to the device status word by a kernel that gave up on a wait ----
// (the value also says which role of the pipeline waited)
constexpr unsigned kDevOk = 0;
constexpr unsigned kDevTimeoutProducer = 0x101;  // TMA producer waiting for a free smem stage
constexpr unsigned kDevTimeoutMma = 0x102;       // MMA issuer waiting for operands
constexpr unsigned kDevTimeoutMmaTmem = 0x103;   // MMA issuer waiting for a drained accumulator
constexpr unsigned kDevTimeoutEpilogue = 0x104;  // epilogue waiting for a finished accumulator
constexpr unsigned kDevTimeoutConvert = 0x105;   // operand converter warps (W4A8) waiting
constexpr unsigned kDevTimeoutPeerCta = 0x106;   // a CTA of a pair waiting for its peer
constexpr unsigned kDevTimeoutSelfTest = 0x1F0;  // the wait self-test (a barrier nothing arrives on)

// Upper bound for any single wait.  Far above every legitimate wait (the longest kernel here runs a few
// milliseconds), so it only fires when the pipeline is broken; copies still in flight have landed by then.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on the barrier at the same smem offset in CTA `cta` of this cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta)
{
    asm volatile(
        "{\n\t"
        ".reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t"
        "}\n" ::"r"(bar),
        "r"(cta)
        : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait that also acquires writes made by other CTAs of the cluster before they arrived on the barrier.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking probe of a barrier phase.  (try_wait may suspend the thread for a hardware-chosen time when the
// phase is not complete; a thread that polls several barriers in turn must not be held up by any one of them.)
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the CTA is being torn down: either this wait exceeded kWaitLimitNs
// (then it records `code` in *status and raises *abort for the other roles) or another role did.
// The caller must leave its loops and fall through to the kernel's common exit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort,
                                          unsigned* status, unsigned code,
                                          unsigned long long limit_ns = kWaitLimitNs)
{
    // The clock is read only after a run of failed probes: a read of the global timer costs far more than a
    // probe, and most waits end within the first few.
    if (mbar_test_wait(bar, parity)) {  // the common case in a pipeline that runs ahead: no suspension involved
        return true;
    }
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    for (;;) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((++spins & 0x3f) == 0) {
            if (*abort != 0) {
                return false;
            }
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort = 1;
                atomicMax(status, code);
                return false;
            }
        }
    }
}

// Bounded wait on a barrier other CTAs of the cluster arrive on (see mbar_wait for the contract).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort,
                                                  unsigned* status, unsigned code,
                                                  unsigned long long limit_ns = kWaitLimitNs)
{
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    for (;;) {
        if (mbar_try_wait_cluster(bar, parity)) {
            return true;
        }
        if ((++spins & 0x3f) == 0) {
            if (*abort != 0) {
                return false;
            }
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort = 1;
                atomicMax(status, code);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------- fences

__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Named barrier among `threads` threads (id 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int32_t x,
                                            int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int32_t x,
                                            int32_t y, int32_t z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
        "[%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Loads for a CTA pair (cta_group::2): data lands in this CTA's smem, the transaction bytes are counted on
// the barrier address given, which may be the peer CTA's barrier (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster,
                                                 int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
        "%4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster,
                                                 int32_t x, int32_t y, int32_t z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
        "%4, %5}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster,
                                                 int32_t x, int32_t y, int32_t z, int32_t w)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
        "%4, %5, %6}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(src), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM

template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t columns)
{
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                     "r"(columns)
                     : "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                     "r"(columns)
                     : "memory");
    }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_relinquish()
{
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
{
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
    } else {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
    }
}

// Shared-memory matrix descriptor of a tile whose rows are 128 bytes wide and 128B-swizzled (the layout a
// TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces; tile base 1024-byte aligned).
//   K-major operand  (rows = M or N index, 128 contiguous bytes of K per row):
//       lbo is not used by the hardware for swizzled K-major tiles (encoded as 1), sbo = bytes between
//       8-row groups (1024 when rows are packed).
//   MN-major operand (rows = K index, 128 contiguous bytes of M or N per row):
//       lbo = bytes between successive 128-byte-wide column panels, sbo = bytes between 8-row groups of K.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;  // descriptor version of the 5th-generation tensor core
    d |= 2ull << 61;  // 128-byte swizzle
    return d;
}

// Descriptor of an unswizzled K-major tile: 8-row x 16-byte core matrices stored contiguously (128 bytes),
// `sbo_bytes` between core matrices along the rows, `lbo_bytes` between core matrices along K.
__device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t smem_addr, uint32_t lbo_bytes,
                                                             uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    return d;
}

// Instruction descriptor of the block-scaled kinds (mxf8f6f4, mxf4) with E8M0 scale factors:
//   bits 4-5 which byte of the B scale column this MMA uses, 7-9 A format, 10-12 B format, 15/16 A/B MN-major,
//   17-22 N/8, 23 scale format (1 = E8M0), 24-28 M/16, 29-30 byte of the A scale column.
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n,
                                                     uint32_t a_sf_id, uint32_t b_sf_id)
{
    return (b_sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) |
           (a_sf_id << 29);
}

// Descriptor of an MN-major tile stored as 32-byte-wide column panels with the 32-byte swizzle (what a TMA
// load with CU_TENSOR_MAP_SWIZZLE_32B produces from a box whose inner extent is 32 bytes): rows = K index,
// 32 contiguous bytes of M or N per row; lbo = bytes between panels, sbo = bytes between 8-row groups of K.
__device__ __forceinline__ uint64_t make_smem_desc_sw32(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    d |= 6ull << 61;  // 32-byte swizzle
    return d;
}

// Instruction descriptor fields (32-bit) shared by the dense kinds.
//   bits 4-5 accumulator format (1 = f32, 2 = s32), 7-9 A format, 10-12 B format, 15 A is MN-major,
//   16 B is MN-major, 17-22 N/8, 24-28 M/16.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, bool a_mn,
                                                  bool b_mn, uint32_t m, uint32_t n)
{
    return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

constexpr uint32_t kFmtS8 = 1;     // signed 8-bit integer operand (kind::i8)
constexpr uint32_t kFmtE4M3 = 0;   // kind::f8f6f4 / mxf8f6f4
constexpr uint32_t kFmtE2M1 = 5;   // 4-bit operand in kind::mxf8f6f4 (unpacked in smem)
constexpr uint32_t kFmtMxf4E2M1 = 1;  // packed 4-bit operand of kind::mxf4
constexpr uint32_t kAccS32 = 2;
constexpr uint32_t kAccF32 = 1;

template <int kCtaGroup>
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate)
{
    if constexpr (kCtaGroup == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Block-scaled MMA: E8M0 scale factors for A and B sit in TMEM at sfa / sfb.
template <bool kFp4>
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate, uint32_t sfa, uint32_t sfb)
{
    if constexpr (kFp4) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
            : "memory");
    }
}

// Make `bar` complete once every MMA this thread issued so far has finished (implies
// tcgen05.fence::before_thread_sync).
template <int kCtaGroup>
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
    } else {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
    }
}

// Same, arriving on the barrier at this offset in every CTA of `cta_mask` (signals only, no data moves).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            bar),
        "h"(cta_mask)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Wait for an earlier tmem_ld_32x32b_x16 into r that was left in flight.  The registers are operands so that no
// use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_wait_x16(uint32_t (&r)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15])
                 :
                 : "memory");
}

// Copy 128-bit x 32 rows from shared memory (described by a no-swizzle descriptor) into the TMEM lanes
// of all four 32-lane quadrants: the form the block-scaled MMA expects its scale factors in.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// No-ops unless the kernel was launched with cudaLaunchAttributeProgrammaticStreamSerialization.
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Blocks until the grids this one depends on have completed and their writes are visible.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------- cluster helpers

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace cb200
