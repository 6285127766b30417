// Hand-written PTX wrappers for sm_100a: mbarrier, async copies, proxy fences
// and the tcgen05 family (TMEM allocation, UMMA issue/commit, TMEM loads).
// They replace the reference's Ampere-era wrappers -- cp.async in
// csrc/AsyncCopy_PTX.cuh:15-78 and ldmatrix / mma.sync in
// csrc/MMA_PTX.cuh:15-210 -- for the Blackwell execution model.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace spmm_b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("{\n\t.reg .b64 state;\n\tmbarrier.arrive.shared::cta.b64 state, [%0];\n\t}" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("{\n\t.reg .b64 state;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 state, [%0], %1;\n\t}" ::"r"(bar),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}

// try_wait that lets the hardware park the thread for up to `suspend_ns` while the phase is
// pending, so that a waiting warp does not compete for issue slots.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t suspend_ns)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity), "r"(suspend_ns)
                 : "memory");
    return done != 0;
}

// Bounded wait.  Each poll may park the thread for up to kSuspendNs; between polls the
// block-wide abort word is checked, and every 256 polls a wall-clock deadline.  Returns
// false if the wait was abandoned, in which case *abort_word has been set so that every
// other role in the block gives up as well.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s
constexpr uint32_t kSuspendNs   = 20000u;

__device__ __forceinline__ bool
mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_word, uint64_t limit_ns = kWaitLimitNs)
{
#ifndef SPMM_B200_PLAIN_POLLS
#define SPMM_B200_PLAIN_POLLS 64
#endif
    // plain polls first: a parked thread wakes up noticeably later than a polling one
#pragma unroll 1
    for (int i = 0; i < SPMM_B200_PLAIN_POLLS; i++)
        if (mbar_try_wait(bar, parity))
            return true;
    uint64_t start = 0;
#pragma unroll 1
    for (uint32_t polls = 0;; polls++) {
        if (mbar_try_wait_suspend(bar, parity, kSuspendNs))
            return true;
        if (*abort_word != 0)
            return false;
        if ((polls & 255u) == 0) {
            const uint64_t now = global_timer_ns();
            if (start == 0)
                start = now;
            else if (now - start > limit_ns) {
                *abort_word = 1;
                return false;
            }
        }
    }
}

// Waits, for at most limit_ns, without looking at the abort word: used on the way out of an
// abandoned block to let a bulk copy that is still in flight land before the block exits.
__device__ __forceinline__ bool mbar_wait_quiet(uint32_t bar, uint32_t parity, uint64_t limit_ns)
{
    const uint64_t start = global_timer_ns();
#pragma unroll 1
    for (;;) {
        if (mbar_try_wait_suspend(bar, parity, kSuspendNs))
            return true;
        if (global_timer_ns() - start > limit_ns)
            return false;
    }
}

// Programmatic dependent launch (a kernel launched with the programmatic-stream-serialization
// attribute may start before its predecessor in the stream has finished).  Both are no-ops for a
// kernel launched the ordinary way.
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Blocks until the predecessor grid has completed and its memory operations are visible.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------- copies
// 16-byte asynchronous copy, bypassing L1.
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async_wait_all()
{
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// Bulk (TMA, untiled) global -> shared copy that reports its bytes to an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src),
                 "r"(bytes),
                 "r"(bar)
                 : "memory");
}

// Adds `bytes` to what the barrier's current phase expects from bulk copies, without arriving.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// Tiled TMA load of one box of a 2-D tensor (x = innermost coordinate, in elements; x * element size
// must be a multiple of 16 bytes).  `tensor_map` is the generic address of a CUtensorMap in
// parameter or global memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tensor_map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     dst_smem),
                 "l"(tensor_map),
                 "r"(x),
                 "r"(y),
                 "r"(bar)
                 : "memory");
}

// The same load issued by either block of a pair (a cluster of two): the box lands in the issuing block's
// shared memory, the bytes are counted on an mbarrier of either block (`bar_cluster`: address in the
// cluster's shared window, see map_to_cta), which is how the partner's half of an operand is reported to
// the block that issues the pair's MMAs.  Every block fetches what it stages itself; nothing is broadcast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tensor_map, int x, int y, uint32_t bar_cluster)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     dst_smem),
                 "l"(tensor_map),
                 "r"(x),
                 "r"(y),
                 "r"(bar_cluster)
                 : "memory");
}

// Asks the memory system to bring `bytes` (a multiple of 16, from a 16-byte aligned address) into L2.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Streaming 128-bit load of read-only data that is used exactly once.
__device__ __forceinline__ uint4 ld_stream_128(const uint4* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_shared_zero_128(uint32_t addr)
{
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
}

// Makes generic-proxy shared-memory writes visible to the async proxy (UMMA operand reads).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, one CTA.  `accumulate` = 0 overwrites D.
__device__ __forceinline__ void
umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc),
                 "l"(b_desc),
                 "r"(idesc),
                 "r"(accumulate),
                 "r"(0u)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with A stored 2:4-compressed (two of every four k values) and
// the selector metadata of the 128 x 32 logical A operand in TMEM.  `e_tmem` is the even column of a
// pair; the instruction descriptor carries the sparse flag and, in its two lowest bits, which column
// of the pair to use (make_idesc_f16_f32(...) | kIdescSparse | column & 1).
__device__ __forceinline__ void
umma_f16_sp_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t e_tmem, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %5, 0;\n\t"
                 "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], %1, %2, [%3], %4, {%6, %6, %6, %6}, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc),
                 "l"(b_desc),
                 "r"(e_tmem),
                 "r"(idesc),
                 "r"(accumulate),
                 "r"(0u)
                 : "memory");
}

// Copies 128 rows x 16 bytes from shared memory (described by a matrix descriptor) to TMEM lanes
// 0..127, four 32-bit columns starting at `taddr`.  Ordered with the MMAs the same thread issues.
__device__ __forceinline__ void tmem_cp_128x128b(uint32_t taddr, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// Arrives on the mbarrier once every UMMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------- pairs of SMs (a cluster of two blocks)
// tcgen05 with .cta_group::2: one thread of the even block of the pair issues MMAs that use the tensor
// cores, shared memory and TMEM of both blocks (M = 256: each block holds 128 rows of A and of the
// accumulator, and half of the columns of B).
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// The address, in the cluster's shared window, of the same shared-memory location in block `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr_cta, uint32_t rank)
{
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr_cta), "r"(rank));
    return out;
}

// Arrives on an mbarrier anywhere in the cluster (address from map_to_cta); what this thread observed
// or wrote before is visible to a cluster-scope acquire of the completed phase.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity, uint32_t suspend_ns)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity), "r"(suspend_ns)
                 : "memory");
    return done != 0;
}

// mbar_wait_bounded for a barrier of this block that the other block of the pair arrives on.
__device__ __forceinline__ bool
mbar_wait_bounded_cluster(uint32_t bar, uint32_t parity, volatile int* abort_word, uint64_t limit_ns = kWaitLimitNs)
{
    uint64_t start = 0;
#pragma unroll 1
    for (uint32_t polls = 0;; polls++) {
        if (mbar_try_wait_cluster(bar, parity, polls < SPMM_B200_PLAIN_POLLS ? 0u : kSuspendNs))
            return true;
        if (*abort_word != 0)
            return false;
        if ((polls & 255u) == 255u) {
            const uint64_t now = global_timer_ns();
            if (start == 0)
                start = now;
            else if (now - start > limit_ns) {
                *abort_word = 1;
                return false;
            }
        }
    }
}

// Barrier over all threads of the cluster (both blocks): every thread arrives, every thread waits.
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_smem, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

// D[tmem of both blocks] (+)= A[shared memory of both blocks] * B[shared memory of both blocks]: the
// descriptors give the offsets of each block's part, the same in both blocks.
__device__ __forceinline__ void
umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc),
                 "l"(b_desc),
                 "r"(idesc),
                 "r"(accumulate)
                 : "memory");
}

// Arrives on an mbarrier of either block of the pair (address in the cluster's shared window) once
// every pair MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Each thread of the warp reads 8 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]),
                   "=r"(r[1]),
                   "=r"(r[2]),
                   "=r"(r[3]),
                   "=r"(r[4]),
                   "=r"(r[5]),
                   "=r"(r[6]),
                   "=r"(r[7]),
                   "=r"(r[8]),
                   "=r"(r[9]),
                   "=r"(r[10]),
                   "=r"(r[11]),
                   "=r"(r[12]),
                   "=r"(r[13]),
                   "=r"(r[14]),
                   "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor (64 bit): start address, leading / stride
// byte offsets (all >> 4), descriptor version 1, swizzle mode in bits 61..63.
constexpr uint64_t kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;

__device__ __forceinline__ uint64_t
make_smem_desc(uint32_t smem_byte_addr, uint32_t leading_bytes, uint32_t stride_bytes, uint64_t swizzle)
{
    return static_cast<uint64_t>((smem_byte_addr >> 4) & 0x3fffu) | (static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16)
           | (static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (swizzle << 61);
}

// Instruction descriptor for kind::f16 with fp16 A and B and an fp32 accumulator.
// a_mn_major / b_mn_major: operand stored with its M (resp. N) index contiguous.
__host__ __device__ constexpr uint32_t make_idesc_f16_f32(int m, int n, bool a_mn_major, bool b_mn_major)
{
    return (1u << 4)                                   // accumulator format: f32
           | (0u << 7) | (0u << 10)                    // A, B formats: f16
           | (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16)
           | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

constexpr uint32_t kIdescSparse = 1u << 2;  // A is 2:4-compressed, metadata in TMEM

}  // namespace ptx
}  // namespace spmm_b200
