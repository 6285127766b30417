// Sum of the ranks' partial results of a row-parallel (split by K) SpMM, read straight out of the
// peers' memory over NVLink: one kernel per rank, no library collective.
//
// The reference is single-GPU; its weight-conversion tool splits out-proj and FFN2 by K
// (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:134-135) and leaves the sum to
// FasterTransformer's NCCL all-reduce.  For the 0.3 MB results of decode-size layers that all-reduce
// is latency-bound (15-30 us against a 76 us SpMM); here every rank
//   1. tells every peer that its partial result is complete (one 32-bit flag per peer, written into
//      the peer's memory after a system-scope fence),
//   2. waits until all peers have told it the same (bounded spin on its own flags),
//   3. adds the g partial results element by element in rank order (16-byte loads from the peers'
//      buffers, fp32 sums, one rounding) and writes the sum to a local output.
// Flags carry the call's epoch, which only grows, so nothing is reset; the callers alternate between
// two result buffers, so a fast rank's next SpMM never overwrites what a slow peer is still reading
// (a rank reaches the flag exchange of call n + 1 only after its reads of call n have finished).
// The epoch comes from the host, or -- so that the call can be captured in a CUDA graph and replayed --
// from a counter in device memory that the last block of every launch advances.
//
// The buffers and flag arrays are symmetric allocations mapped into every rank's address space by
// the caller (torch.distributed._symmetric_memory in the Python mirror); this file only takes
// pointers.  One process per GPU; the ranks must not share a GPU (each waits for the others).
#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/spmm_b200.h"
#include "ptx_sm100.cuh"

namespace spmm_b200 {

__device__ int g_device_status_allreduce;  // 1 after a wait for the peers ran out

constexpr int kMaxRanks = 16;

struct AllReduceParams {
    const uint4* partial[kMaxRanks];  // every rank's partial result, count halves (or floats) each
    const uint4* partial_odd[kMaxRanks];  // fp32 form: the buffers used by calls of odd epoch (partial: even)
    uint32_t*    flags[kMaxRanks];    // flags[p] = rank p's flag array (world entries, one per sender)
    uint4*       out;                 // local result
    size_t       vectors;             // count / 8
    int          rank, world;
    uint32_t     epoch;               // this call's epoch when `state` is null
    uint32_t*    state;               // or: state[0] = epoch of the previous call, state[1] = blocks finished
    int          announced;           // 1: the kernel that wrote the partial result has told the peers already
    unsigned long long limit_ns;
};

// F32: the partial results are fp32 (two 16-byte vectors per eight outputs) and lie in the buffer set of the
// call's epoch parity; they are rounded to fp16 once, after the sum.
template<bool F32>
__global__ void __launch_bounds__(256) allreduce_partials_kernel(const __grid_constant__ AllReduceParams p)
{
    __shared__ int ok;
    ptx::grid_dependency_wait();  // the SpMM before this kernel in the stream wrote this rank's partial result
    if (threadIdx.x == 0)
        ok = 1;
    uint32_t epoch = p.epoch;
    if (p.state != nullptr) {
        // every earlier launch that used this state has completed (stream order), so the counter is stable
        uint32_t previous;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(previous) : "l"(p.state) : "memory");
        epoch = previous + 1;
    }
    if (blockIdx.x == 0 && threadIdx.x < p.world && !p.announced) {
        // this rank's partial result is complete and visible: tell peer threadIdx.x
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[threadIdx.x] + p.rank), "r"(epoch) : "memory");
    }
    __syncthreads();
    if (threadIdx.x < p.world) {
        const uint32_t*          mine  = p.flags[p.rank] + threadIdx.x;
        const unsigned long long start = ptx::global_timer_ns();
        for (unsigned polls = 0;; polls++) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if (static_cast<int32_t>(seen - epoch) >= 0)
                break;
            if ((polls & 255u) == 255u && ptx::global_timer_ns() - start > p.limit_ns) {
                ok = 0;  // a peer never arrived: give up, report, leave the output untouched
                atomicExch(&g_device_status_allreduce, 1);
                break;
            }
        }
    }
    __syncthreads();
    const uint4* const* partial = (F32 && (epoch & 1u)) ? p.partial_odd : p.partial;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; ok && i < p.vectors;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (F32) {
            // all ranks' loads first, then the sums in rank order: one NVLink round trip per eight outputs
            float4 v[kMaxRanks][2];
#pragma unroll
            for (int r = 0; r < kMaxRanks; r++)
                if (r < p.world) {
                    const float4* src = reinterpret_cast<const float4*>(partial[r]) + 2 * i;
                    v[r][0]           = __ldcv(src);
                    v[r][1]           = __ldcv(src + 1);
                }
#pragma unroll
            for (int r = 0; r < kMaxRanks; r++)
                if (r < p.world) {
                    sum[0] += v[r][0].x, sum[1] += v[r][0].y, sum[2] += v[r][0].z, sum[3] += v[r][0].w;
                    sum[4] += v[r][1].x, sum[5] += v[r][1].y, sum[6] += v[r][1].z, sum[7] += v[r][1].w;
                }
        }
        else {
            for (int r = 0; r < p.world; r++) {
                const uint4    v = __ldcv(partial[r] + i);  // peer memory, rewritten every other call: never from a cache
                const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float2 f = __half22float2(h[k]);
                    sum[2 * k] += f.x;
                    sum[2 * k + 1] += f.y;
                }
            }
        }
        uint4    o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int k = 0; k < 4; k++)
            oh[k] = __floats2half2_rn(sum[2 * k], sum[2 * k + 1]);
        p.out[i] = o;
    }
    if (p.state != nullptr) {
        // the last block to get here advances the epoch for the next launch
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(p.state + 1, 1u) == gridDim.x - 1) {
                p.state[1] = 0;
                __threadfence();
                p.state[0] = epoch;
            }
        }
    }
}


// Two-phase form for larger worlds (reduce-scatter, then all-gather by remote stores): every rank adds only
// its own 1 / world of the outputs out of all ranks' fp32 partial results and writes the rounded slice into
// every rank's result buffer; a second flag exchange tells the peers that the slice has arrived.  Against
// the one-phase form, which pulls all ranks' complete partial results into every rank (world * count * 4
// bytes over NVLink per rank), a rank reads count * 4 bytes and writes count * 2: at eight ranks 4.1 MB
// become 0.7 MB per sum, for one more flag round trip.  Flags: entries [0, world) of a rank's flag array are
// "partial result of sender s is complete", entries [world, 2 world) "sender s has written its slice here".
struct TwoPhaseParams {
    const float4* partial[2][kMaxRanks];  // [epoch parity][rank]: fp32 partial results, count floats each
    uint32_t*     flags[kMaxRanks];       // 2 * world words per rank
    uint4*        out[kMaxRanks];         // every rank's result buffer (count halves), mapped here
    size_t        slice_vectors;          // count / 8 / world: outputs this rank sums, in vectors of eight
    int           rank, world;
    uint32_t*     state;                  // [0] epoch of the previous call, [1] blocks finished
    unsigned long long limit_ns;
};

__global__ void __launch_bounds__(256) allreduce_two_phase_kernel(const __grid_constant__ TwoPhaseParams p)
{
    __shared__ int ok, last;
    ptx::grid_dependency_wait();  // the SpMM before this kernel in the stream wrote this rank's partial result
    if (threadIdx.x == 0) {
        ok   = 1;
        last = 0;
    }
    uint32_t previous;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(previous) : "l"(p.state) : "memory");
    const uint32_t epoch = previous + 1;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[threadIdx.x] + p.rank), "r"(epoch) : "memory");
    }
    __syncthreads();
    // bounded wait for `count` flags of this rank's array, starting at entry `first`
    auto wait_flags = [&](int first) {
        if (threadIdx.x < p.world) {
            const uint32_t*          mine  = p.flags[p.rank] + first + threadIdx.x;
            const unsigned long long start = ptx::global_timer_ns();
            for (unsigned polls = 0;; polls++) {
                uint32_t seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
                if (static_cast<int32_t>(seen - epoch) >= 0)
                    break;
                if ((polls & 255u) == 255u && ptx::global_timer_ns() - start > p.limit_ns) {
                    ok = 0;  // a peer never arrived: give up and report
                    atomicExch(&g_device_status_allreduce, 1);
                    break;
                }
            }
        }
        __syncthreads();
    };
    wait_flags(0);
    const float4* const* partial = p.partial[epoch & 1u];
    const size_t         begin   = p.slice_vectors * p.rank;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; ok && i < p.slice_vectors;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        // all ranks' loads first, then the sums in rank order: one NVLink round trip
        float4 v[kMaxRanks][2];
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if (r < p.world) {
                const float4* src = partial[r] + 2 * (begin + i);
                v[r][0]           = __ldcv(src);
                v[r][1]           = __ldcv(src + 1);
            }
        float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if (r < p.world) {
                sum[0] += v[r][0].x, sum[1] += v[r][0].y, sum[2] += v[r][0].z, sum[3] += v[r][0].w;
                sum[4] += v[r][1].x, sum[5] += v[r][1].y, sum[6] += v[r][1].z, sum[7] += v[r][1].w;
            }
        uint4    o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int k = 0; k < 4; k++)
            oh[k] = __floats2half2_rn(sum[2 * k], sum[2 * k + 1]);
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if (r < p.world)
                p.out[r][begin + i] = o;  // every rank gets the same bits
    }
    // The last block of this rank to finish tells every peer that the slice has arrived (the block's stores are
    // ordered before thread 0's system-scope fence by the barrier), then waits for the peers' slices: when
    // this kernel completes, this rank's result buffer is complete.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(p.state + 1, 1u) == gridDim.x - 1) {
            p.state[1] = 0;
            last       = 1;
        }
    }
    __syncthreads();
    if (last) {
        if (threadIdx.x < p.world)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[threadIdx.x] + p.world + p.rank), "r"(epoch) : "memory");
        wait_flags(p.world);
        if (threadIdx.x == 0) {
            __threadfence();
            p.state[0] = epoch;
        }
    }
}

}  // namespace spmm_b200

namespace spmm_b200 {
namespace {
int launch_allreduce(void* stream, const void* const* partial_buffers, void* const* flag_arrays, int rank, int world, void* out,
                     size_t count, uint32_t epoch, uint32_t* state, unsigned limit_ms, bool f32 = false, bool announced = false)
{
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || count % 8 != 0 || !out || !partial_buffers
        || !flag_arrays || (epoch == 0 && state == nullptr) || (f32 && state == nullptr))
        return static_cast<int>(cudaErrorInvalidValue);
    AllReduceParams p;
    for (int r = 0; r < world; r++) {
        if (!partial_buffers[r] || !flag_arrays[r] || (reinterpret_cast<uintptr_t>(partial_buffers[r]) & 15u))
            return static_cast<int>(cudaErrorInvalidValue);
        p.partial[r]     = static_cast<const uint4*>(partial_buffers[r]);
        p.partial_odd[r] = p.partial[r];
        if (f32) {  // two buffer sets, parity-major: [parity * world + rank]
            if (!partial_buffers[world + r] || (reinterpret_cast<uintptr_t>(partial_buffers[world + r]) & 15u))
                return static_cast<int>(cudaErrorInvalidValue);
            p.partial_odd[r] = static_cast<const uint4*>(partial_buffers[world + r]);
        }
        p.flags[r] = static_cast<uint32_t*>(flag_arrays[r]);
    }
    if (reinterpret_cast<uintptr_t>(out) & 15u)
        return static_cast<int>(cudaErrorInvalidValue);
    p.out      = static_cast<uint4*>(out);
    p.vectors  = count / 8;
    p.rank     = rank;
    p.world    = world;
    p.epoch    = epoch;
    p.state     = state;
    p.announced = announced ? 1 : 0;
    p.limit_ns = static_cast<unsigned long long>(limit_ms ? limit_ms : 2000u) * 1000000ull;
    const int blocks = static_cast<int>(p.vectors < 256 * 148 ? (p.vectors + 255) / 256 : 148);
    cudaLaunchConfig_t config = {};
    config.gridDim            = dim3(blocks > 0 ? blocks : 1);
    config.blockDim           = dim3(256);
    config.stream             = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                       = attr;
    config.numAttrs                                    = 1;
    cudaError_t e = f32 ? cudaLaunchKernelEx(&config, allreduce_partials_kernel<true>, p)
                        : cudaLaunchKernelEx(&config, allreduce_partials_kernel<false>, p);
    return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}
}  // namespace
}  // namespace spmm_b200

extern "C" int spmm_b200_allreduce_partials(void*              stream,
                                            const void* const* partial_buffers,
                                            void* const*       flag_arrays,
                                            int                rank,
                                            int                world,
                                            void*              out,
                                            size_t             count,
                                            uint32_t           epoch,
                                            unsigned           limit_ms)
{
    return spmm_b200::launch_allreduce(stream, partial_buffers, flag_arrays, rank, world, out, count, epoch, nullptr, limit_ms);
}

extern "C" int spmm_b200_allreduce_partials_replayable(void*              stream,
                                                       const void* const* partial_buffers,
                                                       void* const*       flag_arrays,
                                                       int                rank,
                                                       int                world,
                                                       void*              out,
                                                       size_t             count,
                                                       void*              state,
                                                       unsigned           limit_ms)
{
    if (state == nullptr || (reinterpret_cast<uintptr_t>(state) & 3u))
        return static_cast<int>(cudaErrorInvalidValue);
    return spmm_b200::launch_allreduce(stream, partial_buffers, flag_arrays, rank, world, out, count, 0,
                                       static_cast<uint32_t*>(state), limit_ms);
}

extern "C" int spmm_b200_allreduce_status(int reset)
{
    int         status = 0;
    cudaError_t e      = cudaDeviceSynchronize();
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    e = cudaMemcpyFromSymbol(&status, spmm_b200::g_device_status_allreduce, sizeof(int));
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    if (reset) {
        const int zero = 0;
        cudaMemcpyToSymbol(spmm_b200::g_device_status_allreduce, &zero, sizeof(int));
    }
    return status;
}

extern "C" int spmm_b200_allreduce_partials_f32(void*              stream,
                                                const void* const* partial_buffers,
                                                void* const*       flag_arrays,
                                                int                rank,
                                                int                world,
                                                void*              out,
                                                size_t             count,
                                                void*              state,
                                                unsigned           limit_ms)
{
    if (state == nullptr || (reinterpret_cast<uintptr_t>(state) & 3u))
        return static_cast<int>(cudaErrorInvalidValue);
    return spmm_b200::launch_allreduce(stream, partial_buffers, flag_arrays, rank, world, out, count, 0,
                                       static_cast<uint32_t*>(state), limit_ms, true);
}

extern "C" int spmm_b200_allreduce_partials_f32_announced(void*              stream,
                                                          const void* const* partial_buffers,
                                                          void* const*       flag_arrays,
                                                          int                rank,
                                                          int                world,
                                                          void*              out,
                                                          size_t             count,
                                                          void*              state,
                                                          unsigned           limit_ms)
{
    if (state == nullptr || (reinterpret_cast<uintptr_t>(state) & 3u))
        return static_cast<int>(cudaErrorInvalidValue);
    return spmm_b200::launch_allreduce(stream, partial_buffers, flag_arrays, rank, world, out, count, 0,
                                       static_cast<uint32_t*>(state), limit_ms, true, true);
}

extern "C" int spmm_b200_allreduce_partials_f32_two_phase(void*              stream,
                                                          const void* const* partial_buffers,
                                                          void* const*       flag_arrays,
                                                          void* const*       out_buffers,
                                                          int                rank,
                                                          int                world,
                                                          size_t             count,
                                                          void*              state,
                                                          unsigned           limit_ms)
{
    using namespace spmm_b200;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || count == 0 || count % (8 * static_cast<size_t>(world)) != 0
        || !partial_buffers || !flag_arrays || !out_buffers || !state || (reinterpret_cast<uintptr_t>(state) & 3u))
        return static_cast<int>(cudaErrorInvalidValue);
    TwoPhaseParams p;
    for (int r = 0; r < world; r++) {
        for (int parity = 0; parity < 2; parity++) {
            const void* buffer = partial_buffers[parity * world + r];
            if (!buffer || (reinterpret_cast<uintptr_t>(buffer) & 15u))
                return static_cast<int>(cudaErrorInvalidValue);
            p.partial[parity][r] = static_cast<const float4*>(buffer);
        }
        if (!flag_arrays[r] || !out_buffers[r] || (reinterpret_cast<uintptr_t>(out_buffers[r]) & 15u))
            return static_cast<int>(cudaErrorInvalidValue);
        p.flags[r] = static_cast<uint32_t*>(flag_arrays[r]);
        p.out[r]   = static_cast<uint4*>(out_buffers[r]);
    }
    p.slice_vectors = count / 8 / world;
    p.rank          = rank;
    p.world         = world;
    p.state         = static_cast<uint32_t*>(state);
    p.limit_ns      = static_cast<unsigned long long>(limit_ms ? limit_ms : 2000u) * 1000000ull;
    const int blocks = static_cast<int>(p.slice_vectors < 256 * 148 ? (p.slice_vectors + 255) / 256 : 148);
    cudaLaunchConfig_t config = {};
    config.gridDim            = dim3(blocks > 0 ? blocks : 1);
    config.blockDim           = dim3(256);
    config.stream             = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                       = attr;
    config.numAttrs                                    = 1;
    cudaError_t e = cudaLaunchKernelEx(&config, allreduce_two_phase_kernel, p);
    return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}
