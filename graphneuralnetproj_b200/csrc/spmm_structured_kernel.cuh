// Structured (2:4) half of the heterogeneous SpMM for sm_100a: C = A1 * B with A1 holding at most
// two nonzeros in every aligned group of four along K, multiplied by the sparse tensor-core
// instruction tcgen05.mma.sp straight from its compressed form.
//
// Replaces the structured half of the reference's SpMM_Kernel (csrc/SpMM_Kernel.cuh:293-735:
// value vectors + 64-bit index words restored to a 2:4-compressed tile in shared memory, selector
// metadata in registers, mma.sp.m16n8k16 through csrc/MMA_PTX.cuh:43-86,195-210 and
// csrc/MatMulUtilities.cuh:247-302).  Here nothing is restored on the GPU: the host packer
// (pack_a1_tcgen05.cu) stores every 128 x 128 block of A1 as the exact shared-memory image the
// tensor core reads,
//
//   values   16 KB  128 rows x 64 kept halves, K-major, 128-byte swizzle (chunk ^= row % 8)
//   metadata  2 KB  128 x 16 bytes: entry L = m0 + 8 * h + 16 * g (m0 < 8, h < 2, g < 8) holds four
//                   32-bit words, one per 32-wide k step; a word's low half describes row 16 g + m0,
//                   its high half row 16 g + m0 + 8, k columns 16 h .. 16 h + 15 of the step: four
//                   4-bit codes (index of the first kept element | index of the second << 2),
//
// so a block reaches shared memory with two bulk copies, the metadata goes on to TMEM with one
// tcgen05.cp.128x128b, and four tcgen05.mma.sp (M = 128, K = 32 each) consume the block.  The path is
// bound by the bytes of A1 (1.125 bytes per element of the dense matrix).
//
// One persistent block per SM takes a contiguous chunk of the block sequence (row of blocks after
// row of blocks, as schedule.h partitions it).  Roles by warp:
//   0..3  epilogue, as in spmm_decode_kernel.cuh (fp32 slots + last-arriver reduction for rows of
//         blocks whose K range is shared); the result goes to C as fp16 or, when a residual product
//         follows, to an fp32 array that the residual kernel adds before its single rounding
//   4     MMA issue (one lane), owner of the TMEM allocation
//   5     producer: bulk copies of values and metadata, a ring of STAGES stages
//   6..7  B loaders: 128 x N slice of B[K][N] per block, 16-byte async copies into the
//         N-contiguous swizzled layout, arrival lagging three stages behind the issue
//
// Every wait is bounded as in the decode kernel; a wait that gives up raises the block-wide abort
// word and the status word.
#pragma once

#include <cuda_fp16.h>

#include "ptx_sm100.cuh"
#include "schedule.h"
#include "spmm_decode_kernel.cuh"

namespace spmm_b200 {

constexpr int kBlockK            = 128;                      // logical k extent of a packed A1 block
constexpr int kBlockValueBytes   = kTileRows * kBlockK;      // 128 rows x 64 kept halves
constexpr int kBlockMetaBytes    = kTileRows * 16;
constexpr int kStructuredThreads = 8 * 32;
constexpr int kBLoaderWarps      = 2;
constexpr int kBLag              = 3;  // a B slice is announced this many blocks after its copies were issued

struct StructuredParams {
    const uint4* values = nullptr;  // blocks * 16 KB
    const uint4* meta   = nullptr;  // blocks * 2 KB
    const half*  B      = nullptr;  // [K][ld]
    half*        C      = nullptr;  // [M][ld] fp16 result, used when C32 == nullptr
    float*       C32    = nullptr;  // [M][N] fp32 result for a following residual product, or nullptr
    float*       slots  = nullptr;  // fp32 partial blocks of split rows
    int          n        = 0;
    int          blocks_k = 0;  // K / 128
    int          m        = 0;
    int          ld       = 0;
    int          counter_set   = 0;  // which set of arrival counters this launch uses
    int          weights_early = 0;  // as DecodeParams::weights_early
    Schedule     sched;
};

template<int NB, int STAGES>
constexpr int structured_smem_bytes()
{
    return 1024 + STAGES * (kBlockValueBytes + kBlockMetaBytes + kBlockK * NB * 2) + 512;
}

template<int N, int STAGES>
__global__ void __launch_bounds__(kStructuredThreads, 1) spmm_structured_kernel(const __grid_constant__ StructuredParams p)
{
    constexpr int NB = N < 16 ? 16 : N;
    using BT         = BTile<NB>;
    constexpr int kBBytes = kBlockK * NB * 2;
    static_assert(kBLag < STAGES, "a B slice must be announced before its stage is needed again");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base    = smem_base;
    const uint32_t b_base    = a_base + STAGES * kBlockValueBytes;
    const uint32_t e_base    = b_base + STAGES * kBBytes;
    const uint32_t bar_base  = e_base + STAGES * kBlockMetaBytes;
    // barriers: values+metadata landed, B landed, stage free (x STAGES), accumulator full / free (x 2)
    auto ae_full  = [&](int s) { return bar_base + 8u * s; };
    auto b_full   = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto empty    = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    auto acc_full = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };
    auto acc_free = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 + b); };
    static_assert(8 * (3 * STAGES + 4) + 8 <= 512, "barrier block");
    const uint32_t tmem_slot_addr = bar_base + 8u * (3 * STAGES + 4);
    uint8_t*       smem_generic   = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
    volatile uint32_t* tmem_slot  = reinterpret_cast<volatile uint32_t*>(smem_generic + (tmem_slot_addr - smem_base));
    volatile int*      abort_word = reinterpret_cast<volatile int*>(smem_generic + (tmem_slot_addr + 4 - smem_base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta  = blockIdx.x;

    const int tile_begin = p.sched.chunk_begin[cta];
    const int tile_end   = p.sched.chunk_begin[cta + 1];
    const int num_tiles  = tile_end - tile_begin;
    const int tiles_k    = p.blocks_k;
    // TMEM: two accumulators of NB columns, then four metadata columns per stage
    constexpr uint32_t kTmemCols = tmem_columns(2 * NB + 4 * STAGES);
    static_assert(2 * NB + 4 * STAGES <= 512, "TMEM columns");

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            ptx::mbar_init(ae_full(s), 1);
            ptx::mbar_init(b_full(s), kBLoaderWarps);
            ptx::mbar_init(empty(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            ptx::mbar_init(acc_full(b), 1);
            ptx::mbar_init(acc_free(b), kEpilogueWarps);
        }
        *abort_word = 0;
        ptx::mbar_init_fence();
    }
    // Columns N..NB-1 of the staged B slices (N == 8) are never written: clear the B ring once.
    for (uint32_t off = threadIdx.x * 16u; off < static_cast<uint32_t>(STAGES * kBBytes); off += blockDim.x * 16u)
        ptx::st_shared_zero_128(b_base + off);
    if (warp == kFirstMmaWarp) {
        ptx::tmem_alloc(tmem_slot_addr, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_e    = tmem_base + 2 * NB;
    // Programmatic dependent launch, as in the decode kernel: B, C, the workspace and the arrival counters
    // are touched only after the predecessor grid has finished; the packed weights are requested at
    // once if p.weights_early says they were complete before the predecessor started.
    ptx::grid_launch_dependents();

    if (warp == kFirstMmaWarp + 1) {
        // ------------------------------------------------------------ producer: values and metadata
        // Lane 0 copies the values, lane 1 the metadata, in one instruction: issuing a bulk copy
        // costs the issuing thread a few hundred cycles, and one thread issuing both copies of every
        // block would be close to the time a block may take at full memory bandwidth.
        if (!p.weights_early)
            ptx::grid_dependency_wait();
        if (lane < 2) {
            int            issued = 0;
            const uint32_t bytes  = lane == 0 ? kBlockValueBytes : kBlockMetaBytes;
            const uint32_t dst0   = lane == 0 ? a_base : e_base;
            const uint4*   src0   = lane == 0 ? p.values : p.meta;
#pragma unroll 1
            for (int l = 0; l < num_tiles; l++, issued++) {
                const int s = l % STAGES, u = l / STAGES;
                if (u > 0 && !ptx::mbar_wait_bounded(empty(s), (u - 1) & 1, abort_word))
                    break;
                const size_t t = static_cast<size_t>(tile_begin + l);
                if (lane == 0)
                    ptx::mbar_arrive_expect_tx(ae_full(s), kBlockValueBytes + kBlockMetaBytes);
                ptx::bulk_copy_g2s(dst0 + s * bytes, src0 + t * (bytes / 16), bytes, ae_full(s));
            }
            if (*abort_word != 0) {
                // copies that nobody will wait for any more must land before the block exits
#pragma unroll 1
                for (int l = max(0, issued - STAGES); l < issued; l++)
                    ptx::mbar_wait_quiet(ae_full(l % STAGES), (l / STAGES) & 1, 1000000ull);
            }
        }
    }
    else if (warp > kFirstMmaWarp + 1) {
        // ------------------------------------------------------------ B loaders
        constexpr int kChunksPerRow = N / 8;                 // 16-byte chunks of a row that exist in B
        constexpr int kChunks       = kBlockK * kChunksPerRow;
        constexpr int kLoaders      = kBLoaderWarps * 32;
        const int     loader        = (warp - kFirstMmaWarp - 2) * 32 + lane;
        auto announce = [&](int l) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(b_full(l % STAGES));
        };
        int  announced = 0;
        bool ok        = true;
        ptx::grid_dependency_wait();
#pragma unroll 1
        for (int l = 0; l < num_tiles; l++) {
            const int s = l % STAGES, u = l / STAGES;
            if (u > 0 && !ptx::mbar_wait_bounded(empty(s), (u - 1) & 1, abort_word)) {
                ok = false;
                break;
            }
            const int      kb    = (tile_begin + l) % tiles_k;
            const half*    b_src = p.B + static_cast<size_t>(kb) * kBlockK * p.ld;
            const uint32_t dst   = b_base + s * kBBytes;
#pragma unroll
            for (int i = 0; i < (kChunks + kLoaders - 1) / kLoaders; i++) {
                const uint32_t c = loader + i * kLoaders;
                if (kChunks % kLoaders == 0 || c < kChunks) {
                    const uint32_t row = c / kChunksPerRow, col = c % kChunksPerRow;
                    ptx::cp_async_16(dst + BT::swizzle(row * BT::kRowBytes + col * 16u),
                                     b_src + static_cast<size_t>(row) * p.ld + col * 8);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (l >= kBLag) {
                asm volatile("cp.async.wait_group %0;" ::"n"(kBLag) : "memory");
                announce(announced++);
            }
        }
        ptx::cp_async_wait_all();
        if (ok)
            while (announced < num_tiles)
                announce(announced++);
    }
    else if (warp == kFirstMmaWarp) {
        // ------------------------------------------------------------ MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_f16_f32(kTileRows, NB, false, true) | ptx::kIdescSparse;
            const uint64_t a_desc0 = ptx::make_smem_desc(a_base, 16, 1024, ptx::kSwizzle128B);
            const uint64_t b_desc0 = ptx::make_smem_desc(b_base, BT::kGroupBytes, BT::kGroupBytes, BT::kSwizzleMode);
            const uint64_t e_desc0 = ptx::make_smem_desc(e_base, 128, 128, ptx::kSwizzleNone);
            bool ok  = true;
            int  seg = 0;
#pragma unroll 1
            for (int l0 = 0; l0 < num_tiles && ok; ++seg) {
                const int      j0     = (tile_begin + l0) % tiles_k;
                const int      len    = min(tiles_k - j0, num_tiles - l0);
                const uint32_t d_tmem = tmem_base + (seg & 1) * NB;
                if (seg >= 2)
                    ok = ptx::mbar_wait_bounded(acc_free(seg & 1), ((seg >> 1) - 1) & 1, abort_word);
                uint32_t accumulate = 0;
#pragma unroll 1
                for (int l = l0; l < l0 + len && ok; l++) {
                    const int      s      = l % STAGES;
                    const uint32_t parity = (l / STAGES) & 1;
                    ok = ptx::mbar_wait_bounded(ae_full(s), parity, abort_word)
                         && ptx::mbar_wait_bounded(b_full(s), parity, abort_word);
                    if (!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (kBlockValueBytes >> 4));
                    const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(s * (kBBytes >> 4));
                    ptx::tmem_cp_128x128b(tmem_e + 4 * s, e_desc0 + static_cast<uint64_t>(s * (kBlockMetaBytes >> 4)));
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; k++) {
                        // A: 16 kept halves = 32 bytes along the swizzled row; B: 32 k rows = four 8-row groups
                        // the metadata address names a pair of columns; the descriptor's low bits pick one
                        ptx::umma_f16_sp_ss(d_tmem,
                                            a_desc + static_cast<uint64_t>((k * 32) >> 4),
                                            b_desc + static_cast<uint64_t>((k * 4 * BT::kGroupBytes) >> 4),
                                            tmem_e + 4 * s + (k & ~1),
                                            idesc | static_cast<uint32_t>(k & 1),
                                            k == 0 ? accumulate : 1u);
                    }
                    ptx::umma_commit(empty(s));
                    accumulate = 1;
                }
                if (ok)
                    ptx::umma_commit(acc_full(seg & 1));
                l0 += len;
            }
        }
    }
    else {
        // ------------------------------------------------------------ epilogue
        const int row_in_tile = warp * 32 + lane;
        int       seg         = 0;
        ptx::grid_dependency_wait();
#pragma unroll 1
        for (int l = 0; l < num_tiles; ++seg) {
            const int  t0       = tile_begin + l;
            const int  row_tile = t0 / tiles_k;
            const int  j0       = t0 % tiles_k;
            const int  len      = min(tiles_k - j0, num_tiles - l);
            const bool whole    = (j0 == 0) && (len == tiles_k);
            if (!warp_wait(acc_full(seg & 1), (seg >> 1) & 1, abort_word, lane))
                break;
            ptx::tc_fence_after_sync();
            constexpr int CH = N < 16 ? 8 : 16;  // columns handled at a time
            auto load_chunk = [&](int c, float* out) {
                const uint32_t taddr = tmem_base + (seg & 1) * NB + c * CH + (static_cast<uint32_t>(warp * 32) << 16);
                if (CH == 8)
                    ptx::tmem_ld_x8(taddr, reinterpret_cast<uint32_t*>(out));
                else
                    ptx::tmem_ld_x16(taddr, reinterpret_cast<uint32_t*>(out));
                ptx::tmem_ld_wait();
            };
            auto store_chunk = [&](int c, const float* v) {
                const size_t row = static_cast<size_t>(row_tile) * kTileRows + row_in_tile;
                if (p.C32 != nullptr) {
                    float4* dst = reinterpret_cast<float4*>(p.C32 + row * N + c * CH);
#pragma unroll
                    for (int i = 0; i < CH / 4; i++)
                        dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    return;
                }
                uint4* dst = reinterpret_cast<uint4*>(p.C + row * p.ld + c * CH);
#pragma unroll
                for (int i = 0; i < CH / 8; i++) {
                    __half2 h0 = __floats2half2_rn(v[8 * i], v[8 * i + 1]);
                    __half2 h1 = __floats2half2_rn(v[8 * i + 2], v[8 * i + 3]);
                    __half2 h2 = __floats2half2_rn(v[8 * i + 4], v[8 * i + 5]);
                    __half2 h3 = __floats2half2_rn(v[8 * i + 6], v[8 * i + 7]);
                    uint4   o;
                    o.x    = *reinterpret_cast<uint32_t*>(&h0);
                    o.y    = *reinterpret_cast<uint32_t*>(&h1);
                    o.z    = *reinterpret_cast<uint32_t*>(&h2);
                    o.w    = *reinterpret_cast<uint32_t*>(&h3);
                    dst[i] = o;
                }
            };
            if (whole) {
#pragma unroll 1
                for (int c = 0; c < N / CH; c++) {
                    float v[CH];
                    load_chunk(c, v);
                    store_chunk(c, v);
                }
            }
            else {
                // Park the partial row, count arrivals, let the last arriver sum in owner order.
                const int  head_row  = tile_begin / tiles_k;
                const bool head_part = (tile_begin % tiles_k != 0) || (tile_end < (head_row + 1) * tiles_k);
                const int  above     = p.sched.split_rows_above[cta] + ((row_tile != head_row && head_part) ? 1 : 0);
                int        g_first = cta, g_last = cta;
                while (p.sched.chunk_begin[g_first] > row_tile * tiles_k)
                    g_first--;
                while (p.sched.chunk_begin[g_last + 1] < (row_tile + 1) * tiles_k)
                    g_last++;
                // slots as [N / 4 groups of four columns][128 rows] float4: a warp's 32 rows are contiguous (see spmm_decode_kernel)
                auto slot_of = [&](int g) {
                    return reinterpret_cast<float4*>(p.slots) + static_cast<size_t>(g + above) * (kTileRows * N / 4) + row_in_tile;
                };
                float4* const mine = slot_of(cta);
#pragma unroll 1
                for (int c = 0; c < N / CH; c++) {
                    float v[CH];
                    load_chunk(c, v);
#pragma unroll
                    for (int i = 0; i < CH / 4; i++)
                        __stcg(mine + (c * (CH / 4) + i) * kTileRows, make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
                }
                __threadfence();
                __syncwarp();
                unsigned int  arrived = 0;
                unsigned int* counter = &g_row_arrivals[p.counter_set][row_tile * kEpilogueWarps + warp];
                if (lane == 0)
                    arrived = atomicAdd(counter, 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == static_cast<unsigned int>(g_last - g_first)) {
                    if (lane == 0)
                        *counter = 0;
                    __threadfence();
#pragma unroll 1
                    for (int c = 0; c < N / CH; c++) {
                        float own[CH], sum[CH];
                        load_chunk(c, own);
#pragma unroll
                        for (int n = 0; n < CH; n++)
                            sum[n] = 0.0f;
#pragma unroll 1
                        for (int g = g_first; g <= g_last; g++) {
                            if (g == cta) {
#pragma unroll
                                for (int n = 0; n < CH; n++)
                                    sum[n] += own[n];
                            }
                            else {
                                const float4* theirs = slot_of(g) + c * (CH / 4) * kTileRows;
#pragma unroll
                                for (int i = 0; i < CH / 4; i++) {
                                    const float4 x = __ldcg(theirs + i * kTileRows);
                                    sum[4 * i] += x.x;
                                    sum[4 * i + 1] += x.y;
                                    sum[4 * i + 2] += x.z;
                                    sum[4 * i + 3] += x.w;
                                }
                            }
                        }
                        store_chunk(c, sum);
                    }
                }
            }
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(acc_free(seg & 1));
            l += len;
        }
    }

    // ---------------------------------------------------------------- exit
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word != 0)
        atomicExch(&g_device_status, static_cast<int>(kStatusWaitTimeout));
    if (warp == kFirstMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace spmm_b200
