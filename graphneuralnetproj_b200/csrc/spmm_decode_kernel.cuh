// Decode-size (N <= 64) "load-as-sparse, compute-as-dense" SpMM for sm_100a.
//
// Replaces the reference's SpMM_Kernel (csrc/SpMM_Kernel.cuh:293-735) and its
// Ampere pipeline -- cp.async staging, ldmatrix, mma.sync m16n8k16
// (csrc/MatMulUtilities.cuh:190-245, csrc/MMA_PTX.cuh:15-193) -- and folds
// the split-K reduction (csrc/Reduction_Kernel.cuh:24-47) into the epilogue.
//
// One persistent thread block per SM works through a contiguous chunk of the
// tile sequence (see schedule.h).  Roles, by warp:
//
//   warps 0..3     epilogue: TMEM -> registers -> C, or -> an fp32 slot plus the
//                  last-arriver reduction for rows whose K range is shared
//   warp  4        allocates TMEM; one lane issues tcgen05.mma and commits
//   warps 5..5+D-1 decoders, one 128 x 64 tile at a time each, round-robin:
//                  128-bit streaming loads of the tile's words into registers,
//                  zero the warp's own 16 KB A buffer, scatter the values to
//                  the half-word positions the words carry, stage the matching
//                  64 x N slice of B, hand the pair to the MMA lane
//
// The position stored in each word, row * 64 + (col ^ ((row % 8) << 3))
// (csrc/SpMM_API.cu:330-339), is the element offset of (row, col) in a K-major
// 128 x 64 fp16 tile in the tensor core's 128-byte-swizzle layout, so the
// scatter needs no index arithmetic and the restored tile is read by
// tcgen05.mma as it lies.  B[K][N] is row-major, i.e. N-contiguous ("MN-major"
// for the tensor core); a 64 x N slice is copied chunk by chunk into the
// matching 32/64/128-byte-swizzle layout.  Accumulation is fp32 in TMEM, two
// accumulators so that the epilogue of one row of tiles overlaps the next.
//
// Every wait is bounded (ptx::mbar_wait_bounded); a wait that gives up raises
// a block-wide abort word, all roles fall through to the common exit, TMEM is
// released and a status word in global memory records the event.
#pragma once

#include <cuda_fp16.h>

#include "ptx_sm100.cuh"
#include "schedule.h"

namespace spmm_b200 {

constexpr int kTileRows        = 128;    // rows of an encoded tile = UMMA M
constexpr int kTileCols        = 64;     // k extent of an encoded tile
constexpr int kATileBytes      = kTileRows * kTileCols * 2;
constexpr int kEpilogueWarps   = 4;
constexpr int kMmaWarp         = 4;
constexpr int kFirstDecodeWarp = 5;
constexpr int kMaxRowTiles     = 8192;  // arrival counters are sized for M <= 128 * 8192

enum DeviceStatus : int { kStatusOk = 0, kStatusWaitTimeout = 1 };

// Arrival counters for rows of tiles whose K range is split between blocks, four per
// row (one per 32-row quarter, i.e. per epilogue warp).  Zero between launches: the
// last arriver resets its counter.
__device__ unsigned int g_row_arrivals[kMaxRowTiles * kEpilogueWarps];
__device__ int          g_device_status;

struct DecodeParams {
    const uint4* words;         // tiled-CSL words, viewed as 4-word vectors
    const int*   tile_offsets;  // vectors before each tile
    const half*  B;             // [K][N] row-major
    half*        C;             // [M][N] row-major
    float*       slots;         // fp32 partial tiles, 128 * N floats each
    int          n;             // N (8, 16, 32 or 64)
    int          tiles_k;       // K / 64
    Schedule     sched;
};

template<int NB>
struct BTile {
    static constexpr int      kRowBytes    = NB * 2;
    static constexpr int      kBytes       = kTileCols * kRowBytes;
    static constexpr int      kSwizzleBits = NB == 16 ? 1 : (NB == 32 ? 2 : 3);
    static constexpr uint64_t kSwizzleMode =
        NB == 16 ? ptx::kSwizzle32B : (NB == 32 ? ptx::kSwizzle64B : ptx::kSwizzle128B);
    static constexpr int kGroupBytes = 8 * kRowBytes;  // eight k rows: the descriptor's stride offset
    // XOR the 16-byte chunk index with address bits 7.. (Swizzle<bits,4,3> on byte offsets).
    __device__ static __forceinline__ uint32_t swizzle(uint32_t byte_offset)
    {
        return byte_offset ^ (((byte_offset >> 7) & ((1u << kSwizzleBits) - 1u)) << 4);
    }
};

template<int NB, int D>
constexpr int decode_smem_bytes()
{
    return 1024 + D * (kATileBytes + BTile<NB>::kBytes) + 256;
}

// N  : columns of B / C (8, 16, 32, 64);   NB : columns of the staged B tile (16 when N == 8)
// D  : decoder warps = depth of the A/B tile ring;   VPL : 4-word vectors held per lane
template<int N, int D, int VPL>
__global__ void __launch_bounds__((kFirstDecodeWarp + D) * 32, 1)
spmm_decode_kernel(const __grid_constant__ DecodeParams p)
{
    constexpr int NB = N < 16 ? 16 : N;
    using BT         = BTile<NB>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base    = smem_base;
    const uint32_t b_base    = a_base + D * kATileBytes;
    const uint32_t bar_base  = b_base + D * BT::kBytes;
    // barrier map (8 bytes each): [0,D) tile full, [D,2D) tile free, then acc full x2, acc free x2
    auto tile_full = [&](int s) { return bar_base + 8u * s; };
    auto tile_free = [&](int s) { return bar_base + 8u * (D + s); };
    auto acc_full  = [&](int b) { return bar_base + 8u * (2 * D + b); };
    auto acc_free  = [&](int b) { return bar_base + 8u * (2 * D + 2 + b); };
    const uint32_t tmem_slot_addr = bar_base + 8u * (2 * D + 4);
    uint8_t*       smem_generic   = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
    volatile uint32_t* tmem_slot  = reinterpret_cast<volatile uint32_t*>(smem_generic + (tmem_slot_addr - smem_base));
    volatile int*      abort_word = reinterpret_cast<volatile int*>(smem_generic + (tmem_slot_addr + 4 - smem_base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta  = blockIdx.x;

    const int tile_begin = p.sched.chunk_begin[cta];
    const int tile_end   = p.sched.chunk_begin[cta + 1];
    const int num_tiles  = tile_end - tile_begin;
    const int tiles_k    = p.tiles_k;
    constexpr uint32_t kTmemCols = 2 * NB < 32 ? 32 : 2 * NB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < D; s++) {
            ptx::mbar_init(tile_full(s), 1);
            ptx::mbar_init(tile_free(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            ptx::mbar_init(acc_full(b), 1);
            ptx::mbar_init(acc_free(b), kEpilogueWarps);
        }
        *abort_word = 0;
        ptx::mbar_init_fence();
    }
    if (N < NB) {
        // Columns N..NB-1 of the staged B tiles are never written; clear them once.
        for (uint32_t off = threadIdx.x * 16u; off < static_cast<uint32_t>(D * BT::kBytes); off += blockDim.x * 16u)
            ptx::st_shared_zero_128(b_base + off);
    }
    if (warp == kMmaWarp) {
        ptx::tmem_alloc(tmem_slot_addr, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= kFirstDecodeWarp) {
        // ------------------------------------------------------------ decoder
        const int      w      = warp - kFirstDecodeWarp;
        const uint32_t a_tile = a_base + w * kATileBytes;
        const uint32_t b_tile = b_base + w * BT::kBytes;
        int off0 = 0, off1 = 0;
        if (w < num_tiles) {
            off0 = __ldg(p.tile_offsets + tile_begin + w);
            off1 = __ldg(p.tile_offsets + tile_begin + w + 1);
        }
        int use = 0;
#pragma unroll 1
        for (int l = w; l < num_tiles; l += D, ++use) {
            const int    t    = tile_begin + l;
            const int    nvec = off1 - off0;
            const uint4* src  = p.words + off0;
            uint4        r[VPL];
#pragma unroll
            for (int v = 0; v < VPL; v++)
                if (v * 32 + lane < nvec)
                    r[v] = ptx::ld_stream_128(src + v * 32 + lane);
            if (l + D < num_tiles) {
                off0 = __ldg(p.tile_offsets + t + D);
                off1 = __ldg(p.tile_offsets + t + D + 1);
            }
            if (use > 0 && !ptx::mbar_wait_bounded(tile_free(w), (use - 1) & 1, abort_word))
                break;
            // B slice of this k tile: 64 rows of N halves, contiguous in global memory.
            {
                const uint4* b_src = reinterpret_cast<const uint4*>(p.B + static_cast<size_t>(t % tiles_k) * kTileCols * N);
                constexpr int kChunksPerRow = N / 8;
#pragma unroll
                for (int c = lane; c < kTileCols * kChunksPerRow; c += 32) {
                    const uint32_t row = c / kChunksPerRow, col = c % kChunksPerRow;
                    ptx::cp_async_16(b_tile + BT::swizzle(row * BT::kRowBytes + col * 16u), b_src + c);
                }
            }
#pragma unroll
            for (int i = 0; i < kATileBytes / (32 * 16); i++)
                ptx::st_shared_zero_128(a_tile + (i * 32 + lane) * 16u);
            __syncwarp();
#pragma unroll
            for (int v = 0; v < VPL; v++)
                if (v * 32 + lane < nvec) {
                    ptx::st_shared_u16(a_tile + ((r[v].x >> 16) << 1), r[v].x);
                    ptx::st_shared_u16(a_tile + ((r[v].y >> 16) << 1), r[v].y);
                    ptx::st_shared_u16(a_tile + ((r[v].z >> 16) << 1), r[v].z);
                    ptx::st_shared_u16(a_tile + ((r[v].w >> 16) << 1), r[v].w);
                }
#pragma unroll 1
            for (int idx = VPL * 32 + lane; idx < nvec; idx += 32) {  // tiles denser than VPL * 32 vectors
                const uint4 x = ptx::ld_stream_128(src + idx);
                ptx::st_shared_u16(a_tile + ((x.x >> 16) << 1), x.x);
                ptx::st_shared_u16(a_tile + ((x.y >> 16) << 1), x.y);
                ptx::st_shared_u16(a_tile + ((x.z >> 16) << 1), x.z);
                ptx::st_shared_u16(a_tile + ((x.w >> 16) << 1), x.w);
            }
            ptx::cp_async_wait_all();
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(tile_full(w));
        }
        ptx::cp_async_wait_all();
    }
    else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_f16_f32(kTileRows, NB, false, true);
            int                seg   = 0;
#pragma unroll 1
            for (int l = 0; l < num_tiles; l++) {
                const int  j     = (tile_begin + l) % tiles_k;
                const int  s     = l % D;
                const bool first = (l == 0) || (j == 0);
                if (first && seg >= 2 && !ptx::mbar_wait_bounded(acc_free(seg & 1), ((seg >> 1) - 1) & 1, abort_word))
                    break;
                if (!ptx::mbar_wait_bounded(tile_full(s), (l / D) & 1, abort_word))
                    break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (seg & 1) * NB;
                const uint64_t a_desc = ptx::make_smem_desc(a_base + s * kATileBytes, 16, 1024, ptx::kSwizzle128B);
                const uint64_t b_desc =
                    ptx::make_smem_desc(b_base + s * BT::kBytes, BT::kGroupBytes, BT::kGroupBytes, BT::kSwizzleMode);
#pragma unroll
                for (int k = 0; k < kTileCols / 16; k++) {
                    // A: 16 k values = 32 bytes along the swizzled row; B: 16 k rows = two 8-row groups.
                    ptx::umma_f16_ss(d_tmem,
                                     a_desc + static_cast<uint64_t>((k * 32) >> 4),
                                     b_desc + static_cast<uint64_t>((k * 2 * BT::kGroupBytes) >> 4),
                                     idesc,
                                     (first && k == 0) ? 0u : 1u);
                }
                ptx::umma_commit(tile_free(s));
                if (j == tiles_k - 1 || l == num_tiles - 1) {
                    ptx::umma_commit(acc_full(seg & 1));
                    seg++;
                }
            }
        }
    }
    else {
        // ------------------------------------------------------------ epilogue
        const int row_in_tile = warp * 32 + lane;
        int       seg         = 0;
#pragma unroll 1
        for (int l = 0; l < num_tiles; ++seg) {
            const int  t0       = tile_begin + l;
            const int  row_tile = t0 / tiles_k;
            const int  j0       = t0 % tiles_k;
            const int  len      = min(tiles_k - j0, num_tiles - l);
            const bool whole    = (j0 == 0) && (len == tiles_k);
            if (!ptx::mbar_wait_bounded(acc_full(seg & 1), (seg >> 1) & 1, abort_word))
                break;
            ptx::tc_fence_after_sync();
            float          acc[N];
            const uint32_t taddr = tmem_base + (seg & 1) * NB + (static_cast<uint32_t>(warp * 32) << 16);
            if (N == 8) {
                ptx::tmem_ld_x8(taddr, reinterpret_cast<uint32_t*>(acc));
            }
            else {
#pragma unroll
                for (int c = 0; c < N / 16; c++)
                    ptx::tmem_ld_x16(taddr + c * 16, reinterpret_cast<uint32_t*>(acc) + c * 16);
            }
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(acc_free(seg & 1));

            bool write_c = whole;
            if (!whole) {
                // Park the partial row, count arrivals, let the last arriver sum in owner order.
                const int  head_row  = tile_begin / tiles_k;
                const bool head_part = (tile_begin % tiles_k != 0) || (tile_end < (head_row + 1) * tiles_k);
                const int  above     = p.sched.split_rows_above[cta] + ((row_tile != head_row && head_part) ? 1 : 0);
                int        g_first = cta, g_last = cta;
                while (p.sched.chunk_begin[g_first] > row_tile * tiles_k)
                    g_first--;
                while (p.sched.chunk_begin[g_last + 1] < (row_tile + 1) * tiles_k)
                    g_last++;
                float* mine = p.slots + (static_cast<size_t>(cta + above) * kTileRows + row_in_tile) * N;
#pragma unroll
                for (int c = 0; c < N / 4; c++)
                    __stcg(reinterpret_cast<float4*>(mine) + c, make_float4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]));
                __threadfence();
                __syncwarp();
                unsigned int arrived = 0;
                unsigned int* counter = &g_row_arrivals[row_tile * kEpilogueWarps + warp];
                if (lane == 0)
                    arrived = atomicAdd(counter, 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == static_cast<unsigned int>(g_last - g_first)) {
                    if (lane == 0)
                        *counter = 0;
                    __threadfence();
                    float sum[N];
#pragma unroll
                    for (int n = 0; n < N; n++)
                        sum[n] = 0.0f;
#pragma unroll 1
                    for (int g = g_first; g <= g_last; g++) {
                        if (g == cta) {
#pragma unroll
                            for (int n = 0; n < N; n++)
                                sum[n] += acc[n];
                        }
                        else {
                            const float4* theirs = reinterpret_cast<const float4*>(
                                p.slots + (static_cast<size_t>(g + above) * kTileRows + row_in_tile) * N);
#pragma unroll
                            for (int c = 0; c < N / 4; c++) {
                                const float4 x = __ldcg(theirs + c);
                                sum[4 * c] += x.x;
                                sum[4 * c + 1] += x.y;
                                sum[4 * c + 2] += x.z;
                                sum[4 * c + 3] += x.w;
                            }
                        }
                    }
#pragma unroll
                    for (int n = 0; n < N; n++)
                        acc[n] = sum[n];
                    write_c = true;
                }
            }
            if (write_c) {
                uint4* dst = reinterpret_cast<uint4*>(p.C + (static_cast<size_t>(row_tile) * kTileRows + row_in_tile) * N);
#pragma unroll
                for (int c = 0; c < N / 8; c++) {
                    __half2 h0 = __floats2half2_rn(acc[8 * c], acc[8 * c + 1]);
                    __half2 h1 = __floats2half2_rn(acc[8 * c + 2], acc[8 * c + 3]);
                    __half2 h2 = __floats2half2_rn(acc[8 * c + 4], acc[8 * c + 5]);
                    __half2 h3 = __floats2half2_rn(acc[8 * c + 6], acc[8 * c + 7]);
                    uint4   o;
                    o.x    = *reinterpret_cast<uint32_t*>(&h0);
                    o.y    = *reinterpret_cast<uint32_t*>(&h1);
                    o.z    = *reinterpret_cast<uint32_t*>(&h2);
                    o.w    = *reinterpret_cast<uint32_t*>(&h3);
                    dst[c] = o;
                }
            }
            l += len;
        }
    }

    // ---------------------------------------------------------------- exit
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word != 0)
        atomicExch(&g_device_status, static_cast<int>(kStatusWaitTimeout));
    if (warp == kMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace spmm_b200
