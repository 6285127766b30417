// "Load-as-sparse, compute-as-dense" SpMM for sm_100a: C[M][N] = A * B with A in the reference's
// tiled-CSL format (128 x 64 tiles of value|position words, csrc/SpMM_API.cu:241-438).
//
// Replaces the reference's SpMM_Kernel (csrc/SpMM_Kernel.cuh:293-735) and its
// Ampere pipeline -- cp.async staging, ldmatrix, mma.sync m16n8k16
// (csrc/MatMulUtilities.cuh:190-245, csrc/MMA_PTX.cuh:15-193) -- and folds
// the split-K reduction (csrc/Reduction_Kernel.cuh:24-47) into the epilogue.
//
// One persistent thread block per SM works through a contiguous chunk of the
// tile sequence (see schedule.h).  The block keeps a ring of S slots, each a
// 16 KB buffer for a restored 128 x 64 fp16 tile of A plus one or two staged
// 64 x N slices of B.  Roles, by warp:
//
//   warps 0..3      epilogue: TMEM -> registers -> C, or -> an fp32 slot plus the
//                   last-arriver reduction for rows whose K range is shared
//   warps 4..4+Q-1  MMA issue: one lane each; warp q takes tiles q, q + Q, ... of the
//                   chunk and accumulates them in its own TMEM accumulator (the
//                   epilogue adds the Q accumulators in a fixed order).  Several
//                   issuers because one lane, sharing its scheduler with busy
//                   decoder warps, cannot issue four MMAs and a commit per tile fast
//                   enough; warp 4 also allocates TMEM.  Where B arrives by tiled TMA
//                   loads a lap ahead (BM == 2) these lanes issue them, and they ask
//                   for the words two laps ahead to be brought into L2.
//   warps 4+Q..     decoders: D teams of WPT warps; team t restores tiles t, t + D, ...
//                   of the chunk into slot (tile % S).  Per tile a team
//                     - holds the tile's words in registers: 128-bit streaming loads, issued
//                       as soon as the previous tile has been scattered, without a branch
//                       around them so that they pipeline (the words were asked into L2
//                       two laps earlier),
//                     - waits until the tensor core has finished with the slot,
//                     - clears the A buffer with 128-bit stores,
//                     - scatters the values to the half-word positions the words carry,
//                     - hands the slot to an MMA lane (mbarrier arrive).
//
// The position stored in each word, row * 64 + (col ^ ((row % 8) << 3))
// (csrc/SpMM_API.cu:330-339), is the element offset of (row, col) in a K-major
// 128 x 64 fp16 tile in the tensor core's 128-byte-swizzle layout, so the
// scatter needs no index arithmetic and the restored tile is read by
// tcgen05.mma as it lies.  B[K][N] is row-major, i.e. N-contiguous ("MN-major"
// for the tensor core); a 64 x N slice is staged in the matching 32/64/128-byte
// swizzle layout.  Accumulation is fp32 in TMEM, two accumulator sets so that
// the epilogue of one row of tiles overlaps the next.
//
// Every wait is bounded (ptx::mbar_wait_bounded); a wait that gives up raises
// a block-wide abort word, all roles fall through to the common exit, TMEM is
// released and a status word in global memory records the event.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"
#include "schedule.h"

namespace spmm_b200 {

constexpr int kTileRows        = 128;  // rows of an encoded tile = UMMA M
constexpr int kTileCols        = 64;   // k extent of an encoded tile
constexpr int kATileBytes      = kTileRows * kTileCols * 2;
constexpr int kEpilogueWarps   = 4;
constexpr int kFirstMmaWarp    = 4;
constexpr int kMaxRowTiles     = 32768;  // arrival counters: rows of tiles x column blocks per launch
constexpr int kCounterSets     = 8;      // independent sets of arrival counters (one per workspace in use)
constexpr int kPrefetchRounds  = 2;      // a tile's words are asked into L2 this many laps before they are copied

enum DeviceStatus : int { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadInput = 2 };

// Arrival counters for rows of tiles whose K range is split between blocks, four per
// row (one per 32-row quarter, i.e. per epilogue warp).  Zero between launches: the
// last arriver resets its counter.  Launches that may overlap in time use different sets.
__device__ unsigned int g_row_arrivals[kCounterSets][kMaxRowTiles * kEpilogueWarps];
__device__ int          g_device_status;

constexpr int kMaxPeers = 8;  // ranks of a row-parallel (split by K) layer whose sum is folded into the epilogue

// Sum over the ranks of a layer split by K, folded into the SpMM's epilogue (no counterpart in the
// reference, which is single-GPU; its FasterTransformer glue all-reduces with NCCL after the product).
// Every rank writes its finished rows, still in fp32, to its own partial buffer instead of C.  When all
// blocks of a rank have written theirs, the last of them tells every rank (one flag per sender, carrying
// the call's epoch, after one system-scope fence); the blocks then take rows of tiles in turn, wait for
// all ranks' flags, add the ranks' partial rows in rank order out of the peers' memory (plain loads over
// NVLink) and round once to fp16.  Epochs only grow, so nothing is reset; the partial buffers alternate
// with the epoch's parity, so a fast rank's next product never overwrites what a slow peer is still
// reading.  fp32 partials because fp16 ones put the mean relative error of the sum right at the 1e-3
// acceptance gate (entries much smaller than their partial sums).  (An earlier form flagged every
// quarter of a row of tiles as it was finished, to overlap the sums with the product: all rows finish
// at the end of a balanced persistent kernel, so nothing overlapped and the fences cost 8-16 us.)
struct PeerSumParams {
    float*    partial[2][kMaxPeers] = {};  // [epoch parity][rank]: that rank's partial result, fp32 [M][N], mapped here
    uint32_t* flags[kMaxPeers]      = {};  // flags[r]: rank r's flag array, one word per sender
    uint32_t* state                 = nullptr;  // this rank's: [0] epoch of the previous call, [1] block counter
    int       rank = 0, world = 0;              // world == 0: no sum over ranks
    // 1: only write this rank's fp32 partial rows (buffer of parity (state[0] + 1) & 1); the flags, the sum and
    // the advance of the epoch are left to the reduction kernel launched next in the stream
    // 2: as 1, and the last block of this kernel to finish tells every rank that the partial rows are complete (entry
    //    [rank] of every rank's flag array gets the call's epoch), so that the exchange of flags travels while the
    //    reduction kernel is being launched; that kernel then only waits for the flags
    int       partial_only = 0;
    unsigned long long limit_ns = 0;
};

struct DecodeParams {
    const uint4* words        = nullptr;  // tiled-CSL words, viewed as 4-word vectors
    const int*   tile_offsets = nullptr;  // vectors before each tile
    const half*  B            = nullptr;  // [K][N] row-major
    half*        C            = nullptr;  // [M][N] row-major
    float*       slots        = nullptr;  // fp32 partial tiles, 128 * N floats each
    int          counter_set  = 0;        // which set of arrival counters this launch uses
    int          n            = 0;        // N (8, 16, 32 or 64)
    int          tiles_k      = 0;        // K / 64
    int          m            = 0;        // M
    int          ld           = 0;  // row stride of B[K][ld] and C[M][ld] in halves (row-major layout): the full N
    int          slots_per_block_column = 0;  // workspace slots used by one column block (blockIdx.y)
    // 1: the weights and their offsets were complete before the kernel ahead of this one in the stream
    // started (constant inference weights), so they may be fetched before that kernel has finished;
    // 0: nothing is read before the stream predecessor has completed
    int          weights_early = 0;
    const float* addend = nullptr;  // optional fp32 [M][N] added before the rounding (row-major results, N <= 64 only)
    // B as a 2-D tensor [K][ld] of halves, boxes of 64 k rows x min(N, 64) columns in the swizzle mode of
    // the staged layout: for the forms whose B slices arrive by tiled TMA loads (BM != 0)
    alignas(64) CUtensorMap b_map;
    PeerSumParams peer;
    Schedule     sched;
};

// Staged 64 x NB slice of B[K][N] (N-contiguous, "MN-major" for the tensor core).  Up to 64 columns a
// row of the slice is one swizzle row (32, 64 or 128 bytes); wider slices are cut into atoms of 64
// columns, each a 64 x 128-byte block of its own (the descriptor's leading offset steps over atoms).
template<int NB>
struct BTile {
    static constexpr int      kAtomCols    = NB > 64 ? 64 : NB;
    static constexpr int      kAtoms       = NB / kAtomCols;
    static constexpr int      kRowBytes    = kAtomCols * 2;
    static constexpr int      kAtomBytes   = kTileCols * kRowBytes;
    static constexpr int      kBytes       = kAtoms * kAtomBytes;
    static constexpr int      kSwizzleBits = kAtomCols == 16 ? 1 : (kAtomCols == 32 ? 2 : 3);
    static constexpr uint64_t kSwizzleMode =
        kAtomCols == 16 ? ptx::kSwizzle32B : (kAtomCols == 32 ? ptx::kSwizzle64B : ptx::kSwizzle128B);
    static constexpr int kGroupBytes   = 8 * kRowBytes;  // eight k rows: the descriptor's stride offset
    static constexpr int kLeadingBytes = kAtoms > 1 ? kAtomBytes : kGroupBytes;  // the descriptor's leading offset
    // XOR the 16-byte chunk index with address bits 7.. (Swizzle<bits,4,3> on byte offsets).
    __device__ static __forceinline__ uint32_t swizzle(uint32_t byte_offset)
    {
        return byte_offset ^ (((byte_offset >> 7) & ((1u << kSwizzleBits) - 1u)) << 4);
    }
    // Byte offset of 16-byte chunk `chunk` (of the NB-wide row) of k row `row`.
    __device__ static __forceinline__ uint32_t offset(uint32_t row, uint32_t chunk)
    {
        constexpr uint32_t kChunksPerAtomRow = kRowBytes / 16;
        return (chunk / kChunksPerAtomRow) * kAtomBytes + swizzle(row * kRowBytes + (chunk % kChunksPerAtomRow) * 16u);
    }
};

// Per ring slot one A buffer and one or two (BM == 2) B buffers.
template<int NB, int S, int BM>
constexpr int decode_smem_bytes()
{
    return 1024 + S * (kATileBytes + (BM == 2 ? 2 : 1) * BTile<NB>::kBytes) + 512;
}

template<int D, int Q, int WPT>
constexpr int decode_threads()
{
    return (kFirstMmaWarp + Q + D * WPT) * 32;
}

// TMEM is allocated in powers of two, at least 32 columns.
__host__ __device__ constexpr uint32_t tmem_columns(uint32_t needed)
{
    uint32_t c = 32;
    while (c < needed)
        c *= 2;
    return c;
}

// Lane 0 polls, the warp follows.  Returns false (warp-uniform) when the wait was abandoned.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_word, int lane)
{
    int ok = 1;
    if (lane == 0)
        ok = ptx::mbar_wait_bounded(bar, parity, abort_word) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// The value of each of the four words of `w` goes to the half-word position the word carries, in the
// tile at `tile` (a pointer into shared memory).  Written as plain stores so that the compiler hoists
// the address arithmetic of all vectors of a tile and predicates the stores of a ragged last group:
// measured on one warp, 4.3 cycles per store against 12.9 for the same stores inside a branch per vector.
// Positions are taken modulo the tile (13 bits), so a corrupt word cannot write outside the buffer.
__device__ __forceinline__ void scatter_vector(uint8_t* tile, const uint4& w, bool valid)
{
    if (valid) {
        *reinterpret_cast<uint16_t*>(tile + ((w.x >> 15) & 0x3ffeu)) = static_cast<uint16_t>(w.x);
        *reinterpret_cast<uint16_t*>(tile + ((w.y >> 15) & 0x3ffeu)) = static_cast<uint16_t>(w.y);
        *reinterpret_cast<uint16_t*>(tile + ((w.z >> 15) & 0x3ffeu)) = static_cast<uint16_t>(w.z);
        *reinterpret_cast<uint16_t*>(tile + ((w.w >> 15) & 0x3ffeu)) = static_cast<uint16_t>(w.w);
    }
}

// N    : columns of B / C handled by one block column (8, 16, 32, 64, 128, 256); the staged B tile has
//        NB = max(N, 16) columns
// D    : decoder teams;  Q : MMA-issuing warps;  WPT : decoder warps per team;
// VPL  : 4-word vectors held per lane;  S : ring slots (S >= D, S % Q == 0).  Tile l of the chunk is
//        decoded by team l % D into slot l % S and multiplied by MMA warp l % Q.
// TM   : 1 = token-major activations and results, B[N][K] and C[N][M] (the layout of the upstream
//        library and of its FasterTransformer caller, third_party/ft.patch:2822-2846): the B slice of a
//        k tile is then K-contiguous and is staged in the same 128-byte-swizzle layout as A.
// BM   : how a tile's B slice reaches shared memory.  0: 16-byte async copies by the tile's decoders,
//        1: tiled TMA loads issued by one of them, both once the slot has been handed back (one B
//        buffer per slot); 2: tiled TMA loads issued by the MMA warp one lap ahead into the other of
//        two B buffers per slot (the decoders never touch B).  1 and 2 need p.b_map and row-major B.
template<int N, int D, int Q, int WPT, int VPL, int S, int TM, int BM>
__global__ void __launch_bounds__(decode_threads<D, Q, WPT>(), 1)
spmm_decode_kernel(const __grid_constant__ DecodeParams p)
{
    constexpr int NB   = N < 16 ? 16 : N;
    constexpr int BBUF = BM == 2 ? 2 : 1;  // B buffers per slot
    using BT           = BTile<NB>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base    = smem_base;
    const uint32_t b_base    = a_base + S * kATileBytes;
    const uint32_t bar_base  = b_base + BBUF * S * BT::kBytes;
    // barrier map (8 bytes each): [0,S) tile full, [S,2S) tile free, acc full x2, acc free x2
    auto tile_full  = [&](int s) { return bar_base + 8u * s; };
    auto tile_free  = [&](int s) { return bar_base + 8u * (S + s); };
    auto acc_full   = [&](int b) { return bar_base + 8u * (2 * S + b); };
    auto acc_free   = [&](int b) { return bar_base + 8u * (2 * S + 2 + b); };
    const uint32_t tmem_slot_addr = bar_base + 8u * (2 * S + 4);
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
    constexpr int      kFirstDecodeWarp = kFirstMmaWarp + Q;
    // Who asks for the words kPrefetchRounds laps ahead to be brought into L2: the MMA warps (which have
    // time to spare) wherever the kernel uses the tensor-map forms of loading B, else the decoders.
    constexpr bool     kMmaRequests     = BM != 0;
    constexpr uint32_t kTmemCols        = tmem_columns(2 * Q * NB);  // accumulator (q, b) at column (b * Q + q) * NB
    static_assert(2 * Q * NB <= 512, "accumulators exceed the 512 TMEM columns");
    static_assert(S % Q == 0, "a ring slot must always be served by the same MMA warp (barrier phases alias otherwise)");
    static_assert(S >= D, "every team needs a slot of its own to start with");
    static_assert(BM == 0 || !TM, "tiled loads of B are for the row-major layout");
    static_assert(8 * (2 * S + 4) + 8 <= 512, "barrier block");

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            ptx::mbar_init(tile_full(s), WPT);
            ptx::mbar_init(tile_free(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            ptx::mbar_init(acc_full(b), Q);
            ptx::mbar_init(acc_free(b), kEpilogueWarps);
        }
        *abort_word = 0;
        ptx::mbar_init_fence();
    }
    // Clear the ring once: the first lap scatters into it as it is, and columns N..NB-1 of the
    // staged B slices (N == 8) are never written.
    for (uint32_t off = threadIdx.x * 16u; off < static_cast<uint32_t>(S * (kATileBytes + BBUF * BT::kBytes));
         off += blockDim.x * 16u)
        ptx::st_shared_zero_128(a_base + off);
    if (warp == kFirstMmaWarp) {
        ptx::tmem_alloc(tmem_slot_addr, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: the next kernel in the stream may be scheduled from here on (it
    // still needs this block's resources to start on this SM).  This kernel in turn may have started
    // before its predecessor finished: everything the predecessor may still be writing or reading --
    // B, C, the workspace, the arrival counters, and unless p.weights_early is set the weights and
    // their offsets too -- is touched only after ptx::grid_dependency_wait().
    ptx::grid_launch_dependents();

    if (warp >= kFirstDecodeWarp) {
        // ------------------------------------------------------------ decoder team
        const int s_own = (warp - kFirstDecodeWarp) / WPT;  // this team; also its first tile and first slot
        const int h     = (warp - kFirstDecodeWarp) % WPT;  // this warp's share of the tile
        uint32_t  slot  = s_own;                            // ring slot of the tile being decoded
        auto team_sync = [&]() {
            if (WPT > 1)
                asm volatile("bar.sync %0, %1;" ::"r"(s_own + 1), "n"(WPT * 32) : "memory");
            else
                __syncwarp();
        };
        // B staging by the decoders (BM == 0): a 64 x N slice is kTileCols * N / 8 chunks of 16 bytes,
        // contiguous in global memory; this warp copies chunks first_chunk, first_chunk + WPT * 32, ...
        // Chunk c lands at swizzle(row * row_bytes + col * 16), row = c / chunks_per_row.
        constexpr int kChunksPerRow = N / 8;
        constexpr int kChunks       = kTileCols * kChunksPerRow;
        const int     first_chunk   = h * 32 + lane;
        auto stage_b = [&](int j) {
            if (BM == 2)
                return;
            if (BM == 1) {
                // one box of 64 k rows x 64 columns per swizzle atom; the bytes are counted on the
                // barrier the MMA warp waits on for this tile
                if (h == 0 && lane == 0) {
                    const uint32_t bar = tile_full(slot);
                    ptx::mbar_expect_tx(bar, BT::kBytes);
#pragma unroll
                    for (int a = 0; a < BT::kAtoms; a++)
                        ptx::tma_load_2d(b_base + slot * BT::kBytes + a * BT::kAtomBytes, &p.b_map,
                                         static_cast<int>(blockIdx.y) * N + a * BT::kAtomCols, j * kTileCols, bar);
                }
                return;
            }
            const uint32_t dst = b_base + slot * BT::kBytes;
            if (TM) {
                // row n of the slice: 64 halves of token n starting at column 64 j (eight 16-byte chunks);
                // chunk q of row n lands at n * 128 + ((q ^ (n % 8)) * 16)
                // (with several column blocks, blockIdx.y selects N tokens of B[n][K] and of C[n][M])
                const half* b_src = p.B + static_cast<size_t>(blockIdx.y) * N * (static_cast<size_t>(tiles_k) * kTileCols)
                                    + static_cast<size_t>(j) * kTileCols;
#pragma unroll
                for (int i = 0; i < (N * 8) / (WPT * 32); i++) {
                    const uint32_t c = first_chunk + i * WPT * 32;
                    const uint32_t n = c >> 3, q = c & 7;
                    ptx::cp_async_16(dst + n * 128u + ((q ^ (n & 7u)) << 4),
                                     b_src + static_cast<size_t>(n) * (static_cast<size_t>(tiles_k) * kTileCols) + q * 8);
                }
                return;
            }
            // rows of the slice are ld halves apart; this block's columns start at column_block * N
            const half* b_src = p.B + static_cast<size_t>(j) * kTileCols * p.ld + static_cast<size_t>(blockIdx.y) * N;
#pragma unroll
            for (int i = 0; i < kChunks / (WPT * 32); i++) {
                const uint32_t c   = first_chunk + i * WPT * 32;
                const uint32_t row = c / kChunksPerRow, col = c % kChunksPerRow;
                ptx::cp_async_16(dst + BT::offset(row, col), b_src + static_cast<size_t>(row) * p.ld + col * 8);
            }
        };
        // Vector v of this lane within a tile: teams interleave their warps by groups of 32 vectors.
        const int    lane_vec = h * 32 + lane;
        constexpr int kBatch  = VPL * WPT * 32;  // vectors a team holds in registers at a time
        uint4        r[VPL];                     // this warp's share of the tile's words
        int          nvec = 0, next0 = 0, next1 = 0;
        int          j    = (tile_begin + s_own) % tiles_k;
        // Register loads of this lane's VPL vectors of a batch from `from` (the lane's first vector).  No
        // branch per load (loads inside branches do not pipeline: 11 against 2.8 cycles each): a lane whose
        // vector lies beyond the batch's `count` reads the batch's last vector instead and never scatters it.
        auto load_words = [&](const uint4* from, int count) {
            if (count <= 0)
                return;
#pragma unroll
            for (int v = 0; v < VPL; v++)
                r[v] = ptx::ld_stream_128(from + (min(lane_vec + v * WPT * 32, count - 1) - lane_vec));
        };
        auto scatter_batch = [&](uint8_t* tile, int count) {
#pragma unroll
            for (int v = 0; v < VPL; v++)
                scatter_vector(tile, r[v], lane_vec + v * WPT * 32 < count);
        };
        const uint4* src = p.words + lane_vec;  // always offset by this lane's first vector
        // Offsets are read two tiles ahead (next*: tile l + D, after*: tile l + 2D) so that the words of
        // tile l + 2D can be requested into L2 while tile l is being decoded.
        int  after0 = 0, after1 = 0, pf0 = 0, pf1 = 0;
        auto prefetch_tile = [&](int off0, int off1) {
            if (!kMmaRequests && h == 0 && lane == 0 && off1 > off0)
                ptx::bulk_prefetch_l2(p.words + off0, static_cast<uint32_t>(off1 - off0) * 16u);
        };
        if (!p.weights_early)
            ptx::grid_dependency_wait();
        if (s_own < num_tiles) {
            const int off0 = __ldg(p.tile_offsets + tile_begin + s_own);
            const int off1 = __ldg(p.tile_offsets + tile_begin + s_own + 1);
            nvec           = off1 - off0;
            src            = p.words + off0 + lane_vec;
            load_words(src, nvec);
            if (s_own + D < num_tiles) {
                next0 = __ldg(p.tile_offsets + tile_begin + s_own + D);
                next1 = __ldg(p.tile_offsets + tile_begin + s_own + D + 1);
                prefetch_tile(next0, next1);
            }
            if (s_own + 2 * D < num_tiles) {
                after0 = __ldg(p.tile_offsets + tile_begin + s_own + 2 * D);
                after1 = __ldg(p.tile_offsets + tile_begin + s_own + 2 * D + 1);
                prefetch_tile(after0, after1);
            }
        }
        ptx::grid_dependency_wait();
        int use = 0;  // tiles this team has decoded
#pragma unroll 1
        for (int l = s_own; l < num_tiles; l += D, ++use) {
            const bool     has_next = l + D < num_tiles;
            const int      lap      = l / S;  // how often this slot has been filled before
            uint8_t* const a_tile   = smem_generic + slot * kATileBytes;
            if (use > 0)
                prefetch_tile(pf0, pf1);  // tile l + kPrefetchRounds * D; its offsets were read one iteration ago
            if (lap > 0) {
                if (!ptx::mbar_wait_bounded(tile_free(slot), (lap - 1) & 1, abort_word)) {
                    // A team mate that saw the barrier complete may be waiting at the team barrier below.
                    if (WPT > 1)
                        asm volatile("bar.arrive %0, %1;" ::"r"(s_own + 1), "n"(WPT * 32) : "memory");
                    break;
                }
#pragma unroll
                for (int i = h; i < kATileBytes / (32 * 16); i += WPT)
                    ptx::st_shared_zero_128(a_base + slot * kATileBytes + lane * 16u + i * 512u);
                team_sync();  // the whole buffer is clear before anyone scatters into it
            }
            stage_b(j);  // the slot's B buffer is free as well: this tile's slice (BM == 0, 1)
            scatter_batch(a_tile, nvec);
            // Tiles denser than the register budget (kBatch vectors): the rest follows in further
            // register batches; the tile was requested into L2 two rounds ago, so these loads are short.
#pragma unroll 1
            for (int done = kBatch; done < nvec; done += kBatch) {
                load_words(src + done, nvec - done);
                scatter_batch(a_tile, nvec - done);
            }
            if (has_next) {
                nvec = next1 - next0;
                src  = p.words + next0 + lane_vec;
                load_words(src, nvec);  // the next tile's words: in flight from here
                next0 = after0;
                next1 = after1;
                if (l + 3 * D < num_tiles) {
                    after0 = __ldg(p.tile_offsets + tile_begin + l + 3 * D);
                    after1 = __ldg(p.tile_offsets + tile_begin + l + 3 * D + 1);
                }
            }
            pf0 = pf1 = 0;
            if (l + (kPrefetchRounds + 1) * D < num_tiles) {
                pf0 = __ldg(p.tile_offsets + tile_begin + l + (kPrefetchRounds + 1) * D);
                pf1 = __ldg(p.tile_offsets + tile_begin + l + (kPrefetchRounds + 1) * D + 1);
            }
            if (BM == 0)
                ptx::cp_async_wait_all();  // this tile's B slice has landed
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(tile_full(slot));
            j += D;
            while (j >= tiles_k)
                j -= tiles_k;
            slot += D;
            if (slot >= S)
                slot -= S;
        }
        if (BM == 0)
            ptx::cp_async_wait_all();
    }
    else if (warp >= kFirstMmaWarp) {
        // ------------------------------------------------------------ MMA issue
        // Lane 0 of MMA warp q issues the MMAs of tiles q, q + Q, ... (chunk-local numbering) into
        // accumulator (q, segment parity); a segment is the run of tiles that share a row of tiles.
        // Every MMA warp arrives on the segment's acc_full barrier, through tcgen05.commit if it
        // issued anything for the segment and directly otherwise.
        const int q = warp - kFirstMmaWarp;
        ptx::grid_dependency_wait();
        if (lane == 0) {
            constexpr uint32_t idesc   = ptx::make_idesc_f16_f32(kTileRows, NB, false, TM ? false : true);
            const uint64_t     a_desc0 = ptx::make_smem_desc(a_base, 16, 1024, ptx::kSwizzle128B);
            const uint64_t     b_desc0 =
                TM ? ptx::make_smem_desc(b_base, 16, 1024, ptx::kSwizzle128B)
                   : ptx::make_smem_desc(b_base, BT::kLeadingBytes, BT::kGroupBytes, BT::kSwizzleMode);
            // BM == 2: the B slice of chunk-local tile l goes to buffer (l / S) % 2 of slot l % S and is
            // counted on that slot's tile_full barrier, which is in the phase of tile l once the fill of
            // tile l - S has completed (or from the start, for the first lap).
            auto load_b = [&](int l) {
                const int      s   = l % S;
                const uint32_t bar = tile_full(s);
                const uint32_t dst = b_base + ((((l / S) & 1) * S) + s) * BT::kBytes;
                const int      j   = (tile_begin + l) % tiles_k;
                ptx::mbar_expect_tx(bar, BT::kBytes);
#pragma unroll
                for (int a = 0; a < BT::kAtoms; a++)
                    ptx::tma_load_2d(dst + a * BT::kAtomBytes, &p.b_map, static_cast<int>(blockIdx.y) * N + a * BT::kAtomCols,
                                     j * kTileCols, bar);
            };
            // kMmaRequests: this lane also asks for the words of its tiles two laps ahead to be brought into L2
            auto request_words = [&](int off0, int off1) {
                if (off1 > off0)
                    ptx::bulk_prefetch_l2(p.words + off0, static_cast<uint32_t>(off1 - off0) * 16u);
            };
            if (BM == 2) {
#pragma unroll 1
                for (int l = q; l < S && l < num_tiles; l += Q)
                    load_b(l);
            }
            if (kMmaRequests) {
#pragma unroll 1
                for (int l = q + S; l < kPrefetchRounds * S && l < num_tiles; l += Q)
                    request_words(__ldg(p.tile_offsets + tile_begin + l), __ldg(p.tile_offsets + tile_begin + l + 1));
            }
            bool ok  = true;
            int  seg = 0;
#pragma unroll 1
            for (int l0 = 0; l0 < num_tiles && ok; ++seg) {
                const int j0    = (tile_begin + l0) % tiles_k;
                const int len   = min(tiles_k - j0, num_tiles - l0);
                const int first = l0 + ((q - l0) % Q + Q) % Q;
                const uint32_t d_tmem = tmem_base + ((seg & 1) * Q + q) * NB;
                if (seg >= 2)
                    ok = ptx::mbar_wait_bounded(acc_free(seg & 1), ((seg >> 1) - 1) & 1, abort_word);
                uint32_t accumulate = 0;
#pragma unroll 1
                for (int l = first; l < l0 + len && ok; l += Q) {
                    const int      s      = l % S;
                    const uint32_t parity = (l / S) & 1;
                    int            ahead0 = 0, ahead1 = 0;  // offsets of tile l + kPrefetchRounds * S, read while waiting
                    if (kMmaRequests && l + kPrefetchRounds * S < num_tiles) {
                        ahead0 = __ldg(p.tile_offsets + tile_begin + l + kPrefetchRounds * S);
                        ahead1 = __ldg(p.tile_offsets + tile_begin + l + kPrefetchRounds * S + 1);
                    }
                    ok = ptx::mbar_wait_bounded(tile_full(s), parity, abort_word);
                    if (!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (kATileBytes >> 4));
                    const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(((BBUF == 2 ? parity : 0) * S + s) * (BT::kBytes >> 4));
#pragma unroll
                    for (int k = 0; k < kTileCols / 16; k++) {
                        // A: 16 k values = 32 bytes along the swizzled row; B: 16 k rows = two 8-row groups.
                        ptx::umma_f16_ss(d_tmem,
                                         a_desc + static_cast<uint64_t>((k * 32) >> 4),
                                         b_desc + static_cast<uint64_t>((TM ? k * 32 : k * 2 * BT::kGroupBytes) >> 4),
                                         idesc,
                                         k == 0 ? accumulate : 1u);
                    }
                    ptx::umma_commit(tile_free(s));
                    accumulate = 1;
                    if (BM == 2 && l + S < num_tiles)
                        load_b(l + S);
                    if (kMmaRequests)
                        request_words(ahead0, ahead1);
                }
                if (ok) {
                    if (first < l0 + len)
                        ptx::umma_commit(acc_full(seg & 1));
                    else
                        ptx::mbar_arrive(acc_full(seg & 1));
                }
                l0 += len;
            }
        }
    }
    else {
        // ------------------------------------------------------------ epilogue
        const int row_in_tile = warp * 32 + lane;
        int       seg         = 0;
        ptx::grid_dependency_wait();
        // Sum over ranks folded into this epilogue: finished rows go to this rank's partial buffer of the
        // call's parity, C is written by the sum further down.
        const bool peer_sum = !TM && p.peer.world > 0;
        uint32_t   epoch    = 0;
        float*     c32_out  = nullptr;
        if (peer_sum) {
            uint32_t previous;
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(previous) : "l"(p.peer.state) : "memory");
            epoch   = previous + 1;  // every earlier launch on this state has completed (stream order)
            c32_out = p.peer.partial[epoch & 1][p.peer.rank];
        }
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
            // The segment's result is handled in chunks of CH columns to keep registers low: the sum, in
            // warp order, of the accumulators of the MMA warps that issued for this segment.
            constexpr int CH = N < 16 ? 8 : 16;
            auto load_chunk = [&](int c, float* out) {
#pragma unroll
                for (int n = 0; n < CH; n++)
                    out[n] = 0.0f;
#pragma unroll
                for (int q = 0; q < Q; q++) {
                    if (((q - l) % Q + Q) % Q < len) {
                        float          part[CH];
                        const uint32_t taddr =
                            tmem_base + ((seg & 1) * Q + q) * NB + c * CH + (static_cast<uint32_t>(warp * 32) << 16);
                        if (CH == 8)
                            ptx::tmem_ld_x8(taddr, reinterpret_cast<uint32_t*>(part));
                        else
                            ptx::tmem_ld_x16(taddr, reinterpret_cast<uint32_t*>(part));
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int n = 0; n < CH; n++)
                            out[n] += part[n];
                    }
                }
            };
            auto store_c_chunk = [&](int c, const float* v) {
                if (TM) {
                    half* dst = p.C + static_cast<size_t>(blockIdx.y) * N * p.m + static_cast<size_t>(row_tile) * kTileRows
                                + row_in_tile;  // C[n][m]
#pragma unroll
                    for (int n = 0; n < CH; n++)
                        dst[static_cast<size_t>(c * CH + n) * p.m] = __float2half_rn(v[n]);
                    return;
                }
                if (peer_sum) {
                    // this rank's share of the sum over ranks stays in fp32 (N <= 64, one column block)
                    float4* dst32 = reinterpret_cast<float4*>(c32_out + (static_cast<size_t>(row_tile) * kTileRows + row_in_tile) * N
                                                              + c * CH);
#pragma unroll
                    for (int i = 0; i < CH / 4; i++)
                        dst32[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    return;
                }
                uint4* dst = reinterpret_cast<uint4*>(p.C + (static_cast<size_t>(row_tile) * kTileRows + row_in_tile) * p.ld
                                                      + static_cast<size_t>(blockIdx.y) * N + c * CH);
                float w[CH];
#pragma unroll
                for (int n = 0; n < CH; n++)
                    w[n] = v[n];
                if (p.addend != nullptr) {
                    // the product of the structured half of the same matrix, left in fp32 by its kernel
                    const float4* add = reinterpret_cast<const float4*>(
                        p.addend + (static_cast<size_t>(row_tile) * kTileRows + row_in_tile) * N + c * CH);
#pragma unroll
                    for (int i = 0; i < CH / 4; i++) {
                        const float4 x = __ldcg(add + i);
                        w[4 * i] += x.x;
                        w[4 * i + 1] += x.y;
                        w[4 * i + 2] += x.z;
                        w[4 * i + 3] += x.w;
                    }
                }
                v = w;
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
                    store_c_chunk(c, v);
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
                // A slot holds 128 x N floats as [N / 4 groups of four columns][128 rows] float4, so that the 32 lanes
                // of a warp (32 rows) write and read 512 contiguous bytes per instruction instead of 32 pieces of
                // 16 bytes in 32 different rows.
                float4* const slots = reinterpret_cast<float4*>(p.slots)
                                      + static_cast<size_t>(blockIdx.y) * p.slots_per_block_column * (kTileRows * N / 4);
                auto slot_of = [&](int g) { return slots + static_cast<size_t>(g + above) * (kTileRows * N / 4) + row_in_tile; };
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
                unsigned int* counter =
                    &g_row_arrivals[p.counter_set][(blockIdx.y * (p.m / kTileRows) + row_tile) * kEpilogueWarps + warp];
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
                        load_chunk(c, own);  // the accumulators are still held: read them again
#pragma unroll
                        for (int n = 0; n < CH; n++)
                            sum[n] = 0.0f;
                        // the other owners' slots, four at a time: their loads are issued together (one L2
                        // round trip per group instead of one per owner), the sums follow in owner order
#pragma unroll 1
                        for (int g0 = g_first; g0 <= g_last; g0 += 4) {
                            float4 theirs[4][CH / 4];
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                const int g = g0 + u;
                                if (g <= g_last && g != cta) {
                                    const float4* src = slot_of(g) + c * (CH / 4) * kTileRows;
#pragma unroll
                                    for (int i = 0; i < CH / 4; i++)
                                        theirs[u][i] = __ldcg(src + i * kTileRows);
                                }
                            }
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                const int g = g0 + u;
                                if (g > g_last)
                                    break;
                                if (g == cta) {
#pragma unroll
                                    for (int n = 0; n < CH; n++)
                                        sum[n] += own[n];
                                }
                                else {
#pragma unroll
                                    for (int i = 0; i < CH / 4; i++) {
                                        sum[4 * i] += theirs[u][i].x;
                                        sum[4 * i + 1] += theirs[u][i].y;
                                        sum[4 * i + 2] += theirs[u][i].z;
                                        sum[4 * i + 3] += theirs[u][i].w;
                                    }
                                }
                            }
                        }
                        store_c_chunk(c, sum);
                    }
                }
            }
            // only now may the MMA warps overwrite this accumulator set
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(acc_free(seg & 1));
            l += len;
        }
        if (peer_sum && !p.peer.partial_only && blockIdx.y == 0) {
            // Own tiles done.  When the four epilogue warps of every block of this rank have written their rows, the
            // last block to count itself tells every rank (one system-scope fence for the whole rank: fences per warp
            // and row of tiles at the end of a kernel that keeps the memory system busy cost far more).  Then the
            // blocks take rows of tiles in turn, wait for all ranks' flags -- their own rank's included -- and add
            // the partial rows in rank order.
            asm volatile("bar.sync 15, 128;" ::: "memory");
            if (warp == 0 && lane == 0) {
                // state[1]: low half counts the blocks whose rows are written, high half the blocks that have left
                // (a block without rows to add leaves while others still write, so the two counts interleave)
                __threadfence();
                if ((atomicAdd(p.peer.state + 1, 1u) & 0xffffu) == gridDim.x * gridDim.y - 1) {
                    __threadfence_system();
                    for (int r = 0; r < p.peer.world; r++)
                        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.peer.flags[r] + p.peer.rank), "r"(epoch) : "memory");
                }
            }
            const int      tiles_m = p.m / kTileRows;
            float* const* parts = p.peer.partial[epoch & 1];
            if (cta < tiles_m) {
                if (lane < p.peer.world) {
                    const uint32_t* flag  = p.peer.flags[p.peer.rank] + lane;
                    const uint64_t  start = ptx::global_timer_ns();
#pragma unroll 1
                    for (uint32_t polls = 0;; polls++) {
                        uint32_t seen;
                        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
                        if (static_cast<int32_t>(seen - epoch) >= 0 || *abort_word != 0)
                            break;
                        if ((polls & 255u) == 255u && ptx::global_timer_ns() - start > p.peer.limit_ns) {
                            *abort_word = 1;  // a rank never arrived: give up, the status word reports it
                            break;
                        }
                    }
                }
                __syncwarp();
            }
#pragma unroll 1
            for (int rt = cta; rt < tiles_m && *abort_word == 0; rt += gridDim.x) {
                const size_t row = static_cast<size_t>(rt) * kTileRows + row_in_tile;
#pragma unroll 1
                for (int c = 0; c < N / 8; c++) {
                    // eight columns at a time; all ranks' loads are issued before the first is used, so a chunk
                    // costs one NVLink round trip
                    float4 v[kMaxPeers][2];
#pragma unroll
                    for (int r = 0; r < kMaxPeers; r++)
                        if (r < p.peer.world) {  // a peer's memory, rewritten every other call: never from a cache
                            const float4* src = reinterpret_cast<const float4*>(parts[r] + row * N) + 2 * c;
                            v[r][0] = __ldcv(src);
                            v[r][1] = __ldcv(src + 1);
                        }
                    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int r = 0; r < kMaxPeers; r++)
                        if (r < p.peer.world) {
                            sum[0] += v[r][0].x, sum[1] += v[r][0].y, sum[2] += v[r][0].z, sum[3] += v[r][0].w;
                            sum[4] += v[r][1].x, sum[5] += v[r][1].y, sum[6] += v[r][1].z, sum[7] += v[r][1].w;
                        }
                    uint4    o;
                    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        oh[k] = __floats2half2_rn(sum[2 * k], sum[2 * k + 1]);
                    reinterpret_cast<uint4*>(p.C + row * N)[c] = o;
                }
            }
        }
    }

    // ---------------------------------------------------------------- exit
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word != 0)
        atomicExch(&g_device_status, static_cast<int>(kStatusWaitTimeout));
    if (threadIdx.x == 0 && p.peer.world > 0 && !p.peer.partial_only) {
        // the last block to get here advances the epoch for the next launch on this state
        uint32_t previous;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(previous) : "l"(p.peer.state) : "memory");
        __threadfence();
        // (the low half of state[1] counted the blocks when their rows were written, see the epilogue)
        if ((atomicAdd(p.peer.state + 1, 0x10000u) >> 16) == gridDim.x * gridDim.y - 1) {
            p.peer.state[1] = 0;
            __threadfence();
            p.peer.state[0] = previous + 1;
        }
    }
    if (threadIdx.x == 0 && p.peer.world > 0 && p.peer.partial_only == 2) {
        // Partial rows with the announcement: every block's rows are ordered before its count, the last block to count
        // orders all of them before the flags with one system-scope fence.  state[1] is back at zero before the
        // reduction kernel, which waits for this kernel, uses it.
        uint32_t previous;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(previous) : "l"(p.peer.state) : "memory");
        __threadfence();
        if (atomicAdd(p.peer.state + 1, 1u) == gridDim.x * gridDim.y - 1) {
            p.peer.state[1] = 0;
            __threadfence_system();
            for (int r = 0; r < p.peer.world; r++)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.peer.flags[r] + p.peer.rank), "r"(previous + 1) : "memory");
        }
    }
    if (warp == kFirstMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace spmm_b200
