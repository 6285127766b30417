// Prefill-size "load-as-sparse, compute-as-dense" SpMM on pairs of SMs: C[M][N] = A * B for N a multiple
// of 256 (beyond the reference's N <= 64, csrc/SpMM_API.cu:105-196), A in tiled-CSL.
//
// At these widths the single-block kernel (spmm_decode_kernel.cuh) is bound by shared-memory bandwidth
// -- per restored tile and 256 columns the decoders spend about 450 wavefronts and the tensor core
// reads 128 (A) + 256 (B) -- and by the B slices it pulls out of L2 (32 KB per tile and 256 columns).
// Here two blocks on neighbouring SMs (a cluster of two) work on 256 rows together with
// tcgen05.mma.cta_group::2, M = 256:
//   - each block restores the tiles of its own 128 rows (rows 256 * pr + 128 * rank ...) into its own
//     shared memory, exactly as the single-block kernel does;
//   - each block stages only half of the columns of a B slice (128 of every 256); the pair MMA reads
//     both halves, so the B traffic per block out of L2 and out of shared memory halves;
//   - with NM = 2 a restored tile serves 512 columns (two MMAs of 256 columns per k step), so it is
//     decoded once per 512 columns instead of once per 256.  The accumulators then fill the 512 TMEM
//     columns and the epilogue of a row no longer overlaps the next row (about 2 % at K = 12288).
// Per block and restored tile at NM = 2: 450 (decode) + 2 * (128 + 128) (operands) = 962 wavefronts for
// 1024 cycles of MMA, against 450 + 384 = 834 for 512 cycles in the single-block kernel.  Measured on
// 12288 x 12288 at 80 % sparsity (workspace for Split_K = 8): 71 / 129 / 217 / 403 us at N = 256 / 512 /
// 1024 / 2048 against 87 / 147 / 290 / 543 us for the single-block kernel.
//
// Roles per block: warps 0..3 epilogue; warp 4 allocates TMEM and, in the even block (the leader),
// issues the pair MMAs; warp 5 issues the tiled TMA loads of the block's half of the B slices, buffer
// by buffer as they come free; warps 6.. are D decoder warps.  Synchronisation across the pair: the
// "ready" barrier of a tile lives in the leader; the partner's decoder arrives on it at cluster scope and
// the partner's TMA loads count their bytes on it (cp.async.bulk.tensor with .cta_group::2), so the MMA
// lane waits once per tile (a lane in the partner that forwarded its block's readiness was measured to
// take 0.6 us per tile, more than the MMAs of a tile); the leader's tcgen05.commit arrives on the
// "done" / acc_full barriers of both blocks (one commit per block, the second through the cluster-window
// address of the partner's barrier); the partner's epilogue warps arrive on the leader's acc_free
// barrier.  Every wait is bounded; a block that gives up still reaches the cluster barrier at the end,
// so its partner never waits for it without limit.
#pragma once

#include "spmm_decode_kernel.cuh"

namespace spmm_b200 {

constexpr int kPairColsPerMma = 256;  // columns of one pair MMA; each block stages half of them

// SA buffers for restored tiles of A, SB buffers for this block's half of a B slice (NM * 16 KB each)
template<int NM, int SA, int SB>
constexpr int pair_smem_bytes()
{
    return 1024 + SA * kATileBytes + SB * NM * BTile<kPairColsPerMma / 2>::kBytes + 512;
}

template<int D>
constexpr int pair_threads()
{
    return (kFirstMmaWarp + 2 + D) * 32;
}

// Adds the parked partial rows of one output row -- `owners` slots, 2 * slot4 float4 apart, in owner order -- and
// writes the fp16 result: the chunks first, first + step, ... of 16 columns.  `parked` points at the row's float4 in
// the first owner's slot (slots are [NBLK / 4][128 rows] float4); four owners' loads are in flight together.
// TM: token-major results, C[n][m]: `c_row` then points at (row, first column of the block) and a column is
// `m_stride` halves further.
template<int NBLK, int TM>
__device__ __forceinline__ void
sum_parked_row(const float4* parked, size_t slot4, int owners, half* c_row, size_t m_stride, int first, int step)
{
    constexpr int CH = 16;
#pragma unroll 1
    for (int c = first; c < NBLK / CH; c += step) {
        float sum[CH];
#pragma unroll
        for (int n = 0; n < CH; n++)
            sum[n] = 0.0f;
#pragma unroll 1
        for (int k0 = 0; k0 < owners; k0 += 4) {
            float4 part[4][CH / 4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (k0 + u < owners) {
                    const float4* src = parked + static_cast<size_t>(k0 + u) * 2 * slot4 + c * (CH / 4) * kTileRows;
#pragma unroll
                    for (int i = 0; i < CH / 4; i++)
                        part[u][i] = __ldcg(src + i * kTileRows);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (k0 + u >= owners)
                    break;
#pragma unroll
                for (int i = 0; i < CH / 4; i++) {
                    sum[4 * i] += part[u][i].x;
                    sum[4 * i + 1] += part[u][i].y;
                    sum[4 * i + 2] += part[u][i].z;
                    sum[4 * i + 3] += part[u][i].w;
                }
            }
        }
        if (TM) {
#pragma unroll
            for (int n = 0; n < CH; n++)
                c_row[static_cast<size_t>(c * CH + n) * m_stride] = __float2half_rn(sum[n]);
            continue;
        }
        uint4* dst = reinterpret_cast<uint4*>(c_row + c * CH);
#pragma unroll
        for (int i = 0; i < CH / 8; i++) {
            __half2 h0 = __floats2half2_rn(sum[8 * i], sum[8 * i + 1]);
            __half2 h1 = __floats2half2_rn(sum[8 * i + 2], sum[8 * i + 3]);
            __half2 h2 = __floats2half2_rn(sum[8 * i + 4], sum[8 * i + 5]);
            __half2 h3 = __floats2half2_rn(sum[8 * i + 6], sum[8 * i + 7]);
            uint4   o;
            o.x    = *reinterpret_cast<uint32_t*>(&h0);
            o.y    = *reinterpret_cast<uint32_t*>(&h1);
            o.z    = *reinterpret_cast<uint32_t*>(&h2);
            o.w    = *reinterpret_cast<uint32_t*>(&h3);
            dst[i] = o;
        }
    }
}

// What the last arriver of the chunk's final row leaves for the whole block to sum on the way out.
struct PendingSum {
    int mask;        // quarters (epilogue warps) of the row of tiles whose sum is pending
    int row_tile;    // the row of tiles
    int first_slot;  // this block's slot of the first owner
    int owners;
};

// NM  : pair MMAs per k step = 256-column blocks served by one restored tile (1 or 2); the cluster
//       handles NM * 256 columns (blockIdx.y selects which)
// D   : decoder warps (tile l of the chunk is restored by warp l % D into A buffer l % SA), each holding
//       VPL 4-word vectors per lane -- the decode-size kernel's arrangement; with three to six decoders
//       and more B buffers instead the kernel was measured 0-25 % slower
// SA, SB: ring of A buffers and, separately, of B buffers (tile l uses B buffer l % SB): the B halves are
//       NM times larger than a restored tile, so fewer of them fit
//       p.sched partitions (M / 256) rows of tile pairs x (K / 64) among the clusters;
//       p.slots_per_block_column counts slots of 128 x (NM * 256) floats, two per schedule slot.
// TM  : 1 = token-major activations and results, B[N][K] and C[N][M] (the FasterTransformer caller's layout,
//       third_party/ft.patch:2822-2846): a block's half of a B slice is then 128 tokens x 64 k values, K-contiguous,
//       one TMA box in the 128-byte-swizzle layout the restored A tiles have
template<int NM, int D, int VPL, int SA, int SB, int TM>
__global__ void __launch_bounds__(pair_threads<D>(), 1)
spmm_pair_kernel(const __grid_constant__ DecodeParams p)
{
    constexpr int NBLK = NM * kPairColsPerMma;  // columns per cluster
    constexpr int ACC  = 2 / NM;                // accumulator sets of NBLK columns in the 512 TMEM columns
    using BT           = BTile<kPairColsPerMma / 2>;  // this block's half of a 64 x 256 slice: two 64-column atoms
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base    = smem_base;
    const uint32_t b_base    = a_base + SA * kATileBytes;
    const uint32_t bar_base  = b_base + SB * NM * BT::kBytes;
    // barriers (8 bytes each): per tile "ready" (the leader's: both blocks' tiles are restored and both B halves
    // have landed) and "done" (the pair MMAs that read the tile's A and B buffers have completed); then accumulators
    // full x2, free x2 (leader's).  One wait and two commits per tile for the MMA lane: its time per tile, not the
    // tensor core's, bounded an earlier form with more barriers.  Both kinds form a ring of R = max(SA, SB) entries
    // indexed by the tile (l % R): the decoder of tile l waits for the MMAs of tile l - SA (its A buffer), the
    // loader for those of tile l - SB (its B buffer).
    constexpr int R = SA > SB ? SA : SB;
    auto ready    = [&](int s) { return bar_base + 8u * s; };
    auto done     = [&](int s) { return bar_base + 8u * (R + s); };
    auto acc_full = [&](int b) { return bar_base + 8u * (2 * R + b); };
    auto acc_free = [&](int b) { return bar_base + 8u * (2 * R + 2 + b); };
    const uint32_t tmem_slot_addr = bar_base + 8u * (2 * R + 4);
    uint8_t*       smem_generic   = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
    volatile uint32_t* tmem_slot  = reinterpret_cast<volatile uint32_t*>(smem_generic + (tmem_slot_addr - smem_base));
    volatile int*      abort_word = reinterpret_cast<volatile int*>(smem_generic + (tmem_slot_addr + 4 - smem_base));
    PendingSum* const  pending    = reinterpret_cast<PendingSum*>(smem_generic + (bar_base + 384 - smem_base));
    static_assert(8 * (2 * R + 4) + 8 <= 384, "barrier block");
    static_assert(SA >= D, "every decoder warp needs a buffer of its own to start with");
    static_assert(NM == 1 || NM == 2, "one or two 256-column MMAs per k step");

    const int      warp    = threadIdx.x >> 5;
    const int      lane    = threadIdx.x & 31;
    const uint32_t rank    = ptx::cluster_cta_rank();  // 0: leader (issues the MMAs), 1: its partner
    const int      cluster = blockIdx.x >> 1;

    const int tile_begin = p.sched.chunk_begin[cluster];  // in units of tile pairs: (row of pairs, k tile)
    const int tile_end   = p.sched.chunk_begin[cluster + 1];
    const int num_tiles  = tile_end - tile_begin;
    const int tiles_k    = p.tiles_k;
    // Tile `l` of the chunk is pair tile t = tile_begin + l = (pr, j); this block's tile of it is tile
    // (2 pr + rank, j) of the encoded sequence.
    auto tile_index = [&](int l) {
        const int t = tile_begin + l;
        return t + (t / tiles_k + static_cast<int>(rank)) * tiles_k;
    };
    // Where output row `row` of row of tiles `rt` starts in this cluster's columns: C[m][n] row-major, or C[n][m]
    // (TM), where the next column is p.m halves further.
    auto c_origin = [&](int rt, int row) {
        const size_t m_index = static_cast<size_t>(rt) * kTileRows + row, n0 = static_cast<size_t>(blockIdx.y) * NBLK;
        return TM ? p.C + n0 * p.m + m_index : p.C + m_index * p.ld + n0;
    };
    constexpr int kLoaderWarp      = kFirstMmaWarp + 1;
    constexpr int kFirstDecodeWarp = kFirstMmaWarp + 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < R; s++) {
            ptx::mbar_init(ready(s), 3);  // the leader's: both blocks' decoders and the leader's loader (+ both halves' bytes)
            ptx::mbar_init(done(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            ptx::mbar_init(acc_full(b), 1);
            ptx::mbar_init(acc_free(b), 2 * kEpilogueWarps);
        }
        *abort_word   = 0;
        pending->mask = 0;
        ptx::mbar_init_fence();
    }
    for (uint32_t off = threadIdx.x * 16u; off < static_cast<uint32_t>(SA * kATileBytes + SB * NM * BT::kBytes); off += blockDim.x * 16u)
        ptx::st_shared_zero_128(a_base + off);
    if (warp == kFirstMmaWarp) {
        ptx::tmem_alloc_pair(tmem_slot_addr, 512);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();  // both blocks' barriers exist before anyone arrives on the partner's
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    ptx::grid_launch_dependents();

    if (warp >= kFirstDecodeWarp) {
        // ------------------------------------------------------------ decoder warp (see spmm_decode_kernel)
        const int      s_own         = warp - kFirstDecodeWarp;  // this warp's first tile and first A buffer
        const uint32_t leader_ready0 = ptx::map_to_cta(ready(0), 0);
        uint32_t       slot          = s_own;
        uint4          r[VPL];
        int            nvec = 0, next0 = 0, next1 = 0;
        auto load_words = [&](const uint4* from, int count) {
            if (count <= 0)
                return;
#pragma unroll
            for (int v = 0; v < VPL; v++)
                r[v] = ptx::ld_stream_128(from + (min(lane + v * 32, count - 1) - lane));
        };
        auto scatter_batch = [&](uint8_t* tile, int count) {
#pragma unroll
            for (int v = 0; v < VPL; v++)
                scatter_vector(tile, r[v], lane + v * 32 < count);
        };
        auto request_words = [&](int l) {  // this block's words of chunk tile l into L2, ahead of their turn
            if (lane == 0 && l < num_tiles) {
                const int i    = tile_index(l);
                const int off0 = __ldg(p.tile_offsets + i), off1 = __ldg(p.tile_offsets + i + 1);
                if (off1 > off0)
                    ptx::bulk_prefetch_l2(p.words + off0, static_cast<uint32_t>(off1 - off0) * 16u);
            }
        };
        const uint4* src = p.words + lane;
        if (!p.weights_early)
            ptx::grid_dependency_wait();
        if (s_own < num_tiles) {
            const int i    = tile_index(s_own);
            const int off0 = __ldg(p.tile_offsets + i), off1 = __ldg(p.tile_offsets + i + 1);
            nvec           = off1 - off0;
            src            = p.words + off0 + lane;
            load_words(src, nvec);
            if (s_own + D < num_tiles) {
                const int in = tile_index(s_own + D);
                next0        = __ldg(p.tile_offsets + in);
                next1        = __ldg(p.tile_offsets + in + 1);
            }
            request_words(s_own + D);
            request_words(s_own + 2 * D);
        }
        ptx::grid_dependency_wait();
#pragma unroll 1
        for (int l = s_own; l < num_tiles; l += D) {
            const bool     has_next = l + D < num_tiles;
            const int      before   = l - SA;  // the tile that used this A buffer last
            uint8_t* const a_tile   = smem_generic + slot * kATileBytes;
            request_words(l + 3 * D);
            if (before >= 0) {
                if (!ptx::mbar_wait_bounded_cluster(done(before % R), (before / R) & 1, abort_word))
                    break;
#pragma unroll
                for (int i = 0; i < kATileBytes / (32 * 16); i++)
                    ptx::st_shared_zero_128(a_base + slot * kATileBytes + lane * 16u + i * 512u);
                __syncwarp();  // the whole buffer is clear before any lane scatters into it
            }
            scatter_batch(a_tile, nvec);
#pragma unroll 1
            for (int held = VPL * 32; held < nvec; held += VPL * 32) {  // tiles denser than the register budget
                load_words(src + held, nvec - held);
                scatter_batch(a_tile, nvec - held);
            }
            if (has_next) {
                nvec = next1 - next0;
                src  = p.words + next0 + lane;
                load_words(src, nvec);
                if (l + 2 * D < num_tiles) {
                    const int in = tile_index(l + 2 * D);
                    next0        = __ldg(p.tile_offsets + in);
                    next1        = __ldg(p.tile_offsets + in + 1);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0)
                    ptx::mbar_arrive(ready(l % R));
                else
                    ptx::mbar_arrive_cluster(leader_ready0 + 8u * (l % R));
            }
            slot += D;
            if (slot >= SA)
                slot -= SA;
        }
    }
    else if (warp == kLoaderWarp) {
        // ------------------------------------------------------------ B loader: this block's half of every slice
        // Columns [rank * 128, rank * 128 + 128) of each of the cluster's 256-column blocks, 64 k rows, as boxes
        // of 64 columns; a slot's B buffers are refilled as soon as the pair MMAs that read them have completed.
        ptx::grid_dependency_wait();
        if (lane == 0) {
            const uint32_t leader_ready0 = ptx::map_to_cta(ready(0), 0);
            int j = tile_begin % tiles_k;
#pragma unroll 1
            for (int l = 0; l < num_tiles; l++) {
                // B buffer l % SB was last read by tile l - SB: wait for that tile's MMAs
                const int s = l % SB;
                if (l >= SB && !ptx::mbar_wait_bounded_cluster(done((l - SB) % R), ((l - SB) / R) & 1, abort_word))
                    break;
                // the bytes of both halves are counted on the leader's barrier, announced by the leader's loader
                const uint32_t bar = leader_ready0 + 8u * (l % R);
                if (rank == 0)
                    ptx::mbar_arrive_expect_tx(ready(l % R), 2 * NM * BT::kBytes);
#pragma unroll
                for (int m = 0; m < NM; m++) {
                    const int col0 = static_cast<int>(blockIdx.y) * NBLK + m * kPairColsPerMma + static_cast<int>(rank) * (kPairColsPerMma / 2);
                    if (TM)  // B[N][K]: x = k, y = token; one box of 64 k values x 128 tokens
                        ptx::tma_load_2d_pair(b_base + (s * NM + m) * BT::kBytes, &p.b_map, j * kTileCols, col0, bar);
                    else
#pragma unroll
                        for (int a = 0; a < BT::kAtoms; a++)
                            ptx::tma_load_2d_pair(b_base + (s * NM + m) * BT::kBytes + a * BT::kAtomBytes, &p.b_map,
                                                  col0 + a * BT::kAtomCols, j * kTileCols, bar);
                }
                if (++j == tiles_k)
                    j = 0;
            }
        }
    }
    else if (warp == kFirstMmaWarp) {
        ptx::grid_dependency_wait();
        if (lane == 0 && rank == 0) {
            // ------------------------------------------------------------ leader: MMA issue for the pair
            constexpr uint32_t idesc   = ptx::make_idesc_f16_f32(2 * kTileRows, kPairColsPerMma, false, TM ? false : true);
            const uint64_t     a_desc0 = ptx::make_smem_desc(a_base, 16, 1024, ptx::kSwizzle128B);
            const uint64_t     b_desc0 = TM ? ptx::make_smem_desc(b_base, 16, 1024, ptx::kSwizzle128B)
                                            : ptx::make_smem_desc(b_base, BT::kLeadingBytes, BT::kGroupBytes, BT::kSwizzleMode);
            const uint32_t     partner_done0     = ptx::map_to_cta(done(0), 1);
            const uint32_t     partner_acc_full0 = ptx::map_to_cta(acc_full(0), 1);
            bool ok  = true;
            int  seg = 0;
#pragma unroll 1
            for (int l0 = 0; l0 < num_tiles && ok; ++seg) {
                const int j0  = (tile_begin + l0) % tiles_k;
                const int len = min(tiles_k - j0, num_tiles - l0);
                const int set = seg % ACC, use = seg / ACC;
                const uint32_t d_tmem = tmem_base + set * NBLK;
                if (use >= 1)
                    ok = ptx::mbar_wait_bounded_cluster(acc_free(set), (use - 1) & 1, abort_word);
                uint32_t accumulate = 0;
#pragma unroll 1
                for (int l = l0; l < l0 + len && ok; l++) {
                    const int      sa = l % SA, sb = l % SB, e = l % R;
                    const uint32_t parity = (l / R) & 1;
                    ok = ptx::mbar_wait_bounded_cluster(ready(e), parity, abort_word);
                    if (!ok)
                        break;
                    ptx::tc_fence_after_sync();
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(sa * (kATileBytes >> 4));
#pragma unroll
                    for (int k = 0; k < kTileCols / 16; k++) {
#pragma unroll
                        for (int m = 0; m < NM; m++) {
                            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((sb * NM + m) * (BT::kBytes >> 4));
                            ptx::umma_f16_ss_pair(d_tmem + m * kPairColsPerMma,
                                                  a_desc + static_cast<uint64_t>((k * 32) >> 4),
                                                  b_desc + static_cast<uint64_t>((TM ? k * 32 : k * 2 * BT::kGroupBytes) >> 4),
                                                  idesc,
                                                  k == 0 ? accumulate : 1u);
                        }
                    }
                    ptx::umma_commit_pair(done(e));
                    ptx::umma_commit_pair(partner_done0 + 8u * e);
                    accumulate = 1;
                }
                if (ok) {
                    ptx::umma_commit_pair(acc_full(set));
                    ptx::umma_commit_pair(partner_acc_full0 + 8u * set);
                }
                l0 += len;
            }
        }
    }
    else {
        // ------------------------------------------------------------ epilogue: this block's 128 rows x NBLK columns
        const int      row_in_tile      = warp * 32 + lane;
        const uint32_t leader_acc_free0 = ptx::map_to_cta(acc_free(0), 0);
        int            seg              = 0;
        ptx::grid_dependency_wait();
        constexpr int CH = 16;
#pragma unroll 1
        for (int l = 0; l < num_tiles; ++seg) {
            const int  t0       = tile_begin + l;
            const int  pair_row = t0 / tiles_k;
            const int  row_tile = 2 * pair_row + static_cast<int>(rank);
            const int  j0       = t0 % tiles_k;
            const int  len      = min(tiles_k - j0, num_tiles - l);
            const bool whole    = (j0 == 0) && (len == tiles_k);
            const int  set = seg % ACC, use = seg / ACC;
            if (!warp_wait(acc_full(set), use & 1, abort_word, lane))
                break;
            ptx::tc_fence_after_sync();
            auto load_chunk = [&](int c, float* out) {
                ptx::tmem_ld_x16(tmem_base + set * NBLK + c * CH + (static_cast<uint32_t>(warp * 32) << 16),
                                 reinterpret_cast<uint32_t*>(out));
                ptx::tmem_ld_wait();
            };
            auto store_c_chunk = [&](int c, const float* v) {
                if (TM) {
                    half* dst = c_origin(row_tile, row_in_tile);  // C[n][m]
#pragma unroll
                    for (int n = 0; n < CH; n++)
                        dst[static_cast<size_t>(c * CH + n) * p.m] = __float2half_rn(v[n]);
                    return;
                }
                uint4* dst = reinterpret_cast<uint4*>(c_origin(row_tile, row_in_tile) + c * CH);
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
                for (int c = 0; c < NBLK / CH; c++) {
                    float v[CH];
                    load_chunk(c, v);
                    store_c_chunk(c, v);
                }
            }
            else {
                // A row of pairs whose K range is shared between clusters: park the partial rows, count arrivals
                // per row of tiles, the last arriver adds the owners' slots in owner order (as in spmm_decode_kernel;
                // an owner is a cluster, and each of its two blocks has a slot of its own).
                const int  head_row  = tile_begin / tiles_k;
                const bool head_part = (tile_begin % tiles_k != 0) || (tile_end < (head_row + 1) * tiles_k);
                const int  above     = p.sched.split_rows_above[cluster] + ((pair_row != head_row && head_part) ? 1 : 0);
                int        g_first = cluster, g_last = cluster;
                while (p.sched.chunk_begin[g_first] > pair_row * tiles_k)
                    g_first--;
                while (p.sched.chunk_begin[g_last + 1] < (pair_row + 1) * tiles_k)
                    g_last++;
                float* const slots = p.slots + static_cast<size_t>(blockIdx.y) * p.slots_per_block_column * (kTileRows * NBLK);
                // A slot holds 128 x NBLK floats as [NBLK / 4 groups of four columns][128 rows] float4: the 32 lanes
                // of a warp (32 rows) write and read 512 contiguous bytes per instruction.  (Row-major slots made
                // every store 32 partial sectors and the tail of a launch tens of microseconds long.)
                auto slot_of = [&](int g) {
                    return reinterpret_cast<float4*>(slots) + (static_cast<size_t>(g + above) * 2 + rank) * (kTileRows * NBLK / 4)
                           + row_in_tile;
                };
                float4* const mine = slot_of(cluster);
#pragma unroll 1
                for (int c = 0; c < NBLK / CH; c++) {
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
                // The partial rows are parked, so the accumulators are free: the leader may start the next row of
                // tiles while the last arriver adds the owners' slots -- its own included -- out of memory.
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive_cluster(leader_acc_free0 + 8u * set);
                if (arrived == static_cast<unsigned int>(g_last - g_first)) {
                    if (lane == 0)
                        *counter = 0;
                    __threadfence();
                    const int first_slot = (g_first + above) * 2 + static_cast<int>(rank);
                    if (l + len == num_tiles) {
                        // the chunk's final row: nothing is left to overlap with, so all warps of the block share the
                        // sum on the way out (one warp per quarter would make 32 L2 round trips in a row)
                        if (lane == 0) {
                            pending->row_tile   = row_tile;
                            pending->first_slot = first_slot;
                            pending->owners     = g_last - g_first + 1;
                            atomicOr(&pending->mask, 1 << warp);
                        }
                    }
                    else
                        sum_parked_row<NBLK, TM>(reinterpret_cast<const float4*>(slots)
                                                     + static_cast<size_t>(first_slot) * (kTileRows * NBLK / 4) + row_in_tile,
                                                 kTileRows * NBLK / 4, g_last - g_first + 1, c_origin(row_tile, row_in_tile), p.m, 0, 1);
                }
                l += len;
                continue;
            }
            // only now may the leader overwrite this accumulator set (in both blocks)
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive_cluster(leader_acc_free0 + 8u * set);
            l += len;
        }
    }

    // ---------------------------------------------------------------- exit
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word != 0)
        atomicExch(&g_device_status, static_cast<int>(kStatusWaitTimeout));
    if (const int mask = *reinterpret_cast<volatile int*>(&pending->mask)) {
        const float4* slots4 = reinterpret_cast<const float4*>(p.slots)
                               + static_cast<size_t>(blockIdx.y) * p.slots_per_block_column * (kTileRows * NBLK / 4);
        for (int quarter = 0; quarter < kEpilogueWarps; quarter++)
            if ((mask >> quarter) & 1) {
                const int row = quarter * 32 + lane;
                sum_parked_row<NBLK, TM>(slots4 + static_cast<size_t>(pending->first_slot) * (kTileRows * NBLK / 4) + row,
                                         kTileRows * NBLK / 4, pending->owners, c_origin(pending->row_tile, row), p.m, warp,
                                         static_cast<int>(blockDim.x) / 32);
            }
    }
    // Neither block leaves while its partner may still arrive on its barriers or the leader's MMAs may
    // still read its shared memory (a block that gave up gets here too).
    ptx::cluster_sync_all();
    if (warp == kFirstMmaWarp) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace spmm_b200
