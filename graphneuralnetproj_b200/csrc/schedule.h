// Host-side work partition for the decode-size SpMM kernel.
//
// The encoded matrix is a sequence of 128 x 64 tiles in (row-of-tiles, k-tile)
// order -- the order InitSparseMatrixA_API emits them, so consecutive tiles are
// contiguous in memory.  The sequence is cut into `num_ctas` contiguous chunks
// of equal length (within one tile), one chunk per thread block, instead of the
// reference's grid of (M / 256) * Split_K blocks with fixed K slices
// (csrc/SpMM_API.cu:54-58, csrc/SpMM_Kernel.cuh:307-320).  A chunk boundary
// that falls inside a row of tiles splits that row's K range between blocks;
// every piece of such a row parks an fp32 partial tile in a numbered slot of
// the caller's workspace and the last block to arrive sums the slots in a
// fixed order.
//
// Slot numbering: a piece owned by block g inside row-of-tiles r gets slot
// g + (number of split rows above r).  Pieces of one row have consecutive
// owners, a block owns at most one piece per row, and the last owner of a
// split row may also own the first piece of the next split row, hence the
// increment per split row.  Slot ids are dense: 0 .. slots_used - 1.
#pragma once

#include <cstdint>

namespace spmm_b200 {

constexpr int kMaxCtas = 304;  // two blocks per SM on 148 SMs, rounded up

struct Schedule {
    int      num_ctas;
    int      slots_used;
    int      chunk_begin[kMaxCtas + 1];  // first tile of each chunk; [num_ctas] = total tiles
    uint16_t split_rows_above[kMaxCtas];  // number of split rows above the row holding the chunk's first tile
};

// Fills `s` for exactly `ctas` blocks with boundaries rounded down to multiples of `unit` tiles.
inline void fill_schedule(Schedule& s, int tiles_m, int tiles_k, int ctas, int unit)
{
    const long total = static_cast<long>(tiles_m) * tiles_k;
    const long units = total / unit;
    s.num_ctas       = ctas;
    for (int g = 0; g <= ctas; g++)
        s.chunk_begin[g] = static_cast<int>((units * g / ctas) * unit);
    // A row is split iff a chunk boundary lies strictly inside it.  Boundaries are
    // visited in increasing order, so split rows are discovered in increasing order.
    int split_rows = 0;   // split rows discovered so far
    int last_split = -1;  // the most recent of them
    int max_slot   = -1;
    for (int g = 0; g < ctas; g++) {
        const int begin = s.chunk_begin[g], end = s.chunk_begin[g + 1];
        const int row_head = begin / tiles_k;
        if (g > 0 && begin % tiles_k != 0 && last_split != row_head) {
            last_split = row_head;
            split_rows++;
        }
        const int above       = split_rows - (last_split == row_head ? 1 : 0);
        s.split_rows_above[g] = static_cast<uint16_t>(above);
        const bool head_partial = (begin % tiles_k != 0) || (end < (row_head + 1) * tiles_k);
        if (head_partial && g + above > max_slot)
            max_slot = g + above;
        const int row_tail = (end - 1) / tiles_k;
        if (row_tail != row_head && end % tiles_k != 0) {  // a partial last piece in a later row
            const int above_tail = above + (head_partial ? 1 : 0);
            if (g + above_tail > max_slot)
                max_slot = g + above_tail;
        }
    }
    s.slots_used = max_slot + 1;
}

// Chooses the partition: as many blocks as `max_ctas` allows, reduced until the
// partial-tile slots fit into `slots_avail`; rows are never split when
// `slots_avail` is 0.  Falls back to row-aligned chunks when that balances better.
inline void make_schedule(Schedule& s, int tiles_m, int tiles_k, int max_ctas, long slots_avail)
{
    const long total = static_cast<long>(tiles_m) * tiles_k;
    if (max_ctas > kMaxCtas)
        max_ctas = kMaxCtas;
    int ctas = static_cast<int>(total < max_ctas ? total : max_ctas);
    if (ctas < 1)
        ctas = 1;
    const int aligned_ctas = tiles_m < max_ctas ? tiles_m : max_ctas;
    const long aligned_span = static_cast<long>((tiles_m + aligned_ctas - 1) / aligned_ctas) * tiles_k;
    for (; ctas >= 1; ctas--) {
        fill_schedule(s, tiles_m, tiles_k, ctas, 1);
        if (s.slots_used <= slots_avail)
            break;
    }
    const long span = ctas >= 1 ? (total + ctas - 1) / ctas : total + 1;
    if (ctas < 1 || aligned_span <= span)
        fill_schedule(s, tiles_m, tiles_k, aligned_ctas, tiles_k);
}

}  // namespace spmm_b200
