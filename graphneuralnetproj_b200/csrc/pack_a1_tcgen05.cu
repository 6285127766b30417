// Host packer for the structured (2:4) half A1 of a decomposed weight matrix, in the form the
// sm_100a sparse tensor-core instruction reads (see spmm_structured_kernel.cuh for the layout).
//
// It takes the place of the reference's InitSparseMatrixA1_Vec_Sparse_Load + inspect_metadata pair
// (csrc/SpMM_API.cu:1127-1398 and :1401-1553: value vectors with 64-bit index words, and selector
// metadata ordered for mma.sp.m16n8k16 register fragments), whose formats are tied to the Ampere
// kernel.  The 4-bit selector code of a group of four is the same in both: index of the first kept
// element | index of the second << 2 (csrc/SpMM_API.cu:1404-1416).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <cuda_fp16.h>

#include "../../include/SpMM_API.cuh"
#include "../../include/spmm_b200.h"
#include "host_threads.h"

namespace {

constexpr int kRows = 128, kCols = 128;  // logical extent of a block
constexpr int kValueBytes = kRows * kCols;  // half of the elements, two bytes each
constexpr int kMetaBytes  = kRows * 16;

inline bool kept_as_nonzero(uint16_t bits)
{
    return (bits & 0x7fffu) != 0;  // the test decompose uses: +-0 is zero, NaN is not
}

// Packs block (rb, kb).  Returns false if a group of four holds more than two nonzeros.
bool pack_block(const uint16_t* A1, int K, int rb, int kb, uint8_t* values, uint32_t* meta)
{
    memset(values, 0, kValueBytes);
    memset(meta, 0, kMetaBytes);
    for (int r = 0; r < kRows; r++) {
        const uint16_t* row = A1 + (static_cast<size_t>(rb) * kRows + r) * K + static_cast<size_t>(kb) * kCols;
        for (int g = 0; g < kCols / 4; g++) {
            int idx[2], kept = 0;
            for (int x = 0; x < 4; x++)
                if (kept_as_nonzero(row[4 * g + x])) {
                    if (kept == 2)
                        return false;
                    idx[kept++] = x;
                }
            // fewer than two nonzeros: keep the lowest unused positions as well (their values are zero)
            for (int x = 0; kept < 2; x++)
                if (kept == 0 || idx[0] != x)
                    idx[kept++] = x;
            if (idx[0] > idx[1]) {
                const int t = idx[0];
                idx[0]      = idx[1];
                idx[1]      = t;
            }
            for (int e = 0; e < 2; e++) {
                const int      c      = 2 * g + e;  // column of the kept element in the 128 x 64 value tile
                const uint32_t offset = r * 128 + (((c >> 3) ^ (r & 7)) << 4) + (c & 7) * 2;
                memcpy(values + offset, &row[4 * g + idx[e]], 2);
            }
            const uint32_t code  = static_cast<uint32_t>(idx[0] | (idx[1] << 2));
            const int      step  = g / 8;        // 32 logical k per MMA
            const int      half  = (g % 8) / 4;  // which 16 of the 32
            const int      entry = (r % 8) + 8 * half + 16 * (r / 16);
            const int      shift = 16 * ((r % 16) / 8) + 4 * (g % 4);
            meta[entry * 4 + step] |= code << shift;
        }
    }
    return true;
}

int pack_a1(const uint16_t* A1, int M, int K, void** values_out, void** meta_out)
{
    if (M <= 0 || K <= 0 || M % kRows != 0 || K % kCols != 0) {
        printf("InitSparseMatrixA1_tcgen05: M (%d) must be a positive multiple of %d and K (%d) of %d\n", M, kRows, K, kCols);
        return -1;
    }
    const long blocks_m = M / kRows, blocks_k = K / kCols, blocks = blocks_m * blocks_k;
    uint8_t*  values = static_cast<uint8_t*>(malloc(static_cast<size_t>(blocks) * kValueBytes));
    uint32_t* meta   = static_cast<uint32_t*>(malloc(static_cast<size_t>(blocks) * kMetaBytes));
    if (values == nullptr || meta == nullptr) {
        printf("InitSparseMatrixA1_tcgen05: Error in malloc memory from host memory!\n");
        exit(-1);
    }
    int bad = 0;
    spmm_b200::parallel_for(blocks, [&](long b0, long b1) {
        for (long b = b0; b < b1; b++)
            if (!pack_block(A1, K, static_cast<int>(b / blocks_k), static_cast<int>(b % blocks_k),
                            values + static_cast<size_t>(b) * kValueBytes, meta + static_cast<size_t>(b) * (kMetaBytes / 4)))
                __atomic_store_n(&bad, 1, __ATOMIC_RELAXED);
    });
    if (bad) {
        printf("InitSparseMatrixA1_tcgen05: a group of four consecutive elements holds more than two nonzeros\n");
        free(values);
        free(meta);
        return -1;
    }
    *values_out = values;
    *meta_out   = meta;
    return static_cast<int>(blocks);
}

}  // namespace

__host__ int InitSparseMatrixA1_tcgen05(half* A1_h, int M, int K, half** Values, int** Metadata)
{
    return pack_a1(reinterpret_cast<const uint16_t*>(A1_h), M, K, reinterpret_cast<void**>(Values),
                   reinterpret_cast<void**>(Metadata));
}

extern "C" int spmm_b200_pack_a1(const uint16_t* A1, int M, int K, void** values, void** metadata)
{
    return pack_a1(A1, M, K, values, metadata);
}
