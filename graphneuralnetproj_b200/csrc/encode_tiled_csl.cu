// Host encoders: dense fp16 -> tiled-CSL, bit-identical to the reference's
// InitSparseMatrixA_API (csrc/SpMM_API.cu:241-438) and
// InitSparseMatrixA_API_NoReorder (:441-567), plus the file front end
// GenSparseMatrixBinFile (:1565-1620).
//
// The reference builds 32 per-bank stacks and then, once per emitted word,
// scans all 32 for the fullest one.  That scan has a closed form: "pop the
// fullest stack, lowest index first" visits the stacks level by level -- first
// every stack of the maximal height H in index order, then every stack that
// now has height H-1, and so on -- so the pop sequence is
//     for h = H..1: for b = 0..31: if height[b] >= h: take stack[b][h-1].
// The lane-interleaved LIFO emission (:406-424) is likewise a fixed
// permutation of that sequence.  Both are applied directly here, one tile per
// task, tiles spread over host threads; offsets come from a prefix sum over
// per-tile counts, so the output does not depend on the thread count.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <thread>
#include <vector>

#include "../../include/SpMM_API.cuh"
#include "host_threads.h"

namespace {

constexpr int kTileM = 128;  // rows per encoded tile      (csrc/SpMM_API.cu:249)
constexpr int kTileK = 64;   // columns per encoded tile   (csrc/TilingConfig.h:29)
constexpr int kVec   = 4;    // words per vector           (csrc/SpMM_API.cu:250)
constexpr int kBanks = 32;
constexpr int kBankCap = kTileM * kTileK / kBanks + kVec;  // 256 slots per bank + padding words

// fabs(__half2float(v)) > 0: everything except +-0 and NaN.
inline bool is_nonzero(uint16_t bits)
{
    return static_cast<uint16_t>((bits & 0x7fffu) - 1u) < 0x7c00u;
}

inline uint32_t pack_word(uint16_t value, int position)
{
    return static_cast<uint32_t>(value) | (static_cast<uint32_t>(position) << 16);
}

int count_tile(const uint16_t* tile, int ld)
{
    int nnz = 0;
    for (int m = 0; m < kTileM; m++) {
        const uint16_t* row = tile + static_cast<size_t>(m) * ld;
        for (int n = 0; n < kTileK; n++)
            nnz += is_nonzero(row[n]);
    }
    return nnz;
}

// Encodes one tile into out[0 .. padded_count).
void encode_tile_reordered(const uint16_t* tile, int ld, int padded_count, uint32_t* out, uint32_t* bank_items,
                           uint32_t* pops)
{
    int height[kBanks];
    int first_zero[kBanks];
    for (int b = 0; b < kBanks; b++) {
        height[b]     = 0;
        first_zero[b] = -1;
    }
    int count = 0;
    for (int m = 0; m < kTileM; m++) {
        const uint16_t* row  = tile + static_cast<size_t>(m) * ld;
        const int       mask = (m & 7) << 3;
        for (int n = 0; n < kTileK; n++) {
            const int cp   = n ^ mask;
            const int bank = (cp >> 1) & 31;
            const int pos  = m * kTileK + cp;
            if (is_nonzero(row[n])) {
                bank_items[bank * kBankCap + height[bank]++] = pack_word(row[n], pos);
                count++;
            }
            else if (first_zero[bank] < 0) {
                first_zero[bank] = pos;
            }
        }
    }
    // Padding words go to the emptiest bank (lowest index on ties) and point at that bank's first zero.
    while (count < padded_count) {
        int b = 0;
        for (int i = 1; i < kBanks; i++)
            if (height[i] < height[b])
                b = i;
        bank_items[b * kBankCap + height[b]++] = pack_word(0, first_zero[b]);
        count++;
    }
    // Pop sequence, level by level.
    int top = 0;
    for (int b = 0; b < kBanks; b++)
        top = height[b] > top ? height[b] : top;
    int np = 0;
    for (int h = top; h >= 1; h--)
        for (int b = 0; b < kBanks; b++)
            if (height[b] >= h)
                pops[np++] = bank_items[b * kBankCap + h - 1];
    // Emission permutation.
    const int vectors = count / kVec;
    const int repeat  = vectors / 32;
    const int rem     = vectors % 32;
    uint32_t* tail    = out + repeat * 128;
    for (int k = 0; k < kVec * rem; k++) {
        const int v = k / rem, b = k % rem;
        tail[b * kVec + (kVec - 1 - v)] = pops[k];
    }
    const uint32_t* main_pops = pops + kVec * rem;
    const int       steps     = repeat * kVec;
    for (int s = 0; s < steps; s++) {
        const int       e   = steps - 1 - s;  // emitted in reverse order of filling
        uint32_t*       dst = out + (e / kVec) * 128 + (e % kVec);
        const uint32_t* src = main_pops + s * 32;
        for (int b = 0; b < 32; b++)
            dst[b * kVec] = src[b];
    }
}

void encode_tile_scan_order(const uint16_t* tile, int ld, int pad, uint32_t* out)
{
    int n_out = 0;
    for (int m = 0; m < kTileM; m++) {
        const uint16_t* row  = tile + static_cast<size_t>(m) * ld;
        const int       mask = (m & 7) << 3;
        for (int n = 0; n < kTileK; n++) {
            const int pos = m * kTileK + (n ^ mask);
            if (is_nonzero(row[n])) {
                out[n_out++] = pack_word(row[n], pos);
            }
            else if (pad > 0) {
                pad--;
                out[n_out++] = pack_word(row[n], pos);  // the element's own bits, as the reference stores them
            }
        }
    }
}

int encode_matrix(const uint16_t* A, int M, int K, uint32_t** words_out, int** offsets_out, bool reorder)
{
    if (M % kTileM != 0 || K % kTileK != 0) {
        fprintf(stderr, "InitSparseMatrixA: M (%d) must be a multiple of %d and K (%d) of %d\n", M, kTileM, K, kTileK);
        abort();
    }
    const int  tiles_m = M / kTileM, tiles_k = K / kTileK;
    const long tiles   = static_cast<long>(tiles_m) * tiles_k;
    int*       offsets = static_cast<int*>(malloc((tiles + 2) * sizeof(int)));
    if (!offsets) {
        printf("InitSparseMatrixA: Error in malloc memory from host memory!\n");
        exit(-1);
    }
    std::vector<int> padded(tiles);
    std::vector<int> padding(tiles);
    spmm_b200::parallel_for(tiles, [&](long t0, long t1) {
        for (long t = t0; t < t1; t++) {
            const uint16_t* tile = A + static_cast<size_t>(t / tiles_k) * kTileM * K + (t % tiles_k) * kTileK;
            const int       nnz  = count_tile(tile, K);
            padding[t]           = (kVec - nnz % kVec) % kVec;
            padded[t]            = nnz + padding[t];
        }
    });
    long total = 0;
    offsets[0] = 0;
    for (long t = 0; t < tiles; t++) {
        total += padded[t];
        offsets[t + 1] = static_cast<int>(total / kVec);
    }
    offsets[tiles + 1] = static_cast<int>(total / kVec);
    uint32_t* words    = static_cast<uint32_t*>(malloc(total > 0 ? total * sizeof(uint32_t) : sizeof(uint32_t)));
    if (!words) {
        printf("InitSparseMatrixA: Error in malloc memory from host memory!\n");
        exit(-1);
    }
    spmm_b200::parallel_for(tiles, [&](long t0, long t1) {
        std::vector<uint32_t> bank_items(kBanks * kBankCap);
        std::vector<uint32_t> pops(kTileM * kTileK + kVec);
        for (long t = t0; t < t1; t++) {
            const uint16_t* tile = A + static_cast<size_t>(t / tiles_k) * kTileM * K + (t % tiles_k) * kTileK;
            uint32_t*       out  = words + static_cast<size_t>(offsets[t]) * kVec;
            if (reorder)
                encode_tile_reordered(tile, K, padded[t], out, bank_items.data(), pops.data());
            else
                encode_tile_scan_order(tile, K, padding[t], out);
        }
    });
    *words_out   = words;
    *offsets_out = offsets;
    return static_cast<int>(tiles + 2);
}

}  // namespace

__host__ int InitSparseMatrixA_API(half* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    (void)N;
    return encode_matrix(reinterpret_cast<const uint16_t*>(A_h), M, K, Compressed_A, TileOffsets, true);
}

__host__ int
InitSparseMatrixA_API_NoReorder(half* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    (void)N;
    return encode_matrix(reinterpret_cast<const uint16_t*>(A_h), M, K, Compressed_A, TileOffsets, false);
}

extern "C" void GenSparseMatrixBinFile(char* DenseMatrixFileName,
                                       int   M,
                                       int   K,
                                       char* NZWeightsFileName,
                                       char* TileOffsetsFileName,
                                       char* OutputSizesFileName)
{
    const size_t          want = sizeof(uint16_t) * static_cast<size_t>(M) * K;
    std::vector<uint16_t> dense(static_cast<size_t>(M) * K);
    std::ifstream         in(DenseMatrixFileName, std::ios::in | std::ios::binary);
    if (!in.is_open()) {
        printf("file %s cannot be opened, loadDataArrayFromBin fails. \n", DenseMatrixFileName);
        exit(-1);
    }
    in.read(reinterpret_cast<char*>(dense.data()), static_cast<std::streamsize>(want));
    const size_t got = static_cast<size_t>(in.gcount());
    if (got != want) {
        printf("file %s only has %ld, but request %ld, loading DenseMatrix fails! \n",
               DenseMatrixFileName,
               static_cast<long>(got),
               static_cast<long>(want));
        exit(-1);
    }
    in.close();
    uint32_t* words   = nullptr;
    int*      offsets = nullptr;
    const int n_offsets = encode_matrix(dense.data(), M, K, &words, &offsets, true);
    const int n_words   = offsets[n_offsets - 1] * kVec;
    std::ofstream sizes_file(OutputSizesFileName, std::ios::out | std::ios::binary);
    std::ofstream words_file(NZWeightsFileName, std::ios::out | std::ios::binary);
    std::ofstream offsets_file(TileOffsetsFileName, std::ios::out | std::ios::binary);
    if (!sizes_file.is_open() || !words_file.is_open() || !offsets_file.is_open()) {
        printf("GenSparseMatrixBinFile() ERROR: file %s, %s, or %s cannot be opened or creaetd. \n",
               OutputSizesFileName,
               NZWeightsFileName,
               TileOffsetsFileName);
        exit(-1);
    }
    sizes_file.write(reinterpret_cast<const char*>(&n_words), sizeof(int));
    sizes_file.write(reinterpret_cast<const char*>(&n_offsets), sizeof(int));
    words_file.write(reinterpret_cast<const char*>(words), sizeof(uint32_t) * static_cast<size_t>(n_words));
    offsets_file.write(reinterpret_cast<const char*>(offsets), sizeof(int) * static_cast<size_t>(n_offsets));
    free(words);
    free(offsets);
}
