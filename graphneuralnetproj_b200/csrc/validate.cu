// Checks that a tiled-CSL stream is well formed before it is handed to the SpMM kernels, which trust
// it: a word's position field addresses the 128 x 64 tile buffer in shared memory and consecutive
// TileOffsets entries size the kernels' bulk copies.  The reference checks the same properties with
// asserts inside its encoder (csrc/SpMM_API.cu:354-356, 380, 431) and nowhere on the consuming side;
// weights that come from files (.NZWeights.bin / .TileOffsets.bin) can be truncated or corrupt.
//
// Properties: TileOffsets[0] == 0; entries never decrease; the last entry is repeated
// (TileOffsets[tiles + 1] == TileOffsets[tiles], csrc/SpMM_API.cu:432-435); the words the offsets
// cover are exactly the n_words given; every word's position is below 128 * 64.
// Findings are reported as a bit mask; nothing here traps or reads beyond n_words / tiles + 2.
#include <cstdint>

#include <cuda_runtime.h>

#include "../../include/spmm_b200.h"

namespace spmm_b200 {
namespace {

constexpr int kTileElements = 128 * 64;

__device__ int g_validate_findings;

__global__ void validate_tiled_csl_kernel(const uint32_t* words, size_t n_words, const int* offsets, int tiles)
{
    int          found  = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t first  = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (first == 0) {
        if (offsets[0] != 0)
            found |= SPMM_B200_CSL_FIRST_OFFSET_NOT_ZERO;
        if (offsets[tiles + 1] != offsets[tiles])
            found |= SPMM_B200_CSL_TAIL_NOT_REPEATED;
        if (static_cast<size_t>(static_cast<unsigned int>(offsets[tiles])) * 4u != n_words || offsets[tiles] < 0)
            found |= SPMM_B200_CSL_WORD_COUNT_MISMATCH;
    }
    for (size_t t = first; t < static_cast<size_t>(tiles); t += stride)
        if (offsets[t + 1] < offsets[t])
            found |= SPMM_B200_CSL_OFFSETS_DECREASE;
    for (size_t w = first; w < n_words; w += stride)
        if ((words[w] >> 16) >= static_cast<uint32_t>(kTileElements))
            found |= SPMM_B200_CSL_POSITION_OUT_OF_TILE;
    if (found)
        atomicOr(&g_validate_findings, found);
}

}  // namespace
}  // namespace spmm_b200

extern "C" int spmm_b200_validate_tiled_csl_host(const uint32_t* words, size_t n_words, const int* offsets, int M, int K)
{
    if (!offsets || (!words && n_words) || M <= 0 || K <= 0 || M % 128 || K % 64)
        return SPMM_B200_CSL_BAD_ARGUMENT;
    const long tiles = static_cast<long>(M / 128) * (K / 64);
    int        found = 0;
    if (offsets[0] != 0)
        found |= SPMM_B200_CSL_FIRST_OFFSET_NOT_ZERO;
    if (offsets[tiles + 1] != offsets[tiles])
        found |= SPMM_B200_CSL_TAIL_NOT_REPEATED;
    if (offsets[tiles] < 0 || static_cast<size_t>(offsets[tiles]) * 4u != n_words)
        found |= SPMM_B200_CSL_WORD_COUNT_MISMATCH;
    for (long t = 0; t < tiles; t++)
        if (offsets[t + 1] < offsets[t])
            found |= SPMM_B200_CSL_OFFSETS_DECREASE;
    for (size_t w = 0; w < n_words; w++)
        if ((words[w] >> 16) >= static_cast<uint32_t>(spmm_b200::kTileElements))
            found |= SPMM_B200_CSL_POSITION_OUT_OF_TILE;
    return found;
}

extern "C" int spmm_b200_validate_tiled_csl(void* stream, const void* Compressed_A, size_t n_words, const int* TileOffsets, int M, int K)
{
    using namespace spmm_b200;
    if (!TileOffsets || (!Compressed_A && n_words) || M <= 0 || K <= 0 || M % 128 || K % 64)
        return SPMM_B200_CSL_BAD_ARGUMENT;
    const long tiles = static_cast<long>(M / 128) * (K / 64);
    if (tiles + 2 > 0x7fffffffL)
        return SPMM_B200_CSL_BAD_ARGUMENT;
    cudaStream_t st   = static_cast<cudaStream_t>(stream);
    const int    zero = 0;
    cudaError_t  e    = cudaMemcpyToSymbolAsync(g_validate_findings, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    const size_t work   = n_words > static_cast<size_t>(tiles) ? n_words : static_cast<size_t>(tiles);
    const int    blocks = static_cast<int>(work / 256 + 1 < 1184 ? work / 256 + 1 : 1184);  // 8 blocks per SM on 148 SMs
    validate_tiled_csl_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint32_t*>(Compressed_A), n_words, TileOffsets,
                                                      static_cast<int>(tiles));
    e = cudaGetLastError();
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    int found = 0;
    e         = cudaMemcpyFromSymbolAsync(&found, g_validate_findings, sizeof(int), 0, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess)
        e = cudaStreamSynchronize(st);
    return e != cudaSuccess ? -static_cast<int>(e) : found;
}
