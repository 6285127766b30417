// Host encoders of the reference's 2:4-oriented formats, output-identical restatements kept for
// the completeness of the drop-in header: InitSparseMatrixA_API_NoReorder_v1..v4
// (csrc/SpMM_API.cu:571-1123), InitSparseMatrixA1_Vec_Sparse_Load (:1127-1398) and
// inspect_metadata (:1401-1553).  None of them feeds the sm_100a kernel of this library; they
// exist so that tools written against the reference header keep linking and get the same bytes.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/SpMM_API.cuh"

namespace {

constexpr int kTileM   = 128;  // _TILE_M of the uint32 / half formats (csrc/SpMM_API.cu:579)
constexpr int kTileMA1 = 256;  // TILE_M of the A1 formats (csrc/TilingConfig.h:67-68)
constexpr int kTileK   = 64;
constexpr int kVec     = 4;

// fabs(__half2float(v)) > 0: everything except +-0 and NaN (the test of the padding pass and of v1..v4).
inline bool kept(uint16_t bits)
{
    return static_cast<uint16_t>((bits & 0x7fffu) - 1u) < 0x7c00u;
}
// __half2float(v) != 0.0f: everything except +-0, NaN included (the test of the A1 encoder and the metadata).
inline bool nonzero_or_nan(uint16_t bits)
{
    return (bits & 0x7fffu) != 0;
}

[[noreturn]] void fail(const char* what)
{
    fprintf(stderr, "%s\n", what);
    abort();
}

void* checked_malloc(size_t bytes)
{
    void* p = malloc(bytes ? bytes : 1);
    if (!p) {
        printf("InitSparseMatrixA: Error in malloc memory from host memory!\n");
        exit(-1);
    }
    return p;
}

// Padding words per tile (to a multiple of four nonzeros) and the padded total, :602-624.
long padding_per_tile(const uint16_t* A, int M, int K, std::vector<int>& pad)
{
    long total = 0;
    pad.assign(static_cast<size_t>(M / kTileM) * (K / kTileK), 0);
    for (int i = 0; i < M / kTileM; i++)
        for (int j = 0; j < K / kTileK; j++) {
            const uint16_t* t   = A + static_cast<size_t>(i) * kTileM * K + j * kTileK;
            int             nnz = 0;
            for (int m = 0; m < kTileM; m++)
                for (int n = 0; n < kTileK; n++)
                    nnz += kept(t[static_cast<size_t>(m) * K + n]);
            const int p                 = (kVec - nnz % kVec) % kVec;
            pad[i * (K / kTileK) + j] = p;
            total += nnz + p;
        }
    return total;
}

void check_shape(int M, int K, int tile_m)
{
    if (M <= 0 || K <= 0 || M % tile_m != 0 || K % kTileK != 0)
        fail("InitSparseMatrixA: M must be a multiple of the tile height and K of 64");
}

}  // namespace

// :571-726.  Words carry row * 32 + (col / 4) * 2 + (rank of the nonzero within its group of four);
// padding words carry the element's own bits and (col / 4) * 2 + col % 4.
__host__ int
InitSparseMatrixA_API_NoReorder_v1(half* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    (void)N;
    check_shape(M, K, kTileM);
    const uint16_t*  A = reinterpret_cast<const uint16_t*>(A_h);
    std::vector<int> pad;
    const long       total   = padding_per_tile(A, M, K, pad);
    const int        tiles_k = K / kTileK, tiles = (M / kTileM) * tiles_k;
    uint32_t*        words   = static_cast<uint32_t*>(checked_malloc(static_cast<size_t>(total) * 4));
    int*             offsets = static_cast<int*>(checked_malloc((static_cast<size_t>(tiles) + 2) * sizeof(int)));
    long             n_out   = 0;
    for (int t = 0; t < tiles; t++) {
        const uint16_t* tile      = A + static_cast<size_t>(t / tiles_k) * kTileM * K + (t % tiles_k) * kTileK;
        int             remaining = pad[t];
        int             in_group = 0, rank = 0;
        for (int m = 0; m < kTileM; m++)
            for (int n = 0; n < kTileK; n++) {
                if (in_group == 4) {
                    in_group = 0;
                    rank     = 0;
                }
                in_group++;
                const uint16_t v = tile[static_cast<size_t>(m) * K + n];
                if (kept(v)) {
                    const int pos = m * (kTileK / 2) + (n / 4) * 2 + rank++;
                    words[n_out++] = static_cast<uint32_t>(v) | (static_cast<uint32_t>(static_cast<uint16_t>(pos)) << 16);
                }
                else if (remaining > 0) {
                    remaining--;
                    const int pos = m * (kTileK / 2) + (n / 4) * 2 + n % 4;
                    words[n_out++] = static_cast<uint32_t>(v) | (static_cast<uint32_t>(static_cast<uint16_t>(pos)) << 16);
                }
            }
        offsets[t + 1] = static_cast<int>(n_out / kVec);
    }
    offsets[0]         = 0;
    offsets[tiles + 1] = static_cast<int>(n_out / kVec);
    *Compressed_A      = words;
    *TileOffsets       = offsets;
    return tiles + 2;
}

// :730-859.  Bare halves in scan order (nonzeros plus the first zeros met as padding); offsets count
// groups of eight halves.  The reference asserts that every tile's count is a multiple of eight.
__host__ int InitSparseMatrixA_API_NoReorder_v2(half* A_h, int M, int N, int K, half** Compressed_A, int** TileOffsets)
{
    (void)N;
    check_shape(M, K, kTileM);
    const uint16_t*  A = reinterpret_cast<const uint16_t*>(A_h);
    std::vector<int> pad;
    const long       total   = padding_per_tile(A, M, K, pad);
    const int        tiles_k = K / kTileK, tiles = (M / kTileM) * tiles_k;
    uint16_t*        out     = static_cast<uint16_t*>(checked_malloc(static_cast<size_t>(total) * 2));
    int*             offsets = static_cast<int*>(checked_malloc((static_cast<size_t>(tiles) + 2) * sizeof(int)));
    long             n_out   = 0;
    for (int t = 0; t < tiles; t++) {
        const uint16_t* tile      = A + static_cast<size_t>(t / tiles_k) * kTileM * K + (t % tiles_k) * kTileK;
        int             remaining = pad[t];
        const long      before    = n_out;
        for (int m = 0; m < kTileM; m++)
            for (int n = 0; n < kTileK; n++) {
                const uint16_t v = tile[static_cast<size_t>(m) * K + n];
                if (kept(v)) {
                    out[n_out++] = v;
                }
                else if (remaining > 0) {
                    remaining--;
                    out[n_out++] = v;
                }
            }
        if ((n_out - before) % (2 * kVec) != 0)
            fail("InitSparseMatrixA_API_NoReorder_v2: a tile's padded count is not a multiple of 8");
        offsets[t + 1] = static_cast<int>(n_out / (2 * kVec));
    }
    offsets[0]         = 0;
    offsets[tiles + 1] = static_cast<int>(n_out / (2 * kVec));
    *Compressed_A      = reinterpret_cast<half*>(out);
    *TileOffsets       = offsets;
    return tiles + 2;
}

namespace {

// Two halves per group of four: the group's nonzeros in order, then +0.  More than two is an error (:943).
inline void compress_group(const uint16_t* g, uint16_t* out2)
{
    int n = 0;
    for (int x = 0; x < 4; x++)
        if (kept(g[x])) {
            if (n == 2)
                fail("InitSparseMatrixA_API_NoReorder_v3/v4: more than two nonzeros in a group of four");
            out2[n++] = g[x];
        }
    while (n < 2)
        out2[n++] = 0;
}

int encode_two_four(const uint16_t* A, int M, int K, half** Compressed_A, int** TileOffsets, bool pair_rows)
{
    check_shape(M, K, kTileM);
    const int tiles_k = K / kTileK, tiles = (M / kTileM) * tiles_k;
    uint16_t* out     = static_cast<uint16_t*>(checked_malloc(static_cast<size_t>(M) * K / 2 * 2));
    int*      offsets = static_cast<int*>(checked_malloc((static_cast<size_t>(tiles) + 2) * sizeof(int)));
    long      n_out   = 0;
    uint16_t  rows[kTileK];  // two compressed rows of 32 halves each (:1089-1103)
    for (int t = 0; t < tiles; t++) {
        const uint16_t* tile = A + static_cast<size_t>(t / tiles_k) * kTileM * K + (t % tiles_k) * kTileK;
        for (int m = 0; m < kTileM; m++) {
            uint16_t* dst = pair_rows ? rows + (m & 1) * (kTileK / 2) : out + n_out;
            for (int n = 0; n < kTileK; n += 4)
                compress_group(tile + static_cast<size_t>(m) * K + n, dst + n / 2);
            if (!pair_rows) {
                n_out += kTileK / 2;
            }
            else if (m & 1) {
                const int mask = ((m / 2) % 4) << 3;
                for (int c = 0; c < kTileK; c++)
                    out[n_out++] = rows[c ^ mask];
            }
        }
        offsets[t + 1] = static_cast<int>(n_out / (2 * kVec));
    }
    offsets[0]         = 0;
    offsets[tiles + 1] = static_cast<int>(n_out / (2 * kVec));
    *Compressed_A      = reinterpret_cast<half*>(out);
    *TileOffsets       = offsets;
    return tiles + 2;
}

}  // namespace

// :862-989.  A must be 2:4; each 128 x 64 tile becomes 128 x 32 halves, row by row.
__host__ int InitSparseMatrixA_API_NoReorder_v3(half* A_h, int M, int N, int K, half** Compressed_A, int** TileOffsets)
{
    (void)N;
    return encode_two_four(reinterpret_cast<const uint16_t*>(A_h), M, K, Compressed_A, TileOffsets, false);
}

// :993-1123.  As v3, with two compressed rows per 64-half shared-memory row and the 16-byte chunk
// index XORed with (pair index % 4).
__host__ int InitSparseMatrixA_API_NoReorder_v4(half* A_h, int M, int N, int K, half** Compressed_A, int** TileOffsets)
{
    (void)N;
    return encode_two_four(reinterpret_cast<const uint16_t*>(A_h), M, K, Compressed_A, TileOffsets, true);
}

// :1127-1398.  A1 must be 2:4.  Per 256 x 64 tile: the nonzeros in row-major order, eight to a vector
// (one uint4 of halves), plus one 64-bit index word per vector: bits 63..56 the row of element 0,
// bits 6..0 its compressed column (col / 4) * 2 + rank-in-group, and for element k >= 1 in bits
// 7k+6..7k its distance from element k-1 in the flattened (row * 32 + compressed column) space.
// The last vector of a tile is padded by repeating the last value with distance 0.  TileOffsets
// counts vectors.  As in the reference, a tile without nonzeros is counted as one vector that is
// never written (:1202, :1315-1317).
__host__ int InitSparseMatrixA1_Vec_Sparse_Load(
    half* A1, int M, int K, half** Compressed_A, uint64_t** Ind_data, int** TileOffsets)
{
    check_shape(M, K, kTileMA1);
    constexpr int   kVecA1 = 8, kBits = 7;
    const uint16_t* A       = reinterpret_cast<const uint16_t*>(A1);
    const int       tiles_k = K / kTileK, tiles = (M / kTileMA1) * tiles_k;
    int*            offsets = static_cast<int*>(checked_malloc((static_cast<size_t>(tiles) + 2) * sizeof(int)));
    long            vectors = 0;
    for (int t = 0; t < tiles; t++) {
        const uint16_t* tile = A + static_cast<size_t>(t / tiles_k) * kTileMA1 * K + (t % tiles_k) * kTileK;
        int             nnz  = 0;
        for (int m = 0; m < kTileMA1; m++)
            for (int n = 0; n < kTileK; n++)
                nnz += nonzero_or_nan(tile[static_cast<size_t>(m) * K + n]);
        vectors += (nnz - 1) / kVecA1 + 1;  // C division: an empty tile still counts one vector
        offsets[t + 1] = static_cast<int>(vectors);
    }
    printf("INTO TotalNZCount = %d\n", static_cast<int>(vectors));
    offsets[0]         = 0;
    offsets[tiles + 1] = static_cast<int>(vectors);
    uint16_t* values   = static_cast<uint16_t*>(checked_malloc(static_cast<size_t>(vectors) * kVecA1 * 2));
    uint64_t* index    = static_cast<uint64_t*>(checked_malloc(static_cast<size_t>(vectors) * 8));
    long      v_offset = 0, d_offset = 0;
    int       max_offset = 0;
    std::vector<uint16_t> val;
    std::vector<int>      col, row;
    for (int t = 0; t < tiles; t++) {
        const uint16_t* tile = A + static_cast<size_t>(t / tiles_k) * kTileMA1 * K + (t % tiles_k) * kTileK;
        val.clear();
        col.clear();
        row.clear();
        for (int m = 0; m < kTileMA1; m++)
            for (int n = 0; n < kTileK; n += 4) {
                int rank = 0;
                for (int x = 0; x < 4; x++) {
                    const uint16_t v = tile[static_cast<size_t>(m) * K + n + x];
                    if (nonzero_or_nan(v)) {
                        if (rank == 2)
                            fail("InitSparseMatrixA1_Vec_Sparse_Load: more than two nonzeros in a group of four");
                        val.push_back(v);
                        col.push_back((n / 4) * 2 + rank++);
                        row.push_back(m);
                    }
                }
            }
        const size_t count = val.size();
        int          tile_max = 0;
        bool         any_jump = false;
        auto field = [&](size_t i, int k, uint64_t& word) {  // distance of element i from element i - 1
            if (k == 0) {
                word |= static_cast<uint64_t>(col[i]);
                return;
            }
            uint64_t diff;
            if (row[i] == row[i - 1]) {
                diff = static_cast<uint64_t>(col[i] - col[i - 1]);
            }
            else {
                diff = static_cast<uint64_t>((row[i] * (kTileK / 2) + col[i]) - (row[i - 1] * (kTileK / 2) + col[i - 1]));
                if (diff >= (1u << kBits))
                    fail("InitSparseMatrixA1_Vec_Sparse_Load: distance between nonzeros does not fit 7 bits");
                any_jump = true;
                tile_max = static_cast<int>(diff) > tile_max ? static_cast<int>(diff) : tile_max;
            }
            word |= diff << (kBits * k);
        };
        size_t i = 0;
        for (; i + kVecA1 <= count; i += kVecA1) {
            uint64_t word = static_cast<uint64_t>(row[i]) << (kVecA1 * kBits);
            for (int k = 0; k < kVecA1; k++) {
                values[v_offset + k] = val[i + k];
                field(i + k, k, word);
            }
            index[d_offset++] = word;
            v_offset += kVecA1;
        }
        if (i == count)
            continue;  // (the reference also skips its statistics here)
        uint64_t word = static_cast<uint64_t>(row[i]) << (kVecA1 * kBits);
        int      k    = 0;
        for (; i + k < count; k++) {
            values[v_offset++] = val[i + k];
            field(i + k, k, word);
        }
        const int padding = kVecA1 - static_cast<int>(count % kVecA1);
        for (int x = 0; x < padding; x++)
            values[v_offset++] = val[count - 1];
        index[d_offset++] = word;
        if (any_jump && tile_max > max_offset)
            max_offset = tile_max;
    }
    printf("max_offset = %d\n", max_offset);
    printf("v_offset = %d, d_offset = %d\n", static_cast<int>(v_offset), static_cast<int>(d_offset));
    printf("Into Function: TotalNZCount = %d\n", static_cast<int>(vectors));
    *Compressed_A = reinterpret_cast<half*>(values);
    *Ind_data     = index;
    *TileOffsets  = offsets;
    return tiles + 2;
}

// :1401-1553.  Selector metadata of mma.sp m16n8k16: per 16 x 16 block eight 32-bit words, word r
// holding the 4-bit codes of the four groups of row r (low half) and row r + 8 (high half); then
// regrouped per 256 x 64 tile so that four consecutive k blocks of one row lie in one 16-byte chunk.
// Codes (:1404-1416): 1100->4 1010->8 1001->C 0110->9 0101->D 0011->E 1000->0 0100->1 0010->2 0001->3
// 0000->F; a group with three or four nonzeros gets 0, as the reference's map lookup does.
__host__ void inspect_metadata(half* mat, int* meta, int M, int K)
{
    static const int kCode[16] = {
        // index: bit 3 = first element nonzero ... bit 0 = fourth element nonzero
        0xF, 0x3, 0x2, 0xE, 0x1, 0xD, 0x9, 0x0, 0x0, 0xC, 0x8, 0x0, 0x4, 0x0, 0x0, 0x0};
    const uint16_t* A = reinterpret_cast<const uint16_t*>(mat);
    const int       blocks_k = K / 16;
    std::vector<int> buffer(static_cast<size_t>(M / 16) * blocks_k * 8);
    long            histogram[16] = {0};
    for (int m = 0; m < M / 16; m++)
        for (int k = 0; k < blocks_k; k++)
            for (int r = 0; r < 8; r++) {
                unsigned word = 0;
                for (int half_sel = 0; half_sel < 2; half_sel++)
                    for (int g = 0; g < 4; g++) {
                        const uint16_t* e = A + static_cast<size_t>(m * 16 + r + 8 * half_sel) * K + k * 16 + g * 4;
                        const int pattern = (nonzero_or_nan(e[0]) << 3) | (nonzero_or_nan(e[1]) << 2)
                                            | (nonzero_or_nan(e[2]) << 1) | static_cast<int>(nonzero_or_nan(e[3]));
                        histogram[pattern]++;
                        word |= static_cast<unsigned>(kCode[pattern]) << (g * 4 + 16 * half_sel);
                    }
                buffer[(static_cast<size_t>(m) * blocks_k + k) * 8 + r] = static_cast<int>(word);
            }
    long id = 0;
    for (int i = 0; i < M / kTileMA1; i++)
        for (int j = 0; j < K / kTileK; j++)
            for (int ii = 0; ii < kTileMA1 / 16; ii++)
                for (int r = 0; r < 8; r++)
                    for (int k = 0; k < 4; k++) {
                        const size_t block_row = static_cast<size_t>(i) * (kTileMA1 / 16) + ii;
                        const size_t block_col = static_cast<size_t>(j) * 4 + k;
                        meta[id++] = buffer[(block_row * blocks_k + block_col) * 8 + r];
                    }
    long total = 0;
    for (long h : histogram)
        total += h;
    printf("Metadata Inspection:\n");
    for (int pattern = 0; pattern < 16; pattern++)
        if (histogram[pattern] || kCode[pattern] != 0 || pattern == 7)
            printf("%d%d%d%d %ld %g%%\n", (pattern >> 3) & 1, (pattern >> 2) & 1, (pattern >> 1) & 1, pattern & 1,
                   histogram[pattern], total ? histogram[pattern] * 100.0 / total : 0.0);
}
