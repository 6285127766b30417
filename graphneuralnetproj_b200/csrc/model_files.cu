// The per-rank list files the FasterTransformer glue reads next to the per-matrix weight files, and the
// tensor-parallel shard shapes they go with.
//
// The reference's conversion tool (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py) encodes
// every linear layer of every rank with GenSparseMatrixBinFile and then writes, per rank,
//   NNZ_List.<rank>.bin, NumOffsets_List.<rank>.bin, SplitK_List.<rank>.bin   (:183-195)
// one int32 per (layer, matrix) in the order query_key_value, attention.dense, dense_h_to_4h,
// dense_4h_to_h (:13-18), taken from each matrix's .OutputSizes.bin ({NNZ, NumOffsets}); a matrix that
// was left dense (no .OutputSizes.bin) gets 0, 0, 0.  The loaders size their buffers from these lists
// (third_party/ft.patch:1864-1872, 2352-2401).  Shard shapes per rank: M = {3h/g, h, 4h/g, h},
// K = {h, h/g, h, 4h/g} (:134-135).
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/spmm_b200.h"
#include "schedule.h"

namespace {

const char* const kWeightNames[4] = {
    "model.layers.%d.attention.query_key_value.weight.%d",
    "model.layers.%d.attention.dense.weight.%d",
    "model.layers.%d.mlp.dense_h_to_4h.weight.%d",
    "model.layers.%d.mlp.dense_4h_to_h.weight.%d",
};

bool write_ints(const std::string& path, const std::vector<int32_t>& values)
{
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f)
        return false;
    const bool ok = std::fwrite(values.data(), sizeof(int32_t), values.size(), f) == values.size();
    return std::fclose(f) == 0 && ok;
}

}  // namespace

extern "C" int spmm_b200_shard_shapes(int hidden, int world, int* M, int* K)
{
    if (hidden <= 0 || world <= 0 || hidden % world != 0 || !M || !K)
        return -1;
    M[0] = 3 * hidden / world, M[1] = hidden, M[2] = 4 * hidden / world, M[3] = hidden;
    K[0] = hidden, K[1] = hidden / world, K[2] = hidden, K[3] = 4 * hidden / world;
    for (int k = 0; k < 4; k++)
        if (M[k] % 128 != 0 || K[k] % 64 != 0)
            return -1;  // the tile format cannot describe such a shard
    return 0;
}

extern "C" int spmm_b200_suggest_split_k(int M, int K)
{
    if (M <= 0 || K <= 0 || M % 128 != 0 || K % 64 != 0)
        return 0;
    // The partition over 148 SMs parks at most slots_used partial tiles of 128 x N floats; a workspace of
    // Split_K * M * N halves holds them when Split_K * M >= 256 * slots_used.
    spmm_b200::Schedule s;
    spmm_b200::make_schedule(s, M / 128, K / 64, 148, 1L << 40);
    const long need = (256L * s.slots_used + M - 1) / M;
    return static_cast<int>(need < 1 ? 1 : need);
}

extern "C" int spmm_b200_write_rank_lists(const char* model_dir, int rank, int num_layers, const int* M, const int* K)
{
    if (!model_dir || rank < 0 || num_layers <= 0 || !M || !K)
        return -1;
    const std::string dir(model_dir);
    std::vector<int32_t> nnz, offsets, split_k;
    int sparse = 0;
    for (int layer = 0; layer < num_layers; layer++)
        for (int k = 0; k < 4; k++) {
            char name[256];
            std::snprintf(name, sizeof(name), kWeightNames[k], layer, rank);
            const std::string sizes_path = dir + "/" + name + ".OutputSizes.bin";
            int32_t sizes[2] = {0, 0};
            bool    found    = false;
            if (FILE* f = std::fopen(sizes_path.c_str(), "rb")) {
                found = std::fread(sizes, sizeof(int32_t), 2, f) == 2;
                std::fclose(f);
                if (!found)
                    return -1;  // a truncated sizes file
            }
            nnz.push_back(found ? sizes[0] : 0);
            offsets.push_back(found ? sizes[1] : 0);
            split_k.push_back(found ? spmm_b200_suggest_split_k(M[k], K[k]) : 0);
            sparse += found ? 1 : 0;
        }
    const std::string tail = "." + std::to_string(rank) + ".bin";
    if (!write_ints(dir + "/NNZ_List" + tail, nnz) || !write_ints(dir + "/NumOffsets_List" + tail, offsets)
        || !write_ints(dir + "/SplitK_List" + tail, split_k))
        return -1;
    return sparse;
}
