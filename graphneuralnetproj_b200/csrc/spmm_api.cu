// Launcher and dispatcher: the sm_100a counterpart of SpMM_SplitK_API /
// SpMM_SplitK_Kernel_Ex (csrc/SpMM_API.cu:25-208), plus the extern "C" views
// declared in include/spmm_b200.h.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/SpMM_API.cuh"
#include "../../include/spmm_b200.h"
#include "host_threads.h"
#include "spmm_decode_kernel.cuh"

namespace spmm_b200 {
namespace {

// Decoder warps = depth of the A/B tile ring, bounded by 227 KB of shared memory per block.
template<int N>
constexpr int decode_warps()
{
    return N <= 32 ? 10 : 8;
}
constexpr int kVectorsPerLane = 14;  // 14 * 32 vectors = 7168 bytes of words in flight per decoder warp

struct DeviceInfo {
    int  sm_count = 0;
    bool attrs_set[4] = {false, false, false, false};
};

DeviceInfo& device_info(int device)
{
    static DeviceInfo info[64];
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    DeviceInfo& d = info[device & 63];
    if (d.sm_count == 0)
        cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device);
    return d;
}

// Partition cache: the schedule depends only on the shape and the slot budget.
struct PlanKey {
    int  tiles_m, tiles_k, max_ctas;
    long slots;
    bool operator==(const PlanKey& o) const
    {
        return tiles_m == o.tiles_m && tiles_k == o.tiles_k && max_ctas == o.max_ctas && slots == o.slots;
    }
};

const Schedule& cached_schedule(const PlanKey& key)
{
    constexpr int   kEntries = 32;
    static PlanKey  keys[kEntries];
    static Schedule plans[kEntries];
    static int      used = 0, next = 0;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    for (int i = 0; i < used; i++)
        if (keys[i] == key)
            return plans[i];
    const int slot = used < kEntries ? used++ : (next++ % kEntries);
    keys[slot]     = key;
    make_schedule(plans[slot], key.tiles_m, key.tiles_k, key.max_ctas, key.slots);
    return plans[slot];
}

template<int N>
cudaError_t launch_decode(cudaStream_t stream, DeviceInfo& dev, int n_index, const DecodeParams& params)
{
    constexpr int NB   = N < 16 ? 16 : N;
    constexpr int D    = decode_warps<N>();
    constexpr int smem = decode_smem_bytes<NB, D>();
    auto          kern = spmm_decode_kernel<N, D, kVectorsPerLane>;
    if (!dev.attrs_set[n_index]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();  // do not leave the error behind for an unrelated later call
            return e;
        }
        dev.attrs_set[n_index] = true;
    }
    kern<<<params.sched.num_ctas, (kFirstDecodeWarp + D) * 32, smem, stream>>>(params);
    return cudaGetLastError();
}

bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

}  // namespace
}  // namespace spmm_b200

cudaError_t SpMM_SplitK_API(cudaStream_t    stream,
                            const half*     A,
                            const uint4*    Compressed_A,
                            const uint64_t* A1_Ind_data,
                            const int*      metadata,
                            const int*      TileOffsets,
                            const half*     B,
                            half*           C,
                            const int       M_Global,
                            const int       N_Global,
                            const int       K_Global,
                            half*           Reduction_Workspace,
                            int             Split_K)
{
    using namespace spmm_b200;
    (void)A;
    (void)A1_Ind_data;
    if (N_Global != 8 && N_Global != 16 && N_Global != 32 && N_Global != 64) {
        printf("MM_Sparse_API Error: Unsupported N dimension %d!\n", N_Global);
        return cudaErrorUnknown;
    }
    if (metadata != nullptr)
        return cudaErrorNotSupported;  // structured (2:4) half: not handled by this kernel
    if (M_Global <= 0 || K_Global <= 0 || M_Global % kTileRows != 0 || K_Global % kTileCols != 0
        || M_Global / kTileRows > kMaxRowTiles || Split_K < 1)
        return cudaErrorInvalidValue;
    if (!Compressed_A || !TileOffsets || !B || !C || !aligned16(Compressed_A) || !aligned16(B) || !aligned16(C)
        || !aligned16(Reduction_Workspace))
        return cudaErrorInvalidValue;

    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return e;
    DeviceInfo& dev = device_info(device);

    const int  tiles_m = M_Global / kTileRows, tiles_k = K_Global / kTileCols;
    const long slots   = Reduction_Workspace
                             ? static_cast<long>(static_cast<size_t>(Split_K) * M_Global * N_Global * sizeof(half)
                                                 / (static_cast<size_t>(kTileRows) * N_Global * sizeof(float)))
                             : 0;
    DecodeParams params;
    params.words        = Compressed_A;
    params.tile_offsets = TileOffsets;
    params.B            = B;
    params.C            = C;
    params.slots        = reinterpret_cast<float*>(Reduction_Workspace);
    params.n            = N_Global;
    params.tiles_k      = tiles_k;
    params.sched        = cached_schedule(PlanKey{tiles_m, tiles_k, dev.sm_count, slots});
    switch (N_Global) {
        case 8:
            return launch_decode<8>(stream, dev, 0, params);
        case 16:
            return launch_decode<16>(stream, dev, 1, params);
        case 32:
            return launch_decode<32>(stream, dev, 2, params);
        default:
            return launch_decode<64>(stream, dev, 3, params);
    }
}

// ------------------------------------------------------------------ extern "C"
extern "C" {

int spmm_b200_init_sparse_matrix_a(const uint16_t* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    if (M <= 0 || K <= 0 || M % 128 != 0 || K % 64 != 0)
        return -1;
    return InitSparseMatrixA_API(reinterpret_cast<half*>(const_cast<uint16_t*>(A_h)), M, N, K, Compressed_A, TileOffsets);
}

int spmm_b200_init_sparse_matrix_a_noreorder(
    const uint16_t* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    if (M <= 0 || K <= 0 || M % 128 != 0 || K % 64 != 0)
        return -1;
    return InitSparseMatrixA_API_NoReorder(
        reinterpret_cast<half*>(const_cast<uint16_t*>(A_h)), M, N, K, Compressed_A, TileOffsets);
}

void spmm_b200_free(void* p)
{
    free(p);
}

int spmm_b200_spmm_splitk(void*       stream,
                          const void* A,
                          const void* Compressed_A,
                          const void* A1_Ind_data,
                          const void* metadata,
                          const int*  TileOffsets,
                          const void* B,
                          void*       C,
                          int         M_Global,
                          int         N_Global,
                          int         K_Global,
                          void*       Reduction_Workspace,
                          int         Split_K)
{
    return static_cast<int>(SpMM_SplitK_API(static_cast<cudaStream_t>(stream),
                                            static_cast<const half*>(A),
                                            static_cast<const uint4*>(Compressed_A),
                                            static_cast<const uint64_t*>(A1_Ind_data),
                                            static_cast<const int*>(metadata),
                                            TileOffsets,
                                            static_cast<const half*>(B),
                                            static_cast<half*>(C),
                                            M_Global,
                                            N_Global,
                                            K_Global,
                                            static_cast<half*>(Reduction_Workspace),
                                            Split_K));
}

size_t spmm_b200_workspace_bytes(int M_Global, int N_Global, int Split_K)
{
    return static_cast<size_t>(Split_K) * M_Global * N_Global * sizeof(half);
}

int spmm_b200_device_status(int reset)
{
    int         status = 0;
    cudaError_t e      = cudaDeviceSynchronize();
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    e = cudaMemcpyFromSymbol(&status, spmm_b200::g_device_status, sizeof(int));
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    if (reset) {
        const int zero = 0;
        cudaMemcpyToSymbol(spmm_b200::g_device_status, &zero, sizeof(int));
        void* counters = nullptr;
        if (cudaGetSymbolAddress(&counters, spmm_b200::g_row_arrivals) == cudaSuccess)
            cudaMemset(counters, 0, sizeof(unsigned int) * spmm_b200::kMaxRowTiles * spmm_b200::kEpilogueWarps);
        cudaDeviceSynchronize();
    }
    return status;
}

int spmm_b200_plan(int tiles_m, int tiles_k, int max_ctas, long slots_avail, int* chunk_begin, int* split_rows_above,
                   int* slots_used)
{
    spmm_b200::Schedule s;
    spmm_b200::make_schedule(s, tiles_m, tiles_k, max_ctas, slots_avail);
    for (int g = 0; g <= s.num_ctas; g++)
        chunk_begin[g] = s.chunk_begin[g];
    for (int g = 0; g < s.num_ctas; g++)
        split_rows_above[g] = s.split_rows_above[g];
    *slots_used = s.slots_used;
    return s.num_ctas;
}

}  // extern "C"
