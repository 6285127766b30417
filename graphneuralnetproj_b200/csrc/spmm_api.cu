// Launcher and dispatcher: the sm_100a counterpart of SpMM_SplitK_API /
// SpMM_SplitK_Kernel_Ex (csrc/SpMM_API.cu:25-208), plus the extern "C" views
// declared in include/spmm_b200.h.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/SpMM_API.cuh"
#include "../../include/spmm_b200.h"
#include "host_threads.h"
#include "spmm_decode_kernel.cuh"
#include "spmm_pair_kernel.cuh"
#include "spmm_structured_kernel.cuh"

namespace spmm_b200 {
namespace {

// Shape of the block per width of the B slice (bounded by 227 KB of shared memory and 512 TMEM
// columns): D decoder teams of WPT warps, Q MMA-issuing warps, S ring slots, VPL 4-word vectors
// held per lane (WPT * VPL * 32 vectors = 7168 bytes of words in flight per team, loaded straight into
// registers: staging them through shared memory by bulk copy was measured 2-7 % slower at every width).
// Up to 64 columns the kernel is bound by decoding; 128 and 256 columns serve prefill sizes, where a
// decoded tile feeds four 128 x N x 16 MMAs of 64-128 cycles each and fewer, wider slots are enough.
template<int N>
struct DecodeConfig {
    static constexpr int D    = N <= 64 ? 8 : 4;   // decoder teams
    static constexpr int WPT  = N <= 64 ? 1 : 2;   // warps per team
    static constexpr int Q    = N <= 64 ? 4 : (N == 128 ? 2 : 1);  // MMA-issuing warps (2 * Q * N TMEM columns)
    static constexpr int VPL  = 14 / WPT;
    static constexpr int S    = N <= 64 ? 8 : (N == 128 ? 6 : 4);  // ring slots
    // B slices (row-major layout): tiled TMA loads, issued by the MMA warps a lap ahead into a second
    // B buffer where that fits in shared memory (N <= 16), else by the tile's decoder
    // (N = 8 keeps the 16-byte copies: its staged rows are twice as wide as the rows of B)
    static constexpr int BM   = N == 8 ? 0 : (N == 16 ? 2 : 1);
};

struct DeviceInfo {
    int  sm_count = 0;
    bool attrs_set[20] = {};  // cudaFuncSetAttribute done, per kernel instantiation
    int  pair_clusters[4] = {};  // clusters of the pair kernel the device holds at once, per layout and NM
};

std::mutex g_device_lock;  // guards DeviceInfo, the workspace -> counter set table and the caches below

DeviceInfo& device_info(int device)
{
    static DeviceInfo info[64];
    std::lock_guard<std::mutex> guard(g_device_lock);
    DeviceInfo& d = info[device & 63];
    if (d.sm_count == 0)
        cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device);
    return d;
}

// Launches that may overlap in time must not share arrival counters.  Set 0 belongs to the launches
// that park their partial tiles in the library's own scratch; every caller-provided workspace gets a
// set of its own, remembered by its address (seven at a time per device; the least recently assigned
// is handed on when an eighth workspace appears).
int counter_set_for(int device, const void* workspace)
{
    static const void* owner[64][kCounterSets] = {};
    static int         next[64]                = {};
    if (workspace == nullptr)
        return 0;
    std::lock_guard<std::mutex> guard(g_device_lock);
    const void** mine = owner[device & 63];
    for (int i = 1; i < kCounterSets; i++)
        if (mine[i] == workspace)
            return i;
    const int slot = 1 + (next[device & 63]++ % (kCounterSets - 1));
    mine[slot]     = workspace;
    return slot;
}

// Whether the weights may be fetched ahead of the stream predecessor's completion (see
// spmm_b200_set_weights_constant).
std::atomic<int> g_weights_constant{0};

// Partition cache: the schedule depends only on the shape and the slot budget.
struct PlanKey {
    int  tiles_m, tiles_k, max_ctas;
    long slots;
    bool operator==(const PlanKey& o) const
    {
        return tiles_m == o.tiles_m && tiles_k == o.tiles_k && max_ctas == o.max_ctas && slots == o.slots;
    }
};

// Fills `out` (a copy: the cache entry may be replaced by another thread as soon as the lock is gone).
void cached_schedule(const PlanKey& key, Schedule& out)
{
    constexpr int   kEntries = 32;
    static PlanKey  keys[kEntries];
    static Schedule plans[kEntries];
    static int      used = 0, next = 0;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    for (int i = 0; i < used; i++)
        if (keys[i] == key) {
            out = plans[i];
            return;
        }
    const int slot = used < kEntries ? used++ : (next++ % kEntries);
    keys[slot]     = key;
    make_schedule(plans[slot], key.tiles_m, key.tiles_k, key.max_ctas, key.slots);
    out = plans[slot];
}

template<int N, int TM = 0>
cudaError_t launch_decode(cudaStream_t stream, DeviceInfo& dev, int n_index, const DecodeParams& params,
                          int column_blocks = 1)
{
    constexpr int NB   = N < 16 ? 16 : N;
    using Cfg          = DecodeConfig<N>;
    constexpr int D    = Cfg::D;
    constexpr int BM   = TM ? 0 : Cfg::BM;  // token-major B keeps the 16-byte copies
    constexpr int smem =
        decode_smem_bytes<NB, Cfg::S, BM>();
    static_assert(smem <= 227 * 1024, "ring does not fit in shared memory");
    auto kern = spmm_decode_kernel<N, D, Cfg::Q, Cfg::WPT, Cfg::VPL, Cfg::S, TM, BM>;
    {
        std::lock_guard<std::mutex> guard(g_device_lock);
        if (!dev.attrs_set[n_index]) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) {
                (void)cudaGetLastError();  // do not leave the error behind for an unrelated later call
                return e;
            }
            dev.attrs_set[n_index] = true;
        }
    }
    // Launched so that it may start while the kernel before it in the stream drains (the kernel waits
    // for its predecessor before touching anything it may still be working on).
    cudaLaunchConfig_t config = {};
    config.gridDim            = dim3(params.sched.num_ctas, column_blocks);
    config.blockDim           = dim3(decode_threads<D, Cfg::Q, Cfg::WPT>());
    config.dynamicSmemBytes   = smem;
    config.stream             = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                       = attr;
    config.numAttrs                                    = 1;
    cudaError_t e = cudaLaunchKernelEx(&config, kern, params);
    return e != cudaSuccess ? e : cudaGetLastError();
}


// Widths that are multiples of 256 (prefill) run on pairs of SMs where the shape allows (see
// spmm_pair_kernel.cuh); spmm_b200_set_pair_kernel(0) keeps them on the single-block kernel.
std::atomic<int> g_pair_kernel{1};

// Eight decoder warps with an A buffer each, as at decode sizes (fewer decoders, or teams of two warps, were
// measured slower); what is left of shared memory holds B buffers (of NM * 16 KB).
template<int NM>
struct PairConfig {
    static constexpr int SA = 8, D = 8, VPL = 14;
    static constexpr int SB = NM == 2 ? 3 : 5;
};

// How many clusters of two blocks of the pair kernel the device holds at once (0: cannot run it).
template<int NM, int TM = 0>
int pair_clusters(DeviceInfo& dev, int n_index)
{
    using Cfg          = PairConfig<NM>;
    constexpr int smem = pair_smem_bytes<NM, Cfg::SA, Cfg::SB>();
    static_assert(smem <= 227 * 1024, "ring does not fit in shared memory");
    auto kern = spmm_pair_kernel<NM, Cfg::D, Cfg::VPL, Cfg::SA, Cfg::SB, TM>;
    std::lock_guard<std::mutex> guard(g_device_lock);
    if (!dev.attrs_set[n_index]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        cudaLaunchConfig_t config = {};
        config.gridDim            = dim3(2 * (dev.sm_count / 2));
        config.blockDim           = dim3(pair_threads<Cfg::D>());
        config.dynamicSmemBytes   = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs             = attr;
        config.numAttrs          = 1;
        int clusters             = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kern, &config) != cudaSuccess) {
            (void)cudaGetLastError();
            clusters = 0;
        }
        dev.pair_clusters[2 * TM + NM - 1] = std::min(clusters, dev.sm_count / 2);
        dev.attrs_set[n_index]             = true;
    }
    return dev.pair_clusters[2 * TM + NM - 1];
}

template<int NM, int TM = 0>
cudaError_t launch_pair(cudaStream_t stream, const DecodeParams& params, int column_blocks)
{
    using Cfg                 = PairConfig<NM>;
    auto kern                 = spmm_pair_kernel<NM, Cfg::D, Cfg::VPL, Cfg::SA, Cfg::SB, TM>;
    cudaLaunchConfig_t config = {};
    config.gridDim            = dim3(2 * params.sched.num_ctas, column_blocks);
    config.blockDim           = dim3(pair_threads<Cfg::D>());
    config.dynamicSmemBytes   = pair_smem_bytes<NM, Cfg::SA, Cfg::SB>();
    config.stream             = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id                                         = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x                           = 2;
    attr[0].val.clusterDim.y                           = 1;
    attr[0].val.clusterDim.z                           = 1;
    attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                       = attr;
    config.numAttrs                                    = 2;
    cudaError_t e = cudaLaunchKernelEx(&config, kern, params);
    return e != cudaSuccess ? e : cudaGetLastError();
}


// Scratch for the fp32 partial tiles of split rows, for callers that cannot provide a workspace.
// It lives in the library image: every GPU that loads the library holds these 10 MiB until the
// process exits.  In host code the name below is only a handle; the device address comes from
// cudaGetSymbolAddress.
constexpr size_t kOwnScratchBytes = 10u << 20;
static __device__ __align__(256) float g_own_scratch[kOwnScratchBytes / sizeof(float)];

// Device address of g_own_scratch on `device` (which must be current), looked up once per device.
cudaError_t own_scratch_address(int device, float** out)
{
    static float*     address[64] = {};
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    float*& slot = address[device & 63];
    if (slot == nullptr) {
        void*       p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_own_scratch);
        if (e != cudaSuccess)
            return e;
        slot = static_cast<float*>(p);
    }
    *out = slot;
    return cudaSuccess;
}


// Describes B[K][N] (row-major halves) to the copy engine for the kernels' tiled loads of 64-row
// slices: boxes of min(n_block, 64) columns (16 for N = 8: the columns beyond N read as zero), in the
// swizzle mode of the staged layout.
cudaError_t describe_b(CUtensorMap& map, const half* B, int N_Global, int K_Global, int n_block)
{
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn   encode = nullptr;
    static std::mutex lock;
    {
        std::lock_guard<std::mutex> guard(lock);
        if (encode == nullptr) {
            void*                           fn     = nullptr;
            cudaDriverEntryPointQueryResult status = cudaDriverEntryPointSymbolNotFound;
            cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
            if (e != cudaSuccess || status != cudaDriverEntryPointSuccess || fn == nullptr)
                return e != cudaSuccess ? e : cudaErrorNotSupported;
            encode = reinterpret_cast<EncodeFn>(fn);
        }
    }
    // the description depends only on (B, N, K, block width): callers multiply the same activations
    // buffer again and again, so the last few descriptions are kept
    struct Entry {
        const half* B;
        int         n, k, n_block;
        CUtensorMap map;
    };
    constexpr int kEntries = 16;
    static Entry  cache[kEntries];
    static int    used = 0, next = 0;
    {
        std::lock_guard<std::mutex> guard(lock);
        for (int i = 0; i < used; i++)
            if (cache[i].B == B && cache[i].n == N_Global && cache[i].k == K_Global && cache[i].n_block == n_block) {
                map = cache[i].map;
                return cudaSuccess;
            }
    }
    if (n_block < 0) {
        // token-major B[N][K]: x = k, y = token; boxes of 64 k values x 128 tokens, rows of 128 bytes
        const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(K_Global), static_cast<cuuint64_t>(N_Global)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K_Global) * sizeof(half)};
        const cuuint32_t box[2]     = {static_cast<cuuint32_t>(kTileCols), static_cast<cuuint32_t>(kPairColsPerMma / 2)};
        const cuuint32_t steps[2]   = {1, 1};
        if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<half*>(B), dims, strides, box, steps,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        std::lock_guard<std::mutex> guard(lock);
        const int slot = used < kEntries ? used++ : (next++ % kEntries);
        cache[slot]    = Entry{B, N_Global, K_Global, n_block, map};
        return cudaSuccess;
    }
    const int                box_cols = n_block < 16 ? 16 : (n_block > 64 ? 64 : n_block);
    const CUtensorMapSwizzle swizzle  = box_cols == 16   ? CU_TENSOR_MAP_SWIZZLE_32B
                                        : box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                         : CU_TENSOR_MAP_SWIZZLE_128B;
    const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(N_Global), static_cast<cuuint64_t>(K_Global)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(N_Global) * sizeof(half)};
    const cuuint32_t box[2]     = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(kTileCols)};
    const cuuint32_t steps[2]   = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<half*>(B), dims, strides, box, steps,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
        != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    {
        std::lock_guard<std::mutex> guard(lock);
        const int slot = used < kEntries ? used++ : (next++ % kEntries);
        cache[slot]    = Entry{B, N_Global, K_Global, n_block, map};
    }
    return cudaSuccess;
}

bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

}  // namespace
}  // namespace spmm_b200

namespace spmm_b200 {
namespace {

// Shared by both layouts: validates, partitions, launches.  token_major: B[N][K], C[N][M].
cudaError_t spmm_tiled_csl(cudaStream_t stream, const uint4* Compressed_A, const int* TileOffsets, const half* B, half* C,
                           int M_Global, int N_Global, int K_Global, half* Reduction_Workspace, int Split_K, bool token_major,
                           const float* addend = nullptr, size_t workspace_skip_bytes = 0, const PeerSumParams* peer = nullptr)
{
    // N: 8, 16, 32, 64 as in the reference (csrc/SpMM_API.cu:105-196); multiples of 64 beyond that are
    // served in column blocks (blockIdx.y) of 64 to 512 columns, in both layouts.
    const bool wide = N_Global > 64 && N_Global % 64 == 0 && N_Global <= 8192;
    if (N_Global != 8 && N_Global != 16 && N_Global != 32 && N_Global != 64 && !wide) {
        printf("MM_Sparse_API Error: Unsupported N dimension %d!\n", N_Global);
        return cudaErrorUnknown;
    }
    if (M_Global <= 0 || K_Global <= 0 || M_Global % kTileRows != 0 || K_Global % kTileCols != 0 || Split_K < 1)
        return cudaErrorInvalidValue;
    if (!Compressed_A || !TileOffsets || !B || !C || !aligned16(Compressed_A) || !aligned16(B)
        || !aligned16(Reduction_Workspace) || (!token_major && !aligned16(C)))
        return cudaErrorInvalidValue;

    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return e;
    DeviceInfo& dev = device_info(device);

    // Multiples of 256 columns on 256-row multiples: pairs of SMs, 512 columns per restored tile where N allows.
    int pair_nm = 0, clusters = 0;
    if (wide && N_Global % 256 == 0 && M_Global % (2 * kTileRows) == 0 && addend == nullptr && peer == nullptr
        && g_pair_kernel.load(std::memory_order_relaxed) != 0) {
        pair_nm  = N_Global % 512 == 0 ? 2 : 1;
        clusters = token_major ? (pair_nm == 2 ? pair_clusters<2, 1>(dev, 17) : pair_clusters<1, 1>(dev, 16))
                               : (pair_nm == 2 ? pair_clusters<2>(dev, 15) : pair_clusters<1>(dev, 14));
        if (clusters == 0)
            pair_nm = 0;
    }
    // the widest slice that divides N: the sparse tiles are decoded once per column block
    const int n_block       = !wide ? N_Global
                                    : (pair_nm ? pair_nm * kPairColsPerMma
                                               : (token_major ? 64 : (N_Global % 256 == 0 ? 256 : (N_Global % 128 == 0 ? 128 : 64))));
    const int column_blocks = N_Global / n_block;
    if (static_cast<long>(M_Global / kTileRows) * column_blocks > kMaxRowTiles)
        return cudaErrorInvalidValue;

    const int  tiles_m = M_Global / kTileRows, tiles_k = K_Global / kTileCols;
    // every column block gets an equal share of the workspace for its partial tiles
    // (a caller that keeps the head of the workspace for itself passes its size as workspace_skip_bytes)
    const size_t workspace_bytes = static_cast<size_t>(Split_K) * M_Global * N_Global * sizeof(half);
    const long   slots           = Reduction_Workspace && workspace_bytes > workspace_skip_bytes
                                       ? static_cast<long>((workspace_bytes - workspace_skip_bytes)
                                                           / (static_cast<size_t>(kTileRows) * n_block * sizeof(float)) / column_blocks)
                                       : 0;
    DecodeParams params;
    params.words        = Compressed_A;
    params.tile_offsets = TileOffsets;
    params.B            = B;
    params.C            = C;
    params.slots        = reinterpret_cast<float*>(reinterpret_cast<char*>(Reduction_Workspace) + workspace_skip_bytes);
    long slots_granted  = slots;
    params.counter_set  = counter_set_for(device, slots > 0 ? Reduction_Workspace : nullptr);
    if (!wide) {
        // A workspace sized by a small Split_K hint (the reference's 7168 x 7168 case passes 5) cannot
        // hold the partial tiles of a partition over all SMs; the library's built-in scratch takes its
        // place when it holds more.
        cached_schedule(PlanKey{tiles_m, tiles_k, dev.sm_count, 1L << 40}, params.sched);
        const long own = static_cast<long>(kOwnScratchBytes / (static_cast<size_t>(kTileRows) * n_block * sizeof(float)));
        if (slots < params.sched.slots_used && own > slots) {
            float* scratch = nullptr;
            if (own_scratch_address(device, &scratch) == cudaSuccess) {
                params.slots       = scratch;
                params.counter_set = 0;
                slots_granted      = own;
            }
            else
                (void)cudaGetLastError();
        }
    }
    params.weights_early = g_weights_constant.load(std::memory_order_relaxed);
    if (peer != nullptr) {
        if (wide || token_major)
            return cudaErrorInvalidValue;
        params.peer = *peer;
    }
    params.addend       = addend;
    params.n            = N_Global;
    params.tiles_k      = tiles_k;
    params.m            = M_Global;
    params.ld           = N_Global;
    if (pair_nm != 0) {
        // the schedule is over rows of tile pairs and clusters; each of a cluster's two blocks parks its own rows
        cached_schedule(PlanKey{tiles_m / 2, tiles_k, std::max(1, clusters / std::min(column_blocks, 4)), slots_granted / 2},
                        params.sched);
        params.slots_per_block_column = 2 * params.sched.slots_used;
        e = describe_b(params.b_map, B, N_Global, K_Global, token_major ? -1 : n_block);
        if (e != cudaSuccess)
            return e;
        if (token_major)
            return pair_nm == 2 ? launch_pair<2, 1>(stream, params, column_blocks) : launch_pair<1, 1>(stream, params, column_blocks);
        return pair_nm == 2 ? launch_pair<2>(stream, params, column_blocks) : launch_pair<1>(stream, params, column_blocks);
    }
    // with several column blocks the blocks of one column share the SMs with the other columns
    cached_schedule(PlanKey{tiles_m, tiles_k, wide ? std::max(1, dev.sm_count / std::min(column_blocks, 4)) : dev.sm_count,
                            slots_granted},
                    params.sched);
    params.slots_per_block_column = params.sched.slots_used;
    if (!token_major && N_Global != 8) {
        e = describe_b(params.b_map, B, N_Global, K_Global, n_block);
        if (e != cudaSuccess)
            return e;
    }
    if (wide && token_major)  // 64 tokens per column block
        return launch_decode<64, 1>(stream, dev, 7, params, column_blocks);
    if (wide) {
        switch (n_block) {
            case 256:
                return launch_decode<256>(stream, dev, 13, params, column_blocks);
            case 128:
                return launch_decode<128>(stream, dev, 12, params, column_blocks);
            default:
                return launch_decode<64>(stream, dev, 3, params, column_blocks);
        }
    }
    if (token_major) {
        switch (N_Global) {
            case 8:
                return launch_decode<8, 1>(stream, dev, 4, params);
            case 16:
                return launch_decode<16, 1>(stream, dev, 5, params);
            case 32:
                return launch_decode<32, 1>(stream, dev, 6, params);
            default:
                return launch_decode<64, 1>(stream, dev, 7, params);
        }
    }
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

template<int N, int STAGES>
cudaError_t launch_structured(cudaStream_t stream, DeviceInfo& dev, int n_index, const StructuredParams& params)
{
    constexpr int NB   = N < 16 ? 16 : N;
    constexpr int smem = structured_smem_bytes<NB, STAGES>();
    static_assert(smem <= 227 * 1024, "stages do not fit in shared memory");
    auto kern = spmm_structured_kernel<N, STAGES>;
    {
        std::lock_guard<std::mutex> guard(g_device_lock);
        if (!dev.attrs_set[n_index]) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) {
                (void)cudaGetLastError();
                return e;
            }
            dev.attrs_set[n_index] = true;
        }
    }
    cudaLaunchConfig_t config = {};
    config.gridDim            = dim3(params.sched.num_ctas);
    config.blockDim           = dim3(kStructuredThreads);
    config.dynamicSmemBytes   = smem;
    config.stream             = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                       = attr;
    config.numAttrs                                    = 1;
    cudaError_t e = cudaLaunchKernelEx(&config, kern, params);
    return e != cudaSuccess ? e : cudaGetLastError();
}

// Heterogeneous product C = A1 * B + A2 * B: A1 (at most two nonzeros per aligned group of four along
// K) packed by InitSparseMatrixA1_tcgen05, A2 as tiled-CSL or absent.  With a residual the structured
// kernel leaves its product in fp32 at the head of the workspace and the tiled-CSL kernel adds it
// before the single rounding to fp16.
cudaError_t spmm_hetero(cudaStream_t stream, const half* values, const int* metadata, const uint4* residual_words,
                        const int* residual_offsets, const half* B, half* C, int M_Global, int N_Global, int K_Global,
                        half* Reduction_Workspace, int Split_K)
{
    if (N_Global != 8 && N_Global != 16 && N_Global != 32 && N_Global != 64) {
        printf("MM_Sparse_API Error: Unsupported N dimension %d!\n", N_Global);
        return cudaErrorUnknown;
    }
    if (M_Global <= 0 || K_Global <= 0 || M_Global % kTileRows != 0 || K_Global % kBlockK != 0
        || M_Global / kTileRows > kMaxRowTiles || Split_K < 1)
        return cudaErrorInvalidValue;
    if (!values || !metadata || !B || !C || !aligned16(values) || !aligned16(metadata) || !aligned16(B) || !aligned16(C)
        || !aligned16(Reduction_Workspace))
        return cudaErrorInvalidValue;
    const bool   residual      = residual_words != nullptr && residual_offsets != nullptr;
    const size_t partial_bytes = static_cast<size_t>(M_Global) * N_Global * sizeof(float);
    const size_t workspace     = Reduction_Workspace ? static_cast<size_t>(Split_K) * M_Global * N_Global * sizeof(half) : 0;
    if (residual && workspace < partial_bytes)
        return cudaErrorInvalidValue;  // the fp32 hand-over needs Split_K >= 2 worth of workspace

    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return e;
    DeviceInfo& dev = device_info(device);

    const size_t skip    = residual ? partial_bytes : 0;
    const int    tiles_m = M_Global / kTileRows, blocks_k = K_Global / kBlockK;
    const long   slots   = workspace > skip
                               ? static_cast<long>((workspace - skip) / (static_cast<size_t>(kTileRows) * N_Global * sizeof(float)))
                               : 0;
    StructuredParams params;
    params.values   = reinterpret_cast<const uint4*>(values);
    params.meta     = reinterpret_cast<const uint4*>(metadata);
    params.B        = B;
    params.C        = C;
    params.C32      = residual ? reinterpret_cast<float*>(Reduction_Workspace) : nullptr;
    params.slots    = reinterpret_cast<float*>(reinterpret_cast<char*>(Reduction_Workspace) + skip);
    params.n        = N_Global;
    params.blocks_k = blocks_k;
    params.m        = M_Global;
    params.ld       = N_Global;
    params.counter_set   = counter_set_for(device, slots > 0 ? Reduction_Workspace : nullptr);
    params.weights_early = g_weights_constant.load(std::memory_order_relaxed);
    cached_schedule(PlanKey{tiles_m, blocks_k, dev.sm_count, slots}, params.sched);
    switch (N_Global) {
        case 8:
            e = launch_structured<8, 9>(stream, dev, 8, params);
            break;
        case 16:
            e = launch_structured<16, 9>(stream, dev, 9, params);
            break;
        case 32:
            e = launch_structured<32, 8>(stream, dev, 10, params);
            break;
        default:
            e = launch_structured<64, 6>(stream, dev, 11, params);
            break;
    }
    if (e != cudaSuccess || !residual)
        return e;
    return spmm_tiled_csl(stream, residual_words, residual_offsets, B, C, M_Global, N_Global, K_Global, Reduction_Workspace,
                          Split_K, false, params.C32, skip);
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
    (void)A1_Ind_data;
    if (metadata != nullptr)  // heterogeneous mode: A and metadata from InitSparseMatrixA1_tcgen05
        return spmm_b200::spmm_hetero(stream, A, metadata, Compressed_A, TileOffsets, B, C, M_Global, N_Global, K_Global,
                                      Reduction_Workspace, Split_K);
    return spmm_b200::spmm_tiled_csl(stream, Compressed_A, TileOffsets, B, C, M_Global, N_Global, K_Global,
                                     Reduction_Workspace, Split_K, false);
}

cudaError_t SpMM_SplitK_API(cudaStream_t stream,
                            const half*  A,
                            const uint4* Compressed_A,
                            const int*   TileOffsets,
                            const half*  B,
                            half*        C,
                            const int    M_Global,
                            const int    N_Global,
                            const int    K_Global,
                            half*        Reduction_Workspace,
                            int          Split_K)
{
    (void)A;
    return spmm_b200::spmm_tiled_csl(stream, Compressed_A, TileOffsets, B, C, M_Global, N_Global, K_Global,
                                     Reduction_Workspace, Split_K, true);
}

// ------------------------------------------------------------------ entry point that allocates nothing

extern "C" int spmm_b200_spmm_own_scratch(void*       stream,
                                          const void* Compressed_A,
                                          const int*  TileOffsets,
                                          const void* B,
                                          void*       C,
                                          int         M_Global,
                                          int         N_Global,
                                          int         K_Global)
{
    using namespace spmm_b200;
    if (N_Global != 8 && N_Global != 16 && N_Global != 32 && N_Global != 64) {
        printf("MM_Sparse_API Error: Unsupported N dimension %d!\n", N_Global);
        return static_cast<int>(cudaErrorUnknown);
    }
    if (M_Global <= 0 || K_Global <= 0 || M_Global % kTileRows != 0 || K_Global % kTileCols != 0) {
        printf("spmm_b200_spmm_own_scratch: M (%d) must be a positive multiple of %d and K (%d) of %d\n", M_Global,
               kTileRows, K_Global, kTileCols);
        return static_cast<int>(cudaErrorInvalidValue);
    }
    constexpr int kOwnScratchMaxRowTiles = 8192;
    if (M_Global / kTileRows > kOwnScratchMaxRowTiles) {
        printf("spmm_b200_spmm_own_scratch: M = %d exceeds the supported maximum of %d rows\n", M_Global,
               kOwnScratchMaxRowTiles * kTileRows);
        return static_cast<int>(cudaErrorInvalidValue);
    }
    if (!Compressed_A || !TileOffsets || !B || !C || !aligned16(Compressed_A) || !aligned16(B) || !aligned16(C))
        return static_cast<int>(cudaErrorInvalidValue);
    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    DeviceInfo& dev = device_info(device);
    const int   tiles_m = M_Global / kTileRows, tiles_k = K_Global / kTileCols;
    const long  total   = static_cast<long>(tiles_m) * tiles_k;
    const size_t slot_bytes = static_cast<size_t>(kTileRows) * N_Global * sizeof(float);
    // The balanced partition over all SMs must fit: its partial tiles are what the scratch is for.
    Schedule full;
    const int full_ctas = std::min(dev.sm_count, kMaxCtas);
    fill_schedule(full, tiles_m, tiles_k, static_cast<int>(total < full_ctas ? total : full_ctas), 1);
    if (static_cast<size_t>(full.slots_used) * slot_bytes > kOwnScratchBytes) {
        printf("spmm_b200_spmm_own_scratch: this shape needs %zu bytes of scratch, the built-in array holds %zu\n",
               static_cast<size_t>(full.slots_used) * slot_bytes, kOwnScratchBytes);
        return static_cast<int>(cudaErrorInvalidValue);
    }
    float* scratch = nullptr;
    e              = own_scratch_address(device, &scratch);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    DecodeParams params;
    params.words        = static_cast<const uint4*>(Compressed_A);
    params.tile_offsets = TileOffsets;
    params.B            = static_cast<const half*>(B);
    params.C            = static_cast<half*>(C);
    params.slots        = scratch;
    params.n            = N_Global;
    params.tiles_k      = tiles_k;
    params.m            = M_Global;
    params.ld           = N_Global;
    params.slots_per_block_column = 0;
    if (N_Global != 8) {
        e = describe_b(params.b_map, static_cast<const half*>(B), N_Global, K_Global, N_Global);
        if (e != cudaSuccess)
            return static_cast<int>(e);
    }
    params.counter_set   = 0;
    params.weights_early = g_weights_constant.load(std::memory_order_relaxed);
    cached_schedule(PlanKey{tiles_m, tiles_k, dev.sm_count, static_cast<long>(kOwnScratchBytes / slot_bytes)}, params.sched);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (N_Global) {
        case 8:
            return static_cast<int>(launch_decode<8>(st, dev, 0, params));
        case 16:
            return static_cast<int>(launch_decode<16>(st, dev, 1, params));
        case 32:
            return static_cast<int>(launch_decode<32>(st, dev, 2, params));
        default:
            return static_cast<int>(launch_decode<64>(st, dev, 3, params));
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

int spmm_b200_spmm_splitk_host_io(void*       stream,
                                  const void* Compressed_A,
                                  const int*  TileOffsets,
                                  const void* B_host,
                                  void*       C_host,
                                  void*       B_dev,
                                  void*       C_dev,
                                  int         M_Global,
                                  int         N_Global,
                                  int         K_Global,
                                  void*       Reduction_Workspace,
                                  int         Split_K)
{
    if (!B_host || !C_host || !B_dev || !C_dev || M_Global <= 0 || N_Global <= 0 || K_Global <= 0)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t  e  = cudaMemcpyAsync(B_dev, B_host, static_cast<size_t>(K_Global) * N_Global * sizeof(half),
                                      cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    e = SpMM_SplitK_API(st, nullptr, static_cast<const uint4*>(Compressed_A), nullptr, nullptr, TileOffsets,
                        static_cast<const half*>(B_dev), static_cast<half*>(C_dev), M_Global, N_Global, K_Global,
                        static_cast<half*>(Reduction_Workspace), Split_K);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    return static_cast<int>(cudaMemcpyAsync(C_host, C_dev, static_cast<size_t>(M_Global) * N_Global * sizeof(half),
                                            cudaMemcpyDeviceToHost, st));
}

namespace spmm_b200 {
namespace {
// Copy streams and events of spmm_b200_spmm_splitk_host_io_batch, created on first use, one set per device.
struct HostIoLanes {
    bool         ready = false, have_previous = false;
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t  fork = nullptr, joined = nullptr, products = nullptr;
    cudaEvent_t  landed[SPMM_B200_HOST_IO_MAX_ITEMS] = {};
    cudaEvent_t  multiplied[SPMM_B200_HOST_IO_MAX_ITEMS] = {};
};
std::mutex  g_host_io_lock;
HostIoLanes g_host_io_lanes[64];

cudaError_t host_io_lanes(int device, HostIoLanes** out)
{
    HostIoLanes& lanes = g_host_io_lanes[device & 63];
    if (!lanes.ready) {
        cudaError_t e = cudaStreamCreateWithFlags(&lanes.in, cudaStreamNonBlocking);
        if (e == cudaSuccess)
            e = cudaStreamCreateWithFlags(&lanes.out, cudaStreamNonBlocking);
        if (e == cudaSuccess)
            e = cudaEventCreateWithFlags(&lanes.fork, cudaEventDisableTiming);
        if (e == cudaSuccess)
            e = cudaEventCreateWithFlags(&lanes.joined, cudaEventDisableTiming);
        if (e == cudaSuccess)
            e = cudaEventCreateWithFlags(&lanes.products, cudaEventDisableTiming);
        for (int i = 0; i < SPMM_B200_HOST_IO_MAX_ITEMS && e == cudaSuccess; i++) {
            e = cudaEventCreateWithFlags(&lanes.landed[i], cudaEventDisableTiming);
            if (e == cudaSuccess)
                e = cudaEventCreateWithFlags(&lanes.multiplied[i], cudaEventDisableTiming);
        }
        if (e != cudaSuccess)
            return e;
        lanes.ready = true;
    }
    *out = &lanes;
    return cudaSuccess;
}
}  // namespace
}  // namespace spmm_b200

int spmm_b200_spmm_splitk_host_io_batch(void* stream, int count, const spmm_b200_host_io_item* items)
{
    using namespace spmm_b200;
    if (count < 1 || count > SPMM_B200_HOST_IO_MAX_ITEMS || !items)
        return static_cast<int>(cudaErrorInvalidValue);
    for (int i = 0; i < count; i++)
        if (!items[i].B_host || !items[i].C_host || !items[i].B_dev || !items[i].C_dev || items[i].M <= 0 || items[i].N <= 0
            || items[i].K <= 0)
            return static_cast<int>(cudaErrorInvalidValue);
    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    std::lock_guard<std::mutex> guard(g_host_io_lock);
    HostIoLanes* lanes = nullptr;
    e = host_io_lanes(device, &lanes);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define SPMM_B200_TRY(call)                \
    do {                                   \
        e = (call);                        \
        if (e != cudaSuccess)              \
            return static_cast<int>(e);    \
    } while (0)
    // The copies in start once the staging buffers are free: after everything queued on `stream` so far (first call),
    // or after the products of the previous call (later calls: its copies out may still be under way, so the
    // activations of this call travel while the last results of the previous one do).  The copies out follow their
    // products, which follow `stream`.
    if (!lanes->have_previous) {
        SPMM_B200_TRY(cudaEventRecord(lanes->fork, st));
        SPMM_B200_TRY(cudaStreamWaitEvent(lanes->in, lanes->fork, 0));
    }
    else
        SPMM_B200_TRY(cudaStreamWaitEvent(lanes->in, lanes->products, 0));
    for (int i = 0; i < count; i++) {
        const spmm_b200_host_io_item& it = items[i];
        SPMM_B200_TRY(cudaMemcpyAsync(it.B_dev, it.B_host, static_cast<size_t>(it.K) * it.N * sizeof(half),
                                      cudaMemcpyHostToDevice, lanes->in));
        SPMM_B200_TRY(cudaEventRecord(lanes->landed[i], lanes->in));
    }
    for (int i = 0; i < count; i++) {
        const spmm_b200_host_io_item& it = items[i];
        SPMM_B200_TRY(cudaStreamWaitEvent(st, lanes->landed[i], 0));
        SPMM_B200_TRY(SpMM_SplitK_API(st, nullptr, static_cast<const uint4*>(it.Compressed_A), nullptr, nullptr, it.TileOffsets,
                                      static_cast<const half*>(it.B_dev), static_cast<half*>(it.C_dev), it.M, it.N, it.K,
                                      static_cast<half*>(it.Reduction_Workspace), it.Split_K));
        SPMM_B200_TRY(cudaEventRecord(lanes->multiplied[i], st));
        SPMM_B200_TRY(cudaStreamWaitEvent(lanes->out, lanes->multiplied[i], 0));
        SPMM_B200_TRY(cudaMemcpyAsync(it.C_host, it.C_dev, static_cast<size_t>(it.M) * it.N * sizeof(half),
                                      cudaMemcpyDeviceToHost, lanes->out));
    }
    SPMM_B200_TRY(cudaEventRecord(lanes->products, st));
    lanes->have_previous = true;
    SPMM_B200_TRY(cudaEventRecord(lanes->joined, lanes->out));
    SPMM_B200_TRY(cudaStreamWaitEvent(st, lanes->joined, 0));
#undef SPMM_B200_TRY
    return static_cast<int>(cudaSuccess);
}

int spmm_b200_spmm_row_parallel(void*        stream,
                                const void*  Compressed_A,
                                const int*   TileOffsets,
                                const void*  B,
                                void*        C,
                                int          M_Global,
                                int          N_Global,
                                int          K_Global,
                                void*        Reduction_Workspace,
                                int          Split_K,
                                void* const* partial_buffers,
                                void* const* flag_arrays,
                                int          rank,
                                int          world,
                                void*        state,
                                unsigned     limit_ms,
                                int          partial_only)
{
    using namespace spmm_b200;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || !partial_buffers || !flag_arrays || !state
        || (reinterpret_cast<uintptr_t>(state) & 3u))
        return static_cast<int>(cudaErrorInvalidValue);
    if (N_Global != 8 && N_Global != 16 && N_Global != 32 && N_Global != 64) {
        printf("MM_Sparse_API Error: Unsupported N dimension %d!\n", N_Global);
        return static_cast<int>(cudaErrorUnknown);
    }
    PeerSumParams peer;
    for (int r = 0; r < world; r++) {
        for (int parity = 0; parity < 2; parity++) {
            void* buffer = partial_buffers[parity * world + r];
            if (!buffer || (reinterpret_cast<uintptr_t>(buffer) & 15u))
                return static_cast<int>(cudaErrorInvalidValue);
            peer.partial[parity][r] = static_cast<float*>(buffer);
        }
        if (!flag_arrays[r] || (reinterpret_cast<uintptr_t>(flag_arrays[r]) & 3u))
            return static_cast<int>(cudaErrorInvalidValue);
        peer.flags[r] = static_cast<uint32_t*>(flag_arrays[r]);
    }
    peer.state    = static_cast<uint32_t*>(state);
    peer.rank     = rank;
    peer.world    = world;
    peer.partial_only = partial_only == 2 ? 2 : (partial_only ? 1 : 0);
    peer.limit_ns = static_cast<unsigned long long>(limit_ms ? limit_ms : 2000u) * 1000000ull;
    return static_cast<int>(spmm_tiled_csl(static_cast<cudaStream_t>(stream), static_cast<const uint4*>(Compressed_A), TileOffsets,
                                           static_cast<const half*>(B), static_cast<half*>(C), M_Global, N_Global, K_Global,
                                           static_cast<half*>(Reduction_Workspace), Split_K, false, nullptr, 0, &peer));
}

int spmm_b200_spmm_splitk_token_major(void*       stream,
                                      const void* Compressed_A,
                                      const int*  TileOffsets,
                                      const void* B,
                                      void*       C,
                                      int         M_Global,
                                      int         N_Global,
                                      int         K_Global,
                                      void*       Reduction_Workspace,
                                      int         Split_K)
{
    return static_cast<int>(SpMM_SplitK_API(static_cast<cudaStream_t>(stream), nullptr,
                                            static_cast<const uint4*>(Compressed_A), TileOffsets,
                                            static_cast<const half*>(B), static_cast<half*>(C), M_Global, N_Global,
                                            K_Global, static_cast<half*>(Reduction_Workspace), Split_K));
}

int spmm_b200_set_pair_kernel(int enabled)
{
    return spmm_b200::g_pair_kernel.exchange(enabled ? 1 : 0);
}

int spmm_b200_set_weights_constant(int constant)
{
    return spmm_b200::g_weights_constant.exchange(constant ? 1 : 0);
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
            cudaMemset(counters, 0, sizeof(spmm_b200::g_row_arrivals));
        cudaDeviceSynchronize();
    }
    return status;
}

namespace spmm_b200 {
// One warp waits on a barrier that nothing ever arrives on: the bounded wait must give up after
// limit_ns, record the event in the status word and let the block exit normally.
__global__ void wait_that_runs_out_kernel(unsigned long long limit_ns)
{
    __shared__ __align__(8) uint64_t bar;
    __shared__ int                   abort_word;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_addr(&bar), 1);
        ptx::mbar_init_fence();
        abort_word = 0;
    }
    __syncthreads();
    const bool ok = ptx::mbar_wait_bounded(ptx::smem_addr(&bar), 0, &abort_word, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && !ok)
        atomicExch(&g_device_status, static_cast<int>(kStatusWaitTimeout));
}
}  // namespace spmm_b200

int spmm_b200_selftest_wait_timeout(void* stream, unsigned int limit_ms)
{
    if (limit_ms == 0 || limit_ms > 1000)
        return static_cast<int>(cudaErrorInvalidValue);
    spmm_b200::wait_that_runs_out_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<unsigned long long>(limit_ms) * 1000000ull);
    return static_cast<int>(cudaGetLastError());
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
