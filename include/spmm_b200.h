/* Plain-C boundary of libSpMM_API.so (sm_100a).
 *
 * The reference exports its entry points with C++ linkage
 * (build/SpMM_API.cuh:40-96); SpMM_API.cuh in this directory keeps those
 * symbols for callers that link C++.  The functions below are thin extern "C"
 * views of the same entry points for foreign-function interfaces (Python
 * ctypes, cgo, JNI ...).  fp16 data is passed as raw 16-bit patterns, streams
 * as the cudaStream_t handle cast to void*, and device pointers as void*.
 * Functions returning int return a cudaError_t value unless stated otherwise.
 */
#ifndef SPMM_B200_H
#define SPMM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* InitSparseMatrixA_API, build/SpMM_API.cuh:55 (csrc/SpMM_API.cu:241-438).
 * Host dense A[M][K] -> tiled-CSL words + offsets (malloc'd, release with
 * spmm_b200_free).  Returns the number of offsets (tiles + 2), or -1 if M is
 * not a multiple of 128 or K of 64 (the C++ symbol aborts there, like the
 * reference's assert). */
int spmm_b200_init_sparse_matrix_a(const uint16_t* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets);

/* InitSparseMatrixA_API_NoReorder, build/SpMM_API.cuh:57-62 (csrc/SpMM_API.cu:441-567). */
int spmm_b200_init_sparse_matrix_a_noreorder(
    const uint16_t* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets);

/* free() for buffers returned by the encoders (the reference's callers call free directly,
 * kernel_benchmark/spmm_test.cu:348-349). */
void spmm_b200_free(void* p);

/* SpMM_SplitK_API, build/SpMM_API.cuh:40-52 (csrc/SpMM_API.cu:79-208).  Same
 * argument order and meaning; all pointers are device pointers. */
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
                          int         Split_K);

/* spmm_b200_spmm_splitk (unstructured mode) for activations and results that live in host memory,
 * as the reference's harness holds them around its cudaMemcpy calls (kernel_benchmark/
 * spmm_test.cu:118-137, 520-533): on `stream`, copies B_host[K][N] to B_dev, multiplies, copies
 * C_dev[M][N] to C_host.  B_dev and C_dev are device buffers of K*N and M*N halves provided by the
 * caller (nothing is allocated here); B_host and C_host should be page-locked for the copies to be
 * asynchronous.  Returns the first cudaError_t met, as an int. */
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
                                  int         Split_K);

/* Several spmm_b200_spmm_splitk_host_io products in one call, e.g. the linear layers of a decoder
 * block: the copies of the activations run on a copy stream of the library ahead of the products,
 * and every result travels back on a second copy stream while the next product runs on `stream`.
 * When the call returns everything is queued; `stream` has been made to wait for the last copy, so
 * synchronising `stream` (or queueing more work on it) is enough to read C_host.  The library keeps
 * two streams and a few events per device for this (created by the first call on the device, which
 * should not fall inside a stream capture).  count: 1 .. SPMM_B200_HOST_IO_MAX_ITEMS.  Calls are
 * serialised by a lock.  The staging buffers B_dev and C_dev belong to these calls: the copies in of a
 * call are ordered after the products of the previous call on the device (so they travel while that
 * call's last results still go out), not after other work the caller queued on `stream` in between;
 * a caller that touches B_dev or C_dev itself synchronises first.  Returns the first cudaError_t met, as an int.  The reference's harness
 * does the same copies with blocking cudaMemcpy calls (kernel_benchmark/spmm_test.cu:118-137,
 * 565-567). */
#define SPMM_B200_HOST_IO_MAX_ITEMS 16
typedef struct spmm_b200_host_io_item {
    const void* Compressed_A;
    const int*  TileOffsets;
    const void* B_host; /* K * N halves, page-locked */
    void*       C_host; /* M * N halves, page-locked */
    void*       B_dev;  /* device staging for B */
    void*       C_dev;  /* device staging for C */
    int         M, N, K;
    void*       Reduction_Workspace;
    int         Split_K;
} spmm_b200_host_io_item;
int spmm_b200_spmm_splitk_host_io_batch(void* stream, int count, const spmm_b200_host_io_item* items);

/* The eleven-argument upstream form of SpMM_SplitK_API that the reference's FasterTransformer
 * glue calls (third_party/ft.patch:2822-2846), with token-major layouts: B[N][K], C[N][M].
 * N: 8, 16, 32, 64, and multiples of 64 up to 8192 (the glue's calls with more than 64 tokens,
 * third_party/ft.patch:523,1454): multiples of 256 with M a multiple of 256 run on pairs of SMs
 * (B arrives as K-contiguous TMA boxes, the layout the tensor core reads directly), other widths in
 * column blocks of 64 tokens. */
int spmm_b200_spmm_splitk_token_major(void*       stream,
                                      const void* Compressed_A,
                                      const int*  TileOffsets,
                                      const void* B,
                                      void*       C,
                                      int         M_Global,
                                      int         N_Global,
                                      int         K_Global,
                                      void*       Reduction_Workspace,
                                      int         Split_K);

/* SpMM for callers that can neither allocate device memory nor bring a workspace: a plugin or
 * serving callback that is handed only the tensors of the call, a host that has frozen its
 * allocator after start-up, a latency-critical loop in which cudaMalloc's implicit
 * synchronisation is not acceptable.  It has no counterpart in the reference, whose
 * SpMM_SplitK_API always needs a caller-allocated Reduction_Workspace.  Same result as
 * spmm_b200_spmm_splitk in unstructured mode; the fp32 partial tiles of rows shared between
 * thread blocks go to a 10 MiB array built into the library instead (each GPU that loads the
 * library holds it until the process exits).  Nothing is allocated or freed here, by the CUDA
 * runtime or any other library.  Limits: N in {8, 16, 32, 64}; M a multiple of 128 up to
 * 1,048,576; K a multiple of 64; and the partition's partial tiles must fit the 10 MiB -- a
 * shape beyond that is refused with a message and cudaErrorInvalidValue.  The first call on each
 * device looks up the array's device address (the device must be current); that first call
 * should come before any stream capture begins.  All calls on a device share the array and it keeps the previous
 * call's partial tiles (each slot is rewritten before it is read, so nothing needs clearing);
 * calls that overlap in time on one device race on it, and with every other SpMM of this
 * library through the shared arrival counters. */
int spmm_b200_spmm_own_scratch(void*       stream,
                               const void* Compressed_A,
                               const int*  TileOffsets,
                               const void* B,
                               void*       C,
                               int         M_Global,
                               int         N_Global,
                               int         K_Global);

/* Sum of the partial results of a row-parallel (split by K) layer, read out of the peers' memory over
 * NVLink by one kernel per rank; no counterpart in the reference (single-GPU; its FasterTransformer
 * glue all-reduces with NCCL).  partial_buffers[r] / flag_arrays[r]: rank r's partial result (count
 * halves, 16-byte aligned) and flag array (at least `world` 32-bit words, zero before the first
 * call), both mapped into this process (symmetric memory); host arrays of `world` device pointers.
 * out: local result, count halves.  epoch: 1, 2, 3, ... the same on every rank for the same call;
 * callers alternate between two sets of partial buffers from call to call.  Every rank must make
 * the matching call; a rank whose peers do not arrive within limit_ms (0 = 2000) leaves `out`
 * untouched and raises the status read by spmm_b200_allreduce_status.  One process per GPU. */
int spmm_b200_allreduce_partials(void*              stream,
                                 const void* const* partial_buffers,
                                 void* const*       flag_arrays,
                                 int                rank,
                                 int                world,
                                 void*              out,
                                 size_t             count,
                                 uint32_t           epoch,
                                 unsigned           limit_ms);
/* The same reduction for callers that capture it in a CUDA graph and replay it: the epoch is not an
 * argument but lives on the device.  state: two 32-bit words of this rank's device memory, zero before
 * the first call and used by nothing else; every launch reads its epoch from them and its last block
 * advances it, so every replay carries a new epoch.  All ranks must make the same sequence of calls
 * on the same state.  The partial buffers are fixed at capture time: between two launches that use
 * the same partial buffers there must be another exchange among the same ranks (a second set of
 * buffers used alternately, or another layer's reduction), otherwise a fast rank's next product
 * could overwrite what a slow peer is still reading. */
int spmm_b200_allreduce_partials_replayable(void*              stream,
                                            const void* const* partial_buffers,
                                            void* const*       flag_arrays,
                                            int                rank,
                                            int                world,
                                            void*              out,
                                            size_t             count,
                                            void*              state,
                                            unsigned           limit_ms);
/* spmm_b200_spmm_splitk (unstructured mode, N in {8, 16, 32, 64}) of one rank's K shard of a row-parallel
 * layer with the sum over the ranks folded into the kernel: no second launch and no collective library
 * on the critical path.  No counterpart in the reference (single-GPU; FasterTransformer all-reduces
 * after the product, third_party/ft.patch:2822-2846 is followed by its NCCL call).  Every rank writes
 * its finished rows into its own partial buffer; the last of its thread blocks to do so flags them to
 * all ranks, and the thread blocks then add the ranks' partial rows in rank order out of the peers'
 * memory (plain loads over NVLink, no multimem) into C; every rank ends up with the same bits.
 *   partial_buffers  host array of 2 * world device pointers, [parity * world + rank]: rank's partial
 *                    result of M * N floats (fp32, so that the sum is rounded to fp16 once) for calls
 *                    of that epoch parity, mapped into this process (symmetric memory); 16-byte aligned
 *   flag_arrays      host array of world device pointers: rank r's flag array of at least 2 * world
 *                    32-bit words, zero before the first call, mapped into this process
 *   state            two 32-bit words of this rank's own device memory, zero before the first call and
 *                    used by this sequence of calls only (the epoch lives there, so the call can be
 *                    captured in a CUDA graph and replayed)
 *   limit_ms         how long a block waits for the other ranks (0 = 2000); when it runs out C is left
 *                    incomplete and spmm_b200_device_status() reports 1
 *   partial_only     0: as described.  1: the kernel only writes this rank's fp32 partial rows (into the
 *                    buffer of the coming epoch's parity) and neither flags, sums nor advances the epoch:
 *                    spmm_b200_allreduce_partials_f32 on the same buffers, flag arrays and state, launched
 *                    next in the stream, does that (C is then not written by this call).
 *                    2: as 1, and the last block to finish also tells every rank that the partial rows
 *                    are complete; spmm_b200_allreduce_partials_f32_announced follows.  Measured on two
 *                    B200s the three forms take the same time within 1 % (the sum is bound by one
 *                    system-scope fence, one flag over NVLink and one round trip for the loads).
 * world 1..8 (1 degenerates to a copy through the partial buffer); every rank must make the matching
 * call.  One process per GPU; the ranks must not share a GPU (each waits for the others). */
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
                                int          partial_only);

/* The sum over ranks for spmm_b200_spmm_row_parallel(..., partial_only = 1): the replayable reduction
 * above on fp32 partial results, rounded to fp16 once.  partial_buffers: the same 2 * world pointers
 * (M * N floats each, [parity * world + rank]); flag_arrays: world pointers to at least `world` words
 * each; state: the two words shared with the SpMM calls (this kernel advances the epoch); out: count
 * halves. */
int spmm_b200_allreduce_partials_f32(void*              stream,
                                     const void* const* partial_buffers,
                                     void* const*       flag_arrays,
                                     int                rank,
                                     int                world,
                                     void*              out,
                                     size_t             count,
                                     void*              state,
                                     unsigned           limit_ms);

/* The sum over ranks after spmm_b200_spmm_row_parallel(..., partial_only = 2): that SpMM's last block has
 * already told every rank that this rank's partial rows are complete, so this kernel only waits for the
 * peers' flags, adds and writes (the flag exchange travels while this kernel is being launched).
 * Arguments as for spmm_b200_allreduce_partials_f32; must follow a partial_only = 2 product on the same
 * buffers, flag arrays and state. */
int spmm_b200_allreduce_partials_f32_announced(void*              stream,
                                               const void* const* partial_buffers,
                                               void* const*       flag_arrays,
                                               int                rank,
                                               int                world,
                                               void*              out,
                                               size_t             count,
                                               void*              state,
                                               unsigned           limit_ms);

/* The same sum in two phases, for larger worlds: every rank adds only its own 1 / world of the outputs
 * out of all ranks' fp32 partial results and writes the rounded slice into every rank's result buffer
 * (remote stores over NVLink), then a second flag exchange tells the peers that the slice has arrived;
 * the kernel completes when this rank's buffer is complete.  A rank then moves count * 6 bytes instead
 * of world * count * 4 (0.7 MB instead of 4.1 MB at eight ranks for a 9216 x 16 result).
 *   out_buffers   host array of world device pointers: rank r's result buffer of count halves, mapped
 *                 into this process (symmetric memory); 16-byte aligned
 *   flag_arrays   world pointers to at least 2 * world words each, zero before the first call
 *   count         a multiple of 8 * world
 * partial_buffers, state, limit_ms as for spmm_b200_allreduce_partials_f32.  Plain peer loads and
 * stores (no multimem).  Every rank gets the same bits.  Measured on 2 and 4 B200s with 9216 x 16
 * results this form is 3-5 us slower per sum than the one-phase form: the sums are bound by the flag
 * exchanges, not by the bytes, and this form has two. */
int spmm_b200_allreduce_partials_f32_two_phase(void*              stream,
                                               const void* const* partial_buffers,
                                               void* const*       flag_arrays,
                                               void* const*       out_buffers,
                                               int                rank,
                                               int                world,
                                               size_t             count,
                                               void*              state,
                                               unsigned           limit_ms);

/* 0, or 1 if a wait inside spmm_b200_allreduce_partials ran out (synchronises the device). */
int spmm_b200_allreduce_status(int reset);

/* Tells the library whether the weights of every SpMM (Compressed_A, TileOffsets, and in the
 * heterogeneous mode A and metadata) are constant while kernels run, as inference weights are.
 * The kernels are launched so that they may start while the kernel ahead of them in the stream is
 * still draining (programmatic dependent launch).  By default (0) they read nothing before that
 * predecessor has completed, so a stream in which the preceding kernel produces the weights
 * (dequantisation, a copy, a device-side encoder) is safe.  With 1 the weights and offsets are
 * fetched at once, ahead of the predecessor's completion, which hides the start-up of a launch
 * behind the end of the previous one; the caller then guarantees that the weights were complete
 * before the preceding kernel in the stream started (e.g. by one synchronisation after upload).
 * Process-wide; returns the previous setting.  No counterpart in the reference, whose launches are
 * fully serialised. */
int spmm_b200_set_weights_constant(int constant);

/* Widths that are multiples of 256 columns (prefill; beyond the reference's N <= 64) on matrices whose
 * M is a multiple of 256 run on pairs of SMs (tcgen05.mma.cta_group::2 over a cluster of two blocks:
 * each block restores the tiles of 128 of the pair's 256 rows and stages half of the columns of a B
 * slice; with N a multiple of 512 a restored tile serves 512 columns).  0 keeps such calls on the
 * single-block kernel that serves every other width (for comparison; the results of the two agree
 * within rounding, not bit for bit, because rows are split between blocks at different k).
 * At these widths a partial tile is 128 x 256 or 128 x 512 floats, so the workspace decides how many
 * rows can be split between SMs: size it with the Split_K that spmm_b200_suggest_split_k returns
 * (with less the call still succeeds, on fewer SMs).
 * Process-wide; returns the previous setting (default 1). */
int spmm_b200_set_pair_kernel(int enabled);

/* The reference's workspace contract, build/SpMM_API.cuh:34-38:
 * Split_K * M * N * sizeof(half) bytes. */
size_t spmm_b200_workspace_bytes(int M_Global, int N_Global, int Split_K);

/* decompose / decompose_v1, kernel_benchmark/spmm_decompose.h:12-51 and :53-142:
 * split A into a 2:4-compliant part A1 and the residual A2 (both dense, length
 * elements, caller-allocated). */
void spmm_b200_decompose(const uint16_t* A, uint16_t* A1, uint16_t* A2, int length);

/* Packs the structured half A1[M][K] (host, fp16 bits, at most two nonzeros in every aligned group
 * of four along K, e.g. the A1 that decompose returns) for the heterogeneous mode of
 * spmm_b200_spmm_splitk: *values (16 KB per 128 x 128 block) is passed as its argument A,
 * *metadata (2 KB per block) as its argument metadata, both copied to the device by the caller.
 * M and K multiples of 128.  Both arrays are malloc'd here and owned by the caller (free()).
 * Returns the number of blocks, or -1 (nothing allocated) if a shape or the 2:4 condition is
 * violated.  Takes the place of the reference's InitSparseMatrixA1_Vec_Sparse_Load +
 * inspect_metadata pair (csrc/SpMM_API.cu:1127-1553), whose formats serve its Ampere kernel. */
int spmm_b200_pack_a1(const uint16_t* A1, int M, int K, void** values, void** metadata);
void spmm_b200_decompose_v1(const uint16_t* A, uint16_t* A1, uint16_t* A2, int length);

/* Device-side status of the current device: 0 = ok, 1 = a bounded wait inside a
 * kernel gave up.  Synchronises the device.  With reset != 0 the status and the
 * arrival counters are cleared afterwards.  No counterpart in the reference,
 * whose kernels cannot report anything. */
int spmm_b200_device_status(int reset);

/* Failure-detection self test: launches one warp that waits on a barrier nothing arrives on, with a
 * limit of limit_ms (1..1000) milliseconds.  The bounded wait gives up, the kernel exits normally and
 * spmm_b200_device_status() then reports 1 until it is reset.  No counterpart in the reference. */
int spmm_b200_selftest_wait_timeout(void* stream, unsigned int limit_ms);

/* Seeded synthetic inputs (stand-ins for pruned model weights and
 * activations): element i of the stream is drawn from a counter-based
 * splitmix64 generator, value = fp16(sigma * gaussian), zeroed with
 * probability p_zero.  No counterpart in the reference, whose harness uses
 * rand() (kernel_benchmark/spmm_test_utils.h:108-162). */
void spmm_b200_synth_fp16(uint16_t* out, long count, uint64_t seed, double sigma, double p_zero);

/* The same stream, for the rows x cols block at (row0, col0) of a virtual row-major matrix with ld
 * columns (out is rows x cols, contiguous): element (r, c) of the block is element
 * (row0 + r) * ld + col0 + c of the stream.  Lets a tensor-parallel rank draw only its own shard
 * of a layer, identical to cutting it out of the whole matrix.  No counterpart in the reference. */
void spmm_b200_synth_fp16_block(
    uint16_t* out, long rows, long cols, long ld, long row0, long col0, uint64_t seed, double sigma, double p_zero);

/* Checks a tiled-CSL stream before it is given to the SpMM, whose kernels trust it (a word's position
 * addresses the tile buffer in shared memory, consecutive offsets size the copies): TileOffsets starts
 * at 0, never decreases, repeats its last entry ((M/128)*(K/64) + 2 entries), covers exactly n_words
 * words, and every position is below 128*64.  The reference asserts these inside its encoder only
 * (csrc/SpMM_API.cu:354-356, 380, 431); files can be truncated or corrupt.  Reads nothing beyond
 * n_words words and the offsets; never traps.  Returns 0 if well formed, a mask of the findings
 * below, or minus a cudaError_t.  The device version runs on `stream` and synchronises it. */
#define SPMM_B200_CSL_FIRST_OFFSET_NOT_ZERO 1
#define SPMM_B200_CSL_OFFSETS_DECREASE 2
#define SPMM_B200_CSL_TAIL_NOT_REPEATED 4
#define SPMM_B200_CSL_WORD_COUNT_MISMATCH 8
#define SPMM_B200_CSL_POSITION_OUT_OF_TILE 16
#define SPMM_B200_CSL_BAD_ARGUMENT 32
int spmm_b200_validate_tiled_csl(void* stream, const void* Compressed_A, size_t n_words, const int* TileOffsets, int M, int K);
int spmm_b200_validate_tiled_csl_host(const uint32_t* Compressed_A, size_t n_words, const int* TileOffsets, int M, int K);

/* Tensor-parallel shard shapes of the four linear layers of a decoder block (query_key_value,
 * attention.dense, dense_h_to_4h, dense_4h_to_h) on one of `world` ranks, as the reference's conversion
 * tool splits them (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:134-135):
 * M = {3h/g, h, 4h/g, h}, K = {h, h/g, h, 4h/g}.  Returns 0, or -1 if a shard is not a whole number
 * of 128 x 64 tiles. */
int spmm_b200_shard_shapes(int hidden, int world, int* M, int* K);

/* A Split_K for spmm_b200_spmm_splitk's workspace contract (Split_K * M * N halves) that is large
 * enough for the partition over all SMs of an M x K layer; takes the place of the reference's
 * hand-tuned table (huggingface_opt_convert_Phase2.py:20, kernel_benchmark/benchmark.sh:13-15).
 * 0 for shapes the format cannot describe. */
int spmm_b200_suggest_split_k(int M, int K);

/* Writes NNZ_List.<rank>.bin, NumOffsets_List.<rank>.bin and SplitK_List.<rank>.bin into model_dir
 * (huggingface_opt_convert_Phase2.py:183-195; read by third_party/ft.patch:2352-2401): one int32 per
 * (layer, matrix), matrices in the order above, from the .OutputSizes.bin that GenSparseMatrixBinFile
 * wrote for model.layers.<layer>.<matrix>.weight.<rank>; matrices without one (left dense) get 0.
 * M, K: the rank's four shard shapes.  Returns the number of sparse matrices found, -1 on an I/O error. */
int spmm_b200_write_rank_lists(const char* model_dir, int rank, int num_layers, const int* M, const int* K);

/* The work partition the SpMM kernel would use (for tests of the host logic):
 * fills chunk_begin[0..ctas] and split_rows_above[0..ctas-1], returns the
 * number of thread blocks; *slots_used gets the number of workspace slots. */
int spmm_b200_plan(int tiles_m, int tiles_k, int max_ctas, long slots_avail, int* chunk_begin, int* split_rows_above,
                   int* slots_used);

#ifdef __cplusplus
}
#endif
#endif
