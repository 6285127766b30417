"""Host-side mirror of the reference's SpMM API over the C boundary of libSpMM_API.so.

Function names and argument order follow the reference header
(build/SpMM_API.cuh:40-62) and the decompose entry points
(kernel_benchmark/spmm_decompose.h:12,53).  Everything here is a thin ctypes
call into the CUDA library; there is no Python or CPU implementation behind it,
and importing this module fails if the library cannot be built or loaded.
fp16 host data is carried as numpy float16/uint16 arrays, device data as torch
tensors (or raw integer device pointers).
"""
import ctypes

import numpy as np

from . import build as _build

class HostIoItem(ctypes.Structure):
    """spmm_b200_host_io_item of include/spmm_b200.h."""
    _fields_ = [("Compressed_A", ctypes.c_void_p), ("TileOffsets", ctypes.c_void_p), ("B_host", ctypes.c_void_p),
                ("C_host", ctypes.c_void_p), ("B_dev", ctypes.c_void_p), ("C_dev", ctypes.c_void_p),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("Reduction_Workspace", ctypes.c_void_p), ("Split_K", ctypes.c_int)]


_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_i32p = ctypes.POINTER(ctypes.c_int)

TILE_M = 128  # rows of an encoded tile (csrc/SpMM_API.cu:249)
TILE_K = 64   # columns of an encoded tile (csrc/TilingConfig.h:29)
SUPPORTED_N = (8, 16, 32, 64)  # csrc/SpMM_API.cu:105-196

cudaSuccess = 0
cudaErrorInvalidValue = 1
cudaErrorNotSupported = 801
cudaErrorUnknown = 999


def _load():
    path = _build.build()
    lib = ctypes.CDLL(path)
    enc_args = [_u16p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u32p), ctypes.POINTER(_i32p)]
    lib.spmm_b200_init_sparse_matrix_a.argtypes = enc_args
    lib.spmm_b200_init_sparse_matrix_a.restype = ctypes.c_int
    lib.spmm_b200_init_sparse_matrix_a_noreorder.argtypes = enc_args
    lib.spmm_b200_init_sparse_matrix_a_noreorder.restype = ctypes.c_int
    lib.spmm_b200_free.argtypes = [ctypes.c_void_p]
    lib.spmm_b200_free.restype = None
    lib.spmm_b200_spmm_splitk.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_void_p] + [ctypes.c_void_p] * 2 + \
        [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_int]
    lib.spmm_b200_spmm_splitk.restype = ctypes.c_int
    lib.spmm_b200_spmm_splitk_host_io.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_int]
    lib.spmm_b200_spmm_splitk_host_io.restype = ctypes.c_int
    lib.spmm_b200_spmm_splitk_host_io_batch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(HostIoItem)]
    lib.spmm_b200_spmm_splitk_host_io_batch.restype = ctypes.c_int
    lib.spmm_b200_spmm_own_scratch.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3
    lib.spmm_b200_spmm_own_scratch.restype = ctypes.c_int
    lib.spmm_b200_spmm_splitk_token_major.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_int]
    lib.spmm_b200_spmm_splitk_token_major.restype = ctypes.c_int
    lib.spmm_b200_pack_a1.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                      ctypes.POINTER(ctypes.c_void_p)]
    lib.spmm_b200_pack_a1.restype = ctypes.c_int
    lib.spmm_b200_allreduce_partials.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                                 ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint32,
                                                 ctypes.c_uint]
    lib.spmm_b200_allreduce_partials.restype = ctypes.c_int
    lib.spmm_b200_allreduce_partials_replayable.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                                            ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int,
                                                            ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_uint]
    lib.spmm_b200_allreduce_partials_replayable.restype = ctypes.c_int
    lib.spmm_b200_spmm_row_parallel.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_int] + \
        [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
         ctypes.c_uint, ctypes.c_int]
    lib.spmm_b200_spmm_row_parallel.restype = ctypes.c_int
    lib.spmm_b200_allreduce_partials_f32.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                                     ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int,
                                                     ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_uint]
    lib.spmm_b200_allreduce_partials_f32.restype = ctypes.c_int
    lib.spmm_b200_allreduce_partials_f32_announced.argtypes = lib.spmm_b200_allreduce_partials_f32.argtypes
    lib.spmm_b200_allreduce_partials_f32_announced.restype = ctypes.c_int
    lib.spmm_b200_allreduce_partials_f32_two_phase.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                                               ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                                               ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p,
                                                               ctypes.c_uint]
    lib.spmm_b200_allreduce_partials_f32_two_phase.restype = ctypes.c_int
    lib.spmm_b200_allreduce_status.argtypes = [ctypes.c_int]
    lib.spmm_b200_allreduce_status.restype = ctypes.c_int
    lib.spmm_b200_set_weights_constant.argtypes = [ctypes.c_int]
    lib.spmm_b200_set_weights_constant.restype = ctypes.c_int
    lib.spmm_b200_set_pair_kernel.argtypes = [ctypes.c_int]
    lib.spmm_b200_set_pair_kernel.restype = ctypes.c_int
    lib.spmm_b200_workspace_bytes.argtypes = [ctypes.c_int] * 3
    lib.spmm_b200_workspace_bytes.restype = ctypes.c_size_t
    for name in ("spmm_b200_decompose", "spmm_b200_decompose_v1"):
        f = getattr(lib, name)
        f.argtypes = [_u16p, _u16p, _u16p, ctypes.c_int]
        f.restype = None
    lib.spmm_b200_device_status.argtypes = [ctypes.c_int]
    lib.spmm_b200_device_status.restype = ctypes.c_int
    lib.spmm_b200_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_uint]
    lib.spmm_b200_selftest_wait_timeout.restype = ctypes.c_int
    lib.spmm_b200_synth_fp16.argtypes = [_u16p, ctypes.c_long, ctypes.c_uint64, ctypes.c_double, ctypes.c_double]
    lib.spmm_b200_synth_fp16.restype = None
    lib.spmm_b200_synth_fp16_block.argtypes = [_u16p] + [ctypes.c_long] * 5 + [ctypes.c_uint64, ctypes.c_double, ctypes.c_double]
    lib.spmm_b200_synth_fp16_block.restype = None
    lib.spmm_b200_validate_tiled_csl.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                                 ctypes.c_int, ctypes.c_int]
    lib.spmm_b200_validate_tiled_csl.restype = ctypes.c_int
    lib.spmm_b200_validate_tiled_csl_host.argtypes = [_u32p, ctypes.c_size_t, _i32p, ctypes.c_int, ctypes.c_int]
    lib.spmm_b200_validate_tiled_csl_host.restype = ctypes.c_int
    lib.spmm_b200_shard_shapes.argtypes = [ctypes.c_int, ctypes.c_int, _i32p, _i32p]
    lib.spmm_b200_shard_shapes.restype = ctypes.c_int
    lib.spmm_b200_suggest_split_k.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.spmm_b200_suggest_split_k.restype = ctypes.c_int
    lib.spmm_b200_write_rank_lists.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, _i32p, _i32p]
    lib.spmm_b200_write_rank_lists.restype = ctypes.c_int
    lib.spmm_b200_plan.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_long, _i32p, _i32p, _i32p]
    lib.spmm_b200_plan.restype = ctypes.c_int
    lib.GenSparseMatrixBinFile.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p,
                                           ctypes.c_char_p]
    lib.GenSparseMatrixBinFile.restype = None
    return lib


LIB = _load()
LIB_PATH = _build.LIB_PATH


def _host_u16(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    if a.dtype != np.uint16:
        raise TypeError("fp16 host data must be float16 or uint16, got %s" % a.dtype)
    return a


def _encode(fn, A_h, M, N, K):
    A_h = _host_u16(A_h)
    if A_h.size != M * K:
        raise ValueError("A_h has %d elements, expected M*K = %d" % (A_h.size, M * K))
    wp, op = _u32p(), _i32p()
    n_offsets = fn(A_h.ctypes.data_as(_u16p), M, N, K, ctypes.byref(wp), ctypes.byref(op))
    if n_offsets < 0:
        raise ValueError("M must be a positive multiple of %d and K of %d (got M=%d, K=%d)" % (TILE_M, TILE_K, M, K))
    offsets = np.ctypeslib.as_array(op, shape=(n_offsets,)).copy()
    n_words = int(offsets[-1]) * 4
    words = np.ctypeslib.as_array(wp, shape=(max(n_words, 1),))[:n_words].copy()
    LIB.spmm_b200_free(ctypes.cast(wp, ctypes.c_void_p))
    LIB.spmm_b200_free(ctypes.cast(op, ctypes.c_void_p))
    return words, offsets, n_offsets


def InitSparseMatrixA_API(A_h, M, N, K):
    """Dense host A[M][K] -> (Compressed_A uint32 words, TileOffsets int32, NumOffsets).

    Same output as the reference's InitSparseMatrixA_API (csrc/SpMM_API.cu:241-438);
    NumOffsets is its return value and 4 * TileOffsets[-1] the word count."""
    return _encode(LIB.spmm_b200_init_sparse_matrix_a, A_h, M, N, K)


def InitSparseMatrixA_API_NoReorder(A_h, M, N, K):
    """Scan-order variant (csrc/SpMM_API.cu:441-567)."""
    return _encode(LIB.spmm_b200_init_sparse_matrix_a_noreorder, A_h, M, N, K)


def _dev_ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if not x.is_cuda:
        raise ValueError("expected a CUDA tensor")
    if not x.is_contiguous():
        raise ValueError("expected a contiguous tensor")
    return ctypes.c_void_p(x.data_ptr())


def SpMM_SplitK_API(stream, A, Compressed_A, A1_Ind_data, metadata, TileOffsets, B, C, M_Global, N_Global, K_Global,
                    Reduction_Workspace, Split_K):
    """C[M][N] = A_sparse * B on `stream` (a torch.cuda.Stream, a raw handle, or None for the current stream).

    Argument order and meaning as in the reference (build/SpMM_API.cuh:40-52).
    Returns the cudaError_t of the launch as an int (0 = success); asynchronous."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    handle = stream if isinstance(stream, int) else stream.cuda_stream
    return LIB.spmm_b200_spmm_splitk(ctypes.c_void_p(handle), _dev_ptr(A), _dev_ptr(Compressed_A), _dev_ptr(A1_Ind_data),
                                     _dev_ptr(metadata), _dev_ptr(TileOffsets), _dev_ptr(B), _dev_ptr(C), M_Global,
                                     N_Global, K_Global, _dev_ptr(Reduction_Workspace), Split_K)


def SpMM_SplitK_API_host_io(stream, Compressed_A, TileOffsets, B_host, C_host, B_dev, C_dev, M_Global, N_Global, K_Global,
                            Reduction_Workspace, Split_K):
    """SpMM_SplitK_API for activations and results in (page-locked) host memory: one call that copies
    B_host to B_dev, multiplies and copies C_dev to C_host, all on `stream`.  B_host / C_host: CPU
    tensors; the rest CUDA tensors.  Returns the first cudaError_t met as an int."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    handle = stream if isinstance(stream, int) else stream.cuda_stream
    if B_host.is_cuda or C_host.is_cuda:
        raise ValueError("B_host and C_host must be CPU tensors")
    return LIB.spmm_b200_spmm_splitk_host_io(ctypes.c_void_p(handle), _dev_ptr(Compressed_A), _dev_ptr(TileOffsets),
                                             ctypes.c_void_p(B_host.data_ptr()), ctypes.c_void_p(C_host.data_ptr()),
                                             _dev_ptr(B_dev), _dev_ptr(C_dev), M_Global, N_Global, K_Global,
                                             _dev_ptr(Reduction_Workspace), Split_K)


def host_io_items(layers):
    """Packs dicts with the keys of spmm_b200_host_io_item (tensors or raw pointers) into a ctypes array for
    SpMM_SplitK_API_host_io_batch; build it once and reuse it."""
    arr = (HostIoItem * len(layers))()
    for item, L in zip(arr, layers):
        for key in ("Compressed_A", "TileOffsets", "B_dev", "C_dev", "Reduction_Workspace"):
            setattr(item, key, _dev_ptr(L[key]).value if L[key] is not None else None)
        for key in ("B_host", "C_host"):
            if L[key].is_cuda:
                raise ValueError("%s must be a CPU tensor" % key)
            setattr(item, key, L[key].data_ptr())
        item.M, item.N, item.K, item.Split_K = L["M"], L["N"], L["K"], L["Split_K"]
    return arr


def SpMM_SplitK_API_host_io_batch(stream, items):
    """Several host-buffer products in one call (e.g. the layers of a decoder block): activations are copied in on a
    copy stream ahead of the products, each result is copied out while the next product runs.  `items`: what
    host_io_items returned.  After the call `stream` waits for the last copy.  Returns a cudaError_t as an int."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    handle = stream if isinstance(stream, int) else stream.cuda_stream
    return LIB.spmm_b200_spmm_splitk_host_io_batch(ctypes.c_void_p(handle), len(items), items)


def SpMM_SplitK_API_token_major(stream, Compressed_A, TileOffsets, B, C, M_Global, N_Global, K_Global,
                                Reduction_Workspace, Split_K):
    """The upstream eleven-argument form the FasterTransformer glue calls (third_party/ft.patch:2822-2846):
    token-major activations B[N][K] and results C[N][M]."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    handle = stream if isinstance(stream, int) else stream.cuda_stream
    return LIB.spmm_b200_spmm_splitk_token_major(ctypes.c_void_p(handle), _dev_ptr(Compressed_A), _dev_ptr(TileOffsets),
                                                 _dev_ptr(B), _dev_ptr(C), M_Global, N_Global, K_Global,
                                                 _dev_ptr(Reduction_Workspace), Split_K)


def spmm_own_scratch(stream, Compressed_A, TileOffsets, B, C, M_Global, N_Global, K_Global):
    """SpMM for callers that cannot allocate or pass a workspace: partial tiles go to a 10 MiB array
    built into the library.  Same result as SpMM_SplitK_API; returns the cudaError_t as an int.
    Make the first call on a device before any stream capture begins; calls on one device must not overlap."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    handle = stream if isinstance(stream, int) else stream.cuda_stream
    return LIB.spmm_b200_spmm_own_scratch(ctypes.c_void_p(handle), _dev_ptr(Compressed_A), _dev_ptr(TileOffsets),
                                          _dev_ptr(B), _dev_ptr(C), M_Global, N_Global, K_Global)


def set_weights_constant(constant=True):
    """Whether weights may be fetched before the stream predecessor has completed (see include/spmm_b200.h:
    the caller guarantees they are not produced by the kernel just ahead).  Returns the previous setting."""
    return bool(LIB.spmm_b200_set_weights_constant(1 if constant else 0))


def set_pair_kernel(enabled=True):
    """Whether widths that are multiples of 256 run on pairs of SMs (include/spmm_b200.h).  Returns the previous setting."""
    return bool(LIB.spmm_b200_set_pair_kernel(1 if enabled else 0))


def workspace_bytes(M_Global, N_Global, Split_K):
    """The reference's workspace contract: Split_K * M * N * sizeof(half) (build/SpMM_API.cuh:34-38)."""
    return int(LIB.spmm_b200_workspace_bytes(M_Global, N_Global, Split_K))


def decompose(A, v1=False):
    """2:4 part + residual (kernel_benchmark/spmm_decompose.h:12-51, v1 :53-142). Returns (A1, A2) as uint16 bits."""
    A = _host_u16(A)
    flat = A.reshape(-1)
    if flat.size % 4:
        raise ValueError("length must be a multiple of 4")
    A1 = np.empty_like(flat)
    A2 = np.empty_like(flat)
    fn = LIB.spmm_b200_decompose_v1 if v1 else LIB.spmm_b200_decompose
    fn(flat.ctypes.data_as(_u16p), A1.ctypes.data_as(_u16p), A2.ctypes.data_as(_u16p), flat.size)
    return A1.reshape(A.shape), A2.reshape(A.shape)


def InitSparseMatrixA1_tcgen05(A1_h, M, K):
    """Packs the structured half A1[M][K] (at most two nonzeros per aligned group of four along K, as
    `decompose` returns it) for the heterogeneous mode of SpMM_SplitK_API.

    Returns (values, metadata, blocks): uint8 array of 16 KB per 128 x 128 block (argument A of
    SpMM_SplitK_API once on the device) and uint32 array of 2 KB per block (argument metadata).
    Raises ValueError on a violated precondition."""
    A1_h = _host_u16(A1_h)
    if A1_h.size != M * K:
        raise ValueError("A1 must hold M * K halves")
    values, meta = ctypes.c_void_p(), ctypes.c_void_p()
    blocks = LIB.spmm_b200_pack_a1(A1_h.ctypes.data_as(_u16p), M, K, ctypes.byref(values), ctypes.byref(meta))
    if blocks < 0:
        raise ValueError("M and K must be multiples of 128 and A1 must hold at most two nonzeros per group of four")
    try:
        v = np.ctypeslib.as_array(ctypes.cast(values, ctypes.POINTER(ctypes.c_uint8)), shape=(blocks * 16384,)).copy()
        m = np.ctypeslib.as_array(ctypes.cast(meta, ctypes.POINTER(ctypes.c_uint32)), shape=(blocks * 512,)).copy()
    finally:
        LIB.spmm_b200_free(values)
        LIB.spmm_b200_free(meta)
    return v, m, blocks


def GenSparseMatrixBinFile(dense_path, M, K, nz_path, offsets_path, sizes_path):
    """File front end used by the weight-conversion tools (csrc/SpMM_API.cu:1565-1620)."""
    LIB.GenSparseMatrixBinFile(dense_path.encode(), M, K, nz_path.encode(), offsets_path.encode(), sizes_path.encode())


CSL_FINDINGS = {1: "first offset not zero", 2: "offsets decrease", 4: "last offset not repeated",
                8: "offsets do not cover the words given", 16: "a position lies outside the tile", 32: "bad argument"}


def validate_tiled_csl(words, offsets, M, K, stream=None):
    """0 if the tiled-CSL stream is well formed, else a mask of CSL_FINDINGS keys.  numpy arrays are checked on the
    host, CUDA tensors by a kernel on `stream` (which is synchronised)."""
    if isinstance(words, np.ndarray):
        words = np.ascontiguousarray(words, dtype=np.uint32)
        offsets = np.ascontiguousarray(offsets, dtype=np.int32)
        if offsets.size != (M // TILE_M) * (K // TILE_K) + 2:
            return 32
        return int(LIB.spmm_b200_validate_tiled_csl_host(words.ctypes.data_as(_u32p), words.size,
                                                          offsets.ctypes.data_as(_i32p), M, K))
    import torch
    if offsets.numel() != (M // TILE_M) * (K // TILE_K) + 2:
        return 32
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(LIB.spmm_b200_validate_tiled_csl(ctypes.c_void_p(stream.cuda_stream), _dev_ptr(words), words.numel(),
                                                _dev_ptr(offsets), M, K))


def shard_shapes(hidden, world):
    """(M[4], K[4]) of one rank's shards of query_key_value, attention.dense, dense_h_to_4h, dense_4h_to_h."""
    M, K = (ctypes.c_int * 4)(), (ctypes.c_int * 4)()
    if LIB.spmm_b200_shard_shapes(hidden, world, M, K) != 0:
        raise ValueError("hidden size %d cannot be split %d ways into whole tiles" % (hidden, world))
    return list(M), list(K)


def suggest_split_k(M, K):
    """A Split_K whose workspace (Split_K * M * N halves) holds the partial tiles of the partition over all SMs."""
    return int(LIB.spmm_b200_suggest_split_k(M, K))


def write_rank_lists(model_dir, rank, num_layers, M, K):
    """Writes NNZ_List/NumOffsets_List/SplitK_List.<rank>.bin from the .OutputSizes.bin files in model_dir."""
    n = LIB.spmm_b200_write_rank_lists(model_dir.encode(), rank, num_layers, (ctypes.c_int * 4)(*M), (ctypes.c_int * 4)(*K))
    if n < 0:
        raise OSError("could not read the sizes files or write the list files in " + model_dir)
    return n


def device_status(reset=False):
    """0 if no kernel on the current device ever abandoned a wait; synchronises the device."""
    return int(LIB.spmm_b200_device_status(1 if reset else 0))


def selftest_wait_timeout(limit_ms=50):
    """Launches a wait that nothing satisfies; device_status() must report 1 afterwards (then reset it)."""
    import torch
    return int(LIB.spmm_b200_selftest_wait_timeout(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), limit_ms))


def synth_fp16(shape, seed, sigma, p_zero=0.0):
    """Seeded synthetic fp16 data (uint16 bits): sigma * N(0,1), zeroed with probability p_zero."""
    out = np.empty(shape, np.uint16)
    LIB.spmm_b200_synth_fp16(out.ctypes.data_as(_u16p), out.size, seed, float(sigma), float(p_zero))
    return out


def synth_fp16_block(rows, cols, ld, row0, col0, seed, sigma, p_zero=0.0):
    """The rows x cols block at (row0, col0) of the matrix synth_fp16((R, ld), seed, ...) would return."""
    out = np.empty((rows, cols), np.uint16)
    LIB.spmm_b200_synth_fp16_block(out.ctypes.data_as(_u16p), rows, cols, ld, row0, col0, seed, float(sigma), float(p_zero))
    return out


def plan(tiles_m, tiles_k, max_ctas, slots_avail):
    """The kernel's work partition: (chunk_begin[ctas+1], split_rows_above[ctas], slots_used)."""
    cb = np.zeros(320, np.int32)
    ab = np.zeros(320, np.int32)
    used = ctypes.c_int(0)
    n = LIB.spmm_b200_plan(tiles_m, tiles_k, max_ctas, slots_avail, cb.ctypes.data_as(_i32p), ab.ctypes.data_as(_i32p),
                           ctypes.byref(used))
    return cb[:n + 1].copy(), ab[:n].copy(), used.value
