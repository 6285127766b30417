"""CPU checkers for the sparse-weight SpMM path.  TEST INFRASTRUCTURE ONLY.

Two shared objects sit behind this module, both built by ``oracle/Makefile``:

* ``liboracle.so``  -- the plain-C restatement in ``tiled_csl_oracle.c``
  (every function cites the reference lines it follows);
* ``_ref/libSpMM_API_ref.so`` -- the reference's own ``csrc/SpMM_API.cu``
  compiled unchanged; its host encoders run without a GPU and are what the
  restatement is pinned against.

Nothing in the product package imports this module.  Only the tests, the
smoke check and the benchmark's CPU-baseline leg do, and only as the checker.
fp16 data crosses this boundary as ``numpy.uint16`` bit patterns.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libSpMM_API_ref.so")

_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_i32p = ctypes.POINTER(ctypes.c_int)
_f64p = ctypes.POINTER(ctypes.c_double)


def build():
    """Compile the C restatement and, when the reference tree is present (REFERENCE_ROOT in the environment, or a
    directory named `reference` beside this repository), the reference libraries."""
    beside = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    root = os.environ.get("REFERENCE_ROOT") or (beside if os.path.isfile(os.path.join(beside, "csrc", "SpMM_API.cu")) else "")
    import fcntl
    with open(os.path.join(_HERE, ".build.lock"), "w") as lock:  # several ranks of one job may get here at once
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            subprocess.check_call(["make", "-s", "-C", _HERE] + (["REFERENCE_ROOT=" + root] if root else []))
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_lib = None
_ref = None
_libc = ctypes.CDLL(None)
_libc.free.argtypes = [ctypes.c_void_p]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            build()
        L = ctypes.CDLL(_ORACLE_SO)
        for name in ("oracle_init_sparse_matrix_a", "oracle_init_sparse_matrix_a_noreorder"):
            f = getattr(L, name)
            f.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u32p), ctypes.POINTER(_i32p)]
            f.restype = ctypes.c_int
        L.oracle_decode_tiled_csl.argtypes = [_u32p, _i32p, ctypes.c_int, ctypes.c_int, _u16p]
        L.oracle_decode_tiled_csl.restype = ctypes.c_int
        L.oracle_spmm_f32.argtypes = [_u16p, _u16p, _u16p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.oracle_spmm_f32.restype = None
        L.oracle_spmm_f64.argtypes = [_u16p, _u16p, _f64p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.oracle_spmm_f64.restype = None
        L.oracle_spmm_from_csl.argtypes = [_u32p, _i32p, _u16p, _u16p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.oracle_spmm_from_csl.restype = ctypes.c_int
        for name in ("oracle_decompose", "oracle_decompose_v1"):
            f = getattr(L, name)
            f.argtypes = [_u16p, _u16p, _u16p, ctypes.c_int]
            f.restype = None
        L.oracle_synth_fp16_block.argtypes = [_u16p] + [ctypes.c_long] * 5 + [ctypes.c_uint64, ctypes.c_double, ctypes.c_double]
        L.oracle_synth_fp16_block.restype = None
        _lib = L
    return _lib


def have_ref():
    return os.path.exists(_REF_SO)


_REF_DECOMPOSE_SO = os.path.join(_HERE, "_ref", "libdecompose_ref.so")


def have_ref_decompose():
    return os.path.exists(_REF_DECOMPOSE_SO)


def ref_decompose(A, v1=False):
    """decompose / decompose_v1 of the compiled reference header (kernel_benchmark/spmm_decompose.h:12,53).
    Prints the reference's statistics lines to stdout, as the reference does."""
    R = ctypes.CDLL(_REF_DECOMPOSE_SO)
    fn = getattr(R, "_Z12decompose_v1P6__halfS0_S0_i" if v1 else "_Z9decomposeP6__halfS0_S0_i")
    fn.argtypes = [_u16p, _u16p, _u16p, ctypes.c_int]
    fn.restype = None
    A = _as_u16(A)
    flat = np.ascontiguousarray(A.reshape(-1))
    A1 = np.empty_like(flat)
    A2 = np.empty_like(flat)
    fn(flat.ctypes.data_as(_u16p), A1.ctypes.data_as(_u16p), A2.ctypes.data_as(_u16p), flat.size)
    return A1.reshape(A.shape), A2.reshape(A.shape)


# Itanium-mangled names of the reference's C++ entry points (build/SpMM_API.cuh:54-96).
_REF_ENCODERS = {
    "reorder": "_Z21InitSparseMatrixA_APIP6__halfiiiPPjPPi",
    "noreorder": "_Z31InitSparseMatrixA_API_NoReorderP6__halfiiiPPjPPi",
    "noreorder_v1": "_Z34InitSparseMatrixA_API_NoReorder_v1P6__halfiiiPPjPPi",
}


def ref():
    """The compiled reference library (raises if it was never built here)."""
    global _ref
    if _ref is None:
        if not have_ref():
            raise FileNotFoundError(_REF_SO + " (run `make -C oracle` where the reference tree is mounted)")
        R = ctypes.CDLL(_REF_SO)
        for sym in _REF_ENCODERS.values():
            f = getattr(R, sym)
            f.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u32p), ctypes.POINTER(_i32p)]
            f.restype = ctypes.c_int
        _ref = R
    return _ref


def _as_u16(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


def _take(words_p, offs_p, n_offs):
    offs = np.ctypeslib.as_array(offs_p, shape=(n_offs,)).copy()
    n_words = int(offs[-1]) * 4
    words = np.ctypeslib.as_array(words_p, shape=(max(n_words, 1),))[:n_words].copy()
    _libc.free(ctypes.cast(words_p, ctypes.c_void_p))
    _libc.free(ctypes.cast(offs_p, ctypes.c_void_p))
    return words, offs


def encode(A, variant="reorder"):
    """Tiled-CSL encode with the C restatement. Returns (uint32 words, int32 offsets)."""
    A = _as_u16(A)
    M, K = A.shape
    fn = {"reorder": lib().oracle_init_sparse_matrix_a, "noreorder": lib().oracle_init_sparse_matrix_a_noreorder}[variant]
    wp, op = _u32p(), _i32p()
    n = fn(A.ctypes.data_as(_u16p), M, K, ctypes.byref(wp), ctypes.byref(op))
    if n < 0:
        raise ValueError("M must be a multiple of 128 and K of 64")
    return _take(wp, op, n)


def ref_encode(A, variant="reorder", N=16):
    """Tiled-CSL encode with the reference's own compiled encoder."""
    A = _as_u16(A)
    M, K = A.shape
    fn = getattr(ref(), _REF_ENCODERS[variant])
    wp, op = _u32p(), _i32p()
    n = fn(A.ctypes.data_as(_u16p), M, N, K, ctypes.byref(wp), ctypes.byref(op))
    return _take(wp, op, n)


def decode(words, offsets, M, K):
    words = np.ascontiguousarray(words, dtype=np.uint32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    if words.size == 0:
        words = np.zeros(1, np.uint32)
    dense = np.empty((M, K), np.uint16)
    rc = lib().oracle_decode_tiled_csl(words.ctypes.data_as(_u32p), offsets.ctypes.data_as(_i32p), M, K, dense.ctypes.data_as(_u16p))
    if rc != 0:
        raise ValueError("malformed tiled-CSL stream")
    return dense


def spmm_f32(A, B):
    """fp32-accumulate host product, fp16 result (uint16 bits), row-major C[M][N]."""
    A, B = _as_u16(A), _as_u16(B)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    C = np.empty((M, N), np.uint16)
    lib().oracle_spmm_f32(A.ctypes.data_as(_u16p), B.ctypes.data_as(_u16p), C.ctypes.data_as(_u16p), M, N, K)
    return C


def spmm_f64(A, B):
    """fp64 host product (the tolerance oracle)."""
    A, B = _as_u16(A), _as_u16(B)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    C = np.empty((M, N), np.float64)
    lib().oracle_spmm_f64(A.ctypes.data_as(_u16p), B.ctypes.data_as(_u16p), C.ctypes.data_as(_f64p), M, N, K)
    return C


def synth_fp16_block(rows, cols, ld, row0, col0, seed, sigma, p_zero=0.0, threads=None):
    """Seeded synthetic fp16 bits: the rows x cols block at (row0, col0) of a virtual matrix with ld columns
    (bit-identical to the product library's generator, written independently); row blocks on host threads."""
    import threading
    out = np.empty((rows, cols), np.uint16)
    threads = max(1, min(threads or (os.cpu_count() or 1), 64, rows))
    bounds = [rows * t // threads for t in range(threads + 1)]

    def work(t):
        r0, r1 = bounds[t], bounds[t + 1]
        if r1 > r0:
            lib().oracle_synth_fp16_block(out[r0:r1].ctypes.data_as(_u16p), r1 - r0, cols, ld, row0 + r0, col0, seed,
                                          float(sigma), float(p_zero))

    lib()
    pool = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
    for th in pool:
        th.start()
    for th in pool:
        th.join()
    return out


def spmm_f64_threads(A, B, threads=None):
    """spmm_f64 over row blocks on several host threads (the C loop releases the interpreter lock)."""
    import threading
    A = _as_u16(A)
    M = A.shape[0]
    threads = max(1, min(threads or int(os.environ.get("SPMM_B200_THREADS", 0)) or (os.cpu_count() or 1), 32, M))
    out = np.empty((M, B.shape[1]), np.float64)
    bounds = [M * t // threads for t in range(threads + 1)]

    def work(t):
        if bounds[t + 1] > bounds[t]:
            out[bounds[t]:bounds[t + 1]] = spmm_f64(A[bounds[t]:bounds[t + 1]], B)

    pool = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
    for th in pool:
        th.start()
    for th in pool:
        th.join()
    return out


def spmm_from_csl(words, offsets, B, M, K):
    words = np.ascontiguousarray(words, dtype=np.uint32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    B = _as_u16(B)
    N = B.shape[1]
    C = np.empty((M, N), np.uint16)
    rc = lib().oracle_spmm_from_csl(words.ctypes.data_as(_u32p), offsets.ctypes.data_as(_i32p), B.ctypes.data_as(_u16p),
                                    C.ctypes.data_as(_u16p), M, N, K)
    if rc != 0:
        raise ValueError("malformed tiled-CSL stream")
    return C


def decompose(A, v1=False):
    A = _as_u16(A)
    flat = A.reshape(-1)
    A1 = np.empty_like(flat)
    A2 = np.empty_like(flat)
    fn = lib().oracle_decompose_v1 if v1 else lib().oracle_decompose
    fn(flat.ctypes.data_as(_u16p), A1.ctypes.data_as(_u16p), A2.ctypes.data_as(_u16p), flat.size)
    return A1.reshape(A.shape), A2.reshape(A.shape)


def tolerance_check(C_half_bits, C64, tiny=1e-6):
    """The acceptance gates for C: max |err| <= 1e-2 * max|C64| and
    mean(|err| / max(|C64|, tiny)) <= 1e-3.  Returns (ok, max_err_ratio, mean_rel)."""
    C = _as_u16(C_half_bits).view(np.float16).astype(np.float64)
    err = np.abs(C - C64)
    peak = float(np.max(np.abs(C64))) if C64.size else 0.0
    max_ratio = float(err.max() / peak) if peak > 0 else float(err.max() if err.size else 0.0)
    mean_rel = float(np.mean(err / np.maximum(np.abs(C64), tiny))) if err.size else 0.0
    return (max_ratio <= 1e-2 and mean_rel <= 1e-3), max_ratio, mean_rel
