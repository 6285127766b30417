"""ctypes access to the 2:4-oriented host encoders (C++ symbols shared by the reference's library and
this one) and the seeded inputs used for their golden digests.

    python tests/golden/structured_formats.py      # regenerate structured_digests.json from oracle/_ref
"""
import ctypes
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_u64p = ctypes.POINTER(ctypes.c_uint64)
_i32p = ctypes.POINTER(ctypes.c_int)
_libc = ctypes.CDLL(None)
_libc.free.argtypes = [ctypes.c_void_p]

SYMBOLS = {
    "v1": "_Z34InitSparseMatrixA_API_NoReorder_v1P6__halfiiiPPjPPi",
    "v2": "_Z34InitSparseMatrixA_API_NoReorder_v2P6__halfiiiPS0_PPi",
    "v3": "_Z34InitSparseMatrixA_API_NoReorder_v3P6__halfiiiPS0_PPi",
    "v4": "_Z34InitSparseMatrixA_API_NoReorder_v4P6__halfiiiPS0_PPi",
    "a1": "_Z34InitSparseMatrixA1_Vec_Sparse_LoadP6__halfiiPS0_PPmPPi",
    "meta": "_Z16inspect_metadataP6__halfPiii",
}
CASES = [("m256_k128", 256, 128, 31), ("m512_k256", 512, 256, 32), ("m256_k512", 256, 512, 33)]


def two_four_input(M, K, seed, density=0.9):
    """A 2:4-compliant matrix (at most two nonzeros per aligned group of four), no empty 256 x 64 tile."""
    rng = np.random.default_rng(seed)
    A = (rng.standard_normal((M, K)) * 0.02).astype(np.float16)
    g = A.reshape(M, K // 4, 4)
    order = np.argsort(-np.abs(g.astype(np.float32)), axis=2)
    keep = np.zeros_like(g, dtype=bool)
    np.put_along_axis(keep, order[:, :, :2], True, axis=2)
    keep &= rng.random(g.shape) < density
    return np.where(keep, g, np.float16(0)).reshape(M, K).view(np.uint16).copy()


def multiple_of_eight_input(M, K, seed):
    """Unstructured input whose every 128 x 64 tile holds a multiple of eight nonzeros (what v2 asserts)."""
    rng = np.random.default_rng(seed)
    A = np.zeros((M, K), np.uint16)
    for i in range(M // 128):
        for j in range(K // 64):
            n = 8 * int(rng.integers(50, 300))
            idx = rng.choice(128 * 64, n, replace=False)
            tile = np.zeros(128 * 64, np.uint16)
            tile[idx] = (rng.standard_normal(n) * 0.02).astype(np.float16).view(np.uint16) | 0x0001
            A[i * 128:(i + 1) * 128, j * 64:(j + 1) * 64] = tile.reshape(128, 64)
    return A


def run(lib, which, A):
    """Calls encoder `which` of library `lib`; returns a dict of numpy arrays (copies)."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    M, K = A.shape
    fn = getattr(lib, SYMBOLS[which])
    op = _i32p()
    if which == "meta":
        meta = np.zeros((M // 16) * (K // 16) * 8, np.int32)
        fn.argtypes = [_u16p, _i32p, ctypes.c_int, ctypes.c_int]
        fn.restype = None
        fn(A.ctypes.data_as(_u16p), meta.ctypes.data_as(_i32p), M, K)
        return {"meta": meta}
    if which == "a1":
        vp, ip = _u16p(), _u64p()
        fn.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u16p), ctypes.POINTER(_u64p), ctypes.POINTER(_i32p)]
        fn.restype = ctypes.c_int
        n = fn(A.ctypes.data_as(_u16p), M, K, ctypes.byref(vp), ctypes.byref(ip), ctypes.byref(op))
        offsets = np.ctypeslib.as_array(op, shape=(n,)).copy()
        vectors = int(offsets[-1])
        out = {"offsets": offsets, "values": np.ctypeslib.as_array(vp, shape=(vectors * 8,)).copy(),
               "index": np.ctypeslib.as_array(ip, shape=(vectors,)).copy()}
        for p in (vp, ip, op):
            _libc.free(ctypes.cast(p, ctypes.c_void_p))
        return out
    if which == "v1":
        wp = _u32p()
        fn.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u32p), ctypes.POINTER(_i32p)]
    else:
        wp = _u16p()
        fn.argtypes = [_u16p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u16p), ctypes.POINTER(_i32p)]
    fn.restype = ctypes.c_int
    n = fn(A.ctypes.data_as(_u16p), M, 16, K, ctypes.byref(wp), ctypes.byref(op))
    offsets = np.ctypeslib.as_array(op, shape=(n,)).copy()
    count = int(offsets[-1]) * (4 if which == "v1" else 8)
    data = np.ctypeslib.as_array(wp, shape=(max(count, 1),))[:count].copy()
    _libc.free(ctypes.cast(wp, ctypes.c_void_p))
    _libc.free(ctypes.cast(op, ctypes.c_void_p))
    return {"offsets": offsets, "data": data}


def input_for(which, M, K, seed):
    if which == "v2":
        return multiple_of_eight_input(M, K, seed)
    if which == "v1":
        import graphneuralnetproj_b200 as sp
        return sp.synth_fp16((M, K), seed, 0.02, 0.8)
    return two_four_input(M, K, seed)


def digest(result):
    h = hashlib.sha256()
    for key in sorted(result):
        h.update(key.encode())
        h.update(np.ascontiguousarray(result[key]).tobytes())
    return h.hexdigest()


if __name__ == "__main__":
    import oracle
    ref = oracle.ref()
    out = {}
    for name, M, K, seed in CASES:
        for which in SYMBOLS:
            out["%s__%s" % (name, which)] = digest(run(ref, which, input_for(which, M, K, seed)))
    with open(os.path.join(HERE, "structured_digests.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", len(out), "digests")
