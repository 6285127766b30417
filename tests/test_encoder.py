"""The product's host encoders (C++, tile-parallel) must be bit-identical to the oracle,
to the golden vectors and -- where present -- to the reference's compiled encoder."""
import os
import subprocess
import sys

import numpy as np
import pytest

from golden.make_golden import LARGE, SMALL, make_input

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def small():
    return np.load(os.path.join(GOLDEN, "tiled_csl_small.npz"))


@pytest.mark.parametrize("case", SMALL, ids=[c[0] for c in SMALL])
def test_encoder_matches_golden(sp, small, case):
    name, M, K, p, seed = case
    A = small[f"{name}__A"]
    w, o, n = sp.InitSparseMatrixA_API(A, M, 16, K)
    assert n == (M // 128) * (K // 64) + 2 == o.size
    assert np.array_equal(o, small[f"{name}__reorder__offsets"])
    assert np.array_equal(w, small[f"{name}__reorder__words"])
    w, o, n = sp.InitSparseMatrixA_API_NoReorder(A, M, 16, K)
    assert np.array_equal(o, small[f"{name}__noreorder__offsets"])
    assert np.array_equal(w, small[f"{name}__noreorder__words"])


@pytest.mark.parametrize("case", LARGE, ids=[c[0] for c in LARGE])
def test_encoder_matches_oracle_large(sp, oracle, case):
    name, M, K, p, seed = case
    A = make_input(M, K, p, seed, special=True)
    for fn, variant in ((sp.InitSparseMatrixA_API, "reorder"), (sp.InitSparseMatrixA_API_NoReorder, "noreorder")):
        w, o, n = fn(A, M, 8, K)
        wo, oo = oracle.encode(A, variant)
        assert np.array_equal(o, oo) and np.array_equal(w, wo)


def test_offsets_structure(sp):
    A = sp.synth_fp16((512, 256), 3, 0.02, 0.8)
    w, o, n = sp.InitSparseMatrixA_API(A, 512, 16, 256)
    assert o[0] == 0 and o[-1] == o[-2] and np.all(np.diff(o) >= 0)
    assert w.size == 4 * o[-1]
    nnz = np.count_nonzero(A)
    assert nnz <= w.size <= nnz + 3 * (n - 2)


def test_pad_counts_one_two_three(sp, oracle):
    # tiles with nnz % 4 == 1, 2, 3 need 3, 2, 1 padding words
    for nnz in (1, 2, 3, 5, 4097, 8191):
        A = np.zeros((128, 64), np.uint16)
        A.reshape(-1)[np.random.default_rng(nnz).choice(8192, nnz, replace=False)] = 0x3C00
        w, o, _ = sp.InitSparseMatrixA_API(A, 128, 16, 64)
        wo, oo = oracle.encode(A)
        assert w.size == (nnz + 3) // 4 * 4
        assert np.array_equal(w, wo) and np.array_equal(o, oo)


def test_thread_count_does_not_change_output(sp):
    A = sp.synth_fp16((1024, 512), 9, 0.02, 0.8)
    base = sp.InitSparseMatrixA_API(A, 1024, 16, 512)
    code = ("import sys,numpy as np;sys.path.insert(0,%r);import graphneuralnetproj_b200 as sp;"
            "A=sp.synth_fp16((1024,512),9,0.02,0.8);w,o,n=sp.InitSparseMatrixA_API(A,1024,16,512);"
            "sys.stdout.buffer.write(w.tobytes()+o.tobytes())") % os.path.dirname(os.path.dirname(__file__))
    env = dict(os.environ, SPMM_B200_THREADS="1")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, check=True).stdout
    assert out == base[0].tobytes() + base[1].tobytes()


def test_bad_shapes_are_rejected(sp):
    A = np.zeros((100, 64), np.uint16)
    with pytest.raises(ValueError):
        sp.InitSparseMatrixA_API(A, 100, 16, 64)
    with pytest.raises(ValueError):
        sp.InitSparseMatrixA_API(np.zeros((128, 32), np.uint16), 128, 16, 32)


def test_decompose_matches_oracle(sp, oracle):
    A = sp.synth_fp16((256, 512), 17, 0.02, 0.6)
    A.reshape(-1)[:8] = [0x8000, 0x7E00, 0x3C00, 0x3C00, 0x7E00, 0x7E00, 0x7E00, 0x0001]
    for v1 in (False, True):
        a1, a2 = sp.decompose(A, v1=v1)
        b1, b2 = oracle.decompose(A, v1=v1)
        assert np.array_equal(a1, b1) and np.array_equal(a2, b2)


def test_decompose_matches_compiled_reference(sp, oracle, capfd):
    """decompose / decompose_v1 against the reference's own header (kernel_benchmark/spmm_decompose.h:12-142),
    compiled as it lies into oracle/_ref: groups with 0..4 nonzeros, -0, NaN, subnormals."""
    import pytest
    if not oracle.have_ref_decompose():
        pytest.skip("compiled reference header not present")
    A = sp.synth_fp16((256, 192), 4321, 0.02, 0.55)
    A[0, :8] = [0x8000, 0x0001, 0x7E00, 0x3C00, 0x0000, 0x8000, 0x8000, 0xFC00]  # -0, subnormal, NaN, 1, 0, -0, -0, -inf
    A[1, :4] = 0x3C00                                                           # a full group
    for v1 in (False, True):
        a1, a2 = sp.decompose(A, v1=v1)
        r1, r2 = oracle.ref_decompose(A, v1=v1)
        o1, o2 = oracle.decompose(A, v1=v1)
        assert np.array_equal(a1, r1) and np.array_equal(a2, r2)
        assert np.array_equal(o1, r1) and np.array_equal(o2, r2)
    capfd.readouterr()


def test_decompose_cxx_entry_points(sp):
    """decompose / decompose_v1 with the reference's C++ signatures (include/spmm_decompose.h) agree with the C ABI."""
    import ctypes
    A = sp.synth_fp16((128, 256), 19, 0.02, 0.55)
    for v1, symbol in ((False, "_Z9decomposeP6__halfS0_S0_i"), (True, "_Z12decompose_v1P6__halfS0_S0_i")):
        fn = getattr(sp.spmm_api.LIB, symbol)
        fn.restype = None
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        a1 = np.full(A.shape, 0xFFFF, np.uint16)
        a2 = np.full(A.shape, 0xFFFF, np.uint16)
        fn(A.ctypes.data, a1.ctypes.data, a2.ctypes.data, A.size)
        b1, b2 = sp.decompose(A, v1=v1)
        assert np.array_equal(a1, b1) and np.array_equal(a2, b2)


def test_gen_sparse_matrix_bin_file(sp, tmp_path):
    M, K = 256, 128
    A = sp.synth_fp16((M, K), 23, 0.02, 0.8)
    dense = tmp_path / "dense.bin"
    A.tofile(dense)
    nz, off, sizes = tmp_path / "nz.bin", tmp_path / "off.bin", tmp_path / "sizes.bin"
    sp.GenSparseMatrixBinFile(str(dense), M, K, str(nz), str(off), str(sizes))
    w, o, n = sp.InitSparseMatrixA_API(A, M, 0, K)
    assert np.array_equal(np.fromfile(sizes, np.int32), [w.size, n])
    assert np.array_equal(np.fromfile(nz, np.uint32), w)
    assert np.array_equal(np.fromfile(off, np.int32), o)


def test_synth_is_seeded_and_distributed(sp):
    a = sp.synth_fp16((1 << 16,), 0xA001, 0.02, 0.8)
    b = sp.synth_fp16((1 << 16,), 0xA001, 0.02, 0.8)
    c = sp.synth_fp16((1 << 16,), 0xA002, 0.02, 0.8)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    frac_zero = np.mean(a == 0)
    assert 0.78 < frac_zero < 0.82
    vals = a[a != 0].view(np.float16).astype(np.float64)
    assert abs(vals.std() - 0.02) < 0.002 and abs(vals.mean()) < 0.001
