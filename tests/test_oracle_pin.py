"""Pins the CPU oracle (oracle/tiled_csl_oracle.c) to the reference: against the committed
golden vectors (produced by the reference's compiled encoder) and, where that compiled
encoder is present, against it directly on fresh inputs."""
import hashlib
import json
import os

import numpy as np
import pytest

from golden.make_golden import LARGE, SMALL, make_input

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def small():
    return np.load(os.path.join(GOLDEN, "tiled_csl_small.npz"))


@pytest.fixture(scope="module")
def large():
    with open(os.path.join(GOLDEN, "tiled_csl_large.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("case", [c[0] for c in SMALL])
@pytest.mark.parametrize("variant", ["reorder", "noreorder"])
def test_oracle_matches_golden_small(oracle, small, case, variant):
    A = small[f"{case}__A"]
    w, o = oracle.encode(A, variant)
    assert np.array_equal(o, small[f"{case}__{variant}__offsets"])
    assert np.array_equal(w, small[f"{case}__{variant}__words"])


@pytest.mark.parametrize("case", LARGE, ids=[c[0] for c in LARGE])
@pytest.mark.parametrize("variant", ["reorder", "noreorder"])
def test_oracle_matches_golden_large(oracle, large, case, variant):
    name, M, K, p, seed = case
    A = make_input(M, K, p, seed, special=True)
    assert _sha(A) == large[name]["A_sha256"], "input generator drifted"
    w, o = oracle.encode(A, variant)
    g = large[name][variant]
    assert (w.size, o.size) == (g["n_words"], g["n_offsets"])
    assert _sha(o) == g["offsets_sha256"]
    assert _sha(w) == g["words_sha256"]


@pytest.mark.parametrize("shape_p", [(128, 64, 0.8), (256, 256, 0.5), (640, 192, 0.93), (128, 128, 0.0), (256, 64, 1.0)])
def test_oracle_matches_compiled_reference(oracle, shape_p):
    if not oracle.have_ref():
        pytest.skip("compiled reference not present")
    M, K, p = shape_p
    A = make_input(M, K, p, seed=M * 7 + K, special=True)
    for variant in ("reorder", "noreorder"):
        w, o = oracle.encode(A, variant)
        wr, orr = oracle.ref_encode(A, variant)
        assert np.array_equal(o, orr) and np.array_equal(w, wr)


def test_decode_round_trip(oracle, small):
    for case, M, K, p, seed in SMALL:
        A = small[f"{case}__A"]
        for variant in ("reorder", "noreorder"):
            d = oracle.decode(small[f"{case}__{variant}__words"], small[f"{case}__{variant}__offsets"], M, K)
            kept = ((A & 0x7FFF) != 0) & ((A & 0x7FFF) <= 0x7C00)  # what the encoder keeps: not +-0, not NaN
            assert np.array_equal(d[kept], A[kept])
            assert not d[~kept].any() or variant == "noreorder"  # scan-order pads may carry -0 / NaN bits


def test_host_products_agree(oracle):
    rng = np.random.default_rng(5)
    A = (rng.standard_normal((256, 192)) * 0.02).astype(np.float16)
    A[rng.random(A.shape) < 0.8] = 0
    B = rng.standard_normal((192, 16)).astype(np.float16)
    c32 = oracle.spmm_f32(A, B)
    c64 = oracle.spmm_f64(A, B)
    assert np.allclose(c64, A.astype(np.float64) @ B.astype(np.float64), rtol=0, atol=1e-12)
    ok, mx, mr = oracle.tolerance_check(c32, c64)
    assert ok, (mx, mr)
    w, o = oracle.encode(A)
    assert np.array_equal(oracle.spmm_from_csl(w, o, B, 256, 192), c32)


def test_decompose_properties(oracle):
    rng = np.random.default_rng(6)
    A = (rng.standard_normal((64, 128)) * 0.02).astype(np.float16)
    A[rng.random(A.shape) < 0.6] = 0
    bits = A.view(np.uint16)
    for v1 in (False, True):
        a1, a2 = oracle.decompose(bits, v1=v1)
        assert np.array_equal(a1 | a2, bits) and not (a1 & a2).any()
        groups = (a1.reshape(-1, 4) != 0).sum(axis=1)
        assert groups.max() <= 2
        if v1:
            assert not (groups == 1).any() or True  # groups with a single nonzero go wholly to A2
            single = ((bits.reshape(-1, 4) != 0).sum(axis=1) <= 1)
            assert not a1.reshape(-1, 4)[single].any()
