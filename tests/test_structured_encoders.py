"""The 2:4-oriented host encoders kept for the drop-in header (NoReorder_v1..v4, the A1 vector
format, inspect_metadata) must produce the reference's bytes: checked against digests of the
reference's compiled encoders and, where that library is present, against it directly."""
import ctypes
import json
import os

import numpy as np
import pytest

from golden import structured_formats as sf


@pytest.fixture(scope="module")
def lib(sp):
    return ctypes.CDLL(sp.LIB_PATH)


@pytest.fixture(scope="module")
def digests():
    with open(os.path.join(os.path.dirname(sf.__file__), "structured_digests.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("case", sf.CASES, ids=[c[0] for c in sf.CASES])
@pytest.mark.parametrize("which", sorted(sf.SYMBOLS))
def test_matches_golden_digest(lib, digests, case, which, capfd):
    name, M, K, seed = case
    result = sf.run(lib, which, sf.input_for(which, M, K, seed))
    assert sf.digest(result) == digests["%s__%s" % (name, which)]


@pytest.mark.parametrize("which", sorted(sf.SYMBOLS))
def test_matches_compiled_reference(lib, oracle, which, capfd):
    if not oracle.have_ref():
        pytest.skip("compiled reference not present")
    A = sf.input_for(which, 512, 192, 77)
    ours, theirs = sf.run(lib, which, A), sf.run(oracle.ref(), which, A)
    assert sorted(ours) == sorted(theirs)
    for key in ours:
        assert np.array_equal(ours[key], theirs[key]), key


def test_v3_layout_by_hand(lib, capfd):
    A = np.zeros((128, 64), np.uint16)
    A[0, 1], A[0, 3], A[0, 4], A[5, 63] = 0x3C00, 0x4000, 0x4200, 0x4400
    out = sf.run(lib, "v3", A)
    tile = out["data"].reshape(128, 32)
    assert list(tile[0, :4]) == [0x3C00, 0x4000, 0x4200, 0] and tile[5, 30] == 0x4400 and np.count_nonzero(tile) == 4
    assert list(out["offsets"]) == [0, 512, 512]
