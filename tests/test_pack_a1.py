"""Host packer of the structured (2:4) half for tcgen05.mma.sp: round trip through the oracle's decoder."""
import numpy as np
import pytest


def prune_2_of_4(A_bits, keep_prob, seed):
    """Keeps the two largest magnitudes of every aligned group of four, then zeroes each survivor with 1 - keep_prob."""
    vals = A_bits.view(np.float16).astype(np.float32)
    groups = np.abs(vals).reshape(-1, 4)
    order = np.argsort(-groups, axis=1, kind="stable")
    mask = np.zeros_like(groups, dtype=bool)
    np.put_along_axis(mask, order[:, :2], True, axis=1)
    rng = np.random.default_rng(seed)
    mask &= rng.random(mask.shape) < keep_prob
    out = A_bits.reshape(-1, 4).copy()
    out[~mask] = 0
    return out.reshape(A_bits.shape)


@pytest.mark.parametrize("shape,keep", [((128, 128), 1.0), ((256, 384), 0.5), ((384, 256), 0.0)])
def test_round_trip(sp, shape, keep):
    from oracle.a1_tcgen05 import unpack_a1
    M, K = shape
    A1 = prune_2_of_4(sp.synth_fp16((M, K), 31 + M + K, 0.02, 0.0), keep, 5)
    values, meta, blocks = sp.InitSparseMatrixA1_tcgen05(A1, M, K)
    assert blocks == (M // 128) * (K // 128) and values.size == blocks * 16384 and meta.size == blocks * 512
    assert np.array_equal(unpack_a1(values, meta, M, K), A1)


def test_decompose_output_packs(sp):
    from oracle.a1_tcgen05 import unpack_a1
    A = sp.synth_fp16((256, 256), 77, 0.02, 0.6)
    A.reshape(-1)[:8] = [0x8000, 0x3C00, 0x8000, 0x3C00, 0x7E00, 0x0001, 0, 0]  # -0 is not kept, NaN and subnormals are
    A1, _ = sp.decompose(A)
    values, meta, _ = sp.InitSparseMatrixA1_tcgen05(A1, 256, 256)
    back = unpack_a1(values, meta, 256, 256)
    # -0 in A1 may come back as +0 (it is not a kept value); everything else is bit-exact
    assert np.array_equal(back & 0x7FFF, A1 & 0x7FFF)
    keep = (A1 & 0x7FFF) != 0
    assert np.array_equal(back[keep], A1[keep])


def test_rejects_bad_input(sp):
    dense = sp.synth_fp16((128, 128), 3, 0.02, 0.0)  # four nonzeros per group
    with pytest.raises(ValueError):
        sp.InitSparseMatrixA1_tcgen05(dense, 128, 128)
    with pytest.raises(ValueError):
        sp.InitSparseMatrixA1_tcgen05(np.zeros((128, 64), np.uint16), 128, 64)
