"""The tiled-CSL validator (host side here, device side under -m gpu) and the per-rank list files the
FasterTransformer loaders read (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:134-135, 183-195;
third_party/ft.patch:2352-2401).  A corrupt stream is only ever shown to the validator: the SpMM is not
launched on it."""
import numpy as np
import pytest


def encoded(sp, M=256, K=192, seed=5):
    A = sp.synth_fp16((M, K), seed, 0.02, 0.8)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, 16, K)
    return words, offsets, M, K


def corruptions(words, offsets):
    tiles = offsets.size - 2
    w, o = words.copy(), offsets.copy()
    o[0] = 1
    yield "first offset", w, o, 1
    w, o = words.copy(), offsets.copy()
    o[3], o[4] = o[4], o[3] + 0
    o[3] = o[5] + 7
    yield "offsets decrease", w, o, 2
    w, o = words.copy(), offsets.copy()
    o[tiles + 1] += 1
    yield "tail", w, o, 4
    yield "truncated words", words[:-8].copy(), offsets.copy(), 8
    w, o = words.copy(), offsets.copy()
    w[17] = (8192 << 16) | 0x3C00
    yield "position", w, o, 16


def test_host_validator(sp):
    words, offsets, M, K = encoded(sp)
    assert sp.validate_tiled_csl(words, offsets, M, K) == 0
    for label, w, o, bit in corruptions(words, offsets):
        found = sp.validate_tiled_csl(w, o, M, K)
        assert found & bit, (label, found)
    assert sp.validate_tiled_csl(words, offsets[:-1], M, K) == 32       # wrong number of offsets
    assert sp.validate_tiled_csl(words, offsets, M + 1, K) == 32        # a shape the format cannot describe
    # an all-zero matrix: no words at all
    zw, zo, _ = sp.InitSparseMatrixA_API(np.zeros((128, 64), np.uint16), 128, 16, 64)
    assert zw.size == 0 and sp.validate_tiled_csl(zw, zo, 128, 64) == 0


def test_encoder_output_files_validate(sp, tmp_path):
    """What GenSparseMatrixBinFile writes passes the validator."""
    M, K = 256, 128
    A = sp.synth_fp16((M, K), 9, 0.02, 0.8)
    dense = tmp_path / "w.bin"
    A.tofile(dense)
    sp.GenSparseMatrixBinFile(str(dense), M, K, str(tmp_path / "w.NZWeights.bin"), str(tmp_path / "w.TileOffsets.bin"),
                              str(tmp_path / "w.OutputSizes.bin"))
    sizes = np.fromfile(tmp_path / "w.OutputSizes.bin", np.int32)
    words = np.fromfile(tmp_path / "w.NZWeights.bin", np.uint32)
    offsets = np.fromfile(tmp_path / "w.TileOffsets.bin", np.int32)
    assert sizes[0] == words.size and sizes[1] == offsets.size
    assert sp.validate_tiled_csl(words, offsets, M, K) == 0


def test_shard_shapes_and_split_k(sp):
    assert sp.shard_shapes(9216, 1) == ([27648, 9216, 36864, 9216], [9216, 9216, 9216, 36864])
    assert sp.shard_shapes(12288, 8) == ([4608, 12288, 6144, 12288], [12288, 1536, 12288, 6144])
    with pytest.raises(ValueError):
        sp.shard_shapes(9216, 5)
    with pytest.raises(ValueError):
        sp.shard_shapes(1024, 16)  # K shard of 64 is fine, M shard 3*1024/16 = 192 is not a multiple of 128
    for M, K in ((27648, 9216), (9216, 36864), (7168, 7168), (1152, 9216)):
        sk = sp.suggest_split_k(M, K)
        _, _, used = sp.plan(M // 128, K // 64, 148, 1 << 40)
        assert sk >= 1 and sk * M * 2 >= used * 128 * 4 and (sk == 1 or (sk - 1) * M * 2 < used * 128 * 4)
    assert sp.suggest_split_k(100, 64) == 0


def test_rank_list_files(sp, tmp_path):
    """Two layers, two ranks, a small hidden size: every matrix is encoded with GenSparseMatrixBinFile, one is
    left dense; the list files repeat the sizes files in (layer, matrix) order."""
    hidden, world, layers = 256, 2, 2
    names = ["attention.query_key_value", "attention.dense", "mlp.dense_h_to_4h", "mlp.dense_4h_to_h"]
    for rank in range(world):
        M, K = sp.shard_shapes(hidden, world)
        expect_nnz, expect_off = [], []
        for layer in range(layers):
            for k, name in enumerate(names):
                stem = str(tmp_path / ("model.layers.%d.%s.weight.%d" % (layer, name, rank)))
                sp.synth_fp16((M[k], K[k]), 100 * rank + 10 * layer + k, 0.02, 0.8).tofile(stem + ".bin")
                if (layer, k) == (1, 2) and rank == 1:     # this one stays dense
                    expect_nnz.append(0)
                    expect_off.append(0)
                    continue
                sp.GenSparseMatrixBinFile(stem + ".bin", M[k], K[k], stem + ".NZWeights.bin", stem + ".TileOffsets.bin",
                                          stem + ".OutputSizes.bin")
                sizes = np.fromfile(stem + ".OutputSizes.bin", np.int32)
                expect_nnz.append(int(sizes[0]))
                expect_off.append(int(sizes[1]))
        found = sp.write_rank_lists(str(tmp_path), rank, layers, M, K)
        assert found == layers * 4 - (1 if rank == 1 else 0)
        nnz = np.fromfile(tmp_path / ("NNZ_List.%d.bin" % rank), np.int32)
        off = np.fromfile(tmp_path / ("NumOffsets_List.%d.bin" % rank), np.int32)
        sk = np.fromfile(tmp_path / ("SplitK_List.%d.bin" % rank), np.int32)
        assert nnz.tolist() == expect_nnz and off.tolist() == expect_off
        assert [int(s > 0) for s in sk] == [int(n > 0) for n in expect_off]
        assert all(s == sp.suggest_split_k(M[i % 4], K[i % 4]) for i, s in enumerate(sk) if s)
    with pytest.raises(OSError):
        sp.write_rank_lists(str(tmp_path / "missing"), 0, layers, M, K)


@pytest.mark.gpu
def test_device_validator(sp):
    import torch
    dev = torch.device("cuda:0")
    words, offsets, M, K = encoded(sp, 1024, 2048, 6)

    def on_device(w, o):
        wd = torch.from_numpy(w.view(np.int32)).to(dev)
        od = torch.from_numpy(o).to(dev)
        return sp.validate_tiled_csl(wd, od, M, K)

    assert on_device(words, offsets) == 0
    for label, w, o, bit in corruptions(words, offsets):
        assert on_device(w, o) & bit, label
    assert sp.device_status() == 0
