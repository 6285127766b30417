"""Host-side pieces around the SpMM that need no GPU: the seeded generators (the product library's and the
oracle's independent one must agree bit for bit, and a block drawn on its own must equal the block cut out
of the whole matrix -- what lets a tensor-parallel rank draw only its shard), argument checks of the
host-buffer batch call and of the replayable reduction, and the weights-constant switch."""
import ctypes

import numpy as np


def test_block_equals_slice_of_whole(sp):
    whole = sp.synth_fp16((384, 320), 0xA0A0, 0.02, 0.8)
    assert np.array_equal(sp.synth_fp16_block(384, 320, 320, 0, 0, 0xA0A0, 0.02, 0.8), whole)
    assert np.array_equal(sp.synth_fp16_block(128, 320, 320, 256, 0, 0xA0A0, 0.02, 0.8), whole[256:])      # a row shard
    assert np.array_equal(sp.synth_fp16_block(384, 64, 320, 0, 192, 0xA0A0, 0.02, 0.8), whole[:, 192:256])  # a K shard
    assert 0.75 < np.mean(whole == 0) < 0.85


def test_oracle_generator_matches_the_library(sp, oracle):
    for seed, sigma, p in ((1, 0.02, 0.8), (0xB000, 1.0, 0.0), (77, 0.02, 0.5)):
        a = sp.synth_fp16_block(200, 96, 128, 3, 16, seed, sigma, p)
        b = oracle.synth_fp16_block(200, 96, 128, 3, 16, seed, sigma, p, threads=3)
        assert np.array_equal(a, b)


def test_row_shard_drawn_alone_encodes_like_the_slice(sp):
    """A rank's rows drawn alone and encoded == its slice of the whole matrix's encoding."""
    from graphneuralnetproj_b200 import tensor_parallel as tp
    M, K, world = 1024, 512, 4
    whole = sp.synth_fp16((M, K), 31, 0.02, 0.8)
    words, offsets, _ = sp.InitSparseMatrixA_API(whole, M, 16, K)
    for rank in range(world):
        mine = sp.synth_fp16_block(M // world, K, K, rank * (M // world), 0, 31, 0.02, 0.8)
        w, o, _ = sp.InitSparseMatrixA_API(mine, M // world, 16, K)
        ws, os_, m = tp.row_shard(words, offsets, M, K, rank, world)
        assert m == M // world and np.array_equal(w, ws) and np.array_equal(o, os_)


def test_host_io_batch_argument_checks(sp):
    lib = sp.spmm_api.LIB
    items = (sp.spmm_api.HostIoItem * 1)()
    assert lib.spmm_b200_spmm_splitk_host_io_batch(None, 0, items) == 1       # empty batch
    assert lib.spmm_b200_spmm_splitk_host_io_batch(None, 17, items) == 1      # more than the maximum
    assert lib.spmm_b200_spmm_splitk_host_io_batch(None, 1, None) == 1
    assert lib.spmm_b200_spmm_splitk_host_io_batch(None, 1, items) == 1       # null buffers inside the item


def test_replayable_reduction_argument_checks(sp):
    lib = sp.spmm_api.LIB
    two = (ctypes.c_void_p * 2)(16, 32)
    out = ctypes.c_void_p(16)
    assert lib.spmm_b200_allreduce_partials_replayable(None, two, two, 0, 2, out, 64, None, 0) == 1              # no state
    assert lib.spmm_b200_allreduce_partials_replayable(None, two, two, 0, 2, out, 64, ctypes.c_void_p(18), 0) == 1  # misaligned
    assert lib.spmm_b200_allreduce_partials_replayable(None, two, two, 0, 2, out, 60, ctypes.c_void_p(16), 0) == 1


def test_two_phase_reduction_argument_checks(sp):
    lib = sp.spmm_api.LIB
    four = (ctypes.c_void_p * 4)(16, 32, 48, 64)
    two = (ctypes.c_void_p * 2)(16, 32)
    state = ctypes.c_void_p(16)
    f = lib.spmm_b200_allreduce_partials_f32_two_phase
    assert f(None, four, two, two, 0, 2, 64, None, 0) == 1                 # no state
    assert f(None, four, two, two, 0, 2, 24, state, 0) == 1                # count is no multiple of 8 * world
    assert f(None, four, two, None, 0, 2, 64, state, 0) == 1               # no result buffers
    assert f(None, four, two, two, 2, 2, 64, state, 0) == 1                # rank outside the world
    assert f(None, four, two, (ctypes.c_void_p * 2)(16, 40), 0, 2, 64, state, 0) == 1  # misaligned result buffer


def test_weights_constant_switch(sp):
    before = sp.set_weights_constant(True)
    assert sp.set_weights_constant(False) is True
    assert sp.set_weights_constant(before) is False
