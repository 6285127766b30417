"""The tolerance gate at the sizes the benchmark configurations name, through the C boundary.

Gate: max|C - C64| <= 1e-2 * max|C64| and mean(|C - C64| / max(|C64|, 1e-6)) <= 1e-3 against the
fp64 host product of the oracle, on fp16 N(0, 0.02^2) weights zeroed i.i.d. and N(0, 1) activations
(the seeded stand-ins for pruned OPT weights).  The reference checks its kernels the same way, one
product against a trusted one after the timed loop (kernel_benchmark/spmm_test.cu:1091), over the
grid of kernel_benchmark/benchmark.sh:13-17 (layer shapes x N in {8,16,32,64} x sparsity in {70,80,90} %).

Decode sizes are checked on every row.  At prefill sizes the fp64 product is taken on two rows of
every row of tiles (so every thread block's output and every split row is sampled); the gate's
max|C64| is then the maximum over the sampled rows.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

OPT66B = {"qkv": (27648, 9216), "out_proj": (9216, 9216), "ffn1": (36864, 9216), "ffn2": (9216, 36864)}
SPLIT_K = {"qkv": 4, "out_proj": 8, "ffn1": 4, "ffn2": 8}


def spmm_on_gpu(sp, words, offsets, B_bits, M, N, K, split_k):
    """Exact-size device buffers: Compressed_A holds the encoder's words and nothing after them."""
    import torch
    dev = torch.device("cuda:0")
    wd = torch.from_numpy(words.view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(np.ascontiguousarray(B_bits).view(np.int16)).to(dev)
    Cd = torch.full((M, N), 0x7E00, dtype=torch.int16, device=dev)  # NaN pattern: unwritten rows show up
    ws = torch.zeros(sp.workspace_bytes(M, N, split_k) // 2, dtype=torch.int16, device=dev)
    rc = sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, N, K, ws, split_k)
    torch.cuda.synchronize()
    assert rc == 0, "launch failed with cudaError %d" % rc
    assert sp.device_status() == 0, "a bounded wait inside the kernel gave up"
    return Cd.cpu().numpy().view(np.uint16)


def gate(oracle, C, A, B, rows=None):
    if rows is None:
        c64 = oracle.spmm_f64_threads(A, B)
        ok, max_ratio, mean_rel = oracle.tolerance_check(C, c64)
    else:
        c64 = oracle.spmm_f64_threads(np.ascontiguousarray(A[rows]), B)
        ok, max_ratio, mean_rel = oracle.tolerance_check(np.ascontiguousarray(C[rows]), c64)
    assert ok, "max|err|/max|C| = %.3e, mean relative error = %.3e" % (max_ratio, mean_rel)


def two_rows_per_row_of_tiles(M, seed):
    rng = np.random.default_rng(seed)
    return np.sort(np.concatenate([np.arange(0, M, 128) + rng.integers(0, 64, M // 128),
                                   np.arange(0, M, 128) + rng.integers(64, 128, M // 128)]))


@pytest.mark.parametrize("layer", list(OPT66B))
def test_opt66b_layers_n16_p80(sp, oracle, layer):
    """The four layers of the benchmark step (OPT-66B decoder block, N = 16, 80 % sparse) at full size."""
    M, K = OPT66B[layer]
    N = 16
    A = sp.synth_fp16((M, K), 0xA600 + len(layer), 0.02, 0.8)
    B = sp.synth_fp16((K, N), 0xB600 + len(layer), 1.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    gate(oracle, spmm_on_gpu(sp, words, offsets, B, M, N, K, SPLIT_K[layer]), A, B)


SWEEP_CELLS = [("out_proj", 8, 0.8), ("ffn2", 32, 0.8), ("qkv", 64, 0.8), ("ffn1", 16, 0.7), ("ffn2", 16, 0.9),
               ("out_proj", 64, 0.7), ("qkv", 8, 0.9)]


@pytest.mark.parametrize("cell", SWEEP_CELLS, ids=["%s_N%d_p%g" % c for c in SWEEP_CELLS])
def test_opt66b_sweep_cells(sp, oracle, cell):
    """One full-size cell for each other N and sparsity of the decode sweep."""
    layer, N, p = cell
    M, K = OPT66B[layer]
    A = sp.synth_fp16((M, K), 0xA700 + N + int(100 * p), 0.02, p)
    B = sp.synth_fp16((K, N), 0xB700 + N, 1.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    gate(oracle, spmm_on_gpu(sp, words, offsets, B, M, N, K, SPLIT_K[layer]), A, B)


PREFILL_CELLS = [(12288, 12288, 256, 0.5), (12288, 12288, 2048, 0.8), (49152, 12288, 512, 0.7)]


@pytest.mark.parametrize("cell", PREFILL_CELLS, ids=["M%d_K%d_N%d_p%g" % c for c in PREFILL_CELLS])
def test_prefill_sizes(sp, oracle, cell):
    """Prefill-size products (N >= 256) at the sparsities of that configuration, incl. the 49152 x 12288 layer."""
    M, K, N, p = cell
    A = sp.synth_fp16((M, K), 0xA800 + N, 0.02, p)
    B = sp.synth_fp16((K, N), 0xB800 + N, 1.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = spmm_on_gpu(sp, words, offsets, B, M, N, K, 2)
    assert not np.any((C & 0x7FFF) > 0x7C00), "rows left unwritten"
    gate(oracle, C, A, B, rows=two_rows_per_row_of_tiles(M, N))


TP_SHARDS = [("qkv", 36864, 12288, "rows"), ("ffn1", 49152, 12288, "rows"), ("ffn2", 12288, 49152, "columns")]


@pytest.mark.parametrize("case", TP_SHARDS, ids=[c[0] + "_175b_shard_of_8" for c in TP_SHARDS])
def test_opt175b_shards_of_eight(sp, oracle, case):
    """What one of eight ranks multiplies of an OPT-175B layer (N = 16, 80 % sparse), on one GPU: a row shard
    cut out of the whole-matrix encoding (QKV, FFN1) or the encoding of a column slice (FFN2), as
    end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:134-135 shards them."""
    from graphneuralnetproj_b200 import tensor_parallel as tp
    name, M, K, split = case
    N, world, rank = 16, 8, 5
    B = sp.synth_fp16((K, N), 0xB900, 1.0)
    if split == "rows":
        # the shard of rank 5 only needs rank 5's rows: encode those (bit-identical to the slice of the whole
        # encoding, which tests/test_tensor_parallel.py checks) and one more shard to cut from
        rows = M // world
        A2 = sp.synth_fp16((2 * rows, K), 0xA900 + len(name), 0.02, 0.8)
        words, offsets, _ = sp.InitSparseMatrixA_API(A2, 2 * rows, N, K)
        w, o, m = tp.row_shard(words, offsets, 2 * rows, K, 1, 2)
        assert m == rows
        gate(oracle, spmm_on_gpu(sp, w, o, B, rows, N, K, 4), A2[rows:], B)
    else:
        k = K // world
        A_shard = sp.synth_fp16((M, k), 0xA900 + len(name), 0.02, 0.8)
        B_shard = tp.activation_rows(B, rank, world)
        words, offsets, _ = sp.InitSparseMatrixA_API(A_shard, M, N, k)
        gate(oracle, spmm_on_gpu(sp, words, offsets, B_shard, M, N, k, 8), A_shard, B_shard)


def test_exact_size_compressed_a(sp, oracle):
    """Compressed_A needs no bytes after the last word: the buffer here ends where the encoder's output ends,
    at the end of its allocation, for a matrix whose last tiles are dense, ragged and empty."""
    import torch
    M, K, N = 1024, 4608, 16
    A = sp.synth_fp16((M, K), 0xAA00, 0.02, 0.8)
    A[-128:, -64:] = 0                                   # the very last tile is empty
    A[-128:, -128:-64] = sp.synth_fp16((128, 64), 1, 0.02, 0.0)  # the one before it is dense
    B = sp.synth_fp16((K, N), 0xBA00, 1.0)
    words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, N, K)
    assert words.size == 4 * offsets[n_offsets - 1]
    gate(oracle, spmm_on_gpu(sp, words, offsets, B, M, N, K, 4), A, B)
    # the same words at the very end of a larger allocation (nothing of this tensor lies behind them)
    dev = torch.device("cuda:0")
    pool = torch.zeros(words.size + 1024, dtype=torch.int32, device=dev)
    pool[-words.size:] = torch.from_numpy(words.view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(B.view(np.int16)).to(dev)
    Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
    ws = torch.zeros(sp.workspace_bytes(M, N, 4) // 2, dtype=torch.int16, device=dev)
    assert sp.SpMM_SplitK_API(None, None, pool[-words.size:], None, None, od, Bd, Cd, M, N, K, ws, 4) == 0
    torch.cuda.synchronize()
    gate(oracle, Cd.cpu().numpy().view(np.uint16), A, B)
