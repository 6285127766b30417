"""Prefill widths (N a multiple of 256) on pairs of SMs (tcgen05.mma.cta_group::2 over a cluster of two
blocks), through the C boundary: against the fp64 host product with the gates of the path
(max|C - C64| <= 1e-2 * max|C64|, mean(|C - C64| / max(|C64|, 1e-6)) <= 1e-3), exactly on integer inputs,
and against the single-block kernel that serves the same call when the switch is off."""
import numpy as np
import pytest

from test_spmm_gpu import run_spmm

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch


@pytest.fixture(autouse=True)
def pairs_on(sp):
    before = sp.set_pair_kernel(True)
    yield
    sp.set_pair_kernel(before)


CASES = [  # M, K, N, sparsity, Split_K
    (256, 64, 256, 0.8, 1),      # one pair of tiles, one cluster at work
    (256, 64, 512, 0.8, 1),      # the same with two MMAs per k step
    (512, 640, 256, 0.7, 2),     # 2 x 10 pair tiles over 74 clusters: rows split at every tile
    (512, 640, 512, 0.7, 2),
    (2304, 1152, 768, 0.8, 2),   # three column blocks of 256 (N is no multiple of 512)
    (2304, 1152, 1024, 0.5, 2),  # two column blocks of 512, tiles denser than the register budget
    (2560, 4608, 512, 0.9, 4),   # 10 rows of pairs x 72 k tiles: split rows and whole rows
    (1024, 2048, 256, 1.0, 2),   # all tiles empty
    (768, 256, 512, 0.0, 2),     # fully dense tiles
    (512, 256, 8192, 0.8, 1),    # the widest call: sixteen column blocks, more clusters than the device holds at once
]


@pytest.mark.parametrize("case", CASES, ids=["M%d_K%d_N%d_p%g_sk%d" % c for c in CASES])
def test_matches_oracle(sp, oracle, torch_cuda, case):
    M, K, N, p, sk = case
    A = sp.synth_fp16((M, K), 3000 + M + K + N, 0.02, p)
    B = sp.synth_fp16((K, N), 4000 + M + K + N, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, sk)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A, B))
    assert ok, (max_ratio, mean_rel)
    # repeated: same bits (fixed order of the sums over split rows)
    assert np.array_equal(run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, sk), C)
    # the single-block kernel on the same call: equal up to where rows are split
    sp.set_pair_kernel(False)
    C1 = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, sk)
    sp.set_pair_kernel(True)
    a, b = C.view(np.float16).astype(np.float64), C1.view(np.float16).astype(np.float64)
    assert np.abs(a - b).max() <= 2e-3 * max(np.abs(b).max(), 1e-6)


@pytest.mark.parametrize("N", [256, 512])
def test_without_workspace_rows_are_not_split(sp, oracle, torch_cuda, N):
    M, K = 1536, 1024
    A = sp.synth_fp16((M, K), 71, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 72, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 1, workspace=False)
    assert oracle.tolerance_check(C, oracle.spmm_f64(A, B))[0]


@pytest.mark.parametrize("shape", [(2304, 4608, 512), (4608, 2304, 768)], ids=["N512", "N768"])
def test_integer_inputs_are_exact(sp, torch_cuda, shape):
    """A in {-1, 0, 1}, B in {-1, 1}: every partial sum is a small integer, so fp32 accumulation in TMEM, the
    fp32 slots of split rows and the fp16 result are exact whatever the order."""
    M, K, N = shape
    rng = np.random.default_rng(23)
    A = (rng.integers(0, 2, size=(M, K)) * 2 - 1).astype(np.float16)
    A[rng.random((M, K), dtype=np.float32) < 0.8] = 0
    B = (rng.integers(0, 2, size=(K, N)) * 2 - 1).astype(np.float16)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 4).view(np.float16)
    expect = (torch_cuda.from_numpy(A).cuda().float() @ torch_cuda.from_numpy(B).cuda().float()).cpu().numpy()
    assert np.abs(expect).max() < 2048
    assert np.array_equal(C.astype(np.float32), expect)


def test_rows_not_a_multiple_of_256_stay_on_the_single_block_kernel(sp, oracle, torch_cuda):
    M, K, N = 1152, 1024, 512
    A = sp.synth_fp16((M, K), 81, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 82, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 2)
    sp.set_pair_kernel(False)
    assert np.array_equal(run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 2), C)
    assert oracle.tolerance_check(C, oracle.spmm_f64(A, B))[0]


TOKEN_MAJOR_CASES = [  # M, K, N, sparsity
    (512, 1024, 128, 0.8),    # two column blocks of 64 tokens on the single-block kernel
    (1152, 1024, 192, 0.8),   # M is no multiple of 256: single-block kernel, three column blocks
    (768, 1152, 256, 0.7),    # pairs of SMs, one MMA per k step
    (2304, 1152, 512, 0.8),   # pairs of SMs, two MMAs per k step
    (1536, 640, 768, 0.5),    # three column blocks of 256
    (2560, 4608, 1024, 0.9),  # two column blocks of 512, split rows and whole rows
    (768, 192, 4096, 0.8),    # eight column blocks of 512
]


@pytest.mark.parametrize("case", TOKEN_MAJOR_CASES, ids=["M%d_K%d_N%d_p%g" % c for c in TOKEN_MAJOR_CASES])
def test_token_major_layout_at_prefill_widths(sp, oracle, torch_cuda, case):
    """The upstream eleven-argument form (third_party/ft.patch:2822-2846), B[N][K] and C[N][M], beyond 64 tokens."""
    torch = torch_cuda
    dev = torch.device("cuda:0")
    M, K, N, p = case
    A = sp.synth_fp16((M, K), 5000 + M + N, 0.02, p)
    B = sp.synth_fp16((K, N), 6000 + M + N, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    wd = torch.from_numpy(words.view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bt = torch.from_numpy(np.ascontiguousarray(B.T).view(np.int16)).to(dev)          # [N][K]
    Ct = torch.full((N, M), 0x7E00, dtype=torch.int16, device=dev)                   # [N][M]
    sk = 8
    ws = torch.zeros(sp.workspace_bytes(M, N, sk) // 2, dtype=torch.int16, device=dev)
    assert sp.SpMM_SplitK_API_token_major(None, wd, od, Bt, Ct, M, N, K, ws, sk) == 0
    torch.cuda.synchronize()
    assert sp.device_status() == 0
    C = np.ascontiguousarray(Ct.cpu().numpy().view(np.uint16).T)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A, B))
    assert ok, (max_ratio, mean_rel)
    if M % 256 == 0 and N % 256 == 0:
        # on pairs of SMs both layouts use the same partition and accumulate in the same order: same bits
        assert np.array_equal(C, run_spmm(sp, torch, words, offsets, B, M, N, K, sk))
