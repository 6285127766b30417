"""Heterogeneous mode of SpMM_SplitK_API on the GPU: C = A1 * B (tcgen05.mma.sp) + A2 * B (tiled-CSL),
against the fp64 host product of A = A1 + A2, through the C boundary.  Same tolerance as the
unstructured path: max|C - C64| <= 1e-2 * max|C64| and mean(|C - C64| / max(|C64|, 1e-6)) <= 1e-3."""
import numpy as np
import pytest

from test_pack_a1 import prune_2_of_4

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch


def run_hetero(sp, torch, A1, A2, B_bits, M, N, K, split_k, workspace=True):
    dev = torch.device("cuda:0")
    values, meta, _ = sp.InitSparseMatrixA1_tcgen05(A1, M, K)
    vd = torch.from_numpy(values).to(dev)
    md = torch.from_numpy(meta.view(np.int32)).to(dev)
    wd = od = None
    if A2 is not None:
        words, offsets, _ = sp.InitSparseMatrixA_API(A2, M, N, K)
        wd = torch.from_numpy((words if words.size else np.zeros(4, np.uint32)).view(np.int32)).to(dev)
        od = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(np.ascontiguousarray(B_bits).view(np.int16)).to(dev)
    Cd = torch.full((M, N), 0x7E00, dtype=torch.int16, device=dev)
    ws = torch.zeros(sp.workspace_bytes(M, N, split_k) // 2 + 8, dtype=torch.int16, device=dev) if workspace else None
    rc = sp.SpMM_SplitK_API(None, vd, wd, None, md, od, Bd, Cd, M, N, K, ws, split_k)
    torch.cuda.synchronize()
    assert rc == 0, "launch failed with cudaError %d" % rc
    assert sp.device_status() == 0, "a bounded wait inside the kernel gave up"
    return Cd.cpu().numpy().view(np.uint16)


def pattern_matrix(sp, M, K, seed, pair_of):
    """A 2:4 matrix whose kept pair in group g of row r is pair_of(r, g) (index into the six pairs)."""
    pairs = np.array([(0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3)])
    dense = sp.synth_fp16((M, K), seed, 0.02, 0.0).reshape(M, K // 4, 4)
    r, g = np.meshgrid(np.arange(M), np.arange(K // 4), indexing="ij")
    chosen = pairs[pair_of(r, g) % 6]                       # [M][K/4][2]
    mask = np.zeros((M, K // 4, 4), bool)
    np.put_along_axis(mask, chosen, True, axis=2)
    return np.where(mask, dense, 0).astype(np.uint16).reshape(M, K)


PATTERNS = {
    "first_two_everywhere": lambda r, g: 0 * r,     # one selector code: only the value layout matters
    "by_row": lambda r, g: r,                       # metadata must follow rows
    "by_group": lambda r, g: g,                     # metadata must follow k
    "by_row_and_group": lambda r, g: r * 7 + g * 3,
}


@pytest.mark.parametrize("name", list(PATTERNS))
def test_selector_patterns(sp, oracle, torch_cuda, name):
    M, K, N = 256, 512, 16
    A1 = pattern_matrix(sp, M, K, 41, PATTERNS[name])
    B = sp.synth_fp16((K, N), 43, 1.0, 0.0)
    C = run_hetero(sp, torch_cuda, A1, None, B, M, N, K, 4)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A1, B))
    assert ok, (name, max_ratio, mean_rel)


CASES = [  # M, K, N, Split_K
    (128, 128, 16, 2),
    (256, 384, 8, 2),
    (512, 1024, 32, 4),
    (1024, 2048, 64, 4),
    (2304, 4608, 32, 8),   # 18 x 36 blocks over 148 thread blocks: rows split between blocks
]


@pytest.mark.parametrize("case", CASES, ids=["M%d_K%d_N%d_sk%d" % c for c in CASES])
def test_structured_only(sp, oracle, torch_cuda, case):
    """2:4 magnitude pruning, then half of the survivors zeroed (75 % sparse): no residual."""
    M, K, N, sk = case
    A1 = prune_2_of_4(sp.synth_fp16((M, K), 500 + M + K, 0.02, 0.0), 0.5, 9)
    B = sp.synth_fp16((K, N), 600 + M + N, 1.0, 0.0)
    C = run_hetero(sp, torch_cuda, A1, None, B, M, N, K, sk)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A1, B))
    assert ok, (max_ratio, mean_rel)
    C_again = run_hetero(sp, torch_cuda, A1, None, B, M, N, K, sk)
    assert np.array_equal(C, C_again)


@pytest.mark.parametrize("case", CASES[1:], ids=["M%d_K%d_N%d_sk%d" % c for c in CASES[1:]])
@pytest.mark.parametrize("v1", [False, True])
def test_with_residual(sp, oracle, torch_cuda, case, v1):
    """i.i.d. sparse A: decompose -> A1 (sparse tensor core) + A2 (tiled-CSL), summed before one rounding."""
    M, K, N, sk = case
    A = sp.synth_fp16((M, K), 700 + M + K, 0.02, 0.6)
    B = sp.synth_fp16((K, N), 800 + M + N, 1.0, 0.0)
    A1, A2 = sp.decompose(A, v1=v1)
    assert (A2 != 0).any()
    C = run_hetero(sp, torch_cuda, A1, A2, B, M, N, K, max(sk, 3))
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A, B))
    assert ok, (max_ratio, mean_rel)


def test_integer_inputs_exact(sp, oracle, torch_cuda):
    """Small-integer weights and activations: every partial sum is exact in fp32 and fp16."""
    M, K, N = 512, 1024, 32
    rng = np.random.default_rng(5)
    A = rng.integers(-2, 3, size=(M, K)).astype(np.float16)
    A[rng.random((M, K)) < 0.5] = 0
    B = rng.choice(np.array([-3, -1, 1, 3], np.float16), size=(K, N))
    A_bits = A.view(np.uint16)
    A1, A2 = sp.decompose(A_bits)
    C = run_hetero(sp, torch_cuda, A1, A2, B.view(np.uint16), M, N, K, 4)
    want = (A.astype(np.float64) @ B.astype(np.float64))
    assert np.abs(want).max() <= 2048
    assert np.array_equal(C.view(np.float16).astype(np.float64), want)


def test_config_4_full_size_exact(sp, torch_cuda):
    """BASELINE config 4 at full size (M = K = 12288, N = 32): integer weights pruned 2:4 with half of the
    survivors zeroed, so the residual is empty and the product runs on the sparse tensor core alone; then
    the same weights with a few third nonzeros per group put back, which go through the residual path."""
    torch = torch_cuda
    M = K = 12288
    N = 32
    rng = np.random.default_rng(13)
    A = rng.integers(1, 3, size=(M, K)).astype(np.float16) * (rng.integers(0, 2, size=(M, K)) * 2 - 1).astype(np.float16)
    A_bits = prune_2_of_4(A.view(np.uint16), 0.5, 17)
    B = rng.choice(np.array([-3, -1, 1, 3], np.float16), size=(K, N))
    Bd = torch.from_numpy(B).cuda().float()
    A1, A2 = sp.decompose(A_bits)
    assert not (A2 & 0x7FFF).any()
    C = run_hetero(sp, torch, A1, None, B.view(np.uint16), M, N, K, 8).view(np.float16)
    expect = (torch.from_numpy(A_bits.view(np.float16)).cuda().float() @ Bd).cpu().numpy()
    assert np.abs(expect).max() < 2048
    assert np.array_equal(C.astype(np.float32), expect)
    # a sprinkle of extra nonzeros: groups with three or four of them feed the residual
    extra = rng.random((M, K), dtype=np.float32) < 0.02
    A_more = np.where(extra & (A_bits == 0), np.float16(1).view(np.uint16), A_bits).astype(np.uint16)
    A1, A2 = sp.decompose(A_more)
    assert (A2 & 0x7FFF).any()
    C = run_hetero(sp, torch, A1, A2, B.view(np.uint16), M, N, K, 8).view(np.float16)
    expect = (torch.from_numpy(A_more.view(np.float16)).cuda().float() @ Bd).cpu().numpy()
    assert np.abs(expect).max() < 2048
    assert np.array_equal(C.astype(np.float32), expect)


def test_error_paths(sp, torch_cuda):
    torch = torch_cuda
    dev = torch.device("cuda:0")
    M, K, N = 128, 128, 16
    A1 = np.zeros((M, K), np.uint16)
    values, meta, _ = sp.InitSparseMatrixA1_tcgen05(A1, M, K)
    vd, md = torch.from_numpy(values).to(dev), torch.from_numpy(meta.view(np.int32)).to(dev)
    Bd = torch.zeros((K, N), dtype=torch.int16, device=dev)
    Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
    words, offsets, _ = sp.InitSparseMatrixA_API(A1, M, N, K)
    wd = torch.from_numpy((words if words.size else np.zeros(4, np.uint32)).view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    # unsupported N: the reference's message and cudaErrorUnknown
    assert sp.SpMM_SplitK_API(None, vd, None, None, md, None, Bd, Cd, M, 24, K, None, 1) == 999
    # K not a multiple of 128
    assert sp.SpMM_SplitK_API(None, vd, None, None, md, None, Bd, Cd, M, N, 64, None, 1) == 1
    # a residual without a workspace for the fp32 hand-over
    assert sp.SpMM_SplitK_API(None, vd, wd, None, md, od, Bd, Cd, M, N, K, None, 4) == 1
    ws = torch.zeros(sp.workspace_bytes(M, N, 1) // 2, dtype=torch.int16, device=dev)
    assert sp.SpMM_SplitK_API(None, vd, wd, None, md, od, Bd, Cd, M, N, K, ws, 1) == 1
    torch.cuda.synchronize()
