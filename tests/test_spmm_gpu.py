"""Parity of the CUDA SpMM path, called through the C boundary, against the CPU oracle.

Gates (from the acceptance criteria of the path): the encoded format is bit-exact (checked in
test_encoder.py); C must satisfy max|C - C64| <= 1e-2 * max|C64| and
mean(|C - C64| / max(|C64|, 1e-6)) <= 1e-3 against the fp64 host product.  Integer-valued
inputs, as the reference's harness uses (kernel_benchmark/spmm_test_utils.h:108-141), must
come out exactly."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch


def run_spmm(sp, torch, words, offsets, B_bits, M, N, K, split_k, workspace=True):
    dev = torch.device("cuda:0")
    wd = torch.from_numpy((words if words.size else np.zeros(4, np.uint32)).view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(np.ascontiguousarray(B_bits).view(np.int16)).to(dev)
    Cd = torch.full((M, N), 0x7E00, dtype=torch.int16, device=dev)  # NaN pattern: unwritten rows show up
    ws = torch.zeros(sp.workspace_bytes(M, N, split_k) // 2 + 8, dtype=torch.int16, device=dev) if workspace else None
    rc = sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, N, K, ws, split_k)
    torch.cuda.synchronize()
    assert rc == 0, "launch failed with cudaError %d" % rc
    assert sp.device_status() == 0, "a bounded wait inside the kernel gave up"
    return Cd.cpu().numpy().view(np.uint16)


CASES = [  # M, K, N, sparsity, Split_K
    (128, 64, 16, 0.8, 1),
    (128, 64, 8, 0.5, 1),
    (256, 192, 32, 0.8, 2),
    (384, 128, 64, 0.9, 3),
    (512, 1024, 16, 0.7, 4),      # tiles denser than the register budget: streamed remainder
    (1024, 512, 16, 0.0, 4),      # fully dense tiles (32 KB of words each)
    (1024, 512, 8, 1.0, 4),       # all tiles empty
    (1152, 9216, 16, 0.8, 8),     # many k tiles per row, rows split between blocks
    (2048, 2048, 32, 0.8, 1),     # workspace too small for split rows at Split_K = 1
    (2048, 1024, 64, 0.8, 6),
]


@pytest.mark.parametrize("case", CASES, ids=["M%d_K%d_N%d_p%g_sk%d" % c for c in CASES])
def test_matches_oracle(sp, oracle, torch_cuda, case):
    M, K, N, p, sk = case
    A = sp.synth_fp16((M, K), 1000 + M + K + N, 0.02, p)
    B = sp.synth_fp16((K, N), 2000 + M + K + N, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, sk)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A, B))
    assert ok, (max_ratio, mean_rel)
    # fp32-accumulate CPU product of the decoded words: equal up to summation order
    c32 = oracle.spmm_from_csl(words, offsets, B, M, K).view(np.float16).astype(np.float64)
    diff = np.abs(C.view(np.float16).astype(np.float64) - c32)
    assert diff.max() <= 2e-3 * max(np.abs(c32).max(), 1e-6)


def test_baseline_config_1(sp, oracle, torch_cuda):
    """M = K = 7168, N = 16, 80 % sparse, Split_K = 5: the reference's own CPU-runnable case."""
    M = K = 7168
    N, sk = 16, 5
    A = sp.synth_fp16((M, K), 0xA001, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 0xB001, 1.0, 0.0)
    words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, N, K)
    assert n_offsets == 56 * 112 + 2
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, sk)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A, B))
    assert ok, (max_ratio, mean_rel)


def test_without_workspace(sp, oracle, torch_cuda):
    M, K, N = 1024, 2048, 16
    A = sp.synth_fp16((M, K), 31, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 32, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 1, workspace=False)
    assert oracle.tolerance_check(C, oracle.spmm_f64(A, B))[0]


def test_scan_order_encoding_gives_same_product(sp, torch_cuda):
    M, K, N = 512, 512, 16
    A = sp.synth_fp16((M, K), 41, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 42, 1.0, 0.0)
    w1, o1, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    w2, o2, _ = sp.InitSparseMatrixA_API_NoReorder(A, M, N, K)
    c1 = run_spmm(sp, torch_cuda, w1, o1, B, M, N, K, 4)
    c2 = run_spmm(sp, torch_cuda, w2, o2, B, M, N, K, 4)
    assert np.array_equal(c1, c2)  # same values reach the same tile positions; accumulation order is identical


def test_repeated_calls_are_bitwise_reproducible(sp, torch_cuda):
    M, K, N = 2304, 4608, 16
    A = sp.synth_fp16((M, K), 51, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 52, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    first = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 8)
    for _ in range(3):
        assert np.array_equal(run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 8), first)


@pytest.mark.parametrize("shape", [(27648, 9216), (9216, 36864)], ids=["qkv_66b", "ffn2_66b"])
def test_full_size_integer_inputs_are_exact(sp, torch_cuda, shape):
    """OPT-66B layer shapes with harness-style integer inputs: A in {0, 1}, B in {-3, -1, 1, 3}
    (zero mean, so that sums stay below 2048).  Every partial sum is a small integer, so fp32
    accumulation and the fp16 result are exact."""
    M, K = shape
    N = 16
    rng = np.random.default_rng(7)
    A = np.where(rng.random((M, K), dtype=np.float32) < 0.2, np.float16(1), np.float16(0)).astype(np.float16)
    B = rng.choice(np.array([-3, -1, 1, 3], np.float16), size=(K, N))
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 8).view(np.float16)
    expect = torch_cuda.from_numpy(A).cuda().float() @ torch_cuda.from_numpy(B).cuda().float()
    expect = expect.cpu().numpy()
    assert np.abs(expect).max() < 2048
    assert np.array_equal(C.astype(np.float32), expect)


def test_prefill_full_size_integer_inputs_are_exact(sp, torch_cuda):
    """BASELINE config 3 at full size (M = K = 12288, N = 2048, eight 256-column blocks): A in {-1, 0, 1}
    at 90 % sparsity, B in {-1, 1}; every sum is a small integer, so the fp16 result is exact."""
    M = K = 12288
    N = 2048
    rng = np.random.default_rng(11)
    A = (rng.integers(0, 2, size=(M, K)) * 2 - 1).astype(np.float16)
    A[rng.random((M, K), dtype=np.float32) < 0.9] = 0
    B = (rng.integers(0, 2, size=(K, N)) * 2 - 1).astype(np.float16)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 2).view(np.float16)
    expect = (torch_cuda.from_numpy(A).cuda().float() @ torch_cuda.from_numpy(B).cuda().float()).cpu().numpy()
    assert np.abs(expect).max() < 2048
    assert np.array_equal(C.astype(np.float32), expect)


def test_linearity_at_full_size(sp, torch_cuda):
    """C(A, B1) + C(A, B2) == C(A, B1 + B2) for power-of-two scaled integer inputs (all sums exact)."""
    M, K, N = 9216, 9216, 32
    rng = np.random.default_rng(9)
    A = (rng.integers(-2, 3, size=(M, K)) * (rng.random((M, K)) < 0.25)).astype(np.float16)
    B1 = rng.integers(-2, 3, size=(K, N)).astype(np.float16)
    B2 = rng.integers(-2, 3, size=(K, N)).astype(np.float16)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    c1 = run_spmm(sp, torch_cuda, words, offsets, B1, M, N, K, 6).view(np.float16).astype(np.float32)
    c2 = run_spmm(sp, torch_cuda, words, offsets, B2, M, N, K, 6).view(np.float16).astype(np.float32)
    c12 = run_spmm(sp, torch_cuda, words, offsets, B1 + B2, M, N, K, 6).view(np.float16).astype(np.float32)
    assert np.abs(c12).max() < 2048 and np.array_equal(c1 + c2, c12)


def test_error_paths(sp, torch_cuda, capfd):
    torch = torch_cuda
    dev = torch.device("cuda:0")
    M, K, N = 256, 128, 16
    A = sp.synth_fp16((M, K), 61, 0.02, 0.8)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    wd = torch.from_numpy((words if words.size else np.zeros(4, np.uint32)).view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bd = torch.zeros((K, 64), dtype=torch.int16, device=dev)
    Cd = torch.zeros((M, 64), dtype=torch.int16, device=dev)
    ws = torch.zeros(M * 64 * 4, dtype=torch.int16, device=dev)
    # unsupported N: the reference's message and cudaErrorUnknown (csrc/SpMM_API.cu:192-193)
    assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, 24, K, ws, 4) == 999
    # shapes the tile format cannot describe
    assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, 200, 16, K, ws, 4) == 1
    assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, 16, 100, ws, 4) == 1
    assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, 16, K, ws, 0) == 1
    # misaligned and missing pointers
    assert sp.SpMM_SplitK_API(None, None, wd.data_ptr() + 4, None, None, od, Bd, Cd, M, 16, K, ws, 4) == 1
    assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, None, Cd, M, 16, K, ws, 4) == 1
    # a failed call leaves no sticky error behind
    assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, 16, K, ws, 4) == 0
    torch.cuda.synchronize()
    assert sp.device_status() == 0


@pytest.mark.parametrize("case", [(256, 192, 8, 0.8), (1024, 2048, 16, 0.8), (2304, 4608, 32, 0.7), (1152, 1024, 64, 0.9)],
                         ids=["N8", "N16", "N32", "N64"])
def test_token_major_layout(sp, oracle, torch_cuda, case):
    """The upstream eleven-argument form (third_party/ft.patch:2822-2846): B[N][K], C[N][M]."""
    torch = torch_cuda
    dev = torch.device("cuda:0")
    M, K, N, p = case
    A = sp.synth_fp16((M, K), 300 + N, 0.02, p)
    B = sp.synth_fp16((K, N), 400 + N, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    wd = torch.from_numpy((words if words.size else np.zeros(4, np.uint32)).view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bt = torch.from_numpy(np.ascontiguousarray(B.T).view(np.int16)).to(dev)          # [N][K]
    Ct = torch.full((N, M), 0x7E00, dtype=torch.int16, device=dev)                   # [N][M]
    ws = torch.zeros(sp.workspace_bytes(M, N, 8) // 2, dtype=torch.int16, device=dev)
    assert sp.SpMM_SplitK_API_token_major(None, wd, od, Bt, Ct, M, N, K, ws, 8) == 0
    torch.cuda.synchronize()
    assert sp.device_status() == 0
    C = np.ascontiguousarray(Ct.cpu().numpy().view(np.uint16).T)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A, B))
    assert ok, (max_ratio, mean_rel)
    # same accumulation as the row-major entry point: bitwise equal results
    assert np.array_equal(C, run_spmm(sp, torch, words, offsets, B, M, N, K, 8))


@pytest.mark.parametrize("case", [(512, 1024, 128, 0.8), (1152, 2304, 256, 0.7), (2304, 1152, 512, 0.5),
                                  (1024, 1024, 192, 0.8), (2304, 4608, 384, 0.8), (4608, 9216, 1024, 0.6)],
                         ids=["N128", "N256", "N512", "N192", "N384", "N1024"])
def test_wide_n_in_column_blocks(sp, oracle, torch_cuda, case):
    """N beyond the reference's 64 (prefill sizes): multiples of 64, served in column blocks of 256, 128 or
    64 columns (the widest that divides N), one block per blockIdx.y."""
    M, K, N, p = case
    A = sp.synth_fp16((M, K), 500 + N, 0.02, p)
    B = sp.synth_fp16((K, N), 600 + N, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch_cuda, words, offsets, B, M, N, K, 4)
    ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64(A, B))
    assert ok, (max_ratio, mean_rel)
    # a 64-column slice equals the N = 64 product of that slice of B (the partition may differ, hence a tolerance)
    block = run_spmm(sp, torch_cuda, words, offsets, np.ascontiguousarray(B[:, 64:128]), M, 64, K, 4)
    a, b = C[:, 64:128].view(np.float16).astype(np.float64), block.view(np.float16).astype(np.float64)
    assert np.abs(a - b).max() <= 2e-3 * np.abs(b).max()


def test_peer_reduction_gives_up_when_a_peer_never_arrives(sp, torch_cuda):
    """Failure detection without a fault, for the row-parallel reduction kernel: rank 0 of a world of two whose
    peer never signals.  The bounded wait runs out after 50 ms, the kernel returns, the output is untouched,
    the status says so, and with both flags set the same call then sums the two buffers."""
    import ctypes
    torch = torch_cuda
    dev = torch.device("cuda:0")
    lib = sp.spmm_api.LIB
    count = 4096
    mine = torch.full((count,), 1.5, dtype=torch.float16, device=dev)
    theirs = torch.full((count,), 2.25, dtype=torch.float16, device=dev)
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]
    out = torch.full((count,), -1.0, dtype=torch.float16, device=dev)
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
    fptrs = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.spmm_b200_allreduce_status(1) >= 0
    assert lib.spmm_b200_allreduce_partials(stream, ptrs, fptrs, 0, 2, ctypes.c_void_p(out.data_ptr()), count, 1, 50) == 0
    assert lib.spmm_b200_allreduce_status(1) == 1
    assert bool((out == -1.0).all())
    flags[0][1] = 2  # what the peer would have written for epoch 2
    torch.cuda.synchronize()
    assert lib.spmm_b200_allreduce_partials(stream, ptrs, fptrs, 0, 2, ctypes.c_void_p(out.data_ptr()), count, 2, 50) == 0
    assert lib.spmm_b200_allreduce_status(0) == 0
    assert bool((out == 3.75).all())


def test_host_buffer_entry_point(sp, oracle, torch_cuda):
    """The C call that takes B and C in page-locked host memory gives the result of the device-pointer call."""
    torch = torch_cuda
    dev = torch.device("cuda:0")
    M, K, N, sk = 1152, 2304, 16, 8
    A = sp.synth_fp16((M, K), 901, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 902, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    want = run_spmm(sp, torch, words, offsets, B, M, N, K, sk)
    wd = torch.from_numpy((words if words.size else np.zeros(4, np.uint32)).view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    B_host = torch.from_numpy(B.view(np.int16)).pin_memory()
    C_host = torch.zeros((M, N), dtype=torch.int16).pin_memory()
    B_dev = torch.zeros((K, N), dtype=torch.int16, device=dev)
    C_dev = torch.zeros((M, N), dtype=torch.int16, device=dev)
    ws = torch.zeros(sp.workspace_bytes(M, N, sk) // 2, dtype=torch.int16, device=dev)
    rc = sp.SpMM_SplitK_API_host_io(None, wd, od, B_host, C_host, B_dev, C_dev, M, N, K, ws, sk)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(C_host.numpy().view(np.uint16), want)


def test_host_buffer_batches_back_to_back_share_staging_buffers(sp, oracle, torch_cuda):
    """Batches of two products queued one after the other without a synchronisation in between, each with its
    own activations and results in page-locked host memory but all through the same device staging buffers: the
    copies in of a batch must wait for the products of the batch before it, its products for that batch's copies
    out.  Every batch must give the result of the device-pointer call on its own activations."""
    torch = torch_cuda
    dev = torch.device("cuda:0")
    shapes = [(1152, 2304), (2304, 1152)]
    N, sk, batches = 16, 8, 4
    layers = []
    for li, (M, K) in enumerate(shapes):
        A = sp.synth_fp16((M, K), 910 + li, 0.02, 0.8)
        words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
        layers.append(dict(M=M, K=K, words=words, offsets=offsets,
                           wd=torch.from_numpy(words.view(np.int32)).to(dev), od=torch.from_numpy(offsets).to(dev),
                           B_dev=torch.zeros((K, N), dtype=torch.int16, device=dev),
                           C_dev=torch.zeros((M, N), dtype=torch.int16, device=dev),
                           ws=torch.zeros(sp.workspace_bytes(M, N, sk) // 2, dtype=torch.int16, device=dev)))
    B = [[sp.synth_fp16((L["K"], N), 920 + 10 * b + li, 1.0, 0.0) for li, L in enumerate(layers)] for b in range(batches)]
    want = [[run_spmm(sp, torch, L["words"], L["offsets"], B[b][li], L["M"], N, L["K"], sk) for li, L in enumerate(layers)]
            for b in range(batches)]
    B_host = [[torch.from_numpy(B[b][li].view(np.int16)).pin_memory() for li in range(len(layers))] for b in range(batches)]
    C_host = [[torch.zeros((L["M"], N), dtype=torch.int16).pin_memory() for L in layers] for b in range(batches)]
    items = [sp.host_io_items([dict(Compressed_A=L["wd"], TileOffsets=L["od"], B_host=B_host[b][li], C_host=C_host[b][li],
                                    B_dev=L["B_dev"], C_dev=L["C_dev"], M=L["M"], N=N, K=L["K"],
                                    Reduction_Workspace=L["ws"], Split_K=sk) for li, L in enumerate(layers)])
             for b in range(batches)]
    stream = torch.cuda.Stream()
    for _ in range(2):  # the second round starts with results of the first still on their way out
        for b in range(batches):
            assert sp.SpMM_SplitK_API_host_io_batch(stream, items[b]) == 0
    stream.synchronize()
    assert sp.device_status() == 0
    for b in range(batches):
        for li in range(len(layers)):
            assert np.array_equal(C_host[b][li].numpy().view(np.uint16), want[b][li]), (b, li)


def test_a_wait_that_runs_out_is_reported_not_hung(sp, oracle, torch_cuda):
    """Failure detection without a fault: a kernel waits on a barrier nothing arrives on; the bounded
    wait gives up after 50 ms, the kernel returns, the status word says so, and the device keeps working."""
    torch = torch_cuda
    assert sp.device_status(reset=True) == 0
    assert sp.selftest_wait_timeout(50) == 0
    torch.cuda.synchronize()
    assert sp.device_status() == 1
    assert sp.device_status(reset=True) == 1
    assert sp.device_status() == 0
    M, K, N = 256, 256, 16
    A = sp.synth_fp16((M, K), 91, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 92, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    C = run_spmm(sp, torch, words, offsets, B, M, N, K, 4)
    assert oracle.tolerance_check(C, oracle.spmm_f64(A, B))[0]


def test_weights_written_by_the_preceding_kernel(sp, oracle, torch_cuda):
    """The SpMM is launched so that it may start while its stream predecessor drains.  By default it reads
    nothing before that predecessor has completed, so weights (and offsets) produced by the kernel directly
    ahead of it -- here an elementwise kernel that fills the buffers -- are seen in full."""
    torch = torch_cuda
    dev = torch.device("cuda:0")
    assert sp.set_weights_constant(False) in (True, False)
    M, K, N = 4608, 9216, 16
    A = sp.synth_fp16((M, K), 111, 0.02, 0.8)
    B = sp.synth_fp16((K, N), 112, 1.0, 0.0)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    src_w = torch.from_numpy(words.view(np.int32)).to(dev)
    src_o = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(B.view(np.int16)).to(dev)
    ws = torch.zeros(sp.workspace_bytes(M, N, 8) // 2, dtype=torch.int16, device=dev)
    want = None
    for attempt in range(3):
        wd = torch.zeros_like(src_w)      # all-zero words: every value lands on position 0 with value 0
        od = torch.zeros_like(src_o)
        Cd = torch.full((M, N), 0x7E00, dtype=torch.int16, device=dev)
        torch.cuda.synchronize()
        torch.add(src_o, 0, out=od)       # kernels on the same stream, directly ahead of the SpMM
        torch.add(src_w, 0, out=wd)
        assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, N, K, ws, 8) == 0
        torch.cuda.synchronize()
        assert sp.device_status() == 0
        C = Cd.cpu().numpy().view(np.uint16)
        if want is None:
            ok, max_ratio, mean_rel = oracle.tolerance_check(C, oracle.spmm_f64_threads(A, B))
            assert ok, (max_ratio, mean_rel)
            want = C
        assert np.array_equal(C, want), "attempt %d" % attempt


def test_row_parallel_entry_point_on_one_rank(sp, torch_cuda):
    """spmm_b200_spmm_row_parallel with a world of one, in both forms (the sum inside the SpMM kernel, or the SpMM
    writing fp32 partial rows and spmm_b200_allreduce_partials_f32 following it): the finished rows travel through
    the partial buffer in fp32, the flags are this rank's own, and the sum over 'ranks' is a copy with one rounding.
    Same bits as SpMM_SplitK_API, call after call (the epoch advances and the partial buffers alternate), also when
    replayed from a CUDA graph."""
    torch = torch_cuda
    from graphneuralnetproj_b200 import tensor_parallel as tp
    dev = torch.device("cuda:0")
    for M, K, N in ((2304, 4608, 16), (1152, 9216, 64), (1024, 1024, 8)):
        A = sp.synth_fp16((M, K), 700 + N, 0.02, 0.8)
        B = sp.synth_fp16((K, N), 800 + N, 1.0, 0.0)
        words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
        want = run_spmm(sp, torch, words, offsets, B, M, N, K, 8)
        wd = torch.from_numpy(words.view(np.int32)).to(dev)
        od = torch.from_numpy(offsets).to(dev)
        Bd = torch.from_numpy(B.view(np.int16)).to(dev)
        for fused in (True, False):
            layer = tp.FusedRowParallelSpMM(wd, od, M, N, K, fused=fused)
            for call in range(3):
                layer.C.fill_(float("nan"))
                out = layer.forward(Bd)
                torch.cuda.synchronize()
                assert sp.device_status() == 0
                assert np.array_equal(out.cpu().numpy().view(np.uint16), want), (M, K, N, fused, call)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    out = layer.forward(Bd)
                for replay in range(4):
                    layer.C.fill_(float("nan"))
                    graph.replay()
                    torch.cuda.synchronize()
                    assert np.array_equal(out.cpu().numpy().view(np.uint16), want), (M, K, N, fused, "replay", replay)
            assert int(layer.state[0].item()) == 3 + 4 and int(layer.state[1].item()) == 0
            assert sp.device_status() == 0 and sp.spmm_api.LIB.spmm_b200_allreduce_status(0) == 0
