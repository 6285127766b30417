"""The entry point for callers that cannot allocate (spmm_b200_spmm_own_scratch).

Some callers of this library are handed device tensors but may not call cudaMalloc and have no
workspace to pass: a plugin callback inside a serving stack, a host whose allocator is frozen
after start-up, a latency-critical loop that must not hit cudaMalloc's implicit synchronisation.  For them the library carries its own scratch
array.  This test calls that entry point through the C boundary twice in a row and checks each
result against the regular entry point (which uses a caller-allocated workspace) within the
tolerance the other GPU tests use; the second call runs on the scratch contents the first left
behind.  Collected last so that a failure here cannot hide any other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [(2304, 4608, 16), (1152, 9216, 64), (1024, 1024, 8)]


@pytest.mark.parametrize("shape", SHAPES, ids=["M%d_K%d_N%d" % s for s in SHAPES])
def test_own_scratch_matches_workspace_entry_point(sp, shape):
    import torch
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    M, K, N = shape
    A = sp.synth_fp16((M, K), 71 + N, 0.02, 0.8)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    wd = torch.from_numpy((words if words.size else np.zeros(4, np.uint32)).view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    ws = torch.zeros(sp.workspace_bytes(M, N, 16) // 2, dtype=torch.int16, device=dev)
    for call in range(2):
        B = sp.synth_fp16((K, N), 80 + call, 1.0, 0.0)
        Bd = torch.from_numpy(B.view(np.int16)).to(dev)
        expect = torch.zeros((M, N), dtype=torch.int16, device=dev)
        got = torch.full((M, N), 0x7E00, dtype=torch.int16, device=dev)
        assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, expect, M, N, K, ws, 16) == 0
        assert sp.spmm_own_scratch(None, wd, od, Bd, got, M, N, K) == 0
        torch.cuda.synchronize()
        assert sp.device_status() == 0
        e = expect.cpu().numpy().view(np.float16).astype(np.float64)
        g = got.cpu().numpy().view(np.float16).astype(np.float64)
        assert np.isfinite(g).all()
        assert np.abs(g - e).max() <= 2e-3 * max(np.abs(e).max(), 1e-6), "call %d" % call


def test_own_scratch_rejects_sizes_beyond_its_maximum(sp, capfd):
    import torch
    dev = torch.device("cuda:0")
    dummy = torch.zeros(64, dtype=torch.int32, device=dev)
    too_many_rows = 128 * 8193
    assert sp.spmm_own_scratch(None, dummy, dummy, dummy, dummy, too_many_rows, 16, 64) == 1
    assert sp.spmm_own_scratch(None, dummy, dummy, dummy, dummy, 256, 24, 64) == 999
    assert sp.spmm_own_scratch(None, dummy, dummy, dummy, dummy, 200, 16, 64) == 1
    torch.cuda.synchronize()
