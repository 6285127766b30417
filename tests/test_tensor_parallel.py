"""Tensor-parallel splits of one layer: column-parallel by rows of A (no collective) and
row-parallel by K (one sum all-reduce).  The CPU tests run two gloo ranks with the oracle as the
local product; the GPU test runs two NCCL ranks on two GPUs through the CUDA SpMM."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_shards_are_slices_of_the_whole_encoding(sp):
    from graphneuralnetproj_b200 import tensor_parallel as tp
    M, K = 1024, 512
    A = sp.synth_fp16((M, K), 5, 0.02, 0.8)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, 16, K)
    for world in (1, 2, 4, 8):
        for rank in range(world):
            w, o, m = tp.row_shard(words, offsets, M, K, rank, world)
            rows = A[rank * m:(rank + 1) * m]
            w_alone, o_alone, _ = sp.InitSparseMatrixA_API(rows, m, 16, K)
            assert m == M // world and np.array_equal(w, w_alone) and np.array_equal(o, o_alone)
    with pytest.raises(ValueError):
        tp.row_shard(words, offsets, M, K, 0, 3)


WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, {root!r})
import graphneuralnetproj_b200 as sp
from graphneuralnetproj_b200 import tensor_parallel as tp
import oracle
backend, mode = sys.argv[1], sys.argv[2]
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
if backend == "nccl":
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
else:
    dist.init_process_group("gloo")
M, K, N = 1024, 2048, 16
A = sp.synth_fp16((M, K), 11, 0.02, 0.8)
B = sp.synth_fp16((K, N), 12, 1.0, 0.0)
C64 = oracle.spmm_f64(A, B)
if mode == "column":
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, N, K)
    w, o, m = tp.row_shard(words, offsets, M, K, rank, world)
    if backend == "nccl":
        dev = torch.device("cuda", rank)
        Cd = torch.zeros((m, N), dtype=torch.int16, device=dev)
        ws = torch.zeros(sp.workspace_bytes(m, N, 8) // 2, dtype=torch.int16, device=dev)
        rc = sp.SpMM_SplitK_API(None, None, torch.from_numpy(w.view(np.int32)).to(dev), None, None,
                                torch.from_numpy(o).to(dev), torch.from_numpy(B.view(np.int16)).to(dev), Cd, m, N, K, ws, 8)
        torch.cuda.synchronize(); assert rc == 0 and sp.device_status() == 0
        mine = Cd.cpu().numpy().view(np.uint16)
    else:
        mine = oracle.spmm_from_csl(w, o, B, m, K)
    ok, mx, mr = oracle.tolerance_check(mine, C64[rank * m:(rank + 1) * m])
    assert ok, (mx, mr)
    # no collective on the data path: only the verdicts are gathered
    flag = torch.tensor([1 if ok else 0], device="cuda" if backend == "nccl" else "cpu")
    dist.all_reduce(flag)
    assert int(flag.item()) == world
else:
    As, Bs = tp.column_slice(A, rank, world), tp.activation_rows(B, rank, world)
    k = K // world
    w, o, _ = sp.InitSparseMatrixA_API(As, M, N, k)
    if backend == "nccl":
        dev = torch.device("cuda", rank)
        layer = tp.RowParallelSpMM(torch.from_numpy(w.view(np.int32)).to(dev),
                                   torch.from_numpy(o).to(dev), M, N, k, reduce="peer" if mode == "row_peer" else "nccl")  # row_peer_graph starts from the NCCL answer
        Bd = torch.from_numpy(Bs.view(np.int16)).to(dev)
        C = layer.forward(Bd)
        torch.cuda.synchronize(); assert sp.device_status() == 0
        total = C.cpu().numpy().view(np.uint16)
        if mode == "row_peer":
            # the library's own reduction over peer memory: several calls in a row (the two result buffers
            # alternate), each with the same answer, and the wait for the peers never ran out
            for _ in range(5):
                again = layer.forward(Bd)
            torch.cuda.synchronize()
            assert sp.spmm_api.LIB.spmm_b200_allreduce_status(0) == 0
            assert np.array_equal(again.cpu().numpy().view(np.uint16), total)
        if mode == "row_peer_graph":
            # the replayable form (epoch kept on the device): two layers whose reductions alternate, captured
            # once in a CUDA graph and replayed; every replay must give the un-captured answer
            layers = [tp.RowParallelSpMM(layer.words, layer.offsets, M, N, k, reduce="peer", replayable=True) for _ in range(2)]
            for L in layers:
                L.forward(Bd)
            torch.cuda.synchronize()
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    outs = [L.forward(Bd) for L in layers]
                for replay in range(6):
                    for out in outs:
                        out.zero_()
                    g.replay()
                    torch.cuda.synchronize()
                    for out in outs:
                        assert np.array_equal(out.cpu().numpy().view(np.uint16), total), replay
            assert sp.spmm_api.LIB.spmm_b200_allreduce_status(0) == 0
        if mode in ("row_fused", "row_two_launches", "row_two_phase", "row_announced"):
            # fp32 partial rows summed out of peer memory, inside the SpMM kernel or by the reduction kernel
            # launched after it: un-captured calls, then a captured pair replayed; one rounding, so the result
            # is at least as close to the fp64 product as the all-reduced fp16 results
            # (row_two_phase: every rank sums its half of the rows and stores the result into both ranks' buffers)
            fused = tp.FusedRowParallelSpMM(layer.words, layer.offsets, M, N, k, fused=(mode == "row_fused"),
                                            two_phase=(mode == "row_two_phase"), announce=(mode == "row_announced"))
            for call in range(3):
                fused.C.fill_(float("nan"))
                out = fused.forward(Bd)
                torch.cuda.synchronize()
                if call == 0:
                    total = out.cpu().numpy().view(np.uint16).copy()
                assert np.array_equal(out.cpu().numpy().view(np.uint16), total), call
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    fused.forward(Bd)
                    out = fused.forward(Bd)
                for replay in range(5):
                    fused.C.fill_(float("nan"))
                    g.replay()
                    torch.cuda.synchronize()
                    assert np.array_equal(out.cpu().numpy().view(np.uint16), total), replay
            assert sp.device_status() == 0
    else:
        part = torch.from_numpy(oracle.spmm_from_csl(w, o, Bs, M, k).view(np.float16).astype(np.float32))
        total = tp.all_reduce_partial(part).numpy().astype(np.float16).view(np.uint16)
    ok, mx, mr = oracle.tolerance_check(total, C64)
    assert ok, (mx, mr)
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def run_ranks(world, backend, mode):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER.format(root=ROOT), backend, mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for p, out in zip(procs, outs):
        assert p.returncode == 0, out[-3000:]


@pytest.mark.parametrize("mode", ["column", "row"])
def test_two_gloo_ranks_on_cpu(mode):
    run_ranks(2, "gloo", mode)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["column", "row", "row_peer", "row_peer_graph", "row_fused", "row_two_launches", "row_two_phase", "row_announced"])
def test_two_nccl_ranks_on_gpus(mode):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_ranks(2, "nccl", mode)
