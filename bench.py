"""Benchmark of the sparse-weight SpMM hot path on B200.

A step is one pass over the four linear layers of an OPT-66B decoder block at decode size
(QKV 27648x9216, out-proj 9216x9216, FFN1 36864x9216, FFN2 9216x36864; N = 16 tokens, 80 %
i.i.d. sparsity, fp16 in, fp32 accumulate): four SpMM launches through the C boundary of
libSpMM_API.so.  Weights are seeded synthetic stand-ins for pruned OPT weights, encoded with
the library's InitSparseMatrixA_API and resident in HBM before the timed region.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Prints one JSON line (rank 0).  `value` is effective weight-HBM GB/s: (4*NNZ_pad + 4*NumOffsets)
summed over the step and all ranks, divided by the device time of a step (max over ranks).

With N > 1 the SAME block is sharded tensor-parallel the way the reference's conversion tool shards
it (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:134-135): QKV and FFN1 by output
rows (no collective), out-proj and FFN2 by K with the sum over ranks inside the timed step (strong
scaling).  Every rank draws only its own shard of the seeded matrix, which is bit-identical to
cutting the shard out of the whole matrix.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# name, M, K, how the layer is split over ranks, Split_K (sizes the workspace: Split_K * M * N * 2 bytes)
LAYERS = [
    ("qkv", 27648, 9216, "rows", 4),
    ("out_proj", 9216, 9216, "cols", 8),
    ("ffn1", 36864, 9216, "rows", 4),
    ("ffn2", 9216, 36864, "cols", 8),
]
# OPT-175B layer shapes of the tensor-parallel configuration (hidden 12288, FFN 49152)
LAYERS_175B = [
    ("qkv_175b", 36864, 12288, "rows", 4),
    ("ffn1_175b", 49152, 12288, "rows", 4),
    ("ffn2_175b", 12288, 49152, "cols", 8),
]
N_TOKENS = 16
SPARSITY = 0.8
WORKLOAD = "opt66b_decoder_block_4_spmm_n16_p0.8"
METRIC = "effective weight-HBM GB/s, SpMM (OPT-66B shapes, N=16, 80% sparse)"
HBM_PEAK_FALLBACK_GBS = 6650.0
ROTATE_BYTES = 256e6  # weights a timed loop cycles through: twice what L2 (126 MB) holds
SEED_A, SEED_B = 0xA000, 0xB000
# dram__bytes_read + dram__bytes_write over algorithmic bytes of one launch of the decode kernel, from an
# ncu capture of the FFN1 launch (272.6 + 3.3 MB against 273.5 MB)
DRAM_TRAFFIC_OVER_ALGORITHMIC = 1.009


def measured_peak(key, fallback):
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)[key]), "measured"
    except Exception:
        return fallback, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_flag = threading.Event()
        self.window = None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            names = {
                "hw_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(pynvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            }
            while not self._stop_flag.is_set():
                mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                now = time.time()
                self.samples.append((now, mhz))
                if self.window and self.window[0] <= now and (self.window[1] is None or now <= self.window[1]):
                    for name, bit in names.items():
                        if mask & bit:
                            self.reasons.add(name)
                time.sleep(0.005)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add("nvml_unavailable:%s" % type(e).__name__)

    def stop(self):
        self._stop_flag.set()
        self.join(timeout=2)

    def summary(self, t0, t1):
        inside = [m for (t, m) in self.samples if t0 <= t <= t1]
        return {"sm_mhz": float(np.median(inside)) if inside else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(inside)}


def algorithmic_bytes(n_words, n_offsets, M, K, N):
    """Compulsory traffic of one SpMM: words + offsets + B + C."""
    return 4 * n_words + 4 * n_offsets + 2 * K * N + 2 * M * N


def shard_shape(M, K, split, world):
    return (M // world, K) if split == "rows" else (M, K // world)


def shard_block(M, K, split, rank, world):
    """(rows, cols, row0, col0) of rank's shard inside the M x K matrix."""
    m, k = shard_shape(M, K, split, world)
    return (m, k, rank * m, 0) if split == "rows" else (m, k, 0, rank * k)


# --------------------------------------------------------------------------------------------- GPU arm
class Layer:
    """One rank's shard of one linear layer, resident on the device, with everything the step needs."""

    def __init__(self, sp, torch, dev, name, M, K, split, split_k, seed_a, seed_b, rank, world, N, keep_dense):
        self.name, self.M_full, self.K_full, self.split, self.split_k, self.N = name, M, K, split, split_k, N
        self.seed_a = seed_a
        m, k, row0, col0 = shard_block(M, K, split, rank, world)
        self.M, self.K, self.row0, self.col0 = m, k, row0, col0
        A = sp.synth_fp16_block(m, k, K, row0, col0, seed_a, 0.02, SPARSITY)
        words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, m, N, k)
        self.weight_bytes = 4 * words.size + 4 * n_offsets
        self.algo_bytes = algorithmic_bytes(words.size, n_offsets, m, k, N)
        copies = min(12, max(1, int(np.ceil(ROTATE_BYTES / self.weight_bytes))))
        first = torch.from_numpy(words.view(np.int32)).to(dev)
        self.words = [first] + [first.clone() for _ in range(copies - 1)]
        self.offsets = torch.from_numpy(offsets).to(dev)
        B_full = sp.synth_fp16((K, N), seed_b, 1.0)
        self.B_full = B_full
        B_mine = B_full if split == "rows" else np.ascontiguousarray(B_full[col0:col0 + k])
        self.B_host = torch.from_numpy(B_mine.view(np.int16)).pin_memory()
        self.B = self.B_host.to(dev)
        self.C = torch.zeros((m, N), dtype=torch.int16, device=dev)
        self.C_host = torch.zeros((m, N), dtype=torch.int16).pin_memory()
        self.ws = torch.zeros(sp.workspace_bytes(m, N, split_k) // 2, dtype=torch.int16, device=dev)
        self.dense = None
        if keep_dense:
            dense_copies = min(12, max(1, int(np.ceil(ROTATE_BYTES / (2.0 * m * k)))))
            d0 = torch.from_numpy(A.view(np.float16)).to(dev)
            self.dense = [d0] + [d0.clone() for _ in range(dense_copies - 1)]
        self.pair = None      # row-parallel layers, world > 1: fp32 partial rows + the reduction kernel over peer memory
        self.pair2 = None     # the same partial rows + the two-phase reduction kernel (each rank sums its share of the rows)
        self.paira = None     # partial rows announced to the peers by the SpMM's last block + the reduction kernel
        self.fused = None     # the same sum inside the SpMM kernel
        self.result = self.C  # where the layer's final result lies after a step

    def launch(self, sp, copy, C=None):
        rc = sp.SpMM_SplitK_API(None, None, self.words[copy % len(self.words)], None, None, self.offsets, self.B,
                                self.C if C is None else C, self.M, self.N, self.K, self.ws, self.split_k)
        if rc != 0:
            raise RuntimeError("SpMM_SplitK_API failed with cudaError %d" % rc)


def verify_layer(sp, layer, C_bits, rows_global, label):
    """Checks rows of the layer's result against the oracle's fp64 product (the checker, not the product):
    max|err| <= 1e-2 max|C64| and mean relative error <= 1e-3 over the sampled rows."""
    import oracle
    A_rows = np.concatenate([sp.synth_fp16_block(128, layer.K_full, layer.K_full, int(r0), 0, layer.seed_a, 0.02, SPARSITY)
                             for r0 in rows_global[::128]], axis=0)
    c64 = oracle.spmm_f64_threads(A_rows, layer.B_full)
    ok, max_ratio, mean_rel = oracle.tolerance_check(np.ascontiguousarray(C_bits), c64)
    return {"layer": label, "rows": int(len(rows_global)), "ok": bool(ok), "max_err_over_max_c": float("%.3g" % max_ratio),
            "mean_rel_err": float("%.3g" % mean_rel)}


def sample_rows(sp, layer, rng):
    """Local row indices to verify, whole rows of tiles: the first and the last, up to four whose K range is split
    between thread blocks, and two more picked at random."""
    tiles_m, tiles_k = layer.M // 128, layer.K // 64
    cb, _, _ = sp.plan(tiles_m, tiles_k, 148, 1 << 30)
    split = sorted({int(b) // tiles_k for b in cb[1:-1] if int(b) % tiles_k != 0})
    picks = {0, tiles_m - 1} | set(split[:2] + split[-2:]) | set(int(x) for x in rng.integers(0, tiles_m, 2))
    return np.concatenate([np.arange(t * 128, (t + 1) * 128) for t in sorted(picks)])


def graph_of(torch, stream, fn):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    return g


def run_ours(args):
    import torch
    import torch.distributed as dist

    import graphneuralnetproj_b200 as sp
    from graphneuralnetproj_b200 import tensor_parallel as tp

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:  # the ranks share the host: each gets its share of the cores for generating and encoding its shards
        os.environ.setdefault("SPMM_B200_THREADS", str(max(1, (os.cpu_count() or 8) // world)))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    # inference weights are constant: let every launch fetch them while its predecessor drains
    sp.set_weights_constant(os.environ.get("SPMM_WEIGHTS_CONSTANT", "1") != "0")
    N = N_TOKENS
    warmup = max(args.warmup, 3)
    hbm_peak, peak_kind = measured_peak("hbm_gbs", HBM_PEAK_FALLBACK_GBS)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def leave(code):
        """Ends the process once every rank is done, without tearing down the process group, the captured graphs and
        the symmetric-memory mappings one by one (with several ranks that teardown was seen to hang)."""
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            try:
                torch.cuda.synchronize()
                dist.barrier()
            except Exception:
                pass
            os._exit(code)
        raise SystemExit(code)

    def reduce_max(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def reduce_sum(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t.tolist()

    def build(specs, seed_base, keep_dense):
        out = []
        for li, (name, M, K, split, sk) in enumerate(specs):
            if (M if split == "rows" else K) % (world * (128 if split == "rows" else 64)):
                raise SystemExit("%s cannot be split %d ways" % (name, world))
            out.append(Layer(sp, torch, dev, name, M, K, split, sk, SEED_A + seed_base + li, SEED_B + seed_base + li,
                             rank, world, N, keep_dense))
        return out

    def add_peer_reducers(some_layers):
        for L in some_layers:
            if L.split == "cols":
                L.pair = tp.FusedRowParallelSpMM(L.words[0], L.offsets, L.M, N, L.K, split_k=L.split_k, fused=False)
                L.paira = tp.FusedRowParallelSpMM(L.words[0], L.offsets, L.M, N, L.K, split_k=L.split_k, fused=False,
                                                  announce=True)
                L.pair2 = tp.FusedRowParallelSpMM(L.words[0], L.offsets, L.M, N, L.K, split_k=L.split_k, fused=False,
                                                  two_phase=True)
                L.fused = tp.FusedRowParallelSpMM(L.words[0], L.offsets, L.M, N, L.K, split_k=L.split_k, fused=True)

    layers = build(LAYERS, 0, True)
    # ---- the sum over ranks of the layers split by K: NCCL all-reduce, and the library's own kernel
    peer_ok = False
    if world > 1:
        try:
            add_peer_reducers(layers)
            peer_ok = True
        except Exception as exc:  # symmetric memory not available on this box
            if rank == 0:
                print("peer-memory reduction unavailable:", exc, file=sys.stderr)
        peer_ok = reduce_sum([1.0 if peer_ok else 0.0])[0] == world
    # "peer": fp32 partial rows, then the library's reduction kernel over peer memory (two launches; every rank pulls all
    # ranks' rows); "peer2": the two-phase form of that kernel (every rank sums its share of the rows and pushes the
    # result to all ranks: fewer bytes but one more flag exchange, measured 3-5 us slower per sum on 2 and 4 GPUs);
    # "fused": the sum inside the SpMM kernel (one launch); "nccl": fp16 results all-reduced by NCCL; "none": no sum
    # (timing only)
    # "peera": as "peer", but the SpMM's last block flags the partial rows to the peers, so the exchange of flags
    # overlaps the launch of the reduction kernel
    # The main mode is the first of these that passes the check below: "peera" (1-1.5 % faster per step than "peer" on
    # 2 and 4 GPUs), else "peer", ...
    modes = ["none"] if world == 1 else (["peera", "peer", "peer2", "fused", "nccl", "none"] if peer_ok else ["nccl", "none"])
    main_mode = modes[0]

    def run_layer(L, copy, mode, use):
        """SpMM of layer L (+ the sum over ranks for a layer split by K).  `use`: running count of uses of L, for the
        alternation between its two peer-reduction objects."""
        if L.split == "cols" and mode in ("fused", "peer", "peera", "peer2"):
            layer = {"fused": L.fused, "peer": L.pair, "peera": L.paira, "peer2": L.pair2}[mode]
            L.result = layer.forward(L.B, words=L.words[copy % len(L.words)]).view(torch.int16)
        else:
            L.launch(sp, copy)
            if L.split == "cols" and mode == "nccl":
                dist.all_reduce(L.C.view(torch.float16), op=dist.ReduceOp.SUM)
            L.result = L.C

    def time_launches(stream, fn, count):
        """us per call of fn: a CUDA graph of `count` calls (count even), replayed five times."""
        g = graph_of(torch, stream, lambda: [fn(i) for i in range(count)])
        g.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(5):
            g.replay()
        e1.record(stream)
        barrier()
        return reduce_max([e0.elapsed_time(e1) * 1000.0 / (5 * count)])[0]

    def layer_record(stream, L, with_cublas):
        count = max(8, 2 * len(L.words))
        entry = {"shard": [L.M, L.K], "split": L.split if world > 1 else "none",
                 "spmm_us": round(time_launches(stream, lambda i: L.launch(sp, i), count), 2)}
        if L.split == "cols" and world > 1:
            for mode in modes[:-1]:
                entry["spmm_plus_%s_reduce_us" % mode] = round(
                    time_launches(stream, lambda i, mode=mode: run_layer(L, i, mode, i), count), 2)
        if with_cublas and L.dense is not None:
            Bh = L.B.view(torch.float16)
            out = torch.empty((L.M, N), dtype=torch.float16, device=dev)
            torch.matmul(L.dense[0], Bh, out=out)  # cuBLAS creates its handle and workspace outside the capture
            torch.cuda.synchronize()
            count_d = max(8, 2 * len(L.dense))
            entry["cublas_dense_us"] = round(
                time_launches(stream, lambda i: torch.matmul(L.dense[i % len(L.dense)], Bh, out=out), count_d), 2)
            entry["speedup_vs_cublas"] = round(entry["cublas_dense_us"] / entry["spmm_us"], 3)
        entry["roofline_frac"] = round(L.algo_bytes / entry["spmm_us"] / 1e3 / hbm_peak, 4)
        entry["hbm_floor_us"] = round(L.algo_bytes / hbm_peak / 1e3, 2)
        if L.split == "cols" and world > 1:
            best = entry["spmm_plus_%s_reduce_us" % modes[0]]
            entry["limited_by"] = ("sum over ranks: +%.1f us on a %.1f us product (HBM floor %.1f us)"
                                   % (best - entry["spmm_us"], entry["spmm_us"], entry["hbm_floor_us"]))
        else:
            entry["limited_by"] = ("fixed cost of a launch (prologue, ramp-up, tail): %.1f us against an HBM floor of %.1f us"
                                   % (entry["spmm_us"], entry["hbm_floor_us"])
                                   if entry["roofline_frac"] < 0.45 else "decode work per tile in shared memory")
        return entry

    def verify(some_layers, mode, seed):
        """Runs two steps and checks sampled rows of every layer's result on every rank against the fp64 oracle."""
        for i in range(2):
            for L in some_layers:
                run_layer(L, i, mode, i)
        torch.cuda.synchronize()
        rng = np.random.default_rng(seed + rank)
        checks = []
        for L in some_layers:
            rows_local = sample_rows(sp, L, rng)
            C_bits = L.result.cpu().numpy().view(np.uint16)[rows_local]
            checks.append(verify_layer(sp, L, C_bits, rows_local + L.row0, L.name))
        all_ok = all(c["ok"] for c in checks) and sp.device_status() == 0
        return reduce_sum([1.0 if all_ok else 0.0])[0] == world, checks

    max_copies = max(len(L.words) for L in layers)
    stream = torch.cuda.Stream()
    record = {}
    with torch.cuda.stream(stream):
        # ---- every mode once, checked: a reduction whose bounded waits run out (2 s each) is dropped instead of being
        # timed launch after launch, and the main mode becomes the first one left
        dropped = []
        for mode in list(modes):
            for L in layers:
                run_layer(L, 0, mode, 0)
            torch.cuda.synchronize()
            failed = sp.device_status(reset=True) != 0 or sp.spmm_api.LIB.spmm_b200_allreduce_status(1) != 0
            if reduce_sum([1.0 if failed else 0.0])[0] > 0:
                modes.remove(mode)
                dropped.append(mode)
        if dropped:
            record["dropped_modes"] = dropped
        if not modes or (world > 1 and modes[0] == "none"):
            raise RuntimeError("no form of the sum over ranks passed its check: %r" % dropped)
        main_mode = modes[0]
        # ---- warm-up, un-captured, through every mode
        for mode in modes:
            for i in range(warmup):
                for L in layers:
                    run_layer(L, i, mode, i)
        barrier()
        # ---- what the timed loop computes is checked before it is timed
        verified, checks = verify(layers, main_mode, 1234)

        # ---- one CUDA graph per weight copy and mode: a step = the four layers (+ sums over ranks)
        graphs = {mode: [graph_of(torch, stream, lambda c=c, mode=mode: [run_layer(L, c, mode, c) for L in layers])
                         for c in range(max_copies)] for mode in modes}
        for mode in modes:
            for g in graphs[mode]:
                g.replay()
        barrier()

        def time_block(mode, steps):
            """Device time of exactly `steps` steps, bracketed by a barrier and a synchronise on both sides."""
            gs = graphs[mode]
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(steps):
                gs[i % len(gs)].replay()
            e1.record(stream)
            barrier()
            return e0.elapsed_time(e1)

        # ---- the timed region: repeats of a block of K steps until at least half a second has been timed
        probe = reduce_max([time_block(main_mode, args.steps)])[0]
        repeats = int(min(400, max(5, np.ceil(500.0 / max(probe, 1e-3)))))
        sampler = ClockSampler(local)
        sampler.start()
        time.sleep(0.02)
        t0 = time.time()
        sampler.window = (t0, None)
        blocks = [time_block(main_mode, args.steps) for _ in range(repeats)]
        t1 = time.time()
        sampler.window = (t0, t1)
        sampler.stop()
        blocks = reduce_max(blocks)  # per repeat, the slowest rank
        ms_per_step = float(np.median(blocks)) / args.steps
        record["ms_per_step_min_max"] = [round(min(blocks) / args.steps, 5), round(max(blocks) / args.steps, 5)]
        record["repeats"] = repeats
        other_modes = {}
        for mode in modes[1:]:
            ms = [time_block(mode, args.steps) for _ in range(5)]
            other_modes[mode] = float(np.median(reduce_max(ms))) / args.steps

        # ---- per layer: a graph of back-to-back launches of that layer alone, rotating through its copies
        per_layer = {L.name: layer_record(stream, L, True) for L in layers}

        # ---- end to end: activations from pinned host memory, results back to the host, every step
        if world == 1:
            items = [sp.host_io_items([dict(Compressed_A=L.words[c % len(L.words)], TileOffsets=L.offsets, B_host=L.B_host,
                                             C_host=L.C_host, B_dev=L.B, C_dev=L.C, M=L.M, N=N, K=L.K,
                                             Reduction_Workspace=L.ws, Split_K=L.split_k) for L in layers])
                     for c in range(max_copies)]

            def step_e2e(i):
                rc = sp.SpMM_SplitK_API_host_io_batch(stream, items[i % max_copies])
                if rc != 0:
                    raise RuntimeError("spmm_b200_spmm_splitk_host_io_batch failed with cudaError %d" % rc)
        else:
            def step_e2e(i):
                for L in layers:
                    L.B.copy_(L.B_host, non_blocking=True)
                    run_layer(L, i, main_mode, i)
                    L.C_host.copy_(L.result, non_blocking=True)

        for i in range(3):
            step_e2e(i)
        e2e_blocks = []
        for _ in range(5):
            barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record(stream)
            for i in range(args.steps):
                step_e2e(i)
            f1.record(stream)
            barrier()
            e2e_blocks.append(f0.elapsed_time(f1))
        ms_e2e = float(np.median(reduce_max(e2e_blocks))) / args.steps
        e2e_ok = all(bool(np.array_equal(L.C_host.numpy(), L.result.cpu().numpy())) for L in layers)

        extras = {}
        if not args.no_extras:
            # OPT-175B layer shapes sharded over the ranks: QKV and FFN1 by rows, FFN2 by K with the sum over ranks
            big = build(LAYERS_175B, 0x50, False)
            if peer_ok:
                add_peer_reducers(big)
            for mode in modes:
                for L in big:
                    run_layer(L, 0, mode, 0)
                    run_layer(L, 1, mode, 1)
            big_ok, big_checks = verify(big, main_mode, 99)
            extras["config5"] = {L.name: layer_record(stream, L, False) for L in big}
            extras["config5"]["verified"] = bool(big_ok)
            extras["config5"]["verification"] = big_checks
            verified = verified and big_ok
            del big
            torch.cuda.empty_cache()
            if world == 1:
                extras["prefill"] = prefill_point(sp, torch, dev, 12288, 12288, 1024, 0.8)

    status = sp.device_status()
    if status != 0:
        raise RuntimeError("device status %d: a bounded wait inside the kernel gave up" % status)
    if world > 1 and peer_ok and sp.spmm_api.LIB.spmm_b200_allreduce_status(0) != 0:
        raise RuntimeError("a wait inside the peer-memory reduction ran out")
    weight_bytes, algo_bytes = reduce_sum([sum(L.weight_bytes for L in layers), sum(L.algo_bytes for L in layers)])
    if rank != 0:
        leave(0)
    value = weight_bytes / (ms_per_step * 1e-3) / 1e9
    achieved = algo_bytes / world / (ms_per_step * 1e-3) / 1e9  # per GPU: the roofline is a per-GPU figure
    launches_per_step = len(layers) + (sum(1 for L in layers if L.split == "cols") if main_mode in ("peer", "peera", "peer2") else 0)
    reduce_note = {"none": "no collective (one GPU)", "fused": "fp32 partials summed inside the SpMM kernel, plain NVLink peer loads",
                   "peer": "fp32 partials summed by the library's reduction kernel, plain NVLink peer loads",
                   "peera": "fp32 partials flagged to the peers by the SpMM's last block and summed by the library's reduction "
                            "kernel, plain NVLink peer loads",
                   "peer2": "fp32 partials summed by the library's two-phase reduction kernel (each rank sums its share of the "
                            "rows out of peer memory and stores the result to all ranks over NVLink)",
                   "nccl": "NCCL all-reduce of fp16 results"}[main_mode]
    line = {
        "metric": METRIC,
        "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": [[n, m, k] for n, m, k, _, _ in LAYERS], "n_tokens": N,
                   "sparsity": SPARSITY, "split_k": [s for *_, s in LAYERS],
                   "parallelism": "one GPU" if world == 1 else
                   "tensor-parallel x%d: qkv, ffn1 by rows (no collective); out_proj, ffn2 by K + sum over ranks (%s)"
                   % (world, reduce_note),
                   "l2_policy": "weights rotate through copies: %.0f MB per GPU between two uses of the same bytes"
                                % (sum(L.weight_bytes * len(L.words) for L in layers) / 1e6),
                   "weights_constant": os.environ.get("SPMM_WEIGHTS_CONSTANT", "1") != "0",
                   "per_layer": per_layer, "weight_bytes_per_step": int(weight_bytes)},
        "verified": bool(verified), "verification": checks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4),
                     "traffic": int(algo_bytes / world * DRAM_TRAFFIC_OVER_ALGORITHMIC),
                     "traffic_note": "bytes per step per GPU (4 launches): ncu dram read+write of one launch / its "
                                     "algorithmic bytes = 1.009 (FFN1: 275.9 MB against 273.5 MB), applied to the step",
                     "peak_source": peak_kind, "kernel": "spmm_decode_kernel<16>",
                     "algorithmic_bytes_per_step_per_gpu": int(algo_bytes / world)},
        "e2e": {"value": round(weight_bytes / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
                "h2d_bytes_per_step": int(sum(2 * L.K * N for L in layers)),
                "d2h_bytes_per_step": int(sum(2 * L.M * N for L in layers)),
                "results_match_device_call": bool(e2e_ok),
                "call": "spmm_b200_spmm_splitk_host_io_batch (copies overlap the products)" if world == 1 else
                        "per layer: copy B from pinned memory, SpMM (+ sum over ranks), copy C to pinned memory"},
        "gpu_launches": args.steps * launches_per_step,
        "clocks": sampler.summary(t0, t1),
    }
    line.update(record)
    if world > 1:
        line["step_us_by_reduction"] = {main_mode: round(ms_per_step * 1e3, 2),
                                        **{m: round(v * 1e3, 2) for m, v in other_modes.items()}}
        line["comm_nranks_seen"] = world
    step_cublas = sum(e.get("cublas_dense_us", 0.0) for e in per_layer.values())
    if step_cublas:
        step_spmm = sum(e["spmm_us"] for e in per_layer.values())
        line["vs_cublas"] = {"cublas_dense_us_per_step": round(step_cublas, 2), "spmm_us_per_step": round(step_spmm, 2),
                             "speedup": round(step_cublas / step_spmm, 3),
                             "note": "cuBLAS dense fp16 (fp32 accumulate) on this GPU's pruned shard, same rotation through L2"}
    line.update(extras)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    if not verified:
        line["error"] = "verification against the fp64 oracle failed"
    print(json.dumps(line), flush=True)
    leave(0 if verified else 1)


def prefill_point(sp, torch, dev, M, K, N, p):
    """One prefill-size point: dense-equivalent TFLOP/s = 2*M*N*K / t against the measured dense tensor peak."""
    tensor_peak = measured_peak("bf16_tflops", 1590.0)[0]
    A = sp.synth_fp16((M, K), 0xA300 + int(p * 100), 0.02, p)
    words, offsets, _ = sp.InitSparseMatrixA_API(A, M, 64, K)
    wd = torch.from_numpy(words.view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(sp.synth_fp16((K, N), 0xB300, 1.0).view(np.int16)).to(dev)
    Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
    split_k = sp.suggest_split_k(M, K)  # sizes the workspace: room for the partial tiles of a partition over all SMs
    ws = torch.zeros(sp.workspace_bytes(M, N, split_k) // 2, dtype=torch.int16, device=dev)
    assert sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, N, K, ws, split_k) == 0
    us = time_graph(torch, lambda: sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, N, K, ws, split_k))
    assert sp.device_status() == 0
    return {"M": M, "K": K, "N": N, "sparsity": p, "spmm_us": round(us, 1),
            "dense_equiv_tflops": round(2.0 * M * N * K / us / 1e6, 1),
            "frac_of_tensor_peak": round(2.0 * M * N * K / us / 1e6 / tensor_peak, 4), "tensor_peak_tflops": tensor_peak}


# --------------------------------------------------------------------------------------------- CPU arms
# Nothing below imports the product package: inputs come from the oracle's own generator, the encoder is the
# reference's (oracle/_ref) or its C restatement, the product is the oracle's decode + fp32-accumulate loop.
def cpu_layers(fraction, threads):
    """The four layers of the step, the first `fraction` of each layer's rows of tiles:
    ([(words, offsets, B, rows, K)], seconds the slowest encoder call took)."""
    import oracle
    results = [None] * len(LAYERS)

    def make(li):
        name, M, K, _, _ = LAYERS[li]
        rows = max(128, int(M * fraction) // 128 * 128)
        A = oracle.synth_fp16_block(rows, K, K, 0, 0, SEED_A + li, 0.02, SPARSITY, threads=max(1, threads // len(LAYERS)))
        B = oracle.synth_fp16_block(K, N_TOKENS, N_TOKENS, 0, 0, SEED_B + li, 1.0, threads=1)
        t0 = time.time()
        words, offsets = (oracle.ref_encode(A) if oracle.have_ref() else oracle.encode(A))
        results[li] = ((words, offsets, B, rows, K), time.time() - t0)

    pool = [threading.Thread(target=make, args=(li,)) for li in range(len(LAYERS))]
    for th in pool:
        th.start()
    for th in pool:
        th.join()
    return [r for r, _ in results], max(s for _, s in results)


def cpu_spmm_threads(words, offsets, B, M, K, threads):
    """The oracle's decode + fp32-accumulate product over row blocks of tiles, one block per host thread."""
    import oracle
    tiles_m, tiles_k = M // 128, K // 64
    threads = max(1, min(threads, tiles_m))
    out = [None] * threads

    def work(t):
        r0, r1 = tiles_m * t // threads, tiles_m * (t + 1) // threads
        offs = offsets[r0 * tiles_k:r1 * tiles_k + 1].astype(np.int64)
        sub_offsets = np.concatenate([offs - offs[0], [offs[-1] - offs[0]]]).astype(np.int32)
        sub_words = words[offs[0] * 4:offs[-1] * 4]
        out[t] = oracle.spmm_from_csl(sub_words, sub_offsets, B, (r1 - r0) * 128, K)

    pool = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
    for th in pool:
        th.start()
    for th in pool:
        th.join()
    return np.concatenate(out, axis=0)


def cpu_step(layers, threads):
    for words, offsets, B, rows, K in layers:
        cpu_spmm_threads(words, offsets, B, rows, K, threads)


def cpu_baseline():
    """The CPU path on a bounded sample, timed beside the GPU number: the reference's own InitSparseMatrixA_API
    (single-threaded as shipped, one thread per layer here) and the oracle's decode + fp32 host product on all host
    threads, over the first eighth of the rows of every layer of the step."""
    import oracle
    cores = os.cpu_count() or 1
    layers, enc_s = cpu_layers(0.125, cores)
    cpu_step(layers, cores)
    t0 = time.time()
    reps = 3
    for _ in range(reps):
        cpu_step(layers, cores)
    dt = (time.time() - t0) / reps
    wbytes = sum(4 * w.size + 4 * o.size for w, o, *_ in layers)
    return {"value": round(wbytes / dt / 1e9, 4), "unit": "GB/s", "cores": cores,
            "kind": "reference" if oracle.have_ref() else "port",
            "sample": "first 1/8 of the rows of each of the four layers (N=16, p=0.8): encoder %s, slowest layer %.2f s "
                      "on 1 core; decode + fp32 host product (oracle C code) %.3f s per pass on %d threads"
                      % ("InitSparseMatrixA_API of the compiled reference (oracle/_ref)" if oracle.have_ref()
                         else "oracle restatement of InitSparseMatrixA_API", enc_s, dt, cores),
            "encode_s": round(enc_s, 3), "spmm_s": round(dt, 4)}


def run_reference(args):
    """The reference's CPU implementation of the path on all host cores: its InitSparseMatrixA_API encoding (outside
    the timed loop, as the GPU arm's) and per step the decode of the tiled-CSL words + fp32-accumulate host product of
    all four layers of the block (a bounded share of every layer's rows if a full step would take too long)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle
    cores = os.cpu_count() or 1
    # probe on 1/16 of the rows, then size the sample so that the whole run stays within about two minutes
    probe_layers, _ = cpu_layers(1.0 / 16, cores)
    cpu_step(probe_layers, cores)
    t0 = time.time()
    cpu_step(probe_layers, cores)
    probe = (time.time() - t0) * 16
    budget = 100.0 / max(args.steps + args.warmup, 1)
    fraction = 1.0 if probe <= budget else max(1.0 / 16, budget / probe)
    layers = probe_layers if fraction <= 1.0 / 16 else cpu_layers(fraction, cores)[0]
    for _ in range(args.warmup):
        cpu_step(layers, cores)
    t0 = time.time()
    for _ in range(args.steps):
        cpu_step(layers, cores)
    dt = (time.time() - t0) / args.steps
    wbytes = sum(4 * w.size + 4 * o.size for w, o, *_ in layers)
    value = round(wbytes / dt / 1e9, 4)
    sample = ("all four layers of the block, %s of every layer's rows per step, N=16, p=0.8, %d host threads; encoder: %s"
              % ("all" if fraction >= 1.0 else "the first %.3f" % fraction, cores,
                 "reference (oracle/_ref)" if oracle.have_ref() else "oracle restatement"))
    line = {
        "impl": "reference", "metric": METRIC,
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": [[n, m, k] for n, m, k, _, _ in LAYERS], "n_tokens": N_TOKENS,
                   "sparsity": SPARSITY, "rows_fraction_per_step": round(fraction, 4)},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores,
                         "kind": "reference" if oracle.have_ref() else "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- sweeps
def run_sweep(args):
    """Decode-size sweep over the OPT-66B layer shapes, N and sparsity (one JSON line per point),
    with cuBLAS dense fp16 on the pruned matrix as the comparator.  Device-timed with CUDA graphs;
    every shape's weights exceed or rotate through L2 (copies chosen so that the set is >= 256 MB)."""
    import torch

    import graphneuralnetproj_b200 as sp
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    peak, _ = measured_peak("hbm_gbs", HBM_PEAK_FALLBACK_GBS)
    sp.set_weights_constant(True)
    # "cfg1" = the reference's single-SpMM case (M = K = 7168 with its Split_K hint 5), beside the OPT-66B layers
    shapes = [(n, m, k, 8) for n, m, k, _, _ in LAYERS if n in args.sweep_layers.split(",")]
    if "cfg1" in args.sweep_layers.split(","):
        shapes.append(("cfg1", 7168, 7168, 5))
    n_list = [int(x) for x in args.sweep_n.split(",")]
    p_list = [float(x) for x in args.sweep_p.split(",")]
    for name, M, K, sk in shapes:
        for p in p_list:
            A = sp.synth_fp16((M, K), 0xA100 + int(p * 100), 0.02, p)
            words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, 16, K)
            wbytes = 4 * words.size + 4 * n_offsets
            copies = max(1, int(np.ceil(256e6 / wbytes)))
            wds = [torch.from_numpy(words.view(np.int32)).to(dev)
                   for _ in range(copies)]
            od = torch.from_numpy(offsets).to(dev)
            dense = [torch.from_numpy(A.view(np.float16)).to(dev) for _ in range(max(1, min(copies, 2)))]
            del A, words
            for N in n_list:
                Bd = torch.from_numpy(sp.synth_fp16((K, N), 0xB100, 1.0).view(np.int16)).to(dev)
                Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
                ws = torch.zeros(sp.workspace_bytes(M, N, sk) // 2, dtype=torch.int16, device=dev)

                def ours(i):
                    rc = sp.SpMM_SplitK_API(None, None, wds[i % copies], None, None, od, Bd, Cd, M, N, K, ws, sk)
                    assert rc == 0, rc

                def cublas(i):
                    torch.matmul(dense[i % len(dense)], Bd.view(torch.float16))

                times = {}
                for label, fn in (("spmm", ours), ("cublas_dense", cublas)):
                    stream = torch.cuda.Stream()
                    with torch.cuda.stream(stream):
                        for i in range(4):
                            fn(i)
                        torch.cuda.synchronize()
                        g = torch.cuda.CUDAGraph()
                        reps = 12
                        with torch.cuda.graph(g, stream=stream):
                            for i in range(reps):
                                fn(i)
                        g.replay()
                        torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        for _ in range(5):
                            g.replay()
                        e1.record(stream)
                        torch.cuda.synchronize()
                        times[label] = e0.elapsed_time(e1) * 1000.0 / (5 * reps)
                algo = algorithmic_bytes(wbytes // 4 - n_offsets, n_offsets, M, K, N)
                print(json.dumps({"layer": name, "M": M, "K": K, "N": N, "sparsity": p,
                                  "spmm_us": round(times["spmm"], 2), "cublas_dense_us": round(times["cublas_dense"], 2),
                                  "speedup_vs_cublas": round(times["cublas_dense"] / times["spmm"], 3),
                                  "weight_gbs": round(wbytes / times["spmm"] / 1e3, 1),
                                  "roofline_frac": round(algo / times["spmm"] / 1e3 / peak, 4)}), flush=True)
            del wds, dense
            torch.cuda.empty_cache()
    assert sp.device_status() == 0


def time_graph(torch, fn, launches=10, replays=3):
    """Microseconds per call of `fn`, `launches` calls captured in one CUDA graph and replayed (no host time
    between the kernels), CUDA events on the replaying stream, after warm-up calls and one warm-up replay."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(launches):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(replays):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / (launches * replays)


def run_prefill(args):
    """Prefill-size points (N >= 256): dense-equivalent TFLOP/s = 2*M*N*K / t against the measured
    dense tensor peak, with cuBLAS dense fp16 beside it.  One JSON line per point."""
    import torch

    import graphneuralnetproj_b200 as sp
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    tensor_peak = measured_peak("bf16_tflops", 1590.0)[0]
    shapes = [(12288, 12288), (49152, 12288)] if not args.small else [(12288, 12288)]
    for M, K in shapes:
        for p in [float(x) for x in args.prefill_p.split(",")]:
            A = sp.synth_fp16((M, K), 0xA300 + int(p * 100), 0.02, p)
            words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, 64, K)
            wd = torch.from_numpy(words.view(np.int32)).to(dev)
            od = torch.from_numpy(offsets).to(dev)
            Ad = torch.from_numpy(A.view(np.float16)).to(dev)
            del A, words
            for N in [int(x) for x in args.prefill_n.split(",")]:
                Bd = torch.from_numpy(sp.synth_fp16((K, N), 0xB300, 1.0).view(np.int16)).to(dev)
                Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
                # the workspace of the reference's contract for the Split_K the library suggests: room for the fp32
                # partial tiles of a partition of the rows over all SMs (with less, rows cannot be split and SMs idle)
                split_k = sp.suggest_split_k(M, K)
                ws = torch.zeros(sp.workspace_bytes(M, N, split_k) // 2, dtype=torch.int16, device=dev)
                Bh = Bd.view(torch.float16)
                dense_out = torch.empty((M, N), dtype=torch.float16, device=dev)
                calls = {"spmm": lambda: sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, N, K, ws, split_k),
                         "cublas_dense": lambda: torch.matmul(Ad, Bh, out=dense_out)}
                times = {}
                for label in ("spmm", "single_block", "cublas_dense"):
                    fn = calls["spmm" if label == "single_block" else label]
                    sp.set_pair_kernel(label != "single_block")
                    times[label] = time_graph(torch, fn)
                sp.set_pair_kernel(True)
                flops = 2.0 * M * N * K
                print(json.dumps({"M": M, "K": K, "N": N, "sparsity": p, "spmm_us": round(times["spmm"], 1),
                                  "single_block_kernel_us": round(times["single_block"], 1),
                                  "cublas_dense_us": round(times["cublas_dense"], 1),
                                  "dense_equiv_tflops": round(flops / times["spmm"] / 1e6, 1),
                                  "frac_of_tensor_peak": round(flops / times["spmm"] / 1e6 / tensor_peak, 4),
                                  "tensor_peak_tflops": tensor_peak}), flush=True)
            del wd, Ad
            torch.cuda.empty_cache()
    assert sp.device_status() == 0


class quiet_stdout:
    """Silences what C code prints to stdout (the reference's encoders report statistics with printf)."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        self.null = os.open(os.devnull, os.O_WRONLY)
        os.dup2(self.null, 1)

    def __exit__(self, *exc):
        import ctypes
        ctypes.CDLL(None).fflush(None)
        os.dup2(self.saved, 1)
        os.close(self.saved)
        os.close(self.null)


def reference_sparse_tensor_core_kernel(sp, torch, dev, A1_bits, B_bits, split_k, reps=20):
    """The reference's own GPU kernel for the 2:4 half (csrc/SpMM_Kernel.cuh:293-735: mma.sp.m16n8k16 with fp16
    accumulators), compiled unchanged for sm_100a into oracle/_ref, fed with the A1 vectors, index words and
    metadata of InitSparseMatrixA1_Vec_Sparse_Load / inspect_metadata (this library's, bit-identical to the
    reference's), followed by the sum of its Split_K fp16 slabs (the reference leaves that to the harness's Reduction
    kernel, kernel_benchmark/FSP_Batch8.h:209-229; a torch reduction stands in for it).  Returns
    (microseconds per product or None, note, result as a float32 tensor or None)."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libSpMM_API_ref.so")
    if not os.path.exists(path):
        return None, "unavailable: oracle/_ref/libSpMM_API_ref.so was not built", None
    try:
        ref = ctypes.CDLL(path)
        spmm = getattr(ref, "_Z15SpMM_SplitK_APIP11CUstream_stPK6__halfPK5uint4PKmPKiSA_S3_PS1_iiiSB_i")
    except (OSError, AttributeError) as exc:
        return None, "unavailable: %s" % exc, None
    spmm.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_int]
    spmm.restype = ctypes.c_int
    M, K = A1_bits.shape
    N = B_bits.shape[1]
    if M % 256 or K % 64 or N not in (8, 16, 32, 64):
        return None, "unavailable: the reference kernel needs M %% 256 == 0, K %% 64 == 0, N in {8,16,32,64}", None
    lib = sp.spmm_api.LIB
    u16p, u64p, i32p = ctypes.POINTER(ctypes.c_uint16), ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_int)
    enc = getattr(lib, "_Z34InitSparseMatrixA1_Vec_Sparse_LoadP6__halfiiPS0_PPmPPi")
    enc.argtypes = [u16p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(u16p), ctypes.POINTER(u64p), ctypes.POINTER(i32p)]
    enc.restype = ctypes.c_int
    meta_fn = getattr(lib, "_Z16inspect_metadataP6__halfPiii")
    meta_fn.argtypes = [u16p, i32p, ctypes.c_int, ctypes.c_int]
    meta_fn.restype = None
    A1 = np.ascontiguousarray(A1_bits, dtype=np.uint16)
    vp, ip, op = u16p(), u64p(), i32p()
    meta = np.zeros((M // 16) * (K // 16) * 8, np.int32)
    with quiet_stdout():
        n_off = enc(A1.ctypes.data_as(u16p), M, K, ctypes.byref(vp), ctypes.byref(ip), ctypes.byref(op))
        meta_fn(A1.ctypes.data_as(u16p), meta.ctypes.data_as(i32p), M, K)
    offsets = np.ctypeslib.as_array(op, shape=(n_off,)).copy()
    vectors = int(offsets[-1])
    values = np.ctypeslib.as_array(vp, shape=(vectors * 8,)).copy()
    index = np.ctypeslib.as_array(ip, shape=(vectors,)).copy()
    for ptr in (vp, ip, op):
        lib.spmm_b200_free(ctypes.cast(ptr, ctypes.c_void_p))
    if np.any(np.diff(offsets[:-1]) <= 0):
        return None, "unavailable: an empty 256 x 64 tile (the reference encoder mis-sizes those, csrc/SpMM_API.cu:1202)", None
    vd = torch.from_numpy(values.view(np.int16)).to(dev)
    xd = torch.from_numpy(index.view(np.int64)).to(dev)
    md = torch.from_numpy(meta).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(np.ascontiguousarray(B_bits).view(np.int16)).to(dev)
    ws = torch.zeros((split_k, M, N), dtype=torch.float16, device=dev)
    out = torch.empty((M, N), dtype=torch.float16, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def once():
        rc = spmm(stream, None, vd.data_ptr(), xd.data_ptr(), md.data_ptr(), od.data_ptr(), Bd.data_ptr(), None, M, N, K,
                  ws.data_ptr(), split_k)
        torch.sum(ws, dim=0, dtype=torch.float16, out=out)
        return rc

    rc = once()
    torch.cuda.synchronize()
    if rc != 0:
        return None, "unavailable: the reference launch returned cudaError %d" % rc, None
    for _ in range(3):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        once()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / reps, "Split_K %d, fp16 accumulate, torch sum of the slabs included" % split_k, out.float()



def prune_2_of_4(A_bits, keep_prob, seed):
    """2:4 magnitude pruning along K, then each survivor is zeroed with probability 1 - keep_prob."""
    groups = np.abs(A_bits.view(np.float16).astype(np.float32)).reshape(-1, 4)
    order = np.argsort(-groups, axis=1, kind="stable")
    mask = np.zeros(groups.shape, dtype=bool)
    np.put_along_axis(mask, order[:, :2], True, axis=1)
    mask &= np.random.default_rng(seed).random(mask.shape) < keep_prob
    out = A_bits.reshape(-1, 4).copy()
    out[~mask] = 0
    return out.reshape(A_bits.shape)


def run_hetero(args):
    """Heterogeneous decomposition (M = K = 12288, N = 32): the structured half on tcgen05.mma.sp plus the
    tiled-CSL residual, against the same matrix encoded wholly as tiled-CSL and against cuBLAS dense.
    Two inputs: 2:4 magnitude pruning with half of the survivors zeroed (75 % sparse, empty residual) and
    i.i.d. 80 % sparsity (a few per cent of the nonzeros land in the residual).  One JSON line each."""
    import torch

    import graphneuralnetproj_b200 as sp
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    peak, _ = measured_peak("hbm_gbs", HBM_PEAK_FALLBACK_GBS)
    sp.set_weights_constant(True)
    M = K = args.hetero_size
    N = args.hetero_n

    def timed(fn, copies):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(2 * copies):
                    fn(i)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1000.0 / (reps * 2 * copies)

    B_bits = sp.synth_fp16((K, N), 0xB400, 1.0)
    Bd = torch.from_numpy(B_bits.view(np.int16)).to(dev)
    Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
    ws = torch.zeros(sp.workspace_bytes(M, N, 8) // 2, dtype=torch.int16, device=dev)
    copies = 2  # rotate over two copies of the weights: more than L2 holds

    # The reference's own kernel for the structured half, first on a 512 x 256 case checked against an fp64
    # product; the full-size case runs only if that one came out right.
    small_A = prune_2_of_4(sp.synth_fp16((512, 256), 0xA410, 0.02, 0.0), 0.5, 5)
    small_B = sp.synth_fp16((256, N), 0xB410, 1.0)
    ref_us, ref_note, ref_C = reference_sparse_tensor_core_kernel(sp, torch, dev, small_A, small_B, 2, reps=3)
    reference_kernel_ok = False
    if ref_C is not None:
        want = torch.from_numpy(small_A.view(np.float16)).to(dev).double() @ torch.from_numpy(small_B.view(np.float16)).to(dev).double()
        err = float((ref_C.double() - want).abs().max() / want.abs().max())
        reference_kernel_ok = err <= 2e-2  # fp16 accumulation: looser than the product's own gate
        ref_note = ref_note if reference_kernel_ok else "unavailable: wrong result on the 512 x 256 check (max err / max|C| = %.3g)" % err
    for label, make in (("2:4 pruned, half of the survivors zeroed (75 % sparse)",
                         lambda: prune_2_of_4(sp.synth_fp16((M, K), 0xA400, 0.02, 0.0), 0.5, 4)),
                        ("i.i.d. 80 % sparse", lambda: sp.synth_fp16((M, K), 0xA401, 0.02, 0.8))):
        A = make()
        A1, A2 = sp.decompose(A)
        residual_nnz = int(np.count_nonzero(A2 & 0x7FFF))
        values, meta, _ = sp.InitSparseMatrixA1_tcgen05(A1, M, K)
        vds = [torch.from_numpy(values).to(dev) for _ in range(copies)]
        mds = [torch.from_numpy(meta.view(np.int32)).to(dev) for _ in range(copies)]
        a1_bytes = values.nbytes + meta.nbytes
        r_wds = r_od = None
        residual_bytes = 0
        if residual_nnz:
            rw, ro, rn = sp.InitSparseMatrixA_API(A2, M, N, K)
            r_wds = [torch.from_numpy(rw.view(np.int32)).to(dev) for _ in range(copies)]
            r_od = torch.from_numpy(ro).to(dev)
            residual_bytes = 4 * rw.size + 4 * rn
        words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, N, K)
        wds = [torch.from_numpy(words.view(np.int32)).to(dev) for _ in range(copies)]
        od = torch.from_numpy(offsets).to(dev)
        csl_bytes = 4 * words.size + 4 * n_offsets
        Ad = [torch.from_numpy(A.view(np.float16)).to(dev) for _ in range(copies)]
        Bh = Bd.view(torch.float16)

        def hetero(i):
            rc = sp.SpMM_SplitK_API(None, vds[i % copies], r_wds[i % copies] if r_wds else None, None, mds[i % copies],
                                    r_od, Bd, Cd, M, N, K, ws, 8)
            assert rc == 0, rc

        def csl(i):
            rc = sp.SpMM_SplitK_API(None, None, wds[i % copies], None, None, od, Bd, Cd, M, N, K, ws, 8)
            assert rc == 0, rc

        t_hetero = timed(hetero, copies)
        t_csl = timed(csl, copies)
        t_dense = timed(lambda i: torch.matmul(Ad[i % copies], Bh), copies)
        algo = a1_bytes + residual_bytes + 2 * K * N + 2 * M * N
        reference_kernel = {"reference_kernel": ref_note}
        if reference_kernel_ok and residual_nnz == 0:
            # the structured half alone, as the reference's harness times its A1 kernel (kernel_benchmark/spmm_test.cu:467-506)
            us, note, C_ref = reference_sparse_tensor_core_kernel(sp, torch, dev, A1, B_bits, 9)
            reference_kernel = {"reference_kernel": note}
            if us is not None:
                hetero(0)
                torch.cuda.synchronize()
                ours = Cd.view(torch.float16).float()
                reference_kernel.update({"reference_kernel_us": round(us, 2),
                                         "speedup_vs_reference_kernel": round(us / t_hetero, 3),
                                         "reference_kernel_max_diff_over_max_c": float("%.3g" % float(
                                             (C_ref - ours).abs().max() / ours.abs().max()))})
        elif reference_kernel_ok:
            reference_kernel = {"reference_kernel": "not run: this input has a residual, which the reference multiplies with "
                                                    "separate CUDA-core kernels that are not part of its library"}
        print(json.dumps({"input": label, "M": M, "K": K, "N": N, "residual_nnz": residual_nnz, **reference_kernel,
                          "hetero_us": round(t_hetero, 2), "tiled_csl_only_us": round(t_csl, 2),
                          "cublas_dense_us": round(t_dense, 2),
                          "a1_bytes": a1_bytes, "residual_bytes": residual_bytes, "tiled_csl_bytes": csl_bytes,
                          "hetero_weight_gbs": round((a1_bytes + residual_bytes) / t_hetero / 1e3, 1),
                          "hetero_roofline_frac": round(algo / t_hetero / 1e3 / peak, 4),
                          "tiled_csl_roofline_frac": round((csl_bytes + 2 * K * N + 2 * M * N) / t_csl / 1e3 / peak, 4),
                          "speedup_vs_cublas": round(t_dense / t_hetero, 3)}), flush=True)
        del vds, mds, wds, Ad, r_wds
        torch.cuda.empty_cache()
    assert sp.device_status() == 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the OPT-175B and prefill sub-records of the bench line")
    ap.add_argument("--sweep", action="store_true", help="decode-size sweep (layers x N x sparsity) instead of the bench line")
    ap.add_argument("--sweep-n", default="8,16,32,64")
    ap.add_argument("--sweep-p", default="0.7,0.8,0.9")
    ap.add_argument("--sweep-layers", default="qkv,out_proj,ffn1,ffn2")
    ap.add_argument("--prefill", action="store_true", help="prefill-size points (N >= 256) instead of the bench line")
    ap.add_argument("--prefill-n", default="256,512,1024,2048")
    ap.add_argument("--prefill-p", default="0.5,0.7,0.8")
    ap.add_argument("--small", action="store_true", help="with --prefill: only the 12288 x 12288 shape")
    ap.add_argument("--hetero", action="store_true", help="heterogeneous decomposition points (structured half on the sparse tensor core)")
    ap.add_argument("--hetero-size", type=int, default=12288)
    ap.add_argument("--hetero-n", type=int, default=32)
    args = ap.parse_args()
    if args.hetero:
        run_hetero(args)
    elif args.prefill:
        run_prefill(args)
    elif args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
