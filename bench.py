"""Benchmark of the sparse-weight SpMM hot path on B200.

A step is one pass over the four linear layers of an OPT-66B decoder block at decode size
(QKV 27648x9216, out-proj 9216x9216, FFN1 36864x9216, FFN2 9216x36864; N = 16 tokens, 80 %
i.i.d. sparsity, fp16 in, fp32 accumulate): four SpMM launches through the C boundary of
libSpMM_API.so.  Weights are seeded synthetic stand-ins for pruned OPT weights, encoded with
the library's InitSparseMatrixA_API and resident in HBM before the timed region.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Prints one JSON line (rank 0).  `value` is effective weight-HBM GB/s, (4*NNZ_pad +
4*NumOffsets) summed over the step and all ranks, divided by the device time (max over
ranks).  With N > 1 every rank runs the same per-GPU workload on its own row shard of an
N-times taller, column-parallel layer: no collective on the data path, weak scaling.
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

LAYERS = [  # name, M, K, Split_K (sizes the workspace: Split_K * M * N * 2 bytes)
    ("qkv", 27648, 9216, 4),
    ("out_proj", 9216, 9216, 8),
    ("ffn1", 36864, 9216, 4),
    ("ffn2", 9216, 36864, 8),
]
N_TOKENS = 16
SPARSITY = 0.8
WORKLOAD = "opt66b_decoder_block_4_spmm_n16_p0.8"
HBM_PEAK_FALLBACK_GBS = 6650.0
# dram__bytes_read + dram__bytes_write over algorithmic bytes, from the ncu capture summarised in
# profiles/spmm_decode_n16_ffn1_lsu_counters.md (FFN1 launch: 278.5 MB / 273.5 MB)
DRAM_TRAFFIC_OVER_ALGORITHMIC = 1.018


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_PEAK_FALLBACK_GBS, "fallback"


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
                self.samples.append((time.time(), mhz))
                if self.window and self.window[0] <= time.time():
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
        inside = [m for (t, m) in self.samples if t0 <= t <= t1] or [m for (_, m) in self.samples[-3:]]
        return {"sm_mhz": float(np.median(inside)) if inside else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(inside)}


def algorithmic_bytes(n_words, n_offsets, M, K, N):
    """Compulsory traffic of one SpMM: words + offsets + B + C."""
    return 4 * n_words + 4 * n_offsets + 2 * K * N + 2 * M * N


def make_layer(sp, name, M, K, seed):
    A = sp.synth_fp16((M, K), seed, 0.02, SPARSITY)
    words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, N_TOKENS, K)
    del A
    return words, offsets, n_offsets


def run_ours(args):
    import torch
    import torch.distributed as dist

    import graphneuralnetproj_b200 as sp

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- weights: encoded on the host, resident in HBM (rank r holds row shard r of each layer)
    layers = []
    weight_bytes = algo_bytes = 0
    for li, (name, M, K, sk) in enumerate(LAYERS):
        words, offsets, n_offsets = make_layer(sp, name, M, K, 0xA000 + 16 * rank + li)
        weight_bytes += 4 * words.size + 4 * n_offsets
        algo_bytes += algorithmic_bytes(words.size, n_offsets, M, K, N_TOKENS)
        B_host = torch.from_numpy(sp.synth_fp16((K, N_TOKENS), 0xB000 + li, 1.0).view(np.int16)).pin_memory()
        layers.append(dict(
            name=name, M=M, K=K, sk=sk,
            words=torch.from_numpy(np.concatenate([words, np.zeros(4, np.uint32)]).view(np.int32)).to(dev),
            offsets=torch.from_numpy(offsets).to(dev),
            B_host=B_host, B=B_host.to(dev),
            C=torch.zeros((M, N_TOKENS), dtype=torch.int16, device=dev),
            C_host=torch.zeros((M, N_TOKENS), dtype=torch.int16).pin_memory(),
            ws=torch.zeros(sp.workspace_bytes(M, N_TOKENS, sk) // 2, dtype=torch.int16, device=dev)))
        del words

    def launch(layer):
        rc = sp.SpMM_SplitK_API(None, None, layer["words"], None, None, layer["offsets"], layer["B"], layer["C"],
                                layer["M"], N_TOKENS, layer["K"], layer["ws"], layer["sk"])
        if rc != 0:
            raise RuntimeError("SpMM_SplitK_API failed with cudaError %d" % rc)

    def step():
        for layer in layers:
            launch(layer)

    def step_e2e():
        # the C boundary's host-buffer call: H2D copy of B, SpMM, D2H copy of C, per layer
        for layer in layers:
            rc = sp.SpMM_SplitK_API_host_io(stream, layer["words"], layer["offsets"], layer["B_host"], layer["C_host"],
                                            layer["B"], layer["C"], layer["M"], N_TOKENS, layer["K"], layer["ws"], layer["sk"])
            if rc != 0:
                raise RuntimeError("spmm_b200_spmm_splitk_host_io failed with cudaError %d" % rc)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        # One step captured as a CUDA graph so that launch latency of the host loop is not timed.
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        graph.replay()
        sampler = ClockSampler(local)
        sampler.start()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        sampler.window = (t0, None)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        t1 = time.time()
        sampler.stop()
        ms = e0.elapsed_time(e1)

        # per-layer device time: events around every launch of a few plain (un-captured) steps, so
        # each layer's weights have been evicted from L2 by the other layers in between
        reps, pairs = 10, []
        for _ in range(reps):
            for layer in layers:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                launch(layer)
                b.record(stream)
                pairs.append((layer["name"], a, b))
        torch.cuda.synchronize()
        per_layer = {}
        for name, a, b in pairs:
            per_layer[name] = per_layer.get(name, 0.0) + a.elapsed_time(b) * 1000.0 / reps

        # end to end: activations from pinned host memory, results back to the host, every launch
        for _ in range(3):
            step_e2e()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(args.steps):
            step_e2e()
        f1.record(stream)
        barrier()
        ms_e2e = f0.elapsed_time(f1)
    status = sp.device_status()
    if status != 0:
        raise RuntimeError("device status %d: a bounded wait inside the kernel gave up" % status)

    times = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = times.tolist()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_per_step = ms / args.steps
    value = world * weight_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * weight_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    peak, peak_kind = measured_hbm_peak()
    achieved = algo_bytes / (ms_per_step * 1e-3) / 1e9  # this rank's kernel launches
    line = {
        "metric": "effective weight-HBM GB/s, SpMM (OPT-66B shapes, N=16, 80% sparse)",
        "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": [[n, m, k] for n, m, k, _ in LAYERS], "n_tokens": N_TOKENS,
                   "sparsity": SPARSITY, "split_k": [s for *_, s in LAYERS], "parallelism": "column-parallel by M x%d" % world,
                   "l2_policy": "inputs larger than L2: %.0f MB of weights per step" % (weight_bytes / 1e6),
                   "spmm_us_per_layer": {k: round(v, 2) for k, v in per_layer.items()},
                   "weight_bytes_per_step_per_gpu": weight_bytes},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4),
                     "traffic": int(algo_bytes * DRAM_TRAFFIC_OVER_ALGORITHMIC),
                     "traffic_note": "bytes per step (4 launches): ncu dram read+write of one launch / its algorithmic "
                                     "bytes = 1.018 (FFN1: 278.5 MB against 273.5 MB), applied to the step", "peak_source": peak_kind,
                     "kernel": "spmm_decode_kernel<16>", "algorithmic_bytes_per_step": algo_bytes},
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s",
                "h2d_bytes_per_step": sum(2 * L["K"] * N_TOKENS for L in layers),
                "d2h_bytes_per_step": sum(2 * L["M"] * N_TOKENS for L in layers)},
        "gpu_launches": args.steps * len(layers),
        "clocks": sampler.summary(t0, t1),
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_sample_problem(sp, rows, K, seed):
    A = sp.synth_fp16((rows, K), seed, 0.02, SPARSITY)
    B = sp.synth_fp16((K, N_TOKENS), seed + 1, 1.0)
    return A, B


def cpu_spmm_threads(oracle, words, offsets, B, M, K, threads):
    """The oracle's decode + fp32-accumulate product over row blocks of tiles, one block per host thread."""
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


def cpu_baseline():
    """Reference CPU path on a bounded sample: the reference's own InitSparseMatrixA_API (one
    core; it is single-threaded) and the oracle's decode + fp32 host product (one core)."""
    import graphneuralnetproj_b200 as sp
    import oracle
    M, K = 9216, 9216  # the out-proj layer of the step
    A, B = cpu_sample_problem(sp, M, K, 0xC000)
    t0 = time.time()
    if oracle.have_ref():
        words, offsets = oracle.ref_encode(A)
        encoder = "reference InitSparseMatrixA_API (oracle/_ref)"
    else:
        words, offsets = oracle.encode(A)
        encoder = "oracle port of InitSparseMatrixA_API"
    t_enc = time.time() - t0
    t0 = time.time()
    oracle.spmm_from_csl(words, offsets, B, M, K)
    t_spmm = time.time() - t0
    wbytes = 4 * words.size + 4 * offsets.size
    return {"value": round(wbytes / t_spmm / 1e9, 4), "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": "out-proj layer 9216x9216, N=16, p=0.8: %s %.2f s on 1 core; oracle decode + fp32 host "
                      "product %.2f s on 1 core (value = weight bytes / product time)" % (encoder, t_enc, t_spmm),
            "encode_s": round(t_enc, 3), "spmm_s": round(t_spmm, 3)}


def run_reference(args):
    """The reference's CPU implementation of the path on all host cores: decode of the tiled-CSL
    words + fp32-accumulate host product, a bounded row sample of the out-proj layer per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import graphneuralnetproj_b200 as sp
    import oracle
    cores = os.cpu_count() or 1
    K = 9216
    rows = 9216
    A, B = cpu_sample_problem(sp, rows, K, 0xC000)
    words, offsets = (oracle.ref_encode(A) if oracle.have_ref() else oracle.encode(A))
    t0 = time.time()
    cpu_spmm_threads(oracle, words, offsets, B, rows, K, cores)
    probe = time.time() - t0
    # bound the whole run to about two minutes
    budget = 120.0 / max(args.steps + args.warmup, 1)
    if probe > budget:
        rows = max(128, int(rows * budget / probe) // 128 * 128)
        tiles_k = K // 64
        offs = offsets[:rows // 128 * tiles_k + 1]
        offsets = np.concatenate([offs, offs[-1:]]).astype(np.int32)
        words = words[:int(offs[-1]) * 4]
    for _ in range(args.warmup):
        cpu_spmm_threads(oracle, words, offsets, B, rows, K, cores)
    t0 = time.time()
    for _ in range(args.steps):
        cpu_spmm_threads(oracle, words, offsets, B, rows, K, cores)
    dt = (time.time() - t0) / args.steps
    wbytes = 4 * words.size + 4 * offsets.size
    value = round(wbytes / dt / 1e9, 4)
    sample = "%d x %d rows of the out-proj layer per step, N=16, p=0.8, %d host threads" % (rows, K, cores)
    line = {
        "impl": "reference", "metric": "effective weight-HBM GB/s, SpMM (OPT-66B shapes, N=16, 80% sparse)",
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores,
                         "kind": "port", "sample": sample + "; encoder: " +
                         ("reference (oracle/_ref)" if oracle.have_ref() else "oracle port")},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_sweep(args):
    """Decode-size sweep over the OPT-66B layer shapes, N and sparsity (one JSON line per point),
    with cuBLAS dense fp16 on the pruned matrix as the comparator.  Device-timed with CUDA graphs;
    every shape's weights exceed or rotate through L2 (copies chosen so that the set is >= 256 MB)."""
    import torch

    import graphneuralnetproj_b200 as sp
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    peak, _ = measured_hbm_peak()
    # "cfg1" = the reference's single-SpMM case (M = K = 7168 with its Split_K hint 5), beside the OPT-66B layers
    shapes = [(n, m, k, 8) for n, m, k, _ in LAYERS if n in args.sweep_layers.split(",")]
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
            wds = [torch.from_numpy(np.concatenate([words, np.zeros(4, np.uint32)]).view(np.int32)).to(dev)
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


def run_prefill(args):
    """Prefill-size points (N >= 256): dense-equivalent TFLOP/s = 2*M*N*K / t against the measured
    dense tensor peak, with cuBLAS dense fp16 beside it.  One JSON line per point."""
    import torch

    import graphneuralnetproj_b200 as sp
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tensor_peak = float(json.load(f)["bf16_tflops"])
    except Exception:
        tensor_peak = 1590.0
    shapes = [(12288, 12288), (49152, 12288)] if not args.small else [(12288, 12288)]
    for M, K in shapes:
        for p in [float(x) for x in args.prefill_p.split(",")]:
            A = sp.synth_fp16((M, K), 0xA300 + int(p * 100), 0.02, p)
            words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, 64, K)
            wd = torch.from_numpy(np.concatenate([words, np.zeros(4, np.uint32)]).view(np.int32)).to(dev)
            od = torch.from_numpy(offsets).to(dev)
            Ad = torch.from_numpy(A.view(np.float16)).to(dev)
            del A, words
            for N in [int(x) for x in args.prefill_n.split(",")]:
                Bd = torch.from_numpy(sp.synth_fp16((K, N), 0xB300, 1.0).view(np.int16)).to(dev)
                Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
                ws = torch.zeros(sp.workspace_bytes(M, N, 2) // 2, dtype=torch.int16, device=dev)
                times = {}
                for label, fn in (("spmm", lambda: sp.SpMM_SplitK_API(None, None, wd, None, None, od, Bd, Cd, M, N, K, ws, 2)),
                                  ("cublas_dense", lambda: torch.matmul(Ad, Bd.view(torch.float16)))):
                    for _ in range(3):
                        fn()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    reps = 5
                    e0.record()
                    for _ in range(reps):
                        fn()
                    e1.record()
                    torch.cuda.synchronize()
                    times[label] = e0.elapsed_time(e1) * 1000.0 / reps
                flops = 2.0 * M * N * K
                print(json.dumps({"M": M, "K": K, "N": N, "sparsity": p, "spmm_us": round(times["spmm"], 1),
                                  "cublas_dense_us": round(times["cublas_dense"], 1),
                                  "dense_equiv_tflops": round(flops / times["spmm"] / 1e6, 1),
                                  "frac_of_tensor_peak": round(flops / times["spmm"] / 1e6 / tensor_peak, 4),
                                  "tensor_peak_tflops": tensor_peak}), flush=True)
            del wd, Ad
            torch.cuda.empty_cache()
    assert sp.device_status() == 0


def run_row_parallel(args):
    """Row-parallel (by K) layer across the GPUs of the box: every rank multiplies its K shard of an
    FFN2-shaped layer (M = 9216, 36864 columns of A per rank) and one NCCL sum all-reduce of the M x N
    result finishes it.  Prints one JSON line with the SpMM-only and the SpMM + reduce time (device-timed,
    max over ranks)."""
    import torch
    import torch.distributed as dist

    import graphneuralnetproj_b200 as sp
    from graphneuralnetproj_b200.tensor_parallel import RowParallelSpMM

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    M, K_shard, N = 9216, 36864, N_TOKENS
    words, offsets, n_offsets = make_layer(sp, "ffn2", M, K_shard, 0xA500 + rank)
    wbytes = 4 * words.size + 4 * n_offsets
    wd = torch.from_numpy(np.concatenate([words, np.zeros(4, np.uint32)]).view(np.int32)).to(dev)
    od = torch.from_numpy(offsets).to(dev)
    Bd = torch.from_numpy(sp.synth_fp16((K_shard, N), 0xB500 + rank, 1.0).view(np.int16)).to(dev)
    layer = RowParallelSpMM(wd, od, M, N, K_shard, split_k=8)
    # a second layer's worth of weights between timed launches keeps the first one out of L2
    other = RowParallelSpMM(wd.clone(), od, M, N, K_shard, split_k=8)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def spmm_only():
        for l in (layer, other):
            rc = sp.SpMM_SplitK_API(None, None, l.words, None, None, l.offsets, Bd, l.C, M, N, K_shard, l.workspace, 8)
            assert rc == 0

    def with_reduce():
        for l in (layer, other):
            l.forward(Bd)

    ms_spmm = timed(spmm_only) / 2
    ms_full = timed(with_reduce) / 2
    # the same with the library's own reduction kernel over peer memory instead of NCCL
    ms_peer = None
    if world > 1:
        try:
            peer_layers = [RowParallelSpMM(l.words, l.offsets, M, N, K_shard, split_k=8, reduce="peer") for l in (layer, other)]

            def with_peer_reduce():
                for l in peer_layers:
                    l.forward(Bd)

            ms_peer = timed(with_peer_reduce) / 2
            assert sp.spmm_api.LIB.spmm_b200_allreduce_status(0) == 0
        except Exception as exc:  # symmetric memory not available on this box
            if rank == 0:
                print("peer-memory reduction unavailable:", exc, file=sys.stderr)
    assert sp.device_status() == 0
    if rank == 0:
        peak, src = measured_hbm_peak()
        print(json.dumps({
            "metric": "effective weight-HBM GB/s, row-parallel SpMM + all-reduce (FFN2 shape, N=16, 80% sparse)",
            "value": round(world * wbytes / ((ms_peer or ms_full) * 1e-3) / 1e9, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "scaling": "weak", "higher_is_better": True,
            "spmm_only_us": round(ms_spmm * 1e3, 2), "spmm_plus_allreduce_us": round(ms_full * 1e3, 2),
            "spmm_plus_peer_reduce_us": round(ms_peer * 1e3, 2) if ms_peer else None,
            "spmm_only_gbs_per_gpu": round(wbytes / (ms_spmm * 1e-3) / 1e9, 1),
            "allreduce_bytes": M * N * 2,
            "config": {"workload": "row_parallel_ffn2", "M": M, "K_per_rank": K_shard, "n_tokens": N, "sparsity": SPARSITY,
                       "parallelism": "row-parallel by K x%d; value uses the library's peer-memory reduction when "
                                      "available, the NCCL all-reduce otherwise; both are listed" % world},
            "roofline_frac_spmm_only": round(wbytes / (ms_spmm * 1e-3) / 1e9 / peak, 4), "peak_source": src}))
    if world > 1:
        dist.destroy_process_group()


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
    peak, _ = measured_hbm_peak()
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

    Bd = torch.from_numpy(sp.synth_fp16((K, N), 0xB400, 1.0).view(np.int16)).to(dev)
    Cd = torch.zeros((M, N), dtype=torch.int16, device=dev)
    ws = torch.zeros(sp.workspace_bytes(M, N, 8) // 2, dtype=torch.int16, device=dev)
    copies = 2  # rotate over two copies of the weights: more than L2 holds
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
            r_wds = [torch.from_numpy(np.concatenate([rw, np.zeros(4, np.uint32)]).view(np.int32)).to(dev) for _ in range(copies)]
            r_od = torch.from_numpy(ro).to(dev)
            residual_bytes = 4 * rw.size + 4 * rn
        words, offsets, n_offsets = sp.InitSparseMatrixA_API(A, M, N, K)
        wds = [torch.from_numpy(np.concatenate([words, np.zeros(4, np.uint32)]).view(np.int32)).to(dev) for _ in range(copies)]
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
        print(json.dumps({"input": label, "M": M, "K": K, "N": N, "residual_nnz": residual_nnz,
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
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sweep", action="store_true", help="decode-size sweep (layers x N x sparsity) instead of the bench line")
    ap.add_argument("--sweep-n", default="8,16,32,64")
    ap.add_argument("--sweep-p", default="0.7,0.8,0.9")
    ap.add_argument("--sweep-layers", default="qkv,out_proj,ffn1,ffn2")
    ap.add_argument("--prefill", action="store_true", help="prefill-size points (N >= 256) instead of the bench line")
    ap.add_argument("--prefill-n", default="256,512,1024,2048")
    ap.add_argument("--prefill-p", default="0.5,0.7,0.8")
    ap.add_argument("--small", action="store_true", help="with --prefill: only the 12288 x 12288 shape")
    ap.add_argument("--row-parallel", action="store_true", help="row-parallel (by K) layer with an NCCL all-reduce, one rank per GPU")
    ap.add_argument("--hetero", action="store_true", help="heterogeneous decomposition points (structured half on the sparse tensor core)")
    ap.add_argument("--hetero-size", type=int, default=12288)
    ap.add_argument("--hetero-n", type=int, default=32)
    args = ap.parse_args()
    if args.row_parallel:
        run_row_parallel(args)
    elif args.hetero:
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
