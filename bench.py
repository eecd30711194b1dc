#!/usr/bin/env python
"""Benchmark of the activation-compression hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the attention-map save/restore of a [4,32,512,512] bf16 causal
softmax map, per-row top-k (ratio 0.05) + 4-bit 64-wide groups; one step = ROUND_TRIPS compress +
decompress round trips over a ring of maps.  Prints ONE JSON line.
Under torchrun every rank works on its own shard of maps (weak scaling, no data-path
collective); the time is the maximum over ranks.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MAP_SHAPE = (4, 32, 512, 512)
RATIO = 0.05
QBIT = 4
NBUF = 4          # distinct input/output sets rotated between round trips (4 x 64 MiB in, > L2)
ROUND_TRIPS = 64  # compress + decompress round trips that make one step (a step is about 4 ms of device time)
SAMPLE_SHAPE = (1, 8, 512, 512)     # the slice of the map one step of the CPU arms works on (1/16 of the map)
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch on this workload (bytes), from an ncu --set full capture of
# the two kernels as they are built now (67.16 + 3.40 MB and 24.92 + 10.58 MB); set an entry to None when its kernel
# changes until a new capture is taken
NCU_TRAFFIC = {"hyc::topk_lane_compress_kernel<4,8>": 70.56e6, "hyc::topk_lane_restore_kernel<4,8,false>": 35.50e6}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peaks():
    """(burst, sustained) dense bf16 TFLOP/s and where they come from."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


def make_map(seed, device, shape=MAP_SHAPE):
    g = torch.Generator(device="cpu").manual_seed(seed)
    b, h, s, _ = shape
    logits = 3 * torch.randn(b, h, s, s, generator=g)
    logits = logits + torch.triu(torch.full((s, s), float("-inf")), diagonal=1)
    return torch.softmax(logits, dim=-1).to(torch.bfloat16).to(device)


def algo_bytes(shape, q_bit, ratio):
    """Algorithmic bytes of one compress and of one decompress of a map (equal by symmetry):
    2 B/elem dense side + q/8 packed + 3/64 group metadata + 4 k/S outlier list."""
    s = shape[-1]
    k = int(s * ratio)
    numel = 1
    for d in shape:
        numel *= d
    per_elem = 2.0 + q_bit / 8.0 + 3.0 / 64.0 + 4.0 * k / s
    return numel * per_elem


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


DEFAULT_REFERENCE = os.path.join(os.sep, "root", "reference")


def find_reference():
    """Folder that holds the reference's ``operators/compress_function.py``: $HYC_REFERENCE, the default checkout
    location, or the copy staged by oracle/stage_reference.py (oracle/_ref).  None when there is none."""
    for cand in (os.environ.get("HYC_REFERENCE"), DEFAULT_REFERENCE, os.path.join(ROOT, "oracle", "_ref")):
        if cand and os.path.isfile(os.path.join(cand, "operators", "compress_function.py")):
            return cand
    return None


def load_reference_compress(ref):
    """The reference's operators/compress_function.py imported UNCHANGED (as a sub-module of a synthetic package,
    so that its relative import of the kernel module resolves inside the same folder)."""
    import importlib
    import types
    name = "hyc_reference_operators"
    if name not in sys.modules:
        pkg = types.ModuleType(name)
        pkg.__path__ = [os.path.join(ref, "operators")]
        sys.modules[name] = pkg
    return importlib.import_module(name + ".compress_function")


class CpuArm:
    """The CPU implementation of the attention-map save/restore on the host cores, on a [1,8,512,512] slice of the
    map per step.  kind "reference": the reference's own pure-PyTorch path imported unchanged -- calibration with
    get_statistics_softmax once (compress_function.py:30-32), then per step compression_softmax (mask multiply +
    to_sparse, :309-313) and decompression_softmax (to_dense, :316-317), which is what the reference's layer runs in
    steady state for this tensor.  kind "port": the CPU oracle's restatement of this repository's top-k form, only
    when no copy of the reference is reachable.  Throughput is counted in the SAME unit as the GPU arm: algorithmic
    bytes of the top-k round trip per map element, so the two values compare as maps per second."""

    def __init__(self):
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        self.a = make_map(99, "cpu", SAMPLE_SHAPE)
        self.nbytes = 2 * algo_bytes(SAMPLE_SHAPE, QBIT, RATIO)
        ref = find_reference()
        self.kind, self.why = "port", "no copy of the reference reachable (HYC_REFERENCE, the default checkout location, oracle/_ref)"
        if ref is not None:
            try:
                cf = load_reference_compress(ref)
                thr = cf.get_statistics_softmax(self.a, RATIO)
                self._step = lambda: cf.decompression_softmax(cf.compression_softmax(self.a, thr))
                self.kind, self.why = "reference", ref
            except Exception as e:       # an import that fails (a Triton too old or too new for the kernel module)
                self.why = "reference at %s not importable: %s" % (ref, repr(e)[:200])
        if self.kind == "port":
            import oracle
            self._step = lambda: oracle.topk_decompress(*oracle.topk_compress(self.a, RATIO, QBIT), QBIT, self.a.shape)

    def step(self):
        self._step()

    def describe(self, steps, secs):
        what = ("get_statistics_softmax once, then compression_softmax + decompression_softmax of the reference "
                "(operators/compress_function.py, imported unchanged)") if self.kind == "reference" else \
            "oracle.topk_compress + oracle.topk_decompress (CPU restatement; %s)" % self.why
        return "%d steps of %s on a %s slice of the map (1/16 of it), %.1f s" % (steps, what, list(SAMPLE_SHAPE), secs)


def cpu_baseline_sample(target_s=10.0):
    """About `target_s` seconds of the CPU arm (rank 0, N = 1 only)."""
    arm = CpuArm()
    arm.step()
    t0 = time.perf_counter()
    reps = 0
    while True:
        arm.step()
        reps += 1
        el = time.perf_counter() - t0
        if el >= target_s or reps >= 1000000:
            break
    return {"value": reps * arm.nbytes / el / 1e9, "unit": "GB/s", "cores": arm.cores, "kind": arm.kind,
            "sample": arm.describe(reps, el)}


def run_reference(args):
    """Reference arm: the reference's CPU implementation of the headline path on the host cores (all threads), same
    metric, unit and config as the GPU arm, exactly --steps timed steps after --warmup untimed ones; one step works on a
    [1,8,512,512] slice of the map (stated in config.sample).  Under torchrun rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm()
    for _ in range(args.warmup):
        arm.step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        arm.step()
    el = time.perf_counter() - t0
    v = args.steps * arm.nbytes / el / 1e9
    cfg = config_dict()
    cfg["sample"] = "one step = one save/restore of a %s slice (1/16 of the map, %d of its rows)" % (
        list(SAMPLE_SHAPE), SAMPLE_SHAPE[0] * SAMPLE_SHAPE[1] * SAMPLE_SHAPE[2])
    print(json.dumps({
        "impl": "reference", "metric": "activation compress+decompress GB/s", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16->u8", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": arm.cores, "kind": arm.kind,
                         "sample": arm.describe(args.steps, el)},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def config_dict():
    return {"workload": "attention-map save/restore, softmax [4,32,512,512] bf16 causal, top-k per row "
                        "ratio 0.05 + q_bit 4 groups of 64 (BASELINE configs[1])",
            "q_bit": QBIT, "outlier_ratio": RATIO, "rows_per_gpu": MAP_SHAPE[0] * MAP_SHAPE[1] * MAP_SHAPE[2],
            "round_trips_per_step": ROUND_TRIPS,
            "l2": "inputs and outputs rotated over %d distinct buffer sets (%d MiB dense) > 126 MB L2" % (
                NBUF, NBUF * 64)}


def time_loop(fn, steps, warmup):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3


def extra_workloads(dev, hbm):
    """Secondary lines of the same path (reported under "also"): the per-channel round trip
    (outlier channels + q-bit codes) of the CPU-runnable config and a q_bit sweep at the Mistral MLP
    width.  Outputs are pre-allocated and each pass over the buffer sets is replayed from a CUDA graph,
    so the small config measures the kernels and not the Python call overhead."""
    from hyc_lora_release_b200.operators import compress_function as cf
    out = []
    g = torch.Generator().manual_seed(1234)
    for name, shape, n_out, mult, ratio, qs, nbuf in (
            ("channel-base round trip [4,512,4096] bf16, 0.5% outlier channels x30 (BASELINE configs[0])",
             (4, 512, 4096), 20, 30.0, 0.005, (4,), 12),
            ("channel-base round trip [1,8192,14336] bf16, 1% outlier channels x20 (BASELINE configs[3], per GPU)",
             (1, 8192, 14336), 143, 20.0, 0.01, (2, 4, 8), 2)):
        xs = []
        for _ in range(nbuf):
            x = torch.randn(*shape, generator=g)
            ch = torch.randperm(shape[-1], generator=g)[:n_out]
            x[:, :, ch] *= mult
            xs.append(x.to(torch.bfloat16).to(dev))
        B, M, N = shape
        for q in qs:
            idx, s = cf.get_statistics_channel_base(xs[0], ratio, q, "per-channel")
            k = idx.numel()
            numel = xs[0].numel()
            nbytes = numel * (4 + q / 4.0) + 2 * (B * M) * k * 2
            qb = [torch.empty((B, M, N * q // 8), dtype=torch.uint8, device=dev) for _ in range(nbuf)]
            ob = [torch.empty((B, M, k), dtype=torch.bfloat16, device=dev) for _ in range(nbuf)]
            xb = [torch.empty(shape, dtype=torch.bfloat16, device=dev) for _ in range(nbuf)]

            def one_pass():
                for j in range(nbuf):
                    cf.outlier_subtraction_fuse_compression_quantization(xs[j], s, idx, q, out=(qb[j], ob[j]))
                    cf.outlier_addition_fuse_decompression_dequantization(qb[j], s, ob[j], idx, q, out=xb[j])
            one_pass()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                one_pass()
            reps = max(3, 48 // nbuf)
            t = time_loop(lambda i: graph.replay(), reps, 3)
            gbs = reps * nbuf * nbytes / t / 1e9
            out.append({"workload": name, "q_bit": q, "value": gbs, "unit": "GB/s", "frac_of_hbm": gbs / hbm,
                        "ms_per_step": t / (reps * nbuf) * 1e3, "launch": "CUDA graph replay of %d compress+decompress pairs" % nbuf})
            del graph, qb, ob, xb
        del xs
    out.append(fused_elementwise_workload(dev, hbm))
    out.append(attention_backward_workload(dev, hbm))
    out.append(prune_workload(dev, hbm))
    out.extend(reference_triton_lines(dev, hbm))
    return out


def reference_triton_lines(dev, hbm):
    """The reference's own Triton kernels, compiled by the installed Triton for THIS GPU and timed with CUDA events on
    the tensors of the lines above: the quantize / de-quantize pair (compress_function_kernel.py:47-112, 150-206), the
    channel-base and the softmax-prune round trips through the reference's API, and the two fused LoRA-SiLU-Hadamard
    kernels.  A reported comparison; an error message stands in where Triton refuses a kernel."""
    ref = find_reference()
    if ref is None:
        return [{"workload": "reference Triton kernels on this GPU", "unavailable": "no copy of the reference reachable"}]
    out = []
    try:
        import importlib
        cf = load_reference_compress(ref)
        fwd = importlib.import_module("hyc_reference_operators.triton_fuse_lora_silu_hadamard_forward_kernels")
        bwd = importlib.import_module("hyc_reference_operators.triton_fuse_lora_silu_hadamard_backward_kernels")
        import triton
        ver = triton.__version__
    except Exception as e:
        return [{"workload": "reference Triton kernels on this GPU", "unavailable": repr(e)[:300]}]
    g = torch.Generator().manual_seed(1234)

    def timed(fn, n=10):
        return time_loop(lambda i: fn(), n, 3) / n

    def guarded(name, fn):
        try:
            line = fn()
        except Exception as e:
            line = {"unavailable": repr(e)[:300]}
        line["workload"] = "reference Triton on this GPU (triton %s): %s" % (ver, name)
        out.append(line)
    for shape, n_out, mult, ratio, qs in (((4, 512, 4096), 20, 30.0, 0.005, (4,)), ((1, 8192, 14336), 143, 20.0, 0.01, (2, 4, 8))):
        x = torch.randn(*shape, generator=g)
        x[:, :, torch.randperm(shape[-1], generator=g)[:n_out]] *= mult
        x = x.to(torch.bfloat16).to(dev)
        for q in qs:
            def pair(q=q, x=x):
                s_ = cf.get_statistics_only_quant(x, q, "per-channel")
                s_ = (s_ + (s_ == 0) * 1e-3).to(torch.bfloat16)
                qq = cf.compression_quantization(x, s_, q)
                tc, td = timed(lambda: cf.compression_quantization(x, s_, q)), timed(lambda: cf.decompression_dequantization(qq, s_, q))
                nb = x.numel() * (4 + q / 4.0)
                return {"q_bit": q, "value": nb / (tc + td) / 1e9, "unit": "GB/s", "frac_of_hbm": nb / (tc + td) / 1e9 / hbm,
                        "kernel_ms": {"compress": tc * 1e3, "decompress": td * 1e3}}
            guarded("compression_quantization + decompression_dequantization %s" % list(shape), pair)
        if shape[-1] == 4096:
            def chan(x=x, ratio=ratio):
                idx, sc = cf.get_statistics_channel_base(x, ratio, 4, "per-channel")
                st = {"outlier_channel_index": idx, "scale": sc}

                def rt():
                    xo, qq, i2, s2 = cf.compression_pack_channel_base(x.clone(), ratio, 4, "per-channel", 9, 5, st)
                    return cf.outlier_addition_fuse_decompression_dequantization(qq, s2, xo, i2, 4)
                t = timed(rt)
                nb = x.numel() * 5.0
                return {"q_bit": 4, "value": nb / t / 1e9, "unit": "GB/s", "frac_of_hbm": nb / t / 1e9 / hbm, "ms_per_step": t * 1e3,
                        "note": "as the layer calls it: clone + index gather + zeroing + quant kernel, then dequant kernel + scatter"}
            guarded("channel-base round trip %s" % list(shape), chan)
        del x

    def prune():
        a = make_map(2000, dev)
        thr = cf.get_statistics_softmax(a, RATIO)
        t = timed(lambda: cf.decompression_softmax(cf.compression_softmax(a, thr)), 5)
        nnz = int(cf.compression_softmax(a, thr).values().numel())
        nb = a.numel() * 4 + 20 * nnz
        return {"value": nb / t / 1e9, "unit": "GB/s", "frac_of_hbm": nb / t / 1e9 / hbm, "ms_per_step": t * 1e3}
    guarded("compression_softmax + to_dense [4,32,512,512]", prune)

    def fused():
        T, N, R, q = 8192, 14336, 16, 4
        rn = lambda *sh, sc=1.0: (torch.randn(*sh, generator=g) * sc).to(torch.bfloat16).to(dev)
        xa1, xa2, b1, b2 = rn(1, T, R), rn(1, T, R), rn(R, N, sc=.05), rn(R, N, sc=.05)
        x1, x2, go = rn(1, T, N), rn(1, T, N), rn(1, T, N)
        s1, s2 = cf.get_statistics_only_quant(x1, q, "per-channel"), cf.get_statistics_only_quant(x2, q, "per-channel")
        q1, q2, _ = fwd.triton_fuse_silu_forward(xa1, b1, x1, s1, xa2, b2, x2, s2, q)
        tf = timed(lambda: fwd.triton_fuse_silu_forward(xa1, b1, x1, s1, xa2, b2, x2, s2, q), 6)
        tb = timed(lambda: bwd.triton_fuse_silu_backward(xa1, b1, q1, s1, xa2, b2, q2, s2, go, q), 6)
        nel = T * N
        bf_, bb = nel * (4 + 2 + 2 * q / 8), nel * (2 * q / 8 + 2 + 6)
        return {"q_bit": q, "value": (bf_ + bb) / (tf + tb) / 1e9, "unit": "GB/s", "frac_of_hbm": (bf_ + bb) / (tf + tb) / 1e9 / hbm,
                "forward": {"ms": tf * 1e3, "GBps": bf_ / tf / 1e9}, "backward": {"ms": tb * 1e3, "GBps": bb / tb / 1e9}}
    guarded("triton_fuse_silu_forward + triton_fuse_silu_backward [1,8192,14336]", fused)
    return out


def prune_workload(dev, hbm):
    """The reference's own form of the saved probability map (compress_function.py:309-317): entries above a
    calibrated global threshold as a sparse COO tensor (int64 index + bf16 value), restored by to_dense.  Headline
    map [4,32,512,512], ratio 0.05, through the operator API (which reads the number of kept entries back once per
    call, as to_sparse does).  Algorithmic bytes: the dense map read once and written once, the list written and
    read (10 bytes per kept entry each way)."""
    from hyc_lora_release_b200.operators import compress_function as cf
    maps = [make_map(2000 + i, dev) for i in range(NBUF)]
    thr = cf.get_statistics_softmax(maps[0], RATIO)
    handles = [cf.compression_softmax(m, thr) for m in maps]
    nnz = sum(h.values().numel() for h in handles) / NBUF
    numel = maps[0].numel()
    nbytes = numel * 4 + 2 * 10 * nnz
    nbytes_tiled = numel * 4 + 2 * (4 * nnz + 8 * (numel // 2048))     # 4-byte words + the per-batch directory
    t_c = time_loop(lambda i: cf.compression_softmax(maps[i % NBUF], thr), 20, 3) / 20
    t_d = time_loop(lambda i: cf.decompression_softmax(handles[i % NBUF]), 20, 3) / 20
    gbs = nbytes / (t_c + t_d) / 1e9
    # the form the fused layer uses in steady state: fixed-capacity buffers, the count stays on the device; timed as
    # CUDA-graph replays over the buffer sets (what a captured training step pays) and as plain operator calls
    thr_f = float(thr)
    pm = [cf.compression_softmax_static(m, thr_f, ratio=RATIO) for m in maps]
    dense = [torch.empty(MAP_SHAPE, dtype=torch.bfloat16, device=dev) for _ in range(NBUF)]
    t_cs = time_loop(lambda i: cf.compression_softmax_static(maps[i % NBUF], thr_f, ratio=RATIO), 20, 3) / 20
    t_ds = time_loop(lambda i: pm[i % NBUF].to_dense(out=dense[i % NBUF]), 20, 3) / 20

    def graph_avg(fn):
        for j in range(NBUF):
            fn(j)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for j in range(NBUF):
                fn(j)
        return time_loop(lambda i: gr.replay(), 25, 3) / (25 * NBUF)
    keep = [None] * NBUF

    def comp(j):
        keep[j] = cf.compression_softmax_static(maps[j], thr_f, ratio=RATIO)
    t_cg = graph_avg(comp)
    t_dg = graph_avg(lambda j: pm[j].to_dense(out=dense[j]))
    return {"workload": "attention-map save/restore in the reference's form: global-threshold prune to sparse COO + to_dense, "
                        "[4,32,512,512] (BASELINE configs[1] map)", "value": gbs, "unit": "GB/s", "frac_of_hbm": gbs / hbm,
            "ms_per_step": (t_c + t_d) * 1e3, "kept_fraction": nnz / numel,
            "kernel_ms": {"compress": t_c * 1e3, "restore": t_d * 1e3},
            "without_host_sync": {"GBps": nbytes_tiled / (t_cg + t_dg) / 1e9, "frac_of_hbm": nbytes_tiled / (t_cg + t_dg) / 1e9 / hbm,
                                  "GBps_in_reference_bytes": nbytes / (t_cg + t_dg) / 1e9,
                                  "compress_ms": t_cg * 1e3, "restore_ms": t_dg * 1e3,
                                  "as_operator_calls": {"compress_ms": t_cs * 1e3, "restore_ms": t_ds * 1e3},
                                  "launch": "CUDA graph replay over %d buffer sets" % NBUF,
                                  "api": "compression_softmax_static -> TiledPrunedMap.to_dense (one pass each way, 4-byte "
                                         "entries, count left on the device)"},
            "launch": "operator calls, CUDA events (compress includes one device-to-host read of the count)"}


def attention_backward_workload(dev, hbm):
    """Backward side of the attention-map save: restore of the top-k + 4-bit map fused with softmax_backward
    (the restored map never reaches HBM), on the headline's [4,32,512,512] map.  Algorithmic bytes: the saved
    form (codes, group parameters, outlier list) + the upstream gradient in, the gradient out."""
    from hyc_lora_release_b200.operators import compress_function as cf
    maps = [make_map(2000 + i, dev) for i in range(NBUF)]
    g = torch.Generator().manual_seed(5)
    grads = [torch.randn(*MAP_SHAPE, generator=g).to(torch.bfloat16).to(dev) for _ in range(NBUF)]
    hs = [cf.compression_softmax_topk(m, RATIO, QBIT) for m in maps]
    outs = [torch.empty_like(m) for m in maps]
    del maps
    for j in range(NBUF):
        hs[j].softmax_backward(grads[j], out=outs[j])
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for j in range(NBUF):
            hs[j].softmax_backward(grads[j], out=outs[j])
    t = time_loop(lambda i: graph.replay(), 10, 3) / (10 * NBUF)
    numel = grads[0].numel()
    nbytes = algo_bytes(MAP_SHAPE, QBIT, RATIO) - 2.0 * numel + 4.0 * numel
    return {"workload": "attention-map backward: top-k restore fused with softmax_backward, [4,32,512,512] (BASELINE configs[1] map)",
            "q_bit": QBIT, "value": nbytes / t / 1e9, "unit": "GB/s", "frac_of_hbm": nbytes / t / 1e9 / hbm,
            "ms_per_step": t * 1e3, "launch": "CUDA graph replay over %d buffer sets" % NBUF}


def fused_elementwise_workload(dev, hbm):
    """The two stand-alone fused LoRA-SiLU-Hadamard kernels behind the reference's launch wrappers
    (triton_fuse_silu_forward / triton_fuse_silu_backward) at the Mistral MLP width, 8192 tokens, q_bit 4.
    Algorithmic bytes per element: forward 2+2 in, 2 + 2*q/8 out; backward 2*q/8 + 2 in, 6 out."""
    from hyc_lora_release_b200.operators import compress_function as cf
    from hyc_lora_release_b200.operators.triton_fuse_lora_silu_hadamard_forward_kernels import triton_fuse_silu_forward
    from hyc_lora_release_b200.operators.triton_fuse_lora_silu_hadamard_backward_kernels import triton_fuse_silu_backward
    g = torch.Generator().manual_seed(77)
    T, N, R, q = 8192, 14336, 16, 4
    rn = lambda *sh, sc=1.0: (torch.randn(*sh, generator=g) * sc).to(torch.bfloat16).to(dev)
    xa1, xa2 = rn(1, T, R), rn(1, T, R)
    b1, b2 = rn(N, R, sc=.05).t(), rn(N, R, sc=.05).t()
    x1, x2, go = rn(1, T, N), rn(1, T, N), rn(1, T, N)
    s1 = cf.get_statistics_only_quant(x1, q, "per-channel")
    s2 = cf.get_statistics_only_quant(x2, q, "per-channel")
    q1, q2, _ = triton_fuse_silu_forward(xa1, b1, x1, s1, xa2, b2, x2, s2, q)
    tf = time_loop(lambda i: triton_fuse_silu_forward(xa1, b1, x1, s1, xa2, b2, x2, s2, q), 8, 3) / 8
    tb = time_loop(lambda i: triton_fuse_silu_backward(xa1, b1, q1, s1, xa2, b2, q2, s2, go, q), 8, 3) / 8
    nel = T * N
    bf, bb = nel * (4 + 2 + 2 * q / 8), nel * (2 * q / 8 + 2 + 6)
    return {"workload": "stand-alone fused LoRA-SiLU-Hadamard kernels (triton_fuse_silu_forward/backward drop-ins), "
                        "[1,8192,14336] bf16, q_bit 4",
            "q_bit": q, "value": (bf + bb) / (tf + tb) / 1e9, "unit": "GB/s",
            "frac_of_hbm": (bf + bb) / (tf + tb) / 1e9 / hbm, "ms_per_step": (tf + tb) * 1e3,
            "forward": {"ms": tf * 1e3, "GBps": bf / tf / 1e9}, "backward": {"ms": tb * 1e3, "GBps": bb / tb / 1e9},
            "launch": "one forward + one backward call through the operator wrappers (inputs 3 x 235 MB > L2)"}


def run_profile(args):
    """Minimal launch sequence of one workload (few launches, inputs > L2, < 2 GB on the device)."""
    from hyc_lora_release_b200.operators import compress_function as cf
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.profile == "mlp":
        line = mlp_workload(dev, None, steps=args.steps, warmup=args.warmup)
        print(json.dumps({"profile": "mlp", "steps": args.steps, "ms_per_step": line["ms_per_step"],
                          "tokens_per_s": line["value"], "tflops": line["roofline"]["achieved"],
                          "cuda_graph_replay_ms_per_step": line["cuda_graph_replay_ms_per_step"]}))
        return
    if args.profile == "layer":
        line = layer_workload(dev, None, steps=args.steps, warmup=args.warmup, graph=False)
        print(json.dumps({"profile": "layer", "steps": args.steps, "ms_per_step": line["ms_per_step"],
                          "tokens_per_s": line["value"], "tflops": line["roofline"]["achieved"]}))
        return
    if args.profile == "model":
        line = model_workload(dev, None, steps=args.steps, warmup=args.warmup, n_layers=args.layers)
        print(json.dumps(line))
        return
    if args.profile == "attn_bwd":
        print(json.dumps(attention_backward_workload(dev, peaks()[0])))
        return
    if args.profile == "prune":
        print(json.dumps(prune_workload(dev, peaks()[0])))
        return
    if args.profile == "fused":
        line = fused_elementwise_workload(dev, peaks()[0])
        print(json.dumps({"profile": "fused", "forward": line["forward"], "backward": line["backward"]}))
        return
    if args.profile == "attn_topk":
        maps = [make_map(1000 + i, dev) for i in range(NBUF)]
        nbytes = 2 * algo_bytes(MAP_SHAPE, QBIT, RATIO)

        def step(i):
            cf.compression_softmax_topk(maps[i % NBUF], RATIO, QBIT).to_dense()
    else:
        q = int(args.profile[-1])
        g = torch.Generator().manual_seed(1234)
        xs = []
        for _ in range(2):
            x = torch.randn(1, 8192, 14336, generator=g)
            x[:, :, torch.randperm(14336, generator=g)[:143]] *= 20.0
            xs.append(x.to(torch.bfloat16).to(dev))
        idx, s = cf.get_statistics_channel_base(xs[0], 0.01, q, "per-channel")
        nbytes = xs[0].numel() * (4 + q / 4.0)

        def step(i):
            o, qq = cf.outlier_subtraction_fuse_compression_quantization(xs[i % 2], s, idx, q)
            cf.outlier_addition_fuse_decompression_dequantization(qq, s, o, idx, q)
    t = time_loop(step, args.steps, args.warmup)
    print(json.dumps({"profile": args.profile, "steps": args.steps, "ms_per_step": t / args.steps * 1e3,
                      "GBps": args.steps * nbytes / t / 1e9}))


def ranks_hold_identical(reducer, dist):
    """True when every rank's averaged gradient buffer has the same fingerprint (None on a single rank)."""
    if dist is None:
        return None
    mine = reducer.checksum()
    all_sums = [None] * dist.get_world_size()
    dist.all_gather_object(all_sums, mine)
    return all(v == all_sums[0] for v in all_sums)


def mlp_eager_baseline(dev, B, M, H, I, R, steps=200, warmup=5):
    """The same MLP block in plain PyTorch on the same GPU: library (cuBLAS) matmuls, torch element-wise kernels and
    autograd, LoRA rank R on gate/up/down, frozen bf16 weights, NOTHING compressed (every activation saved in bf16).
    Reported beside the fused path; not part of it."""
    g = torch.Generator().manual_seed(4321)
    rn = lambda *sh, sc=1.0: (torch.randn(*sh, generator=g) * sc).to(torch.bfloat16).to(dev)
    x = rn(B, M, H).requires_grad_(True)
    wg, wu, wd = rn(I, H, sc=.02), rn(I, H, sc=.02), rn(H, I, sc=.02)
    lora = [rn(R, H, sc=.02), rn(I, R, sc=.02), rn(R, H, sc=.02), rn(I, R, sc=.02), rn(R, I, sc=.02), rn(H, R, sc=.02)]
    for t in lora:
        t.requires_grad_(True)
    ag, bg, au, bu, ad, bd = lora
    nw = torch.ones(H, dtype=torch.bfloat16, device=dev)
    gout = rn(B, M, H)

    def step(i):
        xn = torch.nn.functional.rms_norm(x, (H,), nw, 1e-5)
        gate = xn @ wg.t() + (xn @ ag.t()) @ bg.t()
        up = xn @ wu.t() + (xn @ au.t()) @ bu.t()
        had = torch.nn.functional.silu(gate) * up
        y = x + had @ wd.t() + (had @ ad.t()) @ bd.t()
        torch.autograd.grad(y, [x] + lora, gout)
    t = time_loop(step, steps, warmup)
    return {"tokens_per_s": B * M * steps / t, "ms_per_step": t / steps * 1e3,
            "what": "plain PyTorch on the same GPU: cuBLAS matmuls + torch element-wise kernels + autograd, bf16 "
                    "activations kept uncompressed"}


def mlp_workload(dev, dist=None, steps=200, warmup=5, shape="llama", q_bit=4, eager=False):
    """Fused LoRA-SiLU-Hadamard MLP forward + backward.  shape "llama" = BASELINE configs[2]: x [4,512,4096] per
    GPU, intermediate 11008, 0.5 % outlier channels x30; shape "mistral" = BASELINE configs[3]: 8192 tokens per GPU,
    intermediate 14336, 1 % outlier channels x20.  Frozen W ~ N(0, .02), LoRA rank 16, saved activations q_bit
    wide; calibration (5 iterations, statistics synchronised across ranks) happens before the timed region.  With
    several ranks every rank runs its OWN token shard (inputs seeded per rank, weights shared) and the six LoRA
    gradients are averaged over the ranks inside the timed step (one bucketed all-reduce started from the
    backward's hook); after the timed region the ranks' averaged gradients are compared."""
    from hyc_lora_release_b200 import mlp, parallel
    rank = dist.get_rank() if dist is not None else 0
    g = torch.Generator().manual_seed(4321)
    gr = torch.Generator().manual_seed(9000 + rank)          # this rank's token shard
    if shape == "llama":
        B, M, H, I, R, n_out, amp, ratio = 4, 512, 4096, 11008, 16, 20, 30, 0.005
        name = "Llama-2-7B shapes, x [4,512,4096] per GPU, q_bit %d (BASELINE configs[2])" % q_bit
    else:
        B, M, H, I, R, n_out, amp, ratio = 1, 8192, 4096, 14336, 16, 41, 20, 0.01
        name = "Mistral-7B shapes, x [1,8192,4096] per GPU, q_bit %d (BASELINE configs[3])" % q_bit
    T = B * M
    rn = lambda *sh, sc=1.0: (torch.randn(*sh, generator=g) * sc).to(torch.bfloat16).to(dev)
    outlier_channels = torch.randperm(H, generator=g)[:n_out]
    ku = lambda out, inp: ((torch.rand(out, inp, generator=g) * 2 - 1) * (1.0 / inp) ** 0.5).to(torch.bfloat16).to(dev)
    W = mlp.MLPWeights(norm_w=torch.ones(H, dtype=torch.bfloat16, device=dev),
                       wg=rn(I, H, sc=.02), wu=rn(I, H, sc=.02), wd=rn(H, I, sc=.02),
                       ag=ku(R, H), bg=rn(I, R, sc=.02), au=ku(R, H), bu=rn(I, R, sc=.02), ad=ku(R, I), bd=rn(H, R, sc=.02))
    x = torch.randn(B, M, H, generator=gr)
    x[:, :, outlier_channels] *= amp
    x = x.to(torch.bfloat16).to(dev)
    gout = (torch.randn(B, M, H, generator=gr)).to(torch.bfloat16).to(dev)
    state = mlp.MLPState(q_bit=q_bit, layernorm_outlier_ratio=ratio)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    reducer = parallel.LoraGradReducer()

    def step(i):
        out, saved = mlp.mlp_forward(x, W, state, status=st)
        # the LoRA-gradient exchange starts inside the backward pass and overlaps its last two kernels
        mlp.mlp_backward(gout, saved, W, status=st, on_lora_grads=lambda g_: reducer.add("mlp", g_))
        reducer.finish()
    for i in range(6):          # calibration iterations
        step(i)
        if i < state.iteration_threshold:
            parallel.sync_calibration(state.static_value)
    mlp.check_status(st, "mlp")
    t = time_loop(step, steps, warmup)
    mlp.check_status(st, "mlp")
    world = 1
    if dist is not None:
        world = dist.get_world_size()
        tt = torch.tensor([t], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = float(tt.item())
    # the steady-state step is a fixed launch sequence: captured once, replayed without host work between launches
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(7)
    torch.cuda.current_stream().wait_stream(side)
    cg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(cg):
        step(7)
    tg = time_loop(lambda i: cg.replay(), steps, warmup)
    mlp.check_status(st, "mlp (graph replay)")
    if dist is not None:
        tt = torch.tensor([tg], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        tg = float(tt.item())
    flop_per_token = 12 * H * I + R * (18 * H + 22 * I)
    burst, sustained, src = tensor_peaks()
    tf = T * flop_per_token * steps / t / 1e12
    line = {"workload": "fused LoRA-SiLU-Hadamard MLP fwd+bwd, " + name, "q_bit": q_bit,
            "metric": "tokens/s", "value": world * T * steps / t, "unit": "tokens/s", "ms_per_step": t / steps * 1e3,
            "tokens_per_gpu": T, "flop_per_token": flop_per_token, "cuda_graph_replay_ms_per_step": tg / steps * 1e3,
            "steps": steps, "timed_region_s": t,
            "roofline": {"bound": "tensor", "kernel": "tc::mlp_gemm_kernel (gate+up forward, down forward, grad_down, grad_x: "
                                                      "four launches per step)",
                         "achieved": tf, "peak": sustained, "unit": "TFLOP/s", "frac": tf / sustained,
                         "frac_of_burst_peak": tf / burst, "algorithmic_flop_per_step": T * flop_per_token,
                         "traffic": None,
                         "peak_source": src + " (sustained %.0f, burst %.0f TFLOP/s)" % (sustained, burst)},
            "gpu_launches_per_step": 4, "identical_grads_on_all_ranks": ranks_hold_identical(reducer, dist),
            "note": "4 tcgen05 GEMM launches + streaming kernels per step; with n_gpus > 1 every rank has its own token "
                    "shard and the LoRA gradients are averaged by one all-reduce inside the step"}
    if eager:
        del W, x, gout
        torch.cuda.empty_cache()
        line["pytorch_eager_same_gpu"] = mlp_eager_baseline(dev, B, M, H, I, R)
    return line


def layer_workload(dev, dist=None, steps=80, warmup=3, graph=True):
    """One fused decoder layer (attention + MLP) forward + backward at the Llama-2-7B geometry of BASELINE
    configs[4]: hidden 4096, 32 heads of 128, intermediate 11008, sequence 2048, batch 1 per GPU, causal mask,
    LoRA rank 16 on q/k/v/o/gate/up/down, saved activations 4-bit with 0.5 % outlier channels, the probability
    map [1,32,2048,2048] saved as per-row top-k (5 %) + 4-bit groups.  Driven through the layer module and
    autograd (the call a model fork makes); calibration happens before the timed region."""
    import types
    from hyc_lora_release_b200 import mlp, parallel
    from hyc_lora_release_b200.layer import FusedLlamaLayerIntraInterFullFuse
    rank = dist.get_rank() if dist is not None else 0
    g = torch.Generator().manual_seed(777)
    gr = torch.Generator().manual_seed(7000 + rank)          # this rank's sequence
    B, M, H, heads, d, I, R = 1, 2048, 4096, 32, 128, 11008, 16
    bf = torch.bfloat16

    def lin(out, inp, sc=None, grad=False):
        m = torch.nn.Linear(inp, out, bias=False, device=dev, dtype=bf)
        with torch.no_grad():
            if sc is None:
                m.weight.copy_(((torch.rand(out, inp, generator=g) * 2 - 1) * (1.0 / inp) ** 0.5).to(bf))
            else:
                m.weight.copy_((torch.randn(out, inp, generator=g) * sc).to(bf))
        m.weight.requires_grad_(grad)
        return m

    def adapter(out, inp):
        a, b = torch.nn.Module(), torch.nn.Module()
        a.default, b.default = lin(R, inp, grad=True), lin(out, R, sc=.02, grad=True)
        return a, b
    dims = dict(q=(H, H), k=(H, H), v=(H, H), o=(H, H), gate=(I, H), up=(I, H), down=(H, I))
    mods = {n: (lin(o_, i_, sc=.02),) + adapter(o_, i_) for n, (o_, i_) in dims.items()}
    outlier_channels = torch.randperm(H, generator=g)[:20]
    x = torch.randn(B, M, H, generator=gr)
    x[:, :, outlier_channels] *= 30
    x = x.to(bf).to(dev)
    pos = torch.arange(M, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb = torch.cat([torch.outer(pos, inv)] * 2, -1)
    cos, sin = emb.cos().to(bf).to(dev), emb.sin().to(bf).to(dev)
    mask = torch.full((M, M), torch.finfo(bf).min).triu(1).to(bf).reshape(1, 1, M, M).to(dev)
    n1 = torch.ones(H, dtype=bf, device=dev)
    n2 = torch.ones(H, dtype=bf, device=dev)
    gy = (torch.randn(B, M, H, generator=gr)).to(bf).to(dev)
    layer = FusedLlamaLayerIntraInterFullFuse()
    layer.set_hyclora_config(types.SimpleNamespace(use_hyclora=True, iteration_threshold=5, softmax_outlier_ratio=0.05,
                                                   layernorm_outlier_ratio=0.005, q_bit=4, softmax_map_mode="topk"))
    reducer = parallel.LoraGradReducer()
    reducer.attach_layer(0, layer)
    args = [None, n1, None, cos, sin]
    for n in ("q", "k", "v", "o"):
        args += list(mods[n])
    args += [n2, None]
    for n in ("gate", "up", "down"):
        args += list(mods[n])
    args += [mask, heads, d, heads]

    def step(i):
        xin = x.detach().requires_grad_(True)
        args[0] = xin
        y = layer(*args)
        # autograd hands the layer's LOCAL adapter gradients back; the averaged ones are what finish() leaves in .grad
        torch.autograd.grad(y, [xin] + lora_weights, gy)
        reducer.finish()
    lora_weights = [m3[j].default.weight for m3 in mods.values() for j in (1, 2)]
    for i in range(6):
        step(i)
        if i < 5:
            parallel.sync_calibration(layer.attn_state.static_value)
            parallel.sync_calibration(layer.mlp_state.static_value)
    layer.check_kernel_status = True
    layer.track_saved_bytes = True
    step(6)
    layer.check_kernel_status = False
    layer.track_saved_bytes = False
    saved_bytes = layer.last_saved_bytes
    # the same tensors kept as plain bf16 (x, x_norm_1, q, k, v, o, x_medium, x_norm_2: T x H each; gate and up main
    # branches: T x I each; the probability map)
    dense_bytes = 2 * (8 * B * M * H + 2 * B * M * I + B * heads * M * M)
    t = time_loop(step, steps, warmup)
    world = 1
    graph_ms = None
    if dist is not None:
        world = dist.get_world_size()
        tt = torch.tensor([t], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = float(tt.item())
    if graph:
        # the steady-state step (module forward + autograd backward) is a fixed launch sequence: captured once,
        # replayed without host work between the launches
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step(0)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(0)
        tg = time_loop(lambda i: graph.replay(), steps, warmup)
        if dist is not None:       # the captured step holds the all-reduce of the LoRA gradients too
            tt = torch.tensor([tg], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            tg = float(tt.item())
        graph_ms = tg / steps * 1e3
    T = B * M
    # frozen GEMMs (no weight gradient): 2 flop x (fwd + bwd) per weight element; attention products 4 M d per
    # head and token forward (scores + P.V over the full, unskipped square), twice that backward; rank-16 terms:
    # 12 H R per attention projection, R (18 H + 22 I) for the MLP
    flop_per_token = 4 * (4 * H * H + 3 * H * I) + 12 * M * heads * d + R * (48 * H + 18 * H + 22 * I)
    burst, sustained, src = tensor_peaks()
    tf = T * flop_per_token * steps / t / 1e12
    return {"workload": "fused decoder layer fwd+bwd through the layer module, Llama-2-7B geometry, seq 2048, batch 1 per GPU, "
                        "q_bit 4, map top-k 5 % (one of the 32 layers of BASELINE configs[4])",
            "metric": "tokens/s", "value": world * T * steps / t, "unit": "tokens/s (one layer)", "ms_per_step": t / steps * 1e3,
            "tokens_per_gpu": T, "flop_per_token": flop_per_token, "cuda_graph_replay_ms_per_step": graph_ms,
            "saved_for_backward_bytes": saved_bytes, "same_tensors_in_bf16_bytes": dense_bytes,
            "identical_grads_on_all_ranks": ranks_hold_identical(reducer, dist),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": sustained, "unit": "TFLOP/s", "frac": tf / sustained,
                         "peak_source": src + " (sustained)"},
            "note": "the two attention products per direction are library batched GEMMs and, like every pass over the "
                    "[1,32,2048,2048] map (softmax, save, restore, softmax backward), bound by HBM, not by the tensor cores"}


def model_workload(dev, dist=None, steps=4, warmup=3, n_layers=32, graph=True):
    """One training step (forward + backward) of the whole 32-layer stack of BASELINE configs[4]: token embedding
    (vocabulary 32000, hidden 4096), 32 fused decoder layers driven through the layer module (32 heads of 128,
    intermediate 11008, LoRA rank 16 on q/k/v/o/gate/up/down, 4-bit saves, top-k map), final RMSNorm, the
    vocabulary projection and a cross-entropy loss on random token ids uniform in [0,32000), sequence 2048,
    batch 1 per GPU.  Only the adapters train (frozen embedding, norms and head).  Frozen weights are random-init
    bf16 drawn on the device, distinct per layer.  The LoRA gradients of every layer are all-reduced over NCCL
    when there are several ranks.  The loss is read back to the host at the end of every step."""
    import types
    from hyc_lora_release_b200 import mlp, parallel
    from hyc_lora_release_b200.layer import FusedLlamaLayerIntraInterFullFuse
    from hyc_lora_release_b200.operators.rmsnorm_kernels import rmsnorm_backward, rmsnorm_forward
    B, M, H, heads, d, I, R, V = 1, 2048, 4096, 32, 128, 11008, 16, 32000
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(4242 + (dist.get_rank() if dist is not None else 0))

    def lin(out, inp, sc=None, grad=False):
        m = torch.nn.Linear(inp, out, bias=False, device=dev, dtype=bf)
        with torch.no_grad():
            if sc is None:
                m.weight.copy_((torch.rand(out, inp, generator=g, device=dev) * 2 - 1) * (1.0 / inp) ** 0.5)
            else:
                m.weight.copy_(torch.randn(out, inp, generator=g, device=dev) * sc)
        m.weight.requires_grad_(grad)
        return m

    def adapter(out, inp):
        a, b = torch.nn.Module(), torch.nn.Module()
        a.default, b.default = lin(R, inp, grad=True), lin(out, R, sc=.02, grad=True)
        return a, b
    dims = dict(q=(H, H), k=(H, H), v=(H, H), o=(H, H), gate=(I, H), up=(I, H), down=(H, I))
    pos = torch.arange(M, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb_t = torch.cat([torch.outer(pos, inv)] * 2, -1)
    cos, sin = emb_t.cos().to(bf).to(dev), emb_t.sin().to(bf).to(dev)
    mask = torch.full((M, M), torch.finfo(bf).min).triu(1).to(bf).reshape(1, 1, M, M).to(dev)
    cfg = types.SimpleNamespace(use_hyclora=True, iteration_threshold=5, softmax_outlier_ratio=0.05,
                                layernorm_outlier_ratio=0.005, q_bit=4, softmax_map_mode="topk")
    # every layer's LoRA gradients go into one flat buffer; an all-reduce starts for every 10 MB of it that is complete
    reducer = parallel.LoraGradReducer(bucket_bytes=10 << 20)
    layers, adapters = [], []
    gw = torch.Generator(device=dev).manual_seed(4242)       # weights: the same on every rank
    g_rank = g
    g = gw
    for li in range(n_layers):
        mods = {n: (lin(o_, i_, sc=.02),) + adapter(o_, i_) for n, (o_, i_) in dims.items()}
        layer = FusedLlamaLayerIntraInterFullFuse()
        layer.set_hyclora_config(cfg)
        reducer.attach_layer(li, layer)
        args = [None, torch.ones(H, dtype=bf, device=dev), None, cos, sin]
        for n in ("q", "k", "v", "o"):
            args += list(mods[n])
        args += [torch.ones(H, dtype=bf, device=dev), None]
        for n in ("gate", "up", "down"):
            args += list(mods[n])
        args += [mask, heads, d, heads]
        layers.append((layer, args))
        adapters += [m3[j].default.weight for m3 in mods.values() for j in (1, 2)]
    embed = (torch.randn(V, H, generator=g, device=dev) * 0.02).to(bf)
    head_w = (torch.randn(V, H, generator=g, device=dev) * 0.02).to(bf)
    norm_w = torch.ones(H, dtype=bf, device=dev)
    status = mlp._status_tensor(dev)

    class NormHead(torch.autograd.Function):
        """final RMSNorm + vocabulary projection: the norm kernels of the path and the tcgen05 GEMM in both
        weight orientations (logits = h W^T, grad_h = grad_logits W); frozen weights, so no weight gradient"""

        @staticmethod
        def forward(ctx, h):
            h2 = h.reshape(-1, H)
            y, mean, rstd, blk, warps = rmsnorm_forward(h2, norm_w, 1e-5)
            ctx.save_for_backward(h2, rstd)
            ctx.meta = (mean, blk, warps, h.shape)
            return mlp.gemm(y.reshape(-1, H), head_w, status=status)

        @staticmethod
        def backward(ctx, g_logits):
            h2, rstd = ctx.saved_tensors
            mean, blk, warps, shape = ctx.meta
            gy = mlp.gemm(g_logits.contiguous(), head_w, b_is_kn=True, status=status)
            dx, _ = rmsnorm_backward(gy, h2, norm_w, mean, rstd, (True, False), 1e-5, warps, blk)
            return dx.reshape(shape)

    n_ids = 4
    g = g_rank                                                # token ids and labels: this rank's own batch
    ids = [torch.randint(0, V, (B, M), generator=g, device=dev) for _ in range(n_ids)]
    labels = [torch.randint(0, V, (B * M,), generator=g, device=dev) for _ in range(n_ids)]
    loss_box, grads_box = [None], [None]

    def fwd_bwd(i):
        x = embed[ids[i % n_ids]]
        for layer, args in layers:
            x = layer(x, *args[1:])       # (no reference to x is kept: a stale autograd graph would outlive the step)
        logits = NormHead.apply(x)
        loss = torch.nn.functional.cross_entropy(logits.float(), labels[i % n_ids])
        grads_box[0] = torch.autograd.grad(loss, adapters)      # the 14 x n_layers adapter gradients of this rank ...
        reducer.finish()                                        # ... and their average over the ranks, left in .grad
        loss_box[0] = loss.detach()

    def step(i):
        fwd_bwd(i)
        return float(loss_box[0].item())      # the device-to-host read of the step's result
    for i in range(6):                         # calibration iterations of every layer
        step(i)
        if i < 5 and dist is not None:
            for layer, _ in layers:
                parallel.sync_calibration(layer.attn_state.static_value)
                parallel.sync_calibration(layer.mlp_state.static_value)
    mlp.check_status(status, "model step")
    torch.cuda.reset_peak_memory_stats(dev)
    t = time_loop(step, steps, warmup)
    peak_mem = torch.cuda.max_memory_allocated(dev)
    loss_value = step(0)
    world = 1
    if dist is not None:
        world = dist.get_world_size()
        tt = torch.tensor([t], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = float(tt.item())
    graph_ms = None
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fwd_bwd(0)
        torch.cuda.current_stream().wait_stream(side)
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            fwd_bwd(0)

        def replay(i):
            cg.replay()
            return float(loss_box[0].item())
        tg = time_loop(replay, steps, warmup)
        if dist is not None:
            tt = torch.tensor([tg], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            tg = float(tt.item())
        graph_ms = tg / steps * 1e3
        mlp.check_status(status, "model step (graph)")
    T = B * M
    per_layer = 4 * (4 * H * H + 3 * H * I) + 12 * M * heads * d + R * (48 * H + 18 * H + 22 * I)
    flop_per_token = n_layers * per_layer + 4 * H * V
    burst, sustained, src = tensor_peaks()
    tf = T * flop_per_token * steps / t / 1e12
    out = {"workload": "one training step fwd+bwd of the %d-layer Llama-2-7B stack (embedding, fused layers, final norm, "
                       "vocabulary projection, cross-entropy), random-init bf16, LoRA r=16 on all seven projections, q_bit 4, "
                       "seq 2048, batch 1 per GPU (BASELINE configs[4])" % n_layers,
           "metric": "tokens/s", "value": world * T * steps / t, "unit": "tokens/s", "ms_per_step": t / steps * 1e3,
           "tokens_per_gpu": T, "flop_per_token": flop_per_token, "cuda_graph_replay_ms_per_step": graph_ms,
           "loss": loss_value, "peak_memory_bytes": peak_mem,
           "identical_grads_on_all_ranks": ranks_hold_identical(reducer, dist),
           "lora_grad_exchange": {"buffer_bytes": 0 if reducer.flat is None else reducer.flat.numel() * 4,
                                  "all_reduces_per_step": len(reducer._bucket_range)},
           "roofline": {"bound": "tensor", "achieved": tf, "peak": sustained, "unit": "TFLOP/s", "frac": tf / sustained,
                        "peak_source": src + " (sustained)"},
           "note": "embedding lookup and the cross-entropy are torch glue; every other launch is a kernel of this library "
                   "except the batched attention products and the rank-16 skinny products (library GEMMs)"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads and the CPU sample")
    ap.add_argument("--profile", default=None, choices=["attn_topk", "attn_bwd", "channel_q4", "channel_q2", "channel_q8", "mlp", "fused", "layer", "model", "prune"],
                    help="run only W+K steps of one workload and print timing (for a profiler capture)")
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of --profile model")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    if args.profile:
        return run_profile(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the kernels are sm_100a only; there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from hyc_lora_release_b200.operators import compress_function as cf
    hbm, peak_src = peaks()
    maps = [make_map(1000 + rank * NBUF + i, dev) for i in range(NBUF)]
    handles = [None] * NBUF
    dense = [None] * NBUF
    one_way = algo_bytes(MAP_SHAPE, QBIT, RATIO)

    # the saved maps and the restored maps live in rings of NBUF buffers that every step overwrites
    for j in range(NBUF):
        handles[j] = cf.compression_softmax_topk(maps[j], RATIO, QBIT)
        dense[j] = handles[j].to_dense()

    def step(i):
        # one step = ROUND_TRIPS save/restore round trips over the ring of maps (a step is milliseconds, not microseconds)
        for r in range(ROUND_TRIPS):
            j = (i * ROUND_TRIPS + r) % NBUF
            cf.compression_softmax_topk(maps[j], RATIO, QBIT, out=handles[j])
            handles[j].to_dense(out=dense[j])

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    secs = e0.elapsed_time(e1) / 1e3
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        t = torch.tensor([secs], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    value = world * args.steps * ROUND_TRIPS * 2 * one_way / secs / 1e9

    # per-kernel durations of the two kernels (CUDA events on the launching stream)
    # (one pass over the NBUF buffer sets captured in a CUDA graph, so that the average is the kernel's and
    # not the host's launch rate)
    def graph_avg(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for j in range(NBUF):
                fn(j)
        n_rep = 25
        return time_loop(lambda i: g.replay(), n_rep, 3) / (n_rep * NBUF)
    t_c = graph_avg(lambda j: cf.compression_softmax_topk(maps[j], RATIO, QBIT, out=handles[j]))
    t_d = graph_avg(lambda j: handles[j].to_dense(out=dense[j]))
    dom, t_dom = (("hyc::topk_lane_compress_kernel<4,8>", t_c) if t_c >= t_d
                  else ("hyc::topk_lane_restore_kernel<4,8,false>", t_d))
    achieved = one_way / t_dom / 1e9

    # end to end: pinned host map -> device -> compress -> decompress -> pinned host map, every step through the
    # public operators.  Steps alternate between two streams (each with its own buffers), so that the
    # device-to-host copy of one step overlaps the host-to-device copy of the next: PCIe is full duplex.
    n_lanes = 4
    host_in = [m.cpu().pin_memory() for m in maps[:n_lanes]]
    host_out = [torch.empty(MAP_SHAPE, dtype=torch.bfloat16).pin_memory() for _ in range(n_lanes)]
    dev_in = [torch.empty(MAP_SHAPE, dtype=torch.bfloat16, device=dev) for _ in range(n_lanes)]
    e_handles = [cf.compression_softmax_topk(maps[j], RATIO, QBIT) for j in range(n_lanes)]
    e_dense = [torch.empty(MAP_SHAPE, dtype=torch.bfloat16, device=dev) for _ in range(n_lanes)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(n_lanes)]

    def e2e_step(i):
        j = i % n_lanes
        with torch.cuda.stream(streams[j]):
            dev_in[j].copy_(host_in[j], non_blocking=True)
            cf.compression_softmax_topk(dev_in[j], RATIO, QBIT, out=e_handles[j])
            e_handles[j].to_dense(out=e_dense[j])
            host_out[j].copy_(e_dense[j], non_blocking=True)

    def e2e_loop(steps, warm):
        cur = torch.cuda.current_stream()
        for i in range(warm):
            e2e_step(i)
        for s_ in streams:
            cur.wait_stream(s_)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(cur)
        for s_ in streams:
            s_.wait_event(a)
        for i in range(steps):
            e2e_step(i)
        for s_ in streams:
            cur.wait_stream(s_)
        b.record(cur)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 1e3
    n_e = max(8, min(args.steps, 32))        # one map per end-to-end step (PCIe-bound: about 1.5 ms each)
    barrier()
    t_e = e2e_loop(n_e, 4)
    if dist is not None:
        t = torch.tensor([t_e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_e = float(t.item())
    if not torch.equal(host_out[0], dense[0].cpu()):
        raise RuntimeError("the end-to-end result differs from the device-resident run")
    dense_bytes = maps[0].numel() * 2
    e2e = {"value": world * n_e * 2 * one_way / t_e / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": dense_bytes, "d2h_bytes_per_step": dense_bytes, "steps": n_e,
           "round_trips_per_step": 1,
           "api": "compress_function.compression_softmax_topk + TopkMap.to_dense on pinned host maps, four streams "
                  "(the read-back of one step overlaps the upload of the next)"}

    mlp_line = layer_line = model_line = None
    sweep_lines = []
    if not args.no_extras:
        barrier()
        mlp_line = mlp_workload(dev, dist, eager=(world == 1))      # every rank takes part (all-reduce inside)
        sweep_lines = []
        for qb in (2, 4, 8):
            barrier()
            sweep_lines.append(mlp_workload(dev, dist, steps=40, warmup=3, shape="mistral", q_bit=qb))
        barrier()
        layer_line = layer_workload(dev, dist)
        barrier()
        model_line = model_workload(dev, dist)
    if rank == 0:
        also, cpu = [], None
        if not args.no_extras and world == 1:
            also = extra_workloads(dev, hbm)
            cpu = cpu_baseline_sample()
        if mlp_line is not None:
            also.append(mlp_line)
        also.extend(sweep_lines)
        if layer_line is not None:
            also.append(layer_line)
        if model_line is not None:
            also.append(model_line)
        line = {
            "metric": "activation compress+decompress GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16->u8",
            "data": "synthetic", "config": config_dict(), "clocks": clocks, "e2e": e2e,
            "gpu_launches": 2 * ROUND_TRIPS * args.steps,
            "frac_of_hbm_peak": value / world / hbm,
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": hbm, "unit": "GB/s",
                         "frac": achieved / hbm, "peak_source": peak_src,
                         "traffic": NCU_TRAFFIC.get(dom),
                         "algorithmic_bytes_per_launch": one_way,
                         "kernel_ms": {"compress": t_c * 1e3, "decompress": t_d * 1e3}},
            "cpu_baseline": cpu, "mlp": mlp_line, "also": also,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
