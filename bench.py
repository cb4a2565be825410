"""Benchmark of the quantized MatMul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows M]

One JSON line on stdout (rank 0). Metric: quantized MatMul weight GB/s = weight bytes streamed per second, the figure the
reference's own benchmark reports (tests/Sharplight.Cpu.Tests/BenchTests.cs:82-99 of the Sharplight tree).

The workload is the same at every N, so the per-N values form a strong-scaling curve: benchmark configuration 5, the
quantized MatMuls of a Llama-3-70B-shaped layer stack (80 layers, Q4_K, 38.5 GB of weights: it fits one B200), at
decode batch M = --rows (default 1), tensor parallel over the N GPUs -- q/k/v and gate/up column-split (stacked into
one MatMul each), o and down row-split with the f32 partial outputs summed over the ranks. One step = every MatMul of
every layer once, activation quantization included.
  value    : device-resident inputs and outputs, the step replayed as one CUDA graph, timed with CUDA events on the
             launching stream, max over ranks; 38.5 GB / step time.
  e2e      : the same step through the provider API (one compiled segment: SetInput / Execute / GetOutput) with HOST
             buffers: host->device copy of the four activation inputs and a device->host copy of every MatMul output
             into the caller's array, inside the timed region.
  roofline : the dominant kernel alone -- benchmark configuration 2's Q4_K [14336, 4096] mat-vec at M = 1 on
             pre-quantized activations -- algorithmic bytes / measured launch time against the measured HBM peak.
  configs  : (N = 1) every other benchmark configuration: configuration 1 (Q8_0 [3072, 1024]), configuration 2 at
             M = 1 / 4 / 16 / 64, configuration 3 (Q4_0 prefill GEMM, with its own roofline, e2e and CPU baseline),
             configuration 4 (8B decode step at batch 32, with a per-MatMul breakdown).
  tp_stack : the stack at M = 1 / 8 / 64 and the 2048-row prefill.
  cpu_baseline : the CPU restatement of the reference's MatMul (oracle/) on the host cores, bounded sample.
With --impl reference the CPU arm is the measured one (the reference's managed CPU provider cannot be built here: no
.NET toolchain; the restatement is labelled "port").
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NOMINAL_INT8_TOPS = 4500.0
KERNEL_NAMES = {1: "mmvq (dp4a)", 2: "skinny (int8 mma.sync)", 3: "mmq (tcgen05 kind::i8)", 4: "tile (tcgen05 kind::i8, stream-K)"}
# dram__bytes_read.sum + dram__bytes_write.sum of one mat-vec launch on configuration 2 at M = 1, from one ncu capture
# of this kernel (the algorithmic bytes are 33 092 608); quoted only while the kernel family of the run is the captured one
CONFIG2_M1_DRAM_BYTES = 33071872


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "source": "fallback"}
    if os.path.exists(path):
        try:
            j = json.load(open(path))
            out = {"hbm_gbs": float(j["hbm_gbs"]), "bf16_tflops": float(j["bf16_tflops"]), "source": "measured (MEASURED_PEAKS.json)"}
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _once(self):
        nv = self._nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
        try:
            bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
        except Exception:
            bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
                 0x80: "hw_power_brake"}
        for bit, name in names.items():
            if bits & bit:
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._once()
            except Exception:
                return
            self._stop.wait(0.01)

    def start(self):
        if self._nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- the CPU arm -----------------------------------------------------------------------------------------------------

def cpu_p10(fn, budget_s: float, min_runs: int = 3, want_runs: int = 30, warmups: int = 5):
    """The reference's timing rule (tests/Sharplight.Cpu.Tests/BenchTests.cs:82-99): warm-ups, then the 10th percentile of
    at least 30 runs -- cut short (never below min_runs) when the time budget of this bounded sample runs out."""
    t_w = time.perf_counter()
    for i in range(warmups):
        fn()
        if time.perf_counter() - t_w > 0.25 * budget_s and i >= 1:
            break
    times = []
    t0 = time.perf_counter()
    while len(times) < want_runs:
        a = time.perf_counter()
        fn()
        times.append(time.perf_counter() - a)
        if time.perf_counter() - t0 > budget_s and len(times) >= min_runs:
            break
    return float(np.percentile(times, 10)), len(times)


def cpu_stack_baseline(rows: int, seconds: float):
    """The 70B-shaped stack on the host cores: the four MatMuls of one layer (stacked qkv, o, stacked gate_up, down; 481 MB
    of Q4_K blocks, full size), driven as the reference's CPU provider drives them -- integer dots in
    clamp(N / 16, 1, 4 x threads) chunks on a spinning worker pool below 32 rows, the f32 GEMM from 32 rows
    (src/Sharplight.Cpu/MatMulOp.cs:125-213) -- p10 per MatMul, summed; weight GB/s."""
    from oracle import sl_oracle
    from sharplight_b200 import synth, tp
    threads = os.cpu_count() or 1
    mats = []
    for i, (name, parts, k, _, _) in enumerate(tp.fused_layer_matmuls(tp.LLAMA70B)):
        n = sum(parts)
        mats.append((name, synth.weight_blocks("Q4_K", n, k, seed=400 + i), n, k, synth.activations(rows, k, seed=410 + i)))
    layer_bytes = sum(synth.weight_bytes("Q4_K", n, k) for _, _, n, k, _ in mats)
    total, runs = 0.0, []
    for name, b, n, k, x in mats:
        p10, nruns = cpu_p10(lambda: sl_oracle.matmul_run(12, b, n, k, x, threads=threads), seconds / len(mats))
        total += p10
        runs.append(nruns)
    gbs = layer_bytes / total / 1e9
    path = "f32 GEMM (" + sl_oracle.gemm_tile_name() + ")" if rows >= 32 else "integer dots (" + sl_oracle.fast_tier_name() + ")"
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "path": path,
            "sample": f"one layer's four MatMuls at full size ({layer_bytes / 1e6:.0f} MB of Q4_K blocks) at M={rows}, p10 of "
                      f"{min(runs)}-{max(runs)} runs each after warm-ups, {threads} threads; the stack's step time is 80 x the layer's"}, gbs


def cpu_matmul_baseline(type_name: str, n: int, k: int, rows: int, seconds: float):
    """One MatMul shape on the host cores through the reference's row-count dispatch; (seconds per MatMul p10, runs)."""
    from oracle import sl_oracle
    from sharplight_b200 import synth
    fmt = {"Q4_0": 2, "Q8_0": 8, "Q4_K": 12, "Q6_K": 14}[type_name]
    threads = os.cpu_count() or 1
    b = synth.weight_blocks(type_name, n, k, seed=77)
    x = synth.activations(rows, k, seed=78)
    p10, runs = cpu_p10(lambda: sl_oracle.matmul_run(fmt, b, n, k, x, threads=threads), seconds)
    return p10, runs, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import sl_oracle  # noqa: F401  (the reference arm is the one place besides the baseline leg that runs oracle/)
    from sharplight_b200 import tp
    seconds = max(8.0, min(60.0, 0.5 * (args.steps + args.warmup)))
    base, gbs = cpu_stack_baseline(args.rows, seconds)
    total = tp.layer_weight_bytes(tp.LLAMA70B) * tp.LLAMA70B["layers"]
    line = {"impl": "reference", "metric": "quant MatMul weight GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / (gbs * 1e9) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
            "config": {"workload": stack_workload_name(args.rows, 1) + " -- on the host cores (the CPU has no tensor "
                                   "parallelism: one socket, all threads); bounded sample, step time extrapolated to the 38.5 GB stack"},
            "cpu_baseline": base,
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement (oracle/) of the reference's Sharplight.Cpu MatMul; the managed reference cannot be built "
                    "here (no .NET toolchain)"}
    print(json.dumps(line), flush=True)


def stack_workload_name(rows: int, world: int) -> str:
    return (f"configs[4]: Llama-3-70B-shaped layer stack, 80 layers, Q4_K (38.5 GB), decode M={rows}, tensor parallel x{world}: "
            "column-split stacked q/k/v and gate/up, row-split o/down with the f32 partial outputs summed over the ranks")


# ---- GPU legs --------------------------------------------------------------------------------------------------------

class TpStack:
    """benchmark configuration 5: the quantized MatMuls of a Llama-3-70B-shaped layer stack, tensor-parallel over the
    ranks: q / k / v / gate / up column-split (stacked into one qkv and one gate_up MatMul per layer), o / down row-split
    with an all-reduce (sum) of the f32 partial outputs.
    Attention, norms and the activation function are not on the path: the inputs of o and down are fresh synthetic
    activations of the sharded shape. One step = every MatMul of every layer once, for `rows` activation rows (any
    count up to max_rows: decode batches and the prefill run on the same stack)."""

    IN_KERNEL_ROWS = 16   # measured on 8 GPUs: in-kernel sum 2.2x faster than NCCL at 1 row, 1.5x at 8, 0.9x at 64

    def __init__(self, device, torch, dist, N, synth, rank, world, max_rows, layers, arch, type_name="Q4_K"):
        from sharplight_b200 import MatMulOp, SharedActivation, TpComm, TpExchange, tp
        self.torch, self.dist, self.N, self.world, self.device = torch, dist, N, world, device
        self.exchange, self.comm = None, None
        if world > 1:
            # the receive area of the in-kernel all-reduce (one serves o and down of every layer: same output width), and
            # the library's own NCCL communicator for the row counts above it
            self.exchange = TpExchange(device, rank, world, N.TP_MAX_ROWS, arch["hidden"])
            self.exchange.connect_group(dist)
            self.comm = TpComm.for_group(device, dist)
            self.exchange.set_comm(self.comm, self.IN_KERNEL_ROWS)
            dist.barrier()
        rows = max_rows
        self.layers, self.arch, self.type_name = layers, arch, type_name
        self.specs = [(name, sum(parts), k, split, inp) for name, parts, k, split, inp in tp.fused_layer_matmuls(arch)]
        self.total_weight_bytes = tp.layer_weight_bytes(arch, type_name) * layers
        self.weights, self.ops, self.layer_weights = [], [], []
        shard_blocks = {}
        for name, parts, k, split, _ in tp.fused_layer_matmuls(arch):
            nl, kl = tp.fused_shard_shape(parts, k, split, rank, world, type_name, arch["head_dim"])
            shard_blocks[name] = (synth.weight_blocks(type_name, nl, kl, seed=500 + 7 * rank + len(shard_blocks)), nl, kl)
        for _ in range(layers):
            layer_ops, layer_w = {}, {}
            for name, (blocks, nl, kl) in shard_blocks.items():
                w = device.upload_weight(type_name, (nl, kl), blocks)
                self.weights.append(w)
                layer_w[name] = w
                layer_ops[name] = MatMulOp(device, w, rows)
            self.ops.append(layer_ops)
            self.layer_weights.append(layer_w)
        self.dims = {name: (nl, kl) for name, (_, nl, kl) in shard_blocks.items()}
        dims = self.dims
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        mk = lambda r, c: torch.randn((r, c), generator=g, device="cuda", dtype=torch.float32)
        h = arch["hidden"]
        self.x = {"x_attn": mk(rows, h), "x_ffn": mk(rows, h), "x_o": mk(rows, dims["o"][1]), "x_down": mk(rows, dims["down"][1])}
        self.y = {name: torch.empty((rows, dims[name][0]), device="cuda", dtype=torch.float32) for name in dims}
        self.act = {key: SharedActivation(device, rows, v.shape[1]) for key, v in self.x.items()}
        self.launches_per_step = 0

    def step(self, rows, sp, in_kernel=None):
        """Row-split MatMuls go through the exchange: the library sums over the ranks inside the MatMul kernel (peer stores
        over NVLink) up to IN_KERNEL_ROWS rows and by its NCCL communicator above. in_kernel = True / False moves that
        threshold to 64 / 0 rows for this step (the comparison legs)."""
        N = self.N
        launches = 0
        if self.exchange is not None:
            self.exchange.set_comm(self.comm, self.IN_KERNEL_ROWS if in_kernel is None else N.TP_MAX_ROWS if in_kernel else 0)
        for layer_ops in self.ops:
            for key in ("x_attn", "x_o", "x_ffn", "x_down"):
                x = self.x[key]
                # every input of this stack has one consumer (q/k/v and gate/up are stacked): the rows are handed over as
                # they are and the library quantizes them at that MatMul -- inside the mat-vec kernel when K is a short
                # tensor-parallel shard, through the quantizer kernel otherwise (counted in the MatMul's launches)
                self.act[key].set_rows(x.data_ptr(), N.F32, rows, x.shape[1], sp)
                for name, _, _, split, inp in self.specs:
                    if inp != key:
                        continue
                    y = self.y[name]
                    if split == "row" and self.exchange is not None:
                        self.exchange.matmul(layer_ops[name], self.act[key], y.data_ptr(), y.shape[1], sp)
                    else:
                        self.act[key].matmul(layer_ops[name], y.data_ptr(), y.shape[1], sp)
                    launches += layer_ops[name].last_kernel()[1]
        self.launches_per_step = launches

    def segment(self, max_rows: int):
        """The same stack as one compiled segment of the provider API, on the weights already resident: four host inputs,
        every MatMul's output a host output; row-split nodes sum over the ranks through the stack's exchange."""
        from sharplight_b200 import CompileOptions, GraphSegment, MatMulNode, WeightInfo
        nodes, outputs = [], []
        for li, layer_w in enumerate(self.layer_weights):
            for name, _, _, split, inp in self.specs:
                nl, kl = self.dims[name]
                out = f"{name}{li}"
                nodes.append(MatMulNode(out, inp, WeightInfo(self.type_name, (nl, kl), None, resident=layer_w[name]), out,
                                        allreduce=(split == "row" and self.world > 1)))
                outputs.append(out)
        seg = self.device.compile(GraphSegment(nodes, ["x_attn", "x_o", "x_ffn", "x_down"], outputs),
                                  CompileOptions(max_rows=max_rows, exchange=self.exchange))
        return seg, outputs

    def dispose(self):
        if self.exchange is not None:
            self.torch.cuda.synchronize()
            self.dist.barrier()
            self.exchange.dispose()
            self.comm.dispose()
        for layer_ops in self.ops:
            for op in layer_ops.values():
                op.dispose()
        for w in self.weights:
            w.dispose()
        for a in self.act.values():
            a.dispose()


def time_graphed(torch, dist, world, stream, fn, steps, warmup, use_graph=True):
    """fn(stream_ptr) captured into a CUDA graph and replayed; returns ms per step (max over ranks)."""
    for _ in range(2):
        fn(stream.cuda_stream)
    torch.cuda.synchronize()
    run = lambda: fn(stream.cuda_stream)
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=torch.cuda.Stream()):
            fn(torch.cuda.current_stream().cuda_stream)
        run = graph.replay
    for _ in range(warmup):
        run()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        run()
    e1.record(stream)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def stack_e2e(args, torch, dist, world, stack, rows, steps):
    """The stack's step through the provider API with host buffers: SetInput of the four activation inputs (pinned
    staging, host->device), Execute (one quantization per input and layer, every MatMul; a captured graph from the third
    call), GetOutput of every MatMul's result copied into the caller's array."""
    seg, outputs = stack.segment(rows)
    xs = {k: v[:rows].cpu().numpy() for k, v in stack.x.items()}
    got = {}

    def step_host():
        for k, v in xs.items():
            seg.set_input(k, v)
        seg.execute({"T": rows})
        for name in outputs:
            got[name] = seg.get_output(name, copy=True)

    for _ in range(4):
        step_host()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step_host()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / steps   # every step ends with a host-side wait: wall clock is the device's clock here
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # what was timed equals the device-resident path: the last layer's outputs against the graph-replayed stack's
    stack.step(rows, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    last = len(stack.layer_weights) - 1
    same = bool(all(np.array_equal(got[f"{name}{last}"], stack.y[name][:rows].cpu().numpy()) for name in stack.dims))
    h2d = sum(v.nbytes for v in xs.values())
    d2h = sum(rows * stack.dims[name][0] * 4 for name in stack.dims) * len(stack.layer_weights)
    seg.dispose()
    return ms, h2d, d2h, same


def kernel_times(torch, device, N, synth, stream, type_name, n, k, rows, copies, steps, distinct=True, kernel=None, use_graph=True):
    """One MatMul shape over `copies` weight matrices (distinct: rotating copies, so the weights come from HBM; else
    the same matrix every time: L2-resident when it fits). Returns seconds per MatMul for (operator = quantize + kernel,
    each launch waiting for its predecessor; kernel: the step quantizes once and the `copies` MatMuls share that one
    quantization, so their launches are free to run beside each other -- the quantization's 1/copies share is inside
    the figure), and the kernel family."""
    from sharplight_b200 import MatMulOp, SharedActivation
    base = synth.weight_blocks(type_name, n, k, seed=100 + n % 97)
    nw = copies if distinct else 1
    ws = [device.upload_weight(type_name, (n, k), np.roll(base.reshape(n, -1), i * 37, axis=0).reshape(-1)) for i in range(nw)]
    ops = [MatMulOp(device, ws[i % nw], rows) for i in range(copies)]
    if kernel is not None:
        for op in ops:
            op.set_kernel(kernel)
    x = torch.randn((rows, k), device="cuda", dtype=torch.float32)
    y = torch.empty((copies, rows, n), dtype=torch.float32, device="cuda")
    act = SharedActivation(device, rows, k)

    def op_step(sp):
        for i, op in enumerate(ops):
            op.run_pointers(x.data_ptr(), N.F32, rows, k, True, y[i].data_ptr(), n, True, sp)

    def kern_step(sp):
        # one quantization at the head of the step, on the step's stream: the MatMuls that share it may then run beside
        # each other (as the MatMuls of a layer that read the same input do)
        act.quantize(x.data_ptr(), N.F32, rows, k, sp)
        for i, op in enumerate(ops):
            act.matmul(op, y[i].data_ptr(), n, sp)

    t_op = time_graphed(torch, None, 1, stream, op_step, steps, 3, use_graph=use_graph) * 1e-3 / copies
    t_k = time_graphed(torch, None, 1, stream, kern_step, steps, 3, use_graph=use_graph) * 1e-3 / copies
    family, launches = ops[0].last_kernel()
    for op in ops:
        op.dispose()
    for w in ws:
        w.dispose()
    act.dispose()
    return t_op, t_k, family, launches


def hbm_entry(peaks, type_name, n, k, rows, t_op, t_k, family, synth):
    wbytes = synth.weight_bytes(type_name, n, k)
    algo = wbytes + rows * k + rows * (k // 32) * 8 + rows * n * 4
    return {"kernel_us": t_k * 1e6, "operator_us": t_op * 1e6, "achieved": algo / t_k / 1e9, "unit": "GB/s",
            "frac": algo / t_k / 1e9 / peaks["hbm_gbs"], "operator_frac": algo / t_op / 1e9 / peaks["hbm_gbs"],
            "algorithmic_bytes_per_launch": algo, "kernel_family": KERNEL_NAMES.get(family, str(family))}


def config_legs(args, torch, device, N, synth, stream, peaks):
    """Configurations 1 and 2 (HBM-bound mat-vec / skinny shapes): kernel and operator time, achieved GB/s over the
    algorithmic bytes, fraction of the measured HBM peak."""
    steps = max(5, min(args.steps, 20))
    out = {}
    c1 = {}
    t_op, t_k, fam, _ = kernel_times(torch, device, N, synth, stream, "Q8_0", 3072, 1024, 1, 48, steps, distinct=True)
    c1["rotating_48_copies_160MB"] = hbm_entry(peaks, "Q8_0", 3072, 1024, 1, t_op, t_k, fam, synth)
    t_op, t_k, fam, _ = kernel_times(torch, device, N, synth, stream, "Q8_0", 3072, 1024, 1, 48, steps, distinct=False)
    c1["l2_resident"] = hbm_entry(peaks, "Q8_0", 3072, 1024, 1, t_op, t_k, fam, synth)
    c1["workload"] = "configs[0]: Q8_0 [3072,1024] mat-vec, M=1; 3.3 MB of weights per launch (time floor 0.51 us at the measured peak: launch latency dominates)"
    out["config1"] = c1
    c2 = {"workload": "configs[1]: Q4_K [14336,4096], 32 rotating weight copies (1057 MB > L2)"}
    for rows in (1, 4, 16, 64):
        t_op, t_k, fam, _ = kernel_times(torch, device, N, synth, stream, "Q4_K", 14336, 4096, rows, 32, steps)
        c2[f"M={rows}"] = hbm_entry(peaks, "Q4_K", 14336, 4096, rows, t_op, t_k, fam, synth)
    out["config2"] = c2
    return out


def prefill_leg(args, device, torch, N, synth, stream, peaks, with_cpu):
    """benchmark configuration 3: Q4_0 [4096, 4096], bf16 activations [2048, 4096], the tensor-core GEMM.
    Operator time = quantization + GEMM (what the reference's published TFLOPS include,
    tests/Sharplight.Vulkan.Tests/BenchTests.cs:28-46); kernel time = the GEMM alone on quantized activations; e2e = one
    compiled segment with host bf16 activations in and host f32 results out."""
    from sharplight_b200 import CompileOptions, GraphSegment, MatMulNode, MatMulOp, SharedActivation, WeightInfo
    from sharplight_b200.provider import to_bf16_bits
    n, k, m, copies = 4096, 4096, 2048, 8
    steps = max(5, args.steps // 4)
    base = synth.weight_blocks("Q4_0", n, k, seed=300)
    ws = [device.upload_weight("Q4_0", (n, k), np.roll(base.reshape(n, -1), 11 * i, axis=0).reshape(-1)) for i in range(copies)]
    ops = [MatMulOp(device, w, m) for w in ws]
    x_bits = to_bf16_bits(synth.activations(m, k, seed=301))
    x = torch.from_numpy(x_bits.view(np.int16)).cuda()
    y = torch.empty((copies, m, n), dtype=torch.float32, device="cuda")
    act = SharedActivation(device, m, k)

    def op_step(sp):
        for i, op in enumerate(ops):
            op.run_pointers(x.data_ptr(), N.BF16, m, k, True, y[i].data_ptr(), n, True, sp)

    def gemm_step(sp):
        for i, op in enumerate(ops):
            act.matmul(op, y[i].data_ptr(), n, sp)

    t_op = time_graphed(torch, None, 1, stream, op_step, steps, 3) * 1e-3 / copies
    act.quantize(x.data_ptr(), N.BF16, m, k, stream.cuda_stream)
    t_gemm = time_graphed(torch, None, 1, stream, gemm_step, steps, 3) * 1e-3 / copies
    family, _ = ops[0].last_kernel()
    ops_count = 2.0 * m * n * k
    tops = ops_count / t_gemm / 1e12
    # e2e: one segment holding the eight MatMuls, host bf16 in, host f32 out
    nodes = [MatMulNode(f"mm{i}", "x", WeightInfo("Q4_0", (n, k), None, resident=ws[i]), f"y{i}", x_dtype="bf16") for i in range(copies)]
    seg = device.compile(GraphSegment(nodes, ["x"], [f"y{i}" for i in range(copies)]), CompileOptions(max_rows=m))
    got = [None] * copies

    def step_host():
        seg.set_input("x", x_bits)
        seg.execute({"T": m})
        for i in range(copies):
            got[i] = seg.get_output(f"y{i}", copy=True)

    for _ in range(4):
        step_host()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e_steps = max(3, steps // 2)
    for _ in range(e_steps):
        step_host()
    torch.cuda.synchronize()
    t_e2e = (time.perf_counter() - t0) / (e_steps * copies)
    same = bool(np.array_equal(got[0], y[0].cpu().numpy()))
    seg.dispose()
    ceiling = 1100.0
    out = {"workload": "configs[2]: Q4_0 [4096,4096] x bf16 [2048,4096], 8 rotating weight copies",
           "operator_tops": ops_count / t_op / 1e12, "gemm_kernel_tops": tops,
           "operator_us": t_op * 1e6, "gemm_kernel_us": t_gemm * 1e6,
           "kernel_family": KERNEL_NAMES.get(family, str(family)),
           "block_scale_fmas": m * n * (k // 32),
           "roofline": {"bound": "tensor", "achieved": tops, "unit": "TOP/s", "peak": NOMINAL_INT8_TOPS,
                        "frac": tops / NOMINAL_INT8_TOPS, "peak_source": "nominal dense int8 (no int8 figure in MEASURED_PEAKS.json)",
                        "frac_of_2x_measured_bf16": tops / (2.0 * peaks["bf16_tflops"]),
                        "ceiling_tops": ceiling, "frac_of_ceiling": tops / ceiling,
                        "ceiling": "two f32 operations per (row, token, 32-block) on the CUDA cores -- per-block f16 weight "
                                   "scale x f32 activation scale -- at 128 per clock per SM",
                        "traffic": None},
           "e2e": {"value": ops_count / t_e2e / 1e12, "unit": "TOP/s", "h2d_bytes_per_step": int(x_bits.nbytes),
                   "d2h_bytes_per_step": copies * m * n * 4, "us_per_matmul": t_e2e * 1e6, "equals_device_path": same,
                   "note": "host bf16 activations in (16.8 MB once per 8 MatMuls), host f32 results out (33.6 MB per MatMul): the "
                           "copies over PCIe dominate"}}
    if with_cpu:
        p10, runs, threads = cpu_matmul_baseline("Q4_0", n, k, m, 12.0)
        from oracle import sl_oracle
        out["cpu_baseline"] = {"value": ops_count / p10 / 1e12, "unit": "TOP/s (2 M N K / t; the CPU runs them as f32 FLOPs)",
                               "cores": threads, "kind": "port", "ms_per_matmul": p10 * 1e3,
                               "sample": f"p10 of {runs} runs of the reference's f32 GEMM path ({sl_oracle.gemm_tile_name()} micro-kernel, "
                                         "weights dequantized per 256-value slice) on this shape"}
    for op in ops:
        op.dispose()
    for w in ws:
        w.dispose()
    act.dispose()
    return out


def decode_step_leg(args, torch, dist, device, N, synth, stream, peaks):
    """benchmark configuration 4: every quantized MatMul of one decode step of a Llama-3-8B-shaped model on one GPU, a
    continuous batch of 32 sequences: 32 layers of Q4_K weights (qkv, o, gate_up, down) and the Q6_K lm_head
    [128256, 4096]. Attention, norms and sampling are not on the path. With the time of every MatMul type alone."""
    from sharplight_b200 import MatMulOp, SharedActivation, tp
    arch, rows = tp.LLAMA8B, 32
    stack = TpStack(device, torch, dist, N, synth, 0, 1, rows, arch["layers"], arch)
    vocab, h = 128256, arch["hidden"]
    head_w = device.upload_weight("Q6_K", (vocab, h), synth.weight_blocks("Q6_K", vocab, h, seed=900))
    head = MatMulOp(device, head_w, rows)
    head_act = SharedActivation(device, rows, h)
    x = torch.randn((rows, h), device="cuda", dtype=torch.float32)
    logits = torch.empty((rows, vocab), device="cuda", dtype=torch.float32)

    def step(sp):
        stack.step(rows, sp)
        head_act.quantize(x.data_ptr(), N.F32, rows, h, sp)
        head_act.matmul(head, logits.data_ptr(), vocab, sp)

    steps = max(3, min(args.steps, 20))
    ms = time_graphed(torch, dist, 1, stream, step, steps, 3, use_graph=not args.no_graph)
    wbytes = stack.total_weight_bytes + synth.weight_bytes("Q6_K", vocab, h)
    # per-MatMul breakdown: the stack's own ops of one type in turn over the 32 layers (distinct weights), kernel + quantize
    breakdown = {}
    for name, n, k, _, inp in stack.specs:
        def one(sp, name=name, inp=inp):
            xx = stack.x[inp]
            for layer_ops in stack.ops:
                stack.act[inp].quantize(xx.data_ptr(), N.F32, rows, xx.shape[1], sp)
                stack.act[inp].matmul(layer_ops[name], stack.y[name].data_ptr(), stack.y[name].shape[1], sp)
        t = time_graphed(torch, dist, 1, stream, one, steps, 2) * 1e-3 / arch["layers"]
        wb = synth.weight_bytes("Q4_K", n, k)
        breakdown[name] = {"shape": [n, k], "operator_us": t * 1e6, "weight_gbs": wb / t / 1e9, "frac": wb / t / 1e9 / peaks["hbm_gbs"],
                           "kernel_family": KERNEL_NAMES.get(stack.ops[0][name].last_kernel()[0])}

    def head_only(sp):
        head_act.quantize(x.data_ptr(), N.F32, rows, h, sp)
        head_act.matmul(head, logits.data_ptr(), vocab, sp)
    t = time_graphed(torch, dist, 1, stream, head_only, steps, 2) * 1e-3
    wb = synth.weight_bytes("Q6_K", vocab, h)
    breakdown["lm_head"] = {"shape": [vocab, h], "format": "Q6_K", "operator_us": t * 1e6, "weight_gbs": wb / t / 1e9,
                            "frac": wb / t / 1e9 / peaks["hbm_gbs"], "kernel_family": KERNEL_NAMES.get(head.last_kernel()[0])}
    out = {"workload": "configs[3]: Llama-3-8B-shaped decode step, 32 layers Q4_K + Q6_K lm_head, batch 32, one GPU",
           "ms_per_step": ms, "weight_gbs": wbytes / (ms * 1e-3) / 1e9, "frac": wbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
           "weight_bytes_per_step": wbytes, "sequences_per_s": rows / (ms * 1e-3),
           "launches_per_step": stack.launches_per_step + 2, "steps": steps, "per_matmul": breakdown}
    head_act.dispose(); head.dispose(); head_w.dispose(); stack.dispose()
    torch.cuda.synchronize()
    return out


def extras_leg(args, torch, device, N, synth, stream, peaks):
    """The kernels on either side of the MatMul (producers of the 8-bit activations, arg-max) and the f32-activation
    mat-vec: microseconds per launch inside a replayed graph of 32 launches."""
    from sharplight_b200 import MatMulOp, SharedActivation
    steps = max(5, min(args.steps, 20))
    reps = 32
    out = {}

    def timed(fn):
        return time_graphed(torch, None, 1, stream, lambda sp: [fn(sp) for _ in range(reps)], steps, 3) * 1e3 / reps

    for rows, k in ((1, 8192), (32, 4096)):
        x = torch.randn((rows, k), device="cuda")
        w = torch.ones((k,), device="cuda")
        act = SharedActivation(device, rows, k)
        out[f"quantize_{rows}x{k}_us"] = timed(lambda sp: act.quantize(x.data_ptr(), N.F32, rows, k, sp))
        out[f"rmsnorm_quantize_{rows}x{k}_us"] = timed(lambda sp: act.quantize_rmsnorm(x.data_ptr(), N.F32, rows, k, w.data_ptr(), 1e-5, 0, 0, sp))
        act.dispose()
    for rows, k in ((1, 28672), (32, 14336)):
        gu = torch.randn((rows, 2 * k), device="cuda")
        act = SharedActivation(device, rows, k)
        out[f"silu_mul_quantize_{rows}x{k}_us"] = timed(
            lambda sp: act.quantize_silu_mul(gu.data_ptr(), 2 * k, gu.data_ptr() + 4 * k, 2 * k, rows, 0, 0, sp))
        act.dispose()
    logits = torch.randn((32, 128256), device="cuda")
    idx = torch.empty((32,), dtype=torch.int32, device="cuda")
    out["argmax_32x128256_us"] = timed(lambda sp: device.argmax_rows(logits.data_ptr(), 32, 128256, 128256, idx.data_ptr(), sp))
    # f32-activation mat-vec on config 2's shape, 16 rotating weights
    n, k, copies = 14336, 4096, 16
    base = synth.weight_blocks("Q4_K", n, k, seed=77)
    ws = [device.upload_weight("Q4_K", (n, k), np.roll(base.reshape(n, -1), i * 37, axis=0).reshape(-1)) for i in range(copies)]
    wbytes = synth.weight_bytes("Q4_K", n, k)
    for rows in (1, 4):
        ops = [MatMulOp(device, wt, rows, f32_activations=True) for wt in ws]
        x = torch.randn((rows, k), device="cuda")
        y = torch.empty((copies, rows, n), device="cuda")
        ms = time_graphed(torch, None, 1, stream,
                          lambda sp: [op.run_pointers(x.data_ptr(), N.F32, rows, k, True, y[i].data_ptr(), n, True, sp) for i, op in enumerate(ops)],
                          steps, 3)
        us = ms * 1e3 / copies
        out[f"matvec_f32_q4k_14336x4096_M{rows}"] = {"us": us, "weight_gbs": wbytes / us / 1e3, "frac": wbytes / us / 1e3 / peaks["hbm_gbs"]}
        for op in ops:
            op.dispose()
    for wt in ws:
        wt.dispose()
    # the other served formats on the same shape at one row (MatMul launches only, one shared quantization): Q6_K natively;
    # Q5_0 / IQ4_NL as Q8_0 device records, Q5_K as two Q4_K weights (converted at upload)
    x = torch.randn((1, k), device="cuda")
    y = torch.empty((copies, 1, n), device="cuda")
    act = SharedActivation(device, 1, k)
    act.quantize(x.data_ptr(), N.F32, 1, k, stream.cuda_stream)
    more = {}
    for type_name in ("Q6_K", "Q5_K", "Q5_0", "IQ4_NL"):
        base = synth.weight_blocks(type_name, n, k, seed=78)
        ws = [device.upload_weight(type_name, (n, k), np.roll(base.reshape(n, -1), i * 37, axis=0).reshape(-1)) for i in range(copies)]
        ops = [MatMulOp(device, wt, 1) for wt in ws]
        ms = time_graphed(torch, None, 1, stream, lambda sp: [act.matmul(op, y[i].data_ptr(), n, sp) for i, op in enumerate(ops)], steps, 3)
        us = ms * 1e3 / copies
        src = synth.weight_bytes(type_name, n, k)
        more[type_name] = {"us": us, "file_format_gbs": src / us / 1e3, "device_bytes": ws[0].device_bytes, "launches": ops[0].last_kernel()[1]}
        for op in ops:
            op.dispose()
        for wt in ws:
            wt.dispose()
    act.dispose()
    out["more_formats_14336x4096_M1"] = more
    return out


def allreduce_check(stack, torch, dist, world, stream, row_counts):
    """The in-kernel sum against the collective library's, on the last layer's row-split outputs of one step, and across
    ranks (bit-identical everywhere), at row counts on both exchange protocols (word protocol up to 16 rows, arrival
    flags above)."""
    sp = stream.cuda_stream
    check = {}
    for rows in row_counts:
        stack.step(rows, sp, in_kernel=True)
        torch.cuda.synchronize()
        mine = {name: stack.y[name][:rows].clone() for name in ("o", "down")}
        stack.step(rows, sp, in_kernel=False)
        torch.cuda.synchronize()
        worst, same = 0.0, True
        for name, got in mine.items():
            ref = stack.y[name][:rows]
            worst = max(worst, float(((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()))
            everyone = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(everyone, got)
            same = same and all(torch.equal(everyone[0], e) for e in everyone[1:])
        t = torch.tensor([worst], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        check[rows] = {"max_diff_vs_nccl_over_max_abs": float(t.item()), "bit_identical_on_all_ranks": same}
    return check


def run_ours(args):
    import torch
    import torch.distributed as dist
    from sharplight_b200 import CudaExecutionProvider, synth, tp
    from sharplight_b200 import native as N

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    provider = CudaExecutionProvider()
    av = provider.check_availability()
    if not av.available:
        raise RuntimeError("CUDA provider unavailable (no CPU fallback): " + av.reason)
    device = provider.open_device([d for d in provider.get_devices() if d.index == local][0])
    peaks = measured_peaks()
    # an explicit (non-default) launching stream: kernels, CUDA events and graph replays all go to it
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    rows = args.rows
    warmup = max(args.warmup, 3)
    arch = tp.LLAMA70B
    layers = args.layers or arch["layers"]
    row_counts = sorted(set([rows] + ([] if args.tp_main_only else [1, 8, 64, 2048])))
    stack = TpStack(device, torch, dist, N, synth, rank, world, max(row_counts), layers, arch)
    flops_per_row = 2.0 * sum(n * k for _, n, k, _, _ in stack.specs) * layers

    # ---- the headline: the stack at M = rows, exactly --steps steps after --warmup warm-ups
    sampler = ClockSampler(local)
    sampler.start()
    ms_main = time_graphed(torch, dist, world, stream, lambda sp: stack.step(rows, sp), args.steps, warmup, use_graph=not args.no_graph)
    clocks = sampler.stop()
    launches_main = stack.launches_per_step
    families_main = {name: KERNEL_NAMES.get(stack.ops[0][name].last_kernel()[0]) for name in stack.dims}
    value = stack.total_weight_bytes / (ms_main * 1e-3) / 1e9

    check = None
    if world > 1:
        check = allreduce_check(stack, torch, dist, world, stream, [r for r in (1, 8, 33, 64) if r <= max(row_counts)])

    by_rows = {}
    for r in row_counts:
        steps = max(3, min(args.steps, 20 if r <= 64 else 5))
        ms = ms_main if r == rows else time_graphed(torch, dist, world, stream, lambda sp, r=r: stack.step(r, sp), steps, 3,
                                                    use_graph=not args.no_graph)
        in_kernel = world > 1 and r <= TpStack.IN_KERNEL_ROWS
        by_rows[r] = {"ms_per_step": ms, "weight_gbs": stack.total_weight_bytes / (ms * 1e-3) / 1e9,
                      "per_gpu_frac_of_hbm_peak": stack.total_weight_bytes / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                      "tops": flops_per_row * r / (ms * 1e-3) / 1e12, "steps": args.steps if r == rows else steps,
                      "launches_per_step": stack.launches_per_step if r != rows else launches_main,
                      "kernel_families": families_main if r == rows else
                                         {name: KERNEL_NAMES.get(stack.ops[0][name].last_kernel()[0]) for name in stack.dims},
                      "allreduce": "none" if world == 1 else "in the MatMul kernel (peer stores)" if in_kernel else "ncclAllReduce issued by the library",
                      "allreduces_per_step": 2 * layers if world > 1 else 0}
        if world > 1 and r >= 1024 and not args.tp_main_only:
            # prefill: the library's option of summing over ranks in chunks beside the GEMM, against its default (after it)
            stack.comm.set_chunking(1024)
            other = time_graphed(torch, dist, world, stream, lambda sp, r=r: stack.step(r, sp), steps, 3, use_graph=not args.no_graph)
            stack.comm.set_chunking(0)
            by_rows[r]["prefill_sum"] = "after the GEMM"
            by_rows[r]["ms_per_step_chunked"] = other
        if world > 1 and r <= N.TP_MAX_ROWS and not args.tp_main_only:
            other = time_graphed(torch, dist, world, stream, lambda sp, r=r: stack.step(r, sp, in_kernel=not in_kernel),
                                 steps, 3, use_graph=not args.no_graph)
            by_rows[r]["ms_per_step_nccl" if in_kernel else "ms_per_step_in_kernel"] = other

    # ---- end to end through the provider API with host buffers
    e2e = None
    if not args.no_e2e and rows <= N.TP_MAX_ROWS:
        e_steps = max(3, args.steps // 2)
        ms_e2e, h2d, d2h, same = stack_e2e(args, torch, dist, world, stack, rows, e_steps)
        e2e = {"value": stack.total_weight_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "steps": e_steps, "equals_device_path": same,
               "note": "one compiled segment of the provider API over the stack's MatMuls: SetInput of the four host activation "
                       "inputs, Execute, GetOutput of every MatMul's result into the caller's array (copy included); per rank. "
                       "The segment quantizes each input once and shares the 8-bit copy among the MatMuls that read it, as the "
                       "reference's lowering does, whereas `value` quantizes per layer"}
    tp_stack = {"workload": f"configs[4]: Llama-3-70B-shaped stack, {layers} layers, Q4_K, tensor parallel x{world}",
                "weight_bytes_per_step": stack.total_weight_bytes, "by_rows": by_rows}
    if check is not None:
        tp_stack["in_kernel_allreduce_check"] = check
    stack.dispose()
    torch.cuda.synchronize()

    line = None
    if rank == 0:
        line = {"metric": "quant MatMul weight GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": ms_main, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
                "config": {"workload": stack_workload_name(rows, world) +
                                       (" (inside the MatMul kernel over NVLink peer memory up to 16 rows, by an NCCL all-reduce above)" if world > 1 else ""),
                           "l2": f"inputs larger than L2: {stack.total_weight_bytes / world / 1e9:.1f} GB of weights per GPU per step vs 126 MB",
                           "launch": "host launches" if args.no_graph else "CUDA graph replay of the step"},
                "gpu_launches": launches_main * args.steps, "clocks": clocks, "tp_stack": tp_stack,
                "stack_frac_of_hbm_peak": value / world / peaks["hbm_gbs"]}
        if e2e is not None:
            line["e2e"] = e2e

    # ---- the dominant kernel's roofline, and the other benchmark configurations (one GPU)
    if world == 1:
        t_op, t_k, fam, _ = kernel_times(torch, device, N, synth, stream, "Q4_K", 14336, 4096, 1, 32, max(args.steps, 10))
        wbytes = synth.weight_bytes("Q4_K", 14336, 4096)
        algo = wbytes + 4096 + (4096 // 32) * 8 + 14336 * 4
        achieved = algo / t_k / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                            "traffic": CONFIG2_M1_DRAM_BYTES if fam == 1 else None, "peak_source": peaks["source"],
                            "kernel_us": t_k * 1e6, "algorithmic_bytes_per_launch": algo, "frac_of_nominal_8000": achieved / 8000.0,
                            "operator_us": t_op * 1e6, "kernel_family": KERNEL_NAMES.get(fam),
                            "what": "configs[1] at M=1: the mat-vec kernel over 32 rotating weight matrices (1057 MB > L2) that "
                                    "share one quantization per step, launches free to overlap; operator_us is one whole MatMul "
                                    "(quantize + kernel), each launch waiting for its predecessor"}
        if not args.no_configs:
            configs = config_legs(args, torch, device, N, synth, stream, peaks)
            configs["config3_prefill"] = prefill_leg(args, device, torch, N, synth, stream, peaks, with_cpu=not args.no_cpu)
            configs["config4_decode_step_8b"] = decode_step_leg(args, torch, dist, device, N, synth, stream, peaks)
            configs["either_side_of_the_matmul"] = extras_leg(args, torch, device, N, synth, stream, peaks)
            line["configs"] = configs
        if not args.no_cpu:
            base, _ = cpu_stack_baseline(rows, 12.0)
            line["cpu_baseline"] = base
    elif rank == 0:
        per_gpu = value / world
        line["roofline"] = {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": per_gpu / peaks["hbm_gbs"],
                            "traffic": None, "peak_source": peaks["source"],
                            "what": "per-GPU weight bytes of one step / step time (all launches and sums of the step, not one "
                                    "kernel): how much of the step is streaming and how much the latency of its chain of dependent launches"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    device.dispose()
    if world > 1:
        dist.destroy_process_group()


def run_shape(args):
    """--shape TYPE,N,K,ROWS[,FAMILY]: one MatMul shape over --copies rotating weight matrices, kernel and operator time
    (the probe behind the per-kernel profiles: small enough to capture under a profiler). FAMILY: auto, mmvq, skinny, mmq,
    tile."""
    import torch
    from sharplight_b200 import CudaExecutionProvider, synth
    from sharplight_b200 import native as N
    parts = args.shape.split(",")
    type_name, n, k, rows = parts[0], int(parts[1]), int(parts[2]), int(parts[3])
    family = {"auto": None, "mmvq": N.KERNEL_MMVQ, "skinny": N.KERNEL_SKINNY, "mmq": N.KERNEL_MMQ, "tile": N.KERNEL_TILE}[
        parts[4] if len(parts) > 4 else "auto"]
    torch.cuda.set_device(0)
    provider = CudaExecutionProvider()
    device = provider.open_device(provider.get_devices()[0])
    peaks = measured_peaks()
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    t_op, t_k, fam, launches = kernel_times(torch, device, N, synth, stream, type_name, n, k, rows, args.copies, max(args.steps, 1),
                                            kernel=family, use_graph=not args.no_graph)
    entry = hbm_entry(peaks, type_name, n, k, rows, t_op, t_k, fam, synth)
    entry.update({"shape": [type_name, n, k, rows], "copies": args.copies, "launches_per_matmul": launches,
                  "kernel_tops": 2.0 * rows * n * k / t_k / 1e12, "status": device.last_status()})
    print(json.dumps({"probe": entry}), flush=True)
    device.dispose()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=1, help="decode batch of the headline step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-configs", action="store_true", help="N=1: skip the legs of configurations 1-4 (profiling runs)")
    ap.add_argument("--layers", type=int, default=0, help="layers of the stack (default: the architecture's 80)")
    ap.add_argument("--tp-main-only", action="store_true", help="time the stack at --rows only, not at 1, 8, 64 and 2048 rows")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of a CUDA graph")
    ap.add_argument("--shape", default="", help="TYPE,N,K,ROWS[,FAMILY]: time this one MatMul shape and nothing else")
    ap.add_argument("--copies", type=int, default=8, help="--shape: rotating weight matrices")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.shape:
        run_shape(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
