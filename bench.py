"""Benchmark of the quantized MatMul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows M]

One JSON line on stdout (rank 0). Metric: quantized mat-vec HBM GB/s = weight bytes streamed per second, the figure the
reference's own benchmark reports (tests/Sharplight.Cpu.Tests/BenchTests.cs:82-99 of the Sharplight tree).

Workload at N = 1: benchmark configuration 2, the Llama-3-8B FFN shape -- Q4_K weight [14336, 4096], f32 activations ~N(0,1),
M = 1 row. One step = the MatMul (8-bit activation quantization + mat-vec) over each of COPIES independent weight
matrices of that shape (COPIES x 33 MB is far larger than the 126 MB L2, so every weight byte comes from HBM).
  value : device-resident inputs and outputs, timed with CUDA events on the launching stream.
  e2e   : the same step through the provider API (a compiled segment: SetInput / Execute / GetOutput) with HOST
          buffers: host->device copy of x, kernels, device->host copy of every y inside the timed region.
  roofline : the mat-vec kernel alone (activations already quantized), algorithmic bytes / measured launch time.
  cpu_baseline : the CPU restatement of the reference's integer-dot MatMul (oracle/) on the host cores, bounded sample.
With --impl reference the CPU arm is the measured one (the reference's managed CPU provider cannot be built here: no
.NET toolchain; the restatement is labelled "port").
For N > 1 every rank streams its own COPIES matrices (weak scaling, no data-path collective for this workload).
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

TYPE, N_ROWS_W, K_COLS = "Q4_K", 14336, 4096
COPIES = 32
# dram__bytes_read.sum + dram__bytes_write.sum of one matvec_kernel launch on this workload at M = 1, from the ncu capture
# summarised in profiles/matvec_q4k_m1_14336x4096.md (the algorithmic bytes are 33 092 608)
CONFIG2_M1_DRAM_BYTES = 33062656
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


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


def cpu_arm(rows: int, seconds: float = 12.0):
    """The reference's CPU integer-dot MatMul (restated in oracle/) on all host cores; bounded sample."""
    from oracle import sl_oracle
    from sharplight_b200 import synth
    threads = os.cpu_count() or 1
    copies = 8   # 264 MB of distinct weights, so the sample does not sit in the last-level cache
    blocks = [synth.weight_blocks(TYPE, N_ROWS_W, K_COLS, seed=200 + i) for i in range(copies)]
    x = synth.activations(rows, K_COLS, seed=300)
    wbytes = synth.weight_bytes(TYPE, N_ROWS_W, K_COLS)
    for i in range(2):
        sl_oracle.matmul_intdot(12, blocks[i], N_ROWS_W, K_COLS, x, threads=threads, tier=1)
    t0 = time.perf_counter()
    done = 0
    while True:
        sl_oracle.matmul_intdot(12, blocks[done % copies], N_ROWS_W, K_COLS, x, threads=threads, tier=1)
        done += 1
        el = time.perf_counter() - t0
        if el > seconds or done >= 4000:
            break
    return {"value": wbytes * done / el / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "tier": sl_oracle.fast_tier_name(),
            "sample": f"{done} mat-vecs of the {TYPE} [{N_ROWS_W},{K_COLS}] weight at M={rows} over {copies} rotating "
                      f"copies, {el:.1f} s, {threads} threads"}, el / done


def cpu_arm_stack(rows: int, seconds: float):
    """The N > 1 workload on the host cores: the four MatMuls of a Llama-3-70B-shaped layer (stacked qkv, o, stacked
    gate_up, down), an eighth of the output rows of each (60 MB of Q4_K blocks), in rotation; weight GB/s."""
    from oracle import sl_oracle
    from sharplight_b200 import synth, tp
    threads = os.cpu_count() or 1
    mats = []
    for i, (name, parts, k, _, _) in enumerate(tp.fused_layer_matmuls(tp.LLAMA70B)):
        n = sum(parts) // 8
        mats.append((synth.weight_blocks("Q4_K", n, k, seed=400 + i), n, k, synth.activations(rows, k, seed=410 + i)))
    layer_bytes = sum(synth.weight_bytes("Q4_K", n, k) for _, n, k, _ in mats)
    for b, n, k, x in mats:
        sl_oracle.matmul_intdot(12, b, n, k, x, threads=threads, tier=1)
    t0, done = time.perf_counter(), 0
    while True:
        for b, n, k, x in mats:
            sl_oracle.matmul_intdot(12, b, n, k, x, threads=threads, tier=1)
        done += 1
        el = time.perf_counter() - t0
        if el > seconds or done >= 2000:
            break
    gbs = layer_bytes * done / el / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "tier": sl_oracle.fast_tier_name(),
            "sample": f"{done} passes over one layer's four MatMuls at an eighth of their output rows "
                      f"({layer_bytes / 1e6:.0f} MB of Q4_K blocks) at M={rows}, {el:.1f} s, {threads} threads"}, gbs


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    seconds = max(3.0, min(60.0, 0.25 * (args.steps + args.warmup)))
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.gpus > 1:
        # the N > 1 arm's workload: the 70B-shaped stack (the CPU has no tensor parallelism: one socket, all threads)
        from sharplight_b200 import tp
        base, gbs = cpu_arm_stack(args.rows, seconds)
        total = tp.layer_weight_bytes(tp.LLAMA70B) * tp.LLAMA70B["layers"]
        line = {"impl": "reference", "metric": "quant mat-vec HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / (gbs * 1e9) * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
                "config": {"workload": f"configs[4]: Llama-3-70B-shaped stack, 80 layers, Q4_K, decode M={args.rows}, on the "
                                       "host cores; bounded sample, step time extrapolated to the 38.5 GB stack"},
                "cpu_baseline": base,
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "CPU restatement (oracle/) of the reference's Sharplight.Cpu integer-dot MatMul; the managed "
                        "reference cannot be built here (no .NET toolchain)"}
        print(json.dumps(line), flush=True)
        return
    base, per_matvec = cpu_arm(args.rows, seconds)
    line = {"impl": "reference", "metric": "quant mat-vec HBM GB/s", "value": base["value"], "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_matvec * COPIES * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 scales",
            "data": "synthetic",
            "config": {"workload": f"configs[1]: {TYPE} [{N_ROWS_W},{K_COLS}] mat-vec, M={args.rows}; bounded sample, "
                                   f"step time extrapolated to {COPIES} matrices"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement (oracle/) of the reference's Sharplight.Cpu integer-dot MatMul; the managed "
                    "reference cannot be built here (no .NET toolchain)"}
    print(json.dumps(line), flush=True)


def prefill_leg(device, torch, N, synth, stream, steps):
    """benchmark configuration 3: Q4_0 [4096, 4096], bf16 activations [2048, 4096] on the tcgen05 int8 GEMM.
    Operator time = quantization + GEMM (what the reference's published TFLOPS include,
    tests/Sharplight.Vulkan.Tests/BenchTests.cs:28-46); kernel time = the GEMM alone on quantized activations."""
    from sharplight_b200 import MatMulOp, SharedActivation
    from sharplight_b200.provider import to_bf16_bits
    n, k, m, copies = 4096, 4096, 2048, 8
    base = synth.weight_blocks("Q4_0", n, k, seed=300)
    ws = [device.upload_weight("Q4_0", (n, k), np.roll(base.reshape(n, -1), 11 * i, axis=0).reshape(-1))
          for i in range(copies)]
    ops = [MatMulOp(device, w, m) for w in ws]
    x = torch.from_numpy(to_bf16_bits(synth.activations(m, k, seed=301)).view(np.int16)).cuda()
    y = torch.empty((copies, m, n), dtype=torch.float32, device="cuda")
    act = SharedActivation(device, m, k)
    sp = stream.cuda_stream

    def op_step(p=sp):
        for i, op in enumerate(ops):
            op.run_pointers(x.data_ptr(), N.BF16, m, k, True, y[i].data_ptr(), n, True, p)

    def gemm_step(p=sp):
        for i, op in enumerate(ops):
            act.matmul(op, y[i].data_ptr(), n, p)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=torch.cuda.Stream()):
            fn(torch.cuda.current_stream().cuda_stream)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / (steps * copies)

    t_op = timed(op_step)
    act.quantize(x.data_ptr(), N.BF16, m, k, sp)
    t_gemm = timed(gemm_step)
    family, _ = ops[0].last_kernel()
    ops_count = 2.0 * m * n * k
    out = {"workload": "configs[2]: Q4_0 [4096,4096] x bf16 [2048,4096], 8 rotating weight copies",
           "operator_tops": ops_count / t_op / 1e12, "gemm_kernel_tops": ops_count / t_gemm / 1e12,
           "operator_us": t_op * 1e6, "gemm_kernel_us": t_gemm * 1e6,
           "frac_of_nominal_int8_4500": ops_count / t_gemm / 4.5e15,
           "kernel_family": {1: "mmvq (dp4a)", 2: "skinny (int8 mma)", 3: "mmq (tcgen05)"}[family],
           "block_scale_fmas": m * n * (k // 32)}
    for op in ops:
        op.dispose()
    for w in ws:
        w.dispose()
    act.dispose()
    return out


class TpStack:
    """benchmark configuration 5: the quantized MatMuls of a Llama-3-70B-shaped layer stack, tensor-parallel over the ranks:
    q / k / v / gate / up column-split (stacked into one qkv and one gate_up MatMul per layer), o / down row-split with
    an all-reduce (sum) of the f32 partial outputs.
    Attention, norms and the activation function are not on the path: the inputs of o and down are fresh synthetic
    activations of the sharded shape. One step = every MatMul of every layer once, for `rows` activation rows (any
    count up to max_rows: decode batches and the prefill run on the same stack)."""

    def __init__(self, device, torch, dist, N, synth, rank, world, max_rows, layers, arch, type_name="Q4_K"):
        from sharplight_b200 import MatMulOp, SharedActivation, TpExchange, tp
        self.torch, self.dist, self.N, self.world = torch, dist, N, world
        # the receive area of the in-kernel all-reduce (one serves o and down of every layer: same output width)
        self.exchange = None
        if world > 1:
            self.exchange = TpExchange(device, rank, world, N.TP_MAX_ROWS, arch["hidden"])
            self.exchange.connect_group(dist)
            dist.barrier()
        rows = max_rows
        self.layers, self.arch = layers, arch
        # q / k / v and gate / up are stacked along N (one MatMul each), as a runtime stores them
        self.specs = [(name, sum(parts), k, split, inp) for name, parts, k, split, inp in tp.fused_layer_matmuls(arch)]
        self.total_weight_bytes = tp.layer_weight_bytes(arch, type_name) * layers
        h, f = arch["hidden"], arch["ffn"]
        self.weights, self.ops = [], []
        shard_blocks = {}
        for name, parts, k, split, _ in tp.fused_layer_matmuls(arch):
            nl, kl = tp.fused_shard_shape(parts, k, split, rank, world, type_name, arch["head_dim"])
            shard_blocks[name] = (synth.weight_blocks(type_name, nl, kl, seed=500 + 7 * rank + len(shard_blocks)), nl, kl)
        for _ in range(layers):
            layer_ops = {}
            for name, (blocks, nl, kl) in shard_blocks.items():
                w = device.upload_weight(type_name, (nl, kl), blocks)
                self.weights.append(w)
                layer_ops[name] = MatMulOp(device, w, rows)
            self.ops.append(layer_ops)
        dims = {name: (nl, kl) for name, (_, nl, kl) in shard_blocks.items()}
        self.dims = dims
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        mk = lambda r, c: torch.randn((r, c), generator=g, device="cuda", dtype=torch.float32)
        self.x = {"x_attn": mk(rows, h), "x_ffn": mk(rows, h), "x_o": mk(rows, dims["o"][1]), "x_down": mk(rows, dims["down"][1])}
        self.y = {name: torch.empty((rows, dims[name][0]), device="cuda", dtype=torch.float32) for name in dims}
        self.act = {key: SharedActivation(device, rows, v.shape[1]) for key, v in self.x.items()}
        self.launches_per_step = 0

    IN_KERNEL_ROWS = 16   # measured on 8 GPUs: in-kernel sum 2.2x faster than NCCL at 1 row, 1.5x at 8, 0.9x at 64

    def step(self, rows, sp, in_kernel=None):
        """in_kernel: row-split MatMuls sum over the ranks inside their kernel (peer stores over NVLink), possible up
        to 64 rows and the default up to IN_KERNEL_ROWS; otherwise the partial outputs go through an NCCL all-reduce."""
        N = self.N
        launches = 0
        if in_kernel is None:
            in_kernel = rows <= self.IN_KERNEL_ROWS
        in_kernel = in_kernel and self.exchange is not None and rows <= N.TP_MAX_ROWS
        for layer_ops in self.ops:
            for key in ("x_attn", "x_o", "x_ffn", "x_down"):
                x = self.x[key]
                self.act[key].quantize(x.data_ptr(), N.F32, rows, x.shape[1], sp)
                launches += 1
                for name, _, _, split, inp in self.specs:
                    if inp != key:
                        continue
                    y = self.y[name]
                    if split == "row" and in_kernel:
                        self.exchange.matmul(layer_ops[name], self.act[key], y.data_ptr(), y.shape[1], sp)
                    else:
                        self.act[key].matmul(layer_ops[name], y.data_ptr(), y.shape[1], sp)
                        if split == "row" and self.world > 1:
                            self.dist.all_reduce(y[:rows])
                    launches += layer_ops[name].last_kernel()[1]
        self.launches_per_step = launches

    def dispose(self):
        if self.exchange is not None:
            self.torch.cuda.synchronize()
            self.dist.barrier()
            self.exchange.dispose()
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


def decode_step_leg(args, torch, dist, device, N, synth, stream):
    """benchmark configuration 4: every quantized MatMul of one decode step of a Llama-3-8B-shaped model on one GPU, a
    continuous batch of 32 sequences: 32 layers of Q4_K weights (qkv, o, gate_up, down) and the Q6_K lm_head
    [128256, 4096]. Attention, norms and sampling are not on the path."""
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
    out = {"workload": "configs[3]: Llama-3-8B-shaped decode step, 32 layers Q4_K + Q6_K lm_head, batch 32, one GPU",
           "ms_per_step": ms, "weight_gbs": wbytes / (ms * 1e-3) / 1e9, "weight_bytes_per_step": wbytes,
           "sequences_per_s": rows / (ms * 1e-3), "launches_per_step": stack.launches_per_step + 2, "steps": steps}
    head_act.dispose(); head.dispose(); head_w.dispose(); stack.dispose()
    torch.cuda.synchronize()
    return out


def run_tp(args, torch, dist, device, N, synth, stream, world, rank, local):
    """The N > 1 workload (and the "tp_stack" object of the N = 1 line)."""
    from sharplight_b200 import tp
    arch = tp.LLAMA70B
    layers = args.layers or arch["layers"]
    out = {}
    row_counts = sorted(set([args.rows] + ([] if args.tp_main_only else [1, 8, 64, 2048])))
    stack = TpStack(device, torch, dist, N, synth, rank, world, max(row_counts), layers, arch)
    flops_per_row = 2.0 * sum(n * k for _, n, k, _, _ in stack.specs) * layers
    check = None
    if world > 1:
        # the in-kernel sum against the collective library's, on the last layer's row-split outputs of one step
        sp = stream.cuda_stream
        check = {}
        for rows in [r for r in (1, 8) if r <= max(row_counts)]:
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
    for rows in row_counts:
        steps = max(3, min(args.steps, 20 if rows <= 64 else 5))
        ms = time_graphed(torch, dist, world, stream, lambda sp, r=rows: stack.step(r, sp), steps, 3,
                          use_graph=not args.no_graph)
        in_kernel = world > 1 and rows <= TpStack.IN_KERNEL_ROWS
        out[rows] = {"ms_per_step": ms, "weight_gbs": stack.total_weight_bytes / (ms * 1e-3) / 1e9,
                     "tops": flops_per_row * rows / (ms * 1e-3) / 1e12, "steps": steps,
                     "launches_per_step": stack.launches_per_step,
                     "allreduce": "none" if world == 1 else "in the MatMul kernel (peer stores)" if in_kernel else "NCCL",
                     "allreduces_per_step": 2 * layers if world > 1 else 0}
        if world > 1 and rows <= N.TP_MAX_ROWS:
            # the same step with the sum done the other way, for comparison
            other = time_graphed(torch, dist, world, stream, lambda sp, r=rows: stack.step(r, sp, in_kernel=not in_kernel),
                                 steps, 3, use_graph=not args.no_graph)
            out[rows]["ms_per_step_nccl" if in_kernel else "ms_per_step_in_kernel"] = other
    stack.dispose()
    torch.cuda.synchronize()
    res = {"workload": f"configs[4]: Llama-3-70B-shaped stack, {layers} layers, Q4_K, tensor parallel x{world}",
           "weight_bytes_per_step": tp.layer_weight_bytes(arch) * layers, "by_rows": out}
    if check is not None:
        res["in_kernel_allreduce_check"] = check
    return res


def tp_roofline(per_gpu_gbs: float):
    """The N > 1 line's roofline object: the whole step, not one kernel -- every GPU streams its shard of the weights
    once per step, so per-GPU weight bytes over the step time against the measured HBM peak says how much of the step
    is streaming and how much is the latency of its chain of dependent launches."""
    peak, kind = measured_peaks()
    return {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
            "traffic": None, "peak_source": kind,
            "what": "per-GPU weight bytes of one step / step time (all launches and sums of the step, not one kernel)"}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from sharplight_b200 import CudaExecutionProvider, MatMulOp, SharedActivation, synth
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
    rows, n, k = args.rows, N_ROWS_W, K_COLS
    wbytes = synth.weight_bytes(TYPE, n, k)

    if world > 1:
        stream = torch.cuda.Stream()
        torch.cuda.set_stream(stream)
        sampler = ClockSampler(local)
        sampler.start()
        tpr = run_tp(args, torch, dist, device, N, synth, stream, world, rank, local)
        clocks = sampler.stop()
        if rank == 0:
            main = tpr["by_rows"][rows]
            line = {"metric": "quant mat-vec HBM GB/s", "value": main["weight_gbs"], "unit": "GB/s", "n_gpus": world,
                    "steps": max(3, min(args.steps, 20)), "warmup": 3, "ms_per_step": main["ms_per_step"],
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                    "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
                    "config": {"workload": tpr["workload"] + f", decode M={rows}: column-split q/k/v/gate/up, row-split "
                                           "o/down, f32 partial outputs summed inside the MatMul kernel over NVLink peer memory "
                                           "up to 16 rows, by an NCCL all-reduce above",
                               "l2": f"inputs larger than L2: {tpr['weight_bytes_per_step'] / world / 1e9:.1f} GB of weights per GPU per step",
                               "launch": "host launches" if args.no_graph else "CUDA graph replay of the step"},
                    "gpu_launches": main["launches_per_step"] * max(3, min(args.steps, 20)),
                    "roofline": tp_roofline(main["weight_gbs"] / world),
                    "tp_stack": tpr, "clocks": clocks,
                    "e2e": {"value": main["weight_gbs"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                            "note": "activations of this workload are device-resident by construction (they come from the "
                                    "preceding layer); the host-buffer figure is reported by the N=1 run"}}
            print(json.dumps(line), flush=True)
        device.dispose()
        dist.destroy_process_group()
        return

    base_blocks = synth.weight_blocks(TYPE, n, k, seed=100 + rank)
    weights, ops = [], []
    for i in range(COPIES):
        blocks = np.roll(base_blocks.reshape(n, -1), i * 37, axis=0).reshape(-1)   # distinct matrices, cheap to make
        w = device.upload_weight(TYPE, (n, k), blocks)
        weights.append(w)
        ops.append(MatMulOp(device, w, max(rows, 1)))
    x_host = torch.from_numpy(synth.activations(rows, k, seed=7)).pin_memory()
    y_host = torch.empty((COPIES, rows, n), dtype=torch.float32).pin_memory()
    x_dev = x_host.cuda()
    y_dev = torch.empty((COPIES, rows, n), dtype=torch.float32, device="cuda")
    # an explicit (non-default) launching stream: kernels, CUDA events and graph replays all go to it
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sptr = stream.cuda_stream
    assert sptr != 0
    act = SharedActivation(device, max(rows, 1), k)

    def step_device(sp=sptr):
        for i, op in enumerate(ops):
            op.run_pointers(x_dev.data_ptr(), N.F32, rows, k, True, y_dev[i].data_ptr(), n, True, sp)

    def step_kernel_only(sp=sptr):
        for i, op in enumerate(ops):
            act.matmul(op, y_dev[i].data_ptr(), n, sp)

    def graphed(fn):
        """Captures one step of fn into a CUDA graph; returns the replay callable."""
        if args.no_graph:
            return fn
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=torch.cuda.Stream()):
            fn(torch.cuda.current_stream().cuda_stream)
        graphs.append(graph)
        return graph.replay

    graphs = []

    # End to end through the provider API with host buffers: one compiled segment holding the step's MatMul nodes
    # (SetInput copies x from host memory, Execute quantizes once and runs every node, GetOutput reads the results
    # back); the copies in both directions are inside the timed region.
    from sharplight_b200 import CompileOptions, GraphSegment, MatMulNode, WeightInfo
    segment = None
    if not args.no_e2e:
        nodes = [MatMulNode(f"mm{i}", "x", WeightInfo(TYPE, (n, k), np.roll(base_blocks.reshape(n, -1), i * 37, axis=0).reshape(-1)),
                            f"y{i}") for i in range(COPIES)]
        segment = device.compile(GraphSegment(nodes, ["x"], [f"y{i}" for i in range(COPIES)]), CompileOptions(max_rows=max(rows, 1)))
    x_np = x_host.numpy()
    e2e_out = [None] * COPIES
    dev_stream = torch.cuda.ExternalStream(device.stream)

    def step_host():
        segment.set_input("x", x_np)
        segment.execute({"T": rows})
        for i in range(COPIES):
            e2e_out[i] = segment.get_output(f"y{i}", copy=False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    # The step's launches are captured once into a CUDA graph (the decode loop of a real model is launch-bound on the
    # host otherwise); the timed region replays that graph on the launching stream.
    sampler = ClockSampler(local)
    sampler.start()
    ms_step = timed(graphed(step_device), args.steps, max(args.warmup, 3))
    clocks = sampler.stop()
    kernel_family, launches_per_call = ops[0].last_kernel()   # launches of one MatMul call, quantization included
    # kernel pass for the roofline: activations quantized once and shared (as the q/k/v or gate/up MatMuls of a layer
    # share theirs), only the MatMul kernel in the timed loop, every launch free to run beside its predecessor
    act.quantize(x_dev.data_ptr(), N.F32, rows, k, sptr)
    ms_kernel_step = timed(graphed(step_kernel_only), args.steps, 3)
    main_launches = 1 if launches_per_call == 1 else launches_per_call - 1
    # end to end through host buffers
    ms_e2e = float("nan")
    same = None
    if not args.no_e2e:
        for _ in range(3):
            step_host()
        barrier()
        e_steps = max(3, args.steps // 4)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall0 = time.perf_counter()
        e0.record(dev_stream)
        for _ in range(e_steps):
            step_host()
        e1.record(dev_stream)
        barrier()
        wall_ms = (time.perf_counter() - t_wall0) * 1e3 / e_steps
        ms_e2e = max(e0.elapsed_time(e1) / e_steps, wall_ms)   # the step ends with a host-side wait: take the longer clock
        # a last correctness look at what was timed: graph-replayed device result == segment result read on the host
        torch.cuda.synchronize()
        yd = y_dev.cpu().numpy()
        same = bool(all(np.array_equal(yd[i], e2e_out[i]) for i in range(COPIES)))

    tp_stack = None
    if world == 1 and not args.no_tp_stack:
        tp_stack = run_tp(args, torch, dist, device, N, synth, stream, 1, 0, local)
    decode_step = None
    if world == 1 and not args.no_tp_stack:
        decode_step = decode_step_leg(args, torch, dist, device, N, synth, stream)
    prefill = None
    if world == 1 and not args.no_prefill:
        prefill = prefill_leg(device, torch, N, synth, stream, max(5, args.steps // 10))

    peak, peak_kind = measured_peaks()
    algo_bytes = wbytes + rows * k + rows * (k // 32) * 8 + rows * n * 4
    sec_per_launch = ms_kernel_step * 1e-3 / (COPIES * main_launches)
    achieved = algo_bytes / sec_per_launch / 1e9
    value = world * COPIES * wbytes / (ms_step * 1e-3) / 1e9
    e2e = world * COPIES * wbytes / (ms_e2e * 1e-3) / 1e9

    if rank == 0:
        base = None
        if world == 1 and not args.no_cpu:
            base, _ = cpu_arm(rows)
        line = {"metric": "quant mat-vec HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
                "config": {"workload": f"configs[1]: {TYPE} [{n},{k}] mat-vec (quantize + kernel), M={rows}, "
                                       f"{COPIES} weight matrices per step per GPU",
                           "l2": f"inputs larger than L2: {COPIES * wbytes / 1e6:.0f} MB of weights per step vs 126 MB",
                           "kernel_family": {1: "mmvq (dp4a)", 2: "skinny (int8 mma)", 3: "mmq (tcgen05)"}[kernel_family],
                           "launch": "host launches" if args.no_graph else "CUDA graph replay of the step"},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": CONFIG2_M1_DRAM_BYTES if (rows, n, k, TYPE) == (1, 14336, 4096, "Q4_K") else None,
                             "peak_source": peak_kind, "kernel_us": sec_per_launch * 1e6,
                             "algorithmic_bytes_per_launch": algo_bytes, "frac_of_nominal_8000": achieved / 8000.0,
                             "operator_us": ms_step * 1e3 / COPIES,
                             "what": "matvec_kernel on shared, already quantized activations (overlapping launches); "
                                     "operator_us is one whole MatMul of the main loop, quantization included, each "
                                     "launch waiting for its predecessor"},
                "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": rows * k * 4,
                        "d2h_bytes_per_step": COPIES * rows * n * 4, "ms_per_step": ms_e2e,
                        "note": "one compiled segment of the provider API: SetInput (host x), Execute, GetOutput of every "
                                "y; x is quantized once and shared by the step's MatMuls, as the reference's lowering "
                                "shares it, whereas `value` quantizes per MatMul"},
                "gpu_launches": args.steps * COPIES * launches_per_call,
                "clocks": clocks, "device_equals_host_path": same}
        if base is not None:
            line["cpu_baseline"] = base
        if prefill is not None:
            line["prefill"] = prefill
        if tp_stack is not None:
            line["tp_stack"] = tp_stack
        if decode_step is not None:
            line["decode_step_8b"] = decode_step
        print(json.dumps(line), flush=True)
    if segment is not None:
        segment.dispose()
    for op in ops:
        op.dispose()
    for w in weights:
        w.dispose()
    act.dispose()
    device.dispose()
    if world > 1:
        dist.destroy_process_group()


def main():
    global COPIES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--copies", type=int, default=COPIES, help="weight matrices per step (profiling runs use fewer)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--layers", type=int, default=0, help="layers of the tensor-parallel stack (default: the architecture's 80)")
    ap.add_argument("--no-tp-stack", action="store_true", help="N=1: skip the 70B-shaped stack at tensor-parallel degree 1 and the 8B decode step")
    ap.add_argument("--tp-main-only", action="store_true", help="time the stack at --rows only, not at 1, 8, 64 and 2048 rows")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM leg")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of a CUDA graph")
    args = ap.parse_args()
    COPIES = args.copies
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
