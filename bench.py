#!/usr/bin/env python
"""Benchmark of the FP8 W8A8 linear stack (the tensor-parallel linear layers of nano_qwen).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (one "step"): the full 36-layer Qwen3-8B-shaped linear stack — per layer
QKVParallelLinear 4096->6144, RowParallelLinear (o_proj) 4096->4096,
MergedColumnParallelLinear (gate_up) 4096->24576, RowParallelLinear (down)
12288->4096 — run once as a batched-decode pass (M = 256 tokens, replayed from a
CUDA graph, as the model runner does for decode) and once as a chunked-prefill
pass (M = 8192 tokens, eager), tensor-parallel over the N ranks (column layers
sharded on N, row layers on K with a bf16 all-reduce).  Random-init weights
(bf16 N(0, 0.02) quantised to e4m3 with 128x128 block scales), N(0,1)
activations quantised dynamically inside the timed region, synthetic data.
Each linear reads its own activation matrix (layers are not chained through
attention / SiLU, which are outside this path).

One JSON line is printed by rank 0; see the keys at the bottom of main().
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, LAYERS = 4096, 32, 8, 128, 12288, 36
M_DECODE, M_PREFILL = 256, 8192
# 2 * sum(N*K) over the four linears of one layer
FLOPS_PER_TOKEN_LAYER = 2 * (HIDDEN * (HEADS + 2 * KV_HEADS) * HEAD_DIM + HIDDEN * HIDDEN + HIDDEN * 2 * INTER + INTER * HIDDEN)
KINDS = ("qkv", "o_proj", "gate_up", "down")
WORKLOAD = ("Qwen3-8B-shaped 36-layer FP8 linear stack: decode pass M=256 (CUDA graph) + "
            "chunked-prefill pass M=8192 per step")


# DRAM traffic of the dominant kernel: one ncu capture of its qkv launch at M = 8192 read 81.0 MB and wrote 73.9 MB
# for 159.4 MB of algorithmic bytes (e4m3 x, e4m3 W, bf16 y); the other three shapes of the pass are scaled by the
# same ratio (operands are read once, y is written once).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 154.9 / 159.4


def prefill_gemm_traffic_bytes(layers) -> float:
    """dram read + write bytes per launch of the prefill-pass GEMM, averaged over one rank's four shapes."""
    total = 0.0
    for name in KINDS:
        n, k = layers[0][name].weight.shape
        total += M_PREFILL * k + n * k + 2.0 * M_PREFILL * n
    return total / len(KINDS) * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE


def flops_per_step() -> float:
    return float(LAYERS) * FLOPS_PER_TOKEN_LAYER * (M_DECODE + M_PREFILL)


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- #
# CPU arm: the oracle (port of the reference path) timed on the host cores     #
# --------------------------------------------------------------------------- #
def cpu_reference_sample(repeats: int, m_decode: int = 256, m_prefill: int = 8192) -> dict:
    """Times ONE layer of the stack on the CPU: dynamic activation quantisation, dequantisation of
    both operands to fp32 and the reference's ``F.linear`` (fp32), bf16 out — for a decode pass of
    ``m_decode`` tokens and a prefill chunk of ``m_prefill`` tokens.  Returns TFLOP/s."""
    from oracle import fp8_spec as S, ref_linear as R
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; this arm is the only work on the host
    # (the other ranks have left), so it takes every core at every N.
    torch.set_num_threads(os.cpu_count() or 1)
    torch.manual_seed(0)
    shapes = {"qkv": (HIDDEN, (HEADS + 2 * KV_HEADS) * HEAD_DIM), "o_proj": (HIDDEN, HIDDEN),
              "gate_up": (HIDDEN, 2 * INTER), "down": (INTER, HIDDEN)}
    weights = {}
    for name, (k, n) in shapes.items():
        w = (torch.randn(n, k) * 0.02).to(torch.bfloat16)
        weights[name] = S.quantize_weight_block128(w)
    acts = {(name, m): torch.randn(m, shapes[name][0]).to(torch.bfloat16)
            for name in shapes for m in (m_decode, m_prefill)}

    def one_pass(m):
        for name in KINDS:
            wq, sw = weights[name]
            xq, sx = S.quantize_act_group128(acts[(name, m)])
            R.column_forward(S.dequantize_act(xq, sx), S.dequantize_weight(wq, sw)).to(torch.bfloat16)

    one_pass(m_decode)          # warm-up (thread pool, allocator)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        one_pass(m_decode)
        one_pass(m_prefill)
        times.append(time.perf_counter() - t0)
    flops = FLOPS_PER_TOKEN_LAYER * (m_decode + m_prefill)
    best = min(times)
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 of {LAYERS} layers, decode M={m_decode} + prefill M={m_prefill} "
                      f"(act quant + dequant + fp32 F.linear), best of {repeats}, {best:.2f} s",
            "seconds": best, "host_cpus": os.cpu_count()}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_reference_sample(1, 64, 64)
    t0 = time.perf_counter()
    res = cpu_reference_sample(steps)
    wall = time.perf_counter() - t0
    line = {
        "impl": "reference", "metric": "fp8_linear_stack_tflops", "value": res["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": res["seconds"] * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tp": args.gpus, "layers": LAYERS,
                   "l2": "weights of the stack (6.95 GB / tp) exceed L2; no flush needed"},
        "cpu_baseline": res,
        "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": wall,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- #
# GPU arm                                                                      #
# --------------------------------------------------------------------------- #
def row_sum_note(L, tp: int) -> str:
    """Which reduction the row-parallel layers of this run use (decode-sized / prefill-sized outputs)."""
    if tp == 1:
        return "none (tp 1)"
    from nano_qwen_b200.layers import p2p_reduce, sym_reduce
    cls = L.RowParallelLinear
    small = "peer-memory push kernel" if (cls.p2p_reduce and p2p_reduce._reducer is not None) else "NCCL"
    want = cls.sym_reduce if cls.sym_reduce is not None else tp in cls.sym_auto_ranks
    large = (f"peer-memory pull kernel ({cls.overlap_chunks} chunk(s))"
             if (want and sym_reduce._reducer is not None) else "NCCL all-reduce")
    return f"decode-sized: {small}; prefill-sized: {large}"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons, power = [], [], set(), []
        for row in open(self.path):
            f = [c.strip() for c in row.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples taken under load: the upper half by power draw
        order = sorted(range(len(sm)), key=lambda i: power[i])
        hot = [sm[i] for i in order[len(order) // 2:]]
        hot.sort()
        return {"sm_mhz": hot[len(hot) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


class NvmlClock:
    """SM clock read through NVML (read-only queries) from a host thread while a short window is timed; the
    nvidia-smi sampler above needs a few hundred milliseconds to start, too long for a 30 ms window."""

    def __init__(self, gpu_index: int):
        self.samples, self.handle, self._stop = [], None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in visible.split(",") if v.strip().isdigit()]
            phys = int(ids[gpu_index]) if gpu_index < len(ids) else gpu_index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self._read = lambda: pynvml.nvmlDeviceGetClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.handle = None

    def __enter__(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        return self

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self._read())
            except Exception:
                return
            time.sleep(0.004)

    def __exit__(self, *exc):
        self._stop.set()
        if self.handle is not None:
            self.thread.join()

    def median(self):
        if not self.samples:
            return None
        v = sorted(self.samples)
        return v[len(v) // 2]


# Qwen3-32B-shaped layer (config 4 of the contract): hidden, heads, kv heads, head dim, intermediate
DIMS_32B = (5120, 64, 8, 128, 25600)


def build_stack(L, ops, tp_rank: int, tp_size: int, n_layers: int = LAYERS,
                dims=(HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER), seed_base: int = 0):
    """n_layers x 4 drop-in layers on the current device with random-init FP8 weights (this rank's shards)."""
    hidden, heads, kv_heads, head_dim, inter = dims
    torch.set_default_device("cuda")
    torch.set_default_dtype(torch.bfloat16)
    try:
        layers = []
        for li in range(n_layers):
            layer = {
                "qkv": L.QKVParallelLinear(hidden, head_dim, heads, kv_heads),
                "o_proj": L.RowParallelLinear(heads * head_dim, hidden),
                "gate_up": L.MergedColumnParallelLinear(hidden, [inter, inter]),
                "down": L.RowParallelLinear(inter, hidden),
            }
            for ki, (name, mod) in enumerate(layer.items()):
                gen = torch.Generator(device="cuda").manual_seed(seed_base + 1000 * li + 10 * ki + tp_rank)
                n, k = mod.weight.shape
                w = (torch.randn(n, k, generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                wq, sw = ops.weight_quant(w)          # this rank's shard, quantised on the device
                mod.weight.data.copy_(wq)
                mod.weight_scale_inv.data.copy_(sw)
                del w, wq, sw
            layers.append(layer)
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(torch.float32)
    return layers


def input_shapes(m: int, tp: int) -> dict:
    return {"qkv": (m, HIDDEN), "o_proj": (m, HIDDEN // tp), "gate_up": (m, HIDDEN), "down": (m, INTER // tp)}


def run_pass(layers, xs):
    y = None
    for layer in layers:
        for name in KINDS:
            y = layer[name](xs[name])
    return y


def run_gpu_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))

    from nano_qwen_b200 import _cabi, ops
    from nano_qwen_b200.layers import linear as L
    ops.init()
    tp = world
    if args.row_overlap_chunks is not None:                 # default: the layer's own choice (peer-memory sum on 2 and 8 ranks)
        L.RowParallelLinear.sym_reduce = args.row_overlap_chunks > 0
        if args.row_overlap_chunks > 0:
            L.RowParallelLinear.overlap_chunks = args.row_overlap_chunks
    layers = build_stack(L, ops, rank, tp)
    torch.cuda.synchronize()
    if tp > 1:
        # collective set-up of the peer-memory reductions, as a model runner does it once after init_process_group
        # and before graph capture (otherwise the first forward of each kind would do it, inside a warm-up step)
        from nano_qwen_b200.layers import p2p_reduce, sym_reduce
        if L.RowParallelLinear.p2p_reduce:
            p2p_reduce.init()
        want_sym = L.RowParallelLinear.sym_reduce
        if want_sym if want_sym is not None else tp in L.RowParallelLinear.sym_auto_ranks:
            sym_reduce.init()

    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    host = {}
    for tag, m in (("decode", M_DECODE), ("prefill", M_PREFILL)):
        host[tag] = {name: torch.randn(shape, generator=gen, dtype=torch.float32).to(torch.bfloat16).pin_memory()
                     for name, shape in input_shapes(m, tp).items()}
    dev = {tag: {name: t.cuda() for name, t in d.items()} for tag, d in host.items()}
    out_host = {tag: torch.empty((m, HIDDEN), dtype=torch.bfloat16).pin_memory()
                for tag, m in (("decode", M_DECODE), ("prefill", M_PREFILL))}

    # decode pass: captured once, replayed every step (static input buffers, like the model runner's graph_vars)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run_pass(layers, dev["decode"])
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    n_before_capture = ops.launch_count()
    with torch.cuda.graph(graph):
        y_decode = run_pass(layers, dev["decode"])
    graph_kernels = ops.launch_count() - n_before_capture    # this library's kernels inside one replay

    def step_resident():
        graph.replay()
        return run_pass(layers, dev["prefill"])

    # End to end: every step copies its inputs from pinned host memory and its results back.  The prefill inputs
    # (415 MB / tp) are double-buffered: while step i computes, a copy stream brings in the inputs of step i + 1,
    # as a serving loop would; the small decode inputs go on the compute stream in front of the graph replay.
    copy_stream = torch.cuda.Stream()
    stage = [{name: torch.empty_like(t, device="cuda") for name, t in host["prefill"].items()} for _ in range(2)]
    copied = [torch.cuda.Event(), torch.cuda.Event()]       # inputs of the set have arrived
    consumed = [torch.cuda.Event(), torch.cuda.Event()]     # the pass that read the set has finished
    e2e_state = {"step": 0}

    def prefetch(slot: int):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            for name, t in host["prefill"].items():
                stage[slot][name].copy_(t, non_blocking=True)
            copied[slot].record(copy_stream)

    for ev in consumed:
        ev.record()
    prefetch(0)

    def step_e2e():
        i = e2e_state["step"]
        e2e_state["step"] = i + 1
        prefetch((i + 1) % 2)                                # the next step's inputs, behind this step's compute
        for name, t in host["decode"].items():
            dev["decode"][name].copy_(t, non_blocking=True)
        graph.replay()
        out_host["decode"].copy_(y_decode, non_blocking=True)
        torch.cuda.current_stream().wait_event(copied[i % 2])
        y = run_pass(layers, stage[i % 2])
        consumed[i % 2].record()
        # the result goes back on the copy stream as well, behind the next step's compute
        y.record_stream(copy_stream)
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])
            out_host["prefill"].copy_(y, non_blocking=True)
        return y

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = ops.launch_count()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps, ops.launch_count() - n0

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step, launches = timed(step_resident, args.steps, args.warmup)
    launches += graph_kernels * args.steps                   # replays launch the captured kernels without host calls
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, _ = timed(step_e2e, args.steps, args.warmup)
    torch.cuda.synchronize()                                 # the copy stream's last prefetch has landed

    # ---- per-pass and per-kernel timings that explain the headline (same device, after the timed region) ----
    # The decode pass is short kernels whose time follows the SM clock: right behind the power-capped prefill steps
    # the clock is still low, after a pause it is at its maximum.  Both windows are sampled so that the two figures
    # (this one and detail.decode["256"]) can be compared as time x clock.
    def timed_with_clock(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        with NvmlClock(local) as clk:
            ms, _ = timed(fn, steps, 0)
        return ms, clk.median()

    ms_decode, mhz_decode = timed_with_clock(graph.replay, 40, 5)
    ms_prefill, _ = timed(lambda: run_pass(layers, dev["prefill"]), 3, 1)
    # dominant kernel: the GEMM of the prefill pass (256 x 256 tiles on CTA pairs), timed alone on pre-quantised activations
    pre = {name: ops.act_quant(dev["prefill"][name]) for name in KINDS}

    def prefill_gemms_only():
        for layer in layers:
            for name in KINDS:
                mod = layer[name]
                ops.fp8_gemm(pre[name][0], pre[name][1], mod.weight, mod.weight_scale_inv)

    ms_gemm, n_gemm = timed(prefill_gemms_only, 3, 1)
    n_gemm //= 3
    dec_pre = {name: ops.act_quant(dev["decode"][name]) for name in KINDS}
    g2 = torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for layer in layers:
            for name in KINDS:
                ops.fp8_gemm(dec_pre[name][0], dec_pre[name][1], layer[name].weight, layer[name].weight_scale_inv)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(g2):
        for layer in layers:
            for name in KINDS:
                ops.fp8_gemm(dec_pre[name][0], dec_pre[name][1], layer[name].weight, layer[name].weight_scale_inv)
    ms_dec_gemm, _ = timed(g2.replay, 5, 2)
    torch.cuda.synchronize()

    # ---- the other batch sizes of the contract (reported, not part of `value`): one pass over the same
    #      36-layer stack per M; decode sizes replayed from a CUDA graph, prefill sizes eager ----
    detail = {"decode": {}, "prefill": {}}
    if not args.no_detail:
        gen_d = torch.Generator(device="cuda").manual_seed(99 + rank)
        for m, kind in [(1, "decode"), (8, "decode"), (32, "decode"), (64, "decode"), (128, "decode"), (256, "decode"),
                        (2048, "prefill"), (8192, "prefill"), (16384, "prefill")]:
            xs = {name: torch.randn(shape, generator=gen_d, device="cuda", dtype=torch.float32).to(torch.bfloat16)
                  for name, shape in input_shapes(m, tp).items()}
            if kind == "decode":
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    run_pass(layers[:2], xs)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                gm = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gm):
                    run_pass(layers, xs)
                # enough warm-up replays (50-100 ms) for the SM clock to come back up after the power-capped passes
                ms, mhz = timed_with_clock(gm.replay, 20, 40)
                del gm
            else:
                ms, mhz = timed_with_clock(lambda: run_pass(layers, xs), 2, 1)
            shapes_m = {"qkv": (HIDDEN, (HEADS + 2 * KV_HEADS) * HEAD_DIM // tp), "o_proj": (HIDDEN // tp, HIDDEN),
                        "gate_up": (HIDDEN, 2 * INTER // tp), "down": (INTER // tp, HIDDEN)}
            bytes_layer = sum(2 * m * k + n * k + 4 * ((n + 127) // 128) * ((k + 127) // 128) + 2 * m * n
                              for k, n in shapes_m.values())
            layer_us = ms * 1e3 / LAYERS
            detail[kind][str(m)] = {
                "layer_us": round(layer_us, 2),
                "tflops": round(FLOPS_PER_TOKEN_LAYER * m / (layer_us * 1e-6) / 1e12, 1),          # whole job
                "hbm_gbs_per_gpu": round(bytes_layer / (layer_us * 1e-6) / 1e9, 1),
                "sm_mhz": mhz,
            }
            del xs
        torch.cuda.synchronize()
        # ---- config 4: one Qwen3-32B-shaped layer at this TP degree (three copies of the weights are cycled so that
        #      they never come from L2), M = 1 and 64 from a CUDA graph, M = 8192 eager ----
        hid32, heads32, kv32, hd32, inter32 = DIMS_32B
        big = build_stack(L, ops, rank, tp, n_layers=3, dims=DIMS_32B, seed_base=777000)
        flops32 = 2 * (hid32 * (heads32 + 2 * kv32) * hd32 + heads32 * hd32 * hid32 + hid32 * 2 * inter32 + inter32 * hid32)
        shapes32 = {"qkv": (hid32, (heads32 + 2 * kv32) * hd32 // tp), "o_proj": (heads32 * hd32 // tp, hid32),
                    "gate_up": (hid32, 2 * inter32 // tp), "down": (inter32 // tp, hid32)}
        detail["layer_32b"] = {}
        for m in (1, 64, 8192):
            xs = {name: torch.randn((m, k), generator=gen_d, device="cuda", dtype=torch.float32).to(torch.bfloat16)
                  for name, (k, n) in shapes32.items()}
            if m <= 64:
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    run_pass(big[:1], xs)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                gm = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gm):
                    for _ in range(4):
                        run_pass(big, xs)
                ms, _ = timed(gm.replay, 5, 2)
                layer_us = ms * 1e3 / (4 * len(big))
                del gm
            else:
                ms, _ = timed(lambda: run_pass(big, xs), 2, 1)
                layer_us = ms * 1e3 / len(big)
            bytes_layer = sum(2 * m * k + n * k + 4 * ((n + 127) // 128) * ((k + 127) // 128) + 2 * m * n
                              for k, n in shapes32.values())
            detail["layer_32b"][str(m)] = {
                "layer_us": round(layer_us, 2),
                "tflops": round(flops32 * m / (layer_us * 1e-6) / 1e12, 1),
                "hbm_gbs_per_gpu": round(bytes_layer / (layer_us * 1e-6) / 1e9, 1),
            }
            del xs
        del big
        torch.cuda.synchronize()
        # ---- the producers that emit FP8 directly (the rows next to the path): HBM-bound streaming kernels.
        #      Algorithmic bytes: silu-mul 4*M*I in + M*I + 4*M*I/128 out; add+norm 4*M*H in + 2*M*H (residual)
        #      + M*H + 4*M*H/128 out.  Three input copies are cycled; M = 8192 eager, M = 64 from a CUDA graph ----
        detail["producers"] = {}
        for m in (64, 8192):
            gu = [torch.randn((m, 2 * INTER // tp), generator=gen_d, device="cuda", dtype=torch.float32).to(torch.bfloat16)
                  for _ in range(3)]
            xr = [torch.randn((m, HIDDEN), generator=gen_d, device="cuda", dtype=torch.float32).to(torch.bfloat16)
                  for _ in range(3)]
            wn = torch.ones(HIDDEN, dtype=torch.bfloat16, device="cuda")

            def run_silu():
                for t in gu:
                    ops.silu_mul_quant(t)

            def run_norm():
                for t in xr:
                    ops.rmsnorm_quant(t, wn, 1e-6, xr[0])
            res = {}
            for name, fn, nbytes in (("silu_mul_quant", run_silu, m * (INTER // tp) * (4 + 1 + 4 / 128)),
                                     ("add_rmsnorm_quant", run_norm, m * HIDDEN * (4 + 2 + 1 + 4 / 128))):
                if m <= 64:
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        fn()
                    torch.cuda.current_stream().wait_stream(side)
                    torch.cuda.synchronize()
                    gm = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gm):
                        for _ in range(8):
                            fn()
                    ms, _ = timed(gm.replay, 5, 2)
                    us = ms * 1e3 / 24
                    del gm
                else:
                    ms, _ = timed(fn, 5, 2)
                    us = ms * 1e3 / 3
                res[name] = {"us": round(us, 2), "hbm_gbs": round(nbytes / (us * 1e-6) / 1e9, 1)}
            detail["producers"][str(m)] = res
            del gu, xr
        torch.cuda.synchronize()
        # ---- context: what the reference's own GPU path costs on this box.  nano_qwen's layers are bf16 ``F.linear``
        #      (cuBLAS) followed, for row layers, by ``dist.all_reduce`` (layers/linear.py:72-73, :152-156); four layers'
        #      worth of bf16 weights of this rank's shard shapes are cycled (they exceed L2), same token counts ----
        import torch.nn.functional as F
        shapes_r = {"qkv": (HIDDEN, (HEADS + 2 * KV_HEADS) * HEAD_DIM // tp), "o_proj": (HIDDEN // tp, HIDDEN),
                    "gate_up": (HIDDEN, 2 * INTER // tp), "down": (INTER // tp, HIDDEN)}
        n_ref = 4
        wref = [{name: (torch.randn((n, k), generator=gen_d, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
                 for name, (k, n) in shapes_r.items()} for _ in range(n_ref)]
        detail["bf16_f_linear"] = {}
        for m in (M_DECODE, M_PREFILL):
            xs = {name: torch.randn((m, k), generator=gen_d, device="cuda", dtype=torch.float32).to(torch.bfloat16)
                  for name, (k, n) in shapes_r.items()}

            def ref_pass():
                for wl in wref:
                    for name in KINDS:
                        y = F.linear(xs[name], wl[name])
                        if tp > 1 and name in ("o_proj", "down"):
                            dist.all_reduce(y)
            ms, _ = timed(ref_pass, 3, 2)
            layer_us = ms * 1e3 / n_ref
            detail["bf16_f_linear"][str(m)] = {"layer_us": round(layer_us, 2),
                                               "tflops": round(FLOPS_PER_TOKEN_LAYER * m / (layer_us * 1e-6) / 1e12, 1)}
            del xs
        del wref
        torch.cuda.synchronize()
    status = _cabi.device_status()

    if rank == 0:
        peaks = measured_peaks()
        flops = flops_per_step()
        tflops = flops / (ms_step * 1e-3) / 1e12
        prefill_flops = LAYERS * FLOPS_PER_TOKEN_LAYER * M_PREFILL / tp      # per GPU
        kernel_tflops = prefill_flops / (ms_gemm * 1e-3) / 1e12
        fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        # decode: algorithmic bytes of one rank's layer = weights + scales + bf16 in/out of the four linears
        shapes = {"qkv": (HIDDEN, (HEADS + 2 * KV_HEADS) * HEAD_DIM // tp), "o_proj": (HIDDEN // tp, HIDDEN),
                  "gate_up": (HIDDEN, 2 * INTER // tp), "down": (INTER // tp, HIDDEN)}
        layer_bytes = sum(2 * M_DECODE * k + n * k + 4 * ((n + 127) // 128) * ((k + 127) // 128) + 2 * M_DECODE * n
                          for k, n in shapes.values())
        decode_gbs = LAYERS * layer_bytes / (ms_decode * 1e-3) / 1e9
        in_bytes = sum(t.numel() * 2 for d in host.values() for t in d.values())
        out_bytes = sum(t.numel() * 2 for t in out_host.values())
        cpu = cpu_reference_sample(5) if world == 1 else None
        line = {
            "metric": "fp8_linear_stack_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate, bf16 out)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "tp": tp, "layers": LAYERS,
                       "l2": "weights of the stack (6.95 GB / tp) exceed L2; no flush needed",
                       "row_parallel_sum": row_sum_note(L, tp)},
            "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "token_pair_kernel (prefill-pass FP8 GEMM, 256x256 tiles on CTA pairs)",
                         "achieved": kernel_tflops, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": kernel_tflops / fp8_peak,
                         "peak_note": f"2 x bf16_tflops_sustained of {peaks['source']} (the e4m3 UMMA rate is twice the "
                                      "bf16 rate); torch._scaled_mm per-tensor FP8 measured 3046 burst / 2618 sustained here",
                         "launches": n_gemm, "avg_launch_us": ms_gemm * 1e3 / max(n_gemm, 1),
                         "traffic": prefill_gemm_traffic_bytes(layers), "traffic_unit": "bytes per launch",
                         "traffic_note": "ncu dram read+write of the qkv launch (154.9 MB for 159.4 MB algorithmic) "
                                         "scaled to the mean of the four shapes of the pass"},
            "passes": {"decode_ms": ms_decode, "prefill_ms": ms_prefill, "prefill_gemm_only_ms": ms_gemm,
                       "decode_gemm_only_ms": ms_dec_gemm,
                       "decode_layer_us": ms_decode * 1e3 / LAYERS, "decode_sm_mhz": mhz_decode,
                       "prefill_layer_us": ms_prefill * 1e3 / LAYERS,
                       "decode_hbm_gbs": decode_gbs, "decode_hbm_frac_of_measured": decode_gbs / peaks["hbm_gbs"],
                       "prefill_tflops": LAYERS * FLOPS_PER_TOKEN_LAYER * M_PREFILL / (ms_prefill * 1e-3) / 1e12},
            "detail": {"note": "one pass of the same stack per batch size M: act quant + GEMM (+ all-reduce) per linear; "
                               "layer_us = pass time / 36 (layer_32b: one Qwen3-32B-shaped layer at this TP degree, three "
                               "weight copies cycled); hbm_gbs_per_gpu uses the algorithmic bytes of one rank's layer "
                               f"(measured copy peak {peaks['hbm_gbs']} GB/s); tflops is the whole job; bf16_f_linear: "
                               "the reference's own GPU path (cuBLAS bf16 F.linear + NCCL all-reduce, eager) on the same "
                               "shard shapes, for context",
                       **detail},
            "device_status": status["code"],
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    # Normal interpreter exit (at-exit hooks run).  Graphs that captured collectives pin the communicator: drop
    # them first, then tear the group down.  A watchdog only guards against a teardown that never returns.
    del graph, g2, y_decode
    import gc
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()

    def _give_up():
        sys.stderr.write("bench.py: process-group teardown did not return within 60 s; leaving without it\n")
        sys.stderr.flush()
        os._exit(0)

    watchdog = threading.Timer(60.0, _give_up)
    watchdog.daemon = True
    watchdog.start()
    dist.destroy_process_group()
    watchdog.cancel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-detail", action="store_true", help="skip the per-batch-size sweep after the timed region")
    ap.add_argument("--row-overlap-chunks", type=int, default=None,
                    help="row-parallel layers at prefill sizes: N > 0 = sum over the peer-mapped buffer, the GEMM in N "
                         "chunks of token rows (N > 1: exchange of a chunk beside the GEMM of the next); 0 = NCCL's "
                         "all-reduce; default: the layer's own choice (peer-mapped buffer on 2 and 8 ranks, one chunk)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (the product has no CPU fallback); "
                             "use --impl reference for the CPU arm")
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
