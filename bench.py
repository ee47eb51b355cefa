#!/usr/bin/env python
"""MoE-layer throughput on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One step = one forward of the MoE layer (router top-k -> permute -> grouped GEMM + SwiGLU -> combine) over
one batch of seeded synthetic tokens.  The default workload is the decode-sized bf16 layer
(T=128, H=4096, 256 experts, top-6, one shared expert, I=2048), which is HBM-bound: 12.9 GB of expert
weights are streamed every step, far more than the 126 MB L2, so no cache flush is needed between steps.

Prints one JSON line: tokens/s with inputs resident in HBM (`value`), the same through the host-buffer
entry point with the copies timed (`e2e`), the roofline of the dominant kernel, and the CPU baseline.
With --impl reference it times the reference's own CPU ops (compiled in place under oracle/_ref, else the
CPU oracle) on the host cores instead.
"""
import argparse
import ctypes as C
import datetime
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "xstar-infer_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
def kernels_per_step(T):
    """logits, top-k, fused permute+tile-table, scatter, gate/up, down, combine for T <= 256;
    logits, top-k, count, scan, fill, scatter, tile table, gate/up, down, combine above."""
    return 7 if T <= 256 else 10


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only queries)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < 5.0:  # nvidia-smi needs a moment before its first sample
                time.sleep(0.01)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU ops composed into the layer (oracle/_ref), else the CPU oracle
# ------------------------------------------------------------------------------------------------------------
def cpu_forward_tokens_per_s(dims, n, sample_tokens, threads, oracle):
    """Time one CPU pass over `sample_tokens` tokens (routing over all tokens of the batch, experts for the
    sample) and return (tokens/s, seconds, kind)."""
    from xstar_moe import synth

    K = dims["K"]
    sub = np.arange(sample_tokens, dtype=np.int32)
    ref = oracle.ref_lib() if dims["fmt"] == "bf16" else None
    t0 = time.perf_counter()
    if ref is not None:
        xf, rwf = synth.bf16_bits_to_f32(n["x"]), synth.bf16_bits_to_f32(n["router_w"])
        logits = oracle.ref_router_logits(xf, rwf)
        ids, w = oracle.topk(logits, n.get("router_bias"), K)
        counts, offsets, perm, inv = oracle.permute(ids, dims["E"])
        routing = dict(topk_ids=ids, topk_w=w, offsets=offsets, perm=perm, inv=inv)
        oracle.ref_experts_combine(True, n["x"], n["gate_up_w"], n["down_w"], n.get("shared_gate_up_w"), n.get("shared_down_w"),
                                   routing, threads=threads, token_subset=sub)
        kind = "reference"
    else:
        mode = {"bf16": oracle.BF16, "fp8": oracle.FP8, "fp4": oracle.FP4}[dims["fmt"]]
        oracle.moe_forward(mode, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], K, router_bias=n.get("router_bias"),
                           gate_up_scale=n.get("gate_up_scale"), down_scale=n.get("down_scale"),
                           shared_gate_up_w=n.get("shared_gate_up_w"), shared_down_w=n.get("shared_down_w"),
                           shared_gate_up_scale=n.get("shared_gate_up_scale"), shared_down_scale=n.get("shared_down_scale"),
                           threads=threads, token_subset=sub)
        kind = "port"
    dt = time.perf_counter() - t0
    return sample_tokens / dt, dt, kind


def pick_sample(dims, cores):
    """Tokens whose expert work is roughly 10-20 s on `cores` threads at the reference's ~0.15 GMAC/s/thread."""
    macs_per_token = (dims["K"] + dims["S"]) * 3 * dims["H"] * dims["I"]
    rate = 0.15e9 * max(1, min(cores, dims["E"]))
    return int(max(1, min(dims["T"], round(12.0 * rate / macs_per_token))))


def run_reference_arm(args, dims):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import moe_oracle as oracle
    from xstar_moe import synth

    cores = host_cores()
    d = synth.make_inputs(dims, seed=0, device="cuda" if torch.cuda.is_available() else "cpu")
    n = synth.to_numpy_storage(d)
    del d
    per_step = max(1, pick_sample(dims, cores) // 3)  # ~4 s per step keeps steps+warmup within minutes
    kind = "port"
    for _ in range(args.warmup):
        _, _, kind = cpu_forward_tokens_per_s(dims, n, max(1, per_step // 4), cores, oracle)
    t = 0.0
    for _ in range(args.steps):
        _, dt, kind = cpu_forward_tokens_per_s(dims, n, per_step, cores, oracle)
        t += dt
    value = per_step * args.steps / t
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32-accumulate over bf16 storage" if dims["fmt"] == "bf16" else dims["fmt"],
        "data": "synthetic (seeded: weights N(0,0.02), activations N(0,1))",
        "config": dict(workload=args.workload, **{k: dims[k] for k in "THEKIS"}, format=dims["fmt"]),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"{per_step} of {dims['T']} tokens per step (routing over all tokens, experts for the sample)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------
def run_ours(args, dims):
    import torch
    import torch.distributed as dist

    from xstar_moe import capi, synth

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = capi.lib()
    capi.check(L.xs_moe_device_check())

    T, H, E, K, I, S = (dims[k] for k in "THEKIS")
    # every rank holds a full replica of the layer and its own batch of T tokens (weak scaling, no data-path collective)
    d = synth.make_inputs(dims, seed=rank, device="cuda")
    fmt = synth.FMT[dims["fmt"]]
    cfg = capi.make_config(T, H, E, K, I, S, fmt, capi.FP8_BLOCK128 if fmt == capi.FP4_MX32 else fmt)
    nbytes = capi.workspace_bytes(cfg)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()
    st = C.c_void_p(stream.cuda_stream)
    capi.check(L.xs_moe_workspace_init(capi.ptr(ws), nbytes, st))
    w = capi.make_weights(d)
    out = torch.empty_like(d["x"])
    x_host = d["x"].cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    x_stage = torch.empty_like(d["x"])

    def step():
        capi.check(L.xs_moe_forward(C.byref(cfg), C.byref(w), capi.ptr(d["x"]), capi.ptr(out), capi.ptr(ws), nbytes, st))

    def step_host():
        capi.check(L.xs_moe_forward_host(C.byref(cfg), C.byref(w), capi.ptr(x_host), capi.ptr(out_host), capi.ptr(x_stage),
                                         capi.ptr(out), capi.ptr(ws), nbytes, st))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(3, args.warmup)):
        step()
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), st))

    # Decode-sized steps are a handful of short kernels: replay them as one CUDA graph so that launch gaps do not
    # dominate (xs_moe_forward allocates nothing and never synchronises, so it can be captured as it is).
    timed_step, used_graph = step, False
    if args.graph == "on" or (args.graph == "auto" and T <= 1024):
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            st_side = C.c_void_p(side.cuda_stream)
            capi.check(L.xs_moe_forward(C.byref(cfg), C.byref(w), capi.ptr(d["x"]), capi.ptr(out), capi.ptr(ws), nbytes, st_side))
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                capi.check(L.xs_moe_forward(C.byref(cfg), C.byref(w), capi.ptr(d["x"]), capi.ptr(out), capi.ptr(ws), nbytes, st_side))
        stream.wait_stream(side)
        torch.cuda.synchronize()
        out_direct = out.clone()
        graph.replay()
        torch.cuda.synchronize()
        if not torch.equal(out, out_direct):
            raise SystemExit("graph replay and direct launch disagree")
        timed_step, used_graph = graph.replay, True
        for _ in range(3):
            timed_step()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(timed_step, args.steps)
    # end-to-end through the host-buffer entry point: h2d of x and d2h of out inside the timed region
    for _ in range(2):
        step_host()
    ms_e2e = timed(step_host, args.steps)

    # stage times with CUDA events on the launching stream (same steps, same inputs)
    stage = (C.c_float * 6)()
    acc = np.zeros(6)
    prof_steps = max(3, min(args.steps, 20))
    for _ in range(prof_steps):
        capi.check(L.xs_moe_forward_profile(C.byref(cfg), C.byref(w), capi.ptr(d["x"]), capi.ptr(out), capi.ptr(ws), nbytes, st, stage))
        acc += np.array(list(stage))
    stage_ms = acc / prof_steps
    clocks = sampler.stop() if rank == 0 else None
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), st))

    # routing of this batch -> active experts -> algorithmic bytes
    ids = torch.empty((T, K), dtype=torch.int32, device="cuda")
    tw = torch.empty((T, K), dtype=torch.float32, device="cuda")
    capi.check(L.xs_moe_route(C.byref(cfg), capi.ptr(d["x"]), capi.ptr(d["router_w"]), capi.ptr(d.get("router_bias")), None,
                              capi.ptr(ids), capi.ptr(tw), capi.ptr(ws), nbytes, st))
    torch.cuda.synchronize()
    active = int(torch.unique(ids).numel())

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    wbytes = {"bf16": 2.0, "fp8": 1.0, "fp4": 0.5}[dims["fmt"]]
    # the dominant kernel streams the gate and up matrices of every active expert and of the always-on expert
    gate_up_bytes = (active + (S if dims["fmt"] != "fp4" else 0)) * 2 * H * I * wbytes
    dom_ms = float(stage_ms[3])
    # DRAM traffic of the gate/up launch: dram__bytes_read + dram__bytes_write from the ncu capture of a small case
    # (32 experts' weights, 16 tokens; profiles/), which grows in proportion to the experts streamed
    per_expert = {"bf16": (1.074722e9 + 4.153856e6) / 32, "fp8": (537.667072e6 + 3.838208e6) / 32}.get(dims["fmt"])
    traffic = per_expert * (active + S) * (H * I) / (4096 * 2048) if per_expert else None
    layer_bytes = synth.algorithmic_bytes(dims, active)
    roofline = {
        "bound": "hbm", "kernel": f"grouped_gemm_{dims['fmt']}_kernel<gate_up> (routed" + (" + always-on experts)" if dims["fmt"] != "fp4" else " experts)"),
        "achieved": gate_up_bytes / (dom_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "peak_kind": peak_kind,
        "frac": gate_up_bytes / (dom_ms * 1e-3) / 1e9 / peak, "traffic": traffic,
        "traffic_source": "ncu capture of a 32-expert case of the same kernel, scaled by experts streamed (profiles/)" if traffic else None,
        "algorithmic_bytes_per_launch": gate_up_bytes, "ms_per_launch": dom_ms,
        "layer": {"algorithmic_bytes": layer_bytes, "achieved": layer_bytes / (ms / args.steps * 1e-3) / 1e9,
                  "frac": layer_bytes / (ms / args.steps * 1e-3) / 1e9 / peak},
        "stage_ms": {k: float(v) for k, v in zip(("router_logits", "select_permute", "scatter", "gate_up", "down", "combine"), stage_ms)},
    }

    # CPU baseline on a bounded sample of the same batch
    cpu = None
    if not args.no_cpu:
        from oracle import moe_oracle as oracle

        cores = host_cores()
        n = synth.to_numpy_storage(d)
        sample = pick_sample(dims, cores)
        v, dt, kind = cpu_forward_tokens_per_s(dims, n, sample, cores, oracle)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "seconds": dt,
               "sample": f"{sample} of {T} tokens (routing over all tokens, experts for the sample)"}

    tokens = T * world * args.steps
    line = {
        "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dims["fmt"],
        "data": "synthetic (seeded: weights N(0,0.02), activations N(0,1), rounded once to storage)",
        "config": dict(workload=args.workload, **{k: dims[k] for k in "THEKIS"}, format=dims["fmt"], active_experts=active,
                       parallelism=f"replicas x{world}" if world > 1 else "1 gpu", launch="cuda graph replay" if used_graph else "direct launches",
                       l2="inputs larger than L2: expert weights streamed per step exceed 126 MB"),
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 2 + 4,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": kernels_per_step(T) * args.steps,
        "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_ours_ep(args, dims):
    """N > 1: expert parallelism.  Experts are sharded evenly over the ranks, every rank brings its own batch of T
    tokens (weak scaling), rows travel by NCCL all-to-all each way."""
    import torch
    import torch.distributed as dist

    from xstar_moe import capi, ep, synth

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=180))
    capi.check(capi.lib().xs_moe_device_check())
    strong = args.workload == "ep_fp4"  # this workload fixes the GLOBAL batch (16384 tokens) and splits it over the ranks
    if strong:
        dims = dict(dims, T=dims["T"] // world)
    T, H, E, K, I, S = (dims[k] for k in "THEKIS")
    x, weights, shared, bias = synth.make_ep_inputs(dims, rank, world, seed=0, device="cuda")
    ops = ep.CudaOps(dict(dims), weights, shared, rank, world)
    layer = ep.ExpertParallelMoE(ops, weights["router_w"], bias, E, K, S)
    stream = torch.cuda.current_stream()
    x_host = x.cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    peer = args.exchange == "peer"
    px, fallback = None, None
    if peer:
        px = ep.PeerExchange(dims, rank, world)
        try:
            px.connect_ipc()
        except RuntimeError as e:  # agreed on by all ranks: no peer mappings on this box -> all-to-all exchange everywhere
            fallback = str(e)
            px.close()
            px, peer = None, False

    def forward(xd, marks=None):
        return layer.forward_peer(xd, px, marks) if peer else layer.forward(xd, marks)

    use_graph = peer and args.graph != "off"  # nothing in the peer step touches the host: replay it whole at any size
    if use_graph:
        x_static = x.clone()
        graph = None
        try:
            graph, out_static = layer.capture_peer(x_static, px)
        except RuntimeError as e:
            print(f"rank {rank}: graph capture failed ({e}); launching the step eagerly", file=sys.stderr, flush=True)
        agreed = torch.tensor([1 if graph is not None else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)  # every rank replays, or none does
        if int(agreed.item()) == 0:
            if graph is not None:
                graph.reset()
            use_graph = False
    if use_graph:

        def step():
            graph.replay()
            return out_static

        def step_host():
            x_static.copy_(x_host, non_blocking=True)
            graph.replay()
            out_host.copy_(out_static, non_blocking=True)
            torch.cuda.synchronize()
    else:
        def step():
            return forward(x)

        def step_host():
            xd = x_host.to("cuda", non_blocking=True)
            out_host.copy_(forward(xd), non_blocking=True)
            torch.cuda.synchronize()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(3, args.warmup)):
        step()
    ops.check()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(step, args.steps)
    for _ in range(2):
        step_host()
    ms_e2e = timed(step_host, args.steps)
    # the grouped expert MLPs of this rank, timed on their own with CUDA events
    if peer:
        counts_now = torch.empty(world * E, dtype=torch.int32, device="cuda")
        dist.all_gather_into_tensor(counts_now, ops.permute(ops.route(x, weights["router_w"], bias)[0])[0])
        plan = ep.EpPlan(counts_now.view(world, E).cpu().numpy(), rank)
    else:
        plan = layer.last_plan
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    payload = ops.payload(x)
    rows = [torch.zeros((plan.n_recv, *p.shape[1:]), dtype=p.dtype, device="cuda") for p in payload]
    off = torch.from_numpy(plan.offsets_local).cuda()
    ops.grouped_mlp(rows, off, plan.n_recv)
    torch.cuda.synchronize()
    reps = 5
    e0.record(stream)
    for _ in range(reps):
        ops.grouped_mlp(rows, off, plan.n_recv)
    e1.record(stream)
    torch.cuda.synchronize()
    mlp_ms = e0.elapsed_time(e1) / reps
    clocks = sampler.stop() if rank == 0 else None
    ops.check()
    # phase times of one more step (CUDA events on the launching stream; host-side gaps show up in the phase that follows them)
    forward(x)  # the marked step runs eagerly: warm its allocations first when the timed steps were graph replays
    torch.cuda.synchronize()
    marks = []
    forward(x, marks)
    torch.cuda.synchronize()
    phases = {marks[i][0]: marks[i - 1][1].elapsed_time(marks[i][1]) for i in range(1, len(marks))}
    active = int((np.diff(plan.offsets_local) > 0).sum())
    if rank == 0:
        peak, peak_kind = measured_peaks()
        wbytes = {"bf16": 2.0, "fp8": 1.0, "fp4": 0.5}[dims["fmt"]]
        mlp_bytes = active * 3 * H * I * wbytes
        tokens = T * world * args.steps
        line = {
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": dims["fmt"], "data": "synthetic (seeded: weights N(0,0.02), activations N(0,1), rounded once to storage)",
            "config": dict(workload=args.workload, **{k: dims[k] for k in "THEKIS"}, format=dims["fmt"], tokens_per_rank=T,
                           experts_per_rank=E // world, parallelism=f"ep{world}: experts sharded, " + ("dispatch/return by peer-memory stores over NVLink, no host synchronisation"
                                                                           if peer else "NCCL all-to-all dispatch/combine"), cuda_graph=bool(use_graph), exchange_fallback=fallback,
                           l2="inputs larger than L2: expert weights streamed per step exceed 126 MB"),
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 2,
                    "ms_per_step": ms_e2e / args.steps},
            # route 2 | permute 1 or 3 | [peer: plan, dispatch, return | all-to-all: quantise, 2 gathers per payload tensor, return gather]
            # | grouped MLP 3 | always-on expert 3 (+ its own quantise next to FP4 experts) | combine 1
            "gpu_launches": (2 + (1 if T <= 256 else 3) + (3 if peer else 1 + len(payload) * 2 + 1) + 3
                             + S * (4 if dims["fmt"] == "fp4" else 3) + 1) * args.steps,
            "roofline": {"bound": "hbm", "kernel": "grouped expert MLP of rank 0 (tile table + gate/up + down GEMM launches)",
                         "achieved": mlp_bytes / (mlp_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "peak_kind": peak_kind,
                         "frac": mlp_bytes / (mlp_ms * 1e-3) / 1e9 / peak, "traffic": None, "algorithmic_bytes_per_launch": mlp_bytes,
                         "ms_per_launch": mlp_ms, "rows_received_rank0": plan.n_recv, "active_local_experts": active,
                         "phase_ms_rank0": phases},
            "cpu_baseline": None, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    if use_graph:
        graph.reset()  # a live graph holds the communicator; destroy_process_group would block on it
    if px is not None:
        dist.barrier()
        px.close()
    dist.destroy_process_group()


def run_mma_rate():
    """Tables of hardware rates the tile shapes rest on: tcgen05.mma (M = 128) by kind, N and number of independent
    accumulators (cycles per instruction, whole-chip TFLOP/s), and TMEM -> register reads by load shape and warp count
    (bytes per cycle per SM), alone and beside a stream of N = 256 FP8 MMAs."""
    import torch

    from xstar_moe import capi

    torch.cuda.set_device(0)
    L = capi.lib()
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    rows = []
    for kind, name in ((0, "bf16 K=16"), (1, "e4m3 K=32"), (2, "e4m3 x e2m1 block-scaled K=32")):
        for n in (16, 64, 128, 256):
            for chains in (1, 2, 4):
                if chains * n > (496 if kind == 2 else 512):
                    continue
                cyc, iss, tf = C.c_double(), C.c_double(), C.c_double()
                for _ in range(2):  # second run is warm
                    capi.check(L.xs_moe_probe_mma_rate(kind, n, 4000, chains, capi.ptr(ws), ws.numel(), C.byref(cyc), C.byref(iss),
                                                       C.byref(tf), None))
                rows.append({"kind": name, "n": n, "chains": chains, "cycles_per_mma": round(cyc.value, 1),
                             "issue_cycles_per_mma": round(iss.value, 1), "tflops": round(tf.value, 1)})
    print(json.dumps({"mma_rate": rows}), flush=True)
    shapes = {0: "2 x (2 x .x16, wait)", 1: "4 x .x16, wait", 2: "2 x .x32, wait", 3: ".x64, wait"}
    rows = []
    for with_mma in (0, 1):
        for shape, sname in shapes.items():
            for warps in (4, 8, 16):
                bpc, mcyc = C.c_double(), C.c_double()
                for _ in range(2):
                    capi.check(L.xs_moe_probe_tmem_ld_rate(shape, warps, 2000, with_mma, capi.ptr(ws), ws.numel(), C.byref(bpc),
                                                           C.byref(mcyc), None))
                rows.append({"loads": sname, "warps": warps, "beside_mma": bool(with_mma), "bytes_per_cycle_per_sm": round(bpc.value, 1),
                             "mma_cycles_per_mma": round(mcyc.value, 1)})
    print(json.dumps({"tmem_ld_rate": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_bf16")
    ap.add_argument("--tokens", type=int, default=None, help="override the workload's token count")
    ap.add_argument("--experts", type=int, default=None, help="override the routed expert count (small profiling cases)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"], help="replay the step as a CUDA graph (auto: T <= 1024)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: rows travel by peer-memory stores from the dispatch/return kernels (default) or by NCCL all-to-all")
    ap.add_argument("--mma-rate", action="store_true", help="print the tensor-pipe rate probe table and exit")
    args = ap.parse_args()
    if args.mma_rate:
        return run_mma_rate()

    from xstar_moe import synth

    dims = dict(synth.CONFIGS[args.workload])
    if args.tokens is not None:
        dims["T"] = args.tokens
    if args.experts is not None:
        dims["E"] = args.experts
    if args.impl == "reference":
        run_reference_arm(args, dims)
    elif int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_ours_ep(args, dims)
    else:
        run_ours(args, dims)


if __name__ == "__main__":
    main()
