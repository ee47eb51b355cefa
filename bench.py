#!/usr/bin/env python
"""MoE-layer throughput on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One step = one forward of the MoE layer (router top-k -> permute -> grouped GEMM + SwiGLU -> combine) over
one batch of seeded synthetic tokens.  The headline workload is the decode-sized bf16 layer
(T=128, H=4096, 256 experts, top-6, one shared expert, I=2048), which is HBM-bound: 12.9 GB of expert
weights are streamed every step, far more than the 126 MB L2, so no cache flush is needed between steps.

Prints one JSON line: tokens/s with inputs resident in HBM (`value`), the same through the host-buffer
entry point with the copies timed (`e2e`), the roofline of the dominant kernel, and the CPU baseline.  The
same line carries `workloads`: the other layer configurations (FP8 decode at 1/32/256 tokens, FP8 and FP4
prefill, FP4 decode; under N > 1 the 16 384-token FP4 expert-parallel layer), a few steps each, every one
with the roofline that bounds it (HBM for decode shapes, tensor pipe for prefill shapes, NVLink for the
expert-parallel exchange).  With N > 1 the experts are sharded over the ranks and every line carries a
`parity` field: outputs of a seeded subset of tokens against the CPU oracle run on the global problem.
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
DATA = "synthetic (seeded: weights N(0,0.02), activations N(0,1), rounded once to storage)"
NVLINK_GBS = 770.0      # measured peer copy per direction per GPU on this pool
FP8_NOMINAL_TFLOPS = 4500.0
SINGLE_GPU_WORKLOADS = ["decode_fp8_t1", "decode_fp8_t32", "decode_fp8_t256", "prefill_fp8", "decode_fp4", "prefill_fp4"]
TOL = {"bf16": 2e-3, "fp8": 1e-2, "fp4": 1e-2}


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s burst, which): the driver-written measurements of this pool, else the fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


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


def shape_config(workload, dims):
    """The keys both arms print under `config`: the workload's name and shape, nothing descriptive."""
    return dict(workload=workload, **{k: dims[k] for k in "THEKIS"}, format=dims["fmt"])


def stats(ms_list, steps):
    per = sorted(m / steps for m in ms_list)
    return {"median": float(np.median(per)), "min": per[0], "max": per[-1], "repeats": len(per)}


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU ops composed into the layer (oracle/_ref), else the CPU oracle
# ------------------------------------------------------------------------------------------------------------
def cpu_forward_tokens_per_s(dims, n, sample_tokens, threads, oracle):
    """Time one CPU pass of the whole layer over the first `sample_tokens` tokens of the batch (routing and experts
    for exactly those tokens: token rows are independent, so this is the batch's work per token) and return
    (tokens/s, seconds, kind)."""
    from xstar_moe import synth

    K = dims["K"]
    n = dict(n, x=np.ascontiguousarray(n["x"][:sample_tokens]))
    ref = oracle.ref_lib() if dims["fmt"] == "bf16" else None
    t0 = time.perf_counter()
    if ref is not None:
        xf, rwf = synth.bf16_bits_to_f32(n["x"]), synth.bf16_bits_to_f32(n["router_w"])
        logits = oracle.ref_router_logits(xf, rwf)
        ids, w = oracle.topk(logits, n.get("router_bias"), K)
        counts, offsets, perm, inv = oracle.permute(ids, dims["E"])
        routing = dict(topk_ids=ids, topk_w=w, offsets=offsets, perm=perm, inv=inv)
        oracle.ref_experts_combine(True, n["x"], n["gate_up_w"], n["down_w"], n.get("shared_gate_up_w"), n.get("shared_down_w"),
                                   routing, threads=threads)
        kind = "reference"
    else:
        mode = {"bf16": oracle.BF16, "fp8": oracle.FP8, "fp4": oracle.FP4}[dims["fmt"]]
        oracle.moe_forward(mode, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], K, router_bias=n.get("router_bias"),
                           gate_up_scale=n.get("gate_up_scale"), down_scale=n.get("down_scale"),
                           shared_gate_up_w=n.get("shared_gate_up_w"), shared_down_w=n.get("shared_down_w"),
                           shared_gate_up_scale=n.get("shared_gate_up_scale"), shared_down_scale=n.get("shared_down_scale"),
                           threads=threads)
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
        "vs_baseline": None, "dtype": dims["fmt"], "data": DATA, "config": shape_config(args.workload, dims),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"each step = the whole layer (routing and experts) over {per_step} of the batch's {dims['T']} tokens; "
                                   f"ms_per_step is the time of that sample, a full batch takes {dims['T'] / per_step:.1f}x as long"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# GPU arm, one device: the whole layer through xs_moe_forward
# ------------------------------------------------------------------------------------------------------------
NCU_TRAFFIC_PER_EXPERT = {  # dram__bytes_read + dram__bytes_write of the gate/up launch per expert streamed, H=4096, I=2048
    "bf16": (1.074722e9 + 4.153856e6) / 32, "fp8": (537.667072e6 + 3.838208e6) / 32}


def measure_single(name, dims, args, steps, repeats, want_e2e=True, seed=0):
    """Times one workload on the current device.  Returns a dict with per-step statistics, stage times, the routing's
    active experts, the launches counted per step and (want_e2e) the host-buffer figure."""
    import torch

    from xstar_moe import capi, synth

    L = capi.lib()
    T, H, E, K, I, S = (dims[k] for k in "THEKIS")
    d = synth.make_inputs(dims, seed=seed, device="cuda")
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

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return float(e0.elapsed_time(e1))

    for _ in range(max(3, args.warmup)):
        step()
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), st))
    c0 = capi.launch_count()
    step()
    launches_per_step = capi.launch_count() - c0

    # Decode-sized steps are a handful of short kernels: replay them as one CUDA graph so that launch gaps do not
    # dominate (xs_moe_forward allocates nothing and never synchronises, so it can be captured as it is).
    timed_step, used_graph = step, False
    graph = None
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
            raise SystemExit(f"{name}: graph replay and direct launch disagree")
        timed_step, used_graph = graph.replay, True
        for _ in range(3):
            timed_step()

    ms_list = [timed(timed_step, steps) for _ in range(repeats)]
    res = {"ms": stats(ms_list, steps), "used_graph": used_graph, "launches_per_step": int(launches_per_step)}
    if want_e2e:
        for _ in range(2):
            step_host()
        res["ms_e2e"] = stats([timed(step_host, steps) for _ in range(max(1, repeats // 2))], steps)
    # stage times with CUDA events on the launching stream (same steps, same inputs)
    stage = (C.c_float * 6)()
    acc = np.zeros(6)
    prof_steps = max(3, min(steps, 20))
    for _ in range(prof_steps):
        capi.check(L.xs_moe_forward_profile(C.byref(cfg), C.byref(w), capi.ptr(d["x"]), capi.ptr(out), capi.ptr(ws), nbytes, st, stage))
        acc += np.array(list(stage))
    res["stage_ms"] = {k: float(v) for k, v in zip(("router_logits", "select_permute", "scatter", "gate_up", "down", "combine"), acc / prof_steps)}
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), st))
    # routing of this batch -> active experts -> algorithmic bytes
    ids = torch.empty((T, K), dtype=torch.int32, device="cuda")
    tw = torch.empty((T, K), dtype=torch.float32, device="cuda")
    capi.check(L.xs_moe_route(C.byref(cfg), capi.ptr(d["x"]), capi.ptr(d["router_w"]), capi.ptr(d.get("router_bias")), None,
                              capi.ptr(ids), capi.ptr(tw), capi.ptr(ws), nbytes, st))
    torch.cuda.synchronize()
    res["active"] = int(torch.unique(ids).numel())
    tile, prefill = C.c_int32(0), C.c_int32(0)
    capi.check(L.xs_moe_plan_info(C.byref(cfg), C.byref(tile), C.byref(prefill)))
    res["token_tile"], res["prefill_kernels"] = int(tile.value), bool(prefill.value)
    res["inputs"] = d
    if graph is not None:
        graph.reset()
    return res


def roofline_single(dims, res):
    """The roofline of the dominant kernel (the gate/up GEMM launch) and of the whole layer, against the bound the
    shape has: HBM weight streaming for decode shapes, the tensor pipe for shapes that run the prefill kernels."""
    from xstar_moe import synth

    hbm, bf16_tf, kind = measured_peaks()
    T, H, E, K, I, S = (dims[k] for k in "THEKIS")
    fmt = dims["fmt"]
    active = res["active"]
    wbytes = {"bf16": 2.0, "fp8": 1.0, "fp4": 0.5}[fmt]
    merged_shared = S if fmt != "fp4" else 0  # the FP8 always-on expert next to FP4 experts runs in launches of its own
    step_ms = res["ms"]["median"]
    layer_bytes = synth.algorithmic_bytes(dims, active)
    layer_flops = synth.algorithmic_flops(dims)
    gu_ms, down_ms = res["stage_ms"]["gate_up"], res["stage_ms"]["down"]
    family = {"bf16": "grouped_gemm_bf16_kernel", "fp8": "grouped_gemm_fp8_kernel", "fp4": "grouped_gemm_fp4_kernel"}[fmt]
    if res["prefill_kernels"]:
        family = {"fp8": "prefill_gemm_fp8_kernel", "fp4": "prefill_gemm_fp4_kernel"}[fmt]
    kernel = f"{family}<gate_up>" + (f", token tile {res['token_tile']}" if not res["prefill_kernels"] else ", 128 tokens x 256 weight rows per MMA")
    if res["prefill_kernels"]:
        peak = 2.0 * bf16_tf  # no FP8 peak was measured by the driver: twice the measured dense bf16 burst stands in for it
        gu_flops = 2.0 * T * (K + merged_shared) * 2 * I * H
        gemm_flops = 2.0 * T * (K + S) * 3 * I * H
        ach = gu_flops / (gu_ms * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": kernel, "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "peak_kind": f"2 x {kind} dense bf16 burst ({bf16_tf:.1f} TFLOP/s); nominal dense FP8 {FP8_NOMINAL_TFLOPS:.0f}",
                "frac": ach / peak, "frac_of_nominal": ach / FP8_NOMINAL_TFLOPS, "traffic": None,
                "algorithmic_flops_per_launch": gu_flops, "ms_per_launch": gu_ms,
                "gemms": {"tflops": gemm_flops / ((gu_ms + down_ms) * 1e-3) / 1e12, "frac": gemm_flops / ((gu_ms + down_ms) * 1e-3) / 1e12 / peak,
                          "ms": gu_ms + down_ms},
                "layer": {"algorithmic_flops": layer_flops, "tflops": layer_flops / (step_ms * 1e-3) / 1e12,
                          "frac": layer_flops / (step_ms * 1e-3) / 1e12 / peak,
                          "hbm_frac": layer_bytes / (step_ms * 1e-3) / 1e9 / hbm},
                "stage_ms": res["stage_ms"]}
    gate_up_bytes = (active + merged_shared) * 2 * H * I * wbytes
    per_expert = NCU_TRAFFIC_PER_EXPERT.get(fmt)
    traffic = per_expert * (active + merged_shared) * (H * I) / (4096 * 2048) if per_expert else None
    ach = gate_up_bytes / (gu_ms * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": kernel + (" (routed + always-on experts)" if merged_shared else " (routed experts)"),
            "achieved": ach, "peak": hbm, "unit": "GB/s", "peak_kind": kind, "frac": ach / hbm, "traffic": traffic,
            "traffic_source": "ncu capture of a 32-expert case of the same kernel, scaled by experts streamed (profiles/)" if traffic else None,
            "algorithmic_bytes_per_launch": gate_up_bytes, "ms_per_launch": gu_ms,
            "layer": {"algorithmic_bytes": layer_bytes, "achieved": layer_bytes / (step_ms * 1e-3) / 1e9,
                      "frac": layer_bytes / (step_ms * 1e-3) / 1e9 / hbm},
            "stage_ms": res["stage_ms"]}


def l2_note(dims, active):
    from xstar_moe import synth

    b = synth.algorithmic_bytes(dims, active)
    if b > 126e6:
        return f"inputs larger than L2: {b / 1e9:.2f} GB of weights and activations streamed per step exceed 126 MB"
    return f"{b / 1e6:.0f} MB per step fit in the 126 MB L2"


def measure_host_op(dims, d, steps):
    """The layer through the reference-facing C++ op on device tensors: xstar_cpp.moe (synchronous: the call returns when the
    result is finished and checked, as every reference op does) and xstar_cpp.moe_into (enqueue on a stream, caller's scratch and
    output).  CUDA events on the stream the op uses; the synchronous form's time includes its host synchronisation."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "xstar-infer_b200", "xstar_cpp_py"))
    import xstar_cpp as xc

    fmt = dims["fmt"]
    wk = {"bf16": xc.DType.BFloat16, "fp8": xc.DType.Float8E4M3, "fp4": xc.DType.Float4E2M1x2}[fmt]
    sk = {"bf16": None, "fp8": xc.DType.Float32, "fp4": xc.DType.UE8M0}[fmt]
    shk = xc.DType.BFloat16 if fmt == "bf16" else xc.DType.Float8E4M3

    def view(t, dt):
        return xc.from_device_ptr(t.data_ptr(), list(t.shape), dt)

    a = [view(d["x"], xc.DType.BFloat16), view(d["router_w"], xc.DType.BFloat16), view(d["gate_up_w"], wk), view(d["down_w"], wk)]
    kw = {}
    if fmt != "bf16":
        kw.update(gate_up_scale=view(d["gate_up_scale"], sk), down_scale=view(d["down_scale"], sk))
    if dims["S"]:
        kw.update(shared_gate_up_weight=view(d["shared_gate_up_w"], shk), shared_down_weight=view(d["shared_down_w"], shk))
        if fmt != "bf16":
            kw.update(shared_gate_up_scale=view(d["shared_gate_up_scale"], xc.DType.Float32),
                      shared_down_scale=view(d["shared_down_scale"], xc.DType.Float32))
    if d.get("router_bias") is not None:
        kw["router_bias"] = view(d["router_bias"], xc.DType.Float32)
    K = dims["K"]
    stream = torch.cuda.current_stream()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return float(e0.elapsed_time(e1)) / n

    def sync_op():
        xc.moe(*a, K, **kw)

    out_t = torch.empty_like(d["x"])
    out = view(out_t, xc.DType.BFloat16)
    scratch = xc.MoEScratch()

    def stream_op():
        xc.moe_into(a[0], out, scratch, stream.cuda_stream, *a[1:], K, **kw)

    for _ in range(3):
        sync_op()
        stream_op()
    xc.moe_check(scratch, stream.cuda_stream)
    ms_sync = timed(sync_op, steps)
    ms_stream = timed(stream_op, steps)
    xc.moe_check(scratch, stream.cuda_stream)
    T = dims["T"]
    return {"call": "xstar_cpp.moe(x, router_weight, gate_up_weight, down_weight, top_k, ...) on device tensors",
            "ms_per_call": ms_sync, "value": T / (ms_sync * 1e-3), "unit": UNIT,
            "stream_form": {"call": "xstar_cpp.moe_into(x, out, scratch, stream, ...): enqueue only, caller's output and scratch",
                            "ms_per_call": ms_stream, "value": T / (ms_stream * 1e-3), "unit": UNIT}}


def run_ours(args, dims):
    import torch

    from xstar_moe import capi, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    L = capi.lib()
    capi.check(L.xs_moe_device_check())
    T = dims["T"]
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    res = measure_single(args.workload, dims, args, args.steps, args.repeats)
    clocks = sampler.stop()
    roofline = roofline_single(dims, res)
    try:
        host_op = measure_host_op(dims, res["inputs"], args.steps)
    except Exception as e:  # noqa: BLE001 - the host module is optional for the headline
        host_op = {"error": f"{type(e).__name__}: {e}"}

    # CPU baseline on a bounded sample of the same batch
    cpu = None
    if not args.no_cpu:
        from oracle import moe_oracle as oracle

        cores = host_cores()
        n = synth.to_numpy_storage(res["inputs"])
        sample = pick_sample(dims, cores)
        v, dt, kind = cpu_forward_tokens_per_s(dims, n, sample, cores, oracle)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "seconds": dt,
               "sample": f"the whole layer (routing and experts) over {sample} of the batch's {T} tokens"}
        del n
    active = res["active"]
    res.pop("inputs")
    torch.cuda.empty_cache()

    workloads = []
    if args.workloads == "all":
        for name in SINGLE_GPU_WORKLOADS:
            wd = dict(synth.CONFIGS[name])
            try:
                r = measure_single(name, wd, args, args.workload_steps, 5)
                r.pop("inputs")
                torch.cuda.empty_cache()
                rf = roofline_single(wd, r)
                workloads.append({
                    "workload": name, "config": shape_config(name, wd), "value": wd["T"] / (r["ms"]["median"] * 1e-3), "unit": UNIT,
                    "ms_per_step": r["ms"]["median"], "ms_per_step_min_max": [r["ms"]["min"], r["ms"]["max"]], "steps": args.workload_steps,
                    "repeats": r["ms"]["repeats"], "active_experts": r["active"], "launch": "cuda graph replay" if r["used_graph"] else "direct launches",
                    "gpu_launches_per_step": r["launches_per_step"],
                    "e2e": {"value": wd["T"] / (r["ms_e2e"]["median"] * 1e-3), "unit": UNIT, "ms_per_step": r["ms_e2e"]["median"]},
                    "roofline": rf, "l2": l2_note(wd, r["active"])})
            except Exception as e:  # one workload failing must not lose the headline
                workloads.append({"workload": name, "error": f"{type(e).__name__}: {e}"})
                torch.cuda.empty_cache()

    ms = res["ms"]["median"]
    line = {
        "metric": METRIC, "value": T / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms, "ms_per_step_min_max": [res["ms"]["min"], res["ms"]["max"]], "repeats": res["ms"]["repeats"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dims["fmt"], "data": DATA,
        "config": shape_config(args.workload, dims),
        "run": {"active_experts": active, "parallelism": "1 gpu", "launch": "cuda graph replay" if res["used_graph"] else "direct launches",
                "l2": l2_note(dims, active), "timing": f"{res['ms']['repeats']} repeats of {args.steps} steps, CUDA events on the launching stream; value = median repeat"},
        "e2e": {"value": T / (res["ms_e2e"]["median"] * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * dims["H"] * 2,
                "d2h_bytes_per_step": T * dims["H"] * 2 + 4, "ms_per_step": res["ms_e2e"]["median"],
                "ms_per_step_min_max": [res["ms_e2e"]["min"], res["ms_e2e"]["max"]]},
        "host_op": host_op,
        "gpu_launches": res["launches_per_step"] * args.steps,
        "gpu_launches_note": "kernels the library enqueued for one step (counted by the library) x steps of one timed repeat",
        "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks, "workloads": workloads,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# GPU arm, N > 1: expert parallelism
# ------------------------------------------------------------------------------------------------------------
def ep_parity(dims, rank, world, out_local, ids_local, oracle_threads):
    """Outputs of a seeded subset of tokens of rank 0 and of the last rank, and the expert ids of all their tokens,
    against the CPU oracle run on the GLOBAL problem (all ranks' experts; the inputs are regenerated from their seeds on
    rank 0, the device results travel by one small all-gather).  Collective; returns the parity dict on rank 0."""
    import torch
    import torch.distributed as dist

    from xstar_moe import synth

    T, H, E, K = (dims[k] for k in "THEK")
    n_sub = 3
    subs = [np.sort(np.random.default_rng(100 + r).choice(T, min(n_sub, T), replace=False)).astype(np.int64) for r in range(world)]
    mine = out_local[torch.from_numpy(subs[rank]).cuda()].contiguous()
    got_out = torch.empty((world, *mine.shape), dtype=mine.dtype, device="cuda")
    dist.all_gather_into_tensor(got_out.view(-1), mine.view(-1))
    got_ids = torch.empty((world, T, K), dtype=torch.int32, device="cuda")
    dist.all_gather_into_tensor(got_ids.view(-1), ids_local.contiguous().view(-1))
    if rank != 0:
        return None
    from oracle import moe_oracle as oracle

    keys = ("gate_up_w", "down_w", "gate_up_scale", "down_scale")
    parts = {k: [] for k in keys}
    xs, shared, router_w, bias = {}, None, None, None
    check_ranks = sorted({0, world - 1})
    for r in range(world):
        x, wl, sh, b = synth.make_ep_inputs(dims, r, world, seed=0, device="cuda")
        for k in keys:
            if wl.get(k) is not None:
                parts[k].append(synth.to_numpy_storage({k: wl[k]})[k])
        if r in check_ranks:
            xs[r] = synth.to_numpy_storage({"x": x})["x"]
        if r == 0:
            router_w = synth.to_numpy_storage({"w": wl["router_w"]})["w"]
            shared = synth.to_numpy_storage(sh) if sh is not None else {}
            bias = None if b is None else b.cpu().numpy()
        del x, wl, sh
        torch.cuda.empty_cache()
    glob = {k: (np.concatenate(v) if v else None) for k, v in parts.items()}
    mode = {"bf16": oracle.BF16, "fp8": oracle.FP8, "fp4": oracle.FP4}[dims["fmt"]]
    worst, ids_exact, tokens = 0.0, True, 0
    for r in check_ranks:
        ref = oracle.moe_forward(mode, xs[r], router_w, glob["gate_up_w"], glob["down_w"], K, router_bias=bias,
                                 gate_up_scale=glob["gate_up_scale"], down_scale=glob["down_scale"],
                                 shared_gate_up_w=shared.get("shared_gate_up_w"), shared_down_w=shared.get("shared_down_w"),
                                 shared_gate_up_scale=shared.get("shared_gate_up_scale"), shared_down_scale=shared.get("shared_down_scale"),
                                 threads=oracle_threads, token_subset=subs[r].astype(np.int32))
        ids_exact = ids_exact and bool(np.array_equal(got_ids[r].cpu().numpy(), ref["topk_ids"]))
        want = synth.bf16_bits_to_f32(ref["out"])[subs[r]]
        got = got_out[r].float().cpu().numpy()
        worst = max(worst, synth.rel_l2(got, want))
        tokens += len(subs[r])
    tol = TOL[dims["fmt"]]
    return {"rel_l2": worst, "tolerance": tol, "ok": bool(worst <= tol and ids_exact), "ids_exact": ids_exact, "tokens": tokens,
            "ranks_checked": check_ranks, "against": "CPU oracle on the global problem (all ranks' experts), worst rank's rel-L2"}


class CppEpStep:
    """One rank's expert-parallel step through the C++ host: torch owns x / out / the weights, xstar_cpp.EpContext owns the
    exchange buffers and drives the stage calls and NCCL.  The unique id travels through torch.distributed once."""

    def __init__(self, dims, rank, local_rank, world, x, weights, shared, bias, fused_return=True, signal_barriers=True):
        import torch
        import torch.distributed as dist

        sys.path.insert(0, os.path.join(ROOT, "xstar-infer_b200", "xstar_cpp_py"))
        import xstar_cpp

        self.m, self.torch = xstar_cpp, torch
        T, H, E, K, I, S = (dims[k] for k in "THEKIS")
        fmt = dims["fmt"]
        box = [xstar_cpp.ep_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        dt = {"bf16": xstar_cpp.DType.BFloat16, "fp8": xstar_cpp.DType.Float8E4M3, "fp4": xstar_cpp.DType.Float4E2M1x2}[fmt]
        self.ctx = xstar_cpp.EpContext(None, box[0], rank, world, local_rank, T, H, E, K, I, dt, bool(S), 0.0, fused_return, signal_barriers)
        self.fused_return = self.ctx.fused_return()
        self.signal_barriers = self.ctx.signal_barriers()
        self.shape = (T, H)
        self.K = K
        self.keep = (weights, shared, bias)
        wk = dt
        sk = {"bf16": None, "fp8": xstar_cpp.DType.Float32, "fp4": xstar_cpp.DType.UE8M0}[fmt]
        shk = xstar_cpp.DType.BFloat16 if fmt == "bf16" else xstar_cpp.DType.Float8E4M3
        self.w = [self.view(weights["router_w"], xstar_cpp.DType.BFloat16), self.view(weights["gate_up_w"], wk), self.view(weights["down_w"], wk)]
        kw = {}
        if fmt != "bf16":
            kw["gate_up_scale"] = self.view(weights["gate_up_scale"], sk)
            kw["down_scale"] = self.view(weights["down_scale"], sk)
        if S:
            kw["shared_gate_up_weight"] = self.view(shared["shared_gate_up_w"], shk)
            kw["shared_down_weight"] = self.view(shared["shared_down_w"], shk)
            if fmt != "bf16":
                kw["shared_gate_up_scale"] = self.view(shared["shared_gate_up_scale"], xstar_cpp.DType.Float32)
                kw["shared_down_scale"] = self.view(shared["shared_down_scale"], xstar_cpp.DType.Float32)
        if bias is not None:
            kw["router_bias"] = self.view(bias, xstar_cpp.DType.Float32)
        self.kw = kw

    def view(self, t, dtype):
        assert t.is_contiguous() and t.is_cuda
        return self.m.from_device_ptr(t.data_ptr(), list(t.shape), dtype)

    def run(self, x, stream, out=None):
        out = self.torch.empty(self.shape, dtype=self.torch.bfloat16, device="cuda") if out is None else out
        self.ctx.moe_into(self.view(x, self.m.DType.BFloat16), self.view(out, self.m.DType.BFloat16), stream.cuda_stream, *self.w, self.K,
                          **self.kw)
        return out

    def capture(self, x_static):
        torch = self.torch
        out_static = torch.empty(self.shape, dtype=torch.bfloat16, device="cuda")
        warm = torch.cuda.Stream()
        warm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(warm):
            for _ in range(2):
                self.run(x_static, warm, out_static)
        torch.cuda.current_stream().wait_stream(warm)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.run(x_static, torch.cuda.current_stream(), out_static)
        return graph, out_static

    def check(self, stream):
        self.ctx.check(stream.cuda_stream)

    def close(self):
        self.ctx = None


def measure_ep(name, dims, args, steps, repeats, rank, local_rank, world, want_e2e=True):
    """One expert-parallel workload on the initialised process group.  Returns the entry dict on rank 0 (None elsewhere)."""
    import torch
    import torch.distributed as dist

    from xstar_moe import capi, ep, synth

    strong = name == "ep_fp4"  # this workload fixes the GLOBAL batch (16384 tokens) and splits it over the ranks
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

    # The timed step is driven by the C++ host (xstar_cpp.EpContext: NCCL + peer stores, no torch in the step); the Python
    # composition above stays for the phase marks and as the fallback when the context cannot be made on some rank.
    cpp = None
    if peer and args.ep_host == "cpp":
        try:
            cpp = CppEpStep(dims, rank, local_rank, world, x, weights, shared, bias, args.ep_fused_return == "on", args.ep_signal == "on")
        except Exception as e:  # noqa: BLE001 - any failure here means "use the Python host", on every rank
            print(f"rank {rank}: C++ expert-parallel host unavailable ({type(e).__name__}: {e})", file=sys.stderr, flush=True)
        agreed = torch.tensor([1 if cpp is not None else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            cpp = None

    c0 = capi.launch_count()
    if cpp is not None:
        cpp.run(x, stream)
    else:
        forward(x)
    launches_per_step = capi.launch_count() - c0
    use_graph = peer and args.graph != "off"  # nothing in the peer step touches the host: replay it whole at any size
    graph = None
    if use_graph:
        x_static = x.clone()
        try:
            if cpp is not None:
                graph, out_static = cpp.capture(x_static)
            else:
                graph, out_static = layer.capture_peer(x_static, px)
        except RuntimeError as e:
            print(f"rank {rank}: graph capture failed ({e}); launching the step eagerly", file=sys.stderr, flush=True)
        agreed = torch.tensor([1 if graph is not None else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)  # every rank replays, or none does
        if int(agreed.item()) == 0:
            if graph is not None:
                graph.reset()
            graph, use_graph = None, False
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
            return cpp.run(x, stream) if cpp is not None else forward(x)

        def step_host():
            xd = x_host.to("cuda", non_blocking=True)
            out_host.copy_(cpp.run(xd, stream) if cpp is not None else forward(xd), non_blocking=True)
            torch.cuda.synchronize()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(3, args.warmup)):
        step()
    ops.check()
    if cpp is not None:
        cpp.check(stream)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = stats([timed(step, steps) for _ in range(repeats)], steps)
    ms_e2e = None
    if want_e2e:
        for _ in range(2):
            step_host()
        ms_e2e = stats([timed(step_host, steps) for _ in range(max(1, repeats // 2))], steps)
    clocks = sampler.stop() if rank == 0 else None
    # parity of what the timed steps computed (same inputs): one more step, then the collective check
    out_dev = step().clone()
    ids_dev = ops.route(x, weights["router_w"], bias)[0]
    torch.cuda.synchronize()
    ops.check()
    if cpp is not None:
        cpp.check(stream)
    parity = ep_parity(dims, rank, world, out_dev, ids_dev, host_cores())
    # the grouped expert MLPs of this rank, timed on their own with CUDA events
    counts_now = torch.empty(world * E, dtype=torch.int32, device="cuda")
    dist.all_gather_into_tensor(counts_now, ops.permute(ids_dev)[0])
    all_counts = counts_now.view(world, E).cpu().numpy()
    plan = ep.EpPlan(all_counts, rank)
    payload = ops.payload(x)
    rows = [torch.zeros((max(plan.n_recv, 1), *p.shape[1:]), dtype=p.dtype, device="cuda") for p in payload]
    off = torch.from_numpy(plan.offsets_local).cuda()
    ops.grouped_mlp(rows, off, max(plan.n_recv, 1))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record(stream)
    for _ in range(reps):
        ops.grouped_mlp(rows, off, max(plan.n_recv, 1))
    e1.record(stream)
    torch.cuda.synchronize()
    mlp_ms = e0.elapsed_time(e1) / reps
    ops.check()
    # phase times of one more step (CUDA events on the launching stream; host-side gaps show up in the phase that follows them)
    forward(x)  # the marked step runs eagerly: warm its allocations first when the timed steps were graph replays
    torch.cuda.synchronize()
    marks = []
    forward(x, marks)
    torch.cuda.synchronize()
    phases = {marks[i][0]: marks[i - 1][1].elapsed_time(marks[i][1]) for i in range(1, len(marks))}
    active = int((np.diff(plan.offsets_local) > 0).sum())
    entry = None
    if rank == 0:
        hbm, bf16_tf, peak_kind = measured_peaks()
        fmt = dims["fmt"]
        wbytes = {"bf16": 2.0, "fp8": 1.0, "fp4": 0.5}[fmt]
        per_expert = 3 * H * I * wbytes + {"bf16": 0, "fp8": 3 * (H // 128) * (I // 128) * 4, "fp4": 3 * H * I // 32}[fmt]
        shared_bytes = S * (3 * H * I * (2.0 if fmt == "bf16" else 1.0))
        mlp_bytes = active * per_expert
        # bytes this rank must move and flops it must do per step, and the time each bound allows
        remote = 1.0 - 1.0 / world
        sent = float(all_counts[rank].sum() - all_counts[rank, rank * (E // world):(rank + 1) * (E // world)].sum())
        disp_row = H * (2 if fmt == "bf16" else 1) + {"bf16": 0, "fp8": (H // 128) * 4, "fp4": H // 32}[fmt]
        back_row = H * (4 if fmt == "bf16" else 2)
        recv_remote = float(plan.n_recv - all_counts[rank, rank * (E // world):(rank + 1) * (E // world)].sum())
        nv_ms = (max(sent, recv_remote) * disp_row + max(sent, recv_remote) * back_row) / (NVLINK_GBS * 1e9) * 1e3
        hbm_ms = (mlp_bytes + shared_bytes + E * H * 2 + 2 * T * H * 2) / (hbm * 1e9) * 1e3
        flops = 2.0 * (plan.n_recv + S * T) * 3 * H * I + 2.0 * T * H * E
        tensor_peak = (2.0 if fmt != "bf16" else 1.0) * bf16_tf
        tc_ms = flops / (tensor_peak * 1e12) * 1e3
        ideal_ms = max(nv_ms, hbm_ms, tc_ms)
        bound = "nvlink" if ideal_ms == nv_ms else ("hbm" if ideal_ms == hbm_ms else "tensor")
        step_ms = ms["median"]
        disp_ms = phases.get("dispatch (peer stores) + barrier")
        ret_ms = phases.get("return (peer stores) + barrier")
        entry = {
            "workload": name, "config": shape_config(name, dims), "value": T * world / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "ms_per_step": step_ms, "ms_per_step_min_max": [ms["min"], ms["max"]], "steps": steps, "repeats": ms["repeats"],
            "scaling": "strong" if strong else "weak",
            "scaling_note": (f"{dims['T'] * world} tokens in all, split over the ranks; experts sharded" if strong else
                             f"{T} tokens per rank (total grows with N) while each rank streams only its {E // world} of {E} experts: "
                             "neither fixed work per GPU nor fixed total work -- compare ms_per_step with ideal_ms_per_step"),
            "ideal_ms_per_step": ideal_ms, "frac_of_ideal": ideal_ms / step_ms,
            "ideal": {"bound": bound, "nvlink_ms": nv_ms, "hbm_ms": hbm_ms, "tensor_ms": tc_ms,
                      "peaks": f"HBM {hbm:.0f} GB/s ({peak_kind}), NVLink {NVLINK_GBS:.0f} GB/s per direction (measured peer copy), "
                               f"tensor {tensor_peak:.0f} TFLOP/s ({'2 x ' if fmt != 'bf16' else ''}{peak_kind} dense bf16 burst)"},
            "run": {"tokens_per_rank": T, "experts_per_rank": E // world,
                    "parallelism": f"ep{world}: experts sharded, " + ("dispatch/return by peer-memory stores over NVLink, no host synchronisation"
                                                                     if peer else "NCCL all-to-all dispatch/combine"),
                    "cuda_graph": bool(use_graph), "exchange_fallback": fallback,
                    "barriers": ("peer-memory flags (xs_moe_ep_signal), counts exchanged by the same kernel" if (cpp is not None and cpp.signal_barriers)
                                 else "NCCL all-gather + one-element all-reduces"),
                    "return_trip": ("folded into the down GEMM's epilogue" if (cpp is not None and cpp.fused_return) else "separate return kernel"),
                    "host": ("C++ (xstar_cpp.EpContext: NCCL all-gather / all-reduce + peer stores, one process per GPU)" if cpp is not None
                             else "Python composition of the stage calls (torch.distributed for the collectives)"),
                    "l2": "inputs larger than L2: expert weights streamed per step exceed 126 MB"},
            "e2e": None if ms_e2e is None else {"value": T * world / (ms_e2e["median"] * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * H * 2,
                                                "d2h_bytes_per_step": T * H * 2, "ms_per_step": ms_e2e["median"]},
            "gpu_launches_per_step": int(launches_per_step),
            "parity": parity,
            "roofline": {"bound": "hbm" if T * K / max(E, 1) * world <= 20 else "tensor",
                         "kernel": "grouped expert MLP of rank 0 (tile table + gate/up + down GEMM launches)",
                         "achieved": mlp_bytes / (mlp_ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s", "peak_kind": peak_kind,
                         "frac": mlp_bytes / (mlp_ms * 1e-3) / 1e9 / hbm, "traffic": None, "algorithmic_bytes_per_launch": mlp_bytes,
                         "ms_per_launch": mlp_ms, "tflops": 2.0 * plan.n_recv * 3 * H * I / (mlp_ms * 1e-3) / 1e12,
                         "tensor_frac": 2.0 * plan.n_recv * 3 * H * I / (mlp_ms * 1e-3) / 1e12 / tensor_peak,
                         "rows_received_rank0": plan.n_recv, "active_local_experts": active,
                         "exchange": {"bytes_out_dispatch": sent * disp_row, "bytes_in_return": sent * back_row,
                                      "dispatch_frac_of_nvlink": None if not disp_ms else sent * disp_row / (disp_ms * 1e-3) / 1e9 / NVLINK_GBS,
                                      "return_frac_of_nvlink": None if not ret_ms else recv_remote * back_row / (ret_ms * 1e-3) / 1e9 / NVLINK_GBS,
                                      "note": "kernel + the barrier that follows it, one eagerly launched step"},
                         "phase_ms_rank0": phases},
            "clocks": clocks,
        }
    torch.cuda.synchronize()
    if graph is not None:
        graph.reset()  # a live graph holds the communicator; destroy_process_group would block on it
    dist.barrier()
    if px is not None:
        px.close()
    if cpp is not None:
        cpp.close()
        dist.barrier()
    del ops, layer, x, weights, shared
    torch.cuda.empty_cache()
    return entry


def run_ours_ep(args, dims):
    """N > 1: expert parallelism.  Experts are sharded evenly over the ranks; rows travel by peer-memory stores (or NCCL
    all-to-all) each way.  Headline = the --workload layer with T tokens per rank; `workloads` adds the 16 384-token FP4
    expert-parallel layer."""
    import torch
    import torch.distributed as dist

    from xstar_moe import capi, synth

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    # the parity check runs the CPU oracle on rank 0 while the other ranks wait in a barrier: a generous time-out
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=900))
    capi.check(capi.lib().xs_moe_device_check())
    head = measure_ep(args.workload, dims, args, args.steps, args.repeats, rank, local_rank, world)
    extra = []
    if args.workloads == "all" and args.workload != "ep_fp4":
        try:
            e = measure_ep("ep_fp4", dict(synth.CONFIGS["ep_fp4"]), args, args.workload_steps, 5, rank, local_rank, world)
            if e is not None:
                extra.append(e)
        except Exception as ex:
            if rank == 0:
                extra.append({"workload": "ep_fp4", "error": f"{type(ex).__name__}: {ex}"})
            raise
    if rank == 0:
        line = {
            "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": head["ms_per_step"], "ms_per_step_min_max": head["ms_per_step_min_max"], "repeats": head["repeats"],
            "higher_is_better": True, "scaling": head["scaling"], "scaling_note": head["scaling_note"],
            "ideal_ms_per_step": head["ideal_ms_per_step"], "frac_of_ideal": head["frac_of_ideal"], "ideal": head["ideal"],
            "vs_baseline": None, "dtype": head["config"]["format"], "data": DATA, "config": head["config"], "run": head["run"],
            "e2e": head["e2e"], "gpu_launches": head["gpu_launches_per_step"] * args.steps,
            "gpu_launches_note": "kernels the library enqueued for one step on rank 0 (counted by the library) x steps of one timed repeat",
            "parity": head["parity"], "roofline": head["roofline"], "cpu_baseline": None, "clocks": head["clocks"], "workloads": extra,
        }
        print(json.dumps(line), flush=True)
        bad = [e for e in [head] + extra if e.get("parity") and not e["parity"]["ok"]]
        if bad:
            dist.destroy_process_group()
            raise SystemExit("parity out of tolerance: " + ", ".join(f"{e['workload']} rel-L2 {e['parity']['rel_l2']:.3e}" for e in bad))
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
    for kind, name in ((0, "bf16 K=16"), (1, "e4m3 K=32"), (2, "e4m3 x e2m1 block-scaled K=32"),
                       (3, "block-scaled K=32 + 3 tcgen05.cp per 4 MMAs"), (4, "e4m3 K=32, fresh accumulator + 2 commits per 4 MMAs"),
                       (5, "e4m3 K=32, fresh accumulator + 1 commit per 4 MMAs"),
                       (6, "e4m3 K=32, 4 MMAs + commit + wait for it (latency)")):
        for n in (16, 64, 128, 256):
            for chains in (1, 2, 4):
                if chains * n > (496 if kind in (2, 3) else 512) or (kind >= 4 and chains > 1):
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
    ap.add_argument("--repeats", type=int, default=5, help="how many times the timed region of --steps steps is repeated (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_bf16")
    ap.add_argument("--workloads", default=None, choices=["all", "none"],
                    help="also run the other layer configurations, a few steps each (default: all for the default workload)")
    ap.add_argument("--workload-steps", type=int, default=5, help="steps per repeat of each extra workload")
    ap.add_argument("--tokens", type=int, default=None, help="override the workload's token count")
    ap.add_argument("--experts", type=int, default=None, help="override the routed expert count (small profiling cases)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"], help="replay the step as a CUDA graph (auto: T <= 1024)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: rows travel by peer-memory stores from the dispatch/return kernels (default) or by NCCL all-to-all")
    ap.add_argument("--ep-host", default="cpp", choices=["cpp", "py"],
                    help="N > 1 with the peer exchange: the step is driven by the C++ host (xstar_cpp.EpContext, default) or by the "
                         "Python composition of the stage calls")
    ap.add_argument("--ep-fused-return", default="on", choices=["on", "off"],
                    help="N > 1, C++ host: let the down GEMM's epilogue store result rows into their source ranks where the kernels support it")
    ap.add_argument("--ep-signal", default="on", choices=["on", "off"],
                    help="N > 1, C++ host: counts exchange and barriers through peer-memory flags instead of NCCL collectives")
    ap.add_argument("--mma-rate", action="store_true", help="print the tensor-pipe and TMEM read-rate probe tables and exit")
    args = ap.parse_args()
    if args.mma_rate:
        return run_mma_rate()

    from xstar_moe import synth

    if args.workloads is None:
        args.workloads = "all" if (args.workload == "decode_bf16" and args.tokens is None and args.experts is None) else "none"
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
