"""Seeded synthetic inputs for the MoE layer, shaped like the benchmark configurations.

Weights are drawn N(0, 0.02), activations N(0, 1), each rounded ONCE to its storage type; the same
tensors feed the CUDA path and the CPU oracle, so neither side sees an extra rounding.  No dataset or
checkpoint is involved.
"""
import math

import numpy as np
import torch

from . import capi

CONFIGS = {
    # name: T, H, E, K, I, S, format, router bias
    "small_bf16": dict(T=64, H=1024, E=16, K=2, I=512, S=0, fmt="bf16", bias=None),
    "decode_bf16": dict(T=128, H=4096, E=256, K=6, I=2048, S=1, fmt="bf16", bias=None),
    "decode_fp8_t1": dict(T=1, H=4096, E=256, K=6, I=2048, S=1, fmt="fp8", bias=None),
    "decode_fp8_t32": dict(T=32, H=4096, E=256, K=6, I=2048, S=1, fmt="fp8", bias=None),
    "decode_fp8_t256": dict(T=256, H=4096, E=256, K=6, I=2048, S=1, fmt="fp8", bias=None),
    "prefill_fp8": dict(T=8192, H=4096, E=256, K=6, I=2048, S=1, fmt="fp8", bias="zipf"),
    "decode_fp4": dict(T=128, H=4096, E=256, K=6, I=2048, S=1, fmt="fp4", bias=None),
    "prefill_fp4": dict(T=8192, H=4096, E=256, K=6, I=2048, S=1, fmt="fp4", bias="zipf"),
    "ep_fp4": dict(T=16384, H=4096, E=256, K=6, I=2048, S=1, fmt="fp4", bias=None),
}

FMT = {"bf16": capi.BF16, "fp8": capi.FP8_BLOCK128, "fp4": capi.FP4_MX32}


def zipf_bias(E, seed, s=1.1, scale=0.45, cap=6.0):
    """Per-expert router bias from Zipf(s) draws: bias = scale * min(log z, cap), centred.  With router logits of
    standard deviation ~1.3 this skews expert loads from empty to about three times the mean."""
    rng = np.random.default_rng(seed + 7919)
    z = rng.zipf(s, size=E).astype(np.float64)
    b = scale * np.minimum(np.log(z), cap)
    b -= b.mean()
    return torch.from_numpy(b.astype(np.float32))


def _randn_bf16(shape, std, gen, device, chunk_rows=None):
    """N(0,std) rounded once to bf16.  Large tensors are filled slice by slice along dim 0 to bound scratch."""
    out = torch.empty(shape, dtype=torch.bfloat16, device=device)
    n0 = shape[0]
    step = chunk_rows or max(1, min(n0, (1 << 27) // max(1, int(np.prod(shape[1:])))))
    for i in range(0, n0, step):
        j = min(n0, i + step)
        out[i:j] = (torch.randn((j - i, *shape[1:]), generator=gen, device=device, dtype=torch.float32) * std).to(torch.bfloat16)
    return out


def _fp8_block128(shape, std, gen, device):
    """e4m3 codes + f32 scale per 128x128 block (scales log-uniform in [2^-8, 2^-2]); code = e4m3(w / scale)."""
    *lead, R, C = shape
    codes = torch.empty(shape, dtype=torch.uint8, device=device)
    scales = torch.empty((*lead, R // 128, C // 128), dtype=torch.float32, device=device)
    flat_c = codes.view(-1, R, C)
    flat_s = scales.view(-1, R // 128, C // 128)
    for i in range(flat_c.shape[0]):
        w = torch.randn((R, C), generator=gen, device=device, dtype=torch.float32) * std
        s = torch.exp2(torch.rand((R // 128, C // 128), generator=gen, device=device, dtype=torch.float32) * 6.0 - 8.0)
        q = (w.view(R // 128, 128, C // 128, 128) / s.view(R // 128, 1, C // 128, 1)).clamp_(-448.0, 448.0)
        flat_c[i] = q.view(R, C).to(torch.float8_e4m3fn).view(torch.uint8)
        flat_s[i] = s
    return codes, scales


_E2M1_MID = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]


def _fp4_mx32(shape, std, gen, device):
    """Packed e2m1 codes (two per byte, low nibble = even k) + one e8m0 scale per 32 elements of the last dim:
    scale = smallest power of two >= amax / 6, code = nearest e2m1 value of w / scale."""
    *lead, R, C = shape
    codes = torch.empty((*lead, R, C // 2), dtype=torch.uint8, device=device)
    scales = torch.empty((*lead, R, C // 32), dtype=torch.uint8, device=device)
    flat_c = codes.view(-1, R, C // 2)
    flat_s = scales.view(-1, R, C // 32)
    mid = torch.tensor(_E2M1_MID, device=device)
    for i in range(flat_c.shape[0]):
        w = (torch.randn((R, C), generator=gen, device=device, dtype=torch.float32) * std).view(R, C // 32, 32)
        amax = w.abs().amax(-1, keepdim=True).clamp_min(1e-30)
        ex = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
        q = w / torch.exp2(ex)
        idx = torch.bucketize(q.abs(), mid).to(torch.uint8)  # 0..7
        code = (idx | ((q < 0).to(torch.uint8) << 3)).view(R, C)
        flat_c[i] = code[:, 0::2] | (code[:, 1::2] << 4)
        flat_s[i] = (ex.view(R, C // 32) + 127).to(torch.uint8)
    return codes, scales


def make_inputs(cfg, seed=0, device="cpu"):
    """Returns a dict of torch tensors in storage form:
       x (T,H) bf16, router_w (E,H) bf16, router_bias (E) f32 | None,
       gate_up_w (E,2I,H), down_w (E,H,I) [+ *_scale], shared_gate_up_w (2I,H), shared_down_w (H,I) [+ *_scale]."""
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    T, H, E, K, I, S = (cfg[k] for k in "THEKIS")
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    d = {}
    d["x"] = _randn_bf16((T, H), 1.0, gen, device)
    d["router_w"] = _randn_bf16((E, H), 0.02, gen, device)
    d["router_bias"] = zipf_bias(E, seed).to(device) if cfg.get("bias") == "zipf" else None
    fmt = cfg["fmt"]
    if fmt == "bf16":
        d["gate_up_w"] = _randn_bf16((E, 2 * I, H), 0.02, gen, device)
        d["down_w"] = _randn_bf16((E, H, I), 0.02, gen, device)
        if S:
            d["shared_gate_up_w"] = _randn_bf16((2 * I, H), 0.02, gen, device)
            d["shared_down_w"] = _randn_bf16((H, I), 0.02, gen, device)
    elif fmt == "fp8":
        d["gate_up_w"], d["gate_up_scale"] = _fp8_block128((E, 2 * I, H), 0.02, gen, device)
        d["down_w"], d["down_scale"] = _fp8_block128((E, H, I), 0.02, gen, device)
        if S:
            d["shared_gate_up_w"], d["shared_gate_up_scale"] = _fp8_block128((2 * I, H), 0.02, gen, device)
            d["shared_down_w"], d["shared_down_scale"] = _fp8_block128((H, I), 0.02, gen, device)
    elif fmt == "fp4":
        d["gate_up_w"], d["gate_up_scale"] = _fp4_mx32((E, 2 * I, H), 0.02, gen, device)
        d["down_w"], d["down_scale"] = _fp4_mx32((E, H, I), 0.02, gen, device)
        if S:  # the always-on expert is FP8 with 128x128 scales next to FP4 routed experts
            d["shared_gate_up_w"], d["shared_gate_up_scale"] = _fp8_block128((2 * I, H), 0.02, gen, device)
            d["shared_down_w"], d["shared_down_scale"] = _fp8_block128((H, I), 0.02, gen, device)
    else:
        raise NotImplementedError(fmt)
    return d


def make_ep_inputs(cfg, rank, world, seed=0, device="cuda"):
    """Inputs of one expert-parallel rank: the router matrix (and bias) and the always-on expert are replicated
    (same seed everywhere), the rank's own E/world routed experts and its own batch of T tokens are drawn from
    rank-specific seeds.  Returns (x, weights_local, shared_weights | None, router_bias | None)."""
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    T, H, E, K, I, S = (cfg[k] for k in "THEKIS")
    El = E // world
    common = make_inputs(dict(cfg, T=1, E=1, S=S), seed=seed + 3000, device=device)  # always-on expert, replicated
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    router_w = _randn_bf16((E, H), 0.02, gen, device)
    local = make_inputs(dict(cfg, T=T, E=El, S=0, bias=None), seed=seed + 2000 + rank, device=device)
    x = local["x"]
    weights = {k: v for k, v in local.items() if k in ("gate_up_w", "down_w", "gate_up_scale", "down_scale") and v is not None}
    weights["router_w"] = router_w
    shared = {k: v for k, v in common.items() if k.startswith("shared_") and v is not None} if S else None
    bias = zipf_bias(E, seed).to(device) if cfg.get("bias") == "zipf" else None
    return x, weights, shared, bias


def to_numpy_storage(d):
    """Host numpy views of the storage bytes (bf16 as uint16) for the CPU oracle."""
    out = {}
    for k, v in d.items():
        if v is None:
            out[k] = None
        elif v.dtype == torch.bfloat16:
            out[k] = v.detach().cpu().contiguous().view(torch.uint16).numpy()
        else:
            out[k] = v.detach().cpu().contiguous().numpy()
    return out


def bf16_bits_to_f32(a):
    return (a.astype(np.uint32) << 16).view(np.float32)


def algorithmic_bytes(cfg, active_experts):
    """Bytes one layer call must move: weights of every expert that received a token, the shared expert,
    the router matrix, x in and out (bf16)."""
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    T, H, E, K, I, S = (cfg[k] for k in "THEKIS")
    per = {"bf16": 3 * H * I * 2, "fp8": 3 * H * I + 3 * (H // 128) * (I // 128) * 4,
           "fp4": 3 * H * I // 2 + 3 * H * I // 32}[cfg["fmt"]]
    shared = {"bf16": 3 * H * I * 2}.get(cfg["fmt"], 3 * H * I + 3 * (H // 128) * (I // 128) * 4)
    return active_experts * per + S * shared + E * H * 2 + 2 * T * H * 2


def algorithmic_flops(cfg):
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    T, H, E, K, I, S = (cfg[k] for k in "THEKIS")
    return 2 * T * (K + S) * 3 * H * I + 2 * T * H * E


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
