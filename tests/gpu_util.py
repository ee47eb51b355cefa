"""Helpers for the GPU parity tests: torch owns device memory, every compute call goes through the C ABI."""
import ctypes as C

import numpy as np
import torch

from xstar_moe import capi, synth


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def new_workspace(cfg):
    nbytes = capi.workspace_bytes(cfg)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    assert ws.data_ptr() % 256 == 0
    capi.check(capi.lib().xs_moe_workspace_init(capi.ptr(ws), nbytes, stream_ptr()))
    return ws


def cfg_of(dims, gemm_impl=0, T=None):
    return capi.make_config(dims["T"] if T is None else T, dims["H"], dims["E"], dims["K"], dims["I"], dims["S"],
                            synth.FMT[dims["fmt"]], synth.FMT[dims["fmt"]] if dims["fmt"] != "fp4" else capi.FP8_BLOCK128,
                            gemm_impl=gemm_impl)


def forward(dims, d, gemm_impl=0, ws=None):
    """d: dict of CUDA tensors (synth.make_inputs(..., device='cuda')).  Returns out (T,H) bf16 tensor."""
    cfg = cfg_of(dims, gemm_impl, T=d["x"].shape[0])
    ws = new_workspace(cfg) if ws is None else ws
    w = capi.make_weights(d)
    out = torch.empty_like(d["x"])
    L = capi.lib()
    capi.check(L.xs_moe_forward(C.byref(cfg), C.byref(w), capi.ptr(d["x"]), capi.ptr(out), capi.ptr(ws), ws.numel(), stream_ptr()))
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), stream_ptr()))
    return out


def rmsnorm(x, weight, eps):
    out = torch.empty_like(x)
    capi.check(capi.lib().xs_moe_rmsnorm(capi.ptr(x), capi.ptr(weight), capi.ptr(out), x.shape[0], x.shape[1], C.c_float(eps), stream_ptr()))
    torch.cuda.synchronize()
    return out


def block_forward(dims, d, norm_weight, eps):
    """x + moe(rmsnorm(x, norm_weight, eps)) through the C ABI; returns (T,H) bf16."""
    cfg = cfg_of(dims, T=d["x"].shape[0])
    L = capi.lib()
    need = C.c_size_t(0)
    capi.check(L.xs_moe_block_workspace_bytes(C.byref(cfg), C.byref(need)))
    ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    capi.check(L.xs_moe_workspace_init(capi.ptr(ws), ws.numel(), stream_ptr()))
    w = capi.make_weights(d)
    out = torch.empty_like(d["x"])
    capi.check(L.xs_moe_block_forward(C.byref(cfg), C.byref(w), capi.ptr(d["x"]), capi.ptr(norm_weight), C.c_float(eps), capi.ptr(out),
                                      capi.ptr(ws), ws.numel(), stream_ptr()))
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), stream_ptr()))
    return out


def oracle_block(oracle, dims, d, norm_weight, eps, threads=8):
    """The reference composition add(x, moe(rmsnorm(x, w, eps))) on the CPU; returns (out bits, routing of the normalised x)."""
    xb = d["x"].detach().cpu().contiguous().view(torch.uint16).numpy()
    wb = norm_weight.detach().cpu().contiguous().view(torch.uint16).numpy()
    xn = oracle.rmsnorm_bf16(xb, wb, eps)
    dn = dict(d)
    dn["x"] = torch.from_numpy(xn).view(torch.bfloat16)
    r = oracle_forward(oracle, dims, dn, threads=threads)
    return oracle.add_bf16(xb, r["out"]), r, xn


def route(dims, d):
    cfg = cfg_of(dims, T=d["x"].shape[0])
    T, E, K = cfg.num_tokens, cfg.num_experts, cfg.top_k
    logits = torch.empty((T, E), dtype=torch.float32, device="cuda")
    ids = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float32, device="cuda")
    capi.check(capi.lib().xs_moe_route(C.byref(cfg), capi.ptr(d["x"]), capi.ptr(d["router_w"]), capi.ptr(d.get("router_bias")),
                                       capi.ptr(logits), capi.ptr(ids), capi.ptr(w), None, 0, stream_ptr()))
    torch.cuda.synchronize()
    return logits, ids, w


def route_selected(dims, d):
    """xs_moe_route without asking for the logits: large batches take the tensor-core filter + exact refine router.
    Returns ids, w and the refine counters (tokens recomputed in full, exact logits computed)."""
    cfg = cfg_of(dims, T=d["x"].shape[0])
    T, K = cfg.num_tokens, cfg.top_k
    ws = new_workspace(cfg)
    ids = torch.empty((T, K), dtype=torch.int32, device="cuda")
    w = torch.empty((T, K), dtype=torch.float32, device="cuda")
    L = capi.lib()
    capi.check(L.xs_moe_route(C.byref(cfg), capi.ptr(d["x"]), capi.ptr(d["router_w"]), capi.ptr(d.get("router_bias")), None,
                              capi.ptr(ids), capi.ptr(w), capi.ptr(ws), ws.numel(), stream_ptr()))
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), stream_ptr()))
    counters = ws[200:216].view(torch.int64).cpu().tolist()
    return ids, w, counters


def permute(dims, ids):
    T, K = ids.shape
    cfg = cfg_of(dims, T=T)
    E = cfg.num_experts
    ws = new_workspace(cfg)
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    offsets = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    perm = torch.empty(T * K, dtype=torch.int32, device="cuda")
    inv = torch.empty(T * K, dtype=torch.int32, device="cuda")
    L = capi.lib()
    capi.check(L.xs_moe_permute(C.byref(cfg), capi.ptr(ids), capi.ptr(counts), capi.ptr(offsets), capi.ptr(perm), capi.ptr(inv),
                                capi.ptr(ws), ws.numel(), stream_ptr()))
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), stream_ptr()))
    return counts, offsets, perm, inv


def grouped_mlp(dims, d, rows, offsets, gemm_impl=0, row_scales=None):
    """rows (M,H) bf16 cuda, offsets (E+1) int32 cuda -> y (M,H) f32."""
    cfg = cfg_of(dims, gemm_impl, T=1)
    M = rows.shape[0]
    n = C.c_size_t(0)
    L = capi.lib()
    capi.check(L.xs_moe_grouped_mlp_workspace_bytes(C.byref(cfg), M, C.byref(n)))
    ws = torch.zeros(n.value, dtype=torch.uint8, device="cuda")
    y = torch.empty((M, cfg.hidden), dtype=torch.float32, device="cuda")
    w = capi.make_weights(d)
    capi.check(L.xs_moe_grouped_mlp(C.byref(cfg), C.byref(w), capi.ptr(rows), capi.ptr(row_scales), capi.ptr(offsets), M, capi.ptr(y), capi.ptr(ws),
                                    ws.numel(), stream_ptr()))
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), stream_ptr()))
    return y


def oracle_forward(oracle, dims, d, mode=None, threads=8, token_subset=None, want_y=False):
    n = synth.to_numpy_storage(d)
    if mode is None:
        mode = {"bf16": oracle.BF16, "fp8": oracle.FP8, "fp4": oracle.FP4}[dims["fmt"]]
    if mode == oracle.F32:
        n = {k: (synth.bf16_bits_to_f32(v) if v is not None and v.dtype == np.uint16 else v) for k, v in n.items()}
    return oracle.moe_forward(mode, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"], router_bias=n.get("router_bias"),
                              gate_up_scale=n.get("gate_up_scale"), down_scale=n.get("down_scale"),
                              shared_gate_up_w=n.get("shared_gate_up_w"), shared_down_w=n.get("shared_down_w"),
                              shared_gate_up_scale=n.get("shared_gate_up_scale"), shared_down_scale=n.get("shared_down_scale"),
                              threads=threads, token_subset=token_subset, want_y=want_y)


def bf16_to_f32(t):
    return t.float().cpu().numpy()
