"""ctypes binding of the C ABI in include/xs_moe.h and include/xs_moe_tuning.h.

This is plumbing for the tests and the benchmark: it passes raw device pointers (from torch tensors or
from the library's own allocator) straight to the `extern "C"` entry points.  There is no fallback: if the
shared library is missing the import fails, and if a call fails a RuntimeError carries the library's message.
"""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# XS_MOE_LIBRARY: another build of the same library to load instead (a tuning build with -DXS_ROLE_PROFILE=1, say)
LIB_PATH = os.environ.get("XS_MOE_LIBRARY") or os.path.join(_PKG, "libxs_moe.so")

BF16, FP8_BLOCK128, FP4_MX32 = 0, 1, 2


class XsMoeConfig(C.Structure):
    _fields_ = [
        ("num_tokens", C.c_int32),
        ("hidden", C.c_int32),
        ("num_experts", C.c_int32),
        ("top_k", C.c_int32),
        ("intermediate", C.c_int32),
        ("num_shared", C.c_int32),
        ("routed_format", C.c_int32),
        ("shared_format", C.c_int32),
        ("local_expert_begin", C.c_int32),
        ("local_expert_count", C.c_int32),
        ("gemm_impl", C.c_int32),
        ("reserved", C.c_int32 * 5),
    ]


class XsMoeWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "router_w_dev", "router_bias_dev", "gate_up_w_dev", "gate_up_scale_dev", "down_w_dev", "down_scale_dev",
        "shared_gate_up_w_dev", "shared_gate_up_scale_dev", "shared_down_w_dev", "shared_down_scale_dev")]


IPC_HANDLE_BYTES = 64

EXPORTS = [
    "xs_moe_status_string", "xs_moe_last_error", "xs_moe_device_check", "xs_moe_device_count", "xs_moe_set_device", "xs_moe_current_device", "xs_moe_device_alloc", "xs_moe_device_free",
    "xs_moe_memcpy_h2d", "xs_moe_memcpy_d2h", "xs_moe_memcpy_d2d", "xs_moe_device_free_bytes",
    "xs_moe_stream_synchronize", "xs_moe_workspace_bytes", "xs_moe_workspace_init", "xs_moe_forward",
    "xs_moe_forward_host", "xs_moe_forward_profile", "xs_moe_block_workspace_bytes", "xs_moe_block_forward", "xs_moe_rmsnorm", "xs_moe_route", "xs_moe_topk", "xs_moe_permute", "xs_moe_permute_noalloc", "xs_moe_grouped_mlp_workspace_bytes",
    "xs_moe_grouped_mlp", "xs_moe_quantize_rows_fp8", "xs_moe_quantize_rows_mxfp8", "xs_moe_gather_rows", "xs_moe_combine", "xs_moe_combine_bf16_rows", "xs_moe_gather_rows_f32_to_bf16", "xs_moe_check_flags", "xs_moe_debug_counters", "xs_moe_probe_mma_rate", "xs_moe_probe_tmem_ld_rate", "xs_moe_probe_handoff", "xs_moe_launch_count", "xs_moe_plan_info",
    "xs_moe_ipc_export", "xs_moe_ipc_import", "xs_moe_ipc_close", "xs_moe_ep_plan", "xs_moe_ep_dispatch", "xs_moe_ep_return", "xs_moe_ep_signal",
    "xs_moe_grouped_mlp_return_supported", "xs_moe_grouped_mlp_return",
    "xs_moe_comm_available", "xs_moe_comm_unique_id", "xs_moe_comm_create", "xs_moe_comm_destroy", "xs_moe_comm_abort",
    "xs_moe_comm_async_error", "xs_moe_comm_all_gather", "xs_moe_comm_barrier", "xs_moe_comm_all_to_all_v", "xs_moe_stream_create",
    "xs_moe_stream_destroy", "xs_moe_event_create", "xs_moe_event_destroy", "xs_moe_event_record", "xs_moe_stream_wait_event",
    "xs_moe_memset_async", "xs_moe_enable_peer_access",
]

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` (nvcc, sm_100a)")
        L = C.CDLL(LIB_PATH)
        L.xs_moe_status_string.restype = C.c_char_p
        L.xs_moe_status_string.argtypes = [C.c_int]
        L.xs_moe_last_error.restype = C.c_char_p
        vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int32
        cfgp, wp = C.POINTER(XsMoeConfig), C.POINTER(XsMoeWeights)
        sig = {
            "xs_moe_device_check": [],
            "xs_moe_device_count": [C.POINTER(i32)],
            "xs_moe_set_device": [i32],
            "xs_moe_current_device": [C.POINTER(i32)],
            "xs_moe_device_alloc": [C.POINTER(vp), sz],
            "xs_moe_device_free": [vp],
            "xs_moe_memcpy_h2d": [vp, vp, sz],
            "xs_moe_memcpy_d2h": [vp, vp, sz],
            "xs_moe_memcpy_d2d": [vp, vp, sz],
            "xs_moe_device_free_bytes": [C.POINTER(sz)],
            "xs_moe_stream_synchronize": [vp],
            "xs_moe_comm_available": [],
            "xs_moe_comm_unique_id": [vp],
            "xs_moe_comm_create": [C.POINTER(vp), vp, i32, i32],
            "xs_moe_comm_destroy": [vp],
            "xs_moe_comm_abort": [vp],
            "xs_moe_comm_async_error": [vp, C.POINTER(i32)],
            "xs_moe_comm_all_gather": [vp, vp, vp, sz, vp],
            "xs_moe_comm_barrier": [vp, vp, vp],
            "xs_moe_comm_all_to_all_v": [vp, i32, vp, C.POINTER(sz), C.POINTER(sz), vp, C.POINTER(sz), C.POINTER(sz), vp],
            "xs_moe_stream_create": [C.POINTER(vp)],
            "xs_moe_stream_destroy": [vp],
            "xs_moe_event_create": [C.POINTER(vp)],
            "xs_moe_event_destroy": [vp],
            "xs_moe_event_record": [vp, vp],
            "xs_moe_stream_wait_event": [vp, vp],
            "xs_moe_memset_async": [vp, i32, sz, vp],
            "xs_moe_enable_peer_access": [i32],
            "xs_moe_workspace_bytes": [cfgp, C.POINTER(sz)],
            "xs_moe_workspace_init": [vp, sz, vp],
            "xs_moe_forward": [cfgp, wp, vp, vp, vp, sz, vp],
            "xs_moe_forward_host": [cfgp, wp, vp, vp, vp, vp, vp, sz, vp],
            "xs_moe_forward_profile": [cfgp, wp, vp, vp, vp, sz, vp, C.POINTER(C.c_float)],
            "xs_moe_block_workspace_bytes": [cfgp, C.POINTER(sz)],
            "xs_moe_block_forward": [cfgp, wp, vp, vp, C.c_float, vp, vp, sz, vp],
            "xs_moe_rmsnorm": [vp, vp, vp, i32, i32, C.c_float, vp],
            "xs_moe_route": [cfgp, vp, vp, vp, vp, vp, vp, vp, sz, vp],
            "xs_moe_topk": [cfgp, vp, vp, vp, vp, vp],
            "xs_moe_permute": [cfgp, vp, vp, vp, vp, vp, vp, sz, vp],
            "xs_moe_permute_noalloc": [cfgp, vp, vp, vp, vp, vp, vp],
            "xs_moe_grouped_mlp_workspace_bytes": [cfgp, i32, C.POINTER(sz)],
            "xs_moe_grouped_mlp": [cfgp, wp, vp, vp, vp, i32, vp, vp, sz, vp],
            "xs_moe_ep_signal": [i32, i32, vp, i32, vp, vp, vp, vp, vp, vp],
            "xs_moe_grouped_mlp_return_supported": [cfgp, i32, C.POINTER(i32)],
            "xs_moe_grouped_mlp_return": [cfgp, wp, vp, vp, vp, i32, i32, i32, vp, vp, vp, i32, vp, sz, vp],
            "xs_moe_quantize_rows_fp8": [vp, i32, i32, vp, vp, vp],
            "xs_moe_quantize_rows_mxfp8": [vp, i32, i32, vp, vp, vp],
            "xs_moe_gather_rows": [vp, vp, vp, i32, i32, vp],
            "xs_moe_combine": [cfgp, vp, vp, vp, vp, vp, vp],
            "xs_moe_combine_bf16_rows": [cfgp, vp, vp, vp, vp, vp, vp],
            "xs_moe_gather_rows_f32_to_bf16": [vp, vp, vp, i32, i32, vp],
            "xs_moe_check_flags": [vp, vp],
            "xs_moe_probe_mma_rate": [i32, i32, i32, i32, vp, sz, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double), vp],
            "xs_moe_probe_tmem_ld_rate": [i32, i32, i32, i32, vp, sz, C.POINTER(C.c_double), C.POINTER(C.c_double), vp],
            "xs_moe_probe_handoff": [i32, i32, i32, i32, vp, sz, C.POINTER(C.c_double), vp],
            "xs_moe_debug_counters": [vp, C.POINTER(C.c_ulonglong), vp],
            "xs_moe_launch_count": [C.POINTER(C.c_ulonglong)],
            "xs_moe_plan_info": [cfgp, C.POINTER(i32), C.POINTER(i32)],
            "xs_moe_ipc_export": [vp, vp],
            "xs_moe_ipc_import": [vp, C.POINTER(vp)],
            "xs_moe_ipc_close": [vp],
            "xs_moe_ep_plan": [vp, i32, i32, i32, vp, vp, vp, vp],
            "xs_moe_ep_dispatch": [cfgp, i32, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp],
            "xs_moe_ep_return": [cfgp, i32, i32, vp, vp, vp, vp, i32, vp, i32, i32, vp, vp],
        }
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.restype = C.c_int
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        L = lib()
        raise RuntimeError(f"{L.xs_moe_status_string(rc).decode()}: {L.xs_moe_last_error().decode()}")


def make_config(T, H, E, K, I, S, routed_format=BF16, shared_format=BF16, local_begin=0, local_count=None, gemm_impl=0):
    c = XsMoeConfig()
    c.num_tokens, c.hidden, c.num_experts, c.top_k, c.intermediate, c.num_shared = T, H, E, K, I, S
    c.routed_format, c.shared_format = routed_format, shared_format
    c.local_expert_begin = local_begin
    c.local_expert_count = E if local_count is None else local_count
    c.gemm_impl = gemm_impl
    return c


def ptr(t):
    """Device (or host) address of a torch tensor / None."""
    return None if t is None else C.c_void_p(t.data_ptr())


def make_weights(d):
    """d: dict of torch tensors keyed like the oracle's arguments (see synth.make_inputs)."""
    w = XsMoeWeights()
    w.router_w_dev = ptr(d["router_w"])
    w.router_bias_dev = ptr(d.get("router_bias"))
    w.gate_up_w_dev = ptr(d["gate_up_w"])
    w.gate_up_scale_dev = ptr(d.get("gate_up_scale"))
    w.down_w_dev = ptr(d["down_w"])
    w.down_scale_dev = ptr(d.get("down_scale"))
    w.shared_gate_up_w_dev = ptr(d.get("shared_gate_up_w"))
    w.shared_gate_up_scale_dev = ptr(d.get("shared_gate_up_scale"))
    w.shared_down_w_dev = ptr(d.get("shared_down_w"))
    w.shared_down_scale_dev = ptr(d.get("shared_down_scale"))
    return w


def workspace_bytes(cfg):
    n = C.c_size_t(0)
    check(lib().xs_moe_workspace_bytes(C.byref(cfg), C.byref(n)))
    return n.value


def launch_count():
    """Kernels the library has enqueued in this process so far."""
    n = C.c_ulonglong(0)
    check(lib().xs_moe_launch_count(C.byref(n)))
    return int(n.value)
