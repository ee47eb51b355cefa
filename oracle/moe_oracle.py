"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the product
path never does.  `libxs_moe_oracle.so` is the plain-C restatement in moe_oracle.c; `_ref/libxsref.so`
is the reference's own CPU ops compiled in place and composed by ref_compose.cpp.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

F32, BF16, BF16_REFCPU, FP8, FP4 = 0, 1, 2, 3, 4


class _Dims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("T", "H", "E", "K", "I", "S")]


class _Args(C.Structure):
    _fields_ = [
        ("d", _Dims),
        ("mode", C.c_int32),
        ("threads", C.c_int32),
        ("x", C.c_void_p),
        ("router_w", C.c_void_p),
        ("router_bias", C.c_void_p),
        ("gate_up_w", C.c_void_p),
        ("gate_up_scale", C.c_void_p),
        ("down_w", C.c_void_p),
        ("down_scale", C.c_void_p),
        ("shared_gate_up_w", C.c_void_p),
        ("shared_gate_up_scale", C.c_void_p),
        ("shared_down_w", C.c_void_p),
        ("shared_down_scale", C.c_void_p),
        ("out", C.c_void_p),
        ("logits", C.c_void_p),
        ("topk_ids", C.c_void_p),
        ("topk_w", C.c_void_p),
        ("counts", C.c_void_p),
        ("offsets", C.c_void_p),
        ("perm", C.c_void_p),
        ("inv", C.c_void_p),
        ("y_rows", C.c_void_p),
        ("token_subset", C.c_void_p),
        ("n_subset", C.c_int32),
    ]


def reference_root():
    """The reference checkout: $XSTAR_REFERENCE_ROOT, else a directory named `reference` beside this repository."""
    return os.environ.get("XSTAR_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(force=False):
    """Compile the oracle (and the reference composition when the reference tree is present)."""
    so = os.path.join(_HERE, "libxs_moe_oracle.so")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(_HERE, "moe_oracle.c")):
        subprocess.run(["make", "-C", _HERE, "libxs_moe_oracle.so"], check=True, capture_output=True)
    ref = os.path.join(_HERE, "_ref", "libxsref.so")
    if os.path.isdir(os.path.join(reference_root(), "xstar_cpp", "src")) and (force or not os.path.exists(ref)):
        subprocess.run(["make", "-C", _HERE, "ref"], check=True, capture_output=True)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(os.path.join(_HERE, "libxs_moe_oracle.so"))
        _lib.xso_moe_forward.argtypes = [C.POINTER(_Args)]
        _lib.xso_moe_forward.restype = C.c_int
        _lib.xso_f32_to_e4m3.argtypes = [C.c_float]
        _lib.xso_f32_to_e4m3.restype = C.c_uint8
        _lib.xso_e4m3_to_f32.argtypes = [C.c_uint8]
        _lib.xso_e4m3_to_f32.restype = C.c_float
        _lib.xso_f32_to_e2m1.argtypes = [C.c_float]
        _lib.xso_f32_to_e2m1.restype = C.c_uint8
        _lib.xso_e2m1_to_f32.argtypes = [C.c_uint8]
        _lib.xso_e2m1_to_f32.restype = C.c_float
        _lib.xso_f32_to_e8m0_ceil.argtypes = [C.c_float]
        _lib.xso_f32_to_e8m0_ceil.restype = C.c_uint8
        _lib.xso_e8m0_to_f32.argtypes = [C.c_uint8]
        _lib.xso_e8m0_to_f32.restype = C.c_float
        _lib.xso_f32_to_bf16.argtypes = [C.c_float]
        _lib.xso_f32_to_bf16.restype = C.c_uint16
        _lib.xso_expert_mlp.restype = C.c_int
        _lib.xso_expert_mlp.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.xso_quant_act_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _lib.xso_quant_act_fp8.restype = None
        _lib.xso_quant_act_mxfp8.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _lib.xso_quant_act_mxfp8.restype = None
        _lib.xso_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.xso_topk.restype = None
        _lib.xso_permute.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3
        _lib.xso_permute.restype = None
    return _lib


def ref_lib():
    """The reference's own CPU ops (compiled in place); None if it was never built."""
    global _ref
    if _ref is None:
        build()
        p = os.path.join(_HERE, "_ref", "libxsref.so")
        if not os.path.exists(p):
            return None
        _ref = C.CDLL(p)
        _ref.xsref_router_logits.restype = C.c_int
        _ref.xsref_router_logits.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _ref.xsref_moe_experts_combine.restype = C.c_int
        _ref.xsref_moe_experts_combine.argtypes = (
            [C.c_int] * 7 + [C.c_void_p] * 12 + [C.c_int, C.c_void_p, C.c_int]
        )
    return _ref


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype=None):
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if dtype is not None and a.dtype != dtype:
        raise TypeError(f"expected {dtype}, got {a.dtype}")
    return a


def moe_forward(mode, x, router_w, gate_up_w, down_w, top_k, router_bias=None, gate_up_scale=None, down_scale=None,
                shared_gate_up_w=None, shared_down_w=None, shared_gate_up_scale=None, shared_down_scale=None,
                threads=1, token_subset=None, want_y=False):
    """Run the oracle.  Arrays are in STORAGE form (see moe_oracle.h): f32 for mode F32, uint16 bf16 bits
    for x/router_w/bf16 weights, uint8 codes (+ scales) for FP8/FP4.  Returns a dict of numpy arrays."""
    T, H = x.shape
    E = router_w.shape[0]
    I = down_w.shape[2] * (2 if mode == FP4 else 1)
    S = 0 if shared_gate_up_w is None else 1
    keep = [_c(v) for v in (x, router_w, router_bias, gate_up_w, gate_up_scale, down_w, down_scale, shared_gate_up_w,
                            shared_gate_up_scale, shared_down_w, shared_down_scale)]
    out = np.zeros((T, H), np.float32 if mode == F32 else np.uint16)
    res = {
        "out": out,
        "logits": np.zeros((T, E), np.float32),
        "topk_ids": np.zeros((T, top_k), np.int32),
        "topk_w": np.zeros((T, top_k), np.float32),
        "counts": np.zeros(E, np.int32),
        "offsets": np.zeros(E + 1, np.int32),
        "perm": np.zeros(T * top_k, np.int32),
        "inv": np.zeros(T * top_k, np.int32),
    }
    if want_y:
        res["y_rows"] = np.zeros((T * top_k, H), np.float32)
    sub = None if token_subset is None else np.ascontiguousarray(token_subset, dtype=np.int32)
    a = _Args()
    a.d = _Dims(T, H, E, top_k, I, S)
    a.mode, a.threads = mode, threads
    (a.x, a.router_w, a.router_bias, a.gate_up_w, a.gate_up_scale, a.down_w, a.down_scale, a.shared_gate_up_w,
     a.shared_gate_up_scale, a.shared_down_w, a.shared_down_scale) = [_p(v) for v in keep]
    a.out = _p(out)
    for k in ("logits", "topk_ids", "topk_w", "counts", "offsets", "perm", "inv"):
        setattr(a, k, _p(res[k]))
    a.y_rows = _p(res.get("y_rows"))
    a.token_subset = _p(sub)
    a.n_subset = 0 if sub is None else len(sub)
    rc = lib().xso_moe_forward(C.byref(a))
    if rc != 0:
        raise RuntimeError(f"oracle rejected its arguments (code {rc})")
    return res


def topk(logits, bias, k):
    T, E = logits.shape
    logits = _c(logits, np.float32)
    bias = _c(bias, np.float32)
    ids = np.zeros((T, k), np.int32)
    w = np.zeros((T, k), np.float32)
    lib().xso_topk(_p(logits), _p(bias), _p(ids), _p(w), T, E, k)
    return ids, w


def permute(topk_ids, E):
    T, K = topk_ids.shape
    ids = _c(topk_ids, np.int32)
    counts = np.zeros(E, np.int32)
    offsets = np.zeros(E + 1, np.int32)
    perm = np.zeros(T * K, np.int32)
    inv = np.zeros(T * K, np.int32)
    lib().xso_permute(_p(ids), _p(counts), _p(offsets), _p(perm), _p(inv), T, E, K)
    return counts, offsets, perm, inv


def quant_act_fp8(x):
    x = _c(x, np.float32)
    r, c = x.shape
    q = np.zeros((r, c), np.uint8)
    s = np.zeros((r, c // 128), np.float32)
    lib().xso_quant_act_fp8(_p(x), _p(q), _p(s), r, c)
    return q, s


def quant_act_mxfp8(x):
    x = _c(x, np.float32)
    r, c = x.shape
    q = np.zeros((r, c), np.uint8)
    s = np.zeros((r, c // 32), np.uint8)
    lib().xso_quant_act_mxfp8(_p(x), _p(q), _p(s), r, c)
    return q, s


def expert_mlp(mode, x, gate_up_w, down_w):
    rows, H = x.shape
    I = down_w.shape[1]
    x, gate_up_w, down_w = _c(x), _c(gate_up_w), _c(down_w)
    y = np.zeros((rows, H), np.float32)
    rc = lib().xso_expert_mlp(mode, _p(x), _p(gate_up_w), _p(down_w), _p(y), rows, H, I)
    if rc != 0:
        raise RuntimeError("xso_expert_mlp failed")
    return y


def rmsnorm_bf16(x_bits, w_bits, eps):
    """bf16 storage (uint16) in and out; the oracle's restatement of the reference's rmsnorm."""
    x_bits, w_bits = _c(x_bits, np.uint16), _c(w_bits, np.uint16)
    rows, H = x_bits.shape
    out = np.zeros((rows, H), np.uint16)
    L = lib()
    L.xso_rmsnorm_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float]
    L.xso_rmsnorm_bf16.restype = None
    L.xso_rmsnorm_bf16(_p(x_bits), _p(w_bits), _p(out), rows, H, C.c_float(eps))
    return out


def add_bf16(a_bits, b_bits):
    a_bits, b_bits = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    out = np.zeros(a_bits.shape, np.uint16)
    L = lib()
    L.xso_add_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
    L.xso_add_bf16.restype = None
    L.xso_add_bf16(_p(a_bits), _p(b_bits), _p(out), a_bits.size)
    return out


def ref_rmsnorm_bf16(x_bits, w_bits, eps):
    """The reference's own rmsnorm (compiled in place); None if the reference library is absent."""
    r = ref_lib()
    if r is None or not hasattr(r, "xsref_rmsnorm_bf16"):
        return None
    x_bits, w_bits = _c(x_bits, np.uint16), _c(w_bits, np.uint16)
    rows, H = x_bits.shape
    out = np.zeros((rows, H), np.uint16)
    r.xsref_rmsnorm_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float]
    r.xsref_rmsnorm_bf16.restype = C.c_int
    if r.xsref_rmsnorm_bf16(_p(x_bits), _p(w_bits), _p(out), rows, H, C.c_float(eps)) != 0:
        raise RuntimeError("reference rmsnorm failed")
    return out


def ref_add_bf16(a_bits, b_bits):
    r = ref_lib()
    if r is None or not hasattr(r, "xsref_add_bf16"):
        return None
    a_bits, b_bits = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    out = np.zeros(a_bits.shape, np.uint16)
    r.xsref_add_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong]
    r.xsref_add_bf16.restype = C.c_int
    if r.xsref_add_bf16(_p(a_bits), _p(b_bits), _p(out), a_bits.size) != 0:
        raise RuntimeError("reference add failed")
    return out


def ref_router_logits(x_f32, router_w_f32):
    r = ref_lib()
    T, H = x_f32.shape
    E = router_w_f32.shape[0]
    x_f32, router_w_f32 = _c(x_f32, np.float32), _c(router_w_f32, np.float32)
    out = np.zeros((T, E), np.float32)
    if r.xsref_router_logits(_p(x_f32), _p(router_w_f32), _p(out), T, H, E) != 0:
        raise RuntimeError("reference linear failed")
    return out


def ref_experts_combine(bf16, x, gate_up_w, down_w, shared_gate_up_w, shared_down_w, routing, threads=1,
                        token_subset=None):
    """Reference CPU ops (embedding gather + mlp) per expert, then the weighted sum.  `routing` is a dict with
    topk_ids, topk_w, offsets, perm, inv (from the oracle).  Returns (out, y_rows)."""
    r = ref_lib()
    T, H = x.shape
    E, twoI, _ = gate_up_w.shape
    I = twoI // 2
    K = routing["topk_ids"].shape[1]
    S = 0 if shared_gate_up_w is None else 1
    keep = [_c(v) for v in (x, gate_up_w, down_w, shared_gate_up_w, shared_down_w)]
    ids = _c(routing["topk_ids"], np.int32)
    tw = _c(routing["topk_w"], np.float32)
    off = _c(routing["offsets"], np.int32)
    perm = _c(routing["perm"], np.int32)
    inv = _c(routing["inv"], np.int32)
    y = np.zeros((T * K, H), np.float32)
    out = np.zeros((T, H), np.uint16 if bf16 else np.float32)
    sub = None if token_subset is None else np.ascontiguousarray(token_subset, dtype=np.int32)
    rc = r.xsref_moe_experts_combine(int(bool(bf16)), T, H, E, K, I, S, *[_p(v) for v in keep], _p(ids), _p(tw),
                                     _p(off), _p(perm), _p(inv), _p(y), _p(out), threads, _p(sub),
                                     0 if sub is None else len(sub))
    if rc != 0:
        raise RuntimeError(f"reference composition failed ({rc})")
    return out, y
