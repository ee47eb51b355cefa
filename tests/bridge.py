"""torch <-> xstar_cpp.Tensor bridge, bit-exact both ways (the pattern of the reference's tests/bridge.py:
bf16 crosses as uint16 bits, everything else as its own bytes)."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "xstar-infer_b200", "xstar_cpp_py"))
import xstar_cpp  # noqa: E402

_DT = {
    torch.float32: (xstar_cpp.DType.Float32, None),
    torch.bfloat16: (xstar_cpp.DType.BFloat16, torch.uint16),
    torch.int32: (xstar_cpp.DType.Int32, None),
}


def torch_to_cpp(t, dtype=None):
    """dtype overrides the element kind for byte tensors (uint8 -> Float8E4M3 / Float4E2M1x2 / UE8M0)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.uint8:
        if dtype is None:
            raise RuntimeError("byte tensors need an explicit xstar dtype")
        return xstar_cpp.from_numpy_raw(t.numpy(), list(t.shape), dtype)
    xd, view = _DT[t.dtype]
    a = (t.view(view) if view is not None else t).numpy()
    return xstar_cpp.from_numpy_raw(a, list(t.shape), xd)


def cpp_to_torch(t, ref_shape):
    raw = xstar_cpp.to_numpy_raw(t)
    if t.dtype() == xstar_cpp.DType.Float32:
        return torch.from_numpy(raw.view(np.float32).reshape(ref_shape).copy())
    if t.dtype() == xstar_cpp.DType.BFloat16:
        return torch.from_numpy(raw.view(np.uint16).reshape(ref_shape).copy()).view(torch.bfloat16)
    if t.dtype() == xstar_cpp.DType.Int32:
        return torch.from_numpy(raw.view(np.int32).reshape(ref_shape).copy())
    return torch.from_numpy(raw.reshape(ref_shape).copy())
