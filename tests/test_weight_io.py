"""Checkpoint IO of the MoE layer (xstar_cpp.MMapFile / parse_safetensors_header / make_weight_view / load_moe_layer): the
header scanner on well-formed and malformed files, views bit-exact with what was written, experts stacked [gate; up] in all
three storage formats, one rank's slice of the experts, and -- on a GPU -- a layer loaded from a file against the oracle."""
import json
import struct

import numpy as np
import pytest
import torch

from xstar_moe import synth

from bridge import cpp_to_torch, xstar_cpp

_FILE_DTYPE = {torch.float32: "F32", torch.bfloat16: "BF16", torch.uint8: "U8", torch.int32: "I32"}


def _raw(t):
    t = t.detach().cpu().contiguous()
    return (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()


def write_file(path, tensors, metadata=None, header_edit=None, dtype_names=None):
    """tensors: name -> torch tensor (uint8 tensors are written as U8 unless dtype_names overrides, e.g. 'F8_E4M3')."""
    header, blob, off = {}, b"", 0
    for name, t in tensors.items():
        b = _raw(t)
        header[name] = {"dtype": (dtype_names or {}).get(name, _FILE_DTYPE[t.dtype]), "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blob += b
        off += len(b)
        pad = (-off) % 8  # keep every tensor 8-byte aligned inside the data section
        blob += b"\0" * pad
        off += pad
    if metadata is not None:
        header["__metadata__"] = metadata
    text = json.dumps(header)
    if header_edit:
        text = header_edit(text)
    hb = text.encode("utf-8")
    hb += b" " * ((-len(hb)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)) + hb + blob)
    return str(path)


def layer_tensors(d, dims, prefix="model.layers.3.mlp"):
    """The stacked synthetic layer split into the per-expert tensors a checkpoint holds."""
    E, I, fmt = dims["E"], dims["I"], dims["fmt"]
    out, names = {}, {}
    out[f"{prefix}.gate.weight"] = d["router_w"]
    if d.get("router_bias") is not None:
        out[f"{prefix}.gate.e_score_correction_bias"] = d["router_bias"]
    sname = {"fp8": "weight_scale_inv", "fp4": "weight_scale"}.get(fmt)
    for e in range(E):
        p = f"{prefix}.experts.{e}."
        out[p + "gate_proj.weight"], out[p + "up_proj.weight"], out[p + "down_proj.weight"] = d["gate_up_w"][e, :I], d["gate_up_w"][e, I:], d["down_w"][e]
        if fmt == "fp8":
            for k in ("gate_proj.weight", "up_proj.weight", "down_proj.weight"):
                names[p + k] = "F8_E4M3"
        if sname:
            g = d["gate_up_scale"][e]
            half = g.shape[0] // 2
            out[p + f"gate_proj.{sname}"], out[p + f"up_proj.{sname}"], out[p + f"down_proj.{sname}"] = g[:half], g[half:], d["down_scale"][e]
    if dims["S"]:
        p = f"{prefix}.shared_experts."
        out[p + "gate_proj.weight"], out[p + "up_proj.weight"], out[p + "down_proj.weight"] = d["shared_gate_up_w"][:I], d["shared_gate_up_w"][I:], d["shared_down_w"]
        if fmt != "bf16":
            for k in ("gate_proj.weight", "up_proj.weight", "down_proj.weight"):
                names[p + k] = "F8_E4M3"
            g = d["shared_gate_up_scale"]
            half = g.shape[0] // 2
            out[p + "gate_proj.weight_scale_inv"], out[p + "up_proj.weight_scale_inv"] = g[:half], g[half:]
            out[p + "down_proj.weight_scale_inv"] = d["shared_down_scale"]
    return {k: v.contiguous() for k, v in out.items()}, names


def _bytes(t):
    return xstar_cpp.to_numpy_raw(t).tobytes()


def test_header_scan_and_views_are_bit_exact(tmp_path):
    g = torch.Generator().manual_seed(1)
    tensors = {"a.weight": torch.randn((5, 8), generator=g).to(torch.bfloat16), "b": torch.randn(7, generator=g),
               "codes": torch.randint(0, 255, (3, 16), generator=g, dtype=torch.uint8), "idx": torch.arange(6, dtype=torch.int32).reshape(2, 3),
               "empty": torch.zeros((0, 4))}
    path = write_file(tmp_path / "t.safetensors", tensors, metadata={"format": "pt", "note": 'braces } { and "quotes" inside'},
                      dtype_names={"codes": "F8_E4M3"})
    mf = xstar_cpp.MMapFile(path)
    meta = xstar_cpp.parse_safetensors_header(mf)
    assert set(meta) == set(tensors)
    want = {"a.weight": xstar_cpp.DType.BFloat16, "b": xstar_cpp.DType.Float32, "codes": xstar_cpp.DType.Float8E4M3,
            "idx": xstar_cpp.DType.Int32, "empty": xstar_cpp.DType.Float32}
    for name, t in tensors.items():
        m = meta[name]
        assert list(m.shape) == list(t.shape) and m.dtype == want[name]
        assert _bytes(xstar_cpp.make_weight_view(mf, m.offset, m.shape, m.dtype)) == _raw(t)
    with pytest.raises(RuntimeError, match="offset not aligned"):
        xstar_cpp.make_weight_view(mf, meta["b"].offset + 1, [1], xstar_cpp.DType.Float32)
    with pytest.raises(RuntimeError, match="view exceeds mapping"):
        xstar_cpp.make_weight_view(mf, meta["b"].offset, [1 << 20], xstar_cpp.DType.Float32)


@pytest.mark.parametrize("edit,msg", [
    (lambda s: s.replace('"F32"', '"F64"'), "unsupported dtype F64"),
    (lambda s: s.replace('"x"', '"x\\\\n"'), "backslash or non-ASCII"),
    (lambda s: s.replace('"x"', '"xé"'), "backslash or non-ASCII"),
    (lambda s: s.replace('"shape": [2, 3], ', ''), "missing required field"),
    (lambda s: s.replace('[0, 24]', '[0, 20]'), "header inconsistent"),
    (lambda s: s.replace('[0, 24]', '[4096, 4120]'), "out of file bounds"),
    (lambda s: s[:-1], "JSON syntax error"),
    (lambda s: s.replace('[2, 3]', '[2, -3]'), "JSON syntax error"),
    (lambda s: s + " x", "JSON syntax error"),
])
def test_malformed_headers_are_rejected(tmp_path, edit, msg):
    path = write_file(tmp_path / "bad.safetensors", {"x": torch.zeros((2, 3))}, header_edit=edit)
    with pytest.raises(RuntimeError, match=msg):
        xstar_cpp.parse_safetensors_header(xstar_cpp.MMapFile(path))


def test_truncated_files_are_rejected(tmp_path):
    p = tmp_path / "tiny"
    p.write_bytes(b"\x01\x02\x03")
    with pytest.raises(RuntimeError, match="file too small"):
        xstar_cpp.parse_safetensors_header(xstar_cpp.MMapFile(str(p)))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(RuntimeError, match="truncated header"):
        xstar_cpp.parse_safetensors_header(xstar_cpp.MMapFile(str(p)))
    with pytest.raises(RuntimeError, match="mmap: cannot open"):
        xstar_cpp.MMapFile(str(tmp_path / "nope"))


@pytest.mark.parametrize("fmt", ["bf16", "fp8", "fp4"])
def test_experts_are_stacked_gate_then_up_in_every_format(tmp_path, fmt):
    dims = dict(T=4, H=256, E=4, K=2, I=128, S=1, fmt=fmt, bias="zipf")
    d = synth.make_inputs(dims, seed=3)
    tensors, names = layer_tensors(d, dims)
    path = write_file(tmp_path / "layer.safetensors", tensors, dtype_names=names)
    mf = xstar_cpp.MMapFile(path)
    meta = xstar_cpp.parse_safetensors_header(mf)
    w = xstar_cpp.load_moe_layer(mf, meta, "model.layers.3.mlp", 4, 0, 4)
    assert (w.num_experts, w.first_expert, w.expert_count, w.hidden, w.intermediate) == (4, 0, 4, 256, 128)
    kind = {"bf16": xstar_cpp.DType.BFloat16, "fp8": xstar_cpp.DType.Float8E4M3, "fp4": xstar_cpp.DType.Float4E2M1x2}[fmt]
    assert w.gate_up_weight.dtype() == kind and w.gate_up_weight.shape() == list(d["gate_up_w"].shape)
    assert _bytes(w.router_weight) == _raw(d["router_w"]) and _bytes(w.optional("router_bias")) == _raw(d["router_bias"])
    assert _bytes(w.gate_up_weight) == _raw(d["gate_up_w"]) and _bytes(w.down_weight) == _raw(d["down_w"])
    if fmt == "bf16":
        assert w.optional("gate_up_scale") is None
        assert w.optional("shared_gate_up_weight").dtype() == xstar_cpp.DType.BFloat16
    else:
        sk = xstar_cpp.DType.Float32 if fmt == "fp8" else xstar_cpp.DType.UE8M0
        assert w.optional("gate_up_scale").dtype() == sk and w.optional("gate_up_scale").shape() == list(d["gate_up_scale"].shape)
        assert _bytes(w.optional("gate_up_scale")) == _raw(d["gate_up_scale"]) and _bytes(w.optional("down_scale")) == _raw(d["down_scale"])
        assert w.optional("shared_gate_up_weight").dtype() == xstar_cpp.DType.Float8E4M3
        assert _bytes(w.optional("shared_gate_up_scale")) == _raw(d["shared_gate_up_scale"])
    assert _bytes(w.optional("shared_gate_up_weight")) == _raw(d["shared_gate_up_w"])
    assert _bytes(w.optional("shared_down_weight")) == _raw(d["shared_down_w"])
    # one expert-parallel rank's slice: experts [2, 4)
    r = xstar_cpp.load_moe_layer(mf, meta, "model.layers.3.mlp", 4, 2, 2)
    assert r.gate_up_weight.shape()[0] == 2 and _bytes(r.gate_up_weight) == _raw(d["gate_up_w"][2:]) and _bytes(r.down_weight) == _raw(d["down_w"][2:])
    assert _bytes(r.router_weight) == _raw(d["router_w"])  # the router stays whole
    if fmt != "bf16":
        assert _bytes(r.optional("down_scale")) == _raw(d["down_scale"][2:])


def test_loader_errors(tmp_path):
    dims = dict(T=4, H=256, E=4, K=2, I=128, S=0, fmt="bf16", bias=None)
    d = synth.make_inputs(dims, seed=4)
    tensors, names = layer_tensors(d, dims)
    pre = "model.layers.3.mlp"

    def load(t, *a):
        path = write_file(tmp_path / "e.safetensors", t, dtype_names=names)
        mf = xstar_cpp.MMapFile(path)
        return xstar_cpp.load_moe_layer(mf, xstar_cpp.parse_safetensors_header(mf), pre, *a)

    t = dict(tensors)
    del t[f"{pre}.experts.2.up_proj.weight"]
    with pytest.raises(RuntimeError, match=r"missing weight: model.layers.3.mlp.experts.2.up_proj.weight"):
        load(t, 4, 0, 4)
    assert load(t, 4, 0, 2).expert_count == 2  # the slice that does not need the missing tensor loads
    t = dict(tensors)
    t[f"{pre}.experts.1.down_proj.weight"] = t[f"{pre}.experts.1.down_proj.weight"].float()
    with pytest.raises(RuntimeError, match="dtype mismatch: .*experts.1.down_proj.weight"):
        load(t, 4, 0, 4)
    t = dict(tensors)
    t[f"{pre}.experts.3.gate_proj.weight"] = t[f"{pre}.experts.3.gate_proj.weight"][:64].contiguous()
    with pytest.raises(RuntimeError, match="shape mismatch: .*experts.3.gate_proj.weight"):
        load(t, 4, 0, 4)
    with pytest.raises(RuntimeError, match="expert count mismatch"):
        load(tensors, 8, 0, 8)  # the router has 4 rows
    with pytest.raises(RuntimeError, match="expert count mismatch"):
        load(tensors, 4, 3, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-3), ("fp4", 1e-2)])
def test_layer_loaded_from_a_checkpoint_matches_the_oracle(oracle, tmp_path, fmt, tol):
    dims = dict(T=48, H=512, E=8, K=2, I=256, S=1, fmt=fmt, bias=None)
    d = synth.make_inputs(dims, seed=12)
    tensors, names = layer_tensors(d, dims)
    mf = xstar_cpp.MMapFile(write_file(tmp_path / "l.safetensors", tensors, dtype_names=names))
    w = xstar_cpp.load_moe_layer(mf, xstar_cpp.parse_safetensors_header(mf), "model.layers.3.mlp", 8, 0, 8, xstar_cpp.Device.CUDA)
    from bridge import torch_to_cpp
    x = xstar_cpp.to_cuda(torch_to_cpp(d["x"]))
    kw = {k: w.optional(k) for k in ("gate_up_scale", "down_scale", "shared_gate_up_weight", "shared_down_weight", "shared_gate_up_scale",
                                     "shared_down_scale") if w.optional(k) is not None}
    out = cpp_to_torch(xstar_cpp.to_cpu(xstar_cpp.moe(x, w.router_weight, w.gate_up_weight, w.down_weight, 2, **kw)), (48, 512))
    n = synth.to_numpy_storage(d)
    mode = {"bf16": oracle.BF16, "fp4": oracle.FP4}[fmt]
    ref = oracle.moe_forward(mode, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], 2, gate_up_scale=n.get("gate_up_scale"),
                             down_scale=n.get("down_scale"), shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"],
                             shared_gate_up_scale=n.get("shared_gate_up_scale"), shared_down_scale=n.get("shared_down_scale"), threads=4)
    assert synth.rel_l2(out.float().numpy(), synth.bf16_bits_to_f32(ref["out"])) <= tol
