"""The reference-facing boundary: the `xstar_cpp` module (host C++ over the C ABI).  CPU tests cover the
bridge and argument errors; GPU tests call xstar_cpp.moe the way the reference's tests call xstar_cpp.mlp
(tests/ops/test_cpp_cuda_mlp.py in the reference: CUDA op against the CPU oracle)."""
import numpy as np
import pytest
import torch

from xstar_moe import synth

from bridge import cpp_to_torch, torch_to_cpp, xstar_cpp


def test_bridge_roundtrip_is_bit_exact():
    g = torch.Generator().manual_seed(0)
    for t in (torch.randn(3, 5, generator=g), torch.randn(4, 6, generator=g).to(torch.bfloat16),
              torch.randint(-9, 9, (7,), generator=g, dtype=torch.int32)):
        c = torch_to_cpp(t)
        assert c.shape() == list(t.shape) and c.numel() == t.numel()
        back = cpp_to_torch(c, t.shape)
        assert torch.equal(back.view(torch.uint8) if back.dtype != torch.bfloat16 else back.view(torch.uint16),
                           t.view(torch.uint8) if t.dtype != torch.bfloat16 else t.view(torch.uint16))
    b = torch.arange(32, dtype=torch.uint8).reshape(4, 8)
    c = torch_to_cpp(b, xstar_cpp.DType.Float8E4M3)
    assert c.nbytes() == 32 and torch.equal(cpp_to_torch(c, (4, 8)), b)


def test_from_numpy_raw_rejects_wrong_sizes():
    with pytest.raises(RuntimeError, match="itemsize mismatch"):
        xstar_cpp.from_numpy_raw(np.zeros(4, np.float32), [4], xstar_cpp.DType.BFloat16)
    with pytest.raises(RuntimeError, match="byte count mismatch"):
        xstar_cpp.from_numpy_raw(np.zeros(4, np.float32), [5], xstar_cpp.DType.Float32)


def _cpu_tensors(H=128, E=4, I=128, T=3):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    rw = torch.randn(E, H, generator=g).to(torch.bfloat16)
    gu = torch.randn(E, 2 * I, H, generator=g).to(torch.bfloat16)
    dw = torch.randn(E, H, I, generator=g).to(torch.bfloat16)
    return x, rw, gu, dw


def test_moe_argument_errors_match_the_reference_vocabulary():
    x, rw, gu, dw = _cpu_tensors()
    X, RW, GU, DW = (torch_to_cpp(t) for t in (x, rw, gu, dw))
    with pytest.raises(RuntimeError, match="dtype mismatch"):
        xstar_cpp.moe(torch_to_cpp(x.float()), RW, GU, DW, 2)
    with pytest.raises(RuntimeError, match="shape mismatch"):
        xstar_cpp.moe(torch_to_cpp(x[:, :64].contiguous()), RW, GU, DW, 2)
    with pytest.raises(RuntimeError, match="rank mismatch"):
        xstar_cpp.moe(X, RW, torch_to_cpp(gu[0].contiguous()), DW, 2)
    with pytest.raises(RuntimeError, match="top_k out of range"):
        xstar_cpp.moe(X, RW, GU, DW, 5)
    with pytest.raises(RuntimeError, match="expert count mismatch"):
        xstar_cpp.moe(X, RW, torch_to_cpp(gu[:3].contiguous()), DW, 2)
    with pytest.raises(RuntimeError, match="gate_up out must be even"):
        xstar_cpp.moe(X, RW, torch_to_cpp(gu[:, :255].contiguous()), DW, 2)
    with pytest.raises(RuntimeError, match="unsupported device"):  # no host implementation, no fallback
        xstar_cpp.moe(X, RW, GU, DW, 2)


@pytest.mark.gpu
def test_moe_op_matches_oracle_and_does_not_leak(oracle):
    dims = dict(T=70, H=512, E=16, K=4, I=256, S=1, fmt="bf16", bias=None)
    d = synth.make_inputs(dims, seed=2)
    dev = {k: xstar_cpp.to_cuda(torch_to_cpp(v)) for k, v in d.items() if v is not None}
    kw = dict(shared_gate_up_weight=dev["shared_gate_up_w"], shared_down_weight=dev["shared_down_w"])
    out = xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"], **kw)
    assert out.shape() == [70, 512] and out.dtype() == xstar_cpp.DType.BFloat16
    got = cpp_to_torch(xstar_cpp.to_cpu(out), (70, 512)).float().numpy()
    n = synth.to_numpy_storage(d)
    ref = oracle.moe_forward(oracle.BF16, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"],
                             shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"], threads=4)
    assert synth.rel_l2(got, synth.bf16_bits_to_f32(ref["out"])) <= 2e-3
    r = xstar_cpp.moe_route(dev["x"], dev["router_w"], dims["K"])
    for k in ("topk_ids", "counts", "offsets", "perm", "inv"):
        assert np.array_equal(r[k], ref[k]), k
    # leading dims collapse like the reference's mlp: (2, 35, H) -> same values
    x3 = xstar_cpp.to_cuda(torch_to_cpp(d["x"].reshape(2, 35, 512)))
    out3 = xstar_cpp.moe(x3, dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"], **kw)
    assert out3.shape() == [2, 35, 512]
    assert np.array_equal(cpp_to_torch(xstar_cpp.to_cpu(out3), (70, 512)).float().numpy(), got)
    # no-leak probe, as the reference's allocator tests do (100 iterations, 1 MiB slack)
    before = xstar_cpp.cuda_free_bytes()
    for _ in range(100):
        xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"], **kw)
    assert before - xstar_cpp.cuda_free_bytes() <= (1 << 20)


@pytest.mark.gpu
def test_moe_op_rejects_mixed_devices():
    x, rw, gu, dw = _cpu_tensors()
    X, RW, GU, DW = (torch_to_cpp(t) for t in (x, rw, gu, dw))
    with pytest.raises(RuntimeError, match="device mismatch"):
        xstar_cpp.moe(xstar_cpp.to_cuda(X), RW, GU, DW, 2)


@pytest.mark.gpu
def test_moe_op_fp8_experts_through_the_binding(oracle):
    """FP8 e4m3 experts with 128x128 block scales enter as byte tensors tagged Float8E4M3 plus Float32 scale tensors."""
    dims = dict(T=40, H=512, E=8, K=2, I=256, S=1, fmt="fp8", bias=None)
    d = synth.make_inputs(dims, seed=4)
    tag = {"gate_up_w": xstar_cpp.DType.Float8E4M3, "down_w": xstar_cpp.DType.Float8E4M3,
           "shared_gate_up_w": xstar_cpp.DType.Float8E4M3, "shared_down_w": xstar_cpp.DType.Float8E4M3}
    dev = {k: xstar_cpp.to_cuda(torch_to_cpp(v, tag.get(k))) for k, v in d.items() if v is not None}
    out = xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"], gate_up_scale=dev["gate_up_scale"],
                        down_scale=dev["down_scale"], shared_gate_up_weight=dev["shared_gate_up_w"], shared_down_weight=dev["shared_down_w"],
                        shared_gate_up_scale=dev["shared_gate_up_scale"], shared_down_scale=dev["shared_down_scale"])
    got = cpp_to_torch(xstar_cpp.to_cpu(out), (40, 512)).float().numpy()
    n = synth.to_numpy_storage(d)
    ref = oracle.moe_forward(oracle.FP8, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"], gate_up_scale=n["gate_up_scale"],
                             down_scale=n["down_scale"], shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"],
                             shared_gate_up_scale=n["shared_gate_up_scale"], shared_down_scale=n["shared_down_scale"], threads=4)
    assert synth.rel_l2(got, synth.bf16_bits_to_f32(ref["out"])) <= 1e-2
    with pytest.raises(RuntimeError, match="missing scale"):
        xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"])


@pytest.mark.gpu
def test_moe_op_fp4_experts_through_the_binding(oracle):
    """FP4 e2m1 experts enter as packed byte tensors tagged Float4E2M1x2 (last dim counts bytes: K/2) with UE8M0 scale
    tensors (one byte per 32 elements of K); the always-on expert beside them is FP8 with Float32 block scales."""
    dims = dict(T=40, H=512, E=8, K=2, I=256, S=1, fmt="fp4", bias=None)
    d = synth.make_inputs(dims, seed=6)
    D = xstar_cpp.DType
    tag = {"gate_up_w": D.Float4E2M1x2, "down_w": D.Float4E2M1x2, "gate_up_scale": D.UE8M0, "down_scale": D.UE8M0,
           "shared_gate_up_w": D.Float8E4M3, "shared_down_w": D.Float8E4M3}
    dev = {k: xstar_cpp.to_cuda(torch_to_cpp(v, tag.get(k))) for k, v in d.items() if v is not None}
    assert dev["gate_up_w"].shape() == [8, 512, 256] and dev["gate_up_w"].nbytes() == 8 * 512 * 256
    assert dev["gate_up_scale"].shape() == [8, 512, 16] and dev["down_scale"].dtype() == D.UE8M0
    out = xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"], gate_up_scale=dev["gate_up_scale"],
                        down_scale=dev["down_scale"], shared_gate_up_weight=dev["shared_gate_up_w"], shared_down_weight=dev["shared_down_w"],
                        shared_gate_up_scale=dev["shared_gate_up_scale"], shared_down_scale=dev["shared_down_scale"])
    got = cpp_to_torch(xstar_cpp.to_cpu(out), (40, 512)).float().numpy()
    n = synth.to_numpy_storage(d)
    ref = oracle.moe_forward(oracle.FP4, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"], gate_up_scale=n["gate_up_scale"],
                             down_scale=n["down_scale"], shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"],
                             shared_gate_up_scale=n["shared_gate_up_scale"], shared_down_scale=n["shared_down_scale"], threads=4)
    assert synth.rel_l2(got, synth.bf16_bits_to_f32(ref["out"])) <= 1e-2
    with pytest.raises(RuntimeError, match="dtype mismatch"):  # f32 scales next to FP4 experts
        xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"], gate_up_scale=dev["shared_gate_up_scale"],
                      down_scale=dev["shared_down_scale"])


@pytest.mark.gpu
def test_moe_block_op_matches_the_reference_composition(oracle):
    """xstar_cpp.moe_block(x, ln_w, eps, ...) = x + moe(rmsnorm(x)), the call that replaces
    add(attention_x, mlp(rmsnorm(attention_x, ln2_w, eps), ...)) in the reference's transformer block."""
    dims = dict(T=50, H=512, E=8, K=2, I=256, S=0, fmt="bf16", bias=None)
    d = synth.make_inputs(dims, seed=4)
    d["x"] = (d["x"].float() * 3).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(512, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    dev = {k: xstar_cpp.to_cuda(torch_to_cpp(v)) for k, v in d.items() if v is not None}
    NW = xstar_cpp.to_cuda(torch_to_cpp(nw))
    out = xstar_cpp.moe_block(dev["x"], NW, 1e-6, dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"])
    assert out.shape() == [50, 512] and out.dtype() == xstar_cpp.DType.BFloat16
    got = cpp_to_torch(xstar_cpp.to_cpu(out), (50, 512))
    xb = d["x"].view(torch.uint16).numpy()
    xn = oracle.rmsnorm_bf16(xb, nw.view(torch.uint16).numpy(), 1e-6)
    n = synth.to_numpy_storage(d)
    ref = oracle.moe_forward(oracle.BF16, xn, n["router_w"], n["gate_up_w"], n["down_w"], dims["K"], threads=4)
    want = synth.bf16_bits_to_f32(oracle.add_bf16(xb, ref["out"]))
    x32 = d["x"].float().numpy()
    rel = synth.rel_l2(got.float().numpy() - x32, want - x32)
    assert rel <= 2e-3 + 2.0 ** -8 * np.linalg.norm(x32) / np.linalg.norm(want - x32), rel
    # the same call in two steps through the layer op gives the same bits
    xn_dev = xstar_cpp.to_cuda(torch_to_cpp(torch.from_numpy(xn).view(torch.bfloat16)))
    layer = cpp_to_torch(xstar_cpp.to_cpu(xstar_cpp.moe(xn_dev, dev["router_w"], dev["gate_up_w"], dev["down_w"], dims["K"])), (50, 512))
    assert np.array_equal(oracle.add_bf16(xb, layer.view(torch.uint16).numpy()), got.view(torch.uint16).numpy())
    with pytest.raises(RuntimeError, match="shape mismatch"):
        xstar_cpp.moe_block(dev["x"], xstar_cpp.to_cuda(torch_to_cpp(nw[:256].contiguous())), 1e-6, dev["router_w"], dev["gate_up_w"],
                            dev["down_w"], dims["K"])
    with pytest.raises(RuntimeError, match="dtype mismatch"):
        xstar_cpp.moe_block(dev["x"], xstar_cpp.to_cuda(torch_to_cpp(nw.float())), 1e-6, dev["router_w"], dev["gate_up_w"], dev["down_w"],
                            dims["K"])


@pytest.mark.gpu
def test_stream_form_and_recycled_results(oracle):
    """moe_into on a caller's stream with a caller's scratch gives the bits of the synchronous op; results of the synchronous op
    come from the result cache (no device allocation once the size has been seen)."""
    dims = dict(T=40, H=512, E=8, K=2, I=256, S=1, fmt="bf16", bias=None)
    d = synth.make_inputs(dims, seed=8)
    dev = {k: xstar_cpp.to_cuda(torch_to_cpp(v)) for k, v in d.items() if v is not None}
    kw = dict(shared_gate_up_weight=dev["shared_gate_up_w"], shared_down_weight=dev["shared_down_w"])
    ref = cpp_to_torch(xstar_cpp.to_cpu(xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], 2, **kw)), (40, 512))
    stream = torch.cuda.Stream()
    out_t = torch.zeros((40, 512), dtype=torch.bfloat16, device="cuda")
    out = xstar_cpp.from_device_ptr(out_t.data_ptr(), [40, 512], xstar_cpp.DType.BFloat16)
    scratch = xstar_cpp.MoEScratch()
    for _ in range(3):
        xstar_cpp.moe_into(dev["x"], out, scratch, stream.cuda_stream, dev["router_w"], dev["gate_up_w"], dev["down_w"], 2, **kw)
    xstar_cpp.moe_check(scratch, stream.cuda_stream)
    assert scratch.bytes() > 0 and torch.equal(out_t.cpu(), ref)
    with pytest.raises(RuntimeError, match="shape mismatch"):
        bad = xstar_cpp.from_device_ptr(out_t.data_ptr(), [20, 512], xstar_cpp.DType.BFloat16)
        xstar_cpp.moe_into(dev["x"], bad, scratch, 0, dev["router_w"], dev["gate_up_w"], dev["down_w"], 2, **kw)
    # the synchronous op: a dropped result goes to the cache and the next call takes it from there
    xstar_cpp.workspace_trim()
    assert xstar_cpp.result_cache_bytes() == 0
    r1 = xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], 2, **kw)
    del r1
    cached = xstar_cpp.result_cache_bytes()
    assert cached >= 40 * 512 * 2
    r2 = xstar_cpp.moe(dev["x"], dev["router_w"], dev["gate_up_w"], dev["down_w"], 2, **kw)
    assert xstar_cpp.result_cache_bytes() == cached - max(4096, 1 << (40 * 512 * 2 - 1).bit_length())
    assert torch.equal(cpp_to_torch(xstar_cpp.to_cpu(r2), (40, 512)), ref)
