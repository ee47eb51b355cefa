"""CPU tests of the oracle: scalar formats against independent implementations, known answers taken from
the reference's own tests, bit-identity with the reference's compiled CPU ops (golden fixtures, and live
when oracle/_ref is present), and the routing / permutation rules."""
import glob
import os

import numpy as np
import pytest
import torch

from xstar_moe import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _f32(a):
    return synth.bf16_bits_to_f32(a) if a.dtype == np.uint16 else a


# ---- scalar formats ------------------------------------------------------------------------------------
def test_bf16_rne_matches_torch(oracle):
    rng = np.random.default_rng(0)
    v = np.concatenate([rng.standard_normal(5000).astype(np.float32) * 10.0 ** rng.integers(-6, 6, 5000),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38], np.float32)])
    got = np.array([oracle.lib().xso_f32_to_bf16(float(x)) for x in v], np.uint16)
    ref = torch.from_numpy(v).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(got, ref)


def test_e4m3_all_codes_roundtrip(oracle):
    L = oracle.lib()
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    for c in range(256):
        v = L.xso_e4m3_to_f32(c)
        if c & 0x7F == 0x7F:
            assert np.isnan(v)
            continue
        assert v == ref[c], c
        assert L.xso_f32_to_e4m3(v) == c or v == 0.0


def test_e4m3_encode_matches_torch(oracle):
    rng = np.random.default_rng(1)
    v = np.concatenate([rng.uniform(-460, 460, 20000), rng.standard_normal(20000) * 0.01,
                        rng.standard_normal(5000) * 2.0 ** -8, [2.0 ** -10, 3 * 2.0 ** -10, 448.0, 464.0, 1e9, -1e9]]).astype(np.float32)
    got = np.array([oracle.lib().xso_f32_to_e4m3(float(x)) for x in v], np.uint8)
    sat = np.clip(v, -448.0, 448.0)  # the oracle saturates; torch's cast does not
    ref = torch.from_numpy(sat).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got, ref)


def test_e2m1_codes_and_ties(oracle):
    L = oracle.lib()
    vals = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c in range(16):
        v = L.xso_e2m1_to_f32(c)
        assert v == (-1 if c & 8 else 1) * vals[c & 7]
        assert L.xso_f32_to_e2m1(v) == c or v == 0.0
    # midpoints go to the even code
    for mid, code in [(0.25, 0), (0.75, 2), (1.25, 2), (1.75, 4), (2.5, 4), (3.5, 6), (5.0, 6), (7.0, 7), (100.0, 7)]:
        assert L.xso_f32_to_e2m1(mid) == code, mid


def test_e8m0(oracle):
    L = oracle.lib()
    assert L.xso_e8m0_to_f32(127) == 1.0 and L.xso_e8m0_to_f32(120) == 2.0 ** -7
    assert L.xso_f32_to_e8m0_ceil(1.0) == 127 and L.xso_f32_to_e8m0_ceil(1.0001) == 128
    assert L.xso_f32_to_e8m0_ceil(0.26) == 126 and L.xso_f32_to_e8m0_ceil(0.25) == 125


def test_quant_act_fp8_properties(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((7, 256)).astype(np.float32)
    x[3, :128] = 0.0  # an all-zero group must not divide by zero
    q, s = oracle.quant_act_fp8(x)
    deq = torch.from_numpy(q).view(torch.float8_e4m3fn).float().numpy().reshape(7, 2, 128) * s[:, :, None]
    assert np.all(np.isfinite(deq))
    err = np.abs(deq.reshape(7, 256) - x)
    amax = np.abs(x.reshape(7, 2, 128)).max(-1, keepdims=True)
    assert np.all(err.reshape(7, 2, 128) <= amax * 2.0 ** -4 + 1e-12)
    assert np.all(q[3, :128] & 0x7F == 0)
    # the group maximum maps to +-448
    assert np.all(np.abs(deq.reshape(7, 2, 128)).max(-1)[np.arange(7) != 3] > 0)


# ---- known answers from the reference's own tests --------------------------------------------------------
def test_gate_up_order_known_answer(oracle):
    """x = 1, gate rows 0.125, up rows 1.25, hidden 8 (the reference's gate/up order detector,
    tests/ops/test_cpp_mlp.py:127-153): gate = 1, up = 10, act = silu(1) * 10; swapping the halves gives
    silu(10) * 1 instead."""
    H, I = 8, 6
    x = np.ones((2, H), np.float32)
    gu = np.ones((2 * I, H), np.float32)
    gu[:I] = 0.125
    gu[I:] = 1.25
    rng = np.random.default_rng(3)
    dw = rng.standard_normal((H, I)).astype(np.float32)
    y = oracle.expert_mlp(oracle.F32, x, gu, dw)
    act = np.float32(1.0 / (1.0 + np.exp(-1.0)) * 10.0)
    expect = (dw.astype(np.float64) * float(act)).sum(1)
    assert np.allclose(y[0], expect, atol=1e-4) and np.allclose(y[1], expect, atol=1e-4)
    wrong = (dw.astype(np.float64) * (10.0 / (1.0 + np.exp(-10.0)))).sum(1)
    assert not np.allclose(y[0], wrong, atol=1e-2)


def test_expert_mlp_matches_torch_f32(oracle):
    """Same tolerance as the reference's CPU mlp test against PyTorch (tests/ops/test_cpp_mlp.py:34-36)."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(6, 8, generator=g)
    gu = torch.randn(12, 8, generator=g)
    dw = torch.randn(8, 6, generator=g)
    gate, up = (x @ gu.T).chunk(2, dim=-1)
    ref = (torch.nn.functional.silu(gate) * up) @ dw.T
    y = oracle.expert_mlp(oracle.F32, x.numpy(), gu.numpy(), dw.numpy())
    assert np.allclose(y, ref.numpy(), atol=1e-4)


# ---- bit-identity with the reference's compiled CPU ops ----------------------------------------------------
@pytest.mark.parametrize("path", sorted(p for p in glob.glob(os.path.join(GOLDEN, "*.npz")) if not os.path.basename(p).startswith("block_")),
                         ids=os.path.basename)
def test_oracle_reproduces_reference_golden(oracle, path):
    g = np.load(path)
    bf16 = bool(g["bf16"])
    K = int(g["K"])
    S = g["shared_gate_up_w"].size > 0
    conv = (lambda a: a) if bf16 else _f32
    r = oracle.moe_forward(oracle.BF16_REFCPU if bf16 else oracle.F32, conv(g["x"]), conv(g["router_w"]), conv(g["gate_up_w"]),
                           conv(g["down_w"]), K, shared_gate_up_w=conv(g["shared_gate_up_w"]) if S else None,
                           shared_down_w=conv(g["shared_down_w"]) if S else None, want_y=True)
    assert np.array_equal(r["logits"].view(np.uint32), g["ref_logits"].view(np.uint32))
    for k in ("topk_ids", "counts", "offsets", "perm", "inv"):
        assert np.array_equal(r[k], g[k]), k
    assert np.array_equal(r["topk_w"].view(np.uint32), g["topk_w"].view(np.uint32))
    assert np.array_equal(r["y_rows"].view(np.uint32), g["ref_y_rows"].view(np.uint32))
    assert np.array_equal(r["out"].view(np.uint8), g["ref_out"].view(np.uint8))


def test_oracle_equals_live_reference_small_config(oracle):
    """Config 'small_bf16' (T=64, H=1024, E=16, k=2, I=512) against the reference ops compiled in place."""
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built (no reference tree in this container)")
    cfg = synth.CONFIGS["small_bf16"]
    n = synth.to_numpy_storage(synth.make_inputs(cfg, seed=5))
    f = {k: (_f32(v) if v is not None else None) for k, v in n.items()}
    r = oracle.moe_forward(oracle.F32, f["x"], f["router_w"], f["gate_up_w"], f["down_w"], cfg["K"], want_y=True, threads=4)
    assert np.array_equal(oracle.ref_router_logits(f["x"], f["router_w"]).view(np.uint32), r["logits"].view(np.uint32))
    out, y = oracle.ref_experts_combine(False, f["x"], f["gate_up_w"], f["down_w"], None, None, r, threads=4)
    assert np.array_equal(y.view(np.uint32), r["y_rows"].view(np.uint32))
    assert np.array_equal(out.view(np.uint32), r["out"].view(np.uint32))
    rb = oracle.moe_forward(oracle.BF16_REFCPU, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], cfg["K"], want_y=True, threads=4)
    outb, yb = oracle.ref_experts_combine(True, n["x"], n["gate_up_w"], n["down_w"], None, None, rb, threads=4)
    assert np.array_equal(yb.view(np.uint32), rb["y_rows"].view(np.uint32)) and np.array_equal(outb, rb["out"])


def test_rmsnorm_and_add_reproduce_reference_golden(oracle):
    """The two ops around the layer in the reference's transformer block, against outputs of the reference's own
    compiled rmsnorm and add (bf16)."""
    g = np.load(os.path.join(GOLDEN, "block_norm_add.npz"))
    for i in range(2):
        assert np.array_equal(oracle.rmsnorm_bf16(g["x"], g["weight"], float(g["eps"][i])), g["ref_norm_eps%d" % i])
    assert np.array_equal(oracle.add_bf16(g["x"], g["other"]), g["ref_add"])
    # the zero row stays zero (0 * 1/sqrt(eps)), whatever eps
    assert not g["ref_norm_eps0"][3].any()


def test_rmsnorm_and_add_equal_live_reference(oracle):
    if oracle.ref_lib() is None or oracle.ref_rmsnorm_bf16(np.zeros((1, 8), np.uint16), np.zeros(8, np.uint16), 1e-6) is None:
        pytest.skip("oracle/_ref not built (no reference tree in this container)")
    rng = np.random.default_rng(3)
    for rows, H in ((1, 8), (5, 1000), (64, 4096)):
        x = torch.from_numpy(rng.standard_normal((rows, H)).astype(np.float32) * 2.5).to(torch.bfloat16).view(torch.uint16).numpy()
        w = torch.from_numpy(rng.standard_normal(H).astype(np.float32)).to(torch.bfloat16).view(torch.uint16).numpy()
        o = torch.from_numpy(rng.standard_normal((rows, H)).astype(np.float32)).to(torch.bfloat16).view(torch.uint16).numpy()
        assert np.array_equal(oracle.rmsnorm_bf16(x, w, 1e-6), oracle.ref_rmsnorm_bf16(x, w, 1e-6))
        assert np.array_equal(oracle.add_bf16(x, o), oracle.ref_add_bf16(x, o))


def test_rmsnorm_close_to_torch_f32(oracle):
    rng = np.random.default_rng(4)
    x = torch.from_numpy(rng.standard_normal((6, 512)).astype(np.float32)).to(torch.bfloat16)
    w = torch.from_numpy(1 + 0.1 * rng.standard_normal(512).astype(np.float32)).to(torch.bfloat16)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    got = torch.from_numpy(oracle.rmsnorm_bf16(x.view(torch.uint16).numpy(), w.view(torch.uint16).numpy(), 1e-6)).view(torch.bfloat16).float()
    assert torch.allclose(got, ref, rtol=2e-2, atol=1e-3)


def test_threads_do_not_change_results(oracle):
    cfg = dict(T=33, H=128, E=8, K=3, I=128, S=1, fmt="bf16", bias=None)
    n = synth.to_numpy_storage(synth.make_inputs(cfg, seed=6))
    args = (oracle.BF16, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], 3)
    kw = dict(shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"])
    a = oracle.moe_forward(*args, threads=1, **kw)
    b = oracle.moe_forward(*args, threads=5, **kw)
    assert np.array_equal(a["out"], b["out"])
    sub = oracle.moe_forward(*args, threads=3, token_subset=[2, 17, 32], **kw)
    assert np.array_equal(sub["out"][[2, 17, 32]], a["out"][[2, 17, 32]])
    assert np.array_equal(sub["perm"], a["perm"])


# ---- routing rules (no reference implementation: the oracle is normative here) ----------------------------
def test_topk_ties_go_to_lower_id_and_slots_ascend(oracle):
    logits = np.zeros((3, 8), np.float32)
    logits[1] = [1, 5, 5, 0, 5, 0, 0, 0]   # three-way tie for two slots -> experts 1, 2
    logits[2] = [0, 0, 0, 9, 0, 0, 0, 7]
    ids, w = oracle.topk(logits, None, 2)
    assert ids.tolist() == [[0, 1], [1, 2], [3, 7]]
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    assert np.allclose(w[0], [0.5, 0.5]) and w[2, 0] > w[2, 1]


def test_topk_bias_changes_selection_not_weights(oracle):
    logits = np.array([[2.0, 1.0, 0.0, -1.0]], np.float32)
    bias = np.array([0.0, 0.0, 10.0, 10.0], np.float32)
    ids, w = oracle.topk(logits, bias, 2)
    assert ids.tolist() == [[2, 3]]
    e = np.exp(np.array([0.0, -1.0]) - 0.0)
    assert np.allclose(w[0], e / e.sum(), atol=1e-6)


def test_topk_equals_softmax_then_renormalise(oracle):
    rng = np.random.default_rng(7)
    logits = rng.standard_normal((50, 16)).astype(np.float32)
    ids, w = oracle.topk(logits, None, 4)
    p = torch.softmax(torch.from_numpy(logits).double(), -1).numpy()
    for t in range(50):
        top = np.sort(np.argsort(-p[t], kind="stable")[:4])
        assert ids[t].tolist() == top.tolist()
        assert np.allclose(w[t], p[t, top] / p[t, top].sum(), atol=1e-6)


def test_permutation_is_stable_sort(oracle):
    rng = np.random.default_rng(8)
    T, E, K = 300, 16, 3
    ids = np.stack([np.sort(rng.choice(E, K, replace=False)) for _ in range(T)]).astype(np.int32)
    counts, offsets, perm, inv = oracle.permute(ids, E)
    flat = ids.reshape(-1)
    assert np.array_equal(counts, np.bincount(flat, minlength=E))
    assert np.array_equal(offsets, np.concatenate([[0], np.cumsum(counts)]))
    assert np.array_equal(perm, np.argsort(flat, kind="stable"))
    assert np.array_equal(inv[perm], np.arange(T * K))
    # empty experts are legal
    ids2 = np.zeros((4, 1), np.int32)
    c2, o2, p2, i2 = oracle.permute(ids2, 5)
    assert c2.tolist() == [4, 0, 0, 0, 0] and o2.tolist() == [0, 4, 4, 4, 4, 4]


def test_fp8_mode_close_to_dequantised_f32(oracle):
    """FP8 mode against the f32 oracle run on the dequantised weights: bounded by activation quantisation."""
    cfg = dict(T=12, H=256, E=4, K=2, I=128, S=1, fmt="fp8", bias=None)
    d = synth.make_inputs(cfg, seed=9)
    n = synth.to_numpy_storage(d)

    def deq(codes, scales):
        w = torch.from_numpy(codes).view(torch.float8_e4m3fn).float()
        s = torch.from_numpy(scales).repeat_interleave(128, -2).repeat_interleave(128, -1)
        return (w * s).numpy()

    r8 = oracle.moe_forward(oracle.FP8, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], 2, gate_up_scale=n["gate_up_scale"],
                            down_scale=n["down_scale"], shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"],
                            shared_gate_up_scale=n["shared_gate_up_scale"], shared_down_scale=n["shared_down_scale"])
    r32 = oracle.moe_forward(oracle.F32, _f32(n["x"]), _f32(n["router_w"]), deq(n["gate_up_w"], n["gate_up_scale"]),
                             deq(n["down_w"], n["down_scale"]), 2, shared_gate_up_w=deq(n["shared_gate_up_w"], n["shared_gate_up_scale"]),
                             shared_down_w=deq(n["shared_down_w"], n["shared_down_scale"]))
    assert np.array_equal(r8["topk_ids"], r32["topk_ids"])
    assert synth.rel_l2(_f32(r8["out"]), r32["out"]) < 6e-2
