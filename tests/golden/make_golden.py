"""Generates tests/golden/*.npz by running the REFERENCE's own compiled CPU ops (oracle/_ref/libxsref.so,
built from the reference sources where they lie) on small seeded inputs.  Run in a container that has the
reference tree; the fixtures are committed so that the tests need neither the tree nor the library.

    python tests/golden/make_golden.py

Each fixture stores the inputs (storage form) and, from the reference ops: router logits (linear),
per-assignment expert outputs (embedding gather + mlp) and the combined layer output.  Selection and
permutation inputs of the composition come from the oracle (the reference has no such op); they are stored
too so that a change of those rules is caught as well.

block_norm_add.npz holds the two ops either side of the layer in the reference's transformer block: the
reference's bf16 `rmsnorm` (rows with large, tiny and zero entries, two eps values) and bf16 `add`.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "xstar-infer_b200"))

from oracle import moe_oracle as mo  # noqa: E402
from xstar_moe import synth  # noqa: E402

CASES = {
    # name: (dims, seed, bf16?)
    "tiny_f32": (dict(T=9, H=128, E=8, K=2, I=128, S=1, fmt="bf16", bias=None), 11, False),
    "tiny_bf16": (dict(T=9, H=128, E=8, K=2, I=128, S=1, fmt="bf16", bias=None), 12, True),
    "ragged_f32": (dict(T=5, H=128, E=6, K=3, I=128, S=0, fmt="bf16", bias=None), 13, False),
}


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    for name, (cfg, seed, bf16) in CASES.items():
        d = synth.make_inputs(cfg, seed=seed)
        n = synth.to_numpy_storage(d)
        f = {k: (synth.bf16_bits_to_f32(v) if v is not None and v.dtype == np.uint16 else v) for k, v in n.items()}
        logits = mo.ref_router_logits(f["x"], f["router_w"])
        ids, w = mo.topk(logits, None, cfg["K"])
        counts, offsets, perm, inv = mo.permute(ids, cfg["E"])
        routing = dict(topk_ids=ids, topk_w=w, offsets=offsets, perm=perm, inv=inv)
        src = n if bf16 else f
        out, y = mo.ref_experts_combine(bf16, src["x"], src["gate_up_w"], src["down_w"], src.get("shared_gate_up_w"),
                                        src.get("shared_down_w"), routing)
        np.savez_compressed(
            os.path.join(here, name + ".npz"), bf16=np.int32(bf16), K=np.int32(cfg["K"]),
            x=n["x"], router_w=n["router_w"], gate_up_w=n["gate_up_w"], down_w=n["down_w"],
            shared_gate_up_w=n.get("shared_gate_up_w") if cfg["S"] else np.zeros(0, np.uint16),
            shared_down_w=n.get("shared_down_w") if cfg["S"] else np.zeros(0, np.uint16),
            ref_logits=logits, topk_ids=ids, topk_w=w, counts=counts, offsets=offsets, perm=perm, inv=inv,
            ref_y_rows=y, ref_out=out)
        print(name, "written")


def block_fixture(here):
    rng = np.random.default_rng(21)
    R, H = 7, 384
    x = rng.standard_normal((R, H)).astype(np.float32)
    x[1] *= 1e3
    x[2] *= 1e-4
    x[3] = 0.0
    x[4, ::2] = 0.0
    w = (1.0 + 0.25 * rng.standard_normal(H)).astype(np.float32)
    other = rng.standard_normal((R, H)).astype(np.float32) * 3.0
    import torch

    def bits(a):
        return torch.from_numpy(a).to(torch.bfloat16).view(torch.uint16).numpy()

    xb, wb, ob = bits(x), bits(w), bits(other)
    np.savez_compressed(
        os.path.join(here, "block_norm_add.npz"), x=xb, weight=wb, other=ob, eps=np.array([1e-6, 1e-5], np.float32),
        ref_norm_eps0=mo.ref_rmsnorm_bf16(xb, wb, 1e-6), ref_norm_eps1=mo.ref_rmsnorm_bf16(xb, wb, 1e-5), ref_add=mo.ref_add_bf16(xb, ob))
    print("block_norm_add written")


if __name__ == "__main__":
    if mo.ref_lib() is None:
        raise SystemExit("oracle/_ref is not built: the fixtures come from the reference's compiled ops")
    block_fixture(os.path.dirname(os.path.abspath(__file__)))
    main()
