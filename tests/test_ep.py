"""Expert parallelism: the host-side planning on its own, the whole exchange on two CPU ranks (gloo) with a
stand-in for the device ops, and -- where two GPUs are visible -- the real thing over NCCL."""
import ctypes as C
import datetime
import os
import sys
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "xstar-infer_b200"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from xstar_moe import capi, ep, synth  # noqa: E402


# ---- planning (numpy only) --------------------------------------------------------------------------------------
def test_plan_splits_and_maps():
    rng = np.random.default_rng(0)
    R, E = 4, 16
    all_counts = rng.integers(0, 5, size=(R, E))
    all_counts[2, 4:8] = 0  # a rank that sends nothing to rank 1
    plans = [ep.EpPlan(all_counts, r) for r in range(R)]
    for r, p in enumerate(plans):
        assert p.send_splits.sum() == all_counts[r].sum()
        for d in range(R):
            assert p.send_splits[d] == plans[d].recv_splits[r]  # what r sends to d is what d expects from r
        # regroup maps are inverse permutations
        assert np.array_equal(np.sort(p.grouped_from_arrival), np.arange(p.n_recv))
        assert np.array_equal(p.grouped_from_arrival[p.arrival_from_grouped], np.arange(p.n_recv))
        # grouped order is (expert, source, token): label every arrival row and check
        labels = []
        for s in range(R):
            for e in range(p.El):
                labels += [(e, s, i) for i in range(int(p.recv_counts[s, e]))]
        grouped = [labels[a] for a in p.grouped_from_arrival]
        assert grouped == sorted(grouped)
        assert np.array_equal(np.diff(p.offsets_local), p.recv_counts.sum(0))


def test_plan_rejects_uneven_sharding():
    with pytest.raises(ValueError, match="expert count mismatch"):
        ep.EpPlan(np.zeros((3, 8), np.int64), 0)


def test_peer_layout_formulas_agree_with_the_plan():
    """The peer-memory exchange addresses rows by closed formulas over the (R, E) count matrix (csrc/xs_ep.cuh):
        row in the owner's buffer  = offsets_local_owner[e mod El] + sum_{s' < s} counts[s'][e] + j
        row in the source's buffer = exclusive prefix of counts[s] at e + j
    Restated here in numpy and checked against EpPlan's regroup maps: both describe the same grouped order."""
    rng = np.random.default_rng(3)
    R, E = 4, 16
    El = E // R
    counts = rng.integers(0, 6, size=(R, E))
    counts[1, :] = 0          # a rank without tokens
    counts[:, 5] = 0          # an expert nobody chose
    col = counts.sum(0)
    for d in range(R):
        plan = ep.EpPlan(counts, d)
        offsets_local = np.concatenate([[0], np.cumsum(col[d * El:(d + 1) * El])])
        assert np.array_equal(offsets_local, plan.offsets_local)
        # label every arrival row (all-to-all order: source, expert, j) and map it through the formula
        grouped_of = []
        for s in range(R):
            for el in range(El):
                e = d * El + el
                for j in range(int(counts[s, e])):
                    grouped_of.append(offsets_local[el] + counts[:s, e].sum() + j)
        grouped_of = np.array(grouped_of, dtype=np.int64)
        assert np.array_equal(np.sort(grouped_of), np.arange(plan.n_recv))  # a bijection onto the buffer's rows
        # plan.arrival_from_grouped[a] is the grouped row of arrival row a (the inverse of grouped_from_arrival)
        assert np.array_equal(grouped_of, plan.arrival_from_grouped), "formula and regroup map disagree"
    # the way back: row g of the owner's buffer returns to (source s, row prefix_s[e] + j)
    prefix = np.concatenate([np.zeros((R, 1), np.int64), np.cumsum(counts, 1)[:, :-1]], 1)
    seen = [np.zeros(int(counts[s].sum()), bool) for s in range(R)]
    for d in range(R):
        for el in range(El):
            e = d * El + el
            for s in range(R):
                for j in range(int(counts[s, e])):
                    row = prefix[s, e] + j
                    assert not seen[s][row]
                    seen[s][row] = True
    assert all(v.all() for v in seen)  # every permuted row of every source gets exactly one result


# ---- two CPU ranks over gloo: the exchange logic end to end ----------------------------------------------------------
class OracleOps:
    """Stand-in for the device ops so that the host logic of ep.ExpertParallelMoE runs on CPU ranks: each call is
    the CPU oracle's restatement of the corresponding C-ABI stage (test infrastructure, never shipped)."""

    def __init__(self, oracle, dims, d_local, shared):
        self.o, self.dims, self.d, self.shared = oracle, dims, d_local, shared
        self.H, self.K, self.E = dims["H"], dims["K"], dims["E"]

    @staticmethod
    def _bits(t):
        return t.contiguous().view(torch.uint16).numpy()

    def route(self, x, router_w, router_bias):
        import ctypes as C
        xf, rwf = x.float().numpy(), router_w.float().numpy()
        logits = np.zeros((x.shape[0], self.E), np.float32)
        self.o.lib().xso_router_logits(C.c_void_p(xf.ctypes.data), C.c_void_p(rwf.ctypes.data), C.c_void_p(logits.ctypes.data),
                                       x.shape[0], self.H, self.E)
        ids, w = self.o.topk(logits, None if router_bias is None else router_bias.numpy(), self.K)
        return torch.from_numpy(ids), torch.from_numpy(w)

    def permute(self, ids):
        return tuple(torch.from_numpy(a) for a in self.o.permute(ids.numpy(), self.E))

    def payload(self, x):
        return [x]

    def gather(self, src, index):
        return src.index_select(0, index.long())

    def return_rows(self, y_grouped, index):
        return self.gather(y_grouped, index)

    def grouped_mlp(self, payload, offsets_local, n_rows):
        rows = payload[0]
        y = torch.zeros((n_rows, self.H), dtype=torch.float32)
        off = offsets_local.numpy()
        gu, dw = self._bits(self.d["gate_up_w"]), self._bits(self.d["down_w"])
        for e in range(len(off) - 1):
            if off[e + 1] > off[e]:
                y[off[e]:off[e + 1]] = torch.from_numpy(self.o.expert_mlp(self.o.BF16, self._bits(rows[off[e]:off[e + 1]]), gu[e], dw[e]))
        return y

    def shared_mlp(self, x, payload):
        return torch.from_numpy(self.o.expert_mlp(self.o.BF16, self._bits(x), self._bits(self.shared["shared_gate_up_w"]),
                                                  self._bits(self.shared["shared_down_w"])))

    def combine(self, y, inv, w, shared):
        T, K = w.shape
        acc = np.zeros((T, self.H), np.float32)
        yn, wn, invn = y.numpy(), w.numpy(), inv.numpy().reshape(T, K)
        for j in range(K):
            acc = acc + wn[:, j:j + 1] * yn[invn[:, j]]
        if shared is not None:
            acc = acc + shared.numpy()
        return torch.from_numpy(acc).to(torch.bfloat16)


def _cpu_rank(rank, world, port, dims, seed, result_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import moe_oracle as oracle

        d = synth.make_inputs(dict(dims, T=dims["T"] * world), seed=seed)  # the global problem, same on every rank
        T, El = dims["T"], dims["E"] // world
        x_local = d["x"][rank * T:(rank + 1) * T].contiguous()
        d_local = dict(gate_up_w=d["gate_up_w"][rank * El:(rank + 1) * El], down_w=d["down_w"][rank * El:(rank + 1) * El])
        ops = OracleOps(oracle, dims, d_local, d)
        layer = ep.ExpertParallelMoE(ops, d["router_w"], d["router_bias"], dims["E"], dims["K"], dims["S"])
        out = layer.forward(x_local)
        np.save(os.path.join(result_dir, f"out{rank}.npy"), out.view(torch.uint16).numpy())
        np.save(os.path.join(result_dir, f"recv{rank}.npy"), np.array([layer.last_plan.n_recv]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ep_on_cpu_ranks_equals_single_process_oracle(oracle, tmp_path, world):
    dims = dict(T=24, H=128, E=8, K=3, I=128, S=1, fmt="bf16", bias=None)
    port = 29600 + world
    mp.spawn(_cpu_rank, args=(world, port, dims, 17, str(tmp_path)), nprocs=world, join=True)
    d = synth.make_inputs(dict(dims, T=dims["T"] * world), seed=17)
    n = synth.to_numpy_storage(d)
    ref = oracle.moe_forward(oracle.BF16, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"],
                             shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"])
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    assert np.array_equal(got, ref["out"]), "expert-parallel result differs from the single-process layer"
    total = sum(int(np.load(tmp_path / f"recv{r}.npy")[0]) for r in range(world))
    assert total == dims["T"] * world * dims["K"]


# ---- two GPUs over NCCL ---------------------------------------------------------------------------------------------
def _gpu_rank(rank, world, port, dims, seed, result_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        d = synth.make_inputs(dict(dims, T=dims["T"] * world), seed=seed)  # CPU generator: identical on every rank
        T, El = dims["T"], dims["E"] // world
        keys = ["gate_up_w", "down_w", "gate_up_scale", "down_scale"]
        local = {k: d[k][rank * El:(rank + 1) * El].contiguous().cuda() for k in keys if d.get(k) is not None}
        local["router_w"] = d["router_w"].cuda()
        shared = {k: v.cuda() for k, v in d.items() if k.startswith("shared_") and v is not None} if dims["S"] else None
        ops = ep.CudaOps(dict(dims), local, shared, rank, world)
        bias = d["router_bias"].cuda() if d["router_bias"] is not None else None
        layer = ep.ExpertParallelMoE(ops, local["router_w"], bias, dims["E"], dims["K"], dims["S"])
        x_local = d["x"][rank * T:(rank + 1) * T].contiguous().cuda()
        out = layer.forward(x_local)
        out2 = layer.forward(x_local)
        ops.check()
        torch.cuda.synchronize()
        assert torch.equal(out, out2)
        np.save(os.path.join(result_dir, f"out{rank}.npy"), out.cpu().view(torch.uint16).numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-3), ("fp8", 1e-2), ("fp4", 1e-2)])
def test_ep_on_gpus_matches_oracle(oracle, tmp_path, fmt, tol):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs on one box")
    dims = dict(T=96, H=512, E=16, K=4, I=256, S=1, fmt=fmt, bias=None)
    mp.spawn(_gpu_rank, args=(world, 29650 + ["bf16", "fp8", "fp4"].index(fmt), dims, 23, str(tmp_path)), nprocs=world, join=True)
    d = synth.make_inputs(dict(dims, T=dims["T"] * world), seed=23)
    n = synth.to_numpy_storage(d)
    mode = {"bf16": oracle.BF16, "fp8": oracle.FP8, "fp4": oracle.FP4}[fmt]
    ref = oracle.moe_forward(mode, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"], gate_up_scale=n.get("gate_up_scale"),
                             down_scale=n.get("down_scale"), shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"],
                             shared_gate_up_scale=n.get("shared_gate_up_scale"), shared_down_scale=n.get("shared_down_scale"), threads=8)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    rel = synth.rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(ref["out"]))
    assert rel <= tol, rel


# ---- the exchange over peer memory ------------------------------------------------------------------------------------
def _oracle_ref(oracle, dims, d):
    n = synth.to_numpy_storage(d)
    mode = {"bf16": oracle.BF16, "fp8": oracle.FP8, "fp4": oracle.FP4}[dims["fmt"]]
    return oracle.moe_forward(mode, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"], router_bias=n.get("router_bias"),
                              gate_up_scale=n.get("gate_up_scale"),
                              down_scale=n.get("down_scale"), shared_gate_up_w=n["shared_gate_up_w"], shared_down_w=n["shared_down_w"],
                              shared_gate_up_scale=n.get("shared_gate_up_scale"), shared_down_scale=n.get("shared_down_scale"), threads=8)


def _virtual_ranks(dims, R, seed, capacity=None):
    """R expert-parallel ranks inside one process on one GPU: every rank has its own ops, buffers and index tables, and
    the 'peer' pointers are simply the other ranks' buffers on the same device.  Exercises every kernel and all the
    index arithmetic of the peer exchange without a second GPU; phases run rank after rank on one stream, which is
    what the barriers between them guarantee on real ranks."""
    d = synth.make_inputs(dict(dims, T=dims["T"] * R), seed=seed)
    T, El = dims["T"], dims["E"] // R
    keys = ["gate_up_w", "down_w", "gate_up_scale", "down_scale"]
    shared = {k: v.cuda() for k, v in d.items() if k.startswith("shared_") and v is not None}
    router_w = d["router_w"].cuda()
    ranks = []
    for r in range(R):
        local = {k: d[k][r * El:(r + 1) * El].contiguous().cuda() for k in keys if d.get(k) is not None}
        local["router_w"] = router_w
        ops = ep.CudaOps(dict(dims), local, shared, r, R)
        px = ep.PeerExchange(dims, r, R, capacity)
        bias = d["router_bias"].cuda() if d.get("router_bias") is not None else None
        ranks.append(dict(ops=ops, px=px, x=d["x"][r * T:(r + 1) * T].contiguous().cuda(), bias=bias))
    for k in ranks:
        k["px"].connect([q["px"].rows.data_ptr() for q in ranks], [q["px"].scales.data_ptr() for q in ranks],
                        [q["px"].back.data_ptr() for q in ranks])
    return d, ranks


def _run_virtual(ranks):
    for k in ranks:
        k["ids"], k["w"] = k["ops"].route(k["x"], k["ops"].keep[0]["router_w"], k["bias"])
        k["counts"], k["offsets"], k["perm"], k["inv"] = k["ops"].permute(k["ids"])
    all_counts = torch.cat([k["counts"] for k in ranks])
    for k in ranks:
        k["px"].plan(all_counts)
        k["px"].dispatch(k["x"], k["ids"], k["inv"], k["offsets"], k["ops"].ws)
    for k in ranks:
        px = k["px"]
        y = k["ops"].grouped_mlp([px.rows, px.scales if px.fmt != 0 else None], px.offsets_local, px.capacity)
        px.give_back(y, all_counts, k["ops"].ws)
    outs = []
    for k in ranks:
        sh = k["ops"].shared_mlp(k["x"], None)
        outs.append(k["ops"].combine(k["px"].back, k["inv"], k["w"], sh))
    return all_counts, outs


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-3), ("fp8", 1e-2), ("fp4", 1e-2)])
def test_peer_exchange_virtual_ranks_match_oracle(oracle, fmt, tol):
    R = 4
    dims = dict(T=40, H=512, E=16, K=4, I=256, S=1, fmt=fmt, bias=None)
    d, ranks = _virtual_ranks(dims, R, seed=31)
    try:
        all_counts, outs = _run_virtual(ranks)
        for k in ranks:
            k["ops"].check()
        torch.cuda.synchronize()
        # the device-side plan equals the host-side one
        ac = all_counts.view(R, dims["E"]).cpu().numpy()
        for r, k in enumerate(ranks):
            assert np.array_equal(k["px"].offsets_local.cpu().numpy(), ep.EpPlan(ac, r).offsets_local)
        got = torch.cat(outs).cpu().view(torch.uint16).numpy()
        ref = _oracle_ref(oracle, dims, d)
        rel = synth.rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(ref["out"]))
        assert rel <= tol, rel
    finally:
        torch.cuda.synchronize()
        for k in ranks:
            k["px"].close()


@pytest.mark.gpu
@pytest.mark.parametrize("R,dims", [
    (8, dict(T=16, H=256, E=32, K=6, I=128, S=1, fmt="fp8", bias="zipf")),   # skewed routing: experts (and ranks) with no rows at all
    (2, dict(T=33, H=256, E=8, K=1, I=128, S=1, fmt="bf16", bias="zipf")),   # top-1, ragged token count
    (4, dict(T=1, H=512, E=16, K=4, I=256, S=1, fmt="fp4", bias=None)),      # one token per rank
    (8, dict(T=8, H=256, E=8, K=2, I=128, S=1, fmt="bf16", bias=None)),      # one expert per rank
])
def test_peer_exchange_virtual_ranks_edge_cases(oracle, R, dims):
    d, ranks = _virtual_ranks(dims, R, seed=77)
    try:
        all_counts, outs = _run_virtual(ranks)
        for k in ranks:
            k["ops"].check()
        torch.cuda.synchronize()
        ac = all_counts.view(R, dims["E"]).cpu().numpy()
        assert ac.sum() == R * dims["T"] * dims["K"]
        got = torch.cat(outs).cpu().view(torch.uint16).numpy()
        ref = _oracle_ref(oracle, dims, d)
        assert np.array_equal(torch.cat([k["ids"] for k in ranks]).cpu().numpy(), ref["topk_ids"]), "routing differs from the oracle"
        rel = synth.rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(ref["out"]))
        assert rel <= (2e-3 if dims["fmt"] == "bf16" else 1e-2), rel
    finally:
        torch.cuda.synchronize()
        for k in ranks:
            k["px"].close()


@pytest.mark.gpu
def test_peer_exchange_flags_a_buffer_that_is_too_small(oracle):
    R = 2
    dims = dict(T=32, H=256, E=8, K=2, I=128, S=1, fmt="bf16", bias=None)
    d, ranks = _virtual_ranks(dims, R, seed=5, capacity=8)  # far fewer rows than the routing sends
    try:
        # plan and dispatch only: rows that do not fit are skipped and flagged; an overflowed plan is never handed on
        # to the expert GEMMs or the return trip
        for k in ranks:
            k["ids"], k["w"] = k["ops"].route(k["x"], k["ops"].keep[0]["router_w"], k["bias"])
            k["counts"], k["offsets"], k["perm"], k["inv"] = k["ops"].permute(k["ids"])
        all_counts = torch.cat([k["counts"] for k in ranks])
        for k in ranks:
            k["px"].plan(all_counts)
            k["px"].dispatch(k["x"], k["ids"], k["inv"], k["offsets"], k["ops"].ws)
        torch.cuda.synchronize()
        assert int(ranks[0]["px"].offsets_local[-1]) > 8
        with pytest.raises(RuntimeError, match="out-of-range index"):
            for k in ranks:
                k["ops"].check()
    finally:
        torch.cuda.synchronize()
        for k in ranks:
            k["px"].close()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["bf16", "fp4"])
def test_peer_step_replays_as_cuda_graph_on_one_rank(oracle, fmt):
    """World size 1 (no collective): the whole step -- route, permute, plan, dispatch, grouped MLP, return, always-on
    expert on its side stream, combine -- captured once and replayed on new inputs."""
    dims = dict(T=48, H=512, E=16, K=4, I=256, S=1, fmt=fmt, bias=None)
    d, ranks = _virtual_ranks(dims, 1, seed=41)
    k = ranks[0]
    try:
        layer = ep.ExpertParallelMoE(k["ops"], k["ops"].keep[0]["router_w"], None, dims["E"], dims["K"], dims["S"])
        eager = layer.forward_peer(k["x"], k["px"])
        x_static = k["x"].clone()
        graph, out_static = layer.capture_peer(x_static, k["px"])
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out_static, eager)
        x2 = torch.roll(k["x"], 7, dims=0).contiguous()  # other tokens, other routing counts
        x_static.copy_(x2)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out_static, layer.forward_peer(x2, k["px"]))
        k["ops"].check()
    finally:
        torch.cuda.synchronize()
        k["px"].close()


def _gpu_rank_peer(rank, world, port, dims, seed, result_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    px = None
    done = False
    try:
        d = synth.make_inputs(dict(dims, T=dims["T"] * world), seed=seed)
        T, El = dims["T"], dims["E"] // world
        keys = ["gate_up_w", "down_w", "gate_up_scale", "down_scale"]
        local = {k: d[k][rank * El:(rank + 1) * El].contiguous().cuda() for k in keys if d.get(k) is not None}
        local["router_w"] = d["router_w"].cuda()
        shared = {k: v.cuda() for k, v in d.items() if k.startswith("shared_") and v is not None}
        ops = ep.CudaOps(dict(dims), local, shared, rank, world)
        layer = ep.ExpertParallelMoE(ops, local["router_w"], None, dims["E"], dims["K"], dims["S"])
        px = ep.PeerExchange(dims, rank, world)
        px.connect_ipc()
        x_local = d["x"][rank * T:(rank + 1) * T].contiguous().cuda()
        via_nccl = layer.forward(x_local)
        out = layer.forward_peer(x_local, px)
        out2 = layer.forward_peer(x_local, px)
        ops.check()
        torch.cuda.synchronize()
        assert torch.equal(out, out2)
        assert torch.equal(out, via_nccl), "peer-memory exchange and all-to-all exchange disagree"
        # the same step captured once and replayed as a CUDA graph
        x_static = x_local.clone()
        graph, out_static = layer.capture_peer(x_static, px)
        for _ in range(2):
            out_static.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out_static, out)
        ops.check()
        graph.reset()  # a live graph holds the communicator: release it before the process group goes away
        del graph
        np.save(os.path.join(result_dir, f"out{rank}.npy"), out.cpu().view(torch.uint16).numpy())
        done = True
    finally:
        torch.cuda.synchronize()
        if done:  # a rank that failed leaves without a collective: the other one must not wait for it
            dist.barrier()
            px.close()
            dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-3), ("fp8", 1e-2), ("fp4", 1e-2)])
def test_ep_peer_exchange_on_gpus_matches_oracle(oracle, tmp_path, fmt, tol):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs on one box")
    dims = dict(T=96, H=512, E=16, K=4, I=256, S=1, fmt=fmt, bias=None)
    mp.spawn(_gpu_rank_peer, args=(world, 29660 + ["bf16", "fp8", "fp4"].index(fmt), dims, 23, str(tmp_path)), nprocs=world, join=True)
    d = synth.make_inputs(dict(dims, T=dims["T"] * world), seed=23)
    ref = _oracle_ref(oracle, dims, d)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    rel = synth.rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(ref["out"]))
    assert rel <= tol, rel


@pytest.mark.gpu
def test_signal_barrier_passes_alone_and_gives_up_when_a_peer_never_arrives():
    """xs_moe_ep_signal on one GPU: a one-rank barrier passes at once and carries the counts; with a second rank that never
    stores its flag the bounded wait runs out (about two seconds), the kernel returns, and the status word reports it."""
    L = capi.lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    E = 8
    counts = torch.arange(1, E + 1, dtype=torch.int32, device="cuda")
    all_counts = torch.zeros(2 * E, dtype=torch.int32, device="cuda")
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    t_counts = torch.tensor([all_counts.data_ptr()], dtype=torch.int64, device="cuda")
    t_flags = torch.tensor([flags.data_ptr()], dtype=torch.int64, device="cuda")
    for step in (1, 2, 3):
        capi.check(L.xs_moe_ep_signal(1, 0, capi.ptr(counts), E, capi.ptr(t_counts), capi.ptr(t_flags), capi.ptr(flags), capi.ptr(epoch),
                                      capi.ptr(ws), st))
        capi.check(L.xs_moe_check_flags(capi.ptr(ws), st))
        assert int(epoch.item()) == step and int(flags[0].item()) == step
    assert torch.equal(all_counts[:E], counts)
    # two ranks, of which only rank 0 ever signals: rank 0's wait for flags[1] runs out
    flags.zero_()
    epoch.zero_()
    t_flags2 = torch.tensor([flags.data_ptr(), flags.data_ptr()], dtype=torch.int64, device="cuda")  # "rank 1"'s row is never read
    t0 = time.time()
    capi.check(L.xs_moe_ep_signal(2, 0, None, 0, None, capi.ptr(t_flags2), capi.ptr(flags), capi.ptr(epoch), capi.ptr(ws), st))
    with pytest.raises(RuntimeError, match="wait timed out"):
        capi.check(L.xs_moe_check_flags(capi.ptr(ws), st))
    assert 0.2 < time.time() - t0 < 30.0
    capi.check(L.xs_moe_check_flags(capi.ptr(ws), st))  # the flag is cleared; the context is still usable
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum().item()) == 16.0
