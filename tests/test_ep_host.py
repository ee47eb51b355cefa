"""The C++ host of the expert-parallel layer (xstar_cpp.EpGroup / EpContext: NCCL + peer stores, one thread per GPU).
CPU tests cover the host-side failure detection -- a rank that never posts, a rank that leaves, ranks that disagree --
none of which touches a GPU; GPU tests run the layer through EpContext against the CPU oracle on the global problem."""
import threading
import time

import numpy as np
import pytest
import torch

from xstar_moe import capi, synth

from bridge import cpp_to_torch, torch_to_cpp, xstar_cpp


def _run_threads(fns):
    out = [None] * len(fns)

    def wrap(i):
        try:
            out[i] = ("ok", fns[i]())
        except Exception as e:  # noqa: BLE001 - the test inspects what each rank raised
            out[i] = ("err", e)

    ts = [threading.Thread(target=wrap, args=(i,)) for i in range(len(fns))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(60)
        assert not t.is_alive(), "a rank thread did not come back"
    return out


def test_group_releases_all_ranks_step_after_step():
    g = xstar_cpp.EpGroup(3, 5000)

    def rank(r):
        def run():
            for step in range(20):
                g.arrive(r, 1000 + step)
            return True
        return run

    assert [o[0] for o in _run_threads([rank(r) for r in range(3)])] == ["ok"] * 3
    assert not g.broken()


def test_group_times_out_when_a_rank_never_posts():
    g = xstar_cpp.EpGroup(3, 300)
    t0 = time.monotonic()
    res = _run_threads([lambda: g.arrive(0, 7), lambda: g.arrive(2, 7)])  # rank 1 never shows up
    dt = time.monotonic() - t0
    assert all(k == "err" for k, _ in res)
    assert all("peer timeout: rank 1 did not arrive" in str(e) for _, e in res), res
    assert 0.25 <= dt < 5.0
    assert g.broken()
    with pytest.raises(RuntimeError, match="group is broken: peer timeout"):
        g.arrive(1, 7)  # the late rank learns of it as soon as it does arrive


def test_group_reports_a_rank_that_left():
    g = xstar_cpp.EpGroup(2, 10000)
    res = {}

    def waiter():
        try:
            g.arrive(0, 1)
            res["r"] = "ok"
        except RuntimeError as e:
            res["r"] = str(e)

    t = threading.Thread(target=waiter)
    t.start()
    time.sleep(0.2)
    g.leave(1)  # rank 1 unwinds instead of joining the step
    t.join(10)
    assert not t.is_alive() and "peer left: rank 1" in res["r"]
    # a rank that left before anyone waited is noticed at the next check-in
    g2 = xstar_cpp.EpGroup(2, 10000)
    g2.leave(0)
    with pytest.raises(RuntimeError, match="peer left: rank 0"):
        g2.arrive(1, 1)


def test_group_rejects_ranks_that_disagree_on_the_step():
    g = xstar_cpp.EpGroup(2, 5000)
    res = _run_threads([lambda: g.arrive(0, 11), lambda: g.arrive(1, 12)])
    assert all(k == "err" and "step mismatch" in str(e) for k, e in res), res
    g = xstar_cpp.EpGroup(2, 300)
    g_res = _run_threads([lambda: (g.arrive(0, 1), g.arrive(0, 1))])  # the same rank twice in one step
    assert g_res[0][0] == "err" and ("peer timeout" in str(g_res[0][1]) or "arrived twice" in str(g_res[0][1]))
    with pytest.raises(RuntimeError, match="bad rank"):
        xstar_cpp.EpGroup(2, 100).arrive(5, 0)


def test_capacity_rule():
    assert xstar_cpp.ep_capacity_rows(2048, 6, 8, 0.0) == 8 * 2048 * 6  # worst case: every row of every rank
    assert xstar_cpp.ep_capacity_rows(2048, 6, 8, 2.0) == 2 * 2048 * 6
    assert xstar_cpp.ep_capacity_rows(2048, 6, 8, 100.0) == 8 * 2048 * 6  # never more than the worst case
    assert xstar_cpp.ep_capacity_rows(5, 3, 2, 1.5) == 128  # rounded up to whole 128-row tiles
    with pytest.raises(RuntimeError, match="bad capacity"):
        xstar_cpp.ep_capacity_rows(8, 2, 2, -1.0)


def test_comm_layer_loads_nccl_by_name():
    assert capi.lib().xs_moe_comm_available() == 0, capi.lib().xs_moe_last_error()


def test_fused_return_is_offered_for_fp4_experts_only():
    """xs_moe_grouped_mlp_return_supported needs no GPU: FP4 experts with hidden % 256 == 0 take the tokens-as-M kernels,
    whose down epilogue can store into the source ranks; everything else uses the two-step return."""
    import ctypes as C
    L = capi.lib()
    ok = C.c_int32(-1)
    for fmt, H, want in ((capi.FP4_MX32, 4096, 1), (capi.FP4_MX32, 384, 0), (capi.FP8_BLOCK128, 4096, 0), (capi.BF16, 4096, 0)):
        cfg = capi.make_config(2048, H, 256, 6, 2048, 0, fmt, capi.FP8_BLOCK128 if fmt == capi.FP4_MX32 else fmt, 32, 32)
        assert L.xs_moe_grouped_mlp_return_supported(C.byref(cfg), 12288, C.byref(ok)) == 0, L.xs_moe_last_error()
        assert ok.value == want, (fmt, H)


# ---- on GPUs ---------------------------------------------------------------------------------------------------------
_DT = {"bf16": "BFloat16", "fp8": "Float8E4M3", "fp4": "Float4E2M1x2"}


def _cpp(t, kind=None):
    return torch_to_cpp(t, getattr(xstar_cpp.DType, kind)) if kind else torch_to_cpp(t)


def _rank_tensors(d, dims, rank, world):
    """This rank's tensors on ITS device (the calling thread's current device): router and always-on expert replicated,
    experts [rank * E / world, ...) and the rank's slice of the tokens."""
    fmt, T, El = dims["fmt"], dims["T"], dims["E"] // world
    wk = {"bf16": None, "fp8": "Float8E4M3", "fp4": "Float4E2M1x2"}[fmt]
    sk = {"bf16": None, "fp8": None, "fp4": "UE8M0"}[fmt]
    up = lambda t, k=None: xstar_cpp.to_cuda(_cpp(t.contiguous(), k))  # noqa: E731
    sl = slice(rank * El, (rank + 1) * El)
    kw = {}
    if fmt != "bf16":
        kw["gate_up_scale"] = up(d["gate_up_scale"][sl], sk)
        kw["down_scale"] = up(d["down_scale"][sl], sk)
    if dims["S"]:
        shk = None if fmt == "bf16" else "Float8E4M3"
        kw["shared_gate_up_weight"] = up(d["shared_gate_up_w"], shk)
        kw["shared_down_weight"] = up(d["shared_down_w"], shk)
        if fmt != "bf16":
            kw["shared_gate_up_scale"] = up(d["shared_gate_up_scale"])
            kw["shared_down_scale"] = up(d["shared_down_scale"])
    if d.get("router_bias") is not None:
        kw["router_bias"] = up(d["router_bias"])
    return (up(d["x"][rank * T:(rank + 1) * T]), up(d["router_w"]), up(d["gate_up_w"][sl], wk), up(d["down_w"][sl], wk)), kw


def _oracle(oracle, dims, d):
    n = synth.to_numpy_storage(d)
    mode = {"bf16": oracle.BF16, "fp8": oracle.FP8, "fp4": oracle.FP4}[dims["fmt"]]
    return oracle.moe_forward(mode, n["x"], n["router_w"], n["gate_up_w"], n["down_w"], dims["K"], router_bias=n.get("router_bias"),
                              gate_up_scale=n.get("gate_up_scale"), down_scale=n.get("down_scale"),
                              shared_gate_up_w=n.get("shared_gate_up_w"), shared_down_w=n.get("shared_down_w"),
                              shared_gate_up_scale=n.get("shared_gate_up_scale"), shared_down_scale=n.get("shared_down_scale"), threads=8)


def _run_world(dims, world, seed, capacity_factor=0.0, steps=2, timeout_ms=60000):
    d = synth.make_inputs(dict(dims, T=dims["T"] * world), seed=seed)
    group = xstar_cpp.EpGroup(world, timeout_ms)
    uid = xstar_cpp.ep_unique_id()

    def rank(r):
        def run():
            xstar_cpp.set_device(r)
            (x, rw, gu, dw), kw = _rank_tensors(d, dims, r, world)
            ctx = xstar_cpp.EpContext(group, uid, r, world, r, dims["T"], dims["H"], dims["E"], dims["K"], dims["I"],
                                      getattr(xstar_cpp.DType, _DT[dims["fmt"]]), bool(dims["S"]), capacity_factor)
            outs = [cpp_to_torch(xstar_cpp.to_cpu(ctx.moe(x, rw, gu, dw, dims["K"], **kw)), (dims["T"], dims["H"])) for _ in range(steps)]
            for o in outs[1:]:
                assert torch.equal(o, outs[0])
            return outs[0]
        return run

    return d, _run_threads([rank(r) for r in range(world)])


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-3), ("fp8", 1e-2), ("fp4", 1e-2)])
def test_cpp_ep_single_rank_matches_oracle(oracle, fmt, tol):
    """world = 1: the whole expert-parallel step (NCCL communicator of one rank, dispatch and return kernels storing into this
    rank's own buffers) on one GPU."""
    dims = dict(T=96, H=512, E=16, K=4, I=256, S=1, fmt=fmt, bias=None)
    d, res = _run_world(dims, 1, seed=31)
    assert res[0][0] == "ok", res[0][1]
    ref = _oracle(oracle, dims, d)
    rel = synth.rel_l2(res[0][1].float().numpy(), synth.bf16_bits_to_f32(ref["out"]))
    assert rel <= tol, rel


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-3), ("fp8", 1e-2), ("fp4", 1e-2)])
def test_cpp_ep_two_rank_threads_match_oracle(oracle, fmt, tol):
    """Two host threads, one GPU each, rows crossing NVLink both ways: outputs of both ranks against the oracle on the global
    batch; bf16 experts also bit-identical to the single-GPU layer's contract (same roundings)."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs on one box")
    dims = dict(T=96, H=512, E=16, K=4, I=256, S=1, fmt=fmt, bias=None)
    d, res = _run_world(dims, world, seed=23)
    for k, v in res:
        assert k == "ok", v
    got = torch.cat([v for _, v in res]).float().numpy()
    ref = _oracle(oracle, dims, d)
    rel = synth.rel_l2(got, synth.bf16_bits_to_f32(ref["out"]))
    assert rel <= tol, rel


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["bf16", "fp4"])
def test_cpp_ep_flags_a_receive_buffer_that_is_too_small(fmt):
    """capacity_factor far below the rows that arrive: the dispatch kernel skips the rows that do not fit and flags it, the
    grouped MLP clamps its segments to the capacity (FP4: with the return folded into its epilogue), and check() raises on
    the host -- nothing is written out of bounds."""
    dims = dict(T=256, H=256, E=8, K=4, I=128, S=0, fmt=fmt, bias=None)
    d, res = _run_world(dims, 1, seed=3, capacity_factor=0.25, steps=1)
    assert res[0][0] == "err" and "out-of-range index" in str(res[0][1]), res[0]


@pytest.mark.gpu
def test_cpp_ep_rejects_calls_that_do_not_fit_the_context():
    dims = dict(T=32, H=256, E=8, K=2, I=128, S=0, fmt="bf16", bias=None)
    d = synth.make_inputs(dims, seed=1)
    xstar_cpp.set_device(0)
    (x, rw, gu, dw), kw = _rank_tensors(d, dims, 0, 1)
    ctx = xstar_cpp.EpContext(None, xstar_cpp.ep_unique_id(), 0, 1, 0, 32, 256, 8, 2, 128, xstar_cpp.DType.BFloat16, False)
    with pytest.raises(RuntimeError, match="shape mismatch"):
        ctx.moe(x, rw, gu, dw, 3)  # another top_k than the context was sized for
    with pytest.raises(RuntimeError, match="expert count mismatch"):
        xstar_cpp.EpContext(None, xstar_cpp.ep_unique_id(), 0, 3, 0, 32, 256, 8, 2, 128, xstar_cpp.DType.BFloat16, False)
    out = cpp_to_torch(xstar_cpp.to_cpu(ctx.moe(x, rw, gu, dw, 2)), (32, 256))
    assert torch.isfinite(out.float()).all()


# ---- batch composition and rank workers -------------------------------------------------------------------------------
def test_batch_is_balanced_without_splitting_sequences():
    rng = np.random.default_rng(5)
    lens = rng.integers(1, 400, size=37).tolist()
    cu = np.concatenate([[0], np.cumsum(lens)]).tolist()
    for ranks in (1, 2, 4, 8):
        p = xstar_cpp.ep_balance_batch(cu, ranks)
        assert sorted(s for r in p["sequences_of_rank"] for s in r) == list(range(len(lens)))  # every sequence exactly once
        for r, seqs in enumerate(p["sequences_of_rank"]):
            assert seqs == sorted(seqs) and sum(lens[s] for s in seqs) == p["tokens_of_rank"][r]
            assert all(p["rank_of_sequence"][s] == r for s in seqs)
        mean = sum(lens) / ranks
        assert p["max_tokens"] <= mean + max(lens)  # longest-first greedy: within one sequence of the mean
        assert abs(p["imbalance"] - p["max_tokens"] / mean) < 1e-9
    # a decode batch (one token per sequence) splits evenly
    p = xstar_cpp.ep_balance_batch(list(range(0, 129)), 8)
    assert p["tokens_of_rank"] == [16] * 8 and p["imbalance"] == 1.0
    # fewer sequences than ranks: some ranks stay empty, nothing is split
    p = xstar_cpp.ep_balance_batch([0, 5, 9], 4)
    assert sorted(p["tokens_of_rank"]) == [0, 0, 4, 5]
    assert xstar_cpp.ep_balance_batch([0], 2)["imbalance"] == 1.0


def test_batch_balancer_errors():
    with pytest.raises(RuntimeError, match="batch does not fit: rank 0 would hold 300 tokens, capacity 256"):
        xstar_cpp.ep_balance_batch([0, 300, 310], 2, 256)
    with pytest.raises(RuntimeError, match="bad cu_seqlens"):
        xstar_cpp.ep_balance_batch([1, 5], 2)
    with pytest.raises(RuntimeError, match="bad cu_seqlens"):
        xstar_cpp.ep_balance_batch([0, 5, 3], 2)
    with pytest.raises(RuntimeError, match="bad rank count"):
        xstar_cpp.ep_balance_batch([0, 5], 0)


def _pool_run(oracle, dims, world, tokens_of_rank, seed):
    """One worker thread per rank inside the module; the ranks' batches hold different numbers of tokens."""
    total = sum(tokens_of_rank)
    d = synth.make_inputs(dict(dims, T=total), seed=seed)
    El = dims["E"] // world
    pool = xstar_cpp.EpWorkerPool(world, list(range(world)), max(tokens_of_rank), dims["H"], dims["E"], dims["K"], dims["I"],
                                  getattr(xstar_cpp.DType, _DT[dims["fmt"]]), bool(dims["S"]))
    xs, rw, gu, dw, extra = [], [], [], [], {}
    start = 0
    for r in range(world):
        xstar_cpp.set_device(r)
        T = tokens_of_rank[r]
        (_, a, b, c), kw = _rank_tensors(d, dict(dims, T=0), r, world)  # weights only; the rank's rows are cut here
        x = xstar_cpp.to_cuda(_cpp(d["x"][start:start + T].contiguous()))
        start += T
        xs.append(x), rw.append(a), gu.append(b), dw.append(c)
        for k, v in kw.items():
            extra.setdefault(k, []).append(v)
    xstar_cpp.set_device(0)
    outs = pool.run(xs, rw, gu, dw, dims["K"], **extra)
    got = torch.cat([cpp_to_torch(xstar_cpp.to_cpu(o), (tokens_of_rank[r], dims["H"])) for r, o in enumerate(outs)])
    ref = _oracle(oracle, dict(dims, T=total), d)
    return synth.rel_l2(got.float().numpy(), synth.bf16_bits_to_f32(ref["out"]))


@pytest.mark.gpu
def test_worker_pool_single_rank(oracle):
    dims = dict(T=0, H=512, E=16, K=4, I=256, S=1, fmt="bf16", bias=None)
    assert _pool_run(oracle, dims, 1, [80], seed=41) <= 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-3), ("fp4", 1e-2)])
def test_worker_pool_two_ranks_with_uneven_batches(oracle, fmt, tol):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on one box")
    dims = dict(T=0, H=512, E=16, K=4, I=256, S=1, fmt=fmt, bias=None)
    plan = xstar_cpp.ep_balance_batch([0, 40, 100, 130, 166], 2)  # sequences of 40, 60, 30, 36 tokens
    assert plan["tokens_of_rank"] == [90, 76]
    # the layer does not care which tokens sit on which rank: the global batch in rank order must equal the oracle's
    assert _pool_run(oracle, dims, 2, plan["tokens_of_rank"], seed=42) <= tol


@pytest.mark.gpu
def test_worker_pool_with_a_rank_that_holds_no_tokens(oracle):
    """Fewer sequences than ranks: a rank with an empty batch still takes part in every collective of the step."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on one box")
    dims = dict(T=0, H=512, E=16, K=4, I=256, S=1, fmt="bf16", bias=None)
    assert _pool_run(oracle, dims, 2, [0, 50], seed=43) <= 2e-3
    assert _pool_run(oracle, dims, 2, [33, 0], seed=44) <= 2e-3


# ---- the collective layer by itself (include/xs_moe_comm.h) -----------------------------------------------------------
def _comm_rank(L, uid, rank, world, results):
    """One rank of the collective layer through ctypes: all-gather, barrier, all-to-all with uneven splits."""
    import ctypes as C
    capi.check(L.xs_moe_set_device(rank))
    comm = C.c_void_p()
    capi.check(L.xs_moe_comm_create(C.byref(comm), uid, rank, world))
    stream = C.c_void_p()
    capi.check(L.xs_moe_stream_create(C.byref(stream)))

    def dev(nbytes):
        p = C.c_void_p()
        capi.check(L.xs_moe_device_alloc(C.byref(p), max(nbytes, 256)))
        return p

    def up(p, a):
        capi.check(L.xs_moe_memcpy_h2d(p, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def down(p, n, dtype):
        a = np.empty(n, dtype)
        capi.check(L.xs_moe_memcpy_d2h(a.ctypes.data_as(C.c_void_p), p, a.nbytes))
        return a

    # all-gather of 5 int32 per rank
    mine = np.arange(5, dtype=np.int32) + 100 * rank
    s, r = dev(20), dev(20 * world)
    up(s, mine)
    capi.check(L.xs_moe_comm_all_gather(comm, s, r, 20, stream))
    tok = dev(4)
    capi.check(L.xs_moe_memset_async(tok, 0, 4, stream))
    capi.check(L.xs_moe_comm_barrier(comm, tok, stream))
    capi.check(L.xs_moe_stream_synchronize(stream))
    gathered = down(r, 5 * world, np.int32)
    # all-to-all: rank a sends (a + 1) * (b + 1) bytes of value 16 * a + b to rank b
    send_n = [(rank + 1) * (b + 1) for b in range(world)]
    recv_n = [(a + 1) * (rank + 1) for a in range(world)]
    sbuf = np.concatenate([np.full(send_n[b], 16 * rank + b, np.uint8) for b in range(world)])
    sp, rp = dev(sbuf.nbytes), dev(sum(recv_n))
    up(sp, sbuf)
    sz = C.c_size_t * world
    soff = np.concatenate([[0], np.cumsum(send_n)[:-1]]).tolist()
    roff = np.concatenate([[0], np.cumsum(recv_n)[:-1]]).tolist()
    capi.check(L.xs_moe_comm_all_to_all_v(comm, world, sp, sz(*send_n), sz(*soff), rp, sz(*recv_n), sz(*roff), stream))
    capi.check(L.xs_moe_stream_synchronize(stream))
    got = down(rp, sum(recv_n), np.uint8)
    code = C.c_int32(-1)
    capi.check(L.xs_moe_comm_async_error(comm, C.byref(code)))
    results[rank] = (gathered, got, recv_n, code.value)
    for p in (s, r, tok, sp, rp):
        capi.check(L.xs_moe_device_free(p))
    capi.check(L.xs_moe_stream_destroy(stream))
    capi.check(L.xs_moe_comm_destroy(comm))


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2])
def test_collective_layer_all_gather_barrier_all_to_all(world):
    import ctypes as C
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs on one box")
    L = capi.lib()
    uid = (C.c_uint8 * 128)()
    capi.check(L.xs_moe_comm_unique_id(uid))
    results = [None] * world
    res = _run_threads([(lambda r=r: _comm_rank(L, uid, r, world, results)) for r in range(world)])
    for k, v in res:
        assert k == "ok", v
    for rank in range(world):
        gathered, got, recv_n, code = results[rank]
        assert code == 0
        assert gathered.tolist() == [v + 100 * a for a in range(world) for v in range(5)]
        want = np.concatenate([np.full(recv_n[a], 16 * a + rank, np.uint8) for a in range(world)])
        assert np.array_equal(got, want)
    capi.check(L.xs_moe_set_device(0))
