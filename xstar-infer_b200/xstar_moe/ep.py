"""Expert parallelism for the MoE layer: one process per GPU, experts sharded evenly and contiguously
(expert e lives on rank e // (E / R)), tokens data-parallel, one exchange each way.  Two transports:

`forward_peer` (default in bench.py) -- rows travel by peer-memory stores from kernels of the library:
    local route -> local permute -> all-gather of per-expert counts (stays on the device) -> plan kernel
    -> DISPATCH kernel: each token quantised once and stored into the grouped buffer of the owner of each of its experts
    -> barrier -> grouped expert MLPs straight on that buffer -> RETURN kernel: results stored into the source rank's
    return buffer at their permuted row -> barrier -> local weighted combine (+ the always-on expert, computed locally)
  Nothing returns to the host, so the step can be captured as one CUDA graph (`capture_peer`).

`forward` -- rows travel by NCCL all-to-all (portable baseline; what the CPU/gloo tests drive):
    local route -> local permute (rows sorted by expert => by destination rank)
    -> all-gather of per-expert counts (the one host synchronisation: NCCL needs split sizes on the host)
    -> DISPATCH all-to-all of the permuted rows (payload: bf16 rows, or e4m3 codes + 1x128 f32 / 1x32 e8m0 scales)
    -> regroup received rows by local expert -> grouped expert MLPs -> rows back into arrival order
    -> COMBINE all-to-all back (f32 rows; bf16 rows for the quantised formats) -> local weighted combine

Received rows are ordered by (expert, source rank, source order) in both -- fixed by the data, not by arrival time --
so the result is reproducible, the two transports agree bit for bit, and with bf16 experts the layer equals the
single-device layer bit for bit (the combine still sums each token's k expert outputs in slot order).

This module is host logic over `torch.distributed`; all device compute goes through an `ops` object.
`CudaOps` binds the C ABI (libxs_moe.so).  Tests drive the same host logic on CPU ranks (gloo) with a
stand-in `ops`.
"""
import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import capi


# ------------------------------------------------------------------------------------------------------------
# host-side planning (pure numpy: testable without any device)
# ------------------------------------------------------------------------------------------------------------
class EpPlan:
    """Split sizes and regroup maps from the (R, E) matrix of per-rank, per-expert row counts."""

    def __init__(self, all_counts, rank):
        all_counts = np.asarray(all_counts, dtype=np.int64)
        R, E = all_counts.shape
        if E % R != 0:
            raise ValueError("expert count mismatch: experts must divide evenly over ranks")
        self.R, self.E, self.rank = R, E, rank
        self.El = El = E // R
        mine = all_counts[rank]
        # rows this rank sends to rank d = its rows of d's experts; rows it receives from s = s's rows of my experts
        self.send_splits = mine.reshape(R, El).sum(1).astype(np.int64)
        self.recv_counts = all_counts[:, rank * El:(rank + 1) * El]  # (R, El): source rank x local expert
        self.recv_splits = self.recv_counts.sum(1).astype(np.int64)
        self.n_recv = int(self.recv_splits.sum())
        # grouped order: (local expert, source rank, token); arrival order: (source rank, local expert, token)
        per_expert = self.recv_counts.sum(0)
        self.offsets_local = np.concatenate([[0], np.cumsum(per_expert)]).astype(np.int32)
        # arrival rows carry (source, expert) labels in source-major order; a stable sort by expert gives the grouped order
        expert_of_row = np.repeat(np.tile(np.arange(El, dtype=np.int32), R), self.recv_counts.reshape(-1))
        self.grouped_from_arrival = np.argsort(expert_of_row, kind="stable").astype(np.int32)  # grouped row g <- arrival row
        arrival_from_grouped = np.empty(self.n_recv, np.int32)
        arrival_from_grouped[self.grouped_from_arrival] = np.arange(self.n_recv, dtype=np.int32)
        self.arrival_from_grouped = arrival_from_grouped

    def packed_maps(self):
        """offsets_local | grouped_from_arrival | arrival_from_grouped in one int32 array (one host-to-device copy)."""
        return np.concatenate([self.offsets_local, self.grouped_from_arrival, self.arrival_from_grouped])


# ------------------------------------------------------------------------------------------------------------
# device ops through the C ABI
# ------------------------------------------------------------------------------------------------------------
class CudaOps:
    """Stage calls of libxs_moe.so on torch CUDA tensors (torch = device memory + streams only)."""

    def __init__(self, dims, weights_local, shared_weights, rank, world):
        self.dims = dims
        self.T, self.H, self.E, self.K, self.I, self.S = (dims[k] for k in "THEKIS")
        self.El = self.E // world
        self.fmt = {"bf16": capi.BF16, "fp8": capi.FP8_BLOCK128, "fp4": capi.FP4_MX32}[dims["fmt"]]
        self.fmt_shared = capi.FP8_BLOCK128 if self.fmt == capi.FP4_MX32 else self.fmt  # FP8 always-on expert next to FP4 experts
        self.L = capi.lib()
        self.cfg_route = capi.make_config(self.T, self.H, self.E, self.K, self.I, 0, self.fmt, self.fmt_shared)
        self.cfg_local = capi.make_config(self.T, self.H, self.E, self.K, self.I, 0, self.fmt, self.fmt_shared, rank * self.El, self.El)
        self.cfg_shared = capi.make_config(self.T, self.H, self.E, self.K, self.I, 0, self.fmt_shared, self.fmt_shared, 0, 1)
        self.w_local = capi.make_weights(weights_local)
        self.keep = (weights_local, shared_weights)
        if shared_weights is not None:
            sw = dict(router_w=weights_local["router_w"], gate_up_w=shared_weights["shared_gate_up_w"],
                      down_w=shared_weights["shared_down_w"], gate_up_scale=shared_weights.get("shared_gate_up_scale"),
                      down_scale=shared_weights.get("shared_down_scale"))
            self.w_shared = capi.make_weights(sw)
            self.keep += (sw,)
        self.ws = torch.empty(capi.workspace_bytes(self.cfg_route), dtype=torch.uint8, device="cuda")
        capi.check(self.L.xs_moe_workspace_init(capi.ptr(self.ws), self.ws.numel(), self._st()))
        self._gws = {}
        self.shared_offsets = torch.tensor([0, self.T], dtype=torch.int32, device="cuda")
        self.side_stream = torch.cuda.Stream()

    @staticmethod
    def _st():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def device(self):
        return torch.device("cuda")

    def route(self, x, router_w, router_bias):
        T, K = self.T, self.K
        ids = torch.empty((T, K), dtype=torch.int32, device="cuda")
        w = torch.empty((T, K), dtype=torch.float32, device="cuda")
        capi.check(self.L.xs_moe_route(C.byref(self.cfg_route), capi.ptr(x), capi.ptr(router_w), capi.ptr(router_bias), None,
                                       capi.ptr(ids), capi.ptr(w), capi.ptr(self.ws), self.ws.numel(), self._st()))
        return ids, w

    def permute(self, ids):
        T, K, E = self.T, self.K, self.E
        counts = torch.empty(E, dtype=torch.int32, device="cuda")
        offsets = torch.empty(E + 1, dtype=torch.int32, device="cuda")
        perm = torch.empty(T * K, dtype=torch.int32, device="cuda")
        inv = torch.empty(T * K, dtype=torch.int32, device="cuda")
        capi.check(self.L.xs_moe_permute(C.byref(self.cfg_route), capi.ptr(ids), capi.ptr(counts), capi.ptr(offsets), capi.ptr(perm),
                                         capi.ptr(inv), capi.ptr(self.ws), self.ws.numel(), self._st()))
        return counts, offsets, perm, inv

    def _payload(self, x, fmt):
        if fmt == capi.BF16:
            return [x]
        q = torch.empty(x.shape, dtype=torch.uint8, device="cuda")
        if fmt == capi.FP8_BLOCK128:
            s = torch.empty((x.shape[0], self.H // 128), dtype=torch.float32, device="cuda")
            capi.check(self.L.xs_moe_quantize_rows_fp8(capi.ptr(x), x.shape[0], self.H, capi.ptr(q), capi.ptr(s), self._st()))
        else:
            s = torch.empty((x.shape[0], self.H // 32), dtype=torch.uint8, device="cuda")
            capi.check(self.L.xs_moe_quantize_rows_mxfp8(capi.ptr(x), x.shape[0], self.H, capi.ptr(q), capi.ptr(s), self._st()))
        return [q, s]

    def payload(self, x):
        """What travels per row: [bf16 row], [e4m3 codes, 1x128 f32 scales] (FP8 experts) or
        [e4m3 codes, 1x32 e8m0 scales] (FP4 experts)."""
        return self._payload(x, self.fmt)

    def gather(self, src, index):
        n = index.numel()
        dst = torch.empty((n, *src.shape[1:]), dtype=src.dtype, device="cuda")
        row_bytes = src[0].numel() * src.element_size() if src.shape[0] else int(np.prod(src.shape[1:])) * src.element_size()
        capi.check(self.L.xs_moe_gather_rows(capi.ptr(src), capi.ptr(index), capi.ptr(dst), n, row_bytes, self._st()))
        return dst

    def _grouped(self, cfg, w, payload, offsets, n_rows):
        nb = C.c_size_t(0)
        capi.check(self.L.xs_moe_grouped_mlp_workspace_bytes(C.byref(cfg), n_rows, C.byref(nb)))
        ws = self._gws.get(id(cfg))
        if ws is None or ws.numel() < nb.value:  # grow-only scratch, with headroom so that routing noise does not reallocate
            ws = torch.zeros(int(nb.value * 1.25) + 256, dtype=torch.uint8, device="cuda")
            self._gws[id(cfg)] = ws
        y = torch.empty((n_rows, self.H), dtype=torch.float32, device="cuda")
        scales = payload[1] if len(payload) > 1 else None
        capi.check(self.L.xs_moe_grouped_mlp(C.byref(cfg), C.byref(w), capi.ptr(payload[0]), capi.ptr(scales), capi.ptr(offsets),
                                             n_rows, capi.ptr(y), capi.ptr(ws), ws.numel(), self._st()))
        return y

    def grouped_mlp(self, payload, offsets_local, n_rows):
        return self._grouped(self.cfg_local, self.w_local, payload, offsets_local, n_rows)

    def shared_mlp(self, x, payload):
        if payload is None or self.fmt_shared != self.fmt:
            payload = self._payload(x, self.fmt_shared)
        return self._grouped(self.cfg_shared, self.w_shared, payload, self.shared_offsets, self.T)

    def return_rows(self, y_grouped, index):
        """Expert outputs back into arrival order for the return trip: f32 rows for bf16 experts (bit-identical to the
        single-device layer), bf16 rows for the quantised formats (half the NVLink bytes, inside their tolerance)."""
        if self.fmt == capi.BF16:
            return self.gather(y_grouped, index)
        n = index.numel()
        dst = torch.empty((n, self.H), dtype=torch.bfloat16, device="cuda")
        capi.check(self.L.xs_moe_gather_rows_f32_to_bf16(capi.ptr(y_grouped), capi.ptr(index), capi.ptr(dst), n, self.H, self._st()))
        return dst

    def combine(self, y, inv, w, shared):
        out = torch.empty((self.T, self.H), dtype=torch.bfloat16, device="cuda")
        fn = self.L.xs_moe_combine if y.dtype == torch.float32 else self.L.xs_moe_combine_bf16_rows
        capi.check(fn(C.byref(self.cfg_route), capi.ptr(y), capi.ptr(inv), capi.ptr(w), capi.ptr(shared), capi.ptr(out), self._st()))
        return out

    def check(self):
        capi.check(self.L.xs_moe_check_flags(capi.ptr(self.ws), self._st()))
        for ws in self._gws.values():
            capi.check(self.L.xs_moe_check_flags(capi.ptr(ws), self._st()))


# ------------------------------------------------------------------------------------------------------------
# exchange over peer memory (NVLink stores from the dispatch / return kernels; no host synchronisation)
# ------------------------------------------------------------------------------------------------------------
class DeviceBuffer:
    """Raw device memory from the library's allocator: exportable to the other processes of the box, which a block
    of torch's pooled allocator is not."""

    def __init__(self, nbytes, dtype=torch.uint8):
        self.nbytes, self.dtype = int(nbytes), dtype
        p = C.c_void_p()
        capi.check(capi.lib().xs_moe_device_alloc(C.byref(p), max(self.nbytes, 256)))
        self._ptr = p.value

    def data_ptr(self):
        return self._ptr

    def free(self):
        if self._ptr:
            capi.check(capi.lib().xs_moe_device_free(C.c_void_p(self._ptr)))
            self._ptr = 0


class PeerExchange:
    """This rank's side of the peer-memory exchange: its receive buffers (grouped rows + scales, sized for the worst
    routing: every token of every rank choosing this rank's experts), its return buffer (one row per local (token, slot)),
    the small index tables, and the pointer tables of all ranks' buffers."""

    def __init__(self, dims, rank, world, capacity=None):
        T, H, E, K = (dims[k] for k in "THEK")
        self.T, self.H, self.E, self.K, self.R, self.rank = T, H, E, K, world, rank
        self.El = E // world
        self.fmt = {"bf16": capi.BF16, "fp8": capi.FP8_BLOCK128, "fp4": capi.FP4_MX32}[dims["fmt"]]
        self.capacity = int(capacity) if capacity is not None else world * T * K
        self.back_rows = T * K
        self.wire_bf16 = self.fmt != capi.BF16
        row_bytes = H * 2 if self.fmt == capi.BF16 else H
        scale_bytes = {capi.BF16: 0, capi.FP8_BLOCK128: (H // 128) * 4, capi.FP4_MX32: H // 32}[self.fmt]
        self.rows = DeviceBuffer(self.capacity * row_bytes)
        self.scales = DeviceBuffer(self.capacity * scale_bytes, torch.float32 if self.fmt == capi.FP8_BLOCK128 else torch.uint8)
        self.back = DeviceBuffer(self.back_rows * H * (2 if self.wire_bf16 else 4), torch.bfloat16 if self.wire_bf16 else torch.float32)
        self.dest_base = torch.zeros(E, dtype=torch.int32, device="cuda")
        self.offsets_local = torch.zeros(self.El + 1, dtype=torch.int32, device="cuda")
        self.src_offsets = torch.zeros(world * E, dtype=torch.int32, device="cuda")
        self.cfg = capi.make_config(T, H, E, K, dims["I"], 0, self.fmt, self.fmt)
        self.L = capi.lib()
        self._imported = []
        self.tables = None

    def connect(self, rows_ptrs, scales_ptrs, back_ptrs):
        """Addresses of every rank's buffers as this process sees them (index = rank)."""
        self.tables = torch.tensor([rows_ptrs, scales_ptrs, back_ptrs], dtype=torch.int64, device="cuda")

    def connect_ipc(self, group=None):
        """Exchange handles with the other processes of the box and map their buffers.  Collective; the ranks agree on
        the outcome before any of them raises, so a caller may fall back to the all-to-all exchange on every rank."""
        err = None
        mine = torch.zeros(3, capi.IPC_HANDLE_BYTES, dtype=torch.uint8)
        try:
            for i, b in enumerate((self.rows, self.scales, self.back)):
                capi.check(self.L.xs_moe_ipc_export(C.c_void_p(b.data_ptr()), C.c_void_p(mine[i].data_ptr())))
        except RuntimeError as e:
            err = e
        every = torch.empty(self.R, 3, capi.IPC_HANDLE_BYTES, dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(every.view(-1), mine.cuda().view(-1), group=group)
        every = every.cpu()
        ptrs = [[0] * self.R for _ in range(3)]
        try:
            for r in range(self.R if err is None else 0):
                for i, b in enumerate((self.rows, self.scales, self.back)):
                    if r == self.rank:
                        ptrs[i][r] = b.data_ptr()
                    else:
                        p = C.c_void_p()
                        h = every[r, i].contiguous()
                        capi.check(self.L.xs_moe_ipc_import(C.c_void_p(h.data_ptr()), C.byref(p)))
                        self._imported.append(p.value)
                        ptrs[i][r] = p.value
        except RuntimeError as e:
            err = e
        ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32, device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            self._unmap()
            raise RuntimeError(f"peer mapping failed on at least one rank ({err if err is not None else 'another rank'})")
        self.connect(*ptrs)

    @staticmethod
    def _st():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def plan(self, all_counts):
        capi.check(self.L.xs_moe_ep_plan(capi.ptr(all_counts), self.R, self.E, self.rank, capi.ptr(self.dest_base),
                                         capi.ptr(self.offsets_local), capi.ptr(self.src_offsets), self._st()))

    def dispatch(self, x, ids, inv, offsets, ws):
        capi.check(self.L.xs_moe_ep_dispatch(C.byref(self.cfg), self.R, capi.ptr(x), capi.ptr(ids), capi.ptr(inv), capi.ptr(offsets),
                                             capi.ptr(self.dest_base), capi.ptr(self.tables[0]), capi.ptr(self.tables[1]),
                                             self.capacity, capi.ptr(ws), self._st()))

    def give_back(self, y_grouped, all_counts, ws):
        capi.check(self.L.xs_moe_ep_return(C.byref(self.cfg), self.R, self.rank, capi.ptr(y_grouped), capi.ptr(all_counts),
                                           capi.ptr(self.offsets_local), capi.ptr(self.src_offsets), int(y_grouped.shape[0]),
                                           capi.ptr(self.tables[2]), self.back_rows, int(self.wire_bf16), capi.ptr(ws), self._st()))

    def close(self):
        """Unmap the peers' buffers and free this rank's (call on every rank, after a barrier)."""
        self._unmap()
        for b in (self.rows, self.scales, self.back):
            b.free()

    def _unmap(self):
        for p in self._imported:
            capi.check(self.L.xs_moe_ipc_close(C.c_void_p(p)))
        self._imported = []


# ------------------------------------------------------------------------------------------------------------
# the layer
# ------------------------------------------------------------------------------------------------------------
class ExpertParallelMoE:
    """forward(x_local (T,H)) -> out_local (T,H).  `ops` supplies route / permute / payload / gather / grouped_mlp /
    shared_mlp / combine on this rank's device; `group` is the torch.distributed process group (None = world)."""

    def __init__(self, ops, router_w, router_bias, num_experts, top_k, has_shared, group=None):
        self.ops = ops
        self.router_w, self.router_bias = router_w, router_bias
        self.E, self.K, self.S = num_experts, top_k, has_shared
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.E % self.world != 0:
            raise ValueError("expert count mismatch: experts must divide evenly over ranks")
        self.last_plan = None

    def _all_gather_counts_start(self, counts):
        if self.world == 1:
            return counts
        out = torch.empty(self.world * self.E, dtype=torch.int32, device=counts.device)
        dist.all_gather_into_tensor(out, counts.contiguous(), group=self.group)
        return out

    def _all_gather_counts_finish(self, gathered):
        return gathered.view(self.world, self.E).cpu().numpy()  # the one host synchronisation of the layer

    def _a2a(self, t, out_rows, in_splits, out_splits):
        out = torch.empty((out_rows, *t.shape[1:]), dtype=t.dtype, device=t.device)
        if self.world == 1:
            out.copy_(t)
            return out
        dist.all_to_all_single(out, t.contiguous(), [int(v) for v in out_splits], [int(v) for v in in_splits], group=self.group)
        return out

    def forward_peer(self, x, px, marks=None):
        """The layer with both exchanges as peer-memory kernels (`px`: this rank's connected PeerExchange).  Nothing
        here synchronises with the host; the two barriers are one-element all-reduces on the stream."""
        ops = self.ops

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        side = ops.side_stream
        shared = None
        if self.S:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                shared = ops.shared_mlp(x, None)
        ids, w = ops.route(x, self.router_w, self.router_bias)
        counts, offsets, perm, inv = ops.permute(ids)
        mark("route+permute")
        all_counts = self._all_gather_counts_start(counts)
        px.plan(all_counts)
        mark("counts exchange + plan (device)")
        px.dispatch(x, ids, inv, offsets, ops.ws)
        self._barrier()
        mark("dispatch (peer stores) + barrier")
        y_grouped = ops.grouped_mlp([px.rows, px.scales if px.fmt != capi.BF16 else None], px.offsets_local, px.capacity)
        mark("grouped expert MLP")
        px.give_back(y_grouped, all_counts, ops.ws)
        self._barrier()
        mark("return (peer stores) + barrier")
        if self.S:
            torch.cuda.current_stream().wait_stream(side)
            shared.record_stream(torch.cuda.current_stream())
        mark("always-on expert")
        out = ops.combine(px.back, inv, w, shared)
        mark("combine")
        return out

    def capture_peer(self, x_static, px):
        """forward_peer(x_static, px) as a CUDA graph -- possible because nothing in it returns to the host: every
        size the kernels and the collectives need is fixed (buffers sized for the worst routing), every count is read
        on the device.  Returns (graph, out_static); refill x_static, replay, read out_static.  Collective: every
        rank captures, and later replays, the same number of times.  The graph holds the communicator: call
        graph.reset() before the process group is destroyed, or the destroy blocks."""
        warm = torch.cuda.Stream()
        warm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(warm):
            for _ in range(2):
                self.forward_peer(x_static, px)
        torch.cuda.current_stream().wait_stream(warm)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.forward_peer(x_static, px)
        return graph, out

    def _barrier(self):
        if self.world > 1:
            if not hasattr(self, "_token"):
                self._token = torch.zeros(1, dtype=torch.int32, device="cuda")
            dist.all_reduce(self._token, group=self.group)

    def forward(self, x, marks=None):
        """marks: optional list; when given, (name, cuda event) pairs are appended after each phase (device ops only)."""
        ops, K = self.ops, self.K

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        side = getattr(ops, "side_stream", None)
        shared = None
        if self.S and side is not None:
            # the always-on expert needs only x: it runs on a second stream next to routing and the exchange
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                shared = ops.shared_mlp(x, None)
        ids, w = ops.route(x, self.router_w, self.router_bias)
        counts, offsets, perm, inv = ops.permute(ids)
        mark("route+permute")
        gathered = self._all_gather_counts_start(counts)  # in flight while the rows are quantised and packed
        payload = ops.payload(x)
        tok = torch.div(perm, K, rounding_mode="floor").to(torch.int32)
        send = [ops.gather(p, tok) for p in payload]  # rows in (expert, token) order = grouped by destination rank
        mark("quantise+pack")
        plan = EpPlan(self._all_gather_counts_finish(gathered), self.rank)
        self.last_plan = plan
        mark("counts exchange + plan (host sync)")
        recv = [self._a2a(s, plan.n_recv, plan.send_splits, plan.recv_splits) for s in send]
        mark("dispatch all-to-all")
        maps = torch.from_numpy(plan.packed_maps()).to(x.device, non_blocking=True)
        n_off = plan.El + 1
        off_local, g_from_a, a_from_g = maps[:n_off], maps[n_off:n_off + plan.n_recv], maps[n_off + plan.n_recv:]
        grouped = [ops.gather(r, g_from_a) for r in recv]
        mark("regroup")
        y_grouped = ops.grouped_mlp(grouped, off_local, plan.n_recv)
        mark("grouped expert MLP")
        y_arrival = ops.return_rows(y_grouped, a_from_g)
        y_back = self._a2a(y_arrival, int(plan.send_splits.sum()), plan.recv_splits, plan.send_splits)
        mark("combine all-to-all")
        if self.S and side is None:
            shared = ops.shared_mlp(x, payload)
        elif self.S:
            torch.cuda.current_stream().wait_stream(side)
            shared.record_stream(torch.cuda.current_stream())  # allocated on the side stream, consumed here
        mark("always-on expert")
        out = ops.combine(y_back, inv, w, shared)
        mark("combine")
        return out
