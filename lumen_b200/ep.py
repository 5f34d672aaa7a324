"""Expert-parallel MoE layer over G ranks (one process per GPU, torch.distributed).

The reference is single-GPU (one context, one stream, cuda/ffi.rs:61-87); this is the
additive multi-GPU form of the same layer for multi-token batches:

  tokens are sharded over ranks (each rank routes its own tokens with the replicated
  router weight), experts are sharded E/G per rank. Per layer call:
    1. route locally                               (lumen_moe_route_only)
    2. all-to-all of per-destination row counts    (G x G integers)
    3. dispatch all-to-all-v: activation rows + local expert ids to the owning rank
    4. grouped expert products on the received rows (lumen_moe_prefill_routed, K = 1)
    5. combine all-to-all-v: expert outputs back to the token's home rank
    6. out[t] = residual[t] + sum_slot w[t,slot] * d[t,slot]   in slot order

The stable counting sort by expert (cuda/moe.rs:2115-2147) already groups the
(token, slot) pairs by destination rank, because experts are contiguous per rank.
Batch-1 decode does not use this path (replicas only).

The collective plumbing is backend-agnostic (NCCL on GPUs, gloo on CPU for the
host-logic tests): `route_fn` and `expert_fn` are injectable, the defaults call
the CUDA library.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def dispatch_plan(ids: torch.Tensor, experts_per_rank: int, world: int):
    """ids [T,K] (global expert ids) -> (order, send_counts, local_ids).

    order: permutation of the T*K (token, slot) pairs, stable by destination rank
    then by expert (tokens ascending, slots ascending inside an expert -- the
    reference's compact-column order); send_counts[r]: pairs going to rank r;
    local_ids: expert id relative to the owning rank, in `order`.
    """
    flat = ids.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    sorted_ids = flat[order]
    dest = torch.div(sorted_ids, experts_per_rank, rounding_mode="floor")
    send_counts = torch.bincount(dest, minlength=world)[:world]
    local_ids = (sorted_ids - dest * experts_per_rank).to(torch.int32)
    return order, send_counts, local_ids


def all_to_all_v(t: torch.Tensor, send_counts, recv_counts, group=None) -> torch.Tensor:
    out = t.new_empty((int(sum(recv_counts)),) + tuple(t.shape[1:]))
    dist.all_to_all_single(out, t.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


class ExpertParallelMoe:
    """One MoE layer, experts [rank*E/G, (rank+1)*E/G) resident on this rank.

    route_fn(x [T,H]) -> (ids int32 [T,K], weights f32 [T,K])
    expert_fn(rows [R,H], local_ids int32 [R]) -> d [R,H] (f32): the expert FFN of
        each row's local expert, unweighted.
    """

    def __init__(self, num_experts: int, top_k: int, route_fn: Callable, expert_fn: Callable, group=None,
                 combine_fn: Optional[Callable] = None,
                 wire_dtype: torch.dtype = torch.bfloat16, combine_dtype: torch.dtype = torch.float16,
                 route_takes_slot: bool = False):
        self.E, self.K = num_experts, top_k
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError("num_experts must be divisible by the number of ranks")
        self.epr = num_experts // self.world
        self.route_fn, self.expert_fn = route_fn, expert_fn
        self.combine_fn = combine_fn  # (back [T*K,H] in send order, residual, w, inv_order) -> out; None = torch ops
        self.wire_dtype = wire_dtype        # activation rows on the wire (bf16 inputs travel exactly)
        self.combine_dtype = combine_dtype  # expert outputs on the wire (f16, as the single-GPU path stores them)
        self.last = {}
        self.profile = False
        self._marks = []
        self.route_takes_slot = route_takes_slot  # route_fn(x, slot): one set of output buffers per part of forward_pipelined
        self._side_streams = None

    def _mark(self, name):
        if self.profile and torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def phase_times_ms(self):
        """Per-phase device times of the last forward (profile=True): [(phase, ms), ...]."""
        torch.cuda.synchronize()
        return [(b[0], a[1].elapsed_time(b[1])) for a, b in zip(self._marks[:-1], self._marks[1:])]

    def _send_side(self, normed: torch.Tensor, slot=None) -> dict:
        """Route `normed` and lay out what leaves this rank: rows in destination order, the
        rank-local expert id of every row, rows per destination rank, and what the combine needs."""
        routed = self.route_fn(normed) if slot is None else self.route_fn(normed, slot)
        ids, w = routed[0], routed[1]
        side = {"ids": ids, "w": w, "order": None, "inv": None}
        if len(routed) > 2 and "rows" in routed[2]:
            # the library produced the whole send side in one launch
            tables = routed[2]
            side.update(rows=tables["rows"], local_ids=tables["local_ids"], sc=tables["send_counts"],
                        inv=tables["dst_to_col"])
            return side
        if len(routed) > 2:
            # the router's own counting sort is the send plan (compact-column order)
            tables = routed[2]
            tok = tables["col_src_tok"].to(torch.int64)
            side["inv"] = tables["dst_to_col"]
            if self.combine_fn is None:
                d2c = tables["dst_to_col"].to(torch.int64)
                order = torch.empty_like(d2c)
                order[d2c] = torch.arange(d2c.numel(), device=d2c.device)
                side["order"] = order
            b = tables["expert_bounds"].to(torch.int64)
            edges = b[torch.arange(0, self.E + 1, self.epr, device=b.device)]
            side["sc"] = edges[1:] - edges[:-1]
            side["local_ids"] = (tables["col_expert"] % self.epr).to(torch.int32)
        else:
            order, send_counts, local_ids = dispatch_plan(ids, self.epr, self.world)
            tok = torch.div(order, self.K, rounding_mode="floor")
            side.update(order=order, sc=send_counts, local_ids=local_ids)
        side["rows"] = normed[tok].to(self.wire_dtype)
        return side

    def _combine(self, back: torch.Tensor, residual: torch.Tensor, side: dict) -> torch.Tensor:
        """out[t] = residual[t] + sum_slot w[t,slot] * d[t,slot] in slot order; `back` is in send order."""
        T, H = residual.shape
        w, order = side["w"], side["order"]
        if self.combine_fn is not None:
            inv = side["inv"]
            if inv is None:
                inv = torch.empty(T * self.K, dtype=torch.int32, device=residual.device)
                inv[order] = torch.arange(T * self.K, dtype=torch.int32, device=residual.device)
            return self.combine_fn(back, residual, w, inv)
        dpair = torch.empty((T * self.K, H), dtype=torch.float32, device=residual.device)
        dpair[order] = back.to(torch.float32)
        dpair = dpair.view(T, self.K, H)
        out = residual.clone()
        for slot in range(self.K):
            out += w[:, slot, None] * dpair[:, slot]
        return out

    def forward(self, normed: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        self._marks = []
        self._mark("start")
        side = self._send_side(normed)
        self._mark("route")
        # (2) counts
        sc = side["sc"].to(torch.int64)
        rc = torch.empty_like(sc)
        dist.all_to_all_single(rc, sc, group=self.group)
        send_l, recv_l = sc.tolist(), rc.tolist()  # the one host sync of the call (NCCL sizes are host arguments)
        self._mark("plan+counts")
        # (3) dispatch rows and local expert ids
        recv_rows = all_to_all_v(side["rows"], send_l, recv_l, self.group)
        recv_ids = all_to_all_v(side["local_ids"], send_l, recv_l, self.group)
        self._mark("dispatch")
        # (4) local experts
        d = self.expert_fn(recv_rows, recv_ids)
        self._mark("experts")
        # (5) combine
        back = all_to_all_v(d.to(self.combine_dtype), recv_l, send_l, self.group)
        self._mark("combine_a2a")
        # (6) weighted sum in slot order
        self.last = {"ids": side["ids"], "weights": side["w"], "send_counts": send_l, "recv_counts": recv_l}
        out = self._combine(back, residual, side)
        self._mark("combine")
        return out

    def forward_pipelined(self, normed: torch.Tensor, residual: torch.Tensor, chunks: int = 2) -> torch.Tensor:
        """The same layer with the tokens cut into `chunks` parts whose dispatch, expert products and
        combine overlap: all parts are routed first and their row counts exchanged in ONE
        all-to-all (one host sync), then the collectives run on one side stream and the expert
        products on another, so that part c+1 is on the wire while part c is in the GEMMs and part
        c's outputs travel back under part c+1's GEMMs. `chunks` must be the same on every rank."""
        T = normed.shape[0]
        bounds = [T * c // chunks for c in range(chunks + 1)]
        parts = [(bounds[c], bounds[c + 1]) for c in range(chunks)]
        sides = [self._send_side(normed[b0:b1], c if self.route_takes_slot else None) for c, (b0, b1) in enumerate(parts)]
        sc = torch.stack([s["sc"].to(torch.int64) for s in sides])  # [chunks, G]
        sc_t = sc.t().contiguous()                                  # per destination rank: its `chunks` counts
        rc_t = torch.empty_like(sc_t)
        dist.all_to_all_single(rc_t, sc_t, group=self.group)
        send_l, recv_l = sc.tolist(), rc_t.t().tolist()             # the one host sync of the call
        cuda = normed.is_cuda
        if cuda:
            main = torch.cuda.current_stream()
            if self._side_streams is None:
                self._side_streams = (torch.cuda.Stream(), torch.cuda.Stream())
            s_comm, s_comp = self._side_streams
            s_comm.wait_stream(main)
            s_comp.wait_stream(main)
            on = lambda st: torch.cuda.stream(st)
        else:
            import contextlib
            s_comm = s_comp = None
            on = lambda st: contextlib.nullcontext()

        def mark(st):
            if not cuda:
                return None
            ev = torch.cuda.Event()
            ev.record(st)
            return ev

        recv, d_out, backs = [], [], []
        for c in range(chunks):
            with on(s_comm):
                rr = all_to_all_v(sides[c]["rows"], send_l[c], recv_l[c], self.group)
                ri = all_to_all_v(sides[c]["local_ids"], send_l[c], recv_l[c], self.group)
                recv.append((rr, ri, mark(s_comm)))
        for c in range(chunks):
            with on(s_comp):
                if cuda:
                    s_comp.wait_event(recv[c][2])
                d = self.expert_fn(recv[c][0], recv[c][1]).to(self.combine_dtype)
                d_out.append((d, mark(s_comp)))
        for c in range(chunks):
            with on(s_comm):
                if cuda:
                    s_comm.wait_event(d_out[c][1])
                backs.append(all_to_all_v(d_out[c][0], recv_l[c], send_l[c], self.group))
        if cuda:
            main.wait_stream(s_comm)
            main.wait_stream(s_comp)
        self.last = {"ids": torch.cat([s["ids"] for s in sides]), "weights": torch.cat([s["w"] for s in sides]),
                     "send_counts": [sum(v) for v in zip(*send_l)], "recv_counts": [sum(v) for v in zip(*recv_l)]}
        return torch.cat([self._combine(backs[c], residual[b0:b1], sides[c]) for c, (b0, b1) in enumerate(parts)])


def push_layout(counts, experts_per_rank: int):
    """Host restatement of the layout every rank derives, on the device, from the count matrix
    (ep_dispatch_kernel): counts[s][e] = pairs of source rank s for global expert e. Returns
    base[s][e], the row in the window of e's owner where source s's pairs of expert e start
    (rows grouped by expert, inside an expert by source rank, inside a source in its own
    compact-column order), and rows[r], the rows rank r receives."""
    import numpy as np
    counts = np.asarray(counts, dtype=np.int64)
    G, E = counts.shape
    tot = counts.sum(axis=0)
    base = np.zeros((G, E), dtype=np.int64)
    rows = np.zeros(E // experts_per_rank, dtype=np.int64)
    for e in range(E):
        first = (e // experts_per_rank) * experts_per_rank
        lower = int(tot[first:e].sum())
        base[:, e] = lower + np.concatenate(([0], np.cumsum(counts[:-1, e])))
    for r in range(E // experts_per_rank):
        rows[r] = int(tot[r * experts_per_rank:(r + 1) * experts_per_rank].sum())
    return base, rows


class PushExpertParallel:
    """lumen_moe_prefill_ep behind a torch.distributed rendezvous. The process group is used for
    one thing only, at set-up: gathering the 64-byte handles of the ranks' windows (what a Rust
    host would do over its own launcher's channel). A layer call is one library call per rank;
    rows and results travel by plain peer stores over NVLink, issued by the library's kernels."""

    def __init__(self, H: int, I: int, E: int, K: int, max_tokens: int, rank: int, world: int, device: int,
                 gating_mode: int = 0, group=None, flags: int = 0, recv_rows: int = 0):
        from . import moe
        self.rank, self.world = rank, world
        self.sc = moe.allocate_moe_scratch(H, I, E, K, max_tokens, gating_mode, device, flags)
        handle = self.sc.ep_create(rank, world, max_tokens, recv_rows)
        handles = [handle]
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, handle, group=group)
        self.sc.ep_attach(handles)
        self.group = group

    def prepare_layer(self, full_blob: torch.Tensor, meta):
        return self.sc.ep_prepare_layer(full_blob, meta)

    def forward(self, layer, normed: torch.Tensor, residual: torch.Tensor, out: Optional[torch.Tensor] = None):
        return self.sc.prefill_ep(layer, normed, residual, out)

    def stack_forward(self, layers, gammas, x: torch.Tensor, eps: float, normed: Optional[torch.Tensor] = None):
        return self.sc.stack_prefill_ep(layers, gammas, x, eps, normed)

    def close(self):
        """Collective: no rank frees its window while a peer may still write to it."""
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        self.sc.close()


def cuda_layer_fns(H: int, I: int, E: int, K: int, quant: int, full_blob: torch.Tensor, rank: int, world: int,
                   max_tokens: int, gating_mode: int = 0, contexts=None) -> Tuple[Callable, Callable, dict]:
    """Builds route_fn / expert_fn on the CUDA library for this rank.

    `full_blob` is the complete layer blob (router + all experts) in the reference
    layout; only this rank's expert slice is repacked and kept by the expert
    context (K = 1, E/G experts); a second, router-only context routes from its own
    copy of the router weight, so the caller may drop `full_blob` afterwards.
    `contexts` = (route context, expert context) of an earlier call shares them between
    the layers of a stack (the calls of a stack are sequential)."""
    from . import moe, synth
    epr = E // world
    dev = full_blob.device.index
    lay = synth.LayerLayout(H, I, E, quant)
    meta = lay.meta()
    if contexts is None:
        route_sc = moe.allocate_moe_scratch(H, I, E, K, max_tokens, gating_mode, dev)
        exp_sc = moe.allocate_moe_scratch(H, I, epr, 1, max_tokens * K, gating_mode, dev)
    else:
        route_sc, exp_sc = contexts
    router_blob = full_blob[meta.router_weight_off: meta.router_weight_off + E * H * 4].clone()
    route_layer = route_sc.prepare_router_only(router_blob, 0)
    sl = slice(rank * epr, (rank + 1) * epr)
    local_meta = moe.MoeMeta(0, meta.expert_gate_offs[sl].copy(), meta.expert_up_offs[sl].copy(),
                             meta.expert_down_offs[sl].copy(), quant, quant)
    exp_layer = exp_sc.prepare_layer(full_blob, local_meta)

    def route_eager(x):
        ids, w = route_sc.route_only(route_layer, x.float().contiguous())
        rows, local_ids, send_counts = route_sc.ep_prepare(x.contiguous(), epr)
        d2c = torch.empty(x.shape[0] * K, dtype=torch.int32, device=x.device)
        route_sc.get_routing_device_into(x.shape[0], dst_to_col=d2c)
        return ids, w, {"rows": rows, "local_ids": local_ids, "send_counts": send_counts, "dst_to_col": d2c}

    # The routing side has no host synchronisation and fixed shapes per (tokens, dtype): its dozen
    # launches are replayed from a CUDA graph (static input and output buffers), which matters when a
    # rank holds only a few thousand tokens and the launches, not the kernels, set the time.
    graphs = {}

    def route_fn(x, slot=0):
        key = (tuple(x.shape), x.dtype, slot)  # a slot has its own graph and static output buffers
        entry = graphs.get(key)
        if entry is None:
            out = route_eager(x)  # first call: eager (one-time set-up inside the library must not be captured)
            graphs[key] = "warm"
            return out
        if entry == "warm":
            try:
                static_x = x.clone()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    static_out = route_eager(static_x)
                entry = graphs[key] = (g, static_x, static_out)
            except Exception:
                graphs[key] = "eager"
                return route_eager(x)
        if entry == "eager":
            return route_eager(x)
        g, static_x, static_out = entry
        static_x.copy_(x)
        g.replay()
        return static_out

    def expert_fn(rows, local_ids):
        if rows.shape[0] == 0:
            return torch.zeros((0, H), dtype=torch.float16, device=rows.device)
        return exp_sc.experts_routed_f16(exp_layer, rows.contiguous(), local_ids.contiguous())

    def combine_fn(back, residual, w, inv):
        return moe.combine_f16(back.contiguous(), residual, w.contiguous(), inv)

    return route_fn, expert_fn, {"combine_fn": combine_fn, "route_takes_slot": True, "route": route_sc, "experts": exp_sc,
                                 "layers": (route_layer, exp_layer), "router_blob": router_blob}


class ExpertParallelStack:
    """Stack of MoE FFN layers with identity mixers over G ranks, tokens sharded:
    x <- x + MoE_l(rmsnorm(x; gamma_l, eps)) per layer, the expert-parallel form of
    lumen_moe_stack_prefill. The norm and the residual are local to the token's home rank;
    f32 activations cross the wire as f16, the rounding the single-GPU grouped GEMM applies
    to its operand."""

    def __init__(self, H: int, I: int, E: int, K: int, quant: int, layer_blobs, gammas, rank: int, world: int,
                 max_tokens: int, eps: float, gating_mode: int = 0, group=None, chunks: int = 1):
        from . import moe
        self.eps, self.gammas, self._rmsnorm = eps, list(gammas), moe.rmsnorm
        self.chunks = chunks  # > 1: every layer runs forward_pipelined with that many parts
        self.layers, self._keep, ctx = [], [], None
        for blob in layer_blobs:  # any iterable: a generator lets each full blob be freed after its slice is repacked
            route_fn, expert_fn, keep = cuda_layer_fns(H, I, E, K, quant, blob, rank, world, max_tokens, gating_mode, ctx)
            ctx = (keep["route"], keep["experts"])
            self._keep.append(keep)
            self.layers.append(ExpertParallelMoe(E, K, route_fn, expert_fn, group=group, combine_fn=keep["combine_fn"],
                                                 route_takes_slot=True))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for layer, gamma in zip(self.layers, self.gammas):
            normed = self._rmsnorm(x, gamma, self.eps)
            x = layer.forward(normed, x) if self.chunks < 2 else layer.forward_pipelined(normed, x, self.chunks)
        return x
