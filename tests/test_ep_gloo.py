"""Expert-parallel dispatch/combine plumbing on two CPU ranks (gloo): the
all-to-all bookkeeping of lumen_b200/ep.py with the CPU oracle standing in for
the routing and expert kernels. Output of every rank must equal the
single-process reference layer on that rank's tokens."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

H, I, E, K, QUANT = 64, 64, 8, 2, 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tokens_per_rank, result_q, chunks=1):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lumen_b200 import ep
        from lumen_b200.synth import LayerLayout, make_layer_blob_numpy
        from oracle import oracle
        lay = LayerLayout(H, I, E, QUANT)
        blob = make_layer_blob_numpy(lay, 5, oracle.quantize)
        meta = lay.meta()
        router = blob[:lay.router_bytes].view(np.float32).reshape(E, H)
        epr = E // world
        T = tokens_per_rank[rank]
        rng = np.random.default_rng(100 + rank)
        x = rng.standard_normal((T, H)).astype(np.float32)

        def route_fn(xt):
            ids = np.zeros((xt.shape[0], K), np.uint32)
            w = np.zeros((xt.shape[0], K), np.float32)
            for t in range(xt.shape[0]):
                ids[t], w[t], _ = oracle.router_softmax(xt[t].numpy(), router, H, E, K)
            return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w)

        def expert_fn(rows, local_ids):
            out = np.zeros((rows.shape[0], H), np.float32)
            r = rows.float().numpy()
            for i in range(rows.shape[0]):
                e = rank * epr + int(local_ids[i])
                g = oracle.matvec(blob[int(meta.expert_gate_offs[e]):], r[i], I, H, QUANT)
                u = oracle.matvec(blob[int(meta.expert_up_offs[e]):], r[i], I, H, QUANT)
                out[i] = oracle.matvec(blob[int(meta.expert_down_offs[e]):], oracle.swiglu(g, u), H, I, QUANT)
            return torch.from_numpy(out)

        layer = ep.ExpertParallelMoe(E, K, route_fn, expert_fn, wire_dtype=torch.float32, combine_dtype=torch.float32)
        if chunks > 1:
            out = layer.forward_pipelined(torch.from_numpy(x), torch.from_numpy(x), chunks).numpy()
        else:
            out = layer.forward(torch.from_numpy(x), torch.from_numpy(x)).numpy()
        if T > 0:
            ref, ids, _ = oracle.moe_layer(blob, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs,
                                           QUANT, H, I, E, K, x, x)
            err = float(np.linalg.norm(out - ref) / np.linalg.norm(ref))
            ids_ok = bool(np.array_equal(layer.last["ids"].numpy().astype(np.uint32), ids))
        else:
            err, ids_ok = 0.0, True
        # every pair is sent exactly once and received by the owner of its expert
        sent = sum(layer.last["send_counts"])
        result_q.put((rank, err, ids_ok, sent == T * K, layer.last["recv_counts"]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens_per_rank,chunks", [((5, 9), 1), ((4, 0), 1), ((5, 9), 2), ((7, 1), 3)])
def test_expert_parallel_two_ranks_gloo(tokens_per_rank, chunks):
    """chunks > 1: the pipelined form (tokens cut into parts, one exchange of all parts' counts);
    a rank with fewer tokens than parts has empty parts."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tokens_per_rank, q, chunks)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    total_recv = 0
    for rank, err, ids_ok, sent_ok, recv in results:
        assert ids_ok and sent_ok
        assert err < 1e-6, (rank, err)
        total_recv += sum(recv)
    assert total_recv == sum(tokens_per_rank) * K


def test_dispatch_plan_groups_by_rank_in_compact_column_order():
    from lumen_b200 import ep
    ids = torch.tensor([[3, 1], [1, 5], [3, 0], [1, 3]], dtype=torch.int32)  # the reference's sort fixture
    order, counts, local = ep.dispatch_plan(ids, experts_per_rank=3, world=2)
    assert counts.tolist() == [4, 4]                      # experts 0-2 -> rank 0, 3-5 -> rank 1
    assert (ids.reshape(-1)[order]).tolist() == [0, 1, 1, 1, 3, 3, 3, 5]
    assert order.tolist() == [5, 1, 2, 6, 0, 4, 7, 3]     # stable: tokens ascending inside an expert
    assert local.tolist() == [0, 1, 1, 1, 0, 0, 0, 2]


def _push_worker(rank, world, port, tokens_per_rank, q):
    """The push form's layout logic on CPU ranks: every rank routes its own tokens, the ranks
    exchange only their per-expert counts, and from the count matrix each derives where its
    rows land in the owners' windows (ep.push_layout restates ep_dispatch_kernel). The 'stores'
    are emulated by gathering (owner, row, tag) triples."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lumen_b200 import ep
        from oracle import oracle
        epr = E // world
        T = tokens_per_rank[rank]
        rng = np.random.default_rng(7 + rank)
        ids = np.stack([rng.choice(E, K, replace=False) for _ in range(T)]).astype(np.uint32) if T else np.zeros((0, K), np.uint32)
        col_expert, col_src_tok, dst_to_col, bounds = oracle.counting_sort(ids, E) if T else (
            np.zeros(0, np.int32), np.zeros(0, np.int32), np.zeros(0, np.int32), np.zeros(E + 1, np.int32))
        mine = np.diff(bounds).astype(np.int64)
        allc = [None] * world
        dist.all_gather_object(allc, mine.tolist())
        base, rows = ep.push_layout(np.array(allc), epr)
        pushes = []
        for c in range(T * K):
            e = int(col_expert[c])
            pushes.append((e // epr, int(base[rank, e] + (c - bounds[e])), (rank, c, e, int(col_src_tok[c]))))
        everything = [None] * world
        dist.all_gather_object(everything, pushes)
        q.put((rank, rows.tolist(), [p for src in everything for p in src if p[0] == rank]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens_per_rank", [(6, 11), (5, 0)])
def test_push_layout_two_ranks_gloo(tokens_per_rank):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_push_worker, args=(r, world, port, tokens_per_rank, q), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    epr = E // world
    total = 0
    for rank, rows, landed in results:
        landed.sort(key=lambda p: p[1])
        # every row of the window is written exactly once, none beyond what the rank is sent
        assert [p[1] for p in landed] == list(range(rows[rank]))
        # grouped by expert, then by source rank, then in the source's own compact-column order:
        # the stable order of cuda/moe.rs:2115-2147 applied to all ranks' tokens together
        keys = [(tag[2], tag[0], tag[1]) for _, _, tag in landed]
        assert keys == sorted(keys)
        assert all(rank * epr <= tag[2] < (rank + 1) * epr for _, _, tag in landed)
        total += len(landed)
    assert total == sum(tokens_per_rank) * K
