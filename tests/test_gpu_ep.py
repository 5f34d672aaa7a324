"""Expert-parallel prefill (lumen_moe_prefill_ep: push dispatch/combine over peer memory,
no collective in the data path) against the single-GPU result. The one-rank form runs the
whole machinery (window, flags, dispatch, grouped GEMMs with the return map, combine) on one
GPU; the two-rank form needs two devices and is skipped otherwise (the layout logic is also
covered on CPU by test_ep_gloo.py). The older NCCL all-to-all form is kept as a cross-check."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,act,routing,quant", [(600, torch.bfloat16, "router", 1), (77, torch.float32, "zipf", 1),
                                                 (1, torch.float32, "router", 1), (300, torch.bfloat16, "zipf", 0),
                                                 (300, torch.float32, "router", 2), (1200, torch.bfloat16, "router", 1)])
def test_one_rank_window_equals_plain_prefill(cuda_lib, T, act, routing, quant):
    from lumen_b200 import ep, moe, synth
    from oracle import oracle
    H, I, E, K = 512, 256, 32, 4
    lay = synth.LayerLayout(H, I, E, quant)
    blob = synth.make_layer_blob(lay, 3)
    g = torch.Generator("cuda").manual_seed(4)
    x = torch.randn((T, H), generator=g, device="cuda").to(act)
    res = torch.randn((T, H), generator=g, device="cuda")
    lg = synth.zipf_logits(T, E, 5) if routing == "zipf" else None
    sc = moe.allocate_moe_scratch(H, I, E, K, T)
    full = sc.prepare_layer(blob, lay.meta())
    sc.set_logits_override(lg)
    ref = sc.prefill(full, x, res)
    r_ref = sc.get_routing(T)
    pe = ep.PushExpertParallel(H, I, E, K, max(700, T), 0, 1, 0)
    layer = pe.prepare_layer(blob, lay.meta())
    pe.sc.set_logits_override(lg)
    outs = [pe.forward(layer, x, res).clone() for _ in range(3)]  # the window is reused call after call
    torch.cuda.synchronize()
    assert pe.sc.poll_status() == 0
    for o in outs:
        assert torch.equal(o, ref)
    r = pe.sc.get_routing(T)
    assert np.array_equal(r["ids"], r_ref["ids"]) and np.array_equal(r["dst_to_col"], r_ref["dst_to_col"])
    # and a few tokens against the CPU reference
    sample = sorted(set([0, T // 2, T - 1]))
    xs = x[sample].float().cpu().numpy()
    meta = lay.meta()
    o_out, _, _ = oracle.moe_layer(blob.cpu().numpy(), 0, meta.expert_gate_offs, meta.expert_up_offs,
                                   meta.expert_down_offs, quant, H, I, E, K, xs, res[sample].cpu().numpy(),
                                   ids=r["ids"][sample], weights=r["weights"][sample], threads=8)
    got = outs[0][sample].cpu().numpy() - res[sample].cpu().numpy()
    want = o_out - res[sample].cpu().numpy()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-3


def test_expert_parallel_call_replayed_from_a_cuda_graph(cuda_lib):
    # the call number that tags the flags lives in device memory: a captured call can be replayed
    from lumen_b200 import ep, moe, synth
    H, I, E, K, T = 512, 256, 32, 4, 200
    lay = synth.LayerLayout(H, I, E, 1)
    blob = synth.make_layer_blob(lay, 3)
    g = torch.Generator("cuda").manual_seed(4)
    x = torch.randn((T, H), generator=g, device="cuda")
    res = torch.randn((T, H), generator=g, device="cuda")
    sc = moe.allocate_moe_scratch(H, I, E, K, T)
    ref = sc.prefill(sc.prepare_layer(blob, lay.meta()), x, res)
    pe = ep.PushExpertParallel(H, I, E, K, T, 0, 1, 0)
    layer = pe.prepare_layer(blob, lay.meta())
    out = torch.empty_like(res)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        pe.forward(layer, x, res, out)   # first call outside the capture (one-time set-up inside the library)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pe.forward(layer, x, res, out)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert pe.sc.poll_status() == 0
        assert torch.equal(out, ref)
    # eager calls still work after the replays
    assert torch.equal(pe.forward(layer, x, res), ref)


def test_receive_window_overflow_is_an_error_code(cuda_lib):
    # a window smaller than what the routing sends: no row may land outside it; the context reports it
    from lumen_b200 import _lib, ep, synth
    H, I, E, K, T = 512, 256, 32, 4, 300
    lay = synth.LayerLayout(H, I, E, 1)
    blob = synth.make_layer_blob(lay, 3)
    pe = ep.PushExpertParallel(H, I, E, K, T, 0, 1, 0, recv_rows=256)
    layer = pe.prepare_layer(blob, lay.meta())
    x = torch.randn((T, H), device="cuda")
    pe.forward(layer, x, torch.zeros((T, H), device="cuda"))
    torch.cuda.synchronize()
    assert pe.sc.poll_status() == _lib.INVALID_ARG
    pe.sc.clear_status()
    small = pe.forward(layer, x[:60].contiguous(), torch.zeros((60, H), device="cuda"))  # 240 rows fit
    torch.cuda.synchronize()
    assert pe.sc.poll_status() == _lib.OK and torch.isfinite(small).all()


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from datetime import timedelta
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=timedelta(seconds=120))
    try:
        from lumen_b200 import ep, moe, synth
        H, I, E, K, T = 512, 256, 32, 4, 600
        dev = f"cuda:{rank}"
        lay = synth.LayerLayout(H, I, E, 1)
        blob = synth.make_layer_blob(lay, 3, device=dev)
        g = torch.Generator(device=dev)
        g.manual_seed(4)
        x_all = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)
        res_all = torch.randn((T, H), generator=g, device=dev)
        # uneven shards: rank 0 takes 350 tokens, rank 1 the other 250
        cut = [0, 350, T] if world == 2 else [T * r // world for r in range(world + 1)]
        sl = slice(cut[rank], cut[rank + 1])
        sc = moe.allocate_moe_scratch(H, I, E, K, T, device=rank)  # contexts are per device
        full = sc.prepare_layer(blob, lay.meta())
        results = {}
        for routing in ("router", "zipf"):
            lg = synth.zipf_logits(T, E, 5, device=dev) if routing == "zipf" else None
            sc.set_logits_override(lg)
            ref = sc.prefill(full, x_all, res_all)[sl]
            r = sc.get_routing(T)
            pe = ep.PushExpertParallel(H, I, E, K, 400, rank, world, rank)
            layer = pe.prepare_layer(blob, lay.meta())
            pe.sc.set_logits_override(lg[sl].contiguous() if lg is not None else None)
            outs = [pe.forward(layer, x_all[sl].contiguous(), res_all[sl].contiguous()).clone() for _ in range(3)]
            torch.cuda.synchronize()
            assert pe.sc.poll_status() == 0
            mine = pe.sc.get_routing(cut[rank + 1] - cut[rank])
            results[routing] = (all(torch.equal(o, ref) for o in outs), bool((mine["ids"] == r["ids"][sl]).all()),
                                float((outs[0] - ref).norm() / (ref - res_all[sl]).norm()))
            pe.close()
        # stack of 3 layers, f32 residual stream, against lumen_moe_stack_prefill on one GPU
        sc.set_logits_override(None)
        L = 3
        blobs = [synth.make_layer_blob(lay, 10 + l, device=dev) for l in range(L)]
        gammas = [(1.0 + 0.1 * torch.randn(H, generator=g, device=dev)).contiguous() for _ in range(L)]
        x0 = torch.randn((T, H), generator=g, device=dev)
        want = sc.stack_prefill([sc.prepare_layer(b, lay.meta()) for b in blobs], gammas, x0.clone(), 1e-6)[sl]
        pe = ep.PushExpertParallel(H, I, E, K, 400, rank, world, rank)
        layers = [pe.prepare_layer(b, lay.meta()) for b in blobs]
        ys = [pe.stack_forward(layers, gammas, x0[sl].clone(), 1e-6).clone() for _ in range(2)]
        torch.cuda.synchronize()
        results["stack"] = (all(torch.equal(y, want) for y in ys), True,
                            float((ys[0] - want).norm() / (want - x0[sl]).norm()))
        pe.close()
        # the NCCL all-to-all form of the same layer (older path, kept as a cross-check)
        Tl = T // world
        sl2 = slice(rank * Tl, (rank + 1) * Tl)
        route_fn, expert_fn, keep = ep.cuda_layer_fns(H, I, E, K, 1, blob, rank, world, Tl)
        nl = ep.ExpertParallelMoe(E, K, route_fn, expert_fn, combine_fn=keep["combine_fn"], route_takes_slot=True)
        out2 = nl.forward(x_all[sl2].contiguous(), res_all[sl2].contiguous())
        ref2 = sc.prefill(full, x_all, res_all)[sl2]
        results["nccl"] = (True, True, float((out2 - ref2).norm() / (ref2 - res_all[sl2]).norm()))
        q.put((rank, results))
    except Exception as exc:  # the parent reports it; the process still leaves cleanly
        q.put((rank, {"error": (False, False, repr(exc))}))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_expert_parallel_matches_single_gpu(cuda_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = [q.get(timeout=300) for _ in range(2)]
        for p in procs:
            p.join(timeout=60)
    finally:
        # a rank that stalled must not keep the GPUs (NVLS is off, so ending a rank is safe)
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
            if p.is_alive():
                p.kill()
    for rank, res in results:
        assert "error" not in res, res
        for name, (bit_equal, ids_ok, rel) in res.items():
            assert ids_ok, (rank, name)
            assert rel < 1e-3, (rank, name, rel)
            if name != "nccl":
                assert bit_equal, (rank, name, rel)   # same operands, same order: same bits as one GPU
