"""Expert-parallel layer on 2 GPUs (NCCL) against the single-GPU result. Needs two
devices; skipped otherwise (the host logic is covered on CPU by test_ep_gloo.py)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
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
        Tl = T // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        route_fn, expert_fn, keep = ep.cuda_layer_fns(H, I, E, K, 1, blob, rank, world, Tl)
        layer = ep.ExpertParallelMoe(E, K, route_fn, expert_fn, combine_fn=keep["combine_fn"], route_takes_slot=True)
        # three calls: the first is eager, the second captures the routing side into a CUDA graph,
        # the third replays it; all must give the same result
        outs = [layer.forward(x_all[sl].contiguous(), res_all[sl].contiguous()).clone() for _ in range(3)]
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        out = outs[2]
        # the pipelined form (two parts on side streams; eager, capture, replay): same bits
        for _ in range(3):
            assert torch.equal(layer.forward_pipelined(x_all[sl].contiguous(), res_all[sl].contiguous(), 2), out)
        sc = moe.allocate_moe_scratch(H, I, E, K, T, device=rank)  # contexts are per device
        full = sc.prepare_layer(blob, lay.meta())
        ref = sc.prefill(full, x_all, res_all)[sl]
        rel = float(((out - ref) - 0).norm() / (ref - res_all[sl]).norm())
        r = sc.get_routing(T)
        ids_ok = bool((torch.from_numpy(r["ids"][sl].astype("int32")).to(dev) == layer.last["ids"]).all())
        # stack of 3 layers, f32 activations (f16 on the wire), against lumen_moe_stack_prefill on one GPU
        L = 3
        blobs = [synth.make_layer_blob(lay, 10 + l, device=dev) for l in range(L)]
        gammas = [(1.0 + 0.1 * torch.randn(H, generator=g, device=dev)).contiguous() for _ in range(L)]
        x0 = torch.randn((T, H), generator=g, device=dev)
        stack = ep.ExpertParallelStack(H, I, E, K, 1, blobs, gammas, rank, world, Tl, 1e-6)
        ys = [stack.forward(x0[sl].contiguous()).clone() for _ in range(3)]
        assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[2])
        stack.chunks = 2
        for _ in range(3):
            assert torch.equal(stack.forward(x0[sl].contiguous()), ys[0])
        full_layers = [sc.prepare_layer(b, lay.meta()) for b in blobs]
        want = sc.stack_prefill(full_layers, gammas, x0.clone(), 1e-6)[sl]
        rel_stack = float((ys[2] - want).norm() / (want - x0[sl]).norm())
        q.put((rank, max(rel, rel_stack), ids_ok))
    finally:
        dist.destroy_process_group()


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
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, rel, ids_ok in results:
        assert ids_ok
        assert rel < 1e-3, (rank, rel)
