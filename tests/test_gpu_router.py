"""Router parity on the GPU, through the C ABI: ids and weights bit-exact against
the CPU reference on identical logits; permutation tables bit-exact."""
from pathlib import Path

import numpy as np
import pytest
import torch

from lumen_b200 import moe, synth
from oracle import oracle

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"


def test_device_expf_is_libm_exact(cuda_lib):
    rng = np.random.default_rng(0)
    x = np.concatenate([-np.abs(rng.standard_normal(200000) * 20), rng.standard_normal(100000) * 30,
                        np.array([0.0, -0.0, -103.9, -104.5, -87.4, 88.7, 89.0, -63.0999, 32.564632], np.float64),
                        np.frombuffer(np.array([0xc27c65d9, 0x4202422f, 0xff800000, 0x7f800000], np.uint32).tobytes(),
                                      np.float32).astype(np.float64)]).astype(np.float32)
    got = moe.debug_expf(torch.from_numpy(x).cuda()).cpu().numpy()
    import ctypes
    libm = ctypes.CDLL("libm.so.6")
    libm.expf.restype = ctypes.c_float
    libm.expf.argtypes = [ctypes.c_float]
    ref = np.array([libm.expf(float(v)) for v in x], np.float32)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("gating,tag", [(0, "softmax"), (1, "sigmoid")])
def test_topk_golden_vectors(cuda_lib, gating, tag):
    d = np.load(G / "router_topk.npz")
    lg = d["logits"]
    sc = moe.allocate_moe_scratch(2048, 768, 128, 8, 64, gating)
    for T in (1, 4, 16, lg.shape[0]):  # small-batch kernel and large-batch kernels
        ids, w = sc.topk_from_logits(torch.from_numpy(lg[:T].copy()).cuda())
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), d[f"ids_{tag}"][:T])
        assert np.array_equal(w.cpu().numpy().view(np.uint32), d[f"w_{tag}"][:T].view(np.uint32))


@pytest.mark.parametrize("T,kind", [(1, "normal"), (16, "tau"), (333, "tau"), (4096, "zipf"), (4096, "ties")])
def test_topk_and_permutation_bit_exact(cuda_lib, T, kind):
    E, K = 128, 8
    if kind == "normal":
        lg = synth.uniform_logits(T, E, 3, tau=1.0)
    elif kind == "tau":
        lg = synth.uniform_logits(T, E, 4, tau=0.02)
    elif kind == "zipf":
        lg = synth.zipf_logits(T, E, 5)
    else:
        lg = torch.round(synth.uniform_logits(T, E, 6, tau=2.0)) / 4  # many exact ties
    sc = moe.allocate_moe_scratch(2048, 768, E, K, T)
    ids, w = sc.topk_from_logits(lg)
    r = sc.get_routing(T)
    o_ids, o_w = oracle.topk_from_logits(lg.cpu().numpy(), K, 0)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), o_ids)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), o_w.view(np.uint32))
    ce, cst, d2c, bounds = oracle.counting_sort(o_ids, E)
    assert np.array_equal(r["expert_bounds"], bounds)
    assert np.array_equal(r["col_src_tok"], cst)
    assert np.array_equal(r["dst_to_col"], d2c)
    # size-independent properties
    assert np.all(np.diff(bounds) >= 0) and bounds[-1] == T * K
    assert sorted(d2c.tolist()) == list(range(T * K))
    np.testing.assert_allclose(r["weights"].sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("E,K", [(256, 16), (64, 16), (256, 1), (16, 16)])
@pytest.mark.parametrize("gating", [0, 1])
def test_topk_limits_of_expert_and_slot_counts(cuda_lib, E, K, gating):
    """The reference's fused router serves K <= 16 and E in {64, 128, 256}
    (topk_moe_fused.cu:298-358): ids, weights and permutation stay bit-exact at those
    limits, through the small-batch and the large-batch kernels."""
    for T in (1, 3, 16, 700):
        lg = torch.round(synth.uniform_logits(T, E, 11 + T, tau=0.5) * 64) / 64  # some exact ties
        sc = moe.allocate_moe_scratch(256, 128, E, K, T, gating)
        ids, w = sc.topk_from_logits(lg)
        r = sc.get_routing(T)
        o_ids, o_w = oracle.topk_from_logits(lg.cpu().numpy(), K, gating)
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), o_ids)
        assert np.array_equal(w.cpu().numpy().view(np.uint32), o_w.view(np.uint32))
        ce, cst, d2c, bounds = oracle.counting_sort(o_ids, E)
        assert np.array_equal(r["expert_bounds"], bounds)
        assert np.array_equal(r["col_src_tok"], cst)
        assert np.array_equal(r["dst_to_col"], d2c)


@pytest.mark.parametrize("T", [1, 16, 200])
def test_route_only_against_cpu_router(cuda_lib, T):
    """Logits computed on the GPU sum in a different order than the sequential CPU
    dot product, so ids are compared softly: any mismatch must be a near-tie."""
    from tests.gpu_util import make_layer
    H, I, E, K = 512, 128, 64, 8
    lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, 1, seed=2, max_tokens=T, numpy_blob=True)
    x = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(1), device="cuda")
    ids, w, lg = sc.route_only(layer, x, want_logits=True)
    router = blob_np[:lay.router_bytes].view(np.float32).reshape(E, H)
    xn = x.cpu().numpy()
    for t in range(T):
        o_ids, o_w, o_lg = oracle.router_softmax(xn[t], router, H, E, K)
        np.testing.assert_allclose(lg[t].cpu().numpy(), o_lg, rtol=0, atol=2e-5)
        g = ids[t].cpu().numpy().astype(np.uint32)
        if not np.array_equal(g, o_ids):
            srt = np.sort(o_lg)[::-1]
            assert np.min(np.abs(np.diff(srt[:K + 1]))) < 1e-5, "ids differ without a near-tie"
        else:
            np.testing.assert_allclose(w[t].cpu().numpy(), o_w, rtol=1e-4, atol=1e-6)
    # feeding the GPU's own logits back through the CPU top-k must agree bit for bit
    o_ids, o_w = oracle.topk_from_logits(lg.cpu().numpy(), K, 0)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), o_ids)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), o_w.view(np.uint32))


@pytest.mark.parametrize("T,act", [(1, torch.float32), (3, torch.float32), (16, torch.float32), (4096, torch.float32),
                                   (4096, torch.bfloat16)])
def test_router_logits_at_the_headline_shape(cuda_lib, T, act):
    """logit[t,e] = sum_j W_r[e,j] x[t,j] (cuda/moe.rs:6456-6463) at H = 2048, E = 128 for the
    small-batch router (T <= 16) and the batched one (any T, f32 and bf16 activations). (The
    persistent decode kernel keeps its logits in shared memory; tests/test_gpu_decode.py checks
    the experts it selects from them.)"""
    H, I, E, K = 2048, 768, 128, 8
    lay = synth.LayerLayout(H, I, E, 1)
    blob = synth.make_layer_blob(lay, 21)
    sc = moe.allocate_moe_scratch(H, I, E, K, T)
    layer = sc.prepare_router_only(blob, lay.meta().router_weight_off)
    x = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(T), device="cuda").to(act)
    router = blob[:lay.router_bytes].cpu().numpy().view(np.float32).reshape(E, H)
    xn = x.float().cpu().numpy()
    sample = sorted(set([0, T // 3, T - 1]))
    if act == torch.float32:
        ids, w, lg = sc.route_only(layer, x, want_logits=True)
        for t in sample:
            o_lg = oracle.router_logits(xn[t], router, H, E)
            np.testing.assert_allclose(lg[t].cpu().numpy(), o_lg, rtol=0, atol=3e-5)
        o_ids, o_w = oracle.topk_from_logits(lg.cpu().numpy(), K, 0)
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), o_ids)
        assert np.array_equal(w.cpu().numpy().view(np.uint32), o_w.view(np.uint32))
    else:
        # bf16 activations only enter through the prefill call: ids must be the CPU top-k of logits
        # that agree with the CPU dot products (checked through the set of chosen experts)
        full = synth.make_layer_blob(lay, 21)
        fl = sc.prepare_layer(full, lay.meta())
        sc.prefill(fl, x, torch.zeros((T, H), device="cuda"))
        r = sc.get_routing(T)
        for t in sample:
            o_lg = oracle.router_logits(xn[t], router, H, E)
            o_ids, _ = oracle.topk_from_logits(o_lg[None, :], K, 0)
            srt = np.sort(o_lg)[::-1]
            if np.min(np.abs(np.diff(srt[:K + 1]))) > 1e-4:
                assert np.array_equal(r["ids"][t], o_ids[0])


def test_batched_router_logits_do_not_depend_on_the_batch(cuda_lib):
    """A token's logits must be the same bits whether it is routed alone in a shard or inside the
    whole batch (an expert-parallel rank routes its shard and must pick what one GPU picks)."""
    H, I, E, K = 1024, 128, 64, 4
    lay = synth.LayerLayout(H, I, E, 1)
    blob = synth.make_layer_blob(lay, 5)
    sc = moe.allocate_moe_scratch(H, I, E, K, 3000)
    layer = sc.prepare_router_only(blob, lay.meta().router_weight_off)
    x = torch.randn((3000, H), generator=torch.Generator("cuda").manual_seed(2), device="cuda")
    ids_all, w_all, lg_all = sc.route_only(layer, x, want_logits=True)
    for lo, hi in ((0, 17), (1000, 1777), (2900, 3000)):
        ids, w, lg = sc.route_only(layer, x[lo:hi].contiguous(), want_logits=True)
        assert torch.equal(lg, lg_all[lo:hi]) and torch.equal(ids, ids_all[lo:hi]) and torch.equal(w, w_all[lo:hi])


def test_quantizers_bit_exact(cuda_lib):
    g = torch.Generator("cuda").manual_seed(9)
    w = torch.randn(32 * 4096, generator=g, device="cuda") * 0.02
    w[:32] = 0.0                       # all-zero block
    w[32:64] = 1e-7                    # scale in the f16 subnormal range
    w[64:96] = torch.linspace(-6e5, 6e5, 32, device="cuda")  # scale clamp / saturation
    w[96] = 0.5 * 0.02                 # exact .5 rounding cases
    for quant in (0, 1, 2):
        got = moe.quantize(w, quant).cpu().numpy()
        ref = oracle.quantize(w.cpu().numpy(), quant)
        assert np.array_equal(got, ref), quant


@pytest.mark.parametrize("T,epr,act", [(200, 16, torch.bfloat16), (37, 4, torch.bfloat16), (90, 8, torch.float32)])
def test_ep_prepare_and_device_tables(cuda_lib, T, epr, act):
    """lumen_moe_ep_prepare (send side of the expert-parallel form) and
    lumen_moe_get_routing_device against the host copy of the same routing tables."""
    H, I, E, K = 256, 128, 32, 4
    lay = synth.LayerLayout(H, I, E, 1)
    blob = synth.make_layer_blob(lay, 9)
    sc = moe.allocate_moe_scratch(H, I, E, K, T)
    layer = sc.prepare_router_only(blob, lay.meta().router_weight_off)
    x = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(T), device="cuda").to(act)
    ids, w = sc.route_only(layer, x.float().contiguous())
    rows, local_ids, send_counts = sc.ep_prepare(x, epr)
    dev = sc.get_routing_device(T, x.device)
    torch.cuda.synchronize()
    r = sc.get_routing(T)
    assert np.array_equal(dev["dst_to_col"].cpu().numpy(), r["dst_to_col"])
    assert np.array_equal(dev["expert_bounds"].cpu().numpy(), r["expert_bounds"])
    cst = dev["col_src_tok"].cpu().numpy()
    cex = dev["col_expert"].cpu().numpy()
    # column c holds pair p with dst_to_col[p] == c: its token is p // K and its expert ids[p]
    p_of_col = np.empty(T * K, np.int64)
    p_of_col[r["dst_to_col"]] = np.arange(T * K)
    assert np.array_equal(cst, p_of_col // K)
    assert np.array_equal(cex, r["ids"].reshape(-1)[p_of_col])
    # bf16 activations travel unchanged; f32 ones as f16 (round to nearest)
    wire = x if act == torch.bfloat16 else x.to(torch.float16)
    assert rows.dtype == wire.dtype and torch.equal(rows, wire[torch.from_numpy(cst).cuda().long()])
    assert np.array_equal(local_ids.cpu().numpy(), cex % epr)
    b = r["expert_bounds"]
    assert np.array_equal(send_counts.cpu().numpy(), np.diff(b[::epr]))
