"""Decode path (1..16 tokens) against the CPU reference, through the C ABI."""
from pathlib import Path

import numpy as np
import pytest
import torch

from lumen_b200 import moe, synth
from oracle import oracle
from tests.gpu_util import TOL_REL_L2, make_layer, oracle_layer, rel_l2

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
def test_golden_small_layer(cuda_lib, name):
    d = np.load(G / f"moe_small_{name}.npz")
    H, I, E, K, T, quant = (int(v) for v in d["dims"])
    meta = synth.LayerLayout(H, I, E, quant).meta()
    sc = moe.allocate_moe_scratch(H, I, E, K)
    layer = sc.prepare_layer(torch.from_numpy(d["blob"]).cuda(), meta)
    x = torch.from_numpy(d["x"]).cuda()
    out = sc.decode(layer, x, x.clone())
    r = sc.get_routing(T)
    assert np.array_equal(r["ids"], d["ids"])
    assert rel_l2(out.cpu().numpy(), d["ref_out"]) < TOL_REL_L2


@pytest.mark.parametrize("quant", [1, 0, 2])
@pytest.mark.parametrize("T", [1, 4, 16])
def test_decode_full_shape_identical_logits(cuda_lib, quant, T):
    """Headline shapes (H=2048, E=128, K=8, I=768); both sides route on the same logits."""
    H, I, E, K = 2048, 768, 128, 8
    lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, quant, seed=0)
    g = torch.Generator("cuda").manual_seed(1)
    x = torch.randn((T, H), generator=g, device="cuda")
    lg = synth.uniform_logits(T, E, 2, tau=0.05)
    sc.set_logits_override(lg)
    out = sc.decode(layer, x, x.clone())
    r = sc.get_routing(T)
    sc.set_logits_override(None)
    o_out, o_ids, o_w = oracle_layer(blob_np, meta, lay, K, x.cpu().numpy(), x.cpu().numpy(), logits=lg.cpu().numpy())
    assert np.array_equal(r["ids"], o_ids)
    assert np.array_equal(r["weights"].view(np.uint32), o_w.view(np.uint32))
    ce, cst, d2c, bounds = oracle.counting_sort(o_ids, E)
    assert np.array_equal(r["dst_to_col"], d2c) and np.array_equal(r["expert_bounds"], bounds)
    err = rel_l2(out.cpu().numpy() - x.cpu().numpy(), o_out - x.cpu().numpy())  # error of the MoE term itself
    assert err < TOL_REL_L2, err


@pytest.mark.parametrize("quant", [1, 0])
def test_decode_real_router_and_aliasing(cuda_lib, quant):
    H, I, E, K, T = 2048, 768, 128, 8, 4
    lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, quant, seed=3)
    x = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(5), device="cuda")
    buf = x.clone()
    sc.decode(layer, x, buf, buf)  # output written in place over the residual (backend_impl.rs:3570-3573)
    r = sc.get_routing(T)
    # route the oracle with the ids the GPU chose (its logits differ in the last bits)
    o_out, _, _ = oracle.moe_layer(blob_np, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs,
                                   quant, H, I, E, K, x.cpu().numpy(), x.cpu().numpy(), ids=r["ids"],
                                   weights=r["weights"], threads=8)
    assert rel_l2(buf.cpu().numpy() - x.cpu().numpy(), o_out - x.cpu().numpy()) < TOL_REL_L2
    # determinism: a second run is bit-identical
    buf2 = x.clone()
    sc.decode(layer, x, buf2, buf2)
    assert torch.equal(buf, buf2)


@pytest.mark.parametrize("shape", [(64, 64, 16, 4), (96, 160, 8, 2), (256, 32, 4, 1)])
@pytest.mark.parametrize("quant", [1, 0, 2])
def test_decode_small_and_ragged_shapes(cuda_lib, shape, quant):
    """Shapes that are not multiples of the 128-input tile (zero-padded groups), K=1, E=4."""
    H, I, E, K = shape
    for T in (1, 3, 16):
        lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, quant, seed=4, numpy_blob=True)
        x = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(T), device="cuda")
        res = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(T + 100), device="cuda")
        lg = synth.uniform_logits(T, E, 7, tau=1.0)
        sc.set_logits_override(lg)
        out = sc.decode(layer, x, res)
        o_out, _, _ = oracle_layer(blob_np, meta, lay, K, x.cpu().numpy(), res.cpu().numpy(), logits=lg.cpu().numpy())
        assert rel_l2(out.cpu().numpy() - res.cpu().numpy(), o_out - res.cpu().numpy()) < TOL_REL_L2


def test_decode_fused_norm(cuda_lib):
    H, I, E, K, T = 2048, 768, 128, 8, 2
    lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, 1, seed=6)
    g = torch.Generator("cuda").manual_seed(8)
    x = torch.randn((T, H), generator=g, device="cuda") * 3
    gamma = 1 + 0.01 * torch.randn(H, generator=g, device="cuda")
    normed = torch.empty_like(x)
    out = sc.decode_fused_norm(layer, x, gamma, 1e-6, normed)
    r = sc.get_routing(T)
    o_normed = oracle.rmsnorm(x.cpu().numpy(), gamma.cpu().numpy(), 1e-6)
    np.testing.assert_allclose(normed.cpu().numpy(), o_normed, rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(moe.rmsnorm(x, gamma, 1e-6).cpu().numpy(), o_normed, rtol=2e-6, atol=1e-7)
    o_out, _, _ = oracle.moe_layer(blob_np, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs, 1,
                                   H, I, E, K, o_normed, x.cpu().numpy(), ids=r["ids"], weights=r["weights"], threads=8)
    assert rel_l2(out.cpu().numpy() - x.cpu().numpy(), o_out - x.cpu().numpy()) < TOL_REL_L2


def test_stack_decode_matches_layer_by_layer(cuda_lib):
    H, I, E, K, T, L = 512, 256, 16, 4, 1, 3
    sc = moe.allocate_moe_scratch(H, I, E, K)
    lay = synth.LayerLayout(H, I, E, 1)
    blobs = [synth.make_layer_blob(lay, 20 + l) for l in range(L)]
    layers = [sc.prepare_layer(b, lay.meta()) for b in blobs]
    gammas = [torch.ones(H, device="cuda") for _ in range(L)]
    x0 = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(2), device="cuda")
    x = x0.clone()
    sc.stack_decode(layers, gammas, x, 1e-6)
    ref = x0.cpu().numpy().copy()
    meta = lay.meta()
    for l in range(L):
        normed = oracle.rmsnorm(ref, np.ones(H, np.float32), 1e-6)
        ref, _, _ = oracle.moe_layer(blobs[l].cpu().numpy(), 0, meta.expert_gate_offs, meta.expert_up_offs,
                                     meta.expert_down_offs, 1, H, I, E, K, normed, ref)
    assert rel_l2(x.cpu().numpy(), ref) < TOL_REL_L2


def test_argument_validation(cuda_lib):
    sc = moe.allocate_moe_scratch(128, 64, 8, 2)
    lay = synth.LayerLayout(128, 64, 8, 1)
    layer = sc.prepare_layer(synth.make_layer_blob(lay, 1), lay.meta())
    x = torch.zeros((17, 128), device="cuda")
    with pytest.raises(moe.LumenMoeError):
        sc.decode(layer, x, x.clone())          # more than 16 tokens
    y = torch.zeros((1, 128), device="cuda")
    with pytest.raises(moe.LumenMoeError):
        sc.decode(layer, y, y, y)               # output aliases the normed input
    with pytest.raises(moe.LumenMoeError):
        moe.allocate_moe_scratch(100, 64, 8, 2)  # H not a multiple of 32
    with pytest.raises(moe.LumenMoeError):
        moe.allocate_moe_scratch(128, 64, 300, 2)  # E > 256
    bad = lay.meta()
    bad.expert_down_offs = bad.expert_down_offs + np.uint64(10 ** 9)
    with pytest.raises(moe.LumenMoeError):
        sc.prepare_layer(synth.make_layer_blob(lay, 1), bad)  # slice outside the blob


@pytest.mark.parametrize("T", [1, 3])
def test_decode_when_the_raw_logit_ranking_differs_from_the_exact_selection(cuda_lib, T):
    """The fused kernel requests weights for the top-K by raw logit while the exact gating
    runs, and must notice when the exact selection differs: here all but K-1 probabilities
    underflow to 0, so the exact rule (lowest index among equals, cuda/moe.rs:6486-6497)
    takes expert K-1 while the largest remaining raw logit sits at expert 100."""
    H, I, E, K = 2048, 768, 128, 8
    lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, 1, seed=2)
    x = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(9), device="cuda")
    lg = np.full((T, E), -400.0, np.float32) - np.arange(E, dtype=np.float32)[None, :]
    lg[:, : K - 1] = np.linspace(0.0, 1.0, K - 1, dtype=np.float32)[None, :]
    lg[:, 100] = -300.0
    lg_d = torch.from_numpy(lg).cuda()
    sc.set_logits_override(lg_d)
    out = sc.decode(layer, x, x.clone())
    r = sc.get_routing(T)
    sc.set_logits_override(None)
    o_out, o_ids, o_w = oracle_layer(blob_np, meta, lay, K, x.cpu().numpy(), x.cpu().numpy(), logits=lg)
    assert sorted(o_ids[0].tolist()) == list(range(K))  # the exact rule really picks expert K-1, not 100
    assert np.array_equal(r["ids"], o_ids)
    assert np.array_equal(r["weights"].view(np.uint32), o_w.view(np.uint32))
    assert rel_l2(out.cpu().numpy() - x.cpu().numpy(), o_out - x.cpu().numpy()) < TOL_REL_L2


@pytest.mark.parametrize("shape", [(1024, 512, 64, 6), (2048, 1536, 32, 4), (1536, 384, 256, 8), (512, 768, 128, 8),
                                   (512, 256, 256, 16), (768, 256, 64, 16)])
@pytest.mark.parametrize("quant", [1, 0, 2])
@pytest.mark.parametrize("gating", [0, 1])
def test_fused_decode_shape_sweep_real_router(cuda_lib, shape, quant, gating):
    """Mid-size shapes through the persistent kernel with its own router (no logits override):
    the oracle is routed with the ids and weights the GPU chose, whose own exactness is
    covered by the identical-logits tests; ids must be valid and distinct per token."""
    H, I, E, K = shape
    lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, quant, seed=21, gating=gating)
    for T in (1, 2, 4):
        if T * K > 32 and K < 16:
            continue  # K = 16 also walks the three-kernel chain (T * K = 64)
        g = torch.Generator("cuda").manual_seed(100 + T)
        x = torch.randn((T, H), generator=g, device="cuda")
        res = torch.randn((T, H), generator=g, device="cuda")
        out = sc.decode(layer, x, res)
        r = sc.get_routing(T)
        ids = r["ids"]
        assert ids.max() < E and all(len(set(row.tolist())) == K for row in ids)
        o_out, _, _ = oracle.moe_layer(blob_np, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs,
                                       quant, H, I, E, K, x.cpu().numpy(), res.cpu().numpy(), ids=ids,
                                       weights=r["weights"], threads=8)
        assert rel_l2(out.cpu().numpy() - res.cpu().numpy(), o_out - res.cpu().numpy()) < TOL_REL_L2
        # the router itself: logits recomputed on the host select the same set when no near-tie is involved
        w = np.frombuffer(blob_np[: E * H * 4].tobytes(), np.float32).reshape(E, H)
        lg = x.cpu().numpy().astype(np.float64) @ w.T.astype(np.float64)
        for t in range(T):
            order = np.argsort(-lg[t], kind="stable")
            gap = lg[t][order[K - 1]] - lg[t][order[K]]
            if gap > 1e-4:
                assert set(order[:K].tolist()) == set(ids[t].tolist())


# ---------------------------------------------------------------------------
# Q4_0 chain with the streaming gate/up kernel and the int8 down product (2..16 tokens when the
# context is created with LUMEN_MOE_FLAG_DECODE_SPLIT, 4..16 tokens otherwise)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("T", [2, 3, 4, 5, 8, 13, 16])
def test_streaming_chain_every_batch_size(cuda_lib, T):
    """Same logits on both sides: ids, weights and sort tables exact, output within the tolerance;
    and the chain agrees with the fused kernel where both apply."""
    from lumen_b200 import _lib
    H, I, E, K = 2048, 768, 128, 8
    lay = synth.LayerLayout(H, I, E, 1)
    blob = synth.make_layer_blob(lay, 11)
    torch.cuda.synchronize()
    blob_np = blob.cpu().numpy()
    meta = lay.meta()
    g = torch.Generator("cuda").manual_seed(20 + T)
    x = torch.randn((T, H), generator=g, device="cuda")
    res = torch.randn((T, H), generator=g, device="cuda")
    lg = synth.uniform_logits(T, E, 30 + T, tau=0.5)
    outs = {}
    for flags in (0, _lib.FLAG_DECODE_SPLIT):
        sc = moe.allocate_moe_scratch(H, I, E, K, 16, flags=flags)
        layer = sc.prepare_layer(blob, meta)
        sc.set_logits_override(lg)
        outs[flags] = sc.decode(layer, x, res).clone()
        r = sc.get_routing(T)
        o_out, o_ids, o_w = oracle_layer(blob_np, meta, lay, K, x.cpu().numpy(), res.cpu().numpy(), logits=lg.cpu().numpy())
        assert np.array_equal(r["ids"], o_ids)
        assert np.array_equal(r["weights"].view(np.uint32), o_w.view(np.uint32))
        _, _, d2c, bounds = oracle.counting_sort(o_ids, E)
        assert np.array_equal(r["dst_to_col"], d2c) and np.array_equal(r["expert_bounds"], bounds)
        assert rel_l2(outs[flags].cpu().numpy() - res.cpu().numpy(), o_out - res.cpu().numpy()) < TOL_REL_L2
        layer.close()
        sc.close()
    a, b = outs[0] - res, outs[_lib.FLAG_DECODE_SPLIT] - res
    assert ((a - b).norm() / a.norm()).item() < 1e-4  # two-term int8 against hi+lo f16 activations in the down product


@pytest.mark.parametrize("K", [8, 16])
def test_streaming_chain_experts_with_many_columns(cuda_lib, K):
    """Every token selects the same K experts: each of them has 16 columns (four column groups in
    both expert kernels), all the others none."""
    H, I, E, T = 512, 256, 32, 16
    lay, meta, blob_np, sc, layer = make_layer(H, I, E, K, 1, seed=9)
    g = torch.Generator("cuda").manual_seed(2)
    x = torch.randn((T, H), generator=g, device="cuda")
    res = torch.randn((T, H), generator=g, device="cuda")
    lg = torch.full((T, E), -4.0, device="cuda")
    lg[:, 3:3 + K] = torch.linspace(1.0, 2.0, K, device="cuda")[None, :]
    sc.set_logits_override(lg)
    out = sc.decode(layer, x, res)
    r = sc.get_routing(T)
    assert all(set(row.tolist()) == set(range(3, 3 + K)) for row in r["ids"])
    assert np.diff(r["expert_bounds"]).max() == T
    o_out, o_ids, _ = oracle_layer(blob_np, meta, lay, K, x.cpu().numpy(), res.cpu().numpy(), logits=lg.cpu().numpy())
    assert np.array_equal(r["ids"], o_ids)
    assert rel_l2(out.cpu().numpy() - res.cpu().numpy(), o_out - res.cpu().numpy()) < TOL_REL_L2
    # determinism
    out2 = sc.decode(layer, x, res)
    assert torch.equal(out, out2)
