"""The always-on shared expert (cuda/moe.rs:5455-5520, 2788): a one-expert context whose
weight is sigmoid(dot(ffn_gate_inp_shexp, x)) (or 1), accumulated into the routed result.

The layer blob here is [routed blob][shared blob] with the shared slices addressed by
offsets, as the converter lays them out (lumen-convert/src/arch/qwen35_moe.rs:257-260)."""
import numpy as np
import pytest
import torch

from lumen_b200 import moe, synth
from oracle import oracle
from tests.gpu_util import TOL_REL_L2, rel_l2

pytestmark = pytest.mark.gpu


def _combined(H, I, I_sh, E, quant, seed):
    routed = synth.LayerLayout(H, I, E, quant)
    shared = synth.LayerLayout(H, I_sh, 1, quant)
    b0 = synth.make_layer_blob(routed, seed)
    b1 = synth.make_layer_blob(shared, seed + 1)
    blob = torch.cat([b0, b1]).contiguous()
    torch.cuda.synchronize()
    base = b0.numel()
    m0, m1 = routed.meta(), shared.meta()
    sh_meta = moe.MoeMeta(base + m1.router_weight_off, m1.expert_gate_offs + base, m1.expert_up_offs + base,
                          m1.expert_down_offs + base, quant, quant)
    return routed, shared, blob, m0, sh_meta


def _oracle_shared(blob_np, sh_meta, quant, H, I_sh, x, acc_in, gating):
    # one expert, top-1: the oracle's layer function with the gate vector as its 1 x H router
    return oracle.moe_layer(blob_np, int(sh_meta.router_weight_off), sh_meta.expert_gate_offs, sh_meta.expert_up_offs,
                            sh_meta.expert_down_offs, quant, H, I_sh, 1, 1, x, acc_in, gating=gating,
                            threads=oracle.hardware_threads())[0]


@pytest.mark.parametrize("quant", [moe.Q4_0, moe.Q8_0])
@pytest.mark.parametrize("gating", [moe.SIGMOID_GATE, moe.UNIT_WEIGHT])
@pytest.mark.parametrize("T", [1, 3, 7])
def test_shared_expert_decode_after_routed(quant, gating, T):
    H, I, I_sh, E, K = 512, 256, 384, 16, 4
    routed, shared, blob, m0, sh_meta = _combined(H, I, I_sh, E, quant, seed=11)
    blob_np = blob.cpu().numpy()
    sc = moe.allocate_moe_scratch(H, I, E, K, 16)
    layer = sc.prepare_layer(blob, m0)
    sc_sh = moe.allocate_moe_scratch(H, I_sh, 1, 1, 16, gating)
    layer_sh = sc_sh.prepare_layer(blob, sh_meta)
    g = torch.Generator(device="cuda").manual_seed(T)
    x = torch.randn((T, H), generator=g, device="cuda")
    res = torch.randn((T, H), generator=g, device="cuda")
    out = sc.decode(layer, x, res)
    routed_out = out.clone()
    sc_sh.shared_expert_decode(layer_sh, x, out)
    torch.cuda.synchronize()
    want = _oracle_shared(blob_np, sh_meta, quant, H, I_sh, x.cpu().numpy(), routed_out.cpu().numpy(), gating)
    got = out.cpu().numpy()
    assert rel_l2(got - routed_out.cpu().numpy(), want - routed_out.cpu().numpy()) < TOL_REL_L2
    rt = sc_sh.get_routing(T)
    assert (rt["ids"] == 0).all()
    if gating == moe.UNIT_WEIGHT:
        assert (rt["weights"] == 1.0).all()
    else:
        lg = x.cpu().numpy() @ np.frombuffer(blob_np[int(sh_meta.router_weight_off):][:H * 4].tobytes(), np.float32)
        np.testing.assert_allclose(rt["weights"][:, 0], 1.0 / (1.0 + np.exp(-lg.astype(np.float64))), rtol=2e-5)


@pytest.mark.parametrize("quant", [moe.Q4_0])
@pytest.mark.parametrize("T", [40, 300])
def test_shared_expert_prefill(quant, T):
    H, I_sh = 512, 384
    shared = synth.LayerLayout(H, I_sh, 1, quant)
    blob = synth.make_layer_blob(shared, 5)
    torch.cuda.synchronize()
    blob_np = blob.cpu().numpy()
    meta = shared.meta()
    sc_sh = moe.allocate_moe_scratch(H, I_sh, 1, 1, T, moe.SIGMOID_GATE)
    layer_sh = sc_sh.prepare_layer(blob, meta)
    g = torch.Generator(device="cuda").manual_seed(T)
    x = torch.randn((T, H), generator=g, device="cuda")
    acc = torch.randn((T, H), generator=g, device="cuda")
    acc0 = acc.clone()
    sc_sh.shared_expert_prefill(layer_sh, x, acc)
    torch.cuda.synchronize()
    want = _oracle_shared(blob_np, meta, quant, H, I_sh, x.cpu().numpy(), acc0.cpu().numpy(), moe.SIGMOID_GATE)
    assert rel_l2(acc.cpu().numpy() - acc0.cpu().numpy(), want - acc0.cpu().numpy()) < TOL_REL_L2


def test_shared_expert_entry_point_rejects_routed_context():
    sc = moe.allocate_moe_scratch(256, 128, 8, 2, 16)
    lay = synth.LayerLayout(256, 128, 8, moe.Q4_0)
    layer = sc.prepare_layer(synth.make_layer_blob(lay, 0), lay.meta())
    x = torch.zeros((1, 256), device="cuda")
    with pytest.raises(moe.LumenMoeError):
        sc.shared_expert_decode(layer, x, torch.zeros_like(x))
