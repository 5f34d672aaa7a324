"""A MoE layer read from an LBC file (header + index parsed by the library, layer blob
uploaded byte for byte as cuda/gpu_buffers.rs:1404-1409 does) gives exactly the result of
the same weights prepared from hand-derived offsets."""
import numpy as np
import pytest
import torch

from lumen_b200 import lbc, moe, synth
from oracle import lbc_writer as W
from oracle import oracle
from tests.gpu_util import TOL_REL_L2, rel_l2

pytestmark = pytest.mark.gpu

TAG = {moe.Q4_0: W.Q4_0, moe.Q8_0: W.Q8_0, moe.BF16: W.BF16}


@pytest.mark.parametrize("quant", [moe.Q4_0, moe.Q8_0, moe.BF16])
def test_layer_from_lbc_file(cuda_lib, quant):
    H, I, I_sh, E, K, T = 512, 256, 384, 16, 4, 3
    routed, shared = synth.LayerLayout(H, I, E, quant), synth.LayerLayout(H, I_sh, 1, quant)
    b_routed, b_shared = synth.make_layer_blob(routed, 31), synth.make_layer_blob(shared, 32)
    g = torch.Generator(device="cuda").manual_seed(7)
    norm_w = (1.0 + 0.1 * torch.randn(H, generator=g, device="cuda")).contiguous()
    torch.cuda.synchronize()
    # layer blob of the file: [attention bytes][ffn_norm][router + experts][gate vector + shared expert]
    attn = bytes(range(250)) * 4
    p_norm = len(attn)
    p_routed = p_norm + H * 4
    p_shared = p_routed + b_routed.numel()
    blob = attn + norm_w.cpu().numpy().tobytes() + b_routed.cpu().numpy().tobytes() + b_shared.cpu().numpy().tobytes()
    m0, m1 = routed.meta(), shared.meta()
    q = TAG[quant]
    sl = lambda off, n, tag=q: (int(off), int(n), tag)
    L = W.Layer(wq=sl(0, 400), wk=sl(400, 200), wv=sl(600, 200), wo=sl(800, 200), attn_norm=sl(0, 0, W.F32),
                ffn_norm=sl(p_norm, H * 4, W.F32), router_weight=sl(p_routed, E * H * 4, W.F32),
                experts=[(sl(p_routed + m0.expert_gate_offs[e], routed.gate_bytes),
                          sl(p_routed + m0.expert_up_offs[e], routed.gate_bytes),
                          sl(p_routed + m0.expert_down_offs[e], routed.down_bytes)) for e in range(E)],
                ext={0: sl(p_shared + m1.expert_gate_offs[0], shared.gate_bytes),
                     1: sl(p_shared + m1.expert_up_offs[0], shared.gate_bytes),
                     2: sl(p_shared + m1.expert_down_offs[0], shared.down_bytes),
                     15: sl(p_shared, H * 4, W.F32)}, layer_type=0)
    dense = W.Layer(w_gate=sl(0, 64), w_up=sl(64, 64), w_down=sl(128, 64))
    model = W.Model(num_layers=2, hidden_dim=H, intermediate_dim=I, num_experts=E, num_active_experts=K,
                    norm_eps=1e-6, primary_quant=q)
    data = W.write_lbc(model, [dense, L], [bytes(192), blob])

    idx = lbc.LbcIndex(data)
    cfg = idx.config()
    assert (cfg["hidden_dim"], cfg["num_experts"], cfg["top_k"]) == (H, E, K)
    assert idx.moe_layer(0).meta is None
    info = idx.moe_layer(1)
    assert info.inter_dim == I
    file_blob = torch.frombuffer(bytearray(data[info.layer_offset_bytes: info.layer_offset_bytes + info.layer_length_bytes]),
                                 dtype=torch.uint8).cuda()
    sc = moe.allocate_moe_scratch(H, info.inter_dim, cfg["num_experts"], cfg["top_k"], 16)
    layer = sc.prepare_layer(file_blob, info.meta)
    sh_meta, i_sh, sh_gating = info.shared_expert_meta(H)
    assert (i_sh, sh_gating) == (I_sh, moe.SIGMOID_GATE)
    sc_sh = moe.allocate_moe_scratch(H, i_sh, 1, 1, 16, sh_gating)
    layer_sh = sc_sh.prepare_layer(file_blob, sh_meta)
    no, nl, _ = info.ffn_norm
    norm_from_file = file_blob[no: no + nl].view(torch.float32)
    assert torch.equal(norm_from_file, norm_w)

    # the same weights from the stand-alone blobs and their own offsets
    sc2 = moe.allocate_moe_scratch(H, I, E, K, 16)
    layer2 = sc2.prepare_layer(b_routed, m0)
    sc2_sh = moe.allocate_moe_scratch(H, I_sh, 1, 1, 16, moe.SIGMOID_GATE)
    layer2_sh = sc2_sh.prepare_layer(b_shared, m1)

    x = torch.randn((T, H), generator=g, device="cuda")
    res = torch.randn((T, H), generator=g, device="cuda")
    out = sc.decode(layer, x, res)
    sc_sh.shared_expert_decode(layer_sh, x, out)
    out2 = sc2.decode(layer2, x, res)
    routed_only = out2.clone()
    sc2_sh.shared_expert_decode(layer2_sh, x, out2)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    r = sc.get_routing(T)
    want, _, _ = oracle.moe_layer(np.frombuffer(blob, np.uint8), int(info.meta.router_weight_off),
                                  info.meta.expert_gate_offs, info.meta.expert_up_offs, info.meta.expert_down_offs,
                                  quant, H, I, E, K, x.cpu().numpy(), res.cpu().numpy(), ids=r["ids"],
                                  weights=r["weights"], threads=8)
    assert rel_l2(routed_only.cpu().numpy() - res.cpu().numpy(), want - res.cpu().numpy()) < TOL_REL_L2
    # prefill of the same layer from the file
    Tp = 200
    xp = torch.randn((Tp, H), generator=g, device="cuda").to(torch.bfloat16)
    rp = torch.randn((Tp, H), generator=g, device="cuda")
    assert torch.equal(sc.prefill(layer, xp, rp), sc2.prefill(layer2, xp, rp))
