"""Oracle against the committed golden vectors (tests/golden/, made by
make_golden.py from the reference's own scalar kernels compiled for the host)."""
from pathlib import Path

import numpy as np
import pytest

G = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
def test_oracle_layer_matches_reference_kernels(orc, name):
    from lumen_b200.synth import LayerLayout
    d = np.load(G / f"moe_small_{name}.npz")
    H, I, E, K, T, quant = (int(v) for v in d["dims"])
    meta = LayerLayout(H, I, E, quant).meta()
    out, ids, wts = orc.moe_layer(d["blob"], 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs,
                                  quant, H, I, E, K, d["x"], d["x"])
    assert np.array_equal(ids, d["ids"])
    assert np.array_equal(wts, d["weights"])
    rel = np.linalg.norm(out - d["ref_out"]) / np.linalg.norm(d["ref_out"])
    assert rel < 1e-5  # summation order differs between the CPU reference and its scalar kernels


def test_oracle_topk_matches_golden(orc):
    d = np.load(G / "router_topk.npz")
    for gating, tag in ((0, "softmax"), (1, "sigmoid")):
        ids, w = orc.topk_from_logits(d["logits"], 8, gating)
        assert np.array_equal(ids, d[f"ids_{tag}"])
        assert np.array_equal(w, d[f"w_{tag}"])


def test_reference_scalar_kernels_agree_when_present(orc):
    """Only where the reference tree is mounted: rebuild oracle/_ref and compare."""
    import ctypes
    orc.build(ref=True)
    if not orc.REF_PATH.exists():
        pytest.skip("reference sources not present")
    ref = ctypes.CDLL(str(orc.REF_PATH))
    rng = np.random.default_rng(5)
    H, I = 256, 96
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    for quant in (0, 1):
        g = orc.quantize((rng.standard_normal(I * H) * 0.02).astype(np.float32), quant)
        u = orc.quantize((rng.standard_normal(I * H) * 0.02).astype(np.float32), quant)
        blob = np.concatenate([g, u])
        x = rng.standard_normal(H).astype(np.float32)
        sw = np.zeros(I, np.float32)
        ref.ref_gate_up_swiglu(p(x), p(blob), ctypes.c_ulonglong(0), ctypes.c_ulonglong(g.size), p(sw), H, I, quant)
        mine = orc.swiglu(orc.matvec(g, x, I, H, quant), orc.matvec(u, x, I, H, quant))
        assert np.linalg.norm(sw - mine) / np.linalg.norm(mine) < 1e-5
