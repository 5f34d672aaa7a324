"""Generates the committed golden vectors under tests/golden/.

Run where the reference tree is available (REFERENCE_ROOT; by default a checkout named
`reference` next to this repository): the expert outputs stored here come from the REFERENCE'S OWN
scalar kernels (cuda/shaders/moe_expert.cu, moe_expert_q4_0.cu, moe_accum.cu)
compiled for the host by `make -C oracle ref`; routing comes from the oracle's
restatement of cpu_router_softmax (the reference keeps that function inside a
Rust test module, which cannot be built without cargo).

    python tests/golden/make_golden.py
"""
import ctypes
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle  # noqa: E402
from lumen_b200.synth import LayerLayout, make_layer_blob_numpy  # noqa: E402

HERE = Path(__file__).resolve().parent


def ref_layer(ref, blob, meta, quant, H, I, K, x, ids, wts):
    T = x.shape[0]
    out = np.zeros((T, H), np.float32)
    sw_all = np.zeros((T, K, I), np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    for t in range(T):
        douts = np.zeros((K, H), np.float32)
        for k in range(K):
            e = int(ids[t, k])
            sw = np.zeros(I, np.float32)
            ref.ref_gate_up_swiglu(p(x[t]), p(blob), ctypes.c_ulonglong(int(meta.expert_gate_offs[e])),
                                   ctypes.c_ulonglong(int(meta.expert_up_offs[e])), p(sw), H, I, quant)
            ref.ref_down(p(sw), p(blob), ctypes.c_ulonglong(int(meta.expert_down_offs[e])), p(douts[k]), H, I, quant)
            sw_all[t, k] = sw
        ref.ref_accum_option_a(p(out[t]), p(x[t]), p(douts), p(wts[t]), H, K)
    return out, sw_all


def main():
    oracle.build(ref=True)
    if not oracle.REF_PATH.exists():
        raise SystemExit("oracle/_ref was not built (reference tree absent)")
    ref = ctypes.CDLL(str(oracle.REF_PATH))
    H, I, E, K, T = 128, 64, 8, 2, 3
    for quant, name in ((oracle.Q4_0, "q4_0"), (oracle.Q8_0, "q8_0")):
        lay = LayerLayout(H, I, E, quant)
        blob = make_layer_blob_numpy(lay, 11, oracle.quantize)
        meta = lay.meta()
        rng = np.random.default_rng(12)
        x = rng.standard_normal((T, H)).astype(np.float32)
        o_out, ids, wts = oracle.moe_layer(blob, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs,
                                           quant, H, I, E, K, x, x)
        r_out, r_sw = ref_layer(ref, blob, meta, quant, H, I, K, x, ids, wts)
        rel = np.linalg.norm(r_out - o_out) / np.linalg.norm(r_out)
        print(name, "oracle vs reference scalar kernels rel-L2", rel)
        assert rel < 1e-5
        np.savez_compressed(HERE / f"moe_small_{name}.npz", blob=blob, x=x, ids=ids, weights=wts, ref_out=r_out,
                            ref_swiglu=r_sw, dims=np.array([H, I, E, K, T, quant], np.int32))
    # router vectors: logits -> ids / weights (softmax and sigmoid gating)
    rng = np.random.default_rng(21)
    E, K = 128, 8
    logits = np.concatenate([rng.standard_normal((24, E)).astype(np.float32),
                             (rng.standard_normal((24, E)) * 0.02).astype(np.float32),
                             np.zeros((1, E), np.float32),
                             np.round(rng.standard_normal((8, E)) * 2).astype(np.float32) / 4])  # many exact ties
    ids0, w0 = oracle.topk_from_logits(logits, K, 0)
    ids1, w1 = oracle.topk_from_logits(logits, K, 1)
    np.savez_compressed(HERE / "router_topk.npz", logits=logits, ids_softmax=ids0, w_softmax=w0, ids_sigmoid=ids1,
                        w_sigmoid=w1)
    print("wrote", sorted(q.name for q in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
