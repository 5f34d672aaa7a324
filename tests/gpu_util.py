"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from lumen_b200 import moe, synth
from oracle import oracle

TOL_REL_L2 = 1e-3  # layer output vs CPU reference, relative L2 (f32 accumulation)


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def make_layer(H, I, E, K, quant, seed=0, max_tokens=16, gating=0, numpy_blob=False):
    lay = synth.LayerLayout(H, I, E, quant)
    if numpy_blob:
        blob_np = synth.make_layer_blob_numpy(lay, seed, oracle.quantize)
        blob = torch.from_numpy(blob_np).cuda()
    else:
        blob = synth.make_layer_blob(lay, seed)
        torch.cuda.synchronize()
        blob_np = blob.cpu().numpy()
    meta = lay.meta()
    scratch = moe.allocate_moe_scratch(H, I, E, K, max_tokens, gating)
    layer = scratch.prepare_layer(blob, meta)
    return lay, meta, blob_np, scratch, layer


def oracle_layer(blob_np, meta, lay, K, x, residual, logits=None, gating=0, threads=None):
    threads = threads or oracle.hardware_threads()
    return oracle.moe_layer(blob_np, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs, lay.quant,
                            lay.H, lay.I, lay.E, K, x, residual, gating=gating, logits=logits, threads=threads)
