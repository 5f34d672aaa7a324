"""Synthetic MoE layer blobs with the layout the reference's converter writes
(crates/lumen-convert/src/arch/qwen35_moe.rs:257-260,512-551):
[router f32 [E,H]] [expert 0: gate | up | down] ... [expert E-1], each matrix a run
of raw GGML blocks (rows contiguous along the input dimension).

Weights are drawn on the GPU with a seeded torch generator and quantised on the
GPU by the library's restatement of the reference quantisers, so that a 340 MB
layer takes milliseconds. The quantised BYTES are what both the CUDA path and the
CPU oracle consume.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import moe
from ._lib import BF16, Q4_0, Q8_0


def row_bytes(in_dim: int, quant: int) -> int:
    return {Q8_0: in_dim // 32 * 34, Q4_0: in_dim // 32 * 18, BF16: in_dim * 2}[quant]


@dataclass
class LayerLayout:
    H: int
    I: int
    E: int
    quant: int

    @property
    def router_bytes(self) -> int:
        return self.E * self.H * 4

    @property
    def gate_bytes(self) -> int:
        return self.I * row_bytes(self.H, self.quant)

    @property
    def down_bytes(self) -> int:
        return self.H * row_bytes(self.I, self.quant)

    @property
    def expert_bytes(self) -> int:
        return 2 * self.gate_bytes + self.down_bytes

    @property
    def blob_bytes(self) -> int:
        return self.router_bytes + self.E * self.expert_bytes

    def meta(self) -> moe.MoeMeta:
        base = self.router_bytes
        experts = []
        for e in range(self.E):
            o = base + e * self.expert_bytes
            experts.append({"gate": (o, self.quant), "up": (o + self.gate_bytes, self.quant),
                            "down": (o + 2 * self.gate_bytes, self.quant)})
        return moe.build_moe_meta(0, experts)


def make_layer_blob(layout: LayerLayout, seed: int, device="cuda", std: float = 0.02,
                    router_std: float = 0.02) -> torch.Tensor:
    """Expert weights N(0,std) then router N(0,router_std) from one seeded stream
    (experts first, expert-major, gate/up/down; then the router)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    blob = torch.empty(layout.blob_bytes, dtype=torch.uint8, device=device)
    off = layout.router_bytes
    n_gu, n_dn = layout.I * layout.H, layout.H * layout.I
    for e in range(layout.E):
        w = torch.randn(2 * n_gu + n_dn, generator=g, device=device, dtype=torch.float32) * std
        for n, nb in ((n_gu, layout.gate_bytes), (n_gu, layout.gate_bytes), (n_dn, layout.down_bytes)):
            blob[off:off + nb] = moe.quantize(w[:n].contiguous(), layout.quant)
            w = w[n:]
            off += nb
    r = torch.randn(layout.E * layout.H, generator=g, device=device, dtype=torch.float32) * router_std
    blob[:layout.router_bytes] = r.view(torch.uint8)
    return blob


def make_layer_blob_numpy(layout: LayerLayout, seed: int, quantize_fn, std: float = 0.02,
                          router_std: float = 0.02) -> np.ndarray:
    """CPU variant for small shapes; quantize_fn(w_f32, quant) -> uint8 array."""
    rng = np.random.default_rng(seed)
    blob = np.zeros(layout.blob_bytes, dtype=np.uint8)
    off = layout.router_bytes
    for _ in range(layout.E):
        for n, nb in ((layout.I * layout.H, layout.gate_bytes), (layout.I * layout.H, layout.gate_bytes),
                      (layout.H * layout.I, layout.down_bytes)):
            w = (rng.standard_normal(n) * std).astype(np.float32)
            blob[off:off + nb] = quantize_fn(w, layout.quant)
            off += nb
    r = (rng.standard_normal(layout.E * layout.H) * router_std).astype(np.float32)
    blob[:layout.router_bytes] = r.view(np.uint8)
    return blob


def zipf_logits(T: int, E: int, seed: int, s: float = 1.1, device="cuda") -> torch.Tensor:
    """Router logits whose top-k follows a Zipf(s) expert popularity: ln p_e plus
    Gumbel noise (top-k of that samples k experts without replacement with
    probabilities proportional to p)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    perm = torch.randperm(E, generator=g, device=device)
    p = (torch.arange(1, E + 1, device=device, dtype=torch.float64) ** (-s))
    logp = torch.log(p / p.sum())[perm.argsort()].to(torch.float32)
    u = torch.rand((T, E), generator=g, device=device, dtype=torch.float32).clamp_(1e-7, 1 - 1e-7)
    gumbel = -torch.log(-torch.log(u))
    return (logp[None, :] + gumbel).contiguous()


def uniform_logits(T: int, E: int, seed: int, tau: float = 0.05, device="cuda") -> torch.Tensor:
    """Logits N(0, tau^2): near-uniform expert selection."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn((T, E), generator=g, device=device, dtype=torch.float32) * tau).contiguous()
