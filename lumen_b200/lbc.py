"""LBC checkpoint ingestion for the MoE layer path.

The reference's backend uploads a MoE layer's blob byte for byte
(cuda/gpu_buffers.rs:1404-1409) and takes the operator's offsets from the layer's entry
in the file's index (build_moe_meta, cuda/moe.rs:223-262; entry format
crates/lumen-format/src/reader.rs:522-760). `LbcIndex` reads that index through the
library (`lumen_lbc_read_header`, `lumen_lbc_read_moe_layer`) and returns, per layer,
the `MoeMeta` that `MoeScratch.prepare_layer` takes, the byte range of the layer blob in
the file, and the slices of the shared expert and of the FFN norm.

Only the header and the index are parsed; payload bytes are the caller's to read (mmap or
file reads) and to upload.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Tuple, Union

import numpy as np

from . import _lib
from .moe import MoeMeta

Slice = Optional[Tuple[int, int, int]]  # (offset in the layer blob, length, LBC scheme tag)


def _slice(s: _lib.LbcSlice) -> Slice:
    return (int(s.offset), int(s.length), int(s.quant)) if s.present else None


@dataclass
class LbcMoeLayer:
    layer: int
    layer_offset_bytes: int   # absolute position of the layer blob in the file
    layer_length_bytes: int
    meta: Optional[MoeMeta]   # None for a dense layer (build_moe_meta returns None, cuda/moe.rs:226-231)
    inter_dim: Optional[int]  # I, from the byte length of expert 0's gate slice
    router_weight: Slice
    ffn_norm: Slice
    shared_expert_gate: Slice
    shared_expert_up: Slice
    shared_expert_down: Slice
    ffn_gate_inp_shexp: Slice
    layer_type: Optional[int]

    def shared_expert_meta(self, hidden_dim: int):
        """(MoeMeta, inter_dim, gating_mode) of the always-on shared expert as a one-expert
        layer (the form lumen_moe_shared_expert_decode / _prefill take), or None when the
        layer has none. The gate vector ffn_gate_inp_shexp stands where the router does;
        without it the expert's weight is 1 (cuda/moe.rs:5455-5520)."""
        g, u, d = self.shared_expert_gate, self.shared_expert_up, self.shared_expert_down
        if g is None or u is None or d is None:
            return None
        gq = _lib.lib().lumen_lbc_quant_to_moe(g[2])
        dq = _lib.lib().lumen_lbc_quant_to_moe(d[2])
        if gq < 0 or dq < 0:
            raise _lib.LumenMoeError(_lib.UNSUPPORTED, f"layer {self.layer}: shared expert scheme tags {g[2]}/{d[2]} "
                                                       "have no kernel (Q8_0, Q4_0, BF16 only)")
        gate_vec = self.ffn_gate_inp_shexp
        one = lambda v: np.array([v], dtype=np.uint64)
        meta = MoeMeta(gate_vec[0] if gate_vec else 0, one(g[0]), one(u[0]), one(d[0]), gq, dq)
        return meta, g[1] // _row_bytes(gq, hidden_dim), _lib.SIGMOID_GATE if gate_vec else _lib.UNIT_WEIGHT


def _row_bytes(quant: int, cols: int) -> int:
    return {_lib.Q8_0: cols // 32 * 34, _lib.Q4_0: cols // 32 * 18, _lib.BF16: cols * 2}[quant]


class LbcIndex:
    """Header + layer index of an LBC file (path, bytes or any buffer)."""

    def __init__(self, source: Union[str, Path, bytes, bytearray, memoryview, np.ndarray]):
        if isinstance(source, (str, Path)):
            with open(source, "rb") as f:
                head = f.read(256)
                hdr = self._header(head)
                # the index ends where the payload starts (writer.rs:57-75)
                f.seek(0)
                data = f.read(int(hdr.payload_offset) if hdr.payload_offset else -1)
        else:
            data = bytes(source)
        self._buf = ctypes.create_string_buffer(data, len(data))
        self._n = len(data)
        self.header = self._header(data)

    @staticmethod
    def _header(data: bytes) -> _lib.LbcHeader:
        h = _lib.LbcHeader()
        buf = ctypes.create_string_buffer(data, len(data))
        _lib.check(_lib.lib().lumen_lbc_read_header(buf, len(data), ctypes.byref(h)))
        return h

    def read_layer_blob(self, source, layer: "LbcMoeLayer") -> np.ndarray:
        """The layer's blob bytes (what the backend uploads unchanged, cuda/gpu_buffers.rs:1404-1409)
        from the file (path) or from a buffer holding the whole file."""
        lo, n = layer.layer_offset_bytes, layer.layer_length_bytes
        if isinstance(source, (str, Path)):
            with open(source, "rb") as f:
                f.seek(lo)
                data = f.read(n)
        else:
            data = bytes(memoryview(source)[lo: lo + n])
        if len(data) != n:
            raise _lib.LumenMoeError(_lib.INVALID_ARG, f"layer {layer.layer}: the file ends inside the layer blob")
        return np.frombuffer(data, dtype=np.uint8)

    @property
    def num_layers(self) -> int:
        return int(self.header.num_layers)

    def config(self) -> dict:
        """The operator's dimensions as the file's hyperparameters record them."""
        h = self.header
        return {"hidden_dim": int(h.hidden_dim), "num_experts": int(h.num_experts),
                "top_k": int(h.num_active_experts), "norm_eps": float(h.norm_eps)}

    def moe_layer(self, layer: int) -> LbcMoeLayer:
        out = _lib.LbcMoeLayer()
        cap = max(int(self.header.num_experts), 256)
        offs = [np.zeros(cap, np.uint64) for _ in range(3)]
        _lib.check(_lib.lib().lumen_lbc_read_moe_layer(self._buf, self._n, layer, ctypes.byref(out),
                                                       *(o.ctypes.data for o in offs), cap))
        meta = inter = None
        if out.is_moe:
            E = int(out.num_experts)
            gq = _lib.lib().lumen_lbc_quant_to_moe(out.expert_gate_quant)
            dq = _lib.lib().lumen_lbc_quant_to_moe(out.expert_down_quant)
            if gq < 0 or dq < 0:
                raise _lib.LumenMoeError(_lib.UNSUPPORTED,
                                         f"layer {layer}: expert scheme tags {out.expert_gate_quant}/"
                                         f"{out.expert_down_quant} have no kernel (Q8_0, Q4_0, BF16 only)")
            meta = MoeMeta(int(out.router_weight.offset), offs[0][:E].copy(), offs[1][:E].copy(), offs[2][:E].copy(),
                           gq, dq)
            inter = int(out.expert_gate_bytes) // _row_bytes(gq, int(self.header.hidden_dim))
        return LbcMoeLayer(layer, int(out.layer_offset_bytes), int(out.layer_length_bytes), meta, inter,
                           _slice(out.router_weight), _slice(out.ffn_norm), _slice(out.shared_expert_gate),
                           _slice(out.shared_expert_up), _slice(out.shared_expert_down),
                           _slice(out.ffn_gate_inp_shexp), int(out.layer_type) if out.has_layer_type else None)
