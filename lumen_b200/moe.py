"""Host-side mirror of the reference's MoE operator interface
(crates/lumen-runtime/src/cuda/moe.rs) on top of the C ABI (include/lumen_moe.h).

PyTorch is used for device memory and streams only; every computation is a call
into liblumen_moe_b200.so. Names follow the reference:

    allocate_moe_scratch(...)            -> MoeScratch      (cuda/moe.rs:968)
    build_moe_meta(...)                  -> MoeMeta         (cuda/moe.rs:223)
    MoeScratch.prepare_layer(...)        -> MoeLayer        (build_batched_offsets :272 + build_repacked_down :337)
    encode_moe_ffn_decode(...)                              (cuda/moe.rs:1119)
    encode_moe_ffn_decode_fused_norm(...)                   (cuda/moe.rs:3184)
    encode_moe_ffn_prefill_grouped(...)                     (cuda/moe.rs:1900)
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import (ACT_BF16, ACT_F16, ACT_F32, BF16, Q4_0, Q8_0, SIGMOID_GATE, SIGMOID_RENORM, SOFTMAX_RENORM, UNIT_WEIGHT,
                   LumenMoeError, MoeConfig,
                   check)

__all__ = ["MoeMeta", "MoeScratch", "MoeLayer", "allocate_moe_scratch", "build_moe_meta", "encode_moe_ffn_decode",
           "encode_moe_ffn_decode_fused_norm", "encode_moe_ffn_prefill_grouped", "LumenMoeError", "Q8_0", "Q4_0",
           "BF16", "SOFTMAX_RENORM", "SIGMOID_RENORM", "SIGMOID_GATE", "UNIT_WEIGHT"]


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise LumenMoeError(_lib.INVALID_ARG, f"{name} must be a CUDA tensor (no CPU path)")
    if t.dtype != dtype or not t.is_contiguous():
        raise LumenMoeError(_lib.INVALID_ARG, f"{name} must be contiguous {dtype}")
    return t


@dataclass
class MoeMeta:
    """CudaMoeMeta (cuda/moe.rs:39-59): byte offsets inside the layer blob."""
    router_weight_off: int
    expert_gate_offs: np.ndarray
    expert_up_offs: np.ndarray
    expert_down_offs: np.ndarray
    expert_gate_quant: int
    expert_down_quant: int


def build_moe_meta(router_weight_off: Optional[int], experts: Optional[Sequence[dict]]) -> Optional[MoeMeta]:
    """build_moe_meta (cuda/moe.rs:223-260). `experts` is a list of
    {"gate": (offset, quant), "up": (...), "down": (...)}; returns None when the
    layer has no router or no experts (not an MoE layer), like the reference."""
    if router_weight_off is None or not experts:
        return None
    return MoeMeta(int(router_weight_off),
                   np.array([e["gate"][0] for e in experts], dtype=np.uint64),
                   np.array([e["up"][0] for e in experts], dtype=np.uint64),
                   np.array([e["down"][0] for e in experts], dtype=np.uint64),
                   int(experts[0]["gate"][1]), int(experts[0]["down"][1]))


class MoeLayer:
    """Prepared layer: device offset tables + repacked expert planes."""

    def __init__(self, handle: int, blob: torch.Tensor, meta: MoeMeta):
        self._h = handle
        self.blob = blob  # keeps the caller's blob alive: the router weight is read in place
        self.meta = meta

    @property
    def device_bytes(self) -> int:
        return int(_lib.lib().lumen_moe_layer_bytes(self._h))

    def close(self) -> None:
        if self._h:
            _lib.lib().lumen_moe_layer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MoeScratch:
    """CudaMoeScratch (cuda/moe.rs:101-210) behind lumen_moe_ctx."""

    def __init__(self, hidden_dim: int, inter_dim: int, num_experts: int, top_k: int, max_tokens: int = 16,
                 gating_mode: int = SOFTMAX_RENORM, device: int = 0, flags: int = 0):
        self.H, self.I, self.E, self.K = hidden_dim, inter_dim, num_experts, top_k
        self.device = device
        cfg = MoeConfig(hidden_dim, inter_dim, num_experts, top_k, max_tokens, gating_mode, device, flags)
        h = ctypes.c_void_p()
        check(_lib.lib().lumen_moe_create(ctypes.byref(cfg), ctypes.byref(h)))
        self._h = h.value
        self._override = None

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().lumen_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- preload ----------------------------------------------------------
    def prepare_layer(self, blob: torch.Tensor, meta: MoeMeta) -> MoeLayer:
        _need(blob, torch.uint8, "layer blob")
        if meta.expert_gate_quant != meta.expert_down_quant:
            raise LumenMoeError(_lib.UNSUPPORTED, "gate and down quant schemes differ")
        go = np.ascontiguousarray(meta.expert_gate_offs, dtype=np.uint64)
        uo = np.ascontiguousarray(meta.expert_up_offs, dtype=np.uint64)
        do = np.ascontiguousarray(meta.expert_down_offs, dtype=np.uint64)
        if not (len(go) == len(uo) == len(do) == self.E):
            raise LumenMoeError(_lib.INVALID_ARG, "offset tables must have num_experts entries")
        h = ctypes.c_void_p()
        check(_lib.lib().lumen_moe_layer_prepare(self._h, blob.data_ptr(), blob.numel(), meta.router_weight_off,
                                                 go.ctypes.data, uo.ctypes.data, do.ctypes.data,
                                                 meta.expert_gate_quant, _stream(), ctypes.byref(h)))
        return MoeLayer(h.value, blob, meta)

    def prepare_router_only(self, blob: torch.Tensor, router_weight_off: int = 0) -> MoeLayer:
        """Layer usable for route_only only (no expert planes): the replicated router of
        an expert-parallel rank."""
        _need(blob, torch.uint8, "layer blob")
        h = ctypes.c_void_p()
        check(_lib.lib().lumen_moe_layer_prepare(self._h, blob.data_ptr(), blob.numel(), router_weight_off, None,
                                                 None, None, 0, _stream(), ctypes.byref(h)))
        return MoeLayer(h.value, blob, None)

    def ensure_prefill_grouped(self, batch: int) -> None:
        check(_lib.lib().lumen_moe_ensure_prefill(self._h, batch))

    # -- operators --------------------------------------------------------
    def decode(self, layer: MoeLayer, normed_x: torch.Tensor, residual: torch.Tensor,
               output_x: Optional[torch.Tensor] = None) -> torch.Tensor:
        _need(normed_x, torch.float32, "normed_x")
        _need(residual, torch.float32, "residual")
        T = normed_x.numel() // self.H
        if output_x is None:
            output_x = torch.empty_like(residual)
        _need(output_x, torch.float32, "output_x")
        check(_lib.lib().lumen_moe_decode(self._h, layer._h, normed_x.data_ptr(), residual.data_ptr(),
                                          output_x.data_ptr(), T, _stream()))
        return output_x

    def decode_fused_norm(self, layer: MoeLayer, attn_proj: torch.Tensor, ffn_norm: torch.Tensor, eps: float,
                          normed_x: Optional[torch.Tensor] = None,
                          output_x: Optional[torch.Tensor] = None) -> torch.Tensor:
        _need(attn_proj, torch.float32, "attn_proj")
        _need(ffn_norm, torch.float32, "ffn_norm")
        T = attn_proj.numel() // self.H
        if output_x is None:
            output_x = torch.empty_like(attn_proj)
        check(_lib.lib().lumen_moe_decode_fused_norm(self._h, layer._h, attn_proj.data_ptr(), ffn_norm.data_ptr(),
                                                     _ptr(normed_x), output_x.data_ptr(), eps, T, _stream()))
        return output_x

    def prefill(self, layer: MoeLayer, normed: torch.Tensor, residual: torch.Tensor,
                output: Optional[torch.Tensor] = None) -> torch.Tensor:
        if normed.dtype == torch.float32:
            act = ACT_F32
        elif normed.dtype == torch.bfloat16:
            act = ACT_BF16
        else:
            raise LumenMoeError(_lib.UNSUPPORTED, "activations must be float32 or bfloat16")
        _need(normed, normed.dtype, "normed")
        _need(residual, torch.float32, "residual")
        T = normed.numel() // self.H
        if output is None:
            output = torch.empty_like(residual)
        check(_lib.lib().lumen_moe_prefill(self._h, layer._h, normed.data_ptr(), residual.data_ptr(),
                                           output.data_ptr(), T, act, _stream()))
        return output

    def shared_expert_decode(self, layer: MoeLayer, normed_x: torch.Tensor, output_x: torch.Tensor) -> torch.Tensor:
        """lumen_moe_shared_expert_decode: output_x += gate * FFN_shared(normed_x), in place (this context
        must be a shared-expert context: one expert, top-1, gating mode 2 or 3)."""
        _need(normed_x, torch.float32, "normed_x")
        _need(output_x, torch.float32, "output_x")
        T = normed_x.numel() // self.H
        check(_lib.lib().lumen_moe_shared_expert_decode(self._h, layer._h, normed_x.data_ptr(), output_x.data_ptr(),
                                                        T, _stream()))
        return output_x

    def shared_expert_prefill(self, layer: MoeLayer, normed: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
        """lumen_moe_shared_expert_prefill: the batched form, any number of tokens."""
        act = ACT_F32 if normed.dtype == torch.float32 else ACT_BF16
        _need(normed, normed.dtype, "normed")
        _need(output, torch.float32, "output")
        T = normed.numel() // self.H
        check(_lib.lib().lumen_moe_shared_expert_prefill(self._h, layer._h, normed.data_ptr(), output.data_ptr(),
                                                         T, act, _stream()))
        return output

    def prefill_routed(self, layer: MoeLayer, normed: torch.Tensor, ids: torch.Tensor,
                       weights: Optional[torch.Tensor], residual: torch.Tensor,
                       output: Optional[torch.Tensor] = None) -> torch.Tensor:
        """lumen_moe_prefill_routed: expert products + combine for caller-supplied routing."""
        act = {torch.float32: ACT_F32, torch.bfloat16: ACT_BF16, torch.float16: ACT_F16}[normed.dtype]
        _need(normed, normed.dtype, "normed")
        _need(ids, torch.int32, "ids")
        _need(residual, torch.float32, "residual")
        T = normed.numel() // self.H
        if output is None:
            output = torch.empty_like(residual)
        check(_lib.lib().lumen_moe_prefill_routed(self._h, layer._h, normed.data_ptr(), ids.data_ptr(), _ptr(weights),
                                                  residual.data_ptr(), output.data_ptr(), T, act, _stream()))
        return output

    def experts_routed_f16(self, layer: MoeLayer, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """lumen_moe_experts_routed_f16 (context with top_k = 1): f16 [R,H] expert outputs in row order."""
        act = {torch.float32: ACT_F32, torch.bfloat16: ACT_BF16, torch.float16: ACT_F16}[rows.dtype]
        _need(rows, rows.dtype, "rows")
        _need(ids, torch.int32, "ids")
        R = rows.numel() // self.H
        out = torch.empty((R, self.H), dtype=torch.float16, device=rows.device)
        check(_lib.lib().lumen_moe_experts_routed_f16(self._h, layer._h, rows.data_ptr(), ids.data_ptr(),
                                                      out.data_ptr(), R, act, _stream()))
        return out

    def route_only(self, layer: MoeLayer, normed_x: torch.Tensor, want_logits: bool = False):
        _need(normed_x, torch.float32, "normed_x")
        T = normed_x.numel() // self.H
        ids = torch.empty((T, self.K), dtype=torch.int32, device=normed_x.device)
        w = torch.empty((T, self.K), dtype=torch.float32, device=normed_x.device)
        lg = torch.empty((T, self.E), dtype=torch.float32, device=normed_x.device) if want_logits else None
        check(_lib.lib().lumen_moe_route_only(self._h, layer._h, normed_x.data_ptr(), T, ids.data_ptr(),
                                              w.data_ptr(), _ptr(lg), _stream()))
        return (ids, w, lg) if want_logits else (ids, w)

    def topk_from_logits(self, logits: torch.Tensor):
        _need(logits, torch.float32, "logits")
        T = logits.numel() // self.E
        ids = torch.empty((T, self.K), dtype=torch.int32, device=logits.device)
        w = torch.empty((T, self.K), dtype=torch.float32, device=logits.device)
        check(_lib.lib().lumen_moe_topk_from_logits(self._h, logits.data_ptr(), T, ids.data_ptr(), w.data_ptr(),
                                                    _stream()))
        return ids, w

    def set_logits_override(self, logits: Optional[torch.Tensor]) -> None:
        if logits is not None:
            _need(logits, torch.float32, "logits")
        self._override = logits
        check(_lib.lib().lumen_moe_set_logits_override(self._h, _ptr(logits)))

    def get_routing_device_into(self, tokens: int, dst_to_col=None, col_src_tok=None, col_expert=None,
                                expert_bounds=None) -> None:
        """Copies the chosen sort tables of the last routing call into the caller's int32 device tensors."""
        p = lambda t: t.data_ptr() if t is not None else None
        check(_lib.lib().lumen_moe_get_routing_device(self._h, tokens, p(dst_to_col), p(col_src_tok), p(col_expert),
                                                      p(expert_bounds), _stream()))

    def get_routing_device(self, tokens: int, device):
        """Sort tables of the last routing call as device tensors (no host sync)."""
        C = tokens * self.K
        d2c = torch.empty(C, dtype=torch.int32, device=device)
        cst = torch.empty(C, dtype=torch.int32, device=device)
        cex = torch.empty(C, dtype=torch.int32, device=device)
        bounds = torch.empty(self.E + 1, dtype=torch.int32, device=device)
        check(_lib.lib().lumen_moe_get_routing_device(self._h, tokens, d2c.data_ptr(), cst.data_ptr(), cex.data_ptr(),
                                                      bounds.data_ptr(), _stream()))
        return {"dst_to_col": d2c, "col_src_tok": cst, "col_expert": cex, "expert_bounds": bounds}

    def ep_prepare(self, normed: torch.Tensor, experts_per_rank: int):
        """lumen_moe_ep_prepare after route_only: (rows [T*K,H], local_ids int32 [T*K], send_counts int64 [G]);
        rows are bf16 for bf16 activations and f16 for f32 activations."""
        act = ACT_F32 if normed.dtype == torch.float32 else ACT_BF16
        T = normed.numel() // self.H
        dev = normed.device
        rows = torch.empty((T * self.K, self.H), dtype=torch.float16 if act == ACT_F32 else torch.bfloat16, device=dev)
        local_ids = torch.empty(T * self.K, dtype=torch.int32, device=dev)
        send_counts = torch.empty(self.E // experts_per_rank, dtype=torch.int64, device=dev)
        check(_lib.lib().lumen_moe_ep_prepare(self._h, normed.data_ptr(), act, T, experts_per_rank, rows.data_ptr(),
                                              local_ids.data_ptr(), send_counts.data_ptr(), _stream()))
        return rows, local_ids, send_counts

    def get_routing(self, tokens: int):
        C = tokens * self.K
        ids = np.zeros((tokens, self.K), np.uint32)
        w = np.zeros((tokens, self.K), np.float32)
        d2c = np.zeros(C, np.int32)
        cst = np.zeros(C, np.int32)
        bounds = np.zeros(self.E + 1, np.int32)
        check(_lib.lib().lumen_moe_get_routing(self._h, tokens, ids.ctypes.data, w.ctypes.data, d2c.ctypes.data,
                                               cst.ctypes.data, bounds.ctypes.data, _stream()))
        return {"ids": ids, "weights": w, "dst_to_col": d2c, "col_src_tok": cst, "expert_bounds": bounds}

    # -- expert parallel (lumen_moe_ep_*) ----------------------------------
    def ep_create(self, rank: int, world: int, max_tokens: int, recv_rows: int = 0) -> bytes:
        """lumen_moe_ep_create: allocates this rank's window; returns its 64-byte IPC handle."""
        buf = ctypes.create_string_buffer(64)
        check(_lib.lib().lumen_moe_ep_create(self._h, rank, world, max_tokens, recv_rows, buf))
        self.ep_rank, self.ep_world = rank, world
        return buf.raw

    def ep_attach(self, handles: Sequence[bytes]) -> None:
        """lumen_moe_ep_attach: `handles` = every rank's handle, in rank order."""
        blob = b"".join(handles)
        assert len(blob) == 64 * self.ep_world
        check(_lib.lib().lumen_moe_ep_attach(self._h, blob, self.ep_rank, self.ep_world))

    def ep_prepare_layer(self, blob: torch.Tensor, meta: MoeMeta) -> MoeLayer:
        """lumen_moe_ep_layer_prepare: router + this rank's experts of a full layer blob."""
        _need(blob, torch.uint8, "layer blob")
        go = np.ascontiguousarray(meta.expert_gate_offs, dtype=np.uint64)
        uo = np.ascontiguousarray(meta.expert_up_offs, dtype=np.uint64)
        do = np.ascontiguousarray(meta.expert_down_offs, dtype=np.uint64)
        if not (len(go) == len(uo) == len(do) == self.E):
            raise LumenMoeError(_lib.INVALID_ARG, "offset tables must have num_experts entries")
        h = ctypes.c_void_p()
        check(_lib.lib().lumen_moe_ep_layer_prepare(self._h, blob.data_ptr(), blob.numel(), meta.router_weight_off,
                                                    go.ctypes.data, uo.ctypes.data, do.ctypes.data,
                                                    meta.expert_gate_quant, _stream(), ctypes.byref(h)))
        return MoeLayer(h.value, blob, meta)

    def prefill_ep(self, layer: MoeLayer, normed: torch.Tensor, residual: torch.Tensor,
                   output: Optional[torch.Tensor] = None) -> torch.Tensor:
        """lumen_moe_prefill_ep: one expert-parallel layer call on this rank's tokens (collective)."""
        act = {torch.float32: ACT_F32, torch.bfloat16: ACT_BF16}[normed.dtype]
        _need(normed, normed.dtype, "normed")
        _need(residual, torch.float32, "residual")
        T = normed.numel() // self.H
        if output is None:
            output = torch.empty_like(residual)
        check(_lib.lib().lumen_moe_prefill_ep(self._h, layer._h, normed.data_ptr(), residual.data_ptr(),
                                              output.data_ptr(), T, act, _stream()))
        return output

    EP_PHASES = ("route", "counts+dispatch", "wait_rows+plan", "experts", "wait_results", "combine")

    def ep_profile(self, on: bool) -> None:
        check(_lib.lib().lumen_moe_ep_profile(self._h, 1 if on else 0))

    def ep_phase_ms(self) -> dict:
        out = (ctypes.c_float * 6)()
        check(_lib.lib().lumen_moe_ep_phase_ms(self._h, out))
        return dict(zip(self.EP_PHASES, [float(v) for v in out]))

    def stack_prefill_ep(self, layers: Sequence[MoeLayer], gammas: Sequence[torch.Tensor], x: torch.Tensor,
                         eps: float, normed: Optional[torch.Tensor] = None) -> torch.Tensor:
        _need(x, torch.float32, "x")
        if normed is None:
            normed = torch.empty_like(x)
        n = len(layers)
        lh = (ctypes.c_void_p * n)(*[l._h for l in layers])
        gp = (ctypes.c_void_p * n)(*[g.data_ptr() for g in gammas])
        check(_lib.lib().lumen_moe_stack_prefill_ep(self._h, lh, gp, n, x.data_ptr(), normed.data_ptr(), eps,
                                                    x.numel() // self.H, _stream()))
        return x

    def get_routing_ids_stride_e(self, tokens: int) -> np.ndarray:
        """ids of the last routing call as the reference's batched buffer lays them out: [T, E], first K valid."""
        ids = np.zeros((tokens, self.E), np.uint32)
        check(_lib.lib().lumen_moe_get_routing_ids_stride_e(self._h, tokens, ids.ctypes.data, _stream()))
        return ids

    def poll_status(self) -> int:
        """lumen_moe_poll_status: 0, or the code a kernel of this context recorded when it gave up (no sync)."""
        return int(_lib.lib().lumen_moe_poll_status(self._h))

    def clear_status(self) -> None:
        check(_lib.lib().lumen_moe_clear_status(self._h, _stream()))

    def debug_expire_next_wait(self, which: int) -> None:
        check(_lib.lib().lumen_moe_debug_expire_next_wait(self._h, which))

    def debug_decode_trace(self, layer):
        """Per-CTA phase stamps (ns) of the fused decode kernel for the last decode call: int64 [SMs, 12]."""
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        tr = torch.zeros((sms, 12), dtype=torch.int64, device=f"cuda:{self.device}")
        check(_lib.lib().lumen_moe_debug_decode_trace(self._h, layer._h, tr.data_ptr(), _stream()))
        return tr

    def debug_decode_phase(self, layer: MoeLayer, phase: int) -> None:
        check(_lib.lib().lumen_moe_debug_decode_phase(self._h, layer._h, phase, _stream()))

    def stack_decode(self, layers: Sequence[MoeLayer], gammas: Sequence[torch.Tensor], x: torch.Tensor,
                     eps: float) -> torch.Tensor:
        _need(x, torch.float32, "x")
        n = len(layers)
        lh = (ctypes.c_void_p * n)(*[l._h for l in layers])
        gp = (ctypes.c_void_p * n)(*[g.data_ptr() for g in gammas])
        T = x.numel() // self.H
        check(_lib.lib().lumen_moe_stack_decode(self._h, lh, gp, n, x.data_ptr(), eps, T, _stream()))
        return x


    def stack_prefill(self, layers: Sequence[MoeLayer], gammas: Sequence[torch.Tensor], x: torch.Tensor,
                      eps: float, normed: Optional[torch.Tensor] = None) -> torch.Tensor:
        """lumen_moe_stack_prefill: x <- x + MoE_l(rmsnorm(x)) over the layers, in place, any token count."""
        _need(x, torch.float32, "x")
        if normed is None:
            normed = torch.empty_like(x)
        _need(normed, torch.float32, "normed")
        n = len(layers)
        lh = (ctypes.c_void_p * n)(*[l._h for l in layers])
        gp = (ctypes.c_void_p * n)(*[g.data_ptr() for g in gammas])
        T = x.numel() // self.H
        check(_lib.lib().lumen_moe_stack_prefill(self._h, lh, gp, n, x.data_ptr(), normed.data_ptr(), eps, T,
                                                 _stream()))
        return x


def allocate_moe_scratch(hidden_dim: int, expert_inter_dim: int, num_experts: int, top_k: int,
                         max_tokens: int = 16, gating_mode: int = SOFTMAX_RENORM, device: int = 0,
                         flags: int = 0) -> MoeScratch:
    """allocate_moe_scratch (cuda/moe.rs:968)."""
    return MoeScratch(hidden_dim, expert_inter_dim, num_experts, top_k, max_tokens, gating_mode, device, flags)


def encode_moe_ffn_decode(scratch: MoeScratch, layer: MoeLayer, normed_x, residual, output_x):
    """encode_moe_ffn_decode (cuda/moe.rs:1119): output_x = residual + MoE(normed_x)."""
    return scratch.decode(layer, normed_x, residual, output_x)


def encode_moe_ffn_decode_fused_norm(scratch: MoeScratch, layer: MoeLayer, attn_proj, ffn_norm, normed_x, output_x,
                                     eps: float):
    """encode_moe_ffn_decode_fused_norm (cuda/moe.rs:3184)."""
    return scratch.decode_fused_norm(layer, attn_proj, ffn_norm, eps, normed_x, output_x)


def encode_moe_ffn_prefill_grouped(scratch: MoeScratch, layer: MoeLayer, normed, residual, output):
    """encode_moe_ffn_prefill_grouped (cuda/moe.rs:1900)."""
    return scratch.prefill(layer, normed, residual, output)


def quantize(src: torch.Tensor, quant: int) -> torch.Tensor:
    """Device quantiser (crates/lumen-convert/src/dequant.rs:791-906); returns raw bytes."""
    _need(src, torch.float32, "src")
    n = src.numel()
    nbytes = {Q8_0: n // 32 * 34, Q4_0: n // 32 * 18, BF16: n * 2}[quant]
    dst = torch.empty(nbytes, dtype=torch.uint8, device=src.device)
    check(_lib.lib().lumen_moe_quantize(src.data_ptr(), n, quant, dst.data_ptr(), _stream()))
    return dst


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    _need(x, torch.float32, "x")
    out = torch.empty_like(x)
    H = gamma.numel()
    check(_lib.lib().lumen_moe_rmsnorm(x.data_ptr(), gamma.data_ptr(), out.data_ptr(), x.numel() // H, H, eps,
                                       _stream()))
    return out


def debug_expf(x: torch.Tensor) -> torch.Tensor:
    _need(x, torch.float32, "x")
    out = torch.empty_like(x)
    check(_lib.lib().lumen_moe_debug_expf(x.data_ptr(), out.data_ptr(), x.numel(), _stream()))
    return out


def launch_count(reset: bool = False) -> int:
    return int(_lib.lib().lumen_moe_launch_count(1 if reset else 0))


def route_small_static(logits: torch.Tensor, top_k: int, gating_mode: int = SOFTMAX_RENORM, want_tables: bool = False):
    """lumen_moe_route_small_static: context-free routing of 1..16 tokens for callers
    that may not allocate device memory (the outputs created here are the CALLER's
    buffers; the library itself allocates nothing)."""
    _need(logits, torch.float32, "logits")
    T, E = logits.shape
    ids = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    d2c = torch.empty(T * top_k, dtype=torch.int32, device=logits.device) if want_tables else None
    bounds = torch.empty(E + 1, dtype=torch.int32, device=logits.device) if want_tables else None
    check(_lib.lib().lumen_moe_route_small_static(logits.data_ptr(), T, E, top_k, gating_mode, ids.data_ptr(),
                                                  w.data_ptr(), _ptr(d2c), _ptr(bounds), _stream()))
    return (ids, w, d2c, bounds) if want_tables else (ids, w)


def combine_f16(d16: torch.Tensor, residual: torch.Tensor, weights: torch.Tensor, dst_to_col: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """lumen_moe_combine_f16: out[t] = residual[t] + sum_slot w[t,slot] * d16[dst_to_col[t*K+slot]]."""
    _need(d16, torch.float16, "d16")
    _need(residual, torch.float32, "residual")
    _need(weights, torch.float32, "weights")
    _need(dst_to_col, torch.int32, "dst_to_col")
    T, H = residual.shape
    K = weights.numel() // T
    if out is None:
        out = torch.empty_like(residual)
    check(_lib.lib().lumen_moe_combine_f16(d16.data_ptr(), residual.data_ptr(), weights.data_ptr(),
                                           dst_to_col.data_ptr(), out.data_ptr(), T, H, K, _stream()))
    return out
