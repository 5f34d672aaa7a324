"""Loader of the CUDA library. There is no fallback: if the shared object is
missing or cannot be loaded, importing an operator raises."""
from __future__ import annotations

import ctypes
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "liblumen_moe_b200.so"

OK, INVALID_ARG, UNSUPPORTED, CUDA_ERROR, TIMEOUT, NCCL_ERROR = range(6)
Q8_0, Q4_0, BF16 = 0, 1, 2
SOFTMAX_RENORM, SIGMOID_RENORM, SIGMOID_GATE, UNIT_WEIGHT = 0, 1, 2, 3
ACT_F32, ACT_BF16, ACT_F16 = 0, 1, 2
# lumen_moe_config.flags
FLAG_DECODE_SPLIT, FLAG_PREFILL_MMA, FLAG_SHORT_WAITS, FLAG_PREFILL_F16_WEIGHTS = 0x1, 0x2, 0x4, 0x8


def flag_tc_ctas(n: int) -> int:
    return (n & 0xFF) << 8


class MoeConfig(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("hidden_dim", "inter_dim", "num_experts", "top_k", "max_tokens", "gating_mode", "device", "flags")]


class LbcSlice(ctypes.Structure):
    _fields_ = [("offset", ctypes.c_uint64), ("length", ctypes.c_uint64), ("quant", ctypes.c_uint32),
                ("present", ctypes.c_uint32)]


class LbcHeader(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint32) for n in
                ("version", "num_layers", "num_heads", "num_kv_heads", "head_dim", "hidden_dim", "intermediate_dim",
                 "vocab_size", "max_seq_len", "num_experts", "num_active_experts")] + [
        ("norm_eps", ctypes.c_float), ("primary_quant", ctypes.c_uint32), ("has_expert_index", ctypes.c_uint32),
        ("alignment", ctypes.c_uint64), ("layer_index_offset", ctypes.c_uint64), ("payload_offset", ctypes.c_uint64),
        ("header_bytes", ctypes.c_uint64)]


class LbcMoeLayer(ctypes.Structure):
    _fields_ = [("layer_offset_bytes", ctypes.c_uint64), ("layer_length_bytes", ctypes.c_uint64),
                ("is_moe", ctypes.c_uint32), ("num_experts", ctypes.c_uint32),
                ("expert_gate_quant", ctypes.c_uint32), ("expert_down_quant", ctypes.c_uint32),
                ("expert_gate_bytes", ctypes.c_uint64), ("expert_down_bytes", ctypes.c_uint64),
                ("router_weight", LbcSlice), ("ffn_norm", LbcSlice),
                ("shared_expert_gate", LbcSlice), ("shared_expert_up", LbcSlice), ("shared_expert_down", LbcSlice),
                ("ffn_gate_inp_shexp", LbcSlice),
                ("has_layer_type", ctypes.c_uint32), ("layer_type", ctypes.c_uint32)]


class LumenMoeError(RuntimeError):
    """Mirror of RuntimeError::Compute / ::Unsupported (crates/lumen-runtime/src/error.rs:6-31)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[{['OK','INVALID_ARG','UNSUPPORTED','CUDA_ERROR','TIMEOUT','NCCL_ERROR'][code]}] {msg}")
        self.code = code


_lib = None
vp, i32, i64, u64, f32, sz = (ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_float,
                              ctypes.c_size_t)

# name -> argtypes; every entry point include/lumen_moe.h declares
SIGNATURES = {
    "lumen_moe_create": [ctypes.POINTER(MoeConfig), ctypes.POINTER(vp)],
    "lumen_moe_destroy": [vp],
    "lumen_moe_ensure_prefill": [vp, i32],
    "lumen_moe_layer_prepare": [vp, vp, sz, u64, vp, vp, vp, i32, vp, ctypes.POINTER(vp)],
    "lumen_moe_layer_destroy": [vp],
    "lumen_moe_decode": [vp, vp, vp, vp, vp, i32, vp],
    "lumen_moe_decode_fused_norm": [vp, vp, vp, vp, vp, vp, f32, i32, vp],
    "lumen_moe_prefill": [vp, vp, vp, vp, vp, i32, i32, vp],
    "lumen_moe_prefill_routed": [vp, vp, vp, vp, vp, vp, vp, i32, i32, vp],
    "lumen_moe_experts_routed_f16": [vp, vp, vp, vp, vp, i32, i32, vp],
    "lumen_moe_combine_f16": [vp, vp, vp, vp, vp, i32, i32, i32, vp],
    "lumen_moe_route_only": [vp, vp, vp, i32, vp, vp, vp, vp],
    "lumen_moe_topk_from_logits": [vp, vp, i32, vp, vp, vp],
    "lumen_moe_route_small_static": [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp],
    "lumen_moe_set_logits_override": [vp, vp],
    "lumen_moe_get_routing": [vp, i32, vp, vp, vp, vp, vp, vp],
    "lumen_moe_get_routing_device": [vp, i32, vp, vp, vp, vp, vp],
    "lumen_moe_get_routing_ids_stride_e": [vp, i32, vp, vp],
    "lumen_moe_poll_status": [vp],
    "lumen_moe_clear_status": [vp, vp],
    "lumen_moe_debug_expire_next_wait": [vp, i32],
    "lumen_moe_ep_prepare": [vp, vp, i32, i32, i32, vp, vp, vp, vp],
    "lumen_moe_ep_create": [vp, i32, i32, i32, i32, vp],
    "lumen_moe_ep_attach": [vp, vp, i32, i32],
    "lumen_moe_ep_layer_prepare": [vp, vp, sz, u64, vp, vp, vp, i32, vp, ctypes.POINTER(vp)],
    "lumen_moe_prefill_ep": [vp, vp, vp, vp, vp, i32, i32, vp],
    "lumen_moe_stack_prefill_ep": [vp, vp, vp, i32, vp, vp, f32, i32, vp],
    "lumen_moe_ep_profile": [vp, i32],
    "lumen_moe_ep_phase_ms": [vp, vp],
    "lumen_lbc_read_header": [vp, sz, ctypes.POINTER(LbcHeader)],
    "lumen_lbc_read_moe_layer": [vp, sz, ctypes.c_uint32, ctypes.POINTER(LbcMoeLayer), vp, vp, vp, ctypes.c_uint32],
    "lumen_lbc_quant_to_moe": [ctypes.c_uint32],
    "lumen_moe_quantize": [vp, i64, i32, vp, vp],
    "lumen_moe_rmsnorm": [vp, vp, vp, i32, i32, f32, vp],
    "lumen_moe_stack_decode": [vp, vp, vp, i32, vp, f32, i32, vp],
    "lumen_moe_stack_prefill": [vp, vp, vp, i32, vp, vp, f32, i32, vp],
    "lumen_moe_debug_expf": [vp, vp, i64, vp],
    "lumen_moe_shared_expert_decode": [vp, vp, vp, vp, i32, vp],
    "lumen_moe_shared_expert_prefill": [vp, vp, vp, vp, i32, i32, vp],
    "lumen_moe_debug_decode_trace": [vp, vp, vp, vp],
    "lumen_moe_debug_decode_phase": [vp, vp, i32, vp],
    "lumen_moe_layer_bytes": [vp],
    "lumen_moe_launch_count": [i32],
    "lumen_moe_last_error": [],
    "lumen_moe_version": [],
}
_RESTYPE = {"lumen_moe_destroy": None, "lumen_moe_layer_destroy": None, "lumen_moe_layer_bytes": sz,
            "lumen_moe_launch_count": i64, "lumen_moe_last_error": ctypes.c_char_p,
            "lumen_moe_version": ctypes.c_char_p}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m lumen_b200.build` (nvcc, sm_100a). "
                "lumen_b200 has no CPU or PyTorch fallback.")
        l = ctypes.CDLL(str(LIB_PATH))
        for name, args in SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = _RESTYPE.get(name, i32)
        _lib = l
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise LumenMoeError(code, lib().lumen_moe_last_error().decode())
