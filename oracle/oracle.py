"""ctypes front-end of the CPU oracle (oracle/lumen_moe_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs as the checker / the timed CPU baseline. The product
package (lumen_b200) never imports it.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "liblumen_moe_oracle.so"
REF_PATH = HERE / "_ref" / "liblumen_ref_kernels.so"

Q8_0, Q4_0, BF16 = 0, 1, 2
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18}


def build(ref: bool = True) -> None:
    subprocess.run(["make", "-C", str(HERE), "all"], check=True, capture_output=True)
    if ref:
        subprocess.run(["make", "-C", str(HERE), "ref"], check=False, capture_output=True)


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        src = HERE / "lumen_moe_oracle.cpp"
        if not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
            build(ref=False)
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.orc_f16_bits_to_f32.restype = ctypes.c_float
        _lib.orc_f16_bits_to_f32.argtypes = [ctypes.c_uint16]
        _lib.orc_f32_to_f16_bits.restype = ctypes.c_uint16
        _lib.orc_f32_to_f16_bits.argtypes = [ctypes.c_float]
        _lib.orc_row_bytes.restype = ctypes.c_int64
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def row_bytes(in_dim: int, quant: int) -> int:
    return {Q8_0: in_dim // 32 * 34, Q4_0: in_dim // 32 * 18, BF16: in_dim * 2}[quant]


def quantize(w: np.ndarray, quant: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = w.size
    out = np.zeros(n // 32 * BLOCK_BYTES[quant] if quant != BF16 else n * 2, dtype=np.uint8)
    fn = {Q8_0: lib().orc_quantize_q8_0, Q4_0: lib().orc_quantize_q4_0, BF16: lib().orc_quantize_bf16}[quant]
    fn(_p(w), ctypes.c_int64(n), _p(out))
    return out


def dequantize(raw: np.ndarray, n: int, quant: int) -> np.ndarray:
    out = np.zeros(n, dtype=np.float32)
    lib().orc_dequantize(_p(raw), ctypes.c_int64(n), ctypes.c_int(quant), _p(out))
    return out


def matvec(w_raw, x, out_dim, in_dim, quant):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(out_dim, dtype=np.float32)
    lib().orc_matvec(_p(w_raw), _p(x), _p(out), out_dim, in_dim, quant)
    return out


def swiglu(gate, up):
    g = np.array(gate, dtype=np.float32, copy=True)
    u = np.ascontiguousarray(up, dtype=np.float32)
    lib().orc_swiglu(_p(g), _p(u), g.size)
    return g


def rmsnorm(x, weight, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    out = np.zeros_like(x)
    if x.ndim == 1:
        lib().orc_rmsnorm(_p(out), _p(x), _p(w), x.size, ctypes.c_float(eps))
    else:
        for t in range(x.shape[0]):
            lib().orc_rmsnorm(_p(out[t]), _p(x[t]), _p(w), x.shape[1], ctypes.c_float(eps))
    return out


def router_logits(x, w, H, E):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.zeros(E, dtype=np.float32)
    lib().orc_router_logits(_p(x), _p(w), H, E, _p(out))
    return out


def topk_from_logits(logits, K, gating=0):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    single = logits.ndim == 1
    lg = logits.reshape(-1, logits.shape[-1])
    T, E = lg.shape
    ids = np.zeros((T, K), dtype=np.uint32)
    w = np.zeros((T, K), dtype=np.float32)
    scratch = np.zeros(E, dtype=np.float32)
    for t in range(T):
        lib().orc_topk_from_logits(_p(lg[t]), E, K, gating, _p(ids[t]), _p(w[t]), _p(scratch))
    return (ids[0], w[0]) if single else (ids, w)


def router_softmax(x, w, H, E, K):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    ids = np.zeros(K, dtype=np.uint32)
    wt = np.zeros(K, dtype=np.float32)
    logits = np.zeros(E, dtype=np.float32)
    lib().orc_router_softmax(_p(x), _p(w), H, E, K, _p(ids), _p(wt), _p(logits))
    return ids, wt, logits


def accum_option_a(residual, expert_outputs, expert_weights, H, K):
    out = np.zeros(H, dtype=np.float32)
    lib().orc_accum_option_a(_p(np.ascontiguousarray(residual, np.float32)),
                             _p(np.ascontiguousarray(expert_outputs, np.float32)),
                             _p(np.ascontiguousarray(expert_weights, np.float32)), H, K, _p(out))
    return out


def accum_batched_b(residual, expert_outputs, expert_weights, expert_ids, H, K):
    out = np.zeros(H, dtype=np.float32)
    lib().orc_accum_batched_b(_p(np.ascontiguousarray(residual, np.float32)),
                              _p(np.ascontiguousarray(expert_outputs, np.float32)),
                              _p(np.ascontiguousarray(expert_weights, np.float32)),
                              _p(np.ascontiguousarray(expert_ids, np.uint32)), H, K, _p(out))
    return out


def counting_sort(ids, E, K=None):
    """Host counting sort of cuda/moe.rs:2115-2147. `ids` is [T, K], or, with K given, the reference's
    batched id buffer [T, stride] whose rows hold K valid ids first (stride E, topk_moe_fused.cu:189-191)."""
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    T, ids_stride = ids.shape
    if K is None:
        K = ids_stride
    C = T * K
    col_expert = np.zeros(C, np.int32)
    col_src_tok = np.zeros(C, np.int32)
    dst_to_col = np.full(C, -1, np.int32)
    bounds = np.zeros(E + 1, np.int32)
    lib().orc_counting_sort(_p(ids), T, K, E, ids_stride, _p(col_expert), _p(col_src_tok), _p(dst_to_col), _p(bounds))
    return col_expert, col_src_tok, dst_to_col, bounds


def moe_layer(blob, router_off, gate_offs, up_offs, down_offs, quant, H, I, E, K, normed, residual,
              gating=0, logits=None, ids=None, weights=None, threads=1):
    """Whole layer. Returns (out [T,H], ids [T,K], weights [T,K])."""
    normed = np.ascontiguousarray(normed, dtype=np.float32).reshape(-1, H)
    residual = np.ascontiguousarray(residual, dtype=np.float32).reshape(-1, H)
    T = normed.shape[0]
    go = np.ascontiguousarray(gate_offs, dtype=np.uint64)
    uo = np.ascontiguousarray(up_offs, dtype=np.uint64)
    do = np.ascontiguousarray(down_offs, dtype=np.uint64)
    mode = 0
    lg = None
    if ids is not None:
        mode = 2
        ids_io = np.ascontiguousarray(ids, dtype=np.uint32).reshape(T, K).copy()
        w_io = np.ascontiguousarray(weights, dtype=np.float32).reshape(T, K).copy()
    else:
        ids_io = np.zeros((T, K), np.uint32)
        w_io = np.zeros((T, K), np.float32)
        if logits is not None:
            mode = 1
            lg = np.ascontiguousarray(logits, dtype=np.float32).reshape(T, E)
    out = np.zeros((T, H), np.float32)
    rc = lib().orc_moe_layer(_p(blob), ctypes.c_uint64(router_off), _p(go), _p(uo), _p(do), quant, H, I, E, K, T,
                             gating, mode, _p(normed), _p(residual), _p(lg), _p(ids_io), _p(w_io), _p(out), threads)
    if rc != 0:
        raise ValueError("oracle rejected the arguments")
    return out, ids_io, w_io


def hardware_threads() -> int:
    return int(lib().orc_hardware_threads())
