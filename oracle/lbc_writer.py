"""Writer of LBC files for tests: a Python restatement of the reference's container writer.

TEST INFRASTRUCTURE ONLY (imported by tests/ alone): it produces the files that the
library's LBC index reader is checked on. It follows
crates/lumen-format/src/writer.rs (write_lbc :28-192, serialize_header :219-267,
serialize_hyperparams :270-331, serialize_quant_desc :333-360, serialize_tensor_slice
:362-367, serialize_layer_indices :369-513) and crc.rs.

Pinned by the known answers the reference's own tests hold: the CRC-32 check value
0xCBF43926 of "123456789" (crc.rs known_vectors), the header sizes 183 (v2) / 207 (v3)
bytes (reader.rs genuine_v2_binary_reads_with_v3_reader), and the slice offsets asserted
by reader.rs moe_roundtrip. No LBC file written by the reference itself exists in this
build (no Rust toolchain), so byte-for-byte equality with its writer is unpinned.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

MAGIC = 0x0143424C
F32, F16, BF16, Q8_0, Q4_0 = 0, 1, 2, 3, 4  # scheme tags, quantization.rs:123-137


def crc32(data: bytes) -> int:
    crc = 0xFFFFFFFF
    for b in data:
        crc ^= b
        for _ in range(8):
            crc = (crc >> 1) ^ 0xEDB88320 if crc & 1 else crc >> 1
    return crc ^ 0xFFFFFFFF


Slice = Tuple[int, int, int]  # offset, length, scheme tag


@dataclass
class Layer:
    """SubtensorOffsets (index.rs:30-113); offsets relative to the layer blob."""
    wq: Slice = (0, 0, F32)
    wk: Slice = (0, 0, F32)
    wv: Slice = (0, 0, F32)
    wo: Slice = (0, 0, F32)
    w_gate: Slice = (0, 0, F32)
    w_up: Slice = (0, 0, F32)
    w_down: Slice = (0, 0, F32)
    attn_norm: Slice = (0, 0, F32)
    ffn_norm: Slice = (0, 0, F32)
    bias: Sequence[Optional[Slice]] = (None, None, None)  # bq, bk, bv
    router_weight: Optional[Slice] = None
    experts: Optional[List[Tuple[Slice, Slice, Slice]]] = None  # (gate, up, down) per expert
    # optional slices by extension bit (writer.rs:426-513); bit 12 is the layer type byte
    ext: dict = field(default_factory=dict)  # bit -> Slice
    layer_type: Optional[int] = None


EXT_BITS = {"shared_expert_gate": 0, "shared_expert_up": 1, "shared_expert_down": 2, "attn_gate": 3,
            "attn_post_norm": 4, "ssm_a": 5, "ssm_conv1d": 6, "ssm_dt": 7, "ssm_beta": 8, "ssm_alpha": 9,
            "ssm_norm": 10, "ssm_out": 11, "attn_q_norm": 13, "attn_k_norm": 14, "ffn_gate_inp_shexp": 15}


def _slice(s: Slice) -> bytes:
    return struct.pack("<QQB7x", s[0], s[1], s[2])


def serialize_layer_index(layer_offset: int, layer_length: int, L: Layer) -> bytes:
    b = struct.pack("<QQ", layer_offset, layer_length)
    for s in (L.wq, L.wk, L.wv, L.wo, L.w_gate, L.w_up, L.w_down, L.attn_norm, L.ffn_norm):
        b += _slice(s)
    flags = sum(1 << i for i, s in enumerate(L.bias) if s is not None)
    b += struct.pack("<B7x", flags)
    for s in L.bias:
        if s is not None:
            b += _slice(s)
    ne = len(L.experts) if L.experts else 0
    b += struct.pack("<IB3x", ne, 1 if L.router_weight is not None else 0)
    if L.router_weight is not None:
        b += _slice(L.router_weight)
    for g, u, d in (L.experts or []):
        b += _slice(g) + _slice(u) + _slice(d)
    ext = sum(1 << bit for bit in L.ext) | ((1 << 12) if L.layer_type is not None else 0)
    b += struct.pack("<I4x", ext)
    for bit in range(16):
        if bit == 12:
            if L.layer_type is not None:
                b += struct.pack("<B7x", L.layer_type)
        elif bit in L.ext:
            b += _slice(L.ext[bit])
    return b


@dataclass
class Model:
    num_layers: int
    hidden_dim: int
    intermediate_dim: int
    num_experts: int = 0
    num_active_experts: int = 0
    num_heads: int = 2
    num_kv_heads: int = 2
    head_dim: int = 4
    vocab_size: int = 32
    max_seq_len: int = 64
    norm_eps: float = 1e-5
    rope: Optional[Tuple[float, float, int]] = (10000.0, 1.0, 0)  # theta, scaling factor, scaling type
    gdn: Optional[Tuple[int, int, int, int]] = None                 # v4 block
    version: int = 4
    alignment: int = 128 * 1024
    primary_quant: int = F32
    block_byte_size: int = 4


def serialize_header(m: Model, layer_index_offset=0, payload_offset=0, ranges=((0, 0), (0, 0), (0, 0)),
                     checksum=0) -> bytes:
    b = struct.pack("<IIB3xI", MAGIC, m.version, 0, checksum)
    b += struct.pack("<8I", m.num_layers, m.num_heads, m.num_kv_heads, m.head_dim, m.hidden_dim,
                     m.intermediate_dim, m.vocab_size, m.max_seq_len)
    if m.rope is not None:
        b += struct.pack("<BffBBB", 1, m.rope[0], m.rope[1], m.rope[2], 0, 0)
    else:
        b += bytes(12)
    b += struct.pack("<IIf", m.num_experts, m.num_active_experts, m.norm_eps)
    if m.version >= 4:
        b += struct.pack("<B4I", 1, *m.gdn) if m.gdn is not None else b"\0"
    b += struct.pack("<BBIIBI", m.primary_quant, 0, 0, m.block_byte_size, 0, 0)
    b += struct.pack("<QIB3xQQQ", m.alignment, m.num_layers, 1 if m.num_experts else 0, layer_index_offset, 0,
                     payload_offset)
    for off, ln in ranges:
        b += struct.pack("<QQ", off, ln)
    if m.version >= 2:
        b += struct.pack("<BBBB4x", F32, F32, F32, 0)
    if m.version >= 3:
        b += bytes(24)  # no tokenizer section
    return b


def _align(v: int, a: int) -> int:
    return (v + a - 1) & ~(a - 1)


def write_lbc(m: Model, layers: Sequence[Layer], blobs: Sequence[bytes], globals_=(b"", b"", b"")) -> bytes:
    """Whole file: header, index, padding, global tensors, padding, aligned layer blobs."""
    assert len(layers) == len(blobs) == m.num_layers
    hdr_len = len(serialize_header(m))
    idx_len = sum(len(serialize_layer_index(0, 0, L)) for L in layers)
    globals_start = _align(hdr_len + idx_len, m.alignment)
    layers_start = _align(globals_start + sum(len(g) for g in globals_), m.alignment)
    ranges, cur = [], globals_start
    for g in globals_:
        ranges.append((cur, len(g)))
        cur += len(g)
    idx, cur, starts = b"", layers_start, []
    for L, blob in zip(layers, blobs):
        starts.append(cur)
        idx += serialize_layer_index(cur, len(blob), L)
        cur = _align(cur + len(blob), m.alignment)
    hdr = serialize_header(m, hdr_len, globals_start, ranges, 0)
    hdr = hdr[:12] + struct.pack("<I", crc32(hdr)) + hdr[16:]
    out = bytearray(hdr + idx)
    out += bytes(globals_start - len(out))
    for g in globals_:
        out += g
    out += bytes(layers_start - len(out))
    for i, blob in enumerate(blobs):
        assert len(out) == starts[i]
        out += blob
        if i + 1 < len(blobs):
            out += bytes(starts[i + 1] - len(out))
    return bytes(out)
