"""LBC header / layer index reader of the library (host only, no GPU) against files
written by the test-side restatement of the reference's writer, and against the known
answers the reference's own reader tests assert."""
import ctypes
import struct

import numpy as np
import pytest

from lumen_b200 import _lib, lbc
from oracle import lbc_writer as W


def test_crc_known_answer():
    # crates/lumen-format/src/crc.rs, known_vectors
    assert W.crc32(b"123456789") == 0xCBF43926
    assert W.crc32(b"") == 0


@pytest.mark.parametrize("version,size", [(2, 183), (3, 207), (4, 208)])
def test_header_sizes_per_version(cuda_lib, version, size):
    # 183 / 207: reader.rs genuine_v2_binary_reads_with_v3_reader; v4 adds the 1-byte GDN flag
    m = W.Model(num_layers=0, hidden_dim=8, intermediate_dim=16, version=version)
    data = W.write_lbc(m, [], [])
    idx = lbc.LbcIndex(data)
    assert idx.header.header_bytes == size == len(W.serialize_header(m))
    assert idx.header.layer_index_offset == size
    assert idx.header.version == version
    m4 = W.Model(num_layers=0, hidden_dim=8, intermediate_dim=16, gdn=(32, 16, 128, 4))
    assert lbc.LbcIndex(W.write_lbc(m4, [], [])).header.header_bytes == 224


def moe_roundtrip_file():
    """The file of reader.rs moe_roundtrip (:963-1120): 1 layer, 4 experts, all F32."""
    m = W.Model(num_layers=1, hidden_dim=8, intermediate_dim=16, num_experts=4, num_active_experts=2)
    off = 0
    sl = []
    for ln in (128, 128, 128, 128, 32, 32, 128):
        sl.append((off, ln, W.F32))
        off += ln
    experts = []
    for _ in range(4):
        e = []
        for _ in range(3):
            e.append((off, 512, W.F32))
            off += 512
        experts.append(tuple(e))
    L = W.Layer(wq=sl[0], wk=sl[1], wv=sl[2], wo=sl[3], attn_norm=sl[4], ffn_norm=sl[5], router_weight=sl[6],
                experts=experts)
    blob = bytes([42]) * off
    g = (bytes([1]) * (32 * 8 * 4), bytes([2]) * (8 * 4), bytes([3]) * (32 * 8 * 4))
    return m, W.write_lbc(m, [L], [blob], g), off


def read_layer_raw(data, layer, cap=256):
    out = _lib.LbcMoeLayer()
    offs = [np.zeros(cap, np.uint64) for _ in range(3)]
    buf = ctypes.create_string_buffer(data, len(data))
    code = _lib.lib().lumen_lbc_read_moe_layer(buf, len(data), layer, ctypes.byref(out),
                                               *(o.ctypes.data for o in offs), cap)
    return code, out, offs


def test_moe_roundtrip_known_answers(cuda_lib):
    m, data, blob_len = moe_roundtrip_file()
    idx = lbc.LbcIndex(data)
    h = idx.header
    assert (h.num_layers, h.num_experts, h.num_active_experts, h.has_expert_index) == (1, 4, 2, 1)
    assert h.hidden_dim == 8 and h.intermediate_dim == 16 and abs(h.norm_eps - 1e-5) < 1e-12
    code, out, (g, u, d) = read_layer_raw(data, 0)
    assert code == _lib.OK and out.is_moe == 1 and out.num_experts == 4
    # the values reader.rs:1096-1113 asserts
    assert (out.router_weight.offset, out.router_weight.length) == (576, 128)
    assert (g[0], u[0], d[0]) == (704, 1216, 1728)
    assert out.expert_gate_bytes == 512 and out.expert_down_bytes == 512
    assert g[3] == 704 + 3 * 1536 and d[3] == 704 + 3 * 1536 + 1024
    assert out.layer_length_bytes == blob_len == 6848
    assert out.layer_offset_bytes % h.alignment == 0
    assert data[out.layer_offset_bytes: out.layer_offset_bytes + 4] == bytes([42]) * 4
    # all-F32 experts: no kernel for that scheme, the Python mirror says so
    with pytest.raises(_lib.LumenMoeError) as ei:
        idx.moe_layer(0)
    assert ei.value.code == _lib.UNSUPPORTED


def qwen_like_file(E=8, H=64, I=32, quant=W.Q4_0, with_bias=True, layers=3):
    """Dense layer, MoE layer with shared expert and every optional section, MoE layer without."""
    rb = {W.Q4_0: 18, W.Q8_0: 34}[quant]
    gate_b, down_b = I * (H // 32) * rb, H * (I // 32) * rb
    m = W.Model(num_layers=layers, hidden_dim=H, intermediate_dim=I, num_experts=E, num_active_experts=2,
                gdn=(32, 16, 128, 4), primary_quant=quant, block_byte_size=rb)
    Ls, blobs, expect = [], [], []
    for li in range(layers):
        off = 0

        def take(n, q=W.F32):
            nonlocal off
            s = (off, n, q)
            off += n
            return s
        L = W.Layer(wq=take(100, quant), wk=take(60, quant), wv=take(60, quant), wo=take(100, quant),
                    attn_norm=take(H * 4), ffn_norm=take(H * 4))
        if li == 0:
            L.w_gate, L.w_up, L.w_down = take(gate_b, quant), take(gate_b, quant), take(down_b, quant)
            expect.append(None)
        else:
            if with_bias and li == 1:
                L.bias = (take(16), None, take(16))
            L.router_weight = take(E * H * 4)
            L.experts = [(take(gate_b, quant), take(gate_b, quant), take(down_b, quant)) for _ in range(E)]
            if li == 1:
                for name in ("shared_expert_gate", "shared_expert_up"):
                    L.ext[W.EXT_BITS[name]] = take(gate_b, quant)
                L.ext[W.EXT_BITS["shared_expert_down"]] = take(down_b, quant)
                for name in ("attn_gate", "ssm_a", "ssm_conv1d", "ssm_out", "attn_q_norm", "attn_k_norm"):
                    L.ext[W.EXT_BITS[name]] = take(24)
                L.ext[W.EXT_BITS["ffn_gate_inp_shexp"]] = take(H * 4)
                L.layer_type = 1
            expect.append(L)
        Ls.append(L)
        blobs.append(bytes([li + 1]) * off)
    return m, W.write_lbc(m, Ls, blobs), Ls, blobs


@pytest.mark.parametrize("quant,ours", [(W.Q4_0, _lib.Q4_0), (W.Q8_0, _lib.Q8_0)])
def test_dense_moe_and_optional_sections(cuda_lib, quant, ours):
    m, data, Ls, blobs = qwen_like_file(quant=quant)
    idx = lbc.LbcIndex(data)
    assert idx.config() == {"hidden_dim": 64, "num_experts": 8, "top_k": 2, "norm_eps": pytest.approx(1e-5)}
    assert idx.header.header_bytes == 224
    d0 = idx.moe_layer(0)
    assert d0.meta is None and d0.router_weight is None and d0.ffn_norm == Ls[0].ffn_norm
    for li in (1, 2):
        r = idx.moe_layer(li)
        L = Ls[li]
        assert r.meta is not None and r.inter_dim == 32
        assert r.meta.router_weight_off == L.router_weight[0]
        assert r.meta.expert_gate_offs.tolist() == [e[0][0] for e in L.experts]
        assert r.meta.expert_up_offs.tolist() == [e[1][0] for e in L.experts]
        assert r.meta.expert_down_offs.tolist() == [e[2][0] for e in L.experts]
        assert (r.meta.expert_gate_quant, r.meta.expert_down_quant) == (ours, ours)
        assert r.ffn_norm == L.ffn_norm and r.router_weight == L.router_weight
        assert r.layer_length_bytes == len(blobs[li])
        assert r.layer_offset_bytes % idx.header.alignment == 0
        assert data[r.layer_offset_bytes: r.layer_offset_bytes + len(blobs[li])] == blobs[li]
    r1, r2 = idx.moe_layer(1), idx.moe_layer(2)
    assert r1.shared_expert_gate == Ls[1].ext[0] and r1.shared_expert_up == Ls[1].ext[1]
    assert r1.shared_expert_down == Ls[1].ext[2] and r1.ffn_gate_inp_shexp == Ls[1].ext[15]
    assert r1.layer_type == 1
    assert r2.shared_expert_gate is None and r2.ffn_gate_inp_shexp is None and r2.layer_type is None
    # a path works like bytes, and reads no further than the index
    import tempfile
    with tempfile.NamedTemporaryFile(suffix=".lbc") as f:
        f.write(data)
        f.flush()
        p = lbc.LbcIndex(f.name)
        assert p._n == idx.header.payload_offset
        assert p.moe_layer(2).meta.expert_down_offs.tolist() == r2.meta.expert_down_offs.tolist()
        # the layer blob, from the path and from the bytes
        assert p.read_layer_blob(f.name, r2).tobytes() == blobs[2] == idx.read_layer_blob(data, r2).tobytes()
        with pytest.raises(_lib.LumenMoeError):
            idx.read_layer_blob(data[: r2.layer_offset_bytes + 10], r2)


def test_error_cases_of_the_reference_reader(cuda_lib):
    m, data, _ = moe_roundtrip_file()
    h = _lib.LbcHeader()

    def header_code(b):
        buf = ctypes.create_string_buffer(bytes(b), len(b))
        return _lib.lib().lumen_lbc_read_header(buf, len(b), ctypes.byref(h))

    assert header_code(data) == _lib.OK
    # bad magic (reader.rs bad_magic), truncated (truncated_file)
    assert header_code(b"\xef\xbe\xad\xde" + data[4:]) == _lib.INVALID_ARG
    assert b"magic" in _lib.lib().lumen_moe_last_error()
    assert header_code(data[:20]) == _lib.INVALID_ARG
    assert header_code(b"") == _lib.INVALID_ARG
    # version above 4 (header.rs version_validation)
    assert header_code(data[:4] + struct.pack("<I", 5) + data[8:]) == _lib.UNSUPPORTED
    # one flipped header byte: checksum mismatch
    bad = bytearray(data)
    bad[40] ^= 1
    assert header_code(bad) == _lib.INVALID_ARG
    assert b"checksum" in _lib.lib().lumen_moe_last_error()
    # endianness byte
    bad = bytearray(data)
    bad[8] = 7
    assert header_code(bad) == _lib.INVALID_ARG
    # layer out of range; index cut short; capacity too small
    assert read_layer_raw(data, 1)[0] == _lib.INVALID_ARG
    hdr_len = lbc.LbcIndex(data).header.header_bytes
    assert read_layer_raw(data[: hdr_len + 300], 0)[0] == _lib.INVALID_ARG
    assert read_layer_raw(data, 0, cap=3)[0] == _lib.INVALID_ARG


def test_slice_outside_the_layer_blob_is_rejected(cuda_lib):
    # LayerIndex::validate (index.rs:229-378): offset + length beyond the blob, and u64 overflow
    for bad_slice in ((6848 - 100, 512, W.F32), (2**64 - 1, 2, W.F32)):
        m = W.Model(num_layers=1, hidden_dim=8, intermediate_dim=16, num_experts=1, num_active_experts=1)
        L = W.Layer(router_weight=(0, 32, W.F32), experts=[((32, 512, W.Q8_0), (544, 512, W.Q8_0), bad_slice)])
        data = W.write_lbc(m, [L], [bytes(6848)])
        code, *_ = read_layer_raw(data, 0)
        assert code == _lib.INVALID_ARG
        assert b"outside the layer blob" in _lib.lib().lumen_moe_last_error()
    # an unknown scheme tag (quantization.rs:138-140)
    L = W.Layer(router_weight=(0, 32, W.F32), experts=[((32, 512, 77), (544, 512, W.Q8_0), (1056, 512, W.Q8_0))])
    data = W.write_lbc(m, [L], [bytes(6848)])
    assert read_layer_raw(data, 0)[0] == _lib.UNSUPPORTED


def test_truncated_and_corrupted_files_never_read_out_of_bounds(cuda_lib):
    """Every prefix of a file and a sweep of single-byte corruptions of its index: the reader
    returns a status (no crash), OK only when the data really holds the whole index."""
    m, data, Ls, blobs = qwen_like_file(E=4, H=32, I=32, layers=2, with_bias=True)
    idx = lbc.LbcIndex(data)
    index_end = None
    # the index ends where the next section starts: find it as the shortest prefix that parses layer 1
    lo = int(idx.header.header_bytes)
    for n in list(range(0, lo + 1)) + list(range(lo, lo + 2200, 7)):
        code, out, _ = read_layer_raw(data[:n], 1)
        if code == _lib.OK and index_end is None:
            index_end = n
        if n < lo:
            assert code != _lib.OK
    assert index_end is not None and index_end > lo
    rng = np.random.default_rng(0)
    for _ in range(300):
        bad = bytearray(data[: index_end + 64])
        pos = int(rng.integers(lo, index_end))
        bad[pos] = int(rng.integers(0, 256))
        code, out, _ = read_layer_raw(bytes(bad), 1)
        assert code in (_lib.OK, _lib.INVALID_ARG, _lib.UNSUPPORTED)
        # huge expert counts must be refused, not allocated
        if code == _lib.OK:
            assert out.num_experts <= 256
