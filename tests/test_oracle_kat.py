"""Pins the CPU oracle against the known-answer tests the reference keeps for this
path. Each test names the reference test it re-states (paths relative to the
reference project's root)."""
import math

import numpy as np
import pytest

Q8_0, Q4_0, BF16 = 0, 1, 2


def lcg(seed):
    """The LCG of cuda/moe.rs:6557-6562: s = s*6364136223846793005 + 1442695040888963407;
    value = ((s >> 32) as u32) as f32 / (u32::MAX as f32) - 0.5."""
    state = [seed & 0xFFFFFFFFFFFFFFFF]

    def nxt():
        state[0] = (state[0] * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return np.float32(np.float32(state[0] >> 32) / np.float32(4294967295.0) - np.float32(0.5))
    return nxt


# ---- block formats: crates/lumen-convert/src/convert.rs:1046-1130 ----------
def test_f16_roundtrip_and_truncation(orc):
    l = orc.lib()
    for v in (0.0, 1.0, -2.0, 0.5, 65504.0, 6.103515625e-05, 5.9604645e-08):
        assert l.orc_f16_bits_to_f32(l.orc_f32_to_f16_bits(v)) == np.float32(v)
    # truncation, not rounding (dequant.rs:741): 1 + 2^-11 + 2^-12 keeps only 10 fraction bits
    assert l.orc_f32_to_f16_bits(1.0 + 2 ** -11 + 2 ** -12) == 0x3C00
    # subnormals are kept (dequant.rs:755-783)
    assert l.orc_f32_to_f16_bits(3e-5) != 0
    assert l.orc_f32_to_f16_bits(1e-9) == 0
    assert l.orc_f32_to_f16_bits(1e6) == 0x7C00


def test_dequantize_q8_0_known_block(orc):
    blk = bytearray(int(orc.lib().orc_f32_to_f16_bits(2.0)).to_bytes(2, "little"))
    blk += bytes(range(32))
    v = orc.dequantize(np.frombuffer(bytes(blk), np.uint8), 32, Q8_0)
    np.testing.assert_allclose(v, 2.0 * np.arange(32), atol=1e-2)


def test_dequantize_q8_0_negative_values(orc):
    blk = bytearray(int(orc.lib().orc_f32_to_f16_bits(1.0)).to_bytes(2, "little"))
    blk += bytes((256 - i) & 0xFF for i in range(1, 33))
    v = orc.dequantize(np.frombuffer(bytes(blk), np.uint8), 32, Q8_0)
    np.testing.assert_allclose(v, -np.arange(1, 33), atol=1e-2)


def test_dequantize_q4_0_known_block(orc):
    blk = bytearray(int(orc.lib().orc_f32_to_f16_bits(0.5)).to_bytes(2, "little"))
    blk += bytes(i | ((15 - i) << 4) for i in range(16))
    v = orc.dequantize(np.frombuffer(bytes(blk), np.uint8), 32, Q4_0)
    np.testing.assert_allclose(v[:16], 0.5 * (np.arange(16) - 8.0), atol=1e-2)
    np.testing.assert_allclose(v[16:], 0.5 * ((15 - np.arange(16)) - 8.0), atol=1e-2)


def test_quantize_roundtrip_error_bounds(orc):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal(32 * 64) * 0.02).astype(np.float32)
    for quant, steps in ((Q8_0, 127.0), (Q4_0, 7.0)):
        d = orc.dequantize(orc.quantize(w, quant), w.size, quant)
        amax = np.abs(w.reshape(-1, 32)).max(axis=1, keepdims=True)
        # half a quantisation step plus the f16 truncation of the scale (<= 2^-10 relative, times |q|)
        assert np.all(np.abs(d.reshape(-1, 32) - w.reshape(-1, 32)) <= amax / steps * (0.5 + (steps + 1) * 2 ** -10) + 1e-9)
    z = np.zeros(32, np.float32)
    assert np.all(orc.dequantize(orc.quantize(z, Q4_0), 32, Q4_0) == 0)
    assert np.all(orc.dequantize(orc.quantize(z, Q8_0), 32, Q8_0) == 0)


# ---- router: metal/tests/moe.rs:2114-2223, 2467-2703 -----------------------
def test_router_correct_topk_analytic(orc):
    H, E, K = 4, 4, 2
    x = np.array([1, 0, 0, 0], np.float32)
    gate = np.zeros((E, H), np.float32)
    gate[:, 0] = [1.0, 3.0, 2.0, 0.5]
    ids, w, _ = orc.router_softmax(x, gate, H, E, K)
    assert list(ids) == [1, 2]
    assert abs(w.sum() - 1) < 1e-5 and w[0] > w[1]
    assert abs(w[0] - math.e / (math.e + 1)) < 1e-4 and abs(w[1] - 1 / (math.e + 1)) < 1e-4


def test_router_uniform_logits_tie_breaks_to_lower_index(orc):
    H, E, K = 64, 8, 2
    x = np.ones(H, np.float32)
    gate = np.full((E, H), 0.25, np.float32)
    ids, w, _ = orc.router_softmax(x, gate, H, E, K)
    assert list(ids) == [0, 1]
    assert abs(w[0] - 0.5) < 1e-5 and abs(w[1] - 0.5) < 1e-5


def test_router_epsilon_bias_routes_to_expert_5(orc):
    H, E, K = 64, 8, 2
    x = np.ones(H, np.float32)
    gate = np.full((E, H), 0.25, np.float32)
    gate[5] += 1e-3
    ids, _, _ = orc.router_softmax(x, gate, H, E, K)
    assert ids[0] == 5


def test_router_ramp_rows_pick_highest(orc):
    H, E, K = 256, 8, 2
    x = np.ones(H, np.float32)
    gate = np.stack([np.full(H, (e + 1) / H, np.float32) for e in range(E)])
    ids, _, logits = orc.router_softmax(x, gate, H, E, K)
    np.testing.assert_allclose(logits, np.arange(1, 9), rtol=1e-5)
    assert list(ids) == [7, 6]


def test_router_one_hot_rows_follow_hot_dim(orc):
    H, E, K = 32, 8, 1
    gate = np.zeros((E, H), np.float32)
    for e in range(E):
        gate[e, e] = 1.0
    for hot in range(E):
        x = np.zeros(H, np.float32)
        x[hot] = 5.0
        ids, w, _ = orc.router_softmax(x, gate, H, E, K)
        assert ids[0] == hot and abs(w[0] - 1.0) < 1e-6


# ---- cuda/moe.rs:6551-6588 ---------------------------------------------------
def test_routing_softmax_properties_lcg(orc):
    H, E, K = 64, 16, 4
    nxt = lcg(0xDEADBEEF)
    for _ in range(100):
        x = np.array([nxt() for _ in range(H)], np.float32)
        w = np.array([nxt() for _ in range(E * H)], np.float32)
        ids, wt, _ = orc.router_softmax(x, w, H, E, K)
        assert len(set(ids.tolist())) == K
        assert all(0 <= i < E for i in ids)
        assert abs(float(wt.sum()) - 1.0) < 1e-5
        assert np.all(wt >= 0)
        assert np.all(np.diff(wt) <= 0)  # selection order = descending weight


# ---- cuda/moe.rs:6593-6681 ---------------------------------------------------
def test_expert_accum_closed_form_lcg(orc):
    H, K = 32, 4
    nxt = lcg(0xCAFEBABE)
    for _ in range(50):
        residual = np.array([nxt() for _ in range(H)], np.float32)
        outs = np.array([nxt() for _ in range(K * H)], np.float32)
        raw = np.array([abs(nxt()) + np.float32(1e-3) for _ in range(K)], np.float32)
        wts = (raw / raw.sum(dtype=np.float32)).astype(np.float32)
        got = orc.accum_option_a(residual, outs, wts, H, K)
        exp0 = residual[0] + sum(float(wts[k]) * float(outs[k * H]) for k in range(K))
        assert abs(got[0] - exp0) < 1e-5


def test_dense_vs_sparse_accum_equivalence(orc):
    H, E, K = 32, 8, 3
    nxt = lcg(0xFACEFEED)
    ids = np.array([2, 5, 7], np.uint32)
    raw = np.array([abs(nxt()) + np.float32(1e-3) for _ in range(K)], np.float32)
    wts = (raw / raw.sum(dtype=np.float32)).astype(np.float32)
    residual = np.array([nxt() for _ in range(H)], np.float32)
    dense = np.array([nxt() for _ in range(K * H)], np.float32)
    sparse = np.zeros(E * H, np.float32)
    for k in range(K):
        sparse[ids[k] * H:(ids[k] + 1) * H] = dense[k * H:(k + 1) * H]
    a = orc.accum_option_a(residual, dense, wts, H, K)
    b = orc.accum_batched_b(residual, sparse, wts, ids, H, K)
    assert np.array_equal(a, b)


# ---- metal/tests/moe.rs:10-178 (accum KATs) ------------------------------------
def test_accum_kat_sparse_slots(orc):
    E, H = 8, 256
    outs = np.concatenate([np.full(H, e + 1, np.float32) for e in range(E)])
    got = orc.accum_batched_b(np.zeros(H, np.float32), outs, np.array([0.7, 0.3], np.float32),
                              np.array([2, 5], np.uint32), H, 2)
    np.testing.assert_allclose(got, 0.7 * 3 + 0.3 * 6, atol=1e-4)
    got = orc.accum_batched_b(np.full(H, 10, np.float32), outs, np.array([0.4, 0.6], np.float32),
                              np.array([0, 7], np.uint32), H, 2)
    np.testing.assert_allclose(got, 10 + 0.4 * 1 + 0.6 * 8, atol=1e-4)


# ---- metal/tests/moe.rs:288-364 (sort KAT) ------------------------------------
def test_counting_sort_kat(orc):
    ids = np.array([[3, 1], [1, 5], [3, 0], [1, 3]], np.uint32)
    col_expert, col_src_tok, dst_to_col, bounds = orc.counting_sort(ids, 6)
    assert bounds.tolist() == [0, 1, 4, 4, 7, 7, 8]
    for e in range(6):
        for c in range(bounds[e], bounds[e + 1]):
            assert col_expert[c] == e
    # stable: tokens ascending within an expert, and dst_to_col inverts the placement
    assert col_src_tok.tolist() == [2, 0, 1, 3, 0, 2, 3, 1]
    flat = ids.reshape(-1)
    for p, c in enumerate(dst_to_col):
        assert col_expert[c] == flat[p] and col_src_tok[c] == p // 2


# ---- metal/tests/moe.rs:3182-3447 (gate/up and down+accum constant KATs) ------
def _const_matrix(orc, rows, cols, val, quant=Q8_0):
    return orc.quantize(np.full(rows * cols, val, np.float32), quant)


def test_gate_up_swiglu_constant_kat(orc):
    H = I = 64
    x = np.full(H, 0.1, np.float32)
    for gv, uv in ((0.5, 0.5), (1.0, 0.5), (0.5, 1.0), (2.0, 1.0)):
        g = orc.matvec(_const_matrix(orc, I, H, gv), x, I, H, Q8_0)
        u = orc.matvec(_const_matrix(orc, I, H, uv), x, I, H, Q8_0)
        s = orc.swiglu(g, u)
        gd, ud = gv * 0.1 * H, uv * 0.1 * H
        expected = gd / (1 + math.exp(-gd)) * ud
        assert np.all(np.abs(s - expected) / expected < 0.05)


def test_down_accum_constant_kat(orc):
    H, I = 32, 64
    down = _const_matrix(orc, H, I, 1.0)
    d0 = orc.matvec(down, np.full(I, 2.0, np.float32), H, I, Q8_0)
    d1 = orc.matvec(down, np.full(I, 4.0, np.float32), H, I, Q8_0)
    out = orc.accum_option_a(np.full(H, 10.0, np.float32), np.concatenate([d0, d1]),
                             np.array([0.7, 0.3], np.float32), H, 2)
    assert np.all(np.abs(out - 176.4) / 176.4 < 0.05)


# ---- cuda/moe.rs:6742-6819: fused norm + router == two steps -------------------
def test_fused_norm_router_equals_two_step(orc):
    H, E, K = 64, 16, 4
    nxt = lcg(0xFEEDBEEF)
    x = np.array([nxt() for _ in range(H)], np.float32)
    gamma = np.array([nxt() + np.float32(1.0) for _ in range(H)], np.float32)
    w = np.array([nxt() for _ in range(E * H)], np.float32)
    normed = orc.rmsnorm(x, gamma, 1e-6)
    ms = np.float32(0)
    for v in x:
        ms = np.float32(ms + v * v)
    scale = np.float32(1.0) / np.sqrt(np.float32(ms / np.float32(H) + np.float32(1e-6)))
    np.testing.assert_array_equal(normed, (x * scale * gamma).astype(np.float32))
    ids_a, w_a, _ = orc.router_softmax(normed, w, H, E, K)
    ids_b, w_b = orc.topk_from_logits(orc.router_logits(normed, w, H, E), K)
    assert np.array_equal(ids_a, ids_b) and np.array_equal(w_a, w_b)


# ---- whole layer == composition (metal/tests/moe.rs:884-909) -------------------
@pytest.mark.parametrize("quant", [Q8_0, Q4_0, BF16])
def test_layer_matches_manual_composition(orc, quant):
    from lumen_b200.synth import LayerLayout, make_layer_blob_numpy
    H, I, E, K, T = 64, 96, 8, 3, 5
    lay = LayerLayout(H, I, E, quant)
    blob = make_layer_blob_numpy(lay, 7, orc.quantize)
    meta = lay.meta()
    rng = np.random.default_rng(1)
    x = rng.standard_normal((T, H)).astype(np.float32)
    out, ids, wts = orc.moe_layer(blob, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs, quant,
                                  H, I, E, K, x, x, threads=2)
    router = blob[:lay.router_bytes].view(np.float32).reshape(E, H)
    for t in range(T):
        i2, w2, _ = orc.router_softmax(x[t], router, H, E, K)
        assert np.array_equal(i2, ids[t]) and np.array_equal(w2, wts[t])
        douts = []
        for k in range(K):
            e = int(ids[t, k])
            g = orc.matvec(blob[int(meta.expert_gate_offs[e]):], x[t], I, H, quant)
            u = orc.matvec(blob[int(meta.expert_up_offs[e]):], x[t], I, H, quant)
            s = orc.swiglu(g, u)
            douts.append(orc.matvec(blob[int(meta.expert_down_offs[e]):], s, H, I, quant))
        exp = orc.accum_option_a(x[t], np.concatenate(douts), wts[t], H, K)
        assert np.array_equal(exp, out[t])
        # and against plain dequantised f32 math
        wd = lambda off, r, c: orc.dequantize(blob[int(off):], r * c, quant).reshape(r, c).astype(np.float64)
        acc = x[t].astype(np.float64)
        for k in range(K):
            e = int(ids[t, k])
            gg = wd(meta.expert_gate_offs[e], I, H) @ x[t]
            uu = wd(meta.expert_up_offs[e], I, H) @ x[t]
            acc = acc + float(wts[t, k]) * (wd(meta.expert_down_offs[e], H, I) @ (gg / (1 + np.exp(-gg)) * uu))
        assert np.linalg.norm(acc - out[t]) / np.linalg.norm(acc) < 1e-5


def test_gating_modes_of_the_shared_expert(orc):
    """gating 2 = sigmoid(logit) as the weight, no renormalisation; 3 = unit weight
    (cuda/moe.rs:5455-5485; cuda/shaders/moe_shared_accum.cu:1-12)."""
    lg = np.array([[0.75], [-3.0], [0.0]], np.float32)
    ids, w = orc.topk_from_logits(lg, 1, gating=2)
    assert (ids == 0).all()
    want = (np.float32(1.0) / (np.float32(1.0) + np.exp(-lg[:, 0]).astype(np.float32))).astype(np.float32)
    np.testing.assert_allclose(w[:, 0], want, rtol=1e-6)
    assert w[2, 0] == np.float32(0.5)
    ids, w = orc.topk_from_logits(lg, 1, gating=3)
    assert (ids == 0).all() and (w == 1.0).all()
    # with several experts mode 2 keeps the raw sigmoid values of the selected ones
    lg2 = np.array([[2.0, -1.0, 0.5, 0.0]], np.float32)
    ids, w = orc.topk_from_logits(lg2, 2, gating=2)
    assert ids.tolist() == [[0, 2]]
    np.testing.assert_allclose(w[0], 1.0 / (1.0 + np.exp(-lg2[0, [0, 2]].astype(np.float64))), rtol=1e-6)
