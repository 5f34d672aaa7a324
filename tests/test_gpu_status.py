"""Error path of the operator, through the C ABI: a kernel that gives up must be visible to
the host without a debug readback (the reference returns Result<(), RuntimeError> from every
launch, error.rs:6-31, cuda/moe.rs:1497-1502), and the context must be usable again after a
reset. The waits are made to run out from the host side: the kernel is told to expect one
arrival (or one byte) more than can come, with the limit shortened to 2 ms. Nothing here
faults, traps or hangs the GPU."""
import numpy as np
import pytest
import torch

from lumen_b200 import _lib, moe, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def _ctx(H, I, E, K, max_tokens, flags=0, device=0):
    lay = synth.LayerLayout(H, I, E, 1)
    blob = synth.make_layer_blob(lay, 0, device=f"cuda:{device}")
    sc = moe.allocate_moe_scratch(H, I, E, K, max_tokens, device=device, flags=flags)
    return lay, blob, sc, sc.prepare_layer(blob, lay.meta())


def test_decode_grid_barrier_that_runs_out_is_reported_and_recoverable(cuda_lib):
    H, I, E, K, T = 512, 256, 32, 4, 2
    _, blob, sc, layer = _ctx(H, I, E, K, 16, flags=_lib.FLAG_SHORT_WAITS)
    x = torch.randn((T, H), generator=torch.Generator("cuda").manual_seed(3), device="cuda")
    good = sc.decode(layer, x, x.clone()).clone()
    torch.cuda.synchronize()
    assert sc.poll_status() == _lib.OK
    sc.debug_expire_next_wait(0)
    sc.decode(layer, x, x.clone())           # every CTA's wait at the second grid barrier runs out
    torch.cuda.synchronize()
    assert sc.poll_status() == _lib.TIMEOUT  # no readback needed: the kernel told the host
    with pytest.raises(moe.LumenMoeError) as ei:
        sc.decode(layer, x, x.clone())       # entry points fail instead of launching on a failed context
    assert ei.value.code == _lib.TIMEOUT
    with pytest.raises(moe.LumenMoeError) as ei:
        sc.get_routing(T)                    # reports it once and resets the context
    assert ei.value.code == _lib.TIMEOUT
    assert sc.poll_status() == _lib.OK
    again = sc.decode(layer, x, x.clone())
    # bit-identical to a context that never failed
    _, _, sc2, layer2 = _ctx(H, I, E, K, 16)
    fresh = sc2.decode(layer2, x, x.clone())
    torch.cuda.synchronize()
    assert torch.equal(again, good) and torch.equal(again, fresh)


def test_grouped_gemm_stage_barrier_that_runs_out_is_reported_and_recoverable(cuda_lib):
    H, I, E, K, T = 512, 256, 16, 4, 200
    _, blob, sc, layer = _ctx(H, I, E, K, T, flags=_lib.FLAG_SHORT_WAITS)
    g = torch.Generator("cuda").manual_seed(4)
    x = torch.randn((T, H), generator=g, device="cuda").to(torch.bfloat16)
    res = torch.randn((T, H), generator=g, device="cuda")
    good = sc.prefill(layer, x, res).clone()
    torch.cuda.synchronize()
    sc.debug_expire_next_wait(1)
    sc.prefill(layer, x, res)                # the first stage of the gate/up GEMM never completes
    torch.cuda.synchronize()
    assert sc.poll_status() == _lib.TIMEOUT
    with pytest.raises(moe.LumenMoeError) as ei:
        sc.prefill(layer, x, res)
    assert ei.value.code == _lib.TIMEOUT
    sc.clear_status()
    assert sc.poll_status() == _lib.OK
    again = sc.prefill(layer, x, res)
    torch.cuda.synchronize()
    assert torch.equal(again, good)


def test_expert_id_out_of_range_is_an_error_code_not_a_fault(cuda_lib):
    # caller-supplied routing (what an expert-parallel rank receives over the wire): an id >= E must
    # never index a table; the pair is dropped (expert 0, weight 0) and the context reports INVALID_ARG
    H, I, E, K, T = 256, 128, 8, 2, 50
    _, blob, sc, layer = _ctx(H, I, E, K, T)
    g = torch.Generator("cuda").manual_seed(5)
    x = torch.randn((T, H), generator=g, device="cuda")
    res = torch.randn((T, H), generator=g, device="cuda")
    ids = torch.randint(0, E, (T, K), generator=g, device="cuda", dtype=torch.int32)
    w = torch.rand((T, K), generator=g, device="cuda")
    ok = sc.prefill_routed(layer, x, ids, w, res).clone()
    torch.cuda.synchronize()
    assert sc.poll_status() == _lib.OK
    bad = ids.clone()
    bad[7, 1] = E + 3
    bad[20, 0] = -1                      # 0xffffffff as u32
    out = sc.prefill_routed(layer, x, bad, w, res)
    torch.cuda.synchronize()
    assert sc.poll_status() == _lib.INVALID_ARG
    # rows whose ids were valid are unaffected; the dropped pairs contribute nothing
    w0 = w.clone()
    w0[7, 1] = 0.0
    w0[20, 0] = 0.0
    fixed = ids.clone()
    fixed[7, 1] = 0
    fixed[20, 0] = 0
    sc.clear_status()
    ref = sc.prefill_routed(layer, x, fixed, w0, res)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    assert not torch.equal(out, ok)


def test_ids_in_the_reference_stride_e_layout(cuda_lib):
    E, K, T = 64, 4, 9
    sc = moe.allocate_moe_scratch(256, 128, E, K, 16)
    lg = synth.uniform_logits(T, E, 11, tau=1.0)
    ids, _ = sc.topk_from_logits(lg)
    wide = sc.get_routing_ids_stride_e(T)
    o_ids, _ = oracle.topk_from_logits(lg.cpu().numpy(), K, 0)
    assert wide.shape == (T, E)
    assert np.array_equal(wide[:, :K], o_ids) and not wide[:, K:].any()
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), wide[:, :K])
    # the reference's host counting sort walks this buffer with stride E (cuda/moe.rs:2116-2121)
    r = sc.get_routing(T)
    _, cst, d2c, bounds = oracle.counting_sort(wide, E, K=K)
    assert np.array_equal(r["dst_to_col"], d2c) and np.array_equal(r["col_src_tok"], cst)
    assert np.array_equal(r["expert_bounds"], bounds)


def test_unknown_config_flags_are_rejected(cuda_lib):
    with pytest.raises(moe.LumenMoeError):
        moe.allocate_moe_scratch(256, 128, 8, 2, 16, flags=0x10)


def test_contexts_on_two_devices_in_one_process(cuda_lib):
    # the shared-memory opt-in of a kernel is per device: a second GPU must get its own
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    H, I, E, K = 512, 256, 16, 4
    outs = []
    for dev in (0, 1):
        torch.cuda.set_device(dev)
        _, blob, sc, layer = _ctx(H, I, E, K, 300, device=dev)
        g = torch.Generator(f"cuda:{dev}").manual_seed(6)
        x = torch.randn((300, H), generator=g, device=f"cuda:{dev}")
        res = torch.zeros((300, H), device=f"cuda:{dev}")
        p = sc.prefill(layer, x, res)
        d16 = sc.decode(layer, x[:16].contiguous(), res[:16].contiguous())
        d2 = sc.decode(layer, x[:2].contiguous(), res[:2].contiguous())
        torch.cuda.synchronize()
        outs.append((p.cpu(), d16.cpu(), d2.cpu()))
    torch.cuda.set_device(0)
    for a, b in zip(*outs):
        assert torch.equal(a, b)
