"""lumen_moe_route_small_static, the entry point for hosts that cannot allocate
device memory (all of it belongs to their own pool, or their decode loop must
not enter the driver allocator): it has to give exactly what the context-based
lumen_moe_topk_from_logits gives -- ids, weights and sort tables, bit for bit, which
are also the CPU reference's (cpu_router_softmax + the host counting sort) --
and keep doing so call after call, since every call reuses the same static
working array inside the library.

Collected last on purpose (file name), so that a run stopping at the first
failure has already executed every other test. Passes alone in a fresh process
and after the other tests."""
import numpy as np
import pytest
import torch

from lumen_b200 import moe, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def _reference(logits, K, gating):
    T, E = logits.shape
    sc = moe.allocate_moe_scratch(256, 128, E, K, 16, gating)
    ids, w = sc.topk_from_logits(logits)
    r = sc.get_routing(T)
    return ids.cpu().numpy(), w.cpu().numpy(), r["dst_to_col"], r["expert_bounds"]


def test_static_scratch_routing_matches_context_routing_twice(cuda_lib):
    # two calls in a row with different shapes and contents: the second one finds the
    # first one's tables in the shared array and must not be disturbed by them
    cases = [(16, 128, 8, 0, 5), (3, 64, 4, 1, 6), (16, 256, 16, 0, 7), (1, 128, 8, 0, 8)]
    for T, E, K, gating, seed in cases:
        lg = synth.uniform_logits(T, E, seed, tau=0.05)
        ids, w, d2c, bounds = moe.route_small_static(lg, K, gating, want_tables=True)
        torch.cuda.synchronize()
        r_ids, r_w, r_d2c, r_bounds = _reference(lg, K, gating)
        assert np.array_equal(ids.cpu().numpy(), r_ids)
        assert np.array_equal(w.cpu().numpy().view(np.uint32), r_w.view(np.uint32))
        assert np.array_equal(d2c.cpu().numpy(), r_d2c)
        assert np.array_equal(bounds.cpu().numpy(), r_bounds)
        # and against the CPU reference's routing and host counting sort on the same logits
        o_ids, o_w = oracle.topk_from_logits(lg.cpu().numpy(), K, gating)
        _, _, o_d2c, o_bounds = oracle.counting_sort(o_ids, E)
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), o_ids)
        assert np.array_equal(w.cpu().numpy().view(np.uint32), o_w.view(np.uint32))
        assert np.array_equal(d2c.cpu().numpy(), o_d2c)
        assert np.array_equal(bounds.cpu().numpy(), o_bounds)
    # same input twice: identical output (nothing left over changes the result)
    lg = synth.zipf_logits(16, 128, 9)
    a = moe.route_small_static(lg, 8, want_tables=True)
    b = moe.route_small_static(lg, 8, want_tables=True)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_static_scratch_rejects_sizes_beyond_its_array(cuda_lib):
    for T, E, K in ((17, 128, 8), (4, 257, 8), (4, 128, 17)):
        lg = torch.zeros((T, E), device="cuda")
        with pytest.raises(moe.LumenMoeError) as ei:
            moe.route_small_static(lg, K)
        assert "8 KiB static scratch" in str(ei.value)
