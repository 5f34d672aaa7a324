#!/usr/bin/env python
"""Benchmark of the MoE feed-forward hot path (one JSON line on stdout).

Workload at every N: the configuration the headline metric is quoted on -- one
MoE FFN layer call, Q4_0 experts, batch-1 decode (H=2048, E=128, top-8, I=768),
issued over `--layers` DISTINCT layer blobs per step so that every call streams
its 22 MB of routed expert weights from HBM (48 layers x 21 MB of active weights
is ~8x the L2). One step = one token through all the layer blobs; the metric is
layer calls x tokens per second. Batch-1 decode does not shard: with N > 1 ranks
run as independent replicas ("weak" scaling, no collective in the data path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--quant q4_0|q8_0|bf16]
    python bench.py --impl reference ...   # the CPU reference path on the host cores

The same JSON line carries sub-records for the other configurations of the metric, measured
after the headline in the same run (skip them with --no-sub):
    N = 1:  "decode"  Q4_0 at 4 and 16 tokens, Q8_0 at 1 token (us per call, fraction of the HBM peak)
            "prefill" one 4096-token call, Zipf(1.1) expert loads, Q4_0 / Q8_0 / BF16 experts
                      (ms, tokens/s, TFLOP/s against the measured bf16 peaks, realised expert loads)
            "stack"   the 48-layer stack (RMSNorm + residual, identity mixers): batch-1 decode and an
                      8192-token prefill
    N > 1:  "ep_prefill"    expert-parallel prefill (lumen_moe_prefill_ep) at 16384 and 256 tokens in
                            total, uniform and Zipf(1.1) routing: ms per call, the same call on ONE
                            GPU timed on rank 0 in the same process, speed-up, per-phase ms, and every
                            rank's rows against the one-GPU output (rel-L2, ids compared exactly)
            "stack_prefill" the 48-layer stack at 8192 tokens the same way
each with the CPU reference path timed on a stated token subset (all host threads and one).

Secondary workloads (their own JSON line, not the headline):
    --workload prefill --tokens T [--routing zipf|uniform|router]     one prefill call, tensor roofline
    --workload ep_prefill --tokens T [--ep-chunks C]   (torchrun)     NCCL all-to-all form of expert parallelism
    --workload stack_prefill --tokens T --layers L     (torchrun)     the stack of L layers, NCCL form
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

H, I, E, K = 2048, 768, 128, 8
QUANTS = {"q8_0": 0, "q4_0": 1, "bf16": 2}
BLK = {0: 34, 1: 18, 2: 64}


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# capture summarised under profiles/ (kernel, quant, tokens) -> bytes
NCU_DRAM_BYTES_PER_LAUNCH = {("decode_fused_kernel", "q4_0", 1): 22_372_000}


# arithmetic of the decode path per weight format (f32 activations in and out in all cases)
DECODE_DTYPE = {"q4_0": "u8*s8->s32 (gate/up) and f16*f16->f32 (down) tensor-core products, f32 scales and sums",
                "q8_0": "f16*f16->f32 tensor-core products (exact-integer weights, hi+lo activations), f32 scales and sums",
                "bf16": "bf16*bf16->f32 tensor-core products (hi+lo activations), f32 sums"}


def algorithmic_bytes(T: int, U: int, quant: int) -> int:
    """Compulsory traffic of one layer call: router weight, the three matrices of
    every distinct expert hit, activations in / residual in / output out."""
    return E * H * 4 + U * 3 * (I * H // 32) * BLK[quant] + 3 * T * H * 4


def gate_up_bytes(T: int, U: int, quant: int) -> int:
    """Compulsory traffic of the gate/up + SwiGLU kernel alone."""
    return U * 2 * (I * H // 32) * BLK[quant] + T * H * 4 + T * K * I * 4


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region (read-only)."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons}


def cpu_reference_leg(quant: int, T: int, budget_s: float, blob_np=None, threads=None, max_calls: int = 2000):
    """Times the CPU reference path (oracle restatement) on a bounded sample of the same
    workload: single layer calls of T tokens on one layer blob (340 MB for Q4_0). Every call
    takes different tokens (64 seeded batches in rotation), so successive calls hit different
    experts and the weights come from DRAM, not from the host's last-level cache."""
    import numpy as np
    from oracle import oracle
    from lumen_b200.synth import LayerLayout, make_layer_blob_numpy
    lay = LayerLayout(H, I, E, quant)
    if blob_np is None:
        # 128 experts of seeded N(0,0.02) weights quantised by the oracle's quantiser
        blob_np = make_layer_blob_numpy(lay, 0, oracle.quantize)
    meta = lay.meta()
    threads = threads or oracle.hardware_threads()
    rng = np.random.default_rng(1)
    xs = rng.standard_normal((64, T, H)).astype(np.float32)
    calls, t0 = 0, time.perf_counter()
    while True:
        x = xs[calls % 64]
        oracle.moe_layer(blob_np, 0, meta.expert_gate_offs, meta.expert_up_offs, meta.expert_down_offs, quant, H, I, E,
                         K, x, x, threads=threads)
        calls += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or calls >= max_calls:
            break
    return {"value": calls * T / dt, "unit": "layer_tokens/s", "cores": threads, "kind": "port",
            "sample": f"{calls} single-layer calls of {T} token(s) (different tokens every call) on one layer blob, {dt:.1f} s"}


def cpu_pair(quant: int, T: int, blob_np, budget_s: float = 2.5):
    """all-threads and single-thread CPU figures for a sub-record, on a bounded token subset."""
    a = cpu_reference_leg(quant, T, budget_s, blob_np)
    one = cpu_reference_leg(quant, min(T, 4), budget_s * 0.6, blob_np, threads=1)
    a["single_thread"] = {"value": one["value"], "unit": one["unit"], "sample": one["sample"]}
    return a


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    quant = QUANTS[args.quant]
    from oracle import oracle
    from lumen_b200.synth import LayerLayout, make_layer_blob_numpy
    blob = make_layer_blob_numpy(LayerLayout(H, I, E, quant), 0, oracle.quantize)
    per_step = max(0.5, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_reference_leg(quant, args.tokens, 0.2, blob)
    t0 = time.perf_counter()
    vals = [cpu_reference_leg(quant, args.tokens, per_step, blob) for _ in range(args.steps)]
    dt = time.perf_counter() - t0
    v = statistics.mean(r["value"] for r in vals)
    base = vals[-1]
    base["value"] = v
    base["sample"] = f"{args.steps} steps, each " + base["sample"]
    line = {"impl": "reference", "metric": "moe_layer_decode_tokens_per_s", "value": v, "unit": "layer_tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000 * dt / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args), "cpu_baseline": base,
            "e2e": {"value": v, "unit": "layer_tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args):
    return {"workload": f"moe_ffn_decode_{args.quant}_T{args.tokens}", "hidden": H, "experts": E, "top_k": K,
            "inter": I, "tokens_per_call": args.tokens, "distinct_layer_blobs": args.layers,
            "l2_policy": "inputs larger than L2: every call reads a different layer's experts",
            "parallelism": "replicas only (batch-1 decode does not shard)"}



# ---------------------------------------------------------------------------------------------
# sub-records: the other configurations of the metric, measured after the headline
# ---------------------------------------------------------------------------------------------
def tensor_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    d = json.loads(p.read_text()) if p.exists() else {}
    return (float(d.get("bf16_tflops", 1590.0)), float(d.get("bf16_tflops_sustained", 1400.0)),
            "measured (MEASURED_PEAKS.json)" if d else "fallback (no MEASURED_PEAKS.json)")


def event_ms(torch, fn, n):
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(n):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / n


def sub_decode(torch, np, moe, synth, dev, quant_name, T, n_layers, layers=None, scratch=None, steps=10):
    """One decode sub-record: T tokens per call, the calls rotating over n_layers distinct layer
    blobs (working set larger than L2), launches replayed from a CUDA graph."""
    quant = QUANTS[quant_name]
    lay = synth.LayerLayout(H, I, E, quant)
    own = layers is None
    if own:
        scratch = moe.allocate_moe_scratch(H, I, E, K, 16, device=dev.index)
        layers, blob0 = [], None
        for l in range(n_layers):
            blob = synth.make_layer_blob(lay, l, device=dev)
            layers.append(scratch.prepare_layer(blob, lay.meta()))
    blob0 = layers[0].blob.cpu().numpy()
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    x = torch.randn((T, H), generator=g, device=dev)
    outs = torch.empty((len(layers), T, H), device=dev)

    def step():
        for l, layer in enumerate(layers):
            scratch.decode(layer, x, x, outs[l])
    for _ in range(3):
        step()
    U = []
    for l, layer in enumerate(layers):
        scratch.decode(layer, x, x, outs[l])
        U.append(len(np.unique(scratch.get_routing(T)["ids"])))
    moe.launch_count(reset=True)
    step()
    launches = moe.launch_count(reset=True)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(3):
        graph.replay()
    ms = event_ms(torch, graph.replay, steps) / len(layers)
    peak, _ = peaks()
    nbytes = sum(algorithmic_bytes(T, u, quant) for u in U) / len(U)
    gbs = nbytes / (ms / 1e3) / 1e9
    rec = {"workload": f"moe_ffn_decode_{quant_name}_T{T}", "us_per_call": ms * 1e3, "layer_tokens_per_s": T / (ms / 1e3),
           "distinct_layer_blobs": len(layers), "launches_per_call": launches / len(layers),
           "distinct_experts_per_call": sum(U) / len(U), "algorithmic_bytes_per_call": nbytes,
           "achieved_gbs": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_8tbs": gbs / 8000.0,
           "cpu_baseline": cpu_pair(quant, T, blob0, 2.0)}
    if own:
        for layer in layers:
            layer.close()
        scratch.close()
    return rec


def sub_prefill(torch, np, moe, synth, dev, quant_name, T, routing="zipf", steps=10, n_layers=2, flags=0):
    """One prefill call of T tokens (bf16 activations), Zipf(1.1)-skewed expert loads through the
    logits entry, rotating over n_layers layer blobs."""
    quant = QUANTS[quant_name]
    lay = synth.LayerLayout(H, I, E, quant)
    sc = moe.allocate_moe_scratch(H, I, E, K, T, device=dev.index, flags=flags)
    layers = [sc.prepare_layer(synth.make_layer_blob(lay, l, device=dev), lay.meta()) for l in range(n_layers)]
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    x = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)
    res = torch.zeros((T, H), device=dev)
    out = torch.empty_like(res)
    if routing != "router":
        sc.set_logits_override(synth.zipf_logits(T, E, 2, device=dev) if routing == "zipf" else
                               synth.uniform_logits(T, E, 2, device=dev))

    def step():
        for layer in layers:
            sc.prefill(layer, x, res, out)
    for _ in range(3):
        step()
    r = sc.get_routing(T)  # raises if a device-side wait expired
    loads = np.diff(r["expert_bounds"])
    moe.launch_count(reset=True)
    step()
    launches = moe.launch_count(reset=True) / n_layers
    ms = event_ms(torch, step, steps) / n_layers
    flops = T * (2 * E * H + K * 6 * I * H)
    burst, sustained, src = tensor_peaks()
    tf = flops / (ms / 1e3) / 1e12
    blob0 = layers[0].blob.cpu().numpy()
    cpu = cpu_pair(quant, 64, blob0, 3.0)
    cpu["sample"] = "token subset: " + cpu["sample"]
    cpu["extrapolated_ms_for_this_call"] = 1e3 * T / cpu["value"]
    weights_form = ("plain f16 matrices fed by TMA" if (quant == 2 or flags & 0x8) else
                    "quantised planes dequantised in shared memory")
    rec = {"workload": f"moe_ffn_prefill_{quant_name}_T{T}_{routing}" + ("_f16weights" if flags & 0x8 else ""),
           "weight_operand": weights_form, "layer_device_bytes": layers[0].device_bytes,
           "ms_per_call": ms, "tokens_per_s": T / (ms / 1e3),
           "tflops": tf, "flops_per_call": flops, "frac_of_burst_peak": tf / burst, "frac_of_sustained_peak": tf / sustained,
           "peak_source": src, "launches_per_call": launches,
           "expert_load": {"max": int(loads.max()), "median": float(np.median(loads)), "min": int(loads.min())},
           "activations": "bf16", "operands": "f16 x f16 -> f32 (tcgen05, accumulators in TMEM)", "cpu_baseline": cpu}
    for layer in layers:
        layer.close()
    sc.close()
    return rec


def sub_stack(torch, np, moe, synth, dev, layers, scratch, steps=3):
    """The 48-layer stack (RMSNorm eps 1e-6 + residual, identity mixers) on one GPU: batch-1
    decode (one token through the stack per step) and an 8192-token prefill."""
    L = len(layers)
    gammas = [torch.ones(H, device=dev) for _ in range(L)]
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    x0 = torch.randn((1, H), generator=g, device=dev)
    xw = x0.clone()

    def dstep():
        xw.copy_(x0)
        scratch.stack_decode(layers, gammas, xw, 1e-6)
    for _ in range(3):
        dstep()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        dstep()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        dstep()
    for _ in range(3):
        graph.replay()
    ms_d = event_ms(torch, graph.replay, 20)
    peak, _ = peaks()
    nbytes = L * (algorithmic_bytes(1, K, 1) + H * 4)
    rec = {"decode": {"workload": f"moe_stack_decode_q4_0_L{L}_T1", "ms_per_token": ms_d, "tokens_per_s": 1e3 / ms_d,
                      "algorithmic_bytes_per_token": nbytes, "achieved_gbs": nbytes / (ms_d / 1e3) / 1e9,
                      "frac_of_measured_peak": nbytes / (ms_d / 1e3) / 1e9 / peak}}
    T = 8192
    sc = moe.allocate_moe_scratch(H, I, E, K, T, device=dev.index)
    xp = torch.randn((T, H), generator=g, device=dev)
    normed = torch.empty_like(xp)
    work = xp.clone()

    def pstep():
        work.copy_(xp)
        sc.stack_prefill(layers, gammas, work, 1e-6, normed)
    pstep()
    ms_p = event_ms(torch, pstep, steps)
    flops = L * T * (2 * E * H + K * 6 * I * H)
    burst, sustained, _ = tensor_peaks()
    tf = flops / (ms_p / 1e3) / 1e12
    rec["prefill"] = {"workload": f"moe_stack_prefill_q4_0_L{L}_T{T}_router", "ms_per_pass": ms_p, "ms_per_layer": ms_p / L,
                      "tokens_per_s": T / (ms_p / 1e3), "tflops": tf, "frac_of_sustained_peak": tf / sustained,
                      "frac_of_burst_peak": tf / burst}
    sc.close()
    return rec


def sub_ep(torch, np, dist, moe, synth, ep, dev, rank, world, layers, args):
    """Expert-parallel sub-records (N > 1): lumen_moe_prefill_ep against the same call on one
    GPU (timed on rank 0 in this process), with every rank's output rows compared with the
    one-GPU output. Strong scaling: the total work is fixed, tokens and experts are sharded."""
    lay = synth.LayerLayout(H, I, E, 1)
    meta = lay.meta()
    Tmax = 16384
    pe = ep.PushExpertParallel(H, I, E, K, Tmax // world, rank, world, dev.index)
    ep_layers = [pe.prepare_layer(l.blob, meta) for l in layers]   # identical blobs on every rank
    sc1 = moe.allocate_moe_scratch(H, I, E, K, Tmax, device=dev.index) if rank == 0 else None

    def maxr(v):
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_all(fn, n):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(n):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        dist.barrier()
        return maxr(ev0.elapsed_time(ev1) / n)

    def graphed(fn, collective=True):
        """The launches of one call replayed from a CUDA graph, as the headline does (the reference's
        backend enqueues from Rust; a Python loop would time the interpreter at 256 tokens)."""
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            fn()
        torch.cuda.synchronize()
        if collective:
            dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g.replay

    records = []
    for T, steps in ((16384, 10), (256, 20)):
        Tl = T // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        g = torch.Generator(device=dev)
        g.manual_seed(1)
        x_all = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)   # same on every rank
        res_all = torch.zeros((T, H), device=dev)
        x, res = x_all[sl].contiguous(), res_all[sl].contiguous()
        out = torch.empty_like(res)
        for routing in ("uniform", "zipf"):
            # uniform: the layer's own router (N(0, 0.02) router weights route near-uniformly), so the
            # router products are part of both timings; zipf: logits drawn so that the expert loads
            # follow Zipf(1.1), fed through the logits entry on both sides
            lg_all = synth.zipf_logits(T, E, 2, device=dev) if routing == "zipf" else None
            pe.sc.set_logits_override(lg_all[sl].contiguous() if lg_all is not None else None)
            fwd = lambda: pe.forward(ep_layers[0], x, res, out)
            for _ in range(3):
                fwd()
            ms = timed_all(graphed(fwd), steps)
            pe.sc.ep_profile(True)
            fwd()
            ph = pe.sc.ep_phase_ms()
            pe.sc.ep_profile(False)
            ph_t = torch.tensor([ph[k] for k in moe.MoeScratch.EP_PHASES], device=dev, dtype=torch.float64)
            ph_max = ph_t.clone()
            dist.all_reduce(ph_max, op=dist.ReduceOp.MAX)
            mine = pe.sc.get_routing(Tl)   # raises if this rank's context recorded a failure
            # the same call on one GPU, on rank 0, in this process
            ref = torch.empty((T, H), device=dev)
            ids_ref = torch.empty((T, K), device=dev, dtype=torch.int32)
            ms1 = 0.0
            if rank == 0:
                sc1.set_logits_override(lg_all)
                one = lambda: sc1.prefill(layers[0], x_all, res_all, ref)
                for _ in range(3):
                    one()
                ms1 = event_ms(torch, graphed(one, collective=False), steps)
                ids_ref.copy_(torch.from_numpy(sc1.get_routing(T)["ids"].astype(np.int32)))
            dist.barrier()
            dist.broadcast(ref, 0)
            dist.broadcast(ids_ref, 0)
            ms1 = maxr(ms1)
            mine_ref = ref[sl]
            rel = float((out.double() - mine_ref.double()).norm() / mine_ref.double().norm().clamp_min(1e-30))
            ids_ok = bool((torch.from_numpy(mine["ids"].astype(np.int32)).to(dev) == ids_ref[sl]).all())
            bit = bool(torch.equal(out, mine_ref))
            rel_max = maxr(rel)
            flags = torch.tensor([1.0 if ids_ok else 0.0, 1.0 if bit else 0.0], device=dev, dtype=torch.float64)
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            loads = np.diff(sc1.get_routing(T)["expert_bounds"]) if rank == 0 else None
            if rank == 0:
                records.append({
                    "workload": f"moe_ffn_ep_prefill_q4_0_T{T}_{routing}", "tokens_total": T, "tokens_per_gpu": Tl,
                    "routing": "the layer's router (near-uniform loads)" if routing == "uniform" else
                               "Zipf(1.1) loads through the logits entry",
                    "experts_per_gpu": E // world, "ms_per_call": ms, "tokens_per_s": T / (ms / 1e3),
                    "ms_per_call_1gpu": ms1, "speedup_vs_1gpu": ms1 / ms,
                    "rel_l2_vs_1gpu_max_over_ranks": rel_max, "ids_exact": bool(flags[0].item() > 0.5),
                    "bit_identical_to_1gpu": bool(flags[1].item() > 0.5),
                    "phase_ms_rank0": {k: round(ph[k], 4) for k in moe.MoeScratch.EP_PHASES},
                    "phase_ms_max_over_ranks": {k: round(float(v), 4) for k, v in zip(moe.MoeScratch.EP_PHASES, ph_max.tolist())},
                    "expert_load": {"max": int(loads.max()), "median": float(np.median(loads))},
                    "transport": "plain peer stores into CUDA-IPC windows over NVLink, release/acquire flags; "
                                 "no collective, no host synchronisation in the call",
                    "wire": "f16 rows (the rounding the one-GPU GEMM applies to its operand), f16 results"})
    # the 48-layer stack at 8192 tokens
    T, L = 8192, len(layers)
    Tl = T // world
    sl = slice(rank * Tl, (rank + 1) * Tl)
    pe.sc.set_logits_override(None)
    gammas = [torch.ones(H, device=dev) for _ in range(L)]
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    x0 = torch.randn((T, H), generator=g, device=dev)
    mine0 = x0[sl].contiguous()
    work = mine0.clone()
    normed = torch.empty_like(work)

    def sfwd():
        work.copy_(mine0)
        pe.stack_forward(ep_layers, gammas, work, 1e-6, normed)
    sfwd()
    ms = timed_all(graphed(sfwd), 3)
    ref = torch.empty((T, H), device=dev)
    ms1 = 0.0
    if rank == 0:
        sc1.set_logits_override(None)
        n1 = torch.empty_like(x0)

        def one():
            ref.copy_(x0)
            sc1.stack_prefill(layers, gammas, ref, 1e-6, n1)
        one()
        ms1 = event_ms(torch, graphed(one, collective=False), 2)
    dist.barrier()
    dist.broadcast(ref, 0)
    ms1 = maxr(ms1)
    d = (ref[sl] - mine0).double()
    rel = maxr(float((work.double() - ref[sl].double()).norm() / d.norm().clamp_min(1e-30)))
    bit = torch.tensor([1.0 if torch.equal(work, ref[sl]) else 0.0], device=dev, dtype=torch.float64)
    dist.all_reduce(bit, op=dist.ReduceOp.MIN)
    stack = None
    if rank == 0:
        flops = L * T * (2 * E * H + K * 6 * I * H)
        _, sustained, _ = tensor_peaks()
        tf = flops / (ms / 1e3) / 1e12
        stack = {"workload": f"moe_stack_prefill_q4_0_L{L}_T{T}_router", "ms_per_pass": ms, "ms_per_layer": ms / L,
                 "tokens_per_s": T / (ms / 1e3), "ms_per_pass_1gpu": ms1, "speedup_vs_1gpu": ms1 / ms,
                 "rel_l2_vs_1gpu_max_over_ranks": rel, "bit_identical_to_1gpu": bool(bit.item() > 0.5),
                 "tflops": tf, "frac_of_sustained_peak_all_gpus": tf / (sustained * world)}
    pe.sc.get_routing(Tl)
    pe.close()
    if sc1 is not None:
        sc1.close()
    return records, stack


def run_gpu(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from lumen_b200 import build, moe, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # one rank brings the library up to date (a no-op when it is newer than its sources); the
    # others must not load a file that is being rewritten
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    quant, T, L = QUANTS[args.quant], args.tokens, args.layers
    lay = synth.LayerLayout(H, I, E, quant)
    scratch = moe.allocate_moe_scratch(H, I, E, K, 16, device=local)
    layers, blob0 = [], None
    for l in range(L):
        blob = synth.make_layer_blob(lay, l, device=f"cuda:{local}")  # the same blobs on every replica
        layers.append(scratch.prepare_layer(blob, lay.meta()))
        if l == 0 and rank == 0:
            blob0 = blob.cpu().numpy()
    g = torch.Generator(device=f"cuda:{local}")
    g.manual_seed(1)
    x = torch.randn((T, H), generator=g, device=f"cuda:{local}")
    outs = torch.empty((L, T, H), device=f"cuda:{local}")
    host_x = torch.randn((T, H)).pin_memory()
    host_out = torch.empty((T, H)).pin_memory()

    def step():
        for l in range(L):
            scratch.decode(layers[l], x, x, outs[l])

    def step_e2e():
        x.copy_(host_x, non_blocking=True)
        step()
        host_out.copy_(outs[L - 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(n):
            fn()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=f"cuda:{local}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(3, args.warmup)):
        step()
    # The 3*L launches of a step are replayed from one CUDA graph (the reference's
    # backend enqueues them from Rust; a Python loop would time the interpreter).
    torch.cuda.synchronize()
    moe.launch_count(reset=True)
    step()
    launches_per_step = moe.launch_count(reset=True)  # L with the fused kernel, 3 L with the three-kernel chain
    step_eager = step
    if not args.no_graph:
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        moe.launch_count(reset=True)
        with torch.cuda.graph(graph):
            step()
        launches_per_step = moe.launch_count(reset=True)
        step = graph.replay
        for _ in range(3):
            step()
    # distinct experts per call (for the algorithmic byte count)
    U = []
    torch.cuda.synchronize()
    for l in range(L):
        scratch.decode(layers[l], x, x, outs[l])
        U.append(len(np.unique(scratch.get_routing(T)["ids"])))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(step, args.steps)
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(step_e2e, args.steps)
    units = args.steps * L * T * world
    value = units / (ms / 1e3)
    e2e = units / (ms_e2e / 1e3)

    line = None
    if rank == 0:
        peak, peak_src = peaks()
        layer_bytes = sum(algorithmic_bytes(T, u, quant) for u in U) / L
        layer_gbs = layer_bytes / ((ms / 1e3) / (args.steps * L)) / 1e9
        fused = launches_per_step == L  # one launch per layer call: the persistent fused kernel ran
        if fused:
            # the timed region IS this kernel, launch after launch: average launch duration from the same events
            k_name = "decode_fused_kernel"
            k_ms = ms / (args.steps * L)
            k_bytes = layer_bytes
            achieved = layer_gbs
            tr = scratch.debug_decode_trace(layers[L - 1]).cpu().numpy().astype(np.int64)
            t0 = tr[:, 0].min()
            med = lambda i: float(np.median((tr[:, i][tr[:, i] > 0] - t0) / 1e3))
            stamps = [med(i) for i in range(12)]
            kernel_us = {"decode_fused_kernel": k_ms * 1e3,
                         "phases_us_median_over_ctas": {
                             "wait_previous_kernel": stamps[1], "router_logits": stamps[2] - stamps[1],
                             "grid_barrier_1": stamps[3] - stamps[2], "topk_and_sort": stamps[4] - stamps[3],
                             "gate_up_swiglu": stamps[5] - stamps[4], "grid_barrier_2": stamps[6] - stamps[5],
                             "stage_swiglu": stamps[7] - stamps[6], "down": stamps[8] - stamps[7],
                             "combine": stamps[9] - stamps[8]},
                         "since_kernel_start_us_median": {"tiles_requested": stamps[10], "last_gate_up_tile_arrived": stamps[11],
                                                          "end": stamps[9]}}
        else:
            # each kernel of the chain alone, one launch per layer blob, CUDA events on the launch stream
            # (phase 1 = gate/up + SwiGLU is the dominant kernel)
            def time_phase(phase, reps=5):
                def run():
                    for l in range(L):
                        scratch.debug_decode_phase(layers[l], phase)
                run()
                torch.cuda.synchronize()
                fn = run
                if not args.no_graph:
                    gph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gph):
                        run()
                    fn = gph.replay
                    fn()
                torch.cuda.synchronize()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
                for _ in range(reps):
                    fn()
                ev1.record()
                torch.cuda.synchronize()
                return ev0.elapsed_time(ev1) / (reps * L)
            phase_ms = [time_phase(ph) for ph in (0, 1, 2)]
            k_name = "gate_up_kernel"
            k_ms = phase_ms[1]
            # routing tables in the context belong to the last layer called: same count of experts for every launch
            k_bytes = gate_up_bytes(T, U[-1], quant)
            achieved = k_bytes / (k_ms / 1e3) / 1e9
            kernel_us = {"router_small_kernel": phase_ms[0] * 1e3, "gate_up_kernel": phase_ms[1] * 1e3,
                         "down_combine_kernel": phase_ms[2] * 1e3}
        traffic = NCU_DRAM_BYTES_PER_LAUNCH.get((k_name, args.quant, T))
        cpu = cpu_reference_leg(quant, T, 12.0, blob0)
        one = cpu_reference_leg(quant, T, 3.0, blob0, threads=1)
        cpu["single_thread"] = {"value": one["value"], "unit": one["unit"], "sample": one["sample"]}
        line = {"metric": "moe_layer_decode_tokens_per_s", "value": value, "unit": "layer_tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DECODE_DTYPE[args.quant],
                "data": "synthetic", "config": workload_config(args),
                "e2e": {"value": e2e, "unit": "layer_tokens/s", "h2d_bytes_per_step": T * H * 4,
                        "d2h_bytes_per_step": T * H * 4},
                "gpu_launches": int(launches),
                "roofline": {"bound": "hbm", "kernel": k_name, "achieved": achieved, "peak": peak,
                             "unit": "GB/s", "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                             "algorithmic_bytes_per_launch": k_bytes, "us_per_launch": k_ms * 1e3},
                "kernel_us": kernel_us,
                "layer_roofline": {"algorithmic_bytes_per_call": layer_bytes, "us_per_call": ms * 1e3 / (args.steps * L),
                                   "achieved_gbs": layer_gbs, "frac_of_measured_peak": layer_gbs / peak,
                                   "frac_of_8tbs": layer_gbs / 8000.0},
                "cpu_baseline": cpu, "clocks": clocks}
    # ---- sub-records (after the headline; nothing below changes the numbers above) ----
    dev = torch.device("cuda", local)
    subs = {}
    # A sub-record must never cost the headline: if the section below is still running after ten
    # minutes (a rank that died inside a collective of the comparison code, say), rank 0 prints the
    # line it has and every rank leaves. The library's own cross-rank waits give up after 2 s each.
    watchdog = None
    if world > 1 and not args.no_sub:
        def give_up():
            if rank == 0:
                line["error"] = "sub-records abandoned after 600 s"
                print(json.dumps(line), flush=True)
            os._exit(0)
        watchdog = threading.Timer(600.0, give_up)
        watchdog.daemon = True
        watchdog.start()
    if not args.no_sub and quant == 1 and T == 1:
        try:
            if world == 1:
                subs["decode"] = [sub_decode(torch, np, moe, synth, dev, "q4_0", 4, L, layers, scratch),
                                  sub_decode(torch, np, moe, synth, dev, "q4_0", 16, L, layers, scratch),
                                  sub_decode(torch, np, moe, synth, dev, "q8_0", 1, 8)]
                subs["prefill"] = [sub_prefill(torch, np, moe, synth, dev, q, 4096) for q in ("q4_0", "q8_0", "bf16")]
                # the same call with the layer's own router instead of supplied logits (router products included)
                subs["prefill"].append(sub_prefill(torch, np, moe, synth, dev, "q4_0", 4096, routing="router"))
                # memory traded for speed: the Q4_0 layer also kept as f16 matrices (LUMEN_MOE_FLAG_PREFILL_F16_WEIGHTS)
                subs["prefill"].append(sub_prefill(torch, np, moe, synth, dev, "q4_0", 4096, flags=0x8))
                subs["stack"] = sub_stack(torch, np, moe, synth, dev, layers, scratch)
            else:
                from lumen_b200 import ep
                recs, stack = sub_ep(torch, np, dist, moe, synth, ep, dev, rank, world, layers, args)
                subs["ep_prefill"], subs["stack_prefill"] = recs, stack
        except Exception as exc:  # a failing sub-record must not cost the headline
            subs["error"] = repr(exc)
    if watchdog is not None:
        watchdog.cancel()
    if rank == 0:
        line.update(subs)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_prefill(args):
    """Secondary workload (not the headline line): one prefill call of `--tokens`
    tokens on one layer, Zipf(1.1)-skewed expert loads, bf16 activations; reports
    tokens/s and the tensor roofline of the grouped GEMMs."""
    import torch
    from lumen_b200 import build, moe, synth
    build.build()
    quant, T = QUANTS[args.quant], args.tokens
    lay = synth.LayerLayout(H, I, E, quant)
    sc = moe.allocate_moe_scratch(H, I, E, K, T, flags=0x8 if args.f16_weights else 0)
    layers = [sc.prepare_layer(synth.make_layer_blob(lay, l), lay.meta()) for l in range(min(args.layers, 4))]
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    x = torch.randn((T, H), generator=g, device="cuda").to(torch.bfloat16)
    res = torch.zeros((T, H), device="cuda")
    out = torch.empty_like(res)
    lg = synth.zipf_logits(T, E, 2) if args.routing == "zipf" else synth.uniform_logits(T, E, 2)
    if args.routing != "router":
        sc.set_logits_override(lg)

    def step():
        for l in layers:
            sc.prefill(l, x, res, out)
    for _ in range(max(3, args.warmup)):
        step()
    sc.get_routing(T)  # raises if a device-side wait expired
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / (args.steps * len(layers))
    flops = T * (2 * E * H + K * 6 * I * H)
    peaks_d = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks_d.get("bf16_tflops", 1590.0))
    tf = flops / (ms / 1e3) / 1e12
    print(json.dumps({"metric": "moe_layer_prefill_tokens_per_s", "value": T / (ms / 1e3), "unit": "tokens/s",
                      "n_gpus": 1, "steps": args.steps, "ms_per_call": ms, "dtype": "f16 operands, f32 accumulate",
                      "config": {"workload": f"moe_ffn_prefill_{args.quant}_T{T}_{args.routing}", "layers_rotated": len(layers)},
                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s",
                                   "frac": tf / peak, "flops_per_call": flops}}), flush=True)


def run_ep_prefill(args):
    """Secondary workload: expert-parallel prefill. `--tokens` tokens
    in total, sharded over the ranks; 128 experts split evenly; NCCL all-to-all dispatch
    and combine. Strong scaling: total work fixed as N grows. At N = 1 the same tokens go
    through the single-GPU prefill entry point."""
    import torch
    import torch.distributed as dist
    from lumen_b200 import build, ep, moe, synth
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    quant, T = QUANTS[args.quant], args.tokens
    Tl = T // world
    lay = synth.LayerLayout(H, I, E, quant)
    blob = synth.make_layer_blob(lay, 0, device=dev)        # identical on every rank
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    x_all = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)
    x = x_all[rank * Tl:(rank + 1) * Tl].contiguous()
    res = torch.zeros((Tl, H), device=dev)
    if world == 1:
        sc = moe.allocate_moe_scratch(H, I, E, K, T, device=local)
        layer = sc.prepare_layer(blob, lay.meta())
        fwd = lambda: sc.prefill(layer, x, res)
    else:
        route_fn, expert_fn, keep = ep.cuda_layer_fns(H, I, E, K, quant, blob, rank, world, Tl)
        epl = ep.ExpertParallelMoe(E, K, route_fn, expert_fn, combine_fn=keep["combine_fn"], route_takes_slot=True)
        fwd = (lambda: epl.forward(x, res)) if args.ep_chunks < 2 else (lambda: epl.forward_pipelined(x, res, args.ep_chunks))
    for _ in range(max(3, args.warmup)):
        out = fwd()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        out = fwd()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    phases = None
    if world > 1:
        epl.profile = True
        epl.forward(x, res)
        phases = {k: round(v, 3) for k, v in epl.phase_times_ms()}
        epl.profile = False
    checksum = float(out.float().abs().sum())
    if world > 1:
        t = torch.tensor([ms, checksum], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, checksum = float(tmax[0]), float(t[1])
    if rank == 0:
        print(json.dumps({"metric": "moe_layer_ep_prefill_tokens_per_s", "value": T / (ms / 1e3), "unit": "tokens/s",
                          "n_gpus": world, "steps": args.steps, "ms_per_call": ms, "scaling": "strong",
                          "config": {"workload": f"moe_ffn_ep_prefill_{args.quant}_T{T}", "experts_per_gpu": E // world,
                                     "tokens_per_gpu": Tl, "wire_dtype": "bf16", "collective": "nccl all_to_all_single",
                                     "pipelined_parts": args.ep_chunks if world > 1 else None},
                          "phase_ms_rank0": phases, "abs_sum_of_output": checksum}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_stack_prefill(args):
    """Secondary workload: the stack of `--layers` MoE FFN layers (RMSNorm eps 1e-6 + residual,
    identity mixers) as one prefill of `--tokens` tokens in total, real router, f32 residual
    stream. N = 1: lumen_moe_stack_prefill. N > 1: tokens sharded over the ranks, experts
    sharded E/N, per-layer NCCL dispatch/combine (strong scaling: total work fixed)."""
    import torch
    import torch.distributed as dist
    from lumen_b200 import build, ep, moe, synth
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    quant, T, L = QUANTS[args.quant], args.tokens, args.layers
    Tl = T // world
    lay = synth.LayerLayout(H, I, E, quant)
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    x_all = torch.randn((T, H), generator=g, device=dev)
    gammas = [torch.ones(H, device=dev) for _ in range(L)]
    x0 = x_all[rank * Tl:(rank + 1) * Tl].contiguous()
    blobs = (synth.make_layer_blob(lay, l, device=dev) for l in range(L))  # identical on every rank
    if world == 1:
        sc = moe.allocate_moe_scratch(H, I, E, K, T, device=local)
        layers = [sc.prepare_layer(b, lay.meta()) for b in blobs]
        normed = torch.empty_like(x0)
        fwd = lambda: sc.stack_prefill(layers, gammas, x0.clone(), 1e-6, normed)
    else:
        stack = ep.ExpertParallelStack(H, I, E, K, quant, blobs, gammas, rank, world, Tl, 1e-6, chunks=args.ep_chunks)
        fwd = lambda: stack.forward(x0)
    for _ in range(max(3, args.warmup)):
        out = fwd()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        out = fwd()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    checksum = float(out.double().abs().sum())
    if world > 1:
        t = torch.tensor([ms, checksum], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, checksum = float(tmax[0]), float(t[1])
    if rank == 0:
        flops = L * T * (2 * E * H + K * 6 * I * H)
        peaks_d = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        peak = float(peaks_d.get("bf16_tflops_sustained", peaks_d.get("bf16_tflops", 1590.0)))
        tf = flops / (ms / 1e3) / 1e12
        print(json.dumps({"metric": "moe_stack_prefill_tokens_per_s", "value": T / (ms / 1e3), "unit": "tokens/s",
                          "n_gpus": world, "steps": args.steps, "ms_per_step": ms, "ms_per_layer": ms / L,
                          "scaling": "strong", "dtype": "f16 operands, f32 accumulate and residual stream",
                          "config": {"workload": f"moe_stack_prefill_{args.quant}_L{L}_T{T}_router", "layers": L,
                                     "tokens_per_gpu": Tl, "experts_per_gpu": E // world,
                                     "wire_dtype": "f16" if world > 1 else None,
                                     "pipelined_parts": args.ep_chunks if world > 1 else None},
                          "roofline": {"bound": "tensor", "achieved": tf, "peak": peak * world, "unit": "TFLOP/s",
                                       "frac": tf / (peak * world), "flops_per_step": flops},
                          "abs_sum_of_output": checksum}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "ep_prefill", "stack_prefill"])
    ap.add_argument("--routing", default="zipf", choices=["zipf", "uniform", "router"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--quant", default="q4_0", choices=sorted(QUANTS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ep-chunks", type=int, default=1,
                    help="expert-parallel workloads: parts whose dispatch / expert products / combine overlap (1 = off)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--f16-weights", action="store_true",
                    help="--workload prefill: keep the layers as plain f16 matrices too (LUMEN_MOE_FLAG_PREFILL_F16_WEIGHTS)")
    ap.add_argument("--no-sub", action="store_true", help="headline only: skip the sub-records of the other configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "ep_prefill":
        run_ep_prefill(args)
    elif args.workload == "stack_prefill":
        run_stack_prefill(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
