#!/usr/bin/env python
"""Benchmark of the quantized matrix-product path on B200.

Main line (one JSON object on stdout): the 4-layer expert-parallel MoE layer stack (hidden 7168, 256 experts top-8,
expert intermediate 2048, MXFP4 expert weights, FP8 1x128 activations, one FP8 7168x7168 dense projection per
layer) at a 64-token decode step, in tokens/s, on N GPUs.  The same object carries the decode FP8 GEMV sweep
(GB/s per shape), the single-layer decode MoE, the HBM roofline of the dominant kernel, the end-to-end figure through
host buffers and a CPU baseline timed on this box's host cores.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference        # the CPU restatement of the path, all host threads, same metric
    python bench.py --small-case decode     # a few launches on a few GB: the case the ncu captures under profiles/ use
    python bench.py --small-case prefill --case-mode mx
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

H, I, E, TOPK, LAYERS = 7168, 2048, 256, 8, 4
DENSE_SHAPES = [(4096, 7168), (7168, 2048), (18432, 7168), (7168, 16384)]
METRIC = "moe_layer_stack_decode_tokens_per_s"
# dram__bytes_read.sum + dram__bytes_write.sum of one w13 launch in the ncu small case, divided by its 55 active experts
NCU_W13_DRAM_BYTES_PER_ACTIVE_EXPERT = (858.861312e6 + 4.27136e6) / 55


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def workload_config(tokens, world, eager=False, pdl=True):
    """The `config` object of the JSON line; both arms print the same keys."""
    leg = "decode step" if tokens <= 1024 else "prefill"
    return {"workload": "cfg4: 4 layers x (FP8 7168x7168 dense + 256-expert top-8 MXFP4 MoE), %d-token %s" % (tokens, leg),
            "tokens": tokens, "hidden": H, "experts": E, "topk": TOPK, "inter": I, "layers": LAYERS,
            "parallelism": "ep%d" % world, "step_launch": "eager" if eager else "cuda_graph", "pdl": bool(pdl),
            "l2": "weights read per step (>= 6 GB per GPU) exceed the 126 MB L2"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only queries)."""

    def __init__(self, index=0):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def expert_bytes():
    """Algorithmic HBM bytes of one expert: FP4 codes + UE8M0/32 scales of w13 (2I x H) and w2 (H x I)."""
    w13 = 2 * I * H // 2 + 2 * I * H // 32
    w2 = H * I // 2 + H * I // 32
    return w13, w2


# ---------------------------------------------------------------------------------------------- CPU arm
CPU_SAMPLE_TOKENS = 16


def cpu_prepare(tokens_sample=CPU_SAMPLE_TOKENS, seed=0):
    """Inputs of the CPU sample: `tokens_sample` tokens of ONE layer of the benchmark shape (dense FP8 7168x7168 + routed
    experts top-8 of 256).  Only the experts the sample routes to are materialised (random MXFP4 codes, scales near 2^-7)."""
    import oracle
    import torch
    rng = np.random.default_rng(seed)
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(tokens_sample, H, generator=g)).bfloat16().view(torch.uint16).numpy()
    wd = (torch.randn(H, H, generator=g) * 0.02).bfloat16().view(torch.uint16).numpy()
    wq, ws = oracle.quant_fp8_weight(oracle.MODE_DS, wd)
    logits = torch.randn(tokens_sample, E, generator=g).numpy()
    ids, w = oracle.route(1, logits, None, TOPK)
    used = sorted(set(ids.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    ids_l = np.vectorize(remap.get)(ids).astype(np.int32)
    n = len(used)
    c13 = rng.integers(0, 256, (n, 2 * I, H // 2), dtype=np.uint8)
    s13 = rng.integers(118, 122, (n, 2 * I, H // 32), dtype=np.uint8)
    c2 = rng.integers(0, 256, (n, H, I // 2), dtype=np.uint8)
    s2 = rng.integers(118, 122, (n, H, I // 32), dtype=np.uint8)
    return dict(x=x, wq=wq, ws=ws, ids=ids_l, w=w, c13=c13, s13=s13, c2=c2, s2=s2, tokens=tokens_sample)


def cpu_run(p):
    """One timed pass of the sample through the CPU oracle (all host threads); tokens/s for the 4-layer stack."""
    import oracle
    t0 = time.perf_counter()
    xq, xs = oracle.act_quant(oracle.MODE_DS, p["x"])
    hb, _ = oracle.gemm_fp8(oracle.MODE_DS, p["wq"], p["ws"], xq, xs)
    oracle.moe_layer(oracle.MODE_DS, hb, p["ids"], p["w"], p["c13"], p["s13"], p["c2"], p["s2"])
    dt = time.perf_counter() - t0
    return p["tokens"] / (dt * LAYERS), dt, oracle.num_threads()


def cpu_sample_text(n_runs, dt):
    return ("%d tokens through one layer (FP8 7168x7168 dense + top-8 of 256 MXFP4 experts) on the scalar C oracle with OpenMP, "
            "%d timed passes of %.1f s, extrapolated to %d layers (a 64-token step is 4x the tokens)" % (CPU_SAMPLE_TOKENS, n_runs, dt, LAYERS))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.use_all_host_cores()   # torch.distributed.run exports OMP_NUM_THREADS=1; this arm is timed on every host core
    p = cpu_prepare()
    for _ in range(min(args.warmup, 1)):
        cpu_run(p)
    vals, dts, nthreads = [], [], 1
    t_all = time.perf_counter()
    for _ in range(args.steps):
        v, dt, nthreads = cpu_run(p)
        vals.append(v)
        dts.append(dt)
        if time.perf_counter() - t_all > 120:
            break
    v = float(np.median(vals))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(vals),
        "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * float(np.median(dts)), "step_is": "one timed pass over the bounded sample (cpu_baseline.sample); value extrapolates it to the 64-token, 4-layer step", "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3 x {fp8_e4m3, mxfp4_e2m1}, fp32 accumulate", "data": "synthetic",
        "config": workload_config(64, args.gpus, pdl=args.pdl),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": nthreads, "kind": "port", "sample": cpu_sample_text(len(vals), float(np.median(dts)))},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------- GPU arm
def time_events(torch, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps  # ms per call


def dense_sweep(pkg, ctx, torch, hbm_peak, quick):
    """Decode FP8 GEMV sweep: GB/s of the weight-streaming kernel alone (activations pre-quantized), rotating over
    enough weight copies that every launch reads its weights from HBM, not L2."""
    synth = importlib.import_module(pkg.__name__ + ".synth")
    out = []
    for (n, k) in DENSE_SHAPES:
        wbytes = n * k + 4 * (n // 128) * (k // 128)
        copies = max(2, int(np.ceil(400e6 / wbytes)))
        ws = []
        for c in range(copies):
            tiles, sds = synth.fp8_dense(torch, False, n, k, 0.02, 100 + c, ctx.device)
            ws.append(pkg.Weight(ctx, 0, pkg.MODE_DS, n, k, 1, False, tiles, sds))
        for m in ([1, 16] if quick else [1, 4, 8, 16]):
            x = torch.randn(m, k, device=ctx.device).bfloat16()
            xq, xs = pkg.act_quant(ctx, pkg.MODE_DS, x)
            o = torch.empty(m, n, dtype=torch.bfloat16, device=ctx.device)
            # one CUDA graph of `copies` launches (each on a different weight copy), replayed: GPU time, not launch rate
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for c in range(copies):
                    pkg.gemm_fp8(ctx, ws[c], xq, xs, m, o)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for c in range(copies):
                        pkg.gemm_fp8(ctx, ws[c], xq, xs, m, o)
                # the same with the activation quantizer in front of every GEMV (ops::gemv takes bf16 activations)
                graph_q = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph_q, stream=side):
                    for c in range(copies):
                        pkg.act_quant(ctx, pkg.MODE_DS, x, xq, xs)
                        pkg.gemm_fp8(ctx, ws[c], xq, xs, m, o)
            torch.cuda.current_stream().wait_stream(side)
            ms = time_events(torch, graph.replay, 10, 2) / copies
            ms_q = time_events(torch, graph_q.replay, 10, 2) / copies
            del graph, graph_q
            algo = wbytes + 2 * m * k + 2 * m * n
            gbs = algo / (ms * 1e-3) / 1e9
            out.append({"n": n, "k": k, "m": m, "us": round(ms * 1e3, 2), "gbs": round(gbs, 1),
                        "frac_of_measured_hbm": round(gbs / hbm_peak, 3), "frac_of_8tbs": round(gbs / 8000.0, 3),
                        "us_with_act_quant": round(ms_q * 1e3, 2)})
        del ws
        torch.cuda.empty_cache()
    return out


def lm_head_bench(pkg, ctx, torch, hbm_peak, vocab=129280):
    """The output head (bf16 [vocab][7168] weight, 1.85 GB: larger than L2, read once per call) at 1 and 8 token rows,
    with the sampling records on; microseconds per call and the weight bytes per second."""
    g = torch.Generator(device="cuda").manual_seed(99)
    w = (torch.randn(vocab, H, generator=g, device="cuda") * 0.02).bfloat16()
    out = {"vocab": vocab, "k": H, "weight_bytes": vocab * H * 2, "cases": []}
    for m in (1, 8):
        x = torch.randn(m, H, generator=g, device="cuda").bfloat16()
        logits = torch.empty(m, vocab, dtype=torch.float32, device="cuda")
        rec = torch.zeros(m, vocab // 64, 20, dtype=torch.float32, device="cuda")
        ms = time_events(torch, lambda: pkg.lm_head(ctx, w, x, out=logits, temperature=0.8, records=rec), 10, 3)
        ms_plain = time_events(torch, lambda: pkg.lm_head(ctx, w, x, out=logits), 10, 3)
        gbs = vocab * H * 2 / (ms * 1e-3) / 1e9
        out["cases"].append({"m": m, "us": round(ms * 1e3, 1), "us_without_records": round(ms_plain * 1e3, 1), "gbs": round(gbs, 1),
                             "frac_of_measured_hbm": round(gbs / hbm_peak, 3), "frac_of_8tbs": round(gbs / 8000.0, 3)})
    out["device_status"] = int(ctx.status().code)
    del w
    torch.cuda.empty_cache()
    return out


def _graph_us(torch, launches, reps=10):
    """Microseconds per launch of a list of callables captured into one CUDA graph and replayed (GPU time, not launch rate)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in launches:
            f()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for f in launches:
                f()
    torch.cuda.current_stream().wait_stream(side)
    ms = time_events(torch, graph.replay, reps, 2) / len(launches)
    del graph
    return ms * 1e3


def reference_kernels(pkg, ctx, torch, hbm_peak, quick, use_pdl=False):
    """The reference's own sm_100a kernels (compiled from its sources into oracle/_ref, launched with its own geometry by
    oracle/refkernels.py) timed on this GPU beside this library's kernels on the same codes, in the reference's (MX) scale
    geometry, which is the only one the reference implements.  Decode GEMVs rotate over enough weight copies to defeat L2."""
    import oracle.refkernels as rk
    if not rk.available():
        return {"unavailable": "oracle/_ref cubins or oracle/librefk.so not built (the reference's sources were absent at build time)"}
    rng = np.random.default_rng(0)

    def rand_weight(n, k):
        codes = rng.integers(0, 0x7e, (n, k), dtype=np.uint8) | (rng.integers(0, 2, (n, k), dtype=np.uint8) << 7)   # finite e4m3
        scales = rng.integers(118, 122, (n // 32, k // 32), dtype=np.uint8)
        return codes, scales

    out = {"geometry": "MX (1x32 activations, 32x32 weights, UE8M0 scales): the reference's", "decode_gemv": [], "notes": []}
    for (n, k) in DENSE_SHAPES:
        wbytes = n * k + (n // 32) * (k // 32)
        copies = max(2, int(np.ceil(260e6 / wbytes)))
        codes, scales = rand_weight(n, k)
        ref_w = [rk.GemvWeight(np.roll(codes, c, axis=0), scales) for c in range(copies)]
        ours_w = [pkg.Weight.dense_fp8(ctx, pkg.MODE_MX, np.roll(codes, c, axis=0), scales) for c in range(copies)]
        tc_w = [rk.TcWeight(np.roll(codes, c, axis=0), scales) for c in range(copies)] if rk.tc_gemv_cluster(n, k, ctx.sm_count) else None
        for m in ([1] if quick else [1, 16]):
            x = torch.randn(m, k, device=ctx.device).bfloat16()
            o = torch.empty(m, n, dtype=torch.bfloat16, device=ctx.device)
            xq, xs = pkg.act_quant(ctx, pkg.MODE_MX, x)
            geo = rk.gemv_geometry(n, k, m, ctx.sm_count)
            us_ref = _graph_us(torch, [lambda w=w: rk.gemv_fp8(w, x, o, pdl=use_pdl) for w in ref_w])
            us_ours = _graph_us(torch, [lambda w=w: (pkg.act_quant(ctx, pkg.MODE_MX, x, xq, xs), pkg.gemm_fp8(ctx, w, xq, xs, m, o)) for w in ours_w])
            algo = wbytes + 2 * m * k + 2 * m * n
            row = {"n": n, "k": k, "m": m, "reference_kernel": geo["kernel"], "reference_cluster": geo["cs"], "reference_us": round(us_ref, 2),
                   "reference_gbs": round(algo / us_ref / 1e3, 1), "ours_us_with_act_quant": round(us_ours, 2),
                   "ours_gbs": round(algo / us_ours / 1e3, 1), "speedup": round(us_ref / us_ours, 2)}
            if tc_w is not None and m <= 8:
                us_tc = _graph_us(torch, [lambda w=w: rk.tc_gemv_fp8(w, x, o, pdl=use_pdl) for w in tc_w])
                row["reference_tc_gemv_fp8_us"] = round(us_tc, 2)
                row["speedup_vs_tc_gemv_fp8"] = round(us_tc / us_ours, 2)
            out["decode_gemv"].append(row)
            rk.synchronize()
        del ref_w, ours_w, tc_w
        torch.cuda.empty_cache()
    out["notes"].append("tc_gemv_fp8 (the reference's tcgen05 decode GEMV) accepts only the 7168 x 2048 shape of the four "
                        "(K/cluster <= 1024 and 96..SMs CTAs, crates/engine/src/ops.rs:1105-1107)")
    # prefill dense: tc_quant_rows + tc_gemm_fp8p at the reference's chunk limit of 8192 tokens (PMAX, model.rs:13)
    tokens = 8192
    codes, scales = rand_weight(H, H)
    tw = rk.TcWeight(codes, scales)
    w = pkg.Weight.dense_fp8(ctx, pkg.MODE_MX, codes, scales)
    x = torch.randn(tokens, H, device=ctx.device).bfloat16()
    o = torch.empty(tokens, H, dtype=torch.bfloat16, device=ctx.device)
    aq, sfa = rk.tc_quant_rows(x)
    xq, xs = pkg.act_quant(ctx, pkg.MODE_MX, x)
    flops = 2.0 * tokens * H * H
    ms_ref_q = time_events(torch, lambda: rk.tc_quant_rows(x, aq=aq, sfa=sfa), 5, 2)
    ms_ref = time_events(torch, lambda: rk.tc_gemm(tw, aq, sfa, tokens, out=o), 5, 2)
    rk.synchronize()
    ms_ours_q = time_events(torch, lambda: pkg.act_quant(ctx, pkg.MODE_MX, x, xq, xs), 5, 2)
    ms_ours = time_events(torch, lambda: pkg.gemm_fp8(ctx, w, xq, xs, tokens, o), 5, 2)
    out["prefill_dense"] = {"n": H, "k": H, "tokens": tokens, "reference_kernel": "tc_gemm_fp8p", "reference_ms": round(ms_ref, 4),
                            "reference_tflops": round(flops / ms_ref / 1e9, 1), "reference_tc_quant_rows_ms": round(ms_ref_q, 4),
                            "ours_ms": round(ms_ours, 4), "ours_tflops": round(flops / ms_ours / 1e9, 1), "ours_act_quant_ms": round(ms_ours_q, 4),
                            "speedup_gemm": round(ms_ref / ms_ours, 2), "speedup_quant": round(ms_ref_q / ms_ours_q, 2)}
    # prefill expert GEMMs: tc_moe_w13 + tc_moe_w2 at the largest hidden size the reference's gate/up kernel takes (it keeps
    # the scale atoms of all K tiles of a token tile in 40 shared-memory slots, cu/tcmoe.cu:171: K <= 5120)
    dm, it_, ne, tk = 5120, I, 32, 2048
    rng = np.random.default_rng(11)
    c13 = rng.integers(0, 256, (ne, 2 * it_, dm // 2), dtype=np.uint8)
    s13 = rng.integers(118, 122, (ne, 2 * it_, dm // 32), dtype=np.uint8)
    c2 = rng.integers(0, 256, (ne, dm, it_ // 2), dtype=np.uint8)
    s2 = rng.integers(118, 122, (ne, dm, it_ // 32), dtype=np.uint8)
    xm = torch.randn(tk, dm, device=ctx.device).bfloat16()
    ids, wr = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, torch.randn(tk, ne, device=ctx.device), None, TOPK)
    plan_r = rk.PrefillPlan(ids, wr, ne)
    xq_r, sf_r = rk.moe_gather_quant(xm, torch.ones(dm, dtype=torch.bfloat16, device=ctx.device), 1e-6, plan_r)
    wts = rk.MoeFp4Weights(c13, s13, c2, s2)
    bufs = rk.tc_moe(wts, plan_r, xq_r, sf_r)
    ms_ref_moe = time_events(torch, lambda: rk.tc_moe(wts, plan_r, xq_r, sf_r, out=bufs), 5, 2)
    rk.synchronize()
    plan_l = pkg.MoePlan(ctx, tk, TOPK, ne, 128)
    pkg.moe_perm(ctx, plan_l, ids, wr)
    W13 = pkg.Weight.experts_fp4(ctx, c13, s13, True)
    W2 = pkg.Weight.experts_fp4(ctx, c2, s2, False)
    pr = tk * TOPK
    xq_l = torch.empty(pr, dm, dtype=torch.uint8, device=ctx.device)
    xs_l = torch.empty(pr, dm // 32, dtype=torch.uint8, device=ctx.device)
    pkg.moe_gather_quant(ctx, pkg.MODE_MX, plan_l, xm, xq_l, xs_l)
    act = torch.empty(pr, it_, dtype=torch.bfloat16, device=ctx.device)
    aq_l = torch.empty(pr, it_, dtype=torch.uint8, device=ctx.device)
    as_l = torch.empty(pr, it_ // 32, dtype=torch.uint8, device=ctx.device)
    yr = torch.empty(pr, dm, dtype=torch.float32, device=ctx.device)

    def ours_moe():
        pkg.moe_w13_swiglu(ctx, W13, pkg.MODE_MX, plan_l, xq_l, xs_l, act, 0.0)
        pkg.act_quant(ctx, pkg.MODE_MX, act, aq_l, as_l)
        pkg.moe_w2(ctx, W2, pkg.MODE_MX, plan_l, aq_l, as_l, yr)
    ms_ours_moe = time_events(torch, ours_moe, 5, 2)
    fl = 6.0 * pr * it_ * dm
    out["prefill_moe"] = {"hidden": dm, "inter": it_, "experts": ne, "tokens": tk, "pairs": pr, "reference_kernels": "tc_moe_w13 + tc_moe_w2",
                          "reference_ms": round(ms_ref_moe, 4), "reference_tflops": round(fl / ms_ref_moe / 1e9, 1),
                          "ours_ms_w13_quant_w2": round(ms_ours_moe, 4), "ours_tflops": round(fl / ms_ours_moe / 1e9, 1),
                          "speedup": round(ms_ref_moe / ms_ours_moe, 2)}
    del wts, W13, W2, bufs
    # the decode-size batch (64 tokens, top-8): the reference's decode path takes at most 16 rows (MAX_M,
    # crates/model/src/limits.rs:1; its MoE kernels 97 slots, cu/gemv.cu:9), so a 64-token step takes Rank::ffn_prefill
    # (model.rs:3063): the same tc_moe_w13 / tc_moe_w2, with 128-row tiles that hold a handful of rows each; ours runs its
    # decode kernels on 8-row slots.  128 experts, hidden 5120 (the largest the reference's gate/up kernel takes).
    ne2, tk2 = 128, 64
    c13 = rng.integers(0, 256, (ne2, 2 * it_, dm // 2), dtype=np.uint8)
    s13 = rng.integers(118, 122, (ne2, 2 * it_, dm // 32), dtype=np.uint8)
    c2 = rng.integers(0, 256, (ne2, dm, it_ // 2), dtype=np.uint8)
    s2 = rng.integers(118, 122, (ne2, dm, it_ // 32), dtype=np.uint8)
    xm2 = torch.randn(tk2, dm, device=ctx.device).bfloat16()
    ids2, wr2 = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, torch.randn(tk2, ne2, device=ctx.device), None, TOPK)
    plan_r2 = rk.PrefillPlan(ids2, wr2, ne2)
    xq_r2, sf_r2 = rk.moe_gather_quant(xm2, torch.ones(dm, dtype=torch.bfloat16, device=ctx.device), 1e-6, plan_r2)
    wts2 = rk.MoeFp4Weights(c13, s13, c2, s2)
    bufs2 = rk.tc_moe(wts2, plan_r2, xq_r2, sf_r2)
    ms_ref_dec = time_events(torch, lambda: rk.tc_moe(wts2, plan_r2, xq_r2, sf_r2, out=bufs2), 10, 3)
    rk.synchronize()
    W13d = pkg.Weight.experts_fp4(ctx, c13, s13, True)
    W2d = pkg.Weight.experts_fp4(ctx, c2, s2, False)
    plan_d = pkg.MoePlan(ctx, tk2, TOPK, ne2, 8)
    pkg.moe_perm(ctx, plan_d, ids2, wr2)
    pr2 = tk2 * TOPK
    xq_d = torch.empty(pr2, dm, dtype=torch.uint8, device=ctx.device)
    xs_d = torch.empty(pr2, dm // 32, dtype=torch.uint8, device=ctx.device)
    pkg.moe_gather_quant(ctx, pkg.MODE_MX, plan_d, xm2, xq_d, xs_d)
    act_d = torch.empty(pr2, it_, dtype=torch.bfloat16, device=ctx.device)
    aq_d = torch.empty(pr2, it_, dtype=torch.uint8, device=ctx.device)
    as_d = torch.empty(pr2, it_ // 32, dtype=torch.uint8, device=ctx.device)
    yr_d = torch.empty(pr2, dm, dtype=torch.float32, device=ctx.device)

    def ours_dec():
        pkg.moe_w13_swiglu(ctx, W13d, pkg.MODE_MX, plan_d, xq_d, xs_d, act_d, 0.0)
        pkg.act_quant(ctx, pkg.MODE_MX, act_d, aq_d, as_d)
        pkg.moe_w2(ctx, W2d, pkg.MODE_MX, plan_d, aq_d, as_d, yr_d)
    ms_ours_dec = time_events(torch, ours_dec, 10, 3)
    act_exp = int(torch.unique(ids2).numel())
    wbytes = act_exp * (2 * it_ * dm // 2 + 2 * it_ * dm // 32 + dm * it_ // 2 + dm * it_ // 32)
    out["decode_moe"] = {"hidden": dm, "inter": it_, "experts": ne2, "active_experts": act_exp, "tokens": tk2,
                         "reference_kernels": "tc_moe_w13 + tc_moe_w2 (more than MAX_M = 16 rows: the reference's prefill path)",
                         "reference_ms": round(ms_ref_dec, 4), "reference_gbs": round(wbytes / ms_ref_dec / 1e6, 1),
                         "ours_ms_w13_quant_w2": round(ms_ours_dec, 4), "ours_gbs": round(wbytes / ms_ours_dec / 1e6, 1),
                         "speedup": round(ms_ref_dec / ms_ours_dec, 2)}
    del wts2, W13d, W2d, bufs2
    out["notes"].append("tc_moe_w13 (the reference's prefill gate/up GEMM) keeps the scale atoms of all K tiles of a token tile in 40 "
                        "shared-memory slots (cu/tcmoe.cu:171, SFB_MAX): K <= 5120, so it cannot run at hidden 7168 and is timed at 5120; the fused "
                        "decode MoE entries and comm.cu spin on global memory without a bound and are not launched on a shared GPU")
    out["device_status"] = int(ctx.status().code)
    return out


def zipf_routing(torch, tokens, n_exp, topk, seed, device):
    """cfg3 routing: expert popularity Zipf(s=1.1) over a seeded permutation; each token draws `topk` distinct experts
    without replacement in proportion to popularity (Gumbel top-k); weights = softmax of `topk` fresh N(0,1) logits."""
    g = torch.Generator(device=device).manual_seed(seed)
    perm = torch.randperm(n_exp, generator=g, device=device)
    p = 1.0 / torch.arange(1, n_exp + 1, device=device, dtype=torch.float32) ** 1.1
    logp = torch.empty(n_exp, device=device)
    logp[perm] = torch.log(p / p.sum())
    u = torch.rand(tokens, n_exp, generator=g, device=device).clamp_min(1e-20)
    ids = (logp[None, :] - torch.log(-torch.log(u))).topk(topk, dim=1).indices.to(torch.int32)
    w = torch.softmax(torch.randn(tokens, topk, generator=g, device=device), dim=1)
    return ids.contiguous(), w.contiguous()


def prefill_dense(pkg, ctx, torch, stack, tokens, mode_name):
    """The dense FP8 7168x7168 projection of the stack over a prefill-size batch (the layer's own weight, its geometry)."""
    w = stack.dense[0]
    x = torch.randn(tokens, H, generator=torch.Generator(device="cuda").manual_seed(5), device="cuda").bfloat16()
    xq, xs = pkg.act_quant(ctx, w.mode, x)
    out = torch.empty(tokens, H, dtype=torch.bfloat16, device="cuda")
    ms = time_events(torch, lambda: pkg.gemm_fp8(ctx, w, xq, xs, tokens, out), 5, 2)
    ms_q = time_events(torch, lambda: (pkg.act_quant(ctx, w.mode, x, xq, xs), pkg.gemm_fp8(ctx, w, xq, xs, tokens, out)), 5, 2)
    flops = 2.0 * tokens * H * H
    return {"tokens": tokens, "n": H, "k": H, "geometry": mode_name, "ms": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
            "ms_with_act_quant": round(ms_q, 4), "device_status": int(ctx.status().code)}


def prefill_moe(pkg, ctx, torch, stack, tokens, act_mode=None, tensor_peak=None):
    """cfg3: one routed-expert layer over `tokens` tokens with Zipf-skewed routing on 128-row plans (tcgen05 path);
    TFLOPS = 6 * pairs * inter * hidden / time of the two grouped GEMMs (+ the whole layer's time alongside)."""
    w13, w2 = stack.moe[0].w13, stack.moe[0].w2
    act_mode = stack.cfg.act_mode if act_mode is None else act_mode
    layer = pkg.MoeLayer(ctx, w13, w2, tokens, TOPK, act_mode, tile_rows=128)
    ids, w = zipf_routing(torch, tokens, E, TOPK, 7, ctx.device)
    x = torch.randn(tokens, H, device=ctx.device).bfloat16()
    y = torch.empty(tokens, H, dtype=torch.bfloat16, device=ctx.device)
    ms_layer = time_events(torch, lambda: layer.forward(x, ids, w, y), 3, 2)
    plan = layer.plan

    def gemms():
        pkg.moe_w13_swiglu(ctx, w13, layer.act_mode, plan, layer.xq, layer.xs, layer.act, 0.0)
        pkg.moe_w2(ctx, w2, layer.act_mode, plan, layer.act_q, layer.act_s, layer.yrows)
    ms_g = time_events(torch, gemms, 3, 1)
    flops = 6.0 * tokens * TOPK * I * H
    cnt = torch.bincount(ids.reshape(-1).long(), minlength=E)
    st = ctx.status()
    del layer
    return {"tokens": tokens, "pairs": tokens * TOPK, "ms_grouped_gemms": round(ms_g, 3), "tflops": round(flops / (ms_g * 1e-3) / 1e12, 1),
            "frac_of_fp8_dense_peak_4500": round(flops / (ms_g * 1e-3) / 4.5e15, 4),
            "frac_of_tensor_peak_measured": round(flops / (ms_g * 1e-3) / 1e12 / tensor_peak, 4) if tensor_peak else None,
            "ms_layer": round(ms_layer, 3),
            "layer_tokens_per_s": round(tokens / (ms_layer * 1e-3), 1),
            "tokens_per_expert": {"max": int(cnt.max()), "median": int(cnt.median()), "min": int(cnt.min())},
            "routing": "Zipf(1.1) popularity, Gumbel top-8 without replacement", "device_status": st.code}


def finish(torch, dist, world, graph):
    """Multi-rank exit: tearing the NCCL communicator down while a captured graph still references it can block, so the
    ranks drop the graph, meet at a barrier and leave without the communicator's destructor."""
    del graph
    sys.stdout.flush()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stderr.flush()
        os._exit(0)


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        # a rank that is two minutes late at a barrier has failed: end the run instead of waiting out the default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    pkg = load_package()
    stackmod = importlib.import_module(pkg.__name__ + ".stack")
    ctx = pkg.Ctx(local, pdl=args.pdl)
    hbm_peak, peak_src = peaks()
    T = args.tokens
    amode = pkg.MODE_MX if args.act_mode == "mx" else pkg.MODE_DS
    cfg = stackmod.StackConfig(hidden=H, inter=I, n_experts=E, topk=TOPK, layers=LAYERS, tokens=T, act_mode=amode, dense_mode=amode)
    if world > 1:
        stack = stackmod.EpLayerStack(ctx, cfg, dist, rank, world)
    else:
        stack = stackmod.LayerStack(ctx, cfg)
    t_local = T // world
    g = torch.Generator().manual_seed(1234)
    x_full = torch.randn(T, H, generator=g).bfloat16()       # the step's tokens; rank r owns rows [r*T/W, (r+1)*T/W)
    x_host = x_full[rank * t_local:(rank + 1) * t_local].clone().pin_memory()
    y_host = torch.empty(t_local, H, dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.cuda()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the step as one CUDA graph (kernels + collectives), as the reference replays its decode step (model.rs:3956) ----
    for _ in range(args.warmup):
        stack.forward(x_dev)
    barrier()
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            stack.forward(x_dev)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                y_static = stack.forward(x_dev)
        torch.cuda.current_stream().wait_stream(side)

    def step():
        if graph is not None:
            graph.replay()
            return y_static
        return stack.forward(x_dev)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- device-resident throughput ----
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        # every rank must agree on the figure (and on the number of steps derived from it below: the ranks replay a
        # graph that contains their exchange, so they have to replay it the same number of times)
        tms = torch.tensor([ms], device="cuda")
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    st_mid = ctx.status()
    if st_mid.code:
        raise RuntimeError(f"device status {st_mid.code} (kernel {st_mid.kernel}, site {st_mid.where}) after the timed steps: the result is void")
    # ---- end to end through host buffers: H2D of the step's tokens, the step, D2H of its result; the same K steps, right
    #      after the device-timed ones (the one-second region below runs under the power cap and comes last) ----
    # Every step's tokens come from pinned host memory and its result goes back to it; the two copies run on streams of
    # their own through double-buffered device staging, so step k's result and step k + 1's tokens cross PCIe while the
    # neighbouring steps compute (the step itself reads and writes fixed buffers: it is a captured graph).
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_stage = [torch.empty_like(x_dev) for _ in range(2)]
    y_stage = [torch.empty(t_local, H, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]       # tokens of a step have arrived in x_stage[b]
    ev_xfree = [torch.cuda.Event() for _ in range(2)]    # x_stage[b] has been consumed
    ev_res = [torch.cuda.Event() for _ in range(2)]      # a step's result is in y_stage[b]
    ev_yfree = [torch.cuda.Event() for _ in range(2)]    # y_stage[b] has been read back

    def e2e_steps(n):
        for k in range(n):
            b = k & 1
            with torch.cuda.stream(s_in):
                if k >= 2:
                    s_in.wait_event(ev_xfree[b])
                x_stage[b].copy_(x_host, non_blocking=True)
                ev_in[b].record(s_in)
            main.wait_event(ev_in[b])
            x_dev.copy_(x_stage[b], non_blocking=True)
            ev_xfree[b].record(main)
            y = step()
            if k >= 2:
                main.wait_event(ev_yfree[b])
            y_stage[b].copy_(y, non_blocking=True)
            ev_res[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_res[b])
                y_host.copy_(y_stage[b], non_blocking=True)
                ev_yfree[b].record(s_out)
        main.wait_stream(s_out)      # the last results are on the host before the region's closing event

    e2e_steps(2)
    barrier()
    e0.record()
    e2e_steps(args.steps)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    # ---- the same step over a region of at least a second (the K timed steps above are the contract's number) ----
    n_long = max(args.steps, int(np.ceil(1100.0 / max(ms, 1e-3)))) if args.sustain else 0
    ms_long = None
    if n_long:
        e0.record()
        for _ in range(n_long):
            step()
        e1.record()
        barrier()
        ms_long = e0.elapsed_time(e1) / n_long
    clocks = sampler.stop() if rank == 0 else None
    # ---- dominant kernel: a second capture of the same step with event-record nodes around every gate/up launch, so
    #      its time comes from graph replays like the headline (eager launches when --no-graph) ----
    w13_times = []
    if graph is not None:
        events = []
        with torch.cuda.stream(side):
            graph_ev = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_ev, stream=side):
                stack.forward(x_dev, events=events)
        torch.cuda.current_stream().wait_stream(side)
        for i in range(min(args.steps, 20) + 2):
            graph_ev.replay()
            torch.cuda.synchronize()
            if i >= 2:
                w13_times += [a.elapsed_time(b) for a, b in events]
        del graph_ev
    else:
        events = []
        for _ in range(args.steps):
            stack.forward(x_dev, events=events)
        torch.cuda.synchronize()
        w13_times = [a.elapsed_time(b) for a, b in events]
    barrier()
    st = ctx.status()
    # ---- N > 1: the sharded stack against the single-GPU stack on the same weights, one layer (6 GB of experts) ----
    parity = None
    if world > 1 and not args.skip_parity:
        y_ep = stack.forward(x_dev, layers=1).float()
        torch.cuda.synchronize()
        if rank == 0:
            cfg1 = stackmod.StackConfig(hidden=H, inter=I, n_experts=E, topk=TOPK, layers=1, tokens=T, act_mode=amode, dense_mode=amode)
            ref1 = stackmod.LayerStack(ctx, cfg1)
            y1 = ref1.forward(x_full.cuda(), layers=1)[:t_local].float()
            torch.cuda.synchronize()
            parity = float((y_ep - y1).norm() / y1.norm())
            del ref1, y1
            torch.cuda.empty_cache()
        barrier()
    if world > 1:
        tms = torch.tensor([ms_e2e, ms_long if ms_long is not None else 0.0], device="cuda")
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms_e2e, ml = tms.tolist()
        ms_long = ml if ms_long is not None else None
    if rank != 0:
        finish(torch, dist, world, graph)
        return
    # ---- roofline of the dominant kernel (grouped gate/up GEMM) ----
    w13_b, w2_b = expert_bytes()
    w13_ms = float(np.mean(w13_times))
    n_local = E // world
    ids_counts = []
    for l in range(LAYERS):
        ids, _ = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, stack.logits_full(l) if world > 1 else stack.logits[l], None, TOPK)
        u = torch.unique(ids)
        ids_counts.append(int(((u >= rank * n_local) & (u < (rank + 1) * n_local)).sum()))
    e_act = float(np.mean(ids_counts))
    algo_w13 = e_act * w13_b + T * TOPK * (H + H // 128 * 4) / world + T * TOPK * I * 2 / world
    achieved = algo_w13 / (w13_ms * 1e-3) / 1e9
    roofline = {"kernel": ("tc_stream_kernel" if ctx.tcgen05 else "stream_gemv_kernel") + "<FP4,W13> (grouped gate/up + SwiGLU)", "bound": "hbm", "achieved": round(achieved, 1),
                "peak": hbm_peak, "peak_source": peak_src, "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                "frac_of_8tbs": round(achieved / 8000.0, 4), "avg_launch_ms": round(w13_ms, 4),
                "timed": "CUDA event-record nodes around the kernel inside replays of the captured step" if graph is not None else "CUDA events around eager launches",
                "launches_timed": len(w13_times), "active_experts_per_launch": e_act,
                "algorithmic_bytes_per_launch": int(algo_w13),
                "traffic": args.traffic if args.traffic is not None else int(e_act * NCU_W13_DRAM_BYTES_PER_ACTIVE_EXPERT),
                "traffic_source": "given on the command line" if args.traffic is not None else
                "ncu dram__bytes_read+write of the 64-expert small case (profiles/tc_stream_kernel_decode_small_case.md), "
                "per active expert, times this launch's active experts (traffic grows with the experts streamed)"}
    result = {
        "metric": METRIC if T <= 1024 else "moe_layer_stack_prefill_tokens_per_s", "value": round(T / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3 x {fp8_e4m3, mxfp4_e2m1}, fp32 accumulate", "data": "synthetic",
        "config": workload_config(T, world, args.no_graph, pdl=args.pdl),
        "e2e": {"value": round(T / (ms_e2e * 1e-3), 1), "unit": "tokens/s", "h2d_bytes_per_step": t_local * H * 2 * world,
                "d2h_bytes_per_step": t_local * H * 2 * world, "ms_per_step": round(ms_e2e, 4),
                "note": "every step: tokens from pinned host memory, result back to it; the copies run on their own streams through "
                        "double-buffered staging and overlap the neighbouring steps' compute"},
        "gpu_launches": stack.count_launches() * args.steps,
        "roofline": roofline, "clocks": clocks, "device_status": st.code,
        "exchange": stack.exchange_path() if world > 1 else "none (one GPU)",
    }
    if T > 1024:
        result["stack_tflops"] = round(LAYERS * (2.0 * T * H * H + 6.0 * T * TOPK * I * H) / (ms * 1e-3) / 1e12, 1)
        result["roofline"]["note"] = "prefill-size batch: the HBM figure of the gate/up kernel is not its bound; see stack_tflops"
    if world > 1:
        result["exchange_fallback_reason"] = stack.peer_error
        result["parity_rel_err"] = parity
        result["parity_note"] = ("rank 0's rows after one layer of the sharded stack against a single-GPU LayerStack on the same weights "
                                 "and tokens (relative Frobenius; the ranks' bf16 partial sums differ from one fp32 sum by rounding)")
    if ms_long is not None:
        result["sustained"] = {"steps": n_long, "ms_per_step": round(ms_long, 4), "value": round(T / (ms_long * 1e-3), 1),
                               "note": "the same replayed step over a timed region of at least one second"}
    if world == 1 and not args.skip_sub:
        result["decode_gemv_sweep"] = dense_sweep(pkg, ctx, torch, hbm_peak, args.quick)
        # single routed-expert layer (cfg2): tokens/s of one layer's MoE
        layer0 = stack.moe[0]
        ids, w = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, stack.logits[0], None, TOPK)
        yb = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        ms_l = time_events(torch, lambda: layer0.forward(x_dev, ids, w, yb), 20, 3)
        e_act0 = int(torch.unique(ids).numel())
        result["moe_decode_layer"] = {"tokens": T, "active_experts": e_act0, "ms": round(ms_l, 4), "tokens_per_s": round(T / (ms_l * 1e-3), 1),
                                      "gbs": round(e_act0 * (w13_b + w2_b) / (ms_l * 1e-3) / 1e9, 1),
                                      "note": "L2 holds 126 MB of the ~5 GB read per call; repeated calls on one layer are HBM-bound"}
    if world == 1 and not args.skip_sub and not args.quick:
        # what the tensor cores deliver to the kernels' MMA instruction with no memory traffic at all (measured here;
        # the box's measured-peaks file has no FP8 entry): the ceiling beside the vendor's nominal 4.5 PFLOP/s
        tp = {"n128_e2m1": pkg.probe_tensor_rate(ctx, 128, True), "n256_e2m1": pkg.probe_tensor_rate(ctx, 256, True),
              "n128_e4m3": pkg.probe_tensor_rate(ctx, 128, False), "n256_e4m3": pkg.probe_tensor_rate(ctx, 256, False)}
        tensor_peak = max(tp.values())
        result["tensor_peak_measured"] = {"tflops": round(tensor_peak, 1), "by_shape": {k: round(v, 1) for k, v in tp.items()},
                                          "how": "148 CTAs issuing tcgen05.mma kind::mxf8f6f4.block_scale M=128 K=32 back to back on resident operands, "
                                                 "best of 5 launches of 20000 MMAs per CTA, CUDA events", "nominal_dense_fp8_tflops": 4500}
        result["prefill_moe"] = prefill_moe(pkg, ctx, torch, stack, args.prefill_tokens, tensor_peak=tensor_peak)
        pdn = prefill_dense(pkg, ctx, torch, stack, args.prefill_tokens, "ds" if amode == pkg.MODE_DS else "mx")
        pdn["frac_of_fp8_dense_peak_4500"] = round(pdn["tflops"] / 4500.0, 4)
        pdn["frac_of_tensor_peak_measured"] = round(pdn["tflops"] / tensor_peak, 4)
        result["prefill_dense"] = pdn
        if stack.cfg.act_mode == pkg.MODE_DS:
            # the same two workloads with the reference's own activation geometry (1x32, UE8M0 scales: block scaling in hardware)
            lmx = pkg.MoeLayer(ctx, stack.moe[0].w13, stack.moe[0].w2, T, TOPK, pkg.MODE_MX)
            ms_mx = time_events(torch, lambda: lmx.forward(x_dev, ids, w, yb), 20, 3)
            result["mx_geometry"] = {"moe_decode_layer": {"ms": round(ms_mx, 4), "tokens_per_s": round(T / (ms_mx * 1e-3), 1),
                                                          "gbs": round(e_act0 * (w13_b + w2_b) / (ms_mx * 1e-3) / 1e9, 1)},
                                     "prefill_moe": prefill_moe(pkg, ctx, torch, stack, args.prefill_tokens, pkg.MODE_MX, tensor_peak=tensor_peak)}
            del lmx
        # cfg4's prefill leg on one GPU: the whole 4-layer stack (dense FP8 projection + routed experts) over a
        # prefill-size batch, sharing the decode stack's weights
        tp = args.prefill_tokens
        pcfg = stackmod.StackConfig(hidden=H, inter=I, n_experts=E, topk=TOPK, layers=LAYERS, tokens=tp, act_mode=amode, dense_mode=amode)
        pstack = stackmod.LayerStack(ctx, pcfg, weights_from=stack)
        xp = torch.randn(tp, H, generator=torch.Generator(device="cuda").manual_seed(77), device="cuda").bfloat16()
        ms_p = time_events(torch, lambda: pstack.forward(xp), 3, 1)
        flop_layer = 2.0 * tp * H * H + 6.0 * tp * TOPK * I * H
        result["prefill_stack"] = {"tokens": tp, "layers": LAYERS, "ms": round(ms_p, 3), "tokens_per_s": round(tp / (ms_p * 1e-3), 1),
                                   "tflops": round(LAYERS * flop_layer / (ms_p * 1e-3) / 1e12, 1),
                                   "routing": "softmax of N(0,1) logits, top-8 (near-uniform expert load)",
                                   "launches_per_layer": pstack.count_launches() // LAYERS, "device_status": int(ctx.status().code)}
        del pstack, xp
    if world == 1 and not args.skip_sub and not args.quick:
        result["lm_head"] = lm_head_bench(pkg, ctx, torch, hbm_peak)
    if world == 1 and not args.skip_sub and not args.skip_ref_kernels:
        try:
            result["reference_kernels"] = reference_kernels(pkg, ctx, torch, hbm_peak, args.quick, use_pdl=args.pdl)
        except Exception as ex:  # noqa: BLE001 - the comparison must not take the benchmark line down with it
            result["reference_kernels"] = {"unavailable": f"{type(ex).__name__}: {ex}"}
    if world == 1 and not args.skip_cpu:
        p = cpu_prepare()
        vals, dts, t_all = [], [], time.perf_counter()
        while not vals or (time.perf_counter() - t_all < 12 and len(vals) < 8):
            v, dt, nthr = cpu_run(p)
            vals.append(v)
            dts.append(dt)
        result["cpu_baseline"] = {"value": round(float(np.median(vals)), 3), "unit": "tokens/s", "cores": nthr, "kind": "port",
                                  "sample": cpu_sample_text(len(vals), float(np.median(dts)))}
    print(json.dumps(result))
    finish(torch, dist, world, graph)


def small_case(args):
    """A few launches on a few GB, for `ncu` captures and quick checks (one GPU).
    decode : one dense FP8 GEMV (18432 x 7168 and 7168 x 2048, --case-m token rows) and one decode expert layer
             (default 64 experts of the benchmark shape, 16 tokens, top-8: ~59 active experts, 0.92 GB of gate/up weights),
             each run twice.
    lmhead : the output head over 32320 x 7168 bf16 weights (463 MB), 8 token rows, sampling records on, run twice.
    prefill: one expert layer on 128-row plans (default 8 experts, 2048 tokens, top-8) and one dense 7168 x 7168 GEMM over
             the same tokens, each run twice."""
    import torch
    pkg = load_package()
    synth = importlib.import_module(pkg.__name__ + ".synth")
    torch.manual_seed(0)       # same routing (and the same number of active experts) on every run
    torch.cuda.manual_seed(0)
    mode = pkg.MODE_MX if args.case_mode == "mx" else pkg.MODE_DS
    ctx = pkg.Ctx(0, pdl=args.pdl)
    dev = ctx.device
    if args.small_case == "lmhead":
        # the output head on a quarter of the vocabulary (32320 x 7168 bf16 = 463 MB: larger than L2), 8 token rows, records on
        n = args.case_experts or 32320
        g = torch.Generator(device=dev).manual_seed(99)
        w = (torch.randn(n, H, generator=g, device=dev) * 0.02).bfloat16()
        x = torch.randn(8, H, generator=g, device=dev).bfloat16()
        for _ in range(2):
            logits, rec = pkg.lm_head(ctx, w, x, temperature=0.8)
        torch.cuda.synchronize()
        print(json.dumps({"small_case": "lmhead", "vocab_rows": n, "weight_bytes": n * H * 2, "device_status": int(ctx.status().code)}))
        return
    prefill = args.small_case == "prefill"
    n_exp = args.case_experts or (8 if prefill else 64)
    tokens = args.case_tokens or (2048 if prefill else 16)
    w13 = synth.fp4_experts(torch, n_exp, 2 * I, H, 0.02, 2, True, dev)
    w2 = synth.fp4_experts(torch, n_exp, H, I, 0.02, 3, False, dev)
    layer = pkg.MoeLayer(ctx, pkg.Weight.experts_fp4_packed(ctx, w13, 2 * I, H, n_exp, True),
                         pkg.Weight.experts_fp4_packed(ctx, w2, H, I, n_exp, False), tokens, TOPK, mode,
                         tile_rows=128 if prefill else 8)
    xm = torch.randn(tokens, H, device=dev).bfloat16()
    ids, w = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, torch.randn(tokens, n_exp, device=dev), None, TOPK)
    y = torch.empty(tokens, H, dtype=torch.bfloat16, device=dev)
    dense = []
    for (n, k) in ([(H, H)] if prefill else [(18432, 7168), (7168, 2048)]):
        tiles, sds = synth.fp8_dense(torch, mode == pkg.MODE_MX, n, k, 0.02, 1, dev)
        wd = pkg.Weight(ctx, 0, mode, n, k, 1, False, tiles, sds)
        m = tokens if prefill else args.case_m
        x = torch.randn(m, k, device=dev).bfloat16()
        xq, xs = pkg.act_quant(ctx, mode, x)
        dense.append((wd, xq, xs, m, torch.empty(m, n, dtype=torch.bfloat16, device=dev)))
    for _ in range(2):
        for wd, xq, xs, m, out in dense:
            pkg.gemm_fp8(ctx, wd, xq, xs, m, out)
        layer.forward(xm, ids, w, y)
    torch.cuda.synchronize()
    print(json.dumps({"small_case": args.small_case, "mode": args.case_mode, "experts": n_exp, "tokens": tokens,
                      "active_experts": int(torch.unique(ids).numel()), "device_status": int(ctx.status().code)}))


def exchange_bench(args):
    """The expert-parallel exchanges alone, under torch.distributed.run: this library's peer-memory kernels (gather of
    column slices = dispatch, all-reduce, combine fused with the unpermute) beside NCCL's all-gather / all-reduce on the
    same [64][7168] bf16 rows, each as a CUDA graph of 20 calls replayed 10 times; microseconds per call (max over
    ranks) and the bytes a rank pulls over NVLink per call."""
    import datetime
    import torch
    import torch.distributed as dist
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    pkg = load_package()
    ctx = pkg.Ctx(local)
    ctx.set_wait_budget_us(500000)
    T = args.tokens
    peer = pkg.PeerAllReduce(ctx, dist, rank, world)
    bufs = [peer.buffer((T, H)) for _ in range(2)]
    for b in bufs:
        b.copy_(torch.randn(T, H, device="cuda").bfloat16())
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    plan = pkg.MoePlan(ctx, T, TOPK, E // world, 8)
    owner = torch.randint(0, world, (T, TOPK), generator=torch.Generator(device="cuda").manual_seed(7), device="cuda")
    rows_of = torch.arange(T * TOPK, device="cuda", dtype=torch.int32).view(T, TOPK)
    plan.pair_row.copy_(torch.where(owner == rank, rows_of, torch.full_like(rows_of, -1)).view(-1))
    yrows = torch.randn(T * TOPK, H, device="cuda")
    nccl_buf = torch.randn(T, H, device="cuda").bfloat16()
    sl = H // world
    parts = [torch.empty(T, sl, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    mine = nccl_buf[:, rank * sl:(rank + 1) * sl].contiguous()
    row_bytes = T * H * 2
    ops = {
        "peer_gather_cols (dispatch)": (lambda i: peer.gather_cols(bufs[i & 1], out), row_bytes * (world - 1) // world),
        "peer_allreduce": (lambda i: peer(bufs[i & 1], out), row_bytes * (world - 1)),
        "peer_combine (unpermute + all-reduce)": (lambda i: peer.combine(plan, yrows, None, bufs[i & 1], out), row_bytes * (world - 1)),
        "nccl all_gather (column slices)": (lambda i: dist.all_gather(parts, mine), row_bytes * (world - 1) // world),
        "nccl all_reduce": (lambda i: dist.all_reduce(nccl_buf), None),
    }
    res = {}
    for name, (fn, pulled) in ops.items():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(4):
                fn(i)
            side.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(20):
                    fn(i)
        torch.cuda.current_stream().wait_stream(side)
        dist.barrier()
        torch.cuda.synchronize()
        ms = time_events(torch, graph.replay, 10, 3) / 20
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = {"us_per_call": round(float(t.item()) * 1e3, 2), "bytes_pulled_per_rank": pulled}
        del graph
        dist.barrier()
    st = ctx.status()
    if rank == 0:
        print(json.dumps({"exchange_bench": res, "world": world, "rows": T, "row_elems": H, "device_status": st.code}))
    sys.stdout.flush()
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--pdl", dest="pdl", action="store_true", default=None,
                    help="programmatic dependent launch (as the reference's GemvOpts.pdl); default: on for one GPU, where it "
                         "takes ~0.9 us off the small GEMVs, off for several, where the step measured 1-2 %% slower with it")
    ap.add_argument("--no-pdl", dest="pdl", action="store_false")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--act-mode", default="ds", choices=["ds", "mx"], help="scale geometry: ds = 1x128 fp32 (benchmark configs), mx = 1x32 UE8M0 (reference semantics)")
    ap.add_argument("--quick", action="store_true", help="shorter GEMV sweep")
    ap.add_argument("--skip-sub", action="store_true", help="main line only")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-ref-kernels", action="store_true", help="leave out the reference's own kernels (oracle/_ref) timed beside ours")
    ap.add_argument("--skip-parity", action="store_true", help="N > 1: leave out the one-layer comparison with the single-GPU stack")
    ap.add_argument("--no-sustain", dest="sustain", action="store_false", help="leave out the second timed region of >= 1 s")
    ap.add_argument("--exchange-bench", action="store_true", help="under torch.distributed.run: time the peer-memory exchange kernels beside NCCL and exit")
    ap.add_argument("--small-case", default=None, choices=["decode", "prefill", "lmhead"],
                    help="run a few launches of a small case (a few GB on the device) and exit: the case the ncu captures use")
    ap.add_argument("--case-mode", default="ds", choices=["ds", "mx"], help="scale geometry of --small-case")
    ap.add_argument("--case-experts", type=int, default=None)
    ap.add_argument("--case-tokens", type=int, default=None)
    ap.add_argument("--case-m", type=int, default=1, help="token rows of the dense GEMV in --small-case decode")
    ap.add_argument("--prefill-tokens", type=int, default=16384)
    ap.add_argument("--traffic", type=float, default=None, help="ncu dram bytes per launch of the dominant kernel, if captured")
    args = ap.parse_args()
    if args.pdl is None:
        args.pdl = int(os.environ.get("WORLD_SIZE", "1")) == 1
    if args.exchange_bench:
        exchange_bench(args)
    elif args.small_case:
        small_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
