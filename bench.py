"""Benchmark of the engine on one B200: decode tokens per second of a Llama-3.1-8B-shaped model with random bf16
weights at batch 8 and 8,192 tokens of context per request, with the 2,048-token prefill, the decode roofline and
decode at batch 1 and 64 on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C] [--no-points]
    python bench.py --workload 3b-serving   # 64 requests of mixed lengths through Engine.admit/step, Llama-3.2-3B shape
    python bench.py --workload 1b-long      # 4 prompts of 32,768 tokens in 2,048-token portions, then 256 sampled steps
    python bench.py --kernels               # single kernels against the library on the layer's shapes
    python bench.py --attention --head-dim 64 --queries 2048 --keys 32768     # the attention kernels alone
    python bench.py --timeline --batch 8    # when the kernels of one layer of a decode step start and end
    python bench.py --impl reference        # the reference arm (unavailable here: it needs JAX and a TPU)

A "step" is one decode step of the whole batch.  `value` is timed on the device with CUDA events around K calls of the
engine's step function (inputs sent from pinned host memory each step, no read-back); `e2e` is the same through the
public entry point (Engine.admit / Engine.step: host token ids in, sampled token ids read back every step).  A decode
step reads more than 16 GB, far over the 126 MB L2, so no flush is needed between steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

POINT_PAUSE_S = 2.0          # idle time before each of the extra points (decode at batch 1 and 64)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


def baseline_config():
    """Sizes of BASELINE.json's configs[2] (the Llama-3.1-8B shape), as a typed configuration."""
    from mashbox_b200.config.llama import LlamaConfig, RopeScaling
    return LlamaConfig(architecture="LlamaForCausalLM", num_layers=32, hidden=4096, num_heads=32, num_kv_heads=8,
                       head_dim=128, intermediate=14336, vocab=128256, rms_eps=1e-5, rope_theta=500000.0,
                       rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 8192), tie_embeddings=False,
                       attention_bias=False, max_position=131072)


class Clocks:
    """Samples nvidia-smi every 200 ms while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.remove(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def flops_prefill(c, layers, n_tokens):
    H, KV, HD, D, F, V = c.num_heads, c.num_kv_heads, c.head_dim, c.hidden, c.intermediate, c.vocab
    per_layer = 2 * n_tokens * (D * (H + 2 * KV) * HD + H * HD * D + 3 * D * F)
    attn = 4 * (n_tokens * (n_tokens + 1) // 2) * HD * H
    return layers * (per_layer + attn) + 2 * D * V


def bytes_decode(c, layers, batch, kv_len):
    H, KV, HD, D, F, V = c.num_heads, c.num_kv_heads, c.head_dim, c.hidden, c.intermediate, c.vocab
    weights = layers * 2 * (D * (H + 2 * KV) * HD + H * HD * D + 3 * D * F) + 2 * D * V
    cache = layers * batch * kv_len * 2 * KV * HD * 2
    return weights + cache


def run_ours(a):
    import torch
    from mashbox_b200 import ops
    from mashbox_b200.config.registry import architecture
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import RandomSource

    torch.cuda.set_device(0)
    dev = "cuda:0"
    c = baseline_config()
    layers = a.layers or c.num_layers
    import dataclasses
    cfg = dataclasses.replace(c, num_layers=layers)
    K, W, ctx = a.steps, a.warmup, a.context
    batches = [a.batch] + ([] if a.no_points else [b for b in (1, 64) if b != a.batch])
    max_b = max(batches)
    per_request = -(-(ctx + 1024) // 64) * 64
    pool_tokens = max_b * per_request + 4096
    shapes = architecture(cfg.architecture).stored_tensors(cfg)
    t0 = time.time()
    eng = Engine.from_config(cfg, RandomSource(shapes, 0, torch.bfloat16, dev), dtype="bfloat16", device=dev,
                             page_size=16, max_tokens=pool_tokens, max_requests=max_b, max_tokens_per_step=2048 + max_b,
                             chunk=2048, max_context=per_request, cuda_graphs=not a.no_graphs,
                             options=json.loads(a.options) if a.options else None)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator().manual_seed(1)
    rand_ids = lambda n: torch.randint(0, cfg.vocab, (n,), generator=gen).tolist()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    clocks = Clocks()
    clocks.start()

    # ---- prefill of 2,048 tokens: one step of one fresh request (its first token is sampled in the same step)
    P = a.prefill_tokens
    pre_ms = []
    for i in range(2 + 3):
        rows = eng.admit([dict(ids=rand_ids(P), max_new=1)])
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        eng.step()
        e1.record()
        torch.cuda.synchronize()
        assert rows[0].finish == "length", rows[0].finish
        if i >= 2:
            pre_ms.append(e0.elapsed_time(e1))
    pre = statistics.median(pre_ms)
    pk = peaks()
    tflops = flops_prefill(cfg, layers, P) / (pre / 1e3) / 1e12
    prefill = {"value": P / (pre / 1e3), "tokens": P, "ms": pre, "frac": tflops / pk["bf16_tflops"],
               "tflops": tflops, "frac_of_sustained": tflops / pk["bf16_tflops_sustained"]}

    # ---- decode
    def decode(batch, with_e2e):
        # requests finish their prompts one after the other and decode while the others still prefill: the prompt is
        # shortened by the mean of that head start, so that the mean context in the timed steps is about `ctx`
        chunks = -(-ctx // 2048)
        plen = ctx - 2 * (K + W) - (batch - 1) * chunks // 2 - 2
        rows = eng.admit([dict(ids=rand_ids(plen), max_new=2 * (K + W) + batch * chunks + 16) for _ in range(batch)])
        while any(r.t_first is None for r in rows):
            eng.step()
        res = {}
        if with_e2e:
            for _ in range(W):
                eng.step()
            torch.cuda.synchronize()
            l0 = ops.COUNTERS["launches"]
            e0, e1 = ev(), ev()
            e0.record()
            t0 = time.perf_counter()
            for _ in range(K):
                eng.step()
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            ms = max(e0.elapsed_time(e1), wall * 1e3)
            res["e2e"] = {"value": batch * K / (ms / 1e3), "unit": "tokens/s",
                          "h2d_bytes_per_step": eng.runner.inputs.used * 4, "d2h_bytes_per_step": batch * 4 + 4,
                          "ms_per_step": ms / K}
            res["e2e_launches"] = ops.COUNTERS["launches"] - l0
        # the step function alone: fixed next tokens, no read-back inside the timed region
        runner = eng.runner
        live = [r for r in rows if r.finish is None]
        toks = rand_ids(len(live))
        entries = lambda: [(r.rid, [t], [0]) for r, t in zip(live, toks)]
        for _ in range(W):
            runner.step(entries())
        torch.cuda.synchronize()
        l0 = ops.COUNTERS["launches"]
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(K):
            runner.step(entries())
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        runner.check()
        lens = [runner.cache.get(r.rid).length for r in live]
        res.update(value=len(live) * K / (ms / 1e3), ms_per_step=ms / K, launches=ops.COUNTERS["launches"] - l0,
                   kv_len=sum(lens) / len(lens) - K / 2, batch=len(live))
        eng.cancel(rows)
        return res

    def roof(r):
        gbs = bytes_decode(cfg, layers, r["batch"], r["kv_len"]) / (r["ms_per_step"] / 1e3) / 1e9
        return {"ms_per_step": r["ms_per_step"], "mean_kv_len_timed": round(r["kv_len"], 1), "achieved_gbs": gbs,
                "frac": gbs / pk["hbm_gbs"]}

    main = decode(a.batch, True)
    points, detail = {}, {}
    for b in batches[1:]:
        # a pause, so that the power state the measurement before left (the SM clock stays low for a while after a
        # power-capped run) is not part of this one; the point's own clocks are sampled
        torch.cuda.synchronize()
        time.sleep(POINT_PAUSE_S)
        own = Clocks()
        own.start()
        r = decode(b, False)
        ck = own.stop()
        points[f"decode_b{b}"], detail[f"decode_b{b}"] = r["value"], dict(roof(r), sm_mhz=ck["sm_mhz"])
    points[f"decode_b{a.batch}"], detail[f"decode_b{a.batch}"] = main["value"], roof(main)
    clk = clocks.stop()
    nbytes = bytes_decode(cfg, layers, main["batch"], main["kv_len"])
    achieved = nbytes / (main["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tokens/s, Llama-3.1-8B shape, random bf16 weights", "value": main["value"], "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights made on the GPU, uniform random token ids",
        "config": {"model": "llama-3.1-8b-shape", "layers": layers, "layers_of_config": c.num_layers,
                   "hidden": cfg.hidden, "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate, "vocab": cfg.vocab,
                   "global_batch": main["batch"], "seq_len": ctx, "mean_kv_len_timed": round(main["kv_len"], 1),
                   "page_size": 16,
                   "prefill_tokens": P, "parallelism": "single-gpu", "l2": "inputs larger than L2 (no flush)",
                   "cuda_graphs": bool(eng.runner.use_graphs), "peaks": pk["source"], "load_s": round(load_s, 1),
                   "pause_before_points_s": POINT_PAUSE_S},
        "clocks": clk,
        "e2e": {k: main["e2e"][k] for k in ("value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step")},
        "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "points_roofline": detail,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


WORKLOADS = {
    # BASELINE.json configs[3]: continuous batching of 64 requests, prompts U[128, 4096], outputs U[64, 512], greedy
    "3b-serving": dict(model="llama-3.2-3b-shape", layers=28, hidden=3072, heads=24, kv_heads=8, head_dim=128,
                       intermediate=8192, factor=32.0, requests=64, prompt=(128, 4096), new=(64, 512), temperature=0.0),
    # BASELINE.json configs[4]: 4 prompts of 32,768 tokens in 2,048-token portions, then 256 steps at temperature 1.0
    "1b-long": dict(model="llama-3.2-1b-shape", layers=16, hidden=2048, heads=32, kv_heads=8, head_dim=64,
                    intermediate=8192, factor=32.0, requests=4, prompt=(32768, 32768), new=(256, 256), temperature=1.0),
    # the condition of the reference's published single-user rows: one request, 128 new tokens after a warm request
    # (bf16 here, 4- to 8-bit files there); the last has the shape of Falcon3-1B, which its GGUF calls `llama`
    "1b-single": dict(model="llama-3.2-1b-shape", layers=16, hidden=2048, heads=32, kv_heads=8, head_dim=64,
                      intermediate=8192, factor=32.0, requests=1, prompt=(32, 32), new=(128, 128), temperature=0.0),
    "3b-single": dict(model="llama-3.2-3b-shape", layers=28, hidden=3072, heads=24, kv_heads=8, head_dim=128,
                      intermediate=8192, factor=32.0, requests=1, prompt=(32, 32), new=(128, 128), temperature=0.0),
    "8b-single": dict(model="llama-3.1-8b-shape", layers=32, hidden=4096, heads=32, kv_heads=8, head_dim=128,
                      intermediate=14336, factor=8.0, requests=1, prompt=(32, 32), new=(128, 128), temperature=0.0,
                      tied=False),
    "falcon3-1b-single": dict(model="falcon3-1b-shape", layers=18, hidden=2048, heads=8, kv_heads=4, head_dim=256,
                              intermediate=8192, factor=32.0, requests=1, prompt=(32, 32), new=(128, 128),
                              temperature=0.0, vocab=131072),
}


def run_workload(a):
    """A whole workload through the public entry point (Engine.admit / Engine.step, host token ids in, sampled ids read
    back every step): one JSON line with total, prompt and generated tokens per second, what the scheduler and the
    graph cache did, and how much of the wall time the GPU spent inside steps."""
    import random

    import torch
    from mashbox_b200 import ops
    from mashbox_b200.config.llama import LlamaConfig, RopeScaling
    from mashbox_b200.config.registry import architecture
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import RandomSource

    w = WORKLOADS[a.workload]
    torch.cuda.set_device(0)
    dev = "cuda:0"
    layers = a.layers or w["layers"]
    cfg = LlamaConfig(architecture="LlamaForCausalLM", num_layers=layers, hidden=w["hidden"], num_heads=w["heads"],
                      num_kv_heads=w["kv_heads"], head_dim=w["head_dim"], intermediate=w["intermediate"],
                      vocab=w.get("vocab", 128256),
                      rms_eps=1e-5, rope_theta=500000.0, rope_scaling=RopeScaling("llama3", w["factor"], 1.0, 4.0, 8192),
                      tie_embeddings=w.get("tied", True), attention_bias=False, max_position=131072)
    rng = random.Random(a.seed)
    n_req = a.requests or w["requests"]
    plens = [rng.randint(*w["prompt"]) for _ in range(n_req)]
    news = [rng.randint(*w["new"]) for _ in range(n_req)]
    per_request = max(p + n for p, n in zip(plens, news))
    pool = a.pool_tokens or sum(-(-(p + n) // 64) * 64 for p, n in zip(plens, news)) + 4096
    eng = Engine.from_config(cfg, RandomSource(architecture(cfg.architecture).stored_tensors(cfg), 0, torch.bfloat16, dev),
                             dtype="bfloat16", device=dev, page_size=16, max_tokens=pool, max_requests=n_req,
                             max_tokens_per_step=2048 + n_req, chunk=2048, max_context=-(-per_request // 64) * 64,
                             cuda_graphs=not a.no_graphs, options=json.loads(a.options) if a.options else None)
    gen = torch.Generator().manual_seed(a.seed)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=gen).tolist() for n in plens]
    samp = None if w["temperature"] == 0 else dict(temperature=w["temperature"], seed=a.seed)

    # GPU time inside steps: an event before a step's first launch and one after its sampling kernels
    spans = []
    inner = eng._launch

    def timed_launch(prep, before=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st = eng.runner.stats
        was = (st["graph_captures"], st["graph_replays"])
        e0.record()
        f = inner(prep, before)
        e1.record()
        kind = "captured" if st["graph_captures"] > was[0] else "replayed" if st["graph_replays"] > was[1] else "launched"
        spans.append((e0, e1, sum(p.count for p in prep[0]), kind))
        return f

    def once(timed):
        spans.clear()
        rows = eng.admit([dict(ids=p, max_new=n, samp=samp) for p, n in zip(prompts, news)])
        l0 = ops.COUNTERS["launches"]
        before = dict(eng.runner.stats), dict(eng.scheduler.stats)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps, t_first, new_at_first = 0, None, 0
        while eng.busy():
            eng.step()
            steps += 1
            if t_first is None and all(r.t_first is not None or r.finish is not None for r in rows):
                t_first = time.perf_counter()
                new_at_first = sum(len(r.generated) for r in rows)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        gpu_ms = sum(e0.elapsed_time(e1) for e0, e1, _, _ in spans)
        kinds = {}
        for e0, e1, _, kind in spans:
            k = kinds.setdefault(kind, [0, 0.0])
            k[0] += 1
            k[1] = round(k[1] + e0.elapsed_time(e1), 1)
        new = sum(len(r.generated) for r in rows)
        assert all(r.finish == "length" for r in rows), [r.finish for r in rows]
        rs, ss = eng.runner.stats, eng.scheduler.stats
        return dict(wall_s=wall, steps=steps, new_tokens=new, prompt_tokens=sum(plens), gpu_ms_in_steps=gpu_ms,
                    until_all_first_tokens_s=(t_first or t0 + wall) - t0, new_at_first=new_at_first,
                    preemptions=ss["preemptions"] - before[1]["preemptions"],
                    graph_captures=rs["graph_captures"] - before[0]["graph_captures"],
                    graph_replays=rs["graph_replays"] - before[0]["graph_replays"],
                    capture_s=rs["capture_s"] - before[0]["capture_s"], kinds=kinds,
                    launches=ops.COUNTERS["launches"] - l0, deferred=eng.stats["deferred"])

    eng._launch = timed_launch
    clocks = Clocks()
    if a.workload_warm:
        once(False)                      # a first pass loads every kernel and captures the graphs of recurring shapes
    clocks.start()
    r = once(True)
    clk = clocks.stop()
    wall = r["wall_s"]
    decode_s = wall - r["until_all_first_tokens_s"]
    line = {
        "metric": f"generated tokens/s, {a.workload} workload, {w['model']}, random bf16 weights",
        "value": r["new_tokens"] / wall, "unit": "tokens/s", "n_gpus": 1, "steps": r["steps"], "warmup": int(a.workload_warm),
        "ms_per_step": wall * 1e3 / r["steps"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights made on the GPU, seeded uniform random token ids and lengths",
        "config": {"model": w["model"], "layers": layers, "layers_of_config": w["layers"], "hidden": cfg.hidden,
                   "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate, "vocab": cfg.vocab, "requests": n_req,
                   "prompt_tokens": r["prompt_tokens"], "new_tokens": r["new_tokens"], "temperature": w["temperature"],
                   "pool_tokens": pool, "page_size": 16, "chunk": 2048, "seed": a.seed,
                   "cuda_graphs": bool(eng.runner.use_graphs), "parallelism": "single-gpu"},
        "clocks": clk,
        "workload": {"wall_s": wall, "total_tokens_per_s": (r["prompt_tokens"] + r["new_tokens"]) / wall,
                     "prompt_tokens_per_s_until_all_first_tokens": r["prompt_tokens"] / r["until_all_first_tokens_s"],
                     "generated_tokens_per_s_after_that": (None if decode_s <= 0 else
                                                           (r["new_tokens"] - r["new_at_first"]) / decode_s),
                     "until_all_first_tokens_s": r["until_all_first_tokens_s"],
                     "preemptions": r["preemptions"], "graph_captures": r["graph_captures"],
                     "graph_replays": r["graph_replays"], "graph_capture_s": round(r["capture_s"], 3), "steps_and_gpu_ms_by_kind": r["kinds"], "steps_deferred": r["deferred"],
                     "gpu_s_inside_steps": r["gpu_ms_in_steps"] / 1e3,
                     "share_of_wall_outside_steps": 1.0 - r["gpu_ms_in_steps"] / 1e3 / wall},
        "gpu_launches": r["launches"], "impl": "ours",
    }
    print(json.dumps(line))
    return 0


def run_timeline(a):
    """Start and end of every kernel of one decode step inside its captured graph (CUPTI through torch.profiler; no
    ncu): with programmatic dependent launch the kernels of a step overlap, so their durations alone say little; the
    line gives, for one layer in the middle of the model, when each kernel started, when it ended and how long after
    the END of the kernel before it that was.  One JSON line."""
    import dataclasses

    import torch
    from torch.profiler import ProfilerActivity, profile
    from mashbox_b200.config.registry import architecture
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import RandomSource
    dev = "cuda:0"
    c = baseline_config()
    cfg = dataclasses.replace(c, num_layers=a.layers or c.num_layers)
    B, ctx = a.batch, a.context
    per_request = -(-(ctx + 1024) // 64) * 64
    eng = Engine.from_config(cfg, RandomSource(architecture(cfg.architecture).stored_tensors(cfg), 0, torch.bfloat16, dev),
                             dtype="bfloat16", device=dev, page_size=16, max_tokens=B * per_request + 4096, max_requests=B,
                             max_tokens_per_step=2048 + B, chunk=2048, max_context=per_request,
                             options=json.loads(a.options) if a.options else None)
    gen = torch.Generator().manual_seed(1)
    rows = eng.admit([dict(ids=torch.randint(0, cfg.vocab, (ctx - 64,), generator=gen).tolist(), max_new=256) for _ in range(B)])
    while any(r.t_first is None for r in rows):
        eng.step()
    runner = eng.runner
    entries = lambda: [(r.rid, [5], [0]) for r in rows]
    for _ in range(5):
        runner.step(entries())
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            runner.step(entries())
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type.name == "CUDA" and "emcpy" not in e.name and "emset" not in e.name]
    ev.sort(key=lambda e: e.time_range.start)
    first = max(i for i, e in enumerate(ev) if "embed" in e.name)
    step = ev[first:]
    t0 = step[0].time_range.start
    att = [i for i, e in enumerate(step) if "attn" in e.name]
    lo, hi = att[len(att) // 2], att[len(att) // 2 + 1]
    layer, prev_end = [], step[lo - 1].time_range.end
    for e in step[lo:hi]:
        layer.append({"kernel": e.name.split("(")[0][:60], "start_us": round(e.time_range.start - t0, 1),
                      "end_us": round(e.time_range.end - t0, 1), "after_end_of_previous_us": round(e.time_range.end - prev_end, 1)})
        prev_end = max(prev_end, e.time_range.end)
    tail = [{"kernel": e.name.split("(")[0][:60], "start_us": round(e.time_range.start - t0, 1),
             "end_us": round(e.time_range.end - t0, 1)} for e in step[att[-1] + 1:]]
    print(json.dumps({"impl": "ours", "timeline": {"batch": B, "context": ctx, "layers": cfg.num_layers, "kernels_in_step": len(step),
                                                   "step_us": round(step[-1].time_range.end - t0, 1),
                                                   "layer_us": round(step[hi].time_range.start - step[lo].time_range.start, 1),
                                                   "one_layer": layer, "after_the_last_attention": tail}}))
    return 0


def run_attention(a):
    """Times the attention kernels alone on one layer's cache (one JSON line; also the workload of their ncu captures):
    the prompt form -- a portion of `--queries` tokens at the end of `--keys` tokens of context, tcgen05 kernel against
    the mma.sync kernel -- and the decode form, `--batch` one-token sequences of `--keys` tokens each."""
    import numpy as np
    import torch
    from mashbox_b200 import ops
    dev = "cuda:0"
    H, KV, HD, page = a.heads, a.kv_heads, a.head_dim, 16
    Q, ctx, B = a.queries, a.keys, a.batch
    G = H // KV
    gen = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    err = ops.new_error_word(dev)

    def timed(f, n):
        for _ in range(3):
            f()
        ts = []
        for _ in range(n):
            flush.zero_()
            e0, e1 = ev(), ev()
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    out = {"config": dict(heads=H, kv_heads=KV, head_dim=HD, page_size=page)}
    # ---- prompt form: one sequence, its last Q tokens are the step's
    pages = -(-ctx // page)
    pool = (torch.randn(2, pages, KV, page, HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    table = torch.randperm(pages, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(dev).reshape(1, pages)
    q = (torch.randn(Q, H * HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    o = torch.empty(Q, H * HD, device=dev, dtype=torch.bfloat16)
    args = (i32([0]), i32([Q]), i32([ctx - Q]))
    zero, none = i32([0]), i32([-1])
    flops = 4.0 * HD * H * sum(min(ctx, ctx - Q + t + 1) for t in range(Q))
    res = {"queries": Q, "keys": ctx}
    if ops.attention_tc5_supports(HD, page):
        rows = ops.attention_tc5_rows()
        items = i32([v for m in range(-(-Q * G // rows) - 1, -1, -1) for v in (0, m, 0, 1)])
        n = items.numel() // 4
        us = timed(lambda: ops.attention_tc5(q, H * HD, o, pool[0], pool[1], items, n, *args, zero, table, H, KV, HD, page,
                                             pages, None, HD ** -0.5, err), a.steps)
        res["tcgen05_us"], res["tcgen05_tflops"] = us, flops / us / 1e6
    items = i32([v for m in range(-(-Q * G // 64) - 1, -1, -1) for v in (0, m, 0, 1)])
    n = items.numel() // 4
    us = timed(lambda: ops.attention_tma(q, H * HD, o, pool[0], pool[1], items, n, False, *args, none, zero, table,
                                         None, None, 1, H, KV, HD, page, pages, None, HD ** -0.5, err), a.steps)
    res["mma_sync_us"], res["mma_sync_tflops"] = us, flops / us / 1e6
    out["prompt_form"] = res
    del pool
    # ---- decode form: B sequences of ctx tokens, one token each, the keys cut into the splits the mixer would choose
    pages = B * -(-ctx // page)
    pool = (torch.randn(2, pages, KV, page, HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(B, -1)
    q = (torch.randn(B, H * HD, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    o = torch.empty(B, H * HD, device=dev, dtype=torch.bfloat16)
    ns = max(1, min(32, -(-296 // (B * KV)), ctx // 128))
    ns = 1 << (ns.bit_length() - 1)
    items = i32([v for s in range(B) for sp in range(ns) for v in (s, 0, sp, ns)])
    part_o, part_ml = torch.empty(B * H * ns, HD, device=dev), torch.empty(B * H * ns, 2, device=dev)
    rows, ones, last = i32(list(range(B))), i32([1] * B), i32([ctx - 1] * B)
    us = timed(lambda: ops.attention_tma(q, H * HD, o, pool[0], pool[1], items, B * ns, True, rows, ones, last, rows, rows,
                                         table, part_o, part_ml, ns, H, KV, HD, page, pages, None, HD ** -0.5, err,
                                         merge=ns > 1), a.steps)
    nbytes = B * ctx * KV * HD * 2 * 2
    out["decode_form"] = {"batch": B, "keys": ctx, "splits": ns, "us": us, "gbs": nbytes / us / 1e3,
                          "frac_of_hbm_peak": nbytes / us / 1e3 / peaks()["hbm_gbs"]}
    ops.check_error_word(err)
    print(json.dumps({"impl": "ours", "attention": out, "note": "CUDA-event time of single launches after an L2 flush"}))
    return 0


def run_kernels(a):
    """Times this repo's matrix-product and attention kernels next to the library's on the layer shapes of the
    configuration (2,048 tokens and a decode batch), one JSON line; also the workload of the ncu captures of single
    kernels (few launches, under 2 GB on the device)."""
    import torch
    from mashbox_b200 import ops
    dev = "cuda:0"
    c = baseline_config()
    D, F, QKV, V = c.hidden, c.intermediate, (c.num_heads + 2 * c.num_kv_heads) * c.head_dim, c.vocab
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(f, n=a.steps):
        for _ in range(max(3, a.warmup)):
            f()
        ts = []
        for _ in range(n):
            flush.zero_()                                   # L2 is flushed between timed launches
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    out = {}
    T = a.prefill_tokens
    for name, M, K in (("qkv", QKV, D), ("o", D, D), ("gate_up", 2 * F, D), ("down", D, F)):
        x, w = rnd(T, K), rnd(M, K)
        y = torch.empty(T, M, device=dev, dtype=torch.bfloat16)
        own = timed(lambda: ops.linear_tc5(x, w, y, "plain"))
        lib = timed(lambda: torch.mm(x, w.t(), out=y))
        fl = 2 * T * M * K
        out[f"prefill_{name}"] = {"own_us": own, "library_us": lib, "own_tflops": fl / own / 1e6, "library_tflops": fl / lib / 1e6}
    x, w = rnd(T, D), rnd(2 * F, D)
    y = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
    out["prefill_gate_up_swiglu_fused"] = {"own_us": timed(lambda: ops.linear_tc5(x, w, y, "swiglu"))}
    # decode batch: every product as a captured graph of launches over different weights (more than the L2 holds), so the
    # figure is the time from launch to launch inside a step; library product against the matrix-vector kernel (at most
    # 4 tokens) and the weight-streaming kernel with its folded forms
    def chained(f, n_w):
        for i in range(n_w):
            f(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n_w):
                f(i)
        g.replay()
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / n_w)
        return statistics.median(ts)

    B = a.batch
    for name, M, K in (("o", D, D), ("qkv", QKV, D), ("down", D, F), ("gate_up", 2 * F, D)):
        n_w = max(8, int(600e6 // (M * K * 2)))
        ws = [rnd(M, K) for _ in range(n_w)]
        x, y = rnd(B, K), torch.empty(B, M, device=dev, dtype=torch.bfloat16)
        h = torch.randn(B, K, device=dev, generator=gen)
        hs = torch.randn(B, M, device=dev, generator=gen)
        nw, nw_out = torch.ones(K, device=dev), torch.ones(M, device=dev)
        sums_in = torch.full(((K + 31) // 32, 16), 32.0, device=dev)
        sums_out, scaled_out = torch.empty((M + 31) // 32, 16, device=dev), torch.empty(B, M, device=dev, dtype=torch.bfloat16)
        ops.set_pdl(False)
        r = {"library_us": chained(lambda i: torch.mm(x, ws[i].t(), out=y), n_w),
             "stream_plain_launch_us": chained(lambda i: ops.linear_stream(x, ws[i], y, "plain"), n_w)}
        ops.set_pdl(True)           # from here on as the engine launches them: programmatic dependent launch
        r.update({"stream_us": chained(lambda i: ops.linear_stream(x, ws[i], y, "plain"), n_w),
                  "stream_of_normalised_us": chained(lambda i: ops.linear_stream(x, ws[i], y, "plain", sums_in, 1e-5), n_w),
                  "stream_residual_us": chained(lambda i: ops.linear_stream_residual(x, ws[i], hs, None, sums_out, nw_out, scaled_out), n_w)})
        if B <= 4:
            # the matrix-vector kernels in the forms the engine runs at one token: with the residual add; of the
            # normalised stream (the norm inside the kernel), for gate/up with SwiGLU
            r["gemv_us"] = chained(lambda i: ops.linear_gemv(x, ws[i], y, "plain"), n_w)
            r["gemv_residual_us"] = chained(lambda i: ops.linear_gemv_residual(x, ws[i], hs), n_w)
            if K < 8192 and name != "gate_up":
                r["gemv_of_normalised_us"] = chained(lambda i: ops.linear_gemv_normed(h, nw, 1e-5, ws[i], y), n_w)
            if name == "gate_up":
                act1 = torch.empty(B, F, device=dev, dtype=torch.bfloat16)
                r["gemv_of_normalised_swiglu_us"] = chained(lambda i: ops.linear_gemv_normed(h, nw, 1e-5, ws[i], act1, "swiglu"), n_w)
        if name == "gate_up":
            act, hh = torch.empty(B, F, device=dev, dtype=torch.bfloat16), torch.empty(B, K, device=dev, dtype=torch.bfloat16)
            r["stream_of_normalised_swiglu_us"] = chained(lambda i: ops.linear_stream(x, ws[i], act, "swiglu", sums_in, 1e-5), n_w)
            r["norm_library_gate_us"] = chained(lambda i: (ops.add_rmsnorm(h, None, None, nw, 1e-5, hh, None),
                                                           torch.mm(hh, ws[i].t(), out=y), ops.swiglu(y, act)), n_w)
        r["ideal_us_at_peak"] = M * K * 2 / peaks()["hbm_gbs"] / 1e3
        out[f"decode_b{B}_{name}"] = r
        del ws
    ops.check_error_word(ops.error_word(dev))
    print(json.dumps({"impl": "ours", "kernels": out, "note": "prefill: CUDA-event time of single launches after an L2 flush (launch gaps "
                      "of the Python caller are inside); decode: per launch inside a captured graph of launches over different weights"}))
    return 0


# ---------------------------------------------------------------------------------------------------- another design
# Layer sizes that resemble real models, for `--design luzosun`: the Luzosun decoder beside the Llama decoder of equal
# size -- the same width, layers, query and kv heads, q/k/v rows (two maps of `dim` against one head of 2 dim, values of
# vdim = 2 dim), the same number of feed-forward weights (two matrices of 1.5 F against three of F).
DESIGN_SIZES = {
    "1b": dict(width=2048, heads=32, kv_heads=8, dim=32, ff=8192, block=2048),
    "3b": dict(width=3072, heads=24, kv_heads=8, dim=64, ff=8192, block=4096),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=64, ff=14336, block=8192),
}


def design_configs(size, layers, vocab=32000):
    from mashbox_b200.config.llama import LlamaConfig
    from mashbox_b200.config.luzosun import LuzosunConfig, LuzosunLayer, LuzosunMixer
    z = DESIGN_SIZES[size]
    D, H, KV, dim = z["width"], z["heads"], z["kv_heads"], z["dim"]
    own = LuzosunMixer(heads=H, kv_heads=KV, dim=dim, vdim=2 * dim, diff=0.25, scale=dim ** -0.5, conv=4,
                       mask_size=z["block"], rot_base=10000.0, rot_dims=dim // 2, rot_factor=2.0)
    import dataclasses
    lz = LuzosunConfig("Luzosun", width=D, vocab=vocab, embedding_scale=1.0, norm_eps=1e-6, canon_taps=4, layers=tuple(
        LuzosunLayer("attention", own if i % 2 == 0 else dataclasses.replace(own, kv_from=i - 1), z["ff"] * 3 // 2)
        for i in range(layers)))
    ll = LlamaConfig(architecture="LlamaForCausalLM", num_layers=layers, hidden=D, num_heads=H, num_kv_heads=KV,
                     head_dim=2 * dim, intermediate=z["ff"], vocab=vocab, rms_eps=1e-6, rope_theta=10000.0,
                     rope_scaling=None, tie_embeddings=False, attention_bias=True, max_position=131072)
    return lz, ll


# Layer sizes for `--design sufopel`: three delta-rule layers to one latent-attention layer (which ends each run of four),
# routed experts in all but the first layer, a per-layer token input.  Heads of 128 x 128, latents of 128 values (the head
# sizes the engine's TMA and tcgen05 attention kernels take; models of this kind keep 512), experts of F values of which
# `top` of `experts` are chosen.  The Llama decoder beside it has the same width, layers and heads and as many
# feed-forward weights as a token's chosen experts.
SUFOPEL_SIZES = {
    "1b": dict(width=2048, heads=16, dim=128, q_rank=768, kv_rank=128, ff=1408, experts=64, top=6, groups=8, keep=4, rank=128,
               side=256),
    "3b": dict(width=3072, heads=24, dim=128, q_rank=1024, kv_rank=128, ff=1536, experts=64, top=6, groups=8, keep=4, rank=128,
               side=256),
    "8b": dict(width=4096, heads=32, dim=128, q_rank=1536, kv_rank=128, ff=2048, experts=64, top=8, groups=8, keep=4, rank=128,
               side=256),
}


def sufopel_configs(size, layers, vocab=32000, context=8192):
    from mashbox_b200.config.llama import LlamaConfig
    from mashbox_b200.config.sufopel import DeltaMixer, DenseFF, LatentMixer, RoutedFF, SufopelConfig, SufopelLayer
    z = SUFOPEL_SIZES[size]
    D, H, dim = z["width"], z["heads"], z["dim"]
    dl = DeltaMixer(heads=H, kv_heads=H, dim=dim, vdim=dim, conv=4, a_rank=z["rank"], g_rank=z["rank"])
    la = LatentMixer(heads=H, dim=dim, vdim=dim, q_rank=z["q_rank"], kv_rank=z["kv_rank"], scale=dim ** -0.5)
    moe = RoutedFF(ff=z["ff"], limit=7.0, experts=z["experts"], top=z["top"], groups=z["groups"], keep=z["keep"])
    sf = SufopelConfig("Sufopel", width=D, vocab=vocab, max_positions=context + 2048, embedding_scale=1.0, logit_scale=1.0,
                       norm_eps=1e-6, side_dim=z["side"], layers=tuple(
        SufopelLayer("latent_attention" if i % 4 == 3 else "channel_delta", la if i % 4 == 3 else dl,
                     DenseFF(z["ff"] * z["top"]) if i == 0 else moe) for i in range(layers)))
    ll = LlamaConfig(architecture="LlamaForCausalLM", num_layers=layers, hidden=D, num_heads=H, num_kv_heads=max(1, H // 4),
                     head_dim=dim, intermediate=z["ff"] * z["top"], vocab=vocab, rms_eps=1e-6, rope_theta=10000.0,
                     rope_scaling=None, tie_embeddings=False, attention_bias=False, max_position=131072)
    return sf, ll


# Layer sizes for `--design tosevik`: three retention layers to one layer of two mixers side by side (attention with
# sigmoid weights beside retention), routed experts with a gated shared expert in every layer.  Heads of 128 x 128, a kv
# head to four query heads.  The Sufopel decoder beside it -- the closest design the engine has: recurrent layers with a
# matrix state per head, one attention layer in four, routed experts -- has the same width, layers, heads, head sizes and
# experts.
TOSEVIK_SIZES = {
    "1b": dict(width=2048, heads=16, dim=128, ff=1408, experts=64, top=6, groups=8, keep=4, shared=2816),
    "3b": dict(width=3072, heads=24, dim=128, ff=1536, experts=64, top=6, groups=8, keep=4, shared=3072),
    "8b": dict(width=4096, heads=32, dim=128, ff=2048, experts=64, top=8, groups=8, keep=4, shared=4096),
}


def tosevik_configs(size, layers, vocab=32000, context=8192):
    from mashbox_b200.config.tosevik import ExpertsFF, PairMixer, RetentionMixer, SigmoidMixer, TosevikConfig, TosevikLayer
    z = TOSEVIK_SIZES[size]
    D, H, dim = z["width"], z["heads"], z["dim"]
    decay = tuple(1.0 - 2.0 ** (-5.0 - 3.0 * h / max(1, H - 1)) for h in range(H))
    ret = RetentionMixer(heads=H, dim=dim, vdim=dim, decay=decay, rot_dims=dim, rot_base=10000.0)
    sig = SigmoidMixer(heads=H, kv_heads=max(1, H // 4), dim=dim, vdim=dim, scale=dim ** -0.5, temp_coef=0.1, temp_every=1024)
    moe = ExpertsFF(ff=z["ff"], experts=z["experts"], top=z["top"], scale=2.5, groups=z["groups"], keep=z["keep"],
                    shared_ff=z["shared"])
    tv = TosevikConfig("Tosevik", width=D, vocab=vocab, norm_eps=1e-6, layers=tuple(
        TosevikLayer("parallel", PairMixer(sig, ret), moe) if i % 4 == 3 else TosevikLayer("retention", ret, moe)
        for i in range(layers)))
    sf = sufopel_configs(size, layers, vocab, context)[0]
    return tv, sf


# Layer sizes for `--design fipitar`: a layer of two mixers side by side first (attention with normed heads, capped scores
# and a gate per head over keys of 128 and values of 64, beside a state-space recurrence with heads of 64 over a state of
# 128), two layers of gated linear attention (heads of 128 x 128), a latent-attention layer last (latents of 128 with a
# rotated strip of 64), a dense clamped feed-forward in every layer.  The Sufopel decoder beside it -- the closest design
# the engine has: three recurrent layers with a matrix state per head and a decay per key channel, then a latent-attention
# layer -- has the same width, layers, heads and head sizes and, here, a dense feed-forward of as many weights in every
# layer and no token input.
FIPITAR_SIZES = {
    "1b": dict(width=2048, heads=16, dim=128, q_rank=768, kv_rank=128, rot=64, ff=8448),
    "3b": dict(width=3072, heads=24, dim=128, q_rank=1024, kv_rank=128, rot=64, ff=9216),
    "8b": dict(width=4096, heads=32, dim=128, q_rank=1536, kv_rank=128, rot=64, ff=16384),
}


def fipitar_configs(size, layers, vocab=32000, context=8192):
    from mashbox_b200.config import fipitar as F
    from mashbox_b200.config.sufopel import DeltaMixer, DenseFF, LatentMixer, SufopelConfig, SufopelLayer
    z = FIPITAR_SIZES[size]
    D, H, dim = z["width"], z["heads"], z["dim"]
    left = F.AttentionMixer(heads=H, kv_heads=max(1, H // 4), dim=dim, vdim=dim // 2, scale=dim ** -0.5, softcap=30.0,
                            rot=F.Rotation(dim // 2, 500000.0))
    right = F.SsdMixer(heads=D // 64, vdim=64, state=128, groups=1, norm_groups=8, conv=4)
    pair = F.PairMixer(left, right, 0.6, 1.1)
    gla = F.GlaMixer(heads=H, dim=dim, vdim=dim, tau=16.0, a_rank=16)
    lat = F.LatentMixer(heads=H, dim=dim, vdim=dim, q_rank=z["q_rank"], kv_rank=z["kv_rank"], scale=(dim + z["rot"]) ** -0.5,
                        rot_dim=z["rot"], rot=F.Rotation(z["rot"], 250000.0, (2.0, 2048.0, 32.0, 1.0)))
    kinds = (("parallel", pair), ("gla", gla), ("gla", gla), ("latent_attention", lat))
    fp = F.FipitarConfig("Fipitar", width=D, vocab=vocab, norm_eps=1e-6, layers=tuple(
        F.FipitarLayer(*kinds[i % 4], F.DenseFF(z["ff"], 7.0)) for i in range(layers)))
    dl = DeltaMixer(heads=H, kv_heads=H, dim=dim, vdim=dim, conv=4, a_rank=16, g_rank=16)
    la = LatentMixer(heads=H, dim=dim, vdim=dim, q_rank=z["q_rank"], kv_rank=z["kv_rank"], scale=dim ** -0.5)
    sf = SufopelConfig("Sufopel", width=D, vocab=vocab, max_positions=context + 2048, embedding_scale=1.0, logit_scale=1.0,
                       norm_eps=1e-6, side_dim=None, layers=tuple(
        SufopelLayer("latent_attention" if i % 4 == 3 else "channel_delta", la if i % 4 == 3 else dl, DenseFF(z["ff"]))
        for i in range(layers)))
    return fp, sf


def fipitar_kernels(a, z, P, B, ctx, pk):
    """The kernels of the Fipitar decoder, each beside the like kernel of the Sufopel (or Llama) decoder at equal sizes:
    CUDA-event time of single launches after an L2 flush, and the fraction of the measured peak that the algorithmic bytes
    (copy bandwidth) or FLOPs (bf16 tensor throughput) come to."""
    import torch
    from mashbox_b200 import ops
    from mashbox_b200.parts.attention import PagedAttention
    dev = "cuda:0"
    D, H, dim, R, rd, F, page = z["width"], z["heads"], z["dim"], z["kv_rank"], z["rot"], z["ff"], 16
    KV, HS, PS, NS = max(1, H // 4), D // 64, 64, 128
    gen = torch.Generator(device=dev).manual_seed(0)
    bf = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    f32 = lambda *s: torch.randn(*s, generator=gen, device=dev) * 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    err = ops.new_error_word(dev)

    def timed(f):
        for _ in range(3):
            f()
        ts = []
        for _ in range(max(5, a.steps // 4)):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    mem = lambda us, nbytes: {"us": us, "gbs": nbytes / us / 1e3, "frac_of_copy_peak": nbytes / us / 1e3 / pk["hbm_gbs"]}
    mat = lambda us, flops: {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / pk["bf16_tflops"]}
    res = {}
    # ---- the recurrences: a prompt of P tokens; B sequences of one token (state in, state out)
    for form, N, S in (("prompt", P, 1), ("decode", B, B)):
        seq = (i32([i * (N // S) for i in range(S)]), i32([N // S] * S), i32(list(range(S))))
        q, k, v, o = f32(N, H * dim), f32(N, H * dim), f32(N, H * dim), f32(N, H * dim)
        g, beta = torch.rand(N, H * dim, generator=gen, device=dev), torch.rand(N, H, generator=gen, device=dev)
        state = torch.zeros(S, H * dim * dim, device=dev)
        us = timed(lambda: ops.gated_scan(q, k, v, g, o, state, seq, H, H, dim, dim, False))
        res[f"gla_scan_{form}"] = mem(us, 2 * S * H * dim * dim * 4 + N * H * dim * 5 * 4)
        us = timed(lambda: ops.delta_rule(q, k, v, g, beta, o, state, seq, H, H, dim, dim))
        res[f"delta_rule_sufopel_{form}"] = mem(us, 2 * S * H * dim * dim * 4 + N * H * dim * 5 * 4)
        q, k, v, o = f32(N, NS), f32(N, NS), f32(N, HS * PS), f32(N, HS * PS)
        g = torch.rand(N, HS, generator=gen, device=dev)
        state = torch.zeros(S, HS * NS * PS, device=dev)
        us = timed(lambda: ops.gated_scan(q, k, v, g, o, state, seq, HS, 1, NS, PS, True))
        res[f"ssd_scan_{form}"] = mem(us, 2 * S * HS * NS * PS * 4 + N * (2 * NS + 2 * HS * PS + HS) * 4)
    # ---- attention: P prompt tokens; B tokens over ctx keys.  The side-by-side layer's attention beside Llama's at equal
    # heads and keys (its values are half as wide); latent attention with a rotated strip beside Sufopel's without one
    left = PagedAttention(H, KV, dim, None, dim ** -0.5, vdim=dim // 2, softcap=30.0, sinks=True, gated=True)
    llama = PagedAttention(H, KV, dim)
    lat = PagedAttention(H, 1, R + rd, None, (dim + rd) ** -0.5, vdim=R, sinks=True)
    lat.general = True
    suf = PagedAttention(H, 1, R, None, dim ** -0.5)
    sinks = f32(H)
    for name, core, wk, wv, shared in (("attention_fipitar", left, dim, dim // 2, False), ("attention_llama", llama, dim, dim, False),
                                       ("latent_attention_fipitar", lat, R + rd, R, True),
                                       ("latent_attention_sufopel", suf, R, R, True)):
        for form, N, S, klen in (("prompt", P, 1, P), ("decode", B, B, ctx)):
            pages = S * -(-klen // page)
            table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(S, -1)
            kp = bf(pages, core.KV, page, wk)
            vp = kp if shared else bf(pages, core.KV, page, wv)
            q, o = bf(N, H * wk + 8 * ((H + 7) // 8)), torch.empty(N, H * wv, device=dev, dtype=torch.bfloat16)
            q_len = [N // S] * S
            ctx_ = _PlanContext(ops, dev, q_len, [klen - n for n in q_len], page, pages, err)
            core.prepare(ctx_)
            ctx_.inputs.upload()
            extra = dict(sinks=sinks) if core.general else {}
            if core is left:
                extra["gate"] = q[:, H * wk:H * wk + H]
            us = timed(lambda: core.attend(ctx_, q, q.stride(0), o, table, kp, vp, **extra))
            nbytes = S * klen * core.KV * (wk + (0 if shared else wv)) * 2 + N * H * (wk + wv) * 2
            if form == "prompt":
                res[f"{name}_prompt"] = mat(us, 2 * H * (wk + wv) * P * P / 2)
            else:
                res[f"{name}_decode"] = mem(us, nbytes)
    # ---- rows: what a sublayer's output passes on its way into the stream; the feed-forward's gate; heads before attention
    for form, N in (("prompt", P), ("decode", B)):
        x, y1, y2, w, b = f32(N, D), bf(N, D), bf(N, D), f32(D), f32(D)
        nrm, cp = torch.empty(N, D, device=dev, dtype=torch.bfloat16), torch.empty(N, D, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.ln_add(x, y1, w, b, 1e-6, cp))
        res[f"ln_add_{form}"] = mem(us, N * D * (4 + 4 + 2 + 2))
        us = timed(lambda: ops.ln_add(x, y1, w, b, 1e-6, cp, y2, 0.6, 1.1))
        res[f"ln_add_two_outputs_{form}"] = mem(us, N * D * (4 + 4 + 2 + 2 + 2))
        us = timed(lambda: ops.post_norm_add(x, y1, w, 1e-6, w, 1e-6, nrm))
        res[f"post_norm_add_sufopel_{form}"] = mem(us, N * D * (4 + 4 + 2 + 2))
        gu, act = bf(N, 2 * F), torch.empty(N, F, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.glu_clamped(gu, act, 7.0))
        res[f"glu_clamped_{form}"] = mem(us, N * F * 6)
        us = timed(lambda: ops.swiglu(gu, act))
        res[f"swiglu_llama_{form}"] = mem(us, N * F * 6)
        S = 1 if form == "prompt" else N
        pages = S * -(-(N // S) // page) + 1
        table = torch.arange(pages - 1, dtype=torch.int32, device=dev).reshape(S, -1)
        positions, tok_row = i32([t % (N // S) for t in range(N)]), i32([t // (N // S) for t in range(N)])
        rows = bf(N, (H + KV) * dim + KV * (dim // 2) + 8 * ((H + 7) // 8))
        kp, vp = bf(pages, KV, page, dim), bf(pages, KV, page, dim // 2)
        freqs, qw = f32(dim // 4).abs(), f32(dim)
        us = timed(lambda: ops.norm_rope_kv_write(rows, qw, qw, 1e-6, freqs, dim // 2, 1, 1.0, positions, tok_row, table, kp, vp, H,
                                                  KV, dim, dim // 2, page, pages, err))
        res[f"norm_rope_kv_write_{form}"] = mem(us, N * ((H + KV) * dim * 2 + KV * (dim // 2)) * 2 + N * KV * dim * 2)
        rows2, kp2, vp2 = bf(N, (H + 2 * KV) * dim), bf(pages, KV, page, dim), bf(pages, KV, page, dim)
        us = timed(lambda: ops.rope_kv_write(rows2, None, positions, tok_row, table, kp2, vp2, freqs, H, KV, dim, dim // 2, 1, page,
                                             pages, err))
        res[f"rope_kv_write_llama_{form}"] = mem(us, N * ((H + KV) * dim * 2 + KV * dim) * 2 + N * 2 * KV * dim * 2)
        # the gates of the recurrences and what follows them
        grow, zz, zb = bf(N, 4 * H * dim), f32(N, H * dim), f32(H * dim)
        q, k, v, g = (torch.empty(N, H * dim, device=dev) for _ in range(4))
        us = timed(lambda: ops.gla_gates(grow, zz, zb, 16.0, q, k, v, g, H, dim, dim))
        res[f"gla_gates_{form}"] = mem(us, N * H * dim * (3 * 2 + 4 + 4 * 4))
        o, out = f32(N, H * dim), torch.empty(N, H * dim, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.gated_rms(o, grow[:, 3 * H * dim:], qw, out, H, dim, 1e-6, silu=True))
        res[f"gated_rms_{form}"] = mem(us, N * H * dim * (4 + 2 + 2))
        C = HS * PS + 2 * NS
        xbc, cb, dt, hb = bf(N, C), f32(C), f32(N, HS), f32(HS)
        q2, k2, v2, g2 = torch.empty(N, NS, device=dev), torch.empty(N, NS, device=dev), torch.empty(N, HS * PS, device=dev), torch.empty(N, HS, device=dev)
        us = timed(lambda: ops.ssd_gates(xbc, cb, dt, hb, hb, q2, k2, v2, g2, HS, 1, PS, NS))
        res[f"ssd_gates_{form}"] = mem(us, N * (C * 2 + HS * 4 + (2 * NS + HS * PS + HS) * 4))
        o2, zg, wn, out2 = f32(N, HS * PS), bf(N, HS * PS), f32(HS * PS), torch.empty(N, HS * PS, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.ssd_out(o2, xbc, cb, hb, zg, wn, out2, HS, PS, 8, 1e-6))
        res[f"ssd_out_{form}"] = mem(us, N * HS * PS * (4 + 2 + 2 + 2))
    return res


def run_design(a):
    """`--design luzosun --size 1b|3b|8b`: prefill and decode throughput of the Luzosun decoder and of the Llama decoder
    of equal size through the step function (random bf16 weights, `--layers` layers, default 4), and the kernels that
    differ between the two timed alone with their bytes or FLOPs against the measured peaks.  One JSON line."""
    import numpy as np
    import torch
    from mashbox_b200 import ops
    from mashbox_b200.config.registry import architecture
    from mashbox_b200.engine.engine import Engine
    from mashbox_b200.weights.random_init import RandomSource
    torch.cuda.set_device(0)
    dev = "cuda:0"
    layers = a.layers or 4
    design = a.design
    other = "llama"
    if design == "fipitar":
        z, other = FIPITAR_SIZES[a.size], "sufopel"
        cfgs = dict(zip((design, other), fipitar_configs(a.size, layers, context=a.context)))
        single_kernels = fipitar_kernels
    elif design == "tosevik":
        z, other = TOSEVIK_SIZES[a.size], "sufopel"
        cfgs = dict(zip((design, other), tosevik_configs(a.size, layers, context=a.context)))
        single_kernels = tosevik_kernels
    elif design == "sufopel":
        z = SUFOPEL_SIZES[a.size]
        cfgs = dict(zip((design, "llama"), sufopel_configs(a.size, layers, context=a.context)))
        single_kernels = sufopel_kernels
    else:
        z = DESIGN_SIZES[a.size]
        cfgs = dict(zip((design, "llama"), design_configs(a.size, layers)))
        single_kernels = design_kernels
    K, W, B = a.steps, max(3, a.warmup), a.batch
    ctx = min(a.context, z.get("block", a.context))    # a Luzosun query reads its block of positions: both read `ctx` keys
    P = a.prefill_tokens
    pk = peaks()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    gen = torch.Generator().manual_seed(1)
    clocks = Clocks()
    clocks.start()
    out = {}
    if a.kernels:                               # the single kernels only (also the workload of their ncu captures)
        print(json.dumps({"impl": "ours", "design": design, "size": a.size, "prefill_tokens": P, "batch": B, "context": ctx,
                          "peaks": pk, "kernels": single_kernels(a, z, P, B, ctx, pk), "clocks": clocks.stop()}))
        return 0
    for name, cfg in cfgs.items():
        rand_ids = lambda n: torch.randint(0, cfg.vocab, (n,), generator=gen).tolist()
        per_request = -(-(ctx + 64) // 64) * 64
        shapes = architecture(cfg.architecture).stored_tensors(cfg)
        eng = Engine.from_config(cfg, RandomSource(shapes, 0, torch.bfloat16, dev), dtype="bfloat16", device=dev,
                                 page_size=16, max_tokens=B * per_request + max(P, 2048) + 64, max_requests=B + 1,
                                 max_tokens_per_step=max(P, 2048) + B, chunk=max(P, 2048), max_context=max(per_request, P + 64),
                                 cuda_graphs=not a.no_graphs, options=json.loads(a.options) if a.options else None)
        runner, cache = eng.runner, eng.runner.cache
        ms = []
        for i in range(W + 3):                  # a whole prompt of P tokens in one step
            cache.admit("p")
            ids = rand_ids(P)
            torch.cuda.synchronize()
            e0, e1 = ev(), ev()
            e0.record()
            runner.step([("p", ids, [P - 1])])
            e1.record()
            torch.cuda.synchronize()
            cache.release("p")
            if i >= W:
                ms.append(e0.elapsed_time(e1))
        pre = statistics.median(ms)
        rids = [f"d{i}" for i in range(B)]      # B requests of ctx - K - W tokens, then single tokens
        for r in rids:
            cache.admit(r)
            n = ctx - K - W - 1
            for lo in range(0, n, 2048):
                runner.step([(r, rand_ids(min(2048, n - lo)), [])])
        toks = rand_ids(B)
        step = lambda: runner.step([(r, [t], [0]) for r, t in zip(rids, toks)])
        for _ in range(W):
            step()
        torch.cuda.synchronize()
        l0 = ops.COUNTERS["launches"]
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(K):
            step()
        e1.record()
        torch.cuda.synchronize()
        dec = e0.elapsed_time(e1) / K
        runner.check()
        out[name] = {"prefill_tokens_per_s": P / (pre / 1e3), "prefill_ms": pre, "decode_tokens_per_s": B / (dec / 1e3),
                     "decode_ms_per_step": dec, "decode_launches_per_step": (ops.COUNTERS["launches"] - l0) / K,
                     "weights_bytes": sum(int(np.prod(sh)) for sh, _ in shapes.values()) * 2}
        for r in rids:
            cache.release(r)
        del eng, runner, cache
        torch.cuda.empty_cache()
    out["kernels"] = single_kernels(a, z, P, B, ctx, pk)
    out[f"ratio_{design}_to_{other}"] = {k: out[design][k] / out[other][k] for k in ("prefill_tokens_per_s", "decode_tokens_per_s")}
    print(json.dumps({"impl": "ours", "design": design, "size": a.size, "layers": layers, "prefill_tokens": P, "batch": B,
                      "context": ctx, "dtype": "bf16", "data": "synthetic", "peaks": pk, "clocks": clocks.stop(), **out}))
    return 0


def sufopel_kernels(a, z, P, B, ctx, pk):
    """The kernels of the Sufopel decoder, each beside the Llama decoder's kernel of the like job at equal sizes: CUDA-event
    time of single launches after an L2 flush, and the fraction of the measured peak (copy bandwidth for the memory-bound
    ones, bf16 tensor throughput for the products) that the algorithmic bytes or FLOPs come to."""
    import torch
    from mashbox_b200 import ops
    from mashbox_b200.parts.attention import PagedAttention
    dev = "cuda:0"
    D, H, dim, R, F, E, top, page = z["width"], z["heads"], z["dim"], z["kv_rank"], z["ff"], z["experts"], z["top"], 16
    gen = torch.Generator(device=dev).manual_seed(0)
    bf = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    f32 = lambda *s: torch.randn(*s, generator=gen, device=dev) * 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    err = ops.new_error_word(dev)

    def timed(f):
        for _ in range(3):
            f()
        ts = []
        for _ in range(max(5, a.steps // 4)):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    mem = lambda us, nbytes: {"us": us, "gbs": nbytes / us / 1e3, "frac_of_copy_peak": nbytes / us / 1e3 / pk["hbm_gbs"]}
    mat = lambda us, flops: {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / pk["bf16_tflops"]}
    res = {}
    # ---- the recurrence: a prompt of P tokens; B sequences of one token (state in, state out)
    for form, N, S in (("prompt", P, 1), ("decode", B, B)):
        q, k = f32(N, H * dim), f32(N, H * dim)
        v, g, beta, o = f32(N, H * dim), torch.rand(N, H * dim, generator=gen, device=dev), torch.rand(N, H, generator=gen, device=dev), f32(N, H * dim)
        state = torch.zeros(S, H * dim * dim, device=dev)
        seq = (i32([i * (N // S) for i in range(S)]), i32([N // S] * S), i32(list(range(S))))
        us = timed(lambda: ops.delta_rule(q, k, v, g, beta, o, state, seq, H, H, dim, dim))
        r = mem(us, 2 * S * H * dim * dim * 4 + N * H * dim * 5 * 4)
        r["gflops_fp32"] = N * H * dim * dim * 7 / us / 1e3                 # decay, two dot products, update: 7 per element
        res[f"delta_rule_{form}"] = r
        for lanes in (16, 32):                                                # the same with more threads a column
            ops.delta_rule_lanes(lanes)
            res[f"delta_rule_{form}"][f"us_{lanes}_lanes"] = timed(lambda: ops.delta_rule(q, k, v, g, beta, o, state, seq, H, H, dim, dim))
        ops.delta_rule_lanes(0)
    # ---- Llama's attention at equal heads, beside it: P prompt tokens; B tokens over ctx keys
    att = PagedAttention(H, max(1, H // 4), dim)
    lat = PagedAttention(H, 1, R, None, dim ** -0.5)
    for name, core, width in (("attention_llama", att, dim), ("latent_attention", lat, R)):
        for form, N, S, klen in (("prompt", P, 1, P), ("decode", B, B, ctx)):
            pages = S * -(-klen // page)
            table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(S, -1)
            kp, vp = bf(pages, core.KV, page, width), bf(pages, core.KV, page, width)
            if core is lat:
                vp = kp                                 # a position's latent is key and value at once
            q, o = bf(N, H * width), torch.empty(N, H * width, device=dev, dtype=torch.bfloat16)
            q_len = [N // S] * S
            ctx_ = _PlanContext(ops, dev, q_len, [klen - n for n in q_len], page, pages, err)
            core.prepare(ctx_)
            ctx_.inputs.upload()
            us = timed(lambda: core.attend(ctx_, q, H * width, o, table, kp, vp))
            nbytes = (1 if core is lat else 2) * S * klen * core.KV * width * 2 + 2 * N * H * width * 2
            if form == "prompt":
                res[f"{name}_prompt"] = mat(us, 4 * H * width * P * P / 2)
            else:
                res[f"{name}_decode"] = mem(us, nbytes)
    # ---- the experts: P tokens on tiles; B tokens pair by pair; Llama's feed-forward products of as many weights
    wg, wu, wd = bf(E, F, D), bf(E, F, D), bf(E, D, F)
    for form, N in (("prompt", P), ("decode", B)):
        h = bf(N, D)
        ids = torch.stack([torch.randperm(E, generator=gen, device=dev)[:top] for _ in range(N)]).int().contiguous()
        y = torch.empty(N, top, D, device=dev)
        if form == "prompt":
            act = torch.empty(N * top, F, device=dev, dtype=torch.bfloat16)
            scratch = torch.empty(ops.moe_grouped_scratch(N, top, E), dtype=torch.int32, device=dev)
            us = timed(lambda: ops.moe_grouped(h, ids, wg, wu, wd, y, act, scratch, 7.0, 1.702))
            res["experts_prompt_mma_sync"] = mat(us, 2 * N * top * 3 * F * D)
            T = ops.moe_tc5_tiles(N, top, E)
            wts, out = torch.rand(N, top, generator=gen, device=dev), torch.empty(N, D, device=dev, dtype=torch.bfloat16)
            rows, act2 = torch.empty(128 * T, D, device=dev, dtype=torch.bfloat16), torch.empty(128 * T, F, device=dev, dtype=torch.bfloat16)
            y2, places = torch.empty(128 * T, D, device=dev), torch.empty(N * top + T, dtype=torch.int32, device=dev)
            wgu2 = torch.cat([wg, wu], 1).contiguous()
            us = timed(lambda: ops.moe_tc5(h, ids, wts, wgu2, wd, out, rows, act2, y2, places, 7.0, 1.702))
            res["experts_prompt"] = mat(us, 2 * N * top * 3 * F * D)
            # few rows an expert: every expert's matrices have to be read once, which may take longer than the products
            touched = len(set(ids.flatten().tolist()))
            need = max(2 * N * top * 3 * F * D / (pk["bf16_tflops"] * 1e6), touched * 3 * F * D * 2 / (pk["hbm_gbs"] * 1e3))
            res["experts_prompt"].update(weights_gbs=touched * 3 * F * D * 2 / us / 1e3, frac_of_roofline=need / us)
            del wgu2
            wgu, wdn, a1, o1 = bf(2 * F * top, D), bf(D, F * top), torch.empty(N, F * top, device=dev, dtype=torch.bfloat16), torch.empty(N, D, device=dev, dtype=torch.bfloat16)
            us = timed(lambda: (ops.linear_swiglu(h, wgu, a1), ops.linear(a1, wdn, out=o1)))
            res["feed_forward_llama_prompt"] = mat(us, 2 * N * top * 3 * F * D)
        else:
            us = timed(lambda: ops.moe_experts(h, ids, wg, wu, wd, y, 7.0, 1.702))
            touched = len(set(ids.flatten().tolist()))
            res["experts_decode"] = mem(us, touched * 3 * F * D * 2)
            res["experts_decode"]["experts_touched"] = touched
            wgu, wdn, a1, o1 = bf(2 * F * top, D), bf(D, F * top), torch.empty(N, F * top, device=dev, dtype=torch.bfloat16), torch.empty(N, D, device=dev, dtype=torch.bfloat16)
            us = timed(lambda: (ops.linear_swiglu(h, wgu, a1) if ops.fused_swiglu_supports(N, F * top, D) else
                                ops.linear_stream(h, wgu, a1, "swiglu"), ops.linear(a1, wdn, out=o1)))
            res["feed_forward_llama_decode"] = mem(us, 3 * F * top * D * 2)
    # ---- the norm around a sublayer's output, beside Llama's add + norm
    for form, N in (("prompt", P), ("decode", B)):
        x, delta, w, nrm = f32(N, D), bf(N, D), f32(D), torch.empty(N, D, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.post_norm_add(x, delta, w, 1e-6, w, 1e-6, nrm))
        res[f"post_norm_add_{form}"] = mem(us, N * D * (4 + 4 + 2 + 2))
        us = timed(lambda: ops.add_rmsnorm(x, delta, None, w, 1e-6, nrm))
        res[f"add_norm_llama_{form}"] = mem(us, N * D * (4 + 4 + 2 + 2))
    return res


def tosevik_kernels(a, z, P, B, ctx, pk):
    """The kernels of the Tosevik decoder, each beside the Sufopel decoder's kernel of the like job at equal sizes (the
    recurrence beside the delta rule, attention with sigmoid weights beside latent attention and beside softmax attention
    over as many kv heads, the stream's kernels beside the post norm): CUDA-event time of single launches after an L2
    flush, and the fraction of the measured peak (copy bandwidth for the memory-bound ones, bf16 tensor throughput for
    the products) that the algorithmic bytes or FLOPs come to."""
    import torch
    from mashbox_b200 import ops
    from mashbox_b200.parts.attention import PagedAttention
    from mashbox_b200.parts.sigmoid_attention import SigmoidAttention, geometric_slopes
    dev = "cuda:0"
    D, H, dim, F, E, top, page = z["width"], z["heads"], z["dim"], z["ff"], z["experts"], z["top"], 16
    G = max(1, H // 4)
    gen = torch.Generator(device=dev).manual_seed(0)
    bf = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    f32 = lambda *s: torch.randn(*s, generator=gen, device=dev) * 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    err = ops.new_error_word(dev)

    def timed(f):
        for _ in range(3):
            f()
        ts = []
        for _ in range(max(5, a.steps // 4)):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    mem = lambda us, nbytes: {"us": us, "gbs": nbytes / us / 1e3, "frac_of_copy_peak": nbytes / us / 1e3 / pk["hbm_gbs"]}
    mat = lambda us, flops: {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / pk["bf16_tflops"]}
    res = {}
    # ---- the two recurrences: a prompt of P tokens; B sequences of one token (state in, state out)
    decay = torch.tensor([1.0 - 2.0 ** (-5.0 - 3.0 * h / max(1, H - 1)) for h in range(H)], device=dev)
    for form, N, S in (("prompt", P, 1), ("decode", B, B)):
        q, k, v, o = f32(N, H * dim), f32(N, H * dim) * dim ** -0.5, f32(N, H * dim), f32(N, H * dim)
        state = torch.zeros(S, H * dim * dim, device=dev)
        seq = (i32([i * (N // S) for i in range(S)]), i32([N // S] * S), i32(list(range(S))))
        nbytes = 2 * S * H * dim * dim * 4 + N * H * dim * 4 * 4
        for name, chunked in (("retention_split", True), ("retention_scan", False)):
            if chunked and form == "decode":
                continue
            us = timed(lambda: ops.retention(q, k, v, decay, o, state, seq, H, dim, dim, chunked=chunked))
            r = mem(us, nbytes)
            r["gflops_fp32"] = N * H * dim * dim * 4 / us / 1e3                  # decay + write, read: 4 per element and token
            res[f"{name}_{form}"] = r
            state.zero_()
        # the form the mixer takes at this size
        picked = "retention_split" if ops.retention_splits(N, S, H, dim) else "retention_scan"
        res[f"retention_{form}"] = dict(res[f"{picked}_{form}"], form=picked)
        g, beta = torch.rand(N, H * dim, generator=gen, device=dev), torch.rand(N, H, generator=gen, device=dev)
        us = timed(lambda: ops.delta_rule(q, k, v, g, beta, o, state, seq, H, H, dim, dim))
        res[f"delta_rule_sufopel_{form}"] = mem(us, nbytes + N * H * dim * 4)
        # what stands around the recurrence: rotation and widening of q, k, v; the unit-rms heads times the gate
        rows, freqs = bf(N, 4 * H * dim), torch.rand(dim // 2, generator=gen, device=dev)
        pos = torch.arange(N, dtype=torch.int32, device=dev)
        us = timed(lambda: ops.retention_prep(rows, 0, H * dim, 2 * H * dim, pos, freqs, q, k, v, H, dim, dim, dim, dim ** -0.5))
        res[f"retention_prep_{form}"] = mem(us, N * H * dim * 3 * (2 + 4))
        gated = torch.empty(N, H * dim, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.gated_rms(o, rows[:, 3 * H * dim:], None, gated, H, dim, 1e-6, silu=True))
        res[f"retention_gated_norm_{form}"] = mem(us, N * H * dim * (4 + 2 + 2))
    # ---- attention: sigmoid weights (H heads on G kv heads); beside it softmax attention of the same heads, and Sufopel's
    #      latent attention (one shared row of `dim` values per position)
    sig = SigmoidAttention(D, H, G, dim, dim, dim ** -0.5, 1e-6, slopes=geometric_slopes(H, 8.0), q_temp=(0.1, 1024))
    sig.slopes, sig.pb = torch.tensor(sig.slope_values, device=dev), f32(H)
    att = PagedAttention(H, G, dim)
    lat = PagedAttention(H, 1, dim, None, dim ** -0.5)
    for name, core, KV in (("sigmoid_attention", sig, G), ("attention_softmax", att, G), ("latent_attention_sufopel", lat, 1)):
        for form, N, S, klen in (("prompt", P, 1, P), ("decode", B, B, ctx)):
            pages = S * -(-klen // page)
            table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(S, -1)
            kp, vp = bf(pages, KV, page, dim), bf(pages, KV, page, dim)
            if core is lat:
                vp = kp
            q, o = bf(N, H * dim), torch.empty(N, H * dim, device=dev, dtype=torch.bfloat16)
            q_len = [N // S] * S
            ctx_ = _PlanContext(ops, dev, q_len, [klen - n for n in q_len], page, pages, err)
            core.prepare(ctx_)
            ctx_.inputs.upload()
            if core is sig:
                us = timed(lambda: core.attend(ctx_, q, o, table, kp, vp))
            else:
                us = timed(lambda: core.attend(ctx_, q, H * dim, o, table, kp, vp))
            nbytes = (1 if core is lat else 2) * S * klen * KV * dim * 2 + 2 * N * H * dim * 2
            if form == "prompt":
                res[f"{name}_prompt"] = mat(us, 4 * H * dim * P * P / 2)
                if core is sig:             # a weight goes into the second product as two bf16 numbers: 3 products, not 2
                    res[f"{name}_prompt"]["tflops_issued"] = 6 * H * dim * P * P / 2 / us / 1e6
                    # the same on mma.sync tiles (the form that takes every pair of head sizes)
                    ctx_m = _PlanContext(ops, dev, q_len, [klen - n for n in q_len], page, pages, err)
                    ctx_m.options["attention_prefill_kernel"] = "mma"
                    core.prepare(ctx_m)
                    ctx_m.inputs.upload()
                    res[f"{name}_mma_prompt"] = mat(timed(lambda: core.attend(ctx_m, q, o, table, kp, vp)), 4 * H * dim * P * P / 2)
            else:
                res[f"{name}_decode"] = mem(us, nbytes)
        if core is sig:                      # the kernel in front of it: norms over whole rows, temperature, cache write
            for form, N in (("prompt", P), ("decode", B)):
                rows, qn = bf(N, (H + 2 * G) * dim), torch.empty(N, H * dim, device=dev, dtype=torch.bfloat16)
                pages = -(-N // page)
                table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, -1)
                kp, vp = bf(pages, G, page, dim), bf(pages, G, page, dim)
                pos, row = torch.arange(N, dtype=torch.int32, device=dev), torch.zeros(N, dtype=torch.int32, device=dev)
                qw, kw = f32(H * dim), f32(G * dim)
                us = timed(lambda: ops.sigmoid_attention_prep(rows, qw, kw, pos, row, table, qn, kp, vp, H, G, dim, dim, page,
                                                               pages, 1e-6, 0.1, 1024, err))
                res[f"sigmoid_attention_prep_{form}"] = mem(us, 2 * N * (H + 2 * G) * dim * 2)
    # ---- the experts: the same kernels as Sufopel's with another activation and, in the last one, the gated shared expert
    wg, wu, wd = bf(E, F, D), bf(E, F, D), bf(E, D, F)
    for form, N in (("prompt", P), ("decode", B)):
        h = bf(N, D)
        ids = torch.stack([torch.randperm(E, generator=gen, device=dev)[:top] for _ in range(N)]).int().contiguous()
        wts, shared, gate = torch.rand(N, top, generator=gen, device=dev), bf(N, D), f32(N, 1)
        touched = len(set(ids.flatten().tolist()))
        for name, lim, alpha, shift, extra in (("experts", float("inf"), 1.0, 0.0, (shared, gate)), ("experts_sufopel", 7.0, 1.702, 1.0, (None, None))):
            if form == "prompt":
                T = ops.moe_tc5_tiles(N, top, E)
                out = torch.empty(N, D, device=dev, dtype=torch.bfloat16)
                rows, act2 = torch.empty(128 * T, D, device=dev, dtype=torch.bfloat16), torch.empty(128 * T, F, device=dev, dtype=torch.bfloat16)
                y2, places = torch.empty(128 * T, D, device=dev), torch.empty(N * top + T, dtype=torch.int32, device=dev)
                wgu2 = torch.cat([wg, wu], 1).contiguous()
                us = timed(lambda: ops.moe_tc5(h, ids, wts, wgu2, wd, out, rows, act2, y2, places, lim, alpha, shift, *extra))
                res[f"{name}_prompt"] = mat(us, 2 * N * top * 3 * F * D)
                need = max(2 * N * top * 3 * F * D / (pk["bf16_tflops"] * 1e6), touched * 3 * F * D * 2 / (pk["hbm_gbs"] * 1e3))
                res[f"{name}_prompt"].update(frac_of_roofline=need / us)
                del wgu2, rows, act2, y2
            else:
                y, out = torch.empty(N, top, D, device=dev), torch.empty(N, D, device=dev, dtype=torch.bfloat16)
                us = timed(lambda: (ops.moe_experts(h, ids, wg, wu, wd, y, lim, alpha, None, shift), ops.moe_combine(y, wts, out, *extra)))
                res[f"{name}_decode"] = mem(us, touched * 3 * F * D * 2)
                res[f"{name}_decode"]["experts_touched"] = touched
        z_ = f32(N, E + 1)
        idc, wtc = torch.empty(N, top, dtype=torch.int32, device=dev), torch.empty(N, top, device=dev)
        us = timed(lambda: ops.moe_select(z_, None, idc, wtc, z["groups"], z["keep"], experts=E, softmax=True, worth="max", scale=2.5))
        res[f"choice_softmax_{form}"] = {"us": us}
        corr = f32(E)
        us = timed(lambda: ops.moe_select(z_, corr, idc, wtc, z["groups"], z["keep"], experts=E))
        res[f"choice_sufopel_{form}"] = {"us": us}
    # ---- the stream: add + Dynamic Tanh; add + depth average + next norm; two normed outputs halved; Sufopel's post norm
    L = 4
    for form, N in (("prompt", P), ("decode", B)):
        x, delta, delta2, w, b = f32(N, D), bf(N, D), bf(N, D), f32(D), f32(D)
        nrm = torch.empty(N, D, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.dyt(x, delta, 0.5, w, b, nrm))
        res[f"add_dyt_{form}"] = mem(us, N * D * (4 + 4 + 2 + 2))
        hist, coef = torch.zeros(L + 1, N, D, device=dev), f32(L + 1)
        us = timed(lambda: ops.depth_average(x, delta, hist, coef, L - 1, normed=nrm, next_norm=(0.5, w, b)))
        res[f"depth_average_{form}"] = mem(us, N * D * (4 + 2 + 4 + 4 * L + 4 + 2))       # the last layer's: L earlier results read
        us = timed(lambda: ops.rms_pair_mean(delta, delta2, w, b, nrm, 1e-6))
        res[f"pair_mean_{form}"] = mem(us, N * D * 3 * 2)
        us = timed(lambda: ops.post_norm_add(x, delta, w, 1e-6, w, 1e-6, nrm))
        res[f"post_norm_add_sufopel_{form}"] = mem(us, N * D * (4 + 4 + 2 + 2))
    return res


class _PlanContext:
    """the part of a step's context that the attention plan and kernels read, for timing them outside a model"""

    def __init__(self, ops, dev, q_len, pos0, page, pages, err):
        import numpy as np
        import torch
        from mashbox_b200.parts import StepInputs, Workspace
        S, N = len(q_len), sum(q_len)
        self.ops, self.device, self.dtype, self.err, self.options, self.memo = ops, dev, torch.bfloat16, err, {}, {}
        self.N, self.S, self.q_len, self.pos0 = N, S, list(q_len), list(pos0)
        self.q_start = [int(v) for v in np.concatenate([[0], np.cumsum(q_len)[:-1]])]
        self.rows = list(range(S))
        self.ws = Workspace(dev, N)
        self.inputs = StepInputs(dev)
        self.inputs.add("positions", np.concatenate([p + np.arange(n) for p, n in zip(pos0, q_len)]))
        self.inputs.add("tok_row", np.repeat(np.arange(S), q_len))
        for name, v in (("q_start", self.q_start), ("q_len", q_len), ("pos0", pos0), ("seq_row", self.rows)):
            self.inputs.add(name, v)

        class _Cache:
            page_size, pool_pages = page, pages
        self.cache = _Cache()

    def dev(self, name):
        return self.inputs.get(name)


def design_kernels(a, z, P, B, ctx, pk):
    """The kernels of the Luzosun decoder that the Llama decoder has a like kernel for, each pair on the same sizes:
    CUDA-event time of single launches after an L2 flush, and the fraction of the measured peak (copy bandwidth for
    the memory-bound ones, bf16 tensor throughput for prompt attention) that the algorithmic bytes or FLOPs come to."""
    import torch
    from mashbox_b200 import ops
    from mashbox_b200.parts.diff_attention import plan_diff_attention
    dev = "cuda:0"
    D, H, KV, dim, page = z["width"], z["heads"], z["kv_heads"], z["dim"], 16
    HD, vd, G, F = 2 * dim, 2 * dim, H // KV, z["ff"]
    gen = torch.Generator(device=dev).manual_seed(0)
    bf = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    err = ops.new_error_word(dev)

    def timed(f):
        for _ in range(3):
            f()
        ts = []
        for _ in range(max(5, a.steps // 4)):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    mem = lambda us, nbytes: {"us": us, "gbs": nbytes / us / 1e3, "frac_of_copy_peak": nbytes / us / 1e3 / pk["hbm_gbs"]}
    res = {}
    for form, N, S, klen in (("prompt", P, 1, P), ("decode", B, B, ctx)):
        pages = S * -(-klen // page)
        table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(S, -1)
        kz, vz = bf(pages, KV, page, 2 * dim), bf(pages, KV, page, vd)
        kl, vl = bf(pages, KV, page, HD), bf(pages, KV, page, HD)
        q, o = bf(N, H * HD), torch.empty(N, H * HD, device=dev, dtype=torch.bfloat16)
        q_len = [N // S] * S
        pos0 = [klen - n for n in q_len]
        q_start = [i * (N // S) for i in range(S)]
        seqs = (i32(q_start), i32(q_len), i32(pos0))
        rows = i32(list(range(S)))
        target = int((json.loads(a.options) if a.options else {}).get("attention_target_blocks", 296))
        plan = {k: i32(v or [0]) for k, v in plan_diff_attention(q_len, pos0, G, KV, z["block"], ops.attention_diff_mma_rows(),
                                                                 target=target).items()}
        tail = (*seqs, rows, table, kz, vz, H, KV, dim, vd, page, pages, z["block"], dim ** -0.5, 0.4, 0.7, 1e-6, err)
        if form == "prompt":
            us = timed(lambda: ops.attention_diff_mma(q, o, plan["pre"], plan["pre"].numel() // 2, *tail))
            if ops.attention_tc5_diff_supports(dim, vd, page):      # what the mixer runs at these sizes
                res["attention_prompt_luzosun_mma_sync"] = {"us": us}
                quads = i32(plan_diff_attention(q_len, pos0, G, KV, z["block"], ops.attention_tc5_diff_rows(), quads=True)["pre"])
                us = timed(lambda: ops.attention_tc5_diff(q, o, quads, quads.numel() // 4, *tail))
        else:
            n_slots = plan["slots"].numel() // 2
            n_part = max(1, n_slots * KV * ops.DIFF_MAX_SPLITS * 2 * ops.DIFF_DECODE_ROWS)
            po, pm = torch.empty(n_part, vd, device=dev), torch.empty(n_part, 2, device=dev)
            us = timed(lambda: ops.attention_diff_mma_decode(q, o, plan["dec"], plan["dec"].numel() // 4, plan["slots"],
                                                             n_slots, po, pm, *tail))
        if form == "prompt":
            pairs = P * (P + 1) // 2
            fz, fl = H * pairs * (2 * 2 * dim * 2 + 2 * 2 * vd), H * pairs * 4 * HD       # two maps: scores of 2 dim, values twice
            res["attention_prompt_luzosun"] = {"us": us, "tflops": fz / us / 1e6, "frac_of_bf16_peak": fz / us / 1e6 / pk["bf16_tflops"]}
            rws = ops.attention_tc5_rows() if ops.attention_tc5_supports(HD, page) else 64
            it = i32([v for m in range(-(-P * G // rws) - 1, -1, -1) for v in (0, m, 0, 1)])
            if ops.attention_tc5_supports(HD, page):
                ul = timed(lambda: ops.attention_tc5(q, H * HD, o, kl, vl, it, it.numel() // 4, *seqs, rows, table, H, KV, HD,
                                                     page, pages, None, HD ** -0.5, err))
            else:
                ul = timed(lambda: ops.attention_tma(q, H * HD, o, kl, vl, it, it.numel() // 4, False, *seqs, i32([-1]), rows,
                                                     table, None, None, 1, H, KV, HD, page, pages, None, HD ** -0.5, err))
            res["attention_prompt_llama"] = {"us": ul, "tflops": fl / ul / 1e6, "frac_of_bf16_peak": fl / ul / 1e6 / pk["bf16_tflops"]}
        else:
            nbytes = B * ctx * KV * (2 * dim + vd) * 2
            res["attention_decode_luzosun"] = mem(us, nbytes)
            ns = max(1, min(32, -(-296 // (B * KV)), ctx // 128))
            ns = 1 << (ns.bit_length() - 1)
            it = i32([v for s in range(B) for sp in range(ns) for v in (s, 0, sp, ns)])
            po, pm = torch.empty(B * H * ns, HD, device=dev), torch.empty(B * H * ns, 2, device=dev)
            ul = timed(lambda: ops.attention_tma(q, H * HD, o, kl, vl, it, B * ns, True, *seqs, rows, rows, table, po, pm, ns,
                                                 H, KV, HD, page, pages, None, HD ** -0.5, err, merge=ns > 1))
            res["attention_decode_llama"] = mem(ul, B * ctx * KV * 2 * HD * 2)
        # what follows the q/k/v product: bias, short convolutions, rotation, cache write / bias, rotation, cache write
        C = (H + 2 * KV) * HD
        qkv, qo = bf(N, C), torch.empty(N, H * HD, device=dev, dtype=torch.bfloat16)
        bias, wc = torch.randn(C, device=dev), torch.randn(4, C, device=dev)
        state = torch.zeros(S + 1, 3 * C, device=dev)
        fr = torch.rand(dim // 4, device=dev)
        positions = i32([p + t for p, n in zip(pos0, q_len) for t in range(n)])
        tok_row = i32([s for s, n in enumerate(q_len) for _ in range(n)])
        seq4 = (tok_row, i32(q_start), i32(q_len), rows)
        us = timed(lambda: ops.conv_rope_kv_write(qkv, bias, wc, state, seq4, positions, tok_row, table, qo, kz, vz, fr,
                                                  2 * H, 2 * KV, KV, dim, vd, 2, dim // 2, page, pages, err))
        fl2 = torch.rand(HD // 2, device=dev)
        ul = timed(lambda: ops.rope_kv_write(qkv, bias, positions, tok_row, table, kl, vl, fl2, H, KV, HD, HD, 1, page,
                                             pages, err))
        res[f"after_qkv_{form}_luzosun"] = mem(us, N * C * 2 * 2)
        res[f"after_qkv_{form}_llama"] = mem(ul, N * C * 2 * 2)
        # the norms: one kernel makes both of a Luzosun layer (x, two deltas, two outputs) / one norm (x, delta, output)
        x = torch.randn(N, D, device=dev)
        d1, d2, o1, o2 = bf(N, D), bf(N, D), bf(N, D), bf(N, D)
        w1 = torch.ones(D, device=dev)
        us = timed(lambda: ops.add_rmsnorm_pair(x, d1, d2, w1, w1, 1e-6, o1, o2))
        ul = timed(lambda: ops.add_rmsnorm(x, d1, None, w1, 1e-6, o1))
        res[f"norms_{form}_luzosun"] = mem(us, N * D * (4 + 4 + 4 * 2))
        res[f"norm_{form}_llama"] = mem(ul, N * D * (4 + 4 + 2 * 2))
        st2 = torch.zeros(S + 1, 3 * D, device=dev)
        wd = torch.randn(4, D, device=dev)
        us = timed(lambda: ops.short_conv(d1, wd, st2, seq4, o1, True))
        res[f"input_conv_{form}_luzosun"] = mem(us, N * D * 2 * 2)
        # the activation between the feed-forward's products
        up, act = bf(N, F * 3 // 2), torch.empty(N, F * 3 // 2, device=dev, dtype=torch.bfloat16)
        gu, ga = bf(N, 2 * F), torch.empty(N, F, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.xielu(up, act, 0.8, 1.2))
        ul = timed(lambda: ops.swiglu(gu, ga))
        res[f"activation_{form}_luzosun"] = mem(us, N * (F * 3 // 2) * 2 * 2)
        res[f"activation_{form}_llama"] = mem(ul, N * F * 3 * 2)
        del kz, vz, kl, vl
    ops.check_error_word(err)
    return res


def run_reference(a):
    """The reference arm: mashbox's own engine from baseline/_ref.  mashbox 0.1.15 installs there with --no-deps, but
    its model and engine modules import JAX (not in this image, no network) and it runs on TPU chips."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        import mashbox.runtime.engine  # noqa: F401
        import mashbox.gguf.archs.dense  # noqa: F401
    except Exception as e:
        print(json.dumps({"impl": "reference", "unavailable": f"mashbox's engine cannot be imported here: "
                          f"{type(e).__name__}: {e} (it is a JAX/TPU program; JAX is not installed and there is no network)"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "mashbox imports, but its engine targets TPU chips through JAX "
                      "and has no CUDA path for this metric"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all of them)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel directly (for profilers)")
    ap.add_argument("--options", default="", help="JSON of engine options (kernel choices), for experiments")
    ap.add_argument("--kernels", action="store_true", help="time single kernels against the library instead of the model")
    ap.add_argument("--attention", action="store_true", help="time the attention kernels alone (--heads --kv-heads --head-dim "
                    "--queries --keys --batch)")
    ap.add_argument("--timeline", action="store_true", help="start and end of every kernel of one layer of a decode step "
                    "inside its graph (--batch --context --layers)")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--queries", type=int, default=2048)
    ap.add_argument("--keys", type=int, default=8192)
    ap.add_argument("--workload", default="", choices=("",) + tuple(WORKLOADS),
                    help="run one of the other workloads of the baseline through Engine.admit/step instead")
    ap.add_argument("--requests", type=int, default=0, help="workloads: fewer requests than the workload names")
    ap.add_argument("--pool-tokens", type=int, default=0, help="workloads: size of the cache pool (0: every request fits)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--design", default="", choices=("", "luzosun", "sufopel", "tosevik", "fipitar"),
                    help="another design beside the Llama decoder of equal size (tosevik and fipitar: beside the Sufopel decoder): "
                    "prefill, decode, single kernels")
    ap.add_argument("--size", default="8b", choices=tuple(DESIGN_SIZES), help="--design: the layer sizes")
    ap.add_argument("--workload-warm", type=int, default=1, help="workloads: run the workload once untimed first")
    a = ap.parse_args()
    if a.impl == "reference":
        return run_reference(a)
    if a.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this engine runs on ONE GPU; --gpus {a.gpus} is not measured")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.workload:
        return run_workload(a)
    if a.design:
        return run_design(a)
    if a.attention:
        return run_attention(a)
    if a.timeline:
        return run_timeline(a)
    return run_kernels(a) if a.kernels else run_ours(a)


if __name__ == "__main__":
    sys.exit(main())
