#!/usr/bin/env python3
"""Measures the engine on one B200: Qwen3-8B layer sizes, bf16, random weights, synthetic token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 with 2,048 tokens of context per request,
timed on the device over K replays of the decode step; ``e2e`` is the same through ``Engine.step`` (host token ids
in through pinned memory, sampled token ids out, every step). ``prefill`` is one 2,048-token prompt in one step;
``points`` holds decode at batch 1 and 64, at longer contexts and for 32 requests of very different lengths, a longer prefill
and the two serving workloads; ``roofline`` divides the bytes a decode step has to read (every weight
once, plus the cache of the live requests) by its time. A step's inputs (15 GB of weights) are far larger than L2,
so nothing is cached between timed iterations.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 4096, "intermediate_size": 12288,
    "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "vocab_size": 151936, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 2560, "intermediate_size": 9728,
    "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "vocab_size": 151936, "tie_word_embeddings": True, "max_position_embeddings": 4096,
}
QWEN3_32B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 5120, "intermediate_size": 25600,
    "num_hidden_layers": 64, "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "vocab_size": 151936, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}
CONTEXT = 2048
PREFILL_TOKENS = 2048
LONG_CONTEXTS = (8192, 32768)      # further decode points at batch 8
LONG_PREFILL_TOKENS = 8192         # a further prefill point
UNEVEN_CONTEXTS = [256 + round(i * (8192 - 256) / 31) for i in range(32)]   # a decode point with requests of very different lengths
METRIC = "Qwen3-8B bf16 decode tok/s at batch 8 (context 2048)"


def peaks() -> tuple[float, float, str]:
    """(HBM GB/s, bf16 TFLOP/s, 'measured' | 'fallback')"""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            p = json.loads(path.read_text())
            return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
        except (KeyError, ValueError):
            pass
    return 6650.0, 1590.0, "fallback"


def sustained_tflops() -> float | None:
    """The measured bf16 throughput of a seconds-long loop under the power cap, if the peaks file has it: the figure
    for a product timed inside a long step."""
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["bf16_tflops_sustained"])
    except (OSError, KeyError, ValueError, TypeError):
        return None


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait(timeout=10)
        self.thread.join(timeout=5)
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def reference_arm(args) -> int:
    """The unmodified reference's language path at the same config (see baseline/reference_arm.py); nothing of this
    repository's package is imported on this path."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as arm
    return arm.run(args, QWEN3_8B, args.context, PREFILL_TOKENS, METRIC.replace(str(CONTEXT), str(args.context)), peaks, ClockSampler)


def serving_workload(which: str) -> int:
    """The two serving workloads beside the headline: many requests through ``Engine.generate`` (wall clock, host in the
    loop). ``continuous``: Qwen3-4B sizes (tied head), 256 requests, prompts of 64..2048 and outputs of 32..512 tokens,
    greedy. ``chunked``: Qwen3-32B sizes, 32 requests of 4,096 prompt tokens cut into 2,048-token portions mixed with
    decoding, 256 output tokens each."""
    import random

    import torch

    from oxr_inference_b200 import ops
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.sampling import SamplingParams

    rng = random.Random(0)
    if which == "continuous":
        cfg, kv_gb, max_running, budget = QWEN3_4B, 40.0, 256, 8192
        work = [(rng.randint(64, 2048), rng.randint(32, 512)) for _ in range(256)]
    else:
        cfg, kv_gb, max_running, budget = QWEN3_32B, 40.0, 32, 2048 + 32
        work = [(4096, 256)] * 32
    V = cfg["vocab_size"]
    engine = Engine(random_config=cfg, seed=0, settings=EngineSettings(
        dtype="bfloat16", page_size=16, kv_cache_gb=kv_gb, max_running=max_running, max_step_tokens=budget, prefill_chunk=2048,
        max_positions=cfg["max_position_embeddings"], cuda_graphs=True, profile=True))
    prompts = [[rng.randrange(V) for _ in range(p)] for p, _ in work]
    params = [SamplingParams(max_tokens=o, ignore_eos=True) for _, o in work]
    engine.generate(prompts[:2], [SamplingParams(max_tokens=4, ignore_eos=True)] * 2)   # warm-up: libraries, first graphs
    before = dict(engine.counters)
    launches = ops.launch_count
    engine.profile.steps.clear()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    done = engine.generate(prompts, params)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    # the engine's own per-step log: device milliseconds between two CUDA events around each step
    steps = [(st["ms"], st["tokens"], st["graph"], st["held"]) for st in engine.profile.steps]
    out_tokens = sum(len(c.token_ids) for c in done)
    in_tokens = sum(len(p) for p in prompts)
    assert all(len(c.token_ids) == o for c, (_, o) in zip(done, work))

    def percentiles(values, marks=(50, 90, 99)):
        v = sorted(values)
        return {f"p{q}": round(v[min(len(v) - 1, len(v) * q // 100)], 3) for q in marks} if v else {}

    h, layers, inter = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["intermediate_size"]
    heads, kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    layer_params = h * (heads + 2 * kv) * d + heads * d * h + 3 * h * inter
    weight_bytes = 2 * (layers * layer_params + V * h)           # every matrix a decode step reads, the head included
    kv_bytes_per_token = 2 * 2 * layers * kv * d
    hbm_gbs, bf16_tflops, source = peaks()
    decode = [(ms, n, held) for ms, n, graph, held in steps if graph]
    mixed = [(ms, n) for ms, n, graph, held in steps if not graph]
    decode_fracs = [(weight_bytes + kv_bytes_per_token * held) / (ms * 1e-3) / 1e9 / hbm_gbs for ms, n, held in decode]
    mixed_flops = [2 * n * (layers * layer_params) / (ms * 1e-3) / 1e12 / bf16_tflops for ms, n in mixed if n >= 1024]
    print(json.dumps({
        "workload": which, "model": "Qwen3-4B shape (tied)" if which == "continuous" else "Qwen3-32B shape", "requests": len(work),
        "prompt_tokens": in_tokens, "output_tokens": out_tokens, "seconds": round(seconds, 3),
        "output_tok_s": round(out_tokens / seconds, 1), "total_tok_s": round((in_tokens + out_tokens) / seconds, 1),
        "steps": engine.counters["steps"] - before["steps"], "graph_steps": engine.counters["graph_steps"] - before["graph_steps"],
        "decode_step_ms": percentiles([ms for ms, _, _ in decode]), "mixed_step_ms": percentiles([ms for ms, _ in mixed]),
        "decode_step_hbm_frac": percentiles(decode_fracs, (10, 50, 90)), "mixed_step_gemm_frac": percentiles(mixed_flops, (10, 50, 90)),
        "slowest_steps_ms": [round(ms, 1) for ms, *_ in sorted(steps, reverse=True)[:4]],
        "weight_gb_per_decode_step": round(weight_bytes / 1e9, 2), "peaks": source,
        "stages": engine.profile.summary(),
        "preemptions": engine.preemptions, "gpu_launches": ops.launch_count - launches, "dtype": "bf16",
        "data": "synthetic uniform token ids, random weights N(0, 0.02)"}))
    return 0


def radapel_config(width: int, ff: int, heads: int, kv_heads: int, head_dim: int, layers: int, vocab: int) -> dict:
    """A Radapel model of a real model's layer sizes: its three mixers in turn (Mamba-2, chunked attention with a distance bias twice,
    latent attention), each with a dense feed-forward, at the width, feed-forward size and head sizes of the Qwen3 model beside it."""
    ff_part = {"kind": "dense", "ff": ff, "limit": 7.0}
    attention = {"type": "attention", "mlp": ff_part, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "mask": {"size": 1024},
        "bias_max": 512, "bias_rows": 32}}
    latent = {"type": "latent_attention", "mlp": ff_part, "mixer": {
        "heads": heads, "dim": head_dim, "rot_dim": 64, "rot": {"dims": 64, "base": 10000.0}, "vdim": head_dim, "kv_rank": 192,
        "scale": (head_dim + 64) ** -0.5}}
    mamba = {"type": "mamba2", "mlp": ff_part, "mixer": {
        "heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}}
    turn = [mamba, attention, attention, latent]
    return {"architecture": "Radapel", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "vocab": vocab, "width": width,
            "layers": [turn[i % 4] for i in range(layers)]}


def _flush_l2(buf) -> None:
    buf.add_(1)   # 512 MB written: more than L2 holds


def _time_ms(fn, reps: int = 9, warm: int = 3, flush=None) -> float:
    import torch

    for _ in range(warm):
        fn()
    times = []
    for _ in range(reps):
        if flush is not None:
            _flush_l2(flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def design_throughput(cfg: dict, vocab: int, K: int, W: int, batch: int, context: int, prefill_tokens: int) -> dict:
    """Prefill (one prompt in one step, device time) and decode (``batch`` requests at ``context`` tokens, K replays of the decode
    step's CUDA graph) of one model with random weights, through the engine."""
    import torch

    from oxr_inference_b200 import ops
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.engine.batch import StepEntry
    from oxr_inference_b200.sampling import SamplingParams

    page = 16
    pages = batch * ((context + 2 * (K + W) + 64) // page + 2) + prefill_tokens // page + 64
    engine = Engine(random_config=cfg, seed=0, settings=EngineSettings(
        dtype="bfloat16", page_size=page, num_pages=pages, max_running=batch, max_step_tokens=8192, prefill_chunk=2048,
        max_positions=context + 2 * (K + W) + 128, cuda_graphs=True))
    gen = torch.Generator().manual_seed(0)
    # ---- prefill
    ids = torch.randint(0, vocab, (prefill_tokens,), generator=gen).tolist()

    def prefill():
        rc = engine.runner.cache.open("prefill")
        assert engine.runner.cache.reserve(rc, prefill_tokens)
        engine.runner.step([StepEntry(rc, ids, [prefill_tokens - 1])])
        engine.runner.cache.close(rc)

    before = ops.launch_count
    prefill()
    prefill_launches = ops.launch_count - before
    prefill_ms = _time_ms(prefill, reps=5, warm=W)
    engine.runner.check()
    # ---- decode
    for _ in range(batch):
        engine.add_request(torch.randint(0, vocab, (context,), generator=gen).tolist(), SamplingParams(max_tokens=2 * (K + W) + 8, ignore_eos=True))
    while engine.scheduler.waiting or any(r.pending > 1 for r in engine.scheduler.running):
        engine.step()
    plan = engine.scheduler.schedule()
    assert plan.decode_only and len(plan.entries) == batch
    entries = [StepEntry(p.request.cache, p.request.tokens[p.start:p.start + 1], [0], counter=len(p.request.output)) for p in plan.entries]
    tokens, _ = engine.graphs.run(entries)
    key = engine.graphs.last_key
    graph = engine.graphs._graphs[key][0]
    for _ in range(W):
        graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(K):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / K
    engine.runner.check()
    return {"prefill_tok_s": round(prefill_tokens / (prefill_ms * 1e-3), 1), "prefill_ms": round(prefill_ms, 3), "prefill_launches": prefill_launches,
            "decode_tok_s": round(batch * 1000.0 / ms, 1), "decode_ms_per_step": round(ms, 4), "decode_launches_per_step": engine.graphs.kernels_per_replay[key]}


def radapel_kernels(width: int, heads: int, kv_heads: int, head_dim: int, ff: int) -> list[dict]:
    """Each kernel of the new mixers alone, at one model size, beside the like kernel of the Qwen3 path: device time (median, L2 flushed
    between calls), the bytes or FLOPs it has to move or do, and the fraction of the measured peak."""
    import torch

    from oxr_inference_b200 import ops

    dev = "cuda"
    hbm_gbs, bf16_tflops, _ = peaks()
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    status = ops.new_status(dev)
    bf = torch.bfloat16
    rows = []

    def put(name, like, ms, *, bytes_=None, flops=None):
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            row.update(gb_s=round(bytes_ / (ms * 1e-3) / 1e9, 1), frac=round(bytes_ / (ms * 1e-3) / 1e9 / hbm_gbs, 4), bound="hbm")
        else:
            row.update(tflop_s=round(flops / (ms * 1e-3) / 1e12, 2), frac=round(flops / (ms * 1e-3) / 1e12 / bf16_tflops, 4), bound="tensor")
        rows.append(row)

    P, T, B, CTX = 16, 2048, 8, 2048
    H, KV, D = heads, kv_heads, head_dim
    g = torch.Generator(device=dev).manual_seed(0)

    def rand(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

    # ---- attention: a prompt of T tokens (prefill) and B single tokens over CTX keys (decode)
    n_pages = B * (CTX // P) + T // P + 8
    k_pool, v_pool = rand(n_pages, P, KV, D), rand(n_pages, P, KV, D)
    bias = rand(513, H, dtype=torch.float32)
    sink = rand(H, dtype=torch.float32)

    def tiles_for(specs, q_lens):
        out = {}
        for spec in specs:
            req = [r for r, x in enumerate(q_lens) if spec[1] <= x <= spec[2] for _ in range(0, x, spec[0])]
            tok0 = [t0 for r, x in enumerate(q_lens) if spec[1] <= x <= spec[2] for t0 in range(0, x, spec[0])]
            out[spec] = (torch.tensor(req + [0], dtype=torch.int32, device=dev), torch.tensor(tok0 + [0], dtype=torch.int32, device=dev), len(req))
        return out

    def attention_case(name, like, q_lens, ctx_lens, kv_heads_, k, v, *, tma, **extras):
        n = sum(q_lens)
        q = rand(n, H, k.shape[-1])
        width_ = max(ctx_lens) // P + 1
        table = torch.stack([torch.arange(r * (CTX // P), r * (CTX // P) + width_, dtype=torch.int32) % n_pages for r in range(len(q_lens))]).to(dev).contiguous()
        maps = ops.make_kv_maps(k.unsqueeze(0), v.unsqueeze(0), P) if tma else None
        specs = ops.attention_tile_specs(H, kv_heads_, k.shape[-1], bf, P if tma else None)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        args = dict(tiles=tiles_for(specs, q_lens), cu_q=cu, ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=dev), block_table=table,
                    page_size=P, scale=D ** -0.5, window=0, kv_len_bound=max(ctx_lens), status=status, kv_maps=maps, **extras)
        ms = _time_ms(lambda: ops.paged_attention(q, k, v, **args), flush=flush)
        chunk = extras.get("chunk", 0)
        if q_lens[0] > 1:
            seen = sum(min(p % chunk, p) + 1 if chunk else p + 1 for x, c in zip(q_lens, ctx_lens) for p in range(c - x, c))
            put(name, like, ms, flops=2 * 2 * H * k.shape[-1] * seen)
        else:
            seen = sum(min((c - 1) % chunk, c - 1) + 1 if chunk else c for c in ctx_lens)
            put(name, like, ms, bytes_=seen * kv_heads_ * (k.shape[-1] + (0 if v is k else v.shape[-1])) * 2)

    attention_case("paged_attention prefill (tcgen05, TMA)", None, [T], [T], KV, k_pool, v_pool, tma=True)
    attention_case("paged_attention prefill (cp.async mma)", None, [T], [T], KV, k_pool, v_pool, tma=False)
    attention_case("masked prefill: chunk 1024 + distance bias", "paged_attention prefill (cp.async mma)", [T], [T], KV, k_pool, v_pool, tma=False,
                   chunk=1024, dist_bias=bias)
    latent_pool = rand(n_pages, P, 1, 256)
    attention_case("latent prefill: 256-wide shared row + sink", "paged_attention prefill (cp.async mma)", [T], [T], 1, latent_pool, latent_pool,
                   tma=False, sink=sink)
    attention_case("paged_attention decode b8 (TMA split-KV)", None, [1] * B, [CTX] * B, KV, k_pool, v_pool, tma=True)
    attention_case("paged_attention decode b8 (cp.async split-KV)", None, [1] * B, [CTX] * B, KV, k_pool, v_pool, tma=False)
    attention_case("masked decode b8: chunk 1024 + distance bias", "paged_attention decode b8 (cp.async split-KV)", [1] * B, [CTX] * B, KV, k_pool,
                   v_pool, tma=False, chunk=1024, dist_bias=bias)
    attention_case("latent decode b8: 256-wide shared row + sink", "paged_attention decode b8 (cp.async split-KV)", [1] * B, [CTX] * B, 1, latent_pool,
                   latent_pool, tma=False, sink=sink)

    # ---- Mamba-2: heads of 64 values, 128 states, 8 groups
    MH, MP, MN, MG, taps = 2 * width // 64, 64, 128, 8, 4
    inner, channels = MH * MP, MH * MP + 2 * MG * MN
    state = torch.zeros(B + 1, MH * MP * MN + channels * (taps - 1), dtype=torch.float32, device=dev)
    vec = {k: rand(*shape, dtype=torch.float32, scale=0.1) for k, shape in
           (("conv", (channels, taps)), ("conv.b", (channels,)), ("dt_bias", (MH,)), ("A_log", (MH,)), ("D", (MH,)), ("norm", (inner,)))}
    for name, q_lens in (("prefill 2048", [T]), ("decode b8", [1] * B)):
        n = sum(q_lens)
        proj = rand(n, 2 * inner + 2 * MG * MN + MH, scale=0.5)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        req = torch.repeat_interleave(torch.arange(len(q_lens), dtype=torch.int32), torch.tensor(q_lens)).to(dev)
        slots = torch.arange(len(q_lens), dtype=torch.int32, device=dev)
        common = dict(cu_q=cu, state_slots=slots, n_requests=len(q_lens))
        ms = _time_ms(lambda: ops.mamba_conv(proj, inner, channels, vec["conv"], vec["conv.b"], state[:, MH * MP * MN:], req_of_token=req, **common), flush=flush)
        put(f"mamba_conv {name}", "qk_norm_rope_store", ms, bytes_=n * channels * 2 * 2 + len(q_lens) * channels * (taps - 1) * 8)
        xbc = ops.mamba_conv(proj, inner, channels, vec["conv"], vec["conv.b"], state[:, MH * MP * MN:], req_of_token=req, **common)
        ms = _time_ms(lambda: ops.mamba_scan(xbc, proj, inner + channels, heads=MH, vdim=MP, state=MN, groups=MG, dt_bias=vec["dt_bias"],
                                             a_log=vec["A_log"], d_skip=vec["D"], ssm=state, **common), flush=flush)
        put(f"mamba_scan {name}", "paged_attention (same step)", ms, bytes_=n * (channels * 2 + inner * 4) + len(q_lens) * MH * MP * MN * 8)
        y = torch.randn(n, inner, device=dev)
        ms = _time_ms(lambda: ops.gated_group_norm(y, proj, 0, vec["norm"], 8, 1e-6), flush=flush)
        put(f"gated_group_norm {name}", "add_rms_norm", ms, bytes_=n * inner * (4 + 2 + 2))

    # ---- the stream's norms and the feed-forward's activation, beside the Qwen3 path's
    for n in (T, B):
        x, res, w = rand(n, width), torch.randn(n, width, device=dev), torch.ones(width, device=dev)
        ms = _time_ms(lambda: ops.add_rms_norm(x, res, w, 1e-6), flush=flush)
        put(f"add_rms_norm {n} rows", None, ms, bytes_=n * width * (2 + 4 + 4 + 2))
        ms = _time_ms(lambda: ops.norm_add_norm(res, x, w, 1e-6, w, 1e-6), flush=flush)
        put(f"norm_add_norm {n} rows", f"add_rms_norm {n} rows", ms, bytes_=n * width * (2 + 4 + 4 + 2))
        gu = rand(n, 2 * ff)
        ms = _time_ms(lambda: ops.silu_mul(gu), flush=flush)
        put(f"silu_mul {n} rows", None, ms, bytes_=n * ff * 6)
        ms = _time_ms(lambda: ops.clamped_glu(gu, alpha=1.702, limit=7.0), flush=flush)
        put(f"clamped_glu {n} rows", f"silu_mul {n} rows", ms, bytes_=n * ff * 6)
    # ---- the latent mixer's per-head maps (queries into the latent space, latent output to values)
    for n in (T, B):
        q = rand(n, H, D + 64)
        q_abs = torch.empty(n, H, 256, dtype=bf, device=dev)
        uk = rand(H, D, 192, scale=0.05)
        ms = _time_ms(lambda: ops.head_linear(q_abs, 0, q, 0, uk), flush=flush)
        put(f"head_linear {n} rows", "linear (same FLOPs)", ms, flops=2 * n * H * D * 192)
    ops.check_status(status)
    return rows


def radapel_workload(args) -> int:
    """The new design beside the closest existing one at equal sizes: whole-model prefill and decode throughput at two sizes, and every
    kernel of the new mixers against its roofline beside the like kernel of the Qwen3 path."""
    import torch

    sizes = [("2048 wide, 8 layers", dict(width=2048, ff=8192, heads=16, kv_heads=4, head_dim=128, layers=8, vocab=32768)),
             ("4096 wide, 8 layers (Qwen3-8B layer sizes)", dict(width=4096, ff=12288, heads=32, kv_heads=8, head_dim=128, layers=8, vocab=32768))]
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler()
    sampler.start()
    out = {"workload": "radapel", "dtype": "bf16", "data": "synthetic uniform token ids, random weights N(0, 0.02)", "steps": K, "warmup": W,
           "batch": 8, "context": args.context, "prefill_tokens": PREFILL_TOKENS, "peaks": peaks()[2], "sizes": []}
    for name, s in sizes:
        qwen = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": s["width"], "intermediate_size": s["ff"],
                "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["head_dim"],
                "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "vocab_size": s["vocab"], "tie_word_embeddings": False,
                "max_position_embeddings": 8192}
        row = {"size": name}
        for design, cfg in (("qwen3", qwen), ("radapel", radapel_config(**s))):
            row[design] = design_throughput(cfg, s["vocab"], K, W, 8, args.context, PREFILL_TOKENS)
            torch.cuda.empty_cache()
        out["sizes"].append(row)
    last = sizes[-1][1]
    out["kernels"] = radapel_kernels(last["width"], last["heads"], last["kv_heads"], last["head_dim"], last["ff"])
    out["clocks"] = sampler.stop()
    print(json.dumps(out))
    return 0


def bifusun_config(width: int, ff: int, heads: int, kv_heads: int, head_dim: int, layers: int, vocab: int, experts: int = 16, top: int = 4) -> dict:
    """A Bifusun model of a real model's layer sizes: a matrix-memory layer, then three attention layers (biases, a filter of four taps, a
    query temperature, blended values), in turn; each with a feed-forward of ``experts`` experts of which a token runs ``top``, whose
    ``top`` experts together are as wide as the dense feed-forward of the Qwen3 model beside it."""
    moe = {"kind": "moe", "expert": {"ff": ff // top}, "router": {"experts": experts, "top": top, "scale": 2.0, "groups": {"count": 8, "keep": 4}}}
    attention = {"type": "attention", "mlp": moe, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "conv": 4,
        "q_temp": {"coef": 0.3, "every": 256}, "v_mix": True}}
    mlstm = {"type": "mlstm", "mlp": moe, "mixer": {"heads": 8, "dim": width // 16, "vdim": width // 8, "gate_cap": 15.0}}
    turn = [mlstm, attention, attention, attention]
    return {"architecture": "Bifusun", "embedding": {"scale": 1.0}, "logit_scale": 1.0, "norm": {"eps": 1e-6}, "vocab": vocab, "width": width,
            "layers": [turn[i % 4] for i in range(layers)]}


def bifusun_kernels(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, experts: int = 16, top: int = 4) -> list[dict]:
    """Each kernel of the design alone, at one model size, beside the like kernel of the paths that were there before: device time
    (median, L2 flushed between calls), the bytes or FLOPs it has to move or do, and the fraction of the measured peak."""
    import torch

    from oxr_inference_b200 import ops

    dev = "cuda"
    hbm_gbs, bf16_tflops, _ = peaks()
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    status = ops.new_status(dev)
    bf = torch.bfloat16
    rows = []

    def put(name, like, ms, *, bytes_=None, flops=None):
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            row.update(gb_s=round(bytes_ / (ms * 1e-3) / 1e9, 1), frac=round(bytes_ / (ms * 1e-3) / 1e9 / hbm_gbs, 4), bound="hbm")
        else:
            row.update(tflop_s=round(flops / (ms * 1e-3) / 1e12, 2), frac=round(flops / (ms * 1e-3) / 1e12 / bf16_tflops, 4), bound="tensor")
        rows.append(row)

    P, T, B, CTX = 16, 2048, 8, 2048
    H, KV, D = heads, kv_heads, head_dim
    g = torch.Generator(device=dev).manual_seed(0)

    def rand(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    n_pages = B * (CTX // P) + T // P + 8
    k_pool, v_pool = rand(n_pages, P, KV, D), rand(n_pages, P, KV, D)
    cq, ck, cv = H * D, KV * D, KV * D
    C = cq + ck + cv
    taps = 4
    conv, bias = rand(C, taps, dtype=torch.float32), rand(C, dtype=torch.float32)
    conv_t = conv.t().contiguous()
    cos = torch.ones(8192, D // 2, device=dev)
    ones = torch.ones(D, device=dev)
    tails = torch.zeros(B + 1, C * (taps - 1), device=dev)
    lam = torch.tensor([0.3], device=dev)
    for name, q_lens in (("prefill 2048", [T]), ("decode b8", [1] * B)):
        n = sum(q_lens)
        qkv = rand(n, C, scale=0.5)
        first = rand(n, cv)
        cu = i32([0] + list(torch.tensor(q_lens).cumsum(0)))
        req = torch.repeat_interleave(torch.arange(len(q_lens), dtype=torch.int32), torch.tensor(q_lens)).to(dev)
        pos = i32(list(range(T)) if len(q_lens) == 1 else [CTX - 1] * B)
        slots = i32([(r * (CTX // P)) * P + (i if len(q_lens) == 1 else CTX - 1) for r, x in enumerate(q_lens) for i in range(x)])
        ms = _time_ms(lambda: ops.qk_norm_rope_store(qkv, ones, ones, cos, cos, pos, slots, k_pool, v_pool, H, KV, D, 1e-6, status), flush=flush)
        put(f"qk_norm_rope_store {name}", None, ms, bytes_=n * C * 2 * 2)
        state_slots = i32(list(range(len(q_lens))))
        ms = _time_ms(lambda: ops.conv_qkv_store(qkv, cq, ck, cv, conv=conv, conv_t=conv_t, bias=bias, tails=tails, k_pool=k_pool, v_pool=v_pool, slots=slots,
                                                 req_of_token=req, cu_q=cu, state_slots=state_slots, positions=pos, n_requests=len(q_lens),
                                                 status=status, temp_coef=0.3, temp_every=256, blend=lam, first=first,
                                                 single_tokens=len(q_lens) > 1), flush=flush)
        put(f"conv_qkv_store {name} (bias, 4 taps, temperature, blend, cache write, tail roll)", f"qk_norm_rope_store {name}", ms,
            bytes_=n * (C * 2 * 2 + cv * 2) + len(q_lens) * C * (taps - 1) * 8)

    # ---- matrix memory: 8 heads, keys of width / 16, values of width / 8; beside the Mamba-2 scan of the same inner width
    MH, DK, DV = 8, width // 16, width // 8
    inner = MH * DV
    size = MH * DK * DV + MH * DK + MH
    state = torch.zeros(B + 1, size, device=dev)
    gate_bias = rand(2 * MH, dtype=torch.float32)
    norm_w = torch.ones(inner, device=dev)
    SH, SP, SN, SG = inner // 64, 64, 128, 8
    s_channels = inner + 2 * SG * SN
    ssm = torch.zeros(B + 1, SH * SP * SN, device=dev)
    vec = {k: rand(*shape, dtype=torch.float32, scale=0.1) for k, shape in (("dt_bias", (SH,)), ("A_log", (SH,)), ("D", (SH,)))}
    for name, q_lens in (("prefill 2048", [T]), ("decode b8", [1] * B)):
        n = sum(q_lens)
        proj = rand(n, 2 * MH * DK + 2 * inner, scale=0.5)
        gates = torch.randn(n, 2 * MH, device=dev)
        cu = i32([0] + list(torch.tensor(q_lens).cumsum(0)))
        common = dict(cu_q=cu, state_slots=i32(list(range(len(q_lens)))), n_requests=len(q_lens))
        xbc, sproj = rand(n, s_channels, scale=0.5), rand(n, 2 * inner + 2 * SG * SN + SH, scale=0.5)
        ms = _time_ms(lambda: ops.mamba_scan(xbc, sproj, inner + s_channels, heads=SH, vdim=SP, state=SN, groups=SG, dt_bias=vec["dt_bias"],
                                             a_log=vec["A_log"], d_skip=vec["D"], ssm=ssm, **common), flush=flush)
        put(f"mamba_scan {name}", None, ms, bytes_=n * (s_channels * 2 + inner * 4) + len(q_lens) * SH * SP * SN * 8)
        ms = _time_ms(lambda: ops.mlstm_scan(proj, 0, MH * DK, 2 * MH * DK, gates, gate_bias, heads=MH, key_dim=DK, value_dim=DV, cap=15.0,
                                             q_scale=DK ** -0.5, state=state, **common), flush=flush)
        put(f"mlstm_scan {name}", f"mamba_scan {name}", ms, bytes_=n * ((2 * MH * DK + inner) * 2 + inner * 4) + len(q_lens) * size * 8)
        y = torch.randn(n, inner, device=dev)
        ms = _time_ms(lambda: ops.gated_group_norm(y, proj, 0, norm_w, 8, 1e-6), flush=flush)
        put(f"gated_group_norm {name}", None, ms, bytes_=n * inner * (4 + 2 + 2))
        ms = _time_ms(lambda: ops.head_norm_gate(y, proj, 2 * MH * DK + inner, norm_w, MH, 1e-6), flush=flush)
        put(f"head_norm_gate {name}", f"gated_group_norm {name}", ms, bytes_=n * inner * (4 + 2 + 2))

    # ---- the feed-forward: router, activation, and the layer as a whole beside the dense gated one of equal active width
    E, ffe = experts, ff // top
    router_w, up_w, down_w = rand(E, width, scale=0.02), rand(E * ffe, width, scale=0.02), rand(width, E * ffe, scale=0.02)
    gate_up_w, dense_down_w = rand(2 * ff, width, scale=0.02), rand(width, ff, scale=0.02)
    from oxr_inference_b200.parts.base import Runtime
    from oxr_inference_b200.parts.experts import RoutedExperts

    part = RoutedExperts(Runtime(device=torch.device(dev), dtype=bf, max_positions=1, status=status), hidden_size=width, intermediate_size=ffe,
                         experts=E, top=top, groups=8, keep=4, scale=2.0)
    part.router, part.up, part.down = router_w, up_w, down_w
    part.finish_loading()
    for n in (T, B):
        h = rand(n, width)
        z = torch.randn(n, E, device=dev)
        ms = _time_ms(lambda: ops.route(z, top=top, groups=8, keep=4, scale=2.0), flush=flush)
        put(f"route {n} rows", None, ms, bytes_=n * (E * 8 + top * 8))
        gu = rand(n, 2 * ff)
        ms = _time_ms(lambda: ops.silu_mul(gu), flush=flush)
        put(f"silu_mul {n} rows", None, ms, bytes_=n * ff * 6)
        u = rand(n, E * ffe)
        gate = ops.route(z, top=top, groups=8, keep=4, scale=2.0)[0]
        ms = _time_ms(lambda: ops.gated_relu2(u, gate, ffe), flush=flush)
        put(f"gated_relu2 {n} rows (all {E} experts' columns)", f"silu_mul {n} rows", ms, bytes_=n * E * ffe * 4)
        ms = _time_ms(lambda: ops.linear(ops.silu_mul(ops.linear(h, gate_up_w)), dense_down_w), flush=flush)
        dense_flops, dense_bytes = 2 * n * width * 3 * ff, 3 * ff * width * 2
        moe_flops = 2 * n * width * 2 * ff     # the chosen experts only
        touched = E * (1 - (1 - top / E) ** n)
        moe_bytes = 2 * touched * ffe * width * 2
        if n >= 256:
            put(f"dense gated feed-forward {n} rows (three products of {ff})", None, ms, flops=dense_flops)
        else:
            put(f"dense gated feed-forward {n} rows (three products of {ff})", None, ms, bytes_=dense_bytes)
        ms = _time_ms(lambda: part.forward(h), flush=flush)
        if n >= 256:
            put(f"routed experts {n} rows ({top} of {E} experts of {ffe}; FLOPs of the chosen experts)", f"dense gated feed-forward {n} rows (three products of {ff})", ms,
                flops=moe_flops)
        else:
            put(f"routed experts {n} rows ({top} of {E} experts of {ffe}; bytes of the experts touched)", f"dense gated feed-forward {n} rows (three products of {ff})", ms,
                bytes_=moe_bytes)
    ops.check_status(status)
    return rows


def bifusun_workload(args) -> int:
    """The Bifusun design beside Qwen3 at equal sizes: whole-model prefill and decode throughput at two sizes, and every kernel of the new
    parts against its roofline beside the like kernel of the paths that were there before."""
    import torch

    sizes = [("2048 wide, 8 layers", dict(width=2048, ff=8192, heads=16, kv_heads=4, head_dim=128, layers=8, vocab=32768)),
             ("4096 wide, 8 layers (Qwen3-8B layer sizes)", dict(width=4096, ff=12288, heads=32, kv_heads=8, head_dim=128, layers=8, vocab=32768))]
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler()
    sampler.start()
    out = {"workload": "bifusun", "dtype": "bf16", "data": "synthetic uniform token ids, random weights N(0, 0.02)", "steps": K, "warmup": W,
           "batch": 8, "context": args.context, "prefill_tokens": PREFILL_TOKENS, "peaks": peaks()[2], "sizes": []}
    for name, s in sizes:
        qwen = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": s["width"], "intermediate_size": s["ff"],
                "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["head_dim"],
                "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "vocab_size": s["vocab"], "tie_word_embeddings": False,
                "max_position_embeddings": 8192}
        row = {"size": name}
        for design, cfg in (("qwen3", qwen), ("bifusun", bifusun_config(**s))):
            row[design] = design_throughput(cfg, s["vocab"], K, W, 8, args.context, PREFILL_TOKENS)
            torch.cuda.empty_cache()
        out["sizes"].append(row)
    last = sizes[-1][1]
    out["kernels"] = bifusun_kernels(last["width"], last["heads"], last["kv_heads"], last["head_dim"], last["ff"])
    out["clocks"] = sampler.stop()
    print(json.dumps(out))
    return 0


def vazepel_config(width: int, ff: int, heads: int, kv_heads: int, head_dim: int, layers: int, vocab: int, experts: int = 16, top: int = 4) -> dict:
    """A Vazepel model of a real model's layer sizes: parallel blocks whose attention (biases, rotated pairs, capped and mixed scores, a
    unit sink, an output gate) has the head sizes of the Qwen3 model beside it; the feed-forwards are, in turn, a two-matrix GELU layer with
    as many weights as the gated one beside it (half as wide again) and experts (``top`` of ``experts``, each an eighth of ``ff`` wide, with a
    shared expert of half of ``ff``: a token runs ``ff`` columns in all)."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "softcap": 30.0,
             "rot": {"dims": head_dim // 2, "base": 10000.0}}
    dense = {"kind": "dense", "ff": ff * 3 // 2}
    moe = {"kind": "moe", "expert": {"ff": ff // (2 * top), "limit": 7.0}, "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": ff // 2, "limit": 7.0}}
    return {"architecture": "Vazepel", "norm": {"eps": 1e-5}, "vocab": vocab, "width": width,
            "layers": [{"type": "attention", "mixer": mixer, "mlp": (dense, moe)[i % 2]} for i in range(layers)]}


def vazepel_kernels(width: int, heads: int, kv_heads: int, head_dim: int, ff: int) -> list[dict]:
    """Each kernel of the design alone, at one model size, beside the like kernel of the Qwen3 path: device time (median, L2 flushed
    between calls), the bytes or FLOPs it has to move or do, and the fraction of the measured peak."""
    import torch

    from oxr_inference_b200 import ops

    dev = "cuda"
    hbm_gbs, bf16_tflops, _ = peaks()
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    status = ops.new_status(dev)
    bf = torch.bfloat16
    rows = []

    def put(name, like, ms, *, bytes_=None, flops=None):
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            row.update(gb_s=round(bytes_ / (ms * 1e-3) / 1e9, 1), frac=round(bytes_ / (ms * 1e-3) / 1e9 / hbm_gbs, 4), bound="hbm")
        else:
            row.update(tflop_s=round(flops / (ms * 1e-3) / 1e12, 2), frac=round(flops / (ms * 1e-3) / 1e12 / bf16_tflops, 4), bound="tensor")
        rows.append(row)

    P, T, B, CTX = 16, 2048, 8, 2048
    H, KV, D = heads, kv_heads, head_dim
    g = torch.Generator(device=dev).manual_seed(0)

    def rand(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    n_pages = B * (CTX // P) + T // P + 8
    k_pool, v_pool = rand(n_pages, P, KV, D), rand(n_pages, P, KV, D)
    cq, ck, cv = H * D, KV * D, KV * D
    C = cq + ck + cv + cq      # q | k | v | output gate
    mix = (torch.eye(H, device=dev) + 0.1 * torch.randn(H, H, generator=g, device=dev)).contiguous()
    bias = rand(cq + ck + cv, dtype=torch.float32)
    ones = torch.ones(D, device=dev)
    cos_table = torch.ones(8192, D // 2, device=dev)
    tile = ops.attention_mix_tile(H, KV, D, D, bf)
    maps = ops.make_kv_maps(k_pool.unsqueeze(0), v_pool.unsqueeze(0), P)
    for name, q_lens, ctx_lens in (("prefill 2048", [T], [T]), ("decode b8", [1] * B, [CTX] * B)):
        n, prefill = sum(q_lens), q_lens[0] > 1
        proj = rand(n, C, scale=0.5)
        cu = i32([0] + list(torch.tensor(q_lens).cumsum(0)))
        req = torch.repeat_interleave(torch.arange(len(q_lens), dtype=torch.int32), torch.tensor(q_lens)).to(dev)
        pos = i32(list(range(T)) if prefill else [CTX - 1] * B)
        slots = i32([(r * (CTX // P)) * P + (i if prefill else CTX - 1) for r, x in enumerate(q_lens) for i in range(x)])
        table = torch.stack([torch.arange(r * (CTX // P), r * (CTX // P) + CTX // P + 1, dtype=torch.int32) % n_pages for r in range(len(q_lens))]).to(dev).contiguous()
        # ---- between the product and attention
        qkv = proj[:, :cq + ck + cv].contiguous()
        ms = _time_ms(lambda: ops.qk_norm_rope_store(qkv, ones, ones, cos_table, cos_table, pos, slots, k_pool, v_pool, H, KV, D, 1e-6, status), flush=flush)
        put(f"qk_norm_rope_store {name}", None, ms, bytes_=n * (cq + ck + cv) * 2 * 2)
        cos = torch.ones(n, D // 4, device=dev)
        ms = _time_ms(lambda: ops.bias_rope_store(proj, cq, ck, cv, D, bias=bias, cos=cos, sin=cos, k_pool=k_pool, v_pool=v_pool, slots=slots, status=status), flush=flush)
        put(f"bias_rope_store {name} (biases, rotated pairs, cache write)", f"qk_norm_rope_store {name}", ms, bytes_=n * (cq + ck + cv) * 2 * 2)
        # ---- attention
        def tiles_for(spec):
            r_ = [r for r, x in enumerate(q_lens) if spec[1] <= x <= spec[2] for _ in range(0, x, spec[0])]
            t_ = [t0 for r, x in enumerate(q_lens) if spec[1] <= x <= spec[2] for t0 in range(0, x, spec[0])]
            return i32(r_ + [0]), i32(t_ + [0]), len(r_)
        q3 = rand(n, H, D)
        for tma in (True, False):
            specs = ops.attention_tile_specs(H, KV, D, bf, P if tma else None)
            args = dict(tiles={spec: tiles_for(spec) for spec in specs}, cu_q=cu, ctx_lens=i32(ctx_lens), block_table=table, page_size=P, scale=D ** -0.5,
                        window=0, kv_len_bound=max(ctx_lens), status=status, kv_maps=maps if tma else None)
            ms = _time_ms(lambda: ops.paged_attention(q3, k_pool, v_pool, **args), flush=flush)
            kind = ("tcgen05, TMA" if prefill else "TMA split-KV") if tma else ("cp.async mma" if prefill else "cp.async split-KV")
            if prefill:
                put(f"paged_attention {name} ({kind})", None, ms, flops=2 * 2 * H * D * T * (T + 1) // 2)
            else:
                put(f"paged_attention {name} ({kind})", None, ms, bytes_=sum(ctx_lens) * KV * 2 * D * 2)
        like = f"paged_attention {name} ({'cp.async mma' if prefill else 'cp.async split-KV'})"
        common = dict(positions=pos, block_table=table, scale=D ** -0.5, softcap=30.0, head_mix=mix, unit_sink=True, gate=proj[:, cq + ck + cv:], status=status)
        ms = _time_ms(lambda: ops.attention_mix_tiled(proj, H, k_pool, v_pool, tile=tile, tiles=tiles_for((tile[0], 1, 1 << 30)), cu_q=cu,
                                                      kv_len_bound=max(ctx_lens), single_tokens=not prefill, **common), flush=flush)
        pairs = T * (T + 1) // 2 if prefill else sum(ctx_lens)
        if prefill:
            # q k and p v on the tensor cores, and the H x H mix of every (query, key) place on the fp32 pipes
            put(f"attention_mix_tiled {name} (cap, {H} x {H} mix, sink, gate; mma.sync)", like, ms, flops=pairs * (2 * 2 * H * D + 2 * H * H))
        else:
            put(f"attention_mix_tiled {name} (cap, {H} x {H} mix, sink, gate; split keys)", like, ms, bytes_=pairs * KV * 2 * D * 2)
        if not prefill:
            ms = _time_ms(lambda: ops.attention_mix_rows(proj, H, k_pool, v_pool, req_of_token=req, **common), flush=flush)
            put(f"attention_mix_rows {name} (the 32-bit kernel, on bfloat16 rows)", like, ms, bytes_=pairs * KV * 2 * D * 2)
        # ---- the stream: norm, and the gated add with the depth average
        stream, w, b = torch.randn(n, width, device=dev), torch.ones(width, device=dev), torch.zeros(width, device=dev)
        x = rand(n, width)
        ms = _time_ms(lambda: ops.add_rms_norm(x, stream, w, 1e-6), flush=flush)
        put(f"add_rms_norm {name}", None, ms, bytes_=n * width * (2 + 4 + 4 + 2))
        ms = _time_ms(lambda: ops.stream_layer_norm(stream, w, b, 1e-5, bf), flush=flush)
        put(f"stream_layer_norm {name}", f"add_rms_norm {name}", ms, bytes_=n * width * (4 + 2))
        depth = 5
        history = torch.randn(depth + 1, n, width, device=dev)
        a, f_, gates = rand(n, width), rand(n, width), rand(n, 2 * width)
        gb, ab, dw = torch.zeros(2 * width, device=dev), torch.zeros(width, device=dev), torch.full((depth + 1,), 0.2, device=dev)
        ms = _time_ms(lambda: ops.gated_residual(stream, a, f_, gates=gates, gate_bias=gb, a_bias=ab, history=history, index=depth, weights=dw), flush=flush)
        put(f"gated_residual {name} (two gates, both adds, history of {depth + 1}, weighted sum)", f"add_rms_norm {name}", ms,
            bytes_=n * width * (4 + 2 + 2 + 4 + 4 + depth * 4 + 4))
        ms = _time_ms(lambda: ops.gated_residual(stream, a, f_, gates=gates, gate_bias=gb, a_bias=ab, history=history, index=depth, weights=dw,
                                                 norm=(w, b, 1e-5), out_dtype=bf), flush=flush)
        put(f"gated_residual + layer norm {name} (one kernel: what runs between two blocks)", f"add_rms_norm {name}", ms,
            bytes_=n * width * (4 + 2 + 2 + 4 + 4 + depth * 4 + 4 + 2))
        # ---- feed-forward activations
        gu = rand(n, 2 * ff)
        ms = _time_ms(lambda: ops.silu_mul(gu), flush=flush)
        put(f"silu_mul {name}", None, ms, bytes_=n * ff * 6)
        up = rand(n, ff * 3 // 2)
        ms = _time_ms(lambda: ops.gelu_tanh_(up), flush=flush)
        put(f"gelu_tanh {name} (in place)", f"silu_mul {name}", ms, bytes_=n * (ff * 3 // 2) * 4)
        ms = _time_ms(lambda: ops.clamped_glu(gu, alpha=1.702, limit=7.0), flush=flush)
        put(f"clamped_glu {name} (the shared expert)", f"silu_mul {name}", ms, bytes_=n * ff * 6)
        E, top = 16, 4
        z = torch.randn(n, E, device=dev)
        ms = _time_ms(lambda: ops.route(z, top=top, groups=8, keep=4, scale=2.0), flush=flush)
        put(f"route {name} (sigmoid, best two of a group)", None, ms, bytes_=n * (E * 8 + top * 8))
        ms = _time_ms(lambda: ops.route(z, top=top, groups=4, keep=2, scale=1.0, score="softmax", group_score="max", renormalize=False), flush=flush)
        put(f"route {name} (softmax, best of a group, scores as weights)", f"route {name} (sigmoid, best two of a group)", ms, bytes_=n * (E * 8 + top * 8))
    # ---- the feed-forwards as a whole, beside the dense gated one
    from oxr_inference_b200.parts.base import FEED_FORWARDS, Runtime

    rt = Runtime(device=torch.device(dev), dtype=bf, max_positions=1, status=status)
    E, top, ffe = 16, 4, ff // 8
    gate_up_w, dense_down_w = rand(2 * ff, width, scale=0.02), rand(width, ff, scale=0.02)
    gelu = FEED_FORWARDS.build("gelu_mlp", rt, hidden_size=width, intermediate_size=ff * 3 // 2)
    gelu.assign("up", rand(ff * 3 // 2, width, scale=0.02)); gelu.assign("down", rand(width, ff * 3 // 2, scale=0.02))
    unit = {"hidden_size": width, "intermediate_size": ff // 2, "limit": 7.0, "alpha": 1.702}
    moe = FEED_FORWARDS.build("routed_experts", rt, hidden_size=width, intermediate_size=ffe, experts=E, top=top, groups=4, keep=2, activation="clamped_glu",
                              limit=7.0, score="softmax", group_score="max", renormalize=False, shared={"kind": "clamped_glu", "params": unit})
    for name, info in moe.parameters().items():
        moe.assign(name, rand(*info.shape, scale=0.02))
    for part in (gelu, moe):
        part.finish_loading()
    for n in (T, B):
        h = rand(n, width)
        dense_name = f"dense gated feed-forward {n} rows (three products of {ff})"
        ms = _time_ms(lambda: ops.linear(ops.silu_mul(ops.linear(h, gate_up_w)), dense_down_w), flush=flush)
        weights_dense = 3 * ff * width * 2
        put(dense_name, None, ms, **({"flops": 2 * n * width * 3 * ff} if n >= 256 else {"bytes_": weights_dense}))
        ms = _time_ms(lambda: gelu.forward(h), flush=flush)
        put(f"GELU feed-forward {n} rows (two products of {ff * 3 // 2})", dense_name, ms,
            **({"flops": 2 * n * width * 3 * ff} if n >= 256 else {"bytes_": weights_dense}))
        ms = _time_ms(lambda: moe.forward(h), flush=flush)
        touched = E * (1 - (1 - top / E) ** n)
        put(f"routed clamped experts {n} rows ({top} of {E} of {ffe}, shared {ff // 2})", dense_name, ms,
            **({"flops": 2 * n * width * 3 * ff} if n >= 256 else {"bytes_": 3 * width * 2 * (touched * ffe + ff // 2)}))
    ops.check_status(status)
    return rows


def vazepel_workload(args) -> int:
    """The Vazepel design beside Qwen3 at equal sizes: whole-model prefill and decode throughput at two sizes, and every kernel of the new
    parts against its roofline beside the like kernel of the Qwen3 path."""
    import torch

    sizes = [("2048 wide, 8 layers", dict(width=2048, ff=8192, heads=16, kv_heads=4, head_dim=128, layers=8, vocab=32768)),
             ("4096 wide, 8 layers (Qwen3-8B layer sizes)", dict(width=4096, ff=12288, heads=32, kv_heads=8, head_dim=128, layers=8, vocab=32768))]
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler()
    sampler.start()
    out = {"workload": "vazepel", "dtype": "bf16", "data": "synthetic uniform token ids, random weights N(0, 0.02)", "steps": K, "warmup": W,
           "batch": 8, "context": args.context, "prefill_tokens": PREFILL_TOKENS, "peaks": peaks()[2], "sizes": []}
    for name, s in sizes:
        qwen = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": s["width"], "intermediate_size": s["ff"],
                "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["head_dim"],
                "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "vocab_size": s["vocab"], "tie_word_embeddings": False,
                "max_position_embeddings": 8192}
        row = {"size": name}
        for design, cfg in (("qwen3", qwen), ("vazepel", vazepel_config(**s))):
            row[design] = design_throughput(cfg, s["vocab"], K, W, 8, args.context, PREFILL_TOKENS)
            torch.cuda.empty_cache()
        out["sizes"].append(row)
    last = sizes[-1][1]
    out["kernels"] = vazepel_kernels(last["width"], last["heads"], last["kv_heads"], last["head_dim"], last["ff"])
    out["clocks"] = sampler.stop()
    print(json.dumps(out))
    return 0


def nidudra_config(width: int, ff: int, heads: int, kv_heads: int, head_dim: int, layers: int, vocab: int, experts: int = 16, top: int = 4) -> dict:
    """A Nidudra model of a real model's layer sizes. Its layers take turns of four: windowed attention (the last 1,024 keys beside the first 64;
    q/k norm, a gate per channel); causal attention with half of each head rotated (rescaled in bands), unit-norm q and k, a sink and a gate per
    head; the pair (causal attention behind a filter of 4 taps with rescaled rotation, beside gated linear attention with ``width / 256`` heads
    of 128 keys and 256 values); windowed attention again that reads the first layer's keys and values. All with the head sizes of the Qwen3
    model beside it. The feed-forwards alternate between the gated layer of that model and experts (``top`` of ``experts``, each an eighth of
    ``ff`` wide, with a shared expert of half of ``ff``: a token runs ``ff`` columns in all)."""
    sizes = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // (2 * top)}, "router": {"experts": experts, "top": top}, "shared": {"ff": ff // 2}}
    out = []
    for i in range(layers):
        first = i // 4 * 4
        windowed = {**sizes, "mask": {"size": 1024, "keep_first": 64}}
        sinked = {**sizes, "rot": {"dims": head_dim // 2, "base": 100000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 2048}}}
        pair = {"left": {**sizes, "conv": 4, "rot": {"dims": head_dim // 2, "base": 10000.0, "scaling": {"factor": 4.0, "original": 1024, "fast": 16.0, "slow": 2.0}}},
                "right": {"heads": max(width // 256, 1), "dim": 128, "vdim": 256, "tau": 8.0, "rank": 64}}
        kind, mixer = (("attention", windowed), ("attention_2", sinked), ("parallel", pair), ("attention", {**windowed, "kv_from": first}))[i % 4]
        out.append({"type": kind, "mixer": mixer, "mlp": (dense, moe)[i % 2]})
    return {"architecture": "Nidudra", "norm": {"eps": 1e-6}, "vocab": vocab, "width": width, "logit_softcap": 50.0, "layers": out}


def nidudra_kernels(width: int, heads: int, kv_heads: int, head_dim: int, ff: int) -> list[dict]:
    """Each kernel of the design alone, at one model size, beside the like kernel of the paths that were there before: device time (median, L2
    flushed between calls), the bytes or FLOPs it has to move or do, and the fraction of the measured peak."""
    import torch

    from oxr_inference_b200 import ops

    dev = "cuda"
    hbm_gbs, bf16_tflops, _ = peaks()
    flush = torch.zeros(128 << 20, dtype=torch.float32, device=dev)
    status = ops.new_status(dev)
    bf = torch.bfloat16
    rows = []

    def put(name, like, ms, *, bytes_=None, flops=None):
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1)}
        if bytes_ is not None:
            row.update(gb_s=round(bytes_ / (ms * 1e-3) / 1e9, 1), frac=round(bytes_ / (ms * 1e-3) / 1e9 / hbm_gbs, 4), bound="hbm")
        else:
            row.update(tflop_s=round(flops / (ms * 1e-3) / 1e12, 2), frac=round(flops / (ms * 1e-3) / 1e12 / bf16_tflops, 4), bound="tensor")
        rows.append(row)

    P, T, B, CTX = 16, 2048, 8, 2048
    H, KV, D = heads, kv_heads, head_dim
    WINDOW, KEEP, TAPS = 1024, 64, 4
    g = torch.Generator(device=dev).manual_seed(0)

    def rand(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    n_pages = B * (CTX // P) + T // P + 8
    k_pool, v_pool = rand(n_pages, P, KV, D), rand(n_pages, P, KV, D)
    cq, ck, cv = H * D, KV * D, KV * D
    ones = torch.ones(D, device=dev)
    cos_table = torch.ones(8192, D // 2, device=dev)
    maps = ops.make_kv_maps(k_pool.unsqueeze(0), v_pool.unsqueeze(0), P)
    GH, GK, GV = max(width // 256, 1), 128, 256       # the recurrence's heads, keys and values
    for name, q_lens, ctx_lens in (("prefill 2048", [T], [T]), ("decode b8", [1] * B, [CTX] * B)):
        n, prefill = sum(q_lens), q_lens[0] > 1
        R = len(q_lens)
        cu = i32([0] + list(torch.tensor(q_lens).cumsum(0)))
        req = torch.repeat_interleave(torch.arange(R, dtype=torch.int32), torch.tensor(q_lens)).to(dev)
        pos = i32(list(range(T)) if prefill else [CTX - 1] * B)
        slots = i32([(r * (CTX // P)) * P + (i if prefill else CTX - 1) for r, x in enumerate(q_lens) for i in range(x)])
        table = torch.stack([torch.arange(r * (CTX // P), r * (CTX // P) + CTX // P + 1, dtype=torch.int32) % n_pages for r in range(R)]).to(dev).contiguous()
        state_slots = i32(list(range(R)))
        # ---- between the product and attention
        qkv = rand(n, cq + ck + cv, scale=0.5)
        ms = _time_ms(lambda: ops.qk_norm_rope_store(qkv, ones, ones, cos_table, cos_table, pos, slots, k_pool, v_pool, H, KV, D, 1e-6, status), flush=flush)
        put(f"qk_norm_rope_store {name}", None, ms, bytes_=n * (cq + ck + cv) * 2 * 2)
        cos = torch.ones(n, D // 4, device=dev)
        common = dict(num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=D, k_pool=k_pool, v_pool=v_pool, slots=slots, req_of_token=req, cu_q=cu,
                      state_slots=state_slots, n_requests=R, status=status, eps=1e-5)
        ms = _time_ms(lambda: ops.head_prep(qkv, q_col0=0, k_col0=cq, v_col0=cq + ck, norm="weighted", q_weight=ones, k_weight=ones, **common), flush=flush)
        put(f"head_prep {name} (weighted q/k norm, cache write)", f"qk_norm_rope_store {name}", ms, bytes_=n * (cq + ck + cv) * 2 * 2)
        ms = _time_ms(lambda: ops.head_prep(qkv, q_col0=0, k_col0=cq, v_col0=cq + ck, norm="unit", norm_after_rotation=True, cos=cos, sin=cos, **common), flush=flush)
        put(f"head_prep {name} (half of each head rotated, unit norm, cache write)", f"qk_norm_rope_store {name}", ms, bytes_=n * (cq + ck + cv) * 2 * 2)
        qk = rand(n, cq + ck, scale=0.5)
        bias, taps = rand(cq + ck, dtype=torch.float32), rand(cq + ck, TAPS, dtype=torch.float32)
        taps_t = taps.t().contiguous()
        tails = torch.zeros(R, (cq + ck) * (TAPS - 1), device=dev)
        ms = _time_ms(lambda: ops.head_prep(qk, q_col0=0, k_col0=cq, v_col0=None, values_are_keys=True, bias=bias, taps=taps, taps_t=taps_t, tails=tails, norm="weighted",
                                            q_weight=ones, k_weight=ones, cos=cos, sin=cos, **common), flush=flush)
        put(f"head_prep {name} (biases, {TAPS} taps, values = keys, norm, rotation, cache write, tails)", f"qk_norm_rope_store {name}", ms,
            bytes_=n * ((cq + ck) * 2 + (cq + ck + cv) * 2))
        # ---- attention
        def tiles_for(spec):
            r_ = [r for r, x in enumerate(q_lens) if spec[1] <= x <= spec[2] for _ in range(0, x, spec[0])]
            t_ = [t0 for r, x in enumerate(q_lens) if spec[1] <= x <= spec[2] for t0 in range(0, x, spec[0])]
            return i32(r_ + [0]), i32(t_ + [0]), len(r_)
        q3 = rand(n, H, D)
        sink = torch.zeros(H, device=dev)
        seen_causal = T * (T + 1) // 2 if prefill else sum(ctx_lens)
        seen_window = sum(min(p_ + 1, WINDOW) + max(0, min(KEEP, p_ + 1 - WINDOW)) for p_ in (range(T) if prefill else [CTX - 1] * B))
        for tma in (True, False):
            specs = ops.attention_tile_specs(H, KV, D, bf, P if tma else None)
            args = dict(tiles={spec: tiles_for(spec) for spec in specs}, cu_q=cu, ctx_lens=i32(ctx_lens), block_table=table, page_size=P, scale=D ** -0.5,
                        kv_len_bound=max(ctx_lens), status=status)
            kind = ("tcgen05, TMA" if prefill else "TMA split-KV") if tma else ("cp.async mma" if prefill else "cp.async split-KV")
            ms = _time_ms(lambda: ops.paged_attention(q3, k_pool, v_pool, window=0, kv_maps=maps if tma else None, **args), flush=flush)
            if prefill:
                put(f"paged_attention {name} ({kind})", None, ms, flops=2 * 2 * H * D * seen_causal)
            else:
                put(f"paged_attention {name} ({kind})", None, ms, bytes_=seen_causal * KV * 2 * D * 2)
            if not tma:
                like = f"paged_attention {name} ({kind})"
                ms = _time_ms(lambda: ops.paged_attention(q3, k_pool, v_pool, window=0, sink=sink, **args), flush=flush)
                if prefill:
                    put(f"sink attention {name} (causal, a sink per head; {kind})", like, ms, flops=2 * 2 * H * D * seen_causal)
                else:
                    put(f"sink attention {name} (causal, a sink per head; {kind})", like, ms, bytes_=seen_causal * KV * 2 * D * 2)
                ms = _time_ms(lambda: ops.paged_attention(q3, k_pool, v_pool, window=WINDOW, keep_first=KEEP, **args), flush=flush)
                if prefill:
                    put(f"windowed attention {name} (last {WINDOW} keys beside the first {KEEP}; {kind})", like, ms, flops=2 * 2 * H * D * seen_window)
                else:
                    put(f"windowed attention {name} (last {WINDOW} keys beside the first {KEEP}; {kind})", like, ms, bytes_=seen_window * KV * 2 * D * 2)
        o = rand(n, H * D)
        gates = rand(n, H * D)
        gates_pair = rand(n, 2 * H * D)
        ms = _time_ms(lambda: ops.silu_mul(gates_pair), flush=flush)
        put(f"silu_mul {name} ({H * D} columns)", None, ms, bytes_=n * H * D * 6)
        ms = _time_ms(lambda: ops.sigmoid_gate_(o, gates, 0, D, per_head=False), flush=flush)
        put(f"sigmoid_gate {name} (a gate per channel, in place)", f"silu_mul {name} ({H * D} columns)", ms, bytes_=n * H * D * 6)
        # ---- the recurrences
        inner, keys = GH * GV, GH * GK
        gproj = rand(n, 2 * keys + 2 * inner, scale=0.3)
        z, zb = torch.randn(n, keys, device=dev), torch.full((keys,), 3.0, device=dev)
        gstate = torch.zeros(R + 1, GH * GK * GV, device=dev)
        mgates, mbias = torch.randn(n, 2 * GH, device=dev), torch.zeros(2 * GH, device=dev)
        mstate = torch.zeros(R + 1, GH * GK * GV + GH * GK + GH, device=dev)
        ms = _time_ms(lambda: ops.mlstm_scan(gproj, 0, keys, 2 * keys, mgates, mbias, heads=GH, key_dim=GK, value_dim=GV, cap=15.0, q_scale=GK ** -0.5,
                                             state=mstate, cu_q=cu, state_slots=state_slots, n_requests=R), flush=flush)
        moved = n * (2 * keys + inner) * 2 + n * inner * 4 + R * GH * GK * GV * 4 * 2
        put(f"mlstm_scan {name} ({GH} heads of {GK} x {GV})", None, ms, bytes_=moved)
        ms = _time_ms(lambda: ops.gla_scan(gproj, 0, keys, 2 * keys, z, zb, heads=GH, key_dim=GK, value_dim=GV, tau=16.0, q_scale=GK ** -0.5, state=gstate,
                                           cu_q=cu, state_slots=state_slots, n_requests=R), flush=flush)
        put(f"gla_scan {name} ({GH} heads of {GK} x {GV}, a decay per key channel)", f"mlstm_scan {name} ({GH} heads of {GK} x {GV})", ms, bytes_=moved + n * keys * 4)
        y, wn = torch.randn(n, inner, device=dev), torch.ones(inner, device=dev)
        ms = _time_ms(lambda: ops.head_norm_gate(y, gproj, 2 * keys + inner, wn, GH, 1e-5), flush=flush)
        put(f"head_norm_gate {name} (sigmoid gate)", None, ms, bytes_=n * inner * (4 + 2 + 2))
        ms = _time_ms(lambda: ops.head_norm_gate(y, gproj, 2 * keys + inner, wn, GH, 1e-5, silu=True), flush=flush)
        put(f"head_norm_gate {name} (SiLU gate)", f"head_norm_gate {name} (sigmoid gate)", ms, bytes_=n * inner * (4 + 2 + 2))
        # ---- the stream
        stream, w = torch.randn(n, width, device=dev), torch.ones(width, device=dev)
        x, x2 = rand(n, width), rand(n, width)
        ms = _time_ms(lambda: ops.add_rms_norm(x, stream, w, 1e-6), flush=flush)
        put(f"add_rms_norm {name}", None, ms, bytes_=n * width * (2 + 4 + 4 + 2))
        ms = _time_ms(lambda: ops.norm_add_norm(stream, x, w, 1e-5, rounded=True), flush=flush)
        put(f"norm_add_norm {name} (norm of the output, add, rounded stream)", f"add_rms_norm {name}", ms, bytes_=n * width * (2 + 4 + 4 + 2))
        ms = _time_ms(lambda: ops.pair_norm_mean(x, x2, w, w, 1e-5), flush=flush)
        put(f"pair_norm_mean {name}", f"add_rms_norm {name}", ms, bytes_=n * width * (2 + 2 + 2))
        # ---- experts' activation over all experts' columns
        E, top, ffe = 16, 4, ff // 8
        u = rand(n, E * ffe)
        gate = torch.rand(n, E, device=dev)
        ms = _time_ms(lambda: ops.gated_relu2(u, gate, ffe), flush=flush)
        put(f"gated_relu2 {name} (all {E} experts' columns)", None, ms, bytes_=n * E * ffe * 4)
        gu = rand(n, E * 2 * ffe)
        ms = _time_ms(lambda: ops.expert_silu_glu(gu, gate, ffe, on_input=True), flush=flush)
        put(f"expert_silu_glu {name} (all {E} experts' gate and up columns, weight on the input)", f"gated_relu2 {name} (all {E} experts' columns)", ms,
            bytes_=n * E * ffe * 6)
    # ---- the feed-forwards as a whole, beside the dense gated one
    from oxr_inference_b200.parts.base import FEED_FORWARDS, Runtime

    rt = Runtime(device=torch.device(dev), dtype=bf, max_positions=1, status=status)
    E, top, ffe = 16, 4, ff // 8
    gate_up_w, dense_down_w = rand(2 * ff, width, scale=0.02), rand(width, ff, scale=0.02)
    moe = FEED_FORWARDS.build("routed_experts", rt, hidden_size=width, intermediate_size=ffe, experts=E, top=top, activation="silu_glu", score="sigmoid",
                              renormalize=False, weight_on="input", shared={"kind": "swiglu", "params": {"hidden_size": width, "intermediate_size": ff // 2}},
                              shared_gate=True)
    for name, info in moe.parameters().items():
        moe.assign(name, rand(*info.shape, scale=0.02))
    moe.finish_loading()
    for n in (T, B):
        h = rand(n, width)
        dense_name = f"dense gated feed-forward {n} rows (three products of {ff})"
        ms = _time_ms(lambda: ops.linear(ops.silu_mul(ops.linear(h, gate_up_w)), dense_down_w), flush=flush)
        weights_dense = 3 * ff * width * 2
        put(dense_name, None, ms, **({"flops": 2 * n * width * 3 * ff} if n >= 256 else {"bytes_": weights_dense}))
        ms = _time_ms(lambda: moe.forward(h), flush=flush)
        touched = E * (1 - (1 - top / E) ** n)
        put(f"routed SiLU experts {n} rows ({top} of {E} of {ffe}, gated shared {ff // 2})", dense_name, ms,
            **({"flops": 2 * n * width * 3 * ff} if n >= 256 else {"bytes_": 3 * width * 2 * (touched * ffe + ff // 2)}))
    ops.check_status(status)
    return rows


def nidudra_workload(args) -> int:
    """The Nidudra design beside Qwen3 at equal sizes: whole-model prefill and decode throughput at two sizes, and every kernel of the new
    parts against its roofline beside the like kernel of the paths that were there before."""
    import torch

    sizes = [("2048 wide, 8 layers", dict(width=2048, ff=8192, heads=16, kv_heads=4, head_dim=128, layers=8, vocab=32768)),
             ("4096 wide, 8 layers (Qwen3-8B layer sizes)", dict(width=4096, ff=12288, heads=32, kv_heads=8, head_dim=128, layers=8, vocab=32768))]
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler()
    sampler.start()
    out = {"workload": "nidudra", "dtype": "bf16", "data": "synthetic uniform token ids, random weights N(0, 0.02)", "steps": K, "warmup": W,
           "batch": 8, "context": args.context, "prefill_tokens": PREFILL_TOKENS, "peaks": peaks()[2], "sizes": []}
    for name, s in sizes:
        qwen = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": s["width"], "intermediate_size": s["ff"],
                "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["head_dim"],
                "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "vocab_size": s["vocab"], "tie_word_embeddings": False,
                "max_position_embeddings": 8192}
        row = {"size": name}
        for design, cfg in (("qwen3", qwen), ("nidudra", nidudra_config(**s))):
            row[design] = design_throughput(cfg, s["vocab"], K, W, 8, args.context, PREFILL_TOKENS)
            torch.cuda.empty_cache()
        out["sizes"].append(row)
    last = sizes[-1][1]
    out["kernels"] = nidudra_kernels(last["width"], last["heads"], last["kv_heads"], last["head_dim"], last["ff"])
    out["clocks"] = sampler.stop()
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"], help="fewer layers than the model has (named in config)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64 and the further points (quick runs)")
    ap.add_argument("--skip-serving", action="store_true", help="leave the two serving workloads out of `points`")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each request holds when the decode steps are timed")
    ap.add_argument("--workload", default="decode", choices=("decode", "continuous", "chunked", "radapel", "bifusun", "vazepel", "nidudra"),
                    help="decode: the headline line (default); continuous / chunked: the two serving workloads, one line each; "
                         "radapel / bifusun / vazepel / nidudra: that design beside Qwen3 at equal sizes, whole models and kernel by kernel")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload == "radapel":
        return radapel_workload(args)
    if args.workload == "bifusun":
        return bifusun_workload(args)
    if args.workload == "vazepel":
        return vazepel_workload(args)
    if args.workload == "nidudra":
        return nidudra_workload(args)
    if args.workload != "decode":
        return serving_workload(args.workload)
    K, W = args.steps, max(args.warmup, 3)

    import torch

    from oxr_inference_b200 import ops
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.engine.batch import StepEntry
    from oxr_inference_b200.sampling import SamplingParams

    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    page = 16
    context = args.context
    kv_per_token = 2 * 2 * args.layers * cfg["num_key_value_heads"] * cfg["head_dim"]
    # batch 1 and 64 ride along where 64 requests of this context fit beside the weights (they do at 2,048 tokens)
    batches = (8,) if args.skip_points or 64 * context * kv_per_token > 100e9 else (8, 1, 64)
    # further points: batch 8 at longer contexts, and a longer prompt
    long_contexts = () if args.skip_points else LONG_CONTEXTS
    long_prefill = 0 if args.skip_points else LONG_PREFILL_TOKENS
    spare = 2 * (K + W) + 64
    pages = max([max(batches) * ((context + spare) // page + 2)] + [8 * ((c + spare) // page + 2) for c in long_contexts] +
                ([sum((c + spare) // page + 2 for c in UNEVEN_CONTEXTS)] if long_contexts else [])) + 64
    engine = Engine(random_config=cfg, seed=0, settings=EngineSettings(
        dtype="bfloat16", page_size=page, num_pages=pages, max_running=64, max_step_tokens=8192, prefill_chunk=2048,
        max_positions=max([4096, context + spare + 64, long_prefill + 64] + [c + spare + 64 for c in long_contexts]), cuda_graphs=True))
    model = engine.runner.model
    gen = torch.Generator().manual_seed(0)
    hbm_gbs, bf16_tflops, peak_kind = peaks()

    L, h, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, KV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    layer_params = (H + 2 * KV) * D * h + H * D * h + 2 * I * h + I * h
    weight_bytes = 2 * (L * layer_params + V * h) + 4 * (L * (2 * h + 2 * D) + h)
    kv_bytes_per_token = 2 * L * KV * D * 2

    def fill(batch: int, budget: int, tokens) -> None:
        """`batch` requests, each with `tokens` tokens (one number, or one for each) in the cache and one token left to decode."""
        for r in list(engine.scheduler.running) + list(engine.scheduler.waiting):
            r.cancelled = True
        engine.step()
        for i in range(batch):
            p = torch.randint(0, V, (tokens if isinstance(tokens, int) else tokens[i],), generator=gen).tolist()
            engine.add_request(p, SamplingParams(max_tokens=budget, ignore_eos=True))
        while engine.scheduler.waiting or any(r.pending > 1 for r in engine.scheduler.running):
            engine.step()
        assert len(engine.scheduler.running) == batch

    def decode_device(batch: int, tokens=context) -> tuple[float, int, int]:
        """ms per decode step on the device (K replays after W), kernels per step, context length (of the first request)."""
        fill(batch, 2 * (K + W) + 8, tokens)
        plan = engine.scheduler.schedule()
        assert plan.decode_only and len(plan.entries) == batch
        entries = [StepEntry(p.request.cache, p.request.tokens[p.start:p.start + 1], [0], counter=len(p.request.output))
                   for p in plan.entries]
        tokens, _ = engine.graphs.run(entries)  # captures at first use, fills the static inputs
        key = engine.graphs.last_key
        graph = engine.graphs._graphs[key][0]
        for _ in range(W):
            graph.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(K):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / K
        ctx = plan.entries[0].start + 1
        engine.scheduler.commit(plan, {p.request.id: t for p, t in zip(plan.entries, tokens.tolist())})
        return ms, engine.graphs.kernels_per_replay[key], ctx

    sampler = ClockSampler()
    sampler.start()

    # ---- headline: batch 8, device-timed
    ms8, kernels_per_step, ctx8 = decode_device(8)
    value = 8 * 1000.0 / ms8
    step_bytes = weight_bytes + 8 * ctx8 * kv_bytes_per_token + 8 * h * 2
    achieved = step_bytes / (ms8 * 1e-3) / 1e9

    # ---- the same through the entry point: host tokens in, sampled tokens out, every step
    for _ in range(W):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e = 8 * K / e2e_s
    layout_words = next(v[1].total for k, v in engine.graphs._graphs.items() if k[0] == 8)

    points = {}
    for b in batches[1:]:
        ms, _, ctx = decode_device(b)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
        points[f"decode_b{b}_hbm_frac"] = round((weight_bytes + b * ctx * kv_bytes_per_token) / (ms * 1e-3) / 1e9 / hbm_gbs, 4)
    for c in long_contexts:
        ms, _, ctx = decode_device(8, c)
        points[f"decode_b8_ctx{c}"] = round(8 * 1000.0 / ms, 1)
        points[f"decode_b8_ctx{c}_hbm_frac"] = round((weight_bytes + 8 * ctx * kv_bytes_per_token) / (ms * 1e-3) / 1e9 / hbm_gbs, 4)

    if long_contexts:
        # requests of very different lengths, as a serving engine has them: 32 contexts evenly spaced from 256 to 8,192 tokens
        lens = UNEVEN_CONTEXTS
        ms, _, _ = decode_device(32, lens)
        points["decode_b32_ctx256_to_8192"] = round(32 * 1000.0 / ms, 1)
        points["decode_b32_ctx256_to_8192_hbm_frac"] = round((weight_bytes + (sum(lens) + 32) * kv_bytes_per_token) / (ms * 1e-3) / 1e9 / hbm_gbs, 4)

    # ---- prefill: one prompt in one step
    for r in list(engine.scheduler.running):
        r.cancelled = True
    engine.step()

    def prefill_ms_of(T: int) -> float:
        ids = torch.randint(0, V, (T,), generator=gen).tolist()
        times = []
        for i in range(W + 5):
            rc = engine.runner.cache.open("prefill")
            assert engine.runner.cache.reserve(rc, T)
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.step([StepEntry(rc, ids, [T - 1])])
            end.record()
            torch.cuda.synchronize()
            if i >= W:
                times.append(start.elapsed_time(end))
            engine.runner.cache.close(rc)
        engine.runner.check()
        return statistics.median(times)

    T = PREFILL_TOKENS
    prefill_ms = prefill_ms_of(T)
    # the fraction counts the matrix products alone (attention's flops are named beside it, not added to it)
    flops = 2 * T * L * layer_params + 2 * V * h
    attn_flops = L * 2 * H * D * T * (T + 1)
    prefill_frac = flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12)
    if long_prefill:
        ms = prefill_ms_of(long_prefill)
        points[f"prefill_{long_prefill}"] = round(long_prefill / (ms * 1e-3), 1)
        points[f"prefill_{long_prefill}_gemm_frac"] = round((2 * long_prefill * L * layer_params + 2 * V * h) / (ms * 1e-3) / (bf16_tflops * 1e12), 4)

    clocks = sampler.stop()
    launches_of_step = kernels_per_step * K
    if not (args.skip_points or args.skip_serving):
        # the two serving workloads, each in a process of its own once this one's model is gone
        del engine, model
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for which in ("continuous", "chunked"):
            try:
                res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", which], capture_output=True, text=True, timeout=900)
                line = json.loads(res.stdout.strip().splitlines()[-1])
                points[f"{which}_output_tok_s"] = line["output_tok_s"]
                points[f"{which}_decode_hbm_frac_p50"] = line["decode_step_hbm_frac"].get("p50")
                points[f"{which}_mixed_gemm_frac_p50"] = line["mixed_step_gemm_frac"].get("p50")
            except Exception as exc:   # a serving workload that fails does not take the headline with it
                points[f"{which}_error"] = f"{type(exc).__name__}: {exc}"[:200]
    out = {
        "metric": METRIC.replace(str(CONTEXT), str(context)), "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, random weights N(0, 0.02)", "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": L, "layers_of_model": QWEN3_8B["num_hidden_layers"], "hidden": h,
                   "heads": H, "kv_heads": KV, "head_dim": D, "intermediate": I, "vocab": V, "global_batch": 8,
                   "seq_len": context, "page_size": page, "tied": False, "parallelism": "single GPU",
                   "l2": "step inputs (15 GB of weights) exceed L2", "peaks": peak_kind},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": layout_words * 4, "d2h_bytes_per_step": (8 + 2) * 4},
        "gpu_launches": launches_of_step,
        "prefill": {"value": round(T / (prefill_ms * 1e-3), 1), "tokens": T, "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4),
                    "attention_tflops_in_step": round(attn_flops / 1e12, 3),
                    **({"frac_of_sustained": round(flops / (prefill_ms * 1e-3) / (sustained_tflops() * 1e12), 4)} if sustained_tflops() else {})},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s", "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
