"""Nidudra on the GPU against the plain statement in ``tests/plain/nidudra_plain.py``: each mechanism alone, the stream after every layer,
whole prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests, pages and slots that are used
again, marked keys far back, at page borders and just inside and outside a window and the kept first keys, long decoding, greedy
generation through the engine, and the new kernels against their formulas."""

import math

import pytest
import torch

import nidudra_util as NU
from plain import nidudra_plain as NP
from util import Replay

pytestmark = pytest.mark.gpu

DEV = "cuda"

CLOSE_CALL = 0.004
"""bfloat16 rows at which some router of the plain model decided by less than this (a difference of sigmoid scores) are not compared:
a score that differs by a rounding step may choose another expert there, for no fault. (32-bit compares every row.)"""


def close(got, want, dtype, what, margins=None, spreading=False):
    """32-bit: every row within 2e-4 of the row's spread. bfloat16: within 8e-2, one row in twenty (at least one) up to 0.25. ``spreading``: the
    model has routers below attention layers, so a choice that a bfloat16 rounding step turns over at one token reaches later tokens through
    their attention, and no row can be cleared by its own margins alone: then nine clear rows in ten within 8e-2 and the median within 4e-2
    (32-bit still compares every row)."""
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    d = (got - want) - (got - want).mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std(-1).clamp_min(1e-6)
    if dtype == "float32":
        assert err.max() <= 2e-4, f"{what}: row {int(err.argmax())} is off by {err.max():.2e} of the row's spread (limit 2e-04)"
        return
    if margins is not None:
        clear = margins >= CLOSE_CALL
        assert clear.float().mean() >= 0.4 or len(clear) < 12, f"{what}: most rows are close calls of a router; the test compares too little"
        err = torch.where(clear, err, torch.zeros_like(err))
    over = int((err > 8e-2).sum())
    if spreading:
        assert over <= max(1, len(err) // 10) and err.median() <= 4e-2, (
            f"{what}: {over} of {len(err)} rows are off by more than 8e-02 of the row's spread, the median by {err.median():.2e}")
        return
    assert err.max() <= 0.25 and over <= max(1, len(err) // 20), (
        f"{what}: {over} of {len(err)} rows are off by more than 8e-02 of the row's spread, row {int(err.argmax())} by {err.max():.2e}")


def runner_for(folder, dtype, *, page_size=8, num_pages=64, max_requests=4):
    from oxr_inference_b200.engine.runtime import ModelRunner

    return ModelRunner.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages, max_requests=max_requests)


def feed(runner, rc, ids, lo, hi, want=None):
    from oxr_inference_b200.engine.batch import StepEntry

    assert runner.cache.reserve(rc, hi)
    return StepEntry(rc, ids[lo:hi], list(range(hi - lo)) if want is None else want)


def run_cut(runner, ids, cuts):
    """One request alone, cut into portions; logits of every position."""
    rc = runner.cache.open("r")
    rows, at = [], 0
    for c in cuts:
        rows.append(runner.step([feed(runner, rc, ids, at, at + c)]))
        at += c
    assert at == len(ids)
    runner.check()
    runner.cache.close(rc)
    runner.cache.check()
    return torch.cat(rows)


# ------------------------------------------------------------------------------------------------ each mechanism alone
W, S, P, MOE, DENSE = NU.windowed, NU.sinked, NU.paired, NU.moe, NU.dense
SINGLE = {
    "windowed_alone": NU.model_config([W()]),
    "window_of_one": NU.model_config([W(size=1, keep_first=0)]),
    "window_of_one_and_kept_keys": NU.model_config([W(size=1, keep_first=5)]),
    "window_beyond_the_prompt": NU.model_config([W(size=500, keep_first=2)]),
    "kept_keys_beyond_a_page": NU.model_config([W(size=4, keep_first=11)]),
    "windowed_one_head": NU.model_config([W(heads=1, kv_heads=1, dim=32, vdim=16, size=6, keep_first=1)]),
    "windowed_tiled_sizes": NU.model_config([W(heads=6, kv_heads=2, dim=32, vdim=32, size=13, keep_first=9, scale=0.3)]),
    "borrowed_keys_under_another_mask": NU.model_config([W(size=20, keep_first=0), W(size=3, keep_first=7, kv_from=0), W(size=40, keep_first=1, kv_from=0)]),
    "borrowed_keys_tiled": NU.model_config([W(heads=4, kv_heads=4, dim=16, vdim=16, size=5, keep_first=2),
                                            W(heads=4, kv_heads=4, dim=16, vdim=16, size=11, keep_first=0, kv_from=0)]),
    "sink_alone": NU.model_config([S()]),
    "sink_no_rotation": NU.model_config([S(rot=0)]),
    "sink_all_entries_rotated_plain_frequencies": NU.model_config([S(rot=16, base=7.0, scaling=None)]),
    "sink_two_entries_rotated": NU.model_config([S(rot=2, base=3.0)]),
    "sink_every_band": NU.model_config([S(dim=32, vdim=32, rot=32, base=3000.0, scaling=NU.bands(factor=5.0, low=2.0, high=6.0, original=200), scale=0.4)]),
    "sink_many_heads_on_one": NU.model_config([S(heads=12, kv_heads=1, dim=16, vdim=8, rot=8)]),
    "sink_odd_sizes": NU.model_config([S(heads=3, kv_heads=1, dim=22, vdim=10, rot=6)], width=40),
    "pair_alone": NU.model_config([P()]),
    "pair_one_tap": NU.model_config([P(conv=1)]),
    "pair_six_taps": NU.model_config([P(conv=6, rot=16, scaling=None)]),
    "pair_no_rotation": NU.model_config([P(rot=0)]),
    "pair_slow_decay_wide_keys": NU.model_config([P(r_heads=2, r_dim=72, r_vdim=40, tau=32.0, rank=2)]),
    "pair_fast_decay_one_head": NU.model_config([P(r_heads=1, r_dim=8, r_vdim=8, tau=0.5, rank=8, heads=2, kv_heads=2, dim=32, scale=0.3)]),
    "dense_feed_forward": NU.model_config([W(mlp=DENSE())]),
    "no_logit_cap": NU.model_config([S(mlp=DENSE(ff=24))], softcap=0.0),
    "tight_logit_cap": NU.model_config([S(mlp=DENSE(ff=24))], softcap=1.5),
    "experts": NU.model_config([S(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE())]),
    "experts_no_shared": NU.model_config([S(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(shared=0))]),
    "experts_top_one": NU.model_config([S(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(experts=8, top=1))]),
    "experts_all_chosen": NU.model_config([S(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(experts=4, top=4, ff=20))]),
    "experts_odd_sizes": NU.model_config([S(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(experts=7, top=3, ff=9, shared=13))], width=40),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_mechanism(name, dtype, tmp_path):
    cfg = SINGLE[name]
    folder = NU.make_folder(tmp_path, cfg, name, seed=5)
    ids = NU.tokens(cfg, 61, seed=1)
    want = NU.plain_logits(folder, ids)
    r = runner_for(folder, dtype)
    mg = NU.router_margins(folder, ids)
    close(run_cut(r, ids, [61]), want, dtype, f"{name}, whole prompt", mg)
    close(run_cut(r, ids, [29] + [1] * 32), want, dtype, f"{name}, 29 tokens then one by one", mg)
    close(run_cut(r, ids, [2, 3, 2, 11, 2, 17, 1, 2, 21]), want, dtype, f"{name}, portions", mg)


@pytest.mark.parametrize("width,ff,experts,top", [(64, 16, 6, 2), (40, 20, 5, 1), (72, 36, 3, 2), (48, 9, 4, 3)])
def test_experts_grouped_by_expert_equal_the_two_products_form(width, ff, experts, top, tmp_path):
    """From ``grouped_min_rows`` tokens on every expert multiplies only the rows that chose it (their inputs scaled by the score first); below, all
    experts are two products. Both against the plain sum, in both dtypes, also for widths that are no multiples of 16."""
    cfg = NU.model_config([S(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(experts=experts, top=top, ff=ff, shared=24))], width=width)
    folder = NU.make_folder(tmp_path, cfg, "grouped", seed=8)
    ids = NU.tokens(cfg, 70, seed=3)
    want, mg = NU.plain_logits(folder, ids), NU.router_margins(folder, ids)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(folder, dtype)
        ff = r.model.blocks[0].feed_forward
        for rows in (0, 8):
            ff.grouped_min_rows = rows
            close(run_cut(r, ids, [40, 5, 25]), want, dtype, f"experts, grouped from {rows} rows on, {dtype}", mg)


def test_layer_results_one_by_one(tmp_path):
    """The stream after every layer against the plain statement's, in 32-bit."""
    from oxr_inference_b200.engine.batch import StepEntry

    for name, cfg in (("A", NU.MODEL_A), ("B", NU.MODEL_B)):
        folder = NU.make_folder(tmp_path, cfg, name, seed=2)
        ids = NU.tokens(cfg, 23, seed=6)
        plain_cfg, w = NP.read_model(folder, torch.float64)
        want: list = []
        NP.forward(plain_cfg, w, ids, streams=want)
        r = runner_for(folder, "float32")
        got = []
        blocks = r.model.blocks
        originals = [b.forward for b in blocks]
        for b, f in zip(blocks, originals):
            def wrapped(*a, _f=f, **k):
                out = _f(*a, **k)
                assert out[0] is None
                got.append(out[1].clone())
                return out
            b.forward = wrapped
        rc = r.cache.open("r")
        assert r.cache.reserve(rc, len(ids))
        r.step([StepEntry(rc, ids, [len(ids) - 1])])
        r.cache.close(rc)
        assert len(got) == len(want) == len(cfg["layers"])
        for i, (a, b) in enumerate(zip(got, want)):
            err = (a.double().cpu() - b).abs().max() / b.abs().max()
            assert err < 2e-5, f"model {name}, layer {i} ({cfg['layers'][i]['type']}): off by {err:.2e} of the stream's largest entry"


# ------------------------------------------------------------------------------------------------ whole models, every cutting
MODELS = {"A": NU.MODEL_A, "B": NU.MODEL_B, "C": NU.MODEL_C}
SPREADING = {"A": True, "B": True, "C": False}
"""Whether a model has routers below attention layers (see ``close``)."""


@pytest.fixture(scope="module", params=[(m, d) for m in sorted(MODELS) for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def model(request, tmp_path_factory):
    name, dtype = request.param
    # 32-bit runs take the weights at full strength and compare every row at 2e-4; 16-bit runs of these deep models take them milder
    folder = NU.make_folder(tmp_path_factory.mktemp(f"nidudra_{name}_{dtype}"), MODELS[name], name, seed=11, strength=1.0 if dtype == "float32" else 0.25)
    return name, dtype, folder, runner_for(folder, dtype, page_size=8, num_pages=40)


def test_whole_prompt_equals_token_by_token(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    for n in (1, 2, 9, 75):
        ids = NU.tokens(cfg, n, seed=2)
        want = NU.plain_logits(folder, ids)
        mg = NU.router_margins(folder, ids)
        close(run_cut(r, ids, [n]), want, dtype, f"{name}: whole prompt of {n}", mg, SPREADING[name])
        close(run_cut(r, ids, [1] * n), want, dtype, f"{name}: {n} tokens one by one", mg, SPREADING[name])


def test_portions_of_several_sizes(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = NU.tokens(cfg, 120, seed=3)
    want = NU.plain_logits(folder, ids)
    for cuts in ([2] * 60, [7, 2, 13, 3, 2, 31, 1, 16, 2, 17, 8, 18], [33, 33, 33, 21], [119, 1], [15, 16, 17, 32, 40]):
        close(run_cut(r, ids, cuts), want, dtype, f"{name}: portions {cuts[:4]}...", NU.router_margins(folder, ids), SPREADING[name])


def test_long_decoding(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = NU.tokens(cfg, 260, seed=4)
    close(run_cut(r, ids, [4] + [1] * 256), NU.plain_logits(folder, ids), dtype, f"{name}: 256 decoded tokens", NU.router_margins(folder, ids), SPREADING[name])


def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(model):
    """Four live requests at most, 40 pages of 8 tokens: the lengths below need far more over time, so pages and state slots come back and are
    handed out again (a slot's filter tails and recurrence matrices must start at zero); every request's logits equal those it gets alone."""
    name, dtype, folder, r = model
    cfg = MODELS[name]
    lengths = [97, 3, 64, 30, 1, 121, 45, 18, 70]
    todo = [(f"q{i}", NU.tokens(cfg, n, seed=20 + i)) for i, n in enumerate(lengths)]
    live, got, cuts = {}, {}, {}
    step = 0
    while todo or live:
        while todo and len(live) < 4:
            key, ids = todo.pop(0)
            rc = r.cache.open(key)
            assert rc is not None
            live[key] = [rc, ids, 0]
        entries, order = [], []
        for k, (key, (rc, ids, at)) in enumerate(sorted(live.items())):
            if (step + k) % 3 == 0 and at > 0 and len(live) > 1:
                continue                                   # a request may sit a step out
            left = len(ids) - at
            c = 1 if at >= len(ids) // 2 else min(left, [2, 5, 16, 3, 29][(step + k) % 5])   # portions first, then single tokens
            if r.cache.free_pages * 8 < c + 8:
                continue
            entries.append(feed(r, rc, ids, at, at + c))
            order.append((key, c))
        if not entries:   # everything sat out or lacked pages: let the longest go on alone
            key, (rc, ids, at) = max(live.items(), key=lambda kv: kv[1][2])
            entries, order = [feed(r, rc, ids, at, at + 1)], [(key, 1)]
        out = r.step(entries)
        row = 0
        for key, c in order:
            got.setdefault(key, []).append(out[row:row + c])
            cuts.setdefault(key, []).append(c)
            row += c
            live[key][2] += c
            if live[key][2] == len(live[key][1]):
                r.cache.close(live.pop(key)[0])
        step += 1
    r.check()
    r.cache.check()
    assert sum(-(-n // 8) for n in lengths) > 40, "the requests never needed a page twice"
    for i, n in enumerate(lengths):
        ids = NU.tokens(cfg, n, seed=20 + i)
        mixed = torch.cat(got[f"q{i}"])
        if dtype == "bfloat16" and SPREADING[name]:
            # what the mix must not change is told apart from what 16 bits do to a deep model with routers: the same request alone, cut alike
            alone = run_cut(r, ids, cuts[f"q{i}"]).float().cpu()
            d = (mixed.float().cpu() - alone) - (mixed.float().cpu() - alone).mean(-1, keepdim=True)
            err = d.pow(2).mean(-1).sqrt() / alone.std(-1).clamp_min(1e-6)
            assert int((err > 3e-2).sum()) <= n // 20, f"{name}: request {i} of {n} tokens differs in the mix from itself alone: row {int(err.argmax())} by {err.max():.2e}"
        else:
            close(mixed, NU.plain_logits(folder, ids), dtype, f"{name}: request {i} of {n} tokens in the mix", NU.router_margins(folder, ids))


def test_far_keys_and_a_long_lived_state(tmp_path):
    """A prompt of 700 tokens with peaked attention and slowly decaying state: the last logits rest on keys from hundreds of tokens back,
    across dozens of pages, and on what the recurrence has carried; in 32-bit a lost key shows."""
    cfg = NU.model_config([S(heads=4, kv_heads=2, dim=32, vdim=32, rot=32, base=1e4, scale=0.7, mlp=DENSE(ff=40)),
                           P(heads=2, kv_heads=1, dim=64, conv=4, rot=32, base=1e4, scale=0.2, r_heads=2, r_dim=32, r_vdim=32, tau=64.0, rank=4),
                           W(heads=4, kv_heads=2, dim=32, vdim=32, size=150, keep_first=40, scale=0.3, mlp=MOE(ff=16, experts=4, top=2, shared=16))],
                          width=64, vocab=180)
    folder = NU.make_folder(tmp_path, cfg, "far", seed=3, sharpen=4.0)
    ids = NU.tokens(cfg, 700, seed=9)
    want = NU.plain_logits(folder, ids)
    mg = NU.router_margins(folder, ids)
    r = runner_for(folder, "float32", page_size=16, num_pages=50)
    close(run_cut(r, ids, [650] + [1] * 50), want, "float32", "650 tokens, then 50 one by one")
    close(run_cut(r, ids, [255, 257, 2, 186]), want, "float32", "portions that end beside page borders")
    b = runner_for(folder, "bfloat16", page_size=16, num_pages=50)
    close(run_cut(b, ids, [650] + [1] * 50), want, "bfloat16", "bfloat16: 650 tokens, then 50 one by one", mg)       # its router stands in the last layer
    close(run_cut(b, ids, [255, 257, 2, 186]), want, "bfloat16", "bfloat16: portions that end beside page borders", mg)


def test_replay_program_runs_the_design(tmp_path):
    cfg = NU.MODEL_A
    folder = NU.make_folder(tmp_path, cfg, "A", seed=11)
    ids_a, ids_b = NU.tokens(cfg, 50, seed=7), NU.tokens(cfg, 9, seed=8)
    r = Replay(folder, "float32", tmp_path / "out", max_tokens=128, page_size=16)
    got = r.step([{"id": "a", "tokens": ids_a[:31], "want": [0, 30]}, {"id": "b", "tokens": ids_b[:2], "want": []}])
    close(got, NU.plain_logits(folder, ids_a)[[0, 30]], "float32", "replay: first step")
    assert r.step([{"id": "b", "tokens": ids_b[2:8], "want": []}]) is None
    got = r.step([{"id": "a", "tokens": ids_a[31:], "want": [18]}, {"id": "b", "tokens": ids_b[8:], "want": [0]}], end=["a", "b"])
    close(got, torch.stack([NU.plain_logits(folder, ids_a)[49], NU.plain_logits(folder, ids_b)[8]]), "float32", "replay: last step")
    assert r.close() == 0


# ------------------------------------------------------------------------------------------------ greedy generation through the engine
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_engine(which, graphs, tmp_path):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine, SamplingParams

    cfg = MODELS[which]
    folder = NU.make_folder(tmp_path, cfg, which, seed=11)
    plain_cfg, w = NP.read_model(folder, torch.float64)
    prompts = [NU.tokens(cfg, n, seed=30 + n) for n in (5, 23, 1, 40, 12, 9)]
    engine = Engine(folder, EngineSettings(dtype="float32", num_pages=48, page_size=8, max_running=3, max_step_tokens=32, prefill_chunk=16,
                                           cuda_graphs=graphs))
    done = engine.generate(prompts, SamplingParams(max_tokens=14, ignore_eos=True))
    compared = 0
    for prompt, c in zip(prompts, done):
        want, gaps = NP.greedy(plain_cfg, w, prompt, 14)
        for a, b, gap in zip(c.token_ids, want, gaps):
            if gap < 1e-3:
                break          # a near-tie: from here on the two may differ for no fault
            assert a == b, f"prompt of {len(prompt)}: generated {c.token_ids}, the plain implementation {want}"
            compared += 1
    assert compared >= 60
    if graphs:
        assert engine.counters["graph_steps"] > 0


def test_command_line_generates_with_the_design(tmp_path):
    import json
    import subprocess
    import sys

    import util

    cfg = NU.MODEL_A
    folder = NU.make_folder(tmp_path, cfg, "A", seed=14)
    plain_cfg, w = NP.read_model(folder, torch.float64)
    cmd = [sys.executable, "-m", "oxr_inference_b200", "--model", str(folder), "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6 11 2",
           "--max-tokens", "6", "--dtype", "float32", "--num-pages", "32", "--max-running", "4", "--ignore-eos"]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=str(util.ROOT), timeout=600)
    assert res.returncode == 0, res.stderr
    rows = [json.loads(line) for line in res.stdout.strip().splitlines() if line.startswith("{")]
    for row, prompt in zip(rows, ([5, 17, 3], [9, 8, 7, 6, 11, 2])):
        want, gaps = NP.greedy(plain_cfg, w, prompt, 6)
        for a, b, gap in zip(row["token_ids"], want, gaps):
            if gap < 1e-3:
                break
            assert a == b, f"the command line generated {row['token_ids']}, the plain implementation {want}"
    assert len(rows) == 2


def test_bfloat16_generation_with_graphs_equals_eager(tmp_path):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine, SamplingParams

    cfg = NU.MODEL_C
    folder = NU.make_folder(tmp_path, cfg, "C", seed=12)
    prompts = [NU.tokens(cfg, n, seed=40 + n) for n in (17, 3, 30, 8)]
    out = []
    for graphs in (False, True):
        engine = Engine(folder, EngineSettings(dtype="bfloat16", num_pages=48, page_size=16, max_running=4, cuda_graphs=graphs))
        out.append([c.token_ids for c in engine.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))])
    assert out[0] == out[1]


# ------------------------------------------------------------------------------------------------ marked keys: the attention kernels alone
def plain_attention(q, k, v, pos, *, scale, window, keep_first, sink):
    """One request: q [n, H, D] at positions pos, keys / values [ctx, KV, D] (fp64), by the formulas."""
    per = q.shape[1] // k.shape[1]
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(per, 1)) * scale
    j = torch.arange(k.shape[0])
    seen = j[None, :] <= pos[:, None]
    if window > 0:
        seen &= (pos[:, None] - j[None, :] < window) | (j[None, :] < keep_first)
    s = s.masked_fill(~seen[None], -math.inf)
    m = s.amax(-1, keepdim=True)
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None].expand_as(m))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True) + (torch.exp(sink[:, None, None] - m) if sink is not None else 0.0)
    return torch.einsum("hij,jhd->ihd", e / den, v.repeat_interleave(per, 1))


def marked_case(dtype, H, KV, D, window, keep_first, with_sink, q_lens, ctx_lens, marks, P=8, tiled=False):
    """Requests whose keys are small but for one MARKED key each (a copy of the query direction, so that its score beats all others by far):
    where the mark is visible the output is that key's value, where it is not, an average of the others. ``marks[r]`` is the marked
    position of request r. Pages are dealt out in a shuffled order."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(H * 1000 + D + window * 7 + keep_first)
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    n_pages = sum(-(-c // P) for c in ctx_lens) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    k_pool = torch.zeros(n_pages, P, KV, D, dtype=tdt)
    v_pool = torch.zeros(n_pages, P, KV, D, dtype=tdt)
    width = max(-(-c // P) for c in ctx_lens)
    table = torch.full((len(ctx_lens), width), -1, dtype=torch.int32)
    direction = torch.randn(D, generator=g)
    direction = direction / direction.norm()
    scale = 1.0
    sink = (torch.randn(H, generator=g) * 2 + 1).float() if with_sink else None
    qs, pos, wants = [], [], []
    for r, (c, ql, mark) in enumerate(zip(ctx_lens, q_lens, marks)):
        k = (torch.randn(c, KV, D, generator=g) * 0.3).to(tdt)
        v = torch.randn(c, KV, D, generator=g).to(tdt)
        k[mark] = (direction * 6.0).to(tdt)
        for j in range(c):
            page = order.pop() if j % P == 0 else int(table[r, j // P])
            table[r, j // P] = page
            k_pool[page, j % P], v_pool[page, j % P] = k[j], v[j]
        q = (direction * 4.0 + torch.randn(ql, H, D, generator=g) * 0.3).to(tdt)
        p_r = torch.arange(c - ql, c)
        wants.append(plain_attention(q.double(), k.double(), v.double(), p_r, scale=scale, window=window, keep_first=keep_first,
                                     sink=None if sink is None else sink.double()).reshape(ql, H * D))
        qs.append(q.reshape(ql, H * D))
        pos.append(p_r)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    q_all = torch.cat(qs).to(DEV)
    positions = torch.cat(pos).to(DEV, torch.int32)
    req_of = torch.repeat_interleave(torch.arange(len(q_lens)), torch.tensor(q_lens)).to(DEV, torch.int32)
    if tiled:
        specs = ops.attention_tile_specs(H, KV, D, torch.bfloat16, None)
        tiles = {}
        for spec in specs:
            rows, lo, hi = spec
            treq, ttok = [], []
            for r, ql in enumerate(q_lens):
                if lo <= ql <= hi:
                    for t0 in range(0, ql, rows):
                        treq.append(r); ttok.append(t0)
            tiles[spec] = (i32(treq or [0]), i32(ttok or [0]), len(treq))
        got = ops.paged_attention(q_all.view(-1, H, D), k_pool.to(DEV), v_pool.to(DEV), tiles=tiles, cu_q=i32([0] + torch.tensor(q_lens).cumsum(0).tolist()),
                                  ctx_lens=i32(ctx_lens), block_table=table.to(DEV), page_size=P, scale=scale, window=window, keep_first=keep_first,
                                  kv_len_bound=max(ctx_lens), status=status, sink=None if sink is None else sink.to(DEV)).view(-1, H * D)
    else:
        got = ops.attention_rows(q_all, H, k_pool.to(DEV), v_pool.to(DEV), value_dim=D, positions=positions, req_of_token=req_of, block_table=table.to(DEV),
                                 scale=scale, window=window, keep_first=keep_first, sink=None if sink is None else sink.to(DEV), status=status)
    ops.check_status(status)
    want = torch.cat(wants).float()
    err = (got.float().cpu() - want).abs().max() / want.abs().max()
    assert err < (2e-5 if dtype == "float32" else 2e-2), f"off by {err:.2e} of the largest entry"


# the marked key: far back, on a page's first and last row, just inside and just outside the window, the last kept key and the first one
# that is not kept, the very first key, the query itself
WINDOW, KEEP = 21, 6
MARKS = {"far_back_in_no_window": (0, 0, 3), "page_first_row": (0, 0, 64), "page_last_row": (0, 0, 63), "window_first_inside": (WINDOW, KEEP, 130 - WINDOW),
         "window_last_outside": (WINDOW, KEEP, 129 - WINDOW), "last_kept": (WINDOW, KEEP, KEEP - 1), "first_not_kept": (WINDOW, KEEP, KEEP),
         "first_key": (WINDOW, KEEP, 0), "window_without_kept_keys": (WINDOW, 0, 2), "kept_beyond_a_block": (9, 70, 69), "kept_beyond_a_block_out": (9, 70, 70)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sink", [False, True])
@pytest.mark.parametrize("where", sorted(MARKS))
def test_marked_keys_rows_kernel(where, sink, dtype):
    window, keep, mark = MARKS[where]
    # the last query of request 0 stands at 129; a portion of 5 tokens, a single token, a two-token request
    marked_case(dtype, 6, 2, 24, window, keep, sink, [5, 1, 2], [130, 130, 2], [mark, mark, 0])


@pytest.mark.parametrize("sink", [False, True])
@pytest.mark.parametrize("shape", [(8, 2, 64), (3, 3, 32), (4, 1, 128)])
@pytest.mark.parametrize("where", sorted(MARKS))
def test_marked_keys_tiled_kernels(where, shape, sink):
    window, keep, mark = MARKS[where]
    H, KV, D = shape
    # a long portion (the prefill kernel), single tokens and a short portion (the split-KV kernel), a two-token request
    marked_case("bfloat16", H, KV, D, window, keep, sink, [70, 1, 5, 2], [130, 130, 130, 2], [mark, mark, mark, 0], tiled=True)


# ------------------------------------------------------------------------------------------------ the new kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,DK,taps,half,norm,after,vmode", [(4, 2, 16, 3, 4, "weighted", False, "keys"), (3, 1, 24, 1, 12, "unit", True, "copy"),
                                                                (2, 2, 40, 5, 0, None, False, "copy"), (5, 5, 8, 0, 3, "weighted", True, "keys"),
                                                                (2, 1, 64, 2, 32, "unit", False, None), (4, 2, 128, 4, 32, "weighted", False, "keys"),
                                                                (6, 2, 64, 3, 16, "unit", True, "copy"), (3, 3, 48, 0, 8, "weighted", True, "copy"),
                                                                (5, 1, 256, 2, 128, "weighted", False, "keys"), (2, 2, 24, 3, 0, "unit", False, "keys")])
def test_head_prep_against_the_formulas(dtype, H, KV, DK, taps, half, norm, after, vmode):
    """Two requests in unequal portions down to one token, fed step by step: bias, filter with its tails, the values that are the filtered
    keys, norm before or after the rotation, the rotation of pairs (i, i + half), the cache rows; against float64, token by token."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(H * 100 + DK + taps)
    rnd = lambda *s: torch.randn(*s, generator=g)
    has_k = vmode is not None
    DV = DK if vmode != "copy" else DK + 8
    cq, ck, cv = H * DK, KV * DK if has_k else 0, KV * DV if vmode == "copy" else 0
    ch = cq + ck
    lens = [13, 6]
    proj_all = [rnd(n, cq + ck + cv + 3).to(dtype) for n in lens]
    bias = rnd(ch) if taps != 1 else None
    filt = (rnd(ch, taps) + 0.5) if taps > 0 else None
    qw, kw = 1 + 0.2 * rnd(DK), 1 + 0.2 * rnd(DK)
    eps = 1e-5
    freqs = torch.rand(half, generator=g, dtype=torch.float64) + 0.05 if half else None

    def reference(x, n):
        u = x[:, :ch].double() + (bias.double() if bias is not None else 0.0)
        y = NP.causal_filter(u, filt.double()) if filt is not None else u
        qh, kh = y[:, :cq].reshape(n, H, DK), y[:, cq:].reshape(n, KV, DK) if has_k else None
        vals = kh.clone() if vmode == "keys" else (x[:, ch:ch + cv].double().reshape(n, KV, DV) if vmode == "copy" else None)

        def steps(t, w):
            if norm and not after:
                t = NP.rms(t, eps) * (w.double() if norm == "weighted" else 1.0)
            if half:
                t = NP.rotate_halves(t, freqs.tolist())
            if norm and after:
                t = NP.rms(t, eps) * (w.double() if norm == "weighted" else 1.0)
            return t
        return steps(qh, qw), steps(kh, kw) if has_k else None, vals

    P = 4
    k_pool = torch.zeros(12, P, KV, DK, dtype=dtype, device=DEV)
    v_pool = torch.zeros(12, P, KV, DV, dtype=dtype, device=DEV)
    tails = torch.zeros(3, 8 + ch * max(taps - 1, 0), device=DEV)[:, 8:] if taps > 1 else None     # a view with a row stride of its own
    status = ops.new_status(DEV)
    slot_of = [[(1 + 2 * r + 6 * (j // P // 2 * 0) + (j // P)) * P + j % P for j in range(n)] for r, n in enumerate(lens)]
    slot_of = [[((r * 5 + j // P) + 1) * P + j % P for j in range(n)] for r, n in enumerate(lens)]
    got_q = [[], []]
    at = [0, 0]
    for cut in ([5, 2], [1, 1], [2, 0], [5, 3]):
        rows, slots, req_of, cu, positions = [], [], [], [0], []
        live = [r for r in (0, 1) if cut[r] > 0]
        for i, r in enumerate(live):
            rows.append(proj_all[r][at[r]:at[r] + cut[r]])
            slots += slot_of[r][at[r]:at[r] + cut[r]]
            req_of += [i] * cut[r]
            positions += list(range(at[r], at[r] + cut[r]))
            cu.append(cu[-1] + cut[r])
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        cos = sin = None
        if half:
            ang = torch.tensor(positions, dtype=torch.float64)[:, None] * freqs[None, :]
            cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
        q = ops.head_prep(torch.cat(rows).to(DEV), q_col0=0, k_col0=cq if has_k else None, v_col0=ch if vmode == "copy" else None,
                          values_are_keys=vmode == "keys", num_heads=H, num_kv_heads=KV, key_dim=DK, value_dim=DV, bias=None if bias is None else bias.to(DEV),
                          taps=None if filt is None else filt.to(DEV), taps_t=None if filt is None else filt.t().contiguous().to(DEV), tails=tails, norm=norm, norm_after_rotation=after, q_weight=qw.to(DEV), k_weight=kw.to(DEV),
                          eps=eps, cos=cos, sin=sin, k_pool=k_pool if has_k else None, v_pool=v_pool if has_k else None, slots=i32(slots), req_of_token=i32(req_of),
                          cu_q=i32(cu), state_slots=i32([r + 1 for r in live]), n_requests=len(live), status=status)
        row = 0
        for r in live:
            got_q[r].append(q[row:row + cut[r]].float().cpu())
            row += cut[r]
            at[r] += cut[r]
    ops.check_status(status)
    tol = 3e-5 if dtype == torch.float32 else 2.5e-2
    for r, n in enumerate(lens):
        want_q, want_k, want_v = reference(proj_all[r], n)
        got = torch.cat(got_q[r]).reshape(n, H, DK).double()
        assert (got - want_q).abs().max() < tol * (1 + want_q.abs().max()), f"queries of request {r}"
        if has_k:
            idx = torch.tensor(slot_of[r])
            gk = k_pool.view(-1, KV, DK)[idx].double().cpu()
            gv = v_pool.view(-1, KV, DV)[idx].double().cpu()
            assert (gk - want_k).abs().max() < tol * (1 + want_k.abs().max()), f"keys of request {r}"
            assert (gv - want_v).abs().max() < tol * (1 + want_v.abs().max()), f"values of request {r}"
        if taps > 1:
            u = proj_all[r][:, :ch].double() + bias.double()
            want_tail = u[n - (taps - 1):].reshape(-1)      # the oldest value of every channel first
            assert (tails[r + 1].double().cpu() - want_tail).abs().max() < 1e-5 * (1 + want_tail.abs().max()), f"tails of request {r}"
    if taps > 1:
        assert tails[0].abs().max() == 0, "a slot nobody used was written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_thread", [0, 16, 32])
@pytest.mark.parametrize("H,DK,DV,tau", [(3, 12, 20, 4.0), (1, 70, 33, 1.5), (2, 64, 64, 16.0), (2, 130, 8, 40.0), (2, 128, 40, 8.0)])
def test_gated_linear_attention_scan_continues_from_its_state(dtype, H, DK, DV, tau, per_thread):
    """Two requests in unequal portions over three steps against the recurrence in float64, token by token; the state a step leaves is the
    state the next one starts from; a slot nobody uses stays zero. With both splits of a head's key channels over threads."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(H + DK + DV)
    lens = [41, 11]
    inputs = []
    for n in lens:
        proj = (torch.randn(n, 2 * H * DK + H * DV + 5, generator=g) * 0.7).to(dtype)
        z = torch.randn(n, H * DK, generator=g) * 2
        inputs.append((proj, z))
    zb = torch.randn(H * DK, generator=g) + 2.0
    state = torch.zeros(4, 9 + H * DK * DV, device=DEV)[:, 9:]       # a view with a row stride of its own
    got = [[], []]
    at = [0, 0]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    for cut in ([30, 1], [1, 1], [10, 9]):
        projs, zs, cu = [], [], [0]
        for r in (0, 1):
            projs.append(inputs[r][0][at[r]:at[r] + cut[r]])
            zs.append(inputs[r][1][at[r]:at[r] + cut[r]])
            cu.append(cu[-1] + cut[r])
        y = ops.gla_scan(torch.cat(projs).to(DEV), 0, H * DK, 2 * H * DK, torch.cat(zs).to(DEV), zb.to(DEV), heads=H, key_dim=DK, value_dim=DV, tau=tau,
                         q_scale=DK ** -0.5, state=state, cu_q=i32(cu), state_slots=i32([2, 0]), n_requests=2, key_entries_per_thread=per_thread)
        for r in (0, 1):
            got[r].append(y[cu[r]:cu[r + 1]].cpu())
            at[r] += cut[r]
    for r, n in enumerate(lens):
        proj, z = inputs[r][0].double(), inputs[r][1].double()
        q = proj[:, :H * DK].reshape(n, H, DK) * DK ** -0.5
        k = proj[:, H * DK:2 * H * DK].reshape(n, H, DK)
        v = proj[:, 2 * H * DK:2 * H * DK + H * DV].reshape(n, H, DV)
        alpha = (torch.sigmoid(z + zb.double()) ** (1.0 / tau)).reshape(n, H, DK)
        S = torch.zeros(H, DK, DV, dtype=torch.float64)
        want = torch.zeros(n, H, DV, dtype=torch.float64)
        for t in range(n):
            S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
            want[t] = torch.einsum("hdv,hd->hv", S, q[t])
        err = (torch.cat(got[r]).double().reshape(n, H, DV) - want).abs().max() / want.abs().max()
        assert err < 5e-5, f"request {r}: off by {err:.2e}"
        assert (state[[2, 0][r]].double().cpu().reshape(H, DK, DV) - S).abs().max() < 5e-5 * (1 + S.abs().max()), f"state of request {r}"
    assert state[1].abs().max() == 0 and state[3].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels_against_their_formulas(dtype):
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    near = lambda got, want, what: (lambda e: (_ for _ in ()).throw(AssertionError(f"{what}: off by {e:.2e}")) if e > tol else None)(
        float((got.double().cpu() - want).abs().max() / (1 + want.abs().max())))
    for n, hidden in ((5, 50), (130, 64), (3, 1032)):
        # the output norm's add, with the rounded copy of the new stream
        stream0, y, w = rnd(n, hidden), rnd(n, hidden).to(dtype), 1 + 0.1 * rnd(hidden)
        stream = stream0.clone().to(DEV)
        copy = ops.norm_add_norm(stream, y.to(DEV), w.to(DEV), 1e-5, rounded=True)
        want = stream0.double() + NP.rms(y.double(), 1e-5) * w.double()
        near(stream, want, "stream after the add")
        assert copy.dtype == dtype
        near(copy, want, "rounded copy of the stream")
        # the mean of two normed results
        a, b, wa, wb = rnd(n, hidden).to(dtype), (3 * rnd(n, hidden)).to(dtype), 1 + 0.1 * rnd(hidden), 0.5 + 0.1 * rnd(hidden)
        got = ops.pair_norm_mean(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-6)
        near(got, 0.5 * (NP.rms(a.double(), 1e-6) * wa.double() + NP.rms(b.double(), 1e-6) * wb.double()), "pair_norm_mean")
        # a second result joins behind one gate per row
        yy, s, z = rnd(n, hidden).to(dtype), rnd(n, hidden).to(dtype), rnd(n) * 3
        got = ops.add_row_gated_(yy.clone().to(DEV), s.to(DEV), z.to(DEV))
        near(got, yy.double() + torch.sigmoid(z.double())[:, None] * s.double(), "add_row_gated")
    # the sigmoid gate per channel and per head
    for n, H, DV, lead in ((7, 3, 10, 4), (7, 3, 16, 8), (40, 5, 24, 16)):      # odd sizes, and rows of whole 16-byte words
        o, proj = rnd(n, H * DV).to(dtype), rnd(n, lead + H * DV).to(dtype)
        got = ops.sigmoid_gate_(o.clone().to(DEV), proj.to(DEV), lead, DV, per_head=False)
        near(got, o.double() * torch.sigmoid(proj[:, lead:].double()), "gate per channel")
        got = ops.sigmoid_gate_(o.clone().to(DEV), proj.to(DEV), 2, DV, per_head=True)
        near(got, (o.double().reshape(n, H, DV) * torch.sigmoid(proj[:, 2:2 + H].double())[:, :, None]).reshape(n, -1), "gate per head")
    n, H, DV = 7, 3, 10
    # SiLU-gated experts over stacked columns with the weight on the input, and on the output
    for E, ff in ((4, 6), (3, 16)):
        gu, gate = rnd(n, E * 2 * ff).to(dtype), torch.where(torch.rand(n, E, generator=g) < 0.5, torch.rand(n, E, generator=g), torch.zeros(n, E))
        gud = gu.double().reshape(n, E, 2, ff)
        wd = gate.double()[:, :, None]
        got = ops.expert_silu_glu(gu.to(DEV), gate.to(DEV), ff, on_input=True)
        near(got, (NP.silu(wd * gud[:, :, 0]) * (wd * gud[:, :, 1])).reshape(n, -1), "experts, weight on the input")
        got = ops.expert_silu_glu(gu.to(DEV), gate.to(DEV), ff, on_input=False)
        near(got, (wd * NP.silu(gud[:, :, 0]) * gud[:, :, 1]).reshape(n, -1), "experts, weight on the output")
        got = ops.expert_silu_glu(gu.to(DEV), None, ff, on_input=True)
        near(got, (NP.silu(gud[:, :, 0]) * gud[:, :, 1]).reshape(n, -1), "experts, no weight")
    E, ff = 4, 6
    gu, gate = rnd(n, E * 2 * ff).to(dtype), torch.where(torch.rand(n, E, generator=g) < 0.5, torch.rand(n, E, generator=g), torch.zeros(n, E))
    gud = gu.double().reshape(n, E, 2, ff)
    wd = gate.double()[:, :, None]
    got = ops.expert_silu_glu(gu.to(DEV), gate.to(DEV), ff, on_input=True)
    near(got, (NP.silu(wd * gud[:, :, 0]) * (wd * gud[:, :, 1])).reshape(n, -1), "experts, weight on the input")
    got = ops.expert_silu_glu(gu.to(DEV), gate.to(DEV), ff, on_input=False)
    near(got, (wd * NP.silu(gud[:, :, 0]) * gud[:, :, 1]).reshape(n, -1), "experts, weight on the output")
    # the capped logits (32-bit whatever the dtype)
    x = rnd(9, 77) * 20
    near(ops.tanh_cap_(x.clone().to(DEV), 7.0), 7.0 * torch.tanh(x.double() / 7.0), "tanh cap")
    # the head norm with a SiLU gate
    y, pr, wn = rnd(n, H * DV), rnd(n, 3 + H * DV).to(dtype), 1 + 0.1 * rnd(H * DV)
    got = ops.head_norm_gate(y.to(DEV), pr.to(DEV), 3, wn.to(DEV), H, 1e-5, silu=True)
    near(got, (NP.rms(y.double().reshape(n, H, DV), 1e-5).reshape(n, -1) * wn.double()) * NP.silu(pr[:, 3:].double()), "head norm with a SiLU gate")
