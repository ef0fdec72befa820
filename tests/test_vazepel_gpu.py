"""Vazepel on the GPU against the plain statement in ``tests/plain/vazepel_plain.py``: each mechanism alone, whole prompts against
token-by-token decoding, portions down to two tokens, batches of unequal requests, pages that are used again, keys far back, at page
borders, at a sequence's first positions and at a window's edge, long decoding, greedy generation through the engine, and the new
kernels against their formulas."""

import math

import pytest
import torch

import vazepel_util as VU
from plain import vazepel_plain as VP
from util import Replay

pytestmark = pytest.mark.gpu

DEV = "cuda"

CLOSE_CALL = 0.002
"""bfloat16 rows at which some router of the plain model decided by less than this (a difference of softmax scores) are not compared:
a score that differs by a rounding step may choose another expert there, for no fault. (32-bit compares every row.)"""


def close(got, want, dtype, what, margins=None):
    """32-bit: every row within 2e-4 of the row's spread. bfloat16: within 8e-2, one row in twenty up to 0.25."""
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
    assert err.max() <= 0.25 and over <= len(err) // 20, (
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
    return torch.cat(rows)


# ------------------------------------------------------------------------------------------------ each mechanism alone
L, MOE, DENSE = VU.layer, VU.moe, VU.dense
SINGLE = {
    "attention_alone": VU.model_config([L()]),
    "no_rotation": VU.model_config([L(rot=0)]),
    "all_entries_rotated": VU.model_config([L(rot=16, base=7.0)]),
    "two_entries_rotated": VU.model_config([L(rot=2, base=3.0)]),
    "tight_cap": VU.model_config([L(softcap=0.7, scale=0.6)]),
    "one_head": VU.model_config([L(heads=1, kv_heads=1, dim=32, vdim=16, rot=32)]),
    "as_many_kv_heads_as_heads": VU.model_config([L(heads=3, kv_heads=3, dim=16, vdim=16, rot=8)]),
    "many_heads": VU.model_config([L(heads=12, kv_heads=3, dim=16, vdim=32, rot=16, scale=0.25)], width=64),
    "sixteen_heads_of_64": VU.model_config([L(heads=16, kv_heads=2, dim=64, vdim=64, rot=32, scale=0.12)], width=64),
    "odd_sizes": VU.model_config([L(heads=3, kv_heads=1, dim=22, vdim=10, rot=6)], width=40),
    "values_wider_than_keys": VU.model_config([L(heads=2, kv_heads=2, dim=16, vdim=48, rot=16)]),
    "dense_feed_forward": VU.model_config([L(mlp=DENSE())]),
    "depth_average_over_four": VU.model_config([L(heads=2, kv_heads=1, dim=16, vdim=16, rot=8, mlp=DENSE(ff=24)) for _ in range(4)]),
    "experts": VU.model_config([L(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE())]),
    "experts_no_shared": VU.model_config([L(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(shared=0))]),
    "experts_one_group": VU.model_config([L(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(count=0, top=3))]),
    "experts_groups_of_one": VU.model_config([L(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(experts=5, count=5, keep=3, top=2))]),
    "experts_top_one": VU.model_config([L(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(experts=8, count=2, keep=1, top=1, limit=0.4))]),
    "experts_all_chosen": VU.model_config([L(heads=1, kv_heads=1, dim=16, vdim=16, mlp=MOE(experts=4, count=2, keep=2, top=4, limit=5.0))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_mechanism(name, dtype, tmp_path):
    cfg = SINGLE[name]
    folder = VU.make_folder(tmp_path, cfg, name, seed=5)
    ids = VU.tokens(cfg, 61, seed=1)
    want = VU.plain_logits(folder, ids)
    r = runner_for(folder, dtype)
    mg = VU.router_margins(folder, ids)
    close(run_cut(r, ids, [61]), want, dtype, f"{name}, whole prompt", mg)
    close(run_cut(r, ids, [29] + [1] * 32), want, dtype, f"{name}, 29 tokens then one by one", mg)
    close(run_cut(r, ids, [2, 3, 2, 11, 2, 17, 1, 2, 21]), want, dtype, f"{name}, portions", mg)


def test_layer_results_one_by_one(tmp_path):
    """The stream after every layer (the depth average included) against the plain statement's, in 32-bit."""
    from oxr_inference_b200.engine.batch import StepEntry

    cfg = VU.MODEL_P
    folder = VU.make_folder(tmp_path, cfg, "P", seed=2)
    ids = VU.tokens(cfg, 23, seed=6)
    plain_cfg, w = VP.read_model(folder, torch.float64)
    want: list = []
    VP.forward(plain_cfg, w, ids, layers_out=want)
    r = runner_for(folder, "float32")
    got = []
    blocks = r.model.blocks
    originals = [b.forward for b in blocks]
    for b, f in zip(blocks, originals):
        def wrapped(*a, _f=f, **k):
            out = _f(*a, **k)
            after = out[1].clone()
            if out[0] is not None:   # the add is left to the next block's norm: made here, on the copy
                out[0].apply(after)
            got.append(after)
            return out
        b.forward = wrapped
    rc = r.cache.open("r")
    assert r.cache.reserve(rc, len(ids))
    r.step([StepEntry(rc, ids, [len(ids) - 1])])
    r.cache.close(rc)
    for b, f in zip(blocks, originals):
        b.forward = f
    assert len(got) == len(want) == 4
    for i, (a, b) in enumerate(zip(got, want)):
        err = (a.double().cpu() - b).abs().max() / b.abs().max()
        assert err < 2e-5, f"layer {i}: off by {err:.2e} of the stream's largest entry"


# ------------------------------------------------------------------------------------------------ whole models, every cutting
MODELS = {"P": VU.MODEL_P, "Q": VU.MODEL_Q, "R": VU.MODEL_R, "T": VU.MODEL_T}


@pytest.fixture(scope="module", params=[(m, d) for m in sorted(MODELS) for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def model(request, tmp_path_factory):
    name, dtype = request.param
    folder = VU.make_folder(tmp_path_factory.mktemp(f"vazepel_{name}_{dtype}"), MODELS[name], name, seed=11)
    return name, dtype, folder, runner_for(folder, dtype, page_size=8, num_pages=40)


def test_whole_prompt_equals_token_by_token(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    for n in (1, 2, 9, 75):
        ids = VU.tokens(cfg, n, seed=2)
        want = VU.plain_logits(folder, ids)
        mg = VU.router_margins(folder, ids)
        close(run_cut(r, ids, [n]), want, dtype, f"{name}: whole prompt of {n}", mg)
        close(run_cut(r, ids, [1] * n), want, dtype, f"{name}: {n} tokens one by one", mg)


def test_portions_of_several_sizes(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = VU.tokens(cfg, 120, seed=3)
    want = VU.plain_logits(folder, ids)
    for cuts in ([2] * 60, [7, 2, 13, 3, 2, 31, 1, 16, 2, 17, 8, 18], [33, 33, 33, 21], [119, 1], [15, 16, 17, 32, 40]):
        close(run_cut(r, ids, cuts), want, dtype, f"{name}: portions {cuts[:4]}...", VU.router_margins(folder, ids))


def test_long_decoding(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = VU.tokens(cfg, 260, seed=4)
    close(run_cut(r, ids, [4] + [1] * 256), VU.plain_logits(folder, ids), dtype, f"{name}: 256 decoded tokens", VU.router_margins(folder, ids))


def test_unequal_requests_in_one_batch_with_pages_used_again(model):
    """Four live requests at most, 40 pages of 8 tokens: the lengths below need far more over time, so pages and request slots come
    back and are handed out again; every request's logits equal those it gets alone."""
    name, dtype, folder, r = model
    cfg = MODELS[name]
    lengths = [97, 3, 64, 30, 1, 121, 45, 18, 70]
    todo = [(f"q{i}", VU.tokens(cfg, n, seed=20 + i)) for i, n in enumerate(lengths)]
    live, got, pages_seen = {}, {}, []
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
            row += c
            live[key][2] += c
            if live[key][2] == len(live[key][1]):
                r.cache.close(live.pop(key)[0])
        step += 1
    r.check()
    r.cache.check()
    assert sum(-(-n // 8) for n in lengths) > 40, "the requests never needed a page twice"
    for i, n in enumerate(lengths):
        ids = VU.tokens(cfg, n, seed=20 + i)
        close(torch.cat(got[f"q{i}"]), VU.plain_logits(folder, ids), dtype, f"{name}: request {i} of {n} tokens in the mix", VU.router_margins(folder, ids))


def test_far_keys(tmp_path):
    """A prompt of 700 tokens with peaked attention: the last logits rest on keys from hundreds of tokens back, across dozens of
    pages; in 32-bit a lost one shows."""
    cfg = VU.MODEL_Q
    folder = VU.make_folder(tmp_path, cfg, "far", seed=3, sharpen=16.0)
    ids = VU.tokens(cfg, 700, seed=9)
    want = VU.plain_logits(folder, ids)
    r = runner_for(folder, "float32", page_size=16, num_pages=50)
    close(run_cut(r, ids, [650] + [1] * 50), want, "float32", "650 tokens, then 50 one by one")
    close(run_cut(r, ids, [255, 257, 2, 186]), want, "float32", "portions that end beside page borders")
    b = runner_for(folder, "bfloat16", page_size=16, num_pages=50)
    close(run_cut(b, ids, [650] + [1] * 50), want, "bfloat16", "bfloat16: 650 tokens, then 50 one by one", VU.router_margins(folder, ids))
    close(run_cut(b, ids, [255, 257, 2, 186]), want, "bfloat16", "bfloat16: portions that end beside page borders", VU.router_margins(folder, ids))


def test_replay_program_runs_the_design(tmp_path):
    cfg = VU.MODEL_R
    folder = VU.make_folder(tmp_path, cfg, "R", seed=11)
    ids_a, ids_b = VU.tokens(cfg, 50, seed=7), VU.tokens(cfg, 9, seed=8)
    r = Replay(folder, "float32", tmp_path / "out", max_tokens=128, page_size=16)
    got = r.step([{"id": "a", "tokens": ids_a[:31], "want": [0, 30]}, {"id": "b", "tokens": ids_b[:2], "want": []}])
    close(got, VU.plain_logits(folder, ids_a)[[0, 30]], "float32", "replay: first step")
    assert r.step([{"id": "b", "tokens": ids_b[2:8], "want": []}]) is None
    got = r.step([{"id": "a", "tokens": ids_a[31:], "want": [18]}, {"id": "b", "tokens": ids_b[8:], "want": [0]}], end=["a", "b"])
    close(got, torch.stack([VU.plain_logits(folder, ids_a)[49], VU.plain_logits(folder, ids_b)[8]]), "float32", "replay: last step")
    assert r.close() == 0


# ------------------------------------------------------------------------------------------------ greedy generation through the engine
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("which", ["P", "Q"])
def test_greedy_generation_through_the_engine(which, graphs, tmp_path):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine, SamplingParams

    cfg = MODELS[which]
    folder = VU.make_folder(tmp_path, cfg, which, seed=11)
    plain_cfg, w = VP.read_model(folder, torch.float64)
    prompts = [VU.tokens(cfg, n, seed=30 + n) for n in (5, 23, 1, 40, 12, 9)]
    engine = Engine(folder, EngineSettings(dtype="float32", num_pages=48, page_size=8, max_running=3, max_step_tokens=32, prefill_chunk=16,
                                           cuda_graphs=graphs))
    done = engine.generate(prompts, SamplingParams(max_tokens=14, ignore_eos=True))
    compared = 0
    for prompt, c in zip(prompts, done):
        want, gaps = VP.greedy(plain_cfg, w, prompt, 14)
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

    cfg = VU.MODEL_R
    folder = VU.make_folder(tmp_path, cfg, "R", seed=14)
    plain_cfg, w = VP.read_model(folder, torch.float64)
    cmd = [sys.executable, "-m", "oxr_inference_b200", "--model", str(folder), "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6 11 2",
           "--max-tokens", "6", "--dtype", "float32", "--num-pages", "32", "--max-running", "4", "--ignore-eos"]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=str(util.ROOT), timeout=600)
    assert res.returncode == 0, res.stderr
    rows = [json.loads(line) for line in res.stdout.strip().splitlines() if line.startswith("{")]
    for row, prompt in zip(rows, ([5, 17, 3], [9, 8, 7, 6, 11, 2])):
        want, gaps = VP.greedy(plain_cfg, w, prompt, 6)
        for a, b, gap in zip(row["token_ids"], want, gaps):
            if gap < 1e-3:
                break
            assert a == b, f"the command line generated {row['token_ids']}, the plain implementation {want}"
    assert len(rows) == 2


def test_bfloat16_generation_with_graphs_equals_eager(tmp_path):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine, SamplingParams

    cfg = VU.MODEL_Q
    folder = VU.make_folder(tmp_path, cfg, "Q", seed=12)
    prompts = [VU.tokens(cfg, n, seed=40 + n) for n in (17, 3, 30, 8)]
    out = []
    for graphs in (False, True):
        engine = Engine(folder, EngineSettings(dtype="bfloat16", num_pages=48, page_size=16, max_running=4, cuda_graphs=graphs))
        out.append([c.token_ids for c in engine.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))])
    assert out[0] == out[1]


# ------------------------------------------------------------------------------------------------ the tensor-core attention kernel alone
def plain_mixed_attention(q, k, v, pos, ctx_of, *, scale, cap, mix, sink, window, gate):
    """One request: q [n, H, DK] at positions pos, keys / values k, v [ctx, KV, D*] (fp64), by the formulas."""
    n, H, _ = q.shape
    per = H // k.shape[1]
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(per, 1)) * scale
    if cap > 0:
        s = cap * torch.tanh(s / cap)
    if mix is not None:
        s = torch.einsum("hg,gij->hij", mix, s)
    j = torch.arange(ctx_of)
    seen = j[None, :] <= pos[:, None]
    if window > 0:
        seen &= j[None, :] > pos[:, None] - window
    e = torch.where(seen[None], torch.exp(s - s.amax(-1, keepdim=True)), torch.zeros_like(s))
    denom = e.sum(-1) + (torch.exp(-s.amax(-1)) if sink else 0.0)
    o = torch.einsum("hij,jhd->ihd", e / denom[..., None], v.repeat_interleave(per, 1))
    if gate is not None:
        o = o * torch.sigmoid(gate)
    return o


@pytest.mark.parametrize("H,KV,DK,DV", [(8, 2, 64, 128), (4, 4, 128, 64), (16, 1, 64, 64), (6, 3, 128, 128), (32, 8, 128, 128), (2, 1, 64, 64)])
@pytest.mark.parametrize("window,splits", [(0, None), (0, 3), (37, 1), (21, 2)])
def test_tiled_kernel_against_the_formulas(H, KV, DK, DV, window, splits):
    tiled_case(H, KV, DK, DV, window, splits, [1, 1, 67, 2, 45], False)


@pytest.mark.parametrize("H,KV,DK,DV", [(8, 2, 64, 128), (32, 8, 128, 128), (3 * 2, 3, 64, 64), (16, 16, 128, 64)])
@pytest.mark.parametrize("window,splits", [(0, None), (50, 4), (0, 9)])
def test_tiled_kernel_on_single_tokens(H, KV, DK, DV, window, splits):
    tiled_case(H, KV, DK, DV, window, splits, [1, 1, 1, 1, 1], True)


def tiled_case(H, KV, DK, DV, window, splits, q_lens, single):
    """Requests of unequal lengths and portions (one token, two, a run that ends inside a tile, a long one) over pages dealt out in a
    shuffled order; the keys in one piece and in several; with and without a window; the mix far from the identity."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(H * 1000 + DK + window)
    tile = ops.attention_mix_tile(H, KV, DK, DV, torch.bfloat16)
    assert tile is not None
    P, ctx_lens = 8, [70, 1, 131, 19, 45]
    n_pages = sum(-(-c // P) for c in ctx_lens) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    k_pool = torch.zeros(n_pages, P, KV, DK, dtype=torch.bfloat16)
    v_pool = torch.zeros(n_pages, P, KV, DV, dtype=torch.bfloat16)
    width = max(-(-c // P) for c in ctx_lens)
    table = torch.full((len(ctx_lens), width), -1, dtype=torch.int32)
    mix = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).bfloat16().float()
    scale, cap = 0.5 * DK ** -0.5, 7.0
    qs, gates, pos, wants = [], [], [], []
    for r, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        k = (torch.randn(c, KV, DK, generator=g) * 1.5).bfloat16()
        v = torch.randn(c, KV, DV, generator=g).bfloat16()
        for j in range(c):
            page = order.pop() if j % P == 0 else int(table[r, j // P])
            table[r, j // P] = page
            k_pool[page, j % P], v_pool[page, j % P] = k[j], v[j]
        q = (torch.randn(ql, H, DK, generator=g) * 1.5).bfloat16()
        gate = torch.randn(ql, H, DV, generator=g).bfloat16()
        p_r = torch.arange(c - ql, c)
        wants.append(plain_mixed_attention(q.double(), k.double(), v.double(), p_r, c, scale=scale, cap=cap, mix=mix.double(), sink=True,
                                           window=window, gate=gate.double()).reshape(ql, H * DV))
        qs.append(q.reshape(ql, H * DK)); gates.append(gate.reshape(ql, H * DV)); pos.append(p_r)
    n = sum(q_lens)
    # q and the gate as columns of one stacked row, as the mixer hands them over
    proj = torch.cat([torch.cat(qs), torch.zeros(n, 24, dtype=torch.bfloat16), torch.cat(gates)], 1).to(DEV)
    treq, ttok = [], []
    for r, ql in enumerate(q_lens):
        for t0 in range(0, ql, tile[0]):
            treq.append(r); ttok.append(t0)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    cu = i32([0] + torch.tensor(q_lens).cumsum(0).tolist())
    status = ops.new_status(DEV)
    common = dict(positions=torch.cat(pos).to(DEV, torch.int32), block_table=table.to(DEV), scale=scale, softcap=cap, head_mix=mix.to(DEV),
                  unit_sink=True, window=window, gate=proj[:, H * DK + 24:], status=status)
    got = ops.attention_mix_tiled(proj, H, k_pool.to(DEV), v_pool.to(DEV), tile=tile, tiles=(i32(treq), i32(ttok), len(treq)), cu_q=cu,
                                  kv_len_bound=max(ctx_lens), splits=splits, single_tokens=single, **common)
    rows = ops.attention_mix_rows(proj, H, k_pool.to(DEV), v_pool.to(DEV), req_of_token=torch.repeat_interleave(torch.arange(len(q_lens)), torch.tensor(q_lens)).to(DEV, torch.int32),
                                  **common)
    ops.check_status(status)
    want = torch.cat(wants).float()
    err = (got.float().cpu() - want).abs().max() / want.abs().max()
    err_rows = (rows.float().cpu() - want).abs().max() / want.abs().max()
    assert err_rows < 1e-2, f"the rows kernel is off by {err_rows:.2e}"
    assert err < 1.5e-2, f"the tiled kernel is off by {err:.2e} of the largest entry (the rows kernel: {err_rows:.2e})"


# ------------------------------------------------------------------------------------------------ the stream's kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,hidden", [(5, 50), (3, 4100), (300, 64), (9, 1024)])
@pytest.mark.parametrize("second,depth", [(True, 3), (False, 0), (True, 0), (False, 9)])
def test_gated_add_with_and_without_the_norm_in_the_kernel(dtype, n, hidden, second, depth):
    """The gated add (one or two sublayers, with and without a history) alone and followed by the layer norm in the same kernel, against
    the formulas in float64; widths that are and are not whole 16-byte words; the rows option of the norm."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(n * hidden + depth)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    stream0, a, f = rnd(n, hidden), rnd(n, hidden).to(dtype), rnd(n, hidden).to(dtype) if second else None
    gates = rnd(n, 2 * hidden + 8).to(dtype)
    gate_bias, a_bias, w, b = rnd(2 * hidden), rnd(hidden), 1 + 0.1 * rnd(hidden), rnd(hidden)
    history0 = rnd(depth + 1, n, hidden) if depth else None
    mixw = rnd(depth + 1) if depth else None
    eps = 1e-5
    # the formulas
    x = stream0.double() + (a.double() + a_bias.double()) * torch.sigmoid(gates[:, :hidden].double() + gate_bias[:hidden].double())
    if second:
        x = x + f.double() * torch.sigmoid(gates[:, hidden:2 * hidden].double() + gate_bias[hidden:].double())
    new_stream = x
    if depth:
        new_stream = sum(mixw[j].double() * history0[j].double() for j in range(depth)) + mixw[depth].double() * x
    mean = new_stream.mean(-1, keepdim=True)
    want_h = (new_stream - mean) / torch.sqrt(((new_stream - mean) ** 2).mean(-1, keepdim=True) + eps) * w.double() + b.double()
    dev = lambda t: None if t is None else t.to(DEV)
    for fused in (False, True):
        stream, history = stream0.clone().to(DEV), dev(None if history0 is None else history0.clone())
        kw = dict(gates=dev(gates), gate_bias=dev(gate_bias), a_bias=dev(a_bias), history=history, index=depth, weights=dev(mixw))
        if fused:
            h = ops.gated_residual(stream, dev(a), dev(f), norm=(dev(w), dev(b), eps), out_dtype=dtype, **kw)
        else:
            assert ops.gated_residual(stream, dev(a), dev(f), **kw) is stream
            h = ops.stream_layer_norm(stream, dev(w), dev(b), eps, dtype)
            some = torch.tensor([n - 1, 0], dtype=torch.int32, device=DEV)
            assert torch.equal(ops.stream_layer_norm(stream, dev(w), dev(b), eps, dtype, rows=some), h[some.long()])
        assert (stream.cpu().double() - new_stream).abs().max() < 1e-4 * (1 + new_stream.abs().max()), f"stream, fused={fused}"
        if depth:
            assert (history[depth].cpu().double() - x).abs().max() < 1e-4 * (1 + x.abs().max()), f"history entry, fused={fused}"
            assert torch.equal(history[:depth].cpu(), history0[:depth]), "earlier history entries were touched"
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (h.cpu().double() - want_h).abs().max() < tol * (1 + want_h.abs().max()), f"norm output, fused={fused}"
