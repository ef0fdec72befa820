"""A plain, slow statement of the Nidudra decoder: one function per mechanism, whole sequences at once, no cache.

Shares no code with the engine. Everything runs on the host in one floating-point type (float64 by default), so it is the
yardstick for both the 16-bit and the 32-bit engine. The network: a token embedding; a list of layers, each ``x += norm1(mixer(x))``
and then ``x += norm2(ff(x))`` with the sublayers reading the stream itself and RMS norms on their OUTPUTS only; a final RMS norm; an
output head whose logits are capped by a tanh. Three mixers: windowed attention that also keeps a sequence's first tokens in sight (q/k
norm with weights, no rotation, a gate per channel, optionally reading another layer's keys and values); causal attention with a partial
half-split rotation whose frequencies are rescaled in three bands, unit-norm q and k, a per-head sink and a gate per head; and a pair of
mixers side by side, causal attention behind a short causal filter (values = filtered keys) with ramp-rescaled rotation next to gated
linear attention with a decay per key channel, whose normed outputs are averaged. Feed-forwards: a SiLU-gated layer, or routed experts that
scale their INPUT by the router's score beside a gated shared expert.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


def read_model(folder: str | Path, dtype: torch.dtype = torch.float64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():  # noqa: SIM118
            t = f.get_tensor(name)
            w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


# ------------------------------------------------------------------------------------------------ small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def heads_of(x: torch.Tensor, n: int) -> torch.Tensor:
    return x.reshape(x.shape[0], n, -1)


# ------------------------------------------------------------------------------------------------ rotation
def plain_frequencies(dims: int, base: float) -> list[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def banded_frequencies(dims: int, base: float, s: dict) -> list[float]:
    """Three bands by wavelength: short waves keep their frequency, long ones are slowed by ``factor``, a linear blend between."""
    factor, low, high, original = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
    out = []
    for f in plain_frequencies(dims, base):
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out.append(f)
        elif wave > original / low:
            out.append(f / factor)
        else:
            t = (original / wave - low) / (high - low)
            out.append((1.0 - t) * f / factor + t * f)
    return out


def ramp_frequencies(dims: int, base: float, s: dict) -> tuple[list[float], float]:
    """A ramp over the pair index between the pairs that turn ``fast`` and ``slow`` times within ``original`` positions; returns the
    frequencies and the factor on cos and sin."""
    factor, original, fast, slow = float(s["factor"]), float(s["original"]), float(s["fast"]), float(s["slow"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, freqs: list[float], magnitude: float = 1.0) -> torch.Tensor:
    """x: [T, heads, D]. With n = len(freqs), entry i < n is paired with entry i + n; the pair turns by position * freqs[i] and is
    multiplied by ``magnitude``; entries from 2n on stay."""
    T, n = x.shape[0], len(freqs)
    out = x.clone()
    pos = torch.arange(T, dtype=torch.float64)
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = (torch.cos(a) * magnitude).to(x.dtype)[:, None], (torch.sin(a) * magnitude).to(x.dtype)[:, None]
        u, v = x[:, :, i], x[:, :, i + n]
        out[:, :, i] = u * c - v * s
        out[:, :, i + n] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ softmax attention
def visible(T: int, window: int = 0, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: query i sees key j <= i; with a window only if i - j < window or j < keep_first."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window > 0:
        seen = seen & ((i - j < window) | (j < keep_first))
    return seen


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, seen: torch.Tensor,
                      sink: torch.Tensor | None = None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, DV] -> [T, H, DV]; head h reads key/value head h // (H / G). ``sink`` [H]: exp(sink) joins
    the denominator and nothing else."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def causal_filter(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, n]: y_t = sum_j taps[:, j] * u_(t - n + 1 + j), zeros before the sequence."""
    T, n = u.shape[0], taps.shape[1]
    y = torch.zeros_like(u)
    for j in range(n):
        back = n - 1 - j
        if back < T:
            y[back:] += taps[:, j] * u[:T - back]
    return y


# ------------------------------------------------------------------------------------------------ the three mixers
def windowed_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, borrowed=None):
    """Returns (output, (keys, values)) so that a later layer can borrow this layer's keys and values."""
    H, G = m["heads"], m["kv_heads"]
    q = rms(heads_of(h @ w[p + "q"].T, H), eps) * w[p + "q.norm"]
    if borrowed is None:
        k = rms(heads_of(h @ w[p + "k"].T, G), eps) * w[p + "k.norm"]
        v = heads_of(h @ w[p + "v"].T, G)
    else:
        k, v = borrowed
    seen = visible(h.shape[0], m["mask"]["size"], m["mask"]["keep_first"])
    o = softmax_attention(q, k, v, m["scale"], seen).reshape(h.shape[0], -1)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, (k, v)


def sink_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    H, G = m["heads"], m["kv_heads"]
    q, k, v = heads_of(h @ w[p + "q"].T, H), heads_of(h @ w[p + "k"].T, G), heads_of(h @ w[p + "v"].T, G)
    rot = m.get("rot")
    if rot:
        freqs = banded_frequencies(rot["dims"], rot["base"], rot["scaling"]) if rot.get("scaling") else plain_frequencies(rot["dims"], rot["base"])
        q, k = rotate_halves(q, freqs), rotate_halves(k, freqs)
    q, k = rms(q, eps), rms(k, eps)
    o = softmax_attention(q, k, v, m["scale"], visible(h.shape[0]), sink=w[p + "sink"])
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(h.shape[0], -1) @ w[p + "o"].T


def filtered_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The left side of the pair: biased q and k behind a causal filter, values = filtered keys, then norm and rotation."""
    H, G = m["heads"], m["kv_heads"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    if m.get("conv"):
        q, k = causal_filter(q, w[p + "q.conv"]), causal_filter(k, w[p + "k.conv"])
    v = heads_of(k, G)
    q = rms(heads_of(q, H), eps) * w[p + "q.norm"]
    k = rms(heads_of(k, G), eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        if rot.get("scaling"):
            freqs, mag = ramp_frequencies(rot["dims"], rot["base"], rot["scaling"])
        else:
            freqs, mag = plain_frequencies(rot["dims"], rot["base"]), 1.0
        q, k = rotate_halves(q, freqs, mag), rotate_halves(k, freqs, mag)
    o = softmax_attention(q, k, v, m["scale"], visible(h.shape[0]))
    return o.reshape(h.shape[0], -1) @ w[p + "o"].T


def decayed_linear_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The right side: per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    H, D, DV, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = heads_of(h @ w[p + "q"].T, H) * D ** -0.5
    k = heads_of(h @ w[p + "k"].T, H)
    v = heads_of(h @ w[p + "v"].T, H)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = heads_of(torch.sigmoid(z) ** (1.0 / tau), H)
    S = torch.zeros(H, D, DV, dtype=h.dtype)
    o = torch.zeros(T, H, DV, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = (rms(o, eps) * w[p + "norm"]).reshape(T, -1)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def side_by_side(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    left = filtered_attention(h, w, p + "left.", m["left"], eps)
    right = decayed_linear_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


# ------------------------------------------------------------------------------------------------ feed-forwards
def gated_unit(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def router_scores(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return torch.sigmoid(h @ w[p + "router"].T)


def choose(scores: torch.Tensor, top: int) -> torch.Tensor:
    return torch.topk(scores, top, dim=-1).indices


def choice_margin(scores: torch.Tensor, top: int) -> torch.Tensor:
    """How far the last chosen score is above the best one not chosen (inf when all are chosen)."""
    s = torch.sort(scores, dim=-1, descending=True).values
    if top >= s.shape[1]:
        return torch.full((s.shape[0],), math.inf, dtype=scores.dtype)
    return s[:, top - 1] - s[:, top]


def routed_experts(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    top = mlp["router"]["top"]
    s = router_scores(h, w, p)
    ids = choose(s, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in ids[t].tolist():
            out[t] += gated_unit((s[t, e] * h[t])[None], w, f"{p}e{e}.")[0]      # the score scales the expert's INPUT
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_unit(h, w, p + "shared.")
    return out


def feed_forward(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_unit(h, w, p)
    if mlp["kind"] == "moe":
        return routed_experts(h, w, p, mlp)
    raise ValueError(mlp["kind"])


# ------------------------------------------------------------------------------------------------ the model
def forward(cfg: dict, w: dict, tokens: list[int], streams: list | None = None, margins: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. ``streams`` collects the stream after every layer, ``margins`` the routers' margins."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    kept: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            a, kv = windowed_attention(x, w, p, m, eps, kept[src] if src is not None else None)
            kept[i] = kv
        elif layer["type"] == "attention_2":
            a = sink_attention(x, w, p, m, eps)
        elif layer["type"] == "parallel":
            a = side_by_side(x, w, p, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms(a, eps) * w[f"l{i}.norm1"]
        if layer.get("mlp") is not None:
            if margins is not None and layer["mlp"]["kind"] == "moe":
                margins.append(choice_margin(router_scores(x, w, f"l{i}.mlp."), layer["mlp"]["router"]["top"]))
            x = x + rms(feed_forward(x, w, f"l{i}.mlp.", layer["mlp"]), eps) * w[f"l{i}.norm2"]
        if streams is not None:
            streams.append(x.clone())
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def greedy(cfg: dict, w: dict, prompt: list[int], n: int) -> tuple[list[int], list[float]]:
    """``n`` greedy tokens after ``prompt`` and, for each, how far its logit stood above the runner-up's."""
    tokens, gaps = list(prompt), []
    for _ in range(n):
        last = forward(cfg, w, tokens)[-1]
        best = torch.topk(last, 2).values
        gaps.append(float(best[0] - best[1]))
        tokens.append(int(last.argmax()))
    return tokens[len(prompt):], gaps
