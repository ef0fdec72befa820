"""A plain, slow statement of the Vazepel decoder: one function per mechanism, whole sequences at once, no cache.

Shares no code with the engine. Everything runs on the host in one floating-point type (float64 by default), so it is the
yardstick for both the 16-bit and the 32-bit engine. The network: a token embedding; a list of layers in which ONE layer norm
feeds the mixer and the feed-forward side by side, each result passes a learned sigmoid gate before it joins the stream, and
what a layer hands on is a learned weighted sum of the embedding's output and every layer result so far; a final layer norm;
an output head. The mixer is grouped-query attention with biases, a rotation of entry pairs, capped scores that are mixed
between the heads before the softmax, a softmax whose denominator holds an extra one, and a sigmoid gate on the heads'
output. The feed-forward is a tanh-GELU layer or a set of routed experts beside a shared one.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open

GATE_SLOPE = 1.702


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
def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [T, heads, D]; entries (2i, 2i+1) for 2i < dims turn by the angle p * base^(-2i/dims) at position p; the rest stay."""
    T = x.shape[0]
    out = x.clone()
    pos = torch.arange(T, dtype=torch.float64)
    for i in range(dims // 2):
        a = pos * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a).to(x.dtype)[:, None], torch.sin(a).to(x.dtype)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def clamped_unit(h: torch.Tensor, w: dict, p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ w[p + "down"].T


# ------------------------------------------------------------------------------------------------ the mixer
def mixed_head_attention(h: torch.Tensor, w: dict, p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, DV)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, rot["dims"], rot["base"])
        k = rotate_pairs(k, rot["dims"], rot["base"])
    per = H // G
    k_of = k[:, [a // per for a in range(H)]]          # [T, H, D]
    v_of = v[:, [a // per for a in range(H)]]
    s = torch.einsum("ihd,jhd->hij", q, k_of) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    s = torch.einsum("hg,gij->hij", w[p + "talk"], s)   # every head's score becomes a mixture of all heads' scores
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    s = s.masked_fill(~seen[None], float("-inf"))
    e = torch.exp(s)                                    # scores are capped and mixed: no overflow to guard against here
    pr = e / (1.0 + e.sum(-1, keepdim=True))            # the extra one: a place with score 0 that holds no value
    o = torch.einsum("hij,jhd->ihd", pr, v_of).reshape(T, H * DV)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T + w[p + "o.b"]


# ------------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def choose_experts(z: torch.Tensor, top: int, count: int, keep: int):
    """z: [T, E] router logits. Returns (ids [T, top], weights [T, top], margin [T]); the weights are the softmax scores themselves."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    allowed = torch.ones(T, E, dtype=torch.bool)
    margin = torch.full((T,), float("inf"), dtype=z.dtype)
    if count > 1 and keep < count:
        per = E // count
        gs = s.view(T, count, per).max(-1).values
        order = gs.argsort(dim=-1, descending=True, stable=True)
        kept = torch.zeros(T, count, dtype=torch.bool)
        kept.scatter_(1, order[:, :keep], True)
        allowed = kept.repeat_interleave(per, dim=1)
        sorted_gs = gs.gather(1, order)
        margin = torch.minimum(margin, sorted_gs[:, keep - 1] - sorted_gs[:, keep])
    masked = s.masked_fill(~allowed, -1.0)
    order = masked.argsort(dim=-1, descending=True, stable=True)
    ids = order[:, :top]
    sm = masked.gather(1, order)
    if top < E:
        nxt = sm[:, top]
        margin = torch.minimum(margin, torch.where(nxt >= 0, sm[:, top - 1] - nxt, torch.full_like(nxt, float("inf"))))
    return ids, s.gather(1, ids), margin


def routed_ff(h: torch.Tensor, w: dict, p: str, mlp: dict, margins: list | None = None) -> torch.Tensor:
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = h.to(torch.float32).to(h.dtype) @ w[p + "router"].T
    ids, wts, margin = choose_experts(z, r["top"], groups["count"], groups["keep"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wts[t]):
            out[t] += a * clamped_unit(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_unit(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------------------------ the whole network
def forward(cfg: dict, w: dict, ids: list[int], layers_out: list | None = None, margins: list | None = None) -> torch.Tensor:
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)]
    results = [x]                                       # the embedding's output, then every layer's result
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        a = mixed_head_attention(h, w, p + "mix.", layer["mixer"])
        a = a * torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
        y = x + a
        mlp = layer.get("mlp")
        if mlp is not None:
            f = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp, margins)
            y = y + f * torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
        results.append(y)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["head"].T


def greedy(cfg: dict, w: dict, prompt: list[int], n: int) -> tuple[list[int], list[float]]:
    """``n`` greedy tokens after ``prompt``, and for each the gap between the two largest logits over the logits' spread (a near-tie
    may fall either way under another rounding)."""
    ids, gaps = list(prompt), []
    for _ in range(n):
        row = forward(cfg, w, ids)[-1]
        best = row.topk(2).values
        gaps.append(float((best[0] - best[1]) / row.std()))
        ids.append(int(row.argmax()))
    return ids[len(prompt):], gaps
