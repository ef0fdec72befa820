"""Small Nidudra configurations and model folders for the tests: sizes unlike any real model's, values that differ where a coincidence
(heads == kv_heads, key size == value size, all entries rotated, top == 1, a window that covers everything) would hide a fault, and weights
reshaped so that faults show."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=6, top=2, shared=40):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def windowed(heads=4, kv_heads=2, dim=16, vdim=24, size=9, keep_first=3, scale=0.6, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size, "keep_first": keep_first}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def bands(factor=4.0, low=1.0, high=4.0, original=64):
    return {"factor": factor, "low": low, "high": high, "original": original}


def sinked(heads=4, kv_heads=2, dim=16, vdim=24, rot=12, base=100.0, scaling="default", scale=0.9, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = bands() if scaling == "default" else scaling
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def ramp(factor=6.0, original=32, fast=8.0, slow=1.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def paired(heads=4, kv_heads=2, dim=16, conv=3, rot=8, base=50.0, scaling="default", scale=0.5, r_heads=3, r_dim=12, r_vdim=20, tau=4.0, rank=5,
           mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "conv": conv}
    if rot:
        left["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            left["rot"]["scaling"] = ramp() if scaling == "default" else scaling
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau, "rank": rank}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def model_config(layers, width=48, vocab=131, eps=1e-5, softcap=12.0):
    return {"architecture": "Nidudra", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width, "logit_softcap": softcap}


# Whole models that differ in every size and option.
MODEL_A = model_config([windowed(mlp=dense()), sinked(mlp=moe()), paired(mlp=dense(ff=40)), windowed(kv_from=0, size=5, keep_first=1, mlp=moe(ff=16, experts=5, top=1)),
                        sinked(heads=2, kv_heads=2, dim=8, vdim=8, rot=8, scaling=None)])
MODEL_B = model_config([paired(heads=2, kv_heads=1, dim=32, conv=2, rot=32, base=1e4, scaling=ramp(factor=16.0, original=16, fast=4.0, slow=0.5), r_heads=1, r_dim=40,
                               r_vdim=8, tau=16.0, rank=3, mlp=moe(ff=8, experts=10, top=3, shared=8)),
                        windowed(heads=6, kv_heads=3, dim=32, vdim=32, size=20, keep_first=0, scale=0.3, mlp=dense(ff=72)),
                        windowed(heads=6, kv_heads=3, dim=32, vdim=32, size=7, keep_first=10, scale=0.3, kv_from=1),
                        sinked(heads=8, kv_heads=1, dim=32, vdim=16, rot=6, base=7.0, scaling=bands(factor=2.0, low=0.5, high=2.0, original=24), mlp=dense(ff=24)),
                        paired(heads=3, kv_heads=3, dim=48, conv=4, rot=0, r_heads=4, r_dim=70, r_vdim=33, tau=1.5, rank=9)],
                       width=64, vocab=200, eps=1e-6, softcap=5.0)
# every attention layer has sizes that the tensor-core kernels take in bfloat16 (keys and values of one size, a multiple of 16)
# and its only router stands in the last layer, where a choice that a rounding step turns over spoils one row and no later one
MODEL_C = model_config([windowed(heads=8, kv_heads=2, dim=64, vdim=64, size=33, keep_first=5, scale=0.2, mlp=dense(ff=48)),
                        sinked(heads=6, kv_heads=3, dim=32, vdim=32, rot=32, base=500.0, scale=0.5, mlp=dense(ff=32)),
                        paired(heads=4, kv_heads=1, dim=128, conv=5, rot=64, base=1e3, scale=0.1, r_heads=2, r_dim=64, r_vdim=64, tau=8.0, rank=8),
                        windowed(heads=8, kv_heads=2, dim=64, vdim=64, size=100, keep_first=70, scale=0.2, kv_from=0, mlp=dense(ff=40)),
                        windowed(heads=2, kv_heads=1, dim=48, vdim=48, size=17, keep_first=16, scale=0.25, mlp=moe(ff=32, experts=4, top=2, shared=16))],
                       width=56, vocab=150, eps=1e-5, softcap=30.0)


def make_folder(tmp: Path, config: dict, name: str, seed: int = 0, sharpen: float = 2.0, strength: float = 1.0) -> Path:
    """A model folder with random bfloat16 weights, then reshaped so that faults show: the q/k norm weights are scaled up for peaked attention
    (a lost, doubled or wrongly placed key changes the output), sinks get the size of the scores, biases and filters a visible size, the
    decay's bias keeps the state alive over many tokens, the routers' scores are spread out, gates and experts leave their linear stretch,
    the two sides' output weights differ. ``strength`` < 1 scales all of that down towards plain random weights, for 16-bit runs of deep
    models, where every factor here also multiplies what a rounding step does."""
    from safetensors.torch import load_file, save_file

    from oxr_inference_b200.weights import write_random_model

    def by(factor: float) -> float:
        return 1.0 + (factor - 1.0) * strength

    folder = write_random_model(config, tmp / name, seed, dtype="bfloat16", std=0.06)
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    for k, t in tensors.items():
        f = t.float()
        if k.endswith((".q.norm", ".k.norm")):
            f = f * by(sharpen) ** 0.5
        elif k.endswith(".mix.sink"):
            f = f * 30 + 1.0
        elif k.endswith((".q.b", ".k.b")):
            f = f * by(8)
        elif k.endswith(".conv"):
            f = f * 6 + 0.4
        elif k.endswith(".a2.b"):
            f = f * 10 + 2.5
        elif k.endswith((".a1", ".a2")):
            f = f * by(4)
        elif k.endswith("left.out"):
            f = f * 0.7
        elif k.endswith("right.out"):
            f = f * 1.4
        elif k.endswith((".router", ".shared.sg")):
            f = f * by(2)
        elif k.endswith((".gate", ".up")) and ".mlp." in k:
            f = f * by(4)
        elif k.endswith((".mix.g", ".right.g")):
            f = f * by(5)
        elif k.endswith(("head", "embed")):
            f = f * by(4)
        tensors[k] = f.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


def tokens(config: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed * 104729 + n)
    return torch.randint(0, config["vocab"], (n,), generator=g).tolist()


_cache: dict = {}


def plain_logits(folder: Path, ids: list[int]) -> torch.Tensor:
    from plain import nidudra_plain as NP

    key = (str(folder), tuple(ids))
    if key not in _cache:
        if str(folder) not in _cache:
            _cache[str(folder)] = NP.read_model(folder, torch.float64)
        cfg, w = _cache[str(folder)]
        margins: list = []
        _cache[key] = NP.forward(cfg, w, ids, margins=margins).float()
        _cache[("margin",) + key] = torch.stack(margins).min(0).values.float() if margins else torch.full((len(ids),), float("inf"))
    return _cache[key]


def router_margins(folder: Path, ids: list[int]) -> torch.Tensor:
    """Per position, the smallest margin by which any layer's router decided (``inf`` without routers)."""
    plain_logits(folder, ids)
    return _cache[("margin", str(folder), tuple(ids))]
