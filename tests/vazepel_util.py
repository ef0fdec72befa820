"""Small Vazepel configurations and model folders for the tests: sizes unlike any real model's, values that differ where a coincidence
(heads == kv_heads, key size == value size, all entries rotated, one group, top == 1) would hide a fault, and weights reshaped so that
faults show."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def moe(ff=24, experts=6, top=2, count=3, keep=2, limit=1.1, shared=40, shared_limit=0.8):
    router = {"experts": experts, "top": top}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared:
        out["shared"] = {"ff": shared, "limit": shared_limit}
    return out


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def layer(heads=4, kv_heads=2, dim=16, vdim=24, rot=12, base=100.0, scale=0.3, softcap=6.0, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def model_config(layers, width=48, vocab=131, eps=1e-5):
    return {"architecture": "Vazepel", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


# Three whole models that differ in every size and option.
MODEL_P = model_config([layer(mlp=moe()), layer(heads=2, kv_heads=2, dim=8, vdim=8, rot=8, softcap=2.5, mlp=dense()),
                        layer(heads=6, kv_heads=2, dim=32, vdim=16, rot=20, base=10000.0, scale=0.17),
                        layer(heads=3, kv_heads=1, dim=16, vdim=32, rot=0, mlp=moe(ff=16, experts=8, top=3, count=4, keep=3, shared=0))])
MODEL_Q = model_config([layer(heads=4, kv_heads=1, dim=64, vdim=64, rot=64, base=1e6, scale=0.11, softcap=30.0, mlp=dense(ff=72)),
                        layer(heads=8, kv_heads=4, dim=32, vdim=32, rot=16, scale=0.2, mlp=moe(ff=8, experts=10, top=3, count=10, keep=5, limit=0.5, shared=8, shared_limit=3.0)),
                        layer(heads=2, kv_heads=1, dim=48, vdim=80, rot=48, scale=0.15, softcap=1.5, mlp=dense(ff=24))],
                       width=64, vocab=200, eps=1e-6)
MODEL_R = model_config([layer(heads=5, kv_heads=5, dim=24, vdim=8, rot=2, scale=0.25, softcap=4.0, mlp=moe(ff=32, experts=9, top=2, count=3, keep=1, shared=16)),
                        layer(heads=1, kv_heads=1, dim=70, vdim=40, rot=34, base=50.0, scale=0.12, softcap=9.0, mlp=moe(ff=12, experts=5, top=5, count=1, keep=1))],
                       width=40, vocab=97)
# Every layer has key and value sizes that the tensor-core attention kernel takes in bfloat16, with 4, 1, 16 and 2 query heads per key/value
# head (6 heads: the mixing matrix is padded), key sizes unlike value sizes, few and all entries rotated.
MODEL_T = model_config([layer(heads=8, kv_heads=2, dim=64, vdim=128, rot=40, scale=0.14, softcap=20.0, mlp=dense(ff=40)),
                        layer(heads=2, kv_heads=2, dim=128, vdim=64, rot=128, base=5000.0, scale=0.1, softcap=3.0, mlp=moe(ff=16, experts=4, top=2, count=2, keep=1, shared=24)),
                        layer(heads=16, kv_heads=1, dim=64, vdim=64, rot=6, scale=0.13, softcap=8.0),
                        layer(heads=6, kv_heads=3, dim=64, vdim=64, rot=64, scale=0.12, softcap=50.0, mlp=dense(ff=32))],
                       width=56, vocab=150, eps=1e-5)


def make_folder(tmp: Path, config: dict, name: str, seed: int = 0, sharpen: float = 8.0) -> Path:
    """A model folder with random bfloat16 weights, then reshaped so that faults show: query and key weights are scaled up (peaked
    attention: a lost, doubled or wrongly placed key changes the output), the head-mixing matrix is the identity plus sizeable
    off-diagonal entries of both signs, the depth weights are of the size of one over their count with both signs, biases get a visible
    size, the routers' scores are spread out, expert inputs are large enough that the clamps cut."""
    from safetensors.torch import load_file, save_file

    from oxr_inference_b200.weights import write_random_model

    folder = write_random_model(config, tmp / name, seed, dtype="bfloat16", std=0.06)
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    for k, t in tensors.items():
        f = t.float()
        if k.endswith((".mix.q", ".mix.k")):
            f = f * sharpen ** 0.5
        elif k.endswith(".talk"):
            f = torch.eye(f.shape[0]) * 0.8 + f * 5
        elif k.endswith(".dwa"):
            f = (1.2 + f * 6) / f.numel() ** 0.5
        elif k.endswith((".q.b", ".k.b", ".v.b", ".o.b", ".rg1.b", ".rg2.b")) or (k.endswith(".b") and "norm" in k):
            f = f * 5
        elif k.endswith((".rg1", ".rg2")):
            f = f * 4
        elif k.endswith(".router"):
            f = f * 6
        elif k.endswith((".gate", ".up")) and ".mlp." in k:
            f = f * 5
        elif k.endswith(("head", "embed")):
            f = f * 4
        tensors[k] = f.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


def tokens(config: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed * 104729 + n)
    return torch.randint(0, config["vocab"], (n,), generator=g).tolist()


_cache: dict = {}


def plain_logits(folder: Path, ids: list[int]) -> torch.Tensor:
    from plain import vazepel_plain as VP

    key = (str(folder), tuple(ids))
    if key not in _cache:
        if str(folder) not in _cache:
            _cache[str(folder)] = VP.read_model(folder, torch.float64)
        cfg, w = _cache[str(folder)]
        margins: list = []
        _cache[key] = VP.forward(cfg, w, ids, margins=margins).float()
        _cache[("margin",) + key] = torch.stack(margins).min(0).values.float() if margins else torch.full((len(ids),), float("inf"))
    return _cache[key]


def router_margins(folder: Path, ids: list[int]) -> torch.Tensor:
    """Per position, the smallest margin by which any layer's router decided (``inf`` without routers)."""
    plain_logits(folder, ids)
    return _cache[("margin", str(folder), tuple(ids))]
