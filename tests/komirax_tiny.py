"""Tiny Komirax configurations of the test-suite and their random weights.  They differ in every size
and option: width, vocabulary, eps, order of layers, heads and kv heads, widths of maps and values
(equal, wider, narrower), decays, experts and how many a token uses (one, some, all), layers without a
feed-forward, the looped span (none, one layer, several, from layer 0, several passes), page size."""

from __future__ import annotations

import json
import os

import numpy as np
import torch
from safetensors.torch import save_file

from turingserve_b200.models.komirax import make_config
from turingserve_b200.weights.random_init import random_tensors


def _light(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def _attn(heads, kv, dim, vdim, diff, scale):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff,
                                           "scale": scale}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


# name -> (config arguments, seed, cache page size)
TINY = {
    # attention first, kv heads shared by two query heads, values wider than a map, two of five experts, the
    # first two layers three times, a layer that is only a mixer
    "P": (dict(width=64, vocab=131, eps=1e-5, loop={"start": 0, "stop": 2, "times": 3}, layers=[
        {**_attn(4, 2, 16, 24, 0.3, 0.25), "mlp": _moe(5, 2, 40)},
        {**_light(2, 16, 32, [0.9, 0.99]), "mlp": _dense(72)},
        {**_light(3, 8, 16, [0.5, 0.97, 1.0]), "mlp": None},
        {**_attn(2, 1, 24, 16, 0.8, 0.2), "mlp": _dense(56)},
    ]), 11, 16),
    # no loop at all; all three experts used by every token; values narrower than keys in the linear layer and
    # five times a map's width in the attention layer; as many kv heads as heads
    "Q": (dict(width=96, vocab=257, eps=1e-6, layers=[
        {**_light(4, 32, 16, [0.8, 0.95, 0.99, 0.999]), "mlp": _moe(3, 3, 32)},
        {**_attn(6, 6, 8, 40, 0.5, 0.35), "mlp": None},
        {**_light(1, 48, 48, [0.93]), "mlp": _dense(120)},
    ]), 12, 8),
    # one looped layer in the middle, twice; one of two experts; one head
    "R": (dict(width=48, vocab=97, eps=3e-6, loop={"start": 1, "stop": 2, "times": 2}, layers=[
        {**_light(2, 24, 8, [0.7, 0.98]), "mlp": _dense(64)},
        {**_attn(1, 1, 32, 32, 0.1, 0.18), "mlp": _moe(2, 1, 24)},
        {**_attn(3, 3, 16, 32, 0.6, 0.25), "mlp": _dense(40)},
    ]), 13, 32),
    # sizes the tensor-core kernels take: maps and values in multiples of 16, pages of 64; four of eight experts
    "S": (dict(width=128, vocab=300, eps=1e-6, loop={"start": 1, "stop": 3, "times": 2}, layers=[
        {**_light(2, 64, 64, [0.9, 0.995]), "mlp": _dense(256)},
        {**_attn(4, 2, 64, 128, 0.7, 0.125), "mlp": _moe(8, 4, 64)},
        {**_light(2, 128, 64, [0.97, 0.999]), "mlp": _moe(8, 2, 128)},
        {**_attn(2, 2, 32, 64, 0.4, 0.18), "mlp": None},
    ]), 14, 64),
    # no attention layer at all: the engine runs without a single cache group, on state slots alone
    "Z": (dict(width=32, vocab=50, eps=1e-5, layers=[
        {**_light(2, 8, 8, [0.9, 0.95]), "mlp": None},
        {**_light(1, 16, 8, [0.99]), "mlp": _dense(40)},
    ]), 15, 16),
}

# how much larger than the base deviation a tensor's entries are (by the end of its name): queries and keys
# large enough for scores that tell keys apart, routers for scores that tell experts apart
BOOST = {".q": 4.0, ".k": 4.0, ".router": 6.0, ".q.b": 3.0, ".k.b": 3.0, ".v.b": 3.0, ".lq1": 20.0, ".lk1": 20.0,
         ".lq2": 20.0, ".lk2": 20.0, "embed": 10.0}


def tiny_config(name: str):
    return make_config(**TINY[name][0])


def page_size(name: str) -> int:
    return TINY[name][2]


def make_tiny_folder(name: str, base, std: float = 0.05) -> str:
    kw, seed, _ = TINY[name]
    folder = os.path.join(str(base), f"komirax_{name}")
    if os.path.exists(os.path.join(folder, "model.safetensors")):
        return folder
    cfg = make_config(**kw)
    from turingserve_b200.config.registry import get_architecture
    tensors = random_tensors(cfg, seed, std)
    g = torch.Generator().manual_seed(seed + 1000)
    for n, t in tensors.items():
        if "norm" in n:                              # scales around one, not all equal
            tensors[n] = (1.0 + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        for end, f in BOOST.items():
            if n.endswith(end):
                tensors[n] = (t.float() * f).to(t.dtype)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(get_architecture(cfg.architecture).to_config_json(cfg), f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
