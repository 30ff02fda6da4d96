"""Tiny Pizunex configurations of the test-suite and their random weights.  They differ in every size and
option: width, vocabulary, eps, order of layers, heads and kv heads of all three mixers, key and value widths,
filter taps (one tap: no filter memory at all), windows smaller and larger than a page, the temperature's period
(1: it moves at every position), with and without cap, window, temperature and frequency blending, a rotation over
part of the rotated dimensions only, layers that borrow another layer's tensors, layers without feed-forward,
a model without any attention layer, page size."""

from __future__ import annotations

import json
import os

import numpy as np
import torch
from safetensors.torch import save_file

from turingserve_b200.models.pizunex import make_config
from turingserve_b200.weights.random_init import random_tensors


def _delta(heads, kv, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _attn(heads, kv, dim, scale, window=None, cap=None, temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if cap:
        m["softcap"] = cap
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": m}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims=None, scaling=None):
    rot = {"base": base, "dims": dims or rot_dim}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                                                  "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale, "rot": rot}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


# name -> (config arguments, seed, cache page size)
TINY = {
    # the recurrent mixer first, two query/key heads for four heads; a window shorter than a page with cap and a
    # temperature that moves every 5 positions; blended frequencies; two layers borrow tensors
    "A": (dict(width=64, vocab=131, eps=1e-5, layers=[
        {**_delta(4, 2, 16, 8, 3), "mlp": None},
        {**_attn(4, 2, 16, 0.3, window=9, cap=6.0, temp=(0.4, 5)), "mlp": _dense(72)},
        {**_latent(2, 8, 8, 12, 24, 20, 0.3, 100.0, scaling=(2.5, 16, 4.0, 1.0)), "mlp": _dense(40)},
        {**_delta(4, 2, 16, 8, 3), "mlp": None, "weights_of": 0},
        {**_latent(2, 8, 8, 12, 24, 20, 0.3, 100.0, scaling=(2.5, 16, 4.0, 1.0)), "mlp": _dense(40), "weights_of": 2},
    ]), 21, 16),
    # latent attention first, rotation over 4 of 6 rotated dimensions and no blending; a window wider than a page and
    # neither cap nor temperature; one query/key head for two heads, keys of 24 (no multiple of 16), two taps; a window
    # of 3 with the temperature moving at every position
    "B": (dict(width=96, vocab=257, eps=1e-6, layers=[
        {**_latent(3, 16, 6, 8, 16, 40, 0.2, 10000.0, dims=4), "mlp": None},
        {**_attn(6, 6, 8, 0.4, window=33), "mlp": _dense(120)},
        {**_delta(2, 1, 24, 20, 2), "mlp": _dense(56)},
        {**_attn(2, 1, 40, 0.15, window=3, cap=20.0, temp=(0.25, 1)), "mlp": None},
        {**_attn(6, 6, 8, 0.4, window=33), "mlp": _dense(120), "weights_of": 1},
    ]), 22, 8),
    # sizes in multiples of 16 and pages of 64: keys of 128 in the recurrent mixer (32 rows a lane), heads of 64, a
    # cached latent row of 80; attention without a window at all
    "C": (dict(width=128, vocab=300, eps=1e-6, layers=[
        {**_attn(4, 2, 64, 0.125, cap=30.0, temp=(0.3, 16)), "mlp": _dense(256)},
        {**_delta(2, 2, 128, 64, 4), "mlp": None},
        {**_latent(4, 32, 16, 32, 48, 64, 0.14, 50000.0, scaling=(4.0, 64, 16.0, 2.0)), "mlp": _dense(192)},
        {**_attn(4, 4, 32, 0.18, window=70), "mlp": None},
    ]), 23, 64),
    # no attention layer at all: the engine runs without a single cache group, on state slots alone; one tap (no
    # filter memory) and eight
    "D": (dict(width=32, vocab=50, eps=1e-5, layers=[
        {**_delta(2, 2, 8, 8, 1), "mlp": None},
        {**_delta(3, 1, 16, 4, 8), "mlp": _dense(40)},
    ]), 24, 16),
}

# how much larger than the base deviation a tensor's entries are (by the end of its name): queries and keys large
# enough for scores that tell keys apart, filters and gates of the recurrence away from their resting values
BOOST = {"mix.q": 4.0, "mix.k": 4.0, "mix.uq": 4.0, "mix.uk": 4.0, "mix.dkv": 3.0, "mix.dq": 3.0, ".conv": 8.0,
         "A_log": 15.0, "dt_bias": 15.0, "mix.a": 4.0, "mix.b": 6.0, "mix.g": 4.0, "embed": 10.0}


def tiny_config(name: str):
    return make_config(**TINY[name][0])


def page_size(name: str) -> int:
    return TINY[name][2]


def make_tiny_folder(name: str, base, std: float = 0.05) -> str:
    kw, seed, _ = TINY[name]
    folder = os.path.join(str(base), f"pizunex_{name}")
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
