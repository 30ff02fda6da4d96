"""A plain, slow Pizunex decoder in PyTorch on the CPU: whole sequences, no cache, token by token where the
design has a recurrence, one function per mechanism.  It is the oracle of the Pizunex tests and shares no
code with ``turingserve_b200``: it reads ``config.json`` as a dict and the checkpoint as a dict of tensors
by name.

The design, in this file's notation (x is the residual stream, one row a token, p a token's position):

* layer:     x += mixer(rms(x) * w1);  x += ff(rms(x) * w2)   (a layer may have no ff; a layer may borrow
             another layer's tensors and still keeps memory of its own)
* delta:     q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h)), conv a causal filter of a few
             taps per channel; q, k to unit length per head, q / sqrt(dim); b = sigmoid(Wb h);
             g = exp(-exp(A) softplus(Wa h + dt)); head by head the memory M fades, is corrected and read:
             M <- g M; e = b (v - M^T k); M <- M + k e^T; y = M^T q; y / rms(y) * w_norm * silu(Wg h); Wo
* attention: q = Wq h, k = Wk h, values = k; q and k normed over the WHOLE row (all heads at once) with a
             weight; q *= 1 + c ln(floor((p+1)/every) + 1); s = cap tanh(q.k scale / cap) - m_h (i - j), with
             the slopes m_h = 2^(-8 (h+1) / H) for h = 0 .. H-1; keys i - w < j <= i; softmax; Wo
* latent:    cq = rms(Wdq h) * w; q = Wuq cq, per head [plain | rotated]; Wdkv h = [c_raw | kr];
             c = rms(c_raw) * w; per head k = [Wuk c | rot(kr)], v = Wuv c; causal softmax of q.k scale; Wo.
             rot: interleaved pairs, YaRN-blended frequencies, cos and sin times 0.1 ln(factor) + 1
* ff:        Wdown relu(Wup h)^2
"""

from __future__ import annotations

import json
import math
import os

import torch
import torch.nn.functional as F
from safetensors.torch import load_file


def read_folder(folder: str, dtype=torch.float32):
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return cfg, {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in tensors.items()}


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


# ---------------------------------------------------------------------------------------------- delta rule
def short_filter(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n] (last column multiplies the present token): y_t = sum_i taps[:, i] x_(t-n+1+i),
    zeros before the sequence."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for i in range(n):
        y = y + padded[i:i + T] * taps[:, i]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_scan(q, k, v, g, b, S=None):
    """One head, token by token.  q, k [T, D], v [T, V], g, b [T]; returns (o [T, V], last state)."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype) if S is None else S.clone()
    out = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for t in range(T):
        S = g[t] * S
        u = b[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.t() @ q[t]
    return out, S


def delta(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit(F.silu(short_filter(F.linear(h, w[p + "q"]), w[p + "q.conv"])).view(T, G, D)) * D ** -0.5
    k = unit(F.silu(short_filter(F.linear(h, w[p + "k"]), w[p + "k.conv"])).view(T, G, D))
    v = F.silu(short_filter(F.linear(h, w[p + "v"]), w[p + "v.conv"])).view(T, H, V)
    b = torch.sigmoid(F.linear(h, w[p + "b"]))
    g = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(F.linear(h, w[p + "a"]) + w[p + "dt_bias"]))
    per = H // G
    o = torch.stack([delta_scan(q[:, a // per], k[:, a // per], v[:, a], g[:, a], b[:, a])[0] for a in range(H)], 1)
    o = rms(o, eps) * w[p + "norm"] * F.silu(F.linear(h, w[p + "g"])).view(T, H, V)
    return F.linear(o.reshape(T, H * V), w[p + "o"])


# ---------------------------------------------------------------------------------- attention with a window
def slopes(H: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)])


def query_heat(pos: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    return 1.0 + coef * torch.log(torch.floor((pos + 1) / every) + 1.0)


def capped_scores(q, k, scale: float, cap: float | None, slope: float, window: int | None, first_pos: int = 0):
    """q [Tq, D] at positions first_pos.., k [Tk, D] at positions 0..: masked scores before the softmax."""
    Tq, Tk = q.shape[0], k.shape[0]
    i = torch.arange(Tq)[:, None] + first_pos
    j = torch.arange(Tk)[None, :]
    s = (q @ k.t()) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    s = s - slope * (i - j).to(s.dtype)
    hidden = j > i
    if window:
        hidden = hidden | (i - j >= window)
    return s.masked_fill(hidden, float("-inf"))


def window_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q_raw, k_raw = F.linear(h, w[p + "q"]), F.linear(h, w[p + "k"])
    q = rms(q_raw, eps) * w[p + "q.norm"]
    k = (rms(k_raw, eps) * w[p + "k.norm"]).view(T, G, D)
    v = k_raw.view(T, G, D)
    if m.get("q_temp"):
        q = q * query_heat(torch.arange(T, dtype=h.dtype), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None]
    q = q.view(T, H, D)
    sl = slopes(H)
    win = (m.get("mask") or {}).get("size")
    outs = []
    for a in range(H):
        s = capped_scores(q[:, a], k[:, a // (H // G)], m["scale"], m.get("softcap"), float(sl[a]), win)
        outs.append(torch.softmax(s, -1) @ v[:, a // (H // G)])
    return F.linear(torch.cat(outs, -1), w[p + "o"])


# --------------------------------------------------------------------------------------- latent attention
def yarn_angles(rot: dict, positions: torch.Tensor):
    """(cos, sin) [T, dims / 2] of the rotation, with the blended frequencies and the magnitude factor."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        def pair_at(turns):
            return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        begin = max(math.floor(pair_at(sc["fast"])), 0)
        end = min(math.ceil(pair_at(sc["slow"])), dims - 1)
        t = ((i - begin) / max(end - begin, 0.001)).clamp(0, 1)
        f = (1 - t) * f + t * (f / sc["factor"])
        mag = 1.0 + 0.1 * math.log(sc["factor"])
    a = positions.to(torch.float64)[:, None] * f[None, :]
    return torch.cos(a) * mag, torch.sin(a) * mag


def rotate_pairs(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, ..., R]: the first 2 * cos.shape[1] dims in pairs (2i, 2i+1); cos, sin [T, dims/2]."""
    n = cos.shape[1]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n]
    c, s = cos.view(shape).to(x.dtype), sin.view(shape).to(x.dtype)
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


def latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(F.linear(h, w[p + "dq"]), eps) * w[p + "dq.norm"]
    q = F.linear(cq, w[p + "uq"]).view(T, H, D + R)
    both = F.linear(h, w[p + "dkv"])
    c = rms(both[:, :rank], eps) * w[p + "dkv.norm"]
    cos, sin = yarn_angles(m["rot"], torch.arange(T))
    kr = rotate_pairs(both[:, rank:], cos, sin)
    qr = rotate_pairs(q[..., D:], cos, sin)
    ku = F.linear(c, w[p + "uk"]).view(T, H, D)
    v = F.linear(c, w[p + "uv"]).view(T, H, V)
    hidden = torch.arange(T)[None, :] > torch.arange(T)[:, None]
    outs = []
    for a in range(H):
        s = (q[:, a, :D] @ ku[:, a].t() + qr[:, a] @ kr.t()) * m["scale"]
        outs.append(torch.softmax(s.masked_fill(hidden, float("-inf")), -1) @ v[:, a])
    return F.linear(torch.cat(outs, -1), w[p + "o"])


# ---------------------------------------------------------------------------------------------- the rest
def dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    return F.linear(F.relu(F.linear(h, w[p + "up"])) ** 2, w[p + "down"])


MIXERS = {"delta": delta, "attention": window_attention, "latent_attention": latent_attention}


def forward(cfg: dict, w: dict, tokens, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``streams``: receives x after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."
        x = x + MIXERS[layer["type"]](rms(x, eps) * w[p + "norm1"], w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + dense_ff(rms(x, eps) * w[p + "norm2"], w, p + "mlp.")
        if streams is not None:
            streams.append(x.clone())
    return F.linear(rms(x, eps) * w["final.norm"], w["head"])
