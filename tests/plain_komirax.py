"""A plain, slow Komirax decoder in PyTorch on the CPU: whole sequences, no cache, token by token where
the design has a recurrence, one function per mechanism.  It is the oracle of the Komirax tests and
shares no code with ``turingserve_b200``: it reads ``config.json`` as a dict and the checkpoint as a
dict of tensors by name.

The design, in this file's notation (x is the residual stream, one row a token):

* layer:      x += mixer(rms(x) * w1);  x += ff(rms(x) * w2)   (a layer may have no ff)
* lightning:  q, k, v = silu(Wq h), silu(Wk h), silu(Wv h), head by head;
              S_t = lam_h S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t;  heads side by side, one rms norm with a
              weight over all of them, times sigmoid(Wg h), then Wo
* attention:  two score maps a head (q and k rows come as [map 1 | map 2] for every head), both over the
              same values; causal softmax each; o = a1 - L a2 with L = exp(lq1.lk1) - exp(lq2.lk2) + diff;
              o / rms(o) over the head's values, times (1 - diff); then Wo.  No positions.
* ff dense:   Wdown gelu_tanh(Wup h)
* ff routed:  s = sigmoid(Wr h); the `top` largest; y = sum_e Wdown_e relu(Wup_e (s_e h))^2
* schedule:   layers before `start` once, layers start..stop-1 `times` times (each pass its own memory; every
              pass but the first begins by adding the embedding rows to x), then the rest once.
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


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def decayed_state_scan(q, k, v, lam: float, S=None):
    """One head, token by token: S <- lam S + k_t v_t^T, o_t = S^T q_t.  q, k [T, D], v [T, V]; returns
    (o [T, V], the state after the last token)."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype) if S is None else S.clone()
    out = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for t in range(T):
        S = lam * S + torch.outer(k[t], v[t])
        out[t] = S.t() @ q[t]
    return out, S


def lightning(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = F.silu(F.linear(h, w[p + "q"])).view(T, H, D)
    k = F.silu(F.linear(h, w[p + "k"])).view(T, H, D)
    v = F.silu(F.linear(h, w[p + "v"])).view(T, H, V)
    out = torch.stack([decayed_state_scan(q[:, a], k[:, a], v[:, a], float(m["decay"][a]))[0] for a in range(H)], dim=1)
    o = rms(out.reshape(T, H * V), eps) * w[p + "norm"]
    o = o * torch.sigmoid(F.linear(h, w[p + "g"]))
    return F.linear(o, w[p + "o"])


def two_map_head(q1, k1, q2, k2, v, scale: float, L: float, eps: float, out_scale: float, first_pos: int = 0):
    """One head: queries q1, q2 [Tq, D] at positions first_pos.., keys k1, k2 [Tk, D] and values [Tk, V] at
    positions 0..; causal softmax for each map, o = a1 - L a2, o / rms(o) * out_scale."""
    Tq, Tk = q1.shape[0], k1.shape[0]
    hidden = torch.arange(Tk)[None, :] > (torch.arange(Tq)[:, None] + first_pos)
    maps = []
    for q, k in ((q1, k1), (q2, k2)):
        s = ((q @ k.t()) * scale).masked_fill(hidden, float("-inf"))
        maps.append(torch.softmax(s, -1) @ v)
    return rms(maps[0] - L * maps[1], eps) * out_scale


def mixing_constant(w: dict, p: str, diff: float) -> float:
    return (math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum()))
            + diff)


def two_map_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """h [T, width] -> [T, width]; every head on its own."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.linear(h, w[p + "q"], w[p + "q.b"]).view(T, H, 2, D)
    k = F.linear(h, w[p + "k"], w[p + "k.b"]).view(T, G, 2, D)
    v = F.linear(h, w[p + "v"], w[p + "v.b"]).view(T, G, V)
    L = mixing_constant(w, p, m["diff"])
    per = H // G
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        g = a // per
        out[:, a] = two_map_head(q[:, a, 0], k[:, g, 0], q[:, a, 1], k[:, g, 1], v[:, g], m["scale"], L, eps,
                                 1.0 - m["diff"])
    return F.linear(out.reshape(T, H * V), w[p + "o"])


def dense_ff(h, w, p):
    return F.linear(gelu_tanh(F.linear(h, w[p + "up"])), w[p + "down"])


def route(h, router_w, top: int):
    """(experts [T, top], weights [T, top]): the largest sigmoid scores of every token, largest first."""
    s = torch.sigmoid(F.linear(h.float(), router_w.float()))
    best = s.topk(top, dim=-1)
    return best.indices, best.values


def routing_margin(h, router_w, top: int):
    """Per token, how far the last chosen expert's router logit lies above the first one left out (inf when
    every expert is chosen): a small margin is a close call that lower precision may decide the other way."""
    z = F.linear(h.float(), router_w.float()).sort(-1, descending=True).values
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else torch.full((h.shape[0],), float("inf"))


def routed_ff(h, w, p, ff: dict, margins: list | None = None):
    top = ff["router"]["top"]
    experts, weights = route(h, w[p + "router"], top)
    if margins is not None:
        margins.append(routing_margin(h, w[p + "router"], top))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for r in range(top):
            e, weight = int(experts[t, r]), weights[t, r].to(h.dtype)
            z = F.linear(weight * h[t], w[f"{p}e{e}.up"])
            out[t] += F.linear(torch.relu(z) ** 2, w[f"{p}e{e}.down"])
    return out


def order(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, whether this run opens a pass after the first) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for r in range(times):
        runs += [(i, r > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


@torch.inference_mode()
def forward(cfg: dict, w: dict, ids, return_streams: bool = False, margins: list | None = None):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run).  ``margins``: a list
    that receives every routed layer run's per-token routing margin."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(ids, dtype=torch.long)]
    x = x0.clone()
    streams = []
    for i, opens in order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if opens:
            x = x + x0
        hn = rms(x, eps) * w[p + "norm1"]
        mix = lightning if L["type"] == "lightning" else two_map_attention
        x = x + mix(hn, w, p + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            hn = rms(x, eps) * w[p + "norm2"]
            x = x + (dense_ff(hn, w, p + "mlp.") if L["mlp"]["kind"] == "dense" else routed_ff(hn, w, p + "mlp.", L["mlp"], margins))
        streams.append(x.clone())
    logits = F.linear(rms(x, eps) * w["final.norm"], w["head"])
    return (logits, torch.stack(streams)) if return_streams else logits


def greedy(cfg: dict, w: dict, prompt: list[int], max_new_tokens: int) -> list[int]:
    """Greedy continuation, the whole sequence run again for every token."""
    ids, out = list(prompt), []
    for _ in range(max_new_tokens):
        out.append(int(forward(cfg, w, ids)[-1].argmax()))
        ids.append(out[-1])
    return out
