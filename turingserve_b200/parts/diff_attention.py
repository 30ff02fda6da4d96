"""Differential attention over the paged cache: two causal softmax maps a head over the same values.

One fused projection gives, per token, H x [q map 1 | q map 2], G x [k map 1 | k map 2] and G x v
(+ biases).  The new key rows (2 key_dim wide) and value rows (value_dim wide) go to the cache first,
then every query attends from the cache, so a prompt portion and a single decoded token take one path.
o = a1 - lam a2 with lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (one number a layer, from four learned
vectors, computed once when the weights arrive); each head's o is divided by its root mean square
(no learned scale) and multiplied by 1 - diff; then the output projection.  Positions do not enter.
"""

from __future__ import annotations

import math

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, CacheNeed, Mixer, ParamSpec, register


class DiffAttention(Mixer):
    MAX_DIM = 256               # the any-size kernel's limit on a map's width and on the value width

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.G = int(spec.num_heads), int(spec.num_kv_heads)
        self.D, self.V = int(spec.key_dim), int(spec.value_dim)
        if self.G < 1 or self.H % self.G:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not (0 < self.D <= self.MAX_DIM and 0 < self.V <= self.MAX_DIM):
            raise ValueError(f"diff_attention: maps of {self.D}, values of {self.V}: the kernels take up to {self.MAX_DIM}")
        self.scale, self.diff, self.eps = float(spec.scale), float(spec.diff), float(spec.norm_eps)
        self.qkv_bias, self.out_bias = bool(spec.qkv_bias), bool(spec.out_bias)
        self.q_dim, self.k_dim, self.v_dim = self.H * 2 * self.D, self.G * 2 * self.D, self.G * self.V
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None
        self.lam = 0.0

    def parameters(self) -> dict[str, ParamSpec]:
        p = {"q": ParamSpec((self.q_dim, self.hidden)), "k": ParamSpec((self.k_dim, self.hidden)),
             "v": ParamSpec((self.v_dim, self.hidden)), "o": ParamSpec((self.hidden, self.H * self.V))}
        if self.qkv_bias:
            p.update({"q.b": ParamSpec((self.q_dim,)), "k.b": ParamSpec((self.k_dim,)), "v.b": ParamSpec((self.v_dim,))})
        if self.out_bias:
            p["o.b"] = ParamSpec((self.hidden,))
        for n in ("lq1", "lk1", "lq2", "lk2"):
            p[n] = ParamSpec((self.D,), compute_dtype=False)
        return p

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([t["q"], t["k"], t["v"]], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([t["q.b"], t["k.b"], t["v.b"]], dim=0).contiguous()
        self.w_o = t["o"].contiguous()
        if self.out_bias:
            self.b_o = t["o.b"].contiguous()
        one = float((t["lq1"].float() * t["lk1"].float()).sum())
        two = float((t["lq2"].float() * t["lk2"].float()).sum())
        self.lam = math.exp(one) - math.exp(two) + self.diff

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.G, 2 * self.D, None, value_dim=self.V)

    def forward(self, x: torch.Tensor, step, cache, state=None) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        grp = step.groups[cache.group]
        proj = torch.empty((T, self.q_dim + self.k_dim + self.v_dim), dtype=x.dtype, device=x.device)
        ops.linear(proj, x, self.w_qkv, self.b_qkv)
        if cache.writable:
            ops.kv_write_pair(proj, self.q_dim, self.q_dim + self.k_dim, cache.k, cache.v, grp.slot_mapping,
                              self.G, 2 * self.D, self.V, cache.page_size)
        attn = torch.empty((T, self.H * self.V), dtype=x.dtype, device=x.device)
        ops.attention_diff(attn, proj, cache.k, cache.v, grp.block_tables, step, self.H, self.G, self.D, self.V,
                           cache.page_size, self.scale, self.lam, self.eps, 1.0 - self.diff)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, attn, self.w_o, self.b_o, may_defer=True)


register("mixer", "diff_attention", DiffAttention)
