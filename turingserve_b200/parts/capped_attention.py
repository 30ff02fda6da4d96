"""Grouped-query attention whose values are its keys, over the paged cache.

One fused projection gives, per token, [q (H D) | k (G D)].  q and k are RMS-normed over their WHOLE rows
(all heads at once) with learned weights; the query is then multiplied by a temperature that grows with its
position p: 1 + coef ln(floor((p + 1) / every) + 1).  The cache keeps the normed key rows as keys and the key
rows as projected (before the norm) as values.  score = cap tanh(q.k scale / cap) - slope_h (i - j) with
slope_h = 2^(-power (h + 1) / H); position i sees i - window < j <= i; ordinary softmax; output projection.
Positions enter through the temperature, the bias and the window only.  Cap, bias, window and temperature
are each optional in the spec.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, CacheNeed, Mixer, ParamSpec, register


class CappedAttention(Mixer):
    MAX_DIM = 512               # the kernel's limit on a head's width

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.G, self.D = int(spec.num_heads), int(spec.num_kv_heads), int(spec.head_dim)
        if self.G < 1 or self.H % self.G:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not 0 < self.D <= self.MAX_DIM:
            raise ValueError(f"capped_attention: heads of {self.D} (the kernel takes up to {self.MAX_DIM})")
        self.scale, self.eps = float(spec.scale), float(spec.norm_eps)
        self.softcap = float(spec.softcap) if spec.softcap else 0.0
        self.window = int(spec.window) if spec.window else None
        self.q_temp = (float(spec.q_temp[0]), int(spec.q_temp[1])) if spec.q_temp else (0.0, 1)
        self.slope_power = None if spec.slope_power is None else float(spec.slope_power)
        self.slopes = None
        if self.slope_power is not None:
            self.slopes = torch.tensor([2.0 ** (-self.slope_power * (h + 1) / self.H) for h in range(self.H)],
                                       dtype=torch.float32, device=ctx.device)
        self.w_qk = self.w_o = self.q_w = self.k_w = None

    def parameters(self) -> dict[str, ParamSpec]:
        hd, gd = self.H * self.D, self.G * self.D
        return {"q": ParamSpec((hd, self.hidden)), "k": ParamSpec((gd, self.hidden)),
                "q.norm": ParamSpec((hd,), compute_dtype=False, init="ones"),
                "k.norm": ParamSpec((gd,), compute_dtype=False, init="ones"),
                "o": ParamSpec((self.hidden, hd))}

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_qk = torch.cat([t["q"], t["k"]], dim=0).contiguous()
        self.w_o = t["o"].contiguous()
        self.q_w, self.k_w = t["q.norm"].float().contiguous(), t["k.norm"].float().contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.G, self.D, self.window)

    def forward(self, x: torch.Tensor, step, cache, state=None) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        H, G, D = self.H, self.G, self.D
        grp = step.groups[cache.group]
        proj = torch.empty((T, (H + G) * D), dtype=x.dtype, device=x.device)
        ops.linear(proj, x, self.w_qk)
        # q normed and heated in place; normed keys and raw keys (the values) into the cache
        ops.qk_rownorm_write(proj, self.q_w, self.k_w, self.eps, step.positions, self.q_temp[0], self.q_temp[1],
                             cache.k, cache.v, grp.slot_mapping if cache.writable else None, H, G, D, cache.page_size)
        attn = torch.empty((T, H, D), dtype=x.dtype, device=x.device)
        ops.attention_biased(attn, proj[:, :H * D].view(T, H, D), cache.k, cache.v, grp.block_tables, step, G,
                             cache.page_size, self.scale, self.softcap, self.slopes, self.window)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, attn.view(T, H * D), self.w_o, may_defer=True)


register("mixer", "capped_attention", CappedAttention)
