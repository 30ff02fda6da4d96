"""The gated delta rule: a recurrent mixer with a matrix state per head and short causal filters.

One fused projection gives, per token, [q (G D) | k (G D) | v (H V) | gate (H V) | b (H) | a (H)].  q, k and v
pass a causal filter of a few taps per channel and SiLU; q and k are brought to unit length per head and q is
divided by sqrt(D); write strength w = sigmoid(b); fade d = exp(-exp(A) softplus(a + dt)).  Per head, in 32-bit,
with M the head's memory [D, V]:   M <- d M;   e = w (v - M^T k);   M <- M + k e^T;   y = M^T q   (the read-out
comes after the token's own write).  Every head's y is normed by its own root mean square, scaled by a weight
common to the heads and gated by silu(gate); then the output projection.

Nothing is cached per token.  The mixer declares one flat 32-bit state per request:
[H D V values of M | (taps - 1) x (2 G D + H V) last filter inputs], zeroed when the request is admitted, so
the first portion needs no branch and a captured step's padding rows update the null slot.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, Mixer, ParamSpec, StateNeed, register


class DeltaRule(Mixer):
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.G = int(spec.num_heads), int(spec.num_kv_heads)
        self.D, self.V, self.taps = int(spec.key_dim), int(spec.value_dim), int(spec.conv_taps)
        if self.G < 1 or self.H % self.G:
            raise ValueError("delta_rule: num_heads must be a multiple of num_kv_heads")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"delta_rule: a filter of {self.taps} taps (the kernels take 1 to 8)")
        self.eps, self.unit_eps = float(spec.norm_eps), float(spec.unit_eps)
        self.qk, self.hv = self.G * self.D, self.H * self.V
        self.channels = 2 * self.qk + self.hv                   # what passes the filter
        self.w_in = self.w_o = self.conv = self.a_log = self.dt_bias = self.norm_w = None

    def parameters(self) -> dict[str, ParamSpec]:
        h, t = self.hidden, self.taps
        return {"q": ParamSpec((self.qk, h)), "k": ParamSpec((self.qk, h)), "v": ParamSpec((self.hv, h)),
                "g": ParamSpec((self.hv, h)), "b": ParamSpec((self.H, h)), "a": ParamSpec((self.H, h)),
                "q.conv": ParamSpec((self.qk, t), compute_dtype=False), "k.conv": ParamSpec((self.qk, t), compute_dtype=False),
                "v.conv": ParamSpec((self.hv, t), compute_dtype=False),
                "A_log": ParamSpec((self.H,), compute_dtype=False), "dt_bias": ParamSpec((self.H,), compute_dtype=False),
                "norm": ParamSpec((self.V,), compute_dtype=False, init="ones"),
                "o": ParamSpec((self.hidden, self.hv))}

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([t["q"], t["k"], t["v"], t["g"], t["b"], t["a"]], dim=0).contiguous()
        self.w_o = t["o"].contiguous()
        self.conv = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).float().contiguous()
        self.a_log, self.dt_bias = t["A_log"].float().contiguous(), t["dt_bias"].float().contiguous()
        self.norm_w = t["norm"].float().contiguous()

    def state_need(self) -> StateNeed:
        return StateNeed((self.H * self.D * self.V + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x: torch.Tensor, step, cache, state: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        H, G, D, V = self.H, self.G, self.D, self.V
        proj = torch.empty((T, self.channels + self.hv + 2 * H), dtype=x.dtype, device=x.device)
        ops.linear(proj, x, self.w_in)
        # 32-bit rows [q | k | v | g | beta | k.q] for the scan
        ready = torch.empty((T, self.channels + 2 * H + G), dtype=torch.float32, device=x.device)
        ops.delta_prepare(ready, proj, self.conv, self.a_log, self.dt_bias, state, step, H, G, D, V, self.taps,
                          self.unit_eps)
        o = torch.empty((T, self.hv), dtype=torch.float32, device=x.device)
        ops.delta_scan(o, ready, proj, state, step, H, G, D, V, self.taps)
        y = torch.empty((T, self.hv), dtype=x.dtype, device=x.device)
        ops.head_gated_rmsnorm(y, o, proj[:, self.channels:self.channels + self.hv], self.norm_w, self.eps, H, V)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, y, self.w_o, may_defer=True)


register("mixer", "delta_rule", DeltaRule)
