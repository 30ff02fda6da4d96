"""Attention through low-rank latents, over the paged cache.

One fused projection gives, per token, [dq (q_rank) | latent (kv_rank) | rotated key part (R)].  Queries:
q = W_uq rms(dq), per head [D plain | R rotated].  Per token the cache keeps ONE row [c | kr] for all heads:
c = rms(latent) with its weight, kr the rotated key part.  Per head the plain key is W_uk c and the value
W_uv c; neither is ever formed for the cached tokens: the query is carried into the latent space instead,
qa_h = W_uk,h^T q_plain,h, so that  q_plain . (W_uk c) = qa . c, every head attends over the one cached row
(score = (qa . c + q_rot . kr) * scale, causal softmax, weighted sum of the c rows), and the head's output
is W_uv,h applied to that sum.  The rotation (neighbouring pairs, angle = position * frequency in 32-bit)
comes from the position encoding the spec names.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, CacheNeed, Mixer, ParamSpec, build, register


class LatentAttention(Mixer):
    MAX_ROW = 640               # the kernel's limit on the cached row's width (latent + rotated part)

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.H, self.D, self.R, self.V = int(spec.num_heads), int(spec.nope_dim), int(spec.rope_dim), int(spec.value_dim)
        self.q_rank, self.rank = int(spec.q_rank), int(spec.kv_rank)
        if self.rank + self.R > self.MAX_ROW:
            raise ValueError(f"latent_attention: cached rows of {self.rank + self.R} (the kernel takes up to {self.MAX_ROW})")
        self.scale, self.eps = float(spec.scale), float(spec.norm_eps)
        if spec.position is None:
            raise ValueError("latent_attention needs a position encoding for its rotated parts")
        self.rotary = build("position", spec.position, ctx)
        if self.rotary.dims > self.R:
            raise ValueError("the rotation covers more dimensions than the rotated part has")
        self.w_d = self.w_uq = self.w_ukt = self.w_uv = self.w_o = self.dq_w = self.dkv_w = None

    def parameters(self) -> dict[str, ParamSpec]:
        H, D, R, V = self.H, self.D, self.R, self.V
        return {"dq": ParamSpec((self.q_rank, self.hidden)), "dq.norm": ParamSpec((self.q_rank,), compute_dtype=False, init="ones"),
                "uq": ParamSpec((H * (D + R), self.q_rank)),
                "dkv": ParamSpec((self.rank + R, self.hidden)),
                "dkv.norm": ParamSpec((self.rank,), compute_dtype=False, init="ones"),
                "uk": ParamSpec((H * D, self.rank)), "uv": ParamSpec((H * V, self.rank)),
                "o": ParamSpec((self.hidden, H * V))}

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_d = torch.cat([t["dq"], t["dkv"]], dim=0).contiguous()
        self.w_uq = t["uq"].contiguous()
        # [H, rank, D]: head h's rows of W_uk, transposed, so that qa = W_ukT[h] q_plain is a product like any other
        self.w_ukt = t["uk"].view(self.H, self.D, self.rank).transpose(1, 2).contiguous()
        self.w_uv = t["uv"].view(self.H, self.V, self.rank).contiguous()
        self.w_o = t["o"].contiguous()
        self.dq_w, self.dkv_w = t["dq.norm"].float().contiguous(), t["dkv.norm"].float().contiguous()

    def cache_need(self) -> CacheNeed:
        # one row a token for all heads, and no value rows: the values are the row's first kv_rank columns
        return CacheNeed(1, self.rank + self.R, None, value_dim=0)

    def forward(self, x: torch.Tensor, step, cache, state=None) -> torch.Tensor:
        ops = kernels.ops()
        T = x.shape[0]
        H, D, R, V, rank = self.H, self.D, self.R, self.V, self.rank
        grp = step.groups[cache.group]
        rot = self.rotary
        proj = torch.empty((T, self.q_rank + rank + R), dtype=x.dtype, device=x.device)
        ops.linear(proj, x, self.w_d)
        if cache.writable:
            ops.latent_kv_write(proj, self.q_rank, self.dkv_w, self.eps, step.positions, rot.freq, rot.magnitude, rot.dims,
                                cache.k, grp.slot_mapping, rank, R, cache.page_size)
        cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
        ops.rms_rows(cq, proj, 0, self.dq_w, self.eps)
        q = torch.empty((T, H, D + R), dtype=x.dtype, device=x.device)
        ops.linear(q.view(T, H * (D + R)), cq, self.w_uq)
        qa = torch.empty((T, H, rank + R), dtype=x.dtype, device=x.device)
        ops.batched_linear(qa[:, :, :rank], q[:, :, :D], self.w_ukt)
        ops.rotate_pairs(qa[:, :, rank:], q[:, :, D:], step.positions, rot.freq, rot.magnitude, rot.dims)
        mixed = torch.empty((T, H, rank), dtype=x.dtype, device=x.device)
        ops.attention_biased(mixed, qa, cache.k, None, grp.block_tables, step, 1, cache.page_size, self.scale, 0.0,
                             None, None)
        heads = torch.empty((T, H, V), dtype=x.dtype, device=x.device)
        ops.batched_linear(heads, mixed, self.w_uv)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        return ops.linear(out, heads.view(T, H * V), self.w_o, may_defer=True)


register("mixer", "latent_attention", LatentAttention)
