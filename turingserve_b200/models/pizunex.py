"""Pizunex: config.json keys -> ``ModelConfig``, and checkpoint tensor names.

A decoder whose layers are, in the order the configuration lists them, one of three mixers (``delta``: the
gated delta rule over a matrix state with short causal filters on q, k, v; ``attention``: grouped-query
attention whose values are its keys, with whole-row query/key norms, a query temperature that grows with the
position, capped scores, a distance bias per head and a sliding window; ``latent_attention``: attention
through low-rank latents with a rotated part (pairs of neighbouring dimensions, YaRN-blended frequencies))
and a dense squared-ReLU feed-forward or none.  What is fixed for the family: pre-norm layers over a residual
stream kept in 32-bit; RMS norms with a learned scale named by the norm's own prefix; no biases; separate
input embedding and output head; a layer may name another layer whose tensors it uses (``weights_of``)
while keeping memory of its own.  Every size and constant comes from config.json.
"""

from __future__ import annotations

from turingserve_b200.config.model_config import (
    CappedAttentionSpec, DeltaRuleSpec, LatentAttentionSpec, LayerRun, LayerSpec, MLPSpec, ModelConfig,
    StreamRMSNormSpec, YarnRotarySpec)
from turingserve_b200.config.registry import (
    Architecture, LayerTensorNames, TensorNames, register_architecture)

NAME = "Pizunex"
# nothing in the design bounds a sequence (the rotation's angles are computed from the position itself)
NO_POSITION_LIMIT = 1 << 30
# the distance bias of the attention mixer: slope_h = 2^(-SLOPE_POWER (h + 1) / heads)
SLOPE_POWER = 8.0


def _require(c: dict, key: str, where: str = "config.json"):
    if key not in c:
        raise ValueError(f"{where} is missing required key {key!r}")
    return c[key]


def _rotation(rot: dict, where: str) -> YarnRotarySpec:
    sc = rot.get("scaling") or None
    kw = {}
    if sc:
        kw = dict(factor=float(_require(sc, "factor", where)), original=float(_require(sc, "original", where)),
                  fast=float(_require(sc, "fast", where)), slow=float(_require(sc, "slow", where)))
    return YarnRotarySpec(base=float(_require(rot, "base", where)), dims=int(_require(rot, "dims", where)), **kw)


def _mixer(kind: str, m: dict, eps: float, where: str):
    heads = int(_require(m, "heads", where))
    if kind == "delta":
        return DeltaRuleSpec(num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)),
                             key_dim=int(_require(m, "dim", where)), value_dim=int(_require(m, "vdim", where)),
                             conv_taps=int(_require(m, "conv", where)), norm_eps=eps)
    if kind == "attention":
        dim = int(_require(m, "dim", where))
        if int(m.get("vdim", dim)) != dim:
            raise ValueError(f"{where}: the values of this mixer are its keys, so vdim must equal dim")
        qt = m.get("q_temp") or None
        mask = m.get("mask") or None
        cap = m.get("softcap")
        return CappedAttentionSpec(
            num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)), head_dim=dim,
            scale=float(_require(m, "scale", where)), norm_eps=eps, softcap=float(cap) if cap else None,
            window=int(_require(mask, "size", where)) if mask else None,
            q_temp=(float(_require(qt, "coef", where)), int(_require(qt, "every", where))) if qt else None,
            slope_power=SLOPE_POWER)
    if kind == "latent_attention":
        rope_dim = int(_require(m, "rot_dim", where))
        rot = _rotation(_require(m, "rot", where), where)
        if rot.dims > rope_dim or rot.dims % 2:
            raise ValueError(f"{where}: rot.dims {rot.dims} must be even and at most rot_dim {rope_dim}")
        return LatentAttentionSpec(
            num_heads=heads, nope_dim=int(_require(m, "dim", where)), rope_dim=rope_dim,
            value_dim=int(_require(m, "vdim", where)), q_rank=int(_require(m, "q_rank", where)),
            kv_rank=int(_require(m, "kv_rank", where)), scale=float(_require(m, "scale", where)), norm_eps=eps,
            position=rot)
    raise ValueError(f"{where}: unknown layer type {kind!r} (known: delta, attention, latent_attention)")


def _feed_forward(f: dict | None, where: str):
    if f is None:
        return None
    kind = _require(f, "kind", where)
    if kind == "dense":
        return MLPSpec(intermediate_size=int(_require(f, "ff", where)), activation="relu2")
    raise ValueError(f"{where}: unknown feed-forward kind {kind!r} (known: dense)")


def parse_config(c: dict, gen: dict | None = None) -> ModelConfig:
    eps = float(_require(_require(c, "norm"), "eps", "norm"))
    norm = StreamRMSNormSpec(eps=eps, weight_name="")
    entries = _require(c, "layers")
    layers, ids, place, runs = [], [], {}, []
    for i, entry in enumerate(entries):
        where = f"layers[{i}]"
        src = entry.get("weights_of")
        if src is not None:
            src = int(src)
            if src not in place:
                raise ValueError(f"{where}: weights_of {src} must name an earlier layer with tensors of its own")
            if entry.get("type") != entries[src].get("type"):
                raise ValueError(f"{where}: uses the tensors of layer {src}, which is of another type")
            runs.append(LayerRun(place[src]))
            continue
        mixer = _mixer(_require(entry, "type", where), _require(entry, "mixer", where), eps, where)
        ff = _feed_forward(entry.get("mlp"), where)
        roles = dict(mixer=mixer, mixer_norm=norm)
        if ff is not None:
            roles.update(feed_forward=ff, ffn_norm=norm)
        place[i] = len(layers)
        ids.append(i)
        layers.append(LayerSpec("pre_norm_stream", **roles))
        runs.append(LayerRun(place[i]))
    eos = (gen or {}).get("eos_token_id", c.get("eos_token_id"))
    eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
    # which entry of config.json every set of weights belongs to (its tensors are named 'l<entry>.'), and which
    # entry every run of the schedule is
    extras = (("layer_ids", tuple(ids)),)
    return ModelConfig(
        architecture=NAME, hidden_size=int(_require(c, "width")), vocab_size=int(_require(c, "vocab")),
        layers=tuple(layers), schedule=tuple(runs), final_norm=norm, tie_word_embeddings=False,
        max_position_embeddings=int(c.get("max_positions", NO_POSITION_LIMIT)), eos_token_ids=eos_ids,
        bos_token_id=c.get("bos_token_id"), extras=extras)


def tensor_names(cfg: ModelConfig) -> TensorNames:
    """'l<i>.norm1', 'l<i>.mix.<name>', 'l<i>.norm2', 'l<i>.mlp.<name>'; 'embed', 'final.norm', 'head'; i counts
    the entries of config.json's layer list, so the numbers of layers that borrow their tensors are skipped."""
    ids = cfg.extra("layer_ids") or tuple(range(len(cfg.layers)))
    layers = []
    for i, spec in zip(ids, cfg.layers):
        names = dict(mixer=f"l{i}.mix.", mixer_norm=f"l{i}.norm1")
        if "feed_forward" in spec.roles:
            names.update(feed_forward=f"l{i}.mlp.", ffn_norm=f"l{i}.norm2")
        layers.append(LayerTensorNames(**names))
    return TensorNames(embedding="embed", lm_head="head", final_norm="final.norm", layers=tuple(layers))


def _entry(spec: LayerSpec) -> dict:
    m = spec.mixer
    if isinstance(m, DeltaRuleSpec):
        entry = {"type": "delta", "mixer": {"heads": m.num_heads, "kv_heads": m.num_kv_heads, "dim": m.key_dim,
                                            "vdim": m.value_dim, "conv": m.conv_taps}}
    elif isinstance(m, CappedAttentionSpec):
        mix = {"heads": m.num_heads, "kv_heads": m.num_kv_heads, "dim": m.head_dim, "vdim": m.head_dim,
               "scale": m.scale}
        if m.softcap:
            mix["softcap"] = m.softcap
        if m.window:
            mix["mask"] = {"size": m.window}
        if m.q_temp:
            mix["q_temp"] = {"coef": m.q_temp[0], "every": m.q_temp[1]}
        entry = {"type": "attention", "mixer": mix}
    else:
        r = m.position
        rot = {"base": r.base, "dims": r.dims}
        if r.factor:
            rot["scaling"] = {"factor": r.factor, "original": r.original, "fast": r.fast, "slow": r.slow}
        entry = {"type": "latent_attention",
                 "mixer": {"heads": m.num_heads, "dim": m.nope_dim, "rot_dim": m.rope_dim, "vdim": m.value_dim,
                           "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "rot": rot}}
    f = spec.roles.get("feed_forward")
    entry["mlp"] = None if f is None else {"kind": "dense", "ff": f.intermediate_size}
    return entry


def to_config_json(cfg: ModelConfig) -> dict:
    """The layer list in schedule order: a run of a layer that ran before borrows its tensors."""
    first_run: dict[int, int] = {}
    layers = []
    for r, run in enumerate(cfg.schedule):
        entry = _entry(cfg.layers[run.layer])
        if run.layer in first_run:
            entry["weights_of"] = first_run[run.layer]
        else:
            first_run[run.layer] = r
        layers.append(entry)
    out = {"architecture": NAME, "width": cfg.hidden_size, "vocab": cfg.vocab_size, "layers": layers,
           "norm": {"eps": cfg.final_norm.eps}}
    if cfg.max_position_embeddings != NO_POSITION_LIMIT:
        out["max_positions"] = cfg.max_position_embeddings
    if cfg.eos_token_ids:
        out["eos_token_id"] = list(cfg.eos_token_ids) if len(cfg.eos_token_ids) > 1 else cfg.eos_token_ids[0]
    return out


def make_config(*, width: int, vocab: int, layers: list[dict], eps: float = 1e-6,
                eos_token_id: int | None = None) -> ModelConfig:
    """A Pizunex ``ModelConfig`` from sizes (through the same parser as config.json); ``layers`` as the
    configuration file lists them."""
    c = {"architecture": NAME, "width": width, "vocab": vocab, "layers": layers, "norm": {"eps": eps}}
    if eos_token_id is not None:
        c["eos_token_id"] = eos_token_id
    return parse_config(c)


register_architecture(Architecture(NAME, parse_config, tensor_names, to_config_json))
