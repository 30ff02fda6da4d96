"""Komirax: config.json keys -> ``ModelConfig``, and checkpoint tensor names.

A decoder whose layers alternate, in an order the configuration gives, between two mixers (linear
attention with a decaying matrix state: ``lightning``; softmax attention with two score maps a head:
``attention``) and two feed-forwards (dense with the tanh form of GELU; routed, with squared-ReLU experts,
sigmoid scores that are not renormalised and that multiply the expert's input) or none.  What is fixed for
the family: pre-norm layers over a residual stream kept in 32-bit; RMS norms with a learned scale; no
position encoding anywhere; biases on q/k/v of the attention mixer only; separate input embedding and output
head; a span of layers (``loop``: start, stop, times) that runs several times in a row with the same weights,
every pass with memory of its own and every pass but the first opened by adding the embedding rows to the
stream.  Every size and constant comes from config.json.
"""

from __future__ import annotations

from turingserve_b200.config.model_config import (
    DiffAttentionSpec, LayerRun, LayerSpec, LightningSpec, MLPSpec, ModelConfig, RoutedMLPSpec, StreamRMSNormSpec)
from turingserve_b200.config.registry import (
    Architecture, LayerTensorNames, TensorNames, register_architecture)

NAME = "Komirax"
# the design has no position encoding, hence no longest sequence of its own
NO_POSITION_LIMIT = 1 << 30


def _require(c: dict, key: str, where: str = "config.json"):
    if key not in c:
        raise ValueError(f"{where} is missing required key {key!r}")
    return c[key]


def _mixer(kind: str, m: dict, eps: float, where: str):
    if kind == "lightning":
        heads = int(_require(m, "heads", where))
        decay = _require(m, "decay", where)
        if not isinstance(decay, (list, tuple)):
            decay = [decay] * heads
        return LightningSpec(num_heads=heads, key_dim=int(_require(m, "dim", where)),
                             value_dim=int(_require(m, "vdim", where)), decays=tuple(float(d) for d in decay),
                             norm_eps=eps)
    if kind == "attention":
        heads = int(_require(m, "heads", where))
        return DiffAttentionSpec(num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)),
                                 key_dim=int(_require(m, "dim", where)), value_dim=int(_require(m, "vdim", where)),
                                 scale=float(_require(m, "scale", where)), diff=float(_require(m, "diff", where)),
                                 norm_eps=eps, qkv_bias=True, out_bias=False)
    raise ValueError(f"{where}: unknown layer type {kind!r} (known: lightning, attention)")


def _feed_forward(f: dict | None, where: str):
    if f is None:
        return None
    kind = _require(f, "kind", where)
    if kind == "dense":
        return MLPSpec(intermediate_size=int(_require(f, "ff", where)), activation="gelu_tanh")
    if kind == "moe":
        router = _require(f, "router", where)
        return RoutedMLPSpec(num_experts=int(_require(router, "experts", where)), top_k=int(_require(router, "top", where)),
                             intermediate_size=int(_require(_require(f, "expert", where), "ff", where)),
                             activation="relu2", scoring="sigmoid", renormalize=False, weight_on="input")
    raise ValueError(f"{where}: unknown feed-forward kind {kind!r} (known: dense, moe)")


def run_order(n_layers: int, loop: dict | None) -> tuple[LayerRun, ...]:
    """Layers before ``start`` once, layers start..stop-1 ``times`` times, the rest once; the first run of
    every pass after the first takes the embedding rows into the stream."""
    if not loop:
        return tuple(LayerRun(i) for i in range(n_layers))
    a, b, times = int(_require(loop, "start", "loop")), int(_require(loop, "stop", "loop")), int(loop.get("times", 1))
    if not (0 <= a <= b <= n_layers) or times < 1:
        raise ValueError(f"loop {loop!r} does not fit {n_layers} layers")
    runs = [LayerRun(i) for i in range(a)]
    for p in range(times):
        runs += [LayerRun(i, add_embedding=(p > 0 and i == a)) for i in range(a, b)]
    return tuple(runs + [LayerRun(i) for i in range(b, n_layers)])


def parse_config(c: dict, gen: dict | None = None) -> ModelConfig:
    eps = float(_require(_require(c, "norm"), "eps", "norm"))
    norm = StreamRMSNormSpec(eps=eps, weight_name="")
    layers = []
    for i, entry in enumerate(_require(c, "layers")):
        where = f"layers[{i}]"
        mixer = _mixer(_require(entry, "type", where), _require(entry, "mixer", where), eps, where)
        ff = _feed_forward(entry.get("mlp"), where)
        roles = dict(mixer=mixer, mixer_norm=norm)
        if ff is not None:
            roles.update(feed_forward=ff, ffn_norm=norm)
        layers.append(LayerSpec("pre_norm_stream", **roles))
    eos = (gen or {}).get("eos_token_id", c.get("eos_token_id"))
    eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
    loop = c.get("loop") or None
    extras = (("loop", tuple(sorted(loop.items()))),) if loop else ()
    return ModelConfig(
        architecture=NAME, hidden_size=int(_require(c, "width")), vocab_size=int(_require(c, "vocab")),
        layers=tuple(layers), schedule=run_order(len(layers), loop), final_norm=norm, tie_word_embeddings=False,
        max_position_embeddings=int(c.get("max_positions", NO_POSITION_LIMIT)), eos_token_ids=eos_ids,
        bos_token_id=c.get("bos_token_id"), extras=extras)


def tensor_names(cfg: ModelConfig) -> TensorNames:
    """'l<i>.norm1', 'l<i>.mix.<name>', 'l<i>.norm2', 'l<i>.mlp.<name>'; 'embed', 'final.norm', 'head'.  The
    norms' scales are named by the prefix itself (their local name is '')."""
    layers = []
    for i, spec in enumerate(cfg.layers):
        names = dict(mixer=f"l{i}.mix.", mixer_norm=f"l{i}.norm1")
        if "feed_forward" in spec.roles:
            names.update(feed_forward=f"l{i}.mlp.", ffn_norm=f"l{i}.norm2")
        layers.append(LayerTensorNames(**names))
    return TensorNames(embedding="embed", lm_head="head", final_norm="final.norm", layers=tuple(layers))


def to_config_json(cfg: ModelConfig) -> dict:
    layers = []
    for spec in cfg.layers:
        m = spec.mixer
        if isinstance(m, LightningSpec):
            entry = {"type": "lightning", "mixer": {"heads": m.num_heads, "dim": m.key_dim, "vdim": m.value_dim,
                                                    "decay": list(m.decays)}}
        else:
            entry = {"type": "attention", "mixer": {"heads": m.num_heads, "kv_heads": m.num_kv_heads, "dim": m.key_dim,
                                                    "vdim": m.value_dim, "scale": m.scale, "diff": m.diff}}
        f = spec.roles.get("feed_forward")
        if f is None:
            entry["mlp"] = None
        elif isinstance(f, MLPSpec):
            entry["mlp"] = {"kind": "dense", "ff": f.intermediate_size}
        else:
            entry["mlp"] = {"kind": "moe", "expert": {"ff": f.intermediate_size},
                            "router": {"experts": f.num_experts, "top": f.top_k}}
        layers.append(entry)
    out = {"architecture": NAME, "width": cfg.hidden_size, "vocab": cfg.vocab_size, "layers": layers,
           "norm": {"eps": cfg.final_norm.eps}}
    loop = cfg.extra("loop")
    if loop:
        out["loop"] = dict(loop)
    if cfg.max_position_embeddings != NO_POSITION_LIMIT:
        out["max_positions"] = cfg.max_position_embeddings
    if cfg.eos_token_ids:
        out["eos_token_id"] = list(cfg.eos_token_ids) if len(cfg.eos_token_ids) > 1 else cfg.eos_token_ids[0]
    return out


def make_config(*, width: int, vocab: int, layers: list[dict], eps: float = 1e-6, loop: dict | None = None,
                eos_token_id: int | None = None) -> ModelConfig:
    """A Komirax ``ModelConfig`` from sizes (through the same parser as config.json); ``layers`` as the
    configuration file lists them."""
    c = {"architecture": NAME, "width": width, "vocab": vocab, "layers": layers, "norm": {"eps": eps}}
    if loop:
        c["loop"] = loop
    if eos_token_id is not None:
        c["eos_token_id"] = eos_token_id
    return parse_config(c)


register_architecture(Architecture(NAME, parse_config, tensor_names, to_config_json))
