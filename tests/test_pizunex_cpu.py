"""Pizunex without a GPU: the parser and its refusals, the checkpoint names of layers that borrow tensors, the
cache groups its mixers ask for, the engine's host logic (pages and state slots going round, portions down to two
tokens, mixed batches) through the kernel twins against the plain model, and the plain model against closed forms."""

from __future__ import annotations

import json
import math

import pytest
import torch

from tests import pizunex_tiny as pt
from tests import plain_pizunex as plain
from tests import schedules
from turingserve_b200.cache.manager import CacheManager, RunNeeds
from turingserve_b200.config.model_config import CappedAttentionSpec, DeltaRuleSpec, LatentAttentionSpec
from turingserve_b200.config.registry import get_architecture, load_model_config
from turingserve_b200.parts.base import CacheNeed, StateNeed


def test_parser_reads_every_size_and_option():
    cfg = pt.tiny_config("A")
    assert cfg.architecture == "Pizunex" and cfg.hidden_size == 64 and cfg.vocab_size == 131
    assert len(cfg.layers) == 3 and [r.layer for r in cfg.schedule] == [0, 1, 2, 0, 2]
    d, a, l = (cfg.layers[i].mixer for i in range(3))
    assert isinstance(d, DeltaRuleSpec) and (d.num_heads, d.num_kv_heads, d.key_dim, d.value_dim, d.conv_taps) == (4, 2, 16, 8, 3)
    assert isinstance(a, CappedAttentionSpec) and (a.window, a.softcap, a.q_temp, a.slope_power) == (9, 6.0, (0.4, 5), 8.0)
    assert isinstance(l, LatentAttentionSpec) and (l.nope_dim, l.rope_dim, l.value_dim, l.q_rank, l.kv_rank) == (8, 8, 12, 24, 20)
    assert l.position.factor == 2.5 and l.position.original == 16 and l.norm_eps == 1e-5
    assert "feed_forward" not in cfg.layers[0].roles and cfg.layers[1].feed_forward.activation == "relu2"
    b = pt.tiny_config("B")
    assert b.layers[1].mixer.softcap is None and b.layers[1].mixer.q_temp is None and b.layers[0].mixer.position.factor is None
    assert b.layers[0].mixer.position.dims == 4 and pt.tiny_config("C").layers[0].mixer.window is None


def test_names_of_layers_that_lend_their_tensors_and_round_trip(tmp_path):
    arch = get_architecture("Pizunex")
    cfg = pt.tiny_config("B")
    names = arch.tensor_names(cfg)
    assert [n.mixer for n in names.layers] == ["l0.mix.", "l1.mix.", "l2.mix.", "l3.mix."]
    assert names.layers[1].ffn_norm == "l1.norm2" and "ffn_norm" not in names.layers[0].roles()
    again = arch.parse_config(arch.to_config_json(cfg))
    assert again.layers == cfg.layers and again.schedule == cfg.schedule
    # a borrowed layer in the middle: the numbers of the layers behind it are not moved up
    c = arch.to_config_json(cfg)
    c["layers"] = [c["layers"][0], {**c["layers"][0], "weights_of": 0}, c["layers"][2]]
    moved = arch.parse_config(c)
    assert [n.mixer for n in arch.tensor_names(moved).layers] == ["l0.mix.", "l2.mix."]
    assert [r.layer for r in moved.schedule] == [0, 0, 1]
    folder = pt.make_tiny_folder("D", tmp_path)
    assert load_model_config(folder).architecture == "Pizunex"


def test_parser_refusals():
    arch = get_architecture("Pizunex")
    good = arch.to_config_json(pt.tiny_config("A"))
    for edit, match in ((lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
                        (lambda c: c["layers"][3].update(weights_of=7), "weights_of"),
                        (lambda c: c["layers"][3].update(weights_of=1), "another type"),
                        (lambda c: c["layers"][1]["mixer"].update(vdim=24), "vdim"),
                        (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
                        (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
                        (lambda c: c.pop("norm"), "norm")):
        bad = json.loads(json.dumps(good))
        edit(bad)
        with pytest.raises(ValueError, match=match):
            arch.parse_config(bad)


def test_cache_groups_and_state_of_the_three_mixers(tmp_path):
    """A latent layer caches one row a token and no value rows; a windowed layer gives its pages back; the
    recurrent layer owns a flat state (matrix and filter memory) that starts clean in a slot used again."""
    from turingserve_b200.engine.runner import run_needs
    from turingserve_b200.weights.loader import load_model
    model, cfg = load_model(pt.make_tiny_folder("A", tmp_path), torch.float32, "cpu")
    needs = run_needs(model)
    assert needs[0].state.shape == (4 * 16 * 8 + 2 * (2 * 2 * 16 + 4 * 8),) and needs[0].cache is None
    assert needs[1].cache == CacheNeed(2, 16, 9) and needs[2].cache == CacheNeed(1, 28, None, value_dim=0)
    cm = CacheManager(needs, 16, 6, 3, torch.float32, "cpu")
    assert len(cm.groups) == 2 and cm.groups[1].runs == [2, 4]
    lat = cm.view(4)
    assert lat.k.shape == (6, 1, 16, 28) and lat.v.numel() == 0 and lat.k.data_ptr() != cm.view(2).k.data_ptr()
    assert cm.states[0].data_ptr() != cm.states[3].data_ptr()          # a borrowed layer's memory is its own
    rc = cm.admit("a")
    cm.grow(rc, 40)
    cm.advance(rc, 40)
    assert rc.tables[0][0] == 0 and rc.tables[0][1] == 0 and rc.tables[0][2] != 0      # window of 9: pages 0, 1 returned
    assert all(p != 0 for p in rc.tables[1])
    cm.states[0][rc.slot].fill_(3.0)
    cm.release(rc)
    cm.check()
    assert float(cm.states[0][cm.admit("b").slot].abs().sum()) == 0.0


def _replay_cpu(folder, name, steps):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    from tests.twin_ops import TwinOps
    kernels.use(TwinOps())
    try:
        rp = Replayer(folder, torch.float32, schedules.peak_tokens(steps), "cpu", page_size=pt.page_size(name))
        outs = {}
        with torch.inference_mode():
            for s in steps:
                o = rp.step(s)
                if o is not None:
                    outs[s["step"]] = o
                rp.cache.check()
        assert not rp.cache.live
    finally:
        kernels.use(None)
    return schedules.collect(steps, outs)


@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("schedule", ["decode_tail", "portions", "mixed"])
def test_host_logic_against_plain(tmp_path, name, schedule):
    """More requests than state slots, a pool that makes pages go round, portions down to two tokens."""
    folder = pt.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    reqs = {f"r{i}": pt.random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate([1, 9, 34, 21, 17, 40])}
    steps = getattr(schedules, schedule)(reqs, tail=5) if schedule != "portions" else schedules.portions(reqs)
    got = _replay_cpu(folder, name, steps)
    expected = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    bad = schedules.first_bad(got, expected, 2e-4)
    assert bad is None, f"first wrong place (request, position, error): {bad}"


def test_the_plain_functions_agree_with_closed_forms():
    g = torch.Generator().manual_seed(0)
    T, D, V = 9, 5, 3
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (D, D, V))
    gate, beta = torch.rand(T, generator=g, dtype=torch.float64), torch.rand(T, generator=g, dtype=torch.float64)
    out, S = plain.delta_scan(q, k, v, gate, beta)
    # with beta = 0 nothing is ever written; with g = 1, beta = 1 and one unit key the state holds that key's value
    zero, _ = plain.delta_scan(q, k, v, gate, torch.zeros(T, dtype=torch.float64))
    assert float(zero.abs().max()) == 0.0
    e = torch.zeros(1, D, dtype=torch.float64)
    e[0, 2] = 1.0
    o, S1 = plain.delta_scan(e, e, v[:1], torch.ones(1, dtype=torch.float64), torch.ones(1, dtype=torch.float64))
    assert torch.allclose(o[0], v[0]) and torch.allclose(S1[2], v[0])
    o2, _ = plain.delta_scan(e, e, v[1:2], torch.ones(1, dtype=torch.float64), torch.ones(1, dtype=torch.float64), S1)
    assert torch.allclose(o2[0], v[1])                                    # the same key again: its value is replaced
    half, S_half = plain.delta_scan(q[:4], k[:4], v[:4], gate[:4], beta[:4])
    rest, S_end = plain.delta_scan(q[4:], k[4:], v[4:], gate[4:], beta[4:], S_half)
    assert torch.allclose(torch.cat([half, rest]), out, atol=1e-12) and torch.allclose(S_end, S, atol=1e-12)
    # the filter: the last tap multiplies the present token, zeros before the sequence
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    y = plain.short_filter(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    # the window keeps the query's own position and window - 1 before it; the bias grows with the distance
    s = plain.capped_scores(torch.ones(6, 2, dtype=torch.float64), torch.ones(6, 2, dtype=torch.float64), 1.0, None, 0.5, 3)
    assert torch.isinf(s[5, 2]) and s[5, 3] == 2.0 - 1.0 and s[5, 5] == 2.0 and torch.isinf(s[2, 3])
    capped = plain.capped_scores(100 * torch.ones(1, 2, dtype=torch.float64), torch.ones(1, 2, dtype=torch.float64), 1.0, 7.0, 0.0, None)
    assert abs(float(capped[0, 0]) - 7.0) < 1e-9
    assert plain.slopes(4).tolist() == [0.25, 0.0625, 0.015625, 0.00390625]
    heat = plain.query_heat(torch.tensor([0.0, 3.0, 4.0, 9.0]), 0.5, 5)
    assert torch.allclose(heat, torch.tensor([1.0, 1.0, 1.0 + 0.5 * math.log(2.0), 1.0 + 0.5 * math.log(3.0)]))
    # rotation: a pair keeps its length times the magnitude; without blending the angle is position * base^(-2i/dims)
    cos, sin = plain.yarn_angles({"base": 100.0, "dims": 4}, torch.tensor([3]))
    assert torch.allclose(cos[0], torch.cos(torch.tensor([3.0, 0.3], dtype=torch.float64)))
    r = plain.rotate_pairs(torch.tensor([[1.0, 0.0, 0.0, 2.0, 5.0]], dtype=torch.float64), cos, sin)
    assert torch.allclose(r[0, :2].norm(), torch.tensor(1.0, dtype=torch.float64)) and float(r[0, 4]) == 5.0
    cos, sin = plain.yarn_angles({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}},
                                 torch.tensor([1]))
    mag = 0.1 * math.log(4.0) + 1.0
    assert torch.allclose(cos[0, 0], torch.cos(torch.tensor(1.0, dtype=torch.float64)) * mag)      # fastest pair: not slowed
    assert torch.allclose(cos[0, 3] ** 2 + sin[0, 3] ** 2, torch.tensor(mag * mag, dtype=torch.float64))
    slow = 100.0 ** (-6.0 / 8.0)
    assert torch.allclose(sin[0, 3], torch.sin(torch.tensor(slow / 4.0, dtype=torch.float64)) * mag)  # slowest: by the factor
