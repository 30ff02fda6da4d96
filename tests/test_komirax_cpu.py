"""Komirax without a GPU: the configuration parser and the run order, tensor names, the cache group whose
value rows have their own width, and the engine's host logic (batch builder, cache manager, state slots,
step function, replay) driven through the kernels' plain twins against the plain whole-sequence model."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import komirax_tiny as kt
from tests import plain_komirax as plain
from tests import schedules
from turingserve_b200.cache.manager import CacheManager, RunNeeds
from turingserve_b200.config.registry import get_architecture, load_model_config
from turingserve_b200.models import komirax
from turingserve_b200.parts.base import CacheNeed, StateNeed


@pytest.mark.parametrize("loop,want", [
    (None, [0, 1, 2, 3]),
    ({"start": 0, "stop": 4, "times": 1}, [0, 1, 2, 3]),
    ({"start": 1, "stop": 3, "times": 3}, [0, 1, 2, 1, 2, 1, 2, 3]),
    ({"start": 0, "stop": 1, "times": 2}, [0, 0, 1, 2, 3]),
    ({"start": 2, "stop": 4, "times": 2}, [0, 1, 2, 3, 2, 3]),
    ({"start": 2, "stop": 2, "times": 5}, [0, 1, 2, 3]),
])
def test_run_order(loop, want):
    runs = komirax.run_order(4, loop)
    assert [r.layer for r in runs] == want
    opens = [i for i, r in enumerate(runs) if r.add_embedding]
    if loop and loop["times"] > 1 and loop["stop"] > loop["start"]:
        span = loop["stop"] - loop["start"]
        assert opens == [loop["start"] + span * p for p in range(1, loop["times"])]
    else:
        assert opens == []
    assert [(i, o) for i, o in plain.order({"layers": [0] * 4, "loop": loop})] == [(r.layer, r.add_embedding) for r in runs]


def test_parser_reads_every_size_and_refuses_what_it_does_not_know(tmp_path):
    cfg = kt.tiny_config("P")
    a, l = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (a.num_heads, a.num_kv_heads, a.key_dim, a.value_dim, a.diff, a.scale) == (4, 2, 16, 24, 0.3, 0.25)
    assert (l.num_heads, l.key_dim, l.value_dim, l.decays) == (2, 16, 32, (0.9, 0.99))
    assert "feed_forward" not in cfg.layers[2].roles and cfg.layers[0].feed_forward.top_k == 2
    assert cfg.final_norm.eps == 1e-5 and cfg.num_runs == 2 * 3 + 2
    arch = get_architecture("Komirax")
    again = arch.parse_config(arch.to_config_json(cfg))
    assert again.layers == cfg.layers and again.schedule == cfg.schedule
    bad = arch.to_config_json(cfg)
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError, match="unknown layer type"):
        arch.parse_config(bad)
    bad = arch.to_config_json(cfg)
    bad["layers"][1]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError, match="unknown feed-forward"):
        arch.parse_config(bad)
    bad = arch.to_config_json(cfg)
    del bad["layers"][1]["mixer"]["decay"]
    with pytest.raises(ValueError, match="decay"):
        arch.parse_config(bad)
    folder = kt.make_tiny_folder("R", tmp_path)
    assert load_model_config(folder).architecture == "Komirax"      # chosen by config.json's "architecture"


def test_a_cache_group_with_value_rows_of_their_own_width():
    needs = [RunNeeds(CacheNeed(2, 32, None, value_dim=24), None), RunNeeds(None, StateNeed((2, 4, 6))),
             RunNeeds(CacheNeed(2, 32, None, value_dim=24), None), RunNeeds(CacheNeed(2, 32), None)]
    cm = CacheManager(needs, 8, 5, 3, torch.float32, "cpu")
    assert len(cm.groups) == 2 and cm.groups[0].runs == [0, 2] and cm.groups[1].runs == [3]
    v0, v2, v3 = cm.view(0), cm.view(2), cm.view(3)
    assert v0.k.shape == (5, 2, 8, 32) and v0.v.shape == (5, 2, 8, 24) and v3.v.shape == (5, 2, 8, 32)
    assert v0.k.data_ptr() != v2.k.data_ptr() and v0.group == v2.group != v3.group
    assert cm.states[1].shape == (4, 2, 4, 6)
    assert CacheManager.bytes_per_page(needs, 8, torch.float32) == 4 * 8 * (2 * 2 * (32 + 24) + 2 * 64)
    rc = cm.admit("a")
    cm.states[1][rc.slot].fill_(3.0)
    cm.release(rc)
    assert float(cm.states[1][cm.admit("b").slot].abs().sum()) == 0.0          # a slot used again starts clean


def _replay_cpu(folder, name, steps):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    from tests.twin_ops import TwinOps
    kernels.use(TwinOps())
    try:
        rp = Replayer(folder, torch.float32, schedules.peak_tokens(steps), "cpu", page_size=kt.page_size(name))
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


@pytest.mark.parametrize("name", ["P", "Q", "R", "Z"])
@pytest.mark.parametrize("schedule", ["decode_tail", "portions", "mixed"])
def test_host_logic_against_plain(tmp_path, name, schedule):
    """More requests than state slots, a pool that makes pages go round, portions down to two tokens."""
    folder = kt.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    reqs = {f"r{i}": kt.random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate([1, 9, 34, 21, 17, 40])}
    steps = getattr(schedules, schedule)(reqs, tail=5) if schedule != "portions" else schedules.portions(reqs)
    got = _replay_cpu(folder, name, steps)
    expected = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    bad = schedules.first_bad(got, expected, 2e-4)
    assert bad is None, f"first wrong place (request, position, error): {bad}"


def test_the_plain_functions_agree_with_closed_forms():
    """The oracle against itself: the token-by-token scan equals the sum it stands for, and one score map
    that sees a single key returns that key's value."""
    g = torch.Generator().manual_seed(0)
    T, D, V, lam = 9, 5, 3, 0.8
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (D, D, V))
    out, S = plain.decayed_state_scan(q, k, v, lam)
    for t in range(T):
        want = sum(lam ** (t - j) * float(q[t] @ k[j]) * v[j] for j in range(t + 1))
        assert torch.allclose(out[t], want, atol=1e-12)
    half, S_half = plain.decayed_state_scan(q[:4], k[:4], v[:4], lam)
    rest, S_end = plain.decayed_state_scan(q[4:], k[4:], v[4:], lam, S_half)
    assert torch.allclose(torch.cat([half, rest]), out, atol=1e-12) and torch.allclose(S_end, S, atol=1e-12)
    o = plain.two_map_head(q[:1], k[:1], q[:1], k[:1], v[:1], 0.3, 0.25, 0.0, 2.0)
    assert torch.allclose(o, 2.0 * plain.rms(0.75 * v[:1], 0.0), atol=1e-12)
