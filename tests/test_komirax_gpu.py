"""Komirax through the engine on the GPU against the plain whole-sequence model: the same requests whole,
with their last tokens decoded one by one, in portions down to two tokens, and mixed with other requests
in a pool so small that pages and state slots are used again; in 32-bit and in bfloat16; captured steps;
greedy generation through the public entry points and the scheduler; ``bin/trace_run`` as a user starts it."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import komirax_tiny as kt
from tests import plain_komirax as plain
from tests import schedules

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"Z": [4, 40, 19, 70, 33, 8], "P": [5, 17, 33, 70, 41, 64], "Q": [1, 9, 40, 70, 97, 33], "R": [3, 50, 77, 120, 64, 31],
           "S": [2, 130, 200, 70, 257, 64]}
F32_REL = 2e-5          # of the largest expected logit of the request
BF16_REL = 3e-2
# A token whose router logits leave less than this between the last expert chosen and the first left out is a
# close call: bfloat16 may send it elsewhere than the 32-bit plain model, which moves its logits (and, a little,
# those of later tokens) by any amount.  Such positions are not held to the bfloat16 bound; the rest are.
CLOSE_CALL = 0.12


def requests_for(name, folder):
    cfg, _ = plain.read_folder(folder)
    return {f"r{i}": kt.random_ids(n, cfg["vocab"], 100 + i) for i, n in enumerate(LENGTHS[name])}


def expected_logits(folder, reqs, close=None):
    """``close``: a dict that receives, per request, the positions whose routing is a close call."""
    cfg, w = plain.read_folder(folder)
    out = {}
    for rid, toks in reqs.items():
        margins = []
        out[rid] = plain.forward(cfg, w, toks, margins=margins).numpy()
        if close is not None:
            least = torch.stack(margins).min(0).values if margins else torch.full((len(toks),), float("inf"))
            close[rid] = set(np.nonzero((least < CLOSE_CALL).numpy())[0].tolist())
    return out


def check(got, expected, dtype, close=None):
    """Every position within the bound; in bfloat16 but for the close calls of the routers (fewer than half of
    all positions).  A token that went to another expert also leaves other keys, values and state behind: in
    these tiny models with their short contexts that moves every later position of the request, so positions
    after a request's first close call get ten times the bound; those before it, and everything in float32,
    the bound itself."""
    rel = F32_REL if dtype == "float32" else BF16_REL
    total = skipped = 0
    for rid, rows in got.items():
        bound = rel * float(np.abs(expected[rid]).max())
        calls = (close or {}).get(rid, set()) if dtype != "float32" else set()
        first = min(calls) if calls else None
        for pos in sorted(rows):
            total += 1
            if pos in calls:
                skipped += 1
                continue
            err = float(np.abs(rows[pos] - expected[rid][pos]).max())
            limit = bound * (10.0 if first is not None and pos > first else 1.0)
            assert err <= limit, f"first wrong place (request, position, error / bound): {(rid, pos, err / bound)}"
    assert skipped <= 0.5 * total


def replay(folder, name, steps, dtype, graphs=(), portions=(), page=None):
    from turingserve_b200 import kernels
    from turingserve_b200.engine.replay import Replayer
    kernels.use(None)
    rp = Replayer(folder, getattr(torch, dtype), schedules.peak_tokens(steps), "cuda", page_size=page or kt.page_size(name),
                  graph_batch_sizes=graphs, graph_portion_sizes=portions)
    outs = {}
    with torch.inference_mode():
        for s in steps:
            o = rp.step(s)
            if o is not None:
                outs[s["step"]] = o
            rp.cache.check()
    assert not rp.cache.live
    return schedules.collect(steps, outs), rp


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S", "Z"])
@pytest.mark.parametrize("schedule", ["whole", "decode_tail", "portions", "mixed"])
def test_schedules_match_plain(tmp_path, name, schedule, dtype):
    folder = kt.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    steps = getattr(schedules, schedule)(reqs)
    got, _ = replay(folder, name, steps, dtype)
    assert sum(len(v) for v in got.values()) == sum(len(t) for t in reqs.values())
    close = {}
    check(got, expected_logits(folder, reqs, close), dtype, close)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "S"])
def test_captured_steps_match_plain(tmp_path, name, dtype):
    """Single-token steps replayed from captured graphs of 1, 2 and 4 rows (3 live requests: a padding row that
    points at the null state slot and the null page), and steps of decoding requests beside one 16-token portion
    from graphs of (rows, portion): the state slots, the block tables and the routing all come from device
    arrays, so one capture serves every later step of its shape."""
    folder = kt.make_tiny_folder(name, tmp_path)
    reqs = requests_for(name, folder)
    close = {}
    expected = expected_logits(folder, reqs, close)
    got, rp = replay(folder, name, schedules.batched_tail(reqs), dtype, graphs=(1, 2, 4))
    assert rp.runner._graphs, "no step was captured"
    check(got, expected, dtype, close)
    served = schedules.served(reqs)
    got, rp = replay(folder, name, served, dtype, graphs=(1, 2, 4), portions=(16,))
    assert any(k[1] == 16 for k in rp.runner._graphs), "no step with a portion was captured"
    check(got, expected, dtype, close)


def test_results_do_not_depend_on_batch_mates_or_pages(tmp_path):
    """float32: a request alone in a fresh pool and the same request among others in a shuffled pool with other
    page sizes give the same logits to the last bits that the order of sums leaves."""
    folder = kt.make_tiny_folder("P", tmp_path)
    reqs = requests_for("P", folder)
    alone, _ = replay(folder, "P", schedules.whole(reqs), "float32", page=64)
    among, _ = replay(folder, "P", schedules.mixed(reqs, seed=3), "float32", page=8)
    for rid in reqs:
        for pos, row in alone[rid].items():
            assert float(np.abs(row - among[rid][pos]).max()) <= 2e-5 * float(np.abs(row).max()), (rid, pos)


def engine(folder, dtype="float32", **kw):
    from turingserve_b200 import EngineConfig, LLMEngine, kernels
    kernels.use(None)
    opts = dict(num_blocks=200, max_num_seqs=8, max_num_batched_tokens=64, block_size=16, max_model_len=512)
    opts.update(kw)
    return LLMEngine.from_config(EngineConfig(model=folder, dtype=dtype, **opts))


def greedy(n):
    from turingserve_b200 import SamplingParams
    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


def tokens_are_best(cfg, w, prompt, tokens, slack):
    ids = list(prompt)
    for tok in tokens:
        lg = plain.forward(cfg, w, ids)[-1]
        assert lg[tok] >= lg.max() - slack * lg.abs().max(), (len(ids), tok, int(lg.argmax()))
        ids.append(tok)


@pytest.mark.parametrize("name", ["P", "Q", "R", "Z"])
def test_greedy_generation_float32_equals_plain(tmp_path, name):
    """Through LLMEngine.generate: the scheduler cuts the prompts into portions of at most 24 tokens beside
    the decoding requests; more requests than fit at once."""
    folder = kt.make_tiny_folder(name, tmp_path)
    cfg, w = plain.read_folder(folder)
    prompts = [kt.random_ids(n, cfg["vocab"], 20 + n) for n in (5, 17, 33, 1, 50)]
    eng = engine(folder, block_size=kt.page_size(name), max_num_batched_tokens=24, max_num_seqs=3)
    outs = eng.generate(prompts, greedy(8))
    for p, o in zip(prompts, outs):
        tokens_are_best(cfg, w, p, o.token_ids, 1e-5)
        assert o.finish_reason == "length" and len(o.token_ids) == 8 and o.prompt_tokens == len(p)
    assert not eng.cache.live and (not eng.cache.groups or eng.cache.min_free() == eng.cache.num_pages - 1)


def test_entry_point_and_long_decoding_from_the_first_token(tmp_path):
    """generate_greedy from a one-token prompt: 150 tokens decoded one by one through captured graphs, every one
    the plain model's choice (the state of the linear layers is carried 150 times)."""
    from turingserve_b200 import generate_greedy
    folder = kt.make_tiny_folder("R", tmp_path)
    cfg, w = plain.read_folder(folder)
    toks = generate_greedy(folder, [7], 150, dtype="float32", num_blocks=40, max_num_seqs=2, block_size=32, max_model_len=256)
    assert len(toks) == 150
    tokens_are_best(cfg, w, [7], toks, 1e-5)


def test_graphs_look_ahead_and_preemption_do_not_change_tokens(tmp_path):
    """bfloat16: graphs on or off, the next step launched ahead or not, and a pool so small that requests are
    preempted and recomputed (their state slot zeroed again): the same tokens."""
    from turingserve_b200 import SamplingParams
    folder = kt.make_tiny_folder("P", tmp_path)
    cfg, _ = plain.read_folder(folder)
    prompts = [kt.random_ids(n, cfg["vocab"], 40 + n) for n in (7, 21, 2, 50, 11, 33, 5)]
    params = [SamplingParams(temperature=0.0, max_tokens=m, ignore_eos=True) for m in (20, 3, 31, 9, 14, 1, 26)]
    runs = {}
    for graphs, ahead, pages in ((False, False, 200), (True, True, 200), (True, False, 200), (False, True, 200), (True, True, 14)):
        eng = engine(folder, "bfloat16", cuda_graphs=graphs, async_decode=ahead, block_size=8, max_num_seqs=8,
                     graph_batch_sizes=(1, 2, 4, 8), max_num_batched_tokens=32, num_blocks=pages)
        runs[(graphs, ahead, pages)] = [o.token_ids for o in eng.generate(prompts, params)]
        assert not eng.cache.live
    base = runs[(False, False, 200)]
    assert [len(t) for t in base] == [20, 3, 31, 9, 14, 1, 26]
    for key, got in runs.items():
        assert got == base, key


def test_trace_run_as_a_subprocess(tmp_path):
    folder = kt.make_tiny_folder("Q", tmp_path)
    reqs = requests_for("Q", folder)
    steps = schedules.mixed(reqs, seed=5)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(schedules.peak_tokens(steps)), "--block-size", "16"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    cfg, _ = plain.read_folder(folder)
    outs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for s in steps
            if any(e["want"] for e in s["entries"])}
    check(schedules.collect(steps, outs), expected_logits(folder, reqs), "float32")


def test_command_line_generates_the_plain_models_tokens(tmp_path):
    """``python -m turingserve_b200.cli generate`` on a Komirax folder: config.json alone chooses the model class;
    a stop token ends the request where the plain model's own continuation has it."""
    import turingserve_b200
    folder = kt.make_tiny_folder("P", tmp_path)
    cfg, w = plain.read_folder(folder)
    prompt = kt.random_ids(6, cfg["vocab"], 12)
    want = plain.greedy(cfg, w, prompt, 6)
    r = subprocess.run([sys.executable, "-m", "turingserve_b200.cli", "generate", "--model", folder, "--dtype", "float32",
                        "--num-blocks", "32", "--max-num-seqs", "2", "--max-model-len", "128", "--prompt-ids",
                        ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0", "--ignore-eos"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["token_ids"] == want
    cut = next((i for i, t in enumerate(want) if t not in want[:i] and i > 0), None)
    if cut is not None:
        stopped = turingserve_b200.generate_greedy(folder, prompt, 6, eos_ids=(want[cut],), dtype="float32", num_blocks=32,
                                                   max_model_len=128)
        assert stopped == want[:cut + 1]
