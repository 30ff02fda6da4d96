"""Each Komirax mechanism's kernels alone on the GPU against the plain functions of
``tests/plain_komirax.py``: sizes that are no powers of two, values that a real configuration makes
equal made different, and inputs built so that one wrong key, state or expert shows."""

from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

from tests import plain_komirax as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def ops():
    from turingserve_b200 import kernels
    kernels.use(None)
    return kernels.ops()


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# -- the stream norm, the gated norm, the activations ---------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [48, 200, 1030])
def test_stream_norm_adds_then_norms(ops, dtype, hidden):
    g = torch.Generator(device=DEV).manual_seed(hidden)
    T, eps = 7, 1e-5
    a, b = (torch.randn(T, hidden, generator=g, device=DEV).to(dtype) * 3 for _ in range(2))
    w = (1 + 0.2 * torch.randn(hidden, generator=g, device=DEV)).to(dtype)
    stream = torch.full((T, hidden), 99.0, device=DEV)
    out = torch.empty(T, hidden, dtype=dtype, device=DEV)
    ops.rmsnorm_stream(out, stream, a, None, w, eps, first=True)                   # starts the stream: 99 is not read
    assert torch.equal(stream, a.float())
    assert torch.allclose(out.float(), plain.rms(a.float(), eps) * w.float(), **tol(dtype))
    ops.rmsnorm_stream(out, stream, b, a, w, eps)                                    # two pending tensors
    want = a.float() + b.float() + a.float()
    assert torch.allclose(stream, want, atol=1e-5)
    assert torch.allclose(out.float(), plain.rms(want, eps) * w.float(), **tol(dtype))
    tiny = torch.full((T, hidden), 1e-4, device=DEV).to(dtype)                       # eps sits inside the root
    ops.rmsnorm_stream(out, stream, tiny, None, w, 1e-2, first=True)
    assert torch.allclose(out.float(), tiny.float() / math.sqrt(float(tiny[0, 0]) ** 2 + 1e-2) * w.float(), rtol=2e-2, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_norm_and_activations(ops, dtype):
    g = torch.Generator(device=DEV).manual_seed(3)
    T, n = 5, 72
    x = torch.randn(T, n, generator=g, device=DEV) * 4
    wide = torch.randn(T, 3 * n, generator=g, device=DEV).to(dtype)
    w = (1 + 0.2 * torch.randn(n, generator=g, device=DEV)).to(dtype)
    out = torch.empty(T, n, dtype=dtype, device=DEV)
    ops.gated_rmsnorm(out, x, wide[:, 2 * n:], w, 1e-6)
    want = plain.rms(x, 1e-6) * w.float() * torch.sigmoid(wide[:, 2 * n:].float())
    assert torch.allclose(out.float(), want, **tol(dtype))
    z = torch.linspace(-6, 6, 1001, device=DEV).to(dtype)
    for kind, f in (("gelu_tanh", lambda t: plain.gelu_tanh(t)), ("relu2", lambda t: torch.relu(t) ** 2), ("silu", F.silu)):
        y = torch.empty_like(z)
        ops.activation(y, z, kind)
        assert torch.allclose(y.float(), f(z.float()), **tol(dtype)), kind


# -- the decaying state -----------------------------------------------------------------------------------------
def run_lightning(ops, proj, state, decay, cuts, slots, H, D, V):
    """The rows of ``proj`` belong to len(slots) requests of equal length; ``cuts`` are the step sizes."""
    n_req, T = len(slots), proj.shape[0] // len(slots)
    out = torch.empty(proj.shape[0], H * V, device=DEV)
    at = 0
    for c in cuts:
        rows = torch.cat([torch.arange(r * T + at, r * T + at + c) for r in range(n_req)]).to(DEV)
        step = SimpleNamespace(q_start=i32([i * c for i in range(n_req + 1)]), state_slots=i32(slots), num_requests=n_req)
        o = torch.empty(len(rows), H * V, device=DEV)
        ops.lightning(o, proj[rows].contiguous(), state, decay, step, H, D, V)
        out[rows] = o
        at += c
    assert at == T
    return out


def plain_lightning(proj, decay, H, D, V, dtype):
    act = lambda t: F.silu(t.float()).to(dtype).float().cpu()
    T = proj.shape[0]
    q, k = act(proj[:, :H * D]).view(T, H, D), act(proj[:, H * D:2 * H * D]).view(T, H, D)
    v = act(proj[:, 2 * H * D:2 * H * D + H * V]).view(T, H, V)
    outs, states = zip(*[plain.decayed_state_scan(q[:, h].double(), k[:, h].double(), v[:, h].double(), float(decay[h]))
                         for h in range(H)])
    return torch.stack(outs, 1).reshape(T, H * V).float(), torch.stack(states).float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,V", [(3, 8, 24), (2, 48, 16), (1, 64, 40), (2, 256, 256), (2, 12, 20), (3, 5, 33)])
def test_state_scan_whole_in_portions_and_token_by_token(ops, dtype, H, D, V):
    """The same tokens as one portion, as portions down to two tokens and one, and one by one: the same
    outputs and the same state; two requests in one launch with slots that are not their batch rows.  Sizes
    that are multiples of 8 (rows fetched by 16-byte asynchronous copies), sizes that are not (plain loads), a
    state of 256 x 256 (32 row parts a block)."""
    g = torch.Generator(device=DEV).manual_seed(D + V)
    T = 37
    decay = torch.tensor([0.6, 0.97, 1.0][:H], device=DEV)
    width = 2 * H * D + 2 * H * V + 5
    proj = (torch.randn(2 * T, width, generator=g, device=DEV)).to(dtype)
    want = [plain_lightning(proj[r * T:(r + 1) * T], decay.tolist(), H, D, V, dtype) for r in range(2)]
    for cuts in ([T], [16, 2, 1, 17, 1], [1] * T, [36, 1]):
        state = torch.zeros(5, H, D, V, device=DEV)
        state[1].fill_(7.0)                                                          # a slot nobody uses stays as it is
        out = run_lightning(ops, proj, state, decay, cuts, [3, 0], H, D, V)
        for r, slot in enumerate([3, 0]):
            # (bfloat16: the kernel's own exponential may round one activation the other way)
            rel = 1e-5 if dtype == torch.float32 else 2e-3
            assert torch.allclose(out[r * T:(r + 1) * T].cpu(), want[r][0], rtol=10 * rel, atol=rel * float(want[r][0].abs().max())), (cuts, r)
            assert torch.allclose(state[slot].cpu(), want[r][1], rtol=10 * rel, atol=rel * float(want[r][1].abs().max()))
        assert float((state[1] - 7.0).abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


def test_state_scan_keeps_a_far_token_and_forgets_with_its_decay(ops):
    """Head 0 does not decay: a key 400 tokens back, the only one the last query is aligned with, comes back
    whole.  Head 1 halves its state every token: the same key is gone, its neighbour one token back is not."""
    H, D, V, T = 2, 16, 8, 401
    proj = torch.full((T, 2 * H * D + 2 * H * V), -30.0, device=DEV)                  # silu(-30) = 0
    def put(row, col, width, value):
        proj[row, col:col + width] = value
    for h in range(H):
        put(0, H * D + h * D, 1, 5.0)                      # token 0: key along axis 0, value 5 * ones
        put(0, 2 * H * D + h * V, V, 5.0)
        put(T - 2, H * D + h * D + 1, 1, 5.0)              # token T-2: key along axis 1, value 3 * ones
        put(T - 2, 2 * H * D + h * V, V, 3.0)
        put(T - 1, h * D, 2, 5.0)                          # the last query looks along axes 0 and 1
    decay = torch.tensor([1.0, 0.5], device=DEV)
    state = torch.zeros(1, H, D, V, device=DEV)
    out = run_lightning(ops, proj, state, decay, [300, 99, 1, 1], [0], H, D, V)
    s5, s3 = float(F.silu(torch.tensor(5.0))), float(F.silu(torch.tensor(3.0)))
    last = out[-1].view(H, V).cpu()
    assert torch.allclose(last[0], torch.full((V,), s5 * s5 * s5 + s5 * s5 * s3), rtol=1e-5)
    assert torch.allclose(last[1], torch.full((V,), 0.5 * s5 * s5 * s3), rtol=1e-5)


def test_state_scan_long_decoding(ops):
    H, D, V, T = 2, 32, 32, 600
    g = torch.Generator(device=DEV).manual_seed(9)
    proj = torch.randn(T, 2 * H * D + 2 * H * V, generator=g, device=DEV)
    decay = torch.tensor([0.999, 0.9], device=DEV)
    want, _ = plain_lightning(proj, decay.tolist(), H, D, V, torch.float32)
    out = run_lightning(ops, proj, torch.zeros(1, H, D, V, device=DEV), decay, [1] * T, [0], H, D, V)
    assert torch.allclose(out.cpu(), want, rtol=2e-4, atol=2e-4 * float(want.abs().max()))


# -- the two-map attention --------------------------------------------------------------------------------------
def paged(ops, q, k, v, lens_new, H, G, D, V, page, scale, lam, eps, out_scale, dtype, shuffle_seed=0):
    """q [T, H, 2, D], k [T, G, 2, D], v [T, G, V]: the tokens of len(lens_new) requests one after the other;
    request r brings lens_new[r][1] new tokens after lens_new[r][0] cached ones.  Everything goes through
    kv_write_pair into a shuffled pool, the cached part in an earlier call."""
    total_pages = sum(-(-(a + b) // page) for a, b in lens_new) + 1
    perm = torch.randperm(total_pages - 1, generator=torch.Generator().manual_seed(shuffle_seed)) + 1
    kc = torch.zeros(total_pages, G, page, 2 * D, dtype=dtype, device=DEV)
    vc = torch.zeros(total_pages, G, page, V, dtype=dtype, device=DEV)
    tables, at_page, at_tok = [], 0, 0
    width = max(-(-(a + b) // page) for a, b in lens_new)
    spans = []
    for a, b in lens_new:
        n = -(-(a + b) // page)
        t = perm[at_page:at_page + n].tolist()
        tables.append(t + [0] * (width - n))
        at_page += n
        spans.append((at_tok, a, b, t))
        at_tok += a + b
    proj = torch.cat([q.reshape(q.shape[0], -1), k.reshape(k.shape[0], -1), v.reshape(v.shape[0], -1)], 1).to(dtype).contiguous()
    qd, kd = H * 2 * D, G * 2 * D
    def slots_of(first, count, table, base):
        pos = torch.arange(first, first + count)
        return (torch.tensor(table)[pos // page] * page + pos % page).to(torch.int32), torch.arange(base + first, base + first + count)
    old = [slots_of(0, a, t, base) for base, a, b, t in spans if a]
    if old:
        rows = torch.cat([r for _, r in old]).to(DEV)
        ops.kv_write_pair(proj[rows].contiguous(), qd, qd + kd, kc, vc, torch.cat([s for s, _ in old]).to(DEV), G, 2 * D, V, page)
    new = [slots_of(a, b, t, base) for base, a, b, t in spans]
    rows = torch.cat([r for _, r in new]).to(DEV)
    slots = torch.cat([s for s, _ in new]).to(DEV)
    step_proj = proj[rows].contiguous()
    ops.kv_write_pair(step_proj, qd, qd + kd, kc, vc, slots, G, 2 * D, V, page)
    qs = [0]
    for a, b in lens_new:
        qs.append(qs[-1] + b)
    step = SimpleNamespace(q_start=i32(qs), seq_lens=i32([a + b for a, b in lens_new]), num_requests=len(lens_new),
                           max_q_len=max(b for _, b in lens_new))
    out = torch.empty(len(rows), H * V, dtype=dtype, device=DEV)
    ops.attention_diff(out, step_proj, kc, vc, i32(tables), step, H, G, D, V, page, scale, lam, eps, out_scale)
    return out, rows.cpu()


def plain_two_maps(q, k, v, lens_new, H, G, D, V, scale, lam, eps, out_scale, dtype):
    rd = lambda t: t.to(dtype).double().cpu()
    q, k, v = rd(q), rd(k), rd(v)
    outs, base = [], 0
    for a, b in lens_new:
        n = a + b
        o = torch.zeros(b, H, V, dtype=torch.float64)
        for h in range(H):
            g = h // (H // G)
            o[:, h] = plain.two_map_head(q[base + a:base + n, h, 0], k[base:base + n, g, 0], q[base + a:base + n, h, 1],
                                         k[base:base + n, g, 1], v[base:base + n, g], scale, lam, eps, out_scale, first_pos=a)
        outs.append(o.reshape(b, H * V))
        base += n
    return torch.cat(outs).float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V,page", [(4, 2, 16, 24, 8), (6, 6, 8, 40, 16), (3, 1, 40, 72, 4), (2, 2, 128, 256, 32),
                                          (4, 2, 64, 128, 64), (4, 4, 32, 64, 16), (6, 2, 32, 128, 8), (2, 1, 64, 64, 32)])
def test_two_map_attention_portions_and_single_tokens(ops, dtype, H, G, D, V, page):
    """A batch of unequal requests: a whole prompt, a portion after a cached part that ends in the middle of a
    page, single tokens after 1, page - 1, page and many cached tokens; against every head computed alone."""
    g = torch.Generator(device=DEV).manual_seed(H * D)
    lens = [(0, 33), (page + 3, 18), (1, 1), (page - 1, 1), (page, 1), (3 * page + 5, 1), (0, 1), (2 * page, 2), (5, 150),
            (300, 1)]
    T = sum(a + b for a, b in lens)
    q = torch.randn(T, H, 2, D, generator=g, device=DEV) * 2
    k = torch.randn(T, G, 2, D, generator=g, device=DEV) * 2
    v = torch.randn(T, G, V, generator=g, device=DEV)
    scale, lam, eps, out_scale = 0.21, 0.37, 1e-5, 0.45
    out, _ = paged(ops, q, k, v, lens, H, G, D, V, page, scale, lam, eps, out_scale, dtype)
    want = plain_two_maps(q, k, v, lens, H, G, D, V, scale, lam, eps, out_scale, dtype)
    t = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    assert torch.allclose(out.float().cpu(), want, **t)


@pytest.mark.parametrize("D,V,dtype", [(16, 8, torch.float32), (32, 64, torch.bfloat16), (64, 128, torch.bfloat16)])
@pytest.mark.parametrize("new", [1, 40])
def test_two_map_attention_finds_one_far_key_and_stops_at_the_causal_edge(ops, new, D, V, dtype):
    """Among 700 cached keys one (at a page's last place, then at a page's first) answers the last query's map 1
    with a score far above the rest: the output is that key's value, normed.  The same key placed one token
    AFTER a query must not reach it.  Map 2 answers another key; with lam = 1 and equal values the head's output
    before the norm is their difference."""
    H, G, page = 2, 1, 16
    atol = 1e-4 if dtype == torch.float32 else 3e-2
    for needle in (page * 20 - 1, page * 20):
        cached = 700
        T = cached + new
        g = torch.Generator(device=DEV).manual_seed(needle)
        q = torch.randn(T, H, 2, D, generator=g, device=DEV) * 0.1
        k = torch.randn(T, G, 2, D, generator=g, device=DEV) * 0.1
        v = torch.randn(T, G, V, generator=g, device=DEV)
        q[-1, :, 0, 3] = 30.0
        k[needle, 0, 0, 3] = 30.0                               # map 1 of the last query: key `needle`
        q[-1, :, 1, 5] = 30.0
        k[needle + 7, 0, 1, 5] = 30.0                            # map 2: key needle + 7
        if new > 1:
            q[-3, :, 0, 9] = 30.0                                # a query two places before the end, on an axis of its own,
            k[needle, 0, 0, 9] = 30.0                            # answered by the same far key ...
            k[T - 2, 0, 0, 9] = 60.0                             # ... must not see the louder key one place after it
        out, _ = paged(ops, q, k, v, [(cached, new)], H, G, D, V, page, 1.0, 1.0, 0.0, 1.0, dtype, shuffle_seed=needle)
        diff = (v[needle, 0] - v[needle + 7, 0]).cpu()
        want = diff / diff.pow(2).mean().sqrt()
        assert torch.allclose(out[-1].view(H, V)[0].float().cpu(), want, atol=atol), needle
        if new > 1:
            full = plain_two_maps(q, k, v, [(cached, new)], H, G, D, V, 1.0, 1.0, 0.0, 1.0, dtype)
            # (rows whose two maps are both nearly uniform subtract two nearly equal averages: after the norm their
            # bfloat16 noise is of order one, so in bfloat16 only the rows with a loud key are compared)
            rows = slice(None) if dtype == torch.float32 else [-3, -1]
            assert torch.allclose(out.float().cpu()[rows], full[rows], atol=2 * atol)
            seen = out[-3].view(H, V)[0].float().cpu()                   # that query's map 1 answers `needle` too, not T - 2
            leak = v[T - 2, 0].cpu()
            assert not torch.allclose(seen, leak / leak.pow(2).mean().sqrt(), atol=0.2)


def test_kv_write_pair_skips_rows_without_a_slot(ops):
    G, DK, DV, page = 2, 6, 10, 4
    proj = torch.randn(5, 3 + G * DK + G * DV, device=DEV)
    kc, vc = torch.zeros(3, G, page, DK, device=DEV), torch.zeros(3, G, page, DV, device=DEV)
    ops.kv_write_pair(proj, 3, 3 + G * DK, kc, vc, i32([4, -1, 11, 5, -1]), G, DK, DV, page)
    for row, slot in ((0, 4), (2, 11), (3, 5)):
        assert torch.equal(kc[slot // page, :, slot % page], proj[row, 3:3 + G * DK].view(G, DK))
        assert torch.equal(vc[slot // page, :, slot % page], proj[row, 3 + G * DK:].view(G, DV))
    assert int((kc != 0).sum()) == 3 * G * DK and int((vc != 0).sum()) == 3 * G * DV


# -- the routed feed-forward --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,K", [(5, 2, 64), (3, 3, 40), (40, 6, 96), (2, 1, 200)])
def test_router_picks_the_largest_scores(ops, dtype, E, top, K):
    g = torch.Generator(device=DEV).manual_seed(E)
    T = 33
    x = torch.randn(T, K, generator=g, device=DEV).to(dtype)
    wr = torch.randn(E, K, generator=g, device=DEV) * 0.1          # logits of a few units: no score saturates
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    ops.router_topk(idx, wts, x, wr, False, False)
    experts, weights = plain.route(x.float().cpu(), wr.cpu(), top)
    assert torch.equal(idx.cpu().long(), experts)                    # largest first; random scores do not tie
    assert torch.allclose(wts.cpu(), weights, atol=1e-5)
    ops.router_topk(idx, wts, x, wr, True, True)                     # softmax over all experts, chosen ones renormalised
    p = torch.softmax(F.linear(x.float().cpu(), wr.cpu()), -1).gather(1, experts)
    assert torch.allclose(wts.cpu(), p / p.sum(-1, keepdim=True), atol=1e-5)


def test_router_breaks_ties_towards_the_lower_index(ops):
    x = torch.ones(2, 8, device=DEV)
    wr = torch.zeros(37, 8, device=DEV)
    wr[[4, 20, 36]] = 0.5
    idx = torch.empty(2, 4, dtype=torch.int32, device=DEV)
    wts = torch.empty(2, 4, device=DEV)
    ops.router_topk(idx, wts, x, wr, False, False)
    assert idx.cpu().tolist() == [[4, 20, 36, 0]] * 2
    assert torch.allclose(wts.cpu(), torch.sigmoid(torch.tensor([4.0, 4.0, 4.0, 0.0])).expand(2, 4))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top", [(150, 3, 2), (9, 12, 1), (70, 7, 7), (1, 4, 2)])
def test_grouped_products_and_the_sum_of_choices(ops, dtype, T, E, top):
    """Tokens sorted by expert (groups longer than a row tile, experts nobody chose), up product with the
    weighted input and the squared ReLU, down product, sum over a token's choices: against one token at a time."""
    g = torch.Generator(device=DEV).manual_seed(T)
    K, ff = 48, 40
    x = torch.randn(T, K, generator=g, device=DEV).to(dtype)
    up = (torch.randn(E, ff, K, generator=g, device=DEV) * 0.2).to(dtype)
    down = (torch.randn(E, K, ff, generator=g, device=DEV) * 0.2).to(dtype)
    idx = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(t))[:top] for t in range(T)]).to(torch.int32).to(DEV)
    if E == 12:
        idx.fill_(5)
        idx[0] = 11                                                  # experts 0..4 and 6..10 get nobody
    wts = torch.rand(T, top, generator=g, device=DEV) + 0.25
    for on_input in (True, False):
        offsets, order, place, tiles = ops.moe_align(idx, E)
        counts = torch.bincount(idx.flatten().long().cpu(), minlength=E)
        assert offsets[:E + 1].cpu().tolist() == [0] + counts.cumsum(0).tolist()
        assert sorted(order[:T * top].cpu().tolist()) == list(range(T * top))
        assert torch.equal(order[:T * top][place[:T * top].long()].cpu(), torch.arange(T * top, dtype=torch.int32))
        a = torch.empty(T * top, ff, dtype=dtype, device=DEV)
        ops.grouped_linear(a, x, up, order, wts if on_input else None, offsets, tiles, top, "relu2")
        y = torch.empty(T * top, K, device=DEV)
        ops.grouped_linear(y, a, down, None, None, offsets, tiles, 1)
        out = torch.empty(T, K, dtype=dtype, device=DEV)
        ops.moe_combine(out, y, place, None if on_input else wts, top)
        want = torch.zeros(T, K)
        for t in range(T):
            for r in range(top):
                e, wt = int(idx[t, r]), float(wts[t, r])
                h = x[t].float().cpu()
                h_in = (h * wt).to(dtype).float() if on_input else h
                act = (torch.relu(F.linear(h_in, up[e].float().cpu())) ** 2).to(dtype).float()
                o = F.linear(act, down[e].float().cpu())
                want[t] += o if on_input else wt * o
        t_ = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        assert torch.allclose(out.float().cpu(), want, **t_), on_input


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_part_many_row_path_equals_the_grouped_kernels(ops, dtype, monkeypatch):
    """The routed feed-forward as a part: with every expert's rows launched as a product of their own (what steps
    of many tokens do) and with the grouped kernels (what few tokens and captured steps do), against one token at a
    time; three of six experts, one of them chosen by nobody."""
    from turingserve_b200.config.model_config import RoutedMLPSpec
    from turingserve_b200.parts.base import BuildContext
    from turingserve_b200.parts.routed_mlp import RoutedMLP
    g = torch.Generator(device=DEV).manual_seed(5)
    W, ff, E, top, T = 64, 48, 6, 3, 90
    part = RoutedMLP(RoutedMLPSpec(num_experts=E, top_k=top, intermediate_size=ff), BuildContext(W, dtype, torch.device(DEV), 0))
    t = {"router": torch.randn(E, W, generator=g, device=DEV) * 0.2}
    t["router"][4] = -5.0 * t["router"][0].abs()                       # expert 4 never wins ...
    for e in range(E):
        t[f"e{e}.up"] = (torch.randn(ff, W, generator=g, device=DEV) * 0.2).to(dtype)
        t[f"e{e}.down"] = (torch.randn(W, ff, generator=g, device=DEV) * 0.2).to(dtype)
    part.load(t)
    x = (torch.randn(T, W, generator=g, device=DEV).abs() + 0.1).to(dtype)          # ... on inputs that are all positive
    monkeypatch.setattr(RoutedMLP, "LIBRARY_ROWS", 1)
    by_expert = part.forward(x).float().cpu()
    monkeypatch.setattr(RoutedMLP, "LIBRARY_ROWS", 10 ** 9)
    grouped = part.forward(x).float().cpu()
    w = {f"p.{k}": v.float().cpu() for k, v in t.items()}
    want = plain.routed_ff(x.float().cpu(), w, "p.", {"router": {"experts": E, "top": top}})
    experts, _ = plain.route(x.float().cpu(), w["p.router"], top)
    assert 4 not in experts.unique().tolist()
    # (bfloat16: the plain model rounds neither the weighted input nor the activation; 3 % of the largest output)
    t_ = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2 * float(want.abs().max()))
    assert torch.allclose(grouped, want, **t_) and torch.allclose(by_expert, want, **t_)
    assert torch.allclose(grouped, by_expert, **t_)
