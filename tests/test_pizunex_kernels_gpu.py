"""Each Pizunex mechanism's kernels alone on the GPU against the plain functions of ``tests/plain_pizunex.py``:
sizes that are no powers of two, values that a real configuration makes equal made different, and inputs built
so that one wrong key, state, tap or position shows."""

from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

from tests import plain_pizunex as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def ops():
    from turingserve_b200 import kernels
    kernels.use(None)
    return kernels.ops()


def tol(dtype):
    return dict(rtol=3e-5, atol=3e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# -- the gated delta rule ---------------------------------------------------------------------------------------
def delta_step(n_req, c, slots):
    req = [r for r in range(n_req) for _ in range(c)]
    return SimpleNamespace(q_start=i32([i * c for i in range(n_req + 1)]), state_slots=i32(slots), num_requests=n_req,
                           token_request=i32(req), max_q_len=c)


def run_delta(ops, proj, conv_w, a_log, dt, state, cuts, slots, H, G, D, V, taps):
    """The rows of ``proj`` belong to len(slots) requests of equal length; ``cuts`` are the step sizes."""
    n_req, T = len(slots), proj.shape[0] // len(slots)
    C = 2 * G * D + H * V
    out = torch.empty(proj.shape[0], H * V, device=DEV)
    at = 0
    for c in cuts:
        rows = torch.cat([torch.arange(r * T + at, r * T + at + c) for r in range(n_req)]).to(DEV)
        step = delta_step(n_req, c, slots)
        p = proj[rows].contiguous()
        ready = torch.empty(len(rows), C + 2 * H + G, device=DEV)
        ops.delta_prepare(ready, p, conv_w, a_log, dt, state, step, H, G, D, V, taps, 1e-6)
        o = torch.empty(len(rows), H * V, device=DEV)
        ops.delta_scan(o, ready, p, state, step, H, G, D, V, taps)
        out[rows] = o
        at += c
    assert at == T
    return out


def plain_delta(proj, conv_w, a_log, dt, H, G, D, V):
    """One request's rows through the plain functions, in 64-bit."""
    p = proj.double().cpu()
    T = p.shape[0]
    qk, hv = G * D, H * V
    C = 2 * qk + hv
    y = F.silu(plain.short_filter(p[:, :C], conv_w.double().cpu()))
    q = plain.unit(y[:, :qk].view(T, G, D)) * D ** -0.5
    k = plain.unit(y[:, qk:2 * qk].view(T, G, D))
    v = y[:, 2 * qk:].view(T, H, V)
    b = torch.sigmoid(p[:, C + hv:C + hv + H])
    g = torch.exp(-torch.exp(a_log.double().cpu()) * F.softplus(p[:, C + hv + H:C + hv + 2 * H] + dt.double().cpu()))
    per = H // G
    outs, states = zip(*[plain.delta_scan(q[:, h // per], k[:, h // per], v[:, h], g[:, h], b[:, h]) for h in range(H)])
    return torch.stack(outs, 1).reshape(T, hv).float(), torch.stack(states).float(), p[:, :C].float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,V,taps", [(4, 2, 16, 8, 3), (2, 1, 24, 20, 2), (2, 2, 128, 64, 4), (3, 3, 5, 33, 1),
                                          (2, 1, 72, 40, 8), (1, 1, 256, 48, 4), (6, 2, 64, 16, 4)])
def test_delta_rule_whole_in_portions_and_token_by_token(ops, dtype, H, G, D, V, taps):
    """The same tokens as one portion, as portions down to two tokens and one, and one by one: the same outputs,
    the same matrix state and the same filter memory; two requests in one launch with slots that are not their
    batch rows.  Keys of 16 rows a lane and of 32, widths that are no multiple of 4 (no 16-byte copies), fewer
    query/key heads than heads, one tap (no memory) to eight."""
    g = torch.Generator(device=DEV).manual_seed(D + V)
    T = 37
    C = 2 * G * D + H * V
    proj = (torch.randn(2 * T, C + H * V + 2 * H, generator=g, device=DEV) * 2).to(dtype)
    conv_w = torch.randn(C, taps, generator=g, device=DEV) * 0.6
    a_log, dt = torch.randn(H, generator=g, device=DEV), torch.randn(H, generator=g, device=DEV)
    want = [plain_delta(proj[r * T:(r + 1) * T], conv_w, a_log, dt, H, G, D, V) for r in range(2)]
    width = H * D * V + (taps - 1) * C
    for cuts in ([T], [16, 2, 1, 17, 1], [1] * T, [36, 1], [2, 3, 32]):
        state = torch.zeros(5, width, device=DEV)
        state[1].fill_(7.0)                                                          # a slot nobody uses stays as it is
        out = run_delta(ops, proj, conv_w, a_log, dt, state, cuts, [3, 0], H, G, D, V, taps)
        for r, slot in enumerate([3, 0]):
            o, S, raw = want[r]
            assert torch.allclose(out[r * T:(r + 1) * T].cpu(), o, rtol=2e-4, atol=2e-5), (cuts, r)
            assert torch.allclose(state[slot, :H * D * V].cpu().view(H, D, V), S, rtol=2e-4, atol=2e-5), (cuts, r)
            if taps > 1:
                assert torch.equal(state[slot, H * D * V:].cpu().view(taps - 1, C), raw[T - (taps - 1):]), (cuts, r)
        assert float((state[1] - 7.0).abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


def test_delta_rule_keeps_a_far_write_and_replaces_a_repeated_key(ops):
    """Built inputs: with g = 1 (no decay) and beta = 1 a key written 500 tokens back is read out whole by the
    same query, and writing the same key again replaces its value instead of adding to it; with a decay of one
    half a token the far write is gone."""
    H, G, D, V, taps, T = 2, 2, 8, 4, 1, 520
    C = 2 * G * D + H * V
    proj = torch.zeros(T, C + H * V + 2 * H, device=DEV)
    big = 30.0                                                   # silu(30) = 30: unit vectors after the norm
    for h in range(G):
        proj[:, G * D + h * D + 1] = big                         # every token's key: axis 1 ...
        proj[3, G * D + h * D + 1] = 0.0
        proj[3, G * D + h * D + 5] = big                         # ... but token 3 writes on axis 5
        proj[T - 1, h * D + 5] = big                             # the last query asks for axis 5
        proj[T - 1, G * D + h * D + 1] = 0.0
        proj[T - 1, G * D + h * D + 2] = big
    proj[:, 2 * G * D:C] = 1.0
    proj[3, 2 * G * D:C] = torch.arange(1.0, 1.0 + H * V, device=DEV)
    proj[:, C + H * V:C + H * V + H] = 40.0                      # beta = 1
    proj[:, C + H * V + H] = -80.0                               # head 0: softplus = 0, g = 1
    proj[:, C + H * V + H + 1] = math.log(math.e ** (math.log(2.0)) - 1.0)      # head 1: softplus = ln 2, g = 1/2
    a_log, dt = torch.zeros(H, device=DEV), torch.zeros(H, device=DEV)
    conv_w = torch.ones(C, 1, device=DEV)
    state = torch.zeros(2, H * D * V, device=DEV)
    out = run_delta(ops, proj, conv_w, a_log, dt, state, [T], [1], H, G, D, V, taps)
    v3 = F.silu(torch.arange(1.0, 1.0 + H * V)).view(H, V)
    got = out[T - 1].cpu().view(H, V) * math.sqrt(D)
    assert torch.allclose(got[0], v3[0], rtol=1e-4), got[0]                      # kept whole over 516 tokens
    assert float(got[1].abs().max()) < 1e-20                                       # halved 516 times
    S = state[1].cpu().view(H, D, V)
    assert torch.allclose(S[0, 1], F.silu(torch.ones(V)), rtol=1e-4)             # axis 1 written 518 times: one value, not a sum


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_gated_norm(ops, dtype):
    g = torch.Generator(device=DEV).manual_seed(3)
    T, H, V = 5, 3, 20
    x = torch.randn(T, H * V, generator=g, device=DEV) * 4
    x[:, V:2 * V] *= 50                                                              # a head's scale is its own
    wide = torch.randn(T, 3 * H * V, generator=g, device=DEV).to(dtype)
    w = 1 + 0.3 * torch.randn(V, generator=g, device=DEV)
    out = torch.empty(T, H * V, dtype=dtype, device=DEV)
    ops.head_gated_rmsnorm(out, x, wide[:, H * V:2 * H * V], w, 1e-5, H, V)
    want = plain.rms(x.view(T, H, V), 1e-5) * w * F.silu(wide[:, H * V:2 * H * V].float()).view(T, H, V)
    assert torch.allclose(out.float(), want.reshape(T, H * V), **tol(dtype))


# -- norms, rotation, per-head products ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_norm_slice_and_eps_inside_the_root(ops, dtype):
    g = torch.Generator(device=DEV).manual_seed(5)
    x = (torch.randn(6, 100, generator=g, device=DEV) * 3).to(dtype)
    w = 1 + 0.3 * torch.randn(37, generator=g, device=DEV)
    out = torch.empty(6, 37, dtype=dtype, device=DEV)
    ops.rms_rows(out, x, 41, w, 1e-5)
    assert torch.allclose(out.float(), plain.rms(x[:, 41:78].float(), 1e-5) * w, **tol(dtype))
    tiny = torch.full((2, 37), 1e-4, device=DEV).to(dtype)
    ops.rms_rows(out[:2], tiny, 0, w, 1e-2)
    assert torch.allclose(out[:2].float(), tiny.float() / math.sqrt(float(tiny[0, 0]) ** 2 + 1e-2) * w, rtol=2e-2, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,every", [(4, 2, 16, 5), (3, 3, 10, 1), (2, 1, 72, 64)])
def test_whole_row_norms_temperature_and_cache_rows(ops, dtype, H, G, D, every):
    """The norm runs over ALL heads of a row at once (one head a hundred times larger shrinks the others); the
    temperature steps where floor((p + 1) / every) does; normed keys become keys, raw keys values; slot -1 writes nothing."""
    g = torch.Generator(device=DEV).manual_seed(D)
    T, page, pages = 9, 4, 6
    proj = torch.randn(T, (H + G) * D, generator=g, device=DEV)
    proj[:, :D] *= 100
    proj = proj.to(dtype)
    q_w, k_w = 1 + 0.3 * torch.randn(H * D, generator=g, device=DEV), 1 + 0.3 * torch.randn(G * D, generator=g, device=DEV)
    positions = i32([0, every - 2 if every > 1 else 3, every - 1, every, 2 * every - 1, 3 * every - 1, 50, 1000, 7])
    slots = i32([5, 9, -1, 0, 23, 14, 3, 2, 1])
    k_cache = torch.zeros(pages, G, page, D, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    raw = proj.clone()
    ops.qk_rownorm_write(proj, q_w, k_w, 1e-6, positions, 0.35, every, k_cache, v_cache, slots, H, G, D, page)
    heat = plain.query_heat(positions.double().cpu(), 0.35, every).float().to(DEV)
    want_q = plain.rms(raw[:, :H * D].float(), 1e-6) * q_w * heat[:, None]
    assert torch.allclose(proj[:, :H * D].float(), want_q, **tol(dtype))
    assert torch.equal(proj[:, H * D:], raw[:, H * D:])
    want_k = plain.rms(raw[:, H * D:].float(), 1e-6) * k_w
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert torch.allclose(k_cache[s // page, :, s % page].float().reshape(-1), want_k[t], **tol(dtype))
        assert torch.equal(v_cache[s // page, :, s % page].reshape(-1), raw[t, H * D:])
    assert int((k_cache.float().abs().sum(-1) > 0).sum()) == 8 * G


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,dims,scaling", [(8, 8, (2.5, 16, 4.0, 1.0)), (6, 4, None), (32, 32, (4.0, 64, 16.0, 2.0)), (5, 2, None)])
def test_pair_rotation_and_latent_rows(ops, dtype, R, dims, scaling):
    from turingserve_b200.config.model_config import YarnRotarySpec
    from turingserve_b200.parts.base import BuildContext
    from turingserve_b200.parts.rotary import PairRotaryEncoding
    kw = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else {}
    enc = PairRotaryEncoding(YarnRotarySpec(base=500.0, dims=dims, **kw), BuildContext(8, dtype, torch.device(DEV), 0))
    rot = {"base": 500.0, "dims": dims}
    if scaling:
        rot["scaling"] = kw
    g = torch.Generator(device=DEV).manual_seed(R)
    T, H, D, rank, page = 7, 3, 6, 10, 4
    positions = i32([0, 1, 2, 17, 300, 4095, 5])
    cos, sin = plain.yarn_angles(rot, positions.cpu())
    src = torch.randn(T, H, D + R, generator=g, device=DEV).to(dtype)
    dst = torch.zeros(T, H, rank + R, dtype=dtype, device=DEV)
    ops.rotate_pairs(dst[:, :, rank:], src[:, :, D:], positions, enc.freq, enc.magnitude, enc.dims)
    want = plain.rotate_pairs(src[:, :, D:].double().cpu(), cos, sin).float()
    assert torch.allclose(dst[:, :, rank:].float().cpu(), want, **tol(dtype))
    assert float(dst[:, :, :rank].abs().max()) == 0.0
    proj = torch.randn(T, 4 + rank + R, generator=g, device=DEV).to(dtype)
    w = 1 + 0.3 * torch.randn(rank, generator=g, device=DEV)
    cache = torch.zeros(3, 1, page, rank + R, dtype=dtype, device=DEV)
    slots = i32([4, 0, 11, -1, 7, 6, 1])
    ops.latent_kv_write(proj, 4, w, 1e-6, positions, enc.freq, enc.magnitude, enc.dims, cache, slots, rank, R, page)
    c = (plain.rms(proj[:, 4:4 + rank].float(), 1e-6) * w).cpu()
    kr = plain.rotate_pairs(proj[:, 4 + rank:].double().cpu(), cos, sin).float()
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert torch.allclose(cache[s // page, 0, s % page].float().cpu(), torch.cat([c[t], kr[t]]), **tol(dtype)), t
    assert int((cache.float().abs().sum(-1) > 0).sum()) == 6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 11, 16, 17, 70, 200])
@pytest.mark.parametrize("K,off", [(20, 9), (64, 8), (136, 16)])
def test_per_head_products_over_strided_rows(ops, dtype, T, K, off):
    """Rows that start on 16-byte boundaries and rows that do not; up to 16 rows (the kernel that streams the weights),
    more (tiles, or the vendor's batched product in bfloat16)."""
    g = torch.Generator(device=DEV).manual_seed(T)
    H, N = 3, 37
    wide = torch.randn(T, H, K + off, generator=g, device=DEV).to(dtype)
    w = torch.randn(H, N, K, generator=g, device=DEV).to(dtype)
    out = torch.zeros(T, H, N + 4, dtype=dtype, device=DEV)
    ops.batched_linear(out[:, :, :N], wide[:, :, off:], w)
    want = torch.einsum("thk,hnk->thn", wide[:, :, off:].float(), w.float())
    assert torch.allclose(out[:, :, :N].float(), want, rtol=2e-2 if dtype == torch.bfloat16 else 2e-5, atol=1e-1 if dtype == torch.bfloat16 else 3e-5)
    assert float(out[:, :, N:].abs().max()) == 0.0


# -- the attention with capped scores, distance bias and window -----------------------------------------------------
def paged(rows, page, order=None):
    """rows [T, KVH, D] -> (cache [pages + 1, KVH, page, D], block table row): pages in ``order`` (shuffled pool)."""
    T, KVH, D = rows.shape
    n = -(-T // page)
    order = order or list(range(1, n + 1))
    cache = torch.zeros(max(order) + 1, KVH, page, D, dtype=rows.dtype, device=DEV)
    for j in range(T):
        cache[order[j // page], :, j % page] = rows[j]
    return cache, order


def attention_step(q_lens, seq_lens):
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    return SimpleNamespace(q_start=i32(starts), seq_lens=i32(seq_lens), num_requests=len(q_lens),
                           num_decode=sum(1 for n in q_lens if n == 1), max_q_len=max(q_lens), max_seq_len=max(seq_lens))


def plain_attention(q, k, v, KVH, scale, cap, slopes, window, first_pos):
    """q [Tq, H, Dk] at positions first_pos.., k [Tk, KVH, Dk], v [Tk, KVH, Dv] -> [Tq, H, Dv] in 64-bit."""
    H = q.shape[1]
    outs = []
    for h in range(H):
        s = plain.capped_scores(q[:, h].double().cpu(), k[:, h // (H // KVH)].double().cpu(), scale, cap,
                                float(slopes[h]) if slopes is not None else 0.0, window, first_pos)
        outs.append(torch.softmax(s, -1) @ v[:, h // (H // KVH)].double().cpu())
    return torch.stack(outs, 1).float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KVH,Dk,Dv,page,window,cap,shared", [
    (4, 2, 16, 16, 8, 9, 6.0, False), (6, 6, 8, 8, 4, 33, None, False), (2, 1, 40, 40, 16, 3, 20.0, False),
    (4, 1, 28, 20, 16, None, None, True), (3, 1, 80, 64, 64, None, None, True), (4, 2, 64, 64, 64, 70, 30.0, False),
    (20, 1, 30, 30, 8, None, 4.0, False), (6, 2, 128, 128, 16, 48, 25.0, False), (5, 1, 576, 512, 64, None, None, True),
    (3, 1, 320, 256, 16, None, None, True), (4, 4, 64, 64, 8, None, None, False), (20, 1, 64, 64, 8, None, 4.0, False),
    (24, 1, 320, 256, 16, None, None, True), (40, 1, 128, 128, 16, 25, None, False)])
def test_biased_attention_in_batches_of_unequal_requests(ops, dtype, H, KVH, Dk, Dv, page, window, cap, shared):
    """A prompt from position 0, a portion in the middle of a context, two single tokens (one with a context of one
    key), in one launch, pages in a shuffled pool; against each request alone in the plain functions.  ``shared``:
    no value tensor, the values are the first Dv columns of the key rows.  In bfloat16 the widths 64, 128, 320 and 576
    go to the tensor-core kernel (values in chunks of 256 columns, keys of single tokens cut over blocks; up to 16 heads a
    kv head, up to 32 and more than 32: the three instances for single tokens)."""
    g = torch.Generator(device=DEV).manual_seed(H * Dk)
    q_lens, seq_lens = [1, 1, 21, 13], [1, 77, 21, 90]
    slopes = plain.slopes(H).to(DEV) if not shared else None
    ks, vs, tables, pools_k, pools_v = [], [], [], [], []
    base = 1
    for T in seq_lens:
        k = (torch.randn(T, KVH, Dk, generator=g, device=DEV) * 1.5).to(dtype)
        v = k[:, :, :Dv] if shared else torch.randn(T, KVH, Dv, generator=g, device=DEV).to(dtype)
        n = -(-T // page)
        order = list(range(base, base + n))[::-1]
        base += n
        ks.append(k), vs.append(v), tables.append(order)
    k_cache = torch.zeros(base, KVH, page, Dk, dtype=dtype, device=DEV)
    v_cache = None if shared else torch.zeros(base, KVH, page, Dv, dtype=dtype, device=DEV)
    for k, v, order in zip(ks, vs, tables):
        for j in range(k.shape[0]):
            k_cache[order[j // page], :, j % page] = k[j]
            if not shared:
                v_cache[order[j // page], :, j % page] = v[j]
    width = max(len(t) for t in tables)
    bt = i32([t + [0] * (width - len(t)) for t in tables])
    pad = 8 if Dk % 64 == 0 else 3                      # (the tensor-core kernel wants query rows on 16-byte boundaries)
    q = (torch.randn(sum(q_lens), H, Dk + pad, generator=g, device=DEV) * 1.5).to(dtype)[:, :, pad:]
    out = torch.zeros(sum(q_lens), H, Dv + 2, dtype=dtype, device=DEV)[:, :, :Dv]
    step = attention_step(q_lens, seq_lens)
    for splits in (0, 1, 3):
        ops.biased_decode_splits = splits
        out.zero_()
        ops.attention_biased(out, q, k_cache, v_cache, bt, step, KVH, page, 0.3, cap or 0.0, slopes, window)
        at = 0
        for n, T, k, v in zip(q_lens, seq_lens, ks, vs):
            want = plain_attention(q[at:at + n], k, v, KVH, 0.3, cap, slopes, window, T - n)
            # (32-bit sums of Dk products of size 2: the rounding of a score grows with the row's width)
            loose = {k_: v_ * max(1.0, Dk / 64) for k_, v_ in tol(dtype).items()} if dtype == torch.float32 else tol(dtype)
            assert torch.allclose(out[at:at + n].float().cpu(), want, **loose), (splits, n, T)
            at += n
    ops.biased_decode_splits = 0


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,page", [(48, 16), (64, 64), (5, 8), (None, 16)])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 12), (torch.bfloat16, 64), (torch.bfloat16, 128)])
def test_one_loud_key_far_away_at_page_edges_and_at_the_windows_edge(ops, window, page, decode, dtype, D):
    """Built inputs (float32 on the any-size kernel, bfloat16 on the tensor cores): all keys are silent but one, whose value is marked.  The query finds it hundreds of
    tokens back (no window), at a page's last and first place, at the last place the window still holds; and it
    must not find it one place further back, nor one place ahead of itself.  ``decode``: the query comes alone
    (keys cut over several blocks) or at the end of a portion of 30."""
    H, KVH = 2, 1
    T = 700
    n_q = 1 if decode else 30
    i = T - 1
    cases = [i, i - 1, i - (i % page), i - (i % page) - 1, 0, 1]
    if window:
        cases += [i - window + 1, i - window]
    else:
        cases += [i - 500, 3 * page - 1, 3 * page]
    for j in cases:
        k = torch.zeros(T + 1, KVH, D, dtype=dtype, device=DEV)
        v = torch.zeros(T + 1, KVH, D, dtype=dtype, device=DEV)
        k[j, 0, 3] = 60.0
        v[j, 0, 7] = 1.0
        k[T, 0, 3] = 90.0                                      # one place ahead of the query: in the cache's page, unseen
        v[T, 0, 5] = 1.0
        k_cache, order = paged(k, page, order=list(range(-(-(T + 1) // page), 0, -1)))
        v_cache, _ = paged(v, page, order=order)
        q = torch.zeros(n_q, H, D, dtype=dtype, device=DEV)
        q[:, :, 3] = 1.0
        out = torch.empty(n_q, H, D, dtype=dtype, device=DEV)
        step = attention_step([n_q], [T])
        ops.attention_biased(out, q, k_cache, v_cache, i32([order]), step, KVH, page, 1.0, 0.0, None, window)
        seen = window is None or i - j < window
        assert abs(float(out[-1, 0, 7]) - (1.0 if seen else 0.0)) < 1e-6, (j, seen)
        assert float(out[-1, :, 5].abs().max()) == 0.0, j


def test_the_bias_is_a_distance_and_the_cap_bounds_a_score(ops):
    """Two equal keys at distances 2 and 10: their weights differ by exp(-slope_h * 8), head by head.  A score of
    1000 is capped at 5: a key with score 0 keeps weight 1 / (1 + e^5)."""
    H, D, page = 4, 4, 8
    T = 30
    k = torch.zeros(T, 1, D, device=DEV)
    v = torch.zeros(T, 1, D, device=DEV)
    v[T - 3, 0, 0] = 1.0
    v[T - 11, 0, 1] = 1.0
    k[T - 3, 0, 2] = k[T - 11, 0, 2] = 50.0
    k_cache, order = paged(k, page)
    v_cache, _ = paged(v, page)
    q = torch.zeros(1, H, D, device=DEV)
    q[:, :, 2] = 1.0
    out = torch.empty(1, H, D, device=DEV)
    sl = plain.slopes(H).to(DEV)
    ops.attention_biased(out, q, k_cache, v_cache, i32([order]), attention_step([1], [T]), 1, page, 1.0, 0.0, sl, None)
    for h in range(H):
        assert abs(float(out[0, h, 1] / out[0, h, 0]) - math.exp(-float(sl[h]) * 8)) < 1e-5, h
    k.zero_(), v.zero_()
    k[5, 0, 2] = 1000.0
    v[5, 0, 0] = 1.0
    k_cache, order = paged(k[:7], page)
    v_cache, _ = paged(v[:7], page)
    ops.attention_biased(out, q, k_cache, v_cache, i32([order]), attention_step([1], [7]), 1, page, 1.0, 5.0, None, None)
    assert abs(float(out[0, 0, 0]) - math.e ** 5 / (math.e ** 5 + 6)) < 1e-5
