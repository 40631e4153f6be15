"""The Sotazen family on the GPU against the plain implementation: every new kernel alone, then the engine
under every way of cutting the work (whole prompts, a decoded tail, portions down to two tokens, mixed batches
with pages and state slots used again), in true 32-bit and in bfloat16, on small configurations that differ in
every size; greedy generation through `Engine`; the trace replay command and the command line."""
import json
import math
import os
import subprocess

import pytest
import torch

import plain_sotazen as P
from helpers import random_ids, rel_err
from sotazen_helpers import CONFIGS, Plain, make_sharp_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"
F64 = torch.float64
# max |engine - plain| / max |plain| over the compared logits.  fp32 sums a few hundred products per output
# against float64; in bfloat16 projections and activations are rounded to 8 bits.
TOL = {"float32": 3e-5, "bfloat16": 6e-2}
DTYPES = ["float32", "bfloat16"]
NAMES = sorted(CONFIGS)


def K():
    from rustinfer_b200.ops import kernels
    return kernels


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float32) * scale


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# =============================================================================== kernels alone
@pytest.mark.parametrize("d", [83, 96])
def test_embed_scaled(d):
    table = rnd(50, d, seed=1).to(torch.bfloat16)
    ids = [3, 49, 0, 3, 17]
    out = torch.empty((len(ids), d), dtype=torch.float32, device=DEV)
    K().embed_scaled(i32(ids), table.to(DEV), 0.37, out)
    assert rel_err(out, table.to(F64)[ids] * 0.37) < 1e-6


@pytest.mark.parametrize("d", [83, 96, 1032])
@pytest.mark.parametrize("ddtype", [torch.float32, torch.bfloat16])
def test_scale_add_norm(d, ddtype):
    """h <- w * rms(alpha h + delta + bias) in place, and the same rounded for the next product; alpha above and
    below one; without a sublayer's output the stream is only normed."""
    T, eps = 7, 1e-4
    w, b = (1.0 + 0.3 * rnd(d, seed=6)).to(torch.bfloat16), rnd(d, seed=7).to(torch.bfloat16)
    for alpha, bias in ((3.0, None), (0.5, b), (1.0, None)):
        h0, delta = rnd(T, d, seed=1), rnd(T, d, seed=2).to(ddtype)
        h = h0.to(DEV)
        act = torch.empty((T, d), dtype=torch.bfloat16, device=DEV)
        K().scale_add_norm(h, delta.to(DEV), bias.to(DEV) if bias is not None else None, alpha, w.to(DEV), eps, act)
        s = alpha * h0.to(F64) + delta.to(F64) + (bias.to(F64) if bias is not None else 0.0)
        ref = P.rms_norm(s, w.to(F64), eps)
        assert rel_err(h, ref) < 2e-6
        assert rel_err(act, ref) < 1e-2 and torch.equal(act.cpu(), h.cpu().to(torch.bfloat16))
    h = h0.to(DEV)
    K().scale_add_norm(h, None, None, 2.0, w.to(DEV), eps, None)
    assert rel_err(h, P.rms_norm(2.0 * h0.to(F64), w.to(F64), eps)) < 2e-6


@pytest.mark.parametrize("n", [36, 120, 1000])
def test_row_norm_gate(n):
    T, eps = 5, 1e-3
    o, w = rnd(T, n, seed=1, scale=30.0), (1.0 + 0.3 * rnd(n, seed=2)).to(torch.bfloat16)
    wide = rnd(T, n + 9, seed=3)                                          # the gate is a column view of wider rows
    for odt in (torch.float32, torch.bfloat16):
        out = torch.empty((T, n), dtype=odt, device=DEV)
        K().row_norm_gate(o.to(DEV), wide.to(DEV)[:, 9:], w.to(DEV), eps, out)
        ref = P.rms_norm(o.to(F64), w.to(F64), eps) * torch.sigmoid(wide[:, 9:].to(F64))
        assert rel_err(out, ref) < (2e-6 if odt == torch.float32 else 1e-2)
    K().row_norm_gate(o.to(DEV), None, w.to(DEV), eps, out)
    assert rel_err(out, P.rms_norm(o.to(F64), w.to(F64), eps)) < 1e-2


@pytest.mark.parametrize("H,vd", [(4, 24), (1, 8), (6, 16), (3, 100)])
def test_diff_combine(H, vd):
    """(1 - diff) * rms_head(a1 - lam a2) * sigmoid(gate) from a head's two maps side by side."""
    T, eps, lam, diff = 6, 1e-4, 0.83, 0.3
    a = rnd(T, H * 2 * vd, seed=1)
    wide = rnd(T, 5 + H * vd, seed=2)
    ref = P.difference_of_maps(a.to(F64).view(T, H, 2, vd), lam, diff, eps).reshape(T, H * vd)
    out = torch.empty((T, H * vd), dtype=torch.float32, device=DEV)
    K().diff_combine(a.to(DEV), lam, 1.0 - diff, eps, wide.to(DEV)[:, 5:], out, H, vd)
    assert rel_err(out, ref * torch.sigmoid(wide[:, 5:].to(F64))) < 2e-6
    out16 = torch.empty((T, H * vd), dtype=torch.bfloat16, device=DEV)
    K().diff_combine(a.to(DEV), lam, 1.0 - diff, eps, None, out16, H, vd)
    assert rel_err(out16, ref) < 1e-2
    # equal maps and lam = 1: the difference is zero, and eps keeps the norm finite
    same = a.view(T, H, 2, vd)[:, :, :1].repeat(1, 1, 2, 1).reshape(T, -1)
    K().diff_combine(same.to(DEV), 1.0, 1.0, eps, None, out, H, vd)
    assert float(out.abs().max()) == 0.0


def _tables(positions, dims, base, rows=4096):
    cos, sin = torch.zeros(rows, max(dims // 2, 1)), torch.zeros(rows, max(dims // 2, 1))
    if dims:
        f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
        ang = positions.to(F64)[:, None] * f[None, :]
        cos[positions], sin[positions] = torch.cos(ang).float(), torch.sin(ang).float()
    return cos, sin


@pytest.mark.parametrize("H,G,dk,dv,rot", [(4, 2, 16, 24, 8), (6, 1, 8, 16, 8), (2, 2, 32, 32, 0), (1, 1, 40, 8, 20)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qkv_prepare_two_maps(H, G, dk, dv, rot, dtype):
    """q [H][map][dk], k [G][map][dk], v [G][dv]: bias, a norm per head and map with one weight for all, rotary
    pairs (2i, 2i+1) on the first `rot` channels of every map, far positions, two key heads a value head into
    scrambled pages, nothing where the slot is -1."""
    T, page, eps, base = 9, 4, 1e-3, 700.0
    nq, nk, nv = H * 2 * dk, G * 2 * dk, G * dv
    wide = rnd(T, nq + nk + nv + 11, seed=1)                              # q, k, v are the leading columns
    bias = rnd(nq + nk + nv, seed=2, scale=0.5)
    qw, kw = 1.0 + 0.3 * rnd(dk, seed=3), 1.0 + 0.3 * rnd(dk, seed=4)
    pos = torch.tensor([0, 1, 2, 1000, 1001, 4095, 7, 8, 9])
    cos, sin = _tables(pos, rot, base)
    slots = [13, 2, 7, 0, -1, 22, 9, 5, 30]
    pages = 9
    per_page = page * (nk + nv)
    cache = torch.full((pages, per_page), 77.0, dtype=dtype, device=DEV)
    q_out = torch.empty((T, nq), dtype=dtype, device=DEV)
    K().qkv_prepare(wide.to(DEV)[:, : nq + nk + nv], bias.to(DEV), qw.to(DEV), kw.to(DEV), 1, eps, i32(pos.tolist()),
                    cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, rot, True, i32(slots), cache, q_out,
                    2 * H, 2 * G, dk, dv, True, value_heads=G)
    x = wide[:, : nq + nk + nv].to(F64) + bias.to(F64)
    q = P.rotate_pairs(P.rms_norm(x[:, :nq].reshape(T, H, 2, dk), qw.to(F64), eps), pos, rot, base)
    k = P.rotate_pairs(P.rms_norm(x[:, nq: nq + nk].reshape(T, G, 2, dk), kw.to(F64), eps), pos, rot, base)
    v = x[:, nq + nk:].reshape(T, G, dv)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert rel_err(q_out, q.reshape(T, nq)) < tol
    c = cache.cpu().to(F64)
    touched = torch.zeros_like(c, dtype=torch.bool)
    for t, s in enumerate(slots):
        if s < 0:
            continue
        pg, off = s // page, s % page
        for kh in range(2 * G):
            a = (kh * page + off) * dk
            assert rel_err(c[pg, a: a + dk], k[t, kh // 2, kh % 2]) < tol
            touched[pg, a: a + dk] = True
        for g in range(G):
            a = 2 * G * page * dk + (g * page + off) * dv
            assert rel_err(c[pg, a: a + dv], v[t, g]) < tol
            touched[pg, a: a + dv] = True
    assert bool((c[~touched] == 77.0).all())


@pytest.mark.parametrize("H,d,r,rank", [(4, 24, 8, 40), (2, 32, 16, 48), (3, 20, 4, 20), (1, 8, 0, 12)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare(H, d, r, rank, dtype):
    """From one projection [every head's plain and rotated query channels, the low-rank vector, the shared key
    part]: plain query parts, rotated query parts at the end of every head's row, and the cache row [normed
    low-rank vector, rotated key part] at scrambled slots."""
    T, page, eps, base = 9, 4, 1e-3, 300.0
    kd = rank + r
    proj = rnd(T, H * (d + r) + kd, seed=1)
    cw = (1.0 + 0.3 * rnd(rank, seed=2)).to(torch.bfloat16)
    pos = torch.tensor([0, 1, 2, 1000, 1001, 4095, 7, 8, 9])
    cos, sin = _tables(pos, r, base)
    if not r:
        cos, sin = torch.zeros(4096, 0), torch.zeros(4096, 0)
    slots = [13, 2, 7, 0, -1, 22, 9, 5, 30]
    cache = torch.full((9, page * kd), 77.0, dtype=dtype, device=DEV)
    q_plain = torch.empty((T, H * d), dtype=dtype, device=DEV)
    q_full = torch.full((T, H * kd), 5.0, dtype=dtype, device=DEV)
    K().latent_prepare(proj.to(DEV), cw.to(DEV), eps, i32(pos.tolist()), cos.to(DEV), sin.to(DEV), i32(slots), cache,
                       q_plain, q_full, H, d, r, rank)
    p64 = proj.to(F64)
    q = p64[:, : H * (d + r)].reshape(T, H, d + r)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert rel_err(q_plain, q[..., :d].reshape(T, H * d)) < tol
    full = q_full.cpu().to(F64).view(T, H, kd)
    if r:
        assert rel_err(full[..., rank:], P.rotate_pairs(q[..., d:], pos, r, base)) < tol
    assert bool((full[..., :rank] == 5.0).all())                         # left for the product with the up-projection
    c = P.rms_norm(p64[:, H * (d + r): H * (d + r) + rank], cw.to(F64), eps)
    kr = P.rotate_pairs(p64[:, H * (d + r) + rank:], pos, r, base)
    got = cache.cpu().to(F64).view(9 * page, kd)
    used = [s for s in slots if s >= 0]
    want = torch.cat([c, kr], dim=1)[[t for t, s in enumerate(slots) if s >= 0]]
    assert rel_err(got[used], want) < tol
    rest = torch.ones(9 * page, dtype=torch.bool)
    rest[used] = False
    assert bool((got[rest] == 77.0).all())


# ---------------------------------------------------------------------------------- the decay recurrence
def _pieces(T, cuts):
    at, out = 0, []
    for c in cuts:
        out.append((at, at + c))
        at += c
    assert at == T
    return out


@pytest.mark.parametrize("dk,dv,H", [(16, 40, 3), (32, 32, 4), (64, 32, 2), (20, 12, 1), (100, 9, 1)])
def test_decay_scan_kernel(dk, dv, H):
    """Two requests walked in pieces of changing size (one token, two, many), side by side in one launch where
    their pieces meet, their states in slots 3 and 1 of a state tensor whose other rows stay as they were; q, k
    and v are column views of one fp32 projection, as the mixer hands them over."""
    T = 45
    buf = [rnd(T, 2 * H * dk + H * dv + 3, seed=s) for s in (1, 2)]
    decay = torch.tensor([0.5, 0.97, 0.999, 0.8][:H], dtype=F64)
    row = decay.float().repeat_interleave(dk).to(DEV)
    state = torch.full((5, H, dv, K().recurrent_state_rows(dk)), 9.0, device=DEV)
    state[3] = 0
    state[1] = 0
    cuts = [_pieces(T, [1, 2, 17, 1, 8, 16]), _pieces(T, [20, 1, 1, 3, 9, 11])]
    outs = [torch.zeros(T, H * dv), torch.zeros(T, H * dv)]
    for (a0, a1), (b0, b1) in zip(*cuts):
        x = torch.cat([buf[0][a0:a1], buf[1][b0:b1]]).to(DEV)
        n = x.shape[0]
        o = torch.empty((n, H * dv), dtype=torch.float32, device=DEV)
        K().decay_scan(x[:, 3: 3 + H * dk], x[:, 3 + H * dk: 3 + 2 * H * dk], x[:, 3 + 2 * H * dk:], row, 1.0, o, state,
                       i32([0, a1 - a0, n]), i32([3, 1]), 2, H, dk, dv)
        outs[0][a0:a1] = o[: a1 - a0].cpu()
        outs[1][b0:b1] = o[a1 - a0:].cpu()
    for r in range(2):
        b64 = buf[r].to(F64)
        q = b64[:, 3: 3 + H * dk].view(T, H, dk)
        k = b64[:, 3 + H * dk: 3 + 2 * H * dk].view(T, H, dk)
        v = b64[:, 3 + 2 * H * dk:].view(T, H, dv)
        want, S = P.decay_recurrence(q, k, v, decay)
        assert rel_err(outs[r], want.reshape(T, -1)) < 2e-5
        got_S = state[[3, 1][r]].cpu().to(F64)[:, :, :dk].transpose(1, 2)                # [H, dk, dv]
        assert rel_err(got_S, S) < 2e-5
    assert bool((state[[0, 2, 4]] == 9.0).all())


def test_decay_scan_keeps_a_far_key_and_forgets_at_its_rate():
    """Keys along the axes, a query along one axis: the output is the sum of the values written along that axis,
    each times decay^(distance), 600 tokens in portions read by a single token.  With a decay of one nothing is
    lost; with 0.99 the far values count for what the closed form says; with 0.5 only the last one counts."""
    dk, dv, T, H = 16, 8, 600, 3
    decay = [1.0, 0.99, 0.5]
    k = torch.zeros(T + 1, H, dk)
    for t in range(T):
        k[t, :, t % dk] = 1.0
    v = rnd(T + 1, H, dv, seed=1)
    q = torch.zeros(T + 1, H, dk)
    q[T, :, 5] = 1.0
    row = torch.tensor(decay).repeat_interleave(dk).to(DEV)
    state = torch.zeros((1, H, dv, K().recurrent_state_rows(dk)), device=DEV)
    at = 0
    for n in (64, 2, 300, 1, 233, 1):
        o = torch.empty((n, H * dv), dtype=torch.float32, device=DEV)
        K().decay_scan(q[at: at + n].reshape(n, -1).to(DEV), k[at: at + n].reshape(n, -1).to(DEV),
                       v[at: at + n].reshape(n, -1).to(DEV), row, 1.0, o, state, i32([0, n]), i32([0]), 1, H, dk, dv)
        at += n
    got = o[-1].cpu().to(F64).view(H, dv)
    for h, a in enumerate(decay):
        want = sum(a ** (T - s) * v[s, h].to(F64) for s in range(5, T, dk))
        assert float((got[h] - want).abs().max()) < 1e-4, h
    last = max(range(5, T, dk))
    assert float((got[2] - 0.5 ** (T - last) * v[last, 2].to(F64)).abs().max()) < 1e-4     # the last write on axis 5


# ------------------------------------------------------------------------------- attention of two maps
def paged_maps(keys, vals, page, table, dtype):
    """A cache [pages, page * (G*maps*dk + G*dv)] that holds keys [n, G, maps, dk] and vals [n, G, dv] of one
    request in the pages `table` names (a page's key heads [kv head][map], then its value heads); the rest is
    poison."""
    n, G, maps, dk = keys.shape
    dv = vals.shape[2]
    pages = max(table) + 2
    c = torch.full((pages, page * (G * maps * dk + G * dv)), 1e4, dtype=torch.float32)
    for t in range(n):
        pg, off = table[t // page], t % page
        for g in range(G):
            for m in range(maps):
                a = ((g * maps + m) * page + off) * dk
                c[pg, a: a + dk] = keys[t, g, m]
            b = G * maps * page * dk + (g * page + off) * dv
            c[pg, b: b + dv] = vals[t, g]
    return c.to(dtype).to(DEV)


@pytest.mark.parametrize("dk,dv,window,cap", [(16, 24, 20, 20.0), (32, 32, 16, None), (40, 8, 33, 1.5), (8, 16, None, 50.0)])
def test_two_map_attention_edges_and_far_keys(dk, dv, window, cap):
    """For every query and map one key stands out (the two maps look for different keys, at different distances):
    a map's output is that key's value when the key is inside the window and something else when it is one
    further.  Keys just inside and just outside the window, in prompt portions and for single tokens, the
    window's edge inside a page and at a page's edge, pages scrambled and poisoned outside; without a window a
    key hundreds of tokens back among hundreds.  A cap on the scores (a small one flattens what stands out) is
    held against the plain model like the rest.  (Keys are unit vectors with a channel of 1 appended, queries
    the looked-for key times a gain with -gain appended: q . k = gain * (cos - 1).)"""
    page, H, G, n = 8, 4, 2, 330
    table = torch.randperm(48, generator=torch.Generator().manual_seed(5)).tolist()[: (n + page - 1) // page]
    unit = torch.nn.functional.normalize(rnd(n, 2, dk, seed=2), dim=-1)              # a set of keys a map
    top = max(float((unit[:, m] @ unit[:, m].T - 2.0 * torch.eye(n)).max()) for m in range(2))
    gain = 30.0 / (1.0 - top)
    keys = torch.cat([unit, torch.ones(n, 2, 1)], dim=-1)[:, None].repeat(1, G, 1, 1)    # [n, G, 2, dk+1]
    vals = rnd(n, G, dv, seed=1)
    d1 = dk + 1
    cache = paged_maps(keys, vals, page, table, torch.float32)
    bt = i32([table])

    def queries(targets):                    # targets: [(key of map 1, key of map 2)]
        q = torch.zeros(len(targets), H, 2, d1)
        for i, tg in enumerate(targets):
            for m in range(2):
                q[i, :, m, :dk] = unit[tg[m], m] * gain
                q[i, :, m, dk] = -gain
        return q

    def plain_rows(first, targets):
        T = first + len(targets)
        q = torch.zeros(T, H, 2, d1, dtype=F64)
        q[first:] = queries(targets).to(F64)
        return P.two_map_attention(q, keys[:T].to(F64), vals[:T].to(F64), 1.0, cap, window)[first:]

    def attend(first, targets):
        count = len(targets)
        out = torch.empty((count, H * 2 * dv), dtype=torch.float32, device=DEV)
        tiles = list(range(0, count, 16))
        K().attention_plain(queries(targets).reshape(count, -1).to(DEV), out, cache, bt, i32([0, count]),
                            i32([first + count]), i32([0] * len(tiles)), i32(tiles), 2 * H, G, d1, 1.0, window, None, dv,
                            softcap=cap, maps=2)
        return out.cpu().view(count, H, 2, dv)

    def attend_single(pos, tg, splits=1):
        out = torch.empty((1, H * 2 * dv), dtype=torch.float32, device=DEV)
        part = torch.full((K().attention_single_scratch_floats(1, 2 * H, dv, splits),), float("nan"), device=DEV)
        K().attention_single(queries([tg]).reshape(1, -1).to(DEV), out, cache, bt, i32([0, 1]), i32([pos + 1]), i32([0]),
                             2 * H, G, d1, 1.0, window, None, dv, splits=splits, part=part, softcap=cap, maps=2)
        return out.cpu().view(H, 2, dv)

    w = window or 10 ** 9
    first, count = 45, 70
    sharp = cap is None or cap >= 20.0                      # whether what stands out still does under the cap
    for shift in ((0, 1, w - 1, w, w + 1) if window else (0, 1, 40, 100)):
        other = max(0, shift - 3)
        targets = [(max(0, p - shift), max(0, p - other)) for p in range(first, first + count)]
        got, ref = attend(first, targets), plain_rows(first, targets)
        assert float((got.to(F64) - ref).abs().max()) < 2e-4, shift
        if sharp:
            for m, s in ((0, shift), (1, other)):
                lead = float((ref[-1, 0, m] - vals[targets[-1][m], 0].to(F64)).abs().max())
                assert (lead < 1e-3) == (s < w), (shift, m)
    if window:
        singles = [(p, t) for p in (w - 1, w, w + 1, 2 * w + 3, n - 1) for t in (p, p - w + 1, p - w, 0) if 0 <= t <= p]
    else:
        singles = [(n - 1, 3), (n - 1, n - 1), (300, 0), (64, 63), (7, 0)]
    for p, tgt in singles:
        tg = (tgt, min(p, tgt + 1))
        ref = plain_rows(p, [tg])[0]
        assert float((attend(p, [tg])[0].to(F64) - ref).abs().max()) < 2e-4, (p, tgt)
        if K().attention_single_supports(2 * H, G, d1, dv, maps=2):
            for splits in (1, 2, 5):
                assert float((attend_single(p, tg, splits).to(F64) - ref).abs().max()) < 2e-4, (p, tgt, splits)


# ------------------------------------------------------------ attention over one cached row a token, with a sink
@pytest.mark.parametrize("rank,r,H", [(40, 8, 4), (48, 16, 2), (20, 4, 3), (88, 16, 6)])
def test_latent_rows_attention_far_keys_and_sink(rank, r, H):
    """One row [low-rank vector, shared key part] a token is every head's key, and its first `rank` channels
    the value.  One key stands out with score 0: a head whose sink is 0 gives it the weight 1/2, a head whose
    sink is far below gives it all, a head whose sink is far above gives nearly nothing; 326 tokens back among
    hundreds, in prompt portions and for single tokens with the keys in 1, 2 and 5 ranges, pages scrambled."""
    page, n = 8, 330
    kd = rank + r
    table = torch.randperm(48, generator=torch.Generator().manual_seed(7)).tolist()[: (n + page - 1) // page]
    unit = torch.nn.functional.normalize(rnd(n, kd - 1, seed=2), dim=-1)
    gain = 30.0 / (1.0 - float((unit @ unit.T - 2.0 * torch.eye(n)).max()))
    rows = torch.cat([unit, torch.ones(n, 1)], dim=-1)                    # [n, kd]
    cache = torch.full((max(table) + 2, page * kd), 1e4)
    for t in range(n):
        cache[table[t // page], (t % page) * kd: (t % page + 1) * kd] = rows[t]
    cache = cache.to(DEV)
    bt = i32([table])
    sink = torch.tensor(([0.0, -1e4, 40.0, 1.0] * 2)[:H])

    def queries(targets):
        q = torch.zeros(len(targets), H, kd)
        for i, tgt in enumerate(targets):
            q[i, :, : kd - 1] = unit[tgt] * gain
            q[i, :, kd - 1] = -gain
        return q

    def plain_rows(first, targets):
        T = first + len(targets)
        q = torch.zeros(T, H, kd, dtype=F64)
        q[first:] = queries(targets).to(F64)
        s = torch.einsum("ihd,jd->hij", q, rows[:T].to(F64)) * 0.5
        p = P.softmax_rows(s, P.visible(T, None), sink.to(F64))
        return torch.einsum("hij,jv->ihv", p, rows[:T, :rank].to(F64))[first:]

    def attend(first, targets):
        count = len(targets)
        out = torch.empty((count, H * rank), dtype=torch.float32, device=DEV)
        tiles = list(range(0, count, 16))
        K().attention_plain(queries(targets).reshape(count, -1).to(DEV), out, cache, bt, i32([0, count]),
                            i32([first + count]), i32([0] * len(tiles)), i32(tiles), H, 1, kd, 0.5, None, None, rank,
                            sink=True, sink_values=sink.to(DEV), value_in_key=True)
        return out.cpu().view(count, H, rank)

    def attend_single(pos, tgt, splits):
        out = torch.empty((1, H * rank), dtype=torch.float32, device=DEV)
        part = torch.full((K().attention_single_scratch_floats(1, H, rank, splits),), float("nan"), device=DEV)
        K().attention_single(queries([tgt]).reshape(1, -1).to(DEV), out, cache, bt, i32([0, 1]), i32([pos + 1]), i32([0]),
                             H, 1, kd, 0.5, None, None, rank, sink=True, splits=splits, part=part,
                             sink_values=sink.to(DEV), value_in_key=True)
        return out.cpu().view(H, rank)

    first, count = 45, 70
    for shift in (0, 1, 40, 100):
        targets = [max(0, p - shift) for p in range(first, first + count)]
        got, ref = attend(first, targets), plain_rows(first, targets)
        assert float((got.to(F64) - ref).abs().max()) < 2e-4, shift
        val = rows[targets[-1], :rank].to(F64)
        assert float((ref[-1, 0] - 0.5 * val).abs().max()) < 1e-3                   # sink 0 beside a score of 0
        if H > 1:
            assert float((ref[-1, 1] - val).abs().max()) < 1e-3                     # no sink to speak of
        if H > 2:
            assert float(ref[-1, 2].abs().max()) < 1e-6                             # the sink takes it all
    for p, tgt in [(n - 1, 3), (n - 1, n - 1), (300, 0), (64, 63), (7, 0), (0, 0)]:
        ref = plain_rows(p, [tgt])[0]
        assert float((attend(p, [tgt])[0].to(F64) - ref).abs().max()) < 2e-4, (p, tgt)
        if K().attention_single_supports(H, 1, kd, rank):
            for splits in (1, 2, 5):
                assert float((attend_single(p, tgt, splits).to(F64) - ref).abs().max()) < 2e-4, (p, tgt, splits)


# ------------------------------------------------------------ the same two attentions on the tensor cores
BF = torch.bfloat16


def bf_round(x):
    return x.to(BF).to(torch.float32)


@pytest.mark.parametrize("dk,dv,H,G,window,cap", [(15, 32, 4, 2, 20, 20.0), (31, 16, 6, 1, 16, None), (47, 80, 4, 1, 24, 45.0),
                                                  (63, 128, 2, 2, None, 30.0)])
def test_two_map_attention_on_tensor_cores(dk, dv, H, G, window, cap):
    """`attention_rows` against the plain model on inputs that bfloat16 holds exactly: for every query and map one
    key stands out, just inside and just outside the window, in prompt portions (from the first token on, and from
    the middle of a page) and for single tokens, pages scrambled and poisoned outside; without a window a key
    hundreds of tokens back."""
    page, n = 8, 330
    table = torch.randperm(48, generator=torch.Generator().manual_seed(5)).tolist()[: (n + page - 1) // page]
    unit = torch.nn.functional.normalize(rnd(n, 2, dk, seed=2), dim=-1)
    top = max(float((unit[:, m] @ unit[:, m].T - 2.0 * torch.eye(n)).max()) for m in range(2))
    gain = 30.0 / (1.0 - top)
    keys = bf_round(torch.cat([unit, torch.ones(n, 2, 1)], dim=-1))[:, None].repeat(1, G, 1, 1)    # [n, G, 2, dk+1]
    vals = bf_round(rnd(n, G, dv, seed=1))
    d1 = dk + 1
    cache = paged_maps(keys, vals, page, table, BF)
    bt = i32([table])
    tpt = K().attention_rows_tokens_per_tile(2 * H, G, d1, dv, 2)
    assert tpt == 64 // (H // G)

    def queries(targets):
        q = torch.zeros(len(targets), H, 2, d1)
        for i, tg in enumerate(targets):
            for m in range(2):
                q[i, :, m, :dk] = unit[tg[m], m] * gain
                q[i, :, m, dk] = -gain
        return bf_round(q)

    def plain_rows(first, targets):
        T = first + len(targets)
        q = torch.zeros(T, H, 2, d1, dtype=F64)
        q[first:] = queries(targets).to(F64)
        return P.two_map_attention(q, keys[:T].to(F64), vals[:T].to(F64), 1.0, cap, window)[first:]

    def attend(first, targets, splits=1):
        count = len(targets)
        out = torch.full((count, H * 2 * dv), float("nan"), dtype=torch.float32, device=DEV)
        tiles = list(range(0, count, tpt))
        part = torch.full((K().attention_rows_scratch_floats(len(tiles), 2 * H, G, dv, 2, splits),), float("nan"), device=DEV)
        K().attention_rows(queries(targets).reshape(count, -1).to(BF).to(DEV), out, cache, bt, i32([0, count]),
                           i32([first + count]), i32([0] * len(tiles)), i32(tiles), 2 * H, G, d1, 1.0, window, dv,
                           softcap=cap, maps=2, splits=splits, part=part)
        return out.cpu().view(count, H, 2, dv)

    w = window or 10 ** 9
    for first, count in ((45, 70), (0, 67), (128, 1)):
        for shift in ((0, 1, w - 1, w, w + 1) if window else (0, 1, 40, 100)):
            other = max(0, shift - 3)
            targets = [(max(0, p - shift), max(0, p - other)) for p in range(first, first + count)]
            got, ref = attend(first, targets), plain_rows(first, targets)
            assert float((got.to(F64) - ref).abs().max()) < 2e-4, (first, shift)
            for m, sh in ((0, shift), (1, other)):
                if targets[-1][m] == first + count - 1 - sh:           # not clamped at the first token
                    lead = float((ref[-1, 0, m] - vals[targets[-1][m], 0].to(F64)).abs().max())
                    assert (lead < 1e-2) == (sh < w), (first, shift, m)
    for p, tgt in [(n - 1, 3), (n - 1, n - 1), (300, 0), (64, 63), (7, 0), (0, 0)]:
        tg = (tgt, min(p, tgt + 1))
        ref = plain_rows(p, [tg])[0]
        for splits in (1, 2, 7):            # key ranges: some hold no visible key, some are empty
            assert float((attend(p, [tg], splits)[0].to(F64) - ref).abs().max()) < 2e-4, (p, tgt, splits)
    targets = [(max(0, p - 2), max(0, p - 40)) for p in range(250, 320)]
    assert float((attend(250, targets, 3).to(F64) - plain_rows(250, targets)).abs().max()) < 2e-4


@pytest.mark.parametrize("rank,r,H", [(32, 16, 4), (80, 16, 3), (64, 48, 20), (16, 16, 70), (256, 32, 8)])
def test_latent_rows_attention_on_tensor_cores(rank, r, H):
    """`attention_rows` over one cached row a token with a sink a head: 3, 20 and 70 heads on one key head (a tile
    of 64 rows then holds 21, 3 and 1 tokens; 70 heads take two CTAs), a key 326 tokens back among hundreds."""
    page, n = 8, 330
    kd = rank + r
    table = torch.randperm(48, generator=torch.Generator().manual_seed(7)).tolist()[: (n + page - 1) // page]
    unit = torch.nn.functional.normalize(rnd(n, kd - 1, seed=2), dim=-1)
    gain = 30.0 / (1.0 - float((unit @ unit.T - 2.0 * torch.eye(n)).max()))
    rows = bf_round(torch.cat([unit, torch.ones(n, 1)], dim=-1))
    cache = torch.full((max(table) + 2, page * kd), 1e4)
    for t in range(n):
        cache[table[t // page], (t % page) * kd: (t % page + 1) * kd] = rows[t]
    cache = cache.to(BF).to(DEV)
    bt = i32([table])
    sink = torch.tensor(([0.0, -1e4, 40.0, 1.0] * 18)[:H])
    tpt = K().attention_rows_tokens_per_tile(H, 1, kd, rank, 1)
    assert tpt == max(1, 64 // H)

    def queries(targets):
        q = torch.zeros(len(targets), H, kd)
        for i, tgt in enumerate(targets):
            q[i, :, : kd - 1] = unit[tgt] * gain
            q[i, :, kd - 1] = -gain
        return bf_round(q)

    def plain_rows(first, targets):
        T = first + len(targets)
        q = torch.zeros(T, H, kd, dtype=F64)
        q[first:] = queries(targets).to(F64)
        sc = torch.einsum("ihd,jd->hij", q, rows[:T].to(F64)) * 0.5
        p = P.softmax_rows(sc, P.visible(T, None), sink.to(F64))
        return torch.einsum("hij,jv->ihv", p, rows[:T, :rank].to(F64))[first:]

    def attend(first, targets, dtype=torch.float32, splits=1):
        count = len(targets)
        out = torch.full((count, H * rank), float("nan"), dtype=dtype, device=DEV)
        tiles = list(range(0, count, tpt))
        part = torch.full((K().attention_rows_scratch_floats(len(tiles), H, 1, rank, 1, splits),), float("nan"), device=DEV)
        K().attention_rows(queries(targets).reshape(count, -1).to(BF).to(DEV), out, cache, bt, i32([0, count]),
                           i32([first + count]), i32([0] * len(tiles)), i32(tiles), H, 1, kd, 0.5, None, rank,
                           sink=True, sink_values=sink.to(DEV), value_in_key=True, splits=splits, part=part)
        return out.float().cpu().view(count, H, rank)

    for first, count in ((45, 70), (0, 33)):
        for shift in (0, 1, 40, 100):
            targets = [max(0, p - shift) for p in range(first, first + count)]
            got, ref = attend(first, targets), plain_rows(first, targets)
            assert float((got.to(F64) - ref).abs().max()) < 2e-4, (first, shift)
    assert float((attend(45, list(range(45, 115)), BF).to(F64) - plain_rows(45, list(range(45, 115)))).abs().max()) < 1e-2
    for p, tgt in [(n - 1, 3), (n - 1, n - 1), (300, 0), (64, 63), (7, 0), (0, 0)]:
        ref = plain_rows(p, [tgt])[0]
        for splits in (1, 2, 5, 16):        # key ranges joined by the second launch; the sink counts once
            assert float((attend(p, [tgt], splits=splits)[0].to(F64) - ref).abs().max()) < 2e-4, (p, tgt, splits)
    targets = [max(0, p - 100) for p in range(200, 270)]
    assert float((attend(200, targets, splits=4).to(F64) - plain_rows(200, targets)).abs().max()) < 2e-4
    assert float((attend(n - 1, [5], BF, splits=3)[0].to(F64) - plain_rows(n - 1, [5])[0]).abs().max()) < 1e-2


# ============================================================================ the engine
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("sotazen")
    out = {}
    for n in NAMES:
        folder = make_sharp_model(str(root / n), n, seed=31 + ord(n))
        out[n] = (folder, Plain(folder))
    return out


def close(got, ref, dtype):
    return rel_err(got, ref) <= TOL[dtype]


def runner(folder, dtype, max_tokens=512, page=16, seqs=4, pages=None, capture=None):
    from rustinfer_b200.engine.runner import ModelRunner
    return ModelRunner(folder, dtype=dtype, max_model_len=max_tokens, page_size=page,
                       num_pages=pages if pages is not None else max_tokens // page,
                       max_batch_seqs=seqs, max_batch_tokens=max_tokens, capture_sizes=capture)


def run_cuts(r, rid, ids, cuts):
    from rustinfer_b200.engine.runner import StepEntry
    r.open(rid)
    outs, at = [], 0
    for c in cuts:
        outs.append(r.step([StepEntry(rid, ids[at: at + c], list(range(c)))]))
        at += c
    assert at == len(ids)
    r.close(rid)
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_layers_one_by_one(models, name, dtype):
    """The stream after every layer against the plain model's, for a whole prompt and for the same prompt cut
    in two with three single tokens at its end."""
    from rustinfer_b200.engine.runner import StepEntry
    folder, plain = models[name]
    ids = random_ids(50, CONFIGS[name]["vocab"], 7)
    want = []
    P.forward(plain.cfg, plain.w, ids, want)
    r = runner(folder, dtype)
    taps = []
    r.model.layer_tap = lambda i, hidden: taps.append((i, hidden.stream.clone().cpu()))
    r.open("a")
    r.step([StepEntry("a", ids, [0])])
    r.close("a")
    assert [i for i, _ in taps] == list(range(len(want)))
    for (i, g), w in zip(taps, want):
        assert close(g, w, dtype), i
    taps.clear()
    r.open("b")
    for a, b in ((0, 21), (21, 47), (47, 48), (48, 49), (49, 50)):
        r.step([StepEntry("b", ids[a:b], [0])])
    L = len(want)
    for i, w in enumerate(want):
        got = torch.cat([taps[s * L + i][1] for s in range(5)])
        assert close(got, w, dtype), i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_tail_and_portions(models, name, dtype):
    folder, plain = models[name]
    V = CONFIGS[name]["vocab"]
    r = runner(folder, dtype, page=8 if name == "B" else 16)
    for n, seed in [(130, 1), (61, 2), (1, 3), (3, 4)]:
        ids = random_ids(n, V, seed)
        ref = plain.logits(ids)
        assert close(run_cuts(r, "w", ids, [n]), ref, dtype)                   # the first tokens included
        if n < 40:
            continue
        tail = run_cuts(r, "t", ids, [n - 45] + [1] * 45)                      # windows pass over decoded tokens
        assert close(tail, ref, dtype)
        cuts, left, sizes = [], n, [2, 7, 1, 16, 2, 33, 24, 5, 2, 64]
        while left:
            c = min(sizes[len(cuts) % len(sizes)], left)
            cuts.append(c)
            left -= c
        assert close(run_cuts(r, "p", ids, cuts), ref, dtype)
        assert close(run_cuts(r, "two", ids[:40], [2] * 20), ref[:40], dtype)
        assert close(run_cuts(r, "one", ids[:40], [1] * 40), ref[:40], dtype)  # token by token from the start
    r.cache.check_invariants()
    torch.cuda.synchronize()
    r.check_kernel_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Three state slots and a pool that holds far less than the requests' sum: requests come and go, portions
    of prompts run beside single tokens, and every request's logits are those it has alone."""
    from rustinfer_b200.engine.runner import StepEntry
    folder, plain = models[name]
    V = CONFIGS[name]["vocab"]
    r = runner(folder, dtype, max_tokens=256, page=16, seqs=3, pages=20)
    lens = {"a": 150, "b": 37, "c": 90, "d": 2, "e": 120, "f": 64}
    ids = {k: random_ids(n, V, 100 + i) for i, (k, n) in enumerate(lens.items())}
    at = {k: 0 for k in ids}
    got = {k: [] for k in ids}
    waiting = list(ids)
    live = []
    portion = {"a": [33, 1, 1, 50, 2], "b": [5, 1, 1], "c": [64, 1, 25], "d": [1], "e": [2, 100, 1], "f": [16, 47, 1]}
    turn = 0
    while waiting or live:
        while waiting and len(live) < 3:
            k = waiting.pop(0)
            r.open(k)
            live.append(k)
        entries = []
        for k in live:
            if (turn + ord(k)) % 4 == 3 and len(live) > 1 and len(entries) + 1 < len(live):
                continue                                         # a request sits a step out now and then
            plan = portion[k]
            n = min(plan[min(len(got[k]), len(plan) - 1)], lens[k] - at[k])
            entries.append(StepEntry(k, ids[k][at[k]: at[k] + n], list(range(n))))
        if not entries:
            turn += 1
            continue
        lg = r.step(entries)
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.request_id].append(lg[row: row + n])
            row += n
            at[e.request_id] += n
            if at[e.request_id] == lens[e.request_id]:
                r.close(e.request_id)
                live.remove(e.request_id)
        r.cache.check_invariants()
        turn += 1
    for k in ids:
        assert close(torch.cat(got[k]), plain.logits(ids[k]), dtype), k
    torch.cuda.synchronize()
    r.check_kernel_errors()


def test_fp32_logits_do_not_depend_on_the_cut(models):
    """Attention, the recurrence and the norms add in an order that the cut does not change; the library's batched
    products of the latent layer may add in another order for another count of rows, so the logits agree to
    rounding, not to the bit."""
    folder, _ = models["A"]
    r = runner(folder, "float32")
    ids = random_ids(90, CONFIGS["A"]["vocab"], 9)
    whole = run_cuts(r, "w", ids, [90])
    assert rel_err(run_cuts(r, "p", ids, [31, 2, 1, 24, 32]), whole) <= 2e-6
    assert rel_err(run_cuts(r, "t", ids, [60] + [1] * 30), whole) <= 2e-6


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_long_decoding_and_graphs(models, name):
    """300 single tokens after a short prompt, eager and from captured steps: windows pass, their pages are
    given back, the states carry, and the logits stay those of the plain model."""
    from rustinfer_b200.engine.runner import StepEntry
    folder, plain = models[name]
    ids = random_ids(310, CONFIGS[name]["vocab"], 5)
    ref = plain.logits(ids)
    for dtype, capture in (("float32", None), ("float32", [1, 2]), ("bfloat16", [1, 2])):
        r = runner(folder, dtype, max_tokens=320, page=16, seqs=2, pages=20, capture=capture)
        r.open("a")
        out = [r.step([StepEntry("a", ids[:10], list(range(10)))])]
        for t in range(10, 310):
            out.append(r.step([StepEntry("a", ids[t: t + 1], [0])]))
        assert close(torch.cat(out), ref, dtype)
        if capture:
            assert r.graph_replays == 300
        r.close("a")
        r.cache.check_invariants()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(models, name):
    """`Engine.generate`: scheduler, chunked prefill, continuous batching, device argmax, decode graphs."""
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, plain = models[name]
    V = CONFIGS[name]["vocab"]
    prompts = [random_ids(n, V, 50 + n) for n in (45, 3, 70, 1, 26)]
    want = [plain.greedy(p, 12) for p in prompts]
    eng = Engine(folder, dtype="float32", max_batch_seqs=3, max_model_len=128, paged_block_size=16,
                 num_blocks=24, max_batch_tokens=64, chunked_prefill_size=32)
    got = [res.tokens for res in eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))]
    assert got == want
    eng16 = Engine(folder, dtype="bfloat16", max_batch_seqs=3, max_model_len=128, paged_block_size=16,
                   num_blocks=24, max_batch_tokens=64, chunked_prefill_size=32)
    got16 = [res.tokens for res in eng16.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))]
    same = sum(a == b for g, w in zip(got16, want) for a, b in zip(g, w))
    assert same >= 0.5 * 12 * len(prompts), (got16, want)


def test_trace_replay_command(models, tmp_path):
    folder, plain = models["B"]
    V = CONFIGS["B"]["vocab"]
    a, b = random_ids(70, V, 1), random_ids(20, V, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[33:69], "want": []}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0]}, {"id": "a", "tokens": a[69:], "want": [0]}], "end": ["a", "b"]},
    ]
    import numpy as np
    ra, rb = plain.logits(a), plain.logits(b)
    for dtype in DTYPES:
        out = tmp_path / dtype
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4")).view(2, V)
        assert rel_err(g0, ra[[0, 32]]) <= TOL[dtype]
        g1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4")).view(1, V)
        assert rel_err(g1, rb[[18]]) <= TOL[dtype]
        g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4")).view(2, V)
        assert rel_err(g2, torch.stack([rb[19], ra[69]])) <= TOL[dtype]


def test_command_line_and_sampler_serve_a_sotazen_folder(models, tmp_path):
    """`bin/rustinfer --config run.toml` on a Sotazen folder: greedy tokens are the plain model's.  Through `Engine`
    with temperature, top-k and top-p: a seeded request gives the same tokens twice, and every drawn token is among
    the most likely at its place."""
    import sys
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, plain = models["C"]
    V = CONFIGS["C"]["vocab"]
    prompt = random_ids(21, V, 8)
    (tmp_path / "run.toml").write_text(f"""
model = "{folder}"
dtype = "float32"
max_batch_tokens = 64
max_batch_seqs = 3
max_model_len = 96
paged_block_size = 16
chunked_prefill_size = 8
num_blocks = 18
ignore_eos = true
capture_sizes = [1, 2, 4]

[sampling]
temperature = 0.0
max_tokens = 7

[[request]]
prompt_ids = {prompt}

[[request]]
prompt_ids = {prompt[:5]}
""")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rustinfer"), "--config", str(tmp_path / "run.toml")],
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.strip()]
    assert [l["request"] for l in lines] == [0, 1]
    assert lines[0]["tokens"] == plain.greedy(prompt, 7) and lines[1]["tokens"] == plain.greedy(prompt[:5], 7)
    eng = Engine(folder, dtype="float32", max_batch_seqs=3, max_model_len=96, paged_block_size=16, num_blocks=18,
                 max_batch_tokens=64, chunked_prefill_size=8)
    sp = SamplingParams(temperature=0.9, top_k=12, top_p=0.8, seed=11, max_tokens=7, ignore_eos=True)
    first = [r.tokens for r in eng.generate([prompt[:5], prompt], sp)]
    again = [r.tokens for r in eng.generate([prompt[:5], prompt], sp)]
    assert first == again and all(len(t) == 7 for t in first)
    ids = list(prompt[:5])
    for tok in first[0]:
        assert tok in torch.topk(plain.logits(ids)[-1], 12).indices.tolist()
        ids.append(tok)
