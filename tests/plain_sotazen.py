"""A plain statement of the Sotazen decoder in float64, one function per mechanism, written from the
design's equations and sharing no code with the package.  Everything runs on whole sequences on the
CPU; nothing is cached, so whatever the engine does with pages, slots and portions is held against
a computation that has none of them.

Notation: h [T, width] is a sublayer's input, p the position of a token (from 0), W x a projection
with W stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times the weight if there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, ..., d]: channels (2i, 2i+1), i < dims/2, turn by the angle p * base^(-2i/dims); the other
    channels pass."""
    if not dims:
        return x
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]                  # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T: int, window: Optional[int]) -> torch.Tensor:
    """[T, T] True where query i sees key j: 0 <= i - j (< window where there is one)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok = ok & (i - j < window)
    return ok


def softmax_rows(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax over the visible keys of scores [H, T, T]; with `sink` [H] the denominator also holds
    exp(sink_h), a term without key or value."""
    s = scores.masked_fill(~mask[None], -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.reshape(-1, 1, 1))
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.reshape(-1, 1, 1) - m)
    return e / den


def two_map_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: Optional[float],
                      window: Optional[int]) -> torch.Tensor:
    """q [T, H, 2, d], k [T, G, 2, d], v [T, G, vd] (already normed and rotated): for every head and map an
    ordinary softmax attention of its own over the values of the head's kv head; [T, H, 2, vd]."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    rep = H // G
    mask = visible(T, window)
    vh = v.permute(1, 0, 2).repeat_interleave(rep, dim=0)                  # [H, T, vd]
    out = []
    for j in range(2):
        qj = q[:, :, j].permute(1, 0, 2)                                   # [H, T, d]
        kj = k[:, :, j].permute(1, 0, 2).repeat_interleave(rep, dim=0)     # [H, T, d]
        s = (qj @ kj.transpose(1, 2)) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        out.append(softmax_rows(s, mask) @ vh)
    return torch.stack(out, dim=2).permute(1, 0, 2, 3)                     # [T, H, 2, vd]


def map_weight(w: Mapping[str, torch.Tensor], diff: float) -> float:
    """lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff."""
    return math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + diff


def difference_of_maps(maps: torch.Tensor, lam: float, diff: float, eps: float) -> torch.Tensor:
    """maps [T, H, 2, vd] -> (1 - diff) * rms_head(a1 - lam a2), [T, H, vd]."""
    return rms_norm(maps[:, :, 0] - lam * maps[:, :, 1], None, eps) * (1.0 - diff)


def differential_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values, the second subtracted with a learned weight."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    pos = torch.arange(T)

    def proj(name):
        y = h @ w[name].T
        return y + w[name + ".b"] if name + ".b" in w else y
    q = proj("q").reshape(T, H, 2, d)
    k = proj("k").reshape(T, G, 2, d)
    v = proj("v").reshape(T, G, vd)
    if "q.norm" in w:
        q = rms_norm(q, w["q.norm"], eps)
        k = rms_norm(k, w["k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, pos, rot["dims"], rot["base"])
        k = rotate_pairs(k, pos, rot["dims"], rot["base"])
    maps = two_map_attention(q, k, v, m["scale"], m.get("softcap"), (m.get("mask") or {}).get("size"))
    diff = float(m["diff"])
    o = difference_of_maps(maps, map_weight(w, diff), diff, eps).reshape(T, H * vd)
    if "g" in w:
        o = o * torch.sigmoid(h @ w["g"].T)
    y = o @ w["o"].T
    return y + w["o.b"] if "o.b" in w else y


def decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                     state: Optional[torch.Tensor] = None):
    """q, k [T, H, d], v [T, H, vd], decay [H]: S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, token by
    token from `state` [H, d, vd] (zero if None).  Returns (o [T, H, vd], the last state)."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=F64) if state is None else state.clone()
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


def lightning_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head, silu on q, k and v, a norm over all heads and a gate."""
    T = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w["q"].T).reshape(T, H, d)
    k = silu(h @ w["k"].T).reshape(T, H, d)
    v = silu(h @ w["v"].T).reshape(T, H, vd)
    out, _ = decay_recurrence(q, k, v, torch.tensor([float(x) for x in m["decay"]], dtype=F64))
    o = rms_norm(out.reshape(T, H * vd), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def latent_scores_attention(q_plain: torch.Tensor, q_rot: torch.Tensor, c: torch.Tensor, k_rot: torch.Tensor,
                            uk: torch.Tensor, uv: torch.Tensor, scale: float, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q_plain [T, H, d], q_rot [T, H, r] (rotated), c [T, rank] (normed), k_rot [T, r] (rotated), uk [H*d, rank],
    uv [H*vd, rank]: keys and values of every head are made from c; causal softmax with exp(sink_h) in the
    denominator; [T, H, vd]."""
    T, H, d = q_plain.shape
    k_plain = (c @ uk.T).reshape(T, H, d)
    v = (c @ uv.T).reshape(T, H, -1)
    s = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)
    p = softmax_rows(s * scale, visible(T, None), sink)
    return torch.einsum("hij,jhv->ihv", p, v)


def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float) -> torch.Tensor:
    """Keys and values made from one normed low-rank vector per token, plus one rotated key part shared by
    the heads; a softmax whose denominator holds a learned term per head."""
    T = h.shape[0]
    H, d, r, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    base = (m.get("rot") or {}).get("base", 10000.0)
    q = (h @ w["q"].T).reshape(T, H, d + r)
    dkv = h @ w["dkv"].T
    c = rms_norm(dkv[:, :rank], w["dkv.norm"], eps)
    o = latent_scores_attention(q[..., :d], rotate_pairs(q[..., d:], pos, r, base), c,
                                rotate_pairs(dkv[:, rank:], pos, r, base), w["uk"], w["uv"], m["scale"], w.get("sink"))
    return o.reshape(T, H * vd) @ w["o"].T


def feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    """down( relu(up h)^2 )."""
    return (torch.relu(h @ w["up"].T) ** 2) @ w["down"].T


MIXERS = {"attention": differential_attention, "lightning": lightning_attention,
          "latent_attention": latent_attention}


def _sub(weights: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in weights.items() if k.startswith(prefix)}


def read_model_folder(folder: str):
    """(config.json as a dict, tensors by name) of a model folder."""
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))


def forward(cfg: Mapping, weights: Mapping[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  `taps` collects the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    alpha = float(cfg.get("postln_alpha", 1.0))
    E = weights["embed"].to(F64)
    x = E[torch.tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        y = MIXERS[layer["type"]](x, _sub(weights, f"l{i}.mix."), layer["mixer"], eps)
        x = rms_norm(alpha * x + y, weights[f"l{i}.norm1"].to(F64), eps)
        if layer.get("mlp") is not None:
            y = feed_forward(x, _sub(weights, f"l{i}.mlp."))
            x = rms_norm(alpha * x + y, weights[f"l{i}.norm2"].to(F64), eps)
        if taps is not None:
            taps.append(x.clone())
    x = rms_norm(x, weights["final.norm"].to(F64), eps)
    return x @ E.T
