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
    rep = H // G
    mask = visible(T, (m.get("mask") or {}).get("size"))
    diff = float(m["diff"])
    lam = (math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + diff)
    maps = []
    for j in range(2):
        qj = q[:, :, j].permute(1, 0, 2)                                  # [H, T, d]
        kj = k[:, :, j].permute(1, 0, 2).repeat_interleave(rep, dim=0)    # [H, T, d]
        s = (qj @ kj.transpose(1, 2)) * m["scale"]
        cap = m.get("softcap")
        if cap:
            s = cap * torch.tanh(s / cap)
        p = softmax_rows(s, mask)
        maps.append(p @ v.permute(1, 0, 2).repeat_interleave(rep, dim=0))  # [H, T, vd]
    o = maps[0] - lam * maps[1]
    o = rms_norm(o, None, eps) * (1.0 - diff)
    o = o.permute(1, 0, 2).reshape(T, H * vd)
    if "g" in w:
        o = o * torch.sigmoid(h @ w["g"].T)
    y = o @ w["o"].T
    return y + w["o.b"] if "o.b" in w else y


def lightning_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float) -> torch.Tensor:
    """S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per head, token by token from a zero state."""
    T = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w["q"].T).reshape(T, H, d)
    k = silu(h @ w["k"].T).reshape(T, H, d)
    v = silu(h @ w["v"].T).reshape(T, H, vd)
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=F64)
    S = torch.zeros(H, d, vd, dtype=F64)
    out = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(out.reshape(T, H * vd), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float) -> torch.Tensor:
    """Keys and values made from one normed low-rank vector per token, plus one rotated key part shared by
    the heads; a softmax whose denominator holds a learned term per head."""
    T = h.shape[0]
    H, d, r, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    base = m["rot"]["base"]
    q = (h @ w["q"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, r, base)
    dkv = h @ w["dkv"].T
    c = rms_norm(dkv[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_pairs(dkv[:, rank:], pos, r, base)                     # [T, r]
    k_plain = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, vd)
    s = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)
    p = softmax_rows(s * m["scale"], visible(T, None), w["sink"] if "sink" in w else None)
    o = torch.einsum("hij,jhv->ihv", p, v).reshape(T, H * vd)
    return o @ w["o"].T


def feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    """down( relu(up h)^2 )."""
    return (torch.relu(h @ w["up"].T) ** 2) @ w["down"].T


MIXERS = {"attention": differential_attention, "lightning": lightning_attention,
          "latent_attention": latent_attention}


def _sub(weights: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in weights.items() if k.startswith(prefix)}


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
