"""A plain statement of the Linedra decoder in float64, one function per mechanism, written from the
design's equations and sharing no code with the package.  Everything runs on whole sequences on the
CPU; nothing is cached, so whatever the engine does with pages, slots and portions is held against
a computation that has none of them.

Notation: h [T, width] is a sublayer's input, p the position of a token (from 0), W x a projection
with W stored [out, in]; a model is (cfg, tensors): config.json's dict and name -> tensor.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, offset: float = 0.0) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times (offset + weight) if there is a weight."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * (offset + weight)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], w [C, taps]: y_t = sum_j w[:, j] x_(t - taps + 1 + j) (+ bias), zeros before the start; the
    last column of w meets the current token."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * x[: T - back]
    return y if bias is None else y + bias


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, ..., d]: channel i turns with channel i + dims/2 (i < dims/2) by the angle p * base^(-2i/dims);
    channels from dims on pass."""
    if not dims:
        return x
    half = dims // 2
    out = x.clone()
    freq = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(T: int, window: Optional[int]) -> torch.Tensor:
    """[T, T] True where query i sees key j: 0 <= i - j (< window where there is one)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok = ok & (i - j < window)
    return ok


def softmax_with_sink(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
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


def distance_slopes(heads: int) -> torch.Tensor:
    """slope_h = 2^(-8 (h + 1) / H)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


def attend_with_distance_bias(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                              window: Optional[int], sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, vd]: score(i, j) = q_i . k_j * scale - slope_h (i - j) over the keys the
    window leaves, softmax with the sink's term; [T, H, vd]."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    qh = q.permute(1, 0, 2)
    kh = k.permute(1, 0, 2).repeat_interleave(H // G, dim=0)
    vh = v.permute(1, 0, 2).repeat_interleave(H // G, dim=0)
    s = (qh @ kh.transpose(1, 2)) * scale
    i = torch.arange(T, dtype=F64)
    s = s - distance_slopes(H)[:, None, None] * (i[:, None] - i[None, :])[None]
    p = softmax_with_sink(s, visible(T, window), sink)
    return (p @ vh).permute(1, 0, 2)


def biased_window_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping) -> torch.Tensor:
    """Grouped-query attention without rotation: score = q.k * scale - slope_h (i - j) inside a window, a
    learned sink in the softmax, every head's output times sigmoid of one number of W_g h, then W_o."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = (h @ w["v"].T).reshape(T, G, vd)
    window = m["mask"]["size"] if m.get("mask") else None
    o = attend_with_distance_bias(q, k, v, m["scale"], window, w["sink"])       # [T, H, vd]
    gate = torch.sigmoid(h @ w["g"].T)                                    # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * vd) @ w["o"].T


def gated_recurrent_unit(u: torch.Tensor, w: Mapping[str, torch.Tensor], blocks: int) -> torch.Tensor:
    """u [T, C] -> S [T, C]: per block b of channels r = sigmoid(ra[b] u_b + ra.b[b]), i = sigmoid(ri[b] u_b +
    ri.b[b]); a = exp(-8 r softplus(lam)); S_t = a S_(t-1) + sqrt(1 - a^2) i u, from S = 0."""
    T, C = u.shape
    ub = u.reshape(T, blocks, C // blocks)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ra"]) + w["ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ri"]) + w["ri.b"]).reshape(T, C)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(w["lam"]))
    x = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(C, dtype=F64)
    out = []
    for t in range(T):
        S = a[t] * S + x[t]
        out.append(S)
    return torch.stack(out)


def recurrent_block(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping) -> torch.Tensor:
    """y = gelu_tanh(W_y h + b); u = conv(W_x h + b) + b_conv; out = W_o (S(u) * y)."""
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_conv(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    return (gated_recurrent_unit(u, w, m["blocks"]) * y) @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping) -> torch.Tensor:
    left = {k[len("left."):]: v for k, v in w.items() if k.startswith("left.")}
    right = {k[len("right."):]: v for k, v in w.items() if k.startswith("right.")}
    return (m["left_scale"] * biased_window_attention(h, left, m["left"])
            + m["right_scale"] * recurrent_block(h, right, m["right"]))


def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float) -> torch.Tensor:
    """Queries through a normed low-rank vector; keys and values of all heads made from one normed low-rank
    vector c a token plus rot_dim rotated key channels all heads share; causal, a sink, an output gate."""
    T = h.shape[0]
    H, d, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    base = m["rot"]["base"] if m.get("rot") else 10000.0
    if "dq" in w:
        q = rms_norm(h @ w["dq"].T, w["dq.norm"], eps) @ w["uq"].T
    else:                                                                 # no low-rank vector: q = W_q h
        q = h @ w["q"].T
    q = q.reshape(T, H, d + rd)
    q_plain, q_rot = q[..., :d], rotate_half(q[..., d:], pos, rd, base)
    dkv = h @ w["dkv"].T
    c = rms_norm(dkv[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, rank:], pos, rd, base)                      # [T, rd], one for all heads
    k_plain = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, vd)
    s = torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, k_rot)
    p = softmax_with_sink(s * m["scale"], visible(T, None), w["sink"])
    o = torch.einsum("hts,shv->thv", p, v).reshape(T, H * vd)
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def route(z: torch.Tensor, top: int):
    """Router logits z [T, E] -> (ids [T, top], weights [T, top]): the `top` largest logits (the lower index
    among equals), weights their softmax among themselves."""
    vals, ids = torch.sort(z, dim=-1, descending=True, stable=True)
    vals, ids = vals[:, :top], ids[:, :top]
    return ids, torch.softmax(vals, dim=-1)


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def mixture_of_experts(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, router_input=None) -> torch.Tensor:
    z = (h if router_input is None else router_input) @ w["router"].T
    ids, weights = route(z, m["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(ids[t].tolist(), weights[t]):
            out[t] += p * expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], m["expert"]["limit"])
    return out


def sub(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def layer(cfg: Mapping, tensors: Mapping[str, torch.Tensor], i: int, x: torch.Tensor) -> torch.Tensor:
    """One layer on its input x (the depth average that the layer before left): norms around both sublayers,
    the input convolution in front of the mixer.  Returns the layer's own result, before it is averaged."""
    spec, eps, mult = cfg["layers"][i], cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    w = sub(tensors, f"l{i}.")
    h = rms_norm(x, w["norm1"], eps, 1.0)
    h = h + causal_conv(h, w["canon1"])
    mix = sub(w, "mix.")
    if spec["type"] == "parallel":
        y = parallel_mixer(h, mix, spec["mixer"])
    elif spec["type"] == "latent_attention":
        y = latent_attention(h, mix, spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    x = x + mult * rms_norm(y, w["norm1b"], eps, 1.0)
    if spec.get("mlp") is not None:
        y = mixture_of_experts(rms_norm(x, w["norm2"], eps, 1.0), sub(w, "mlp."), spec["mlp"])
        x = x + mult * rms_norm(y, w["norm2b"], eps, 1.0)
    return x


def forward(cfg: Mapping, tensors: Mapping[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  `taps`, if a list, receives what every layer hands on (after the
    depth average)."""
    ids = torch.tensor(tokens, dtype=torch.long)
    table = tensors["embed"].to(F64)
    x = table[ids] * cfg.get("embedding", {}).get("scale", 1.0)
    results = [x]                                                         # X_0, X_1, ...
    for i in range(len(cfg["layers"])):
        results.append(layer(cfg, tensors, i, x))
        dwa = tensors[f"l{i}.dwa"].to(F64)
        x = sum(dwa[j] * results[j] for j in range(i + 2))
        if taps is not None:
            taps.append(x)
    n = rms_norm(x, tensors["final.norm"].to(F64), cfg["norm"]["eps"], 1.0)
    logits = n @ table.T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg: Mapping, tensors: Mapping[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(forward(cfg, tensors, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


def read_model_folder(folder: str):
    """(config.json as a dict, tensors by name) of a model folder."""
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))
