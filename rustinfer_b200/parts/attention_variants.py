"""Two more attention mixers over the paged cache, beside `gqa_attention`:

    differential_attention   every head has two softmax maps, with queries and keys of their own, over one
                             set of values; out = rms_head(a1 - lambda a2) * (1 - diff), gated and projected
    latent_attention         keys and values of all heads are made from one cached low-rank vector per token
                             (plus a few rotated key channels the heads share); only that vector is cached

Both run on the fp32-arithmetic attention kernels in both engine precisions: scores, softmax weights and
the weighted sum of values are 32-bit there.  The reference engine has one attention
(crates/infer-worker/src/components/attention.rs:21-37); these are parts of the same kind with caches of
their own shapes.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import (BuildContext, Mixer, PagedKV, PagedLayerCache, ParamDecl, POSITIONS, StepContext,
                   register_mixer, single_token_entries, token_tiles)
from .linear import Linear
from .spec import PartSpec


class PlainAttend:
    """How a mixer sends its queries to the attention kernels with fp32 scores and softmax weights.  The bfloat16
    engine: prompt portions go to the tensor-core kernel in tiles of 64 (token, head) rows (where the sizes are
    multiples of 16).  Entries of one token go there too where eight or more query heads share a key head (one
    cached row for all heads, say: the arithmetic of so many heads a key outgrows the fp32 pipes), else to the
    kernel that reads a key head once for all its query heads (where it takes the geometry).  Both cut the keys
    into ranges when few CTAs would walk many keys.  What neither takes runs on the fp32-arithmetic kernel in
    tiles of 16 query rows.  The 32-bit engine uses that last kernel alone, whose sums do not depend on how the
    tokens were cut into steps."""
    MAX_SPLITS = 16             # of the one-CTA-a-key-head kernel
    ROWS_MAX_SPLITS = 32        # of the tensor-core kernel

    def __init__(self, ctx: BuildContext, heads: int, kv_heads: int, head_dim: int, value_dim: int, maps: int = 1,
                 value_in_key: bool = False, window: Optional[int] = None):
        self.ctx = ctx
        self.Hq, self.Hkv, self.hd, self.vd, self.maps = heads, kv_heads, head_dim, value_dim, maps
        self.value_in_key, self.window = value_in_key, window
        fast = (ctx.dtype == torch.bfloat16 and os.environ.get("RUSTINFER_B200_BLOCK_ATTENTION", "fast") != "plain")
        self.rows = fast and K.attention_rows_supports(head_dim, value_dim, value_in_key)
        group = heads // (kv_heads * maps)
        self.rows_single = self.rows and group >= 8
        self.fast_single = (fast and not self.rows_single
                            and K.attention_single_supports(heads, kv_heads, head_dim, value_dim, maps))
        rows = K.attention_rows_tokens_per_tile(heads, kv_heads, head_dim, value_dim, maps) if self.rows else 16
        self._single = self.part = None
        if self.fast_single:
            self._single = single_token_entries()
            key = ("single_scratch", heads, value_dim)
            if key not in ctx.shared:
                n = K.attention_single_scratch_floats(ctx.max_batch_seqs, heads, value_dim, self.MAX_SPLITS)
                ctx.shared[key] = torch.empty(n, dtype=torch.float32, device=ctx.device)
            self.part = ctx.shared[key]
        elif self.rows_single:
            self._single = single_token_entries()
            self.ctas_per_tile = kv_heads * maps * -(-group // 64)
            # ranges are made until the CTAs fill the SMs once: one CTA more than fit at once costs a second turn
            self.slots = ctx.num_sms * K.attention_rows_ctas_per_sm(head_dim, value_dim, value_in_key,
                                                                    torch.float32 if maps > 1 else ctx.dtype)
            key = ("rows_scratch", value_dim)
            if key not in ctx.shared or ctx.shared[key].numel() < self.slots * 64 * (value_dim + 2):
                ctx.shared[key] = torch.empty(self.slots * 64 * (value_dim + 2), dtype=torch.float32, device=ctx.device)
            self.part = ctx.shared[key]
            if "zero_tok0" not in ctx.shared:
                ctx.shared["zero_tok0"] = torch.zeros(ctx.max_batch_seqs + 4, dtype=torch.int32, device=ctx.device)
            self.zero_tok0 = ctx.shared["zero_tok0"]
        self._tiles = token_tiles(rows, skip_single_token=self._single is not None)

    def step_indices(self):
        return [self._tiles] if self._single is None else [self._single, self._tiles]

    def _span(self, max_kv_len: int) -> int:
        return min(max_kv_len, self.window) if self.window else max_kv_len

    def _splits(self, n_single: int, max_kv_len: int) -> int:
        want = -(-4 * self.ctx.num_sms // max(1, n_single * self.Hkv * self.maps))
        return max(1, min(want, -(-self._span(max_kv_len) // 128), self.MAX_SPLITS))

    def _rows_splits(self, n_single: int, max_kv_len: int) -> int:
        ctas = max(1, n_single * self.ctas_per_tile)
        return max(1, min(self.slots // ctas, -(-self._span(max_kv_len) // 128), self.ROWS_MAX_SPLITS))

    def __call__(self, q: torch.Tensor, out: torch.Tensor, step: StepContext, cache: PagedLayerCache, scale: float,
                 softcap: Optional[float] = None, sink_values: Optional[torch.Tensor] = None,
                 slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
        g = step.groups[cache.group]
        opts = dict(value_dim=self.vd, sink=sink_values is not None, softcap=softcap, sink_values=sink_values,
                    maps=self.maps, value_in_key=self.value_in_key, slopes=slopes)
        if self._single is not None:
            (single,) = step.index(self._single)
            if single.numel() and self.fast_single:
                K.attention_single(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, single, self.Hq, self.Hkv,
                                   self.hd, scale, self.window, None, splits=self._splits(single.numel(), step.max_kv_len),
                                   part=self.part, **opts)
            elif single.numel():
                K.attention_rows(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, single,
                                 self.zero_tok0[: single.numel()], self.Hq, self.Hkv, self.hd, scale, self.window,
                                 splits=self._rows_splits(single.numel(), step.max_kv_len), part=self.part, **opts)
        tile_entry, tile_tok0 = step.index(self._tiles)
        if tile_entry.numel():
            if self.rows:
                K.attention_rows(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry, tile_tok0,
                                 self.Hq, self.Hkv, self.hd, scale, self.window, **opts)
            else:
                K.attention_plain(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry, tile_tok0,
                                  self.Hq, self.Hkv, self.hd, scale, self.window, None, **opts)
        return out


def project_out(o: Linear, y: torch.Tensor, add_to: Optional[torch.Tensor]) -> torch.Tensor:
    """y W_o^T in fp32; with `add_to` (fp32 [T, hidden]) added into it (inside the product where the weight can) and
    `add_to` returned."""
    if add_to is None:
        return o(y, out_dtype=torch.float32)
    if not o.add_into(y, add_to):
        K.residual_add(add_to, o(y, out_dtype=torch.float32))
    return add_to


def _shared_position(ctx: BuildContext, spec: Optional[PartSpec]):
    if spec is None:
        return None
    key = ("position", spec.key(), ctx.max_model_len)
    if key not in ctx.shared:
        part = POSITIONS.build(spec)
        part.prepare(ctx)
        ctx.shared[key] = part
    return ctx.shared[key]


@register_mixer("differential_attention")
class DifferentialAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim (of one map's queries and keys), value_dim,
    scale, diff, softcap (None: scores are not capped), window (None: every earlier key), position
    (PartSpec of a rotary encoding over head_dim, or None), qk_norm_eps (None: q and k are not normed),
    norm_eps (of the norm after the difference), bias (q, k, v and o have biases), gate (the heads'
    outputs are multiplied by sigmoid(W_g h)), tensor_names.

    q [H*2*hd] and k [G*2*hd] come head by head as [map 1, map 2]; each (head, map) is normed by its own
    root mean square (weights `q.norm`, `k.norm` [hd] shared by all), rotated, and attends over the same
    values as the other map: score = softcap * tanh(q.k * scale / softcap), softmax over the window.
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff is one number of the layer (formed once, at load).
    out = W_o( (1 - diff) * rms_head(a1 - lambda a2) * sigmoid(W_g h) ) + b_o.  The cache keeps 2G key
    heads and G value heads; the two maps' results leave the attention kernel in fp32."""
    graph_safe = True

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p.get("num_kv_heads") or p["num_heads"])
        self.hd, self.vd = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"])
        self.scale, self.diff = float(p["scale"]), float(p["diff"])
        self.softcap = float(p["softcap"]) if p.get("softcap") else None
        self.window = int(p["window"]) if p.get("window") else None
        self.qk_norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") is not None else None
        self.norm_eps = float(p["norm_eps"])
        self.bias, self.gate = bool(p.get("bias", False)), bool(p.get("gate", False))
        self.tensor_names = dict(p.get("tensor_names") or {})
        self.position_spec: Optional[PartSpec] = p.get("position")
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} kv heads")
        if not (1 <= self.hd <= 512 and 1 <= self.vd <= 512):
            raise ValueError(f"head sizes {self.hd}, {self.vd}: the attention kernel takes sizes up to 512")
        self.nq, self.nk, self.nv = self.H * 2 * self.hd, self.G * 2 * self.hd, self.G * self.vd

    def _name(self, local: str) -> str:
        return self.tensor_names.get(local, local)

    def param_decls(self) -> Dict[str, ParamDecl]:
        n = self._name
        d = {n("q"): ParamDecl((self.nq, self.hidden)), n("k"): ParamDecl((self.nk, self.hidden)),
             n("v"): ParamDecl((self.nv, self.hidden)), n("o"): ParamDecl((self.hidden, self.H * self.vd))}
        for x in ("lq1", "lk1", "lq2", "lk2"):
            d[n(x)] = ParamDecl((self.hd,))
        if self.gate:
            d[n("g")] = ParamDecl((self.H * self.vd, self.hidden))
        if self.qk_norm_eps is not None:
            d[n("q.norm")] = ParamDecl((self.hd,), init="ones")
            d[n("k.norm")] = ParamDecl((self.hd,), init="ones")
        if self.bias:
            d[n("q.b")] = ParamDecl((self.nq,), init="zeros")
            d[n("k.b")] = ParamDecl((self.nk,), init="zeros")
            d[n("v.b")] = ParamDecl((self.nv,), init="zeros")
            d[n("o.b")] = ParamDecl((self.hidden,), init="zeros")
        return d

    def cache_need(self):
        return PagedKV(self.G, self.hd, self.window, value_dim=self.vd, key_maps=2)

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        self.attend = PlainAttend(ctx, 2 * self.H, self.G, self.hd, self.vd, maps=2, window=self.window)
        self.position = _shared_position(ctx, self.position_spec)

    def step_indices(self):
        return self.attend.step_indices()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._name
        parts = [tensors[n(x)] for x in (("q", "k", "v", "g") if self.gate else ("q", "k", "v"))]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.proj = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.o = Linear(tensors[n("o")], self.ctx.num_sms)
        self.q_norm = self.k_norm = self.qkv_bias = self.o_bias = None
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[n("q.norm")].contiguous()
            self.k_norm = tensors[n("k.norm")].to(self.q_norm.dtype).contiguous()
        if self.bias:
            self.qkv_bias = torch.cat([tensors[n(x)].to(torch.float32) for x in ("q.b", "k.b", "v.b")]).contiguous()
            self.o_bias = tensors[n("o.b")].to(torch.float32).contiguous()
        dot = lambda a, b: float((tensors[n(a)].double() * tensors[n(b)].double()).sum())
        self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff

    def forward(self, x: torch.Tensor, step: StepContext, cache: PagedLayerCache) -> torch.Tensor:
        T, dt = x.shape[0], self.ctx.dtype
        g = step.groups[cache.group]
        proj = self.proj(x, out_dtype=torch.float32)
        nqkv = self.nq + self.nk + self.nv
        q = torch.empty((T, self.nq), dtype=dt, device=x.device)
        pos = self.position
        K.qkv_prepare(proj[:, :nqkv], self.qkv_bias, self.q_norm, self.k_norm, 0 if self.qk_norm_eps is None else 1,
                      self.qk_norm_eps or 0.0, step.positions, pos.cos if pos else None, pos.sin if pos else None,
                      pos.rotary_dim if pos else 0, bool(pos and pos.layout == "interleaved"),
                      g.slot_of_token if cache.writes else None, cache.kv if cache.writes else None, q,
                      2 * self.H, 2 * self.G, self.hd, self.vd, True, value_heads=self.G)
        maps = torch.empty((T, 2 * self.H * self.vd), dtype=torch.float32, device=x.device)
        self.attend(q, maps, step, cache, self.scale, softcap=self.softcap)
        y = torch.empty((T, self.H * self.vd), dtype=dt, device=x.device)
        K.diff_combine(maps, self.lam, 1.0 - self.diff, self.norm_eps, proj[:, nqkv:] if self.gate else None, y,
                       self.H, self.vd)
        out = self.o(y, out_dtype=torch.float32)
        if self.o_bias is not None:
            K.bias_rows(out, self.o_bias)
        return out


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (plain query/key channels of a head), rot_dim (rotated ones),
    value_dim, kv_rank, scale, rot_base, norm_eps, sink (the softmax's denominator holds exp(sink_h), a
    learned number per head), q_rank (None: q = W_q h; else queries go through a low-rank vector of that size,
    c_q = rmsnorm(W_dq h) * `dq.norm`, q = W_uq c_q), rot_layout ("interleaved", the default: channels (2i, 2i+1)
    turn together; "half": (i, i + rot_dim/2)), gate (the heads' outputs are multiplied element by element with
    sigmoid(W_g h) before W_o), tensor_names.

    q = W_q h, per head [head_dim plain, rot_dim rotated].  W_dkv h = [kv_rank, rot_dim]: the first part,
    RMS-normed with `dkv.norm`, is the latent c; the second, rotated, is a key part all heads share.  A
    head's plain key is W_uk c and its value W_uv c, so with q' = W_uk^T q_plain the score is
    (q' . c + q_rot . k_rot) * scale and the output W_uv (sum_j p_j c_j): one cached row [c, k_rot] per
    token serves every head as key, and its first kv_rank channels as value.  Pairs (2i, 2i+1) of the
    rotated parts turn by p * rot_base^(-2i/rot_dim).  Causal; out = W_o on the heads' outputs.  The two
    products with W_uk and W_uv are batched library products over the heads."""
    graph_safe = True

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.hd, self.rd = int(p["num_heads"]), int(p["head_dim"]), int(p["rot_dim"])
        self.vd, self.rank = int(p["value_dim"]), int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.rot_base = float(p.get("rot_base", 10000.0))
        self.norm_eps = float(p["norm_eps"])
        self.sink = bool(p.get("sink", False))
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else None
        self.rot_layout = str(p.get("rot_layout", "interleaved"))
        if self.rot_layout not in ("half", "interleaved"):
            raise ValueError(f"rot_layout {self.rot_layout!r}: known are 'half' and 'interleaved'")
        self.gate = bool(p.get("gate", False))
        self.tensor_names = dict(p.get("tensor_names") or {})
        self.kd = self.rank + self.rd                       # a cached row
        if self.rd % 2 or self.rd < 0:
            raise ValueError("rot_dim is even")
        if not 1 <= self.kd <= 512:
            raise ValueError(f"kv_rank + rot_dim = {self.kd}: the attention kernel takes rows up to 512")

    def _name(self, local: str) -> str:
        return self.tensor_names.get(local, local)

    def param_decls(self) -> Dict[str, ParamDecl]:
        n = self._name
        nq = self.H * (self.hd + self.rd)
        d = {n("dkv"): ParamDecl((self.kd, self.hidden)), n("dkv.norm"): ParamDecl((self.rank,), init="ones"),
             n("uk"): ParamDecl((self.H * self.hd, self.rank)), n("uv"): ParamDecl((self.H * self.vd, self.rank)),
             n("o"): ParamDecl((self.hidden, self.H * self.vd))}
        if self.q_rank:
            d[n("dq")] = ParamDecl((self.q_rank, self.hidden))
            d[n("dq.norm")] = ParamDecl((self.q_rank,), init="ones")
            d[n("uq")] = ParamDecl((nq, self.q_rank))
        else:
            d[n("q")] = ParamDecl((nq, self.hidden))
        if self.gate:
            d[n("g")] = ParamDecl((self.H * self.vd, self.hidden))
        if self.sink:
            d[n("sink")] = ParamDecl((self.H,), init="zeros")
        return d

    def cache_need(self):
        return PagedKV(1, self.kd, None, value_dim=self.rank, value_in_key=True)

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        self.attend = PlainAttend(ctx, self.H, 1, self.kd, self.rank, value_in_key=True)
        self.position = _shared_position(ctx, PartSpec("rope", {
            "head_dim": self.rd, "rotary_dim": self.rd, "theta": self.rot_base, "scaling": None,
            "layout": self.rot_layout})) if self.rd else None

    def step_indices(self):
        return self.attend.step_indices()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._name
        # one product for everything that reads the mixer's input: queries (or their low-rank vector), the
        # cached row, the gate
        parts = [tensors[n("dq") if self.q_rank else n("q")], tensors[n("dkv")]] + ([tensors[n("g")]] if self.gate else [])
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.proj = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.uq = self.q_norm = None
        if self.q_rank:
            self.uq = Linear(tensors[n("uq")], self.ctx.num_sms)
            self.q_norm = tensors[n("dq.norm")].to(torch.float32).contiguous()
        self.c_norm = tensors[n("dkv.norm")].contiguous()
        act = self.ctx.dtype
        self.w_uk = tensors[n("uk")].to(act).view(self.H, self.hd, self.rank).contiguous()
        self.w_uv = tensors[n("uv")].to(act).view(self.H, self.vd, self.rank).transpose(1, 2)     # [H, rank, vd]
        self.o = Linear(tensors[n("o")], self.ctx.num_sms)
        self.sink_values = tensors[n("sink")].to(torch.float32).contiguous() if self.sink else None
        if not self.rd:
            self._no_rot = torch.zeros((self.ctx.max_model_len, 0), dtype=torch.float32, device=self.ctx.device)

    def forward(self, x: torch.Tensor, step: StepContext, cache: PagedLayerCache) -> torch.Tensor:
        T, dt, H = x.shape[0], self.ctx.dtype, self.H
        g = step.groups[cache.group]
        proj = self.proj(x, out_dtype=torch.float32)
        q_plain = torch.empty((T, H * self.hd), dtype=dt, device=x.device)
        q_full = torch.empty((T, H * self.kd), dtype=dt, device=x.device)
        cos, sin = (self.position.cos, self.position.sin) if self.position is not None else (self._no_rot, self._no_rot)
        nq = self.q_rank or H * (self.hd + self.rd)
        if self.q_rank:
            cq = torch.empty((T, self.q_rank), dtype=dt, device=x.device)
            K.rms_sandwich(proj[:, :nq], None, None, None, self.q_norm, cq, self.norm_eps)
            queries, low = self.uq(cq, out_dtype=torch.float32), proj[:, nq: nq + self.kd]
        else:
            queries, low = proj[:, : nq + self.kd], None
        K.latent_prepare(queries, self.c_norm, self.norm_eps, step.positions, cos, sin,
                         g.slot_of_token if cache.writes else None, cache.kv if cache.writes else None,
                         q_plain, q_full, H, self.hd, self.rd, self.rank, low=low,
                         interleaved=self.rot_layout == "interleaved")
        # q' of every head into the first kv_rank channels of its row of q_full
        torch.bmm(q_plain.view(T, H, self.hd).transpose(0, 1), self.w_uk,
                  out=q_full.view(T, H, self.kd)[:, :, : self.rank].transpose(0, 1))
        lat = torch.empty((T, H * self.rank), dtype=dt, device=x.device)
        self.attend(q_full, lat, step, cache, self.scale, sink_values=self.sink_values)
        y = torch.empty((T, H * self.vd), dtype=dt, device=x.device)
        torch.bmm(lat.view(T, H, self.rank).transpose(0, 1), self.w_uv, out=y.view(T, H, self.vd).transpose(0, 1))
        if self.gate:
            gated = torch.empty_like(y)
            K.sigmoid_gate(y, proj[:, nq + self.kd:], 1, gated)
            y = gated
        return self.o(y, out_dtype=torch.float32)


@register_mixer("distance_bias_attention")
class DistanceBiasAttention(Mixer):
    """Grouped-query attention without rotation, whose scores carry a linear distance bias:

        score(i, j) = q_i . k_j * scale - slope_h * (i - j),    slope_h = 2^(-slope_exponent * (h + 1) / H)

    for head h of H, over the keys of a sliding window (None: every earlier key).  params: hidden_size, num_heads,
    num_kv_heads, head_dim, value_dim, scale, window, slope_exponent (default 8), sink (the softmax's denominator
    holds exp(sink_h), a learned number per head with no key or value), head_gate (head h's output is multiplied
    by sigmoid of the h-th of H numbers W_g x), tensor_names.  Tensors: q, k, v, o, and `sink` [H], `g` [H, hidden]
    where asked for; no biases.  q, k, v and the gates are one product of the input; scores, softmax weights and
    their product with the values are fp32 in both engines (the kernels `PlainAttend` picks).  Beside another mixer
    (`parallel_mixers`) it takes the joint product's columns as `proj`, and with a gate a head an `out_scale` on what
    its output product reads and an `add_to` that product is added into."""
    graph_safe = True
    joins_input = True

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p.get("num_kv_heads") or p["num_heads"])
        self.hd, self.vd = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"])
        self.scale = float(p["scale"])
        self.window = int(p["window"]) if p.get("window") else None
        self.slope_exponent = float(p.get("slope_exponent", 8.0))
        self.sink, self.head_gate = bool(p.get("sink", False)), bool(p.get("head_gate", False))
        self.tensor_names = dict(p.get("tensor_names") or {})
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} kv heads")
        if not (1 <= self.hd <= 512 and 1 <= self.vd <= 512):
            raise ValueError(f"head sizes {self.hd}, {self.vd}: the attention kernel takes sizes up to 512")
        self.nq, self.nk, self.nv = self.H * self.hd, self.G * self.hd, self.G * self.vd
        self.scales_output = self.head_gate          # the gate's kernel is where a factor on the output is free

    def _name(self, local: str) -> str:
        return self.tensor_names.get(local, local)

    def param_decls(self) -> Dict[str, ParamDecl]:
        n = self._name
        d = {n("q"): ParamDecl((self.nq, self.hidden)), n("k"): ParamDecl((self.nk, self.hidden)),
             n("v"): ParamDecl((self.nv, self.hidden)), n("o"): ParamDecl((self.hidden, self.H * self.vd))}
        if self.sink:
            d[n("sink")] = ParamDecl((self.H,), init="zeros")
        if self.head_gate:
            d[n("g")] = ParamDecl((self.H, self.hidden))
        return d

    def cache_need(self):
        return PagedKV(self.G, self.hd, self.window, value_dim=self.vd if self.vd != self.hd else None)

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        self.attend = PlainAttend(ctx, self.H, self.G, self.hd, self.vd, window=self.window)
        slopes = [2.0 ** (-self.slope_exponent * (h + 1) / self.H) for h in range(self.H)]
        self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(ctx.device)

    def step_indices(self):
        return self.attend.step_indices()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._name
        parts = [tensors[n(x)] for x in (("q", "k", "v", "g") if self.head_gate else ("q", "k", "v"))]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.proj = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.o = Linear(tensors[n("o")], self.ctx.num_sms)
        self.sink_values = tensors[n("sink")].to(torch.float32).contiguous() if self.sink else None

    def forward(self, x: torch.Tensor, step: StepContext, cache: PagedLayerCache, proj: Optional[torch.Tensor] = None,
                out_scale: float = 1.0, add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, dt = x.shape[0], self.ctx.dtype
        g = step.groups[cache.group]
        if proj is None:
            proj = self.proj(x, out_dtype=torch.float32)
        nqkv = self.nq + self.nk + self.nv
        q = torch.empty((T, self.nq), dtype=dt, device=x.device)
        K.qkv_prepare(proj[:, :nqkv], None, None, None, 0, 0.0, step.positions, None, None, 0, False,
                      g.slot_of_token if cache.writes else None, cache.kv if cache.writes else None, q,
                      self.H, self.G, self.hd, self.vd, True)
        if self.head_gate:
            o = torch.empty((T, self.H * self.vd), dtype=torch.float32, device=x.device)
            self.attend(q, o, step, cache, self.scale, sink_values=self.sink_values, slopes=self.slopes)
            y = torch.empty((T, self.H * self.vd), dtype=dt, device=x.device)
            K.sigmoid_gate(o, proj[:, nqkv:], self.vd, y, scale=out_scale)
        else:
            if out_scale != 1.0:
                raise ValueError("a factor on the output rides on the heads' gate; this mixer has none")
            y = torch.empty((T, self.H * self.vd), dtype=dt, device=x.device)
            self.attend(q, y, step, cache, self.scale, sink_values=self.sink_values, slopes=self.slopes)
        return project_out(self.o, y, add_to)
