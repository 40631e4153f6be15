"""Mixers that keep a matrix per head instead of keys and values: the state S [key channel,
value channel] of every live request sits in a slot of a fixed-state cache group, in fp32, and a
step walks each entry's tokens through the recurrence from where the last step left it.  A whole
prompt, a portion of one and a single decoded token are the same kernel launch.

    gated_linear_attention   S_t = diag(alpha_t) S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t
                             alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau),  q scaled by key_dim^(-1/2);
                             out = W_o( rms_head(o) * w * silu(W_g h) )
    delta_rule               S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T,  o_t = S_t^T r_t
                             u = k / sqrt(|k|^2 + unit_eps),  w = exp(-decay_rate * sigmoid(W_w2 tanh(W_w1 h) + w0)),
                             a = sigmoid(W_a h + b);  out = W_o( rms_head(o) * w * sigmoid(W_g h) )

The projections of one input are one matrix product (rows of the weights joined); the low-rank
pair that makes the decay is two small products, the second with fp32 output.  Decays, gates of
the recurrence, unit keys, the state and every sum over key channels are fp32 in both engine
precisions.  The reference engine has no such mixer (its only one is
crates/infer-worker/src/components/attention.rs); these stand beside `gqa_attention` as parts of
the same kind.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from .base import FixedState, Mixer, ParamDecl, StateLayerCache, StepContext, register_mixer
from .linear import Linear


class _StateMixer(Mixer):
    """What the two recurrences share: names, the joined projection, the output path."""
    graph_safe = True
    joined: List[str] = []                      # local names of the projections of the mixer's input, in order

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.dk = int(p["key_dim"])
        self.dv = int(p.get("value_dim") or self.dk)
        self.norm_eps = float(p["norm_eps"])
        self.rank = int(p["decay_rank"]) if p.get("decay_rank") else -1     # -1: whatever the file has
        self.tensor_names = dict(p.get("tensor_names") or {})
        if not (1 <= self.dk <= 512 and self.dv >= 1):
            raise ValueError(f"key size {self.dk}: the recurrence kernels take key sizes up to 512")

    def _name(self, local: str) -> str:
        return self.tensor_names.get(local, local)

    def cache_need(self):
        # a request's state: per head and value channel the column of S over the key channels, padded
        # to the rows the kernel keeps (the padding stays zero)
        return FixedState((self.H, self.dv, K.recurrent_state_rows(self.dk)), "float32")

    def _widths(self) -> Dict[str, int]:
        raise NotImplementedError

    def _load_joined(self, tensors: Dict[str, torch.Tensor]) -> None:
        parts = [tensors[self._name(n)] for n in self.joined]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.proj = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.cols = {}
        at = 0
        for n in self.joined:
            self.cols[n] = (at, at + self._widths()[n])
            at += self._widths()[n]

    def _split(self, proj: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {n: proj[:, a:b] for n, (a, b) in self.cols.items()}

    def _check_rank(self, first: torch.Tensor, second: torch.Tensor, what: str) -> None:
        if first.shape[0] != second.shape[1]:
            raise ValueError(f"{what}: the low-rank pair's sizes {tuple(first.shape)} and {tuple(second.shape)} do not meet")


@register_mixer("gated_linear_attention")
class GatedLinearAttention(_StateMixer):
    """params: hidden_size, num_heads, key_dim, value_dim, tau, norm_eps, decay_rank (None: read off
    the tensors), tensor_names.  Tensors: q, k [H*dk, hidden]; v, g [H*dv, hidden]; o [hidden, H*dv];
    norm [dv] (shared by the heads); a1 [rank, hidden]; a2 [H*dk, rank]; a2.b [H*dk]."""
    joined = ["q", "k", "v", "g"]

    def __init__(self, params):
        super().__init__(params)
        self.tau = float(params["tau"])
        if not self.tau > 0:
            raise ValueError("tau must be positive")

    def _widths(self):
        return {"q": self.H * self.dk, "k": self.H * self.dk, "v": self.H * self.dv, "g": self.H * self.dv}

    def param_decls(self) -> Dict[str, ParamDecl]:
        n, w = self._name, self._widths()
        d = {n(x): ParamDecl((w[x], self.hidden)) for x in self.joined}
        d[n("o")] = ParamDecl((self.hidden, self.H * self.dv))
        d[n("norm")] = ParamDecl((self.dv,), init="ones")
        d[n("a1")] = ParamDecl((self.rank, self.hidden))
        d[n("a2")] = ParamDecl((self.H * self.dk, self.rank))
        d[n("a2.b")] = ParamDecl((self.H * self.dk,), init="zeros")
        return d

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._name
        self._load_joined(tensors)
        self._check_rank(tensors[n("a1")], tensors[n("a2")], "gated_linear_attention")
        sms = self.ctx.num_sms
        self.a1, self.a2 = Linear(tensors[n("a1")], sms), Linear(tensors[n("a2")], sms)
        self.a_bias = tensors[n("a2.b")].contiguous()
        self.norm_w = tensors[n("norm")].contiguous()
        self.o = Linear(tensors[n("o")], sms)

    def forward(self, x: torch.Tensor, step: StepContext, cache: StateLayerCache) -> torch.Tensor:
        T, dt = x.shape[0], self.ctx.dtype
        p = self._split(self.proj(x, out_dtype=dt))
        z = self.a2(self.a1(x, out_dtype=dt), out_dtype=torch.float32)
        o = torch.empty((T, self.H * self.dv), dtype=torch.float32, device=x.device)
        K.gated_scan(p["q"], p["k"], p["v"], z, self.a_bias, self.dk ** -0.5, self.tau, o, cache.state,
                     step.cu_q, step.state_slots, step.num_entries, self.H, self.dk, self.dv)
        y = torch.empty((T, self.H * self.dv), dtype=dt, device=x.device)
        K.gated_head_norm(o, p["g"], self.norm_w, False, K.GATE_SILU, self.norm_eps, y, self.H, self.dv)
        return self.o(y, out_dtype=dt)


@register_mixer("delta_rule")
class DeltaRule(_StateMixer):
    """params: hidden_size, num_heads, key_dim (values have the same size), norm_eps, decay_rate
    (default exp(-1/2)), unit_eps (default 1e-6), decay_rank (None: read off the tensors),
    tensor_names.  Tensors: r, k, v, g, a [H*d, hidden]; a.b, w0, norm [H*d]; w1 [rank, hidden];
    w2 [H*d, rank]; o [hidden, H*d]."""
    joined = ["r", "k", "v", "g", "a"]

    def __init__(self, params):
        super().__init__(params)
        if self.dv != self.dk:
            raise ValueError("the delta rule's values have the keys' size")
        self.decay_rate = float(params.get("decay_rate", math.exp(-0.5)))
        self.unit_eps = float(params.get("unit_eps", 1e-6))

    def _widths(self):
        return {x: self.H * self.dk for x in self.joined}

    def param_decls(self) -> Dict[str, ParamDecl]:
        n, hd = self._name, self.H * self.dk
        d = {n(x): ParamDecl((hd, self.hidden)) for x in self.joined}
        d[n("a.b")] = ParamDecl((hd,), init="zeros")
        d[n("w0")] = ParamDecl((hd,), init="zeros")
        d[n("norm")] = ParamDecl((hd,), init="ones")
        d[n("w1")] = ParamDecl((self.rank, self.hidden))
        d[n("w2")] = ParamDecl((hd, self.rank))
        d[n("o")] = ParamDecl((self.hidden, hd))
        return d

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._name
        self._load_joined(tensors)
        self._check_rank(tensors[n("w1")], tensors[n("w2")], "delta_rule")
        sms = self.ctx.num_sms
        self.w1, self.w2 = Linear(tensors[n("w1")], sms), Linear(tensors[n("w2")], sms)
        self.w_bias = tensors[n("w0")].contiguous()
        self.a_bias = tensors[n("a.b")].to(self.w_bias.dtype).contiguous()
        self.norm_w = tensors[n("norm")].contiguous()
        self.o = Linear(tensors[n("o")], sms)

    def forward(self, x: torch.Tensor, step: StepContext, cache: StateLayerCache) -> torch.Tensor:
        T, dt = x.shape[0], self.ctx.dtype
        p = self._split(self.proj(x, out_dtype=dt))
        low = self.w1(x, out_dtype=dt)
        K.activation(low, low, K.ACT_TANH)
        zw = self.w2(low, out_dtype=torch.float32)
        o = torch.empty((T, self.H * self.dk), dtype=torch.float32, device=x.device)
        K.delta_scan(p["r"], p["k"], p["v"], p["a"], self.a_bias, zw, self.w_bias, self.decay_rate, self.unit_eps,
                     o, cache.state, step.cu_q, step.state_slots, step.num_entries, self.H, self.dk, self.dk)
        y = torch.empty((T, self.H * self.dk), dtype=dt, device=x.device)
        K.gated_head_norm(o, p["g"], self.norm_w, True, K.GATE_SIGMOID, self.norm_eps, y, self.H, self.dk)
        return self.o(y, out_dtype=dt)


@register_mixer("lightning_attention")
class LightningAttention(Mixer):
    """Linear attention with one fixed decay per head:

        q = silu(W_q h), k = silu(W_k h), v = silu(W_v h);  S_t = decay_h S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t
        out = W_o( w * rms(o over all heads) * sigmoid(W_g h) )

    params: hidden_size, num_heads, key_dim, value_dim, decay (one number per head), norm_eps, q_scale
    (default 1), tensor_names.  Tensors: q, k [H*dk, hidden]; v, g [H*dv, hidden]; norm [H*dv]; o [hidden,
    H*dv].  The four projections are one product whose result stays fp32: the activations are formed from
    it in fp32 and the recurrence reads them unrounded, so the decays, the state and everything that
    enters it are 32-bit in both engine precisions.  The walk is the gated recurrence's with the same row
    of decays for every token."""
    graph_safe = True
    joined = ["q", "k", "v", "g"]

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.dk = int(p["num_heads"]), int(p["key_dim"])
        self.dv = int(p.get("value_dim") or self.dk)
        self.decay = [float(x) for x in p["decay"]]
        self.norm_eps = float(p["norm_eps"])
        self.q_scale = float(p.get("q_scale", 1.0))
        self.tensor_names = dict(p.get("tensor_names") or {})
        if len(self.decay) != self.H:
            raise ValueError(f"{len(self.decay)} decays for {self.H} heads")
        if not (1 <= self.dk <= 512 and self.dv >= 1):
            raise ValueError(f"key size {self.dk}: the recurrence kernels take key sizes up to 512")

    def _name(self, local: str) -> str:
        return self.tensor_names.get(local, local)

    def param_decls(self) -> Dict[str, ParamDecl]:
        n, qk, vg = self._name, self.H * self.dk, self.H * self.dv
        return {n("q"): ParamDecl((qk, self.hidden)), n("k"): ParamDecl((qk, self.hidden)),
                n("v"): ParamDecl((vg, self.hidden)), n("g"): ParamDecl((vg, self.hidden)),
                n("norm"): ParamDecl((vg,), init="ones"), n("o"): ParamDecl((self.hidden, vg))}

    def cache_need(self):
        return FixedState((self.H, self.dv, K.recurrent_state_rows(self.dk)), "float32")

    def prepare(self, ctx) -> None:
        super().prepare(ctx)
        per_channel = [d for d in self.decay for _ in range(self.dk)]
        self.decay_row = torch.tensor(per_channel, dtype=torch.float64).to(torch.float32).to(ctx.device)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._name
        parts = [tensors[n(x)] for x in self.joined]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.proj = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.norm_w = tensors[n("norm")].contiguous()
        self.o = Linear(tensors[n("o")], self.ctx.num_sms)

    def forward(self, x: torch.Tensor, step: StepContext, cache: StateLayerCache) -> torch.Tensor:
        T, qk, vg = x.shape[0], self.H * self.dk, self.H * self.dv
        p = self.proj(x, out_dtype=torch.float32)
        K.activation_cols(p[:, : 2 * qk + vg], K.ACT_SILU)
        o = torch.empty((T, vg), dtype=torch.float32, device=x.device)
        K.decay_scan(p[:, :qk], p[:, qk: 2 * qk], p[:, 2 * qk: 2 * qk + vg], self.decay_row, self.q_scale, o,
                     cache.state, step.cu_q, step.state_slots, step.num_entries, self.H, self.dk, self.dv)
        y = torch.empty((T, vg), dtype=self.ctx.dtype, device=x.device)
        K.row_norm_gate(o, p[:, 2 * qk + vg:], self.norm_w, self.norm_eps, y)
        return self.o(y, out_dtype=torch.float32)
