"""The recurrent block with a real-gated linear recurrent unit (De et al., "Griffin: Mixing Gated Linear
Recurrences with Local Attention for Efficient Language Models"): two branches of `width` channels,

    y = gelu_tanh(W_y h + b_y)
    u = conv(W_x h + b_x) + b_conv                 a short causal convolution per channel
    r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b)      per block b of width / blocks channels
    a = exp(-decay_scale * r * softplus(lam));     S_t = a S_(t-1) + sqrt(1 - a^2) * i * u
    out = W_o (S * y)

The state S (fp32, zero for a new request) and the convolution's last taps - 1 inputs sit in slots of two
fixed-state cache groups.  The projections are matrix products of the engine's precision with fp32 results; the
convolution, the gates' products, the decay, the recurrence and the gelu are fp32 in both engines, and S * y is
rounded once for the output product.  Beside another mixer (`parallel_mixers`) the part takes the joint product's
columns as `proj`, an `out_scale` on S * y and an `add_to` its output product is added into.  The reference engine has no recurrent mixer
(crates/infer-worker/src/components/attention.rs is its only one).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .attention_variants import project_out
from .base import BuildContext, FixedState, Mixer, ParamDecl, StepContext, register_mixer
from .linear import Linear
from .short_conv import ConvState


@register_mixer("gated_recurrent_unit")
class GatedRecurrentUnit(Mixer):
    """params: hidden_size, width, blocks, conv_taps, decay_scale (default 8), tensor_names (local name -> name in the
    file).  Tensors: y, x [width, hidden] with biases y.b, x.b; conv [width, taps], conv.b; ra, ri
    [blocks, width/blocks, width/blocks] ([out, in]) with biases ra.b, ri.b [blocks, width/blocks]; lam [width];
    o [hidden, width]."""
    graph_safe = True
    joins_input = True
    scales_output = True

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden, self.width, self.blocks = int(p["hidden_size"]), int(p["width"]), int(p["blocks"])
        self.decay_scale = float(p.get("decay_scale", 8.0))
        self.tensor_names = dict(p.get("tensor_names") or {})
        if self.blocks <= 0 or self.width % self.blocks:
            raise ValueError(f"width {self.width} is not a multiple of {self.blocks} blocks")
        self.conv = ConvState(self.width, int(p["conv_taps"]))

    def _name(self, local: str) -> str:
        return self.tensor_names.get(local, local)

    def param_decls(self) -> Dict[str, ParamDecl]:
        n, W, bs = self._name, self.width, self.width // self.blocks
        return {n("y"): ParamDecl((W, self.hidden)), n("y.b"): ParamDecl((W,), init="zeros"),
                n("x"): ParamDecl((W, self.hidden)), n("x.b"): ParamDecl((W,), init="zeros"),
                n("conv"): ParamDecl((W, self.conv.taps)), n("conv.b"): ParamDecl((W,), init="zeros"),
                n("ra"): ParamDecl((self.blocks, bs, bs)), n("ra.b"): ParamDecl((self.blocks, bs), init="zeros"),
                n("ri"): ParamDecl((self.blocks, bs, bs)), n("ri.b"): ParamDecl((self.blocks, bs), init="zeros"),
                n("lam"): ParamDecl((W,)), n("o"): ParamDecl((self.hidden, W))}

    def cache_need(self):
        return (self.conv.need(), FixedState((self.width,)))

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._name
        f32 = lambda name: tensors[n(name)].to(torch.float32).reshape(-1).contiguous()
        parts = [tensors[n("y")], tensors[n("x")]]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.proj = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.y_bias, self.x_bias = f32("y.b"), f32("x.b")
        self.conv.load(tensors[n("conv")], tensors[n("conv.b")])
        self.wa, self.wi = tensors[n("ra")].contiguous(), tensors[n("ri")].to(tensors[n("ra")].dtype).contiguous()
        self.ba, self.bi, self.lam = f32("ra.b"), f32("ri.b"), f32("lam")
        self.o = Linear(tensors[n("o")], self.ctx.num_sms)

    def forward(self, h: torch.Tensor, step: StepContext, cache, proj: Optional[torch.Tensor] = None,
                out_scale: float = 1.0, add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
        conv_cache, state_cache = cache
        T, W, dev = h.shape[0], self.width, h.device
        if proj is None:
            proj = self.proj(h, out_dtype=torch.float32)                     # [T, 2W]: y, then x
        u = torch.empty((T, W), dtype=torch.float32, device=dev)
        self.conv.run(proj[:, W:], step, conv_cache, u, residual=False, in_bias=self.x_bias)
        sy = torch.empty((T, W), dtype=self.ctx.dtype, device=dev)
        if step.max_q_len == 1 and step.num_entries == T:
            # every entry brings one token: gates, the recurrence's step and the gelu in one launch
            K.rglru_step(u, self.wa, self.wi, self.ba, self.bi, self.lam, self.decay_scale, proj[:, :W], self.y_bias,
                         state_cache.state, step.state_slots, sy, out_scale)
            return project_out(self.o, sy, add_to)
        a = torch.empty((T, W), dtype=torch.float32, device=dev)
        x = torch.empty((T, W), dtype=torch.float32, device=dev)
        K.rglru_gates(u, self.wa, self.wi, self.ba, self.bi, self.lam, self.decay_scale, a, x)
        K.rglru_scan(a, x, proj[:, :W], self.y_bias, state_cache.state, step.cu_q, step.state_slots, sy,
                     step.num_entries, step.max_q_len, out_scale)
        return project_out(self.o, sy, add_to)
