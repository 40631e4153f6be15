"""The stem and the tail of a decoder as parts of their own: the embedding that starts the
residual stream and the head that turns normed rows into logits.

`token_embedding`: h[t, :] = E[ids[t], :], no scaling, no position table
(crates/infer-worker/src/components/embed.rs:78-81).  `linear_head`: logits = n W^T in fp32;
when the file has no weight for it, it takes the matrix the embedding offers to share, as
the reference ties the head to the embedding table when `lm_head.weight` is absent
(crates/infer-worker/src/models/decoder.rs:245-262).  An embedding multiplier, learned
positions or a soft cap on the logits would be other kinds registered beside these.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Embedding, Head, ParamDecl, StepContext, register_embedding, register_head
from .linear import Linear


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab_size, hidden_size."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.table: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((self.vocab, self.hidden))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors["weight"].contiguous()

    def shared_table(self) -> Optional[torch.Tensor]:
        return self.table

    def forward(self, step: StepContext, h: torch.Tensor) -> None:
        K.embed_gather(step.token_ids[: step.num_tokens], self.table, h)


@register_embedding("scaled_embedding")
class ScaledEmbedding(TokenEmbedding):
    """h[t, :] = scale * E[ids[t], :], the product in fp32.  The table itself is not scaled, so a head that
    shares it multiplies by the stored rows.  params: vocab_size, hidden_size, scale, weight_name (default
    "weight")."""

    def __init__(self, params):
        super().__init__(params)
        self.scale = float(params.get("scale", 1.0))
        self.weight_name = str(params.get("weight_name", "weight"))

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {self.weight_name: ParamDecl((self.vocab, self.hidden))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.weight_name].contiguous()

    def forward(self, step: StepContext, h: torch.Tensor) -> None:
        K.embed_scaled(step.token_ids[: step.num_tokens], self.table, self.scale, h)


@register_embedding("sinusoid_embedding")
class SinusoidEmbedding(TokenEmbedding):
    """h[t, :] = E[ids[t], :] + s(p_t), with s(p)[2i] = sin(p * base^(-2i/hidden)) and s(p)[2i+1] the
    cosine of the same angle.  params: vocab_size, hidden_size, base (default 10000), weight_name
    (default "weight").  Frequencies are made in float64 on the host and the angle in float64 on
    the device, so the vector is exact to fp32 rounding at every position."""

    def __init__(self, params):
        super().__init__(params)
        self.base = float(params.get("base", 10000.0))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.freq: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {self.weight_name: ParamDecl((self.vocab, self.hidden))}

    def prepare(self, ctx) -> None:
        super().prepare(ctx)
        pairs = (self.hidden + 1) // 2
        f = [self.base ** (-2.0 * i / self.hidden) for i in range(pairs)]
        self.freq = torch.tensor(f, dtype=torch.float64).to(ctx.device)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.weight_name].contiguous()

    def forward(self, step: StepContext, h: torch.Tensor) -> None:
        K.embed_sinusoid(step.token_ids[: step.num_tokens], step.positions[: step.num_tokens], self.table,
                         self.freq, h)


@register_embedding("normed_embedding")
class NormedEmbedding(TokenEmbedding):
    """h[t, :] = rmsnorm(E[ids[t], :]) * w: the looked-up row divided by its root mean square (eps inside the
    root) and multiplied by a weight, in fp32.  params: vocab_size, hidden_size, eps, weight_name (the
    table's local name, default "weight"), norm_name (the norm weight's, default "norm.weight")."""

    def __init__(self, params):
        super().__init__(params)
        self.eps = float(params["eps"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.norm_name = str(params.get("norm_name", "norm.weight"))
        self.norm_weight: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {self.weight_name: ParamDecl((self.vocab, self.hidden)),
                self.norm_name: ParamDecl((self.hidden,), init="ones")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.weight_name].contiguous()
        self.norm_weight = tensors[self.norm_name].contiguous()

    def forward(self, step: StepContext, h: torch.Tensor) -> None:
        K.embed_rmsnorm(step.token_ids[: step.num_tokens], self.table, self.norm_weight, self.eps, h)


@register_head("linear_head")
class LinearHead(Head):
    """params: vocab_size, hidden_size, tied (the configuration says the head is the embedding
    table: the file need not have a weight for it), weight_name (the tensor's local name, default "weight"),
    softcap (c > 0: logits <- c * tanh(logits / c); None: none)."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.tied = bool(params.get("tied", False))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        self.linear: Optional[Linear] = None
        self.is_tied = False

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {self.weight_name: ParamDecl((self.vocab, self.hidden), optional=self.tied)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.get(self.weight_name)
        self.is_tied = w is None
        if w is None:
            shared = self.shared
            if shared is None or tuple(shared.shape) != (self.vocab, self.hidden):
                raise ValueError("the head has no weight of its own and the embedding offers none of its shape")
            w = shared
        self.linear = Linear(w, self.ctx.num_sms)

    def forward(self, normed: torch.Tensor) -> torch.Tensor:
        logits = self.linear(normed, out_dtype=torch.float32)
        if self.softcap:
            logits = logits.contiguous()
            K.softcap(logits, self.softcap)
        return logits
