"""RMSNorm fused with the residual add: y = x * w / sqrt(mean(x^2) + eps), the weight
multiplying directly (crates/infer-worker/src/components/norm.rs:10-27,
crates/infer-backend-cuda/src/kernels/rmsnorm/rmsnorm.cu:52-113).  Sum of squares, the
scale and the residual sum are fp32."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Norm, ParamDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, weight_name (the tensor's local name, default "weight"), offset (added to the stored
    weight: 1 for a weight stored around zero; default 0), scale (a factor on the norm's output, the residual's
    factor of a norm that follows a sublayer, say; default 1).  With an offset or a scale the part keeps
    (offset + w) * scale in fp32.

    `add_norm` takes as `delta` a tensor (added as it is), None, a `NormedDelta` (normed by the RMS norm it names,
    then added) or a `DepthPending` (see parts/block.py); the last two run as one kernel with this norm."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.offset = float(params.get("offset", 0.0))
        self.scale = float(params.get("scale", 1.0))
        self.weight: Optional[torch.Tensor] = None
        self._weight32: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {self.weight_name: ParamDecl((self.size,), init="zeros" if self.offset == 1.0 else "ones")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name].contiguous()
        if self.offset != 0.0 or self.scale != 1.0:
            w = ((w.to(torch.float32) + self.offset) * self.scale).contiguous()
        self.weight = w
        self._weight32 = None

    @property
    def weight32(self) -> torch.Tensor:
        if self._weight32 is None:
            self._weight32 = self.weight.to(torch.float32).contiguous()
        return self._weight32

    def add_norm(self, h, delta, rows=None, out_dtype=None, conv=None):
        """`conv` (weight, state, state slots), in a step of single tokens: the short convolution that follows this norm
        runs in the norm's launch (see `kernels.rms_sandwich`)."""
        from .block import DepthPending
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.ctx.dtype, device=h.device)
        if isinstance(delta, DepthPending):
            if rows is None and delta.eps == self.eps:
                delta.run(self.weight32, out, conv)
            else:
                delta.run(None, None)
                K.rms_sandwich(delta.avg_out, None, None, None, self.weight32, out, self.eps, rows=rows, conv=conv)
            return out
        if isinstance(delta, NormedDelta):
            post = delta.norm
            if rows is None and post.eps == self.eps:
                K.rms_sandwich(h, delta.delta, post.weight32, h, self.weight32, out, self.eps, conv=conv)
            else:
                post.add_into(h, delta.delta)
                K.rms_sandwich(h, None, None, None, self.weight32, out, self.eps, rows=rows, conv=conv)
            return out
        if conv is not None or (self.weight.dtype == torch.float32
                                and (delta is None or delta.dtype != out.dtype or self.ctx.dtype != out.dtype)):
            if delta is not None:
                K.residual_add(h, delta)
            K.rms_sandwich(h, None, None, None, self.weight32, out, self.eps, rows=rows, conv=conv)
            return out
        K.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
        return out

    def add_into(self, h: torch.Tensor, delta: torch.Tensor, h_out: Optional[torch.Tensor] = None) -> None:
        """h_out (default h itself) <- h + rms(delta) * w."""
        K.rms_sandwich(h, delta, self.weight32, h if h_out is None else h_out, None, None, self.eps)


@register_norm("post_rmsnorm")
class PostRMSNorm(Norm):
    """The norm of a block that norms after the sum: h <- w * rms(alpha * h + y), the stream itself
    replaced.  params: size, eps, alpha (default 1), weight_name (default "weight").  `renorm` does
    that in one kernel and returns the new stream in the activation dtype for the next sublayer's
    products (the stream itself in a 32-bit engine); `add_norm` is the plain RMS norm, so the part
    can stand wherever an `rmsnorm` can."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.alpha = float(params.get("alpha", 1.0))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {self.weight_name: ParamDecl((self.size,), init="ones")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def renorm(self, h: torch.Tensor, delta: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.ctx.dtype == torch.float32:
            K.scale_add_norm(h, delta, bias, self.alpha, self.weight, self.eps, None)
            return h
        act = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        K.scale_add_norm(h, delta, bias, self.alpha, self.weight, self.eps, act)
        return act

    def add_norm(self, h, delta, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=h.device)
        K.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
        return out


@dataclass
class NormedDelta:
    """A sublayer's output that is to pass through `norm` before it is added to the stream (a
    block with a norm after each sublayer leaves this as its pending delta)."""
    delta: torch.Tensor
    norm: Norm                          # a `layernorm` or an `rmsnorm`; the norm that adds it is of the same kind


@register_norm("layernorm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w + b over the last axis, var the mean of the squared
    deviations; mean, variance, scale and the residual sum are fp32.  params: size, eps, bias
    (True: the file has a bias; False: none; None: used when the file has one).  The weight's
    tensor is named by the part's prefix alone, the bias by prefix + `.b`, unless `weight_name` /
    `bias_name` say otherwise.

    `add_norm` takes as `delta` a tensor (added as it is), None, or a `NormedDelta` (normed by the
    norm it names, then added): one kernel does that norm, the add and this norm."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.has_bias = params.get("bias", True)
        self.weight_name = str(params.get("weight_name", ""))
        self.bias_name = str(params.get("bias_name", ".b"))
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {self.weight_name: ParamDecl((self.size,), init="ones")}
        if self.has_bias is None or self.has_bias:
            d[self.bias_name] = ParamDecl((self.size,), init="zeros", optional=self.has_bias is None)
        return d

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        b = tensors.get(self.bias_name)
        self.bias = b.to(self.weight.dtype).contiguous() if b is not None else None

    def add_norm(self, h, delta, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=h.device)
        if isinstance(delta, NormedDelta):
            post = delta.norm
            if post.eps != self.eps:            # two norms of one kernel share eps; else two launches
                post.add_into(h, delta.delta)
                K.sandwich_norm(h, None, None, None, self.weight, self.bias, out, self.eps, rows)
            else:
                K.sandwich_norm(h, delta.delta, post.weight, post.bias, self.weight, self.bias, out, self.eps, rows)
            return out
        if delta is not None:
            K.residual_add(h, delta)
        K.sandwich_norm(h, None, None, None, self.weight, self.bias, out, self.eps, rows)
        return out

    def add_into(self, h: torch.Tensor, delta: torch.Tensor) -> None:
        """h += LN(delta)."""
        K.sandwich_norm(h, delta, self.weight, self.bias, None, None, None, self.eps)


@register_norm("depth_average")
class DepthAverage(Norm):
    """The weights of a layer's average over depth (see the `sandwich_depth_average` arrangement): `count` numbers,
    one for the stem's output and one for every layer's result up to this layer's own.  params: count,
    weight_name (default "weight").  It norms nothing; it stands among a block's norms because, like them, it is a
    small tensor of the block that the kernel around the sublayers reads."""

    def __init__(self, params):
        super().__init__(params)
        self.count = int(params["count"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weights: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {self.weight_name: ParamDecl((self.count,), init="depth_last")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weights = tensors[self.weight_name].to(torch.float32).contiguous()

    def add_norm(self, h, delta, rows=None):
        raise TypeError("depth_average holds weights only: it runs in the `sandwich_depth_average` block arrangement")
