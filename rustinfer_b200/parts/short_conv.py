"""A short causal convolution over time in front of a mixer: the mixer reads x + conv(x) instead of x.

    conv(x)_t = sum_j w[:, j] * x_(t - taps + 1 + j)      per channel, zeros before the sequence's start

`conv_input` wraps any registered mixer.  The last taps - 1 inputs of every live request are state (a slot of a
fixed-state cache group of the part's own), so a prompt cut into portions and a token decoded alone see the same
inputs as the whole prompt would.  The convolution runs in fp32 on the fp32 output of the norm before it and is
rounded once, for the mixer's products.  `ConvState` is the same convolution for mixers that have one inside
(the recurrent unit's input branch).  The reference engine has no such part (its blocks are
crates/infer-worker/src/components/decoder_block.rs:13-32).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..ops import kernels as K
from .base import MIXERS, BuildContext, FixedState, Mixer, ParamDecl, StateLayerCache, StepContext, StepIndex, register_mixer


class ConvState:
    """The convolution's weights ([channels, taps], kept fp32) and how it is run on a step."""

    def __init__(self, channels: int, taps: int):
        self.channels, self.taps = int(channels), int(taps)
        if not 1 <= self.taps <= 8:
            raise ValueError(f"a short convolution has 1 to 8 taps, got {self.taps}")
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def need(self) -> FixedState:
        return FixedState((self.taps - 1, self.channels))

    def load(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        self.weight = weight.to(torch.float32).contiguous()
        self.bias = bias.to(torch.float32).contiguous() if bias is not None else None

    def run(self, x: torch.Tensor, step: StepContext, cache: StateLayerCache, out: torch.Tensor, residual: bool,
            in_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        K.short_conv(x, self.weight, self.bias, cache.state, step.cu_q, step.state_slots, out, step.num_entries,
                     step.max_q_len, residual, in_bias)
        return out


@register_mixer("conv_input")
class ConvInput(Mixer):
    """params: inner (PartSpec of the mixer behind the convolution), size, taps, weight_name (the convolution's
    tensor, default "conv"), inner_prefix (prefix of the inner mixer's tensors inside this part, default "")."""
    input_float32 = True                # the block hands this part the fp32 output of the norm before it

    def __init__(self, params):
        super().__init__(params)
        self.inner: Mixer = MIXERS.build(params["inner"])
        self.conv = ConvState(int(params["size"]), int(params["taps"]))
        self.weight_name = str(params.get("weight_name", "conv"))
        self.inner_prefix = str(params.get("inner_prefix", ""))
        need = self.inner.cache_need()
        self._inner_needs = () if need is None else tuple(need) if isinstance(need, (tuple, list)) else (need,)
        self._inner_single = need is not None and not isinstance(need, (tuple, list))

    @property
    def graph_safe(self) -> bool:
        return self.inner.graph_safe

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {self.weight_name: ParamDecl((self.conv.channels, self.conv.taps))}
        d.update({self.inner_prefix + n: decl for n, decl in self.inner.param_decls().items()})
        return d

    def cache_need(self):
        return (self.conv.need(),) + self._inner_needs

    def step_indices(self) -> Sequence[StepIndex]:
        return self.inner.step_indices()

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        self.inner.prepare(ctx)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.conv.load(tensors[self.weight_name])
        pre = self.inner_prefix
        self.inner.load({n: tensors[pre + n] for n in self.inner.param_decls() if pre + n in tensors})

    @property
    def input_conv(self) -> ConvState:
        """The convolution, for a block that can run it in the launch of the norm before it (it then calls
        `forward(..., conv_done=True)` with x + conv(x) in the activation dtype)."""
        return self.conv

    def forward(self, x: torch.Tensor, step: StepContext, cache, conv_done: bool = False) -> torch.Tensor:
        caches = list(cache)
        if conv_done:
            out = x
        else:
            out = torch.empty(x.shape, dtype=self.ctx.dtype, device=x.device)
            self.conv.run(x, step, caches[0], out, residual=True)
        rest = caches[1:]
        inner_cache = None if not rest else rest[0] if self._inner_single else tuple(rest)
        return self.inner.forward(out, step, inner_cache)
