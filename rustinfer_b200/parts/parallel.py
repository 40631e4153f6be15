"""Two mixers side by side on one input: out = left_scale * left(x) + right_scale * right(x).

Two optional understandings with the sides save launches.  A side that sets `joins_input` keeps the projections of
its input as one `Linear` called `proj` (fp32 out) and takes `proj=` (that product's result, a column view) in
`forward`: where both sides do, the part multiplies the input by both matrices at once.  A side that sets
`scales_output` takes `out_scale=` (applied before its output product, where its last rounding is) and `add_to=` (an
fp32 tensor its output product is added into): where both do, no kernel of its own sums the sides.

Each side is a mixer of any registered kind with its own tensors (under the prefixes `left.` and
`right.` unless the spec names others) and its own cache: the part declares both sides' needs
and hands each side the cache that belongs to it.  The reference engine has one mixer per block
(crates/infer-worker/src/components/decoder_block.rs:13-32); this is the part that lets a block
keep attention over recent keys beside a recurrent state.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..ops import kernels as K
from .base import MIXERS, BuildContext, Mixer, ParamDecl, StepContext, StepIndex, register_mixer
from .spec import PartSpec


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    """params: left, right (PartSpec of a mixer each), left_scale, right_scale, left_prefix,
    right_prefix (tensor-name prefixes inside this part, default "left." and "right.")."""

    def __init__(self, params):
        super().__init__(params)
        self.sides: List[Mixer] = [MIXERS.build(params["left"]), MIXERS.build(params["right"])]
        self.scales = [float(params.get("left_scale", 1.0)), float(params.get("right_scale", 1.0))]
        self.prefixes = [str(params.get("left_prefix", "left.")), str(params.get("right_prefix", "right."))]
        # a side's needs as a tuple (a side may itself keep several things: a state beside a convolution's inputs)
        self._needs = [m.cache_need() for m in self.sides]
        self._counts = [0 if n is None else len(n) if isinstance(n, (tuple, list)) else 1 for n in self._needs]

    @property
    def graph_safe(self) -> bool:
        return all(m.graph_safe for m in self.sides)

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {pre + name: d for pre, m in zip(self.prefixes, self.sides) for name, d in m.param_decls().items()}

    def cache_need(self):
        needs = tuple(x for n in self._needs if n is not None for x in (n if isinstance(n, (tuple, list)) else (n,)))
        return needs or None

    def step_indices(self) -> Sequence[StepIndex]:
        return [need for m in self.sides for need in m.step_indices()]

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        for m in self.sides:
            m.prepare(ctx)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        from .linear import Linear
        for pre, m in zip(self.prefixes, self.sides):
            m.load({name: tensors[pre + name] for name in m.param_decls() if pre + name in tensors})
        self.joint = None
        if all(getattr(m, "joins_input", False) for m in self.sides):
            ws = [m.proj.weight for m in self.sides]
            if ws[0].dtype == ws[1].dtype and ws[0].shape[1] == ws[1].shape[1]:
                self.joint = Linear(torch.cat(ws, dim=0), self.ctx.num_sms)
                self.split = ws[0].shape[0]
                for m in self.sides:
                    m.proj = None                        # the joint matrix holds its rows now
        self.accumulate = all(getattr(m, "scales_output", False) for m in self.sides)

    def forward(self, x: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        caches = list(cache) if isinstance(cache, (tuple, list)) else [cache]
        outs = []
        projs = [None, None]
        if self.joint is not None:
            both = self.joint(x, out_dtype=torch.float32)
            projs = [both[:, : self.split], both[:, self.split:]]
        for i, (m, need, count) in enumerate(zip(self.sides, self._needs, self._counts)):
            mine = [caches.pop(0) for _ in range(count)]
            kw = {"proj": projs[i]} if projs[i] is not None else {}
            if self.accumulate:
                kw["out_scale"] = self.scales[i]
                if i == 1:
                    kw["add_to"] = outs[0]
            outs.append(m.forward(x, step, None if need is None else tuple(mine) if isinstance(need, (tuple, list))
                                  else mine[0], **kw))
        if self.accumulate:
            return outs[0]
        if outs[0].dtype != outs[1].dtype:                   # one side leaves in 32-bit, the other rounded
            outs = [o.to(torch.float32) for o in outs]
        out = torch.empty_like(outs[0])
        K.scaled_sum(outs[0], outs[1], self.scales[0], self.scales[1], out)
        return out
