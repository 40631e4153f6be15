"""How a layer's parts are arranged.  "pre_norm": the stream h is only ever changed by
adding what a sublayer returned, and that add is fused into the next norm:

    x = mixer_norm(h += pending);  pending = mixer(x)
    x = ffn_norm(h += pending);    pending = ffn(x)

(crates/infer-worker/src/components/decoder_block.rs:13-32 over
crates/infer-core/src/component.rs:8-27).  h is fp32; pending is in the activation dtype.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch

from .base import FEED_FORWARDS, MIXERS, NORMS, BuildContext, FeedForward, Mixer, Norm, StepContext
from .spec import LayerSpec


@dataclass
class Hidden:
    stream: torch.Tensor                # [T, hidden] fp32 ([streams, T, hidden] in a model of several streams)
    pending: Optional[torch.Tensor]     # [T, hidden] activation dtype, not yet added
    fresh: bool = False                 # several streams of which only the first is written yet (all are equal)
    act: Optional[torch.Tensor] = None  # the stream rounded to the activation dtype, where a block keeps one


class Block:
    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer: Mixer = MIXERS.build(spec.mixer)
        self.mixer_norm: Optional[Norm] = NORMS.build(spec.mixer_norm) if spec.mixer_norm else None
        self.ffn: Optional[FeedForward] = FEED_FORWARDS.build(spec.ffn) if spec.ffn else None
        self.ffn_norm: Optional[Norm] = NORMS.build(spec.ffn_norm) if spec.ffn_norm else None
        self.extra_norms: Dict[str, Norm] = {role: NORMS.build(ps) for role, ps in spec.extra_norms.items()}
        fn = ARRANGEMENTS.get(spec.arrangement)
        if fn is None:
            raise KeyError(f"no block arrangement '{spec.arrangement}'; known: {sorted(ARRANGEMENTS)}")
        self._run = fn
        missing = [r for r in self.roles() if r not in spec.names]
        if missing:
            raise KeyError(f"layer names no tensor prefix for {missing}")

    def roles(self):
        """role -> part, for every part the layer has."""
        named = {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "ffn": self.ffn, "ffn_norm": self.ffn_norm}
        named.update(self.extra_norms)
        return {role: part for role, part in named.items() if part is not None}

    def prepare(self, ctx: BuildContext) -> None:
        for part in self.roles().values():
            part.prepare(ctx)

    @property
    def graph_safe(self) -> bool:
        return self.mixer.graph_safe and (self.ffn is None or self.ffn.graph_safe)

    def forward(self, hidden: Hidden, step: StepContext, cache) -> None:
        self._run(self, hidden, step, cache)


def _pre_norm(block: Block, hidden: Hidden, step: StepContext, cache) -> None:
    if block.mixer_norm is None or block.ffn is None or block.ffn_norm is None:
        raise ValueError("the pre_norm arrangement wants a mixer, a feed-forward and a norm before each")
    # a part that declares `adds_to_residual` may add its output into the stream itself
    # (inside its last product's epilogue) and return None; otherwise the add rides on the
    # next norm
    x = block.mixer_norm.add_norm(hidden.stream, hidden.pending)
    if getattr(block.mixer, "adds_to_residual", False):
        hidden.pending = block.mixer.forward(x, step, cache, residual=hidden.stream)
    else:
        hidden.pending = block.mixer.forward(x, step, cache)
    x = block.ffn_norm.add_norm(hidden.stream, hidden.pending)
    if getattr(block.ffn, "adds_to_residual", False):
        hidden.pending = block.ffn.forward(x, step, residual=hidden.stream)
    else:
        hidden.pending = block.ffn.forward(x, step)


def _sandwich(block: Block, hidden: Hidden, step: StepContext, cache) -> None:
    """A norm before and a norm after each sublayer:

        h += post_mixer_norm(mixer(mixer_norm(h)));  h += post_ffn_norm(ffn(ffn_norm(h)))

    (the second line only when the layer has a feed-forward).  The norms after the sublayers go
    by the roles `post_mixer_norm` and `post_ffn_norm` in `extra_norms`.  A sublayer's output stays
    pending as a `NormedDelta`; the next norm that reads the stream, of this layer, the next or
    the model's last, norms it, adds it and norms the sum in one kernel."""
    from .norm import NormedDelta
    post_mixer, post_ffn = block.extra_norms.get("post_mixer_norm"), block.extra_norms.get("post_ffn_norm")
    if block.mixer_norm is None or post_mixer is None:
        raise ValueError("the sandwich arrangement wants a norm before and a norm after the mixer")
    x = block.mixer_norm.add_norm(hidden.stream, hidden.pending)
    hidden.pending = NormedDelta(block.mixer.forward(x, step, cache), post_mixer)
    if block.ffn is None:
        return
    if block.ffn_norm is None or post_ffn is None:
        raise ValueError("the sandwich arrangement wants a norm before and a norm after the feed-forward")
    x = block.ffn_norm.add_norm(hidden.stream, hidden.pending)
    hidden.pending = NormedDelta(block.ffn.forward(x, step), post_ffn)


def _hyper(block: Block, hidden: Hidden, step: StepContext, cache) -> None:
    """Several residual streams (see parts/hyper.py): each sublayer reads a weighted sum of the streams
    through its `hyper_rmsnorm`, and its output stays pending until the next read of the streams mixes
    them and adds it to each with a weight of its own.  The feed-forward is optional."""
    from .hyper import HyperPending, HyperRMSNorm
    if not isinstance(block.mixer_norm, HyperRMSNorm) or (block.ffn is not None and not isinstance(block.ffn_norm, HyperRMSNorm)):
        raise ValueError("the hyper arrangement wants a hyper_rmsnorm before each sublayer")
    x = block.mixer_norm.collect(hidden)
    hidden.pending = HyperPending(block.mixer.forward(x, step, cache), block.mixer_norm)
    if block.ffn is not None:
        x = block.ffn_norm.collect(hidden)
        hidden.pending = HyperPending(block.ffn.forward(x, step), block.ffn_norm)


def _post_norm(block: Block, hidden: Hidden, step: StepContext, cache) -> None:
    """The norm after the sum, and the stream replaced by it:

        h <- mixer_norm(alpha h + mixer(h));  h <- ffn_norm(alpha h + ffn(h))

    (the second line only when the layer has a feed-forward).  The sublayers read the stream itself;
    both norms are `post_rmsnorm` parts, which hold alpha.  The stream is fp32; each norm also hands
    out its result rounded to the activation dtype, which is what the next sublayer's products read
    (`hidden.act`; the first block of a model rounds the stem's output itself)."""
    from ..ops import kernels as K
    from .norm import PostRMSNorm
    if not isinstance(block.mixer_norm, PostRMSNorm) or (block.ffn is not None and not isinstance(block.ffn_norm, PostRMSNorm)):
        raise ValueError("the post_norm arrangement wants a post_rmsnorm after each sublayer")
    if hidden.pending is not None:
        raise ValueError("the post_norm arrangement follows blocks that leave nothing pending")
    x = hidden.act
    if x is None:
        x = hidden.stream
        if block.mixer_norm.ctx.dtype != torch.float32:
            x = torch.empty(hidden.stream.shape, dtype=block.mixer_norm.ctx.dtype, device=hidden.stream.device)
            K.round_rows(hidden.stream, x)
    x = block.mixer_norm.renorm(hidden.stream, block.mixer.forward(x, step, cache))
    if block.ffn is not None:
        x = block.ffn_norm.renorm(hidden.stream, block.ffn.forward(x, step))
    hidden.act = x


ARRANGEMENTS: Dict[str, Callable] = {"pre_norm": _pre_norm, "sandwich": _sandwich, "hyper": _hyper,
                                     "post_norm": _post_norm}


def register_arrangement(name: str, fn: Callable) -> None:
    ARRANGEMENTS[name] = fn
