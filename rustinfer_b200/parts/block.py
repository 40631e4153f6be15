"""How a layer's parts are arranged.  "pre_norm": the stream h is only ever changed by
adding what a sublayer returned, and that add is fused into the next norm:

    x = mixer_norm(h += pending);  pending = mixer(x)
    x = ffn_norm(h += pending);    pending = ffn(x)

(crates/infer-worker/src/components/decoder_block.rs:13-32 over
crates/infer-core/src/component.rs:8-27).  h is fp32; pending is in the activation dtype.
"""
from __future__ import annotations

import os
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
    # a model whose layers read a weighted average of all earlier results: [results, T, hidden] fp32 (entry 0 the
    # stem's output), how many entries are written, and the buffer the averages go to
    history: Optional[torch.Tensor] = None
    depth: int = 0
    average: Optional[torch.Tensor] = None


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


_FUSE_INPUT_CONV = os.environ.get("RUSTINFER_B200_FUSE_INPUT_CONV", "1") != "0"


@dataclass
class DepthPending:
    """The end of a layer of the `sandwich_depth_average` arrangement that has not run yet: the last sublayer's
    output is normed and added to the stream, the sum is the layer's result (entry `n_prev` of the history), and
    the weighted average of all results so far is what the next reader gets.  The next norm that reads the stream
    (of the next layer, or the model's last) runs this together with itself, in one kernel."""
    h_in: torch.Tensor
    delta: torch.Tensor
    post_w: torch.Tensor
    result: torch.Tensor                # history[n_prev]
    history: torch.Tensor
    n_prev: int
    weights: torch.Tensor               # fp32 [n_prev + 1]
    avg_out: torch.Tensor
    eps: float

    def run(self, next_w: Optional[torch.Tensor], out: Optional[torch.Tensor], conv=None) -> None:
        from ..ops import kernels as K
        K.rms_sandwich(self.h_in, self.delta, self.post_w, self.result, next_w, out, self.eps, history=self.history,
                       n_prev=self.n_prev, dwa=self.weights, avg_out=self.avg_out, conv=conv)


def settle_depth(hidden: Hidden) -> torch.Tensor:
    """Run what a layer of `sandwich_depth_average` left pending; returns the stream (the depth average)."""
    if isinstance(hidden.pending, DepthPending):
        hidden.pending.run(None, None)
        hidden.pending = None
    return hidden.stream


def _sandwich_depth_average(block: Block, hidden: Hidden, step: StepContext, cache) -> None:
    """A norm before and after each sublayer, and a weighted average over depth.  With x the layer's input:

        x <- x + post_mixer_norm(mixer(mixer_norm(x)));  x <- x + post_ffn_norm(ffn(ffn_norm(x)))

    (the second only when the layer has a feed-forward; the post norms hold the residual's factor as their
    `scale`).  x is then the layer's result X_n, kept in the model's history beside X_0 (the stem's output) and the
    earlier results, and the next layer's input (after the last layer, the final norm's) is sum_j w[j] X_j over
    j = 0 .. n with the weights of this layer's `depth_average` part.  All norms are `rmsnorm` parts.  A mixer that
    sets `input_float32` gets its norm's output unrounded."""
    from ..ops import kernels as K
    post_mixer, post_ffn = block.extra_norms.get("post_mixer_norm"), block.extra_norms.get("post_ffn_norm")
    avg = block.extra_norms.get("depth_average")
    if block.mixer_norm is None or post_mixer is None or avg is None:
        raise ValueError("the sandwich_depth_average arrangement wants a norm before and after the mixer and a "
                         "depth_average part")
    if hidden.history is None or hidden.average is None:
        raise ValueError("the sandwich_depth_average arrangement runs in a model whose spec sets depth_average")
    n = hidden.depth                      # this layer's result is entry n of the history
    if avg.count != n + 1:
        raise ValueError(f"the layer's depth_average has {avg.count} weights; {n + 1} results exist after it")
    x_in = hidden.stream
    # a mixer behind a short convolution (`conv_input`), in a step of single tokens: the convolution runs in the norm's
    # launch and the mixer is told that its input has passed it
    conv = getattr(block.mixer, "input_conv", None) if _FUSE_INPUT_CONV else None
    if conv is not None and conv.bias is None and step.max_q_len == 1 and step.num_entries == step.num_tokens:
        x = block.mixer_norm.add_norm(x_in, hidden.pending, conv=(conv.weight, cache[0].state, step.state_slots))
        hidden.pending = None
        y = block.mixer.forward(x, step, cache, conv_done=True)
    else:
        want = torch.float32 if getattr(block.mixer, "input_float32", False) else None
        x = block.mixer_norm.add_norm(x_in, hidden.pending, out_dtype=want)
        hidden.pending = None
        y = block.mixer.forward(x, step, cache)
    result = hidden.history[n]
    if block.ffn is None:
        last_in, last_y, last_post = x_in, y, post_mixer
    else:
        if block.ffn_norm is None or post_ffn is None:
            raise ValueError("the sandwich_depth_average arrangement wants a norm before and after the feed-forward")
        x2 = torch.empty((x_in.shape[0], x_in.shape[1]), dtype=block.ffn_norm.ctx.dtype, device=x_in.device)
        if post_mixer.eps == block.ffn_norm.eps:
            K.rms_sandwich(x_in, y, post_mixer.weight32, result, block.ffn_norm.weight32, x2, post_mixer.eps)
        else:
            post_mixer.add_into(x_in, y, h_out=result)
            K.rms_sandwich(result, None, None, None, block.ffn_norm.weight32, x2, block.ffn_norm.eps)
        last_in, last_y, last_post = result, block.ffn.forward(x2, step), post_ffn
    hidden.pending = DepthPending(last_in, last_y, last_post.weight32, result, hidden.history, n, avg.weights,
                                  hidden.average, last_post.eps)
    hidden.stream = hidden.average
    hidden.depth = n + 1


ARRANGEMENTS: Dict[str, Callable] = {"pre_norm": _pre_norm, "sandwich": _sandwich, "hyper": _hyper,
                                     "post_norm": _post_norm, "sandwich_depth_average": _sandwich_depth_average}


def register_arrangement(name: str, fn: Callable) -> None:
    ARRANGEMENTS[name] = fn
