"""A feed-forward of routed experts: every token runs through `top` of `experts` small gated feed-forwards,
chosen by a router, and through a shared one where the model has it.

    z = W_r x (32-bit);  s = sigmoid(z);  choice score c = s + correction
    with groups: the experts form `groups_count` equal groups of neighbours; a group's score is the sum of
        its two largest c; only experts of the `groups_keep` best groups can be chosen
    the `top` largest c are chosen; their weights are the s (divided by their sum when `renormalize`)
    y = sum_chosen weight_e * down_e( silu(gate_e x) * up_e x ) + shared(x)

With `score` "softmax_chosen" the `top` largest logits z are chosen as they are and the weights are their softmax
among themselves.  With `activation` "clamped" an expert is down_e( g' sigmoid(alpha g') (u' + 1) ) with
g' = min(gate_e x, limit) and u' = clamp(up_e x, -limit, limit).

The router's product, scores and choice are fp32.  The (token, choice) pairs are sorted by expert on the
device and the experts' products run over the sorted rows; no count visits the host, so the part can be
captured in a step's CUDA graph.  The reference engine has dense feed-forwards only
(crates/infer-worker/src/components/ffn_dense.rs:26-33); its loader names expert tensors but runs none.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import FEED_FORWARDS, FeedForward, ParamDecl, StepContext, register_feed_forward
from .spec import PartSpec


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """params: hidden_size, expert_ff, experts, top, groups_count / groups_keep (None: no groups), shared_ff
    (None: no shared expert), score ("sigmoid", or "softmax_chosen"), activation ("silu", or "clamped" with
    `limit` and `alpha`, default 1.702), correction (the router has a tensor added to the scores for
    the choice), renormalize, output ("float32", the default, or the activation dtype); tensor names:
    expert_prefix (default "e{}."; `{}` is the expert's number), gate_name / up_name / down_name (default
    "gate" / "up" / "down"), router_name ("router"), correction_name ("correction"), shared_prefix ("shared.")."""

    TC_ROWS_PER_EXPERT = 24              # rows an expert on average from which the tcgen05 products pay

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden, self.ff = int(p["hidden_size"]), int(p["expert_ff"])
        self.E, self.top = int(p["experts"]), int(p["top"])
        self.groups = int(p["groups_count"]) if p.get("groups_count") else 0
        self.keep = int(p["groups_keep"]) if p.get("groups_keep") else 0
        self.shared_ff = int(p["shared_ff"]) if p.get("shared_ff") else None
        self.score = str(p.get("score", "sigmoid"))
        if self.score not in ("sigmoid", "softmax_chosen"):
            raise ValueError(f"router score {self.score!r}: known are 'sigmoid' and 'softmax_chosen'")
        activation = str(p.get("activation", "silu"))
        if activation not in ("silu", "clamped"):
            raise ValueError(f"expert activation {activation!r}: known are 'silu' and 'clamped'")
        # (limit, alpha) of the clamped pair, None for silu(gate) * up
        self.act = (float(p["limit"]), float(p.get("alpha", 1.702))) if activation == "clamped" else None
        if self.act is not None and not self.act[0] > 0:
            raise ValueError("the clamp's limit is positive")
        self.has_correction = bool(p.get("correction", False))
        self.renorm = bool(p.get("renormalize", False))
        self.out_fp32 = str(p.get("output", "float32")) == "float32"
        self.expert_prefix = str(p.get("expert_prefix", "e{}."))
        self.names = {k: str(p.get(k + "_name", k)) for k in ("gate", "up", "down", "router", "correction")}
        self.shared_prefix = str(p.get("shared_prefix", "shared."))
        if not 1 <= self.top <= min(self.E, 32):
            raise ValueError(f"a token uses 1 to min(experts, 32) experts, got {self.top} of {self.E}")
        if self.groups and (self.E % self.groups or not 0 < self.keep <= self.groups
                            or self.keep * (self.E // self.groups) < self.top):
            raise ValueError("groups_count divides experts, and the groups kept hold at least `top` experts")
        self.shared: Optional[FeedForward] = None
        if self.shared_ff:
            self.shared = FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": self.hidden,
                                                                  "intermediate_size": self.shared_ff,
                                                                  "output": "float32"}))
        self._shared_names = {"gate_proj.weight": self.names["gate"], "up_proj.weight": self.names["up"],
                              "down_proj.weight": self.names["down"]}

    @property
    def graph_safe(self) -> bool:
        return True

    def param_decls(self) -> Dict[str, ParamDecl]:
        d: Dict[str, ParamDecl] = {}
        for e in range(self.E):
            pre = self.expert_prefix.format(e)
            d[pre + self.names["gate"]] = ParamDecl((self.ff, self.hidden))
            d[pre + self.names["up"]] = ParamDecl((self.ff, self.hidden))
            d[pre + self.names["down"]] = ParamDecl((self.hidden, self.ff))
        d[self.names["router"]] = ParamDecl((self.E, self.hidden))
        if self.has_correction:
            d[self.names["correction"]] = ParamDecl((self.E,), init="zeros")
        if self.shared is not None:
            for local, decl in self.shared.param_decls().items():
                d[self.shared_prefix + self._shared_names[local]] = decl
        return d

    def prepare(self, ctx) -> None:
        super().prepare(ctx)
        if self.shared is not None:
            self.shared.prepare(ctx)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        pre = [self.expert_prefix.format(e) for e in range(self.E)]
        # per expert the rows alternate gate_j, up_j, so that a product's epilogue has both of a pair at hand:
        # [E, 2 ff, hidden]; the down matrices [E, hidden, ff]
        self.gate_up = torch.stack([torch.stack([tensors[p + n["gate"]], tensors[p + n["up"]]], dim=1)
                                   .reshape(2 * self.ff, self.hidden) for p in pre]).contiguous()
        self.down = torch.stack([tensors[p + n["down"]] for p in pre]).contiguous()
        # the router is 32-bit in both engines; the choice kernel forms its product itself
        self.router = tensors[n["router"]].to(torch.float32).contiguous()
        self.correction = tensors[n["correction"]].to(torch.float32).contiguous() if self.has_correction else None
        self.counts = torch.zeros(self.E, dtype=torch.int32, device=self.gate_up.device)   # the kernels leave it zero
        self.tensor_memory = (self.gate_up.dtype == torch.bfloat16 and self.gate_up.is_cuda
                              and K.gemm_tc_grouped_supports(0, 2 * self.ff, self.hidden)
                              and K.gemm_tc_grouped_supports(0, self.hidden, self.ff)
                              and os.environ.get("RUSTINFER_B200_EXPERTS", "tc") != "mma")
        if self.shared is not None:
            self.shared.load({local: tensors[self.shared_prefix + name] for local, name in self._shared_names.items()})

    def route(self, x: torch.Tensor):
        """(ids int32 [T, top], weights fp32 [T, top]); adds the choices to `self.counts`."""
        T = x.shape[0]
        ids = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        K.moe_route(None, self.correction, self.top, self.groups, self.keep, self.renorm, ids, weights, self.counts,
                    x=x if x.is_contiguous() else x.contiguous(), router=self.router, score=self.score)
        return ids, weights

    def forward(self, x: torch.Tensor, step: StepContext, residual: Optional[torch.Tensor] = None):
        T, dev = x.shape[0], x.device
        N = T * self.top
        ids, weights = self.route(x)
        offsets = torch.empty(self.E + 1, dtype=torch.int32, device=dev)
        order = torch.empty(N, dtype=torch.int32, device=dev)
        place = torch.empty(N, dtype=torch.int32, device=dev)
        K.moe_sort(ids, self.counts, offsets, order, place)
        mid = torch.empty((N, self.ff), dtype=self.gate_up.dtype, device=dev)
        Y = torch.empty((N, self.hidden), dtype=torch.float32, device=dev)
        xin = x if x.dtype == self.gate_up.dtype else x.to(self.gate_up.dtype)
        if (self.tensor_memory and N >= self.TC_ROWS_PER_EXPERT * self.E and xin.dtype == torch.bfloat16
                and xin.is_contiguous()):
            # many rows an expert: the rows gathered into expert order, both products on tcgen05 with TMA-fed
            # tiles of 128 rows that never cross from one expert's rows into the next one's results
            xs = torch.empty((N, self.hidden), dtype=torch.bfloat16, device=dev)
            K.moe_gather(xin, order, self.top, xs)
            K.gemm_tc_grouped(xs, self.gate_up, mid, offsets, K.EPI_SILU, act=self.act)
            K.gemm_tc_grouped(mid, self.down, Y, offsets, K.EPI_F32)
        else:
            K.moe_product(xin, self.gate_up, mid, offsets, order, self.top, gated=True, act=self.act)
            K.moe_product(mid, self.down, Y, offsets, None, self.top, gated=False)
        shared = self.shared.forward(x, step) if self.shared is not None else None
        out = torch.empty((T, self.hidden), dtype=torch.float32 if self.out_fp32 else self.ctx.dtype, device=dev)
        K.moe_combine(Y, place, weights, shared, out, self.counts)
        return out
