"""Shared by the Linedra tests: small configurations that differ from one another in every size, constant
and layer order, weights that make faults show, model folders, the plain model's logits."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch

import plain_linedra


def _parallel(heads, kv, dim, vdim, scale, mask, width, blocks, conv, ls, rs):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if mask:
        left["mask"] = {"size": mask}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv},
                                          "left_scale": ls, "right_scale": rs}}


def _latent(heads, dim, rot_dim, vdim, rank, q_rank, scale, base):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if q_rank:
        m["q_rank"] = q_rank
    return {"type": "latent_attention", "mixer": m}


def _layer(mixer, moe=None):
    mlp = None
    if moe:
        ff, limit, experts, top = moe
        mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    return dict(mixer, mlp=mlp)


# A: a parallel layer first, two kv heads for four heads, values wider than keys, a window of 20 (a page and a
#    quarter), four blocks in the recurrent unit whose convolution has two taps while the input convolution has
#    three; a latent layer with low-rank queries; a last parallel layer without a window, one kv head for six heads,
#    one block, and no feed-forward
# B: no `embedding`, `residual_mult` and `logit_softcap` keys; latent attention first, without `q_rank`; every token
#    uses one expert of three; a window equal to the page; as many kv heads as heads
# C: one head where it can be; an input convolution of one tap (no state) and a recurrent unit's of one; a window of
#    9 inside one page; keys much wider than values; every expert used by every token (top = experts); three heads
#    on a rotated part of four channels
# D: every attention size a multiple of 16, so that the bfloat16 engine's prompt portions run on the tensor-core
#    attention; a latent layer of eight heads and a last parallel layer of eight heads on one kv head, whose single
#    tokens run there too; a window of 50 (three pages and two tokens); five blocks
CONFIGS = {
    "A": {"architecture": "Linedra", "width": 96, "vocab": 211, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
          "embedding": {"scale": 0.7}, "residual_mult": 0.5, "logit_softcap": 20.0, "layers": [
              _layer(_parallel(4, 2, 16, 24, 0.3, 20, 64, 4, 2, 0.7, 0.9), (40, 1.5, 5, 2)),
              _layer(_latent(4, 24, 8, 16, 40, 24, 0.2, 500.0), (56, 3.0, 4, 3)),
              _layer(_parallel(6, 1, 8, 16, 0.4, None, 48, 1, 4, 1.1, 0.4))]},
    "B": {"architecture": "Linedra", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "canon": {"taps": 4}, "layers": [
        _layer(_latent(2, 32, 16, 64, 48, None, 0.15, 10000.0), (64, 2.5, 3, 1)),
        _layer(_parallel(2, 2, 32, 32, 0.2, 16, 128, 2, 4, 0.5, 0.5), (96, 1.0, 6, 2))]},
    "C": {"architecture": "Linedra", "width": 64, "vocab": 97, "norm": {"eps": 3e-6}, "canon": {"taps": 1},
          "embedding": {"scale": 2.0}, "residual_mult": 1.5, "logit_softcap": 5.0, "layers": [
              _layer(_parallel(1, 1, 40, 8, 0.25, 9, 24, 3, 1, 0.8, 1.2), (24, 0.7, 3, 3)),
              _layer(_latent(3, 20, 4, 36, 20, 12, 0.35, 50.0)),
              _layer(_parallel(1, 1, 8, 40, 0.5, 33, 72, 2, 3, 1.0, 1.0), (72, 4.0, 2, 1))]},
    "D": {"architecture": "Linedra", "width": 80, "vocab": 150, "norm": {"eps": 2e-5}, "canon": {"taps": 2},
          "embedding": {"scale": 1.5}, "residual_mult": 0.25, "logit_softcap": 30.0, "layers": [
              _layer(_parallel(4, 2, 16, 32, 0.25, 50, 80, 5, 3, 0.6, 0.5), (48, 2.0, 4, 2)),
              _layer(_latent(8, 16, 16, 32, 32, 40, 0.2, 1000.0), (32, 2.0, 8, 2)),
              _layer(_parallel(8, 1, 32, 32, 0.3, None, 32, 2, 4, 0.9, 0.3), (40, 6.0, 3, 2))]},
}


def tensor_shapes(name: str) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint, written out here so that the tests do not lean on the framework's own list."""
    cfg = CONFIGS[name]
    d, v, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    s = {"embed": (v, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        s.update({p + "norm1": (d,), p + "norm1b": (d,), p + "canon1": (d, taps), p + "dwa": (i + 2,)})
        if layer["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, W, nb = l["heads"], l["kv_heads"], r["width"], r["blocks"]
            s.update({p + "mix.left.q": (H * l["dim"], d), p + "mix.left.k": (G * l["dim"], d),
                      p + "mix.left.v": (G * l["vdim"], d), p + "mix.left.sink": (H,), p + "mix.left.g": (H, d),
                      p + "mix.left.o": (d, H * l["vdim"]),
                      p + "mix.right.y": (W, d), p + "mix.right.y.b": (W,), p + "mix.right.x": (W, d),
                      p + "mix.right.x.b": (W,), p + "mix.right.conv": (W, r["conv"]), p + "mix.right.conv.b": (W,),
                      p + "mix.right.ra": (nb, W // nb, W // nb), p + "mix.right.ra.b": (nb, W // nb),
                      p + "mix.right.ri": (nb, W // nb, W // nb), p + "mix.right.ri.b": (nb, W // nb),
                      p + "mix.right.lam": (W,), p + "mix.right.o": (d, W)})
        else:
            H, kd, nq = m["heads"], m["kv_rank"] + m["rot_dim"], m["heads"] * (m["dim"] + m["rot_dim"])
            if m.get("q_rank"):
                s.update({p + "mix.dq": (m["q_rank"], d), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (nq, m["q_rank"])})
            else:
                s[p + "mix.q"] = (nq, d)
            s.update({p + "mix.dkv": (kd, d), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                      p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.sink": (H,), p + "mix.g": (H * m["vdim"], d),
                      p + "mix.o": (d, H * m["vdim"])})
        if layer["mlp"]:
            ff, E = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"]
            s.update({p + "norm2": (d,), p + "norm2b": (d,), p + "mlp.router": (E, d)})
            for e in range(E):
                s.update({p + f"mlp.e{e}.gate": (ff, d), p + f"mlp.e{e}.up": (ff, d), p + f"mlp.e{e}.down": (d, ff)})
    return s


def sharp_weights(name: str, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Matrices of size 1/sqrt(fan_in) (q, k and the router several times that, so that attention and the choice of
    experts are peaked), norm weights spread around 0 (the model adds 1) except the two low-rank norms' (around 1),
    biases around 0, sinks and decay parameters with a spread of 1, depth weights that favour the newest result."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for n, shape in tensor_shapes(name).items():
        parts = n.split(".")
        leaf = parts[-1]
        if leaf == "dwa":
            t = 0.3 * torch.randn(shape, generator=g)
            t[-1] += 1.0
        elif leaf in ("sink", "lam"):
            t = torch.randn(shape, generator=g)
        elif leaf in ("canon1", "conv"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
            if parts[-2] in ("dq", "dkv"):
                t = t + 1.0
        elif n == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            if leaf in ("q", "k", "dkv", "uk", "uq", "router"):
                t = t * 2.0
        out[n] = t.to(dtype)
    return out


def write_model(folder: str, name: str, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(CONFIGS[name], f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def make_sharp_model(folder: str, name: str, seed: int = 0) -> str:
    return write_model(folder, name, sharp_weights(name, seed))


class Plain:
    """The plain implementation over one model folder, with per-sequence memo."""

    def __init__(self, folder: str):
        self.cfg, self.w = plain_linedra.read_model_folder(folder)
        self._memo = {}

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = plain_linedra.forward(self.cfg, self.w, list(ids))
        return self._memo[key]

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        ids, out = list(prompt), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(ids)[-1]))
            out.append(t)
            ids.append(t)
        return out
