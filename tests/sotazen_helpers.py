"""Shared by the Sotazen tests: small configurations that differ from one another in every size, constant
and layer order, weights that make faults show, model folders, the plain model's logits."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch

import plain_sotazen


def _att(heads, kv, dim, vdim, scale, diff, mask=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if mask:
        m["mask"] = {"size": mask}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def _lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                                                  "kv_rank": rank, "scale": scale,
                                                  "rot": {"dims": rot_dim, "base": base}}}


def _layer(mixer, ff=None):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


# A: attention first (the stem's output is rounded by the block itself); two kv heads for four heads, values wider
#    than keys, a window of 20 (a page and a quarter), a cap on the scores, rotation on half of a map; a lightning
#    layer without a feed-forward, keys and values of different sizes; a latent layer; a second attention layer
#    without window or cap, one kv head for six heads, whole maps rotated (its pages are a group of their own)
# B: no `embedding` and no `postln_alpha` key (both 1); latent attention first; a lightning layer with keys wider
#    than values and a decay close to one; attention with as many kv heads as heads, no rotation, a window equal
#    to the page
# C: one head everywhere it can be; a lightning layer first; attention with a window of 9 inside one page and no
#    feed-forward (its `diff` small: with scores capped at 1.5 the two maps are nearly alike, and a weight near one on
#    the second would leave a difference that is mostly rounding in bfloat16); a latent layer of three heads with a
#    rotated part of four channels; alpha below one
# D: every attention size a multiple of 16, so that the bfloat16 engine's prompt portions run on the tensor-core
#    attention; a latent layer of eight heads, whose single tokens run there too with their keys in ranges once the
#    context passes 128; attention with a window of 50 (three pages and two tokens) over two kv heads, whole maps rotated;
#    a last attention layer of eight heads on one kv head without a window, whose single tokens take the same way
#    with two maps
CONFIGS = {
    "A": {"architecture": "Sotazen", "width": 96, "vocab": 211, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.7},
          "postln_alpha": 2.0, "layers": [
              _layer(_att(4, 2, 16, 24, 0.3, 0.3, mask=20, rot=(8, 10000.0), softcap=20.0), 136),
              _layer(_lightning(3, 16, 40, [0.5, 0.9, 0.99])),
              _layer(_latent(4, 24, 8, 16, 40, 0.2, 500.0), 72),
              _layer(_att(6, 1, 8, 16, 0.4, 0.5, rot=(8, 300.0)), 104)]},
    "B": {"architecture": "Sotazen", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "layers": [
        _layer(_latent(2, 32, 16, 64, 48, 0.15, 10000.0), 256),
        _layer(_lightning(2, 64, 32, [0.8, 0.999]), 192),
        _layer(_att(2, 2, 32, 32, 0.2, 0.2, mask=16, softcap=5.0), 160)]},
    "C": {"architecture": "Sotazen", "width": 64, "vocab": 97, "norm": {"eps": 3e-6}, "embedding": {"scale": 2.0},
          "postln_alpha": 0.5, "layers": [
              _layer(_lightning(1, 20, 12, [0.95]), 72),
              _layer(_att(1, 1, 40, 8, 0.25, 0.15, mask=9, rot=(20, 1e6), softcap=1.5)),
              _layer(_latent(3, 20, 4, 36, 20, 0.35, 50.0), 80)]},
    "D": {"architecture": "Sotazen", "width": 80, "vocab": 150, "norm": {"eps": 2e-5}, "embedding": {"scale": 1.5},
          "postln_alpha": 1.5, "layers": [
              _layer(_lightning(2, 16, 16, [0.7, 0.97]), 96),
              _layer(_att(4, 2, 16, 32, 0.25, 0.4, mask=50, rot=(16, 20000.0), softcap=10.0), 112),
              _layer(_latent(8, 16, 16, 24, 32, 0.2, 1000.0), 64),
              _layer(_att(8, 1, 16, 16, 0.3, 0.25, rot=(8, 700.0)))]},
}


def tensor_shapes(name: str) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint, written out here so that the tests do not lean on the framework's own list."""
    cfg = CONFIGS[name]
    d, v = cfg["width"], cfg["vocab"]
    s = {"embed": (v, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        s[p + "norm1"] = (d,)
        if layer["type"] == "attention":
            q, k, vv, hv = m["heads"] * 2 * m["dim"], m["kv_heads"] * 2 * m["dim"], m["kv_heads"] * m["vdim"], m["heads"] * m["vdim"]
            s.update({p + "mix.q": (q, d), p + "mix.q.b": (q,), p + "mix.k": (k, d), p + "mix.k.b": (k,),
                      p + "mix.v": (vv, d), p + "mix.v.b": (vv,), p + "mix.q.norm": (m["dim"],), p + "mix.k.norm": (m["dim"],),
                      p + "mix.lq1": (m["dim"],), p + "mix.lk1": (m["dim"],), p + "mix.lq2": (m["dim"],),
                      p + "mix.lk2": (m["dim"],), p + "mix.g": (hv, d), p + "mix.o": (d, hv), p + "mix.o.b": (d,)})
        elif layer["type"] == "lightning":
            qk, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            s.update({p + "mix.q": (qk, d), p + "mix.k": (qk, d), p + "mix.v": (hv, d), p + "mix.g": (hv, d),
                      p + "mix.o": (d, hv), p + "mix.norm": (hv,)})
        else:
            H, kd = m["heads"], m["kv_rank"] + m["rot_dim"]
            s.update({p + "mix.q": (H * (m["dim"] + m["rot_dim"]), d), p + "mix.dkv": (kd, d),
                      p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                      p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.sink": (H,), p + "mix.o": (d, H * m["vdim"])})
        if layer["mlp"]:
            s.update({p + "norm2": (d,), p + "mlp.up": (layer["mlp"]["ff"], d), p + "mlp.down": (d, layer["mlp"]["ff"])})
    return s


def sharp_weights(name: str, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Matrices of size 1/sqrt(fan_in) (q and k several times that, so that attention is peaked), norm weights
    spread around 1, biases around 0, sinks around 0 with a spread of 1, and the four vectors behind lambda small
    enough that lambda stays of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for n, shape in tensor_shapes(name).items():
        leaf = n.split(".")[-1]
        if leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "sink":
            t = torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
            if leaf != "b":
                t = t + 1.0
        elif n == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf in ("q", "k", "dkv", "uk"):
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
        self.cfg, self.w = plain_sotazen.read_model_folder(folder)
        self._memo = {}

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = plain_sotazen.forward(self.cfg, self.w, list(ids))
        return self._memo[key]

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        ids, out = list(prompt), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(ids)[-1]))
            out.append(t)
            ids.append(t)
        return out
