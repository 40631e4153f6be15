"""Typed configuration of the Sotazen decoder, read from config.json's own keys.

config.json names the width, the vocabulary, the norms' eps, the embedding's scale, the factor the
stream is multiplied by before a sublayer's output is added (`postln_alpha`) and a list of layers;
every layer names its mixer (`type`: `attention`, `lightning` or `latent_attention`), the mixer's sizes
and constants (`mixer`) and its feed-forward (`mlp`: `dense`, or null for none).  Every size and
constant is a field here.  What config.json leaves out does not exist in the model (no `mask`: every
earlier key is seen; no `rot`: no rotation; no `softcap`: scores are not capped; no `kv_heads`: a key
head a query head; no `embedding`: scale 1; no `postln_alpha`: 1).  An unknown mixer type or
feed-forward kind is an error, a key the engine does not know is named in a warning.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .dirurax_config import DenseMlpConfig, _only
from .model_config import ConfigError, _eos_ids, _need
from .pikalix_config import _table


def _rot(d: Mapping[str, Any], where: str) -> Tuple[int, float]:
    rot = _table(d, "rot", where)
    if rot is None:
        return 0, 10000.0
    _only(rot, ("base", "dims"), "a rotation")
    dims, base = _need(rot, "dims"), _need(rot, "base", float)
    if dims < 0 or dims % 2 or not base > 0:
        raise ConfigError(f"config.json: {where}: rot.dims is even and rot.base positive")
    return dims, base


@dataclass(frozen=True)
class DiffAttentionConfig:
    """Differential attention: every head has two softmax maps with queries and keys of their own (size
    `dim`) over one set of values (size `vdim`); the second map is subtracted with a learned weight that
    `diff` enters.  Grouped key/value heads, biased projections, q and k normed per head and map, rotary
    pairs on the first `rot_dims` channels, scores capped at `softcap`, a window of `mask_size` keys, an
    output gate."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    softcap: Optional[float] = None
    mask_size: Optional[int] = None
    rot_dims: int = 0
    rot_base: float = 10000.0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DiffAttentionConfig":
        where = "an attention mixer"
        _only(d, ("heads", "kv_heads", "dim", "vdim", "scale", "diff", "softcap", "mask", "rot"), where)
        mask = _table(d, "mask", where)
        if mask is not None:
            _only(mask, ("size",), "an attention mask")
        rot_dims, rot_base = _rot(d, where)
        heads = _need(d, "heads")
        c = cls(heads, int(d["kv_heads"]) if d.get("kv_heads") is not None else heads, _need(d, "dim"),
                _need(d, "vdim"), _need(d, "scale", float), _need(d, "diff", float),
                float(d["softcap"]) if d.get("softcap") is not None else None,
                _need(mask, "size") if mask is not None else None, rot_dims, rot_base)
        if min(c.heads, c.kv_heads, c.dim, c.vdim) <= 0 or c.heads % c.kv_heads:
            raise ConfigError("config.json: an attention mixer needs positive sizes and heads a multiple of kv_heads")
        if c.mask_size is not None and c.mask_size <= 0:
            raise ConfigError("config.json: mask.size must be positive")
        if c.softcap is not None and not c.softcap > 0:
            raise ConfigError("config.json: softcap must be positive")
        if c.rot_dims > c.dim:
            raise ConfigError("config.json: rot.dims is at most dim")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale, "diff": self.diff}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.mask_size is not None:
            d["mask"] = {"size": self.mask_size}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class LightningConfig:
    """Linear attention with one fixed decay per head: a state [dim, vdim] per head and request."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LightningConfig":
        _only(d, ("heads", "dim", "vdim", "decay"), "a lightning mixer")
        decay = d.get("decay")
        if not isinstance(decay, (list, tuple)):
            raise ConfigError("config.json: a lightning mixer lists one 'decay' per head")
        try:
            c = cls(_need(d, "heads"), _need(d, "dim"), _need(d, "vdim"), tuple(float(x) for x in decay))
        except (TypeError, ValueError):
            raise ConfigError("config.json: a lightning mixer's decays are numbers")
        if min(c.heads, c.dim, c.vdim) <= 0 or len(c.decay) != c.heads:
            raise ConfigError("config.json: a lightning mixer needs positive sizes and one decay per head")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class LatentAttentionConfig:
    """Attention whose keys and values are made from one cached vector of `kv_rank` channels per token
    plus `rot_dim` rotated key channels all heads share; a head's queries have `dim` plain and `rot_dim`
    rotated channels.  Causal, with a learned term per head in the softmax's denominator."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float = 10000.0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LatentAttentionConfig":
        where = "a latent attention mixer"
        _only(d, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), where)
        rot_dim = _need(d, "rot_dim")
        dims, base = _rot(d, where)
        if d.get("rot") is not None and dims != rot_dim:
            raise ConfigError("config.json: a latent attention mixer rotates its whole rotated part: rot.dims = rot_dim")
        c = cls(_need(d, "heads"), _need(d, "dim"), rot_dim, _need(d, "vdim"), _need(d, "kv_rank"),
                _need(d, "scale", float), base)
        if min(c.heads, c.dim, c.vdim, c.kv_rank) <= 0 or c.rot_dim < 0 or c.rot_dim % 2:
            raise ConfigError("config.json: a latent attention mixer needs positive sizes and an even rot_dim")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dim}}


MixerConfig = Union[DiffAttentionConfig, LightningConfig, LatentAttentionConfig]
_MIXERS = {"attention": DiffAttentionConfig, "lightning": LightningConfig, "latent_attention": LatentAttentionConfig}
_MLPS = {"dense": DenseMlpConfig}


@dataclass(frozen=True)
class SotazenLayer:
    type: str
    mixer: MixerConfig
    mlp: Optional[DenseMlpConfig]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], index: int) -> "SotazenLayer":
        _only(d, ("type", "mixer", "mlp"), f"layer {index}")
        kind = d.get("type")
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: layer {index} has mixer type {kind!r}; known: {sorted(_MIXERS)}")
        if not isinstance(d.get("mixer"), Mapping):
            raise ConfigError(f"config.json: layer {index} has no 'mixer'")
        mlp = _table(d, "mlp", f"layer {index}")
        if mlp is not None and mlp.get("kind") not in _MLPS:
            raise ConfigError(f"config.json: layer {index}: feed-forward kind {mlp.get('kind')!r} is not built; "
                              f"known: {sorted(_MLPS)}")
        return cls(kind, _MIXERS[kind].from_dict(d["mixer"]),
                   _MLPS[mlp["kind"]].from_dict(mlp) if mlp is not None else None)

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class SotazenConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: Tuple[SotazenLayer, ...]
    embedding_scale: float = 1.0
    postln_alpha: float = 1.0
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Sotazen"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Optional[Mapping[str, Any]] = None) -> "SotazenConfig":
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: required key 'norm' is missing")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        emb = _table(d, "embedding", "the model")
        if emb is not None:
            _only(emb, ("scale",), "the embedding")
        vocab = _need(d, "vocab")
        cfg = cls(width=_need(d, "width"), vocab=vocab, norm_eps=_need(norm, "eps", float),
                  layers=tuple(SotazenLayer.from_dict(l, i) for i, l in enumerate(layers)),
                  embedding_scale=float(emb["scale"]) if emb is not None and emb.get("scale") is not None else 1.0,
                  postln_alpha=float(d["postln_alpha"]) if d.get("postln_alpha") is not None else 1.0,
                  eos_token_ids=_eos_ids(d, generation, vocab),
                  architecture=str(d.get("architecture") or "Sotazen"))
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: width, vocab and norm.eps must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "layers": [l.to_dict() for l in self.layers]}
        if self.embedding_scale != 1.0:
            d["embedding"] = {"scale": self.embedding_scale}
        if self.postln_alpha != 1.0:
            d["postln_alpha"] = self.postln_alpha
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
