"""Typed configuration of the Linedra decoder, read from config.json's own keys.

config.json names the width, the vocabulary, the norms' eps, the embedding's scale, the factor on every
sublayer's normed output (`residual_mult`), the taps of the convolution in front of every mixer (`canon.taps`),
a cap on the logits (`logit_softcap`) and a list of layers; every layer names its mixer (`type`: `parallel` or
`latent_attention`), the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`: `moe`, or null for
none).  Every size and constant is a field here.  What config.json leaves out does not exist in the model (no
`mask`: every earlier key is seen; no `kv_heads`: a key head a query head; no `embedding`: scale 1; no
`residual_mult`: 1; no `logit_softcap`: logits are not capped; no `q_rank`: queries come straight from the
input).  An unknown mixer type or feed-forward kind is an error, a key the engine does not know is named in a
warning.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .dirurax_config import _only
from .model_config import ConfigError, _eos_ids, _need
from .pikalix_config import _table


@dataclass(frozen=True)
class BiasAttentionConfig:
    """The attention side of a parallel mixer: grouped-query attention without rotation, a linear distance bias on
    the scores, a window of `mask_size` keys, a learned sink, a gate per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask_size: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BiasAttentionConfig":
        where = "the attention side of a parallel mixer"
        _only(d, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), where)
        mask = _table(d, "mask", where)
        if mask is not None:
            _only(mask, ("size",), "an attention mask")
        heads = _need(d, "heads")
        dim = _need(d, "dim")
        c = cls(heads, int(d["kv_heads"]) if d.get("kv_heads") is not None else heads, dim,
                int(d["vdim"]) if d.get("vdim") is not None else dim, _need(d, "scale", float),
                _need(mask, "size") if mask is not None else None)
        if min(c.heads, c.kv_heads, c.dim, c.vdim) <= 0 or c.heads % c.kv_heads:
            raise ConfigError("config.json: an attention mixer needs positive sizes and heads a multiple of kv_heads")
        if c.mask_size is not None and c.mask_size <= 0:
            raise ConfigError("config.json: mask.size must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.mask_size is not None:
            d["mask"] = {"size": self.mask_size}
        return d


@dataclass(frozen=True)
class RecurrentUnitConfig:
    """The recurrent side of a parallel mixer: `width` channels in `blocks` equal parts, a convolution of `conv` taps
    on the unit's input."""
    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RecurrentUnitConfig":
        _only(d, ("width", "blocks", "conv"), "the recurrent side of a parallel mixer")
        c = cls(_need(d, "width"), _need(d, "blocks"), _need(d, "conv"))
        if min(c.width, c.blocks, c.conv) <= 0 or c.width % c.blocks:
            raise ConfigError("config.json: a recurrent unit needs positive sizes and a width that its blocks divide")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class ParallelConfig:
    left: BiasAttentionConfig
    right: RecurrentUnitConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ParallelConfig":
        _only(d, ("left", "right", "left_scale", "right_scale"), "a parallel mixer")
        for side in ("left", "right"):
            if not isinstance(d.get(side), Mapping):
                raise ConfigError(f"config.json: a parallel mixer has no {side!r}")
        return cls(BiasAttentionConfig.from_dict(d["left"]), RecurrentUnitConfig.from_dict(d["right"]),
                   float(d["left_scale"]) if d.get("left_scale") is not None else 1.0,
                   float(d["right_scale"]) if d.get("right_scale") is not None else 1.0)

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class LatentConfig:
    """Attention whose keys and values are made from one cached vector of `kv_rank` channels per token plus `rot_dim`
    rotated key channels all heads share; queries through a vector of `q_rank` channels where that is given."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    q_rank: Optional[int] = None
    rot_base: float = 10000.0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LatentConfig":
        where = "a latent attention mixer"
        _only(d, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"), where)
        rot_dim = _need(d, "rot_dim")
        rot = _table(d, "rot", where)
        base = 10000.0
        if rot is not None:
            _only(rot, ("base", "dims"), "a rotation")
            base = _need(rot, "base", float)
            if rot.get("dims") is not None and int(rot["dims"]) != rot_dim:
                raise ConfigError("config.json: a latent attention mixer rotates its whole rotated part: rot.dims = rot_dim")
        c = cls(_need(d, "heads"), _need(d, "dim"), rot_dim, _need(d, "vdim"), _need(d, "kv_rank"),
                _need(d, "scale", float), int(d["q_rank"]) if d.get("q_rank") is not None else None, base)
        if min(c.heads, c.dim, c.vdim, c.kv_rank) <= 0 or c.rot_dim < 0 or c.rot_dim % 2 or not c.rot_base > 0:
            raise ConfigError("config.json: a latent attention mixer needs positive sizes and an even rot_dim")
        if c.q_rank is not None and c.q_rank <= 0:
            raise ConfigError("config.json: q_rank must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                             "kv_rank": self.kv_rank, "scale": self.scale,
                             "rot": {"base": self.rot_base, "dims": self.rot_dim}}
        if self.q_rank is not None:
            d["q_rank"] = self.q_rank
        return d


@dataclass(frozen=True)
class ClampedExpertsConfig:
    """`experts` gated feed-forwards of `ff` channels whose gate and up products are clamped at `limit`; a token
    uses the `top` with the largest router logits."""
    ff: int
    limit: float
    experts: int
    top: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ClampedExpertsConfig":
        _only(d, ("kind", "expert", "router"), "a feed-forward of experts")
        expert, router = _table(d, "expert", "a feed-forward"), _table(d, "router", "a feed-forward")
        if expert is None or router is None:
            raise ConfigError("config.json: a feed-forward of experts names its 'expert' and its 'router'")
        _only(expert, ("ff", "limit"), "an expert")
        _only(router, ("experts", "top"), "a router")
        c = cls(_need(expert, "ff"), _need(expert, "limit", float), _need(router, "experts"), _need(router, "top"))
        if c.ff <= 0 or not c.limit > 0 or not 1 <= c.top <= c.experts:
            raise ConfigError("config.json: experts need a positive ff and limit, and 1 <= top <= experts")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top}}


MixerConfig = Union[ParallelConfig, LatentConfig]
_MIXERS = {"parallel": ParallelConfig, "latent_attention": LatentConfig}
_MLPS = {"moe": ClampedExpertsConfig}


@dataclass(frozen=True)
class LinedraLayer:
    type: str
    mixer: MixerConfig
    mlp: Optional[ClampedExpertsConfig]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], index: int) -> "LinedraLayer":
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
class LinedraConfig:
    width: int
    vocab: int
    norm_eps: float
    canon_taps: int
    layers: Tuple[LinedraLayer, ...]
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    logit_softcap: Optional[float] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Linedra"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Optional[Mapping[str, Any]] = None) -> "LinedraConfig":
        norm, canon = d.get("norm"), d.get("canon")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: required key 'norm' is missing")
        if not isinstance(canon, Mapping):
            raise ConfigError("config.json: required key 'canon' is missing")
        _only(canon, ("taps",), "the input convolution")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        emb = _table(d, "embedding", "the model")
        if emb is not None:
            _only(emb, ("scale",), "the embedding")
        vocab = _need(d, "vocab")
        cfg = cls(width=_need(d, "width"), vocab=vocab, norm_eps=_need(norm, "eps", float),
                  canon_taps=_need(canon, "taps"),
                  layers=tuple(LinedraLayer.from_dict(l, i) for i, l in enumerate(layers)),
                  embedding_scale=float(emb["scale"]) if emb is not None and emb.get("scale") is not None else 1.0,
                  residual_mult=float(d["residual_mult"]) if d.get("residual_mult") is not None else 1.0,
                  logit_softcap=float(d["logit_softcap"]) if d.get("logit_softcap") is not None else None,
                  eos_token_ids=_eos_ids(d, generation, vocab),
                  architecture=str(d.get("architecture") or "Linedra"))
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.norm_eps > 0 or cfg.canon_taps <= 0:
            raise ConfigError("config.json: width, vocab, norm.eps and canon.taps must be positive")
        if cfg.logit_softcap is not None and not cfg.logit_softcap > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
                             "layers": [l.to_dict() for l in self.layers]}
        if self.embedding_scale != 1.0:
            d["embedding"] = {"scale": self.embedding_scale}
        if self.residual_mult != 1.0:
            d["residual_mult"] = self.residual_mult
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
