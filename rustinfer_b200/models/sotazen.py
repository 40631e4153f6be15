"""The Sotazen decoder as a registry entry: configuration -> model spec.

A token embedding times a scale; layers in the order config.json lists them, each normed AFTER the
residual sum (the `post_norm` arrangement: h <- norm1(alpha h + mixer(h)), h <- norm2(alpha h + ffn(h)),
the sublayers reading the stream itself); three kinds of mixer, differential attention (`attention`),
linear attention with fixed decays (`lightning`) and attention over a cached low-rank vector
(`latent_attention`); a dense feed-forward with the square of relu where the layer has one; a last RMS
norm and a head that is the embedding table without its scale.  Nothing here computes: the spec names
registered parts and hands them the numbers of config.json.

Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*` (a bias with
`.b`, a norm weight with `.norm` added to the projection's name), `l<i>.mlp.up`, `l<i>.mlp.down`.
"""
from __future__ import annotations

from ..config.registry import ArchitectureFamily, register_architecture
from ..config.sotazen_config import DiffAttentionConfig, LatentAttentionConfig, LightningConfig, SotazenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer_spec(cfg: SotazenConfig, m) -> PartSpec:
    if isinstance(m, DiffAttentionConfig):
        rope = None
        if m.rot_dims:
            rope = PartSpec("rope", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                     "scaling": None, "layout": "interleaved"})
        return PartSpec("differential_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
            "value_dim": m.vdim, "scale": m.scale, "diff": m.diff, "softcap": m.softcap, "window": m.mask_size,
            "position": rope, "qk_norm_eps": cfg.norm_eps, "norm_eps": cfg.norm_eps, "bias": True, "gate": True})
    if isinstance(m, LightningConfig):
        return PartSpec("lightning_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
            "decay": list(m.decay), "norm_eps": cfg.norm_eps})
    if isinstance(m, LatentAttentionConfig):
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
            "value_dim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale, "rot_base": m.rot_base,
            "norm_eps": cfg.norm_eps, "sink": True})
    raise TypeError(f"no mixer for {type(m).__name__}")


def sotazen_model_spec(cfg: SotazenConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."

        def norm(q: int) -> PartSpec:
            return PartSpec("post_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "alpha": cfg.postln_alpha,
                                             "weight_name": f"norm{q}"})
        names = {"mixer": p + "mix.", "mixer_norm": p}
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff,
                                         "activation": "relu_squared", "up_name": "up", "down_name": "down",
                                         "output": "float32"})
            names.update({"ffn": p + "mlp.", "ffn_norm": p})
        layers.append(LayerSpec(mixer=_mixer_spec(cfg, layer.mixer), mixer_norm=norm(1), ffn=ffn,
                                ffn_norm=norm(2) if ffn else None, names=names, arrangement="post_norm"))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""}),
        embed_name="embed", final_norm_name="final.norm", head_name="head.",
        tie_head=True, eos_token_ids=cfg.eos_token_ids,
        embed=PartSpec("scaled_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                            "scale": cfg.embedding_scale, "weight_name": ""}))


SOTAZEN = ArchitectureFamily(name="sotazen", parse_config=SotazenConfig.from_dict, model_spec=sotazen_model_spec)
register_architecture(["sotazen"], SOTAZEN)
