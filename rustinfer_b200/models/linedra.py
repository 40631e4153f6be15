"""The Linedra decoder as a registry entry: configuration -> model spec.

A token embedding times a scale; layers in the order config.json lists them, each with an RMS norm (weights stored
around zero) before and after each sublayer and the factor `residual_mult` on what is added, a short causal
convolution in front of the mixer, and a weighted average over all earlier layers' results as the next layer's
input (the `sandwich_depth_average` arrangement).  Two kinds of mixer: `parallel` (attention with a linear distance
bias, a window, a sink and a gate per head, beside a gated linear recurrent unit) and `latent_attention` (queries
through a low-rank vector, keys and values from one cached low-rank vector a token).  The feed-forward is routed
experts with clamped gated pairs; the head is the embedding table without its scale, the logits capped by a tanh.
Nothing here computes: the spec names registered parts and hands them the numbers of config.json.

Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`,
`l<i>.canon1`, `l<i>.dwa`, `l<i>.mix.*` (a parallel mixer's sides under `left.` and `right.`; a bias with `.b`, a
norm weight with `.norm` added to the projection's name), `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`.
"""
from __future__ import annotations

from ..config.linedra_config import LatentConfig, LinedraConfig, ParallelConfig
from ..config.registry import ArchitectureFamily, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

SLOPE_EXPONENT = 8.0         # the attention's distance slopes are 2^(-8 (h + 1) / heads)
DECAY_SCALE = 8.0            # log a = -8 r softplus(lam) in the recurrent unit
GATE_ALPHA = 1.702           # an expert's gate is g sigmoid(1.702 g)


def _mixer_spec(cfg: LinedraConfig, m) -> PartSpec:
    if isinstance(m, ParallelConfig):
        left = PartSpec("distance_bias_attention", {
            "hidden_size": cfg.width, "num_heads": m.left.heads, "num_kv_heads": m.left.kv_heads,
            "head_dim": m.left.dim, "value_dim": m.left.vdim, "scale": m.left.scale, "window": m.left.mask_size,
            "slope_exponent": SLOPE_EXPONENT, "sink": True, "head_gate": True})
        right = PartSpec("gated_recurrent_unit", {
            "hidden_size": cfg.width, "width": m.right.width, "blocks": m.right.blocks, "conv_taps": m.right.conv,
            "decay_scale": DECAY_SCALE})
        return PartSpec("parallel_mixers", {"left": left, "right": right, "left_scale": m.left_scale,
                                            "right_scale": m.right_scale})
    if isinstance(m, LatentConfig):
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
            "value_dim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "rot_base": m.rot_base,
            "rot_layout": "half", "norm_eps": cfg.norm_eps, "sink": True, "gate": True})
    raise TypeError(f"no mixer for {type(m).__name__}")


def linedra_model_spec(cfg: LinedraConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."

        def norm(name: str, scale: float = 1.0) -> PartSpec:
            return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": name, "offset": 1.0,
                                        "scale": scale})
        mixer = PartSpec("conv_input", {"inner": _mixer_spec(cfg, layer.mixer), "size": cfg.width,
                                        "taps": cfg.canon_taps, "weight_name": "canon1", "inner_prefix": "mix."})
        extra = {"post_mixer_norm": norm("norm1b", cfg.residual_mult),
                 "depth_average": PartSpec("depth_average", {"count": i + 2, "weight_name": "dwa"})}
        names = {"mixer": p, "mixer_norm": p, "post_mixer_norm": p, "depth_average": p}
        ffn = None
        if layer.mlp is not None:
            e = layer.mlp
            ffn = PartSpec("routed_experts", {"hidden_size": cfg.width, "expert_ff": e.ff, "experts": e.experts,
                                              "top": e.top, "score": "softmax_chosen", "activation": "clamped",
                                              "limit": e.limit, "alpha": GATE_ALPHA, "output": "float32"})
            extra["post_ffn_norm"] = norm("norm2b", cfg.residual_mult)
            names.update({"ffn": p + "mlp.", "ffn_norm": p, "post_ffn_norm": p})
        layers.append(LayerSpec(mixer=mixer, mixer_norm=norm("norm1"), ffn=ffn,
                                ffn_norm=norm("norm2") if ffn else None, names=names,
                                arrangement="sandwich_depth_average", extra_norms=extra))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": "", "offset": 1.0}),
        embed_name="embed", final_norm_name="final.norm", head_name="head.",
        tie_head=True, eos_token_ids=cfg.eos_token_ids,
        embed=PartSpec("scaled_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                            "scale": cfg.embedding_scale, "weight_name": ""}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": True,
                                      "softcap": cfg.logit_softcap}),
        depth_average=True)


LINEDRA = ArchitectureFamily(name="linedra", parse_config=LinedraConfig.from_dict, model_spec=linedra_model_spec)
register_architecture(["linedra"], LINEDRA)
