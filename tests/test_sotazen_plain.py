"""The plain Sotazen model against closed forms and hand-made cases, and what the package derives from a
config.json without a GPU: the typed configuration, the declared tensors, the cache layout, configuration
errors, the random-weights mode."""
import json
import math

import pytest
import torch

import plain_sotazen as P
from sotazen_helpers import CONFIGS, tensor_shapes

F64 = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# ------------------------------------------------------------------------ the plain model
def test_rotation_by_hand():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 7.0]]], dtype=F64).repeat(3, 1, 1)      # [T=3, 1, 6], dims 4
    y = P.rotate_pairs(x, torch.arange(3), 4, 100.0)
    assert torch.equal(y[0], x[0])                                                       # position 0: no turn
    for p in (1, 2):
        a0, a1 = p * 1.0, p * 100.0 ** (-2.0 / 4)
        want = [math.cos(a0), math.sin(a0), -2.0 * math.sin(a1), 2.0 * math.cos(a1), 5.0, 7.0]
        assert torch.allclose(y[p, 0], torch.tensor(want, dtype=F64))
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))


def test_window_is_exactly_its_size():
    m = P.visible(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True]
    assert m[1].tolist() == [True, True, False, False, False, False]
    assert P.visible(4, None)[3].tolist() == [True] * 4


def test_softmax_with_a_sink():
    """One key of score s beside a sink of the same exponent: weight 1/2; a sink far above: weight ~0; none: 1."""
    s = torch.zeros(2, 1, 1, dtype=F64) + 0.7
    mask = torch.ones(1, 1, dtype=torch.bool)
    assert torch.allclose(P.softmax_rows(s, mask, torch.tensor([0.7, 30.7], dtype=F64)).flatten(),
                          torch.tensor([0.5, 1.0 / (1.0 + math.exp(30.0))], dtype=F64))
    assert torch.allclose(P.softmax_rows(s, mask), torch.ones(2, 1, 1, dtype=F64))


def test_two_maps_and_their_difference():
    """Equal maps cancel to lam-dependent multiples of one vector, which the head norm makes a unit-rms vector."""
    T, H, G, d, vd = 5, 4, 2, 6, 3
    q, k, v = rnd(T, H, 1, d).repeat(1, 1, 2, 1), rnd(T, G, 1, d, seed=1).repeat(1, 1, 2, 1), rnd(T, G, vd, seed=2)
    maps = P.two_map_attention(q, k, v, 0.4, None, None)
    assert torch.allclose(maps[:, :, 0], maps[:, :, 1])
    assert torch.allclose(maps[0, 0, 0], v[0, 0]) and torch.allclose(maps[0, 3, 1], v[0, 1])    # token 0 sees itself
    o = P.difference_of_maps(maps, 0.25, 0.4, 0.0)
    assert torch.allclose(o, P.rms_norm(maps[:, :, 0], None, 0.0) * 0.6)
    # a cap far above the scores changes nothing; a small one flattens the softmax towards the mean of the values
    assert torch.allclose(P.two_map_attention(q, k, v, 0.4, 1e6, None), maps)
    flat = P.two_map_attention(q, k, v, 0.4, 1e-6, None)
    assert torch.allclose(flat[4, 0, 0], v[:, 0].mean(0), atol=1e-5)
    w = {"lq1": torch.tensor([1.0, 2.0]), "lk1": torch.tensor([0.5, 0.25]), "lq2": torch.tensor([0.0, 1.0]),
         "lk2": torch.tensor([3.0, -1.0])}
    assert math.isclose(P.map_weight(w, 0.3), math.e - math.exp(-1.0) + 0.3)


def test_decay_recurrence_closed_form():
    """o_t = sum_{s <= t} decay^(t-s) (q_t . k_s) v_s, and a walk in two pieces through the state is the walk in one."""
    T, H, d, vd = 9, 2, 5, 3
    q, k, v = rnd(T, H, d), rnd(T, H, d, seed=1), rnd(T, H, vd, seed=2)
    decay = torch.tensor([0.5, 0.97], dtype=F64)
    out, S = P.decay_recurrence(q, k, v, decay)
    for h in range(H):
        for t in (0, 4, 8):
            want = sum(decay[h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(out[t, h], want)
    a, Sa = P.decay_recurrence(q[:4], k[:4], v[:4], decay)
    b, Sb = P.decay_recurrence(q[4:], k[4:], v[4:], decay, Sa)
    assert torch.allclose(torch.cat([a, b]), out) and torch.allclose(Sb, S)


def test_latent_attention_is_attention_over_made_keys():
    T, H, d, r, vd, rank = 6, 3, 4, 2, 5, 7
    qp, qr, c, kr = rnd(T, H, d), rnd(T, H, r, seed=1), rnd(T, rank, seed=2), rnd(T, r, seed=3)
    uk, uv, sink = rnd(H * d, rank, seed=4), rnd(H * vd, rank, seed=5), rnd(H, seed=6)
    got = P.latent_scores_attention(qp, qr, c, kr, uk, uv, 0.3, sink)
    for h in range(H):
        K_ = torch.cat([c @ uk[h * d:(h + 1) * d].T, kr], dim=1)
        V_ = c @ uv[h * vd:(h + 1) * vd].T
        for t in range(T):
            s = (torch.cat([qp[t, h], qr[t, h]]) @ K_[: t + 1].T) * 0.3
            e = torch.exp(s)
            want = (e[:, None] * V_[: t + 1]).sum(0) / (e.sum() + torch.exp(sink[h]))
            assert torch.allclose(got[t, h], want)


def test_feed_forward_and_norm():
    x, w = rnd(4, 9), rnd(9, seed=1)
    assert torch.allclose(P.rms_norm(x, w, 0.5), x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 0.5) * w)
    up, down = rnd(6, 9, seed=2), rnd(9, 6, seed=3)
    assert torch.allclose(P.feed_forward(x, {"up": up, "down": down}), (torch.clamp(x @ up.T, min=0) ** 2) @ down.T)


def test_block_norms_after_the_sum():
    """One lightning layer by hand: x1 = norm1(alpha x + mixer(x)), x2 = norm2(alpha x1 + ff(x1)); the logits
    use the unscaled table."""
    cfg = {"width": 8, "vocab": 5, "norm": {"eps": 1e-3}, "embedding": {"scale": 3.0}, "postln_alpha": 1.5,
           "layers": [{"type": "lightning", "mixer": {"heads": 2, "dim": 3, "vdim": 2, "decay": [0.9, 0.5]},
                       "mlp": {"kind": "dense", "ff": 6}}]}
    shapes = {"embed": (5, 8), "final.norm": (8,), "l0.norm1": (8,), "l0.norm2": (8,), "l0.mix.q": (6, 8), "l0.mix.k": (6, 8),
              "l0.mix.v": (4, 8), "l0.mix.g": (4, 8), "l0.mix.o": (8, 4), "l0.mix.norm": (4,), "l0.mlp.up": (6, 8),
              "l0.mlp.down": (8, 6)}
    w = {n: rnd(*s, seed=i) for i, (n, s) in enumerate(shapes.items())}
    ids = [4, 0, 2]
    taps = []
    logits = P.forward(cfg, w, ids, taps)
    x = w["embed"][ids] * 3.0
    sub = {k[len("l0.mix."):]: v for k, v in w.items() if k.startswith("l0.mix.")}
    x1 = P.rms_norm(1.5 * x + P.lightning_attention(x, sub, cfg["layers"][0]["mixer"], 1e-3), w["l0.norm1"], 1e-3)
    x2 = P.rms_norm(1.5 * x1 + P.feed_forward(x1, {"up": w["l0.mlp.up"], "down": w["l0.mlp.down"]}), w["l0.norm2"], 1e-3)
    assert torch.allclose(taps[0], x2)
    assert torch.allclose(logits, P.rms_norm(x2, w["final.norm"], 1e-3) @ w["embed"].T)


# --------------------------------------------------------------------- configuration, registry
def test_registry_and_declared_tensors():
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    for name, cfg in CONFIGS.items():
        fam = resolve_architecture(cfg)
        assert fam.name == "sotazen"
        typed = fam.parse_config(cfg, None)
        assert typed.to_dict() == cfg
        spec = fam.model_spec(typed)
        decls = Decoder(spec).param_decls()
        assert {n: tuple(d.shape) for n, d in decls.items() if not d.optional} == tensor_shapes(name)   # the tied head is optional
        assert [ls.arrangement for ls in spec.layers] == ["post_norm"] * len(cfg["layers"])


def test_cache_layout_of_mixed_layers():
    """Lightning layers share one group of state slots; a latent layer keeps one row of kv_rank + rot_dim a token
    and no values; an attention layer keeps two key heads a value head, and layers with different windows (or
    sizes) have page groups of their own."""
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.cache.manager import CacheLayout
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    from rustinfer_b200.parts.base import FixedState, PagedKV
    fam = resolve_architecture(CONFIGS["A"])
    dec = Decoder(fam.model_spec(fam.parse_config(CONFIGS["A"], None)))
    needs = [n for _, n, _ in dec.cache_needs()]
    assert needs[0] == PagedKV(2, 16, 20, value_dim=24, key_maps=2) and needs[0].elems_per_token() == 2 * 2 * 16 + 2 * 24
    assert isinstance(needs[1], FixedState) and needs[1].shape[:2] == (3, 40)
    assert needs[2] == PagedKV(1, 48, None, value_dim=40, value_in_key=True) and needs[2].elems_per_token() == 48
    assert needs[3].window is None and needs[3].key_maps == 2 and not needs[3].plain
    layout = CacheLayout.from_needs(dec.cache_needs())
    assert len(layout.groups) == 4 and len(layout.paged_groups()) == 3
    # pages before a window are given back; none of a layer that sees every key
    assert needs[0].first_key_kept(100) == 81 and needs[2].first_key_kept(100) == 0


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].__setitem__("type", "gla"), "mixer type"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "feed-forward kind"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("softcap", 0.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.9]), "one decay per head"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 4), "rot.dims = rot_dim"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("rot_dim", 7), "rot"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_configuration_errors(change, needle):
    from rustinfer_b200.config.model_config import ConfigError
    from rustinfer_b200.config.sotazen_config import SotazenConfig
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    change(cfg)
    with pytest.raises(ConfigError, match=needle):
        SotazenConfig.from_dict(cfg)


def test_what_config_leaves_out_does_not_exist():
    from rustinfer_b200.config.sotazen_config import SotazenConfig
    c = SotazenConfig.from_dict(CONFIGS["B"])
    assert c.embedding_scale == 1.0 and c.postln_alpha == 1.0
    att = c.layers[2].mixer
    assert att.rot_dims == 0 and att.mask_size == 16 and att.softcap == 5.0
    a3 = SotazenConfig.from_dict(CONFIGS["A"]).layers[3].mixer
    assert a3.mask_size is None and a3.softcap is None and a3.rot_dims == 8
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    cfg["layers"][0]["mixer"]["taper"] = 3
    with pytest.warns(UserWarning, match="taper"):
        SotazenConfig.from_dict(cfg)


def test_random_weights_mode(tmp_path):
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.weights.random_init import write_random_model
    folder = write_random_model(str(tmp_path / "m"), CONFIGS["C"], seed=3, norm_std=0.1)
    cfg, w = P.read_model_folder(folder)
    assert {n: tuple(t.shape) for n, t in w.items()} == tensor_shapes("C")
    assert cfg["postln_alpha"] == 0.5 and cfg["layers"][1]["mlp"] is None
    logits = P.forward(cfg, w, [1, 5, 9, 96])
    assert logits.shape == (4, 97) and bool(torch.isfinite(logits).all())
