"""The plain Linedra model against closed forms and hand-made cases, and what the package derives from a
config.json without a GPU: the typed configuration, the declared tensors, the cache layout, configuration
errors, the random-weights mode."""
import json
import math

import pytest
import torch

import plain_linedra as P
from linedra_helpers import CONFIGS, tensor_shapes

F64 = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# ------------------------------------------------------------------------ the plain model
def test_rotation_by_hand():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 7.0]]], dtype=F64).repeat(3, 1, 1)      # [T=3, 1, 6], dims 4
    y = P.rotate_half(x, torch.arange(3), 4, 100.0)
    assert torch.equal(y[0], x[0])                                                       # position 0: no turn
    for p in (1, 2):
        a0, a1 = p * 1.0, p * 100.0 ** (-2.0 / 4)                                        # pairs (0, 2) and (1, 3)
        want = [math.cos(a0), -2.0 * math.sin(a1), math.sin(a0), 2.0 * math.cos(a1), 5.0, 7.0]
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
    assert torch.allclose(P.softmax_with_sink(s, mask, torch.tensor([0.7, 30.7], dtype=F64)).flatten(),
                          torch.tensor([0.5, 1.0 / (1.0 + math.exp(30.0))], dtype=F64))
    assert torch.allclose(P.softmax_with_sink(s, mask, None), torch.ones(2, 1, 1, dtype=F64))


def test_causal_convolution_by_hand():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=F64)                                       # last column: the current token
    assert P.causal_conv(x, w).flatten().tolist() == [1.0, 12.0, 123.0, 1230.0]
    assert P.causal_conv(x, w[:, 2:], torch.tensor([0.5], dtype=F64)).flatten().tolist() == [1.5, 10.5, 100.5, 1000.5]


def test_distance_bias_and_head_gate():
    """With zero queries the scores are the bias alone: weights fall off by exp(-slope) a token, the sink counts
    once, and a head's output is scaled by the sigmoid of its own gate number."""
    T, H, d = 4, 2, 3
    m = {"heads": H, "kv_heads": 1, "dim": d, "vdim": d, "scale": 1.0}
    h = rnd(T, 5)
    eye = torch.eye(d, dtype=F64)
    w = {"q": torch.zeros(H * d, 5, dtype=F64), "k": rnd(d, 5, seed=1), "v": rnd(d, 5, seed=2),
         "sink": torch.tensor([0.0, -50.0], dtype=F64), "g": torch.zeros(H, 5, dtype=F64),
         "o": torch.cat([eye, torch.zeros(d, d, dtype=F64)], dim=1)}                     # reads head 0 only
    v = h @ w["v"].T
    s0 = 2.0 ** (-8.0 / H)
    assert torch.allclose(P.distance_slopes(H), torch.tensor([s0, 2.0 ** -8.0], dtype=F64))
    e = torch.tensor([math.exp(-s0 * k) for k in range(T)], dtype=F64)                  # weight of the key k tokens back
    want3 = sum(e[k] * v[3 - k] for k in range(T)) / (e.sum() + 1.0) * 0.5               # the sink's exp(0) = 1; gate 1/2
    out = P.biased_window_attention(h, w, m)
    assert torch.allclose(out[3], want3)
    w["o"] = torch.cat([torch.zeros(d, d, dtype=F64), eye], dim=1)                       # head 1: a negligible sink
    e1 = torch.tensor([math.exp(-(2.0 ** -8.0) * k) for k in range(T)], dtype=F64)
    assert torch.allclose(P.biased_window_attention(h, w, m)[3], sum(e1[k] * v[3 - k] for k in range(T)) / e1.sum() * 0.5)
    m["mask"] = {"size": 2}
    assert torch.allclose(P.biased_window_attention(h, w, m)[3], (e1[0] * v[3] + e1[1] * v[2]) / (e1[0] + e1[1]) * 0.5)


def test_recurrent_unit_closed_form():
    """With zero gate matrices r = sigmoid(ra.b), i = sigmoid(ri.b) are constants, so S_t is a geometric sum of u."""
    C, T, blocks = 4, 6, 2
    u = rnd(T, C)
    w = {"ra": torch.zeros(blocks, 2, 2, dtype=F64), "ri": torch.zeros(blocks, 2, 2, dtype=F64),
         "ra.b": rnd(blocks, 2, seed=1), "ri.b": rnd(blocks, 2, seed=2), "lam": rnd(C, seed=3)}
    a = torch.exp(-8.0 * torch.sigmoid(w["ra.b"].flatten()) * torch.log1p(torch.exp(w["lam"])))
    g = torch.sqrt(1 - a * a) * torch.sigmoid(w["ri.b"].flatten())
    want = sum(a ** (T - 1 - t) * g * u[t] for t in range(T))
    assert torch.allclose(P.gated_recurrent_unit(u, w, blocks)[-1], want)
    # a block's gates read only the block's own channels
    w["ra"] = rnd(blocks, 2, 2, seed=4)
    base = P.gated_recurrent_unit(u, w, blocks)
    u2 = u.clone()
    u2[:, 2:] += 1.0
    assert torch.allclose(P.gated_recurrent_unit(u2, w, blocks)[:, :2], base[:, :2])


def test_router_and_expert_by_hand():
    z = torch.tensor([[0.1, 2.0, -1.0, 2.0, 1.0]], dtype=F64)
    ids, wts = P.route(z, 3)
    assert ids.tolist() == [[1, 3, 4]]                                                   # the lower index among equals first
    e = torch.tensor([math.exp(2.0), math.exp(2.0), math.exp(1.0)], dtype=F64)
    assert torch.allclose(wts[0], e / e.sum())
    h = torch.tensor([1.0], dtype=F64)
    one = torch.ones(1, 1, dtype=F64)
    # gate 5 is cut to 2, up -7 to -2: 2 sigmoid(3.404) (-2 + 1)
    assert torch.allclose(P.expert(h, 5.0 * one, -7.0 * one, one, 2.0), torch.tensor([-2.0 / (1 + math.exp(-3.404))], dtype=F64))
    # a very negative gate is not cut from below
    assert torch.allclose(P.expert(h, -9.0 * one, 0.5 * one, one, 2.0), torch.tensor([-9.0 / (1 + math.exp(9 * 1.702)) * 1.5], dtype=F64))


def test_latent_attention_is_attention_over_made_keys():
    """One head, no rotated part, no sink to speak of, a gate of zeros: softmax attention with keys W_uk c and values
    W_uv c, halved by the gate."""
    T, d = 5, 8
    m = {"heads": 1, "dim": 4, "rot_dim": 0, "vdim": 3, "kv_rank": 6, "scale": 0.5}
    h = rnd(T, d)
    w = {"q": rnd(4, d, seed=1), "dkv": rnd(6, d, seed=2), "dkv.norm": rnd(6, seed=3), "uk": rnd(4, 6, seed=4),
         "uv": rnd(3, 6, seed=5), "sink": torch.tensor([-60.0], dtype=F64), "g": torch.zeros(3, d, dtype=F64),
         "o": torch.eye(3, dtype=F64)}
    c = P.rms_norm(h @ w["dkv"].T, w["dkv.norm"], 1e-6)
    s = ((h @ w["q"].T) @ (c @ w["uk"].T).T) * 0.5
    p = torch.softmax(s.masked_fill(~P.visible(T, None), -math.inf), dim=-1)
    assert torch.allclose(P.latent_attention(h, w, m, 1e-6), 0.5 * p @ (c @ w["uv"].T))


def test_layer_and_depth_average():
    """A model of one layer without a feed-forward, written out: norm, convolution, mixer, norm, residual factor,
    the average of the stem's output and the layer's result, the last norm, the capped logits."""
    cfg = {"width": 8, "vocab": 11, "norm": {"eps": 1e-3}, "canon": {"taps": 2}, "embedding": {"scale": 3.0},
           "residual_mult": 0.4, "logit_softcap": 2.0,
           "layers": [{"type": "latent_attention", "mlp": None, "mixer": {
               "heads": 2, "dim": 4, "rot_dim": 2, "vdim": 3, "kv_rank": 5, "q_rank": 6, "scale": 0.3, "rot": {"dims": 2, "base": 10.0}}}]}
    shapes = {"embed": (11, 8), "final.norm": (8,), "l0.norm1": (8,), "l0.norm1b": (8,), "l0.canon1": (8, 2), "l0.dwa": (2,),
              "l0.mix.dq": (6, 8), "l0.mix.dq.norm": (6,), "l0.mix.uq": (12, 6), "l0.mix.dkv": (7, 8), "l0.mix.dkv.norm": (5,),
              "l0.mix.uk": (8, 5), "l0.mix.uv": (6, 5), "l0.mix.sink": (2,), "l0.mix.g": (6, 8), "l0.mix.o": (8, 6)}
    w = {n: rnd(*s, seed=i) for i, (n, s) in enumerate(shapes.items())}
    ids = [3, 9, 0, 3]
    x0 = w["embed"][ids] * 3.0
    h = P.rms_norm(x0, None, 1e-3) * (1.0 + w["l0.norm1"])
    h = h + P.causal_conv(h, w["l0.canon1"])
    y = P.latent_attention(h, P.sub(w, "l0.mix."), cfg["layers"][0]["mixer"], 1e-3)
    x1 = x0 + 0.4 * P.rms_norm(y, None, 1e-3) * (1.0 + w["l0.norm1b"])
    avg = w["l0.dwa"][0] * x0 + w["l0.dwa"][1] * x1
    taps = []
    logits = P.forward(cfg, w, ids, taps)
    assert torch.allclose(taps[0], avg)
    z = (P.rms_norm(avg, None, 1e-3) * (1.0 + w["final.norm"])) @ w["embed"].T
    assert torch.allclose(logits, 2.0 * torch.tanh(z / 2.0))


# --------------------------------------------------------------------- configuration, registry
def test_registry_and_declared_tensors():
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    for name, cfg in CONFIGS.items():
        fam = resolve_architecture(cfg)
        assert fam.name == "linedra"
        typed = fam.parse_config(cfg, None)
        assert typed.to_dict() == cfg
        spec = fam.model_spec(typed)
        decls = Decoder(spec).param_decls()
        assert {n: tuple(d.shape) for n, d in decls.items() if not d.optional} == tensor_shapes(name)   # the tied head is optional
        assert [ls.arrangement for ls in spec.layers] == ["sandwich_depth_average"] * len(cfg["layers"])
        assert spec.depth_average


def test_cache_layout_of_mixed_layers():
    """Every layer keeps its input convolution's last inputs; a parallel layer also the attention's pages (a window's
    worth), the recurrent unit's convolution inputs and its state; a latent layer one row of kv_rank + rot_dim a
    token and no values."""
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.cache.manager import CacheLayout
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    from rustinfer_b200.parts.base import FixedState, PagedKV
    fam = resolve_architecture(CONFIGS["A"])
    dec = Decoder(fam.model_spec(fam.parse_config(CONFIGS["A"], None)))
    needs = [n for _, n, _ in dec.cache_needs()]
    assert needs[0] == (FixedState((2, 96)), PagedKV(2, 16, 20, value_dim=24), FixedState((1, 64)), FixedState((64,)))
    assert needs[1] == (FixedState((2, 96)), PagedKV(1, 48, None, value_dim=40, value_in_key=True))
    assert needs[2][1] == PagedKV(1, 8, None, value_dim=16) and needs[2][2:] == (FixedState((3, 48)), FixedState((48,)))
    layout = CacheLayout.from_needs(dec.cache_needs())
    assert len(layout.paged_groups()) == 3
    assert needs[0][1].first_key_kept(100) == 81 and needs[1][1].first_key_kept(100) == 0
    # an input convolution of one tap keeps nothing
    famc = resolve_architecture(CONFIGS["C"])
    decc = Decoder(famc.model_spec(famc.parse_config(CONFIGS["C"], None)))
    assert decc.cache_needs()[0][1][0] == FixedState((0, 64))


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].__setitem__("type", "gla"), "mixer type"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "feed-forward kind"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("blocks", 5), "blocks divide"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top <= experts"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 4), "rot.dims = rot_dim"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("rot_dim", 7), "rot"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("q_rank", 0), "q_rank"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("canon"), "canon"),
    (lambda c: c.__setitem__("logit_softcap", 0.0), "logit_softcap"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_configuration_errors(change, needle):
    from rustinfer_b200.config.linedra_config import LinedraConfig
    from rustinfer_b200.config.model_config import ConfigError
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    change(cfg)
    with pytest.raises(ConfigError, match=needle):
        LinedraConfig.from_dict(cfg)


def test_what_config_leaves_out_does_not_exist():
    from rustinfer_b200.config.linedra_config import LinedraConfig
    c = LinedraConfig.from_dict(CONFIGS["B"])
    assert c.embedding_scale == 1.0 and c.residual_mult == 1.0 and c.logit_softcap is None
    assert c.layers[0].mixer.q_rank is None and c.layers[1].mixer.left.mask_size == 16
    a = LinedraConfig.from_dict(CONFIGS["A"])
    assert a.layers[2].mixer.left.mask_size is None and a.layers[2].mlp is None and a.layers[1].mixer.q_rank == 24
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    cfg["layers"][0]["mixer"]["left"]["taper"] = 3
    with pytest.warns(UserWarning, match="taper"):
        LinedraConfig.from_dict(cfg)


def test_random_weights_mode(tmp_path):
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.weights.random_init import write_random_model
    folder = write_random_model(str(tmp_path / "m"), CONFIGS["C"], seed=3, norm_std=0.1)
    cfg, w = P.read_model_folder(folder)
    assert {n: tuple(t.shape) for n, t in w.items()} == tensor_shapes("C")
    assert cfg["residual_mult"] == 1.5 and cfg["layers"][1]["mlp"] is None
    assert abs(float(w["l1.dwa"][-1]) - 1.0) < 0.5 and abs(float(w["l1.dwa"][0])) < 0.5     # the newest result leads
    logits = P.forward(cfg, w, [1, 5, 9, 96])
    assert logits.shape == (4, 97) and bool(torch.isfinite(logits).all())
