"""Tagelorn without a GPU: configuration and refusals, tensor names against a drawn model file, what each layer
keeps between steps and how the cache manager groups it, and properties of the plain mechanisms that the GPU
tests lean on."""

import copy
import math

import pytest
import torch

from tagelorn_helpers import CONFIGS, TP, attn, delta, dense, draw_weights, file_config, layer, model, moe


def build(raw, shapes=None):
    from prism_b200.model_registry import build_model
    return build_model(copy.deepcopy(raw), shapes)


def test_the_registry_finds_the_design_and_every_tensor_has_a_taker():
    from prism_b200.model_registry import registered_architectures
    assert "Tagelorn" in registered_architectures()
    for name, (raw, seed, _) in CONFIGS.items():
        w = draw_weights(raw, seed)
        cfg, mdl = build(file_config(raw), {k: tuple(v.shape) for k, v in w.items()})
        asked = {s.name: tuple(s.shape) for _, spec in mdl.named_params() for s in spec.sources if not spec.optional}
        assert asked == {k: tuple(v.shape) for k, v in w.items()}, name


def test_sizes_come_from_the_file_where_only_the_file_has_them():
    from prism_b200.config.model_config import ConfigError
    raw = file_config(CONFIGS["A"][0])
    with pytest.raises(ConfigError, match="bias_rows"):
        build(raw)
    shapes = {"l0.mix.rel": (14, 6), "l2.mix.rel": (4, 4), "l1.mix.w1": (9, 72), "l3.mix.w1": (2, 72)}
    cfg, _ = build(raw, shapes)
    assert (cfg.layers[0].mixer.bias_rows, cfg.layers[2].mixer.bias_rows) == (14, 4)
    assert (cfg.layers[1].mixer.decay_rank, cfg.layers[3].mixer.decay_rank) == (9, 2)
    del shapes["l3.mix.w1"]
    with pytest.raises(ConfigError, match="l3.mix.w1"):
        build(raw, shapes)


@pytest.mark.parametrize("edit, text", [
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["canon"].update(taps=0), "taps"),
    (lambda r: r.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda r: r["layers"][0].update(type="conv"), "general_delta"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "divisible"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda r: r["layers"][1]["mixer"].pop("dim"), "dim"),
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "dense"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda r: r["token_side"].update(dim=0), "dim"),
])
def test_refusals_name_the_key(edit, text):
    from prism_b200.config.model_config import ConfigError
    raw = copy.deepcopy(CONFIGS["A"][0])
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        build(raw)


def test_what_the_layers_keep_between_steps():
    from prism_b200.cache.manager import plan_groups
    _, mdl = build(CONFIGS["A"][0])
    needs = mdl.cache_needs()
    a, tail = needs[0]
    assert a.kind == "paged" and (a.num_kv_heads, a.head_dim, a.value_dim, a.window, a.keep_first) == (2, 12, 20, 9, 2)
    assert tail.kind == "state" and tail.state_shape == (1, 72)              # two taps: one row of the normed input
    assert [n.state_shape for n in needs[1]] == [(3, 7, 7), (1, 72)]
    assert needs[2][0].window == 40 and needs[2][0].keep_first == 0
    groups, where = plan_groups(needs, [e.reads_cache_of for e in mdl.schedule])
    tails = {w[-1][0] for w in where}
    assert len(tails) == 1 and groups[tails.pop()].num_planes == 4            # every layer's tail in one state group
    _, mdl = build(CONFIGS["D"][0])
    groups, _ = plan_groups(mdl.cache_needs(), [e.reads_cache_of for e in mdl.schedule])
    assert all(g.kind == "state" for g in groups)
    _, mdl = build(CONFIGS["C"][0])                                          # one tap: no tail at all
    needs = mdl.cache_needs()
    assert needs[0].kind == "paged" and needs[1].state_shape == (1, 1, 1)


def test_options_that_a_file_leaves_out():
    raw = model(40, 16, [layer("general_delta", delta(2, 4, 3), None)], taps=2)
    cfg, mdl = build(raw)
    assert cfg.side_dim is None and cfg.logit_softcap is None
    names = [s.name for _, spec in mdl.named_params() for s in spec.sources]
    assert not [n for n in names if "side" in n or "norm2" in n or "mlp" in n]
    raw.pop("canon")
    names = [s.name for _, spec in build(raw)[1].named_params() for s in spec.sources]
    assert not [n for n in names if "canon" in n] and len(build(raw)[1].cache_needs()[0].state_shape) == 3
    raw = model(40, 16, [layer("attention", attn(2, 1, 4), None)])
    for key in ("mask", "bias_max", "bias_rows"):
        raw["layers"][0]["mixer"].pop(key)
    cfg, mdl = build(raw)                                   # no mask: causal; no bias_max: no table of distances
    assert cfg.layers[0].mixer.window is None and cfg.layers[0].mixer.bias_max is None
    assert "l0.mix.rel" not in [s.name for _, spec in mdl.named_params() for s in spec.sources]
    raw = model(40, 16, [layer("attention", attn(2, 1, 4), moe(8, 4, 2))], taps=2, side=3)
    names = [s.name for _, spec in build(raw)[1].named_params() for s in spec.sources]
    assert "side.embed" in names and "l0.side.proj" in names and "l0.mlp.correction" in names
    assert not [n for n in names if "shared" in n or n.endswith("mlp.e0.gate")]


def test_distance_rows():
    from prism_b200.parts.attention import distance_bucket
    for rows, far in [(24, 200), (10, 30), (6, 11), (16, 64), (64, 512), (2, 3), (1, 1), (8, 4)]:
        got = [distance_bucket(n, rows, far) for n in range(3 * far + 5)]
        assert got == [TP.distance_bucket(n, rows, far) for n in range(3 * far + 5)]
        assert got[:rows // 2] == list(range(rows // 2))                      # a row each below half the table
        assert all(b >= a for a, b in zip(got, got[1:])) and max(got) == rows - 1
        assert all(g == rows - 1 for g in got[far:])
    # where the logarithms' quotient is a whole number in exact arithmetic the distance opens its row
    assert distance_bucket(64, 64, 512) == 32 + 8 and distance_bucket(63, 64, 512) == 32 + 7
    assert distance_bucket(128, 64, 512) == 32 + 16 and distance_bucket(256, 64, 512) == 32 + 24


def test_plain_prefix_property():
    """The plain model is causal: the logits of a prefix are those of the whole sequence (what lets the GPU tests
    compare any cutting of a prompt with one plain pass)."""
    raw, seed, _ = CONFIGS["A"]
    w = {k: v.double() for k, v in draw_weights(raw, seed).items()}
    seq = torch.randint(0, raw["vocab"], (30,), generator=torch.Generator().manual_seed(1)).tolist()
    full = TP.forward(raw, w, seq)
    assert torch.allclose(TP.forward(raw, w, seq[:17]), full[:17], atol=1e-9)


def test_plain_window_keeps_the_first_positions():
    assert [j for j in range(12) if TP.visible(11, j, 4, 2)] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(3) if TP.visible(2, j, 4, 2)] == [0, 1, 2]
    assert [j for j in range(12) if TP.visible(11, j, 1, 0)] == [11]


def test_plain_generalized_delta_rule_against_closed_forms():
    """Without removal and with a constant decay the state is a decayed sum of outer products."""
    g = torch.Generator().manual_seed(2)
    T, W, d = 7, 5, 4
    h = torch.randn(T, W, generator=g).double()
    w = {n: torch.randn(d, W, generator=g).double() for n in ("r", "k", "v", "g")}
    w.update({"a": torch.zeros(d, W).double(), "a.b": torch.full((d,), -60.0).double(), "w1": torch.zeros(1, W).double(),
              "w2": torch.zeros(d, 1).double(), "w0": torch.zeros(d).double(), "norm": torch.ones(d).double(),
              "o": torch.eye(d).double()})
    out = TP.general_delta(h, w, "", dict(heads=1, dim=d), 1e-5)
    decay = math.exp(-math.exp(-0.5) * 0.5)
    r, k, v = h @ w["r"].T, h @ w["k"].T, h @ w["v"].T
    S, ref = torch.zeros(d, d).double(), []
    for t in range(T):
        S = decay * S + k[t][:, None] * v[t][None, :]
        ref.append(TP.rms((S.T @ r[t])[None], 1e-5)[0] * torch.sigmoid(h[t] @ w["g"].T))
    assert torch.allclose(out, torch.stack(ref), atol=1e-9)


def test_plain_routing_keeps_the_best_groups_and_weighs_without_the_correction():
    z = torch.tensor([2.0, 0.1, 0.0, 1.9, -1.0, 1.5]).double()
    s = torch.softmax(z, -1)
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.9, 0.0]).double()
    chosen, weights = TP.route(z, corr, 2, 3, 2, 2.0)
    # groups (0,1) (2,3) (4,5): with the correction expert 4 leads its group, and groups 2 and 0 are kept
    assert sorted(chosen) == [0, 4]
    total = s[0] + s[4]
    assert abs(float(sum(weights)) - 2.0) < 1e-12 and abs(float(weights[chosen.index(4)]) - 2.0 * float(s[4] / total)) < 1e-12
    chosen, _ = TP.route(z, torch.zeros(6).double(), 2, 3, 1, 1.0)
    assert sorted(chosen) == [0, 1]                            # one group kept: both choices from the best group


def test_random_weights_mode_writes_every_tensor(tmp_path):
    from prism_b200.weights.loader import read_safetensors_header
    from prism_b200.weights.random_init import write_model_folder
    raw = copy.deepcopy(CONFIGS["A"][0])                       # keeps bias_rows and decay_rank: there is no file to ask
    write_model_folder(raw, 3, str(tmp_path))
    header = read_safetensors_header(str(tmp_path / "model.safetensors"))
    w = draw_weights(CONFIGS["A"][0], 1)
    assert {k: v[0] for k, v in header.items()} == {k: tuple(v.shape) for k, v in w.items()}
