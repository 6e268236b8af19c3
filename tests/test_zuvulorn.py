"""Zuvulorn without a GPU: configuration and refusals, tensor names against a drawn model file, what each layer
keeps between steps and how the cache manager groups it, and properties of the plain mechanisms that the GPU
tests lean on."""

import copy
import math

import pytest
import torch

from zuvulorn_helpers import CONFIGS, ZP, attn, delta, draw_weights, experts, file_config, layer, model, rglru


def build(raw, shapes=None):
    from prism_b200.model_registry import build_model
    return build_model(copy.deepcopy(raw), shapes)


def test_the_registry_finds_the_design_and_every_tensor_has_a_taker():
    from prism_b200.model_registry import registered_architectures
    assert "Zuvulorn" in registered_architectures()
    for name, (raw, seed, _) in CONFIGS.items():
        w = draw_weights(raw, seed)
        cfg, mdl = build(file_config(raw), {k: tuple(v.shape) for k, v in w.items()})
        asked = {s.name: tuple(s.shape) for _, spec in mdl.named_params() for s in spec.sources if not spec.optional}
        assert asked == {k: tuple(v.shape) for k, v in w.items()}, name


def test_ranks_come_from_the_file_where_only_the_file_has_them():
    from prism_b200.config.model_config import ConfigError
    raw = file_config(CONFIGS["E"][0])
    with pytest.raises(ConfigError, match="decay_rank"):
        build(raw)
    cfg, _ = build(raw, {"l1.mix.a1": (9, 48), "l1.mix.g1": (2, 48)})
    assert (cfg.layers[1].mixer.decay_rank, cfg.layers[1].mixer.gate_rank) == (9, 2)
    with pytest.raises(ConfigError, match="l1.mix.g1"):
        build(raw, {"l1.mix.a1": (9, 48)})


@pytest.mark.parametrize("edit, text", [
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.update(streams=9), "streams"),
    (lambda r: r["layers"][0].update(type="conv"), "channel_delta"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "divisible"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda r: r["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=8), "layer 0"),
    (lambda r: r["layers"][3]["mixer"].update(blocks=3), "divisible"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=7), "top"),
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
    assert needs[0].kind == "paged" and (needs[0].num_kv_heads, needs[0].head_dim, needs[0].value_dim) == (2, 16, 24)
    assert needs[0].window is None and needs[0].chunk is None
    assert needs[2] is None                                    # reads layer 0's plane
    assert [n.state_shape for n in needs[1]] == [(4, 20, 12), (2, 2 * 2 * 12 + 4 * 20)]
    assert [n.state_shape for n in needs[3]] == [(40,), (3, 40)]
    groups, where = plan_groups(needs, [e.reads_cache_of for e in mdl.schedule])
    assert where[2] == (where[0][0], where[0][1], False)
    _, mdl = build(CONFIGS["E"][0])
    groups, _ = plan_groups(mdl.cache_needs(), [e.reads_cache_of for e in mdl.schedule])
    assert all(g.kind == "state" for g in groups)
    _, mdl = build(CONFIGS["C"][0])                             # one tap: a tail of no rows
    assert mdl.cache_needs()[1][1].state_shape == (0, 8)


def test_a_model_without_copies_has_no_connection_weights():
    _, mdl = build(CONFIGS["D"][0])
    names = [s.name for _, spec in mdl.named_params() for s in spec.sources]
    assert not [n for n in names if ".hc" in n]
    _, mdl = build(CONFIGS["C"][0])                             # one copy, but with weights
    assert "l0.hc1.mix" in [s.name for _, spec in mdl.named_params() for s in spec.sources]


def test_the_frequency_table_is_the_plain_one():
    from prism_b200.parts.positions import ScaledRotaryEmbedding
    for base, dims, sc in [(50.0, 8, (4.0, 1.0, 3.0, 64)), (30000.0, 64, None), (500000.0, 32, (8.0, 1.0, 4.0, 8192)),
                           (100.0, 6, (2.0, 0.5, 8.0, 16))]:
        part = ScaledRotaryEmbedding(dims, base, None if sc is None else dict(zip(("factor", "low", "high", "original"), sc)),
                                     interleaved=False)
        ref = ZP.band_frequencies(base, dims, None if sc is None else dict(zip(("factor", "low", "high", "original"), sc)),
                                  torch.float32)
        assert torch.allclose(part.frequencies(), ref, rtol=1e-6, atol=0)


def test_plain_sink_softmax_adds_one_to_the_denominator():
    s = torch.tensor([[0.3, -1.0, 2.0, float("-inf")], [-40.0, -50.0, -45.0, -60.0], [90.0, 10.0, 0.0, 3.0]])
    p = ZP.sink_softmax(s)
    e = torch.exp(s.double())
    assert torch.allclose(p.double(), e / (1.0 + e.sum(-1, keepdim=True)), atol=1e-7)
    assert float(p[1].sum()) < 1e-15 and abs(float(p[2].sum()) - 1.0) < 1e-6


def test_plain_prefix_property():
    """The plain model is causal: the logits of a prefix are those of the whole sequence (what lets the GPU
    tests compare any cutting of a prompt with one plain pass)."""
    raw, seed, _ = CONFIGS["A"]
    w = {k: v.double() for k, v in draw_weights(raw, seed).items()}
    seq = torch.randint(0, raw["vocab"], (30,), generator=torch.Generator().manual_seed(1)).tolist()
    full = ZP.forward(raw, w, seq)
    assert torch.allclose(ZP.forward(raw, w, seq[:17]), full[:17], atol=1e-9)


def test_plain_recurrences_against_closed_forms():
    # rglru with a constant decay: S_t = sum_j a^(t-j) b_j
    T, C = 9, 4
    g = torch.Generator().manual_seed(2)
    m = dict(width=C, blocks=2, conv=1)
    w = {"y": torch.zeros(C, 3), "y.b": torch.full((C,), 1.0), "x": torch.randn(C, 3, generator=g), "x.b": torch.zeros(C),
         "conv": torch.ones(C, 1), "conv.b": torch.zeros(C), "ra": torch.zeros(2, 2, 2), "ri": torch.zeros(2, 2, 2),
         "ra.b": torch.zeros(2, 2), "ri.b": torch.full((2, 2), 30.0), "lam": torch.zeros(C), "o": torch.eye(C)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, 3, generator=g).double()
    out = ZP.rglru(h, w, "", m)
    a = math.exp(-8.0 * 0.5 * math.log(2.0))
    u = h @ w["x"].T
    S, ref = torch.zeros(C).double(), []
    for t in range(T):
        S = a * S + math.sqrt(1 - a * a) * u[t]
        ref.append(S * ZP.gelu_tanh(torch.tensor(1.0).double()))
    assert torch.allclose(out, torch.stack(ref), atol=1e-9)


def test_plain_experts_with_every_expert_chosen_is_a_sum_over_all():
    g = torch.Generator().manual_seed(3)
    W, F, E = 6, 4, 3
    w = {"router": torch.randn(E, W, generator=g)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (torch.randn(F, W, generator=g), torch.randn(F, W, generator=g),
                                                         torch.randn(W, F, generator=g))
    h = torch.randn(5, W, generator=g)
    out = ZP.moe(h, w, "", experts(F, E, E))
    s = torch.sigmoid(h @ w["router"].T)
    ref = sum((ZP.silu((s[:, e:e + 1] * h) @ w[f"e{e}.gate"].T) * ((s[:, e:e + 1] * h) @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
              for e in range(E))
    assert torch.allclose(out, ref, atol=1e-5)
