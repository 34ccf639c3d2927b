"""Configuration of the Migosun design, its plan and its tensor list, without a GPU; and the plain restatement against
itself (causality; the chunked mask; the learned sink; the delta rule against its closed form for one key)."""
import copy
import math

import pytest
import torch

import plain_migosun as plain
from migosun_cases import case

from esp_b200.config import config_from_dict, config_from_json
from esp_b200.config.migosun import MigosunConfig
from esp_b200.errors import InvalidConfig, Unsupported
from esp_b200.weights.random_init import parameter_specs, write_model_folder


def with_ranks(name):
    raw, (decay_rank, gate_rank) = case(name)
    raw["ranks"] = {}
    for i, layer in enumerate(raw["layers"]):
        raw["ranks"][f"{i}:a1"] = decay_rank
        if layer["type"] == "parallel":
            raw["ranks"][f"{i}:g1"] = gate_rank
    return raw, (decay_rank, gate_rank)


def test_registry_finds_the_design_by_its_architecture_string():
    raw, _ = with_ranks("A")
    cfg = config_from_dict(raw)
    assert isinstance(cfg, MigosunConfig)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_tensor_names_and_shapes_are_the_designs(name):
    raw, ranks = with_ranks(name)
    mine = {s.name: tuple(s.shape) for s in parameter_specs(config_from_dict(raw))}
    plain_raw, _ = case(name)
    assert mine == plain.tensor_shapes(plain_raw, *ranks)


def test_inner_widths_come_from_the_tensors():
    raw, _ = case("A")
    cfg = config_from_dict(raw)
    shapes = plain.tensor_shapes(raw, 12, 20)
    cfg.bind_shapes(shapes)
    plan = cfg.plan()
    gla, par = plan.blocks[0].mixer, plan.blocks[1].mixer
    assert gla.decay_rank == 12
    assert (par.branches[1].decay_rank, par.branches[1].gate_rank) == (12, 20)
    assert {s.name: tuple(s.shape) for s in parameter_specs(cfg)} == shapes


def test_plan_takes_every_size_and_constant_from_the_configuration():
    raw, _ = case("A")
    plan = config_from_dict(raw).plan()
    assert plan.embed_scale == 1.7 and plan.head_weight is None and plan.embed_weight == "embed"
    gla, par, par2, gla2 = (b.mixer for b in plan.blocks)
    assert (gla.num_heads, gla.key_dim, gla.value_dim, gla.tau) == (3, 24, 40, 4.0)
    left, right = par.branches
    assert par.scales == (0.7, 1.3)
    assert (left.num_heads, left.num_kv_heads, left.key_dim, left.value_dim, left.scale) == (6, 2, 40, 24, 0.2)
    assert (left.position.rotary_dim, left.position.theta, left.chunk) == (16, 500.0, 37)
    assert (right.num_heads, right.num_kv_heads, right.key_dim, right.value_dim, right.taps) == (4, 2, 24, 40, 4)
    assert par2.branches[0].chunk == 70 and par2.branches[1].taps == 2
    assert gla2.tau == 1.0
    assert all(b.streams == 2 for b in plan.blocks)
    assert plan.blocks[1].ffn is None and plan.blocks[1].ffn_norm is None
    ffn = plan.blocks[2].ffn
    assert (ffn.intermediate, ffn.limit, ffn.alpha, ffn.up_shift) == (136, 0.8, 1.702, 1.0)
    assert all(b.mixer_norm.eps == 1e-5 for b in plan.blocks)
    b = config_from_dict(case("B")[0]).plan()
    assert b.blocks[0].streams == 1 and b.blocks[0].mixer.branches[0].chunk == 1


@pytest.mark.parametrize("change, error", [
    (lambda c: c["layers"][0].update(type="conv"), Unsupported),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4), InvalidConfig),
    (lambda c: c["layers"][1]["mixer"]["right"].update(kv_heads=3), InvalidConfig),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), InvalidConfig),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=48), InvalidConfig),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), InvalidConfig),
    (lambda c: c["layers"][1]["mixer"].pop("right_scale"), InvalidConfig),
    (lambda c: c["layers"][0]["mixer"].update(tau=0), InvalidConfig),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), Unsupported),
    (lambda c: c["layers"][0]["mlp"].update(limit=0), InvalidConfig),
    (lambda c: c["norm"].update(eps=0), InvalidConfig),
    (lambda c: c.update(layers=[]), InvalidConfig),
])
def test_refusals(change, error):
    raw, _ = case("A")
    change(raw)
    with pytest.raises(error):
        config_from_dict(raw)


def test_random_model_folder_round_trips(tmp_path):
    raw, ranks = with_ranks("C")
    cfg = config_from_dict(raw)
    write_model_folder(cfg, 5, tmp_path)
    again = config_from_json(tmp_path)
    assert again.to_dict() == cfg.to_dict()
    from esp_b200.weights.loader import FolderSource
    src = FolderSource(tmp_path)
    assert {n: tuple(src.shape(n)) for n in src.names()} == plain.tensor_shapes(case("C")[0], *ranks)


# ------------------------------------------------------------------------------------ the restatement against itself
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_restatement_is_causal_and_finite(name):
    raw, ranks = case(name)
    w = plain.random_weights(raw, 11, *ranks)
    toks = [int(t) for t in torch.randint(0, raw["vocab"], (90,), generator=torch.Generator().manual_seed(1))]
    a = plain.forward(raw, w, toks)
    b = plain.forward(raw, w, toks + [3])
    assert torch.isfinite(a).all() and torch.allclose(a, b[:-1], atol=1e-10)


def test_chunks_are_counted_from_the_sequences_start():
    pos = torch.arange(10)
    vis = plain.chunk_visible(pos, pos, 4)
    assert vis[3].tolist() == [True, True, True, True] + [False] * 6
    assert vis[4].tolist() == [False] * 4 + [True] + [False] * 5
    assert vis[9].tolist() == [False] * 8 + [True, True]
    # a portion that starts at position 6 sees position 4 (its own chunk) and not position 3
    part = plain.chunk_visible(pos[6:], pos, 4)
    assert part[0].tolist() == [False] * 4 + [True, True, True] + [False] * 3


def test_sink_counts_once_and_is_not_scaled():
    q, k = torch.ones(1, 2, 4, dtype=torch.float64), torch.ones(3, 1, 4, dtype=torch.float64)
    v = torch.full((3, 1, 2), 5.0, dtype=torch.float64)
    sink = torch.tensor([0.3, -50.0], dtype=torch.float64)
    out = plain.attend_learned_sink(q, k, v, 0.1, torch.ones(1, 3, dtype=torch.bool), sink)
    assert abs(float(out[0, 0, 0]) - 5.0 * 3 * math.exp(0.4) / (3 * math.exp(0.4) + math.exp(0.3))) < 1e-12
    assert abs(float(out[0, 1, 0]) - 5.0) < 1e-12


def test_delta_rule_with_one_key_moves_the_stored_value_towards_the_new_one():
    T, K, V = 6, 4, 3
    k = torch.zeros(T, 1, K, dtype=torch.float64)
    k[:, 0, 2] = 1.0
    v = torch.randn(T, 1, V, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    beta = torch.full((T, 1), 0.25, dtype=torch.float64)
    decay = torch.full((T, 1, K), 0.5, dtype=torch.float64)
    o, S = plain.delta_rule(k, k, v, decay, beta, torch.zeros(1, K, V, dtype=torch.float64))
    stored = torch.zeros(V, dtype=torch.float64)
    for t in range(T):
        stored = 0.5 * stored
        stored = stored + 0.25 * (v[t, 0] - stored)
        assert torch.allclose(o[t, 0], stored, atol=1e-12)
    assert torch.allclose(S[0, 2], stored) and float(S[0, [0, 1, 3]].abs().max()) == 0


def test_rotation_leaves_the_channels_behind_the_rotated_ones():
    x = torch.randn(5, 2, 12, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    pos = torch.tensor([0, 1, 2, 50, 1000])
    y = plain.rotate_half_layout(x, pos, 6, 100.0)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    a = 50 * 100.0 ** (-2.0 / 6)                       # pair (1, 4) at position 50
    assert abs(float(y[3, 0, 1]) - float(x[3, 0, 1] * math.cos(a) - x[3, 0, 4] * math.sin(a))) < 1e-12
    assert abs(float(y[3, 0, 4]) - float(x[3, 0, 4] * math.cos(a) + x[3, 0, 1] * math.sin(a))) < 1e-12
