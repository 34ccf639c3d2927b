"""Configuration of the Sebevik design, its plan and its tensor list, without a GPU; and the plain restatement against
itself (causality; the window's edge; the sink; the corrected, group-limited choice; pass-through router outputs; the
selective scan against its closed form)."""
import copy
import math

import pytest
import torch

import plain_sebevik as plain
from sebevik_cases import case

from esp_b200.config import config_from_dict, config_from_json
from esp_b200.config.sebevik import SebevikConfig
from esp_b200.errors import InvalidConfig, Unsupported
from esp_b200.weights.random_init import parameter_specs, write_model_folder


def test_registry_finds_the_design_by_its_architecture_string():
    cfg = config_from_dict(case("A"))
    assert isinstance(cfg, SebevikConfig)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_tensor_names_and_shapes_are_the_designs(name):
    raw = case(name)
    mine = {s.name: tuple(s.shape) for s in parameter_specs(config_from_dict(raw))}
    assert mine == plain.tensor_shapes(raw)


def test_plan_takes_every_size_and_constant_from_the_configuration():
    raw = case("A")
    plan = config_from_dict(raw).plan()
    assert plan.head_weight is None and plan.embed_weight == "embed" and plan.final_norm.kind == "rmsnorm_offset"
    scan, att, lat, att2, att3 = (b.mixer for b in plan.blocks)
    assert (scan.inner, scan.state, scan.dt_rank, scan.taps) == (80, 24, 5, 3)
    assert (att.num_heads, att.num_kv_heads, att.key_dim, att.value_dim, att.scale, att.window) == (6, 2, 40, 24, 0.21, 37)
    assert (att.position.rotary_dim, att.position.theta) == (16, 500.0) and att.eps == 1e-5
    # the first blending layer is marked; later ones blend; a layer that does not say so does neither
    assert (att.value_blend, att2.value_blend, att3.value_blend) == ("first", None, "blend")
    assert (lat.num_heads, lat.nope_dim, lat.value_dim, lat.kv_rank, lat.scale) == (3, 24, 40, 48, 0.19)
    assert lat.q_rank is None and lat.rot_dim == 0 and lat.position is None and lat.window is None and lat.head_gate
    moe = plan.blocks[1].ffn
    assert (moe.num_experts, moe.identity_experts, moe.top_k, moe.groups, moe.keep_groups) == (7, 2, 2, 3, 2)
    assert (moe.expert_intermediate, moe.shared_intermediate, moe.norm_topk) == (40, 56, False)
    assert plan.blocks[3].ffn.shared_intermediate is None and plan.blocks[3].ffn.groups == 0
    assert plan.blocks[2].ffn is None and plan.blocks[2].ffn_norm is None
    assert plan.blocks[0].ffn.kind == "relu2" and plan.blocks[0].ffn.intermediate == 72


def _set(path, value):
    def change(raw):
        d = raw
        for key in path[:-1]:
            d = d[key]
        if value is KeyError:
            del d[path[-1]]
        else:
            d[path[-1]] = value
    return change


@pytest.mark.parametrize("change, error", [
    (_set(("layers", 0, "type"), "mamba2"), Unsupported),
    (_set(("layers", 1, "mixer", "kv_heads"), 4), InvalidConfig),
    (_set(("layers", 1, "mixer", "rot", "dims"), 15), InvalidConfig),
    (_set(("layers", 1, "mixer", "rot", "dims"), 42), InvalidConfig),
    (_set(("layers", 1, "mixer", "mask", "size"), 0), InvalidConfig),
    (_set(("layers", 1, "mlp", "router", "groups", "count"), 2), InvalidConfig),        # nine outputs in two groups
    (_set(("layers", 1, "mlp", "router", "groups", "keep"), 4), InvalidConfig),
    (_set(("layers", 1, "mlp", "router", "top"), 10), InvalidConfig),
    (_set(("layers", 1, "mlp", "kind"), "glu"), Unsupported),
    (_set(("layers", 4, "mixer", "vdim"), 16), InvalidConfig),                           # blended values of another size
    (_set(("layers", 0, "mixer", "state"), 0), InvalidConfig),
    (_set(("norm", "eps"), 0.0), InvalidConfig),
    (_set(("layers", 2, "mixer", "kv_rank"), KeyError), InvalidConfig),
])
def test_refusals(change, error):
    raw = case("A")
    change(raw)
    with pytest.raises(error):
        config_from_dict(raw)


def test_kept_groups_must_hold_the_chosen_experts():
    raw = case("C")
    raw["layers"][0]["mlp"]["router"]["top"] = 5          # four groups of four outputs, one kept
    with pytest.raises(InvalidConfig):
        config_from_dict(raw)


def test_random_model_folder_round_trips(tmp_path):
    cfg = config_from_dict(case("C"))
    write_model_folder(cfg, 5, tmp_path)
    again = config_from_json(tmp_path)
    assert again.to_dict() == cfg.to_dict()
    from esp_b200.weights.loader import FolderSource
    src = FolderSource(tmp_path)
    assert {n: tuple(src.shape(n)) for n in src.names()} == plain.tensor_shapes(case("C"))


# ------------------------------------------------------------------------------------ the restatement against itself
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_restatement_is_causal_and_finite(name):
    raw = case(name)
    w = plain.random_weights(raw, 3)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, raw["vocab"], (90,), generator=g).tolist()
    full = plain.forward(raw, w, toks)
    assert torch.isfinite(full).all()
    other = list(toks)
    other[-1] = (other[-1] + 1) % raw["vocab"]
    moved = plain.forward(raw, w, other)
    assert torch.equal(full[:-1], moved[:-1]) and not torch.equal(full[-1], moved[-1])
    assert torch.allclose(plain.forward(raw, w, toks[:40]), full[:40], atol=1e-9)


def test_window_holds_the_query_and_its_predecessors():
    T, size = 12, 5
    h = torch.zeros(T, 8, dtype=torch.float64)
    mix = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 1.0, "mask": {"size": size}}
    w = {"q": torch.zeros(4, 8), "k": torch.zeros(4, 8), "v": torch.zeros(4, 8), "o": torch.eye(4).repeat(2, 1),
         "q.b": torch.ones(4), "k.b": torch.ones(4), "v.b": torch.zeros(4), "sink": torch.tensor([-1e9])}
    w = {k: v.double() for k, v in w.items()}
    # values: position t carries t in every channel, through the value projection of a one-hot input
    h[:, 0] = torch.arange(T, dtype=torch.float64)
    w["v"][:, 0] = 1.0
    y, _ = plain.window_sink_attention(h, w, "", mix, 1e-6, torch.arange(T), None)
    for t in range(T):
        seen = range(max(0, t - size + 1), t + 1)
        assert abs(float(y[t, 0]) - sum(seen) / len(seen)) < 1e-9        # equal scores: the mean over the visible keys


def test_sink_counts_once_and_is_not_scaled():
    scores = torch.zeros(2, 1, 3, dtype=torch.float64)
    p = plain.causal_softmax_rows(scores, torch.ones(1, 3, dtype=torch.bool), extra=torch.tensor([0.0, math.log(3.0)], dtype=torch.float64))
    assert torch.allclose(p[0].sum(), torch.tensor(3 / 4, dtype=torch.float64))
    assert torch.allclose(p[1].sum(), torch.tensor(3 / 6, dtype=torch.float64))


def test_choice_uses_the_correction_and_the_weights_do_not():
    D = 6
    w = {"router": torch.zeros(4, D, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 0.0, 0.5], dtype=torch.float64)}
    w["router"][:, 0] = torch.tensor([3.0, 2.0, 1.0, 0.0])
    h = torch.zeros(1, D, dtype=torch.float64)
    h[0, 0] = 1.0
    ids, wts, s = plain.route(h, w, "", {"experts": 4, "top": 2})
    assert sorted(ids[0].tolist()) == [0, 3]                      # the last output wins through its correction alone
    assert torch.allclose(wts[0].sort().values, torch.stack([s[0, 3], s[0, 0]]))
    assert float(wts.sum()) < 1.0                                 # not renormalised


def test_groups_shut_out_better_experts_of_other_groups_also_with_negative_scores():
    D = 4
    w = {"router": torch.zeros(6, D, dtype=torch.float64), "correction": torch.full((6,), -2.0, dtype=torch.float64)}
    w["router"][:, 0] = torch.tensor([5.0, 0.0, 4.9, 4.8, 0.0, 0.0])          # groups {0, 1}, {2, 3}, {4, 5}
    h = torch.zeros(1, D, dtype=torch.float64)
    h[0, 0] = 1.0
    ids, _, _ = plain.route(h, w, "", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert sorted(ids[0].tolist()) == [0, 1]                      # every corrected score is negative; 2 and 3 are still out


def test_pass_through_outputs_return_the_input_times_the_score():
    raw = {"router": {"experts": 1, "top": 1, "identity": 1}, "expert": {"ff": 2}}
    D = 3
    w = {"router": torch.tensor([[0.0] * D, [9.0] * D], dtype=torch.float64), "correction": torch.zeros(2, dtype=torch.float64),
         "e0.gate": torch.ones(2, D, dtype=torch.float64), "e0.up": torch.ones(2, D, dtype=torch.float64),
         "e0.down": torch.ones(D, 2, dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float64)
    y = plain.moe_ffn(h, w, "", raw)
    s = torch.softmax(h @ w["router"].T, -1)[0, 1]
    assert torch.allclose(y, s * h)


def test_selective_scan_with_constant_inputs_has_a_closed_form():
    T, C, N = 9, 2, 3
    x = torch.full((T, C), 0.7, dtype=torch.float64)
    dt = torch.full((T, C), 0.3, dtype=torch.float64)
    A = -torch.rand(C, N, dtype=torch.float64, generator=torch.Generator().manual_seed(0)) - 0.1
    B = torch.ones(T, N, dtype=torch.float64)
    Cm = torch.ones(T, N, dtype=torch.float64)
    y = plain.selective_scan(x, dt, A, B, Cm, torch.zeros(C, dtype=torch.float64))
    a = torch.exp(0.3 * A)
    want = (0.3 * 0.7 * (1 - a ** T) / (1 - a)).sum(-1)           # a geometric series per state entry
    assert torch.allclose(y[-1], want)


def test_rotation_pairs_neighbours_and_leaves_the_rest():
    x = torch.arange(8, dtype=torch.float64).view(1, 1, 8) + 1
    y = plain.rotate_neighbours(x, torch.tensor([3]), 4, 10.0)
    assert torch.equal(y[..., 4:], x[..., 4:])
    for i in range(2):
        a = 3 * 10.0 ** (-2.0 * i / 4)
        u, v = float(x[0, 0, 2 * i]), float(x[0, 0, 2 * i + 1])
        assert abs(float(y[0, 0, 2 * i]) - (u * math.cos(a) - v * math.sin(a))) < 1e-12
        assert abs(float(y[0, 0, 2 * i + 1]) - (v * math.cos(a) + u * math.sin(a))) < 1e-12
