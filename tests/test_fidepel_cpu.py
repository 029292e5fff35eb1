"""Fidepel without a GPU: the configuration reader, the spec and its schedule, the tensor list, and the oracle
against itself (windows, rotation, routing)."""
import copy

import pytest
import torch

import plain_fidepel as plain
from fidepel_util import CFG_A, CFG_B, CFG_C, CONFIGS, attn, config, doubles, moe, prompts, random_weights, write_folder
from trapetum_b200.config import ConfigError, load_config
from trapetum_b200.engine.model import tensor_specs_for_config

F = torch.float64


def test_every_size_and_constant_is_read_by_key():
    cfg, spec = load_config(copy.deepcopy(CFG_A))
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.residual_mult) == (150, 48, 1e-5, 1.0)
    assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 2, 3)
    a = cfg.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.rot_dims, a.rot_base, a.rot_factor) == \
        (3, 3, 8, 12, 0.4, 5, 4, 100.0, 1.0)
    b = cfg.layers[1].mixer
    assert (b.heads, b.kv_heads, b.window, b.rot_dims, b.rot_factor) == (2, 1, 33, 16, 8.0)
    m = cfg.layers[1].mlp
    assert (m.experts, m.top, m.ff, m.scale, m.groups, m.keep, m.shared_ff) == (6, 3, 16, 1.5, 3, 2, 40)
    m0 = cfg.layers[0].mlp
    assert (m0.scale, m0.groups, m0.keep, m0.shared_ff) == (1.0, 1, 1, None) and cfg.layers[2].mlp is None
    assert all(l.block.kind == "parallel" and l.mixer.kind == "attention" for l in spec.layers)
    assert [l.feed_forward.kind for l in spec.layers] == ["routed_experts", "routed_experts", "none"]
    assert spec.layers[0].block.params["scale"] == 1.0 and spec.final_norm.params["scalar"]
    p = spec.layers[1].mixer.params
    assert p["position"].params["scaling_factor"] == 8.0 and p["window"] == 33 and p["value_dim"] == 16
    f = spec.layers[1].feed_forward.params
    assert (f["score"], f["gated"], f["activation"], f["route_scale"], f["weight_eps"]) == ("softmax", False, "relu2", 1.5, 1e-20)
    cb, spec_b = load_config(copy.deepcopy(CFG_B))
    assert cb.loop is None and cb.residual_mult == 0.7
    assert cb.layers[0].mixer.window is None and cb.layers[0].mixer.rot_dims == 0
    assert spec_b.layers[0].mixer.params["position"].kind == "none" and spec_b.layers[0].mixer.params["window"] is None
    assert spec_b.layers[1].feed_forward.params["shared"] is None


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_schedule_names_every_layer_run(name):
    cfg = CONFIGS[name]
    _, spec = load_config(copy.deepcopy(cfg))
    assert [e.layer for e in spec.schedule] == plain.schedule(cfg)
    assert all(e.cache_of is None and e.before is None for e in spec.schedule)      # every pass has a cache of its own
    lp = cfg.get("loop")
    n = len(cfg["layers"])
    assert len(spec.schedule) == n + ((lp["stop"] - lp["start"]) * (lp["times"] - 1) if lp else 0)


@pytest.mark.parametrize("path, value, word", [
    (("layers", 1, "type"), "rwkv", "type"),
    (("layers", 0, "mixer", "heads"), None, "layers[0].mixer.heads"),
    (("layers", 0, "mixer", "scale"), None, "mixer.scale"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "rot.dims"),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0, "factor"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mlp", "kind"), "dense", "mlp.kind"),
    (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 5, "groups"),
    (("layers", 0, "mlp", "expert"), None, "mlp.expert"),
    (("loop", "stop"), 7, "loop"),
    (("loop", "times"), 0, "loop"),
    (("norm",), None, "norm"),
    (("vocab",), "many", "vocab"),
])
def test_errors_name_the_key(path, value, word):
    c = copy.deepcopy(CFG_A)
    d = c
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        load_config(c)
    assert word in str(e.value)


def test_kept_groups_must_hold_enough_experts():
    c = copy.deepcopy(CFG_A)
    c["layers"][1]["mlp"]["router"].update(top=3, groups={"count": 3, "keep": 1})
    with pytest.raises(ConfigError):
        load_config(c)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_tensor_list_is_the_files(name):
    cfg = CONFIGS[name]
    w = random_weights(cfg, 1)
    specs = tensor_specs_for_config(copy.deepcopy(cfg))
    assert set(specs) == set(w)
    assert all(tuple(s.shape) == tuple(w[k].shape) for k, s in specs.items())
    assert specs["l0.norm1"].shape == () and specs["final.norm"].shape == ()


def test_wrong_and_missing_tensors_are_reported(tmp_path):
    from trapetum_b200.weights.loader import WeightError, load_tensors
    cfg = CFG_B
    w = random_weights(cfg, 3)
    specs = tensor_specs_for_config(copy.deepcopy(cfg))
    got = load_tensors(write_folder(str(tmp_path / "ok"), cfg, w), specs, torch.float32, "cpu")
    assert got["l1.norm1"].dim() == 0 and got["l0.mix.temp"].shape == (4,)
    bad = dict(w)
    bad["l0.mix.g"] = w["l0.mix.g"][:-1].contiguous()
    del bad["l2.mlp.shared.up"]
    with pytest.raises(WeightError) as e:
        load_tensors(write_folder(str(tmp_path / "bad"), cfg, bad), specs, torch.float32, "cpu")
    assert "l0.mix.g" in str(e.value) and "l2.mlp.shared.up" in str(e.value)


# ---------------------------------------------------------------------------------------------------------------
# the oracle against itself
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_agrees_with_itself_step_by_step(name):
    cfg = CONFIGS[name]
    w = doubles(random_weights(cfg, 2))
    ids = prompts(cfg["vocab"], [80 if name == "C" else 23], seed=1)[0]
    whole = plain.forward(cfg, w, ids)
    for first in (1, 2, 9):
        assert torch.allclose(plain.forward_stepwise(cfg, w, ids, first), whole, atol=1e-9, rtol=1e-9)


def test_a_window_counts_the_query_itself():
    q, k = torch.arange(6), torch.arange(6)
    v = plain.visible(q, k, 3)
    assert v[5].tolist() == [False, False, False, True, True, True]
    assert v[1].tolist() == [True, True, False, False, False, False]
    assert plain.visible(q, k, 1).int().tolist() == torch.eye(6, dtype=torch.int32).tolist()
    assert plain.visible(q, k, None)[5].all()


def test_rotation_pairs_the_halves_of_the_rotated_part_and_scales_positions():
    x = torch.zeros(1, 1, 6, dtype=F)
    x[0, 0, 0], x[0, 0, 5] = 1.0, 7.0
    pos = torch.tensor([3])
    y = plain.rotate_half(x, pos, 4, 100.0, 2.0)
    a = 3.0 / 2.0                                     # frequency 0 is 1, divided by the factor
    assert torch.allclose(y[0, 0], torch.tensor([torch.cos(torch.tensor(a)), 0, torch.sin(torch.tensor(a)), 0, 0, 7.0], dtype=F))
    # scores depend on the distance only
    g = torch.Generator().manual_seed(0)
    u, v = torch.randn(1, 1, 8, generator=g, dtype=F), torch.randn(1, 1, 8, generator=g, dtype=F)
    s = [float((plain.rotate_half(u, torch.tensor([p + 4]), 8, 50.0, 3.0) * plain.rotate_half(v, torch.tensor([p]), 8, 50.0, 3.0)).sum())
         for p in (0, 11, 300)]
    assert abs(s[0] - s[1]) < 1e-9 and abs(s[0] - s[2]) < 1e-9


def test_routing_in_the_plain_implementation():
    """A group that is not kept is out although it holds the second largest score of all."""
    z = torch.tensor([[2.0, 0.0, 1.9, 1.8, 0.1, 0.2]], dtype=F)
    t = {"router": torch.eye(6, dtype=F)}
    r = {"experts": 6, "top": 2, "scale": 2.5, "groups": {"count": 3, "keep": 1}}
    idx, wt = plain.route(z, r, t, "")
    assert sorted(idx[0].tolist()) == [0, 1]                  # group maxima: 2.0, 1.9, 0.2
    assert torch.allclose(wt.sum(-1), torch.tensor([2.5], dtype=F))
    s = torch.softmax(z, -1)[0]
    assert torch.allclose(wt[0].sort().values, (s[[1, 0]] / (s[0] + s[1]) * 2.5))
    r["groups"]["keep"] = 2
    assert sorted(plain.route(z, r, t, "")[0][0].tolist()) == [0, 2]
    del r["groups"]
    assert sorted(plain.route(z, r, t, "")[0][0].tolist()) == [0, 2]
    r["top"] = 6
    assert torch.allclose(plain.route(z, r, t, "")[1].sum(-1), torch.tensor([2.5], dtype=F))


def test_the_expert_squares_what_relu_lets_through():
    up, down = torch.tensor([[1.0], [-1.0]], dtype=F), torch.tensor([[1.0, 10.0]], dtype=F)
    assert plain.expert(torch.tensor([[3.0]], dtype=F), up, down).item() == 9.0
    assert plain.expert(torch.tensor([[-2.0]], dtype=F), up, down).item() == 40.0


def test_layers_outside_the_window_do_not_see_a_token():
    """One layer, a window of four: changing token 2 changes the logits of positions 2..5 and of no other."""
    cfg = config(40, 32, [(attn(2, 1, 8, 8, 0.5, window=4, rot=(8, 100.0)), moe(4, 2, 8, shared=8))])
    w = doubles(random_weights(cfg, 4))
    ids = prompts(40, [12], seed=2)[0]
    other = list(ids)
    other[2] = (ids[2] + 1) % 40
    d = (plain.forward(cfg, w, ids) - plain.forward(cfg, w, other)).abs().amax(-1)
    assert (d[:2] == 0).all() and (d[6:] == 0).all() and (d[2:6] > 1e-6).all()
