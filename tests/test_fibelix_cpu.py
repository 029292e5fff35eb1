"""Fibelix without a GPU: the configuration reader, the spec, the tensor names, the frequencies' table, the blocks of
a step, and the plain implementation against itself."""
import copy

import pytest
import torch

import plain_fibelix as plain
from fibelix_util import CONFIGS, config, difference, doubles, latent, mixed, moe, position_errors, prompts, random_weights, rot
from trapetum_b200.config import ConfigError, FibelixConfig, load_config
from trapetum_b200.engine.model import tensor_specs_for_config
from trapetum_b200.parts.rope import rotary_frequencies


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_spec_names_the_tensors_of_a_model_folder(name):
    cfg = CONFIGS[name]
    w = random_weights(cfg, 1)
    specs = tensor_specs_for_config(cfg)
    needed = {n for n, s in specs.items() if not s.optional}
    assert needed == set(w)
    for n in needed:
        assert tuple(specs[n].shape) == tuple(w[n].shape), n


def test_the_schedule_reads_another_layers_cache_where_the_configuration_says_so():
    _, spec = load_config(CONFIGS["A"])
    assert [e.cache_of for e in spec.schedule] == [None, None, None, 1]
    assert spec.layers[3].mixer.params["k"] is None and spec.layers[1].mixer.params["k"] == "mix.k"
    assert spec.layers[1].mixer.params["keep_all"]          # its reader looks 70 back, itself 33
    _, spec = load_config(CONFIGS["B"])
    assert [e.cache_of for e in spec.schedule] == [None, None, None, None, 2, None]
    assert spec.head.params["weight"] == spec.embedding.params["weight"]


def test_every_constant_comes_from_the_configuration():
    cfg = FibelixConfig.from_dict(CONFIGS["B"])
    m = cfg.layers[0].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.window) == (4, 32, 32, 64, 48, 40, 64)
    assert m.rot.scaling == {"factor": 8.0, "original": 64.0, "fast": 16.0, "slow": 2.0}
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.block, a.rot.dims, a.rot.base, a.rot.scaling) == (4, 2, 64, 32, 250000.0, {"factor": 4.0})
    d = cfg.layers[4].mixer
    assert (d.diff, d.block, d.kv_from) == (0.1, 64, 2)
    assert cfg.layers[3].mlp is None and cfg.layers[2].mlp.top == 4


@pytest.mark.parametrize("change, says", [
    (lambda c: c["layers"][0].__setitem__("type", "attention_3"), "known mixers"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "layers[1].mixer.diff"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 3), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("dim", 16), "differ"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "layers[2].mixer.kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"), "scaling.slow"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top=9"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_wrong_configuration_is_refused_with_the_keys_name(change, says):
    c = copy.deepcopy(CONFIGS["A"])
    change(c)
    with pytest.raises(ConfigError) as e:
        FibelixConfig.from_dict(c)
    assert says in str(e.value)


@pytest.mark.parametrize("dims, base, factor, blend", [(16, 50000.0, 4.0, (2048, 32.0, 1.0)), (4, 1000.0, 2.0, (16, 4.0, 1.0)),
                                                      (32, 500.0, 3.0, (128, 8.0, 1.0)), (8, 100.0, 40.0, (4096, 1.0, 1.0))])
def test_blended_frequencies(dims, base, factor, blend):
    got, mult = rotary_frequencies(dims, base, {"factor": factor, "original": blend[0], "fast": blend[1], "slow": blend[2]})
    want, want_mult = plain.blended_frequencies(dims, base, factor, *blend)
    assert got.dtype == torch.float32 and torch.equal(got, want.float()) and mult == want_mult
    plain_f, one = rotary_frequencies(dims, base, {"factor": factor})
    assert one == 1.0 and torch.equal(plain_f, plain.linear_frequencies(dims, base, factor).float())
    # the blend lies between the two it blends
    lo, hi = plain.linear_frequencies(dims, base, factor), plain.linear_frequencies(dims, base)
    assert bool(((want >= lo * (1 - 1e-12)) & (want <= hi * (1 + 1e-12))).all())


def test_the_blocks_of_a_step_are_sequences_of_their_own():
    from types import SimpleNamespace
    from trapetum_b200.parts.diff_attention import block_sequences
    ctx = SimpleNamespace(seq_lens=[1, 12, 5, 10], memo={}, positions=torch.zeros(1))
    starts, token_block, lens, longest = block_sequences(ctx, 5)
    assert lens == [1, 5, 5, 2, 5, 5, 5] and longest == 5
    assert starts.tolist() == [0, 1, 6, 11, 13, 18, 23, 28]
    assert token_block.tolist() == [0] + [1] * 5 + [2] * 5 + [3] * 2 + [4] * 5 + [5] * 5 + [6] * 5
    assert block_sequences(ctx, 5)[0] is starts                   # once per step


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_fed_in_pieces_equals_itself(name):
    cfg = CONFIGS[name]
    w = doubles(random_weights(cfg, 2))
    ids = prompts(cfg["vocab"], [150], seed=1)[0]
    whole = plain.forward(cfg, w, ids)
    for pieces in ([149, 1], [1] + [1] * 149, [64, 1, 2, 63, 20], [5, 5, 5, 135]):
        assert float(position_errors(plain.logits(cfg, w, ids, pieces), whole).max()) < 1e-9


def test_what_the_masks_of_the_plain_implementation_let_through():
    pos = torch.arange(12)
    blocks = plain.same_block(pos, pos, 5)
    assert blocks[4, 0] and not blocks[5, 4] and blocks[5, 5] and blocks[9, 5] and not blocks[10, 9] and not blocks[3, 4]
    window = plain.in_window(pos, pos, 5)
    assert window[4, 0] and not window[5, 0] and window[5, 1] and not window[3, 4]
    one = plain.softmax_seen(torch.zeros(1, 3, dtype=plain.F), torch.ones(1, 3, dtype=torch.bool), extra_one=True)
    assert torch.allclose(one, torch.full((1, 3), 0.25, dtype=plain.F))


def test_a_single_layer_model_of_every_mixer_builds():
    for layer in (mixed(2, 1, 16, 24, 0.25, size=9, rot=rot(8, 100.0, 2.0)), difference(2, 1, 16, 24, 0.25, 0.4, size=7),
                  latent(2, 16, 8, 24, 32, 24, 0.2, size=6, rot=rot(8, 1000.0, 4.0, (32, 8.0, 1.0)))):
        cfg = config(50, 32, [(layer, None), (layer, moe(3, 1, 8))])
        specs = tensor_specs_for_config(cfg)
        assert "l0.norm2" in specs and specs["l0.norm2"].optional and not specs["l1.norm2"].optional
