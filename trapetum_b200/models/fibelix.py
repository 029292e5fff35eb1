"""Fibelix as data: its configuration turned into a :class:`ModelSpec`.

Nothing here computes.  A Fibelix layer is a ``pre_norm`` block (RMS norms whose stored weights lie around zero)
around one of three mixers and a feed-forward of experts:

* ``attention`` is :mod:`trapetum_b200.parts.attention` with biases, a rotation of the first ``rot.dims`` dims of
  every head with linear position scaling, a number per head on its scores, the heads' scores mixed by a matrix
  before the softmax, blocks of ``mask.size`` positions that see only themselves, and a softmax denominator with
  one added;
* ``attention_2`` is :mod:`trapetum_b200.parts.diff_attention`: two score maps per head over the same values, their
  outputs subtracted and normed; blocks as above; a layer with ``kv_from`` reads that layer's cache line (the
  schedule's ``cache_of``) with its own queries and mask;
* ``latent_attention`` is :mod:`trapetum_b200.parts.latent_attention` with the queries through a latent of their
  own, the rotation over neighbouring pairs with frequencies blended between their own and the scaled ones, a
  sliding window and a sigmoid gate per head on the output;
* the feed-forward is :mod:`trapetum_b200.parts.experts`: gated experts with silu, a bias on the router's logits, the
  ``top`` largest logits win and their weights are the softmax over the winners alone.

The head multiplies with the embedding table.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*`` (``q, k, v, o`` with ``.b`` biases, ``talk``,
``temp``; ``lq1, lk1, lq2, lk2``; ``dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g``), ``l<i>.mlp.router``, ``l<i>.mlp.router.b``,
``l<i>.mlp.e<j>.{gate,up,down}``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
from ..config.fibelix import FibelixConfig

MAX_POSITIONS = 1 << 24          # angles are position x frequency in 32-bit: every integer up to here is exact


def fibelix_spec(cfg: FibelixConfig) -> ModelSpec:
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "weight": name, "unit_offset": True})

    # an owner whose readers look farther back than itself must keep what they need
    farthest = {}
    for i, L in enumerate(cfg.layers):
        if L.type == "attention_2" and L.mixer.kv_from is not None:
            farthest.setdefault(L.mixer.kv_from, []).append(L.mixer.block)

    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "attention":
            position = PartSpec("rope", {"head_dim": m.dim, "rotary_dim": m.rot.dims, "theta": m.rot.base,
                                         "scaling_factor": (m.rot.scaling or {}).get("factor", 1.0)}) \
                if m.rot.dims else PartSpec("none", {"head_dim": m.dim})
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "scale": m.scale, "softcap": None, "window": None, "block": m.block, "unit_sink": True,
                "position": position, "head_temp": "mix.temp", "talk": "mix.talk",
                "bias": {"q": "mix.q.b", "k": "mix.k.b", "v": "mix.v.b", "o": "mix.o.b"},
                "q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o",
            })
        elif L.type == "attention_2":
            reads = m.kv_from is not None
            others = farthest.get(i, [])
            keep_all = any(b is None or (m.block is not None and b > m.block) for b in others) or m.block is None
            mixer = PartSpec("diff_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "dim": m.dim, "value_dim": m.vdim,
                "scale": m.scale, "diff": m.diff, "eps": cfg.norm_eps, "block": m.block, "keep_all": keep_all,
                "q": "mix.q", "k": None if reads else "mix.k", "v": None if reads else "mix.v", "o": "mix.o",
                "lq1": "mix.lq1", "lk1": "mix.lk1", "lq2": "mix.lq2", "lk2": "mix.lk2",
            })
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "heads": m.heads, "plain_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "sink": None, "window": m.window,
                "rotary": {"dims": m.rot.dims, "base": m.rot.base, "scaling": m.rot.scaling, "pairing": "neighbours"},
                "q_latent": {"rank": m.q_rank, "down": "mix.dq", "norm": "mix.dq.norm", "up": "mix.uq"},
                "out_gate": "mix.g",
                "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "o": "mix.o",
            })
        if L.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "experts": L.mlp.experts, "top": L.mlp.top, "intermediate_size": L.mlp.ff,
                "activation": "silu", "score": "softmax", "groups": 1, "keep_groups": 1, "group_score_of": 1,
                "weight_eps": 0.0, "router": "mlp.router", "router_bias": "mlp.router.b", "correction": None,
                "expert": "mlp.e{}.", "gate": "gate", "up": "up", "down": "down", "shared": None,
            })
        else:
            ffn = PartSpec("none", {})
        block = PartSpec("pre_norm", {"pre_mixer_norm": norm("norm1"),
                                      "pre_ffn_norm": norm("norm2") if L.mlp is not None else None,
                                      "idle": {} if L.mlp is not None else {"norm2": W}})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, prefix=f"l{i}."))

    schedule = []
    for i, L in enumerate(cfg.layers):
        src = L.mixer.kv_from if L.type == "attention_2" else None
        schedule.append(ScheduleEntry(i, cache_of=src))          # every layer runs once: entry i is layer i

    return ModelSpec(
        architecture="Fibelix",
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": 1.0, "weight": "embed"}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "softcap": None, "scale": None,
                                      "weight": "embed", "tied_to": None}),
        max_positions=MAX_POSITIONS,
        stop_ids=(),
    )


register_architecture("Fibelix", FibelixConfig, fibelix_spec, native=False)
