"""Fidepel as data: its configuration turned into a :class:`ModelSpec`.

Nothing here computes.  A Fidepel layer is a ``parallel`` block: one RMS norm whose weight is a single number, an
attention mixer and a feed-forward of experts that both read the normed input, and their outputs added to the stream
together, times ``residual_mult``:

* the mixer is :mod:`trapetum_b200.parts.attention` with a sliding window, a rotation of the first ``rot.dims`` dims of
  every head with linear position scaling, q and k RMS-normed over the whole projection, a number per head that
  multiplies its scores, values of their own size, and a sigmoid gate per head on the output;
* the feed-forward is :mod:`trapetum_b200.parts.experts` with softmax scores, groups scored by their best expert,
  experts and a shared expert of the form ``down(relu(up x)^2)``, and a scale on the winners' weights.

A span of layers may run several times in a row with the same weights: the schedule names those layers once per
pass, and every call owns a cache of its own.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.{q,k,v,o,g,temp,q.norm,k.norm}``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.{up,down}``, ``l<i>.mlp.shared.{up,down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
from ..config.fidepel import FidepelConfig

MAX_POSITIONS = 1 << 24          # angles are position x frequency in 32-bit: every integer up to here is exact


def fidepel_spec(cfg: FidepelConfig) -> ModelSpec:
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "weight": name, "scalar": True})

    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        position = PartSpec("rope", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                     "scaling_factor": m.rot_factor}) if m.rot_dims else PartSpec("none", {"head_dim": m.dim})
        mixer = PartSpec("attention", {
            "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
            "scale": m.scale, "softcap": None, "window": m.window, "position": position,
            "proj_norm": {"q": "mix.q.norm", "k": "mix.k.norm", "eps": cfg.norm_eps},
            "head_temp": "mix.temp", "out_gate": "mix.g",
            "q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o",
        })
        if L.mlp is not None:
            shared = None
            if L.mlp.shared_ff:
                shared = {"intermediate_size": L.mlp.shared_ff, "up": "mlp.shared.up", "down": "mlp.shared.down"}
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "experts": L.mlp.experts, "top": L.mlp.top, "intermediate_size": L.mlp.ff,
                "gated": False, "activation": "relu2", "score": "softmax", "route_scale": L.mlp.scale,
                "groups": L.mlp.groups, "keep_groups": L.mlp.keep, "group_score_of": 1, "weight_eps": 1e-20,
                "router": "mlp.router", "correction": None,
                "expert": "mlp.e{}.", "up": "up", "down": "down", "shared": shared,
            })
        else:
            ffn = PartSpec("none", {})
        block = PartSpec("parallel", {"norm": norm("norm1"), "scale": cfg.residual_mult})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, prefix=f"l{i}."))

    n = len(layers)
    if cfg.loop is None:
        order = list(range(n))
    else:
        lp = cfg.loop
        order = list(range(lp.start)) + list(range(lp.start, lp.stop)) * lp.times + list(range(lp.stop, n))

    return ModelSpec(
        architecture="Fidepel",
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": 1.0, "weight": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in order),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "softcap": None, "scale": None,
                                      "weight": "head", "tied_to": None}),
        max_positions=MAX_POSITIONS,
        stop_ids=(),
    )


register_architecture("Fidepel", FidepelConfig, fidepel_spec, native=False)
