"""Arrangements of a layer's parts around the residual stream.

``sandwich``: a norm before and a norm after each of the two branches
(runtime/src/lib.rs:4527-4540):

    h += post_mixer_norm(mixer(pre_mixer_norm(h)))
    h += post_ffn_norm(feed_forward(pre_ffn_norm(h)))

``pre_norm``: the common two-norm arrangement, branch outputs added as they are:

    h += mixer(pre_mixer_norm(h));  h += feed_forward(pre_ffn_norm(h))

``post_norm``: the norm comes after the sum, the stream is scaled by ``alpha`` on
the way in, and both sublayers read the stream itself:

    h <- mixer_norm(alpha h + mixer(h));  h <- ffn_norm(alpha h + feed_forward(h))

(the second line only if the layer has a feed-forward), then, if the layer has a
``side`` input (a feed-forward that may look at the step's token ids),
``h <- h + side_norm(side(h))``.

``parallel``: one norm, both sublayers read its output, and their outputs are
added together, times ``scale`` (1 if absent):

    x = norm(h);  h += scale * (mixer(x) + feed_forward(x))

(without a feed-forward: ``h += scale * mixer(x)``).

A block only talks to the :class:`~trapetum_b200.parts.stream.ResidualStream`,
which decides how additions and norms are fused.
"""
from __future__ import annotations

from typing import Dict

from ..weights.loader import TensorSpec
from .base import Block, build_part, register_part


class _NormedBlock(Block):
    graph_safe = True          # every launch depends on device data only
    NORMS = ()

    def __init__(self, params, prefix, rt, mixer, feed_forward):
        super().__init__(params, prefix, rt, mixer, feed_forward)
        self.norms = {n: build_part("norm", params[n], prefix, rt) for n in self.NORMS}

    def parts(self):
        return list(self.norms.values()) + [self.mixer, self.feed_forward]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for p in self.parts():
            specs.update(p.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        for p in self.parts():
            p.bind(tensors)

    def kernel_files(self):
        out = ()
        for p in self.parts():
            out += tuple(p.kernel_files())
        return out


class SandwichBlock(_NormedBlock):
    NORMS = ("pre_mixer_norm", "post_mixer_norm", "pre_ffn_norm", "post_ffn_norm")

    def forward(self, stream, ctx, cache) -> None:
        dt = self.rt.dtype
        x = stream.normed(self.norms["pre_mixer_norm"], dt)
        stream.add_normed(self.mixer.forward(x, ctx, cache), self.norms["post_mixer_norm"])
        x = stream.normed(self.norms["pre_ffn_norm"], dt)
        stream.add_normed(self.feed_forward.forward(x, ctx), self.norms["post_ffn_norm"])


class PreNormBlock(_NormedBlock):
    """``pre_ffn_norm`` may be None for a layer whose feed-forward is of kind "none": the second line is then left out."""
    NORMS = ("pre_mixer_norm", "pre_ffn_norm")

    def __init__(self, params, prefix, rt, mixer, feed_forward):
        Block.__init__(self, params, prefix, rt, mixer, feed_forward)
        self.has_ffn = not getattr(feed_forward, "absent", False)
        if self.has_ffn and not params.get("pre_ffn_norm"):
            raise ValueError("pre_norm: a layer with a feed-forward needs 'pre_ffn_norm'")
        self.norms = {n: build_part("norm", params[n], prefix, rt) for n in self.NORMS
                      if n == "pre_mixer_norm" or self.has_ffn}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = super().tensor_specs()
        # ``idle``: tensor name -> size of vectors that a file may carry for a layer without feed-forward (the norm
        # that nothing follows); they are accepted and not used
        for name, size in (self.params.get("idle") or {}).items():
            specs.setdefault(self.prefix + name, TensorSpec((int(size),), "norm", optional=True))
        return specs

    def forward(self, stream, ctx, cache) -> None:
        dt = self.rt.dtype
        x = stream.normed(self.norms["pre_mixer_norm"], dt)
        stream.add(self.mixer.forward(x, ctx, cache))
        if self.has_ffn:
            x = stream.normed(self.norms["pre_ffn_norm"], dt)
            stream.add(self.feed_forward.forward(x, ctx))


class PostNormBlock(_NormedBlock):
    """Parameters: ``alpha``, ``mixer_norm``, ``ffn_norm`` (None when the layer's feed-forward is of kind "none"),
    ``side`` (a feed-forward spec or None) and ``side_norm``."""

    def __init__(self, params, prefix, rt, mixer, feed_forward):
        Block.__init__(self, params, prefix, rt, mixer, feed_forward)
        self.alpha = float(params["alpha"])
        self.has_ffn = not getattr(feed_forward, "absent", False)
        self.norms = {"mixer_norm": build_part("norm", params["mixer_norm"], prefix, rt)}
        if self.has_ffn:
            if not params.get("ffn_norm"):
                raise ValueError("post_norm: a layer with a feed-forward needs 'ffn_norm'")
            self.norms["ffn_norm"] = build_part("norm", params["ffn_norm"], prefix, rt)
        self.side = None
        if params.get("side"):
            self.side = build_part("feed_forward", params["side"], prefix, rt)
            self.norms["side_norm"] = build_part("norm", params["side_norm"], prefix, rt)

    @property
    def graph_safe(self):
        return self.side is None or getattr(self.side, "graph_safe", False)

    def parts(self):
        return list(self.norms.values()) + [self.mixer, self.feed_forward] + ([self.side] if self.side else [])

    def forward(self, stream, ctx, cache) -> None:
        dt = self.rt.dtype
        stream.fold_normed(self.mixer.forward(stream.read(dt), ctx, cache), self.norms["mixer_norm"], self.alpha)
        if self.has_ffn:
            stream.fold_normed(self.feed_forward.forward(stream.read(dt), ctx), self.norms["ffn_norm"], self.alpha)
        if self.side is not None:
            stream.add_normed(self.side.forward(stream.read(dt), ctx), self.norms["side_norm"])


class ParallelBlock(_NormedBlock):
    """Parameters: ``norm`` (the one norm's spec) and ``scale``."""
    NORMS = ("norm",)

    def __init__(self, params, prefix, rt, mixer, feed_forward):
        super().__init__(params, prefix, rt, mixer, feed_forward)
        self.scale = float(params.get("scale", 1.0))
        self.has_ffn = not getattr(feed_forward, "absent", False)

    def forward(self, stream, ctx, cache) -> None:
        x = stream.normed(self.norms["norm"], self.rt.dtype)
        branches = [self.mixer.forward(x, ctx, cache)]
        if self.has_ffn:
            branches.append(self.feed_forward.forward(x, ctx))
        stream.add_scaled(branches, self.scale)


register_part("block", "parallel", ParallelBlock)
register_part("block", "post_norm", PostNormBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "pre_norm", PreNormBlock)
