"""Fidepel's configuration, read from the keys of its config.json.

Top level: ``architecture`` ("Fidepel"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (absent: 1), ``loop``
(``start``, ``stop``, ``times``; absent: every layer runs once) and ``layers``, a list whose entries give ``type``
("attention"), ``mixer`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``rot.dims``,
``rot.base``, ``rot.scaling.factor``) and ``mlp`` (``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top",
"scale", "groups": {"count", "keep"}}, "shared": {"ff"}}`` or null).  Every size and constant is read by key, with an
error that names the key; nothing is assumed equal between layers.  What a layer leaves out does not exist for it:
no ``mask``, no window; no ``rot``, no rotation; no ``scaling``, factor 1; no ``groups``, one group; no ``shared``,
no shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, _get
from .divanex import _obj, _sub
from .lofirax import Loop

MIXERS = ("attention",)


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]        # a query sees itself and the window - 1 tokens before it; None: all of them
    rot_dims: int                # how many of a head's first dims the rotation turns (0: none)
    rot_base: float
    rot_factor: float            # linear position scaling: every frequency divided by this


@dataclass(frozen=True)
class SoftmaxMoe:
    experts: int
    top: int
    ff: int
    scale: float                 # the winners' weights times this
    groups: int                  # 1: no groups
    keep: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class FidepelLayer:
    type: str
    mixer: WindowAttention
    mlp: Optional[SoftmaxMoe]


@dataclass(frozen=True)
class FidepelConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    loop: Optional[Loop]
    layers: Tuple[FidepelLayer, ...]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FidepelConfig":
        vocab = _get(d, "vocab", int)
        width = _get(d, "width", int)
        if vocab < 1 or width < 1:
            raise ConfigError(f"config.json: vocab={vocab} and width={width} must be positive")
        norm = _obj(d, "norm", "")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            typ = _sub(L, "type", str, where)
            if typ not in MIXERS:
                raise ConfigError(f"config.json: {where}type is '{typ}'; known mixers: {', '.join(MIXERS)}")
            m = _obj(L, "mixer", where)
            mw = where + "mixer."
            heads = _sub(m, "heads", int, mw)
            dim = _sub(m, "dim", int, mw)
            mask = _obj(m, "mask", mw, nullable=True)
            rot = _obj(m, "rot", mw, nullable=True)
            scaling = _obj(rot, "scaling", mw + "rot.", nullable=True) if rot else None
            mixer = WindowAttention(
                heads, _sub(m, "kv_heads", int, mw, heads), dim, _sub(m, "vdim", int, mw, dim), _sub(m, "scale", float, mw),
                _sub(mask, "size", int, mw + "mask.") if mask else None,
                _sub(rot, "dims", int, mw + "rot.", dim) if rot else 0,
                _sub(rot, "base", float, mw + "rot.", 10000.0) if rot else 10000.0,
                _sub(scaling, "factor", float, mw + "rot.scaling.") if scaling else 1.0)
            if min(mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim) < 1 or mixer.heads % mixer.kv_heads:
                raise ConfigError(f"config.json: {mw}heads, kv_heads, dim and vdim must be positive and kv_heads divide heads")
            if mixer.window is not None and mixer.window < 1:
                raise ConfigError(f"config.json: {mw}mask.size={mixer.window} must be positive")
            if mixer.rot_dims % 2 or not (0 <= mixer.rot_dims <= mixer.dim):
                raise ConfigError(f"config.json: {mw}rot.dims={mixer.rot_dims} must be even and at most dim={mixer.dim}")
            if not mixer.rot_factor > 0.0 or not mixer.rot_base > 0.0:
                raise ConfigError(f"config.json: {mw}rot.base and rot.scaling.factor must be positive")
            mlp = None
            ml = _obj(L, "mlp", where, nullable=True)
            if ml is not None:
                lw = where + "mlp."
                kind = _sub(ml, "kind", str, lw)
                if kind != "moe":
                    raise ConfigError(f"config.json: {lw}kind is '{kind}'; known kinds: moe")
                r = _obj(ml, "router", lw)
                g = _obj(r, "groups", lw + "router.", nullable=True)
                sh = _obj(ml, "shared", lw, nullable=True)
                mlp = SoftmaxMoe(_sub(r, "experts", int, lw + "router."), _sub(r, "top", int, lw + "router."),
                                 _sub(_obj(ml, "expert", lw), "ff", int, lw + "expert."),
                                 _sub(r, "scale", float, lw + "router.", 1.0),
                                 _sub(g, "count", int, lw + "router.groups.") if g else 1,
                                 _sub(g, "keep", int, lw + "router.groups.") if g else 1,
                                 _sub(sh, "ff", int, lw + "shared.") if sh else None)
                if mlp.experts < 1 or mlp.ff < 1 or not (1 <= mlp.top <= mlp.experts):
                    raise ConfigError(f"config.json: {lw}router: top={mlp.top} of experts={mlp.experts}, ff={mlp.ff}")
                if mlp.groups < 1 or mlp.experts % mlp.groups or not (1 <= mlp.keep <= mlp.groups):
                    raise ConfigError(f"config.json: {lw}router.groups: {mlp.experts} experts do not form "
                                      f"{mlp.groups} equal groups of which {mlp.keep} are kept")
                if mlp.keep * (mlp.experts // mlp.groups) < mlp.top:
                    raise ConfigError(f"config.json: {lw}router: {mlp.keep} kept groups hold fewer than "
                                      f"top={mlp.top} experts")
                if mlp.shared_ff is not None and mlp.shared_ff < 1:
                    raise ConfigError(f"config.json: {lw}shared.ff={mlp.shared_ff} must be positive")
            layers.append(FidepelLayer(typ, mixer, mlp))
        loop = None
        lp = _obj(d, "loop", "", nullable=True)
        if lp is not None:
            loop = Loop(_sub(lp, "start", int, "loop."), _sub(lp, "stop", int, "loop."), _sub(lp, "times", int, "loop."))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError(f"config.json: loop start={loop.start} stop={loop.stop} times={loop.times} does not "
                                  f"fit {len(layers)} layers")
        return cls(vocab=vocab, width=width, norm_eps=_sub(norm, "eps", float, "norm."),
                   residual_mult=_get(d, "residual_mult", float, 1.0), loop=loop, layers=tuple(layers))
