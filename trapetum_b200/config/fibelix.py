"""Fibelix's configuration, read from the keys of its config.json.

Top level: ``architecture`` ("Fibelix"), ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list whose entries give
``type`` (one of the mixers below), ``mixer`` (its sizes and constants) and ``mlp`` (``{"kind": "moe", "expert":
{"ff"}, "router": {"experts", "top"}}`` or null).

``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (blocks of that many positions),
``rot.dims``, ``rot.base``, ``rot.scaling.factor``.
``attention_2``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``diff``, ``mask.size`` (blocks), ``kv_from`` (the
layer whose keys and values it reads; absent: its own).
``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``mask.size`` (a sliding
window), ``rot.dims``, ``rot.base``, ``rot.scaling`` (``factor``; with ``original``, ``fast``, ``slow`` a blend per frequency).

Every size and constant is read by key, with an error that names the key; nothing is assumed equal between layers.
What a layer leaves out does not exist for it: no ``mask``, every earlier token is seen; no ``rot``, no rotation; no
``scaling``, frequencies as they are; ``mlp`` null, no feed-forward.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, _get
from .divanex import _obj, _sub

MIXERS = ("attention", "attention_2", "latent_attention")


@dataclass(frozen=True)
class Rotation:
    dims: int                    # how many of a head's first dims (of the rotated part) the rotation turns; 0: none
    base: float
    scaling: Optional[Dict[str, float]]     # None, {"factor"} or {"factor", "original", "fast", "slow"}


@dataclass(frozen=True)
class MixedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    block: Optional[int]
    rot: Rotation


@dataclass(frozen=True)
class DifferenceAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    block: Optional[int]
    kv_from: Optional[int]


@dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: Optional[int]
    rot: Rotation


@dataclass(frozen=True)
class TopMoe:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class FibelixLayer:
    type: str
    mixer: object
    mlp: Optional[TopMoe]


def _mask(m, mw) -> Optional[int]:
    mask = _obj(m, "mask", mw, nullable=True)
    if not mask:
        return None
    size = _sub(mask, "size", int, mw + "mask.")
    if size < 1:
        raise ConfigError(f"config.json: {mw}mask.size={size} must be positive")
    return size


def _rotation(m, mw, default_dims: int) -> Rotation:
    rot = _obj(m, "rot", mw, nullable=True)
    if not rot:
        return Rotation(0, 10000.0, None)
    rw = mw + "rot."
    dims = _sub(rot, "dims", int, rw, default_dims)
    base = _sub(rot, "base", float, rw, 10000.0)
    if dims % 2 or not (0 <= dims <= default_dims) or not base > 0.0:
        raise ConfigError(f"config.json: {rw}dims={dims} must be even and at most {default_dims}, {rw}base positive")
    sc = _obj(rot, "scaling", rw, nullable=True)
    scaling = None
    if sc:
        sw = rw + "scaling."
        scaling = {"factor": _sub(sc, "factor", float, sw)}
        if not scaling["factor"] > 0.0:
            raise ConfigError(f"config.json: {sw}factor must be positive")
        if any(key in sc for key in ("original", "fast", "slow")):
            for key in ("original", "fast", "slow"):
                scaling[key] = _sub(sc, key, float, sw)
                if not scaling[key] > 0.0:
                    raise ConfigError(f"config.json: {sw}{key} must be positive")
    return Rotation(dims, base, scaling)


@dataclass(frozen=True)
class FibelixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FibelixLayer, ...]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FibelixConfig":
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
            vdim = _sub(m, "vdim", int, mw, dim)
            scale = _sub(m, "scale", float, mw)
            if min(heads, dim, vdim) < 1:
                raise ConfigError(f"config.json: {mw}heads, dim and vdim must be positive")
            if typ == "latent_attention":
                rot_dim = _sub(m, "rot_dim", int, mw)
                mixer = LatentAttention(heads, dim, rot_dim, vdim, _sub(m, "kv_rank", int, mw), _sub(m, "q_rank", int, mw),
                                        scale, _mask(m, mw), _rotation(m, mw, rot_dim))
                if min(mixer.kv_rank, mixer.q_rank) < 1 or rot_dim < 0:
                    raise ConfigError(f"config.json: {mw}kv_rank and q_rank must be positive, rot_dim not negative")
            else:
                kv_heads = _sub(m, "kv_heads", int, mw, heads)
                if kv_heads < 1 or heads % kv_heads:
                    raise ConfigError(f"config.json: {mw}kv_heads={kv_heads} must be positive and divide heads={heads}")
                if typ == "attention":
                    mixer = MixedAttention(heads, kv_heads, dim, vdim, scale, _mask(m, mw), _rotation(m, mw, dim))
                else:
                    kv_from = _sub(m, "kv_from", int, mw, None, nullable=True) if "kv_from" in m else None
                    mixer = DifferenceAttention(heads, kv_heads, dim, vdim, scale, _sub(m, "diff", float, mw), _mask(m, mw),
                                                kv_from)
            mlp = None
            ml = _obj(L, "mlp", where, nullable=True)
            if ml is not None:
                lw = where + "mlp."
                kind = _sub(ml, "kind", str, lw)
                if kind != "moe":
                    raise ConfigError(f"config.json: {lw}kind is '{kind}'; known kinds: moe")
                r = _obj(ml, "router", lw)
                mlp = TopMoe(_sub(r, "experts", int, lw + "router."), _sub(r, "top", int, lw + "router."),
                             _sub(_obj(ml, "expert", lw), "ff", int, lw + "expert."))
                if mlp.experts < 1 or mlp.ff < 1 or not (1 <= mlp.top <= mlp.experts):
                    raise ConfigError(f"config.json: {lw}router: top={mlp.top} of experts={mlp.experts}, ff={mlp.ff}")
            layers.append(FibelixLayer(typ, mixer, mlp))
        for i, L in enumerate(layers):
            j = L.mixer.kv_from if L.type == "attention_2" else None
            if j is None:
                continue
            src = layers[j] if 0 <= j < i else None
            if src is None or src.type != "attention_2" or src.mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} must name an earlier attention_2 layer "
                                  "that has keys and values of its own")
            a, b = L.mixer, src.mixer
            if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layers[{j}], whose kv_heads, dim "
                                  "and vdim differ from its own")
        return cls(vocab=vocab, width=width, norm_eps=_sub(norm, "eps", float, "norm."), layers=tuple(layers))
