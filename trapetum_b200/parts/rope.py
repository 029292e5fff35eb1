"""Rotary position encoding (rotate-half pairing).

For each head and i in [0, R/2): ``angle = pos * theta^(-2i/R)`` and the pair
``(x[i], x[i+R/2])`` is rotated by it (runtime/cuda/codebook_gemv.cu:219-230;
the table of inverse frequencies is made as in model/export_gemma.py:53).  R is
``rotary_dim`` (the whole head for Gemma-2).  ``scaling_factor`` f (1 if absent)
is linear position scaling: every frequency is divided by f.  The table is made once, in
32-bit; the kernel multiplies by the position and takes sin and cos in 32-bit.
The rotation is fused with the cache write, so a mixer hands this part its qkv
matrix and its cache line in one call.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import PositionEncoding, register_part


def rotary_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """(frequencies float32 [dims / 2], factor on cos and sin) of a rotation over ``dims`` numbers.

    ``f_i = base^(-2i / dims)``.  ``scaling`` None: as they are.  ``{"factor": s}``: every frequency divided by s (linear
    position scaling).  ``{"factor": s, "original": L, "fast": a, "slow": b}``: a blend per frequency between ``f_i``
    (dims that turn more than ``a`` times over L positions) and ``f_i / s`` (dims that turn fewer than ``b`` times):
    with ``d(t) = dims * ln(L / (2 pi t)) / (2 ln base)``, ``lo = max(floor(d(a)), 0)``, ``hi = min(ceil(d(b)), dims - 1)``
    and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency is ``f_i / s * ramp_i + f_i * (1 - ramp_i)``,
    and cos and sin come times ``0.1 ln(s) + 1``.  Computed in 64-bit, stored in 32."""
    import math
    half = dims // 2
    f = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    mult = 1.0
    sc = dict(scaling or {})
    if "original" in sc:
        s, L = float(sc["factor"]), float(sc["original"])

        def dim_of(turns):
            return dims * math.log(L / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)]
        f = [x / s * r + x * (1.0 - r) for x, r in zip(f, ramp)]
        mult = 0.1 * math.log(s) + 1.0
    elif sc.get("factor"):
        f = [x / float(sc["factor"]) for x in f]
    return torch.tensor(f, dtype=torch.float64).to(torch.float32), mult


class Rope(PositionEncoding):
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        self.scaling_factor = float(params.get("scaling_factor") or 1.0)
        if not self.scaling_factor > 0.0:
            raise ValueError(f"rope: scaling_factor must be positive, got {self.scaling_factor}")
        self._inv_freq_cpu = 1.0 / (torch.tensor(self.theta, dtype=torch.float32) ** (idx / self.rotary_dim))
        if self.scaling_factor != 1.0:
            self._inv_freq_cpu = self._inv_freq_cpu / self.scaling_factor
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, tensors) -> None:
        self.inv_freq = self._inv_freq_cpu.to(self.rt.device)

    def kernel_files(self):
        return ("rope_kv",)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim

    def rotate_and_store(self, qkv, n_heads, n_kv_heads, ctx, line, store: bool, partial=None) -> None:
        """Rotate q and k inside ``qkv`` at the step's positions; with ``store`` also
        write k and v into the cache line.  ``partial``: split-K partial sums of the projection
        ([splits, tokens, width] float32) to take the values from; ``qkv`` is then only written."""
        ops.rope_kv(qkv, n_heads, n_kv_heads, self.head_dim, self.rotary_dim, self.inv_freq,
                    ctx.positions, ctx.token_seq, ctx.len_after,
                    line.k if store else None, line.v if store else None,
                    line.page_table if store else None, line.ring_rows if store else 0, partial)


class NoPosition(PositionEncoding):
    """No position encoding: keys and values are stored as they are."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.head_dim = int(params["head_dim"])

    def kernel_files(self):
        return ("rope_kv",)

    def rotary_table(self):
        return None, 0

    def rotate_and_store(self, qkv, n_heads, n_kv_heads, ctx, line, store: bool, partial=None) -> None:
        if store or partial is not None:
            ops.rope_kv(qkv, n_heads, n_kv_heads, self.head_dim, 0, None, ctx.positions, ctx.token_seq,
                        ctx.len_after, line.k if store else None, line.v if store else None,
                        line.page_table if store else None, line.ring_rows if store else 0, partial)


register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
