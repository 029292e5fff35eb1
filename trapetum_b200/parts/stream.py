"""The residual stream of a step: a 32-bit [tokens, hidden] matrix and the one
branch output that still waits to be added.

Blocks never add into the stream themselves.  They call :meth:`add` or
:meth:`add_normed` with a branch output and :meth:`normed` when they need the
next normalised input; the stream holds an addition back until the next read
so that ``h += norm_a(a); x = norm_b(h)`` runs as one kernel, also across the
border between two layers.  The sum itself is always 32-bit.

Arrangements that norm AFTER the sum replace the stream instead of adding to it:
:meth:`fold_normed` is ``h <- norm(alpha * h + a)``, and their sublayers read the
stream itself through :meth:`read` (a copy in the compute dtype when that is not
32-bit), which rides along with whatever was still waiting.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import Norm


class ResidualStream:
    def __init__(self, h: torch.Tensor):
        assert h.dtype == torch.float32
        self.h = h
        self._pending = None          # (branch output, its norm or None, alpha or None)

    def add(self, a: torch.Tensor) -> None:
        """h += a (no norm on the branch output)."""
        self._flush()
        self._pending = (a, None, None)

    def add_normed(self, a: torch.Tensor, norm: Norm) -> None:
        """h += norm(a)."""
        self._flush()
        self._pending = (a, norm, None)

    def add_scaled(self, branches, scale: float) -> None:
        """h += scale * (sum of one or two branch outputs, float32 or their split-K partial sums)."""
        self._flush()
        self._pending = (list(branches), None, ("scaled", float(scale)))

    def fold_normed(self, a: torch.Tensor, norm: Norm, alpha: float) -> None:
        """h <- norm(alpha * h + a): the norm after the sum."""
        self._flush()
        self._pending = (a, norm, float(alpha))

    def normed(self, norm: Norm, out_dtype: torch.dtype) -> torch.Tensor:
        """norm(h), after whatever addition was still waiting."""
        if self._pending is not None and isinstance(self._pending[2], tuple):
            branches, _, (_, scale) = self._pending
            if hasattr(norm, "add_scaled_apply"):
                self._pending = None
                return norm.add_scaled_apply(self.h, branches, scale, out_dtype)      # the scaled sum and the norm in one kernel
        if self._pending is not None and self._pending[2] is None:
            a, post, _ = self._pending
            self._pending = None
            if post is not None:
                return post.add_to(self.h, a, norm, out_dtype)
            if hasattr(norm, "add_apply"):
                return norm.add_apply(self.h, a, out_dtype)      # the sum and the norm in one kernel
            ops.residual_add(self.h, a)
        self._flush()
        return norm.apply(self.h, out_dtype)

    def read(self, out_dtype: torch.dtype) -> torch.Tensor:
        """The stream itself for a sublayer that reads it unnormed: ``h`` when the compute dtype is 32-bit, else a
        rounded copy, made by the kernel that applies what was still waiting."""
        want = None if out_dtype == torch.float32 else out_dtype
        if self._pending is not None and self._pending[1] is not None:
            a, norm, alpha = self._pending
            self._pending = None
            out = norm.fold(self.h, a, alpha, want)
            return self.h if want is None else out
        self._flush()
        return self.h if want is None else ops.cast(self.h, want)

    def add_rows(self, rows: Optional[torch.Tensor], vector: Optional[torch.Tensor]) -> None:
        """h += rows (a float32 matrix of the stream's shape) + vector (one float32 row, added to every token)."""
        self._flush()
        ops.add_rows(self.h, rows, vector)

    def value(self) -> torch.Tensor:
        self._flush()
        return self.h

    def _flush(self) -> None:
        if self._pending is None:
            return
        a, post, alpha = self._pending
        self._pending = None
        if isinstance(alpha, tuple):
            ops.add_scaled_rmsnorm(self.h, a, alpha[1])
        elif alpha is not None:
            post.fold(self.h, a, alpha, None)
        elif post is not None:
            post.add_to(self.h, a, None, None)
        else:
            ops.residual_add(self.h, a)
