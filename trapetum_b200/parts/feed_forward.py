"""Gated dense feed-forward: ``down(act(gate(x)) * up(x))``.

Gemma-2's form is GeGLU with the tanh approximation of GELU
(runtime/src/lib.rs:4511-4516; runtime/cuda/codebook_gemv.cu:531-537); the
activation is a parameter, as are both widths and the three tensor names.  The
gate and up matrices are fused into one when the weights are bound.  The
activation ``clamped_swish`` takes a ``limit`` L and bounds both branches:
``g' = min(g, L)``, ``u' = clamp(u, -L, L)``, ``g' sigmoid(1.702 g') (u' + 1)``.

``mlp`` is the form without a gate branch, ``down(act(up(x)))``, with a unary
activation (``relu2``: the square of relu).

Also here: ``none`` (a layer without a feed-forward) and ``token_gated``, a narrow
side input that is looked up by token id:
``proj(gelu_tanh(gate(x)) * table[token][first_col : first_col + dim])``.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear, linear_partials


class GatedMLP(FeedForward):
    graph_safe = True          # every launch depends on device data only
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params["activation"]
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated_mlp: unknown activation '{self.activation}' (known: {sorted(ops.ACTIVATIONS)})")
        self.limit = float(params.get("limit") or 0.0)
        if self.activation in ops.ACTIVATIONS_WITH_LIMIT and not self.limit > 0.0:
            raise ValueError(f"gated_mlp: activation '{self.activation}' needs a positive 'limit'")
        self.w_gu: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            self._name("gate"): TensorSpec((self.inter, self.hidden)),
            self._name("up"): TensorSpec((self.inter, self.hidden)),
            self._name("down"): TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors) -> None:
        g, u = tensors[self._name("gate")], tensors[self._name("up")]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        # With bfloat16 weights of tensor-core sizes the activation runs in the product's epilogue; the gate
        # and up rows are then interleaved in blocks of 16.  Otherwise: [gate; up] and a kernel of its own.
        self.fused = (dt == torch.bfloat16 and self.rt.dtype == torch.bfloat16 and self.inter % 16 == 0
                      and self.hidden % 8 == 0 and ops.gemm_tc_gates(self.activation))
        if self.fused:
            self.w_gu = ops.interleave_gate_up(g, u)
        else:
            self.w_gu = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = tensors[self._name("down")]

    def kernel_files(self):
        return linear_kernels(self.rt.dtype) + ("activation",)

    def forward(self, x, ctx):
        if self.fused and ops.gemm_tc_takes(x, self.w_gu):
            act = ops.gemm_tc(x, self.w_gu, self.rt.dtype, gated_act=self.activation, act_limit=self.limit)
            return linear_partials(act, self.w_down)
        if self.fused:
            raise RuntimeError("gated_mlp: the interleaved weights need the tensor-core product, which does not take "
                               f"an input of shape {tuple(x.shape)} with strides {x.stride()}")
        # an activation with thresholds gets its inputs unrounded, as the fused epilogue gives them
        gu = linear(x, self.w_gu, torch.float32 if self.limit else self.rt.dtype)
        act = ops.gated_act(gu, self.activation, self.rt.dtype, self.limit)
        return linear_partials(act, self.w_down)


class PlainMLP(FeedForward):
    """``down(act(up(x)))``.  Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` (a unary one: "relu2")
    and the tensor names ``up`` and ``down``.  With many tokens the activation runs in the tensor-core product's
    epilogue; with few, the product keeps its split-K partial sums and a small kernel adds and activates them."""
    graph_safe = True          # every launch depends on device data only

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params["activation"]
        if self.activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"mlp: unknown activation '{self.activation}' (known: {sorted(ops.UNARY_ACTIVATIONS)})")
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self._name("up"): TensorSpec((self.inter, self.hidden)),
                self._name("down"): TensorSpec((self.hidden, self.inter))}

    def bind(self, tensors) -> None:
        self.w_up = tensors[self._name("up")]
        self.w_down = tensors[self._name("down")]

    def kernel_files(self):
        return linear_kernels(self.rt.dtype) + ("activation",)

    def forward(self, x, ctx):
        if x.shape[0] > 128 and x.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and ops.gemm_tc_takes(x, self.w_up):
            act = ops.gemm_tc(x, self.w_up, self.rt.dtype, unary_act=self.activation)
        else:
            act = ops.unary_act(linear_partials(x, self.w_up), self.activation, self.rt.dtype)
        return linear_partials(act, self.w_down)

    def finish(self, part: torch.Tensor, col0: int) -> torch.Tensor:
        """The rest of the part when its first product was made together with another one: ``part`` holds
        ``up(x)`` as 32-bit partial sums in the columns from ``col0`` on."""
        act = ops.unary_act(part, self.activation, self.rt.dtype, col0, self.inter)
        return linear_partials(act, self.w_down)


class NoFeedForward(FeedForward):
    """A layer without a feed-forward: arrangements that allow it look at ``absent`` and skip the branch."""
    graph_safe = True
    absent = True

    def forward(self, x, ctx):
        raise RuntimeError("this layer has no feed-forward; its block must not call it")


class TokenGated(FeedForward):
    """``proj(gelu_tanh(gate(x)) * table[token][first_col : first_col + dim])``.  Parameters: ``hidden_size``, ``dim``,
    ``vocab_size``, ``table_width`` and ``first_col`` (the table is shared by the layers, each reads its own columns;
    its name is taken as it stands, without the layer's prefix), and the tensor names ``table``, ``gate``, ``proj``."""
    graph_safe = True          # the token ids are read on the device

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden_size"])
        self.dim = int(params["dim"])
        self.vocab = int(params["vocab_size"])
        self.table_width = int(params["table_width"])
        self.first_col = int(params["first_col"])
        if not (0 <= self.first_col and self.first_col + self.dim <= self.table_width):
            raise ValueError(f"token_gated: columns {self.first_col}..{self.first_col + self.dim} lie outside a table "
                             f"of width {self.table_width}")
        self.table = self.w_gate = self.w_proj = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            self.params["table"]: TensorSpec((self.vocab, self.table_width), "embedding"),
            self._name("gate"): TensorSpec((self.dim, self.hidden)),
            self._name("proj"): TensorSpec((self.hidden, self.dim)),
        }

    def bind(self, tensors) -> None:
        self.table = tensors[self.params["table"]]
        self.w_gate = tensors[self._name("gate")]
        self.w_proj = tensors[self._name("proj")]

    def kernel_files(self):
        return linear_kernels(self.rt.dtype) + ("activation",)

    def forward(self, x, ctx):
        if ctx.token_ids is None:
            raise RuntimeError("token_gated: the step's context carries no token ids")
        g = linear_partials(x, self.w_gate)                # narrow: 32-bit (partial sums) up to the activation
        return linear_partials(ops.token_gate(g, ctx.token_ids, self.table, self.first_col, self.rt.dtype), self.w_proj)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "mlp", PlainMLP)
register_part("feed_forward", "none", NoFeedForward)
register_part("feed_forward", "token_gated", TokenGated)
