"""A feed-forward made of experts behind a router, with an optional gated shared expert.

``experts`` small gated feed-forwards ``down_e(act(gate_e x) * up_e x)`` without biases; each token uses ``top``
of them.  The router (all of it 32-bit): logits ``z = R x``, scores ``s = sigmoid(z)``; *choice scores* are
``s + correction``; the experts form ``groups`` equal groups of neighbours, a group's score is the sum of its
``group_score_of`` largest choice scores, and only experts of the ``keep_groups`` best groups can be chosen (the
others' choice scores count as minus infinity); the ``top`` largest choice scores win; the winners' weights are
their ``s`` (without the correction) divided by their sum plus ``weight_eps``.  The output is the weighted sum
of the winners' outputs, plus, if there is a shared expert, ``sigmoid(g . x)`` times its output for every token.

Two more forms of the same part: ``score`` "softmax" takes ``s = softmax(z)`` over all experts, and ``gated``
False makes the experts ``down_e(act(up_e x))`` with a unary activation ("relu2", the square of relu) and no gate
matrix; the shared expert is then of that form too.  ``route_scale`` multiplies the winners' weights.
``router_bias`` (a tensor name, one number per expert) is added to the logits themselves, by the routing kernel.  A softmax over the
winners' logits only is ``score`` "softmax" with ``weight_eps`` 0: the winners' shares of the softmax over all
experts, divided by their sum, are exactly that.

Parameters (none is fixed in code): ``hidden_size``, ``experts``, ``top``, ``intermediate_size``, ``activation``
("silu"), ``score`` ("sigmoid"), ``groups``, ``keep_groups``, ``group_score_of``, ``weight_eps``, the tensor names
``router``, ``correction`` (None: no correction), ``expert`` (a pattern with ``{}`` for the expert's number) with
``gate``, ``up``, ``down`` below it, and ``shared``: None or ``{"intermediate_size", "gate", "up", "down",
"token_gate"}`` (``token_gate`` None: the shared expert is added as it is; no ``gate`` with ungated experts).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part
from .feed_forward import GatedMLP, PlainMLP
from .linear import kernel_files as linear_kernels
from .linear import linear_partials


FUSED_UP_TOKENS = 128     # up to here a product comes as split-K partial sums anyway (the swapped tensor-core form)


class RoutedExperts(FeedForward):
    graph_safe = True          # the routing stays on the device: no launch depends on which experts were chosen

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden_size"])
        self.E = int(p["experts"])
        self.top = int(p["top"])
        self.ff = int(p["intermediate_size"])
        self.groups = int(p.get("groups") or 1)
        self.keep = int(p.get("keep_groups") or self.groups)
        self.group_top = int(p.get("group_score_of") or 1)
        self.weight_eps = float(p.get("weight_eps") or 0.0)
        self.gated = bool(p.get("gated", True))
        self.activation = p.get("activation", "silu")
        self.score = p.get("score", "sigmoid")
        self.route_scale = float(p.get("route_scale", 1.0))
        if self.activation != ("silu" if self.gated else "relu2") or self.score not in ("sigmoid", "softmax"):
            raise ValueError("routed_experts: the kernels know gated experts with silu, ungated experts with relu2, and "
                             "sigmoid or softmax scores")
        if not (1 <= self.top <= self.E) or self.E % self.groups or not (1 <= self.keep <= self.groups) \
                or self.keep * (self.E // self.groups) < self.top:
            raise ValueError(f"routed_experts: experts={self.E} top={self.top} groups={self.groups} keep={self.keep}")
        self.shared = None
        self._ones = []
        self.shared_gate_name = None
        sh = p.get("shared")
        if sh and self.gated:
            self.shared = GatedMLP({"hidden_size": self.hidden, "intermediate_size": int(sh["intermediate_size"]),
                                    "activation": "silu", "gate": sh["gate"], "up": sh["up"], "down": sh["down"]}, prefix, rt)
        elif sh:
            self.shared = PlainMLP({"hidden_size": self.hidden, "intermediate_size": int(sh["intermediate_size"]),
                                    "activation": self.activation, "up": sh["up"], "down": sh["down"]}, prefix, rt)
        if sh:
            self.shared_gate_name = sh.get("token_gate")

    def _expert(self, e: int, key: str) -> str:
        return self.prefix + self.params["expert"].format(e) + self.params[key]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self._name("router"): TensorSpec((self.E, self.hidden))}
        if self.params.get("correction"):
            specs[self._name("correction")] = TensorSpec((self.E,), "norm")
        if self.params.get("router_bias"):
            specs[self._name("router_bias")] = TensorSpec((self.E,), "norm")
        for e in range(self.E):
            if self.gated:
                specs[self._expert(e, "gate")] = TensorSpec((self.ff, self.hidden))
            specs[self._expert(e, "up")] = TensorSpec((self.ff, self.hidden))
            specs[self._expert(e, "down")] = TensorSpec((self.hidden, self.ff))
        if self.shared is not None:
            specs.update(self.shared.tensor_specs())
            if self.shared_gate_name:
                specs[self.prefix + self.shared_gate_name] = TensorSpec((1, self.hidden))
        return specs

    def bind(self, tensors) -> None:
        router = tensors[self._name("router")]
        self.correction = tensors[self._name("correction")].float().contiguous() if self.params.get("correction") else None
        self.router_bias = None
        if self.params.get("router_bias"):
            self.router_bias = tensors[self._name("router_bias")].float().contiguous()      # the routing kernel adds it
        dt = tensors[self._expert(0, "up")].dtype
        self.w_gate = torch.stack([tensors[self._expert(e, "gate")].to(dt) for e in range(self.E)]).contiguous() \
            if self.gated else None
        self.w_up = torch.stack([tensors[self._expert(e, "up")].to(dt) for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")].to(dt) for e in range(self.E)]).contiguous()
        # for many tokens: every expert's gate and up rows interleaved, as the tensor-core product's gated epilogue
        # wants them (a second copy of those rows; steps of few tokens read the plain ones)
        self.w_gate_up = None
        if self.gated and dt == torch.bfloat16 and self.rt.dtype == torch.bfloat16 and self.ff % 16 == 0 and self.hidden % 8 == 0:
            self.w_gate_up = torch.stack([ops.interleave_gate_up(self.w_gate[e], self.w_up[e]) for e in range(self.E)]).contiguous()
        rows = [router]
        self.has_gate = False
        if self.shared is not None:
            self.shared.bind(tensors)
            if self.shared_gate_name:
                rows.append(tensors[self.prefix + self.shared_gate_name].to(router.dtype).reshape(1, -1))
                self.has_gate = True
        # one product gives the router's logits and the shared expert's gate; rows of zeros up to a multiple of 16
        n = self.E + int(self.has_gate)
        rows.append(torch.zeros((-n % 16, self.hidden), dtype=router.dtype, device=router.device))
        self.w_router = torch.cat(rows, dim=0).contiguous()
        # an ungated shared expert: its up rows lie right behind the router's, so that a step of few tokens makes the
        # logits and the shared expert's first product with ONE product (both are read as 32-bit partial sums there);
        # the router and the shared expert keep views of their rows, nothing is stored twice
        self.w_router_up = None
        if isinstance(self.shared, PlainMLP) and self.shared.w_up.dtype == self.w_router.dtype:
            n = self.w_router.shape[0]
            self.w_router_up = torch.cat([self.w_router, self.shared.w_up], dim=0).contiguous()
            self.w_router = self.w_router_up[:n]
            self.shared.w_up = self.w_router_up[n:]

    def kernel_files(self):
        return linear_kernels(self.rt.dtype) + ("moe", "activation")

    def forward(self, x, ctx):
        fused_up = self.w_router_up is not None and x.shape[0] <= FUSED_UP_TOKENS
        # 32-bit sums; the routing itself is 32-bit throughout
        logits = linear_partials(x, self.w_router_up if fused_up else self.w_router)
        idx, weight, gate = ops.moe_route(logits, self.E, self.correction, self.has_gate, self.top, self.groups,
                                          self.keep, self.group_top, self.weight_eps, self.score, self.route_scale,
                                          self.router_bias)
        shared = None
        if self.shared is not None:
            # float32 partial sums [splits, T, hidden]
            shared = self.shared.finish(logits, self.w_router.shape[0]) if fused_up else self.shared.forward(x, ctx)
            if gate is None:
                # the shared expert is added as it is: a gate of ones, made once and kept (no launch in a step); a
                # smaller one that a captured step may still read stays alive beside its successor
                if not self._ones or self._ones[-1].numel() < x.shape[0]:
                    self._ones.append(torch.ones(max(256, 2 * x.shape[0]), dtype=torch.float32, device=x.device))
                gate = self._ones[-1]
        return ops.moe_experts(x, self.w_gate, self.w_up, self.w_down, idx, weight, shared, gate, self.w_gate_up)


register_part("feed_forward", "routed_experts", RoutedExperts)
