"""Attention as a mixer: grouped-query, causal, optionally windowed and soft-capped.

In the order the reference computes it (runtime/src/lib.rs:4483-4496):
q, k, v projections without bias; position encoding of q and k; k and v appended
to the cache; per query ``s = (q.k) * scale``, ``s = cap * tanh(s / cap)`` if a
cap is set, softmax over the visible keys, weighted sum of v
(runtime/cuda/codebook_gemv.cu:240-270); output projection.  Query head ``h``
reads kv head ``h // (num_heads // num_kv_heads)`` (codebook_gemv.cu:244).

Parameters (none is fixed in code): ``hidden_size``, ``num_heads``,
``num_kv_heads``, ``head_dim``, ``scale``, ``softcap`` (None: off), ``window``
(None: every earlier token is visible; W: the last W tokens, the query's own
included), ``position`` (a position-encoding spec) and the four tensor names.
Optional, absent in Gemma-2: ``bias`` (tensor names of biases under the keys
``q``, ``k``, ``v``, ``o``; any subset) and ``q_norm`` / ``k_norm`` (norm specs
applied to every query / key head, over ``head_dim``, before the position
encoding).  What the fused decode kernel can do by itself is declared by
:meth:`Attention.fused_decode`: the plain projection followed by a rotate-half
rotation.  With a bias or a head norm the same steps run as kernels of their
own, so such a mixer is a matter of parameters, not of a change to a kernel.
The reference fixes ``scale = rsqrt(head_dim)`` (codebook_gemv.cu:250) and has
no window (runtime/src/lib.rs:4455).

Three more options serve mixers whose positions do not enter through a rotation
(``position`` of kind "none"); they run in one kernel between the projection and
the attention kernel (``ops.headnorm_kv``), all in 32-bit:

* ``v`` None: there is no v matrix, v is the raw output of the k projection (the cache still
  keeps keys and values, because the keys may be normed and the values are not);
* ``head_unit_norm`` ``{"q": bool, "k": bool, "eps": e}``: every query / key head is
  divided by its root mean square over ``head_dim`` (no weight);
* ``q_temp`` ``{"coef": c, "every": n}``: the query at position p is multiplied by
  ``1 + c * ln(floor((p + 1) / n) + 1)``.

Four more options serve mixers that norm q and k over the WHOLE projection; they
go with a rotation or with none, and run in one kernel between the projection and
the attention kernel (``ops.projnorm_kv``), all in 32-bit:

* ``proj_norm`` ``{"q": name, "k": name, "eps": e}``: q (all heads at once) and k are
  divided by their root mean square and multiplied by a weight of the projection's
  size, before the rotation;
* ``head_temp`` (a tensor name, one number per head): head h's scores are multiplied
  by it (applied to the query, in which the score is linear);
* ``value_dim``: values of another size than the keys.  Keys and values are then
  stored with one padded head size (``ops.attn_padded_head``), zeros in the padding,
  which changes neither a score nor the kept part of the output; the output
  projection gets zero columns to match;
* ``out_gate`` (a tensor name, [heads, hidden]): head h's output is multiplied by
  ``sigmoid(G x)[h]`` before the output projection; its rows ride in the fused
  projection.

Three more options change who sees whom and how the scores become weights; they ride on the same path
(``ops.projnorm_kv``, which then also adds the biases), and their attention kernels are ``ops.attn_mixed_*``:

* ``block`` B (instead of ``window``): the query at position i sees key j iff ``j <= i`` and both lie in the same
  block of B positions, blocks counted from position 0 of the sequence; the cache line is a ring of B rows;
* ``unit_sink``: the softmax denominator also holds ``exp(0)``, a sink without a key and without a value;
* ``talk`` (a tensor name, [heads, heads]): the heads' scores are mixed before the mask and the softmax,
  ``s_h <- sum_g talk[h, g] s_g``.  Scale and ``head_temp`` are folded into the matrix when the weights are bound.

The three projections are fused into one matrix when the weights are bound, so
a step runs one product for q, k and v.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, build_part, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear, linear_partials


class Attention(Mixer):
    graph_safe = True          # every launch depends on device data only
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.window = int(p["window"]) if p.get("window") else None
        if self.n_heads % self.n_kv:
            raise ValueError(f"attention: {self.n_heads} heads cannot share {self.n_kv} kv heads")
        self.position = build_part("position", p["position"], prefix, rt)
        self.qd = self.n_heads * self.hd
        self.kvd = self.n_kv * self.hd
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.bias_names = dict(p.get("bias") or {})
        unknown = set(self.bias_names) - {"q", "k", "v", "o"}
        if unknown:
            raise ValueError(f"attention: 'bias' names {sorted(unknown)}; it knows q, k, v and o")
        self.q_norm = build_part("norm", p["q_norm"], prefix, rt) if p.get("q_norm") else None
        self.k_norm = build_part("norm", p["k_norm"], prefix, rt) if p.get("k_norm") else None
        self.b_qkv: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None
        self.v_from_k = p.get("v", "") is None
        unit = p.get("head_unit_norm") or {}
        self.q_unit, self.k_unit = bool(unit.get("q")), bool(unit.get("k"))
        self.unit_eps = float(unit.get("eps", 0.0))
        temp = p.get("q_temp") or {}
        self.temp_coef = float(temp.get("coef", 0.0))
        self.temp_every = int(temp.get("every", 0)) if self.temp_coef else 0
        if temp and self.temp_coef and self.temp_every < 1:
            raise ValueError(f"attention: q_temp 'every' must be at least 1, got {temp.get('every')!r}")
        self.prepared = self.v_from_k or self.q_unit or self.k_unit or self.temp_every > 0
        if self.prepared and (self.position.rotary_table() != (None, 0) or self.bias_names or self.q_norm or self.k_norm):
            raise ValueError("attention: 'v' None, 'head_unit_norm' and 'q_temp' go with position 'none' and without "
                             "biases or weighted head norms")
        self.vd = int(p.get("value_dim") or self.hd)
        pn = dict(p.get("proj_norm") or {})
        self.proj_norm_names = {key: pn[key] for key in ("q", "k") if pn.get(key)}
        self.proj_norm_eps = float(pn.get("eps", 0.0))
        self.head_temp_name = p.get("head_temp")
        self.out_gate_name = p.get("out_gate")
        self.block = int(p["block"]) if p.get("block") else None
        self.unit_sink = bool(p.get("unit_sink"))
        self.talk_name = p.get("talk")
        self.mixed = bool(self.block or self.unit_sink or self.talk_name)
        if self.block and self.window:
            raise ValueError("attention: 'block' and 'window' exclude each other")
        if self.block is not None and self.block < 1:
            raise ValueError(f"attention: block={self.block} must be positive")
        self.projected = bool(self.proj_norm_names or self.head_temp_name or self.out_gate_name or self.vd != self.hd
                              or self.mixed)
        if self.projected:
            if self.prepared or self.q_norm or self.k_norm or self.softcap:
                raise ValueError("attention: 'proj_norm', 'head_temp', 'value_dim', 'out_gate', 'block', 'unit_sink' and 'talk' "
                                 "go without head norms, a cap, 'v' None, 'head_unit_norm' and 'q_temp'")
            if self.position.rotary_table() is None:
                raise ValueError("attention: 'proj_norm', 'head_temp', 'value_dim' and 'out_gate' go with a rotate-half "
                                 "rotation or with no position encoding")
            # the mixing kernels take any head size; the tensor-core kernels want one of theirs
            self.pad = ops.attn_mixed_padded_head(rt.dtype, self.n_heads, max(self.hd, self.vd)) if self.mixed \
                else ops.attn_padded_head(rt.dtype, max(self.hd, self.vd))
        self.wq_norm = self.wk_norm = self.head_temp = self.w_o_padded = self.mix = self.b_proj = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {
            self._name("q"): TensorSpec((self.qd, self.hidden)),
            self._name("k"): TensorSpec((self.kvd, self.hidden)),
            self._name("o"): TensorSpec((self.hidden, self.n_heads * self.vd)),
        }
        if not self.v_from_k:
            specs[self._name("v")] = TensorSpec((self.n_kv * self.vd, self.hidden))
        for key, n in (("q", self.qd), ("k", self.kvd)):
            if key in self.proj_norm_names:
                specs[self.prefix + self.proj_norm_names[key]] = TensorSpec((n,), "gain")
        if self.head_temp_name:
            specs[self.prefix + self.head_temp_name] = TensorSpec((self.n_heads,), "gain")
        if self.out_gate_name:
            specs[self.prefix + self.out_gate_name] = TensorSpec((self.n_heads, self.hidden))
        if self.talk_name:
            specs[self.prefix + self.talk_name] = TensorSpec((self.n_heads, self.n_heads))
        sizes = {"q": self.qd, "k": self.kvd, "v": self.n_kv * self.vd, "o": self.hidden}
        for key, name in self.bias_names.items():
            specs[self.prefix + name] = TensorSpec((sizes[key],))
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                specs.update(n.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        mats = [tensors[self._name(n)] for n in (("q", "k") if self.v_from_k else ("q", "k", "v"))]
        q = mats[0]
        if self.projected:
            if self.out_gate_name:
                mats.append(tensors[self.prefix + self.out_gate_name])
            n = sum(m.shape[0] for m in mats)
            mats.append(torch.zeros((-n % 16, self.hidden), dtype=q.dtype, device=q.device))     # whole tiles of weight rows
            # short vectors that enter 32-bit arithmetic: kept in 32 bits (exact for what a file stores in 16)
            if "q" in self.proj_norm_names:
                self.wq_norm = tensors[self.prefix + self.proj_norm_names["q"]].float().contiguous()
            if "k" in self.proj_norm_names:
                self.wk_norm = tensors[self.prefix + self.proj_norm_names["k"]].float().contiguous()
            if self.head_temp_name:
                self.head_temp = tensors[self.prefix + self.head_temp_name].float().contiguous()
            if self.mixed:
                # s_h = sum_g talk[h, g] * temp[g] * scale * (q_g . k): one 32-bit matrix
                mix = tensors[self.prefix + self.talk_name].float() if self.talk_name \
                    else torch.eye(self.n_heads, dtype=torch.float32, device=q.device)
                if self.head_temp is not None:
                    mix = mix * self.head_temp[None, :]
                self.mix = (mix * self.scale).contiguous()
            if any(key in self.bias_names for key in "qkv"):
                parts = [tensors[self.prefix + self.bias_names[key]].float() if key in self.bias_names
                         else torch.zeros(m, dtype=torch.float32, device=q.device)
                         for key, m in (("q", self.qd), ("k", self.kvd), ("v", self.n_kv * self.vd))]
                parts.append(torch.zeros(n - sum(x.numel() for x in parts) + (-n % 16), dtype=torch.float32, device=q.device))
                self.b_proj = torch.cat(parts).contiguous()
            w_o = tensors[self._name("o")]
            if self.pad != self.vd:
                wide = torch.zeros((self.hidden, self.n_heads, self.pad), dtype=w_o.dtype, device=w_o.device)
                wide[:, :, :self.vd] = w_o.view(self.hidden, self.n_heads, self.vd)
                w_o = wide.view(self.hidden, self.n_heads * self.pad).contiguous()
            self.w_o_padded = w_o
        dt = q.dtype if all(m.dtype == q.dtype for m in mats) else torch.float32
        self.w_qkv = torch.cat([m.to(dt) for m in mats], dim=0).contiguous()
        self.w_o = self.w_o_padded if self.projected else tensors[self._name("o")]
        self.position.bind(tensors)
        if not self.projected and any(key in self.bias_names for key in "qkv"):
            # one bias row for the fused projection, 32-bit; a projection without a bias of its own gets zeros
            parts = [tensors[self.prefix + self.bias_names[key]].float() if key in self.bias_names
                     else torch.zeros(n, dtype=torch.float32, device=q.device)
                     for key, n in (("q", self.qd), ("k", self.kvd), ("v", self.kvd))]
            self.b_qkv = torch.cat(parts).contiguous()
        if "o" in self.bias_names:
            self.b_o = tensors[self.prefix + self.bias_names["o"]].float().contiguous()
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                n.bind(tensors)

    def fused_decode(self) -> bool:
        """Whether this mixer is what the decode kernel's own prologue computes: the plain q/k/v projection
        (no bias, no head norm), then a rotate-half rotation (or none)."""
        return self.b_qkv is None and self.q_norm is None and self.k_norm is None \
            and self.position.rotary_table() is not None

    def _finish_projection(self, qkv: torch.Tensor, n_q: int, n_kv: int) -> None:
        """Bias and head norms on a freshly projected [tokens, (n_q + 2 n_kv) * head_dim] matrix, in place."""
        if self.b_qkv is not None:
            ops.add_bias(qkv, self.b_qkv[:qkv.shape[1]])
        T = qkv.shape[0]
        for norm, lo, n in ((self.q_norm, 0, n_q), (self.k_norm, n_q * self.hd, n_kv)):
            if norm is not None and n:
                heads = qkv[:, lo:lo + n * self.hd]
                normed = norm.apply(heads.reshape(T * n, self.hd).contiguous(), qkv.dtype)
                heads.copy_(normed.view(T, n * self.hd))

    def _out(self, o: torch.Tensor) -> torch.Tensor:
        part = linear_partials(o, self.w_o)
        if self.b_o is not None:
            ops.add_bias(part[0], self.b_o)
        return part

    def kernel_files(self):
        if self.mixed:
            return linear_kernels(self.rt.dtype) + ("projnorm_kv", "attention_mixed") + (("activation",) if "o" in self.bias_names else ())
        if self.projected:
            fast = ("projnorm_kv",)
            if ops.attn_decode_takes(self.rt.dtype, self.n_heads, self.n_kv, self.pad):
                fast += ("attention_decode",)
            if ops.attn_prefill_tc_takes(self.rt.dtype, self.pad):
                fast += (ops.attn_prefill_tc_lib(self.pad),)
            elif ops.attn_prefill_takes(self.rt.dtype, self.pad):
                fast += (ops.attn_prefill_lib(self.pad),)
            return linear_kernels(self.rt.dtype) + ("attention_simt",) + fast
        fast = ("attention_decode",) if ops.attn_decode_takes(self.rt.dtype, self.n_heads, self.n_kv, self.hd) else ()
        if self.prepared:
            fast += ("headnorm_kv",)
        if self.bias_names:
            fast += ("activation",)
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                fast += tuple(n.kernel_files())
        if ops.attn_prefill_tc_takes(self.rt.dtype, self.hd):
            fast += (ops.attn_prefill_tc_lib(self.hd),)
        elif ops.attn_prefill_takes(self.rt.dtype, self.hd):
            fast += (ops.attn_prefill_lib(self.hd),)
        return linear_kernels(self.rt.dtype) + self.position.kernel_files() + ("attention_simt",) + fast

    def cache_need(self):
        return KVNeed(self.n_kv, self.pad if self.projected else self.hd, self.block or self.window)

    def forward(self, x, ctx, line):
        dt = self.rt.dtype
        if self.projected:
            return self._forward_projected(x, ctx, line)
        if self.prepared:
            return self._forward_prepared(x, ctx, line)
        if line.owner:
            plain = self.b_qkv is None and self.q_norm is None and self.k_norm is None
            if plain and dt == torch.bfloat16 and x.shape[0] <= 128 and ops.gemm_tc_takes(x, self.w_qkv):
                # few tokens: the product comes as split-K partial sums, which the rotation kernel adds up
                part = ops.gemm_tc(x, self.w_qkv, torch.float32, partials=True)
                rotate = self.position.rotary_table()
                if not ctx.is_prefill and self.fused_decode() and ops.attn_decode_rotates(dt, self.n_heads, self.n_kv, self.hd):
                    # decoding: the attention kernel adds them up, rotates and appends to the cache by itself
                    o = ops.attn_decode(part, line.k, line.v, line.page_table, ctx.len_after, self.n_heads, self.n_kv,
                                        self.hd, self.scale, self.softcap, self.window or 0, line.ring_rows,
                                        ctx.len_bucket, ctx.uneven, rotate)
                    return self._out(o)
                qkv = torch.empty(part.shape[1:], dtype=dt, device=x.device)
                self.position.rotate_and_store(qkv, self.n_heads, self.n_kv, ctx, line, store=True, partial=part)
            else:
                qkv = linear(x, self.w_qkv, dt)
                self._finish_projection(qkv, self.n_heads, self.n_kv)
                self.position.rotate_and_store(qkv, self.n_heads, self.n_kv, ctx, line, store=True)
            q = qkv[:, :self.qd]
            k = qkv[:, self.qd:self.qd + self.kvd]
            v = qkv[:, self.qd + self.kvd:]
            if ctx.is_prefill and line.shared:
                ctx.step_kv[line.entry] = (k, v)      # a later call that reads this cache needs them
        else:
            # this call reads another call's cache: only its queries are new
            q = linear(x, self.w_qkv[:self.qd], dt)
            self._finish_projection(q, self.n_heads, 0)
            self.position.rotate_and_store(q, self.n_heads, 0, ctx, line, store=False)
            k, v = ctx.step_kv[line.entry] if ctx.is_prefill else (None, None)
        if ctx.is_prefill:
            o = ops.attn_prefill(q, k, v, ctx.seq_start, ctx.token_seq, self.n_heads, self.n_kv, self.hd,
                                 self.scale, self.softcap, self.window or 0, ctx.max_seq_len, ctx.seq_lens, ctx.memo)
        else:
            o = ops.attn_decode(q, line.k, line.v, line.page_table, ctx.len_after, self.n_heads, self.n_kv,
                                self.hd, self.scale, self.softcap, self.window or 0, line.ring_rows, ctx.len_bucket,
                                ctx.uneven)
        return self._out(o)


    def _forward_prepared(self, x, ctx, line):
        """The path of ``v`` None / ``head_unit_norm`` / ``q_temp``: the projection as 32-bit partial sums, one kernel
        that norms, scales, rounds and fills the cache, then the same attention kernels as every other mixer."""
        dt = self.rt.dtype
        if not line.owner:
            raise NotImplementedError("attention: a prepared mixer that reads another call's cache is not built")
        part = linear_partials(x, self.w_qkv)
        qkv = ops.headnorm_kv(part, self.n_heads, self.n_kv, self.hd, dt, self.q_unit, self.k_unit, self.v_from_k,
                              self.unit_eps, self.temp_coef, self.temp_every, ctx.positions, ctx.token_seq,
                              ctx.len_after, line.k, line.v, line.page_table, line.ring_rows)
        q = qkv[:, :self.qd]
        k = qkv[:, self.qd:self.qd + self.kvd]
        v = qkv[:, self.qd + self.kvd:]
        if ctx.is_prefill:
            o = ops.attn_prefill(q, k, v, ctx.seq_start, ctx.token_seq, self.n_heads, self.n_kv, self.hd,
                                 self.scale, self.softcap, self.window or 0, ctx.max_seq_len, ctx.seq_lens, ctx.memo)
        else:
            o = ops.attn_decode(q, line.k, line.v, line.page_table, ctx.len_after, self.n_heads, self.n_kv,
                                self.hd, self.scale, self.softcap, self.window or 0, line.ring_rows, ctx.len_bucket,
                                ctx.uneven)
        return self._out(o)


    def _forward_projected(self, x, ctx, line):
        """The path of ``proj_norm`` / ``head_temp`` / ``value_dim`` / ``out_gate``: the fused projection as 32-bit partial
        sums, one kernel that norms, weighs, rotates, pads, rounds, fills the cache and takes the gate's sigmoid, then the
        same attention kernels as every other mixer at the padded head size."""
        dt = self.rt.dtype
        if not line.owner:
            raise NotImplementedError("attention: a mixer with a projection-wide norm that reads another call's cache is not built")
        H, G, D = self.n_heads, self.n_kv, self.pad
        inv_freq, rotary = self.position.rotary_table()
        part = linear_partials(x, self.w_qkv)
        qkv, gate = ops.projnorm_kv(part, H, G, self.hd, self.vd, D, dt, self.wq_norm, self.wk_norm, self.proj_norm_eps,
                                    None if self.mixed else self.head_temp, rotary, inv_freq, bool(self.out_gate_name),
                                    ctx.positions, ctx.token_seq, ctx.len_after, line.k, line.v, line.page_table,
                                    line.ring_rows, self.b_proj)
        q = qkv[:, :H * D]
        k = qkv[:, H * D:(H + G) * D]
        v = qkv[:, (H + G) * D:]
        if self.mixed:
            seen = -self.block if self.block else (self.window or 0)
            if ctx.is_prefill:
                o = ops.attn_mixed_prefill(q, k, v, ctx.seq_start, ctx.token_seq, H, G, D, self.mix, seen, self.unit_sink,
                                           ctx.max_seq_len)
            else:
                o = ops.attn_mixed_decode(q, line.k, line.v, line.page_table, ctx.len_after, H, G, D, self.mix, seen,
                                          self.unit_sink, line.ring_rows, ctx.len_bucket)
        elif ctx.is_prefill:
            o = ops.attn_prefill(q, k, v, ctx.seq_start, ctx.token_seq, H, G, D, self.scale, 0.0, self.window or 0,
                                 ctx.max_seq_len, ctx.seq_lens, ctx.memo)
        else:
            o = ops.attn_decode(q, line.k, line.v, line.page_table, ctx.len_after, H, G, D, self.scale, 0.0,
                                self.window or 0, line.ring_rows, ctx.len_bucket, ctx.uneven)
        if gate is not None:
            ops.head_gate(o, gate, H)
        return self._out(o)


register_part("mixer", "attention", Attention)
