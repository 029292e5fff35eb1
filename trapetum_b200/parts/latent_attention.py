"""Latent attention: causal softmax attention whose keys and values are made from one cached latent per token.

With ``H`` heads, per head ``plain_dim`` unrotated and ``rot_dim`` rotated query/key dims, ``value_dim`` value
dims and a latent of ``kv_rank`` numbers:

* ``q = W_q h`` laid out head by head as ``[plain | rot]``; ``W_dkv h`` gives ``kv_rank + rot_dim`` numbers: the first
  ``kv_rank``, RMS-normed times a weight, are the latent ``c``; the rest are ONE rotated key part ``r`` for all heads;
* per head ``k = [W_uk c | r]``, ``v = W_uv c``; the rotation (rotate-half pairing over the first ``rotary_dims`` of
  the rotated part, angle = position x theta^(-2i / rotary_dims)) turns q's rotated part and ``r``, never v;
* score = ``q . k * scale``; causal; the softmax denominator also holds ``exp(sink_h)``, a learned number per head
  that has no key and no value;
* output product ``W_o`` over the concatenated heads.

Only ``[c | r]`` is cached: one row of ``kv_rank + rot_dim`` numbers per token in the paged cache (a key pool
without a value pool).  A step of whole prompts makes every head's keys and values from the step's rows with one
product (the matrix that does it also copies ``r`` into every head: a row of it holds a single one) and runs
the framework's prefill attention; a step of one token each maps the queries into the latent's space instead
(``q' = [W_uk^T q_plain | q_rot]``), so that all heads read the same cached rows, and maps the weighted sum of
latents back through ``W_uv``.  Both are the same function of the same cached rows.

32-bit: the down projection's sums, the norm of the latent, angles, sines and cosines, scores and softmax.

Parameters (none is fixed in code): ``hidden_size``, ``heads``, ``plain_dim``, ``rot_dim``, ``value_dim``,
``kv_rank``, ``scale``, ``rotary_dims``, ``theta``, ``eps`` and the tensor names ``q``, ``dkv``, ``dkv_norm``,
``uk``, ``uv``, ``o``, ``sink`` (None: a plain softmax).

Optional:

* ``q_latent`` ``{"rank", "down", "norm", "up"}`` (instead of ``q``): the queries go through a latent of their own,
  ``c_q = rmsnorm(W_down h) * norm`` (the layer's eps), ``q = W_up c_q``; the down product rides with ``dkv``'s;
* ``rotary`` ``{"dims", "base", "scaling", "pairing"}`` (instead of ``rotary_dims`` / ``theta``): ``scaling`` as
  :func:`~trapetum_b200.parts.rope.rotary_frequencies` takes it; ``pairing`` "halves" (i, i + dims/2) or "neighbours"
  (2i, 2i + 1).  Neighbours are a matter of the weights' row order: the rows that make the rotated numbers of q and
  of ``r`` are sorted evens first when the weights are bound, which turns the pairing into halves and changes no
  dot product.  The factor that a blended scaling puts on cos and sin is applied twice to ``r`` and not to q;
* ``window`` W: the query at position i sees j iff ``0 <= i - j < W``; the cache line is then a ring;
* ``out_gate`` (a tensor name, [heads, hidden]): head h's output times ``sigmoid(G h)[h]``; its rows ride with ``dkv``'s.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear, linear_partials
from .rope import rotary_frequencies


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class LatentAttention(Mixer):
    graph_safe = True          # every launch depends on device data only

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["heads"])
        self.D = int(p["plain_dim"])
        self.R = int(p["rot_dim"])
        self.V = int(p["value_dim"])
        self.C = int(p["kv_rank"])
        self.scale = float(p["scale"])
        rot = p.get("rotary")
        self.rot_dims = int(rot["dims"]) if rot else int(p.get("rotary_dims", self.R))
        self.theta = float(rot["base"]) if rot else float(p["theta"])
        self.neighbours = bool(rot) and rot.get("pairing", "halves") == "neighbours"
        if rot and rot.get("pairing", "halves") not in ("halves", "neighbours"):
            raise ValueError(f"latent_attention: pairing '{rot.get('pairing')}' is neither 'halves' nor 'neighbours'")
        self.eps = float(p["eps"])
        self.window = int(p["window"]) if p.get("window") else None
        self.q_latent = dict(p["q_latent"]) if p.get("q_latent") else None
        self.Q = int(self.q_latent["rank"]) if self.q_latent else 0
        self.out_gate_name = p.get("out_gate")
        if self.rot_dims % 2 or not (0 <= self.rot_dims <= self.R):
            raise ValueError(f"latent_attention: rotary_dims {self.rot_dims} must be even and at most rot_dim {self.R}")
        # the prefill kernels want one head size for q, k and v: the larger of the two, a multiple of 16; the
        # padding is zero columns of the matrices below, so it changes no sum
        self.hd = _round_up(max(self.D + self.R, self.V), 16)
        if rt.dtype == torch.bfloat16:
            # the tcgen05 kernel takes 64, 128 and 256: more padding, a faster kernel
            self.hd = next((n for n in (64, 128, 256) if n >= self.hd), self.hd)
        self.has_sink = p.get("sink") is not None
        self.rot_mult = 1.0
        if rot:
            self._inv_freq_cpu, self.rot_mult = rotary_frequencies(self.rot_dims, self.theta, rot.get("scaling"))
        else:
            idx = torch.arange(0, self.rot_dims, 2, dtype=torch.float32)
            self._inv_freq_cpu = 1.0 / (torch.tensor(self.theta, dtype=torch.float32) ** (idx / max(self.rot_dims, 1)))

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {
            self._name("dkv"): TensorSpec((self.C + self.R, self.hidden)),
            self._name("dkv_norm"): TensorSpec((self.C,), "gain"),
            self._name("uk"): TensorSpec((self.H * self.D, self.C)),
            self._name("uv"): TensorSpec((self.H * self.V, self.C)),
            self._name("o"): TensorSpec((self.hidden, self.H * self.V)),
        }
        if self.has_sink:
            specs[self._name("sink")] = TensorSpec((self.H,), "norm")
        if self.q_latent:
            ql = self.q_latent
            specs[self.prefix + ql["down"]] = TensorSpec((self.Q, self.hidden))
            specs[self.prefix + ql["norm"]] = TensorSpec((self.Q,), "gain")
            specs[self.prefix + ql["up"]] = TensorSpec((self.H * (self.D + self.R), self.Q))
        else:
            specs[self._name("q")] = TensorSpec((self.H * (self.D + self.R), self.hidden))
        if self.out_gate_name:
            specs[self.prefix + self.out_gate_name] = TensorSpec((self.H, self.hidden))
        return specs

    def bind(self, tensors) -> None:
        H, D, R, V, C, hd = self.H, self.D, self.R, self.V, self.C, self.hd
        wq = tensors[self.prefix + self.q_latent["up"]] if self.q_latent else tensors[self._name("q")]
        dt, dev = wq.dtype, wq.device
        q_in = wq.shape[1]
        # the order in which the rotated numbers are made: neighbours (2i, 2i + 1) become halves (i, i + dims/2)
        order = torch.arange(R, device=dev)
        if self.neighbours:
            order = torch.cat([torch.arange(0, self.rot_dims, 2, device=dev), torch.arange(1, self.rot_dims, 2, device=dev),
                               torch.arange(self.rot_dims, R, device=dev)])
        # queries head by head as [rot | plain | zeros]: the rotation kernel turns the FIRST dims of a head, and a dot
        # product does not care in which order q and k list their dims as long as they agree
        q3 = wq.view(H, D + R, q_in)
        wq_p = torch.zeros((H, hd, q_in), dtype=dt, device=dev)
        wq_p[:, :R] = q3[:, D:][:, order]
        wq_p[:, R:R + D] = q3[:, :D]
        self.w_q = wq_p.view(H * hd, q_in).contiguous()
        w_dkv = tensors[self._name("dkv")]
        if self.neighbours:
            w_dkv = torch.cat([w_dkv[:C], w_dkv[C:][order]], dim=0)
        # what rides with the down projection: the queries' latent and the heads' gates, rows of zeros up to 16
        rows = [w_dkv]
        self.w_cq_norm = None
        if self.q_latent:
            rows.append(tensors[self.prefix + self.q_latent["down"]].to(w_dkv.dtype))
            self.w_cq_norm = tensors[self.prefix + self.q_latent["norm"]].float().contiguous()
        if self.out_gate_name:
            rows.append(tensors[self.prefix + self.out_gate_name].to(w_dkv.dtype))
        if len(rows) > 1:
            n = sum(r.shape[0] for r in rows)
            rows.append(torch.zeros((-n % 16, self.hidden), dtype=w_dkv.dtype, device=dev))
        self.w_dkv = torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else w_dkv.contiguous()
        self.w_c_norm = tensors[self._name("dkv_norm")].float().contiguous()
        uk = tensors[self._name("uk")].to(dt).view(H, D, C)
        uv = tensors[self._name("uv")].to(dt).view(H, V, C)
        # keys and values of every head from a cached row [c | r]: k_h = [r | Uk_h c | 0], v_h = [Uv_h c | 0]
        up = torch.zeros((2, H, hd, C + R), dtype=dt, device=dev)
        up[0, :, :R, C:] = torch.eye(R, dtype=dt, device=dev)
        up[0, :, R:R + D, :C] = uk
        up[1, :, :V, :C] = uv
        self.w_up = up.view(2 * H * hd, C + R).contiguous()
        # a query in the latent's space: q'_h = [Uk_h^T q_plain | q_rot] from a head laid out [rot | plain | 0]
        qmap = torch.zeros((H, C + R, hd), dtype=dt, device=dev)
        qmap[:, :C, R:R + D] = uk.transpose(1, 2)
        qmap[:, C:, :R] = torch.eye(R, dtype=dt, device=dev)
        self.w_qmap = qmap.contiguous()
        # and a weighted sum of latents back into a head's values: [Uv_h ; 0]
        vmap = torch.zeros((H, hd, C), dtype=dt, device=dev)
        vmap[:, :V] = uv
        self.w_vmap = vmap.contiguous()
        wo = tensors[self._name("o")]
        wo_p = torch.zeros((self.hidden, H, hd), dtype=wo.dtype, device=dev)
        wo_p[:, :, :V] = wo.view(self.hidden, H, V)
        self.w_o = wo_p.view(self.hidden, H * hd).contiguous()
        self.sink = tensors[self._name("sink")].float().contiguous() if self.has_sink else None
        self.inv_freq = self._inv_freq_cpu.to(dev)

    def kernel_files(self):
        fast = ()
        if ops.attn_prefill_tc_takes(self.rt.dtype, self.hd):
            fast = (ops.attn_prefill_tc_lib(self.hd),)
        elif ops.attn_prefill_takes(self.rt.dtype, self.hd):
            fast = (ops.attn_prefill_lib(self.hd),)
        return linear_kernels(self.rt.dtype) + ("rope_kv", "attention_latent", "attention_simt") + fast \
            + (("projnorm_kv",) if self.out_gate_name else ())

    def cache_need(self):
        return KVNeed(1, self.C + self.R, self.window, values=False)

    def forward(self, x, ctx, line):
        dt = self.rt.dtype
        H, C, R, hd = self.H, self.C, self.R, self.hd
        if not line.owner:
            raise NotImplementedError("latent_attention: reading another call's cache is not built")
        part = linear_partials(x, self.w_dkv)             # 32-bit sums: they enter a norm and a rotation
        gate = None
        if self.q_latent or self.out_gate_name:
            rows, cq, gate = ops.latent_rows(part, self.w_c_norm, self.eps, self.inv_freq, self.rot_dims, C, R, ctx.positions,
                                             ctx.token_seq, line.k, line.page_table, dt, line.ring_rows, ctx.len_after,
                                             self.rot_mult * self.rot_mult, self.w_cq_norm,
                                             H if self.out_gate_name else 0)
        else:
            cq = None
            rows = ops.latent_rows(part, self.w_c_norm, self.eps, self.inv_freq, self.rot_dims, C, R, ctx.positions,
                                   ctx.token_seq, line.k, line.page_table, dt, line.ring_rows, ctx.len_after,
                                   self.rot_mult * self.rot_mult)
        # the queries: 32-bit sums in, rotated and rounded once
        q_part = linear_partials(cq if self.q_latent else x, self.w_q)
        q = torch.empty(q_part.shape[1:], dtype=dt, device=x.device)
        ops.rope_kv(q, H, 0, hd, self.rot_dims, self.inv_freq if self.rot_dims else None, ctx.positions, ctx.token_seq,
                    ctx.len_after, None, None, None, 0, q_part)
        if ctx.is_prefill:
            kv = linear(rows, self.w_up, dt)              # [T, 2 H hd]: every head's keys, then every head's values
            o = ops.attn_prefill_sink(q, kv[:, :H * hd], kv[:, H * hd:], ctx.seq_start, ctx.token_seq, H, hd, self.scale,
                                      self.sink, ctx.max_seq_len, ctx.seq_lens, self.window or 0)
        else:
            ql = ops.head_linear(q, self.w_qmap, H)       # [B, H (C + R)]
            ol = ops.latent_decode(ql, line.k, line.page_table, ctx.len_after, self.sink, H, C, R, self.scale,
                                   ctx.len_bucket, self.window or 0, line.ring_rows)
            o = ops.head_linear(ol, self.w_vmap, H)       # [B, H hd]
        if gate is not None:
            ops.head_gate(o, gate, H)
        return linear_partials(o, self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
