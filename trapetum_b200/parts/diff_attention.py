"""Difference attention: every head takes two softmax attentions over the same values and subtracts them.

With ``H`` query heads, ``G`` key/value heads (query head h reads kv head ``h // (H / G)``), per-head and per-map
query/key size ``dim`` and value size ``value_dim``:

* ``q = W_q h`` has ``H * 2 * dim`` numbers, laid out head by head as ``[map 1 | map 2]``; ``k = W_k h`` has
  ``G * 2 * dim`` laid out the same way; ``v = W_v h`` has ``G * value_dim``.  No biases, no position encoding;
* per map m: ``a_m = softmax_j((q_m . k_m) * scale) v`` over the keys the query sees;
* ``o = a_1 - lam * a_2`` with ``lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` (four learned vectors of ``dim``
  numbers, one number for the whole layer), then ``o / sqrt(mean(o^2) + eps)`` over the head's values (no weight),
  times ``1 - diff``; output product over the heads side by side.

Who sees whom: ``block`` B: key j from query i iff ``j <= i`` and both lie in the same block of B positions, blocks
counted from position 0 of the sequence; ``window`` W: iff ``0 <= i - j < W``; neither: every earlier key.

How it runs on the framework's attention kernels: a map is an attention head of its own whose query is padded with
zeros where the other map's numbers lie (``[q_1 | 0]`` and ``[0 | q_2]``), against keys ``[k_1 | k_2]`` as the
projection gives them.  That is ``2 H`` query heads over ``G`` kv heads of ``2 * dim`` numbers, which every kernel
takes; the zeros are rows of zeros in the bound query matrix.  A prompt's blocks are independent causal sequences,
so a step of whole prompts hands the kernels the blocks' starts instead of the sequences'.  The pairs are folded by
``ops.head_difference`` in 32-bit.

A layer may read another layer's keys and values (the schedule's ``cache_of``): it then has no k and v matrices
(``k`` and ``v`` None), makes only its queries and attends over the owner's cache line with its own mask.  The owner
keeps every key (no ring) when ``keep_all`` is set, which an owner must be told if a reader's mask reaches farther
than its own.

Parameters (none is fixed in code): ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``dim``, ``value_dim``,
``scale``, ``diff``, ``eps``, ``block`` / ``window``, ``keep_all`` and the tensor names ``q``, ``k``, ``v``, ``o``, ``lq1``,
``lk1``, ``lq2``, ``lk2``.
"""
from __future__ import annotations

import math
from typing import Dict

import numpy as np
import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear_partials


def block_sequences(ctx, block: int):
    """A step of whole prompts whose sequences are cut into blocks of ``block`` positions: (first row of every block
    int32 [blocks + 1], block of every token int32 [tokens], the blocks' lengths, the longest).  Kept per step."""
    key = ("block_sequences", block)
    if key not in ctx.memo:
        starts, lens, tok = [0], [], []
        for n in ctx.seq_lens:
            for lo in range(0, n, block):
                m = min(block, n - lo)
                tok.extend([len(lens)] * m)
                lens.append(m)
                starts.append(starts[-1] + m)
        dev = ctx.positions.device
        both = torch.from_numpy(np.asarray(starts + tok, dtype=np.int32)).to(dev)
        ctx.memo[key] = (both[:len(starts)], both[len(starts):], lens, max(lens))
    return ctx.memo[key]


class DiffAttention(Mixer):
    graph_safe = True          # every launch depends on device data only

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.G = int(p["num_kv_heads"])
        self.dim = int(p["dim"])
        self.vd = int(p.get("value_dim") or self.dim)
        self.scale = float(p["scale"])
        self.diff = float(p["diff"])
        self.eps = float(p["eps"])
        self.block = int(p["block"]) if p.get("block") else None
        self.window = int(p["window"]) if p.get("window") else None
        self.keep_all = bool(p.get("keep_all"))
        self.reader = p.get("k") is None
        if self.H % self.G:
            raise ValueError(f"diff_attention: {self.H} heads cannot share {self.G} kv heads")
        if self.block and self.window:
            raise ValueError("diff_attention: 'block' and 'window' exclude each other")
        # one head size for the padded queries, the keys [k_1 | k_2] and the values
        self.D = ops.attn_padded_head(rt.dtype, max(2 * self.dim, self.vd))
        self.lam = 0.0

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self._name("q"): TensorSpec((self.H * 2 * self.dim, self.hidden)),
                 self._name("o"): TensorSpec((self.hidden, self.H * self.vd))}
        if not self.reader:
            specs[self._name("k")] = TensorSpec((self.G * 2 * self.dim, self.hidden))
            specs[self._name("v")] = TensorSpec((self.G * self.vd, self.hidden))
        for key in ("lq1", "lk1", "lq2", "lk2"):
            specs[self._name(key)] = TensorSpec((self.dim,), "norm")
        return specs

    def bind(self, tensors) -> None:
        H, G, dim, D = self.H, self.G, self.dim, self.D
        wq = tensors[self._name("q")]
        dt, dev = wq.dtype, wq.device
        # query head (h, m) is [q_1 | 0] or [0 | q_2]: rows of zeros where the other map's numbers would lie
        q4 = wq.view(H, 2, dim, self.hidden)
        wide = torch.zeros((H, 2, 2 * dim, self.hidden), dtype=dt, device=dev)
        wide[:, 0, :dim] = q4[:, 0]
        wide[:, 1, dim:] = q4[:, 1]
        mats = [wide.view(H * 4 * dim, self.hidden)]
        if not self.reader:
            mats += [tensors[self._name("k")].to(dt), tensors[self._name("v")].to(dt)]
        n = sum(m.shape[0] for m in mats)
        mats.append(torch.zeros((-n % 16, self.hidden), dtype=dt, device=dev))
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        wo = tensors[self._name("o")]
        wo_p = torch.zeros((self.hidden, H, D), dtype=wo.dtype, device=dev)
        wo_p[:, :, :self.vd] = wo.view(self.hidden, H, self.vd)
        self.w_o = wo_p.view(self.hidden, H * D).contiguous()
        f = {key: tensors[self._name(key)].float() for key in ("lq1", "lk1", "lq2", "lk2")}
        # one number for the layer, 32-bit
        lam = torch.exp((f["lq1"] * f["lk1"]).sum()) - torch.exp((f["lq2"] * f["lk2"]).sum()) + torch.tensor(self.diff, dtype=torch.float32)
        self.lam = float(lam)

    def kernel_files(self):
        fast = ("projnorm_kv", "attention_simt")
        if ops.attn_decode_takes(self.rt.dtype, 2 * self.H, self.G, self.D):
            fast += ("attention_decode",)
        if ops.attn_prefill_tc_takes(self.rt.dtype, self.D):
            fast += (ops.attn_prefill_tc_lib(self.D),)
        elif ops.attn_prefill_takes(self.rt.dtype, self.D):
            fast += (ops.attn_prefill_lib(self.D),)
        return linear_kernels(self.rt.dtype) + fast

    def cache_need(self):
        if self.reader:
            return None
        # a line that keeps the last `window` rows is a ring; blocks are read by the decode kernels from a line that
        # keeps every key
        return KVNeed(self.G, self.D, None if (self.keep_all or self.block) else self.window)

    def forward(self, x, ctx, line):
        dt = self.rt.dtype
        H2, G, D = 2 * self.H, self.G, self.D
        own = line.owner
        if own == self.reader:
            raise ValueError("diff_attention: a layer without k and v matrices reads another call's cache, and only such a layer does")
        part = linear_partials(x, self.w_qkv)
        qkv, _ = ops.projnorm_kv(part, H2, G if own else 0, 2 * self.dim, self.vd, D, dt, None, None, 0.0, None, 0, None,
                                 False, ctx.positions, ctx.token_seq, ctx.len_after, line.k if own else None,
                                 line.v if own else None, line.page_table if own else None, line.ring_rows if own else 0)
        q = qkv[:, :H2 * D]
        if ctx.is_prefill:
            if own:
                k, v = qkv[:, H2 * D:(H2 + G) * D], qkv[:, (H2 + G) * D:]
                if line.shared:
                    ctx.step_kv[line.entry] = (k, v)          # a later call that reads this cache needs them
            else:
                k, v = ctx.step_kv[line.entry]
            if self.block:
                starts, token_block, lens, longest = block_sequences(ctx, self.block)
                o = ops.attn_prefill(q, k, v, starts, token_block, H2, G, D, self.scale, 0.0, 0, longest, lens, ctx.memo)
            else:
                o = ops.attn_prefill(q, k, v, ctx.seq_start, ctx.token_seq, H2, G, D, self.scale, 0.0, self.window or 0,
                                     ctx.max_seq_len, ctx.seq_lens, ctx.memo)
        else:
            seen = -self.block if self.block else (self.window or 0)
            bucket = ctx.len_bucket
            if seen and not line.ring_rows:
                # what a query reaches, rounded up to whole pages and a power of two: launch shapes may depend on it
                bucket = min(bucket, 1 << max(6, math.ceil(math.log2(abs(seen) + ops.PAGE_ROWS))))
            o = ops.attn_decode(q, line.k, line.v, line.page_table, ctx.len_after, H2, G, D, self.scale, 0.0, seen,
                                line.ring_rows, bucket, ctx.uneven)
        o = ops.head_difference(o, self.H, D, self.vd, self.lam, self.eps, 1.0 - self.diff)
        return linear_partials(o, self.w_o)


register_part("mixer", "diff_attention", DiffAttention)
