"""Fidepel, stated plainly: one slow function per mechanism, in 64-bit floats on the CPU.

This file is the tests' oracle.  It shares no code with the library: it reads a
configuration dictionary (the keys of config.json) and a dictionary of tensors by
name, and keeps, per layer run, the keys and values of the tokens it has seen.

Notation: ``W`` is the model's width, ``h`` a sublayer's input [tokens, W], all
matrices are stored [out, in].

    layer      h = x / rms(x) * g            (g one number);  x <- x + m (mix(h) + ff(h))
    attention  q, k RMS-normed over the whole projection (weights the projection's size), then split into
               heads; the first R dims of every head turned by pos * base^(-2i/R) / factor, pair (i, i + R/2);
               score = q.k * scale * temp[head]; key j is seen from i iff 0 <= i - j < window; softmax;
               head output times sigmoid(G h)[head]; output product
    experts    s = softmax(R h); a group's score is its largest s; only experts of the `keep` best groups can
               be chosen; the `top` largest s win; weights s / (sum + 1e-20) * router scale;
               expert(h) = D relu(U h)^2; plus the shared expert of the same form for every token
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

F = torch.float64


def f64(t: torch.Tensor) -> torch.Tensor:
    return t.to(F)


def same(x):
    return x


def to_bf16(x: torch.Tensor) -> torch.Tensor:
    """What a 16-bit engine stores: the value rounded to bfloat16 (used only to size the tests' tolerances)."""
    return x.to(torch.bfloat16).to(F)


def rms(x, eps):
    return torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return x / rms(x, eps) * g.reshape(())


def rms_norm(x, w, eps):
    return x / rms(x, eps) * w


def relu2(z):
    return torch.relu(z) ** 2


def rotate_half(x, pos, dims: int, base: float, factor: float = 1.0):
    """The first ``dims`` entries of the last axis, pair (i, i + dims/2), turned by pos * base^(-2i/dims) / factor."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(half)], dtype=F)
    a = pos.to(F)[:, None] * f
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., dims:]], dim=-1)


def visible(qpos, kpos, window: Optional[int]):
    """[queries, keys]: key j is seen from query i iff 0 <= i - j (< window)."""
    d = qpos[:, None] - kpos[None, :]
    ok = d >= 0
    if window:
        ok &= d < window
    return ok


def attention(h, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float, first_pos: int = 0, past=None, rnd=same):
    """Windowed attention over one sequence.  ``past`` = (keys, values) of the earlier tokens, all of them (the window is
    applied here, by position)."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    base = float(rot.get("base", 10000.0))
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rms_norm(h @ t[p + "q"].T, t[p + "q.norm"], eps).view(T, H, D)
    k = rms_norm(h @ t[p + "k"].T, t[p + "k.norm"], eps).view(T, G, D)
    v = rnd(h @ t[p + "v"].T).view(T, G, V)
    q = rnd(rotate_half(q, pos, dims, base, factor))
    k = rnd(rotate_half(k, pos, dims, base, factor))
    if past is not None:
        k, v = torch.cat([past[0], k]), torch.cat([past[1], v])
    n = k.shape[0]
    rep = H // G
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)          # head i reads kv head i // rep
    s = torch.einsum("thd,nhd->htn", q, kk) * float(m["scale"]) * t[p + "temp"][:, None, None]
    window = (m.get("mask") or {}).get("size")
    s = s.masked_fill(~visible(pos, torch.arange(n), window)[None], float("-inf"))
    w = torch.softmax(s, dim=-1)
    o = torch.einsum("htn,nhv->thv", rnd(w), vv)                 # tensor-core kernels round the weights that meet v
    o = o * torch.sigmoid(h @ t[p + "g"].T)[:, :, None]
    return rnd(o.reshape(T, H * V)) @ t[p + "o"].T, (k, v)


MARGINS = None          # a list to collect, per router call, every token's smallest margin (see route)


def route(h, r: dict, t: Dict[str, torch.Tensor], p: str):
    """(chosen experts [tokens, top], their weights [tokens, top]).  If MARGINS is a list, also appends [tokens]: how far
    the choice was from going another way (relative lead of the last winner over the best loser, and of the last kept
    group over the best group left out)."""
    E, top = r["experts"], r["top"]
    z = h @ t[p + "router"].T
    s = torch.softmax(z, dim=-1)
    choice = s
    margin = torch.full((h.shape[0],), float("inf"), dtype=F)
    g = r.get("groups")
    if g and g["count"] > 1:
        per = E // g["count"]
        grouped = s.view(-1, g["count"], per)
        gs = grouped.max(-1).values
        keep = gs.topk(g["keep"], dim=-1).indices
        if g["keep"] < g["count"]:
            both = gs.topk(g["keep"] + 1, dim=-1).values
            margin = torch.log(both[:, -2] / both[:, -1])
        ok = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, keep, True)
        choice = grouped.masked_fill(~ok[..., None], float("-inf")).reshape(-1, E)
    idx = choice.topk(top, dim=-1).indices
    if top < E:
        both = choice.topk(top + 1, dim=-1).values
        lead = torch.log(both[:, -2] / both[:, -1].clamp_min(1e-300))
        margin = torch.minimum(margin, lead)
    if MARGINS is not None:
        MARGINS.append(margin)
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))


def expert(h, up, down, rnd=same):
    return rnd(relu2(h @ up.T)) @ down.T


def moe(h, mlp: dict, t: Dict[str, torch.Tensor], p: str, rnd=same):
    idx, w = route(h, mlp["router"], t, p)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=F)
    for i in range(h.shape[0]):
        for j, e in enumerate(idx[i].tolist()):
            q = f"{p}e{e}."
            out[i] += w[i, j] * expert(h[i:i + 1], t[q + "up"], t[q + "down"], rnd)[0]
    if mlp.get("shared"):
        out = out + expert(h, t[p + "shared.up"], t[p + "shared.down"], rnd)
    return out


def routing_margins(cfg: dict, tensors, ids) -> torch.Tensor:
    """Per position: the smallest margin of any of its routing decisions (infinite for a model without experts)."""
    global MARGINS
    MARGINS = []
    try:
        forward(cfg, tensors, ids)
        out = torch.full((len(ids),), float("inf"), dtype=F)
        for m in MARGINS:
            out = torch.minimum(out, m)
        return out
    finally:
        MARGINS = None


def schedule(cfg: dict) -> List[int]:
    """The layer runs in order (a repeated span names its layers once per pass)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


class Plain:
    """One sequence, fed in pieces: ``feed(tokens)`` returns (logits of these tokens, stream after every layer run)."""

    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor], rnd=same):
        self.cfg = cfg
        self.rnd = rnd
        self.t = {k: f64(v) for k, v in tensors.items()}
        self.runs = schedule(cfg)
        self.memory = [None] * len(self.runs)
        self.n = 0

    def feed(self, tokens):
        cfg, t, rnd = self.cfg, self.t, self.rnd
        eps = float(cfg["norm"]["eps"])
        mult = float(cfg.get("residual_mult", 1.0))
        x = t["embed"][torch.as_tensor(tokens)].clone()
        after = []
        for r, i in enumerate(self.runs):
            L = cfg["layers"][i]
            p = f"l{i}."
            h = rnd(scalar_norm(x, t[p + "norm1"], eps))
            if L["type"] != "attention":
                raise ValueError(L["type"])
            y, self.memory[r] = attention(h, L["mixer"], t, p + "mix.", eps, self.n, self.memory[r], rnd)
            if L.get("mlp"):
                y = y + moe(h, L["mlp"], t, p + "mlp.", rnd)
            x = x + mult * y
            after.append(x.clone())
        self.n += len(tokens)
        z = rnd(scalar_norm(x, t["final.norm"], eps)) @ t["head"].T
        return z, torch.stack(after)


def forward(cfg: dict, tensors, ids, rnd=same) -> torch.Tensor:
    """Logits of a whole sequence, [tokens, vocab]."""
    return Plain(cfg, tensors, rnd).feed(list(ids))[0]


def forward_stepwise(cfg: dict, tensors, ids, first: int = 1) -> torch.Tensor:
    """The same logits, from ``first`` tokens at once and then one token at a time."""
    m = Plain(cfg, tensors)
    out = [m.feed(list(ids[:first]))[0]] + [m.feed([t])[0] for t in ids[first:]]
    return torch.cat(out)


def generate_greedy(cfg: dict, tensors, prompt, n_new: int) -> List[int]:
    m = Plain(cfg, tensors)
    z = m.feed(list(prompt))[0]
    out = []
    for _ in range(n_new):
        out.append(int(z[-1].argmax()))
        z = m.feed([out[-1]])[0]
    return out
