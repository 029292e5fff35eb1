"""Fibelix, stated plainly: one slow function per mechanism, in 64-bit floats on the CPU.

This file is the tests' oracle.  It shares no code with the library: it reads a configuration dictionary (the
keys of config.json) and a dictionary of tensors by name, and keeps, per layer, what the tokens it has seen left
behind (keys and values, or latent rows), so that a sequence can be fed in pieces.

Notation: ``W`` is the model's width, ``h`` a sublayer's input [tokens, W], matrices are stored [out, in].

    layer       x <- x + mix(n1(x));  x <- x + ff(n2(x));   n(x) = x / rms(x) * (1 + w)
    attention   q, k, v with biases; the first R dims of every head turned by pos * base^(-2i/R) / factor, pair
                (i, i + R/2); s_g = q_g.k * scale * temp[g]; s'_h = sum_g T[h, g] s_g; key j is seen from i iff
                j <= i and both lie in the same block of `size` positions; p = exp(s') / (1 + sum exp(s'));
                output product with bias
    attention_2 two score maps per head over the same values; softmax each; o = a1 - lam a2 with
                lam = exp(lq1.lk1) - exp(lq2.lk2) + diff; o / rms(o) * (1 - diff); may read another layer's keys
                and values
    latent      c_q = rmsnorm(Dq h) wq;  q = Uq c_q = [plain | rot] per head;  Dkv h = [c' | r],  c = rmsnorm(c') wc;
                k_h = [Uk_h c | r], v_h = Uv_h c;  r and q's rot part turned, pair (2i, 2i+1), frequencies blended
                between f and f / factor, cos and sin times 0.1 ln(factor) + 1; window; softmax; head output times
                sigmoid(G h)[head]; output product
    experts     z = R h + b; the `top` largest z win; weights softmax over the winners' z; expert(h) = D (silu(G h) * U h)
"""
from __future__ import annotations

import math
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


def offset_norm(x, w, eps):
    """RMS norm whose stored weight lies around zero."""
    return x / rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return x / rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------
# positions
# ---------------------------------------------------------------------------

def linear_frequencies(dims: int, base: float, factor: float = 1.0) -> torch.Tensor:
    return torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(dims // 2)], dtype=F)


def blended_frequencies(dims: int, base: float, factor: float, original: float, fast: float, slow: float):
    """Frequencies between f_i (fast-turning dims) and f_i / factor (slow ones), and the factor on cos and sin."""
    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), dims - 1)
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def turn_halves(x, pos, freq):
    """The first 2 len(freq) entries of the last axis, pair (i, i + len(freq)), turned by pos * freq[i]."""
    half = freq.numel()
    if half == 0:
        return x
    a = pos.to(F)[:, None] * freq
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
    u, w = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., 2 * half:]], dim=-1)


def turn_neighbours(x, pos, freq, mult: float = 1.0):
    """The first 2 len(freq) entries of the last axis, pair (2i, 2i + 1), turned by pos * freq[i]; cos and sin
    times ``mult``."""
    half = freq.numel()
    if half == 0:
        return x
    a = pos.to(F)[:, None] * freq
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = (torch.cos(a) * mult).view(shape), (torch.sin(a) * mult).view(shape)
    u, w = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
    out = x.clone()
    out[..., 0:2 * half:2] = u * c - w * s
    out[..., 1:2 * half:2] = w * c + u * s
    return out


def rotation_of(m: dict):
    """(frequencies, factor on cos and sin) of a mixer's ``rot`` entry, or (no frequencies, 1)."""
    rot = m.get("rot")
    if not rot:
        return torch.zeros(0, dtype=F), 1.0
    dims = rot.get("dims", m.get("rot_dim", m["dim"]))
    sc = rot.get("scaling") or {}
    if "original" in sc:
        return blended_frequencies(dims, rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
    return linear_frequencies(dims, rot["base"], sc.get("factor", 1.0)), 1.0


# ---------------------------------------------------------------------------
# who sees whom
# ---------------------------------------------------------------------------

def same_block(qpos, kpos, size: Optional[int]):
    """[queries, keys]: key j is seen from query i iff j <= i and floor(i / size) == floor(j / size)."""
    ok = kpos[None, :] <= qpos[:, None]
    if size:
        ok &= (qpos[:, None] // size) == (kpos[None, :] // size)
    return ok


def in_window(qpos, kpos, size: Optional[int]):
    """[queries, keys]: key j is seen from query i iff 0 <= i - j (< size)."""
    d = qpos[:, None] - kpos[None, :]
    ok = d >= 0
    if size:
        ok &= d < size
    return ok


def softmax_seen(s, ok, extra_one: bool = False):
    """Softmax over the seen keys of every row; ``extra_one``: the denominator also holds exp(0)."""
    s = s.masked_fill(~ok, -math.inf)
    m = s.max(-1, keepdim=True).values
    if extra_one:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if extra_one:
        den = den + torch.exp(-m)
    return e / den


def _mask_size(m):
    return (m.get("mask") or {}).get("size")


# ---------------------------------------------------------------------------
# mixers.  ``past``: a dictionary the function keeps what later tokens need in; ``first_pos``: the position of
# h's first row.  ``rnd`` rounds what a 16-bit engine stores (identity for the oracle proper).
# ---------------------------------------------------------------------------

def mixed_attention(h, m, t, p, first_pos=0, past=None, rnd=same):
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    q = (h @ f64(t[p + "q"]).T + f64(t[p + "q.b"])).view(T, H, D)
    k = (h @ f64(t[p + "k"]).T + f64(t[p + "k.b"])).view(T, G, D)
    v = (h @ f64(t[p + "v"]).T + f64(t[p + "v.b"])).view(T, G, V)
    freq, _ = rotation_of(m)
    q, k, v = rnd(turn_halves(q, pos, freq)), rnd(turn_halves(k, pos, freq)), rnd(v)
    if past is not None:
        if "k" in past:
            k, v = torch.cat([past["k"], k]), torch.cat([past["v"], v])
        past["k"], past["v"] = k, v
    kpos = torch.arange(k.shape[0])
    temp, talk = f64(t[p + "temp"]), f64(t[p + "talk"])
    s = torch.stack([q[:, g] @ k[:, g // (H // G)].T * m["scale"] * temp[g] for g in range(H)])    # [H, T, keys]
    s = torch.einsum("hg,gtj->htj", talk, s)
    ok = same_block(pos, kpos, _mask_size(m))
    out = []
    for g in range(H):
        w = rnd(softmax_seen(s[g], ok, extra_one=True))       # tensor-core kernels round the weights that meet v
        out.append(w @ v[:, g // (H // G)])
    o = rnd(torch.cat(out, dim=-1))
    return o @ f64(t[p + "o"]).T + f64(t[p + "o.b"])


def difference_attention(h, m, t, p, eps, first_pos=0, past=None, rnd=same, source=None):
    """``source``: the ``past`` of the layer whose keys and values this one reads (already holding this step's), or None."""
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    q = rnd(h @ f64(t[p + "q"]).T).view(T, H, 2, D)
    if source is None:
        k = rnd(h @ f64(t[p + "k"]).T).view(T, G, 2, D)
        v = rnd(h @ f64(t[p + "v"]).T).view(T, G, V)
        if past is not None:
            if "k" in past:
                k, v = torch.cat([past["k"], k]), torch.cat([past["v"], v])
            past["k"], past["v"] = k, v
    else:
        k, v = source["k"], source["v"]
    kpos = torch.arange(k.shape[0])
    ok = same_block(pos, kpos, _mask_size(m))
    lam = math.exp(float((f64(t[p + "lq1"]) * f64(t[p + "lk1"])).sum())) \
        - math.exp(float((f64(t[p + "lq2"]) * f64(t[p + "lk2"])).sum())) + m["diff"]
    out = []
    for g in range(H):
        kv = g // (H // G)
        # a 16-bit engine stores each map's output (and its tensor-core kernels the weights that meet v)
        a = [rnd(rnd(softmax_seen(q[:, g, i] @ k[:, kv, i].T * m["scale"], ok)) @ v[:, kv]) for i in range(2)]
        o = a[0] - lam * a[1]
        out.append(o / rms(o, eps) * (1.0 - m["diff"]))
    o = rnd(torch.cat(out, dim=-1))
    return o @ f64(t[p + "o"]).T


def latent_attention(h, m, t, p, eps, first_pos=0, past=None, rnd=same, mapped=False):
    """``mapped``: the same sums in the order in which an engine that reads the cached latents directly makes them (the
    query mapped into the latent's space, the weighted sum of latents mapped back); it matters to ``rnd`` only."""
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    freq, mult = rotation_of(m)
    cq = rnd(plain_norm(h @ f64(t[p + "dq"]).T, f64(t[p + "dq.norm"]), eps))
    q = (cq @ f64(t[p + "uq"]).T).view(T, H, D + R)
    q = rnd(torch.cat([q[..., :D], turn_neighbours(q[..., D:], pos, freq, mult)], dim=-1))
    down = h @ f64(t[p + "dkv"]).T
    c = rnd(plain_norm(down[:, :C], f64(t[p + "dkv.norm"]), eps))
    r = rnd(turn_neighbours(down[:, C:], pos, freq, mult))
    if past is not None:
        if "c" in past:
            c, r = torch.cat([past["c"], c]), torch.cat([past["r"], r])
        past["c"], past["r"] = c, r
    kpos = torch.arange(c.shape[0])
    ok = in_window(pos, kpos, _mask_size(m))
    uk = f64(t[p + "uk"]).view(H, D, C)
    uv = f64(t[p + "uv"]).view(H, V, C)
    gate = torch.sigmoid(h @ f64(t[p + "g"]).T)                     # [T, H]
    out = []
    for g in range(H):
        if mapped:
            s = (rnd(q[:, g, :D] @ uk[g]) @ c.T + q[:, g, D:] @ r.T) * m["scale"]
            w = rnd(softmax_seen(s, ok))
            out.append(rnd(rnd(w @ c) @ uv[g].T) * gate[:, g:g + 1])
            continue
        s = (q[:, g, :D] @ rnd(c @ uk[g].T).T + q[:, g, D:] @ r.T) * m["scale"]
        w = rnd(softmax_seen(s, ok))
        out.append(rnd(w @ rnd(c @ uv[g].T)) * gate[:, g:g + 1])
    o = rnd(torch.cat(out, dim=-1))
    return o @ f64(t[p + "o"]).T


# ---------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------

def route(h, f, t, p):
    """(indices [T, top], weights [T, top], logits [T, experts])."""
    z = h @ f64(t[p + "router"]).T + f64(t[p + "router.b"])
    top = f["router"]["top"]
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    zs = torch.gather(z, 1, order)
    return order, torch.softmax(zs, dim=-1), z


def route_margin(h, f, t, p):
    """Per token: how far the last winner's logit lies above the best loser's (infinite when every expert wins)."""
    z = route(h, f, t, p)[2]
    top = f["router"]["top"]
    zs = torch.sort(z, dim=-1, descending=True).values
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), math.inf, dtype=F)
    return zs[:, top - 1] - zs[:, top]


def experts(h, f, t, p, rnd=same):
    idx, w, _ = route(h, f, t, p)
    out = torch.zeros_like(h)
    for n in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[n, j])
            x = h[n]
            a = rnd(silu(f64(t[f"{p}e{e}.gate"]) @ x) * (f64(t[f"{p}e{e}.up"]) @ x))
            out[n] += w[n, j] * (f64(t[f"{p}e{e}.down"]) @ a)
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------

class Sequence:
    """One sequence fed in pieces: ``feed(tokens)`` returns the logits of the piece's tokens [n, vocab]."""

    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor], rnd=same):
        self.cfg, self.t, self.rnd = cfg, tensors, rnd
        self.n = 0
        self.past: List[dict] = [{} for _ in cfg["layers"]]
        self.streams: List[torch.Tensor] = []          # after the last piece: the stream after every layer
        self.margins: List[torch.Tensor] = []          # per piece: every token's smallest routing margin over the layers

    def feed(self, tokens) -> torch.Tensor:
        cfg, t, rnd = self.cfg, self.t, self.rnd
        eps = cfg["norm"]["eps"]
        x = f64(t["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
        self.streams = []
        margin = torch.full((len(tokens),), math.inf, dtype=F)
        for i, L in enumerate(cfg["layers"]):
            p, m = f"l{i}.", L["mixer"]
            h = rnd(offset_norm(x, f64(t[p + "norm1"]), eps))
            if L["type"] == "attention":
                y = mixed_attention(h, m, t, p + "mix.", self.n, self.past[i], rnd)
            elif L["type"] == "attention_2":
                src = self.past[m["kv_from"]] if m.get("kv_from") is not None else None
                y = difference_attention(h, m, t, p + "mix.", eps, self.n, self.past[i], rnd, src)
            elif L["type"] == "latent_attention":
                y = latent_attention(h, m, t, p + "mix.", eps, self.n, self.past[i], rnd, mapped=self.n > 0)
            else:
                raise ValueError(L["type"])
            x = x + y
            if L.get("mlp") is not None:
                h2 = rnd(offset_norm(x, f64(t[p + "norm2"]), eps))
                margin = torch.minimum(margin, route_margin(h2, L["mlp"], t, p + "mlp."))
                x = x + experts(h2, L["mlp"], t, p + "mlp.", rnd)
            self.streams.append(x.clone())
        self.margins.append(margin)
        self.n += len(tokens)
        return rnd(offset_norm(x, f64(t["final.norm"]), eps)) @ f64(t["embed"]).T


def logits(cfg, tensors, tokens, pieces=None, rnd=same) -> torch.Tensor:
    """Logits of every token of one sequence, fed whole or in the given pieces."""
    seq = Sequence(cfg, tensors, rnd)
    out, at = [], 0
    for n in (pieces or [len(tokens)]):
        out.append(seq.feed(tokens[at:at + n]))
        at += n
    return torch.cat(out)


def forward(cfg, tensors, tokens, rnd=same) -> torch.Tensor:
    return logits(cfg, tensors, tokens, None, rnd)


def routing_margins(cfg, tensors, tokens) -> torch.Tensor:
    seq = Sequence(cfg, tensors)
    seq.feed(tokens)
    return seq.margins[0]


def generate_greedy(cfg, tensors, prompt, n: int) -> List[int]:
    """``n`` tokens after ``prompt``, each the first of the largest logits."""
    seq = Sequence(cfg, tensors)
    nxt = int(torch.argmax(seq.feed(prompt)[-1]))
    out = [nxt]
    while len(out) < n:
        nxt = int(torch.argmax(seq.feed([nxt])[-1]))
        out.append(nxt)
    return out
