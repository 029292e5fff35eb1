"""Shared pieces of the Fibelix tests: small configurations made up here, model folders with random weights drawn
here (not by the library), and tolerances taken from the plain implementation alone."""
import math

import torch

import plain_fibelix as plain
from lofirax_util import position_errors, prompts, worst_ratio, write_folder  # noqa: F401  (the tests import them from here)


def rot(dims, base, factor=None, blend=None):
    """``blend`` = (original, fast, slow)."""
    r = {"dims": dims, "base": base}
    if factor is not None:
        r["scaling"] = {"factor": factor}
        if blend:
            r["scaling"].update({"original": blend[0], "fast": blend[1], "slow": blend[2]})
    return r


def mixed(heads, kv_heads, dim, vdim, scale, size=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if rot:
        m["rot"] = rot
    return "attention", m


def difference(heads, kv_heads, dim, vdim, scale, diff, size=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if size:
        m["mask"] = {"size": size}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "attention_2", m


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, size=None, rot=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if rot:
        m["rot"] = rot
    return "latent_attention", m


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(vocab, width, layers, eps=1e-5):
    return {"architecture": "Fibelix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{"type": t, "mixer": m, "mlp": f} for (t, m), f in layers]}


# A: small and odd-shaped.  Blocks of 5 and 33, a window of 7; as many kv heads as heads in one layer and fewer in
#    others; values wider and narrower than keys; half of a head rotated without scaling; a blend of frequencies
#    whose ramp lies inside the table; a reader whose blocks are larger than its owner's; a layer without feed-forward;
#    one expert chosen.
CFG_A = config(150, 48, [
    (mixed(3, 3, 8, 12, 0.4, size=5, rot=rot(4, 100.0)), moe(4, 1, 24)),
    (difference(2, 1, 8, 12, 0.3, 0.3, size=33), moe(6, 3, 16)),
    (latent(2, 8, 4, 12, 16, 24, 0.3, size=7, rot=rot(4, 1000.0, 2.0, (16, 4.0, 1.0))), None),
    (difference(2, 1, 8, 12, 0.25, 0.55, size=70, kv_from=1), moe(3, 3, 8)),
], eps=1e-5)
# B: sizes that the tensor-core kernels take in bfloat16 (heads of 64 and 128, a cached row of 80 numbers); blocks
#    of 64 (a page) and 100, windows of 64 and 65; linear position scaling; every expert chosen in one layer; the
#    reader's blocks smaller than its owner's.
CFG_B = config(512, 128, [
    (latent(4, 32, 32, 64, 48, 40, 0.12, size=64, rot=rot(32, 10000.0, 8.0, (64, 16.0, 2.0))), moe(8, 2, 64)),
    (mixed(4, 2, 64, 64, 0.125, size=64, rot=rot(32, 250000.0, 4.0)), moe(4, 4, 64)),
    (difference(2, 2, 32, 64, 0.18, 0.8, size=100), moe(16, 4, 32)),
    (latent(2, 96, 32, 128, 96, 64, 0.09, size=65, rot=rot(32, 500.0, 3.0, (128, 8.0, 1.0))), None),
    (difference(2, 2, 32, 64, 0.2, 0.1, size=64, kv_from=2), moe(8, 2, 64)),
    (mixed(2, 1, 128, 96, 0.09, size=100, rot=rot(128, 10000.0)), None),
], eps=1e-6)
# C: sizes that fit no fast path and no vector load (a width of 50, a vocabulary of 77, heads of 6 and 10); layers
#    without a mask and without a rotation; one head; the latent layer last.
CFG_C = config(77, 50, [
    (difference(3, 1, 6, 10, 0.4, 0.45), moe(5, 2, 12)),
    (mixed(2, 1, 10, 6, 0.3), moe(2, 1, 10)),
    (mixed(1, 1, 6, 6, 0.5, size=3, rot=rot(2, 50.0, 2.0)), None),
    (latent(3, 6, 2, 10, 14, 10, 0.35, rot=rot(2, 20.0)), moe(7, 2, 10)),
], eps=1e-3)

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C}


def random_weights(cfg: dict, seed: int, sharp: float = 2.0) -> dict:
    """bfloat16 weights, drawn here: matrices N(0, 1/fan_in) (those of q and k ``sharp`` times larger, so that the
    scores single keys out), norm weights around zero, gains near 1, a number per head between 0.5 and 2, a mixing
    matrix near the unit matrix."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def mat(o, i, scale=1.0):
        return torch.randn(o, i, generator=g) * (scale / math.sqrt(i))

    def small(n, s=0.2):
        return s * torch.randn(n, generator=g)
    out["embed"] = torch.randn(V, W, generator=g)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = small(W)
        H, D, Vd = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            G = m["kv_heads"]
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = mat(H * D, W, sharp), mat(G * D, W, sharp), mat(G * Vd, W, 1.5)
            out[p + "mix.q.b"], out[p + "mix.k.b"], out[p + "mix.v.b"] = small(H * D, 0.5), small(G * D, 0.5), small(G * Vd, 0.5)
            out[p + "mix.talk"] = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
            out[p + "mix.temp"] = 0.5 + 1.5 * torch.rand(H, generator=g)
            out[p + "mix.o"], out[p + "mix.o.b"] = mat(W, H * Vd, 1.5), small(W, 0.5)
        elif L["type"] == "attention_2":
            G = m["kv_heads"]
            out[p + "mix.q"] = mat(H * 2 * D, W, sharp)
            if m.get("kv_from") is None:
                out[p + "mix.k"], out[p + "mix.v"] = mat(G * 2 * D, W, sharp), mat(G * Vd, W, 1.5)
            for key in ("lq1", "lk1", "lq2", "lk2"):
                out[p + "mix." + key] = small(D, 0.4)
            out[p + "mix.o"] = mat(W, H * Vd, 1.5)
        else:
            R, C, Q = m["rot_dim"], m["kv_rank"], m["q_rank"]
            out[p + "mix.dq"], out[p + "mix.dq.norm"] = mat(Q, W, 1.5), 1.0 + small(Q)
            out[p + "mix.uq"] = mat(H * (D + R), Q, sharp)
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = mat(C + R, W, sharp), 1.0 + small(C)
            out[p + "mix.uk"], out[p + "mix.uv"] = mat(H * D, C, sharp), mat(H * Vd, C, 1.5)
            out[p + "mix.g"] = mat(H, W, 2.0)
            out[p + "mix.o"] = mat(W, H * Vd, 1.5)
        f = L["mlp"]
        if f is not None:
            out[p + "norm2"] = small(W)
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            out[p + "mlp.router"], out[p + "mlp.router.b"] = mat(E, W, 2.0), small(E, 0.5)
            for e in range(E):
                q = f"{p}mlp.e{e}."
                out[q + "gate"], out[q + "up"], out[q + "down"] = mat(ff, W, 1.5), mat(ff, W, 1.5), mat(W, ff)
    out["final.norm"] = small(W)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in out.items()}


def doubles(w: dict) -> dict:
    return {k: v.double() for k, v in w.items()}


TOL32 = 3e-5
ROUTING_MARGIN = 0.05          # logits of size 2 are sums of a few dozen products of 16-bit numbers; one of two experts may win
ROUTING_TURNS = 0.02           # under this margin the 16-bit engine is taken to have chosen otherwise (a token of one
                               # configuration, margin 0.012, did: where one expert of four is chosen, every later token
                               # that reads it differs)
BF16_FLOOR, BF16_FACTOR = 2e-2, 3.0
_BUDGET = {}


def tolerance(key, cfg, w, ids, dtype: str, first=None) -> torch.Tensor:
    """One tolerance per position.  float32: rounding only.  bfloat16: the larger of 2e-2 and three times what the plain
    implementation itself loses at that position when it rounds what a 16-bit engine stores (never taken from the
    library's output); positions whose routing hangs on less than ROUTING_MARGIN are not compared, nor is anything
    after a position whose routing hangs on less than ROUTING_TURNS.  ``first``: the sequence is fed as ``first`` tokens and
    then one by one, and the plain implementation rounds what the engine stores in such steps."""
    if dtype == "float32":
        return torch.full((len(ids),), TOL32, dtype=torch.float64)
    k = (key, tuple(ids), first)
    if k not in _BUDGET:
        truth = plain.forward(cfg, w, ids)
        lost = position_errors(plain.forward(cfg, w, ids, rnd=plain.to_bf16), truth)
        if first is not None and first < len(ids):
            pieces = [first] + [1] * (len(ids) - first)
            lost = torch.maximum(lost, position_errors(plain.logits(cfg, w, ids, pieces, rnd=plain.to_bf16), truth))
        tol = torch.clamp(BF16_FACTOR * lost, min=max(BF16_FLOOR, float(lost.median()) * BF16_FACTOR))
        margins = plain.routing_margins(cfg, w, ids)
        tol[margins < ROUTING_MARGIN] = float("inf")
        turned = (margins < ROUTING_TURNS).nonzero().flatten()
        if turned.numel():
            tol[int(turned[0]):] = float("inf")
        _BUDGET[k] = tol
    return _BUDGET[k]
