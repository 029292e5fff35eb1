"""Shared pieces of the Fidepel tests: small configurations made up here, model folders with random weights drawn
here (not by the library), and tolerances taken from the plain implementation alone."""
import math

import torch

import plain_fidepel as plain
from lofirax_util import position_errors, prompts, worst_ratio, write_folder  # noqa: F401  (the tests import them from here)


def attn(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    """``rot`` = (dims, base) or (dims, base, factor) or None."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = {"factor": rot[2]}
    return m


def moe(experts, top, ff, scale=None, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if scale is not None:
        r["scale"] = scale
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(vocab, width, layers, loop=None, mult=None, eps=1e-5):
    c = {"architecture": "Fidepel", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [{"type": "attention", "mixer": m, "mlp": f} for m, f in layers]}
    if mult is not None:
        c["residual_mult"] = mult
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# A: as many kv heads as heads; values wider than keys; a window of five; half of every head rotated, no position scaling;
#    no groups, no shared expert; a layer without a feed-forward; no residual multiplier; the middle layer alone runs
#    three times.
CFG_A = config(150, 48, [
    (attn(3, 3, 8, 12, 0.4, window=5, rot=(4, 100.0)), moe(4, 1, 24)),
    (attn(2, 1, 16, 16, 0.3, window=33, rot=(16, 10000.0, 8.0)), moe(6, 3, 16, scale=1.5, groups=(3, 2), shared=40)),
    (attn(1, 1, 24, 8, 0.2, window=2, rot=(24, 500.0, 1.5)), None),
], loop=(1, 2, 3), eps=1e-5)
# B: no window and no rotation in the first layer (positions enter through the second); values narrower than keys;
#    a window of one (a token sees itself only); six experts of which all groups are kept; a width that is no multiple
#    of 16.
CFG_B = config(301, 72, [
    (attn(4, 2, 16, 8, 0.25), moe(6, 2, 24, scale=0.5, groups=(2, 2), shared=16)),
    (attn(2, 2, 12, 20, 0.3, window=1, rot=(12, 50.0)), moe(3, 3, 16)),
    (attn(6, 3, 8, 8, 0.35, window=64, rot=(2, 10000.0, 3.0)), moe(8, 2, 8, groups=(4, 1), shared=24)),
], mult=0.7, eps=1e-4)
# C: sizes that the tensor-core kernels take in bfloat16 (heads padded to 64, 128 and 256); windows of 64 (a page), 65
#    and 100; the whole model is one repeated span that runs twice.
CFG_C = config(512, 128, [
    (attn(4, 2, 64, 64, 0.125, window=64, rot=(64, 10000.0, 2.0)), moe(8, 2, 64, scale=2.0, groups=(4, 2), shared=128)),
    (attn(2, 1, 128, 96, 0.09, window=65, rot=(32, 250000.0)), moe(4, 4, 64, groups=(4, 4))),
    (attn(4, 4, 32, 48, 0.2, window=100, rot=(32, 1000.0, 4.0)), moe(16, 4, 32, scale=1.0, groups=(2, 1), shared=64)),
    (attn(1, 1, 160, 144, 0.08, rot=(96, 10000.0)), None),
], loop=(0, 4, 2), mult=0.4, eps=1e-6)
# D: sizes that fit no fast path and no vector load: a width of 50, a vocabulary of 77, heads of 6 and 10, as many groups
#    as experts, the first layer alone repeated.
CFG_D = config(77, 50, [
    (attn(2, 1, 6, 10, 0.5, window=3, rot=(2, 50.0, 2.0)), moe(5, 2, 12, scale=3.0, groups=(5, 3), shared=20)),
    (attn(3, 1, 10, 6, 0.3, window=70, rot=(6, 20.0)), moe(2, 1, 10)),
], loop=(0, 1, 2), mult=1.25, eps=1e-3)

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}


def random_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 weights, drawn here: matrices N(0, 1/fan_in), gains near 1, a temperature per head between 0.5 and 2."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def mat(o, i, scale=1.0):
        return torch.randn(o, i, generator=g) * (scale / math.sqrt(i))

    def gain(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)
    out["embed"] = torch.randn(V, W, generator=g)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = gain(1).reshape(())
        out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = mat(H * D, W), mat(G * D, W), mat(G * Vd, W, 1.5)
        out[p + "mix.q.norm"], out[p + "mix.k.norm"] = gain(H * D) * 1.5, gain(G * D) * 1.5
        out[p + "mix.temp"] = 0.5 + 1.5 * torch.rand(H, generator=g)
        out[p + "mix.g"] = mat(H, W, 2.0)
        out[p + "mix.o"] = mat(W, H * Vd, 1.5)
        f = L["mlp"]
        if f is not None:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            out[p + "mlp.router"] = mat(E, W, 2.0)
            for e in range(E):
                out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = mat(ff, W, 1.5), mat(W, ff, 1.5)
            if f.get("shared"):
                out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = mat(f["shared"]["ff"], W, 1.5), mat(W, f["shared"]["ff"])
    out["final.norm"] = gain(1).reshape(())
    out["head"] = mat(V, W)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in out.items()}


def doubles(w: dict) -> dict:
    return {k: v.double() for k, v in w.items()}


TOL32 = 3e-5
ROUTING_MARGIN = 0.03          # scores are softmaxes of sums of a few dozen products of 16-bit numbers
ROUTING_TURNS = 0.005          # under this margin the 16-bit engine is taken to have chosen otherwise
BF16_FLOOR, BF16_FACTOR = 2e-2, 3.0
_BUDGET = {}


def tolerance(key, cfg, w, ids, dtype: str) -> torch.Tensor:
    """One tolerance per position.  float32: rounding only.  bfloat16: the larger of 2e-2 and three times what the plain
    implementation itself loses at that position when it rounds what a 16-bit engine stores (never taken from the
    library's output); positions whose routing hangs on less than ROUTING_MARGIN are not compared."""
    if dtype == "float32":
        return torch.full((len(ids),), TOL32, dtype=torch.float64)
    k = (key, tuple(ids))
    if k not in _BUDGET:
        lost = position_errors(plain.forward(cfg, w, ids, rnd=plain.to_bf16), plain.forward(cfg, w, ids))
        tol = torch.clamp(BF16_FACTOR * lost, min=max(BF16_FLOOR, float(lost.median()) * BF16_FACTOR))
        margins = plain.routing_margins(cfg, w, ids)
        tol[margins < ROUTING_MARGIN] = float("inf")
        turned = (margins < ROUTING_TURNS).nonzero().flatten()
        if turned.numel():
            # a token that went another way changes what every later token reads from the cache
            tol[int(turned[0]):] = float("inf")
        _BUDGET[k] = tol
    return _BUDGET[k]
