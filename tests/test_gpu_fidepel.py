"""Fidepel on the GPU against the plain implementation: each mechanism alone, then the model through the engine
(whole prompts, the stream after every layer run, token by token, unequal batches, reused slots and pages, keys at the
edges of windows and pages, the first tokens, long decoding, greedy generation, the command line, trace replay)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_fidepel as plain
import trapetum_b200 as tb
from conftest import ROOT, within
from fidepel_util import (CONFIGS, TOL32, attn, config, doubles, moe, position_errors, prompts, random_weights, tolerance,
                          worst_ratio, write_folder)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64


@pytest.fixture(scope="module")
def weights():
    return {name: random_weights(cfg, 31 + ord(name)) for name, cfg in CONFIGS.items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory, weights):
    return {name: write_folder(str(tmp_path_factory.mktemp("fidepel" + name)), cfg, weights[name]) for name, cfg in CONFIGS.items()}


@pytest.fixture(scope="module")
def oracles(weights):
    return {name: (cfg, doubles(weights[name])) for name, cfg in CONFIGS.items()}


_MODELS = {}


def model_of(folders, name, dtype):
    if (name, dtype) not in _MODELS:
        _MODELS[(name, dtype)] = tb.load_model(folders[name], dtype, DEV)
    return _MODELS[(name, dtype)]


def close(got, want, tol, what, dtype):
    within(worst_ratio(got, want, tol), 1.0, dtype, what + " (error / tolerance)")


def near(got, want, dtype, what, rel32=2e-5, rel16=2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= (rel32 if dtype == "float32" else rel16), f"{what} [{dtype}]: {err:.3e}"


def dev(t, dt=None):
    return t.to(device=DEV, dtype=dt) if dt is not None else t.to(DEV)


# =================================================================================================================
# Mechanisms alone
# =================================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, width, splits", [(5, 72, (1, 1)), (130, 320, (3, 1)), (3, 1000, (2, 4)), (7, 50, (1, 0))])
def test_the_scaled_sum_of_two_branches_and_the_norm_of_one_number(rows, width, splits, dtype):
    """h += m (a + b) with each branch as partial sums or not, one branch or two; then h / rms(h) * g."""
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(width)
    h = torch.randn(rows, width, generator=g) * 3
    branches = [torch.randn(n, rows, width, generator=g) for n in splits if n]
    gain, m, eps = 1.3, 0.37, 1e-3
    w = torch.full((width,), gain)
    hd = dev(h)
    out = ops.add_scaled_rmsnorm(hd, [dev(b) if b.shape[0] > 1 else dev(b[0]) for b in branches], m, dev(w), eps, 0.0, DTYPES[dtype])
    s = h.double() + m * sum(b.double().sum(0) for b in branches)
    near(hd, s, "float32", "the scaled sum")
    near(out, plain.scalar_norm(s, torch.tensor(gain, dtype=F), eps), dtype, "the norm after it")
    hd2 = dev(h)
    assert ops.add_scaled_rmsnorm(hd2, [dev(b) for b in branches], m) is None          # the sum alone (the model's last layer)
    near(hd2, s, "float32", "the scaled sum alone")
    near(ops.rmsnorm(dev(h), dev(w), eps, 0.0, DTYPES[dtype]), plain.scalar_norm(h.double(), torch.tensor(gain, dtype=F), eps), dtype,
         "the norm alone")


def _cache_line(pages, n_kv, hd, dtype):
    from trapetum_b200.csrc.ops import PAGE_ROWS
    return (torch.zeros(pages, n_kv, PAGE_ROWS, hd, dtype=dtype, device=DEV),
            torch.zeros(pages, n_kv, PAGE_ROWS, hd, dtype=dtype, device=DEV))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, d, vd, pad, R, factor, normed, gated", [
    (4, 2, 16, 16, 16, 16, 2.0, True, True), (3, 1, 24, 40, 40, 8, 1.0, True, True), (2, 2, 80, 64, 128, 80, 4.0, True, False),
    (8, 1, 128, 128, 128, 64, 1.0, False, True), (5, 5, 6, 10, 16, 0, 1.0, True, True), (1, 1, 32, 8, 64, 2, 3.0, True, False)])
def test_projection_norm_head_weights_rotation_padding_gate_and_cache_write(H, G, d, vd, pad, R, factor, normed, gated, dtype):
    """Two sequences (the second one's tokens sit at positions 130..132, on its third page) through the kernel that
    stands between the fused projection and the attention kernels."""
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(d + vd)
    lens, pos0 = [70, 3], [0, 130]
    T = sum(lens)
    in_w = H * d + G * (d + vd) + (H if gated else 0)
    part = torch.randn(3, T, (in_w + 15) // 16 * 16, generator=g) * torch.tensor([1.0, 0.1, 3.0])[:, None, None]
    x = part.double().sum(0)
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(pos0, lens)]).int()
    token_seq = torch.repeat_interleave(torch.arange(2), torch.tensor(lens)).int()
    len_after = torch.tensor([p + n for p, n in zip(pos0, lens)]).int()
    table = torch.tensor([[5, 2, 0], [1, 4, 3]]).int()
    kp, vp = _cache_line(6, G, pad, dt)
    eps, base = 1e-3, 300.0
    wq, wk = 1 + 0.3 * torch.randn(H * d, generator=g), 1 + 0.3 * torch.randn(G * d, generator=g)
    temp = 0.5 + torch.rand(H, generator=g)
    inv_freq = torch.tensor([base ** (-2.0 * i / R) / factor for i in range(R // 2)], dtype=torch.float32) if R else None
    out, gate = ops.projnorm_kv(dev(part), H, G, d, vd, pad, dt, dev(wq) if normed else None, dev(wk) if normed else None, eps,
                                dev(temp), R, dev(inv_freq) if R else None, gated, dev(positions), dev(token_seq), dev(len_after),
                                kp, vp, dev(table), 0)
    q, k = x[:, :H * d], x[:, H * d:(H + G) * d]
    if normed:
        q, k = plain.rms_norm(q, wq.double(), eps), plain.rms_norm(k, wk.double(), eps)
    q = plain.rotate_half(q.view(T, H, d), positions.long(), R, base, factor) * temp.double()[None, :, None]
    k = plain.rotate_half(k.view(T, G, d), positions.long(), R, base, factor)
    v = x[:, (H + G) * d:(H + G) * d + G * vd].view(T, G, vd)

    def padded(t):
        return torch.cat([t, torch.zeros(T, t.shape[1], pad - t.shape[2], dtype=F)], dim=2).reshape(T, -1)
    want = torch.cat([padded(q), padded(k), padded(v)], dim=1)
    # angles are 32-bit products of a position and a 32-bit frequency: up to 132 * 2^-24 off, times the values' size
    tol = 3e-5 if dtype == "float32" else 2 ** -8
    assert float(((out.double().cpu() - want).abs() / (want.abs() + 1.0)).max()) <= tol
    if pad > max(d, vd):
        assert float(out.view(T, H + 2 * G, pad)[:, :, max(d, vd):].abs().max()) == 0.0
    if gated:
        near(gate, torch.sigmoid(x[:, in_w - H:in_w]), "float32", "the heads' gates")
    else:
        assert gate is None
    for t in range(T):
        b, p = int(token_seq[t]), int(positions[t])
        page = int(table[b, p // 64])
        assert torch.equal(kp[page, :, p % 64].cpu(), out[t, H * pad:(H + G) * pad].view(G, pad).cpu())
        assert torch.equal(vp[page, :, p % 64].cpu(), out[t, (H + G) * pad:].view(G, pad).cpu())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_head_times_its_gate(dtype):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    o, gate = torch.randn(37, 3 * 40, generator=g).to(DTYPES[dtype]), torch.rand(37, 3, generator=g)
    want = (o.double().view(37, 3, 40) * gate.double()[:, :, None]).view(37, 120)
    near(ops.head_gate(dev(o), dev(gate), 3), want, dtype, "gated heads", rel16=2 ** -8)


@pytest.mark.parametrize("E, top, groups, keep, scale", [(8, 2, 4, 2, 2.5), (6, 3, 3, 2, 1.0), (5, 2, 5, 3, 0.5), (16, 4, 2, 1, 1.0),
                                                         (3, 3, 1, 1, 2.0), (4, 1, 1, 1, 1.0), (64, 6, 8, 3, 1.5)])
def test_routing_by_softmax_scores(E, top, groups, keep, scale):
    """Logits as partial sums; the chosen sets, and the weights in the kernel's order, against the plain routing."""
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(E * top)
    T = 200
    logits = torch.randn(2, T, (E + 15) // 16 * 16, generator=g) * 2
    r = {"experts": E, "top": top, "scale": scale}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    z = logits.double().sum(0)[:, :E]
    idx, wt = plain.route(z, r, {"router": torch.eye(E, dtype=F)}, "")
    gi, gw, gate = ops.moe_route(dev(logits), E, None, False, top, groups, keep, 1, 1e-20, "softmax", scale)
    assert gate is None
    gi, gw = gi.cpu().long(), gw.cpu().double()
    assert torch.equal(gi.sort(-1).values, idx.sort(-1).values)
    assert torch.allclose(gw.sum(-1), torch.full((T,), scale, dtype=F), rtol=1e-5)
    want = torch.zeros(T, E, dtype=F).scatter_(1, idx, wt)
    assert torch.allclose(torch.zeros(T, E, dtype=F).scatter_(1, gi, gw), want, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, W, E, top, ff, shared", [(5, 48, 4, 2, 24, True), (70, 72, 6, 3, 16, False), (300, 64, 8, 2, 32, True),
                                                      (1100, 128, 8, 2, 64, True), (3, 50, 5, 1, 12, False)])
def test_experts_without_a_gate_matrix(T, W, E, top, ff, shared, dtype):
    """down_e(relu(up_e x)^2), weighed and summed, plus a shared branch given as partial sums: a few tokens (one block
    per pair), more (grouped), and many (the tensor-core product with the activation in its epilogue)."""
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, W, generator=g).to(dt)
    uw, dw = (torch.randn(E, a, b, generator=g).to(dt) / 4 for a, b in ((ff, W), (W, ff)))
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    wt = torch.rand(T, top, generator=g)
    sh = torch.randn(2, T, W, generator=g) if shared else None
    ones = torch.ones(T) if shared else None
    out = ops.moe_experts(dev(x), None, dev(uw), dev(dw), dev(idx), dev(wt), dev(sh) if shared else None, dev(ones) if shared else None, None)
    rnd = plain.to_bf16 if dtype == "bfloat16" else plain.same
    want = sh.double().sum(0) if shared else torch.zeros(T, W, dtype=F)
    for e in range(E):
        y = plain.expert(x.double(), uw[e].double(), dw[e].double(), rnd)
        for j in range(top):
            hit = idx[:, j] == e
            want[hit] += wt[hit, j].double()[:, None] * y[hit]
    got = out.double().sum(0) if out.dim() == 3 else out
    near(got, want, dtype, "experts", rel16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, W, ff", [(4, 72, 40), (200, 128, 96), (9, 50, 20)])
def test_the_shared_expert_as_a_part(T, W, ff, dtype):
    from trapetum_b200.parts.base import Runtime, build_part
    from trapetum_b200.config.base import PartSpec
    from trapetum_b200.csrc import build
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(ff)
    up, down = (torch.randn(ff, W, generator=g) / 6).to(dt), (torch.randn(W, ff, generator=g) / 6).to(dt)
    part = build_part("feed_forward", PartSpec("mlp", {"hidden_size": W, "intermediate_size": ff, "activation": "relu2",
                                                       "up": "s.up", "down": "s.down"}), "", Runtime(dt, torch.device(DEV)))
    build.require(part.kernel_files())
    part.bind({"s.up": dev(up), "s.down": dev(down)})
    x = torch.randn(T, W, generator=g).to(dt)
    out = part.forward(dev(x), None)
    rnd = plain.to_bf16 if dtype == "bfloat16" else plain.same
    near(out.double().sum(0) if out.dim() == 3 else out, plain.expert(x.double(), up.double(), down.double(), rnd), dtype, "down(relu(up x)^2)")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W, E, top, ff, sff, groups", [(64, 8, 2, 32, 48, (4, 2)), (72, 6, 3, 16, 40, None), (128, 16, 4, 64, 128, (2, 1))])
def test_router_and_shared_expert_from_one_product_or_two(W, E, top, ff, sff, groups, dtype):
    """Few tokens take the router's logits and the shared expert's first product from one product over the rows of
    both, many tokens from two: both agree with the plain implementation, token by token."""
    from trapetum_b200.parts.base import Runtime, build_part
    from trapetum_b200.config.base import PartSpec
    from trapetum_b200.csrc import build
    from trapetum_b200.parts import experts as experts_part
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(W + E)
    mlp = moe(E, top, ff, scale=1.5, groups=groups, shared=sff)
    t = {"f.router": torch.randn(E, W, generator=g) * 0.5,
         "f.shared.up": torch.randn(sff, W, generator=g) / 6, "f.shared.down": torch.randn(W, sff, generator=g) / 6}
    for e in range(E):
        t[f"f.e{e}.up"], t[f"f.e{e}.down"] = torch.randn(ff, W, generator=g) / 6, torch.randn(W, ff, generator=g) / 6
    t = {k: v.to(dt) for k, v in t.items()}
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": W, "experts": E, "top": top, "intermediate_size": ff, "gated": False, "activation": "relu2",
        "score": "softmax", "route_scale": 1.5, "groups": groups[0] if groups else 1, "keep_groups": groups[1] if groups else 1,
        "group_score_of": 1, "weight_eps": 1e-20, "router": "router", "correction": None, "expert": "e{}.", "up": "up",
        "down": "down", "shared": {"intermediate_size": sff, "up": "shared.up", "down": "shared.down"}}), "f.", Runtime(dt, torch.device(DEV)))
    build.require(part.kernel_files())
    part.bind({k: dev(v) for k, v in t.items()})
    assert part.w_router_up is not None and part.shared.w_up.data_ptr() == part.w_router_up[part.w_router.shape[0]:].data_ptr()
    rnd = plain.to_bf16 if dtype == "bfloat16" else plain.same
    td = {k: v.double() for k, v in t.items()}

    class Ctx:
        memo = {}
    for T in (3, experts_part.FUSED_UP_TOKENS, experts_part.FUSED_UP_TOKENS + 70):
        x = torch.randn(T, W, generator=g).to(dt)
        out = part.forward(dev(x), Ctx())
        got = (out.double().sum(0) if out.dim() == 3 else out.double()).cpu()
        want = plain.moe(x.double(), mlp, td, "f.", rnd)
        plain.MARGINS = []
        plain.route(x.double(), mlp["router"], td, "f.")
        sure = plain.MARGINS[0] > (1e-4 if dtype == "float32" else 0.05)      # a rounded product may turn a close call
        plain.MARGINS = None
        assert int(sure.sum()) >= T // 2
        near(got[sure], want[sure], dtype, f"experts with a shared expert, {T} tokens", rel16=2e-2)


@pytest.mark.parametrize("T, N, K", [(256, 128, 128), (300, 96, 72)])
def test_the_tensor_core_product_squares_what_relu_lets_through(T, N, K):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(N)
    a, w = torch.randn(T, K, generator=g).to(torch.bfloat16), (torch.randn(N, K, generator=g) / 8).to(torch.bfloat16)
    if not ops.gemm_tc_takes(dev(a), dev(w)):
        pytest.skip("sizes the tensor-core product does not take")
    got = ops.gemm_tc(dev(a), dev(w), torch.float32, unary_act="relu2")
    near(got, plain.relu2(a.double() @ w.double().T), "float32", "relu(a w^T)^2 in the product's epilogue", rel32=1e-5)


# =================================================================================================================
# The model through the engine
# =================================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(folders, oracles, name, dtype):
    cfg, w = oracles[name]
    model = model_of(folders, name, dtype)
    eng = tb.Engine(model, max_tokens=1024)
    for ids in prompts(cfg["vocab"], [1, 2, 64, 65, 150], seed=1):
        s = eng.start(1)
        got = eng.step(s, [ids], [list(range(len(ids)))])
        eng.release(s)
        close(got, plain.forward(cfg, w, ids), tolerance(name, cfg, w, ids, dtype), f"{name}: whole prompt of {len(ids)}", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_residual_stream_after_every_layer_run(folders, oracles, name, monkeypatch):
    from trapetum_b200.parts.block import ParallelBlock
    cfg, w = oracles[name]
    ids = prompts(cfg["vocab"], [37], seed=2)[0]
    want = plain.Plain(cfg, w).feed(ids)[1]
    seen, orig = [], ParallelBlock.forward

    def spy(self, stream, ctx, cache):
        orig(self, stream, ctx, cache)
        seen.append(stream.value().clone())
    monkeypatch.setattr(ParallelBlock, "forward", spy)
    eng = tb.Engine(model_of(folders, name, "float32"), max_tokens=256)
    eng.step(eng.start(1), [ids], [[0]])
    assert len(seen) == want.shape[0] == len(plain.schedule(cfg))
    for r, x in enumerate(seen):
        near(x, want[r], "float32", f"{name}: the stream after layer run {r}", rel32=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, first", [("A", 1), ("A", 2), ("B", 63), ("B", 64), ("C", 65), ("C", 7), ("D", 3)])
def test_prompt_then_token_by_token(folders, oracles, name, first, dtype):
    """Decoding runs across a page's border (64, 128), over every window's edge (windows of 1 to 100 pass over decoded
    tokens, and the rows of their caches are used again) and through the capture of the step's graph."""
    cfg, w = oracles[name]
    ids = prompts(cfg["vocab"], [215], seed=first)[0]
    truth = plain.forward(cfg, w, ids)
    assert float(position_errors(plain.forward_stepwise(cfg, w, ids[:70], first), truth[:70]).max()) < 1e-9
    eng = tb.Engine(model_of(folders, name, dtype), max_tokens=512)
    s = eng.start(1)
    got = [eng.step(s, [ids[:first]], [list(range(first))])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[first:]]
    eng.release(s)
    assert dtype == "float32" or eng.graphs_captured >= 1
    close(torch.cat(got), truth, tolerance(name, cfg, w, ids, dtype), f"{name}: {first} tokens, then one by one", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_batch_equals_each_alone_and_slots_are_reused(folders, oracles, name, dtype):
    cfg, w = oracles[name]
    eng = tb.Engine(model_of(folders, name, dtype), max_tokens=1024, max_slots=4)
    rounds = [prompts(cfg["vocab"], [1, 90, 33], seed=4), prompts(cfg["vocab"], [70, 2, 129], seed=5)]
    for ps in rounds:                                            # the second round takes the first one's slots and pages
        n_new = 6
        full = [p + q for p, q in zip(ps, prompts(cfg["vocab"], [n_new] * 3, seed=6))]
        truth = [plain.forward(cfg, w, f) for f in full]
        s = eng.start(3)
        got = [[] for _ in ps]
        out = eng.step(s, ps, [[len(p) - 1] for p in ps])
        for i in range(3):
            got[i].append(out[i:i + 1].clone())
        live = [0, 1, 2]
        for j in range(n_new):
            if j == 3:
                eng.release([s[1]])                              # the middle one ends early; the others go on
                live = [0, 2]
            out = eng.step([s[i] for i in live], [[full[i][len(ps[i]) + j]] for i in live], [[0]] * len(live))
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1].clone())
        eng.release([s[i] for i in live])
        eng.cache.check()
        for i in range(3):
            g = torch.cat(got[i])
            lo = len(ps[i]) - 1
            close(g, truth[i][lo:lo + g.shape[0]], tolerance(name + "u", cfg, w, full[i], dtype)[lo:lo + g.shape[0]],
                  f"{name}: request {i} of an unequal batch", dtype)
    eng.check_kernels()


def _needle(tmp_path, window, key_pos, n):
    """A one-layer model without experts whose scores are sharpened, and a prompt of one repeated token with a single
    other token at ``key_pos``, chosen (with the plain implementation) as the one that the queries single out most."""
    cfg = config(50, 32, [(attn(2, 1, 16, 24, 0.25, window=window, rot=(8, 10000.0, 2.0)), None)], mult=1.5)
    w = {k: v.float() for k, v in random_weights(cfg, 5).items()}
    w["l0.mix.temp"][:] = torch.tensor([2.5, 3.5])
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    wd = doubles(w)
    base = [3] * n
    seen_from = min(n - 1, key_pos + (window or n) - 1)          # the last query that still sees the key
    without = plain.forward(cfg, wd, base)[seen_from:seen_from + 1]
    best, ids = -1.0, None
    for cand in range(4, 24):
        trial = list(base)
        trial[key_pos] = cand
        e = float(position_errors(plain.forward(cfg, wd, trial)[seen_from:seen_from + 1], without))
        if e > best:
            best, ids = e, trial
    assert best > 0.1, best
    folder = write_folder(str(tmp_path / f"needle{window}_{key_pos}_{n}"), cfg, w)
    return cfg, wd, ids, folder, seen_from


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key_pos, n", [(0, 200), (63, 130), (64, 130), (127, 129), (5, 700)])
def test_a_far_key_is_found_in_prompts_and_in_decoding(tmp_path, key_pos, n, dtype):
    """No window: every earlier token is seen, also the first one and those at a page's edge, hundreds of tokens back."""
    cfg, w, ids, folder, _ = _needle(tmp_path, None, key_pos, n)
    truth = plain.forward(cfg, w, ids)
    tol = tolerance(("far", key_pos, n), cfg, w, ids, dtype)
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), max_tokens=1024)
    s = eng.start(1)
    close(eng.step(s, [ids], [[n - 1]]), truth[-1:], tol[-1:], f"needle at {key_pos} of {n}, prompt", dtype)
    eng.release(s)
    s = eng.start(1)
    eng.step(s, [ids[:n - 3]], [[]])
    got = torch.cat([eng.step(s, [[t]], [[0]]).clone() for t in ids[n - 3:]])
    close(got, truth[-3:], tol[-3:], f"needle at {key_pos} of {n}, decoded", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window, key_pos", [(48, 1), (48, 30), (64, 0), (64, 70), (65, 63), (65, 64), (130, 2), (2, 77), (1, 50), (129, 127)])
def test_a_key_at_the_edge_of_the_window_in_prompts_and_in_decoding(tmp_path, window, key_pos, dtype):
    """The key is seen by the queries up to key_pos + window - 1 and by none after it: the logits of the last query that
    sees it and of the first that does not, computed as part of a prompt and decoded one by one."""
    last = key_pos + window - 1
    n = last + 3
    cfg, w, ids, folder, seen_from = _needle(tmp_path, window, key_pos, n)
    assert seen_from == last
    truth = plain.forward(cfg, w, ids)
    blind = plain.forward(cfg, w, [3] * n)
    # the oracle: the key shows at `last` and not after it (one layer: nothing carries it further)
    assert float(position_errors(truth[last:last + 1], blind[last:last + 1])) > 0.1 or window == 1
    assert float((truth[last + 1:] - blind[last + 1:]).abs().max()) == 0.0
    tol = tolerance(("edge", window, key_pos), cfg, w, ids, dtype)
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), max_tokens=512)
    s = eng.start(1)
    close(eng.step(s, [ids], [list(range(n))]), truth, tol, f"window {window}, key at {key_pos}: prompt", dtype)
    eng.release(s)
    s = eng.start(1)
    first = max(1, last - 2)
    got = [eng.step(s, [ids[:first]], [[first - 1]])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[first:]]
    close(torch.cat(got), truth[first - 1:], tol[first - 1:], f"window {window}, key at {key_pos}: decoded", dtype)
    eng.release(s)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_head_without_a_gate_or_its_number_would_show(tmp_path, dtype):
    """Gates near zero on one head and a large number on the other: the logits follow the plain implementation, and the
    plain implementation without either is far away."""
    cfg = config(60, 40, [(attn(2, 2, 8, 12, 0.5, window=9, rot=(8, 100.0)), moe(4, 2, 16, scale=2.0, shared=16))], mult=0.8)
    w = {k: v.float() for k, v in random_weights(cfg, 9).items()}
    w["l0.mix.g"][0] *= 6.0
    w["l0.mix.temp"][:] = torch.tensor([0.25, 3.0])
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    wd = doubles(w)
    ids = prompts(60, [40], seed=3)[0]
    truth = plain.forward(cfg, wd, ids)
    for name, value in (("l0.mix.g", torch.zeros(2, 40, dtype=F)), ("l0.mix.temp", torch.ones(2, dtype=F))):
        other = dict(wd)
        other[name] = value
        assert float(position_errors(plain.forward(cfg, other, ids), truth).median()) > 0.03
    eng = tb.Engine(tb.load_model(write_folder(str(tmp_path / "gates"), cfg, w), dtype, DEV), max_tokens=256)
    s = eng.start(1)
    got = [eng.step(s, [ids[:30]], [list(range(30))])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[30:]]
    close(torch.cat(got), truth, tolerance("gates", cfg, wd, ids, dtype), "gates and head numbers, prompt then decoding", dtype)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_library(folders, oracles, name):
    cfg, w = oracles[name]
    ps = prompts(cfg["vocab"], [5, 1, 70, 12], seed=9)
    want = [plain.generate_greedy(cfg, w, p, 10) for p in ps]
    model = model_of(folders, name, "float32")
    assert tb.generate(model, ps, max_tokens=10, stop_ids=[]) == want
    assert tb.generate(model, ps, max_tokens=10, stop_ids=[], max_batch=2) == want      # two batches, slots used again
    got16 = tb.generate(model_of(folders, name, "bfloat16"), ps, max_tokens=10, stop_ids=[])
    assert all(len(o) == 10 for o in got16)


def test_command_line_runs_the_model(folders, oracles):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gemma_run"), folders["B"], "--prompt_ids", "5,17,3",
                           "--max_tokens", "5", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    cfg, w = oracles["B"]
    assert f"continuation ids: {plain.generate_greedy(cfg, w, [5, 17, 3], 5)}" in proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay(folders, oracles, tmp_path, dtype):
    name = "A"
    cfg, w = oracles[name]
    V = cfg["vocab"]
    reqs = prompts(V, [40, 75, 130], seed=3)
    truth = [plain.forward(cfg, w, r) for r in reqs]
    steps, expect = [], {}                                            # step -> [(request, position)] of its wanted rows

    def add(entries, end=()):
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})
        return len(steps) - 1
    n = add([{"id": "w", "tokens": reqs[0], "want": list(range(40))}], end=["w"])
    expect[n] = [(0, p) for p in range(40)]
    cut = [1, 60, 33]                                                # together; one starts with a single token
    ids = [f"b{i}" for i in range(3)]
    n = add([{"id": ids[i], "tokens": reqs[i][:cut[i]], "want": [cut[i] - 1]} for i in range(3)])
    expect[n] = [(i, cut[i] - 1) for i in range(3)]
    live, t = [0, 1, 2], 0
    while live:
        nxt = [i for i in live if cut[i] + t + 1 < len(reqs[i])]
        quiet = t % 5 == 3
        n = add([{"id": ids[i], "tokens": [reqs[i][cut[i] + t]], "want": [] if quiet else [0]} for i in live],
                end=[ids[i] for i in live if i not in nxt])
        if not quiet:
            expect[n] = [(i, cut[i] + t) for i in live]
        live, t = nxt, t + 1
    out = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name], "--dtype", dtype,
                           "--out", out, "--max-tokens", str(40 + 75 + 130)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    assert sorted(os.listdir(out)) == sorted(f"{n}.f32" for n in expect)
    tols = [tolerance(name, cfg, w, r, dtype) for r in reqs]
    for n, rows in expect.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V))
        want = torch.stack([truth[i][p] for i, p in rows])
        assert got.shape == want.shape
        close(got, want, torch.stack([tols[i][p] for i, p in rows]), f"replay step {n}", dtype)
