"""Fibelix on the GPU against the plain implementation: each mechanism alone, then the model through the engine
(whole prompts, the stream after every layer, token by token, unequal batches, reused slots and pages, keys at the
edges of blocks, windows and pages, the first tokens, long decoding, greedy generation, the command line, trace
replay)."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_fibelix as plain
import trapetum_b200 as tb
from conftest import ROOT, within
from fibelix_util import (CONFIGS, config, difference, doubles, latent, mixed, moe, position_errors, prompts, random_weights,
                          rot, tolerance, worst_ratio, write_folder)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64
PAGE = 64


@pytest.fixture(scope="module")
def weights():
    # B's heads are wide: with the other models' sharpening its scores reach the hundreds, where the rounding of one
    # 16-bit key decides which token a query reads, in the plain implementation as in the engine
    return {name: random_weights(cfg, 17 + ord(name), sharp=1.25 if name == "B" else 2.0) for name, cfg in CONFIGS.items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory, weights):
    return {name: write_folder(str(tmp_path_factory.mktemp("fibelix" + name)), cfg, weights[name]) for name, cfg in CONFIGS.items()}


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


def rounded(t, dtype):
    """What the kernel gets: the values as the dtype stores them, in 64-bit for the oracle."""
    return t.to(DTYPES[dtype]).to(F)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------

def _mixed_reference(q, k, v, mix, H, G, seen, unit_sink, first_pos=0):
    """q [T, H, D] at positions first_pos.., k and v [keys, G, D] at positions 0..: the oracle's pieces put together."""
    T = q.shape[0]
    pos, kpos = torch.arange(first_pos, first_pos + T), torch.arange(k.shape[0])
    s = torch.stack([q[:, g] @ k[:, g // (H // G)].T for g in range(H)])
    s = torch.einsum("hg,gtj->htj", mix, s)
    ok = plain.same_block(pos, kpos, -seen) if seen < 0 else plain.in_window(pos, kpos, seen or None)
    return torch.stack([plain.softmax_seen(s[h], ok, unit_sink) @ v[:, h // (H // G)] for h in range(H)], dim=1)


def _paged(rows, n_kv, D, dtype, ring_rows=0, pages_total=24, seed=0):
    """``rows`` [B][len_b, n_kv, D] written into pools whose pages lie out of order; returns (k-like pool, table)."""
    g = torch.Generator().manual_seed(seed)
    pool = torch.full((pages_total, n_kv, PAGE, D), float("nan"), dtype=torch.float32)
    order = torch.randperm(pages_total, generator=g).tolist()
    table, at = [], 0
    for r in rows:
        held = min(r.shape[0], ring_rows) if ring_rows else r.shape[0]
        n_pages = (held + PAGE - 1) // PAGE
        mine = order[at:at + n_pages]
        at += n_pages
        first = max(0, r.shape[0] - ring_rows) if ring_rows else 0
        for p in range(first, r.shape[0]):
            row = p % ring_rows if ring_rows else p
            pool[mine[row // PAGE], :, row % PAGE] = r[p].float()
        table.append(mine)
    width = max(len(t) for t in table)
    tab = torch.tensor([t + [0] * (width - len(t)) for t in table], dtype=torch.int32)
    return pool.nan_to_num(0.0).to(DTYPES[dtype]).to(DEV).contiguous(), tab.to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, seen, sink", [(3, 3, 8, -5, True), (6, 3, 24, -33, True), (4, 2, 64, -64, False), (2, 1, 40, 0, True),
                                                 (5, 1, 16, 7, False), (1, 1, 8, -1, True), (32, 8, 16, -70, True), (6, 3, 96, -33, True),
                                                 (16, 4, 128, -100, True), (3, 1, 32, 20, False), (8, 8, 64, 0, True), (2, 2, 128, -3, True),
                                                 (32, 8, 128, -100, True), (24, 3, 64, -33, False), (20, 4, 32, 0, True), (17, 17, 32, 9, True)])
def test_scores_mixed_across_heads_in_prompts(H, G, D, seen, sink, dtype):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(H * 100 + D)
    lens = [1, 2, 37, 140]
    T = sum(lens)
    q = rounded(torch.randn(T, H, D, generator=g), dtype)
    k = rounded(torch.randn(T, G, D, generator=g), dtype)
    v = rounded(torch.randn(T, G, D, generator=g), dtype)
    mix = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).float() * 0.3
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    token_seq = sum([[b] * n for b, n in enumerate(lens)], [])
    want = torch.cat([_mixed_reference(q[a:b], k[a:b], v[a:b], mix.double(), H, G, seen, sink)
                      for a, b in zip(starts, starts[1:])])
    for longest in (0, max(lens)):           # without the longest sequence's length the generic kernel runs, with it the tensor cores' where they can
        got = ops.attn_mixed_prefill(dev(q.reshape(T, -1), DTYPES[dtype]), dev(k.reshape(T, -1), DTYPES[dtype]),
                                     dev(v.reshape(T, -1), DTYPES[dtype]), i32(starts), i32(token_seq), H, G, D, dev(mix), seen, sink, longest)
        near(got.view(T, H, D), want, dtype, f"mixed attention, prompts ({longest})", rel16=1.5e-2)


@pytest.mark.parametrize("H, G, D, seen, sink", [(4, 2, 64, 0, True), (6, 3, 96, -300, True), (2, 1, 128, 500, False), (24, 3, 32, -256, True)])
def test_scores_mixed_across_heads_in_a_long_prompt_whose_keys_are_cut_into_pieces(H, G, D, seen, sink):
    """One long prompt is fewer tiles of queries than the GPU has SMs: the tensor-core kernel cuts every tile's keys
    into pieces and folds them."""
    from trapetum_b200.csrc import ops
    dtype = "bfloat16"
    g = torch.Generator().manual_seed(H + D)
    lens = [3, 900]
    T = sum(lens)
    q = rounded(torch.randn(T, H, D, generator=g), dtype)
    k = rounded(torch.randn(T, G, D, generator=g), dtype)
    v = rounded(torch.randn(T, G, D, generator=g), dtype)
    mix = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).float() * 0.2
    starts = [0, 3, T]
    token_seq = [0] * 3 + [1] * 900
    want = torch.cat([_mixed_reference(q[a:b], k[a:b], v[a:b], mix.double(), H, G, seen, sink) for a, b in zip(starts, starts[1:])])
    got = ops.attn_mixed_prefill(dev(q.reshape(T, -1), DTYPES[dtype]), dev(k.reshape(T, -1), DTYPES[dtype]),
                                 dev(v.reshape(T, -1), DTYPES[dtype]), i32(starts), i32(token_seq), H, G, D, dev(mix), seen, sink, 900)
    near(got.view(T, H, D), want, dtype, "mixed attention, a long prompt in pieces", rel16=1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, seen, ring, sink", [(3, 3, 8, -5, 64, True), (6, 3, 24, -33, 0, True), (4, 2, 64, -64, 64, False),
                                                       (2, 1, 40, 0, 0, True), (5, 1, 16, 70, 128, False), (4, 4, 16, -100, 128, True)])
def test_scores_mixed_across_heads_one_query_against_the_cache(H, G, D, seen, ring, sink, dtype):
    """Lengths just before, at and after the edges of blocks, windows and pages; pages out of order; a ring that has
    wrapped; the keys cut into pieces (a long bucket) and not."""
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(D)
    size = abs(seen) or 50
    lens = sorted({1, 2, size, size + 1, 2 * size, 2 * size + 1, 64, 65, 128, 129, 3 * size - 1, 700})
    B = len(lens)
    ks = [rounded(torch.randn(n, G, D, generator=g), dtype) for n in lens]
    vs = [rounded(torch.randn(n, G, D, generator=g), dtype) for n in lens]
    q = rounded(torch.randn(B, H, D, generator=g), dtype)
    mix = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).float() * 0.3
    k_pool, table = _paged(ks, G, D, dtype, ring, pages_total=48, seed=1)
    v_pool, _ = _paged(vs, G, D, dtype, ring, pages_total=48, seed=1)
    want = torch.cat([_mixed_reference(q[b:b + 1], ks[b], vs[b], mix.double(), H, G, seen, sink, first_pos=lens[b] - 1)
                      for b in range(B)])
    for bucket in (64, 1024):
        got = ops.attn_mixed_decode(dev(q.reshape(B, -1), DTYPES[dtype]), k_pool, v_pool, table, i32(lens), H, G, D, dev(mix),
                                    seen, sink, ring, bucket)
        near(got.view(B, H, D), want, dtype, f"mixed attention, decode, bucket {bucket}", rel16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, block", [(4, 2, 64, 64), (4, 1, 128, 100), (2, 2, 64, 5), (6, 3, 16, 33), (3, 1, 24, 70)])
def test_blocks_on_the_decode_kernels(H, G, D, block, dtype):
    """The framework's decode kernels with a block in place of a window: lengths around the edges of blocks and pages."""
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(block)
    lens = sorted({1, block, block + 1, 2 * block, 2 * block + 1, 64, 65, 128, 129, 5 * block + 2, 600})
    B = len(lens)
    ks = [rounded(torch.randn(n, G, D, generator=g), dtype) for n in lens]
    vs = [rounded(torch.randn(n, G, D, generator=g), dtype) for n in lens]
    q = rounded(torch.randn(B, H, D, generator=g), dtype)
    k_pool, table = _paged(ks, G, D, dtype, 0, pages_total=48, seed=2)
    v_pool, _ = _paged(vs, G, D, dtype, 0, pages_total=48, seed=2)
    scale = 0.3
    mix = torch.eye(H, dtype=F) * scale
    want = torch.cat([_mixed_reference(q[b:b + 1], ks[b], vs[b], mix, H, G, -block, False, first_pos=lens[b] - 1) for b in range(B)])
    for bucket, uneven in ((256, 0), (1024, 3)):
        got = ops.attn_decode(dev(q.reshape(B, -1), DTYPES[dtype]), k_pool, v_pool, table, i32(lens), H, G, D, scale, 0.0, -block,
                              0, bucket, uneven)
        near(got.view(B, H, D), want, dtype, f"blocks on the decode kernels, bucket {bucket}", rel16=1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, D, vd", [(2, 64, 64), (3, 16, 10), (1, 128, 96)])
def test_two_maps_folded_into_their_difference(H, D, vd, dtype):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(D)
    T, lam, eps, diff = 9, 0.37, 1e-5, 0.6
    a = rounded(torch.randn(T, H, 2, D, generator=g), dtype)
    got = ops.head_difference(dev(a.reshape(T, -1), DTYPES[dtype]), H, D, vd, lam, eps, 1.0 - diff).view(T, H, D)
    o = a[:, :, 0, :vd] - lam * a[:, :, 1, :vd]
    want = o / plain.rms(o, eps) * (1.0 - diff)
    near(got[:, :, :vd], want, dtype, "head difference", rel16=1e-2)
    assert float(got[:, :, vd:].abs().max()) == 0.0 if vd < D else True


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C, R, Q, n_gate, ring, mult", [(16, 4, 24, 2, 64, 1.07), (48, 32, 40, 4, 0, 1.2), (14, 2, 0, 3, 128, 1.0),
                                                         (96, 32, 64, 0, 64, 1.1)])
def test_latent_rows_with_the_queries_latent_the_gates_and_a_ring(C, R, Q, n_gate, ring, mult, dtype):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(C)
    lens = [3, 150, 64]
    T, eps = sum(lens), 1e-5
    width = C + R + Q + n_gate
    part = torch.randn(2, T, width + (-width % 4), generator=g)
    w_c, w_q = 1.0 + 0.2 * torch.randn(C, generator=g), 1.0 + 0.2 * torch.randn(max(Q, 1), generator=g)
    freq = plain.linear_frequencies(R, 100.0)
    pos = torch.cat([torch.arange(n) for n in lens])
    token_seq = sum([[b] * n for b, n in enumerate(lens)], [])
    pool = torch.zeros((16, 1, PAGE, C + R), dtype=DTYPES[dtype], device=DEV)
    table = torch.tensor([[3, 9, 1], [7, 2, 11], [5, 0, 4]], dtype=torch.int32, device=DEV)
    rows, cq, gates = ops.latent_rows(dev(part), dev(w_c.float()), eps, dev(freq.float()), R, C, R, dev(pos.int()), i32(token_seq), pool,
                                      table, DTYPES[dtype], ring, i32(lens), mult, dev(w_q.float()) if Q else None, n_gate)
    x = part.double().sum(0)
    want_c = plain.plain_norm(x[:, :C], w_c.double(), eps)
    want_r = plain.turn_halves(x[:, C:C + R], pos, freq.float().double()) * mult
    near(rows[:, :C], want_c, dtype, "latent rows: the latent")
    near(rows[:, C:], want_r, dtype, "latent rows: the rotated part")
    if Q:
        near(cq, plain.plain_norm(x[:, C + R:C + R + Q], w_q.double(), eps), dtype, "latent rows: the queries' latent")
    if n_gate:
        near(gates, torch.sigmoid(x[:, C + R + Q:width]), "float32", "latent rows: gates")
    # the cache: every kept token where its position says
    at = 0
    for b, n in enumerate(lens):
        for p in range(max(0, n - ring) if ring else 0, n):
            r = p % ring if ring else p
            cached = pool[int(table[b, r // PAGE]), 0, r % PAGE]
            assert torch.equal(cached, rows[at + p]), (b, p)
        at += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, C, R, window, ring", [(2, 16, 4, 7, 64), (4, 48, 32, 64, 64), (4, 48, 32, 65, 128), (3, 14, 2, 0, 0),
                                                  (20, 96, 32, 100, 128), (2, 16, 16, 130, 0)])
def test_cached_latents_read_through_a_window(H, C, R, window, ring, dtype):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(C + window)
    lens = sorted({1, 2, 33, 64, 65, 128, 129, 300, max(1, window), window + 1, window + 64, 2 * window + 3})
    B, KD = len(lens), C + R
    rows = [rounded(torch.randn(n, 1, KD, generator=g) * 0.5, dtype) for n in lens]
    q = rounded(torch.randn(B, H, KD, generator=g), dtype)
    pool, table = _paged(rows, 1, KD, dtype, ring, pages_total=48, seed=3)
    scale = 0.2
    want = []
    for b, n in enumerate(lens):
        r = rows[b][:, 0]
        ok = plain.in_window(torch.tensor([n - 1]), torch.arange(n), window or None)
        want.append(torch.stack([plain.softmax_seen(q[b, h:h + 1] @ r.T * scale, ok) @ r[:, :C] for h in range(H)], dim=1))
    for bucket in (64, 2048):
        got = ops.latent_decode(dev(q.reshape(B, -1), DTYPES[dtype]), pool, table, i32(lens), None, H, C, R, scale, bucket, window, ring)
        near(got.view(B, H, C), torch.cat(want), dtype, f"latent decode through a window, bucket {bucket}", rel16=1.5e-2)


@pytest.mark.parametrize("E, top", [(12, 2), (5, 1), (7, 7), (16, 4)])
def test_routing_by_the_largest_logits_with_a_bias(E, top):
    """The winners' softmax over their own logits is their share of the softmax over all, divided by the winners' sum."""
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(E)
    T, W = 50, 24
    h, R, b = torch.randn(T, W, generator=g).double(), torch.randn(E, W, generator=g).double(), torch.randn(E, generator=g).double()
    t = {"router": R, "router.b": b}
    idx, w, z = plain.route(h, {"router": {"top": top}}, t, "")
    part = torch.zeros(2, T, 16)
    part[0, :, :E] = (z - b).float() * 0.25
    part[1, :, :E] = (z - b).float() * 0.75
    gi, gw, _ = ops.moe_route(dev(part), E, None, False, top, 1, 1, 1, 0.0, "softmax", 1.0, dev(b.float()))
    order = torch.argsort(gi.cpu().long(), dim=1)
    want_order = torch.argsort(idx, dim=1)
    assert torch.equal(torch.gather(gi.cpu().long(), 1, order), torch.gather(idx, 1, want_order))
    near(torch.gather(gw.cpu(), 1, order), torch.gather(w, 1, want_order), "float32", "routing weights", rel32=1e-5)


# ---------------------------------------------------------------------------
# the model through the engine
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(folders, oracles, name, dtype):
    cfg, w = oracles[name]
    eng = tb.Engine(model_of(folders, name, dtype), max_tokens=1024)
    for ids in prompts(cfg["vocab"], [1, 2, 64, 65, 150], seed=1):
        s = eng.start(1)
        got = eng.step(s, [ids], [list(range(len(ids)))])
        eng.release(s)
        close(got, plain.forward(cfg, w, ids), tolerance(name, cfg, w, ids, dtype), f"{name}: whole prompt of {len(ids)}", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_residual_stream_after_every_layer(folders, oracles, name, monkeypatch):
    from trapetum_b200.parts.block import PreNormBlock
    cfg, w = oracles[name]
    ids = prompts(cfg["vocab"], [75], seed=2)[0]
    seq = plain.Sequence(cfg, w)
    seq.feed(ids)
    seen, orig = [], PreNormBlock.forward

    def spy(self, stream, ctx, cache):
        orig(self, stream, ctx, cache)
        seen.append(stream.value().clone())
    monkeypatch.setattr(PreNormBlock, "forward", spy)
    eng = tb.Engine(model_of(folders, name, "float32"), max_tokens=256)
    eng.step(eng.start(1), [ids], [[0]])
    assert len(seen) == len(seq.streams) == len(cfg["layers"])
    for r, x in enumerate(seen):
        near(x, seq.streams[r], "float32", f"{name}: the stream after layer {r} ({cfg['layers'][r]['type']})", rel32=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, first", [("A", 1), ("A", 2), ("B", 63), ("B", 64), ("B", 7), ("C", 65), ("C", 3)])
def test_prompt_then_token_by_token(folders, oracles, name, first, dtype):
    """Decoding runs across pages' borders (64, 128, 192), over every block's and window's edge (blocks of 3 to 100,
    windows of 7 to 65 pass over decoded tokens, and the rows of their rings are used again) and through the capture of
    the step's graph."""
    cfg, w = oracles[name]
    ids = prompts(cfg["vocab"], [215], seed=first)[0]
    truth = plain.forward(cfg, w, ids)
    eng = tb.Engine(model_of(folders, name, dtype), max_tokens=512)
    s = eng.start(1)
    got = [eng.step(s, [ids[:first]], [list(range(first))])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[first:]]
    eng.release(s)
    assert dtype == "float32" or eng.graphs_captured >= 1
    close(torch.cat(got), truth, tolerance(name, cfg, w, ids, dtype, first), f"{name}: {first} tokens, then one by one", dtype)
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
            close(g, truth[i][lo:lo + g.shape[0]], tolerance(name + "u", cfg, w, full[i], dtype, len(ps[i]))[lo:lo + g.shape[0]],
                  f"{name}: request {i} of an unequal batch", dtype)
    eng.check_kernels()


def _layer(kind, size):
    if kind == "attention":
        return mixed(2, 1, 16, 24, 0.25, size=size, rot=rot(8, 10000.0, 2.0))
    if kind == "attention_2":
        return difference(2, 1, 16, 24, 0.25, 0.4, size=size)
    return latent(2, 16, 8, 24, 32, 24, 0.2, size=size, rot=rot(8, 1000.0, 4.0, (32, 8.0, 1.0)))


def _needle(tmp_path, kind, size, key_pos, n, probe):
    """A one-layer model without experts whose scores are sharpened, and a prompt of one repeated token with a single
    other token at ``key_pos``, chosen (with the plain implementation) as the one that the query at ``probe`` singles
    out most."""
    cfg = config(50, 32, [(_layer(kind, size), None)])
    w = random_weights(cfg, 5, sharp=3.0)
    wd = doubles(w)
    base = [3] * n
    without = plain.forward(cfg, wd, base)[probe:probe + 1]
    best, ids = -1.0, None
    for cand in range(4, 24):
        trial = list(base)
        trial[key_pos] = cand
        e = float(position_errors(plain.forward(cfg, wd, trial)[probe:probe + 1], without))
        if e > best:
            best, ids = e, trial
    assert best > 0.05, best
    folder = write_folder(str(tmp_path / f"needle_{kind}_{size}_{key_pos}_{n}"), cfg, w)
    return cfg, wd, ids, folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "attention_2", "latent_attention"])
@pytest.mark.parametrize("key_pos, n", [(0, 200), (63, 130), (64, 130), (5, 700)])
def test_a_far_key_is_found_in_prompts_and_in_decoding(tmp_path, kind, key_pos, n, dtype):
    """No mask: every earlier token is seen, also the first one and those at a page's edge, hundreds of tokens back."""
    cfg, w, ids, folder = _needle(tmp_path, kind, None, key_pos, n, n - 1)
    truth = plain.forward(cfg, w, ids)
    tol = tolerance(("far", kind, key_pos, n), cfg, w, ids, dtype, n - 3)
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), max_tokens=1024)
    s = eng.start(1)
    close(eng.step(s, [ids], [[n - 1]]), truth[-1:], tol[-1:], f"{kind}: needle at {key_pos} of {n}, prompt", dtype)
    eng.release(s)
    s = eng.start(1)
    eng.step(s, [ids[:n - 3]], [[]])
    got = torch.cat([eng.step(s, [[t]], [[0]]).clone() for t in ids[n - 3:]])
    close(got, truth[-3:], tol[-3:], f"{kind}: needle at {key_pos} of {n}, decoded", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind, size, key_pos", [
    ("attention", 48, 48), ("attention", 48, 70), ("attention", 64, 64), ("attention", 65, 130), ("attention", 5, 77), ("attention", 1, 50),
    ("attention", 130, 131), ("attention_2", 48, 96), ("attention_2", 64, 64), ("attention_2", 64, 127), ("attention_2", 65, 65),
    ("attention_2", 100, 150), ("attention_2", 2, 76), ("latent_attention", 48, 1), ("latent_attention", 64, 0), ("latent_attention", 64, 70),
    ("latent_attention", 65, 63), ("latent_attention", 130, 2), ("latent_attention", 2, 77), ("latent_attention", 1, 50)])
def test_a_key_at_the_edge_of_what_is_seen_in_prompts_and_in_decoding(tmp_path, kind, size, key_pos, dtype):
    """The key is seen by the queries up to the end of its block (or of the window that starts at it) and by none after
    it: the logits of the last query that sees it and of the first that does not, in a prompt and decoded."""
    last = (key_pos // size + 1) * size - 1 if kind != "latent_attention" else key_pos + size - 1
    n = last + 3
    cfg, w, ids, folder = _needle(tmp_path, kind, size, key_pos, n, last)
    truth = plain.forward(cfg, w, ids)
    blind = plain.forward(cfg, w, [3] * n)
    assert float(position_errors(truth[last:last + 1], blind[last:last + 1])) > 0.05 or size == 1
    assert float((truth[last + 1:] - blind[last + 1:]).abs().max()) == 0.0
    first = max(1, last - 2)
    tol = tolerance(("edge", kind, size, key_pos), cfg, w, ids, dtype, first)
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), max_tokens=512)
    s = eng.start(1)
    close(eng.step(s, [ids], [list(range(n))]), truth, tol, f"{kind} {size}, key at {key_pos}: prompt", dtype)
    eng.release(s)
    s = eng.start(1)
    got = [eng.step(s, [ids[:first]], [[first - 1]])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[first:]]
    close(torch.cat(got), truth[first - 1:], tol[first - 1:], f"{kind} {size}, key at {key_pos}: decoded", dtype)
    eng.release(s)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_what_the_design_adds_to_plain_attention_would_show(tmp_path, dtype):
    """The engine follows the plain implementation, and the plain implementation without the one in the denominator,
    without the mixing of the heads' scores, without the biases, with the other pairing of the rotation or without
    the gates is far away."""
    cfg = config(60, 40, [(mixed(2, 2, 8, 12, 0.5, size=9, rot=rot(8, 100.0)), moe(4, 2, 16)),
                          (latent(2, 8, 8, 12, 16, 16, 0.4, size=6, rot=rot(8, 100.0, 4.0, (16, 4.0, 1.0))), None)])
    w = {k: v.float() for k, v in random_weights(cfg, 9).items()}
    w["l0.mix.talk"] = torch.tensor([[0.6, 0.9], [-0.8, 1.2]])
    w["l1.mix.g"][0] *= 6.0
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    wd = doubles(w)
    ids = prompts(60, [40], seed=3)[0]
    truth = plain.forward(cfg, wd, ids)
    for name, value in (("l0.mix.talk", torch.eye(2, dtype=F)), ("l0.mix.q.b", torch.zeros(16, dtype=F)), ("l1.mix.g", torch.zeros(2, 40, dtype=F)),
                        ("l0.mix.temp", torch.ones(2, dtype=F))):
        other = dict(wd)
        other[name] = value
        assert float(position_errors(plain.forward(cfg, other, ids), truth).median()) > 0.03, name
    eng = tb.Engine(tb.load_model(write_folder(str(tmp_path / "adds"), cfg, w), dtype, DEV), max_tokens=256)
    s = eng.start(1)
    got = [eng.step(s, [ids[:30]], [list(range(30))])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[30:]]
    close(torch.cat(got), truth, tolerance("adds", cfg, wd, ids, dtype, 30), "mixing, sink, biases, gates: prompt then decoding", dtype)


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
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gemma_run"), folders["A"], "--prompt_ids", "5,17,3",
                           "--max_tokens", "5", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    cfg, w = oracles["A"]
    assert f"continuation ids: {plain.generate_greedy(cfg, w, [5, 17, 3], 5)}" in proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay(folders, oracles, tmp_path, dtype):
    """Two requests start together, are decoded together, one ends early; a third starts from one token later and
    takes the freed slot and pages."""
    cfg, w = oracles["B"]
    a, b, c = prompts(cfg["vocab"], [70, 9, 1], seed=11)
    tail = prompts(cfg["vocab"], [4, 4, 70], seed=12)
    steps = []

    def add(entries, end=()):
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})
    add([{"id": "a", "tokens": a, "want": [0, 69]}, {"id": "b", "tokens": b, "want": [8]}])
    for j in range(4):
        add([{"id": "a", "tokens": [tail[0][j]], "want": [0]}, {"id": "b", "tokens": [tail[1][j]], "want": [0] if j % 2 else []}],
            end=["b"] if j == 1 else [])
        if j == 1:
            break
    add([{"id": "a", "tokens": [tail[0][2]], "want": [0]}], end=["a"])
    add([{"id": "c", "tokens": c, "want": [0]}])
    for j in range(66):
        add([{"id": "c", "tokens": [tail[2][j]], "want": [0] if j >= 60 else []}])
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "512"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=1200)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    full = {"a": a + tail[0][:3], "b": b + tail[1][:2], "c": c + tail[2][:66]}
    truth = {k: plain.forward(cfg, w, v) for k, v in full.items()}
    at = {k: 0 for k in full}
    for st in steps:
        rows = []
        for e in st["entries"]:
            rows += [(e["id"], at[e["id"]] + p) for p in e["want"]]
            at[e["id"]] += len(e["tokens"])
        path = out / f"{st['step']}.f32"
        if not rows:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(rows), cfg["vocab"]))
        for r, (i, p) in enumerate(rows):
            tol = tolerance("trace" + i, cfg, w, full[i], dtype)[p:p + 1]
            close(got[r:r + 1], truth[i][p:p + 1], tol, f"trace: request {i}, position {p}", dtype)
