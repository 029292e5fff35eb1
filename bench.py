#!/usr/bin/env python3
"""Benchmark: decode tokens per second of Gemma-2-shaped models with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 2b|9b|27b] [--batch 8] [--context 8192] [--layers L]
    python bench.py --impl reference ...        # the reference arm: not installable here

A step is one decode step: one new token for each of ``batch`` sequences whose caches hold about
``context`` tokens.  Prints ONE JSON line.  ``value`` is timed on the device with CUDA events around
K steps, as the median of five such regions (``spread`` gives the least and the most, and each region's
median SM clock); ``e2e`` runs the same steps through the public Python API with host token lists in and
host token ids out (a pinned host-to-device copy of the step's inputs and a device-to-host read of the
chosen tokens every step).  ``prefill`` times one 2,048-token prompt; ``roofline`` sets the bytes a decode
step has to read (every weight once, the live requests' cache) against its time; ``points`` repeats the
decode measurement at batch 1 and 64; ``runs`` holds the other measurements that the three model shapes
are quoted on (caches of 2,048 tokens, the 9B shape's unequal batch of 8, the 27B shape from 2,048-token
prompts, each shape's prefill), every one with its bytes or FLOPs, its time and its fraction of the peak.
Weights are made on the device by the counter-based generator (``tb.random_model``).  Peaks come from
MEASURED_PEAKS.json beside this file when the driver wrote it, otherwise from the fallback figures
(6.65 TB/s, 1.59 PFLOP/s).

    python bench.py --design divanex [--sizes small,medium,large] [--batch 8] [--context 2048]
    python bench.py --design lofirax [--sizes small,medium,large] [--batch 8] [--context 2048]
    python bench.py --design fidepel [--sizes small,medium,large] [--batch 8] [--context 2048]
    python bench.py --design fibelix [--sizes small,medium,large] [--batch 8] [--context 2048]

``--design divanex`` is a measurement of its own (the default workload and its line stay as they are): Divanex
models with random weights at a few layer sizes, a 2,048-token prompt and decode steps of ``batch`` sequences
at ``context`` tokens, each beside a Gemma-2 model of the same width, depth, head counts, head size, feed-forward
width and vocabulary on the same host, and the design's own kernels timed alone beside the like kernels of
Gemma-2, each with its fraction of its roofline.

This library runs on one GPU: for --gpus > 1 it says so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

def _shape(L, H, nh, nkv, hd, I, qpas):
    return {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": L, "hidden_size": H,
            "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": I,
            "vocab_size": 256000, "rope_theta": 10000.0, "sliding_window": 4096, "query_pre_attn_scalar": qpas,
            "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6,
            "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "max_position_embeddings": 8192}


# Layer sizes of Gemma-2-2B, -9B and -27B; weights are random (seeds 2, 3, 4).
MODELS = {"2b": _shape(26, 2304, 8, 4, 256, 9216, 256), "9b": _shape(42, 3584, 16, 8, 256, 14336, 256),
          "27b": _shape(46, 4608, 32, 16, 128, 36864, 144)}
SEEDS = {"2b": 2, "9b": 3, "27b": 4}
GEMMA2_2B = MODELS["2b"]
PREFILL_TOKENS = 2048
REPEATS = 5              # timed regions per measurement; the median is reported


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons (NVML, else nvidia-smi) while a timed region runs.  Reads only."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.stamps, self._stop, self._t = [], [], threading.Event(), None

    def _run_nvml(self) -> bool:
        """Reads the same values through NVML every 5 ms (an nvidia-smi call takes longer than a short timed
        region); False if NVML cannot be used here."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(0)
            top = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), reasons(h)
        except Exception:
            return False
        bits = (0x8, 0x40, 0x20, 0x4)          # hw_slowdown, hw_thermal_slowdown, sw_thermal_slowdown, sw_power_cap
        while not self._stop.is_set():
            try:
                mhz, mask = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), int(reasons(h))
                self.rows.append([str(mhz), str(top)] + ["Active" if mask & b else "Not Active" for b in bits])
                self.stamps.append(time.perf_counter())
            except Exception:
                pass
            self._stop.wait(0.005)
        return True

    def _run(self):
        if self._run_nvml():
            return
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    self.rows.append([x.strip() for x in out[0].split(",")])
                    self.stamps.append(time.perf_counter())
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def mhz_between(self, t0, t1):
        """Median SM clock of the samples taken between two host times (None if there is none)."""
        m = sorted(int(r[0]) for r, t in zip(self.rows, self.stamps) if t0 <= t <= t1 and r[0].isdigit())
        return m[len(m) // 2] if m else None

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no samples"]}
        mhz = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(self.rows[0][1]) if self.rows[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(self.rows)}


# ---------------------------------------------------------------------------------------------------------------
# --design divanex: the design at sizes that resemble real layers, beside Gemma-2 at equal size
# ---------------------------------------------------------------------------------------------------------------
# name -> (width, layers, heads, kv heads, head size, ff, state-space heads, their head size, state, vocabulary)
DESIGN_SIZES = {"small": (1024, 12, 8, 2, 128, 4096, 32, 64, 64, 32768),
                "medium": (2048, 16, 16, 4, 128, 8192, 64, 64, 128, 65536),
                "large": (4096, 16, 32, 8, 128, 14336, 128, 64, 128, 131072)}
FP32_TFLOPS_NOMINAL = 72.0      # 148 SMs x 128 FMA x 2 x 1.9 GHz: the bound of 32-bit arithmetic outside the tensor cores


def divanex_config(size):
    W, L, H, G, d, ff, mh, mp, N, V = DESIGN_SIZES[size]
    attn = {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "softcap": 50.0,
                                           "q_temp": {"coef": 0.3, "every": 128}},
            "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}}
    ssm = {"type": "mamba2", "mixer": {"heads": mh, "vdim": mp, "state": N, "groups": 1, "conv": 4, "norm_groups": 1}, "mlp": None}
    return {"architecture": "Divanex", "vocab": V, "width": W, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "postln_alpha": 1.5, "logit_scale": 0.5, "token_side": {"dim": 64},
            "layers": [attn if i % 2 == 0 else ssm for i in range(L)]}


def gemma_like(size):
    W, L, H, G, d, ff, mh, mp, N, V = DESIGN_SIZES[size]
    return dict(_shape(L, W, H, G, d, ff, d), vocab_size=V, sliding_window=4096)


def divanex_bytes_flops(cfg, tokens, ctx, batch):
    """(weight bytes a decode step reads, cache and state bytes per sequence at ``ctx`` tokens, tensor-core FLOPs and
    32-bit recurrence FLOPs of one ``tokens``-token prompt)."""
    W, V = cfg["width"], cfg["vocab"]
    wb, cb, fl, rf = V * W + W, 0, 2 * V * W, 0
    sd = cfg["token_side"]["dim"]
    for L in cfg["layers"]:
        m = L["mixer"]
        per = 2 * sd * W + 2 * W                                    # side gate and proj, norms
        if L["type"] == "attention":
            qd, kvd = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            per += (qd + kvd) * W + W * qd
            cb += 2 * kvd * ctx * 2
            fl += 4 * qd * tokens * (tokens + 1) // 2
        else:
            inner = m["heads"] * m["vdim"]
            ch = inner + 2 * m["groups"] * m["state"]
            per += (inner + ch + m["heads"]) * W + W * inner + ch * m["conv"]
            cb += 2 * 4 * (inner * m["state"] + (m["conv"] - 1) * ch)      # the state is read and written, 32-bit
            rf += tokens * inner * m["state"] * 5
        if L["mlp"]:
            per += 3 * L["mlp"]["ff"] * W
        wb += per
        fl += 2 * tokens * per
    return 2 * wb, cb, fl, rf


def _median_us(torch, fn, flush, reps=15, warm=3):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(reps):
        flush.zero_()                                               # a buffer larger than L2 between timed launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return sorted(ts)[len(ts) // 2]


def design_kernels(torch, size, hbm_gbs, tokens=PREFILL_TOKENS):
    """The design's own kernels alone at ``tokens`` tokens of one prompt, each beside the like kernel of Gemma-2:
    microseconds, algorithmic bytes (or FLOPs) and the fraction of the roofline."""
    from trapetum_b200.csrc import ops
    W, _, H, G, d, ff, mh, mp, N, _ = DESIGN_SIZES[size]
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    T = tokens
    out = {}

    def rec(name, us, nbytes, flops=0.0, like=None, tensor_flops=0.0):
        t_mem, t_fl = nbytes / (hbm_gbs * 1e9) * 1e6, flops / (FP32_TFLOPS_NOMINAL * 1e12) * 1e6
        t_tc = tensor_flops / (peaks()[1] * 1e12) * 1e6
        best = max(t_mem, t_fl, t_tc)
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "roofline_us": round(best, 1), "frac": round(best / us, 3),
                     "bound": "tensor" if best == t_tc else ("fp32" if best == t_fl else "hbm")}
        if like:
            out[name]["like"] = like
    pos = torch.arange(T, device=dev).int()
    tseq = torch.zeros(T, device=dev).int()
    la = torch.tensor([T], device=dev).int()
    pages = (T + 63) // 64
    kp = torch.zeros(pages, G, 64, d, dtype=bf, device=dev)
    vp = torch.zeros_like(kp)
    table = torch.arange(pages, device=dev).int().view(1, pages)
    part = torch.randn(1, T, (H + G) * d, device=dev)
    rec("headnorm_kv", _median_us(torch, lambda: ops.headnorm_kv(part, H, G, d, bf, True, True, True, 1e-5, 0.5, 64, pos, tseq, la, kp, vp, table, 0), flush),
        part.numel() * 4 + T * (H + 2 * G) * d * 2 + T * 2 * G * d * 2, like="rope_kv")
    qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    inv = torch.rand(d // 2, device=dev)
    rec("rope_kv", _median_us(torch, lambda: ops.rope_kv(qkv, H, G, d, d, inv, pos, tseq, la, kp, vp, table, 0), flush),
        T * (H + 2 * G) * d * 2 * 2 + T * 2 * G * d * 2)
    h = torch.randn(T, W, device=dev)
    a = torch.randn(1, T, W, device=dev)
    w = torch.ones(W, device=dev).to(bf)
    rec("fold_rmsnorm", _median_us(torch, lambda: ops.fold_rmsnorm(h, a, w, 1e-5, 0.0, 2.0, bf), flush), T * W * 14, like="add_rmsnorm")
    rec("add_rmsnorm", _median_us(torch, lambda: ops.add_rmsnorm(h, a, w, 1e-5, 0.0, w, 1e-5, 0.0, bf), flush), T * W * 14)
    inner, ch = mh * mp, mh * mp + 2 * N
    proj = torch.randn(T, inner + ch, device=dev).to(bf)
    dtr = torch.randn(T, mh, device=dev)
    f32 = lambda *s: torch.randn(*s, device=dev)
    cw, cb, dtb, Al, D, nw = f32(ch, 4) * .3, f32(ch) * .1, f32(mh) - 1, f32(mh) * .5, f32(mh), f32(inner)
    state = torch.zeros(1, ops.mamba2_state_size(mh, mp, N, 1, 4), device=dev)
    ss = torch.tensor([0, T], device=dev).int()
    slots = torch.zeros(1, device=dev).int()
    # conv + recurrence + gated norm together (three launches, four with the state's update): bytes of the rows
    # they read and write once, FLOPs of the recurrence (5 per state element and token, 32-bit)
    rec("mamba2 (conv, scan, gated norm)",
        _median_us(torch, lambda: ops.mamba2(proj, dtr, mh, mp, N, 1, 4, 1, cw, cb, dtb, Al, D, nw, 1e-5, state, ss, tseq, slots, 1, False,
                                             max_seq_len=T), flush),
        T * (ch * 2 * 3 + inner * 2 + inner * 4 * 2 + inner * 2), flops=T * inner * N * 5.0, like="attention (prefill)")
    # the mixer kernel of the closest model (and of this design's attention layers): causal attention of the prompt
    q = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    rec("attention (prefill)",
        _median_us(torch, lambda: ops.attn_prefill(q[:, :H * d], q[:, H * d:(H + G) * d], q[:, (H + G) * d:], ss, tseq, H, G, d,
                                                   d ** -0.5, 30.0, 0, T, [T], {}), flush),
        T * (H + 2 * G) * d * 2 + T * H * d * 2, tensor_flops=4.0 * H * d * T * (T + 1) / 2)
    # one token for each of 64 sequences: the state is read and written once
    B = 64
    proj1 = torch.randn(B, inner + ch, device=dev).to(bf)
    dtr1 = torch.randn(B, mh, device=dev)
    state64 = torch.zeros(B, ops.mamba2_state_size(mh, mp, N, 1, 4), device=dev)
    ss1 = torch.arange(B + 1, device=dev).int()
    tseq1 = torch.arange(B, device=dev).int()
    rec("mamba2, one token for each of 64 sequences",
        _median_us(torch, lambda: ops.mamba2(proj1, dtr1, mh, mp, N, 1, 4, 1, cw, cb, dtb, Al, D, nw, 1e-5, state64, ss1, tseq1, tseq1, B, True), flush),
        state64.numel() * 8, like="attention (decode)")
    return out


def design_compare(args, torch):
    """Prints one JSON line: per size, Divanex and the Gemma-2 model of equal size (prefill of one 2,048-token prompt,
    decode at ``batch`` x ``context``), with bytes, FLOPs and roofline fractions, and the kernels alone."""
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    hbm_gbs, bf16_tflops, peak_src = peaks()
    warmup = max(3, args.warmup)
    ctx, batch = args.context, args.batch
    sizes = [s for s in args.sizes.split(",") if s in DESIGN_SIZES]
    out = {"design": "divanex", "sizes": {}, "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src,
                                                         "fp32_tflops_nominal": FP32_TFLOPS_NOMINAL},
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "batch": batch, "context": ctx,
           "timing": "CUDA events; decode: median of five regions of --steps steps; kernels alone: a 256 MB buffer is written "
                     "between timed launches (larger than L2)"}
    clocks = ClockSampler()
    clocks.__enter__()
    for size in sizes:
        row = {}
        for which in ("divanex", "gemma2"):
            cfg = divanex_config(size) if which == "divanex" else gemma_like(size)
            V = cfg["vocab"] if which == "divanex" else cfg["vocab_size"]
            model = tb.random_model(cfg, 7, 0.02, 0.1, "bfloat16", "cuda:0", host="python")
            engine = tb.Engine(model, max_tokens=batch * (ctx + 64), max_slots=batch)
            random_cache(engine)
            pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=5, warmup=warmup)
            r = time_decode(engine, torch, [ctx] * batch, args.steps, warmup, V, clocks=clocks)
            if which == "divanex":
                wb, cb, fl, rf = divanex_bytes_flops(cfg, PREFILL_TOKENS, ctx, batch)
                nbytes = wb + batch * cb
                pre_ideal = fl / (bf16_tflops * 1e12) + rf / (FP32_TFLOPS_NOMINAL * 1e12)
            else:
                nbytes = weight_bytes(cfg) + batch * cache_bytes(cfg, ctx)
                fl, rf = prefill_flops(cfg, PREFILL_TOKENS), 0
                pre_ideal = fl / (bf16_tflops * 1e12)
            row[which] = {
                "prefill": {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tok_s": round(PREFILL_TOKENS * 1e3 / pms, 1),
                            "tensor_flops": fl, "fp32_recurrence_flops": rf, "frac_of_roofline": round(pre_ideal * 1e3 / pms, 4)},
                "decode": {"ms": r["ms"], "tok_s": round(batch * 1e3 / r["ms"], 1), "bytes": nbytes,
                           "gbs": round(nbytes / (r["ms"] * 1e-3) / 1e9, 1),
                           "frac_of_hbm": round(nbytes / (r["ms"] * 1e-3) / 1e9 / hbm_gbs, 4), "launches": r["launches"]},
            }
            engine.check_kernels()
            del engine, model
            torch.cuda.empty_cache()
        row["kernels_alone"] = design_kernels(torch, size, hbm_gbs)
        out["sizes"][size] = row
    clocks.__exit__()
    out["clocks"] = clocks.summary()
    out["kernel_errors"] = ops.kernel_errors()
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# --design lofirax: the design at sizes that resemble real layers, beside Divanex (the closest model of the
# library: recurrent and attention layers in turn, on the same host) at equal width, depth and vocabulary
# ---------------------------------------------------------------------------------------------------------------
# name -> (gla heads, key dim, value dim; latent heads, plain dim, rotated dim, value dim, latent rank; experts, top,
#          expert ff, groups, kept groups, shared ff); width, depth, dense ff and vocabulary are DESIGN_SIZES'
LOFIRAX_SIZES = {"small": (4, 128, 256, 8, 128, 64, 128, 448, 16, 4, 512, 4, 2, 1024),
                 "medium": (8, 128, 256, 16, 128, 64, 128, 448, 32, 4, 1024, 8, 4, 2048),
                 "large": (16, 128, 256, 32, 128, 64, 128, 448, 32, 4, 2048, 8, 4, 4096)}
LOFIRAX_RANK = 16


def lofirax_config(size):
    W, L, _, _, _, ff, _, _, _, V = DESIGN_SIZES[size]
    gh, gd, gv, lh, ld, lr, lv, lc, E, top, eff, groups, keep, sff = LOFIRAX_SIZES[size]
    gla = {"type": "gla", "mixer": {"heads": gh, "dim": gd, "vdim": gv, "tau": 8.0, "rank": LOFIRAX_RANK},
           "mlp": {"kind": "dense", "ff": ff}}
    lat = {"type": "latent_attention", "mixer": {"heads": lh, "dim": ld, "rot_dim": lr, "vdim": lv, "kv_rank": lc,
                                                 "scale": (ld + lr) ** -0.5, "rot": {"base": 10000.0, "dims": lr}},
           "mlp": {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}},
                   "shared": {"ff": sff}}}
    # the first two layers run twice: L layer runs from L - 2 layers
    return {"architecture": "Lofirax", "vocab": V, "width": W, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "logit_softcap": 30.0, "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [gla if i % 2 == 0 else lat for i in range(L - 2)]}


def lofirax_bytes_flops(cfg, tokens, ctx, batch):
    """(weight bytes a decode step of ``batch`` sequences reads, with every matrix once and of the experts those that
    ``batch`` tokens are expected to choose; cache and state bytes per sequence at ``ctx`` tokens; tensor-core FLOPs and
    32-bit recurrence FLOPs of one ``tokens``-token prompt)."""
    W, V = cfg["width"], cfg["vocab"]
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    runs = [1] * n
    if lp:
        for i in range(lp["start"], lp["stop"]):
            runs[i] = lp["times"]
    wb, cb, fl, rf = V * W, 0, 2 * V * W * tokens, 0
    for L, r in zip(cfg["layers"], runs):
        m, f = L["mixer"], L["mlp"]
        if L["type"] == "gla":
            HD, HV = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            per = (2 * HD + 2 * HV) * W + W * HV + LOFIRAX_RANK * (W + HD)
            cb += r * 2 * 4 * HD * m["vdim"]                            # the state is read and written, 32-bit
            rf += r * tokens * HD * m["vdim"] * 5
        else:
            H, D, R, Vd, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            per = H * (D + R) * W + (C + R) * W + H * (D + Vd) * C + W * H * Vd
            cb += r * (C + R) * ctx * 2
            fl += r * 2 * (H * (D + R) + H * Vd) * tokens * (tokens + 1) // 2
        used = per
        if f and f["kind"] == "dense":
            per += 3 * f["ff"] * W
            used = per
        elif f:
            E, top = f["router"]["experts"], f["router"]["top"]
            one = 3 * f["expert"]["ff"] * W
            sh = 3 * f["shared"]["ff"] * W + W if f.get("shared") else 0
            used = per + E * W + sh + top * one                          # what a token's products touch
            per += E * W + sh + one * E * (1.0 - (1.0 - top / E) ** batch)   # what a step of ``batch`` tokens is expected to read
        wb += per
        fl += r * 2 * tokens * used
    return int(2 * wb), cb, fl, rf


def lofirax_kernels(torch, size, hbm_gbs, tokens=PREFILL_TOKENS):
    """The design's own kernels alone, each beside the like kernel of the closest model: microseconds, algorithmic
    bytes (or FLOPs) and the fraction of the roofline.  One prompt of ``tokens`` tokens, or one token for each of 64
    sequences at a context of 2,048."""
    from trapetum_b200.csrc import ops
    W, _, H, G, d, ff, mh, mp, N, _ = DESIGN_SIZES[size]
    gh, gd, gv, lh, ld, lr, lv, lc, E, top, eff, groups, keep, sff = LOFIRAX_SIZES[size]
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    T = tokens
    out = {}
    tc_peak = peaks()[1]

    def rec(name, us, nbytes, flops=0.0, like=None, tensor_flops=0.0):
        t_mem, t_fl = nbytes / (hbm_gbs * 1e9) * 1e6, flops / (FP32_TFLOPS_NOMINAL * 1e12) * 1e6
        t_tc = tensor_flops / (tc_peak * 1e12) * 1e6
        best = max(t_mem, t_fl, t_tc)
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "roofline_us": round(best, 1), "frac": round(best / us, 3),
                     "bound": "tensor" if best == t_tc else ("fp32" if best == t_fl else "hbm")}
        if like:
            out[name]["like"] = like
    f32 = lambda *s: torch.randn(*s, device=dev)
    pos = torch.arange(T, device=dev).int()
    tseq = torch.zeros(T, device=dev).int()
    ss = torch.tensor([0, T], device=dev).int()
    slots = torch.zeros(1, device=dev).int()
    # ---- norms
    h, a = f32(T, W), f32(1, T, W)
    w32, b32, wbf = torch.ones(W, device=dev), torch.zeros(W, device=dev), torch.ones(W, device=dev).to(bf)
    rec("add_layernorm", _median_us(torch, lambda: ops.add_layernorm(h, a, w32, b32, 1e-6, bf), flush), T * W * 14, like="add_rmsnorm")
    rec("add_rmsnorm", _median_us(torch, lambda: ops.add_rmsnorm(h, a, wbf, 1e-5, 0.0, wbf, 1e-5, 0.0, bf), flush), T * W * 14)
    # ---- the recurrent mixers: whole prompt
    HD, HV = gh * gd, gh * gv
    proj = torch.randn(T, 2 * HD + 2 * HV, device=dev).to(bf)
    low = f32(1, T, LOFIRAX_RANK)
    a2, a2b, nw = f32(HD, LOFIRAX_RANK) * .3, f32(HD) + 2, torch.ones(gv, device=dev)
    gstate = torch.zeros(1, HD * gv, device=dev)
    rec("gla (decay, scan, gated norm)",
        _median_us(torch, lambda: ops.gla(proj, low, a2, a2b, 8.0, gd ** -0.5, nw, 1e-6, gh, gd, gv, gstate, ss, tseq, slots, 1, max_seq_len=T), flush),
        T * ((2 * HD + 2 * HV) * 2 + HD * 4 * 2 + HV * 4 * 2 + HV * 2), flops=T * HD * gv * 5.0, like="mamba2 (conv, scan, gated norm)")
    inner, ch = mh * mp, mh * mp + 2 * N
    mproj = torch.randn(T, inner + ch, device=dev).to(bf)
    dtr = f32(T, mh)
    cw, cb, dtb, Al, D, mnw = f32(ch, 4) * .3, f32(ch) * .1, f32(mh) - 1, f32(mh) * .5, f32(mh), f32(inner)
    mstate = torch.zeros(1, ops.mamba2_state_size(mh, mp, N, 1, 4), device=dev)
    rec("mamba2 (conv, scan, gated norm)",
        _median_us(torch, lambda: ops.mamba2(mproj, dtr, mh, mp, N, 1, 4, 1, cw, cb, dtb, Al, D, mnw, 1e-5, mstate, ss, tseq, slots, 1, False,
                                             max_seq_len=T), flush),
        T * (ch * 2 * 3 + inner * 2 + inner * 4 * 2 + inner * 2), flops=T * inner * N * 5.0)
    # ---- one token for each of 64 sequences: the states are read and written once
    B = 64
    ss1, tseq1 = torch.arange(B + 1, device=dev).int(), torch.arange(B, device=dev).int()
    proj1, low1 = torch.randn(B, 2 * HD + 2 * HV, device=dev).to(bf), f32(1, B, LOFIRAX_RANK)
    gstate64 = torch.zeros(B, HD * gv, device=dev)
    rec("gla, one token for each of 64 sequences",
        _median_us(torch, lambda: ops.gla(proj1, low1, a2, a2b, 8.0, gd ** -0.5, nw, 1e-6, gh, gd, gv, gstate64, ss1, tseq1, tseq1, B), flush),
        gstate64.numel() * 8, like="mamba2, one token for each of 64 sequences")
    mproj1, dtr1 = torch.randn(B, inner + ch, device=dev).to(bf), f32(B, mh)
    mstate64 = torch.zeros(B, ops.mamba2_state_size(mh, mp, N, 1, 4), device=dev)
    rec("mamba2, one token for each of 64 sequences",
        _median_us(torch, lambda: ops.mamba2(mproj1, dtr1, mh, mp, N, 1, 4, 1, cw, cb, dtb, Al, D, mnw, 1e-5, mstate64, ss1, tseq1, tseq1, B, True), flush),
        mstate64.numel() * 8)
    # ---- what stands between the attention's products and its kernel
    KD = lc + lr
    pages = (T + 63) // 64
    pool = torch.zeros(pages, 1, 64, KD, dtype=bf, device=dev)
    table = torch.arange(pages, device=dev).int().view(1, pages)
    part = f32(1, T, KD)
    inv = torch.rand(lr // 2, device=dev)
    cn = torch.ones(lc, device=dev)
    rec("latent_rows", _median_us(torch, lambda: ops.latent_rows(part, cn, 1e-6, inv, lr, lc, lr, pos, tseq, pool, table, bf), flush),
        T * KD * (4 + 2 + 2), like="headnorm_kv")
    la = torch.tensor([T], device=dev).int()
    kp = torch.zeros(pages, G, 64, d, dtype=bf, device=dev)
    vp = torch.zeros_like(kp)
    hpart = f32(1, T, (H + G) * d)
    rec("headnorm_kv", _median_us(torch, lambda: ops.headnorm_kv(hpart, H, G, d, bf, True, True, True, 1e-5, 0.5, 64, pos, tseq, la, kp, vp, table, 0), flush),
        hpart.numel() * 4 + T * (H + 2 * G) * d * 2 + T * 2 * G * d * 2)
    # ---- causal attention of the prompt
    hd = next(n for n in (64, 128, 256) if n >= max(ld + lr, lv))       # as the part pads it in bfloat16
    q, k, v = (torch.randn(T, lh * hd, device=dev).to(bf) for _ in range(3))
    sink = torch.zeros(lh, device=dev)
    rec("attention with a sink (prefill)", _median_us(torch, lambda: ops.attn_prefill_sink(q, k, v, ss, tseq, lh, hd, 0.07, sink, T, [T]), flush),
        T * lh * hd * 2 * 4, tensor_flops=2.0 * lh * (ld + lr + lv) * T * (T + 1) / 2, like="attention (prefill)")
    q2 = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    rec("attention (prefill)",
        _median_us(torch, lambda: ops.attn_prefill(q2[:, :H * d], q2[:, H * d:(H + G) * d], q2[:, (H + G) * d:], ss, tseq, H, G, d,
                                                   d ** -0.5, 30.0, 0, T, [T], {}), flush),
        T * (H + 2 * G) * d * 2 + T * H * d * 2, tensor_flops=4.0 * H * d * T * (T + 1) / 2)
    # ---- decode attention: 64 sequences at a context of 2,048
    ctx = 2048
    pg = ctx // 64
    lpool = torch.randn(B * pg, 1, 64, KD, device=dev).to(bf)
    ltab = torch.arange(B * pg, device=dev).int().view(B, pg)
    lens = torch.full((B,), ctx, device=dev).int()
    ql = torch.randn(B, lh * KD, device=dev).to(bf)
    rec("latent_decode", _median_us(torch, lambda: ops.latent_decode(ql, lpool, ltab, lens, sink, lh, lc, lr, 0.07, ctx), flush),
        lpool.numel() * 2, like="attention (decode)")
    kp2 = torch.randn(B * pg, G, 64, d, device=dev).to(bf)
    vp2 = torch.randn(B * pg, G, 64, d, device=dev).to(bf)
    qd = torch.randn(B, H * d, device=dev).to(bf)
    rec("attention (decode)", _median_us(torch, lambda: ops.attn_decode(qd, kp2, vp2, ltab, lens, H, G, d, d ** -0.5, 30.0, 0, 0, ctx, 0), flush),
        kp2.numel() * 4)
    # ---- the experts: routing, then the grouped products; beside a dense gated feed-forward's two products
    x = torch.randn(T, W, device=dev).to(bf)
    corr = f32(E) * .1
    logits = f32(1, T, (E + 16) // 16 * 16)
    rec("moe_route", _median_us(torch, lambda: ops.moe_route(logits, E, corr, True, top, groups, keep, 2, 1e-20), flush),
        logits.numel() * 4 + T * top * 8, like="add_rmsnorm")
    idx, wt, gate = ops.moe_route(logits, E, corr, True, top, groups, keep, 2, 1e-20)
    gw, uw, dw = (torch.randn(E, a_, b_, device=dev).to(bf) * .02 for a_, b_ in ((eff, W), (eff, W), (W, eff)))
    gu = torch.stack([ops.interleave_gate_up(gw[e], uw[e]) for e in range(E)]).contiguous()      # as the part binds them
    rec("experts (grouped products)", _median_us(torch, lambda: ops.moe_experts(x, gw, uw, dw, idx, wt, gate_up_w=gu), flush),
        3 * E * eff * W * 2 + T * W * 2, tensor_flops=2.0 * T * top * 3 * eff * W, like="gated feed-forward (two products)")
    wgu = ops.interleave_gate_up(torch.randn(ff, W, device=dev).to(bf) * .02, torch.randn(ff, W, device=dev).to(bf) * .02)
    wdn = torch.randn(W, ff, device=dev).to(bf) * .02

    def dense_ff():
        act = ops.gemm_tc(x, wgu, bf, gated_act="gelu_tanh")
        return ops.gemm_tc(act, wdn, torch.float32, partials=True)
    rec("gated feed-forward (two products)", _median_us(torch, dense_ff, flush), 3 * ff * W * 2 + T * W * 2,
        tensor_flops=2.0 * T * 3 * ff * W)
    return out


def lofirax_compare(args, torch):
    """Prints one JSON line: per size, Lofirax and the Divanex model of equal width, depth and vocabulary (prefill of
    one 2,048-token prompt, decode at ``batch`` x ``context``), with bytes, FLOPs and roofline fractions, and the
    design's kernels alone beside their like kernels."""
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    hbm_gbs, bf16_tflops, peak_src = peaks()
    warmup = max(3, args.warmup)
    ctx, batch = args.context, args.batch
    sizes = [s for s in args.sizes.split(",") if s in DESIGN_SIZES]
    out = {"design": "lofirax", "beside": "divanex", "sizes": {},
           "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src, "fp32_tflops_nominal": FP32_TFLOPS_NOMINAL},
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "batch": batch, "context": ctx,
           "timing": "CUDA events; decode: median of five regions of --steps steps; kernels alone: a 256 MB buffer is written "
                     "between timed launches (larger than L2)"}
    clocks = ClockSampler()
    clocks.__enter__()
    for size in sizes:
        row = {}
        for which in ("lofirax", "divanex"):
            cfg = lofirax_config(size) if which == "lofirax" else divanex_config(size)
            V = cfg["vocab"]
            model = tb.random_model(cfg, 7, 0.02, 0.1, "bfloat16", "cuda:0", host="python")
            engine = tb.Engine(model, max_tokens=batch * (ctx + 64), max_slots=batch)
            random_cache(engine)
            pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=5, warmup=warmup)
            r = time_decode(engine, torch, [ctx] * batch, args.steps, warmup, V, clocks=clocks)
            wb, cb, fl, rf = (lofirax_bytes_flops if which == "lofirax" else divanex_bytes_flops)(cfg, PREFILL_TOKENS, ctx, batch)
            nbytes = wb + batch * cb
            pre_ideal = fl / (bf16_tflops * 1e12) + rf / (FP32_TFLOPS_NOMINAL * 1e12)
            row[which] = {
                "prefill": {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tok_s": round(PREFILL_TOKENS * 1e3 / pms, 1),
                            "tensor_flops": fl, "fp32_recurrence_flops": rf, "frac_of_roofline": round(pre_ideal * 1e3 / pms, 4)},
                "decode": {"ms": r["ms"], "tok_s": round(batch * 1e3 / r["ms"], 1), "bytes": nbytes,
                           "gbs": round(nbytes / (r["ms"] * 1e-3) / 1e9, 1),
                           "frac_of_hbm": round(nbytes / (r["ms"] * 1e-3) / 1e9 / hbm_gbs, 4), "launches": r["launches"]},
            }
            engine.check_kernels()
            del engine, model
            torch.cuda.empty_cache()
        if not args.no_points:
            row["kernels_alone"] = lofirax_kernels(torch, size, hbm_gbs)
        out["sizes"][size] = row
    clocks.__exit__()
    out["clocks"] = clocks.summary()
    out["kernel_errors"] = ops.kernel_errors()
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# --design fidepel: the design at sizes that resemble real layers, beside Gemma-2 (the closest model of the library:
# every layer a rotary, windowed, grouped-query attention over the same cache and attention kernels) at equal width,
# depth, head counts, head size and vocabulary; its experts' kernels beside Lofirax's gated ones at equal sizes
# ---------------------------------------------------------------------------------------------------------------
# name -> (value size, window; experts, top, expert ff, groups, kept groups, shared ff); width, depth, heads, kv heads,
#          head size and vocabulary are DESIGN_SIZES'
FIDEPEL_SIZES = {"small": (128, 4096, 16, 4, 512, 4, 2, 1024),
                 "medium": (128, 4096, 32, 4, 1024, 8, 4, 2048),
                 "large": (128, 4096, 32, 4, 2048, 8, 4, 4096)}


def fidepel_config(size):
    W, L, H, G, d, _, _, _, _, V = DESIGN_SIZES[size]
    vd, window, E, top, eff, groups, keep, sff = FIDEPEL_SIZES[size]
    layer = {"type": "attention",
             "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": vd, "scale": d ** -0.5, "mask": {"size": window},
                       "rot": {"dims": d, "base": 10000.0, "scaling": {"factor": 2.0}}},
             "mlp": {"kind": "moe", "expert": {"ff": eff},
                     "router": {"experts": E, "top": top, "scale": 2.0, "groups": {"count": groups, "keep": keep}},
                     "shared": {"ff": sff}}}
    # the first two layers run twice: L layer runs from L - 2 layers
    return {"architecture": "Fidepel", "vocab": V, "width": W, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [layer for _ in range(L - 2)]}


def fidepel_bytes_flops(cfg, tokens, ctx, batch):
    """(weight bytes a decode step of ``batch`` sequences reads, with every matrix once and of the experts those that
    ``batch`` tokens are expected to choose; cache bytes per sequence at ``ctx`` tokens; tensor-core FLOPs of one
    ``tokens``-token prompt)."""
    W, V = cfg["width"], cfg["vocab"]
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    runs = [1] * n
    if lp:
        for i in range(lp["start"], lp["stop"]):
            runs[i] = lp["times"]
    wb, cb, fl = V * W, 0, 2 * V * W * tokens
    for L, r in zip(cfg["layers"], runs):
        m, f = L["mixer"], L["mlp"]
        H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        per = (H * D + G * (D + Vd) + H) * W + W * H * Vd
        pad = next((s for s in (64, 128, 256) if max(D, Vd) <= s), (max(D, Vd) + 15) // 16 * 16)
        seen = min(ctx, (m.get("mask") or {}).get("size") or ctx)
        cb += r * 2 * G * pad * seen * 2
        span = min(tokens, (m.get("mask") or {}).get("size") or tokens)
        pairs = span * (span + 1) // 2 + (tokens - span) * span          # (query, key) pairs that a window leaves
        fl += r * 2 * H * (D + Vd) * pairs
        used = per
        if f:
            E, top = f["router"]["experts"], f["router"]["top"]
            one = 2 * f["expert"]["ff"] * W
            sh = 2 * f["shared"]["ff"] * W if f.get("shared") else 0
            used = per + E * W + sh + top * one
            per += E * W + sh + one * E * (1.0 - (1.0 - top / E) ** batch)
        wb += per
        fl += r * 2 * tokens * used
    return int(2 * wb), cb, fl, 0


def fidepel_kernels(torch, size, hbm_gbs, tokens=PREFILL_TOKENS):
    """The design's own kernels alone, each beside the like kernel of the closest model: microseconds, algorithmic
    bytes (or FLOPs) and the fraction of the roofline.  One prompt of ``tokens`` tokens."""
    from trapetum_b200.csrc import ops
    W, _, H, G, d, ff, _, _, _, _ = DESIGN_SIZES[size]
    vd, window, E, top, eff, groups, keep, sff = FIDEPEL_SIZES[size]
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    T = tokens
    out = {}
    tc_peak = peaks()[1]

    def rec(name, us, nbytes, like=None, tensor_flops=0.0):
        t_mem, t_tc = nbytes / (hbm_gbs * 1e9) * 1e6, tensor_flops / (tc_peak * 1e12) * 1e6
        best = max(t_mem, t_tc)
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "roofline_us": round(best, 1), "frac": round(best / us, 3),
                     "bound": "tensor" if best == t_tc else "hbm"}
        if like:
            out[name]["like"] = like
    f32 = lambda *s: torch.randn(*s, device=dev)
    pos = torch.arange(T, device=dev).int()
    tseq = torch.zeros(T, device=dev).int()
    la = torch.tensor([T], device=dev).int()
    ss = torch.tensor([0, T], device=dev).int()
    # ---- the scaled sum of both branches with the next layer's norm; beside the sum of one branch with two norms
    h, a, b = f32(T, W), f32(1, T, W), f32(1, T, W)
    w32, wbf = torch.ones(W, device=dev), torch.ones(W, device=dev).to(bf)
    rec("add_scaled_rmsnorm (two branches)", _median_us(torch, lambda: ops.add_scaled_rmsnorm(h, [a, b], 0.5, w32, 1e-6, 0.0, bf), flush),
        T * W * 18, like="add_rmsnorm")
    rec("add_rmsnorm", _median_us(torch, lambda: ops.add_rmsnorm(h, a, wbf, 1e-5, 0.0, wbf, 1e-5, 0.0, bf), flush), T * W * 14)
    # ---- what stands between the fused projection and the attention kernel
    D = ops.attn_padded_head(bf, max(d, vd))
    pages = (T + 63) // 64
    kp = torch.zeros(pages, G, 64, D, dtype=bf, device=dev)
    vp = torch.zeros_like(kp)
    table = torch.arange(pages, device=dev).int().view(1, pages)
    in_w = (H * d + G * (d + vd) + H + 15) // 16 * 16
    part = f32(1, T, in_w)
    wq, wk, temp = torch.ones(H * d, device=dev), torch.ones(G * d, device=dev), torch.ones(H, device=dev)
    inv = torch.rand(d // 2, device=dev)
    rec("projnorm_kv", _median_us(torch, lambda: ops.projnorm_kv(part, H, G, d, vd, D, bf, wq, wk, 1e-6, temp, d, inv, True, pos, tseq, la,
                                                                 kp, vp, table, 0), flush),
        part.numel() * 4 + T * (H + 2 * G) * D * 2 + T * 2 * G * D * 2, like="rope_kv")
    qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    kp2 = torch.zeros(pages, G, 64, d, dtype=bf, device=dev)
    vp2 = torch.zeros_like(kp2)
    rec("rope_kv", _median_us(torch, lambda: ops.rope_kv(qkv, H, G, d, d, inv, pos, tseq, la, kp2, vp2, table, 0), flush),
        T * (H + 2 * G) * d * 2 * 2 + T * 2 * G * d * 2)
    o, gate = torch.randn(T, H * D, device=dev).to(bf), torch.rand(T, H, device=dev)
    rec("head_gate", _median_us(torch, lambda: ops.head_gate(o, gate, H), flush), T * H * D * 4 + T * H * 4, like="add_rmsnorm")
    # ---- causal attention of the prompt: the design's and the closest model's are one kernel
    rec("attention (prefill)",
        _median_us(torch, lambda: ops.attn_prefill(qkv[:, :H * d], qkv[:, H * d:(H + G) * d], qkv[:, (H + G) * d:], ss, tseq, H, G, d,
                                                   d ** -0.5, 0.0, window, T, [T], {}), flush),
        T * (H + 2 * G) * d * 2 + T * H * d * 2, tensor_flops=4.0 * H * d * T * (T + 1) / 2)
    # ---- routing and the experts; beside the gated experts of equal sizes and a dense gated feed-forward
    x = torch.randn(T, W, device=dev).to(bf)
    logits = f32(1, T, (E + 15) // 16 * 16)
    rec("moe_route (softmax)", _median_us(torch, lambda: ops.moe_route(logits, E, None, False, top, groups, keep, 1, 1e-20, "softmax", 2.0), flush),
        logits.numel() * 4 + T * top * 8, like="moe_route (sigmoid)")
    corr = f32(E) * .1
    rec("moe_route (sigmoid)", _median_us(torch, lambda: ops.moe_route(logits, E, corr, False, top, groups, keep, 2, 1e-20), flush),
        logits.numel() * 4 + T * top * 8)
    idx, wt, _ = ops.moe_route(logits, E, None, False, top, groups, keep, 1, 1e-20, "softmax", 2.0)
    gw, uw, dw = (torch.randn(E, a_, b_, device=dev).to(bf) * .02 for a_, b_ in ((eff, W), (eff, W), (W, eff)))
    rec("experts without a gate (grouped products)", _median_us(torch, lambda: ops.moe_experts(x, None, uw, dw, idx, wt), flush),
        2 * E * eff * W * 2 + T * W * 2, tensor_flops=2.0 * T * top * 2 * eff * W, like="gated experts (grouped products)")
    gu = torch.stack([ops.interleave_gate_up(gw[e], uw[e]) for e in range(E)]).contiguous()
    rec("gated experts (grouped products)", _median_us(torch, lambda: ops.moe_experts(x, gw, uw, dw, idx, wt, gate_up_w=gu), flush),
        3 * E * eff * W * 2 + T * W * 2, tensor_flops=2.0 * T * top * 3 * eff * W)
    su, sd = torch.randn(sff, W, device=dev).to(bf) * .02, torch.randn(W, sff, device=dev).to(bf) * .02

    def shared_ff():
        return ops.gemm_tc(ops.gemm_tc(x, su, bf, unary_act="relu2"), sd, torch.float32, partials=True)
    rec("shared expert (two products)", _median_us(torch, shared_ff, flush), 2 * sff * W * 2 + T * W * 2,
        tensor_flops=2.0 * T * 2 * sff * W, like="gated feed-forward (two products)")
    wgu = ops.interleave_gate_up(torch.randn(sff, W, device=dev).to(bf) * .02, torch.randn(sff, W, device=dev).to(bf) * .02)

    def dense_ff():
        return ops.gemm_tc(ops.gemm_tc(x, wgu, bf, gated_act="gelu_tanh"), sd, torch.float32, partials=True)
    rec("gated feed-forward (two products)", _median_us(torch, dense_ff, flush), 3 * sff * W * 2 + T * W * 2,
        tensor_flops=2.0 * T * 3 * sff * W)
    # ---- one token for each of 64 sequences at a context of 2,048: what a decode step adds to the closest model's
    B, ctx = 64, 2048
    pg = ctx // 64
    pos1, tseq1 = torch.full((B,), ctx - 1, device=dev).int(), torch.arange(B, device=dev).int()
    la1 = torch.full((B,), ctx, device=dev).int()
    kp3 = torch.randn(B * pg, G, 64, D, device=dev).to(bf)
    vp3 = torch.randn(B * pg, G, 64, D, device=dev).to(bf)
    tab = torch.arange(B * pg, device=dev).int().view(B, pg)
    part1 = f32(4, B, in_w)
    rec("projnorm_kv, one token for each of 64 sequences",
        _median_us(torch, lambda: ops.projnorm_kv(part1, H, G, d, vd, D, bf, wq, wk, 1e-6, temp, d, inv, True, pos1, tseq1, la1, kp3, vp3, tab, 0), flush),
        part1.numel() * 4 + B * (H + 4 * G) * D * 2, like="rope_kv, one token for each of 64 sequences")
    part2 = f32(4, B, (H + 2 * G) * d)
    qkv1 = torch.empty(B, (H + 2 * G) * d, dtype=bf, device=dev)
    kp4 = torch.zeros(B * pg, G, 64, d, dtype=bf, device=dev)
    vp4 = torch.zeros_like(kp4)
    rec("rope_kv, one token for each of 64 sequences",
        _median_us(torch, lambda: ops.rope_kv(qkv1, H, G, d, d, inv, pos1, tseq1, la1, kp4, vp4, tab, 0, partial=part2), flush),
        part2.numel() * 4 + B * (H + 4 * G) * d * 2)
    del kp4, vp4
    qd = torch.randn(B, H * D, device=dev).to(bf)
    rec("attention (decode)", _median_us(torch, lambda: ops.attn_decode(qd, kp3, vp3, tab, la1, H, G, D, d ** -0.5, 0.0, window, 0, ctx, 0), flush),
        kp3.numel() * 4)
    x1 = torch.randn(B, W, device=dev).to(bf)
    idx1 = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(B)]).int()
    wt1 = torch.rand(B, top, device=dev)
    touched = E * (1.0 - (1.0 - top / E) ** B)
    rec("experts without a gate, one token for each of 64 sequences", _median_us(torch, lambda: ops.moe_experts(x1, None, uw, dw, idx1, wt1), flush),
        2 * touched * eff * W * 2, like="gated experts, one token for each of 64 sequences")
    rec("gated experts, one token for each of 64 sequences", _median_us(torch, lambda: ops.moe_experts(x1, gw, uw, dw, idx1, wt1, gate_up_w=gu), flush),
        3 * touched * eff * W * 2)
    return out


def fidepel_compare(args, torch):
    """Prints one JSON line: per size, Fidepel and the Gemma-2 model of equal width, depth, heads and vocabulary
    (prefill of one 2,048-token prompt, decode at ``batch`` x ``context``), with bytes, FLOPs and roofline fractions,
    and the design's kernels alone beside their like kernels."""
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    hbm_gbs, bf16_tflops, peak_src = peaks()
    warmup = max(3, args.warmup)
    ctx, batch = args.context, args.batch
    sizes = [s for s in args.sizes.split(",") if s in DESIGN_SIZES]
    out = {"design": "fidepel", "beside": "gemma2", "sizes": {},
           "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src},
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "batch": batch, "context": ctx,
           "timing": "CUDA events; decode: median of five regions of --steps steps; kernels alone: a 256 MB buffer is written "
                     "between timed launches (larger than L2)"}
    clocks = ClockSampler()
    clocks.__enter__()
    for size in sizes:
        row = {}
        for which in ("fidepel", "gemma2"):
            cfg = fidepel_config(size) if which == "fidepel" else gemma_like(size)
            V = cfg["vocab"] if which == "fidepel" else cfg["vocab_size"]
            model = tb.random_model(cfg, 7, 0.02, 0.1, "bfloat16", "cuda:0", host="python")
            engine = tb.Engine(model, max_tokens=batch * (ctx + 64), max_slots=batch)
            random_cache(engine)
            pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=5, warmup=warmup)
            r = time_decode(engine, torch, [ctx] * batch, args.steps, warmup, V, clocks=clocks)
            if which == "fidepel":
                wb, cb, fl, _ = fidepel_bytes_flops(cfg, PREFILL_TOKENS, ctx, batch)
                nbytes = wb + batch * cb
            else:
                nbytes = weight_bytes(cfg) + batch * cache_bytes(cfg, ctx)
                fl = prefill_flops(cfg, PREFILL_TOKENS)
            pre_ideal = fl / (bf16_tflops * 1e12)
            row[which] = {
                "prefill": {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tok_s": round(PREFILL_TOKENS * 1e3 / pms, 1),
                            "tensor_flops": fl, "frac_of_roofline": round(pre_ideal * 1e3 / pms, 4)},
                "decode": {"ms": r["ms"], "tok_s": round(batch * 1e3 / r["ms"], 1), "bytes": nbytes,
                           "gbs": round(nbytes / (r["ms"] * 1e-3) / 1e9, 1),
                           "frac_of_hbm": round(nbytes / (r["ms"] * 1e-3) / 1e9 / hbm_gbs, 4), "launches": r["launches"]},
            }
            engine.check_kernels()
            del engine, model
            torch.cuda.empty_cache()
        if not args.no_points:
            row["kernels_alone"] = fidepel_kernels(torch, size, hbm_gbs)
        out["sizes"][size] = row
    clocks.__exit__()
    out["clocks"] = clocks.summary()
    out["kernel_errors"] = ops.kernel_errors()
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# --design fibelix: the design at sizes that resemble real layers, beside Fidepel (the closest model of the library:
# rotary attention with a number per head, a mask that bounds what a query sees, values of their own size, and
# softmax-routed experts, on the same host) at equal width, depth, head counts, head size and vocabulary
# ---------------------------------------------------------------------------------------------------------------
# name -> (blocks of the mixed attention, blocks of the difference attention, window of the latent attention,
#          latent: rotated dims, kv rank, q rank; experts, top, expert ff); the rest are DESIGN_SIZES'
FIBELIX_SIZES = {"small": (1024, 512, 1024, 64, 448, 768, 16, 4, 512),
                 "medium": (1024, 512, 1024, 64, 448, 1024, 32, 4, 1024),
                 "large": (1024, 512, 1024, 64, 448, 1536, 32, 4, 2048)}


def fibelix_config(size):
    W, L, H, G, d, _, _, _, _, V = DESIGN_SIZES[size]
    blk, blk2, win, R, C, Q, E, top, eff = FIBELIX_SIZES[size]
    mlp = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}}
    layers, last_own = [], None
    for i in range(L):
        kind = i % 3
        if kind == 0:
            layer = {"type": "latent_attention",
                     "mixer": {"heads": H, "dim": d, "rot_dim": R, "vdim": d, "kv_rank": C, "q_rank": Q, "scale": (d + R) ** -0.5,
                               "mask": {"size": win},
                               "rot": {"dims": R, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
        elif kind == 1:
            layer = {"type": "attention",
                     "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": blk},
                               "rot": {"dims": d // 2, "base": 500000.0, "scaling": {"factor": 8.0}}}}
        else:
            m = {"heads": H // 2, "kv_heads": G, "dim": d // 2, "vdim": d, "scale": (d // 2) ** -0.5, "diff": 0.6,
                 "mask": {"size": blk2}}
            if last_own is None:
                last_own = i
            else:
                m["kv_from"], last_own = last_own, None          # every second one reads the one before it
            layer = {"type": "attention_2", "mixer": m}
        layer["mlp"] = mlp
        layers.append(layer)
    return {"architecture": "Fibelix", "vocab": V, "width": W, "norm": {"eps": 1e-6}, "layers": layers}


def fibelix_bytes_flops(cfg, tokens, ctx, batch):
    """(weight bytes a decode step of ``batch`` sequences reads, with every matrix once and of the experts those that
    ``batch`` tokens are expected to choose; cache bytes per sequence that a step at ``ctx`` tokens reads; tensor-core
    FLOPs of one ``tokens``-token prompt, the (query, key) pairs that the masks leave)."""
    W, V = cfg["width"], cfg["vocab"]
    wb, cb, fl = V * W, 0, 2 * V * W * tokens

    def pairs(span, blocks):
        span = min(tokens, span or tokens)
        if blocks:
            full, rest = divmod(tokens, span)
            return full * span * (span + 1) // 2 + rest * (rest + 1) // 2
        return span * (span + 1) // 2 + (tokens - span) * span
    for L in cfg["layers"]:
        m, f = L["mixer"], L["mlp"]
        H, D, Vd = m["heads"], m["dim"], m["vdim"]
        size = (m.get("mask") or {}).get("size")
        if L["type"] == "latent_attention":
            R, C, Q = m["rot_dim"], m["kv_rank"], m["q_rank"]
            per = (Q + C + R + H) * W + H * (D + R) * Q + H * (D + Vd) * C + W * H * Vd
            cb += (C + R) * min(ctx, size or ctx) * 2
            fl += 2 * H * (D + R + Vd) * pairs(size, False) + 2 * tokens * H * (D + Vd) * C
        elif L["type"] == "attention":
            G = m["kv_heads"]
            per = (H * D + G * (D + Vd)) * W + W * H * Vd
            seen = (ctx - 1) % size + 1 if size else ctx
            cb += G * (D + Vd) * seen * 2
            fl += 2 * H * (D + Vd) * pairs(size, True)
        else:
            G = m["kv_heads"]
            own = m.get("kv_from") is None
            per = H * 2 * D * W + (G * (2 * D + Vd) * W if own else 0) + W * H * Vd
            seen = (ctx - 1) % size + 1 if size else ctx
            cb += G * (2 * D + Vd) * seen * 2
            fl += 2 * 2 * H * (D + Vd) * pairs(size, True)
        used = per
        if f:
            E, top = f["router"]["experts"], f["router"]["top"]
            one = 3 * f["expert"]["ff"] * W
            used = per + E * W + top * one
            per += E * W + one * E * (1.0 - (1.0 - top / E) ** batch)
        wb += per
        fl += 2 * tokens * used
    return int(2 * wb), cb, fl, 0


def fibelix_kernels(torch, size, hbm_gbs, tokens=PREFILL_TOKENS):
    """The design's own kernels alone, each beside the like kernel of the closest model: microseconds, algorithmic
    bytes (or FLOPs) and the fraction of the roofline.  One prompt of ``tokens`` tokens; 64 sequences at 2,048 for
    the one-token kernels."""
    from trapetum_b200.csrc import ops
    W, _, H, G, d, _, _, _, _, _ = DESIGN_SIZES[size]
    blk, blk2, win, R, C, Q, E, top, eff = FIBELIX_SIZES[size]
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    T = tokens
    out = {}
    tc_peak = peaks()[1]

    def rec(name, us, nbytes, like=None, tensor_flops=0.0, fp32_flops=0.0):
        t_mem, t_tc = nbytes / (hbm_gbs * 1e9) * 1e6, tensor_flops / (tc_peak * 1e12) * 1e6
        t_fma = fp32_flops / (FP32_TFLOPS_NOMINAL * 1e12) * 1e6
        best = max(t_mem, t_tc, t_fma)
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "roofline_us": round(best, 1), "frac": round(best / us, 3),
                     "bound": "tensor" if best == t_tc else ("fp32" if best == t_fma else "hbm")}
        if like:
            out[name]["like"] = like
    rb = lambda *s: (torch.randn(*s, device=dev) * 0.5).to(bf)
    pos = torch.arange(T, device=dev).int()
    tseq = torch.zeros(T, device=dev).int()
    ss = torch.tensor([0, T], device=dev).int()
    # ---- prompts: scores mixed across heads (blocks, a unit sink) beside the plain attention kernel over the same blocks
    q, k, v = rb(T, H * d), rb(T, G * d), rb(T, G * d)
    mix = (torch.eye(H, device=dev) + 0.1 * torch.randn(H, H, device=dev)) * d ** -0.5
    n_pairs = (T // blk) * blk * (blk + 1) // 2 + (T % blk) * (T % blk + 1) // 2
    starts = torch.arange(0, T + 1, blk, device=dev).int()
    lens = [blk] * (T // blk)
    rec("attention with mixed scores (prefill)", _median_us(torch, lambda: ops.attn_mixed_prefill(q, k, v, ss, tseq, H, G, d, mix, -blk, True, T), flush),
        (2 * H + 2 * G) * d * T * 2, like="attention (prefill)", tensor_flops=4.0 * H * d * n_pairs)
    rec("attention (prefill)", _median_us(torch, lambda: ops.attn_prefill(q, k, v, starts, tseq, H, G, d, d ** -0.5, 0.0, 0, blk, lens), flush),
        (2 * H + 2 * G) * d * T * 2, tensor_flops=4.0 * H * d * n_pairs)
    # ---- difference attention: twice the heads at half the size over the same kernel, then the fold of the pairs
    H2, d2 = H // 2, d // 2
    qd, kd, vd_ = rb(T, 2 * H2 * d), rb(T, G * d), rb(T, G * d)
    starts2 = torch.arange(0, T + 1, blk2, device=dev).int()
    n_pairs2 = (T // blk2) * blk2 * (blk2 + 1) // 2
    rec("difference attention (prefill: two maps a head)", _median_us(torch, lambda: ops.attn_prefill(qd, kd, vd_, starts2, tseq, 2 * H2, G, d, d2 ** -0.5, 0.0, 0, blk2, [blk2] * (T // blk2)), flush),
        (4 * H2 + 2 * G) * d * T * 2, like="attention (prefill)", tensor_flops=4.0 * 2 * H2 * d * n_pairs2)
    o2 = rb(T, 2 * H2 * d)
    rec("head_difference", _median_us(torch, lambda: ops.head_difference(o2, H2, d, d, 0.55, 1e-6, 0.4), flush), 3 * H2 * d * T * 2, like="head_gate")
    og, gate = rb(T, H * d), torch.rand(T, H, device=dev)
    rec("head_gate", _median_us(torch, lambda: ops.head_gate(og, gate, H), flush), 2 * H * d * T * 2)
    # ---- latent rows with the queries' latent and the gates, beside the rows alone
    wide = C + R + Q + H
    wide += -wide % 16
    part, part0 = torch.randn(1, T, wide, device=dev), torch.randn(1, T, C + R, device=dev)
    wc, wq = torch.ones(C, device=dev), torch.ones(Q, device=dev)
    inv = torch.rand(R // 2, device=dev)
    pool = torch.zeros((T // 64 + 1, 1, 64, C + R), dtype=bf, device=dev)
    table = torch.arange(T // 64 + 1, device=dev).int()[None]
    la = torch.tensor([T], device=dev).int()
    rec("latent_rows with the queries' latent and gates", _median_us(torch, lambda: ops.latent_rows(part, wc, 1e-6, inv, R, C, R, pos, tseq, pool, table, bf, 0, la, 1.3, wq, H), flush),
        T * ((C + R + Q + H) * 4 + (2 * (C + R) + Q) * 2 + H * 4), like="latent_rows")
    rec("latent_rows", _median_us(torch, lambda: ops.latent_rows(part0, wc, 1e-6, inv, R, C, R, pos, tseq, pool, table, bf), flush),
        T * (C + R) * (4 + 4))
    # ---- one token for each of 64 sequences at 2,048
    B, ctx = 64, 2048
    pages = ctx // 64
    lens_d = torch.full((B,), ctx, device=dev).int()
    tab = torch.arange(B * pages, device=dev).int().view(B, pages)
    kp, vp = rb(B * pages, G, 64, d), rb(B * pages, G, 64, d)
    q1 = rb(B, H * d)
    seen = (ctx - 1) % blk + 1
    rec("attention with mixed scores (decode), 64 sequences", _median_us(torch, lambda: ops.attn_mixed_decode(q1, kp, vp, tab, lens_d, H, G, d, mix, -blk, True, 0, ctx), flush),
        B * 2 * G * d * seen * 2, like="attention (decode) over the same blocks")
    rec("attention (decode) over the same blocks", _median_us(torch, lambda: ops.attn_decode(q1, kp, vp, tab, lens_d, H, G, d, d ** -0.5, 0.0, -blk, 0, 2048), flush),
        B * 2 * G * d * seen * 2)
    lp = rb(B * pages, 1, 64, C + R)
    ql = rb(B, H * (C + R))
    rec("latent_decode through a window, 64 sequences", _median_us(torch, lambda: ops.latent_decode(ql, lp, tab, lens_d, None, H, C, R, 0.07, ctx, win, 0), flush),
        B * (C + R) * min(win, ctx) * 2, like="latent_decode")
    rec("latent_decode", _median_us(torch, lambda: ops.latent_decode(ql, lp, tab, lens_d, None, H, C, R, 0.07, ctx), flush),
        B * (C + R) * ctx * 2)
    return out


def fibelix_compare(args, torch):
    """Prints one JSON line: per size, Fibelix and the Fidepel model of equal width, depth, heads and vocabulary
    (prefill of one 2,048-token prompt, decode at ``batch`` x ``context``), with bytes, FLOPs and roofline fractions,
    and the design's kernels alone beside their like kernels."""
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    hbm_gbs, bf16_tflops, peak_src = peaks()
    warmup = max(3, args.warmup)
    ctx, batch = args.context, args.batch
    sizes = [s for s in args.sizes.split(",") if s in DESIGN_SIZES]
    out = {"design": "fibelix", "beside": "fidepel", "sizes": {},
           "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src},
           "dtype": "bf16", "data": "synthetic (random weights, random token ids)", "batch": batch, "context": ctx,
           "timing": "CUDA events; decode: median of five regions of --steps steps; kernels alone: a 256 MB buffer is written "
                     "between timed launches (larger than L2)"}
    clocks = ClockSampler()
    clocks.__enter__()
    for size in sizes:
        row = {}
        for which in ("fibelix", "fidepel"):
            cfg = fibelix_config(size) if which == "fibelix" else fidepel_config(size)
            V = cfg["vocab"]
            model = tb.random_model(cfg, 7, 0.02, 0.1, "bfloat16", "cuda:0", host="python")
            engine = tb.Engine(model, max_tokens=batch * (ctx + 64), max_slots=batch)
            random_cache(engine)
            pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=5, warmup=warmup)
            r = time_decode(engine, torch, [ctx] * batch, args.steps, warmup, V, clocks=clocks)
            wb, cb, fl, _ = (fibelix_bytes_flops if which == "fibelix" else fidepel_bytes_flops)(cfg, PREFILL_TOKENS, ctx, batch)
            nbytes = wb + batch * cb
            pre_ideal = fl / (bf16_tflops * 1e12)
            row[which] = {
                "prefill": {"tokens": PREFILL_TOKENS, "ms": round(pms, 3), "tok_s": round(PREFILL_TOKENS * 1e3 / pms, 1),
                            "tensor_flops": fl, "frac_of_roofline": round(pre_ideal * 1e3 / pms, 4)},
                "decode": {"ms": r["ms"], "tok_s": round(batch * 1e3 / r["ms"], 1), "bytes": nbytes,
                           "gbs": round(nbytes / (r["ms"] * 1e-3) / 1e9, 1),
                           "frac_of_hbm": round(nbytes / (r["ms"] * 1e-3) / 1e9 / hbm_gbs, 4), "launches": r["launches"]},
            }
            engine.check_kernels()
            del engine, model
            torch.cuda.empty_cache()
        if not args.no_points:
            row["kernels_alone"] = fibelix_kernels(torch, size, hbm_gbs)
        out["sizes"][size] = row
    clocks.__exit__()
    out["clocks"] = clocks.summary()
    out["kernel_errors"] = ops.kernel_errors()
    print(json.dumps(out))
    return 0


HOST = None              # which host runs the models (None: the library's default, the native host for these models)


def build_model(cfg, seed):
    import trapetum_b200 as tb
    return tb.random_model(cfg, seed, 0.02, 0.1, "bfloat16", "cuda:0", host=HOST)


def launches():
    """Kernel launches of this process so far, on whichever host runs the steps."""
    import sys as _sys
    from trapetum_b200.csrc import ops
    nat = _sys.modules.get("trapetum_b200.native")
    return ops.launches() + (nat.launches() if nat is not None and nat._lib is not None else 0)


def weight_bytes(cfg):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (qd + 2 * kvd) * H + H * qd + 2 * I * H + H * I + 4 * H
    return 2 * (L * per_layer + V * H + H)          # the embedding table is read once, as the output head


def cache_bytes(cfg, ctx):
    """Key and value bytes one sequence with ``ctx`` tokens makes a decode step read."""
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    W = cfg["sliding_window"]
    total = 0
    for i in range(cfg["num_hidden_layers"]):
        rows = min(ctx, W) if i % 2 == 0 else ctx
        total += rows * kvd * 2 * 2
    return total


def prefill_flops(cfg, lens):
    """FLOPs of one step that brings whole prompts of these lengths (the head runs on each last position)."""
    if isinstance(lens, int):
        lens = [lens]
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    lin = 2 * sum(lens) * ((qd + 2 * kvd) * H + H * qd + 2 * I * H + H * I)
    W = cfg["sliding_window"]
    att = 0
    for i in range(L):
        for T in lens:
            if i % 2 == 0 and T > W:
                pairs = W * (W + 1) // 2 + (T - W) * W
            else:
                pairs = T * (T + 1) // 2
            att += 4 * qd * pairs
    return L * lin + att + 2 * V * H * len(lens)


def fill_cache(engine, lens):
    """Sequences whose caches hold ``lens`` tokens of random keys and values (no prefill is run:
    the decode step's work does not depend on what the keys are)."""
    slots = engine.start(len(lens))
    engine.cache.grow({s: n for s, n in zip(slots, lens)})
    return slots


def time_decode(engine, torch, ctxs, steps, warmup, vocab, repeats=REPEATS, e2e=False, clocks=None):
    """Decode steps of a batch whose caches hold about ``ctxs`` tokens (one number per sequence; they end the
    measurement at these lengths).  ``repeats`` regions of ``steps`` steps each are timed with CUDA events.
    Returns a dict: ms (median per step), ms_min, ms_max, regions [{ms, sm_mhz}], mean_ctx (per sequence, over
    the timed steps), launches (per step), and with ``e2e`` also e2e_ms and h2d."""
    from trapetum_b200.csrc import ops
    batch = len(ctxs)
    g = torch.Generator().manual_seed(batch)
    total = warmup + repeats * steps + (2 * warmup + steps if e2e else 0)
    start = [max(1, c - total) for c in ctxs]
    slots = fill_cache(engine, start)
    out = {}
    try:
        toks = torch.randint(0, vocab, (total + 2, batch), generator=g).tolist()
        it = iter(toks)
        for _ in range(warmup):
            engine.step(slots, [[t] for t in next(it)], borrow=True)
        torch.cuda.synchronize()
        regions, done = [], warmup
        n0 = launches()
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e0.record()
            for _ in range(steps):
                engine.step(slots, [[t] for t in next(it)], borrow=True)
            e1.record()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            regions.append({"ms": round(e0.elapsed_time(e1) / steps, 4),
                            "sm_mhz": clocks.mhz_between(t0, t1) if clocks is not None else None})
        out["launches"] = (launches() - n0) // (repeats * steps)
        ms = sorted(r["ms"] for r in regions)
        out.update(ms=ms[len(ms) // 2], ms_min=ms[0], ms_max=ms[-1], regions=regions)
        # the context each timed step reads: the tokens before it, and its own
        first = [s0 + warmup + 1 for s0 in start]
        out["mean_ctx"] = [f + (repeats * steps - 1) / 2.0 for f in first]
        if e2e:
            # end to end: host token lists in, chosen token ids out, each step feeding the next
            cur = next(it)
            for _ in range(warmup):
                cur = engine.step_tokens(slots, [[t] for t in cur])
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                cur = engine.step_tokens(slots, [[t] for t in cur])
            torch.cuda.synchronize()
            out["e2e_ms"] = (time.perf_counter() - t0) * 1e3 / steps
            out["h2d"] = engine.last_h2d_bytes
        return out
    finally:
        engine.release(slots)


def time_generate(engine, torch, ctx, batch, steps, warmup, vocab):
    """Decode steps through the generation entry point (``tb.generate``: host prompts in, host tokens out through the
    per-token callback): prompts that fill the caches to about ``ctx`` tokens, then ``warmup + steps`` new tokens
    each; the times between the callbacks of a request's tokens give ms per step: (median, mean).  Every step
    copies its inputs from pinned host memory and its chosen ids back to the host.  The median is the steady step:
    right after the prompts' own step (tens of thousands of tokens on the tensor cores at the power cap) the clocks
    stay low for some tens of milliseconds, which the mean of a short run shows and the median does not."""
    import trapetum_b200 as tb
    g = torch.Generator().manual_seed(1000 + batch)
    warmup = warmup + 100          # the clocks need about 120 ms to come back after the prompts' step: those steps are not timed
    n_new = warmup + steps + 1
    prompts = torch.randint(0, vocab, (batch, max(1, ctx - n_new)), generator=g).tolist()
    stamps = []

    def on_token(request, token):
        if request == 0:
            stamps.append(time.perf_counter())
    tb.generate(engine, prompts, max_tokens=n_new, stop_ids=[], max_batch=batch, on_token=on_token)
    torch.cuda.synchronize()
    gaps = sorted((b - a) * 1e3 for a, b in zip(stamps[warmup:], stamps[warmup + 1:]))
    return gaps[len(gaps) // 2], (stamps[-1] - stamps[warmup]) * 1e3 / (len(stamps) - 1 - warmup)


def decode_record(cfg, r, hbm_gbs):
    """What a decode measurement says against the memory roofline."""
    nbytes = weight_bytes(cfg) + sum(cache_bytes(cfg, int(round(c))) for c in r["mean_ctx"])
    gbs = nbytes / (r["ms"] * 1e-3) / 1e9
    return {"value": round(len(r["mean_ctx"]) * 1e3 / r["ms"], 1), "unit": "tokens/s", "ms": r["ms"],
            "ms_min": r["ms_min"], "ms_max": r["ms_max"], "bytes": nbytes, "gbs": round(gbs, 1),
            "frac": round(gbs / hbm_gbs, 4)}


def time_prefill(engine, torch, lens, vocab, reps, warmup):
    """One step that brings whole prompts of ``lens`` tokens: (median ms on the device, median ms of host time
    to issue the step, median ms from the call to the logits' arrival on the host)."""
    if isinstance(lens, int):
        lens = [lens]
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    dev, host, whole = [], [], []
    for i in range(warmup + reps):
        s = engine.start(len(lens))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        logits = engine.step(s, prompts, borrow=True)
        e1.record()
        t1 = time.perf_counter()
        logits[:, :8].cpu()
        t2 = time.perf_counter()
        torch.cuda.synchronize()
        engine.release(s)
        if i >= warmup:
            dev.append(e0.elapsed_time(e1)); host.append((t1 - t0) * 1e3); whole.append((t2 - t0) * 1e3)
    med = lambda v: sorted(v)[len(v) // 2]
    return med(dev), med(host), med(whole)


def prefill_record(cfg, lens, ms, host_ms, e2e_ms, bf16_tflops):
    lens = [lens] if isinstance(lens, int) else lens
    fl = prefill_flops(cfg, lens)
    return {"value": round(sum(lens) * 1e3 / ms, 1), "unit": "tokens/s", "tokens": sum(lens), "ms": round(ms, 3),
            "host_ms": round(host_ms, 3), "e2e_ms": round(e2e_ms, 3), "flops": fl,
            "frac": round(fl / (ms * 1e-3) / (bf16_tflops * 1e12), 4)}


def random_cache(engine):
    for g in engine.cache.groups:                         # random keys and values, small enough for a sane softmax
        g.k.normal_(0.0, 0.5)
        g.v.normal_(0.0, 0.5)


def other_runs(torch, which, steps, warmup, hbm_gbs, bf16_tflops, have=None):
    """The measurements beside the headline: per model shape, decode at batch 1/8/64 with caches of 2,048 tokens
    (the 9B shape: its unequal batch of 8, prompts U[64, 2048], decode and the prompts' own step), and a
    2,048-token prompt.  ``have``: (name, model) already built.  Models are built and freed one after another."""
    from trapetum_b200 import Engine
    runs = {}
    for name in which:
        cfg = MODELS[name]
        V = cfg["vocab_size"]
        model = have[1] if have and have[0] == name else build_model(cfg, SEEDS[name])
        engine = Engine(model, max_tokens=64 * 2112, max_slots=64)
        random_cache(engine)
        st = max(8, steps // 2)
        for b in (1, 8, 64):
            r = time_decode(engine, torch, [2048] * b, st, warmup, V, repeats=3)
            runs[f"{name}_decode_b{b}_ctx2048"] = decode_record(cfg, r, hbm_gbs)
        if name == "9b":
            lens = torch.randint(64, 2049, (8,), generator=torch.Generator().manual_seed(3)).tolist()
            r = time_decode(engine, torch, lens, st, warmup, V, repeats=3)
            rec = decode_record(cfg, r, hbm_gbs)
            rec["prompt_lens"] = " ".join(map(str, lens))
            runs["9b_decode_unequal_b8"] = rec
            runs["9b_prefill_unequal_b8"] = prefill_record(cfg, lens, *time_prefill(engine, torch, lens, V, 3, 3), bf16_tflops)
        if name != "2b":
            runs[f"{name}_prefill_{PREFILL_TOKENS}"] = prefill_record(
                cfg, PREFILL_TOKENS, *time_prefill(engine, torch, PREFILL_TOKENS, V, 3, 3), bf16_tflops)
        del engine, model
        have = None
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    return runs


def leave_out_report(engine, model, cfg, torch, args, warmup) -> int:
    """What each kind of launch costs inside the step's graph: the step is timed whole, then with that kind
    replaced by a stand-in that launches nothing and returns a buffer of the right shape."""
    from trapetum_b200.csrc import ops
    from trapetum_b200.engine import Engine
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    real = {k: getattr(ops, k) for k in ("attn_decode", "add_rmsnorm", "gemm_tc")}
    bufs = {}

    def buf(key, shape, dtype):
        k = (key, tuple(shape), dtype)
        if k not in bufs:
            bufs[k] = torch.zeros(shape, dtype=dtype, device="cuda:0")
        return bufs[k]

    def no_attn(q, *a, **kw):
        rows = q.shape[1] if q.dim() == 3 else q.shape[0]
        return buf("attn", (rows, qd), torch.bfloat16)

    def no_norm(h, a, wa, ea, oa, wb=None, eps_b=0.0, off_b=0.0, out_dtype=None):
        return buf("norm", h.shape, out_dtype) if wb is not None else None

    def no_gemm(shape):
        def f(a, w, out_dtype, softcap=0.0, splits=None, out=None, partials=False, gated_act=None):
            if tuple(w.shape) != shape:
                return real["gemm_tc"](a, w, out_dtype, softcap, splits, out, partials, gated_act)
            M, N = a.shape[0], w.shape[0]
            if gated_act:
                return buf("g", (M, N // 2), torch.bfloat16)
            return buf("p", (1, M, N), torch.float32) if partials else buf("o", (M, N), out_dtype)
        return f

    kinds = {"nothing": {}, "attention": {"attn_decode": no_attn}, "add_rmsnorm": {"add_rmsnorm": no_norm},
             "gemm qkv": {"gemm_tc": no_gemm((qd + 2 * kvd, H))}, "gemm o": {"gemm_tc": no_gemm((H, qd))},
             "gemm gate_up": {"gemm_tc": no_gemm((2 * I, H))}, "gemm down": {"gemm_tc": no_gemm((H, I))},
             "gemm head": {"gemm_tc": no_gemm((V, H))}}
    whole = None
    try:
        for name, patch in kinds.items():
            for k, v in real.items():
                setattr(ops, k, v)
            for k, v in patch.items():
                setattr(ops, k, v)
            eng = Engine(model, max_tokens=args.batch * args.context, max_slots=args.batch)
            r = time_decode(eng, torch, [args.context] * args.batch, args.steps, warmup, V, repeats=1)
            ms, launches = r["ms"], r["launches"]
            whole = ms if whole is None else whole
            print(json.dumps({"left_out": name, "ms_per_step": round(ms, 4), "launches": launches,
                              "saves_us": round((whole - ms) * 1e3, 1),
                              "saves_us_per_layer": round((whole - ms) * 1e3 / args.layers, 2)}), flush=True)
            del eng
    finally:
        for k, v in real.items():
            setattr(ops, k, v)
    return 0


def gemm_compare(cfg, torch, tokens, bf16_tflops):
    """The four products of a layer at ``tokens`` tokens, this library's tensor-core kernel beside torch.matmul
    (cuBLAS), as a comparison only: neither result feeds a bench number.  Each launch gets another of three weight
    matrices, so the weights come from memory; 12 launches are captured in a CUDA graph and timed as one."""
    from trapetum_b200.csrc import ops
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    shapes = [("qkv", qd + 2 * kvd, H), ("o", H, qd), ("gate_up", 2 * I, H), ("down", H, I)]
    g0 = torch.Generator(device="cuda").manual_seed(1)

    def timed(fn, reps=12):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                fn(i)
        best = None
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); graph.replay(); e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) / reps
            best = t if best is None else min(best, t)
        return best

    for name, N, K in shapes:
        a = (torch.randn(tokens, K, device="cuda", generator=g0) * 0.5).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device="cuda", generator=g0) * 0.05).to(torch.bfloat16) for _ in range(3)]
        outs = [torch.empty(tokens, N, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
        ours = timed(lambda i: ops.gemm_tc(a, ws[i % 3], torch.bfloat16))
        lib = timed(lambda i: torch.matmul(a, ws[i % 3].t(), out=outs[i % 3]))
        fl = 2.0 * tokens * N * K
        print(json.dumps({"product": name, "tokens": tokens, "weight_rows": N, "k": K,
                          "ours_us": round(ours * 1e3, 1), "ours_tflops": round(fl / ours / 1e9, 1),
                          "torch_matmul_us": round(lib * 1e3, 1), "torch_matmul_tflops": round(fl / lib / 1e9, 1),
                          "ours_over_torch": round(lib / ours, 3),
                          "ours_frac_of_peak": round(fl / (ours * 1e-3) / (bf16_tflops * 1e12), 3)}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="2b", choices=sorted(MODELS), help="the headline's model shape")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has (same layer sizes); both numbers are reported")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points, the prefill and the other runs")
    ap.add_argument("--no-e2e", action="store_true",
                    help="skip the end-to-end run through tb.generate (it starts with 8 prompts of about 8,000 tokens); the "
                         "step-loop figure then stands in its place (for short captures under a profiler)")
    ap.add_argument("--runs", default="2b,9b,27b",
                    help="model shapes whose other measurements (caches of 2,048 tokens, prefill) are taken: a comma "
                         "list out of 2b, 9b, 27b, or 'none'")
    ap.add_argument("--host", default=None, choices=["native", "python"],
                    help="the host that runs the steps (default: the library's own choice, the native host)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="instead of the bench line: time only the prompt of 2,048 tokens and print one line about it")
    ap.add_argument("--leave-out", action="store_true",
                    help="instead of the bench line: the decode step re-timed with one kind of launch left out at a "
                         "time (its results are then wrong; only its time is of interest), one line per kind")
    ap.add_argument("--design", default=None, choices=["divanex", "lofirax", "fidepel", "fibelix"],
                    help="instead of the bench line: this design at the layer sizes of --sizes beside the library's closest "
                         "model at equal size (divanex beside Gemma-2, lofirax beside divanex, fidepel beside Gemma-2, fibelix beside fidepel)")
    ap.add_argument("--sizes", default="small,medium,large", help="with --design: which of small, medium, large")
    ap.add_argument("--gemm-compare", type=int, default=0, metavar="TOKENS",
                    help="instead of the bench line: the four products of a layer of --model at TOKENS tokens, this "
                         "library's kernel beside torch.matmul, one line per product (a comparison only)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "neuralboot/trapetum is a Rust crate (no setup.py or pyproject.toml: pip reports 'not "
                          "installable'); no cargo/rustc in this image, and its Gemma-2 path runs 4-bit codebook "
                          "weights only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: trapetum_b200 is a single-GPU library; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    warmup = max(3, args.warmup)

    import torch
    if args.design:
        if args.context == 8192:
            args.context = 2048
        if args.design == "fidepel":
            return fidepel_compare(args, torch)
        if args.design == "fibelix":
            return fibelix_compare(args, torch)
        return lofirax_compare(args, torch) if args.design == "lofirax" else design_compare(args, torch)
    if args.gemm_compare:
        return gemm_compare(MODELS[args.model], torch, args.gemm_compare, peaks()[1])
    from trapetum_b200 import Engine
    global HOST
    HOST = "python" if args.leave_out else args.host
    full = MODELS[args.model]
    args.layers = args.layers or full["num_hidden_layers"]
    cfg = dict(full, num_hidden_layers=args.layers)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    model = build_model(cfg, SEEDS[args.model])
    V = cfg["vocab_size"]
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    per_token = 4 * cfg["num_key_value_heads"] * cfg["head_dim"] * cfg["num_hidden_layers"]      # key and value bytes
    if max_batch > args.batch and max_batch * args.context * per_token + weight_bytes(cfg) > 150e9:
        max_batch = args.batch                            # the batch-64 point does not fit beside these weights
    engine = Engine(model, max_tokens=max_batch * args.context, max_slots=max(max_batch, args.batch))
    random_cache(engine)

    if args.leave_out:
        return leave_out_report(engine, model, cfg, torch, args, warmup)
    if args.prefill_only:
        pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=max(1, args.steps), warmup=warmup)
        print(json.dumps({"prefill_ms": round(pms, 3), "host_ms": round(hms, 3), "e2e_ms": round(wms, 3),
                          "tokens": PREFILL_TOKENS, "layers": args.layers,
                          "frac": round(prefill_flops(cfg, PREFILL_TOKENS) / (pms * 1e-3) / (bf16_tflops * 1e12), 4),
                          "of": peak_src}))
        return 0

    with ClockSampler() as clocks:
        r = time_decode(engine, torch, [args.context] * args.batch, args.steps, warmup, V, e2e=True, clocks=clocks)
    dev_ms, loop_ms = r["ms"], r["e2e_ms"]
    e2e_ms = e2e_mean_ms = loop_ms                     # replaced below by the run through tb.generate
    rec = decode_record(cfg, r, hbm_gbs)
    csum = clocks.summary()
    mhz = csum.get("sm_mhz")

    out = {
        "metric": "decode tok/s at batch %d (Gemma-2-%s)" % (args.batch, args.model.upper()),
        "value": rec["value"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights seed %d made on the device, uniform token ids, random "
                                 "cache contents)" % SEEDS[args.model],
        "config": {"model": "gemma-2-%s-shape" % args.model, "global_batch": args.batch, "seq_len": args.context,
                   "parallelism": "1 gpu", "layers": args.layers, "layers_of_model": full["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "window": cfg["sliding_window"],
                   "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (each step reads every weight)",
                   "timed": "median of %d regions of %d steps" % (REPEATS, args.steps), "peaks": peak_src,
                   "host": type(engine).__module__.split(".")[-1].replace("engine", "python")},
        "clocks": csum,
        "spread": {"ms_min": r["ms_min"], "ms_max": r["ms_max"], "regions": r["regions"],
                   "ms_x_ghz": round(dev_ms * mhz / 1e3, 4) if mhz else None},
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": 4 * args.batch,
                "how": "engine.step_tokens in a loop: host tokens in, the chosen tokens back on the host, every step",
                "mean_ms_per_step": round(e2e_mean_ms, 4),
                "step_loop_value": round(args.batch * 1e3 / loop_ms, 1), "step_loop_ms": round(loop_ms, 4)},
        "gpu_launches": r["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": rec["gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": rec["frac"], "of": peak_src, "bytes_per_step": rec["bytes"]},
    }
    if not args.no_points:
        pts, runs = {}, {}
        for b in (1, 64):
            if b > engine.cache.max_slots:
                continue
            rb = time_decode(engine, torch, [args.context] * b, max(8, args.steps // 2), warmup, V, repeats=3, e2e=(b == 1))
            rr = decode_record(cfg, rb, hbm_gbs)
            pts[f"decode_b{b}"] = rr["value"]
            if b == 1:
                pts["e2e_b1_step_loop"] = round(1e3 / rb["e2e_ms"], 1)
            runs[f"{args.model}_decode_b{b}_ctx{args.context}"] = rr
        pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=5, warmup=3)
        prec = prefill_record(cfg, PREFILL_TOKENS, pms, hms, wms, bf16_tflops)
        out["prefill"] = dict(prec, of=peak_src)
        out["points"] = pts
        if not args.no_e2e:
            pts["e2e_b1"] = round(1e3 / time_generate(engine, torch, args.context, 1, max(8, args.steps // 2), warmup, V)[0], 1)
        if not args.no_e2e:
            e2e_ms, e2e_mean_ms = time_generate(engine, torch, args.context, args.batch, args.steps, warmup, V)
            out["e2e"].update(value=round(args.batch * 1e3 / e2e_ms, 1), ms_per_step=round(e2e_ms, 4),
                              mean_ms_per_step=round(e2e_mean_ms, 4),
                              how="tb.generate: host prompts in, tokens out through its callback; median time between a "
                                  "request's tokens, the first hundred after the prompts' step left out")
        which = [] if args.runs == "none" else [w for w in args.runs.split(",") if w in MODELS]
        if args.layers != full["num_hidden_layers"]:
            which = []                                  # the other runs are of whole models
        del engine
        torch.cuda.empty_cache()
        have = (args.model, model)
        del model
        runs.update(other_runs(torch, which, args.steps, warmup, hbm_gbs, bf16_tflops, have))
        for k, v in runs.items():
            if "decode" in k:
                pts.setdefault(k, v["value"])
        out["runs"] = runs
    from trapetum_b200.csrc import ops
    err = ops.kernel_errors()
    if err:
        out["error"] = f"a bounded wait ran out: {err}"
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
