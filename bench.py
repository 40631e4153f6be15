"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference] [--shape 1b|3b|8b]

A step is one decode step of the whole batch.  The default run has the layer sizes of the
Llama-3.2-1B-shaped benchmark configuration with random weights ~N(0, 0.02) (seed 2), a
batch of 8 and a context that reaches 4,096 tokens.  `value` is decoded tokens a second
timed on the device over K steps fed with the previous step's tokens on the device; `e2e`
is the same through `Engine.add_request` / `Engine.step`, host token ids in and out.
Every timed window is repeated (five times for the headline) and the median is reported with the
smallest and largest beside it.  Also reported: a 2,048-token prefill, the decode step against the
HBM roofline, clocks sampled while timing, how many of this package's kernels ran, and under
`points`: decode and end-to-end decode at batch 1 and 64, decode at batch 8 with temperature
sampling, the Llama-3.1-8B-shaped model at 8 of its 32 layers (decode at batch 1, 8, 64, a
2,048-token prefill, one 32,768-token prompt in portions of 8,192 with the share of time spent in
attention), the Llama-3.2-3B-shaped model at 8 of its 28 layers serving 64 requests at once, and
this engine's attention and GEMM kernels timed against the reference's own attention kernels
(compiled unmodified, see baseline/reference_kernels.py) and the library GEMM on the same data.
`--shape` takes the layer sizes of the 3B or 8B benchmark configuration for the headline instead;
`--only decode|prefill|serve` runs one part alone and prints its time.  `--family dirurax` (or `pikalix`, `sotazen`, `linedra`) leaves
all of that aside and prints a line of its own: prefill and decode of that family's models at two sizes beside
Llama models of the same width, depth, feed-forward width and vocabulary, and that family's kernels alone against
their rooflines.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

def _llama(layers, hidden, heads, kv_heads, head_dim, inter, factor, tied):
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=layers,
                hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                intermediate_size=inter, vocab_size=128256, rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192),
                rms_norm_eps=1e-5, tie_word_embeddings=tied, max_position_embeddings=131072)


# the benchmark configurations: the Llama-3.2-1B shape is the default and the headline; the
# 3B and 8B shapes are there for --shape (further sizes, head size 128, an untied head)
SHAPES = {"1b": ("Llama-3.2-1B-shaped", _llama(16, 2048, 32, 8, 64, 8192, 32.0, True)),
          "3b": ("Llama-3.2-3B-shaped", _llama(28, 3072, 24, 8, 128, 8192, 32.0, True)),
          "8b": ("Llama-3.1-8B-shaped", _llama(32, 4096, 32, 8, 128, 14336, 8.0, False))}
SEED, STD = 2, 0.02
CONTEXT, PREFILL_TOKENS, PAGE = 4096, 2048, 16
# Decode steps run untimed between the burst that fills the context and the warm-up: for some 80
# steps after such a burst a step takes up to 14 % longer (1.20, 1.14, 1.11, 1.07, 1.06, 1.055 ms in
# windows of 16 steps at batch 8), the GPU's clocks coming back from the burst's power draw; what
# is measured is the steady state the metric names.
SETTLE_STEPS = 96
NOMINAL_HBM_GBS, NOMINAL_BF16_TFLOPS = 6650.0, 1590.0      # fallback when no measured peaks are given


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return NOMINAL_HBM_GBS, NOMINAL_BF16_TFLOPS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        # the timed regions are tens of milliseconds long and follow one another closely:
        # every sample from the first region's start to the last one's end was taken under load
        if windows:
            windows = [(min(a for a, _ in windows), max(b for _, b in windows))]
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, c in self.rows:
            if len(c) < 7 or not any(a <= t <= b for a, b in windows):
                continue
            try:
                sm.append(float(c[0])); mx = max(mx, float(c[1]))
            except ValueError:
                continue
            for n, v in zip(names, c[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, layers):
    d, inter, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (q + 2 * kv) + q * d + 3 * d * inter
    weight_bytes = 2 * (layers * (per_layer + 2 * d) + V * d + d)       # bf16; the head is the tied table
    kv_bytes_per_token = layers * 2 * kv * 2
    return per_layer, weight_bytes, kv_bytes_per_token, q


def fill_context(engine, batch, ctx0, vocab, seed):
    """Open `batch` requests and bring each to ctx0 cached tokens through the step function."""
    import random
    from rustinfer_b200.engine.runner import StepEntry
    r = engine.runner
    rng = random.Random(seed)
    ids = []
    for b in range(batch):
        rid = ("bench", seed, b)
        r.open(rid)
        ids.append(rid)
        at = 0
        while at < ctx0:
            n = min(ctx0 - at, r.max_batch_tokens)
            r.step([StepEntry(rid, [rng.randrange(vocab) for _ in range(n)], [])])
            at += n
    return ids


def median_of(run, repeats):
    """`run()` -> (ms, ...): the run whose ms is the median of `repeats` runs, with all the ms."""
    runs = sorted((run() for _ in range(repeats)), key=lambda r: r[0])
    return runs[len(runs) // 2], [round(r[0], 4) for r in runs]


def decode_device_timed(engine, batch, steps, warmup, vocab, seed, context=CONTEXT, sampling=None):
    """K decode steps of `batch` requests that end at `context` tokens; device time.  With
    `sampling` (SamplingParams) every row's token is drawn on the device instead of the argmax."""
    import torch
    from rustinfer_b200.engine.runner import StepEntry
    from rustinfer_b200.ops import library
    r = engine.runner
    settle = min(SETTLE_STEPS, max(0, context - (steps + warmup) - 16))     # (a short context leaves less room)
    ctx0 = context - (steps + warmup + settle)
    ids = fill_context(engine, batch, ctx0, vocab, seed)
    tokens = torch.randint(0, vocab, (batch,), dtype=torch.int32, device=r.device)
    entries = [StepEntry(rid, [0], [0]) for rid in ids]

    at = [ctx0]

    def one():
        nonlocal tokens
        logits = r.step(entries, device_tokens=tokens)
        if sampling is None:
            tokens = engine.sampler.argmax_device(logits)
        else:
            at[0] += 1
            tokens = engine.sampler.sample_device(logits, [sampling] * batch, list(range(batch)), [at[0]] * batch)

    r_step = r.step
    r.step = lambda e, device_tokens=None: r_step(e, device_tokens=device_tokens, borrow_logits=True)
    for _ in range(settle + warmup):
        one()
    torch.cuda.synchronize()
    l0 = library.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    w1 = time.time()
    ms = e0.elapsed_time(e1)
    launches = library.launch_count - l0
    r.step = r_step
    for rid in ids:
        r.close(rid)
    return ms / steps, launches, (w0, w1)


def decode_e2e(engine, batch, steps, warmup, vocab, seed, trace=False):
    """The same decode steps through the public entry point: host token ids in and out.  With
    `trace`, `engine.stats.host_seconds` holds the host's time in the timed steps afterwards."""
    import random
    import torch
    from rustinfer_b200.sampling.params import SamplingParams
    rng = random.Random(seed)
    # requests whose prompt is done keep decoding while the others' prompts are computed, so
    # leave room for those extra tokens and end nothing inside the timed region
    ctx0 = CONTEXT - (steps + warmup + SETTLE_STEPS) - 4 * batch - 8
    if batch > 8:                                            # prompts of 64 requests take many steps of 8,192 tokens
        ctx0 = CONTEXT - (steps + warmup + SETTLE_STEPS) - (batch * CONTEXT) // 8192 - batch - 16
    sp = SamplingParams(max_tokens=CONTEXT, ignore_eos=True)
    for _ in range(batch):
        engine.add_request([rng.randrange(vocab) for _ in range(ctx0)], sp)
    while any(q.computed < len(q.prompt) for q in engine._requests.values()):
        engine.step()                                       # prompts (untimed)
    for _ in range(SETTLE_STEPS + warmup):
        engine.step()
    torch.cuda.synchronize()
    if trace:
        engine.stats.host_seconds.clear()
        engine.trace_host = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    got = 0
    for _ in range(steps - 1):
        got += len(engine.step())
    e1.record()
    engine.trace_host = False
    torch.cuda.synchronize()
    w1 = time.time()
    ms = e0.elapsed_time(e1) / (steps - 1)
    h2d = engine.runner.h2d_bytes_last
    for rid in list(engine._requests):
        engine.abort(rid)
    torch.cuda.synchronize()
    assert got == batch * (steps - 1), (got, batch, steps)
    return ms, h2d, batch * 8, (w0, w1)       # read back per step: a token id and a stop flag per request


def prefill_timed(engine, vocab, tokens, repeats=3):
    import random
    import torch
    from rustinfer_b200.engine.runner import StepEntry
    r = engine.runner
    rng = random.Random(7)
    times, windows = [], []
    for i in range(repeats + 1):                            # the first run warms up
        rid = ("prefill", i)
        r.open(rid)
        prompt = [rng.randrange(vocab) for _ in range(tokens)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        logits = r.step([StepEntry(rid, prompt, [tokens - 1])])
        engine.sampler.argmax_device(logits)
        e1.record()
        torch.cuda.synchronize()
        windows.append((w0, time.time()))
        ms = e0.elapsed_time(e1)
        r.close(rid)
        if i > 0:
            times.append(ms)
    return statistics.median(times), windows[1:]


def serve_workload(folder, vocab, layers, quiet=False):
    """Continuous batching through the public entry point: 64 requests arrive at once, prompt
    lengths uniform in [128, 2048], 256 tokens out each, prompts computed in portions of 512
    beside the decoding of the others.  Tokens a second over the whole run (host time:
    scheduling, launches and the reading of every token included), and the time from one
    step's launch to the next."""
    import random
    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=64, max_model_len=CONTEXT,
                    paged_block_size=PAGE, chunked_prefill_size=512, num_blocks=64 * 2560 // PAGE,
                    ignore_eos=True)
    rng = random.Random(3)
    prompts = [[rng.randrange(vocab) for _ in range(rng.randint(128, 2048))] for _ in range(64)]
    engine.generate([p[:64] for p in prompts[:8]], SamplingParams(max_tokens=8, ignore_eos=True))   # warm-up
    torch.cuda.synchronize()
    steps0 = engine.stats.steps
    ids = [engine.add_request(p, SamplingParams(max_tokens=256, ignore_eos=True)) for p in prompts]
    marks = []
    t0 = time.perf_counter()
    while engine.has_unfinished():
        engine.step()
        marks.append(time.perf_counter())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    results = [engine.take_finished(i) for i in ids]
    gaps = sorted((b - a) * 1e3 for a, b in zip(marks, marks[1:]))
    n_in, n_out = sum(len(p) for p in prompts), sum(len(r.tokens) for r in results)
    out = {"seconds": round(dt, 4), "out_tok_s": round(n_out / dt, 1), "tok_s": round((n_in + n_out) / dt, 1),
           "steps": engine.stats.steps - steps0, "preemptions": engine.stats.preemptions,
           "step_ms_mean": round(sum(gaps) / len(gaps), 4), "step_ms_p99": round(gaps[int(0.99 * (len(gaps) - 1))], 4),
           "prompt_tokens": n_in, "out_tokens": n_out}
    if not quiet:
        print(f"serve layers{layers}: {len(prompts)} requests, {n_in} prompt tokens, {n_out} tokens out in {dt:.3f} s: "
              f"{n_out / dt:.0f} out tok/s, {(n_in + n_out) / dt:.0f} tok/s in all, {out['steps']} steps "
              f"(mean {out['step_ms_mean']} ms, p99 {out['step_ms_p99']} ms), {out['preemptions']} preemptions")
    del engine
    torch.cuda.empty_cache()
    return out


def long_prompt(folder, vocab, cfg, layers, tokens=32768, portion=8192):
    """One prompt of `tokens` tokens computed in portions through the step function; the time of
    the attention kernels alone is taken with events around every layer's attention."""
    import random
    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.engine.runner import StepEntry
    from rustinfer_b200.parts.attention import GQAAttention
    engine = Engine(folder, dtype="bfloat16", max_batch_tokens=portion, max_batch_seqs=1, max_model_len=tokens + 64,
                    paged_block_size=PAGE, num_blocks=(tokens + 64) // PAGE + 8, capture_sizes=[], ignore_eos=True)
    r = engine.runner
    rng = random.Random(5)
    prompt = [rng.randrange(vocab) for _ in range(tokens)]
    marks = []
    plain_attend = GQAAttention.attend

    def timed_attend(self, q, step, cache, out=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        res = plain_attend(self, q, step, cache, out)
        e1.record()
        marks.append((e0, e1))
        return res

    best = None
    for rep in range(2):                                    # the first run warms up
        r.open(("long", rep))
        marks.clear()
        GQAAttention.attend = timed_attend if rep == 1 else plain_attend
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for at in range(0, tokens, portion):
            n = min(portion, tokens - at)
            logits = r.step([StepEntry(("long", rep), prompt[at: at + n], [n - 1] if at + n == tokens else [])])
        engine.sampler.argmax_device(logits)
        e1.record()
        torch.cuda.synchronize()
        best = e0.elapsed_time(e1)
        r.close(("long", rep))
    GQAAttention.attend = plain_attend
    attn_ms = sum(a.elapsed_time(b) for a, b in marks)
    per_layer, _, _, q_dim = model_numbers(cfg, layers)
    flops = 2 * tokens * layers * per_layer + 2 * vocab * cfg["hidden_size"] + 2 * tokens * tokens * q_dim * layers
    del engine
    torch.cuda.empty_cache()
    return {"ms": round(best, 2), "tok_s": round(tokens / best * 1e3, 1), "attention_share": round(attn_ms / best, 4),
            "tflops": round(flops / (best * 1e-3) / 1e12, 1)}


def time_kernel(fn, repeats=20, flush=None):
    """Median device time of fn() in microseconds; `flush` (a large tensor) is rewritten between
    runs so that nothing of the last run stays in L2."""
    import torch
    for _ in range(3):
        fn()
    times = []
    for _ in range(repeats):
        if flush is not None:
            flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(times)


def kernel_ratios():
    """This engine's attention kernels against the reference's own (compiled unmodified, called
    through their C launchers with the cache laid out their way), and its tcgen05 GEMM against the
    library's, on the same data.  reference time / own time: above 1, this engine's kernel is the
    faster.  The reference's kernels are absent where baseline/_ref was never built: null then."""
    import math
    import torch
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_kernels as R
    from rustinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    out = {}
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)           # 256 MB: twice the L2
    have_ref = R.load() is not None
    g = torch.Generator(device="cuda").manual_seed(1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    for tag, (Hq, Hkv, hd) in {"1b": (32, 8, 64), "8b": (32, 8, 128)}.items():
        scale = 1 / math.sqrt(hd)
        # ---- decode: 8 requests at 4,096 keys
        B, ctx = 8, CONTEXT
        blocks = ctx // PAGE
        cache = torch.randn(B * blocks, 2, Hkv, PAGE, hd, generator=g, device=dev, dtype=torch.float32).bfloat16()
        table = torch.randperm(B * blocks, device=dev).to(torch.int32).view(B, blocks).contiguous()
        q = torch.randn(B, Hq * hd, generator=g, device=dev, dtype=torch.float32).bfloat16()
        o = torch.empty_like(q)
        kv_len, cu = i32([ctx] * B), i32(list(range(B + 1)))
        from rustinfer_b200.parts.base import MIXERS, BuildContext
        from rustinfer_b200.parts.spec import PartSpec
        part = MIXERS.build(PartSpec("gqa_attention", {"hidden_size": 64, "num_heads": Hq, "num_kv_heads": Hkv,
                                                       "head_dim": hd, "scale": scale, "window": None, "position": None}))
        part.prepare(BuildContext(dev, torch.bfloat16, ctx, PAGE, max_batch_seqs=64, num_sms=sms))
        splits = part._splits(B, ctx)
        no, nl = K.decode_scratch_floats(B, Hq, hd, splits)
        po, pl = torch.empty(no, device=dev), torch.empty(nl, device=dev)
        own = time_kernel(lambda: K.attention_decode_bf16(q, o, cache, table, cu, kv_len, None, B, Hq, Hkv, hd, scale,
                                                          None, splits, po, pl), flush=flush)
        out[f"attn_decode_{tag}_b8_us"] = round(own, 1)
        if have_ref:
            kp, vp = R.pools_from_pages(cache, PAGE)
            ws = R.decode_workspace(B, Hq, hd)
            o2 = torch.empty_like(q)
            ref = time_kernel(lambda: R.paged_decode(q, kp, vp, o2, table, kv_len, ws, Hq, Hkv, hd, scale, sms,
                                                     [ctx] * B), flush=flush)
            out[f"attn_decode_{tag}_b8_ref_us"] = round(ref, 1)
            out[f"attn_decode_{tag}_b8_vs_ref"] = round(ref / own, 2)
            del kp, vp
        # ---- prompt portion: one request of 2,048 tokens
        T = PREFILL_TOKENS
        qp = torch.randn(T, Hq * hd, generator=g, device=dev, dtype=torch.float32).bfloat16()
        op = torch.empty_like(qp)
        kvl, cup = i32([T]), i32([0, T])
        tbl = table[:1, : T // PAGE].contiguous()
        tc = K.tc_attention_supports(Hq, Hkv, hd, PAGE)
        tpt = K.tc_tokens_per_tile(Hq, Hkv) if tc else K.mma_tokens_per_tile(Hq, Hkv)
        te, tq = i32([0] * (T // tpt)), i32(list(range(0, T, tpt)))
        fn = K.attention_prefill_tc if tc else K.attention_prefill_bf16
        own = time_kernel(lambda: fn(qp, op, cache, tbl, cup, kvl, te, tq, Hq, Hkv, hd, scale, None), flush=flush)
        out[f"attn_prefill_{tag}_2048_us"] = round(own, 1)
        if have_ref:
            kp, vp = R.pools_from_pages(cache, PAGE)
            tiles = R.prefill_tiles([T])
            o2 = torch.empty_like(qp)
            ref = time_kernel(lambda: R.paged_prefill(qp, kp, vp, o2, tbl, kvl, cup, tiles, [T], [T], Hq, Hkv, hd, scale),
                              flush=flush)
            out[f"attn_prefill_{tag}_2048_ref_us"] = round(ref, 1)
            out[f"attn_prefill_{tag}_2048_vs_ref"] = round(ref / own, 2)
            del kp, vp
        del cache
    # ---- GEMM: the 2,048-token products of the 1B shape against the library's
    for name, (M, N, Kd) in {"qkv": (2048, 3072, 2048), "gate_up": (2048, 16384, 2048), "down": (2048, 2048, 8192),
                             "square8192": (8192, 8192, 8192)}.items():
        x = (torch.randn(M, Kd, generator=g, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, Kd, generator=g, device=dev) * 0.02).bfloat16()
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        own = time_kernel(lambda: K.gemm_tc(x, w, y, K.EPI_BF16, num_sms=sms), flush=flush)
        lib = time_kernel(lambda: torch.mm(x, w.t(), out=y), flush=flush)
        out[f"gemm_{name}_tflops"] = round(2 * M * N * Kd / own / 1e6, 1)
        out[f"gemm_{name}_vs_library"] = round(lib / own, 2)
        del x, w, y
    del flush
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------- the Dirurax family beside Llama at equal size
def _dirurax(width, layers, ff, vocab, gla, attn, delta, block):
    """`layers` layers, every fourth attention over blocks of `block` positions beside a delta rule,
    the others gated linear attention; a dense feed-forward in each."""
    gh, gd, gv = gla
    ah, akv, ad, av = attn
    dh, dd = delta
    out = []
    for i in range(layers):
        mlp = {"ff": ff, "kind": "dense"}
        if i % 4 == 3:
            out.append({"type": "parallel", "mlp": mlp, "mixer": {
                "left": {"heads": ah, "kv_heads": akv, "dim": ad, "vdim": av, "scale": ad ** -0.5, "mask": {"size": block}},
                "right": {"heads": dh, "dim": dd}, "left_scale": 0.5, "right_scale": 0.5}})
        else:
            out.append({"type": "gla", "mlp": mlp, "mixer": {"heads": gh, "dim": gd, "vdim": gv, "tau": 16.0}})
    return {"architecture": "Dirurax", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "layers": out}


def _llama_like(width, layers, ff, vocab, heads, kv_heads, head_dim):
    return dict(_llama(layers, width, heads, kv_heads, head_dim, ff, 32.0, True), vocab_size=vocab)


# width, layers, feed-forward width, vocabulary; Dirurax: gla (heads, key, value), attention (heads, kv heads,
# key, value), delta rule (heads, size), block of positions; Llama at the same width, layers, ff, vocabulary
FAMILY_SIZES = {
    "w1024": dict(width=1024, layers=8, ff=4096, vocab=32768, gla=(4, 128, 256), attn=(16, 4, 64, 64),
                  delta=(8, 128), block=512, llama=(16, 4, 64)),
    "w2048": dict(width=2048, layers=8, ff=8192, vocab=32768, gla=(8, 128, 256), attn=(32, 8, 64, 64),
                  delta=(16, 128), block=1024, llama=(32, 8, 64)),
}


def dirurax_kernels(hbm_gbs, size):
    """The new family's kernels alone at one size, 2,048 tokens of one request and 64 single tokens:
    microseconds, and what that is of the bytes they must move at the measured copy bandwidth (or, for
    the walks over tokens, of the fp32 multiply-adds at the CUDA cores' rate)."""
    import torch
    from rustinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    sz = FAMILY_SIZES[size]
    d = sz["width"]
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)
    out = {}
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    fma_per_s = sms * 128 * 1.9e9                            # fp32 multiply-adds a second on the CUDA cores
    for tag, T, entries in (("prefill2048", 2048, 1), ("decode64", 64, 64)):
        cu = i32([i * (T // entries) for i in range(entries + 1)])
        slots = i32(list(range(entries)))
        # gated linear attention
        H, dk, dv = sz["gla"]
        proj = bf(T, 2 * H * dk + 2 * H * dv)
        z = torch.randn(T, H * dk, device=dev)
        bias = bf(H * dk)
        o = torch.empty(T, H * dv, device=dev)
        state = torch.zeros(entries + 1, H, dv, K.recurrent_state_rows(dk), device=dev)
        us = time_kernel(lambda: K.gated_scan(proj[:, :H * dk], proj[:, H * dk:2 * H * dk], proj[:, 2 * H * dk:2 * H * dk + H * dv],
                                              z, bias, dk ** -0.5, 16.0, o, state, cu, slots, entries, H, dk, dv), flush=flush)
        moved = T * (2 * H * dk * 2 + H * dv * 2 + H * dk * 4 + H * dv * 4) + 2 * entries * H * dk * dv * 4
        out[f"gated_scan_{tag}"] = {"us": round(us, 1), "hbm_frac": round(moved / (us * 1e-6) / 1e9 / hbm_gbs, 4),
                                    "fma_frac": round(2 * T * H * dk * dv / (us * 1e-6) / fma_per_s, 4)}
        y = torch.empty(T, H * dv, device=dev, dtype=torch.bfloat16)
        w = bf(dv)
        us = time_kernel(lambda: K.gated_head_norm(o, proj[:, 2 * H * dk + H * dv:], w, False, K.GATE_SILU, 1e-6, y, H, dv), flush=flush)
        out[f"gated_head_norm_{tag}"] = {"us": round(us, 1), "hbm_frac": round(T * H * dv * 8 / (us * 1e-6) / 1e9 / hbm_gbs, 4)}
        # delta rule
        H, dk = sz["delta"]
        proj = bf(T, 5 * H * dk)
        zw = torch.randn(T, H * dk, device=dev)
        b1, b2 = bf(H * dk), bf(H * dk)
        o = torch.empty(T, H * dk, device=dev)
        state = torch.zeros(entries + 1, H, dk, K.recurrent_state_rows(dk), device=dev)
        us = time_kernel(lambda: K.delta_scan(proj[:, :H * dk], proj[:, H * dk:2 * H * dk], proj[:, 2 * H * dk:3 * H * dk],
                                              proj[:, 4 * H * dk:], b1, zw, b2, 0.6065306597, 1e-6, o, state, cu, slots,
                                              entries, H, dk, dk), flush=flush)
        moved = T * (4 * H * dk * 2 + 2 * H * dk * 4) + 2 * entries * H * dk * dk * 4
        out[f"delta_scan_{tag}"] = {"us": round(us, 1), "hbm_frac": round(moved / (us * 1e-6) / 1e9 / hbm_gbs, 4),
                                    "fma_frac": round(3 * T * H * dk * dk / (us * 1e-6) / fma_per_s, 4)}
        # layer norm around a sublayer beside the fused add + RMSNorm of the Llama blocks
        h = torch.randn(T, d, device=dev)
        delta = bf(T, d)
        ws = [bf(d) for _ in range(4)]
        xo = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.sandwich_norm(h, delta, ws[0], ws[1], ws[2], ws[3], xo, 1e-6), flush=flush)
        us_rms = time_kernel(lambda: K.add_rmsnorm(h, delta, ws[0], 1e-6, xo), flush=flush)
        moved = T * d * (4 + 4 + 2 + 2)
        out[f"sandwich_norm_{tag}"] = {"us": round(us, 1), "hbm_frac": round(moved / (us * 1e-6) / 1e9 / hbm_gbs, 4),
                                       "add_rmsnorm_us": round(us_rms, 1),
                                       "add_rmsnorm_hbm_frac": round(moved / (us_rms * 1e-6) / 1e9 / hbm_gbs, 4)}
    # attention over the current block of positions (fp32 arithmetic) beside the tcgen05 causal attention
    # of the Llama blocks on the same heads, 2,048 tokens of one request
    Hq, Hkv, hd, vd = sz["attn"]
    T, page, block = 2048, PAGE, sz["block"]
    pages = T // page
    cache = bf(pages, 2, Hkv, page, hd)
    table = i32([list(range(pages))])
    q = bf(T, Hq * hd)
    ao = torch.empty(T, Hq * vd, device=dev, dtype=torch.bfloat16)
    tiles = list(range(0, T, 16))
    te, t0 = i32([0] * len(tiles)), i32(tiles)
    cu, kv = i32([0, T]), i32([T])
    us = time_kernel(lambda: K.attention_plain(q, ao, cache, table, cu, kv, te, t0, Hq, Hkv, hd, hd ** -0.5, None, block, vd),
                     repeats=5, flush=flush)
    pairs = sum(min(p % block, p) + 1 for p in range(T))     # (query, key) pairs inside the blocks
    out["block_attention_prefill2048"] = {"us": round(us, 1), "tflops": round(2 * pairs * Hq * (hd + vd) / (us * 1e-6) / 1e12, 2)}
    if hd == vd and hd % 16 == 0:
        rows = K.mma_tokens_per_tile(Hq, Hkv)
        tl = list(range(0, T, rows))
        te1, t01 = i32([0] * len(tl)), i32(tl)
        us1 = time_kernel(lambda: K.attention_prefill_bf16(q, ao, cache, table, cu, kv, te1, t01, Hq, Hkv, hd, hd ** -0.5,
                                                           None, block, precise=True), flush=flush)
        out["block_attention_prefill2048"].update(
            fp32_arithmetic_us=out["block_attention_prefill2048"]["us"], us=round(us1, 1),
            tflops=round(2 * pairs * Hq * (hd + 3 * vd) / (us1 * 1e-6) / 1e12, 2))
    if K.tc_attention_supports(Hq, Hkv, hd, page):
        rows = K.tc_tokens_per_tile(Hq, Hkv)
        tl = list(range(0, T, rows))
        te2, t02 = i32([0] * len(tl)), i32(tl)
        us2 = time_kernel(lambda: K.attention_prefill_tc(q, ao, cache, table, cu, kv, te2, t02, Hq, Hkv, hd, hd ** -0.5, None),
                          flush=flush)
        out["block_attention_prefill2048"].update(
            causal_tc_us=round(us2, 1), causal_tc_tflops=round(2 * (T * (T + 1) // 2) * Hq * 2 * hd / (us2 * 1e-6) / 1e12, 2))
    return out


def _pikalix(width, layers, ff, vocab, attn, window, rot, experts, top, expert_ff, shared_ff, groups, streams):
    """`layers` layers of attention with a sliding window; every odd layer reads the keys and values of the layer
    before it; feed-forwards alternate between a dense one and routed experts."""
    h, kv, dim, vdim = attn
    out = []
    for i in range(layers):
        mixer = {"heads": h, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "mask": {"size": window},
                 "rot": {"dims": rot, "base": 500000.0}}
        if i % 2 == 1:
            mixer["kv_from"] = i - 1
        mlp = {"kind": "dense", "ff": ff} if i % 2 == 0 else {
            "kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff},
            "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}}
        out.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Pikalix", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "streams": streams, "layers": out}


# Pikalix at the same widths: a token's feed-forward work equals the dense one's (top x expert_ff + shared_ff = ff)
PIKALIX_SIZES = {
    "w1024": dict(width=1024, layers=8, ff=4096, vocab=32768, attn=(16, 4, 64, 64), window=1024, rot=32, experts=32, top=4,
                  expert_ff=768, shared_ff=1024, groups=(8, 4), streams=2, llama=(16, 4, 64)),
    "w2048": dict(width=2048, layers=8, ff=8192, vocab=32768, attn=(32, 8, 64, 64), window=1024, rot=32, experts=32, top=4,
                  expert_ff=1536, shared_ff=2048, groups=(8, 4), streams=2, llama=(32, 8, 64)),
}


def pikalix_kernels(hbm_gbs, bf16_tflops, size):
    """The Pikalix kernels alone at one size, each beside the like kernel of the Llama path on the same shapes:
    microseconds, and what that is of the bytes they must move at the measured copy bandwidth (or of the
    measured library GEMM rate for the experts' products over a prompt)."""
    import torch
    from rustinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    sz = PIKALIX_SIZES[size]
    d, S = sz["width"], sz["streams"]
    Hq, Hkv, hd, vd = sz["attn"]
    E, top, fe = sz["experts"], sz["top"], sz["expert_ff"]
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)
    frac = lambda moved, us: round(moved / (us * 1e-6) / 1e9 / hbm_gbs, 4)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    out = {}
    for tag, T in (("prefill2048", 2048), ("decode64", 64)):
        # the streams' update + weighted sum + norm beside the add + RMSNorm of one stream
        X = torch.randn(S, T, d, device=dev)
        y = torch.randn(T, d, device=dev)
        mix, wr, rd = torch.randn(S, S, device=dev), torch.randn(S, device=dev), torch.randn(S, device=dev)
        w = bf(d)
        xo = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.hyper_collect(X, False, y, mix, wr, rd, w, 1e-6, xo), flush=flush)
        h, delta = torch.randn(T, d, device=dev), bf(T, d)
        us_rms = time_kernel(lambda: K.add_rmsnorm(h, delta, w, 1e-6, xo), flush=flush)
        out[f"stream_norm_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * d * (8 * S + 4 + 2), us),
                                     "add_rmsnorm_us": round(us_rms, 1), "add_rmsnorm_hbm_frac": frac(T * d * (4 + 4 + 2 + 2), us_rms)}
        # q, k, v from the projection to the attention and the cache beside the rotary + cache-write kernel
        cols = (Hq + Hkv) * hd + Hkv * vd
        pages = T // PAGE + 1
        cache = bf(pages, 2, Hkv, PAGE, hd)
        qkv32, bias = torch.randn(T, cols, device=dev), torch.randn(cols, device=dev)
        qw, kw = bf(Hq * hd), bf(Hkv * hd)
        pos, slots = i32(list(range(T))), i32(list(range(T)))
        cos, sin = torch.randn(T, sz["rot"] // 2, device=dev), torch.randn(T, sz["rot"] // 2, device=dev)
        q_out = torch.empty(T, Hq * hd, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.qkv_prepare(qkv32, bias, qw, kw, 2, 1e-6, pos, cos, sin, sz["rot"], True, slots, cache, q_out,
                                               Hq, Hkv, hd, vd, True), flush=flush)
        qkv16 = bf(T, cols)
        cos2, sin2 = torch.randn(T, hd // 2, device=dev), torch.randn(T, hd // 2, device=dev)
        us_rope = time_kernel(lambda: K.rope_scatter(qkv16, pos, cos2, sin2, slots, cache, Hq, Hkv, hd, hd), flush=flush)
        out[f"qkv_prepare_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * cols * (4 + 2), us),
                                     "rope_scatter_us": round(us_rope, 1), "rope_scatter_hbm_frac": frac(T * cols * (2 + 2), us_rope)}
        # the experts: choice and sort, the two products, the weighted sum
        N = T * top
        xr, rw, corr = bf(T, d), torch.randn(E, d, device=dev) * 0.02, torch.randn(E, device=dev) * 0.1
        ids = torch.empty(T, top, dtype=torch.int32, device=dev)
        wts = torch.empty(T, top, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        offsets, order, place = (torch.empty(n, dtype=torch.int32, device=dev) for n in (E + 1, N, N))

        def choose():
            counts.zero_()
            K.moe_route(None, corr, top, sz["groups"][0], sz["groups"][1], False, ids, wts, counts, x=xr, router=rw)
            K.moe_sort(ids, counts, offsets, order, place)
        us = time_kernel(choose, flush=flush)
        out[f"experts_choice_{tag}"] = {"us": round(us, 1), "launches": 2}
        x = bf(T, d)
        gate_up, down = bf(E, 2 * fe, d) * 0.02, bf(E, d, fe) * 0.02
        mid = torch.empty(N, fe, device=dev, dtype=torch.bfloat16)
        Y = torch.empty(N, d, device=dev)
        used = int((offsets[1:] > offsets[:-1]).sum())
        us1 = time_kernel(lambda: K.moe_product(x, gate_up, mid, offsets, order, top, gated=True), flush=flush)
        us2 = time_kernel(lambda: K.moe_product(mid, down, Y, offsets, None, top, gated=False), flush=flush)
        mma_us = us1 + us2
        tensor_memory = N >= 24 * E                      # what the experts part does from that many rows on
        if tensor_memory:
            xs = torch.empty(N, d, device=dev, dtype=torch.bfloat16)
            us0 = time_kernel(lambda: K.moe_gather(x, order, top, xs), flush=flush)
            us1 = time_kernel(lambda: K.gemm_tc_grouped(xs, gate_up, mid, offsets, K.EPI_SILU), flush=flush) + us0
            us2 = time_kernel(lambda: K.gemm_tc_grouped(mid, down, Y, offsets, K.EPI_F32), flush=flush)
        flops = 2 * N * d * fe * 3
        moved = used * 3 * fe * d * 2 + N * (d * 2 + fe * 4 + d * 4)
        # the like work of the Llama path: one dense product pair over the same rows (N rows, the tcgen05 GEMM)
        xd, wd1, wd2 = bf(N, d), bf(2 * fe, d) * 0.02, bf(d, fe) * 0.02
        m2, y2 = torch.empty(N, fe, device=dev, dtype=torch.bfloat16), torch.empty(N, d, device=dev)
        usd = time_kernel(lambda: (K.gemm_tc(xd, wd1, m2, K.EPI_SILU, num_sms=sms), K.gemm_tc(m2, wd2, y2, K.EPI_F32, num_sms=sms)),
                          flush=flush)
        out[f"experts_products_{tag}"] = {"us": round(us1 + us2, 1), "gate_up_us": round(us1, 1), "down_us": round(us2, 1),
                                          "tflops": round(flops / ((us1 + us2) * 1e-6) / 1e12, 1),
                                          "gemm_frac": round(flops / ((us1 + us2) * 1e-6) / 1e12 / bf16_tflops, 4),
                                          "hbm_frac": frac(moved, us1 + us2), "experts_used": used,
                                          "kernel": "tcgen05 (gather + two grouped products)" if tensor_memory else "mma.sync",
                                          "mma_sync_us": round(mma_us, 1),
                                          "dense_pair_same_rows_us": round(usd, 1),
                                          "dense_pair_tflops": round(flops / (usd * 1e-6) / 1e12, 1)}
        shared = torch.randn(T, d, device=dev)
        o = torch.empty(T, d, device=dev)
        us = time_kernel(lambda: K.moe_combine(Y, place, wts, shared, o, counts), flush=flush)
        out[f"experts_sum_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * d * (4 * top + 4 + 4), us)}
    # attention: 64 single tokens at 4,096 keys of which the window keeps 1,024, beside the split-KV kernel with the same window
    B, ctx, win = 64, 4096, sz["window"]
    blocks = ctx // PAGE
    cache = bf(B * blocks, 2, Hkv, PAGE, hd)
    table = torch.randperm(B * blocks, device=dev).to(torch.int32).view(B, blocks).contiguous()
    q, ao = bf(B, Hq * hd), torch.empty(B, Hq * vd, device=dev, dtype=torch.bfloat16)
    kv_len, cu, ent = i32([ctx] * B), i32(list(range(B + 1))), i32(list(range(B)))
    from rustinfer_b200.parts.base import MIXERS, BuildContext
    from rustinfer_b200.parts.spec import PartSpec
    own = MIXERS.build(PartSpec("gqa_attention", {"hidden_size": 64, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd,
                                                  "value_dim": vd, "scale": hd ** -0.5, "window": win, "position": None,
                                                  "sink": True}))
    own.prepare(BuildContext(dev, torch.bfloat16, ctx, PAGE, max_batch_seqs=64, num_sms=sms))
    ranges = own._single_splits(B, ctx)
    us = time_kernel(lambda: K.attention_single(q, ao, cache, table, cu, kv_len, ent, Hq, Hkv, hd, hd ** -0.5, win, None, vd,
                                                sink=True, splits=ranges, part=own.single_part), flush=flush)
    moved = B * Hkv * win * (hd + vd) * 2
    part = MIXERS.build(PartSpec("gqa_attention", {"hidden_size": 64, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd,
                                                   "scale": hd ** -0.5, "window": win, "position": None}))
    part.prepare(BuildContext(dev, torch.bfloat16, ctx, PAGE, max_batch_seqs=64, num_sms=sms))
    splits = part._splits(B, ctx)
    no, nl = K.decode_scratch_floats(B, Hq, hd, splits)
    po, pl = torch.empty(no, device=dev), torch.empty(nl, device=dev)
    us_d = time_kernel(lambda: K.attention_decode_bf16(q, ao, cache, table, cu, kv_len, None, B, Hq, Hkv, hd, hd ** -0.5, win,
                                                       splits, po, pl), flush=flush)
    out["window_attention_decode64"] = {"us": round(us, 1), "ranges": ranges, "hbm_frac": frac(moved, us), "split_kv_us": round(us_d, 1),
                                        "split_kv_hbm_frac": frac(moved, us_d)}
    # a prompt of 2,048 tokens: fp32 softmax weights with the sink beside the tcgen05 kernel with the same window
    T = 2048
    tbl = table[:1, : T // PAGE].contiguous()
    qp, op = bf(T, Hq * hd), torch.empty(T, Hq * vd, device=dev, dtype=torch.bfloat16)
    cup, kvl = i32([0, T]), i32([T])
    pairs = sum(min(p + 1, win) for p in range(T))
    rows = K.mma_tokens_per_tile(Hq, Hkv)
    tl = list(range(0, T, rows))
    te, t0 = i32([0] * len(tl)), i32(tl)
    us = time_kernel(lambda: K.attention_prefill_bf16(qp, op, cache, tbl, cup, kvl, te, t0, Hq, Hkv, hd, hd ** -0.5, win, None,
                                                      precise=True, sink=True), flush=flush)
    res = {"us": round(us, 1), "tflops": round(2 * pairs * Hq * (hd + 3 * vd) / (us * 1e-6) / 1e12, 2),
           "useful_tflops": round(2 * pairs * Hq * (hd + vd) / (us * 1e-6) / 1e12, 2)}
    if K.tc_attention_supports(Hq, Hkv, hd, PAGE):
        rows = K.tc_tokens_per_tile(Hq, Hkv)
        tl = list(range(0, T, rows))
        te2, t02 = i32([0] * len(tl)), i32(tl)
        us2 = time_kernel(lambda: K.attention_prefill_tc(qp, op, cache, tbl, cup, kvl, te2, t02, Hq, Hkv, hd, hd ** -0.5, win),
                          flush=flush)
        res.update(window_tc_us=round(us2, 1), window_tc_tflops=round(2 * pairs * Hq * 2 * hd / (us2 * 1e-6) / 1e12, 2))
    out["window_attention_prefill2048"] = res
    return out


def _sotazen(width, layers, ff, vocab, lightning, latent, attn, window, rot):
    """`layers` layers in the order lightning, lightning, latent attention, differential attention (norms after the
    sums), a dense feed-forward with the square of relu in each."""
    lh, ld, lv = lightning
    th, td, tr, tv, rank = latent
    ah, akv, ad, av = attn
    out = []
    for i in range(layers):
        mlp = {"ff": ff, "kind": "dense"}
        if i % 4 == 3:
            mixer = {"heads": ah, "kv_heads": akv, "dim": ad, "vdim": av, "scale": ad ** -0.5, "diff": 0.8, "softcap": 50.0,
                     "mask": {"size": window}, "rot": {"dims": rot, "base": 500000.0}}
            out.append({"type": "attention", "mixer": mixer, "mlp": mlp})
        elif i % 4 == 2:
            mixer = {"heads": th, "dim": td, "rot_dim": tr, "vdim": tv, "kv_rank": rank, "scale": (td + tr) ** -0.5,
                     "rot": {"dims": tr, "base": 10000.0}}
            out.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
        else:
            decay = [1.0 - 2.0 ** (-5.0 - 3.0 * h / max(lh - 1, 1)) for h in range(lh)]
            out.append({"type": "lightning", "mixer": {"heads": lh, "dim": ld, "vdim": lv, "decay": decay}, "mlp": mlp})
    return {"architecture": "Sotazen", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "postln_alpha": 2.0, "layers": out}


# Sotazen at the same widths: lightning (heads, key, value), latent attention (heads, plain, rotated, value, rank),
# differential attention (heads, kv heads, key of one map, value), its window and rotated channels
SOTAZEN_SIZES = {
    "w1024": dict(width=1024, layers=8, ff=4096, vocab=32768, lightning=(8, 128, 128), latent=(16, 64, 32, 64, 128),
                  attn=(8, 2, 64, 128), window=1024, rot=32, llama=(16, 4, 64)),
    "w2048": dict(width=2048, layers=8, ff=8192, vocab=32768, lightning=(16, 128, 128), latent=(32, 64, 32, 64, 256),
                  attn=(16, 4, 64, 128), window=1024, rot=32, llama=(32, 8, 64)),
}


def sotazen_kernels(hbm_gbs, bf16_tflops, size):
    """The Sotazen kernels alone at one size, each beside the like kernel of the nearest existing family on the same
    shapes (the gated recurrence and head norm of Dirurax, the window attention with a sink and the q/k/v preparation
    of Pikalix, the add + RMSNorm and rotary kernels of the Llama path): microseconds, and what that is of the bytes
    they must move at the measured copy bandwidth."""
    import torch
    from rustinfer_b200.ops import kernels as K
    from rustinfer_b200.parts.attention_variants import PlainAttend
    from rustinfer_b200.parts.base import BuildContext
    dev = torch.device("cuda:0")
    sz = SOTAZEN_SIZES[size]
    d = sz["width"]
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)
    f32 = lambda *s: torch.randn(*s, device=dev)
    frac = lambda moved, us: round(moved / (us * 1e-6) / 1e9 / hbm_gbs, 4)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    fma_per_s = sms * 128 * 1.9e9
    out = {}
    ah, akv, ad, av = sz["attn"]
    th, td, tr, tv, rank = sz["latent"]
    kd = rank + tr
    for tag, T, entries in (("prefill2048", 2048, 1), ("decode64", 64, 64)):
        cu = i32([i * (T // entries) for i in range(entries + 1)])
        slots = i32(list(range(entries)))
        # the norm after the sum beside the add + RMSNorm before a sublayer
        h, delta, w = f32(T, d), f32(T, d), bf(d)
        xo = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.scale_add_norm(h, delta, None, 2.0, w, 1e-6, xo), flush=flush)
        d16 = bf(T, d)
        us_rms = time_kernel(lambda: K.add_rmsnorm(h, d16, w, 1e-6, xo), flush=flush)
        out[f"scale_add_norm_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * d * (4 + 4 + 4 + 2), us),
                                        "add_rmsnorm_us": round(us_rms, 1), "add_rmsnorm_hbm_frac": frac(T * d * (4 + 4 + 2 + 2), us_rms)}
        # lightning: the walk with fixed decays beside the gated walk on the same sizes, the row norm beside the head norm
        H, dk, dv = sz["lightning"]
        p32 = f32(T, 2 * H * dk + 2 * H * dv)
        decay = torch.full((H * dk,), 0.97, device=dev)
        o = torch.empty(T, H * dv, device=dev)
        state = torch.zeros(entries + 1, H, dv, K.recurrent_state_rows(dk), device=dev)
        us = time_kernel(lambda: K.decay_scan(p32[:, :H * dk], p32[:, H * dk:2 * H * dk], p32[:, 2 * H * dk:2 * H * dk + H * dv],
                                              decay, 1.0, o, state, cu, slots, entries, H, dk, dv), flush=flush)
        moved = T * (2 * H * dk * 4 + H * dv * 4 + H * dv * 4) + 2 * entries * H * dk * dv * 4
        p16, z = bf(T, 2 * H * dk + 2 * H * dv), f32(T, H * dk)
        zb = bf(H * dk)
        us_g = time_kernel(lambda: K.gated_scan(p16[:, :H * dk], p16[:, H * dk:2 * H * dk], p16[:, 2 * H * dk:2 * H * dk + H * dv],
                                                z, zb, 1.0, 16.0, o, state, cu, slots, entries, H, dk, dv), flush=flush)
        moved_g = T * (2 * H * dk * 2 + H * dv * 2 + H * dk * 4 + H * dv * 4) + 2 * entries * H * dk * dv * 4
        out[f"decay_scan_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(moved, us),
                                    "fma_frac": round(2 * T * H * dk * dv / (us * 1e-6) / fma_per_s, 4),
                                    "gated_scan_us": round(us_g, 1), "gated_scan_hbm_frac": frac(moved_g, us_g)}
        y = torch.empty(T, H * dv, device=dev, dtype=torch.bfloat16)
        wn = bf(H * dv)
        us = time_kernel(lambda: K.row_norm_gate(o, p32[:, 2 * H * dk + H * dv:], wn, 1e-6, y), flush=flush)
        whd = bf(dv)
        us_h = time_kernel(lambda: K.gated_head_norm(o, p16[:, 2 * H * dk + H * dv:], whd, False, K.GATE_SILU, 1e-6, y, H, dv), flush=flush)
        out[f"row_norm_gate_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * H * dv * (4 + 4 + 2), us),
                                       "gated_head_norm_us": round(us_h, 1), "gated_head_norm_hbm_frac": frac(T * H * dv * (4 + 2 + 2), us_h)}
        # differential attention: q, k, v from the projection (two maps), the maps' difference with its norm and gate
        cols = (ah + akv) * 2 * ad + akv * av
        pages = T // PAGE + 1
        cache = bf(pages, PAGE * (akv * 2 * ad + akv * av))
        qkv32, bias = f32(T, cols), f32(cols)
        qw, kw = bf(ad), bf(ad)
        pos, slot_t = i32(list(range(T))), i32(list(range(T)))
        cos, sin = f32(T, sz["rot"] // 2), f32(T, sz["rot"] // 2)
        q_out = torch.empty(T, ah * 2 * ad, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.qkv_prepare(qkv32, bias, qw, kw, 1, 1e-6, pos, cos, sin, sz["rot"], True, slot_t, cache, q_out,
                                               2 * ah, 2 * akv, ad, av, True, value_heads=akv), flush=flush)
        lh, lkv, lhd = sz["llama"]
        lcols = (lh + 2 * lkv) * lhd
        qkv16 = bf(T, lcols)
        lcache = bf(pages, 2, lkv, PAGE, lhd)
        cos2, sin2 = f32(T, lhd // 2), f32(T, lhd // 2)
        us_rope = time_kernel(lambda: K.rope_scatter(qkv16, pos, cos2, sin2, slot_t, lcache, lh, lkv, lhd, lhd), flush=flush)
        out[f"qkv_prepare_two_maps_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * cols * (4 + 2), us),
                                              "rope_scatter_us": round(us_rope, 1), "rope_scatter_hbm_frac": frac(T * lcols * (2 + 2), us_rope)}
        maps, gate = f32(T, ah * 2 * av), f32(T, ah * av)
        yd = torch.empty(T, ah * av, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.diff_combine(maps, 0.7, 0.2, 1e-6, gate, yd, ah, av), flush=flush)
        o2, g16, w2 = f32(T, ah * av), bf(T, ah * av), bf(av)
        us_h = time_kernel(lambda: K.gated_head_norm(o2, g16, w2, False, K.GATE_SILU, 1e-6, yd, ah, av), flush=flush)
        out[f"diff_combine_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * ah * av * (8 + 4 + 2), us),
                                      "gated_head_norm_us": round(us_h, 1), "gated_head_norm_hbm_frac": frac(T * ah * av * (4 + 2 + 2), us_h)}
        # latent attention: queries and the cached row from the projection
        pcols = th * (td + tr) + kd
        proj, cw = f32(T, pcols), bf(rank)
        lat_cache = bf(pages, PAGE * kd)
        cos3, sin3 = f32(T, tr // 2), f32(T, tr // 2)
        q_plain = torch.empty(T, th * td, device=dev, dtype=torch.bfloat16)
        q_full = torch.empty(T, th * kd, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.latent_prepare(proj, cw, 1e-6, pos, cos3, sin3, slot_t, lat_cache, q_plain, q_full, th, td, tr, rank),
                         flush=flush)
        out[f"latent_prepare_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * (pcols * 4 + (th * (td + tr) + kd) * 2), us),
                                        "rope_scatter_us": round(us_rope, 1), "rope_scatter_hbm_frac": frac(T * lcols * (2 + 2), us_rope)}
    # attention of 64 single tokens at 4,096 keys: two maps under the window, rows of the latent cache, and Pikalix's
    # window attention with a sink on the Llama heads
    B, ctx, win = 64, 4096, sz["window"]
    blocks = ctx // PAGE
    bctx = BuildContext(dev, torch.bfloat16, ctx, PAGE, max_batch_seqs=B, num_sms=sms)
    kv_len, cu, ent = i32([ctx] * B), i32(list(range(B + 1))), i32(list(range(B)))
    table = torch.randperm(B * blocks, device=dev).to(torch.int32).view(B, blocks).contiguous()
    lh, lkv, lhd = sz["llama"]

    def single(Hq, Hkv, hd, vd, maps, vik, window, softcap, sink_values):
        att = PlainAttend(bctx, Hq, Hkv, hd, vd, maps=maps, value_in_key=vik, window=window)
        per = Hkv * maps * hd + (0 if vik else Hkv * vd)
        cache = bf(B * blocks, PAGE * per)
        q = bf(B, Hq * hd)
        o = torch.empty(B, Hq * vd, device=dev, dtype=torch.float32 if maps > 1 else torch.bfloat16)
        span = min(ctx, window) if window else ctx
        if att.fast_single:
            ranges, kernel = att._splits(B, ctx), "one CTA a key head"
            us = time_kernel(lambda: K.attention_single(q, o, cache, table, cu, kv_len, ent, Hq, Hkv, hd, hd ** -0.5, window, None, vd,
                                                        sink=sink_values is not None, splits=ranges, part=att.part, softcap=softcap,
                                                        sink_values=sink_values, maps=maps, value_in_key=vik), flush=flush)
        elif att.rows_single:
            ranges, kernel = att._rows_splits(B, ctx), "tensor cores, 64 (token, head) rows a CTA"
            us = time_kernel(lambda: K.attention_rows(q, o, cache, table, cu, kv_len, ent, att.zero_tok0[:B], Hq, Hkv, hd, hd ** -0.5,
                                                      window, vd, sink=sink_values is not None, softcap=softcap,
                                                      sink_values=sink_values, maps=maps, value_in_key=vik, splits=ranges,
                                                      part=att.part), flush=flush)
        else:
            ranges, t0 = 0, i32([0] * B)
            fn, kernel = ((K.attention_rows, "tensor cores, 64 (token, head) rows a CTA") if att.rows else
                          (lambda *a, **k: K.attention_plain(*a[:13], None, *a[13:], **k), "fp32 arithmetic, 16 rows a head"))
            us = time_kernel(lambda: fn(q, o, cache, table, cu, kv_len, ent, t0, Hq, Hkv, hd, hd ** -0.5, window, vd,
                                        sink=sink_values is not None, softcap=softcap, sink_values=sink_values,
                                        maps=maps, value_in_key=vik), repeats=5, flush=flush)
        return {"us": round(us, 1), "ranges": ranges, "hbm_frac": frac(B * span * per * 2, us), "kernel": kernel,
                "useful_tflops": round(2 * B * span * Hq * (hd + vd) / (us * 1e-6) / 1e12, 2)}
    res = single(2 * ah, akv, ad, av, 2, False, win, 50.0, None)
    like = single(lh, lkv, lhd, lhd, 1, False, win, None, torch.zeros(lh, device=dev))
    res.update(window_sink_us=like["us"], window_sink_hbm_frac=like["hbm_frac"])
    out["two_map_attention_decode64"] = res
    res = single(th, 1, kd, rank, 1, True, None, None, torch.zeros(th, device=dev))
    like = single(lh, lkv, lhd, lhd, 1, False, None, None, torch.zeros(lh, device=dev))
    res.update(causal_sink_us=like["us"], causal_sink_hbm_frac=like["hbm_frac"], causal_sink_useful_tflops=like["useful_tflops"])
    out["latent_attention_decode64"] = res
    # a prompt of 2,048 tokens: the fp32-arithmetic tiles beside Pikalix's tensor-core kernel with fp32 weights
    T = 2048
    tbl = i32([list(range(T // PAGE))])
    cup, kvl = i32([0, T]), i32([T])
    tiles = list(range(0, T, 16))
    te, t0 = i32([0] * len(tiles)), i32(tiles)

    def prompt(Hq, Hkv, hd, vd, maps, vik, window, softcap, sink_values):
        per = Hkv * maps * hd + (0 if vik else Hkv * vd)
        cache = bf(T // PAGE, PAGE * per)
        q = bf(T, Hq * hd)
        o = torch.empty(T, Hq * vd, device=dev, dtype=torch.float32 if maps > 1 else torch.bfloat16)
        opts = dict(sink=sink_values is not None, softcap=softcap, sink_values=sink_values, maps=maps, value_in_key=vik)
        us32 = time_kernel(lambda: K.attention_plain(q, o, cache, tbl, cup, kvl, te, t0, Hq, Hkv, hd, hd ** -0.5, window, None, vd, **opts),
                           repeats=5, flush=flush)
        pairs = sum(min(p + 1, window) if window else p + 1 for p in range(T))
        res = {"fp32_arithmetic_us": round(us32, 1), "fp32_arithmetic_fma_frac": round(pairs * Hq * (hd + vd) / (us32 * 1e-6) / fma_per_s, 4)}
        if K.attention_rows_supports(hd, vd, vik):
            tpt = K.attention_rows_tokens_per_tile(Hq, Hkv, hd, vd, maps)
            tl = list(range(0, T, tpt))
            ter, t0r = i32([0] * len(tl)), i32(tl)
            us = time_kernel(lambda: K.attention_rows(q, o, cache, tbl, cup, kvl, ter, t0r, Hq, Hkv, hd, hd ** -0.5, window, vd, **opts),
                             flush=flush)
            res.update(us=round(us, 1), useful_tflops=round(2 * pairs * Hq * (hd + vd) / (us * 1e-6) / 1e12, 2),
                       tflops=round(2 * pairs * Hq * (hd + 3 * vd) / (us * 1e-6) / 1e12, 2))
        return res
    res = prompt(2 * ah, akv, ad, av, 2, False, win, 50.0, None)
    pcache = bf(T // PAGE, 2, lkv, PAGE, lhd)
    qp, op = bf(T, lh * lhd), torch.empty(T, lh * lhd, device=dev, dtype=torch.bfloat16)
    rows = K.mma_tokens_per_tile(lh, lkv)
    tl = list(range(0, T, rows))
    te1, t01 = i32([0] * len(tl)), i32(tl)
    for name, w_ in (("window", win), ("causal", None)):
        pairs = sum(min(p + 1, w_) if w_ else p + 1 for p in range(T))
        us1 = time_kernel(lambda: K.attention_prefill_bf16(qp, op, pcache, tbl, cup, kvl, te1, t01, lh, lkv, lhd, lhd ** -0.5, w_, None,
                                                           precise=True, sink=True), flush=flush)
        like = {f"{name}_sink_mma_us": round(us1, 1), f"{name}_sink_mma_useful_tflops": round(2 * pairs * lh * 2 * lhd / (us1 * 1e-6) / 1e12, 2)}
        if name == "window":
            res.update(like)
            out["two_map_attention_prefill2048"] = res
            res = prompt(th, 1, kd, rank, 1, True, None, None, torch.zeros(th, device=dev))
        else:
            res.update(like)
            out["latent_attention_prefill2048"] = res
    return out


def _linedra(width, layers, ff, vocab, attn, window, recurrent, latent, experts, top, expert_ff, taps):
    """`layers` layers in the order parallel, parallel, parallel, latent attention (norms around the sublayers, the
    input convolution, the depth average), routed experts with clamped pairs in each."""
    h, kv, dim, vdim = attn
    rw, blocks, conv = recurrent
    th, td, tr, tv, rank, q_rank = latent
    out = []
    for i in range(layers):
        mlp = {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0}, "router": {"experts": experts, "top": top}}
        if i % 4 == 3:
            mixer = {"heads": th, "dim": td, "rot_dim": tr, "vdim": tv, "kv_rank": rank, "q_rank": q_rank,
                     "scale": (td + tr) ** -0.5, "rot": {"dims": tr, "base": 10000.0}}
            out.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
        else:
            mixer = {"left": {"heads": h, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "mask": {"size": window}},
                     "right": {"width": rw, "blocks": blocks, "conv": conv}, "left_scale": 0.6, "right_scale": 0.5}
            out.append({"type": "parallel", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Linedra", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "canon": {"taps": taps},
            "embedding": {"scale": 1.0}, "residual_mult": 0.5, "logit_softcap": 30.0, "layers": out}


# Linedra at the same widths: attention (heads, kv heads, key, value), the recurrent unit (width, blocks, taps), latent
# attention (heads, plain, rotated, value, rank, query rank); a token's feed-forward work equals the dense one's
# (top x expert_ff = ff).  `pikalix`: the Pikalix model of the same width, depth and vocabulary (attention with a sink
# and a window, routed experts), the nearest of the families the engine had
LINEDRA_SIZES = {
    "w1024": dict(width=1024, layers=8, ff=4096, vocab=32768, attn=(16, 4, 64, 64), window=1024, recurrent=(1024, 8, 4),
                  latent=(16, 64, 32, 64, 128, 384), experts=32, top=4, expert_ff=1024, taps=4, llama=(16, 4, 64)),
    "w2048": dict(width=2048, layers=8, ff=8192, vocab=32768, attn=(32, 8, 64, 64), window=1024, recurrent=(2048, 16, 4),
                  latent=(32, 64, 32, 64, 256, 768), experts=32, top=4, expert_ff=2048, taps=4, llama=(32, 8, 64)),
}


def linedra_kernels(hbm_gbs, bf16_tflops, size):
    """The Linedra kernels alone at one size, each beside the like kernel of the nearest existing family on the same
    shapes (the add + RMSNorm of the Llama path, the layer norm around a sublayer of Dirurax, the streams kernel of
    Pikalix, the walk with fixed decays of Sotazen, the attention with a sink of Pikalix): microseconds, and what that
    is of the bytes they must move at the measured copy bandwidth."""
    import torch
    from rustinfer_b200.ops import kernels as K
    from rustinfer_b200.parts.attention_variants import PlainAttend
    from rustinfer_b200.parts.base import BuildContext
    dev = torch.device("cuda:0")
    sz = LINEDRA_SIZES[size]
    d = sz["width"]
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)
    f32 = lambda *s: torch.randn(*s, device=dev)
    frac = lambda moved, us: round(moved / (us * 1e-6) / 1e9 / hbm_gbs, 4)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    fma_per_s = sms * 128 * 1.9e9
    out = {}
    ah, akv, ad, av = sz["attn"]
    W, blocks, taps = sz["recurrent"]
    layers = sz["layers"]
    for tag, T, entries in (("prefill2048", 2048, 1), ("decode64", 64, 64)):
        cu = i32([i * (T // entries) for i in range(entries + 1)])
        slots = i32(list(range(entries)))
        # the norms around a sublayer beside the add + RMSNorm of the Llama path and Dirurax's layer norms
        h, delta, pw, nw = f32(T, d), f32(T, d), f32(d), f32(d)
        h2, xo = torch.empty(T, d, device=dev), torch.empty(T, d, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.rms_sandwich(h, delta, pw, h2, nw, xo, 1e-6), flush=flush)
        d16, w16 = bf(T, d), bf(d)
        us_rms = time_kernel(lambda: K.add_rmsnorm(h, d16, w16, 1e-6, xo), flush=flush)
        us_ln = time_kernel(lambda: K.sandwich_norm(h, d16, w16, w16, w16, w16, xo, 1e-6), flush=flush)
        out[f"rms_sandwich_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * d * (4 + 4 + 4 + 2), us),
                                      "add_rmsnorm_us": round(us_rms, 1), "add_rmsnorm_hbm_frac": frac(T * d * (4 + 4 + 2 + 2), us_rms),
                                      "layer_sandwich_us": round(us_ln, 1), "layer_sandwich_hbm_frac": frac(T * d * (4 + 4 + 2 + 2), us_ln)}
        # the end of a layer in the middle of the model: norm and add, the average over depth, the next layer's norm
        n_prev = layers // 2
        hist, dwa, avg = f32(n_prev + 1, T, d), f32(n_prev + 1), torch.empty(T, d, device=dev)
        x32 = torch.empty(T, d, device=dev)
        us = time_kernel(lambda: K.rms_sandwich(h, delta, pw, hist[n_prev], nw, x32, 1e-6, history=hist, n_prev=n_prev, dwa=dwa,
                                                avg_out=avg), flush=flush)
        streams, y = f32(2, T, d), f32(T, d)
        mix, wr, rd = f32(2, 2), f32(2), f32(2)
        us_h = time_kernel(lambda: K.hyper_collect(streams, False, y, mix, wr, rd, w16, 1e-6, xo, None), flush=flush)
        out[f"depth_average_{tag}"] = {"us": round(us, 1), "earlier_results": n_prev,
                                       "hbm_frac": frac(T * d * 4 * (n_prev + 5), us),
                                       "streams_us": round(us_h, 1), "streams_hbm_frac": frac(T * d * (4 * 5 + 2), us_h)}
        # the convolution in front of the mixer
        xin, cw = f32(T, d), f32(d, sz["taps"])
        cstate = torch.zeros(entries + 1, sz["taps"] - 1, d, device=dev)
        us = time_kernel(lambda: K.short_conv(xin, cw, None, cstate, cu, slots, xo, entries, T // entries, True), flush=flush)
        out[f"conv_input_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * d * (4 + 2) + 2 * entries * (sz["taps"] - 1) * d * 4, us)}
        # the recurrent unit: gates (two block-diagonal fp32 products), the walk beside Sotazen's walk with fixed decays
        bs = W // blocks
        u, wa, wi = f32(T, W), bf(blocks, bs, bs), bf(blocks, bs, bs)
        ba, bi, lam = f32(W), f32(W), f32(W)
        a, xg = torch.empty(T, W, device=dev), torch.empty(T, W, device=dev)
        us = time_kernel(lambda: K.rglru_gates(u, wa, wi, ba, bi, lam, 8.0, a, xg), flush=flush)
        # beside the framework's exact fp32 product on a shape of the same work: [T, bs] x [2 W, bs]
        ga, gw, go = f32(T, bs), f32(2 * W, bs), torch.empty(T, 2 * W, device=dev)
        us_g = time_kernel(lambda: K.gemm_f32(ga, gw, go), flush=flush)
        out[f"recurrent_gates_{tag}"] = {"us": round(us, 1), "fma_frac": round(2 * T * W * bs / (us * 1e-6) / fma_per_s, 4),
                                         "hbm_frac": frac(T * W * 12 + 2 * W * bs * 2, us),
                                         "gemm_f32_us": round(us_g, 1), "gemm_f32_fma_frac": round(2 * T * W * bs / (us_g * 1e-6) / fma_per_s, 4)}
        a.uniform_(0.5, 0.99)
        yv, sy = f32(T, W), torch.empty(T, W, device=dev, dtype=torch.bfloat16)
        rstate = torch.zeros(entries + 1, W, device=dev)
        us = time_kernel(lambda: K.rglru_scan(a, xg, yv, ba, rstate, cu, slots, sy, entries), flush=flush)
        H, dk, dv = max(1, W // 128), 128, 128
        p32 = f32(T, 2 * H * dk + H * dv)
        decay, o = torch.full((H * dk,), 0.97, device=dev), torch.empty(T, H * dv, device=dev)
        dstate = torch.zeros(entries + 1, H, dv, K.recurrent_state_rows(dk), device=dev)
        us_d = time_kernel(lambda: K.decay_scan(p32[:, :H * dk], p32[:, H * dk:2 * H * dk], p32[:, 2 * H * dk:], decay, 1.0, o,
                                                dstate, cu, slots, entries, H, dk, dv), flush=flush)
        out[f"recurrent_walk_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * W * (12 + 2) + 2 * entries * W * 4, us),
                                        "decay_scan_us": round(us_d, 1),
                                        "decay_scan_hbm_frac": frac(T * (2 * H * dk + 2 * H * dv) * 4 + 2 * entries * H * dk * dv * 4, us_d)}
        # a gate a head on the attention's output beside Sotazen's norm over all heads with its gate
        o32, gate = f32(T, ah * av), f32(T, ah)
        y16 = torch.empty(T, ah * av, device=dev, dtype=torch.bfloat16)
        us = time_kernel(lambda: K.sigmoid_gate(o32, gate, av, y16), flush=flush)
        g32, wn = f32(T, ah * av), bf(ah * av)
        us_n = time_kernel(lambda: K.row_norm_gate(o32, g32, wn, 1e-6, y16), flush=flush)
        out[f"head_gate_{tag}"] = {"us": round(us, 1), "hbm_frac": frac(T * ah * av * (4 + 2), us),
                                   "row_norm_gate_us": round(us_n, 1), "row_norm_gate_hbm_frac": frac(T * ah * av * (4 + 4 + 2), us_n)}
    # attention with the distance bias beside the same kernels without it (Pikalix's attention with a sink and a window)
    B, ctx, win = 64, 4096, sz["window"]
    nblk = ctx // PAGE
    bctx = BuildContext(dev, torch.bfloat16, ctx, PAGE, max_batch_seqs=B, num_sms=sms)
    kv_len, cu, ent = i32([ctx] * B), i32(list(range(B + 1))), i32(list(range(B)))
    table = torch.randperm(B * nblk, device=dev).to(torch.int32).view(B, nblk).contiguous()
    sink = torch.zeros(ah, device=dev)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / ah) for h in range(ah)], device=dev)
    att = PlainAttend(bctx, ah, akv, ad, av, window=win)
    per = akv * (ad + av)
    cache = bf(B * nblk, 2, akv, PAGE, ad) if ad == av else bf(B * nblk, PAGE * per)
    q, o = bf(B, ah * ad), torch.empty(B, ah * av, device=dev)
    res = {}
    for name, sl in (("us", slopes), ("no_bias_us", None)):
        if att.fast_single:
            ranges = att._splits(B, ctx)
            us = time_kernel(lambda: K.attention_single(q, o, cache, table, cu, kv_len, ent, ah, akv, ad, ad ** -0.5, win, None, av,
                                                        sink=True, splits=ranges, part=att.part, sink_values=sink, slopes=sl), flush=flush)
        else:
            ranges = att._rows_splits(B, ctx) if att.rows_single else 1
            us = time_kernel(lambda: K.attention_rows(q, o, cache, table, cu, kv_len, ent, att.zero_tok0[:B] if att.rows_single else i32([0] * B),
                                                      ah, akv, ad, ad ** -0.5, win, av, sink=True, sink_values=sink, splits=ranges,
                                                      part=att.part, slopes=sl), flush=flush)
        res[name] = round(us, 1)
    res.update(ranges=ranges, hbm_frac=frac(B * min(ctx, win) * per * 2, res["us"]),
               no_bias_hbm_frac=frac(B * min(ctx, win) * per * 2, res["no_bias_us"]))
    out["distance_bias_attention_decode64"] = res
    T = 2048
    tbl, cup, kvl = i32([list(range(T // PAGE))]), i32([0, T]), i32([T])
    pcache = bf(T // PAGE, 2, akv, PAGE, ad) if ad == av else bf(T // PAGE, PAGE * per)
    qp, op = bf(T, ah * ad), torch.empty(T, ah * av, device=dev)
    pairs = sum(min(p + 1, win) for p in range(T))
    res = {}
    if K.attention_rows_supports(ad, av):
        tpt = K.attention_rows_tokens_per_tile(ah, akv, ad, av)
        tl = list(range(0, T, tpt))
        ter, t0r = i32([0] * len(tl)), i32(tl)
        for name, sl in (("us", slopes), ("no_bias_us", None)):
            us = time_kernel(lambda: K.attention_rows(qp, op, pcache, tbl, cup, kvl, ter, t0r, ah, akv, ad, ad ** -0.5, win, av,
                                                      sink=True, sink_values=sink, slopes=sl), flush=flush)
            res[name] = round(us, 1)
            res[name.replace("us", "useful_tflops")] = round(2 * pairs * ah * (ad + av) / (us * 1e-6) / 1e12, 2)
    out["distance_bias_attention_prefill2048"] = res
    return out


def family_bench(args) -> int:
    """`--family dirurax|pikalix|sotazen|linedra`: prefill and decode throughput of that family's models at a few sizes beside
    Llama models of the same width, depth, feed-forward width and vocabulary (random weights), and the
    family's own kernels alone.  One JSON line."""
    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.weights.random_init import write_random_model
    hbm_gbs, bf16_tflops, peak_kind = peaks()
    clocks = ClockSampler()
    clocks.start()
    windows = []
    say = lambda msg: print(f"[bench] {msg}", file=sys.stderr, flush=True)
    ctx, tokens = min(args.context, 4096), max(2, min(args.prompt_tokens, 8192))
    family = args.family
    table = {"pikalix": PIKALIX_SIZES, "sotazen": SOTAZEN_SIZES, "linedra": LINEDRA_SIZES}.get(family, FAMILY_SIZES)
    result = {"family": family, "dtype": "bf16", "data": "synthetic", "peaks": peak_kind, "points": {}, "kernels": {}}
    sizes = [s for s in table if not args.size or s in args.size.split(",")]
    for size in sizes:
        sz = table[size]
        if family == "pikalix":
            own = _pikalix(**{k: v for k, v in sz.items() if k != "llama"})
        elif family == "sotazen":
            own = _sotazen(**{k: v for k, v in sz.items() if k != "llama"})
        elif family == "linedra":
            own = _linedra(**{k: v for k, v in sz.items() if k != "llama"})
        else:
            own = _dirurax(sz["width"], sz["layers"], sz["ff"], sz["vocab"], sz["gla"], sz["attn"], sz["delta"], sz["block"])
        configs = {family: own, "llama": _llama_like(sz["width"], sz["layers"], sz["ff"], sz["vocab"], *sz["llama"])}
        if family == "linedra":                      # also beside the nearest of the other families, at equal size
            configs["pikalix"] = _pikalix(**{k: v for k, v in PIKALIX_SIZES[size].items() if k != "llama"})
        point = {}
        for fam, cfg in configs.items():
            with tempfile.TemporaryDirectory(prefix="rustinfer_b200_bench_") as tmp:
                folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=SEED, std=STD)
                weights = os.path.getsize(os.path.join(folder, "model.safetensors"))
                seqs = max(args.batch, 1)
                longest = max(ctx, tokens)
                engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=seqs, max_model_len=longest,
                                paged_block_size=PAGE, num_blocks=seqs * longest // PAGE + 64,
                                capture_sizes=[1, 2, 4, 8, 16, 32, 64], ignore_eos=True)
                ms_p, pw = prefill_timed(engine, sz["vocab"], tokens, repeats=3)
                windows += pw
                steps = max(args.steps, 32)
                decode_device_timed(engine, args.batch, steps, args.warmup, sz["vocab"], 1, ctx)      # graphs captured: untimed
                (ms_d, launches, w), _all = median_of(
                    lambda: decode_device_timed(engine, args.batch, steps, args.warmup, sz["vocab"], 2, ctx), 3)
                windows.append(w)
                point[fam] = {"prefill_tokens_per_s": round(tokens / ms_p * 1e3), "prefill_ms": round(ms_p, 3),
                              "decode_tokens_per_s": round(args.batch / ms_d * 1e3, 1), "decode_ms_per_step": round(ms_d, 4),
                              "decode_launches_per_step": launches // steps, "weight_mb": round(weights / 1e6, 1),
                              "decode_weight_hbm_frac": round(weights / (ms_d * 1e-3) / 1e9 / hbm_gbs, 4)}
                say(f"{size} {fam}: prefill {tokens} tokens {ms_p:.3f} ms, decode b{args.batch} ctx{ctx} {ms_d:.4f} ms/step")
                del engine
                torch.cuda.empty_cache()
        point["prefill_ratio"] = round(point[family]["prefill_tokens_per_s"] / point["llama"]["prefill_tokens_per_s"], 3)
        point["decode_ratio"] = round(point[family]["decode_tokens_per_s"] / point["llama"]["decode_tokens_per_s"], 3)
        if "pikalix" in point and family != "pikalix":
            point["prefill_ratio_to_pikalix"] = round(point[family]["prefill_tokens_per_s"] / point["pikalix"]["prefill_tokens_per_s"], 3)
            point["decode_ratio_to_pikalix"] = round(point[family]["decode_tokens_per_s"] / point["pikalix"]["decode_tokens_per_s"], 3)
        result["points"][size] = point
        result["kernels"][size] = (pikalix_kernels(hbm_gbs, bf16_tflops, size) if family == "pikalix"
                                   else sotazen_kernels(hbm_gbs, bf16_tflops, size) if family == "sotazen"
                                   else linedra_kernels(hbm_gbs, bf16_tflops, size) if family == "linedra"
                                   else dirurax_kernels(hbm_gbs, size))
        say(f"{size} kernels: {result['kernels'][size]}")
    clocks.stop()
    result["config"] = {"batch": args.batch, "context": ctx, "prompt_tokens": tokens,
                        "sizes": {s: {k: v for k, v in table[s].items()} for s in sizes},
                        "l2": "a 256 MB buffer is rewritten between timed kernel runs; model steps read weights larger than L2"}
    result["clocks"] = clocks.summary(windows)
    print(json.dumps(result))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes (default: the 1B shape)")
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--skip-points", action="store_true", help="leave out everything under `points`")
    ap.add_argument("--repeats", type=int, default=5, help="timed windows of the headline (the median is reported)")
    ap.add_argument("--only", choices=["decode", "prefill", "serve", "e2e"],
                    help="run one part alone and print its time (for profiler captures; no JSON line); "
                         "serve: 64 requests, prompts of 128 to 2,048 tokens, 256 tokens out each, "
                         "prompt portions of 512, through Engine.generate; e2e: the decode steps through "
                         "Engine.step with host tokens in and out, and where the host's time in a step goes")
    ap.add_argument("--eager", action="store_true", help="with --only decode: no CUDA graphs")
    ap.add_argument("--sampled", action="store_true",
                    help="with --only decode: every token drawn (temperature 0.8, top-k 50, top-p 0.9) instead of the argmax")
    ap.add_argument("--context", type=int, default=CONTEXT, help="with --only: context the decode ends at")
    ap.add_argument("--prompt-tokens", type=int, default=PREFILL_TOKENS,
                    help="with --only prefill: length of the prompt, computed in one step (up to 8192)")
    ap.add_argument("--family", default="llama", choices=["llama", "dirurax", "pikalix", "sotazen", "linedra"],
                    help="dirurax, pikalix: that family's prefill and decode at a few sizes beside Llama models of equal size, "
                         "and its kernels alone (one JSON line of its own; the default workload is unchanged)")
    ap.add_argument("--size", default="", help="with --family dirurax or pikalix: sizes to run, with commas (default: all)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: --gpus {args.gpus} is not supported by this engine")
        return 2
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip install of the reference fails at metadata generation (a Rust workspace whose "
                          "pyproject.toml declares no Python package) and no cargo/rustc is in this image"}))
        return 0
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 2)
    if args.family in ("dirurax", "pikalix", "sotazen", "linedra"):
        return family_bench(args)

    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.weights.random_init import write_random_model

    hbm_gbs, bf16_tflops, peak_kind = peaks()
    shape_name, shape = SHAPES[args.shape]
    if args.layers <= 0:
        args.layers = shape["num_hidden_layers"]
    cfg = dict(shape, num_hidden_layers=args.layers)
    vocab = cfg["vocab_size"]
    per_layer, weight_bytes, kv_per_token, q_dim = model_numbers(cfg, args.layers)
    clocks = ClockSampler()
    clocks.start()
    windows = []
    with tempfile.TemporaryDirectory(prefix="rustinfer_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=SEED, std=STD)
        if args.only == "serve":
            serve_workload(folder, vocab, args.layers)
            clocks.stop()
            return 0
        if args.only:
            seqs = max(args.batch, 1)
            longest = max(CONTEXT, min(args.prompt_tokens, 8192))
            engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=seqs,
                            max_model_len=longest, paged_block_size=PAGE, num_blocks=seqs * longest // PAGE + 64,
                            capture_sizes=[] if args.eager else [1, 2, 4, 8, 16, 32, 64], ignore_eos=True)
            if args.only == "e2e":
                decode_e2e(engine, args.batch, args.steps, args.warmup, vocab, 1)          # graphs captured: untimed
                ms, _, _, _ = decode_e2e(engine, args.batch, args.steps, args.warmup, vocab, 2, trace=True)
                host = dict(engine.stats.host_seconds)
                ms_dev, _, _ = decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, 3)
                print(f"e2e b{args.batch} layers{args.layers}: {ms:.4f} ms/step through Engine.step, {ms_dev:.4f} device-timed")
                n = args.steps - 1
                for what, sec in host.items():
                    print(f"  host, {what}: {sec / n * 1e6:8.1f} us a step")
                busy = sum(sec for what, sec in host.items() if not what.startswith("wait"))
                print(f"  host busy {busy / n * 1e6:.1f} us of the step's {ms * 1e3:.1f} us; the rest it waits for the GPU")
            elif args.only == "decode":
                global_ctx = args.context
                sp = None
                if args.sampled:
                    from rustinfer_b200.sampling.params import SamplingParams
                    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1, max_tokens=CONTEXT, ignore_eos=True)
                ms, n, _ = decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, 1, global_ctx, sampling=sp)
                print(f"decode b{args.batch} ctx{global_ctx} layers{args.layers}{' sampled' if sp else ''}: {ms:.4f} ms/step, {n} launches")
            else:
                tokens = max(2, min(args.prompt_tokens, 8192))
                ms, _ = prefill_timed(engine, vocab, tokens, repeats=max(1, min(args.steps, 3)))
                print(f"prefill {tokens} layers{args.layers}: {ms:.3f} ms")
            clocks.stop()
            return 0
        engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=64,
                        max_model_len=CONTEXT, paged_block_size=PAGE, chunked_prefill_size=0,
                        num_blocks=64 * CONTEXT // PAGE + 64, capture_sizes=[1, 2, 4, 8, 16, 32, 64],
                        ignore_eos=True)
        say = lambda msg: print(f"[bench] {msg}", file=sys.stderr, flush=True)
        reps = args.repeats
        seeds = iter(range(100, 10_000))
        # ---- the headline: K decode steps at the asked batch, device-timed, repeated
        (ms_step, launches, w), decode_ms = median_of(
            lambda: decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, next(seeds)), reps)
        windows.append(w)
        say(f"decode b{args.batch}: {ms_step:.4f} ms/step (of {decode_ms})")
        (e2e_ms, h2d, d2h, w), e2e_all = median_of(
            lambda: decode_e2e(engine, args.batch, args.steps, args.warmup, vocab, next(seeds)), reps)
        windows.append(w)
        say(f"e2e b{args.batch}: {e2e_ms:.4f} ms/step (of {e2e_all})")
        prefill_ms, pw = prefill_timed(engine, vocab, PREFILL_TOKENS, repeats=reps)
        windows += pw
        say(f"prefill {PREFILL_TOKENS}: {prefill_ms:.3f} ms")
        points = {}
        if not args.skip_points:
            from rustinfer_b200.sampling.params import SamplingParams
            k = max(args.steps, 64)                       # (the headline keeps exactly --steps; these are its company)
            for b in (1, 64):
                (ms_b, _, w), _all = median_of(lambda: decode_device_timed(engine, b, k, args.warmup, vocab, next(seeds)), 3)
                windows.append(w)
                points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)
                points[f"decode_b{b}_hbm_frac"] = round(step_bytes_of(cfg, args.layers, b, CONTEXT - k / 2) / (ms_b * 1e-3) / 1e9 / hbm_gbs, 4)
                (ms_e, _, _, w), _all = median_of(lambda: decode_e2e(engine, b, k, args.warmup, vocab, next(seeds)), 3)
                windows.append(w)
                points[f"e2e_b{b}"] = round(b / ms_e * 1e3, 1)
                say(f"decode b{b}: {ms_b:.4f} ms/step, e2e {ms_e:.4f}")
            # the same steps with every token drawn (temperature 0.8, top-k 50, top-p 0.9) instead of the
            # argmax.  Windows of the two kinds alternate and each drawn one is set against the greedy
            # one before it: minutes into a run the clocks under the power cap move a window by
            # several per cent, more than the sampler costs.
            sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1, max_tokens=CONTEXT, ignore_eos=True)
            drawn, ratios = [], []
            for _ in range(3):
                ms_g, _, w = decode_device_timed(engine, args.batch, k, args.warmup, vocab, next(seeds))
                windows.append(w)
                ms_s, _, w = decode_device_timed(engine, args.batch, k, args.warmup, vocab, next(seeds), sampling=sp)
                windows.append(w)
                drawn.append(ms_s)
                ratios.append(ms_g / ms_s)
            ms_s = statistics.median(drawn)
            points[f"decode_b{args.batch}_sampled"] = round(args.batch / ms_s * 1e3, 1)
            points[f"decode_b{args.batch}_sampled_vs_greedy"] = round(statistics.median(ratios), 4)
            say(f"decode b{args.batch} sampled: {ms_s:.4f} ms/step, {statistics.median(ratios):.3f} of greedy windows beside it")
        del engine
        torch.cuda.empty_cache()
    if not args.skip_points and args.shape == "1b":
        points.update(further_shapes(args, hbm_gbs, bf16_tflops, windows, say))
        try:
            points.update(kernel_ratios())
        except Exception as e:                                # the comparison must not cost the headline its line
            points["kernel_ratios_error"] = f"{type(e).__name__}: {e}"[:200]
    clocks.stop()

    value = args.batch / ms_step * 1e3
    mean_ctx = CONTEXT - args.steps / 2
    step_bytes = step_bytes_of(cfg, args.layers, args.batch, mean_ctx)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    T = PREFILL_TOKENS
    prefill_flops = prefill_flops_of(cfg, args.layers, T)
    prefill_frac = prefill_flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12)
    out = {
        "metric": f"decode tok/s @ batch {args.batch}, context {CONTEXT} ({shape_name}, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids",
        "config": {"model": shape_name, "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "tied_head": cfg["tie_word_embeddings"],
                   "page_size": PAGE, "prefill_tokens": T, "cuda_graphs": True,
                   "l2": "each step reads %.2f GB of weights and cache, far beyond the 126 MB L2" % (step_bytes / 1e9),
                   "peaks": peak_kind,
                   "windows": f"median of {reps} windows of {args.steps} steps, each after {SETTLE_STEPS} untimed "
                              f"decode steps behind the burst that fills the context, then the warm-up"},
        "spread": {"decode_ms": decode_ms, "e2e_ms": e2e_all},
        "e2e": {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4)},
        "gpu_launches": launches,
        "prefill": {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
        "clocks": clocks.summary(windows),
    }
    print(json.dumps(out))
    return 0


def step_bytes_of(cfg, layers, batch, mean_ctx):
    """Bytes a decode step has to read: every weight once, and the cache of the live requests."""
    _, weight_bytes, kv_per_token, _ = model_numbers(cfg, layers)
    if not cfg["tie_word_embeddings"]:
        weight_bytes += 0                                    # the untied head is the table counted; the embedding is only gathered
    return weight_bytes + batch * mean_ctx * kv_per_token


def prefill_flops_of(cfg, layers, T):
    per_layer, _, _, q_dim = model_numbers(cfg, layers)
    return 2 * T * layers * per_layer + 2 * cfg["vocab_size"] * cfg["hidden_size"] + 2 * T * T * q_dim * layers


def further_shapes(args, hbm_gbs, bf16_tflops, windows, say):
    """The other benchmark configurations, at 8 of their layers each (both numbers are in the
    keys): the 8B shape (decode at batch 1, 8, 64, a 2,048-token prefill, one 32,768-token prompt)
    and the 3B shape serving 64 requests at once."""
    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.weights.random_init import write_random_model
    out = {}
    seeds = iter(range(20_000, 30_000))
    # (windows as long as the headline's: the steps right after the burst that fills the context run
    # several per cent slower than the ones that follow, and a short window is mostly those)
    k = max(args.steps, 64)
    # ---- Llama-3.1-8B-shaped, 8 of 32 layers
    name, shape = SHAPES["8b"]
    layers = 8
    cfg = dict(shape, num_hidden_layers=layers)
    tag = f"8b_l{layers}of{shape['num_hidden_layers']}"
    with tempfile.TemporaryDirectory(prefix="rustinfer_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=4, std=STD)
        engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=64, max_model_len=CONTEXT,
                        paged_block_size=PAGE, num_blocks=64 * CONTEXT // PAGE + 64,
                        capture_sizes=[1, 2, 4, 8, 16, 32, 64], ignore_eos=True)
        for b in (1, 8, 64):
            (ms_b, _, w), _all = median_of(lambda: decode_device_timed(engine, b, k, args.warmup, cfg["vocab_size"], next(seeds)), 3)
            windows.append(w)
            out[f"{tag}_decode_b{b}"] = round(b / ms_b * 1e3, 1)
            out[f"{tag}_decode_b{b}_hbm_frac"] = round(step_bytes_of(cfg, layers, b, CONTEXT - k / 2) / (ms_b * 1e-3) / 1e9 / hbm_gbs, 4)
            say(f"{tag} decode b{b}: {ms_b:.4f} ms/step")
        ms_p, pw = prefill_timed(engine, cfg["vocab_size"], PREFILL_TOKENS, repeats=3)
        windows += pw
        out[f"{tag}_prefill_2048"] = round(PREFILL_TOKENS / ms_p * 1e3, 1)
        out[f"{tag}_prefill_2048_tc_frac"] = round(prefill_flops_of(cfg, layers, PREFILL_TOKENS) / (ms_p * 1e-3) / (bf16_tflops * 1e12), 4)
        say(f"{tag} prefill 2048: {ms_p:.3f} ms")
        del engine
        torch.cuda.empty_cache()
        w0 = time.time()
        lp = long_prompt(folder, cfg["vocab_size"], cfg, layers)
        windows.append((w0, time.time()))
        out[f"{tag}_prompt_32768"] = lp["tok_s"]
        out[f"{tag}_prompt_32768_attention_share"] = lp["attention_share"]
        out[f"{tag}_prompt_32768_tc_frac"] = round(lp["tflops"] / bf16_tflops, 4)
        say(f"{tag} prompt of 32,768: {lp['ms']} ms, attention {lp['attention_share']:.0%}")
    # ---- Llama-3.2-3B-shaped, 8 of 28 layers: 64 requests at once through Engine
    name, shape = SHAPES["3b"]
    cfg = dict(shape, num_hidden_layers=layers)
    tag = f"3b_l{layers}of{shape['num_hidden_layers']}"
    with tempfile.TemporaryDirectory(prefix="rustinfer_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=3, std=STD)
        w0 = time.time()
        sv = serve_workload(folder, cfg["vocab_size"], layers, quiet=True)
        windows.append((w0, time.time()))
        out[f"{tag}_serve64_tok_s"] = sv["tok_s"]
        out[f"{tag}_serve64_out_tok_s"] = sv["out_tok_s"]
        out[f"{tag}_serve64_step_ms_mean"] = sv["step_ms_mean"]
        out[f"{tag}_serve64_step_ms_p99"] = sv["step_ms_p99"]
        out[f"{tag}_serve64_preemptions"] = sv["preemptions"]
        say(f"{tag} serve: {sv}")
    return out


if __name__ == "__main__":
    sys.exit(main())
