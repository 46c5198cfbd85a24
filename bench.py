#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
    python bench.py --case prefill|decode [--shape 8b|1b|13b] [--dtype bfloat16|float32] [--layers L] [--batch B]
                    [--context C] [--prompt-tokens T]                 one phase alone (for profilers and sweeps)
    python bench.py --case workload-1b      64 prompts of 16..1,024 tokens in one step, then 128 steps (1B shape)
    python bench.py --case workload-13b     8 prompts of 2,048 tokens, then 256 steps (13B shape)
    python bench.py --case float32 [--layers L]    the 8B shape in true 32-bit: a 2,048-token prompt, decode at batch 1 and 8
    python bench.py --case reference-kernels [--context C]     the reference's CUDA kernels alone, if they were built
    python bench.py --case tumatar [--shape 1b|8b] [--layers L]    the Tumatar design beside Llama at equal width, its kernels alone
    python bench.py --case tikalix [--shape 1b|8b] [--layers L]    the Tikalix design beside Llama at equal width, its kernels alone
    python bench.py --case vilazen [--shape 1b|8b] [--layers L]    the Vilazen design beside Llama at equal width, its kernels alone
    python bench.py --case lipadra [--shape 1b|8b] [--layers L]    the Lipadra design beside Tumatar and Llama at equal width, its kernels alone

A "step" is one decode step of a batch of 8 sequences at a context of 4096
tokens.  ``value`` is decoded tokens a second, timed on the device with CUDA
events over exactly K steps after W warm-up steps, each with its greedy choice
on the device; ``e2e`` is the same K steps inside ``Engine.generate``, the call a
user makes: prompts of host token ids in, every step's integers copied from
pinned host memory, every step's sampled ids read back, timed by the wall clock.  The line
also carries the prefill of 2,048 tokens, the decode step's memory roofline,
decode at batch 1 and 64, the SM clocks seen during the timed region and the
number of kernels launched in it.  Weights are random N(0, 0.02) in bfloat16
and token ids are uniform random: there is no dataset or checkpoint here.

The reference (a Zig program with one CUDA file) has no Python package and no
Zig toolchain is installed, so ``--impl reference`` reports itself unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from ziglm_b200.config.shapes import shape as _shape  # noqa: E402  (plain dictionaries, no CUDA needed)

LLAMA_8B, LLAMA_1B, LLAMA_13B = _shape("llama-8b"), _shape("llama-1b"), _shape("llama-13b")
SHAPES = {"8b": LLAMA_8B, "1b": LLAMA_1B, "13b": LLAMA_13B}
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
        return out
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.samples = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(int(float(s[0])))
                mx = max(mx, int(float(s[1])))
            except ValueError:
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


def decode_bytes(cfg, n_layers, batch, context, bytes_per_el=2, cached_tokens=None):
    """Bytes a decode step has to read: every weight it uses once and the cache of the live requests
    (``cached_tokens``: the sum of their lengths; default batch * context).  A tied head is the embedding
    table, read once as the head; an untied model reads its head and `batch` rows of the embedding."""
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * q + 2 * d * kv + q * d + 3 * d * i + 2 * d
    weights = n_layers * per_layer + v * d + d
    if cached_tokens is None:
        cached_tokens = context * batch
    cache = n_layers * 2 * kv * cached_tokens
    return (weights + cache) * bytes_per_el + batch * d * bytes_per_el


def prefill_flops(cfg, n_layers, tokens, wanted=1):
    """FLOPs of one prompt of ``tokens`` tokens whose last ``wanted`` places go through the head."""
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2 * tokens * (d * q + 2 * d * kv + q * d + 3 * d * i)
    attn = 2 * 2 * q * tokens * (tokens + 1) / 2               # QK^T and PV over the causal half
    return n_layers * (linear + attn) + wanted * 2 * d * v


def wait_errors(kernels):
    """The error words of the kernels' bounded waits, as a list in a fixed order (0: none)."""
    codes = kernels.wait_errors()
    return [codes.get(k, 0) for k in ("gemm_tc", "attention_tc", "attention_fmha")]


def run_ours(args):
    import torch
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams, config_from_dict, kernels

    torch.cuda.set_device(0)
    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg["num_hidden_layers"] = n_layers
    pk = peaks()
    steps, warmup = args.steps, max(3, args.warmup)
    slack = 64
    max_seq = CONTEXT + slack
    kernels.require(("sampling",))

    def make_engine(batch):
        opts = EngineOptions(dtype="bfloat16", max_batch=batch, max_seq_len=max_seq,
                             max_tokens=batch * (-(-max_seq // 64) * 64), seed=1234)
        return Engine.from_config(config_from_dict(cfg), opts)

    gen = torch.Generator().manual_seed(7)

    def random_ids(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()

    def fill(engine, batch, context):
        """Give `batch` sequences `context` cached tokens each, by real prompt steps of at most 2048 tokens."""
        slots = [engine.alloc_slot() for _ in range(batch)]
        for s in slots:
            done = 0
            while done < context:
                n = min(2048, context - done)
                engine.step([(s, random_ids(n))], [[]])
                done += n
        return slots

    def time_decode(engine, slots, n_warm, n_steps):
        """Device time of n_steps decode steps, each with its greedy choice on the device (ms per step), and
        the kernels launched in them."""
        ids = [random_ids(len(slots)) for _ in range(n_warm + n_steps)]
        picked = torch.empty(len(slots), dtype=torch.int32, device="cuda")
        for k in range(n_warm):
            kernels.argmax(engine.step([(s, [t]) for s, t in zip(slots, ids[k])]), picked)
        torch.cuda.synchronize()
        kernels.reset_launches()
        engine.graph_launched_kernels()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(n_warm, n_warm + n_steps):
            kernels.argmax(engine.step([(s, [t]) for s, t in zip(slots, ids[k])]), picked)
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / n_steps, kernels.launches() + engine.graph_launched_kernels()

    def time_end_to_end(engine, batch, n_warm, n_steps):
        """The same steps through the Python entry point, ``Engine.generate``: prompts of host token ids in, the
        generated ids out.  Every step copies its integers (positions, lengths, block tables) from pinned host
        memory and its sampled ids are read back; the loop runs one step ahead of the ids it reads.  One call
        generates n_warm + n_steps + 1 tokens per sequence; the per-token callback of the entry point stamps
        the wall clock when a step's ids have arrived on the host, and the last n_steps steps are the timed
        ones.  The warm-up is 30 steps longer than asked for: the first ten or so steps after the long prompts
        run a quarter slower, on a GPU that the prompts have just driven into its power cap (measured: 4.7 ms
        a step against 3.83 from the twentieth step on, batch 8), and the first decode step of a batch size is
        captured."""
        n_warm += 30
        prompts = [random_ids(max(1, CONTEXT - n_warm - n_steps - 1)) for _ in range(batch)]
        stamps = []

        def stamp(request, token):
            if request == 0:
                stamps.append(time.perf_counter())
            return True

        opts = GenerationOptions(max_tokens=n_warm + n_steps + 1, ignore_eos=True, sampler=SamplerParams(greedy=True))
        results, _ = engine.generate(prompts, opts, callback=stamp)
        assert all(len(r.tokens) == n_warm + n_steps + 1 for r in results) and len(stamps) == n_warm + n_steps + 1
        return (stamps[-1] - stamps[-1 - n_steps]) * 1000.0 / n_steps, engine.last_step_h2d_bytes

    def frac(batch, ms):
        return decode_bytes(cfg, n_layers, batch, CONTEXT) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]

    # each phase starts so far below the context that its warm-up and timed steps end at it
    start_ctx = max(1, CONTEXT - (warmup + steps) - 1)
    # ---------------------------------------------------------------- prefill, 2048 tokens of one sequence
    engine = make_engine(8)
    prompt = random_ids(PREFILL_TOKENS)
    times = []
    for k in range(3 + 3):
        slot = engine.alloc_slot()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([(slot, prompt)])
        e.record()
        torch.cuda.synchronize()
        if k >= 3:
            times.append(s.elapsed_time(e))
        engine.free_slot(slot)
    pre_ms = sorted(times)[len(times) // 2]
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / pre_ms * 1000.0, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---------------------------------------------------------------- decode, batch 8 at the context length
    batch = 8
    slots = fill(engine, batch, start_ctx)
    with ClockSampler() as clocks:
        ms, launched = time_decode(engine, slots, warmup, steps)
    clock_summary = clocks.summary()
    tok_s = batch / ms * 1000.0
    bytes_step = decode_bytes(cfg, n_layers, batch, CONTEXT)
    achieved = bytes_step / (ms * 1e-3) / 1e9
    for s in slots:
        engine.free_slot(s)
    e2e_ms, h2d = time_end_to_end(engine, batch, warmup, steps)

    # ---------------------------------------------------------------- decode at batch 1 and 64
    points = {}
    s1 = fill(engine, 1, start_ctx)
    ms1, _ = time_decode(engine, s1, warmup, steps)
    engine.free_slot(s1[0])
    e2e1, _ = time_end_to_end(engine, 1, warmup, steps)
    del engine
    torch.cuda.empty_cache()
    engine = make_engine(64)
    s64 = fill(engine, 64, start_ctx)
    ms64, _ = time_decode(engine, s64, warmup, steps)
    for s in s64:
        engine.free_slot(s)
    e2e64, _ = time_end_to_end(engine, 64, warmup, steps)
    points["decode_b1"] = round(1 / ms1 * 1000.0, 1)
    points["decode_b64"] = round(64 / ms64 * 1000.0, 1)
    points["decode_b1_hbm_frac"] = round(frac(1, ms1), 4)
    points["decode_b64_hbm_frac"] = round(frac(64, ms64), 4)
    points["e2e_b1"] = round(1 / e2e1 * 1000.0, 1)
    points["e2e_b64"] = round(64 / e2e64 * 1000.0, 1)

    line = {
        "metric": "decode tok/s at batch 8 (Llama-3.1-8B shape, context 4096)",
        "value": round(tok_s, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Llama-3.1-8B shape", "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
            "layers": n_layers, "layers_of_config": full_layers, "hidden_size": cfg["hidden_size"],
            "intermediate_size": cfg["intermediate_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"],
            "rope_theta": cfg["rope_theta"], "rope_scaling": "llama3 factor 8 low 1 high 4 orig 8192",
            "rms_norm_eps": cfg["rms_norm_eps"], "tied": False, "prefill_tokens": PREFILL_TOKENS,
            "l2": "inputs larger than L2 (weights read each step exceed 126 MB)", "peaks": pk["source"],
        },
        "e2e": {"value": round(batch / e2e_ms * 1000.0, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": batch * 4},
        "gpu_launches": int(launched),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
        "wait_errors": wait_errors(kernels),
    }
    print(json.dumps(line))
    return 0


def _engine_for(cfg, dtype, batch, max_seq, tokens=None, seed=1234):
    from ziglm_b200 import Engine, EngineOptions, config_from_dict
    page = 64
    max_tokens = tokens if tokens is not None else batch * (-(-max_seq // page) * page)
    return Engine.from_config(config_from_dict(cfg), EngineOptions(dtype=dtype, max_batch=batch, max_seq_len=max_seq,
                                                                   max_tokens=max_tokens, seed=seed))


def _time_prompt(eng, prompt, warmup, steps):
    """Median device time (ms) of one prompt step of a fresh sequence."""
    import torch
    times = []
    for k in range(warmup + steps):
        slot = eng.alloc_slot()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        eng.step([(slot, prompt)])
        e.record()
        torch.cuda.synchronize()
        if k >= warmup:
            times.append(s.elapsed_time(e))
        eng.free_slot(slot)
    return sorted(times)[len(times) // 2]


def _time_decode_at(eng, batch, context, warmup, steps, ids):
    """Median device time (ms) of a decode step of ``batch`` sequences that hold ``context`` tokens when the timed
    steps end.  The cache is given its length without being computed: a decode step's time does not depend on
    what the cache holds."""
    import torch
    slots = [eng.alloc_slot() for _ in range(batch)]
    grow = {s: max(1, context - warmup - steps - 1) for s in slots}
    eng.cache.slots.reserve(grow)
    eng.cache.slots.advance(grow)
    times = []
    for k in range(warmup + steps):
        toks = ids(batch)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        eng.step([(sl, [t]) for sl, t in zip(slots, toks)])
        e.record()
        torch.cuda.synchronize()
        if k >= warmup:
            times.append(s.elapsed_time(e))
    for s in slots:
        eng.free_slot(s)
    return sorted(times)[len(times) // 2]


def run_case(args):
    """A single phase on a (possibly shallower) model, for profilers and sweeps: a prompt, or decode steps."""
    import torch
    from ziglm_b200 import kernels
    torch.cuda.set_device(0)
    cfg = dict(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or full_layers
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], args.context + 64, args.prompt_tokens + 64)
    batch, context = args.batch, args.context
    max_seq = max(context, args.prompt_tokens) + 64
    eng = _engine_for(cfg, args.dtype, batch, max_seq)
    gen = torch.Generator().manual_seed(7)
    ids = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()
    pk = peaks()
    el = 2 if args.dtype == "bfloat16" else 4
    out = {"case": args.case, "shape": args.shape, "dtype": args.dtype, "layers": cfg["num_hidden_layers"],
           "layers_of_config": full_layers, "batch": batch, "context": context}
    if args.case == "prefill":
        ms = _time_prompt(eng, ids(args.prompt_tokens), args.warmup, args.steps)
        flops = prefill_flops(cfg, cfg["num_hidden_layers"], args.prompt_tokens)
        out.update({"prompt_tokens": args.prompt_tokens, "ms": round(ms, 4),
                    "tok_s": round(args.prompt_tokens / ms * 1000.0, 1), "tflops": round(flops / ms / 1e9, 1)})
        if args.dtype == "bfloat16":
            out["frac_of_bf16_peak"] = round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
    else:
        ms = _time_decode_at(eng, batch, context, args.warmup, args.steps, ids)
        nbytes = decode_bytes(cfg, cfg["num_hidden_layers"], batch, context, el)
        out.update({"ms": round(ms, 4), "tok_s": round(batch / ms * 1000.0, 1), "gb_per_step": round(nbytes / 1e9, 3),
                    "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)})
    out["peaks"] = pk["source"]
    out["wait_errors"] = wait_errors(kernels)
    print(json.dumps(out))
    return 0


def _timed(fn, warmup, steps, flush):
    """Median device time (ms) of ``fn()``, with a buffer larger than L2 rewritten before every timed call."""
    import torch
    times = []
    for k in range(warmup + steps):
        flush.add_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        if k >= warmup:
            times.append(s.elapsed_time(e))
    return sorted(times)[len(times) // 2]


def run_tumatar(args):
    """The Tumatar design beside the Llama shape of the same width, with random weights: a prompt of
    ``--prompt-tokens`` and decode steps of ``--batch`` sequences at ``--context``, ``--layers`` layer runs of each
    (default 4), and every kernel the design adds, alone, against its own roofline (the larger of bytes / measured
    copy bandwidth and FLOPs / measured bf16 peak), beside the library's kernels of the like kind."""
    import torch
    from types import SimpleNamespace
    from ziglm_b200 import kernels
    from ziglm_b200.config.shapes import shape
    torch.cuda.set_device(0)
    pk = peaks()
    size = "8b" if args.shape == "8b" else "1b"
    layers = args.layers or 4
    T, batch, context = args.prompt_tokens, args.batch, args.context
    max_seq = max(context, T) + 64
    gen = torch.Generator().manual_seed(7)
    out = {"case": "tumatar", "width_of": "llama-" + size, "dtype": "bf16", "layer_runs": layers, "prompt_tokens": T,
           "batch": batch, "context": context, "data": "synthetic", "l2": "a 256 MiB buffer is rewritten before every timed call",
           "peaks": pk["source"], "models": {}}
    for name in ("tumatar-" + size, "llama-" + size):
        cfg = shape(name)
        if "layers" in cfg:
            cfg["layers"] = cfg["layers"][:layers]
            vocab = cfg["vocab"]
        else:
            cfg["num_hidden_layers"] = layers
            cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], max_seq)
            vocab = cfg["vocab_size"]
        eng = _engine_for(cfg, "bfloat16", batch, max_seq)
        ids = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        pre = _time_prompt(eng, ids(T), args.warmup, args.steps)
        dec = _time_decode_at(eng, batch, context, args.warmup, args.steps, ids)
        out["models"][name] = {"prefill_ms": round(pre, 3), "prefill_tok_s": round(T / pre * 1e3, 1),
                               "decode_ms": round(dec, 4), "decode_tok_s": round(batch / dec * 1e3, 1)}
        del eng
        torch.cuda.empty_cache()
    # ---- the kernels, alone
    cfg = shape("tumatar-" + size)
    d = cfg["width"]
    lat, rec = cfg["layers"][1]["mixer"], cfg["layers"][0]["mixer"]
    moe = cfg["layers"][1]["mlp"]
    H, D, R, C, K = lat["heads"], lat["dim"], lat["kv_rank"], rec["width"], rec["conv"]
    nb = rec["blocks"]
    E, top, ff = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"]
    dev = torch.device("cuda:0")
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    bf = lambda *sh: (torch.randn(*sh, device=dev) * 0.05).to(torch.bfloat16)
    f32 = lambda *sh: torch.randn(*sh, device=dev) * 0.05
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = []

    def report(what, like, ms, nbytes, flops):
        floor = max(nbytes / hbm, flops / peak) * 1e3
        rows.append({"kernel": what, "like": like, "ms": round(ms, 4), "roofline_ms": round(floor, 4),
                     "frac_of_roofline": round(floor / ms, 4)})

    kernels.require(("elementwise", "block_linear", "recurrent", "moe", "gemm_generic", "gemm_tc"))
    for n_tok, tag in ((T, f"prompt of {T}"), (batch, f"decode batch {batch}")):
        st = SimpleNamespace(seq_of_token=torch.zeros(n_tok, dtype=torch.int32, device=dev) if n_tok == T else
                             torch.arange(n_tok, dtype=torch.int32, device=dev),
                             cu_seqlens=(torch.tensor([0, n_tok], dtype=torch.int32, device=dev) if n_tok == T else
                                         torch.arange(n_tok + 1, dtype=torch.int32, device=dev)),
                             slots=torch.arange(1 if n_tok == T else n_tok, dtype=torch.int32, device=dev),
                             n_seqs=1 if n_tok == T else n_tok, max_new=n_tok if n_tok == T else 1, n_tokens=n_tok)
        # the library's like kernels at the same width: a dense product, a norm
        x, w, y = bf(n_tok, d), bf(d, d), torch.empty(n_tok, d, dtype=torch.bfloat16, device=dev)
        ms = _timed(lambda: kernels.gemm_tc(x, w, y), args.warmup, args.steps, flush)
        report(f"gemm_tc {d}x{d}, {tag}", "-", ms, 2 * (n_tok * d * 2) + d * d * 2, 2.0 * n_tok * d * d)
        xr, wn, yn = f32(n_tok, d), bf(d), torch.empty(n_tok, d, dtype=torch.bfloat16, device=dev)
        ms = _timed(lambda: kernels.rmsnorm(xr, wn, yn, 1e-6), args.warmup, args.steps, flush)
        report(f"rmsnorm, {tag}", "-", ms, n_tok * d * 6 + d * 2, 0)
        # the design's own
        res = f32(n_tok, d)
        ms = _timed(lambda: kernels.rmsnorm_rows(xr, wn, res, 1e-6, add=True), args.warmup, args.steps, flush)
        report(f"rmsnorm_rows (post-norm + residual sum), {tag}", "rmsnorm", ms, n_tok * d * 12 + d * 2, 0)
        q, ukt = bf(n_tok, H * D), bf(H, R, D)
        qc = torch.empty(n_tok, (H + 1) * R, dtype=torch.bfloat16, device=dev)
        ms = _timed(lambda: kernels.block_linear(q, ukt, qc[:, :H * R]), args.warmup, args.steps, flush)
        report(f"block_linear (queries into the latent, {H} heads {D}->{R}), {tag}", "gemm_tc", ms,
               n_tok * H * (D + R) * 2 + H * R * D * 2, 2.0 * n_tok * H * D * R)
        u, gw, gb = bf(n_tok, C), bf(nb, 2 * C // nb, C // nb), f32(2 * C)
        gates = torch.empty(n_tok, 2 * C, dtype=torch.float32, device=dev)
        ms = _timed(lambda: kernels.block_linear(u, gw, gates, bias=gb, epilogue="sigmoid"), args.warmup, args.steps, flush)
        report(f"block_linear (gates of the recurrence, {nb} blocks of {C // nb}), {tag}", "gemm_tc", ms,
               n_tok * C * 2 + n_tok * 2 * C * 4 + gw.numel() * 2, 2.0 * n_tok * 2 * C * (C // nb))
        proj, taps, cb, lam = bf(n_tok, 2 * C), f32(K, C), f32(C), f32(C)
        state = torch.zeros(st.n_seqs, K, C, device=dev)
        uo = torch.empty(n_tok, C, dtype=torch.bfloat16, device=dev)
        ms = _timed(lambda: kernels.causal_conv(proj[:, C:], taps, cb, state, st, uo), args.warmup, args.steps, flush)
        report(f"causal_conv ({K} taps), {tag}", "rmsnorm", ms, n_tok * C * 4, 0)
        gates.uniform_(0.1, 0.9)
        so = torch.empty_like(uo)
        ms = _timed(lambda: kernels.gated_scan(uo, gates, C // nb, proj[:, :C], proj[:, C:], lam, 8.0, state, st, so),
                    args.warmup, args.steps, flush)
        report(f"gated_scan, {tag}", "rmsnorm", ms, n_tok * C * (2 + 8 + 2 + 2), 0)
        # the experts: routing, grouping, the two grouped products, the sum
        P = n_tok * top
        h, z = bf(n_tok, d), f32(n_tok, E) * 40
        ids = torch.empty(n_tok, top, dtype=torch.int32, device=dev)
        wts = torch.empty(n_tok, top, dtype=torch.float32, device=dev)
        corr = f32(E)
        ms = _timed(lambda: kernels.moe_route(z, corr, top, 4, 2, 2, ids, wts), args.warmup, args.steps, flush)
        report(f"moe_route ({E} experts), {tag}", "rmsnorm", ms, n_tok * (E * 4 + top * 8), 0)
        mt = kernels.moe_max_tiles(P, E)
        i32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
        offs, order, place, te, tr, nt = i32(E + 1), i32(P), i32(P), i32(mt), i32(mt), i32(1)
        grp = (offs, order, te, tr, nt)
        ms = _timed(lambda: kernels.moe_group(ids.view(-1), E, offs, order, place, te, tr, nt), args.warmup, args.steps, flush)
        report(f"moe_group, {tag}", "-", ms, P * 12, 0)
        wgu, wd = bf(E, 2 * ff, d), bf(E, d, ff)
        act = torch.empty(P, ff, dtype=torch.bfloat16, device=dev)
        yy = torch.empty(P, d, dtype=torch.float32, device=dev)
        used = min(E, P)
        gu_bytes, gu_flops = used * 2 * ff * d * 2 + P * d * 2 + P * ff * 2, 2.0 * P * 2 * ff * d
        dn_bytes, dn_flops = used * ff * d * 2 + P * ff * 2 + P * d * 4, 2.0 * P * ff * d
        if n_tok >= 128:
            import ctypes
            hrows = torch.empty(P, d, dtype=torch.bfloat16, device=dev)
            ms = _timed(lambda: kernels.moe_gather(h, order, top, hrows), args.warmup, args.steps, flush)
            report(f"moe_gather, {tag}", "rmsnorm", ms, P * d * 4, 0)
            host_offs = offs.cpu()
            hp = ctypes.c_void_p(host_offs.data_ptr())
            ms = _timed(lambda: kernels.gemm_tc_groups(hrows, wgu, act, hp, glu="silu"), args.warmup, args.steps, flush)
            report(f"gemm_tc per expert, gate/up ({ff} per expert, {E} launches), {tag}", "gemm_tc (gated)", ms, gu_bytes, gu_flops)
            ms = _timed(lambda: kernels.gemm_tc_groups(act, wd, yy, hp), args.warmup, args.steps, flush)
            report(f"gemm_tc per expert, down ({E} launches), {tag}", "gemm_tc", ms, dn_bytes, dn_flops)
        else:
            ms = _timed(lambda: kernels.moe_grouped(h, wgu, act, True, P, top, *grp, interleaved=True, skinny=True),
                        args.warmup, args.steps, flush)
            report(f"moe_grouped gate/up, streaming ({ff} per expert), {tag}", "gemm_tc (gated)", ms, gu_bytes, gu_flops)
            ms = _timed(lambda: kernels.moe_grouped(act, wd, yy, False, P, top, *grp, skinny=True), args.warmup, args.steps, flush)
            report(f"moe_grouped down, streaming, {tag}", "gemm_tc", ms, dn_bytes, dn_flops)
        ms = _timed(lambda: kernels.moe_combine(yy, wts, res, True), args.warmup, args.steps, flush)
        report(f"moe_combine, {tag}", "rmsnorm", ms, P * d * 4 + n_tok * d * 8, 0)
    out["kernels"] = rows
    out["wait_errors"] = wait_errors(kernels)
    print(json.dumps(out))
    return 0


def run_tikalix(args):
    """The Tikalix design beside the Llama shape of the same width and heads, with random weights: a prompt of
    ``--prompt-tokens`` and decode steps of ``--batch`` sequences at ``--context``, ``--layers`` layers of each
    (default 4), and every kernel the design adds or changes, alone, against its own roofline (the larger of bytes /
    measured copy bandwidth and FLOPs / measured bf16 peak), each beside the library's like kernel timed in the same
    run on operands of the same size."""
    import ctypes
    import torch
    from types import SimpleNamespace
    from ziglm_b200 import kernels
    from ziglm_b200.config.shapes import shape
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts.base import LayerIO
    torch.cuda.set_device(0)
    pk = peaks()
    size = "8b" if args.shape == "8b" else "1b"
    layers = args.layers or 4
    T, batch, context = args.prompt_tokens, args.batch, args.context
    max_seq = max(context, T) + 64
    gen = torch.Generator().manual_seed(7)
    out = {"case": "tikalix", "width_of": "llama-" + size, "dtype": "bf16", "layers": layers, "prompt_tokens": T,
           "batch": batch, "context": context, "data": "synthetic", "l2": "a 256 MiB buffer is rewritten before every timed call",
           "peaks": pk["source"], "models": {}}
    for name in ("tikalix-" + size, "llama-" + size):
        cfg = shape(name)
        if "layers" in cfg:
            cfg["layers"] = cfg["layers"][:layers]
            vocab = cfg["vocab"]
        else:
            cfg["num_hidden_layers"] = layers
            cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], max_seq)
            vocab = cfg["vocab_size"]
        eng = _engine_for(cfg, "bfloat16", batch, max_seq)
        ids = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        pre = _time_prompt(eng, ids(T), args.warmup, args.steps)
        dec = _time_decode_at(eng, batch, context, args.warmup, args.steps, ids)
        out["models"][name] = {"prefill_ms": round(pre, 3), "prefill_tok_s": round(T / pre * 1e3, 1),
                               "decode_ms": round(dec, 4), "decode_tok_s": round(batch / dec * 1e3, 1)}
        del eng
        torch.cuda.empty_cache()
    # ---- the kernels, alone
    cfg = shape("tikalix-" + size)
    d = cfg["width"]
    mix, moe = cfg["layers"][0]["mixer"], cfg["layers"][1]["mlp"]
    ff = cfg["layers"][0]["mlp"]["ff"]
    H, G, hd, cap, scale = mix["heads"], mix["kv_heads"], mix["dim"], mix["softcap"], mix["scale"]
    E, top, eff, limit = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"], moe["expert"]["limit"]
    dev = torch.device("cuda:0")
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    bf = lambda *sh: (torch.randn(*sh, device=dev) * 0.05).to(torch.bfloat16)
    f32 = lambda *sh: torch.randn(*sh, device=dev) * 0.05
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = []

    def report(what, like, ms, nbytes, flops):
        floor = max(nbytes / hbm, flops / peak) * 1e3
        rows.append({"kernel": what, "like": like, "ms": round(ms, 4), "roofline_ms": round(floor, 4),
                     "frac_of_roofline": round(floor / ms, 4)})

    def timed(fn):
        return _timed(fn, args.warmup, args.steps, flush)

    kernels.require(("elementwise", "attention", "attention_tc", "attention_fmha", "moe", "gemm_generic", "gemm_tc"))
    page = 64
    inv_freq = torch.rand(hd // 2, device=dev)
    for n_tok, tag in ((T, f"prompt of {T}"), (batch, f"decode batch {batch}")):
        decode = n_tok != T
        past = context - 1 if decode else 0
        n_seq = n_tok if decode else 1
        per_seq = -(-(past + (1 if decode else T)) // page)
        k_pages, v_pages = bf(n_seq * per_seq, G, page, hd), bf(n_seq * per_seq, G, page, hd)
        table = torch.arange(n_seq * per_seq, dtype=torch.int32, device=dev).view(n_seq, per_seq)
        new = [1] * n_seq if decode else [T]
        cu = [0]
        for n in new:
            cu.append(cu[-1] + n)
        step = SimpleNamespace(
            n_tokens=n_tok, n_seqs=n_seq, single_token=decode, max_new=max(new), max_total=past + max(new),
            positions=i32([past + i for n in new for i in range(n)]), seq_of_token=i32([b for b, n in enumerate(new) for _ in range(n)]),
            cu_seqlens=i32(cu), past_lens=i32([past] * n_seq), total_lens=i32([past + n for n in new]), ws=Workspace(dev))
        io = LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table, page_size=page)
        # rotation + unit norm + cache write, beside the library's rotation + cache write
        proj = bf(n_tok, (2 * H + 2 * G) * hd)
        qkv = bf(n_tok, (H + 2 * G) * hd)
        rope_bytes = n_tok * (H + G) * hd * 4 + n_tok * G * hd * 2 * 3
        ms = timed(lambda: kernels.rope_store(qkv, H, G, hd, hd, inv_freq, step.positions, step.seq_of_token, table, k_pages,
                                              v_pages, page))
        report(f"rope_store (rotation + cache write), {tag}", "-", ms, rope_bytes, 0)
        ms = timed(lambda: kernels.rope_norm_store(proj, H, G, hd, hd, inv_freq, 1.1, hd, 1e-6, step.positions,
                                                   step.seq_of_token, table, k_pages, v_pages, page))
        report(f"rope_norm_store (rotation + unit norm + cache write), {tag}", "rope_store", ms, rope_bytes, 0)
        # attention with and without the soft cap
        att_out = torch.empty(n_tok, H * hd, dtype=torch.bfloat16, device=dev)
        if decode:
            att_bytes, att_flops = n_seq * (past + 1) * G * hd * 2 * 2 + n_tok * H * hd * 4, 4.0 * n_tok * H * hd * (past + 1)
        else:
            att_bytes, att_flops = n_tok * (H + 2 * G) * hd * 2 + n_tok * H * hd * 2, 2.0 * H * hd * T * T
        ms = timed(lambda: kernels.attention(step, qkv, att_out, H, G, hd, scale, None, io))
        report(f"attention, {tag}", "-", ms, att_bytes, att_flops)
        ms = timed(lambda: kernels.attention(step, proj, att_out, H, G, hd, scale, None, io, softcap=cap))
        report(f"attention with a soft cap of {cap}, {tag}", "attention", ms, att_bytes, att_flops)
        ms = timed(lambda: kernels.sigmoid_mul(att_out, proj[:, (H + 2 * G) * hd:], att_out))
        report(f"sigmoid_mul (output gate), {tag}", "rmsnorm", ms, n_tok * H * hd * 6, 0)
        # norms
        xr, wn, yn = f32(n_tok, d), bf(d), torch.empty(n_tok, d, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: kernels.rmsnorm(xr, wn, yn, 1e-6))
        report(f"rmsnorm, {tag}", "-", ms, n_tok * d * 6 + d * 2, 0)
        res = f32(n_tok, d)
        ms = timed(lambda: kernels.norm_add_scaled(xr, wn, 1e-6, 0.5, res, yn, weight_offset=1.0))
        report(f"norm_add_scaled (norm behind a sublayer + residual sum + next rows), {tag}", "rmsnorm", ms,
               n_tok * d * 14 + d * 2, 0)
        # the dense feed-forward's first product with its activation, beside the gated product of as many rows
        x, wu, act = bf(n_tok, d), bf(ff, d), torch.empty(n_tok, ff, dtype=torch.bfloat16, device=dev)
        wg, actg = bf(ff, d), torch.empty(n_tok, ff // 2, dtype=torch.bfloat16, device=dev)
        up_bytes, up_flops = n_tok * d * 2 + ff * d * 2 + n_tok * ff * 2, 2.0 * n_tok * d * ff
        ms = timed(lambda: kernels.gemm_tc(x, wg, actg, glu="silu"))
        report(f"gemm_tc gated silu ({ff} rows of weights), {tag}", "-", ms, up_bytes - n_tok * ff, up_flops)
        ms = timed(lambda: kernels.gemm_tc_unary(x, wu, act, "relu2"))
        report(f"gemm_tc_unary squared relu ({ff} rows of weights), {tag}", "gemm_tc gated silu", ms, up_bytes, up_flops)
        # the experts
        P = n_tok * top
        h, z = bf(n_tok, d), f32(n_tok, E) * 40
        ids_t = torch.empty(n_tok, top, dtype=torch.int32, device=dev)
        wts = torch.empty(n_tok, top, dtype=torch.float32, device=dev)
        ms = timed(lambda: kernels.moe_route(z, None, top, 1, 1, 2, ids_t, wts, softmax_scores=1, renormalize=True))
        report(f"moe_route softmax ({E} experts), {tag}", "-", ms, n_tok * (E * 4 + top * 8), 0)
        ms = timed(lambda: kernels.moe_route(z, None, top, 1, 1, 2, ids_t, wts, softmax_scores=2))
        report(f"moe_route softmax over the chosen ({E} experts), {tag}", "moe_route softmax", ms, n_tok * (E * 4 + top * 8), 0)
        mt = kernels.moe_max_tiles(P, E)
        e32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
        offs, order, place, te, tr, nt = e32(E + 1), e32(P), e32(P), e32(mt), e32(mt), e32(1)
        grp = (offs, order, te, tr, nt)
        kernels.moe_group(ids_t.view(-1), E, offs, order, place, te, tr, nt)
        wgu = bf(E, 2 * eff, d)
        eact = torch.empty(P, eff, dtype=torch.bfloat16, device=dev)
        used = min(E, P)
        gu_bytes, gu_flops = used * 2 * eff * d * 2 + P * d * 2 + P * eff * 2, 2.0 * P * 2 * eff * d
        if n_tok >= 128:
            hrows = torch.empty(P, d, dtype=torch.bfloat16, device=dev)
            kernels.moe_gather(h, order, top, hrows)
            host_offs = offs.cpu()
            hp = ctypes.c_void_p(host_offs.data_ptr())
            ms = timed(lambda: kernels.gemm_tc_groups(hrows, wgu, eact, hp, glu="silu"))
            report(f"gemm_tc per expert, gate/up silu ({eff} per expert), {tag}", "-", ms, gu_bytes, gu_flops)
            ms = timed(lambda: kernels.gemm_tc_groups(hrows, wgu, eact, hp, glu="silu", limit=limit, slope=1.702))
            report(f"gemm_tc per expert, gate/up clamped ({eff} per expert), {tag}", "gemm_tc per expert silu", ms, gu_bytes, gu_flops)
        else:
            ms = timed(lambda: kernels.moe_grouped(h, wgu, eact, True, P, top, *grp, interleaved=True, skinny=True))
            report(f"moe_grouped gate/up silu, streaming ({eff} per expert), {tag}", "-", ms, gu_bytes, gu_flops)
            ms = timed(lambda: kernels.moe_grouped(h, wgu, eact, True, P, top, *grp, interleaved=True, skinny=True,
                                                   limit=limit, slope=1.702))
            report(f"moe_grouped gate/up clamped, streaming ({eff} per expert), {tag}", "moe_grouped silu", ms, gu_bytes, gu_flops)
        del k_pages, v_pages
    out["kernels"] = rows
    out["wait_errors"] = wait_errors(kernels)
    print(json.dumps(out))
    return 0


def run_vilazen(args):
    """The Vilazen design beside the Llama shape of the same width and heads, with random weights: a prompt of
    ``--prompt-tokens`` and decode steps of ``--batch`` sequences at ``--context``, ``--layers`` layers of each
    (default 4: one of every kind and the value-mixing pair), and every kernel the design adds or changes, alone,
    against its own roofline (the larger of bytes / measured copy bandwidth and FLOPs / measured bf16 peak; float32
    FMA work against 2 x 128 lanes x 148 SMs x the clock), each beside the library's like kernel timed in the same run
    on operands of the same size."""
    import torch
    from types import SimpleNamespace
    from ziglm_b200 import kernels
    from ziglm_b200.config.shapes import shape
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts.base import LayerIO
    torch.cuda.set_device(0)
    pk = peaks()
    size = "8b" if args.shape == "8b" else "1b"
    layers = args.layers or 4
    T, batch, context = args.prompt_tokens, args.batch, args.context
    max_seq = max(context, T) + 64
    gen = torch.Generator().manual_seed(7)
    out = {"case": "vilazen", "width_of": "llama-" + size, "dtype": "bf16", "layers": layers, "prompt_tokens": T,
           "batch": batch, "context": context, "data": "synthetic", "l2": "a 256 MiB buffer is rewritten before every timed call",
           "peaks": pk["source"], "models": {}}
    for name in ("vilazen-" + size, "llama-" + size):
        cfg = shape(name)
        if "layers" in cfg:
            cfg["layers"] = cfg["layers"][:layers]
            vocab = cfg["vocab"]
        else:
            cfg["num_hidden_layers"] = layers
            cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], max_seq)
            vocab = cfg["vocab_size"]
        eng = _engine_for(cfg, "bfloat16", batch, max_seq)
        ids = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        pre = _time_prompt(eng, ids(T), args.warmup, args.steps)
        dec = _time_decode_at(eng, batch, context, args.warmup, args.steps, ids)
        out["models"][name] = {"prefill_ms": round(pre, 3), "prefill_tok_s": round(T / pre * 1e3, 1),
                               "decode_ms": round(dec, 4), "decode_tok_s": round(batch / dec * 1e3, 1)}
        del eng
        torch.cuda.empty_cache()
    # ---- the kernels, alone
    cfg = shape("vilazen-" + size)
    d = cfg["width"]
    par, att = cfg["layers"][0]["mixer"], cfg["layers"][1]["mixer"]
    lin = par["right"]
    ff = cfg["layers"][0]["mlp"]["ff"]
    H, G, hd, scale = att["heads"], att["kv_heads"], att["dim"], att["scale"]
    rot, window, keep = att["rot"]["dims"], att["mask"]["size"], att["mask"]["keep_first"]
    LH, LD, LV = lin["heads"], lin["dim"], lin["vdim"]
    dev = torch.device("cuda:0")
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    bf = lambda *sh: (torch.randn(*sh, device=dev) * 0.05).to(torch.bfloat16)
    f32 = lambda *sh: torch.randn(*sh, device=dev) * 0.05
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fma = 2.0 * 128 * 148 * 1.9e9
    rows = []

    def report(what, like, ms, nbytes, flops, fma_flops=0.0):
        floor = max(nbytes / hbm, flops / peak, fma_flops / fma) * 1e3
        rows.append({"kernel": what, "like": like, "ms": round(ms, 4), "roofline_ms": round(floor, 4),
                     "frac_of_roofline": round(floor / ms, 4)})

    def timed(fn):
        return _timed(fn, args.warmup, args.steps, flush)

    kernels.require(("elementwise", "attention", "attention_tc", "attention_fmha", "linear_attention", "gemm_generic", "gemm_tc"))
    page = 64
    inv_freq = torch.rand(rot // 2, device=dev)
    sinks = f32(H) * 20
    chunk = kernels.linear_attention_chunk()
    pows = torch.tensor([[a ** n for n in range(chunk + 1)] for a in lin["decay"]], dtype=torch.float64).float().to(dev)
    for n_tok, tag in ((T, f"prompt of {T}"), (batch, f"decode batch {batch}")):
        decode = n_tok != T
        past = context - 1 if decode else 0
        n_seq = n_tok if decode else 1
        per_seq = -(-(past + (1 if decode else T)) // page)
        k_pages, v_pages = bf(n_seq * per_seq, G, page, hd), bf(n_seq * per_seq, G, page, hd)
        table = torch.arange(n_seq * per_seq, dtype=torch.int32, device=dev).view(n_seq, per_seq)
        new = [1] * n_seq if decode else [T]
        cu = [0]
        for n in new:
            cu.append(cu[-1] + n)
        step = SimpleNamespace(
            n_tokens=n_tok, n_seqs=n_seq, single_token=decode, max_new=max(new), max_total=past + max(new),
            positions=i32([past + i for n in new for i in range(n)]), seq_of_token=i32([b for b, n in enumerate(new) for _ in range(n)]),
            cu_seqlens=i32(cu), past_lens=i32([past] * n_seq), total_lens=i32([past + n for n in new]),
            slots=i32(list(range(n_seq))), ws=Workspace(dev))
        io = LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table, page_size=page)
        # norm of the whole q and k + rotation + mixed values + cache write, beside the library's rotation + cache write
        gcols = -(-H // 8) * 8
        proj = bf(n_tok, (H + 2 * G) * hd + gcols)
        qkv = bf(n_tok, (H + 2 * G) * hd)
        wq, wk = f32(H * hd) + 1, f32(G * hd) + 1
        mixb = bf(n_tok, G * hd)
        rope_bytes = n_tok * (H + G) * hd * 4 + n_tok * G * hd * 2 * 3
        ms = timed(lambda: kernels.rope_store(qkv, H, G, hd, rot, inv_freq, step.positions, step.seq_of_token, table, k_pages,
                                              v_pages, page))
        report(f"rope_store (rotation + cache write), {tag}", "-", ms, rope_bytes, 0)
        ms = timed(lambda: kernels.qk_prep(proj, H, G, hd, rot, inv_freq, wq, wk, H * hd, G * hd, 1e-6, 2, 0.25, mixb, hd,
                                           step.positions, step.seq_of_token, table, k_pages, v_pages, page))
        report(f"qk_prep (norm of whole q and k + rotation + mixed values + cache write), {tag}", "rope_store", ms,
               rope_bytes + n_tok * G * hd * 2 + (H + G) * hd * 4, 0)
        # attention: a window, a window that keeps the first tokens; all keys, all keys with a number in the denominator
        att_out = torch.empty(n_tok, H * hd, dtype=torch.bfloat16, device=dev)
        for w, kf, sk, what, like in ((window, 0, None, f"attention, window {window}", "-"),
                                      (window, keep, None, f"attention, window {window} keeping the first {keep}", f"attention, window {window}"),
                                      (None, 0, None, "attention, every key", "-"),
                                      (None, 0, sinks, "attention, every key, with sinks", "attention, every key")):
            seen = lambda i: min(i + 1, (w + kf) if w else i + 1)
            if decode:
                keys = seen(past)
                att_bytes, att_flops = n_seq * keys * G * hd * 2 * 2 + n_tok * H * hd * 4, 4.0 * n_tok * H * hd * keys
            else:
                pairs = sum(seen(i) for i in range(T))
                att_bytes, att_flops = n_tok * (H + 2 * G) * hd * 2 + n_tok * H * hd * 2, 4.0 * H * hd * pairs
            ms = timed(lambda: kernels.attention(step, qkv, att_out, H, G, hd, scale, w, io, keep_first=kf, sinks=sk))
            report(f"{what}, {tag}", like, ms, att_bytes, att_flops)
        ms = timed(lambda: kernels.sigmoid_mul(att_out, qkv[:, :H * hd], att_out))
        report(f"sigmoid_mul (a gate an element), {tag}", "-", ms, n_tok * H * hd * 6, 0)
        ms = timed(lambda: kernels.gate_heads(att_out, proj[:, (H + 2 * G) * hd:(H + 2 * G) * hd + H], att_out, H, 1.2))
        report(f"gate_heads (a gate a head), {tag}", "sigmoid_mul", ms, n_tok * H * (hd * 4 + 2), 0)
        # linear attention with a decay, beside attention over every key with as many heads of that size
        lproj = bf(n_tok, LH * (2 * LD + 2 * LV))
        state = torch.zeros(n_seq, LH, LD, LV, device=dev)
        mixed = torch.empty(n_tok, LH * LV, device=dev)
        la_bytes = n_tok * LH * (2 * LD + LV) * 2 + n_tok * LH * LV * 4 + n_seq * LH * LD * LV * 8
        c = min(chunk, max(new))
        la_fma = 2.0 * n_tok * LH * (c * LD + c * LV + 2 * LD * LV)
        ms = timed(lambda: kernels.decayed_linear_attention(lproj, 0, LH * LD, 2 * LH * LD, LH, LD, LV, "silu", pows, state,
                                                            step, mixed))
        report(f"decayed_linear_attention ({LH} heads of {LD}), {tag}", "attention, every key", ms, la_bytes, 0, la_fma)
        xr, wn, yn = f32(n_tok, d), bf(d), torch.empty(n_tok, d, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: kernels.rmsnorm(xr, wn, yn, 1e-6))
        report(f"rmsnorm, {tag}", "-", ms, n_tok * d * 6 + d * 2, 0)
        lout = torch.empty(n_tok, LH * LV, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: kernels.norm_gate(mixed, wq[:LH * LV].contiguous(), lproj[:, LH * (2 * LD + LV):], lout, 1e-6, 1.1))
        report(f"norm_gate (norm of the heads + gate), {tag}", "rmsnorm", ms, n_tok * LH * LV * 8 + LH * LV * 4, 0)
        # the feed-forward's first product with the exact gelu, beside the gated product of as many rows
        x, wu, act = bf(n_tok, d), bf(ff, d), torch.empty(n_tok, ff, dtype=torch.bfloat16, device=dev)
        wg, actg = bf(ff, d), torch.empty(n_tok, ff // 2, dtype=torch.bfloat16, device=dev)
        up_bytes, up_flops = n_tok * d * 2 + ff * d * 2 + n_tok * ff * 2, 2.0 * n_tok * d * ff
        ms = timed(lambda: kernels.gemm_tc(x, wg, actg, glu="silu"))
        report(f"gemm_tc gated silu ({ff} rows of weights), {tag}", "-", ms, up_bytes - n_tok * ff, up_flops)
        ms = timed(lambda: kernels.gemm_tc_unary(x, wu, act, "gelu"))
        report(f"gemm_tc_unary exact gelu ({ff} rows of weights), {tag}", "gemm_tc gated silu", ms, up_bytes, up_flops)
        del k_pages, v_pages
    out["kernels"] = rows
    out["wait_errors"] = wait_errors(kernels)
    print(json.dumps(out))
    return 0


def run_lipadra(args):
    """The Lipadra design beside the Tumatar design (the library's closest: a recurrence behind a short convolution and
    grouped experts) and the Llama shape, all of the same width and with random weights: a prompt of ``--prompt-tokens``
    and decode steps of ``--batch`` sequences at ``--context``, ``--layers`` layer runs of each (default 4: retention,
    scan, chunked attention, and the first once more), and every kernel the design adds or changes, alone, against its
    own roofline (the larger of bytes / measured copy bandwidth and FLOPs / measured bf16 peak; float32 FMA work
    against 2 x 128 lanes x 148 SMs x the clock), each beside the library's like kernel timed in the same run on
    operands of the same size."""
    import torch
    from types import SimpleNamespace
    from ziglm_b200 import kernels
    from ziglm_b200.config.shapes import shape
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts.base import LayerIO
    torch.cuda.set_device(0)
    pk = peaks()
    size = "8b" if args.shape == "8b" else "1b"
    layers = args.layers or 4
    T, batch, context = args.prompt_tokens, args.batch, args.context
    max_seq = max(context, T) + 64
    gen = torch.Generator().manual_seed(7)
    out = {"case": "lipadra", "width_of": "llama-" + size, "dtype": "bf16", "layer_runs": layers, "prompt_tokens": T,
           "batch": batch, "context": context, "data": "synthetic", "l2": "a 256 MiB buffer is rewritten before every timed call",
           "peaks": pk["source"], "models": {}}
    for name in ("lipadra-" + size, "tumatar-" + size, "llama-" + size):
        cfg = shape(name)
        if "layers" in cfg:
            cfg["layers"] = cfg["layers"][:layers]
            vocab = cfg["vocab"]
        else:
            cfg["num_hidden_layers"] = layers
            cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], max_seq)
            vocab = cfg["vocab_size"]
        eng = _engine_for(cfg, "bfloat16", batch, max_seq)
        ids = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        pre = _time_prompt(eng, ids(T), args.warmup, args.steps)
        dec = _time_decode_at(eng, batch, context, args.warmup, args.steps, ids)
        out["models"][name] = {"prefill_ms": round(pre, 3), "prefill_tok_s": round(T / pre * 1e3, 1),
                               "decode_ms": round(dec, 4), "decode_tok_s": round(batch / dec * 1e3, 1)}
        del eng
        torch.cuda.empty_cache()
    # ---- the kernels, alone
    cfg = shape("lipadra-" + size)
    d = cfg["width"]
    ret, scan, att = (cfg["layers"][i]["mixer"] for i in range(3))
    router = cfg["layers"][0]["mlp"]["router"]
    H, G, hd, scale = att["heads"], att["kv_heads"], att["dim"], att["scale"]
    rot, chunk_size = att["rot"]["dims"], att["mask"]["size"]
    LH, LD, LV, lrot = ret["heads"], ret["dim"], ret["vdim"], ret["rot"]["dims"]
    C, N, K, rank = scan["inner"], scan["state"], scan["conv"], scan["dt_rank"]
    E, ident, top = router["experts"], router["identity"], router["top"]
    dev = torch.device("cuda:0")
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    bf = lambda *sh: (torch.randn(*sh, device=dev) * 0.05).to(torch.bfloat16)
    f32 = lambda *sh: torch.randn(*sh, device=dev) * 0.05
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    hbm, peak = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fma = 2.0 * 128 * 148 * 1.9e9
    rows = []

    def report(what, like, ms, nbytes, flops, fma_flops=0.0):
        floor = max(nbytes / hbm, flops / peak, fma_flops / fma) * 1e3
        rows.append({"kernel": what, "like": like, "ms": round(ms, 4), "roofline_ms": round(floor, 4),
                     "frac_of_roofline": round(floor / ms, 4)})

    def timed(fn):
        return _timed(fn, args.warmup, args.steps, flush)

    kernels.require(("elementwise", "attention", "attention_tc", "attention_fmha", "linear_attention", "recurrent", "moe"))
    page = 64
    inv_freq, linv = torch.rand(rot // 2, device=dev), torch.rand(lrot // 2, device=dev)
    la_chunk = kernels.linear_attention_chunk()
    pows = torch.tensor([[a ** n for n in range(la_chunk + 1)] for a in ret["decay"]], dtype=torch.float64).float().to(dev)
    for n_tok, tag in ((T, f"prompt of {T}"), (batch, f"decode batch {batch}")):
        decode = n_tok != T
        past = context - 1 if decode else 0
        n_seq = n_tok if decode else 1
        per_seq = -(-(past + (1 if decode else T)) // page)
        k_pages, v_pages = bf(n_seq * per_seq, G, page, hd), bf(n_seq * per_seq, G, page, hd)
        table = torch.arange(n_seq * per_seq, dtype=torch.int32, device=dev).view(n_seq, per_seq)
        new = [1] * n_seq if decode else [T]
        cu = [0]
        for n in new:
            cu.append(cu[-1] + n)
        step = SimpleNamespace(
            n_tokens=n_tok, n_seqs=n_seq, single_token=decode, max_new=max(new), max_total=past + max(new),
            positions=i32([past + i for n in new for i in range(n)]), seq_of_token=i32([b for b, n in enumerate(new) for _ in range(n)]),
            cu_seqlens=i32(cu), past_lens=i32([past] * n_seq), total_lens=i32([past + n for n in new]),
            slots=i32(list(range(n_seq))), ws=Workspace(dev))
        io = LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table, page_size=page)
        # the norm behind a sum, beside the norm that adds (the post-norm arrangement's) and the plain norm
        x, br, w_n = f32(n_tok, d), f32(n_tok, d), bf(d)
        hrow = torch.empty(n_tok, d, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: kernels.rmsnorm(x, w_n, hrow, 1e-6))
        report(f"rmsnorm, {tag}", "-", ms, n_tok * d * 6 + d * 2, 0)
        ms = timed(lambda: kernels.norm_add_scaled(br, w_n, 1e-6, 0.5, x, hrow))
        report(f"norm_add_scaled (x += m norm(branch), and the next rows), {tag}", "rmsnorm", ms, n_tok * d * 18 + d * 2, 0)
        ms = timed(lambda: kernels.sum_norm(br, w_n, 1e-6, 2.0, x, hrow))
        report(f"sum_norm (x = norm(alpha x + branch), and the next rows), {tag}", "norm_add_scaled", ms, n_tok * d * 18 + d * 2, 0)
        # the weighted norm of every head before the rotation, beside the unit norm behind it
        qkv = bf(n_tok, (H + 2 * G) * hd)
        wq, wk = f32(hd) + 1, f32(hd) + 1
        rope_bytes = n_tok * (H + G) * hd * 4 + n_tok * G * hd * 2 * 3
        ms = timed(lambda: kernels.rope_norm_store(qkv, H, G, hd, rot, inv_freq, 1.0, hd, 1e-6, step.positions, step.seq_of_token,
                                                   table, k_pages, v_pages, page))
        report(f"rope_norm_store (rotation + unit norm + cache write), {tag}", "-", ms, rope_bytes, 0)
        ms = timed(lambda: kernels.rope_norm_store(qkv, H, G, hd, rot, inv_freq, 1.0, hd, 1e-6, step.positions, step.seq_of_token,
                                                   table, k_pages, v_pages, page, norm_first=True, q_weight=wq, k_weight=wk))
        report(f"rope_norm_store (weighted norm + rotation + cache write), {tag}", "rope_norm_store", ms, rope_bytes, 0)
        # attention within chunks with one more 1 in the denominator, beside a window of the same size with sinks
        att_out = torch.empty(n_tok, H * hd, dtype=torch.bfloat16, device=dev)
        zero = torch.zeros(H, device=dev)
        for w, ck, what, like in ((chunk_size, None, f"attention, window {chunk_size}, with sinks", "-"),
                                  (None, chunk_size, f"attention, chunks of {chunk_size}, one more 1", f"attention, window {chunk_size}")):
            seen = (lambda i: min(i + 1, w)) if w else (lambda i: i % ck + 1)
            if decode:
                keys = seen(past)
                att_bytes, att_flops = n_seq * keys * G * hd * 2 * 2 + n_tok * H * hd * 4, 4.0 * n_tok * H * hd * keys
            else:
                pairs = sum(seen(i) for i in range(T))
                att_bytes, att_flops = n_tok * (H + 2 * G) * hd * 2 + n_tok * H * hd * 2, 4.0 * H * hd * pairs
            ms = timed(lambda: kernels.attention(step, qkv, att_out, H, G, hd, scale, w, io, sinks=zero, chunk=ck))
            report(f"{what}, {tag}", like, ms, att_bytes, att_flops)
        # retention: the recurrence with rotated q and k and a factor on k, the norm of every head with a gate; beside the
        # recurrence without them and the norm of the heads together
        lproj = bf(n_tok, LH * (2 * LD + 2 * LV))
        state = torch.zeros(n_seq, LH, LD, LV, device=dev)
        mixed = torch.empty(n_tok, LH * LV, device=dev)
        la_bytes = n_tok * LH * (2 * LD + LV) * 2 + n_tok * LH * LV * 4 + n_seq * LH * LD * LV * 8
        c = min(la_chunk, max(new))
        la_fma = 2.0 * n_tok * LH * (c * LD + c * LV + 2 * LD * LV)
        ms = timed(lambda: kernels.decayed_linear_attention(lproj, 0, LH * LD, 2 * LH * LD, LH, LD, LV, None, pows, state,
                                                            step, mixed))
        report(f"decayed_linear_attention ({LH} heads of {LD}), {tag}", "-", ms, la_bytes, 0, la_fma)
        ms = timed(lambda: kernels.decayed_linear_attention(lproj, 0, LH * LD, 2 * LH * LD, LH, LD, LV, None, pows, state,
                                                            step, mixed, rotary_dim=lrot, inv_freq=linv, key_scale=LD ** -0.5))
        report(f"decayed_linear_attention with rotated q and k and a factor on k ({LH} heads of {LD}), {tag}",
               "decayed_linear_attention", ms, la_bytes, 0, la_fma)
        lout = torch.empty(n_tok, LH * LV, dtype=torch.bfloat16, device=dev)
        wl = f32(LH * LV) + 1
        ms = timed(lambda: kernels.norm_gate(mixed, wl, lproj[:, LH * (2 * LD + LV):], lout, 1e-6, 1.0))
        report(f"norm_gate (norm of the heads together + sigmoid gate), {tag}", "-", ms, n_tok * LH * LV * 8 + LH * LV * 4, 0)
        ms = timed(lambda: kernels.head_norm_gate(mixed, None, lproj[:, LH * (2 * LD + LV):], lout, LH, 1e-6, "silu", 1.0))
        report(f"head_norm_gate (norm of every head + silu gate), {tag}", "norm_gate", ms, n_tok * LH * LV * 8, 0)
        # the scan: the convolution with silu, the selective scan; beside the convolution and the gated scan of a diagonal recurrence
        proj = bf(n_tok, 2 * C)
        u = torch.empty(n_tok, C, dtype=torch.bfloat16, device=dev)
        taps, cbias = f32(K, C), f32(C)
        st_rec = torch.zeros(n_seq, K, C, device=dev)
        st_scan = torch.zeros(n_seq, K - 1 + N, C, device=dev)
        ms = timed(lambda: kernels.causal_conv(proj[:, C:], taps, cbias, st_rec, step, u))
        report(f"causal_conv ({C} channels), {tag}", "-", ms, n_tok * C * 4, 0)
        ms = timed(lambda: kernels.causal_conv(proj[:, :C], taps, cbias, st_scan, step, u, activation="silu"))
        report(f"causal_conv with silu ({C} channels), {tag}", "causal_conv", ms, n_tok * C * 4, 0)
        gates = torch.rand(n_tok, 2 * C, device=dev)
        lam = f32(C)
        sout = torch.empty(n_tok, C, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: kernels.gated_scan(u, gates, 128, proj[:, :C], proj[:, C:], lam, 8.0, st_rec, step, sout))
        report(f"gated_scan (one state a channel, {C} channels), {tag}", "-", ms, n_tok * C * (2 + 8 + 2 + 2) + n_seq * K * C * 8, 0,
               2.0 * n_tok * C * 8)
        dbc = bf(n_tok, rank + 2 * N)
        dtp = f32(n_tok, C)
        a_t, dvec = -torch.rand(N, C, device=dev) - 0.1, f32(C)
        passes = 1 if max(new) < 32 else 2
        ms = timed(lambda: kernels.selective_scan(u, dtp, dbc, rank, rank + N, N, proj[:, C:], proj[:, :C], a_t, dvec, K,
                                                  st_scan, step, sout))
        report(f"selective_scan ({N} states a channel, {C} channels), {tag}", "gated_scan", ms,
               n_tok * C * (2 + 4 + 2 + 2) + n_seq * (K - 1 + N) * C * 8, 0, passes * n_tok * C * N * 12.0)
        # routing over experts and identity experts with a softmax, and the sum over a token's pairs with identity
        # experts and a gated shared expert; beside routing with sigmoid scores and the plain sum
        routed = E + ident
        z = f32(n_tok, routed + 1) * 40
        corr = f32(routed)
        ids = torch.empty(n_tok, top, dtype=torch.int32, device=dev)
        wts = torch.empty(n_tok, top, device=dev)
        ms = timed(lambda: kernels.moe_route(z[:, :routed].contiguous(), corr, top, 6, 3, 2, ids, wts))
        report(f"moe_route, sigmoid scores ({routed} outputs), {tag}", "-", ms, n_tok * (routed * 4 + top * 8), 0)
        ms = timed(lambda: kernels.moe_route(z, corr, top, 6, 3, 1, ids, wts, softmax_scores=1, weight_scale=2.0, n_extra=1))
        report(f"moe_route, softmax scores, identity experts, a factor ({routed} outputs), {tag}", "moe_route, sigmoid scores", ms,
               n_tok * (routed * 4 + top * 8), 0)
        y, shared_y = f32(n_tok * top, d), f32(n_tok, d)
        res = f32(n_tok, d)
        hb = bf(n_tok, d)
        ms = timed(lambda: kernels.moe_combine(y, wts, res, False))
        report(f"moe_combine, {tag}", "-", ms, n_tok * top * d * 4 + n_tok * d * 4, 0)
        ms = timed(lambda: kernels.moe_combine(y, wts, res, False, ids=ids, n_real=E, h=hb, shared=shared_y, gate=z[:, routed:]))
        report(f"moe_combine with identity experts and a gated shared expert, {tag}", "moe_combine", ms,
               n_tok * top * d * 4 + n_tok * d * 10, 0)
        del k_pages, v_pages
    out["kernels"] = rows
    out["wait_errors"] = wait_errors(kernels)
    print(json.dumps(out))
    return 0


def run_workload(args):
    """The two workloads beside the headline one, through ``Engine.generate`` (host token ids in, ids out):

    workload-1b   Llama-3.2-1B shape (tied head): 64 prompts with seeded lengths in [16, 1024] in one step of
                  unequal lengths, then 128 decode steps;
    workload-13b  Llama-2-13B shape (every head its own keys): 8 prompts of 2,048 tokens, then 256 decode steps.

    Times are the loop's own wall-clock times (they include the copies and the read-back of every step); the
    roofline fractions divide the bytes every decode step has to read (weights once, the live sequences' cache
    at its length in that step) and the prompt step's FLOPs by those times and the measured peaks."""
    import random
    import torch
    from ziglm_b200 import GenerationOptions, SamplerParams, kernels
    torch.cuda.set_device(0)
    which = "1b" if args.case == "workload-1b" else "13b"
    cfg = dict(SHAPES[which])
    full_layers = cfg["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg["num_hidden_layers"] = n_layers
    if which == "1b":
        rng = random.Random(1)
        lens = [rng.randint(16, 1024) for _ in range(64)]
        new = 128
    else:
        lens = [2048] * 8
        new = 256
    B = len(lens)
    max_seq = max(lens) + new + 64
    tokens_needed = sum(-(-(l + new + 1) // 64) * 64 for l in lens)
    eng = _engine_for(cfg, "bfloat16", B, max_seq, tokens=tokens_needed + 64 * B, seed=5)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab_size"], (l,), generator=g).tolist() for l in lens]
    # the first token comes from the prompt step, the other `new` from decode steps
    opts = GenerationOptions(max_tokens=new + 1, sampler=SamplerParams(greedy=True), ignore_eos=True)
    pk = peaks()
    runs = []
    with ClockSampler() as clocks:
        for rep in range(1 + max(1, args.repeats)):
            torch.cuda.synchronize()
            results, stats = eng.generate(prompts, opts)
            torch.cuda.synchronize()
            if rep:
                runs.append(stats)
    stats = sorted(runs, key=lambda st: st.generation_time_ms)[len(runs) // 2]
    assert all(len(r.tokens) == new + 1 for r in results)
    flops = sum(prefill_flops(cfg, n_layers, l) for l in lens)
    step_bytes = [decode_bytes(cfg, n_layers, B, 0, cached_tokens=sum(lens) + B * (k + 1)) for k in range(new)]
    ms_step = stats.generation_time_ms / new
    out = {
        "case": args.case, "model": {"1b": "Llama-3.2-1B shape", "13b": "Llama-2-13B shape"}[which], "dtype": "bf16",
        "layers": n_layers, "layers_of_config": full_layers, "batch": B, "prompt_tokens": sum(lens),
        "prompt_lengths": [min(lens), max(lens)], "decode_steps": new,
        "prefill_ms": round(stats.prefill_time_ms, 2), "prefill_tok_s": round(stats.prefill_tokens_per_sec(), 1),
        "prefill_tflop": round(flops / 1e12, 2),
        "prefill_frac_of_bf16_peak": round(flops / (stats.prefill_time_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
        "ms_per_step": round(ms_step, 4), "decode_tok_s": round(B * new / stats.generation_time_ms * 1000.0, 1),
        "decode_gb_per_step": [round(step_bytes[0] / 1e9, 3), round(step_bytes[-1] / 1e9, 3)],
        "decode_hbm_frac": round(sum(step_bytes) / (stats.generation_time_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
        "peaks": pk["source"], "clocks": clocks.summary(), "wait_errors": wait_errors(kernels),
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids; through Engine.generate, wall clock",
    }
    print(json.dumps(out))
    return 0


def run_float32(args):
    """The 8B shape in true 32-bit (CUDA-core products and attention, float32 weights, activations and cache):
    a prompt of 2,048 tokens and decode steps at batch 1 and 8, context 4,096."""
    import torch
    from ziglm_b200 import kernels
    torch.cuda.set_device(0)
    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg["num_hidden_layers"] = n_layers
    max_seq = CONTEXT + 64
    eng = _engine_for(cfg, "float32", 8, max_seq)
    gen = torch.Generator().manual_seed(7)
    ids = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()
    pk = peaks()
    steps, warmup = max(3, min(args.steps, 10)), 3
    pre_ms = _time_prompt(eng, ids(PREFILL_TOKENS), 1, 3)
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    out = {"case": "float32", "model": "Llama-3.1-8B shape", "dtype": "float32 (no tensor cores, no reduced-precision mode)",
           "layers": n_layers, "layers_of_config": full_layers, "context": CONTEXT,
           "prefill": {"tokens": PREFILL_TOKENS, "ms": round(pre_ms, 2), "tok_s": round(PREFILL_TOKENS / pre_ms * 1000.0, 1),
                       "tflops": round(flops / pre_ms / 1e9, 2)}}
    for batch in (1, 8):
        ms = _time_decode_at(eng, batch, CONTEXT, warmup, steps, ids)
        nbytes = decode_bytes(cfg, n_layers, batch, CONTEXT, 4)
        out[f"decode_b{batch}"] = {"ms": round(ms, 3), "tok_s": round(batch / ms * 1000.0, 1),
                                   "gb_per_step": round(nbytes / 1e9, 2),
                                   "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
    out["peaks"] = pk["source"]
    out["wait_errors"] = wait_errors(kernels)
    print(json.dumps(out))
    return 0


REFERENCE_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "libziglm_cuda.so")


def run_reference_kernels(args):
    """The reference's own CUDA kernels (its src/cuda_bridge.cu, unmodified, compiled for sm_100a into
    baseline/_ref/libziglm_cuda.so), timed at the shapes of this benchmark and put together in the order its
    decode step calls them for one Llama layer (src/model.zig:600-760): one sequence, float32 activations and
    cache, bf16 weights.  This is not the reference arm (its engine is a Zig program): it says what the
    reference's kernels alone would give on this GPU."""
    import ctypes
    from ctypes import c_float, c_int, c_void_p
    import torch
    if not os.path.isfile(REFERENCE_LIB):
        print(json.dumps({"case": "reference-kernels", "unavailable":
                          "baseline/_ref/libziglm_cuda.so is not there (build it from the reference's "
                          "src/cuda_bridge.cu with nvcc -shared -gencode arch=compute_100a,code=sm_100a)"}))
        return 0
    lib = ctypes.CDLL(REFERENCE_LIB)
    P = c_void_p
    protos = {
        "cuda_gemv_bf16": [P, P, P, c_int, c_int, P],
        "cuda_rmsnorm": [P, P, P, c_int, c_float, c_int, P],
        "cuda_rope": [P, P, c_int, c_int, c_int, c_int, c_int, c_float, P],
        "cuda_kv_cache_put": [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, P],
        "cuda_attention_forward": [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, P],
        "cuda_swiglu": [P, P, P, c_int, P],
        "cuda_add": [P, P, c_int, P],
    }
    for name, argtypes in protos.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, None
    torch.cuda.set_device(0)
    dev = "cuda:0"
    c = LLAMA_8B
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    ctx = args.context
    stream = torch.cuda.current_stream().cuda_stream
    bf = lambda r, k: (torch.randn(r, k, device=dev) * 0.02).to(torch.bfloat16)
    f32 = lambda n: torch.randn(n, device=dev)
    w = {"q": bf(nh * hd, H), "k": bf(nkv * hd, H), "v": bf(nkv * hd, H), "o": bf(H, nh * hd), "gate": bf(I, H),
         "up": bf(I, H), "down": bf(H, I), "head": bf(V, H)}
    g1, g2 = torch.ones(H, device=dev), torch.ones(H, device=dev)
    x, h, q, k, v, att, o = f32(H), f32(H), f32(nh * hd), f32(nkv * hd), f32(nkv * hd), f32(nh * hd), f32(H)
    gate, up, act, down, logits = f32(I), f32(I), f32(I), f32(H), f32(V)
    kc = torch.randn(ctx, nkv * hd, device=dev)
    vc = torch.randn(ctx, nkv * hd, device=dev)
    pos, eps, scale = ctx - 1, c["rms_norm_eps"], 1.0 / hd ** 0.5
    p = lambda t: t.data_ptr()
    steps = {
        "rmsnorm": lambda: lib.cuda_rmsnorm(p(x), p(g1), p(h), H, eps, 0, stream),
        "gemv_q": lambda: lib.cuda_gemv_bf16(p(w["q"]), p(h), p(q), nh * hd, H, stream),
        "gemv_k": lambda: lib.cuda_gemv_bf16(p(w["k"]), p(h), p(k), nkv * hd, H, stream),
        "gemv_v": lambda: lib.cuda_gemv_bf16(p(w["v"]), p(h), p(v), nkv * hd, H, stream),
        "rope": lambda: lib.cuda_rope(p(q), p(k), pos, nh, nkv, hd, hd, c["rope_theta"], stream),
        "kv_put": lambda: lib.cuda_kv_cache_put(p(kc), p(vc), p(k), p(v), 0, pos, ctx, nkv, hd, nkv * hd, stream),
        "attention": lambda: lib.cuda_attention_forward(p(q), p(kc), p(vc), p(att), 0, pos, ctx, nh, nkv, hd, nkv * hd,
                                                        scale, 0.0, 0, stream),
        "gemv_o": lambda: lib.cuda_gemv_bf16(p(w["o"]), p(att), p(o), H, nh * hd, stream),
        "add_1": lambda: lib.cuda_add(p(x), p(o), H, stream),
        "rmsnorm_2": lambda: lib.cuda_rmsnorm(p(x), p(g2), p(h), H, eps, 0, stream),
        "gemv_gate": lambda: lib.cuda_gemv_bf16(p(w["gate"]), p(h), p(gate), I, H, stream),
        "gemv_up": lambda: lib.cuda_gemv_bf16(p(w["up"]), p(h), p(up), I, H, stream),
        "swiglu": lambda: lib.cuda_swiglu(p(gate), p(up), p(act), I, stream),
        "gemv_down": lambda: lib.cuda_gemv_bf16(p(w["down"]), p(act), p(down), H, I, stream),
        "add_2": lambda: lib.cuda_add(p(x), p(down), H, stream),
    }
    # The reference's cuda_argmax is left out: it hands its kernels the host-side names of two __device__
    # arrays as pointers (src/cuda_bridge.cu:2943-2944, 3075-3076), which is an illegal memory access on
    # this GPU; it ran here once and is not run again.
    tail = {
        "gemv_head": lambda: lib.cuda_gemv_bf16(p(w["head"]), p(h), p(logits), V, H, stream),
    }
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)       # larger than L2

    def timed(fn, reps):
        ts = []
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1000.0)
        return sorted(ts)[len(ts) // 2]

    for name, fn in {**steps, **tail}.items():        # one by one first: a failing launch is named
        fn()
        try:
            torch.cuda.synchronize()
        except RuntimeError as e:
            print(json.dumps({"case": "reference-kernels", "unavailable": "%s failed: %s" % (name, str(e).splitlines()[0])}))
            return 0
    each = {name: round(timed(fn, 7), 1) for name, fn in {**steps, **tail}.items()}

    def layer():
        for fn in steps.values():
            fn()
    layer_us = timed(layer, 7)
    tail_us = each["rmsnorm"] + each["gemv_head"]
    token_ms = (layer_us * c["num_hidden_layers"] + tail_us) / 1000.0
    print(json.dumps({"case": "reference-kernels", "what": "simonproyt/ziglm src/cuda_bridge.cu compiled for sm_100a, one "
                      "sequence, context %d, Llama-3.1-8B layer shapes; L2 flushed before every timing; without its argmax "
                      "(faults here)" % ctx,
                      "kernel_us": each, "layer_us": round(layer_us, 1),
                      "decode_b1_ms_per_token": round(token_ms, 3), "decode_b1_tok_s": round(1000.0 / token_ms, 1)}))
    return 0


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--case", default="full",
                    choices=["full", "prefill", "decode", "workload-1b", "workload-13b", "float32", "reference-kernels",
                             "tumatar", "tikalix", "vilazen", "lipadra"],
                    help="full: the whole measurement; prefill / decode: that phase alone (for profilers and sweeps); "
                         "workload-1b / workload-13b: the two other workloads through Engine.generate; float32: the "
                         "8B shape in true 32-bit; reference-kernels: the reference's CUDA kernels alone, if built; tumatar: the "
                         "Tumatar design beside the Llama shape of the same width (--shape 1b or 8b), and its kernels alone; tikalix: "
                         "the same for the Tikalix design; vilazen: the same for the Vilazen design; lipadra: the Lipadra design "
                         "beside the Tumatar design and the Llama shape of the same width, and its kernels alone")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="--case prefill/decode: layer sizes")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="--case prefill/decode")
    ap.add_argument("--repeats", type=int, default=2, help="workload cases: timed repetitions after one warm-up")
    ap.add_argument("--batch", type=int, default=8, help="--case decode: sequences in the batch")
    ap.add_argument("--context", type=int, default=CONTEXT, help="--case decode: tokens each sequence holds")
    ap.add_argument("--prompt-tokens", type=int, default=PREFILL_TOKENS, help="--case prefill: tokens of the prompt")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Zig program (no setup.py or pyproject.toml, pip reports it is not "
                          "installable) and no Zig toolchain is installed here or on the GPU box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    if args.case == "reference-kernels":
        return run_reference_kernels(args)
    if args.case in ("workload-1b", "workload-13b"):
        return run_workload(args)
    if args.case == "float32":
        return run_float32(args)
    if args.case == "tumatar":
        return run_tumatar(args)
    if args.case == "tikalix":
        return run_tikalix(args)
    if args.case == "vilazen":
        return run_vilazen(args)
    if args.case == "lipadra":
        return run_lipadra(args)
    if args.case != "full":
        return run_case(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
