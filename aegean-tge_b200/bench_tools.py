"""Timed prefill and decode steps with their roofline fractions, shared by `tge bench` and bench.py.

Timing is with CUDA events on the launching stream after warm-up, with a
synchronize on both sides.  A decode step reads every weight once (about
15 GB for the 7B shape) plus the cache of the live requests, far more than
the 126 MB L2, so no extra flush is needed between steps; the prefill's
weights are likewise larger than L2.
"""
from __future__ import annotations

import random
from typing import Dict, List

import torch

from . import peaks as _peaks
from .engine.batch import Portion


def _random_tokens(vocab: int, count: int, seed: int) -> List[int]:
    rnd = random.Random(seed)
    return [rnd.randrange(vocab) for _ in range(count)]


def prefill_flops(engine, tokens: int) -> float:
    """Operations of one whole prompt (a multiply-add is two): what the model's parts report for ``tokens``
    tokens under a causal mask, and one row of logits."""
    return engine.model.step_flops(tokens, tokens * (tokens + 1) / 2.0, 1)


def bench_prefill(engine, prompt_len: int, repeat: int = 3, warmup: int = 2, sustain_seconds: float = 0.0) -> Dict[str, float]:
    """A whole prompt in one step, timed on the device: the mean of ``repeat`` runs after ``warmup``.

    A B200 under its power cap runs the first steps after a pause faster than it sustains (a 2,048-token
    prompt of the 7B shape: 20.3 ms for two or three runs, then 22.5-23.5 ms).  With ``sustain_seconds`` > 0 two
    more figures are taken, to be read against the two peaks measured the same ways: ``burst_ms`` (the best of
    three runs after a pause of two seconds; the burst peak is a best of ten) and ``sustained_ms`` (the mean over
    a loop of that many seconds; the sustained peak is a loop of four seconds)."""
    import time
    vocab = engine.spec.vocab_size
    counter = [0]

    def one() -> float:
        tokens = _random_tokens(vocab, prompt_len, seed=100 + counter[0] % 7)
        counter[0] += 1
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.runner.step([Portion("bench-prefill", tokens, [prompt_len - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.runner.finish("bench-prefill")
        return start.elapsed_time(stop)

    for _ in range(warmup):
        one()
    times = [one() for _ in range(repeat)]
    ms = sum(times) / len(times)
    flops = prefill_flops(engine, prompt_len)
    peak, source = _peaks.load()
    tflops = flops / (ms * 1e-3) / 1e12
    out = {"tokens": prompt_len, "ms": ms, "tok_s": prompt_len / (ms * 1e-3), "tflops": tflops,
           "peak_tflops": peak["bf16_tflops"], "frac": tflops / peak["bf16_tflops"], "peak_source": source,
           "flops": flops}
    if sustain_seconds > 0:
        begin = time.perf_counter()
        loop = []
        while time.perf_counter() - begin < sustain_seconds:
            loop.append(one())
        out["sustained_ms"] = sum(loop) / len(loop)
        sustained_peak = peak.get("bf16_tflops_sustained", peak["bf16_tflops"])
        out["sustained_frac"] = flops / (out["sustained_ms"] * 1e-3) / 1e12 / sustained_peak
        time.sleep(2.0)
        out["burst_ms"] = min(one() for _ in range(3))
        out["burst_frac"] = flops / (out["burst_ms"] * 1e-3) / 1e12 / peak["bf16_tflops"]
    return out


def fill_cache(engine, batch: int, prompt_len: int, chunk: int = 2048, prefix: str = "bench") -> List[str]:
    """Prefills ``batch`` requests of ``prompt_len`` random tokens (untimed); returns their ids."""
    vocab = engine.spec.vocab_size
    names = []
    for b in range(batch):
        name = f"{prefix}-{b}"
        tokens = _random_tokens(vocab, prompt_len, seed=1000 + b)
        for begin in range(0, prompt_len, chunk):
            engine.runner.step([Portion(name, tokens[begin:begin + chunk], [])])
        names.append(name)
    return names


def decode_step_bytes(engine, names: List[str]) -> float:
    """Bytes a decode step must read: every weight it uses once, and the cache of the live requests."""
    cached = sum(engine.cache.computed(n) for n in names)
    return engine.model.step_param_bytes() + cached * engine.model.cache_bytes_per_token()


def bench_decode(engine, batch: int, prompt_len: int, steps: int = 64, warmup: int = 3) -> Dict[str, float]:
    """Device-timed decode steps (model and sampling kernels; the sampled ids stay on the device)."""
    from . import ops
    names = fill_cache(engine, batch, prompt_len)
    vocab = engine.spec.vocab_size
    zeros = torch.zeros(batch, dtype=torch.float32, device=engine.device)
    feed = [_random_tokens(vocab, warmup + steps, seed=5000 + b) for b in range(batch)]
    def one(step: int):
        logits = engine.runner.step([Portion(n, [feed[b][step]], [0]) for b, n in enumerate(names)])
        return ops.sample(logits, zeros, zeros)
    for step in range(warmup):
        one(step)
    torch.cuda.synchronize()
    bytes_first = decode_step_bytes(engine, names)
    launches_before = ops.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(warmup, warmup + steps):
        one(step)
    stop.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = start.elapsed_time(stop) / steps
    bytes_last = decode_step_bytes(engine, names)
    for n in names:
        engine.runner.finish(n)
    step_bytes = (bytes_first + bytes_last) / 2
    peak, source = _peaks.load()
    gbs = step_bytes / (ms * 1e-3) / 1e9
    return {"batch": batch, "ms_per_step": ms, "tok_s": batch / (ms * 1e-3), "step_bytes": step_bytes, "gbs": gbs,
            "peak_gbs": peak["hbm_gbs"], "frac": gbs / peak["hbm_gbs"], "peak_source": source,
            "launches": ops.launches - launches_before, "steps": steps}


def bench_mixed(engine, decodes: int, prompt_len: int, portion: int, repeat: int = 3) -> Dict[str, float]:
    """One step of ``decodes`` single tokens (each request holding ``prompt_len`` tokens) beside one prompt
    portion of ``portion`` tokens, timed on the device: what a scheduler's step looks like while a prompt arrives."""
    names = fill_cache(engine, decodes, prompt_len, prefix="mixed")
    prompt = _random_tokens(engine.spec.vocab_size, portion, seed=31)
    times = []
    for it in range(repeat + 1):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.runner.step([Portion(n, [7 + it], [0]) for n in names] + [Portion("mixed-prompt", prompt, [portion - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.runner.finish("mixed-prompt")
        if it:
            times.append(start.elapsed_time(stop))
    for n in names:
        engine.runner.finish(n)
    ms = sum(times) / len(times)
    return {"ms": ms, "decodes": decodes, "portion": portion, "tok_s": (decodes + portion) / (ms * 1e-3)}


def step_timeline(engine, batch: int, prompt_len: int, prefill: bool, portion: int = 0) -> List[Dict[str, float]]:
    """Where one step's time goes, by kernel name, from the CUDA activity records of one step after
    warm-up: a prompt of ``prompt_len`` tokens (``prefill``) or one token for each of ``batch`` requests
    that hold ``prompt_len`` tokens, with ``portion`` > 0 beside one prompt portion of that many tokens.

    A kernel launched as the dependent of another starts early and waits, so its own duration says
    little.  What is charged to a kernel here is the time from the end of the kernel that ended before it
    (or from its own start, if later) to its own end: the charges add up to the span of the step less the
    gaps in which nothing ran.
    """
    from torch.profiler import ProfilerActivity, profile
    vocab = engine.spec.vocab_size
    if prefill:
        tokens = _random_tokens(vocab, prompt_len, seed=77)

        def run():
            engine.runner.step([Portion("timeline", tokens, [prompt_len - 1])])
            engine.runner.finish("timeline")
        names = []
    else:
        names = fill_cache(engine, batch, prompt_len, prefix="timeline")
        beside = _random_tokens(vocab, portion, seed=78) if portion > 0 else []

        def run():
            engine.runner.step([Portion(n, [5], [0]) for n in names] +
                               ([Portion("timeline-portion", beside, [portion - 1])] if portion > 0 else []))
            if portion > 0:
                engine.runner.finish("timeline-portion")
    for _ in range(4):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    for n in names:
        engine.runner.finish(n)
    events = [(e.time_range.start, e.time_range.start + e.device_time_total, e.name) for e in prof.events()
              if e.device_time_total > 0]
    events.sort(key=lambda e: e[1])
    first = min(e[0] for e in events)
    by_name: Dict[str, List[float]] = {}
    previous_end = first
    for start, end, raw in events:
        name = raw.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0].strip()
        by_name.setdefault(name, []).append(end - max(previous_end, start))
        previous_end = max(previous_end, end)
    span = previous_end - first
    rows = [{"kernel": name, "launches": len(v), "us": sum(v), "share": sum(v) / span} for name, v in by_name.items()]
    rows.sort(key=lambda r: -r["us"])
    rows.append({"kernel": "span of the step under the profiler", "launches": len(events), "us": span, "share": 1.0})
    return rows
