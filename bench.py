#!/usr/bin/env python3
"""Headline measurement: decode tokens/s of the Qwen2.5-7B shape in bfloat16 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One "step" is one decode step of a batch of 8 requests, each after a prompt of
2,048 tokens (random weights, random token ids), with cache pages of 16 tokens
as the benchmark configuration has them.  Prints one JSON line: ``value`` is
decoded tokens per second timed on the device over K steps, ``e2e`` the same
through the Python entry point with host tokens in and out, ``prefill`` a
2,048-token prompt in one step against the bf16 tensor peak, ``roofline`` the
decode step against HBM bandwidth.  ``points`` holds decode at batch 1 and 64
(device-timed and end to end), a mixed step (63 decode rows beside a prompt
portion), the same figures with the engine's default pages of 64 tokens, long
contexts, and the 14B and 32B shapes.  This engine runs on one GPU: for --gpus
above 1 it says so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The Qwen2.5-7B shape of BASELINE.json's configs[2]
with open(os.path.join(ROOT, "aegean-tge_b200", "config", "shapes", "qwen2.5-7b.json"), "r", encoding="utf-8") as _handle:
    CONFIG_7B = json.load(_handle)
PROMPT = 2048
CONTEXT = 4096
BATCH = 8
PAGE = 16           # the benchmark configuration's page; the engine's own default is 64 (reported under points)


def load_shape(name):
    with open(os.path.join(ROOT, "aegean-tge_b200", "config", "shapes", name), "r", encoding="utf-8") as handle:
        return json.load(handle)


def reference_arm() -> int:
    """The reference is a C++/CMake CPU engine for Windows with no Python packaging: it cannot be
    installed with pip, has no CUDA path, and never ran this model."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = ("the reference is a CMake C++ CPU engine without setup.py/pyproject.toml: 'pip install' of its source tree "
           "finds nothing to build, and it has no GPU path or bf16 model to run this metric with")
    if os.path.isdir(ref) and os.listdir(ref):
        why = "baseline/_ref holds no importable package that exposes the reference's generate path; " + why
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ["clocks.sm", "clocks.max.sm", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self):
        self.path = os.path.join(tempfile.gettempdir(), f"tge_clocks_{os.getpid()}.csv")
        self.proc = None

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=" + ",".join(self.FIELDS),
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        self.out.close()
        clocks, peak, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as handle:
            for line in handle:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) != len(self.FIELDS):
                    continue
                try:
                    clocks.append(float(parts[0]))
                    peak = float(parts[1])
                except ValueError:
                    continue
                for name, value in zip(names, parts[2:]):
                    if value.lower().startswith("active"):
                        reasons.add(name)
        os.remove(self.path)
        clocks.sort()
        median = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": median, "sm_max_mhz": peak, "reasons": sorted(reasons), "samples": len(clocks)}


def end_to_end(engine, batch, steps, warmup, sampling=None):
    """Decode steps through the public entry point: host token ids in, sampled ids out, every step (greedy, or
    with ``sampling``).  Returns (tokens per second, host-to-device bytes per step, device-to-host bytes per step)."""
    import time
    import torch
    from aegean_tge_b200.bench_tools import _random_tokens
    vocab = engine.spec.vocab_size
    for b in range(batch):
        engine.add_request(_random_tokens(vocab, PROMPT, seed=2000 + b), n=warmup + steps + batch + 4, sampling=sampling)
    while any(not r.output for r in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()                                   # prefill and the first token, untimed
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    h2d = engine.runner.h2d_bytes_last + 8 * batch
    d2h = engine.d2h_bytes_last
    while engine.has_unfinished():
        engine.step()
    return batch * steps / seconds, h2d, d2h


def prefill_record(run):
    """The prefill figures of the JSON line.  Under its power cap a B200 runs the first steps after a pause faster
    than it sustains, and the two measured peaks were taken in those two ways; so both are given, each against
    its own peak: `ms`/`value`/`frac` the best of three runs after a two-second pause against the burst peak (a
    best of ten), `sustained_*` the mean over a one-second loop against the sustained peak (a four-second loop),
    `mean3_ms` the mean of three runs right after two warm-up runs (what earlier lines of this bench reported)."""
    if "burst_ms" not in run:
        return {"value": round(run["tok_s"], 1), "tokens": run["tokens"], "ms": round(run["ms"], 3),
                "frac": round(run["frac"], 4), "how": "mean of 3 after 2 warm-up runs, against the burst peak"}
    return {"value": round(run["tokens"] / (run["burst_ms"] * 1e-3), 1), "tokens": run["tokens"],
            "ms": round(run["burst_ms"], 3), "frac": round(run["burst_frac"], 4),
            "how": "best of 3 after a 2 s pause, against the burst peak",
            "sustained_ms": round(run["sustained_ms"], 3), "sustained_frac": round(run["sustained_frac"], 4),
            "sustained_value": round(run["tokens"] / (run["sustained_ms"] * 1e-3), 1), "mean3_ms": round(run["ms"], 3)}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=CONFIG_7B["num_hidden_layers"],
                        help="fewer layers than the model has, if memory or time needs it (both numbers are reported)")
    parser.add_argument("--skip-points", action="store_true", help="the headline only: no points")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import gc
    import torch
    import aegean_tge_b200 as tge
    from aegean_tge_b200 import ops, peaks
    from aegean_tge_b200.bench_tools import bench_decode, bench_mixed, bench_prefill

    raw = dict(CONFIG_7B, num_hidden_layers=args.layers)
    need = args.warmup + args.steps + BATCH + 8
    most_batch = BATCH if args.skip_points else 64
    short = min(args.steps, 32)

    def engine_for(config, page_size, batch=most_batch, context=CONTEXT, prompt=PROMPT):
        gc.collect()
        torch.cuda.empty_cache()
        return tge.Engine(random_config=config, seed=0, dtype="bfloat16", context=context, page_size=page_size,
                          max_tokens=batch * (prompt + need + 64) + (0 if args.skip_points else PROMPT),
                          max_batch_tokens=PROMPT, max_requests=batch + 1)

    engine = engine_for(raw, PAGE)
    peak, peak_source = peaks.load()
    prefill = bench_prefill(engine, PROMPT, repeat=3, warmup=2, sustain_seconds=0 if args.skip_points else 1.0)

    def rested():
        """Two seconds without work.  Under its 1 kW cap the GPU runs what comes first after a pause a few per
        cent faster than what comes later (a decode step of this shape 3.03 ms, 3.2 ms after ten seconds of
        work), so every figure that is compared with another starts from the same rest."""
        torch.cuda.synchronize()
        time.sleep(2.0)

    sampler = ClockSampler()
    rested()
    sampler.start()
    main_run = bench_decode(engine, BATCH, PROMPT, steps=args.steps, warmup=args.warmup)
    clocks = sampler.stop()
    rested()
    e2e, h2d, d2h = end_to_end(engine, BATCH, args.steps, args.warmup)
    queued_ahead = engine.stats()["steps_queued_ahead"]["used"]
    ops.check_status()

    points = {}
    rnd = lambda value, digits=1: round(value, digits)

    def group(name, body):
        """One group of points; a failure (out of memory on a smaller GPU, say) is recorded and the headline stands."""
        try:
            body()
        except Exception as error:       # noqa: BLE001
            points[f"{name}_error"] = f"{type(error).__name__}: {error}"[:200]
            gc.collect()
            torch.cuda.empty_cache()

    if not args.skip_points:
        def other_batches():
            for batch in (1, 64):
                rested()
                run = bench_decode(engine, batch, PROMPT, steps=short, warmup=args.warmup)
                points[f"decode_b{batch}"] = rnd(run["tok_s"])
                points[f"decode_b{batch}_hbm_frac"] = rnd(run["frac"], 4)
                rested()
                points[f"e2e_b{batch}"] = rnd(end_to_end(engine, batch, short, args.warmup)[0])
            points["mixed_step_ms"] = rnd(bench_mixed(engine, 63, PROMPT, PROMPT - 63)["ms"], 3)
            cuts = tge.SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1)     # what the cuts cost a step
            rested()
            points["e2e_b8_top_k50_top_p"] = rnd(end_to_end(engine, BATCH, short, args.warmup, sampling=cuts)[0])
        group("batches", other_batches)
        del engine

        def default_pages():        # the engine's own default page of 64 tokens
            engine = engine_for(raw, 64)
            run = bench_prefill(engine, PROMPT, repeat=3, warmup=2, sustain_seconds=0.5)
            points["page64_prefill"] = rnd(PROMPT / (run["burst_ms"] * 1e-3))
            for batch in (8, 64):
                points[f"page64_decode_b{batch}"] = rnd(bench_decode(engine, batch, PROMPT, steps=short, warmup=args.warmup)["tok_s"])
        group("page64", default_pages)

        def long_contexts():
            for batch, context in ((4, 30000), (32, 8000)):
                engine = engine_for(raw, 64, batch=batch, context=32768, prompt=context)
                run = bench_decode(engine, batch, context, steps=short, warmup=args.warmup)
                points[f"decode_b{batch}_ctx{context}"] = rnd(run["tok_s"])
                points[f"decode_b{batch}_ctx{context}_hbm_frac"] = rnd(run["frac"], 4)
                del engine
        group("long_context", long_contexts)

        def larger_shapes():
            for label, shape in (("14b", "qwen2.5-14b.json"), ("32b", "qwen2.5-32b.json")):
                engine = engine_for(load_shape(shape), PAGE, batch=BATCH)
                if label == "14b":
                    run = bench_prefill(engine, PROMPT, repeat=3, warmup=2, sustain_seconds=1.0)
                    points["prefill_14b"] = rnd(PROMPT / (run["burst_ms"] * 1e-3))
                    points["prefill_14b_frac"] = rnd(run["burst_frac"], 4)
                    points["prefill_14b_sustained_frac"] = rnd(run["sustained_frac"], 4)
                run = bench_decode(engine, BATCH, PROMPT, steps=short, warmup=args.warmup)
                points[f"decode_b8_{label}"], points[f"decode_b8_{label}_hbm_frac"] = rnd(run["tok_s"]), rnd(run["frac"], 4)
                del engine
        group("larger_shapes", larger_shapes)
        try:
            ops.check_status()
        except Exception as error:       # noqa: BLE001
            points["status_error"] = str(error)[:200]

    line = {
        "metric": "decode tok/s at batch 8 after 2,048-token prompts; Qwen2.5-7B shape bf16 (with prefill tok/s at "
                  "2,048 tokens and decode at batch 1/64)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) seed 0, uniform random token ids",
        "config": {
            "model": "Qwen2.5-7B shape", "layers": args.layers, "layers_of_model": CONFIG_7B["num_hidden_layers"],
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
            "global_batch": BATCH, "seq_len": PROMPT, "context_limit": CONTEXT, "page_size": PAGE,
            "prefill_tokens": PROMPT, "parallelism": "1 GPU", "cuda_graph": True,
            "l2": "each step reads all weights (>> 126 MB L2), no flush needed",
            "peaks": peak_source, "rest": "2 s without work before value, e2e and the batch-1/64 points",
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps_queued_ahead": queued_ahead},
        "gpu_launches": main_run["launches"],
        "prefill": prefill_record(prefill),
        "roofline": {"bound": "hbm", "achieved": round(main_run["gbs"], 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["frac"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
