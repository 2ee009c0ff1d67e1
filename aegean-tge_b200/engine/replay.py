"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and schedules nothing.  It drives the same model, step
function, cache and kernels that generation uses (an :class:`Engine` without
its scheduler and sampler).  The nearest things in the reference are the
teacher-forced stepping of its fidelity command (apps/cli/main.cpp:2505-2509)
and the all-row logits of ``verify_draft_logits`` (src/models/qwen2.cpp:2518-2532).

Input, one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  A request appears with its first
tokens, may be left out of steps, and is given back when a step lists it
under ``end``.  For a step that wants logits, ``<out>/<step>.f32`` receives
them as little-endian float32 ``[wanted, vocab]`` in the order of the entries
and of ``want``.  After every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np

from .. import ops as _ops
from .batch import Portion
from .engine import Engine


def run_trace(engine: Engine, lines: IO[str], out_dir: str, reply: IO[str]) -> int:
    os.makedirs(out_dir, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        portions = [Portion(entry["id"], list(entry["tokens"]), list(entry.get("want", [])))
                    for entry in record.get("entries", [])]
        logits = engine.runner.step(portions) if portions else None
        if logits is not None:
            host = logits.float().cpu().numpy().astype("<f4", copy=False)
            host.tofile(os.path.join(out_dir, f"{step}.f32"))
        _ops.check_status()
        for request in record.get("end", []):
            if engine.runner.is_live(request):
                engine.runner.finish(request)
        reply.write(f"done {step}\n")
        reply.flush()
    return 0


def main(argv: Optional[list] = None) -> int:
    import argparse
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder that receives <step>.f32")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (the cache pool is made for this many)")
    parser.add_argument("--trace", help="file of steps, one JSON object a line (default: standard input)")
    args = parser.parse_args(argv)
    if args.max_tokens <= 0:
        parser.error("--max-tokens must be positive")
    print(f"[trace_run] loading {args.model} ({args.dtype}); kernels are compiled on first use", file=sys.stderr,
          flush=True)
    engine = Engine(args.model, dtype=args.dtype, context=args.max_tokens, max_tokens=args.max_tokens,
                    max_requests=8, max_batch_tokens=max(args.max_tokens, 1))
    print(f"[trace_run] ready: {engine.describe()}", file=sys.stderr, flush=True)
    if args.trace:
        with open(args.trace, "r", encoding="utf-8") as handle:
            return run_trace(engine, handle, args.out, sys.stdout)
    return run_trace(engine, sys.stdin, args.out, sys.stdout)


if __name__ == "__main__":
    sys.exit(main())
