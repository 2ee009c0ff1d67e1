"""The `tge` command line, in the manner of the reference's (apps/cli/main.cpp:45-140).

    tge info [--json]
    tge plan --model DIR [--context N] [--sessions N] [--bandwidth GB/s]
    tge generate --model DIR --tokens "a b c" [--n N] [--temp T] [--top-k N] [--top-p P] [--min-p P]
                 [--repeat-penalty R] [--penalty-window N] [--seed N] [--context N] [--print-ids]
    tge bench prefill|decode --model DIR [--prompt-len N] [--batch B] [--n N] [--repeat R]
    tge bench mixed --model DIR [--batch B] [--prompt-len N] [--portion P]      (B single tokens beside a prompt portion)
    tge fidelity --model DIR [--context N] [--tokens N] [--corpus FILE]
    tge bench continuous --model DIR [--requests N] [--tokens N] [--sequences N] [--prompt-tokens N] [--prompt-max N]
    tge make-random --config FILE --out DIR [--seed S] [--dtype float32|bfloat16]
    tge replay --model DIR --dtype D --out DIR --max-tokens N          (same as bin/trace_run)
    tge version

Options shared with the reference keep its names, defaults and meanings:
``--n`` tokens to generate (default 32), ``--context`` cache length (default
4096, capped by the model), ``--temp`` 0 is greedy, ``--top-k`` / ``--top-p`` /
``--min-p`` / ``--repeat-penalty`` / ``--penalty-window`` / ``--seed`` as in
its sampler, ``--print-ids``.  Output lines carry its labels (``load``,
``resolved``, ``model``, ``prefill``, ``decode``, ``ids``; decode excludes the
first generated token, main.cpp:1216-1219).  Exit codes: 2 for a usage error,
1 for a load or run-time failure (main.cpp:3061-3072).  ``--prompt`` / ``--text``
need a tokenizer, which this engine does not have: it takes and returns ids.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional

from . import __version__


class UsageError(Exception):
    pass


class _Parser(argparse.ArgumentParser):
    def error(self, message):
        raise UsageError(f"{self.prog}: {message}")


def _model_args(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--model", help="model folder (config.json + model.safetensors)")
    parser.add_argument("--random-config", "--config", dest="random_config",
                        help="config.json file: run with seeded random weights instead of --model")
    parser.add_argument("--random-weights", action="store_true", help="(implied by --random-config / --config)")
    parser.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    parser.add_argument("--context", type=int, default=4096, help="KV cache length (default 4096, capped by model)")
    parser.add_argument("--num-pages", type=int, help="pages in the cache pool (default: from free memory)")
    parser.add_argument("--page-size", type=int, default=None, help="tokens per page: 64 (default), 32, 16 or 8")
    parser.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of one step")
    parser.add_argument("--chunk", type=int, help="largest prompt portion in one step (default: the budget)")
    parser.add_argument("--max-requests", type=int, default=64)


def _sampling_args(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--temp", type=float, default=0.0, help="sampling temperature; 0 is greedy (default 0)")
    parser.add_argument("--top-k", type=int, default=0, help="keep the N best tokens (default off)")
    parser.add_argument("--top-p", type=float, default=1.0, help="nucleus probability mass (default 1.0)")
    parser.add_argument("--min-p", type=float, default=0.0, help="drop tokens below this fraction of the best")
    parser.add_argument("--repeat-penalty", type=float, default=1.0, help="penalty for already seen tokens (default 1)")
    parser.add_argument("--penalty-window", type=int, default=64, help="recent tokens the penalty sees; 0 is all")
    parser.add_argument("--seed", type=int, default=0, help="random seed for sampling")


def build_parser() -> argparse.ArgumentParser:
    parser = _Parser(prog="tge", description=f"aegean-tge b200 {__version__} - Qwen2.5 inference engine for one B200")
    commands = parser.add_subparsers(dest="command", parser_class=_Parser)
    info = commands.add_parser("info", help="GPU, memory and kernel report")
    info.add_argument("--json", action="store_true")
    plan = commands.add_parser("plan", help="memory budget and decode ceiling, before loading")
    plan.add_argument("--model", required=True)
    plan.add_argument("--context", type=int, default=4096)
    plan.add_argument("--sessions", type=int, default=1)
    plan.add_argument("--bandwidth", type=float, help="GB/s (default: the measured or nominal HBM figure)")
    plan.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    generate = commands.add_parser("generate", help="generate tokens and report token rates")
    _model_args(generate)
    _sampling_args(generate)
    generate.add_argument("--tokens", help='prompt token ids, "a b c"')
    generate.add_argument("--prompt", help="(needs a tokenizer: not supported, give --tokens)")
    generate.add_argument("--prompt-len", type=int, help="random prompt of this many ids instead of --tokens")
    generate.add_argument("--n", type=int, default=32, help="tokens to generate (default 32)")
    generate.add_argument("--print-ids", action="store_true", help="print generated token ids")
    generate.add_argument("--text", action="store_true", help="(needs a tokenizer: not supported)")
    bench = commands.add_parser("bench", help="prefill or decode throughput with its roofline fraction")
    bench.add_argument("what", choices=["prefill", "decode", "mixed", "continuous"])
    _model_args(bench)
    bench.add_argument("--prompt-len", type=int, default=2048)
    bench.add_argument("--batch", type=int, default=1)
    bench.add_argument("--n", type=int, default=64, help="decode steps to time")
    bench.add_argument("--repeat", type=int, default=3)
    bench.add_argument("--portion", type=int, default=1985,
                       help="mixed: tokens of the prompt portion that runs beside --batch single tokens (default 1985)")
    bench.add_argument("--timeline", action="store_true", help="prefill/decode/mixed: also list one step's kernels with their device times")
    # bench continuous, with the reference's names (apps/cli/main.cpp:2825-2890)
    bench.add_argument("--requests", type=int, default=8, help="continuous: requests to serve (default 8)")
    bench.add_argument("--tokens", type=int, default=32, help="continuous: tokens generated per request (default 32)")
    bench.add_argument("--sequences", type=int, default=4, help="continuous: requests live at a time (default 4)")
    bench.add_argument("--prompt-tokens", type=int, default=1, help="continuous: prompt length (default 1)")
    bench.add_argument("--prompt-max", type=int, help="continuous: draw each prompt's length from [prompt-tokens, this]")
    fidelity = commands.add_parser("fidelity", help="the float32 path against the bfloat16 kernels, teacher-forced")
    _model_args(fidelity)
    fidelity.add_argument("--corpus", help="file of token ids separated by white space (default: seeded random ids)")
    fidelity.add_argument("--tokens", type=int, default=256, help="positions to compare (default 256)")
    make = commands.add_parser("make-random", help="write a model folder with seeded random weights")
    make.add_argument("--config", required=True, help="a config.json")
    make.add_argument("--out", required=True)
    make.add_argument("--seed", type=int, default=0)
    make.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    replay = commands.add_parser("replay", help="feed token ids step by step and write logits (bin/trace_run)")
    replay.add_argument("--model", required=True)
    replay.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    replay.add_argument("--out", required=True)
    replay.add_argument("--max-tokens", type=int, required=True)
    replay.add_argument("--trace", help="file of steps (default: standard input)")
    commands.add_parser("version", help="print the engine version")
    return parser


def _engine_from(args):
    from .engine.engine import Engine
    if bool(args.model) == bool(args.random_config):
        raise UsageError("give --model DIR or --random-config FILE")
    random_config = None
    if args.random_config:
        with open(args.random_config, "r", encoding="utf-8") as handle:
            random_config = json.load(handle)
    return Engine(args.model, random_config=random_config, seed=args.weights_seed, dtype=args.dtype,
                  context=args.context, num_pages=args.num_pages, max_batch_tokens=args.max_batch_tokens,
                  chunk=args.chunk, max_requests=args.max_requests,
                  **({} if args.page_size is None else {"page_size": args.page_size}))


def command_info(args) -> int:
    import torch
    from .csrc import build
    from .engine.engine import PAGE_SIZE
    facts = {"version": __version__, "cuda_available": torch.cuda.is_available(), "torch": torch.__version__,
             "cuda_runtime": torch.version.cuda, "page_size": PAGE_SIZE, "kernel_target": "sm_100a",
             "kernel_sources": build.CORE_SOURCES + ["attention_mma.cu"]}
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(0)
        free, total = torch.cuda.mem_get_info(0)
        facts.update({"gpu": props.name, "sms": props.multi_processor_count,
                      "compute_capability": f"{props.major}.{props.minor}", "memory_total_bytes": total,
                      "memory_free_bytes": free})
    if args.json:
        print(json.dumps(facts))
    else:
        for key, value in facts.items():
            print(f"{key:<20}: {value}")
    return 0


def command_plan(args) -> int:
    """Bytes before loading, in the manner of the reference's planner (src/models/plan.cpp:28-133).  The model
    is put together on paper (its parts, no weights, no GPU) and asked what it holds and what a step reads."""
    import torch
    from .config.common import read_config_json
    from .engine.engine import PAGE_SIZE
    from .models.decoder import DecoderModel
    from .parts.base import BuildEnv
    from .peaks import hbm_gbs
    from .registry import architecture_of
    from .weights.random_init import parse_dtype
    raw = read_config_json(args.model)
    arch = architecture_of(raw)
    spec = arch.build_spec(arch.parse_config(raw))
    env = BuildEnv(dtype=parse_dtype(args.dtype), device=torch.device("cpu"), hidden_size=spec.hidden_size,
                   max_positions=min(spec.max_positions, args.context), page_size=PAGE_SIZE, ops=None)
    model = DecoderModel(spec, env)
    weights = model.weight_bytes()
    decode_bytes = model.step_param_bytes()                 # everything but the embedding rows (plan.cpp:42-46)
    kv_per_token = model.cache_bytes_per_token()
    bandwidth = args.bandwidth or hbm_gbs()
    total = weights + args.sessions * args.context * kv_per_token
    print(f"weights  : {weights / 2**30:.2f} GiB ({args.dtype})")
    print(f"kv       : {kv_per_token} bytes per token; {args.sessions} x {args.context} tokens = "
          f"{args.sessions * args.context * kv_per_token / 2**30:.2f} GiB")
    print(f"total    : {total / 2**30:.2f} GiB")
    print(f"decode   : {decode_bytes / 2**20:.1f} MiB read per token; ceiling {bandwidth * 1e9 / decode_bytes:.1f} tok/s "
          f"at {bandwidth:.0f} GB/s")
    return 0


def _parse_ids(text: str) -> List[int]:
    try:
        return [int(part) for part in text.replace(",", " ").split()]
    except ValueError:
        raise UsageError('--tokens takes integers, "a b c"')


def command_generate(args) -> int:
    import random
    import torch
    from . import ops
    from .sampling.params import SamplingParams
    if args.prompt or args.text:
        raise UsageError("generate: --prompt and --text need a tokenizer, which this engine does not have; give --tokens")
    if args.n <= 0:
        raise UsageError("generate: token count must be positive")
    sampling = SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                              repeat_penalty=args.repeat_penalty, penalty_window=args.penalty_window, seed=args.seed)
    try:
        sampling.validate()
    except ValueError as error:
        raise UsageError(f"generate: {error}")
    started = time.time()
    engine = _engine_from(args)
    print(f"load     : {(time.time() - started) * 1e3:.1f} ms")
    facts = engine.describe()
    print(f"resolved : dtype={facts['dtype']} context={facts['max_model_len']} page={facts['page_size']} "
          f"pages={facts['pages_per_group']} budget={args.max_batch_tokens} kernels=sm_100a")
    if args.tokens:
        prompt = _parse_ids(args.tokens)
    elif args.prompt_len:
        rnd = random.Random(0)
        prompt = [rnd.randrange(engine.spec.vocab_size) for _ in range(args.prompt_len)]
    else:
        raise UsageError("generate: at least one prompt token is required")
    if not prompt:
        raise UsageError("generate: at least one prompt token is required")
    if len(prompt) + args.n + 1 > engine.max_model_len:
        raise UsageError(f"generate: {len(prompt)} prompt tokens + {args.n} generated exceeds the "
                         f"{engine.max_model_len} token context")
    for token in prompt:
        if not 0 <= token < engine.spec.vocab_size:
            raise UsageError(f"generate: token {token} is outside the vocabulary")
    print(f"model    : {args.model or args.random_config}, {facts['layers']} layers ({facts['layer_kinds']}), "
          f"{facts['hidden_size']} dim, vocab {facts['vocab_size']}")
    if not engine.spec.end_token_ids:
        print("generate: warning: model declares no end-of-generation ids; stopping only at --n", file=sys.stderr)
    request_id = engine.add_request(prompt, args.n, sampling)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    finished = []
    request = engine.scheduler.waiting[0]
    while not request.output and not finished:
        finished = engine.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    print(f"prefill  : {len(prompt)} tokens in {(t1 - t0) * 1e3:.2f} ms ({len(prompt) / (t1 - t0):.1f} tok/s)")
    while not finished:
        finished = engine.step()
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    ops.check_status()
    output = finished[0].output
    if finished[0].finish_reason == "end_token":
        print(f"stop     : end token {output[-1]} after {len(output)} tokens")
    timed = len(output) - 1
    if timed > 0:
        print(f"decode   : {timed} tokens in {(t2 - t1) * 1e3:.2f} ms ({timed / (t2 - t1):.2f} tok/s)")
    if args.print_ids:
        print("ids      : " + " ".join(str(t) for t in output))
    return 0


def command_fidelity(args) -> int:
    """The reference's ``fidelity`` (apps/cli/main.cpp:2379-2596) runs its full-scalar oracle and the selected
    kernels over the same tokens, teacher-forced, and reports KL, the largest logit difference and top-1
    agreement.  Here the oracle is the engine's own true 32-bit path and the candidate its bfloat16 kernels;
    the first half of the tokens runs as one prompt, the second half one token at a time."""
    import gc
    import random
    import time
    import torch
    from .engine.batch import Portion
    if args.tokens < 2:
        raise UsageError("fidelity: at least two tokens")
    started = time.time()
    logits = {}
    tokens = None
    load_seconds = 0.0
    for dtype in ("float32", "bfloat16"):
        args.dtype = dtype
        args.max_requests = 1
        t0 = time.time()
        engine = _engine_from(args)
        load_seconds += time.time() - t0
        if tokens is None:
            vocab = engine.spec.vocab_size
            if args.corpus:
                with open(args.corpus, "r", encoding="utf-8") as handle:
                    tokens = [int(t) for t in handle.read().split()]
                if any(not 0 <= t < vocab for t in tokens):
                    raise UsageError(f"fidelity: the corpus holds ids outside the vocabulary of {vocab}")
            else:
                rnd = random.Random(4321)
                tokens = [rnd.randrange(vocab) for _ in range(args.tokens)]
            tokens = tokens[:min(args.tokens, engine.max_model_len)]
            if len(tokens) < 2:
                raise UsageError(f"fidelity: corpus needs two tokens within the {engine.max_model_len}-token context")
        half = max(len(tokens) // 2, 1)
        rows = [engine.runner.step([Portion("f", tokens[:half], list(range(half)))]).double()]
        for t in range(half, len(tokens)):
            rows.append(engine.runner.step([Portion("f", tokens[t:t + 1], [0])]).double())
        logits[dtype] = torch.cat(rows)
        from . import ops
        ops.check_status()
        del engine, rows
        gc.collect()
        torch.cuda.empty_cache()
    reference, candidate = logits["float32"], logits["bfloat16"]
    log_p = torch.log_softmax(reference, dim=-1)
    log_q = torch.log_softmax(candidate, dim=-1)
    kl = (log_p.exp() * (log_p - log_q)).sum(-1)
    agree = int((reference.argmax(-1) == candidate.argmax(-1)).sum())
    positions = reference.shape[0]
    print("fidelity : float32 path vs bfloat16 kernels (prompt of %d tokens, then %d single tokens)"
          % (max(len(tokens) // 2, 1), positions - max(len(tokens) // 2, 1)))
    print(f"load     : {load_seconds * 1e3:.1f} ms")
    print(f"corpus   : {positions} positions")
    print(f"KL       : mean {float(kl.mean()):.3e}, worst {float(kl.max()):.3e} nats")
    print(f"logits   : max |diff| {float((reference - candidate).abs().max()):.3e} (largest |logit| {float(reference.abs().max()):.3e})")
    print(f"top-1    : {agree}/{positions} agree")
    print(f"time     : {time.time() - started:.2f} s")
    return 0


def command_bench_continuous(args) -> int:
    """Continuous batching as the reference's ``bench continuous`` runs it (apps/cli/main.cpp:1451-1644):
    ``requests`` requests through ``sequences`` live slots, greedy, ``tokens`` new tokens each.  With one
    prompt for all (the default) the transcripts must be identical whatever shared a step with what; with
    ``--prompt-max`` the prompts differ in length and content and only the rate is reported."""
    import random
    import time
    import torch
    if min(args.requests, args.tokens, args.sequences, args.prompt_tokens) <= 0:
        raise UsageError("bench continuous: requests, tokens, sequences and prompt-tokens must be positive")
    if args.prompt_max is not None and args.prompt_max < args.prompt_tokens:
        raise UsageError("bench continuous: --prompt-max must not be below --prompt-tokens")
    args.max_requests = args.sequences
    started = time.time()
    engine = _engine_from(args)
    load_seconds = time.time() - started
    longest = args.prompt_max or args.prompt_tokens
    if longest + args.tokens > engine.max_model_len:
        raise UsageError(f"bench continuous: prompt-tokens + tokens ({longest + args.tokens}) exceeds the "
                         f"{engine.max_model_len}-token context")
    rnd = random.Random(1234)
    vocab = engine.spec.vocab_size
    seed_prompt = [rnd.randrange(vocab) for _ in range(args.prompt_tokens)]
    prompts = []
    for _ in range(args.requests):
        if args.prompt_max is None:
            prompts.append(seed_prompt)
        else:
            prompts.append([rnd.randrange(vocab) for _ in range(rnd.randint(args.prompt_tokens, args.prompt_max))])
    ids = [engine.add_request(p, args.tokens) for p in prompts]
    torch.cuda.synchronize()
    begin = time.time()
    done = {}
    steps = 0
    while engine.has_unfinished():
        for request in engine.step():
            done[request.id] = request
        steps += 1
    torch.cuda.synchronize()
    seconds = time.time() - begin
    transcripts = [done[i].output for i in ids]
    generated = sum(len(t) for t in transcripts)
    prompt_total = sum(len(p) for p in prompts)
    stats = engine.stats()
    print(f"continuous: {args.requests} requests, {args.sequences} slots, {args.tokens} tokens")
    print(f"load      : {load_seconds * 1e3:.1f} ms")
    print(f"wall      : {seconds:.3f} s in {steps} steps ({stats['preemptions']} preemptions)")
    print(f"prompts   : {prompt_total} tokens, lengths {min(map(len, prompts))}..{max(map(len, prompts))}")
    print(f"decode    : {generated} tokens, {generated / seconds:.2f} t/s aggregate "
          f"({(generated + prompt_total) / seconds:.1f} t/s with the prompts)")
    if args.prompt_max is None:
        identical = all(t == transcripts[0] for t in transcripts)
        if identical:
            print("state     : independent (all transcripts identical)")
        elif engine.dtype == torch.float32:
            print("state     : LEAKED - transcripts differ")
        else:
            print("state     : transcripts differ (bfloat16 rounds differently in different batches and may flip a "
                  "near-tie; --dtype float32 is exact)")
        print("first     : " + " ".join(str(t) for t in transcripts[0][:32]) + (" ..." if len(transcripts[0]) > 32 else ""))
        return 0 if identical or engine.dtype != torch.float32 else 1
    print("state     : not compared (prompts differ)")
    return 0


def command_bench(args) -> int:
    from .bench_tools import bench_decode, bench_prefill
    if args.what == "continuous":
        return command_bench_continuous(args)
    engine = _engine_from(args)
    if args.what == "mixed":
        from .bench_tools import bench_mixed
        result = bench_mixed(engine, args.batch, args.prompt_len, args.portion, repeat=args.repeat)
        print(f"mixed    : {result['decodes']} single tokens at context {args.prompt_len} beside a portion of "
              f"{result['portion']} tokens: {result['ms']:.3f} ms/step ({result['tok_s']:.1f} tok/s)")
    elif args.what == "prefill":
        result = bench_prefill(engine, args.prompt_len, repeat=args.repeat, sustain_seconds=1.0)
        print(f"prefill  : {result['tokens']} tokens in {result['ms']:.2f} ms ({result['tok_s']:.1f} tok/s), "
              f"{result['tflops']:.1f} TFLOP/s = {result['frac']:.3f} of {result['peak_tflops']:.0f} ({result['peak_source']})")
        print(f"           after a pause {result['burst_ms']:.2f} ms = {result['burst_frac']:.3f} of the burst peak; "
              f"sustained {result['sustained_ms']:.2f} ms = {result['sustained_frac']:.3f} of the sustained peak")
    else:
        result = bench_decode(engine, args.batch, args.prompt_len, steps=args.n)
        print(f"decode   : batch {args.batch} at context {args.prompt_len}: {result['ms_per_step']:.3f} ms/step "
              f"({result['tok_s']:.1f} tok/s), {result['gbs']:.0f} GB/s = {result['frac']:.3f} of "
              f"{result['peak_gbs']:.0f} ({result['peak_source']})")
    if args.timeline:
        from .bench_tools import step_timeline
        print("one step's time by kernel (each charged from the end of the kernel before it to its own end):")
        for row in step_timeline(engine, args.batch, args.prompt_len, args.what == "prefill",
                                 portion=args.portion if args.what == "mixed" else 0):
            print(f"  {row['us']:9.1f} us  {100 * row['share']:5.1f} %  x{row['launches']:<4d} {row['kernel']}")
    return 0


def command_make_random(args) -> int:
    from .weights.random_init import write_random_model
    with open(args.config, "r", encoding="utf-8") as handle:
        raw = json.load(handle)
    write_random_model(args.out, raw, args.seed, args.dtype)
    print(f"wrote    : {args.out}/config.json and model.safetensors (seed {args.seed}, {args.dtype})")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    parser = build_parser()
    try:
        args = parser.parse_args(argv)
        if args.command is None:
            parser.print_help()
            return 0
        if args.command == "version":
            print(f"aegean-tge b200 {__version__}")
            return 0
        if args.command == "info":
            return command_info(args)
        if args.command == "plan":
            return command_plan(args)
        if args.command == "generate":
            return command_generate(args)
        if args.command == "bench":
            return command_bench(args)
        if args.command == "fidelity":
            return command_fidelity(args)
        if args.command == "make-random":
            return command_make_random(args)
        if args.command == "replay":
            from .engine.replay import main as replay_main
            return replay_main(["--model", args.model, "--dtype", args.dtype, "--out", args.out,
                                "--max-tokens", str(args.max_tokens)] + (["--trace", args.trace] if args.trace else []))
        raise UsageError(f"unknown command {args.command}")
    except SystemExit as stop:          # argparse prints --help itself and leaves through here
        return int(stop.code or 0)
    except UsageError as error:
        print(str(error), file=sys.stderr)
        return 2
    except Exception as error:  # load and run-time failures
        print(f"tge: {type(error).__name__}: {error}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
