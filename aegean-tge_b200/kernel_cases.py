"""Runs one kernel on one workload a few times and prints its time: the unit that profiles are taken of.

    python -m aegean_tge_b200.kernel_cases gemm --m 2048 --n 9472 --k 3584 --epilogue swiglu
    python -m aegean_tge_b200.kernel_cases attention --batch 64 --context 2048 --q-len 1
    python -m aegean_tge_b200.kernel_cases attention --batch 1 --context 2048 --q-len 2048
    python -m aegean_tge_b200.kernel_cases fill --elements 545000000
    python -m aegean_tge_b200.kernel_cases sample --rows 8 --top-k 50 --top-p 0.9

Weights are rotated between launches so that a launch never finds them in L2; attention reads a
freshly shuffled page table.  Sizes default to the Qwen2.5-7B layer shapes.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import ops

EPILOGUES = {"store": ops.GEMM_STORE, "f32": ops.GEMM_STORE_F32, "add": ops.GEMM_ADD_F32, "swiglu": ops.GEMM_SWIGLU}


def run_gemm(args) -> None:
    dev = "cuda:0"
    epilogue = EPILOGUES[args.epilogue]
    ops.set_pair_gemm(args.pair)
    copies = max(2, int(300e6 // (args.n * args.k * 2)) + 1)
    weights = [torch.randn(args.n, args.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(args.m, args.k, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(args.m, args.n, device=dev, dtype=torch.float32) if args.epilogue in ("f32", "add") else None
    times = []
    for i in range(args.repeat):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        ops.linear(x, weights[i % copies], None, epilogue, out=out)
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop) * 1e3)
    us = sorted(times[2:])[len(times[2:]) // 2]
    print(f"gemm M={args.m} N={args.n} K={args.k} {args.epilogue}: {us:.1f} us, "
          f"{2 * args.m * args.n * args.k / us / 1e6:.1f} TFLOP/s, weights at {args.n * args.k * 2 / us / 1e3:.0f} GB/s")


def run_attention(args) -> None:
    dev = "cuda:0"
    heads, kv_heads, head_dim, page = args.heads, args.kv_heads, args.head_dim, args.page_size
    batch, context, q_len = args.batch, args.context, args.q_len
    pages_per = -(-context // page)
    num_pages = batch * pages_per + 1
    k = torch.randn(num_pages, kv_heads, page, head_dim, device=dev, dtype=torch.bfloat16)
    v = torch.randn(num_pages, kv_heads, page, head_dim, device=dev, dtype=torch.bfloat16)
    table = torch.randperm(batch * pages_per, device=dev).to(torch.int32).view(batch, pages_per)
    start_position = context - q_len
    positions = (torch.arange(q_len, device=dev, dtype=torch.int32)[None, :] + start_position).repeat(batch, 1).reshape(-1)
    seq_of = torch.arange(batch, device=dev, dtype=torch.int32).repeat_interleave(q_len).contiguous()
    q_start = (torch.arange(batch + 1, device=dev, dtype=torch.int32) * q_len).contiguous()
    start_pos = torch.full((batch,), start_position, device=dev, dtype=torch.int32)
    q = torch.randn(batch * q_len, heads * head_dim, device=dev, dtype=torch.bfloat16)
    positions = positions.contiguous()
    run = lambda: ops.attention(q, k, v, table, q_start, start_pos, positions, seq_of, batch, q_len, context, heads,
                                kv_heads, head_dim, 1.0 / math.sqrt(head_dim), split_tokens=args.split)
    for _ in range(3):
        run()
    # launches queued back to back between two events: the device time of one, without the host's launch cost
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.repeat):
        run()
    stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1e3 / args.repeat
    kv_bytes = batch * context * kv_heads * head_dim * 2 * 2
    flops = 4.0 * heads * head_dim * batch * q_len * (start_position + (q_len + 1) / 2.0)
    print(f"attention batch={batch} context={context} q_len={q_len}: {us:.1f} us (pages of {page}), "
          f"K/V {kv_bytes / 1e6:.1f} MB at {kv_bytes / us / 1e3:.0f} GB/s, {flops / us / 1e6:.1f} TFLOP/s")


def run_fill(args) -> None:
    """The random-weights kernel writing one bfloat16 tensor (the default: an embedding table of the 7B shape)."""
    from .weights import normal, random_tensor
    times = []
    for i in range(args.repeat):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        tensor = random_tensor(f"tensor.{i}", (args.elements,), normal(0.02), 0, torch.bfloat16, torch.device("cuda:0"))
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop) * 1e3)
        del tensor
    us = sorted(times[1:])[len(times[1:]) // 2]
    print(f"fill {args.elements} bfloat16 elements: {us:.1f} us, written at {args.elements * 2 / us / 1e3:.0f} GB/s")


def run_sample(args) -> None:
    """The sampling kernels on rows of scores as peaked as a language model's (a normal spread of ``--spread``)."""
    dev = "cuda:0"
    gen = torch.Generator(device=dev).manual_seed(3)
    scores = torch.randn(args.rows, args.vocab, generator=gen, device=dev) * args.spread
    temperature = torch.full((args.rows,), args.temperature, device=dev)
    uniform = torch.rand(args.rows, generator=gen, device=dev)
    top_k = torch.full((args.rows,), args.top_k, dtype=torch.int32, device=dev)
    top_p = torch.full((args.rows,), args.top_p, device=dev)
    min_p = torch.full((args.rows,), args.min_p, device=dev)
    cuts = args.top_k > 0 or args.top_p < 1.0 or args.min_p > 0.0
    run = (lambda: ops.sample_cuts(scores, temperature, top_k, top_p, min_p, uniform)) if cuts else \
          (lambda: ops.sample(scores, temperature, uniform))
    for _ in range(3):
        run()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.repeat):
        run()
    stop.record()
    torch.cuda.synchronize()
    print(f"sample rows={args.rows} vocab={args.vocab} temperature={args.temperature} top_k={args.top_k} top_p={args.top_p} min_p={args.min_p}: "
          f"{start.elapsed_time(stop) * 1e3 / args.repeat:.1f} us per call (with the host's launch cost)")


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="kernel_cases", description=__doc__.split("\n\n")[0])
    sub = parser.add_subparsers(dest="what", required=True)
    gemm = sub.add_parser("gemm")
    gemm.add_argument("--m", type=int, default=8)
    gemm.add_argument("--n", type=int, default=37888)
    gemm.add_argument("--k", type=int, default=3584)
    gemm.add_argument("--epilogue", choices=sorted(EPILOGUES), default="swiglu")
    gemm.add_argument("--repeat", type=int, default=8)
    gemm.add_argument("--pair", type=int, default=1, choices=[0, 1, 2],
                      help="two SMs on one tile: 0 never, 1 where its cost model says so (default), 2 always")
    attn = sub.add_parser("attention")
    attn.add_argument("--batch", type=int, default=8)
    attn.add_argument("--context", type=int, default=2048)
    attn.add_argument("--q-len", type=int, default=1)
    attn.add_argument("--heads", type=int, default=28)
    attn.add_argument("--kv-heads", type=int, default=4)
    attn.add_argument("--head-dim", type=int, default=128)
    attn.add_argument("--page-size", type=int, default=64)
    attn.add_argument("--split", type=int, default=0, help="keys per split (a multiple of 64); 0 lets the wrapper choose")
    attn.add_argument("--repeat", type=int, default=8)
    fill = sub.add_parser("fill")
    fill.add_argument("--elements", type=int, default=152064 * 3584)
    fill.add_argument("--repeat", type=int, default=5)
    sample = sub.add_parser("sample")
    sample.add_argument("--rows", type=int, default=8)
    sample.add_argument("--vocab", type=int, default=152064)
    sample.add_argument("--spread", type=float, default=3.0)
    sample.add_argument("--temperature", type=float, default=0.8, help="0: greedy")
    sample.add_argument("--top-k", type=int, default=0)
    sample.add_argument("--top-p", type=float, default=1.0)
    sample.add_argument("--min-p", type=float, default=0.0)
    sample.add_argument("--repeat", type=int, default=10)
    args = parser.parse_args(argv)
    if args.what == "gemm":
        run_gemm(args)
    elif args.what == "fill":
        run_fill(args)
    elif args.what == "sample":
        run_sample(args)
    else:
        run_attention(args)
    ops.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
