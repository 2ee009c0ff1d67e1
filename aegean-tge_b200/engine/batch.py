"""One step's work as the caller states it, and its device-side description.

A step is a list of portions: for each request in the step its next tokens
(one token for a decoding request, any number for a prompt portion) and the
places among them whose logits are wanted.  The reference's nearest notion is
the row list ``(token, position, sequence)`` of ``forward_batch``
(src/models/qwen2.cpp:1613-1639); positions are not given here because the
cache knows how many tokens a request already holds.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Sequence

import torch

from ..parts.base import StepContext


@dataclass
class Portion:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into ``tokens``

    def validate(self, vocab_size: int) -> None:
        if len(self.tokens) == 0:
            raise ValueError(f"request {self.request!r}: a portion needs at least one token")
        for token in self.tokens:
            if not 0 <= int(token) < vocab_size:
                raise ValueError(f"request {self.request!r}: token {token} is outside the vocabulary of {vocab_size}")
        for place in self.want:
            if not 0 <= int(place) < len(self.tokens):
                raise ValueError(f"request {self.request!r}: wanted place {place} is outside its {len(self.tokens)} tokens")


def build_context(portions: Sequence[Portion], start_positions: Sequence[int], slots: Sequence[int],
                  block_tables: Sequence[Sequence[Sequence[int]]], device: torch.device):
    """Packs the step's index arrays into one pinned buffer, copies it once, and slices it.

    Returns (StepContext, logit_rows tensor or None).
    """
    num_seqs = len(portions)
    lengths = [len(p.tokens) for p in portions]
    total = sum(lengths)
    token_ids: List[int] = []
    positions: List[int] = []
    seq_of_token: List[int] = []
    q_start = [0]
    logit_rows: List[int] = []
    for index, (portion, start) in enumerate(zip(portions, start_positions)):
        base = q_start[-1]
        token_ids.extend(int(t) for t in portion.tokens)
        positions.extend(range(start, start + lengths[index]))
        seq_of_token.extend([index] * lengths[index])
        logit_rows.extend(base + int(w) for w in portion.want)
        q_start.append(base + lengths[index])
    ctx_len = [s + n for s, n in zip(start_positions, lengths)]
    widths = [len(table[0]) if table else 1 for table in block_tables]
    flat: List[int] = []
    offsets = {}

    def put(name: str, values: Sequence[int]) -> None:
        offsets[name] = (len(flat), len(values))
        flat.extend(values)

    put("token_ids", token_ids)
    put("positions", positions)
    put("seq_of_token", seq_of_token)
    put("q_start", q_start)
    put("start_pos", list(start_positions))
    put("ctx_len", ctx_len)
    put("slots", list(slots))
    put("logit_rows", logit_rows)
    for g, table in enumerate(block_tables):
        put(f"table{g}", [page for row in table for page in row])
    host = torch.tensor(flat, dtype=torch.int32)
    if device.type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)

    def take(name: str) -> torch.Tensor:
        begin, count = offsets[name]
        return dev[begin:begin + count]

    ctx = StepContext(
        num_tokens=total, num_seqs=num_seqs, token_ids=take("token_ids"), positions=take("positions"),
        seq_of_token=take("seq_of_token"), q_start=take("q_start"), start_pos=take("start_pos"),
        ctx_len=take("ctx_len"), slots=take("slots"),
        block_tables=[take(f"table{g}").view(num_seqs, widths[g]) for g in range(len(block_tables))],
        max_q_len=max(lengths), max_ctx_len=max(ctx_len), host_q_lens=lengths,
        host_start_pos=list(start_positions), host_slots=list(slots))
    rows = take("logit_rows") if logit_rows else None
    return ctx, rows, host.numel() * 4
