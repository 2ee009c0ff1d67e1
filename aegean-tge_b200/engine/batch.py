"""One step's work as the caller states it, and its device-side description.

A step is a list of portions: for each request in the step its next tokens
(one token for a decoding request, any number for a prompt portion) and the
places among them whose logits are wanted.  The reference's nearest notion is
the row list ``(token, position, sequence)`` of ``forward_batch``
(src/models/qwen2.cpp:1613-1639); positions are not given here because the
cache knows how many tokens a request already holds.

The index arrays of a step (token ids, positions, portion of each token,
portion starts, start positions, context lengths, state slots, wanted rows,
one block table per cache group) are packed by the host runtime
(csrc/runtime.cpp: ``pack_step``) into one int32 buffer in pinned memory, which
is copied to the device once.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import runtime as _rt
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


def _int32(values: Sequence[int], what: str, request: Hashable) -> np.ndarray:
    try:
        return np.ascontiguousarray(values, dtype=np.int32)
    except (OverflowError, ValueError, TypeError) as error:
        raise ValueError(f"request {request!r}: {what} are not 32-bit integers ({error})") from None


class PortionArrays:
    """The portions of one step as the arrays the runtime's packer reads."""

    def __init__(self, cache, portions: Sequence[Portion]):
        count = len(portions)
        self.count = count
        self.requests = [p.request for p in portions]
        self.tokens = [_int32(p.tokens, "tokens", p.request) for p in portions]
        self.wants = [_int32(p.want, "wanted places", p.request) for p in portions]
        self.handles = (ctypes.c_int64 * count)(*[cache.handle_of(r, create=True) for r in self.requests])
        self.token_ptrs = (ctypes.c_void_p * count)(*[t.ctypes.data for t in self.tokens])
        self.token_counts = (ctypes.c_int * count)(*[t.size for t in self.tokens])
        self.want_ptrs = (ctypes.c_void_p * count)(*[w.ctypes.data for w in self.wants])
        self.want_counts = (ctypes.c_int * count)(*[w.size for w in self.wants])
        self.single_tokens = all(t.size == 1 for t in self.tokens)


def context_from_packed(dev: torch.Tensor, host: np.ndarray, layout: "_rt.StepLayout", groups: int,
                        max_ctx_len: Optional[int] = None, typical_ctx_len: int = 0) -> Tuple[StepContext, Optional[torch.Tensor]]:
    """Slices the packed device buffer into a :class:`StepContext`; host lists come from the host copy."""
    L = layout
    T, S, R = L.num_tokens, L.num_seqs, L.num_rows
    take = lambda begin, count: dev[begin:begin + count]
    q_start = host[L.q_start:L.q_start + S + 1]
    q_lens = np.diff(q_start)
    # decoding requests usually come first in a step (the scheduler plans running requests before new ones)
    longer = np.flatnonzero(q_lens != 1)
    decode_prefix = int(longer[0]) if longer.size else 0
    ctx = StepContext(
        num_tokens=T, num_seqs=S, token_ids=take(L.token_ids, T), positions=take(L.positions, T),
        seq_of_token=take(L.seq_of_token, T), q_start=take(L.q_start, S + 1), start_pos=take(L.start_pos, S),
        ctx_len=take(L.ctx_len, S), slots=take(L.slots, S),
        block_tables=[take(L.table[g], S * L.width[g]).view(S, L.width[g]) for g in range(groups)],
        max_q_len=L.max_q_len, max_ctx_len=L.max_ctx_len if max_ctx_len is None else max_ctx_len,
        typical_ctx_len=typical_ctx_len, decode_prefix=decode_prefix, host_q_lens=q_lens.tolist(),
        host_start_pos=host[L.start_pos:L.start_pos + S].tolist(), host_slots=host[L.slots:L.slots + S].tolist())
    rows = take(L.logit_rows, R) if R else None
    return ctx, rows
