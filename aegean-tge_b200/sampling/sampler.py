"""Turns logits rows into token ids on the device.

Follows src/models/sampling.cpp:183-410: scores are the logits with the
repetition penalty applied (each distinct token of the recent history window
once); a non-positive temperature takes the first maximal index; otherwise
``exp((z - max) / T)``, the top-k / min-p / top-p cuts over candidates ordered
by probability, a uniform draw scaled by the kept mass, and the first
candidate at which the running remainder drops to zero or below.  Each request
owns its xorshift32 state on the host; one draw is consumed per sampled token
(none for greedy rows) and passed to the kernel.  Rows without cuts take the
kernel that needs no sort.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .params import SamplingParams, XorShift32


class Sampler:
    def __init__(self, ops, device: torch.device):
        self.ops = ops
        self.device = device
        self._zeros = {}            # rows -> float32 zeros [2, rows] on the device (greedy: temperature 0, no draw)
        self._pinned = {}           # rows -> ring of pinned int32 buffers for ids on their way to the host

    def _to_device(self, values, dtype) -> torch.Tensor:
        host = torch.tensor(values, dtype=dtype)
        if self.device.type == "cuda":
            host = host.pin_memory()
        return host.to(self.device, non_blocking=True)

    @staticmethod
    def stays_on_device(params: Sequence[SamplingParams]) -> bool:
        """True when no row needs its token history (the repetition penalty): greedy rows, temperature draws and
        the top-k / top-p / min-p cuts are all settled by kernels that read only what is on the device."""
        return all(not p.has_penalty for p in params)

    def _draw(self, scores: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[XorShift32]) -> torch.Tensor:
        """Token ids on the device for rows of scores: one kernel for all rows, one more for the rows with cuts."""
        rows = scores.shape[0]
        if all(p.greedy for p in params):
            if rows not in self._zeros:
                self._zeros[rows] = torch.zeros((2, rows), dtype=torch.float32, device=self.device)
            floats = self._zeros[rows]
            return self.ops.sample(scores, floats[0], floats[1])
        cuts = any(p.has_cuts and not p.greedy for p in params)
        table = [[max(float(p.temperature), 0.0) for p in params],
                 [0.0 if p.greedy else rng.next_uniform() for p, rng in zip(params, rngs)]]
        if cuts:
            off = lambda p: p.greedy or not p.has_cuts
            table.append([1.0 if off(p) else float(p.top_p) for p in params])
            table.append([0.0 if off(p) else float(p.min_p) for p in params])
        floats = self._to_device(table, torch.float32)
        ids = self.ops.sample(scores, floats[0], floats[1])
        if cuts:
            top_k = self._to_device([0 if p.greedy or not p.has_cuts else int(p.top_k) for p in params], torch.int32)
            self.ops.sample_cuts(scores, floats[0], top_k, floats[2], floats[3], floats[1], out=ids)
        return ids

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[XorShift32]):
        """Like :meth:`sample` for rows that stay on the device, without waiting: returns the ids on the
        device, their copy in pinned host memory, and the event after which that copy is complete."""
        rows = logits.shape[0]
        ids = self._draw(logits, params, rngs)
        turn = self._turn = (getattr(self, "_turn", -1) + 1) % 4
        if rows not in self._pinned:
            self._pinned[rows] = [torch.empty(rows, dtype=torch.int32).pin_memory() for _ in range(4)]
        host = self._pinned[rows][turn]
        host.copy_(ids, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return ids, host, event

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[XorShift32],
               histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """One token id per row of ``logits`` (float32 [R, vocab]).

        ``histories`` (prompt plus generated tokens of each row's request) feeds only the penalty.
        """
        rows = logits.shape[0]
        if rows != len(params) or rows != len(rngs):
            raise ValueError("sampler: one SamplingParams and one generator per logits row")
        for p in params:
            p.validate()
        scores = logits
        if any(p.has_penalty for p in params):
            if histories is None:
                raise ValueError("sampler: a repetition penalty needs the token histories")
            flat: List[int] = []
            starts = [0]
            for p, history in zip(params, histories):
                if p.has_penalty:
                    window = history[-p.penalty_window:] if p.penalty_window > 0 else history
                    flat.extend(int(t) for t in window)
                starts.append(len(flat))
            scores = self.ops.apply_penalty(logits, self._to_device(flat or [0], torch.int32),
                                            self._to_device(starts, torch.int32),
                                            self._to_device([float(p.repeat_penalty) for p in params], torch.float32))
        return self._draw(scores, params, rngs).cpu().tolist()
