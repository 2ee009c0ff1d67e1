"""Turns logits rows into token ids on the device.

Greedy and temperature sampling follow src/models/sampling.cpp:183-228:
the first maximal index when the temperature is not positive; otherwise
``exp((z - max) / T)`` summed in index order, a uniform draw scaled by the
sum, and the first index at which the running remainder drops to zero or
below.  Each request owns its xorshift32 state on the host; one draw is
consumed per sampled token and passed to the kernel.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .params import SamplingParams, XorShift32


class Sampler:
    def __init__(self, ops, device: torch.device):
        self.ops = ops
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[XorShift32],
               histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """One token id per row of ``logits`` (float32 [R, vocab])."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(rngs):
            raise ValueError("sampler: one SamplingParams and one generator per logits row")
        temperatures, uniforms = [], []
        for p, rng in zip(params, rngs):
            p.validate()
            if p.has_cuts or p.has_penalty:
                raise NotImplementedError("sampler: top-k / top-p / min-p / repeat penalty are not built yet")
            temperatures.append(max(float(p.temperature), 0.0))
            uniforms.append(0.0 if p.greedy else rng.next_uniform())
        host = torch.tensor([temperatures, uniforms], dtype=torch.float32)
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        ids = self.ops.sample(logits, dev[0], dev[1])
        return ids.cpu().tolist()
