"""The generic decoder: built from a ModelSpec, knows no architecture.

It owns the parts (embedding, one block per layer, final norm, head), says
which tensors it expects from a checkpoint, tells the cache manager what each
layer keeps, and runs one step: embed the step's tokens, run the layers in
the order the spec's ``schedule`` gives, gather the wanted rows, norm them and
project them to float32 logits (the reference computes the head for the last
row only in prefill, src/models/qwen2.cpp:2494-2499, and for every row in a
mixed batch, :1935-1945; here the caller says which rows).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.manager import CacheManager
from ..config.model_spec import ModelSpec, PartSpec
from ..parts.base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, Block, BuildEnv, LayerCache,
                          ParamSpec, Part, StepContext, build_part)


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        spec.validate()
        self.spec = spec
        self.env = env
        self.embedding = build_part(EMBEDDINGS, spec.embedding, env)
        self.final_norm = build_part(NORMS, spec.final_norm, env)
        self.head = build_part(HEADS, spec.head, env)
        self.blocks: List[Block] = []
        for layer in spec.layers:
            mixer = build_part(MIXERS, layer.mixer, env)
            ffn = build_part(FEED_FORWARDS, layer.feed_forward, env)
            norm1 = build_part(NORMS, layer.mixer_norm, env)
            norm2 = build_part(NORMS, layer.ffn_norm, env)
            self.blocks.append(BLOCKS.get(layer.block)(mixer, ffn, norm1, norm2, env))
        self.layer_caches: List[LayerCache] = [LayerCache() for _ in spec.layers]
        # single-token steps may be replayed from a CUDA graph only if every part says so
        self.graph_safe = all(part.graph_safe for _where, part, _spec in self.named_parts())

    # -- parameters -----------------------------------------------------------
    def named_parts(self) -> List[Tuple[str, Part, PartSpec]]:
        out: List[Tuple[str, Part, PartSpec]] = [("embedding", self.embedding, self.spec.embedding),
                                                 ("final_norm", self.final_norm, self.spec.final_norm),
                                                 ("head", self.head, self.spec.head)]
        for index, (block, layer) in enumerate(zip(self.blocks, self.spec.layers)):
            out.append((f"layers[{index}].mixer_norm", block.mixer_norm, layer.mixer_norm))
            out.append((f"layers[{index}].mixer", block.mixer, layer.mixer))
            out.append((f"layers[{index}].ffn_norm", block.ffn_norm, layer.ffn_norm))
            out.append((f"layers[{index}].feed_forward", block.feed_forward, layer.feed_forward))
        return out

    def manifest(self) -> Dict[str, Tuple[ParamSpec, str]]:
        """Checkpoint tensor name -> (what it must look like, where it is used)."""
        wanted: Dict[str, Tuple[ParamSpec, str]] = {}
        for where, part, spec in self.named_parts():
            for local, param in part.param_specs().items():
                if local not in spec.weights:
                    raise ValueError(f"{where}: the model spec names no tensor for parameter '{local}'")
                name = spec.weights[local]
                if name in wanted and (wanted[name][0].shape != param.shape or wanted[name][0].role != param.role):
                    raise ValueError(f"tensor '{name}' is wanted as {wanted[name][0]} by {wanted[name][1]} "
                                     f"and as {param} by {where}.{local}")
                wanted.setdefault(name, (param, f"{where}.{local}"))
        return wanted

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hands every part its parameters (``tensors`` is keyed by checkpoint name)."""
        for where, part, spec in self.named_parts():
            mine = {}
            for local, param in part.param_specs().items():
                name = spec.weights[local]
                if name in tensors:
                    mine[local] = tensors[name]
                elif not param.optional:
                    raise KeyError(f"{where}.{local}: tensor '{name}' was not loaded")
            if mine or part.param_specs():
                part.load(mine)

    def step_param_bytes(self) -> int:
        """Bytes of parameters one step reads: every part once per visit, the embedding rows not counted."""
        total = self.final_norm.param_bytes() + self.head.param_bytes()
        for index in self.spec.schedule:
            total += sum(part.param_bytes() for part in self.blocks[index].parts().values())
        return total

    # -- cache ----------------------------------------------------------------
    def declare_cache(self, manager: CacheManager) -> None:
        for index, (block, layer) in enumerate(zip(self.blocks, self.spec.layers)):
            if layer.cache_from is None:
                manager.add_layer(index, block.mixer.cache_spec(), block.mixer.state_spec())
            else:
                manager.add_layer(index, None, block.mixer.state_spec())

    def attach_cache(self, manager: CacheManager) -> None:
        self.layer_caches = [manager.layer_cache(index, source=layer.cache_from)
                             for index, layer in enumerate(self.spec.layers)]

    def cache_bytes_per_token(self) -> int:
        """Bytes of paged cache one token adds, over all layers that keep one (their ``cache_spec``)."""
        total = 0
        for block, layer in zip(self.blocks, self.spec.layers):
            spec = block.mixer.cache_spec() if layer.cache_from is None else None
            if spec is not None:
                for _name, shape in spec.entries:
                    count = 1
                    for extent in shape:
                        count *= int(extent)
                    total += count * self.env.dtype.itemsize
        return total

    def weight_bytes(self) -> int:
        """Bytes of all parameters on the device, a tensor that two parts share counted once."""
        total = 0
        for param, _where in self.manifest().values():
            count = 1
            for extent in param.shape:
                count *= int(extent)
            total += count * (self.env.dtype.itemsize if param.role == "matrix" else 4)
        return total

    def step_flops(self, tokens: int, pairs: float, rows: int) -> float:
        """Floating-point operations of one step: ``tokens`` tokens through every scheduled layer, their queries
        meeting ``pairs`` (query, key) pairs per layer, and ``rows`` rows of logits."""
        total = self.head.flops(rows, 0.0)
        for index in self.spec.schedule:
            total += sum(part.flops(tokens, pairs) for part in self.blocks[index].parts().values())
        return total

    # -- one step -------------------------------------------------------------
    def forward(self, ctx: StepContext, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs the step's tokens through all layers; returns float32 logits [R, vocab] of the wanted rows."""
        x = self.embedding.forward(ctx.token_ids)
        schedule = self.spec.schedule
        h = None                              # the next layer's first norm, when the previous layer produced it
        for step, index in enumerate(schedule):
            after = self.blocks[schedule[step + 1]] if step + 1 < len(schedule) else None
            following = after.mixer_norm if after is not None else None
            block = self.blocks[index]
            more = ({"next_takes_deferred": after is not None and after.mixer.takes_deferred_rows}
                    if block.passes_deferred_rows else {})
            h = block.forward(x, ctx, self.layer_caches[index], h=h, next_norm=following, **more)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        h = self.final_norm.forward(x, rows=logit_rows)
        return self.head.forward(h)
