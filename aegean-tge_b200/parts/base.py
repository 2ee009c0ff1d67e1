"""Interfaces of the parts a layer is put together from, and their registries.

Five kinds of part exist: norm, position encoding, mixer, feed-forward, and
the block that arranges them.  Each kind has a registry from a name to a
class; a ``PartSpec`` names the kind and carries the sizes and constants.  A
part sees only its own ``PartSpec`` and the :class:`BuildEnv`; it never learns
which model it belongs to.

What every part does:

* ``param_specs()`` declares its parameters by local name (shape and role);
* ``load(tensors)`` receives them, already on the device and in the dtype the
  role asks for, and may repack them (fuse q/k/v rows, interleave gate/up);
* its ``forward`` runs on a flat batch of tokens ``[T, ...]`` described by a
  :class:`StepContext`.

A mixer additionally declares what it keeps between steps: paged per-token
cache (``cache_spec``) and/or fixed-size per-request state (``state_spec``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple, Type

import torch

from ..config.model_spec import PartSpec


# ----------------------------------------------------------------------------
# declarations
# ----------------------------------------------------------------------------
@dataclass(frozen=True)
class ParamSpec:
    """One parameter of a part.

    role "matrix": operand of a matrix product or an embedding table; held in
    the run dtype (bfloat16 or float32).  role "vector": norm weight or bias;
    always held in float32 (a vector stored in 32-bit stays so, one stored in
    bfloat16 is widened exactly).  role "table": integers, held as int32.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclass(frozen=True)
class PagedCacheSpec:
    """Per-token cache a mixer needs, in pages.

    ``entries`` are the tensors kept per token (name -> trailing shape), for
    attention ``{"k": (kv_heads, head_dim), "v": (kv_heads, head_dim)}``.
    ``window`` is None when every earlier token stays readable, else the
    number of most recent tokens (the current one included) a query may read;
    pages wholly behind the window are given back.
    """

    entries: Tuple[Tuple[str, Tuple[int, ...]], ...]
    window: Optional[int] = None

    def group_key(self) -> Tuple:
        return (self.entries, self.window)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state a mixer keeps: name -> shape, float32."""

    entries: Tuple[Tuple[str, Tuple[int, ...]], ...]


@dataclass
class BuildEnv:
    """What a part may know about its surroundings when it is built."""

    dtype: torch.dtype                 # torch.bfloat16 or torch.float32
    device: torch.device
    hidden_size: int
    max_positions: int
    page_size: int
    ops: Any                           # the kernel bindings (aegean_tge_b200.ops)


@dataclass
class LayerCache:
    """The storage one layer's mixer reads and writes during a step."""

    paged: Dict[str, torch.Tensor] = field(default_factory=dict)   # name -> [pages, ...]
    group: Optional[int] = None                                    # index of its page group
    state: Dict[str, torch.Tensor] = field(default_factory=dict)   # name -> [slots, ...]
    owner: bool = True                                             # False: reads another layer's cache, stores nothing


@dataclass
class StepContext:
    """Device-side description of one step's batch.  All index tensors int32.

    A step holds ``num_seqs`` portions (one per request in the step), laid
    out one after another in the flat token dimension.
    """

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T] absolute position of each token
    seq_of_token: torch.Tensor         # [T] which portion a token belongs to
    q_start: torch.Tensor              # [S+1] first token of each portion
    start_pos: torch.Tensor            # [S] position of a portion's first token
    ctx_len: torch.Tensor              # [S] tokens the request holds after this step
    slots: torch.Tensor                # [S] per-request state slot
    block_tables: List[torch.Tensor]   # per page group: [S, max_pages] physical page ids
    max_q_len: int                     # host copies, for launch geometry
    max_ctx_len: int                   # an upper bound (launch geometry); contexts may be shorter
    typical_ctx_len: int = 0           # what contexts are expected to be (0: the bound); tunes splitting only
    host_q_lens: List[int] = field(default_factory=list)
    host_start_pos: List[int] = field(default_factory=list)
    host_slots: List[int] = field(default_factory=list)
    attn_split_tokens: int = 0         # 0 = let the kernel wrapper decide
    decode_prefix: int = 0             # in a step with longer portions: how many leading portions are single tokens
    scratch: Dict[str, Any] = field(default_factory=dict)


# ----------------------------------------------------------------------------
# part base classes
# ----------------------------------------------------------------------------
class Part:
    kind_name = "part"
    # True when ``forward`` only launches kernels that read the step's device arrays: nothing taken from the
    # step's host-side values (lengths, slots), no synchronisation, no allocation that depends on the data.
    # Steps of single tokens are then captured once into a CUDA graph and replayed; one part that leaves
    # this False makes the whole model run eagerly.
    graph_safe = False
    # Rows that a fused product and norm hands on may lack the norm's factor (``ops.DeferredRows``), which
    # saves the kernel that makes them a whole-row reduction.  A mixer or feed-forward whose ``forward_add``
    # accepts ``defer=True`` and passes it to ``ops.linear_add_norm`` sets ``can_defer_norm``; one whose first
    # use of ``h`` is ``ops.linear`` or ``ops.linear_qkv_rope_store`` (which apply the factor) sets
    # ``takes_deferred_rows``.  Both False: the part only ever sees plain tensors.
    can_defer_norm = False
    takes_deferred_rows = False

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env
        self.ops = env.ops

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no parameters")

    def param_bytes(self) -> int:
        """Bytes this part reads from its parameters in one step (for the roofline and the planner): every
        declared parameter once, matrices in the run dtype, vectors in float32, tables in int32.  It needs
        no loaded weights."""
        total = 0
        for param in self.param_specs().values():
            count = 1
            for extent in param.shape:
                count *= int(extent)
            total += count * (self.env.dtype.itemsize if param.role == "matrix" else 4)
        return total

    def flops(self, tokens: int, pairs: float) -> float:
        """Floating-point operations of one step of ``tokens`` tokens whose queries meet ``pairs`` (query, key)
        pairs in all (a whole prompt of T tokens: T (T + 1) / 2), a multiply-add counted as two.  Parts that
        only move or scale data report 0."""
        return 0.0


class Norm(Part):
    """``forward(x, rows=None)``: x float32 [T, H] -> run dtype [T or R, H]."""

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def fusable(self) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight, eps) if this is a plain RMSNorm that a product's epilogue kernel may apply, else None."""
        return None


class PositionEncoding(Part):
    """Rotates or shifts queries and keys by position.

    ``apply(q, k, positions)`` works in place on ``q [T, heads, head_dim]``
    and ``k [T, kv_heads, head_dim]`` views.  A position encoding that the
    fused rotate-and-store kernel knows returns its tables from
    ``rotary_tables()``; others return None and are applied on their own.
    """

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request."""

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """h: run dtype [T, H] (already normed) -> [T, H] to be added to the stream."""
        raise NotImplementedError

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: LayerCache,
                    next_norm: Optional["Norm"] = None) -> Optional[torch.Tensor]:
        """Adds the mixer's output to the float32 stream ``x`` in place.

        The default adds ``forward``'s result with the add kernel; a mixer
        whose last product can add in its epilogue overrides this.  ``next_norm``
        is the norm that will be applied to ``x`` next: a mixer that can apply it
        in the same kernel returns the normed rows, everyone else returns None
        and the caller runs the norm itself.
        """
        self.ops.add_to_stream(x, self.forward(h, ctx, cache))
        return None


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext,
                    next_norm: Optional["Norm"] = None) -> Optional[torch.Tensor]:
        """As ``Mixer.forward_add``: adds into ``x``; may return ``next_norm(x)`` if it computed it."""
        self.ops.add_to_stream(x, self.forward(h, ctx))
        return None


class Block:
    """Arrangement of one layer's parts around the residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm,
                 env: BuildEnv):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm
        self.env = env

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache, h: Optional[torch.Tensor] = None,
                next_norm: Optional[Norm] = None) -> Optional[torch.Tensor]:
        """Runs the layer on the stream ``x`` in place.

        ``h``: ``mixer_norm(x)`` if the previous layer already computed it.  ``next_norm``: the norm the
        next layer will apply to ``x`` first; the block may return its result (else None).  A block that
        sets ``passes_deferred_rows`` is also given ``next_takes_deferred``: whether the next layer's mixer
        takes rows without their norm factor.
        """
        raise NotImplementedError

    passes_deferred_rows = False

    def parts(self) -> Dict[str, Part]:
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "feed_forward": self.feed_forward}


# ----------------------------------------------------------------------------
# registries
# ----------------------------------------------------------------------------
class Registry:
    def __init__(self, what: str):
        self.what = what
        self._classes: Dict[str, Any] = {}

    def register(self, name: str) -> Callable[[Any], Any]:
        def wrap(cls: Any) -> Any:
            if name in self._classes and self._classes[name] is not cls:
                raise ValueError(f"{self.what} '{name}' is already registered")
            self._classes[name] = cls
            return cls
        return wrap

    def unregister(self, name: str) -> None:
        self._classes.pop(name, None)

    def get(self, name: str) -> Any:
        if name not in self._classes:
            raise KeyError(f"no {self.what} named '{name}'; registered: {', '.join(sorted(self._classes))}")
        return self._classes[name]

    def names(self) -> Tuple[str, ...]:
        return tuple(sorted(self._classes))


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")


def build_part(registry: Registry, spec: PartSpec, env: BuildEnv) -> Part:
    return registry.get(spec.kind)(spec, env)
