"""What every part is built from: the registries, the runtime (device and
precision), the description of one step's batch that parts receive, the cache
needs a mixer declares and the residual stream with its pending add.

A part never knows which model it is in.  It is built from a `PartSpec` (sizes
and constants as parameters, a prefix for its tensors), declares its tensors
with `tensors(spec)` and works on the rows it is handed.

Interfaces (duck-typed; the classes below marked "interface" document them):

  mixer         tensors(spec); __init__(spec, store, runtime); cache_need();
                forward(h [T,H], ctx: StepContext, cache: CacheBinding) -> delta
                optional: batch_annotations() -> [BatchAnnotation] (integer data about the
                batch that its kernels want packed with the step), shape_key(q_lens) -> hashable
                (what, beyond the step's sizes, decides which kernels it launches: part of a
                captured graph's key), advance_decode(ctx, cache) (move per-request state on
                after a device-side decoding step), graph_safe = True (launches depend on
                device-side metadata only)
  feed_forward  tensors(spec); __init__(spec, store, runtime); forward(h [T,H]) -> delta
                (delta is [T,H] in the compute dtype, or float32 partial sums [S,T,H]
                that the residual stream adds up in index order)
  norm          tensors(spec); __init__(spec, store, runtime);
                forward(x f32 [T,H], delta=None, rows=None) -> h (compute dtype)
  position      tensors(spec); __init__(spec, store, runtime); tables used by the mixer
  block         PARTS = {name: category}; __init__(**parts by those names), kept as attributes
                of those names (`mixer` is the part whose cache need the cache manager
                serves); forward(stream, ctx, cache)
  embedding     forward(ids) -> x f32 [T,H];   head  forward(stream, rows) -> logits f32
  gate          tensors(spec); __init__(spec, store, runtime); weight, bias (a projection of a
                sublayer's input whose sigmoid scales the sublayer's output); forward(h) -> pre
  injection     tensors(spec); __init__(spec, store, runtime); needs_embedding (bool);
                forward(stream, embedded) (changes the stream in front of a call of the order;
                `embedded` is the embedding's output, kept for the parts that ask for it)
  filter        tensors(spec); __init__(spec, store, runtime); state_need() -> StateNeed | None;
                forward(h [T,H], ctx, state) -> what a sublayer reads instead of h (it may keep
                its last inputs per request in `state`, the arena of the call's side state)
  scale         tensors(spec); __init__(spec, store, runtime); vector (float32 [H]): a learned
                scale, element by element, on a sublayer's output before it is added
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..config.spec import ConfigError, PartSpec
from ..kernels import ops

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head", "gate", "injection",
              "filter", "scale")
_REGISTRY: Dict[str, Dict[str, Any]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: Any) -> None:
    """Make `cls` buildable from a PartSpec of this `kind`."""
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")
    _REGISTRY[category][kind] = cls


def part_class(category: str, kind: str) -> Any:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY[category])) or "none"
        raise ConfigError(f"no {category} of kind {kind!r} is registered (registered: {known})") from None


def registered(category: str) -> List[str]:
    return sorted(_REGISTRY[category])


# --------------------------------------------------------------------------- #
@dataclass
class Runtime:
    """Where and in which precision a model runs.  `dtype` is the type of the
    matrix-product operands and of the cache: bfloat16 for serving, float32
    for the true 32-bit path.  The residual stream, norm gains, biases and
    logits are float32 in both."""

    device: torch.device
    dtype: torch.dtype

    def __post_init__(self):
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype is float32 or bfloat16, found {self.dtype}")

    def matrix(self, stored: torch.Tensor) -> torch.Tensor:
        """A matrix-product operand in the compute dtype, on the device."""
        return stored.to(device=self.device, dtype=self.dtype).contiguous()

    def vector(self, stored: torch.Tensor) -> torch.Tensor:
        """A gain or bias: widened to float32 (exact for bfloat16)."""
        return stored.to(device=self.device, dtype=torch.float32).contiguous()

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class KVNeed:
    """Keys and values per token: `kv_heads` x `head_dim` each (`planes` = 2), or one row of
    that size which the mixer reads as both (`planes` = 1).  With a `window`, only the last
    window + 1 positions are ever read, and pages wholly before them are given back.  With a
    `chunk`, a query reads the keys of its own chunk of that many positions (counted from 0) only,
    and pages wholly before the chunk of a request's next position are given back."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    planes: int = 2      # 2: keys and values; 1: one row a token that serves as both (a cached latent)
    chunk: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request (float32), zeroed when a request starts."""

    shape: Tuple[int, ...]


@dataclass(frozen=True)
class CacheNeed:
    """What one call of the order keeps per request: keys and values in pages (`kv`), the mixer's
    state (`state`) and, beside it, a state of whatever the layer's arrangement puts around the
    mixer (`side_state`: the last inputs of a convolution in front of it, say).  The two states are
    arenas of their own, so a mixer with a state needs to know nothing of the arrangement."""

    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None
    side_state: Optional[StateNeed] = None


@dataclass
class GroupView:
    """The batch as one cache group sees it: where each row's keys go and the
    block table of each request (logical block -> page, -1 where none)."""

    page_size: int
    slots: torch.Tensor          # [T] int32: page * page_size + offset
    block_table: torch.Tensor    # [R, max_blocks] int32


@dataclass
class StepContext:
    """One step's batch, as parts see it: T rows of R requests.  Row t belongs
    to request `row_req[t]` and sits at absolute position `pos[t]`; a request's
    rows are contiguous and in order (`q_start[r]` .. `q_start[r+1]`)."""

    n_tokens: int
    n_requests: int
    ids: torch.Tensor            # [T] int32
    pos: torch.Tensor            # [T] int32
    row_req: torch.Tensor        # [T] int32
    q_start: torch.Tensor        # [R + 1] int32
    kv_len: torch.Tensor         # [R] int32, tokens held after this step
    state_slot: torch.Tensor     # [R] int32
    groups: List[GroupView]
    # what the model's parts asked to have packed with the batch (`BatchAnnotation`), by key:
    # (the annotation's device view, the count its `fill` returned)
    views: Dict[str, Tuple[Any, int]] = field(default_factory=dict)
    # the block that runs after the one running now (None after the last): a part that asks for
    # memory ahead of its use may look at what that block starts with
    next_block: Any = None
    # host copies, for choosing kernels and for mixers that loop over requests
    q_lens: List[int] = field(default_factory=list)
    kv_lens: List[int] = field(default_factory=list)
    state_slots: List[int] = field(default_factory=list)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_kv_len(self) -> int:
        return max(self.kv_lens) if self.kv_lens else 0


class BatchAnnotation:
    """Interface.  Integer data about a step's batch that a part's kernels want beside the
    rows, positions and tables every part gets: a cut of the rows into tiles, a schedule, a
    sorted order.  A part lists its annotations in `batch_annotations()`; the engine packs each
    (once per `key`, however many layers ask) into the step's one metadata buffer, at an
    offset that depends on the step's capacities only, so a captured graph finds it again; the
    part reads `ctx.views[key]`.  The batch builder knows none of them.

      key                         a string; equal keys are one annotation
      capacity(T, R) -> int       int32 words for a step of up to T rows of R requests
      fill(out, first_rows, counts, starts, padded) -> int
                                  write the step's data into `out` (a zeroed numpy int32 array of
                                  `capacity` words) from the requests' spans: request r brings
                                  rows first_rows[r] .. + counts[r], the first at position
                                  starts[r] (numpy arrays).  `padded`: the step will be replayed
                                  from a graph, so the count returned must be the most the
                                  capacities allow.  The count travels with the view.
      view(words) -> Any          the device-side int32 words (a tensor of `capacity`) as the
                                  part wants to see them
    """

    key = ""

    def capacity(self, n_tokens: int, n_requests: int) -> int:
        raise NotImplementedError

    def fill(self, out, first_rows, counts, starts, padded: bool) -> int:
        raise NotImplementedError

    def view(self, words):
        return words


@dataclass
class CacheBinding:
    """What one call of a mixer may touch in the cache.  `writes` is False when
    the call reads the cache that an earlier call wrote."""

    group: int = -1                           # index into StepContext.groups, -1: no keys
    k_pool: Optional[torch.Tensor] = None     # [pages * page_size, kv_heads, head_dim]
    v_pool: Optional[torch.Tensor] = None     # None where the group keeps one row a token
    state: Optional[torch.Tensor] = None      # [state slots, *shape] float32
    side_state: Optional[torch.Tensor] = None # [state slots, *shape] float32: the arrangement's, not the mixer's
    writes: bool = True


# --------------------------------------------------------------------------- #
@dataclass
class GatedDelta:
    """A sublayer's output that is still to be scaled by its gate: (y + bias) * sigmoid(pre +
    pre_bias), with y [T, H] or float32 partial sums [S, T, H], pre float32 [T, H] (possibly a
    column slice of a wider product) and the biases float32 [H] or None."""

    y: torch.Tensor
    bias: Optional[torch.Tensor]
    pre: torch.Tensor
    pre_bias: Optional[torch.Tensor]


@dataclass
class ScaledTerms:
    """A mixer's output that is a sum of scaled terms (two mixers side by side): [(y, scale)], y
    [T, H] or float32 partial sums [S, T, H].  Whoever adds it to the stream, or norms it first,
    sums the terms in float32 on the way."""

    terms: List[Tuple[torch.Tensor, float]]


@dataclass
class VectorScaledTerms:
    """Sublayer outputs that are each multiplied, element by element, by a learned vector over the
    width before they are added: [(y, vector float32 [H])], y [T, H] or float32 partial sums
    [S, T, H] (a layer whose mixer and feed-forward read one norm adds both at once)."""

    terms: List[Tuple[torch.Tensor, torch.Tensor]]


class ResidualStream:
    """The residual sum, kept in float32.  A part's output is not added at once:
    it stays pending until the next norm, which adds it while it reads the row
    (one pass over memory instead of two).  A gated output (`add_gated`) stays pending with its
    gate unapplied: a norm that offers `forward_gated` applies the gate, adds and norms in one
    kernel; anything else that asks for `pending` gets the gated product as a float32 tensor."""

    def __init__(self, x: torch.Tensor):
        if x.dtype != torch.float32:
            raise ValueError("the residual stream is float32")
        self.x = x
        self._pending: Optional[torch.Tensor] = None
        self._gated: Optional[GatedDelta] = None
        self._normed = None      # (terms, norm): a sublayer's output that is normed before it is added
        self._scaled: Optional[VectorScaledTerms] = None     # outputs still to be scaled by their vectors

    @property
    def pending(self) -> Optional[torch.Tensor]:
        if self._normed is not None:
            (terms, post), self._normed = self._normed, None
            post.add_to(self.x, terms)            # in place: nothing stays pending
        if self._scaled is not None:
            scaled, self._scaled = self._scaled, None
            ops.scaled_add_norm(self.x, scaled.terms)      # in place as well
        if self._gated is not None:
            g, self._gated = self._gated, None
            self._pending = torch.empty(self.x.shape, dtype=torch.float32, device=self.x.device)
            ops.gated_delta(g.y, g.bias, g.pre, self._pending, pre_bias=g.pre_bias)
        return self._pending

    @pending.setter
    def pending(self, value: Optional[torch.Tensor]) -> None:
        self._pending, self._gated, self._normed, self._scaled = value, None, None, None

    def add(self, delta) -> None:
        self.flush()
        if isinstance(delta, ScaledTerms):
            summed = torch.empty(self.x.shape, dtype=torch.float32, device=self.x.device)
            ops.scaled_sum(delta.terms, summed)
            delta = summed
        self.pending = delta

    def add_normed(self, delta, post) -> None:
        """x += post(delta), with the norm `post` on the sublayer's OUTPUT: it stays pending, so
        that the next norm (`normed`) can take the norm, the add and itself in one kernel.  `post`
        offers `add_to(x, terms, then=None)`."""
        self.flush()
        self._normed = (delta.terms if isinstance(delta, ScaledTerms) else [(delta, 1.0)], post)

    def add_scaled(self, delta: VectorScaledTerms) -> None:
        """x += sum of vector * output: stays pending, so that a norm that offers `forward_scaled`
        scales, adds and norms in one kernel."""
        self.flush()
        self._scaled = delta

    def add_gated(self, delta: GatedDelta) -> None:
        self.flush()
        self._gated = delta

    def flush(self) -> torch.Tensor:
        pending = self.pending
        if pending is not None:
            ops.residual_add(self.x, pending)
            self.pending = None
        return self.x

    # Up to this many rows the gate, the add and the norm run as one kernel (a decoding step is
    # bound by its launches: 0.290 -> 0.274 ms a step of 8 rows at width 1,024); with more rows the
    # gate's own kernel and the norm that adds a pending tensor are faster together (a step of 2,048
    # tokens at width 2,048: 2.29 against 2.36 ms), both moving 16 bytes a thread over many blocks.
    GATED_NORM_ROWS = 64

    def normed(self, norm) -> torch.Tensor:
        if self._normed is not None:
            (terms, post), self._normed = self._normed, None
            return post.add_to(self.x, terms, then=norm)
        scaled = getattr(norm, "forward_scaled", None)
        if self._scaled is not None and scaled is not None:
            terms, self._scaled = self._scaled, None
            return scaled(self.x, terms)
        fused = getattr(norm, "forward_gated", None)
        if self._gated is not None and fused is not None and self.x.shape[0] <= self.GATED_NORM_ROWS:
            gated, self._gated = self._gated, None
            return fused(self.x, gated)
        delta, self.pending = self.pending, None
        return norm.forward(self.x, delta=delta)


def build_part(category: str, spec: PartSpec, store, runtime: Runtime):
    return part_class(category, spec.kind)(spec, store, runtime)
