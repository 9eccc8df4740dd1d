"""Interfaces of the parts a model is put together from, and their registries.

A model is data: a :class:`ModelPlan` names, layer by layer, which mixer, feed-forward,
norm and block arrangement to use and with which sizes and constants, plus the order in
which the layers run.  The parts themselves know nothing of the model they are in: they
get their sizes as constructor arguments, declare the checkpoint tensors they want
(:class:`TensorSource`), the cache they need (:class:`PagedKvSpec`, :class:`StateSpec`)
and implement ``forward``.  New kinds are added with ``register_mixer`` and friends; the
reference has one hook table per architecture instead (``ArchSpec``,
src/locus/model/arch.hpp:19-53).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


# ---------------------------------------------------------------------------
# data that describes a model


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by kind, with its sizes and constants."""

    kind: str
    args: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the tensor-name prefix, the arrangement and the parts it arranges."""

    prefix: str
    arrangement: PartSpec
    norm: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run ``layer``; ``cache_of`` names an earlier entry of the
    order (by its index) whose cache this call reads instead of keeping its own."""

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    eos_token_id: int
    embedding: PartSpec
    layers: List[LayerSpec]
    order: List[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    config: Any = None
    # checkpoint tensors (shell-style patterns) that files of this architecture may hold and the model
    # does not read: left-overs of the format such as tables that are recomputed
    ignorable_tensors: Tuple[str, ...] = ()

    def describe(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture,
            "layers": len(self.layers),
            "calls": len(self.order),
            "hidden": self.hidden_size,
            "vocab": self.vocab_size,
        }


# ---------------------------------------------------------------------------
# what a part asks of the weight loader and the cache manager


@dataclass(frozen=True)
class TensorSource:
    """A checkpoint tensor and where it goes: rows ``row0 .. row0 + shape[0]`` of the part's
    parameter ``param`` (seen as [rows, cols], or as a vector when 1-D).  ``init`` names the
    random distribution of the random-weights mode: "linear", "bias" or "norm"."""

    name: str
    shape: Tuple[int, ...]
    param: str
    row0: int = 0
    init: str = "linear"


@dataclass(frozen=True)
class PagedKvSpec:
    """What a mixer keeps per token, in pages: a key row of ``n_kv_heads * head_dim`` elements, a value row
    of the same width unless ``has_v`` is off (a mixer that keeps one row per token: keys only, or a latent),
    and ``extra_width`` further elements per token in a tensor of their own (per-token fields beside the
    rows, as the reference appends them to its cache row, src/locus/model/arch.cpp:539-542).  ``window`` > 0:
    only the last ``window`` tokens are kept; pages behind the window go back while the request lives."""

    n_kv_heads: int
    head_dim: int
    window: int = 0
    has_v: bool = True
    extra_width: int = 0

    @property
    def planes(self) -> int:
        return 2 if self.has_v else 1

    def elements_per_token(self) -> int:
        return self.planes * self.n_kv_heads * self.head_dim + self.extra_width


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (one tensor of ``shape`` per request), zero at start."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of every part.  ``params`` holds the loaded device tensors by parameter name."""

    def __init__(self, prefix: str) -> None:
        self.prefix = prefix
        self.params: Dict[str, torch.Tensor] = {}

    # -- weights ------------------------------------------------------------
    def param_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Shape of every parameter this part owns."""
        return {}

    def sources(self) -> List[TensorSource]:
        """Checkpoint tensors that fill the parameters."""
        return []

    # -- lifecycle ----------------------------------------------------------
    def kernel_modules(self, dtype: torch.dtype) -> List[str]:
        """CUDA modules (files of csrc/) this part launches."""
        return []

    def bind(self, rt: "Runtime") -> None:
        """Called once after the parameters are on the device."""

    def sub_parts(self) -> List["Part"]:
        return []


class PendingAdd:
    """An addition to the residual stream that a feed-forward left undone so that the next norm can
    fold it into its own pass over the rows: x[t] += sum over slots of pair_out[pair_pos[t * k + slot]].
    Whoever takes it from the runtime must either hand it to a norm that folds it or ``apply`` it."""

    def __init__(self, pair_out: torch.Tensor, pair_pos: torch.Tensor, top_k: int) -> None:
        self.pair_out, self.pair_pos, self.top_k = pair_out, pair_pos, top_k

    def apply(self, x: torch.Tensor) -> None:
        from .. import kernels as K

        K.moe_combine(x, self.pair_out, self.pair_pos, self.top_k)


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                add: Optional[PendingAdd] = None) -> None:
        """out = norm(x) (rows: gather of x rows); statistics in float32.  ``add``: a pending
        addition to x that must be done (in x) before the norm: fold it in or call ``add.apply(x)``.
        A caller that gives ``rows`` as well reads x no more afterwards, so the addition then only
        has to show in ``out``."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How a mixer encodes positions.  A rotary encoding exposes its table so that the
    mixer can fuse the rotation into its cache write; any encoding may instead implement
    ``apply`` to transform q and k in place."""

    def rotary_table(self) -> Optional["RotaryTable"]:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError


@dataclass
class RotaryTable:
    inv_freq: torch.Tensor  # float32 [rot_dim / 2] on the device
    rot_dim: int
    interleaved: bool


class StepPlan:
    """Work lists that a part wants for every step, planned on the host from the step's segments: which
    tiles of queries its kernels run, which segments take which kernel, and the like.  The step function knows
    nothing of their meaning: it asks every distinct plan of the model (distinct by ``key``) once per step to
    write its lists behind the step's descriptors, into the same pinned buffer, so that they reach the device
    in the step's one copy; the part finds them as ``batch.plans[key]``.

    ``capacity(max_tokens, max_segments)``: the most int32 values the plan writes for any step.
    ``build(seg_q0, seg_qn, seg_ctx, out)``: the three arguments are host arrays (numpy int32 views of the
    pinned buffer, one entry per segment); write the lists into ``out`` (numpy int32, ``capacity`` long) and
    return ``{name: (offset in out, length, trailing shape or None)}`` for lists and ``{name: int}`` for plain
    numbers (counts) that the part wants back."""

    key: Tuple = ()

    def capacity(self, max_tokens: int, max_segments: int) -> int:
        raise NotImplementedError

    def build(self, seg_q0, seg_qn, seg_ctx, out) -> Dict[str, Any]:
        raise NotImplementedError


class Mixer(Part):
    """Mixes information across the tokens of a request (attention here)."""

    def cache_needs(self) -> Tuple[Optional[PagedKvSpec], Optional[StateSpec]]:
        return None, None

    def step_plans(self) -> List[StepPlan]:
        """Host-planned work lists this mixer wants for every step (see :class:`StepPlan`)."""
        return []

    def forward(self, h: torch.Tensor, batch: "StepBatch", cache: "LayerCache",
                residual: torch.Tensor, rt: "Runtime") -> None:
        """Add the mixer's output for the ``batch.T`` rows of ``h`` into ``residual`` (float32)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, batch: "StepBatch", residual: torch.Tensor, rt: "Runtime") -> None:
        """Add the feed-forward output of ``h`` into ``residual`` (float32)."""
        raise NotImplementedError


class Arrangement(Part):
    """How norm, mixer and feed-forward are arranged around the residual stream.

    ``takes_pending_add``: the arrangement starts by taking ``rt.take_pending()`` and completing
    it (usually inside its first norm); only then may the block before it leave its last addition
    pending."""

    takes_pending_add = False

    def forward(self, x: torch.Tensor, batch: "StepBatch", cache: "LayerCache", rt: "Runtime") -> None:
        raise NotImplementedError


# ---------------------------------------------------------------------------
# registries

_REGISTRIES: Dict[str, Dict[str, Callable[..., Part]]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position": {},
    "arrangement": {},
    "embedding": {},
    "head": {},
}


def _register(family: str, kind: str, factory: Callable[..., Part]) -> None:
    _REGISTRIES[family][kind] = factory


def register_mixer(kind: str, factory: Callable[..., Part]) -> None:
    _register("mixer", kind, factory)


def register_feed_forward(kind: str, factory: Callable[..., Part]) -> None:
    _register("feed_forward", kind, factory)


def register_norm(kind: str, factory: Callable[..., Part]) -> None:
    _register("norm", kind, factory)


def register_position(kind: str, factory: Callable[..., Part]) -> None:
    _register("position", kind, factory)


def register_arrangement(kind: str, factory: Callable[..., Part]) -> None:
    _register("arrangement", kind, factory)


def register_embedding(kind: str, factory: Callable[..., Part]) -> None:
    _register("embedding", kind, factory)


def register_head(kind: str, factory: Callable[..., Part]) -> None:
    _register("head", kind, factory)


def make_part(family: str, spec: PartSpec, prefix: str, **extra) -> Part:
    """Instantiate the part ``spec`` of ``family`` with tensor-name prefix ``prefix``."""
    try:
        factory = _REGISTRIES[family][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "(none)"
        raise ValueError(f"unknown {family} kind {spec.kind!r} (registered: {known})") from None
    return factory(prefix, **spec.args, **extra)


def registered(family: str) -> List[str]:
    return sorted(_REGISTRIES[family])


def iter_parts(part: Part):
    """The part and every part nested in it."""
    yield part
    for s in part.sub_parts():
        yield from iter_parts(s)
