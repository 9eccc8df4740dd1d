"""What a step hands to the parts: the runtime (device, element type, reusable buffers),
the batch descriptors and a layer's view of the cache.

A batch is ragged: ``n_seg`` segments, one per request in the step, each with ``seg_qn``
new tokens that follow the ``seg_ctx`` tokens the request already has in the cache.  The
tokens of all segments are laid end to end (``T`` rows).  Positions always come from
these descriptors, never from a counter inside a kernel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


class Runtime:
    """Device, element type and the buffers that live across steps.

    ``buf(key, shape, dtype)`` returns the same device tensor for the same key on every
    call, allocated once at its first use (sized by the caller for the largest step), so a
    step allocates nothing once every shape has been seen and CUDA graphs can hold the
    addresses.
    """

    def __init__(self, device: torch.device, dtype: torch.dtype, max_tokens: int, max_segments: int,
                 max_wanted: int) -> None:
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_tokens = max_tokens
        self.max_segments = max_segments
        self.max_wanted = max_wanted
        self._bufs: Dict[Tuple, torch.Tensor] = {}
        self._objects: Dict[Tuple, object] = {}
        # An addition to the residual stream that the last feed-forward left to the next norm
        # (parts.base.PendingAdd).  A feed-forward may leave one only while ``defer_add`` is set:
        # the model sets it when the next block, or the final norm, takes pending additions.
        self.defer_add = False
        self._pending = None
        # a second stream for work that does not depend on the main chain (forked and joined
        # with events, also inside a CUDA graph capture)
        self.side_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._fork_event = torch.cuda.Event() if self.side_stream is not None else None
        self._join_event = torch.cuda.Event() if self.side_stream is not None else None

    def leave_pending(self, add) -> None:
        assert self.defer_add and self._pending is None
        self._pending = add

    def take_pending(self):
        p, self._pending = self._pending, None
        return p

    def side(self):
        """Context in which launches go to the side stream, ordered after everything launched so
        far on the main stream; :meth:`join` makes the main stream wait for it.  On a device
        without streams (tests on the CPU) it is a no-op."""
        return _SideScope(self)

    def join(self) -> None:
        if self.side_stream is not None:
            torch.cuda.current_stream(self.device).wait_event(self._join_event)

    def buf(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        k = (key, tuple(shape), dtype)
        t = self._bufs.get(k)
        if t is None:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._bufs[k] = t
        return t

    def rows(self, key: str, width: int, dtype: torch.dtype, n: int, per_token: int = 1) -> torch.Tensor:
        """First ``n`` rows of a [max_tokens * per_token, width] buffer."""
        return self.buf(key, (self.max_tokens * per_token, width), dtype)[:n]

    def shared_object(self, key: Tuple, factory):
        """One object per key for the whole model (for instance a routing layout that every
        layer with the same expert count shares)."""
        o = self._objects.get(key)
        if o is None:
            o = factory()
            self._objects[key] = o
        return o

    def bytes_held(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._bufs.values())


class _SideScope:
    def __init__(self, rt: "Runtime") -> None:
        self.rt = rt

    def __enter__(self):
        rt = self.rt
        if rt.side_stream is None:
            return self
        from .. import kernels as K

        rt._fork_event.record(torch.cuda.current_stream(rt.device))
        rt.side_stream.wait_event(rt._fork_event)
        self._ctx = torch.cuda.stream(rt.side_stream)
        self._ctx.__enter__()
        self._scope = K.stream_scope()
        self._scope.__enter__()
        K.timing_restart()
        return self

    def __exit__(self, *exc):
        rt = self.rt
        if rt.side_stream is None:
            return False
        rt._join_event.record(rt.side_stream)
        self._scope.__exit__(*exc)
        self._ctx.__exit__(*exc)
        return False


@dataclass
class GroupBatch:
    """Descriptors of one cache group for the step."""

    block_table: torch.Tensor  # int32 [n_seg, table_width]
    slots: torch.Tensor        # int32 [T]  page * page_tokens + offset of each new token
    page_tokens: int


@dataclass
class StepBatch:
    T: int
    n_seg: int
    tokens: torch.Tensor      # int32 [T]
    positions: torch.Tensor   # int32 [T]
    seg_q0: torch.Tensor      # int32 [n_seg] first row of each segment
    seg_qn: torch.Tensor      # int32 [n_seg] new tokens
    seg_ctx: torch.Tensor     # int32 [n_seg] tokens cached before the step
    state_slots: torch.Tensor # int32 [n_seg] per-request state slot
    want_rows: torch.Tensor   # int32 [n_want] rows whose logits are returned
    n_want: int
    longest: int = 0          # the longest context of the step, its new tokens included
    # True: the step may be replayed with other lengths (a CUDA graph), so nothing that is launched may
    # depend on ``longest`` or on other lengths known only to the host
    static_shapes: bool = False
    groups: Dict[int, GroupBatch] = field(default_factory=dict)
    # what the parts' own step plans (parts.base.StepPlan) wrote, by the plan's key: device tensors of the
    # work lists by name, and the plain numbers the plan returned
    plans: Dict[Tuple, Dict[str, object]] = field(default_factory=dict)
    # host copies, for parts that plan on the host
    host_seg_q0: List[int] = field(default_factory=list)
    host_seg_qn: List[int] = field(default_factory=list)
    host_seg_ctx: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)


@dataclass
class LayerCache:
    """One layer call's view of the cache: its pages (if it keeps keys and values), the
    descriptors of its group, and its per-request state (if it has any)."""

    group: Optional[int]              # cache group id, key into StepBatch.groups
    pool: Optional[torch.Tensor]      # [n_pages, planes (K, V or K alone), n_kv_heads, page_tokens, head_dim]
    page_tokens: int
    state: Optional[torch.Tensor]     # [n_state_slots, *StateSpec.shape]
    writes: bool = True               # False: the call reads another call's cache
    extra: Optional[torch.Tensor] = None  # [n_pages, page_tokens, extra_width] per-token fields beside the rows
