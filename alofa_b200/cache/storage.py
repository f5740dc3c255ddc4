"""Device memory of the caches.

For every run entry that owns a cache the model says what it needs
(:class:`~alofa_b200.parts.base.PagedKV` or
:class:`~alofa_b200.parts.base.SlotState`).  Paged caches are sorted into
groups by their window (all keys, or the last ``window``); a group's page ids
are valid in every layer cache of the group.  A layer cache is two tensors
``k, v: [num_pages * block_size, kv_heads, head_dim]``; cache slot
``page * block_size + offset`` holds one token (the reference keeps
``[layers * blocks, block_size, kv_dim]`` and offsets the block id by the
layer, src/alofa/engine/executor.mojo:117-127, 301-310).  Slot-state caches
are one tensor ``[max_requests, *shape]`` each.  A cache of one row per token
(:class:`~alofa_b200.parts.base.PagedRows`) is one tensor
``[num_pages * block_size, width]`` in a group like any other."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..errors import AlofaError
from ..parts.base import PagedKV, PagedRows, SlotState


@dataclass
class LayerCache:
    """Paged keys and values of one layer cache."""

    group: int
    k: torch.Tensor
    v: Optional[torch.Tensor] = None  # None: a cache of one row per token (PagedRows), held in ``k``


@dataclass
class StateCache:
    """Fixed-size per-request state of one layer cache: ``state[slot]``."""

    state: torch.Tensor


def flat_specs(plan: dict) -> list:
    """Every cache spec of a plan, the members of tuples (mixers made of
    several side by side) taken one by one."""
    out = []
    for spec in plan.values():
        out.extend(spec if isinstance(spec, (tuple, list)) else [spec])
    return out


def group_windows(plan: dict) -> list:
    """The distinct windows of a cache plan, all-keys (None) first; empty when
    no layer wants pages (the model then has state slots only, and neither the
    cache manager nor the scheduler books a page for it)."""
    windows = {spec.window for spec in flat_specs(plan) if isinstance(spec, (PagedKV, PagedRows))}
    return ([None] if None in windows else []) + sorted(w for w in windows if w is not None)


class CacheStorage:
    def __init__(self, plan: dict, groups: list, max_requests: int, dtype: torch.dtype, device):
        """``plan``: run index -> cache spec (owners only); ``groups``: the
        :class:`GroupSpec` list in the order of :func:`group_windows`."""
        windows = [g.window for g in groups]
        self.groups = groups
        self.caches = {}
        self.bytes = 0
        self.device, self.dtype, self.max_requests = device, dtype, max_requests
        self._windows = windows
        self._states = []
        for idx, spec in plan.items():
            if isinstance(spec, (tuple, list)):  # a mixer made of several: the tuple of their caches
                self.caches[idx] = tuple(self._make(idx, one) for one in spec)
            elif spec is not None:
                self.caches[idx] = self._make(idx, spec)

    def _make(self, idx, spec):
        windows, groups, dtype, device = self._windows, self.groups, self.dtype, self.device
        if isinstance(spec, (PagedKV, PagedRows)):
            if spec.window not in windows:
                raise AlofaError("invalid_argument", "no cache group for this window", f"window={spec.window} groups={windows}")
            gi = windows.index(spec.window)
            g = groups[gi]
            if isinstance(spec, PagedKV):
                slots = g.num_pages * g.block_size
                k = torch.zeros((slots, spec.num_kv_heads, spec.head_dim), dtype=dtype, device=device)
                v = torch.zeros((slots, spec.v_heads or spec.num_kv_heads, spec.v_head_dim or spec.head_dim), dtype=dtype, device=device)
                self.bytes += (k.numel() + v.numel()) * k.element_size()
                return LayerCache(gi, k, v)
            rows = torch.zeros((g.num_pages * g.block_size, spec.width), dtype=dtype, device=device)
            self.bytes += rows.numel() * rows.element_size()
            return LayerCache(gi, rows, None)
        if isinstance(spec, SlotState):
            st = torch.zeros((self.max_requests,) + tuple(spec.shape), dtype=spec.dtype, device=device)
            self.bytes += st.numel() * st.element_size()
            self._states.append(st)
            return StateCache(st)
        if spec is None:
            return None
        raise AlofaError("unsupported", "unknown cache spec", f"entry={idx} spec={spec!r}")

    def reset_slot(self, slot: int) -> None:
        """Zero the fixed-size state of a slot when a request starts in it."""
        for state in self._states:
            state[slot].zero_()

    @staticmethod
    def bytes_per_token(plan: dict, dtype: torch.dtype) -> dict:
        """window -> bytes of paged cache one token takes in that group."""
        width = torch.empty((), dtype=dtype).element_size()
        out = {}
        for spec in flat_specs(plan):
            if isinstance(spec, PagedKV):
                out[spec.window] = out.get(spec.window, 0) + (spec.num_kv_heads * spec.head_dim + (spec.v_heads or spec.num_kv_heads) * (spec.v_head_dim or spec.head_dim)) * width
            elif isinstance(spec, PagedRows):
                out[spec.window] = out.get(spec.window, 0) + spec.width * width
        return out
