"""The cache manager: pages of keys and values, block tables, state slots.

Layers whose mixers ask for the same ``KVCacheSpec`` form a group.  A group
has its own page pool (one tensor per layer, the same page id naming the same
page in each of the group's layers, as the reference's single id does across
all layers, rosellm/roseinfer/engine.py:4370-4408), its own allocator and its
own block table ``[slots, pages per sequence]``.  A group with a window gives
pages back as soon as no later query can see any key in them; every group
gives all of a request's pages back when the request ends.

Beside the pages, each live request owns one slot: a row of every block
table, and one row of every per-request state tensor that a mixer asked for
with a ``StateSpec``.  A slot's state rows are zeroed before the first step
that uses the slot.

Pool layout of one layer: ``[pages, 2 (key, value), kv heads, page size, head
dim]``; the reference keeps K and V as two ``[layers, blocks, heads, 64, dim]``
tensors (rosellm/roseinfer/engine.py:4397-4408).

All bookkeeping is on the host; device tensors are touched only by
``sync_to_device`` (dirty block-table rows, state resets).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import KVCacheSpec, StateSpec
from .allocator import IdAllocator


@dataclass
class CacheGroup:
    spec: KVCacheSpec
    layers: list[int]
    allocator: IdAllocator
    table: np.ndarray  # int32 [slots, max_pages_per_seq]; -1 where no page is held
    first_page: np.ndarray  # int64 [slots]: lowest logical page still held (window groups)
    pools: dict[int, torch.Tensor] = field(default_factory=dict)
    device_table: torch.Tensor | None = None
    host_table: torch.Tensor | None = None  # tensor view of ``table``
    snapshots: list = field(default_factory=list)  # pinned copies of the table that uploads read
    snapshot_at: int = 0


TABLE_SNAPSHOTS = 4  # uploads that may be in flight before the host waits for the oldest


def _key_order(key) -> tuple:
    """Cache keys are a layer's index, or (layer, name) for a layer's further mixers."""
    return (key, "") if isinstance(key, int) else (key[0], str(key[1]))


def pages_for(num_tokens: int, page_size: int) -> int:
    return -(-num_tokens // page_size)


class CacheManager:
    def __init__(
        self,
        kv_specs: dict[int, KVCacheSpec],
        state_specs: dict[int, StateSpec],
        *,
        page_size: int,
        num_pages: int,
        max_slots: int,
        max_seq_len: int,
        dtype: torch.dtype = torch.float32,
        device: str | torch.device = "cpu",
        allocate_pools: bool = True,
    ) -> None:
        self.page_size = int(page_size)
        self.num_pages = int(num_pages)
        self.max_slots = int(max_slots)
        self.max_seq_len = int(max_seq_len)
        self.max_pages_per_seq = pages_for(self.max_seq_len, self.page_size)
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = IdAllocator(self.max_slots, "slot")
        self.num_tokens = np.zeros(self.max_slots, dtype=np.int64)
        self.groups: list[CacheGroup] = []
        self.group_of_layer: dict[int, int] = {}
        by_spec: dict[KVCacheSpec, list[int]] = {}
        for layer in sorted(kv_specs, key=_key_order):
            by_spec.setdefault(kv_specs[layer], []).append(layer)
        for spec, layers in by_spec.items():
            host_table = torch.full(
                (self.max_slots, self.max_pages_per_seq), -1, dtype=torch.int32,
            )
            group = CacheGroup(
                spec=spec,
                layers=layers,
                allocator=IdAllocator(self.num_pages, "page"),
                table=host_table.numpy(),
                first_page=np.zeros(self.max_slots, dtype=np.int64),
                host_table=host_table,
            )
            if allocate_pools:
                for layer in layers:
                    group.pools[layer] = torch.zeros(
                        (self.num_pages, 2, spec.num_kv_heads, self.page_size, spec.head_dim),
                        dtype=dtype, device=self.device,
                    )
                group.device_table = torch.full(
                    (self.max_slots, self.max_pages_per_seq), -1, dtype=torch.int32,
                    device=self.device,
                )
            for layer in layers:
                self.group_of_layer[layer] = len(self.groups)
            self.groups.append(group)
        self.state_specs = dict(state_specs)
        self.states: dict[int, torch.Tensor] = {}
        if allocate_pools:
            for layer, spec in self.state_specs.items():
                self.states[layer] = torch.zeros(
                    (self.max_slots, *spec.shape), dtype=spec.dtype, device=self.device
                )
        self._dirty_rows: set[int] = set()
        self.h2d_bytes = 0  # bytes of block-table rows copied to the device so far
        self._slots_to_reset: list[int] = []

    # ---- what parts read -------------------------------------------------
    def kv_pool(self, layer) -> torch.Tensor:
        return self.groups[self.group_of_layer[layer]].pools[layer]

    def block_table(self, layer) -> torch.Tensor:
        return self.groups[self.group_of_layer[layer]].device_table

    def state(self, layer) -> torch.Tensor:
        return self.states[layer]

    # ---- requests ----------------------------------------------------------
    def new_request(self) -> int | None:
        """A slot for a new request, or ``None`` when all are taken."""
        got = self.slots.alloc(1)
        if got is None:
            return None
        slot = got[0]
        self.num_tokens[slot] = 0
        for g in self.groups:
            g.first_page[slot] = 0
        if self.state_specs:
            self._slots_to_reset.append(slot)
        return slot

    def _first_needed_page(self, group: CacheGroup, first_query_pos: int) -> int:
        """Lowest logical page holding a key that a query at ``first_query_pos`` or later sees."""
        if group.spec.window is None:
            return 0
        first_key = max(0, first_query_pos - group.spec.window + 1)
        return first_key // self.page_size

    def pages_needed(self, slot: int, n_new: int) -> list[int]:
        """Per group, how many new pages ``reserve(slot, n_new)`` would take."""
        cur = int(self.num_tokens[slot])
        out = []
        for g in self.groups:
            have_upto = max(pages_for(cur, self.page_size), int(g.first_page[slot]))
            want_upto = pages_for(cur + n_new, self.page_size)
            first = max(self._first_needed_page(g, cur), have_upto)
            out.append(max(0, want_upto - first))
        return out

    def can_reserve(self, slot: int, n_new: int) -> bool:
        return all(
            need <= g.allocator.num_free for need, g in zip(self.pages_needed(slot, n_new), self.groups)
        )

    def reserve(self, slot: int, n_new: int) -> bool:
        """Pages for ``n_new`` more tokens of ``slot`` in every group, or nothing.

        The reference reserves before the forward pass too
        (rosellm/roseinfer/engine.py:790-794, 1896-1900) but raises when the
        pool is empty; this returns ``False`` and takes no page.
        """
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not live")
        if n_new <= 0:
            raise ValueError("n_new must be positive")
        cur = int(self.num_tokens[slot])
        if cur + n_new > self.max_seq_len:
            raise ValueError(
                f"slot {slot}: {cur} + {n_new} tokens exceed the longest sequence {self.max_seq_len}"
            )
        if (cur % self.page_size) and (cur % self.page_size) + n_new <= self.page_size:
            return True  # the tokens fit the last page the request already holds, in every group
        if not self.can_reserve(slot, n_new):
            return False
        for g in self.groups:
            have_upto = max(pages_for(cur, self.page_size), int(g.first_page[slot]))
            want_upto = pages_for(cur + n_new, self.page_size)
            first = max(self._first_needed_page(g, cur), have_upto)
            if want_upto > first:
                pages = g.allocator.alloc(want_upto - first)
                assert pages is not None
                g.table[slot, first:want_upto] = pages
                # pages of a window group that the portion skips entirely stay -1
                self._dirty_rows.add(slot)
        return True

    def commit(self, slot: int, n_new: int) -> None:
        """The step that used ``reserve(slot, n_new)`` has been issued: count the tokens
        and give back pages that a window has passed."""
        self.num_tokens[slot] += n_new
        cur = int(self.num_tokens[slot])
        for g in self.groups:
            if g.spec.window is None:
                continue
            keep_from = self._first_needed_page(g, cur)
            lo = int(g.first_page[slot])
            if keep_from > lo:
                row = g.table[slot, lo:keep_from]
                g.allocator.free(int(p) for p in row if p >= 0)
                row[:] = -1
                g.first_page[slot] = keep_from
                self._dirty_rows.add(slot)

    def release(self, slot: int) -> None:
        """The request is over (finished, aborted or preempted): everything it holds goes back."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not live")
        for g in self.groups:
            row = g.table[slot]
            g.allocator.free(int(p) for p in row if p >= 0)
            row[:] = -1
            g.first_page[slot] = 0
        self.num_tokens[slot] = 0
        self.slots.free([slot])
        self._dirty_rows.add(slot)
        if slot in self._slots_to_reset:
            self._slots_to_reset.remove(slot)

    # ---- numbers -------------------------------------------------------------
    @property
    def num_free_pages(self) -> int:
        return min(g.allocator.num_free for g in self.groups) if self.groups else 0

    @property
    def num_free_slots(self) -> int:
        return self.slots.num_free

    def pages_of(self, slot: int, group: int = 0) -> list[int]:
        return [int(p) for p in self.groups[group].table[slot] if p >= 0]

    # ---- device side -----------------------------------------------------------
    def sync_to_device(self) -> None:
        """Upload block-table rows that changed and zero the state of newly taken slots.

        Ordered on the current stream before the step's kernels.
        """
        if self._dirty_rows:
            rows = sorted(self._dirty_rows)
            for g in self.groups:
                if g.device_table is None:
                    continue
                # The copy runs when the stream reaches it, and the host goes on changing the
                # table meanwhile (a finished request's row, a slot taken again): so it reads
                # a snapshot that stays as it is until the copy's event has passed.
                if self.device.type != "cuda":
                    g.device_table.copy_(g.host_table)
                    continue
                from ..ops.kernels import copy_to_device_raw, record_event

                # One copy of the rows from the first to the last changed one: rows in between
                # that did not change hold on the host what the device holds already.
                snap, done = self._snapshot(g)
                lo, hi = rows[0], rows[-1] + 1
                snap.numpy()[lo:hi] = g.table[lo:hi]
                width = g.table.shape[1]
                copy_to_device_raw(g.device_table.data_ptr() + lo * width * 4, snap.data_ptr() + lo * width * 4,
                                   (hi - lo) * width * 4)
                record_event(done)
                self.h2d_bytes += (hi - lo) * width * 4
            self._dirty_rows.clear()
        if self._slots_to_reset:
            if self.states:  # nothing to zero (and no copy of the indices) where no part keeps state
                idx = torch.tensor(self._slots_to_reset, dtype=torch.long, device=self.device)
                for t in self.states.values():
                    t.index_fill_(0, idx, 0)
            self._slots_to_reset.clear()

    def _snapshot(self, g: CacheGroup) -> tuple[torch.Tensor, "torch.cuda.Event"]:
        """The next of the group's pinned table snapshots, once its last copy is over."""
        if not g.snapshots:
            g.snapshots = [(torch.empty_like(g.host_table, pin_memory=True), torch.cuda.Event())
                           for _ in range(TABLE_SNAPSHOTS)]
        g.snapshot_at = (g.snapshot_at + 1) % len(g.snapshots)
        snap, done = g.snapshots[g.snapshot_at]
        done.synchronize()  # returns at once for an event that was never recorded
        return snap, done

    # ---- checking ----------------------------------------------------------------
    def check(self) -> None:
        """No page lost, none held twice, tables consistent with the allocators."""
        self.slots.check()
        for gi, g in enumerate(self.groups):
            g.allocator.check()
            seen: dict[int, tuple[int, int]] = {}
            for slot in range(self.max_slots):
                row = g.table[slot]
                held = [(i, int(p)) for i, p in enumerate(row) if p >= 0]
                if held and not self.slots.is_held(slot):
                    raise AssertionError(f"group {gi}: free slot {slot} holds pages")
                for i, p in held:
                    if p in seen:
                        raise AssertionError(
                            f"group {gi}: page {p} held twice: {seen[p]} and {(slot, i)}"
                        )
                    if not g.allocator.is_held(p):
                        raise AssertionError(f"group {gi}: page {p} in a table but free")
                    seen[p] = (slot, i)
                if self.slots.is_held(slot):
                    cur = int(self.num_tokens[slot])
                    lo = self._first_needed_page(g, cur)
                    for i in range(lo, pages_for(cur, self.page_size)):
                        if row[i] < 0:
                            raise AssertionError(
                                f"group {gi}: slot {slot} with {cur} tokens lacks page {i}"
                            )
            if len(seen) != g.allocator.num_held:
                raise AssertionError(
                    f"group {gi}: {g.allocator.num_held} pages held, {len(seen)} in tables (lost pages)"
                )
