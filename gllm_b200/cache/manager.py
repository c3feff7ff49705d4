"""The cache manager.

Layers whose mixers ask for the same kind of pages (kv heads, head size,
window) form a *group*: one page id addresses that page in every layer of the
group, and each request has one block list per group.  Groups with a window
give pages back as soon as the window has moved past them; all groups give
everything back when a request ends.  Freed pages are handed out again.
Beside the pages, every live request holds one *state slot*, the row of its
block tables and of every fixed-size state tensor a mixer declared.

The reference has one pool for all layers, sized so it can never run short,
and keeps block tables in the runner (gllm/model/kv_cache/paged_kv_cache.py:30-57,
gllm/llm/llm.py:71-82,163-231).

Pool layout per group: ``[cache_layers, pages, block_size * elements per
token]``; inside a page the tensors a mixer declared lie one after the other,
each ``[heads, block_size, width]`` (for attention: ``[2 (k|v), kv_heads,
block_size, head_dim]``, one (page, head) being one contiguous chunk).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from gllm_b200.cache.allocator import BlockAllocator, CacheError, OutOfPages, SlotAllocator
from gllm_b200.parts.base import KVPageRequirement, MixerCache, StateRequirement


@dataclass
class CacheGroup:
    index: int
    requirement: KVPageRequirement
    block_size: int
    allocator: BlockAllocator
    # plan entries that own a pool layer in this group, in plan order
    owner_entries: list[int] = field(default_factory=list)
    pool: torch.Tensor | None = None           # [layers, pages + 1, block_size * elements_per_token]
    block_table: torch.Tensor | None = None    # device [max_batch, max_blocks] int32
    block_table_host: np.ndarray | None = None
    # (slot, first column, end column) ranges of block_table_host that the device copy lacks
    dirty: list = field(default_factory=list)

    @property
    def window(self) -> int | None:
        return self.requirement.window


@dataclass
class RequestCache:
    request_id: object
    slot: int
    num_tokens: int = 0                         # tokens whose keys/values are cached
    # per group: logical block index -> page id, or -1 once the window passed it
    blocks: dict[int, list[int]] = field(default_factory=dict)


class CacheManager:
    def __init__(
        self,
        requirements,
        block_size: int,
        num_blocks: int,
        max_batch_size: int,
        max_seq_len: int,
        dtype: torch.dtype,
        device: torch.device | str,
        allocate_pools: bool = True,
    ):
        """``requirements``: per plan entry ``(KVPageRequirement | None,
        StateRequirement | None, reads_cache_of | None)``."""
        self.block_size = int(block_size)
        self.num_blocks = int(num_blocks)
        self.max_batch_size = int(max_batch_size)
        self.max_seq_len = int(max_seq_len)
        self.max_blocks_per_request = -(-self.max_seq_len // self.block_size)
        self.dtype = dtype
        self.device = torch.device(device)
        self.groups: list[CacheGroup] = []
        self.slots = SlotAllocator(self.max_batch_size)
        self.requests: dict[object, RequestCache] = {}
        self._entry_group: list[int | None] = []
        self._entry_layer: list[int | None] = []
        self._entry_writes: list[bool] = []
        self._states: list[torch.Tensor | None] = []
        self._state_reqs: list[StateRequirement | None] = []
        by_req: dict[KVPageRequirement, CacheGroup] = {}
        for idx, (kv, state, reads) in enumerate(requirements):
            if reads is not None:
                if self._entry_group[reads] is None and self._states[reads] is None:
                    raise CacheError(f"plan entry {idx} reads the cache of entry {reads}, which has none")
                self._entry_group.append(self._entry_group[reads])
                self._entry_layer.append(self._entry_layer[reads])
                self._entry_writes.append(False)
                self._states.append(self._states[reads])
                self._state_reqs.append(None)
                continue
            if kv is not None:
                group = by_req.get(kv)
                if group is None:
                    group = CacheGroup(len(self.groups), kv, self.block_size, BlockAllocator(self.num_blocks))
                    by_req[kv] = group
                    self.groups.append(group)
                self._entry_group.append(group.index)
                self._entry_layer.append(len(group.owner_entries))
                group.owner_entries.append(idx)
            else:
                self._entry_group.append(None)
                self._entry_layer.append(None)
            self._entry_writes.append(True)
            self._state_reqs.append(state)
            if state is not None and allocate_pools:
                # one row more than there are slots: the null row, for rows that pad a batch
                self._states.append(
                    torch.zeros((self.max_batch_size + 1, *state.shape), dtype=state.dtype, device=self.device)
                )
            else:
                self._states.append(None)
        for g in self.groups:
            r = g.requirement
            # One page more than the allocator hands out: the *null page* (id num_blocks).
            # Rows that pad a batch to a fixed size store there and read from there.
            if allocate_pools:
                g.pool = torch.zeros(
                    (len(g.owner_entries), self.num_blocks + 1, self.block_size * r.elements_per_token),
                    dtype=dtype, device=self.device,
                )
            # One row more than there are state slots: the *null row* (index max_batch_size),
            # every entry of which is the null page.
            g.block_table = torch.full(
                (self.max_batch_size + 1, self.max_blocks_per_request), -1, dtype=torch.int32, device=self.device
            )
            g.block_table[self.max_batch_size].fill_(self.num_blocks)
            g.block_table_host = np.full((self.max_batch_size + 1, self.max_blocks_per_request), -1, dtype=np.int32)
            g.block_table_host[self.max_batch_size] = self.num_blocks

    @property
    def null_page(self) -> int:
        return self.num_blocks

    @property
    def null_row(self) -> int:
        return self.max_batch_size

    # ------------------------------------------------------------- accounting
    def bytes_per_token(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.requirement.elements_per_token * item * len(g.owner_entries) for g in self.groups)

    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.num_free if self.groups else 0

    def min_free_pages(self) -> int:
        return min((g.allocator.num_free for g in self.groups), default=1 << 30)

    # --------------------------------------------------------------- requests
    def add_request(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already live")
        slot = self.slots.allocate()
        rc = RequestCache(request_id, slot, 0, {g.index: [] for g in self.groups})
        self.requests[request_id] = rc
        for state in self._states:
            if state is not None:
                state[slot].zero_()
        return rc

    def pages_needed(self, request_id, n_new: int) -> dict[int, int]:
        rc = self.requests[request_id]
        total = rc.num_tokens + n_new
        want = -(-total // self.block_size)
        return {g.index: max(0, want - len(rc.blocks[g.index])) for g in self.groups}

    def pages_for_tokens(self, n_tokens: int) -> int:
        return -(-n_tokens // self.block_size)

    def pages_for_admission(self, n_tokens: int) -> dict[int, int]:
        """Pages each group needs for the first ``n_tokens`` tokens of a request that holds nothing yet
        (a window group gives pages back only after the step that stored them)."""
        return {g.index: -(-n_tokens // g.block_size) for g in self.groups}

    def can_append(self, request_id, n_new: int) -> bool:
        rc = self.requests[request_id]
        if rc.num_tokens + n_new > self.max_seq_len:
            return False
        need = self.pages_needed(request_id, n_new)
        return all(self.groups[g].allocator.can_allocate(n) for g, n in need.items())

    def append(self, request_id, n_new: int) -> dict[int, np.ndarray]:
        """Reserve pages for the request's next ``n_new`` tokens in every group
        (all groups or none) and return each group's slot mapping
        ``page * block_size + offset`` for those tokens."""
        rc = self.requests[request_id]
        if n_new <= 0:
            raise CacheError("append needs at least one token")
        if rc.num_tokens + n_new > self.max_seq_len:
            raise CacheError(
                f"request {request_id!r} would hold {rc.num_tokens + n_new} tokens, max_seq_len is {self.max_seq_len}"
            )
        need = self.pages_needed(request_id, n_new)
        for g, n in need.items():
            alloc = self.groups[g].allocator
            if not alloc.can_allocate(n):
                raise OutOfPages(n, alloc.num_free)
        out = {}
        positions = np.arange(rc.num_tokens, rc.num_tokens + n_new, dtype=np.int64)
        for g, n in need.items():
            group = self.groups[g]
            blocks = rc.blocks[g]
            if n:
                first = len(blocks)
                new = group.allocator.allocate(n)
                blocks.extend(new)
                group.block_table_host[rc.slot, first:first + n] = new
                group.dirty.append((rc.slot, first, first + n))
            table = np.asarray(blocks, dtype=np.int64)
            pages = table[positions // self.block_size]
            if (pages < 0).any():
                raise CacheError("a token would be stored into a page its window already released")
            out[g] = (pages * self.block_size + positions % self.block_size).astype(np.int32)
        return out

    def commit(self, request_id, n_new: int) -> None:
        """The step that stored ``n_new`` tokens has been issued: count them and
        give back the pages every later token's window has passed."""
        rc = self.requests[request_id]
        rc.num_tokens += n_new
        for group in self.groups:
            w = group.window
            if w is None:
                continue
            blocks = rc.blocks[group.index]
            # the next token sits at position >= num_tokens and sees keys >= num_tokens - w + 1
            dead = max(0, (rc.num_tokens - w + 1)) // self.block_size
            release = []
            for b in range(min(dead, len(blocks))):
                if blocks[b] >= 0:
                    release.append(blocks[b])
                    blocks[b] = -1
                    group.block_table_host[rc.slot, b] = -1
                    group.dirty.append((rc.slot, b, b + 1))
            if release:
                group.allocator.free(release)

    def free_request(self, request_id) -> None:
        rc = self.requests.pop(request_id, None)
        if rc is None:
            raise CacheError(f"request {request_id!r} is not live")
        for group in self.groups:
            blocks = [b for b in rc.blocks[group.index] if b >= 0]
            group.allocator.free(blocks)
            n = len(rc.blocks[group.index])
            if n:
                group.block_table_host[rc.slot, :n] = -1
                group.dirty.append((rc.slot, 0, n))
        self.slots.free(rc.slot)

    def rollback(self, request_id, n_tokens_before: int) -> None:
        """Undo an ``append`` that was not followed by a step: release the
        pages beyond what ``n_tokens_before`` tokens need."""
        rc = self.requests[request_id]
        keep = -(-n_tokens_before // self.block_size)
        for group in self.groups:
            blocks = rc.blocks[group.index]
            extra = [b for b in blocks[keep:] if b >= 0]
            if extra:
                group.allocator.free(extra)
            if len(blocks) > keep:
                group.block_table_host[rc.slot, keep:len(blocks)] = -1
                group.dirty.append((rc.slot, keep, len(blocks)))
                del blocks[keep:]

    # ------------------------------------------------------------ device side
    def take_table_updates(self) -> dict[int, tuple[np.ndarray, np.ndarray]]:
        """What the device copies of the block tables lack, per group: (flat indices ``slot *
        max_blocks + column``, page ids), both int32, each entry once with its newest value.  The step
        function uploads them with the step's metadata and scatters them on the device, so the host never
        waits for a copy; the lists are cleared."""
        out = {}
        for group in self.groups:
            if not group.dirty:
                continue
            width = self.max_blocks_per_request
            spans = [np.arange(slot * width + a, slot * width + b, dtype=np.int32) for slot, a, b in group.dirty]
            group.dirty.clear()
            idx = np.unique(np.concatenate(spans))
            out[group.index] = (idx, group.block_table_host.reshape(-1)[idx])
        return out

    def flush_block_tables(self) -> int:
        """Bring the device copies of the block tables up to date with a blocking copy of the changed
        entries (for callers without a step function); returns the bytes copied."""
        copied = 0
        for g, (idx, values) in self.take_table_updates().items():
            table = self.groups[g].block_table.view(-1)
            table[torch.from_numpy(idx.astype(np.int64)).to(table.device)] = torch.from_numpy(values).to(table.device)
            copied += 8 * idx.size
        return copied

    def mixer_caches(self) -> list[MixerCache]:
        """One MixerCache per plan entry."""
        out = []
        for idx in range(len(self._entry_group)):
            g = self._entry_group[idx]
            pages = None
            if g is not None and self.groups[g].pool is not None:
                pages = self.groups[g].pool[self._entry_layer[idx]]
            out.append(MixerCache(group=g, pages=pages, writes=self._entry_writes[idx], state=self._states[idx],
                                  requirement=None if g is None else self.groups[g].requirement,
                                  block_size=self.block_size))
        return out

    # ---------------------------------------------------------------- checking
    def check_invariants(self) -> None:
        """No page lost, none held twice: every page of every group is either
        free or in exactly one live request's block list."""
        for group in self.groups:
            seen: dict[int, object] = {}
            for rc in self.requests.values():
                for b in rc.blocks[group.index]:
                    if b < 0:
                        continue
                    if b in seen:
                        raise CacheError(f"page {b} of group {group.index} is held by {seen[b]!r} and {rc.request_id!r}")
                    seen[b] = rc.request_id
                    if not group.allocator.is_held(b):
                        raise CacheError(f"page {b} is in a block list but the allocator has it free")
            if len(seen) != group.allocator.num_held:
                raise CacheError(
                    f"group {group.index}: {group.allocator.num_held} pages held, {len(seen)} in block lists (lost pages)"
                )
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots):
            raise CacheError("two live requests share a state slot")
