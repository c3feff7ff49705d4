"""The step function: one flat batch in, logits at the wanted places out.

A batch is a list of (request, its next tokens): portions of prompts beside
single decoded tokens, cut anywhere.  Only the tokens given are run; all that
came before is read from the cache.  The reference's step is a padded
``[B, T_q]`` rectangle in which a new request always brings its whole prompt
(gllm/llm/llm.py:145-308), builds a dense ``[B, T_q, T]`` bias and a gathered
copy of the context, and computes logits at every position
(gllm/llm/llm.py:311-340).  Here the batch is flat (no padding rows, no bias,
no gather), metadata is built in numpy and uploaded in one copy, and logits
exist only for the rows asked for.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from gllm_b200 import ops
from gllm_b200.cache.manager import CacheManager
from gllm_b200.parts.base import GroupView, StepContext


@dataclass
class StepEntry:
    request_id: object
    tokens: list[int]
    # places among ``tokens`` whose logits are wanted (may be empty)
    want: list[int] = field(default_factory=list)


class Workspace:
    """Named device scratch buffers that kernels share; grown on demand and
    kept, so steady-state steps allocate nothing."""

    def __init__(self, device):
        self.device = device
        self._buffers: dict[str, torch.Tensor] = {}
        # buffers that were outgrown stay allocated: a captured graph may still hold their address
        self._retired: list[torch.Tensor] = []

    def get(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            if buf is not None:
                self._retired.append(buf)
            buf = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._buffers[name] = buf
        return buf[:numel]


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepRunner:
    """Owns the staging buffers of the batch metadata and runs steps."""

    def __init__(self, model, cache: CacheManager, max_tokens_per_step: int, cuda_graphs: bool = True,
                 prefill_graph_tokens: tuple[int, ...] = ()):
        self.model = model
        self.cuda_graphs = bool(cuda_graphs) and torch.cuda.is_available()
        # portion sizes (the scheduler's full prefill portion) whose steps are captured as graphs too
        self.prefill_graph_tokens = tuple(int(n) for n in prefill_graph_tokens)
        if not getattr(model, "graph_safe_portions", False):
            self.prefill_graph_tokens = ()                 # some part reads the step's host-side description
        self._graphs: dict = {}
        self._graph_pool = None
        self.graph_replays = 0
        self.cache = cache
        self.device = model.device
        self.dtype = model.dtype
        self.max_tokens = int(max_tokens_per_step)
        n_groups = len(cache.groups)
        cap = _align4(self.max_tokens) * (5 + n_groups) + 4 * _align4(cache.max_batch_size + 1) + 64
        # room for every entry of every block table (index and page id): the most a step can change
        cap += 2 * n_groups * _align4((cache.max_batch_size + 1) * cache.max_blocks_per_request)
        self._capacity = cap
        self._pinned = [torch.empty(cap, dtype=torch.int32).pin_memory() if torch.cuda.is_available()
                        else torch.empty(cap, dtype=torch.int32) for _ in range(2)]
        self._flip = 0
        self._meta = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.workspace = Workspace(self.device)
        self.mixer_caches = cache.mixer_caches()
        # The token last sampled (argmax) for every state slot stays on the device: the next step's
        # embedding reads it from here when the host passes a token id < 0.
        self.sampled = torch.zeros(cache.max_batch_size + 1, dtype=torch.int32, device=self.device)
        self._snapshots = [
            (torch.zeros(cache.max_batch_size + 2, dtype=torch.int32).pin_memory() if torch.cuda.is_available()
             else torch.zeros(cache.max_batch_size + 2, dtype=torch.int32))
            for _ in range(4)
        ]
        self._snapshot_turn = 0
        self.last_argmax = None
        self.steps_run = 0
        self.last_h2d_bytes = 0

    # ------------------------------------------------------------------ build
    def build(self, entries: list[StepEntry], pad_to: int = 0, seq_bucket: int = 0, pad_tokens_to: int = 0):
        """Reserve pages, lay the flat batch out on the host and upload it.
        Returns (tokens, StepContext, logit_rows).

        ``pad_to`` (decode-only steps): pad the batch with rows that belong to
        no request up to that many, so a captured graph sees fixed shapes; the
        padding rows use the cache's null row and null page and want logits
        like everybody else.  ``seq_bucket`` then stands in for the longest
        sequence.  ``pad_tokens_to`` (a step that is one prompt portion): a
        second portion that belongs to no request follows the real one and
        brings the step to that many tokens; it writes into the null page and
        attends over it, and nobody wants its logits."""
        cache = self.cache
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        n_total = 0
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if not e.tokens:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            n_total += len(e.tokens)
        if n_total > self.max_tokens:
            raise ValueError(f"step of {n_total} tokens exceeds the limit of {self.max_tokens}")
        if len(entries) > cache.max_batch_size:
            raise ValueError("more requests in a step than state slots")

        # wanted rows keep the caller's order of entries; the flat batch itself puts
        # multi-token portions first and single tokens after them
        caller_order = {id(e): i for i, e in enumerate(entries)}
        entries = sorted(entries, key=lambda e: (len(e.tokens) == 1, caller_order[id(e)]))
        appended = []
        slot_maps = {g.index: [] for g in cache.groups}
        try:
            for e in entries:
                if e.request_id not in cache.requests:
                    cache.add_request(e.request_id)
                    appended.append((e.request_id, None))
                before = cache.requests[e.request_id].num_tokens
                maps = cache.append(e.request_id, len(e.tokens))
                appended.append((e.request_id, before))
                for g, m in maps.items():
                    slot_maps[g].append(m)
        except Exception:
            for rid, before in reversed(appended):
                if before is None:
                    cache.free_request(rid)
                else:
                    cache.rollback(rid, before)
            raise

        real_r = len(entries)
        pad = max(0, pad_to - real_r)
        null_portion = max(0, pad_tokens_to - n_total)
        if null_portion == 1 or (null_portion and pad):
            raise ValueError("a null portion has at least two tokens and does not mix with padding rows")
        r = real_r + pad + (1 if null_portion else 0)
        n_total += pad + null_portion
        tokens = np.zeros(n_total, dtype=np.int32)
        positions = np.zeros(n_total, dtype=np.int32)
        token_row = np.full(n_total, cache.null_row, dtype=np.int32)
        cu_q = np.zeros(r + 1, dtype=np.int32)
        ctx_lens = np.zeros(r, dtype=np.int32)
        slots = np.full(r, cache.null_row, dtype=np.int32)
        rows_of = {}
        q_lens = []
        off = 0
        n_prefill = 0
        for i, e in enumerate(entries):
            rc = cache.requests[e.request_id]
            n = len(e.tokens)
            tokens[off:off + n] = e.tokens
            positions[off:off + n] = np.arange(rc.num_tokens, rc.num_tokens + n, dtype=np.int32)
            token_row[off:off + n] = rc.slot
            ctx_lens[i] = rc.num_tokens
            slots[i] = rc.slot
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request_id!r} wants place {w} of {n} tokens")
            rows_of[caller_order[id(e)]] = [off + w for w in e.want]
            q_lens.append(n)
            if n > 1:
                n_prefill += n
            off += n
            cu_q[i + 1] = off
        row_list = [x for i in sorted(rows_of) for x in rows_of[i]]
        if null_portion:
            positions[off:off + null_portion] = np.arange(null_portion, dtype=np.int32)
            q_lens.append(null_portion)
            n_prefill += null_portion
            off += null_portion
            cu_q[real_r + 1] = off
        for k in range(pad):
            q_lens.append(1)
            cu_q[real_r + k + 1] = off + k + 1
            row_list.append(off + k)
        logit_rows = np.asarray(row_list, dtype=np.int32)
        null_slots = np.full(pad, cache.null_page * cache.block_size, dtype=np.int32)
        if null_portion:
            null_slots = (cache.null_page * cache.block_size
                          + np.arange(null_portion, dtype=np.int32) % cache.block_size).astype(np.int32)

        # pack everything into one pinned buffer, one copy to the device
        pinned = self._pinned[self._flip]
        self._flip ^= 1
        host = pinned.numpy()
        cursor = 0
        views = {}

        def put(name, arr):
            nonlocal cursor
            n = arr.size
            host[cursor:cursor + n] = arr
            views[name] = (cursor, n)
            cursor = _align4(cursor + n)

        put("tokens", tokens)
        put("positions", positions)
        put("token_row", token_row)
        put("cu_q", cu_q)
        put("ctx_lens", ctx_lens)
        put("slots", slots)
        put("rows", logit_rows)
        # state slot of the request that owns each wanted row (padding rows: the null row)
        row_owner = token_row[logit_rows] if logit_rows.size else np.zeros(0, dtype=np.int32)
        put("row_slots", row_owner)
        for g in cache.groups:
            put(f"slotmap{g.index}", np.concatenate(slot_maps[g.index] + [null_slots]))
        # block-table entries that changed since the last step ride along and are scattered on the device
        table_updates = cache.take_table_updates()
        for g, (idx, values) in table_updates.items():
            put(f"table_idx{g}", idx)
            put(f"table_val{g}", values)
        self._meta[:cursor].copy_(pinned[:cursor], non_blocking=True)
        self.last_h2d_bytes = cursor * 4
        for g in table_updates:
            (i0, n), (v0, _) = views.pop(f"table_idx{g}"), views.pop(f"table_val{g}")
            ops.scatter_int32(cache.groups[g].block_table, self._meta[i0:i0 + n], self._meta[v0:v0 + n])

        def dev(name):
            start, n = views[name]
            return self._meta[start:start + n]

        ctx = StepContext(
            num_tokens=n_total,
            num_requests=r,
            dtype=self.dtype,
            positions=dev("positions"),
            token_row=dev("token_row"),
            cu_q=dev("cu_q"),
            context_lens=dev("ctx_lens"),
            state_slots=dev("slots"),
            groups={
                g.index: GroupView(g.block_size, g.block_table, dev(f"slotmap{g.index}")) for g in cache.groups
            },
            q_lens_host=tuple(q_lens),
            context_lens_host=tuple(int(c) for c in ctx_lens),
            max_q_len=max(pad_tokens_to, max(q_lens)),
            max_seq_len=max(seq_bucket, max(int(c) + q for c, q in zip(ctx_lens, q_lens))),
            num_prefill_tokens=n_prefill,
            num_prefill_requests=sum(1 for n in q_lens if n > 1),
            workspace=self.workspace,
            sampled=self.sampled,
        )
        self._row_slots = dev("row_slots")
        self._last_views = views
        return dev("tokens"), ctx, dev("rows")

    # -------------------------------------------------------------------- run
    def _graph_key(self, entries: list[StepEntry]):
        """The key of the captured graph this step can run as, or None.

        ("decode", batch bucket, sequence bucket): every entry brings one token and wants its logits.
        ("prefill", token bucket, wanted rows, padded): one request brings a portion of up to the
        largest size named in ``prefill_graph_tokens``; the step is brought to the bucket's size by a null
        portion (see ``build``).  Neither the portion's length nor what the request has cached before
        enters the launch geometry of any kernel (they read both from device memory), so one graph
        serves every length of the bucket and every context length."""
        if not self.cuda_graphs:
            return None
        if len(entries) == 1 and len(entries[0].tokens) > 1 and self.prefill_graph_tokens:
            bucket = self._prefill_bucket(len(entries[0].tokens))
            if bucket:
                return ("prefill", bucket, len(entries[0].want), bucket != len(entries[0].tokens))
        if not all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return None
        bucket = 1
        while bucket < len(entries):
            bucket *= 2
        bucket = min(bucket, self.cache.max_batch_size)
        if bucket < len(entries) or bucket > self.max_tokens:
            return None
        longest = 1
        for e in entries:
            rc = self.cache.requests.get(e.request_id)
            longest = max(longest, (rc.num_tokens if rc else 0) + 1)
        seq_bucket = 1024
        while seq_bucket < longest:
            seq_bucket *= 2
        return ("decode", bucket, min(seq_bucket, max(self.cache.max_seq_len, longest)))

    def _prefill_bucket(self, n: int) -> int:
        """The step size a lone portion of ``n`` tokens is padded to: 16, 32, 64 (the token buckets of
        the products for few tokens: a short prompt costs what a decode step of that many tokens
        costs), then multiples of 128 up to 1,024, of 256 beyond, with room for a null portion of at
        least two tokens unless ``n`` fits exactly; 0 when it is larger than the largest graphed
        portion or than a step may be."""
        limit = min(max(self.prefill_graph_tokens), self.max_tokens)
        if n > limit:
            return 0
        if n in self.prefill_graph_tokens:
            return n
        for need in (n, n + 2):
            step = 128 if need <= 1024 else 256
            bucket = next((b for b in (16, 32, 64) if need <= b), -(-need // step) * step)
            if bucket == n or bucket >= n + 2:
                # the null portion is a sequence of its own: it has to fit a block-table row
                fits = bucket <= self.max_tokens and bucket - n <= self.cache.max_seq_len
                return bucket if fits else 0
        return 0

    def run(self, entries: list[StepEntry], check: bool = True, greedy: bool = False) -> torch.Tensor:
        """Run one step; returns fp32 logits ``[wanted, vocab]`` on the device,
        in the order of the entries and of their ``want`` lists; they may lie in
        a buffer that the next ``run`` overwrites (copy what has to outlive it).  With
        ``greedy`` the argmax of every wanted row is written to
        ``self.sampled[state slot of the row's request]`` (see ``snapshot``).

        A step in which every request brings a single token runs as a CUDA
        graph captured once per (batch bucket, sequence bucket): same kernels,
        same buffers, one launch.  So does a step that is one full prefill
        portion of one request (see ``_graph_key``)."""
        wanted = sum(len(e.want) for e in entries)
        key = self._graph_key(entries)
        self.last_argmax = None
        if key is None:
            tokens, ctx, rows = self.build(entries)
            logits = self.model.forward(tokens, ctx, self.mixer_caches, rows)
            if greedy and wanted:
                ops.argmax(logits, out=self.sampled, scatter_index=self._row_slots)
        else:
            if key[0] == "decode":
                tokens, ctx, rows = self.build(entries, pad_to=key[1], seq_bucket=key[2])
            else:
                tokens, ctx, rows = self.build(entries, pad_tokens_to=key[1])
            key = key + (bool(greedy),)
            record = self._graphs.get(key)
            # every graph writes its logits into the one workspace buffer (kept, not freed, when it is
            # outgrown): a buffer of its own per captured key would add up to gigabytes at a large
            # vocabulary
            vocab = self.model.spec.vocab_size
            logits_out = self.workspace.get("graph_logits", rows.numel() * vocab, torch.float32).view(-1, vocab)
            if record is None:
                # first time: run it plainly (this is the step's result), then capture for later
                logits = self.model.forward(tokens, ctx, self.mixer_caches, rows, logits_out=logits_out)
                if greedy:
                    ops.argmax(logits, out=self.sampled, scatter_index=self._row_slots)
                torch.cuda.synchronize(self.device)
                graph = torch.cuda.CUDAGraph()
                if self._graph_pool is None:
                    self._graph_pool = torch.cuda.graph_pool_handle()
                launches_before = ops.launch_count
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    g_logits = self.model.forward(tokens, ctx, self.mixer_caches, rows, logits_out=logits_out)
                    if greedy:
                        ops.argmax(g_logits, out=self.sampled, scatter_index=self._row_slots)
                launches = ops.launch_count - launches_before
                ops.launch_count = launches_before          # captured, not run
                self._graphs[key] = (graph, g_logits, dict(self._last_views), launches)
            else:
                graph, logits, views, launches = record
                if views != self._last_views:
                    raise RuntimeError("the batch layout of a captured decode step changed")
                graph.replay()
                self.graph_replays += 1
                ops.launch_count += launches
            logits = logits[:wanted]
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        if check:
            ops.check_status(self.device)
        return logits

    def snapshot(self):
        """Queue a copy of the sampled tokens (by state slot) and of the kernels' status word to
        pinned host memory; returns ``(host tensor, event)``.  After ``event.synchronize()`` the
        tensor holds ``sampled[0 .. max_batch_size]`` followed by the status word."""
        host = self._snapshots[self._snapshot_turn]
        self._snapshot_turn = (self._snapshot_turn + 1) % len(self._snapshots)
        n = self.sampled.numel()
        host[:n].copy_(self.sampled, non_blocking=True)
        host[n:n + 1].copy_(ops.status_word(self.device), non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return host, event

    def finish(self, request_id) -> None:
        """The request is over: its pages and its slot are given back."""
        self.cache.free_request(request_id)
