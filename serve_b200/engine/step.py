"""The step function: one batch of (request, its next tokens) through the model.

A step takes any mix of prompt portions and single decoded tokens, cut
anywhere. It reserves cache pages for the new tokens, packs the batch into one
int32 buffer (one host-to-device copy), runs the model on exactly the tokens it
was given, against the cache earlier steps left, and returns float32 logits at
the wanted places. The reference has two separate functions that cannot be
mixed (serve/run.py:63-106) and whose prefill assumes position 0
(serve/kernels/attn_prefill.py:116-134); this is the one function that
replaces both.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch


# In place of a token id: "the token that was last sampled for this request" (it is still on the device).
FROM_DEVICE = -1


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # places among ``tokens`` whose logits are wanted


@dataclass(frozen=True)
class BatchShape:
    """Host-side facts about a batch that kernels size their grids from."""

    rows: int          # requests in the step
    tokens: int        # tokens in the step
    max_q: int         # most tokens any request brings
    min_q: int         # fewest tokens any request brings
    max_kv: int        # longest sequence after the step
    pure_decode: bool  # every request brings exactly one token
    # Requests ordered by how many tokens they bring, most first: their indices on the device, and the negated counts
    # on the host (ascending, for bisect). A kernel that serves only requests with more than n tokens launches blocks
    # for the first bisect_left(neg_q_sorted, -n) entries of rows_by_q. None: not given.
    rows_by_q: object = None
    neg_q_sorted: Optional[tuple] = None


@dataclass
class StepContext:
    rt: object
    shape: BatchShape
    tokens: torch.Tensor        # [T] int32
    positions: torch.Tensor     # [T] int32 absolute position of each token
    token_row: torch.Tensor     # [T] int32 row (request index in the step) of each token
    cu_q: torch.Tensor          # [R+1] int32 prefix sums of tokens per row
    kv_len: torch.Tensor        # [R] int32 sequence length after this step
    slots: torch.Tensor         # [R] int32 state slot of each row
    logit_rows: torch.Tensor    # [L] int32 indices into the T tokens
    block_tables: List[torch.Tensor]   # per cache group: [R, W] int32
    rids: List[Hashable] = field(default_factory=list)
    last_token: Optional[torch.Tensor] = None   # [max_slots] int32: the token last sampled for each state slot
    memo: Dict[Hashable, object] = field(default_factory=dict)   # what a part derives from the step's arrays alone
    #                                                               (one layer makes it, the layers after it find it)


def _align4(n: int) -> int:
    return (n + 3) & ~3


class _Layout:
    """Where each array of a step lies in the packed int32 buffer."""

    def __init__(self, t: int, r: int, l: int, widths: Sequence[int]):
        off = 0
        self.spans: Dict[str, tuple] = {}
        for name, n in (("tokens", t), ("positions", t), ("token_row", t), ("cu_q", r + 1), ("kv_len", r),
                        ("slots", r), ("logit_rows", l), ("rows_by_q", r)):
            self.spans[name] = (off, n)
            off += _align4(max(n, 1))
        self.tables = []
        for w in widths:
            self.tables.append((off, r, w))
            off += _align4(r * w)
        self.total = off


class Stepper:
    def __init__(self, model, cache, runtime, max_tokens_per_step: int, use_cuda_graphs: bool = False):
        self.model = model
        self.cache = cache
        self.rt = runtime
        self.max_tokens_per_step = max_tokens_per_step
        self.views = cache.views()
        self.on_cuda = runtime.device.type == "cuda"
        self.use_cuda_graphs = use_cuda_graphs and self.on_cuda
        # two pinned staging buffers used in turn: one may still be in flight to the device
        self._hosts: List[Optional[torch.Tensor]] = [None, None]
        self._events: List[object] = [None, None]
        self._turn = 0
        self._dev: Optional[torch.Tensor] = None
        self._graphs: Dict[tuple, object] = {}     # in order of last use
        self._graph_pool = None                    # memory pool shared by all captured graphs
        self.launched_graphs = 0
        # the token last sampled for each state slot (written by the sampling kernel, read by the embedding)
        self.last_token = torch.zeros(cache.max_slots, dtype=torch.int32, device=runtime.device)
        self.last_h2d_bytes = 0
        self.last_slots = None      # device view of the state slots of the last step's rows

    def _pinned_stream(self):
        """The kernels object looks the current stream up once for a whole forward pass."""
        return self.rt.kernels.on_current_stream()

    # ---- buffers ----------------------------------------------------------
    def _buffers(self, n: int):
        self._turn ^= 1
        i = self._turn
        if self._dev is None or self._dev.numel() < n:
            cap = 1 << (max(n, 4096) - 1).bit_length()
            if self.on_cuda:
                torch.cuda.current_stream(self.rt.device).synchronize()
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.rt.device)
            self._hosts = [None, None]
        if self._hosts[i] is None:
            self._hosts[i] = torch.empty(self._dev.numel(), dtype=torch.int32, pin_memory=self.on_cuda)
            self._events[i] = torch.cuda.Event() if self.on_cuda else None
        elif self._events[i] is not None:
            self._events[i].synchronize()   # the copy that last used this buffer has finished
        return self._hosts[i], self._dev

    # ---- the step -----------------------------------------------------------
    def plan(self, entries: Sequence[StepEntry]):
        """Validate a batch and reserve its pages (raises OutOfPages, changing nothing). Returns what the step needs of
        every request, each a list in the order of the entries: (batch of (request, length after the step), request
        ids, tokens brought, tokens held before, state slots, number of wanted places)."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        rids, q_lens = [], []
        total = n_want = 0
        for e in entries:                        # one pass: a step may have a thousand entries
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.rid!r} brings no tokens")
            want = e.want
            if want:
                for w in want:
                    if not (0 <= w < n):
                        raise ValueError(f"request {e.rid!r} wants place {w} of {n} tokens")
                n_want += len(want)
            total += n
            rids.append(e.rid)
            q_lens.append(n)
        if len(set(rids)) != len(rids):
            raise ValueError("a request appears twice in one step")
        if total > self.max_tokens_per_step:
            raise ValueError(f"the step holds {total} tokens; the limit is {self.max_tokens_per_step}")
        cache = self.cache
        opened = []
        try:
            for rid in rids:
                if not cache.is_open(rid):
                    cache.open(rid)
                    opened.append(rid)
            starts, slots = cache.lengths_and_slots(rids)
            batch = [(rid, have + n) for rid, have, n in zip(rids, starts, q_lens)]
            cache.reserve(batch)
        except Exception:
            for rid in opened:
                cache.close(rid)
            raise
        return batch, rids, q_lens, starts, slots, n_want

    def _undo_plan(self, batch) -> None:
        """A step that is refused after its pages were reserved gives back requests it had just opened."""
        for rid, _n in batch:
            if self.cache.is_open(rid) and self.cache.length(rid) == 0:
                self.cache.close(rid)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch; returns [wanted, vocab] float32 logits (None if nothing is wanted)."""
        batch, rids, q_lens, starts, slots, n_want = self.plan(entries)
        r = len(entries)
        new_lens = [n for _, n in batch]
        t = sum(q_lens)
        pure_decode = t == r                     # every entry brings at least one token
        graphable = self.use_cuda_graphs and pure_decode and n_want == r and r <= 512
        longest = max(new_lens)
        if graphable:
            widths = [self.cache.max_blocks for _ in self.cache.groups]
        else:
            widths = [self.cache.blocks_for(longest) for _ in self.cache.groups]
        lay = _Layout(t, r, n_want, widths)
        host, dev = self._buffers(lay.total)
        h = host.numpy()
        o, _ = lay.spans["tokens"]
        pos_o, _ = lay.spans["positions"]
        row_o, _ = lay.spans["token_row"]
        cu_o, _ = lay.spans["cu_q"]
        kv_o, _ = lay.spans["kv_len"]
        sl_o, _ = lay.spans["slots"]
        lr_o, _ = lay.spans["logit_rows"]
        # vectorised packing: a handful of numpy calls however many requests the step has
        ql = np.asarray(q_lens, dtype=np.int64)
        cu = np.zeros(r + 1, dtype=np.int64)
        np.cumsum(ql, out=cu[1:])
        if pure_decode:
            toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=r)
            row_of = np.arange(r, dtype=np.int64)
            pos = np.asarray(starts, dtype=np.int64)
        else:
            toks = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
            row_of = np.repeat(np.arange(r, dtype=np.int64), ql)
            pos = np.arange(t, dtype=np.int64) - cu[:-1][row_of] + np.asarray(starts, dtype=np.int64)[row_of]
        vocab = self.model.spec.vocab_size
        if toks.min() < 0:
            # FROM_DEVICE becomes -(slot + 1): the embedding kernel then reads the slot's last sampled token
            slot_of = np.asarray(slots, dtype=np.int64)[row_of]
            toks = np.where(toks == FROM_DEVICE, -(slot_of + 1), np.where(toks < 0, vocab, toks))
        if toks.max() >= vocab:
            self._undo_plan(batch)
            raise ValueError(f"a token id is outside the vocabulary of {vocab}")
        h[o: o + t] = toks
        h[pos_o: pos_o + t] = pos
        h[row_o: row_o + t] = row_of
        h[cu_o: cu_o + r + 1] = cu
        h[kv_o: kv_o + r] = new_lens
        h[sl_o: sl_o + r] = slots
        rq_o, _ = lay.spans["rows_by_q"]
        if pure_decode:
            h[rq_o: rq_o + r] = row_of
            neg_q_sorted = None
        else:
            order = np.argsort(-ql, kind="stable")
            h[rq_o: rq_o + r] = order
            neg_q_sorted = tuple((-ql[order]).tolist())
        if n_want:
            if pure_decode and n_want == r:
                h[lr_o: lr_o + r] = np.arange(r)
            else:
                h[lr_o: lr_o + n_want] = [int(cu[i]) + w for i, e in enumerate(entries) for w in e.want]
        for gi, (off, rr, w) in enumerate(lay.tables):
            rows = self.cache.table_rows(gi, rids, w, slots=slots)
            h[off: off + rr * w] = rows.reshape(-1)
        self.rt.kernels.fetch_ints(host, dev, lay.total)          # lay.total is a multiple of 4: every span is
        self.last_h2d_bytes = lay.total * 4
        if self._events[self._turn] is not None:
            self._events[self._turn].record()

        def view(name):
            off, n = lay.spans[name]
            return dev[off: off + n]

        ctx = StepContext(
            rt=self.rt,
            shape=BatchShape(r, t, max(q_lens), min(q_lens), longest, pure_decode,
                             rows_by_q=view("rows_by_q") if neg_q_sorted is not None else None, neg_q_sorted=neg_q_sorted),
            tokens=view("tokens"), positions=view("positions"), token_row=view("token_row"),
            cu_q=view("cu_q"), kv_len=view("kv_len"), slots=view("slots"), logit_rows=view("logit_rows"),
            block_tables=[dev[off: off + rr * w].view(rr, w) for off, rr, w in lay.tables],
            rids=rids, last_token=self.last_token,
        )
        self.last_slots = ctx.slots
        if graphable:
            logits = self._run_graph(ctx, r, longest)
        else:
            with self._pinned_stream():
                logits = self.model.forward(ctx, self.views)
        self.cache.commit_many(batch)
        return logits

    # ---- CUDA graphs for pure-decode steps ------------------------------------
    # Captured graphs kept; the least recently used goes. All graphs allocate from one shared pool (they never run at
    # the same time), so a graph costs its nodes, not another copy of the activations.
    MAX_GRAPHS = 1024

    def _graph_key(self, r: int, longest: int):
        return (r, min(self.cache.max_context, max(1024, 1 << (longest - 1).bit_length())))

    def _run_graph(self, ctx: StepContext, r: int, longest: int):
        """Replay (capturing on first use) the decode step for ``r`` requests.

        The packed buffer has the same layout and address for a given r, and grids
        are sized from a length class (the next power of two above the longest
        sequence, at least 1024, at most the context limit) rather than from this
        batch's lengths, so one captured graph serves every decode step of that
        batch size until a sequence grows into the next class.
        """
        key = self._graph_key(r, longest)
        bucket = key[1]
        g = self._graphs.pop(key, None)
        if g is not None:
            self._graphs[key] = g              # most recently used last
        if g is None:
            while len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            shape = BatchShape(r, r, 1, 1, bucket, True)
            static_ctx = StepContext(**{**ctx.__dict__, "shape": shape, "memo": {}})
            # The first step of a kind runs eagerly, with the grids the graph will have, and its logits are this
            # step's result (it also warms allocator pools, library workspaces and lazy module loads). The graph is
            # captured afterwards and first replayed by the next step of the kind: capturing runs nothing, so a
            # mixer with state of its own sees this step's tokens exactly once.
            with self._pinned_stream():
                first = self.model.forward(static_ctx, self.views)
            # what the eager run derived from the step's arrays must be derived again inside the graph: a replay has
            # other positions in the same arrays
            static_ctx.memo.clear()
            graph = torch.cuda.CUDAGraph()
            k = self.rt.kernels
            before = (k.launches, k.library_calls)
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self._graph_pool), self._pinned_stream():
                out = self.model.forward(static_ctx, self.views)
            counts = (k.launches - before[0], k.library_calls - before[1])
            k.launches, k.library_calls = before              # capturing launched nothing
            self._graphs[key] = (graph, out, self._dev, counts)
            return first
        graph, out, dev, counts = g
        if dev is not self._dev:
            # the packed buffer was re-made larger since capture: capture again
            del self._graphs[key]
            return self._run_graph(ctx, r, longest)
        graph.replay()
        self.launched_graphs += 1
        k = self.rt.kernels
        k.launches += counts[0]
        k.library_calls += counts[1]
        return out

    def drop_graphs(self) -> None:
        self._graphs.clear()
