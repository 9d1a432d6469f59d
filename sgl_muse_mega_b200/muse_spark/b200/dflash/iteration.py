"""One fused DFlash2 decode iteration on a rank: the draft's launches, then the target's verify step and greedy accept.

Mirrors the reference's ``sm103/dflash/iteration.py:670-684`` (``Iteration.launches``: draft_entry, draft_qkv, the draft
layers, draft_head, then the verify launches and verify_accept) and ``runtime/iteration.py:384-412`` (``Fused.step``: one
CUDA graph replay per step). Everything a step needs from the previous one lives on the device:

    accept -> step words (P, anchor, commit)            -> the draft's positions, anchor row, context rows
    verify -> the capture layers' output residuals      -> the draft's fc input rows
    draft  -> the verify window's ids [anchor, drafts]  -> the target entry's ids

so ``step()`` is a graph replay with no host input.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..stack import Stack
from .draft import DraftRank
from .weights import DraftConfig, DraftWeights, TargetShared


class Iteration:
    def __init__(self, stack: Stack, dcfg: DraftConfig, dw: DraftWeights, *, capture: Optional[Sequence[int]] = None,
                 pool_rows: int = 4096, rope_rows: Optional[int] = None, peers: Optional[Sequence] = None, exchange=None,
                 wait_budget: int = 0, packed: Optional[int] = None):  # fmt: skip
        """``stack``: the bound target stack of this rank (greedy tail). ``capture``: indices into ``stack.layers`` whose
        output residual feeds the draft (default: ``dcfg.capture`` relative to the stack's first layer). ``peers`` /
        ``exchange``: the draft's exchange buffers of a world of several processes (``DraftRank.bind``)."""
        assert stack.bound and stack.accept is not None, "the iteration ends with the accept (greedy or sampled) of a bound stack"
        cfg = stack.case.cfg
        assert (dcfg.hidden, dcfg.vocab) == (cfg.hidden, cfg.vocab), "the draft borrows the target's embedding and lm_head"
        first = stack.case.first_layer
        capture = list(capture) if capture is not None else [c - first for c in dcfg.capture]
        assert len(capture) == dcfg.features and all(0 <= c < len(stack.layers) for c in capture), capture
        self.stack, self.capture = stack, capture
        caps = [stack.layers[c].o["stream_out"] for c in capture]
        t = TargetShared(stack.embed, stack.lm_head_w)
        rope_rows = rope_rows or stack.kv_rows
        self.draft = DraftRank(
            dcfg, dw, t, stack.rank, cfg.tp, stack.device, rows=stack.case.rows, pool_rows=pool_rows, rope_rows=rope_rows,
            lib=stack.lib, module=stack.module, words=stack.accept.words, caps=caps, verify_ids=stack.tokens, exchange=exchange,
            wait_budget=wait_budget, packed=packed, lm_head_packed=stack.packed,
            samp=stack.samp, cand=stack.draft_cand, walk_q=stack.draft_walk_q, sample_too=stack.sample_too,
        )  # fmt: skip
        self.draft.bind(peers)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        # a token-tree window (the stack was built with ``tree=True``): the tree walk over the head's lattice between the
        # draft and the verify step (it rewrites the window's ids and its rotation feeds), the compaction of the accepted
        # path's K / V and captured rows behind the accept
        self.tree_walk = self.tree_compact = None
        if stack.tree_table is not None:
            from . import tree as TR

            dr, f = self.draft, stack.feeds
            self.tree_walk = TR.TreeWalk(stack.lib, stack.module, cand=dr.cand, scores=dr.scores, words=stack.accept.words,
                                         verify_ids=stack.tokens, loc_full=f.loc_full, loc_swa=f.loc_swa, table=stack.tree_table,
                                         cos_sin_cache=stack.cos_sin_cache, cos_sin=f.cos_sin)  # fmt: skip
            swa = [t for lr, kv in zip(stack.layers, stack.pools) if not lr.case.global_attn for t in kv]
            full = [t for lr, kv in zip(stack.layers, stack.pools) if lr.case.global_attn for t in kv]
            self.tree_compact = TR.TreeCompact(stack.lib, stack.module, table=stack.tree_table, swa=swa, full=full,
                                               caps=list(dict.fromkeys(caps)))  # fmt: skip

    @classmethod
    def connect(cls, stack: Stack, stack_peers: Sequence, dcfg: DraftConfig, dw: DraftWeights, group=None, **kw) -> "Iteration":
        """A world of one process per GPU: ``stack_peers`` is what ``stack.connect_world`` returned (the peers' arenas hold
        their embedding shards); the draft's own exchange arena is allocated, swapped and mapped here."""
        from ....common import symm
        from . import draft as DR

        ranks = stack.case.cfg.tp
        arena = symm.Arena(stack.lib, DR.exchange_layout(dcfg, ranks, stack.case.rows), stack.device)
        embeds = [None if p is None or p is stack else p.view.embed for p in stack_peers]
        own, peers = DR.connect_exchange(arena, stack.embed, embeds, stack.rank, ranks, group)
        it = cls(stack, dcfg, dw, peers=peers, exchange=own, **kw)
        it.peers = peers  # the mappings live as long as the iteration launches
        return it

    @property
    def kernels(self) -> int:
        return self.draft.kernels() + self.stack.kernels + (2 if self.tree_walk is not None else 0)

    def launch_all(self, s: int, pdl: bool = True, sample: Optional[bool] = None, feeds: bool = False) -> None:
        """``sample``: which of a dual-bound iteration's two forms runs (False the greedy walk and accept, True the sampled
        ones); default: the form the stack was built for. ``feeds``: the window feeds' kernel first (a serving framework's
        batch tensors changed since the last step)."""
        if feeds:
            self.stack.feeds.launch(s, False)
        self.draft.launch_all(s, pdl, sample)
        if self.tree_walk is not None:
            self.tree_walk.launch(s, pdl)
        if sample is None:
            # the iteration ends with an accept: the stack's own tail when that is one, else the accept bound beside it
            # (a serving stack's own tail is the soft cap of the plain verify step)
            own = self.stack.tail is self.stack.tails.get("greedy") or self.stack.tail is self.stack.tails.get("sample")
            tail = None if own else ("greedy" if "greedy" in self.stack.tails else "sample")
        else:
            tail = "sample" if sample else "greedy"
        self.stack.launch_all(s, pdl, tail=tail)
        if self.tree_compact is not None:
            self.tree_compact.launch(s, pdl)

    def capture_graph(self, pdl: bool = True, warmup: bool = True, sample: Optional[bool] = None, feeds: bool = False,
                      after=None) -> torch.cuda.CUDAGraph:  # fmt: skip
        """One CUDA graph of the iteration on a side stream. ``after()``: torch work captured behind the launches (the
        export of the step's results). The default form's graph is kept as ``self.graph`` (``step`` replays it)."""
        dev = self.stack.device
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            if warmup:
                self.launch_all(side.cuda_stream, pdl, sample, feeds)
                side.synchronize()
            with torch.cuda.graph(g, stream=side):
                self.launch_all(torch.cuda.current_stream(dev).cuda_stream, pdl, sample, feeds)
                if after is not None:
                    after()
        torch.cuda.current_stream(dev).wait_stream(side)
        if sample is None:
            self.graph = g
        return g

    def step(self) -> None:
        self.graph.replay()

    def statuses(self) -> list:
        return self.draft.statuses() + self.stack.statuses()
