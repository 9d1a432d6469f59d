"""One rank's verify step over a run of decoder layers, bound once and replayed: window feeds, the fused entry, layer
0's head, the layer launches chained through their shared buffers, the lm_head shard and the greedy accept (or the
soft cap when the caller wants the logits).

Counterpart of the reference's ``Stack`` (``sm103/verify.py:90-470``): every launch record is bound at construction,
``launch_all`` enqueues them in order with programmatic dependent launch between neighbours, ``capture`` records that
sequence into one CUDA graph, ``step`` replays it. ``StackWorld`` holds every rank of a tensor-parallel world on one
device (parity tests and single-GPU runs): the ranks' launches are interleaved group by group so that every exchange
has all its contributions before any rank reads it.
"""

from __future__ import annotations

from typing import Optional

import torch

from ...common import host
from . import headtail as HT
from .head import QkvHead
from .layer import STAGE_GROUPS, LayerRank


class Stack:
    def __init__(self, case, rank: int, device, lib: Optional[host.Library] = None, module=None, *,
                 kv_rows: Optional[int] = None, tensor_cores: bool = True, keep_plain_experts: bool = True,
                 greedy: bool = True, accept_override: Optional[torch.Tensor] = None, ring: int = 64,
                 b_live: int = 0):  # fmt: skip
        """``case``: a ``synthetic.StackCase``; ``rank`` must be one of ``case.ranks``. ``greedy`` False ends the step
        with the soft cap (the logits go to ``self.logits_out``) instead of the accept."""
        self.lib = lib or host.library()
        if module is None:
            with torch.cuda.device(device):
                module = self.lib.load()
        self.module, self.case, self.rank, self.device = module, case, rank, device
        cfg, M = case.cfg, case.rows
        self.b_live = b_live or M
        slot = case.ranks.index(rank)
        dev = lambda t: t.to(device).contiguous()  # noqa: E731
        i64, i32, bf = torch.int64, torch.int32, torch.bfloat16
        kv_rows = kv_rows or (case.ctx + 8 * M + 127) // 128 * 128
        kvw = cfg.kv_heads_rank * cfg.head_dim
        self.kv_rows = kv_rows
        # ---- the serving framework's side of the feeds: identity slots (position p lives in pool row p) ----
        self.positions = torch.arange(case.ctx, case.ctx + M, dtype=i64, device=device)
        self.out_cache_loc = self.positions.clone()
        self.seq_lens = torch.tensor([case.ctx], dtype=i64, device=device)
        self.req_pool_indices = torch.zeros(1, dtype=i64, device=device)
        self.req_to_token = torch.arange(kv_rows, dtype=i32, device=device)[None].contiguous()
        self.full_to_swa = torch.cat([torch.arange(kv_rows, dtype=i64), torch.tensor([-1])]).to(device)
        self.swa_out_cache_loc = self.out_cache_loc.clone()
        self.cos_sin_cache = dev(case.cos_sin_cache)
        self.tokens = torch.zeros(M, dtype=i64, device=device)
        self.feeds = HT.WindowFeeds(
            self.lib, module, positions=self.positions, cos_sin_cache=self.cos_sin_cache,
            out_cache_loc=self.out_cache_loc, swa_out_cache_loc=self.swa_out_cache_loc, seq_lens=self.seq_lens,
            req_pool_indices=self.req_pool_indices, req_to_token=self.req_to_token, full_to_swa=self.full_to_swa,
            kv_row_bytes=kvw * 2,
        )  # fmt: skip
        f = self.feeds
        # ---- weights of the head and tail; peers' embedding shards are wired in bind() ----
        self.embed = dev(case.embed[slot])
        self.pre_w0 = dev(case.pre_w0)
        self.qkv0 = dev(case.qkv0[slot])
        self.lm_head_w = dev(case.lm_head[slot])
        self.gathered = torch.zeros(M, cfg.vocab, dtype=torch.float32, device=device)
        self.logits_out = None if greedy else torch.zeros(M, cfg.vocab, dtype=torch.float32, device=device)
        self.greedy, self.accept_override, self.ring = greedy, accept_override, ring
        # ---- the KV pools: one pair per layer; context rows from the case ----
        self.pools = []
        for lc in case.layers:
            t = lc.ranks[slot]
            k, v = (torch.zeros(kv_rows, kvw, dtype=bf, device=device) for _ in range(2))
            k[: case.ctx] = t.k_ctx.reshape(case.ctx, kvw).to(device)
            v[: case.ctx] = t.v_ctx.reshape(case.ctx, kvw).to(device)
            self.pools.append((k, v))
        # ---- layers, chained through io ----
        self.entry = None
        self.layers: list[LayerRank] = []
        self._slot = slot
        self._keep_plain = keep_plain_experts
        self._tensor_cores = tensor_cores
        self.normed0 = torch.zeros(M, cfg.hidden, dtype=bf, device=device)
        self.residual0 = torch.zeros(M, cfg.hidden, dtype=torch.float32, device=device)
        self.qkv_in0 = torch.zeros(M, cfg.qkv_row, dtype=bf, device=device)
        qkv_in, stream_in = self.qkv_in0, self.residual0
        n = len(case.layers)
        for j, lc in enumerate(case.layers):
            k, v = self.pools[j]
            nk, nv = self.pools[j + 1] if j + 1 < n else self.pools[j]
            nxt_global = j + 1 < n and case.layers[j + 1].global_attn
            io = dict(qkv_in=qkv_in, stream_in=stream_in, k_cache=k, v_cache=v, next_k=nk, next_v=nv,
                      page_table=f.pt_full if lc.global_attn else f.pt_swa, kv_len=f.kv_len,
                      cache_loc=f.loc_full if nxt_global else f.loc_swa,
                      next_cos_sin=None if (lc.tail or lc.next_global) else f.cos_sin)  # fmt: skip
            if io["next_cos_sin"] is None:
                io.pop("next_cos_sin")
            lr = LayerRank(self.lib, module, lc, rank, device, tensors=lc.ranks[slot], tensor_cores=tensor_cores,
                           keep_plain_experts=keep_plain_experts, io=io)  # fmt: skip
            self.layers.append(lr)
            qkv_in, stream_in = lr.o["qkv_next"], lr.o["stream_out"]
        self.hidden = self.layers[-1].o["h3_next"]
        self.bound = False

    # ---- binding ----
    def bind(self, peers: Optional[list] = None) -> None:
        """``peers``: every rank's ``Stack`` (own included, None for absent ranks) or None for a lone rank."""
        cfg, case, M = self.case.cfg, self.case, self.case.rows
        n = cfg.tp
        f = self.feeds
        if peers is None:
            peers = [self if r == self.rank else None for r in range(n)]
        # the entry reads the owner rank's shard: an absent rank's rows read this rank's shard (a lone-rank timing run)
        shards = [(p.embed if p is not None else self.embed) for p in peers]
        self.entry = HT.Entry(self.lib, self.module, ids=self.tokens, embed_shards=shards, pre_w=self.pre_w0,
                              eps_embed=cfg.rms_eps, eps_pre=cfg.rms_eps)  # fmt: skip
        self.residual0, self.normed0 = self.entry.residual, self.entry.normed
        l0 = case.layers[0]
        self.qkv_head = QkvHead(
            self.lib, self.module, w=self.qkv0, x=self.normed0, q_heads=cfg.q_heads_rank, kv_heads=cfg.kv_heads_rank,
            q_scale=cfg.q_scale, eps=cfg.rms_eps, cos_sin=None if l0.global_attn else f.cos_sin,
            cache_loc=f.loc_full if l0.global_attn else f.loc_swa, k_cache=self.pools[0][0], v_cache=self.pools[0][1],
        )  # fmt: skip
        # layer 0 was built before the entry and the head existed: point it at their outputs
        self.layers[0].w["qkv_in"] = self.qkv_head.out
        self.layers[0].w["stream_in"] = self.residual0
        for j, lr in enumerate(self.layers):
            lr.bind([None if p is None else p.layers[j] for p in peers], self.b_live if self.b_live != M else 0)
        self.lm_head = HT.LmHead(self.lib, self.module, w=self.lm_head_w, x=self.hidden,
                                 gathered=[None if p is None else p.gathered for p in peers], rank=self.rank)  # fmt: skip
        if self.greedy:
            self.accept = HT.Accept(
                self.lib, self.module, logits=self.gathered, tokens=self.tokens, b_live=self.b_live,
                scale=cfg.output_multiplier, cap=cfg.softcap, ring=self.ring, accept_override=self.accept_override,
                cos_sin_cache=self.cos_sin_cache, cos_sin=f.cos_sin, loc_full=f.loc_full, loc_swa=f.loc_swa,
                kv_len=f.kv_len,
            )  # fmt: skip
            self.accept.words[HT.WORDS["P"]] = case.ctx
            self.tail = self.accept
        else:
            self.tail = HT.Softcap(self.lib, self.module, x=self.gathered, out=self.logits_out,
                                   scale=cfg.output_multiplier, cap=cfg.softcap)  # fmt: skip
        self.bound = True

    # ---- launching ----
    @property
    def kernels(self) -> int:
        """Kernel launches of one step (feeds excluded: they run once, the accept refreshes them)."""
        k = 1 + self.qkv_head.launch_record.info().kernels + 2
        return k + sum(lr.launch_record.info().kernels for lr in self.layers)

    def launch_head(self, s: int, pdl: bool = False) -> None:
        self.entry.launch(s, pdl)
        self.qkv_head.launch(s, pdl)

    def launch_all(self, s: int, pdl: bool = True, feeds: bool = False) -> None:
        if feeds:
            self.feeds.launch(s, False)
        self.entry.launch(s, False)
        self.qkv_head.launch(s, pdl)
        for lr in self.layers:
            lr.launch(s, pdl)
        self.lm_head.launch(s, pdl)
        self.tail.launch(s, pdl)

    def capture(self, pdl: bool = True) -> torch.cuda.CUDAGraph:
        """One CUDA graph of the whole step on a side stream; ``step`` replays it."""
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self.launch_all(side.cuda_stream, pdl)  # warm-up outside the capture
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                self.launch_all(torch.cuda.current_stream(self.device).cuda_stream, pdl)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.graph = g
        return g

    def step(self) -> None:
        self.graph.replay()

    def statuses(self) -> list:
        """(launch name, code) of every launch whose device status word is non-zero."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        bad = []
        for name, rec in [("feeds", self.feeds.launch), ("lm_head", self.lm_head.launch)] + [
            (f"layer{j}", lr.launch_record) for j, lr in enumerate(self.layers)
        ]:
            st = rec.status(s)
            if st.code:
                bad.append((name, st.code, st.stage, st.observed))
        return bad


class StackWorld:
    """Every rank of the world on one device; see the module docstring."""

    def __init__(self, case, device, lib: Optional[host.Library] = None, **kw):
        self.lib = lib or host.library()
        with torch.cuda.device(device):
            self.module = self.lib.load()
        self.case, self.device = case, device
        self.ranks = [Stack(case, r, device, self.lib, self.module, **kw) for r in case.ranks]
        full = [None] * case.cfg.tp
        for st in self.ranks:
            full[st.rank] = st
        for st in self.ranks:
            st.bind(full)

    def run_interleaved(self, feeds: bool = True) -> None:
        s = torch.cuda.current_stream(self.device).cuda_stream
        for st in self.ranks:
            if feeds:
                st.feeds.launch(s)
            st.launch_head(s)
        for j in range(len(self.case.layers)):
            for first, count in STAGE_GROUPS:
                for st in self.ranks:
                    st.layers[j].launch_record.step(s, first, count)
        for st in self.ranks:
            st.lm_head.launch(s)
        for st in self.ranks:
            st.tail.launch(s)
