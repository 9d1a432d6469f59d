"""One rank's verify step over a run of decoder layers, bound once and replayed: window feeds, the fused entry, layer
0's head, the layer launches chained through their shared buffers, the lm_head shard and the greedy accept (or the
soft cap when the caller wants the logits).

Counterpart of the reference's ``Stack`` (``sm103/verify.py:90-470``): every launch record is bound at construction,
``launch_all`` enqueues them in order with programmatic dependent launch between neighbours, ``capture`` records that
sequence into one CUDA graph, ``step`` replays it.

Everything a peer rank reads or writes (the exchange buffers all layers share, the flag block, the gathered logits and
the embedding shard) lives in one arena per rank (``common/symm.py``): a CUDA-IPC allocation when the ranks are separate
processes on separate GPUs, ordinary tensors when ``StackWorld`` holds every rank of the world on one device (parity
tests and single-GPU runs; there the ranks' launches are interleaved group by group so that every exchange has all its
contributions before any rank reads it).
"""

from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ...common import host, symm
from . import headtail as HT
from .head import QkvHead
from .layer import STAGE_GROUPS, LayerRank

EXCHANGE = ("ar", "pool_ag", "unpool_ag", "z", "z16", "z_sf", "z_ex", "zb", "flags", "gathered", "embed")


def exchange_layout(cfg, rows: int) -> symm.Layout:
    """The arena of one rank; depends on the model and the window only, so every rank carves the same offsets."""
    u8, bf = torch.uint8, torch.bfloat16
    slots = rows * cfg.topk
    lay = symm.Layout()
    lay.add("flags", (64,), torch.int32)
    lay.add("ar", (cfg.tp * rows * cfg.hidden * 2,), u8)
    lay.add("pool_ag", (rows, cfg.moe_hidden), bf)
    lay.add("unpool_ag", (rows, cfg.hidden), bf)
    lay.add("z", (slots * cfg.moe_inter // 2,), u8)  # the NVFP4 layers' h codes
    lay.add("z16", (slots * cfg.moe_inter * 2,), u8)  # the bf16-expert layers' h rows, kept apart: see LayerRank
    lay.add("z_sf", (slots * cfg.moe_inter // 16,), u8)
    lay.add("z_ex", (slots * cfg.moe_inter // 16,), u8)
    lay.add("zb", (slots * cfg.moe_hidden * 2,), u8)
    lay.add("gathered", (rows, cfg.vocab), torch.float32)
    lay.add("embed", (cfg.vocab_rank, cfg.hidden), bf)
    return lay


class ExchangeView:
    """A rank's exchange buffers by device address (own arena or a peer's mapped one)."""

    def __init__(self, arena):
        for name in EXCHANGE:
            setattr(self, name, arena.ptr(name))


class PeerStack:
    """What a rank needs of a peer that lives in another process: its arena, mapped."""

    def __init__(self, arena):
        self.arena, self.view = arena, ExchangeView(arena)


class Stack:
    def __init__(self, case, rank: int, device, lib: Optional[host.Library] = None, module=None, *, arena=None,
                 kv_rows: Optional[int] = None, tensor_cores: bool = True, keep_plain_experts: bool = True,
                 greedy: bool = True, accept_override: Optional[torch.Tensor] = None, ring: int = 64,
                 b_live: int = 0, wait_budget: int = 0, fused: bool = False, frame: Optional[dict] = None,
                 pools: Optional[list] = None, packed: Optional[int] = None, sampling: Optional[torch.Tensor] = None,
                 block_verify: bool = True, shared_status: bool = False, accept_too: bool = False,
                 sample_too: bool = False, identity_slots: bool = True, tree: bool = False,
                 packets: Optional[bool] = None):  # fmt: skip
        """``identity_slots`` False (a serving framework's pools: position p does not live in pool row p): the accept writes
        no feeds for the next window (it can only write identity slots); the window feeds' kernel must run before every
        step (``launch_all(feeds=True)``) on the framework's batch tensors.
        ``accept_too``: a stack whose step ends with the soft cap (``greedy`` False) binds the accept as well
        (``self.accept``), for a fused iteration on the same buffers; ``launch_all(tail=...)`` picks the tail.
        ``sample_too`` (with ``sampling``): the greedy accept stays bound beside the sampled one (``self.accept`` and
        ``self.accept_sampled``, one set of step words), so that greedy and sampled requests share the stack.
        ``tree``: the verify window is a token tree (``dflash/tree.py``): every layer's attention reads ``self.tree_table``
        (rows placed by depth, window keys masked by ancestors) and the greedy accept follows the tree's matching path;
        the iteration that owns the stack runs the tree walk before the step and the compaction after it.
        ``packets``: the layers' bf16 exchanges carry their own validity (``LayerRank.bind(packets=...)``) instead of counting
        in the flag block; default: on for a world of several processes (peers over NVLink: it saves every producer's
        system-scope fence and the flag's extra trip), off otherwise (a lone rank or an emulated world orders by stream).
        ``shared_status``: every layer launch of the stack records into ONE status block (``self.shared_status``) instead
        of one per layer: a wait that gave up then makes every later wait of the step give up at once (they see the
        recorded failure) instead of each spending its own budget, and a host reads one block per step.
        ``sampling``: the sampled step's words (``dflash.draft.sampling_words``): the step then ends with the sampled
        accept over the draft head's candidates and walk probabilities (``self.draft_cand`` / ``self.draft_walk_q``, which
        the draft of the iteration writes), block verification or token by token.
        ``case``: a ``synthetic.StackCase``; ``rank`` must be one of ``case.ranks``. ``arena``: the rank's exchange
        memory carved by ``exchange_layout`` (default: ordinary tensors, for a world inside one process). ``greedy``
        False ends the step with the soft cap (the logits go to ``self.logits_out``) instead of the accept."""
        self.lib = lib or host.library()
        if module is None:
            with torch.cuda.device(device):
                module = self.lib.load()
        self.module, self.case, self.rank, self.device = module, case, rank, device
        cfg, M = case.cfg, case.rows
        self.b_live, self.wait_budget, self.fused = b_live or M, wait_budget, fused
        self.samp = None if sampling is None else sampling.to(device)
        self.block_verify = block_verify
        self.packets = packets
        assert not (tree and sampling is not None), "the token tree's accept is greedy"
        self.tree_table = torch.zeros(96, dtype=torch.int32, device=device) if tree else None
        self.draft_cand = self.draft_walk_q = None
        if self.samp is not None:
            self.draft_cand = torch.zeros(M - 1, 16, dtype=torch.int64, device=device)
            self.draft_walk_q = torch.zeros(M - 1, 16, dtype=torch.float32, device=device)
        slot = case.ranks.index(rank)
        dev = lambda t: t.to(device).contiguous()  # noqa: E731
        i64, i32, bf = torch.int64, torch.int32, torch.bfloat16
        kv_rows = kv_rows or (case.ctx + 8 * M + 127) // 128 * 128
        kvw = cfg.kv_heads_rank * cfg.head_dim
        self.kv_rows = kv_rows
        self.arena = arena if arena is not None else symm.LocalArena(exchange_layout(cfg, M), device)
        self.view = ExchangeView(self.arena)
        # ---- the serving framework's side of the feeds: identity slots (position p lives in pool row p) ----
        # (a serving framework hands its own batch tensors in through ``frame``; they are read on the device every step)
        frame = dict(frame or {})
        self.positions = frame.get("positions", torch.arange(case.ctx, case.ctx + M, dtype=i64, device=device))
        self.out_cache_loc = frame.get("out_cache_loc", self.positions.clone())
        self.seq_lens = frame.get("seq_lens", torch.tensor([case.ctx], dtype=i64, device=device))
        self.req_pool_indices = frame.get("req_pool_indices", torch.zeros(1, dtype=i64, device=device))
        self.req_to_token = frame.get("req_to_token")
        if self.req_to_token is None:
            self.req_to_token = torch.arange(kv_rows, dtype=i32, device=device)[None].contiguous()
        self.full_to_swa = frame.get("full_to_swa")
        if self.full_to_swa is None:
            self.full_to_swa = torch.cat([torch.arange(kv_rows, dtype=i64), torch.tensor([-1])]).to(device)
        self.swa_out_cache_loc = frame.get("swa_out_cache_loc", self.out_cache_loc.clone())
        self.cos_sin_cache = dev(case.cos_sin_cache)
        self.tokens = torch.zeros(M, dtype=i64, device=device)
        self.feeds = f = HT.WindowFeeds(
            self.lib, module, positions=self.positions, cos_sin_cache=self.cos_sin_cache,
            out_cache_loc=self.out_cache_loc, swa_out_cache_loc=self.swa_out_cache_loc, seq_lens=self.seq_lens,
            req_pool_indices=self.req_pool_indices, req_to_token=self.req_to_token, full_to_swa=self.full_to_swa,
            kv_row_bytes=kvw * 2,
        )  # fmt: skip
        # ---- weights of the head and tail (the embedding shard sits in the arena: the peers' entries read it) ----
        self.embed = self.arena.tensor("embed")
        self.embed.copy_(case.embed[slot])
        self.pre_w0 = dev(case.pre_w0)
        self.qkv0 = dev(case.qkv0[slot])
        # the dense weights and the lm_head in the dense engine's layout (``LayerRank``): 2 tile images (tensor cores; the
        # default where every K is a multiple of 128), 1 item images, 0 row-major
        tiles_ok = cfg.oproj_k % 128 == 0 and cfg.hidden % 128 == 0 and cfg.moe_hidden % 128 == 0
        self.packed = (2 if tiles_ok else 0) if packed is None else int(packed)
        self.lm_head_w = dev(case.lm_head[slot])
        if self.packed:
            from . import weights as W

            self.lm_head_w = W.pack_dense(self.lm_head_w, self.packed)
        self.gathered = self.arena.tensor("gathered")
        self.logits_out = None if greedy else torch.zeros(M, cfg.vocab, dtype=torch.float32, device=device)
        self.greedy, self.accept_override, self.ring = greedy, accept_override, ring
        self.accept_too, self.sample_too, self.identity_slots = accept_too, sample_too, identity_slots
        self.accept = self.accept_sampled = self.softcap = None
        # ---- the KV pools: one pair per layer; context rows from the case ----
        n = len(case.layers)
        self.pools = pools
        if self.pools is None:
            self.pools = [tuple(torch.zeros(kv_rows, kvw, dtype=bf, device=device) for _ in range(2)) for _ in range(n)]
        assert len(self.pools) == n and all(k.shape[1] == kvw for k, _ in self.pools), "one (K, V) pool pair per layer"
        self.kv_rows = min(int(k.shape[0]) for k, _ in self.pools)
        # ---- the entry and layer 0's head (the peers' shards are wired in bind) ----
        self.residual0 = torch.zeros(M, cfg.hidden, dtype=torch.float32, device=device)
        self.normed0 = torch.zeros(M, cfg.hidden, dtype=bf, device=device)
        global0 = cfg.is_global(case.first_layer)
        self.qkv_head = QkvHead(
            self.lib, module, w=self.qkv0, x=self.normed0, q_heads=cfg.q_heads_rank, kv_heads=cfg.kv_heads_rank,
            q_scale=cfg.q_scale, eps=cfg.rms_eps, cos_sin=None if global0 else f.cos_sin,
            cache_loc=f.loc_full if global0 else f.loc_swa, k_cache=self.pools[0][0], v_cache=self.pools[0][1],
        )  # fmt: skip
        # ---- layers, chained through io; the exchange buffers are the arena's, shared by all layers. One layer's
        # weights at a time: ``case.layers`` may draw them on demand, and without ``keep_plain_experts`` nothing of a
        # layer but its packed images and dense weights stays on the device ----
        shared = {k: self.arena.tensor(k) for k in ("ar", "pool_ag", "unpool_ag", "z", "z16", "z_sf", "z_ex", "zb", "flags")}
        self.shared_status = torch.zeros(4096, dtype=torch.uint8, device=device) if shared_status else None
        if shared_status:
            shared["status"] = self.shared_status
        self.layers: list[LayerRank] = []
        qkv_in, stream_in = self.qkv_head.out, self.residual0
        for j in range(n):
            lc = case.layers[j]
            t = lc.ranks[slot]
            k, v = self.pools[j]
            k[: case.ctx] = t.k_ctx.reshape(case.ctx, kvw).to(device)
            v[: case.ctx] = t.v_ctx.reshape(case.ctx, kvw).to(device)
            nk, nv = self.pools[j + 1] if j + 1 < n else self.pools[j]
            io = dict(shared, qkv_in=qkv_in, stream_in=stream_in, k_cache=k, v_cache=v, next_k=nk, next_v=nv,
                      page_table=f.pt_full if lc.global_attn else f.pt_swa, kv_len=f.kv_len,
                      cache_loc=f.loc_full if lc.next_global else f.loc_swa)  # fmt: skip
            if not (lc.tail or lc.next_global):
                io["next_cos_sin"] = f.cos_sin
            lr = LayerRank(self.lib, module, lc, rank, device, tensors=t, tensor_cores=tensor_cores,
                           keep_plain_experts=keep_plain_experts, io=io, packed=self.packed)  # fmt: skip
            if not keep_plain_experts:
                lr.case = dataclasses.replace(lc, ranks=[])  # the device copies live in lr.w
            del lc, t
            self.layers.append(lr)
            qkv_in, stream_in = lr.o["qkv_next"], lr.o["stream_out"]
        self.hidden = self.layers[-1].o["h3_next"]
        self.bound = False

    # ---- binding ----
    def bind(self, peers: Optional[list] = None) -> None:
        """``peers``: per rank a ``Stack`` (same process) or ``PeerStack`` (mapped arena), own included, None for an
        absent rank; or None altogether for a lone rank."""
        cfg, case, M = self.case.cfg, self.case, self.case.rows
        n = cfg.tp
        f = self.feeds
        if peers is None:
            peers = [self if r == self.rank else None for r in range(n)]
        views = [None if p is None else p.view for p in peers]
        present = sum(v is not None for v in views)
        # the fused segment kernels only on request, and never for peers that live in this process (they are launched one
        # after the other on this GPU, and a segment's exchange waits poll for ranks that run at the same time)
        fused = self.fused and not any(isinstance(p, Stack) and p is not self for p in peers)
        # the entry reads the owner rank's shard; in a slice of a larger world an absent rank's rows read a present rank's
        # shard, the same one on every present rank (present rank number r mod present): the ranks must embed the same rows
        # or their residual streams part ways
        here = [i for i, v in enumerate(views) if v is not None]
        shards = [(v.embed if v is not None else views[here[i % len(here)]].embed) for i, v in enumerate(views)]
        self.entry = HT.Entry(self.lib, self.module, ids=self.tokens, embed_shards=shards, pre_w=self.pre_w0,
                              eps_embed=cfg.rms_eps, eps_pre=cfg.rms_eps, shard_rows=cfg.vocab_rank, hidden=cfg.hidden,
                              residual=self.residual0, normed=self.normed0)  # fmt: skip
        live = self.b_live if self.b_live != M else 0
        packets = self.packets
        if packets is None:
            packets = not fused and any(isinstance(p, PeerStack) for p in peers)
        self.packets = bool(packets)
        for lr in self.layers:
            lr.bind(views, live, self.wait_budget, fused=fused, tree=self.tree_table, packets=self.packets)
        flags = self.arena.tensor("flags")
        self.lm_head = HT.LmHead(self.lib, self.module, w=self.lm_head_w, x=self.hidden,
                                 gathered=[None if v is None else v.gathered for v in views], rank=self.rank,
                                 flags=flags, flags_peer=[None if v is None else v.flags for v in views],
                                 v_total=cfg.vocab, w_packed=self.packed, n_out=cfg.vocab_rank, hidden=cfg.hidden)  # fmt: skip
        self.tails = {}
        if self.greedy or self.accept_too:
            common = dict(
                logits=self.gathered, tokens=self.tokens, b_live=self.b_live, scale=cfg.output_multiplier, cap=cfg.softcap,
                ring=self.ring, accept_override=self.accept_override, flags=flags, contributors=present,
                wait_budget=self.wait_budget,
            )  # fmt: skip
            if self.identity_slots:
                common.update(cos_sin_cache=self.cos_sin_cache, cos_sin=f.cos_sin, loc_full=f.loc_full, loc_swa=f.loc_swa,
                              kv_len=f.kv_len, pool_rows=self.kv_rows)  # fmt: skip
            sampled = dict(samp=self.samp, cand=self.draft_cand, walk_q=self.draft_walk_q, block_verify=self.block_verify)
            if self.samp is None or self.sample_too:
                self.accept = HT.Accept(self.lib, self.module, **common, tree=self.tree_table)
                self.tails["greedy"] = self.accept
            if self.samp is not None:
                self.accept_sampled = HT.Accept(self.lib, self.module, **common, **sampled, share=self.accept)
                self.tails["sample"] = self.accept_sampled
                if self.accept is None:  # a sampled-only stack: ``accept`` names its one accept, as before
                    self.accept = self.accept_sampled
            self.accept.words[HT.WORDS["P"]] = case.ctx
        if not self.greedy:
            self.softcap = HT.Softcap(self.lib, self.module, x=self.gathered, out=self.logits_out,
                                      scale=cfg.output_multiplier, cap=cfg.softcap, flags=flags, contributors=present,
                                      wait_budget=self.wait_budget)  # fmt: skip
            self.tails["softcap"] = self.softcap
        self.tail = self.softcap if not self.greedy else (self.accept_sampled if self.samp is not None and not self.sample_too else self.accept)
        self.bound = True

    # ---- launching ----
    @property
    def kernels(self) -> int:
        """Kernel launches of one step (feeds excluded: they run once, the accept refreshes them)."""
        k = 1 + self.qkv_head.launch_record.info().kernels + 2
        return k + sum(lr.launch_record.info().kernels for lr in self.layers)

    def launch_head(self, s: int, pdl: bool = False) -> None:
        self.entry.launch(s, False)
        self.qkv_head.launch(s, pdl)

    def launch_all(self, s: int, pdl: bool = True, feeds: bool = False, tail: Optional[str] = None) -> None:
        """``tail``: "softcap", "greedy" or "sample" (one of the bound tails); default: the stack's own."""
        if feeds:
            self.feeds.launch(s, False)
        self.launch_head(s, pdl)
        for lr in self.layers:
            lr.launch(s, pdl)
        self.lm_head.launch(s, pdl)
        (self.tail if tail is None else self.tails[tail]).launch(s, pdl)

    def capture(self, pdl: bool = True, warmup: bool = True) -> torch.cuda.CUDAGraph:
        """One CUDA graph of the whole step on a side stream; ``step`` replays it. ``warmup`` runs the step once before
        the capture (it advances the step's state like any step). A world of several processes must capture with
        ``warmup`` on every rank or on none: the exchange counters have to stay in step."""
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            if warmup:
                self.launch_all(side.cuda_stream, pdl)
                side.synchronize()
            with torch.cuda.graph(g, stream=side):
                self.launch_all(torch.cuda.current_stream(self.device).cuda_stream, pdl)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.graph = g
        return g

    def step(self) -> None:
        self.graph.replay()

    def rewind(self) -> None:
        """Back to the state before the first step (words, ring, feeds, window rows of the pools); the exchange
        counters keep counting."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        if self.greedy:
            self.accept.words.zero_()
            self.accept.words[HT.WORDS["P"]] = self.case.ctx
            self.accept.out_ring.zero_()
        self.feeds.launch(s)
        for k, v in self.pools:
            k[self.case.ctx :].zero_(), v[self.case.ctx :].zero_()

    def statuses(self) -> list:
        """(launch name, code, stage, observed) of every launch whose device status word is non-zero."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        recs = [("feeds", self.feeds.launch), ("lm_head", self.lm_head.launch)]
        recs += [(f"tail:{k}", t.launch) for k, t in self.tails.items()]
        recs += [(f"layer{j}", lr.launch_record) for j, lr in enumerate(self.layers)]
        bad = []
        for name, rec in recs:
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

    def run_interleaved(self, feeds: bool = True, after_layer=None) -> None:
        """``after_layer(j)`` is called once layer j is enqueued on every rank (the parity tests read the shared exchange
        buffers there, before the next layer overwrites them)."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        for st in self.ranks:
            if feeds:
                st.feeds.launch(s)
            st.launch_head(s)
        for j in range(len(self.case.layers)):
            for first, count in STAGE_GROUPS:
                for st in self.ranks:
                    st.layers[j].launch_record.step(s, first, count)
            if after_layer is not None:
                after_layer(j)
        for st in self.ranks:
            st.lm_head.launch(s)
        for st in self.ranks:
            st.tail.launch(s)


def connect_world(stack: Stack, group=None) -> list:
    """A world of one process per GPU: swaps the arenas' handles over ``torch.distributed``, maps the peers and binds
    ``stack`` against them. Returns the peer list (keep it alive as long as the stack launches)."""
    import torch.distributed as dist

    n, r = dist.get_world_size(group), stack.rank
    tp = stack.case.cfg.tp
    assert n <= tp and dist.get_rank(group) == r, "one process per present rank of the model's world, ranks 0 .. n - 1"
    arenas = symm.connect(stack.arena, r, n, group, stack.lib)
    # a world smaller than the model's (ranks n .. tp - 1 absent) exchanges among the present ranks only
    peers = [stack if i == r else PeerStack(a) for i, a in enumerate(arenas)] + [None] * (tp - n)
    stack.bind(peers)
    dist.barrier(group)
    return peers
