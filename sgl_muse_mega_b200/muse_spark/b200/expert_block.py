"""The NVFP4 expert block on its own, with whole experts per rank (expert parallelism).

The reference shards every expert over the tensor-parallel ranks (W1 on I, W2 on H; ``test/reference/muse_spark.py:170-180``)
and exchanges the h planes and the zb columns. The isolated-block benchmark case instead gives each of ``ep`` ranks
E / ep WHOLE experts: a rank then runs the lone-rank kernels (no h-plane exchange: it holds the full I of its experts)
on the routed (row, slot) pairs that fall on its experts, and only the zb rows cross ranks. The results are bit-identical
to ep = 1: the h requantisation is per 16-group with the row exponent taken over the full row, and every (row, slot)
pair is computed by exactly one rank with the same kernels, tiles and order.

``ExpertBlock`` holds the ``ep`` ranks of such a world on ONE device (``LayerRank`` objects of a lone-rank shape bound with
``MkLayerBind.expert_lo`` / ``expert_hi``, each keeping and packing its own experts only, all writing the same ``zb``).
``ExpertBlockRank`` is one rank of the same world with one process per GPU: its zb rows and its flag block live in an
arena the peers map (``common/symm.py``), g2 stores the zb rows of its (row, slot) pairs into every rank's zb and signals
the expert-output exchange, and every rank's combine waits for all ranks (``MkLayerBind.ep_rank`` / ``ep_world``).
The stages run through the C ABI by index: pooler + router (the block's inputs: h rows ~ N(0, 1) against N(0, 1 / H)
weights give pooled rows and router logits ~ N(0, 1)), routing + pre-expert norm + input quantisation, g1, h-row view,
g2 on every rank, then one combine. ``time_experts`` times the expert kernels (g1, g2) of each rank between CUDA events with
L2 flushed before every sample (``bench.py --config 2`` prints the sweep over rows and ranks).
"""

from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ...common import host, symm
from ..config import Config
from . import layer as L
from . import synthetic

ST_POOLER, ST_G1, ST_COMBINE = 4, 9, 12
EXPERT_BYTES = 3 * 4096 * (2048 + 256)  # codes + scales of gate, up and W2 of one whole expert at the full shape


def block_config(experts: int = 256, moe_hidden: int = 4096, moe_inter: int = 4096, hidden: int = 1024) -> Config:
    """A lone rank with the full expert shape; the dense side (not part of the block) is kept small."""
    return Config(hidden=hidden, q_heads=64, kv_heads=8, experts=experts, topk=8, moe_hidden=moe_hidden,
                  moe_inter=moe_inter, bf16_moe_layers=(), tp=1, node_ranks=1)  # fmt: skip


def draw_case(cfg: Config, rows: int, device, seed: int = 2, band: str = "baseline"):
    """Weights and inputs drawn on ``device`` (7.25 GB of expert bytes at the full shape)."""
    synthetic.set_device(device)
    try:
        return synthetic.layer_case(cfg, rows=rows, ctx=16, band=band, seed=seed)
    finally:
        synthetic.set_device("cpu")


def with_rows(case, rows: int):
    """The same layer with a window of ``rows`` <= case.rows rows (weights shared, row inputs sliced)."""
    t = case.ranks[0]
    cut = lambda x: None if x is None else x[:rows]  # noqa: E731
    t = dataclasses.replace(t, qkv_in=cut(t.qkv_in), stream_in=cut(t.stream_in), next_cos_sin=cut(t.next_cos_sin))
    return dataclasses.replace(case, rows=rows, ranks=[t])


class ExpertBlock:
    def __init__(self, case, device, ep: int = 1, lib: Optional[host.Library] = None, module=None, seed: int = 0):
        """``case``: a drawn lone-rank layer (``draw_case``, ``with_rows``); its expert tensors are shared by every world
        built on it. ``seed`` draws the block's input rows."""
        cfg = case.cfg
        assert cfg.tp == 1 and cfg.experts % ep == 0
        self.lib = lib or host.library()
        self.case, self.device, self.ep = case, device, ep
        self.rows = case.rows
        with torch.cuda.device(device):
            self.module = module or self.lib.load()
        c = self.lib.layer_constants(L.layer_shape(cfg, case, 0))
        self.zb = torch.zeros(int(c.zb_bytes), dtype=torch.uint8, device=device)
        per = cfg.experts // ep
        self.ranks = []
        for r in range(ep):
            lr = L.LayerRank(self.lib, self.module, case, 0, device, tensors=case.ranks[0], keep_plain_experts=True,
                             io={"zb": self.zb}, expert_range=(r * per, (r + 1) * per) if ep > 1 else None)  # fmt: skip
            lr.bind()
            self.ranks.append(lr)
        g = torch.Generator(device=device)
        g.manual_seed(1000 + seed)
        h = torch.randn(case.rows, cfg.hidden, generator=g, device=device).to(torch.bfloat16)
        for lr in self.ranks:
            lr.o["h3"].copy_(h)
            lr.o["h3f"].copy_(h.float())

    def run(self, stream: Optional[int] = None) -> None:
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        for lr in self.ranks:
            lr.launch_record.step(s, ST_POOLER, ST_COMBINE - ST_POOLER)
        self.ranks[0].launch_record.step(s, ST_COMBINE, 1)

    def statuses(self) -> list:
        s = torch.cuda.current_stream(self.device).cuda_stream
        return [lr.launch_record.status(s).code for lr in self.ranks]

    def local_experts(self) -> list:
        """Distinct routed experts per rank (after ``run``)."""
        ids = self.ranks[0].o["ids"][: self.rows].flatten().cpu()
        per = self.case.cfg.experts // self.ep
        return [int(torch.unique(ids[(ids >= r * per) & (ids < (r + 1) * per)]).numel()) for r in range(self.ep)]

    def time_experts(self, iters: int = 10, flush_mb: int = 512) -> list:
        """Median microseconds of g1 + g2 (the h-row view rides g2's staging) per rank, L2 flushed before each sample."""
        s = torch.cuda.current_stream(self.device)
        flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device=self.device)
        out = []
        for lr in self.ranks:
            ts = []
            for _ in range(iters + 2):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(s)
                lr.launch_record.step(s.cuda_stream, ST_G1, ST_COMBINE - ST_G1)
                b.record(s)
                b.synchronize()
                ts.append(a.elapsed_time(b) * 1e3)
            out.append(sorted(ts[2:])[len(ts[2:]) // 2])
        return out


def ep_layout(zb_bytes: int) -> symm.Layout:
    """The arena of one rank of an expert-parallel world: its flag block and its zb rows."""
    lay = symm.Layout()
    lay.add("flags", (64,), torch.int32)
    lay.add("zb", (zb_bytes,), torch.uint8)
    return lay


class _EpPeer:
    """A peer's zb rows and flag block by device address (its arena, mapped)."""

    def __init__(self, arena):
        self.arena, self.zb, self.flags = arena, arena.ptr("zb"), arena.ptr("flags")


class ExpertBlockRank:
    """Rank ``rank`` of an expert-parallel world of ``world`` processes, one per GPU (``torch.distributed`` initialised: it
    only swaps the arenas' handles). Every rank draws the same case (same seed) and keeps its experts
    [rank E / world, (rank + 1) E / world); the block's input rows are the same on every rank, so every rank routes alike.
    ``run`` enqueues pooler + router, routing, g1, g2 and the combine; afterwards ``y`` holds the combined rows on every
    rank."""

    def __init__(self, case, device, rank: int, world: int, lib: Optional[host.Library] = None, module=None, seed: int = 0,
                 group=None, wait_budget: int = 1 << 24):  # fmt: skip
        cfg = case.cfg
        assert cfg.tp == 1 and cfg.experts % world == 0 and world >= 2
        self.lib = lib or host.library()
        self.case, self.device, self.rank, self.world, self.rows = case, device, rank, world, case.rows
        with torch.cuda.device(device):
            self.module = module or self.lib.load()
        c = self.lib.layer_constants(L.layer_shape(cfg, case, 0))
        self.arena = symm.Arena(self.lib, ep_layout(int(c.zb_bytes)), device)
        per = cfg.experts // world
        self.lr = L.LayerRank(self.lib, self.module, case, 0, device, tensors=case.ranks[0], keep_plain_experts=False,
                              io={"zb": self.arena.tensor("zb"), "flags": self.arena.tensor("flags")},
                              expert_range=(rank * per, (rank + 1) * per))  # fmt: skip
        arenas = symm.connect(self.arena, rank, world, group, self.lib)
        self.peers = [None if r == rank else _EpPeer(a) for r, a in enumerate(arenas)]  # the mappings live with this object
        self.lr.bind(ep_peers=self.peers, ep_rank=rank, wait_budget=wait_budget)
        g = torch.Generator(device=device)
        g.manual_seed(1000 + seed)
        h = torch.randn(case.rows, cfg.hidden, generator=g, device=device).to(torch.bfloat16)
        self.lr.o["h3"].copy_(h)
        self.lr.o["h3f"].copy_(h.float())
        import torch.distributed as dist

        dist.barrier(group)  # every rank is bound before any rank launches (a launch stores into the peers' zb)

    @property
    def y(self) -> torch.Tensor:
        return self.lr.o["y"]

    def run(self, stream: Optional[int] = None) -> None:
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        self.lr.launch_record.step(s, ST_POOLER, ST_COMBINE - ST_POOLER + 1)

    def run_experts(self, stream: int) -> None:
        """g1, g2 and the combine (which waits for every rank's zb rows): what ``time_block`` times."""
        self.lr.launch_record.step(stream, ST_G1, ST_COMBINE - ST_G1 + 1)

    def status(self) -> int:
        return self.lr.launch_record.status(torch.cuda.current_stream(self.device).cuda_stream).code

    def local_experts(self) -> int:
        ids = self.lr.o["ids"][: self.rows].flatten().cpu()
        per = self.case.cfg.experts // self.world
        return int(torch.unique(ids[(ids >= self.rank * per) & (ids < (self.rank + 1) * per)]).numel())
