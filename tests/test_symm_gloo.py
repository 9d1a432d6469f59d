"""Host side of the multi-GPU world on CPU: two gloo ranks carve their exchange arenas, swap the handles and end up with
each other's buffers at base + the same offsets; a rank that carved another layout is refused. The device calls are a
fake of the C ABI's mk_symm_* (no GPU here)."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sgl_muse_mega_b200.common import symm
from sgl_muse_mega_b200.muse_spark.b200 import stack as S
from sgl_muse_mega_b200.muse_spark.config import Config


class FakeLib:
    """mk_symm_alloc / mk_symm_open stand-ins: a rank's allocation 'lives' at 0x10000000 x (rank + 1)."""

    def __init__(self, rank):
        self.rank, self.opened, self.closed = rank, [], []

    def symm_alloc(self, nbytes):
        return 0x10000000 * (self.rank + 1), bytes([self.rank]) * 64

    def symm_open(self, handle):
        self.opened.append(handle[0])
        return 0x10000000 * (handle[0] + 1)

    def symm_close(self, ptr):
        self.closed.append(ptr)


class FakeArena:
    def __init__(self, lib, layout):
        self.lib, self.layout = lib, layout
        self.base, self.handle = lib.symm_alloc(layout.nbytes)

    def ptr(self, name):
        return self.base + self.layout.offset(name)


def _worker(rank, world, port, mismatch, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, vocab=4096,
                     tp=2, node_ranks=2)  # fmt: skip
        rows = 16 if not (mismatch and rank == 1) else 8
        lib = FakeLib(rank)
        arena = FakeArena(lib, S.exchange_layout(cfg, rows))
        try:
            peers = symm.connect(arena, rank, world, lib=lib)
        except RuntimeError as e:
            out[rank] = ("refused", str(e))
            return
        views = [S.ExchangeView(a) for a in peers]
        lay = arena.layout
        ok = all(getattr(views[r], k) == 0x10000000 * (r + 1) + lay.offset(k) for r in range(world) for k in S.EXCHANGE)
        out[rank] = ("ok", ok, lib.opened, peers[rank] is arena, sorted(lay.items))
    finally:
        dist.destroy_process_group()


def _run(mismatch):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        out = m.dict()
        port = 29600 + os.getpid() % 300 + (50 if mismatch else 0)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, mismatch, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        return dict(out)


def test_two_ranks_map_each_others_arena():
    out = _run(False)
    for r in (0, 1):
        kind, ok, opened, own_is_arena, names = out[r]
        assert kind == "ok" and ok and own_is_arena
        assert opened == [1 - r]  # the peer's handle was opened, one's own was not
        assert names == sorted(S.EXCHANGE)


def test_a_rank_with_another_layout_is_refused():
    out = _run(True)
    assert out[0][0] == "refused" and out[1][0] == "refused"
    assert "different exchange layout" in out[0][1]


def test_layout_is_aligned_and_sized_for_the_full_model():
    cfg = Config()
    lay = S.exchange_layout(cfg, 16)
    assert all(off % symm.ALIGN == 0 for off, _, _ in lay.items.values())
    sizes = {k: symm._nbytes(s, d) for k, (_, s, d) in lay.items.items()}
    assert sizes["ar"] == 8 * 16 * 8192 * 2 and sizes["gathered"] == 16 * 202048 * 4
    assert sizes["embed"] == 25256 * 8192 * 2 and sizes["z16"] == 128 * 4096 * 2 and sizes["z"] == 128 * 4096 // 2
    assert lay.nbytes < 450 * 2**20
    with pytest.raises(ValueError):
        lay.add("ar", (1,), torch.uint8)
