"""The multi-GPU bench's parity record on CPU: two gloo ranks compare their end states (``bench.ranks_equal``), and
``bench.parity_n`` turns that and the emulated world's verdict into the record the line carries."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import bench  # noqa: E402


def _worker(rank, world, port, differ, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        logits = torch.arange(32, dtype=torch.float32).view(4, 8)
        words = torch.tensor([40, 7, 5, 6], dtype=torch.int64)
        resid = torch.full((2, 16), 0.5)
        if differ and rank == 1:
            resid[1, 3] = -0.0 + 0.5000001  # one element of one rank
            logits[0, 0] = -0.0  # equal as a number to rank 0's 0.0, not as bits
        out[rank] = bench.ranks_equal({"logits": logits, "words": words, "capture_residuals": resid}, world)
    finally:
        dist.destroy_process_group()


def _run(differ):
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(2, 29741 + int(differ), differ, out), nprocs=2, join=True)
        return dict(out)


def test_equal_ranks_report_true_per_tensor():
    got = _run(False)
    assert got[0] == got[1] == {"logits": True, "words": True, "capture_residuals": True}


def test_a_rank_that_differs_is_named_with_its_count():
    got = _run(True)
    assert got[0] == got[1]
    assert got[0]["words"] is True
    assert got[0]["capture_residuals"] == {"differing_elements": 1, "of": 32}
    assert got[0]["logits"] is not True  # the comparison is bitwise: -0.0 is not 0.0


def test_parity_record_needs_every_part():
    same = {"logits": True, "words": True}
    emu = {"bit_equal": True, "mismatch": [], "status": []}
    assert bench.parity_n(2, {"ranks_equal": same}, emu)["bit_equal"] is True
    assert bench.parity_n(2, {"ranks_equal": dict(same, words={"differing_elements": 1, "of": 8})}, emu)["bit_equal"] is False
    assert bench.parity_n(2, {"ranks_equal": same}, dict(emu, bit_equal=False))["bit_equal"] is False
    assert bench.parity_n(2, {"ranks_equal": same}, dict(emu, status=["code 1"]))["bit_equal"] is False
    assert bench.parity_n(2, {}, emu)["bit_equal"] is False
    # the fused form: ranks equal to each other, the emulated per-stage world only to a distance
    assert bench.parity_n(2, {"ranks_equal": same}, dict(emu, bit_equal=False, ranks_bit_equal=True))["bit_equal"] is True
