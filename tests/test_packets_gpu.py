"""Packet mode of the layer's bf16 exchanges (``MkLayerBind.packets``: rows that carry their own validity instead of a
counter word) on worlds emulated on one GPU: the same results bit for bit as the counter-word form, the marks back in
place after every launch, and a poll that runs out recorded without a hang."""

import pytest
import torch
from golden_cases import CASES

from sgl_muse_mega_b200.muse_spark.b200 import layer as L
from sgl_muse_mega_b200.muse_spark.b200 import stack as S
from sgl_muse_mega_b200.muse_spark.b200 import synthetic

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
OUTS = ("x_attn", "branch", "stream_mid", "h3", "ids", "w", "xq", "x_sf", "y", "stream_out", "h3_next", "qkv_next")


def stream() -> int:
    return torch.cuda.current_stream(DEV).cuda_stream


def marks_only(t: torch.Tensor) -> bool:
    return bool((t.view(torch.uint8) == 0xFF).all())


@pytest.mark.parametrize("name,b_live", [("small_fp4_swa_tp2", 0), ("small_fp4_swa_tp8", 0), ("small_fp4_global_tp8_baseline", 11),
                                         ("small_bf16_global_tp8", 0), ("small_bf16_tail_tp4", 0), ("small_fp4_swa_tp1_m5", 0)])  # fmt: skip
def test_packet_world_equals_the_counter_world(name, b_live):
    """Every rank's outputs of two launches in a row, packets against counter words; after each launch the four exchange
    buffers hold nothing but marks wherever a consumer read them (the rows of the live window)."""
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    plain = L.LayerWorld(case, DEV, b_live=b_live)
    pk = L.LayerWorld(case, DEV, b_live=b_live)
    for r in pk.ranks:
        r.bind(pk.ranks, b_live, packets=True)
    M, K = case.rows, cfg.topk
    live = b_live or M
    for rep in range(2):
        plain.run_interleaved()
        pk.run_interleaved()
        torch.cuda.synchronize()
        for a, b in zip(plain.ranks, pk.ranks):
            assert b.launch_record.status(stream()).code == 0
            for k in OUTS:
                if k in a.o and not (case.tail and k in ("h3_next", "qkv_next")):
                    assert torch.equal(a.o[k], b.o[k]), (rep, a.rank, k)
            assert marks_only(b.ar) and marks_only(b.pool_ag) and marks_only(b.unpool_ag), (rep, a.rank)
            zb = b.zb.view(torch.bfloat16).view(M * K, cfg.moe_hidden)
            assert marks_only(zb[: live * K]), (rep, a.rank)


def test_packet_stack_world_equals_the_counter_world():
    """A four-layer stack (one bf16-expert layer) of a two-rank world, three verify steps: step words, arg-max and gathered
    logits of both ranks, packets against counter words, bit for bit."""
    from sgl_muse_mega_b200.muse_spark.config import Config

    cfg = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7,
                 vocab=4096, layers=4, bf16_moe_layers=(0,), tp=2, node_ranks=2)  # fmt: skip
    case = synthetic.stack_case(cfg, n_layers=4, rows=16, ctx=24, seed=21)
    forced = torch.tensor([6], dtype=torch.int32, device=DEV)
    plain = S.StackWorld(case, DEV, accept_override=forced)
    pk = S.StackWorld(case, DEV, accept_override=forced, packets=True)
    assert all(st.packets for st in pk.ranks) and not any(st.packets for st in plain.ranks)
    gen = torch.Generator().manual_seed(5)
    for i in range(3):
        t = torch.randint(0, cfg.vocab, (16,), generator=gen)
        for w in (plain, pk):
            for st in w.ranks:
                st.tokens.copy_(t)
            w.run_interleaved(feeds=i == 0)
        torch.cuda.synchronize()
        for a, b in zip(plain.ranks, pk.ranks):
            assert b.statuses() == []
            assert torch.equal(a.accept.words, b.accept.words) and torch.equal(a.accept.top1, b.accept.top1)
            assert torch.equal(a.gathered, b.gathered), (i, a.rank)


def test_a_packet_that_never_arrives_runs_the_poll_out():
    """Failure detection without a fault: rank 0 of a two-rank world launched alone in packet mode with a budget of 64
    polls a thread. Rank 1's all-reduce partial never arrives: the launch returns, the status names the poll (code 1, the
    post-norm stage), the later polls of the launch give up at once; the next launch on the device is clean."""
    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    world = L.LayerWorld(case, DEV)
    r0 = world.ranks[0]
    r0.bind(world.ranks, wait_budget=64, packets=True)
    r0.launch(stream(), pdl=True)
    torch.cuda.synchronize()
    st = r0.launch_record.status(stream())
    assert (st.code, st.stage) == (1, L.STAGE_NAMES.index("post_norm")), (st.code, st.stage)
    cfg1, kw1 = CASES["small_fp4_swa_tp1_m5"]
    clean = L.LayerWorld(synthetic.layer_case(cfg1, **kw1), DEV)
    clean.run_interleaved()
    torch.cuda.synchronize()
    assert clean.ranks[0].launch_record.status(stream()).code == 0
