"""Long-context decode attention (the 131072-token case of the benchmark configurations): the split-KV attention and its
merge over a 131088-key paged cache against the oracle's f64 attention, on a sample of kv-head groups (the full f64
attention over every head takes minutes on the CPU; every group runs the same code path)."""

import pytest
import torch

from oracle import muse_layer as O
from sgl_muse_mega_b200.muse_spark.b200 import layer as L
from sgl_muse_mega_b200.muse_spark.b200 import synthetic
from sgl_muse_mega_b200.muse_spark.config import Config

pytestmark = pytest.mark.gpu


def test_global_attention_over_131072_tokens():
    cfg = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7,
                 bf16_moe_layers=(), tp=1, node_ranks=1)  # fmt: skip
    rows, ctx = 16, 131072
    case = synthetic.layer_case(cfg, rows=rows, ctx=ctx, global_attn=True, band="reference", seed=41)
    dev = torch.device("cuda:0")
    world = L.LayerWorld(case, dev)
    rank = world.ranks[0]
    s = torch.cuda.current_stream().cuda_stream
    rank.launch_record.step(s, 0, 2)  # attention split + merge
    torch.cuda.synchronize()
    assert rank.launch_record.status(s).code == 0
    got = rank.o["x_attn"].cpu()
    t = case.ranks[0]
    grp = cfg.q_heads_rank // cfg.kv_heads_rank
    q, k, v, og = O.split_heads(t.qkv_in, cfg.q_heads_rank, cfg.kv_heads_rank)
    for g in (0, 5):
        hs = slice(g * grp, (g + 1) * grp)
        small = torch.cat([q[:, hs].reshape(rows, -1), k[:, g], v[:, g], og[:, hs].reshape(rows, -1)], 1)
        ref = O.attention(small, t.k_ctx[:, g : g + 1], t.v_ctx[:, g : g + 1], None)
        _, rel, ok = O.compare(got[:, g * grp * 64 : (g + 1) * grp * 64], ref, "x_attn")
        assert ok, (g, rel)
