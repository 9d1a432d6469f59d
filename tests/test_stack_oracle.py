"""The chained CPU oracle of a verify step (entry -> layers -> logits -> accept) on a small two-rank model: it is the
checker of the GPU stack tests, so its own wiring is pinned here against the per-layer oracle."""

import torch

from oracle import cases
from oracle import muse_layer as O
from oracle import stack as OS
from sgl_muse_mega_b200.muse_spark.b200 import synthetic
from sgl_muse_mega_b200.muse_spark.config import Config


def test_run_stack_chains_the_layer_oracle():
    cfg = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7,
                 vocab=4096, layers=3, bf16_moe_layers=(0,), tp=2, node_ranks=2)  # fmt: skip
    case = synthetic.stack_case(cfg, n_layers=3, rows=4, ctx=12, seed=3)
    assert [(lc.global_attn, lc.bf16, lc.tail, lc.next_global) for lc in case.layers] == [
        (False, True, False, True), (True, False, False, False), (False, False, True, False)]  # fmt: skip
    tokens = torch.tensor([5, 4095, 2048, 77])
    out = OS.run_stack(case, tokens, 12)
    assert out["logits"].shape == (4, 4096) and len(out["layers"]) == 3
    # layer 1 of the chain is the layer oracle on layer 0's outputs
    from dataclasses import replace

    l0 = out["layers"][0]
    rl = [replace(x, qkv=l0[r]["qkv_next"], stream_in=l0[r]["stream_out"]) for r, x in enumerate(cases.rank_layers(case.layers[1]))]
    again = O.run_layer(rl, cfg.node_ranks)
    assert torch.equal(again[1]["stream_out"], out["layers"][1][1]["stream_out"])
    # the ranks agree on the replicated values, the accept is the arg-max of row 0 when no draft is confirmed
    assert torch.equal(out["layers"][2][0]["h3_next"], out["layers"][2][1]["h3_next"])
    acc = out["accept"]
    assert acc.commit_len == acc.accept_len + 1 and acc.new_pos == 12 + acc.commit_len
    forced = OS.run_stack(case, tokens, 12, forced_accept=2)["accept"]
    assert forced.accept_len == 2 and forced.bonus == int(out["logits"][2].argmax())
