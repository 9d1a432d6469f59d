"""The seeded layer cases behind ``tests/golden/*.pt`` (same table as ``tests/golden/make_golden.py``)."""

from sgl_muse_mega_b200.muse_spark.config import Config, downscaled


def small_cfg(tp: int) -> Config:
    return Config(
        hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024,
        swa_window=7, bf16_moe_layers=(), tp=tp, node_ranks=min(4, tp),
    )  # fmt: skip


CASES = {
    "small_fp4_swa_tp8": (small_cfg(8), dict(rows=16, ctx=40, band="reference", seed=11)),
    "small_fp4_global_tp8_baseline": (small_cfg(8), dict(rows=16, ctx=40, global_attn=True, band="baseline", seed=12)),
    "small_bf16_global_tp8": (small_cfg(8), dict(rows=16, ctx=40, global_attn=True, bf16=True, seed=13)),
    "small_fp4_swa_tp2": (small_cfg(2), dict(rows=16, ctx=24, band="baseline", next_global=True, seed=14)),
    "small_fp4_swa_tp1_m5": (small_cfg(1), dict(rows=5, ctx=33, band="baseline", seed=15)),
    "small_bf16_tail_tp4": (small_cfg(4), dict(rows=16, ctx=19, global_attn=True, bf16=True, tail=True, seed=16)),
    "downscaled_m1": (downscaled(), dict(rows=1, ctx=4096, band="baseline", seed=0)),
}
