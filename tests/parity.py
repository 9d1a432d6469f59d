"""Shared checks of the GPU parity tests: the reference's per-stage method (muse_spark.py:738-743): every oracle stage is
fed the kernel's own inputs, so each stage is held to its own bound."""

import torch

from oracle import muse_layer as O
from oracle.cases import rank_layers

FLOAT_STAGES = ("x_attn", "branch", "stream_mid", "h3", "pooled", "logits", "w", "x", "x_scale", "zb", "y", "ffn_out",
                "stream_out", "h3_next", "qkv_next")  # fmt: skip
# end-to-end bounds against the unforced golden outputs (relative L2 per row), as the reference's numerics table for the
# whole path (muse_spark/spec.py:178-193): attention 6e-3, post-attention 5e-3, MoE output 0.15, layer output 5e-2
E2E = {"x_attn": 6e-3, "branch": 6e-3, "stream_mid": 5e-3, "h3": 6e-3, "pooled": 8e-3, "logits": 5e-3,
       "zb": 0.15, "y": 0.15, "ffn_out": 0.15, "stream_out": 5e-2, "h3_next": 5e-2, "qkv_next": 8e-2}  # fmt: skip


def nvfp4_rows_close(codes, sf, ref_codes, ref_sf, what):
    """The reference's NVFP4 boundary-flip rule (test_verify_step.py:54-75): scale bytes within one e4m3 step, at most
    1 % of the codes differ (an approximate rsqrt moves a value across a rounding boundary, never further)."""
    dsf = (sf.int() - ref_sf.int()).abs()
    assert int(dsf.max()) <= 1, f"{what}: scale bytes differ by {int(dsf.max())}"
    same_sf = (dsf == 0).repeat_interleave(8, -1)
    c, r = O.nibbles_unpack(codes.cpu()), O.nibbles_unpack(ref_codes.cpu())
    flips = ((c != r) & same_sf.cpu().repeat_interleave(2, -1)).float().mean().item()
    assert flips <= 0.01, f"{what}: {flips:.4f} of the codes differ"
    assert float((dsf != 0).float().mean()) <= 0.01, f"{what}: too many scale bytes moved"


def check_world(world, ranks_to_check, b_live=None, golden=None):
    """Runs nothing: compares the world's device values against the oracle fed those values."""
    case = world.case
    cfg = case.cfg
    got = [{k: v.detach().cpu() for k, v in r.values().items()} for r in world.ranks]
    forced = [dict(g) for g in got]
    ref = O.run_layer(rank_layers(case), cfg.node_ranks, forced=forced, b_live=b_live)
    report = {}
    for r in ranks_to_check:
        g, o = got[r], ref[r]
        assert torch.equal(g["ids"], o["ids"]), f"rank {r}: routed ids differ from the oracle's on the kernel's logits"
        for name in FLOAT_STAGES:
            if name not in o:
                continue
            mx, rel, ok = O.compare(g[name], o[name], name)
            report[(r, name)] = rel
            assert ok, f"rank {r} stage {name}: rel {rel:.3e} > {O.TOLERANCES[name]:.1e} (max abs {mx:.3e})"
        if not case.bf16:
            nvfp4_rows_close(g["xq"], g["x_sf"], o["xq"], o["x_sf"], f"rank {r} expert input")
        if golden is not None and r in golden["ranks"]:
            for name, tol in E2E.items():
                if name in golden["outputs"][r] and name in g:
                    _, rel, _ = O.compare(g[name], golden["outputs"][r][name], name, tol=tol)
                    assert rel <= tol, f"rank {r} {name} against the golden output: rel {rel:.3e} > {tol}"
    return report
