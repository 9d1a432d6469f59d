"""Generates ``tests/golden/draft.pt`` from the REFERENCE's own DFlash2 draft functions.

    python tests/golden/make_draft_golden.py

Imports (read-only) the reference's ``test/reference/dflash2.py`` and runs its ``draft_step`` (context update, block
forward, candidates, lattice, greedy walk; SGLang's ``post_ar`` order) over thread-emulated ranks on the seeded synthetic
cases that ``tests/test_draft_oracle.py`` re-creates; the fixture holds the reference's outputs. Nothing at test time reads
the reference checkout.
"""

from __future__ import annotations

import dataclasses
import os
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def reference_checkout() -> Path:
    """The reference checkout this script imports read-only: named by the environment, never assumed."""
    if "MUSE_REFERENCE" not in os.environ:
        raise SystemExit("set MUSE_REFERENCE to the reference checkout (this script imports its oracle read-only)")
    return Path(os.environ["MUSE_REFERENCE"])


# (name, ranks, rows, pos, commit, seed): a window that clips the history (pos > sliding window) and one that does not
CASES = [("tp2_b16", 2, 16, 40, 7, 1), ("tp1_b8", 1, 8, 12, 3, 2), ("tp4_b16", 4, 16, 33, 16, 3)]


PHILOX_CASES = [((0, 0, 0, 0), (0, 0)), ((1, 2, 3, 4), (5, 6)), ((0xFFFFFFFF, 0x12345678, 1, 3), (0xDEADBEEF, 0x0BADF00D))]
SAMPLE_SEED, SAMPLE_TEMP = 0x1234567887654321, 0.7


def small_cfg():
    from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig

    return DraftConfig(hidden=512, layers=2, q_heads=8, kv_heads=4, head_dim=128, inter=1024, vocab=2048, sliding_window=24,
                       mask_id=2002, selector_rank=64, top_k=16)  # fmt: skip


def main() -> None:
    REF = reference_checkout()
    sys.path[:0] = [str(REPO), str(REF), str(REF / "test")]
    from reference import dflash2 as R2  # the reference's DFlash2 oracle

    from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic

    cfg = small_cfg()
    rcfg = R2.DraftConfig(**dataclasses.asdict(cfg))
    out = {"cfg": dataclasses.asdict(cfg), "cases": {}}
    for name, ranks, rows, pos, commit, seed in CASES:
        case = synthetic.draft_case(cfg, ranks, rows, pos, commit, seed)
        feats = torch.cat([c.to(torch.bfloat16) for c in case.caps], 1)

        def run(comm, case=case, feats=feats, ranks=ranks, rows=rows, pos=pos, commit=commit):
            mine, tgt = case.shards[comm.rank]
            lw = [R2.LayerWeights(**{f.name: getattr(l, f.name) for f in dataclasses.fields(l) if "conv" not in f.name},
                                  attn_conv=R2.ConvWeights(l.attn_conv.base, l.attn_conv.proj),
                                  mlp_conv=R2.ConvWeights(l.mlp_conv.base, l.mlp_conv.proj)) for l in mine.layers]  # fmt: skip
            w = R2.DraftWeights(lw, mine.fc, mine.hidden_norm, mine.norm, mine.pred_codebook, mine.succ_codebook, mine.hidden_proj)
            t = R2.TargetShared(tgt.embed, tgt.lm_head)
            kv = R2.DraftKV.empty(rcfg, pos + rows, ranks, torch.bfloat16)
            kvh = cfg.kv_heads // ranks
            for li in range(cfg.layers):
                kv.k[li][: pos - commit] = case.hist_k[li][:, comm.rank * kvh : (comm.rank + 1) * kvh]
                kv.v[li][: pos - commit] = case.hist_v[li][:, comm.rank * kvh : (comm.rank + 1) * kvh]
            state = R2.DecodeState(pos, case.anchor, feats, commit)
            d = R2.draft_step(rcfg, w, t, kv, state, rows, comm, torch.bfloat16)
            return dict(tokens=d.tokens, y=d.y, cand=d.cand, unary=d.unary, scores=d.scores, ctx_k=[k for k, _ in d.ctx],
                        ctx_v=[v for _, v in d.ctx], kv_k=[k[pos - commit : pos + rows].clone() for k in kv.k],
                        kv_v=[v[pos - commit : pos + rows].clone() for v in kv.v])  # fmt: skip

        res = R2.emulate_ranks(run, ranks)
        for r in range(1, ranks):  # the replicated results agree on every rank
            for k in ("tokens", "y", "cand", "unary", "scores"):
                assert torch.equal(res[0][k], res[r][k]), (name, k, r)
        out["cases"][name] = dict(ranks=ranks, rows=rows, pos=pos, commit=commit, seed=seed, tokens=res[0]["tokens"], y=res[0]["y"],
                                  cand=res[0]["cand"], unary=res[0]["unary"], scores=res[0]["scores"],
                                  per_rank=[{k: r[k] for k in ("ctx_k", "ctx_v", "kv_k", "kv_v")} for r in res])  # fmt: skip
        print(name, "tokens", res[0]["tokens"].tolist())
    # the sampled walk: Philox known answers, the step's uniforms, and the walk over each case's lattice
    out["philox"] = [dict(counter=c, key=k, out=R2.philox(c, k)) for c, k in PHILOX_CASES]
    out["sampled"] = {}
    for name, g in out["cases"].items():
        u = R2.uniforms(SAMPLE_SEED, g["pos"], 3, R2.PURPOSE_WALK)
        toks, q = R2.selector_walk(g["cand"], g["scores"], greedy=False, uniforms=u, temperature=SAMPLE_TEMP)
        out["sampled"][name] = dict(u=u, tokens=toks, q=q)
    torch.save(out, HERE / "draft.pt")
    print("wrote", HERE / "draft.pt", (HERE / "draft.pt").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
