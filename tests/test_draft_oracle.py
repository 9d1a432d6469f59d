"""The CPU restatement of the DFlash2 draft step against outputs of the reference's own functions
(``tests/golden/draft.pt``, made by ``tests/golden/make_draft_golden.py``) on the seeded cases re-created here."""

from pathlib import Path

import pytest
import torch

from oracle import dflash_draft as D
from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic
from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig

GOLD = torch.load(Path(__file__).parent / "golden" / "draft.pt", weights_only=False)
CFG = DraftConfig(**{k: tuple(v) if isinstance(v, list) else v for k, v in GOLD["cfg"].items()})


def run_case(g):
    case = synthetic.draft_case(CFG, g["ranks"], g["rows"], g["pos"], g["commit"], g["seed"])
    kv = D.DraftKV.empty(CFG, g["ranks"], g["pos"] + g["rows"])
    kvh = CFG.kv_heads // g["ranks"]
    n_hist = g["pos"] - g["commit"]
    for r in range(g["ranks"]):
        for li in range(CFG.layers):
            kv.k[r][li][:n_hist] = case.hist_k[li][:, r * kvh : (r + 1) * kvh]
            kv.v[r][li][:n_hist] = case.hist_v[li][:, r * kvh : (r + 1) * kvh]
    return case, kv, D.draft_step(CFG, case.shards, kv, case.caps, case.anchor, g["pos"], g["commit"], g["rows"])


def ulps_apart(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (a.view(torch.int16).int() - b.view(torch.int16).int()).abs()


@pytest.mark.parametrize("name", sorted(GOLD["cases"]))
def test_draft_step_matches_the_reference(name):
    g = GOLD["cases"][name]
    case, kv, got = run_case(g)
    # the context rows: bit-exact (GEMMs in f64, one rounding; no reduction-order freedom)
    for r, pr in enumerate(g["per_rank"]):
        for li in range(CFG.layers):
            k, v = got["ctx"]["kv"][r][li]
            assert torch.equal(k, pr["ctx_k"][li]) and torch.equal(v, pr["ctx_v"][li]), (r, li)
            lo = g["pos"] - g["commit"]
            assert torch.equal(kv.k[r][li][lo : g["pos"] + g["rows"]], pr["kv_k"][li]), (r, li)
            assert torch.equal(kv.v[r][li][lo : g["pos"] + g["rows"]], pr["kv_v"][li]), (r, li)
    # the block: the per-head f64 softmax here and the reference's batched one may differ in the last f64 bits before
    # the bf16 rounding; everything else is the same arithmetic. Hold y to one bf16 ulp on a vanishing fraction of elements.
    apart = ulps_apart(got["y"], g["y"])
    assert int(apart.max()) <= 1 and float((apart > 0).float().mean()) < 1e-3, (int(apart.max()), float((apart > 0).float().mean()))
    if int(apart.max()) == 0:
        assert torch.equal(got["cand"], g["cand"]) and torch.equal(got["unary"], g["unary"])
        assert torch.equal(got["scores"], g["scores"]) and torch.equal(got["tokens"], g["tokens"])
    # the head on the REFERENCE's y: candidates, lattice and walk are exact functions of y
    cand, unary, _ = D.candidates(CFG, case.shards, g["y"][1:])
    assert torch.equal(cand, g["cand"]) and torch.equal(unary, g["unary"])
    scores, _ = D.lattice(case.shards[0][0], g["y"][1:], cand, unary, case.anchor)
    assert torch.equal(scores, g["scores"])
    drafts, _ = D.walk(cand, scores)
    assert torch.equal(torch.cat([torch.tensor([case.anchor]), drafts]), g["tokens"])


def test_topk_ties_go_to_the_smaller_id():
    vals = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0]])
    ids = torch.tensor([[9, 7, 2, 5, 4]])
    v, i = D.topk_low_id(vals, ids, 3)
    assert i.tolist() == [[2, 4, 7]] and v.tolist() == [[3.0, 3.0, 3.0]]


def test_conv_row_zero_has_no_second_tap():
    x = torch.randn(4, 32).to(torch.bfloat16)
    delta = torch.randn(4, 2, 2).to(torch.bfloat16)
    base = torch.randn(2, 32).to(torch.bfloat16)
    out = D.grouped_conv(x, delta, base)
    want0 = ((base[0].float() + delta[0, 0].float().repeat_interleave(16)) * x[0].float()).to(torch.bfloat16)
    assert torch.equal(out[0], want0)
