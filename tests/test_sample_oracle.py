"""The sampled-verify oracle against the reference's own outputs (``tests/golden/sample.pt``): the target distributions
bit for bit in f64, accept length and bonus token exact, scale and mass to 1e-12."""

from pathlib import Path

import pytest
import torch

from oracle import dflash_draft as D
from oracle import dflash_sample as S

GOLDEN = torch.load(Path(__file__).parent / "golden" / "sample.pt")


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_matches_the_reference(name):
    c = GOLDEN[name]
    probs = S.target_probs(c["logits"], c["temperature"], c["top_k"], c["top_p"])
    assert probs.dtype == torch.float64 and torch.equal(probs, c["probs"])
    u = D.uniforms(0x0123456789ABCDEF + c["seed"], 3, 100 + c["seed"], S.PURPOSE_ACCEPT)
    assert torch.equal(u, c["u"])
    a = S.sampled_accept(c["tokens"], probs, c["cand"], c["q"], u, c["block"])
    assert (a.accept_len, a.bonus) == (c["accept_len"], c["bonus"])
    assert a.scale == pytest.approx(c["scale"], rel=1e-12) and a.norm == pytest.approx(c["norm"], rel=1e-12)


def test_the_cases_cover_every_branch():
    lens = {n: c["accept_len"] for n, c in GOLDEN.items()}
    assert any(0 < c["scale"] < 1 for c in GOLDEN.values()), "no prefix accepted with a scaled residual"
    assert 15 in lens.values() and 0 in lens.values()
    assert any(not c["block"] for c in GOLDEN.values()) and any(c["top_k"] < 512 for c in GOLDEN.values())
    kept = [int((c["probs"] > 0).sum(-1).max()) for c in GOLDEN.values() if c["top_k"] < 512 and c["top_p"] >= 1.0]
    assert any(k > 8 for k in kept), "no tie kept at the top-k boundary"


def test_top_p_keeps_ties_together():
    logits = torch.tensor([[2.0, 2.0, 1.0, 1.0, 0.0, -1.0]])
    p = S.target_probs(logits, 1.0, 6, 0.5)
    # the two largest hold 0.61 of the mass: the mass above them is 0 < 0.5, above the next pair 0.61 >= 0.5
    assert (p > 0).tolist() == [[True, True, False, False, False, False]]
    assert p.sum().item() == pytest.approx(1.0)
    p = S.target_probs(logits, 1.0, 3, 1.0)
    assert (p > 0).tolist() == [[True, True, True, True, False, False]]
