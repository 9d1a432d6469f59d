"""Generates ``tests/golden/sample.pt`` from the REFERENCE's own sampled-verify functions.

    python tests/golden/make_sample_golden.py

Imports (read-only) the reference's ``test/reference/dflash2.py`` and runs its ``target_probs``, ``uniforms`` and
``sampled_accept`` on seeded cases (drawn here, stored in the fixture): plain temperature, top-k, top-p, both, logits on a
coarse grid (ties at the top-k and top-p boundaries), block and token-wise verification, drafts the target likes (long
accepts), drafts it does not, and prefixes accepted with a scaled residual (0 < r < 1). Nothing at test time reads the
reference checkout.
"""

from __future__ import annotations

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


VOCAB, ROWS, CANDS = 512, 16, 16
# (name, temperature, top_k, top_p, block, boost of the drafted token's target logit, logit grid or 0, seed)
CASES = [
    ("plain_block_liked", 0.7, VOCAB, 1.0, True, 9.0, 0.0, 1),
    ("plain_block_disliked", 1.0, VOCAB, 1.0, True, 0.0, 0.0, 2),
    ("topk_topp_block", 0.9, 40, 0.9, True, 7.0, 0.0, 3),
    ("topp_tokenwise", 0.8, VOCAB, 0.95, False, 8.0, 0.0, 4),
    ("topk_tokenwise_ties", 1.3, 8, 1.0, False, 4.0, 0.5, 5),
    ("ties_block", 1.0, 24, 0.8, True, 6.0, 1.0, 6),
    ("scaled_residual_block", 0.8, VOCAB, 1.0, True, 4.0, 0.0, 50),
    ("scaled_residual_topk_topp", 1.0, 64, 0.95, True, 5.0, 0.0, 48),
    ("scaled_residual_long_prefix", 0.8, VOCAB, 1.0, True, 6.0, 0.0, 52),
    ("full_accept_block", 0.5, VOCAB, 1.0, True, 30.0, 0.0, 7),
    ("full_accept_tokenwise", 0.5, VOCAB, 1.0, False, 30.0, 0.0, 8),
]


def draw(seed: int, boost: float, grid: float):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(ROWS, VOCAB, generator=g) * 3.0
    if grid:
        logits = (logits / grid).round() * grid
    cand = torch.stack([torch.randperm(VOCAB, generator=g)[:CANDS] for _ in range(ROWS - 1)])
    q = torch.softmax(torch.randn(ROWS - 1, CANDS, generator=g) / 0.7, -1)
    pick = torch.randint(0, CANDS, (ROWS - 1,), generator=g)
    drafts = cand.gather(1, pick[:, None])[:, 0]
    tokens = torch.cat([torch.randint(0, VOCAB, (1,), generator=g), drafts])
    logits[torch.arange(ROWS - 1), drafts] += boost
    return logits, cand, q, tokens


def main() -> None:
    REF = reference_checkout()
    sys.path[:0] = [str(REPO), str(REF), str(REF / "test")]
    from reference import dflash2 as R2  # the reference's DFlash2 oracle

    out = {}
    for name, temp, top_k, top_p, block, boost, grid, seed in CASES:
        logits, cand, q, tokens = draw(seed, boost, grid)
        u = R2.uniforms(0x0123456789ABCDEF + seed, 3, 100 + seed, R2.PURPOSE_ACCEPT)
        probs = R2.target_probs(logits, temp, top_k, top_p)
        a = R2.sampled_accept(tokens, probs, cand, q, u, block)
        out[name] = dict(
            temperature=temp, top_k=top_k, top_p=top_p, block=block, seed=seed, logits=logits, cand=cand, q=q, tokens=tokens,
            u=u, probs=probs, accept_len=a.accept_len, bonus=a.bonus, scale=a.scale, norm=a.norm,
        )  # fmt: skip
        print(name, a.accept_len, a.bonus, f"{a.scale:.4f} {a.norm:.4f}", int((probs > 0).sum(-1).min()), int((probs > 0).sum(-1).max()))
    torch.save(out, HERE / "sample.pt")


if __name__ == "__main__":
    main()
