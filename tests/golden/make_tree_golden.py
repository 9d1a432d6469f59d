"""Generates ``tests/golden/tree.pt`` from the REFERENCE's own token-tree functions.

    MUSE_REFERENCE=<checkout> python tests/golden/make_tree_golden.py

Imports (read-only) the reference's ``test/reference/dflash2.py`` (``token_tree``, ``tree_accept``); the lattices are seeded
draws that the test re-creates, the fixture holds the reference's outputs. Nothing at test time reads the reference checkout.
"""

from __future__ import annotations

import os
import random
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
GAMMA, ROWS = 15, 16
LATTICES = [(s, t) for s in range(6) for t in (0.3, 1.0, 3.0)]  # seed, temperature of the scores


def reference_checkout() -> Path:
    """The reference checkout this script imports read-only: named by the environment, never assumed."""
    if "MUSE_REFERENCE" not in os.environ:
        raise SystemExit("set MUSE_REFERENCE to the reference checkout (this script imports its oracle read-only)")
    return Path(os.environ["MUSE_REFERENCE"])


def lattice(seed: int, temp: float):
    """Distinct candidate ids per slot and N(0, temp^2) scores; seed 5 carries exact ties in every row."""
    g = torch.Generator().manual_seed(1000 + seed)
    cand = torch.randperm(4000, generator=g)[: GAMMA * 16].view(GAMMA, 16) + 7000
    scores = torch.randn(GAMMA, 16, 16, generator=g) * temp
    if seed == 5:
        scores = (scores * 2).round() / 2
    return cand, scores


def peaked():
    cand, _ = lattice(0, 1.0)
    scores = torch.full((GAMMA, 16, 16), -80.0)
    scores[..., :4] = torch.tensor([0.0, -50.0, -60.0, -70.0])
    return cand, scores


def accept_inputs(tree_tokens, tree_mask, seed: int):
    """A target arg-max per row that confirms the path to a seeded leaf and nothing below it."""
    rnd = random.Random(seed)
    leaf = rnd.randrange(ROWS)
    want = [r for r in range(1, ROWS) if (tree_mask[leaf] >> r) & 1]
    t1 = [rnd.randrange(10**6, 2 * 10**6) for _ in range(ROWS)]
    node = 0
    for r in want:
        t1[node] = tree_tokens[r]
        node = r
    return leaf, t1


def main() -> None:
    ref = reference_checkout()
    sys.path[:0] = [str(REPO), str(ref), str(ref / "test")]
    from reference import dflash2 as R2  # the reference's DFlash2 oracle

    out = {"gamma": GAMMA, "lattices": LATTICES, "trees": [], "accepts": []}
    cases = [lattice(s, t) for s, t in LATTICES] + [peaked()]
    for i, (cand, scores) in enumerate(cases):
        tr = R2.token_tree(7 + i, cand, scores)
        out["trees"].append(dict(parent=tr.parent, depth=tr.depth, mask=tr.mask, tokens=tr.tokens))
        leaf, t1 = accept_inputs(tr.tokens, tr.mask, i)
        for forced in (None, (leaf + 5) % ROWS):
            a, path = R2.tree_accept(tr, torch.tensor(t1), 100 + i, forced=forced)
            out["accepts"].append(dict(tree=i, top1=t1, pos=100 + i, forced=forced, accept=a.accept, commit=a.commit, bonus=a.bonus,
                                       new_pos=a.pos, committed=a.committed.tolist(), path=path))  # fmt: skip
    torch.save(out, HERE / "tree.pt")
    print("tree.pt", (HERE / "tree.pt").stat().st_size, "bytes;", len(out["trees"]), "trees,", len(out["accepts"]), "accepts")


if __name__ == "__main__":
    main()
