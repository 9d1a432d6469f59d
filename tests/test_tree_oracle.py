"""The token-tree oracle (``oracle/dflash_tree.py``) against the reference's own outputs (``tests/golden/tree.pt``, made by
``tests/golden/make_tree_golden.py``) and against the tree's defining properties (the reference's
``test/unit/test_dflash_tree.py``): preorder, ancestor masks, distinct siblings ascending by rank, best-first selection."""

import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import make_tree_golden as G  # noqa: E402  (the seeded inputs; nothing here reads the reference)

from oracle import dflash_tree as T  # noqa: E402

GOLD = torch.load(Path(__file__).resolve().parent / "golden" / "tree.pt")
CASES = [G.lattice(s, t) for s, t in GOLD["lattices"]] + [G.peaked()]


@pytest.mark.parametrize("i", range(len(CASES)))
def test_tree_equals_the_references(i):
    cand, scores = CASES[i]
    tr = T.token_tree(7 + i, cand, scores)
    want = GOLD["trees"][i]
    assert (tr.parent, tr.depth, tr.mask, tr.tokens) == (want["parent"], want["depth"], want["mask"], want["tokens"])


@pytest.mark.parametrize("j", range(len(GOLD["accepts"])))
def test_accept_equals_the_references(j):
    a = GOLD["accepts"][j]
    cand, scores = CASES[a["tree"]]
    tr = T.token_tree(7 + a["tree"], cand, scores)
    got = T.tree_accept(tr, torch.tensor(a["top1"]), a["pos"], forced=a["forced"])
    assert (got.accept_len, got.commit_len, got.bonus, got.new_pos, got.committed, got.path) == (
        a["accept"], a["commit"], a["bonus"], a["new_pos"], a["committed"], a["path"])  # fmt: skip


@pytest.mark.parametrize("i", [0, 4, 8, 16])
def test_the_tree_is_a_preorder_tree_of_distinct_siblings(i):
    cand, scores = CASES[i]
    tr = T.token_tree(3, cand, scores)
    assert tr.parent[0] == -1 and tr.depth[0] == 0 and tr.mask[0] == 1 and tr.tokens[0] == 3
    for r in range(1, T.ROWS):
        p = tr.parent[r]
        assert 0 <= p < r and tr.depth[r] == tr.depth[p] + 1 <= G.GAMMA
        assert tr.mask[r] == tr.mask[p] | (1 << r)
        assert tr.tokens[r] in cand[tr.depth[r] - 1].tolist()
    for p in range(T.ROWS):
        kids = [r for r in range(1, T.ROWS) if tr.parent[r] == p]
        assert len({tr.tokens[r] for r in kids}) == len(kids)
        subtree = [[c for c in range(T.ROWS) if (tr.mask[c] >> r) & 1] for r in kids]
        assert all(kids[j + 1] > max(subtree[j]) for j in range(len(kids) - 1))  # a child precedes the next one's subtree


def test_a_peaked_lattice_gives_the_greedy_chain():
    cand, scores = G.peaked()
    tr = T.token_tree(7, cand, scores)
    assert tr.parent == [-1] + list(range(T.ROWS - 1)) and tr.depth == list(range(T.ROWS))
    assert tr.tokens[1:] == [int(cand[e, 0]) for e in range(T.ROWS - 1)]  # every slot's best successor


def test_fan_logprobs_normalise_in_fp32():
    lps = T.fan_logprobs([1.5, 1.25, -0.5, -3.0])
    assert lps[0] > lps[1] > lps[2] > lps[3] and abs(sum(pow(2.718281828459045, x) for x in lps) - 1.0) < 1e-6
    assert all(float(torch.tensor(x, dtype=torch.float32)) == x for x in lps)  # every value is an fp32 number
