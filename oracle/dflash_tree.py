"""CPU restatement of the DFlash2 token tree: the draft head's tree over its lattice and the verify step's tree accept.

TEST INFRASTRUCTURE ONLY: imported by ``tests/`` as the checker, never by the product path.

Follows the reference's ``test/reference/dflash2.py:1295-1391`` (``tree_fan_lp``, ``token_tree``, ``tree_accept``), which
restate ``kernels/dflash/tree.cuh`` (fan_row, walk, accept_leaf). Pinned by ``tests/golden/tree.pt`` (outputs of the
reference's own functions on seeded lattices, ``tests/golden/make_tree_golden.py``).

The window's 16 rows form a tree rooted at the anchor. Every lattice row (slot e, predecessor candidate p) offers its four
best successors with their log-probabilities inside those four; the tree grows best-first by path log-probability (fp32
per operation) until it has 16 rows, then the rows are laid out in preorder with the better-ranked child first.
"""

from __future__ import annotations

import dataclasses
import heapq
import math
from typing import List, Optional, Tuple

import numpy as np
import torch

ROWS, FAN = 16, 4
F = np.float32


def fan_logprobs(vals: List[float]) -> List[float]:
    """The four best scores of a lattice row, best first -> their log-probabilities within them, every operation rounded to
    fp32 (exp and log of the fp32 argument evaluated in double, then rounded: dflash2.py:1304-1313)."""
    top = F(vals[0])
    shifted = [F(F(v) - top) for v in vals]
    total = F(0.0)
    for d in shifted:
        total = F(total + F(math.exp(float(d))))
    lse = F(math.log(float(total)))
    return [float(F(d - lse)) for d in shifted]


@dataclasses.dataclass
class Tree:
    """The window's rows in preorder: parent (-1 for the anchor), depth, ancestor mask (bit j set: row j is the row itself
    or one of its ancestors), token."""

    parent: List[int]
    depth: List[int]
    mask: List[int]
    tokens: List[int]


def token_tree(anchor: int, cand: torch.Tensor, scores: torch.Tensor) -> Tree:
    """cand [gamma, 16] candidate ids per slot, scores [gamma, 16, 16] (slot, predecessor candidate, successor candidate;
    slot 0's predecessor row is row 0). dflash2.py:1325-1372."""
    gamma = cand.shape[0]
    order = torch.argsort(scores, dim=-1, descending=True, stable=True)[..., :FAN]
    best = scores.gather(-1, order).tolist()
    order = order.tolist()

    def offers(slot: int, pred: int) -> List[Tuple[float, int]]:
        """(log-probability, successor candidate index) of the row's four best, best first."""
        return list(zip(fan_logprobs(best[slot][pred]), order[slot][pred]))

    # nodes in the order they join the tree: (slot, candidate index, parent node, depth, rank among the parent's offers)
    nodes = [(-1, 0, -1, 0, 0)]
    heap: list = []  # (-path log-probability, push number, slot, candidate, parent node, rank)
    pushes = 0
    for k, (lp, c) in enumerate(offers(0, 0)):
        heapq.heappush(heap, (-lp, pushes, 0, c, 0, k + 1))
        pushes += 1
    while len(nodes) < ROWS:
        neg, _, slot, c, par, rank = heapq.heappop(heap)  # the largest log-probability, the earlier push on a tie
        me = len(nodes)
        nodes.append((slot, c, par, slot + 1, rank))
        if slot + 1 < gamma:
            for k, (lp, nxt) in enumerate(offers(slot + 1, c)):
                heapq.heappush(heap, (-float(F(F(-neg) + F(lp))), pushes, slot + 1, nxt, me, k + 1))
                pushes += 1
    # preorder, the better-ranked child first
    kids = {i: [] for i in range(ROWS)}
    for i, (_, _, par, _, rank) in enumerate(nodes):
        if par >= 0:
            kids[par].append((rank, i))
    row_of, stack = {}, [0]
    while stack:
        i = stack.pop()
        row_of[i] = len(row_of)
        stack.extend(j for _, j in sorted(kids[i], reverse=True))
    parent, depth, tokens = [0] * ROWS, [0] * ROWS, [0] * ROWS
    for i, (slot, c, par, d, _) in enumerate(nodes):
        r = row_of[i]
        parent[r] = -1 if i == 0 else row_of[par]
        depth[r] = d
        tokens[r] = anchor if i == 0 else int(cand[slot, c])
    mask = [1] + [0] * (ROWS - 1)
    for r in range(1, ROWS):
        mask[r] = mask[parent[r]] | (1 << r)
    return Tree(parent, depth, mask, tokens)


@dataclasses.dataclass
class TreeAccept:
    accept_len: int
    commit_len: int
    bonus: int
    new_pos: int
    committed: List[int]  # the accepted path's tokens, then the bonus
    path: List[int]  # the window rows at depths 1 .. accept_len


def tree_accept(tree: Tree, top1: torch.Tensor, pos: int, forced: Optional[int] = None) -> TreeAccept:
    """A row matches when its token is the target's arg-max at its parent; it is accepted when it and all its ancestors
    match; the leaf is the deepest (= largest, the rows being in preorder) accepted row, or the row ``forced`` names
    (dflash2.py:1375-1391)."""
    t1 = [int(x) for x in top1]
    match = 1
    for r in range(1, ROWS):
        if tree.tokens[r] == t1[tree.parent[r]]:
            match |= 1 << r
    leaf = max(r for r in range(ROWS) if tree.mask[r] & ~match == 0)
    if forced is not None:
        leaf = max(0, min(int(forced), ROWS - 1))
    path = [r for r in range(1, ROWS) if (tree.mask[leaf] >> r) & 1]
    n = tree.depth[leaf]
    return TreeAccept(n, n + 1, t1[leaf], pos + n + 1, [tree.tokens[r] for r in path] + [t1[leaf]], path)
