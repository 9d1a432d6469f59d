"""Generates ``tests/golden/accept.pt`` from the REFERENCE's own DFlash2 functions.

    python tests/golden/make_accept_golden.py

Imports (read-only) the reference's ``test/reference/dflash2.py`` (first_argmax, greedy_accept, softcap) and the
``draft_feeds`` of its ``sm103/dflash/head.py``; the inputs are seeded draws that the test re-creates, the fixture holds
the reference's outputs. Nothing at test time reads the reference checkout.
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


SEED, ROWS, VOCAB, CASES = 4242, 16, 1000, 12


def draw_case(i: int):
    """Case i's window ids and raw (pre-cap) logits: the logits' arg-max row r is steered to confirm a prefix of i + 1
    drafts (capped at ROWS - 1); case 3 holds an exact tie, case 5 a NaN row."""
    g = torch.Generator().manual_seed(SEED + i)
    logits = torch.randn(ROWS, VOCAB, generator=g) * 8
    tokens = torch.randint(0, VOCAB, (ROWS,), generator=g)
    want = min(i + 1, ROWS - 1) if i != 11 else ROWS - 1
    for r in range(want):
        logits[r, int(tokens[r + 1])] = 90.0 + r
    if i == 3:  # an exact tie on row 0: the lower id wins
        a, b = sorted((int(tokens[1]), (int(tokens[1]) + 17) % VOCAB))
        logits[0, a] = logits[0, b] = 95.0
    if i == 5:  # NaN first
        logits[2, 123] = float("nan")
        logits[2, 700] = float("nan")
    return tokens, logits


def main() -> None:
    REF = reference_checkout()
    sys.path[:0] = [str(REPO), str(REF), str(REF / "test")]
    from reference import dflash2 as R2  # the reference's DFlash2 oracle

    out = {"seed": SEED, "rows": ROWS, "vocab": VOCAB, "cases": []}
    pos = 4099
    for i in range(CASES):
        tokens, logits = draw_case(i)
        capped = R2.softcap(logits, 32**-0.5, 20.0)
        t = R2.first_argmax(capped)
        acc = R2.greedy_accept(tokens, capped, pos)
        out["cases"].append(
            dict(top1=t, accept_len=acc.accept_len, commit_len=acc.commit_len, bonus=acc.bonus, out_tokens=acc.out_tokens,
                 new_pos=acc.new_pos, pos=pos)
        )  # fmt: skip
        pos = acc.new_pos
    try:
        from sgl_muse_mega.muse_spark.sm103.dflash.head import WORDS, draft_feeds

        g = torch.Generator().manual_seed(SEED)
        cache = torch.randn(300, 128, generator=g)
        out["words"] = dict(WORDS)
        out["draft_feeds"] = [
            dict(pos=p, commit=c, b=b, dring=d, **draft_feeds(cache, p, c, b, d))
            for p, c, b, d in ((40, 3, 16, 64), (100, 16, 16, 64), (17, 1, 8, 32), (250, 9, 16, 128))
        ]
    except Exception as e:  # the head module binds native code at import on some checkouts
        print("draft_feeds not generated:", e)
    torch.save(out, HERE / "accept.pt")
    print("accept.pt", (HERE / "accept.pt").stat().st_size, "bytes;", [c["accept_len"] for c in out["cases"]])


if __name__ == "__main__":
    main()
