"""CPU restatement of the tail of a DFlash2 verify step: per-row first-arg-max of the soft-capped logits, the greedy
prefix accept, the step words, the committed-token ring and the next iteration's feeds.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU legs as the
checker, never by the product path.

Follows the reference's ``test/reference/dflash2.py:362-368`` (first_argmax), ``:649-660`` (greedy_accept),
``sgl_muse_mega/muse_spark/sm103/dflash/head.py:54-55`` (the word indices) and ``:64-86`` (draft_feeds), and the window
feeds of ``kernels/head.cu:39-110`` as its host side uses them (``runtime/iteration.py``). Pinned by
``tests/golden/accept.pt`` (outputs of the reference's own functions on seeded inputs).
"""

from __future__ import annotations

import dataclasses
from typing import Optional

import torch

WORDS = {"P": 0, "ANCHOR": 1, "ACCEPT": 2, "COMMIT": 3, "ITER": 4, "OUT_COUNT": 5}
N_WORDS = 8


def first_argmax(x: torch.Tensor) -> torch.Tensor:
    """Per row: the first NaN if the row has one, else the first maximum (dflash2.py:362-368)."""
    out = torch.empty(x.shape[0], dtype=torch.int64)
    for r in range(x.shape[0]):
        row = x[r]
        nan = torch.isnan(row)
        if bool(nan.any()):
            out[r] = int(torch.nonzero(nan)[0])
        else:
            out[r] = int(torch.nonzero(row == row.max())[0])
    return out


@dataclasses.dataclass
class Accept:
    accept_len: int
    commit_len: int
    bonus: int
    out_tokens: torch.Tensor
    new_pos: int


def greedy_accept(tokens: torch.Tensor, capped_logits: torch.Tensor, pos: int, forced: Optional[int] = None) -> Accept:
    """tokens [B] = [anchor, d_1 .. d_(B-1)], post-softcap f32 logits [B, V] -> the longest prefix of drafts that the
    target's own arg-max confirms, then the bonus token (dflash2.py:649-660). ``forced`` replaces the prefix length
    (clamped to [0, B - 1]) the way the kernel's accept-override table does."""
    t = first_argmax(capped_logits)
    b = tokens.shape[0]
    acc = 0
    while acc < b - 1 and int(tokens[acc + 1]) == int(t[acc]):
        acc += 1
    if forced is not None:
        acc = 0 if forced < 0 else min(int(forced), b - 1)
    out = torch.cat([tokens[1:], torch.zeros(1, dtype=tokens.dtype)])
    out[acc] = t[acc]
    return Accept(acc, acc + 1, int(t[acc]), out, pos + acc + 1)


def step_words(words: torch.Tensor, out_ring: torch.Tensor, acc: Accept, tokens: torch.Tensor):
    """The words and the ring after one accept: P += commit, ANCHOR = bonus, ACCEPT, COMMIT, ITER += 1,
    OUT_COUNT += commit; ring rows [OUT_COUNT, OUT_COUNT + commit) = the accepted drafts then the bonus."""
    w, ring = words.clone(), out_ring.clone()
    cnt = int(w[WORDS["OUT_COUNT"]])
    for j in range(acc.accept_len):
        ring[(cnt + j) % ring.shape[0]] = int(tokens[j + 1])
    ring[(cnt + acc.accept_len) % ring.shape[0]] = acc.bonus
    w[WORDS["P"]] += acc.commit_len
    w[WORDS["ANCHOR"]] = acc.bonus
    w[WORDS["ACCEPT"]] = acc.accept_len
    w[WORDS["COMMIT"]] = acc.commit_len
    w[WORDS["ITER"]] += 1
    w[WORDS["OUT_COUNT"]] += acc.commit_len
    return w, ring


def target_feeds(cos_sin_cache: torch.Tensor, pos: int, rows: int) -> dict:
    """The verify window of the next iteration: rows at positions pos .. pos + rows - 1 in identity cache slots."""
    p = torch.arange(rows) + pos
    return {
        "cos_sin": cos_sin_cache[p.clamp(max=cos_sin_cache.shape[0] - 1)],
        "loc": p.int(),
        "kv_len": torch.tensor([pos + rows], dtype=torch.int32),
    }


def draft_feeds(dcos_sin_cache: torch.Tensor, pos: int, commit: int, b: int, dring: int) -> dict:
    """The draft model's 2 b rows: [0, b) the block at pos .., [b, 2 b) the committed context at pos - commit .. (rows
    past the commit masked: slot -1, rope row pos); slot = position mod the ring; kv_len = pos + b (head.py:64-86)."""
    q = torch.arange(2 * b)
    live = (q < b) | (q - b < commit)
    p = torch.where(q < b, pos + q, pos - commit + q - b)
    rows = torch.where(live, p, torch.full_like(p, pos))
    return {
        "dcos_sin": dcos_sin_cache[rows.clamp(max=dcos_sin_cache.shape[0] - 1)],
        "dslot": torch.where(live, p % dring, torch.full_like(p, -1)).int(),
        "dkv_len": torch.tensor([pos + b], dtype=torch.int32),
    }


def window_feeds(positions, cos_sin_cache, out_cache_loc, swa_out_cache_loc, seq_lens, req_pool_indices, req_to_token,
                 full_to_swa, kv_row_bytes: int) -> dict:  # fmt: skip
    """The step's feeds from the serving framework's batch (kernels/head.cu:39-110): rope rows by position, int32 cache
    slots, kv_len = seq_len + rows, and the request's position -> byte-offset tables (full and, through the
    full-to-swa map whose index -1 reads the appended last row, sliding-window)."""
    rows = positions.shape[0]
    row = req_to_token[int(req_pool_indices[0])].long()
    out = {
        "cos_sin": cos_sin_cache[positions.long()],
        "loc_full": out_cache_loc.int(),
        "kv_len": torch.tensor([int(seq_lens[0]) + rows], dtype=torch.int32),
        "pt_full": row * kv_row_bytes,
    }
    if swa_out_cache_loc is not None:
        out["loc_swa"] = swa_out_cache_loc.int()
    if full_to_swa is not None:
        out["pt_swa"] = full_to_swa[row].long() * kv_row_bytes
    return out
