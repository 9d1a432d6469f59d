"""CPU restatement of one greedy verify step over a run of decoder layers: entry, layer 0's head, the layers, the
vocab-sharded logits, the greedy accept. Chains the per-layer oracle the way the reference's ``Stack`` chains its
launches (``sm103/verify.py:400-470``: each layer reads its predecessor's qkv row and residual stream).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs.
"""

from __future__ import annotations

from dataclasses import replace

import torch

from . import cases, dflash_accept
from . import muse_layer as O


def run_stack(case, tokens: torch.Tensor, pos: int, forced_accept=None, b_live=None) -> dict:
    """``case``: a synthetic ``StackCase`` with every rank of the world drawn. Returns per-rank layer values, the
    gathered soft-capped logits and the accept."""
    cfg = case.cfg
    n = cfg.tp
    ent = O.entry(tokens, case.embed, case.pre_w0, cfg.rms_eps, cfg.rms_eps)
    cos_sin = case.cos_sin_cache[pos : pos + case.rows]
    qkv = [O.qkv_rowops(ent["normed"], case.qkv0[r], cfg.q_heads_rank, cfg.kv_heads_rank, cfg.q_scale, cfg.rms_eps,
                        None if cfg.is_global(0) else cos_sin) for r in range(n)]  # fmt: skip
    qkv_first = qkv
    stream = [ent["residual"] for _ in range(n)]
    assert pos == case.ctx, "the window starts where the drawn context ends"
    per_layer = []
    for lc in case.layers:
        rl = [replace(x, qkv=qkv[r], stream_in=stream[r], next_cos_sin=None if x.next_cos_sin is None else cos_sin)
              for r, x in enumerate(cases.rank_layers(lc))]  # fmt: skip
        out = O.run_layer(rl, cfg.node_ranks, b_live=b_live)
        per_layer.append(out)
        stream = [o["stream_out"] for o in out]
        if not lc.tail:
            qkv = [o["qkv_next"] for o in out]
    hidden = per_layer[-1][0]["h3_next"]
    logits = O.logits_out(hidden, case.lm_head, cfg.output_multiplier, cfg.softcap)
    live = b_live or case.rows
    acc = dflash_accept.greedy_accept(tokens[:live], logits[:live], pos, forced_accept)
    return dict(entry=ent, qkv0=qkv_first, layers=per_layer, hidden=hidden, logits=logits, accept=acc)
