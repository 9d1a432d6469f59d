"""CPU restatement of the DFlash2 draft's half of a decode iteration: context update, the block forward through the
draft's layers, the candidate head, the selector lattice and the greedy walk.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU legs as the
checker, never by the product path.

Follows the reference's ``test/reference/dflash2.py``: ``all_reduce`` :214-222, ``rms_norm`` / ``add_rms_norm`` :245-266,
``silu_mul`` :269-272, ``head_norm_rope`` :275-294, ``grouped_conv`` / ``conv_prepare`` / ``conv_finish`` :297-335,
``attention`` :338-361, ``embed`` :364-374, ``topk_low_id`` :391-399, ``context_update`` :410-452,
``draft_layer_normed`` :502-542 (order ``post_ar``, SGLang's), ``draft_block`` :545-567, ``candidates`` :570-584,
``lattice`` :587-606, ``selector_walk`` :609-640, ``draft_step`` :823-846. Precision policy as there: every dot product
accumulates in f64 and is rounded once to bf16, every elementwise step is f32 in the stated operation order. Pinned by
``tests/golden/draft.pt`` (outputs of the reference's own functions on seeded inputs).

The world is walked in lockstep: functions take the list of every rank's shard and return per-rank lists where ranks
differ; ``all_gather`` is then a concatenation in rank order.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import ConvWeights, DraftConfig, rope_cos_sin

BF = torch.bfloat16
F64 = torch.float64


def mm(x: torch.Tensor, w: torch.Tensor, out=BF) -> torch.Tensor:
    """x [M, K] . w [N, K]^T with f64 accumulation, one rounding."""
    xa = x.to(F64)
    cols = [(xa @ w[n : n + 4096].to(F64).T).to(out) for n in range(0, w.shape[0], 4096)]
    return torch.cat(cols, 1)


def _ms(x: torch.Tensor) -> torch.Tensor:
    return x.to(F64).square().mean(-1, keepdim=True).float()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(_ms(xf) + eps) * w.float()).to(BF)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float):
    """-> (normed bf16, residual' bf16): the f32 sum is normed unrounded and stored rounded."""
    s = x.float() + residual.float()
    return (s * torch.rsqrt(_ms(s) + eps) * w.float()).to(BF), s.to(BF)


def all_reduce(parts: List[torch.Tensor]) -> torch.Tensor:
    """bf16 partials summed in rank order in f32, rounded to bf16."""
    acc = parts[0].float()
    for p in parts[1:]:
        acc = acc + p.float()
    return acc.to(BF)


def grouped_conv(x: torch.Tensor, delta: torch.Tensor, base: torch.Tensor) -> torch.Tensor:
    """out[n, ch] = sum_{t <= n} (base[t, ch] + delta[n, t, ch // group]) x[n - t, ch]; f32, one rounding.
    x [B, H], delta [B, taps, groups], base [taps, H]."""
    b, h = x.shape
    taps, groups = delta.shape[1], delta.shape[2]
    per = h // groups
    xf = x.float()
    d = delta.float().repeat_interleave(per, dim=2)  # [B, taps, H]
    out = (base[0].float()[None] + d[:, 0]) * xf
    for t in range(1, taps):
        out[t:] = out[t:] + (base[t].float()[None] + d[t:, t]) * xf[: b - t]
    return out.to(BF)


def conv_prepare(conv: ConvWeights, h: torch.Tensor, taps: int):
    """-> (side-0 conv of h, side-1 coefficients [B, taps, groups], the raw projection [B, 2 taps groups])."""
    c = mm(h, conv.proj)
    c4 = c.view(h.shape[0], 2, taps, -1)
    return grouped_conv(h, c4[:, 0], conv.base[0]), c4[:, 1], c


def head_norm_rope(x: torch.Tensor, w: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor, round_normed: bool):
    """x [n, heads, D]: per-head RMS norm, then neox rotation over the whole head."""
    xf = x.float()
    xn = xf * torch.rsqrt(_ms(xf) + eps) * w.float()
    if round_normed:
        xn = xn.to(BF).float()
    half = xn.shape[-1] // 2
    lo, hi = xn[..., :half], xn[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], -1).to(BF)


def window_attention(q, k, v, pos_q, pos_k, left: int) -> torch.Tensor:
    """Non-causal sliding-window GQA: q [B, qh, D], k / v [n, kvh, D] -> [B, qh D] f64; a query at p sees keys at
    p - left .. p + left; scale D^-0.5."""
    b, qh, d = q.shape
    kvh = k.shape[1]
    grp = qh // kvh
    out = torch.zeros(b, qh, d, dtype=F64)
    seen = (pos_k[None, :] >= pos_q[:, None] - left) & (pos_k[None, :] <= pos_q[:, None] + left)
    for hd in range(qh):
        kk, vv = k[:, hd // grp].to(F64), v[:, hd // grp].to(F64)
        s = (q[:, hd].to(F64) @ kk.T) * d**-0.5
        s = s.masked_fill(~seen, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ vv
    return out.reshape(b, qh * d)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    g = gate.float()
    return (g / (1.0 + torch.exp(-g)) * up.float()).to(BF)


def softcap(x: torch.Tensor, mult: float, cap: float) -> torch.Tensor:
    return torch.tanh(x.float() * mult / cap) * cap


def first_argmax(row: torch.Tensor) -> int:
    nan = torch.isnan(row)
    if bool(nan.any()):
        return int(torch.nonzero(nan)[0])
    return int(torch.nonzero(row == row.max())[0])


def topk_low_id(vals: torch.Tensor, ids: torch.Tensor, k: int):
    """Per row the k largest values, descending, ties to the smaller id."""
    order = torch.argsort(ids, dim=-1, stable=True)
    vals, ids = vals.gather(-1, order), ids.gather(-1, order)
    top = torch.argsort(vals, dim=-1, descending=True, stable=True)[..., :k]
    return vals.gather(-1, top), ids.gather(-1, top)


# ---- (A) context update ------------------------------------------------------------------------------------------


def feats_of(caps: torch.Tensor) -> torch.Tensor:
    """Captured f32 residuals [features, n, H] -> fc's input rows bf16 [n, features H]."""
    return torch.cat([c.to(BF) for c in caps], 1)


def context_update(cfg: DraftConfig, shards: list, feats: torch.Tensor, pos0: int) -> dict:
    """feats [n, features H], row i at position pos0 + i -> ctx_raw / ctx [n, H] (the same on every rank) and per rank,
    per layer the context K (normed, rotated; not rounded in between) and V rows [n, kvh_r, D]."""
    ctx_raw = torch.cat([mm(feats, w.fc) for w, _ in shards], 1)
    ctx = rms_norm(ctx_raw, shards[0][0].hidden_norm, cfg.rms_eps)
    n, d = feats.shape[0], cfg.head_dim
    cos, sin = rope_cos_sin(pos0 + torch.arange(n), d, cfg.rope_theta)
    kv = []
    for w, _ in shards:
        per_layer = []
        for lw in w.layers:
            q_rows = lw.o.shape[1]
            rows = mm(ctx, lw.qkv[q_rows:])
            kvh = rows.shape[1] // (2 * d)
            r4 = rows.view(n, 2, kvh, d)
            per_layer.append((head_norm_rope(r4[:, 0], lw.k_norm, cfg.rms_eps, cos, sin, False), r4[:, 1].clone()))
        kv.append(per_layer)
    return dict(ctx_raw=ctx_raw, ctx=ctx, kv=kv)


# ---- (B) the block ----------------------------------------------------------------------------------------------------


def embed_rows(cfg: DraftConfig, shards: list, anchor: int, rows: int) -> torch.Tensor:
    """The block's input rows [anchor, mask x (rows - 1)] of the vocab-sharded target embedding."""
    n = shards[0][1].embed.shape[0]
    out = []
    for tok in [anchor] + [cfg.mask_id] * (rows - 1):
        out.append(shards[tok // n][1].embed[tok % n].to(BF))
    return torch.stack(out)


@dataclass
class DraftKV:
    """Per rank, per layer K / V by position: bf16 [capacity, kvh_r, D]."""

    k: list
    v: list

    @classmethod
    def empty(cls, cfg: DraftConfig, ranks: int, capacity: int) -> "DraftKV":
        shape = (capacity, cfg.kv_heads // ranks, cfg.head_dim)
        mk = lambda: [[torch.zeros(shape, dtype=BF) for _ in range(cfg.layers)] for _ in range(ranks)]  # noqa: E731
        return cls(mk(), mk())


def layer_forward(cfg: DraftConfig, shards: list, li: int, h: torch.Tensor, residual: torch.Tensor, kv: DraftKV, pos: int) -> dict:
    """One draft layer from its normed input h [B, H] and the residual it was normed from -> every stage's result. The
    replicated stages are computed once; ``q`` / ``o`` / the partials are per rank."""
    b, d, eps = h.shape[0], cfg.head_dim, cfg.rms_eps
    lw0 = shards[0][0].layers[li]
    out = {}
    xa, c_att1, out["c_att"] = conv_prepare(lw0.attn_conv, h, cfg.conv_taps)
    out["xa"] = xa
    positions = pos + torch.arange(b)
    cos, sin = rope_cos_sin(positions, d, cfg.rope_theta)
    lo = max(0, pos - cfg.window_left)
    out["qkv"], out["q"], out["o"], parts = [], [], [], []
    for r, (w, _) in enumerate(shards):
        lw = w.layers[li]
        qh = lw.o.shape[1] // d
        kvh = (lw.qkv.shape[0] // d - qh) // 2
        qkv = mm(xa, lw.qkv)
        q, k, v = qkv.split([qh * d, kvh * d, kvh * d], 1)
        q = head_norm_rope(q.reshape(b, qh, d), lw.q_norm, eps, cos, sin, True)
        kv.k[r][li][pos : pos + b] = head_norm_rope(k.reshape(b, kvh, d), lw.k_norm, eps, cos, sin, True)
        kv.v[r][li][pos : pos + b] = v.reshape(b, kvh, d)
        o = window_attention(q, kv.k[r][li][lo : pos + b], kv.v[r][li][lo : pos + b], positions, torch.arange(lo, pos + b),
                             cfg.window_left).to(BF)  # fmt: skip
        out["qkv"].append(qkv), out["q"].append(q.reshape(b, qh * d)), out["o"].append(o)
        parts.append(mm(o, lw.o))
    out["attn_parts"] = parts
    a = grouped_conv(all_reduce(parts), c_att1, lw0.attn_conv.base[1])
    out["a"] = a
    h2, residual = add_rms_norm(a, residual, lw0.post_norm, eps)
    out["h_post"], out["res_post"] = h2, residual
    xm, c_mlp1, out["c_mlp"] = conv_prepare(lw0.mlp_conv, h2, cfg.conv_taps)
    out["xm"] = xm
    out["gate_up"], out["m"], parts = [], [], []
    for w, _ in shards:
        lw = w.layers[li]
        gu = mm(xm, lw.gate_up)
        gate, up = gu.chunk(2, 1)
        m = silu_mul(gate, up)
        out["gate_up"].append(gu), out["m"].append(m)
        parts.append(mm(m, lw.down))
    out["mlp_parts"] = parts
    out["x"] = grouped_conv(all_reduce(parts), c_mlp1, lw0.mlp_conv.base[1])
    out["residual"] = residual
    return out


def block_forward(cfg: DraftConfig, shards: list, kv: DraftKV, anchor: int, pos: int, rows: int) -> dict:
    """-> the final-normed hidden y [rows, H], every layer's stage record and the input of each layer (h, residual)."""
    x = embed_rows(cfg, shards, anchor, rows)
    w0 = shards[0][0]
    layers, inputs = [], []
    residual: Optional[torch.Tensor] = None
    for li in range(cfg.layers):
        lw = w0.layers[li]
        if residual is None:
            residual, h = x, rms_norm(x, lw.input_norm, cfg.rms_eps)
        else:
            h, residual = add_rms_norm(x, residual, lw.input_norm, cfg.rms_eps)
        inputs.append((h, residual))
        rec = layer_forward(cfg, shards, li, h, residual, kv, pos)
        layers.append(rec)
        x, residual = rec["x"], rec["residual"]
    y, _ = add_rms_norm(x, residual, w0.norm, cfg.rms_eps)
    return dict(y=y, layers=layers, inputs=inputs, embed=embed_rows(cfg, shards, anchor, rows))


# ---- (C) head, lattice, walk -----------------------------------------------------------------------------------------


def candidates_from_logits(cfg: DraftConfig, logits: torch.Tensor):
    """The global top-K of bf16-rounded logits [gamma, V] (ties to the smaller id) and their soft-capped values."""
    lg = logits.to(BF).float()
    ids = torch.arange(lg.shape[1]).expand_as(lg)
    v, i = topk_low_id(lg, ids, cfg.top_k)
    return i, softcap(v, cfg.output_multiplier, cfg.softcap)


def candidates(cfg: DraftConfig, shards: list, y: torch.Tensor):
    """y [gamma, H] (block rows 1..) -> (ids [gamma, K] i64, unary [gamma, K] f32, the bf16-rounded logits [gamma, V]):
    per rank top-K of its vocab rows, then the global top-K of the gathered lists, then the soft cap."""
    vals, ids, logits = [], [], []
    for r, (_, t) in enumerate(shards):
        lg = mm(y, t.lm_head).float()
        n = t.lm_head.shape[0]
        gid = (torch.arange(n) + r * n).expand_as(lg)
        v, i = topk_low_id(lg, gid, cfg.top_k)
        vals.append(v), ids.append(i), logits.append(lg)
    v, i = topk_low_id(torch.cat(vals, 1), torch.cat(ids, 1), cfg.top_k)
    return i, softcap(v, cfg.output_multiplier, cfg.softcap), torch.cat(logits, 1)


def lattice(w, y: torch.Tensor, cand: torch.Tensor, unary: torch.Tensor, anchor: int):
    """score[e, p, c] = unary[e, c] + bf16(sum_r bf16(A[pred(e, p), r] hid[e, r]) S[cand[e, c], r]); pred(0, .) = the
    anchor, pred(e, p) = cand[e - 1, p]. -> (scores f32 [gamma, K, K], hid bf16 [gamma, R])."""
    hid = mm(y, w.hidden_proj)
    return lattice_from_hid(w, hid, cand, unary, anchor), hid


def lattice_from_hid(w, hid: torch.Tensor, cand: torch.Tensor, unary: torch.Tensor, anchor: int) -> torch.Tensor:
    """The lattice from the projected rows hid = bf16(W_P y) [gamma, R]."""
    pred = torch.cat([torch.full((1, cand.shape[1]), anchor, dtype=cand.dtype), cand[:-1]])
    prod = (w.pred_codebook[pred].float() * hid.float()[:, None, :]).to(BF)
    dot = torch.einsum("epr,ecr->epc", prod.to(F64), w.succ_codebook[cand].to(F64))
    return unary[:, None, :] + dot.to(BF).float()


def walk(cand: torch.Tensor, scores: torch.Tensor):
    """Greedy: slot e takes the first arg-max of the score row of slot e - 1's pick (row 0 at slot 0)."""
    toks, picks, prev = [], [], 0
    for e in range(cand.shape[0]):
        idx = first_argmax(scores[e, prev].float())
        toks.append(int(cand[e, idx])), picks.append(idx)
        prev = idx
    return torch.tensor(toks, dtype=torch.int64), torch.tensor(picks, dtype=torch.int64)


# ---- the sampled walk (temperature > 0): dflash2.py:663-700 (Philox4x32-10 uniforms), :609-640 (selector_walk) ----------

PHILOX_M = (0xD2511F53, 0xCD9E8D57)
PHILOX_W = (0x9E3779B9, 0xBB67AE85)
PURPOSE_WALK, PURPOSE_ACCEPT = 0, 1
_M32 = 0xFFFFFFFF


def philox(counter, key):
    """Philox4x32-10 (Salmon et al., SC'11): 4 counter words, 2 key words -> 4 output words."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0, p1 = PHILOX_M[0] * c0, PHILOX_M[1] * c2
        c0, c1, c2, c3 = (p1 >> 32) ^ c1 ^ k0, p1 & _M32, (p0 >> 32) ^ c3 ^ k1, p0 & _M32
        k0, k1 = (k0 + PHILOX_W[0]) & _M32, (k1 + PHILOX_W[1]) & _M32
    return c0, c1, c2, c3


def uniforms(seed: int, stream: int, iteration: int, purpose: int) -> torch.Tensor:
    """u_i in [0, 1), i < 16: the top 24 bits of word i % 4 of philox({iteration, stream, purpose, i / 4}, seed)."""
    seed &= 2**64 - 1
    key = (seed & _M32, seed >> 32)
    out = [(philox((iteration & _M32, stream & _M32, purpose, i // 4), key)[i % 4] >> 8) * 2.0**-24 for i in range(16)]
    return torch.tensor(out, dtype=torch.float32)


def walk_sampled(cand: torch.Tensor, scores: torch.Tensor, u: torch.Tensor, temperature: float):
    """Slot e draws from softmax(score row of slot e - 1's pick / T): index = #{c : u_e >= cumsum(q)_c}, clamped to
    K - 1. -> (tokens, picks, q [gamma, K] f32)."""
    slots, k = cand.shape
    toks, picks, prev = [], [], 0
    q = torch.empty(slots, k, dtype=torch.float32)
    for e in range(slots):
        scaled = scores[e, prev].float() / temperature
        ex = torch.exp(scaled - scaled.max())
        q[e] = ex / ex.sum()
        idx = min(int((u[e] >= torch.cumsum(q[e], 0)).sum()), k - 1)
        toks.append(int(cand[e, idx])), picks.append(idx)
        prev = idx
    return torch.tensor(toks, dtype=torch.int64), torch.tensor(picks, dtype=torch.int64), q


def draft_step(cfg: DraftConfig, shards: list, kv: DraftKV, caps: torch.Tensor, anchor: int, pos: int, commit: int, rows: int) -> dict:
    """(A) + (B) + (C). caps f32 [features, n >= commit, H]: the last verify's captured residuals, row i at position
    pos - commit + i; the first ``commit`` context rows are written to the KV."""
    pos0 = pos - commit
    ctx = context_update(cfg, shards, feats_of(caps), pos0)
    for r in range(len(shards)):
        for li, (k, v) in enumerate(ctx["kv"][r]):
            kv.k[r][li][pos0 : pos0 + commit] = k[:commit]
            kv.v[r][li][pos0 : pos0 + commit] = v[:commit]
    blk = block_forward(cfg, shards, kv, anchor, pos, rows)
    y = blk["y"]
    cand, unary, logits = candidates(cfg, shards, y[1:])
    scores, hid = lattice(shards[0][0], y[1:], cand, unary, anchor)
    drafts, picks = walk(cand, scores)
    tokens = torch.cat([torch.tensor([anchor]), drafts])
    return dict(ctx=ctx, block=blk, y=y, cand=cand, unary=unary, logits=logits, scores=scores, hid=hid, drafts=drafts,
                picks=picks, tokens=tokens)  # fmt: skip
