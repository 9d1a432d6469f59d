"""CPU restatement of the sampled verify of a DFlash2 step (temperature > 0). TEST INFRASTRUCTURE: the checker for a sampled
accept, never part of the product path.

Follows the reference's ``test/reference/dflash2.py``: ``target_probs`` (:703-727), ``sampled_accept`` (:739-791); the
uniforms are ``oracle.dflash_draft.uniforms`` (Philox4x32-10, ``dflash2.py:676-700``) with purpose 1, coin e - 1 for
prefix length e and uniform 15 for the bonus. Pinned by ``tests/golden/sample.pt`` (``tests/golden/make_sample_golden.py``
runs the reference's own functions on seeded cases).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

PURPOSE_ACCEPT = 1
BONUS_UNIFORM = 15


def target_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """The verify rows' sampling distributions, f64 [rows, V]: softmax of f32(logits / T) over the rows' top_k largest
    values (every value equal to the k-th is kept), then the top-p set inside it (a value stays while the mass of the
    strictly larger ones is below top_p; equal values stand or fall together), renormalised."""
    y = (logits.to(torch.float32) / torch.tensor(temperature, dtype=torch.float32)).to(torch.float64)
    vocab = y.shape[-1]
    if top_k < vocab:
        floor = y.topk(top_k, dim=-1).values[:, top_k - 1 : top_k]
        y = y.masked_fill(y < floor, float("-inf"))
    p = torch.softmax(y, dim=-1)
    if top_p >= 1.0:
        return p
    desc, order = p.sort(dim=-1, descending=True)
    before = desc.cumsum(-1) - desc  # mass ahead of each sorted position
    # a run of equal values takes the mass ahead of its first member
    pos = torch.arange(vocab).expand_as(desc)
    opens = torch.ones_like(desc, dtype=torch.bool)
    opens[:, 1:] = desc[:, 1:] != desc[:, :-1]
    head = torch.where(opens, pos, torch.zeros_like(pos)).cummax(-1).values
    larger = torch.empty_like(p).scatter_(-1, order, before.gather(-1, head))
    kept = torch.where(larger < top_p, p, torch.zeros_like(p))
    return kept / kept.sum(-1, keepdim=True)


@dataclass
class SampledAccept:
    accept_len: int
    bonus: int
    scale: float  # the accepted prefix's probability ratio the residual is scaled by (1 token-wise)
    norm: float   # the mass of the distribution the bonus is drawn from


def sampled_accept(tokens, probs, cand, q, u, block: bool) -> SampledAccept:
    """tokens [B] = the anchor then the drafts, probs [B, V] = ``target_probs`` of the verify rows, cand / q [B - 1, K] =
    each slot's candidates and the walk's probabilities over them (the draft's distribution: q at the candidates, 0
    elsewhere), u [16] the step's uniforms. Token-wise: slot e is accepted while u[e] q_e(d) < p_e(d). Block verification
    (arXiv:2403.10444, Algorithm 2): with r_e = min(r_(e-1) p_e(d) / q_e(d), 1), the longest prefix e (tried from the
    longest) whose coin u[e-1] is below r_e and, for a proper prefix with 0 < r_e < 1, below m / (m + 1 - r_e) with m the
    mass of max(r_e P_e - Q_e, 0). The bonus token: the first id whose running sum of max(s P_a - Q_a, 0) (P alone after a
    full accept) exceeds u[15] times the mass; the last id if none does."""
    gamma, vocab = tokens.shape[0] - 1, probs.shape[1]
    P = probs.to(torch.float64)
    Q = torch.zeros(gamma, vocab, dtype=torch.float64).scatter_(1, cand.long(), q.to(torch.float64))
    drafted = tokens[1:].long()
    p_d = [float(P[e, drafted[e]]) for e in range(gamma)]
    q_d = [float(Q[e, drafted[e]]) for e in range(gamma)]

    def leftover(row: int, s: float) -> torch.Tensor:
        return (s * P[row] - Q[row]).clamp(min=0.0)

    accepted, scale, mass = 0, 1.0, None
    if block:
        ratio = [1.0]
        for e in range(gamma):
            ok = 0.0 < q_d[e] <= 1.0
            ratio.append(min(ratio[-1] * p_d[e] / q_d[e], 1.0) if ok else 0.0)
        for e in range(gamma, 0, -1):
            coin = float(u[e - 1])
            if not coin < ratio[e]:
                continue
            bar, m = ratio[e], None
            if e < gamma and 0.0 < ratio[e] < 1.0:
                m = float(leftover(e, ratio[e]).sum())
                bar = m / (m + 1.0 - ratio[e])
            if coin < bar:
                accepted, scale, mass = e, ratio[e], m
                break
    else:
        while accepted < gamma and 0.0 < q_d[accepted] <= 1.0 and float(u[accepted]) * q_d[accepted] < p_d[accepted]:
            accepted += 1
    dist = P[accepted] if accepted == gamma else leftover(accepted, scale)
    if mass is None:
        mass = float(dist.sum())
    over = (dist.cumsum(0) > float(u[BONUS_UNIFORM]) * mass).nonzero()
    bonus = int(over[0]) if over.numel() else vocab - 1
    return SampledAccept(accepted, bonus, scale, mass)
