"""Seeded synthetic DFlash2 draft weights at the checkpoint's scales (there is no checkpoint to read): dense rows
~ N(0, 1 / K) in bf16, conv base kernels N(0, 0.05) with tap 0 near 1, conv projections sigma 0.01, norms 1 + 0.1 N,
codebooks sigma 0.05, W_P sigma 0.01 - the distributions of the reference's ``test/kernels/synthetic.py:271-337``.
The unsharded model is drawn once; ``weights.shard`` cuts a rank's part, so every world size sees the same model."""

from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from .weights import ConvWeights, DraftConfig, DraftWeights, LayerWeights, TargetShared, shard


def _draw(gen: torch.Generator, shape, std: float) -> torch.Tensor:
    return (torch.randn(shape, generator=gen) * std).to(torch.bfloat16)


def _near_one(gen: torch.Generator, n: int) -> torch.Tensor:
    return (1 + _draw(gen, (n,), 0.1).float()).to(torch.bfloat16)


def draft_weights(cfg: DraftConfig, seed: int = 0) -> DraftWeights:
    g = torch.Generator().manual_seed(1000 + seed)
    h, d = cfg.hidden, cfg.head_dim

    def conv() -> ConvWeights:
        base = _draw(g, (2, cfg.conv_taps, h), 0.05)
        base[:, 0] += 1
        return ConvWeights(base, _draw(g, (cfg.coeffs, h), 0.01))

    layers: List[LayerWeights] = []
    for _ in range(cfg.layers):
        layers.append(
            LayerWeights(
                input_norm=_near_one(g, h),
                post_norm=_near_one(g, h),
                q_norm=_near_one(g, d),
                k_norm=_near_one(g, d),
                qkv=_draw(g, ((cfg.q_heads + 2 * cfg.kv_heads) * d, h), h**-0.5),
                o=_draw(g, (h, cfg.q_heads * d), (cfg.q_heads * d) ** -0.5),
                gate_up=_draw(g, (2 * cfg.inter, h), h**-0.5),
                down=_draw(g, (h, cfg.inter), cfg.inter**-0.5),
                attn_conv=conv(),
                mlp_conv=conv(),
            )
        )
    return DraftWeights(
        layers,
        fc=_draw(g, (h, cfg.features * h), (cfg.features * h) ** -0.5),
        hidden_norm=_near_one(g, h),
        norm=_near_one(g, h),
        pred_codebook=_draw(g, (cfg.vocab, cfg.selector_rank), 0.05),
        succ_codebook=_draw(g, (cfg.vocab, cfg.selector_rank), 0.05),
        hidden_proj=_draw(g, (cfg.selector_rank, h), 0.01),
    )


def target_shared(cfg: DraftConfig, seed: int = 0) -> TargetShared:
    g = torch.Generator().manual_seed(2000 + seed)
    return TargetShared(_draw(g, (cfg.vocab, cfg.hidden), 1.0), _draw(g, (cfg.vocab, cfg.hidden), cfg.hidden**-0.5))


@dataclass
class DraftCase:
    """One seeded draft step: the unsharded model, every rank's shard, the state the step starts from (the last verify's
    captured residuals of its window rows, the anchor, the position, the commit length) and ``ctx`` earlier positions whose
    context K / V rows the draft's pools already hold (drawn, not computed: any bf16 rows serve)."""

    cfg: DraftConfig
    ranks: int
    rows: int
    w: DraftWeights
    t: TargetShared
    shards: list  # [(DraftWeights, TargetShared)] per rank
    caps: torch.Tensor  # f32 [features, rows, H]
    anchor: int
    pos: int
    commit: int
    hist_k: list  # per layer bf16 [pos - commit, kv_heads, D]
    hist_v: list


def draft_case(cfg: DraftConfig, ranks: int, rows: int, pos: int, commit: int, seed: int = 0) -> DraftCase:
    w, t = draft_weights(cfg, seed), target_shared(cfg, seed)
    g = torch.Generator().manual_seed(3000 + seed)
    caps = torch.randn(cfg.features, rows, cfg.hidden, generator=g)
    anchor = int(torch.randint(0, cfg.vocab, (1,), generator=g))
    n_hist = pos - commit
    hist_k = [_draw(g, (n_hist, cfg.kv_heads, cfg.head_dim), 1.0) for _ in range(cfg.layers)]
    hist_v = [_draw(g, (n_hist, cfg.kv_heads, cfg.head_dim), 1.0) for _ in range(cfg.layers)]
    return DraftCase(cfg, ranks, rows, w, t, [shard(cfg, w, t, r, ranks) for r in range(ranks)], caps, anchor, pos, commit,
                     hist_k, hist_v)  # fmt: skip


def device_shard(cfg: DraftConfig, rank: int, ranks: int, device, seed: int = 0) -> DraftWeights:
    """One rank's shard drawn directly on the device at the same scales (timing runs at the public size: the unsharded
    model is 9.8 GB and is never materialised; shards of different ranks are independent draws, the replicated tensors are
    keyed by the seed alone)."""
    g = torch.Generator(device=device).manual_seed(4000 + seed * 16 + rank)
    gr = torch.Generator(device=device).manual_seed(5000 + seed)  # replicated tensors: the same on every rank
    h, d = cfg.hidden, cfg.head_dim
    q, kv, inter = cfg.q_rank(ranks), cfg.kv_rank(ranks), cfg.inter // ranks

    def draw(gen, shape, std):
        return (torch.randn(shape, generator=gen, device=device) * std).to(torch.bfloat16)

    def near_one(n):
        return (1 + draw(gr, (n,), 0.1).float()).to(torch.bfloat16)

    def conv():
        base = draw(gr, (2, cfg.conv_taps, h), 0.05)
        base[:, 0] += 1
        return ConvWeights(base, draw(gr, (cfg.coeffs, h), 0.01))

    layers = [
        LayerWeights(
            input_norm=near_one(h), post_norm=near_one(h), q_norm=near_one(d), k_norm=near_one(d),
            qkv=draw(g, ((q + 2 * kv) * d, h), h**-0.5), o=draw(g, (h, q * d), (cfg.q_heads * d) ** -0.5),
            gate_up=draw(g, (2 * inter, h), h**-0.5), down=draw(g, (h, inter), cfg.inter**-0.5),
            attn_conv=conv(), mlp_conv=conv(),
        )
        for _ in range(cfg.layers)
    ]  # fmt: skip
    return DraftWeights(
        layers, fc=draw(g, (h // ranks, cfg.features * h), (cfg.features * h) ** -0.5), hidden_norm=near_one(h), norm=near_one(h),
        pred_codebook=draw(gr, (cfg.vocab, cfg.selector_rank), 0.05), succ_codebook=draw(gr, (cfg.vocab, cfg.selector_rank), 0.05),
        hidden_proj=draw(gr, (cfg.selector_rank, h), 0.01),
    )  # fmt: skip
