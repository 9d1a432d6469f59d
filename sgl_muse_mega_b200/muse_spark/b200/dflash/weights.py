"""The DFlash2 draft's constants and one rank's weights.

Field names follow the reference's ``sgl_muse_mega/muse_spark/sm103/dflash/weights.py:27-150`` (``DraftConfig``,
``ConvWeights``, ``LayerWeights``, ``DraftWeights``) so that a checkpoint loader written for one feeds the other. The
kernels here stream the plain row-major shards (no tile packing): every GEMM of the draft runs on the item engine, whose
items are 64 weight rows x 512 k fetched by one bulk copy per row.

Sharding over ``ranks`` (``shard_layer``, the reference's ``weights.py:158-174`` and ``test/reference/dflash2.py:104-120``):
qkv and gate_up by output heads / rows, o and down by input columns, fc by output rows, embedding and lm_head by vocab rows;
the conv projections, the norms and the selector are replicated.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import List, Tuple

import torch


@dataclass(frozen=True)
class DraftConfig:
    hidden: int = 8192
    layers: int = 5
    q_heads: int = 64
    kv_heads: int = 8
    head_dim: int = 128
    inter: int = 28672
    vocab: int = 202048
    sliding_window: int = 2048  # counts the query's own position
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    conv_taps: int = 2
    conv_group: int = 16
    capture: Tuple[int, ...] = (1, 16, 30, 44, 59)  # target layers whose output residual feeds fc
    mask_id: int = 200002
    selector_rank: int = 256
    top_k: int = 16
    output_multiplier: float = 0.1767766952966369
    softcap: float = 20.0

    @property
    def window_left(self) -> int:
        return self.sliding_window - 1

    @property
    def conv_groups(self) -> int:
        return self.hidden // self.conv_group

    @property
    def features(self) -> int:
        return len(self.capture)

    @property
    def coeffs(self) -> int:
        """Conv coefficients one projection yields per row: (side, tap, group)."""
        return 2 * self.conv_taps * self.conv_groups

    def q_rank(self, ranks: int) -> int:
        return self.q_heads // ranks

    def kv_rank(self, ranks: int) -> int:
        return self.kv_heads // ranks

    def qkv_row(self, ranks: int) -> int:
        return (self.q_rank(ranks) + 2 * self.kv_rank(ranks)) * self.head_dim


@dataclass
class ConvWeights:
    base: torch.Tensor  # [2 sides, taps, H]
    proj: torch.Tensor  # [2 taps groups, H], output n = (side, tap, group)


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    q_norm: torch.Tensor  # [D]
    k_norm: torch.Tensor  # [D]
    qkv: torch.Tensor  # [(q + 2 kv) D, H]: the rank's q rows, then k rows, then v rows
    o: torch.Tensor  # [H, q D]
    gate_up: torch.Tensor  # [2 I_r, H]: the rank's gate rows, then its up rows
    down: torch.Tensor  # [H, I_r]
    attn_conv: ConvWeights
    mlp_conv: ConvWeights


@dataclass
class DraftWeights:
    layers: List[LayerWeights]
    fc: torch.Tensor  # [H / ranks, features H]
    hidden_norm: torch.Tensor
    norm: torch.Tensor
    pred_codebook: torch.Tensor  # [V, R]
    succ_codebook: torch.Tensor  # [V, R]
    hidden_proj: torch.Tensor  # [R, H]


@dataclass
class TargetShared:
    """The target's tensors the draft borrows, the rank's vocab rows of each."""

    embed: torch.Tensor
    lm_head: torch.Tensor


def block(x: torch.Tensor, rank: int, ranks: int, dim: int = 0) -> torch.Tensor:
    n, rem = divmod(x.shape[dim], ranks)
    if rem:
        raise ValueError(f"dim {dim} of {tuple(x.shape)} does not split over {ranks} ranks")
    return x.narrow(dim, rank * n, n)


def shard_layer(cfg: DraftConfig, lw: LayerWeights, rank: int, ranks: int) -> LayerWeights:
    d = cfg.head_dim
    q, k, v = lw.qkv.split([cfg.q_heads * d, cfg.kv_heads * d, cfg.kv_heads * d])
    gate, up = lw.gate_up.chunk(2)
    return replace(
        lw,
        qkv=torch.cat([block(t, rank, ranks) for t in (q, k, v)]).contiguous(),
        o=block(lw.o, rank, ranks, 1).contiguous(),
        gate_up=torch.cat([block(gate, rank, ranks), block(up, rank, ranks)]).contiguous(),
        down=block(lw.down, rank, ranks, 1).contiguous(),
    )


def shard(cfg: DraftConfig, w: DraftWeights, t: TargetShared, rank: int, ranks: int):
    """Unsharded weights -> (rank's DraftWeights, rank's TargetShared)."""
    return (
        replace(w, layers=[shard_layer(cfg, lw, rank, ranks) for lw in w.layers], fc=block(w.fc, rank, ranks).contiguous()),
        TargetShared(block(t.embed, rank, ranks).contiguous(), block(t.lm_head, rank, ranks).contiguous()),
    )


def rope_cos_sin(pos: torch.Tensor, dim: int, theta: float):
    """Rows of the f32 neox cos / sin cache at ``pos`` -> two [n, dim / 2] (reference ``weights.py:243-249``)."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def rope_table(rows: int, dim: int, theta: float) -> torch.Tensor:
    """[rows, dim] f32: cos in the first half of a row, sin in the second (what the draft's kernels gather by position)."""
    c, s = rope_cos_sin(torch.arange(rows), dim, theta)
    return torch.cat([c, s], 1).contiguous()
