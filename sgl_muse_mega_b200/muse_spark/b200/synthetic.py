"""Seeded synthetic weights and inputs of one decoder layer, per rank, in plain row-major layouts.

Plays the part of the reference's ``test/kernels/synthetic.py:56-270`` (keyed generators, one draw per
(seed, name, layer[, rank]); replicated tensors carry no rank in the key so every rank holds identical bytes). Two value
bands are offered for the NVFP4 experts:

  ``"baseline"``   e2m1 codes uniform over the 16 codes, one e4m3 scale per 16 drawn as |N(0,1)| x 0.02, global
                   (per-expert) scales 1.0, KV and activations ~ N(0,1);
  ``"reference"``  the reference's own band (scale exponent field 6 or 7, per-expert scales that put the dequantised
                   weights at RMS 1/sqrt(K), KV ~ U(-0.1, 0.1)) as ``synthetic.py:74-133,372-388``.

Everything is drawn on the CPU so that the CPU oracle and the GPU kernels see the same bytes; the benchmark moves the
tensors to the device once.
"""

from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..config import Config

E2M1_RMS = math.sqrt(sum(v * v for v in (0, 0.5, 1, 1.5, 2, 3, 4, 6)) / 8)


# Draws happen on this device: the CPU by default (oracle and kernels then see the same bytes); the benchmark sets a
# CUDA device to draw its gigabytes of weights in place (a different stream of numbers, same distributions).
_DEVICE = torch.device("cpu")


def set_device(device) -> None:
    global _DEVICE
    _DEVICE = torch.device(device)


def keyed(*key) -> torch.Generator:
    g = torch.Generator(device=_DEVICE)
    g.manual_seed(int.from_bytes(hashlib.sha256(repr(key).encode()).digest()[:7], "little"))
    return g


def normal(shape, std, dtype, *key):
    return (torch.randn(shape, generator=keyed(*key), device=_DEVICE) * std).to(dtype)


def uniform(shape, lo, hi, dtype, *key):
    return (torch.rand(shape, generator=keyed(*key), device=_DEVICE) * (hi - lo) + lo).to(dtype)


def code_bytes(shape, *key):
    return torch.randint(0, 256, shape, generator=keyed(*key), dtype=torch.uint8, device=_DEVICE)


def scale_bytes(shape, band: str, *key):
    g = keyed(*key)
    if band == "reference":
        ex = torch.randint(6, 8, shape, generator=g, dtype=torch.uint8, device=_DEVICE)
        return (ex << 3) | torch.randint(0, 8, shape, generator=g, dtype=torch.uint8, device=_DEVICE)
    v = torch.randn(shape, generator=g, device=_DEVICE).abs() * 0.02
    return v.clamp(max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def _ref_sf_rms() -> float:
    vals = [2.0 ** (e - 7) * (1 + m / 8) for e in (6, 7) for m in range(8)]
    return math.sqrt(sum(v * v for v in vals) / len(vals))


@dataclass
class RankTensors:
    """One rank's weights of one layer plus the successor's head, and the launch inputs; names follow the reference's
    ``LayerWeights`` (``sm103/weights.py:14-41``). Experts: NVFP4 fields or bf16 fields are None per variant."""

    qkv_in: torch.Tensor  # [rows, qkv_row] bf16: this layer's head row
    k_ctx: torch.Tensor  # [ctx, kv_heads_rank, 64] bf16
    v_ctx: torch.Tensor
    stream_in: torch.Tensor  # [rows, H] f32
    o_proj: torch.Tensor  # [H, oproj_k] bf16
    post_alpha: torch.Tensor
    post_beta: torch.Tensor
    post_pre_w: torch.Tensor
    pooler: torch.Tensor  # [P, H] bf16
    router: torch.Tensor  # [E, H] f32
    expert_bias: torch.Tensor
    pre_gamma: torch.Tensor
    gamma_p1: torch.Tensor
    unpooler: torch.Tensor  # [H, P] bf16
    cross_alpha: torch.Tensor
    cross_beta: torch.Tensor
    cross_pre_w: torch.Tensor
    cross_post_w: torch.Tensor
    next_qkv: Optional[torch.Tensor]  # [qkv_row, H] bf16
    next_cos_sin: Optional[torch.Tensor]  # [rows, 64] f32 (None: global successor)
    # NVFP4 experts
    gate_q: Optional[torch.Tensor] = None
    gate_sf: Optional[torch.Tensor] = None
    up_q: Optional[torch.Tensor] = None
    up_sf: Optional[torch.Tensor] = None
    w2_q: Optional[torch.Tensor] = None
    w2_sf: Optional[torch.Tensor] = None
    g1_alphas: Optional[torch.Tensor] = None
    g1_scale_c: Optional[torch.Tensor] = None
    g2_alphas: Optional[torch.Tensor] = None
    # bf16 experts
    gate: Optional[torch.Tensor] = None
    up: Optional[torch.Tensor] = None
    w2: Optional[torch.Tensor] = None


@dataclass
class LayerCase:
    cfg: Config
    rows: int
    ctx: int
    global_attn: bool
    bf16: bool
    next_global: bool
    tail: bool
    band: str
    seed: int
    ranks: list = field(default_factory=list)  # RankTensors per rank

    @property
    def window(self) -> Optional[int]:
        return None if self.global_attn else self.cfg.swa_window

    @property
    def router_mult(self) -> float:
        return self.cfg.output_multiplier

    @property
    def pre_eps(self) -> float:
        return self.cfg.rms_eps


def rope_rows(cfg: Config, positions: torch.Tensor) -> torch.Tensor:
    """{cos[32] | sin[32]} of position x theta^(-2p/64), computed in float64 and stored float32, as the reference's
    identity feeds (``synthetic.py:343-358``)."""
    d = cfg.head_dim
    inv = cfg.rope_theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
    ang = positions.to(torch.float64)[:, None] * inv[None]
    return torch.cat((ang.cos(), ang.sin()), 1).float()


def layer_case(
    cfg: Config,
    *,
    rows: int,
    ctx: int,
    global_attn: bool = False,
    bf16: bool = False,
    next_global: bool = False,
    tail: bool = False,
    band: str = "baseline",
    seed: int = 0,
    layer: int = 2,
    only_ranks: Optional[list] = None,
    experts_subset: Optional[torch.Tensor] = None,
    bias_scale: float = 0.0,
) -> LayerCase:
    """Draws one layer for every rank of ``cfg.tp`` (or ``only_ranks``). ``experts_subset``: only these experts' NVFP4
    bytes are drawn (others zero) and a +1 bias keeps the routing inside the subset, the trick of the reference's
    real-dims CPU test (``test/unit/test_reference.py:463-475``) that bounds CPU memory at full width."""
    cfg.validate()
    H, P, E, I = cfg.hidden, cfg.moe_hidden, cfg.experts, cfg.moe_inter
    i_s, h_s = cfg.inter_rank, cfg.moe_hidden_rank
    bf, f32 = torch.bfloat16, torch.float32
    case = LayerCase(cfg, rows, ctx, global_attn, bf16, next_global, tail, band, seed)
    kv_lo_hi = None if band == "baseline" else (-0.1, 0.1)

    def norm_w(name, n):
        return uniform((n,), 0.8, 1.2, bf, seed, name, layer)

    bias = torch.zeros(E, dtype=f32, device=_DEVICE)
    if bias_scale:
        bias = normal((E,), 1.0, f32, seed, "popularity", layer) * bias_scale
    if experts_subset is not None:
        bias = bias.clone()
        bias[experts_subset.long()] += 1.0
    rep = dict(
        post_alpha=uniform((H,), 0.9, 1.0, f32, seed, "post_alpha", layer),
        post_beta=uniform((H,), 0.4, 0.6, f32, seed, "post_beta", layer),
        post_pre_w=norm_w("post_pre_w", H),
        pooler=normal((P, H), H**-0.5, bf, seed, "pooler", layer),
        router=normal((E, H), H**-0.5, bf, seed, "router", layer).float(),
        expert_bias=bias,
        pre_gamma=norm_w("pre_gamma", P),
        gamma_p1=norm_w("gamma_p1", P),
        unpooler=normal((H, P), P**-0.5, bf, seed, "unpooler", layer),
        cross_alpha=uniform((H,), 0.9, 1.0, f32, seed, "cross_alpha", layer),
        cross_beta=uniform((H,), 0.4, 0.6, f32, seed, "cross_beta", layer),
        cross_pre_w=norm_w("cross_pre_w", H),
        cross_post_w=norm_w("cross_post_w", H),
        stream_in=normal((rows, H), 1.0, f32, seed, "stream_in", layer),
    )
    pos = torch.arange(ctx, ctx + rows)
    cos_sin = None if (next_global or tail) else rope_rows(cfg, pos).to(_DEVICE)
    if band == "reference":
        s2 = 1.0 / (math.sqrt(P) * E2M1_RMS * _ref_sf_rms())
        alphas = dict(
            g1_alphas=uniform((E,), 0.9 * s2, 1.1 * s2, f32, seed, "g1a", layer),
            g1_scale_c=uniform((E,), 0.9, 1.1, f32, seed, "g1c", layer),
            g2_alphas=uniform((E,), 0.9 * s2, 1.1 * s2, f32, seed, "g2a", layer),
        )
    else:
        one = torch.ones(E, device=_DEVICE)
        alphas = dict(g1_alphas=one, g1_scale_c=one.clone(), g2_alphas=one.clone())
    for r in only_ranks if only_ranks is not None else range(cfg.tp):

        def kv(name):
            shape = (ctx, cfg.kv_heads_rank, cfg.head_dim)
            if kv_lo_hi is None:
                return normal(shape, 1.0, bf, seed, name, layer, r)
            return uniform(shape, *kv_lo_hi, bf, seed, name, layer, r)

        t = dict(rep)
        t.update(
            qkv_in=normal((rows, cfg.qkv_row), 1.0, bf, seed, "qkv_in", layer, r),
            k_ctx=kv("k_ctx"),
            v_ctx=kv("v_ctx"),
            o_proj=normal((H, cfg.oproj_k), (cfg.oproj_k * cfg.tp) ** -0.5, bf, seed, "o_proj", layer, r),
            next_qkv=None if tail else normal((cfg.qkv_row, H), H**-0.5, bf, seed, "next_qkv", layer, r),
            next_cos_sin=cos_sin,
        )
        if bf16:

            def rows16(name, nrows, k):
                if experts_subset is None:
                    return normal((E, nrows, k), k**-0.5, bf, seed, name, layer, r)
                w = torch.zeros(E, nrows, k, dtype=bf, device=_DEVICE)
                w[experts_subset.long()] = normal((len(experts_subset), nrows, k), k**-0.5, bf, seed, name, layer, r)
                return w

            t.update(gate=rows16("gate", i_s, P), up=rows16("up", i_s, P), w2=rows16("w2", h_s, I))
        else:

            def fp4(name, nrows, k):
                if experts_subset is None:
                    return (
                        code_bytes((E, nrows, k // 2), seed, name, layer, r),
                        scale_bytes((E, nrows, k // 16), band, seed, name + "_sf", layer, r),
                    )
                q = torch.zeros(E, nrows, k // 2, dtype=torch.uint8, device=_DEVICE)
                s = torch.zeros(E, nrows, k // 16, dtype=torch.uint8, device=_DEVICE)
                n = len(experts_subset)
                q[experts_subset.long()] = code_bytes((n, nrows, k // 2), seed, name, layer, r)
                s[experts_subset.long()] = scale_bytes((n, nrows, k // 16), band, seed, name + "_sf", layer, r)
                return q, s

            gq, gs = fp4("gate", i_s, P)
            uq, us = fp4("up", i_s, P)
            wq, ws = fp4("w2", h_s, I)
            t.update(gate_q=gq, gate_sf=gs, up_q=uq, up_sf=us, w2_q=wq, w2_sf=ws, **alphas)
        case.ranks.append(RankTensors(**t))
    return case


@dataclass
class StackCase:
    """A run of decoder layers with the step's head and tail: per rank the vocab shard of the embedding and of the
    lm_head and layer 0's qkv weights; replicated: layer 0's pre-attention norm weight and the RoPE cache."""

    cfg: Config
    rows: int
    ctx: int
    seed: int
    layers: list  # LayerCase per layer, in order
    embed: list  # per drawn rank: [vocab_rank, H] bf16
    lm_head: list  # per drawn rank: [vocab_rank, H] bf16
    qkv0: list  # per drawn rank: [qkv_row, H] bf16
    pre_w0: torch.Tensor  # [H] bf16
    cos_sin_cache: torch.Tensor  # [positions, 64] f32
    ranks: list  # the ranks drawn, in the order of the per-rank lists
    first_layer: int = 0  # model index of layers[0]


class LazyLayers:
    """The layers of a stack drawn on demand, one ``LayerCase`` per access and none kept: a 62-layer model's plain
    weights never sit in memory together."""

    def __init__(self, n: int, draw):
        self.n, self.draw = n, draw

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, j: int) -> LayerCase:
        if not 0 <= j < self.n:
            raise IndexError(j)
        return self.draw(j)


def stack_case(cfg: Config, *, n_layers: int, rows: int, ctx: int, seed: int = 0, band: str = "baseline",
               only_ranks: Optional[list] = None, max_pos: Optional[int] = None, first_layer: int = 0,
               lazy: bool = False) -> StackCase:  # fmt: skip
    """Layers ``first_layer .. first_layer + n_layers - 1`` of a model of ``cfg.layers`` layers with the variants the
    model gives them (sliding-window / global by ``cfg.is_global``, bf16 experts by ``cfg.bf16_moe_layers``); the last
    drawn layer is the tail (its cross-layer norm is the final norm, no successor head)."""
    ranks = list(only_ranks) if only_ranks is not None else list(range(cfg.tp))
    bf = torch.bfloat16

    def draw(j: int) -> LayerCase:
        i = first_layer + j
        tail = j == n_layers - 1
        return layer_case(cfg, rows=rows, ctx=ctx, global_attn=cfg.is_global(i), bf16=cfg.is_bf16(i),
                          next_global=(not tail) and cfg.is_global(i + 1), tail=tail, band=band, seed=seed, layer=i,
                          only_ranks=ranks)  # fmt: skip

    layers = LazyLayers(n_layers, draw) if lazy else [draw(j) for j in range(n_layers)]
    H = cfg.hidden
    cache = rope_rows(cfg, torch.arange(max_pos or (ctx + 64 * rows))).to(_DEVICE)
    return StackCase(
        cfg, rows, ctx, seed, layers,
        embed=[normal((cfg.vocab_rank, H), 1.0, bf, seed, "embed", r) for r in ranks],
        lm_head=[normal((cfg.vocab_rank, H), H**-0.5, bf, seed, "lm_head", r) for r in ranks],
        qkv0=[normal((cfg.qkv_row, H), H**-0.5, bf, seed, "qkv0", r) for r in ranks],
        pre_w0=uniform((H,), 0.8, 1.2, bf, seed, "pre_w0"),
        cos_sin_cache=cache,
        ranks=ranks,
        first_layer=first_layer,
    )  # fmt: skip
