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

    @classmethod
    def from_hf(cls, cfg: dict) -> "DraftConfig":
        """From a DFlash2 ``config.json`` (a dict). Raises ValueError for the variants the kernels do not implement (another
        architecture, causal or non-sliding layers, an activation other than silu, attention bias, a scaled rope), KeyError
        for a config without the DFlash2 keys; same refusals as the reference's ``sm103/dflash/weights.py:64-110``."""
        d = cfg["dflash_config"]
        checks = {
            f"architectures {cfg['architectures']}": cfg["architectures"] == ["DFlash2DraftModel"],
            "a causal or non-sliding layer": cfg["is_causal"] is False and set(cfg["layer_types"]) == {"sliding_attention"},
            "an activation other than silu, or attention bias": cfg["hidden_act"] == "silu" and not cfg["attention_bias"],
            "a rope type other than default": cfg["rope_parameters"]["rope_type"] == "default",
        }
        for what, ok in checks.items():
            if not ok:
                raise ValueError(what)
        return cls(
            hidden=cfg["hidden_size"], layers=cfg["num_hidden_layers"], q_heads=cfg["num_attention_heads"],
            kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"], inter=cfg["intermediate_size"],
            vocab=cfg["vocab_size"], sliding_window=cfg["sliding_window"],
            rope_theta=float(cfg["rope_parameters"]["rope_theta"]), rms_eps=cfg["rms_norm_eps"],
            conv_taps=d["conv_kernel_size"], conv_group=d["conv_group_size"], capture=tuple(d["target_layer_ids"]),
            mask_id=d["mask_token_id"], selector_rank=d["selector_rank"], top_k=d["selector_top_k"],
            output_multiplier=d["output_multiplier"], softcap=float(d["final_logit_softcapping"]),
        )  # fmt: skip


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


# ---- a DFlash2 checkpoint -> one rank's weights ---------------------------------------------------------------------------------

DRAFT_FILE = "model.safetensors"  # the published draft's single weight file in its directory


def safetensors_reader(path: str):
    """``read(names) -> {name: tensor}`` over a safetensors file (only a real checkpoint needs the package)."""

    def read(names):
        from safetensors import safe_open

        with safe_open(path, framework="pt") as f:
            return {n: f.get_tensor(n) for n in names}

    return read


def load_shard(read, rank: int, ranks: int, cfg: DraftConfig = DraftConfig()) -> DraftWeights:
    """Rank ``rank``'s shard of a DFlash2 checkpoint. ``read(names)`` returns the named bf16 tensors (``safetensors_reader``
    or a test's dict lookup); the entry names are the checkpoint's (reference ``sm103/dflash/weights.py:185-243``): per
    layer the q / k / v / o and gate / up / down projections, four norms and the two grouped convs' base kernels and
    kernel projections; globally fc, two norms and the candidate selector's codebooks and projection. Row-parallel shards
    are copied so that the unsharded tensors can be freed."""
    layers = []
    for i in range(cfg.layers):
        p, a = f"layers.{i}.", f"layers.{i}.self_attn."
        norms = [p + "input_layernorm.weight", p + "post_attention_layernorm.weight", a + "q_norm.weight", a + "k_norm.weight"]
        convs = [f"{p}{c}.{n}" for c in ("attention_conv", "mlp_conv") for n in ("base_kernel", "kernel_projection.weight")]
        proj = [f"{a}{n}_proj.weight" for n in "qkvo"] + [f"{p}mlp.{n}_proj.weight" for n in ("gate", "up", "down")]
        t = read(norms + convs + proj)
        for n, x in t.items():
            if x.dtype != torch.bfloat16:
                raise ValueError(f"{n} is {x.dtype}, not bfloat16")
        whole = LayerWeights(
            *(t[n] for n in norms),
            qkv=torch.cat([t[f"{a}{n}_proj.weight"] for n in "qkv"]), o=t[a + "o_proj.weight"],
            gate_up=torch.cat([t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"]]), down=t[p + "mlp.down_proj.weight"],
            attn_conv=ConvWeights(t[convs[0]], t[convs[1]]), mlp_conv=ConvWeights(t[convs[2]], t[convs[3]]),
        )  # fmt: skip
        layers.append(shard_layer(cfg, whole, rank, ranks))
    sel = "candidate_selector."
    names = ["fc.weight", "hidden_norm.weight", "norm.weight", sel + "predecessor_codebook", sel + "successor_codebook",
             sel + "hidden_projection.weight"]  # fmt: skip
    g = read(names)
    return DraftWeights(layers, fc=block(g[names[0]], rank, ranks).clone(), hidden_norm=g[names[1]], norm=g[names[2]],
                        pred_codebook=g[names[3]], succ_codebook=g[names[4]], hidden_proj=g[names[5]])  # fmt: skip
