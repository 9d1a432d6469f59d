"""SGLang-facing: the build that runs after the model loads: which of SGLang's tensors the kernels alias, whether the
loaded model has them in the kernels' shapes, the experts read from the checkpoint, and the bound verify step.

Mirrors the reference's ``muse_spark/runtime/build.py`` (``_alias_specs`` :153-199, ``alias_reasons`` :202-236,
``layer_experts`` :118-147, ``model_weights`` :239-265, ``build`` :272-330): every dense weight, norm weight, residual
coefficient, the router, the lm_head and the rope rows are SGLang's own tensors (no copy); the vocab shard is copied
into the rank's exchange arena (the peers' entry kernels read it); the experts are read from the checkpoint's
safetensors, every expert's rows of this rank (SGLang holds them expert-parallel, the kernels run them tensor-parallel).

SGLang itself is not importable where this package is developed: ``build`` takes the tensor-parallel group, the
checkpoint's expert reader and the model path as optional arguments (tests pass stand-ins, ``runtime/shim.py``) and
asks SGLang's ``runtime_context`` only when they are absent.
"""

from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Callable, Optional

import torch

from ...common import host, symm
from ..b200 import stack as S
from ..b200 import synthetic, weights
from ..config import Config
from .executor import Verify

INDEX = "model.safetensors.index.json"
BF16, F32 = torch.bfloat16, torch.float32
# the target's built object of this process: the draft spec's build (``muse_spark/draft.py``) leaves the draft's weights
# on it, the worker hooks (``runtime/iteration.py``) find it through the model (reference build.py ``TARGET``)
TARGET: Optional[Verify] = None


def alias_specs(model, cfg: Config) -> dict:
    """(layer or None, field) -> (tensor, shape, dtype) of every SGLang tensor the kernels read in place; the field
    names are this package's ``RankTensors`` fields (the reference's ``LayerWeights`` fields, build.py:153-199)."""
    lm = model.model.language_model
    h, mh = cfg.hidden, cfg.moe_hidden
    out = {
        (None, "pre_w0"): (lm.layers[0].input_layernorm._frozen_weight, (h,), BF16),
        (None, "qkv0"): (lm.layers[0].self_attn.qkv_proj.weight, (cfg.qkv_row, h), BF16),
        (None, "lm_head"): (model.lm_head.weight[: cfg.vocab_rank], (cfg.vocab_rank, h), BF16),
        (None, "cos_sin_cache"): (lm.layers[0].self_attn.rotary_emb.cos_sin_cache, None, F32),
    }
    n = len(lm.layers)
    for i, layer in enumerate(lm.layers):
        att, mlp = layer.self_attn, layer.mlp
        nxt = lm.layers[i + 1].input_layernorm if i + 1 < n else lm.norm
        fields = dict(
            o_proj=(att.o_proj.weight, (h, cfg.oproj_k), BF16),
            pooler=(mlp.pre_expert_proj.weight, (mh, h), BF16),
            router=(mlp.gate.weight, (cfg.experts, h), F32),
            unpooler=(mlp.post_expert_proj.weight, (h, mh), BF16),
            expert_bias=(mlp.gate.e_score_correction_bias, (cfg.experts,), F32),
            post_alpha=(layer.post_attention_residual_gate._alpha.view(-1), (h,), F32),
            post_beta=(layer.post_attention_residual_gate._beta.view(-1), (h,), F32),
            post_pre_w=(layer.pre_feedforward_layernorm._frozen_weight, (h,), BF16),
            cross_alpha=(layer.post_feedforward_residual_gate._alpha.view(-1), (h,), F32),
            cross_beta=(layer.post_feedforward_residual_gate._beta.view(-1), (h,), F32),
            cross_pre_w=(nxt._frozen_weight, (h,), BF16),
            cross_post_w=(layer.post_feedforward_layernorm._frozen_weight, (h,), BF16),
            pre_gamma=(mlp.pre_expert_norm._frozen_weight, (mh,), BF16),
            gamma_p1=(mlp.experts.post_expert_norm._frozen_weight, (mh,), BF16),
        )
        if i + 1 < n:
            fields["next_qkv"] = (lm.layers[i + 1].self_attn.qkv_proj.weight, (cfg.qkv_row, h), BF16)
        out.update({(i, k): v for k, v in fields.items()})
    return out


def alias_reasons(model, cfg: Config, rank: int = 0) -> list:
    """Every aliased tensor that is missing or not in the kernels' shape, dtype and row-major layout, and a vocab shard
    that is not this rank's rows (same checks and wording as the reference's build.py:202-236)."""
    try:
        specs = alias_specs(model, cfg)
    except (AttributeError, IndexError, TypeError) as e:
        return [f"the loaded model lacks a tensor the kernels read: {type(e).__name__}: {e}"]
    reasons = []
    for (layer, name), (t, shape, dtype) in specs.items():
        where = name if layer is None else f"layer {layer} {name}"
        if t is None:
            reasons.append(f"{where} is not set")
        elif (shape is not None and tuple(t.shape) != shape) or t.dtype != dtype or not t.is_contiguous():
            reasons.append(f"{where} is {tuple(t.shape)} {t.dtype}, want {shape} {dtype} contiguous")
    lm = model.model.language_model
    if tuple(lm.layers[0].self_attn.rotary_emb.cos_sin_cache.shape[1:]) != (cfg.head_dim,):
        reasons.append(f"the rope rows are not {cfg.head_dim} wide (cos | sin)")
    for name, mod in (("embed_tokens", lm.embed_tokens), ("lm_head", model.lm_head)):
        start = mod.shard_indices.org_vocab_start_index
        if mod.weight.shape[0] != cfg.vocab and start != rank * cfg.vocab_rank:
            reasons.append(f"{name}'s shard starts at row {start}, not {rank * cfg.vocab_rank}")
    if model.lm_head.weight.shape[0] == cfg.vocab and cfg.tp > 1:
        reasons.append("the lm_head is replicated (full vocabulary on every rank)")
    return reasons


class Checkpoint:
    """A safetensors checkpoint directory; a tensor slice reads only its own rows (reference build.py:103-115)."""

    def __init__(self, path):
        self.path = Path(path)
        self.weight_map = json.loads((self.path / INDEX).read_text())["weight_map"]
        self._files: dict = {}

    def slice(self, name: str):
        from safetensors import safe_open  # only a real checkpoint needs it

        f = self.weight_map[name]
        if f not in self._files:
            self._files[f] = safe_open(str(self.path / f), framework="pt")
        return self._files[f].get_slice(name)


def layer_experts(ck, cfg: Config, layer: int, rank: int, device) -> dict:
    """Layer ``layer``'s expert fields of ``RankTensors`` for ``rank`` from a checkpoint (anything with ``slice(name)``
    returning an indexable [E, rows, ...] tensor): codes and scale bytes move unchanged, the per-expert global scales
    fold into the epilogue constants g1_alphas = s2_gate, g1_scale_c = s2_up / s2_gate, g2_alphas = s2_down
    (reference build.py:118-147)."""
    p = f"model.language_model.layers.{layer}.mlp.experts."

    def w13(name):
        return [t.to(device).contiguous() for t in weights.shard_w13(ck.slice(p + name)[:], rank, cfg.tp, cfg.moe_inter)]

    def w2(name):
        return weights.shard_w2(ck.slice(p + name)[:], rank, cfg.tp, cfg.moe_hidden).to(device).contiguous()

    if cfg.is_bf16(layer):
        gate, up = w13("gate_up_proj")
        return dict(gate=gate, up=up, w2=w2("down_proj"))
    (gate_q, up_q), (gate_sf, up_sf) = w13("gate_up_proj"), w13("gate_up_proj_weight_scale")
    s2 = ck.slice(p + "gate_up_proj_weight_scale_2")[:].to(device)
    return dict(
        gate_q=gate_q.view(torch.uint8), gate_sf=gate_sf.view(torch.uint8), up_q=up_q.view(torch.uint8),
        up_sf=up_sf.view(torch.uint8), w2_q=w2("down_proj").view(torch.uint8),
        w2_sf=w2("down_proj_weight_scale").view(torch.uint8), g1_alphas=s2[:, 0].contiguous(),
        g1_scale_c=(s2[:, 1] / s2[:, 0]).contiguous(), g2_alphas=ck.slice(p + "down_proj_weight_scale_2")[:].to(device),
    )  # fmt: skip


def model_case(model, cfg: Config, rank: int, device, rows: int, experts: Callable[[int], dict]) -> synthetic.StackCase:
    """The loaded model as the ``StackCase`` the stack binds: SGLang's tensors in place, ``experts(layer)`` giving each
    layer's expert fields (``layer_experts`` on a checkpoint, or a test's own). Context length 0: the KV pools are the
    serving framework's."""
    specs = alias_specs(model, cfg)
    lm = model.model.language_model
    n = len(lm.layers)
    kvh = cfg.kv_heads_rank
    none_kv = torch.zeros(0, kvh, cfg.head_dim, dtype=BF16, device=device)

    def draw(j: int) -> synthetic.LayerCase:
        tail = j == n - 1
        nxt_global = (not tail) and cfg.is_global(j + 1)
        lc = synthetic.LayerCase(cfg, rows, 0, cfg.is_global(j), cfg.is_bf16(j), nxt_global, tail, "model", 0)
        fields = {k: specs[(j, k)][0] for k in synthetic.RankTensors.__dataclass_fields__ if (j, k) in specs}
        fields.setdefault("next_qkv", None)
        t = synthetic.RankTensors(
            qkv_in=torch.zeros(rows, cfg.qkv_row, dtype=BF16, device=device), k_ctx=none_kv, v_ctx=none_kv,
            stream_in=torch.zeros(rows, cfg.hidden, dtype=F32, device=device),
            next_cos_sin=None if (tail or nxt_global) else torch.zeros(rows, cfg.head_dim, device=device),
            **fields, **experts(j),
        )  # fmt: skip
        lc.ranks.append(t)
        return lc

    embed = lm.embed_tokens.weight
    lo = rank * cfg.vocab_rank
    if embed.shape[0] == cfg.vocab:
        embed = embed[lo : lo + cfg.vocab_rank]
    return synthetic.StackCase(
        cfg, rows, 0, 0, synthetic.LazyLayers(n, draw), embed=[embed], lm_head=[specs[(None, "lm_head")][0]],
        qkv0=[specs[(None, "qkv0")][0]], pre_w0=specs[(None, "pre_w0")][0],
        cos_sin_cache=specs[(None, "cos_sin_cache")][0], ranks=[rank], first_layer=0,
    )  # fmt: skip


# opt-in, as the reference's runtime/build.py:94-100: the fused DFlash2 iteration verifies a token tree of the draft's 15
# likeliest continuations instead of its chain (a 16-row block; greedy requests only: sampled ones run SGLang's step)
TREE_ENV = "SGLANG_MUSE_MEGA_TREE"


def tree_enabled() -> bool:
    return os.environ.get(TREE_ENV, "0") == "1"


def build(model, hf_config, ctx, *, parallel=None, experts: Optional[Callable[[int], dict]] = None, model_path=None,
          cfg: Optional[Config] = None) -> Verify:  # fmt: skip
    """The verify step of a DFlash2 block (``ctx.tokens_per_request`` rows) on this rank: the library loaded (built
    in-tree when stale), the exchange arena on the tensor-parallel group, the weights (SGLang's tensors, the vocab
    shard, the experts read from the checkpoint). The stack itself is bound on the first step, when SGLang's KV pools
    exist (``Verify.forward``)."""
    t0 = time.perf_counter()
    if parallel is None:
        from sglang.srt.runtime_context import get_model, get_parallel  # the serving process

        parallel = get_parallel().tp_group
        model_path = model_path or get_model().model_path
    rank, world = parallel.rank_in_group, parallel.world_size
    device = torch.device("cuda", torch.cuda.current_device())
    cfg = cfg or Config(tp=world)
    assert cfg.tp == world, (cfg.tp, world)
    cfg.validate()
    block = int(ctx.tokens_per_request)
    assert 1 <= block <= cfg.rows, f"a block of {block} rows does not fit the {cfg.rows}-row verify window"
    lib = host.library()
    module = lib.load()
    if experts is None:
        ck = Checkpoint(model_path)
        experts = lambda layer: layer_experts(ck, cfg, layer, rank, device)  # noqa: E731
    layout = S.exchange_layout(cfg, block)
    arena = symm.Arena(lib, layout, device) if world > 1 else symm.LocalArena(layout, device)
    case = model_case(model, cfg, rank, device, block, experts)
    tree = tree_enabled() and block == 16
    summary = (f"TP{cfg.tp}, block {block}{', token tree' if tree else ''}, sm_100a library {lib.path.name}; "
               f"built in {time.perf_counter() - t0:.1f} s")  # fmt: skip
    global TARGET
    TARGET = Verify(cfg, block, case, lib, module, arena, model, rank, device, getattr(parallel, "device_group", None), summary,
                    tree=tree)  # fmt: skip
    try:
        model.built_megakernel = TARGET  # where the hooks of an SGLang without the binding module look it up
    except AttributeError:
        pass
    from . import iteration  # the two hooks on SGLang's DFlash2 worker, before SGLang builds the worker

    iteration.install()
    return TARGET
