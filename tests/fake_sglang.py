"""A stand-in for a loaded SGLang Muse Spark model, built from a synthetic ``StackCase`` of one rank: the attribute paths
the runtime's ``alias_specs`` reads (reference ``runtime/build.py:47-97`` lists them), holding the case's tensors."""

from types import SimpleNamespace as NS

import torch


def _norm(w):
    return NS(_frozen_weight=w)


def fake_model(case, slot: int = 0, device="cpu"):
    cfg = case.cfg
    dev = lambda t: None if t is None else t.to(device)  # noqa: E731
    layers = []
    n = len(case.layers)
    drawn = [case.layers[j] for j in range(n)]
    for j, lc in enumerate(drawn):
        t = lc.ranks[slot]
        qkv = case.qkv0[slot] if j == 0 else drawn[j - 1].ranks[slot].next_qkv
        layers.append(NS(
            input_layernorm=_norm(dev(case.pre_w0) if j == 0 else dev(drawn[j - 1].ranks[slot].cross_pre_w)),
            self_attn=NS(qkv_proj=NS(weight=dev(qkv)), o_proj=NS(weight=dev(t.o_proj)),
                         rotary_emb=NS(cos_sin_cache=dev(case.cos_sin_cache))),
            mlp=NS(pre_expert_proj=NS(weight=dev(t.pooler)), post_expert_proj=NS(weight=dev(t.unpooler)),
                   gate=NS(weight=dev(t.router), e_score_correction_bias=dev(t.expert_bias)),
                   pre_expert_norm=_norm(dev(t.pre_gamma)), experts=NS(post_expert_norm=_norm(dev(t.gamma_p1)))),
            post_attention_residual_gate=NS(_alpha=dev(t.post_alpha), _beta=dev(t.post_beta)),
            post_feedforward_residual_gate=NS(_alpha=dev(t.cross_alpha), _beta=dev(t.cross_beta)),
            pre_feedforward_layernorm=_norm(dev(t.post_pre_w)),
            post_feedforward_layernorm=_norm(dev(t.cross_post_w)),
        ))  # fmt: skip
    final = _norm(dev(drawn[-1].ranks[slot].cross_pre_w))
    shard = NS(org_vocab_start_index=case.ranks[slot] * cfg.vocab_rank)
    lm = NS(layers=layers, norm=final, embed_tokens=NS(weight=dev(case.embed[slot]), shard_indices=shard))
    return NS(model=NS(language_model=lm), lm_head=NS(weight=dev(case.lm_head[slot]), shard_indices=shard))


def experts_of(case, slot: int = 0, device="cpu"):
    """layer -> the expert fields of ``RankTensors`` (what ``layer_experts`` reads from a checkpoint)."""
    names = ("gate_q", "gate_sf", "up_q", "up_sf", "w2_q", "w2_sf", "g1_alphas", "g1_scale_c", "g2_alphas", "gate", "up", "w2")

    def get(layer: int) -> dict:
        t = case.layers[layer].ranks[slot]
        return {k: getattr(t, k).to(device) for k in names if getattr(t, k) is not None}

    return get


class FakeCheckpoint:
    """``Checkpoint.slice`` over in-memory tensors named like the safetensors entries of a layer's experts."""

    def __init__(self, tensors: dict):
        self.tensors = tensors

    def slice(self, name: str) -> torch.Tensor:
        return self.tensors[name]
