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


def draft_checkpoint(cfg, w) -> dict:
    """Unsharded ``DraftWeights`` -> the DFlash2 checkpoint's entries by name (what ``load_shard`` reads)."""
    d = cfg.head_dim
    out = {"fc.weight": w.fc, "hidden_norm.weight": w.hidden_norm, "norm.weight": w.norm,
           "candidate_selector.predecessor_codebook": w.pred_codebook, "candidate_selector.successor_codebook": w.succ_codebook,
           "candidate_selector.hidden_projection.weight": w.hidden_proj}  # fmt: skip
    for i, lw in enumerate(w.layers):
        p, a = f"layers.{i}.", f"layers.{i}.self_attn."
        q, k, v = lw.qkv.split([cfg.q_heads * d, cfg.kv_heads * d, cfg.kv_heads * d])
        gate, up = lw.gate_up.chunk(2)
        out.update({
            p + "input_layernorm.weight": lw.input_norm, p + "post_attention_layernorm.weight": lw.post_norm,
            a + "q_norm.weight": lw.q_norm, a + "k_norm.weight": lw.k_norm,
            a + "q_proj.weight": q, a + "k_proj.weight": k, a + "v_proj.weight": v, a + "o_proj.weight": lw.o,
            p + "mlp.gate_proj.weight": gate, p + "mlp.up_proj.weight": up, p + "mlp.down_proj.weight": lw.down,
            p + "attention_conv.base_kernel": lw.attn_conv.base, p + "attention_conv.kernel_projection.weight": lw.attn_conv.proj,
            p + "mlp_conv.base_kernel": lw.mlp_conv.base, p + "mlp_conv.kernel_projection.weight": lw.mlp_conv.proj,
        })  # fmt: skip
    return out


def draft_hf_config(cfg) -> dict:
    """A DFlash2 ``config.json`` that ``DraftConfig.from_hf`` turns back into ``cfg``."""
    return {
        "architectures": ["DFlash2DraftModel"], "is_causal": False, "layer_types": ["sliding_attention"] * cfg.layers,
        "hidden_act": "silu", "attention_bias": False, "rope_parameters": {"rope_type": "default", "rope_theta": cfg.rope_theta},
        "hidden_size": cfg.hidden, "num_hidden_layers": cfg.layers, "num_attention_heads": cfg.q_heads,
        "num_key_value_heads": cfg.kv_heads, "head_dim": cfg.head_dim, "intermediate_size": cfg.inter, "vocab_size": cfg.vocab,
        "sliding_window": cfg.sliding_window, "rms_norm_eps": cfg.rms_eps,
        "dflash_config": {"conv_kernel_size": cfg.conv_taps, "conv_group_size": cfg.conv_group,
                          "target_layer_ids": list(cfg.capture), "mask_token_id": cfg.mask_id, "selector_rank": cfg.selector_rank,
                          "selector_top_k": cfg.top_k, "output_multiplier": cfg.output_multiplier,
                          "final_logit_softcapping": cfg.softcap},
    }  # fmt: skip


class FakeRequest:
    def __init__(self, rid: str, temperature: float = 1.0, top_k: int = 1, top_p: float = 1.0, seed=None):
        self.rid = rid
        self.sampling_params = NS(temperature=temperature, top_k=top_k, top_p=top_p, sampling_seed=seed)


class FakeMode:
    def __init__(self, name: str = "decode"):
        self.name = name

    def is_extend(self) -> bool:
        return self.name == "extend"

    def is_idle(self) -> bool:
        return self.name == "idle"


def plain_sampling_info(**over):
    """A sampling_info with nothing that edits the logits."""
    base = dict(penalizer_orchestrator=None, need_min_p_sampling=False, has_custom_logit_processor=False, grammar_mask=None,
                logit_bias=None, sampling_mask_batch_indices=None)  # fmt: skip
    base.update(over)
    return NS(**base)


def decode_batch(reqs, spec_info, seq_lens=None, req_pool_indices=None, mode: str = "decode", sampling_info="plain", **over):
    """A stand-in of the scheduler's batch as the DFlash2 worker's step sees it."""
    b = NS(forward_mode=FakeMode(mode), is_extend_in_batch=False, reqs=list(reqs), spec_info=spec_info, seq_lens=seq_lens,
           req_pool_indices=req_pool_indices, has_grammar=False, return_logprob=False,
           sampling_info=plain_sampling_info() if sampling_info == "plain" else sampling_info)  # fmt: skip
    for k, v in over.items():
        setattr(b, k, v)
    return b
