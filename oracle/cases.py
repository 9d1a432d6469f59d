"""Adapters from the synthetic layer cases (plain per-rank tensors) to the oracle's ``RankLayer`` records.
Test infrastructure only."""

from __future__ import annotations

from . import muse_layer as O


def rank_layers(case) -> list:
    """``synthetic.LayerCase`` -> [``muse_layer.RankLayer``] (one per rank), same tensors, no copies."""
    cfg, out = case.cfg, []
    for t in case.ranks:
        if case.bf16:
            ex = O.Bf16Experts(t.gate, t.up, t.w2)
        else:
            ex = O.Fp4Experts(
                t.gate_q, t.gate_sf, t.up_q, t.up_sf, t.w2_q, t.w2_sf, t.g1_alphas, t.g1_scale_c, t.g2_alphas
            )
        out.append(
            O.RankLayer(
                w_o=t.o_proj, post_alpha=t.post_alpha, post_beta=t.post_beta, post_pre_w=t.post_pre_w,
                w_pool=t.pooler, w_router=t.router, expert_bias=t.expert_bias, router_mult=case.router_mult,
                route_scale=cfg.route_scale, pre_gamma=t.pre_gamma, pre_eps=case.pre_eps, experts=ex,
                gamma_p1=t.gamma_p1, w_unpool=t.unpooler, x_alpha=t.cross_alpha, x_beta=t.cross_beta,
                x_pre_w=t.cross_pre_w, x_post_w=t.cross_post_w, qkv=t.qkv_in, k_ctx=t.k_ctx, v_ctx=t.v_ctx,
                stream_in=t.stream_in, window=case.window, next_w_qkv=t.next_qkv, next_q_scale=cfg.q_scale,
                next_eps=cfg.rms_eps, next_cos_sin=t.next_cos_sin, next_q_heads=cfg.q_heads_rank,
                next_kv_heads=cfg.kv_heads_rank, topk=cfg.topk,
            )  # fmt: skip
        )
    return out
