"""Generates the golden fixtures of ``tests/golden/*.pt`` from the REFERENCE's own torch oracle.

Run once, in a container where the reference checkout is mounted (the environment variable ``MUSE_REFERENCE`` names it):

    MUSE_REFERENCE=<checkout> python tests/golden/make_golden.py

It imports the reference's ``test/reference/muse_spark.py`` read-only, draws the seeded synthetic layer cases of
``sgl_muse_mega_b200.muse_spark.b200.synthetic``, repacks their plain tensors into the reference's kernel layouts with the
reference's own packers (``sm103/weights.py:96-143``) and stores the reference's outputs. The fixtures hold outputs
only; the inputs are re-drawn from the seeds by the tests. Nothing at test time reads the reference checkout.
"""

from __future__ import annotations

import os
import sys
from dataclasses import replace
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def reference_checkout() -> Path:
    """The reference checkout this script imports read-only: named by the environment, never assumed."""
    if "MUSE_REFERENCE" not in os.environ:
        raise SystemExit("set MUSE_REFERENCE to the reference checkout (this script imports its oracle read-only)")
    return Path(os.environ["MUSE_REFERENCE"])

REF = reference_checkout()
sys.path[:0] = [str(REPO), str(REF), str(REF / "test")]

from reference import muse_spark as R  # noqa: E402  (the reference's oracle)
from sgl_muse_mega.muse_spark.sm103 import weights as RW  # noqa: E402  (the reference's packers)

from sgl_muse_mega_b200.muse_spark.b200 import synthetic  # noqa: E402
from sgl_muse_mega_b200.muse_spark.config import Config, downscaled  # noqa: E402

torch.set_num_threads(8)


def small_cfg(tp: int) -> Config:
    """Reduced dims with the real head and quantisation grains (as the reference's SMALL, test_reference.py:163-172)."""
    return Config(
        hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024,
        swa_window=7, bf16_moe_layers=(), tp=tp, node_ranks=min(4, tp),
    )  # fmt: skip


CASES = {
    # name: (cfg, kwargs of synthetic.layer_case)
    "small_fp4_swa_tp8": (small_cfg(8), dict(rows=16, ctx=40, band="reference", seed=11)),
    "small_fp4_global_tp8_baseline": (small_cfg(8), dict(rows=16, ctx=40, global_attn=True, band="baseline", seed=12)),
    "small_bf16_global_tp8": (small_cfg(8), dict(rows=16, ctx=40, global_attn=True, bf16=True, seed=13)),
    "small_fp4_swa_tp2": (small_cfg(2), dict(rows=16, ctx=24, band="baseline", next_global=True, seed=14)),
    "small_fp4_swa_tp1_m5": (small_cfg(1), dict(rows=5, ctx=33, band="baseline", seed=15)),
    "small_bf16_tail_tp4": (small_cfg(4), dict(rows=16, ctx=19, global_attn=True, bf16=True, tail=True, seed=16)),
    "downscaled_m1": (downscaled(), dict(rows=1, ctx=4096, band="baseline", seed=0)),
}


def ref_weights(case, t) -> tuple:
    cfg = case.cfg
    if case.bf16:
        ex = R.Bf16Experts(RW.pack_w1_bf16(t.gate, t.up), RW.pack_w2_bf16(t.w2))
    else:
        w1, w1_sf = RW.pack_w1_fp4(t.gate_q, t.gate_sf, t.up_q, t.up_sf)
        w2, w2_sf = RW.pack_w2_fp4(t.w2_q, t.w2_sf)
        ex = R.Fp4Experts(w1, w1_sf, w2, w2_sf, t.g1_alphas, t.g1_scale_c, t.g2_alphas)
    w = R.LayerWeights(
        t.o_proj, t.post_alpha, t.post_beta, t.post_pre_w, t.pooler, t.router, t.expert_bias, case.router_mult,
        cfg.route_scale, t.pre_gamma, case.pre_eps, ex, t.gamma_p1, t.unpooler, t.cross_alpha, t.cross_beta,
        t.cross_pre_w, t.cross_post_w,
    )  # fmt: skip
    x = R.LayerInputs(t.qkv_in, t.k_ctx, t.v_ctx, t.stream_in, case.window)
    nxt = None
    if not case.tail:
        nxt = R.NextHead(
            t.next_qkv, cfg.q_scale, cfg.rms_eps, t.next_cos_sin, cfg.q_heads_rank, cfg.kv_heads_rank
        )
    return w, x, nxt


def ref_layer_k(w, x, comm, nxt, k: int) -> dict:
    """The reference's layer with ``k`` experts per row: ``ref_layer`` (muse_spark.py:721-794) binds the top-8 default
    and does not forward k, so the downscaled top-4 case composes the reference's own stage functions in the same
    order."""
    o = {}
    o["x_attn"] = R.attention(x.qkv, x.k_ctx, x.v_ctx, x.window)
    o["branch"] = R.o_proj_allreduce(o["x_attn"], w.w_o, comm)
    o["stream_mid"], o["h3"] = R.residual_norm(o["branch"], x.stream_in, w.post_alpha, w.post_beta, w.post_pre_w)
    o["pooled"] = R.node_sharded_linear(o["h3"], w.w_pool, comm)
    o["logits"] = R.router(o["h3"], w.w_router)
    o["ids"], o["w"] = R.topk(o["logits"], w.router_mult, w.expert_bias, w.route_scale, k=k)
    nrm = R.pre_expert_norm(o["pooled"], w.pre_gamma, w.pre_eps)
    o["xq"], o["x_sf"], o["x_scale"] = R.quantize_expert_input(nrm)
    o["zb"] = R.experts_fp4(o["xq"], o["x_sf"], o["x_scale"], o["ids"], w.experts, comm)
    o["y"] = R.combine(o["zb"], o["w"], w.gamma_p1)
    o["ffn_out"] = R.node_sharded_linear(o["y"], w.w_unpool, comm)
    o["stream_out"], o["h3_next"] = R.residual_norm(
        o["ffn_out"], o["stream_mid"], w.x_alpha, w.x_beta, w.x_pre_w, w.x_post_w
    )
    o["qkv_next"] = R.qkv_head(o["h3_next"], nxt.w_qkv, nxt.q_heads, nxt.kv_heads, nxt.q_scale, nxt.eps, nxt.cos_sin)
    return o


def layer_fixture(name: str) -> dict:
    cfg, kw = CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    packed = [ref_weights(case, t) for t in case.ranks]

    def run(comm):
        w, x, nxt = packed[comm.rank]
        if cfg.topk != R.TOPK:
            return ref_layer_k(w, x, comm, nxt, cfg.topk)
        return R.ref_layer(w, x, comm, nxt)

    outs = R.emulate_ranks(run, cfg.tp, cfg.node_ranks)
    keep = sorted({0, cfg.tp - 1})
    return {"ranks": keep, "outputs": {r: outs[r] for r in keep}}


def b_live_fixture() -> dict:
    """A block of 8 verified as rows 0-7 of the 16-row window (``b_live``, muse_spark.py:741-743)."""
    cfg, kw = CASES["small_fp4_swa_tp2"]
    case = synthetic.layer_case(cfg, **kw)
    packed = [ref_weights(case, t) for t in case.ranks]
    outs = R.emulate_ranks(
        lambda c: R.ref_layer(*packed[c.rank][:2], c, packed[c.rank][2], b_live=8), cfg.tp, cfg.node_ranks
    )
    return {"ranks": [0], "outputs": {0: outs[0]}}


def codec_fixture() -> dict:
    g = torch.Generator().manual_seed(1234)
    x = torch.cat((
        torch.randn(4096, generator=g) * 3,
        torch.tensor([0.0, -0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -5.0, 6.0, 7.0, -9.0, 1e-8]),
    ))  # fmt: skip
    y = torch.cat((torch.randn(4096, generator=g) * 50, torch.tensor([448.0, 500.0, -1000.0, 0.0, 2.0**-9, 2.0**-10])))
    amax = torch.cat((torch.rand(2048, generator=g) * 1000, torch.rand(2048, generator=g) * 1e-3)) + 1e-30
    byte = torch.arange(0, 0x7F, dtype=torch.uint8).repeat_interleave(16)
    delta = torch.arange(16).repeat(0x7F)
    z = torch.randn(24, 256, generator=g) * torch.logspace(-6, 3, 24)[:, None]
    zc, zs, ze = R.h_quant(z)
    xr = (torch.randn(16, 512, generator=g) * torch.logspace(-3, 2, 16)[:, None]).bfloat16()
    q, qs, qx = R.quantize_expert_input(xr)
    wq, wsf = R.quantize_nvfp4(torch.randn(8, 256, generator=g))
    cb = torch.randint(0, 256, (8, 128), generator=g, dtype=torch.uint8)
    sb = torch.randint(0, 0x7F, (8, 16), generator=g, dtype=torch.uint8)
    return dict(
        e2m1_in=x, e2m1_codes=R.e2m1_encode(x), e2m1_table=R.e2m1_decode(torch.arange(16)),
        e4m3_in=y, e4m3_bytes=R.e4m3_encode(y), e4m3_table=R.e4m3_decode(torch.arange(256, dtype=torch.uint8)),
        tf32_in=y, tf32_out=R.tf32(y),
        amax=amax, prov_exp=R._prov_exp(amax),
        sd_byte=byte, sd_delta=delta, sd_out=R._scale_down_byte(byte, delta),
        z=z, z_codes=zc, z_sf=zs, z_exp=ze, z_deq=R.h_dequant(zc, zs, ze),
        xr=xr, xr_q=q, xr_sf=qs, xr_scale=qx,
        static_codes=wq, static_sf=wsf, deq_codes=cb, deq_sf=sb, deq_out=R.dequant_nvfp4(cb, sb),
        rope=R.rope_cos_sin(torch.arange(100, 116), 500000.0),
    )  # fmt: skip


def head_tail_fixture() -> dict:
    """Entry (vocab-sharded embedding + norms) and logits (sharded lm_head + soft cap), 4 ranks (muse_spark.py:797-838)."""
    g = torch.Generator().manual_seed(77)
    ranks, vr, h = 4, 96, 256
    emb = [torch.randn(vr, h, generator=g).bfloat16() for _ in range(ranks)]
    head = [(torch.randn(vr, h, generator=g) / 16).bfloat16() for _ in range(ranks)]
    pre_w = (1 + 0.1 * torch.randn(h, generator=g)).bfloat16()
    ids = torch.randint(0, ranks * vr, (16,), generator=g)
    hid = torch.randn(16, h, generator=g).bfloat16()
    e = R.emulate_ranks(lambda c: R.ref_entry(ids, emb[c.rank], pre_w, c), ranks, 4)
    lg = R.emulate_ranks(lambda c: R.ref_logits(hid, head[c.rank], c, 32**-0.5, 20.0), ranks, 4)
    return dict(entry=e[0], logits=lg[0], seed=77)


def main() -> None:
    out = {}
    for name in CASES:
        print("layer case", name, flush=True)
        torch.save(layer_fixture(name), HERE / f"{name}.pt")
    torch.save(b_live_fixture(), HERE / "small_fp4_swa_tp2_blive8.pt")
    torch.save(codec_fixture(), HERE / "codecs.pt")
    torch.save(head_tail_fixture(), HERE / "head_tail.pt")
    for p in sorted(HERE.glob("*.pt")):
        print(f"{p.name}: {p.stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
