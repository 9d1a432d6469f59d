"""The isolated NVFP4 expert block (window of 1 / 4 / 8 / 16 rows, whole experts over 1 / 2 / 4 / 8 expert-parallel ranks)
through the C ABI: every stage of the block against the oracle fed the kernels' own inputs (the reference's per-stage
method, muse_spark.py:738-743, at its bounds :868-888), and every expert-parallel split bit for bit against the lone
rank's result."""

import pytest
import torch

from oracle import muse_layer as O
from parity import nvfp4_rows_close
from sgl_muse_mega_b200.muse_spark.b200 import expert_block as X

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    assert torch.cuda.is_available(), "these tests need the B200"
    return torch.device("cuda:0")


class DeviceExperts:
    """One per-expert weight array left on the device; the oracle indexes it by the routed expert id only."""

    def __init__(self, t):
        self.t, self.shape = t, t.shape

    def __getitem__(self, e):
        return self.t[e].cpu()


def oracle_experts(t):
    f = lambda x: DeviceExperts(x)  # noqa: E731
    return O.Fp4Experts(f(t.gate_q), f(t.gate_sf), f(t.up_q), f(t.up_sf), f(t.w2_q), f(t.w2_sf), t.g1_alphas.cpu(),
                        t.g1_scale_c.cpu(), t.g2_alphas.cpu())  # fmt: skip


def block_values(blk):
    lr = blk.ranks[0]
    names = ("h3", "h3f", "logits", "ids", "w", "xq", "x_sf", "x_scale", "y")
    v = {k: lr.o[k].cpu() for k in names}
    v["pooled"] = lr.pool_ag.cpu()
    cfg = blk.case.cfg
    v["zb"] = blk.zb.view(torch.bfloat16).view(blk.rows, cfg.topk, cfg.moe_hidden).cpu()
    return v


def check_against_oracle(blk):
    case, cfg = blk.case, blk.case.cfg
    t = case.ranks[0]
    v = block_values(blk)
    cpu = lambda x: x.cpu()  # noqa: E731

    def close(name, ref):
        mx, rel, ok = O.compare(v[name], ref, name)
        assert ok, f"{name}: rel {rel:.3e} > {O.TOLERANCES[name]:.1e} (max abs {mx:.3e})"

    close("pooled", O.linear_block(v["h3"], cpu(t.pooler)))
    close("logits", O.router_logits(v["h3f"], cpu(t.router)))
    own, w = O.route_topk(v["logits"], case.router_mult, cpu(t.expert_bias), cfg.route_scale, cfg.topk)
    assert torch.equal(v["ids"], own), "routed ids differ from the oracle's on the kernel's logits"
    close("w", w)
    xq, x_sf, x_scale = O.quantize_rows(O.pre_expert_norm(v["pooled"], cpu(t.pre_gamma), case.pre_eps))
    nvfp4_rows_close(v["xq"], v["x_sf"], xq, x_sf, "expert input")
    close("x_scale", x_scale)
    close("zb", O._experts_fp4(v["xq"], v["x_sf"], v["x_scale"], v["ids"], [oracle_experts(t)]))
    close("y", O.combine(v["zb"], v["w"], cpu(t.gamma_p1)))
    return v


def run_block(case, device, ep):
    blk = X.ExpertBlock(case, device, ep=ep)
    blk.run()
    torch.cuda.synchronize()
    assert not any(blk.statuses()), blk.statuses()
    return blk


@pytest.mark.parametrize("rows", [1, 5, 16])
def test_small_block_and_its_expert_parallel_splits(rows, device):
    cfg = X.block_config(experts=16, moe_hidden=1024, moe_inter=1024)
    case = X.draw_case(cfg, rows, device, seed=70 + rows)
    one = run_block(case, device, 1)
    assert one.ranks[0].tensor_cores
    ref = check_against_oracle(one)
    for ep in (2, 4, 8):
        blk = run_block(case, device, ep)
        assert sum(blk.local_experts()) == sum(one.local_experts())
        got = block_values(blk)
        for k in ("ids", "w", "xq", "x_sf", "zb", "y"):
            assert torch.equal(got[k], ref[k]), f"ep {ep}: {k} differs from the lone rank's"


@pytest.fixture(scope="module")
def full_case(device):
    return X.draw_case(X.block_config(), 16, device)


@pytest.mark.parametrize("rows", [1, 4, 8, 16])
def test_full_shape_block(rows, full_case, device):
    """256 experts of 4096 x 4096 (28.31 MB each), logits and rows ~ N(0, 1), top-8: the lone rank against the oracle on
    the routed experts, then 2 / 4 / 8 ranks of whole experts bit for bit against the lone rank."""
    case = X.with_rows(full_case, rows)
    one = run_block(case, device, 1)
    assert one.ranks[0].tensor_cores
    ref = check_against_oracle(one)
    del one
    for ep in (2, 4, 8):
        torch.cuda.empty_cache()
        blk = run_block(case, device, ep)
        got = block_values(blk)
        for k in ("ids", "w", "xq", "x_sf", "zb", "y"):
            assert torch.equal(got[k], ref[k]), f"ep {ep}: {k} differs from the lone rank's"
        del blk
