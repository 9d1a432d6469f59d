"""The CPU oracle against the golden fixtures produced by the reference's own torch oracle: bit-exact."""

import pytest
import torch

from golden_cases import CASES
from oracle import muse_layer as O
from oracle.cases import rank_layers
from sgl_muse_mega_b200.muse_spark.b200 import synthetic

torch.set_num_threads(8)


def _same(a, b):
    if a.is_floating_point():
        return torch.equal(a.float().nan_to_num(7.0), b.float().nan_to_num(7.0))
    return torch.equal(a, b)


@pytest.mark.parametrize("name", list(CASES))
def test_layer_matches_reference(name, golden_dir):
    cfg, kw = CASES[name]
    gold = torch.load(golden_dir / f"{name}.pt")
    case = synthetic.layer_case(cfg, **kw)
    outs = O.run_layer(rank_layers(case), cfg.node_ranks)
    for r in gold["ranks"]:
        ref = gold["outputs"][r]
        assert set(ref) == set(outs[r]), (sorted(ref), sorted(outs[r]))
        for k, v in ref.items():
            assert outs[r][k].dtype == v.dtype and outs[r][k].shape == v.shape, (name, r, k)
            assert _same(outs[r][k], v), (name, r, k)


def test_b_live(golden_dir):
    cfg, kw = CASES["small_fp4_swa_tp2"]
    gold = torch.load(golden_dir / "small_fp4_swa_tp2_blive8.pt")["outputs"][0]
    outs = O.run_layer(rank_layers(synthetic.layer_case(cfg, **kw)), cfg.node_ranks, b_live=8)
    for k, v in gold.items():
        assert _same(outs[0][k], v), k
    assert not outs[0]["y"][8:].any()


def test_forced_ids_only_move_weights(golden_dir):
    """Forcing the kernel's ids keeps the oracle's own ids and takes the weights at the forced ones (R1:389-390)."""
    cfg, kw = CASES["small_fp4_swa_tp1_m5"]
    case = synthetic.layer_case(cfg, **kw)
    base = O.run_layer(rank_layers(case), cfg.node_ranks)[0]
    ids = base["ids"].clone()
    ids[0, [0, 1]] = ids[0, [1, 0]]
    forced = O.run_layer(rank_layers(case), cfg.node_ranks, forced=[{"ids": ids}])[0]
    assert torch.equal(forced["ids"], base["ids"])
    assert torch.equal(forced["w"][0, 0], base["w"][0, 1])


def test_codecs(golden_dir):
    g = torch.load(golden_dir / "codecs.pt")
    assert torch.equal(O.e2m1_encode(g["e2m1_in"]), g["e2m1_codes"])
    assert torch.equal(O.e2m1_decode(torch.arange(16)), g["e2m1_table"])
    assert torch.equal(O.e4m3_encode(g["e4m3_in"]), g["e4m3_bytes"])
    assert _same(O.e4m3_decode(torch.arange(256, dtype=torch.uint8)), g["e4m3_table"])
    assert torch.equal(O.tf32_truncate(g["tf32_in"]), g["tf32_out"])
    assert torch.equal(O.provisional_exponent(g["amax"]), g["prov_exp"])
    assert torch.equal(O.scale_down_byte(g["sd_byte"], g["sd_delta"]), g["sd_out"])
    c, s, e = O.h_quant(g["z"])
    assert torch.equal(c, g["z_codes"]) and torch.equal(s, g["z_sf"]) and torch.equal(e, g["z_exp"])
    assert torch.equal(O.h_dequant(c, s, e), g["z_deq"])
    q, qs, qx = O.quantize_rows(g["xr"])
    assert torch.equal(q, g["xr_q"]) and torch.equal(qs, g["xr_sf"]) and torch.equal(qx, g["xr_scale"])
    assert torch.equal(O.nvfp4_dequant(g["deq_codes"], g["deq_sf"]), g["deq_out"])
    assert torch.equal(O.rope_rows(torch.arange(100, 116), 500000.0), g["rope"])


def test_codec_known_answers():
    """Known answers of the number formats, the ones the reference pins in test/unit/test_reference.py:30-59."""
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert O.e2m1_encode(mids).tolist() == [0, 2, 2, 4, 4, 6, 6]  # ties go to the even code
    assert O.e2m1_encode(torch.tensor([100.0, -100.0, -0.0])).tolist() == [7, 15, 8]
    assert O.e4m3_encode(torch.tensor([448.0, 1e6, -1e6])).tolist() == [0x7E, 0x7E, 0xFE]
    x = torch.tensor([1.0 + 2**-11, 1.0 + 2**-10])
    assert O.tf32_truncate(x).tolist() == [1.0, 1.0 + 2**-10]
    rt = O.nibbles_unpack(O.nibbles_pack(torch.arange(16, dtype=torch.uint8)))
    assert rt.tolist() == list(range(16))


def test_head_tail(golden_dir):
    g = torch.load(golden_dir / "head_tail.pt")
    gen = torch.Generator().manual_seed(77)
    ranks, vr, h = 4, 96, 256
    emb = [torch.randn(vr, h, generator=gen).bfloat16() for _ in range(ranks)]
    head = [(torch.randn(vr, h, generator=gen) / 16).bfloat16() for _ in range(ranks)]
    pre_w = (1 + 0.1 * torch.randn(h, generator=gen)).bfloat16()
    ids = torch.randint(0, ranks * vr, (16,), generator=gen)
    hid = torch.randn(16, h, generator=gen).bfloat16()
    e = O.entry(ids, emb, pre_w)
    for k in ("emb", "normed", "residual"):
        assert torch.equal(e[k], g["entry"][k]), k
    assert torch.equal(O.logits_out(hid, head, 32**-0.5, 20.0), g["logits"])
