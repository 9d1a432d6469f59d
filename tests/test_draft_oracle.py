"""The CPU restatement of the DFlash2 draft step against outputs of the reference's own functions
(``tests/golden/draft.pt``, made by ``tests/golden/make_draft_golden.py``) on the seeded cases re-created here."""

from pathlib import Path

import pytest
import torch

from oracle import dflash_draft as D
from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic
from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig

GOLD = torch.load(Path(__file__).parent / "golden" / "draft.pt", weights_only=False)
CFG = DraftConfig(**{k: tuple(v) if isinstance(v, list) else v for k, v in GOLD["cfg"].items()})


def run_case(g):
    case = synthetic.draft_case(CFG, g["ranks"], g["rows"], g["pos"], g["commit"], g["seed"])
    kv = D.DraftKV.empty(CFG, g["ranks"], g["pos"] + g["rows"])
    kvh = CFG.kv_heads // g["ranks"]
    n_hist = g["pos"] - g["commit"]
    for r in range(g["ranks"]):
        for li in range(CFG.layers):
            kv.k[r][li][:n_hist] = case.hist_k[li][:, r * kvh : (r + 1) * kvh]
            kv.v[r][li][:n_hist] = case.hist_v[li][:, r * kvh : (r + 1) * kvh]
    return case, kv, D.draft_step(CFG, case.shards, kv, case.caps, case.anchor, g["pos"], g["commit"], g["rows"])


def ulps_apart(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (a.view(torch.int16).int() - b.view(torch.int16).int()).abs()


@pytest.mark.parametrize("name", sorted(GOLD["cases"]))
def test_draft_step_matches_the_reference(name):
    g = GOLD["cases"][name]
    case, kv, got = run_case(g)
    # the context rows: bit-exact (GEMMs in f64, one rounding; no reduction-order freedom)
    for r, pr in enumerate(g["per_rank"]):
        for li in range(CFG.layers):
            k, v = got["ctx"]["kv"][r][li]
            assert torch.equal(k, pr["ctx_k"][li]) and torch.equal(v, pr["ctx_v"][li]), (r, li)
            lo = g["pos"] - g["commit"]
            assert torch.equal(kv.k[r][li][lo : g["pos"] + g["rows"]], pr["kv_k"][li]), (r, li)
            assert torch.equal(kv.v[r][li][lo : g["pos"] + g["rows"]], pr["kv_v"][li]), (r, li)
    # the block: the per-head f64 softmax here and the reference's batched one may differ in the last f64 bits before
    # the bf16 rounding; everything else is the same arithmetic. Hold y to one bf16 ulp on a vanishing fraction of elements.
    apart = ulps_apart(got["y"], g["y"])
    assert int(apart.max()) <= 1 and float((apart > 0).float().mean()) < 1e-3, (int(apart.max()), float((apart > 0).float().mean()))
    if int(apart.max()) == 0:
        assert torch.equal(got["cand"], g["cand"]) and torch.equal(got["unary"], g["unary"])
        assert torch.equal(got["scores"], g["scores"]) and torch.equal(got["tokens"], g["tokens"])
    # the head on the REFERENCE's y: candidates, lattice and walk are exact functions of y
    cand, unary, _ = D.candidates(CFG, case.shards, g["y"][1:])
    assert torch.equal(cand, g["cand"]) and torch.equal(unary, g["unary"])
    scores, _ = D.lattice(case.shards[0][0], g["y"][1:], cand, unary, case.anchor)
    assert torch.equal(scores, g["scores"])
    drafts, _ = D.walk(cand, scores)
    assert torch.equal(torch.cat([torch.tensor([case.anchor]), drafts]), g["tokens"])


def test_topk_ties_go_to_the_smaller_id():
    vals = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0]])
    ids = torch.tensor([[9, 7, 2, 5, 4]])
    v, i = D.topk_low_id(vals, ids, 3)
    assert i.tolist() == [[2, 4, 7]] and v.tolist() == [[3.0, 3.0, 3.0]]


def test_conv_row_zero_has_no_second_tap():
    x = torch.randn(4, 32).to(torch.bfloat16)
    delta = torch.randn(4, 2, 2).to(torch.bfloat16)
    base = torch.randn(2, 32).to(torch.bfloat16)
    out = D.grouped_conv(x, delta, base)
    want0 = ((base[0].float() + delta[0, 0].float().repeat_interleave(16)) * x[0].float()).to(torch.bfloat16)
    assert torch.equal(out[0], want0)


def test_draft_binds_validate_without_a_gpu():
    """Pack-only binds (no module): operand checks and kernel counts of the draft's launch records."""
    from sgl_muse_mega_b200.common import host

    lib = host.library()
    P = 1 << 20  # any aligned non-null address: a pack-only record never launches
    shape = dict(rows=16, hidden=512, layers=2, q_heads=4, kv_heads=2, inter=512, features=5, ranks=2, rank=1, window_left=23,
                 conv_groups=32, vocab=2048, selector_rank=64)  # fmt: skip
    sh = host.make("MkDflashShape", **shape)
    c = lib.dflash_constants(sh)
    assert (c.coeffs, c.qkv_row, c.kv_rows_n, c.attn_splits, c.topk_chunks) == (128, 1024, 1024, 2, 1)
    assert c.ws_bytes >= (5 * 512 // 256) * 16 * 256 * 4 + 512
    common = dict(ws=P, flags=0, flags_peer=[], status=P, wait_budget=0, eps=1e-5, packed=0)
    entry = dict(cap=[P] * 5, words=P, embed_peer=[P, P], shard_rows=1024, mask_id=2002, w_fc=P, hid_norm=P, in_norm=P, w_kv=P,
                 k_norm=[P, P], k_pool=[P, P], v_pool=[P, P], pool_rows=64, rope=P, rope_rows=64, feats=P, ctx_raw_peer=[0, P], ctx=P,
                 kv=P, x=P, h=P, **common)  # fmt: skip
    assert lib.dflash_bind("mk_dflash_entry_bind", None, sh, host.make("MkDflashEntryBind", **entry)).info().kernels == 6
    with pytest.raises(RuntimeError, match="pool_rows"):
        lib.dflash_bind("mk_dflash_entry_bind", None, sh, host.make("MkDflashEntryBind", **{**entry, "pool_rows": 30}))
    with pytest.raises(RuntimeError, match="ctx_raw_peer"):
        lib.dflash_bind("mk_dflash_entry_bind", None, sh, host.make("MkDflashEntryBind", **{**entry, "ctx_raw_peer": [P, 0]}))
    layer = dict(h_in=P, res_in=P, words=P, attn_proj=P, attn_base=P, mlp_proj=P, mlp_base=P, w_qkv=P, q_norm=P, k_norm=P, w_o=P,
                 post_norm=P, w_gate_up=P, w_down=P, next_norm=P, k_pool=P, v_pool=P, pool_rows=64, rope=P, rope_rows=64, c_att=P,
                 xa=P, qkv=P, q=P, attn_ws=P, o=P, ar_attn_peer=[P, P], a=0, h_post=P, res_post=P, c_mlp=P, xm=P, m=P,
                 ar_mlp_peer=[P, P], x_out=0, h_out=P, res_out=0, **common)  # fmt: skip
    assert lib.dflash_bind("mk_dflash_layer_bind", None, sh, host.make("MkDflashLayerBind", **layer)).info().kernels == 10
    with pytest.raises(RuntimeError, match="w_down"):
        lib.dflash_bind("mk_dflash_layer_bind", None, sh, host.make("MkDflashLayerBind", **{**layer, "w_down": 0}))
    head = dict(y=P, w_hproj=P, hid=P, logits=P, pred_codebook=P, succ_codebook=P, words=P, keys=P, cand=P, unary=P, scores=P,
                pick=P, drafts=P, verify_ids=P, mult=0.17, cap=20.0, ws=P, flags=0, contributors=0, status=P, wait_budget=0, packed=1, samp=0, walk_q=0)  # fmt: skip
    assert lib.dflash_bind("mk_dflash_draft_head_bind", None, sh, host.make("MkDflashDraftHeadBind", **head)).info().kernels == 3
    for bad, why in ((dict(q_heads=3), "heads"), (dict(hidden=768), "hidden"), (dict(inter=300), "inter"), (dict(rows=17), "rows"),
                     (dict(conv_groups=128), "conv_groups"), (dict(selector_rank=600), "selector_rank")):  # fmt: skip
        with pytest.raises(RuntimeError, match=why):
            lib.dflash_constants(host.make("MkDflashShape", **{**shape, **bad}))
    sync = dict(words=P, window=P, state=P, ring=P, pool=P, n_buf=10, row_bytes=256, ring_rows=4096, lag=1, status=P)
    assert lib.bind("mk_dflash_kv_sync_bind", None, host.make("MkDflashKvSyncBind", **sync)).info().kernels == 1
    with pytest.raises(RuntimeError, match="row_bytes"):
        lib.bind("mk_dflash_kv_sync_bind", None, host.make("MkDflashKvSyncBind", **{**sync, "row_bytes": 100}))


def test_item_images_hold_the_matrix():
    from sgl_muse_mega_b200.muse_spark.b200 import weights as W

    g = torch.Generator().manual_seed(0)
    for dtype, bn, pad in ((torch.bfloat16, 64, 32), (torch.float32, 16, 16)):
        w = torch.randn(150, 1024, generator=g).to(dtype)
        img = W.pack_items(w)
        nb = (150 + bn - 1) // bn
        assert img.shape == (nb, 2, bn, 512 + pad) and img.is_contiguous()
        for n, k in ((0, 0), (63, 511), (64, 512), (149, 1023), (100, 600)):
            assert img[n // bn, k // 512, n % bn, k % 512] == w[n, k]
        assert float(img[..., 512:].abs().sum()) == 0  # the row padding
        assert float(img[nb - 1, :, 150 - (nb - 1) * bn :].abs().sum()) == 0  # rows past N
    with pytest.raises(ValueError):
        W.pack_items(torch.zeros(64, 300, dtype=torch.bfloat16))


def test_philox_and_sampled_walk_match_the_reference():
    """Philox4x32-10 known answers, the step's uniforms and the sampled walk (softmax of the score row / T, inverse CDF)
    against the reference's own outputs."""
    for k in GOLD["philox"]:
        assert tuple(D.philox(tuple(k["counter"]), tuple(k["key"]))) == tuple(k["out"])
    seed, temp = 0x1234567887654321, 0.7
    for name, s in GOLD["sampled"].items():
        g = GOLD["cases"][name]
        u = D.uniforms(seed, g["pos"], 3, D.PURPOSE_WALK)
        assert torch.equal(u, s["u"]) and float(u.min()) >= 0 and float(u.max()) < 1
        toks, picks, q = D.walk_sampled(g["cand"], g["scores"], u, temp)
        assert torch.equal(toks, s["tokens"]) and torch.equal(q, s["q"])
        assert torch.equal(g["cand"].gather(1, picks[:, None])[:, 0], toks)
