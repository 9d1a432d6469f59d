"""The accept oracle against the fixture made from the reference's own DFlash2 functions (tests/golden/accept.pt), and the
host-side checks of the head / tail binds that need no GPU."""

import sys
from pathlib import Path

import pytest
import torch

from oracle import dflash_accept as A
from sgl_muse_mega_b200.common import host

GOLDEN = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_accept_golden as G  # noqa: E402  (draw_case only: the module imports the reference lazily in main)


def test_make_accept_golden_imports_without_reference():
    assert hasattr(G, "draw_case")


def cap(x):
    return torch.tanh((x * 32**-0.5) / 20.0) * 20.0


def test_accept_matches_reference_outputs():
    fx = torch.load(GOLDEN / "accept.pt")
    assert fx["words"] == A.WORDS
    lens = []
    for i, ref in enumerate(fx["cases"]):
        tokens, logits = G.draw_case(i)
        capped = cap(logits)
        assert torch.equal(A.first_argmax(capped), ref["top1"])
        acc = A.greedy_accept(tokens, capped, ref["pos"])
        assert (acc.accept_len, acc.commit_len, acc.bonus, acc.new_pos) == (
            ref["accept_len"], ref["commit_len"], ref["bonus"], ref["new_pos"])  # fmt: skip
        assert torch.equal(acc.out_tokens, ref["out_tokens"])
        lens.append(acc.accept_len)
    assert lens[3] >= 1 and lens[5] == 2 and lens[11] == 15  # the tie, the NaN row and the full accept are exercised


def test_draft_feeds_match_reference_outputs():
    fx = torch.load(GOLDEN / "accept.pt")
    cache = torch.randn(300, 128, generator=torch.Generator().manual_seed(fx["seed"]))
    for ref in fx["draft_feeds"]:
        got = A.draft_feeds(cache, ref["pos"], ref["commit"], ref["b"], ref["dring"])
        for k in ("dcos_sin", "dslot", "dkv_len"):
            assert torch.equal(got[k], ref[k]), k


def test_step_words_and_ring():
    words = torch.tensor([4099, 77, 0, 3, 5, 62, 0, 0])
    ring = torch.full((64,), -1, dtype=torch.int32)
    tokens = torch.arange(100, 116)
    acc = A.Accept(3, 4, 9, torch.zeros(16, dtype=torch.int64), 4103)
    w, r = A.step_words(words, ring, acc, tokens)
    assert w.tolist() == [4103, 9, 3, 4, 6, 66, 0, 0]
    assert r[62].item() == 101 and r[63].item() == 102 and r[0].item() == 103 and r[1].item() == 9  # wraps at 64


def test_forced_accept_clamps():
    tokens, logits = G.draw_case(0)
    capped = cap(logits)
    assert A.greedy_accept(tokens, capped, 0, forced=40).accept_len == 15
    assert A.greedy_accept(tokens, capped, 0, forced=-2).accept_len == 0
    acc = A.greedy_accept(tokens, capped, 0, forced=6)
    assert acc.accept_len == 6 and acc.bonus == int(A.first_argmax(capped)[6])


# ---- the binds' argument checks (pack-only: no module, no GPU) ----


def _lib():
    return host.library()


def _expect(fn, struct, match):
    with pytest.raises(RuntimeError, match=match):
        _lib().bind(fn, None, struct)


def test_bind_argument_checks():
    one = torch.zeros(64)
    p = one.data_ptr()
    base = dict(positions=p, cos_sin_cache=0, cos_sin_rows=0, out_cache_loc=p, swa_out_cache_loc=0, seq_lens=p,
                req_pool_indices=p, req_to_token=p, r2t_rows=1, r2t_width=32, full_to_swa=0, swa_map_len=0, cos_sin=0,
                loc_full=p, loc_swa=0, kv_len=p, pt_full=p, pt_swa=0, rows=16, head_dim=64, kv_row_bytes=256, status=0)  # fmt: skip
    assert _lib().bind("mk_feeds_bind", None, host.make("MkFeedsBind", **base)).info().kernels == 1
    _expect("mk_feeds_bind", host.make("MkFeedsBind", **{**base, "rows": 17}), "rows 17")
    _expect("mk_feeds_bind", host.make("MkFeedsBind", **{**base, "loc_swa": p}), "go together")
    _expect("mk_feeds_bind", host.make("MkFeedsBind", **{**base, "r2t_width": 8}), "req_to_token")
    e = dict(ids=p, embed_peer=[p, p], shard_rows=10, ranks=2, pre_w=p, residual=p, normed=p, rows=4, hidden=1024,
             eps_embed=1e-5, eps_pre=1e-5)  # fmt: skip
    assert _lib().bind("mk_entry_bind", None, host.make("MkEntryBind", **e)).info().kernels == 1
    _expect("mk_entry_bind", host.make("MkEntryBind", **{**e, "hidden": 1000}), "hidden 1000")
    _expect("mk_entry_bind", host.make("MkEntryBind", **{**e, "ranks": 3}), r"embed_peer\[2\]")
    h = dict(w=p, x=p, out_peer=[p], rank=0, v_total=1000, col0=0, n_out=250, hidden=1024, rows=16, status=0, flags=0,
             flags_peer=[], ws=0, ws_bytes=0, w_packed=0)
    assert _lib().bind("mk_lm_head_bind", None, host.make("MkLmHeadBind", **h)).info().kernels == 1
    need = (1024 // 256) * 16 * 250 * 4 + 512  # with scratch the GEMM runs on the item engine
    assert _lib().bind("mk_lm_head_bind", None, host.make("MkLmHeadBind", **{**h, "ws": 4096, "ws_bytes": need})).info().kernels == 1
    _expect("mk_lm_head_bind", host.make("MkLmHeadBind", **{**h, "ws": 4096, "ws_bytes": need - 16}), "ws_bytes")
    _expect("mk_lm_head_bind", host.make("MkLmHeadBind", **{**h, "col0": 800}), "columns")
    _expect("mk_lm_head_bind", host.make("MkLmHeadBind", **{**h, "rank": 1}), "out_peer")
    a = dict(logits=p, vocab=1000, rows=16, b_live=16, scale=1.0, cap=20.0, tokens=p, accept_override=0, n_override=0,
             words=p, out_ring=p, ring=64, top1=p, counter=p, cos_sin_cache=0, cos_sin_rows=0, cos_sin=0, loc_full=0,
             loc_swa=0, kv_len=0, dcos_sin_cache=0, dcos_sin_rows=0, dcos_sin=0, dslot=0, dkv_len=0, dring=0, flags=0,
             contributors=0, wait_budget=0, status=0, pool_rows=0, samp=0, cand=0, walk_q=0, block_verify=0, sample_ws=0,
             sample_ws_bytes=0, sample_out=0, tree=0)  # fmt: skip
    assert _lib().bind("mk_accept_bind", None, host.make("MkAcceptBind", **a)).info().kernels == 1
    # the token tree: the greedy accept follows the table's tree; the tree's own launches check their operands
    assert _lib().bind("mk_accept_bind", None, host.make("MkAcceptBind", **{**a, "tree": p})).info().kernels == 1
    t = dict(cand=p, scores=p, words=p, table=p, verify_ids=p, loc_full=0, loc_swa=0, rows=16, cos_sin_cache=0, cos_sin_rows=0, cos_sin=0)
    assert _lib().bind("mk_dflash_tree_bind", None, host.make("MkDflashTreeBind", **t)).info().kernels == 1
    _expect("mk_dflash_tree_bind", host.make("MkDflashTreeBind", **{**t, "rows": 17}), "rows")
    _expect("mk_dflash_tree_bind", host.make("MkDflashTreeBind", **{**t, "table": 0}), "table")
    c = dict(table=p, rows=p, n_swa=3, n_full=1, n_cap=5, kv_row_bytes=256, cap_row_bytes=4096)
    assert _lib().bind("mk_dflash_tree_compact_bind", None, host.make("MkDflashTreeCompactBind", **c)).info().kernels == 1
    _expect("mk_dflash_tree_compact_bind", host.make("MkDflashTreeCompactBind", **{**c, "kv_row_bytes": 250}), "multiples of 16")
    _expect("mk_dflash_tree_compact_bind", host.make("MkDflashTreeCompactBind", **{**c, "n_swa": 0, "n_full": 0, "n_cap": 0}), "no buffers")
    # the sampled accept: its operands and scratch (rows x vocab x 12 bytes + 256, 256-byte aligned)
    need = 16 * 1000 * 12 + 256
    smp = {**a, "samp": p, "cand": p, "walk_q": p, "sample_ws": 4096, "sample_ws_bytes": need, "top1": 0}
    assert _lib().bind("mk_accept_bind", None, host.make("MkAcceptBind", **smp)).info().kernels == 1
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**smp, "sample_ws_bytes": need - 1}), "sample_ws_bytes")
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**smp, "cand": 0}), "cand")
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**smp, "sample_ws": 4100}), "aligned")
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**smp, "tree": p}), "exclusive")
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**a, "top1": 0}), "top1")
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**a, "b_live": 17}), "b_live")
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**a, "ring": 8}), "ring")
    _expect("mk_accept_bind", host.make("MkAcceptBind", **{**a, "dslot": p}), "dslot")
    s = dict(x=p, out=p, numel=0, scale=1.0, cap=20.0, flags=0, contributors=0, wait_budget=0, status=0)
    _expect("mk_softcap_bind", host.make("MkSoftcapBind", **s), "numel")
