"""The launches around the decoder layers (window feeds, entry, lm_head, soft cap, greedy accept) through the C-ABI
against the CPU oracle and the fixtures made from the reference's own functions."""

import sys
from pathlib import Path

import pytest
import torch

from oracle import dflash_accept as A
from oracle import muse_layer as O
from sgl_muse_mega_b200.common import host
from sgl_muse_mega_b200.muse_spark.b200 import headtail as HT

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_accept_golden as G  # noqa: E402  (the seeded inputs of accept.pt; the reference is imported in its main only)

DEV = torch.device("cuda:0")
MULT, CAP = 32**-0.5, 20.0


def stream():
    return torch.cuda.current_stream().cuda_stream


def ctx():
    lib = host.library()
    return lib, lib.load()


def head_tail_inputs():
    gen = torch.Generator().manual_seed(77)
    ranks, vr, h = 4, 96, 256
    emb = [torch.randn(vr, h, generator=gen).bfloat16() for _ in range(ranks)]
    head = [(torch.randn(vr, h, generator=gen) / 16).bfloat16() for _ in range(ranks)]
    pre_w = (1 + 0.1 * torch.randn(h, generator=gen)).bfloat16()
    ids = torch.randint(0, ranks * vr, (16,), generator=gen)
    hid = torch.randn(16, h, generator=gen).bfloat16()
    return emb, head, pre_w, ids, hid


def test_entry_golden_bit_exact():
    lib, module = ctx()
    emb, _, pre_w, ids, _ = head_tail_inputs()
    g = torch.load(GOLDEN / "head_tail.pt")["entry"]
    e = HT.Entry(lib, module, ids=ids.to(DEV), embed_shards=[t.to(DEV) for t in emb], pre_w=pre_w.to(DEV))
    e.launch(stream())
    torch.cuda.synchronize()
    # the norms are x * rsqrt(mean + eps) in f32 rounded to bf16: one-ulp flips where rsqrt.approx and the sum order move
    # a value across a rounding boundary
    for name, got in (("residual", e.residual.cpu()), ("normed", e.normed.cpu())):
        _, rel, ok = O.compare(got, g[name], name)
        assert ok, (name, rel)
    assert (e.residual.cpu() != g["residual"]).float().mean() < 0.01


@pytest.mark.parametrize("rows,hidden,ranks,shard", [(16, 8192, 8, 25256), (5, 2048, 2, 1000), (1, 1024, 1, 512)])
def test_entry_oracle(rows, hidden, ranks, shard):
    lib, module = ctx()
    gen = torch.Generator().manual_seed(rows * 7 + ranks)
    used = torch.randint(0, ranks * shard, (rows,), generator=gen)
    used[0], used[-1] = ranks * shard - 1, 0  # the last row of the last shard and the first row of the first
    emb = [torch.zeros(shard, hidden, dtype=torch.bfloat16) for _ in range(ranks)]
    for t in used.tolist():  # only the rows the window reads hold values (the shards are large)
        emb[t // shard][t % shard] = torch.randn(hidden, generator=gen).bfloat16()
    pre_w = (1 + 0.1 * torch.randn(hidden, generator=gen)).bfloat16()
    ref = O.entry(used, emb, pre_w)
    e = HT.Entry(lib, module, ids=used.to(DEV), embed_shards=[t.to(DEV) for t in emb], pre_w=pre_w.to(DEV))
    e.launch(stream())
    torch.cuda.synchronize()
    for name, got in (("residual", e.residual.cpu()), ("normed", e.normed.cpu())):
        _, rel, ok = O.compare(got, ref[name], name)
        assert ok, (name, rel)


def test_lm_head_softcap_golden():
    """Four ranks' lm_head shards write one gathered row each through the peer list; the soft-capped result is the
    reference's logits."""
    lib, module = ctx()
    _, head, _, _, hid = head_tail_inputs()
    g = torch.load(GOLDEN / "head_tail.pt")["logits"]
    gathered = [torch.zeros(16, 4 * 96, dtype=torch.float32, device=DEV) for _ in range(4)]
    x = hid.to(DEV)
    heads = [HT.LmHead(lib, module, w=head[r].to(DEV), x=x, gathered=gathered, rank=r) for r in range(4)]
    for h in heads:
        h.launch(stream())
    out = torch.zeros_like(gathered[0])
    cap = HT.Softcap(lib, module, x=gathered[2], out=out, scale=MULT, cap=CAP)
    cap.launch(stream())
    torch.cuda.synchronize()
    for r in range(1, 4):
        assert torch.equal(gathered[r], gathered[0])  # every rank holds the same gathered row, bit for bit
    _, rel, ok = O.compare(out.cpu(), g, "logits_out")
    assert ok, rel
    assert all(int(h.status[0]) == 0 for h in heads)


@pytest.mark.parametrize("packed", [0, 2])
def test_lm_head_full_shard_ragged_tile(packed):
    """The 816B model's shard: 25256 vocab rows (not a multiple of the 64- or 128-row tile) x 8192, 16 rows, one of eight
    ranks, against an f32 matmul of the same bf16 operands; columns outside the shard stay untouched. ``packed`` 2: tile
    images on the tensor-core engine (198 tiles over 148 CTAs: tiles shared by two CTAs meet through the ticketed partial
    sums), 0: row-major weights on the item engine."""
    from sgl_muse_mega_b200.muse_spark.b200 import weights as W

    lib, module = ctx()
    gen = torch.Generator(device=DEV).manual_seed(5)
    n, k, vt = 25256, 8192, 25256 * 8
    w = (torch.randn(n, k, generator=gen, device=DEV) / 64).bfloat16()
    x = torch.randn(16, k, generator=gen, device=DEV).bfloat16()
    own = torch.full((16, vt), 7.0, dtype=torch.float32, device=DEV)
    gathered = [None] * 8
    gathered[3] = own
    h = HT.LmHead(lib, module, w=W.pack_dense(w, packed), x=x, gathered=gathered, rank=3, w_packed=packed, n_out=n, hidden=k)
    h.launch(stream())
    torch.cuda.synchronize()
    ref = x.float() @ w.float().T
    got = own[:, 3 * n : 4 * n]
    rel = ((got - ref).norm(dim=1) / ref.norm(dim=1)).max().item()
    assert rel < 1e-4, rel  # exact bf16 products into f32: accumulation order only
    assert bool((own[:, : 3 * n] == 7.0).all()) and bool((own[:, 4 * n :] == 7.0).all())
    assert int(h.status[0]) == 0


def test_window_feeds():
    lib, module = ctx()
    gen = torch.Generator().manual_seed(9)
    rows, width, kvb = 16, 4200, 256
    cache = torch.randn(5000, 64, generator=gen)
    positions = torch.arange(4099, 4099 + rows)
    out_loc = torch.randint(0, 10000, (rows,), generator=gen)
    r2t = torch.randint(0, 10000, (3, width), generator=gen, dtype=torch.int32)
    r2t[1, 4150:] = -1  # unwritten tail entries read the map's appended last row
    f2s = torch.cat([torch.randint(0, 3000, (10000,), generator=gen), torch.tensor([-1])])
    swa_loc = f2s[out_loc]
    seq = torch.tensor([4099])
    req = torch.tensor([1])
    ref = A.window_feeds(positions, cache, out_loc, swa_loc, seq, req, r2t, f2s, kvb)
    d = lambda t: t.to(DEV)  # noqa: E731
    f = HT.WindowFeeds(lib, module, positions=d(positions), cos_sin_cache=d(cache), out_cache_loc=d(out_loc),
                       swa_out_cache_loc=d(swa_loc), seq_lens=d(seq), req_pool_indices=d(req), req_to_token=d(r2t),
                       full_to_swa=d(f2s), kv_row_bytes=kvb)  # fmt: skip
    f.launch(stream())
    torch.cuda.synchronize()
    for k in ("cos_sin", "loc_full", "loc_swa", "kv_len", "pt_full", "pt_swa"):
        assert torch.equal(getattr(f, k).cpu(), ref[k]), k
    assert f.launch.status(stream()).code == 0


def test_window_feeds_records_a_bad_position():
    """A position past the rope cache is clamped and recorded in the status words; nothing traps."""
    lib, module = ctx()
    d = lambda t: t.to(DEV)  # noqa: E731
    f = HT.WindowFeeds(lib, module, positions=d(torch.tensor([3, 99])), cos_sin_cache=d(torch.ones(10, 64)),
                       out_cache_loc=d(torch.tensor([1, 2])), swa_out_cache_loc=None, seq_lens=d(torch.tensor([3])),
                       req_pool_indices=d(torch.tensor([0])), req_to_token=d(torch.zeros(1, 8, dtype=torch.int32)),
                       full_to_swa=None, kv_row_bytes=256)  # fmt: skip
    f.launch(stream())
    st = f.launch.status(stream())
    assert (st.code, st.stage, st.observed) == (4, 300, 99)


def test_accept_chain_matches_reference_fixture():
    """Twelve chained iterations on the fixture's inputs: per-row arg-max, accept, words, ring and the next feeds are the
    reference's, bit for bit."""
    lib, module = ctx()
    fx = torch.load(GOLDEN / "accept.pt")
    gen = torch.Generator().manual_seed(1)
    cache, dcache = torch.randn(5000, 64, generator=gen), torch.randn(5000, 128, generator=gen)
    logits = torch.zeros(G.ROWS, G.VOCAB, dtype=torch.float32, device=DEV)
    tokens = torch.zeros(G.ROWS, dtype=torch.int64, device=DEV)
    cs = torch.zeros(G.ROWS, 64, device=DEV)
    loc_f, loc_s = (torch.zeros(G.ROWS, dtype=torch.int32, device=DEV) for _ in range(2))
    kv_len = torch.zeros(1, dtype=torch.int32, device=DEV)
    acc = HT.Accept(lib, module, logits=logits, tokens=tokens, b_live=G.ROWS, scale=MULT, cap=CAP, ring=40,
                    cos_sin_cache=cache.to(DEV), cos_sin=cs, loc_full=loc_f, loc_swa=loc_s, kv_len=kv_len,
                    dcos_sin_cache=dcache.to(DEV), dring=64)  # fmt: skip
    acc.words[A.WORDS["P"]] = fx["cases"][0]["pos"]
    words, ring = acc.words.cpu(), acc.out_ring.cpu()
    for i, ref in enumerate(fx["cases"]):
        tok, lg = G.draw_case(i)
        logits.copy_(lg)
        tokens.copy_(tok)
        acc.launch(stream())
        torch.cuda.synchronize()
        assert torch.equal(acc.top1.cpu().long(), ref["top1"]), i
        step = A.greedy_accept(tok, torch.tanh((lg * MULT) / CAP) * CAP, int(words[0]))
        assert (step.accept_len, step.bonus, step.new_pos) == (ref["accept_len"], ref["bonus"], ref["new_pos"])
        words, ring = A.step_words(words, ring, step, tok)
        assert torch.equal(acc.words.cpu(), words), (i, acc.words.cpu(), words)
        assert torch.equal(acc.out_ring.cpu(), ring), i
        tf = A.target_feeds(cache, step.new_pos, G.ROWS)
        assert torch.equal(cs.cpu(), tf["cos_sin"]) and torch.equal(loc_f.cpu(), tf["loc"])
        assert torch.equal(loc_s.cpu(), tf["loc"]) and torch.equal(kv_len.cpu(), tf["kv_len"])
        df = A.draft_feeds(dcache, step.new_pos, step.commit_len, G.ROWS, 64)
        assert torch.equal(acc.dcos_sin.cpu(), df["dcos_sin"]) and torch.equal(acc.dslot.cpu(), df["dslot"])
        assert torch.equal(acc.dkv_len.cpu(), df["dkv_len"])
    assert int(acc.counter[0]) == 0  # the arrival counter is back at zero after every launch


def test_accept_forced_table_and_b_live():
    lib, module = ctx()
    tok, lg = G.draw_case(8)
    logits, tokens = lg.to(DEV), tok.to(DEV)
    forced = torch.tensor([3, 0, 40, -1], dtype=torch.int32, device=DEV)
    acc = HT.Accept(lib, module, logits=logits, tokens=tokens, b_live=8, scale=MULT, cap=CAP, accept_override=forced)
    capped = torch.tanh((lg * MULT) / CAP) * CAP
    words, ring = acc.words.cpu(), acc.out_ring.cpu()
    for it in range(6):
        acc.launch(stream())
        torch.cuda.synchronize()
        step = A.greedy_accept(tok[:8], capped[:8], int(words[0]), forced=int(forced[it % 4]))
        words, ring = A.step_words(words, ring, step, tok)
        assert torch.equal(acc.words.cpu(), words), it
        assert torch.equal(acc.out_ring.cpu(), ring), it
    # without the table, b_live 8 caps the accept at 7 although the logits confirm 9 drafts
    acc2 = HT.Accept(lib, module, logits=logits, tokens=tokens, b_live=8, scale=MULT, cap=CAP)
    acc2.launch(stream())
    torch.cuda.synchronize()
    assert acc2.words.cpu()[:4].tolist() == [8, int(A.first_argmax(capped)[7]), 7, 8]


def test_accept_full_vocab_argmax():
    """202048 columns x 16 rows: arg-max of the soft-capped row equals the oracle's, with duplicated maxima and a NaN row."""
    lib, module = ctx()
    gen = torch.Generator().manual_seed(3)
    lg = torch.randn(16, 202048, generator=gen) * 6
    lg[4, 150000] = lg[4, 777] = 60.0  # a tie: the lower id
    lg[9, 201000] = float("nan")
    lg[12, 202047] = 70.0  # the last column
    tok = torch.randint(0, 202048, (16,), generator=gen)
    acc = HT.Accept(lib, module, logits=lg.to(DEV), tokens=tok.to(DEV), b_live=16, scale=MULT, cap=CAP)
    acc.launch(stream())
    torch.cuda.synchronize()
    ref = A.first_argmax(torch.tanh((lg * MULT) / CAP) * CAP)
    assert torch.equal(acc.top1.cpu().long(), ref)
    assert ref[4] == 777 and ref[9] == 201000 and ref[12] == 202047


@pytest.mark.parametrize("n,k,rows", [(8192, 1024, 16), (2304, 8192, 16), (1000, 512, 5), (25256, 8192, 16)])
def test_tensor_core_gemm_replays_with_alternating_weights(n, k, rows):
    """The tensor-core dense engine launched back to back with programmatic dependent launch on ONE output, partial-sum
    scratch and ticket block, alternating between two weight images: every launch's result must be its own image's (a
    launch that overtook its predecessor's epilogue, or a ticket left out of step, would mix the two), and the tickets
    are back at zero after every launch."""
    from sgl_muse_mega_b200.common import host
    from sgl_muse_mega_b200.muse_spark.b200 import weights as W

    lib, module = ctx()
    gen = torch.Generator(device=DEV).manual_seed(n + k)
    ws = [(torch.randn(n, k, generator=gen, device=DEV) * k**-0.5).bfloat16() for _ in range(2)]
    x = torch.randn(rows, k, generator=gen, device=DEV).bfloat16()
    refs = [x.float() @ w.float().T for w in ws]
    out = torch.zeros(rows, n, dtype=torch.float32, device=DEV)
    tiles = (n + 127) // 128
    ticket_bytes = (tiles * 4 + 255) // 256 * 256
    ws_bytes = (2 * 148 + 2 * tiles) * 2048 * 4 + ticket_bytes + 512
    scratch = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(16, dtype=torch.int32, device=DEV)
    launches = []
    images = [W.pack_umma(w) for w in ws]  # kept alive: the binds hold their addresses
    for img in images:
        bind = host.make("MkLmHeadBind", w=img, x=x, out_peer=[out], rank=0, v_total=n, col0=0, n_out=n, hidden=k,
                         rows=rows, status=status, flags=None, flags_peer=[], ws=scratch, ws_bytes=ws_bytes, w_packed=2)  # fmt: skip
        launches.append((lib.bind("mk_lm_head_bind", module, bind), bind))
    for count, pdl in ((1, False), (4, True), (7, True), (2, False)):
        for i in range(count):
            launches[i % 2][0](stream(), pdl)
        torch.cuda.synchronize()
        ref = refs[(count - 1) % 2]
        rel = ((out - ref).norm(dim=1) / ref.norm(dim=1)).max().item()
        assert rel < 1e-4, (count, pdl, rel)
        tickets = scratch[ws_bytes - 512 - ticket_bytes : ws_bytes - 512].view(torch.int32)
        assert not bool(tickets.any()), "a tile's ticket did not wrap back to zero"
    assert int(status[0]) == 0
