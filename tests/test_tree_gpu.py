"""The token tree on the GPU through the C ABI: the draft head's tree walk, the tree accept and the compaction of the
accepted path, each against the oracle (``oracle/dflash_tree.py``, pinned to the reference's outputs) on the kernels' own
inputs. Bit-exact: the tree is integer work over fp32 log-probabilities that the oracle forms with the same roundings."""

import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import make_tree_golden as G  # noqa: E402  (the seeded lattices; nothing here reads the reference)

from oracle import dflash_accept as A  # noqa: E402
from oracle import dflash_tree as T  # noqa: E402
from sgl_muse_mega_b200.common import host  # noqa: E402
from sgl_muse_mega_b200.muse_spark.b200 import headtail as HT  # noqa: E402
from sgl_muse_mega_b200.muse_spark.b200.dflash import tree as TR  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROWS = 16
_ctx = {}


def ctx():
    if "lib" not in _ctx:
        _ctx["lib"] = host.library()
        with torch.cuda.device(DEV):
            _ctx["module"] = _ctx["lib"].load()
    return _ctx["lib"], _ctx["module"]


def stream() -> int:
    return torch.cuda.current_stream(DEV).cuda_stream


def walk(cand, scores, anchor):
    lib, module = ctx()
    words = torch.zeros(8, dtype=torch.int64, device=DEV)
    words[1] = anchor
    ids = torch.zeros(ROWS, dtype=torch.int64, device=DEV)
    loc_full = (torch.arange(ROWS, dtype=torch.int32) + 40).to(DEV)
    loc_swa = (torch.arange(ROWS, dtype=torch.int32) + 7).to(DEV)
    w = TR.TreeWalk(lib, module, cand=cand.to(DEV), scores=scores.to(DEV).contiguous(), words=words, verify_ids=ids,
                    loc_full=loc_full, loc_swa=loc_swa)  # fmt: skip
    w.launch(stream(), False)
    torch.cuda.synchronize()
    return w, ids


CASES = [G.lattice(s, t) for s, t in G.LATTICES] + [G.peaked()]


@pytest.mark.parametrize("i", range(len(CASES)))
def test_tree_walk_equals_the_oracle(i):
    cand, scores = CASES[i]
    w, ids = walk(cand, scores, 7 + i)
    want = T.token_tree(7 + i, cand, scores)
    got = w.rows()
    assert (got["parent"], got["depth"], got["mask"]) == (want.parent, want.depth, want.mask)
    assert ids.cpu().tolist() == want.tokens
    t = w.table.cpu().tolist()
    assert t[TR.SLOT_FULL : TR.SLOT_FULL + ROWS] == list(range(40, 56)) and t[TR.SLOT_SWA : TR.SLOT_SWA + ROWS] == list(range(7, 23))


@pytest.mark.parametrize("i,forced", [(0, None), (3, None), (7, None), (11, None), (18, None), (5, 9), (12, 0), (14, 15)])
def test_tree_accept_equals_the_oracle(i, forced):
    """The greedy accept with the tree's table: logits whose arg-max confirms a seeded path of the tree (and nothing below
    it): accept length, committed tokens, bonus, step words and the path left in the table."""
    lib, module = ctx()
    cand, scores = CASES[i]
    w, ids = walk(cand, scores, 7 + i)
    tree = T.token_tree(7 + i, cand, scores)
    vocab = 12000
    leaf, t1 = G.accept_inputs(tree.tokens, tree.mask, i)
    t1 = [x % vocab for x in t1]  # the seeded ids of rows off the path: any id no child carries
    for r in range(ROWS):
        kids = {tree.tokens[c] for c in range(1, ROWS) if tree.parent[c] == r}
        on = {c for c in range(1, ROWS) if (tree.mask[leaf] >> c) & 1}
        nxt = [c for c in on if tree.parent[c] == r]
        if not nxt:
            while t1[r] in kids:
                t1[r] = (t1[r] + 1) % vocab
    gen = torch.Generator().manual_seed(50 + i)
    logits = torch.randn(ROWS, vocab, generator=gen)
    for r in range(ROWS):
        logits[r, t1[r]] = 30.0
    override = None if forced is None else torch.tensor([forced], dtype=torch.int32, device=DEV)
    acc = HT.Accept(lib, module, logits=logits.to(DEV), tokens=ids, b_live=ROWS, scale=1.0, cap=20.0, ring=64,
                    accept_override=override, tree=w.table)  # fmt: skip
    pos = 100 + i
    acc.words[A.WORDS["P"]] = pos
    acc.launch(stream(), False)
    torch.cuda.synchronize()
    want = T.tree_accept(tree, torch.tensor(t1), pos, forced=forced)
    assert acc.top1.cpu().tolist() == t1
    words = acc.words.cpu().tolist()
    assert (words[A.WORDS["P"]], words[A.WORDS["ANCHOR"]], words[A.WORDS["ACCEPT"]], words[A.WORDS["COMMIT"]]) == (
        want.new_pos, want.bonus, want.accept_len, want.commit_len)  # fmt: skip
    assert acc.out_ring.cpu().tolist()[: want.commit_len] == want.committed
    path = w.rows()["path"]
    assert path[0] == want.accept_len and path[1 : 1 + want.accept_len] == want.path
    if forced is None:
        assert want.path == [c for c in range(1, ROWS) if (tree.mask[leaf] >> c) & 1]


@pytest.mark.parametrize("i,leaf,path", [(2, 13, None), (5, 13, None), (11, 13, None), (14, 12, None), (8, 5, None),
                                         (2, None, [2, 3, 5, 6, 15]), (2, None, [15])])  # fmt: skip
def test_tree_compact_moves_the_accepted_path(i, leaf, path):
    """K / V pools (by the table's slots, sliding-window and full) and capture buffers (by window row): after the launch the
    rows at depths 1 .. accept hold what the path's rows held; every other row is untouched. Paths of a tree's leaves that
    are no chain prefix, and two written by hand (a path whose source rows are also destinations; one row)."""
    lib, module = ctx()
    cand, scores = CASES[i]
    w, _ = walk(cand, scores, 3)
    if path is None:
        tree = T.token_tree(3, cand, scores)
        path = [r for r in range(1, ROWS) if (tree.mask[leaf] >> r) & 1]
        assert len(path) >= 3
    assert path != list(range(1, len(path) + 1))  # a path that moves rows
    tab = w.table.cpu()
    tab[TR.PATH] = len(path)
    tab[TR.PATH + 1 : TR.PATH + 1 + len(path)] = torch.tensor(path, dtype=torch.int32)
    w.table.copy_(tab)
    gen = torch.Generator().manual_seed(9)
    swa = [torch.randn(64, 128, generator=gen).bfloat16().to(DEV) for _ in range(3)]
    full = [torch.randn(96, 128, generator=gen).bfloat16().to(DEV) for _ in range(2)]
    caps = [torch.randn(ROWS, 1024, generator=gen).to(DEV) for _ in range(5)]
    before = [t.clone() for t in swa + full + caps]
    c = TR.TreeCompact(lib, module, table=w.table, swa=swa, full=full, caps=caps)
    c.launch(stream(), False)
    torch.cuda.synchronize()
    for j, (now, was) in enumerate(zip(swa + full + caps, before)):
        base = 7 if j < 3 else 40 if j < 5 else 0  # the window's first slot in the pool (capture buffers: window rows)
        want = was.clone()
        for d, r in enumerate(path, start=1):
            want[base + d] = was[base + r]
        assert torch.equal(now, want), j


@pytest.mark.parametrize("name", ["small_fp4_swa_tp2", "small_fp4_global_tp8_baseline"])
def test_tree_window_attention_follows_the_ancestor_masks(name):
    """A layer bound with a tree table: the attention places row r at the context length + depth(r) and lets it see, of the
    window's own keys, its ancestors only (sliding-window layers count the window from that position). x_attn of every
    rank against the oracle's attention with the same tree on the rank's own qkv rows and context."""
    from golden_cases import CASES as LAYER_CASES
    from oracle import muse_layer as O
    from sgl_muse_mega_b200.muse_spark.b200 import layer as L
    from sgl_muse_mega_b200.muse_spark.b200 import synthetic

    cfg, kw = LAYER_CASES[name]
    case = synthetic.layer_case(cfg, **kw)
    assert case.rows == ROWS
    cand, scores = CASES[7]
    tree = T.token_tree(1, cand, scores)
    assert max(tree.depth) < ROWS - 1 and tree.parent != [-1] + list(range(ROWS - 1))  # a branching tree
    table = torch.zeros(TR.TABLE_WORDS, dtype=torch.int32)
    table[TR.PARENT : TR.PARENT + ROWS] = torch.tensor(tree.parent, dtype=torch.int32)
    table[TR.DEPTH : TR.DEPTH + ROWS] = torch.tensor(tree.depth, dtype=torch.int32)
    table[TR.MASK : TR.MASK + ROWS] = torch.tensor(tree.mask, dtype=torch.int32)
    table = table.to(DEV)
    world = L.LayerWorld(case, DEV)
    for r in world.ranks:
        r.bind(world.ranks, tree=table)
    world.run_interleaved()
    torch.cuda.synchronize()
    chain = L.LayerWorld(case, DEV)
    chain.run_interleaved()
    torch.cuda.synchronize()
    for r, plain in zip(world.ranks, chain.ranks):
        assert r.launch_record.status(stream()).code == 0
        t = case.ranks[r.rank]
        want = O.attention(t.qkv_in, t.k_ctx, t.v_ctx, case.window, tree=(tree.depth, tree.mask)).float()
        got = r.o["x_attn"].cpu().float()
        rel = float((got - want).norm() / want.norm())
        assert rel < 6e-3, (r.rank, rel)
        off = float((plain.o["x_attn"].cpu().float() - want).norm() / want.norm())
        assert off > 10 * rel, (rel, off)  # the chain's attention is something else


def test_tree_iteration_walks_accepts_and_compacts():
    """Three fused iterations of a stack built with ``tree=True`` (draft, tree walk, verify step, tree accept, compaction),
    launched piece by piece so that the rows can be read before the compaction moves them: the table equals the oracle's
    tree over the draft head's own lattice, the step words equal the oracle's
    tree accept on the step's own arg-max ids (forced leaves: the natural accept is covered above), and the compaction leaves the accepted
    path's K / V and captured rows where a chain would have written them."""
    from sgl_muse_mega_b200.muse_spark.b200 import stack as S
    from sgl_muse_mega_b200.muse_spark.b200 import synthetic
    from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic as dsyn
    from sgl_muse_mega_b200.muse_spark.b200.dflash.iteration import Iteration
    from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig, shard
    from sgl_muse_mega_b200.muse_spark.config import Config

    cfg = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7,
                 vocab=4096, layers=4, bf16_moe_layers=(0,), tp=1, node_ranks=1)  # fmt: skip
    dcfg = DraftConfig(hidden=1024, layers=2, q_heads=8, kv_heads=4, head_dim=128, inter=1024, vocab=4096, sliding_window=24,
                       mask_id=4001, selector_rank=64, top_k=16, capture=(0, 1, 2, 3, 2))  # fmt: skip
    ctx_len = 24
    case = synthetic.stack_case(cfg, n_layers=4, rows=ROWS, ctx=ctx_len, seed=12)
    forced = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = S.Stack(case, 0, DEV, tree=True, accept_override=forced)
    st.bind()
    dw, dt = dsyn.draft_weights(dcfg, 4), dsyn.target_shared(dcfg, 4)
    w0, _ = shard(dcfg, dw, dt, 0, 1)
    it = Iteration(st, dcfg, w0, capture=list(dcfg.capture), pool_rows=64, rope_rows=128)
    assert it.tree_walk is not None and it.kernels == it.draft.kernels() + st.kernels + 2
    s = stream()
    st.feeds.launch(s)
    torch.cuda.synchronize()
    pos, anchor = ctx_len, 0
    moved = 0
    for i, leaf in enumerate([0, 9, 14]):
        # forced leaves: rows a natural accept of random weights never reaches
        forced.fill_(leaf)
        it.draft.launch_all(s, False, None)
        it.tree_walk.launch(s, False)
        st.launch_all(s, False)
        torch.cuda.synchronize()
        assert it.statuses() == []
        tree = T.token_tree(anchor, it.draft.cand.cpu(), it.draft.scores.cpu())
        got = it.tree_walk.rows()
        assert (got["parent"], got["depth"], got["mask"]) == (tree.parent, tree.depth, tree.mask), i
        assert st.tokens.cpu().tolist() == tree.tokens
        acc = T.tree_accept(tree, st.accept.top1.cpu(), pos, forced=leaf)
        words = st.accept.words.cpu().tolist()
        assert (words[A.WORDS["P"]], words[A.WORDS["ANCHOR"]], words[A.WORDS["ACCEPT"]], words[A.WORDS["COMMIT"]]) == (
            acc.new_pos, acc.bonus, acc.accept_len, acc.commit_len), i  # fmt: skip
        path = it.tree_walk.rows()["path"]
        assert path[0] == acc.accept_len and path[1 : 1 + acc.accept_len] == acc.path
        tab = st.tree_table.cpu().tolist()
        slots = {True: tab[TR.SLOT_FULL : TR.SLOT_FULL + ROWS], False: tab[TR.SLOT_SWA : TR.SLOT_SWA + ROWS]}
        pools = [(lr.case.global_attn, t) for lr, kv in zip(st.layers, st.pools) for t in kv]
        caps = list(dict.fromkeys(st.layers[c].o["stream_out"] for c in it.capture))
        before = [t.clone() for _, t in pools] + [t.clone() for t in caps]
        it.tree_compact.launch(s, False)
        torch.cuda.synchronize()
        for j, was in enumerate(before):
            now = pools[j][1] if j < len(pools) else caps[j - len(pools)]
            want = was.clone()
            for d, r in enumerate(acc.path, start=1):
                if j < len(pools):
                    sl = slots[pools[j][0]]
                    want[sl[d]] = was[sl[r]]
                else:
                    want[d] = was[r]
                moved += int(d != r)
            assert torch.equal(now, want), (i, j)
        pos, anchor = acc.new_pos, acc.bonus
    assert moved > 0  # at least one forced path was no chain prefix
    # the same iteration as one graph: three more replays run clean and keep advancing
    forced.fill_(5)
    it.capture_graph(warmup=False)
    for i in range(3):
        it.step()
        torch.cuda.synchronize()
        assert it.statuses() == []
        w = st.accept.words.cpu().tolist()
        d = it.tree_walk.rows()["depth"][5]
        pos += d + 1
        assert w[A.WORDS["P"]] == pos and w[A.WORDS["ACCEPT"]] == d
