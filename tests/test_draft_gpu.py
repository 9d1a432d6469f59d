"""The DFlash2 draft step on the GPU against the CPU oracle: every stage fed the kernels' own inputs (GEMMs to a
tolerance, the f32 row work to one bf16 ulp, integer results exactly), the whole step end to end, replay as a CUDA graph,
and the pool sync."""

import pytest
import torch

from oracle import dflash_draft as D
from sgl_muse_mega_b200.common import host
from sgl_muse_mega_b200.muse_spark.b200.dflash import draft as DR
from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic
from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig, rope_cos_sin

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
BF = torch.bfloat16

CFG = DraftConfig(hidden=512, layers=2, q_heads=8, kv_heads=4, head_dim=128, inter=1024, vocab=2048, sliding_window=24,
                  mask_id=2002, selector_rank=64, top_k=16)  # fmt: skip
GEMM_TOL = 6e-3  # f32 tensor-core accumulation against f64, both rounded once to bf16
ATTN_TOL = 1e-2


def rel(got: torch.Tensor, ref: torch.Tensor) -> float:
    g, r = got.double().flatten(), ref.double().flatten()
    return float((g - r).norm() / r.norm().clamp_min(1e-30))


def ulps(got: torch.Tensor, ref: torch.Tensor) -> int:
    """Largest distance in bf16 steps (sign-magnitude patterns mapped to a line)."""
    def line(x):
        i = x.contiguous().view(torch.int16).int()
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return int((line(got) - line(ref)).abs().max())


def close_rows(got, ref, name, frac=2e-3):
    """Elementwise f32 work: at most one bf16 step apart, and on few elements (the f64 sums of squares here and the
    reference's differ in the last bits before their f32 rounding)."""
    g, r = got.cpu(), ref.cpu()
    if ulps(g, r) > 1:
        # an element far below its row's largest (a rotation that cancels) moves by several of its own bf16 steps when a
        # cosine differs in its last f32 bit between this host's libm and the device: such elements are held to one step
        # of 1/64 of the row's largest value instead
        gf, rf = g.float(), r.float()
        floor = rf.abs().amax(dim=-1, keepdim=True) / 64
        allowed = torch.maximum(rf.abs(), floor) * 2.0**-7
        assert bool(((gf - rf).abs() <= allowed).all()), (name, ulps(g, r), float(((gf - rf).abs() / allowed).max()))
    assert float((g != r).float().mean()) <= frac, (name, float((g != r).float().mean()))


class Checker:
    def __init__(self, world: DR.DraftWorld):
        self.world, self.case, self.cfg = world, world.case, world.case.cfg
        self.worst = {}

    def note(self, name, v):
        self.worst[name] = max(self.worst.get(name, 0.0), v)

    def gemm(self, got, x, w, name, tol=GEMM_TOL):
        r = rel(got.cpu(), D.mm(x.cpu(), w.cpu()))
        self.note(name, r)
        assert r < tol, (name, r)

    def entry(self):
        case, cfg = self.case, self.cfg
        pos0 = case.pos - case.commit
        ctx_raw = None
        for r, dr in enumerate(self.world.ranks):
            w, t = case.shards[r]
            assert torch.equal(dr.feats.cpu(), D.feats_of(case.caps))
            n = cfg.hidden // case.ranks
            self.gemm(dr.x.ctx_raw[:, r * n : (r + 1) * n], dr.feats, w.fc, "fc")
            if ctx_raw is None:
                ctx_raw = dr.x.ctx_raw.cpu()
            assert torch.equal(dr.x.ctx_raw.cpu(), ctx_raw)  # every rank gathered the same rows
            close_rows(dr.ctx, D.rms_norm(ctx_raw, w.hidden_norm, cfg.rms_eps), "ctx")
            w_kv = torch.cat([lw.qkv[cfg.q_rank(case.ranks) * cfg.head_dim :] for lw in w.layers])  # dr.w holds the packed image
            self.gemm(dr.kv, dr.ctx, w_kv, "ctx_kv")
            cos, sin = rope_cos_sin(pos0 + torch.arange(case.rows), cfg.head_dim, cfg.rope_theta)
            kvh = cfg.kv_rank(case.ranks)
            kv = dr.kv.cpu().view(case.rows, cfg.layers, 2, kvh, cfg.head_dim)
            for li, lw in enumerate(w.layers):
                k = D.head_norm_rope(kv[:, li, 0], lw.k_norm, cfg.rms_eps, cos, sin, False)
                close_rows(dr.k_pool[li][pos0 : case.pos], k[: case.commit], "ctx_k")
                assert torch.equal(dr.v_pool[li][pos0 : case.pos].cpu(), kv[: case.commit, li, 1])
                # rows past the commit are not written (the block's own rows land there later); history is untouched
                assert torch.equal(dr.k_pool[li][:pos0].cpu(), case.hist_k[li][:, r * kvh : (r + 1) * kvh])
            emb = D.embed_rows(cfg, case.shards, case.anchor, case.rows)
            assert torch.equal(dr.emb.cpu(), emb)
            close_rows(dr.h[0], D.rms_norm(emb, w.layers[0].input_norm, cfg.rms_eps), "h0")

    def layer(self, li):
        case, cfg = self.case, self.cfg
        b, d, eps = case.rows, cfg.head_dim, cfg.rms_eps
        parts_a = [dr.x.ar_attn[r].cpu()[:b] for r, dr in enumerate(self.world.ranks)]
        parts_m = [dr.x.ar_mlp[r].cpu()[:b] for r, dr in enumerate(self.world.ranks)]
        cos, sin = rope_cos_sin(case.pos + torch.arange(b), d, cfg.rope_theta)
        lo = max(0, case.pos - cfg.window_left)
        for r, dr in enumerate(self.world.ranks):
            lw, f = case.shards[r][0].layers[li], dr.f
            h_in, res_in = dr.h[li].cpu(), dr.res[li].cpu()
            qh, kvh = cfg.q_rank(case.ranks), cfg.kv_rank(case.ranks)
            self.gemm(f["c_att"], h_in, lw.attn_conv.proj, "c_att")
            c = f["c_att"].cpu().view(b, 2, cfg.conv_taps, -1)
            close_rows(f["xa"], D.grouped_conv(h_in, c[:, 0], lw.attn_conv.base[0]), "xa", frac=0.0)
            self.gemm(f["qkv"], f["xa"], lw.qkv, "qkv")
            q, k, v = f["qkv"].cpu().split([qh * d, kvh * d, kvh * d], 1)
            close_rows(f["q"], D.head_norm_rope(q.reshape(b, qh, d), lw.q_norm, eps, cos, sin, True).reshape(b, -1), "q")
            close_rows(dr.k_pool[li][case.pos : case.pos + b], D.head_norm_rope(k.reshape(b, kvh, d), lw.k_norm, eps, cos, sin, True), "k")
            assert torch.equal(dr.v_pool[li][case.pos : case.pos + b].cpu(), v.reshape(b, kvh, d))
            o = D.window_attention(f["q"].cpu().view(b, qh, d), dr.k_pool[li][lo : case.pos + b].cpu(), dr.v_pool[li][lo : case.pos + b].cpu(),
                                   case.pos + torch.arange(b), torch.arange(lo, case.pos + b), cfg.window_left).to(BF)  # fmt: skip
            ra = rel(f["o"].cpu(), o)
            self.note("attn", ra)
            assert ra < ATTN_TOL, ("attn", ra)
            self.gemm(parts_a[r], f["o"], lw.o, "o_proj")
            for other in self.world.ranks:  # the partial reached every rank's workspace
                assert torch.equal(other.x.ar_attn[r].cpu()[:b], parts_a[r])
            a = D.grouped_conv(D.all_reduce(parts_a), c[:, 1], lw.attn_conv.base[1])
            close_rows(f["a"], a, "a", frac=0.0)
            hp, rp = D.add_rms_norm(f["a"].cpu(), res_in, lw.post_norm, eps)
            close_rows(f["h_post"], hp, "h_post")
            assert torch.equal(f["res_post"].cpu(), rp)
            self.gemm(f["c_mlp"], f["h_post"], lw.mlp_conv.proj, "c_mlp")
            c2 = f["c_mlp"].cpu().view(b, 2, cfg.conv_taps, -1)
            close_rows(f["xm"], D.grouped_conv(f["h_post"].cpu(), c2[:, 0], lw.mlp_conv.base[0]), "xm", frac=0.0)
            gate, up = D.mm(f["xm"].cpu(), lw.gate_up).chunk(2, 1)
            rm = rel(f["m"].cpu(), D.silu_mul(gate, up))
            self.note("swiglu", rm)
            assert rm < 2 * GEMM_TOL, ("swiglu", rm)
            self.gemm(parts_m[r], f["m"], lw.down, "down")
            x = D.grouped_conv(D.all_reduce(parts_m), c2[:, 1], lw.mlp_conv.base[1])
            close_rows(f["x_out"], x, "x_out", frac=0.0)
            last = li == cfg.layers - 1
            nw = case.shards[r][0].norm if last else case.shards[r][0].layers[li + 1].input_norm
            hn, rn = D.add_rms_norm(f["x_out"].cpu(), f["res_post"].cpu(), nw, eps)
            close_rows(dr.h[li + 1], hn, "h_next")
            if not last:
                assert torch.equal(dr.res[li + 1].cpu(), rn)

    def head(self):
        case, cfg = self.case, self.cfg
        g0 = self.world.ranks[0].x.gathered.cpu()
        n = cfg.vocab // case.ranks
        for r, dr in enumerate(self.world.ranks):
            assert torch.equal(dr.x.gathered.cpu(), g0)
            ref = D.mm(dr.y[1:].cpu(), case.shards[r][1].lm_head, torch.float32)
            rr = rel(g0[:, r * n : (r + 1) * n], ref)
            self.note("lm_head", rr)
            assert rr < 1e-3, rr
            w = case.shards[r][0]
            self.gemm(dr.hid, dr.y[1:], w.hidden_proj, "hproj")
            cand, unary = D.candidates_from_logits(cfg, g0)
            assert torch.equal(dr.cand.cpu(), cand)
            assert torch.allclose(dr.unary.cpu(), unary, rtol=0, atol=2e-6)
            scores = D.lattice_from_hid(w, dr.hid.cpu(), cand, dr.unary.cpu(), case.anchor)
            assert torch.equal(dr.scores.cpu(), scores)
            drafts, picks = D.walk(cand, dr.scores.cpu())
            assert torch.equal(dr.drafts.cpu(), drafts) and torch.equal(dr.pick.cpu().long(), picks)
            assert dr.verify_ids.cpu().tolist() == [case.anchor] + drafts.tolist()


def run_world(ranks, rows, pos, commit, seed):
    case = synthetic.draft_case(CFG, ranks, rows, pos, commit, seed)
    world = DR.DraftWorld(case, DEV)
    chk = Checker(world)
    n_layers = CFG.layers

    def after(li):
        torch.cuda.synchronize()
        if li == 0:
            chk.entry()
        elif li <= n_layers:
            chk.layer(li - 1)
        elif li == n_layers + 2:
            chk.head()

    world.run_interleaved(after)
    torch.cuda.synchronize()
    for dr in world.ranks:
        assert dr.statuses() == [], dr.statuses()
    return case, world, chk


@pytest.mark.parametrize("ranks,rows,pos,commit", [(2, 16, 40, 7), (1, 8, 12, 3), (1, 16, 33, 16)])
def test_draft_stagewise_and_end_to_end(ranks, rows, pos, commit):
    case, world, chk = run_world(ranks, rows, pos, commit, 11)
    print({k: f"{v:.2e}" for k, v in sorted(chk.worst.items())})
    # end to end against the oracle's own chain (its all-reduce order and GEMM roundings differ by ulps per stage)
    kv = D.DraftKV.empty(CFG, ranks, pos + rows)
    kvh = CFG.kv_rank(ranks)
    for r in range(ranks):
        for li in range(CFG.layers):
            kv.k[r][li][: pos - commit] = case.hist_k[li][:, r * kvh : (r + 1) * kvh]
            kv.v[r][li][: pos - commit] = case.hist_v[li][:, r * kvh : (r + 1) * kvh]
    ref = D.draft_step(CFG, case.shards, kv, case.caps, case.anchor, pos, commit, rows)
    y = world.ranks[0].y.cpu()
    d = (y.float() - ref["y"].float()).norm(dim=1) / ref["y"].float().norm(dim=1)
    assert float(d.max()) < 3e-2, d


def test_draft_item_images_give_the_same_bits():
    """The draft's GEMM weights as item images: bit-identical results to row-major weights."""
    case = synthetic.draft_case(CFG, 2, 16, 40, 7, 11)
    a, b = DR.DraftWorld(case, DEV, packed=0), DR.DraftWorld(case, DEV, packed=1)
    a.run_interleaved()
    b.run_interleaved()
    torch.cuda.synchronize()
    for ra, rb in zip(a.ranks, b.ranks):
        assert ra.statuses() == [] and rb.statuses() == []
        for k in ("y", "scores", "verify_ids", "cand", "unary", "hid", "kv", "ctx"):
            assert torch.equal(getattr(ra, k), getattr(rb, k)), k
        assert torch.equal(ra.x.gathered, rb.x.gathered)
        for li in range(CFG.layers):
            assert torch.equal(ra.k_pool[li], rb.k_pool[li]) and torch.equal(ra.v_pool[li], rb.v_pool[li])


def test_sampled_walk_matches_the_oracle():
    """Temperature > 0: the head walks the lattice by sampling with the step's Philox uniforms. Uniforms, picks and tokens
    exactly as the oracle's walk over the kernel's own lattice, probabilities to f32 rounding."""
    seed, stream, temp = 0x1234567887654321, 40, 0.7
    case = synthetic.draft_case(CFG, 1, 16, 40, 7, 11)
    samp = DR.sampling_words(seed, stream, temp).to(DEV)
    world = DR.DraftWorld(case, DEV, samp=samp)
    dr = world.ranks[0]
    for iteration in (0, 5):
        dr.words[4] = iteration  # the step counter keys the uniforms
        world.run_interleaved()
        torch.cuda.synchronize()
        assert dr.statuses() == []
        u = D.uniforms(seed, stream, iteration, D.PURPOSE_WALK)
        toks, picks, q = D.walk_sampled(dr.cand.cpu(), dr.scores.cpu(), u, temp)
        got_q = dr.walk_q.cpu()
        # the walk conditions slot e on slot e - 1's pick: compare slot by slot along the kernel's own path
        prev = 0
        for e in range(case.rows - 1):
            row = dr.scores[e, prev].cpu() / temp
            ref_q = torch.softmax(row, 0)
            assert torch.allclose(got_q[e], ref_q, rtol=0, atol=2e-6), (iteration, e)
            cum = torch.cumsum(got_q[e], 0)
            idx = min(int((u[e] >= cum).sum()), 15)
            if float((cum - u[e]).abs().min()) > 1e-5:  # away from a boundary of the CDF the draw is unambiguous
                assert int(dr.pick[e]) == idx, (iteration, e)
            prev = int(dr.pick[e])
            assert int(dr.drafts[e]) == int(dr.cand[e, prev]) == int(dr.verify_ids[1 + e])
        if torch.equal(dr.pick.cpu().long(), picks):
            assert torch.equal(dr.drafts.cpu(), toks)
    # another iteration count draws other uniforms
    assert not torch.equal(D.uniforms(seed, stream, 0, 0), D.uniforms(seed, stream, 5, 0))


def test_draft_step_replays_as_a_graph():
    """A lone rank: the whole launch list under programmatic dependent launch, eager and as one CUDA graph, gives the
    stagewise run's results bit for bit; a second replay after new step words moves the block."""
    case = synthetic.draft_case(CFG, 1, 16, 40, 7, 5)
    world = DR.DraftWorld(case, DEV)
    dr = world.ranks[0]
    world.run_interleaved()
    torch.cuda.synchronize()
    want = dict(y=dr.y.cpu().clone(), ids=dr.verify_ids.cpu().clone(), scores=dr.scores.cpu().clone(), k=dr.k_pool[1].cpu().clone())
    s = torch.cuda.current_stream().cuda_stream
    assert dr.kernels() == 6 + 10 * CFG.layers + 1 + 3
    dr.launch_all(s, pdl=True)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(DEV)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            dr.launch_all(torch.cuda.current_stream().cuda_stream, pdl=True)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        dr.y.zero_(), dr.verify_ids.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(dr.y.cpu(), want["y"]) and torch.equal(dr.verify_ids.cpu(), want["ids"])
        assert torch.equal(dr.scores.cpu(), want["scores"]) and torch.equal(dr.k_pool[1].cpu(), want["k"])
    # the next iteration: 5 tokens committed, a new anchor; the graph reads it all from the words
    dr.set_state(45, 77, 5)
    g.replay()
    torch.cuda.synchronize()
    assert dr.statuses() == []
    assert int(dr.verify_ids[0]) == 77
    assert not torch.equal(dr.k_pool[1][45:61].cpu(), want["k"][45:61])
    assert torch.equal(dr.k_pool[1][:40].cpu(), want["k"][:40])


def test_kv_sync_moves_committed_rows():
    lib = host.library()
    mod = lib.load()
    ring_rows, row_bytes, n_buf = 64, 256, 4
    g = torch.Generator().manual_seed(3)
    rings = [torch.randint(0, 255, (ring_rows, row_bytes), dtype=torch.uint8, generator=g).to(DEV) for _ in range(n_buf)]
    pools = [torch.zeros(200, row_bytes, dtype=torch.uint8, device=DEV) for _ in range(n_buf)]
    ring_ptr = torch.tensor([t.data_ptr() for t in rings], dtype=torch.int64, device=DEV)
    pool_ptr = torch.tensor([t.data_ptr() for t in pools], dtype=torch.int64, device=DEV)
    words = torch.zeros(8, dtype=torch.int64, device=DEV)
    words[0], words[3] = 75, 5  # P, last commit: the rings hold positions < 70
    state = torch.zeros(17, dtype=torch.int64, device=DEV)
    state[0] = 66
    slots = torch.arange(16) * 3 + 100
    state[1:] = slots.to(DEV)
    window = (torch.arange(16) + 20).to(DEV)
    status = torch.zeros(16, dtype=torch.int32, device=DEV)
    bind = host.make("MkDflashKvSyncBind", words=words, window=window, state=state, ring=ring_ptr, pool=pool_ptr, n_buf=n_buf,
                     row_bytes=row_bytes, ring_rows=ring_rows, lag=1, status=status)  # fmt: skip
    launch = lib.bind("mk_dflash_kv_sync_bind", mod, bind)
    s = torch.cuda.current_stream().cuda_stream
    launch(s, False)
    torch.cuda.synchronize()
    assert launch.status(s).code == 0
    for b in range(n_buf):
        for i in range(4):  # positions 66..69 -> slots 100, 103, 106, 109
            assert torch.equal(pools[b][int(slots[i])].cpu(), rings[b][(66 + i) % ring_rows].cpu())
        assert int(pools[b].sum()) == int(sum(rings[b][(66 + i) % ring_rows].sum() for i in range(4)))
    assert int(state[0]) == 70 and state[1:].tolist() == window.tolist()
    # a pool that lags by more than a window: nothing copied, recorded
    state[0] = 10
    launch(s, False)
    torch.cuda.synchronize()
    st = launch.status(s)
    assert st.code == 4 and st.stage == 440
