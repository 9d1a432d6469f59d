"""The fused DFlash2 iteration as the serving framework's worker drives it (``runtime/iteration.py`` ``Fused``): requests
whose slots are scattered over the framework's pools, against a plain ``Iteration`` on identity slots. The tokens, commit
lengths, bonus tokens and committed lengths must be equal step by step (same kernels, same values; only the addressing and
the state hand-over differ), the target's K / V rows must land in the slots the request table names, and the draft's K / V
of every committed position must reach the framework's draft pool (one iteration late, the run's last commit by the
flush)."""

from types import SimpleNamespace as NS

import pytest
import torch

from fake_sglang import FakeRequest, decode_batch, draft_checkpoint, draft_hf_config, experts_of, fake_model
from sgl_muse_mega_b200.muse_spark import draft as DS
from sgl_muse_mega_b200.muse_spark.b200 import headtail as HT
from sgl_muse_mega_b200.muse_spark.b200 import stack as S
from sgl_muse_mega_b200.muse_spark.b200 import synthetic
from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic as dsyn
from sgl_muse_mega_b200.muse_spark.b200.dflash.draft import sampling_words
from sgl_muse_mega_b200.muse_spark.b200.dflash.iteration import Iteration
from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig, shard
from sgl_muse_mega_b200.muse_spark.config import Config
from sgl_muse_mega_b200.muse_spark.runtime import build as B
from sgl_muse_mega_b200.muse_spark.runtime import iteration as IT
from sgl_muse_mega_b200.muse_spark.runtime import shim

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
BF = torch.bfloat16
W = HT.WORDS

CFG = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7, vocab=4096,
             layers=4, bf16_moe_layers=(0,), tp=1, node_ranks=1)  # fmt: skip
DCFG = DraftConfig(hidden=1024, layers=2, q_heads=8, kv_heads=4, head_dim=128, inter=1024, vocab=4096, sliding_window=24,
                   mask_id=4001, selector_rank=64, top_k=16, capture=(0, 1, 2, 3, 2))  # fmt: skip
ROWS, CTX, STEPS = 16, 24, 4
SLOTS_FULL, SLOTS_SWA, WIDTH = 1024, 768, 256
BONUS = 77


def plain_run(case, w0, draft_ctx, sampling=None, **stack_kw):
    """STEPS iterations of a plain stack on identity slots from the request's state: per step (tokens, commit, bonus, P)
    and the draft's rings at the end."""
    st = S.Stack(case, 0, DEV, sampling=sampling, **stack_kw)
    st.bind()
    it = Iteration(st, DCFG, w0, capture=list(DCFG.capture), pool_rows=256, rope_rows=WIDTH + 2 * ROWS)
    for l, (k, v) in enumerate(draft_ctx):
        it.draft.k_pool[l].view(256, -1)[:CTX] = k.to(DEV)
        it.draft.v_pool[l].view(256, -1)[:CTX] = v.to(DEV)
    st.accept.words[W["ANCHOR"]] = BONUS
    s = torch.cuda.current_stream().cuda_stream
    st.feeds.launch(s)
    steps = []
    for _ in range(STEPS):
        it.launch_all(s, pdl=False)
        torch.cuda.synchronize()
        assert it.statuses() == []
        w = st.accept.words.cpu().tolist()
        commit, count = w[W["COMMIT"]], w[W["OUT_COUNT"]]
        ring = st.accept.out_ring.cpu()
        toks = [int(ring[(count - commit + i) % ring.shape[0]]) for i in range(commit)]
        steps.append((toks, commit, w[W["ANCHOR"]], w[W["P"]]))
    return st, it, steps


class Serving:
    """The framework's side: scattered target pools holding the context, a draft pool holding the draft's context, a
    request table whose rows 1 and 2 share the context's slots (a shared prefix) and own different slots past it."""

    def __init__(self, case, gen):
        need = CTX + (STEPS + 2) * ROWS
        perm_full = torch.randperm(SLOTS_FULL, generator=gen)
        perm_swa = torch.randperm(SLOTS_SWA, generator=gen)
        self.slots = {1: perm_full[:need], 2: torch.cat([perm_full[:CTX], perm_full[need : 2 * need - CTX]])}
        self.full_to_swa = torch.full((SLOTS_FULL + 1,), -1, dtype=torch.int64)
        used = torch.cat([self.slots[1], self.slots[2][CTX:]])
        self.full_to_swa[used] = perm_swa[: used.numel()]
        r2t = torch.zeros(3, WIDTH, dtype=torch.int32)
        for row, s in self.slots.items():
            r2t[row, :need] = s.int()
        kvh = CFG.kv_heads_rank
        ks, vs = [], []
        ctx_slots = self.slots[1][:CTX]
        for lc in case.layers:
            n = SLOTS_FULL if lc.global_attn else SLOTS_SWA
            k, v = (torch.zeros(n, kvh, 64, dtype=BF) for _ in range(2))
            where = ctx_slots if lc.global_attn else self.full_to_swa[ctx_slots]
            k[where], v[where] = lc.ranks[0].k_ctx, lc.ranks[0].v_ctx
            ks.append(k.to(DEV)), vs.append(v.to(DEV))
        self.pool = shim.KVPool(ks, vs, self.full_to_swa.to(DEV))
        self.r2t = shim.ReqToTokenPool(r2t.to(DEV))
        self.view = NS(kv_pool=self.pool, req_to_token_pool=self.r2t)
        # the draft's pool: the context's rows hold what the draft's prefill would have left there
        dk = DCFG.kv_heads
        self.draft_ctx = [tuple((torch.randn(CTX, dk * 128, generator=gen) * 0.5).to(BF) for _ in range(2)) for _ in range(DCFG.layers)]
        dks, dvs = [], []
        for k, v in self.draft_ctx:
            pk, pv = (torch.zeros(SLOTS_FULL, dk, 128, dtype=BF) for _ in range(2))
            pk.view(SLOTS_FULL, -1)[ctx_slots], pv.view(SLOTS_FULL, -1)[ctx_slots] = k, v
            dks.append(pk.to(DEV)), dvs.append(pv.to(DEV))
        self.draft_pool = shim.KVPool(dks, dvs, None)
        self.draft_model = NS(layers=[NS(self_attn=NS(attn=NS(layer_id=i))) for i in range(DCFG.layers)])


def built(case, dw):
    shim.install()
    shim.install(capture_mode=True, tp_group=shim.Parallel(0, 1), context_length=WIDTH,
                 server_spec=NS(speculative_draft_model_path="", speculative_use_block_verification=True))  # fmt: skip
    model = fake_model(case, device=DEV)
    model.model.language_model.layers_to_capture = [c + 1 for c in DCFG.capture]
    verify = B.build(model, None, shim.Context(ROWS), parallel=shim.Parallel(0, 1), experts=experts_of(case, device=DEV), cfg=CFG)
    assert B.TARGET is verify and model.built_megakernel is verify
    entries = draft_checkpoint(DCFG, dw)
    hf = NS(to_dict=lambda: draft_hf_config(DCFG))
    assert DS.model_disable_reasons(None, hf) != []  # the test's small draft is not the published one...
    DS.build(None, hf, None, read=lambda names: {n: entries[n] for n in names}, cfg=DCFG)  # ...its build takes a config
    assert verify.draft is not None and verify.draft_cfg is DCFG
    return verify


def drive(fused, serving, row: int, rid: str, req, steps_ref, published):
    """One request's run through the worker's call: each step's batch carries the framework's state of the request."""
    seq, bonus = CTX, torch.tensor([BONUS], device=DEV)
    for i, (toks, commit, ref_bonus, ref_p) in enumerate(steps_ref):
        batch = decode_batch([req], shim.DraftInput(bonus_tokens=bonus), seq_lens=torch.tensor([seq], device=DEV),
                             req_pool_indices=torch.tensor([row], device=DEV))  # fmt: skip
        out = fused(batch, needs_logits=False, on_publish=published.append)
        assert out is not None, (rid, i)
        torch.cuda.synchronize()
        assert fused.statuses() == [], (rid, i)
        n = int(out.accept_lens[0])
        assert n == commit and out.next_token_ids[:n].tolist() == toks and not out.next_token_ids[n:].any(), (rid, i)
        assert int(out.next_draft_input.bonus_tokens[0]) == ref_bonus and int(out.new_seq_lens[0]) == ref_p, (rid, i)
        assert out.logits_output.next_token_logits is None and out.speculative_num_draft_tokens == ROWS and out.can_run_cuda_graph
        assert published[-1] is out.new_seq_lens
        seq, bonus = int(out.new_seq_lens[0]), out.next_draft_input.bonus_tokens
    return seq


def test_fused_iteration_serves_greedy_and_sampled_requests_on_scattered_slots():
    gen = torch.Generator().manual_seed(21)
    case = synthetic.stack_case(CFG, n_layers=4, rows=ROWS, ctx=CTX, seed=9)
    dw, dt = dsyn.draft_weights(DCFG, 4), dsyn.target_shared(DCFG, 4)
    w0, _ = shard(DCFG, dw, dt, 0, 1)
    serving = Serving(case, gen)
    ref_st, ref_it, ref_steps = plain_run(case, w0, serving.draft_ctx)
    verify = built(case, dw)
    verify.prepare(serving.view)
    st = verify.stack
    assert st.accept is not None and st.accept_sampled is not None and st.softcap is not None and not st.identity_slots
    fused = verify.dflash_iteration(block_size=ROWS, draft_model=serving.draft_model, draft_kv_pool=serving.draft_pool)
    assert isinstance(fused, IT.Fused) and fused.sample and set(fused.graphs) == {"greedy", "sample"}
    published = []
    # ---- request A (table row 1), greedy ----
    req_a = FakeRequest("req-a")
    end = drive(fused, serving, 1, "a", req_a, ref_steps, published)
    assert fused.pending and fused.rid == "req-a"
    # the target's K / V rows of every window landed in the slots the request table names
    kvh = CFG.kv_heads_rank
    slots = serving.slots[1]
    for j, lc in enumerate(case.layers):
        where = slots[CTX:end] if lc.global_attn else serving.full_to_swa[slots[CTX:end]]
        got = serving.pool.get_key_buffer(j).view(-1, kvh * 64)[where.to(DEV)]
        assert torch.equal(got, ref_st.pools[j][0][CTX:end]), j
    # the draft's K / V of the committed positions, all but the last commit, are in the framework's draft pool
    last = ref_steps[-1][1]
    for l in range(DCFG.layers):
        ring = ref_it.draft.k_pool[l].view(256, -1)
        got = serving.draft_pool.get_key_buffer(l).view(SLOTS_FULL, -1)[slots[CTX : end - last].to(DEV)]
        assert torch.equal(got, ring[CTX : end - last]), l
        tail = serving.draft_pool.get_key_buffer(l).view(SLOTS_FULL, -1)[slots[end - last : end].to(DEV)]
        assert not tail.any(), l
    # ---- a step that is not the fused iteration's (a prefill): the run's last commit is flushed, the step is SGLang's ----
    prefill = decode_batch([FakeRequest("other")], None, mode="extend")
    assert fused(prefill, needs_logits=True, on_publish=None) is None and not fused.pending and fused.rid is None
    torch.cuda.synchronize()
    ref_it.draft.launch_all(torch.cuda.current_stream().cuda_stream, False)  # the plain draft folds the last commit too
    torch.cuda.synchronize()
    for l in range(DCFG.layers):
        for ring, pool in ((ref_it.draft.k_pool[l], serving.draft_pool.get_key_buffer(l)),
                           (ref_it.draft.v_pool[l], serving.draft_pool.get_value_buffer(l))):  # fmt: skip
            got = pool.view(SLOTS_FULL, -1)[slots[CTX:end].to(DEV)]
            assert torch.equal(got, ring.view(256, -1)[CTX:end]), l
    # ---- request B (table row 2: the same prefix, other slots past it) restarts from the framework's state ----
    drive(fused, serving, 2, "b", FakeRequest("req-b"), ref_steps, published)
    # ---- request C, sampled, on row 1 again (its slots are overwritten): against a plain sampled iteration ----
    seed, temp, top_k, top_p = 0x0123456789ABCDEF, 0.8, 50, 0.9
    _, _, sampled_steps = plain_run(case, w0, serving.draft_ctx, sampling=sampling_words(seed, CTX, temp, top_k, top_p))
    assert sampled_steps != ref_steps
    req_c = FakeRequest("req-c", temperature=temp, top_k=top_k, top_p=top_p, seed=seed)
    seq, bonus = CTX, torch.tensor([BONUS], device=DEV)
    for i, (toks, commit, ref_bonus, ref_p) in enumerate(sampled_steps):
        batch = decode_batch([req_c], shim.DraftInput(bonus_tokens=bonus), seq_lens=torch.tensor([seq], device=DEV),
                             req_pool_indices=torch.tensor([1], device=DEV))  # fmt: skip
        assert fused.mode(batch, needs_logits=True) == "sample"
        out = fused(batch, needs_logits=True, on_publish=None)
        torch.cuda.synchronize()
        assert fused.statuses() == []
        n = int(out.accept_lens[0])
        assert (n, out.next_token_ids[:n].tolist(), int(out.next_draft_input.bonus_tokens[0]), int(out.new_seq_lens[0])) == (
            commit, toks, ref_bonus, ref_p), i  # fmt: skip
        seq, bonus = ref_p, out.next_draft_input.bonus_tokens
    # the plain verify step still runs on the same bound stack (SGLang's own DFlash step calls it between fused runs)
    ids = torch.randint(0, CFG.vocab, (ROWS,), generator=gen).to(DEV)
    fb = shim.ForwardBatch(shim.ForwardMode("target_verify"), 1, torch.tensor([CTX], device=DEV), torch.tensor([1], device=DEV),
                           serving.slots[1][CTX : CTX + ROWS].to(DEV))  # fmt: skip
    step = verify.plan(ids, fb, view=serving.view)
    out = verify.forward(step, None, ids, torch.arange(CTX, CTX + ROWS, device=DEV), fb)
    torch.cuda.synchronize()
    assert out.next_token_logits.shape == (ROWS, CFG.vocab) and out.hidden_states.shape == (ROWS, 5 * CFG.hidden)
    assert verify.stack.statuses() == []
    shim.install()


def test_simulated_acceptance_forces_the_commit_lengths(monkeypatch):
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_LEN", "2.5")
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_METHOD", "match-expected")
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_TOKEN_MODE", "fixed")
    gen = torch.Generator().manual_seed(22)
    case = synthetic.stack_case(CFG, n_layers=4, rows=ROWS, ctx=CTX, seed=9)
    dw = dsyn.draft_weights(DCFG, 4)
    serving = Serving(case, gen)
    verify = built(case, dw)
    shim.install(fixed_token_id=9)
    verify.prepare(serving.view)
    fused = verify.dflash_iteration(block_size=ROWS, draft_model=serving.draft_model, draft_kv_pool=serving.draft_pool)
    assert not fused.sample and set(fused.graphs) == {"greedy"} and fused.fixed == 9
    table = IT.simulated_accepts(ROWS)
    seq, bonus = CTX, torch.tensor([BONUS], device=DEV)
    req = FakeRequest("req-s")
    for i in range(STEPS):
        batch = decode_batch([req], shim.DraftInput(bonus_tokens=bonus), seq_lens=torch.tensor([seq], device=DEV),
                             req_pool_indices=torch.tensor([1], device=DEV))  # fmt: skip
        out = fused(batch, needs_logits=False, on_publish=None)
        torch.cuda.synchronize()
        assert fused.statuses() == []
        commit = int(table[i]) + 1
        assert int(out.accept_lens[0]) == commit and int(out.new_seq_lens[0]) == seq + commit
        assert out.next_token_ids.tolist() == [9] * ROWS and int(out.next_draft_input.bonus_tokens[0]) == 9
        seq, bonus = seq + commit, out.next_draft_input.bonus_tokens
    # a sampled request is SGLang's under simulated acceptance
    sampled = decode_batch([FakeRequest("req-t", temperature=0.7, top_k=40)], shim.DraftInput(bonus_tokens=bonus),
                           seq_lens=torch.tensor([seq], device=DEV), req_pool_indices=torch.tensor([1], device=DEV))  # fmt: skip
    assert fused(sampled, needs_logits=True, on_publish=None) is None
    shim.install()


def test_token_tree_iteration_on_scattered_slots(monkeypatch):
    """``SGLANG_MUSE_MEGA_TREE=1``: the fused iteration verifies a token tree. With a simulated acceptance (here: the forced
    leaf rows) the accepted paths move K / V and captured rows; tokens, commits, bonus tokens and lengths of every step, and
    the target's K / V rows in the framework's scattered slots, equal a plain tree iteration's on identity slots. A sampled
    request is not the tree's (SGLang's step serves it), and the plain verify step on the tree-bound stack sees a chain."""
    monkeypatch.setenv(B.TREE_ENV, "1")
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_LEN", "6")
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_METHOD", "match-expected")
    gen = torch.Generator().manual_seed(23)
    case = synthetic.stack_case(CFG, n_layers=4, rows=ROWS, ctx=CTX, seed=9)
    dw, dt = dsyn.draft_weights(DCFG, 4), dsyn.target_shared(DCFG, 4)
    w0, _ = shard(DCFG, dw, dt, 0, 1)
    serving = Serving(case, gen)
    verify = built(case, dw)
    assert verify.tree and "token tree" in verify.summary()
    table = IT.simulated_accepts(ROWS)
    assert table is not None
    ref_st, ref_it, ref_steps = plain_run(case, w0, serving.draft_ctx, tree=True, accept_override=table.to(DEV))
    assert ref_it.tree_walk is not None and len({c for _, c, _, _ in ref_steps}) > 1  # commits of several lengths
    verify.prepare(serving.view)
    st = verify.stack
    assert st.tree_table is not None and st.accept is not None and st.accept_sampled is None
    fused = verify.dflash_iteration(block_size=ROWS, draft_model=serving.draft_model, draft_kv_pool=serving.draft_pool)
    assert not fused.sample and set(fused.graphs) == {"greedy"} and fused.it.tree_walk is not None
    published = []
    end = drive(fused, serving, 1, "t", FakeRequest("req-t"), ref_steps, published)
    kvh = CFG.kv_heads_rank
    slots = serving.slots[1]
    for j, lc in enumerate(case.layers):
        where = slots[CTX:end] if lc.global_attn else serving.full_to_swa[slots[CTX:end]]
        got = serving.pool.get_key_buffer(j).view(-1, kvh * 64)[where.to(DEV)]
        assert torch.equal(got, ref_st.pools[j][0][CTX:end]), j
    sampled = FakeRequest("req-u", temperature=0.8, top_k=50, top_p=0.9, seed=1)
    batch = decode_batch([sampled], shim.DraftInput(bonus_tokens=torch.tensor([BONUS], device=DEV)),
                         seq_lens=torch.tensor([CTX], device=DEV), req_pool_indices=torch.tensor([2], device=DEV))  # fmt: skip
    assert fused.mode(batch, needs_logits=True) is None
    # SGLang's own verify step on the tree-bound stack: a chain window gives what a chain-bound stack gives
    ids = torch.randint(0, CFG.vocab, (ROWS,), generator=gen).to(DEV)
    fb = shim.ForwardBatch(shim.ForwardMode("target_verify"), 1, torch.tensor([CTX], device=DEV), torch.tensor([1], device=DEV),
                           serving.slots[1][CTX : CTX + ROWS].to(DEV))  # fmt: skip
    step = verify.plan(ids, fb, view=serving.view)
    out = verify.forward(step, None, ids, torch.arange(CTX, CTX + ROWS, device=DEV), fb)
    torch.cuda.synchronize()
    assert verify.stack.statuses() == []
    chain = S.Stack(case, 0, DEV, greedy=False)
    chain.bind()
    chain.tokens.copy_(ids)
    chain.launch_all(torch.cuda.current_stream().cuda_stream, pdl=False, feeds=True)
    torch.cuda.synchronize()
    assert torch.equal(out.next_token_logits, chain.logits_out)
    shim.install()
