"""The fused decode iteration (draft launches, then the target's verify step and greedy accept) on one rank: what one half
hands the other stays on the device and arrives where the other half reads it."""

import pytest
import torch

from oracle import dflash_accept as A
from oracle import dflash_draft as D
from sgl_muse_mega_b200.muse_spark.b200 import headtail as HT
from sgl_muse_mega_b200.muse_spark.b200 import stack as S
from sgl_muse_mega_b200.muse_spark.b200 import synthetic
from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic as dsyn
from sgl_muse_mega_b200.muse_spark.b200.dflash.iteration import Iteration
from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig, shard
from sgl_muse_mega_b200.muse_spark.config import Config

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
BF = torch.bfloat16

CFG = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7, vocab=4096,
             layers=4, bf16_moe_layers=(0,), tp=1, node_ranks=1)  # fmt: skip
DCFG = DraftConfig(hidden=1024, layers=2, q_heads=8, kv_heads=4, head_dim=128, inter=1024, vocab=4096, sliding_window=24,
                   mask_id=4001, selector_rank=64, top_k=16, capture=(0, 1, 2, 3, 2))  # fmt: skip
ROWS, CTX = 16, 24


def build():
    case = synthetic.stack_case(CFG, n_layers=4, rows=ROWS, ctx=CTX, seed=9)
    st = S.Stack(case, 0, DEV)
    st.bind()
    dw, dt = dsyn.draft_weights(DCFG, 4), dsyn.target_shared(DCFG, 4)
    w0, _ = shard(DCFG, dw, dt, 0, 1)
    it = Iteration(st, DCFG, w0, capture=list(DCFG.capture), pool_rows=64, rope_rows=128)
    st.feeds.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return case, st, it, w0


def capped(st):
    return torch.tanh((st.gathered.cpu() * CFG.output_multiplier) / CFG.softcap) * CFG.softcap


def test_two_iterations_hand_over_on_the_device():
    case, st, it, w0 = build()
    s = torch.cuda.current_stream().cuda_stream
    dr = it.draft
    assert dr.words.data_ptr() == st.accept.words.data_ptr() and dr.verify_ids.data_ptr() == st.tokens.data_ptr()
    assert it.kernels == dr.kernels() + st.kernels
    # iteration 1: nothing committed yet, the anchor word is 0
    it.launch_all(s, pdl=False)
    torch.cuda.synchronize()
    assert it.statuses() == []
    tokens1 = st.tokens.cpu().clone()
    assert int(tokens1[0]) == 0 and tokens1[1:].tolist() == dr.drafts.cpu().tolist()
    assert int((dr.k_pool[0][:CTX].float().abs().sum())) == 0  # commit 0: no context rows written
    acc1 = A.greedy_accept(tokens1, capped(st), CTX)
    w1 = st.accept.words.cpu().tolist()
    assert w1[:4] == [acc1.new_pos, acc1.bonus, acc1.accept_len, acc1.commit_len]
    caps1 = torch.stack([st.layers[c].o["stream_out"].cpu().clone() for c in it.capture])
    # iteration 2 reads the words and the capture of iteration 1
    it.launch_all(s, pdl=False)
    torch.cuda.synchronize()
    assert it.statuses() == []
    assert torch.equal(dr.feats.cpu(), D.feats_of(caps1))
    tokens2 = st.tokens.cpu()
    assert int(tokens2[0]) == acc1.bonus
    ref = D.context_update(DCFG, [(w0, None)], dr.feats.cpu(), CTX)
    for li in range(DCFG.layers):
        k, v = ref["kv"][0][li]
        got_k, got_v = dr.k_pool[li][CTX : CTX + acc1.commit_len].cpu(), dr.v_pool[li][CTX : CTX + acc1.commit_len].cpu()
        assert float((got_k.float() - k[: acc1.commit_len].float()).norm() / k[: acc1.commit_len].float().norm()) < 1e-2
        assert float((got_v.float() - v[: acc1.commit_len].float()).norm() / v[: acc1.commit_len].float().norm()) < 1e-2
        # the block's own rows sit at the new position
        assert float(dr.k_pool[li][acc1.new_pos : acc1.new_pos + ROWS].float().abs().sum()) > 0
    acc2 = A.greedy_accept(tokens2, capped(st), acc1.new_pos)
    w2 = st.accept.words.cpu().tolist()
    assert w2[:5] == [acc2.new_pos, acc2.bonus, acc2.accept_len, acc2.commit_len, 2]
    # the target's window moved with it
    assert st.feeds.kv_len.item() == acc2.new_pos + ROWS


def test_iteration_replays_as_one_graph():
    case, st, it, w0 = build()
    forced = torch.tensor([3], dtype=torch.int32, device=DEV)
    st2 = S.Stack(case, 0, DEV, accept_override=forced)
    st2.bind()
    it2 = Iteration(st2, DCFG, w0, capture=list(DCFG.capture), pool_rows=64, rope_rows=128)
    st2.feeds.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    it2.capture_graph(warmup=False)
    for i in range(3):
        it2.step()
        torch.cuda.synchronize()
        w = st2.accept.words.cpu().tolist()
        assert w[HT.WORDS["P"]] == CTX + 4 * (i + 1) and w[HT.WORDS["ITER"]] == i + 1 and w[HT.WORDS["COMMIT"]] == 4
        assert int(st2.tokens[0]) == (0 if i == 0 else prev_bonus)
        prev_bonus = w[HT.WORDS["ANCHOR"]]
    assert it2.statuses() == []
    assert st2.accept.out_ring.cpu()[:12].count_nonzero() > 0


def test_eight_row_window_iteration():
    """DFlash block 8 (1 anchor + 7 drafts): the same launch lists with an 8-row window, three graph replays."""
    rows = 8
    case = synthetic.stack_case(CFG, n_layers=4, rows=rows, ctx=CTX, seed=10)
    forced = torch.tensor([2], dtype=torch.int32, device=DEV)
    st = S.Stack(case, 0, DEV, accept_override=forced)
    st.bind()
    dw, dt = dsyn.draft_weights(DCFG, 4), dsyn.target_shared(DCFG, 4)
    w0, _ = shard(DCFG, dw, dt, 0, 1)
    it = Iteration(st, DCFG, w0, capture=list(DCFG.capture), pool_rows=64, rope_rows=128)
    st.feeds.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    it.capture_graph(warmup=False)
    for i in range(3):
        it.step()
        torch.cuda.synchronize()
        w = st.accept.words.cpu().tolist()
        assert w[HT.WORDS["P"]] == CTX + 3 * (i + 1) and w[HT.WORDS["COMMIT"]] == 3 and w[HT.WORDS["ITER"]] == i + 1
        assert st.tokens.shape[0] == rows and it.draft.drafts.shape[0] == rows - 1
        assert st.tokens.cpu()[1:].tolist() == it.draft.drafts.cpu().tolist()
    assert it.statuses() == []


def test_sampled_iteration_matches_the_oracle_on_its_own_tensors():
    """Temperature > 0: the draft head walks by Philox uniforms (purpose 0), the verify ends with the sampled accept
    (purpose 1) over the draft's candidates and walk probabilities; three graph replays, each checked against the oracle
    fed the step's own gathered logits, candidates, probabilities and ids."""
    from oracle import dflash_sample as SM
    from sgl_muse_mega_b200.muse_spark.b200.dflash.draft import sampling_words

    seed, strm, temp, top_k, top_p = 0x1122334455667788, 2, 0.9, 64, 0.95
    case = synthetic.stack_case(CFG, n_layers=4, rows=ROWS, ctx=CTX, seed=11)
    st = S.Stack(case, 0, DEV, sampling=sampling_words(seed, strm, temp, top_k, top_p))
    st.bind()
    dw, dt = dsyn.draft_weights(DCFG, 4), dsyn.target_shared(DCFG, 4)
    w0, _ = shard(DCFG, dw, dt, 0, 1)
    it = Iteration(st, DCFG, w0, capture=list(DCFG.capture), pool_rows=64, rope_rows=128)
    assert it.draft.cand.data_ptr() == st.draft_cand.data_ptr() and it.draft.samp is st.samp
    st.feeds.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    it.capture_graph(warmup=False)
    pos = CTX
    for i in range(3):
        it.step()
        torch.cuda.synchronize()
        assert it.statuses() == []
        tokens, cand, q = st.tokens.cpu(), st.draft_cand.cpu(), st.draft_walk_q.cpu()
        assert tokens[1:].tolist() == it.draft.drafts.cpu().tolist()
        y = capped(st) / torch.tensor(temp, dtype=torch.float32)
        probs = SM.target_probs(y, 1.0, top_k, float(torch.tensor(top_p, dtype=torch.float32)))
        ref = SM.sampled_accept(tokens, probs, cand, q, D.uniforms(seed, strm, i, SM.PURPOSE_ACCEPT), True)
        w = st.accept.words.cpu().tolist()
        pos += ref.accept_len + 1
        assert (w[HT.WORDS["ACCEPT"]], w[HT.WORDS["ANCHOR"]], w[HT.WORDS["P"]], w[HT.WORDS["ITER"]]) == (
            ref.accept_len, ref.bonus, pos, i + 1)  # fmt: skip
