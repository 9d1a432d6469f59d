"""The SGLang-facing executor on the GPU: ``build`` on a stand-in model and ``Verify.forward`` on a stand-in KV pool whose
slots are scattered (request table and full -> sliding-window map are not the identity). The logits must equal, bit for
bit, the same model run by a plain ``Stack`` with identity slots: same kernels, same values, only the addressing
differs; and the window's K / V rows must land in the slots the batch names."""

import pytest
import torch

from fake_sglang import experts_of, fake_model
from sgl_muse_mega_b200.muse_spark.b200 import stack as S
from sgl_muse_mega_b200.muse_spark.b200 import synthetic
from sgl_muse_mega_b200.muse_spark.config import Config
from sgl_muse_mega_b200.muse_spark.runtime import build as B
from sgl_muse_mega_b200.muse_spark.runtime import executor as X
from sgl_muse_mega_b200.muse_spark.runtime import shim

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def test_verify_forward_on_scattered_slots_equals_the_identity_stack():
    cfg = Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7,
                 vocab=4096, layers=4, bf16_moe_layers=(0,), tp=1, node_ranks=1)  # fmt: skip
    rows, ctx = 16, 40
    case = synthetic.stack_case(cfg, n_layers=4, rows=rows, ctx=ctx, seed=8)
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab, (rows,), generator=gen)
    # ---- the plain stack, identity slots, soft-capped logits ----
    ref = S.Stack(case, 0, DEV, greedy=False)
    ref.bind()
    s = torch.cuda.current_stream().cuda_stream
    ref.tokens.copy_(ids)
    ref.launch_all(s, pdl=False, feeds=True)
    torch.cuda.synchronize()
    # ---- the serving side: scattered slots, a request table with two requests, a swa map that is not the identity ----
    slots_full, slots_swa, width = 512, 384, 128
    perm_full = torch.randperm(slots_full, generator=gen)
    perm_swa = torch.randperm(slots_swa, generator=gen)
    pos_to_full = perm_full[: ctx + rows]  # position p of the request lives in full-pool slot pos_to_full[p]
    full_to_swa = torch.full((slots_full + 1,), -1, dtype=torch.int64)
    full_to_swa[pos_to_full] = perm_swa[: ctx + rows]
    r2t = torch.zeros(2, width, dtype=torch.int32)
    r2t[1, : ctx + rows] = pos_to_full.int()
    kvh = cfg.kv_heads_rank
    k_bufs, v_bufs = [], []
    for j, lc in enumerate(case.layers):
        n = slots_full if lc.global_attn else slots_swa
        k, v = (torch.zeros(n, kvh, 64, dtype=torch.bfloat16) for _ in range(2))
        where = pos_to_full[:ctx] if lc.global_attn else full_to_swa[pos_to_full[:ctx]]
        k[where], v[where] = lc.ranks[0].k_ctx, lc.ranks[0].v_ctx
        k_bufs.append(k.to(DEV)), v_bufs.append(v.to(DEV))
    pool = shim.KVPool(k_bufs, v_bufs, full_to_swa.to(DEV))
    view = type("View", (), {})()
    view.kv_pool, view.req_to_token_pool = pool, shim.ReqToTokenPool(r2t.to(DEV))
    # ---- build and step ----
    shim.install()
    shim.install(capture_mode=True, tp_group=shim.Parallel(0, 1))
    model = fake_model(case, device=DEV)
    model.model.language_model.layers_to_capture = [2, 4]  # the inputs of layers 2 and 4 = the outputs of layers 1 and 3
    assert B.alias_reasons(model, cfg, 0) == []
    verify = B.build(model, None, shim.Context(rows), parallel=shim.Parallel(0, 1), experts=experts_of(case, device=DEV), cfg=cfg)
    assert isinstance(verify, X.Verify) and verify.widths == (rows,) and "block 16" in verify.summary()
    fb = shim.ForwardBatch(shim.ForwardMode("target_verify"), 1, torch.tensor([ctx], device=DEV),
                           torch.tensor([1], device=DEV), pos_to_full[ctx:].to(DEV))  # fmt: skip
    positions = torch.arange(ctx, ctx + rows, device=DEV)
    step = verify.plan(ids.to(DEV), fb, view=view)
    assert step is not None
    out = verify.forward(step, None, ids.to(DEV), positions, fb)
    torch.cuda.synchronize()
    assert verify.stack.statuses() == []
    assert torch.equal(out.next_token_logits, ref.logits_out)
    # hidden_states: the capture layers' output residuals in capture order, bf16 (what the draft's fc reads)
    want = torch.cat([ref.layers[c].o["stream_out"].to(torch.bfloat16) for c in (1, 3)], 1)
    assert out.hidden_states.shape == (rows, 2 * cfg.hidden) and torch.equal(out.hidden_states, want)
    verify.check_status()  # clean: nothing raised
    # the window's rows landed where the batch said: layer 1 is global (full pool), layer 2 sliding-window (swa pool)
    for j, lc in enumerate(case.layers):
        where = pos_to_full[ctx:] if lc.global_attn else full_to_swa[pos_to_full[ctx:]]
        got = pool.get_key_buffer(j).view(-1, kvh * 64)[where.to(DEV)]
        assert torch.equal(got, ref.pools[j][0][ctx : ctx + rows]), j
    # a second step on the same bound stack (the pools have not moved) gives the same logits again
    out2 = verify.forward(step, None, ids.to(DEV), positions, fb)
    torch.cuda.synchronize()
    assert torch.equal(out2.next_token_logits, ref.logits_out)
    # pools that moved are refused
    pool.k[0] = pool.k[0].clone()
    with pytest.raises(RuntimeError, match="KV pools moved"):
        verify.forward(step, None, ids.to(DEV), positions, fb)
