"""The SGLang-facing surface without a GPU: plugin registration and the spec's lookups (as the reference's
test/unit/test_plugin.py), the refusal hooks, the tensors the build aliases, the expert reader's sharding and scale
folding, and the executor's plan()."""

from types import SimpleNamespace as NS

import pytest
import torch

from fake_sglang import FakeCheckpoint, experts_of, fake_model
from sgl_muse_mega_b200 import plugin, sglang_api
from sgl_muse_mega_b200.muse_spark import spec as SP
from sgl_muse_mega_b200.muse_spark.b200 import synthetic
from sgl_muse_mega_b200.muse_spark.config import Config
from sgl_muse_mega_b200.muse_spark.runtime import build as B
from sgl_muse_mega_b200.muse_spark.runtime import executor as X
from sgl_muse_mega_b200.muse_spark.runtime import shim


def small_cfg(tp: int) -> Config:
    return Config(hidden=1024, q_heads=64, kv_heads=8, experts=16, topk=8, moe_hidden=1024, moe_inter=1024, swa_window=7,
                  vocab=4096, layers=3, bf16_moe_layers=(0,), tp=tp, node_ranks=min(4, tp))  # fmt: skip


@pytest.fixture(scope="module")
def case1():
    return synthetic.stack_case(small_cfg(1), n_layers=3, rows=16, ctx=8, seed=2)


def test_plugin_registers_the_spec_under_the_architecture():
    plugin.register()
    assert sglang_api.ENTRY_POINT == "nvidia_megakernel" and sglang_api.MEGAKERNEL_API_VERSION == 1
    found, why = sglang_api.find_spec(architectures=["MuseSparkForConditionalGeneration"], isa="sm_100")
    assert found is SP.SPEC and why is None
    found, why = sglang_api.find_spec(architectures=["MuseSparkForConditionalGeneration"], isa="sm_103")
    assert found is None and "sm_100" in why  # not this build's isa
    found, why = sglang_api.find_spec(architectures=["LlamaForCausalLM"], isa="sm_100")
    assert found is None and "no megakernel spec" in why
    r = SP.SPEC.requires
    assert r.isas == frozenset({"sm_100"}) and r.tp_sizes == frozenset({1, 2, 4, 8}) and r.resident_blocks == 148
    assert SP.SPEC.max_rows == 16 and SP.SPEC.api_version == 1


def test_alias_reasons_accept_the_model_and_name_what_is_wrong(case1):
    cfg = case1.cfg
    model = fake_model(case1)
    assert B.alias_reasons(model, cfg, 0) == []
    specs = B.alias_specs(model, cfg)
    assert specs[(1, "cross_pre_w")][0] is model.model.language_model.layers[2].input_layernorm._frozen_weight
    assert specs[(2, "cross_pre_w")][0] is model.model.language_model.norm._frozen_weight
    assert (2, "next_qkv") not in specs and specs[(0, "next_qkv")][0] is model.model.language_model.layers[1].self_attn.qkv_proj.weight
    # a wrong shape and a wrong dtype are named with their layer
    lm = model.model.language_model
    lm.layers[1].mlp.gate.weight = lm.layers[1].mlp.gate.weight.bfloat16()
    lm.layers[2].self_attn.o_proj.weight = lm.layers[2].self_attn.o_proj.weight[:, :-64]
    reasons = B.alias_reasons(model, cfg, 0)
    assert any(r.startswith("layer 1 router is") and "bfloat16" in r for r in reasons)
    assert any(r.startswith("layer 2 o_proj is") for r in reasons) and len(reasons) == 2
    # a model without the expected modules is one reason, not an exception
    del lm.layers[0].mlp.pre_expert_proj
    assert B.alias_reasons(model, cfg, 0)[0].startswith("the loaded model lacks a tensor the kernels read")


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_model_disable_reasons_use_the_serving_world(tp):
    """The spec's model hook checks every rank's tensors against the per-rank shapes of the SERVING world (its TP degree
    and this process's rank in it): a valid full-width model of any supported world passes on every rank, and all ranks
    reach the same verdict. The tensors here are zero-stride views of the right shapes (the hook reads shapes, dtypes
    and the vocab shard's first row only)."""
    from sgl_muse_mega_b200.muse_spark.config import Config as C

    cfg = C().with_tp(tp)
    for rank in sorted({0, tp - 1}):
        shim.install()
        shim.install(tp_group=shim.Parallel(rank, tp))
        model = shaped_model(cfg, rank)
        assert SP.model_disable_reasons(model, None) == [], (tp, rank)
    # a model sharded for another world is refused, with the offending tensors named
    shim.install(tp_group=shim.Parallel(0, tp))
    other = shaped_model(C().with_tp(8 if tp != 8 else 4), 0)
    assert any("qkv0 is" in r for r in SP.model_disable_reasons(other, None))
    shim.install()


def shaped_model(cfg, rank: int):
    """A model whose tensors have the per-rank shapes of ``cfg`` without their memory (expanded scalars made 'contiguous'
    is impossible, so each tensor is an empty meta tensor: shape, dtype and contiguity are all the hook reads)."""
    bf, f32 = torch.bfloat16, torch.float32
    m = lambda shape, dt=bf: torch.empty(shape, dtype=dt, device="meta")  # noqa: E731
    h, mh = cfg.hidden, cfg.moe_hidden
    norm = lambda n: NS(_frozen_weight=m((n,)))  # noqa: E731
    layers = []
    for _ in range(cfg.layers):
        layers.append(NS(
            input_layernorm=norm(h),
            self_attn=NS(qkv_proj=NS(weight=m((cfg.qkv_row, h))), o_proj=NS(weight=m((h, cfg.oproj_k))),
                         rotary_emb=NS(cos_sin_cache=m((64, cfg.head_dim), f32))),
            mlp=NS(pre_expert_proj=NS(weight=m((mh, h))), post_expert_proj=NS(weight=m((h, mh))),
                   gate=NS(weight=m((cfg.experts, h), f32), e_score_correction_bias=m((cfg.experts,), f32)),
                   pre_expert_norm=norm(mh), experts=NS(post_expert_norm=norm(mh))),
            post_attention_residual_gate=NS(_alpha=m((h,), f32), _beta=m((h,), f32)),
            post_feedforward_residual_gate=NS(_alpha=m((h,), f32), _beta=m((h,), f32)),
            pre_feedforward_layernorm=norm(h), post_feedforward_layernorm=norm(h),
        ))  # fmt: skip
    shard = NS(org_vocab_start_index=rank * cfg.vocab_rank)
    lm = NS(layers=layers, norm=norm(h), embed_tokens=NS(weight=m((cfg.vocab_rank, h)), shard_indices=shard))
    return NS(model=NS(language_model=lm), lm_head=NS(weight=m((cfg.vocab_rank, h)), shard_indices=shard))


def test_vocab_shard_must_be_this_ranks_rows():
    cfg = small_cfg(2)
    case = synthetic.stack_case(cfg, n_layers=3, rows=16, ctx=8, seed=2, only_ranks=[1])
    model = fake_model(case)
    assert B.alias_reasons(model, cfg, 1) == []
    assert any("shard starts at row" in r for r in B.alias_reasons(model, cfg, 0))


def test_layer_experts_shards_the_checkpoint_and_folds_the_scales():
    """A two-rank world's plain shards are stitched into checkpoint-shaped tensors [E, 2 I, ...] / [E, P, ...]; the reader
    must hand each rank its own shard back, with g1_alphas = s2_gate, g1_scale_c = s2_up / s2_gate, g2_alphas = s2_down."""
    cfg = small_cfg(2)
    lc = synthetic.layer_case(cfg, rows=4, ctx=4, seed=9, layer=1, band="reference")
    a, b = lc.ranks
    p = "model.language_model.layers.1.mlp.experts."
    cat = lambda x, y: torch.cat([x, y], 1)  # noqa: E731
    s2 = torch.stack([a.g1_alphas, a.g1_alphas * a.g1_scale_c], 1)
    ck = FakeCheckpoint({
        p + "gate_up_proj": torch.cat([cat(a.gate_q, b.gate_q), cat(a.up_q, b.up_q)], 1),
        p + "gate_up_proj_weight_scale": torch.cat([cat(a.gate_sf, b.gate_sf), cat(a.up_sf, b.up_sf)], 1),
        p + "down_proj": cat(a.w2_q, b.w2_q),
        p + "down_proj_weight_scale": cat(a.w2_sf, b.w2_sf),
        p + "gate_up_proj_weight_scale_2": s2,
        p + "down_proj_weight_scale_2": a.g2_alphas,
    })  # fmt: skip
    for rank, t in enumerate((a, b)):
        got = B.layer_experts(ck, cfg, 1, rank, "cpu")
        for k in ("gate_q", "gate_sf", "up_q", "up_sf", "w2_q", "w2_sf", "g1_alphas", "g2_alphas"):
            assert torch.equal(got[k], getattr(t, k)), (rank, k)
        assert torch.allclose(got["g1_scale_c"], t.g1_scale_c, rtol=1e-6)


def test_model_case_aliases_the_models_tensors(case1):
    cfg = case1.cfg
    model = fake_model(case1)
    mc = B.model_case(model, cfg, 0, "cpu", 16, experts_of(case1))
    assert len(mc.layers) == 3 and mc.ctx == 0 and mc.ranks == [0]
    l1 = mc.layers[1]
    assert (l1.global_attn, l1.bf16, l1.tail, l1.next_global) == (True, False, False, False)
    t = l1.ranks[0]
    assert t.pooler.data_ptr() == model.model.language_model.layers[1].mlp.pre_expert_proj.weight.data_ptr()
    assert t.next_qkv.data_ptr() == model.model.language_model.layers[2].self_attn.qkv_proj.weight.data_ptr()
    assert torch.equal(t.gate_q, case1.layers[1].ranks[0].gate_q)
    assert mc.layers[2].tail and mc.layers[2].ranks[0].next_qkv is None and mc.layers[0].bf16


def test_plan_takes_only_the_batch_1_verify_step_of_one_block(case1):
    shim.install()
    shim.install(capture_mode=True)
    v = X.Verify(case1.cfg, 16, case1, None, None, None, None, 0, "cpu", None, "test build")
    assert v.widths == (16,) and v.summary() == "test build" and v.draft_sampler is None
    fb = lambda mode, bs: shim.ForwardBatch(shim.ForwardMode(mode), bs, torch.tensor([40]), torch.tensor([0]), torch.arange(16))  # noqa: E731
    ids = torch.zeros(16, dtype=torch.int64)
    step = v.plan(ids, fb("target_verify", 1), view=NS())
    assert step is not None and (step.mode, step.rows) == ("target_verify", 16)
    assert v.plan(None, fb("target_verify", 1)) is None  # a forward without ids
    assert v.plan(ids, fb("decode", 1)) is None
    assert v.plan(ids, fb("target_verify", 2)) is None
    assert v.plan(ids[:8], fb("target_verify", 1)) is None
    shim.install(capture_mode=False)  # outside SGLang's decode-graph capture the step is SGLang's own
    assert v.plan(ids, fb("target_verify", 1), view=NS()) is None
    shim.install()
    with pytest.raises(RuntimeError, match="plan"):
        v.forward(None, None, ids, None, fb("target_verify", 1))


# ---- the DFlash2 draft's spec and the fused iteration's host side ----------------------------------------------------------------


def test_plugin_registers_the_draft_spec_too():
    from sgl_muse_mega_b200.muse_spark import draft as DS

    plugin.register()
    found, why = sglang_api.find_spec(architectures=["DFlash2DraftModel"], isa="sm_100")
    assert found is DS.SPEC and why is None
    assert DS.SPEC.max_rows == 0 and DS.Draft().widths == () and DS.SPEC.requires.tp_sizes == frozenset({1, 2, 4, 8})


def test_draft_spec_refuses_other_drafts_and_a_missing_target(monkeypatch):
    from fake_sglang import draft_hf_config
    from sgl_muse_mega_b200.muse_spark import draft as DS
    from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig

    hf = lambda d: NS(to_dict=lambda: d)  # noqa: E731
    good = draft_hf_config(DraftConfig())
    assert DraftConfig.from_hf(good) == DraftConfig()
    monkeypatch.setattr(B, "TARGET", object())
    assert DS.model_disable_reasons(None, hf(good)) == []
    monkeypatch.setattr(B, "TARGET", None)
    assert DS.model_disable_reasons(None, hf(good)) == ["the target's megakernel is not built in this process"]
    monkeypatch.setattr(B, "TARGET", object())
    other = dict(good, num_hidden_layers=good["num_hidden_layers"] + 1, layer_types=good["layer_types"] + ["sliding_attention"])
    assert any(r.startswith("layers ") for r in DS.model_disable_reasons(None, hf(other)))
    causal = dict(good, is_causal=True)
    assert "a causal or non-sliding layer" in DS.model_disable_reasons(None, hf(causal))[0]
    assert "KeyError" in DS.model_disable_reasons(None, hf({"architectures": ["DFlash2DraftModel"]}))[0]
    with pytest.raises(RuntimeError, match="not built"):
        monkeypatch.setattr(B, "TARGET", None)
        DS.build(None, hf(good), None)


@pytest.mark.parametrize("ranks", [1, 2])
def test_draft_build_reads_this_ranks_shard_onto_the_target(monkeypatch, ranks):
    from fake_sglang import draft_checkpoint, draft_hf_config
    from sgl_muse_mega_b200.muse_spark import draft as DS
    from sgl_muse_mega_b200.muse_spark.b200.dflash import synthetic as dsyn
    from sgl_muse_mega_b200.muse_spark.b200.dflash.weights import DraftConfig, load_shard, shard

    dcfg = DraftConfig(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=64, inter=256, vocab=512, sliding_window=24,
                       mask_id=500, selector_rank=16, top_k=8, capture=(0, 1))  # fmt: skip
    w, t = dsyn.draft_weights(dcfg, 3), dsyn.target_shared(dcfg, 3)
    entries = draft_checkpoint(dcfg, w)
    read = lambda names: {n: entries[n] for n in names}  # noqa: E731
    for rank in range(ranks):
        target = NS(draft=None, draft_cfg=None, device="cpu")
        monkeypatch.setattr(B, "TARGET", target)
        shim.install()
        shim.install(tp_group=shim.Parallel(rank, ranks))
        built = DS.build(None, NS(to_dict=lambda: draft_hf_config(dcfg)), None, read=read, cfg=dcfg)
        assert built.widths == () and target.draft_cfg is dcfg
        want, _ = shard(dcfg, w, t, rank, ranks)
        assert torch.equal(target.draft.fc, want.fc) and torch.equal(target.draft.pred_codebook, w.pred_codebook)
        for got, ref in zip(target.draft.layers, want.layers):
            for name in ("input_norm", "post_norm", "q_norm", "k_norm", "qkv", "o", "gate_up", "down"):
                assert torch.equal(getattr(got, name), getattr(ref, name)), name
            assert torch.equal(got.attn_conv.base, ref.attn_conv.base) and torch.equal(got.mlp_conv.proj, ref.mlp_conv.proj)
    shim.install()
    with pytest.raises(ValueError, match="not bfloat16"):
        load_shard(lambda names: {n: entries[n].float() for n in names}, 0, 1, dcfg)


def test_simulated_accepts_meet_the_expected_length(monkeypatch):
    from sgl_muse_mega_b200.muse_spark.runtime import iteration as IT

    monkeypatch.delenv("SGLANG_SIMULATE_ACC_LEN", raising=False)
    assert IT.simulated_accepts(16) is None and IT.fixed_token() is None
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_LEN", "3.3")
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_METHOD", "match-expected")
    t = IT.simulated_accepts(16)
    assert t.dtype == torch.int32 and t.shape == (IT.SIMULATED_STEPS,) and set(t.tolist()) == {2, 3}
    commits = (t + 1).double()
    assert abs(float(commits.mean()) - 3.3) < 1e-2
    # any run of consecutive steps stays within a few commits of the expected total
    run = commits.cumsum(0)
    for lo in (0, 100, 1777):
        for n in (10, 64, 500):
            assert abs(float(run[lo + n] - run[lo]) - 3.3 * n) < 2.0, (lo, n)
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_METHOD", "multinomial")
    m = IT.simulated_accepts(16) + 1
    assert int(m.min()) >= 1 and int(m.max()) <= 16 and abs(float(m.double().mean()) - 3.3) < 0.1
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_LEN", "40")
    assert set(IT.simulated_accepts(16).tolist()) == {15}  # clamped to the block
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_METHOD", "other")
    with pytest.raises(ValueError, match="simulate_acc_method"):
        IT.simulated_accepts(16)
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_METHOD", "multinomial")
    monkeypatch.setenv("SGLANG_SIMULATE_ACC_TOKEN_MODE", "fixed")
    shim.install(fixed_token_id=7)
    assert IT.fixed_token() == 7
    shim.install()


def test_fused_mode_takes_only_the_steps_its_graphs_serve():
    from fake_sglang import FakeRequest, decode_batch, plain_sampling_info
    from sgl_muse_mega_b200.muse_spark.runtime import iteration as IT

    f = IT.Fused.__new__(IT.Fused)  # mode() reads only ``sample``
    f.sample = True
    spec = shim.DraftInput(bonus_tokens=torch.tensor([5]))
    greedy, sampled = FakeRequest("a"), FakeRequest("b", temperature=0.7, top_k=40, top_p=0.9)
    assert f.mode(decode_batch([greedy], spec), needs_logits=False) == "greedy"
    assert f.mode(decode_batch([greedy], spec), needs_logits=True) is None  # logprobs and the like read the logits
    assert f.mode(decode_batch([greedy], spec, sampling_info=None), needs_logits=False) == "greedy"
    assert f.mode(decode_batch([sampled], spec), needs_logits=True) == "sample"
    assert f.mode(decode_batch([greedy, sampled], spec), needs_logits=False) is None
    assert f.mode(decode_batch([greedy], spec, mode="extend"), needs_logits=False) is None
    assert f.mode(decode_batch([greedy], spec, mode="idle"), needs_logits=False) is None
    assert f.mode(decode_batch([greedy], spec, is_extend_in_batch=True), needs_logits=False) is None
    assert f.mode(decode_batch([greedy], object()), needs_logits=False) is None  # not the DFlash2 draft's input
    for edit in (dict(need_min_p_sampling=True), dict(has_custom_logit_processor=True), dict(grammar_mask=torch.ones(1)),
                 dict(logit_bias=torch.ones(1)), dict(sampling_mask_batch_indices=torch.ones(1)),
                 dict(penalizer_orchestrator=NS(is_required=True))):  # fmt: skip
        assert f.mode(decode_batch([sampled], spec, sampling_info=plain_sampling_info(**edit)), needs_logits=True) is None, edit
    assert f.mode(decode_batch([sampled], spec, sampling_info=plain_sampling_info(penalizer_orchestrator=NS(is_required=False))),
                  needs_logits=True) == "sample"  # fmt: skip
    assert f.mode(decode_batch([sampled], spec, has_grammar=True), needs_logits=True) is None
    assert f.mode(decode_batch([sampled], spec, return_logprob=True), needs_logits=True) is None
    f.sample = False  # a simulated accept length: sampled steps are SGLang's
    assert f.mode(decode_batch([sampled], spec), needs_logits=True) is None


def test_token_tree_is_opt_in_by_environment(monkeypatch):
    """``SGLANG_MUSE_MEGA_TREE=1`` (the reference's switch, runtime/build.py:94-100) turns the fused iteration's window into
    a token tree; a tree-bound stack gives SGLang's own verify step (a chain) the chain's table."""
    from sgl_muse_mega_b200.muse_spark.runtime import build as B

    monkeypatch.delenv(B.TREE_ENV, raising=False)
    assert not B.tree_enabled()
    monkeypatch.setenv(B.TREE_ENV, "0")
    assert not B.tree_enabled()
    monkeypatch.setenv(B.TREE_ENV, "1")
    assert B.tree_enabled()
    # the chain as a tree table: parent r - 1, depth r, ancestors = every earlier row (what Verify.forward writes)
    r = torch.arange(16, dtype=torch.int32)
    mask = ((2 << r) - 1).tolist()
    assert mask[0] == 1 and mask[15] == 0xFFFF and all(m == (1 << (i + 1)) - 1 for i, m in enumerate(mask))


def test_request_seed_is_the_same_on_every_rank():
    from fake_sglang import FakeRequest
    from sgl_muse_mega_b200.muse_spark.runtime import iteration as IT

    assert IT.request_seed(FakeRequest("r", seed=12345)) == 12345
    assert IT.request_seed(FakeRequest("r", seed=2**64 - 1)) == -1  # wrapped into a signed 64-bit word
    a, b = IT.request_seed(FakeRequest("req-1")), IT.request_seed(FakeRequest("req-1"))
    assert a == b and -(2**63) <= a < 2**63 and a != IT.request_seed(FakeRequest("req-2"))


def test_hooks_wrap_the_worker_and_fall_back_to_its_own_step(monkeypatch):
    import sys
    import types

    from sgl_muse_mega_b200.muse_spark.runtime import iteration as IT

    calls = []

    class Worker:
        def __init__(self, model):
            self.target_worker = NS(model_runner=NS(model=model))
            self.draft_model, self.draft_model_runner = "draft", NS(token_to_kv_pool="pool")

        def init_cuda_graphs(self):
            calls.append("graphs")
            return "ok"

        def forward_batch_generation(self, batch, on_publish=None):
            calls.append(("own", batch))
            return "own step"

        def _can_skip_verify_logits(self, batch, info):
            return True

    mod = types.ModuleType("sglang.srt.speculative.dflash_worker_v2")
    mod.DFlashWorkerV2 = Worker
    for name in ("sglang", "sglang.srt", "sglang.srt.speculative"):
        monkeypatch.setitem(sys.modules, name, types.ModuleType(name))
    monkeypatch.setitem(sys.modules, "sglang.srt.speculative.dflash_worker_v2", mod)
    IT.install()

    class Target(X.Verify):
        def __init__(self):
            self.block, self.fused = 16, None

        def dflash_iteration(self, *, block_size, draft_model, draft_kv_pool):
            calls.append(("bind", block_size, draft_model, draft_kv_pool))
            return lambda batch, needs_logits, on_publish: None if batch.kind == "prefill" else f"fused {batch.kind} {needs_logits}"

    w = Worker(NS(built_megakernel=Target()))
    assert w.init_cuda_graphs() == "ok" and calls == ["graphs", ("bind", 16, "draft", "pool")]
    decode, prefill = NS(kind="decode", sampling_info=None), NS(kind="prefill", sampling_info=None)
    assert w.forward_batch_generation(decode) == "fused decode False"
    assert w.forward_batch_generation(prefill) == "own step" and calls[-1] == ("own", prefill)
    # a worker whose target model has no megakernel build keeps its own step
    plain = Worker(NS())
    assert plain.init_cuda_graphs() == "ok" and plain.forward_batch_generation(decode) == "own step"
