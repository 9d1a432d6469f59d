"""SGLang-facing: the fused DFlash2 iteration inside SGLang's DFlash worker. For a batch-1 decode step one CUDA graph runs
the draft, the target's verify step and the accept (``b200/dflash/iteration.py``) in place of the worker's step and
returns what the worker returns. A greedy request takes the greedy graph, a sampled one (temperature, top-k, top-p) the
sampled graph; every other step (prefill, logprobs, grammar, penalties, logit bias, min-p, custom logit processors,
sampling masks, larger batches) is SGLang's own.

Same surface as the reference's ``muse_spark/runtime/iteration.py:153-462``: ``simulated_accepts`` (the forced-accept
table behind ``SGLANG_SIMULATE_ACC_LEN``), ``Fused`` with ``mode()``, ``__call__(batch, needs_logits=, on_publish=)``,
``step``, graphs per mode and output parity, the request start from SGLang's state, the export in the worker's form, the
flush of a run's last commit into SGLang's draft pool, and ``install()`` with the two worker hooks for an SGLang without
the iteration slot. The arithmetic is the kernels'; this file only moves state between SGLang's objects and the bound
launches. SGLang's classes are imported where they exist and replaced by the stand-ins of ``runtime/shim.py`` otherwise.

How a graph meets SGLang's state: before each replay the request's committed length and slot-table row are copied into the
window feeds' static inputs; inside the graph the window's positions and their slots in both pools are gathered from
SGLang's request table, so the target's K / V rows go to the slots SGLang allocated. The draft keeps its context K / V in
rings of its own; at a request's first fused step (or after a step SGLang ran) the rings are filled from SGLang's draft
pool, which holds the context of every committed position up to then. A committed position's draft K / V reaches the
rings one iteration after its commit; each graph's last launch (``mk_dflash_kv_sync_bind``) copies the rows that arrived
into SGLang's draft pool, and the run's last commit is flushed (the draft alone, then the copy) before any step that is
not the run's next fused one. The token tree of the reference (``SGLANG_MUSE_MEGA_TREE``) is not built here.
"""

from __future__ import annotations

import hashlib
import logging
import math
from typing import Optional

import torch

from ...common import host
from ..b200 import headtail as HT
from ..b200.dflash.draft import sampling_words
from ..b200.dflash.iteration import Iteration
from . import shim
from .executor import WAIT_BUDGET, Verify

try:  # pragma: no cover - only where SGLang is installed
    from sglang.srt.layers.logits_processor import LogitsProcessorOutput  # type: ignore
    from sglang.srt.managers.utils import GenerationBatchResult  # type: ignore
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType  # type: ignore
    from sglang.srt.speculative.dflash_info_v2 import DFlashDraftInputV2 as DraftInput  # type: ignore
    from sglang.srt.speculative.draft_worker_common import make_draft_input_v2  # type: ignore

    AFTER, AROUND = HookType.AFTER, HookType.AROUND
except ImportError:
    from .shim import DraftInput, GenerationBatchResult, HookRegistry, LogitsProcessorOutput

    AFTER, AROUND = "after", "around"

    def make_draft_input_v2(*, bonus_tokens, new_seq_lens):
        return DraftInput(bonus_tokens=bonus_tokens, new_seq_lens=new_seq_lens)


WORKER = "sglang.srt.speculative.dflash_worker_v2.DFlashWorkerV2"
logger = logging.getLogger(__name__)
SIMULATED_STEPS = 4096  # the accept reads its forced-accept table at the iteration word modulo the table's length
RING_ROWS = 4096  # rows of the draft's K / V rings (position modulo this)
WORDS = HT.WORDS


def simulated_accepts(b: int) -> Optional[torch.Tensor]:
    """The forced accepts (commit length - 1, i32 [4096]) behind SGLang's simulated acceptance, or None when it is off. The
    commit lengths follow the distribution SGLang's simulated step draws from, but at the golden-ratio sequence's
    quantiles instead of random draws: any run of consecutive steps meets the expected total within a few commits, and
    every rank computes the same table (reference iteration.py:153-170).
      match-expected   commit = floor(x) + [u < frac(x)],  x = the length clamped to [1, b]
      multinomial      commit = round(length + Phi^-1(u)) clamped to [1, b]"""
    length, method, _ = shim.simulated_acceptance()
    if length <= 0:
        return None
    golden = (math.sqrt(5) - 1) / 2
    u = torch.remainder(0.5 + golden * torch.arange(SIMULATED_STEPS, dtype=torch.float64), 1.0)
    if method == "match-expected":
        x = min(max(length, 1.0), float(b))
        commit = math.floor(x) + (u < x - math.floor(x)).long()
    elif method == "multinomial":
        commit = torch.round(length + torch.special.ndtri(u)).clamp(1, b).long()
    else:
        raise ValueError(f"Invalid simulate_acc_method: {method}")
    return (commit - 1).to(torch.int32)


def fixed_token() -> Optional[int]:
    """The token id SGLang's simulated step commits in its "fixed" token mode, or None (real tokens)."""
    length, _, token_mode = shim.simulated_acceptance()
    if length <= 0 or token_mode != "fixed":
        return None
    try:
        import inspect

        from sglang.srt.speculative.dflash_utils import apply_dflash_simulated_acceptance  # type: ignore

        return int(inspect.signature(apply_dflash_simulated_acceptance).parameters["fixed_token_id"].default)
    except ImportError:
        return int(shim._STANDINS.get("fixed_token_id", 0))


def request_seed(req) -> int:
    """The request's signed 64-bit seed: its ``sampling_seed``, else one derived from its id (the same on every rank)."""
    seed = req.sampling_params.sampling_seed
    if seed is None:
        seed = int.from_bytes(hashlib.sha256(req.rid.encode()).digest()[:8], "little")
    return (seed + 2**63) % 2**64 - 2**63


def plain_sampling(batch) -> bool:
    """A sampled batch the sampled graph serves exactly: nothing that edits the logits (SGLang's step applies those)."""
    info = batch.sampling_info
    pen = info.penalizer_orchestrator
    return not (
        batch.has_grammar or batch.return_logprob or info.need_min_p_sampling or info.has_custom_logit_processor
        or (pen is not None and pen.is_required) or info.grammar_mask is not None or info.logit_bias is not None
        or info.sampling_mask_batch_indices is not None
    )  # fmt: skip


class Fused:
    """One process's fused iteration of the target's block size: the greedy graph, the sampled graph (not with a simulated
    accept length, nor with the token tree, whose accept is the greedy one) and the flush graph, each captured twice (the outputs alternate between two sets so that a step's
    results stay intact while the overlap scheduler launches the next step)."""

    def __init__(self, target: Verify, draft_model, draft_kv_pool):
        st, cfg, b = target.stack, target.cfg, target.block
        assert st is not None and st.accept is not None, "the verify stack was bound without its accept tail"
        self.target, self.st, self.b, self.device = target, st, b, target.device
        sim_len, sim_method, sim_tokens = shim.simulated_acceptance()
        self.sample = sim_len <= 0 and st.accept_sampled is not None
        self.fixed = fixed_token()
        dcfg = target.draft_cfg
        kw = dict(capture=list(target.capture), pool_rows=RING_ROWS, rope_rows=shim.context_length() + 2 * cfg.rows,
                  wait_budget=WAIT_BUDGET)  # fmt: skip
        if cfg.tp > 1:
            self.it = Iteration.connect(st, target.peers, dcfg, target.draft, target.group, **kw)
        else:
            self.it = Iteration(st, dcfg, target.draft, **kw)
        dr = self.it.draft
        dev = self.device
        # SGLang's draft KV pool, layer by layer, as rows of this rank's kv heads x 128, indexed by the target's slot ids
        layer_ids = [layer.self_attn.attn.layer_id for layer in draft_model.layers]
        assert len(layer_ids) == dcfg.layers, (len(layer_ids), dcfg.layers)
        row = dr.k_pool[0][0].numel()
        full_slots = min(int(k.shape[0]) for (k, _), lr in zip(st.pools, st.layers) if lr.case.global_attn) if any(
            lr.case.global_attn for lr in st.layers) else int(st.pools[0][0].shape[0])  # fmt: skip
        self.draft_kv = []
        for lid in layer_ids:
            kv = (draft_kv_pool.get_key_buffer(lid), draft_kv_pool.get_value_buffer(lid))
            for t in kv:
                assert t.dtype == torch.bfloat16 and t.is_contiguous() and t[0].numel() == row and t.shape[0] >= full_slots, (
                    lid, t.dtype, tuple(t.shape), row, full_slots)  # fmt: skip
            self.draft_kv.append(tuple(t.view(t.shape[0], -1) for t in kv))
        # ring -> pool copies: one launch at the end of every iteration (lag 1: the rings hold the positions below
        # P - commit) and one after the draft ran alone (lag 0: below P)
        rings = [t for l in range(dcfg.layers) for t in (dr.k_pool[l], dr.v_pool[l])]
        pools = [t for kv in self.draft_kv for t in kv]
        self.ring_ptr = torch.tensor([t.data_ptr() for t in rings], dtype=torch.int64, device=dev)
        self.pool_ptr = torch.tensor([t.data_ptr() for t in pools], dtype=torch.int64, device=dev)
        self.sync_state = torch.zeros(17, dtype=torch.int64, device=dev)
        self.sync_status = torch.zeros(16, dtype=torch.int32, device=dev)
        self.f = target.frame

        def sync_bind(lag: int):
            bind = host.make("MkDflashKvSyncBind", words=st.accept.words, window=self.f["out_cache_loc"], state=self.sync_state,
                             ring=self.ring_ptr, pool=self.pool_ptr, n_buf=len(rings), row_bytes=row * 2, ring_rows=RING_ROWS,
                             lag=lag, status=self.sync_status)  # fmt: skip
            return st.lib.bind("mk_dflash_kv_sync_bind", st.module, bind)

        self.sync, self.flush_sync = sync_bind(1), sync_bind(0)
        self.r2t = st.req_to_token
        self.width = int(self.r2t.shape[1])
        self.offsets = torch.arange(b, dtype=torch.int64, device=dev)
        self.cols = torch.arange(b, dtype=torch.int64, device=dev)
        self.outs = [self._outputs() for _ in range(2)]
        modes = ("greedy", "sample") if self.sample else ("greedy",)
        self.graphs = {m: [self._capture(out, m) for out in self.outs] for m in modes}
        self.flush_graph = self._capture_flush()
        self.parity = 0
        self.rid = None
        self.pending = False  # the run's last commit is not in SGLang's draft pool yet
        logger.info("fused DFlash2 iteration: block %d, %d launches in one graph%s%s%s", b, self.it.kernels + 2,
                    " (token tree)" if st.tree_table is not None else "",
                    " (and a sampled graph)" if self.sample else "",
                    f"; simulated accept length {sim_len:g} ({sim_method}, {sim_tokens} tokens; sampled steps run SGLang's)"
                    if sim_len > 0 else "")  # fmt: skip

    # ---- graphs ----
    def _outputs(self) -> dict:
        dev = self.device
        return dict(tokens=torch.zeros(1, self.b, dtype=torch.int64, device=dev), commit=torch.zeros(1, dtype=torch.int32, device=dev),
                    bonus=torch.zeros(1, dtype=torch.int64, device=dev), new_seq_lens=torch.zeros(1, dtype=torch.int64, device=dev))  # fmt: skip

    def window_slots(self) -> None:
        """The window's positions (the committed length + 0 .. b - 1) and their slots in both pools, from the request's
        slot-table row (torch work on static buffers: captured with the graph)."""
        f = self.f
        torch.add(f["seq_lens"], self.offsets, out=f["positions"])
        flat = f["req_pool_indices"] * self.width + f["positions"]
        f["out_cache_loc"].copy_(self.r2t.view(-1)[flat])
        torch.index_select(self.st.full_to_swa, 0, f["out_cache_loc"], out=f["swa_out_cache_loc"])

    def _export(self, out: dict) -> None:
        """The step's results in the worker's form: the committed tokens (the accepted drafts, then the bonus; zeros past
        the commit), the commit length, the bonus and the new committed length. In the fixed token mode every token and
        the bonus are the fixed id, which the next draft also starts from."""
        w, ring = self.st.accept.words, self.st.accept.out_ring
        commit = w[WORDS["COMMIT"]]
        if self.fixed is None:
            idx = torch.remainder(w[WORDS["OUT_COUNT"]] - commit + self.cols, ring.shape[0])
            out["tokens"][0].copy_(torch.where(self.cols < commit, ring[idx].long(), 0))
        else:
            w[WORDS["ANCHOR"]].fill_(self.fixed)
            out["tokens"].fill_(self.fixed)
        out["commit"].copy_(commit)
        out["bonus"].copy_(w[WORDS["ANCHOR"]])
        out["new_seq_lens"].copy_(w[WORDS["P"]])

    def _capture(self, out: dict, mode: str) -> torch.cuda.CUDAGraph:
        dev = self.device
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.cuda.graph(g, stream=side):
            s = torch.cuda.current_stream(dev).cuda_stream
            self.window_slots()
            self.it.launch_all(s, True, sample=(mode == "sample") if self.st.sample_too else None, feeds=True)
            self.sync(s, True)
            self._export(out)
        torch.cuda.current_stream(dev).wait_stream(side)
        return g

    def _capture_flush(self) -> torch.cuda.CUDAGraph:
        """The draft alone (its context update writes the last commit's rows into the rings), then their pool copy."""
        dev = self.device
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.cuda.graph(g, stream=side):
            s = torch.cuda.current_stream(dev).cuda_stream
            self.it.draft.launch_all(s, True, sample=False if self.st.sample_too else None)
            self.flush_sync(s, True)
        torch.cuda.current_stream(dev).wait_stream(side)
        return g

    # ---- eligibility ----
    def mode(self, batch, needs_logits: bool) -> Optional[str]:
        """The graph of a step: "greedy" (a batch-1 greedy decode step that needs no logits), "sample" (a batch-1 sampled
        decode step with temperature, top-k and top-p only), or None (SGLang's step)."""
        fm = batch.forward_mode
        if fm.is_extend() or batch.is_extend_in_batch or fm.is_idle():
            return None
        if len(batch.reqs) != 1 or not isinstance(batch.spec_info, DraftInput):
            return None
        # per request, as SGLang's draft does: the batch's is_all_greedy is not recomputed when a sampled request leaves
        if batch.sampling_info is None or batch.reqs[0].sampling_params.top_k <= 1:
            return None if needs_logits else "greedy"
        return "sample" if self.sample and plain_sampling(batch) else None

    def __call__(self, batch, *, needs_logits: bool, on_publish):
        """A step of SGLang's DFlash2 worker: the fused iteration for an eligible batch (``mode``), else None (SGLang's
        step; the request's next fused step restarts it). Before any step but the run's next fused one, the run's last
        commit goes into SGLang's draft pool."""
        mode = self.mode(batch, needs_logits)
        if self.pending and (mode is None or batch.reqs[0].rid != self.rid):
            self.flush_graph.replay()
            self.pending = False
        if mode is None:
            self.rid = None
            return None
        return self.step(batch, mode, on_publish)

    # ---- a run ----
    def _start(self, batch, mode: str) -> None:
        """The request's state from SGLang's: the committed length P0 and the bonus token as the anchor, no commit to
        fold into the draft's context (its K / V is the pool's: the rings are filled from SGLang's draft pool with the
        positions the draft window reaches), the pool complete up to P0, and (sampled) the request's sampling words."""
        st, dr = self.st, self.it.draft
        w = st.accept.words
        p0 = int(batch.seq_lens[0])
        steps = w[WORDS["ITER"]].clone() if st.accept_override is not None else None  # the forced table continues across runs
        w.zero_()
        w[WORDS["P"]] = p0
        if steps is not None:
            w[WORDS["ITER"]].copy_(steps)
        w[WORDS["ANCHOR"]].copy_(batch.spec_info.bonus_tokens[0])
        self.sync_state.zero_()
        self.sync_state[0] = p0
        lo = max(0, p0 - (RING_ROWS - 2 * self.b))
        pos = torch.arange(lo, p0, device=self.device)
        slots = self.r2t[batch.req_pool_indices[0], lo:p0].long()
        rows = pos % RING_ROWS
        for l, (k, v) in enumerate(self.draft_kv):
            dr.k_pool[l].view(RING_ROWS, -1)[rows] = k[slots]
            dr.v_pool[l].view(RING_ROWS, -1)[rows] = v[slots]
        if mode == "sample":
            sp = batch.reqs[0].sampling_params
            st.samp.copy_(sampling_words(request_seed(batch.reqs[0]), p0, sp.temperature, sp.top_k, sp.top_p))

    def step(self, batch, mode: str, on_publish):
        batch.seq_lens.record_stream(torch.cuda.current_stream())
        rid = batch.reqs[0].rid
        if rid != self.rid:
            self._start(batch, mode)
            self.rid = rid
            logger.info("fused DFlash2 iteration: request %s starts (%s)", rid, mode)
        self.f["seq_lens"].copy_(batch.seq_lens)
        self.f["req_pool_indices"].copy_(batch.req_pool_indices)
        self.graphs[mode][self.parity].replay()
        self.pending = True
        out = self.outs[self.parity]
        self.parity ^= 1
        if on_publish is not None:
            on_publish(out["new_seq_lens"])
        return GenerationBatchResult(
            logits_output=LogitsProcessorOutput(next_token_logits=None), next_token_ids=out["tokens"].view(-1),
            accept_lens=out["commit"], can_run_cuda_graph=True,
            next_draft_input=make_draft_input_v2(bonus_tokens=out["bonus"], new_seq_lens=out["new_seq_lens"]),
            speculative_num_draft_tokens=self.b, new_seq_lens=out["new_seq_lens"],
        )  # fmt: skip

    def statuses(self) -> list:
        bad = self.it.statuses()
        code = int(self.sync_status[0])
        return bad + ([("draft_kv_sync", code, int(self.sync_status[1]), int(self.sync_status[3]))] if code else [])


# ---- the hooks of an SGLang without the iteration slot -------------------------------------------------------------------------


def _target(worker) -> Optional[Verify]:
    try:
        from sglang.srt.kernel_plugins.nvidia.binding import built_megakernel  # type: ignore

        built = built_megakernel(worker.target_worker.model_runner.model)
    except ImportError:
        built = getattr(worker.target_worker.model_runner.model, "built_megakernel", None)
    return built if isinstance(built, Verify) else None


def after_init_cuda_graphs(result, worker, *args, **kwargs):
    """Binds and captures the fused iteration once SGLang's graphs exist (a server with the target's spec built)."""
    target = _target(worker)
    if target is not None:
        target.fused = target.dflash_iteration(block_size=target.block, draft_model=worker.draft_model,
                                               draft_kv_pool=worker.draft_model_runner.token_to_kv_pool)  # fmt: skip
    return result


def around_forward_batch_generation(original, worker, batch, *args, on_publish=None, **kwargs):
    """The fused iteration for an eligible step, else SGLang's step."""
    target = _target(worker)
    out = None
    if target is not None and target.fused is not None:
        out = target.fused(batch, needs_logits=not worker._can_skip_verify_logits(batch, batch.sampling_info), on_publish=on_publish)
    if out is None:
        return original(worker, batch, *args, on_publish=on_publish, **kwargs)
    return out


def install() -> None:
    """The two hooks on SGLang's DFlash2 worker (the target spec's build calls this once per process, before SGLang
    builds the worker)."""
    HookRegistry.register(f"{WORKER}.init_cuda_graphs", after_init_cuda_graphs, AFTER)
    HookRegistry.register(f"{WORKER}.forward_batch_generation", around_forward_batch_generation, AROUND)
    HookRegistry.apply_hooks()
