"""SGLang-facing: the object the spec's ``build`` returns. SGLang asks it whether it takes a step (``plan``) and, if so,
calls ``forward`` instead of the model's own forward.

Same surface as the reference's ``Verify`` (``runtime/executor.py:112-265``): ``widths``, ``draft_sampler``,
``summary()``, ``plan(input_ids, forward_batch, ...) -> Step | None``, ``forward(step, original, input_ids, positions,
forward_batch, input_embeds=None) -> LogitsProcessorOutput`` and ``dflash_iteration(block_size=, draft_model=,
draft_kv_pool=)``, which returns the fused draft + verify + accept step (``runtime/iteration.py``). It takes the batch-1
target-verify step of a DFlash2 block under SGLang's decode-graph capture and nothing else; any other step returns None
and SGLang runs its own path.

The stack is bound on the first step it takes: only then do SGLang's KV pools and request table exist. Binding allocates,
packs weights and (in a world of several ranks) swaps handles over ``torch.distributed`` with a barrier, none of which
may run inside a stream capture: ``forward`` therefore binds only when the stream is not capturing, and a first step that
arrives inside a capture is refused with an error naming ``prepare`` (call it once before SGLang captures its graphs:
the DFlash2 worker's graph initialisation does). The step's batch tensors are copied into fixed device buffers (the
launches are bound to addresses, and a CUDA graph replays them), the window feeds are refreshed by their kernel, and the
launches of the step are enqueued on the current stream.

Device waits never trap: a peer that does not signal makes a wait give up and record itself in the stack's one status
block (all launches of the stack share it, so every later wait of the step gives up at once instead of waiting a full
budget). ``forward`` copies the block's head to pinned memory after each step and checks the previous step's copy before
the next: a recorded failure raises ``RuntimeError`` (SGLang's fallback path can take over) and the block is cleared.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..b200 import stack as S
from ..config import Config
from . import shim
from .shim import LogitsProcessorOutput

# polls an exchange wait spends before it gives up (a poll is one round trip to the L2, 0.5 - 1 us: seconds)
WAIT_BUDGET = 1 << 22
STATUS_NAMES = {1: "an exchange wait ran out (a peer never signalled)", 2: "a grid barrier ran out",
                3: "a bulk copy or tensor-core barrier never completed", 4: "an out-of-range position or slot was clamped",
                6: "a row's router scores were NaN"}  # fmt: skip


@dataclass
class Step:
    mode: str
    rows: int
    view: object = None  # the serving framework's step view: ``kv_pool`` and ``req_to_token_pool`` are read from it


def kv_buffers(pool, layers: int) -> list:
    """Every layer's (K, V) buffer of the pool as [slots, kv heads x 64] rows."""
    out = []
    for layer in range(layers):
        k, v = pool.get_key_buffer(layer), pool.get_value_buffer(layer)
        assert k.dtype == v.dtype == torch.bfloat16 and k.is_contiguous() and v.is_contiguous(), layer
        out.append((k.view(k.shape[0], -1), v.view(v.shape[0], -1)))
    return out


def _addresses(kv) -> list:
    return [(k.data_ptr(), tuple(k.shape), v.data_ptr(), tuple(v.shape)) for k, v in kv]


def capture_layers(cfg: Config, layers_to_capture) -> list:
    """The target layers whose OUTPUT residual the draft reads. SGLang's model lists the layers whose INPUT it
    captures (``layers_to_capture``: layer i + 1 for the draft's target layer i, reference sm103/dflash/iteration.py
    ``capture_layers``); an index equal to the layer count names the last layer's output."""
    out = [int(i) - 1 for i in layers_to_capture]
    assert all(0 <= i < cfg.layers for i in out), (list(layers_to_capture), cfg.layers)
    return out


class Verify:
    draft_sampler = None

    def __init__(self, cfg: Config, block: int, case, lib, module, arena, model, rank: int, device, group, summary: str,
                 tree: bool = False):  # fmt: skip
        self.cfg, self.block, self.case, self.lib, self.module, self.arena = cfg, block, case, lib, module, arena
        self.model, self.rank, self.device, self.group = model, rank, device, group
        self.widths, self._summary = (block,), summary
        self.tree = tree  # the fused iteration verifies a token tree (runtime.build.tree_enabled)
        self._chain_table: Optional[torch.Tensor] = None
        self.stack: Optional[S.Stack] = None
        self.peers = None
        self.kv_pool = None
        self.kv_bound: list = []
        # the draft spec's weights (``muse_spark/draft.py`` build) and the fused iteration, when DFlash2 builds them
        self.draft = None
        self.draft_cfg = None
        self.fused = None
        self.capture: list = []
        self.aux: Optional[torch.Tensor] = None
        i64 = torch.int64
        # fixed device copies of the step's batch tensors (the launches are bound to these addresses)
        self.frame = dict(
            positions=torch.zeros(block, dtype=i64, device=device),
            out_cache_loc=torch.zeros(block, dtype=i64, device=device),
            swa_out_cache_loc=torch.zeros(block, dtype=i64, device=device),
            seq_lens=torch.zeros(1, dtype=i64, device=device),
            req_pool_indices=torch.zeros(1, dtype=i64, device=device),
        )
        self._status_host: Optional[torch.Tensor] = None
        self._status_event = None

    def summary(self) -> str:
        return self._summary

    def plan(self, input_ids, forward_batch, *args, **kwargs) -> Optional[Step]:
        """A Step for the batch-1 target-verify forward of exactly one block under SGLang's decode-graph capture, else
        None (SGLang's own path runs), as reference executor.py:160-172."""
        if input_ids is None or not shim.is_capture_mode():  # the prefill of a multimodal model re-enters without ids
            return None
        if not forward_batch.forward_mode.is_target_verify() or int(forward_batch.batch_size) != 1:
            return None
        if int(input_ids.shape[0]) != self.block:
            return None
        return Step(mode="target_verify", rows=self.block, view=kwargs.get("view"))

    # ---- binding ----
    def prepare(self, view) -> None:
        """Binds the stack on the framework's KV pools (each layer's rows in its attention type's pool), request table
        and full -> sliding-window slot map. Allocates and synchronises: never inside a stream capture."""
        if self.stack is not None:
            return
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the verify stack is not bound yet and the stream is capturing: call Verify.prepare(view) "
                               "before the decode graphs are captured (binding allocates and synchronises)")  # fmt: skip
        cfg = self.cfg
        pool = self.kv_pool = view.kv_pool
        pools = kv_buffers(pool, len(self.case.layers))
        for layer, (k, _) in enumerate(pools):
            assert k.shape[1] * 2 == cfg.kv_row_bytes, (layer, tuple(k.shape))
        self.kv_bound = _addresses(pools)
        r2t = getattr(view, "req_to_token_pool", None) or shim.req_to_token_pool()
        frame = dict(self.frame, req_to_token=r2t.req_to_token, full_to_swa=pool.full_to_swa_index_mapping)
        # With the DFlash2 draft built, the stack also binds the accepts of the fused iteration (greedy and sampled, one set
        # of step words) beside the soft cap of the plain verify step; SGLang's simulated acceptance becomes the accept's
        # forced table.
        extra = {}
        if self.draft is not None:
            from .iteration import simulated_accepts

            table = simulated_accepts(self.block)
            extra = dict(accept_too=True, sample_too=True, sampling=torch.zeros(4, dtype=torch.int64),
                         accept_override=None if table is None else table.to(self.device), ring=4096,
                         block_verify=bool(getattr(shim.server_spec(), "speculative_use_block_verification", True)))  # fmt: skip
            if self.tree:  # the tree's accept is the greedy one: no sampled accept beside it (sampled steps run SGLang's)
                extra = dict(accept_too=True, tree=True, accept_override=extra["accept_override"], ring=4096)
        self.stack = S.Stack(self.case, self.rank, self.device, self.lib, self.module, arena=self.arena, greedy=False,
                             keep_plain_experts=False, frame=frame, pools=pools, wait_budget=WAIT_BUDGET,
                             shared_status=True, identity_slots=False, packets=True, **extra)  # fmt: skip
        if cfg.tp > 1:
            self.peers = S.connect_world(self.stack, self.group)
        else:
            self.stack.bind()
        # the DFlash2 capture layers' output residuals, packed in capture order as bf16: what the model's own forward
        # returns as hidden_states and the draft's fc consumes (reference executor.py:205-218, 255-265)
        lm = self.model.model.language_model if self.model is not None else None
        want = getattr(lm, "layers_to_capture", None)
        self.capture = capture_layers(cfg, want) if want else []
        n = max(len(self.capture), 1)
        self.aux = torch.empty(self.block, n * cfg.hidden, dtype=torch.bfloat16, device=self.device)
        self._status_host = torch.zeros(8, dtype=torch.int32).pin_memory()
        self._status_event = torch.cuda.Event()

    def check_kv(self, pool) -> None:
        """Raises unless the framework's KV buffers are still the ones the launches were bound to."""
        now = _addresses(kv_buffers(pool, len(self.case.layers)))
        if now != self.kv_bound:
            bad = [j for j, (x, y) in enumerate(zip(now, self.kv_bound)) if x != y]
            raise RuntimeError(f"the KV pools moved since the stack was bound (the launches hold their addresses): layers {bad}")

    def check_status(self) -> None:
        """Raises if the last step this object enqueued recorded a device failure; clears the block so the next step
        starts clean. Called at the start of every ``forward``; a host may also call it after synchronising."""
        if self._status_event is None or not self._status_event.query():
            return
        code, stage, block, observed = (int(x) for x in self._status_host[:4])
        if code == 0:
            return
        self._status_host.zero_()
        self.stack.shared_status.zero_()
        raise RuntimeError(f"the verify step failed on the device: {STATUS_NAMES.get(code, f'status {code}')} "
                           f"(stage {stage}, block {block}, observed {observed}); its outputs were meaningless")  # fmt: skip

    def dflash_iteration(self, *, block_size: int, draft_model, draft_kv_pool):
        """The fused DFlash2 iteration (``runtime/iteration.py``), bound once SGLang's graphs are captured: called by
        SGLang's DFlash iteration slot, or by this package's hook on a worker without one (reference executor.py:226-241)."""
        from .iteration import Fused  # iteration imports this module

        assert block_size == self.block, (block_size, self.block)
        assert self.stack is not None, "the target's batch-1 verify step was never bound (Verify.prepare)"
        assert self.draft is not None, "the DFlash2 draft's spec did not build (muse_spark/draft.py)"
        self.check_kv(self.kv_pool)
        return Fused(self, draft_model, draft_kv_pool)

    # ---- the step ----
    def forward(self, step: Step, original, input_ids, positions, forward_batch, input_embeds=None) -> LogitsProcessorOutput:
        """One verify step: ids and the batch's slot tensors in; out the block's soft-capped f32 logits and the capture
        layers' output residuals [block, n_capture x hidden] bf16 (what the draft's fc reads). ``original`` (the model's
        own forward) is what SGLang would have called; it is not used."""
        if step is None or step.mode != "target_verify":
            raise RuntimeError("Verify.forward takes the steps its plan() accepted")
        if self.stack is None:
            self.prepare(step.view)
        capturing = torch.cuda.is_current_stream_capturing()
        if not capturing:
            self.check_status()
        pool = step.view.kv_pool
        self.check_kv(pool)
        f, st = self.frame, self.stack
        st.tokens.copy_(input_ids, non_blocking=True)
        f["positions"].copy_(positions, non_blocking=True)
        f["out_cache_loc"].copy_(forward_batch.out_cache_loc, non_blocking=True)
        torch.index_select(pool.full_to_swa_index_mapping, 0, f["out_cache_loc"], out=f["swa_out_cache_loc"])
        f["seq_lens"].copy_(forward_batch.seq_lens[:1], non_blocking=True)
        f["req_pool_indices"].copy_(forward_batch.req_pool_indices[:1], non_blocking=True)
        if st.tree_table is not None:
            # a stack bound for the token tree reads its rows' places and masks from the tree's table: SGLang's own verify
            # step sends a chain, whose table is parent r - 1, depth r, every earlier row an ancestor
            if self._chain_table is None:
                r = torch.arange(16, dtype=torch.int32)
                t = torch.zeros(96, dtype=torch.int32)
                t[0:16], t[16:32], t[32:48] = r - 1, r, (2 << r) - 1
                self._chain_table = t.to(self.device)
            st.tree_table.copy_(self._chain_table, non_blocking=True)
        s = torch.cuda.current_stream(self.device).cuda_stream
        st.launch_all(s, pdl=True, feeds=True)
        if self.capture:
            H = self.cfg.hidden
            for j, c in enumerate(self.capture):
                self.aux[:, j * H : (j + 1) * H].copy_(st.layers[c].o["stream_out"][: self.block])
        else:  # no draft asked for captures: the last layer's normed rows, as before the draft existed
            self.aux.copy_(st.hidden[: self.block])
        if not capturing:
            self._status_host.copy_(st.shared_status.view(torch.int32)[:8], non_blocking=True)
            self._status_event.record(torch.cuda.current_stream(self.device))
        return LogitsProcessorOutput(next_token_logits=st.logits_out, hidden_states=self.aux)
