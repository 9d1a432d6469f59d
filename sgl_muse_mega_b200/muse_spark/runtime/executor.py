"""SGLang-facing: the object the spec's ``build`` returns. SGLang asks it whether it takes a step (``plan``) and, if so,
calls ``forward`` instead of the model's own forward.

Same surface as the reference's ``Verify`` (``runtime/executor.py:112-265``): ``widths``, ``draft_sampler``,
``summary()``, ``plan(input_ids, forward_batch, ...) -> Step | None`` and ``forward(step, original, input_ids,
positions, forward_batch, input_embeds=None) -> LogitsProcessorOutput``. It takes the batch-1 target-verify step of a
DFlash2 block and nothing else; any other step returns None and SGLang runs its own path.

The stack is bound on the first step it takes: only then do SGLang's KV pools and request table exist. The step's batch
tensors are copied into fixed device buffers (the launches are bound to addresses, and a CUDA graph replays them), the
window feeds are refreshed by their kernel, and the launches of the step are enqueued on the current stream.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..b200 import stack as S
from ..config import Config
from .shim import LogitsProcessorOutput


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


class Verify:
    draft_sampler = None

    def __init__(self, cfg: Config, block: int, case, lib, module, arena, model, rank: int, device, group, summary: str):
        self.cfg, self.block, self.case, self.lib, self.module, self.arena = cfg, block, case, lib, module, arena
        self.model, self.rank, self.device, self.group = model, rank, device, group
        self.widths, self._summary = (block,), summary
        self.stack: Optional[S.Stack] = None
        self.peers = None
        self.kv_bound: list = []
        i64 = torch.int64
        # fixed device copies of the step's batch tensors (the launches are bound to these addresses)
        self.frame = dict(
            positions=torch.zeros(block, dtype=i64, device=device),
            out_cache_loc=torch.zeros(block, dtype=i64, device=device),
            swa_out_cache_loc=torch.zeros(block, dtype=i64, device=device),
            seq_lens=torch.zeros(1, dtype=i64, device=device),
            req_pool_indices=torch.zeros(1, dtype=i64, device=device),
        )

    def summary(self) -> str:
        return self._summary

    def plan(self, input_ids, forward_batch, *args, **kwargs) -> Optional[Step]:
        """A Step for the batch-1 target-verify forward of exactly one block, else None (SGLang's own path runs)."""
        if input_ids is None:  # the prefill of a multimodal model re-enters its forward without ids
            return None
        if not forward_batch.forward_mode.is_target_verify() or int(forward_batch.batch_size) != 1:
            return None
        if int(input_ids.shape[0]) != self.block:
            return None
        return Step(mode="target_verify", rows=self.block, view=kwargs.get("view"))

    def _bind(self, step: Step) -> None:
        """The stack on the framework's KV pools (each layer's rows in its attention type's pool), request table and
        full -> sliding-window slot map."""
        pool = step.view.kv_pool
        pools = kv_buffers(pool, len(self.case.layers))
        self.kv_bound = [(k.data_ptr(), tuple(k.shape), v.data_ptr(), tuple(v.shape)) for k, v in pools]
        frame = dict(self.frame, req_to_token=step.view.req_to_token_pool.req_to_token,
                     full_to_swa=pool.full_to_swa_index_mapping)  # fmt: skip
        self.stack = S.Stack(self.case, self.rank, self.device, self.lib, self.module, arena=self.arena, greedy=False,
                             keep_plain_experts=False, frame=frame, pools=pools)  # fmt: skip
        if self.cfg.tp > 1:
            self.peers = S.connect_world(self.stack, self.group)
        else:
            self.stack.bind()

    def forward(self, step: Step, original, input_ids, positions, forward_batch, input_embeds=None) -> LogitsProcessorOutput:
        """One verify step: ids and the batch's slot tensors in, the block's soft-capped f32 logits out. ``original``
        (the model's own forward) is what SGLang would have called; it is not used."""
        if step is None or step.mode != "target_verify":
            raise RuntimeError("Verify.forward takes the steps its plan() accepted")
        if self.stack is None:
            self._bind(step)
        pool = step.view.kv_pool
        now = [(k.data_ptr(), tuple(k.shape), v.data_ptr(), tuple(v.shape)) for k, v in kv_buffers(pool, len(self.case.layers))]
        if now != self.kv_bound:
            raise RuntimeError("the KV pools moved since the stack was bound (the launches hold their addresses)")
        f, st = self.frame, self.stack
        st.tokens.copy_(input_ids, non_blocking=True)
        f["positions"].copy_(positions, non_blocking=True)
        f["out_cache_loc"].copy_(forward_batch.out_cache_loc, non_blocking=True)
        torch.index_select(pool.full_to_swa_index_mapping, 0, f["out_cache_loc"], out=f["swa_out_cache_loc"])
        f["seq_lens"].copy_(forward_batch.seq_lens[:1], non_blocking=True)
        f["req_pool_indices"].copy_(forward_batch.req_pool_indices[:1], non_blocking=True)
        s = torch.cuda.current_stream(self.device).cuda_stream
        st.launch_all(s, pdl=True, feeds=True)
        return LogitsProcessorOutput(next_token_logits=st.logits_out, hidden_states=st.hidden)
