"""Stand-ins for the SGLang objects the runtime reads, with exactly the fields it reads.

SGLang is not importable where this package is developed; the runtime (``build.py``, ``executor.py``) takes these duck
types: a real ``ForwardBatch`` / KV pool / request-to-token pool has the same attribute names (listed in the reference's
``runtime/executor.py:40-60`` and ``runtime/build.py:47-97``), so the same code serves both. Tests build the stand-ins
from synthetic tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


class ForwardMode:
    """``forward_batch.forward_mode``: only ``is_target_verify`` is asked."""

    def __init__(self, name: str):
        self.name = name

    def is_target_verify(self) -> bool:
        return self.name == "target_verify"


@dataclass
class ForwardBatch:
    forward_mode: ForwardMode
    batch_size: int
    seq_lens: torch.Tensor  # i64 [batch]
    req_pool_indices: torch.Tensor  # i64 [batch]
    out_cache_loc: torch.Tensor  # i64 [rows]


class KVPool:
    """Per-layer K and V buffers ``[slots, kv heads, 64]`` bf16 and the full -> sliding-window slot map."""

    def __init__(self, k: list, v: list, full_to_swa_index_mapping: torch.Tensor):
        self.k, self.v, self.full_to_swa_index_mapping = k, v, full_to_swa_index_mapping

    def get_key_buffer(self, layer: int) -> torch.Tensor:
        return self.k[layer]

    def get_value_buffer(self, layer: int) -> torch.Tensor:
        return self.v[layer]


@dataclass
class ReqToTokenPool:
    req_to_token: torch.Tensor  # i32 [requests, width]


@dataclass
class Parallel:
    """The tensor-parallel group as the build sees it (SGLang: ``get_parallel().tp_group``)."""

    rank_in_group: int
    world_size: int
    device_group: object = None


@dataclass
class Context:
    """What ``build(model, hf_config, ctx)`` receives: the block's rows per request."""

    tokens_per_request: int


@dataclass
class LogitsProcessorOutput:
    next_token_logits: torch.Tensor
    hidden_states: Optional[torch.Tensor] = None
    extras: dict = field(default_factory=dict)
