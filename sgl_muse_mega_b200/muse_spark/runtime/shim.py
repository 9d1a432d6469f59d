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


# ---- the serving process's singletons ----------------------------------------------------------------------------------------
# The runtime asks SGLang for a few process-wide objects (reference runtime/build.py:272-279, executor.py:15-20,
# iteration.py:44-58). Each accessor below asks SGLang when it imports and otherwise returns the stand-in a test (or an
# embedding host) installed with ``install``; nothing is guessed: a missing stand-in raises.

_STANDINS: dict = {}


def install(**objects) -> None:
    """Stand-ins by name: ``tp_group`` (a ``Parallel``), ``capture_mode`` (bool or callable), ``req_to_token_pool``,
    ``context_length`` (int), ``server_spec`` (an object with ``speculative_draft_model_path`` and
    ``speculative_use_block_verification``). ``install()`` with no arguments clears them."""
    if not objects:
        _STANDINS.clear()
    _STANDINS.update(objects)


def _standin(name: str):
    if name not in _STANDINS:
        raise RuntimeError(f"SGLang is not importable and no stand-in for {name!r} was installed (runtime.shim.install)")
    v = _STANDINS[name]
    return v() if callable(v) and name == "capture_mode" else v


def tp_group():
    """The tensor-parallel group: ``rank_in_group``, ``world_size``, ``device_group``."""
    try:
        from sglang.srt.runtime_context import get_parallel  # type: ignore
    except ImportError:
        return _standin("tp_group")
    return get_parallel().tp_group


def is_capture_mode() -> bool:
    """True while SGLang captures its decode graphs."""
    try:
        from sglang.srt.model_executor.runner import get_is_capture_mode  # type: ignore
    except ImportError:
        return bool(_standin("capture_mode"))
    return bool(get_is_capture_mode())


def req_to_token_pool():
    try:
        from sglang.srt.model_executor.forward_context import get_req_to_token_pool  # type: ignore
    except ImportError:
        return _standin("req_to_token_pool")
    return get_req_to_token_pool()


def context_length() -> int:
    try:
        from sglang.srt.runtime_context import get_model  # type: ignore
    except ImportError:
        return int(_standin("context_length"))
    return int(get_model().context_length)


def server_spec():
    """The server's speculative-decoding arguments."""
    try:
        from sglang.srt.runtime_context import get_spec  # type: ignore
    except ImportError:
        return _standin("server_spec")
    return get_spec()


def simulated_acceptance() -> tuple:
    """(length, method, token mode) of SGLang's simulated acceptance: its ``spec_utils`` constants when SGLang imports,
    else the environment variables those constants are read from (``SGLANG_SIMULATE_ACC_LEN`` / ``_METHOD`` /
    ``_TOKEN_MODE``)."""
    try:
        from sglang.srt.speculative.spec_utils import SIMULATE_ACC_LEN, SIMULATE_ACC_METHOD, SIMULATE_ACC_TOKEN_MODE  # type: ignore

        return float(SIMULATE_ACC_LEN), str(SIMULATE_ACC_METHOD), str(SIMULATE_ACC_TOKEN_MODE)
    except ImportError:
        import os

        return (float(os.environ.get("SGLANG_SIMULATE_ACC_LEN", "-1")), os.environ.get("SGLANG_SIMULATE_ACC_METHOD", "multinomial"),
                os.environ.get("SGLANG_SIMULATE_ACC_TOKEN_MODE", "real"))  # fmt: skip


@dataclass
class DraftInput:
    """Stand-in of SGLang's ``DFlashDraftInputV2``: what the fused step reads (``bonus_tokens``) and hands on."""

    bonus_tokens: torch.Tensor
    new_seq_lens: Optional[torch.Tensor] = None


@dataclass
class GenerationBatchResult:
    """Stand-in of SGLang's ``GenerationBatchResult`` with the fields the fused step fills
    (reference runtime/iteration.py:395-412)."""

    logits_output: LogitsProcessorOutput
    next_token_ids: torch.Tensor
    accept_lens: torch.Tensor
    can_run_cuda_graph: bool
    next_draft_input: DraftInput
    speculative_num_draft_tokens: int
    new_seq_lens: torch.Tensor


class HookRegistry:
    """Stand-in of SGLang's ``HookRegistry``: records (target, hook, kind) and wraps the named attribute when applied."""

    hooks: list = []

    @classmethod
    def register(cls, target: str, hook, kind: str) -> None:
        cls.hooks.append((target, hook, kind))

    @classmethod
    def apply_hooks(cls) -> None:
        import importlib

        for target, hook, kind in cls.hooks:
            mod_name, cls_name, attr = target.rsplit(".", 2)
            try:
                owner = getattr(importlib.import_module(mod_name), cls_name)
            except ImportError:
                continue  # the hooked class does not exist in this process
            original = getattr(owner, attr)
            if kind == "after":
                def wrapped(self, *a, _o=original, _h=hook, **kw):
                    return _h(_o(self, *a, **kw), self, *a, **kw)
            else:
                def wrapped(self, *a, _o=original, _h=hook, **kw):
                    return _h(_o, self, *a, **kw)
            setattr(owner, attr, wrapped)
        cls.hooks = []
