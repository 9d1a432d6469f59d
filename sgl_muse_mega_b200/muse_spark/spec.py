"""Muse Spark Open's megakernel spec for B200: the batch-1 DFlash2 verify step (16 rows at a block of 16, 8 at a block
of 8) on sm_100a, tensor-parallel over 1, 2, 4 or 8 GPUs of one NVLink 5 / NVSwitch box.

Same object the reference exports (``sgl_muse_mega/muse_spark/spec.py:143-199``): a ``MegakernelSpec`` with its
requirements, tolerances and the two refusal hooks, each returning reason strings (a non-empty list makes SGLang fall
back to its own path). What differs is what the kernels serve: isa ``sm_100``, any TP degree in {1, 2, 4, 8} on one
node, 148 resident blocks (one CTA per SM for the persistent kernels), and a toolchain check for nvcc >= 12.8 (the first
release that assembles tcgen05 for sm_100a) instead of 13.1.
"""

from __future__ import annotations

import json
import re
import subprocess
from pathlib import Path

from ..common import build as _build
from ..sglang_api import Feature, MegakernelSpec, Numerics, NumericsKind, Requirements
from .config import Config

INDEX = "model.safetensors.index.json"  # the checkpoint index the expert reader walks (reference runtime/build.py)
DRAFT_FILE = "model.safetensors"  # the DFlash2 draft's single weight file (reference sm103/dflash/weights.py)
# The longest a step can take when a peer never signals, seconds: an exchange wait gives up after the bind's poll budget
# (runtime.executor.WAIT_BUDGET polls of one L2 round trip each: seconds) and records a status instead of trapping; once
# a launch's status block holds a failure, its later waits give up after 1024 polls, and the executor raises on the status
# at the next step. SGLang's watchdog only has to exceed the first wait plus a step.
LONGEST_WAIT_S = 1.0


def toolchain_reasons() -> list:
    """nvcc must be present and able to build sm_100a tcgen05 code (the reference's check: common/jit.py:85-97)."""
    try:
        out = subprocess.run([_build.nvcc(), "--version"], capture_output=True, text=True, check=True).stdout
    except (OSError, RuntimeError, subprocess.CalledProcessError) as e:
        return [f"nvcc is not runnable ({type(e).__name__}): the kernels are built in-tree for sm_100a"]
    m = re.search(r"release (\d+)\.(\d+)", out)
    if m is None or (int(m[1]), int(m[2])) < (12, 8):
        return [f"nvcc {m[0] if m else '?'} cannot assemble tcgen05 for sm_100a (needs >= 12.8)"]
    return []


def draft_reasons(path) -> list:
    """The fused iteration's draft must be a local DFlash2 directory with its one safetensors file
    (reference spec.py:71-91)."""
    d = Path(path or "")
    try:
        arch = json.loads((d / "config.json").read_text())["architectures"]
    except (OSError, ValueError, KeyError) as e:
        return [f"--speculative-draft-model-path {path!r} has no local config.json naming its architecture ({type(e).__name__})"]
    reasons = []
    if arch != ["DFlash2DraftModel"]:
        reasons.append(f"the draft's architectures {arch} are not ['DFlash2DraftModel']")
    if not (d / DRAFT_FILE).is_file():
        reasons.append(f"the draft build reads {DRAFT_FILE} under --speculative-draft-model-path (one local file)")
    return reasons


def config_disable_reasons(cfg, hf_config) -> list:
    """Refusals that need only the server arguments and the checkpoint's config (reference spec.py:94-122)."""
    model = Config()
    reasons = model.hf_reasons(hf_config)
    if cfg.context_length is None:
        reasons.append("--context-length is unset (the rope rows bound it)")
    if cfg.nnodes != 1:
        reasons.append(f"{cfg.nnodes} nodes: the B200 kernels exchange over one box's NVLink / NVSwitch domain")
    if cfg.tp_size not in (1, 2, 4, 8):
        reasons.append(f"tp_size {cfg.tp_size} is not 1, 2, 4 or 8")
    if getattr(cfg, "watchdog_timeout", LONGEST_WAIT_S) < LONGEST_WAIT_S:
        reasons.append(f"--watchdog-timeout {cfg.watchdog_timeout} is under the kernels' {LONGEST_WAIT_S:g} s wait bound")
    if cfg.load_format == "dummy" or not (Path(cfg.model_path) / INDEX).is_file():
        reasons.append(f"the build reads the experts from {INDEX} under --model-path, a local checkpoint")
    return reasons + draft_reasons(cfg.speculative_draft_model_path) + toolchain_reasons()


def model_disable_reasons(model, hf_config) -> list:
    """Refusals that need the loaded model: every tensor the build aliases in place must have the per-rank shape and
    dtype the kernels read (reference spec.py:125-140 via runtime/build.alias_reasons)."""
    from .runtime import shim
    from .runtime.build import alias_reasons

    # the serving world's degree and this process's rank in it: the per-rank shapes (and the vocab shard's first row)
    # depend on both, so every rank checks its own tensors and all ranks reach the same verdict
    tp = shim.tp_group()
    return alias_reasons(model, Config().with_tp(tp.world_size), tp.rank_in_group)


def build(model, hf_config, ctx):
    """Post-load build; imported lazily so that registering the spec loads no kernel code."""
    from .runtime.build import build as _runtime_build

    return _runtime_build(model, hf_config, ctx)


SPEC = MegakernelSpec(
    name="Muse Spark Open (B200)",
    requires=Requirements(
        isas=frozenset({"sm_100"}),
        tp_sizes=frozenset({1, 2, 4, 8}),
        resident_blocks=148,
        dtypes=frozenset({"bfloat16"}),
        decode_graph_backends=frozenset({"full"}),
        server_args={
            "kv_cache_dtype": frozenset({"bf16", "bfloat16"}),
            "speculative_algorithm": frozenset({"DFLASH"}),
            "speculative_num_draft_tokens": frozenset({8, 16}),
            "speculative_draft_kv_cache_dtype": frozenset({None, "auto", "bf16", "bfloat16"}),
            "speculative_draft_window_size": frozenset({None}),
            "enable_unified_memory": frozenset({False}),
            "disable_hybrid_swa_memory": frozenset({False}),
            "moe_a2a_backend": frozenset({"none"}),
            "startup_weight_load_mode": frozenset({"serial"}),
        },
        hf_config={"model_type": "muse_spark"},
        env={"SGLANG_USE_HND_KVCACHE": False},
    ),
    features=frozenset({Feature.SPECULATIVE_DECODING, Feature.EXPERT_PARALLEL}),
    # per-stage relative bounds against the reference's torch path, the reference's own table (spec.py:178-193)
    numerics=Numerics(
        kind=NumericsKind.TOLERANCE,
        tolerances={
            "attention.rel": 6e-3, "post_attention.rel": 5e-3, "router_logits.rel": 5e-3, "moe_output.rel": 0.15,
            "layer_output.rel": 5e-2, "logits.rel": 0.14,
        },  # fmt: skip
    ),
    max_rows=16,
    build=build,
    api_version=1,
    model_disable_reasons=model_disable_reasons,
    config_disable_reasons=config_disable_reasons,
)
