"""The DFlash2 draft's megakernel spec (architecture ``DFlash2DraftModel``).

Same role as the reference's ``sgl_muse_mega/muse_spark/draft.py:42-94``: the spec covers no step of the draft model on
its own (``widths`` is empty, ``max_rows`` 0); its build reads this rank's shard of the draft checkpoint into the layouts
the draft's kernels stream and leaves it on the target's built object (``runtime.build.TARGET.draft``), before SGLang
sizes its KV pools. The fused iteration (``runtime/iteration.py``), which replaces the DFlash2 worker's batch-1 greedy and
sampled steps, binds it later, when the pools exist.
"""

from __future__ import annotations

import dataclasses
from pathlib import Path

import torch

from ..sglang_api import Feature, MegakernelSpec, Numerics, NumericsKind, Requirements
from .b200.dflash.weights import DRAFT_FILE, DraftConfig, load_shard, safetensors_reader


class Draft:
    """What the draft spec's build returns: an object that takes no step."""

    widths = ()
    draft_sampler = None

    def summary(self) -> str:
        return "DFlash2 draft in the kernels' layouts"


def model_disable_reasons(model, hf_config) -> list:
    """Every way the draft checkpoint differs from the DFlash2 draft the kernels are cut for (one reason string each), and
    a missing target build (the draft's tensors live on the target's built object)."""
    from .runtime import build as runtime_build

    try:
        cfg = DraftConfig.from_hf(hf_config.to_dict())
    except (ValueError, KeyError) as e:
        return [f"not a DFlash2 draft the kernels implement: {type(e).__name__}: {e}"]
    want = DraftConfig()
    reasons = [
        f"{f.name} {getattr(cfg, f.name)!r} is not {getattr(want, f.name)!r}"
        for f in dataclasses.fields(DraftConfig)
        if getattr(cfg, f.name) != getattr(want, f.name)
    ]
    if runtime_build.TARGET is None:
        reasons.append("the target's megakernel is not built in this process")
    return reasons


def build(model, hf_config, ctx, *, read=None, cfg: DraftConfig = DraftConfig()) -> Draft:
    """Loads this rank's draft shard next to the target's weights. ``read``: the checkpoint reader (tests pass their own;
    default: the safetensors file under the server's ``--speculative-draft-model-path``)."""
    from .runtime import build as runtime_build
    from .runtime import shim

    target = runtime_build.TARGET
    if target is None:
        raise RuntimeError("the target's megakernel is not built in this process: the draft's tensors live on it")
    tp = shim.tp_group()
    if read is None:
        read = safetensors_reader(str(Path(shim.server_spec().speculative_draft_model_path) / DRAFT_FILE))
    target.draft = load_shard(read, tp.rank_in_group, tp.world_size, cfg)
    target.draft_cfg = cfg
    if torch.cuda.is_available():
        torch.cuda.synchronize(target.device)
        torch.cuda.empty_cache()
    return Draft()


SPEC = MegakernelSpec(
    name="DFlash2 draft for Muse Spark Open (B200)",
    requires=Requirements(
        isas=frozenset({"sm_100"}),
        tp_sizes=frozenset({1, 2, 4, 8}),
        resident_blocks=148,
        dtypes=frozenset({"bfloat16"}),
        decode_graph_backends=frozenset({"full"}),
    ),
    features=frozenset({Feature.SPECULATIVE_DECODING}),
    # each draft stage against the draft's arithmetic in a fixed order (the kernel tests' band)
    numerics=Numerics(kind=NumericsKind.TOLERANCE, tolerances={"draft_unit.rel": 2e-2}),
    max_rows=0,
    build=build,
    api_version=1,
    model_disable_reasons=model_disable_reasons,
)
