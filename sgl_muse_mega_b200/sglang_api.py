"""The slice of SGLang's megakernel-plugin API this package talks to, with a local stand-in when SGLang is absent.

The reference imports ``Feature, MegakernelSpec, Numerics, NumericsKind, Requirements`` and ``register`` from
``sglang.kernels.plugin_kernels.nvidia.spec`` (``sgl_muse_mega/muse_spark/spec.py:11-17``, ``plugin.py:26-31``). SGLang is
not a dependency that can be assumed at test time, so the same names are re-exported from here: SGLang's own when it
imports, otherwise dataclasses with exactly the fields the reference's specs fill (``spec.py:143-199``) and a registry
with the lookups the reference's tests use (``test/unit/test_plugin.py:46-95``: ``register``, ``find_spec``).
The stand-in pins field names only: behaviour of the real SGLang classes is not reproduced.
"""

from __future__ import annotations

import enum
import importlib
from dataclasses import dataclass, field
from typing import Callable, Optional

try:  # pragma: no cover - exercised only where SGLang with the plugin framework is installed
    from sglang.kernels.plugin_kernels.nvidia.spec import (  # type: ignore
        ENTRY_POINT,
        MEGAKERNEL_API_VERSION,
        Feature,
        MegakernelSpec,
        Numerics,
        NumericsKind,
        Requirements,
        find_spec,
        register,
    )

    HAVE_SGLANG = True
except ImportError:
    HAVE_SGLANG = False
    ENTRY_POINT = "nvidia_megakernel"
    MEGAKERNEL_API_VERSION = 1

    class Feature(enum.Enum):
        SPECULATIVE_DECODING = "speculative_decoding"
        MULTI_NODE_TP = "multi_node_tp"
        EXPERT_PARALLEL = "expert_parallel"

    class NumericsKind(enum.Enum):
        BITWISE = "bitwise"
        TOLERANCE = "tolerance"

    @dataclass(frozen=True)
    class Numerics:
        kind: NumericsKind
        tolerances: dict = field(default_factory=dict)

    @dataclass(frozen=True)
    class Requirements:
        isas: frozenset
        tp_sizes: frozenset
        resident_blocks: int
        dtypes: frozenset
        decode_graph_backends: frozenset
        server_args: dict = field(default_factory=dict)
        hf_config: dict = field(default_factory=dict)
        env: dict = field(default_factory=dict)

    @dataclass(frozen=True)
    class MegakernelSpec:
        name: str
        requires: Requirements
        features: frozenset
        numerics: Numerics
        max_rows: int
        build: Callable
        api_version: int = MEGAKERNEL_API_VERSION
        model_disable_reasons: Optional[Callable] = None
        config_disable_reasons: Optional[Callable] = None

    _REGISTRY: dict[str, str] = {}

    def register(*, architecture: str, path: str) -> None:
        """Registers a spec by import path ("module:ATTR"); nothing is imported until the spec is looked up."""
        _REGISTRY[architecture] = path

    def find_spec(*, architectures, isa: str):
        """-> (spec, None) for the first registered architecture whose spec serves ``isa``, else (None, why)."""
        why = f"no megakernel spec is registered for {list(architectures)}"
        for arch in architectures:
            path = _REGISTRY.get(arch)
            if path is None:
                continue
            mod, attr = path.split(":")
            spec = getattr(importlib.import_module(mod), attr)
            if isa in spec.requires.isas:
                return spec, None
            why = f"{spec.name} serves {sorted(spec.requires.isas)}, not {isa}"
        return None, why
