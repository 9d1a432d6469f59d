"""The SGLang general-plugin entry point (group ``sglang.srt.plugins``, name ``nvidia_megakernel``).

Same surface as the reference's ``sgl_muse_mega/plugin.py:9-31``: ``register`` takes no arguments, runs in every SGLang
process and only records each model's spec by import path; SGLang imports a spec when ``--enable-nvidia-megakernel``
serves its architecture. No model code is imported here.
"""

SPECS = {
    "MuseSparkForConditionalGeneration": "sgl_muse_mega_b200.muse_spark.spec:SPEC",
    "DFlash2DraftModel": "sgl_muse_mega_b200.muse_spark.draft:SPEC",
}


def register() -> None:
    """Called by SGLang's plugin loader."""
    from .sglang_api import register as register_spec

    for architecture, path in SPECS.items():
        register_spec(architecture=architecture, path=path)
