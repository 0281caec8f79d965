"""B200-native per-token-scaled FP4 MLA decode.

Drop-in for ``flashinfer_mla_fp4.BatchMLADecodeCuteDSLFP4Wrapper`` (reference
``flashinfer_mla_fp4/__init__.py:8-10``): same ``plan()/run()`` API and cache format,
backed by hand-written sm_100a kernels behind a C ABI (``include/mla_fp4_b200.h``).

The public names are resolved on first use: importing a helper module that needs no kernel
(``synth``, ``kvcache.quantize_tokens``, ``planner`` constants) does not load the C-ABI library,
while touching the wrapper or the adapter does, and fails loudly if the library is missing.
"""
from importlib import import_module

_EXPORTS = {
    "BatchMLADecodeCuteDSLFP4Wrapper": ".wrapper",
    "FP4MLADecodeBackend": ".adapter",
    "FP4MLAPagedCache": ".adapter",
    "decode_slot_mapping": ".adapter",
    "StandardAttention": ".variants",
    "AttentionWithSink": ".variants",
    "SoftCappingAttention": ".variants",
}

__all__ = list(_EXPORTS)


def __getattr__(name):
    if name in _EXPORTS:
        value = getattr(import_module(_EXPORTS[name], __name__), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
