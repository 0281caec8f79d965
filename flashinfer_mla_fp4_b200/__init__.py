"""B200-native per-token-scaled FP4 MLA decode.

Drop-in for ``flashinfer_mla_fp4.BatchMLADecodeCuteDSLFP4Wrapper`` (reference
``flashinfer_mla_fp4/__init__.py:8-10``): same ``plan()/run()`` API and cache format,
backed by hand-written sm_100a kernels behind a C ABI (``include/mla_fp4_b200.h``).
"""
from .wrapper import BatchMLADecodeCuteDSLFP4Wrapper
from .adapter import FP4MLADecodeBackend, FP4MLAPagedCache, decode_slot_mapping

__all__ = ["BatchMLADecodeCuteDSLFP4Wrapper", "FP4MLADecodeBackend", "FP4MLAPagedCache", "decode_slot_mapping"]
