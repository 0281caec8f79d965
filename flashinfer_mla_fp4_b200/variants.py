"""Attention variants of the decode path, ahead-of-time form.

The reference forwards an ``AttentionVariant`` object to its kernel, which JIT-traces the object's hooks
(``score_mod``, ``update_statistics``, ``transform_output``; reference ``wrappers/batch_mla_fp4.py:237-253``,
flashinfer ``cute_dsl/attention/fusion/variant.py``).  Nothing is traced here: the two variants in use are compiled into
the kernels and selected by data (``MlaFp4DecodeArgs.logits_soft_cap`` / ``.sink``).  ``plan(variant=...)`` accepts the
classes below, and flashinfer's own ``StandardAttention`` / ``AttentionWithSink`` objects by duck typing; anything else
(a variant with its own hooks, or one that replaces the softmax through ``has_logits_transform``) raises ``ValueError``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


class StandardAttention:
    """Plain softmax attention."""


class AttentionWithSink:
    """One virtual token per head with logit ``sink[h]`` and a zero value row: exp(sink[h]) joins the softmax
    denominator (counted once per request, with its first tile)."""

    def __init__(self, sink: torch.Tensor) -> None:
        self._sink = sink

    @property
    def extra_params(self) -> torch.Tensor:
        return self._sink


class SoftCappingAttention:
    """Raw scores s = q.k pass through cap * tanh(s / cap) before the softmax scale (a separate kernel instantiation:
    the standard kernel carries none of its instructions).  ``sink`` optionally adds the sink of ``AttentionWithSink``."""

    def __init__(self, cap: float = 50.0, sink: Optional[torch.Tensor] = None) -> None:
        self.cap = float(cap)
        self._sink = sink

    @property
    def extra_params(self) -> Optional[torch.Tensor]:
        return self._sink


def resolve(variant, num_heads: int, device) -> Tuple[float, Optional[torch.Tensor]]:
    """(logits_soft_cap, sink on `device` or None) of a variant object; ValueError for what has no compiled form."""
    if variant is None:
        return 0.0, None
    name = type(variant).__name__
    if getattr(variant, "has_logits_transform", False):
        raise ValueError("MLA decode does not support logits_transform. Use score_mod, update_statistics, or transform_output instead.")
    if name == "StandardAttention":
        return 0.0, None
    if name not in ("AttentionWithSink", "SoftCappingAttention"):
        raise ValueError(
            f"unsupported attention variant {name}: the compiled variants are StandardAttention, AttentionWithSink and "
            "SoftCappingAttention (score_mod / update_statistics / transform_output hooks are JIT-traced callbacks in the "
            "reference and have no ahead-of-time form)")
    cap = 0.0
    if name == "SoftCappingAttention":
        cap = float(getattr(variant, "cap"))
        if not cap > 0.0:
            raise ValueError(f"SoftCappingAttention needs cap > 0, got {cap}")
    sink = getattr(variant, "extra_params", None)
    if name == "AttentionWithSink" and sink is None:
        raise ValueError("AttentionWithSink needs a sink tensor")
    if sink is not None:
        if not isinstance(sink, torch.Tensor) or sink.numel() != num_heads:
            raise ValueError(f"the sink must be a tensor of num_heads = {num_heads} values")
        sink = sink.detach().to(device=device, dtype=torch.float32).reshape(num_heads).contiguous()
    return cap, sink
