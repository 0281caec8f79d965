"""Host view of the split-KV work partition.

The decode kernel derives its partition on the device from ``seq_lens``; this
module asks the library for the same partition computed on the host, for
inspection, tests and capacity planning.  It replaces the reference's
``mla_get_split_kv_simplified`` + static tile scheduler (flashinfer
``cute_dsl/attention/scheduler/mla_persistent.py:137-282``), which split every
request the same number of times whatever its length.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Sequence

from . import _cabi


@dataclass(frozen=True)
class Segment:
    cta: int
    request: int
    group: int
    tile_begin: int
    tile_end: int
    slot: int  # -1: the segment covers its request and writes the final output


def num_groups(q_len: int, num_heads: int) -> int:
    return q_len * ((num_heads + _cabi.GROUP_HEADS - 1) // _cabi.GROUP_HEADS)


def tiles_of(seq_len: int) -> int:
    return (seq_len + _cabi.TILE_TOKENS - 1) // _cabi.TILE_TOKENS if seq_len > 0 else 0


def plan_partition(seq_lens: Sequence[int], q_len: int, num_heads: int, num_ctas: int) -> List[Segment]:
    """All segments of all CTAs, in CTA order."""
    n = len(seq_lens)
    arr = (C.c_int32 * max(n, 1))(*[int(x) for x in seq_lens])
    count = C.c_int32(0)
    cap = num_ctas + n * num_groups(q_len, num_heads) + 8
    bufs = [(C.c_int32 * cap)() for _ in range(6)]
    _cabi.check(_cabi.lib.mla_fp4_plan_partition(arr, n, q_len, num_heads, num_ctas, cap, *bufs, C.byref(count)))
    if count.value > cap:
        raise RuntimeError("partition larger than its bound")
    return [Segment(*(int(b[i]) for b in bufs)) for i in range(count.value)]


def workspace_bytes(batch: int, q_len: int, num_heads: int, num_ctas: int) -> int:
    """Scratch bytes one decode step needs (two partial slots per CTA)."""
    return _cabi.workspace_bytes(batch, q_len, num_heads, num_ctas)
