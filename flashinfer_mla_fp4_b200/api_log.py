"""Env-gated call logging and NVTX ranges for the public entry points.

The reference's wrapper is decorated with FlashInfer's ``@flashinfer_api`` (reference
wrappers/batch_mla_fp4.py:189, :320), which logs calls under ``FLASHINFER_LOGLEVEL`` /
``FLASHINFER_LOGDEST``.  The same debugging aid here:

* ``MLA_FP4_LOGLEVEL``  0 off (default), 1 function names, 3 + every argument's metadata (tensors:
  shape, dtype, device, strides, data pointer; scalars: value), 5 + tensor statistics (min, max,
  mean, NaN and Inf counts; this level synchronises, is skipped while a stream is capturing and for
  tensors of more than 16 M elements), 10 + a dump of every tensor argument and of the result to
  ``MLA_FP4_DUMP_DIR`` (default ``mla_fp4_dumps``): one directory per call, ``<call>_<name>/``, holding
  ``inputs.pt`` and ``outputs.pt`` (``torch.save`` of a dict name -> CPU tensor) and ``meta.json``; tensors
  larger than ``MLA_FP4_DUMP_MAX_MB`` (default 256) are recorded in ``meta.json`` but not written.  The
  level-10 dump of FlashInfer's decorator, which the reference inherits, is its model;
* ``MLA_FP4_LOGDEST``   ``stdout`` (default), ``stderr`` or a file path (``%i`` becomes the process id);
* ``MLA_FP4_NVTX``      ``1`` wraps every call in an NVTX range named after the function.

``configure()`` changes the settings at run time.  With everything off a decorated call costs one
attribute test.
"""
from __future__ import annotations

import functools
import inspect
import os
import sys
import time
from typing import Any, Callable, Optional, TextIO

import torch


_STATS_MAX_ELEMENTS = 1 << 24  # level 5 converts a tensor to FP32 for its statistics: not for a whole cache pool


class _State:
    level: int = 0
    nvtx: bool = False
    dest: str = "stdout"
    stream: Optional[TextIO] = None
    active: bool = False
    dump_dir: str = "mla_fp4_dumps"
    dump_max_bytes: int = 256 << 20
    calls: int = 0


_state = _State()


def configure(level: Optional[int] = None, dest: Optional[str] = None, nvtx: Optional[bool] = None,
              dump_dir: Optional[str] = None, dump_max_mb: Optional[float] = None) -> None:
    """Set the log level, destination, NVTX switch and dump directory / size limit (None keeps a setting)."""
    if dump_dir is not None:
        _state.dump_dir = dump_dir
    if dump_max_mb is not None:
        _state.dump_max_bytes = int(dump_max_mb * (1 << 20))
    if level is not None:
        _state.level = int(level)
    if nvtx is not None:
        _state.nvtx = bool(nvtx)
    if dest is not None and dest != _state.dest:
        if _state.stream not in (None, sys.stdout, sys.stderr):
            _state.stream.close()
        _state.dest, _state.stream = dest, None
    _state.active = _state.level > 0 or _state.nvtx


def _out() -> TextIO:
    if _state.stream is None:
        if _state.dest == "stdout":
            _state.stream = sys.stdout
        elif _state.dest == "stderr":
            _state.stream = sys.stderr
        else:
            _state.stream = open(_state.dest.replace("%i", str(os.getpid())), "a")
    return _state.stream


def _describe(v: Any, stats: bool) -> str:
    if isinstance(v, torch.Tensor):
        s = (f"Tensor(shape={tuple(v.shape)}, dtype={v.dtype}, device={v.device}, stride={tuple(v.stride())}, "
             f"ptr=0x{v.data_ptr():x}, contiguous={v.is_contiguous()}")
        if stats and v.numel() > _STATS_MAX_ELEMENTS:
            s += f", statistics skipped ({v.numel()} elements)"
        elif stats and v.numel() > 0:
            f = v.float() if v.dtype != torch.uint8 else v.to(torch.float32)
            finite = f[torch.isfinite(f)]
            s += (f", min={finite.min().item() if finite.numel() else float('nan'):.6g}"
                  f", max={finite.max().item() if finite.numel() else float('nan'):.6g}"
                  f", mean={finite.mean().item() if finite.numel() else float('nan'):.6g}"
                  f", nan={int(torch.isnan(f).sum())}, inf={int(torch.isinf(f).sum())}")
        return s + ")"
    if isinstance(v, (tuple, list)) and any(isinstance(x, torch.Tensor) for x in v):
        return "[" + ", ".join(_describe(x, stats) for x in v) + "]"
    r = repr(v)
    return r if len(r) <= 120 else r[:117] + "..."


def _tensors_of(items) -> dict:
    out = {}
    for k, v in items:
        if isinstance(v, torch.Tensor):
            out[k] = v
        elif isinstance(v, (tuple, list)):
            for i, x in enumerate(v):
                if isinstance(x, torch.Tensor):
                    out[f"{k}.{i}"] = x
    return out


def _dump(call_dir: str, fname: str, tensors: dict, meta: dict) -> None:
    """Write the tensors that fit the size limit to <call_dir>/<fname> and describe all of them in `meta`."""
    os.makedirs(call_dir, exist_ok=True)
    keep = {}
    for k, t in tensors.items():
        nbytes = t.numel() * t.element_size()
        entry = {"shape": list(t.shape), "dtype": str(t.dtype), "device": str(t.device), "stride": list(t.stride()), "bytes": nbytes}
        if nbytes <= _state.dump_max_bytes:
            keep[k] = t.detach().to("cpu")
        else:
            entry["skipped"] = "larger than the dump limit"
        meta[k] = entry
    torch.save(keep, os.path.join(call_dir, fname))


def _capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


def api_logged(fn: Callable) -> Callable:
    """Decorator for a public entry point: logs the call (and its result) per the current settings."""
    name = fn.__qualname__
    sig = inspect.signature(fn)

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if not _state.active:
            return fn(*args, **kwargs)
        level = _state.level
        call_dir, meta = None, None
        if level >= 1:
            out = _out()
            stamp = time.strftime("%Y-%m-%d %H:%M:%S")
            out.write(f"[{stamp}] mla_fp4 API call: {name}\n")
            if level >= 3:
                stats = level >= 5 and not _capturing()
                try:
                    bound = sig.bind_partial(*args, **kwargs)
                    items = list(bound.arguments.items())
                except TypeError:  # the call itself will raise the proper error
                    items = [(f"arg{i}", a) for i, a in enumerate(args)] + list(kwargs.items())
                items = [(k, v) for k, v in items if k != "self"]
                for k, v in items:
                    out.write(f"    {k} = {_describe(v, stats)}\n")
                if level >= 10 and not _capturing():  # the dump copies to the host: not while a graph is being captured
                    _state.calls += 1
                    call_dir = os.path.join(_state.dump_dir, f"{_state.calls:06d}_{name.replace('.', '_')}")
                    meta = {"function": name, "time": stamp, "inputs": {}, "outputs": {},
                            "scalars": {k: repr(v) for k, v in items if not isinstance(v, (torch.Tensor, tuple, list))}}
                    _dump(call_dir, "inputs.pt", _tensors_of(items), meta["inputs"])
                    out.write(f"    inputs dumped to {call_dir}\n")
            out.flush()
        if _state.nvtx:
            torch.cuda.nvtx.range_push(f"mla_fp4::{name}")
        try:
            result = fn(*args, **kwargs)
        finally:
            if _state.nvtx:
                torch.cuda.nvtx.range_pop()
        if level >= 3 and result is not None:
            out = _out()
            out.write(f"    -> {_describe(result, level >= 5 and not _capturing())}\n")
            out.flush()
        if call_dir is not None:
            import json

            _dump(call_dir, "outputs.pt", _tensors_of([("result", result)]), meta["outputs"])
            with open(os.path.join(call_dir, "meta.json"), "w") as f:
                json.dump(meta, f, indent=1)
        return result

    return wrapper


configure(level=int(os.environ.get("MLA_FP4_LOGLEVEL", "0") or 0), dest=os.environ.get("MLA_FP4_LOGDEST", "stdout"),
          nvtx=os.environ.get("MLA_FP4_NVTX", "0") == "1", dump_dir=os.environ.get("MLA_FP4_DUMP_DIR", "mla_fp4_dumps"),
          dump_max_mb=float(os.environ.get("MLA_FP4_DUMP_MAX_MB", "256") or 256))

__all__ = ["api_logged", "configure"]
