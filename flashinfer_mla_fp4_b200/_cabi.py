"""ctypes binding of libmla_fp4_b200.so (declarations: include/mla_fp4_b200.h).

The library is required: there is no Python or CPU fallback.  If it is missing
or fails to load, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# MLA_FP4_B200_LIB overrides the library location (for instance a debug build)
LIB_PATH = Path(os.environ.get("MLA_FP4_B200_LIB") or (Path(__file__).resolve().parent / "libmla_fp4_b200.so"))
ABI_VERSION = 5

OK = 0
ERR_BAD_ARG = 1
ERR_UNSUPPORTED = 2
ERR_WORKSPACE_TOO_SMALL = 3
ERR_CUDA = 4
ERR_DEVICE_TIMEOUT = 5
ERR_NOT_BUILT = 6

KERNEL_TCGEN05 = 0
KERNEL_FP32_CHECK = 1
KERNEL_TCGEN05_2PASS = 2
WORKSPACE_HEADER_BYTES = 2048
IN_BF16, IN_F16, IN_F32 = 0, 1, 2
OUT_BF16 = 0
OUT_F32 = 1
OUT_E4M3 = 2

TILE_TOKENS = 128
GROUP_HEADS = 64
PHANTOM_TILES = 2  # MLA_FP4_PHANTOM_TILES: tiles the work partition charges for a request's start


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("q_stride_batch", C.c_int64), ("q_stride_qpos", C.c_int64), ("q_stride_head", C.c_int64),
        ("kv_cache", C.c_void_p),
        ("kv_cache_sf", C.c_void_p),
        ("block_tables", C.c_void_p),
        ("block_table_stride", C.c_int64),
        ("seq_lens", C.c_void_p),
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("batch", C.c_int32), ("q_len", C.c_int32), ("num_heads", C.c_int32), ("page_size", C.c_int32),
        ("num_pages", C.c_int64),
        ("softmax_scale", C.c_float), ("output_scale", C.c_float),
        ("out_dtype", C.c_int32),
        ("kernel", C.c_int32),
        ("num_ctas", C.c_int32),
        ("enable_pdl", C.c_int32),
        ("phase_mask", C.c_int32),
        ("stream", C.c_void_p),
        ("max_pages_per_request", C.c_int32),
        ("wait_polls", C.c_int32),
        ("logits_soft_cap", C.c_float), ("sink", C.c_void_p),
    ]


EXPORTS = (
    "mla_fp4_abi_version",
    "mla_fp4_last_error",
    "mla_fp4_workspace_bytes",
    "mla_fp4_workspace_init",
    "mla_fp4_plan_partition",
    "mla_fp4_decode",
    "mla_fp4_merge_partials",
    "mla_fp4_dequant_e2m1_to_e4m3",
    "mla_fp4_cache_write",
    "mla_fp4_decode_static",
    "mla_fp4_static_reset",
    "mla_fp4_cp_exchange_bytes",
    "mla_fp4_cp_alloc",
    "mla_fp4_cp_open",
    "mla_fp4_cp_close",
    "mla_fp4_cp_free",
    "mla_fp4_cp_exchange_merge",
)
CP_MAX_RANKS = 8
CP_HANDLE_BYTES = 64
CP_AUTO, CP_ALL_GATHER, CP_REDUCE_SCATTER = 0, 1, 2


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m flashinfer_mla_fp4_b200.build` "
            "(nvcc, sm_100a). There is no fallback path."
        )
    lib = C.CDLL(str(LIB_PATH))
    lib.mla_fp4_abi_version.restype = C.c_int
    lib.mla_fp4_last_error.restype = C.c_char_p
    lib.mla_fp4_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_size_t)]
    lib.mla_fp4_workspace_bytes.restype = C.c_int
    lib.mla_fp4_workspace_init.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    lib.mla_fp4_workspace_init.restype = C.c_int
    i32p = C.POINTER(C.c_int32)
    lib.mla_fp4_plan_partition.argtypes = [i32p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                           i32p, i32p, i32p, i32p, i32p, i32p, i32p]
    lib.mla_fp4_plan_partition.restype = C.c_int
    lib.mla_fp4_decode.argtypes = [C.POINTER(DecodeArgs)]
    lib.mla_fp4_decode.restype = C.c_int
    lib.mla_fp4_decode_static.argtypes = [C.POINTER(DecodeArgs)]
    lib.mla_fp4_decode_static.restype = C.c_int
    lib.mla_fp4_static_reset.argtypes = [C.c_void_p]
    lib.mla_fp4_static_reset.restype = C.c_int
    lib.mla_fp4_cp_exchange_bytes.argtypes = [C.c_int32, C.c_int64, C.POINTER(C.c_size_t)]
    lib.mla_fp4_cp_exchange_bytes.restype = C.c_int
    lib.mla_fp4_cp_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]
    lib.mla_fp4_cp_alloc.restype = C.c_int
    lib.mla_fp4_cp_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.mla_fp4_cp_open.restype = C.c_int
    lib.mla_fp4_cp_close.argtypes = [C.c_void_p]
    lib.mla_fp4_cp_close.restype = C.c_int
    lib.mla_fp4_cp_free.argtypes = [C.c_void_p]
    lib.mla_fp4_cp_free.restype = C.c_int
    lib.mla_fp4_cp_exchange_merge.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p,
                                              C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    lib.mla_fp4_cp_exchange_merge.restype = C.c_int
    lib.mla_fp4_merge_partials.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
                                           C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]
    lib.mla_fp4_merge_partials.restype = C.c_int
    lib.mla_fp4_dequant_e2m1_to_e4m3.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    lib.mla_fp4_dequant_e2m1_to_e4m3.restype = C.c_int
    lib.mla_fp4_cache_write.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p,
                                        C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    lib.mla_fp4_cache_write.restype = C.c_int
    v = lib.mla_fp4_abi_version()
    if v != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {v}, expected {ABI_VERSION}: rebuild it")
    return lib


lib = _load()


def last_error() -> str:
    return (lib.mla_fp4_last_error() or b"").decode("utf-8", "replace")


def check(rc: int) -> None:
    """Map a non-zero status to the exception type the reference wrapper raises for it."""
    if rc == OK:
        return
    msg = last_error()
    if rc in (ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE_TOO_SMALL):
        raise ValueError(msg)
    raise RuntimeError(f"mla_fp4 error {rc}: {msg}")


def workspace_init(ptr: int, nbytes: int, stream: int) -> None:
    """Zero the header of a workspace (asynchronous, on `stream`)."""
    check(lib.mla_fp4_workspace_init(ptr, nbytes, stream))


def workspace_bytes(batch: int, q_len: int, num_heads: int, num_ctas: int) -> int:
    out = C.c_size_t(0)
    check(lib.mla_fp4_workspace_bytes(batch, q_len, num_heads, num_ctas, C.byref(out)))
    return int(out.value)
