"""ctypes binding of ``libitk_b200.so`` (the C ABI declared in ``include/itk_b200.h``).

There is no fallback: if the shared library is missing or does not load, every
operator call raises.  Tensors are passed as raw device pointers
(``tensor.data_ptr()``) together with the current torch CUDA stream.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_longlong, c_size_t, c_uint64, c_void_p
from pathlib import Path
from typing import Any

import os

# ITK_B200_LIBRARY points the loader at another build of the same library (timing studies).
LIBRARY_PATH = Path(os.environ.get("ITK_B200_LIBRARY") or Path(__file__).resolve().parent / "libitk_b200.so")

TOP_K = 2048
HEADS = 64
HEAD_DIM = 128
BLOCK_Q = 4
REPAIR_CHUNK = 16384
SPILL_U64_PER_ROW = 5632
MAX_KEYS = 262144
MAX_PAIR_SOURCES = 16
MAX_CTAS = 256
STATIC_MAX_ROWS = 256
STATUS_WAIT_EXPIRED = 1

EXPORTED_SYMBOLS = (
    "itk_version", "itk_last_error", "itk_init", "itk_resource_report", "itk_workspace_bytes",
    "itk_gather_sampled_kv", "itk_sample_thresholds", "itk_fused_topk", "itk_update_chunk_ranges",
    "itk_repair_produce", "itk_chunk_local_topk", "itk_merge_topk_pairs", "itk_finalize_repair",
    "itk_merge_candidate_lists", "itk_fused_topk_static", "itk_quantize_rows_e4m3",
    "itk_gather_sampled_kv_paged", "itk_repair_produce_paged", "itk_merge_shard_lists",
    "itk_compact_flagged_rows", "itk_repair_merge_chunk", "itk_flagged_scope_begin", "itk_flagged_scope_end",
)


class ItkError(RuntimeError):
    """A C-ABI call returned a negative status."""


class WorkspaceSizes(ctypes.Structure):
    _fields_ = [
        ("spill_bytes", c_size_t), ("repair_pairs_bytes", c_size_t), ("pairs_bytes", c_size_t),
        ("counts_bytes", c_size_t), ("flags_bytes", c_size_t), ("thresholds_bytes", c_size_t),
        ("chunk_ranges_bytes", c_size_t), ("repair_chunks", c_int),
    ]


class FusedArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("kv", c_void_p), ("kv_scales", c_void_p), ("weights", c_void_p),
        ("k_start", c_void_p), ("k_end", c_void_p), ("thresholds", c_void_p),
        ("out_ids", c_void_p), ("out_pairs", c_void_p), ("out_counts", c_void_p),
        ("failure_flags", c_void_p), ("spill", c_void_p),
        ("shard_pairs", c_void_p), ("shard_counts", c_void_p), ("shard_flags", c_void_p), ("diag_logits", c_void_p),
        ("diag_stride", c_longlong), ("trace", c_void_p), ("status", c_void_p),
        ("wait_limit_ns", ctypes.c_ulonglong), ("withhold_loads", c_int),
        ("rows", c_int), ("keys", c_int), ("key_lo", c_int), ("key_hi", c_int), ("shards", c_int),
        ("split_blocks", c_int), ("block_begin", c_int), ("block_stride", c_int), ("num_blocks", c_int),
        ("force_compute", c_int), ("max_ctas", c_int), ("exit_when_no_keys", c_int),
        ("tile_table", c_void_p), ("physical_keys", c_int),
        ("sampled_kv", c_void_p), ("sampled_scales", c_void_p), ("sample_ids", c_void_p), ("thresholds_out", c_void_p),
        ("samples", c_int), ("sample_rank", c_int), ("target_candidates", c_int),
    ]


_library: ctypes.CDLL | None = None


def load_library() -> ctypes.CDLL:
    """Load the shared library once; raise if it is not there."""

    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists():
        raise ItkError(
            f"{LIBRARY_PATH} is missing: build it with `python -m fusedindextopk_b200.build` "
            "(there is no CPU or PyTorch fallback)"
        )
    library = ctypes.CDLL(str(LIBRARY_PATH))
    library.itk_version.restype = c_char_p
    library.itk_last_error.restype = c_char_p
    library.itk_init.argtypes = [c_int]
    library.itk_resource_report.argtypes = [c_char_p, c_size_t]
    library.itk_workspace_bytes.argtypes = [c_int, c_int, c_int, POINTER(WorkspaceSizes)]
    library.itk_gather_sampled_kv.argtypes = [c_void_p] * 5 + [c_int, c_int, c_void_p]
    library.itk_sample_thresholds.argtypes = (
        [c_void_p] * 8 + [c_int] * 8 + [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p]
    )
    library.itk_fused_topk.argtypes = [POINTER(FusedArgs), c_void_p]
    library.itk_fused_topk_static.argtypes = [POINTER(FusedArgs), c_void_p]
    library.itk_update_chunk_ranges.argtypes = [c_void_p] * 4 + [c_int, c_int, c_void_p]
    library.itk_repair_produce.argtypes = [c_void_p] * 8 + [c_int] * 7 + [c_void_p, c_void_p]
    library.itk_chunk_local_topk.argtypes = [c_void_p] * 7 + [c_int, c_int, c_void_p]
    library.itk_merge_topk_pairs.argtypes = [c_void_p] * 6 + [c_int, c_int, c_void_p]
    library.itk_finalize_repair.argtypes = [c_void_p] * 7 + [c_int, c_void_p]
    library.itk_merge_candidate_lists.argtypes = (
        [POINTER(c_void_p), POINTER(c_void_p), c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    )
    library.itk_merge_shard_lists.argtypes = (
        [POINTER(c_void_p), POINTER(c_void_p), c_int, c_void_p, c_void_p, c_void_p, c_int]
        + [c_void_p] * 4 + [c_int] * 5 + [c_void_p, c_void_p, c_void_p]
    )
    library.itk_flagged_scope_begin.argtypes = [c_void_p, c_int, c_void_p, POINTER(c_void_p)]
    library.itk_flagged_scope_end.argtypes = [c_void_p, c_void_p]
    library.itk_compact_flagged_rows.argtypes = [c_void_p] * 5 + [c_int, c_int] + [c_void_p] * 6
    library.itk_repair_merge_chunk.argtypes = (
        [c_void_p] * 5 + [c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int] + [c_void_p] * 5
    )
    library.itk_gather_sampled_kv_paged.argtypes = [c_void_p] * 6 + [c_int, c_int, c_int, c_void_p]
    library.itk_repair_produce_paged.argtypes = [c_void_p] * 8 + [c_int] * 7 + [c_void_p, c_int, c_void_p, c_void_p]
    library.itk_quantize_rows_e4m3.argtypes = [c_void_p, c_int] + [c_void_p] * 4 + [c_longlong, c_void_p]
    for name in EXPORTED_SYMBOLS:
        function = getattr(library, name)
        if name not in ("itk_version", "itk_last_error"):
            function.restype = c_int
    _library = library
    return library


def check(status: int) -> None:
    if status != 0:
        message = load_library().itk_last_error().decode(errors="replace")
        raise ItkError(f"libitk_b200 error {status}: {message}")


def ptr(tensor: Any) -> int | None:
    """Device address of a tensor, or NULL for ``None``."""

    return None if tensor is None else int(tensor.data_ptr())


def current_stream(torch: Any, device: Any) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def version() -> str:
    return load_library().itk_version().decode()


def resource_report() -> dict[str, str]:
    """Registers / shared memory / launch shape of the kernels on the current device."""

    buffer = ctypes.create_string_buffer(8192)
    check(load_library().itk_resource_report(buffer, len(buffer)))
    report: dict[str, str] = {}
    for line in buffer.value.decode().splitlines():
        if "=" in line:
            key, value = line.split("=", 1)
            report[key] = value
    return report


def workspace_sizes(rows: int, keys: int, shards: int = 1) -> WorkspaceSizes:
    sizes = WorkspaceSizes()
    check(load_library().itk_workspace_bytes(rows, keys, shards, ctypes.byref(sizes)))
    return sizes


def pointer_table(tensors: list[Any]) -> Any:
    table = (c_void_p * len(tensors))()
    for index, tensor in enumerate(tensors):
        table[index] = tensor.data_ptr()
    return table


__all__ = [
    "BLOCK_Q", "EXPORTED_SYMBOLS", "FusedArgs", "HEADS", "HEAD_DIM", "ItkError", "LIBRARY_PATH", "MAX_KEYS",
    "MAX_PAIR_SOURCES", "REPAIR_CHUNK", "SPILL_U64_PER_ROW", "STATUS_WAIT_EXPIRED", "TOP_K", "WorkspaceSizes",
    "check", "current_stream", "load_library", "pointer_table", "ptr", "resource_report", "version",
    "workspace_sizes", "c_int32", "c_uint64",
]
