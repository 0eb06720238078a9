"""Index keys in a paged cache.

Serving stacks keep keys in fixed-size pages handed out by an allocator, so a
sequence's keys are not contiguous.  The reference supports contiguous keys only
(``src/fused_index_topk/inputs.py:31-32``).  Here the pool is
``kv_pool [pages, page_size, 128]`` e4m3 with ``scale_pool [pages, page_size]``
fp32, and ``block_table`` (int32) lists the pages of the logical key sequence in
order.  ``page_size`` must be a multiple of 128, the kernel's key tile: the TMA
producer, the epilogue's scale load and the sample gather then only swap the
tile's row offset (``tile_table[t] * 128``), and everything a caller sees (ids,
``[k_start, k_end)``, the number of keys) stays in logical positions.

Together with ``batched.varlen_ranges`` one block table serves a whole batch: the
logical key space is the concatenation of the sequences, each starting on a page
boundary.
"""

from __future__ import annotations

from typing import Any

from . import _lib
from .operator import _WORKSPACES, Workspace, _require, make_workspace, replay_or_run

TILE_KEYS = 128


def expand_block_table(block_table: Any, page_size: int) -> Any:
    """int32 ``[pages_used]`` pages -> int32 ``[pages_used * page_size / 128]`` physical 128-key tiles."""

    import torch

    _require(page_size >= TILE_KEYS and page_size % TILE_KEYS == 0, "page_size must be a positive multiple of 128")
    _require(block_table.dtype == torch.int32 and block_table.dim() == 1, "block_table must be int32 [pages]")
    per_page = page_size // TILE_KEYS
    within = torch.arange(per_page, device=block_table.device, dtype=torch.int32)
    return (block_table.unsqueeze(1) * per_page + within.unsqueeze(0)).reshape(-1).contiguous()


def _tile_table_buffers(workspace: Workspace, pages_used: int, per_page: int, device: Any) -> dict[str, Any]:
    """Workspace-owned buffers of the per-call block-table expansion (allocated once per table length)."""

    import torch

    key = f"paged_{pages_used}_{per_page}"
    buffers = workspace.buffers.get(key)
    if buffers is None:
        buffers = {
            "pages": torch.empty(pages_used, device=device, dtype=torch.int32),
            "tiles": torch.empty(pages_used * per_page, device=device, dtype=torch.int32),
            "within": torch.arange(per_page, device=device, dtype=torch.int32),
            "bad": torch.zeros(pages_used, device=device, dtype=torch.bool),
            "bad_any": torch.zeros(1, device=device, dtype=torch.bool),
        }
        workspace.buffers[key] = buffers
    return buffers


def _expand_on_device(buffers: dict[str, Any], block_table: Any, pages: int) -> None:
    """Physical 128-key tiles of the block table as it is NOW, into the workspace's buffer.

    Enqueued on every call (and part of the replayed CUDA graph), because a serving engine updates its
    block table in place, often from its own kernels, without any host-visible version change.  An
    entry outside the pool is clamped, so that the kernels never read outside the pool, and recorded:
    ``block_table_was_valid`` reports it.
    """

    import torch

    per_page = int(buffers["within"].numel())
    torch.clamp(block_table, 0, pages - 1, out=buffers["pages"])
    torch.ne(block_table, buffers["pages"], out=buffers["bad"])
    torch.any(buffers["bad"], dim=0, keepdim=True, out=buffers["bad_any"])
    torch.mul(buffers["pages"], per_page, out=buffers["pages"])
    torch.add(buffers["pages"].unsqueeze(1), buffers["within"].unsqueeze(0), out=buffers["tiles"].view(-1, per_page))


def block_table_was_valid(workspace: Workspace) -> bool:
    """Whether every block-table entry of the paged calls made through this workspace named a pool page.

    Synchronises; meant for tests and for debugging a serving integration, not for the hot path.
    """

    for name, buffers in workspace.buffers.items():
        if name.startswith("paged_") and bool(buffers["bad_any"].item()):
            return False
    return True


def scatter_to_pages(kv: Any, kv_scales: Any, page_size: int, *, pool_pages: int | None = None,
                     generator: Any = None) -> tuple[Any, Any, Any]:
    """Place contiguous keys into randomly chosen pages of a fresh pool.

    Returns ``(kv_pool [P, page_size, 128], scale_pool [P, page_size], block_table int32)``; unused
    pool rows are filled with a byte pattern and NaN scales so that a wrong page shows up in results.
    For tests and for callers migrating a contiguous cache.
    """

    import torch

    keys = int(kv.shape[0])
    used = (keys + page_size - 1) // page_size
    pool_pages = max(used, pool_pages or used + 3)
    order = torch.randperm(pool_pages, generator=generator)[:used].to(torch.int32)
    kv_pool = torch.full((pool_pages * page_size, _lib.HEAD_DIM), 0x3C, dtype=torch.uint8, device=kv.device)
    scale_pool = torch.full((pool_pages * page_size,), float("nan"), dtype=torch.float32, device=kv.device)
    rows = torch.arange(keys, device=kv.device)
    target = order.to(kv.device).long()[rows // page_size] * page_size + rows % page_size
    kv_pool[target] = kv.view(torch.uint8)
    scale_pool[target] = kv_scales
    return (kv_pool.view(torch.float8_e4m3fn).view(pool_pages, page_size, _lib.HEAD_DIM),
            scale_pool.view(pool_pages, page_size), order.to(kv.device))


def fused_index_topk_paged(q: Any, kv_pool_pair: tuple[Any, Any], block_table: Any, keys: int, weights: Any,
                           k_start: Any, k_end: Any, top_k: int = _lib.TOP_K, *, workspace: Workspace | None = None,
                           seed: int = 0, use_graph: bool = True) -> Any:
    """Exact Top-K ids (logical key positions) with the keys read through a block table.

    ``kv_pool_pair = (kv_pool [P, page_size, 128] e4m3, scale_pool [P, page_size] fp32)``;
    ``block_table`` int32 ``[ceil(keys / page_size)]`` on the same device; ``keys`` is the logical
    number of keys.  Returns int32 ``[Q, K]`` like ``fused_index_topk`` (the workspace's output buffer; from the
    second call with the same tensors and block table on, one CUDA-graph replay).
    """

    import torch

    kv_pool, scale_pool = kv_pool_pair
    _require(top_k == _lib.TOP_K, f"top_k must be {_lib.TOP_K}")
    _require(q.is_cuda, "q must be a CUDA tensor (there is no CPU path)")
    _require(kv_pool.dim() == 3 and kv_pool.shape[2] == _lib.HEAD_DIM, "kv_pool must have shape [P, page_size, 128]")
    pages, page_size = int(kv_pool.shape[0]), int(kv_pool.shape[1])
    _require(page_size % TILE_KEYS == 0, "page_size must be a positive multiple of 128")
    _require(tuple(scale_pool.shape) == (pages, page_size) and scale_pool.dtype == torch.float32,
             "scale_pool must be float32 [P, page_size]")
    _require(q.dtype == torch.float8_e4m3fn and kv_pool.dtype == torch.float8_e4m3fn, "q and kv_pool must be float8_e4m3fn")
    _require(q.dim() == 3 and q.shape[1] == _lib.HEADS and q.shape[2] == _lib.HEAD_DIM, "q must have shape [Q, 64, 128]")
    rows = int(q.shape[0])
    _require(rows > 0 and 0 < keys <= _lib.MAX_KEYS, f"need Q > 0 and 0 < keys <= {_lib.MAX_KEYS}")
    _require(weights.dtype == torch.float32 and tuple(weights.shape) == (rows, _lib.HEADS), "weights must be float32 [Q, 64]")
    _require(k_start.dtype == torch.int32 and k_end.dtype == torch.int32 and tuple(k_start.shape) == (rows,)
             and tuple(k_end.shape) == (rows,), "k_start and k_end must be int32 [Q]")
    for name, tensor in (("q", q), ("kv_pool", kv_pool), ("scale_pool", scale_pool), ("weights", weights),
                         ("k_start", k_start), ("k_end", k_end), ("block_table", block_table)):
        _require(tensor.is_contiguous(), f"{name} must be contiguous")
        _require(tensor.device == q.device, f"{name} must live on the same device as q")
    _require(block_table.dtype == torch.int32 and block_table.dim() == 1, "block_table must be int32 [pages]")
    _require(int(block_table.numel()) * page_size >= keys, "block_table does not cover the keys")

    if workspace is None:
        key = (rows, keys, str(q.device), int(seed))
        workspace = _WORKSPACES.get(key)
        if workspace is None:
            workspace = make_workspace(rows, keys, q.device, seed=seed)
            _WORKSPACES[key] = workspace
    _require(workspace.rows == rows and workspace.keys == keys, "workspace was made for a different problem size")
    flat_kv = kv_pool.view(pages * page_size, _lib.HEAD_DIM)
    flat_scales = scale_pool.view(pages * page_size)
    buffers = _tile_table_buffers(workspace, int(block_table.numel()), page_size // TILE_KEYS, q.device)
    return replay_or_run(workspace, (q, flat_kv, flat_scales, weights, k_start, k_end), tile_table=buffers["tiles"],
                         use_graph=use_graph, prologue=lambda: _expand_on_device(buffers, block_table, pages),
                         key_extra=(int(block_table.data_ptr()),))


__all__ = ["block_table_was_valid", "expand_block_table", "fused_index_topk_paged", "scatter_to_pages"]
