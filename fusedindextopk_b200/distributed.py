"""Multi-GPU partitioning of the operator: one process per GPU, torch.distributed for plumbing.

The reference is single-GPU (it has no collective anywhere); both partitionings below
are new design on top of the same kernels.

* Query-row sharding (replicated keys): rank r owns the query blocks (4 rows each)
  r, r+G, r+2G, ...  Rows are independent, so there is no collective on the data path;
  the round-robin deal balances the causal row lengths across ranks.
* Key-range sharding (short Q, long context): rank r scores keys [lo_r, hi_r), treats
  its slice as a stand-alone problem (ranges rebased like the reference's per-chunk
  ranges, ``kernel/csrc/long_context_repair.cu:653-669``), and produces its exact local
  Top-2048 as (ordered score, key) pairs.  The per-rank lists are all-gathered
  (1 MiB per rank at Q = 64) and every rank merges them with the pair Top-K kernel:
  the union of exact local Top-2048 lists contains the global Top-2048.
"""

from __future__ import annotations

from dataclasses import replace
from typing import Any, Callable

from . import _lib

BLOCK_Q = _lib.BLOCK_Q
TILE_KEYS = 128


def owned_rows(rows: int, rank: int, world: int) -> list[int]:
    """Global row indices of the query blocks dealt to ``rank`` (blocks rank, rank+world, ...)."""

    if not 0 <= rank < world:
        raise ValueError("need 0 <= rank < world")
    blocks = range(rank, (rows + BLOCK_Q - 1) // BLOCK_Q, world)
    return [row for block in blocks for row in range(block * BLOCK_Q, min(rows, (block + 1) * BLOCK_Q))]


def shard_rows(inputs: Any, rank: int, world: int) -> tuple[Any, Any]:
    """Inputs restricted to the rows of ``rank`` (keys replicated) and their global row ids."""

    import torch

    rows = inputs.case.query_tokens
    if world == 1:
        return inputs, torch.arange(rows)
    row_ids = torch.tensor(owned_rows(rows, rank, world), dtype=torch.long)
    device_ids = row_ids.to(inputs.q.device)
    local = replace(
        inputs,
        case=replace(inputs.case, query_tokens=int(row_ids.numel())),
        q=inputs.q[device_ids].contiguous(),
        weights=inputs.weights[device_ids].contiguous(),
        k_start=inputs.k_start[device_ids].contiguous(),
        k_end=inputs.k_end[device_ids].contiguous(),
    )
    return local, row_ids


def key_range(keys: int, rank: int, world: int) -> tuple[int, int]:
    """Key slice ``[lo, hi)`` of ``rank``: equal parts rounded up to whole 128-key tiles."""

    if not 0 <= rank < world:
        raise ValueError("need 0 <= rank < world")
    per_rank = -(-keys // world)
    per_rank = -(-per_rank // TILE_KEYS) * TILE_KEYS
    lo = min(keys, rank * per_rank)
    hi = min(keys, lo + per_rank)
    return lo, hi


def shard_keys(inputs: Any, rank: int, world: int) -> tuple[Any, int]:
    """The key slice of ``rank`` as a stand-alone problem: sliced kv/scales, rebased ranges."""

    lo, hi = key_range(inputs.case.context_tokens, rank, world)
    width = hi - lo
    local = replace(
        inputs,
        case=replace(inputs.case, context_tokens=width),
        kv=inputs.kv[lo:hi].contiguous(),
        kv_scales=inputs.kv_scales[lo:hi].contiguous(),
        k_start=(inputs.k_start - lo).clamp(min=0, max=width).contiguous(),
        k_end=(inputs.k_end - lo).clamp(min=0, max=width).contiguous(),
        generation_context_tokens=width,
    )
    return local, lo


def gpu_local_pairs(workspace: Any, local: Any, key_offset: int) -> tuple[Any, Any]:
    """Exact local Top-2048 of one key slice on the GPU: int64 pairs with global keys, counts."""

    from . import operator

    tensors = (local.q, local.kv, local.kv_scales, local.weights, local.k_start, local.k_end)
    operator.run_sample_thresholds(workspace, *tensors)
    operator.run_fused_topk(workspace, *tensors, want_pairs=True)
    if "repair_pairs" in workspace.buffers:
        operator.run_repair(workspace, *tensors, want_pairs=True)
    # keys sit in the low 32 bits; empty slots are 0 and stay behind the counts
    return workspace.output_pairs + key_offset, workspace.output_counts


def gpu_merge(gathered_pairs: Any, gathered_counts: Any, out_ids: Any) -> Any:
    """Exact Top-2048 of ``[G,Q,2048]`` gathered pairs / ``[G,Q]`` counts into int32 ``[Q,2048]``."""

    import torch

    sources, rows = int(gathered_pairs.shape[0]), int(gathered_pairs.shape[1])
    pair_table = _lib.pointer_table([gathered_pairs[s] for s in range(sources)])
    count_table = _lib.pointer_table([gathered_counts[s] for s in range(sources)])
    _lib.check(_lib.load_library().itk_merge_candidate_lists(
        pair_table, count_table, sources, _lib.ptr(out_ids), None, None, rows,
        _lib.current_stream(torch, gathered_pairs.device),
    ))
    return out_ids


def key_sharded_topk(
    inputs: Any,
    rank: int,
    world: int,
    *,
    local_pairs: Callable[[Any, int], tuple[Any, Any]],
    merge: Callable[[Any, Any], Any],
    all_gather: Callable[[Any], Any],
) -> Any:
    """Key-range sharded operator call of one rank.

    ``local_pairs(local_inputs, key_offset)`` -> (int64 ``[Q,2048]`` pairs, int32 ``[Q]`` counts),
    ``all_gather(tensor)`` -> stacked ``[G, ...]`` tensor of every rank's ``tensor``,
    ``merge(pairs [G,Q,2048], counts [G,Q])`` -> int32 ``[Q,2048]`` ids.
    The three are injected so that the same control flow runs with NCCL + CUDA kernels
    or, in CPU tests, with gloo + the oracle.
    """

    local, offset = shard_keys(inputs, rank, world)
    pairs, counts = local_pairs(local, offset)
    return merge(all_gather(pairs), all_gather(counts))


def dist_all_gather(tensor: Any, group: Any = None) -> Any:
    """All-gather into a stacked ``[G, ...]`` tensor (NCCL or gloo)."""

    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    out = torch.empty((world, *tensor.shape), dtype=tensor.dtype, device=tensor.device)
    dist.all_gather([out[index] for index in range(world)], tensor.contiguous(), group=group)
    return out
