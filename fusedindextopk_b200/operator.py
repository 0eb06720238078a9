"""The operator: sampled thresholds -> fused score + exact Top-K -> device-masked repair.

``fused_index_topk(q, (kv, kv_scales), weights, k_start, k_end, top_k=2048)``
returns the exact, unordered Top-K key ids of every query row as int32
``[Q,K]`` (``-1`` padded) and keeps the argument layout of
``deep_gemm.fp8_mqa_logits`` as the reference calls it
(``src/fused_index_topk/variants/common.py:19-26``).  ``Workspace`` owns every
scratch buffer, like ``FusedIndexTopK.prepare`` does in the reference
(``src/fused_index_topk/kernel/plugin.py:202-257``); the stage functions mirror
the reference's five stage closures (``kernel/plugin.py:259-380``) and only
launch kernels on the current stream: no allocation, no host synchronisation.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import Any

from . import _lib, sampling
from ._lib import FusedArgs, check, current_stream, load_library, ptr

TOP_K = _lib.TOP_K


def _require(condition: bool, message: str) -> None:
    if not condition:
        raise ValueError(message)


def validate_operator_inputs(q: Any, kv: Any, kv_scales: Any, weights: Any, k_start: Any, k_end: Any) -> tuple[int, int]:
    """Shape / dtype / layout / device contract of the six inputs; returns ``(Q, N)``.

    Same checks as the reference's host binding
    (``kernel/csrc/long_fused_bindings.cpp:119-153``).
    """

    import torch

    _require(q.is_cuda, "q must be a CUDA tensor (there is no CPU path)")
    _require(q.dim() == 3 and q.shape[1] == _lib.HEADS and q.shape[2] == _lib.HEAD_DIM,
             "q must have shape [Q, 64, 128]")
    _require(kv.dim() == 2 and kv.shape[1] == _lib.HEAD_DIM, "kv must have shape [N, 128]")
    _require(q.dtype == torch.float8_e4m3fn and kv.dtype == torch.float8_e4m3fn, "q and kv must be float8_e4m3fn")
    rows, keys = int(q.shape[0]), int(kv.shape[0])
    _require(rows > 0 and keys > 0, "Q and N must be positive")
    _require(keys <= _lib.MAX_KEYS, f"N must not exceed {_lib.MAX_KEYS}")
    _require(kv_scales.dtype == torch.float32 and tuple(kv_scales.shape) == (keys,), "kv_scales must be float32 [N]")
    _require(weights.dtype == torch.float32 and tuple(weights.shape) == (rows, _lib.HEADS),
             "weights must be float32 [Q, 64]")
    _require(k_start.dtype == torch.int32 and k_end.dtype == torch.int32, "k_start and k_end must be int32")
    _require(tuple(k_start.shape) == (rows,) and tuple(k_end.shape) == (rows,), "k_start and k_end must have shape [Q]")
    for name, tensor in (("q", q), ("kv", kv), ("kv_scales", kv_scales), ("weights", weights),
                         ("k_start", k_start), ("k_end", k_end)):
        _require(tensor.is_contiguous(), f"{name} must be contiguous")
        _require(tensor.device == q.device, f"{name} must live on the same device as q")
    return rows, keys


@dataclass
class SamplePlan:
    """Host-side decisions of the threshold prepass for one context length."""

    context_tokens: int
    sample_elements: int
    sample_rank: int
    target_candidates: int
    sample_ids: Any          # int32 [S] on the device, sorted
    enabled: bool            # False: every row has few enough keys, thresholds are -inf
    retry_rank: int = 0      # sampled rank of the lower threshold that flagged rows are retried with


# Flagged rows are retried as a compact problem of this many rows (8 query blocks; with up to 16 key
# shards each that is one wave of CTAs); rows beyond it go straight to the dense repair.
RETRY_SLOTS = 32
RETRY_TARGET_FACTOR = 2      # the retry threshold aims at this many times the first pass's candidates
CONDITIONAL_REPAIR_MIN_LAUNCHES = 9


def make_sample_plan(context_tokens: int, *, seed: int, device: Any, guard_sigmas: float = 2.0) -> SamplePlan:
    """Sample size, guarded rank and sample positions (``kernel/plugin.py:187-201``)."""

    import torch

    target = sampling.TARGET_CANDIDATES
    if context_tokens <= target:
        empty = torch.zeros(0, dtype=torch.int32, device=device)
        return SamplePlan(context_tokens, 0, 0, target, empty, False, 0)
    # Beyond the reference's longest context (163840 keys) its schedule would ask for more samples than
    # the prepass kernel keeps per row (2048); the guarded rank is valid for any sample size, so clamp.
    elements = min(sampling.production_sample_elements(context_tokens), TOP_K)
    rank = sampling.guarded_sample_rank(
        elements, context_tokens, target_candidates=target, guard_sigmas=guard_sigmas
    )
    ids = sampling.common_random_sample_ids(
        torch, context_tokens, elements, seed=sampling.sampling_seed(seed), device=device
    )
    # A row whose first threshold came out too high (fewer than 2048 keys above it) or too low (more
    # candidates than the bounded lists hold) is rerun with a threshold aimed at twice as many candidates,
    # spread over key shards with a list each.
    retry_rank = sampling.guarded_sample_rank(
        elements, context_tokens, target_candidates=min(RETRY_TARGET_FACTOR * target, context_tokens),
        guard_sigmas=guard_sigmas,
    )
    return SamplePlan(context_tokens, elements, rank, target, ids, True, retry_rank)


@dataclass
class Workspace:
    """All scratch buffers of one (Q, N) problem on one device."""

    rows: int
    keys: int
    device: Any
    plan: SamplePlan
    block_begin: int = 0
    block_stride: int = 1
    num_blocks: int = 0
    buffers: dict = field(default_factory=dict)
    # CUDA graphs of whole operator calls, keyed by the input tensors' addresses (they die with the workspace)
    graphs: dict = field(default_factory=dict)
    seen_inputs: set = field(default_factory=set)
    retry: Any = None        # RetryBuffers, or None when no row of this problem can be flagged
    split_blocks: int = 0    # owned blocks (the lowest numbered ones) whose key range is cut into shards

    def __getattr__(self, name: str) -> Any:
        buffers = self.__dict__.get("buffers", {})
        if name in buffers:
            return buffers[name]
        raise AttributeError(name)

    def check_status(self) -> None:
        """Raise if a kernel reported an expired bounded wait.  Synchronises; not for timed code."""

        value = int(self.status.item())
        if value != 0:
            raise _lib.ItkError(f"device status word is {value:#x} (bit 0: a bounded wait expired)")


def make_workspace(
    rows: int,
    keys: int,
    device: Any,
    *,
    seed: int = 0,
    guard_sigmas: float = 2.0,
    block_begin: int = 0,
    block_stride: int = 1,
    with_pairs: bool = False,
    repair: bool = True,
    key_shards: int | None = None,
    split_blocks_hint: int | None = None,
    shard_buffers: int = 0,
    second_spill: bool = False,
) -> Workspace:
    """Allocate every buffer once, outside any timed region.

    ``key_shards`` > 1 cuts the key range of ``split_blocks_hint`` query blocks (default: all of them)
    into that many work units each; ``None`` lets ``plan_key_shards`` choose both from Q, N and the SM
    count: the blocks of the last, partly filled wave of units are split so that they fill it.
    ``shard_buffers`` and ``second_spill`` serve a chunked call: shard buffers for chunks that are cut
    into more shards than the whole problem would be, and a second spill area, because the spill is
    addressed by CTA and two launches that run at the same time (on two streams) must not share it.
    """

    import torch

    load_library()
    sizes = _lib.workspace_sizes(rows, keys, 1)
    plan = make_sample_plan(keys, seed=seed, device=device, guard_sigmas=guard_sigmas)
    total_blocks = (rows + _lib.BLOCK_Q - 1) // _lib.BLOCK_Q
    owned = len(range(block_begin, total_blocks, block_stride))
    u8, i32, i64, f32 = torch.uint8, torch.int32, torch.int64, torch.float32

    def empty(shape, dtype):
        return torch.empty(shape, device=device, dtype=dtype)

    samples = max(plan.sample_elements, 1)
    buffers = {
        "output_ids": empty((rows, TOP_K), i32),
        "failure_flags": torch.zeros(rows, device=device, dtype=u8),
        "thresholds": torch.full((rows,), -math.inf, device=device, dtype=f32),
        # bounded overflow of the shared-memory lists: one region per CTA and unit row, not per query row
        "spill_pairs": empty((sizes.spill_bytes // 8,), i64),
        "sampled_kv": empty((samples, _lib.HEAD_DIM), u8),
        "sampled_scales": empty((samples,), f32),
        "status": torch.zeros(1, device=device, dtype=i32),
    }
    if with_pairs:
        buffers["output_pairs"] = empty((rows, TOP_K), i64)
        buffers["output_counts"] = torch.zeros(rows, device=device, dtype=i32)
    if repair:
        # The dense repair is the last resort behind the retry: one 16384-key chunk of pairs at a time
        # (128 KiB per row), as in the reference.
        buffers.update(
            repair_pairs=empty((rows, _lib.REPAIR_CHUNK), i64),
            accumulator_pairs=empty((rows, TOP_K), i64),
            accumulator_counts=torch.zeros(rows, device=device, dtype=i32),
            repair_error_flags=torch.zeros(rows, device=device, dtype=u8),
        )
    sm_count = torch.cuda.get_device_properties(device).multi_processor_count
    if key_shards is None:
        split_blocks, key_shards = plan_key_shards(owned, keys, sm_count)
    else:
        split_blocks = owned if key_shards > 1 else 0
        if split_blocks_hint is not None and key_shards > 1:
            split_blocks = max(1, min(owned, int(split_blocks_hint)))
    planes = max(key_shards, shard_buffers)   # a chunked call may cut single chunks into more shards than the whole
    if planes > 1:
        shard_sizes = _lib.workspace_sizes(rows, keys, planes)
        buffers.update(
            shard_pairs=empty((planes, rows, TOP_K), i64),
            shard_counts=torch.zeros((planes, rows), device=device, dtype=i32),
            shard_flags=torch.zeros((planes, rows), device=device, dtype=u8),
            shard_spill=empty((shard_sizes.spill_bytes // 8,), i64),
            merged_counts=torch.zeros(rows, device=device, dtype=i32),
        )
        if second_spill:
            buffers["shard_spill_second"] = empty((shard_sizes.spill_bytes // 8,), i64)
    if second_spill:
        buffers["spill_pairs_second"] = empty((sizes.spill_bytes // 8,), i64)
    workspace = Workspace(rows, keys, device, plan, block_begin, block_stride, owned, buffers)
    workspace.split_blocks = split_blocks if key_shards > 1 else 0
    if repair and plan.enabled:
        workspace.retry = _make_retry_buffers(rows, keys, device)
    return workspace


@dataclass
class RetryBuffers:
    """The compact problem that flagged rows are rerun as: ``RETRY_SLOTS`` rows, ``shards`` key shards."""

    shards: int
    q: Any
    weights: Any
    k_start: Any
    k_end: Any
    slot_rows: Any           # int32 [slots]: the query row in slot b, -1 for an empty slot
    thresholds: Any
    shard_pairs: Any
    shard_counts: Any
    shard_flags: Any
    spill: Any
    counts: Any              # int32 [rows]: pairs the merge wrote per query row (scratch)


def retry_key_shards(keys: int) -> int:
    """Key shards of the retry problem: units of at least 32 tiles; at least 2 (a split block returns
    pairs, which is what the merge into the operator output reads), at most 16 (8 blocks x 16 fill the SMs)."""

    tiles = (keys + 127) // 128
    return max(2, min(_lib.MAX_PAIR_SOURCES, tiles // 32))


def _make_retry_buffers(rows: int, keys: int, device: Any) -> RetryBuffers:
    import torch

    slots, shards = RETRY_SLOTS, retry_key_shards(keys)
    u8, i32, i64, f32 = torch.uint8, torch.int32, torch.int64, torch.float32
    spill_bytes = _lib.workspace_sizes(slots, keys, shards).spill_bytes

    def empty(shape, dtype):
        return torch.empty(shape, device=device, dtype=dtype)

    return RetryBuffers(
        shards=shards,
        q=torch.zeros((slots, _lib.HEADS, _lib.HEAD_DIM), device=device, dtype=u8),
        weights=torch.zeros((slots, _lib.HEADS), device=device, dtype=f32),
        k_start=torch.zeros(slots, device=device, dtype=i32),
        k_end=torch.zeros(slots, device=device, dtype=i32),
        slot_rows=torch.full((slots,), -1, device=device, dtype=i32),
        thresholds=torch.full((slots,), -math.inf, device=device, dtype=f32),
        shard_pairs=empty((shards, slots, TOP_K), i64),
        shard_counts=torch.zeros((shards, slots), device=device, dtype=i32),
        shard_flags=torch.zeros((shards, slots), device=device, dtype=u8),
        spill=empty((spill_bytes // 8,), i64),
        counts=torch.zeros(rows, device=device, dtype=i32),
    )


@dataclass(frozen=True)
class Part:
    """The query blocks one launch handles, when that is not the workspace's whole share: a row chunk of a
    pipelined call.  ``split_blocks`` of them (the first ones) are cut into ``shards`` key shards."""

    block_begin: int
    num_blocks: int
    split_blocks: int = 0
    shards: int = 1


def _launch_part(ws: "Workspace", part: Part | None) -> Part:
    if part is not None:
        return part
    shards = int(ws.shard_pairs.shape[0]) if "shard_pairs" in ws.buffers else 1
    return Part(ws.block_begin, ws.num_blocks, ws.split_blocks if shards > 1 else 0, shards)


# Cost model of one launch of the fused kernel, in microseconds (B200, measured): a 128-key tile of a unit,
# a full selection per unit, a selection that only copies (a shard that found fewer than 2048 candidates),
# the fixed cost of a unit, and the merge of a row's shard lists (one CTA per row).
_TILE_US, _SELECT_US, _COPY_US, _UNIT_US, _MERGE_ROW_US, _MERGE_LAUNCH_US = 0.70, 16.0, 4.0, 3.0, 12.0, 5.0


def plan_key_shards(query_blocks: int, keys: int, sm_count: int) -> tuple[int, int]:
    """``(split_blocks, shards)`` for a call with ``query_blocks`` blocks of 4 rows.

    The units of a launch run in waves of ``sm_count``.  The blocks of the last, partly filled wave (all
    blocks when there are fewer than SMs) can be cut into S key shards each: S times as many units of 1/S
    the length fill the wave better (128 blocks per rank of an 8-GPU run: 8 shards turn one wave of 128
    long units into 7 waves of 148 short ones; 68 left-over blocks: 2 shards make 136 half units), at the
    price of a selection per shard and of the merge launch.  The shard count with the smallest modelled
    time of that last wave is returned, ``(0, 1)`` when not splitting is best; shards have at least 4096 keys.
    """

    if query_blocks <= 0:
        return 0, 1
    tail = query_blocks % sm_count if query_blocks > sm_count else query_blocks
    if tail == 0:
        return 0, 1
    tiles = (keys + 127) // 128
    best, best_time = 1, None
    for shards in range(1, min(8, keys // 4096) + 1):
        waves = -(-tail * shards // sm_count)
        select = _SELECT_US if shards == 1 else _COPY_US
        time = waves * (_UNIT_US + tiles / shards * _TILE_US + select)
        if shards > 1:
            time += _MERGE_LAUNCH_US + -(-tail * 4 // (3 * sm_count)) * _MERGE_ROW_US
        if best_time is None or time < best_time * 0.95:   # a new count must win by 5 % to be taken
            best, best_time = shards, time
    return (tail, best) if best > 1 else (0, 1)


def auto_key_shards(query_blocks: int, keys: int, sm_count: int) -> int:
    """The shard count of ``plan_key_shards``."""

    return plan_key_shards(query_blocks, keys, sm_count)[1]


# --------------------------------------------------------------------------- stages


def _on_workspace_device(function):
    """Run a stage with the workspace's device current.

    The library sizes its grid, resolves its per-device state and launches on the current device, so a
    call for tensors on cuda:1 while cuda:0 is current would use a foreign stream handle.
    """

    import functools

    @functools.wraps(function)
    def wrapper(ws, *args, **kwargs):
        import torch

        with torch.cuda.device(ws.device):
            return function(ws, *args, **kwargs)

    return wrapper



@_on_workspace_device
def run_sample_thresholds(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, diag_logits=None,
                          trace=None, tile_table=None, only_blocks: int | None = None, part: Part | None = None,
                          gather: bool = True) -> Any:
    """Stages ``sample_gather`` + ``sample_indexer`` + ``sample_threshold`` of the reference graph.

    ``only_blocks`` limits the threshold launch to the first that many owned query blocks (0: the
    sample keys are gathered and nothing else), for calls whose other blocks take their thresholds
    inside the fused launch.  ``part`` names the query blocks of a chunked call; ``gather`` = False
    when the sample keys of this key cache are in the workspace already.
    """

    import torch

    if not ws.plan.enabled:
        ws.thresholds.fill_(-math.inf)
        return ws.thresholds
    library = load_library()
    stream = current_stream(torch, ws.device)
    plan = ws.plan
    if gather:
        check(library.itk_gather_sampled_kv_paged(
            ptr(kv), ptr(kv_scales), ptr(plan.sample_ids), ptr(tile_table), ptr(ws.sampled_kv), ptr(ws.sampled_scales),
            ws.keys, int(kv.shape[0]), plan.sample_elements, stream,
        ))
    owned = _launch_part(ws, part)
    blocks = owned.num_blocks if only_blocks is None else min(only_blocks, owned.num_blocks)
    if blocks > 0:
        check(library.itk_sample_thresholds(
            ptr(q), ptr(ws.sampled_kv), ptr(ws.sampled_scales), ptr(weights), ptr(plan.sample_ids),
            ptr(k_start), ptr(k_end), ptr(ws.thresholds), ws.rows, plan.sample_elements, plan.sample_rank,
            plan.target_candidates, owned.block_begin, ws.block_stride, blocks, 0,
            ptr(diag_logits), 0 if diag_logits is None else int(diag_logits.stride(0)),
            ptr(trace), ptr(ws.status), stream,
        ))
    return ws.thresholds


@_on_workspace_device
def run_fused_topk(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, thresholds=None,
                   diag_logits=None, trace=None, force_compute: bool = False, max_ctas: int = 0,
                   wait_limit_ns: int = 0, withhold_loads: bool = False,
                   key_lo: int = 0, key_hi: int | None = None, want_pairs: bool = False, tile_table=None,
                   thresholds_in_kernel: bool = False, part: Part | None = None, second_spill: bool = False) -> Any:
    """Stage ``fused_topk``: one launch of the persistent fused kernel.

    With ``tile_table`` (int32, one physical 128-key tile per logical tile) ``kv`` and ``kv_scales`` are
    the physical pool of a paged key cache.  With ``thresholds_in_kernel`` the whole blocks score the
    gathered sample keys themselves and write their thresholds to ``ws.thresholds``; only the rows of
    split blocks need thresholds from ``run_sample_thresholds`` then.
    """

    import torch

    args = FusedArgs()
    args.q, args.kv, args.kv_scales, args.weights = ptr(q), ptr(kv), ptr(kv_scales), ptr(weights)
    args.k_start, args.k_end = ptr(k_start), ptr(k_end)
    args.thresholds = ptr(ws.thresholds if thresholds is None else thresholds)
    args.out_ids = ptr(ws.output_ids)
    if want_pairs:
        args.out_pairs = ptr(ws.output_pairs)
        args.out_counts = ptr(ws.output_counts)
    args.failure_flags = ptr(ws.failure_flags)
    args.spill = ptr(ws.spill_pairs_second if second_spill else ws.spill_pairs)
    args.diag_logits = ptr(diag_logits)
    args.diag_stride = 0 if diag_logits is None else int(diag_logits.stride(0))
    args.trace = ptr(trace)
    args.wait_limit_ns = int(wait_limit_ns)
    args.withhold_loads = 1 if withhold_loads else 0
    args.status = ptr(ws.status)
    args.rows, args.keys = ws.rows, ws.keys
    args.key_lo = key_lo
    args.key_hi = ws.keys if key_hi is None else key_hi
    args.shards = 1
    owned = _launch_part(ws, part)
    args.block_begin, args.block_stride, args.num_blocks = owned.block_begin, ws.block_stride, owned.num_blocks
    args.force_compute = 1 if force_compute else 0
    args.max_ctas = max_ctas
    args.tile_table = ptr(tile_table)
    args.physical_keys = int(kv.shape[0]) if tile_table is not None else 0
    if thresholds_in_kernel:
        _require(thresholds is None and diag_logits is None and ws.plan.enabled,
                 "thresholds_in_kernel needs the workspace's own thresholds, a sample plan and no dense output")
        plan = ws.plan
        args.sampled_kv, args.sampled_scales = ptr(ws.sampled_kv), ptr(ws.sampled_scales)
        args.sample_ids, args.thresholds_out = ptr(plan.sample_ids), ptr(ws.thresholds)
        args.samples, args.sample_rank, args.target_candidates = plan.sample_elements, plan.sample_rank, plan.target_candidates
    sharded = owned.shards > 1 and owned.split_blocks > 0 and diag_logits is None
    if sharded:
        # the blocks of the last wave are cut into key shards: every (block, shard) is a work unit, the
        # shards share the row's threshold and return pairs, which the merge below turns into the row's ids
        _require(owned.shards <= int(ws.shard_pairs.shape[0]), "the workspace has too few shard buffers for this part")
        args.shards = owned.shards
        args.split_blocks = owned.split_blocks
        args.shard_pairs, args.shard_counts = ptr(ws.shard_pairs), ptr(ws.shard_counts)
        args.shard_flags = ptr(ws.shard_flags)
        args.spill = ptr(ws.shard_spill_second if second_spill else ws.shard_spill)
    library = load_library()
    stream = current_stream(torch, ws.device)
    check(library.itk_fused_topk(ctypes.byref(args), stream))
    if sharded:
        shards = args.shards
        pair_table = _lib.pointer_table([ws.shard_pairs[s] for s in range(shards)])
        count_table = _lib.pointer_table([ws.shard_counts[s] for s in range(shards)])
        # the merge also decides which rows are complete: no shard overflowed and the union holds
        # min(2048, valid keys) candidates; the others go to the repair graph.  The split blocks are
        # the first `split_blocks` owned ones.
        check(library.itk_merge_shard_lists(
            pair_table, count_table, shards, ptr(ws.output_ids), ptr(ws.output_pairs) if want_pairs else None,
            ptr(ws.output_counts) if want_pairs else ptr(ws.merged_counts), ws.rows,
            ptr(ws.shard_flags), ptr(ws.failure_flags), ptr(k_start), ptr(k_end), key_lo, args.key_hi,
            owned.block_begin, ws.block_stride, owned.split_blocks, None, None, stream))
    return ws.output_ids


@_on_workspace_device
def run_retry(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, key_lo: int = 0,
              key_hi: int | None = None, want_pairs: bool = False, tile_table=None, stream: int | None = None,
              mirror=None) -> Any:
    """Flagged rows once more, with a lower threshold and a candidate list per key shard.

    Four launches, all of them over the compact problem of ``RETRY_SLOTS`` rows and returning at once
    when no row is flagged: compaction of the flagged rows, their thresholds at ``plan.retry_rank``,
    the fused kernel with key shards, and the merge that writes the ids of repaired rows into the
    operator output and clears their flags.  What is still flagged afterwards goes to ``run_repair``.
    The reference has only the dense rescan (``kernel/plugin.py:333-377``).
    """

    import torch

    retry, plan = ws.retry, ws.plan
    if retry is None:
        return ws.output_ids
    library = load_library()
    if stream is None:
        stream = current_stream(torch, ws.device)
    slots = int(retry.slot_rows.shape[0])
    key_hi = ws.keys if key_hi is None else key_hi
    check(library.itk_compact_flagged_rows(
        ptr(ws.failure_flags), ptr(q), ptr(weights), ptr(k_start), ptr(k_end), ws.rows, slots,
        ptr(retry.q), ptr(retry.weights), ptr(retry.k_start), ptr(retry.k_end), ptr(retry.slot_rows), stream,
    ))
    blocks = slots // _lib.BLOCK_Q
    check(library.itk_sample_thresholds(
        ptr(retry.q), ptr(ws.sampled_kv), ptr(ws.sampled_scales), ptr(retry.weights), ptr(plan.sample_ids),
        ptr(retry.k_start), ptr(retry.k_end), ptr(retry.thresholds), slots, plan.sample_elements, plan.retry_rank,
        plan.target_candidates, 0, 1, blocks, 1, None, 0, None, ptr(ws.status), stream,
    ))
    args = FusedArgs()
    args.q, args.kv, args.kv_scales, args.weights = ptr(retry.q), ptr(kv), ptr(kv_scales), ptr(retry.weights)
    args.k_start, args.k_end = ptr(retry.k_start), ptr(retry.k_end)
    args.thresholds = ptr(retry.thresholds)
    args.shard_pairs, args.shard_counts = ptr(retry.shard_pairs), ptr(retry.shard_counts)
    args.shard_flags, args.spill = ptr(retry.shard_flags), ptr(retry.spill)
    args.status = ptr(ws.status)
    args.rows, args.keys = slots, ws.keys
    args.key_lo, args.key_hi = key_lo, key_hi
    args.shards = retry.shards
    args.split_blocks = blocks
    args.block_begin, args.block_stride, args.num_blocks = 0, 1, blocks
    args.exit_when_no_keys = 1
    args.tile_table = ptr(tile_table)
    args.physical_keys = int(kv.shape[0]) if tile_table is not None else 0
    check(library.itk_fused_topk(ctypes.byref(args), stream))
    pair_table = _lib.pointer_table([retry.shard_pairs[s] for s in range(retry.shards)])
    count_table = _lib.pointer_table([retry.shard_counts[s] for s in range(retry.shards)])
    check(library.itk_merge_shard_lists(
        pair_table, count_table, retry.shards, ptr(ws.output_ids), ptr(ws.output_pairs) if want_pairs else None,
        ptr(ws.output_counts) if want_pairs else ptr(retry.counts), slots,
        ptr(retry.shard_flags), ptr(ws.failure_flags), ptr(retry.k_start), ptr(retry.k_end), key_lo, key_hi,
        0, 1, 0, ptr(retry.slot_rows), ptr(mirror), stream))
    return ws.output_ids


@_on_workspace_device
def run_repair(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, key_lo: int = 0,
               key_hi: int | None = None, want_pairs: bool = False, tile_table=None, retry: bool = True,
               mirror=None) -> Any:
    """Stage ``hierarchical_repair``: always launched, masked on the device by the failure flags.

    First the retry of the flagged rows (``run_retry``), then, for what is still flagged, the dense
    rescan: per 16384-key chunk one launch of the dense producer and one that selects the chunk's pairs
    into the running Top-2048 of each flagged row (the last one writes the ids and clears the flags).
    ``mirror`` (int32 ``[Q, 2048]``, e.g. the pinned host buffer the fast path's ids were copied to
    already) receives a second copy of the ids of every repaired row.
    """

    import torch

    library = load_library()
    outer = current_stream(torch, ws.device)
    key_hi = ws.keys if key_hi is None else key_hi
    physical_keys = int(kv.shape[0]) if tile_table is not None else 0
    chunks = [(lo, min(ws.keys, lo + _lib.REPAIR_CHUNK)) for lo in range(0, ws.keys, _lib.REPAIR_CHUNK)]
    chunks = [(lo, hi) for lo, hi in chunks if hi > key_lo and lo < key_hi]
    # Inside a graph capture the whole stage can be the body of an IF node on "some row is flagged".  A replay
    # without flagged rows then pays for the node (about 13 us) instead of about 1.5 us per launch that
    # returns at once, which is the better deal from nine launches on (contexts beyond 32 K keys).
    launches = (4 if retry and ws.retry is not None else 0) + 2 * len(chunks)
    body = ctypes.c_void_p(outer)
    if launches >= CONDITIONAL_REPAIR_MIN_LAUNCHES:
        check(library.itk_flagged_scope_begin(ptr(ws.failure_flags), ws.rows, outer, ctypes.byref(body)))
    stream = body.value
    try:
        if retry:
            run_retry(ws, q, kv, kv_scales, weights, k_start, k_end, key_lo=key_lo, key_hi=key_hi,
                      want_pairs=want_pairs, tile_table=tile_table, stream=stream, mirror=mirror)
        for index, (chunk_lo, chunk_hi) in enumerate(chunks):
            check(library.itk_repair_produce_paged(
                ptr(q), ptr(kv), ptr(kv_scales), ptr(weights), ptr(k_start), ptr(k_end), ptr(ws.failure_flags),
                ptr(ws.repair_pairs), ws.rows, ws.keys, chunk_lo, chunk_hi, ws.block_begin, ws.block_stride,
                ws.num_blocks, ptr(tile_table), physical_keys, ptr(ws.status), stream,
            ))
            last = index == len(chunks) - 1
            check(library.itk_repair_merge_chunk(
                ptr(ws.accumulator_pairs), ptr(ws.accumulator_counts), ptr(ws.repair_pairs), ptr(k_start), ptr(k_end),
                chunk_lo, chunk_hi, ptr(ws.failure_flags), ptr(ws.repair_error_flags), ws.rows,
                1 if index == 0 else 0, 1 if last else 0, ptr(ws.output_ids),
                ptr(ws.output_pairs) if want_pairs else None, ptr(ws.output_counts) if want_pairs else None,
                ptr(mirror), stream,
            ))
    finally:
        check(library.itk_flagged_scope_end(outer, stream))
    return ws.output_ids


# Up to this many sample keys the threshold of a row is picked by one warp, which is cheap enough to do
# inside the fused launch (four sample tiles in front of a block's own keys): contexts up to 32 K keys.
IN_KERNEL_THRESHOLD_SAMPLES = 512


def run_operator(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, tile_table=None,
                 part: Part | None = None, gather: bool = True, repair: bool = True, second_spill: bool = False) -> Any:
    """Sampling + fused kernel + repair on the current stream; returns ``ws.output_ids``.

    ``part``, ``gather`` and ``repair`` serve a chunked call (``HostPipeline``): the fast path of one
    range of query blocks, with the sample keys gathered once and the repair stage run once at the end.
    """

    in_kernel = ws.plan.enabled and ws.plan.sample_elements <= IN_KERNEL_THRESHOLD_SAMPLES
    owned = _launch_part(ws, part)
    # the separate threshold launch serves the rows of split blocks (all rows when the fused launch does not sample)
    run_sample_thresholds(ws, q, kv, kv_scales, weights, k_start, k_end, tile_table=tile_table, part=part, gather=gather,
                          only_blocks=(owned.split_blocks if owned.shards > 1 else 0) if in_kernel else None)
    run_fused_topk(ws, q, kv, kv_scales, weights, k_start, k_end, tile_table=tile_table, thresholds_in_kernel=in_kernel,
                   part=part, second_spill=second_spill)
    if repair and "repair_pairs" in ws.buffers:
        run_repair(ws, q, kv, kv_scales, weights, k_start, k_end, tile_table=tile_table)
    return ws.output_ids


_WORKSPACES: dict[tuple, Workspace] = {}


def fused_index_topk(q, kv_pair, weights, k_start, k_end, top_k: int = TOP_K, *, workspace: Workspace | None = None,
                     seed: int = 0, use_graph: bool = True) -> Any:
    """Exact unordered Top-K key ids per query row, int32 ``[Q, K]``, ``-1`` padded.

    ``kv_pair`` is ``(kv, kv_scales)``.  Without ``workspace`` one is cached per
    (Q, N, device, seed); the returned tensor is that workspace's output buffer
    and is overwritten by the next call with the same key.  From the second call with the
    same tensors (same storage) and workspace on, the launches of the call are replayed as one
    CUDA graph: a long context has dozens of small repair launches whose host-side cost
    would otherwise exceed the kernels' time on calls with few query rows.
    """

    kv, kv_scales = kv_pair
    _require(top_k == TOP_K, f"top_k must be {TOP_K}")
    rows, keys = validate_operator_inputs(q, kv, kv_scales, weights, k_start, k_end)
    if workspace is None:
        key = (rows, keys, str(q.device), int(seed))
        workspace = _WORKSPACES.get(key)
        if workspace is None:
            workspace = make_workspace(rows, keys, q.device, seed=seed)
            _WORKSPACES[key] = workspace
    _require(workspace.rows == rows and workspace.keys == keys, "workspace was made for a different problem size")
    return replay_or_run(workspace, (q, kv, kv_scales, weights, k_start, k_end), use_graph=use_graph)


@_on_workspace_device
def replay_or_run(workspace: Workspace, tensors, *, tile_table=None, use_graph: bool = True, prologue=None,
                  key_extra: tuple = ()) -> Any:
    """One operator call: a graph replay from the second call with the same tensor addresses on.

    ``prologue`` (optional callable) is enqueued in front of the operator and is part of the replayed
    graph: device-side preparation that has to be redone on every call (the paged variant expands the
    live block table there); ``key_extra`` are the addresses it reads.
    """

    import torch

    if use_graph and not torch.cuda.is_current_stream_capturing():
        key = tuple(int(tensor.data_ptr()) for tensor in tensors) + tuple(key_extra)
        if tile_table is not None:
            key += (int(tile_table.data_ptr()),)
        graph = workspace.graphs.get(key)
        if graph is None and key in workspace.seen_inputs and len(workspace.graphs) < 4:
            graph = _capture_operator(workspace, tensors, tile_table, prologue)
            if graph is not None:
                workspace.graphs[key] = graph
        if len(workspace.seen_inputs) < 64:
            workspace.seen_inputs.add(key)
        if graph is not None:
            graph.replay()
            return workspace.output_ids
    if prologue is not None:
        prologue()
    return run_operator(workspace, *tensors, tile_table=tile_table)


def _capture_operator(workspace: Workspace, tensors, tile_table=None, prologue=None) -> Any:
    """One operator call as a CUDA graph, or None when the capture fails (the caller launches directly)."""

    import torch

    graph = torch.cuda.CUDAGraph()
    try:
        torch.cuda.synchronize(workspace.device)
        with torch.cuda.graph(graph):
            if prologue is not None:
                prologue()
            run_operator(workspace, *tensors, tile_table=tile_table)
        return graph
    except _lib.ItkError:
        raise   # an argument or launch error of the library is not a capture problem
    except RuntimeError as error:
        # stream capture refused (e.g. another capture is active on the device): launch directly
        _warn_once(f"CUDA graph capture of the operator failed, launching directly: {error}")
        torch.cuda.synchronize(workspace.device)
        return None


_WARNED: set[str] = set()


def _warn_once(message: str) -> None:
    import warnings

    key = message.split(":")[0]
    if key not in _WARNED:
        _WARNED.add(key)
        warnings.warn(message, RuntimeWarning, stacklevel=3)


# --------------------------------------------------------------------------- host buffers


class HostPipeline:
    """The operator for callers whose tensors live in pinned host memory.

    Query rows are independent, so the call is cut into row chunks that flow through four streams:
    the host-to-device copy of chunk c+1, the fast path (thresholds + fused kernel) of chunk c and
    the device-to-host copy of the ids of chunk c-1 overlap (the PCIe link is full duplex and the
    copy engines run beside the SMs).  Keys, scales and the small per-row tensors are copied once,
    ahead of the first chunk, and the sample keys are gathered once.  All chunks share one workspace;
    a chunk is a range of its query blocks.  Consecutive chunks alternate between two compute
    streams, so that the CTAs of chunk c+1 start on the SMs that the shorter units of chunk c have
    left.  The repair stage runs once, after the last chunk: it writes the ids of repaired rows
    into the device output and, through the mapping of the pinned buffer, straight into ``out``
    (their stale fast-path ids were copied there before), so no second copy of the output is needed.
    Everything is allocated here, nothing per call, and repeated calls with the same host tensors
    replay one CUDA graph.
    """

    UNIT_BLOCKS = 148                     # one wave of work units
    EDGE_BLOCKS = 37                      # a quarter wave: the first and the last chunk of a long call
    UNIT_ROWS = UNIT_BLOCKS * _lib.BLOCK_Q
    EDGE_ROWS = EDGE_BLOCKS * _lib.BLOCK_Q

    def __init__(self, rows: int, keys: int, device: Any, *, chunk_units: int = 1, seed: int = 0,
                 use_graph: bool = True):
        import torch

        # From the second call with the same host tensors on, the whole pipeline (some forty copies
        # and launches on four streams) is replayed as one CUDA graph.
        self.use_graph = use_graph
        self._graphs: dict[tuple, Any] = {}
        self._seen: set[tuple] = set()

        self.rows, self.keys, self.device = rows, keys, device
        self.bounds = self.chunk_bounds(rows, chunk_units)
        sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.parts = []
        for lo, hi in self.bounds:
            blocks = (hi - lo + _lib.BLOCK_Q - 1) // _lib.BLOCK_Q
            split, shards = plan_key_shards(blocks, keys, sm_count)
            self.parts.append(Part(lo // _lib.BLOCK_Q, blocks, split, shards))
        f8, i32, f32 = torch.float8_e4m3fn, torch.int32, torch.float32
        self.q = torch.empty((rows, _lib.HEADS, _lib.HEAD_DIM), device=device, dtype=f8)
        self.kv = torch.empty((keys, _lib.HEAD_DIM), device=device, dtype=f8)
        self.kv_scales = torch.empty((keys,), device=device, dtype=f32)
        self.weights = torch.empty((rows, _lib.HEADS), device=device, dtype=f32)
        self.k_start = torch.empty((rows,), device=device, dtype=i32)
        self.k_end = torch.empty((rows,), device=device, dtype=i32)
        self.workspace = make_workspace(rows, keys, device, seed=seed, key_shards=1, second_spill=True,
                                        shard_buffers=max(part.shards for part in self.parts))
        self.copy_in = torch.cuda.Stream(device=device)
        self.compute = (torch.cuda.Stream(device=device), torch.cuda.Stream(device=device))
        self.copy_out = torch.cuda.Stream(device=device)

    @classmethod
    def chunk_bounds(cls, rows: int, chunk_units: int = 1) -> list[tuple[int, int]]:
        """Row ranges of the chunks (every boundary a multiple of 4 rows, the block of a work unit).

        The copies into the device are what bounds a long call, so what counts is how soon the first
        kernel can start and how little is left to do after the last copy: a call of more than two
        waves begins and ends with a chunk of 148 rows (a quarter wave of units; the planner cuts their
        key ranges into shards, so that they still use every SM), with whole multiples of 148 work
        units (592 rows) and one remainder chunk between them.  Shorter calls are one remainder chunk
        followed by whole waves.
        """

        if rows <= 0:
            raise ValueError("rows must be positive")
        blocks = (rows + _lib.BLOCK_Q - 1) // _lib.BLOCK_Q
        step = max(1, chunk_units) * cls.UNIT_BLOCKS
        if blocks > 2 * step + 2 * cls.EDGE_BLOCKS:
            middle = blocks - 2 * cls.EDGE_BLOCKS
            sizes = [cls.EDGE_BLOCKS] + [step] * (middle // step) + ([middle % step] if middle % step else []) + [cls.EDGE_BLOCKS]
        else:
            first = blocks % step or min(blocks, step)
            sizes = [first] + [step] * ((blocks - first) // step)
        bounds, begin = [], 0
        for size in sizes:
            bounds.append((begin * _lib.BLOCK_Q, min(rows, (begin + size) * _lib.BLOCK_Q)))
            begin += size
        return bounds

    def __call__(self, q, kv_pair, weights, k_start, k_end, out) -> Any:
        """All arguments are pinned host tensors; ``out`` is int32 ``[Q, 2048]`` and is returned.

        The copies and kernels are ordered after the work already queued on the caller's current
        stream, and that stream waits for the last write into ``out``.
        """

        import torch

        kv, kv_scales = kv_pair
        for tensor in (q, kv, kv_scales, weights, k_start, k_end, out):
            _require(not tensor.is_cuda and tensor.is_pinned() and tensor.is_contiguous(),
                     "HostPipeline takes contiguous pinned host tensors")
        _require(tuple(q.shape) == (self.rows, _lib.HEADS, _lib.HEAD_DIM) and q.dtype == torch.float8_e4m3fn,
                 "q must be float8_e4m3fn [Q, 64, 128]")
        _require(tuple(kv.shape) == (self.keys, _lib.HEAD_DIM) and kv.dtype == torch.float8_e4m3fn,
                 "kv must be float8_e4m3fn [N, 128]")
        _require(tuple(kv_scales.shape) == (self.keys,) and kv_scales.dtype == torch.float32, "kv_scales must be float32 [N]")
        _require(tuple(weights.shape) == (self.rows, _lib.HEADS) and weights.dtype == torch.float32,
                 "weights must be float32 [Q, 64]")
        _require(tuple(k_start.shape) == (self.rows,) and tuple(k_end.shape) == (self.rows,)
                 and k_start.dtype == torch.int32 and k_end.dtype == torch.int32, "k_start and k_end must be int32 [Q]")
        _require(tuple(out.shape) == (self.rows, TOP_K) and out.dtype == torch.int32, "out must be int32 [Q, 2048]")
        tensors = (q, kv, kv_scales, weights, k_start, k_end, out)
        with torch.cuda.device(self.device):
            return self._run(tensors)

    def _run(self, tensors) -> Any:
        out = tensors[-1]
        if self.use_graph:
            key = tuple(int(tensor.data_ptr()) for tensor in tensors)
            graph = self._graphs.get(key)
            if graph is None and key in self._seen and len(self._graphs) < 4:
                graph = self._capture(tensors)
                if graph is not None:
                    self._graphs[key] = graph
            self._seen.add(key)
            if graph is not None:
                graph.replay()
                return out
        self._enqueue(tensors)
        return out

    def _capture(self, tensors) -> Any:
        """The pipeline as a CUDA graph, or None (graphs are then switched off) when capture fails."""

        import torch

        graph = torch.cuda.CUDAGraph()
        try:
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(graph):
                self._enqueue(tensors)
            return graph
        except _lib.ItkError:
            raise
        except RuntimeError as error:
            _warn_once(f"CUDA graph capture of the host pipeline failed, using the stream version: {error}")
            self.use_graph = False
            torch.cuda.synchronize(self.device)
            return None

    def _enqueue(self, tensors) -> None:
        import torch

        q, kv, kv_scales, weights, k_start, k_end, out = tensors
        ws = self.workspace
        device_tensors = (self.q, self.kv, self.kv_scales, self.weights, self.k_start, self.k_end)
        caller = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(caller)
        for stream in (self.copy_in, *self.compute, self.copy_out):
            stream.wait_event(start)
        with torch.cuda.stream(self.copy_in):
            self.kv.copy_(kv, non_blocking=True)
            self.kv_scales.copy_(kv_scales, non_blocking=True)
            # a megabyte of weights and ranges in three copies, not three small copies per chunk
            self.weights.copy_(weights, non_blocking=True)
            self.k_start.copy_(k_start, non_blocking=True)
            self.k_end.copy_(k_end, non_blocking=True)
        gathered = torch.cuda.Event()
        scored = None
        for index, ((lo, hi), part) in enumerate(zip(self.bounds, self.parts)):
            arrived, scored = torch.cuda.Event(), torch.cuda.Event()
            compute = self.compute[index % 2]
            with torch.cuda.stream(self.copy_in):
                self.q[lo:hi].copy_(q[lo:hi], non_blocking=True)
                arrived.record(self.copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(arrived)
                if index == 1:
                    compute.wait_event(gathered)    # the other compute stream gathered the sample keys
                run_operator(ws, *device_tensors, part=part, gather=index == 0, repair=False,
                             second_spill=index % 2 == 1)
                if index == 0:
                    gathered.record(compute)
                scored.record(compute)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(scored)
                out[lo:hi].copy_(ws.output_ids[lo:hi], non_blocking=True)
        copied = torch.cuda.Event()
        copied.record(self.copy_out)
        # The repair stage, once for all rows, after every fast-path id has reached `out`: what it repairs
        # it writes to the device output and, through the mapped pinned buffer, over the stale ids in `out`.
        closing, other = self.compute[(len(self.bounds) - 1) % 2], self.compute[len(self.bounds) % 2]
        joined = torch.cuda.Event()
        joined.record(other)
        with torch.cuda.stream(closing):
            closing.wait_event(copied)
            closing.wait_event(joined)
            if "repair_pairs" in ws.buffers:
                run_repair(ws, *device_tensors, mirror=out)
            done = torch.cuda.Event()
            done.record(closing)
        caller.wait_event(done)

    def check_status(self) -> None:
        self.workspace.check_status()


_HOST_PIPELINES: dict[tuple, HostPipeline] = {}


def fused_index_topk_host(q, kv_pair, weights, k_start, k_end, out, *, device: Any = None, seed: int = 0) -> Any:
    """``fused_index_topk`` for pinned host tensors: chunked copies overlapped with the kernels.

    Returns ``out`` (pinned int32 ``[Q, 2048]``); the caller's current stream is ordered after the last
    copy, so synchronise that stream before reading ``out``.  One pipeline (device staging and
    workspaces) is cached per (Q, N, device, seed).
    """

    import torch

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    rows, keys = int(q.shape[0]), int(kv_pair[0].shape[0])
    key = (rows, keys, str(device), int(seed))
    pipeline = _HOST_PIPELINES.get(key)
    if pipeline is None:
        pipeline = HostPipeline(rows, keys, device, seed=seed)
        _HOST_PIPELINES[key] = pipeline
    return pipeline(q, kv_pair, weights, k_start, k_end, out)
