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


REPAIR_ALL_CHUNKS_BYTES_LIMIT = 16 << 30


def make_sample_plan(context_tokens: int, *, seed: int, device: Any, guard_sigmas: float = 2.0) -> SamplePlan:
    """Sample size, guarded rank and sample positions (``kernel/plugin.py:187-201``)."""

    import torch

    target = sampling.TARGET_CANDIDATES
    if context_tokens <= target:
        empty = torch.zeros(0, dtype=torch.int32, device=device)
        return SamplePlan(context_tokens, 0, 0, target, empty, False)
    # Beyond the reference's longest context (163840 keys) its schedule would ask for more samples than
    # the prepass kernel keeps per row (2048); the guarded rank is valid for any sample size, so clamp.
    elements = min(sampling.production_sample_elements(context_tokens), TOP_K)
    rank = sampling.guarded_sample_rank(
        elements, context_tokens, target_candidates=target, guard_sigmas=guard_sigmas
    )
    ids = sampling.common_random_sample_ids(
        torch, context_tokens, elements, seed=sampling.sampling_seed(seed), device=device
    )
    return SamplePlan(context_tokens, elements, rank, target, ids, True)


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
) -> Workspace:
    """Allocate every buffer once, outside any timed region.

    ``key_shards`` > 1 cuts every query block's key range into that many work units (for calls with
    too few query blocks to fill the GPU); ``None`` chooses it from Q, N and the SM count.
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
        "spill_pairs": empty((rows, _lib.SPILL_U64_PER_ROW), i64),
        "sampled_kv": empty((samples, _lib.HEAD_DIM), u8),
        "sampled_scales": empty((samples,), f32),
        "status": torch.zeros(1, device=device, dtype=i32),
    }
    assert buffers["spill_pairs"].numel() * 8 == sizes.spill_bytes
    if with_pairs:
        buffers["output_pairs"] = empty((rows, TOP_K), i64)
        buffers["output_counts"] = torch.zeros(rows, device=device, dtype=i32)
    if repair:
        chunks = sizes.repair_chunks
        # One buffer per chunk lets a single launch rescan all chunks of the flagged rows on different SMs
        # (a flagged row of a 160 K context otherwise keeps one SM busy for a whole pass over the context);
        # 512 MiB per chunk at 4096 rows, which a 180 GB device affords.  Very large problems keep the
        # one-chunk buffer and the chunk-by-chunk launches.
        all_chunks_bytes = chunks * rows * _lib.REPAIR_CHUNK * 8
        parallel_chunks = chunks > 1 and all_chunks_bytes <= REPAIR_ALL_CHUNKS_BYTES_LIMIT
        buffers.update(
            repair_pairs=empty((chunks, rows, _lib.REPAIR_CHUNK) if parallel_chunks else (rows, _lib.REPAIR_CHUNK), i64),
            local_pairs=empty((chunks, rows, TOP_K) if parallel_chunks else (rows, TOP_K), i64),
            local_counts=torch.zeros((chunks, rows) if parallel_chunks else (rows,), device=device, dtype=i32),
            accumulator_pairs=empty((rows, TOP_K), i64),
            accumulator_counts=torch.zeros(rows, device=device, dtype=i32),
            repair_error_flags=torch.zeros(rows, device=device, dtype=u8),
            chunk_starts=empty((chunks, rows), i32),
            chunk_ends=empty((chunks, rows), i32),
        )
    if key_shards is None:
        key_shards = auto_key_shards(owned, keys, torch.cuda.get_device_properties(device).multi_processor_count)
    if key_shards > 1:
        shard_sizes = _lib.workspace_sizes(rows, keys, key_shards)
        buffers.update(
            shard_pairs=empty((key_shards, rows, TOP_K), i64),
            shard_counts=torch.zeros((key_shards, rows), device=device, dtype=i32),
            shard_flags=torch.zeros((key_shards, rows), device=device, dtype=u8),
            shard_spill=empty((key_shards * rows, _lib.SPILL_U64_PER_ROW), i64),
            merged_counts=torch.zeros(rows, device=device, dtype=i32),
        )
        assert buffers["shard_spill"].numel() * 8 == shard_sizes.spill_bytes
    return Workspace(rows, keys, device, plan, block_begin, block_stride, owned, buffers)


def auto_key_shards(query_blocks: int, keys: int, sm_count: int) -> int:
    """Key-range shards per query block for a call with ``query_blocks`` blocks of 4 rows.

    One shard while the blocks alone fill half the SMs; otherwise as many shards as fit the SMs,
    at most 8 (the merge kernel's source limit) and with at least 4096 keys per shard.
    """

    if query_blocks <= 0 or 2 * query_blocks > sm_count:
        return 1
    return max(1, min(_lib.MAX_PAIR_SOURCES, sm_count // query_blocks, keys // 4096))


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
                          trace=None, tile_table=None) -> Any:
    """Stages ``sample_gather`` + ``sample_indexer`` + ``sample_threshold`` of the reference graph."""

    import torch

    if not ws.plan.enabled:
        ws.thresholds.fill_(-math.inf)
        return ws.thresholds
    library = load_library()
    stream = current_stream(torch, ws.device)
    plan = ws.plan
    check(library.itk_gather_sampled_kv_paged(
        ptr(kv), ptr(kv_scales), ptr(plan.sample_ids), ptr(tile_table), ptr(ws.sampled_kv), ptr(ws.sampled_scales),
        ws.keys, int(kv.shape[0]), plan.sample_elements, stream,
    ))
    check(library.itk_sample_thresholds(
        ptr(q), ptr(ws.sampled_kv), ptr(ws.sampled_scales), ptr(weights), ptr(plan.sample_ids),
        ptr(k_start), ptr(k_end), ptr(ws.thresholds), ws.rows, plan.sample_elements, plan.sample_rank,
        plan.target_candidates, ptr(diag_logits), 0 if diag_logits is None else int(diag_logits.stride(0)),
        ptr(trace), ptr(ws.status), stream,
    ))
    return ws.thresholds


@_on_workspace_device
def run_fused_topk(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, thresholds=None,
                   diag_logits=None, trace=None, force_compute: bool = False, max_ctas: int = 0,
                   wait_limit_ns: int = 0, withhold_loads: bool = False,
                   key_lo: int = 0, key_hi: int | None = None, want_pairs: bool = False, tile_table=None) -> Any:
    """Stage ``fused_topk``: one launch of the persistent fused kernel.

    With ``tile_table`` (int32, one physical 128-key tile per logical tile) ``kv`` and ``kv_scales`` are
    the physical pool of a paged key cache.
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
    args.spill = ptr(ws.spill_pairs)
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
    args.block_begin, args.block_stride, args.num_blocks = ws.block_begin, ws.block_stride, ws.num_blocks
    args.force_compute = 1 if force_compute else 0
    args.max_ctas = max_ctas
    args.tile_table = ptr(tile_table)
    args.physical_keys = int(kv.shape[0]) if tile_table is not None else 0
    sharded = "shard_pairs" in ws.buffers and diag_logits is None
    if sharded:
        # every (query block, key shard) is a work unit; the shards share the row's threshold and
        # return pairs, which the merge below turns into the row's ids
        args.shards = int(ws.shard_pairs.shape[0])
        args.thresholds_per_row = 1
        args.out_ids = None
        args.out_pairs, args.out_counts = ptr(ws.shard_pairs), ptr(ws.shard_counts)
        args.failure_flags, args.spill = ptr(ws.shard_flags), ptr(ws.shard_spill)
    library = load_library()
    stream = current_stream(torch, ws.device)
    check(library.itk_fused_topk(ctypes.byref(args), stream))
    if sharded:
        shards = args.shards
        pair_table = _lib.pointer_table([ws.shard_pairs[s] for s in range(shards)])
        count_table = _lib.pointer_table([ws.shard_counts[s] for s in range(shards)])
        # the merge also decides which rows are complete: no shard overflowed and the union holds
        # min(2048, valid keys) candidates; the others go to the repair graph
        check(library.itk_merge_shard_lists(
            pair_table, count_table, shards, ptr(ws.output_ids), ptr(ws.output_pairs) if want_pairs else None,
            ptr(ws.output_counts) if want_pairs else ptr(ws.merged_counts), ws.rows,
            ptr(ws.shard_flags), ptr(ws.failure_flags), ptr(k_start), ptr(k_end), key_lo, args.key_hi, stream))
    return ws.output_ids


@_on_workspace_device
def run_repair(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, key_lo: int = 0,
               key_hi: int | None = None, want_pairs: bool = False, tile_table=None) -> Any:
    """Stage ``hierarchical_repair``: always launched, masked on the device by the failure flags."""

    import torch

    library = load_library()
    stream = current_stream(torch, ws.device)
    key_hi = ws.keys if key_hi is None else key_hi
    check(library.itk_update_chunk_ranges(
        ptr(k_start), ptr(k_end), ptr(ws.chunk_starts), ptr(ws.chunk_ends), ws.rows, ws.keys, stream
    ))
    physical_keys = int(kv.shape[0]) if tile_table is not None else 0
    all_chunks = ws.repair_pairs.dim() == 3 and key_lo == 0 and key_hi == ws.keys
    if all_chunks:
        check(library.itk_repair_produce_all(
            ptr(q), ptr(kv), ptr(kv_scales), ptr(weights), ptr(k_start), ptr(k_end), ptr(ws.failure_flags),
            ptr(ws.repair_pairs), ws.rows, ws.keys, ws.block_begin, ws.block_stride, ws.num_blocks,
            ptr(tile_table), physical_keys, ptr(ws.status), stream,
        ))
        chunks = int(ws.repair_pairs.shape[0])
        check(library.itk_chunk_local_topk_all(
            ptr(ws.repair_pairs), ptr(ws.chunk_starts), ptr(ws.chunk_ends), ptr(ws.failure_flags),
            ptr(ws.local_pairs), ptr(ws.local_counts), ptr(ws.repair_error_flags), ws.rows, chunks, stream,
        ))
        check(library.itk_merge_local_lists(
            ptr(ws.local_pairs), ptr(ws.local_counts), chunks, ptr(ws.accumulator_pairs),
            ptr(ws.accumulator_counts), ptr(ws.failure_flags), ptr(ws.repair_error_flags), ws.rows, stream,
        ))
    first = True
    for chunk_index, chunk_lo in enumerate(range(0, ws.keys, _lib.REPAIR_CHUNK)):
        chunk_hi = min(ws.keys, chunk_lo + _lib.REPAIR_CHUNK)
        if all_chunks or chunk_hi <= key_lo or chunk_lo >= key_hi:
            continue
        chunk_pairs = ws.repair_pairs[0] if ws.repair_pairs.dim() == 3 else ws.repair_pairs
        local_pairs = ws.local_pairs[0] if ws.local_pairs.dim() == 3 else ws.local_pairs
        local_counts = ws.local_counts[0] if ws.local_counts.dim() == 2 else ws.local_counts
        check(library.itk_repair_produce_paged(
            ptr(q), ptr(kv), ptr(kv_scales), ptr(weights), ptr(k_start), ptr(k_end), ptr(ws.failure_flags),
            ptr(chunk_pairs), ws.rows, ws.keys, chunk_lo, chunk_hi, ws.block_begin, ws.block_stride,
            ws.num_blocks, ptr(tile_table), physical_keys, ptr(ws.status), stream,
        ))
        check(library.itk_chunk_local_topk(
            ptr(chunk_pairs), ptr(ws.chunk_starts[chunk_index]), ptr(ws.chunk_ends[chunk_index]),
            ptr(ws.failure_flags), ptr(local_pairs), ptr(local_counts), ptr(ws.repair_error_flags),
            ws.rows, 1 if first else 0, stream,
        ))
        check(library.itk_merge_topk_pairs(
            ptr(ws.accumulator_pairs), ptr(ws.accumulator_counts), ptr(local_pairs), ptr(local_counts),
            ptr(ws.failure_flags), ptr(ws.repair_error_flags), ws.rows, 1 if first else 0, stream,
        ))
        first = False
    check(library.itk_finalize_repair(
        ptr(ws.accumulator_pairs), ptr(ws.accumulator_counts), ptr(ws.output_ids),
        ptr(ws.output_pairs) if want_pairs else None, ptr(ws.output_counts) if want_pairs else None,
        ptr(ws.failure_flags), ptr(ws.repair_error_flags), ws.rows, stream,
    ))
    return ws.output_ids


def run_operator(ws: Workspace, q, kv, kv_scales, weights, k_start, k_end, *, tile_table=None) -> Any:
    """Sampling + fused kernel + repair on the current stream; returns ``ws.output_ids``."""

    run_sample_thresholds(ws, q, kv, kv_scales, weights, k_start, k_end, tile_table=tile_table)
    run_fused_topk(ws, q, kv, kv_scales, weights, k_start, k_end, tile_table=tile_table)
    if "repair_pairs" in ws.buffers:
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

    Query rows are independent, so the call is cut into a few row chunks that flow through three
    streams: host-to-device copies of chunk c+1, the operator on chunk c and the device-to-host
    copy of the ids of chunk c-1 overlap (the PCIe link is full duplex and the copy engines run
    beside the SMs).  Keys and scales are copied once, ahead of the first chunk.  Chunks are whole
    multiples of 148 work units (592 rows) where the row count allows, so that every chunk fills
    the persistent kernel's CTAs evenly; the short chunk goes first, which also shortens the
    time before the first kernel can start.  Everything is allocated here, nothing per call, and
    repeated calls with the same host tensors replay one CUDA graph.
    """

    UNIT_ROWS = 148 * _lib.BLOCK_Q

    def __init__(self, rows: int, keys: int, device: Any, *, chunk_units: int = 1, seed: int = 0,
                 use_graph: bool = True):
        import torch

        # From the second call with the same host tensors on, the whole pipeline (some sixty copies
        # and launches on three streams) is replayed as one CUDA graph.
        self.use_graph = use_graph
        self._graphs: dict[tuple, Any] = {}
        self._seen: set[tuple] = set()

        self.rows, self.keys, self.device = rows, keys, device
        self.bounds = self.chunk_bounds(rows, chunk_units)
        f8, i32, f32 = torch.float8_e4m3fn, torch.int32, torch.float32
        self.q = torch.empty((rows, _lib.HEADS, _lib.HEAD_DIM), device=device, dtype=f8)
        self.kv = torch.empty((keys, _lib.HEAD_DIM), device=device, dtype=f8)
        self.kv_scales = torch.empty((keys,), device=device, dtype=f32)
        self.weights = torch.empty((rows, _lib.HEADS), device=device, dtype=f32)
        self.k_start = torch.empty((rows,), device=device, dtype=i32)
        self.k_end = torch.empty((rows,), device=device, dtype=i32)
        self.workspaces = [make_workspace(hi - lo, keys, device, seed=seed) for lo, hi in self.bounds]
        self.copy_in = torch.cuda.Stream(device=device)
        self.compute = torch.cuda.Stream(device=device)
        self.copy_out = torch.cuda.Stream(device=device)

    @classmethod
    def chunk_bounds(cls, rows: int, chunk_units: int = 1) -> list[tuple[int, int]]:
        """Row ranges of the chunks: the remainder first, then whole multiples of 148 work units."""

        if rows <= 0:
            raise ValueError("rows must be positive")
        step = max(1, chunk_units) * cls.UNIT_ROWS
        bounds = []
        first = rows % step or min(rows, step)
        begin = 0
        while begin < rows:
            size = first if begin == 0 else min(step, rows - begin)
            bounds.append((begin, begin + size))
            begin += size
        return bounds

    def __call__(self, q, kv_pair, weights, k_start, k_end, out) -> Any:
        """All arguments are pinned host tensors; ``out`` is int32 ``[Q, 2048]`` and is returned.

        The copies and kernels are ordered after the work already queued on the caller's current
        stream, and that stream waits for the last copy into ``out``.
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
        q_bytes, kv_bytes = q, kv
        caller = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(caller)
        for stream in (self.copy_in, self.compute, self.copy_out):
            stream.wait_event(start)
        with torch.cuda.stream(self.copy_in):
            self.kv.copy_(kv_bytes, non_blocking=True)
            self.kv_scales.copy_(kv_scales, non_blocking=True)
        last = None
        for (lo, hi), ws in zip(self.bounds, self.workspaces):
            arrived, scored = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(self.copy_in):
                self.q[lo:hi].copy_(q_bytes[lo:hi], non_blocking=True)
                self.weights[lo:hi].copy_(weights[lo:hi], non_blocking=True)
                self.k_start[lo:hi].copy_(k_start[lo:hi], non_blocking=True)
                self.k_end[lo:hi].copy_(k_end[lo:hi], non_blocking=True)
                arrived.record(self.copy_in)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(arrived)
                ids = run_operator(ws, self.q[lo:hi], self.kv, self.kv_scales, self.weights[lo:hi],
                                   self.k_start[lo:hi], self.k_end[lo:hi])
                scored.record(self.compute)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(scored)
                out[lo:hi].copy_(ids, non_blocking=True)
                last = torch.cuda.Event()
                last.record(self.copy_out)
        caller.wait_event(last)

    def check_status(self) -> None:
        for ws in self.workspaces:
            ws.check_status()


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
