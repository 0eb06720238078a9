"""Host logic of the multi-GPU partitionings, run as two gloo ranks on the CPU.

The CUDA kernels are replaced by the oracle (local exact Top-2048 pairs, pair merge); what is
under test is the partition arithmetic, the rebasing of the ranges, the gather layout and the
control flow of ``key_sharded_topk``.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from oracle import oracle  # noqa: E402

from fusedindextopk_b200 import distributed  # noqa: E402
from fusedindextopk_b200.inputs import make_workload_inputs  # noqa: E402

TOP_K = 2048


def test_row_deal_is_a_partition():
    for rows, world in ((4096, 8), (10, 4), (7, 2), (3, 4)):
        seen = []
        for rank in range(world):
            seen += distributed.owned_rows(rows, rank, world)
        assert sorted(seen) == list(range(rows))
    assert distributed.owned_rows(16, 1, 2) == [4, 5, 6, 7, 12, 13, 14, 15]
    with pytest.raises(ValueError):
        distributed.owned_rows(8, 2, 2)


def test_key_ranges_tile_the_context():
    for keys, world in ((131072, 8), (163840, 4), (9000, 2), (300, 4)):
        cursor = 0
        for rank in range(world):
            lo, hi = distributed.key_range(keys, rank, world)
            assert lo == cursor and lo % 128 == 0 or lo == keys
            cursor = hi
        assert cursor == keys
    assert distributed.key_range(131072, 3, 8) == (49152, 65536)


def test_shard_rows_and_keys_slice_the_inputs():
    host = make_workload_inputs("c0", query_tokens=10, context_tokens=1024)
    local, row_ids = distributed.shard_rows(host, 1, 2)
    assert row_ids.tolist() == [4, 5, 6, 7]
    assert torch.equal(local.q.view(torch.uint8), host.q.view(torch.uint8)[4:8])
    assert local.case.query_tokens == 4 and torch.equal(local.k_end, host.k_end[4:8])
    sliced, offset = distributed.shard_keys(host, 1, 2)
    assert offset == 512 and sliced.case.context_tokens == 512
    assert torch.equal(sliced.kv.view(torch.uint8), host.kv.view(torch.uint8)[512:])
    assert sliced.k_start.tolist() == [0] * 10
    assert sliced.k_end.tolist() == [int(e) - 512 for e in host.k_end.tolist()]


def _oracle_local_pairs(local, offset):
    logits = oracle.dense_logits(local.q, local.kv, local.kv_scales, local.weights, local.k_start, local.k_end)
    rows = logits.shape[0]
    pairs = np.zeros((rows, TOP_K), dtype=np.uint64)
    counts = np.zeros(rows, dtype=np.int32)
    for row in range(rows):
        end = int(local.k_end[row])
        start = int(local.k_start[row])
        keys = np.arange(start, end)
        packed = oracle.pack_score_id(logits[row, start:end].numpy(), keys + offset)
        best = oracle.topk_pairs(packed, TOP_K)
        pairs[row, : best.size] = best
        counts[row] = best.size
    return torch.from_numpy(pairs.view(np.int64)), torch.from_numpy(counts)


def _oracle_merge(pairs, counts):
    world, rows, _ = pairs.shape
    out = np.full((rows, TOP_K), -1, dtype=np.int32)
    raw = pairs.numpy().view(np.uint64)
    for row in range(rows):
        union = np.concatenate([raw[s, row, : int(counts[s, row])] for s in range(world)])
        best = oracle.topk_pairs(union, TOP_K)
        out[row, : best.size] = (best & np.uint64(0xFFFFFFFF)).astype(np.int32)
    return torch.from_numpy(out)


def _worker(rank: int, world: int, port: int, result_path: str) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        host = make_workload_inputs("c3s", query_tokens=6, context_tokens=6144)
        ids = distributed.key_sharded_topk(
            host, rank, world,
            local_pairs=_oracle_local_pairs, merge=_oracle_merge, all_gather=distributed.dist_all_gather,
        )
        # every rank must hold the same, exact answer
        want, _ = oracle.fused_index_topk(host.q, host.kv, host.kv_scales, host.weights, host.k_start, host.k_end)
        same = torch.equal(ids.sort(dim=-1).values, want[:, 0, :].sort(dim=-1).values)
        gathered = [None] * world
        dist.all_gather_object(gathered, bool(same))
        if rank == 0:
            Path(result_path).write_text("ok" if all(gathered) else f"mismatch {gathered}")
    finally:
        dist.destroy_process_group()


def test_key_sharded_control_flow_on_two_gloo_ranks(tmp_path):
    result = tmp_path / "result.txt"
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"
