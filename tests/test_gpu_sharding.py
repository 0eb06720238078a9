"""The two multi-GPU partitionings, emulated rank by rank on one GPU (same kernels, the
collective replaced by stacking), against the unsharded operator."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from oracle import oracle  # noqa: E402

from fusedindextopk_b200 import distributed, operator  # noqa: E402
from fusedindextopk_b200.api import PrefillCase  # noqa: E402
from fusedindextopk_b200.correctness import tolerance_set_report, validate_topk_indices  # noqa: E402
from fusedindextopk_b200.inputs import inputs_to, make_workload_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _single(gpu, device):
    rows, keys = gpu.case.query_tokens, gpu.case.context_tokens
    ws = operator.make_workspace(rows, keys, device)
    ids = operator.run_operator(ws, gpu.q, gpu.kv, gpu.kv_scales, gpu.weights, gpu.k_start, gpu.k_end)
    torch.cuda.synchronize()
    ws.check_status()
    assert int(ws.failure_flags.sum()) == 0
    return ids.clone()


@pytest.mark.parametrize("world", [2, 4])
def test_query_row_shards_reassemble_the_unsharded_result(device, world):
    host = make_workload_inputs("c1", query_tokens=42, context_tokens=8192)
    gpu = inputs_to(host, device)
    whole = _single(gpu, device)
    assembled = torch.full_like(whole, -7)
    for rank in range(world):
        local, row_ids = distributed.shard_rows(gpu, rank, world)
        assembled[row_ids.to(device)] = _single(local, device)
    assert torch.equal(assembled.sort(dim=-1).values, whole.sort(dim=-1).values)


@pytest.mark.parametrize("world,rows,keys", [(2, 8, 16384), (4, 6, 32768), (8, 4, 65536)])
def test_key_range_shards_merge_to_the_exact_topk(device, world, rows, keys):
    host = make_workload_inputs("c3s", query_tokens=rows, context_tokens=keys)
    gpu = inputs_to(host, device)
    case = PrefillCase("keys", rows, keys, 2048, 0)
    pairs, counts = [], []
    for rank in range(world):
        local, offset = distributed.shard_keys(gpu, rank, world)
        ws = operator.make_workspace(rows, local.case.context_tokens, device, with_pairs=True)
        rank_pairs, rank_counts = distributed.gpu_local_pairs(ws, local, offset)
        torch.cuda.synchronize()
        ws.check_status()
        assert int(ws.failure_flags.sum()) == 0
        pairs.append(rank_pairs.clone())
        counts.append(rank_counts.clone())
    out = torch.empty((rows, 2048), dtype=torch.int32, device=device)
    distributed.gpu_merge(torch.stack(pairs), torch.stack(counts), out)
    torch.cuda.synchronize()
    indices = out.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    want = oracle.dense_logits(host.q, host.kv, host.kv_scales, host.weights, host.k_start, host.k_end)
    tolerance_set_report(indices, want, case, relative_tolerance=1e-3)
    whole = _single(gpu, device)
    assert torch.equal(out.sort(dim=-1).values, whole.sort(dim=-1).values)
