"""Paged index keys: table expansion on the CPU; on the GPU the paged call against the
contiguous call on the same keys (plain, key-sharded, forced through the repair path)."""

from __future__ import annotations

import math

import pytest
import torch

from fusedindextopk_b200 import operator, paged
from fusedindextopk_b200.inputs import make_workload_inputs


def test_block_table_expands_to_128_key_tiles():
    table = torch.tensor([3, 0, 5], dtype=torch.int32)
    assert paged.expand_block_table(table, 128).tolist() == [3, 0, 5]
    assert paged.expand_block_table(table, 256).tolist() == [6, 7, 0, 1, 10, 11]
    assert paged.expand_block_table(table, 512).dtype == torch.int32
    with pytest.raises(ValueError):
        paged.expand_block_table(table, 64)
    with pytest.raises(ValueError):
        paged.expand_block_table(table.long(), 128)


def test_scatter_to_pages_places_every_key_where_the_table_says():
    generator = torch.Generator().manual_seed(1)
    kv = torch.randn((1000, 128), generator=generator).to(torch.float8_e4m3fn)
    scales = torch.rand(1000, generator=generator)
    pool, scale_pool, block_table = paged.scatter_to_pages(kv, scales, 256, generator=generator)
    assert pool.shape[1:] == (256, 128) and pool.shape[0] >= 4 and block_table.numel() == 4
    assert block_table.unique().numel() == 4
    tiles = paged.expand_block_table(block_table, 256).long()
    rows = torch.arange(1000)
    stored = tiles[rows // 128] * 128 + rows % 128
    assert torch.equal(pool.view(-1, 128).view(torch.uint8)[stored], kv.view(torch.uint8))
    assert torch.equal(scale_pool.view(-1)[stored], scales)
    assert torch.isnan(scale_pool).sum() == scale_pool.numel() - 1000      # everything else is poison


@pytest.fixture(scope="module")
def device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _both(host, device, page_size, seed, **kwargs):
    from fusedindextopk_b200 import fused_index_topk

    q, kv, scales = host.q.to(device), host.kv.to(device), host.kv_scales.to(device)
    weights, k_start, k_end = host.weights.to(device), host.k_start.to(device), host.k_end.to(device)
    want = fused_index_topk(q, (kv, scales), weights, k_start, k_end).clone()
    generator = torch.Generator().manual_seed(seed)
    pool, scale_pool, block_table = paged.scatter_to_pages(kv, scales, page_size, generator=generator)
    got = paged.fused_index_topk_paged(q, (pool, scale_pool), block_table, int(kv.shape[0]), weights, k_start, k_end,
                                       **kwargs).clone()
    torch.cuda.synchronize()
    return got, want


@pytest.mark.gpu
@pytest.mark.parametrize("rows,keys,page_size", [(64, 8192, 128), (37, 5000, 256), (256, 16384, 512), (8, 40000, 1024)])
def test_paged_call_equals_the_contiguous_call(device, rows, keys, page_size):
    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=rows)
    got, want = _both(host, device, page_size, seed=keys)
    assert torch.equal(got.sort(dim=-1).values, want.sort(dim=-1).values)


@pytest.mark.gpu
def test_paged_repair_path_equals_the_contiguous_call(device):
    """Thresholds of -inf overflow every row's candidate buffer, so all rows come from the paged repair producer."""

    from fusedindextopk_b200 import operator

    rows, keys, page_size = 32, 20000, 256
    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=5)
    q, kv, scales = host.q.to(device), host.kv.to(device), host.kv_scales.to(device)
    weights, k_start, k_end = host.weights.to(device), host.k_start.to(device), host.k_end.to(device)
    plain = operator.make_workspace(rows, keys, device, key_shards=1)
    operator.run_operator(plain, q, kv, scales, weights, k_start, k_end)
    want = plain.output_ids.clone()

    pool, scale_pool, block_table = paged.scatter_to_pages(kv, scales, page_size, generator=torch.Generator().manual_seed(2))
    tiles = paged.expand_block_table(block_table, page_size)
    flat_kv, flat_scales = pool.view(-1, 128), scale_pool.view(-1)
    forced = operator.make_workspace(rows, keys, device, key_shards=1)
    forced.thresholds.fill_(-math.inf)
    operator.run_fused_topk(forced, q, flat_kv, flat_scales, weights, k_start, k_end, tile_table=tiles)
    assert bool(forced.failure_flags.bool().all()), "the forced overflow did not flag every row"
    operator.run_repair(forced, q, flat_kv, flat_scales, weights, k_start, k_end, tile_table=tiles)
    torch.cuda.synchronize()
    forced.check_status()
    assert not bool(forced.failure_flags.bool().any())
    assert torch.equal(forced.output_ids.sort(dim=-1).values, want.sort(dim=-1).values)


@pytest.mark.gpu
def test_paged_batch_through_one_block_table(device):
    """Two sequences, each starting on a page boundary of one logical key space."""

    from fusedindextopk_b200 import batched, fused_index_topk

    page_size = 256
    shapes = [(40, 5120), (24, 3072)]
    made = [make_workload_inputs("c1", query_tokens=r, context_tokens=n, seed=9 + i) for i, (r, n) in enumerate(shapes)]
    q, cu_q = batched.pack_sequences([m.q.view(torch.uint8) for m in made])
    kv, cu_k = batched.pack_sequences([m.kv.view(torch.uint8) for m in made])
    scales, _ = batched.pack_sequences([m.kv_scales for m in made])
    weights, _ = batched.pack_sequences([m.weights for m in made])
    q = q.view(torch.float8_e4m3fn).to(device)
    kv = kv.view(torch.float8_e4m3fn).to(device)
    scales, weights = scales.to(device), weights.to(device)
    k_start, k_end, offset = batched.varlen_ranges(cu_q.to(device), cu_k.to(device))
    pool, scale_pool, block_table = paged.scatter_to_pages(kv, scales, page_size, generator=torch.Generator().manual_seed(3))
    ids = paged.fused_index_topk_paged(q, (pool, scale_pool), block_table, int(kv.shape[0]), weights, k_start, k_end).clone()
    local = torch.where(ids >= 0, ids - offset.unsqueeze(-1), ids)
    for index, m in enumerate(made):
        rows = slice(int(cu_q[index]), int(cu_q[index + 1]))
        alone = fused_index_topk(m.q.to(device), (m.kv.to(device), m.kv_scales.to(device)), m.weights.to(device),
                                 m.k_start.to(device), m.k_end.to(device)).clone()
        assert torch.equal(local[rows].sort(dim=-1).values, alone.sort(dim=-1).values), f"sequence {index}"


@pytest.mark.gpu
def test_repeated_paged_calls_replay_a_graph_and_follow_a_changed_table(device):
    from fusedindextopk_b200 import fused_index_topk

    host = make_workload_inputs("c1", query_tokens=48, context_tokens=8192, seed=3)
    q, kv, scales = host.q.to(device), host.kv.to(device), host.kv_scales.to(device)
    weights, k_start, k_end = host.weights.to(device), host.k_start.to(device), host.k_end.to(device)
    want = fused_index_topk(q, (kv, scales), weights, k_start, k_end).clone().sort(dim=-1).values
    pool, scale_pool, block_table = paged.scatter_to_pages(kv, scales, 256, generator=torch.Generator().manual_seed(8))
    results = [paged.fused_index_topk_paged(q, (pool, scale_pool), block_table, 8192, weights, k_start, k_end).clone()
               for _ in range(4)]
    for got in results:
        assert torch.equal(got.sort(dim=-1).values, want)
    # move two pages inside the pool and update the table in place: the next call must follow
    a, b = int(block_table[0]), int(block_table[1])
    raw = pool.view(torch.uint8)
    raw[[a, b]] = raw[[b, a]]
    scale_pool[[a, b]] = scale_pool[[b, a]]
    block_table[0], block_table[1] = b, a
    again = paged.fused_index_topk_paged(q, (pool, scale_pool), block_table, 8192, weights, k_start, k_end).clone()
    assert torch.equal(again.sort(dim=-1).values, want)
    # ... also when the table is rewritten behind torch's back (a serving engine's own kernel): the
    # expansion is redone on the device on every call, replayed graphs included
    c, d = int(block_table[2]), int(block_table[3])
    raw[[c, d]] = raw[[d, c]]
    scale_pool[[c, d]] = scale_pool[[d, c]]
    alias = torch.as_strided(block_table.detach(), block_table.shape, block_table.stride())
    alias.data[2], alias.data[3] = d, c
    for _ in range(3):
        again = paged.fused_index_topk_paged(q, (pool, scale_pool), block_table, 8192, weights, k_start, k_end).clone()
        assert torch.equal(again.sort(dim=-1).values, want)


@pytest.mark.gpu
def test_paged_argument_errors(device):
    host = make_workload_inputs("c1", query_tokens=8, context_tokens=2048, seed=1)
    q, kv, scales = host.q.to(device), host.kv.to(device), host.kv_scales.to(device)
    weights, k_start, k_end = host.weights.to(device), host.k_start.to(device), host.k_end.to(device)
    pool, scale_pool, block_table = paged.scatter_to_pages(kv, scales, 256, generator=torch.Generator().manual_seed(4))
    with pytest.raises(ValueError, match="does not cover"):
        paged.fused_index_topk_paged(q, (pool, scale_pool), block_table[:-1].contiguous(), 2048, weights, k_start, k_end)
    # a page outside the pool is clamped on the device (nothing is read outside the pool) and recorded
    bad = block_table.clone()
    bad[0] = pool.shape[0]
    workspace = operator.make_workspace(8, 2048, device)
    paged.fused_index_topk_paged(q, (pool, scale_pool), bad, 2048, weights, k_start, k_end, workspace=workspace)
    assert not paged.block_table_was_valid(workspace)
    paged.fused_index_topk_paged(q, (pool, scale_pool), block_table, 2048, weights, k_start, k_end, workspace=workspace)
    assert paged.block_table_was_valid(workspace)
    with pytest.raises(ValueError, match="multiple of 128"):
        paged.fused_index_topk_paged(q, (pool.view(-1, 64, 128), scale_pool.view(-1, 64)), block_table, 2048,
                                     weights, k_start, k_end)
