"""Packed variable-length batches: range construction on the CPU, and on the GPU one packed
call against one call per sequence and against the kernel's own dense scores."""

from __future__ import annotations

import math

import pytest
import torch

from fusedindextopk_b200 import batched
from fusedindextopk_b200.inputs import make_workload_inputs

SHAPES = [(64, 8192), (37, 4500), (100, 3000), (5, 2048), (16, 16384)]


def test_varlen_ranges_match_per_sequence_causal_ranges():
    cu_q = torch.tensor([0, 3, 5, 9], dtype=torch.int32)
    cu_k = torch.tensor([0, 10, 12, 40], dtype=torch.int32)
    k_start, k_end, offset = batched.varlen_ranges(cu_q, cu_k)
    assert k_start.tolist() == [0, 0, 0, 10, 10, 12, 12, 12, 12]
    assert k_end.tolist() == [8, 9, 10, 11, 12, 37, 38, 39, 40]
    assert offset.tolist() == k_start.tolist()
    _, full_end, _ = batched.varlen_ranges(cu_q, cu_k, causal=False)
    assert full_end.tolist() == [10, 10, 10, 12, 12, 40, 40, 40, 40]
    assert k_start.dtype == torch.int32 and k_end.dtype == torch.int32


def test_varlen_ranges_reject_bad_prefix_sums():
    good = torch.tensor([0, 4, 8], dtype=torch.int32)
    with pytest.raises(ValueError, match="int32"):
        batched.varlen_ranges(good.long(), good)
    with pytest.raises(ValueError, match="start at 0"):
        batched.varlen_ranges(torch.tensor([1, 4, 8], dtype=torch.int32), torch.tensor([0, 8, 16], dtype=torch.int32))
    with pytest.raises(ValueError, match="0 < Q_b <= N_b"):
        batched.varlen_ranges(good, torch.tensor([0, 3, 9], dtype=torch.int32))
    with pytest.raises(ValueError, match=r"\[B\+1\]"):
        batched.varlen_ranges(good, torch.tensor([0, 8], dtype=torch.int32))


def test_pack_sequences_builds_prefix_sums():
    parts = [torch.zeros((3, 2)), torch.ones((5, 2))]
    packed, cu = batched.pack_sequences(parts)
    assert packed.shape == (8, 2) and cu.tolist() == [0, 3, 8] and cu.dtype == torch.int32


@pytest.mark.gpu
def test_packed_batch_equals_one_call_per_sequence_and_is_exact_on_its_own_scores():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fusedindextopk_b200 import fused_index_topk, operator

    device = torch.device("cuda:0")
    made = [make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=index + 1)
            for index, (rows, keys) in enumerate(SHAPES)]
    q, cu_q = batched.pack_sequences([m.q.view(torch.uint8) for m in made])
    kv, cu_k = batched.pack_sequences([m.kv.view(torch.uint8) for m in made])
    scales, _ = batched.pack_sequences([m.kv_scales for m in made])
    weights, _ = batched.pack_sequences([m.weights for m in made])
    q = q.view(torch.float8_e4m3fn).to(device)
    kv = kv.view(torch.float8_e4m3fn).to(device)
    scales, weights = scales.to(device), weights.to(device)

    local = batched.fused_index_topk_varlen(q, (kv, scales), weights, cu_q, cu_k).clone()
    packed_ids = batched.fused_index_topk_varlen(q, (kv, scales), weights, cu_q, cu_k, local_ids=False).clone()
    assert local.shape == (int(cu_q[-1]), 2048) and local.dtype == torch.int32

    for index, m in enumerate(made):
        rows = slice(int(cu_q[index]), int(cu_q[index + 1]))
        alone = fused_index_topk(m.q.to(device), (m.kv.to(device), m.kv_scales.to(device)), m.weights.to(device),
                                 m.k_start.to(device), m.k_end.to(device)).clone()
        assert torch.equal(local[rows].sort(dim=-1).values, alone.sort(dim=-1).values), f"sequence {index}"
        shifted = packed_ids[rows]
        rebased = torch.where(shifted >= 0, shifted - int(cu_k[index]), shifted)
        assert torch.equal(rebased.sort(dim=-1).values, local[rows].sort(dim=-1).values)   # the order is free

    # exact Top-K of the kernel's own dense scores over the packed problem
    total_rows, total_keys = int(cu_q[-1]), int(cu_k[-1])
    k_start, k_end, _ = batched.varlen_ranges(cu_q.to(device), cu_k.to(device))
    ws = operator.make_workspace(total_rows, total_keys, device, key_shards=1)
    operator.run_sample_thresholds(ws, q, kv, scales, weights, k_start, k_end)
    logits = torch.full((total_rows, total_keys), -math.inf, device=device)
    operator.run_fused_topk(ws, q, kv, scales, weights, k_start, k_end, diag_logits=logits, force_compute=True)
    torch.cuda.synchronize()
    inside = torch.isfinite(logits)
    hits = torch.zeros(logits.shape, dtype=torch.int32, device=device)
    hits.scatter_add_(1, packed_ids.clamp_min(0).long(), (packed_ids >= 0).int())
    assert int(hits.max()) <= 1, "duplicate ids in a row"
    chosen = hits > 0
    assert bool((chosen & ~inside).sum() == 0), "an id outside its sequence's visible range"
    want_count = torch.minimum(inside.sum(dim=1), torch.tensor(2048, device=device))
    assert torch.equal(chosen.sum(dim=1), want_count)
    worst_in = torch.where(chosen, logits, torch.full_like(logits, math.inf)).amin(dim=1)
    best_out = torch.where(inside & ~chosen, logits, torch.full_like(logits, -math.inf)).amax(dim=1)
    assert bool((worst_in >= best_out).all()), "a better key was left out"
