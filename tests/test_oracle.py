"""The CPU oracle against independent restatements and known answers."""

from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from oracle import oracle  # noqa: E402

from fusedindextopk_b200.api import PrefillCase  # noqa: E402
from fusedindextopk_b200.correctness import score_threshold_check, validate_topk_indices  # noqa: E402
from fusedindextopk_b200.inputs import make_workload_inputs  # noqa: E402


def test_e4m3_table_matches_torch_decode():
    codes = torch.arange(256, dtype=torch.uint8)
    decoded = codes.view(torch.float8_e4m3fn).float().numpy()
    table = oracle.e4m3_table()
    same = (decoded == table) | (np.isnan(decoded) & np.isnan(table))
    assert same.all()
    assert table[0x7E] == 448.0 and table[0x01] == 2.0 ** -9


def test_dense_logits_match_scalar_loops():
    made = make_workload_inputs("c0", query_tokens=3, context_tokens=40)
    logits = oracle.dense_logits(made.q, made.kv, made.kv_scales, made.weights, made.k_start, made.k_end)
    table = oracle.e4m3_table().astype(np.float64)
    q = table[made.q.view(torch.uint8).numpy()]
    kv = table[made.kv.view(torch.uint8).numpy()]
    for row in range(3):
        for key in range(40):
            if key >= int(made.k_end[row]):
                assert logits[row, key] == -math.inf
                continue
            total = 0.0
            for head in range(64):
                dot = float(np.dot(q[row, head], kv[key]))
                total += float(made.weights[row, head]) * max(dot, 0.0)
            expected = np.float32(total * float(made.kv_scales[key]))
            assert abs(float(logits[row, key]) - expected) <= 2e-6 * abs(expected) + 1e-30


def test_float32_accumulation_stays_inside_the_stated_tolerance():
    made = make_workload_inputs("c1", query_tokens=8, context_tokens=512)
    true = oracle.dense_logits(made.q, made.kv, made.kv_scales, made.weights, made.k_start, made.k_end)
    plain = oracle.dense_logits(
        made.q, made.kv, made.kv_scales, made.weights, made.k_start, made.k_end, accumulate=torch.float32
    )
    finite = torch.isfinite(true)
    row_max = torch.where(finite, true, torch.zeros_like(true)).abs().amax(dim=1, keepdim=True)
    error = torch.where(finite, (true - plain).abs(), torch.zeros_like(true))
    assert bool((error <= 1e-3 * row_max).all())


def test_ordered_bits_are_monotone_and_invertible():
    values = np.array([-np.inf, -3.5, -1e-30, -0.0, 0.0, 1e-30, 2.0, np.inf], dtype=np.float32)
    ordered = oracle.ordered_bits(values)
    assert ordered[3] == ordered[4] == 0x80000000
    assert (np.diff(ordered.astype(np.int64)) >= 0).all()
    back = oracle.ordered_to_float(ordered)
    assert (back == values).all()
    rng = np.random.default_rng(0)
    random = rng.standard_normal(1000).astype(np.float32)
    order = np.argsort(random, kind="stable")
    assert (np.diff(oracle.ordered_bits(random)[order].astype(np.int64)) >= 0).all()
    packed = oracle.pack_score_id(np.array([1.0, -1.0], dtype=np.float32), np.array([7, 9]))
    assert packed[0] > packed[1] and int(packed[0]) & 0xFFFFFFFF == 7


def test_reference_topk_contract_and_exactness():
    made = make_workload_inputs("c0", query_tokens=6, context_tokens=64)
    case = PrefillCase("small", 6, 64, top_k=16, seed=0)
    indices, logits = oracle.fused_index_topk(
        made.q, made.kv, made.kv_scales, made.weights, made.k_start, made.k_end, top_k=16
    )
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits, case)
    short = PrefillCase("short", 4, 5, top_k=8, seed=0)
    made = make_workload_inputs("c0", query_tokens=4, context_tokens=5)
    indices, _ = oracle.fused_index_topk(
        made.q, made.kv, made.kv_scales, made.weights, made.k_start, made.k_end, top_k=8
    )
    validate_topk_indices(indices, short)
    assert sorted(indices[0, 0].tolist()) == [-1] * 6 + [0, 1]


def test_sampled_threshold_rule():
    scores = torch.tensor([[5.0, 1.0, 4.0, -0.0, math.inf, 3.0]] * 4)
    ids = torch.tensor([0, 10, 20, 30, 40, 50], dtype=torch.int32)
    k_start = torch.tensor([0, 0, 15, 0], dtype=torch.int32)
    k_end = torch.tensor([100, 100, 100, 4], dtype=torch.int32)
    out = oracle.sampled_thresholds(scores, ids, k_start, k_end, sample_rank=3, target_candidates=5)
    # row 0/1: valid finite scores 5,1,4,0,3 -> third largest 3
    assert out[0] == 3.0 and out[1] == 3.0
    # row 2: ids >= 15 only: 4,0,3 -> third largest 0 (the -0 reads as +0)
    assert out[2] == 0.0 and not np.signbit(out[2].item())
    # row 3: range no larger than the target -> -inf
    assert out[3] == -math.inf
    few = oracle.sampled_thresholds(scores, ids, k_start, k_end, sample_rank=6, target_candidates=5)
    assert few[0] == -math.inf


def test_chunk_ranges_known_answers():
    k_start = torch.tensor([0, 5, 20000], dtype=torch.int32)
    k_end = torch.tensor([10, 16390, 40000], dtype=torch.int32)
    starts, ends = oracle.chunk_ranges(k_start, k_end, 40000)
    assert starts.tolist() == [[0, 5, 16384], [0, 0, 3616], [0, 0, 0]]
    assert ends.tolist() == [[10, 16384, 16384], [0, 6, 16384], [0, 0, 7232]]


def test_topk_pairs_and_flops():
    pairs = oracle.pack_score_id(np.arange(10, dtype=np.float32), np.arange(10))
    top = oracle.topk_pairs(pairs, 3)
    assert [int(p) & 0xFFFFFFFF for p in top] == [9, 8, 7]
    assert oracle.algorithmic_flops(4096, 16384) == 16384 * (4096 * 12288 + 4096 * 4097 // 2)
    assert abs(oracle.algorithmic_flops(4096, 16384) - 9.6211e11) < 1e8
