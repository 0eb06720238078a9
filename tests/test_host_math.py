"""Sample schedule, guarded rank, sample positions and RNG streams (host arithmetic).

Known answers come from the reference's own tests
(``tests/test_fused_index_topk.py:74-93``) and from fixtures recorded by
running the reference's Python layer (``tests/golden/make_golden.py``).
"""

from __future__ import annotations

import hashlib

import pytest
import torch

from fusedindextopk_b200 import sampling
from fusedindextopk_b200.api import PrefillCase
from fusedindextopk_b200.inputs import (
    WORKLOADS,
    input_stream_seeds,
    make_prefill_inputs,
    make_workload_inputs,
)


def _digest(tensor: torch.Tensor) -> str:
    return hashlib.sha256(tensor.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def test_long_context_schedule_known_answers():
    assert sampling.long_context_sample_elements(32768) == 512
    assert sampling.long_context_sample_elements(40000) == 1024
    assert sampling.long_context_sample_elements(65536) == 1024
    assert sampling.long_context_sample_elements(131072) == 1536
    assert sampling.long_context_sample_elements(163840) == 2048
    with pytest.raises(ValueError):
        sampling.long_context_sample_elements(16384)


def test_production_schedule_known_answers():
    assert sampling.production_sample_elements(8192) == 512
    assert sampling.production_sample_elements(16384) == 256
    assert sampling.production_sample_elements(32768) == 512


def test_guarded_rank_rejects_invalid_contracts():
    with pytest.raises(ValueError):
        sampling.guarded_sample_rank(0, 16384)
    with pytest.raises(ValueError):
        sampling.guarded_sample_rank(256, 16384, target_candidates=0)
    with pytest.raises(ValueError):
        sampling.guarded_sample_rank(256, 16384, guard_sigmas=-1.0)


def test_schedule_rank_and_positions_match_recorded_reference(golden):
    for entry in golden["sampling"]:
        context = entry["context_tokens"]
        samples = sampling.production_sample_elements(context)
        assert samples == entry["sample_elements"], context
        rank = sampling.guarded_sample_rank(
            samples, context, target_candidates=sampling.TARGET_CANDIDATES, guard_sigmas=2.0
        )
        assert rank == entry["sample_rank"], context
        loose = sampling.guarded_sample_rank(samples, context, target_candidates=3072, guard_sigmas=0.5)
        assert loose == entry["sample_rank_target3072_guard0p5"], context
        seed = sampling.sampling_seed(0)
        assert seed == entry["sampling_seed"]
        ids = sampling.common_random_sample_ids(torch, context, samples, seed=seed, device="cpu")
        assert ids.dtype == torch.int32 and ids.numel() == samples
        assert ids[:8].tolist() == entry["sample_ids_head"]
        assert ids[-4:].tolist() == entry["sample_ids_tail"]
        assert _digest(ids) == entry["sample_ids_sha256"]
        assert bool((ids[1:] > ids[:-1]).all())


def test_stream_seeds_match_recorded_reference(golden):
    for key, expected in golden["stream_seeds"].items():
        seed, fixture = key.split(":")
        assert input_stream_seeds(int(seed), fixture) == expected
    first = input_stream_seeds(20260803, "A")
    assert len(set(first.values())) == 3
    assert first != input_stream_seeds(20260803, "B")
    with pytest.raises(ValueError, match="fixture_id"):
        input_stream_seeds(1, "C")


def test_standard_recipe_bytes_match_recorded_reference(golden):
    for entry in golden["input_recipe"]:
        case = PrefillCase(
            "golden", entry["query_tokens"], entry["context_tokens"],
            top_k=min(2048, entry["context_tokens"]), seed=entry["seed"],
        )
        made = make_prefill_inputs(case, device="cpu", fixture_id=entry["fixture_id"])
        for name, expected in entry["sha256"].items():
            assert _digest(getattr(made, name)) == expected, (entry, name)
        assert made.q.dtype == torch.float8_e4m3fn and made.kv.dtype == torch.float8_e4m3fn
        assert made.k_end[-1].item() == entry["context_tokens"]


def test_workload_generators_are_seeded_and_shaped():
    a = make_workload_inputs("c1", query_tokens=16, context_tokens=512)
    b = make_workload_inputs("c1", query_tokens=16, context_tokens=512)
    other = make_workload_inputs("c1", query_tokens=16, context_tokens=512, fixture_id="B")
    assert torch.equal(a.kv.view(torch.uint8), b.kv.view(torch.uint8))
    assert torch.equal(a.q.view(torch.uint8), b.q.view(torch.uint8))
    assert not torch.equal(a.kv.view(torch.uint8), other.kv.view(torch.uint8))
    assert a.q.shape == (16, 64, 128) and a.kv.shape == (512, 128)
    assert a.weights.shape == (16, 64) and a.weights.dtype == torch.float32
    assert a.k_start.dtype == torch.int32 and a.k_end.tolist() == list(range(497, 513))
    assert bool((a.kv_scales > 0).all()) and bool(torch.isfinite(a.weights).all())
    # every quantised row uses the full e4m3 range
    assert a.kv.float().abs().amax(dim=1).eq(448).all()


def test_tie_workload_has_few_distinct_keys():
    made = make_workload_inputs("c4", query_tokens=8, context_tokens=1024)
    distinct = torch.unique(made.kv.view(torch.uint8), dim=0)
    assert distinct.shape[0] <= WORKLOADS["c4"].tie_vectors
    assert torch.unique(made.kv_scales).numel() <= WORKLOADS["c4"].tie_vectors


def test_workload_table_matches_benchmark_shapes():
    shapes = {name: (w.query_tokens, w.context_tokens) for name, w in WORKLOADS.items()}
    assert shapes == {
        "c0": (8, 8192), "c1": (4096, 16384), "c2": (4096, 65536),
        "c3": (4096, 163840), "c3s": (64, 131072), "c4": (512, 32768),
    }


def test_host_pipeline_chunks_cover_the_rows_in_whole_waves():
    from fusedindextopk_b200.operator import HostPipeline

    unit = HostPipeline.UNIT_ROWS
    assert unit == 148 * 4
    edge = HostPipeline.EDGE_ROWS
    assert edge == 148
    # a long call: a quarter wave first and last, whole waves and one remainder between them
    assert HostPipeline.chunk_bounds(4096, 1) == [(0, 148), (148, 740), (740, 1332), (1332, 1924), (1924, 2516),
                                                  (2516, 3108), (3108, 3700), (3700, 3948), (3948, 4096)]
    assert HostPipeline.chunk_bounds(4096, 2) == [(0, 148), (148, 1332), (1332, 2516), (2516, 3700), (3700, 3948),
                                                  (3948, 4096)]
    # short calls: the remainder, then whole waves
    assert HostPipeline.chunk_bounds(1184, 2) == [(0, 1184)]
    assert HostPipeline.chunk_bounds(1400, 1) == [(0, 216), (216, 808), (808, 1400)]
    assert HostPipeline.chunk_bounds(5, 2) == [(0, 5)]
    for rows in (1, 591, 592, 593, 1480, 1481, 4095, 4096, 10000, 10001):
        for units in (1, 2, 3):
            bounds = HostPipeline.chunk_bounds(rows, units)
            assert bounds[0][0] == 0 and bounds[-1][1] == rows
            assert all(a[1] == b[0] and a[1] > a[0] and a[1] % 4 == 0 for a, b in zip(bounds, bounds[1:]))
            whole = [hi - lo for lo, hi in bounds[1:-1]] if len(bounds) > 2 else []
            assert sum(1 for size in whole if size % (units * unit)) <= 1
    with pytest.raises(ValueError):
        HostPipeline.chunk_bounds(0)
