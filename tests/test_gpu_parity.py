"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same seeded inputs.

Three levels, as the operator's contract defines them:
(i)   diagnostic dense scores vs the float64-accumulated oracle: ``|err| <= 1e-3 * rowmax``;
(ii)  the returned id sets are a bit-exact Top-K of the kernel's own fp32 scores under
      the tie rule (no tolerance);
(iii) vs the oracle's sets, differences only inside the tolerance window, counted.
"""

from __future__ import annotations

import math
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from oracle import oracle  # noqa: E402

from fusedindextopk_b200 import _lib, operator  # noqa: E402
from fusedindextopk_b200.api import PrefillCase, RunMode, execute_graph  # noqa: E402
from fusedindextopk_b200.correctness import (  # noqa: E402
    score_threshold_check,
    tolerance_set_report,
    validate_topk_indices,
)
from fusedindextopk_b200.inputs import inputs_to, make_prefill_inputs, make_workload_inputs  # noqa: E402

pytestmark = pytest.mark.gpu
RELATIVE_TOLERANCE = 1e-3  # of the row maximum, for fp32 scores


@pytest.fixture(scope="module")
def device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _tensors(inputs):
    return (inputs.q, inputs.kv, inputs.kv_scales, inputs.weights, inputs.k_start, inputs.k_end)


def _assert_close_to_oracle(got: torch.Tensor, want: torch.Tensor) -> float:
    finite = torch.isfinite(want)
    assert torch.equal(finite, torch.isfinite(got)), "mask pattern differs"
    row_max = torch.where(finite, want, torch.zeros_like(want)).abs().amax(dim=1, keepdim=True)
    error = torch.where(finite, (got - want).abs(), torch.zeros_like(want))
    worst = float((error / row_max.clamp_min(1e-30)).max())
    assert worst <= RELATIVE_TOLERANCE, f"score error {worst:.3e} of the row maximum"
    return worst


def _run_with_diagnostics(host, device, *, thresholds=None, repair=True, retry=True):
    rows, keys = host.case.query_tokens, host.case.context_tokens
    gpu = inputs_to(host, device)
    ws = operator.make_workspace(rows, keys, device, seed=host.case.seed)
    operator.run_sample_thresholds(ws, *_tensors(gpu))   # also gathers the sampled keys the retry reads
    if thresholds is not None:
        ws.thresholds.fill_(thresholds)
    logits = torch.full((rows, keys), -math.inf, device=device)
    operator.run_fused_topk(ws, *_tensors(gpu), diag_logits=logits, force_compute=True)
    fast_flags = ws.failure_flags.clone()
    if repair:
        operator.run_repair(ws, *_tensors(gpu), retry=retry)
    torch.cuda.synchronize()
    ws.check_status()
    return ws, logits, fast_flags


def test_library_loads_and_reports_resources(device):
    report = _lib.resource_report()
    assert int(report["fused_topk.registers_per_thread"]) <= 128
    assert int(report["fused_topk.dynamic_shared_bytes"]) <= 232448
    assert int(report["sm_count"]) >= 100


@pytest.mark.parametrize(
    "workload,rows,keys",
    [("c0", 8, 8192), ("c0", 5, 8192), ("c0", 1, 9000),      # 512 samples: one-warp selection, 16 values per lane
     ("c1", 16, 16384), ("c4", 9, 16384),                   # 256 samples: 8 values per lane; c4 ties everywhere
     ("c4", 8, 8192), ("c2", 4, 40000), ("c3", 3, 163840)],   # ties with 512; 1024 and 2048 samples: radix rounds
)
def test_sampled_scores_and_thresholds(device, workload, rows, keys):
    host = make_workload_inputs(workload, query_tokens=rows, context_tokens=keys)
    gpu = inputs_to(host, device)
    ws = operator.make_workspace(rows, keys, device)
    plan = ws.plan
    diag = torch.full((rows, plan.sample_elements), math.nan, device=device)
    operator.run_sample_thresholds(ws, *_tensors(gpu), diag_logits=diag)
    torch.cuda.synchronize()
    ws.check_status()
    want = oracle.sampled_logits(host.q, host.kv, host.kv_scales, host.weights, plan.sample_ids.cpu())
    _assert_close_to_oracle(diag.cpu(), want)
    # the threshold is the exact guarded rank of the kernel's own sampled scores
    expected = oracle.sampled_thresholds(
        diag.cpu(), plan.sample_ids.cpu(), host.k_start, host.k_end, plan.sample_rank, plan.target_candidates
    )
    assert torch.equal(ws.thresholds.cpu(), expected)
    # the production build (no dense output) gives the same thresholds
    first = ws.thresholds.clone()
    ws.thresholds.fill_(123.0)
    operator.run_sample_thresholds(ws, *_tensors(gpu))
    torch.cuda.synchronize()
    assert torch.equal(ws.thresholds, first)


@pytest.mark.parametrize(
    "workload,rows,keys",
    [("c0", 8, 8192), ("c1", 16, 16384), ("c0", 7, 9000), ("c0", 1, 8192), ("c1", 6, 3000), ("c0", 3, 100)],
)
def test_fused_scores_and_topk_against_oracle(device, workload, rows, keys):
    host = make_workload_inputs(workload, query_tokens=rows, context_tokens=keys)
    case = PrefillCase("parity", rows, keys, 2048, 0)
    ws, logits, _ = _run_with_diagnostics(host, device)
    want = oracle.dense_logits(host.q, host.kv, host.kv_scales, host.weights, host.k_start, host.k_end)
    _assert_close_to_oracle(logits.cpu(), want)
    assert int(ws.failure_flags.sum()) == 0
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)          # (ii) bit-exact on own scores
    report = tolerance_set_report(indices, want, case, relative_tolerance=RELATIVE_TOLERANCE)  # (iii)
    assert report["status"] == "passed"
    print(f"\nPARITY {workload} Q={rows} N={keys}: rows_with_set_difference {report['rows_with_set_difference']}, "
          f"ids_swapped_within_tolerance {report['ids_swapped_within_tolerance']}")


@pytest.mark.parametrize("threshold", [-math.inf, math.inf])
def test_forced_spill_and_forced_repair(device, threshold):
    """-inf floods the candidate segments (spill, then overflow); +inf starves them (underflow)."""

    host = make_workload_inputs("c1", query_tokens=12, context_tokens=16384)
    case = PrefillCase("forced", 12, 16384, 2048, 0)
    ws, logits, fast_flags = _run_with_diagnostics(host, device, thresholds=threshold)
    assert int(fast_flags.sum()) == 12, "every row must have been flagged by the fast path"
    assert int(ws.failure_flags.sum()) == 0 and int(ws.repair_error_flags.sum()) == 0
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)


@pytest.mark.parametrize("rows,keys", [(10, 40000), (6, 70001), (4, 150000)])   # 3, 5 and 10 chunks
def test_forced_repair_by_the_dense_rescan_and_by_the_retry(device, rows, keys):
    """+inf thresholds starve every row.  The dense rescan alone (a producer and a merge launch per 16384-key
    chunk) and the retry alone (lower sampled threshold, key shards, merge) must both clear every flag and agree."""

    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=keys)
    case = PrefillCase("forced-chunks", rows, keys, 2048, 0)
    ws, logits, fast_flags = _run_with_diagnostics(host, device, thresholds=math.inf, retry=False)
    assert int(fast_flags.sum()) == rows
    assert int(ws.failure_flags.sum()) == 0 and int(ws.repair_error_flags.sum()) == 0
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)

    again, _, again_flags = _run_with_diagnostics(host, device, thresholds=math.inf, repair=False)
    assert int(again_flags.sum()) == rows
    again.output_ids.fill_(-7)
    operator.run_retry(again, *_tensors(inputs_to(host, device)))
    torch.cuda.synchronize()
    again.check_status()
    assert again.retry.shards == operator.retry_key_shards(keys) > 1
    assert sorted(again.retry.slot_rows.tolist()) == [-1] * (operator.RETRY_SLOTS - rows) + list(range(rows))
    assert int(again.failure_flags.sum()) == 0
    retried = again.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(retried, case)
    verdict = score_threshold_check(retried, logits.cpu(), case)
    if verdict["rows_with_cutoff_ties"] == 0:
        assert torch.equal(again.output_ids.sort(dim=-1).values, ws.output_ids.sort(dim=-1).values)


def test_flagged_rows_beyond_the_retry_slots_go_to_the_dense_rescan(device):
    """40 starved rows: the first 32 (in row order) fit the retry problem, the other 8 stay flagged for
    the dense rescan; the whole repair stage leaves no flag and an exact result."""

    rows, keys = 40, 20000
    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=3)
    case = PrefillCase("beyond-slots", rows, keys, 2048, 0)
    ws, logits, fast_flags = _run_with_diagnostics(host, device, thresholds=math.inf, repair=False)
    assert int(fast_flags.sum()) == rows
    tensors = _tensors(inputs_to(host, device))
    operator.run_retry(ws, *tensors)
    torch.cuda.synchronize()
    left = ws.failure_flags.nonzero().flatten().tolist()
    assert left == list(range(operator.RETRY_SLOTS, rows))
    operator.run_repair(ws, *tensors, retry=False)
    torch.cuda.synchronize()
    ws.check_status()
    assert int(ws.failure_flags.sum()) == 0 and int(ws.repair_error_flags.sum()) == 0
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)


def test_overflowing_rows_are_retried_with_a_sampled_threshold(device):
    """-inf thresholds on a 40000-key context overflow lists and spill of every row (10000 candidates per
    segment); the retry gives each row a sampled threshold and a list per key shard."""

    rows, keys = 8, 40000
    host = make_workload_inputs("c2", query_tokens=rows, context_tokens=keys, seed=5)
    case = PrefillCase("overflow", rows, keys, 2048, 0)
    ws, logits, fast_flags = _run_with_diagnostics(host, device, thresholds=-math.inf, repair=False)
    assert int(fast_flags.sum()) == rows
    operator.run_retry(ws, *_tensors(inputs_to(host, device)))
    torch.cuda.synchronize()
    ws.check_status()
    assert int(ws.failure_flags.sum()) == 0
    assert bool(torch.isfinite(ws.retry.thresholds[:rows]).all())
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)


def test_a_rank_touches_only_its_own_query_blocks(device):
    """Every third query block, with and without key shards: thresholds, ids and flags of the other blocks
    keep what the caller put there, the owned rows match the full problem's exact sets."""

    rows, keys = 48, 32768
    host = make_workload_inputs("c2", query_tokens=rows, context_tokens=keys, seed=11)
    gpu = inputs_to(host, device)
    tensors = _tensors(gpu)
    case = PrefillCase("ownership", rows, keys, 2048, 0)
    full = operator.make_workspace(rows, keys, device, key_shards=1)
    want = operator.run_operator(full, *tensors).clone()
    logits = torch.full((rows, keys), -math.inf, device=device)
    operator.run_fused_topk(full, *tensors, diag_logits=logits)
    ties = score_threshold_check(want.unsqueeze(1).contiguous().cpu(), logits.cpu(), case)["rows_with_cutoff_ties"]
    owned = torch.arange(rows, device=device).view(-1, 4)[1::3].flatten()
    other = torch.ones(rows, dtype=torch.bool, device=device)
    other[owned] = False
    for shards in (1, 4):
        ws = operator.make_workspace(rows, keys, device, block_begin=1, block_stride=3, key_shards=shards)
        assert ws.num_blocks == 4
        ws.thresholds.fill_(123.0)
        ws.output_ids.fill_(-5)
        ws.failure_flags.fill_(0)
        got = operator.run_operator(ws, *tensors)
        torch.cuda.synchronize()
        ws.check_status()
        assert bool((ws.thresholds[other] == 123.0).all()) and bool((ws.thresholds[owned] != 123.0).all())
        assert bool((got[other] == -5).all())
        assert int(ws.failure_flags.sum()) == 0
        if ties == 0:
            assert torch.equal(got[owned].sort(dim=-1).values, want[owned].sort(dim=-1).values)
        # exact on the kernel's own scores: nothing outside the set beats anything inside it
        picked = torch.zeros_like(logits[owned], dtype=torch.bool)
        picked.scatter_(1, got[owned].long(), True)
        assert bool((picked.sum(dim=1) == 2048).all())
        inside = torch.where(picked, logits[owned], torch.full_like(logits[owned], math.inf)).amin(dim=1)
        outside = torch.where(picked, torch.full_like(logits[owned], -math.inf), logits[owned]).amax(dim=1)
        assert bool((inside >= outside).all())


def test_spill_path_without_overflow(device):
    """N = 8192 with threshold -inf: 2048 candidates per segment, 1248 in shared memory and 800 spilled;
    all distances to the threshold are infinite, so the selection takes its radix fallback."""

    host = make_workload_inputs("c0", query_tokens=8, context_tokens=8192)
    case = PrefillCase("spill", 8, 8192, 2048, 0)
    ws, logits, fast_flags = _run_with_diagnostics(host, device, thresholds=-math.inf, repair=False)
    assert int(fast_flags.sum()) == 0
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)


def test_tie_workload_is_exact_under_the_tie_rule(device):
    host = make_workload_inputs("c4", query_tokens=32, context_tokens=32768)
    case = PrefillCase("ties", 32, 32768, 2048, 0)
    ws, logits, _ = _run_with_diagnostics(host, device)
    assert int(ws.failure_flags.sum()) == 0 and int(ws.repair_error_flags.sum()) == 0
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    verdict = score_threshold_check(indices, logits.cpu(), case)
    assert verdict["rows_with_cutoff_ties"] > 0, "the tie workload must actually tie at the cutoff"


def test_zero_queries_tie_everywhere(device):
    """All-zero queries make every score 0: any K valid ids are an exact answer."""

    host = make_workload_inputs("c0", query_tokens=4, context_tokens=8192)
    host.q = torch.zeros_like(host.q.view(torch.uint8)).view(torch.float8_e4m3fn)
    case = PrefillCase("zero", 4, 8192, 2048, 0)
    ws, logits, _ = _run_with_diagnostics(host, device)
    assert int(ws.failure_flags.sum()) == 0
    indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)


def test_public_callable_and_ab_fixtures_share_one_workspace(device):
    case = PrefillCase("ab", 24, 8192, 2048, seed=3)
    results = {}
    for fixture in ("A", "B", "A"):
        host = make_prefill_inputs(case, device="cpu", fixture_id=fixture)
        gpu = inputs_to(host, device)
        from fusedindextopk_b200 import fused_index_topk

        ids = fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end, seed=case.seed)
        torch.cuda.synchronize()
        assert ids.shape == (24, 2048) and ids.dtype == torch.int32
        want_ids, want_logits = oracle.fused_index_topk(
            host.q, host.kv, host.kv_scales, host.weights, host.k_start, host.k_end
        )
        indices = ids.unsqueeze(1).contiguous().cpu()
        validate_topk_indices(indices, case)
        tolerance_set_report(indices, want_logits, case, relative_tolerance=RELATIVE_TOLERANCE)
        results.setdefault(fixture, []).append(indices.clone())
    assert torch.equal(results["A"][0].sort(dim=-1).values, results["A"][1].sort(dim=-1).values)
    assert not torch.equal(results["A"][0].sort(dim=-1).values, results["B"][0].sort(dim=-1).values)


@pytest.mark.parametrize("rows,keys,shards", [(8, 32768, 8), (24, 16384, 4), (7, 65536, 2)])
def test_key_shards_inside_one_gpu_give_the_unsharded_sets(device, rows, keys, shards):
    """Short-Q calls cut every query block's key range into work units that share the row thresholds;
    the merged result must be the same exact Top-2048 (checked on the kernel's own scores)."""

    host = make_workload_inputs("c3", query_tokens=rows, context_tokens=keys)
    gpu = inputs_to(host, device)
    tensors = (gpu.q, gpu.kv, gpu.kv_scales, gpu.weights, gpu.k_start, gpu.k_end)
    case = PrefillCase("shards", rows, keys, 2048, 0)
    plain = operator.make_workspace(rows, keys, device, key_shards=1)
    cut = operator.make_workspace(rows, keys, device, key_shards=shards)
    assert "shard_pairs" in cut.buffers and "shard_pairs" not in plain.buffers
    want = operator.run_operator(plain, *tensors).clone()
    got = operator.run_operator(cut, *tensors)
    torch.cuda.synchronize()
    plain.check_status()
    cut.check_status()
    assert int(cut.failure_flags.sum()) == 0
    logits = torch.full((rows, keys), -math.inf, device=device)
    operator.run_fused_topk(plain, *tensors, diag_logits=logits)
    indices = got.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    score_threshold_check(indices, logits.cpu(), case)
    verdict = score_threshold_check(want.unsqueeze(1).contiguous().cpu(), logits.cpu(), case)
    if verdict["rows_with_cutoff_ties"] == 0:
        assert torch.equal(got.sort(dim=-1).values, want.sort(dim=-1).values)
    # the automatic choice: few query blocks, many keys -> shards; enough blocks -> none
    assert operator.auto_key_shards(16, 163840, 148) == 8
    assert operator.auto_key_shards(64, 65536, 148) == 2
    assert operator.auto_key_shards(1024, 16384, 148) == 1
    assert operator.auto_key_shards(2, 8192, 148) == 2


@pytest.mark.parametrize("rows,keys,shards,split", [(48, 32768, 4, 5), (40, 16384, 2, 1), (30, 65536, 8, 7)])
def test_only_the_blocks_of_the_last_wave_are_split(device, rows, keys, shards, split):
    """`split` of the query blocks (the lowest numbered ones) are cut into key shards and merged, the others
    run as whole units in the same launch; every row must be the exact Top-2048 of the kernel's own scores."""

    host = make_workload_inputs("c2", query_tokens=rows, context_tokens=keys, seed=rows)
    gpu = inputs_to(host, device)
    tensors = _tensors(gpu)
    case = PrefillCase("tail-split", rows, keys, 2048, 0)
    plain = operator.make_workspace(rows, keys, device, key_shards=1)
    want = operator.run_operator(plain, *tensors).clone()
    logits = torch.full((rows, keys), -math.inf, device=device)
    operator.run_fused_topk(plain, *tensors, diag_logits=logits)
    cut = operator.make_workspace(rows, keys, device, key_shards=shards, split_blocks_hint=split)
    assert cut.split_blocks == split
    cut.output_ids.fill_(-9)
    cut.failure_flags.fill_(1)
    got = operator.run_operator(cut, *tensors)
    torch.cuda.synchronize()
    cut.check_status()
    assert int(cut.failure_flags.sum()) == 0
    # the whole blocks did not touch the shard buffers
    assert int(cut.shard_counts[:, 4 * split:].abs().sum()) == 0
    indices = got.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    verdict = score_threshold_check(indices, logits.cpu(), case)
    if verdict["rows_with_cutoff_ties"] == 0:
        assert torch.equal(got.sort(dim=-1).values, want.sort(dim=-1).values)
    assert operator.plan_key_shards(512, 16384, 148) == (68, 2)
    assert operator.plan_key_shards(1024, 16384, 148) == (0, 1)
    assert operator.plan_key_shards(296, 16384, 148) == (0, 1)


@pytest.mark.parametrize("workload,rows,keys,shards,split", [
    ("c1", 24, 16384, 1, 0), ("c2", 40, 32768, 1, 0), ("c0", 8, 8192, 1, 0), ("c2", 48, 32768, 4, 5), ("c4", 64, 32768, 1, 0),
])
def test_thresholds_taken_inside_the_fused_launch_match_the_prepass(device, workload, rows, keys, shards, split):
    """Up to 512 sample keys the whole blocks score the samples themselves; the thresholds they write must be
    bit-identical to the prepass kernel's and the ids the same exact sets."""

    host = make_workload_inputs(workload, query_tokens=rows, context_tokens=keys, seed=rows + 1)
    gpu = inputs_to(host, device)
    tensors = _tensors(gpu)
    case = PrefillCase("in-kernel", rows, keys, 2048, 0)
    prepass = operator.make_workspace(rows, keys, device, seed=host.case.seed, key_shards=1)
    assert prepass.plan.enabled and prepass.plan.sample_elements <= operator.IN_KERNEL_THRESHOLD_SAMPLES
    want_thresholds = operator.run_sample_thresholds(prepass, *tensors).clone()
    logits = torch.full((rows, keys), -math.inf, device=device)
    operator.run_fused_topk(prepass, *tensors, diag_logits=logits)
    operator.run_repair(prepass, *tensors)
    want = prepass.output_ids.clone()
    ws = operator.make_workspace(rows, keys, device, seed=host.case.seed, key_shards=shards,
                                 split_blocks_hint=split if shards > 1 else None)
    ws.thresholds.fill_(777.0)
    got = operator.run_operator(ws, *tensors)
    torch.cuda.synchronize()
    ws.check_status()
    prepass.check_status()
    assert torch.equal(ws.thresholds.view(torch.int32), want_thresholds.view(torch.int32))
    assert int(ws.failure_flags.sum()) == 0
    indices = got.unsqueeze(1).contiguous().cpu()
    validate_topk_indices(indices, case)
    verdict = score_threshold_check(indices, logits.cpu(), case)
    same = torch.ones(rows, dtype=torch.bool, device=device)
    same[torch.tensor(verdict["cutoff_tie_rows"], dtype=torch.long, device=device)] = False
    assert torch.equal(got[same].sort(dim=-1).values, want[same].sort(dim=-1).values)


def test_repair_stage_is_a_conditional_part_of_a_captured_graph(device):
    """Captured into a CUDA graph the repair stage is the body of an IF node on "some row is flagged".  One graph,
    replayed with thresholds that flag no row, then every row (+inf: the retry repairs 32 of them, the dense
    rescan the other 8), then none again, must give the exact result each time and leave no flag."""

    rows, keys = 40, 50000   # four chunks: enough launches for the stage to be made conditional
    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=9)
    gpu = inputs_to(host, device)
    tensors = _tensors(gpu)
    case = PrefillCase("conditional", rows, keys, 2048, 0)
    assert 4 + 2 * 4 >= operator.CONDITIONAL_REPAIR_MIN_LAUNCHES
    ws = operator.make_workspace(rows, keys, device, seed=host.case.seed)
    sampled = operator.run_sample_thresholds(ws, *tensors).clone()
    logits = torch.full((rows, keys), -math.inf, device=device)
    operator.run_fused_topk(ws, *tensors, diag_logits=logits, force_compute=True)
    thresholds = sampled.clone()
    fast_flags = torch.zeros_like(ws.failure_flags)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        operator.run_fused_topk(ws, *tensors, thresholds=thresholds)
        fast_flags.copy_(ws.failure_flags)
        operator.run_repair(ws, *tensors)
    for fill, flagged in ((None, 0), (math.inf, rows), (None, 0), (math.inf, rows)):
        thresholds.copy_(sampled) if fill is None else thresholds.fill_(fill)
        ws.output_ids.fill_(-3)
        graph.replay()
        torch.cuda.synchronize()
        ws.check_status()
        assert int(fast_flags.sum()) == flagged
        assert int(ws.failure_flags.sum()) == 0 and int(ws.repair_error_flags.sum()) == 0
        indices = ws.output_ids.unsqueeze(1).contiguous().cpu()
        validate_topk_indices(indices, case)
        score_threshold_check(indices, logits.cpu(), case)


def test_public_callable_replays_a_graph_with_the_same_result(device):
    """From its second call with the same tensors on the callable replays one CUDA graph."""

    from fusedindextopk_b200 import fused_index_topk

    host = make_workload_inputs("c3s", query_tokens=16, context_tokens=40000)   # key shards + 3 repair chunks
    gpu = inputs_to(host, device)
    args = (gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end)
    workspace = operator.make_workspace(16, 40000, device)
    want = fused_index_topk(*args, workspace=workspace, use_graph=False).sort(dim=-1).values.clone()
    for _ in range(3):
        got = fused_index_topk(*args, workspace=workspace)
        torch.cuda.synchronize()
        assert torch.equal(got.sort(dim=-1).values, want)
    assert len(workspace.graphs) == 1
    # new contents in the same storage are picked up by the replay
    gpu.weights.neg_()
    flipped = fused_index_topk(*args, workspace=workspace, use_graph=False).sort(dim=-1).values.clone()
    assert not torch.equal(flipped, want)
    assert torch.equal(fused_index_topk(*args, workspace=workspace).sort(dim=-1).values, flipped)


def test_repaired_rows_are_mirrored_into_a_mapped_host_buffer(device):
    """The repair stage writes the ids of the rows it repairs a second time, into a pinned host buffer
    (the host pipeline's output, which holds the stale fast-path ids of those rows by then)."""

    rows, keys = 40, 20000
    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=4)
    ws, _, fast_flags = _run_with_diagnostics(host, device, thresholds=math.inf, repair=False)
    assert int(fast_flags.sum()) == rows
    mirror = torch.full((rows, 2048), -11, dtype=torch.int32).pin_memory()
    operator.run_repair(ws, *_tensors(inputs_to(host, device)), mirror=mirror)   # 32 rows by the retry, 8 by the rescan
    torch.cuda.synchronize()
    ws.check_status()
    assert int(ws.failure_flags.sum()) == 0
    assert torch.equal(mirror, ws.output_ids.cpu())


def test_host_pipeline_repairs_a_flagged_row_of_a_long_context(device):
    """c3 (4096 x 163840) from pinned host buffers: nine chunks, one of which holds the row the fast path
    flags; the repair stage at the end of the pipeline must put its ids into the host output."""

    from fusedindextopk_b200 import fused_index_topk
    from fusedindextopk_b200.operator import HostPipeline

    host = make_workload_inputs("c3")
    rows, keys = host.case.query_tokens, host.case.context_tokens
    gpu = inputs_to(host, device)
    want = fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end).clone()
    pinned = [getattr(host, name).contiguous().pin_memory() for name in ("q", "kv", "kv_scales", "weights", "k_start", "k_end")]
    out = torch.empty((rows, 2048), dtype=torch.int32).pin_memory()
    pipeline = HostPipeline(rows, keys, device)
    for call in range(3):
        out.fill_(-7)
        pipeline(pinned[0], (pinned[1], pinned[2]), pinned[3], pinned[4], pinned[5], out)
        torch.cuda.synchronize()
        pipeline.check_status()
        assert int(pipeline.workspace.failure_flags.sum()) == 0
        assert int((out < 0).sum()) == 0 and int((out >= keys).sum()) == 0
        differing = (out.sort(dim=-1).values != want.cpu().sort(dim=-1).values).any(dim=1)
        assert int(differing.sum()) <= 4, f"call {call}: {int(differing.sum())} rows differ from the device call"   # cutoff ties only
        assert torch.equal(out, pipeline.workspace.output_ids.cpu())


def test_host_pipeline_matches_the_device_call(device):
    """Pinned host tensors through the chunked pipeline give the device call's sets."""

    from fusedindextopk_b200 import fused_index_topk
    from fusedindextopk_b200.operator import HostPipeline

    rows, keys = 1500, 8192      # five row chunks (148 + 592 + 592 + 20 + 148), ragged blocks
    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys)
    gpu = inputs_to(host, device)
    want = fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end).clone()
    pinned = [getattr(host, name).contiguous().pin_memory() for name in ("q", "kv", "kv_scales", "weights", "k_start", "k_end")]
    out = torch.full((rows, 2048), -7, dtype=torch.int32).pin_memory()
    pipeline = HostPipeline(rows, keys, device)
    assert [hi - lo for lo, hi in pipeline.bounds] == [148, 592, 592, 20, 148]
    for _ in range(3):   # the first call runs on the streams, the second captures a CUDA graph, the third replays it
        out.fill_(-7)
        result = pipeline(pinned[0], (pinned[1], pinned[2]), pinned[3], pinned[4], pinned[5], out)
        torch.cuda.synchronize()
        pipeline.check_status()
        assert result is out
        assert torch.equal(out.sort(dim=-1).values, want.cpu().sort(dim=-1).values)
    with pytest.raises(ValueError):
        pipeline(gpu.q, (pinned[1], pinned[2]), pinned[3], pinned[4], pinned[5], out)


def test_plugin_graph_matches_reference_output_contract(device):
    from fusedindextopk_b200 import create_variant

    case = PrefillCase("plugin", 16, 8192, 2048, seed=5)
    plugin = create_variant({"diagnostic": True})
    assert plugin.supports(case)
    host = make_prefill_inputs(case, device="cpu")
    graph = plugin.prepare(case, inputs_to(host, device), options={"diagnostic": True}, mode=RunMode.CORRECTNESS)
    assert [node.spec.stage_id for node in graph.nodes] == ["sample_threshold", "fused_topk", "hierarchical_repair"]
    indices = execute_graph(graph, case)
    torch.cuda.synchronize()
    assert tuple(indices.shape) == (16, 1, 2048) and indices.dtype == torch.int32
    indices = indices.contiguous().cpu()
    validate_topk_indices(indices, case)
    want = oracle.dense_logits(host.q, host.kv, host.kv_scales, host.weights, host.k_start, host.k_end)
    tolerance_set_report(indices, want, case, relative_tolerance=RELATIVE_TOLERANCE)
    # fixture B through the same prepared graph
    host_b = make_prefill_inputs(case, device="cpu", fixture_id="B")
    indices_b = execute_graph(graph, case, inputs=inputs_to(host_b, device)).contiguous().cpu()
    torch.cuda.synchronize()
    want_b = oracle.dense_logits(host_b.q, host_b.kv, host_b.kv_scales, host_b.weights, host_b.k_start, host_b.k_end)
    tolerance_set_report(indices_b, want_b, case, relative_tolerance=RELATIVE_TOLERANCE)


def test_invalid_arguments_raise(device):
    host = make_workload_inputs("c0", query_tokens=4, context_tokens=8192)
    gpu = inputs_to(host, device)
    from fusedindextopk_b200 import fused_index_topk

    with pytest.raises(ValueError, match="top_k"):
        fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end, top_k=1024)
    with pytest.raises(ValueError, match="CUDA"):
        fused_index_topk(host.q, (host.kv, host.kv_scales), host.weights, host.k_start, host.k_end)
    with pytest.raises(ValueError, match="int32"):
        fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start.long(), gpu.k_end)
    ws = operator.make_workspace(4, 8192, device)
    args = _lib.FusedArgs()
    with pytest.raises(_lib.ItkError, match="must not be null"):
        _lib.check(_lib.load_library().itk_fused_topk(args, None))
    assert ws.status.item() == 0


ORACLE_ROWS = 128   # evenly spaced query rows compared with the float64 oracle at full size


@pytest.mark.parametrize(
    "workload,rows,keys",
    [("c1", 4096, 16384), ("c2", 4096, 65536), ("c3", 4096, 163840), ("c3s", 64, 131072), ("c4", 512, 32768)],
)
def test_full_size_parity(device, workload, rows, keys):
    """The benchmark configurations at their full size, all three levels.

    (ii) on the device over every row: the result is a bit-exact Top-K of the kernel's own dense
    scores (tie rule), satisfies the output contract and leaves no row flagged; the production build
    (no dense output) returns the same sets where scores are distinct.  (i) and (iii) against the
    float64 oracle on 128 evenly spaced rows: scores within 1e-3 of the row maximum, set differences
    only inside the tolerance window of the oracle's 2048th value, counted and printed.
    """

    host = make_workload_inputs(workload, query_tokens=rows, context_tokens=keys)
    case = PrefillCase("full", rows, keys, 2048, 0)
    ws, logits, fast_flags = _run_with_diagnostics(host, device)
    assert int(ws.failure_flags.sum()) == 0 and int(ws.repair_error_flags.sum()) == 0
    if workload == "c3":
        # at 160 K keys the sampled threshold starves about one row in a thousand: the fast path must
        # flag it and the exact repair must complete it
        assert int(fast_flags.sum()) >= 1, "expected the fast path to flag at least one row at this size"
    indices = ws.output_ids.unsqueeze(1).contiguous()
    validate_topk_indices(indices, case)
    own = score_threshold_check(indices, logits, case)
    gpu = inputs_to(host, device)
    first = indices.clone()
    operator.run_operator(ws, *_tensors(gpu))
    torch.cuda.synchronize()
    ws.check_status()
    again = ws.output_ids.unsqueeze(1).contiguous()
    validate_topk_indices(again, case)
    score_threshold_check(again, logits, case)
    # the production build returns the same sets, except that a row whose cutoff score is shared by more
    # keys than fit may complete its Top-K with any of them
    same = torch.ones(rows, dtype=torch.bool, device=device)
    same[torch.tensor(own["cutoff_tie_rows"], dtype=torch.long, device=device)] = False
    assert torch.equal(first[same].sort(dim=-1).values, again[same].sort(dim=-1).values)

    sample = torch.linspace(0, rows - 1, min(rows, ORACLE_ROWS)).round().long().unique()
    want = oracle.dense_logits(host.q[sample], host.kv, host.kv_scales, host.weights[sample], host.k_start[sample],
                               host.k_end[sample])
    worst = _assert_close_to_oracle(logits[sample.to(device)].cpu(), want)
    report = tolerance_set_report(again[sample.to(device)].cpu(), want, case, relative_tolerance=RELATIVE_TOLERANCE,
                                  rows=sample)
    assert report["status"] == "passed" and report["rows_checked"] > 0
    print(f"\nPARITY {workload} Q={rows} N={keys}: fast-path flags {int(fast_flags.sum())}, rows with cutoff ties "
          f"{own['rows_with_cutoff_ties']}/{own['rows_checked']}; vs oracle on {int(sample.numel())} rows: score error "
          f"{worst:.2e} of row max, rows_with_set_difference {report['rows_with_set_difference']}, "
          f"ids_swapped_within_tolerance {report['ids_swapped_within_tolerance']}")


def test_phase_trace_report_of_the_diagnostic_build(device):
    """`python -m fusedindextopk_b200.trace`: the counters of one traced launch add up."""

    from fusedindextopk_b200.trace import phase_trace

    report = phase_trace("c0", rows=16, keys=8192)
    assert report["active_ctas"] == 4                       # four blocks of four rows, one unit each
    fields = report["fields"]
    assert fields["issuer: tiles"][0] == 64                 # 8192 keys in 128-key tiles
    total = fields["epilogue (row 0): total"][0]
    assert 0 < fields["epilogue: selection"][0] < total
    assert fields["issuer: wait for a free accumulator"][0] < fields["issuer: total"][0]
    assert fields["selection: rows that fell back to the radix rounds"][2] <= 7
    assert 0 < report["cta_wall_us"][0] < 10_000 and 0.5 < report["sm_ghz"] < 3.0
