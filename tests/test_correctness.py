"""Output contract and tie rule.

The known-answer cases restate the reference's own tests
(``tests/test_correctness.py:47-177``, ``tests/test_lifecycle_gpu.py:158-206``);
the recorded cases replay what the reference's implementation returned.
"""

from __future__ import annotations

import copy
import math

import pytest
import torch

from fusedindextopk_b200.api import PrefillCase
from fusedindextopk_b200.correctness import (
    CorrectnessError,
    build_score_threshold_oracle,
    compare_topk_indices,
    score_threshold_check,
    tolerance_set_report,
    validate_topk_indices,
)


class FakeTensor:
    """Exposes only shape / dtype / is_contiguous / tolist, like a foreign array."""

    def __init__(self, data, *, dtype="int32", contiguous=True):
        self._data = data
        self.dtype = dtype
        self.shape = (len(data), len(data[0]), len(data[0][0]))
        self._contiguous = contiguous

    def is_contiguous(self):
        return self._contiguous

    def tolist(self):
        return copy.deepcopy(self._data)


PADDING_CASE = PrefillCase("small", query_tokens=3, context_tokens=3, top_k=4, seed=1)
GOOD = [[[0, -1, -1, -1]], [[1, 0, -1, -1]], [[2, 0, 1, -1]]]


@pytest.mark.parametrize("wrap", [FakeTensor, lambda d: torch.tensor(d, dtype=torch.int32)])
def test_padded_causal_output_is_accepted(wrap):
    assert validate_topk_indices(wrap(GOOD), PADDING_CASE) == {
        "status": "passed", "rows": 3, "top_k": 4, "valid_ids": 6, "padding_ids": 6,
        "dtype": "int32", "contiguous": True,
    }


@pytest.mark.parametrize(
    ("tensor", "message"),
    [
        (FakeTensor(GOOD, dtype="int64"), "dtype"),
        (FakeTensor(GOOD, contiguous=False), "contiguous"),
        (FakeTensor([[[0, -1, -1, -1]], [[1, 1, -1, -1]], [[2, 0, 1, -1]]]), "duplicate"),
        (FakeTensor([[[1, -1, -1, -1]], [[1, 0, -1, -1]], [[2, 0, 1, -1]]]), "outside"),
        (FakeTensor([[[0, -1, -1, -1]], [[1, 0, -1, -1]], [[2, 0, -1, -1]]]), "expected 3 valid IDs"),
        (FakeTensor([[[0, -2, -1, -1]], [[1, 0, -1, -1]], [[2, 0, 1, -1]]]), "invalid negative"),
    ],
)
def test_contract_violations_are_rejected(tensor, message):
    with pytest.raises(CorrectnessError, match=message):
        validate_topk_indices(tensor, PADDING_CASE)


def test_shape_must_be_q_one_k():
    tensor = FakeTensor(GOOD)
    tensor.shape = (1, 3, 4)
    with pytest.raises(CorrectnessError, match="shape"):
        validate_topk_indices(tensor, PADDING_CASE)


def test_recorded_contract_verdicts(golden):
    recorded = golden["output_contract"]
    good = torch.tensor(GOOD, dtype=torch.int32)
    assert validate_topk_indices(good, PADDING_CASE) == recorded["good_summary"]
    for violation in recorded["violations"]:
        assert violation["message"] is not None
        with pytest.raises(CorrectnessError):
            validate_topk_indices(torch.tensor(violation["data"], dtype=torch.int32), PADDING_CASE)


def test_order_is_irrelevant():
    candidate = FakeTensor([[[-1, 0, -1, -1]], [[-1, 0, 1, -1]], [[1, -1, 2, 0]]])
    result = compare_topk_indices(candidate, FakeTensor(GOOD), PADDING_CASE)
    assert result["comparison"] == "unordered_exact_id_set"
    assert result["cutoff_tie_rows_substituted"] == 0


TIE_CASE = PrefillCase("cutoff-tie", query_tokens=1, context_tokens=5, top_k=3, seed=1)
TIE_ROWS = {0: {"boundary_ids": (2, 3), "required_boundary_selections": 1, "strictly_greater_count": 2}}


def test_set_difference_is_reported():
    with pytest.raises(CorrectnessError, match="missing=.*2.*unexpected=.*3"):
        compare_topk_indices(FakeTensor([[[0, 1, 3]]]), FakeTensor([[[0, 1, 2]]]), TIE_CASE)


def test_tied_substitution_is_accepted_only_at_the_cutoff():
    result = compare_topk_indices(
        FakeTensor([[[0, 1, 3]]]), FakeTensor([[[0, 1, 2]]]), TIE_CASE, cutoff_tie_rows=TIE_ROWS
    )
    assert result["comparison"] == "unordered_exact_topk_score_threshold"
    assert result["cutoff_tie_rows_available"] == 1
    assert result["cutoff_tie_rows_substituted"] == 1
    with pytest.raises(CorrectnessError, match="not an exact score-threshold TopK"):
        compare_topk_indices(
            FakeTensor([[[0, 3, 4]]]), FakeTensor([[[0, 1, 2]]]), TIE_CASE, cutoff_tie_rows=TIE_ROWS
        )


def test_tie_oracle_known_answers():
    scores = torch.tensor([[5.0, 4.0, 3.0, 3.0, 1.0]])
    baseline = torch.tensor([[[0, 1, 2]]], dtype=torch.int32)
    summary, tie_rows = build_score_threshold_oracle(scores, baseline, TIE_CASE)
    assert summary["rows_with_cutoff_ties"] == 1
    assert summary["tie_rows"][0]["boundary_candidate_count"] == 2
    accepted = compare_topk_indices(
        torch.tensor([[[0, 1, 3]]], dtype=torch.int32), baseline, TIE_CASE, cutoff_tie_rows=tie_rows
    )
    assert accepted["status"] == "passed" and accepted["cutoff_tie_rows_substituted"] == 1
    with pytest.raises(CorrectnessError, match="not an exact score-threshold TopK"):
        compare_topk_indices(
            torch.tensor([[[0, 3, 4]]], dtype=torch.int32), baseline, TIE_CASE, cutoff_tie_rows=tie_rows
        )
    with pytest.raises(CorrectnessError, match="below the TopK cutoff"):
        build_score_threshold_oracle(
            torch.tensor([[5.0, 4.0, 3.0, 2.0, 1.0]]),
            torch.tensor([[[0, 1, 4]]], dtype=torch.int32),
            TIE_CASE,
        )


def _scores(entry):
    return torch.tensor(
        [[-math.inf if v is None else v for v in row] for row in entry["scores"]], dtype=torch.float32
    )


def test_recorded_tie_oracles(golden):
    for entry in golden["tie_oracle"]:
        case = PrefillCase("tie", entry["rows"], entry["keys"], top_k=entry["top_k"], seed=0)
        scores = _scores(entry)
        baseline = torch.tensor(entry["baseline"], dtype=torch.int32)
        summary, tie_rows = build_score_threshold_oracle(scores, baseline, case)
        assert summary == entry["summary"]
        recorded = {
            int(row): {key: tuple(value) if isinstance(value, list) else value for key, value in tie.items()}
            for row, tie in entry["tie_rows"].items()
        }
        assert tie_rows == recorded
        swapped = torch.tensor(entry["swapped"], dtype=torch.int32)
        assert compare_topk_indices(swapped, baseline, case, cutoff_tie_rows=tie_rows) == entry["swapped_verdict"]
        # the direct score check agrees with the pairwise comparison
        score_threshold_check(baseline, scores, case)
        score_threshold_check(swapped, scores, case)
        if entry["broken_rejected"]:
            broken = torch.tensor(entry["broken"], dtype=torch.int32)
            with pytest.raises(CorrectnessError):
                compare_topk_indices(broken, baseline, case, cutoff_tie_rows=tie_rows)
            with pytest.raises(CorrectnessError):
                score_threshold_check(broken, scores, case)


def test_tolerance_report_counts_only_swaps_inside_the_window():
    case = PrefillCase("tol", query_tokens=1, context_tokens=6, top_k=3, seed=0)
    scores = torch.tensor([[10.0, 9.0, 5.000, 4.999, 1.0, 0.5]])
    exact = torch.tensor([[[0, 1, 2]]], dtype=torch.int32)
    near = torch.tensor([[[0, 1, 3]]], dtype=torch.int32)
    far = torch.tensor([[[0, 1, 4]]], dtype=torch.int32)
    assert tolerance_set_report(exact, scores, case)["ids_swapped_within_tolerance"] == 0
    report = tolerance_set_report(near, scores, case)
    assert report["ids_swapped_within_tolerance"] == 1 and report["rows_with_set_difference"] == 1
    with pytest.raises(CorrectnessError, match="outside the tolerance window"):
        tolerance_set_report(far, scores, case)
